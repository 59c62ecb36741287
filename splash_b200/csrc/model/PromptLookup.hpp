// Proposals a request's own tokens make (prompt lookup): where the request's latest tokens occurred before, the tokens
// that followed them there are a guess at what follows now, which a verify step can check as its block's chain.
//
// Same results as the reference's LookupIndex (runtime/model/LookupProposals.hpp:17-66: the match is the earlier
// occurrence of the longest suffix of the tokens, its length counted up to kLongestMatch, the most recent among those of
// that length, none shorter than kMinimumMatch; proposals() the tokens after it, at most as far as the latest token), by
// another structure. The reference keeps a suffix automaton; here every position is filed under the hash of the k-gram
// that ends at it, for three gram lengths (3, 8 and 24 tokens), each file a chain from the most recent position to the
// oldest. A match of at least g tokens ends at a position of the latest g-gram's chain, so the search walks the chain of
// the longest gram length whose chain is not empty, most recent first, comparing backwards from the candidate, and stops
// at the first candidate that reaches kLongestMatch (no later one can be more recent). Chains of natural text are a few
// entries long; a run of one repeated token stops at its first candidate.
#pragma once

#include <algorithm>
#include <array>
#include <cstdint>
#include <unordered_map>
#include <vector>

namespace splash::b200::model {

class LookupIndex {
 public:
  static constexpr uint32_t kMinimumMatch = 3;
  static constexpr uint32_t kLongestMatch = 64;

  struct Match {
    uint32_t length = 0;  // kMinimumMatch..kLongestMatch; 0: the latest tokens occurred nowhere before
    uint32_t end = 0;     // the index of the earlier occurrence's last token
    bool operator==(const Match &o) const { return length == o.length && end == o.end; }
  };

  void append(const uint32_t *tokens, size_t count) {
    for (size_t i = 0; i < count; ++i) extend(tokens[i]);
  }
  const std::vector<uint32_t> &tokens() const { return tokens_; }
  Match match() const { return match_; }
  // Up to `count` tokens that followed the match's occurrence, at most as far as the latest token; none without a match.
  size_t proposals(uint32_t count, const uint32_t **out) const {
    if (!match_.length) return *out = nullptr, 0;
    const size_t begin = size_t(match_.end) + 1;
    *out = tokens_.data() + begin;
    return std::min<size_t>(count, tokens_.size() - begin);
  }

 private:
  static constexpr std::array<uint32_t, 3> kGrams{3, 8, 24};
  static constexpr uint32_t kNone = UINT32_MAX;

  static uint64_t mix(uint64_t x) {
    x = (x ^ (x >> 33)) * 0xff51afd7ed558ccdull;
    x = (x ^ (x >> 33)) * 0xc4ceb9fe1a85ec53ull;
    return x ^ (x >> 33);
  }
  // Hash of the g tokens that end at `position` (position + 1 >= g).
  uint64_t gramHash(uint32_t position, uint32_t g) const {
    uint64_t h = g;
    for (uint32_t i = 0; i < g; ++i) h = mix(h ^ tokens_[position - i]) + i;
    return h;
  }
  // How many tokens ending at `candidate` equal those ending at `position`, counted up to kLongestMatch.
  uint32_t common(uint32_t candidate, uint32_t position) const {
    const uint32_t limit = std::min<uint32_t>(kLongestMatch, candidate + 1);
    uint32_t n = 0;
    while (n < limit && tokens_[candidate - n] == tokens_[position - n]) ++n;
    return n;
  }
  void extend(uint32_t token) {
    const uint32_t position = uint32_t(tokens_.size());
    tokens_.push_back(token);
    // The chains' heads before this position is filed: the latest g-gram's earlier occurrences.
    std::array<uint32_t, kGrams.size()> head{};
    std::array<uint64_t, kGrams.size()> hash{};
    for (size_t level = 0; level < kGrams.size(); ++level) {
      head[level] = kNone;
      if (position + 1 < kGrams[level]) continue;
      hash[level] = gramHash(position, kGrams[level]);
      const auto it = heads_[level].find(hash[level]);
      if (it != heads_[level].end()) head[level] = it->second;
    }
    match_ = Match{};
    // The longest gram length with an earlier occurrence bounds the match from below, and every occurrence of a match
    // that long lies on that gram's chain. (A chain may also hold other grams of the same hash: common() tells.)
    for (size_t level = kGrams.size(); level-- > 0;) {
      uint32_t best = 0, end = 0;
      for (uint32_t candidate = head[level]; candidate != kNone; candidate = previous_[level][candidate]) {
        const uint32_t n = common(candidate, position);
        if (n > best) best = n, end = candidate;  // (most recent first: an equal length later in the chain is older)
        if (best == kLongestMatch) break;
      }
      if (best >= kGrams[level]) {
        match_ = Match{best, end};
        break;
      }
    }
    for (size_t level = 0; level < kGrams.size(); ++level) {
      previous_[level].push_back(head[level]);
      if (position + 1 >= kGrams[level]) heads_[level][hash[level]] = position;
    }
  }

  std::vector<uint32_t> tokens_;
  std::array<std::unordered_map<uint64_t, uint32_t>, kGrams.size()> heads_;  // gram hash -> the most recent position it ends at
  std::array<std::vector<uint32_t>, kGrams.size()> previous_;                // position -> the next older position of its chain
  Match match_;
};

// How a lookup token compares with the draft's candidates at its depth (16 a proposal position, the most likely first):
// 0 the most likely, 1 another candidate, 2 none of them, 3 unknown (the draft proposes nothing at that depth).
// (lookupAgreement, runtime/model/LookupProposals.cpp:170-178.)
inline uint32_t lookupAgreement(uint32_t token, uint32_t depth, const uint32_t *candidates, size_t count) {
  constexpr uint32_t kCandidates = 16;
  if ((uint64_t(depth) + 1) * kCandidates > count) return 3;
  const uint32_t *at = candidates + size_t(depth) * kCandidates;
  if (at[0] == token) return 0;
  return std::find(at, at + kCandidates, token) != at + kCandidates ? 1 : 2;
}

}  // namespace splash::b200::model
