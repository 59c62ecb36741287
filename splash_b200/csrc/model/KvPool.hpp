// The pages of a target's INT8 cache as a pool the lanes draw from: a lane holds the pages its tokens need and gives them
// back when its request ends, so lanes of short contexts leave room for long ones. Host bookkeeping only; the kernels
// reach a lane's pages through its row of the page table (SbKvLayer / page_table of sb_attn_store, sb_attn_verify), which
// write_tables fills.
//
// The reference's pool (runtime/engine/KvPool.hpp: acquire / release of pages for a request's table, KvPageAcquisition with a
// refusal instead of a crash when memory is short, the counts of KvPoolSnapshot) also grows and shrinks by extents, moves
// pages to empty extents and shares prefix pages between requests; none of that is here: the pool is the fixed set of pages
// the target allocated.
#pragma once

#include <algorithm>
#include <cstdint>
#include <stdexcept>
#include <vector>

namespace splash::b200::model {

class KvPool {
 public:
  // pages: the page ids 0 .. pages - 1 of every layer's page arrays; laneCap: the most pages one lane may hold (the width of
  // a lane's row of the page table).
  KvPool(uint32_t pages, uint32_t lanes, uint32_t laneCap, uint32_t pageTokens) : held_(lanes), laneCap_(laneCap), pageTokens_(pageTokens) {
    if (!pages || !lanes || !laneCap || !pageTokens) throw std::invalid_argument("KvPool: no pages, lanes, lane cap or page size");
    free_.resize(pages);
    for (uint32_t i = 0; i < pages; ++i) free_[i] = pages - 1 - i;  // (handed out lowest id first)
  }
  // Makes sure `lane` holds the pages of `tokens` tokens. False, with nothing taken, when the pool cannot give them.
  bool acquire(uint32_t lane, uint64_t tokens) {
    std::vector<uint32_t> &mine = held_.at(lane);
    const uint64_t need = (tokens + pageTokens_ - 1) / pageTokens_;
    if (need > laneCap_) throw std::invalid_argument("KvPool::acquire: more tokens than a lane's page table holds");
    if (need <= mine.size()) return true;
    if (need - mine.size() > free_.size()) return false;
    while (mine.size() < need) {
      mine.push_back(free_.back());
      free_.pop_back();
    }
    return true;
  }
  // Gives the lane's pages back (its request ended); the most recently taken are handed out again first.
  void release(uint32_t lane) {
    std::vector<uint32_t> &mine = held_.at(lane);
    for (auto it = mine.rbegin(); it != mine.rend(); ++it) free_.push_back(*it);
    mine.clear();
  }
  const std::vector<uint32_t> &table(uint32_t lane) const { return held_.at(lane); }
  uint32_t lanes() const { return uint32_t(held_.size()); }
  uint32_t laneCap() const { return laneCap_; }
  uint32_t pagesFree() const { return uint32_t(free_.size()); }
  uint32_t pagesHeld() const {
    size_t n = 0;
    for (const auto &h : held_) n += h.size();
    return uint32_t(n);
  }
  // The lanes' rows of a page table of `stride` entries a lane: a lane's pages in the order it took them, the entries past
  // them a page the lane holds (or page 0), which no kernel reads while the lane's tokens stay within what it acquired.
  std::vector<uint32_t> tables(uint32_t stride) const {
    if (stride < laneCap_) throw std::invalid_argument("KvPool::tables: a row narrower than the lane cap");
    std::vector<uint32_t> out(size_t(stride) * held_.size(), 0);
    for (size_t lane = 0; lane < held_.size(); ++lane) {
      const std::vector<uint32_t> &mine = held_[lane];
      for (uint32_t i = 0; i < stride; ++i) out[lane * stride + i] = i < mine.size() ? mine[i] : (mine.empty() ? 0u : mine.back());
    }
    return out;
  }

 private:
  std::vector<uint32_t> free_;
  std::vector<std::vector<uint32_t>> held_;
  uint32_t laneCap_, pageTokens_;
};

}  // namespace splash::b200::model
