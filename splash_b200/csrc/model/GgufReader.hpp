// GGUF (version 3) header reader over a read-only mapping of the file: scalar and string metadata, small numeric
// arrays, the tensor table, and where each tensor's bytes lie. Host code only; nothing is copied out of the mapping
// but the header's own strings.
//
// Stands where the reference has its header parser (runtime/model/GgufFile.hpp:23-141: tensors, metadata by key, find /
// require, numeric arrays; ggml's type table :38-57) for one file or the parts of a split one; the rotation keys are not read.
// File layout as llama.cpp's gguf.h documents it: magic "GGUF", u32 version, u64 tensor count, u64 key count; per key a
// string, a u32 value type and the value; per tensor a string, u32 dimensions, u64 extents (fastest first), u32 ggml
// type, u64 offset into the data section, which starts at the next multiple of general.alignment (32 by default).
#pragma once

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdint>
#include <cstring>
#include <map>
#include <optional>
#include <stdexcept>
#include <string>
#include <string_view>
#include <vector>

namespace splash::b200::model {

class GgufError : public std::runtime_error {
 public:
  using std::runtime_error::runtime_error;
};

namespace ggml {
constexpr uint32_t kF32 = 0, kF16 = 1, kQ8_0 = 8, kQ4_K = 12, kQ6_K = 14, kBF16 = 30;
}

struct GgmlType {
  const char *name;
  uint32_t blockElements, blockBytes;
};
// Name and block shape of a ggml tensor type by its id (ggml's own numbers), for the types this reader can size; a tensor
// of another type is refused, since its extent in the file could not be checked.
inline bool ggmlTypeOf(uint32_t id, GgmlType &t) {
  switch (id) {
    // plain element types
    case 0: t = {"F32", 1, 4}; return true;
    case 1: t = {"F16", 1, 2}; return true;
    case 30: t = {"BF16", 1, 2}; return true;
    case 28: t = {"F64", 1, 8}; return true;
    case 24: t = {"I8", 1, 1}; return true;
    case 25: t = {"I16", 1, 2}; return true;
    case 26: t = {"I32", 1, 4}; return true;
    case 27: t = {"I64", 1, 8}; return true;
    // blocks of 32 weights
    case 2: t = {"Q4_0", 32, 18}; return true;
    case 3: t = {"Q4_1", 32, 20}; return true;
    case 6: t = {"Q5_0", 32, 22}; return true;
    case 7: t = {"Q5_1", 32, 24}; return true;
    case 8: t = {"Q8_0", 32, 34}; return true;
    case 9: t = {"Q8_1", 32, 36}; return true;
    case 20: t = {"IQ4_NL", 32, 18}; return true;
    case 39: t = {"MXFP4", 32, 17}; return true;
    case 40: t = {"NVFP4", 64, 36}; return true;  // (64 weights)
    // super-blocks of 256 weights
    case 10: t = {"Q2_K", 256, 84}; return true;
    case 11: t = {"Q3_K", 256, 110}; return true;
    case 12: t = {"Q4_K", 256, 144}; return true;
    case 13: t = {"Q5_K", 256, 176}; return true;
    case 14: t = {"Q6_K", 256, 210}; return true;
    case 15: t = {"Q8_K", 256, 292}; return true;
    case 16: t = {"IQ2_XXS", 256, 66}; return true;
    case 17: t = {"IQ2_XS", 256, 74}; return true;
    case 22: t = {"IQ2_S", 256, 82}; return true;
    case 18: t = {"IQ3_XXS", 256, 98}; return true;
    case 21: t = {"IQ3_S", 256, 110}; return true;
    case 19: t = {"IQ1_S", 256, 50}; return true;
    case 29: t = {"IQ1_M", 256, 56}; return true;
    case 23: t = {"IQ4_XS", 256, 136}; return true;
    default: return false;
  }
}
inline std::string ggmlTypeName(uint32_t id) {
  GgmlType t;
  return ggmlTypeOf(id, t) ? std::string(t.name) : "type " + std::to_string(id);
}

struct GgufTensor {
  std::string name;
  uint32_t type = 0;
  std::vector<uint64_t> dims;  // dims[0] is the fastest (a row's length)
  uint64_t offset = 0;         // in its part's data section
  uint32_t part = 0;           // which file of a split GGUF holds it
  uint64_t bytes = 0;
  const uint8_t *data = nullptr;  // in the mapping
  uint64_t columns() const { return dims.empty() ? 0 : dims[0]; }
  uint64_t rows() const { return elements() / (columns() ? columns() : 1); }
  uint64_t elements() const {
    uint64_t n = dims.empty() ? 0 : 1;
    for (uint64_t d : dims) n *= d;
    return n;
  }
};

// Scalar metadata by key: integers and booleans as unsigned (a negative one as its two's complement), floats as double.
struct GgufMetadata {
  std::map<std::string, uint64_t, std::less<>> unsigneds;
  std::map<std::string, double, std::less<>> floats;
  std::map<std::string, std::string, std::less<>> strings;
  std::optional<uint64_t> integer(std::string_view key) const {
    auto it = unsigneds.find(key);
    return it == unsigneds.end() ? std::nullopt : std::optional<uint64_t>(it->second);
  }
  std::optional<double> number(std::string_view key) const {
    auto it = floats.find(key);
    if (it != floats.end()) return it->second;
    if (auto u = integer(key)) return double(*u);
    return std::nullopt;
  }
  std::optional<std::string> text(std::string_view key) const {
    auto it = strings.find(key);
    return it == strings.end() ? std::nullopt : std::optional<std::string>(it->second);
  }
  std::string architecture() const { return text("general.architecture").value_or(""); }
};

class GgufReader {
 public:
  explicit GgufReader(const std::string &path) : GgufReader(std::vector<std::string>{path}) {}
  // The parts of a split GGUF in split order (llama.cpp's gguf-split: every part a GGUF of its own with the keys split.no,
  // split.count and split.tensors.count; the first holds the model's metadata), or one whole file. A part read alone, parts
  // out of order or of another split are refused (the reference's GgufFile over several sources,
  // runtime/model/GgufFile.hpp:104-111).
  explicit GgufReader(const std::vector<std::string> &paths) {
    if (paths.empty()) throw GgufError("no GGUF file given");
    try {
      for (const std::string &path : paths) {
        open(path);
        GgufMetadata own;
        parse(parts_.size() - 1, parts_.size() == 1 ? metadata_ : own);
        const GgufMetadata &meta = parts_.size() == 1 ? metadata_ : own;
        const uint64_t count = meta.integer("split.count").value_or(1), number = meta.integer("split.no").value_or(0);
        if (count != paths.size() || number != parts_.size() - 1)
          throw GgufError(path + " is part " + std::to_string(number + 1) + " of " + std::to_string(count) + " of a split GGUF, given as part " +
                          std::to_string(parts_.size()) + " of " + std::to_string(paths.size()));
      }
      if (const auto total = metadata_.integer("split.tensors.count"); total && *total != tensors_.size())
        throw GgufError(paths.front() + ": the parts hold " + std::to_string(tensors_.size()) + " tensors, the split " + std::to_string(*total));
    } catch (...) {
      close();
      throw;
    }
  }
  ~GgufReader() { close(); }
  GgufReader(const GgufReader &) = delete;
  GgufReader &operator=(const GgufReader &) = delete;

  const GgufMetadata &metadata() const { return metadata_; }
  const std::vector<GgufTensor> &tensors() const { return tensors_; }
  const GgufTensor *find(std::string_view name) const {
    auto it = index_.find(name);
    return it == index_.end() ? nullptr : &tensors_[it->second];
  }
  const GgufTensor &require(std::string_view name) const {
    const GgufTensor *t = find(name);
    if (!t) throw GgufError("the GGUF has no tensor " + std::string(name));
    return *t;
  }
  // A numeric array's values (of the first part's metadata), nullptr for a key that holds none (arrays of up to 65536
  // numbers are kept).
  const std::vector<double> *numericArray(std::string_view key) const {
    auto it = arrays_.find(key);
    return it == arrays_.end() ? nullptr : &it->second;
  }
  size_t parts() const { return parts_.size(); }
  uint64_t dataStart(size_t part = 0) const { return parts_[part].dataStart; }
  uint32_t alignment(size_t part = 0) const { return parts_[part].alignment; }
  const std::string &path(size_t part = 0) const { return parts_[part].path; }

 private:
  // GGUF value types.
  enum : uint32_t { kU8, kI8, kU16, kI16, kU32, kI32, kF32, kBool, kString, kArray, kU64, kI64, kF64 };
  struct Part {
    std::string path;
    const uint8_t *base = nullptr;
    uint64_t size = 0, at = 0, dataStart = 0;
    uint32_t alignment = 32;
  };

  void open(const std::string &path) {
    const int fd = ::open(path.c_str(), O_RDONLY);
    if (fd < 0) throw GgufError("cannot open " + path);
    struct stat st {};
    if (::fstat(fd, &st) != 0 || st.st_size < 24) {
      ::close(fd);
      throw GgufError(path + " is not a GGUF file (too short)");
    }
    void *m = ::mmap(nullptr, size_t(st.st_size), PROT_READ, MAP_PRIVATE, fd, 0);
    ::close(fd);
    if (m == MAP_FAILED) throw GgufError("cannot map " + path);
    Part part;
    part.path = path, part.base = static_cast<const uint8_t *>(m), part.size = uint64_t(st.st_size);
    parts_.push_back(part);
  }
  void close() {
    for (Part &part : parts_)
      if (part.base) ::munmap(const_cast<uint8_t *>(part.base), part.size);
    parts_.clear();
  }
  template <class T> T take(Part &f) {
    if (f.at + sizeof(T) > f.size) throw GgufError(f.path + ": the header runs past the end of the file");
    T v;
    std::memcpy(&v, f.base + f.at, sizeof(T));
    f.at += sizeof(T);
    return v;
  }
  std::string takeString(Part &f) {
    const uint64_t n = take<uint64_t>(f);
    if (n > f.size - f.at) throw GgufError(f.path + ": a string runs past the end of the file");
    std::string s(reinterpret_cast<const char *>(f.base + f.at), size_t(n));
    f.at += n;
    return s;
  }
  // One scalar of `type` as (is it a float, unsigned bits, double).
  bool takeScalar(Part &f, uint32_t type, uint64_t &u, double &d) {
    switch (type) {
      case kU8: u = take<uint8_t>(f); return false;
      case kI8: u = uint64_t(int64_t(take<int8_t>(f))); return false;
      case kU16: u = take<uint16_t>(f); return false;
      case kI16: u = uint64_t(int64_t(take<int16_t>(f))); return false;
      case kU32: u = take<uint32_t>(f); return false;
      case kI32: u = uint64_t(int64_t(take<int32_t>(f))); return false;
      case kBool: u = take<uint8_t>(f) != 0; return false;
      case kU64: u = take<uint64_t>(f); return false;
      case kI64: u = uint64_t(take<int64_t>(f)); return false;
      case kF32: d = take<float>(f); return true;
      case kF64: d = take<double>(f); return true;
      default: throw GgufError(f.path + ": metadata value type " + std::to_string(type) + " is not one of GGUF's");
    }
  }
  // Part `index`: its metadata into `meta` (the first part's numeric arrays are kept), its tensors appended.
  void parse(size_t index, GgufMetadata &meta) {
    Part &f = parts_[index];
    if (std::memcmp(f.base, "GGUF", 4) != 0) throw GgufError(f.path + " is not a GGUF file (magic)");
    f.at = 4;
    const uint32_t version = take<uint32_t>(f);
    if (version != 3) throw GgufError(f.path + ": GGUF version " + std::to_string(version) + " (version 3 is read)");
    const uint64_t tensorCount = take<uint64_t>(f), keyCount = take<uint64_t>(f);
    if (tensorCount > f.size / 24 || keyCount > f.size / 12) throw GgufError(f.path + ": counts exceed what the file can hold");
    for (uint64_t k = 0; k < keyCount; ++k) {
      const std::string key = takeString(f);
      const uint32_t type = take<uint32_t>(f);
      if (type == kString) {
        meta.strings[key] = takeString(f);
      } else if (type == kArray) {
        const uint32_t inner = take<uint32_t>(f);
        const uint64_t n = take<uint64_t>(f);
        if (inner == kArray) throw GgufError(f.path + ": nested arrays (" + key + ")");
        std::vector<double> kept;
        const bool keep = inner != kString && n <= 65536 && index == 0;
        for (uint64_t i = 0; i < n; ++i) {
          if (inner == kString) {
            (void)takeString(f);
            continue;
          }
          uint64_t u = 0;
          double d = 0;
          const bool isFloat = takeScalar(f, inner, u, d);
          if (keep) kept.push_back(isFloat ? d : (inner == kI8 || inner == kI16 || inner == kI32 || inner == kI64 ? double(int64_t(u)) : double(u)));
        }
        if (keep) arrays_[key] = std::move(kept);
      } else {
        uint64_t u = 0;
        double d = 0;
        if (takeScalar(f, type, u, d)) meta.floats[key] = d;
        else meta.unsigneds[key] = u;
      }
    }
    f.alignment = uint32_t(meta.integer("general.alignment").value_or(32));
    if (!f.alignment || (f.alignment & (f.alignment - 1))) throw GgufError(f.path + ": general.alignment is not a power of two");
    const size_t first = tensors_.size();
    tensors_.reserve(first + size_t(tensorCount));
    for (uint64_t t = 0; t < tensorCount; ++t) {
      GgufTensor tensor;
      tensor.name = takeString(f);
      const uint32_t nd = take<uint32_t>(f);
      if (nd < 1 || nd > 4) throw GgufError(f.path + ": " + tensor.name + " has " + std::to_string(nd) + " dimensions");
      uint64_t elements = 1;
      for (uint32_t d = 0; d < nd; ++d) {
        const uint64_t e = take<uint64_t>(f);
        if (!e || elements > UINT64_MAX / e) throw GgufError(f.path + ": " + tensor.name + " has an empty or overflowing extent");
        elements *= e;
        tensor.dims.push_back(e);
      }
      tensor.type = take<uint32_t>(f);
      tensor.offset = take<uint64_t>(f);
      tensor.part = uint32_t(index);
      GgmlType type;
      if (!ggmlTypeOf(tensor.type, type)) throw GgufError(f.path + ": " + tensor.name + " is of ggml type " + std::to_string(tensor.type) + ", which this reader cannot size");
      if (tensor.dims[0] % type.blockElements) throw GgufError(f.path + ": " + tensor.name + " rows are not whole " + type.name + " blocks");
      tensor.bytes = elements / type.blockElements * type.blockBytes;
      if (tensor.offset % f.alignment) throw GgufError(f.path + ": " + tensor.name + " does not start on the file's alignment");
      if (!index_.emplace(tensor.name, tensors_.size()).second) throw GgufError(f.path + ": two tensors named " + tensor.name);
      tensors_.push_back(std::move(tensor));
    }
    f.dataStart = (f.at + f.alignment - 1) / f.alignment * f.alignment;
    for (size_t t = first; t < tensors_.size(); ++t) {
      GgufTensor &tensor = tensors_[t];
      if (f.dataStart > f.size || tensor.offset > f.size - f.dataStart || tensor.bytes > f.size - f.dataStart - tensor.offset)
        throw GgufError(f.path + ": " + tensor.name + " lies past the end of the file");
      tensor.data = f.base + f.dataStart + tensor.offset;
    }
  }

  std::vector<Part> parts_;
  GgufMetadata metadata_;
  std::map<std::string, std::vector<double>, std::less<>> arrays_;
  std::vector<GgufTensor> tensors_;
  std::map<std::string, size_t, std::less<>> index_;
};

}  // namespace splash::b200::model
