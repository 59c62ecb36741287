// Host operator layer over the C ABI (include/splash_b200.h): the seam the reference's operators see as
// splash::metal::MetalBackend + CommandGraph (runtime/metal/MetalBackend.hpp:375-547,
// runtime/metal/CommandGraph.hpp:26-146). Operators never touch CUDA; they append launches to a
// CommandGraph, which here is a stream (optionally under CUDA-graph capture).
//
// Errors follow the reference: an argument or extent error throws std::invalid_argument before anything
// is enqueued (runtime/ops/BufferExtent.hpp:19-27); a backend failure throws BackendError.
#pragma once
#include <cstddef>
#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>

#include "../../../include/splash_b200.h"

namespace splash::b200 {

class BackendError : public std::runtime_error {
 public:
  BackendError(int status, const std::string &what) : std::runtime_error(what), status_(status) {}
  int status() const noexcept { return status_; }
  bool outOfMemory() const noexcept { return status_ == SB_ERR_OOM; }

 private:
  int status_;
};

// Throws for a non-zero status: invalid_argument for SB_ERR_INVALID, BackendError otherwise.
inline void check(int status) {
  if (status == SB_OK) return;
  if (status == SB_ERR_INVALID) throw std::invalid_argument(sb_last_error());
  throw BackendError(status, sb_last_error());
}

// A device allocation shared by its views: a view keeps the base alive (MetalBackend.hpp:42-78).
class Buffer {
 public:
  Buffer() = default;
  static Buffer allocate(size_t bytes) {
    void *p = nullptr;
    check(sb_alloc(bytes + kSlack, &p));
    Buffer b;
    b.base_ = std::shared_ptr<void>(p, [](void *q) { sb_free(q); });
    b.data_ = static_cast<uint8_t *>(p);
    b.bytes_ = bytes;
    return b;
  }
  // Memory owned elsewhere (a tensor-parallel group's window); the owner outlives the buffer.
  static Buffer wrap(void *p, size_t bytes) {
    Buffer b;
    b.data_ = static_cast<uint8_t *>(p);
    b.bytes_ = bytes;
    return b;
  }
  Buffer view(size_t offset, size_t bytes) const {
    if (offset + bytes > bytes_) throw std::invalid_argument("Buffer::view past the allocation");
    Buffer b = *this;
    b.data_ = data_ + offset;
    b.bytes_ = bytes;
    return b;
  }
  template <class T = void> T *as() const { return reinterpret_cast<T *>(data_); }
  size_t bytes() const noexcept { return bytes_; }
  explicit operator bool() const noexcept { return data_ != nullptr; }

 private:
  static constexpr size_t kSlack = 256;  // quantized rows are fetched in 16-byte units past their last byte
  std::shared_ptr<void> base_;
  uint8_t *data_ = nullptr;
  size_t bytes_ = 0;
};

// A binding's byte extent, checked before anything is enqueued (BufferExtent.hpp:19-27).
inline void requireBytes(const Buffer &b, size_t bytes, const char *what) {
  if (!b || b.bytes() < bytes)
    throw std::invalid_argument(std::string(what) + ": buffer holds " + std::to_string(b.bytes()) + " bytes, " +
                                std::to_string(bytes) + " needed");
}

// The sequence of launches of one command. `pdl` asks every launch for programmatic stream
// serialization, so a kernel's weight prefetch overlaps the previous kernel's tail.
struct CommandGraph {
  void *stream = nullptr;
  bool pdl = true;
  uint32_t launches = 0;  // kernels appended so far
};

}  // namespace splash::b200
