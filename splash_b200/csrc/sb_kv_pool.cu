// C ABI of the KV page pool (include/splash_b200.h, "KV page pool"): host bookkeeping, and the upload of the lanes' page
// tables into a target.
#include <memory>
#include <new>

#include "model/KvPool.hpp"
#include "sb_internal.h"

using splash::b200::model::KvPool;

namespace {
template <class F> int pool_guarded(F &&f) {
  try {
    return f();
  } catch (const std::invalid_argument &e) {
    return sb::fail(SB_ERR_INVALID, "%s", e.what());
  } catch (const std::out_of_range &) {
    return sb::fail(SB_ERR_INVALID, "sb_kv_pool: no such lane");
  } catch (const std::bad_alloc &) {
    return sb::fail(SB_ERR_OOM, "sb_kv_pool: out of host memory");
  }
}
}  // namespace

extern "C" {

int sb_kv_pool_create(uint32_t pages, uint32_t lanes, uint32_t lane_cap_pages, uint32_t page_tokens, void **out_pool) {
  if (!out_pool) return sb::fail(SB_ERR_INVALID, "sb_kv_pool_create: null pointer");
  return pool_guarded([&] {
    *out_pool = new KvPool(pages, lanes, lane_cap_pages, page_tokens);
    return int(SB_OK);
  });
}
int sb_kv_pool_for_target(void *target, void **out_pool) {
  if (!target || !out_pool) return sb::fail(SB_ERR_INVALID, "sb_kv_pool_for_target: null pointer");
  SbTargetConfig c;
  int st = sb_target_config(target, &c);
  if (st != SB_OK) return st;
  void *table = nullptr;
  uint64_t bytes = 0;
  st = sb_target_tensor(target, -1, "page_table", &table, &bytes);
  if (st != SB_OK) return st;
  const uint32_t lanes = std::max(1u, c.lanes), pages = uint32_t(bytes / 4);
  return sb_kv_pool_create(pages, lanes, pages / lanes, c.page_tokens, out_pool);
}
int sb_kv_pool_destroy(void *pool) {
  delete static_cast<KvPool *>(pool);
  return SB_OK;
}
int sb_kv_pool_acquire(void *pool, uint32_t lane, uint64_t tokens) {
  if (!pool) return sb::fail(SB_ERR_INVALID, "sb_kv_pool_acquire: null pool");
  return pool_guarded([&] {
    KvPool &p = *static_cast<KvPool *>(pool);
    if (!p.acquire(lane, tokens)) return sb::fail(SB_ERR_OOM, "sb_kv_pool_acquire: lane %u needs pages for %llu tokens, %u pages are free", lane, (unsigned long long)tokens, p.pagesFree());
    return int(SB_OK);
  });
}
int sb_kv_pool_release(void *pool, uint32_t lane) {
  if (!pool) return sb::fail(SB_ERR_INVALID, "sb_kv_pool_release: null pool");
  return pool_guarded([&] {
    static_cast<KvPool *>(pool)->release(lane);
    return int(SB_OK);
  });
}
int sb_kv_pool_table(void *pool, uint32_t lane, const uint32_t **out_pages, uint32_t *out_count) {
  if (!pool || !out_pages || !out_count) return sb::fail(SB_ERR_INVALID, "sb_kv_pool_table: null pointer");
  return pool_guarded([&] {
    const std::vector<uint32_t> &t = static_cast<KvPool *>(pool)->table(lane);
    *out_pages = t.data(), *out_count = uint32_t(t.size());
    return int(SB_OK);
  });
}
int sb_kv_pool_counts(void *pool, uint32_t *out_free, uint32_t *out_held) {
  if (!pool || !out_free || !out_held) return sb::fail(SB_ERR_INVALID, "sb_kv_pool_counts: null pointer");
  const KvPool &p = *static_cast<KvPool *>(pool);
  *out_free = p.pagesFree(), *out_held = p.pagesHeld();
  return SB_OK;
}
int sb_kv_pool_write_tables(void *pool, void *target) {
  SB_NEED_DEVICE();
  if (!pool || !target) return sb::fail(SB_ERR_INVALID, "sb_kv_pool_write_tables: null pointer");
  return pool_guarded([&] {
    const KvPool &p = *static_cast<KvPool *>(pool);
    void *table = nullptr;
    uint64_t bytes = 0;
    int st = sb_target_tensor(target, -1, "page_table", &table, &bytes);
    if (st != SB_OK) return st;
    const uint32_t stride = uint32_t(bytes / 4 / p.lanes());
    if (uint64_t(stride) * p.lanes() * 4 != bytes) return sb::fail(SB_ERR_INVALID, "sb_kv_pool_write_tables: the pool has %u lanes, the target's table another count", p.lanes());
    const std::vector<uint32_t> rows = p.tables(stride);
    SB_CUDA(cudaDeviceSynchronize());  // (no step in flight reads the table while it changes)
    SB_CUDA(cudaMemcpy(table, rows.data(), rows.size() * 4, cudaMemcpyHostToDevice));
    return int(SB_OK);
  });
}

}  // extern "C"
