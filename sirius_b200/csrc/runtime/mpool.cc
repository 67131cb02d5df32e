// Page pool + allocators behind the training step: the piece that makes "memory handover" possible.
//
// The reference wraps an external library (third_party/mpool, an empty submodule in the reference
// tree) whose contract is visible only through its call sites in common/cuda_allocator.{h,cc}:
// one pool of fixed-size physical pages per GPU, a caching allocator for training and a direct
// allocator for inference that each own a virtual range and map pool pages into it, per-page
// ownership ("belong": FREE / TRAIN / INFER), EmptyCache() that returns wholly-free pages to FREE
// so the other side can map them, usage statistics, and an out-of-memory observer. This file
// rebuilds that contract on the CUDA virtual-memory-management driver API (cuMemCreate /
// cuMemAddressReserve / cuMemMap / cuMemSetAccess / cuMemUnmap), looked up at run time so the library
// loads on machines without a driver. A host backend (mmap + mprotect) implements the same page
// operations for CPU tests. Pool and allocators live in one process; sharing physical pages across
// processes (exported handles) is not implemented.
#include <cuda.h>
#include <sys/mman.h>

#include <algorithm>
#include <map>
#include <atomic>
#include <chrono>
#include <thread>
#include <mutex>
#include <string>
#include <vector>

#include "../../../include/sirius_pool.h"
#include "rt_common.h"

namespace srt {
namespace {

// ---- page backends ------------------------------------------------------------------------
struct Backend {
  virtual ~Backend() {}
  virtual int granularity(size_t* out) = 0;
  virtual int reserve(size_t bytes, uint64_t* base) = 0;
  virtual int unreserve(uint64_t base, size_t bytes) = 0;
  virtual int create_page(size_t bytes, uint64_t* handle) = 0;
  virtual int release_page(uint64_t handle) = 0;
  // map() backs one page slot; the range becomes usable only after allow() over it. allow() and unmap()
  // take any run of whole, consecutively mapped slots, so a handover costs one driver call per run
  // rather than one per page.
  virtual int map(uint64_t va, size_t bytes, uint64_t handle) = 0;
  virtual int allow(uint64_t va, size_t bytes) = 0;
  virtual int unmap(uint64_t va, size_t bytes, size_t page_bytes) = 0;
};

#define DRV(name) ((decltype(&name))drv(#name))
static void* drv(const char* sym) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(sym, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
    return nullptr;
  return p;
}
#define CU_CALL(expr)                                                        \
  do {                                                                       \
    CUresult _r = (expr);                                                    \
    if (_r != CUDA_SUCCESS) {                                                \
      set_error("%s -> CUresult %d", #expr, (int)_r);                        \
      return _r == CUDA_ERROR_OUT_OF_MEMORY ? SRT_ERR_NOMEM : SRT_ERR_CUDA;  \
    }                                                                        \
  } while (0)

struct CudaVmmBackend : Backend {
  int device;
  decltype(&cuMemCreate) f_create = nullptr;
  decltype(&cuMemRelease) f_release = nullptr;
  decltype(&cuMemAddressReserve) f_reserve = nullptr;
  decltype(&cuMemAddressFree) f_free = nullptr;
  decltype(&cuMemMap) f_map = nullptr;
  decltype(&cuMemUnmap) f_unmap = nullptr;
  decltype(&cuMemSetAccess) f_access = nullptr;
  decltype(&cuMemGetAllocationGranularity) f_gran = nullptr;
  CUmemAllocationProp prop{};
  explicit CudaVmmBackend(int dev) : device(dev) {
    f_create = DRV(cuMemCreate); f_release = DRV(cuMemRelease); f_reserve = DRV(cuMemAddressReserve);
    f_free = DRV(cuMemAddressFree); f_map = DRV(cuMemMap); f_unmap = DRV(cuMemUnmap);
    f_access = DRV(cuMemSetAccess); f_gran = DRV(cuMemGetAllocationGranularity);
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = dev;
  }
  bool ok() const { return f_create && f_release && f_reserve && f_free && f_map && f_unmap && f_access && f_gran; }
  int granularity(size_t* out) override {
    CU_CALL(f_gran(out, &prop, CU_MEM_ALLOC_GRANULARITY_MINIMUM));
    return SRT_OK;
  }
  int reserve(size_t bytes, uint64_t* base) override {
    CUdeviceptr p = 0;
    CU_CALL(f_reserve(&p, bytes, 0, 0, 0));
    *base = (uint64_t)p;
    return SRT_OK;
  }
  int unreserve(uint64_t base, size_t bytes) override {
    CU_CALL(f_free((CUdeviceptr)base, bytes));
    return SRT_OK;
  }
  int create_page(size_t bytes, uint64_t* handle) override {
    CUmemGenericAllocationHandle h;
    CU_CALL(f_create(&h, bytes, &prop, 0));
    *handle = (uint64_t)h;
    return SRT_OK;
  }
  int release_page(uint64_t handle) override {
    CU_CALL(f_release((CUmemGenericAllocationHandle)handle));
    return SRT_OK;
  }
  int map(uint64_t va, size_t bytes, uint64_t handle) override {
    CU_CALL(f_map((CUdeviceptr)va, bytes, 0, (CUmemGenericAllocationHandle)handle, 0));
    return SRT_OK;
  }
  int allow(uint64_t va, size_t bytes) override {
    CUmemAccessDesc acc{};
    acc.location = prop.location;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    CU_CALL(f_access((CUdeviceptr)va, bytes, &acc, 1));
    return SRT_OK;
  }
  int unmap(uint64_t va, size_t bytes, size_t page_bytes) override {
    // one call over the whole run; a driver that wants one call per mapping gets that instead
    if (!per_page_unmap && bytes > page_bytes) {
      if (f_unmap((CUdeviceptr)va, bytes) == CUDA_SUCCESS) return SRT_OK;
      per_page_unmap = true;
    }
    for (size_t o = 0; o < bytes; o += page_bytes) CU_CALL(f_unmap((CUdeviceptr)(va + o), page_bytes));
    return SRT_OK;
  }
  bool per_page_unmap = false;
};

// Host stand-in: a "page" is just a token; mapping makes the address range accessible.
struct HostBackend : Backend {
  uint64_t next = 1;
  int granularity(size_t* out) override { *out = 2u << 20; return SRT_OK; }
  int reserve(size_t bytes, uint64_t* base) override {
    void* p = mmap(nullptr, bytes, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE, -1, 0);
    if (p == MAP_FAILED) { set_error("host backend: mmap of %zu bytes failed", bytes); return SRT_ERR_NOMEM; }
    *base = (uint64_t)(uintptr_t)p;
    return SRT_OK;
  }
  int unreserve(uint64_t base, size_t bytes) override { munmap((void*)(uintptr_t)base, bytes); return SRT_OK; }
  int create_page(size_t, uint64_t* handle) override { *handle = next++; return SRT_OK; }
  int release_page(uint64_t) override { return SRT_OK; }
  int map(uint64_t va, size_t bytes, uint64_t) override {
    if (mprotect((void*)(uintptr_t)va, bytes, PROT_READ | PROT_WRITE) != 0) { set_error("host backend: mprotect failed"); return SRT_ERR_STATE; }
    return SRT_OK;
  }
  int allow(uint64_t, size_t) override { return SRT_OK; }
  int unmap(uint64_t va, size_t bytes, size_t) override {
    madvise((void*)(uintptr_t)va, bytes, MADV_DONTNEED);
    mprotect((void*)(uintptr_t)va, bytes, PROT_NONE);
    return SRT_OK;
  }
};

enum Belong { kFree = 0, kTrain = 1, kInfer = 2 };

}  // namespace

// One allocator = one virtual range of `slots` page slots; a slot is either unmapped or backed by a
// pool page. Free space is tracked over the whole range; ranges over unmapped slots count as free
// and get pages mapped when an allocation lands on them.
struct Pool;
struct Allocator {
  Pool* pool = nullptr;
  Belong who = kTrain;
  uint64_t base = 0;
  size_t slots = 0;
  std::vector<int> slot_page;            // -1 = not backed, else index into pool->pages (page owned by this allocator)
  std::vector<int> kept_page;            // -1, or the page a not-backed slot is still mapped to (mapping kept after
                                         // the page went back to the pool; reused without a driver call if the page
                                         // is free when the slot is needed again)
  std::map<uint64_t, uint64_t> free_;    // offset -> length, coalesced
  std::map<uint64_t, uint64_t> live_;    // offset -> length of allocated blocks
  size_t allocated = 0, peak = 0, mapped_pages = 0;
  size_t align = 512;
};

struct Pool {
  std::mutex mu;
  // Inference goes first: a training call waits (bounded) while an inference call is queued for the
  // lock, so the few pages of a cold request are not mapped behind the trainer's whole regain.
  std::atomic<int> infer_waiting{0};
  Backend* be = nullptr;
  int device = 0;
  size_t page_bytes = 0, n_pages = 0;
  std::vector<uint64_t> pages;    // physical handles
  std::vector<int> belong;        // per page
  size_t free_pages = 0;
  Allocator train, infer;
  srt_pool_oom_fn oom = nullptr;
  void* oom_user = nullptr;
  long long n_map = 0, n_unmap = 0, n_reuse = 0;
  bool unmap_on_release = false;
  ~Pool() {
    for (Allocator* a : {&train, &infer}) {
      if (!a->base) continue;
      for (size_t s = 0; s < a->slots; ++s)
        if (a->slot_page[s] >= 0 || a->kept_page[s] >= 0) be->unmap(a->base + s * page_bytes, page_bytes, page_bytes);
      be->unreserve(a->base, a->slots * page_bytes);
    }
    for (uint64_t h : pages) be->release_page(h);
    delete be;
  }
};

namespace {

void free_insert(Allocator& a, uint64_t off, uint64_t len) {
  auto next = a.free_.lower_bound(off);
  if (next != a.free_.begin()) {
    auto prev = std::prev(next);
    if (prev->first + prev->second == off) { off = prev->first; len += prev->second; a.free_.erase(prev); }
  }
  if (next != a.free_.end() && off + len == next->first) { len += next->second; a.free_.erase(next); }
  a.free_[off] = len;
}

int take_free_page(Pool& p, Belong who, int* page) {
  for (size_t i = 0; i < p.n_pages; ++i)
    if (p.belong[i] == kFree) { p.belong[i] = who; p.free_pages--; *page = (int)i; return SRT_OK; }
  set_error("page pool: no free page left (%zu pages of %zu MiB)", p.n_pages, p.page_bytes >> 20);
  return SRT_ERR_NOMEM;
}

int map_slots(Pool& p, Allocator& a, uint64_t off, uint64_t len) {
  const size_t s0 = off / p.page_bytes, s1 = (off + len - 1) / p.page_bytes;
  size_t run0 = 0, run_n = 0;  // run of freshly mapped slots waiting for access rights
  auto flush = [&]() -> int {
    if (!run_n) return SRT_OK;
    int rc = p.be->allow(a.base + run0 * p.page_bytes, run_n * p.page_bytes);
    run_n = 0;
    return rc;
  };
  for (size_t s = s0; s <= s1; ++s) {
    if (a.slot_page[s] >= 0) { int rc = flush(); if (rc) return rc; continue; }
    const int kept = a.kept_page[s];
    if (kept >= 0 && p.belong[kept] == kFree) {
      // the slot is still mapped to a page that is free again: take it back without touching the driver
      p.belong[kept] = a.who;
      p.free_pages--;
      a.slot_page[s] = kept;
      a.kept_page[s] = -1;
      a.mapped_pages++;
      p.n_reuse++;
      int rc = flush();
      if (rc) return rc;
      continue;
    }
    int page;
    int rc = take_free_page(p, a.who, &page);
    if (rc) { flush(); return rc; }
    if (kept >= 0) {  // mapped to a page that now serves someone else: drop that mapping first
      int r2 = p.be->unmap(a.base + s * p.page_bytes, p.page_bytes, p.page_bytes);
      if (r2) { p.belong[page] = kFree; p.free_pages++; flush(); return r2; }
      a.kept_page[s] = -1;
      p.n_unmap++;
    }
    rc = p.be->map(a.base + s * p.page_bytes, p.page_bytes, p.pages[page]);
    if (rc) { p.belong[page] = kFree; p.free_pages++; flush(); return rc; }
    a.slot_page[s] = page;
    a.mapped_pages++;
    p.n_map++;
    if (!run_n) run0 = s;
    run_n++;
  }
  return flush();
}

// Pages needed to back [off, off+len) that are not mapped yet.
size_t unmapped_in(const Pool& p, const Allocator& a, uint64_t off, uint64_t len) {
  const size_t s0 = off / p.page_bytes, s1 = (off + len - 1) / p.page_bytes;
  size_t n = 0;
  for (size_t s = s0; s <= s1; ++s) n += a.slot_page[s] < 0 ? 1 : 0;
  return n;
}

int alloc_locked(Pool& p, Allocator& a, size_t nbytes, uint64_t* out) {
  const uint64_t need = (nbytes + a.align - 1) / a.align * a.align;
  // best fit by "new pages required", then by smallest range: reuses mapped memory first
  auto best = a.free_.end();
  size_t best_pages = ~(size_t)0;
  uint64_t best_len = ~0ull;
  for (auto it = a.free_.begin(); it != a.free_.end(); ++it) {
    if (it->second < need) continue;
    const size_t np = unmapped_in(p, a, it->first, need);
    if (np < best_pages || (np == best_pages && it->second < best_len)) {
      best = it; best_pages = np; best_len = it->second;
      if (np == 0 && it->second == need) break;
    }
  }
  if (best == a.free_.end()) {
    set_error("allocator: no contiguous virtual range of %zu bytes", (size_t)need);
    return SRT_ERR_NOMEM;
  }
  if (best_pages > p.free_pages) {
    set_error("allocator: needs %zu more pages, pool has %zu free", best_pages, p.free_pages);
    return SRT_ERR_NOMEM;
  }
  const uint64_t off = best->first, len = best->second;
  int rc = map_slots(p, a, off, need);
  if (rc) return rc;
  a.free_.erase(best);
  if (len > need) a.free_[off + need] = len - need;
  a.live_[off] = need;
  a.allocated += need;
  a.peak = std::max(a.peak, a.allocated);
  *out = a.base + off;
  return SRT_OK;
}

int free_locked(Pool& p, Allocator& a, uint64_t ptr) {
  SRT_REQUIRE(ptr >= a.base && ptr < a.base + a.slots * p.page_bytes, "allocator: pointer %#llx is not from this allocator",
              (unsigned long long)ptr);
  auto it = a.live_.find(ptr - a.base);
  SRT_REQUIRE(it != a.live_.end(), "allocator: double free or unknown block %#llx", (unsigned long long)ptr);
  const uint64_t off = it->first, len = it->second;
  a.live_.erase(it);
  a.allocated -= len;
  free_insert(a, off, len);
  return SRT_OK;
}

// Unmap every mapped slot that lies wholly inside free space and give its page back to the pool.
int empty_cache_locked(Pool& p, Allocator& a, size_t* released_pages) {
  size_t n = 0;
  for (auto& fr : a.free_) {
    const uint64_t b = fr.first, e = fr.first + fr.second;
    const size_t s0 = (b + p.page_bytes - 1) / p.page_bytes;
    const size_t s1 = e / p.page_bytes;  // exclusive
    size_t s = s0;
    while (s < s1) {
      if (a.slot_page[s] < 0) { ++s; continue; }
      size_t t = s;
      while (t < s1 && a.slot_page[t] >= 0) ++t;  // [s, t): a run of backed slots inside free space
      if (p.unmap_on_release) {
        int rc = p.be->unmap(a.base + s * p.page_bytes, (t - s) * p.page_bytes, p.page_bytes);
        if (rc) return rc;
      }
      for (; s < t; ++s) {
        p.belong[a.slot_page[s]] = kFree;
        p.free_pages++;
        if (p.unmap_on_release) p.n_unmap++;
        else a.kept_page[s] = a.slot_page[s];
        a.slot_page[s] = -1;
        a.mapped_pages--;
        ++n;
      }
    }
  }
  if (released_pages) *released_pages = n;
  return SRT_OK;
}

Allocator* pick(Pool* p, int kind) { return kind == SRT_POOL_INFER ? &p->infer : &p->train; }

// Takes the pool lock with the inference-first rule. The wait of a training caller is bounded (50 ms)
// so a stuck inference thread cannot stall training for good.
struct PoolLock {
  std::unique_lock<std::mutex> lk;
  PoolLock(Pool* p, int kind) : lk(p->mu, std::defer_lock) {
    if (kind == SRT_POOL_INFER) {
      p->infer_waiting.fetch_add(1, std::memory_order_acq_rel);
      lk.lock();
      p->infer_waiting.fetch_sub(1, std::memory_order_acq_rel);
    } else {
      const auto give_up = std::chrono::steady_clock::now() + std::chrono::milliseconds(50);
      while (p->infer_waiting.load(std::memory_order_acquire) > 0 && std::chrono::steady_clock::now() < give_up)
        std::this_thread::yield();
      lk.lock();
    }
  }
};

}  // namespace
}  // namespace srt

using namespace srt;

extern "C" {

int srt_pool_create(const srt_pool_config* cfg, srt_pool** out) {
  SRT_REQUIRE(cfg && out, "pool_create: null argument");
  SRT_REQUIRE(cfg->pool_nbytes > 0, "pool_create: pool_nbytes must be positive");
  Pool* p = new Pool();
  p->device = cfg->device;
  p->unmap_on_release = cfg->unmap_on_release != 0;
  if (cfg->backend == SRT_POOL_BACKEND_HOST) {
    p->be = new HostBackend();
  } else {
    SRT_CHECK_CUDA(cudaSetDevice(cfg->device));
    SRT_CHECK_CUDA(cudaFree(0));  // make sure the primary context exists
    CudaVmmBackend* b = new CudaVmmBackend(cfg->device);
    if (!b->ok()) { delete b; delete p; set_error("pool_create: CUDA VMM driver entry points unavailable"); return SRT_ERR_UNSUPPORTED; }
    p->be = b;
  }
  size_t gran = 0;
  int rc = p->be->granularity(&gran);
  if (rc) { delete p; return rc; }
  size_t page = cfg->page_nbytes ? cfg->page_nbytes : (32u << 20);  // CUDAMemPool::PageNbytes() = 32 MiB
  page = (page + gran - 1) / gran * gran;
  p->page_bytes = page;
  p->n_pages = cfg->pool_nbytes / page;
  if (p->n_pages == 0) { delete p; set_error("pool_create: pool smaller than one page"); return SRT_ERR_INVALID; }
  p->pages.reserve(p->n_pages);
  for (size_t i = 0; i < p->n_pages; ++i) {
    uint64_t h;
    rc = p->be->create_page(page, &h);
    if (rc) { delete p; return rc; }
    p->pages.push_back(h);
  }
  p->belong.assign(p->n_pages, kFree);
  p->free_pages = p->n_pages;
  const int scale_t = cfg->train_va_scale > 0 ? cfg->train_va_scale : 8;   // cuda_allocator.cc: va_range_scale 8
  const int scale_i = cfg->infer_va_scale > 0 ? cfg->infer_va_scale : 1;
  struct { Allocator* a; Belong who; int scale; size_t align; } defs[2] = {
      {&p->train, kTrain, scale_t, 1024}, {&p->infer, kInfer, scale_i, 512}};
  for (auto& d : defs) {
    d.a->pool = p;
    d.a->who = d.who;
    d.a->slots = p->n_pages * (size_t)d.scale;
    d.a->align = d.align;
    rc = p->be->reserve(d.a->slots * page, &d.a->base);
    if (rc) { delete p; return rc; }
    d.a->slot_page.assign(d.a->slots, -1);
    d.a->kept_page.assign(d.a->slots, -1);
    d.a->free_[0] = d.a->slots * page;
  }
  *out = (srt_pool*)p;
  return SRT_OK;
}

int srt_pool_destroy(srt_pool* h) {
  delete (Pool*)h;
  return SRT_OK;
}

int srt_pool_alloc(srt_pool* h, int kind, size_t nbytes, void** out) {
  Pool* p = (Pool*)h;
  SRT_REQUIRE(p && out && nbytes > 0, "pool_alloc: bad argument");
  PoolLock guard(p, kind);
  std::unique_lock<std::mutex>& lk = guard.lk;
  uint64_t ptr = 0;
  int rc = alloc_locked(*p, *pick(p, kind), nbytes, &ptr);
  if (rc == SRT_ERR_NOMEM && p->oom) {
    // the reference notifies OOM observers before failing (common/cuda_allocator.cc:311-328)
    srt_pool_oom_fn fn = p->oom;
    void* user = p->oom_user;
    lk.unlock();
    fn(user, kind, nbytes);
    lk.lock();
    rc = alloc_locked(*p, *pick(p, kind), nbytes, &ptr);
  }
  if (rc) return rc;
  *out = (void*)(uintptr_t)ptr;
  return SRT_OK;
}

int srt_pool_free(srt_pool* h, int kind, void* ptr) {
  Pool* p = (Pool*)h;
  SRT_REQUIRE(p, "pool_free: null pool");
  if (!ptr) return SRT_OK;
  PoolLock guard(p, kind);
  return free_locked(*p, *pick(p, kind), (uint64_t)(uintptr_t)ptr);
}

int srt_pool_empty_cache(srt_pool* h, int kind, size_t* released_bytes) {
  Pool* p = (Pool*)h;
  SRT_REQUIRE(p, "pool_empty_cache: null pool");
  PoolLock guard(p, kind);
  size_t n = 0;
  int rc = empty_cache_locked(*p, *pick(p, kind), &n);
  if (released_bytes) *released_bytes = n * p->page_bytes;
  return rc;
}

int64_t srt_pool_stat(srt_pool* h, int which) {
  Pool* p = (Pool*)h;
  if (!p) return -1;
  std::lock_guard<std::mutex> lk(p->mu);
  switch (which) {
    case SRT_POOL_STAT_INFER_USAGE: return (int64_t)(p->infer.mapped_pages * p->page_bytes);
    case SRT_POOL_STAT_TRAIN_USAGE: return (int64_t)p->train.allocated;
    case SRT_POOL_STAT_TRAIN_PEAK: return (int64_t)p->train.peak;
    case SRT_POOL_STAT_TRAIN_ALL: return (int64_t)(p->train.mapped_pages * p->page_bytes);
    case SRT_POOL_STAT_FREE_PAGES: return (int64_t)p->free_pages;
    case SRT_POOL_STAT_POOL_NBYTES: return (int64_t)(p->n_pages * p->page_bytes);
    case SRT_POOL_STAT_PAGE_NBYTES: return (int64_t)p->page_bytes;
    case SRT_POOL_STAT_NUM_MAP: return (int64_t)p->n_map;
    case SRT_POOL_STAT_NUM_UNMAP: return (int64_t)p->n_unmap;
    case SRT_POOL_STAT_INFER_ALLOCATED: return (int64_t)p->infer.allocated;
    case SRT_POOL_STAT_NUM_REUSE: return (int64_t)p->n_reuse;
    default: return -1;
  }
}

int srt_pool_set_oom_handler(srt_pool* h, srt_pool_oom_fn fn, void* user) {
  Pool* p = (Pool*)h;
  SRT_REQUIRE(p, "pool_set_oom_handler: null pool");
  std::lock_guard<std::mutex> lk(p->mu);
  p->oom = fn;
  p->oom_user = user;
  return SRT_OK;
}

}  // extern "C"
