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
// loads on machines without a driver. A host backend (a memfd whose pages are mmap-ed into the
// reserved ranges) implements the same page operations for CPU tests.
//
// Across processes (the reference's pool is a set of mpool::SharableObject in POSIX shared memory that the
// inference server creates and every trainer opens, common/cuda_allocator.cc:61-99): the process that
// creates a shared pool owns the physical pages and a named segment with the page ownership table, the
// free-page count, the usage counters of both sides and the pool lock (process-shared, robust). It serves
// the pages' shareable handles (POSIX file descriptors from cuMemExportToShareableHandle; the memfd of
// the host backend) on an abstract Unix socket named after the pool. A process that attaches connects
// there, imports the handles, maps the segment, and builds its own allocators with their own virtual
// ranges over the same physical pages: a page the trainer's EmptyCache marks FREE is mapped by the
// server's allocator a moment later, in another process. The free maps of an allocator are private
// to the process that uses it (the trainer never allocates from the inference range, nor the
// server from the training range); what the other side needs of them is in the shared counters.
#include <cuda.h>
#include <pthread.h>
#include <sys/mman.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>
#include <fcntl.h>
#include <poll.h>
#include <sys/stat.h>
#include <stddef.h>

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
  // Cross-process sharing of the physical pages. prepare_pages() creates all pages of the pool in one go
  // (shareable when asked for); export_fds() yields file descriptors a peer process can turn into page handles
  // with import_fds() (one per page for CUDA, one for the whole pool for the host backend). The caller
  // closes the descriptors.
  virtual int export_fds(const std::vector<uint64_t>& handles, std::vector<int>* fds) = 0;
  virtual int import_fds(const std::vector<int>& fds, size_t n_pages, size_t page_bytes, std::vector<uint64_t>* handles) = 0;
  virtual void set_shareable(bool) {}
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
  decltype(&cuMemExportToShareableHandle) f_export = nullptr;
  decltype(&cuMemImportFromShareableHandle) f_import = nullptr;
  CUmemAllocationProp prop{};
  explicit CudaVmmBackend(int dev) : device(dev) {
    f_create = DRV(cuMemCreate); f_release = DRV(cuMemRelease); f_reserve = DRV(cuMemAddressReserve);
    f_free = DRV(cuMemAddressFree); f_map = DRV(cuMemMap); f_unmap = DRV(cuMemUnmap);
    f_access = DRV(cuMemSetAccess); f_gran = DRV(cuMemGetAllocationGranularity);
    f_export = DRV(cuMemExportToShareableHandle); f_import = DRV(cuMemImportFromShareableHandle);
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
  void set_shareable(bool on) override {
    prop.requestedHandleTypes = on ? CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR : CU_MEM_HANDLE_TYPE_NONE;
  }
  int export_fds(const std::vector<uint64_t>& handles, std::vector<int>* fds) override {
    SRT_REQUIRE(f_export != nullptr, "page pool: cuMemExportToShareableHandle is not available");
    for (uint64_t h : handles) {
      int fd = -1;
      CU_CALL(f_export(&fd, (CUmemGenericAllocationHandle)h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
      fds->push_back(fd);
    }
    return SRT_OK;
  }
  int import_fds(const std::vector<int>& fds, size_t n_pages, size_t, std::vector<uint64_t>* handles) override {
    SRT_REQUIRE(f_import != nullptr, "page pool: cuMemImportFromShareableHandle is not available");
    SRT_REQUIRE(fds.size() == n_pages, "page pool: got %zu page descriptors for %zu pages", fds.size(), n_pages);
    for (int fd : fds) {
      CUmemGenericAllocationHandle h;
      CU_CALL(f_import(&h, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
      handles->push_back((uint64_t)h);
    }
    return SRT_OK;
  }
};

// Host stand-in: the pool is one memfd, page i is its bytes [i * page, (i + 1) * page); mapping a slot is a
// shared mmap of that window over the reserved range, so two processes that map the same page see the same bytes.
struct HostBackend : Backend {
  int memfd = -1;
  size_t created = 0, page = 0;
  ~HostBackend() override { if (memfd >= 0) close(memfd); }
  int granularity(size_t* out) override { *out = 2u << 20; return SRT_OK; }
  int reserve(size_t bytes, uint64_t* base) override {
    void* p = mmap(nullptr, bytes, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE, -1, 0);
    if (p == MAP_FAILED) { set_error("host backend: mmap of %zu bytes failed", bytes); return SRT_ERR_NOMEM; }
    *base = (uint64_t)(uintptr_t)p;
    return SRT_OK;
  }
  int unreserve(uint64_t base, size_t bytes) override { munmap((void*)(uintptr_t)base, bytes); return SRT_OK; }
  int create_page(size_t bytes, uint64_t* handle) override {
    if (memfd < 0) {
      memfd = memfd_create("srt_pool_pages", MFD_CLOEXEC);
      if (memfd < 0) { set_error("host backend: memfd_create failed"); return SRT_ERR_NOMEM; }
      page = bytes;
    }
    if (ftruncate(memfd, (off_t)((created + 1) * page)) != 0) { set_error("host backend: ftruncate failed"); return SRT_ERR_NOMEM; }
    *handle = created++;
    return SRT_OK;
  }
  int release_page(uint64_t) override { return SRT_OK; }
  int map(uint64_t va, size_t bytes, uint64_t handle) override {
    void* r = mmap((void*)(uintptr_t)va, bytes, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_FIXED, memfd, (off_t)(handle * page));
    if (r == MAP_FAILED) { set_error("host backend: mapping a page failed"); return SRT_ERR_STATE; }
    return SRT_OK;
  }
  int allow(uint64_t, size_t) override { return SRT_OK; }
  int unmap(uint64_t va, size_t bytes, size_t) override {
    void* r = mmap((void*)(uintptr_t)va, bytes, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE | MAP_FIXED, -1, 0);
    if (r == MAP_FAILED) { set_error("host backend: unmapping a page failed"); return SRT_ERR_STATE; }
    return SRT_OK;
  }
  int export_fds(const std::vector<uint64_t>&, std::vector<int>* fds) override {
    int fd = dup(memfd);
    SRT_REQUIRE(fd >= 0, "host backend: dup of the page file failed");
    fds->push_back(fd);
    return SRT_OK;
  }
  int import_fds(const std::vector<int>& fds, size_t n_pages, size_t page_bytes, std::vector<uint64_t>* handles) override {
    SRT_REQUIRE(fds.size() == 1, "host backend: expected one descriptor, got %zu", fds.size());
    memfd = dup(fds[0]);
    SRT_REQUIRE(memfd >= 0, "host backend: dup of the page file failed");
    page = page_bytes;
    created = n_pages;
    for (size_t i = 0; i < n_pages; ++i) handles->push_back(i);
    return SRT_OK;
  }
};

// State both sides of a shared pool see. A private pool keeps the same struct on the heap.
struct Shared {
  uint64_t magic;
  uint64_t nonce;          // names this incarnation of the pool: handed out with the page descriptors
  uint32_t ready;
  int32_t backend, device, unmap_on_release;
  uint64_t page_bytes, n_pages;
  int32_t train_va_scale, infer_va_scale;
  pthread_mutex_t mu;
  std::atomic<int> infer_waiting;
  uint64_t free_pages;
  uint64_t mapped_pages[3], allocated[3], peak[3];  // by owner (Belong)
  long long n_map, n_unmap, n_reuse;
  int32_t belong[1];       // n_pages entries
};
constexpr uint64_t kPoolMagic = 0x5352545f504f4f4cull;  // "SRT_POOL"
inline size_t shared_bytes(size_t n_pages) { return sizeof(Shared) + n_pages * sizeof(int32_t); }

void shared_mutex_init(pthread_mutex_t* m, bool process_shared) {
  pthread_mutexattr_t a;
  pthread_mutexattr_init(&a);
  if (process_shared) {
    pthread_mutexattr_setpshared(&a, PTHREAD_PROCESS_SHARED);
    pthread_mutexattr_setrobust(&a, PTHREAD_MUTEX_ROBUST);
  }
  pthread_mutex_init(m, &a);
  pthread_mutexattr_destroy(&a);
}

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
  std::map<uint64_t, uint64_t> hollow_;  // offset -> length of blocks whose memory was given up while their owner
                                         // still holds the address: the range is not handed out again until the
                                         // owner frees it, but counts as free space when pages are released
  size_t allocated = 0, peak = 0, mapped_pages = 0;
  size_t align = 512;
};

struct Pool {
  Shared* sh = nullptr;           // heap (private pool) or the mapped shared segment
  bool shared = false, creator = true;
  std::string name;               // shared pools: segment "/<name>", socket "\0srt_pool.<name>"
  size_t sh_bytes = 0;
  int listen_fd = -1;
  std::thread server;             // creator of a shared pool: hands the page descriptors to attaching processes
  std::atomic<bool> stop{false};
  Backend* be = nullptr;
  int device = 0;
  size_t page_bytes = 0, n_pages = 0;
  std::vector<uint64_t> pages;    // physical handles (this process's)
  Allocator train, infer;
  srt_pool_oom_fn oom = nullptr;
  void* oom_user = nullptr;
  std::mutex oom_mu;
  bool unmap_on_release = false;
  ~Pool() {
    stop.store(true);
    if (listen_fd >= 0) { shutdown(listen_fd, SHUT_RDWR); close(listen_fd); }
    if (server.joinable()) server.join();
    if (be) {
      for (Allocator* a : {&train, &infer}) {
        if (!a->base) continue;
        // pages this process still holds go back to the pool: the other side may outlive it
        if (sh && shared) {
          pthread_mutex_lock(&sh->mu);
          for (size_t s = 0; s < a->slots; ++s)
            if (a->slot_page[s] >= 0) { sh->belong[a->slot_page[s]] = 0; sh->free_pages++; }
          sh->mapped_pages[a->who] -= a->mapped_pages;
          sh->allocated[a->who] -= a->allocated;
          pthread_mutex_unlock(&sh->mu);
        }
        for (size_t s = 0; s < a->slots; ++s)
          if (a->slot_page[s] >= 0 || a->kept_page[s] >= 0) be->unmap(a->base + s * page_bytes, page_bytes, page_bytes);
        be->unreserve(a->base, a->slots * page_bytes);
      }
      for (uint64_t h : pages) be->release_page(h);
      delete be;
    }
    if (sh) {
      if (shared) {
        munmap(sh, sh_bytes);
        if (creator) shm_unlink(("/" + name).c_str());
      } else {
        pthread_mutex_destroy(&sh->mu);
        free(sh);
      }
    }
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
    if (p.sh->belong[i] == kFree) { p.sh->belong[i] = who; p.sh->free_pages--; *page = (int)i; return SRT_OK; }
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
    if (kept >= 0 && p.sh->belong[kept] == kFree) {
      // the slot is still mapped to a page that is free again: take it back without touching the driver
      p.sh->belong[kept] = a.who;
      p.sh->free_pages--;
      a.slot_page[s] = kept;
      a.kept_page[s] = -1;
      a.mapped_pages++;
      p.sh->mapped_pages[a.who]++;
      p.sh->n_reuse++;
      int rc = flush();
      if (rc) return rc;
      continue;
    }
    int page;
    int rc = take_free_page(p, a.who, &page);
    if (rc) { flush(); return rc; }
    if (kept >= 0) {  // mapped to a page that now serves someone else: drop that mapping first
      int r2 = p.be->unmap(a.base + s * p.page_bytes, p.page_bytes, p.page_bytes);
      if (r2) { p.sh->belong[page] = kFree; p.sh->free_pages++; flush(); return r2; }
      a.kept_page[s] = -1;
      p.sh->n_unmap++;
    }
    rc = p.be->map(a.base + s * p.page_bytes, p.page_bytes, p.pages[page]);
    if (rc) { p.sh->belong[page] = kFree; p.sh->free_pages++; flush(); return rc; }
    a.slot_page[s] = page;
    a.mapped_pages++;
    p.sh->mapped_pages[a.who]++;
    p.sh->n_map++;
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
  if (best_pages > p.sh->free_pages) {
    set_error("allocator: needs %zu more pages, pool has %zu free", best_pages, p.sh->free_pages);
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
  p.sh->allocated[a.who] += need;
  p.sh->peak[a.who] = std::max(p.sh->peak[a.who], p.sh->allocated[a.who]);
  *out = a.base + off;
  return SRT_OK;
}

int free_locked(Pool& p, Allocator& a, uint64_t ptr) {
  SRT_REQUIRE(ptr >= a.base && ptr < a.base + a.slots * p.page_bytes, "allocator: pointer %#llx is not from this allocator",
              (unsigned long long)ptr);
  auto hit = a.hollow_.find(ptr - a.base);
  if (hit != a.hollow_.end()) {  // the owner lets go of an address whose memory went back earlier
    const uint64_t off = hit->first, len = hit->second;
    a.hollow_.erase(hit);
    free_insert(a, off, len);
    return SRT_OK;
  }
  auto it = a.live_.find(ptr - a.base);
  SRT_REQUIRE(it != a.live_.end(), "allocator: double free or unknown block %#llx", (unsigned long long)ptr);
  const uint64_t off = it->first, len = it->second;
  a.live_.erase(it);
  a.allocated -= len;
  p.sh->allocated[a.who] -= len;
  free_insert(a, off, len);
  return SRT_OK;
}

// Gives up the memory of a live block but keeps its address range out of circulation.
int hollow_locked(Pool& p, Allocator& a, uint64_t ptr) {
  SRT_REQUIRE(ptr >= a.base && ptr < a.base + a.slots * p.page_bytes, "allocator: pointer %#llx is not from this allocator",
              (unsigned long long)ptr);
  auto it = a.live_.find(ptr - a.base);
  SRT_REQUIRE(it != a.live_.end(), "allocator: unknown block %#llx", (unsigned long long)ptr);
  a.hollow_[it->first] = it->second;
  a.allocated -= it->second;
  p.sh->allocated[a.who] -= it->second;
  a.live_.erase(it);
  return SRT_OK;
}

// Unmap every mapped slot that lies wholly inside free space (free ranges and hollow blocks together) and give
// its page back to the pool.
int empty_cache_locked(Pool& p, Allocator& a, size_t* released_pages) {
  size_t n = 0;
  std::vector<std::pair<uint64_t, uint64_t>> spans;  // [begin, end), sorted, adjacent ones merged
  {
    auto f = a.free_.begin();
    auto h = a.hollow_.begin();
    while (f != a.free_.end() || h != a.hollow_.end()) {
      const bool take_f = h == a.hollow_.end() || (f != a.free_.end() && f->first < h->first);
      const uint64_t b = take_f ? f->first : h->first, e = b + (take_f ? f->second : h->second);
      if (take_f) ++f; else ++h;
      if (!spans.empty() && spans.back().second == b) spans.back().second = e;
      else spans.emplace_back(b, e);
    }
  }
  for (auto& fr : spans) {
    const uint64_t b = fr.first, e = fr.second;
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
        p.sh->belong[a.slot_page[s]] = kFree;
        p.sh->free_pages++;
        if (p.unmap_on_release) p.sh->n_unmap++;
        else a.kept_page[s] = a.slot_page[s];
        a.slot_page[s] = -1;
        a.mapped_pages--;
        p.sh->mapped_pages[a.who]--;
        ++n;
      }
    }
  }
  if (released_pages) *released_pages = n;
  return SRT_OK;
}

Allocator* pick(Pool* p, int kind) { return kind == SRT_POOL_INFER ? &p->infer : &p->train; }

// Takes the pool lock with the inference-first rule. The wait of a training caller is bounded (50 ms)
// so a stuck inference thread cannot stall training for good. The lock lives in the shared block: in a
// shared pool it is process-shared and robust (a holder that died leaves plain data behind).
struct PoolLock {
  Pool* p;
  bool held = false;
  PoolLock(Pool* pool, int kind) : p(pool) {
    if (kind == SRT_POOL_INFER) {
      p->sh->infer_waiting.fetch_add(1, std::memory_order_acq_rel);
      lock();
      p->sh->infer_waiting.fetch_sub(1, std::memory_order_acq_rel);
    } else {
      const auto give_up = std::chrono::steady_clock::now() + std::chrono::milliseconds(50);
      while (p->sh->infer_waiting.load(std::memory_order_acquire) > 0 && std::chrono::steady_clock::now() < give_up)
        std::this_thread::yield();
      lock();
    }
  }
  ~PoolLock() { unlock(); }
  void lock() {
    if (pthread_mutex_lock(&p->sh->mu) == EOWNERDEAD) pthread_mutex_consistent(&p->sh->mu);
    held = true;
  }
  void unlock() {
    if (held) pthread_mutex_unlock(&p->sh->mu);
    held = false;
  }
};

// ---- handing the page descriptors to another process ------------------------------------------------
struct FdHello { uint64_t magic, nonce, n_fds; };

sockaddr_un pool_sockaddr(const std::string& name, socklen_t* len) {
  sockaddr_un a{};
  a.sun_family = AF_UNIX;
  const std::string path = "srt_pool." + name;   // abstract namespace: vanishes with the creating process
  const size_t n = std::min(path.size(), sizeof(a.sun_path) - 2);
  memcpy(a.sun_path + 1, path.data(), n);
  *len = (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + n);
  return a;
}

int send_fds(int sock, const int* fds, int n) {
  char byte = 'F';
  iovec iov{&byte, 1};
  std::vector<char> ctl(CMSG_SPACE(sizeof(int) * n));
  msghdr msg{};
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctl.data();
  msg.msg_controllen = ctl.size();
  cmsghdr* c = CMSG_FIRSTHDR(&msg);
  c->cmsg_level = SOL_SOCKET;
  c->cmsg_type = SCM_RIGHTS;
  c->cmsg_len = CMSG_LEN(sizeof(int) * n);
  memcpy(CMSG_DATA(c), fds, sizeof(int) * n);
  return sendmsg(sock, &msg, MSG_NOSIGNAL) == 1 ? 0 : -1;
}

int recv_fds(int sock, std::vector<int>* out, int max_n) {
  char byte;
  iovec iov{&byte, 1};
  std::vector<char> ctl(CMSG_SPACE(sizeof(int) * max_n));
  msghdr msg{};
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctl.data();
  msg.msg_controllen = ctl.size();
  if (recvmsg(sock, &msg, MSG_CMSG_CLOEXEC) != 1) return -1;
  for (cmsghdr* c = CMSG_FIRSTHDR(&msg); c; c = CMSG_NXTHDR(&msg, c)) {
    if (c->cmsg_level != SOL_SOCKET || c->cmsg_type != SCM_RIGHTS) continue;
    const int n = (int)((c->cmsg_len - CMSG_LEN(0)) / sizeof(int));
    const int* f = (const int*)CMSG_DATA(c);
    out->insert(out->end(), f, f + n);
  }
  return 0;
}

constexpr int kFdBatch = 64;

void serve_descriptors(Pool* p) {
  while (!p->stop.load()) {
    pollfd pf{p->listen_fd, POLLIN, 0};
    if (poll(&pf, 1, 100) <= 0) continue;
    const int c = accept4(p->listen_fd, nullptr, nullptr, SOCK_CLOEXEC);
    if (c < 0) continue;
    std::vector<int> fds;
    if (p->be->export_fds(p->pages, &fds) == SRT_OK) {
      FdHello h{kPoolMagic, p->sh->nonce, (uint64_t)fds.size()};
      bool ok = send(c, &h, sizeof(h), MSG_NOSIGNAL) == (ssize_t)sizeof(h);
      for (size_t o = 0; ok && o < fds.size(); o += kFdBatch)
        ok = send_fds(c, fds.data() + o, (int)std::min<size_t>(kFdBatch, fds.size() - o)) == 0;
    }
    for (int fd : fds) close(fd);
    close(c);
  }
}

int build_allocators(Pool* p, int scale_t, int scale_i) {
  struct { Allocator* a; Belong who; int scale; size_t align; } defs[2] = {
      {&p->train, kTrain, scale_t, 1024}, {&p->infer, kInfer, scale_i, 512}};
  for (auto& d : defs) {
    d.a->pool = p;
    d.a->who = d.who;
    d.a->slots = p->n_pages * (size_t)d.scale;
    d.a->align = d.align;
    int rc = p->be->reserve(d.a->slots * p->page_bytes, &d.a->base);
    if (rc) return rc;
    d.a->slot_page.assign(d.a->slots, -1);
    d.a->kept_page.assign(d.a->slots, -1);
    d.a->free_[0] = d.a->slots * p->page_bytes;
  }
  return SRT_OK;
}

int make_backend(Pool* p, int backend, int device) {
  if (backend == SRT_POOL_BACKEND_HOST) {
    p->be = new HostBackend();
    return SRT_OK;
  }
  SRT_CHECK_CUDA(cudaSetDevice(device));
  SRT_CHECK_CUDA(cudaFree(0));  // make sure the primary context exists
  CudaVmmBackend* b = new CudaVmmBackend(device);
  if (!b->ok()) { delete b; set_error("page pool: CUDA VMM driver entry points unavailable"); return SRT_ERR_UNSUPPORTED; }
  p->be = b;
  return SRT_OK;
}

int create_pool(const srt_pool_config* cfg, const char* shared_name, srt_pool** out) {
  SRT_REQUIRE(cfg && out, "pool_create: null argument");
  SRT_REQUIRE(cfg->pool_nbytes > 0, "pool_create: pool_nbytes must be positive");
  Pool* p = new Pool();
  p->device = cfg->device;
  p->unmap_on_release = cfg->unmap_on_release != 0;
  p->shared = shared_name != nullptr;
  if (p->shared) p->name = shared_name;
  int rc = make_backend(p, cfg->backend, cfg->device);
  if (rc) { delete p; return rc; }
  p->be->set_shareable(p->shared);
  size_t gran = 0;
  rc = p->be->granularity(&gran);
  if (rc) { delete p; return rc; }
  size_t page = cfg->page_nbytes ? cfg->page_nbytes : (32u << 20);  // CUDAMemPool::PageNbytes() = 32 MiB
  page = (page + gran - 1) / gran * gran;
  p->page_bytes = page;
  p->n_pages = cfg->pool_nbytes / page;
  if (p->n_pages == 0) { delete p; set_error("pool_create: pool smaller than one page"); return SRT_ERR_INVALID; }
  // the shared block: page ownership, counters, lock
  p->sh_bytes = shared_bytes(p->n_pages);
  if (p->shared) {
    // the socket first: binding it proves no live pool has the name, before the old segment is touched
    p->listen_fd = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
    socklen_t alen;
    sockaddr_un addr = pool_sockaddr(p->name, &alen);
    if (p->listen_fd < 0 || bind(p->listen_fd, (sockaddr*)&addr, alen) != 0 || listen(p->listen_fd, 16) != 0) {
      delete p;
      set_error("pool_create: cannot listen on the pool's socket (is a pool named %s alive already?)", shared_name);
      return SRT_ERR_STATE;
    }
    const std::string seg = "/" + p->name;
    shm_unlink(seg.c_str());  // a segment left by a crashed owner; nobody can reach it any more (see attach)
    const int fd = shm_open(seg.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
    if (fd < 0 || ftruncate(fd, (off_t)p->sh_bytes) != 0) {
      if (fd >= 0) close(fd);
      delete p;
      set_error("pool_create: cannot create the shared segment %s", seg.c_str());
      return SRT_ERR_STATE;
    }
    void* m = mmap(nullptr, p->sh_bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    close(fd);
    if (m == MAP_FAILED) { delete p; set_error("pool_create: cannot map the shared segment"); return SRT_ERR_STATE; }
    p->sh = (Shared*)m;
    memset((void*)p->sh, 0, p->sh_bytes);
  } else {
    p->sh = (Shared*)calloc(1, p->sh_bytes);
  }
  Shared* sh = p->sh;
  shared_mutex_init(&sh->mu, p->shared);
  new (&sh->infer_waiting) std::atomic<int>(0);
  sh->backend = cfg->backend; sh->device = cfg->device; sh->unmap_on_release = cfg->unmap_on_release;
  sh->page_bytes = page; sh->n_pages = p->n_pages;
  sh->train_va_scale = cfg->train_va_scale > 0 ? cfg->train_va_scale : 8;   // cuda_allocator.cc: va_range_scale 8
  sh->infer_va_scale = cfg->infer_va_scale > 0 ? cfg->infer_va_scale : 1;
  sh->free_pages = p->n_pages;
  p->pages.reserve(p->n_pages);
  for (size_t i = 0; i < p->n_pages; ++i) {
    uint64_t h;
    rc = p->be->create_page(page, &h);
    if (rc) { delete p; return rc; }
    p->pages.push_back(h);
  }
  rc = build_allocators(p, sh->train_va_scale, sh->infer_va_scale);
  if (rc) { delete p; return rc; }
  if (p->shared) {
    timespec ts;
    clock_gettime(CLOCK_REALTIME, &ts);
    sh->nonce = ((uint64_t)getpid() << 32) ^ (uint64_t)ts.tv_nsec ^ ((uint64_t)ts.tv_sec << 20);
    sh->magic = kPoolMagic;
    __atomic_store_n(&sh->ready, 1u, __ATOMIC_RELEASE);
    p->server = std::thread(serve_descriptors, p);
  }
  *out = (srt_pool*)p;
  return SRT_OK;
}

}  // namespace
}  // namespace srt

using namespace srt;

extern "C" {

int srt_pool_create(const srt_pool_config* cfg, srt_pool** out) { return create_pool(cfg, nullptr, out); }

int srt_pool_create_shared(const srt_pool_config* cfg, const char* name, srt_pool** out) {
  SRT_REQUIRE(name && *name && strlen(name) < 80 && !strchr(name, '/'), "pool_create_shared: bad name");
  return create_pool(cfg, name, out);
}

int srt_pool_attach(const char* name, int device, int timeout_ms, srt_pool** out) {
  SRT_REQUIRE(name && *name && strlen(name) < 80 && !strchr(name, '/') && out, "pool_attach: bad argument");
  // 1. the owner's socket: exists only while the owning process lives, so a segment left behind by a crashed
  //    owner is never mistaken for a live pool; it also tells which incarnation of the segment to expect
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms > 0 ? timeout_ms : 0);
  int sock = -1;
  for (;;) {
    sock = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
    socklen_t alen;
    sockaddr_un addr = pool_sockaddr(name, &alen);
    if (sock >= 0 && connect(sock, (sockaddr*)&addr, alen) == 0) break;
    if (sock >= 0) close(sock);
    sock = -1;
    if (std::chrono::steady_clock::now() >= deadline) {
      set_error("pool_attach: no live pool named %s (its owner is not listening)", name);
      return SRT_ERR_STATE;
    }
    std::this_thread::sleep_for(std::chrono::milliseconds(5));
  }
  FdHello hello{};
  std::vector<int> fds;
  bool ok = recv(sock, &hello, sizeof(hello), MSG_WAITALL) == (ssize_t)sizeof(hello) && hello.magic == kPoolMagic;
  while (ok && fds.size() < hello.n_fds) ok = recv_fds(sock, &fds, kFdBatch) == 0;
  close(sock);
  auto close_all = [&] { for (int fd : fds) close(fd); };
  if (!ok || fds.size() != hello.n_fds) {
    close_all();
    set_error("pool_attach: the owner of %s did not send its page descriptors", name);
    return SRT_ERR_STATE;
  }
  // 2. the segment of that incarnation
  Pool* p = new Pool();
  p->shared = true;
  p->creator = false;
  p->name = name;
  const std::string seg = std::string("/") + name;
  const int fd = shm_open(seg.c_str(), O_RDWR, 0600);
  struct stat st{};
  if (fd < 0 || fstat(fd, &st) != 0 || (size_t)st.st_size < sizeof(Shared)) {
    if (fd >= 0) close(fd);
    close_all();
    delete p;
    set_error("pool_attach: cannot open the shared segment %s", seg.c_str());
    return SRT_ERR_STATE;
  }
  p->sh_bytes = (size_t)st.st_size;
  void* m = mmap(nullptr, p->sh_bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (m == MAP_FAILED) { close_all(); delete p; set_error("pool_attach: cannot map the shared segment"); return SRT_ERR_STATE; }
  p->sh = (Shared*)m;
  Shared* sh = p->sh;
  if (__atomic_load_n(&sh->ready, __ATOMIC_ACQUIRE) != 1u || sh->magic != kPoolMagic || sh->nonce != hello.nonce ||
      shared_bytes(sh->n_pages) > p->sh_bytes) {
    close_all();
    delete p;
    set_error("pool_attach: segment %s does not belong to the pool that answered (stale segment?)", seg.c_str());
    return SRT_ERR_STATE;
  }
  p->device = device;
  p->unmap_on_release = sh->unmap_on_release != 0;
  p->page_bytes = sh->page_bytes;
  p->n_pages = sh->n_pages;
  int rc = make_backend(p, sh->backend, device);
  if (rc == SRT_OK) rc = p->be->import_fds(fds, p->n_pages, p->page_bytes, &p->pages);
  close_all();
  if (rc == SRT_OK) rc = build_allocators(p, sh->train_va_scale, sh->infer_va_scale);
  if (rc) { delete p; return rc; }
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
  uint64_t ptr = 0;
  int rc = alloc_locked(*p, *pick(p, kind), nbytes, &ptr);
  if (rc == SRT_ERR_NOMEM) {
    // the reference notifies OOM observers before failing (common/cuda_allocator.cc:311-328)
    srt_pool_oom_fn fn;
    void* user;
    { std::lock_guard<std::mutex> lk(p->oom_mu); fn = p->oom; user = p->oom_user; }
    if (fn) {
      guard.unlock();
      fn(user, kind, nbytes);
      guard.lock();
      rc = alloc_locked(*p, *pick(p, kind), nbytes, &ptr);
    }
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

int srt_pool_hollow(srt_pool* h, int kind, void* ptr) {
  Pool* p = (Pool*)h;
  SRT_REQUIRE(p && ptr, "pool_hollow: bad argument");
  PoolLock guard(p, kind);
  return hollow_locked(*p, *pick(p, kind), (uint64_t)(uintptr_t)ptr);
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

// Usage figures come from the shared block, so either process sees both sides (the server reads the trainer's
// footprint, cuda_allocator.cc:259-302).
int64_t srt_pool_stat(srt_pool* h, int which) {
  Pool* p = (Pool*)h;
  if (!p) return -1;
  PoolLock guard(p, SRT_POOL_INFER);
  const Shared* sh = p->sh;
  switch (which) {
    case SRT_POOL_STAT_INFER_USAGE: return (int64_t)(sh->mapped_pages[kInfer] * p->page_bytes);
    case SRT_POOL_STAT_TRAIN_USAGE: return (int64_t)sh->allocated[kTrain];
    case SRT_POOL_STAT_TRAIN_PEAK: return (int64_t)sh->peak[kTrain];
    case SRT_POOL_STAT_TRAIN_ALL: return (int64_t)(sh->mapped_pages[kTrain] * p->page_bytes);
    case SRT_POOL_STAT_FREE_PAGES: return (int64_t)sh->free_pages;
    case SRT_POOL_STAT_POOL_NBYTES: return (int64_t)(p->n_pages * p->page_bytes);
    case SRT_POOL_STAT_PAGE_NBYTES: return (int64_t)p->page_bytes;
    case SRT_POOL_STAT_NUM_MAP: return (int64_t)sh->n_map;
    case SRT_POOL_STAT_NUM_UNMAP: return (int64_t)sh->n_unmap;
    case SRT_POOL_STAT_INFER_ALLOCATED: return (int64_t)sh->allocated[kInfer];
    case SRT_POOL_STAT_NUM_REUSE: return (int64_t)sh->n_reuse;
    default: return -1;
  }
}

int srt_pool_set_oom_handler(srt_pool* h, srt_pool_oom_fn fn, void* user) {
  Pool* p = (Pool*)h;
  SRT_REQUIRE(p, "pool_set_oom_handler: null pool");
  std::lock_guard<std::mutex> lk(p->oom_mu);
  p->oom = fn;
  p->oom_user = user;
  return SRT_OK;
}

}  // extern "C"
