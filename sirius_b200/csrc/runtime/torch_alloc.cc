// The PyTorch allocator seam: raw alloc / free entry points with the signature of
// torch.cuda.memory.CUDAPluggableAllocator, on top of the training allocator of the page pool.
//
// The reference installs a C++ subclass of c10::cuda::CUDACachingAllocator::CUDAAllocator whose
// raw_alloc_with_stream / raw_delete go to CUDAMemPool, whose recordStream defers a block's reuse until the
// streams that used it have caught up, and which remembers the intermediate (saved-for-backward) tensors so
// that an adjust can drop them all at once (pytorch/torch_col/csrc/torch_allocator_plugin.cc:108-178 alloc and
// free, :200-229 recordStream, :322-375 tagging and ReleaseIntermMemory, :383-412 ProcessEvents). Here the same
// behaviour sits behind plain C functions, so any PyTorch can load it without a fork:
//
//   torch.cuda.memory.change_current_allocator(
//       torch.cuda.memory.CUDAPluggableAllocator(libsirius_b200.so, "srt_alloc", "srt_free"))
//
// One default pool per device and process, made by srt_pool_init: created here, or attached to the pool a
// server process created under the same name (COLTRAIN_HAS_SHARED_TENSOR_SERVER=1). Every entry point returns
// a status and never aborts; srt_alloc, whose signature has no room for one, returns NULL and leaves the
// message in srt_last_error().
#include <map>
#include <mutex>
#include <set>
#include <string>
#include <vector>

#include "../../../include/sirius_pool.h"
#include "../../../include/sirius_runtime.h"
#include "rt_common.h"

namespace srt {
namespace {

struct Block {
  size_t nbytes = 0;
  cudaStream_t alloc_stream = nullptr;
  std::set<cudaStream_t> used_on;  // streams recorded with srt_record_stream (other than alloc_stream)
  bool tagged = false;             // an intermediate tensor: srt_release_interm frees it
};

struct Pending {  // a freed block some stream may still be using
  void* ptr;
  std::vector<cudaEvent_t> events;
};

struct DeviceState {
  srt_pool* pool = nullptr;
  bool owns_pool = false;
  std::map<void*, Block> live;
  std::set<void*> dropped;         // released by srt_release_interm while the framework still holds the pointer
  std::vector<Pending> pending;
  long long n_alloc = 0, n_free = 0, n_deferred = 0;
};

std::mutex g_mu;                   // order: this, then the pool's own lock (as interm_memory_mutex_ -> entry_mutex_)
DeviceState g_dev[SRT_MAX_DEVICE_NUM];
bool g_in_model_setup = false;     // between tag_model_begin and tag_model_end: parameters, never intermediates

std::string pool_name(int device) { return default_shm_prefix() + "_pool_dev" + std::to_string(device); }

// Frees the pending blocks whose recorded streams have all passed the point of the free.
void process_events(DeviceState& d) {
  for (size_t i = 0; i < d.pending.size();) {
    Pending& p = d.pending[i];
    bool done = true;
    for (cudaEvent_t e : p.events)
      if (cudaEventQuery(e) == cudaErrorNotReady) { done = false; break; }
    if (!done) { ++i; continue; }
    for (cudaEvent_t e : p.events) cudaEventDestroy(e);
    srt_pool_free(d.pool, SRT_POOL_TRAIN, p.ptr);
    d.pending.erase(d.pending.begin() + (long)i);
  }
}

int free_block(DeviceState& d, void* ptr, const Block& b) {
  if (b.used_on.empty()) return srt_pool_free(d.pool, SRT_POOL_TRAIN, ptr);
  Pending p{ptr, {}};
  for (cudaStream_t s : b.used_on) {
    cudaEvent_t e;
    SRT_CHECK_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    SRT_CHECK_CUDA(cudaEventRecord(e, s));
    p.events.push_back(e);
  }
  d.pending.push_back(p);
  d.n_deferred++;
  return SRT_OK;
}

}  // namespace
}  // namespace srt

using namespace srt;

extern "C" {

int srt_pool_init(int device, size_t nbytes, int cleanup) {
  SRT_REQUIRE(device >= 0 && device < SRT_MAX_DEVICE_NUM, "pool_init: bad device %d", device);
  std::lock_guard<std::mutex> lk(g_mu);
  DeviceState& d = g_dev[device];
  if (d.pool) return SRT_OK;
  const char* has_server = getenv("COLTRAIN_HAS_SHARED_TENSOR_SERVER");
  const std::string name = pool_name(device);
  if (has_server && atoi(has_server) != 0 && !cleanup) {
    // the inference server made the pool; this trainer opens it
    int rc = srt_pool_attach(name.c_str(), device, 30000, &d.pool);
    if (rc) return rc;
  } else {
    SRT_REQUIRE(nbytes > 0, "pool_init: pool size must be positive");
    srt_pool_config cfg{};
    cfg.device = device;
    cfg.backend = getenv("SIRIUS_B200_POOL_HOST_BACKEND") ? SRT_POOL_BACKEND_HOST : SRT_POOL_BACKEND_CUDA_VMM;
    cfg.pool_nbytes = nbytes;
    if (const char* pg = getenv("SIRIUS_B200_POOL_PAGE_MB")) cfg.page_nbytes = (size_t)atoi(pg) << 20;
    if (const char* um = getenv("SIRIUS_B200_POOL_UNMAP_ON_RELEASE")) cfg.unmap_on_release = atoi(um) != 0;  // the reference's unmap-at-release
    int rc = srt_pool_create_shared(&cfg, name.c_str(), &d.pool);
    if (rc) return rc;
  }
  d.owns_pool = true;
  return SRT_OK;
}

int srt_pool_shutdown(int device) {
  SRT_REQUIRE(device >= 0 && device < SRT_MAX_DEVICE_NUM, "pool_shutdown: bad device %d", device);
  std::lock_guard<std::mutex> lk(g_mu);
  DeviceState& d = g_dev[device];
  if (!d.pool) return SRT_OK;
  for (Pending& p : d.pending) {
    for (cudaEvent_t e : p.events) { cudaEventSynchronize(e); cudaEventDestroy(e); }
    srt_pool_free(d.pool, SRT_POOL_TRAIN, p.ptr);
  }
  d.pending.clear();
  d.live.clear();
  d.dropped.clear();
  if (d.owns_pool) srt_pool_destroy(d.pool);
  d.pool = nullptr;
  return SRT_OK;
}

int srt_pool_default(int device, srt_pool** out) {
  SRT_REQUIRE(device >= 0 && device < SRT_MAX_DEVICE_NUM && out, "pool_default: bad argument");
  std::lock_guard<std::mutex> lk(g_mu);
  SRT_REQUIRE(g_dev[device].pool != nullptr, "pool_default: srt_pool_init was not called for device %d", device);
  *out = g_dev[device].pool;
  return SRT_OK;
}

void* srt_alloc(size_t nbytes, int device, void* stream) {
  if (nbytes == 0) return nullptr;
  if (device < 0 || device >= SRT_MAX_DEVICE_NUM) { set_error("srt_alloc: bad device %d", device); return nullptr; }
  std::lock_guard<std::mutex> lk(g_mu);
  DeviceState& d = g_dev[device];
  if (!d.pool) { set_error("srt_alloc: srt_pool_init was not called for device %d", device); return nullptr; }
  process_events(d);
  void* p = nullptr;
  int rc = srt_pool_alloc(d.pool, SRT_POOL_TRAIN, nbytes, &p);
  if (rc == SRT_ERR_NOMEM && !d.pending.empty()) {
    // blocks waiting for their streams are the only memory left: wait for them, as the reference's allocator
    // synchronises and retries before it gives up
    for (Pending& q : d.pending)
      for (cudaEvent_t e : q.events) cudaEventSynchronize(e);
    process_events(d);
    rc = srt_pool_alloc(d.pool, SRT_POOL_TRAIN, nbytes, &p);
  }
  if (rc) return nullptr;
  Block b;
  b.nbytes = nbytes;
  b.alloc_stream = (cudaStream_t)stream;
  d.live[p] = b;
  d.n_alloc++;
  return p;
}

void srt_free(void* ptr, size_t /*nbytes*/, int device, void* /*stream*/) {
  if (!ptr || device < 0 || device >= SRT_MAX_DEVICE_NUM) return;
  std::lock_guard<std::mutex> lk(g_mu);
  DeviceState& d = g_dev[device];
  if (!d.pool) return;
  if (d.dropped.erase(ptr)) {  // its memory went back with srt_release_interm; now the address does too
    srt_pool_free(d.pool, SRT_POOL_TRAIN, ptr);
    return;
  }
  auto it = d.live.find(ptr);
  if (it == d.live.end()) { set_error("srt_free: %p was not allocated by srt_alloc", ptr); return; }
  Block b = it->second;
  d.live.erase(it);
  d.n_free++;
  free_block(d, ptr, b);
  process_events(d);
}

int srt_record_stream(void* ptr, int device, void* stream) {
  SRT_REQUIRE(device >= 0 && device < SRT_MAX_DEVICE_NUM, "record_stream: bad device %d", device);
  std::lock_guard<std::mutex> lk(g_mu);
  DeviceState& d = g_dev[device];
  auto it = d.live.find(ptr);
  SRT_REQUIRE(it != d.live.end(), "record_stream: %p is not a live block", ptr);
  if ((cudaStream_t)stream != it->second.alloc_stream) it->second.used_on.insert((cudaStream_t)stream);
  return SRT_OK;
}

int srt_empty_cache(int device, size_t* released_bytes) {
  SRT_REQUIRE(device >= 0 && device < SRT_MAX_DEVICE_NUM, "empty_cache: bad device %d", device);
  std::lock_guard<std::mutex> lk(g_mu);
  DeviceState& d = g_dev[device];
  SRT_REQUIRE(d.pool != nullptr, "empty_cache: srt_pool_init was not called for device %d", device);
  process_events(d);
  return srt_pool_empty_cache(d.pool, SRT_POOL_TRAIN, released_bytes);
}

// Model set-up (parameters, optimizer state) happens between begin and end: nothing allocated there is ever an
// intermediate. Outside, the framework's saved-tensor hook tags what backward will need.
int srt_tag_model_begin(void) { std::lock_guard<std::mutex> lk(g_mu); g_in_model_setup = true; return SRT_OK; }
int srt_tag_model_end(void) { std::lock_guard<std::mutex> lk(g_mu); g_in_model_setup = false; return SRT_OK; }

int srt_tag_interm(void* ptr, int device) {
  SRT_REQUIRE(device >= 0 && device < SRT_MAX_DEVICE_NUM, "tag_interm: bad device %d", device);
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_in_model_setup) return SRT_OK;
  DeviceState& d = g_dev[device];
  auto it = d.live.find(ptr);
  SRT_REQUIRE(it != d.live.end(), "tag_interm: %p is not a live block", ptr);
  it->second.tagged = true;
  return SRT_OK;
}

int srt_untag_interm(int device) {
  SRT_REQUIRE(device >= 0 && device < SRT_MAX_DEVICE_NUM, "untag_interm: bad device %d", device);
  std::lock_guard<std::mutex> lk(g_mu);
  for (auto& kv : g_dev[device].live) kv.second.tagged = false;
  return SRT_OK;
}

// Drops every tagged block although the framework still holds the pointers (the batch they belong to was
// killed and will be recomputed); their later srt_free is then a no-op. The caller has synchronised the
// training streams (the kill protocol drains them first). Pages the blocks leave empty go back to the pool.
int srt_release_interm(int device, size_t* released_bytes) {
  SRT_REQUIRE(device >= 0 && device < SRT_MAX_DEVICE_NUM, "release_interm: bad device %d", device);
  std::lock_guard<std::mutex> lk(g_mu);
  DeviceState& d = g_dev[device];
  SRT_REQUIRE(d.pool != nullptr, "release_interm: srt_pool_init was not called for device %d", device);
  for (auto it = d.live.begin(); it != d.live.end();) {
    if (!it->second.tagged) { ++it; continue; }
    // the memory goes, the address stays reserved until the framework frees it (no other block can get it meanwhile)
    int rc = srt_pool_hollow(d.pool, SRT_POOL_TRAIN, it->first);
    if (rc) return rc;
    d.dropped.insert(it->first);
    it = d.live.erase(it);
  }
  return srt_pool_empty_cache(d.pool, SRT_POOL_TRAIN, released_bytes);
}

int64_t srt_pool_stat_dev(int device, int which) {
  if (device < 0 || device >= SRT_MAX_DEVICE_NUM) return -1;
  srt_pool* p;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    p = g_dev[device].pool;
  }
  return p ? srt_pool_stat(p, which) : -1;
}

int srt_alloc_counters(int device, int64_t* allocs, int64_t* frees, int64_t* deferred, int64_t* pending, int64_t* live) {
  SRT_REQUIRE(device >= 0 && device < SRT_MAX_DEVICE_NUM, "alloc_counters: bad device %d", device);
  std::lock_guard<std::mutex> lk(g_mu);
  DeviceState& d = g_dev[device];
  if (allocs) *allocs = d.n_alloc;
  if (frees) *frees = d.n_free;
  if (deferred) *deferred = d.n_deferred;
  if (pending) *pending = (int64_t)d.pending.size();
  if (live) *live = (int64_t)d.live.size();
  return SRT_OK;
}

}  // extern "C"
