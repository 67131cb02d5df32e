// SM partition for colocated training, the B200 way.
//
// The reference confines training kernels to a TPC mask by writing a private field of the CUDA
// stream before every launch (common/sm_partition.cu:316-336, SetStreamTpcMask), so that inference
// kernels always find idle SMs. Here the same effect comes from CUDA green contexts: for a ladder of
// SM counts the device's SM resource is split once (cuDevSmResourceSplitByCount), a green context is
// created on each group and two streams (a main one and a low-priority companion) on each green context. A kernel launched on such a stream can
// only be scheduled on the SMs of its group. Following the mask then means: between two launches,
// move to the stream of the widest group that does not exceed the allowed SM count (an event orders
// the new stream after the old one). Nothing is poked, no kernel has to cooperate.
//
// The ladder is built lazily per device and lives for the life of the process.
#include <cuda.h>

#include <mutex>
#include <vector>

#include "../../include/sirius_b200.h"
#include "common.cuh"

namespace srt {
namespace {

#define DRVFN(name) ((decltype(&name))drv_entry(#name))
void* drv_entry(const char* sym) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(sym, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
    return nullptr;
  return p;
}

struct Rung {
  int sms = 0;
  CUgreenCtx ctx = nullptr;
  cudaStream_t stream = nullptr;
  cudaStream_t side = nullptr;  // second stream on the same SMs, lowest priority (overlapped weight gradients)
};

struct Ladder {
  bool tried = false;
  int status = SRT_ERR_UNSUPPORTED;
  int total = 0;
  std::vector<Rung> rungs;  // strictly decreasing SM counts, all below `total`
};

std::mutex g_mu;
Ladder g_ladder[16];
thread_local int tl_sm_limit = 0;  // 0 = no limit

#define CU_TRY(expr)                                                   \
  do {                                                                 \
    CUresult _r = (expr);                                              \
    if (_r != CUDA_SUCCESS) {                                          \
      set_error("%s -> CUresult %d", #expr, (int)_r);                  \
      return SRT_ERR_CUDA;                                             \
    }                                                                  \
  } while (0)

int build_ladder(int device, int stride, Ladder& L) {
  auto f_dev = DRVFN(cuDeviceGet);
  auto f_res = DRVFN(cuDeviceGetDevResource);
  auto f_split = DRVFN(cuDevSmResourceSplitByCount);
  auto f_desc = DRVFN(cuDevResourceGenerateDesc);
  auto f_create = DRVFN(cuGreenCtxCreate);
  auto f_stream = DRVFN(cuGreenCtxStreamCreate);
  if (!f_dev || !f_res || !f_split || !f_desc || !f_create || !f_stream) {
    set_error("sm partition: green-context driver entry points unavailable");
    return SRT_ERR_UNSUPPORTED;
  }
  SRT_CHECK_CUDA(cudaSetDevice(device));
  SRT_CHECK_CUDA(cudaFree(0));
  CUdevice dev;
  CU_TRY(f_dev(&dev, device));
  CUdevResource all;
  CU_TRY(f_res(dev, &all, CU_DEV_RESOURCE_TYPE_SM));
  L.total = (int)all.sm.smCount;
  int last = L.total;
  for (int want = L.total - stride; want >= 8; want -= stride) {
    CUdevResource grp, rest;
    unsigned int n = 1;
    CU_TRY(f_split(&grp, &n, &all, &rest, 0, (unsigned int)want));
    if (n < 1) break;
    const int got = (int)grp.sm.smCount;
    if (got >= last) continue;  // the driver rounded up to a count we already have
    CUdevResourceDesc desc;
    CU_TRY(f_desc(&desc, &grp, 1));
    Rung r;
    r.sms = got;
    CU_TRY(f_create(&r.ctx, desc, dev, CU_GREEN_CTX_DEFAULT_STREAM));
    CUstream st;
    CU_TRY(f_stream(&st, r.ctx, CU_STREAM_NON_BLOCKING, 0));
    r.stream = (cudaStream_t)st;
    int lo = 0, hi = 0;
    SRT_CHECK_CUDA(cudaDeviceGetStreamPriorityRange(&lo, &hi));
    CU_TRY(f_stream(&st, r.ctx, CU_STREAM_NON_BLOCKING, lo));
    r.side = (cudaStream_t)st;
    L.rungs.push_back(r);
    last = got;
  }
  return SRT_OK;
}

}  // namespace

int sm_limit() { return tl_sm_limit; }
void set_sm_limit(int n) { tl_sm_limit = n; }

// Stream of the widest rung with at most `allowed` SMs; *stream = nullptr when the whole device is
// allowed (the caller keeps its own stream). *sms = SM count of the choice.
int partition_streams(int device, int allowed, cudaStream_t* stream, cudaStream_t* side, int* sms);
int partition_stream(int device, int allowed, cudaStream_t* stream, int* sms) {
  cudaStream_t side = nullptr;
  return partition_streams(device, allowed, stream, &side, sms);
}
// Same, also returning the low-priority companion stream of the partition.
int partition_streams(int device, int allowed, cudaStream_t* stream, cudaStream_t* side, int* sms) {
  SRT_REQUIRE(device >= 0 && device < 16, "sm partition: device %d out of range", device);
  std::lock_guard<std::mutex> lk(g_mu);
  Ladder& L = g_ladder[device];
  if (!L.tried) {
    L.tried = true;
    L.status = build_ladder(device, 16, L);
  }
  if (L.status != SRT_OK) return L.status;
  *stream = nullptr;
  *side = nullptr;
  *sms = L.total;
  if (allowed >= L.total || L.rungs.empty()) return SRT_OK;
  const Rung* pick = &L.rungs.back();  // never below the narrowest rung
  for (const Rung& r : L.rungs)
    if (r.sms <= allowed) { pick = &r; break; }
  *stream = pick->stream;
  *side = pick->side;
  *sms = pick->sms;
  return SRT_OK;
}

int partition_levels(int device, int* sms, int cap, int* n) {
  cudaStream_t st;
  int s;
  int rc = partition_stream(device, 1 << 30, &st, &s);
  if (rc) return rc;
  std::lock_guard<std::mutex> lk(g_mu);
  Ladder& L = g_ladder[device];
  int k = 0;
  if (k < cap) sms[k] = L.total;
  ++k;
  for (const Rung& r : L.rungs) {
    if (k < cap) sms[k] = r.sms;
    ++k;
  }
  *n = k;
  return SRT_OK;
}

namespace {
__global__ void smid_probe_kernel(unsigned long long* mask, int spin) {
  if (threadIdx.x == 0) {
    const uint32_t s = smid();
    atomicOr(&mask[(s >> 6) % 3], 1ull << (s & 63));
  }
  // stay resident for a moment so that the blocks spread over every SM the stream may use
  const long long t0 = clock64();
  while (clock64() - t0 < spin) {}
}
}  // namespace

int smid_probe(unsigned long long* device_mask3, cudaStream_t stream) {
  SRT_CHECK_CUDA(cudaMemsetAsync(device_mask3, 0, 3 * sizeof(unsigned long long), stream));
  smid_probe_kernel<<<148 * 8, 128, 0, stream>>>(device_mask3, 20000);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}

}  // namespace srt

extern "C" {

int srt_smp_partition_levels(int device, int* sms, int cap, int* n) {
  SRT_REQUIRE(sms && n && cap > 0, "partition_levels: bad argument");
  return srt::partition_levels(device, sms, cap, n);
}

int srt_smp_partition_stream(int device, int allowed_sms, void** stream, int* sms) {
  SRT_REQUIRE(stream && sms, "partition_stream: null argument");
  cudaStream_t st = nullptr;
  int rc = srt::partition_stream(device, allowed_sms, &st, sms);
  *stream = (void*)st;
  return rc;
}

int srt_debug_smid_probe(void* device_mask3, void* stream) {
  SRT_REQUIRE(device_mask3, "smid_probe: null buffer");
  return srt::smid_probe((unsigned long long*)device_mask3, (cudaStream_t)stream);
}

}  // extern "C"
