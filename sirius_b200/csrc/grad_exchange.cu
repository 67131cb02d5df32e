// Gradient exchange between data-parallel ranks: one NCCL sum all-reduce per gradient bucket on the library's own
// communication stream, each ordered behind the event the step executor records when the bucket's gradients are
// final, so the exchange runs beside the rest of backward. Replaces the reference's c10d Reducer + ProcessGroupNCCL
// extension (pytorch/torch_col/csrc/dist_ext.h:109-243, dist_ext.cc:59-123; abort and restart of the communicator:
// dist_ext.cc:673-784).
//
// All NCCL traffic lands in this rank's own buffers (plain ncclAllReduce on local pointers; no kernel of this library
// reads a peer's memory). NCCL is resolved at run time (dlopen of libnccl.so.2, the copy PyTorch has loaded when there
// is one), so the library loads and its CPU tests run on hosts without NCCL or a GPU.
//
// Wire format: SRT_F32 exchanges the fp32 gradients in place. SRT_BF16 rounds each bucket to bf16 into a staging
// buffer owned by the communicator, exchanges half the bytes, and widens the sum back into the gradient buffer;
// both conversions run on the communication stream, behind the bucket's event.
#include <dlfcn.h>
#include <nccl.h>

#include <mutex>
#include <vector>

#include "common.cuh"

namespace srt {
namespace {

struct NcclApi {
  void* lib = nullptr;
  ncclResult_t (*GetVersion)(int*) = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRankConfig)(ncclComm_t*, int, ncclUniqueId, int, ncclConfig_t*) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  std::string why;
};

NcclApi* nccl() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    const char* names[] = {getenv("SIRIUS_B200_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
      if (!n || !*n) continue;
      api.lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
      if (api.lib) break;
      api.why = dlerror();
    }
    if (!api.lib) return;
    bool ok = true;
    auto sym = [&](const char* name) {
      void* p = dlsym(api.lib, name);
      if (!p) { ok = false; api.why = std::string("missing symbol ") + name; }
      return p;
    };
    api.GetVersion = (decltype(api.GetVersion))sym("ncclGetVersion");
    api.GetUniqueId = (decltype(api.GetUniqueId))sym("ncclGetUniqueId");
    api.CommInitRankConfig = (decltype(api.CommInitRankConfig))sym("ncclCommInitRankConfig");
    api.CommDestroy = (decltype(api.CommDestroy))sym("ncclCommDestroy");
    api.CommAbort = (decltype(api.CommAbort))sym("ncclCommAbort");
    api.CommGetAsyncError = (decltype(api.CommGetAsyncError))sym("ncclCommGetAsyncError");
    api.AllReduce = (decltype(api.AllReduce))sym("ncclAllReduce");
    api.GroupStart = (decltype(api.GroupStart))sym("ncclGroupStart");
    api.GroupEnd = (decltype(api.GroupEnd))sym("ncclGroupEnd");
    api.GetErrorString = (decltype(api.GetErrorString))sym("ncclGetErrorString");
    if (!ok) { dlclose(api.lib); api.lib = nullptr; }
  });
  return api.lib ? &api : nullptr;
}

#define SRT_CHECK_NCCL(expr)                                                                        \
  do {                                                                                              \
    ncclResult_t _r = (expr);                                                                       \
    if (_r != ncclSuccess && _r != ncclInProgress) {                                                \
      ::srt::set_error("%s:%d %s -> %s", __FILE__, __LINE__, #expr, nccl()->GetErrorString(_r));    \
      return SRT_ERR_CUDA;                                                                          \
    }                                                                                               \
  } while (0)

constexpr int NT = 256;

// 16 bytes of bf16 out per thread and iteration, two 16-byte fp32 loads in.
__global__ void __launch_bounds__(NT) pack_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, int64_t n) {
  const int64_t nv = n / 8;
  for (int64_t v = (int64_t)blockIdx.x * NT + threadIdx.x; v < nv; v += (int64_t)gridDim.x * NT) {
    const float4 a = *reinterpret_cast<const float4*>(src + v * 8);
    const float4 b = *reinterpret_cast<const float4*>(src + v * 8 + 4);
    const float f[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    Vec16<__nv_bfloat16> o;
    o.pack(f);
    o.store(dst + v * 8);
  }
  if (blockIdx.x == 0 && threadIdx.x < (int)(n - nv * 8)) dst[nv * 8 + threadIdx.x] = __float2bfloat16_rn(src[nv * 8 + threadIdx.x]);
}
__global__ void __launch_bounds__(NT) unpack_bf16_kernel(const __nv_bfloat16* __restrict__ src, float* __restrict__ dst, int64_t n) {
  const int64_t nv = n / 8;
  for (int64_t v = (int64_t)blockIdx.x * NT + threadIdx.x; v < nv; v += (int64_t)gridDim.x * NT) {
    Vec16<__nv_bfloat16> x;
    x.load(src + v * 8);
    float f[8];
    x.unpack(f);
    *reinterpret_cast<float4*>(dst + v * 8) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(dst + v * 8 + 4) = make_float4(f[4], f[5], f[6], f[7]);
  }
  if (blockIdx.x == 0 && threadIdx.x < (int)(n - nv * 8)) dst[nv * 8 + threadIdx.x] = __bfloat162float(src[nv * 8 + threadIdx.x]);
}

int conv_grid(int64_t n) {
  const int64_t want = (n / 8 + NT - 1) / NT;
  const int64_t cap = (int64_t)sm_count() * 4;
  return (int)(want < 1 ? 1 : (want < cap ? want : cap));
}

}  // namespace

struct Comm {
  ncclComm_t comm = nullptr;
  int rank = 0, world = 1, device = 0, max_ctas = 0;
  cudaStream_t stream = nullptr;  // the communication stream
  cudaEvent_t done = nullptr;     // behind the last collective of the exchange begun last
  bool pending = false;
  __nv_bfloat16* wire = nullptr;  // bf16 staging of the whole gradient buffer, indexed like it
  size_t wire_elems = 0;
  int64_t exchanges = 0, bytes_on_wire = 0;
};

static int comm_init(Comm* c, const void* id) {
  NcclApi* api = nccl();
  SRT_REQUIRE(api != nullptr, "NCCL is not available: %s", nccl() ? "" : "libnccl.so.2 could not be loaded");
  ncclUniqueId uid;
  static_assert(sizeof(uid) == SRT_DDP_ID_BYTES, "NCCL unique id size");
  memcpy(&uid, id, sizeof(uid));
  ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
  cfg.blocking = 1;
  // Cap on the CTAs NCCL's kernels occupy: the training kernels beside them are persistent grids of one CTA
  // per SM, and every SM NCCL takes delays one of their tiles by a whole collective.
  if (c->max_ctas > 0) { cfg.minCTAs = 1; cfg.maxCTAs = c->max_ctas; }
  SRT_CHECK_NCCL(api->CommInitRankConfig(&c->comm, c->world, uid, c->rank, &cfg));
  return SRT_OK;
}

// One exchange: per bucket [off, off + cnt) of `grad`, wait for ready[i] (or for nothing when null), reduce.
int grad_exchange_begin(Comm* c, float* grad, int nbuckets, const int64_t* offsets, const int64_t* counts,
                        const cudaEvent_t* ready, int wire_dtype) {
  SRT_REQUIRE(c && c->comm && grad && nbuckets > 0 && offsets && counts, "allreduce_begin: bad argument");
  SRT_REQUIRE(wire_dtype == SRT_F32 || wire_dtype == SRT_BF16, "allreduce_begin: wire dtype must be SRT_F32 or SRT_BF16");
  NcclApi* api = nccl();
  int64_t end = 0;
  for (int i = 0; i < nbuckets; ++i) {
    SRT_REQUIRE(offsets[i] >= 0 && counts[i] > 0, "allreduce_begin: empty or negative bucket %d", i);
    if (offsets[i] + counts[i] > end) end = offsets[i] + counts[i];
  }
  if (wire_dtype == SRT_BF16 && c->wire_elems < (size_t)end) {
    SRT_CHECK_CUDA(cudaStreamSynchronize(c->stream));
    if (c->wire) SRT_CHECK_CUDA(cudaFree(c->wire));
    c->wire = nullptr;
    c->wire_elems = 0;
    SRT_CHECK_CUDA(cudaMalloc(&c->wire, (size_t)end * sizeof(__nv_bfloat16)));
    c->wire_elems = (size_t)end;
  }
  for (int i = 0; i < nbuckets; ++i) {
    if (ready && ready[i]) SRT_CHECK_CUDA(cudaStreamWaitEvent(c->stream, ready[i], 0));
    float* g = grad + offsets[i];
    const int64_t n = counts[i];
    if (wire_dtype == SRT_BF16) {
      SRT_REQUIRE(offsets[i] % 8 == 0, "allreduce_begin: bf16 wire format needs bucket offsets that are multiples of 8");
      __nv_bfloat16* w = c->wire + offsets[i];
      pack_bf16_kernel<<<conv_grid(n), NT, 0, c->stream>>>(g, w, n);
      SRT_LAUNCH_CHECK();
      SRT_CHECK_NCCL(api->AllReduce(w, w, (size_t)n, ncclBfloat16, ncclSum, c->comm, c->stream));
      unpack_bf16_kernel<<<conv_grid(n), NT, 0, c->stream>>>(w, g, n);
      SRT_LAUNCH_CHECK();
      c->bytes_on_wire += n * 2;
    } else {
      SRT_CHECK_NCCL(api->AllReduce(g, g, (size_t)n, ncclFloat32, ncclSum, c->comm, c->stream));
      c->bytes_on_wire += n * 4;
    }
  }
  SRT_CHECK_CUDA(cudaEventRecord(c->done, c->stream));
  c->pending = true;
  c->exchanges++;
  return SRT_OK;
}

int grad_exchange_wait(Comm* c, cudaStream_t consumer) {
  SRT_REQUIRE(c, "allreduce_wait: null communicator");
  if (!c->pending) return SRT_OK;
  SRT_CHECK_CUDA(cudaStreamWaitEvent(consumer, c->done, 0));
  c->pending = false;
  return SRT_OK;
}

void tc_set_wgrad_pairs(bool on);  // igemm_tcgen05.cu

}  // namespace srt

using namespace srt;

extern "C" {

int srt_ddp_available(void) { return nccl() != nullptr ? 1 : 0; }

int srt_ddp_nccl_version(int* version) {
  SRT_REQUIRE(version, "comm_nccl_version: null argument");
  NcclApi* api = nccl();
  SRT_REQUIRE(api != nullptr, "NCCL is not available (libnccl.so.2 could not be loaded)");
  SRT_CHECK_NCCL(api->GetVersion(version));
  return SRT_OK;
}

int srt_ddp_unique_id(void* id) {
  SRT_REQUIRE(id, "comm_unique_id: null argument");
  NcclApi* api = nccl();
  SRT_REQUIRE(api != nullptr, "NCCL is not available (libnccl.so.2 could not be loaded)");
  ncclUniqueId uid;
  SRT_CHECK_NCCL(api->GetUniqueId(&uid));
  memcpy(id, &uid, sizeof(uid));
  return SRT_OK;
}

int srt_ddp_create(const void* id, int rank, int world, int device, int max_ctas, srt_ddp** out) {
  SRT_REQUIRE(id && out && world >= 1 && rank >= 0 && rank < world && device >= 0, "comm_create: bad argument");
  SRT_REQUIRE(nccl() != nullptr, "NCCL is not available (libnccl.so.2 could not be loaded)");
  SRT_CHECK_CUDA(cudaSetDevice(device));
  Comm* c = new Comm();
  c->rank = rank; c->world = world; c->device = device; c->max_ctas = max_ctas;
  int lo = 0, hi = 0;
  cudaDeviceGetStreamPriorityRange(&lo, &hi);
  cudaError_t e = cudaStreamCreateWithPriority(&c->stream, cudaStreamNonBlocking, hi);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->done, cudaEventDisableTiming);
  if (e != cudaSuccess) {
    set_error("comm_create: %s", cudaGetErrorString(e));
    delete c;
    return SRT_ERR_CUDA;
  }
  if (int rc = comm_init(c, id)) {
    cudaStreamDestroy(c->stream);
    cudaEventDestroy(c->done);
    delete c;
    return rc;
  }
  // Data-parallel runs keep every filter gradient on the single-CTA kernel: a grid of CTA pairs that is not resident
  // all at once (NCCL's kernels hold SMs while they wait for their peers) is the one configuration of this library
  // with an unexplained stall on record, and a stalled rank stalls every rank. srt_conv_wgrad_pairs(1) undoes it.
  if (world > 1) tc_set_wgrad_pairs(false);
  SRT_LOG(LOG_NCCL_PROCESS_GROUP, "[ProcessGroupNCCL] rank %d of %d created its communicator on device %d (max CTAs %d)", rank,
          world, device, max_ctas);
  *out = (srt_ddp*)c;
  return SRT_OK;
}

int srt_ddp_destroy(srt_ddp* h) {
  Comm* c = (Comm*)h;
  if (!c) return SRT_OK;
  if (c->stream) cudaStreamSynchronize(c->stream);
  if (c->comm && nccl()) nccl()->CommDestroy(c->comm);
  if (c->wire) cudaFree(c->wire);
  if (c->done) cudaEventDestroy(c->done);
  if (c->stream) cudaStreamDestroy(c->stream);
  delete c;
  return SRT_OK;
}

int srt_ddp_abort(srt_ddp* h) {
  Comm* c = (Comm*)h;
  SRT_REQUIRE(c, "comm_abort: null communicator");
  if (c->comm) {
    SRT_LOG(LOG_NCCL_PROCESS_GROUP, "[ProcessGroupNCCL] rank %d aborts its communicator (%lld exchanges so far)", c->rank,
            (long long)c->exchanges);
    SRT_CHECK_NCCL(nccl()->CommAbort(c->comm));
    c->comm = nullptr;
  }
  c->pending = false;
  return SRT_OK;
}

int srt_ddp_restart(srt_ddp* h, const void* id) {
  Comm* c = (Comm*)h;
  SRT_REQUIRE(c && id, "comm_restart: bad argument");
  if (c->comm) {
    if (int rc = srt_ddp_abort(h)) return rc;
  }
  SRT_CHECK_CUDA(cudaSetDevice(c->device));
  SRT_LOG(LOG_NCCL_PROCESS_GROUP, "[ProcessGroupNCCL] rank %d of %d restarts its communicator", c->rank, c->world);
  return comm_init(c, id);
}

void* srt_ddp_stream(srt_ddp* h) { return h ? (void*)((Comm*)h)->stream : nullptr; }

int srt_ddp_stats(srt_ddp* h, int64_t* exchanges, int64_t* bytes_on_wire) {
  Comm* c = (Comm*)h;
  SRT_REQUIRE(c, "comm_stats: null communicator");
  if (exchanges) *exchanges = c->exchanges;
  if (bytes_on_wire) *bytes_on_wire = c->bytes_on_wire;
  return SRT_OK;
}

int srt_allreduce_begin(srt_ddp* h, float* grad, int nbuckets, const int64_t* offsets, const int64_t* counts,
                        void* const* ready_events, int wire_dtype) {
  return grad_exchange_begin((Comm*)h, grad, nbuckets, offsets, counts, (const cudaEvent_t*)ready_events, wire_dtype);
}

int srt_allreduce_wait(srt_ddp* h, void* stream) { return grad_exchange_wait((Comm*)h, (cudaStream_t)stream); }

int srt_ddp_allreduce(srt_ddp* h, void* buf, int64_t count, int dtype, void* stream) {
  Comm* c = (Comm*)h;
  SRT_REQUIRE(c && c->comm && buf && count > 0, "comm_allreduce: bad argument");
  SRT_REQUIRE(dtype == SRT_F32 || dtype == SRT_BF16, "comm_allreduce: dtype must be SRT_F32 or SRT_BF16");
  SRT_CHECK_NCCL(nccl()->AllReduce(buf, buf, (size_t)count, dtype == SRT_F32 ? ncclFloat32 : ncclBfloat16, ncclSum, c->comm,
                                   (cudaStream_t)stream));
  return SRT_OK;
}

}  // extern "C"
