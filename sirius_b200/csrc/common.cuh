// Shared device/host helpers for the sm_100a kernel library.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <string>

#include "../../include/sirius_b200.h"

namespace srt {

// Thread-local last-error text surfaced through srt_last_error().
void set_error(const char* fmt, ...);

#define SRT_CHECK_CUDA(expr)                                                        \
  do {                                                                              \
    cudaError_t _e = (expr);                                                        \
    if (_e != cudaSuccess) {                                                        \
      ::srt::set_error("%s:%d %s -> %s", __FILE__, __LINE__, #expr,                 \
                       cudaGetErrorString(_e));                                     \
      return SRT_ERR_CUDA;                                                          \
    }                                                                               \
  } while (0)

#define SRT_REQUIRE(cond, ...)                                                      \
  do {                                                                              \
    if (!(cond)) {                                                                  \
      ::srt::set_error(__VA_ARGS__);                                                \
      return SRT_ERR_INVALID;                                                       \
    }                                                                               \
  } while (0)

void count_launch();  // bumps the process-wide launch counter

// Diagnostic lines on stderr, silent unless the environment asks for them: the reference's
// LOG_IF(INFO, TorchColConfig::log_*) with the same variables (pytorch/torch_col/csrc/config.cc:66-69,91-98):
// COLTRAIN_LOG_ALL=1 or the variable of the kind. Read at every call (the call sites are per command, not per kernel).
enum LogKind { LOG_CONTROL_STUB = 0, LOG_DYNAMIC_BATCH = 1, LOG_NCCL_PROCESS_GROUP = 2 };
bool log_on(LogKind kind);
void log_line(LogKind kind, const char* fmt, ...);
#define SRT_LOG(kind, ...)                                                          \
  do {                                                                              \
    if (::srt::log_on(kind)) ::srt::log_line(kind, __VA_ARGS__);                    \
  } while (0)

#define SRT_LAUNCH_CHECK()                                                          \
  do {                                                                              \
    ::srt::count_launch();                                                          \
    cudaError_t _e = cudaGetLastError();                                            \
    if (_e != cudaSuccess) {                                                        \
      ::srt::set_error("%s:%d launch -> %s", __FILE__, __LINE__,                    \
                       cudaGetErrorString(_e));                                     \
      return SRT_ERR_CUDA;                                                          \
    }                                                                               \
  } while (0)

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
static inline long long ceil_div_ll(long long a, long long b) { return (a + b - 1) / b; }

int sm_count();  // SM count kernels should size their grids for: the device's, or the calling thread's limit
int sm_limit();                  // 0 = none
void set_sm_limit(int n);        // per thread: a step that runs inside an SM partition sets its width
// Stream of the widest green-context partition with at most `allowed` SMs (nullptr = whole device).
int partition_stream(int device, int allowed, cudaStream_t* stream, int* sms);
int partition_streams(int device, int allowed, cudaStream_t* stream, cudaStream_t* side, int* sms);

// ---- element type traits ---------------------------------------------------------------
template <typename T> struct ElemTraits;
template <> struct ElemTraits<float> {
  static constexpr int kVec = 4;  // elements per 16-byte vector
  __device__ static inline float to_f(float v) { return v; }
  __device__ static inline float from_f(float v) { return v; }
};
template <> struct ElemTraits<__nv_bfloat16> {
  static constexpr int kVec = 8;
  __device__ static inline float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  __device__ static inline __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};

// 16-byte vector of T, loaded/stored in one transaction and unpacked to floats.
template <typename T> struct Vec16;
template <> struct Vec16<float> {
  static constexpr int N = 4;
  float4 raw;
  __device__ inline void load(const float* p) { raw = *reinterpret_cast<const float4*>(p); }
  __device__ inline void store(float* p) const { *reinterpret_cast<float4*>(p) = raw; }
  __device__ inline void unpack(float (&f)[4]) const { f[0] = raw.x; f[1] = raw.y; f[2] = raw.z; f[3] = raw.w; }
  __device__ inline void pack(const float (&f)[4]) { raw = make_float4(f[0], f[1], f[2], f[3]); }
};
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  uint4 raw;
  __device__ inline void load(const __nv_bfloat16* p) { raw = *reinterpret_cast<const uint4*>(p); }
  __device__ inline void store(__nv_bfloat16* p) const { *reinterpret_cast<uint4*>(p) = raw; }
  __device__ inline void unpack(float (&f)[8]) const {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  __device__ inline void pack(const float (&f)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    raw = make_uint4(w[0], w[1], w[2], w[3]);
  }
};

// ---- programmatic dependent launch ---------------------------------------------------------------
// Chains of short kernels on one stream lose a few microseconds at every boundary (launch latency and
// the ramp of the next grid). A kernel launched with launch_pdl() may be scheduled while its
// predecessor on the stream still runs; it must call pdl_enter() before it touches global memory:
// that waits until the predecessor has completed and its writes are visible, then lets the kernel
// after this one be scheduled in turn (one kernel deep, so waiting blocks never pile up on the SMs).
// In a kernel launched the ordinary way both instructions do nothing.
__device__ inline void pdl_enter() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;");
}
// Which kernel classes launch early: bit 0 BatchNorm, bit 1 tensor-core GEMMs, bit 2 everything else.
// SIRIUS_B200_PDL overrides the default at process start (a tuning aid).
enum { PDL_NORM = 1, PDL_GEMM = 2, PDL_MISC = 4 };
int pdl_classes();
// Per thread: launches made while this is off are ordinary ones (used for work queued on a second stream,
// where blocks that sit resident waiting for their predecessor take SM room from the main stream).
void set_pdl_enabled(bool on);
struct PdlOff {  // scope guard
  bool off;
  explicit PdlOff(bool o) : off(o) { if (off) set_pdl_enabled(false); }
  ~PdlOff() { if (off) set_pdl_enabled(true); }
};
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_if(bool early, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                 cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = early ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args&&... args) {
  return launch_pdl_if((pdl_classes() & PDL_MISC) != 0, kernel, grid, block, smem, st, static_cast<Args&&>(args)...);
}
// Kernels that hold most of an SM's shared memory (the tensor-core GEMMs) should not sit resident waiting
// for their predecessor while another stream could use that SM; the step executor turns early launch
// of those off while it overlaps streams.
bool pdl_big_kernels();
void set_pdl_big_kernels(bool on);


// ---- allowed-SM mask ---------------------------------------------------------------------
// Bit i set = SM i may run training CTAs. Passed by value to persistent kernels, which read
// %smid and retire at once when their SM is not allowed.
struct SmMask {
  uint64_t w[3];
};
__device__ inline uint32_t smid() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%smid;" : "=r"(r));
  return r;
}
__device__ inline bool sm_allowed(const SmMask& m) {
  uint32_t s = smid();
  return (m.w[(s >> 6) % 3] >> (s & 63)) & 1ull;
}
SmMask current_sm_mask();          // process-wide mask (all ones by default)
void set_current_sm_mask(const SmMask& m);

}  // namespace srt
