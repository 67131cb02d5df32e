// extern "C" surface of the kernel library: argument checks, dtype / kernel-family dispatch.
#include <stdarg.h>
#include <time.h>
#include <unistd.h>

#include <atomic>
#include <stdlib.h>
#include <mutex>

#include "common.cuh"
#include "conv_geom.cuh"
#include "grad_buckets.cuh"
#include "ops.cuh"

namespace srt {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

static bool env_is_one(const char* name) {
  const char* e = getenv(name);
  return e && e[0] == '1' && e[1] == 0;
}
bool log_on(LogKind kind) {
  static const char* const names[] = {"COLTRAIN_LOG_CONTROL_STUB", "COLTRAIN_LOG_DYNAMIC_BATCH",
                                      "COLTRAIN_LOG_NCCL_PROCESS_GROUP"};
  return env_is_one("COLTRAIN_LOG_ALL") || env_is_one(names[kind]);
}
void log_line(LogKind kind, const char* fmt, ...) {
  static const char* const tags[] = {"control_stub", "dynamic_batch", "nccl_process_group"};
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  timespec ts;
  clock_gettime(CLOCK_REALTIME, &ts);
  // one write per line, so lines of several ranks do not interleave inside a line
  fprintf(stderr, "[torch_col %s %lld.%03ld pid %d] %s\n", tags[kind], (long long)ts.tv_sec, ts.tv_nsec / 1000000,
          (int)getpid(), buf);
}

static std::atomic<long long> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

int sm_count() {
  static int cached[16] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached[dev] = n;
  }
  const int lim = sm_limit();
  return lim > 0 && lim < cached[dev] ? lim : cached[dev];
}

static thread_local bool tl_pdl_on = true;
void set_pdl_enabled(bool on) { tl_pdl_on = on; }
int pdl_classes() {
  static const int v = [] { const char* e = getenv("SIRIUS_B200_PDL"); return e ? atoi(e) : 7; }();
  return tl_pdl_on ? v : 0;
}
static thread_local bool tl_pdl_big = true;
bool pdl_big_kernels() { return tl_pdl_big; }
void set_pdl_big_kernels(bool on) { tl_pdl_big = on; }

static std::mutex g_mask_mu;
static SmMask g_mask = {{~0ull, ~0ull, ~0ull}};
SmMask current_sm_mask() {
  std::lock_guard<std::mutex> lk(g_mask_mu);
  return g_mask;
}
void set_current_sm_mask(const SmMask& m) {
  std::lock_guard<std::mutex> lk(g_mask_mu);
  g_mask = m;
}

int tc_status_fetch(int* out);
void tc_set_conv_plan(int gather, int tile_n, int pair);
void tc_set_wgrad_pairs(bool on);
bool tc_wgrad_pairs();

static int check_desc(const srt_conv_desc& d) {
  SRT_REQUIRE(d.N > 0 && d.H > 0 && d.W > 0 && d.C > 0 && d.K > 0 && d.R > 0 && d.S > 0 &&
                  d.stride > 0 && d.pad >= 0,
              "conv: non-positive extent");
  SRT_REQUIRE(d.P == (d.H + 2 * d.pad - d.R) / d.stride + 1 &&
                  d.Q == (d.W + 2 * d.pad - d.S) / d.stride + 1,
              "conv: P/Q (%d,%d) inconsistent with H/W/pad/stride", d.P, d.Q);
  SRT_REQUIRE(d.C % 8 == 0 && d.K % 8 == 0, "conv: C (%d) and K (%d) must be multiples of 8", d.C, d.K);
  SRT_REQUIRE((long long)d.N * d.H * d.W * d.C < (1ll << 31) &&
                  (long long)d.N * d.P * d.Q * d.K < (1ll << 31),
              "conv: tensor exceeds 2^31 elements");
  return SRT_OK;
}

static bool use_tc(int dtype, int impl) {
  return dtype == SRT_BF16 && impl != SRT_IMPL_SIMT;
}

int conv_fprop(const srt_conv_desc& d, int dtype, int impl, const void* x, const void* w, void* y,
               const srt_conv_epilogue* ep, cudaStream_t st) {
  int rc = check_desc(d);
  if (rc) return rc;
  SRT_REQUIRE(!(dtype == SRT_F32 && impl == SRT_IMPL_TCGEN05), "conv: tcgen05 path is bf16 only");
  GatherGeom g = make_fprop_geom(d);
  if (use_tc(dtype, impl)) return conv_gather_gemm_tc(g, x, w, y, ep, st);
  return conv_gather_gemm_simt(g, dtype, x, w, y, ep, st);
}

bool conv_fprop_stats_supported(const srt_conv_desc& d, int dtype, int impl) {
  return use_tc(dtype, impl) && conv_col_stats_available() && d.C % 8 == 0 && d.K % 8 == 0;
}

size_t conv_fprop_stats_bytes(const srt_conv_desc& d) {
  return conv_col_stats_bytes((int64_t)d.N * d.P * d.Q, d.K);
}

int conv_fprop_stats(const srt_conv_desc& d, int dtype, int impl, const void* x, const void* w, void* y,
                     const srt_conv_epilogue* ep, void* partial, size_t partial_bytes, int* slabs, cudaStream_t st) {
  int rc = check_desc(d);
  if (rc) return rc;
  SRT_REQUIRE(conv_fprop_stats_supported(d, dtype, impl),
              "conv_fprop_bn_stats: only the bf16 tensor-core path computes the column sums");
  GatherGeom g = make_fprop_geom(d);
  return conv_gather_gemm_tc_stats(g, x, w, y, ep, (double*)partial, partial_bytes, slabs, st);
}

int conv_dgrad(const srt_conv_desc& d, int dtype, int impl, const void* dy, const void* wt,
               void* dx, const srt_conv_epilogue* ep, cudaStream_t st) {
  int rc = check_desc(d);
  if (rc) return rc;
  SRT_REQUIRE(!(dtype == SRT_F32 && impl == SRT_IMPL_TCGEN05), "conv: tcgen05 path is bf16 only");
  GatherGeom g = make_dgrad_geom(d);
  if (use_tc(dtype, impl)) return conv_gather_gemm_tc(g, dy, wt, dx, ep, st);
  return conv_gather_gemm_simt(g, dtype, dy, wt, dx, ep, st);
}

size_t conv_wgrad_scratch_bytes(const srt_conv_desc& d, int dtype, int impl) {
  GatherGeom g = make_fprop_geom(d);
  return use_tc(dtype, impl) ? conv_wgrad_tc_scratch_bytes(g) : conv_wgrad_simt_scratch_bytes(g);
}

int conv_wgrad(const srt_conv_desc& d, int dtype, int impl, const void* dy, const void* x,
               float* dw, void* scratch, size_t scratch_bytes, cudaStream_t st) {
  int rc = check_desc(d);
  if (rc) return rc;
  SRT_REQUIRE(!(dtype == SRT_F32 && impl == SRT_IMPL_TCGEN05), "conv: tcgen05 path is bf16 only");
  GatherGeom g = make_fprop_geom(d);
  if (use_tc(dtype, impl)) return conv_wgrad_tc(g, dy, x, dw, scratch, scratch_bytes, st);
  return conv_wgrad_simt(g, dtype, dy, x, dw, scratch, scratch_bytes, st);
}

}  // namespace srt

using namespace srt;

#define ST(s) ((cudaStream_t)(s))
#define CHECK_DTYPE(dt) SRT_REQUIRE((dt) == SRT_F32 || (dt) == SRT_BF16, "unknown dtype %d", (int)(dt))

extern "C" {

const char* srt_last_error(void) { return g_err; }
const char* srt_version(void) { return "sirius_b200 0.1 (sm_100a)"; }

int srt_conv_fprop(const srt_conv_desc* d, int dtype, int impl, const void* x, const void* w,
                   void* y, const srt_conv_epilogue* ep, void* stream) {
  SRT_REQUIRE(d && x && w && y, "conv_fprop: null argument");
  CHECK_DTYPE(dtype);
  return conv_fprop(*d, dtype, impl, x, w, y, ep, ST(stream));
}
int srt_conv_fprop_bn_stats(const srt_conv_desc* d, int dtype, int impl, const void* x, const void* w,
                            void* y, const srt_conv_epilogue* ep, void* partial, size_t partial_bytes,
                            int* slabs, void* stream) {
  SRT_REQUIRE(d && x && w && y && partial && slabs, "conv_fprop_bn_stats: null argument");
  CHECK_DTYPE(dtype);
  return conv_fprop_stats(*d, dtype, impl, x, w, y, ep, partial, partial_bytes, slabs, ST(stream));
}
size_t srt_conv_fprop_bn_stats_bytes(const srt_conv_desc* d) { return d ? conv_fprop_stats_bytes(*d) : 0; }
int srt_conv_fprop_bn_stats_supported(const srt_conv_desc* d, int dtype, int impl) {
  return d && conv_fprop_stats_supported(*d, dtype, impl) ? 1 : 0;
}
int srt_conv_dgrad(const srt_conv_desc* d, int dtype, int impl, const void* dy, const void* wt,
                   void* dx, const srt_conv_epilogue* ep, void* stream) {
  SRT_REQUIRE(d && dy && wt && dx, "conv_dgrad: null argument");
  CHECK_DTYPE(dtype);
  return conv_dgrad(*d, dtype, impl, dy, wt, dx, ep, ST(stream));
}
int srt_conv_wgrad(const srt_conv_desc* d, int dtype, int impl, const void* dy, const void* x,
                   float* dw, void* scratch, size_t scratch_bytes, void* stream) {
  SRT_REQUIRE(d && dy && x && dw, "conv_wgrad: null argument");
  CHECK_DTYPE(dtype);
  return conv_wgrad(*d, dtype, impl, dy, x, dw, scratch, scratch_bytes, ST(stream));
}
size_t srt_conv_wgrad_scratch_bytes(const srt_conv_desc* d, int dtype, int impl) {
  if (!d) return 0;
  return conv_wgrad_scratch_bytes(*d, dtype, impl);
}
int srt_conv_filter_transpose(const srt_conv_desc* d, int dtype, const void* w, void* wt,
                              void* stream) {
  SRT_REQUIRE(d && w && wt, "filter_transpose: null argument");
  CHECK_DTYPE(dtype);
  return filter_transpose(dtype, w, wt, d->K, d->R * d->S, d->C, ST(stream));
}

int srt_bn_stats(int dtype, const void* z, int64_t rows, int C, const float* gamma,
                 const float* beta, float eps, float momentum, float* running_mean,
                 float* running_var, float* mean, float* invstd, float* scale, float* shift,
                 void* scratch, size_t scratch_bytes, void* stream) {
  SRT_REQUIRE(z && mean && invstd && scale && shift, "bn_stats: null argument");
  CHECK_DTYPE(dtype);
  return bn_stats(dtype, z, rows, C, gamma, beta, eps, momentum, running_mean, running_var, mean,
                  invstd, scale, shift, scratch, scratch_bytes, ST(stream));
}
size_t srt_bn_scratch_bytes(int64_t rows, int C) { return bn_scratch_bytes(rows, C); }
int srt_bn_finalize(const void* partial, int slabs, int C, int64_t rows, const float* gamma, const float* beta,
                    float eps, float momentum, float* running_mean, float* running_var, float* mean,
                    float* invstd, float* scale, float* shift, void* stream) {
  SRT_REQUIRE(partial && mean && invstd && scale && shift, "bn_finalize: null argument");
  return bn_finalize(partial, slabs, C, rows, gamma, beta, eps, momentum, running_mean, running_var, mean, invstd,
                     scale, shift, ST(stream));
}
int srt_bn_stats_static(int dtype, const void* z, int64_t rows, int C, const float* gamma,
                        const float* beta, float eps, float momentum, float* running_mean,
                        float* running_var, float* mean, float* invstd, float* scale, float* shift,
                        void* stream) {
  SRT_REQUIRE(z && mean && invstd && scale && shift, "bn_stats_static: null argument");
  CHECK_DTYPE(dtype);
  return bn_stats_static(dtype, z, rows, C, gamma, beta, eps, momentum, running_mean, running_var,
                         mean, invstd, scale, shift, ST(stream));
}
int srt_bn_static_prepare(void) { return bn_static_prepare(true, nullptr); }
int srt_bn_apply(int dtype, const void* z, const void* residual, void* y, int64_t rows, int C,
                 const float* scale, const float* shift, int relu, void* stream) {
  SRT_REQUIRE(z && y && scale && shift, "bn_apply: null argument");
  CHECK_DTYPE(dtype);
  return bn_apply(dtype, z, residual, y, rows, C, scale, shift, relu, ST(stream));
}
int srt_bn_backward(int dtype, const void* dy, const void* y, const void* z, int64_t rows, int C,
                    const float* gamma, const float* mean, const float* invstd, const float* scale,
                    const float* shift, int relu, void* dz, void* dresidual, float* dgamma,
                    float* dbeta, void* scratch, size_t scratch_bytes, void* stream) {
  SRT_REQUIRE(dy && z && mean && invstd && dz, "bn_backward: null argument");
  CHECK_DTYPE(dtype);
  return bn_backward(dtype, dy, y, z, rows, C, gamma, mean, invstd, scale, shift, relu, dz, dresidual,
                     dgamma, dbeta, scratch, scratch_bytes, ST(stream));
}

int srt_bn_apply_bits(int dtype, const void* z, const void* residual, void* y, int64_t rows, int C,
                      const float* scale, const float* shift, uint8_t* relu_bits, void* stream) {
  SRT_REQUIRE(z && y && scale && shift && relu_bits, "bn_apply_bits: null argument");
  CHECK_DTYPE(dtype);
  return bn_apply(dtype, z, residual, y, rows, C, scale, shift, 1, ST(stream), relu_bits);
}
int srt_bn_backward_bits(int dtype, const void* dy, const uint8_t* relu_bits, const void* z, int64_t rows, int C,
                         const float* gamma, const float* mean, const float* invstd, void* dz, void* dresidual,
                         float* dgamma, float* dbeta, void* scratch, size_t scratch_bytes, int one_launch, void* stream) {
  SRT_REQUIRE(dy && relu_bits && z && mean && invstd && dz, "bn_backward_bits: null argument");
  CHECK_DTYPE(dtype);
  if (one_launch) {
    SRT_REQUIRE(C % 8 == 0 && rows > 0, "bn_backward_bits: C (%d) must be a multiple of 8", C);
    return bn_backward_fused(dtype, dy, nullptr, z, rows, C, gamma, mean, invstd, nullptr, nullptr, 1, dz, dresidual, dgamma,
                             dbeta, ST(stream), relu_bits);
  }
  return bn_backward(dtype, dy, nullptr, z, rows, C, gamma, mean, invstd, nullptr, nullptr, 1, dz, dresidual, dgamma, dbeta,
                     scratch, scratch_bytes, ST(stream), relu_bits);
}

int srt_bn_fused_fits(int dtype, int64_t rows, int C, int backward) { return bn_fused_fits(dtype, rows, C, backward) ? 1 : 0; }
int srt_bn_forward_fused(int dtype, const void* z, const void* residual, void* y, int64_t rows, int C, const float* gamma,
                         const float* beta, float eps, float momentum, float* running_mean, float* running_var, float* mean,
                         float* invstd, float* scale, float* shift, int relu, void* stream) {
  SRT_REQUIRE(z && y && mean && invstd && scale && shift, "bn_forward_fused: null argument");
  CHECK_DTYPE(dtype);
  SRT_REQUIRE(C % 8 == 0 && rows > 0, "bn_forward_fused: C (%d) must be a multiple of 8", C);
  return bn_forward_fused(dtype, z, residual, y, rows, C, gamma, beta, eps, momentum, running_mean, running_var, mean, invstd,
                          scale, shift, relu, ST(stream));
}
int srt_bn_backward_fused(int dtype, const void* dy, const void* y, const void* z, int64_t rows, int C, const float* gamma,
                          const float* mean, const float* invstd, const float* scale, const float* shift, int relu, void* dz,
                          void* dresidual, float* dgamma, float* dbeta, void* stream) {
  SRT_REQUIRE(dy && z && mean && invstd && dz, "bn_backward_fused: null argument");
  CHECK_DTYPE(dtype);
  SRT_REQUIRE(C % 8 == 0 && rows > 0, "bn_backward_fused: C (%d) must be a multiple of 8", C);
  return bn_backward_fused(dtype, dy, y, z, rows, C, gamma, mean, invstd, scale, shift, relu, dz, dresidual, dgamma, dbeta,
                           ST(stream));
}

int srt_maxpool3x3s2_fwd(int dtype, const void* x, void* y, uint8_t* argmax, int N, int H, int W,
                         int C, void* stream) {
  SRT_REQUIRE(x && y && argmax, "maxpool_fwd: null argument");
  CHECK_DTYPE(dtype);
  return maxpool_fwd(dtype, x, y, argmax, N, H, W, C, ST(stream));
}
int srt_maxpool3x3s2_bwd(int dtype, const void* dy, const uint8_t* argmax, void* dx, int N, int H,
                         int W, int C, void* stream) {
  SRT_REQUIRE(dy && dx && argmax, "maxpool_bwd: null argument");
  CHECK_DTYPE(dtype);
  return maxpool_bwd(dtype, dy, argmax, dx, N, H, W, C, ST(stream));
}
int srt_avgpool_fwd(int dtype, const void* x, void* y, int N, int HW, int C, void* stream) {
  SRT_REQUIRE(x && y, "avgpool_fwd: null argument");
  CHECK_DTYPE(dtype);
  return avgpool_fwd(dtype, x, y, N, HW, C, ST(stream));
}
int srt_avgpool_bwd(int dtype, const void* dy, void* dx, int N, int HW, int C, void* stream) {
  SRT_REQUIRE(dy && dx, "avgpool_bwd: null argument");
  CHECK_DTYPE(dtype);
  return avgpool_bwd(dtype, dy, dx, N, HW, C, ST(stream));
}

int srt_softmax_ce(int dtype, const void* logits, const int64_t* labels, int B, int classes,
                   float grad_scale, float* row_loss, void* dlogits, void* stream) {
  SRT_REQUIRE(logits && labels, "softmax_ce: null argument");
  CHECK_DTYPE(dtype);
  return softmax_ce(dtype, logits, labels, B, classes, grad_scale, row_loss, dlogits, ST(stream));
}
int srt_sum_f32(const float* v, int n, float* out, int accumulate, void* stream) {
  SRT_REQUIRE(v && out && n >= 0, "sum_f32: bad argument");
  return sum_f32(v, n, out, accumulate, ST(stream));
}
int srt_colsum(int dtype, const void* dy, int64_t rows, int K, float* out, void* stream) {
  SRT_REQUIRE(dy && out, "colsum: null argument");
  CHECK_DTYPE(dtype);
  return colsum(dtype, dy, rows, K, out, ST(stream));
}

int srt_sgd_momentum(float* p, const float* g, float* m, void* p_bf16, int64_t n, float lr,
                     float mu, float wd, int first_step, void* stream) {
  SRT_REQUIRE(p && g && m && n >= 0, "sgd_momentum: bad argument");
  return sgd_momentum(p, g, m, p_bf16, n, lr, mu, wd, first_step, ST(stream));
}
int srt_adamw(float* p, const float* g, float* m, float* v, void* p_bf16, int64_t n, float lr,
              float beta1, float beta2, float eps, float wd, int step, void* stream) {
  SRT_REQUIRE(p && g && m && v && n >= 0, "adamw: bad argument");
  return adamw(p, g, m, v, p_bf16, n, lr, beta1, beta2, eps, wd, step, ST(stream));
}
int srt_grad_accumulate(float* acc, float* g, int64_t n, void* stream) {
  SRT_REQUIRE(acc && g && n >= 0, "grad_accumulate: bad argument");
  return grad_accumulate(acc, g, n, ST(stream));
}

int srt_nchw_to_nhwc(int dtype, const float* src, void* dst, int N, int C, int H, int W, int Cpad,
                     void* stream) {
  SRT_REQUIRE(src && dst, "nchw_to_nhwc: null argument");
  CHECK_DTYPE(dtype);
  return nchw_to_nhwc(dtype, src, dst, N, C, H, W, Cpad, ST(stream));
}
int srt_cast_f32_to_bf16(const float* src, void* dst, int64_t n, void* stream) {
  SRT_REQUIRE(src && dst && n >= 0, "cast: bad argument");
  return cast_f32_to_bf16(src, dst, n, ST(stream));
}
int srt_cast_bf16_to_f32(const void* src, float* dst, int64_t n, void* stream) {
  SRT_REQUIRE(src && dst && n >= 0, "cast: bad argument");
  return cast_bf16_to_f32(src, dst, n, ST(stream));
}

int srt_set_sm_mask(const uint64_t mask[3]) {
  SRT_REQUIRE(mask != nullptr, "set_sm_mask: null mask");
  SRT_REQUIRE((mask[0] | mask[1] | mask[2]) != 0, "set_sm_mask: mask disables every SM");
  SmMask m = {{mask[0], mask[1], mask[2]}};
  set_current_sm_mask(m);
  return SRT_OK;
}
int srt_get_sm_mask(uint64_t mask[3]) {
  SRT_REQUIRE(mask != nullptr, "get_sm_mask: null mask");
  SmMask m = current_sm_mask();
  mask[0] = m.w[0]; mask[1] = m.w[1]; mask[2] = m.w[2];
  return SRT_OK;
}

int64_t srt_launch_count(void) { return (int64_t)g_launches.load(); }

int srt_tc_status(int* status) {
  SRT_REQUIRE(status != nullptr, "tc_status: null argument");
  return tc_status_fetch(status);
}
int srt_conv_wgrad_pairs(int on) {
  const int was = tc_wgrad_pairs() ? 1 : 0;
  if (on >= 0) tc_set_wgrad_pairs(on != 0);
  return was;
}

int srt_conv_plan_override(int gather, int tile_n, int pair) {
  SRT_REQUIRE(gather == 0 || gather == 1, "conv_plan_override: gather must be 0 or 1");
  SRT_REQUIRE(tile_n == 0 || tile_n == 64 || tile_n == 128 || tile_n == 256,
              "conv_plan_override: tile_n must be 0, 64, 128 or 256");
  SRT_REQUIRE(pair >= -1 && pair <= 1, "conv_plan_override: pair must be -1, 0 or 1");
  tc_set_conv_plan(gather, tile_n, pair);
  return SRT_OK;
}

int srt_bgemm(const srt_bgemm_desc* d, const void* A, const void* B, void* D, void* stream) {
  SRT_REQUIRE(d && A && B && D, "bgemm: null argument");
  BgemmDesc g = {d->M, d->N, d->K, d->Z1, d->Z2, d->lda, d->a_s1, d->a_s2, d->ldb, d->b_s1, d->b_s2,
                 d->ldd, d->d_s1, d->d_s2, d->alpha, d->causal, d->k_causal};
  return bgemm_bf16(g, A, B, D, (cudaStream_t)stream);
}
int srt_layernorm_fwd(const void* x, const float* gamma, const float* beta, void* y, float* mean, float* rstd,
                      int64_t rows, int C, float eps, void* stream) {
  SRT_REQUIRE(x && gamma && beta && y && mean && rstd, "layernorm_fwd: null argument");
  return layernorm_fwd(x, gamma, beta, y, mean, rstd, rows, C, eps, (cudaStream_t)stream);
}
size_t srt_layernorm_bwd_scratch_bytes(int C) { return layernorm_bwd_scratch_bytes(C); }
int srt_layernorm_bwd(const void* dy, const void* x, const float* gamma, const float* mean, const float* rstd,
                      const void* addend, void* dx, float* dgamma, float* dbeta, int64_t rows, int C, void* scratch,
                      size_t scratch_bytes, void* stream) {
  SRT_REQUIRE(dy && x && gamma && mean && rstd && dx && dgamma && dbeta, "layernorm_bwd: null argument");
  return layernorm_bwd(dy, x, gamma, mean, rstd, addend, dx, dgamma, dbeta, rows, C, scratch, scratch_bytes,
                       (cudaStream_t)stream);
}
int srt_gelu_fwd(const void* x, void* y, int64_t n, void* stream) {
  SRT_REQUIRE(x && y, "gelu_fwd: null argument");
  return gelu_fwd(x, y, n, (cudaStream_t)stream);
}
int srt_gelu_bwd(const void* dy, const void* x, void* dx, int64_t n, void* stream) {
  SRT_REQUIRE(dy && x && dx, "gelu_bwd: null argument");
  return gelu_bwd(dy, x, dx, n, (cudaStream_t)stream);
}
int srt_causal_softmax_fwd(void* scores, int64_t Z, int S, void* stream) {
  SRT_REQUIRE(scores, "causal_softmax_fwd: null argument");
  return causal_softmax_fwd(scores, Z, S, (cudaStream_t)stream);
}
int srt_causal_softmax_bwd(const void* P, void* dP, int64_t Z, int S, void* stream) {
  SRT_REQUIRE(P && dP, "causal_softmax_bwd: null argument");
  return causal_softmax_bwd(P, dP, Z, S, (cudaStream_t)stream);
}
int srt_batched_transpose(const void* in, void* out, int R, int C, int64_t ld_in, int64_t s1, int64_t s2, int Z1,
                          int Z2, void* stream) {
  SRT_REQUIRE(in && out, "batched_transpose: null argument");
  return batched_transpose(in, out, R, C, ld_in, s1, s2, Z1, Z2, (cudaStream_t)stream);
}
int srt_lm_cross_entropy(void* logits, const int32_t* labels, int64_t rows, int V, int ld, float grad_scale,
                         float* row_loss, void* stream) {
  SRT_REQUIRE(logits && labels && row_loss, "lm_cross_entropy: null argument");
  return lm_cross_entropy(logits, labels, rows, V, ld, grad_scale, row_loss, (cudaStream_t)stream);
}

int srt_gb_count(void* gb) { return gb ? (int)((GradBuckets*)gb)->list.size() : -1; }
int srt_gb_get(void* gb, int i, int64_t* offset, int64_t* count) {
  GradBuckets* b = (GradBuckets*)gb;
  SRT_REQUIRE(b && offset && count && i >= 0 && i < (int)b->list.size(), "gb_get: bad argument");
  *offset = (int64_t)b->list[i].off;
  *count = (int64_t)b->list[i].count;
  return SRT_OK;
}
int srt_gb_wait(void* gb, int i, void* stream) {
  GradBuckets* b = (GradBuckets*)gb;
  SRT_REQUIRE(b && i >= 0 && i < (int)b->list.size(), "gb_wait: bad argument");
  SRT_CHECK_CUDA(cudaStreamWaitEvent((cudaStream_t)stream, b->list[i].ev, 0));
  return SRT_OK;
}
int srt_gb_allreduce_begin(void* gb, float* grad, srt_ddp* c, int wire_dtype) {
  GradBuckets* b = (GradBuckets*)gb;
  SRT_REQUIRE(b && grad && c, "gb_allreduce_begin: null argument");
  std::vector<int64_t> off, cnt;
  std::vector<cudaEvent_t> ev;
  for (auto& k : b->list) {
    off.push_back((int64_t)k.off);
    cnt.push_back((int64_t)k.count);
    ev.push_back(k.ev);
  }
  return grad_exchange_begin((Comm*)c, grad, (int)off.size(), off.data(), cnt.data(), ev.data(), wire_dtype);
}
int srt_stream_wait_event(void* stream, void* event) {
  SRT_REQUIRE(event, "stream_wait_event: null event");
  SRT_CHECK_CUDA(cudaStreamWaitEvent((cudaStream_t)stream, (cudaEvent_t)event, 0));
  return SRT_OK;
}

}  // extern "C"
