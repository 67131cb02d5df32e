// Internal C++ declarations of the kernel launchers (one per C-ABI compute entry point).
#pragma once
#include "common.cuh"
#include "conv_geom.cuh"

namespace srt {

size_t bn_scratch_bytes(int64_t rows, int C);
// Second half of bn_stats for partial sums somebody else produced (double2 [slabs][C]: sum, sum of squares).
int bn_finalize(const void* partial, int slabs, int C, int64_t rows, const float* gamma, const float* beta, float eps,
                float momentum, float* rm, float* rv, float* mean, float* invstd, float* scale, float* shift,
                cudaStream_t st);
int bn_stats(int dtype, const void* z, int64_t rows, int C, const float* gamma, const float* beta,
             float eps, float momentum, float* rm, float* rv, float* mean, float* invstd,
             float* scale, float* shift, void* scratch, size_t scratch_bytes, cudaStream_t st);
int bn_eval_params(const float* gamma, const float* beta, const float* rmean, const float* rvar, float eps, int C,
                   float* scale, float* shift, cudaStream_t st);
int bn_stats_static(int dtype, const void* z, int64_t rows, int C, const float* gamma,
                    const float* beta, float eps, float momentum, float* rm, float* rv, float* mean,
                    float* invstd, float* scale, float* shift, cudaStream_t st);
int bn_static_prepare(bool refresh, void** out);
// relu_bits: one bit per element of a bf16 tensor under a ReLU (bit e of byte i = element 8i + e came out positive).
// bn_apply writes them when given a buffer of rows * C / 8 bytes; the backward functions read them instead of the
// stored output y (a sixteenth of its bytes).
int bn_apply(int dtype, const void* z, const void* residual, void* y, int64_t rows, int C,
             const float* scale, const float* shift, int relu, cudaStream_t st, uint8_t* relu_bits = nullptr);
int bn_backward(int dtype, const void* dy, const void* y, const void* z, int64_t rows, int C,
                const float* gamma, const float* mean, const float* invstd, const float* scale,
                const float* shift, int relu, void* dz, void* dres, float* dgamma, float* dbeta,
                void* scratch, size_t scratch_bytes, cudaStream_t st, const uint8_t* relu_bits = nullptr);

// One-launch BatchNorm (cooperative grid with two grid-wide barriers, see norm_grid.cu); bn_fused_fits says
// whether a shape qualifies.
bool bn_fused_fits(int dtype, int64_t rows, int C, int backward);
bool bn_fused_pays(int dtype, int64_t rows, int C, int backward);  // fits and is small enough to beat the three-kernel path
int bn_forward_fused(int dtype, const void* z, const void* residual, void* y, int64_t rows, int C, const float* gamma,
                     const float* beta, float eps, float momentum, float* rm, float* rv, float* mean, float* invstd,
                     float* scale, float* shift, int relu, cudaStream_t st);
int bn_backward_fused(int dtype, const void* dy, const void* y, const void* z, int64_t rows, int C, const float* gamma,
                      const float* mean, const float* invstd, const float* scale, const float* shift, int relu, void* dz,
                      void* dres, float* dgamma, float* dbeta, cudaStream_t st, const uint8_t* relu_bits = nullptr);

int maxpool_fwd(int dtype, const void* x, void* y, uint8_t* argmax, int N, int H, int W, int C,
                cudaStream_t st);
int maxpool_bwd(int dtype, const void* dy, const uint8_t* argmax, void* dx, int N, int H, int W,
                int C, cudaStream_t st);
int avgpool_fwd(int dtype, const void* x, void* y, int N, int HW, int C, cudaStream_t st);
int avgpool_bwd(int dtype, const void* dy, void* dx, int N, int HW, int C, cudaStream_t st);
int softmax_ce(int dtype, const void* logits, const int64_t* labels, int B, int classes,
               float grad_scale, float* row_loss, void* dlogits, cudaStream_t st);
int sum_f32(const float* v, int n, float* out, int accumulate, cudaStream_t st);
int colsum(int dtype, const void* dy, int64_t rows, int K, float* out, cudaStream_t st);
int sgd_momentum(float* p, const float* g, float* m, void* pb, int64_t n, float lr, float mu,
                 float wd, int first_step, cudaStream_t st);
int adamw(float* p, const float* g, float* m, float* v, void* pb, int64_t n, float lr, float b1,
          float b2, float eps, float wd, int step, cudaStream_t st);
int grad_accumulate(float* acc, float* g, int64_t n, cudaStream_t st);
int nchw_to_nhwc(int dtype, const float* src, void* dst, int N, int C, int H, int W, int Cpad,
                 cudaStream_t st);
int cast_f32_to_bf16(const float* s, void* d, int64_t n, cudaStream_t st);
int cast_bf16_to_f32(const void* s, float* d, int64_t n, cudaStream_t st);
int filter_transpose(int dtype, const void* w, void* wt, int K, int RS, int C, cudaStream_t st);
// Stride-2 data gradient by output parity: the filter taps of one parity class, and the merge of the four classes.
int subfilter(int dtype, const void* wt, void* sub, int C, int K, int RS, const int* taps, int ntaps, cudaStream_t st);
int parity_interleave(int dtype, const void* c00, const void* c01, const void* c10, const void* c11, const void* addend,
                      void* dx, int N, int H, int W, int C, cudaStream_t st);

// Convolution front ends: validate, pick the kernel family, launch.
int conv_fprop(const srt_conv_desc& d, int dtype, int impl, const void* x, const void* w, void* y,
               const srt_conv_epilogue* ep, cudaStream_t st);
int conv_dgrad(const srt_conv_desc& d, int dtype, int impl, const void* dy, const void* wt,
               void* dx, const srt_conv_epilogue* ep, cudaStream_t st);
// fprop that also leaves the column sums of y for bn_finalize (bf16 tensor-core path only; ask
// conv_fprop_stats_supported first). `partial` needs conv_fprop_stats_bytes(d) bytes; *slabs receives the number
// of partial rows written.
bool conv_fprop_stats_supported(const srt_conv_desc& d, int dtype, int impl);
size_t conv_fprop_stats_bytes(const srt_conv_desc& d);
int conv_fprop_stats(const srt_conv_desc& d, int dtype, int impl, const void* x, const void* w, void* y,
                     const srt_conv_epilogue* ep, void* partial, size_t partial_bytes, int* slabs, cudaStream_t st);
int conv_wgrad(const srt_conv_desc& d, int dtype, int impl, const void* dy, const void* x,
               float* dw, void* scratch, size_t scratch_bytes, cudaStream_t st);
size_t conv_wgrad_scratch_bytes(const srt_conv_desc& d, int dtype, int impl);


// ---- transformer step ---------------------------------------------------------------------------------
// Batched GEMM D[z][m][n] = alpha * sum_k A[z][m][k] * B[z][n][k] (bf16, fp32 accumulate, tcgen05), z = (z1, z2)
// with per-operand element strides; see igemm_tcgen05.cu.
struct BgemmDesc {
  int M, N, K, Z1, Z2;
  long long lda, a_s1, a_s2;
  long long ldb, b_s1, b_s2;
  long long ldd, d_s1, d_s2;
  float alpha;
  int causal;    // skip output tiles wholly above the diagonal (n > m)
  int k_causal;  // 0 none; 1: A is zero for k > m; 2: A is zero for k < m (trims the reduction range per tile)
  int b_div = 1; // B's first batch coordinate is z1 / b_div: several A heads share one B head (grouped-query attention)
};
int bgemm_bf16(const BgemmDesc& d, const void* A, const void* B, void* D, cudaStream_t st);

int layernorm_fwd(const void* x, const float* gamma, const float* beta, void* y, float* mean, float* rstd,
                  int64_t rows, int C, float eps, cudaStream_t st);
// RMSNorm: y = x * rsqrt(mean(x^2) + eps) * gamma. Backward through layernorm_bwd with rms = 1 (mean holds zeros).
int rmsnorm_fwd(const void* x, const float* gamma, void* y, float* mean, float* rstd, int64_t rows, int C, float eps,
                cudaStream_t st);
int rmsnorm_bwd(const void* dy, const void* x, const float* gamma, const float* mean, const float* rstd, const void* addend,
                void* dx, float* dgamma, int64_t rows, int C, void* scratch, size_t scratch_bytes, cudaStream_t st);
// Rotary embedding on the heads of a [tokens][ld] matrix, in place: pairs (d, d + D/2) of every head are rotated by
// pos * theta^(-2d/D); inverse = 1 applies the transposed rotation (the gradient).
int rope_apply(void* x, int64_t tokens, int S, int heads, int D, int64_t ld, float theta, int inverse, cudaStream_t st);
// SwiGLU: y = silu(gate) * up for gu = [tokens][2F] (gate first); backward writes d(gu).
int swiglu_fwd(const void* gu, void* y, int64_t tokens, int F, cudaStream_t st);
int swiglu_bwd(const void* dy, const void* gu, void* dgu, int64_t tokens, int F, cudaStream_t st);
// out[t][g*D + d] = sum over the `group` heads of in[(b, g*group + j)][s][d]; in is [B][heads][S][D], out rows have pitch ld.
int head_group_sum(const void* in, void* out, int B, int S, int heads, int group, int D, int64_t ld, cudaStream_t st);
size_t layernorm_bwd_scratch_bytes(int C);
int layernorm_bwd(const void* dy, const void* x, const float* gamma, const float* mean, const float* rstd,
                  const void* addend, void* dx, float* dgamma, float* dbeta, int64_t rows, int C, void* scratch,
                  size_t scratch_bytes, cudaStream_t st);
int gelu_fwd(const void* x, void* y, int64_t n, cudaStream_t st);
int gelu_bwd(const void* dy, const void* x, void* dx, int64_t n, cudaStream_t st);
int causal_softmax_fwd(void* scores, int64_t Z, int S, cudaStream_t st);
int causal_softmax_bwd(const void* P, void* dP, int64_t Z, int S, cudaStream_t st);
int softmax_rows_fwd(void* scores, int64_t rows, int S, cudaStream_t st);  // whole rows, in place
// causal = 1: `in` is lower triangular and `out` feeds a GEMM with k_causal = 2; tiles that GEMM never reads are skipped.
int batched_transpose(const void* in, void* out, int R, int C, int64_t ld_in, int64_t s1, int64_t s2, int Z1, int Z2,
                      cudaStream_t st, int causal = 0);
// Column sums of a bf16 matrix, two-stage and deterministic (bias gradients): out[c] = sum_r dy[r][c].
size_t colsum_scratch_bytes(int C);
int colsum_bf16(const void* dy, int64_t rows, int C, float* out, void* scratch, size_t scratch_bytes, cudaStream_t st);
int embedding_fwd(const int32_t* ids, const float* wte, const float* wpe, void* x, int64_t tokens, int S, int C,
                  cudaStream_t st);
int embedding_bwd(const void* dx, const int32_t* ids, const int32_t* order, const int32_t* seg, int n_unique, float* dwte,
                  float* dwpe, int B, int S, int C, cudaStream_t st);
int gelu_erf_fwd(const void* x, void* y, int64_t n, cudaStream_t st);
int gelu_erf_bwd(const void* dy, const void* x, void* dx, int64_t n, cudaStream_t st);
// Shifted-window attention (Swin): tokens in natural [B][Hs][Ws] order, windows of WS x WS, cyclic shift.
struct WindowShape { int B, Hs, Ws, WS, shift; };
int window_permute(const void* in, void* out, const WindowShape& w, int C, int to_natural, cudaStream_t st);
int window_qkv(void* nat, void* qw, void* kw, void* vw, const WindowShape& w, int heads, int D, int to_natural,
               cudaStream_t st);
int relbias_build(const float* table, float* relbias, int heads, int WS, cudaStream_t st);
int window_softmax_fwd(void* scores, const float* relbias, const WindowShape& w, int heads, int ld, cudaStream_t st);
int window_softmax_bwd(const void* P, void* dP, int64_t Z, int L, int ld, cudaStream_t st);
int relbias_grad(const void* dS, float* dbias_scratch, float* dtable, int64_t windows, int heads, int WS, int ld,
                 cudaStream_t st);
int patch_merge(const void* in, void* out, int B, int Hs, int Ws, int C, int inverse, cudaStream_t st);
int transpose_pad(const void* in, void* out, int R, int C, int64_t ld_in, int64_t z_in, int64_t Z, int ld_out,
                  cudaStream_t st);
int lm_cross_entropy(void* logits, const int32_t* labels, int64_t rows, int V, int ld, float grad_scale, float* row_loss,
                     cudaStream_t st);


// Gradient exchange between data-parallel ranks (grad_exchange.cu): one all-reduce per bucket on the
// communicator's stream, bucket i behind ready[i]; the consumer stream then waits for the whole exchange.
struct Comm;
int grad_exchange_begin(Comm* c, float* grad, int nbuckets, const int64_t* offsets, const int64_t* counts,
                        const cudaEvent_t* ready, int wire_dtype);
int grad_exchange_wait(Comm* c, cudaStream_t consumer);

}  // namespace srt
