// Row-wise and elementwise kernels of the decoder-only transformer step (GPT-2 layout): LayerNorm,
// GELU (tanh form), causal softmax, token/position embedding, next-token cross-entropy, batched
// transposes for the attention products. bf16 activations, fp32 arithmetic and parameters.
//
// All of them are HBM-bound streaming passes: 16-byte vector accesses along the contiguous axis, one
// warp per row with shuffle reductions for the row-wise ones, fixed-order (deterministic) partial sums
// for the column reductions.
#include "common.cuh"
#include "ops.cuh"

namespace srt {

int* tc_status_device_ptr();  // igemm_tcgen05.cu: the status word srt_tc_status() reads

namespace {

using bf16 = __nv_bfloat16;
constexpr int NT = 256;
constexpr int WARPS = NT / 32;

__device__ inline float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ inline float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---- LayerNorm ------------------------------------------------------------------------------------
// y = (x - mean) * rstd * gamma + beta over the last axis (C % 8 == 0); one warp per row.
__global__ void __launch_bounds__(NT)
layernorm_fwd_kernel(const bf16* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
                     bf16* __restrict__ y, float* __restrict__ mean, float* __restrict__ rstd, int64_t rows, int C,
                     float eps, int rms) {
  pdl_enter();
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * WARPS + (threadIdx.x >> 5);
  if (row >= rows) return;
  const bf16* xr = x + row * C;
  const int nv = C / 8;
  float s = 0.f;
  if (!rms) {
    for (int v = lane; v < nv; v += 32) {
      Vec16<bf16> a;
      a.load(xr + v * 8);
      float f[8];
      a.unpack(f);
#pragma unroll
      for (int e = 0; e < 8; ++e) s += f[e];
    }
  }
  const float mu = rms ? 0.f : warp_sum(s) / (float)C;
  float q = 0.f;
  for (int v = lane; v < nv; v += 32) {
    Vec16<bf16> a;
    a.load(xr + v * 8);
    float f[8];
    a.unpack(f);
#pragma unroll
    for (int e = 0; e < 8; ++e) { const float d = f[e] - mu; q = fmaf(d, d, q); }
  }
  const float rs = rsqrtf(warp_sum(q) / (float)C + eps);
  if (lane == 0) { mean[row] = mu; rstd[row] = rs; }
  bf16* yr = y + row * C;
  for (int v = lane; v < nv; v += 32) {
    Vec16<bf16> a;
    a.load(xr + v * 8);
    float f[8];
    a.unpack(f);
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = (f[e] - mu) * rs * gamma[v * 8 + e] + (beta ? beta[v * 8 + e] : 0.f);
    Vec16<bf16> o;
    o.pack(f);
    o.store(yr + v * 8);
  }
}

// dx = rstd * (g - mean(g) - xhat * mean(g * xhat)), g = dy * gamma; plus an optional addend (the gradient
// that reaches x through the residual connection). One warp per row.
__global__ void __launch_bounds__(NT)
layernorm_bwd_dx_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, const float* __restrict__ gamma,
                        const float* __restrict__ mean, const float* __restrict__ rstd,
                        const bf16* __restrict__ addend, bf16* __restrict__ dx, int64_t rows, int C, int rms) {
  pdl_enter();
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * WARPS + (threadIdx.x >> 5);
  if (row >= rows) return;
  const bf16 *dr = dy + row * C, *xr = x + row * C;
  const float mu = mean[row], rs = rstd[row];
  const int nv = C / 8;
  float sg = 0.f, sgx = 0.f;
  for (int v = lane; v < nv; v += 32) {
    Vec16<bf16> a, b;
    a.load(dr + v * 8);
    b.load(xr + v * 8);
    float g[8], f[8];
    a.unpack(g);
    b.unpack(f);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float ge = g[e] * gamma[v * 8 + e];
      sg += ge;
      sgx = fmaf(ge, (f[e] - mu) * rs, sgx);
    }
  }
  const float mg = rms ? 0.f : warp_sum(sg) / (float)C, mgx = warp_sum(sgx) / (float)C;
  for (int v = lane; v < nv; v += 32) {
    Vec16<bf16> a, b;
    a.load(dr + v * 8);
    b.load(xr + v * 8);
    float g[8], f[8], r[8];
    a.unpack(g);
    b.unpack(f);
    if (addend) {
      Vec16<bf16> c;
      c.load(addend + row * C + v * 8);
      c.unpack(r);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) r[e] = 0.f;
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float xh = (f[e] - mu) * rs;
      r[e] += rs * (g[e] * gamma[v * 8 + e] - mg - xh * mgx);
    }
    Vec16<bf16> o;
    o.pack(r);
    o.store(dx + row * C + v * 8);
  }
}

// Column reductions over a [rows][C] bf16 matrix, deterministic and two-stage. MODE 0: sum of dy (bias gradients).
// MODE 1: (sum of dy * xhat, sum of dy) with xhat = (x - mean[row]) * rstd[row] (LayerNorm / RMSNorm parameter gradients).
// Stage 1: grid (ceil(C/256), slabs); a block is 32 vector lanes (8 columns each) x 8 row lanes and walks its slab of
// rows with 16-byte loads; partial[(slab * NOUT + o) * C + c]. Stage 2 adds the slabs in order.
constexpr int CR_MAX_SLABS = 600;
template <int MODE>
__global__ void __launch_bounds__(NT)
colreduce_partial_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, const float* __restrict__ mean,
                         const float* __restrict__ rstd, int64_t rows, int C, int64_t rows_per_slab,
                         float* __restrict__ partial) {
  pdl_enter();
  constexpr int NOUT = MODE == 0 ? 1 : 2;
  __shared__ float sh[NOUT][8][256 + 8];
  const int vl = threadIdx.x & 31, rl = threadIdx.x >> 5;
  const int c0 = blockIdx.x * 256 + vl * 8;
  const int64_t r0 = (int64_t)blockIdx.y * rows_per_slab;
  const int64_t r1 = r0 + rows_per_slab < rows ? r0 + rows_per_slab : rows;
  float a0[8], a1[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) { a0[e] = 0.f; a1[e] = 0.f; }
  if (c0 < C) {
    for (int64_t r = r0 + rl; r < r1; r += 8) {
      Vec16<bf16> g;
      g.load(dy + r * C + c0);
      float gf[8];
      g.unpack(gf);
      if (MODE == 0) {
#pragma unroll
        for (int e = 0; e < 8; ++e) a0[e] += gf[e];
      } else {
        Vec16<bf16> xv;
        xv.load(x + r * C + c0);
        float xf[8];
        xv.unpack(xf);
        const float mu = mean[r], rs = rstd[r];
#pragma unroll
        for (int e = 0; e < 8; ++e) { a0[e] = fmaf(gf[e], (xf[e] - mu) * rs, a0[e]); a1[e] += gf[e]; }
      }
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    sh[0][rl][vl * 8 + e] = a0[e];
    if (NOUT == 2) sh[NOUT - 1][rl][vl * 8 + e] = a1[e];
  }
  __syncthreads();
  const int c = blockIdx.x * 256 + threadIdx.x;  // one column per thread for the lane sum
  if (c < C) {
#pragma unroll
    for (int o = 0; o < NOUT; ++o) {
      float t = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) t += sh[o][j][threadIdx.x];
      partial[((size_t)blockIdx.y * NOUT + o) * C + c] = t;
    }
  }
}
// Stage 2: block = 32 columns x 8 slab lanes; lane l adds slabs l, l + 8, ... in order, then the eight lane sums are
// added in lane order (fixed shape: deterministic).
__global__ void __launch_bounds__(NT)
colreduce_final_kernel(const float* __restrict__ partial, int slabs, int nout, int C, float* __restrict__ out0,
                       float* __restrict__ out1) {
  pdl_enter();
  __shared__ float sh[2][8][33];
  const int cl = threadIdx.x & 31, lane = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cl;
  float t0 = 0.f, t1 = 0.f;
  if (c < C) {
    for (int b = lane; b < slabs; b += 8) {
      t0 += partial[((size_t)b * nout) * C + c];
      if (nout == 2) t1 += partial[((size_t)b * nout + 1) * C + c];
    }
  }
  sh[0][lane][cl] = t0;
  sh[1][lane][cl] = t1;
  __syncthreads();
  if (lane == 0 && c < C) {
    float a = 0.f, b = 0.f;
#pragma unroll
    for (int l = 0; l < 8; ++l) { a += sh[0][l][cl]; b += sh[1][l][cl]; }
    out0[c] = a;
    if (nout == 2) out1[c] = b;
  }
}

// ---- GELU, tanh form ("gelu_new") -------------------------------------------------------------------
__device__ inline float gelu_f(float x) {
  const float k = 0.7978845608028654f;  // sqrt(2/pi)
  return 0.5f * x * (1.f + tanhf(k * (x + 0.044715f * x * x * x)));
}
__device__ inline float gelu_grad_f(float x) {
  const float k = 0.7978845608028654f;
  const float u = k * (x + 0.044715f * x * x * x);
  const float t = tanhf(u);
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * k * (1.f + 3.f * 0.044715f * x * x);
}
__global__ void __launch_bounds__(NT)
gelu_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, int64_t nvec) {
  pdl_enter();
  for (int64_t v = (int64_t)blockIdx.x * NT + threadIdx.x; v < nvec; v += (int64_t)gridDim.x * NT) {
    Vec16<bf16> a;
    a.load(x + v * 8);
    float f[8];
    a.unpack(f);
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = gelu_f(f[e]);
    Vec16<bf16> o;
    o.pack(f);
    o.store(y + v * 8);
  }
}
__global__ void __launch_bounds__(NT)
gelu_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, bf16* __restrict__ dx, int64_t nvec) {
  pdl_enter();
  for (int64_t v = (int64_t)blockIdx.x * NT + threadIdx.x; v < nvec; v += (int64_t)gridDim.x * NT) {
    Vec16<bf16> a, b;
    a.load(dy + v * 8);
    b.load(x + v * 8);
    float g[8], f[8];
    a.unpack(g);
    b.unpack(f);
#pragma unroll
    for (int e = 0; e < 8; ++e) g[e] *= gelu_grad_f(f[e]);
    Vec16<bf16> o;
    o.pack(g);
    o.store(dx + v * 8);
  }
}

// ---- causal softmax over [Z][S][S] scores, in place ---------------------------------------------------
// Row r keeps columns 0..r; the rest of the row is written as zero (the tiles above the diagonal were never
// produced by the score GEMM, and the products that follow read whole rows). One warp per row.
__global__ void __launch_bounds__(NT)
causal_softmax_fwd_kernel(bf16* __restrict__ s, int64_t total_rows, int S) {
  pdl_enter();
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * WARPS + (threadIdx.x >> 5);
  if (row >= total_rows) return;
  const int r = (int)(row % S);
  bf16* p = s + row * S;
  const int nv = S / 8, lastv = r / 8;  // vectors 0..lastv hold valid columns
  float mx = -INFINITY;
  for (int v = lane; v <= lastv; v += 32) {
    Vec16<bf16> a;
    a.load(p + v * 8);
    float f[8];
    a.unpack(f);
#pragma unroll
    for (int e = 0; e < 8; ++e) if (v * 8 + e <= r) mx = fmaxf(mx, f[e]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
  for (int v = lane; v <= lastv; v += 32) {
    Vec16<bf16> a;
    a.load(p + v * 8);
    float f[8];
    a.unpack(f);
#pragma unroll
    for (int e = 0; e < 8; ++e) if (v * 8 + e <= r) sum += __expf(f[e] - mx);
  }
  const float inv = 1.f / warp_sum(sum);
  for (int v = lane; v < nv; v += 32) {
    float f[8];
    if (v <= lastv) {
      Vec16<bf16> a;
      a.load(p + v * 8);
      a.unpack(f);
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = v * 8 + e <= r ? __expf(f[e] - mx) * inv : 0.f;
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = 0.f;
    }
    Vec16<bf16> o;
    o.pack(f);
    o.store(p + v * 8);
  }
}
// Softmax over whole rows of S columns, in place (bidirectional attention without a padding mask). One warp per row.
__global__ void __launch_bounds__(NT)
softmax_rows_kernel(bf16* __restrict__ s, int64_t total_rows, int S) {
  pdl_enter();
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * WARPS + (threadIdx.x >> 5);
  if (row >= total_rows) return;
  bf16* p = s + row * S;
  const int nv = S / 8;
  float mx = -INFINITY;
  for (int v = lane; v < nv; v += 32) {
    Vec16<bf16> a;
    a.load(p + v * 8);
    float f[8];
    a.unpack(f);
#pragma unroll
    for (int e = 0; e < 8; ++e) mx = fmaxf(mx, f[e]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
  for (int v = lane; v < nv; v += 32) {
    Vec16<bf16> a;
    a.load(p + v * 8);
    float f[8];
    a.unpack(f);
#pragma unroll
    for (int e = 0; e < 8; ++e) sum += __expf(f[e] - mx);
  }
  const float inv = 1.f / warp_sum(sum);
  for (int v = lane; v < nv; v += 32) {
    Vec16<bf16> a;
    a.load(p + v * 8);
    float f[8];
    a.unpack(f);
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = __expf(f[e] - mx) * inv;
    Vec16<bf16> o;
    o.pack(f);
    o.store(p + v * 8);
  }
}
// dS = P * (dP - sum_j P_j dP_j) on the valid part of each row, zero elsewhere; in place over dP.
__global__ void __launch_bounds__(NT)
causal_softmax_bwd_kernel(const bf16* __restrict__ P, bf16* __restrict__ dP, int64_t total_rows, int S) {
  pdl_enter();
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * WARPS + (threadIdx.x >> 5);
  if (row >= total_rows) return;
  const int r = (int)(row % S);
  const bf16* p = P + row * S;
  bf16* d = dP + row * S;
  const int nv = S / 8, lastv = r / 8;
  float dot = 0.f;
  for (int v = lane; v <= lastv; v += 32) {
    Vec16<bf16> a, b;
    a.load(p + v * 8);
    b.load(d + v * 8);
    float pf[8], df[8];
    a.unpack(pf);
    b.unpack(df);
#pragma unroll
    for (int e = 0; e < 8; ++e) if (v * 8 + e <= r) dot = fmaf(pf[e], df[e], dot);
  }
  dot = warp_sum(dot);
  for (int v = lane; v < nv; v += 32) {
    float o[8];
    if (v <= lastv) {
      Vec16<bf16> a, b;
      a.load(p + v * 8);
      b.load(d + v * 8);
      float pf[8], df[8];
      a.unpack(pf);
      b.unpack(df);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = v * 8 + e <= r ? pf[e] * (df[e] - dot) : 0.f;
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = 0.f;
    }
    Vec16<bf16> w;
    w.pack(o);
    w.store(d + v * 8);
  }
}

// ---- batched transpose: out[z][c][r] = in[z][r][c] ----------------------------------------------------
// in: row stride ld_in, batch strides (s1 for z1, s2 for z2), z = z2 * Z1 + z1; out: contiguous [Z][C][R].
__global__ void __launch_bounds__(256)
transpose_kernel(const bf16* __restrict__ in, bf16* __restrict__ out, int R, int C, int64_t ld_in, int64_t s1,
                 int64_t s2, int Z1, int causal) {
  pdl_enter();
  // causal: the input is lower triangular and the consumer of out (a GEMM whose reduction starts at the 128-aligned
  // row block of each output tile) never reads out[c][r] with r below the 128-row block that holds c
  if (causal && (int)blockIdx.y * 32 + 32 <= ((int)blockIdx.x * 32 / 128) * 128) return;
  __shared__ bf16 tile[32][33];
  const int z = blockIdx.z, z1 = z % Z1, z2 = z / Z1;
  const bf16* src = in + (int64_t)z1 * s1 + (int64_t)z2 * s2;
  bf16* dst = out + (int64_t)z * R * C;
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = r0 + ty + i * 8, c = c0 + tx;
    if (r < R && c < C) tile[ty + i * 8][tx] = src[(int64_t)r * ld_in + c];
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = c0 + ty + i * 8, r = r0 + tx;
    if (r < R && c < C) dst[(int64_t)c * R + r] = tile[tx][ty + i * 8];
  }
}

// ---- embedding ----------------------------------------------------------------------------------------
__global__ void __launch_bounds__(NT)
embedding_fwd_kernel(const int32_t* __restrict__ ids, const float* __restrict__ wte, const float* __restrict__ wpe,
                     bf16* __restrict__ x, int64_t tokens, int S, int C) {
  pdl_enter();
  const int nv = C / 8;
  for (int64_t i = (int64_t)blockIdx.x * NT + threadIdx.x; i < tokens * nv; i += (int64_t)gridDim.x * NT) {
    const int64_t t = i / nv;
    const int v = (int)(i - t * nv);
    const float* a = wte + (int64_t)ids[t] * C + v * 8;
    float f[8];
    if (wpe) {
      const float* b = wpe + (int64_t)(t % S) * C + v * 8;
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = a[e] + b[e];
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = a[e];
    }
    Vec16<bf16> o;
    o.pack(f);
    o.store(x + t * C + v * 8);
  }
}
// Position table gradient: dwpe[s][c] = sum over the batch, in batch order.
__global__ void __launch_bounds__(NT)
embedding_bwd_pos_kernel(const bf16* __restrict__ dx, float* __restrict__ dwpe, int B, int S, int C) {
  pdl_enter();
  for (int64_t i = (int64_t)blockIdx.x * NT + threadIdx.x; i < (int64_t)S * C; i += (int64_t)gridDim.x * NT) {
    float acc = 0.f;
    for (int b = 0; b < B; ++b) acc += __bfloat162float(dx[(int64_t)b * S * C + i]);
    dwpe[i] = acc;
  }
}
// Token table gradient, added to what the tied output projection left there. `order` lists the token
// positions sorted by token id (ties by position), seg[u]..seg[u+1] is the run of the u-th distinct id:
// one block per distinct id adds its occurrences in that fixed order (deterministic, no atomics).
__global__ void __launch_bounds__(NT)
embedding_bwd_tok_kernel(const bf16* __restrict__ dx, const int32_t* __restrict__ ids, const int32_t* __restrict__ order,
                         const int32_t* __restrict__ seg, int n_unique, float* __restrict__ dwte, int C) {
  pdl_enter();
  const int u = blockIdx.x;
  if (u >= n_unique) return;
  const int a = seg[u], b = seg[u + 1];
  const int64_t tok = ids[order[a]];
  for (int c = threadIdx.x; c < C; c += NT) {
    float acc = 0.f;
    for (int j = a; j < b; ++j) acc += __bfloat162float(dx[(int64_t)order[j] * C + c]);
    dwte[tok * C + c] += acc;
  }
}

// ---- next-token cross-entropy -------------------------------------------------------------------------
// logits [rows][ld] (V valid columns); label[row] < 0 = no target (the last position of each sequence).
// row_loss[row] = -log softmax(logits)[label]; logits are overwritten with (softmax - onehot) * grad_scale,
// zero in rows without a target and in the padding columns. One block per row.
__global__ void __launch_bounds__(NT)
lm_cross_entropy_kernel(bf16* __restrict__ logits, const int32_t* __restrict__ labels, int V, int ld, float grad_scale,
                        float* __restrict__ row_loss, int* __restrict__ status) {
  pdl_enter();
  __shared__ float red[WARPS];
  __shared__ float bcast;
  const int64_t row = blockIdx.x;
  bf16* z = logits + row * ld;
  const int label = labels[row];
  const int nv = ld / 8, lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  // label < 0 marks a position without a target (the last token of a sequence); a label at or beyond the
  // vocabulary is a caller error: neither may index the row, both give no loss and no gradient, the second is
  // reported through the status word.
  if (label < 0 || label >= V) {
    for (int v = threadIdx.x; v < nv; v += NT) *reinterpret_cast<uint4*>(z + v * 8) = make_uint4(0, 0, 0, 0);
    if (threadIdx.x == 0) {
      row_loss[row] = 0.f;
      if (label >= V && status) atomicCAS(status, 0, 0xCE);
    }
    return;
  }
  float mx = -INFINITY;
  for (int v = threadIdx.x; v < nv; v += NT) {
    Vec16<bf16> a;
    a.load(z + v * 8);
    float f[8];
    a.unpack(f);
#pragma unroll
    for (int e = 0; e < 8; ++e) if (v * 8 + e < V) mx = fmaxf(mx, f[e]);
  }
  mx = warp_max(mx);
  if (lane == 0) red[w] = mx;
  __syncthreads();
  if (threadIdx.x == 0) { float m = red[0]; for (int i = 1; i < WARPS; ++i) m = fmaxf(m, red[i]); bcast = m; }
  __syncthreads();
  mx = bcast;
  __syncthreads();
  float sum = 0.f;
  for (int v = threadIdx.x; v < nv; v += NT) {
    Vec16<bf16> a;
    a.load(z + v * 8);
    float f[8];
    a.unpack(f);
#pragma unroll
    for (int e = 0; e < 8; ++e) if (v * 8 + e < V) sum += __expf(f[e] - mx);
  }
  sum = warp_sum(sum);
  if (lane == 0) red[w] = sum;
  __syncthreads();
  if (threadIdx.x == 0) { float t = 0.f; for (int i = 0; i < WARPS; ++i) t += red[i]; bcast = t; }
  __syncthreads();
  const float total = bcast;
  const float inv = 1.f / total;
  if (threadIdx.x == 0) row_loss[row] = logf(total) + mx - __bfloat162float(z[label]);
  __syncthreads();  // the label's logit is read before anyone overwrites it
  for (int v = threadIdx.x; v < nv; v += NT) {
    Vec16<bf16> a;
    a.load(z + v * 8);
    float f[8];
    a.unpack(f);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int c = v * 8 + e;
      f[e] = c < V ? (__expf(f[e] - mx) * inv - (c == label ? 1.f : 0.f)) * grad_scale : 0.f;
    }
    Vec16<bf16> o;
    o.pack(f);
    o.store(z + v * 8);
  }
}

// ---- GELU, erf form (torch.nn.GELU default) -------------------------------------------------------------
__device__ inline float gelu_erf_f(float x) { return 0.5f * x * (1.f + erff(x * 0.7071067811865476f)); }
__device__ inline float gelu_erf_grad_f(float x) {
  return 0.5f * (1.f + erff(x * 0.7071067811865476f)) + x * 0.3989422804014327f * __expf(-0.5f * x * x);
}
__global__ void __launch_bounds__(NT)
gelu_erf_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, int64_t nvec) {
  pdl_enter();
  for (int64_t v = (int64_t)blockIdx.x * NT + threadIdx.x; v < nvec; v += (int64_t)gridDim.x * NT) {
    Vec16<bf16> a;
    a.load(x + v * 8);
    float f[8];
    a.unpack(f);
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = gelu_erf_f(f[e]);
    Vec16<bf16> o;
    o.pack(f);
    o.store(y + v * 8);
  }
}
__global__ void __launch_bounds__(NT)
gelu_erf_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, bf16* __restrict__ dx, int64_t nvec) {
  pdl_enter();
  for (int64_t v = (int64_t)blockIdx.x * NT + threadIdx.x; v < nvec; v += (int64_t)gridDim.x * NT) {
    Vec16<bf16> a, b;
    a.load(dy + v * 8);
    b.load(x + v * 8);
    float g[8], f[8];
    a.unpack(g);
    b.unpack(f);
#pragma unroll
    for (int e = 0; e < 8; ++e) g[e] *= gelu_erf_grad_f(f[e]);
    Vec16<bf16> o;
    o.pack(g);
    o.store(dx + v * 8);
  }
}

// ---- shifted-window attention helpers (Swin) ------------------------------------------------------------
// Tokens live in the natural [B][Hs][Ws] order. A window of WS x WS tokens of the cyclically shifted map is
// window (wy, wx), token (iy, ix): shifted position (wy*WS+iy, wx*WS+ix), natural position that plus `shift`
// modulo the map size.
struct WinGeom {
  int B, Hs, Ws, WS, shift, nWy, nWx;
};
__device__ inline int64_t win_token_to_natural(const WinGeom& g, int64_t win, int tok) {
  const int wx = (int)(win % g.nWx);
  const int wy = (int)((win / g.nWx) % g.nWy);
  const int64_t b = win / ((int64_t)g.nWx * g.nWy);
  const int iy = tok / g.WS, ix = tok - iy * g.WS;
  int h = wy * g.WS + iy + g.shift, w = wx * g.WS + ix + g.shift;
  if (h >= g.Hs) h -= g.Hs;
  if (w >= g.Ws) w -= g.Ws;
  return (b * g.Hs + h) * g.Ws + w;
}
// dir 0: out_win[win][tok][c] = in_nat[natural][c]; dir 1: out_nat[natural][c] = in_win[win][tok][c]. C % 8 == 0.
__global__ void __launch_bounds__(NT)
window_permute_kernel(const bf16* __restrict__ in, bf16* __restrict__ out, WinGeom g, int C, int dir) {
  pdl_enter();
  const int nv = C / 8, L = g.WS * g.WS;
  const int64_t total = (int64_t)g.B * g.nWy * g.nWx * L * nv;
  for (int64_t i = (int64_t)blockIdx.x * NT + threadIdx.x; i < total; i += (int64_t)gridDim.x * NT) {
    const int v = (int)(i % nv);
    const int64_t wt = i / nv;
    const int tok = (int)(wt % L);
    const int64_t win = wt / L;
    const int64_t nat = win_token_to_natural(g, win, tok);
    const int64_t a = wt * C + v * 8, b = nat * C + v * 8;
    *reinterpret_cast<uint4*>(out + (dir ? b : a)) = *reinterpret_cast<const uint4*>(in + (dir ? a : b));
  }
}
// Fused projection [tokens][3][heads][D] <-> per-head windowed Q, K, V [win][head][tok][D].
// dir 0: natural -> windowed; dir 1: windowed -> natural (the gradient path).
__global__ void __launch_bounds__(NT)
window_qkv_kernel(bf16* __restrict__ nat, bf16* __restrict__ qw, bf16* __restrict__ kw, bf16* __restrict__ vw, WinGeom g,
                  int heads, int D, int dir, int parts) {
  pdl_enter();
  const int dv = D / 8, L = g.WS * g.WS, C = heads * D;
  const int64_t total = (int64_t)g.B * g.nWy * g.nWx * L * parts * heads * dv;
  for (int64_t i = (int64_t)blockIdx.x * NT + threadIdx.x; i < total; i += (int64_t)gridDim.x * NT) {
    int64_t r = i;
    const int v = (int)(r % dv); r /= dv;
    const int hd = (int)(r % heads); r /= heads;
    const int part = (int)(r % parts); r /= parts;
    const int tok = (int)(r % L);
    const int64_t win = r / L;
    const int64_t n = win_token_to_natural(g, win, tok);
    bf16* natp = nat + n * parts * C + (int64_t)part * C + hd * D + v * 8;
    bf16* w = (part == 0 ? qw : part == 1 ? kw : vw) + ((win * heads + hd) * L + tok) * D + v * 8;
    if (dir == 0) *reinterpret_cast<uint4*>(w) = *reinterpret_cast<const uint4*>(natp);
    else *reinterpret_cast<uint4*>(natp) = *reinterpret_cast<const uint4*>(w);
  }
}
// relbias[head][i][j] = table[index(i, j)][head], index = (iy_i - iy_j + WS-1) * (2WS-1) + (ix_i - ix_j + WS-1)
__device__ inline int relpos_index(int i, int j, int WS) {
  const int iy = i / WS, ix = i - iy * WS, jy = j / WS, jx = j - jy * WS;
  return (iy - jy + WS - 1) * (2 * WS - 1) + (ix - jx + WS - 1);
}
__global__ void __launch_bounds__(NT)
relbias_build_kernel(const float* __restrict__ table, float* __restrict__ relbias, int heads, int WS) {
  pdl_enter();
  const int L = WS * WS;
  for (int i = blockIdx.x * NT + threadIdx.x; i < heads * L * L; i += gridDim.x * NT) {
    const int j = i % L, r = (i / L) % L, hd = i / (L * L);
    relbias[i] = table[relpos_index(r, j, WS) * heads + hd];
  }
}
__device__ inline int shift_region(int p, int size, int WS, int shift) {  // region of a shifted coordinate
  return p < size - WS ? 0 : (p < size - shift ? 1 : 2);
}
// scores [Z][L][ld] (Z = windows * heads, head fastest): P = softmax(scores + relbias + mask) over the L valid
// columns, columns L..ld-1 are written as zero. One warp per row.
__global__ void __launch_bounds__(NT)
window_softmax_fwd_kernel(bf16* __restrict__ s, const float* __restrict__ relbias, WinGeom g, int heads, int ld,
                          int64_t total_rows) {
  pdl_enter();
  const int lane = threadIdx.x & 31, L = g.WS * g.WS;
  const int64_t row = (int64_t)blockIdx.x * WARPS + (threadIdx.x >> 5);
  if (row >= total_rows) return;
  const int i = (int)(row % L);
  const int64_t z = row / L;
  const int hd = (int)(z % heads);
  const int64_t win = z / heads;
  bf16* p = s + row * ld;
  const float* rb = relbias + ((int64_t)hd * L + i) * L;
  int reg_i = 0;
  const int wx = (int)(win % g.nWx), wy = (int)((win / g.nWx) % g.nWy);
  if (g.shift > 0) {
    const int iy = i / g.WS, ix = i - iy * g.WS;
    reg_i = shift_region(wy * g.WS + iy, g.Hs, g.WS, g.shift) * 3 + shift_region(wx * g.WS + ix, g.Ws, g.WS, g.shift);
  }
  float vals[4];  // L <= 128 columns per warp
  float mx = -INFINITY;
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const int j = lane + 32 * t;
    float v = -INFINITY;
    if (j < L) {
      v = __bfloat162float(p[j]) + rb[j];
      if (g.shift > 0) {
        const int jy = j / g.WS, jx = j - jy * g.WS;
        const int reg_j = shift_region(wy * g.WS + jy, g.Hs, g.WS, g.shift) * 3 + shift_region(wx * g.WS + jx, g.Ws, g.WS, g.shift);
        if (reg_j != reg_i) v += -100.f;
      }
      mx = fmaxf(mx, v);
    }
    vals[t] = v;
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const int j = lane + 32 * t;
    if (j < L) { vals[t] = __expf(vals[t] - mx); sum += vals[t]; }
  }
  const float inv = 1.f / warp_sum(sum);
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const int j = lane + 32 * t;
    if (j < ld) p[j] = __float2bfloat16_rn(j < L ? vals[t] * inv : 0.f);
  }
}
__global__ void __launch_bounds__(NT)
window_softmax_bwd_kernel(const bf16* __restrict__ P, bf16* __restrict__ dP, int L, int ld, int64_t total_rows) {
  pdl_enter();
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * WARPS + (threadIdx.x >> 5);
  if (row >= total_rows) return;
  const bf16* p = P + row * ld;
  bf16* d = dP + row * ld;
  float pv[4], dv[4], dot = 0.f;
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const int j = lane + 32 * t;
    pv[t] = j < L ? __bfloat162float(p[j]) : 0.f;
    dv[t] = j < L ? __bfloat162float(d[j]) : 0.f;
    dot = fmaf(pv[t], dv[t], dot);
  }
  dot = warp_sum(dot);
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const int j = lane + 32 * t;
    if (j < ld) d[j] = __float2bfloat16_rn(j < L ? pv[t] * (dv[t] - dot) : 0.f);
  }
}
// Gradient of the relative-position table. Stage 1: sum dS over the windows for every (head, i, j), in window
// order; stage 2: add the (i, j) pairs that share a table entry, in (i, j) order.
__global__ void __launch_bounds__(512)
relbias_grad_sum_kernel(const bf16* __restrict__ dS, float* __restrict__ dbias, int64_t windows, int heads, int L, int ld) {
  pdl_enter();
  // block = (head, i); 64 columns x 8 window lanes; lane l adds windows l, l + 8, ... in order
  __shared__ float sh[8][65];
  const int i = blockIdx.x % L, hd = blockIdx.x / L;
  const int j = threadIdx.x & 63, lane = threadIdx.x >> 6;
  float acc = 0.f;
  if (j < L)
    for (int64_t w = lane; w < windows; w += 8) acc += __bfloat162float(dS[((w * heads + hd) * L + i) * ld + j]);
  sh[lane][j] = acc;
  __syncthreads();
  if (lane == 0 && j < L) {
    float t = 0.f;
#pragma unroll
    for (int l = 0; l < 8; ++l) t += sh[l][j];
    dbias[((int64_t)hd * L + i) * L + j] = t;
  }
}
// entry t = (dy, dx) of the table collects the pairs (i, j) with i - j = (dy, dx): at most L of them, walked in j order
__global__ void __launch_bounds__(NT)
relbias_grad_table_kernel(const float* __restrict__ dbias, float* __restrict__ dtable, int heads, int WS) {
  pdl_enter();
  const int L = WS * WS, side = 2 * WS - 1;
  const int idx = blockIdx.x * NT + threadIdx.x;
  if (idx >= side * side * heads) return;
  const int hd = idx % heads, t = idx / heads;
  const int dy = t / side - (WS - 1), dx = t % side - (WS - 1);
  float acc = 0.f;
  for (int jy = max(0, -dy); jy < min(WS, WS - dy); ++jy)
    for (int jx = max(0, -dx); jx < min(WS, WS - dx); ++jx) {
      const int j = jy * WS + jx, i = (jy + dy) * WS + jx + dx;
      acc += dbias[((int64_t)hd * L + i) * L + j];
    }
  dtable[idx] = acc;
}

// Patch merging: out[b][h/2][w/2][part*C + c] = in[b][h][w][c], part = (w odd) * 2 + (h odd). dir 1 is the inverse.
__global__ void __launch_bounds__(NT)
patch_merge_kernel(const bf16* __restrict__ in, bf16* __restrict__ out, int B, int Hs, int Ws, int C, int dir) {
  pdl_enter();
  const int nv = C / 8;
  const int64_t total = (int64_t)B * Hs * Ws * nv;
  for (int64_t i = (int64_t)blockIdx.x * NT + threadIdx.x; i < total; i += (int64_t)gridDim.x * NT) {
    int64_t r = i;
    const int v = (int)(r % nv); r /= nv;
    const int w = (int)(r % Ws); r /= Ws;
    const int h = (int)(r % Hs);
    const int64_t b = r / Hs;
    const int part = (w & 1) * 2 + (h & 1);
    const int64_t src = ((b * Hs + h) * Ws + w) * C + v * 8;
    const int64_t dst = (((b * (Hs / 2) + h / 2) * (Ws / 2) + w / 2) * 4 + part) * (int64_t)C + v * 8;
    *reinterpret_cast<uint4*>(out + (dir ? src : dst)) = *reinterpret_cast<const uint4*>(in + (dir ? dst : src));
  }
}

// out[z][c][r] = in[z][r][c] with output row pitch ld_out >= R; the pad columns are written as zero.
__global__ void __launch_bounds__(256)
transpose_pad_kernel(const bf16* __restrict__ in, bf16* __restrict__ out, int R, int C, int64_t ld_in, int64_t z_in,
                     int ld_out) {
  pdl_enter();
  __shared__ bf16 tile[32][33];
  const bf16* src = in + (int64_t)blockIdx.z * z_in;
  bf16* dst = out + (int64_t)blockIdx.z * C * ld_out;
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = r0 + ty + i * 8, c = c0 + tx;
    tile[ty + i * 8][tx] = (r < R && c < C) ? src[(int64_t)r * ld_in + c] : __float2bfloat16_rn(0.f);
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = c0 + ty + i * 8, r = r0 + tx;
    if (c < C && r < ld_out) dst[(int64_t)c * ld_out + r] = tile[tx][ty + i * 8];
  }
}


// ---- rotary embedding, SwiGLU, grouped-head sums (Qwen2 layout) ----------------------------------------------
__global__ void __launch_bounds__(NT)
rope_kernel(bf16* __restrict__ x, int64_t tokens, int S, int heads, int D, int64_t ld, float log_theta, int inverse) {
  pdl_enter();
  const int half = D / 2;
  const int64_t total = tokens * heads * half;
  for (int64_t i = (int64_t)blockIdx.x * NT + threadIdx.x; i < total; i += (int64_t)gridDim.x * NT) {
    const int d = (int)(i % half);
    const int hd = (int)((i / half) % heads);
    const int64_t t = i / ((int64_t)half * heads);
    const float ang = (float)(t % S) * __expf(-log_theta * (2.f * (float)d / (float)D));
    float sn, cs;
    sincosf(ang, &sn, &cs);
    if (inverse) sn = -sn;
    bf16* p = x + t * ld + (int64_t)hd * D + d;
    const float a = __bfloat162float(p[0]), b = __bfloat162float(p[half]);
    p[0] = __float2bfloat16_rn(a * cs - b * sn);
    p[half] = __float2bfloat16_rn(b * cs + a * sn);
  }
}
__global__ void __launch_bounds__(NT)
swiglu_fwd_kernel(const bf16* __restrict__ gu, bf16* __restrict__ y, int64_t tokens, int F) {
  pdl_enter();
  const int nv = F / 8;
  for (int64_t i = (int64_t)blockIdx.x * NT + threadIdx.x; i < tokens * nv; i += (int64_t)gridDim.x * NT) {
    const int64_t t = i / nv;
    const int v = (int)(i - t * nv);
    Vec16<bf16> a, b;
    a.load(gu + t * 2 * F + v * 8);
    b.load(gu + t * 2 * F + F + v * 8);
    float g[8], u[8];
    a.unpack(g);
    b.unpack(u);
#pragma unroll
    for (int e = 0; e < 8; ++e) g[e] = g[e] / (1.f + __expf(-g[e])) * u[e];
    Vec16<bf16> o;
    o.pack(g);
    o.store(y + t * F + v * 8);
  }
}
__global__ void __launch_bounds__(NT)
swiglu_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ gu, bf16* __restrict__ dgu, int64_t tokens, int F) {
  pdl_enter();
  const int nv = F / 8;
  for (int64_t i = (int64_t)blockIdx.x * NT + threadIdx.x; i < tokens * nv; i += (int64_t)gridDim.x * NT) {
    const int64_t t = i / nv;
    const int v = (int)(i - t * nv);
    Vec16<bf16> a, b, c;
    a.load(gu + t * 2 * F + v * 8);
    b.load(gu + t * 2 * F + F + v * 8);
    c.load(dy + t * F + v * 8);
    float g[8], u[8], d[8], dg[8], du[8];
    a.unpack(g);
    b.unpack(u);
    c.unpack(d);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float sg = 1.f / (1.f + __expf(-g[e]));
      const float silu = g[e] * sg;
      du[e] = d[e] * silu;
      dg[e] = d[e] * u[e] * (sg + silu * (1.f - sg));
    }
    Vec16<bf16> o1, o2;
    o1.pack(dg);
    o2.pack(du);
    o1.store(dgu + t * 2 * F + v * 8);
    o2.store(dgu + t * 2 * F + F + v * 8);
  }
}
__global__ void __launch_bounds__(NT)
head_group_sum_kernel(const bf16* __restrict__ in, bf16* __restrict__ out, int B, int S, int heads, int group, int D,
                      int64_t ld) {
  pdl_enter();
  const int dv = D / 8, kvh = heads / group;
  const int64_t total = (int64_t)B * S * kvh * dv;
  for (int64_t i = (int64_t)blockIdx.x * NT + threadIdx.x; i < total; i += (int64_t)gridDim.x * NT) {
    int64_t r = i;
    const int v = (int)(r % dv); r /= dv;
    const int g = (int)(r % kvh); r /= kvh;
    const int s = (int)(r % S);
    const int64_t b = r / S;
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    for (int j = 0; j < group; ++j) {
      Vec16<bf16> a;
      a.load(in + (((b * heads + g * group + j) * S + s) * (int64_t)D) + v * 8);
      float f[8];
      a.unpack(f);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += f[e];
    }
    Vec16<bf16> o;
    o.pack(acc);
    o.store(out + (b * S + s) * ld + (int64_t)g * D + v * 8);
  }
}

inline unsigned rows_grid(int64_t rows) { return (unsigned)((rows + WARPS - 1) / WARPS); }
inline unsigned stream_blocks(int64_t work_items) {
  int64_t b = (work_items + NT - 1) / NT;
  const int64_t cap = (int64_t)sm_count() * 8;
  return (unsigned)(b < 1 ? 1 : b > cap ? cap : b);
}

}  // namespace

int layernorm_fwd(const void* x, const float* gamma, const float* beta, void* y, float* mean, float* rstd,
                  int64_t rows, int C, float eps, cudaStream_t st) {
  SRT_REQUIRE(rows > 0 && C % 8 == 0, "layernorm: C (%d) must be a multiple of 8", C);
  launch_pdl(layernorm_fwd_kernel, dim3(rows_grid(rows)), dim3(NT), 0, st, (const bf16*)x, gamma, beta, (bf16*)y, mean,
             rstd, rows, C, eps, 0);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}

int rmsnorm_fwd(const void* x, const float* gamma, void* y, float* mean, float* rstd, int64_t rows, int C, float eps,
                cudaStream_t st) {
  SRT_REQUIRE(rows > 0 && C % 8 == 0, "rmsnorm: C (%d) must be a multiple of 8", C);
  launch_pdl(layernorm_fwd_kernel, dim3(rows_grid(rows)), dim3(NT), 0, st, (const bf16*)x, gamma, (const float*)nullptr,
             (bf16*)y, mean, rstd, rows, C, eps, 1);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}

size_t layernorm_bwd_scratch_bytes(int C) { return (size_t)CR_MAX_SLABS * 2 * C * sizeof(float) + (size_t)C * sizeof(float) + 256; }

// Two-stage column reduction front end (see colreduce_partial_kernel). mode 0: out0 = column sums of dy; mode 1: norm
// parameter gradients (out0 = sum dy * xhat, out1 = sum dy).
static int colreduce(int mode, const void* dy, const void* x, const float* mean, const float* rstd, int64_t rows, int C,
                     float* out0, float* out1, void* scratch, size_t scratch_bytes, cudaStream_t st) {
  const int gx = ceil_div(C, 256), nout = mode == 0 ? 1 : 2;
  int64_t slabs = (int64_t)4 * sm_count() / gx;
  if (slabs > CR_MAX_SLABS) slabs = CR_MAX_SLABS;
  if (slabs > (rows + 63) / 64) slabs = (rows + 63) / 64;
  if (slabs < 1) slabs = 1;
  const int64_t per = (rows + slabs - 1) / slabs;
  slabs = (rows + per - 1) / per;
  SRT_REQUIRE(scratch && scratch_bytes >= (size_t)slabs * nout * C * sizeof(float), "column reduction: scratch too small");
  if (mode == 0)
    launch_pdl(colreduce_partial_kernel<0>, dim3(gx, (unsigned)slabs), dim3(NT), 0, st, (const bf16*)dy, (const bf16*)nullptr,
               (const float*)nullptr, (const float*)nullptr, rows, C, per, (float*)scratch);
  else
    launch_pdl(colreduce_partial_kernel<1>, dim3(gx, (unsigned)slabs), dim3(NT), 0, st, (const bf16*)dy, (const bf16*)x, mean,
               rstd, rows, C, per, (float*)scratch);
  SRT_LAUNCH_CHECK();
  launch_pdl(colreduce_final_kernel, dim3(ceil_div(C, 32)), dim3(NT), 0, st, (const float*)scratch, (int)slabs, nout, C, out0,
             out1);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}

size_t colsum_scratch_bytes(int C) { return (size_t)CR_MAX_SLABS * C * sizeof(float) + 256; }
int colsum_bf16(const void* dy, int64_t rows, int C, float* out, void* scratch, size_t scratch_bytes, cudaStream_t st) {
  SRT_REQUIRE(rows > 0 && C % 8 == 0, "colsum: C (%d) must be a multiple of 8", C);
  return colreduce(0, dy, nullptr, nullptr, nullptr, rows, C, out, nullptr, scratch, scratch_bytes, st);
}

static int norm_bwd(const void* dy, const void* x, const float* gamma, const float* mean, const float* rstd,
                    const void* addend, void* dx, float* dgamma, float* dbeta, int64_t rows, int C, void* scratch,
                    size_t scratch_bytes, int rms, cudaStream_t st) {
  SRT_REQUIRE(rows > 0 && C % 8 == 0, "layernorm_bwd: C (%d) must be a multiple of 8", C);
  launch_pdl(layernorm_bwd_dx_kernel, dim3(rows_grid(rows)), dim3(NT), 0, st, (const bf16*)dy, (const bf16*)x, gamma,
             mean, rstd, (const bf16*)addend, (bf16*)dx, rows, C, rms);
  SRT_LAUNCH_CHECK();
  return colreduce(1, dy, x, mean, rstd, rows, C, dgamma, dbeta, scratch, scratch_bytes, st);
}
int layernorm_bwd(const void* dy, const void* x, const float* gamma, const float* mean, const float* rstd,
                  const void* addend, void* dx, float* dgamma, float* dbeta, int64_t rows, int C, void* scratch,
                  size_t scratch_bytes, cudaStream_t st) {
  return norm_bwd(dy, x, gamma, mean, rstd, addend, dx, dgamma, dbeta, rows, C, scratch, scratch_bytes, 0, st);
}
// The column sums of dy (what would be d beta) land in the tail of the scratch and are dropped.
int rmsnorm_bwd(const void* dy, const void* x, const float* gamma, const float* mean, const float* rstd, const void* addend,
                void* dx, float* dgamma, int64_t rows, int C, void* scratch, size_t scratch_bytes, cudaStream_t st) {
  const size_t part = (size_t)CR_MAX_SLABS * 2 * C * sizeof(float);
  SRT_REQUIRE(scratch_bytes >= part + (size_t)C * sizeof(float), "rmsnorm_bwd: scratch too small");
  float* dummy = (float*)((char*)scratch + part);
  return norm_bwd(dy, x, gamma, mean, rstd, addend, dx, dgamma, dummy, rows, C, scratch, part, 1, st);
}

int gelu_fwd(const void* x, void* y, int64_t n, cudaStream_t st) {
  SRT_REQUIRE(n > 0 && n % 8 == 0, "gelu: element count must be a multiple of 8");
  launch_pdl(gelu_fwd_kernel, dim3(stream_blocks(n / 8)), dim3(NT), 0, st, (const bf16*)x, (bf16*)y, n / 8);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}
int gelu_bwd(const void* dy, const void* x, void* dx, int64_t n, cudaStream_t st) {
  SRT_REQUIRE(n > 0 && n % 8 == 0, "gelu: element count must be a multiple of 8");
  launch_pdl(gelu_bwd_kernel, dim3(stream_blocks(n / 8)), dim3(NT), 0, st, (const bf16*)dy, (const bf16*)x, (bf16*)dx,
             n / 8);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}

int causal_softmax_fwd(void* scores, int64_t Z, int S, cudaStream_t st) {
  SRT_REQUIRE(Z > 0 && S % 8 == 0, "causal_softmax: S (%d) must be a multiple of 8", S);
  launch_pdl(causal_softmax_fwd_kernel, dim3(rows_grid(Z * S)), dim3(NT), 0, st, (bf16*)scores, Z * S, S);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}
int softmax_rows_fwd(void* scores, int64_t rows, int S, cudaStream_t st) {
  SRT_REQUIRE(rows > 0 && S % 8 == 0, "softmax_rows: S (%d) must be a multiple of 8", S);
  launch_pdl(softmax_rows_kernel, dim3(rows_grid(rows)), dim3(NT), 0, st, (bf16*)scores, rows, S);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}
int causal_softmax_bwd(const void* P, void* dP, int64_t Z, int S, cudaStream_t st) {
  SRT_REQUIRE(Z > 0 && S % 8 == 0, "causal_softmax: S (%d) must be a multiple of 8", S);
  launch_pdl(causal_softmax_bwd_kernel, dim3(rows_grid(Z * S)), dim3(NT), 0, st, (const bf16*)P, (bf16*)dP, Z * S, S);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}

int batched_transpose(const void* in, void* out, int R, int C, int64_t ld_in, int64_t s1, int64_t s2, int Z1, int Z2,
                      cudaStream_t st, int causal) {
  SRT_REQUIRE(R > 0 && C > 0 && Z1 > 0 && Z2 > 0 && (int64_t)Z1 * Z2 <= 65535, "transpose: bad shape");
  launch_pdl(transpose_kernel, dim3(ceil_div(C, 32), ceil_div(R, 32), Z1 * Z2), dim3(256), 0, st, (const bf16*)in,
             (bf16*)out, R, C, ld_in, s1, s2, Z1, causal);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}

int embedding_fwd(const int32_t* ids, const float* wte, const float* wpe, void* x, int64_t tokens, int S, int C,
                  cudaStream_t st) {
  SRT_REQUIRE(tokens > 0 && C % 8 == 0, "embedding: C must be a multiple of 8");
  launch_pdl(embedding_fwd_kernel, dim3(stream_blocks(tokens * (C / 8))), dim3(NT), 0, st, ids, wte, wpe, (bf16*)x, tokens,
             S, C);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}
int embedding_bwd(const void* dx, const int32_t* ids, const int32_t* order, const int32_t* seg, int n_unique, float* dwte,
                  float* dwpe, int B, int S, int C, cudaStream_t st) {
  if (dwpe) {  // models with a learned position table
    launch_pdl(embedding_bwd_pos_kernel, dim3(stream_blocks((int64_t)S * C)), dim3(NT), 0, st, (const bf16*)dx, dwpe, B, S,
               C);
    SRT_LAUNCH_CHECK();
  }
  launch_pdl(embedding_bwd_tok_kernel, dim3(n_unique), dim3(NT), 0, st, (const bf16*)dx, ids, order, seg, n_unique, dwte,
             C);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}

int lm_cross_entropy(void* logits, const int32_t* labels, int64_t rows, int V, int ld, float grad_scale, float* row_loss,
                     cudaStream_t st) {
  SRT_REQUIRE(rows > 0 && ld % 8 == 0 && V <= ld, "lm_cross_entropy: ld (%d) must be a multiple of 8 and >= V", ld);
  launch_pdl(lm_cross_entropy_kernel, dim3((unsigned)rows), dim3(NT), 0, st, (bf16*)logits, labels, V, ld, grad_scale,
             row_loss, tc_status_device_ptr());
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}


int gelu_erf_fwd(const void* x, void* y, int64_t n, cudaStream_t st) {
  SRT_REQUIRE(n > 0 && n % 8 == 0, "gelu: element count must be a multiple of 8");
  launch_pdl(gelu_erf_fwd_kernel, dim3(stream_blocks(n / 8)), dim3(NT), 0, st, (const bf16*)x, (bf16*)y, n / 8);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}
int gelu_erf_bwd(const void* dy, const void* x, void* dx, int64_t n, cudaStream_t st) {
  SRT_REQUIRE(n > 0 && n % 8 == 0, "gelu: element count must be a multiple of 8");
  launch_pdl(gelu_erf_bwd_kernel, dim3(stream_blocks(n / 8)), dim3(NT), 0, st, (const bf16*)dy, (const bf16*)x,
             (bf16*)dx, n / 8);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}

static WinGeom make_geom(const WindowShape& w) {
  WinGeom g = {w.B, w.Hs, w.Ws, w.WS, w.shift, w.Hs / w.WS, w.Ws / w.WS};
  return g;
}
static int check_geom(const WindowShape& w) {
  SRT_REQUIRE(w.B > 0 && w.WS > 0 && w.Hs % w.WS == 0 && w.Ws % w.WS == 0 && w.shift >= 0 && w.shift < w.WS &&
                  w.WS * w.WS <= 128,
              "window attention: the map (%d x %d) must be a multiple of the window (%d), window area <= 128", w.Hs, w.Ws, w.WS);
  return SRT_OK;
}
int window_permute(const void* in, void* out, const WindowShape& w, int C, int to_natural, cudaStream_t st) {
  if (int rc = check_geom(w)) return rc;
  SRT_REQUIRE(C % 8 == 0, "window_permute: C must be a multiple of 8");
  const int64_t items = (int64_t)w.B * w.Hs * w.Ws * (C / 8);
  launch_pdl(window_permute_kernel, dim3(stream_blocks(items)), dim3(NT), 0, st, (const bf16*)in, (bf16*)out, make_geom(w), C,
             to_natural);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}
int window_qkv(void* nat, void* qw, void* kw, void* vw, const WindowShape& w, int heads, int D, int to_natural,
               cudaStream_t st) {
  if (int rc = check_geom(w)) return rc;
  SRT_REQUIRE(D % 8 == 0, "window_qkv: head size must be a multiple of 8");
  const int parts = kw ? 3 : 1;  // one tensor [tokens][heads*D] or the fused [tokens][3][heads*D]
  const int64_t items = (int64_t)w.B * w.Hs * w.Ws * parts * heads * (D / 8);
  launch_pdl(window_qkv_kernel, dim3(stream_blocks(items)), dim3(NT), 0, st, (bf16*)nat, (bf16*)qw, (bf16*)kw, (bf16*)vw,
             make_geom(w), heads, D, to_natural, parts);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}
int relbias_build(const float* table, float* relbias, int heads, int WS, cudaStream_t st) {
  launch_pdl(relbias_build_kernel, dim3(ceil_div(heads * WS * WS * WS * WS, NT)), dim3(NT), 0, st, table, relbias, heads, WS);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}
int window_softmax_fwd(void* scores, const float* relbias, const WindowShape& w, int heads, int ld, cudaStream_t st) {
  if (int rc = check_geom(w)) return rc;
  const int64_t rows = (int64_t)w.B * (w.Hs / w.WS) * (w.Ws / w.WS) * heads * w.WS * w.WS;
  SRT_REQUIRE(ld >= w.WS * w.WS && ld <= 128, "window_softmax: bad row pitch %d", ld);
  launch_pdl(window_softmax_fwd_kernel, dim3(rows_grid(rows)), dim3(NT), 0, st, (bf16*)scores, relbias, make_geom(w), heads,
             ld, rows);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}
int window_softmax_bwd(const void* P, void* dP, int64_t Z, int L, int ld, cudaStream_t st) {
  SRT_REQUIRE(Z > 0 && L <= ld && ld <= 128, "window_softmax_bwd: bad shape");
  launch_pdl(window_softmax_bwd_kernel, dim3(rows_grid(Z * L)), dim3(NT), 0, st, (const bf16*)P, (bf16*)dP, L, ld, Z * L);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}
int relbias_grad(const void* dS, float* dbias_scratch, float* dtable, int64_t windows, int heads, int WS, int ld,
                 cudaStream_t st) {
  const int L = WS * WS;
  SRT_REQUIRE(L <= 64, "relbias_grad: window area above 64");
  launch_pdl(relbias_grad_sum_kernel, dim3(heads * L), dim3(512), 0, st, (const bf16*)dS, dbias_scratch, windows, heads, L, ld);
  SRT_LAUNCH_CHECK();
  launch_pdl(relbias_grad_table_kernel, dim3(ceil_div((2 * WS - 1) * (2 * WS - 1) * heads, NT)), dim3(NT), 0, st,
             (const float*)dbias_scratch, dtable, heads, WS);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}
int patch_merge(const void* in, void* out, int B, int Hs, int Ws, int C, int inverse, cudaStream_t st) {
  SRT_REQUIRE(Hs % 2 == 0 && Ws % 2 == 0 && C % 8 == 0, "patch_merge: even map and C % 8 == 0 required");
  launch_pdl(patch_merge_kernel, dim3(stream_blocks((int64_t)B * Hs * Ws * (C / 8))), dim3(NT), 0, st, (const bf16*)in,
             (bf16*)out, B, Hs, Ws, C, inverse);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}
int transpose_pad(const void* in, void* out, int R, int C, int64_t ld_in, int64_t z_in, int64_t Z, int ld_out,
                  cudaStream_t st) {
  SRT_REQUIRE(R > 0 && C > 0 && Z > 0 && ld_out >= R, "transpose_pad: bad shape");
  // z is spread over grid.z in chunks (the grid's z extent is limited to 65535)
  for (int64_t z0 = 0; z0 < Z; z0 += 65535) {
    const int64_t zn = Z - z0 < 65535 ? Z - z0 : 65535;
    launch_pdl(transpose_pad_kernel, dim3(ceil_div(C, 32), ceil_div(ld_out, 32), (unsigned)zn), dim3(256), 0, st,
               (const bf16*)in + z0 * z_in, (bf16*)out + z0 * C * ld_out, R, C, ld_in, z_in, ld_out);
    SRT_LAUNCH_CHECK();
  }
  return SRT_OK;
}

int rope_apply(void* x, int64_t tokens, int S, int heads, int D, int64_t ld, float theta, int inverse, cudaStream_t st) {
  SRT_REQUIRE(tokens > 0 && D % 2 == 0 && heads > 0, "rope: head size must be even");
  launch_pdl(rope_kernel, dim3(stream_blocks(tokens * heads * (D / 2))), dim3(NT), 0, st, (bf16*)x, tokens, S, heads, D, ld,
             logf(theta), inverse);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}
int swiglu_fwd(const void* gu, void* y, int64_t tokens, int F, cudaStream_t st) {
  SRT_REQUIRE(tokens > 0 && F % 8 == 0, "swiglu: F must be a multiple of 8");
  launch_pdl(swiglu_fwd_kernel, dim3(stream_blocks(tokens * (F / 8))), dim3(NT), 0, st, (const bf16*)gu, (bf16*)y, tokens, F);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}
int swiglu_bwd(const void* dy, const void* gu, void* dgu, int64_t tokens, int F, cudaStream_t st) {
  SRT_REQUIRE(tokens > 0 && F % 8 == 0, "swiglu: F must be a multiple of 8");
  launch_pdl(swiglu_bwd_kernel, dim3(stream_blocks(tokens * (F / 8))), dim3(NT), 0, st, (const bf16*)dy, (const bf16*)gu,
             (bf16*)dgu, tokens, F);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}
int head_group_sum(const void* in, void* out, int B, int S, int heads, int group, int D, int64_t ld, cudaStream_t st) {
  SRT_REQUIRE(heads % group == 0 && D % 8 == 0, "head_group_sum: bad grouping");
  launch_pdl(head_group_sum_kernel, dim3(stream_blocks((int64_t)B * S * (heads / group) * (D / 8))), dim3(NT), 0, st,
             (const bf16*)in, (bf16*)out, B, S, heads, group, D, ld);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}

}  // namespace srt
