// Streaming (HBM-bound) kernels of the training step: pooling, softmax cross-entropy, bias
// gradient, fused optimizers, gradient accumulation, layout and dtype conversion.
#include "common.cuh"
#include "conv_geom.cuh"

namespace srt {

int* tc_status_device_ptr();  // igemm_tcgen05.cu: the status word srt_tc_status() reads

namespace {
constexpr int NT = 256;

inline unsigned stream_grid(int64_t n_items, int per_sm = 16) {
  int64_t blocks = (n_items + NT - 1) / NT;
  const int64_t cap = (int64_t)sm_count() * per_sm;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (unsigned)blocks;
}

// ---- max pool 3x3 stride 2 pad 1 ---------------------------------------------------------
template <typename T>
__global__ void maxpool_fwd_kernel(const T* __restrict__ x, T* __restrict__ y,
                                   uint8_t* __restrict__ argmax, int N, int H, int W, int C, int P,
                                   int Q) {
  pdl_enter();
  constexpr int V = Vec16<T>::N;
  const int CV = C / V;
  const int64_t total = (int64_t)N * P * Q * CV;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    const int cv = (int)(i % CV);
    int64_t r = i / CV;
    const int q = (int)(r % Q); r /= Q;
    const int p = (int)(r % P);
    const int n = (int)(r / P);
    float best[V];
    uint8_t arg[V];
#pragma unroll
    for (int v = 0; v < V; ++v) { best[v] = -INFINITY; arg[v] = 0; }
    for (int a = 0; a < 3; ++a) {
      const int h = p * 2 - 1 + a;
      if (h < 0 || h >= H) continue;
      for (int b = 0; b < 3; ++b) {
        const int w = q * 2 - 1 + b;
        if (w < 0 || w >= W) continue;
        Vec16<T> t;
        t.load(x + (((int64_t)n * H + h) * W + w) * C + cv * V);
        float f[V];
        t.unpack(f);
#pragma unroll
        for (int v = 0; v < V; ++v) {
          // first maximum in scan order wins; NaN propagates (torch max_pool2d semantics)
          if (f[v] > best[v] || f[v] != f[v]) { best[v] = f[v]; arg[v] = (uint8_t)(a * 3 + b); }
        }
      }
    }
    Vec16<T> o;
    o.pack(best);
    o.store(y + i * V);
#pragma unroll
    for (int v = 0; v < V; ++v) argmax[i * V + v] = arg[v];
  }
}

template <typename T>
__global__ void maxpool_bwd_kernel(const T* __restrict__ dy, const uint8_t* __restrict__ argmax,
                                   T* __restrict__ dx, int N, int H, int W, int C, int P, int Q) {
  pdl_enter();
  constexpr int V = Vec16<T>::N;
  const int CV = C / V;
  const int64_t total = (int64_t)N * H * W * CV;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    const int cv = (int)(i % CV);
    int64_t r = i / CV;
    const int w = (int)(r % W); r /= W;
    const int h = (int)(r % H);
    const int n = (int)(r / H);
    float acc[V];
#pragma unroll
    for (int v = 0; v < V; ++v) acc[v] = 0.f;
    const int p_lo = h >> 1 /* ceil((h-1)/2) */, p_hi = (h + 1) >> 1;
    const int q_lo = w >> 1, q_hi = (w + 1) >> 1;
    for (int p = p_lo; p <= p_hi; ++p) {
      if (p >= P) continue;
      const int a = h - (p * 2 - 1);
      if (a < 0 || a > 2) continue;
      for (int q = q_lo; q <= q_hi; ++q) {
        if (q >= Q) continue;
        const int b = w - (q * 2 - 1);
        if (b < 0 || b > 2) continue;
        const int64_t o = ((((int64_t)n * P + p) * Q + q) * CV + cv) * V;
        Vec16<T> t;
        t.load(dy + o);
        float f[V];
        t.unpack(f);
        const uint8_t code = (uint8_t)(a * 3 + b);
#pragma unroll
        for (int v = 0; v < V; ++v)
          if (argmax[o + v] == code) acc[v] += f[v];
      }
    }
    Vec16<T> o;
    o.pack(acc);
    o.store(dx + i * V);
  }
}

// ---- global average pool ------------------------------------------------------------------
template <typename T>
__global__ void avgpool_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, int N, int HW,
                                   int C) {
  pdl_enter();
  constexpr int V = Vec16<T>::N;
  const int CV = C / V;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)N * CV) return;
  const int cv = (int)(i % CV);
  const int n = (int)(i / CV);
  float acc[V];
#pragma unroll
  for (int v = 0; v < V; ++v) acc[v] = 0.f;
  for (int j = 0; j < HW; ++j) {
    Vec16<T> t;
    t.load(x + ((int64_t)n * HW + j) * C + cv * V);
    float f[V];
    t.unpack(f);
#pragma unroll
    for (int v = 0; v < V; ++v) acc[v] += f[v];
  }
  const float inv = 1.f / (float)HW;
#pragma unroll
  for (int v = 0; v < V; ++v) acc[v] *= inv;
  Vec16<T> o;
  o.pack(acc);
  o.store(y + i * V);
}

template <typename T>
__global__ void avgpool_bwd_kernel(const T* __restrict__ dy, T* __restrict__ dx, int N, int HW,
                                   int C) {
  pdl_enter();
  constexpr int V = Vec16<T>::N;
  const int CV = C / V;
  const int64_t total = (int64_t)N * HW * CV;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const float inv = 1.f / (float)HW;
  for (; i < total; i += stride) {
    const int cv = (int)(i % CV);
    const int n = (int)(i / ((int64_t)HW * CV));
    Vec16<T> t;
    t.load(dy + ((int64_t)n * CV + cv) * V);
    float f[V];
    t.unpack(f);
#pragma unroll
    for (int v = 0; v < V; ++v) f[v] *= inv;
    Vec16<T> o;
    o.pack(f);
    o.store(dx + i * V);
  }
}

// ---- softmax cross-entropy, one block per row ----------------------------------------------
__device__ inline float block_reduce(float v, bool is_max) {
  __shared__ float sh[32];
  __shared__ float result;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, other) : v + other;
  }
  if (lane == 0) sh[wid] = v;
  __syncthreads();
  if (wid == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    v = lane < nw ? sh[lane] : (is_max ? -INFINITY : 0.f);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, v, o);
      v = is_max ? fmaxf(v, other) : v + other;
    }
    if (lane == 0) result = v;
  }
  __syncthreads();
  const float r = result;
  __syncthreads();
  return r;
}

constexpr int kStatusBadLabel = 0xCE;  // status code: a label outside [0, classes) was skipped

template <typename T>
__global__ void softmax_ce_kernel(const T* __restrict__ logits, const int64_t* __restrict__ labels,
                                  int classes, float grad_scale, float* __restrict__ row_loss,
                                  T* __restrict__ dlogits, int* __restrict__ status) {
  pdl_enter();
  const int row = blockIdx.x;
  const T* l = logits + (size_t)row * classes;
  // A label outside [0, classes) (an ignore index, a data set with more classes than the head) must not index
  // the row: such a row contributes no loss and no gradient, and the status word reports it.
  const int64_t lab64 = labels[row];
  if (lab64 < 0 || lab64 >= (int64_t)classes) {
    if (dlogits) {
      T* d = dlogits + (size_t)row * classes;
      for (int c = threadIdx.x; c < classes; c += blockDim.x) d[c] = ElemTraits<T>::from_f(0.f);
    }
    if (threadIdx.x == 0) {
      if (row_loss) row_loss[row] = 0.f;
      if (status) atomicCAS(status, 0, kStatusBadLabel);
    }
    return;
  }
  float mx = -INFINITY;
  for (int c = threadIdx.x; c < classes; c += blockDim.x) mx = fmaxf(mx, ElemTraits<T>::to_f(l[c]));
  mx = block_reduce(mx, true);
  float se = 0.f;
  for (int c = threadIdx.x; c < classes; c += blockDim.x) se += expf(ElemTraits<T>::to_f(l[c]) - mx);
  se = block_reduce(se, false);
  const int lab = (int)lab64;
  const float inv = 1.f / se;
  if (dlogits) {
    T* d = dlogits + (size_t)row * classes;
    for (int c = threadIdx.x; c < classes; c += blockDim.x) {
      float p = expf(ElemTraits<T>::to_f(l[c]) - mx) * inv;
      if (c == lab) p -= 1.f;
      d[c] = ElemTraits<T>::from_f(p * grad_scale);
    }
  }
  if (threadIdx.x == 0 && row_loss)
    row_loss[row] = -(ElemTraits<T>::to_f(l[lab]) - mx - logf(se)) * grad_scale;
}

// out[0] (+)= sum of v[0..n) in a fixed order (single block).
__global__ void sum_f32_kernel(const float* __restrict__ v, int n, float* out, int accumulate) {
  pdl_enter();
  __shared__ double sh[NT];
  double s = 0.0;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += (double)v[i];
  sh[threadIdx.x] = s;
  __syncthreads();
  for (int o = NT / 2; o > 0; o >>= 1) {
    if (threadIdx.x < o) sh[threadIdx.x] += sh[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) out[0] = (accumulate ? out[0] : 0.f) + (float)sh[0];
}

// out[k] = sum_rows dy[r][k]; one thread per column chunk, two-stage through shared memory.
template <typename T>
__global__ void colsum_kernel(const T* __restrict__ dy, int64_t rows, int K, float* __restrict__ out) {
  pdl_enter();
  // blockDim = (32 columns, 8 row lanes)
  __shared__ float sh[8][33];
  const int k = blockIdx.x * 32 + threadIdx.x;
  float s = 0.f;
  if (k < K)
    for (int64_t r = threadIdx.y; r < rows; r += 8) s += ElemTraits<T>::to_f(dy[r * K + k]);
  sh[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && k < K) {
    float t = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) t += sh[j][threadIdx.x];
    out[k] = t;
  }
}

// ---- optimizers --------------------------------------------------------------------------
__global__ void sgd_momentum_kernel(float* __restrict__ p, const float* __restrict__ g,
                                    float* __restrict__ m, __nv_bfloat16* __restrict__ pb,
                                    int64_t n4, int64_t n, float lr, float mu, float wd,
                                    int first_step) {
  pdl_enter();
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n4; i += stride) {
    float4 pv = reinterpret_cast<float4*>(p)[i];
    const float4 gv = reinterpret_cast<const float4*>(g)[i];
    float4 mv = first_step ? make_float4(0.f, 0.f, 0.f, 0.f) : reinterpret_cast<float4*>(m)[i];
    float pp[4] = {pv.x, pv.y, pv.z, pv.w};
    const float gg[4] = {gv.x, gv.y, gv.z, gv.w};
    float mm[4] = {mv.x, mv.y, mv.z, mv.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float d = fmaf(wd, pp[j], gg[j]);
      mm[j] = first_step ? d : fmaf(mu, mm[j], d);
      pp[j] = fmaf(-lr, mm[j], pp[j]);
    }
    reinterpret_cast<float4*>(p)[i] = make_float4(pp[0], pp[1], pp[2], pp[3]);
    reinterpret_cast<float4*>(m)[i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    if (pb) {
      __nv_bfloat162 a = __floats2bfloat162_rn(pp[0], pp[1]), b = __floats2bfloat162_rn(pp[2], pp[3]);
      uint2 o;
      o.x = *reinterpret_cast<uint32_t*>(&a);
      o.y = *reinterpret_cast<uint32_t*>(&b);
      reinterpret_cast<uint2*>(pb)[i] = o;
    }
  }
  // scalar tail
  if (blockIdx.x == 0) {
    for (int64_t j = n4 * 4 + threadIdx.x; j < n; j += blockDim.x) {
      const float d = fmaf(wd, p[j], g[j]);
      const float mj = first_step ? d : fmaf(mu, m[j], d);
      m[j] = mj;
      p[j] = fmaf(-lr, mj, p[j]);
      if (pb) pb[j] = __float2bfloat16_rn(p[j]);
    }
  }
}

__global__ void adamw_kernel(float* __restrict__ p, const float* __restrict__ g,
                             float* __restrict__ m, float* __restrict__ v,
                             __nv_bfloat16* __restrict__ pb, int64_t n, float lr, float b1, float b2,
                             float eps, float wd, float bc1, float bc2_sqrt) {
  pdl_enter();
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const float step_size = lr / bc1;
  for (; i < n; i += stride) {
    const float gi = g[i];
    float pi = p[i] * (1.f - lr * wd);
    const float mi = b1 * m[i] + (1.f - b1) * gi;
    const float vi = b2 * v[i] + (1.f - b2) * gi * gi;
    const float denom = sqrtf(vi) / bc2_sqrt + eps;
    pi -= step_size * (mi / denom);
    p[i] = pi; m[i] = mi; v[i] = vi;
    if (pb) pb[i] = __float2bfloat16_rn(pi);
  }
}

__global__ void grad_accumulate_kernel(float* __restrict__ acc, float* __restrict__ g, int64_t n4,
                                       int64_t n) {
  pdl_enter();
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n4; i += stride) {
    float4 a = reinterpret_cast<float4*>(acc)[i];
    const float4 b = reinterpret_cast<float4*>(g)[i];
    a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
    reinterpret_cast<float4*>(acc)[i] = a;
    reinterpret_cast<float4*>(g)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (blockIdx.x == 0)
    for (int64_t j = n4 * 4 + threadIdx.x; j < n; j += blockDim.x) { acc[j] += g[j]; g[j] = 0.f; }
}

// ---- layout / dtype -----------------------------------------------------------------------
template <typename T>
__global__ void nchw_to_nhwc_kernel(const float* __restrict__ src, T* __restrict__ dst, int N, int C,
                                    int H, int W, int Cpad) {
  pdl_enter();
  const int64_t total = (int64_t)N * H * W * Cpad;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    const int c = (int)(i % Cpad);
    int64_t r = i / Cpad;
    const int w = (int)(r % W); r /= W;
    const int h = (int)(r % H);
    const int n = (int)(r / H);
    const float v = c < C ? src[(((int64_t)n * C + c) * H + h) * W + w] : 0.f;
    dst[i] = ElemTraits<T>::from_f(v);
  }
}

__global__ void cast_f32_bf16_kernel(const float* __restrict__ s, __nv_bfloat16* __restrict__ d,
                                     int64_t n) {
  pdl_enter();
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) d[i] = __float2bfloat16_rn(s[i]);
}
__global__ void cast_bf16_f32_kernel(const __nv_bfloat16* __restrict__ s, float* __restrict__ d,
                                     int64_t n) {
  pdl_enter();
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) d[i] = __bfloat162float(s[i]);
}

// wt[c][rs][k] = w[k][rs][c]; 32x32 shared-memory tiles, blockIdx.z = rs.
template <typename T>
__global__ void filter_transpose_kernel(const T* __restrict__ w, T* __restrict__ wt, int K, int RS,
                                        int C) {
  pdl_enter();
  __shared__ T tile[32][33];
  const int rs = blockIdx.z;
  const int c0 = blockIdx.x * 32, k0 = blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int k = k0 + j, c = c0 + threadIdx.x;
    if (k < K && c < C) tile[j][threadIdx.x] = w[((size_t)k * RS + rs) * C + c];
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int c = c0 + j, k = k0 + threadIdx.x;
    if (k < K && c < C) wt[((size_t)c * RS + rs) * K + k] = tile[threadIdx.x][j];
  }
}


// Stride-2 data gradient by output parity. sub[c][t][k] = wt[c][taps[t]][k]: the filter taps that reach one
// parity class of output pixels, in the order the class's stride-1 gather walks them.
struct TapList { int n; int rs[4]; };
template <typename T>
__global__ void subfilter_kernel(const T* __restrict__ wt, T* __restrict__ sub, int C, int K, int RS, TapList taps) {
  pdl_enter();
  constexpr int V = Vec16<T>::N;
  const int kv = K / V;
  const int64_t total = (int64_t)C * taps.n * kv;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int v = (int)(i % kv);
    const int t = (int)((i / kv) % taps.n);
    const int64_t c = i / ((int64_t)kv * taps.n);
    Vec16<T> a;
    a.load(wt + (c * RS + taps.rs[t]) * K + v * V);
    a.store(sub + (c * taps.n + t) * K + v * V);
  }
}
// dx[n][h][w][:] = class(h & 1, w & 1)[n][h / 2][w / 2][:] (+ addend); a null class contributes zero.
template <typename T>
__global__ void parity_interleave_kernel(const T* __restrict__ c00, const T* __restrict__ c01, const T* __restrict__ c10,
                                         const T* __restrict__ c11, const T* __restrict__ addend, T* __restrict__ dx, int N,
                                         int H, int W, int C) {
  pdl_enter();
  constexpr int V = Vec16<T>::N;
  const int cv = C / V;
  const int64_t total = (int64_t)N * H * W * cv;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t r = i;
    const int v = (int)(r % cv); r /= cv;
    const int w = (int)(r % W); r /= W;
    const int h = (int)(r % H);
    const int64_t n = r / H;
    const T* src = (h & 1) ? ((w & 1) ? c11 : c10) : ((w & 1) ? c01 : c00);
    float f[V];
    if (src) {
      Vec16<T> a;
      a.load(src + (((n * (H / 2) + h / 2) * (W / 2) + w / 2) * (int64_t)C) + v * V);
      a.unpack(f);
    } else {
#pragma unroll
      for (int e = 0; e < V; ++e) f[e] = 0.f;
    }
    if (addend) {
      Vec16<T> b;
      b.load(addend + i * V);
      float g[V];
      b.unpack(g);
#pragma unroll
      for (int e = 0; e < V; ++e) f[e] += g[e];
    }
    Vec16<T> o;
    o.pack(f);
    o.store(dx + i * V);
  }
}

}  // namespace

#define DISPATCH_T(dtype, ...)                                   \
  if ((dtype) == SRT_F32) { using T = float; __VA_ARGS__; }      \
  else { using T = __nv_bfloat16; __VA_ARGS__; }

int maxpool_fwd(int dtype, const void* x, void* y, uint8_t* argmax, int N, int H, int W, int C,
                cudaStream_t st) {
  SRT_REQUIRE(C % 8 == 0, "maxpool: C (%d) must be a multiple of 8", C);
  const int P = (H + 2 - 3) / 2 + 1, Q = (W + 2 - 3) / 2 + 1;
  DISPATCH_T(dtype, {
    const int64_t total = (int64_t)N * P * Q * (C / Vec16<T>::N);
    launch_pdl(maxpool_fwd_kernel<T>, dim3(stream_grid(total)), dim3(NT), 0, st, (const T*)x, (T*)y, argmax, N, H, W, C, P, Q);
  });
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}

int maxpool_bwd(int dtype, const void* dy, const uint8_t* argmax, void* dx, int N, int H, int W,
                int C, cudaStream_t st) {
  SRT_REQUIRE(C % 8 == 0, "maxpool: C (%d) must be a multiple of 8", C);
  const int P = (H + 2 - 3) / 2 + 1, Q = (W + 2 - 3) / 2 + 1;
  DISPATCH_T(dtype, {
    const int64_t total = (int64_t)N * H * W * (C / Vec16<T>::N);
    launch_pdl(maxpool_bwd_kernel<T>, dim3(stream_grid(total)), dim3(NT), 0, st, (const T*)dy, argmax, (T*)dx, N, H, W, C, P, Q);
  });
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}

int avgpool_fwd(int dtype, const void* x, void* y, int N, int HW, int C, cudaStream_t st) {
  SRT_REQUIRE(C % 8 == 0, "avgpool: C (%d) must be a multiple of 8", C);
  DISPATCH_T(dtype, {
    const int64_t total = (int64_t)N * (C / Vec16<T>::N);
    launch_pdl(avgpool_fwd_kernel<T>, dim3((unsigned)((total + NT - 1) / NT)), dim3(NT), 0, st, (const T*)x, (T*)y, N, HW, C);
  });
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}

int avgpool_bwd(int dtype, const void* dy, void* dx, int N, int HW, int C, cudaStream_t st) {
  SRT_REQUIRE(C % 8 == 0, "avgpool: C (%d) must be a multiple of 8", C);
  DISPATCH_T(dtype, {
    const int64_t total = (int64_t)N * HW * (C / Vec16<T>::N);
    launch_pdl(avgpool_bwd_kernel<T>, dim3(stream_grid(total)), dim3(NT), 0, st, (const T*)dy, (T*)dx, N, HW, C);
  });
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}

int softmax_ce(int dtype, const void* logits, const int64_t* labels, int B, int classes,
               float grad_scale, float* row_loss, void* dlogits, cudaStream_t st) {
  SRT_REQUIRE(B > 0 && classes > 0, "softmax_ce: empty input");
  DISPATCH_T(dtype, {
    launch_pdl(softmax_ce_kernel<T>, dim3(B), dim3(NT), 0, st, (const T*)logits, labels, classes, grad_scale, row_loss, (T*)dlogits,
               tc_status_device_ptr());
  });
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}

int sum_f32(const float* v, int n, float* out, int accumulate, cudaStream_t st) {
  launch_pdl(sum_f32_kernel, dim3(1), dim3(NT), 0, st, v, n, out, accumulate);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}

int colsum(int dtype, const void* dy, int64_t rows, int K, float* out, cudaStream_t st) {
  DISPATCH_T(dtype, {
    launch_pdl(colsum_kernel<T>, dim3(ceil_div(K, 32)), dim3(dim3(32, 8)), 0, st, (const T*)dy, rows, K, out);
  });
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}

int sgd_momentum(float* p, const float* g, float* m, void* pb, int64_t n, float lr, float mu,
                 float wd, int first_step, cudaStream_t st) {
  if (n == 0) return SRT_OK;
  const int64_t n4 = n / 4;
  launch_pdl(sgd_momentum_kernel, dim3(stream_grid(n4 > 0 ? n4 : 1, 8)), dim3(NT), 0, st, 
      p, g, m, (__nv_bfloat16*)pb, n4, n, lr, mu, wd, first_step);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}

int adamw(float* p, const float* g, float* m, float* v, void* pb, int64_t n, float lr, float b1,
          float b2, float eps, float wd, int step, cudaStream_t st) {
  if (n == 0) return SRT_OK;
  SRT_REQUIRE(step >= 1, "adamw: step counts from 1");
  const float bc1 = 1.f - powf(b1, (float)step);
  const float bc2 = 1.f - powf(b2, (float)step);
  launch_pdl(adamw_kernel, dim3(stream_grid(n, 8)), dim3(NT), 0, st, p, g, m, v, (__nv_bfloat16*)pb, n, lr, b1, b2, eps,
                                                 wd, bc1, sqrtf(bc2));
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}

int grad_accumulate(float* acc, float* g, int64_t n, cudaStream_t st) {
  if (n == 0) return SRT_OK;
  const int64_t n4 = n / 4;
  launch_pdl(grad_accumulate_kernel, dim3(stream_grid(n4 > 0 ? n4 : 1, 8)), dim3(NT), 0, st, acc, g, n4, n);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}

int nchw_to_nhwc(int dtype, const float* src, void* dst, int N, int C, int H, int W, int Cpad,
                 cudaStream_t st) {
  SRT_REQUIRE(Cpad >= C, "nchw_to_nhwc: Cpad < C");
  const int64_t total = (int64_t)N * H * W * Cpad;
  DISPATCH_T(dtype, {
    launch_pdl(nchw_to_nhwc_kernel<T>, dim3(stream_grid(total)), dim3(NT), 0, st, src, (T*)dst, N, C, H, W, Cpad);
  });
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}

int cast_f32_to_bf16(const float* s, void* d, int64_t n, cudaStream_t st) {
  if (n == 0) return SRT_OK;
  launch_pdl(cast_f32_bf16_kernel, dim3(stream_grid(n)), dim3(NT), 0, st, s, (__nv_bfloat16*)d, n);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}
int cast_bf16_to_f32(const void* s, float* d, int64_t n, cudaStream_t st) {
  if (n == 0) return SRT_OK;
  launch_pdl(cast_bf16_f32_kernel, dim3(stream_grid(n)), dim3(NT), 0, st, (const __nv_bfloat16*)s, d, n);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}

int filter_transpose(int dtype, const void* w, void* wt, int K, int RS, int C, cudaStream_t st) {
  dim3 grid(ceil_div(C, 32), ceil_div(K, 32), RS);
  DISPATCH_T(dtype, {
    launch_pdl(filter_transpose_kernel<T>, dim3(grid), dim3(dim3(32, 8)), 0, st, (const T*)w, (T*)wt, K, RS, C);
  });
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}

int subfilter(int dtype, const void* wt, void* sub, int C, int K, int RS, const int* taps, int ntaps, cudaStream_t st) {
  SRT_REQUIRE(ntaps >= 1 && ntaps <= 4 && K % 8 == 0, "subfilter: 1..4 taps, K a multiple of 8");
  TapList tl;
  tl.n = ntaps;
  for (int i = 0; i < 4; ++i) tl.rs[i] = i < ntaps ? taps[i] : 0;
  const int64_t total = (int64_t)C * ntaps * (K / (dtype == SRT_F32 ? 4 : 8));
  DISPATCH_T(dtype, {
    launch_pdl(subfilter_kernel<T>, dim3(stream_grid(total)), dim3(NT), 0, st, (const T*)wt, (T*)sub, C, K, RS, tl);
  });
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}

int parity_interleave(int dtype, const void* c00, const void* c01, const void* c10, const void* c11, const void* addend,
                      void* dx, int N, int H, int W, int C, cudaStream_t st) {
  SRT_REQUIRE(H % 2 == 0 && W % 2 == 0 && C % 8 == 0, "parity_interleave: even map and C % 8 == 0 required");
  const int64_t total = (int64_t)N * H * W * (C / (dtype == SRT_F32 ? 4 : 8));
  DISPATCH_T(dtype, {
    launch_pdl(parity_interleave_kernel<T>, dim3(stream_grid(total)), dim3(NT), 0, st, (const T*)c00, (const T*)c01,
               (const T*)c10, (const T*)c11, (const T*)addend, (T*)dx, N, H, W, C);
  });
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}

}  // namespace srt
