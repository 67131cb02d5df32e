// BatchNorm (training mode) over NHWC rows: statistics, fused apply (+residual, +ReLU), backward.
//
// All kernels are HBM-bound streaming passes: 16-byte vector loads along the channel axis (the
// contiguous one), fp32 per-thread accumulation over a short run of rows, double-precision
// combination of the per-thread and per-slab partial sums in a fixed order (deterministic, and
// accurate enough for the fp32 parity mode).
#include "common.cuh"

namespace srt {

namespace {

constexpr int NT = 256;
constexpr int ROWS_PER_THREAD = 32;

struct RowMap {
  int CV;    // 16-byte vectors per row
  int TC;    // threads across channel vectors in a block
  int RL;    // row lanes in a block
  int slab;  // rows per block
  int S;     // number of slabs (grid.x)
  int GY;    // channel chunks (grid.y)
};

inline RowMap make_row_map(int64_t rows, int C, int V) {
  RowMap m;
  m.CV = C / V;
  m.TC = m.CV < NT ? m.CV : NT;
  m.RL = NT / m.TC;
  m.slab = m.RL * ROWS_PER_THREAD;
  m.S = (int)((rows + m.slab - 1) / m.slab);
  m.GY = (m.CV + m.TC - 1) / m.TC;
  return m;
}

// Reduce per-thread accumulators a[V], b[V] over the block's row lanes; lane 0 of each channel
// vector writes the slab partial as doubles: partial[(slab*C + c)*2 + {0,1}].
template <int V>
__device__ inline void block_reduce_store(const float (&a)[V], const float (&b)[V], const RowMap& m,
                                          int tc, int rl, int cv, int C, double* partial) {
  __shared__ float sh_a[NT * V];
  __shared__ float sh_b[NT * V];
  const int t = threadIdx.x;
#pragma unroll
  for (int v = 0; v < V; ++v) { sh_a[t * V + v] = a[v]; sh_b[t * V + v] = b[v]; }
  __syncthreads();
  if (rl == 0 && cv < m.CV) {
#pragma unroll
    for (int v = 0; v < V; ++v) {
      double sa = 0.0, sb = 0.0;
      for (int r = 0; r < m.RL; ++r) {
        sa += (double)sh_a[(r * m.TC + tc) * V + v];
        sb += (double)sh_b[(r * m.TC + tc) * V + v];
      }
      const size_t o = ((size_t)blockIdx.x * C + (size_t)cv * V + v) * 2;
      partial[o] = sa;
      partial[o + 1] = sb;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(NT)
bn_stats_partial(const T* __restrict__ z, int64_t rows, int C, RowMap m, double* partial) {
  constexpr int V = Vec16<T>::N;
  const int t = threadIdx.x;
  const int tc = t % m.TC, rl = t / m.TC;
  const int cv = blockIdx.y * m.TC + tc;
  float s[V], q[V];
#pragma unroll
  for (int v = 0; v < V; ++v) { s[v] = 0.f; q[v] = 0.f; }
  if (rl < m.RL && cv < m.CV) {
    const int64_t r0 = (int64_t)blockIdx.x * m.slab;
    const int64_t r1 = r0 + m.slab < rows ? r0 + m.slab : rows;
    for (int64_t r = r0 + rl; r < r1; r += m.RL) {
      Vec16<T> x;
      x.load(z + r * C + (int64_t)cv * V);
      float f[V];
      x.unpack(f);
#pragma unroll
      for (int v = 0; v < V; ++v) { s[v] += f[v]; q[v] = fmaf(f[v], f[v], q[v]); }
    }
  }
  block_reduce_store<V>(s, q, m, tc, rl, cv, C, partial);
}

__global__ void bn_stats_finalize(const double* __restrict__ partial, int S, int C, int64_t rows,
                                  const float* __restrict__ gamma, const float* __restrict__ beta,
                                  float eps, float momentum, float* running_mean,
                                  float* running_var, float* mean, float* invstd, float* scale,
                                  float* shift) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  double s = 0.0, q = 0.0;
  for (int i = 0; i < S; ++i) {
    s += partial[((size_t)i * C + c) * 2];
    q += partial[((size_t)i * C + c) * 2 + 1];
  }
  const double mu = s / (double)rows;
  double var = q / (double)rows - mu * mu;
  if (var < 0.0) var = 0.0;
  const float is = (float)(1.0 / sqrt(var + (double)eps));
  const float g = gamma ? gamma[c] : 1.f, b = beta ? beta[c] : 0.f;
  mean[c] = (float)mu;
  invstd[c] = is;
  const float sc = g * is;
  scale[c] = sc;
  shift[c] = b - (float)mu * sc;
  if (running_mean) running_mean[c] = (1.f - momentum) * running_mean[c] + momentum * (float)mu;
  if (running_var) {
    const double unbiased = rows > 1 ? var * (double)rows / (double)(rows - 1) : var;
    running_var[c] = (1.f - momentum) * running_var[c] + momentum * (float)unbiased;
  }
}

template <typename T>
__global__ void __launch_bounds__(NT)
bn_apply_kernel(const T* __restrict__ z, const T* residual, T* y, int64_t nvec, int CV,
                const float* __restrict__ scale, const float* __restrict__ shift, int relu) {
  constexpr int V = Vec16<T>::N;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < nvec; i += stride) {
    const int cv = (int)(i % CV);
    Vec16<T> x;
    x.load(z + i * V);
    float f[V];
    x.unpack(f);
    float sc[V], sh[V];
#pragma unroll
    for (int v = 0; v < V; v += 4) {
      float4 a = *reinterpret_cast<const float4*>(scale + cv * V + v);
      float4 b = *reinterpret_cast<const float4*>(shift + cv * V + v);
      sc[v] = a.x; sc[v + 1] = a.y; sc[v + 2] = a.z; sc[v + 3] = a.w;
      sh[v] = b.x; sh[v + 1] = b.y; sh[v + 2] = b.z; sh[v + 3] = b.w;
    }
#pragma unroll
    for (int v = 0; v < V; ++v) f[v] = fmaf(f[v], sc[v], sh[v]);
    if (residual) {
      Vec16<T> rv;
      rv.load(residual + i * V);
      float rf[V];
      rv.unpack(rf);
#pragma unroll
      for (int v = 0; v < V; ++v) f[v] += rf[v];
    }
    if (relu) {
#pragma unroll
      for (int v = 0; v < V; ++v) f[v] = fmaxf(f[v], 0.f);
    }
    Vec16<T> o;
    o.pack(f);
    o.store(y + i * V);
  }
}

template <typename T>
__global__ void __launch_bounds__(NT)
bn_bwd_partial(const T* __restrict__ dy, const T* __restrict__ y, const T* __restrict__ z,
               int64_t rows, int C, RowMap m, const float* __restrict__ mean,
               const float* __restrict__ invstd, int relu, double* partial) {
  constexpr int V = Vec16<T>::N;
  const int t = threadIdx.x;
  const int tc = t % m.TC, rl = t / m.TC;
  const int cv = blockIdx.y * m.TC + tc;
  float sg[V], sgx[V];
#pragma unroll
  for (int v = 0; v < V; ++v) { sg[v] = 0.f; sgx[v] = 0.f; }
  if (rl < m.RL && cv < m.CV) {
    float mu[V], is[V];
#pragma unroll
    for (int v = 0; v < V; ++v) { mu[v] = mean[cv * V + v]; is[v] = invstd[cv * V + v]; }
    const int64_t r0 = (int64_t)blockIdx.x * m.slab;
    const int64_t r1 = r0 + m.slab < rows ? r0 + m.slab : rows;
    for (int64_t r = r0 + rl; r < r1; r += m.RL) {
      const int64_t o = r * C + (int64_t)cv * V;
      Vec16<T> a, b;
      a.load(dy + o);
      b.load(z + o);
      float g[V], x[V];
      a.unpack(g);
      b.unpack(x);
      if (relu) {
        Vec16<T> c;
        c.load(y + o);
        float yy[V];
        c.unpack(yy);
#pragma unroll
        for (int v = 0; v < V; ++v) g[v] = yy[v] > 0.f ? g[v] : 0.f;
      }
#pragma unroll
      for (int v = 0; v < V; ++v) {
        sg[v] += g[v];
        sgx[v] = fmaf(g[v], (x[v] - mu[v]) * is[v], sgx[v]);
      }
    }
  }
  block_reduce_store<V>(sg, sgx, m, tc, rl, cv, C, partial);
}

// coef[c*4 + {0,1,2}] = gamma*invstd, dbeta/rows, dgamma/rows
__global__ void bn_bwd_finalize(const double* __restrict__ partial, int S, int C, int64_t rows,
                                const float* __restrict__ gamma, const float* __restrict__ invstd,
                                float* dgamma, float* dbeta, float* coef) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  double s = 0.0, q = 0.0;
  for (int i = 0; i < S; ++i) {
    s += partial[((size_t)i * C + c) * 2];
    q += partial[((size_t)i * C + c) * 2 + 1];
  }
  if (dbeta) dbeta[c] = (float)s;
  if (dgamma) dgamma[c] = (float)q;
  const float g = gamma ? gamma[c] : 1.f;
  coef[c * 4 + 0] = g * invstd[c];
  coef[c * 4 + 1] = (float)(s / (double)rows);
  coef[c * 4 + 2] = (float)(q / (double)rows);
  coef[c * 4 + 3] = 0.f;
}

template <typename T>
__global__ void __launch_bounds__(NT)
bn_bwd_apply(const T* __restrict__ dy, const T* __restrict__ y, const T* __restrict__ z, T* dz,
             T* dres, int64_t nvec, int CV, const float* __restrict__ mean,
             const float* __restrict__ invstd, const float* __restrict__ coef, int relu) {
  constexpr int V = Vec16<T>::N;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < nvec; i += stride) {
    const int cv = (int)(i % CV);
    Vec16<T> a, b;
    a.load(dy + i * V);
    b.load(z + i * V);
    float g[V], x[V];
    a.unpack(g);
    b.unpack(x);
    if (relu) {
      Vec16<T> c;
      c.load(y + i * V);
      float yy[V];
      c.unpack(yy);
#pragma unroll
      for (int v = 0; v < V; ++v) g[v] = yy[v] > 0.f ? g[v] : 0.f;
    }
    if (dres) {
      Vec16<T> o;
      o.pack(g);
      o.store(dres + i * V);
    }
    float out[V];
#pragma unroll
    for (int v = 0; v < V; ++v) {
      const int c = cv * V + v;
      const float4 k = *reinterpret_cast<const float4*>(coef + c * 4);
      const float xhat = (x[v] - mean[c]) * invstd[c];
      out[v] = k.x * (g[v] - k.y - xhat * k.z);
    }
    Vec16<T> o;
    o.pack(out);
    o.store(dz + i * V);
  }
}

inline unsigned stream_grid(int64_t nvec) {
  int64_t blocks = (nvec + NT - 1) / NT;
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (unsigned)blocks;
}

}  // namespace

size_t bn_scratch_bytes(int64_t rows, int C) {
  // worst case over both element types: fp32 has the fewest channels per vector
  RowMap m4 = make_row_map(rows, C, 4), m8 = make_row_map(rows, C, 8);
  const size_t S = (size_t)(m4.S > m8.S ? m4.S : m8.S);
  return S * C * 2 * sizeof(double) + (size_t)C * 4 * sizeof(float) + 256;
}

template <typename T>
static int bn_stats_t(const void* z, int64_t rows, int C, const float* gamma, const float* beta,
                      float eps, float momentum, float* rm, float* rv, float* mean, float* invstd,
                      float* scale, float* shift, void* scratch, cudaStream_t st) {
  RowMap m = make_row_map(rows, C, Vec16<T>::N);
  double* partial = (double*)scratch;
  bn_stats_partial<T><<<dim3(m.S, m.GY), NT, 0, st>>>((const T*)z, rows, C, m, partial);
  SRT_LAUNCH_CHECK();
  bn_stats_finalize<<<ceil_div(C, 128), 128, 0, st>>>(partial, m.S, C, rows, gamma, beta, eps,
                                                     momentum, rm, rv, mean, invstd, scale, shift);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}

int bn_stats(int dtype, const void* z, int64_t rows, int C, const float* gamma, const float* beta,
             float eps, float momentum, float* rm, float* rv, float* mean, float* invstd,
             float* scale, float* shift, void* scratch, size_t scratch_bytes, cudaStream_t st) {
  SRT_REQUIRE(C % 8 == 0 && rows > 0, "bn_stats: C (%d) must be a multiple of 8, rows > 0", C);
  SRT_REQUIRE(scratch && scratch_bytes >= bn_scratch_bytes(rows, C), "bn_stats: scratch too small");
  if (dtype == SRT_F32)
    return bn_stats_t<float>(z, rows, C, gamma, beta, eps, momentum, rm, rv, mean, invstd, scale,
                             shift, scratch, st);
  return bn_stats_t<__nv_bfloat16>(z, rows, C, gamma, beta, eps, momentum, rm, rv, mean, invstd,
                                   scale, shift, scratch, st);
}

int bn_apply(int dtype, const void* z, const void* residual, void* y, int64_t rows, int C,
             const float* scale, const float* shift, int relu, cudaStream_t st) {
  SRT_REQUIRE(C % 8 == 0, "bn_apply: C (%d) must be a multiple of 8", C);
  if (dtype == SRT_F32) {
    const int64_t nvec = rows * C / 4;
    bn_apply_kernel<float><<<stream_grid(nvec), NT, 0, st>>>(
        (const float*)z, (const float*)residual, (float*)y, nvec, C / 4, scale, shift, relu);
  } else {
    const int64_t nvec = rows * C / 8;
    bn_apply_kernel<__nv_bfloat16><<<stream_grid(nvec), NT, 0, st>>>(
        (const __nv_bfloat16*)z, (const __nv_bfloat16*)residual, (__nv_bfloat16*)y, nvec, C / 8,
        scale, shift, relu);
  }
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}

template <typename T>
static int bn_backward_t(const void* dy, const void* y, const void* z, int64_t rows, int C,
                         const float* gamma, const float* mean, const float* invstd, int relu,
                         void* dz, void* dres, float* dgamma, float* dbeta, void* scratch,
                         cudaStream_t st) {
  constexpr int V = Vec16<T>::N;
  RowMap m = make_row_map(rows, C, V);
  double* partial = (double*)scratch;
  float* coef = (float*)((char*)scratch + (size_t)m.S * C * 2 * sizeof(double));
  bn_bwd_partial<T><<<dim3(m.S, m.GY), NT, 0, st>>>((const T*)dy, (const T*)y, (const T*)z, rows, C,
                                                    m, mean, invstd, relu, partial);
  SRT_LAUNCH_CHECK();
  bn_bwd_finalize<<<ceil_div(C, 128), 128, 0, st>>>(partial, m.S, C, rows, gamma, invstd, dgamma,
                                                   dbeta, coef);
  SRT_LAUNCH_CHECK();
  const int64_t nvec = rows * C / V;
  bn_bwd_apply<T><<<stream_grid(nvec), NT, 0, st>>>((const T*)dy, (const T*)y, (const T*)z, (T*)dz,
                                                    (T*)dres, nvec, C / V, mean, invstd, coef, relu);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}

int bn_backward(int dtype, const void* dy, const void* y, const void* z, int64_t rows, int C,
                const float* gamma, const float* mean, const float* invstd, int relu, void* dz,
                void* dres, float* dgamma, float* dbeta, void* scratch, size_t scratch_bytes,
                cudaStream_t st) {
  SRT_REQUIRE(C % 8 == 0 && rows > 0, "bn_backward: C (%d) must be a multiple of 8", C);
  SRT_REQUIRE(scratch && scratch_bytes >= bn_scratch_bytes(rows, C),
              "bn_backward: scratch too small");
  SRT_REQUIRE(!relu || y, "bn_backward: relu mask needs y");
  if (dtype == SRT_F32)
    return bn_backward_t<float>(dy, y, z, rows, C, gamma, mean, invstd, relu, dz, dres, dgamma,
                                dbeta, scratch, st);
  return bn_backward_t<__nv_bfloat16>(dy, y, z, rows, C, gamma, mean, invstd, relu, dz, dres,
                                      dgamma, dbeta, scratch, st);
}

}  // namespace srt
