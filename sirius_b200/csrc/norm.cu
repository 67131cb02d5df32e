// BatchNorm (training mode) over NHWC rows: statistics, fused apply (+residual, +ReLU), backward.
//
// All kernels are HBM-bound streaming passes: 16-byte vector loads along the channel axis (the
// contiguous one), fp32 per-thread accumulation over a short run of rows, double-precision
// combination of the per-thread and per-slab partial sums in a fixed order (deterministic, and
// accurate enough for the fp32 parity mode).
#include <cstdlib>
#include <mutex>

#include "common.cuh"

namespace srt {

namespace {

constexpr int NT = 256;
constexpr int ROWS_PER_THREAD = 8;   // rows per thread and batch
constexpr int BWD_ROWS = 4;          // rows in flight per thread in the backward sums (two or three tensors per row)
constexpr int FIN_CH = 8;            // channels per finalize block (8 x 16 B = one 128-byte line)
constexpr int FIN_LANES = 32;        // slab lanes per channel in the finalize kernels
constexpr int RESIDENT_BLOCKS = 3 * 148;  // blocks of the partial-sum kernels the device holds at once (80 registers)
constexpr int MAX_ITERS = 16;

// How a partial-sum kernel covers the rows x C matrix. A block owns `slab` consecutive rows of one
// chunk of TC channel vectors and writes one partial per channel, so the partial-sum traffic is
// 16 bytes per channel per slab: tall slabs keep it small against the rows*C input (a 16-row slab of
// a 1024-channel bf16 tensor would write half as many bytes as it reads). Narrow channel chunks
// (down to one 128-byte line per row) buy the height without starving the device of blocks.
struct RowMap {
  int CV;     // 16-byte vectors per row
  int TC;     // threads across channel vectors in a block
  int RL;     // row lanes in a block
  int iters;  // batches of ROWS_PER_THREAD rows per thread
  int slab;   // rows per block = RL * ROWS_PER_THREAD * iters
  int S;      // number of slabs (grid.x)
  int GY;     // channel chunks (grid.y)
};

inline RowMap row_map_for(int64_t rows, int CV, int TC, int iters) {
  RowMap m;
  m.CV = CV;
  m.TC = TC;
  m.RL = NT / TC;
  m.iters = iters;
  m.slab = m.RL * ROWS_PER_THREAD * iters;
  m.S = (int)((rows + m.slab - 1) / m.slab);
  m.GY = (CV + TC - 1) / TC;
  return m;
}

// One wave of long-lived blocks: the shape with the most blocks among those the device holds at once (a block
// that loops over several batches of rows keeps loads in flight while earlier ones are summed, and no second,
// partly filled wave follows); a tensor too large for that gets the fewest blocks possible. Ties go to the
// taller slab (fewer partial sums).
inline RowMap make_row_map(int64_t rows, int C, int V) {
  const int CV = C / V;
  const int widest = CV < NT ? CV : NT;
  constexpr int min_tc = 8;  // one 128-byte line per row and block
  RowMap best = row_map_for(rows, CV, widest, 1);
  // fp32 is the parity mode: whole rows per block and eight rows per thread keep the fp32 part of every sum short
  // (three SGD steps at lr 0.1 amplify rounding differences of the statistics into percent of the loss)
  if (V == 4) return best;
  auto blocks = [](const RowMap& m) { return (int64_t)m.S * m.GY; };
  auto better = [&](const RowMap& a, const RowMap& b) {  // is a better than b
    const bool fa = blocks(a) <= RESIDENT_BLOCKS, fb = blocks(b) <= RESIDENT_BLOCKS;
    if (fa != fb) return fa;
    if (blocks(a) != blocks(b)) return fa ? blocks(a) > blocks(b) : blocks(a) < blocks(b);
    return a.slab != b.slab ? a.slab > b.slab : a.TC > b.TC;
  };
  for (int tc = widest; tc >= 1; tc = (tc > min_tc ? (tc % 2 == 0 ? tc / 2 : min_tc) : 0)) {
    for (int iters = 1; iters <= MAX_ITERS; iters *= 2) {
      const RowMap m = row_map_for(rows, CV, tc, iters);
      if (better(m, best)) best = m;
    }
    if (tc <= min_tc) break;
  }
  return best;
}

// Reduce per-thread accumulators a[V], b[V] over the block's row lanes; lane 0 of each channel
// vector writes the slab partial as doubles: partial[(slab*C + c)*2 + {0,1}].
template <int V>
__device__ inline void block_reduce_store(const float (&a)[V], const float (&b)[V], const RowMap& m,
                                          int C, double* partial) {
  __shared__ float sh_a[NT * V];
  __shared__ float sh_b[NT * V];
  const int t = threadIdx.x;
#pragma unroll
  for (int v = 0; v < V; ++v) { sh_a[t * V + v] = a[v]; sh_b[t * V + v] = b[v]; }
  __syncthreads();
  // Row lanes are summed in a fixed order. A narrow chunk leaves most threads without a channel of
  // their own, so the lanes of a channel are dealt to NT/chunk threads first and those sums combined.
  const int chunk = m.TC * V;
  const int nparts = chunk < NT ? NT / chunk : 1;
  if (nparts == 1) {
    for (int ch = t; ch < chunk; ch += NT) {
      const int c = blockIdx.y * chunk + ch;
      if (c >= C) break;
      double sa = 0.0, sb = 0.0;
      for (int r = 0; r < m.RL; ++r) {
        sa += (double)sh_a[r * chunk + ch];
        sb += (double)sh_b[r * chunk + ch];
      }
      double2* out = reinterpret_cast<double2*>(partial) + (size_t)blockIdx.x * C + c;
      *out = make_double2(sa, sb);
    }
    return;
  }
  __shared__ double2 sh_d[NT];
  const int ch = t % chunk, part = t / chunk;
  if (part < nparts) {
    double sa = 0.0, sb = 0.0;
    for (int r = part; r < m.RL; r += nparts) {
      sa += (double)sh_a[r * chunk + ch];
      sb += (double)sh_b[r * chunk + ch];
    }
    sh_d[part * chunk + ch] = make_double2(sa, sb);
  }
  __syncthreads();
  const int c = blockIdx.y * chunk + ch;
  if (part == 0 && c < C) {
    double2 tot = sh_d[ch];
    for (int q = 1; q < nparts; ++q) {
      tot.x += sh_d[q * chunk + ch].x;
      tot.y += sh_d[q * chunk + ch].y;
    }
    reinterpret_cast<double2*>(partial)[(size_t)blockIdx.x * C + c] = tot;
  }
}

// Sum of the S slab partials of channel c: FIN_LANES lanes stride over the slabs, then a fixed-shape
// tree through shared memory (deterministic). Call with blockDim = (FIN_CH channels, LANES). The partial sums a
// convolution epilogue leaves come one row per 128-row tile (up to 1568 rows for the layer1 tensors): those get
// FIN_LANES_TALL lanes, so that a lane still has only a dozen loads in a row.
constexpr int FIN_LANES_TALL = 128;
template <int LANES = FIN_LANES>
__device__ inline double2 reduce_partials(const double* __restrict__ partial, int S, int C, int c) {
  __shared__ double2 sh[LANES][FIN_CH];
  double2 acc = make_double2(0.0, 0.0);
  if (c < C) {
    const double2* p = reinterpret_cast<const double2*>(partial);
#pragma unroll 4
    for (int i = threadIdx.y; i < S; i += LANES) {
      const double2 v = p[(size_t)i * C + c];
      acc.x += v.x;
      acc.y += v.y;
    }
  }
  sh[threadIdx.y][threadIdx.x] = acc;
  __syncthreads();
#pragma unroll
  for (int o = LANES / 2; o > 0; o >>= 1) {
    if ((int)threadIdx.y < o) {
      double2 a = sh[threadIdx.y][threadIdx.x];
      const double2 b = sh[threadIdx.y + o][threadIdx.x];
      a.x += b.x;
      a.y += b.y;
      sh[threadIdx.y][threadIdx.x] = a;
    }
    __syncthreads();
  }
  return sh[0][threadIdx.x];
}

template <typename T>
__global__ void __launch_bounds__(NT)
bn_stats_partial(const T* __restrict__ z, int64_t rows, int C, RowMap m, double* partial) {
  pdl_enter();
  constexpr int V = Vec16<T>::N;
  const int t = threadIdx.x;
  const int tc = t % m.TC, rl = t / m.TC;
  const int cv = blockIdx.y * m.TC + tc;
  float s[V], q[V];
#pragma unroll
  for (int v = 0; v < V; ++v) { s[v] = 0.f; q[v] = 0.f; }
  if (rl < m.RL && cv < m.CV) {
    for (int it = 0; it < m.iters; ++it) {
      const int64_t batch0 = (int64_t)blockIdx.x * m.slab + (int64_t)it * ROWS_PER_THREAD * m.RL;
      if (batch0 >= rows) break;  // the last slab may be short
      const int64_t r0 = batch0 + rl;
      Vec16<T> x[ROWS_PER_THREAD];
#pragma unroll
      for (int i = 0; i < ROWS_PER_THREAD; ++i) {
        const int64_t r = r0 + (int64_t)i * m.RL;
        if (r < rows) x[i].load(z + r * C + (int64_t)cv * V);
      }
#pragma unroll
      for (int i = 0; i < ROWS_PER_THREAD; ++i) {
        const int64_t r = r0 + (int64_t)i * m.RL;
        if (r < rows) {
          float f[V];
          x[i].unpack(f);
#pragma unroll
          for (int v = 0; v < V; ++v) { s[v] += f[v]; q[v] = fmaf(f[v], f[v], q[v]); }
        }
      }
    }
  }
  block_reduce_store<V>(s, q, m, C, partial);
}

template <int LANES>
__global__ void __launch_bounds__(FIN_CH * LANES)
bn_stats_finalize(const double* __restrict__ partial, int S, int C, int64_t rows,
                  const float* __restrict__ gamma, const float* __restrict__ beta, float eps,
                  float momentum, float* running_mean, float* running_var, float* mean, float* invstd,
                  float* scale, float* shift) {
  pdl_enter();
  const int c = blockIdx.x * FIN_CH + threadIdx.x;
  // the channel's parameters are fetched before the reduction, so their latency hides behind its loads
  float g = 1.f, b = 0.f, rm0 = 0.f, rv0 = 0.f;
  if (threadIdx.y == 0 && c < C) {
    if (gamma) g = gamma[c];
    if (beta) b = beta[c];
    if (running_mean) rm0 = running_mean[c];
    if (running_var) rv0 = running_var[c];
  }
  const double2 tot = reduce_partials<LANES>(partial, S, C, c);
  if (threadIdx.y != 0 || c >= C) return;
  const double mu = tot.x / (double)rows;
  double var = tot.y / (double)rows - mu * mu;
  if (var < 0.0) var = 0.0;
  const float is = (float)(1.0 / sqrt(var + (double)eps));
  mean[c] = (float)mu;
  invstd[c] = is;
  const float sc = g * is;
  scale[c] = sc;
  shift[c] = b - (float)mu * sc;
  if (running_mean) running_mean[c] = (1.f - momentum) * rm0 + momentum * (float)mu;
  if (running_var) {
    const double unbiased = rows > 1 ? var * (double)rows / (double)(rows - 1) : var;
    running_var[c] = (1.f - momentum) * rv0 + momentum * (float)unbiased;
  }
}

constexpr int UNR = 4;  // independent 16-byte vectors per thread in the elementwise kernels

// relu_bits (optional, 8-element vectors only): byte i receives the ReLU mask of vector i of y, bit e set when
// element e came out positive. The backward pass of a residual unit reads those bits instead of the stored y.
template <typename T, bool HAS_RES>
__global__ void __launch_bounds__(NT)
bn_apply_kernel(const T* __restrict__ z, const T* __restrict__ residual, T* __restrict__ y, int64_t nvec,
                int CV, const float* __restrict__ scale, const float* __restrict__ shift, int relu,
                uint8_t* __restrict__ relu_bits) {
  pdl_enter();
  constexpr int V = Vec16<T>::N;
  const int64_t base = (int64_t)blockIdx.x * (NT * UNR) + threadIdx.x;
  Vec16<T> x[UNR], rv[UNR];
#pragma unroll
  for (int u = 0; u < UNR; ++u) {
    const int64_t i = base + (int64_t)u * NT;
    if (i < nvec) {
      x[u].load(z + i * V);
      if (HAS_RES) rv[u].load(residual + i * V);
    }
  }
#pragma unroll
  for (int u = 0; u < UNR; ++u) {
    const int64_t i = base + (int64_t)u * NT;
    if (i >= nvec) continue;
    const int cv = (int)(i % CV);
    float f[V];
    x[u].unpack(f);
#pragma unroll
    for (int v = 0; v < V; v += 4) {
      const float4 a = *reinterpret_cast<const float4*>(scale + cv * V + v);
      const float4 b = *reinterpret_cast<const float4*>(shift + cv * V + v);
      f[v] = fmaf(f[v], a.x, b.x); f[v + 1] = fmaf(f[v + 1], a.y, b.y);
      f[v + 2] = fmaf(f[v + 2], a.z, b.z); f[v + 3] = fmaf(f[v + 3], a.w, b.w);
    }
    if (HAS_RES) {
      float rf[V];
      rv[u].unpack(rf);
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
    if (V == 8 && relu_bits) {
      // the mask of the value as stored (after rounding): what a reader of y would see
      float r[V];
      o.unpack(r);
      unsigned bits = 0u;
#pragma unroll
      for (int v = 0; v < V; ++v) bits |= (r[v] > 0.f ? 1u : 0u) << v;
      relu_bits[i] = (uint8_t)bits;
    }
  }
}

// ReLU mask of y = relu(z*scale + shift): taken from the stored y when given (residual units),
// otherwise recomputed from z with the same fused multiply-add the forward pass used, which has
// the same sign as the stored (rounded) y.
template <typename T, int V>
__device__ __forceinline__ void apply_relu_mask(float (&g)[V], const float (&x)[V], const Vec16<T>* y_vec,
                                                const float* __restrict__ scale,
                                                const float* __restrict__ shift, int c0) {
  if (y_vec) {
    const Vec16<T>& yv = *y_vec;
    float yy[V];
    yv.unpack(yy);
#pragma unroll
    for (int v = 0; v < V; ++v) g[v] = yy[v] > 0.f ? g[v] : 0.f;
  } else {
#pragma unroll
    for (int v = 0; v < V; v += 4) {
      const float4 a = *reinterpret_cast<const float4*>(scale + c0 + v);
      const float4 b = *reinterpret_cast<const float4*>(shift + c0 + v);
      g[v] = fmaf(x[v], a.x, b.x) > 0.f ? g[v] : 0.f;
      g[v + 1] = fmaf(x[v + 1], a.y, b.y) > 0.f ? g[v + 1] : 0.f;
      g[v + 2] = fmaf(x[v + 2], a.z, b.z) > 0.f ? g[v + 2] : 0.f;
      g[v + 3] = fmaf(x[v + 3], a.w, b.w) > 0.f ? g[v + 3] : 0.f;
    }
  }
}

template <int V>
__device__ __forceinline__ void apply_relu_bits(float (&g)[V], unsigned bits) {
#pragma unroll
  for (int v = 0; v < V; ++v) g[v] = ((bits >> v) & 1u) ? g[v] : 0.f;
}

// MASK: 0 no ReLU, 1 mask from the stored output y, 2 mask recomputed from z, 3 mask from one bit per element
// (the y pointer then holds the bytes bn_apply_kernel wrote; 8-element vectors only). A compile-time choice, so
// the per-channel vectors and loads of the unused variants take no registers.
template <typename T, int MASK>
__global__ void __launch_bounds__(NT, 3)
bn_bwd_partial(const T* __restrict__ dy, const T* __restrict__ y, const T* __restrict__ z,
               int64_t rows, int C, RowMap m, const float* __restrict__ mean,
               const float* __restrict__ invstd, const float* __restrict__ scale,
               const float* __restrict__ shift, int relu, double* partial) {
  pdl_enter();
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
    for (int it = 0; it < m.iters * (ROWS_PER_THREAD / BWD_ROWS); ++it) {
      const int64_t batch0 = (int64_t)blockIdx.x * m.slab + (int64_t)it * BWD_ROWS * m.RL;
      if (batch0 >= rows) break;  // the last slab may be short
      const int64_t r0 = batch0 + rl;
      Vec16<T> a[BWD_ROWS], b[BWD_ROWS], yv[BWD_ROWS];  // the stored output travels with the other two loads
      unsigned mb[BWD_ROWS];
#pragma unroll
      for (int i = 0; i < BWD_ROWS; ++i) {
        const int64_t r = r0 + (int64_t)i * m.RL;
        if (r < rows) {
          const int64_t o = r * C + (int64_t)cv * V;
          a[i].load(dy + o);
          b[i].load(z + o);
          if (MASK == 1) yv[i].load(y + o);
          if (MASK == 3) mb[i] = reinterpret_cast<const uint8_t*>(y)[o / V];
        }
      }
#pragma unroll
      for (int i = 0; i < BWD_ROWS; ++i) {
        const int64_t r = r0 + (int64_t)i * m.RL;
        if (r >= rows) continue;
        float g[V], x[V];
        a[i].unpack(g);
        b[i].unpack(x);
        if (MASK == 3) apply_relu_bits<V>(g, mb[i]);
        else if (MASK != 0) apply_relu_mask<T, V>(g, x, MASK == 1 ? &yv[i] : nullptr, scale, shift, cv * V);
#pragma unroll
        for (int v = 0; v < V; ++v) {
          sg[v] += g[v];
          sgx[v] = fmaf(g[v], (x[v] - mu[v]) * is[v], sgx[v]);
        }
      }
    }
  }
  block_reduce_store<V>(sg, sgx, m, C, partial);
}

__global__ void __launch_bounds__(FIN_CH * FIN_LANES)
bn_bwd_finalize(const double* __restrict__ partial, int S, int C, int64_t rows,
                const float* __restrict__ gamma, const float* __restrict__ invstd, float* dgamma,
                float* dbeta, float* coef) {
  pdl_enter();
  const int c = blockIdx.x * FIN_CH + threadIdx.x;
  float g = 1.f, is = 0.f;  // fetched before the reduction, so their latency hides behind its loads
  if (threadIdx.y == 0 && c < C) {
    if (gamma) g = gamma[c];
    is = invstd[c];
  }
  const double2 tot = reduce_partials(partial, S, C, c);
  if (threadIdx.y != 0 || c >= C) return;
  if (dbeta) dbeta[c] = (float)tot.x;
  if (dgamma) dgamma[c] = (float)tot.y;
  // dz = k0*(g - mean_g - xhat*mean_gx), xhat = (x - mean)*invstd, stored as three per-channel
  // vectors so the elementwise pass reads them with 16-byte loads: dz = ka*g + kb*(x - mean) + kd
  const float k0 = g * is;
  const float mg = (float)(tot.x / (double)rows), mgx = (float)(tot.y / (double)rows);
  coef[c] = k0;
  coef[C + c] = -k0 * mgx * is;
  coef[2 * C + c] = -k0 * mg;
}

template <typename T, int MASK>
__global__ void __launch_bounds__(NT, 4)
bn_bwd_apply(const T* __restrict__ dy, const T* __restrict__ y, const T* __restrict__ z, T* __restrict__ dz,
             T* __restrict__ dres, int64_t nvec, int CV, int C, const float* __restrict__ mean,
             const float* __restrict__ coef,
             const float* __restrict__ scale, const float* __restrict__ shift, int relu) {
  pdl_enter();
  constexpr int V = Vec16<T>::N;
  const int64_t base = (int64_t)blockIdx.x * (NT * UNR) + threadIdx.x;
  Vec16<T> a[UNR], b[UNR], yv[UNR];
  unsigned mb[UNR];
#pragma unroll
  for (int u = 0; u < UNR; ++u) {
    const int64_t i = base + (int64_t)u * NT;
    if (i < nvec) {
      a[u].load(dy + i * V);
      b[u].load(z + i * V);
      if (MASK == 1) yv[u].load(y + i * V);
      if (MASK == 3) mb[u] = reinterpret_cast<const uint8_t*>(y)[i];
    }
  }
#pragma unroll
  for (int u = 0; u < UNR; ++u) {
    const int64_t i = base + (int64_t)u * NT;
    if (i >= nvec) continue;
    const int cv = (int)(i % CV);
    float g[V], x[V];
    a[u].unpack(g);
    b[u].unpack(x);
    if (MASK == 3) apply_relu_bits<V>(g, mb[u]);
    else if (MASK != 0) apply_relu_mask<T, V>(g, x, MASK == 1 ? &yv[u] : nullptr, scale, shift, cv * V);
    if (dres) {
      Vec16<T> o;
      o.pack(g);
      o.store(dres + i * V);
    }
    float out[V];
#pragma unroll
    for (int v = 0; v < V; v += 4) {
      const int c = cv * V + v;
      const float4 ka = *reinterpret_cast<const float4*>(coef + c);
      const float4 kb = *reinterpret_cast<const float4*>(coef + C + c);
      const float4 kd = *reinterpret_cast<const float4*>(coef + 2 * C + c);
      const float4 mu = *reinterpret_cast<const float4*>(mean + c);
      out[v] = fmaf(ka.x, g[v], fmaf(kb.x, x[v] - mu.x, kd.x));
      out[v + 1] = fmaf(ka.y, g[v + 1], fmaf(kb.y, x[v + 1] - mu.y, kd.y));
      out[v + 2] = fmaf(ka.z, g[v + 2], fmaf(kb.z, x[v + 2] - mu.z, kd.z));
      out[v + 3] = fmaf(ka.w, g[v + 3], fmaf(kb.w, x[v + 3] - mu.w, kd.w));
    }
    Vec16<T> o;
    o.pack(out);
    o.store(dz + i * V);
  }
}

inline unsigned unrolled_grid(int64_t nvec) {
  const int64_t per_block = (int64_t)NT * UNR;
  const int64_t blocks = (nvec + per_block - 1) / per_block;
  return (unsigned)(blocks < 1 ? 1 : blocks);
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
  launch_pdl_if((pdl_classes() & PDL_NORM) != 0, bn_stats_partial<T>, dim3(m.S, m.GY), dim3(NT), 0, st, (const T*)z, rows, C, m, partial);
  SRT_LAUNCH_CHECK();
  launch_pdl_if((pdl_classes() & PDL_NORM) != 0, bn_stats_finalize<FIN_LANES>, dim3(ceil_div(C, FIN_CH)), dim3(FIN_CH, FIN_LANES), 0, st,
      partial, m.S, C, rows, gamma, beta, eps, momentum, rm, rv, mean, invstd, scale, shift);
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

int bn_finalize(const void* partial, int slabs, int C, int64_t rows, const float* gamma, const float* beta, float eps,
                float momentum, float* rm, float* rv, float* mean, float* invstd, float* scale, float* shift,
                cudaStream_t st) {
  SRT_REQUIRE(partial && slabs > 0 && C > 0 && rows > 0, "bn_finalize: empty input");
  SRT_REQUIRE(((uintptr_t)partial & 15) == 0, "bn_finalize: partial sums must be 16-byte aligned");
  const bool early = (pdl_classes() & PDL_NORM) != 0;
  if (slabs > 8 * FIN_LANES)
    launch_pdl_if(early, bn_stats_finalize<FIN_LANES_TALL>, dim3(ceil_div(C, FIN_CH)), dim3(FIN_CH, FIN_LANES_TALL), 0, st,
        (const double*)partial, slabs, C, rows, gamma, beta, eps, momentum, rm, rv, mean, invstd, scale, shift);
  else
    launch_pdl_if(early, bn_stats_finalize<FIN_LANES>, dim3(ceil_div(C, FIN_CH)), dim3(FIN_CH, FIN_LANES), 0, st,
        (const double*)partial, slabs, C, rows, gamma, beta, eps, momentum, rm, rv, mean, invstd, scale, shift);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}

template <typename T>
static void bn_apply_t(const void* z, const void* residual, void* y, int64_t rows, int C,
                       const float* scale, const float* shift, int relu, uint8_t* relu_bits, cudaStream_t st) {
  constexpr int V = Vec16<T>::N;
  const int64_t nvec = rows * C / V;
  if (residual)
    launch_pdl_if((pdl_classes() & PDL_NORM) != 0, bn_apply_kernel<T, true>, dim3(unrolled_grid(nvec)), dim3(NT), 0, st, (const T*)z,
               (const T*)residual, (T*)y, nvec, C / V, scale, shift, relu, relu_bits);
  else
    launch_pdl_if((pdl_classes() & PDL_NORM) != 0, bn_apply_kernel<T, false>, dim3(unrolled_grid(nvec)), dim3(NT), 0, st, (const T*)z,
               (const T*)nullptr, (T*)y, nvec, C / V, scale, shift, relu, relu_bits);
}

// ---- allocation-free variant of bn_stats ----------------------------------------------------
// The slab partial sums normally live in caller-provided scratch. Some callers cannot provide any:
// a colocated trainer that is in the middle of handing its memory pool to the inference server has
// promised every free byte of the device to the other process, so a cudaMalloc at that moment
// either fails or takes memory the server was just told it may use; and a control thread that has
// to stay responsive cannot afford cudaMalloc/cudaFree, which may synchronise the whole device.
// For them the partials go into this fixed array, which is part of the library image: every GPU
// that loads the library holds these 4 MiB until the process exits.
static __device__ __align__(256) unsigned char g_bn_static_scratch[SRT_BN_STATIC_SCRATCH_BYTES];

// In host code `g_bn_static_scratch` is only a handle for the runtime, not a device address; the
// address a kernel can use is looked up once per device (with that device current) and cached.
static std::mutex g_static_mu;
static void* g_static_ptr[64] = {nullptr};

// Looks the array's device address up for the current device (again, if asked to: a cudaDeviceReset
// invalidates an address looked up before it). The first look-up on a device may be the moment the CUDA
// runtime loads this file's module and backs the array (lazy module loading), so a caller who must not touch
// the allocator later does it here, at start-up.
int bn_static_prepare(bool refresh, void** out) {
  int dev = -1;
  SRT_CHECK_CUDA(cudaGetDevice(&dev));
  SRT_REQUIRE(dev >= 0 && dev < 64, "bn_stats_static: unsupported device ordinal %d", dev);
  std::lock_guard<std::mutex> lk(g_static_mu);
  if (refresh || g_static_ptr[dev] == nullptr) {
    void* p = nullptr;
    SRT_CHECK_CUDA(cudaGetSymbolAddress(&p, g_bn_static_scratch));
    g_static_ptr[dev] = p;
  }
  if (out) *out = g_static_ptr[dev];
  return SRT_OK;
}

int bn_stats_static(int dtype, const void* z, int64_t rows, int C, const float* gamma,
                    const float* beta, float eps, float momentum, float* rm, float* rv, float* mean,
                    float* invstd, float* scale, float* shift, cudaStream_t st) {
  SRT_REQUIRE(C % 8 == 0 && rows > 0, "bn_stats_static: C (%d) must be a multiple of 8, rows > 0", C);
  const size_t need = bn_scratch_bytes(rows, C);
  SRT_REQUIRE(need <= (size_t)SRT_BN_STATIC_SCRATCH_BYTES,
              "bn_stats_static: rows=%lld, C=%d needs %zu bytes of partial sums, the built-in scratch "
              "holds %zu; use srt_bn_stats with caller-provided scratch",
              (long long)rows, C, need, (size_t)SRT_BN_STATIC_SCRATCH_BYTES);
  void* ptr = nullptr;
  if (int rc = bn_static_prepare(false, &ptr)) return rc;
  // Nothing in the array has to start at zero: every slab partial that the finalize kernel reads
  // is written by the partial kernel of the same call first.
  return bn_stats(dtype, z, rows, C, gamma, beta, eps, momentum, rm, rv, mean, invstd, scale, shift,
                  ptr, (size_t)SRT_BN_STATIC_SCRATCH_BYTES, st);
}

__global__ void bn_eval_params_kernel(const float* __restrict__ gamma, const float* __restrict__ beta,
                                      const float* __restrict__ rmean, const float* __restrict__ rvar,
                                      float eps, int C, float* scale, float* shift) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const float sc = (gamma ? gamma[c] : 1.f) * rsqrtf(rvar[c] + eps);
  scale[c] = sc;
  shift[c] = (beta ? beta[c] : 0.f) - rmean[c] * sc;
}

// scale/shift of inference-mode BatchNorm: y = (z - running_mean) / sqrt(running_var + eps) * g + b.
int bn_eval_params(const float* gamma, const float* beta, const float* rmean, const float* rvar, float eps, int C,
                   float* scale, float* shift, cudaStream_t st) {
  bn_eval_params_kernel<<<ceil_div(C, 128), 128, 0, st>>>(gamma, beta, rmean, rvar, eps, C, scale, shift);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}

int bn_apply(int dtype, const void* z, const void* residual, void* y, int64_t rows, int C,
             const float* scale, const float* shift, int relu, cudaStream_t st, uint8_t* relu_bits) {
  SRT_REQUIRE(C % 8 == 0, "bn_apply: C (%d) must be a multiple of 8", C);
  SRT_REQUIRE(!relu_bits || (dtype == SRT_BF16 && relu), "bn_apply: the ReLU bit mask is written for bf16 tensors under a ReLU");
  if (dtype == SRT_F32) bn_apply_t<float>(z, residual, y, rows, C, scale, shift, relu, nullptr, st);
  else bn_apply_t<__nv_bfloat16>(z, residual, y, rows, C, scale, shift, relu, relu_bits, st);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}

template <typename T>
static int bn_backward_t(const void* dy, const void* y, const void* z, int64_t rows, int C,
                         const float* gamma, const float* mean, const float* invstd,
                         const float* scale, const float* shift, int relu, void* dz, void* dres,
                         float* dgamma, float* dbeta, void* scratch, cudaStream_t st, const uint8_t* relu_bits) {
  constexpr int V = Vec16<T>::N;
  RowMap m = make_row_map(rows, C, V);
  double* partial = (double*)scratch;
  float* coef = (float*)((char*)scratch + (size_t)m.S * C * 2 * sizeof(double));
  const int mask = !relu ? 0 : relu_bits ? 3 : (y ? 1 : 2);
  if (mask == 3) y = relu_bits;  // the kernels find the bytes where the stored output would be
  const bool early = (pdl_classes() & PDL_NORM) != 0;
  auto partial_k = mask == 0 ? bn_bwd_partial<T, 0> : mask == 1 ? bn_bwd_partial<T, 1> : mask == 2 ? bn_bwd_partial<T, 2>
                                                                                               : bn_bwd_partial<T, 3>;
  launch_pdl_if(early, partial_k, dim3(m.S, m.GY), dim3(NT), 0, st, (const T*)dy, (const T*)y, (const T*)z, rows, C, m, mean,
                invstd, scale, shift, relu, partial);
  SRT_LAUNCH_CHECK();
  launch_pdl_if(early, bn_bwd_finalize, dim3(ceil_div(C, FIN_CH)), dim3(FIN_CH, FIN_LANES), 0, st, partial, m.S, C, rows,
                gamma, invstd, dgamma, dbeta, coef);
  SRT_LAUNCH_CHECK();
  const int64_t nvec = rows * C / V;
  auto apply_k = mask == 0 ? bn_bwd_apply<T, 0> : mask == 1 ? bn_bwd_apply<T, 1> : mask == 2 ? bn_bwd_apply<T, 2> : bn_bwd_apply<T, 3>;
  launch_pdl_if(early, apply_k, dim3(unrolled_grid(nvec)), dim3(NT), 0, st, (const T*)dy, (const T*)y, (const T*)z, (T*)dz,
                (T*)dres, nvec, C / V, C, mean, (const float*)coef, scale, shift, relu);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}

int bn_backward(int dtype, const void* dy, const void* y, const void* z, int64_t rows, int C,
                const float* gamma, const float* mean, const float* invstd, const float* scale,
                const float* shift, int relu, void* dz, void* dres, float* dgamma, float* dbeta,
                void* scratch, size_t scratch_bytes, cudaStream_t st, const uint8_t* relu_bits) {
  SRT_REQUIRE(C % 8 == 0 && rows > 0, "bn_backward: C (%d) must be a multiple of 8", C);
  SRT_REQUIRE(scratch && scratch_bytes >= bn_scratch_bytes(rows, C),
              "bn_backward: scratch too small");
  SRT_REQUIRE(!relu || y || relu_bits || (scale && shift), "bn_backward: the ReLU mask needs y, its bits or scale/shift");
  SRT_REQUIRE(!relu_bits || (dtype == SRT_BF16 && relu), "bn_backward: the ReLU bit mask goes with bf16 tensors under a ReLU");
  if (dtype == SRT_F32)
    return bn_backward_t<float>(dy, y, z, rows, C, gamma, mean, invstd, scale, shift, relu, dz, dres,
                                dgamma, dbeta, scratch, st, nullptr);
  return bn_backward_t<__nv_bfloat16>(dy, y, z, rows, C, gamma, mean, invstd, scale, shift, relu, dz,
                                      dres, dgamma, dbeta, scratch, st, relu_bits);
}

}  // namespace srt
