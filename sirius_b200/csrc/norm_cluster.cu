// BatchNorm (training mode) as ONE kernel per direction, for activations small enough to stay on chip.
//
// The three-kernel path (statistics, finalize, apply) reads the activation twice from HBM and pays three
// launches; for the deep layers of a ResNet (6-25 MB per tensor, most of the network's BatchNorms) the launches
// dominate. Here a thread-block cluster of 8 CTAs owns a group of 16 or 32 channels: every CTA loads its eighth of
// the rows into shared memory once, the per-channel sums are combined across the cluster through distributed
// shared memory in rank order (deterministic), and the normalised result is written from shared memory. One read,
// one write, one launch. The backward kernel does the same with (masked gradient, input) resident.
//
// Launched with a cluster dimension of 8 (cudaLaunchKernelEx); the hardware co-schedules the CTAs of a cluster, the
// only inter-CTA waits are cluster barriers. When a tensor's slab does not fit in shared memory the caller uses the
// three-kernel path.
#include <cooperative_groups.h>
#include <stdlib.h>

#include "common.cuh"
#include "ops.cuh"

namespace cg = cooperative_groups;

namespace srt {

namespace {

constexpr int CL = 8;      // CTAs per cluster
constexpr int NTC = 256;   // threads per CTA
constexpr size_t SMEM_BUDGET = 200 * 1024;

struct FusedPlan {
  int CH;            // channels per cluster
  int rows_per_cta;
  size_t smem;
  bool ok;
};

// tiles: number of [rows_per_cta][CH] slabs kept in shared memory (1 forward, 2 backward)
inline FusedPlan make_plan(int64_t rows, int C, int esz, int tiles) {
  FusedPlan p;
  p.ok = false;
  const int V = 16 / esz;
  const int64_t rpc = (rows + CL - 1) / CL;
  for (int CH : {C <= 512 ? 16 : 32, 16}) {
    if (C % CH != 0 || CH % V != 0) continue;
    const size_t slab = (size_t)rpc * CH * esz * tiles;
    const size_t extra = (size_t)NTC * V * 2 * sizeof(float) + (size_t)CH * (2 * sizeof(double) + 4 * sizeof(float)) + 256;
    if (slab + extra <= SMEM_BUDGET && rpc < (1 << 30)) {
      p.CH = CH; p.rows_per_cta = (int)rpc; p.smem = slab + extra; p.ok = true;
      return p;
    }
  }
  return p;
}

template <typename T>
struct SmemView {
  T* tile0;
  T* tile1;
  float* red;      // [NTC][V][2]
  double* part;    // [CH][2]
  float* coef;     // [CH][4]
};
template <typename T>
__device__ inline SmemView<T> carve(unsigned char* raw, int rows_per_cta, int CH, int tiles) {
  constexpr int V = Vec16<T>::N;
  SmemView<T> s;
  s.tile0 = reinterpret_cast<T*>(raw);
  s.tile1 = s.tile0 + (size_t)rows_per_cta * CH;
  unsigned char* p = raw + (size_t)rows_per_cta * CH * sizeof(T) * tiles;
  p = (unsigned char*)(((uintptr_t)p + 15) & ~(uintptr_t)15);
  s.part = reinterpret_cast<double*>(p);
  p += (size_t)CH * 2 * sizeof(double);
  s.coef = reinterpret_cast<float*>(p);
  p += (size_t)CH * 4 * sizeof(float);
  s.red = reinterpret_cast<float*>(p);
  (void)V;
  return s;
}

// Sum the per-thread accumulators a[V], b[V] over the row lanes of the block; channel c of the chunk gets
// part[c*2 + {0,1}] in double. Threads are (tv = t % VPR, rl = t / VPR).
template <int V>
__device__ inline void block_sums(const float (&a)[V], const float (&b)[V], float* red, double* part, int VPR, int CH) {
  const int t = threadIdx.x;
#pragma unroll
  for (int v = 0; v < V; ++v) {
    red[(t * V + v) * 2] = a[v];
    red[(t * V + v) * 2 + 1] = b[v];
  }
  __syncthreads();
  if (t < CH) {
    const int tv = t / V, v = t % V, RL = NTC / VPR;
    double sa = 0.0, sb = 0.0;
    for (int rl = 0; rl < RL; ++rl) {
      const int src = rl * VPR + tv;
      sa += (double)red[(src * V + v) * 2];
      sb += (double)red[(src * V + v) * 2 + 1];
    }
    part[t * 2] = sa;
    part[t * 2 + 1] = sb;
  }
}

template <typename T, bool HAS_RES>
__global__ void __launch_bounds__(NTC)
bn_fwd_cluster_kernel(const T* __restrict__ z, const T* __restrict__ residual, T* __restrict__ y, int64_t rows, int C,
                      int CH, int rows_per_cta, const float* __restrict__ gamma, const float* __restrict__ beta, float eps,
                      float momentum, float* running_mean, float* running_var, float* mean, float* invstd, float* scale,
                      float* shift, int relu) {
  pdl_enter();
  constexpr int V = Vec16<T>::N;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank();
  const int c0 = (int)(blockIdx.x / CL) * CH;
  SmemView<T> sm = carve<T>(smem_raw, rows_per_cta, CH, 1);
  const int VPR = CH / V, RL = NTC / VPR;
  const int t = threadIdx.x, tv = t % VPR, rl = t / VPR;
  const int64_t r0 = (int64_t)rank * rows_per_cta;
  const int nrows = (int)(r0 + rows_per_cta <= rows ? rows_per_cta : (rows > r0 ? rows - r0 : 0));

  float s[V], q[V];
#pragma unroll
  for (int v = 0; v < V; ++v) { s[v] = 0.f; q[v] = 0.f; }
  for (int r = rl; r < nrows; r += 4 * RL) {
    Vec16<T> x[4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (r + u * RL < nrows) x[u].load(z + (r0 + r + u * RL) * C + c0 + tv * V);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (r + u * RL >= nrows) continue;
      x[u].store(sm.tile0 + (size_t)(r + u * RL) * CH + tv * V);
      float f[V];
      x[u].unpack(f);
#pragma unroll
      for (int v = 0; v < V; ++v) { s[v] += f[v]; q[v] = fmaf(f[v], f[v], q[v]); }
    }
  }
  block_sums<V>(s, q, sm.red, sm.part, VPR, CH);
  cluster.sync();
  if (t < CH) {
    double ts = 0.0, tq = 0.0;
    for (int k = 0; k < CL; ++k) {
      const double* rp = cluster.map_shared_rank(sm.part, k);
      ts += rp[t * 2];
      tq += rp[t * 2 + 1];
    }
    const int c = c0 + t;
    const double mu = ts / (double)rows;
    double var = tq / (double)rows - mu * mu;
    if (var < 0.0) var = 0.0;
    const float is = (float)(1.0 / sqrt(var + (double)eps));
    const float g = gamma ? gamma[c] : 1.f, b = beta ? beta[c] : 0.f;
    const float sc = g * is, sh = b - (float)mu * sc;
    sm.coef[t * 2] = sc;
    sm.coef[t * 2 + 1] = sh;
    if (rank == 0) {
      mean[c] = (float)mu;
      invstd[c] = is;
      scale[c] = sc;
      shift[c] = sh;
      if (running_mean) running_mean[c] = (1.f - momentum) * running_mean[c] + momentum * (float)mu;
      if (running_var) {
        const double unbiased = rows > 1 ? var * (double)rows / (double)(rows - 1) : var;
        running_var[c] = (1.f - momentum) * running_var[c] + momentum * (float)unbiased;
      }
    }
  }
  cluster.sync();  // nobody leaves (or reuses its partials) while a peer may still read them; also publishes coef
  float sc[V], sh[V];
#pragma unroll
  for (int v = 0; v < V; ++v) { sc[v] = sm.coef[(tv * V + v) * 2]; sh[v] = sm.coef[(tv * V + v) * 2 + 1]; }
  for (int r = rl; r < nrows; r += RL) {
    Vec16<T> x;
    x.load(sm.tile0 + (size_t)r * CH + tv * V);
    float f[V];
    x.unpack(f);
#pragma unroll
    for (int v = 0; v < V; ++v) f[v] = fmaf(f[v], sc[v], sh[v]);
    const int64_t o = (r0 + r) * C + c0 + tv * V;
    if (HAS_RES) {
      Vec16<T> rv;
      rv.load(residual + o);
      float rf[V];
      rv.unpack(rf);
#pragma unroll
      for (int v = 0; v < V; ++v) f[v] += rf[v];
    }
    if (relu) {
#pragma unroll
      for (int v = 0; v < V; ++v) f[v] = fmaxf(f[v], 0.f);
    }
    Vec16<T> out;
    out.pack(f);
    out.store(y + o);
  }
}

template <typename T>
__global__ void __launch_bounds__(NTC)
bn_bwd_cluster_kernel(const T* __restrict__ dy, const T* __restrict__ y, const T* __restrict__ z, T* __restrict__ dz,
                      T* __restrict__ dres, int64_t rows, int C, int CH, int rows_per_cta, const float* __restrict__ gamma,
                      const float* __restrict__ mean, const float* __restrict__ invstd, const float* __restrict__ scale,
                      const float* __restrict__ shift, int relu, float* dgamma, float* dbeta) {
  pdl_enter();
  constexpr int V = Vec16<T>::N;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank();
  const int c0 = (int)(blockIdx.x / CL) * CH;
  SmemView<T> sm = carve<T>(smem_raw, rows_per_cta, CH, 2);
  const int VPR = CH / V, RL = NTC / VPR;
  const int t = threadIdx.x, tv = t % VPR, rl = t / VPR;
  const int64_t r0 = (int64_t)rank * rows_per_cta;
  const int nrows = (int)(r0 + rows_per_cta <= rows ? rows_per_cta : (rows > r0 ? rows - r0 : 0));

  float mu[V], is[V], sc[V], sh[V];
#pragma unroll
  for (int v = 0; v < V; ++v) {
    const int c = c0 + tv * V + v;
    mu[v] = mean[c]; is[v] = invstd[c];
    sc[v] = scale ? scale[c] : 0.f; sh[v] = shift ? shift[c] : 0.f;
  }
  float sg[V], sgx[V];
#pragma unroll
  for (int v = 0; v < V; ++v) { sg[v] = 0.f; sgx[v] = 0.f; }
  for (int r = rl; r < nrows; r += 2 * RL) {
    Vec16<T> a[2], b[2], yv[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (r + u * RL >= nrows) continue;
      const int64_t o = (r0 + r + u * RL) * C + c0 + tv * V;
      a[u].load(dy + o);
      b[u].load(z + o);
      if (relu && y) yv[u].load(y + o);
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (r + u * RL >= nrows) continue;
      float g[V], x[V];
      a[u].unpack(g);
      b[u].unpack(x);
      if (relu) {
        if (y) {
          float yy[V];
          yv[u].unpack(yy);
#pragma unroll
          for (int v = 0; v < V; ++v) g[v] = yy[v] > 0.f ? g[v] : 0.f;
        } else {
#pragma unroll
          for (int v = 0; v < V; ++v) g[v] = fmaf(x[v], sc[v], sh[v]) > 0.f ? g[v] : 0.f;
        }
      }
      Vec16<T> gm;
      gm.pack(g);
      gm.store(sm.tile0 + (size_t)(r + u * RL) * CH + tv * V);
      b[u].store(sm.tile1 + (size_t)(r + u * RL) * CH + tv * V);
      if (dres) gm.store(dres + (r0 + r + u * RL) * C + c0 + tv * V);
      // the sums use the gradient as it is stored (rounded to the element type), like the three-kernel path
      float gr[V];
      gm.unpack(gr);
#pragma unroll
      for (int v = 0; v < V; ++v) {
        sg[v] += gr[v];
        sgx[v] = fmaf(gr[v], (x[v] - mu[v]) * is[v], sgx[v]);
      }
    }
  }
  block_sums<V>(sg, sgx, sm.red, sm.part, VPR, CH);
  cluster.sync();
  if (t < CH) {
    double tg = 0.0, tgx = 0.0;
    for (int k = 0; k < CL; ++k) {
      const double* rp = cluster.map_shared_rank(sm.part, k);
      tg += rp[t * 2];
      tgx += rp[t * 2 + 1];
    }
    const int c = c0 + t;
    const float g = gamma ? gamma[c] : 1.f;
    const float k0 = g * invstd[c];
    const float mg = (float)(tg / (double)rows), mgx = (float)(tgx / (double)rows);
    sm.coef[t * 4] = k0;
    sm.coef[t * 4 + 1] = -k0 * mgx * invstd[c];
    sm.coef[t * 4 + 2] = -k0 * mg;
    if (rank == 0) {
      if (dbeta) dbeta[c] = (float)tg;
      if (dgamma) dgamma[c] = (float)tgx;
    }
  }
  cluster.sync();
  float ka[V], kb[V], kd[V];
#pragma unroll
  for (int v = 0; v < V; ++v) {
    ka[v] = sm.coef[(tv * V + v) * 4];
    kb[v] = sm.coef[(tv * V + v) * 4 + 1];
    kd[v] = sm.coef[(tv * V + v) * 4 + 2];
  }
  for (int r = rl; r < nrows; r += RL) {
    Vec16<T> gv, xv;
    gv.load(sm.tile0 + (size_t)r * CH + tv * V);
    xv.load(sm.tile1 + (size_t)r * CH + tv * V);
    float g[V], x[V];
    gv.unpack(g);
    xv.unpack(x);
#pragma unroll
    for (int v = 0; v < V; ++v) g[v] = fmaf(ka[v], g[v], fmaf(kb[v], x[v] - mu[v], kd[v]));
    Vec16<T> out;
    out.pack(g);
    out.store(dz + (r0 + r) * C + c0 + tv * V);
  }
}

template <typename K, typename... Args>
int launch_cluster(K kernel, int clusters, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)clusters * CL);
  cfg.blockDim = dim3(NTC);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CL;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = (pdl_classes() & PDL_NORM) != 0 ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  SRT_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kernel, args...));
  count_launch();
  return SRT_OK;
}

template <typename K>
int ensure_smem(K kernel, size_t smem, bool* done, size_t* have) {
  if (!*done || smem > *have) {
    SRT_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BUDGET));
    *done = true;
    *have = SMEM_BUDGET;
  }
  return SRT_OK;
}

}  // namespace

bool bn_fused_fits(int dtype, int64_t rows, int C, int backward) {
  return make_plan(rows, C, dtype == SRT_F32 ? 4 : 2, backward ? 2 : 1).ok;
}

// Whether the step executor should take the one-kernel path. Measured on the ResNet-152 step (batch 64, B200) it does
// NOT pay: a channel group is 32-64 bytes of every row, so the loads are 32-byte pieces 512-4096 bytes apart instead
// of whole rows, and the step got slower for every channel threshold that covers the common layers (27.1-27.7 ms
// against 25.2 ms; neutral when only the 2048-channel layers use it). The executor therefore keeps the three-kernel
// path unless SIRIUS_B200_FUSED_BN_MINC names a minimum channel count; the operators stay available and tested.
bool bn_fused_pays(int dtype, int64_t rows, int C, int backward) {
  static const int min_c = [] { const char* e = getenv("SIRIUS_B200_FUSED_BN_MINC"); return e ? atoi(e) : (1 << 30); }();
  return C >= min_c && bn_fused_fits(dtype, rows, C, backward);
}

template <typename T>
static int bn_forward_fused_t(const void* z, const void* residual, void* y, int64_t rows, int C, const float* gamma,
                              const float* beta, float eps, float momentum, float* rm, float* rv, float* mean, float* invstd,
                              float* scale, float* shift, int relu, cudaStream_t st) {
  const FusedPlan p = make_plan(rows, C, (int)sizeof(T), 1);
  SRT_REQUIRE(p.ok, "bn_forward_fused: tensor does not fit on chip (rows %lld, C %d)", (long long)rows, C);
  static bool done[2] = {false, false};
  static size_t have[2] = {0, 0};
  int rc;
  if (residual) {
    if ((rc = ensure_smem(bn_fwd_cluster_kernel<T, true>, p.smem, &done[1], &have[1]))) return rc;
    return launch_cluster(bn_fwd_cluster_kernel<T, true>, C / p.CH, p.smem, st, (const T*)z, (const T*)residual, (T*)y, rows, C,
                          p.CH, p.rows_per_cta, gamma, beta, eps, momentum, rm, rv, mean, invstd, scale, shift, relu);
  }
  if ((rc = ensure_smem(bn_fwd_cluster_kernel<T, false>, p.smem, &done[0], &have[0]))) return rc;
  return launch_cluster(bn_fwd_cluster_kernel<T, false>, C / p.CH, p.smem, st, (const T*)z, (const T*)nullptr, (T*)y, rows, C,
                        p.CH, p.rows_per_cta, gamma, beta, eps, momentum, rm, rv, mean, invstd, scale, shift, relu);
}

int bn_forward_fused(int dtype, const void* z, const void* residual, void* y, int64_t rows, int C, const float* gamma,
                     const float* beta, float eps, float momentum, float* rm, float* rv, float* mean, float* invstd,
                     float* scale, float* shift, int relu, cudaStream_t st) {
  if (dtype == SRT_F32)
    return bn_forward_fused_t<float>(z, residual, y, rows, C, gamma, beta, eps, momentum, rm, rv, mean, invstd, scale, shift,
                                     relu, st);
  return bn_forward_fused_t<__nv_bfloat16>(z, residual, y, rows, C, gamma, beta, eps, momentum, rm, rv, mean, invstd, scale,
                                           shift, relu, st);
}

template <typename T>
static int bn_backward_fused_t(const void* dy, const void* y, const void* z, int64_t rows, int C, const float* gamma,
                               const float* mean, const float* invstd, const float* scale, const float* shift, int relu,
                               void* dz, void* dres, float* dgamma, float* dbeta, cudaStream_t st) {
  const FusedPlan p = make_plan(rows, C, (int)sizeof(T), 2);
  SRT_REQUIRE(p.ok, "bn_backward_fused: tensor does not fit on chip (rows %lld, C %d)", (long long)rows, C);
  static bool done = false;
  static size_t have = 0;
  int rc;
  if ((rc = ensure_smem(bn_bwd_cluster_kernel<T>, p.smem, &done, &have))) return rc;
  return launch_cluster(bn_bwd_cluster_kernel<T>, C / p.CH, p.smem, st, (const T*)dy, (const T*)y, (const T*)z, (T*)dz,
                        (T*)dres, rows, C, p.CH, p.rows_per_cta, gamma, mean, invstd, scale, shift, relu, dgamma, dbeta);
}

int bn_backward_fused(int dtype, const void* dy, const void* y, const void* z, int64_t rows, int C, const float* gamma,
                      const float* mean, const float* invstd, const float* scale, const float* shift, int relu, void* dz,
                      void* dres, float* dgamma, float* dbeta, cudaStream_t st) {
  SRT_REQUIRE(!relu || y || (scale && shift), "bn_backward_fused: the ReLU mask needs y or scale/shift");
  if (dtype == SRT_F32)
    return bn_backward_fused_t<float>(dy, y, z, rows, C, gamma, mean, invstd, scale, shift, relu, dz, dres, dgamma, dbeta, st);
  return bn_backward_fused_t<__nv_bfloat16>(dy, y, z, rows, C, gamma, mean, invstd, scale, shift, relu, dz, dres, dgamma,
                                            dbeta, st);
}

}  // namespace srt
