// BatchNorm (training mode) as ONE launch per direction.
//
// The three-kernel path (partial sums, finalize, apply) pays three launches and their ramps; for the deep
// layers of a ResNet (6-25 MB per tensor, most of the network's BatchNorms) those dominate: the tensors sit
// in L2 and each pass has a few microseconds of work. Here one grid of at most one block per SM does all
// three phases, separated by two grid-wide barriers:
//
//   phase 1  every block sums its work items (a slab of rows x a chunk of channels) into a partial per channel
//   barrier
//   finalize the channels are dealt to the warps of the grid; each sums the slab partials of its channels in a
//            fixed order and writes the per-channel coefficients
//   barrier
//   phase 2  every block applies the coefficients to the same work items (re-read from L2)
//
// The work items depend on the tensor shape only, not on the grid: a trainer confined to a narrower SM
// partition runs the same items on fewer blocks and gets bit-identical results.
//
// The grid is launched cooperatively (all blocks co-resident or the launch fails), so the barriers cannot
// wait for a block that never starts; every barrier wait is bounded all the same, and a wait that gives up
// records code 0xB1 in the kernel status word instead of hanging the GPU. Barrier words and partial sums
// live in a small workspace owned by the library, one per (device, stream): launches on one stream are
// serialised, so they can share it.
#include <atomic>
#include <cstdlib>
#include <map>
#include <mutex>

#include "common.cuh"
#include "ops.cuh"

namespace srt {

int* tc_status_device_ptr();  // igemm_tcgen05.cu: the status word srt_tc_status() reads

namespace {

constexpr int NTG = 512;     // threads per block
// Registers per thread: 512 x 80 leaves a third of the register file to the kernels of other streams (the
// overlapped weight-gradient GEMMs) and to the tail of the predecessor, so the cooperative grid need not wait
// for whole SMs to drain before all of its blocks are resident.
constexpr int MAX_REGS = 104;
constexpr int ITEMS = 148;   // work items per tensor (upper bound), a property of the algorithm, not the device
constexpr int MAX_TC = 64;   // channel vectors per item: 1 KB of bf16 per row
constexpr int RPT_F = 8;     // rows in flight per thread, forward sums
constexpr int RPT_B = 4;     // backward sums (two or three tensors per row)
constexpr int UNR = 4;       // rows in flight per thread in the apply phases
constexpr unsigned long long BARRIER_LIMIT_NS = 4000000000ull;
constexpr int STATUS_BARRIER_TIMEOUT = 0xB1;

struct GridMap {
  int CV;   // 16-byte vectors per row
  int TC;   // threads across channel vectors
  int RL;   // row lanes
  int GY;   // channel chunks
  int NS;   // row slabs
  int R;    // rows per slab
};

inline GridMap make_grid_map(int64_t rows, int C, int V) {
  GridMap m;
  m.CV = C / V;
  m.TC = m.CV < MAX_TC ? m.CV : MAX_TC;
  m.RL = NTG / m.TC;
  m.GY = (m.CV + m.TC - 1) / m.TC;
  int ns = ITEMS / m.GY;
  if (ns < 1) ns = 1;
  if ((int64_t)ns > rows) ns = (int)rows;
  m.R = (int)((rows + ns - 1) / ns);
  m.NS = (int)((rows + m.R - 1) / m.R);
  return m;
}

// ---- workspace ------------------------------------------------------------------------------------
constexpr size_t WS_BAR_BYTES = 256;
constexpr size_t WS_PARTIAL_ELEMS = (size_t)ITEMS * MAX_TC * 8;  // NS * C never exceeds this while GY <= ITEMS
constexpr size_t WS_COEF_ELEMS = WS_PARTIAL_ELEMS;               // 4 floats per channel, C <= ITEMS*MAX_TC*8 / 4
constexpr size_t WS_BYTES = WS_BAR_BYTES + WS_PARTIAL_ELEMS * sizeof(double2) + WS_COEF_ELEMS * sizeof(float);

struct Workspace {
  unsigned* bar;     // [0] arrivals, [1] generation
  double2* partial;  // [NS][C]
  float* coef;       // [4][C]
};

std::mutex g_ws_mu;
std::map<std::pair<int, cudaStream_t>, void*> g_ws;

int workspace_for(cudaStream_t st, Workspace* w) {
  int dev = 0;
  SRT_CHECK_CUDA(cudaGetDevice(&dev));
  void* base = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_ws_mu);
    auto it = g_ws.find({dev, st});
    if (it == g_ws.end()) {
      SRT_REQUIRE(g_ws.size() < 256, "bn (one launch): more than 256 streams have used it in this process");
      SRT_CHECK_CUDA(cudaMalloc(&base, WS_BYTES));
      SRT_CHECK_CUDA(cudaMemset(base, 0, WS_BAR_BYTES));
      g_ws[{dev, st}] = base;
    } else {
      base = it->second;
    }
  }
  w->bar = (unsigned*)base;
  w->partial = (double2*)((char*)base + WS_BAR_BYTES);
  w->coef = (float*)((char*)base + WS_BAR_BYTES + WS_PARTIAL_ELEMS * sizeof(double2));
  return SRT_OK;
}

// ---- grid barrier ---------------------------------------------------------------------------------
__device__ inline unsigned ld_acquire_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ inline unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// All blocks of the grid arrive; the last one resets the arrival count and bumps the generation, the others
// wait for the generation to change. The words end every barrier as they began it (count 0), so launches
// that follow on the same stream need no reset. Global writes made before the barrier by any thread of any
// block are visible after it to loads that bypass L1 (__ldcg).
//
// One round trip to L2 per arrival: the arrival is an acq_rel atomic (releases this block's writes, which
// thread 0 has observed through __syncthreads; the last arriver acquires everybody's), the generation a block
// waits on is read once when the kernel starts (`gen`, thread 0 only) and counted up locally.
__device__ inline unsigned barrier_generation(const unsigned* bar) {
  unsigned v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(bar + 1) : "memory");
  return v;
}
__device__ inline void grid_barrier(unsigned* bar, unsigned& gen, int* status) {
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned arrived;
    asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(arrived) : "l"(bar) : "memory");
    if (arrived == gridDim.x - 1) {
      asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(bar), "r"(0u) : "memory");
      asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(bar + 1) : "memory");
    } else {
      const unsigned long long t0 = global_ns();
      unsigned spins = 0;
      while (ld_acquire_u32(bar + 1) == gen) {
        if ((++spins & 1023u) == 0 && global_ns() - t0 > BARRIER_LIMIT_NS) {
          if (status) atomicExch(status, STATUS_BARRIER_TIMEOUT);
          break;
        }
      }
    }
    ++gen;
  }
  __syncthreads();
}

// Sum per-thread accumulators a[V], b[V] over the block's row lanes in a fixed order (fp32 lanes combined in
// double); thread layout t = rl * TC + tc. The result for channel c of chunk gy goes to out[c].
template <int V>
__device__ inline void item_reduce_store(const float (&a)[V], const float (&b)[V], const GridMap& m, int gy, int C,
                                         double2* out, float* sh_a, float* sh_b, double2* sh_d) {
  const int t = threadIdx.x;
  __syncthreads();  // the previous item's readers are done with the shared arrays
#pragma unroll
  for (int v = 0; v < V; ++v) { sh_a[t * V + v] = a[v]; sh_b[t * V + v] = b[v]; }
  __syncthreads();
  const int chunk = m.TC * V;
  const int nparts = NTG / chunk;  // >= 1: TC <= 64, V <= 8
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
  const int c = gy * chunk + ch;
  if (part == 0 && c < C) {
    double2 tot = sh_d[ch];
    for (int q = 1; q < nparts; ++q) {
      tot.x += sh_d[q * chunk + ch].x;
      tot.y += sh_d[q * chunk + ch].y;
    }
    out[c] = tot;
  }
}

// One warp per channel: the NS slab partials are summed by lane (strided, in slab order) and combined by a
// fixed butterfly. Every lane returns the total.
__device__ inline double2 warp_sum_partials(const double2* partial, int NS, int C, int c) {
  double2 acc = make_double2(0.0, 0.0);
  for (int s = threadIdx.x & 31; s < NS; s += 32) {
    const double2 v = __ldcg(partial + (size_t)s * C + c);
    acc.x += v.x;
    acc.y += v.y;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    acc.x += __shfl_xor_sync(0xffffffffu, acc.x, o);
    acc.y += __shfl_xor_sync(0xffffffffu, acc.y, o);
  }
  return acc;
}

template <int V>
__device__ inline void load_vec_f32(float (&dst)[V], const float* src) {
#pragma unroll
  for (int v = 0; v < V; v += 4) {
    const float4 a = __ldcg(reinterpret_cast<const float4*>(src + v));
    dst[v] = a.x; dst[v + 1] = a.y; dst[v + 2] = a.z; dst[v + 3] = a.w;
  }
}

// ---- forward ----------------------------------------------------------------------------------------
struct FwdArgs {
  const void* z;
  const void* residual;
  void* y;
  int64_t rows;
  int C;
  GridMap m;
  const float* gamma;
  const float* beta;
  float eps, momentum;
  float* running_mean;
  float* running_var;
  float* mean;
  float* invstd;
  float* scale;
  float* shift;
  int relu;
  Workspace ws;
  int* status;
};

template <typename T>
__global__ void __maxnreg__(MAX_REGS) bn_fwd_grid(const FwdArgs p) {
  pdl_enter();
  constexpr int V = Vec16<T>::N;
  __shared__ float sh_a[NTG * V];
  __shared__ float sh_b[NTG * V];
  __shared__ double2 sh_d[NTG];
  const GridMap& m = p.m;
  const int C = p.C;
  const int64_t rows = p.rows;
  const T* z = (const T*)p.z;
  const int t = threadIdx.x;
  const int tc = t % m.TC, rl = t / m.TC;
  const int n_items = m.NS * m.GY;
  unsigned gen = t == 0 ? barrier_generation(p.ws.bar) : 0u;

  // phase 1: per-item sums of z and z*z
  for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
    const int s = item / m.GY, gy = item % m.GY;
    const int cv = gy * m.TC + tc;
    float sa[V], sq[V];
#pragma unroll
    for (int v = 0; v < V; ++v) { sa[v] = 0.f; sq[v] = 0.f; }
    if (rl < m.RL && cv < m.CV) {
      const int64_t r_begin = (int64_t)s * m.R;
      const int64_t r_end = r_begin + m.R < rows ? r_begin + m.R : rows;
      for (int64_t r0 = r_begin + rl; r0 < r_end; r0 += (int64_t)RPT_F * m.RL) {
        Vec16<T> x[RPT_F];
#pragma unroll
        for (int i = 0; i < RPT_F; ++i) {
          const int64_t r = r0 + (int64_t)i * m.RL;
          if (r < r_end) x[i].load(z + r * C + (int64_t)cv * V);
        }
#pragma unroll
        for (int i = 0; i < RPT_F; ++i) {
          const int64_t r = r0 + (int64_t)i * m.RL;
          if (r < r_end) {
            float f[V];
            x[i].unpack(f);
#pragma unroll
            for (int v = 0; v < V; ++v) { sa[v] += f[v]; sq[v] = fmaf(f[v], f[v], sq[v]); }
          }
        }
      }
    }
    item_reduce_store<V>(sa, sq, m, gy, C, p.ws.partial + (size_t)s * C, sh_a, sh_b, sh_d);
  }
  grid_barrier(p.ws.bar, gen, p.status);

  // finalize: one warp per channel
  {
    const int lane = t & 31;
    const int gw = blockIdx.x * (NTG / 32) + (t >> 5), n_warps = gridDim.x * (NTG / 32);
    for (int c = gw; c < C; c += n_warps) {
      const double2 tot = warp_sum_partials(p.ws.partial, m.NS, C, c);
      if (lane != 0) continue;
      const double mu = tot.x / (double)rows;
      double var = tot.y / (double)rows - mu * mu;
      if (var < 0.0) var = 0.0;
      const float is = (float)(1.0 / sqrt(var + (double)p.eps));
      const float g = p.gamma ? p.gamma[c] : 1.f, b = p.beta ? p.beta[c] : 0.f;
      p.mean[c] = (float)mu;
      p.invstd[c] = is;
      const float sc = g * is;
      p.scale[c] = sc;
      p.shift[c] = b - (float)mu * sc;
      if (p.running_mean) p.running_mean[c] = (1.f - p.momentum) * p.running_mean[c] + p.momentum * (float)mu;
      if (p.running_var) {
        const double unbiased = rows > 1 ? var * (double)rows / (double)(rows - 1) : var;
        p.running_var[c] = (1.f - p.momentum) * p.running_var[c] + p.momentum * (float)unbiased;
      }
    }
  }
  grid_barrier(p.ws.bar, gen, p.status);

  // phase 2: y = relu(z*scale + shift + residual) over the same items
  const T* res = (const T*)p.residual;
  T* y = (T*)p.y;
  for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
    const int s = item / m.GY, gy = item % m.GY;
    const int cv = gy * m.TC + tc;
    if (rl >= m.RL || cv >= m.CV) continue;
    float sc[V], sf[V];
    load_vec_f32<V>(sc, p.scale + cv * V);
    load_vec_f32<V>(sf, p.shift + cv * V);
    const int64_t r_begin = (int64_t)s * m.R;
    const int64_t r_end = r_begin + m.R < rows ? r_begin + m.R : rows;
    for (int64_t r0 = r_begin + rl; r0 < r_end; r0 += (int64_t)UNR * m.RL) {
      Vec16<T> x[UNR], rv[UNR];
#pragma unroll
      for (int i = 0; i < UNR; ++i) {
        const int64_t r = r0 + (int64_t)i * m.RL;
        if (r < r_end) {
          const int64_t o = r * C + (int64_t)cv * V;
          x[i].load(z + o);
          if (res) rv[i].load(res + o);
        }
      }
#pragma unroll
      for (int i = 0; i < UNR; ++i) {
        const int64_t r = r0 + (int64_t)i * m.RL;
        if (r >= r_end) continue;
        float f[V];
        x[i].unpack(f);
#pragma unroll
        for (int v = 0; v < V; ++v) f[v] = fmaf(f[v], sc[v], sf[v]);
        if (res) {
          float rf[V];
          rv[i].unpack(rf);
#pragma unroll
          for (int v = 0; v < V; ++v) f[v] += rf[v];
        }
        if (p.relu) {
#pragma unroll
          for (int v = 0; v < V; ++v) f[v] = fmaxf(f[v], 0.f);
        }
        Vec16<T> o;
        o.pack(f);
        o.store(y + r * C + (int64_t)cv * V);
      }
    }
  }
}

// ---- backward ---------------------------------------------------------------------------------------
struct BwdArgs {
  const void* dy;
  const void* y;   // stored output for the ReLU mask (residual units); null = recompute the mask from z
  const void* z;
  void* dz;
  void* dres;      // masked gradient for the residual branch, or null
  int64_t rows;
  int C;
  GridMap m;
  const float* gamma;
  const float* mean;
  const float* invstd;
  const float* scale;
  const float* shift;
  int relu;
  float* dgamma;
  float* dbeta;
  Workspace ws;
  int* status;
};

// ReLU mask of y = relu(z*scale + shift [+ residual]): from the stored y when given, otherwise recomputed
// from z with the fused multiply-add of the forward pass (same sign as the stored, rounded y).
template <typename T, int V>
__device__ __forceinline__ void mask_gradient(float (&g)[V], const float (&x)[V], const Vec16<T>* y_vec,
                                              const float (&sc)[V], const float (&sf)[V]) {
  if (y_vec) {
    const Vec16<T>& yv = *y_vec;
    float yy[V];
    yv.unpack(yy);
#pragma unroll
    for (int v = 0; v < V; ++v) g[v] = yy[v] > 0.f ? g[v] : 0.f;
  } else {
#pragma unroll
    for (int v = 0; v < V; ++v) g[v] = fmaf(x[v], sc[v], sf[v]) > 0.f ? g[v] : 0.f;
  }
}

template <int V>
__device__ __forceinline__ void mask_gradient_bits(float (&g)[V], unsigned bits) {
#pragma unroll
  for (int v = 0; v < V; ++v) g[v] = ((bits >> v) & 1u) ? g[v] : 0.f;
}

// MASK: 0 no ReLU, 1 mask from the stored output y, 2 mask recomputed from z, 3 mask from one bit per element (the
// y pointer then holds the bytes the forward apply kernel wrote; 8-element vectors) (compile-time, so the vectors and
// loads of the unused variants take no registers)
template <typename T, int MASK>
__global__ void __maxnreg__(MAX_REGS) bn_bwd_grid(const BwdArgs p) {
  pdl_enter();
  constexpr int V = Vec16<T>::N;
  __shared__ float sh_a[NTG * V];
  __shared__ float sh_b[NTG * V];
  __shared__ double2 sh_d[NTG];
  const GridMap& m = p.m;
  const int C = p.C;
  const int64_t rows = p.rows;
  const T* dy = (const T*)p.dy;
  const T* yk = (const T*)p.y;
  const T* z = (const T*)p.z;
  T* dres = (T*)p.dres;
  const int t = threadIdx.x;
  const int tc = t % m.TC, rl = t / m.TC;
  const int n_items = m.NS * m.GY;
  constexpr bool recompute_mask = MASK == 2;
  unsigned gen = t == 0 ? barrier_generation(p.ws.bar) : 0u;

  // phase 1: sums of g and g*xhat per item, g = dy under the ReLU mask; g is also what the residual branch gets
  for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
    const int s = item / m.GY, gy = item % m.GY;
    const int cv = gy * m.TC + tc;
    float sg[V], sgx[V];
#pragma unroll
    for (int v = 0; v < V; ++v) { sg[v] = 0.f; sgx[v] = 0.f; }
    if (rl < m.RL && cv < m.CV) {
      float mu[V], is[V], sc[V], sf[V];
      load_vec_f32<V>(mu, p.mean + cv * V);
      load_vec_f32<V>(is, p.invstd + cv * V);
      if (recompute_mask) {
        load_vec_f32<V>(sc, p.scale + cv * V);
        load_vec_f32<V>(sf, p.shift + cv * V);
      } else {
#pragma unroll
        for (int v = 0; v < V; ++v) { sc[v] = 0.f; sf[v] = 0.f; }
      }
      const int64_t r_begin = (int64_t)s * m.R;
      const int64_t r_end = r_begin + m.R < rows ? r_begin + m.R : rows;
      for (int64_t r0 = r_begin + rl; r0 < r_end; r0 += (int64_t)RPT_B * m.RL) {
        Vec16<T> a[RPT_B], b[RPT_B], yv[RPT_B];  // the stored output travels with the other two loads
        unsigned mb[RPT_B];
#pragma unroll
        for (int i = 0; i < RPT_B; ++i) {
          const int64_t r = r0 + (int64_t)i * m.RL;
          if (r < r_end) {
            const int64_t o = r * C + (int64_t)cv * V;
            a[i].load(dy + o);
            b[i].load(z + o);
            if (MASK == 1) yv[i].load(yk + o);
            if (MASK == 3) mb[i] = reinterpret_cast<const uint8_t*>(p.y)[o / V];
          }
        }
#pragma unroll
        for (int i = 0; i < RPT_B; ++i) {
          const int64_t r = r0 + (int64_t)i * m.RL;
          if (r >= r_end) continue;
          const int64_t o = r * C + (int64_t)cv * V;
          float g[V], x[V];
          a[i].unpack(g);
          b[i].unpack(x);
          if (MASK == 3) mask_gradient_bits<V>(g, mb[i]);
          else if (MASK != 0) mask_gradient<T, V>(g, x, MASK == 1 ? &yv[i] : nullptr, sc, sf);
          if (dres) {
            Vec16<T> w;
            w.pack(g);
            w.store(dres + o);
          }
#pragma unroll
          for (int v = 0; v < V; ++v) {
            sg[v] += g[v];
            sgx[v] = fmaf(g[v], (x[v] - mu[v]) * is[v], sgx[v]);
          }
        }
      }
    }
    item_reduce_store<V>(sg, sgx, m, gy, C, p.ws.partial + (size_t)s * C, sh_a, sh_b, sh_d);
  }
  grid_barrier(p.ws.bar, gen, p.status);

  // finalize: dgamma, dbeta and the coefficients of dz = ka*g + kb*(x - mean) + kd
  {
    const int lane = t & 31;
    const int gw = blockIdx.x * (NTG / 32) + (t >> 5), n_warps = gridDim.x * (NTG / 32);
    float* coef = p.ws.coef;
    for (int c = gw; c < C; c += n_warps) {
      const double2 tot = warp_sum_partials(p.ws.partial, m.NS, C, c);
      if (lane != 0) continue;
      if (p.dbeta) p.dbeta[c] = (float)tot.x;
      if (p.dgamma) p.dgamma[c] = (float)tot.y;
      const float g = p.gamma ? p.gamma[c] : 1.f;
      const float k0 = g * p.invstd[c];
      const float mg = (float)(tot.x / (double)rows), mgx = (float)(tot.y / (double)rows);
      coef[c] = k0;
      coef[C + c] = -k0 * mgx * p.invstd[c];
      coef[2 * C + c] = -k0 * mg;
    }
  }
  grid_barrier(p.ws.bar, gen, p.status);

  // phase 2: dz over the same items; the masked gradient comes back from dres where phase 1 stored it
  T* dz = (T*)p.dz;
  const T* gsrc = dres ? (const T*)dres : dy;
  const bool mask_again = MASK != 0 && !dres;
  for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
    const int s = item / m.GY, gy = item % m.GY;
    const int cv = gy * m.TC + tc;
    if (rl >= m.RL || cv >= m.CV) continue;
    float ka[V], kb[V], kd[V], mu[V], sc[V], sf[V];
    load_vec_f32<V>(ka, p.ws.coef + cv * V);
    load_vec_f32<V>(kb, p.ws.coef + C + cv * V);
    load_vec_f32<V>(kd, p.ws.coef + 2 * C + cv * V);
    load_vec_f32<V>(mu, p.mean + cv * V);
    if (MASK == 2 && mask_again) {
      load_vec_f32<V>(sc, p.scale + cv * V);
      load_vec_f32<V>(sf, p.shift + cv * V);
    } else {
#pragma unroll
      for (int v = 0; v < V; ++v) { sc[v] = 0.f; sf[v] = 0.f; }
    }
    const int64_t r_begin = (int64_t)s * m.R;
    const int64_t r_end = r_begin + m.R < rows ? r_begin + m.R : rows;
    for (int64_t r0 = r_begin + rl; r0 < r_end; r0 += (int64_t)UNR * m.RL) {
      Vec16<T> a[UNR], b[UNR], yv[UNR];
      unsigned mb[UNR];
#pragma unroll
      for (int i = 0; i < UNR; ++i) {
        const int64_t r = r0 + (int64_t)i * m.RL;
        if (r < r_end) {
          const int64_t o = r * C + (int64_t)cv * V;
          a[i].load(gsrc + o);
          b[i].load(z + o);
          if (MASK == 1 && mask_again) yv[i].load(yk + o);
          if (MASK == 3 && mask_again) mb[i] = reinterpret_cast<const uint8_t*>(p.y)[o / V];
        }
      }
#pragma unroll
      for (int i = 0; i < UNR; ++i) {
        const int64_t r = r0 + (int64_t)i * m.RL;
        if (r >= r_end) continue;
        const int64_t o = r * C + (int64_t)cv * V;
        float g[V], x[V];
        a[i].unpack(g);
        b[i].unpack(x);
        if (MASK == 3 && mask_again) mask_gradient_bits<V>(g, mb[i]);
        else if (mask_again) mask_gradient<T, V>(g, x, MASK == 1 ? &yv[i] : nullptr, sc, sf);
        float out[V];
#pragma unroll
        for (int v = 0; v < V; ++v) out[v] = fmaf(ka[v], g[v], fmaf(kb[v], x[v] - mu[v], kd[v]));
        Vec16<T> w;
        w.pack(out);
        w.store(dz + o);
      }
    }
  }
}

// Cooperative launch of a one-block-per-SM grid; early (programmatic) launch on top when the driver takes
// both attributes together, which is probed once.
template <typename Args>
int launch_grid(void (*kernel)(const Args), int blocks, cudaStream_t st, const Args& a) {
  static std::atomic<int> early_ok{1};
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)blocks);
  cfg.blockDim = dim3(NTG);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  const bool early = (pdl_classes() & PDL_NORM) != 0 && early_ok.load(std::memory_order_relaxed) != 0;
  cfg.numAttrs = early ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, a);
  if (e != cudaSuccess && early) {
    (void)cudaGetLastError();
    early_ok.store(0, std::memory_order_relaxed);
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, kernel, a);
  }
  SRT_CHECK_CUDA(e);
  count_launch();
  return SRT_OK;
}

inline int grid_blocks(const GridMap& m) {
  const int items = m.NS * m.GY, sms = sm_count();
  return items < sms ? items : sms;
}

inline size_t env_mb(const char* name, long dflt) {
  const char* e = getenv(name);
  return (size_t)(e ? atol(e) : dflt) << 20;
}

}  // namespace

// Any tensor whose channel count is a multiple of the 16-byte vector and small enough for the partial-sum
// workspace qualifies.
// After a barrier wait has given up, arrival counts may be left non-zero; with the device idle (the caller
// has synchronised) put the barrier words of every workspace of the current device back to zero.
void bn_grid_reset_barriers() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return;
  std::lock_guard<std::mutex> lk(g_ws_mu);
  for (auto& kv : g_ws)
    if (kv.first.first == dev) (void)cudaMemset(kv.second, 0, WS_BAR_BYTES);
}

bool bn_fused_fits(int dtype, int64_t rows, int C, int backward) {
  (void)backward;
  const int V = dtype == SRT_F32 ? 4 : 8;
  if (rows <= 0 || C <= 0 || C % V != 0) return false;
  const GridMap m = make_grid_map(rows, C, V);
  return m.GY <= ITEMS && (size_t)m.NS * C <= WS_PARTIAL_ELEMS && (size_t)4 * C <= WS_COEF_ELEMS;
}

// Where the one-launch kernels pay inside a training step (measured on ResNet-152, batch 64): alone on the GPU
// they beat the three-kernel path in backward at every size (0.6x the time on the large residual tensors) and
// tie or lose in forward. SIRIUS_B200_FUSED_BN_BWD_MIN_MB / SIRIUS_B200_FUSED_BN_FWD_MAX_MB move the lines.
bool bn_fused_pays(int dtype, int64_t rows, int C, int backward) {
  static const size_t bwd_min = env_mb("SIRIUS_B200_FUSED_BN_BWD_MIN_MB", 16);
  static const size_t fwd_max = env_mb("SIRIUS_B200_FUSED_BN_FWD_MAX_MB", 0);
  const size_t bytes = (size_t)rows * C * (dtype == SRT_F32 ? 4 : 2);
  if (!bn_fused_fits(dtype, rows, C, backward)) return false;
  return backward ? bytes >= bwd_min : bytes <= fwd_max;
}

int bn_forward_fused(int dtype, const void* z, const void* residual, void* y, int64_t rows, int C, const float* gamma,
                     const float* beta, float eps, float momentum, float* rm, float* rv, float* mean, float* invstd,
                     float* scale, float* shift, int relu, cudaStream_t st) {
  SRT_REQUIRE(bn_fused_fits(dtype, rows, C, 0), "bn_forward_fused: unsupported shape (rows %lld, C %d)", (long long)rows, C);
  FwdArgs a;
  a.z = z; a.residual = residual; a.y = y; a.rows = rows; a.C = C;
  a.m = make_grid_map(rows, C, dtype == SRT_F32 ? 4 : 8);
  a.gamma = gamma; a.beta = beta; a.eps = eps; a.momentum = momentum;
  a.running_mean = rm; a.running_var = rv; a.mean = mean; a.invstd = invstd; a.scale = scale; a.shift = shift;
  a.relu = relu;
  a.status = tc_status_device_ptr();
  if (int rc = workspace_for(st, &a.ws)) return rc;
  const int blocks = grid_blocks(a.m);
  if (dtype == SRT_F32) return launch_grid(bn_fwd_grid<float>, blocks, st, a);
  return launch_grid(bn_fwd_grid<__nv_bfloat16>, blocks, st, a);
}

int bn_backward_fused(int dtype, const void* dy, const void* y, const void* z, int64_t rows, int C, const float* gamma,
                      const float* mean, const float* invstd, const float* scale, const float* shift, int relu, void* dz,
                      void* dres, float* dgamma, float* dbeta, cudaStream_t st, const uint8_t* relu_bits) {
  SRT_REQUIRE(bn_fused_fits(dtype, rows, C, 1), "bn_backward_fused: unsupported shape (rows %lld, C %d)", (long long)rows, C);
  SRT_REQUIRE(!relu || y || relu_bits || (scale && shift), "bn_backward_fused: the ReLU mask needs y, its bits or scale/shift");
  SRT_REQUIRE(!relu_bits || (dtype == SRT_BF16 && relu), "bn_backward_fused: the ReLU bit mask goes with bf16 tensors under a ReLU");
  BwdArgs a;
  a.dy = dy; a.y = relu_bits ? (const void*)relu_bits : y; a.z = z; a.dz = dz; a.dres = dres; a.rows = rows; a.C = C;
  a.m = make_grid_map(rows, C, dtype == SRT_F32 ? 4 : 8);
  a.gamma = gamma; a.mean = mean; a.invstd = invstd; a.scale = scale; a.shift = shift; a.relu = relu;
  a.dgamma = dgamma; a.dbeta = dbeta;
  a.status = tc_status_device_ptr();
  if (int rc = workspace_for(st, &a.ws)) return rc;
  const int blocks = grid_blocks(a.m);
  const int mask = !relu ? 0 : relu_bits ? 3 : (y ? 1 : 2);
  if (dtype == SRT_F32)
    return launch_grid(mask == 0 ? bn_bwd_grid<float, 0> : mask == 1 ? bn_bwd_grid<float, 1> : bn_bwd_grid<float, 2>, blocks, st, a);
  return launch_grid(mask == 0 ? bn_bwd_grid<__nv_bfloat16, 0> : mask == 1 ? bn_bwd_grid<__nv_bfloat16, 1>
                     : mask == 2 ? bn_bwd_grid<__nv_bfloat16, 2> : bn_bwd_grid<__nv_bfloat16, 3>, blocks, st, a);
}

}  // namespace srt
