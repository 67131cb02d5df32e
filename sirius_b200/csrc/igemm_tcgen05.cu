// bf16 implicit-GEMM convolution on the sm_100a tensor cores.
//
// Two warp-specialised kernels:
//
//   igemm_fwd_persistent<BN, NS, PAIR>   fprop and dgrad.  D[m][n] = sum_k A(m,k) B[n][k]
//       Persistent: one CTA (or one CTA pair, cta_group::2) per SM walks output tiles of 128 (256 for a pair)
//       rows x BN filters; 704 threads.
//       A: 128 output positions x 64 reduction elements per stage, gathered from the NHWC source with 16-byte
//          cp.async (zero-fill outside the image) straight into the 128-byte-swizzled K-major layout
//          tcgen05.mma reads; for 1x1 stride-1 filters the tile is a plain matrix block and comes by TMA.
//       B: BN filters x 64 reduction elements per stage by TMA (K-major, 128-byte swizzle); in a pair each CTA
//          loads its half of the filters and the leader's MMA reads both halves.
//       Warps: 0 TMA producer, 1 MMA issuer (allocates tensor memory), 2-3 and 20-21 gather producers, 4-19
//       four epilogue groups of four warps (warp w of a group owns TMEM lanes 32w..32w+31). The accumulator is
//       double-buffered in tensor memory (2 x BN columns) so the epilogue of tile t overlaps the main loop of
//       tile t+1; 64-column slabs of a tile are dealt round-robin to the epilogue groups, each slab announced
//       on its own mbarrier per (group, accumulator buffer) so that a waiter never falls two phases behind.
//       The epilogue converts to bf16, adds bias / residual, optionally accumulates per-channel sums for
//       BatchNorm, stages the slab in shared memory and stores it with TMA.
//   igemm_wgrad_kernel                   filter gradient.  dW[k][j] = sum_pix dy[pix][k] X(pix,j)
//       192 threads, one 128-filter tile per CTA.
//       A: dy block, 64 pixels x 128 filters per stage by TMA (MN-major, two 64-wide boxes).
//       B: 64 pixels x BN gathered input channels per stage by cp.async (MN-major).
//       The pixel range is split across blockIdx.z; partial sums go to scratch and are reduced in a fixed
//       order afterwards.
//
// A ring of NS shared-memory stages is handed over with mbarriers. No load uses cluster multicast: every CTA
// loads its own tiles (the pair's commit is the only cluster-scope signal). Every wait is bounded and reports
// through a status word.
#include <cuda.h>

#include <mutex>

#include "common.cuh"
#include "conv_geom.cuh"
#include "ops.cuh"
#include "ptx.cuh"

namespace srt {

static int g_force_gather = 0;  // plan override: fetch plain-matrix operands with the gather threads
static int g_force_pair = getenv("SIRIUS_B200_CONV_PAIR") ? atoi(getenv("SIRIUS_B200_CONV_PAIR")) : -1;  // plan override: 0 never pairs CTAs
static int g_im2col_enabled = getenv("SIRIUS_B200_CONV_IM2COL") ? atoi(getenv("SIRIUS_B200_CONV_IM2COL")) : 1;  // 0: gather filters wider than 1x1

namespace {

using namespace ptx;
using bf16 = __nv_bfloat16;

constexpr int BM = 128;       // output rows per CTA (= TMEM lanes)
constexpr int BK = 64;        // reduction elements per stage (one 128-byte swizzle row of bf16)
constexpr int NTHREADS = 192;
constexpr int NPROD = 128;    // gather / epilogue threads
constexpr int LAG = 2;        // cp.async groups kept in flight per producer thread
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KiB

__device__ int g_tc_status;  // 0 = ok; otherwise the code of the first wait that gave up

enum WaitCode { W_PROD_EMPTY = 1, W_TMA_EMPTY = 2, W_MMA_FULL = 3, W_EPI_TMEM = 4 };

// Phase time stamps of the persistent kernel, compiled in only for timing studies (-DSRT_PHASE_STAMPS; the shipped
// library does not define it): slot i of CTA b is written to stamps[b * 16 + i] as a %globaltimer reading.
#ifdef SRT_PHASE_STAMPS
__device__ unsigned long long* g_phase_stamps;
__device__ __forceinline__ void phase_stamp(int i) {
  if (g_phase_stamps) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    g_phase_stamps[blockIdx.x * 16 + i] = t;
  }
}
#define SRT_STAMP(i) phase_stamp(i)
#else
#define SRT_STAMP(i)
#endif

// n / d for 0 <= n < 2^31 with a precomputed multiplier and shift (d >= 1).
__host__ inline void fastdiv_make(uint32_t d, uint32_t* mul, uint32_t* shr) {
  uint32_t p = 0;
  while ((1u << p) < d) ++p;
  if (d == 1) { *mul = 0; *shr = 0; return; }
  *mul = (uint32_t)((((uint64_t)1 << (31 + p)) + d - 1) / d);
  *shr = p - 1;
}
__device__ __forceinline__ int fastdiv(int n, int d, uint32_t mul, uint32_t shr) {
  return d == 1 ? n : (int)(__umulhi((uint32_t)n, mul) >> shr);
}


struct WgradParams {
  GatherGeom g;  // fprop geometry: rows = output pixels, gather from x
  const bf16* x;
  float* out;          // [splits][Kout][J] partials, or dW itself when splits == 1
  int pix_per_split;   // multiple of 64
  int b_tma;           // how X arrives: 0 gathered with cp.async, 1 plain [pixels][C] matrix by TMA (1x1 stride-1
                       // filters), 2 im2col TMA (one 64-pixel x 64-channel block per filter tap and channel chunk)
  uint32_t hw_mul, hw_shr, w_mul, w_shr;  // fast division by out_h*out_w and out_w
  int* status;
};

struct SmemLayout {
  uint8_t* a;
  uint8_t* b;
  uint64_t* full;
  uint64_t* empty;
  uint64_t* tmem_full;
  uint32_t* tmem_ptr;
};

template <int NS, int B_STAGE_BYTES>
__device__ __forceinline__ SmemLayout carve_smem(uint8_t* raw) {
  SmemLayout s;
  uint8_t* base = (uint8_t*)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
  s.a = base;
  s.b = base + NS * A_STAGE_BYTES;
  uint8_t* tail = s.b + NS * B_STAGE_BYTES;
  s.full = (uint64_t*)tail;
  s.empty = s.full + NS;
  s.tmem_full = s.empty + NS;
  s.tmem_ptr = (uint32_t*)(s.tmem_full + 1);
  return s;
}

template <int NS, int B_STAGE_BYTES>
constexpr size_t smem_bytes() {
  return 1024 + (size_t)NS * (A_STAGE_BYTES + B_STAGE_BYTES) + (2 * NS + 1) * 8 + 16;
}

// Issue the NI 16-byte copies of one stage for this producer thread, then hand over the stage
// that was issued LAG iterations ago (its copies have landed once at most LAG groups are pending).
template <int NS>
__device__ __forceinline__ void producer_handover(int kb, uint64_t* full) {
  cp_async_commit();
  if (kb >= LAG) {
    cp_async_wait<LAG>();
    fence_proxy_async_smem();
    mbar_arrive(smem_u32(&full[(kb - LAG) % NS]));
  }
}
template <int NS>
__device__ __forceinline__ void producer_drain(int issued, uint64_t* full) {
  cp_async_wait<0>();
  fence_proxy_async_smem();
  for (int kb = issued > LAG ? issued - LAG : 0; kb < issued; ++kb)
    mbar_arrive(smem_u32(&full[kb % NS]));
}

// ------------------------------------------------------------------------------------------

// ------------------------------------------------------------------------------------------
template <int BN, int NS>
__global__ void __launch_bounds__(NTHREADS)
igemm_wgrad_kernel(const WgradParams p, const __grid_constant__ CUtensorMap tmap_dy,
                   const __grid_constant__ CUtensorMap tmap_x) {
  constexpr int B_STAGE_BYTES = BN * BK * 2;  // BN/64 blocks of [64 pixels][128 bytes]
  constexpr int CPR = BN / 8;                 // 16-byte chunks per pixel row
  constexpr int RSTEP = NPROD / CPR;          // pixel rows covered per pass
  constexpr int NI = BK / RSTEP;              // copies per thread per stage
  extern __shared__ uint8_t smem_raw[];
  SmemLayout sm = carve_smem<NS, B_STAGE_BYTES>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const GatherGeom& g = p.g;
  const int Kout = g.Nout, J = g.Kg;
  const int j0 = blockIdx.x * BN, ko0 = blockIdx.y * BM;
  const int pbeg = blockIdx.z * p.pix_per_split;
  const int pend = min(g.M, pbeg + p.pix_per_split);
  const int nkb = (pend - pbeg + BK - 1) / BK;

  if (tid == 0) {
    const uint32_t full_count = p.b_tma ? 1u : (uint32_t)(NPROD + 1);
    for (int s = 0; s < NS; ++s) {
      mbar_init(smem_u32(&sm.full[s]), full_count);
      mbar_init(smem_u32(&sm.empty[s]), 1);
    }
    mbar_init(smem_u32(sm.tmem_full), 1);
    mbar_fence_init();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&tmap_dy);
    if (p.b_tma) tma_prefetch_desc(&tmap_x);
  }
  if (warp == 5) {
    tmem_alloc(smem_u32(sm.tmem_ptr), BN);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *sm.tmem_ptr;
  // Everything above touches only shared memory, tensor memory and the kernel parameters, so under an early
  // (programmatic dependent) launch it runs beside the predecessor's tail; global memory is first touched below.
  pdl_enter();

  if (warp < 4) {
    // ---------------- gather producers: x(pix, j) for 64 pixels x BN columns ----------------
    if (!p.b_tma) {
    const int cj = tid % CPR, r0 = tid / CPR;
    const int jj = j0 + cj * 8;
    const bool j_ok = jj < J;
    const int tap = jj / g.src_c, c = jj - tap * g.src_c;
    const int r = tap / g.S, sf = tap - r * g.S;
    const int hw = g.out_h * g.out_w;
    // destination of row r0 in block cj/8; later rows step RSTEP*128 bytes (RSTEP % 8 == 0)
    const uint32_t dst_off = (uint32_t)(cj >> 3) * 8192u + (uint32_t)r0 * 128u +
                             (uint32_t)(((cj & 7) ^ (r0 & 7)) << 4);
    // This thread's pixels are pbeg + r0, + RSTEP, + 2 RSTEP, ... through all k-blocks (NI * RSTEP = BK): decoded
    // once, then advanced with carries; the tap's source position follows from (oh, ow) with two multiply-adds.
    int pix = pbeg + r0;
    int n = fastdiv(pix, hw, p.hw_mul, p.hw_shr);
    int oh = fastdiv(pix - n * hw, g.out_w, p.w_mul, p.w_shr), ow = pix - n * hw - oh * g.out_w;
    int issued = 0;
    for (int kb = 0; kb < nkb; ++kb) {
      const int s = kb % NS;
      const uint32_t ph = (uint32_t)(kb / NS) & 1u;
      if (!mbar_wait(smem_u32(&sm.empty[s]), ph ^ 1u, p.status, W_PROD_EMPTY)) break;
      const uint32_t dst0 = smem_u32(sm.b + s * B_STAGE_BYTES) + dst_off;
#pragma unroll
      for (int i = 0; i < NI; ++i) {
        const int ih = oh * g.stride - g.pad + r, iw = ow * g.stride - g.pad + sf;
        const bool v = j_ok && pix < pend && (unsigned)ih < (unsigned)g.src_h && (unsigned)iw < (unsigned)g.src_w;
        const int off = v ? ((n * g.src_h + ih) * g.src_w + iw) * g.src_c + c : 0;
        cp_async_16(dst0 + (uint32_t)i * (uint32_t)(RSTEP * 128), p.x + off, v ? 16u : 0u);
        pix += RSTEP;
        ow += RSTEP;
        while (ow >= g.out_w) {
          ow -= g.out_w;
          if (++oh == g.out_h) { oh = 0; ++n; }
        }
      }
      producer_handover<NS>(kb, sm.full);
      issued = kb + 1;
    }
    producer_drain<NS>(issued, sm.full);
    }

    // ---------------- epilogue: fp32 partial tile ----------------
    const bool ready = mbar_wait(smem_u32(sm.tmem_full), 0u, p.status, W_EPI_TMEM);
    tc_fence_after_sync();
    const int ko = ko0 + warp * 32 + lane;
    float* out = p.out + (size_t)blockIdx.z * Kout * J;
#pragma unroll 1
    for (int cb = 0; cb < BN / 32; ++cb) {
      uint32_t acc[32];
      tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(cb * 32), acc);
      tmem_ld_wait();
      if (ready && ko < Kout) {
#pragma unroll
        for (int v = 0; v < 8; ++v) {
          const int col = j0 + cb * 32 + v * 4;
          if (col < J) {
            float4 o = make_float4(__uint_as_float(acc[v * 4]), __uint_as_float(acc[v * 4 + 1]),
                                   __uint_as_float(acc[v * 4 + 2]), __uint_as_float(acc[v * 4 + 3]));
            *reinterpret_cast<float4*>(out + (size_t)ko * J + col) = o;
          }
        }
      }
    }
  } else if (warp == 4) {
    if (lane == 0) {
      // im2col: 64-column block blk of the tile is one filter tap and one 64-channel chunk of it; blocks at and
      // beyond the last column are not loaded (their products land in columns the epilogue does not store)
      int blk_c[BN / 64], blk_live = 0;
      uint16_t blk_r[BN / 64], blk_s[BN / 64];
#pragma unroll
      for (int blk = 0; blk < BN / 64; ++blk) {
        const int j = j0 + blk * 64;
        const int tap = j / g.src_c;
        blk_c[blk] = j - tap * g.src_c;
        blk_r[blk] = (uint16_t)(tap / g.S);
        blk_s[blk] = (uint16_t)(tap - (tap / g.S) * g.S);
        if (j < J) ++blk_live;
      }
      const int hw = g.out_h * g.out_w;
      const uint32_t b_bytes = p.b_tma == 1 ? (uint32_t)B_STAGE_BYTES : p.b_tma == 2 ? (uint32_t)blk_live * 8192u : 0u;
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % NS;
        const uint32_t ph = (uint32_t)(kb / NS) & 1u;
        if (!mbar_wait(smem_u32(&sm.empty[s]), ph ^ 1u, p.status, W_TMA_EMPTY)) break;
        const uint32_t bar = smem_u32(&sm.full[s]);
        mbar_arrive_expect_tx(bar, (uint32_t)A_STAGE_BYTES + b_bytes);
        const uint32_t dst = smem_u32(sm.a + s * A_STAGE_BYTES);
        const int pix0 = pbeg + kb * BK;
        tma_load_2d(dst, &tmap_dy, bar, ko0, pix0);
        tma_load_2d(dst + 8192u, &tmap_dy, bar, ko0 + 64, pix0);
        const uint32_t dstb = smem_u32(sm.b + s * B_STAGE_BYTES);
        if (p.b_tma == 1) {
#pragma unroll
          for (int blk = 0; blk < BN / 64; ++blk)
            tma_load_2d(dstb + (uint32_t)blk * 8192u, &tmap_x, bar, j0 + blk * 64, pix0);
        } else if (p.b_tma == 2) {
          // base pixel of the k-block's first output position; the 64 positions are consecutive base pixels
          const int n = fastdiv(pix0, hw, p.hw_mul, p.hw_shr);
          const int rem = pix0 - n * hw;
          const int oh = fastdiv(rem, g.out_w, p.w_mul, p.w_shr), ow = rem - oh * g.out_w;
          const int bw = ow * g.stride - g.pad, bh = oh * g.stride - g.pad;
#pragma unroll
          for (int blk = 0; blk < BN / 64; ++blk)
            if (blk < blk_live)
              tma_load_im2col_4d(dstb + (uint32_t)blk * 8192u, &tmap_x, bar, blk_c[blk], bw, bh, n, blk_s[blk], blk_r[blk]);
        }
      }
    }
  } else {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, 1, 1);
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % NS;
        const uint32_t ph = (uint32_t)(kb / NS) & 1u;
        if (!mbar_wait(smem_u32(&sm.full[s]), ph, p.status, W_MMA_FULL)) break;
        tc_fence_after_sync();
        const uint32_t a0 = smem_u32(sm.a + s * A_STAGE_BYTES);
        const uint32_t b0 = smem_u32(sm.b + s * B_STAGE_BYTES);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k) {
          // 16 pixels = two groups of 8 K-rows (1024 bytes each); 64-wide M/N blocks 8192 apart
          const uint64_t ad = make_smem_desc_sw128(a0 + k * 2048, 8192, 1024);
          const uint64_t bd = make_smem_desc_sw128(b0 + k * 2048, 8192, 1024);
          umma_bf16(tmem_base, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
        }
        umma_commit(smem_u32(&sm.empty[s]));
      }
      umma_commit(smem_u32(sm.tmem_full));
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 5) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, BN);
  }
}


// ------------------------------------------------------------------------------------------
// Filter gradient on CTA pairs (tcgen05 cta_group::2): a pair owns a 256-filter x 256-column tile of dW for one
// split of the pixel range. CTA r of the pair stages, per k-block of 64 pixels, its 128 filters of dy (two
// 64-filter boxes) and its 128 of the tile's columns of X (two 64-channel blocks, plain or im2col TMA), the
// leader issues 256 x 256 x 16 MMAs over both CTAs' shared memory, and each CTA finds its 128 filter rows x 256
// columns in its own tensor memory. Per k-block an SM then receives 32 KB for 128 x 256 x 64 multiply-adds, half of
// what the single-CTA kernel's 128 x 128 tile needs, and one CTA per SM with a six-stage ring covers the load
// latency. The fp32 tile leaves through shared memory (the ring's stages, free by then) and TMA stores of
// 128 rows x 32 columns, which write whole lines where a store per thread and row would write 16-byte pieces.
// Both operands must come by TMA (the gather path stays with the single-CTA kernel). No load is multicast.
constexpr int WP_NS = 6;
constexpr int WP_STAGE_BYTES = 32768;  // 16 KB of dy + 16 KB of X per CTA and k-block
constexpr size_t wgrad_pair_smem_bytes() { return 1024 + (size_t)WP_NS * WP_STAGE_BYTES + (2 * WP_NS + 1) * 8 + 16; }

__global__ void __launch_bounds__(NTHREADS, 1)
igemm_wgrad_pair(const WgradParams p, const __grid_constant__ CUtensorMap tmap_dy,
                 const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_out) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = (uint64_t*)(base + WP_NS * WP_STAGE_BYTES);
  uint64_t* empty = full + WP_NS;
  uint64_t* tmem_full = empty + WP_NS;
  uint32_t* tmem_ptr = (uint32_t*)(tmem_full + 1);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const GatherGeom& g = p.g;
  const int Kout = g.Nout, J = g.Kg;
  const uint32_t rank = cluster_ctarank();
  const int j0 = (int)(blockIdx.x >> 1) * 256 + (int)rank * 128;   // this CTA's 128 columns
  const int ko0 = (int)blockIdx.y * 256 + (int)rank * 128;         // ... and its 128 filters
  // A CTA whose 128 filters all lie beyond the last one (the second half of a ragged last tile) still takes part in
  // the pair's protocol, but no box of its loads or stores may lie wholly outside the tensor: it loads the first
  // filters instead and stores nothing.
  const bool rows_live = ko0 < Kout;
  const int ko_load = rows_live ? ko0 : 0;
  const int pbeg = blockIdx.z * p.pix_per_split;
  const int pend = min(g.M, pbeg + p.pix_per_split);
  const int nkb = (pend - pbeg + BK - 1) / BK;

  if (tid == 0) {
    for (int s = 0; s < WP_NS; ++s) {
      mbar_init(smem_u32(&full[s]), 1);
      mbar_init(smem_u32(&empty[s]), 1);
    }
    mbar_init(smem_u32(tmem_full), 1);
    mbar_fence_init();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&tmap_dy);
    tma_prefetch_desc(&tmap_x);
    tma_prefetch_desc(&tmap_out);
  }
  if (warp == 5) {
    tmem_alloc_pair(smem_u32(tmem_ptr), 256);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers and tensor memory exist before anything refers to them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr;
  pdl_enter();

  if (warp == 4) {
    if (lane == 0) {
      // live 64-column blocks of either CTA (a block at or beyond the last column is not loaded)
      auto live_blocks = [&](int jbase) { return jbase >= J ? 0 : (jbase + 64 >= J ? 1 : 2); };
      const int my_live = live_blocks(j0);
      const int pair_j0 = (int)(blockIdx.x >> 1) * 256;
      const uint32_t pair_bytes = 2u * 16384u + (uint32_t)(live_blocks(pair_j0) + live_blocks(pair_j0 + 128)) * 8192u;
      int blk_c[2];
      uint16_t blk_r[2], blk_s[2];
#pragma unroll
      for (int blk = 0; blk < 2; ++blk) {
        const int j = j0 + blk * 64;
        const int tap = j / g.src_c;
        blk_c[blk] = j - tap * g.src_c;
        blk_r[blk] = (uint16_t)(tap / g.S);
        blk_s[blk] = (uint16_t)(tap - (tap / g.S) * g.S);
      }
      const int hw = g.out_h * g.out_w;
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % WP_NS;
        const uint32_t ph = (uint32_t)(kb / WP_NS) & 1u;
        if (!mbar_wait(smem_u32(&empty[s]), ph ^ 1u, p.status, W_TMA_EMPTY)) break;
        const uint32_t lbar = map_to_cta(smem_u32(&full[s]), 0u);
        if (rank == 0) mbar_arrive_expect_tx(smem_u32(&full[s]), pair_bytes);
        const uint32_t dst = smem_u32(base + s * WP_STAGE_BYTES);
        const int pix0 = pbeg + kb * BK;
        tma_load_2d_pair(dst, &tmap_dy, lbar, ko_load, pix0);
        tma_load_2d_pair(dst + 8192u, &tmap_dy, lbar, ko_load + 64 < Kout ? ko_load + 64 : ko_load, pix0);
        const uint32_t dstb = dst + 16384u;
        if (p.b_tma == 1) {
#pragma unroll
          for (int blk = 0; blk < 2; ++blk)
            if (blk < my_live) tma_load_2d_pair(dstb + (uint32_t)blk * 8192u, &tmap_x, lbar, j0 + blk * 64, pix0);
        } else {
          const int n = fastdiv(pix0, hw, p.hw_mul, p.hw_shr);
          const int rem = pix0 - n * hw;
          const int oh = fastdiv(rem, g.out_w, p.w_mul, p.w_shr), ow = rem - oh * g.out_w;
          const int bw = ow * g.stride - g.pad, bh = oh * g.stride - g.pad;
#pragma unroll
          for (int blk = 0; blk < 2; ++blk)
            if (blk < my_live)
              tma_load_im2col_4d_pair(dstb + (uint32_t)blk * 8192u, &tmap_x, lbar, blk_c[blk], bw, bh, n, blk_s[blk], blk_r[blk]);
        }
      }
    }
  } else if (warp == 5) {
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(256, 256, 1, 1);
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % WP_NS;
        const uint32_t ph = (uint32_t)(kb / WP_NS) & 1u;
        if (!mbar_wait_cluster(smem_u32(&full[s]), ph, p.status, W_MMA_FULL)) break;
        tc_fence_after_sync();
        const uint32_t a0 = smem_u32(base + s * WP_STAGE_BYTES);
        const uint32_t b0 = a0 + 16384u;
#pragma unroll
        for (int k = 0; k < BK / 16; ++k) {
          const uint64_t ad = make_smem_desc_sw128(a0 + k * 2048, 8192, 1024);
          const uint64_t bd = make_smem_desc_sw128(b0 + k * 2048, 8192, 1024);
          umma_bf16_pair(tmem_base, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
        }
        umma_commit_pair(smem_u32(&empty[s]), (uint16_t)3);
      }
      umma_commit_pair(smem_u32(tmem_full), (uint16_t)3);
    }
  } else {
    // ---------------- epilogue: this CTA's 128 filter rows x 256 columns, fp32, through shared memory ----------------
    const bool ready = mbar_wait(smem_u32(tmem_full), 0u, p.status, W_EPI_TMEM);
    tc_fence_after_sync();
    // every MMA has completed, so every stage has been consumed: the ring is free for staging
    const int row = warp * 32 + lane;
    const int pair_j0 = (int)(blockIdx.x >> 1) * 256;
#pragma unroll 1
    for (int cb = 0; cb < 8; ++cb) {
      uint32_t acc[32];
      tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(cb * 32), acc);
      tmem_ld_wait();
      uint8_t* stage = base + cb * 16384;  // [128 rows][128 bytes], 16-byte chunks swizzled by the row
#pragma unroll
      for (int v = 0; v < 8; ++v)
        *reinterpret_cast<uint4*>(stage + (uint32_t)row * 128u + (uint32_t)((v ^ (row & 7)) << 4)) =
            make_uint4(acc[v * 4], acc[v * 4 + 1], acc[v * 4 + 2], acc[v * 4 + 3]);
      fence_proxy_async_smem();
      named_bar_sync(1, NPROD);
      if (tid == 0 && ready && rows_live && pair_j0 + cb * 32 < J) {
        tma_store_3d(&tmap_out, smem_u32(stage), pair_j0 + cb * 32, ko0, (int)blockIdx.z);
        bulk_commit_group();
      }
    }
    if (tid == 0) bulk_wait_group_read<0>();
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves while the other may still signal its barriers or read its operands
  if (warp == 5) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, 256);
  }
}

// ------------------------------------------------------------------------------------------
// Persistent fprop/dgrad kernel: one CTA per SM walks the output tiles t = blockIdx.x, +gridDim.x,
// ... (t = m_tile * n_tiles + n_tile). 704 threads:
//   warp 0        TMA producer: B tile every stage, A tile too when it is a plain matrix block
//   warp 1        tensor-memory allocation, tcgen05.mma issue (lane 0)
//   warps 2-3, 20-21   A gather producers (cp.async), idle when A comes by TMA
//   warps 4-19    four epilogue groups of four warps: TMEM -> registers -> (+bias, +addend) -> bf16 -> swizzled
//                 smem -> TMA store, one 64-column slab of a tile at a time, slabs dealt round-robin
// The shared-memory stage ring runs across tile boundaries, and the accumulator is double-buffered
// in tensor memory (2 x BN columns), so the loads of tile i+1 and the MMAs of tile i+1 overlap the
// epilogue of tile i.
//
// PAIR = true runs two CTAs (a cluster of two, on the two SMs of one TPC) as one unit on a 256 x BN tile:
// CTA r of the pair loads rows [128r, 128r+128) of A and filters [BN/2 * r, BN/2 * (r+1)) of B, the
// leader (rank 0) issues tcgen05.mma.cta_group::2 over both CTAs' shared memory, and each CTA finds its 128
// output rows in its own tensor memory and runs its own epilogue. An SM then stages 16 KB + BN x 64 bytes
// per k-block instead of 16 KB + BN x 128 bytes for the same 128 x BN outputs: the L2-to-SM operand stream,
// which bounds these main loops, shrinks by a quarter (BN = 128) to a third (BN = 256), and the smaller stages
// allow a deeper ring. Every load is a plain per-CTA TMA load (none is multicast); what crosses the pair is
// barrier traffic only: both CTAs' loads and gather threads signal the leader's "full" barriers, the MMA's
// commits signal the "empty" and "accumulator ready" barriers of both CTAs, and the peer's epilogue
// releases the accumulator on the leader's barrier.
constexpr int P_THREADS = 704;
constexpr int EPI_GROUPS = 4;            // epilogue warp groups (a power of two)
constexpr int OUT_SLAB_BYTES = BM * 128;  // 128 rows x 64 bf16

struct PersistParams {
  GatherGeom g;
  const bf16* src;
  const float* bias;
  const bf16* addend;
  const uint8_t* addend_bits;  // optional: one bit per element of addend; a cleared bit leaves the element out
  int k_blocks;
  int a_tma;             // how the A operand arrives: 0 gathered with cp.async, 1 plain matrix by TMA, 2 im2col TMA
  int im_lower_w, im_lower_h;  // im2col: base pixel of output position (oh, ow) = (oh, ow) * im_stride + lower
  int im_stride;
  int im_cpt;            // im2col: 64-channel chunks per filter tap (k-block kb = tap * im_cpt + chunk)
  int im_flip;           // im2col: taps run backwards (data gradient)
  int m_tiles, n_tiles;  // 128-row tiles and BN-column tiles of the output
  int gather_lag;        // cp.async groups a gather thread keeps in flight before it hands a stage over (1..NS-2)
  int* status;
  // Optional: per 128-row tile and output column, the sum and the sum of squares of the stored (rounded) values,
  // as double2 [m_tiles][Nout]. The BatchNorm that follows a convolution finalizes its statistics from these and
  // never reads the tensor for them.
  double* col_partial;
};

enum WaitCode2 { W_MMA_TMEM_EMPTY = 5 };

template <int BN, int NS, bool PAIR>
constexpr size_t persist_smem_bytes() {
  return 1024 + (size_t)NS * (A_STAGE_BYTES + (PAIR ? BN / 2 : BN) * BK * 2) + EPI_GROUPS * OUT_SLAB_BYTES + (2 * NS + 2 * EPI_GROUPS + 2) * 8 + 16;
}

// One lane's share of a staged 128 x 64 bf16 slab for the column sums: 32 rows (rp0/rp1 point at the lane's even
// and odd row of the first group of eight, later groups lie 1024 bytes apart) of one column pair, summed and
// square-summed as packed fp32 pairs. MASKED zeroes the rows at and beyond nvalid (the ragged last tile).
template <bool MASKED>
__device__ inline void slab_col_sums(const uint8_t* rp0, const uint8_t* rp1, int rgl, int nvalid, uint64_t& s01,
                                     uint64_t& q01) {
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    uint32_t wv = *reinterpret_cast<const uint32_t*>(((i & 1) ? rp1 : rp0) + (i >> 1) * 1024);
    if (MASKED) {
      const int r = (i >> 1) * 8 + rgl * 2 + (i & 1);
      if (r >= nvalid) wv = 0u;
    }
    uint64_t x01;
    asm("mov.b64 %0, {%1, %2};" : "=l"(x01) : "r"(wv << 16), "r"(wv & 0xffff0000u));
    asm("add.rn.f32x2 %0, %0, %1;" : "+l"(s01) : "l"(x01));
    asm("fma.rn.f32x2 %0, %1, %1, %0;" : "+l"(q01) : "l"(x01));
  }
}

// cp.async.wait_group takes an immediate: wait until at most `lag` of this thread's groups are pending.
__device__ __forceinline__ void cp_async_wait_lag(int lag) {
  switch (lag) {
    case 1: cp_async_wait<1>(); break;
    case 2: cp_async_wait<2>(); break;
    case 3: cp_async_wait<3>(); break;
    default: cp_async_wait<4>(); break;
  }
}

template <int BN, int NS, bool PAIR>
__global__ void __launch_bounds__(P_THREADS, 1)
igemm_fwd_persistent(const PersistParams p, const __grid_constant__ CUtensorMap tmap_b,
                     const __grid_constant__ CUtensorMap tmap_a,
                     const __grid_constant__ CUtensorMap tmap_d) {
  constexpr int B_ROWS = PAIR ? BN / 2 : BN;    // filters this CTA stages per k-block
  constexpr int B_STAGE_BYTES = B_ROWS * BK * 2;
  constexpr int NCTA = PAIR ? 2 : 1;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = base;
  uint8_t* sB = sA + NS * A_STAGE_BYTES;
  uint8_t* sOut = sB + NS * B_STAGE_BYTES;
  uint64_t* full = (uint64_t*)(sOut + EPI_GROUPS * OUT_SLAB_BYTES);
  uint64_t* empty = full + NS;
  uint64_t* acc_ready = empty + NS;      // [EPI_GROUPS][2]: per epilogue group and accumulator buffer, see the MMA branch
  uint64_t* tmem_empty = acc_ready + 2 * EPI_GROUPS;  // [2]: one per accumulator buffer
  uint32_t* tmem_ptr = (uint32_t*)(tmem_empty + 2);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const GatherGeom& g = p.g;
  const int nkb = p.k_blocks;
  if (tid == 0) SRT_STAMP(0);
  // In a pair the unit of work is a 256-row tile; rank r owns its rows 128r..128r+127.
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
  const int unit = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int nunits = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  const int total_tiles = (PAIR ? (p.m_tiles + 1) / 2 : p.m_tiles) * p.n_tiles;

  if (tid == 0) {
    // "full" is waited on by the MMA thread (the leader's, in a pair): one arrival from the TMA thread that
    // announces the bytes, plus one per gather warp of every CTA of the unit when A is gathered (lane 0 arrives
    // for its warp: an arrival on the other CTA's barrier is a remote transaction, and 128 of them per stage
    // cost more than the loads).
    const uint32_t full_count = p.a_tma ? 1u : (uint32_t)(NCTA * (NPROD / 32) + 1);
    for (int s = 0; s < NS; ++s) {
      mbar_init(smem_u32(&full[s]), full_count);
      mbar_init(smem_u32(&empty[s]), 1);
    }
    for (int gi = 0; gi < 2 * EPI_GROUPS; ++gi) mbar_init(smem_u32(&acc_ready[gi]), 1);
    for (int b = 0; b < 2; ++b)
      mbar_init(smem_u32(&tmem_empty[b]), (uint32_t)(NCTA * (NPROD / 32) * (BN / 64)));  // one arrival per warp and slab
    mbar_fence_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_b);
    tma_prefetch_desc(&tmap_d);
    if (p.a_tma) tma_prefetch_desc(&tmap_a);
  }
  if (warp == 1) {
    if (PAIR) {
      tmem_alloc_pair(smem_u32(tmem_ptr), 2 * BN);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(tmem_ptr), 2 * BN);
      tmem_relinquish();
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (PAIR) cluster_sync_all();  // the peer's barriers and tensor memory exist before anything refers to them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr;
  if (tid == 0) SRT_STAMP(1);
  // Everything above touches only shared memory, tensor memory and the kernel parameters, so under an early
  // (programmatic dependent) launch it runs beside the predecessor's tail; global memory is first touched below.
  pdl_enter();
  if (tid == 0) SRT_STAMP(2);

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      // bytes that land on one "full" barrier per stage: from both CTAs of a pair
      const uint32_t bytes = (uint32_t)NCTA * ((uint32_t)B_STAGE_BYTES + (p.a_tma ? (uint32_t)A_STAGE_BYTES : 0u));
      int it = 0;
      bool ok = true;
      for (int t = unit; t < total_tiles && ok; t += nunits) {
        const int m0 = ((t / p.n_tiles) * NCTA + (int)rank) * BM;
        const int n0 = (t % p.n_tiles) * BN + (int)rank * B_ROWS;
        // im2col: the tile's 128 output positions are consecutive base pixels from that of row m0 (the walk wraps
        // rows and images inside the tensor map's bounding box; positions past the last image read as zero). A
        // half-tile without rows (a pair's odd last tile) loads the first tile's pixels, which nobody stores.
        int iw0 = 0, ih0 = 0, in0 = 0, tap_r = 0, tap_s = 0, chunk = 0;
        if (p.a_tma == 2) {
          const RowCoord rc = decode_row(g, m0 < g.M ? m0 : 0);
          iw0 = rc.ow * p.im_stride + p.im_lower_w;
          ih0 = rc.oh * p.im_stride + p.im_lower_h;
          in0 = rc.n;
        }
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % NS;
          const uint32_t ph = (uint32_t)(it / NS) & 1u;
          if (!mbar_wait(smem_u32(&empty[s]), ph ^ 1u, p.status, W_TMA_EMPTY)) { ok = false; break; }
          const uint16_t off_w = (uint16_t)(p.im_flip ? g.S - 1 - tap_s : tap_s);
          const uint16_t off_h = (uint16_t)(p.im_flip ? g.R - 1 - tap_r : tap_r);
          if (PAIR) {
            const uint32_t lbar = map_to_cta(smem_u32(&full[s]), 0u);
            if (rank == 0) mbar_arrive_expect_tx(smem_u32(&full[s]), bytes);
            tma_load_2d_pair(smem_u32(sB + s * B_STAGE_BYTES), &tmap_b, lbar, kb * BK, n0);
            if (p.a_tma == 1) tma_load_2d_pair(smem_u32(sA + s * A_STAGE_BYTES), &tmap_a, lbar, kb * BK, m0);
            else if (p.a_tma == 2)
              tma_load_im2col_4d_pair(smem_u32(sA + s * A_STAGE_BYTES), &tmap_a, lbar, chunk * BK, iw0, ih0, in0, off_w, off_h);
          } else {
            const uint32_t bar = smem_u32(&full[s]);
            mbar_arrive_expect_tx(bar, bytes);
            tma_load_2d(smem_u32(sB + s * B_STAGE_BYTES), &tmap_b, bar, kb * BK, n0);
            if (p.a_tma == 1) tma_load_2d(smem_u32(sA + s * A_STAGE_BYTES), &tmap_a, bar, kb * BK, m0);
            else if (p.a_tma == 2)
              tma_load_im2col_4d(smem_u32(sA + s * A_STAGE_BYTES), &tmap_a, bar, chunk * BK, iw0, ih0, in0, off_w, off_h);
          }
          if (p.a_tma == 2 && ++chunk == p.im_cpt) {
            chunk = 0;
            if (++tap_s == g.S) { tap_s = 0; ++tap_r; }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (the leader's, in a pair) ----------------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM * NCTA, BN, 0, 0);
      int it = 0, tc = 0;
      bool ok = true;
      for (int t = unit; t < total_tiles && ok; t += nunits, ++tc) {
        const int b = tc & 1;
        const uint32_t aph = (uint32_t)(tc >> 1) & 1u;
        const bool got = PAIR ? mbar_wait_cluster(smem_u32(&tmem_empty[b]), aph ^ 1u, p.status, W_MMA_TMEM_EMPTY)
                              : mbar_wait(smem_u32(&tmem_empty[b]), aph ^ 1u, p.status, W_MMA_TMEM_EMPTY);
        if (!got) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t acc = tmem_base + (uint32_t)(b * BN);
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % NS;
          const uint32_t ph = (uint32_t)(it / NS) & 1u;
          const bool fl = PAIR ? mbar_wait_cluster(smem_u32(&full[s]), ph, p.status, W_MMA_FULL)
                               : mbar_wait(smem_u32(&full[s]), ph, p.status, W_MMA_FULL);
          if (!fl) { ok = false; break; }
          if (it == 0) SRT_STAMP(3);
          tc_fence_after_sync();
          const uint32_t a0 = smem_u32(sA + s * A_STAGE_BYTES);
          const uint32_t b0 = smem_u32(sB + s * B_STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t ad = make_smem_desc_sw128(a0 + k * 32, 0, 1024);
            const uint64_t bd = make_smem_desc_sw128(b0 + k * 32, 0, 1024);
            if (PAIR) umma_bf16_pair(acc, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
            else umma_bf16(acc, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          if (PAIR) umma_commit_pair(smem_u32(&empty[s]), (uint16_t)3);
          else umma_commit(smem_u32(&empty[s]));
        }
        // The tile is announced to the epilogue groups that own one of its slabs, each on its own barrier for
        // this accumulator buffer. A parity wait cannot tell phase n from phase n + 2, so a waiter must never
        // fall two completions behind its barrier: with one barrier per buffer polled by every group, a group
        // that owns no slab of a tile (or is still busy with an earlier one) can; with one barrier per group
        // across both buffers, the MMA warp can complete tiles t + 1 and t + 2 while the group still works on
        // tile t. On a barrier of its own per buffer a group sees exactly the tiles it owns there, and the
        // next completion after one it has not consumed needs that very accumulator handed back first.
#pragma unroll
        for (int c = 0; c < BN / 64; ++c) {
          const uint32_t gbar = smem_u32(&acc_ready[2 * ((tc * (BN / 64) + c) & (EPI_GROUPS - 1)) + b]);
          if (PAIR) umma_commit_pair(gbar, (uint16_t)3);
          else umma_commit(gbar);
        }
        SRT_STAMP(4);  // last write wins: the issue of the last tile's last MMA
      }
    }
  } else if (warp >= 4 && warp < 4 + 4 * EPI_GROUPS) {
    // ---------------- epilogue ----------------
    // Four groups of four warps (warps 4-19; the four warps of a group cover the four TMEM lane quarters, which a
    // warp can only read by its index modulo 4). The unit of epilogue work is one 64-column slab of one tile; the
    // slabs are dealt to the groups round-robin across tiles, so a 256-column tile has its four slabs converted
    // side by side and narrower tiles keep groups busy with consecutive tiles (both accumulator buffers are then
    // being read while the MMA warp waits for the first to come back). Each group has its own staging slab,
    // named barrier and store issuer. Per slab a warp waits for tensor memory, converts and stages 32 columns
    // at a time; with one or two such warps per scheduler (the earlier layout) those dependent chains, not the
    // memory system, bounded the epilogue: 2.05 us per slab, 4.1 us per 128 x 256 tile, a third of a
    // layer-3 reduce convolution and most of an expand one.
    constexpr int NSLAB = BN / 64;
    const int grp = (warp - 4) >> 2;
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    const int row = q * 32 + lane;          // row of the tile held by this thread
    const int et = ((warp - 4) & 3) * 32 + lane;  // 0..127 within the group
    const bool issuer = et == 0;
    const uint32_t swz_row = (uint32_t)row * 128u;
    uint8_t* stage = sOut + grp * OUT_SLAB_BYTES;
    const uint32_t bar_id = 1u + (uint32_t)grp;
    int tc = 0;
    uint32_t owned[2] = {0u, 0u};  // tiles of this group seen so far, per accumulator buffer
    bool ok = true;
    for (int t = unit; t < total_tiles; t += nunits, ++tc) {
      // the slab of this tile that falls to this group, if any (at most one: a tile has at most EPI_GROUPS slabs)
      const int c = (grp - tc * NSLAB) & (EPI_GROUPS - 1);
      if (c >= NSLAB) continue;
      const int m_tile = (t / p.n_tiles) * NCTA + (int)rank;
      const int m0 = m_tile * BM, n0 = (t % p.n_tiles) * BN;
      const int b = tc & 1;
      if (ok) ok = mbar_wait(smem_u32(&acc_ready[2 * grp + b]), owned[b] & 1u, p.status, W_EPI_TMEM);
      ++owned[b];
      if (issuer && grp == 0) SRT_STAMP(5);  // last write wins: the last tile's accumulator is complete
      tc_fence_after_sync();
      const int m = m0 + row;
      const bool tile_live = m0 < g.M;  // false only for the second half of a pair's last, odd row tile
      {
        const int col0 = n0 + c * 64;
        const bool live = tile_live && col0 < g.Nout;  // uniform across the group
        if (live) {
          // the store that read this group's staging slab last must be done with it
          if (issuer) bulk_wait_group_read<0>();
          named_bar_sync(bar_id, NPROD);
        }
        // the addend's mask bits of this thread's 64 columns: one 8-byte load when rows are whole 8-byte groups
        uint2 abits = make_uint2(0u, 0u);
        const bool abits_wide = p.addend_bits != nullptr && (g.Nout & 63) == 0;
        if (abits_wide && live && m < g.M)
          abits = *reinterpret_cast<const uint2*>(p.addend_bits + (((size_t)m * g.Nout + col0) >> 3));
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t acc[32];
          if (live) {
            tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * BN + c * 64 + h * 32), acc);
            tmem_ld_wait();
            if (issuer && grp == 0) SRT_STAMP(10 + h);
          }
          if (h == 1) {
            // this slab has been read: one arrival per warp and slab hands the accumulator back to the MMA warp
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
              if (PAIR) mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty[b]), 0u));
              else mbar_arrive(smem_u32(&tmem_empty[b]));
            }
          }
          if (!live) continue;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const int col = col0 + h * 32 + v * 8;
            float f[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(acc[v * 8 + e]);
            if (col < g.Nout) {
              if (p.bias) {
#pragma unroll
                for (int e = 0; e < 8; ++e) f[e] += p.bias[col + e];
              }
              if (p.addend && m < g.M) {
                Vec16<bf16> av;
                av.load(p.addend + (size_t)m * g.Nout + col);
                float af[8];
                av.unpack(af);
                if (p.addend_bits) {
                  const unsigned bits = abits_wide ? ((h ? abits.y : abits.x) >> (v * 8))
                                                   : (unsigned)p.addend_bits[((size_t)m * g.Nout + col) >> 3];
#pragma unroll
                  for (int e = 0; e < 8; ++e) af[e] = ((bits >> e) & 1u) ? af[e] : 0.f;
                }
#pragma unroll
                for (int e = 0; e < 8; ++e) f[e] += af[e];
              }
            }
            Vec16<bf16> ov;
            ov.pack(f);
            const int chunk = h * 4 + v;
            *reinterpret_cast<uint4*>(stage + swz_row + (uint32_t)((chunk ^ (row & 7)) << 4)) = ov.raw;
          }
        }
        if (live) {
          if (issuer && grp == 0) SRT_STAMP(12);
          fence_proxy_async_smem();
          if (issuer && grp == 0) SRT_STAMP(13);
          named_bar_sync(bar_id, NPROD);
          if (issuer) {
            tma_store_2d(&tmap_d, smem_u32(stage), col0, m0);
            bulk_commit_group();
          }
          if (issuer && grp == 0) SRT_STAMP(14);
          if (p.col_partial != nullptr) {
            // Column sums of the slab as it sits in the staging buffer. Warp w of the group takes columns
            // 16w..16w+15; a lane owns one column pair and a quarter of the rows, picked so that the 32 words
            // a warp reads at once fall into 32 different banks of the swizzled slab (the four row classes
            // differ in bits 1-2 of the row, which the swizzle turns into different 16-byte chunks).
            const int wg = et >> 5, cpl = lane & 7, rgl = lane >> 3;
            const int cp = wg * 8 + cpl;
            const uint32_t chunk = (uint32_t)(cp >> 2), within = (uint32_t)(cp & 3) * 4u;
            const int nvalid = g.M - m0;  // rows of this tile that exist
            // both columns of the pair ride in one packed fp32x2 add and one packed fma per row
            uint64_t s01 = 0ull, q01 = 0ull;
            const uint8_t* rp0 = stage + (uint32_t)(rgl * 2) * 128u + ((chunk ^ (uint32_t)(rgl * 2)) << 4) + within;
            const uint8_t* rp1 = stage + (uint32_t)(rgl * 2 + 1) * 128u + ((chunk ^ (uint32_t)(rgl * 2 + 1)) << 4) + within;
            if (nvalid >= BM) slab_col_sums<false>(rp0, rp1, rgl, nvalid, s01, q01);  // every tile but the last
            else slab_col_sums<true>(rp0, rp1, rgl, nvalid, s01, q01);
            float s0, s1, q0, q1;
            {
              uint32_t a, b2, c2, d;
              asm("mov.b64 {%0, %1}, %2;" : "=r"(a), "=r"(b2) : "l"(s01));
              asm("mov.b64 {%0, %1}, %2;" : "=r"(c2), "=r"(d) : "l"(q01));
              s0 = __uint_as_float(a); s1 = __uint_as_float(b2);
              q0 = __uint_as_float(c2); q1 = __uint_as_float(d);
            }
#pragma unroll
            for (int o = 8; o <= 16; o <<= 1) {
              s0 += __shfl_xor_sync(0xffffffffu, s0, o);
              s1 += __shfl_xor_sync(0xffffffffu, s1, o);
              q0 += __shfl_xor_sync(0xffffffffu, q0, o);
              q1 += __shfl_xor_sync(0xffffffffu, q1, o);
            }
            const int col = col0 + 2 * cp;
            if (rgl == 0 && col < g.Nout) {
              double2* out = reinterpret_cast<double2*>(p.col_partial) + (size_t)m_tile * g.Nout + col;
              out[0] = make_double2((double)s0, (double)q0);
              out[1] = make_double2((double)s1, (double)q1);
            }
            if (issuer && grp == 0) SRT_STAMP(15);
          }
        }
      }
    }
    if (issuer && grp == 0) SRT_STAMP(6);
    // the staging slab must outlive the last store's read of it; the data reaches memory before the grid ends
    if (issuer) bulk_wait_group_read<0>();
    if (issuer && grp == 0) SRT_STAMP(7);
  } else {
    // ---------------- A gather producers ----------------
    if (!p.a_tma) {
      const int pt = (warp < 4 ? warp - 2 : warp - 18) * 32 + lane;  // 0..127 over warps 2, 3, 20, 21
      const int j = pt & 7, r0 = pt >> 3;
      const int PLAG = p.gather_lag;
      const uint32_t swz = (uint32_t)((j ^ (r0 & 7)) << 4);
      int it = 0;
      bool ok = true;
      // A stage is complete when every gather warp of the unit has arrived on the MMA thread's barrier. Each
      // thread has waited for its own copies and fenced them towards the async proxy before the warp meets.
      auto stage_done = [&](int k) {
        __syncwarp();
        if (lane == 0) {
          if (PAIR) mbar_arrive_cluster(map_to_cta(smem_u32(&full[k % NS]), 0u));
          else mbar_arrive(smem_u32(&full[k % NS]));
        }
      };
      // A thread copies the same 16-byte chunk j of every row, so within a k-block it stays inside one filter tap when
      // the channel count is a multiple of BK (one tap per k-block) or divides BK (several taps per k-block, one per
      // chunk: the 8-channel stem). Without a dgrad stride the source pixel of a row is then its tap-(0,0) pixel plus
      // a per-thread, per-k-block offset: one element offset per row and tile, one per k-block, an add, two unsigned
      // bounds checks and a select per copy, no division in the loop. Everything else (channel counts like 24, strided
      // dgrad) takes the general loop below.
      const bool fast = ((g.src_c % BK) == 0 || (BK % g.src_c) == 0) && (!g.dgrad || g.stride == 1);
      if (fast) {
        const int sgn = g.dgrad ? -1 : 1;
        for (int t = unit; t < total_tiles && ok; t += nunits) {
          const int m0 = ((t / p.n_tiles) * NCTA + (int)rank) * BM;
          int rowoff[8], ih0[8], iw0[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int m = m0 + r0 + 16 * i;
            if (m < g.M) {
              RowCoord rc = decode_row(g, m);
              ih0[i] = g.dgrad ? rc.oh + g.pad : rc.oh * g.stride - g.pad;
              iw0[i] = g.dgrad ? rc.ow + g.pad : rc.ow * g.stride - g.pad;
              rowoff[i] = ((rc.n * g.src_h + ih0[i]) * g.src_w + iw0[i]) * g.src_c;
            } else {
              ih0[i] = -(1 << 20);
              iw0[i] = 0;
              rowoff[i] = 0;
            }
          }
          // filter tap and first channel of this thread's chunk in the k-block (taps beyond the filter: zero rows of
          // the padded reduction)
          int c0 = j * 8, r = 0, sf = 0;
          while (c0 >= g.src_c) {
            c0 -= g.src_c;
            if (++sf == g.S) { sf = 0; ++r; }
          }
          for (int kb = 0; kb < nkb; ++kb, ++it) {
            const int s = it % NS;
            const uint32_t ph = (uint32_t)(it / NS) & 1u;
            // warp-uniform outcome: the warp leaves the loop together (its lanes meet in stage_done)
            if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&empty[s]), ph ^ 1u, p.status, W_PROD_EMPTY))) { ok = false; break; }
            const int dr = sgn * r, ds = sgn * sf;
            const int tapoff = (dr * g.src_w + ds) * g.src_c + c0;
            const bool tap_ok = r < g.R;
            const uint32_t dst0 = smem_u32(sA + s * A_STAGE_BYTES) + (uint32_t)r0 * 128u + swz;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const bool v = tap_ok && (unsigned)(ih0[i] + dr) < (unsigned)g.src_h && (unsigned)(iw0[i] + ds) < (unsigned)g.src_w;
              const int off = v ? rowoff[i] + tapoff : 0;
              cp_async_16(dst0 + (uint32_t)i * (16u * 128u), p.src + off, v ? 16u : 0u);
            }
            cp_async_commit();
            if (it >= PLAG) {
              cp_async_wait_lag(PLAG);
              fence_proxy_async_smem();
              stage_done(it - PLAG);
            }
            c0 += BK;
            while (c0 >= g.src_c) {
              c0 -= g.src_c;
              if (++sf == g.S) { sf = 0; ++r; }
            }
          }
        }
      }
      for (int t = unit; !fast && t < total_tiles && ok; t += nunits) {
        const int m0 = ((t / p.n_tiles) * NCTA + (int)rank) * BM;
        int pixb[8], ih0[8], iw0[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int m = m0 + r0 + 16 * i;
          if (m < g.M) {
            RowCoord rc = decode_row(g, m);
            pixb[i] = rc.n * g.src_h * g.src_w;
            ih0[i] = g.dgrad ? rc.oh + g.pad : rc.oh * g.stride - g.pad;
            iw0[i] = g.dgrad ? rc.ow + g.pad : rc.ow * g.stride - g.pad;
          } else {
            pixb[i] = 0;
            ih0[i] = -(1 << 20);
            iw0[i] = 0;
          }
        }
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % NS;
          const uint32_t ph = (uint32_t)(it / NS) & 1u;
          if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&empty[s]), ph ^ 1u, p.status, W_PROD_EMPTY))) { ok = false; break; }
          const int kk = kb * BK + j * 8;
          const bool k_ok = kk < g.Kg;
          const int tap = kk / g.src_c, c = kk - tap * g.src_c;
          const int r = tap / g.S, sf = tap - r * g.S;
          const uint32_t dst0 = smem_u32(sA + s * A_STAGE_BYTES) + (uint32_t)r0 * 128u + swz;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            int ih, iw;
            bool v = k_ok;
            if (!g.dgrad) {
              ih = ih0[i] + r;
              iw = iw0[i] + sf;
            } else {
              const int th = ih0[i] - r, tw = iw0[i] - sf;
              v = v && th >= 0 && tw >= 0;
              if (g.stride > 1) {
                v = v && (th % g.stride == 0) && (tw % g.stride == 0);
                ih = th / g.stride;
                iw = tw / g.stride;
              } else {
                ih = th;
                iw = tw;
              }
            }
            v = v && ih >= 0 && iw >= 0 && ih < g.src_h && iw < g.src_w;
            const bf16* ptr = v ? p.src + ((size_t)(pixb[i] + ih * g.src_w + iw) * g.src_c + c) : p.src;
            cp_async_16(dst0 + (uint32_t)i * (16u * 128u), ptr, v ? 16u : 0u);
          }
          cp_async_commit();
          if (it >= PLAG) {
            cp_async_wait_lag(PLAG);
            fence_proxy_async_smem();
            stage_done(it - PLAG);
          }
        }
      }
      // drain: every stage issued but not yet handed over
      cp_async_wait<0>();
      fence_proxy_async_smem();
      for (int k = it > PLAG ? it - PLAG : 0; k < it; ++k) stage_done(k);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0) SRT_STAMP(8);
  // Neither CTA of a pair may retire while the other can still signal its barriers or have its shared and
  // tensor memory read by an MMA in flight.
  if (PAIR) cluster_sync_all();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    if (PAIR) tmem_dealloc_pair(tmem_base, 2 * BN);
    else tmem_dealloc(tmem_base, 2 * BN);
    if (lane == 0) SRT_STAMP(9);
  }
}

// ------------------------------------------------------------------------------------------
// Batched GEMM for attention: D[z][m][n] = alpha * sum_k A[z][m][k] * B[z][n][k], bf16 in, fp32
// accumulate, bf16 out. z = (z1, z2) with independent strides per operand, so the heads of a fused
// [tokens][3*hidden] projection are addressed in place through 4-D tensor maps (k, row, z1, z2).
// One 128 x BN tile per CTA; warps 0-3 epilogue, warp 4 TMA, warp 5 MMA. `causal` skips tiles that
// lie wholly above the diagonal (n > m); `k_causal` trims the reduction range of a tile when the
// A operand is known to be zero beyond (1: k > m) or before (2: k < m) the diagonal.
struct BgemmParams {
  bf16* D;
  int M, N, k_blocks;
  int Z1, b_div;  // b_div: the B operand's first batch coordinate is z1 / b_div (grouped KV heads)
  long long ldd, d_s1, d_s2;
  float alpha;
  int causal, k_causal;
  int* status;
};

template <int BN, int NS>
__global__ void __launch_bounds__(NTHREADS)
bgemm_kernel(const BgemmParams p, const __grid_constant__ CUtensorMap tmap_a,
             const __grid_constant__ CUtensorMap tmap_b) {
  constexpr int B_STAGE_BYTES = BN * BK * 2;
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
  if (p.causal && n0 >= m0 + BM) return;  // wholly above the diagonal: never read by the consumer
  extern __shared__ uint8_t smem_raw[];
  SmemLayout sm = carve_smem<NS, B_STAGE_BYTES>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int z1 = blockIdx.z % p.Z1, z2 = blockIdx.z / p.Z1;
  int kb0 = 0, kb1 = p.k_blocks;
  if (p.k_causal == 1) { const int lim = (m0 + BM + BK - 1) / BK; kb1 = kb1 < lim ? kb1 : lim; }
  if (p.k_causal == 2) kb0 = m0 / BK < kb1 ? m0 / BK : kb1;
  const int nkb = kb1 - kb0;

  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(smem_u32(&sm.full[s]), 1);
      mbar_init(smem_u32(&sm.empty[s]), 1);
    }
    mbar_init(smem_u32(sm.tmem_full), 1);
    mbar_fence_init();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 5) {
    tmem_alloc(smem_u32(sm.tmem_ptr), BN);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *sm.tmem_ptr;
  // Everything above touches only shared memory, tensor memory and the kernel parameters, so under an early
  // (programmatic dependent) launch it runs beside the predecessor's tail; global memory is first touched below.
  pdl_enter();

  if (warp < 4) {
    bool ready = true;
    if (nkb > 0) {
      ready = mbar_wait(smem_u32(sm.tmem_full), 0u, p.status, W_EPI_TMEM);
      tc_fence_after_sync();
    }
    const int m = m0 + warp * 32 + lane;
    bf16* drow = p.D + (long long)z1 * p.d_s1 + (long long)z2 * p.d_s2 + (long long)m * p.ldd;
#pragma unroll 1
    for (int cb = 0; cb < BN / 32; ++cb) {
      uint32_t acc[32];
      if (nkb > 0) {
        tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(cb * 32), acc);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int e = 0; e < 32; ++e) acc[e] = 0u;
      }
      if (ready && m < p.M) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const int col = n0 + cb * 32 + v * 8;
          if (col < p.N) {
            float f[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(acc[v * 8 + e]) * p.alpha;
            Vec16<bf16> ov;
            ov.pack(f);
            ov.store(drow + col);
          }
        }
      }
    }
  } else if (warp == 4) {
    if (lane == 0) {
      for (int i = 0; i < nkb; ++i) {
        const int s = i % NS;
        const uint32_t ph = (uint32_t)(i / NS) & 1u;
        if (!mbar_wait(smem_u32(&sm.empty[s]), ph ^ 1u, p.status, W_TMA_EMPTY)) break;
        const uint32_t bar = smem_u32(&sm.full[s]);
        mbar_arrive_expect_tx(bar, (uint32_t)(A_STAGE_BYTES + B_STAGE_BYTES));
        tma_load_4d(smem_u32(sm.a + s * A_STAGE_BYTES), &tmap_a, bar, (kb0 + i) * BK, m0, z1, z2);
        tma_load_4d(smem_u32(sm.b + s * B_STAGE_BYTES), &tmap_b, bar, (kb0 + i) * BK, n0, z1 / p.b_div, z2);
      }
    }
  } else {
    if (lane == 0 && nkb > 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, 0, 0);
      bool ok = true;
      for (int i = 0; i < nkb && ok; ++i) {
        const int s = i % NS;
        const uint32_t ph = (uint32_t)(i / NS) & 1u;
        if (!mbar_wait(smem_u32(&sm.full[s]), ph, p.status, W_MMA_FULL)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t a0 = smem_u32(sm.a + s * A_STAGE_BYTES);
        const uint32_t b0 = smem_u32(sm.b + s * B_STAGE_BYTES);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k) {
          const uint64_t ad = make_smem_desc_sw128(a0 + k * 32, 0, 1024);
          const uint64_t bd = make_smem_desc_sw128(b0 + k * 32, 0, 1024);
          umma_bf16(tmem_base, ad, bd, idesc, (i | k) != 0 ? 1u : 0u);
        }
        umma_commit(smem_u32(&sm.empty[s]));
      }
      umma_commit(smem_u32(sm.tmem_full));
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 5) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, BN);
  }
}

// ---- host side ------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)sym;
  });
  return fn;
}

typedef CUresult (*EncodeIm2colFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const int*, const int*, cuuint32_t, cuuint32_t,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeIm2colFn get_encode_im2col_fn() {
  static EncodeIm2colFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (EncodeIm2colFn)sym;
  });
  return fn;
}

// The corners of the im2col bounding box (the range of base pixels) for a gather geometry: a convolution reads
// output position o at o * stride - pad + tap, a stride-1 data gradient at o - (R - 1 - pad) + (R - 1 - tap).
struct Im2colBox {
  int lower_w, lower_h, upper_w, upper_h, stride;
};
inline Im2colBox im2col_box(const GatherGeom& g) {
  Im2colBox b;
  if (!g.dgrad) {
    b.lower_w = -g.pad; b.lower_h = -g.pad;
    b.upper_w = g.pad - (g.S - 1); b.upper_h = g.pad - (g.R - 1);
    b.stride = g.stride;
  } else {
    b.lower_w = -(g.S - 1 - g.pad); b.lower_h = -(g.R - 1 - g.pad);
    b.upper_w = -g.pad; b.upper_h = -g.pad;
    b.stride = 1;
  }
  return b;
}
// Whether the source of a gather geometry can be fetched by im2col TMA loads of 64-channel chunks: a k-block must
// not straddle a filter tap, a strided data gradient has holes no box describes, and the corner fields are 8 bits.
bool im2col_ok(const GatherGeom& g) {
  if (g.src_c % 64 != 0 || (g.dgrad && g.stride != 1) || g.stride > 8) return false;
  if (g.pad > g.R - 1 || g.pad > g.S - 1 || g.R > 16 || g.S > 16) return false;
  const Im2colBox b = im2col_box(g);
  // the bounding box must hold exactly out_w x out_h base pixels per image
  const int cw = (g.src_w - 1 + b.upper_w - b.lower_w) / b.stride + 1, ch = (g.src_h - 1 + b.upper_h - b.lower_h) / b.stride + 1;
  return cw == g.out_w && ch == g.out_h && g.src_w + b.upper_w - b.lower_w > 0 && g.src_h + b.upper_h - b.lower_h > 0;
}

// NHWC bf16 tensor [n][h][w][c] for im2col loads of `pixels` base pixels x 64 channels, 128B swizzle.
int make_tmap_im2col(CUtensorMap* tm, const void* base, const GatherGeom& g, uint32_t pixels) {
  EncodeIm2colFn fn = get_encode_im2col_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeIm2col is not available from the CUDA driver");
    return SRT_ERR_CUDA;
  }
  SRT_REQUIRE(((uintptr_t)base & 15) == 0 && g.src_c % 64 == 0, "im2col TMA operand must be 16-byte aligned with 64-channel chunks");
  const Im2colBox b = im2col_box(g);
  cuuint64_t dims[4] = {(cuuint64_t)g.src_c, (cuuint64_t)g.src_w, (cuuint64_t)g.src_h, (cuuint64_t)g.n_img};
  cuuint64_t strides[3] = {(cuuint64_t)g.src_c * 2, (cuuint64_t)g.src_w * g.src_c * 2,
                           (cuuint64_t)g.src_h * g.src_w * g.src_c * 2};
  int lower[2] = {b.lower_w, b.lower_h};
  int upper[2] = {b.upper_w, b.upper_h};
  cuuint32_t estr[4] = {1, (cuuint32_t)b.stride, (cuuint32_t)b.stride, 1};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, lower, upper, 64,
                  pixels, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeIm2col failed with CUresult %d", (int)r);
    return SRT_ERR_CUDA;
  }
  return SRT_OK;
}

// 2-D bf16 row-major matrix [rows][cols] (cols contiguous), box = 64 cols x box_rows, 128B swizzle.
int make_tmap_2d(CUtensorMap* tm, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from the CUDA driver");
    return SRT_ERR_CUDA;
  }
  SRT_REQUIRE(((uintptr_t)base & 15) == 0 && (cols * 2) % 16 == 0,
              "TMA operand must be 16-byte aligned with a 16-byte multiple row pitch");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return SRT_ERR_CUDA;
  }
  return SRT_OK;
}

// Output matrix [rows][cols] bf16 for TMA stores: box = 64 cols x 128 rows, 128B swizzle.
int make_tmap_store(CUtensorMap* tm, void* base, uint64_t rows, uint64_t cols) {
  return make_tmap_2d(tm, base, rows, cols, 128);
}

int* status_ptr() {
  static int* ptr = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_tc_status) == cudaSuccess) ptr = (int*)p;
  });
  return ptr;
}

template <int BN, int NS>
int launch_wgrad(const WgradParams& p, const CUtensorMap& tdy, const CUtensorMap& tx, int splits,
                 cudaStream_t st) {
  constexpr size_t smem = smem_bytes<NS, BN * BK * 2>();
  static bool configured = false;
  if (!configured) {
    SRT_CHECK_CUDA(cudaFuncSetAttribute(igemm_wgrad_kernel<BN, NS>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  dim3 grid(ceil_div(p.g.Kg, BN), ceil_div(p.g.Nout, BM), splits);
  launch_pdl_if(pdl_big_kernels() && (pdl_classes() & PDL_GEMM) != 0, igemm_wgrad_kernel<BN, NS>, dim3(grid), dim3(NTHREADS), smem, st, p, tdy, tx);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}

// fp32 partial sums [splits][filters][columns] for TMA stores of 128 rows x 32 columns, 128B swizzle.
int make_tmap_wgrad_out(CUtensorMap* tm, float* base, uint64_t J, uint64_t Kout, uint64_t splits) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from the CUDA driver");
    return SRT_ERR_CUDA;
  }
  SRT_REQUIRE(((uintptr_t)base & 15) == 0 && (J * 4) % 16 == 0, "wgrad output must be 16-byte aligned with a 16-byte multiple row pitch");
  cuuint64_t dims[3] = {J, Kout, splits};
  cuuint64_t strides[2] = {J * 4, Kout * J * 4};
  cuuint32_t box[3] = {32, 128, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled (wgrad output) failed with CUresult %d", (int)r);
    return SRT_ERR_CUDA;
  }
  return SRT_OK;
}

int launch_wgrad_pair(const WgradParams& p, const CUtensorMap& tdy, const CUtensorMap& tx, const CUtensorMap& tout,
                      int splits, cudaStream_t st) {
  constexpr size_t smem = wgrad_pair_smem_bytes();
  static_assert(smem <= 232448, "pair wgrad: shared memory budget exceeded");
  static bool configured = false;
  if (!configured) {
    SRT_CHECK_CUDA(cudaFuncSetAttribute(igemm_wgrad_pair, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * ceil_div(p.g.Kg, 256), ceil_div(p.g.Nout, 256), splits);
  cfg.blockDim = dim3(NTHREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = (pdl_big_kernels() && (pdl_classes() & PDL_GEMM) != 0) ? 1 : 0;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = 2;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  SRT_CHECK_CUDA(cudaLaunchKernelEx(&cfg, igemm_wgrad_pair, p, tdy, tx, tout));
  return SRT_OK;
}

template <int BN, int NS, bool PAIR>
int launch_persistent(const PersistParams& p, const CUtensorMap& tb, const CUtensorMap& ta,
                      const CUtensorMap& td, cudaStream_t st) {
  constexpr size_t smem = persist_smem_bytes<BN, NS, PAIR>();
  static_assert(smem <= 232448, "persistent igemm: shared memory budget exceeded");
  static bool configured = false;
  if (!configured) {
    SRT_CHECK_CUDA(cudaFuncSetAttribute(igemm_fwd_persistent<BN, NS, PAIR>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  const bool early = pdl_big_kernels() && (pdl_classes() & PDL_GEMM) != 0;
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(P_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = early ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (PAIR) {
    // one unit = two CTAs on the two SMs of a TPC, working on a 256-row tile
    const int units = ceil_div(p.m_tiles, 2) * p.n_tiles;
    const int room = sm_count() / 2;
    cfg.gridDim = dim3(2 * (units < room ? units : room));
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 2;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.numAttrs = 2;
  } else {
    const int tiles = p.m_tiles * p.n_tiles;
    cfg.gridDim = dim3(tiles < sm_count() ? tiles : sm_count());
  }
  cudaLaunchKernelEx(&cfg, igemm_fwd_persistent<BN, NS, PAIR>, p, tb, ta, td);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}

// Tile width: fewest (waves x bytes staged per k-block), the quantity that bounds an L2-fed main loop.
int pick_bn(int M, int N, int forced) {
  if (forced == 64 || forced == 128 || forced == 256) return forced;
  const int mt = ceil_div(M, BM), sms = sm_count();
  int best = 64;
  double best_cost = 1e30;
  for (int bn : {64, 128, 256}) {
    if (bn > 64 && bn / 2 >= N) continue;  // wider than the matrix: wasted columns
    const int tiles = mt * ceil_div(N, bn);
    const int waves = ceil_div(tiles, sms);
    const double cost = (double)waves * (16.0 + bn / 8.0);
    if (cost < best_cost - 1e-9) { best_cost = cost; best = bn; }
  }
  return best;
}

struct WgradPlan {
  int bn, splits, pix_per_split;
  int b_tma;  // how X arrives: 0 gathered, 1 plain matrix by TMA, 2 im2col TMA
  bool pair;  // 256 x 256 tiles on CTA pairs
};

static int g_wgrad_pair = getenv("SIRIUS_B200_WGRAD_PAIR") ? atoi(getenv("SIRIUS_B200_WGRAD_PAIR")) : 1;

// sizing = true asks what the plan would be with every process-wide switch (pair kernel, plan override, im2col) in
// the position that allows the pair kernel: scratch sized from it stays large enough whichever way they are set later.
WgradPlan plan_wgrad(const GatherGeom& g, bool allow_pair = true, bool sizing = false) {
  WgradPlan w;
  const bool plain = g.R == 1 && g.S == 1 && g.stride == 1 && g.pad == 0;
  w.b_tma = g_force_gather ? 0 : plain ? 1 : (im2col_ok(g) && g_im2col_enabled) ? 2 : 0;
  const bool by_tma = sizing ? (plain || im2col_ok(g)) : w.b_tma != 0;
  const bool switched_on = sizing || (g_wgrad_pair && g_force_pair != 0);
  // CTA pairs where both operands come by TMA and the tile is not mostly padding: at least 256 filters (ragged
  // beyond that is fine) and 192 columns
  w.pair = allow_pair && switched_on && by_tma && g.Nout >= 256 && g.Kg >= 192 && g.src_c % 64 == 0 && sm_count() >= 2;
  // ... and only grids of a single wave (every pair resident at once). A grid of several waves of clusters on the
  // low-priority stream, beside the main stream's kernels, stopped making progress in about one process out of
  // three (GPT-2's tied embedding, 591 tiles); the cause was not found by reading, single-wave grids ran 10^4 steps
  // without it, so larger problems stay on the single-CTA kernel.
  if (w.pair && ceil_div(g.Kg, 256) * ceil_div(g.Nout, 256) > sm_count() / 2) w.pair = false;
  if (w.pair) {
    w.bn = 256;
    const int tiles = ceil_div(g.Kg, 256) * ceil_div(g.Nout, 256);
    int want = (sm_count() / 2) / tiles;
    const int max_by_pix = ceil_div(g.M, 4 * BK);
    int splits = want < max_by_pix ? want : max_by_pix;
    if (splits < 1) splits = 1;
    if (splits > 128) splits = 128;
    w.pix_per_split = ceil_div(ceil_div(g.M, splits), BK) * BK;
    w.splits = ceil_div(g.M, w.pix_per_split);
    return w;
  }
  w.bn = g.Kg <= 64 ? 64 : 128;
  // as many splits as fit the machine in one wave (two CTAs per SM), never less than 4 k-blocks each
  const int tiles = ceil_div(g.Kg, w.bn) * ceil_div(g.Nout, BM);
  int want = (2 * sm_count()) / tiles;
  const int max_by_pix = ceil_div(g.M, 4 * BK);
  int splits = want < max_by_pix ? want : max_by_pix;
  if (splits < 1) splits = 1;
  if (splits > 128) splits = 128;
  w.pix_per_split = ceil_div(ceil_div(g.M, splits), BK) * BK;
  w.splits = ceil_div(g.M, w.pix_per_split);
  return w;
}

// 4-D bf16 operand (k contiguous, then rows, then two batch dimensions), box = 64 x box_rows x 1 x 1.
int make_tmap_4d(CUtensorMap* tm, const void* base, uint64_t kdim, uint64_t rows, uint64_t z1, uint64_t z2,
                 uint64_t ld, uint64_t s1, uint64_t s2, uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from the CUDA driver");
    return SRT_ERR_CUDA;
  }
  SRT_REQUIRE(((uintptr_t)base & 15) == 0 && ld % 8 == 0 && s1 % 8 == 0 && s2 % 8 == 0,
              "batched GEMM operand: base and strides must be 16-byte multiples");
  cuuint64_t dims[4] = {kdim, rows, z1, z2};
  cuuint64_t strides[3] = {ld * 2, (z1 > 1 ? s1 : ld * rows) * 2, (z2 > 1 ? s2 : ld * rows) * 2};
  cuuint32_t box[4] = {64, box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled (4-D) failed with CUresult %d", (int)r);
    return SRT_ERR_CUDA;
  }
  return SRT_OK;
}

template <int BN, int NS>
int launch_bgemm(const BgemmParams& p, const CUtensorMap& ta, const CUtensorMap& tb, int zs, cudaStream_t st) {
  constexpr size_t smem = smem_bytes<NS, BN * BK * 2>();
  static bool configured = false;
  if (!configured) {
    SRT_CHECK_CUDA(cudaFuncSetAttribute(bgemm_kernel<BN, NS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  dim3 grid(ceil_div(p.M, BM), ceil_div(p.N, BN), zs);
  launch_pdl_if(pdl_big_kernels() && (pdl_classes() & PDL_GEMM) != 0, bgemm_kernel<BN, NS>, grid, dim3(NTHREADS), smem, st,
                p, ta, tb);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}

}  // namespace

int bgemm_bf16(const BgemmDesc& d, const void* A, const void* B, void* D, cudaStream_t st) {
  SRT_REQUIRE(d.M > 0 && d.N > 0 && d.K > 0 && d.Z1 > 0 && d.Z2 > 0, "bgemm: empty problem");
  SRT_REQUIRE(d.K % 8 == 0 && d.N % 8 == 0 && d.ldd % 8 == 0 && d.d_s1 % 8 == 0 && d.d_s2 % 8 == 0 &&
                  ((uintptr_t)D & 15) == 0,
              "bgemm: K, N and the output strides must be multiples of 8 elements");
  SRT_REQUIRE((long long)d.Z1 * d.Z2 <= 65535, "bgemm: more than 65535 batch entries");
  BgemmParams p;
  p.D = (bf16*)D;
  p.M = d.M; p.N = d.N; p.k_blocks = ceil_div(d.K, BK);
  p.Z1 = d.Z1;
  p.b_div = d.b_div > 1 ? d.b_div : 1;
  SRT_REQUIRE(d.Z1 % p.b_div == 0, "bgemm: Z1 must be a multiple of b_div");
  p.ldd = d.ldd; p.d_s1 = d.d_s1; p.d_s2 = d.d_s2;
  p.alpha = d.alpha;
  p.causal = d.causal; p.k_causal = d.k_causal;
  p.status = status_ptr();
  SRT_REQUIRE(p.status != nullptr, "tcgen05 status word unavailable");
  const int bn = d.N <= 64 ? 64 : 128;
  CUtensorMap ta, tb;
  int rc = make_tmap_4d(&ta, A, (uint64_t)d.K, (uint64_t)d.M, (uint64_t)d.Z1, (uint64_t)d.Z2, (uint64_t)d.lda,
                        (uint64_t)d.a_s1, (uint64_t)d.a_s2, (uint32_t)BM);
  if (rc) return rc;
  rc = make_tmap_4d(&tb, B, (uint64_t)d.K, (uint64_t)d.N, (uint64_t)(d.Z1 / p.b_div), (uint64_t)d.Z2, (uint64_t)d.ldb,
                    (uint64_t)d.b_s1, (uint64_t)d.b_s2, (uint32_t)bn);
  if (rc) return rc;
  if (bn == 64) return launch_bgemm<64, 4>(p, ta, tb, d.Z1 * d.Z2, st);
  return launch_bgemm<128, 3>(p, ta, tb, d.Z1 * d.Z2, st);
}


#ifdef SRT_PHASE_STAMPS
extern "C" int srt_dbg_set_phase_stamps(void* device_buffer) {
  unsigned long long* p = (unsigned long long*)device_buffer;
  SRT_CHECK_CUDA(cudaMemcpyToSymbol(g_phase_stamps, &p, sizeof(p)));
  return SRT_OK;
}
#endif

void bn_grid_reset_barriers();  // norm_grid.cu
int* tc_status_device_ptr() { return status_ptr(); }

// Reads and clears the device status word of the tcgen05 kernels (synchronises the device).
int tc_status_fetch(int* out) {
  int* sp = status_ptr();
  SRT_REQUIRE(sp != nullptr, "tcgen05 status word unavailable");
  SRT_CHECK_CUDA(cudaDeviceSynchronize());
  SRT_CHECK_CUDA(cudaMemcpy(out, sp, sizeof(int), cudaMemcpyDeviceToHost));
  if (*out != 0) {
    int zero = 0;
    SRT_CHECK_CUDA(cudaMemcpy(sp, &zero, sizeof(int), cudaMemcpyHostToDevice));
    bn_grid_reset_barriers();
  }
  return SRT_OK;
}

// Plan override of the fprop/dgrad kernel (a tuning and test aid; 0 / 0 / -1 restores the heuristics):
//   gather  1: fetch plain-matrix (1x1, stride 1) operands with the gather threads instead of TMA
//   tile_n  64, 128 or 256: output-tile width
//   pair    0: one CTA per tile, 1: CTA pairs wherever the shape allows, -1: heuristic
static int g_force_bn = 0;
static int g_gather_lag = getenv("SIRIUS_B200_GATHER_LAG") ? atoi(getenv("SIRIUS_B200_GATHER_LAG")) : 0;  // 0 = stage count - 2
void tc_set_wgrad_pairs(bool on) { g_wgrad_pair = on ? 1 : 0; }
bool tc_wgrad_pairs() { return g_wgrad_pair != 0; }

void tc_set_conv_plan(int gather, int tile_n, int pair) {
  g_force_gather = gather;
  g_force_bn = tile_n;
  g_force_pair = pair;
}

static int conv_gather_gemm_tc_persistent(const GatherGeom& g, const void* src, const void* Bm, void* D,
                                          const srt_conv_epilogue* ep, cudaStream_t st, double* col_partial = nullptr) {
  PersistParams p;
  p.g = g;
  p.col_partial = col_partial;
  p.src = (const bf16*)src;
  p.bias = ep ? ep->bias : nullptr;
  p.addend = ep ? (const bf16*)ep->addend : nullptr;
  p.addend_bits = ep && ep->addend ? ep->addend_bits : nullptr;
  p.k_blocks = ceil_div(g.Kg, BK);
  p.status = status_ptr();
  SRT_REQUIRE(p.status != nullptr, "tcgen05 status word unavailable");
  const bool plain = g.R == 1 && g.S == 1 && g.stride == 1 && g.pad == 0;
  p.a_tma = g_force_gather ? 0 : plain ? 1 : (im2col_ok(g) && g_im2col_enabled) ? 2 : 0;
  p.im_lower_w = p.im_lower_h = p.im_flip = 0;
  p.im_stride = p.im_cpt = 1;
  if (p.a_tma == 2) {
    const Im2colBox b = im2col_box(g);
    p.im_lower_w = b.lower_w; p.im_lower_h = b.lower_h; p.im_stride = b.stride;
    p.im_cpt = g.src_c / BK;
    p.im_flip = g.dgrad;
  }
  p.gather_lag = 0;  // set with the stage count below
  // CTA pairs: the unit is a 256 x tile_n tile of which each CTA stages half the filters, so the operand stream
  // per SM shrinks by a quarter to a third. Measured on the ResNet shapes (16-36 k-blocks per tile) that gain is
  // eaten by the pair's cross-SM signalling (+-5 %); on long reductions it is 13 % (64 k-blocks: 47.3 -> 41.3 us).
  // The heuristic therefore pairs plain-matrix (TMA-fed) problems from 32 k-blocks up whose output is at least
  // 128 columns wide (a 64-column tile would leave each CTA 32 filters per k-block): the MLP down-projections and
  // the data gradients of the wide layers of the transformer steps.
  bool pair = p.a_tma && p.k_blocks >= 32 && g.Nout >= 128 && g_force_bn != 64;
  static const int fwd_pair_env = getenv("SIRIUS_B200_FWD_PAIR") ? atoi(getenv("SIRIUS_B200_FWD_PAIR")) : -1;
  if (fwd_pair_env == 0) pair = false;
  if (g_force_pair == 0) pair = false;
  if (g_force_pair == 1) pair = g.Nout > 64 && g_force_bn != 64;
  if (sm_count() < 2) pair = false;
  int bn;
  if (pair) bn = g_force_bn ? g_force_bn : (g.Nout > 128 ? 256 : 128);
  else bn = pick_bn(g.M, g.Nout, g_force_bn);
  p.m_tiles = ceil_div(g.M, BM);
  p.n_tiles = ceil_div(g.Nout, bn);
  CUtensorMap tb, ta, td;
  int rc = make_tmap_2d(&tb, Bm, (uint64_t)g.Nout, (uint64_t)g.Kg, (uint32_t)(pair ? bn / 2 : bn));
  if (rc != SRT_OK) return rc;
  if (p.a_tma == 1) {
    rc = make_tmap_2d(&ta, src, (uint64_t)g.M, (uint64_t)g.Kg, (uint32_t)BM);
    if (rc != SRT_OK) return rc;
  } else if (p.a_tma == 2) {
    rc = make_tmap_im2col(&ta, src, g, (uint32_t)BM);
    if (rc != SRT_OK) return rc;
  } else {
    ta = tb;
  }
  rc = make_tmap_store(&td, D, (uint64_t)g.M, (uint64_t)g.Nout);
  if (rc != SRT_OK) return rc;
  auto lag = [&](int ns) {
    int l = g_gather_lag > 0 ? g_gather_lag : ns - 2;
    if (l > ns - 2) l = ns - 2;
    if (l > 4) l = 4;
    return l < 1 ? 1 : l;
  };
  if (pair) {
    if (bn == 128) { p.gather_lag = lag(6); return launch_persistent<128, 6, true>(p, tb, ta, td, st); }
    p.gather_lag = lag(5);
    return launch_persistent<256, 5, true>(p, tb, ta, td, st);
  }
  if (bn == 64) { p.gather_lag = lag(6); return launch_persistent<64, 6, false>(p, tb, ta, td, st); }
  if (bn == 128) { p.gather_lag = lag(5); return launch_persistent<128, 5, false>(p, tb, ta, td, st); }
  p.gather_lag = lag(3);
  return launch_persistent<256, 3, false>(p, tb, ta, td, st);
}

int conv_gather_gemm_tc(const GatherGeom& g, const void* src, const void* Bm, void* D,
                        const srt_conv_epilogue* ep, cudaStream_t st) {
  SRT_REQUIRE(g.src_c % 8 == 0 && g.Nout % 8 == 0,
              "tcgen05 conv: channel counts (%d, %d) must be multiples of 8", g.src_c, g.Nout);
  SRT_REQUIRE(((uintptr_t)src & 15) == 0 && ((uintptr_t)D & 15) == 0, "tcgen05 conv: unaligned tensor");
  return conv_gather_gemm_tc_persistent(g, src, Bm, D, ep, st);
}

// Convolution whose epilogue also leaves the per-tile column sums for the BatchNorm that follows
// (double2 [ceil(M/128)][Nout]: sum, sum of squares).
bool conv_col_stats_available() { return true; }
size_t conv_col_stats_bytes(int64_t M, int Nout) { return (size_t)ceil_div_ll(M, BM) * Nout * 2 * sizeof(double); }
int conv_gather_gemm_tc_stats(const GatherGeom& g, const void* src, const void* Bm, void* D, const srt_conv_epilogue* ep,
                              double* col_partial, size_t col_partial_bytes, int* slabs, cudaStream_t st) {
  SRT_REQUIRE(g.src_c % 8 == 0 && g.Nout % 8 == 0,
              "tcgen05 conv: channel counts (%d, %d) must be multiples of 8", g.src_c, g.Nout);
  SRT_REQUIRE(((uintptr_t)src & 15) == 0 && ((uintptr_t)D & 15) == 0, "tcgen05 conv: unaligned tensor");
  SRT_REQUIRE(col_partial && ((uintptr_t)col_partial & 15) == 0 && col_partial_bytes >= conv_col_stats_bytes(g.M, g.Nout),
              "tcgen05 conv: column-sum buffer missing, unaligned or too small (%zu < %zu)", col_partial_bytes,
              conv_col_stats_bytes(g.M, g.Nout));
  if (slabs) *slabs = ceil_div(g.M, BM);
  return conv_gather_gemm_tc_persistent(g, src, Bm, D, ep, st, col_partial);
}

static size_t wgrad_plan_bytes(const GatherGeom& g, const WgradPlan& w) {
  return w.splits > 1 ? (size_t)w.splits * g.Nout * g.Kg * sizeof(float) : 0;
}
// Enough for either kernel: a caller sizes its scratch once, and which kernel a launch takes can change afterwards
// (srt_conv_wgrad_pairs, a plan override).
size_t conv_wgrad_tc_scratch_bytes(const GatherGeom& g) {
  const size_t a = wgrad_plan_bytes(g, plan_wgrad(g, true, true)), b = wgrad_plan_bytes(g, plan_wgrad(g, false));
  return a > b ? a : b;
}

int conv_wgrad_tc(const GatherGeom& g, const void* dy, const void* x, float* dw, void* scratch,
                  size_t scratch_bytes, cudaStream_t st) {
  SRT_REQUIRE(g.src_c % 8 == 0 && g.Nout % 8 == 0,
              "tcgen05 wgrad: channel counts (%d, %d) must be multiples of 8", g.src_c, g.Nout);
  WgradPlan w = plan_wgrad(g);
  const size_t need = wgrad_plan_bytes(g, w);
  SRT_REQUIRE(scratch_bytes >= need && (need == 0 || scratch != nullptr),
              "tcgen05 wgrad: scratch too small (%zu < %zu)", scratch_bytes, need);
  WgradParams p;
  p.g = g;
  p.x = (const bf16*)x;
  p.out = w.splits > 1 ? (float*)scratch : dw;
  p.pix_per_split = w.pix_per_split;
  p.status = status_ptr();
  SRT_REQUIRE(p.status != nullptr, "tcgen05 status word unavailable");
  fastdiv_make((uint32_t)(g.out_h * g.out_w), &p.hw_mul, &p.hw_shr);
  fastdiv_make((uint32_t)g.out_w, &p.w_mul, &p.w_shr);
  p.b_tma = w.b_tma;
  CUtensorMap tdy, tx;
  int rc = make_tmap_2d(&tdy, dy, (uint64_t)g.M, (uint64_t)g.Nout, 64);
  if (rc != SRT_OK) return rc;
  if (p.b_tma == 1) {
    rc = make_tmap_2d(&tx, x, (uint64_t)g.M, (uint64_t)g.src_c, 64);
    if (rc != SRT_OK) return rc;
  } else if (p.b_tma == 2) {
    rc = make_tmap_im2col(&tx, x, g, 64);
    if (rc != SRT_OK) return rc;
  } else {
    tx = tdy;
  }
  if (w.pair) {
    CUtensorMap tout;
    rc = make_tmap_wgrad_out(&tout, p.out, (uint64_t)g.Kg, (uint64_t)g.Nout, (uint64_t)w.splits);
    if (rc != SRT_OK) return rc;
    rc = launch_wgrad_pair(p, tdy, tx, tout, w.splits, st);
    if (rc != SRT_OK) return rc;
    if (w.splits > 1) return launch_split_reduce(p.out, dw, (long long)g.Nout * g.Kg, w.splits, st);
    return SRT_OK;
  }
  // Three stages of 32 KB leave room for two CTAs per SM (the split count assumes them): one CTA's prologue and
  // its fp32 epilogue then run beside the other's main loop. Four stages (one CTA per SM) remain selectable.
  static const int stages = getenv("SIRIUS_B200_WGRAD_STAGES") ? atoi(getenv("SIRIUS_B200_WGRAD_STAGES")) : 3;
  rc = w.bn == 64 ? launch_wgrad<64, 4>(p, tdy, tx, w.splits, st)
       : stages == 4 ? launch_wgrad<128, 4>(p, tdy, tx, w.splits, st)
                     : launch_wgrad<128, 3>(p, tdy, tx, w.splits, st);
  if (rc != SRT_OK) return rc;
  if (w.splits > 1) return launch_split_reduce(p.out, dw, (long long)g.Nout * g.Kg, w.splits, st);
  return SRT_OK;
}

}  // namespace srt
