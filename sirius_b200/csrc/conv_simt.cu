// CUDA-core implicit-GEMM convolution: fp32 accumulate, fp32 or bf16 operands.
//
// This is the exact-arithmetic path (fp32 mode of the training step) and the on-device
// cross-check for the tcgen05 kernels. One gather-GEMM kernel serves fprop and dgrad, one
// split-reduction kernel serves wgrad; partial sums are reduced in a fixed order so results are
// run-to-run deterministic.
#include "common.cuh"
#include "conv_geom.cuh"

namespace srt {

namespace {

constexpr int BM = 64, BN = 64, BK = 16, NT = 256;

template <typename T> struct Ld4;
template <> struct Ld4<float> {
  __device__ static inline void ld(const float* p, float (&v)[4]) {
    float4 r = *reinterpret_cast<const float4*>(p);
    v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
  }
};
template <> struct Ld4<__nv_bfloat16> {
  __device__ static inline void ld(const __nv_bfloat16* p, float (&v)[4]) {
    uint2 r = *reinterpret_cast<const uint2*>(p);
    v[0] = __uint_as_float(r.x << 16); v[1] = __uint_as_float(r.x & 0xffff0000u);
    v[2] = __uint_as_float(r.y << 16); v[3] = __uint_as_float(r.y & 0xffff0000u);
  }
};

// D[m][n] = sum_k A(m,k) * B[n][k], A gathered from an NHWC tensor (see GatherGeom).
template <typename T>
__global__ void __launch_bounds__(NT)
gather_gemm_simt(GatherGeom g, const T* __restrict__ src, const T* __restrict__ Bm,
                 T* __restrict__ D, const float* __restrict__ bias, const T* addend, const uint8_t* __restrict__ addend_bits) {
  __shared__ __align__(16) float As[BK][BM + 4];
  __shared__ __align__(16) float Bs[BK][BN + 4];
  const int t = threadIdx.x;
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
  const int lrow = t >> 2, lk = (t & 3) * 4;

  // fixed per-thread row decode
  const int m = m0 + lrow;
  RowCoord rc = decode_row(g, m);
  const int nb = n0 + lrow;
  const bool nb_ok = nb < g.Nout;
  const T* brow = Bm + (size_t)(nb_ok ? nb : 0) * g.Kg;

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  const int tx = t & 15, ty = t >> 4;
  for (int k0 = 0; k0 < g.Kg; k0 += BK) {
    const int kk = k0 + lk;
    float a[4] = {0.f, 0.f, 0.f, 0.f}, b[4] = {0.f, 0.f, 0.f, 0.f};
    if (kk < g.Kg) {
      const int tap = kk / g.src_c, c = kk - tap * g.src_c;
      const long long off = m < g.M ? gather_offset(g, rc, tap, c) : -1;
      if (off >= 0) Ld4<T>::ld(src + off, a);
      if (nb_ok) Ld4<T>::ld(brow + kk, b);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) { As[lk + i][lrow] = a[i]; Bs[lk + i][lrow] = b[i]; }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float4 av = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
      float4 bv = *reinterpret_cast<const float4*>(&Bs[k][tx * 4]);
      const float ar[4] = {av.x, av.y, av.z, av.w}, br[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int mm = m0 + ty * 4 + i;
    if (mm >= g.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int nn = n0 + tx * 4 + j;
      if (nn >= g.Nout) continue;
      float v = acc[i][j];
      if (bias) v += bias[nn];
      const size_t o = (size_t)mm * g.Nout + nn;
      if (addend && (!addend_bits || ((addend_bits[o >> 3] >> (o & 7)) & 1))) v += ElemTraits<T>::to_f(addend[o]);
      D[o] = ElemTraits<T>::from_f(v);
    }
  }
}

// partial[split][ko][j] = sum over this split's pixels of dy[pix][ko] * x(pix, j), j = (r,s,c).
template <typename T>
__global__ void __launch_bounds__(NT)
wgrad_simt(GatherGeom g /* fprop geometry: rows = output pixels */, const T* __restrict__ dy,
           const T* __restrict__ x, float* __restrict__ partial, int pix_per_split) {
  __shared__ __align__(16) float As[BK][BM + 4];  // [pix][ko]
  __shared__ __align__(16) float Bs[BK][BN + 4];  // [pix][j]
  const int t = threadIdx.x;
  const int j0 = blockIdx.x * BN, ko0 = blockIdx.y * BM;
  const int Kout = g.Nout, J = g.Kg;
  const int pbeg = blockIdx.z * pix_per_split;
  const int pend = min(g.M, pbeg + pix_per_split);
  const int lp = t >> 4, l4 = (t & 15) * 4;

  const int jj = j0 + l4;
  const bool j_ok = jj < J;
  const int tap = j_ok ? jj / g.src_c : 0, c = j_ok ? jj - tap * g.src_c : 0;
  const int kk = ko0 + l4;
  const bool k_ok = kk < Kout;

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  const int tx = t & 15, ty = t >> 4;

  for (int p0 = pbeg; p0 < pend; p0 += BK) {
    const int pix = p0 + lp;
    float a[4] = {0.f, 0.f, 0.f, 0.f}, b[4] = {0.f, 0.f, 0.f, 0.f};
    if (pix < pend) {
      if (k_ok) Ld4<T>::ld(dy + (size_t)pix * Kout + kk, a);
      if (j_ok) {
        RowCoord rc = decode_row(g, pix);
        const long long off = gather_offset(g, rc, tap, c);
        if (off >= 0) Ld4<T>::ld(x + off, b);
      }
    }
    *reinterpret_cast<float4*>(&As[lp][l4]) = make_float4(a[0], a[1], a[2], a[3]);
    *reinterpret_cast<float4*>(&Bs[lp][l4]) = make_float4(b[0], b[1], b[2], b[3]);
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float4 av = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
      float4 bv = *reinterpret_cast<const float4*>(&Bs[k][tx * 4]);
      const float ar[4] = {av.x, av.y, av.z, av.w}, br[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
    }
    __syncthreads();
  }
  float* out = partial + (size_t)blockIdx.z * Kout * J;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int ko = ko0 + ty * 4 + i;
    if (ko >= Kout) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int q = j0 + tx * 4 + j;
      if (q < J) out[(size_t)ko * J + q] = acc[i][j];
    }
  }
}

}  // namespace

__global__ void split_reduce_kernel(const float* __restrict__ partial, float* __restrict__ out,
                                    long long n, int splits) {
  pdl_enter();
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    float s = 0.f;
    for (int k = 0; k < splits; ++k) s += partial[(size_t)k * n + i];
    out[i] = s;
  }
}

int launch_split_reduce(const float* partial, float* out, long long n, int splits,
                        cudaStream_t st) {
  const int threads = 256;
  long long blocks = (n + threads - 1) / threads;
  const long long cap = (long long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  launch_pdl(split_reduce_kernel, dim3((unsigned)blocks), dim3(threads), 0, st, partial, out, n, splits);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}

template <typename T>
static int gather_gemm_simt_launch(const GatherGeom& g, const void* src, const void* Bm, void* D,
                                   const srt_conv_epilogue* ep, cudaStream_t st) {
  dim3 grid(ceil_div(g.M, BM), ceil_div(g.Nout, BN));
  gather_gemm_simt<T><<<grid, NT, 0, st>>>(g, (const T*)src, (const T*)Bm, (T*)D,
                                          ep ? ep->bias : nullptr,
                                          ep ? (const T*)ep->addend : nullptr, ep ? ep->addend_bits : nullptr);
  SRT_LAUNCH_CHECK();
  return SRT_OK;
}

int conv_gather_gemm_simt(const GatherGeom& g, int dtype, const void* src, const void* Bm, void* D,
                          const srt_conv_epilogue* ep, cudaStream_t st) {
  SRT_REQUIRE(g.src_c % 4 == 0, "simt conv: channels per tap (%d) must be a multiple of 4", g.src_c);
  if (dtype == SRT_F32) return gather_gemm_simt_launch<float>(g, src, Bm, D, ep, st);
  return gather_gemm_simt_launch<__nv_bfloat16>(g, src, Bm, D, ep, st);
}

int wgrad_simt_splits(const GatherGeom& g) {
  const int tiles = ceil_div(g.Nout, BM) * ceil_div(g.Kg, BN);
  int want = ceil_div(4 * sm_count(), tiles);
  int max_by_pix = ceil_div(g.M, 4 * BK);
  int splits = want < max_by_pix ? want : max_by_pix;
  if (splits < 1) splits = 1;
  if (splits > 256) splits = 256;
  return splits;
}

size_t conv_wgrad_simt_scratch_bytes(const GatherGeom& g) {
  const int splits = wgrad_simt_splits(g);
  return splits > 1 ? (size_t)splits * g.Nout * g.Kg * sizeof(float) : 0;
}

int conv_wgrad_simt(const GatherGeom& g, int dtype, const void* dy, const void* x, float* dw,
                    void* scratch, size_t scratch_bytes, cudaStream_t st) {
  SRT_REQUIRE(g.src_c % 4 == 0 && g.Nout % 4 == 0,
              "simt wgrad: C (%d) and K (%d) must be multiples of 4", g.src_c, g.Nout);
  int splits = wgrad_simt_splits(g);
  const size_t need = conv_wgrad_simt_scratch_bytes(g);
  SRT_REQUIRE(scratch_bytes >= need && (need == 0 || scratch != nullptr),
              "simt wgrad: scratch too small (%zu < %zu)", scratch_bytes, need);
  int pps = ceil_div(ceil_div(g.M, splits), BK) * BK;
  splits = ceil_div(g.M, pps);
  float* partial = splits > 1 ? (float*)scratch : dw;
  dim3 grid(ceil_div(g.Kg, BN), ceil_div(g.Nout, BM), splits);
  if (dtype == SRT_F32)
    wgrad_simt<float><<<grid, NT, 0, st>>>(g, (const float*)dy, (const float*)x, partial, pps);
  else
    wgrad_simt<__nv_bfloat16><<<grid, NT, 0, st>>>(g, (const __nv_bfloat16*)dy,
                                                    (const __nv_bfloat16*)x, partial, pps);
  SRT_LAUNCH_CHECK();
  if (splits > 1) return launch_split_reduce(partial, dw, (long long)g.Nout * g.Kg, splits, st);
  return SRT_OK;
}

}  // namespace srt
