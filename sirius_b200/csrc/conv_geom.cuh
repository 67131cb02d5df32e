// Implicit-GEMM geometry shared by the CUDA-core and tcgen05 convolution kernels.
//
// A "gather GEMM" computes D[m][n] = sum_k A(m,k) * B[n][k] where row m is one output position
// (image, oh, ow), k = tap * src_c + c walks filter taps (r,s) and source channels, and A(m,k) is
// read from an NHWC source tensor (zero outside it):
//   fprop : source = x,  (ih, iw) = (oh*stride - pad + r, ow*stride - pad + s)
//   dgrad : source = dy, (ih, iw) = ((oh + pad - r)/stride, (ow + pad - s)/stride) when divisible
// wgrad reuses the fprop geometry with the roles of rows and the reduction swapped.
#pragma once
#include "common.cuh"

namespace srt {

struct GatherGeom {
  int n_img, src_h, src_w, src_c;  // source NHWC tensor
  int out_h, out_w;                // row grid: M = n_img*out_h*out_w
  int R, S, stride, pad;
  int dgrad;                       // 0: fprop-style gather, 1: dgrad-style gather
  int M, Kg, Nout;                 // GEMM extents (Kg = R*S*src_c)
};

struct RowCoord {
  int n, oh, ow;
};

__host__ __device__ inline RowCoord decode_row(const GatherGeom& g, int m) {
  RowCoord rc;
  const int hw = g.out_h * g.out_w;
  rc.n = m / hw;
  const int rem = m - rc.n * hw;
  rc.oh = rem / g.out_w;
  rc.ow = rem - rc.oh * g.out_w;
  return rc;
}

// Element offset of source channel c under filter tap `tap` for output position rc, or -1 when the
// tap falls outside the source tensor (contributes zero).
__host__ __device__ inline long long gather_offset(const GatherGeom& g, const RowCoord& rc, int tap,
                                                   int c) {
  const int r = tap / g.S, s = tap - r * g.S;
  int ih, iw;
  if (!g.dgrad) {
    ih = rc.oh * g.stride - g.pad + r;
    iw = rc.ow * g.stride - g.pad + s;
  } else {
    const int th = rc.oh + g.pad - r, tw = rc.ow + g.pad - s;
    if (th < 0 || tw < 0) return -1;
    if (g.stride > 1) {
      if ((th % g.stride) != 0 || (tw % g.stride) != 0) return -1;
      ih = th / g.stride;
      iw = tw / g.stride;
    } else {
      ih = th;
      iw = tw;
    }
  }
  if (ih < 0 || iw < 0 || ih >= g.src_h || iw >= g.src_w) return -1;
  return (((long long)rc.n * g.src_h + ih) * g.src_w + iw) * g.src_c + c;
}

inline GatherGeom make_fprop_geom(const srt_conv_desc& d) {
  GatherGeom g;
  g.n_img = d.N; g.src_h = d.H; g.src_w = d.W; g.src_c = d.C;
  g.out_h = d.P; g.out_w = d.Q;
  g.R = d.R; g.S = d.S; g.stride = d.stride; g.pad = d.pad; g.dgrad = 0;
  g.M = d.N * d.P * d.Q; g.Kg = d.R * d.S * d.C; g.Nout = d.K;
  return g;
}

inline GatherGeom make_dgrad_geom(const srt_conv_desc& d) {
  GatherGeom g;
  g.n_img = d.N; g.src_h = d.P; g.src_w = d.Q; g.src_c = d.K;
  g.out_h = d.H; g.out_w = d.W;
  g.R = d.R; g.S = d.S; g.stride = d.stride; g.pad = d.pad; g.dgrad = 1;
  g.M = d.N * d.H * d.W; g.Kg = d.R * d.S * d.K; g.Nout = d.C;
  return g;
}

// Declared here, defined in conv_simt.cu / igemm_tcgen05.cu.
int conv_gather_gemm_simt(const GatherGeom& g, int dtype, const void* src, const void* Bm, void* D,
                          const srt_conv_epilogue* ep, cudaStream_t st);
int conv_wgrad_simt(const GatherGeom& g, int dtype, const void* dy, const void* x, float* dw,
                    void* scratch, size_t scratch_bytes, cudaStream_t st);
size_t conv_wgrad_simt_scratch_bytes(const GatherGeom& g);
int launch_split_reduce(const float* partial, float* out, long long n, int splits, cudaStream_t st);

int conv_gather_gemm_tc(const GatherGeom& g, const void* src, const void* Bm, void* D,
                        const srt_conv_epilogue* ep, cudaStream_t st);
// The same kernel, whose epilogue also writes per 128-row tile and output column the sum and the sum of squares
// of the stored values (double2 [slabs][Nout]) for the BatchNorm that follows.
bool conv_col_stats_available();
size_t conv_col_stats_bytes(int64_t M, int Nout);
int conv_gather_gemm_tc_stats(const GatherGeom& g, const void* src, const void* Bm, void* D, const srt_conv_epilogue* ep,
                              double* col_partial, size_t col_partial_bytes, int* slabs, cudaStream_t st);
int conv_wgrad_tc(const GatherGeom& g, const void* dy, const void* x, float* dw, void* scratch,
                  size_t scratch_bytes, cudaStream_t st);
size_t conv_wgrad_tc_scratch_bytes(const GatherGeom& g);

}  // namespace srt
