// Training step of a Swin transformer (the reference trains torchvision.models.swin_b,
// train/swin_b.py:38,83-95): 4x4 patch embedding + LayerNorm, four stages of blocks
// [LayerNorm, shifted-window multi-head attention with relative-position bias, LayerNorm, MLP with erf-GELU],
// patch merging between stages, final LayerNorm, average pool, linear head, cross-entropy, AdamW.
//
// Data layout: tokens stay in the natural [batch][row][col] order as [tokens][features] bf16 rows, so every
// linear layer is a 1x1 convolution on the tcgen05 implicit-GEMM kernels (bias / residual in the epilogue).
// Only attention works on windows: Q, K, V are regrouped to [window][head][49][D] (the cyclic shift is folded
// into that permutation), the four small products per window and head are batched tcgen05 GEMMs over all
// windows at once, and the result goes back through the inverse permutation. Rows of 49 are padded to 56
// wherever they are a reduction or output axis.
#include <string.h>

#include <string>
#include <vector>

#include "../../include/sirius_b200.h"
#include "common.cuh"
#include "grad_buckets.cuh"
#include "ops.cuh"
#include "partition_follow.cuh"

namespace srt {

namespace {
inline size_t up_(size_t v, size_t a) { return (v + a - 1) / a * a; }
}

struct Swin {
  srt_swin_config cfg;
  int WS, L, LP;  // window side, tokens per window, padded row length
  cudaStream_t stream = nullptr;

  struct Rec { std::string name; size_t off, count; int64_t shape[4]; int ndim; int kind; int cpad; };  // kind 2 = conv KCRS outside
  std::vector<Rec> params;
  size_t n_flat = 0, n_wt = 0;
  float *P = nullptr, *G = nullptr, *M1 = nullptr, *M2 = nullptr;
  __nv_bfloat16 *Pw = nullptr, *WT = nullptr;
  int opt_steps = 0;

  struct Lin { int w, b, in, out; size_t wt_off; };
  struct Blk {
    int C, heads, D, Hs, shift;
    int n1g, n1b, n2g, n2b, table;
    Lin qkv, proj, fc, fc2;
    __nv_bfloat16 *ln1o, *qw, *kw, *vw, *Pm, *att, *x2, *ln2o, *h, *g, *xout;
    float *m1, *r1, *m2, *r2;
  };
  struct Merge {
    int C, Hs;  // input channels and map side
    int ng, nb;
    Lin red;
    __nv_bfloat16 *merged, *lno, *out;
    float *m, *r;
  };
  std::vector<Blk> blocks;
  std::vector<int> stage_end;   // index one past the last block of each stage
  std::vector<Merge> merges;
  int pe_w, pe_b, pe_ng, pe_nb, fn_g, fn_b;
  Lin head;
  int Cf, Hf;  // final features and map side

  // activations and scratch
  float* stage_images = nullptr;
  int64_t* stage_labels = nullptr;
  __nv_bfloat16 *x_img = nullptr, *e0 = nullptr, *x0 = nullptr, *fno = nullptr, *pooled = nullptr, *logits = nullptr, *dlogits = nullptr;
  float *pe_m = nullptr, *pe_r = nullptr, *fn_m = nullptr, *fn_r = nullptr, *row_loss = nullptr, *loss_acc = nullptr;
  float *relbias = nullptr, *dbias = nullptr;
  __nv_bfloat16 *dxa = nullptr, *dxb = nullptr, *dqkv = nullptr, *dP = nullptr, *tP = nullptr, *tA = nullptr, *tB = nullptr,
                *dOh = nullptr, *dqw = nullptr, *dkw = nullptr, *dvw = nullptr, *dh = nullptr, *dg = nullptr, *datt = nullptr,
                *dln = nullptr, *ow = nullptr, *dpool = nullptr;
  // Weight and bias gradients of a linear layer depend only on (dy, saved input): they run on a second,
  // lowest-priority stream beside the data gradient and whatever follows it in the layer. The main stream waits for
  // them before it overwrites a dy buffer they read (once per layer, before the layer's last kernel) and at the end.
  cudaStream_t side = nullptr;
  PartitionFollower part;   // SM-partition following between layers (off by default)
  cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
  bool side_dirty = false, overlap_wgrad = true;
  void* scratch_side = nullptr;
  int join_side() {
    if (!side || !side_dirty) return SRT_OK;
    side_dirty = false;
    SRT_CHECK_CUDA(cudaEventRecord(ev_join, side));
    SRT_CHECK_CUDA(cudaStreamWaitEvent(stream, ev_join, 0));
    return SRT_OK;
  }
  GradBuckets buckets;      // units: the blocks in forward order, each stage's patch merging counted with its last block
  void* scratch = nullptr;
  size_t scratch_bytes = 0;
  std::vector<void*> allocs;
  size_t bytes_total = 0;
  int cur_B = 0, last_global = 0;

  ~Swin() {
    if (part.home_stream) { stream = part.home_stream; side = part.home_side; }  // partition streams belong to the ladder
    if (ev_fork) cudaEventDestroy(ev_fork);
    if (ev_join) cudaEventDestroy(ev_join);
    if (side) { cudaStreamSynchronize(side); cudaStreamDestroy(side); }
    for (void* p : allocs) cudaFree(p);
    if (stream) cudaStreamDestroy(stream);
  }
  template <class T>
  int dalloc(T** out, size_t bytes, bool zero = false) {
    bytes = up_(bytes ? bytes : 256, 256) + 4096;  // slack: padded window rows are read a little past the last window
    SRT_CHECK_CUDA(cudaMalloc((void**)out, bytes));
    allocs.push_back((void*)*out);
    bytes_total += bytes;
    if (zero) SRT_CHECK_CUDA(cudaMemset(*out, 0, bytes));
    return SRT_OK;
  }
  int add(const std::string& name, std::initializer_list<int64_t> shape, int kind, size_t count, int cpad = 0) {
    Rec r;
    r.name = name; r.off = n_flat; r.count = count; r.kind = kind; r.cpad = cpad;
    r.ndim = (int)shape.size();
    int i = 0;
    for (int64_t d : shape) r.shape[i++] = d;
    for (; i < 4; ++i) r.shape[i] = 0;
    n_flat += up_(count, 64);
    params.push_back(r);
    return (int)params.size() - 1;
  }
  Lin add_lin(const std::string& pre, int in, int out, bool bias = true) {
    Lin l;
    l.in = in; l.out = out;
    l.w = add(pre + ".weight", {out, in}, 0, (size_t)in * out);
    l.b = bias ? add(pre + ".bias", {out}, 0, (size_t)out) : -1;
    l.wt_off = n_wt;
    n_wt += up_((size_t)in * out, 64);
    return l;
  }
  float* pf(int i) { return P + params[i].off; }
  float* gf(int i) { return G + params[i].off; }
  __nv_bfloat16* pw(int i) { return Pw + params[i].off; }
  srt_conv_desc lin_desc(int64_t T, int in, int out) const { return {(int)T, 1, 1, in, out, 1, 1, 1, 0, 1, 1}; }
  int linear_fwd(const Lin& l, const void* x, void* y, const void* residual, int64_t T) {
    srt_conv_epilogue ep = {l.b >= 0 ? pf(l.b) : nullptr, residual};
    return conv_fprop(lin_desc(T, l.in, l.out), SRT_BF16, SRT_IMPL_AUTO, x, pw(l.w), y, &ep, stream);
  }
  int linear_bwd(const Lin& l, const void* dy, const void* x, void* dx, int64_t T) {
    int rc;
    cudaStream_t ws = stream;
    void* wscratch = scratch;
    if (side && overlap_wgrad) {
      SRT_CHECK_CUDA(cudaEventRecord(ev_fork, stream));
      SRT_CHECK_CUDA(cudaStreamWaitEvent(side, ev_fork, 0));
      side_dirty = true;
      ws = side;
      wscratch = scratch_side;
    }
    {
      PdlOff no_early_launch(ws != stream);
      if (l.b >= 0 && (rc = colsum_bf16(dy, T, l.out, gf(l.b), wscratch, scratch_bytes, ws))) return rc;
      if ((rc = conv_wgrad(lin_desc(T, l.in, l.out), SRT_BF16, SRT_IMPL_AUTO, dy, x, gf(l.w), wscratch, scratch_bytes, ws)))
        return rc;
    }
    if (dx) return conv_dgrad(lin_desc(T, l.in, l.out), SRT_BF16, SRT_IMPL_AUTO, dy, WT + l.wt_off, dx, nullptr, stream);
    return SRT_OK;
  }
  srt_conv_desc pe_desc(int B) const {
    const int I = cfg.image, p = cfg.patch;
    return {B, I, I, 8, cfg.embed, p, p, p, 0, I / p, I / p};
  }
  int build();
  int transposes();
  int forward(int B);
  int backward(int B, int global_batch);
  int block_fwd(Blk& k, const __nv_bfloat16* x, int B);
  int block_bwd(Blk& k, const __nv_bfloat16* xin, __nv_bfloat16*& dx, __nv_bfloat16*& dx_other, int B);
};

int Swin::build() {
  WS = cfg.window; L = WS * WS; LP = (int)up_((size_t)L, 8);
  SRT_REQUIRE(cfg.image % cfg.patch == 0 && cfg.max_batch > 0 && cfg.num_classes % 8 == 0 && L <= 64,
              "swin: image must be a multiple of the patch, classes of 8, window area at most 64");
  const int S0 = cfg.image / cfg.patch;
  pe_w = add("features.0.0.weight", {cfg.embed, 3, cfg.patch, cfg.patch}, 2, (size_t)cfg.embed * cfg.patch * cfg.patch * 8, 8);
  pe_b = add("features.0.0.bias", {cfg.embed}, 0, cfg.embed);
  pe_ng = add("features.0.2.weight", {cfg.embed}, 0, cfg.embed);
  pe_nb = add("features.0.2.bias", {cfg.embed}, 0, cfg.embed);
  int C = cfg.embed, Hs = S0;
  for (int s = 0; s < 4; ++s) {
    SRT_REQUIRE(Hs % WS == 0 && C % cfg.heads[s] == 0 && (C / cfg.heads[s]) % 8 == 0,
                "swin: stage %d: map %d must be a multiple of the window and the head size of 8", s, Hs);
    for (int i = 0; i < cfg.depths[s]; ++i) {
      const std::string pre = "features." + std::to_string(2 * s + 1) + "." + std::to_string(i);
      Blk k;
      k.C = C; k.heads = cfg.heads[s]; k.D = C / k.heads; k.Hs = Hs;
      k.shift = (i % 2 == 1 && WS < Hs) ? WS / 2 : 0;
      k.n1g = add(pre + ".norm1.weight", {C}, 0, C);
      k.n1b = add(pre + ".norm1.bias", {C}, 0, C);
      k.table = add(pre + ".attn.relative_position_bias_table", {(2 * WS - 1) * (2 * WS - 1), k.heads}, 0,
                    (size_t)(2 * WS - 1) * (2 * WS - 1) * k.heads);
      k.qkv = add_lin(pre + ".attn.qkv", C, 3 * C);
      k.proj = add_lin(pre + ".attn.proj", C, C);
      k.n2g = add(pre + ".norm2.weight", {C}, 0, C);
      k.n2b = add(pre + ".norm2.bias", {C}, 0, C);
      k.fc = add_lin(pre + ".mlp.0", C, 4 * C);
      k.fc2 = add_lin(pre + ".mlp.3", 4 * C, C);
      blocks.push_back(k);
    }
    stage_end.push_back((int)blocks.size());
    if (s < 3) {
      const std::string pre = "features." + std::to_string(2 * s + 2);
      Merge m;
      m.C = C; m.Hs = Hs;
      m.red = add_lin(pre + ".reduction", 4 * C, 2 * C, false);
      m.ng = add(pre + ".norm.weight", {4 * C}, 0, 4 * C);
      m.nb = add(pre + ".norm.bias", {4 * C}, 0, 4 * C);
      merges.push_back(m);
      C *= 2; Hs /= 2;
    }
  }
  Cf = C; Hf = Hs;
  fn_g = add("norm.weight", {C}, 0, C);
  fn_b = add("norm.bias", {C}, 0, C);
  head = add_lin("head", C, cfg.num_classes);

  int rc;
  if ((rc = dalloc(&P, n_flat * 4, true)) || (rc = dalloc(&G, n_flat * 4, true)) || (rc = dalloc(&M1, n_flat * 4, true)) ||
      (rc = dalloc(&M2, n_flat * 4, true)) || (rc = dalloc(&Pw, n_flat * 2, true)) || (rc = dalloc(&WT, n_wt * 2, true)))
    return rc;
  const size_t B = cfg.max_batch, I = cfg.image;
  auto act = [&](__nv_bfloat16** p, size_t elems) { return dalloc(p, elems * 2, true); };
  if ((rc = dalloc(&stage_images, B * 3 * I * I * 4)) || (rc = dalloc(&stage_labels, B * 8))) return rc;
  const size_t T0 = B * S0 * S0;
  if ((rc = act(&x_img, B * I * I * 8)) || (rc = act(&e0, T0 * cfg.embed)) || (rc = act(&x0, T0 * cfg.embed))) return rc;
  if ((rc = dalloc(&pe_m, T0 * 4)) || (rc = dalloc(&pe_r, T0 * 4))) return rc;
  size_t maxTC = T0 * cfg.embed, maxZLL = 0, maxTable = 0;
  for (Blk& k : blocks) {
    const size_t T = B * k.Hs * k.Hs, TC = T * k.C, Z = T / L * k.heads;
    if ((rc = act(&k.ln1o, TC)) || (rc = act(&k.qw, TC)) || (rc = act(&k.kw, TC)) || (rc = act(&k.vw, TC)) ||
        (rc = act(&k.Pm, Z * L * LP)) || (rc = act(&k.att, TC)) || (rc = act(&k.x2, TC)) || (rc = act(&k.ln2o, TC)) ||
        (rc = act(&k.h, 4 * TC)) || (rc = act(&k.g, 4 * TC)) || (rc = act(&k.xout, TC)))
      return rc;
    if ((rc = dalloc(&k.m1, T * 4)) || (rc = dalloc(&k.r1, T * 4)) || (rc = dalloc(&k.m2, T * 4)) || (rc = dalloc(&k.r2, T * 4)))
      return rc;
    if (TC > maxTC) maxTC = TC;
    if (Z * L * LP > maxZLL) maxZLL = Z * L * LP;
    if ((size_t)k.heads * L * L > maxTable) maxTable = (size_t)k.heads * L * L;
  }
  for (Merge& m : merges) {
    const size_t T = B * (m.Hs / 2) * (m.Hs / 2);
    if ((rc = act(&m.merged, T * 4 * m.C)) || (rc = act(&m.lno, T * 4 * m.C)) || (rc = act(&m.out, T * 2 * m.C))) return rc;
    if ((rc = dalloc(&m.m, T * 4)) || (rc = dalloc(&m.r, T * 4))) return rc;
  }
  const size_t Tf = B * Hf * Hf;
  if ((rc = act(&fno, Tf * Cf)) || (rc = act(&pooled, B * Cf)) || (rc = act(&logits, B * cfg.num_classes)) ||
      (rc = act(&dlogits, B * cfg.num_classes)) || (rc = act(&dpool, B * Cf)))
    return rc;
  if ((rc = dalloc(&fn_m, Tf * 4)) || (rc = dalloc(&fn_r, Tf * 4)) || (rc = dalloc(&row_loss, B * 4)) ||
      (rc = dalloc(&loss_acc, 256, true)) || (rc = dalloc(&relbias, maxTable * 4)) || (rc = dalloc(&dbias, maxTable * 4)))
    return rc;
  const size_t padTC = maxTC * LP / L + 4096;  // [Z][D][LP] buffers
  if ((rc = act(&dxa, maxTC)) || (rc = act(&dxb, maxTC)) || (rc = act(&dqkv, 3 * maxTC)) || (rc = act(&dP, maxZLL)) ||
      (rc = act(&tP, maxZLL)) || (rc = act(&tA, padTC)) || (rc = act(&tB, padTC)) || (rc = act(&dOh, maxTC)) ||
      (rc = act(&dqw, maxTC)) || (rc = act(&dkw, maxTC)) || (rc = act(&dvw, maxTC)) || (rc = act(&dh, 4 * maxTC)) ||
      (rc = act(&dg, 4 * maxTC)) || (rc = act(&datt, maxTC)) || (rc = act(&dln, 4 * maxTC)) || (rc = act(&ow, maxTC)))
    return rc;
  size_t sb = layernorm_bwd_scratch_bytes(4 * Cf);
  if (colsum_scratch_bytes(4 * Cf) > sb) sb = colsum_scratch_bytes(4 * Cf);
  auto wg = [&](const srt_conv_desc& d) {
    const size_t b = conv_wgrad_scratch_bytes(d, SRT_BF16, SRT_IMPL_AUTO);
    if (b > sb) sb = b;
  };
  wg(pe_desc((int)B));
  for (Blk& k : blocks) {
    const int64_t T = (int64_t)B * k.Hs * k.Hs;
    wg(lin_desc(T, k.C, 3 * k.C)); wg(lin_desc(T, k.C, k.C)); wg(lin_desc(T, k.C, 4 * k.C)); wg(lin_desc(T, 4 * k.C, k.C));
  }
  for (Merge& m : merges) wg(lin_desc((int64_t)B * (m.Hs / 2) * (m.Hs / 2), 4 * m.C, 2 * m.C));
  wg(lin_desc((int64_t)B, Cf, cfg.num_classes));
  scratch_bytes = sb;
  if ((rc = dalloc((char**)&scratch, scratch_bytes))) return rc;
  if ((rc = dalloc((char**)&scratch_side, scratch_bytes))) return rc;
  {
    std::vector<size_t> starts;
    for (Blk& k : blocks) starts.push_back(params[k.n1g].off);
    if ((rc = buckets.build(starts, n_flat, (size_t)25 << 18))) return rc;
  }
  SRT_CHECK_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
  {
    int lo = 0, hi = 0;
    SRT_CHECK_CUDA(cudaDeviceGetStreamPriorityRange(&lo, &hi));
    SRT_CHECK_CUDA(cudaStreamCreateWithPriority(&side, cudaStreamNonBlocking, lo));
    SRT_CHECK_CUDA(cudaEventCreateWithFlags(&ev_fork, cudaEventDisableTiming));
    SRT_CHECK_CUDA(cudaEventCreateWithFlags(&ev_join, cudaEventDisableTiming));
  }
  return SRT_OK;
}

// Transposed copies of the linear weights for the data gradients (after the bf16 working copy changed).
int Swin::transposes() {
  int rc;
  auto tr = [&](const Lin& l) { return filter_transpose(SRT_BF16, pw(l.w), WT + l.wt_off, l.out, 1, l.in, stream); };
  for (Blk& k : blocks)
    if ((rc = tr(k.qkv)) || (rc = tr(k.proj)) || (rc = tr(k.fc)) || (rc = tr(k.fc2))) return rc;
  for (Merge& m : merges)
    if ((rc = tr(m.red))) return rc;
  return tr(head);
}

int Swin::block_fwd(Blk& k, const __nv_bfloat16* x, int B) {
  const int64_t T = (int64_t)B * k.Hs * k.Hs;
  const int C = k.C, D = k.D, Hh = k.heads;
  const int nWin = (int)(T / L);
  const WindowShape w = {B, k.Hs, k.Hs, WS, k.shift};
  const float scale = 1.f / sqrtf((float)D);
  int rc;
  if ((rc = layernorm_fwd(x, pf(k.n1g), pf(k.n1b), k.ln1o, k.m1, k.r1, T, C, cfg.ln_eps, stream))) return rc;
  if ((rc = linear_fwd(k.qkv, k.ln1o, dqkv, nullptr, T))) return rc;   // dqkv doubles as the forward staging buffer
  if ((rc = window_qkv(dqkv, k.qw, k.kw, k.vw, w, Hh, D, 0, stream))) return rc;
  const long long hs = (long long)L * D, ws = (long long)Hh * L * D;
  BgemmDesc sc = {L, LP, D, Hh, nWin, D, hs, ws, D, hs, ws, LP, (long long)L * LP, (long long)Hh * L * LP, scale, 0, 0};
  if ((rc = bgemm_bf16(sc, k.qw, k.kw, k.Pm, stream))) return rc;
  if ((rc = relbias_build(pf(k.table), relbias, Hh, WS, stream))) return rc;
  if ((rc = window_softmax_fwd(k.Pm, relbias, w, Hh, LP, stream))) return rc;
  if ((rc = transpose_pad(k.vw, tA, L, D, D, hs, (int64_t)nWin * Hh, LP, stream))) return rc;   // V^T [z][D][LP]
  BgemmDesc av = {L, D, LP, Hh, nWin, LP, (long long)L * LP, (long long)Hh * L * LP, LP, (long long)D * LP,
                  (long long)Hh * D * LP, C, D, (long long)L * C, 1.f, 0, 0};
  if ((rc = bgemm_bf16(av, k.Pm, tA, ow, stream))) return rc;                               // [win][tok][C]
  if ((rc = window_permute(ow, k.att, w, C, 1, stream))) return rc;
  if ((rc = linear_fwd(k.proj, k.att, k.x2, x, T))) return rc;
  if ((rc = layernorm_fwd(k.x2, pf(k.n2g), pf(k.n2b), k.ln2o, k.m2, k.r2, T, C, cfg.ln_eps, stream))) return rc;
  if ((rc = linear_fwd(k.fc, k.ln2o, k.h, nullptr, T))) return rc;
  if ((rc = gelu_erf_fwd(k.h, k.g, T * 4 * C, stream))) return rc;
  return linear_fwd(k.fc2, k.g, k.xout, k.x2, T);
}

// dx: gradient w.r.t. the block's output on entry, w.r.t. its input on return (the two buffers swap roles).
int Swin::block_bwd(Blk& k, const __nv_bfloat16* xin, __nv_bfloat16*& dx, __nv_bfloat16*& dx_other, int B) {
  const int64_t T = (int64_t)B * k.Hs * k.Hs;
  const int C = k.C, D = k.D, Hh = k.heads;
  const int nWin = (int)(T / L);
  const int64_t Z = (int64_t)nWin * Hh;
  const WindowShape w = {B, k.Hs, k.Hs, WS, k.shift};
  const float scale = 1.f / sqrtf((float)D);
  const long long hs = (long long)L * D, ws = (long long)Hh * L * D, ps = (long long)L * LP, pws = (long long)Hh * L * LP,
                  ts = (long long)D * LP, tws = (long long)Hh * D * LP;
  int rc;
  if ((rc = linear_bwd(k.fc2, dx, k.g, dg, T))) return rc;
  if ((rc = gelu_erf_bwd(dg, k.h, dh, T * 4 * C, stream))) return rc;
  if ((rc = linear_bwd(k.fc, dh, k.ln2o, dln, T))) return rc;
  if ((rc = layernorm_bwd(dln, k.x2, pf(k.n2g), k.m2, k.r2, dx, dx_other, gf(k.n2g), gf(k.n2b), T, C, scratch, scratch_bytes,
                          stream)))
    return rc;  // dx_other: gradient w.r.t. x2
  if ((rc = linear_bwd(k.proj, dx_other, k.att, datt, T))) return rc;
  if ((rc = window_qkv(datt, dOh, nullptr, nullptr, w, Hh, D, 0, stream))) return rc;          // dO [win][head][tok][D]
  // dP = dO V^T
  BgemmDesc dp = {L, LP, D, Hh, nWin, D, hs, ws, D, hs, ws, LP, ps, pws, 1.f, 0, 0};
  if ((rc = bgemm_bf16(dp, dOh, k.vw, dP, stream))) return rc;
  // dV = P^T dO
  if ((rc = transpose_pad(k.Pm, tP, L, L, LP, ps, Z, LP, stream))) return rc;
  if ((rc = transpose_pad(dOh, tA, L, D, D, hs, Z, LP, stream))) return rc;
  BgemmDesc dv = {L, D, LP, Hh, nWin, LP, ps, pws, LP, ts, tws, D, hs, ws, 1.f, 0, 0};
  if ((rc = bgemm_bf16(dv, tP, tA, dvw, stream))) return rc;
  // dS, table gradient
  if ((rc = window_softmax_bwd(k.Pm, dP, Z, L, LP, stream))) return rc;
  if ((rc = relbias_grad(dP, dbias, gf(k.table), nWin, Hh, WS, LP, stream))) return rc;
  // dQ = dS K * scale, dK = dS^T Q * scale
  if ((rc = transpose_pad(k.kw, tA, L, D, D, hs, Z, LP, stream))) return rc;
  BgemmDesc dq = {L, D, LP, Hh, nWin, LP, ps, pws, LP, ts, tws, D, hs, ws, scale, 0, 0};
  if ((rc = bgemm_bf16(dq, dP, tA, dqw, stream))) return rc;
  if ((rc = transpose_pad(dP, tP, L, L, LP, ps, Z, LP, stream))) return rc;
  if ((rc = transpose_pad(k.qw, tB, L, D, D, hs, Z, LP, stream))) return rc;
  if ((rc = bgemm_bf16(dq, tP, tB, dkw, stream))) return rc;
  if ((rc = window_qkv(dqkv, dqw, dkw, dvw, w, Hh, D, 1, stream))) return rc;
  if ((rc = linear_bwd(k.qkv, dqkv, k.ln1o, dln, T))) return rc;
  if ((rc = join_side())) return rc;  // the next kernel overwrites dx, which this block's first weight gradient read
  return layernorm_bwd(dln, xin, pf(k.n1g), k.m1, k.r1, dx_other, dx, gf(k.n1g), gf(k.n1b), T, C, scratch, scratch_bytes,
                       stream);
}

int Swin::forward(int B) {
  const int S0 = cfg.image / cfg.patch;
  int rc;
  if ((rc = join_side())) return rc;
  if ((rc = nchw_to_nhwc(SRT_BF16, stage_images, x_img, B, 3, cfg.image, cfg.image, 8, stream))) return rc;
  srt_conv_epilogue ep = {pf(pe_b), nullptr};
  if ((rc = conv_fprop(pe_desc(B), SRT_BF16, SRT_IMPL_AUTO, x_img, pw(pe_w), e0, &ep, stream))) return rc;
  const int64_t T0 = (int64_t)B * S0 * S0;
  if ((rc = layernorm_fwd(e0, pf(pe_ng), pf(pe_nb), x0, pe_m, pe_r, T0, cfg.embed, cfg.ln_eps, stream))) return rc;
  const __nv_bfloat16* x = x0;
  int b0 = 0;
  for (int s = 0; s < 4; ++s) {
    for (int i = b0; i < stage_end[s]; ++i) {
      if ((rc = part.follow(stream, side))) return rc;
      if ((rc = block_fwd(blocks[i], x, B))) return rc;
      x = blocks[i].xout;
    }
    b0 = stage_end[s];
    if (s < 3) {
      Merge& m = merges[s];
      const int64_t T = (int64_t)B * (m.Hs / 2) * (m.Hs / 2);
      if ((rc = patch_merge(x, m.merged, B, m.Hs, m.Hs, m.C, 0, stream))) return rc;
      if ((rc = layernorm_fwd(m.merged, pf(m.ng), pf(m.nb), m.lno, m.m, m.r, T, 4 * m.C, cfg.ln_eps, stream))) return rc;
      if ((rc = linear_fwd(m.red, m.lno, m.out, nullptr, T))) return rc;
      x = m.out;
    }
  }
  const int64_t Tf = (int64_t)B * Hf * Hf;
  if ((rc = layernorm_fwd(x, pf(fn_g), pf(fn_b), fno, fn_m, fn_r, Tf, Cf, cfg.ln_eps, stream))) return rc;
  if ((rc = avgpool_fwd(SRT_BF16, fno, pooled, B, Hf * Hf, Cf, stream))) return rc;
  return linear_fwd(head, pooled, logits, nullptr, B);
}

int Swin::backward(int B, int global_batch) {
  int rc;
  last_global = global_batch;
  buckets.begin_backward();
  if ((rc = softmax_ce(SRT_BF16, logits, stage_labels, B, cfg.num_classes, 1.f / (float)global_batch, row_loss, dlogits, stream)))
    return rc;
  if ((rc = sum_f32(row_loss, B, loss_acc, 0, stream))) return rc;
  if ((rc = linear_bwd(head, dlogits, pooled, dpool, B))) return rc;
  const int64_t Tf = (int64_t)B * Hf * Hf;
  if ((rc = avgpool_bwd(SRT_BF16, dpool, dln, B, Hf * Hf, Cf, stream))) return rc;
  const __nv_bfloat16* x_last = blocks.back().xout;
  __nv_bfloat16 *dx = dxa, *dx_other = dxb;
  if ((rc = layernorm_bwd(dln, x_last, pf(fn_g), fn_m, fn_r, nullptr, dx, gf(fn_g), gf(fn_b), Tf, Cf, scratch, scratch_bytes,
                          stream)))
    return rc;
  for (int s = 3; s >= 0; --s) {
    const int first = s == 0 ? 0 : stage_end[s - 1];
    for (int i = stage_end[s] - 1; i >= first; --i) {
      const __nv_bfloat16* xin = i > first ? blocks[i - 1].xout : (s == 0 ? x0 : merges[s - 1].out);
      if ((rc = part.follow(stream, side))) return rc;
      if ((rc = block_bwd(blocks[i], xin, dx, dx_other, B))) return rc;
      if ((rc = buckets.unit_done(i, stream))) return rc;
    }
    if (s > 0) {
      Merge& m = merges[s - 1];
      const int64_t T = (int64_t)B * (m.Hs / 2) * (m.Hs / 2);
      if ((rc = linear_bwd(m.red, dx, m.lno, dln, T))) return rc;
      if ((rc = layernorm_bwd(dln, m.merged, pf(m.ng), m.m, m.r, nullptr, dh, gf(m.ng), gf(m.nb), T, 4 * m.C, scratch,
                              scratch_bytes, stream)))
        return rc;
      if ((rc = join_side())) return rc;  // dx was read by the reduction's weight gradient
      if ((rc = patch_merge(dh, dx, B, m.Hs, m.Hs, m.C, 1, stream))) return rc;   // back to the finer map
    }
  }
  // patch embedding: LayerNorm, then the convolution's filter and bias gradients
  if ((rc = join_side())) return rc;
  const int S0 = cfg.image / cfg.patch;
  const int64_t T0 = (int64_t)B * S0 * S0;
  if ((rc = layernorm_bwd(dx, e0, pf(pe_ng), pe_m, pe_r, nullptr, dx_other, gf(pe_ng), gf(pe_nb), T0, cfg.embed, scratch,
                          scratch_bytes, stream)))
    return rc;
  if ((rc = colsum_bf16(dx_other, T0, cfg.embed, gf(pe_b), scratch, scratch_bytes, stream))) return rc;
  if ((rc = conv_wgrad(pe_desc(B), SRT_BF16, SRT_IMPL_AUTO, dx_other, x_img, gf(pe_w), scratch, scratch_bytes, stream))) return rc;
  return buckets.all_done(stream);
}

}  // namespace srt

using namespace srt;

extern "C" {

int srt_swin_create(const srt_swin_config* cfg, srt_swin** out) {
  SRT_REQUIRE(cfg && out, "swin_create: null argument");
  Swin* g = new Swin();
  g->cfg = *cfg;
  int rc = g->build();
  if (rc == SRT_OK) rc = cudaStreamSynchronize(g->stream) == cudaSuccess ? SRT_OK : SRT_ERR_CUDA;
  if (rc != SRT_OK) { delete g; return rc; }
  *out = (srt_swin*)g;
  return SRT_OK;
}

int srt_swin_destroy(srt_swin* h) {
  if (!h) return SRT_OK;
  Swin* g = (Swin*)h;
  cudaStreamSynchronize(g->stream);
  delete g;
  return SRT_OK;
}

int srt_swin_num_params(srt_swin* h) { return h ? (int)((Swin*)h)->params.size() : -1; }

int srt_swin_param_info(srt_swin* h, int idx, char* name, int name_cap, int64_t shape[4], int* ndim) {
  Swin* g = (Swin*)h;
  SRT_REQUIRE(g && idx >= 0 && idx < (int)g->params.size(), "swin_param_info: bad index");
  const Swin::Rec& r = g->params[idx];
  if (name && name_cap > 0) { strncpy(name, r.name.c_str(), name_cap - 1); name[name_cap - 1] = 0; }
  if (shape) for (int i = 0; i < 4; ++i) shape[i] = r.shape[i];
  if (ndim) *ndim = r.ndim;
  return SRT_OK;
}

// Host arrays use torchvision's shapes (the patch-embedding filter is [K][C][R][S]).
int srt_swin_set_param(srt_swin* h, int idx, const float* host) {
  Swin* g = (Swin*)h;
  SRT_REQUIRE(g && host && idx >= 0 && idx < (int)g->params.size(), "swin_set_param: bad argument");
  const Swin::Rec& r = g->params[idx];
  if (r.kind == 2) {
    const int K = (int)r.shape[0], C = (int)r.shape[1], R = (int)r.shape[2], S = (int)r.shape[3];
    std::vector<float> t((size_t)K * R * S * r.cpad, 0.f);
    for (int k = 0; k < K; ++k)
      for (int c = 0; c < C; ++c)
        for (int a = 0; a < R; ++a)
          for (int b = 0; b < S; ++b)
            t[(((size_t)k * R + a) * S + b) * r.cpad + c] = host[(((size_t)k * C + c) * R + a) * S + b];
    SRT_CHECK_CUDA(cudaMemcpy(g->P + r.off, t.data(), t.size() * 4, cudaMemcpyHostToDevice));
  } else {
    SRT_CHECK_CUDA(cudaMemcpy(g->P + r.off, host, r.count * 4, cudaMemcpyHostToDevice));
  }
  return SRT_OK;
}

int srt_swin_get_param(srt_swin* h, int idx, float* host, int which) {
  Swin* g = (Swin*)h;
  SRT_REQUIRE(g && host && idx >= 0 && idx < (int)g->params.size(), "swin_get_param: bad argument");
  const Swin::Rec& r = g->params[idx];
  SRT_CHECK_CUDA(cudaStreamSynchronize(g->stream));
  const float* base = which == SRT_GET_GRAD ? g->G : which == SRT_GET_MOMENTUM ? g->M1 : g->P;
  if (r.kind == 2) {
    const int K = (int)r.shape[0], C = (int)r.shape[1], R = (int)r.shape[2], S = (int)r.shape[3];
    std::vector<float> t((size_t)K * R * S * r.cpad);
    SRT_CHECK_CUDA(cudaMemcpy(t.data(), base + r.off, t.size() * 4, cudaMemcpyDeviceToHost));
    for (int k = 0; k < K; ++k)
      for (int c = 0; c < C; ++c)
        for (int a = 0; a < R; ++a)
          for (int b = 0; b < S; ++b)
            host[(((size_t)k * C + c) * R + a) * S + b] = t[(((size_t)k * R + a) * S + b) * r.cpad + c];
  } else {
    SRT_CHECK_CUDA(cudaMemcpy(host, base + r.off, r.count * 4, cudaMemcpyDeviceToHost));
  }
  return SRT_OK;
}

int srt_swin_commit_params(srt_swin* h) {
  Swin* g = (Swin*)h;
  SRT_REQUIRE(g, "swin_commit_params: null handle");
  int rc = cast_f32_to_bf16(g->P, g->Pw, (int64_t)g->n_flat, g->stream);
  if (rc == SRT_OK) rc = g->transposes();
  if (rc) return rc;
  SRT_CHECK_CUDA(cudaStreamSynchronize(g->stream));
  return SRT_OK;
}

// images: [B][3][image][image] fp32 (NCHW, as the reference's loader yields them), labels int64.
int srt_swin_upload_batch(srt_swin* h, const float* host_images, const int64_t* host_labels, int B) {
  Swin* g = (Swin*)h;
  SRT_REQUIRE(g && host_images && host_labels && B > 0 && B <= g->cfg.max_batch, "swin_upload_batch: bad argument");
  const size_t img = (size_t)B * 3 * g->cfg.image * g->cfg.image * 4;
  SRT_CHECK_CUDA(cudaMemcpyAsync(g->stage_images, host_images, img, cudaMemcpyHostToDevice, g->stream));
  SRT_CHECK_CUDA(cudaMemcpyAsync(g->stage_labels, host_labels, (size_t)B * 8, cudaMemcpyHostToDevice, g->stream));
  g->cur_B = B;
  return SRT_OK;
}

int srt_swin_forward_backward(srt_swin* h, int B, int global_batch) {
  Swin* g = (Swin*)h;
  SRT_REQUIRE(g && B > 0 && B == g->cur_B && global_batch >= B, "swin_forward_backward: upload this batch first");
  PartitionFollower::Scope sm_scope(g->part);
  int rc = g->forward(B);
  if (rc) return rc;
  return g->backward(B, global_batch);
}

int srt_swin_forward_only(srt_swin* h, int B) {
  Swin* g = (Swin*)h;
  SRT_REQUIRE(g && B > 0 && B == g->cur_B, "swin_forward_only: upload this batch first");
  PartitionFollower::Scope sm_scope(g->part);
  return g->forward(B);
}

int srt_swin_optimizer(srt_swin* h) {
  Swin* g = (Swin*)h;
  SRT_REQUIRE(g, "swin_optimizer: null handle");
  PartitionFollower::Scope sm_scope(g->part);
  g->opt_steps++;
  int rc = adamw(g->P, g->G, g->M1, g->M2, g->Pw, (int64_t)g->n_flat, g->cfg.lr, g->cfg.beta1, g->cfg.beta2, g->cfg.eps,
                 g->cfg.weight_decay, g->opt_steps, g->stream);
  if (rc) return rc;
  return g->transposes();
}

// Mean cross-entropy of the last micro-batch.
int srt_swin_loss(srt_swin* h, float* host_loss) {
  Swin* g = (Swin*)h;
  SRT_REQUIRE(g && host_loss && g->cur_B > 0 && g->last_global > 0, "swin_loss: nothing has run");
  float sum = 0.f;
  SRT_CHECK_CUDA(cudaMemcpyAsync(&sum, g->loss_acc, 4, cudaMemcpyDeviceToHost, g->stream));
  SRT_CHECK_CUDA(cudaStreamSynchronize(g->stream));
  *host_loss = sum * (float)g->last_global / (float)g->cur_B;  // the rows carry the 1/global_batch gradient scale
  return SRT_OK;
}

int srt_swin_logits(srt_swin* h, float* host, int B) {
  Swin* g = (Swin*)h;
  SRT_REQUIRE(g && host && B > 0 && B <= g->cfg.max_batch, "swin_logits: bad argument");
  const size_t n = (size_t)B * g->cfg.num_classes;
  std::vector<uint16_t> tmp(n);
  SRT_CHECK_CUDA(cudaStreamSynchronize(g->stream));
  SRT_CHECK_CUDA(cudaMemcpy(tmp.data(), g->logits, n * 2, cudaMemcpyDeviceToHost));
  for (size_t i = 0; i < n; ++i) {
    const uint32_t bits = (uint32_t)tmp[i] << 16;
    memcpy(&host[i], &bits, 4);
  }
  return SRT_OK;
}

int srt_swin_follow_infer_tpc(srt_swin* h, srt_comm* comm, int device, int min_train_tpc, int max_train_tpc, int enable) {
  Swin* g = (Swin*)h;
  SRT_REQUIRE(g, "swin_follow_infer_tpc: null handle");
  { int dev = 0; SRT_CHECK_CUDA(cudaGetDevice(&dev)); g->part.device = dev; }
  return g->part.configure(g->stream, g->side, comm, device, min_train_tpc, max_train_tpc, enable != 0);
}

int srt_swin_current_sms(srt_swin* h) { if (!h) return -1;
  const int w = ((Swin*)h)->part.cur_sms;
  return w ? w : PartitionFollower::device_sm_count(); }

int srt_swin_synchronize(srt_swin* h) {
  Swin* g = (Swin*)h;
  SRT_REQUIRE(g, "swin_synchronize: null handle");
  SRT_CHECK_CUDA(cudaStreamSynchronize(g->stream));
  return SRT_OK;
}

void* srt_swin_grad_buckets(srt_swin* h) { return h ? (void*)&((Swin*)h)->buckets : nullptr; }

int srt_swin_grad_buffer(srt_swin* h, void** ptr, int64_t* n) {
  Swin* g = (Swin*)h;
  SRT_REQUIRE(g && ptr && n, "swin_grad_buffer: null argument");
  *ptr = g->G;
  *n = (int64_t)g->n_flat;
  return SRT_OK;
}

void* srt_swin_stream(srt_swin* h) { return h ? (void*)((Swin*)h)->stream : nullptr; }
int64_t srt_swin_memory_bytes(srt_swin* h) { return h ? (int64_t)((Swin*)h)->bytes_total : -1; }

}  // extern "C"
