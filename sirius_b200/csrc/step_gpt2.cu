// Training step of a GPT-2 style decoder (the reference trains transformers.GPT2LMHeadModel,
// train/gpt2.py:26,90-97): token + position embedding, n_layer x [LayerNorm, fused QKV projection, causal
// multi-head attention, output projection, LayerNorm, MLP with tanh-GELU], final LayerNorm, output
// projection tied to the token table, next-token cross-entropy, AdamW.
//
// Data layout: activations are [tokens][features] bf16 rows (tokens = batch * seq); every linear layer is
// a 1x1 convolution over that matrix and runs on the tcgen05 implicit-GEMM kernels (bias and residual
// add in the epilogue); attention products are batched tcgen05 GEMMs that address the heads inside the
// fused [tokens][3*d] projection through 4-D tensor maps; parameters, gradients and both AdamW moments are
// flat fp32 buffers with a bf16 working copy. Linear weights are stored [out][in] (the reference's Conv1D
// keeps [in][out]; set/get transpose).
#include <string.h>

#include <algorithm>
#include <numeric>
#include <string>
#include <vector>

#include "../../include/sirius_b200.h"
#include "../../include/sirius_pool.h"
#include <atomic>
#include "common.cuh"
#include "grad_buckets.cuh"
#include "ops.cuh"
#include "partition_follow.cuh"

namespace srt {

namespace {
inline size_t up(size_t v, size_t a) { return (v + a - 1) / a * a; }
}

struct Gpt2 {
  srt_gpt2_config cfg;
  int C, H, D, V, Vpad, S, L;
  cudaStream_t stream = nullptr;

  struct Rec { std::string name; size_t off, count; int64_t shape[2]; int ndim; int kind; };  // kind 1 = linear [in][out] outside
  std::vector<Rec> params;
  size_t n_flat = 0;
  float *P = nullptr, *G = nullptr, *M1 = nullptr, *M2 = nullptr;
  __nv_bfloat16 *Pw = nullptr, *WT = nullptr;  // bf16 copy; per-linear transposes [in][out] for the data gradients
  int opt_steps = 0;

  struct Lin { int w, b, in, out; size_t wt_off; };
  struct Layer {
    int ln1_g, ln1_b, ln2_g, ln2_b;
    Lin qkv, proj, fc, fc2;
    // saved activations
    __nv_bfloat16 *ln1o, *qkv_o, *Pm, *att, *x2, *ln2o, *h, *g, *xout;
    float *ln1_mean, *ln1_rstd, *ln2_mean, *ln2_rstd;
  };
  std::vector<Layer> layers;
  int wte, wpe, lnf_g, lnf_b;
  size_t wte_wt_off = 0, n_wt = 0;

  // activations / scratch
  __nv_bfloat16 *x0 = nullptr, *lnfo = nullptr, *logits = nullptr;
  float *lnf_mean = nullptr, *lnf_rstd = nullptr, *row_loss = nullptr, *loss_acc = nullptr;
  __nv_bfloat16 *dxa = nullptr, *dxb = nullptr, *dqkv = nullptr, *dP = nullptr, *Tbig = nullptr, *t1 = nullptr, *t2 = nullptr,
                *dh = nullptr, *dg = nullptr, *datt = nullptr, *dln = nullptr;
  void* scratch = nullptr;
  size_t scratch_bytes = 0;
  int32_t *ids = nullptr, *labels = nullptr, *order = nullptr, *seg = nullptr;
  int n_unique = 0, cur_B = 0;
  std::vector<void*> allocs;
  size_t bytes_total = 0;
  // Releasable part (everything sized by the batch): from the training allocator of a page pool when one is
  // attached, so that shrinking the batch hands whole pages to the inference side (as the ResNet executor does).
  srt_pool* pool = nullptr;
  std::vector<void*> act_blocks;
  size_t act_bytes = 0;
  int act_batch = 0;
  float* ACC = nullptr;      // gradients accumulated over the micro-batches of a global batch
  int accum_pending = 0;
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
  GradBuckets buckets;
  std::atomic<int> abort_flag{0};
  static constexpr int kAhead = 4;  // layers the host may run ahead of the GPU (bounds the drain after a kill)
  cudaEvent_t ahead_ev[kAhead] = {nullptr};
  unsigned long long layer_seq = 0;

  ~Gpt2() {
    if (part.home_stream) { stream = part.home_stream; side = part.home_side; }  // partition streams belong to the ladder
    release_activations(nullptr);
    for (auto e : ahead_ev) if (e) cudaEventDestroy(e);
    if (ev_fork) cudaEventDestroy(ev_fork);
    if (ev_join) cudaEventDestroy(ev_join);
    if (side) { cudaStreamSynchronize(side); cudaStreamDestroy(side); }
    for (void* p : allocs) cudaFree(p);
    if (stream) cudaStreamDestroy(stream);
  }
  int aalloc(void** out, size_t bytes) {
    bytes = up(bytes ? bytes : 256, 256);
    if (pool) {
      int rc = srt_pool_alloc(pool, SRT_POOL_TRAIN, bytes, out);
      if (rc) return rc;
    } else {
      SRT_CHECK_CUDA(cudaMalloc(out, bytes));
    }
    act_blocks.push_back(*out);
    act_bytes += bytes;
    return SRT_OK;
  }
  int free_activation_blocks() {
    if (stream && !act_blocks.empty()) SRT_CHECK_CUDA(cudaStreamSynchronize(stream));
    if (side && !act_blocks.empty()) SRT_CHECK_CUDA(cudaStreamSynchronize(side));  // an aborted backward never joined
    side_dirty = false;
    for (void* p : act_blocks) {
      if (pool) { int rc = srt_pool_free(pool, SRT_POOL_TRAIN, p); if (rc) return rc; }
      else cudaFree(p);
    }
    act_blocks.clear();
    act_bytes = 0;
    act_batch = 0;
    return SRT_OK;
  }
  int release_activations(size_t* released) {
    if (released) *released = 0;
    if (act_blocks.empty()) { act_batch = 0; return SRT_OK; }
    size_t freed = act_bytes;
    int rc = free_activation_blocks();
    if (rc) return rc;
    if (pool && (rc = srt_pool_empty_cache(pool, SRT_POOL_TRAIN, &freed))) return rc;
    if (released) *released = freed;
    return SRT_OK;
  }
  int alloc_activations(int B);
  int shrink_activations(int B, size_t* released) {
    if (released) *released = 0;
    if (B <= 0) return release_activations(released);
    SRT_REQUIRE(B <= cfg.max_batch, "gpt2 shrink_activations: batch %d above max_batch %d", B, cfg.max_batch);
    const size_t before = act_bytes;
    int rc = free_activation_blocks();
    if (rc) return rc;
    if ((rc = alloc_activations(B))) return rc;
    size_t freed = before > act_bytes ? before - act_bytes : 0;
    if (pool && (rc = srt_pool_empty_cache(pool, SRT_POOL_TRAIN, &freed))) return rc;
    if (released) *released = freed;
    return SRT_OK;
  }
  // Between layers: kill-batch flag and bounded launch-ahead.
  int checkpoint() {
    if (abort_flag.load(std::memory_order_acquire)) {
      set_error("step aborted between layers (kill batch)");
      return SRT_ERR_ABORTED;
    }
    if (int rc = part.follow(stream, side)) return rc;
    const int slot = (int)(layer_seq % kAhead);
    if (!ahead_ev[slot]) SRT_CHECK_CUDA(cudaEventCreateWithFlags(&ahead_ev[slot], cudaEventDisableTiming));
    else if (layer_seq >= (unsigned long long)kAhead) SRT_CHECK_CUDA(cudaEventSynchronize(ahead_ev[slot]));
    SRT_CHECK_CUDA(cudaEventRecord(ahead_ev[slot], stream));
    ++layer_seq;
    return SRT_OK;
  }
  template <class T>
  int dalloc(T** out, size_t bytes, bool zero = false) {
    bytes = up(bytes ? bytes : 256, 256);
    SRT_CHECK_CUDA(cudaMalloc((void**)out, bytes));
    allocs.push_back((void*)*out);
    bytes_total += bytes;
    if (zero) SRT_CHECK_CUDA(cudaMemset(*out, 0, bytes));
    return SRT_OK;
  }
  int add(const std::string& name, int64_t a, int64_t b, int kind, size_t count) {
    Rec r;
    r.name = name; r.off = n_flat; r.count = count; r.shape[0] = a; r.shape[1] = b; r.ndim = b > 0 ? 2 : 1; r.kind = kind;
    n_flat += up(count, 64);
    params.push_back(r);
    return (int)params.size() - 1;
  }
  Lin add_lin(const std::string& pre, int in, int out) {
    Lin l;
    l.in = in; l.out = out;
    l.w = add(pre + ".weight", in, out, 1, (size_t)in * out);
    l.b = add(pre + ".bias", out, 0, 0, (size_t)out);
    l.wt_off = n_wt;
    n_wt += up((size_t)in * out, 64);
    return l;
  }
  float* pf(int i) { return P + params[i].off; }
  float* gf(int i) { return G + params[i].off; }
  __nv_bfloat16* pw(int i) { return Pw + params[i].off; }

  int build();
  int refresh();
  int forward(int B);
  int backward(int B, int global_batch);
  srt_conv_desc lin_desc(int64_t T, int in, int out) const { return {(int)T, 1, 1, in, out, 1, 1, 1, 0, 1, 1}; }
  int linear_fwd(const Lin& l, const void* x, void* y, const void* residual, int64_t T) {
    srt_conv_epilogue ep = {pf(l.b), residual};
    return conv_fprop(lin_desc(T, l.in, l.out), SRT_BF16, SRT_IMPL_AUTO, x, pw(l.w), y, &ep, stream);
  }
  // dx = dy W, dW = dy^T x, db = column sums of dy
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
      if ((rc = colsum_bf16(dy, T, l.out, gf(l.b), wscratch, scratch_bytes, ws))) return rc;
      if ((rc = conv_wgrad(lin_desc(T, l.in, l.out), SRT_BF16, SRT_IMPL_AUTO, dy, x, gf(l.w), wscratch, scratch_bytes, ws)))
        return rc;
    }
    if (dx) return conv_dgrad(lin_desc(T, l.in, l.out), SRT_BF16, SRT_IMPL_AUTO, dy, WT + l.wt_off, dx, nullptr, stream);
    return SRT_OK;
  }
};

int Gpt2::build() {
  C = cfg.d_model; H = cfg.n_head; V = cfg.vocab; S = cfg.seq; L = cfg.n_layer;
  SRT_REQUIRE(C > 0 && H > 0 && C % H == 0, "gpt2: d_model must be a multiple of n_head");
  D = C / H;
  SRT_REQUIRE(D % 8 == 0 && C % 64 == 0, "gpt2: head size must be a multiple of 8 and d_model of 64");
  SRT_REQUIRE(S % 8 == 0 && S <= cfg.ctx && cfg.max_batch > 0, "gpt2: seq must be a multiple of 8 and at most ctx");
  SRT_REQUIRE((long long)cfg.max_batch * H <= 65535, "gpt2: batch * heads too large");
  Vpad = (int)up((size_t)V, 64);
  wte = add("transformer.wte.weight", V, C, 0, (size_t)Vpad * C);
  wpe = add("transformer.wpe.weight", cfg.ctx, C, 0, (size_t)cfg.ctx * C);
  layers.resize(L);
  for (int i = 0; i < L; ++i) {
    const std::string pre = "transformer.h." + std::to_string(i);
    Layer& y = layers[i];
    y.ln1_g = add(pre + ".ln_1.weight", C, 0, 0, C);
    y.ln1_b = add(pre + ".ln_1.bias", C, 0, 0, C);
    y.qkv = add_lin(pre + ".attn.c_attn", C, 3 * C);
    y.proj = add_lin(pre + ".attn.c_proj", C, C);
    y.ln2_g = add(pre + ".ln_2.weight", C, 0, 0, C);
    y.ln2_b = add(pre + ".ln_2.bias", C, 0, 0, C);
    y.fc = add_lin(pre + ".mlp.c_fc", C, 4 * C);
    y.fc2 = add_lin(pre + ".mlp.c_proj", 4 * C, C);
  }
  lnf_g = add("transformer.ln_f.weight", C, 0, 0, C);
  lnf_b = add("transformer.ln_f.bias", C, 0, 0, C);
  wte_wt_off = n_wt;
  n_wt += up((size_t)Vpad * C, 64);

  int rc;
  if ((rc = dalloc(&P, n_flat * 4, true))) return rc;
  if ((rc = dalloc(&G, n_flat * 4, true))) return rc;
  if ((rc = dalloc(&M1, n_flat * 4, true))) return rc;
  if ((rc = dalloc(&M2, n_flat * 4, true))) return rc;
  if ((rc = dalloc(&Pw, n_flat * 2, true))) return rc;
  if ((rc = dalloc(&WT, n_wt * 2, true))) return rc;

  if ((rc = dalloc(&ACC, n_flat * 4, true))) return rc;
  // scratch: split partials of the largest filter gradient, norm / bias column partials (sized for max_batch)
  const size_t Tmax = (size_t)cfg.max_batch * S;
  size_t sb = layernorm_bwd_scratch_bytes(C);
  if (colsum_scratch_bytes(4 * C) > sb) sb = colsum_scratch_bytes(4 * C);
  auto wg = [&](int in, int out) {
    const size_t b = conv_wgrad_scratch_bytes(lin_desc((int64_t)Tmax, in, out), SRT_BF16, SRT_IMPL_AUTO);
    if (b > sb) sb = b;
  };
  wg(C, 3 * C); wg(C, C); wg(C, 4 * C); wg(4 * C, C); wg(C, Vpad);
  scratch_bytes = sb;
  if ((rc = dalloc((char**)&scratch, scratch_bytes))) return rc;
  if ((rc = dalloc((char**)&scratch_side, scratch_bytes))) return rc;
  if ((rc = dalloc(&ids, Tmax * 4)) || (rc = dalloc(&labels, Tmax * 4)) || (rc = dalloc(&order, Tmax * 4)) ||
      (rc = dalloc(&seg, (Tmax + 1) * 4)) || (rc = dalloc(&loss_acc, 256, true)))
    return rc;
  {
    std::vector<size_t> starts;
    for (Layer& y : layers) starts.push_back(params[y.ln1_g].off);
    if ((rc = buckets.build(starts, n_flat, (size_t)25 << 18))) return rc;  // 25 MiB of fp32 gradients per bucket
  }
  SRT_CHECK_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
  {
    int lo = 0, hi = 0;
    SRT_CHECK_CUDA(cudaDeviceGetStreamPriorityRange(&lo, &hi));
    SRT_CHECK_CUDA(cudaStreamCreateWithPriority(&side, cudaStreamNonBlocking, lo));
    SRT_CHECK_CUDA(cudaEventCreateWithFlags(&ev_fork, cudaEventDisableTiming));
    SRT_CHECK_CUDA(cudaEventCreateWithFlags(&ev_join, cudaEventDisableTiming));
  }
  return alloc_activations(cfg.max_batch);
}

// Everything sized by the batch: saved activations of every layer, logits, backward scratch.
int Gpt2::alloc_activations(int B) {
  SRT_REQUIRE(B > 0 && B <= cfg.max_batch, "gpt2 activations: batch %d outside 1..%d", B, cfg.max_batch);
  if (act_batch == B) return SRT_OK;
  int rc = free_activation_blocks();
  if (rc) return rc;
  const size_t T = (size_t)B * S, BH = (size_t)B * H;
  auto act = [&](__nv_bfloat16** p, size_t elems) { return aalloc((void**)p, elems * 2); };
  auto actf = [&](float** p, size_t elems) { return aalloc((void**)p, elems * 4); };
  if ((rc = act(&x0, T * C))) return rc;
  for (Layer& y : layers) {
    if ((rc = act(&y.ln1o, T * C)) || (rc = act(&y.qkv_o, T * 3 * C)) || (rc = act(&y.Pm, BH * S * S)) ||
        (rc = act(&y.att, T * C)) || (rc = act(&y.x2, T * C)) || (rc = act(&y.ln2o, T * C)) ||
        (rc = act(&y.h, T * 4 * C)) || (rc = act(&y.g, T * 4 * C)) || (rc = act(&y.xout, T * C)))
      return rc;
    if ((rc = actf(&y.ln1_mean, T)) || (rc = actf(&y.ln1_rstd, T)) || (rc = actf(&y.ln2_mean, T)) || (rc = actf(&y.ln2_rstd, T)))
      return rc;
  }
  if ((rc = act(&lnfo, T * C)) || (rc = act(&logits, T * Vpad))) return rc;
  if ((rc = actf(&lnf_mean, T)) || (rc = actf(&lnf_rstd, T)) || (rc = actf(&row_loss, T))) return rc;
  if ((rc = act(&dxa, T * C)) || (rc = act(&dxb, T * C)) || (rc = act(&dqkv, T * 3 * C)) || (rc = act(&dP, BH * S * S)) ||
      (rc = act(&Tbig, BH * S * S)) || (rc = act(&t1, T * C)) || (rc = act(&t2, T * C)) || (rc = act(&dh, T * 4 * C)) ||
      (rc = act(&dg, T * 4 * C)) || (rc = act(&datt, T * C)) || (rc = act(&dln, T * C)))
    return rc;
  act_batch = B;
  return SRT_OK;
}

// bf16 working copy and the transposed weights the data gradients read.
int Gpt2::refresh() {
  int rc;
  if ((rc = cast_f32_to_bf16(P, Pw, (int64_t)n_flat, stream))) return rc;
  auto tr = [&](const Lin& l) { return filter_transpose(SRT_BF16, pw(l.w), WT + l.wt_off, l.out, 1, l.in, stream); };
  for (Layer& y : layers)
    if ((rc = tr(y.qkv)) || (rc = tr(y.proj)) || (rc = tr(y.fc)) || (rc = tr(y.fc2))) return rc;
  return filter_transpose(SRT_BF16, pw(wte), WT + wte_wt_off, Vpad, 1, C, stream);
}

int Gpt2::forward(int B) {
  const int64_t T = (int64_t)B * S;
  const float scale = 1.f / sqrtf((float)D);
  int rc;
  if ((rc = join_side())) return rc;  // an aborted backward may have left weight-gradient kernels in flight
  if ((rc = embedding_fwd(ids, pf(wte), pf(wpe), x0, T, S, C, stream))) return rc;
  const __nv_bfloat16* x = x0;
  for (Layer& y : layers) {
    if ((rc = checkpoint())) return rc;
    if ((rc = layernorm_fwd(x, pf(y.ln1_g), pf(y.ln1_b), y.ln1o, y.ln1_mean, y.ln1_rstd, T, C, cfg.ln_eps, stream))) return rc;
    if ((rc = linear_fwd(y.qkv, y.ln1o, y.qkv_o, nullptr, T))) return rc;
    // scores = Q K^T / sqrt(D), lower triangle only
    BgemmDesc q = {S, S, D, H, B, 3LL * C, D, (long long)S * 3 * C, 3LL * C, D, (long long)S * 3 * C,
                   S, (long long)S * S, (long long)H * S * S, scale, 1, 0};
    if ((rc = bgemm_bf16(q, y.qkv_o, y.qkv_o + C, y.Pm, stream))) return rc;
    if ((rc = causal_softmax_fwd(y.Pm, (int64_t)B * H, S, stream))) return rc;
    // out = P V: B operand is V^T per head, [B][H][D][S]
    if ((rc = batched_transpose(y.qkv_o + 2 * C, t1, S, D, 3LL * C, D, (long long)S * 3 * C, H, B, stream))) return rc;
    BgemmDesc o = {S, D, S, H, B, S, (long long)S * S, (long long)H * S * S, S, (long long)D * S, (long long)H * D * S,
                   C, D, (long long)S * C, 1.f, 0, 1};
    if ((rc = bgemm_bf16(o, y.Pm, t1, y.att, stream))) return rc;
    if ((rc = linear_fwd(y.proj, y.att, y.x2, x, T))) return rc;                       // + residual
    if ((rc = layernorm_fwd(y.x2, pf(y.ln2_g), pf(y.ln2_b), y.ln2o, y.ln2_mean, y.ln2_rstd, T, C, cfg.ln_eps, stream))) return rc;
    if ((rc = linear_fwd(y.fc, y.ln2o, y.h, nullptr, T))) return rc;
    if ((rc = gelu_fwd(y.h, y.g, T * 4 * C, stream))) return rc;
    if ((rc = linear_fwd(y.fc2, y.g, y.xout, y.x2, T))) return rc;                     // + residual
    x = y.xout;
  }
  if ((rc = layernorm_fwd(x, pf(lnf_g), pf(lnf_b), lnfo, lnf_mean, lnf_rstd, T, C, cfg.ln_eps, stream))) return rc;
  // logits = lnf(x) wte^T over the padded vocabulary
  return conv_fprop(lin_desc(T, C, Vpad), SRT_BF16, SRT_IMPL_AUTO, lnfo, pw(wte), logits, nullptr, stream);
}

int Gpt2::backward(int B, int global_batch) {
  const int64_t T = (int64_t)B * S;
  const float scale = 1.f / sqrtf((float)D);
  int rc;
  buckets.begin_backward();
  // mean over the (S - 1) targets of every sequence of the global batch (micro-batches add up to it)
  const float gscale = 1.f / ((float)global_batch * (float)(S - 1));
  if ((rc = lm_cross_entropy(logits, labels, T, V, Vpad, gscale, row_loss, stream))) return rc;
  // loss of this micro-batch: sum of the rows times gscale, done by summing then scaling on read
  if ((rc = sum_f32(row_loss, (int)T, loss_acc, 0, stream))) return rc;
  // tied projection: dwte = dlogits^T lnf(x); d lnf(x) = dlogits wte
  if (side && overlap_wgrad) {
    SRT_CHECK_CUDA(cudaEventRecord(ev_fork, stream));
    SRT_CHECK_CUDA(cudaStreamWaitEvent(side, ev_fork, 0));
    side_dirty = true;
    PdlOff no_early_launch(true);
    if ((rc = conv_wgrad(lin_desc(T, C, Vpad), SRT_BF16, SRT_IMPL_AUTO, logits, lnfo, gf(wte), scratch_side, scratch_bytes, side)))
      return rc;
  } else if ((rc = conv_wgrad(lin_desc(T, C, Vpad), SRT_BF16, SRT_IMPL_AUTO, logits, lnfo, gf(wte), scratch, scratch_bytes,
                              stream))) {
    return rc;
  }
  if ((rc = conv_dgrad(lin_desc(T, C, Vpad), SRT_BF16, SRT_IMPL_AUTO, logits, WT + wte_wt_off, dln, nullptr, stream))) return rc;
  const __nv_bfloat16* x_last = L > 0 ? layers[L - 1].xout : x0;
  if ((rc = layernorm_bwd(dln, x_last, pf(lnf_g), lnf_mean, lnf_rstd, nullptr, dxa, gf(lnf_g), gf(lnf_b), T, C, scratch,
                          scratch_bytes, stream)))
    return rc;
  __nv_bfloat16 *dx = dxa, *dx_other = dxb;  // dx = gradient w.r.t. the layer's output
  for (int i = L - 1; i >= 0; --i) {
    Layer& y = layers[i];
    const __nv_bfloat16* xin = i == 0 ? x0 : layers[i - 1].xout;
    if ((rc = checkpoint())) return rc;
    // MLP
    if ((rc = linear_bwd(y.fc2, dx, y.g, dg, T))) return rc;
    if ((rc = gelu_bwd(dg, y.h, dh, T * 4 * C, stream))) return rc;
    if ((rc = linear_bwd(y.fc, dh, y.ln2o, dln, T))) return rc;
    if ((rc = layernorm_bwd(dln, y.x2, pf(y.ln2_g), y.ln2_mean, y.ln2_rstd, dx, dx_other, gf(y.ln2_g), gf(y.ln2_b), T, C,
                            scratch, scratch_bytes, stream)))
      return rc;  // dx_other = gradient w.r.t. x2
    // attention output projection
    if ((rc = linear_bwd(y.proj, dx_other, y.att, datt, T))) return rc;
    // dP = dO V^T (lower triangle)
    BgemmDesc dp = {S, S, D, H, B, C, D, (long long)S * C, 3LL * C, D, (long long)S * 3 * C,
                    S, (long long)S * S, (long long)H * S * S, 1.f, 1, 0};
    if ((rc = bgemm_bf16(dp, datt, y.qkv_o + 2 * C, dP, stream))) return rc;
    // dV = P^T dO
    if ((rc = batched_transpose(y.Pm, Tbig, S, S, S, (long long)S * S, (long long)H * S * S, H, B, stream, 1))) return rc;
    if ((rc = batched_transpose(datt, t1, S, D, C, D, (long long)S * C, H, B, stream))) return rc;
    BgemmDesc dv = {S, D, S, H, B, S, (long long)S * S, (long long)H * S * S, S, (long long)D * S, (long long)H * D * S,
                    3LL * C, D, (long long)S * 3 * C, 1.f, 0, 2};
    if ((rc = bgemm_bf16(dv, Tbig, t1, dqkv + 2 * C, stream))) return rc;
    // dS = softmax backward, in place over dP
    if ((rc = causal_softmax_bwd(y.Pm, dP, (int64_t)B * H, S, stream))) return rc;
    // dQ = dS K / sqrt(D)
    if ((rc = batched_transpose(y.qkv_o + C, t1, S, D, 3LL * C, D, (long long)S * 3 * C, H, B, stream))) return rc;
    BgemmDesc dq = {S, D, S, H, B, S, (long long)S * S, (long long)H * S * S, S, (long long)D * S, (long long)H * D * S,
                    3LL * C, D, (long long)S * 3 * C, scale, 0, 1};
    if ((rc = bgemm_bf16(dq, dP, t1, dqkv, stream))) return rc;
    // dK = dS^T Q / sqrt(D)
    if ((rc = batched_transpose(dP, Tbig, S, S, S, (long long)S * S, (long long)H * S * S, H, B, stream, 1))) return rc;
    if ((rc = batched_transpose(y.qkv_o, t2, S, D, 3LL * C, D, (long long)S * 3 * C, H, B, stream))) return rc;
    BgemmDesc dk = dq;
    dk.k_causal = 2;
    if ((rc = bgemm_bf16(dk, Tbig, t2, dqkv + C, stream))) return rc;
    // fused projection and the first LayerNorm; dx becomes the gradient w.r.t. the layer's input
    if ((rc = linear_bwd(y.qkv, dqkv, y.ln1o, dln, T))) return rc;
    if ((rc = join_side())) return rc;  // the next kernel overwrites dx, which this layer's first weight gradient read
    if ((rc = layernorm_bwd(dln, xin, pf(y.ln1_g), y.ln1_mean, y.ln1_rstd, dx_other, dx, gf(y.ln1_g), gf(y.ln1_b), T, C,
                            scratch, scratch_bytes, stream)))
      return rc;
    if ((rc = buckets.unit_done(i, stream))) return rc;
  }
  // embedding tables (the token table already holds the output projection's share)
  if ((rc = join_side())) return rc;
  if ((rc = embedding_bwd(dx, ids, order, seg, n_unique, gf(wte), gf(wpe), B, S, C, stream))) return rc;
  return buckets.all_done(stream);
}

}  // namespace srt

using namespace srt;

extern "C" {

int srt_gpt2_create(const srt_gpt2_config* cfg, srt_gpt2** out) { return srt_gpt2_create_with_pool(cfg, nullptr, out); }

int srt_gpt2_create_with_pool(const srt_gpt2_config* cfg, srt_pool* pool, srt_gpt2** out) {
  SRT_REQUIRE(cfg && out, "gpt2_create: null argument");
  Gpt2* g = new Gpt2();
  g->cfg = *cfg;
  g->pool = pool;
  int rc = g->build();
  if (rc == SRT_OK) rc = cudaStreamSynchronize(g->stream) == cudaSuccess ? SRT_OK : SRT_ERR_CUDA;
  if (rc != SRT_OK) { delete g; return rc; }
  *out = (srt_gpt2*)g;
  return SRT_OK;
}

int srt_gpt2_destroy(srt_gpt2* h) {
  if (!h) return SRT_OK;
  Gpt2* g = (Gpt2*)h;
  cudaStreamSynchronize(g->stream);
  delete g;
  return SRT_OK;
}

int srt_gpt2_num_params(srt_gpt2* h) { return h ? (int)((Gpt2*)h)->params.size() : -1; }

int srt_gpt2_param_info(srt_gpt2* h, int idx, char* name, int name_cap, int64_t shape[2], int* ndim) {
  Gpt2* g = (Gpt2*)h;
  SRT_REQUIRE(g && idx >= 0 && idx < (int)g->params.size(), "gpt2_param_info: bad index");
  const Gpt2::Rec& r = g->params[idx];
  if (name && name_cap > 0) { strncpy(name, r.name.c_str(), name_cap - 1); name[name_cap - 1] = 0; }
  if (shape) { shape[0] = r.shape[0]; shape[1] = r.shape[1]; }
  if (ndim) *ndim = r.ndim;
  return SRT_OK;
}

// Host arrays use the reference's shapes: linear weights [in][out], tables [rows][d_model].
int srt_gpt2_set_param(srt_gpt2* h, int idx, const float* host) {
  Gpt2* g = (Gpt2*)h;
  SRT_REQUIRE(g && host && idx >= 0 && idx < (int)g->params.size(), "gpt2_set_param: bad argument");
  const Gpt2::Rec& r = g->params[idx];
  if (r.kind == 1) {
    const int64_t in = r.shape[0], out = r.shape[1];
    std::vector<float> t((size_t)in * out);
    for (int64_t i = 0; i < in; ++i)
      for (int64_t o = 0; o < out; ++o) t[(size_t)o * in + i] = host[(size_t)i * out + o];
    SRT_CHECK_CUDA(cudaMemcpy(g->P + r.off, t.data(), t.size() * 4, cudaMemcpyHostToDevice));
  } else {
    const size_t n = r.ndim == 2 ? (size_t)r.shape[0] * r.shape[1] : (size_t)r.shape[0];
    SRT_CHECK_CUDA(cudaMemcpy(g->P + r.off, host, n * 4, cudaMemcpyHostToDevice));
  }
  return SRT_OK;
}

int srt_gpt2_get_param(srt_gpt2* h, int idx, float* host, int which) {
  Gpt2* g = (Gpt2*)h;
  SRT_REQUIRE(g && host && idx >= 0 && idx < (int)g->params.size(), "gpt2_get_param: bad argument");
  const Gpt2::Rec& r = g->params[idx];
  SRT_CHECK_CUDA(cudaStreamSynchronize(g->stream));
  const float* base = which == SRT_GET_GRAD ? g->G : which == SRT_GET_MOMENTUM ? g->M1 : g->P;
  if (r.kind == 1) {
    const int64_t in = r.shape[0], out = r.shape[1];
    std::vector<float> t((size_t)in * out);
    SRT_CHECK_CUDA(cudaMemcpy(t.data(), base + r.off, t.size() * 4, cudaMemcpyDeviceToHost));
    for (int64_t i = 0; i < in; ++i)
      for (int64_t o = 0; o < out; ++o) host[(size_t)i * out + o] = t[(size_t)o * in + i];
  } else {
    const size_t n = r.ndim == 2 ? (size_t)r.shape[0] * r.shape[1] : (size_t)r.shape[0];
    SRT_CHECK_CUDA(cudaMemcpy(host, base + r.off, n * 4, cudaMemcpyDeviceToHost));
  }
  return SRT_OK;
}

int srt_gpt2_commit_params(srt_gpt2* h) {
  Gpt2* g = (Gpt2*)h;
  SRT_REQUIRE(g, "gpt2_commit_params: null handle");
  int rc = g->refresh();
  if (rc) return rc;
  SRT_CHECK_CUDA(cudaStreamSynchronize(g->stream));
  return SRT_OK;
}

// ids: [B][seq] int32 on the host. Targets are the next token of the same sequence; the last position of a
// sequence has none. Also prepares the sorted token order the embedding gradient uses.
int srt_gpt2_upload_tokens(srt_gpt2* h, const int32_t* host_ids, int B) {
  Gpt2* g = (Gpt2*)h;
  SRT_REQUIRE(g && host_ids && B > 0 && B <= g->cfg.max_batch, "gpt2_upload_tokens: bad argument");
  const int S = g->S;
  const int T = B * S;
  std::vector<int32_t> lab(T), ord(T), sg;
  for (int t = 0; t < T; ++t) {
    SRT_REQUIRE(host_ids[t] >= 0 && host_ids[t] < g->V, "gpt2_upload_tokens: token id %d outside the vocabulary", host_ids[t]);
    lab[t] = (t % S) == S - 1 ? -1 : host_ids[t + 1];
  }
  std::iota(ord.begin(), ord.end(), 0);
  std::stable_sort(ord.begin(), ord.end(), [&](int a, int b) { return host_ids[a] < host_ids[b]; });
  for (int j = 0; j < T; ++j)
    if (j == 0 || host_ids[ord[j]] != host_ids[ord[j - 1]]) sg.push_back(j);
  g->n_unique = (int)sg.size();
  sg.push_back(T);
  SRT_CHECK_CUDA(cudaStreamSynchronize(g->stream));  // the pageable staging below must not race earlier work
  SRT_CHECK_CUDA(cudaMemcpy(g->ids, host_ids, (size_t)T * 4, cudaMemcpyHostToDevice));
  SRT_CHECK_CUDA(cudaMemcpy(g->labels, lab.data(), (size_t)T * 4, cudaMemcpyHostToDevice));
  SRT_CHECK_CUDA(cudaMemcpy(g->order, ord.data(), (size_t)T * 4, cudaMemcpyHostToDevice));
  SRT_CHECK_CUDA(cudaMemcpy(g->seg, sg.data(), sg.size() * 4, cudaMemcpyHostToDevice));
  g->cur_B = B;
  return SRT_OK;
}

int srt_gpt2_forward_backward(srt_gpt2* h, int B, int global_batch) {
  Gpt2* g = (Gpt2*)h;
  SRT_REQUIRE(g && B > 0 && B == g->cur_B && global_batch >= B, "gpt2_forward_backward: upload the tokens of this batch first");
  PartitionFollower::Scope sm_scope(g->part);
  int rc;
  if (g->act_batch < B && (rc = g->alloc_activations(B))) return rc;  // regain after a release or a shrink
  if ((rc = g->forward(B))) return rc;
  return g->backward(B, global_batch);
}

int srt_gpt2_forward_only(srt_gpt2* h, int B) {
  Gpt2* g = (Gpt2*)h;
  SRT_REQUIRE(g && B > 0 && B == g->cur_B, "gpt2_forward_only: upload the tokens of this batch first");
  PartitionFollower::Scope sm_scope(g->part);
  if (g->act_batch < B) { int rc = g->alloc_activations(B); if (rc) return rc; }
  return g->forward(B);
}

int srt_gpt2_optimizer(srt_gpt2* h) {
  Gpt2* g = (Gpt2*)h;
  SRT_REQUIRE(g, "gpt2_optimizer: null handle");
  PartitionFollower::Scope sm_scope(g->part);
  g->opt_steps++;
  const float* grad = g->accum_pending > 0 ? g->ACC : g->G;
  int rc = adamw(g->P, grad, g->M1, g->M2, g->Pw, (int64_t)g->n_flat, g->cfg.lr, g->cfg.beta1, g->cfg.beta2, g->cfg.eps,
                 g->cfg.weight_decay, g->opt_steps, g->stream);
  if (rc) return rc;
  if (g->accum_pending > 0) {
    SRT_CHECK_CUDA(cudaMemsetAsync(g->ACC, 0, g->n_flat * 4, g->stream));
    g->accum_pending = 0;
  }
  auto tr = [&](const Gpt2::Lin& l) {
    return filter_transpose(SRT_BF16, g->pw(l.w), g->WT + l.wt_off, l.out, 1, l.in, g->stream);
  };
  for (Gpt2::Layer& y : g->layers)
    if ((rc = tr(y.qkv)) || (rc = tr(y.proj)) || (rc = tr(y.fc)) || (rc = tr(y.fc2))) return rc;
  return filter_transpose(SRT_BF16, g->pw(g->wte), g->WT + g->wte_wt_off, g->Vpad, 1, g->C, g->stream);
}

// Mean next-token loss of the last micro-batch over its own targets (what the reference's model returns).
int srt_gpt2_loss(srt_gpt2* h, float* host_loss) {
  Gpt2* g = (Gpt2*)h;
  SRT_REQUIRE(g && host_loss && g->cur_B > 0, "gpt2_loss: nothing has run");
  float sum = 0.f;
  SRT_CHECK_CUDA(cudaMemcpyAsync(&sum, g->loss_acc, 4, cudaMemcpyDeviceToHost, g->stream));
  SRT_CHECK_CUDA(cudaStreamSynchronize(g->stream));
  *host_loss = sum / ((float)g->cur_B * (float)(g->S - 1));
  return SRT_OK;
}

int srt_gpt2_logits(srt_gpt2* h, float* host, int B) {
  Gpt2* g = (Gpt2*)h;
  SRT_REQUIRE(g && host && B > 0 && B <= g->cfg.max_batch, "gpt2_logits: bad argument");
  const size_t T = (size_t)B * g->S;
  std::vector<uint16_t> tmp(T * g->Vpad);
  SRT_CHECK_CUDA(cudaStreamSynchronize(g->stream));
  SRT_CHECK_CUDA(cudaMemcpy(tmp.data(), g->logits, tmp.size() * 2, cudaMemcpyDeviceToHost));
  for (size_t t = 0; t < T; ++t)
    for (int v = 0; v < g->V; ++v) {
      const uint32_t bits = (uint32_t)tmp[t * g->Vpad + v] << 16;
      memcpy(&host[t * g->V + v], &bits, 4);
    }
  return SRT_OK;
}

int srt_gpt2_follow_infer_tpc(srt_gpt2* h, srt_comm* comm, int device, int min_train_tpc, int max_train_tpc, int enable) {
  Gpt2* g = (Gpt2*)h;
  SRT_REQUIRE(g, "gpt2_follow_infer_tpc: null handle");
  { int dev = 0; SRT_CHECK_CUDA(cudaGetDevice(&dev)); g->part.device = dev; }
  return g->part.configure(g->stream, g->side, comm, device, min_train_tpc, max_train_tpc, enable != 0);
}

int srt_gpt2_current_sms(srt_gpt2* h) { if (!h) return -1;
  const int w = ((Gpt2*)h)->part.cur_sms;
  return w ? w : PartitionFollower::device_sm_count(); }

int srt_gpt2_synchronize(srt_gpt2* h) {
  Gpt2* g = (Gpt2*)h;
  SRT_REQUIRE(g, "gpt2_synchronize: null handle");
  SRT_CHECK_CUDA(cudaStreamSynchronize(g->stream));
  return SRT_OK;
}

int srt_gpt2_accumulate(srt_gpt2* h) {
  Gpt2* g = (Gpt2*)h;
  SRT_REQUIRE(g, "gpt2_accumulate: null handle");
  g->accum_pending++;
  return grad_accumulate(g->ACC, g->G, (int64_t)g->n_flat, g->stream);
}

int srt_gpt2_release_activations(srt_gpt2* h, size_t* released_bytes) {
  Gpt2* g = (Gpt2*)h;
  SRT_REQUIRE(g, "gpt2_release_activations: null handle");
  return g->release_activations(released_bytes);
}

int srt_gpt2_shrink_activations(srt_gpt2* h, int B, size_t* released_bytes) {
  Gpt2* g = (Gpt2*)h;
  SRT_REQUIRE(g, "gpt2_shrink_activations: null handle");
  return g->shrink_activations(B, released_bytes);
}

int srt_gpt2_request_abort(srt_gpt2* h, int on) {
  Gpt2* g = (Gpt2*)h;
  SRT_REQUIRE(g, "gpt2_request_abort: null handle");
  g->abort_flag.store(on ? 1 : 0, std::memory_order_release);
  return SRT_OK;
}

void* srt_gpt2_grad_buckets(srt_gpt2* h) { return h ? (void*)&((Gpt2*)h)->buckets : nullptr; }

int srt_gpt2_grad_buffer(srt_gpt2* h, void** ptr, int64_t* n) {
  Gpt2* g = (Gpt2*)h;
  SRT_REQUIRE(g && ptr && n, "gpt2_grad_buffer: null argument");
  *ptr = g->G;
  *n = (int64_t)g->n_flat;
  return SRT_OK;
}

void* srt_gpt2_stream(srt_gpt2* h) { return h ? (void*)((Gpt2*)h)->stream : nullptr; }
int64_t srt_gpt2_memory_bytes(srt_gpt2* h) { return h ? (int64_t)(((Gpt2*)h)->bytes_total + ((Gpt2*)h)->act_bytes) : -1; }
int64_t srt_gpt2_num_elements(srt_gpt2* h) { return h ? (int64_t)((Gpt2*)h)->n_flat : -1; }

}  // extern "C"
