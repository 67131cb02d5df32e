// Training step of a Qwen2 style decoder (the reference trains a transformers Qwen2 causal LM,
// train/qwen.py:35-37,80-91): token embedding, n_layer x [RMSNorm, Q/K/V projections with bias, rotary
// embedding, grouped-query causal attention, output projection, RMSNorm, SwiGLU MLP], final RMSNorm, output
// projection tied to the token table, next-token cross-entropy, AdamW.
//
// Same layout as the GPT-2 executor: [tokens][features] bf16 rows, linear layers on the tcgen05 implicit-GEMM
// kernels, attention products as batched tcgen05 GEMMs over 4-D tensor maps. Q, K and V live in one fused
// [tokens][(Hq + 2 Hkv) D] projection (their weights are adjacent rows of one matrix), gate and up in one
// [tokens][2 F] projection. Several query heads read one KV head through the batch divisor of the GEMM; the
// KV gradients are produced per query head and summed per group.
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
inline size_t upq(size_t v, size_t a) { return (v + a - 1) / a * a; }
}

struct Qwen2 {
  srt_qwen2_config cfg;
  int C, Hq, Hkv, D, F, V, Vpad, S, L, QKV, group;
  cudaStream_t stream = nullptr;

  struct Rec { std::string name; size_t off, count; int64_t shape[2]; int ndim; };
  std::vector<Rec> params;
  size_t n_flat = 0, n_wt = 0;
  float *P = nullptr, *G = nullptr, *M1 = nullptr, *M2 = nullptr;
  __nv_bfloat16 *Pw = nullptr, *WT = nullptr;
  int opt_steps = 0;

  struct Lin { size_t w_off; long long b_off; int in, out; size_t wt_off; };  // offsets into the flat buffers; b_off < 0 = no bias
  struct Layer {
    int n1, n2;
    Lin qkv, o, gu, down;
    __nv_bfloat16 *n1o, *qkv_o, *Pm, *att, *x2, *n2o, *gu_o, *act, *xout;
    float *z1, *r1, *z2, *r2;  // "mean" (zeros) and rstd of the two norms
  };
  std::vector<Layer> layers;
  int emb, nf;
  size_t emb_wt_off = 0;

  __nv_bfloat16 *x0 = nullptr, *nfo = nullptr, *logits = nullptr;
  float *zf = nullptr, *rf = nullptr, *row_loss = nullptr, *loss_acc = nullptr;
  __nv_bfloat16 *dxa = nullptr, *dxb = nullptr, *dqkv = nullptr, *dP = nullptr, *Tbig = nullptr, *t1 = nullptr, *t2 = nullptr,
                *dkv_h = nullptr, *dgu = nullptr, *dact = nullptr, *datt = nullptr, *dln = nullptr;
  void* scratch = nullptr;
  size_t scratch_bytes = 0;
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
  int32_t *ids = nullptr, *labels = nullptr, *order = nullptr, *seg = nullptr;
  int n_unique = 0, cur_B = 0;
  std::vector<void*> allocs;
  size_t bytes_total = 0;
  // Releasable part (everything sized by the batch): from the training allocator of a page pool when one is
  // attached, so that shrinking the batch hands whole pages to the inference side (as the other executors do).
  srt_pool* pool = nullptr;
  std::vector<void*> act_blocks;
  size_t act_bytes = 0;
  int act_batch = 0;
  float* ACC = nullptr;      // gradients accumulated over the micro-batches of a global batch
  int accum_pending = 0;
  std::atomic<int> abort_flag{0};
  static constexpr int kAhead = 4;  // layers the host may run ahead of the GPU (bounds the drain after a kill)
  cudaEvent_t ahead_ev[kAhead] = {nullptr};
  unsigned long long layer_seq = 0;

  int aalloc(void** out, size_t bytes) {
    bytes = upq(bytes ? bytes : 256, 256);
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
    SRT_REQUIRE(B <= cfg.max_batch, "qwen2 shrink_activations: batch %d above max_batch %d", B, cfg.max_batch);
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

  ~Qwen2() {
    if (part.home_stream) { stream = part.home_stream; side = part.home_side; }  // partition streams belong to the ladder
    release_activations(nullptr);
    for (auto e : ahead_ev) if (e) cudaEventDestroy(e);
    if (ev_fork) cudaEventDestroy(ev_fork);
    if (ev_join) cudaEventDestroy(ev_join);
    if (side) { cudaStreamSynchronize(side); cudaStreamDestroy(side); }
    for (void* p : allocs) cudaFree(p);
    if (stream) cudaStreamDestroy(stream);
  }
  template <class T>
  int dalloc(T** out, size_t bytes, bool zero = false) {
    bytes = upq(bytes ? bytes : 256, 256);
    SRT_CHECK_CUDA(cudaMalloc((void**)out, bytes));
    allocs.push_back((void*)*out);
    bytes_total += bytes;
    if (zero) SRT_CHECK_CUDA(cudaMemset(*out, 0, bytes));
    return SRT_OK;
  }
  // Registers a parameter; consecutive calls lay their tensors out back to back when every count is a multiple of 64.
  int add(const std::string& name, int64_t a, int64_t b, size_t count) {
    Rec r;
    r.name = name; r.off = n_flat; r.count = count; r.shape[0] = a; r.shape[1] = b; r.ndim = b > 0 ? 2 : 1;
    n_flat += upq(count, 64);
    params.push_back(r);
    return (int)params.size() - 1;
  }
  Lin make_lin(size_t w_off, long long b_off, int in, int out) {
    Lin l = {w_off, b_off, in, out, n_wt};
    n_wt += upq((size_t)in * out, 64);
    return l;
  }
  float* pf(int i) { return P + params[i].off; }
  float* gf(int i) { return G + params[i].off; }

  int build();
  int transposes();
  int forward(int B);
  int backward(int B, int global_batch);
  srt_conv_desc lin_desc(int64_t T, int in, int out) const { return {(int)T, 1, 1, in, out, 1, 1, 1, 0, 1, 1}; }
  int linear_fwd(const Lin& l, const void* x, void* y, const void* residual, int64_t T) {
    srt_conv_epilogue ep = {l.b_off >= 0 ? P + l.b_off : nullptr, residual};
    return conv_fprop(lin_desc(T, l.in, l.out), SRT_BF16, SRT_IMPL_AUTO, x, Pw + l.w_off, y, &ep, stream);
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
      if (l.b_off >= 0 && (rc = colsum_bf16(dy, T, l.out, G + l.b_off, wscratch, scratch_bytes, ws))) return rc;
      if ((rc = conv_wgrad(lin_desc(T, l.in, l.out), SRT_BF16, SRT_IMPL_AUTO, dy, x, G + l.w_off, wscratch, scratch_bytes, ws)))
        return rc;
    }
    if (dx) return conv_dgrad(lin_desc(T, l.in, l.out), SRT_BF16, SRT_IMPL_AUTO, dy, WT + l.wt_off, dx, nullptr, stream);
    return SRT_OK;
  }
};

int Qwen2::build() {
  C = cfg.hidden; Hq = cfg.n_head; Hkv = cfg.n_kv_head; F = cfg.intermediate; V = cfg.vocab; S = cfg.seq; L = cfg.n_layer;
  SRT_REQUIRE(C > 0 && Hq > 0 && Hkv > 0 && C % Hq == 0 && Hq % Hkv == 0, "qwen2: hidden / heads / kv heads do not divide");
  D = C / Hq;
  group = Hq / Hkv;
  QKV = (Hq + 2 * Hkv) * D;
  SRT_REQUIRE(D % 8 == 0 && C % 64 == 0 && F % 64 == 0 && (Hkv * D) % 64 == 0,
              "qwen2: head size must be a multiple of 8; hidden, intermediate and kv width multiples of 64");
  SRT_REQUIRE(S % 128 == 0 && cfg.max_batch > 0 && (long long)cfg.max_batch * Hq <= 65535,
              "qwen2: seq must be a multiple of 128");
  Vpad = (int)upq((size_t)V, 64);
  emb = add("model.embed_tokens.weight", V, C, (size_t)Vpad * C);
  layers.resize(L);
  for (int i = 0; i < L; ++i) {
    const std::string pre = "model.layers." + std::to_string(i);
    Layer& y = layers[i];
    y.n1 = add(pre + ".input_layernorm.weight", C, 0, C);
    // q, k, v weights are adjacent: one [QKV][C] matrix; likewise their biases, and gate/up
    const int qw = add(pre + ".self_attn.q_proj.weight", Hq * D, C, (size_t)Hq * D * C);
    add(pre + ".self_attn.k_proj.weight", Hkv * D, C, (size_t)Hkv * D * C);
    add(pre + ".self_attn.v_proj.weight", Hkv * D, C, (size_t)Hkv * D * C);
    const int qb = add(pre + ".self_attn.q_proj.bias", Hq * D, 0, (size_t)Hq * D);
    add(pre + ".self_attn.k_proj.bias", Hkv * D, 0, (size_t)Hkv * D);
    add(pre + ".self_attn.v_proj.bias", Hkv * D, 0, (size_t)Hkv * D);
    y.qkv = make_lin(params[qw].off, (long long)params[qb].off, C, QKV);
    const int ow = add(pre + ".self_attn.o_proj.weight", C, Hq * D, (size_t)C * Hq * D);
    y.o = make_lin(params[ow].off, -1, Hq * D, C);
    y.n2 = add(pre + ".post_attention_layernorm.weight", C, 0, C);
    const int gw = add(pre + ".mlp.gate_proj.weight", F, C, (size_t)F * C);
    add(pre + ".mlp.up_proj.weight", F, C, (size_t)F * C);
    y.gu = make_lin(params[gw].off, -1, C, 2 * F);
    const int dw = add(pre + ".mlp.down_proj.weight", C, F, (size_t)C * F);
    y.down = make_lin(params[dw].off, -1, F, C);
  }
  nf = add("model.norm.weight", C, 0, C);
  emb_wt_off = n_wt;
  n_wt += upq((size_t)Vpad * C, 64);

  int rc;
  if ((rc = dalloc(&P, n_flat * 4, true)) || (rc = dalloc(&G, n_flat * 4, true)) || (rc = dalloc(&M1, n_flat * 4, true)) ||
      (rc = dalloc(&M2, n_flat * 4, true)) || (rc = dalloc(&Pw, n_flat * 2, true)) || (rc = dalloc(&WT, n_wt * 2, true)))
    return rc;
  if ((rc = dalloc(&ACC, n_flat * 4, true)) || (rc = dalloc(&loss_acc, 256, true))) return rc;
  const size_t T = (size_t)cfg.max_batch * S;
  size_t sb = layernorm_bwd_scratch_bytes(C);
  if (colsum_scratch_bytes(QKV) > sb) sb = colsum_scratch_bytes(QKV);
  auto wg = [&](int in, int out) {
    const size_t b = conv_wgrad_scratch_bytes(lin_desc((int64_t)T, in, out), SRT_BF16, SRT_IMPL_AUTO);
    if (b > sb) sb = b;
  };
  wg(C, QKV); wg(Hq * D, C); wg(C, 2 * F); wg(F, C); wg(C, Vpad);
  scratch_bytes = sb;
  if ((rc = dalloc((char**)&scratch, scratch_bytes))) return rc;
  if ((rc = dalloc((char**)&scratch_side, scratch_bytes))) return rc;
  if ((rc = dalloc(&ids, T * 4)) || (rc = dalloc(&labels, T * 4)) || (rc = dalloc(&order, T * 4)) ||
      (rc = dalloc(&seg, (T + 1) * 4)))
    return rc;
  {
    std::vector<size_t> starts;
    for (Layer& y : layers) starts.push_back(params[y.n1].off);
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
  return alloc_activations(cfg.max_batch);
}

// Everything sized by the batch: saved activations of every layer, logits, backward scratch.
int Qwen2::alloc_activations(int B) {
  SRT_REQUIRE(B > 0 && B <= cfg.max_batch, "qwen2 activations: batch %d outside 1..%d", B, cfg.max_batch);
  if (act_batch == B) return SRT_OK;
  int rc = free_activation_blocks();
  if (rc) return rc;
  const size_t T = (size_t)B * S, BH = (size_t)B * Hq;
  auto act = [&](__nv_bfloat16** p, size_t elems) { return aalloc((void**)p, elems * 2); };
  auto actf = [&](float** p, size_t elems) { return aalloc((void**)p, elems * 4); };
  auto zeros = [&](float** p, size_t elems) -> int {  // the "mean" of an RMSNorm: zeros
    int r = aalloc((void**)p, elems * 4);
    if (r) return r;
    SRT_CHECK_CUDA(cudaMemsetAsync(*p, 0, elems * 4, stream));
    return (int)SRT_OK;
  };
  if ((rc = act(&x0, T * C))) return rc;
  for (Layer& y : layers) {
    if ((rc = act(&y.n1o, T * C)) || (rc = act(&y.qkv_o, T * QKV)) || (rc = act(&y.Pm, BH * S * S)) ||
        (rc = act(&y.att, T * Hq * D)) || (rc = act(&y.x2, T * C)) || (rc = act(&y.n2o, T * C)) ||
        (rc = act(&y.gu_o, T * 2 * F)) || (rc = act(&y.act, T * F)) || (rc = act(&y.xout, T * C)))
      return rc;
    if ((rc = zeros(&y.z1, T)) || (rc = actf(&y.r1, T)) || (rc = zeros(&y.z2, T)) || (rc = actf(&y.r2, T))) return rc;
  }
  if ((rc = act(&nfo, T * C)) || (rc = act(&logits, T * Vpad))) return rc;
  if ((rc = zeros(&zf, T)) || (rc = actf(&rf, T)) || (rc = actf(&row_loss, T))) return rc;
  if ((rc = act(&dxa, T * C)) || (rc = act(&dxb, T * C)) || (rc = act(&dqkv, T * QKV)) || (rc = act(&dP, BH * S * S)) ||
      (rc = act(&Tbig, BH * S * S)) || (rc = act(&t1, T * Hq * D)) || (rc = act(&t2, T * Hq * D)) ||
      (rc = act(&dkv_h, T * Hq * D)) || (rc = act(&dgu, T * 2 * F)) || (rc = act(&dact, T * F)) ||
      (rc = act(&datt, T * Hq * D)) || (rc = act(&dln, T * C)))
    return rc;
  act_batch = B;
  return SRT_OK;
}

int Qwen2::transposes() {
  int rc;
  auto tr = [&](const Lin& l) { return filter_transpose(SRT_BF16, Pw + l.w_off, WT + l.wt_off, l.out, 1, l.in, stream); };
  for (Layer& y : layers)
    if ((rc = tr(y.qkv)) || (rc = tr(y.o)) || (rc = tr(y.gu)) || (rc = tr(y.down))) return rc;
  return filter_transpose(SRT_BF16, Pw + params[emb].off, WT + emb_wt_off, Vpad, 1, C, stream);
}

int Qwen2::forward(int B) {
  const int64_t T = (int64_t)B * S;
  const float scale = 1.f / sqrtf((float)D);
  const int KO = Hq * D, VO = (Hq + Hkv) * D;  // column offsets of K and V inside the fused projection
  const long long SS = (long long)S * S;
  int rc;
  if ((rc = join_side())) return rc;
  if ((rc = embedding_fwd(ids, pf(emb), nullptr, x0, T, S, C, stream))) return rc;
  const __nv_bfloat16* x = x0;
  for (Layer& y : layers) {
    if ((rc = checkpoint())) return rc;
    if ((rc = rmsnorm_fwd(x, pf(y.n1), y.n1o, y.z1, y.r1, T, C, cfg.rms_eps, stream))) return rc;
    if ((rc = linear_fwd(y.qkv, y.n1o, y.qkv_o, nullptr, T))) return rc;
    if ((rc = rope_apply(y.qkv_o, T, S, Hq, D, QKV, cfg.rope_theta, 0, stream))) return rc;
    if ((rc = rope_apply(y.qkv_o + KO, T, S, Hkv, D, QKV, cfg.rope_theta, 0, stream))) return rc;
    BgemmDesc q = {S, S, D, Hq, B, QKV, D, (long long)S * QKV, QKV, D, (long long)S * QKV, S, SS, Hq * SS, scale, 1, 0, group};
    if ((rc = bgemm_bf16(q, y.qkv_o, y.qkv_o + KO, y.Pm, stream))) return rc;
    if ((rc = causal_softmax_fwd(y.Pm, (int64_t)B * Hq, S, stream))) return rc;
    if ((rc = batched_transpose(y.qkv_o + VO, t1, S, D, QKV, D, (long long)S * QKV, Hkv, B, stream))) return rc;  // [B][Hkv][D][S]
    BgemmDesc o = {S, D, S, Hq, B, S, SS, Hq * SS, S, (long long)D * S, (long long)Hkv * D * S, KO, D, (long long)S * KO,
                   1.f, 0, 1, group};
    if ((rc = bgemm_bf16(o, y.Pm, t1, y.att, stream))) return rc;
    if ((rc = linear_fwd(y.o, y.att, y.x2, x, T))) return rc;
    if ((rc = rmsnorm_fwd(y.x2, pf(y.n2), y.n2o, y.z2, y.r2, T, C, cfg.rms_eps, stream))) return rc;
    if ((rc = linear_fwd(y.gu, y.n2o, y.gu_o, nullptr, T))) return rc;
    if ((rc = swiglu_fwd(y.gu_o, y.act, T, F, stream))) return rc;
    if ((rc = linear_fwd(y.down, y.act, y.xout, y.x2, T))) return rc;
    x = y.xout;
  }
  if ((rc = rmsnorm_fwd(x, pf(nf), nfo, zf, rf, T, C, cfg.rms_eps, stream))) return rc;
  return conv_fprop(lin_desc(T, C, Vpad), SRT_BF16, SRT_IMPL_AUTO, nfo, Pw + params[emb].off, logits, nullptr, stream);
}

int Qwen2::backward(int B, int global_batch) {
  const int64_t T = (int64_t)B * S;
  const float scale = 1.f / sqrtf((float)D);
  const int KO = Hq * D, VO = (Hq + Hkv) * D;
  const long long SS = (long long)S * S;
  int rc;
  buckets.begin_backward();
  const float gscale = 1.f / ((float)global_batch * (float)(S - 1));
  if ((rc = lm_cross_entropy(logits, labels, T, V, Vpad, gscale, row_loss, stream))) return rc;
  if ((rc = sum_f32(row_loss, (int)T, loss_acc, 0, stream))) return rc;
  if (side && overlap_wgrad) {
    SRT_CHECK_CUDA(cudaEventRecord(ev_fork, stream));
    SRT_CHECK_CUDA(cudaStreamWaitEvent(side, ev_fork, 0));
    side_dirty = true;
    PdlOff no_early_launch(true);
    if ((rc = conv_wgrad(lin_desc(T, C, Vpad), SRT_BF16, SRT_IMPL_AUTO, logits, nfo, gf(emb), scratch_side, scratch_bytes, side)))
      return rc;
  } else if ((rc = conv_wgrad(lin_desc(T, C, Vpad), SRT_BF16, SRT_IMPL_AUTO, logits, nfo, gf(emb), scratch, scratch_bytes,
                              stream))) {
    return rc;
  }
  if ((rc = conv_dgrad(lin_desc(T, C, Vpad), SRT_BF16, SRT_IMPL_AUTO, logits, WT + emb_wt_off, dln, nullptr, stream))) return rc;
  const __nv_bfloat16* x_last = L > 0 ? layers[L - 1].xout : x0;
  if ((rc = rmsnorm_bwd(dln, x_last, pf(nf), zf, rf, nullptr, dxa, gf(nf), T, C, scratch, scratch_bytes, stream))) return rc;
  __nv_bfloat16 *dx = dxa, *dx_other = dxb;
  for (int i = L - 1; i >= 0; --i) {
    Layer& y = layers[i];
    const __nv_bfloat16* xin = i == 0 ? x0 : layers[i - 1].xout;
    if ((rc = checkpoint())) return rc;
    // MLP
    if ((rc = linear_bwd(y.down, dx, y.act, dact, T))) return rc;
    if ((rc = swiglu_bwd(dact, y.gu_o, dgu, T, F, stream))) return rc;
    if ((rc = linear_bwd(y.gu, dgu, y.n2o, dln, T))) return rc;
    if ((rc = rmsnorm_bwd(dln, y.x2, pf(y.n2), y.z2, y.r2, dx, dx_other, gf(y.n2), T, C, scratch, scratch_bytes, stream)))
      return rc;
    // attention
    if ((rc = linear_bwd(y.o, dx_other, y.att, datt, T))) return rc;
    BgemmDesc dp = {S, S, D, Hq, B, KO, D, (long long)S * KO, QKV, D, (long long)S * QKV, S, SS, Hq * SS, 1.f, 1, 0, group};
    if ((rc = bgemm_bf16(dp, datt, y.qkv_o + VO, dP, stream))) return rc;
    // dV per query head = P^T dO, then summed over the heads of a group
    if ((rc = batched_transpose(y.Pm, Tbig, S, S, S, SS, Hq * SS, Hq, B, stream, 1))) return rc;
    if ((rc = batched_transpose(datt, t1, S, D, KO, D, (long long)S * KO, Hq, B, stream))) return rc;       // dO^T [B][Hq][D][S]
    BgemmDesc dv = {S, D, S, Hq, B, S, SS, Hq * SS, S, (long long)D * S, (long long)Hq * D * S, D, (long long)S * D,
                    (long long)Hq * S * D, 1.f, 0, 2, 1};
    if ((rc = bgemm_bf16(dv, Tbig, t1, dkv_h, stream))) return rc;                                           // [B][Hq][S][D]
    if ((rc = head_group_sum(dkv_h, dqkv + VO, B, S, Hq, group, D, QKV, stream))) return rc;
    if ((rc = causal_softmax_bwd(y.Pm, dP, (int64_t)B * Hq, S, stream))) return rc;
    // dQ = dS K * scale (K of the group's KV head)
    if ((rc = batched_transpose(y.qkv_o + KO, t1, S, D, QKV, D, (long long)S * QKV, Hkv, B, stream))) return rc;  // K^T [B][Hkv][D][S]
    BgemmDesc dq = {S, D, S, Hq, B, S, SS, Hq * SS, S, (long long)D * S, (long long)Hkv * D * S, QKV, D, (long long)S * QKV,
                    scale, 0, 1, group};
    if ((rc = bgemm_bf16(dq, dP, t1, dqkv, stream))) return rc;
    // dK per query head = dS^T Q * scale, summed per group
    if ((rc = batched_transpose(dP, Tbig, S, S, S, SS, Hq * SS, Hq, B, stream, 1))) return rc;
    if ((rc = batched_transpose(y.qkv_o, t2, S, D, QKV, D, (long long)S * QKV, Hq, B, stream))) return rc;        // Q^T [B][Hq][D][S]
    BgemmDesc dk = {S, D, S, Hq, B, S, SS, Hq * SS, S, (long long)D * S, (long long)Hq * D * S, D, (long long)S * D,
                    (long long)Hq * S * D, scale, 0, 2, 1};
    if ((rc = bgemm_bf16(dk, Tbig, t2, dkv_h, stream))) return rc;
    if ((rc = head_group_sum(dkv_h, dqkv + KO, B, S, Hq, group, D, QKV, stream))) return rc;
    // through the rotation (transposed), the fused projection and the first norm
    if ((rc = rope_apply(dqkv, T, S, Hq, D, QKV, cfg.rope_theta, 1, stream))) return rc;
    if ((rc = rope_apply(dqkv + KO, T, S, Hkv, D, QKV, cfg.rope_theta, 1, stream))) return rc;
    if ((rc = linear_bwd(y.qkv, dqkv, y.n1o, dln, T))) return rc;
    if ((rc = join_side())) return rc;  // the next kernel overwrites dx, which this layer's first weight gradient read
    if ((rc = rmsnorm_bwd(dln, xin, pf(y.n1), y.z1, y.r1, dx_other, dx, gf(y.n1), T, C, scratch, scratch_bytes, stream)))
      return rc;
    if ((rc = buckets.unit_done(i, stream))) return rc;
  }
  if ((rc = join_side())) return rc;
  if ((rc = embedding_bwd(dx, ids, order, seg, n_unique, gf(emb), nullptr, B, S, C, stream))) return rc;
  return buckets.all_done(stream);
}

}  // namespace srt

using namespace srt;

extern "C" {

int srt_qwen2_create(const srt_qwen2_config* cfg, srt_qwen2** out) { return srt_qwen2_create_with_pool(cfg, nullptr, out); }

int srt_qwen2_create_with_pool(const srt_qwen2_config* cfg, srt_pool* pool, srt_qwen2** out) {
  SRT_REQUIRE(cfg && out, "qwen2_create: null argument");
  Qwen2* g = new Qwen2();
  g->cfg = *cfg;
  g->pool = pool;
  int rc = g->build();
  if (rc == SRT_OK) rc = cudaStreamSynchronize(g->stream) == cudaSuccess ? SRT_OK : SRT_ERR_CUDA;
  if (rc != SRT_OK) { delete g; return rc; }
  *out = (srt_qwen2*)g;
  return SRT_OK;
}

int srt_qwen2_destroy(srt_qwen2* h) {
  if (!h) return SRT_OK;
  Qwen2* g = (Qwen2*)h;
  cudaStreamSynchronize(g->stream);
  delete g;
  return SRT_OK;
}

int srt_qwen2_num_params(srt_qwen2* h) { return h ? (int)((Qwen2*)h)->params.size() : -1; }

int srt_qwen2_param_info(srt_qwen2* h, int idx, char* name, int name_cap, int64_t shape[2], int* ndim) {
  Qwen2* g = (Qwen2*)h;
  SRT_REQUIRE(g && idx >= 0 && idx < (int)g->params.size(), "qwen2_param_info: bad index");
  const Qwen2::Rec& r = g->params[idx];
  if (name && name_cap > 0) { strncpy(name, r.name.c_str(), name_cap - 1); name[name_cap - 1] = 0; }
  if (shape) { shape[0] = r.shape[0]; shape[1] = r.shape[1]; }
  if (ndim) *ndim = r.ndim;
  return SRT_OK;
}

// Host arrays use the reference's shapes (nn.Linear weights [out][in], which is also the internal layout).
int srt_qwen2_set_param(srt_qwen2* h, int idx, const float* host) {
  Qwen2* g = (Qwen2*)h;
  SRT_REQUIRE(g && host && idx >= 0 && idx < (int)g->params.size(), "qwen2_set_param: bad argument");
  const Qwen2::Rec& r = g->params[idx];
  const size_t n = r.ndim == 2 ? (size_t)r.shape[0] * r.shape[1] : (size_t)r.shape[0];
  SRT_CHECK_CUDA(cudaMemcpy(g->P + r.off, host, n * 4, cudaMemcpyHostToDevice));
  return SRT_OK;
}

int srt_qwen2_get_param(srt_qwen2* h, int idx, float* host, int which) {
  Qwen2* g = (Qwen2*)h;
  SRT_REQUIRE(g && host && idx >= 0 && idx < (int)g->params.size(), "qwen2_get_param: bad argument");
  const Qwen2::Rec& r = g->params[idx];
  SRT_CHECK_CUDA(cudaStreamSynchronize(g->stream));
  const float* base = which == SRT_GET_GRAD ? g->G : which == SRT_GET_MOMENTUM ? g->M1 : g->P;
  const size_t n = r.ndim == 2 ? (size_t)r.shape[0] * r.shape[1] : (size_t)r.shape[0];
  SRT_CHECK_CUDA(cudaMemcpy(host, base + r.off, n * 4, cudaMemcpyDeviceToHost));
  return SRT_OK;
}

int srt_qwen2_commit_params(srt_qwen2* h) {
  Qwen2* g = (Qwen2*)h;
  SRT_REQUIRE(g, "qwen2_commit_params: null handle");
  int rc = cast_f32_to_bf16(g->P, g->Pw, (int64_t)g->n_flat, g->stream);
  if (rc == SRT_OK) rc = g->transposes();
  if (rc) return rc;
  SRT_CHECK_CUDA(cudaStreamSynchronize(g->stream));
  return SRT_OK;
}

int srt_qwen2_upload_tokens(srt_qwen2* h, const int32_t* host_ids, int B) {
  Qwen2* g = (Qwen2*)h;
  SRT_REQUIRE(g && host_ids && B > 0 && B <= g->cfg.max_batch, "qwen2_upload_tokens: bad argument");
  const int S = g->S;
  const int T = B * S;
  std::vector<int32_t> lab(T), ord(T), sg;
  for (int t = 0; t < T; ++t) {
    SRT_REQUIRE(host_ids[t] >= 0 && host_ids[t] < g->V, "qwen2_upload_tokens: token id %d outside the vocabulary", host_ids[t]);
    lab[t] = (t % S) == S - 1 ? -1 : host_ids[t + 1];
  }
  std::iota(ord.begin(), ord.end(), 0);
  std::stable_sort(ord.begin(), ord.end(), [&](int a, int b) { return host_ids[a] < host_ids[b]; });
  for (int j = 0; j < T; ++j)
    if (j == 0 || host_ids[ord[j]] != host_ids[ord[j - 1]]) sg.push_back(j);
  g->n_unique = (int)sg.size();
  sg.push_back(T);
  SRT_CHECK_CUDA(cudaStreamSynchronize(g->stream));
  SRT_CHECK_CUDA(cudaMemcpy(g->ids, host_ids, (size_t)T * 4, cudaMemcpyHostToDevice));
  SRT_CHECK_CUDA(cudaMemcpy(g->labels, lab.data(), (size_t)T * 4, cudaMemcpyHostToDevice));
  SRT_CHECK_CUDA(cudaMemcpy(g->order, ord.data(), (size_t)T * 4, cudaMemcpyHostToDevice));
  SRT_CHECK_CUDA(cudaMemcpy(g->seg, sg.data(), sg.size() * 4, cudaMemcpyHostToDevice));
  g->cur_B = B;
  return SRT_OK;
}

int srt_qwen2_forward_backward(srt_qwen2* h, int B, int global_batch) {
  Qwen2* g = (Qwen2*)h;
  SRT_REQUIRE(g && B > 0 && B == g->cur_B && global_batch >= B, "qwen2_forward_backward: upload the tokens of this batch first");
  PartitionFollower::Scope sm_scope(g->part);
  int rc;
  if (g->act_batch < B && (rc = g->alloc_activations(B))) return rc;  // regain after a release or a shrink
  if ((rc = g->forward(B))) return rc;
  return g->backward(B, global_batch);
}

int srt_qwen2_forward_only(srt_qwen2* h, int B) {
  Qwen2* g = (Qwen2*)h;
  SRT_REQUIRE(g && B > 0 && B == g->cur_B, "qwen2_forward_only: upload the tokens of this batch first");
  PartitionFollower::Scope sm_scope(g->part);
  if (g->act_batch < B) { int rc = g->alloc_activations(B); if (rc) return rc; }
  return g->forward(B);
}

int srt_qwen2_optimizer(srt_qwen2* h) {
  Qwen2* g = (Qwen2*)h;
  SRT_REQUIRE(g, "qwen2_optimizer: null handle");
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
  return g->transposes();
}

int srt_qwen2_loss(srt_qwen2* h, float* host_loss) {
  Qwen2* g = (Qwen2*)h;
  SRT_REQUIRE(g && host_loss && g->cur_B > 0, "qwen2_loss: nothing has run");
  float sum = 0.f;
  SRT_CHECK_CUDA(cudaMemcpyAsync(&sum, g->loss_acc, 4, cudaMemcpyDeviceToHost, g->stream));
  SRT_CHECK_CUDA(cudaStreamSynchronize(g->stream));
  *host_loss = sum / ((float)g->cur_B * (float)(g->S - 1));
  return SRT_OK;
}

int srt_qwen2_logits(srt_qwen2* h, float* host, int B) {
  Qwen2* g = (Qwen2*)h;
  SRT_REQUIRE(g && host && B > 0 && B <= g->cfg.max_batch, "qwen2_logits: bad argument");
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

int srt_qwen2_follow_infer_tpc(srt_qwen2* h, srt_comm* comm, int device, int min_train_tpc, int max_train_tpc, int enable) {
  Qwen2* g = (Qwen2*)h;
  SRT_REQUIRE(g, "qwen2_follow_infer_tpc: null handle");
  { int dev = 0; SRT_CHECK_CUDA(cudaGetDevice(&dev)); g->part.device = dev; }
  return g->part.configure(g->stream, g->side, comm, device, min_train_tpc, max_train_tpc, enable != 0);
}

int srt_qwen2_current_sms(srt_qwen2* h) { if (!h) return -1;
  const int w = ((Qwen2*)h)->part.cur_sms;
  return w ? w : PartitionFollower::device_sm_count(); }

int srt_qwen2_synchronize(srt_qwen2* h) {
  Qwen2* g = (Qwen2*)h;
  SRT_REQUIRE(g, "qwen2_synchronize: null handle");
  SRT_CHECK_CUDA(cudaStreamSynchronize(g->stream));
  return SRT_OK;
}

void* srt_qwen2_grad_buckets(srt_qwen2* h) { return h ? (void*)&((Qwen2*)h)->buckets : nullptr; }

int srt_qwen2_grad_buffer(srt_qwen2* h, void** ptr, int64_t* n) {
  Qwen2* g = (Qwen2*)h;
  SRT_REQUIRE(g && ptr && n, "qwen2_grad_buffer: null argument");
  *ptr = g->G;
  *n = (int64_t)g->n_flat;
  return SRT_OK;
}

void* srt_qwen2_stream(srt_qwen2* h) { return h ? (void*)((Qwen2*)h)->stream : nullptr; }
int64_t srt_qwen2_memory_bytes(srt_qwen2* h) { return h ? (int64_t)(((Qwen2*)h)->bytes_total + ((Qwen2*)h)->act_bytes) : -1; }

int srt_qwen2_accumulate(srt_qwen2* h) {
  Qwen2* g = (Qwen2*)h;
  SRT_REQUIRE(g, "qwen2_accumulate: null handle");
  g->accum_pending++;
  return grad_accumulate(g->ACC, g->G, (int64_t)g->n_flat, g->stream);
}

int srt_qwen2_release_activations(srt_qwen2* h, size_t* released_bytes) {
  Qwen2* g = (Qwen2*)h;
  SRT_REQUIRE(g, "qwen2_release_activations: null handle");
  return g->release_activations(released_bytes);
}

int srt_qwen2_shrink_activations(srt_qwen2* h, int B, size_t* released_bytes) {
  Qwen2* g = (Qwen2*)h;
  SRT_REQUIRE(g, "qwen2_shrink_activations: null handle");
  return g->shrink_activations(B, released_bytes);
}

int srt_qwen2_request_abort(srt_qwen2* h, int on) {
  Qwen2* g = (Qwen2*)h;
  SRT_REQUIRE(g, "qwen2_request_abort: null handle");
  g->abort_flag.store(on ? 1 : 0, std::memory_order_release);
  return SRT_OK;
}

}  // extern "C"
