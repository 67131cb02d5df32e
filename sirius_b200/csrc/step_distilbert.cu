// Forward pass of a DistilBERT-style encoder for the stand-in inference worker (the reference serves
// "distilbert_base" through its TVM graph executor, server/model_store/infer_model.cc:46-58,394-523; the
// arithmetic is that of transformers.DistilBertModel): token + position embedding and LayerNorm, then n_layer x
// [Q/K/V projections, bidirectional multi-head attention, output projection, residual + LayerNorm, MLP with
// erf-GELU, residual + LayerNorm]. Output: the last hidden state.
//
// Same building blocks as the training executors: activations are [tokens][features] bf16 rows, linear layers
// run on the tcgen05 implicit-GEMM kernels (bias and residual add in the epilogue), Q, K and V come from one
// fused [tokens][3*dim] projection (the three weight matrices sit back to back in the flat parameter buffer) and
// the attention products are batched tcgen05 GEMMs addressing the heads in place. Activations come from the
// INFERENCE allocator of a page pool when one is attached, so that a request that finds no memory triggers the
// handover from the colocated trainer, and go back to the pool when the worker idles.
#include <string.h>

#include <string>
#include <vector>

#include "../../include/sirius_b200.h"
#include "../../include/sirius_pool.h"
#include "common.cuh"
#include "ops.cuh"

namespace srt {

namespace {
inline size_t up_to(size_t v, size_t a) { return (v + a - 1) / a * a; }
}

struct Bert {
  srt_bert_config cfg;
  int C, H, D, F, V, S, L;
  cudaStream_t stream = nullptr;
  struct Rec { std::string name; size_t off, count; int64_t shape[2]; int ndim; };
  std::vector<Rec> params;
  size_t n_flat = 0;
  float* P = nullptr;             // fp32 parameters (embedding tables, norms and biases are read from here)
  __nv_bfloat16* Pw = nullptr;    // bf16 copy (linear weights)
  struct Layer {
    int wq, wk, wv, bq, bk, bv, wo, bo, ln1_g, ln1_b, w1, b1, w2, b2, ln2_g, ln2_b;
  };
  std::vector<Layer> layers;
  int wte, wpe, eln_g, eln_b;
  int32_t* ids = nullptr;
  int cur_B = 0;
  std::vector<void*> allocs;
  size_t bytes_total = 0;
  // releasable part
  srt_pool* pool = nullptr;
  std::vector<void*> act_blocks;
  size_t act_bytes = 0;
  __nv_bfloat16 *emb = nullptr, *xa = nullptr, *xb = nullptr, *qkv = nullptr, *Pm = nullptr, *vt = nullptr, *att = nullptr,
                *t1 = nullptr, *sa = nullptr, *h1 = nullptr, *g1 = nullptr;
  float *mean = nullptr, *rstd = nullptr;
  const __nv_bfloat16* out = nullptr;  // last hidden state of the latest forward

  ~Bert() {
    if (stream) cudaStreamSynchronize(stream);
    free_activations();
    for (void* p : allocs) cudaFree(p);
    if (stream) cudaStreamDestroy(stream);
  }
  template <class T>
  int dalloc(T** o, size_t bytes) {
    bytes = up_to(bytes ? bytes : 256, 256);
    SRT_CHECK_CUDA(cudaMalloc((void**)o, bytes));
    SRT_CHECK_CUDA(cudaMemset(*o, 0, bytes));
    allocs.push_back((void*)*o);
    bytes_total += bytes;
    return SRT_OK;
  }
  int aalloc(void** o, size_t bytes) {
    bytes = up_to(bytes ? bytes : 256, 256);
    if (pool) {
      int rc = srt_pool_alloc(pool, SRT_POOL_INFER, bytes, o);
      if (rc) return rc;
    } else {
      SRT_CHECK_CUDA(cudaMalloc(o, bytes));
    }
    act_blocks.push_back(*o);
    act_bytes += bytes;
    return SRT_OK;
  }
  int free_activations() {
    if (stream && !act_blocks.empty()) SRT_CHECK_CUDA(cudaStreamSynchronize(stream));
    for (void* p : act_blocks) {
      if (pool) { int rc = srt_pool_free(pool, SRT_POOL_INFER, p); if (rc) return rc; }
      else cudaFree(p);
    }
    act_blocks.clear();
    act_bytes = 0;
    out = nullptr;
    return SRT_OK;
  }
  int add(const std::string& name, int64_t a, int64_t b) {
    Rec r;
    r.name = name; r.off = n_flat; r.shape[0] = a; r.shape[1] = b; r.ndim = b > 0 ? 2 : 1;
    r.count = b > 0 ? (size_t)a * b : (size_t)a;
    n_flat += up_to(r.count, 64);
    params.push_back(r);
    return (int)params.size() - 1;
  }
  float* pf(int i) { return P + params[i].off; }
  __nv_bfloat16* pw(int i) { return Pw + params[i].off; }
  srt_conv_desc lin_desc(int64_t T, int in, int o) const { return {(int)T, 1, 1, in, o, 1, 1, 1, 0, 1, 1}; }
  int linear(int w, int b, int in, int o, const void* x, void* y, const void* residual, int64_t T) {
    srt_conv_epilogue ep = {pf(b), residual};
    return conv_fprop(lin_desc(T, in, o), SRT_BF16, SRT_IMPL_AUTO, x, pw(w), y, &ep, stream);
  }
  int build();
  int alloc_activations();
  int forward(int B);
};

int Bert::build() {
  C = cfg.dim; H = cfg.n_head; F = cfg.hidden_dim; V = cfg.vocab; S = cfg.seq; L = cfg.n_layer;
  SRT_REQUIRE(C > 0 && H > 0 && C % H == 0 && L > 0 && F > 0, "bert: bad configuration");
  D = C / H;
  SRT_REQUIRE(D % 8 == 0 && C % 64 == 0 && F % 64 == 0, "bert: head size must be a multiple of 8, dim and hidden_dim of 64");
  SRT_REQUIRE(S % 8 == 0 && S > 0 && S <= cfg.max_pos && cfg.max_batch > 0, "bert: seq must be a multiple of 8 and at most max_pos");
  SRT_REQUIRE((long long)cfg.max_batch * H <= 65535, "bert: batch * heads too large");
  wte = add("embeddings.word_embeddings.weight", V, C);
  wpe = add("embeddings.position_embeddings.weight", cfg.max_pos, C);
  eln_g = add("embeddings.LayerNorm.weight", C, 0);
  eln_b = add("embeddings.LayerNorm.bias", C, 0);
  layers.resize(L);
  for (int i = 0; i < L; ++i) {
    const std::string pre = "transformer.layer." + std::to_string(i);
    Layer& y = layers[i];
    // the three projection matrices (and their biases) are adjacent: together they are the fused [3*dim][dim] weight
    y.wq = add(pre + ".attention.q_lin.weight", C, C);
    y.wk = add(pre + ".attention.k_lin.weight", C, C);
    y.wv = add(pre + ".attention.v_lin.weight", C, C);
    y.bq = add(pre + ".attention.q_lin.bias", C, 0);
    y.bk = add(pre + ".attention.k_lin.bias", C, 0);
    y.bv = add(pre + ".attention.v_lin.bias", C, 0);
    y.wo = add(pre + ".attention.out_lin.weight", C, C);
    y.bo = add(pre + ".attention.out_lin.bias", C, 0);
    y.ln1_g = add(pre + ".sa_layer_norm.weight", C, 0);
    y.ln1_b = add(pre + ".sa_layer_norm.bias", C, 0);
    y.w1 = add(pre + ".ffn.lin1.weight", F, C);
    y.b1 = add(pre + ".ffn.lin1.bias", F, 0);
    y.w2 = add(pre + ".ffn.lin2.weight", C, F);
    y.b2 = add(pre + ".ffn.lin2.bias", C, 0);
    y.ln2_g = add(pre + ".output_layer_norm.weight", C, 0);
    y.ln2_b = add(pre + ".output_layer_norm.bias", C, 0);
    SRT_REQUIRE(params[y.wk].off == params[y.wq].off + (size_t)C * C && params[y.wv].off == params[y.wk].off + (size_t)C * C &&
                    params[y.bk].off == params[y.bq].off + (size_t)C && params[y.bv].off == params[y.bk].off + (size_t)C,
                "bert: the fused projection is not contiguous");
  }
  int rc;
  if ((rc = dalloc(&P, n_flat * 4)) || (rc = dalloc(&Pw, n_flat * 2))) return rc;
  if ((rc = dalloc(&ids, (size_t)cfg.max_batch * S * 4))) return rc;
  SRT_CHECK_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
  return alloc_activations();
}

int Bert::alloc_activations() {
  if (!act_blocks.empty()) return SRT_OK;
  const size_t T = (size_t)cfg.max_batch * S, BH = (size_t)cfg.max_batch * H;
  int rc;
  auto act = [&](__nv_bfloat16** p, size_t elems) { return aalloc((void**)p, elems * 2); };
  if ((rc = act(&emb, T * C)) || (rc = act(&xa, T * C)) || (rc = act(&xb, T * C)) || (rc = act(&qkv, T * 3 * C)) ||
      (rc = act(&Pm, BH * S * S)) || (rc = act(&vt, T * C)) || (rc = act(&att, T * C)) || (rc = act(&t1, T * C)) ||
      (rc = act(&sa, T * C)) || (rc = act(&h1, T * F)) || (rc = act(&g1, T * F)))
    return rc;
  if ((rc = aalloc((void**)&mean, T * 4)) || (rc = aalloc((void**)&rstd, T * 4))) return rc;
  return SRT_OK;
}

int Bert::forward(int B) {
  const int64_t T = (int64_t)B * S;
  const float scale = 1.f / sqrtf((float)D);
  int rc;
  if ((rc = alloc_activations())) return rc;
  if ((rc = embedding_fwd(ids, pf(wte), pf(wpe), emb, T, S, C, stream))) return rc;
  if ((rc = layernorm_fwd(emb, pf(eln_g), pf(eln_b), xa, mean, rstd, T, C, cfg.ln_eps, stream))) return rc;
  __nv_bfloat16 *x = xa, *nxt = xb;
  for (Layer& y : layers) {
    if ((rc = linear(y.wq, y.bq, C, 3 * C, x, qkv, nullptr, T))) return rc;
    // scores = Q K^T / sqrt(D) per (batch, head), all S x S entries
    BgemmDesc q = {S, S, D, H, B, 3LL * C, D, (long long)S * 3 * C, 3LL * C, D, (long long)S * 3 * C,
                   S, (long long)S * S, (long long)H * S * S, scale, 0, 0};
    if ((rc = bgemm_bf16(q, qkv, qkv + C, Pm, stream))) return rc;
    if ((rc = softmax_rows_fwd(Pm, (int64_t)B * H * S, S, stream))) return rc;
    // context = P V: the B operand is V^T per head, [B][H][D][S]
    if ((rc = batched_transpose(qkv + 2 * C, vt, S, D, 3LL * C, D, (long long)S * 3 * C, H, B, stream))) return rc;
    BgemmDesc o = {S, D, S, H, B, S, (long long)S * S, (long long)H * S * S, S, (long long)D * S, (long long)H * D * S,
                   C, D, (long long)S * C, 1.f, 0, 0};
    if ((rc = bgemm_bf16(o, Pm, vt, att, stream))) return rc;
    if ((rc = linear(y.wo, y.bo, C, C, att, t1, x, T))) return rc;                                   // + residual
    if ((rc = layernorm_fwd(t1, pf(y.ln1_g), pf(y.ln1_b), sa, mean, rstd, T, C, cfg.ln_eps, stream))) return rc;
    if ((rc = linear(y.w1, y.b1, C, F, sa, h1, nullptr, T))) return rc;
    if ((rc = gelu_erf_fwd(h1, g1, T * F, stream))) return rc;
    if ((rc = linear(y.w2, y.b2, F, C, g1, t1, sa, T))) return rc;                                   // + residual
    if ((rc = layernorm_fwd(t1, pf(y.ln2_g), pf(y.ln2_b), nxt, mean, rstd, T, C, cfg.ln_eps, stream))) return rc;
    std::swap(x, nxt);
  }
  out = x;
  return SRT_OK;
}

}  // namespace srt

using namespace srt;

extern "C" {

int srt_bert_create(const srt_bert_config* cfg, srt_pool* pool, srt_bert** out) {
  SRT_REQUIRE(cfg && out, "bert_create: null argument");
  Bert* g = new Bert();
  g->cfg = *cfg;
  g->pool = pool;
  int rc = g->build();
  if (rc == SRT_OK) rc = cudaStreamSynchronize(g->stream) == cudaSuccess ? SRT_OK : SRT_ERR_CUDA;
  if (rc != SRT_OK) { delete g; return rc; }
  *out = (srt_bert*)g;
  return SRT_OK;
}

int srt_bert_destroy(srt_bert* h) {
  if (!h) return SRT_OK;
  delete (Bert*)h;
  return SRT_OK;
}

int srt_bert_num_params(srt_bert* h) { return h ? (int)((Bert*)h)->params.size() : -1; }

int srt_bert_param_info(srt_bert* h, int idx, char* name, int name_cap, int64_t shape[2], int* ndim) {
  Bert* g = (Bert*)h;
  SRT_REQUIRE(g && idx >= 0 && idx < (int)g->params.size(), "bert_param_info: bad index");
  const Bert::Rec& r = g->params[idx];
  if (name && name_cap > 0) { strncpy(name, r.name.c_str(), name_cap - 1); name[name_cap - 1] = 0; }
  if (shape) { shape[0] = r.shape[0]; shape[1] = r.shape[1]; }
  if (ndim) *ndim = r.ndim;
  return SRT_OK;
}

// Host arrays use the reference's state_dict shapes (nn.Linear weights are [out][in], as stored here).
int srt_bert_set_param(srt_bert* h, int idx, const float* host) {
  Bert* g = (Bert*)h;
  SRT_REQUIRE(g && host && idx >= 0 && idx < (int)g->params.size(), "bert_set_param: bad argument");
  const Bert::Rec& r = g->params[idx];
  SRT_CHECK_CUDA(cudaMemcpy(g->P + r.off, host, r.count * 4, cudaMemcpyHostToDevice));
  return SRT_OK;
}

int srt_bert_commit_params(srt_bert* h) {
  Bert* g = (Bert*)h;
  SRT_REQUIRE(g, "bert_commit_params: null handle");
  int rc = cast_f32_to_bf16(g->P, g->Pw, (int64_t)g->n_flat, g->stream);
  if (rc) return rc;
  SRT_CHECK_CUDA(cudaStreamSynchronize(g->stream));
  return SRT_OK;
}

int srt_bert_upload_tokens(srt_bert* h, const int32_t* host_ids, int B) {
  Bert* g = (Bert*)h;
  SRT_REQUIRE(g && host_ids && B > 0 && B <= g->cfg.max_batch, "bert_upload_tokens: bad argument");
  const int T = B * g->S;
  for (int t = 0; t < T; ++t)
    SRT_REQUIRE(host_ids[t] >= 0 && host_ids[t] < g->V, "bert_upload_tokens: token id %d outside the vocabulary", host_ids[t]);
  SRT_CHECK_CUDA(cudaMemcpyAsync(g->ids, host_ids, (size_t)T * 4, cudaMemcpyHostToDevice, g->stream));
  SRT_CHECK_CUDA(cudaStreamSynchronize(g->stream));
  g->cur_B = B;
  return SRT_OK;
}

int srt_bert_forward(srt_bert* h, int B) {
  Bert* g = (Bert*)h;
  SRT_REQUIRE(g && B > 0 && B == g->cur_B, "bert_forward: upload the tokens of this batch first");
  return g->forward(B);
}

int srt_bert_output(srt_bert* h, float* host, int B) {
  Bert* g = (Bert*)h;
  SRT_REQUIRE(g && host && B > 0 && B <= g->cfg.max_batch && g->out, "bert_output: run a forward pass first");
  const size_t n = (size_t)B * g->S * g->C;
  std::vector<uint16_t> tmp(n);
  SRT_CHECK_CUDA(cudaStreamSynchronize(g->stream));
  SRT_CHECK_CUDA(cudaMemcpy(tmp.data(), g->out, n * 2, cudaMemcpyDeviceToHost));
  for (size_t i = 0; i < n; ++i) {
    const uint32_t bits = (uint32_t)tmp[i] << 16;
    memcpy(&host[i], &bits, 4);
  }
  return SRT_OK;
}

int srt_bert_synchronize(srt_bert* h) {
  Bert* g = (Bert*)h;
  SRT_REQUIRE(g, "bert_synchronize: null handle");
  SRT_CHECK_CUDA(cudaStreamSynchronize(g->stream));
  return SRT_OK;
}

int srt_bert_stream(srt_bert* h, void** stream) {
  Bert* g = (Bert*)h;
  SRT_REQUIRE(g && stream, "bert_stream: null argument");
  *stream = (void*)g->stream;
  return SRT_OK;
}

int srt_bert_release_activations(srt_bert* h, size_t* released_bytes) {
  Bert* g = (Bert*)h;
  SRT_REQUIRE(g, "bert_release_activations: null handle");
  size_t freed = g->act_bytes;
  int rc = g->free_activations();
  if (rc) return rc;
  if (g->pool && (rc = srt_pool_empty_cache(g->pool, SRT_POOL_INFER, &freed))) return rc;
  if (released_bytes) *released_bytes = freed;
  return SRT_OK;
}

int srt_bert_reserve_activations(srt_bert* h) {
  Bert* g = (Bert*)h;
  SRT_REQUIRE(g, "bert_reserve_activations: null handle");
  return g->alloc_activations();
}

int srt_bert_memory_bytes(srt_bert* h, size_t* weights, size_t* activations) {
  Bert* g = (Bert*)h;
  SRT_REQUIRE(g, "bert_memory_bytes: null handle");
  if (weights) *weights = g->bytes_total;
  if (activations) *activations = g->act_bytes;
  return SRT_OK;
}

}  // extern "C"
