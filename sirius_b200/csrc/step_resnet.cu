// Training-step executor for torchvision-layout bottleneck ResNets (ResNet-50/101/152).
//
// One object owns every device buffer of the step (flat fp32 master parameters, gradients,
// momentum, optional bf16 working copy, saved activations, gradient ping-pong buffers, scratch)
// and replays the forward / backward / optimizer sequence as kernel launches on one stream.
// It stands where the reference runs `model(images)`, `criterion`, `scaler.scale(loss).backward()`
// and the optimizer stage of MicroBatchManager (train/resnet152.py:84-91,
// pytorch/torch_col/dynamic_batch.py:112-153, pytorch/torch_col/accumulate.py:7-49).
#include <string.h>

#include <string>
#include <chrono>
#include <vector>

#include <atomic>

#include "../../include/sirius_pool.h"
#include "../../include/sirius_runtime.h"
#include "common.cuh"
#include "ops.cuh"


namespace srt {

namespace {

constexpr int kStemCpad = 8;  // RGB input is zero-padded to 8 channels (16-byte vectors)

struct ParamRec {
  std::string name;
  int kind;          // SRT_PARAM_*
  int64_t shape[4];  // torch layout
  int ndim;
  size_t off;        // element offset into the flat buffers (kind != BUFFER) or buffer arena
  size_t count;      // internal element count (with channel padding)
  int cpad;          // internal channels (conv weights)
};

struct ConvL {
  int C, K, R, S, stride, pad;  // C = internal (padded) channels
  int w;                        // param index
  size_t wt_off;                // element offset of the transposed copy (dgrad operand)
  size_t s2_off;                // 3x3 stride-2 filters: element offset of the four parity sub-filters in the same arena
};
struct BNL {
  int C;
  int gamma, beta, rmean, rvar;  // param indices
  float *mean, *invstd, *scale, *shift;
};
struct Unit {
  ConvL conv;
  BNL bn;
  int relu;
  void* z;  // conv output (pre-BN)
  void* y;  // post BN (+residual) (+ReLU)
  int H, W, P, Q;  // input and output spatial size
  // Residual units in bf16: the ReLU mask of y as one bit per element, written by the forward apply pass. The
  // backward pass reads it instead of y (twice), and the first convolution's data gradient adds the block's output
  // gradient under it, so no masked copy of that gradient is written either.
  uint8_t* bits = nullptr;
  bool bits_valid = false;  // the bits belong to the last forward pass
};
struct Block {
  Unit u1, u2, u3, ds;
  bool has_ds;
};

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace

struct Step {
  srt_resnet_config cfg;
  cudaStream_t stream = nullptr;
  bool own_stream = false;
  size_t esz = 4;  // activation element size

  std::vector<ParamRec> params;
  size_t n_flat = 0;     // elements in P/G/M/ACC
  size_t n_buf = 0;      // elements in BN running-stat arena
  size_t n_wt = 0;       // elements in the transposed-filter arena
  float *P = nullptr, *G = nullptr, *M = nullptr, *ACC = nullptr, *BUF = nullptr;
  void* Pw = nullptr;    // working copy of P in the compute dtype (== P in fp32 mode)
  void* WT = nullptr;    // transposed filters in the compute dtype
  float* bn_vec = nullptr;

  Unit stem;
  std::vector<Block> blocks;
  int fc_w = -1, fc_b = -1;
  int feat_C = 0, final_HW = 0;

  // activations
  void *x0 = nullptr, *pool_y = nullptr, *avg = nullptr, *logits = nullptr, *dlogits = nullptr;
  uint8_t* pool_arg = nullptr;
  void* T[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  void* scratch = nullptr;
  size_t scratch_bytes = 0;
  void* s2_tmp = nullptr;      // the four parity classes of a stride-2 data gradient before they are interleaved
  void* scratch_wg = nullptr;  // split partials of the filter-gradient kernels (they run beside BatchNorm)
  size_t scratch_wg_bytes = 0;
  // Backward overlap: the filter gradient of a unit depends only on (dz, saved input), not on anything
  // later in the chain, so it runs on a second, lowest-priority stream beside the data gradient and the
  // next BatchNorm backward and fills the SMs those leave idle. dz buffers alternate so that the next
  // unit does not have to wait for the reader; a write to a buffer waits for its pending reader.
  cudaStream_t side = nullptr;
  cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
  cudaEvent_t ev_read[6] = {nullptr};
  bool read_pending[6] = {false};  // indexed by position in T; only T[1], T[3], T[5] are ever read by the side
                                   // stream, and those never take part in the T[0]/T[4] swap
  bool side_dirty = false;         // side-stream work queued that the main stream has not waited for
  bool wt_dirty = false;           // ... of which only filter transposes (the forward pass need not wait for those)
  bool overlap_wgrad = getenv("SIRIUS_B200_NO_OVERLAP") == nullptr;  // weight gradients on the second stream
  bool fused_bn = getenv("SIRIUS_B200_NO_FUSED_BN") == nullptr;  // one-launch BatchNorm for the tensors that sit in L2
  bool conv_stats = getenv("SIRIUS_B200_NO_CONV_STATS") == nullptr;  // BatchNorm sums taken in the convolution's epilogue
  bool relu_bits = getenv("SIRIUS_B200_NO_RELU_BITS") == nullptr;    // residual units keep their ReLU mask as bits (bf16)
  // Gradient buckets for the data-parallel all-reduce, in the order backward completes them (fc and the
  // last blocks first). A bucket's event fires when every gradient in its range is final.
  struct GradBucket { size_t off, count; int first_block; cudaEvent_t ev; };
  std::vector<GradBucket> buckets;
  int build_buckets(size_t bucket_elems);
  int bucket_ready(int b, bool on_side);
  bool use_side() const { return side && overlap_wgrad && !prof_on; }
  int t_slot(const void* p) const { for (int i = 0; i < 6; ++i) if (T[i] == p) return i; return -1; }
  int before_write(const void* buf) {   // main stream is about to overwrite buf
    const int i = t_slot(buf);
    if (i >= 0 && read_pending[i]) {
      SRT_CHECK_CUDA(cudaStreamWaitEvent(stream, ev_read[i], 0));
      read_pending[i] = false;
    }
    return SRT_OK;
  }
  int join_side() {                      // main stream continues after everything queued on the side stream
    if (!side || !(side_dirty || wt_dirty)) return SRT_OK;
    side_dirty = wt_dirty = false;
    SRT_CHECK_CUDA(cudaEventRecord(ev_join, side));
    SRT_CHECK_CUDA(cudaStreamWaitEvent(stream, ev_join, 0));
    for (bool& b : read_pending) b = false;
    return SRT_OK;
  }
  float *row_loss = nullptr, *loss_acc = nullptr;
  float* stage_images = nullptr;   // device staging of the NCHW fp32 batch the next forward reads (one of the two below)
  int64_t* stage_labels = nullptr;
  // Double-buffered staging: a host batch is copied on its own stream into the buffer the executor is not reading,
  // so the copy of the next batch runs beside the current step (what pinned memory + non_blocking copies give the
  // reference's loader). ev_up: copy landed; ev_used: the step has consumed the buffer.
  float* stage_images_b[2] = {nullptr, nullptr};
  int64_t* stage_labels_b[2] = {nullptr, nullptr};
  cudaStream_t copy_stream = nullptr;
  cudaEvent_t ev_up[2] = {nullptr, nullptr}, ev_used[2] = {nullptr, nullptr};
  bool used_pending[2] = {false, false};
  int up_next = 0, pending_up = -1, cur_buf = 0;
  std::vector<void*> allocs;

  int opt_steps = 0;
  bool eval_mode = false;  // forward with BatchNorm running statistics (the inference stand-in)
  int accum_pending = 0;
  size_t act_bytes = 0;

  // Releasable part of the step's memory: saved activations, gradient ping-pong buffers, scratch.
  // Taken from the training allocator of a page pool when one is attached (so that releasing them
  // and emptying the allocator's cache hands whole pages to the inference side), else cudaMalloc.
  srt_pool* pool = nullptr;
  int pool_kind = SRT_POOL_TRAIN;  // which allocator of the pool serves this step (INFER for the stand-in worker)
  int act_batch = 0;               // batch size the activation set is currently sized for (0 = released)
  std::vector<void*> act_blocks;
  // Kill-batch support: a flag any thread may raise; forward/backward look at it between units and
  // keep at most kLaunchAhead units in flight, so an abort drains within a bounded time.
  std::atomic<int> abort_flag{0};
  static constexpr int kLaunchAhead = 8;
  cudaEvent_t ahead_ev[kLaunchAhead] = {nullptr};
  unsigned long long unit_seq = 0;

  int aalloc(void** out, size_t bytes) {
    bytes = bytes ? bytes : 256;
    if (pool) {
      int rc = srt_pool_alloc(pool, pool_kind, bytes, out);
      if (rc) return rc;
    } else {
      SRT_CHECK_CUDA(cudaMalloc(out, (bytes + 255) / 256 * 256));
    }
    act_blocks.push_back(*out);
    act_bytes += bytes;
    return SRT_OK;
  }
  // The batch uploaded last becomes the one the next forward reads: wait for its copy, switch buffers.
  int adopt_upload() {
    if (pending_up < 0) return SRT_OK;
    const int idx = pending_up;
    pending_up = -1;
    SRT_CHECK_CUDA(cudaStreamWaitEvent(stream, ev_up[idx], 0));
    cur_buf = idx;
    stage_images = stage_images_b[idx];
    stage_labels = stage_labels_b[idx];
    return SRT_OK;
  }
  // Called once the step's kernels that read the staging buffer are enqueued: a later upload into it must wait for them.
  int staging_consumed() {
    SRT_CHECK_CUDA(cudaEventRecord(ev_used[cur_buf], stream));
    used_pending[cur_buf] = true;
    return SRT_OK;
  }
  int alloc_activations(int B);
  int free_activation_blocks();
  int release_activations(size_t* released_bytes);
  int shrink_activations(int B, size_t* released_bytes);
  // SM partition: when on, the step moves between green-context streams so that its kernels only run
  // on as many SMs as the process-wide allowed-SM mask has bits (see sm_partition.cu).
  bool follow_mask = false;
  cudaStream_t home_stream = nullptr;  // the stream the step was created with (whole device)
  cudaStream_t home_side = nullptr;    // ... and its low-priority companion
  int cur_sms = 0;                     // 0 = whole device
  cudaEvent_t switch_ev = nullptr;
  // Source of the allowed SM count: the inference side's required-TPC counter on the information
  // board when one is attached (what the reference's pre-launch hook reads), else the process-wide mask.
  srt_comm* tpc_comm = nullptr;
  int tpc_device = 0, tpc_min_train = 1, tpc_max_train = 1 << 20;
  int follow_sm_mask() {
    const int total = sm_count_device();
    int allowed = 0;
    if (tpc_comm) {
      int req = 0;
      int rc = srt_comm_infer_tpc(tpc_comm, tpc_device, 3, 0, &req);
      if (rc) return rc;
      allowed = 2 * srt_smp_train_avail_tpc_num(req, total / 2, tpc_min_train, tpc_max_train);
    } else {
      const SmMask m = current_sm_mask();
      for (int i = 0; i < total; ++i) allowed += (int)((m.w[i >> 6] >> (i & 63)) & 1ull);
    }
    cudaStream_t want = nullptr, want_side = nullptr;
    int sms = total;
    int rc = partition_streams(cfg_device, allowed, &want, &want_side, &sms);
    if (rc) return rc;
    if (!want) { want = home_stream; want_side = home_side; sms = 0; }
    if (want == stream) return SRT_OK;
    if (!switch_ev) SRT_CHECK_CUDA(cudaEventCreateWithFlags(&switch_ev, cudaEventDisableTiming));
    SRT_CHECK_CUDA(cudaEventRecord(switch_ev, stream));   // the new stream continues after everything queued so far
    SRT_CHECK_CUDA(cudaStreamWaitEvent(want, switch_ev, 0));
    if (side && want_side && want_side != side) {           // the companion stream moves with it, in order
      SRT_CHECK_CUDA(cudaEventRecord(switch_ev, side));
      SRT_CHECK_CUDA(cudaStreamWaitEvent(want_side, switch_ev, 0));
      side = want_side;
    }
    stream = want;
    cur_sms = sms;
    return SRT_OK;
  }
  int cfg_device = 0;
  static int sm_count_device() {
    const int lim = sm_limit();
    set_sm_limit(0);
    const int n = sm_count();
    set_sm_limit(lim);
    return n;
  }
  // Grid sizing of the calling thread follows the partition while the step's entry points run.
  struct SmScope {
    int saved;
    bool saved_pdl;
    explicit SmScope(const Step* s) : saved(sm_limit()), saved_pdl(pdl_big_kernels()) {
      if (s->follow_mask) set_sm_limit(s->cur_sms);
      set_pdl_big_kernels(true);
    }
    ~SmScope() { set_sm_limit(saved); set_pdl_big_kernels(saved_pdl); }
  };

  // Called between units: abort check + bounded launch-ahead.
  int checkpoint() {
    if (abort_flag.load(std::memory_order_acquire)) {
      set_error("step aborted between units (kill batch)");
      return SRT_ERR_ABORTED;
    }
    if (follow_mask) {
      int rc = follow_sm_mask();
      if (rc) return rc;
      set_sm_limit(cur_sms);
    }
    const int slot = (int)(unit_seq % kLaunchAhead);
    if (!ahead_ev[slot]) SRT_CHECK_CUDA(cudaEventCreateWithFlags(&ahead_ev[slot], cudaEventDisableTiming));
    else if (unit_seq >= (unsigned long long)kLaunchAhead) SRT_CHECK_CUDA(cudaEventSynchronize(ahead_ev[slot]));
    SRT_CHECK_CUDA(cudaEventRecord(ahead_ev[slot], stream));
    ++unit_seq;
    return SRT_OK;
  }

  // Optional per-category device timing (CUDA events on the step's stream around each launch).
  bool prof_on = false;
  struct ProfRec { int cat; double work; cudaEvent_t a, b; };
  std::vector<ProfRec> prof_recs;
  std::vector<cudaEvent_t> prof_pool;
  double prof_ms[SRT_PROF_NCAT] = {0}, prof_work[SRT_PROF_NCAT] = {0};
  long long prof_launches[SRT_PROF_NCAT] = {0};
  template <class F>
  int timed(int cat, double work, F&& f) {
    if (!prof_on) return f();
    auto get = [&]() {
      cudaEvent_t e;
      if (!prof_pool.empty()) { e = prof_pool.back(); prof_pool.pop_back(); }
      else cudaEventCreate(&e);
      return e;
    };
    ProfRec r{cat, work, get(), get()};
    cudaEventRecord(r.a, stream);
    const int rc = f();
    cudaEventRecord(r.b, stream);
    prof_recs.push_back(r);
    return rc;
  }
  void prof_collect() {
    cudaStreamSynchronize(stream);
    for (auto& r : prof_recs) {
      float ms = 0.f;
      if (cudaEventElapsedTime(&ms, r.a, r.b) == cudaSuccess) {
        prof_ms[r.cat] += ms; prof_work[r.cat] += r.work; prof_launches[r.cat]++;
      }
      prof_pool.push_back(r.a); prof_pool.push_back(r.b);
    }
    prof_recs.clear();
  }

  ~Step() {
    for (auto& r : prof_recs) { cudaEventDestroy(r.a); cudaEventDestroy(r.b); }
    for (auto e : prof_pool) cudaEventDestroy(e);
    for (auto e : ahead_ev) if (e) cudaEventDestroy(e);
    release_activations(nullptr);
    for (void* p : allocs) cudaFree(p);
    if (switch_ev) cudaEventDestroy(switch_ev);
    for (int i = 0; i < 2; ++i) { if (ev_up[i]) cudaEventDestroy(ev_up[i]); if (ev_used[i]) cudaEventDestroy(ev_used[i]); }
    if (copy_stream) { cudaStreamSynchronize(copy_stream); cudaStreamDestroy(copy_stream); }
    for (auto& b : buckets) if (b.ev) cudaEventDestroy(b.ev);
    if (ev_fork) cudaEventDestroy(ev_fork);
    if (ev_join) cudaEventDestroy(ev_join);
    for (auto e : ev_read) if (e) cudaEventDestroy(e);
    if (home_side) cudaStreamDestroy(home_side);  // partition streams belong to the ladder
    if (own_stream && home_stream) cudaStreamDestroy(home_stream);  // partition streams belong to the ladder
  }
  int dalloc(void** out, size_t bytes, bool zero) {
    bytes = align_up(bytes ? bytes : 256, 256);
    SRT_CHECK_CUDA(cudaMalloc(out, bytes));
    allocs.push_back(*out);
    if (zero) SRT_CHECK_CUDA(cudaMemset(*out, 0, bytes));
    return SRT_OK;
  }
  int add_param(const std::string& name, int kind, std::initializer_list<int64_t> shape, int cpad) {
    ParamRec r;
    r.name = name;
    r.kind = kind;
    r.ndim = (int)shape.size();
    int i = 0;
    size_t cnt = 1;
    for (int64_t s : shape) { r.shape[i++] = s; cnt *= (size_t)s; }
    for (; i < 4; ++i) r.shape[i] = 1;
    r.cpad = cpad;
    if (kind == SRT_PARAM_CONV) cnt = (size_t)r.shape[0] * r.shape[2] * r.shape[3] * cpad;
    r.count = cnt;
    if (kind == SRT_PARAM_BUFFER) { r.off = n_buf; n_buf += align_up(cnt, 64); }
    else { r.off = n_flat; n_flat += align_up(cnt, 64); }
    params.push_back(r);
    return (int)params.size() - 1;
  }
  ConvL make_conv(const std::string& name, int Cin_real, int K, int R, int stride, int pad) {
    ConvL c;
    c.C = Cin_real < 8 ? kStemCpad : Cin_real;
    c.K = K; c.R = R; c.S = R; c.stride = stride; c.pad = pad;
    c.w = add_param(name + ".weight", SRT_PARAM_CONV, {K, Cin_real, R, R}, c.C);
    c.wt_off = n_wt;
    n_wt += align_up((size_t)K * R * R * c.C, 64);
    c.s2_off = n_wt;
    if (stride == 2 && R == 3) n_wt += align_up((size_t)K * R * R * c.C, 64);  // taps regrouped by output parity
    return c;
  }
  BNL make_bn(const std::string& name, int C) {
    BNL b;
    b.C = C;
    b.gamma = add_param(name + ".weight", SRT_PARAM_VECTOR, {C}, 0);
    b.beta = add_param(name + ".bias", SRT_PARAM_VECTOR, {C}, 0);
    b.rmean = add_param(name + ".running_mean", SRT_PARAM_BUFFER, {C}, 0);
    b.rvar = add_param(name + ".running_var", SRT_PARAM_BUFFER, {C}, 0);
    b.mean = b.invstd = b.scale = b.shift = nullptr;
    return b;
  }
  float* pf(int idx) { return P + params[idx].off; }
  float* gf(int idx) { return G + params[idx].off; }
  float* bf_(int idx) { return BUF + params[idx].off; }
  void* pw(int idx) { return (char*)Pw + params[idx].off * esz; }
  void* wt(const ConvL& c) { return (char*)WT + c.wt_off * esz; }

  int build();
  int refresh_working_copies();
  bool s2_fast(const ConvL& c) const { return cfg.dtype == SRT_BF16 && cfg.impl != SRT_IMPL_SIMT && c.stride == 2 && (c.R == 1 || (c.R == 3 && c.pad == 1)); }
  int build_subfilters(const ConvL& c, cudaStream_t st);
  int dgrad_s2(const Unit& u, const void* dz, void* dx, const void* addend, int B);
  int forward(int B);
  int backward(int B);
};

int Step::build() {
  const int dtype = cfg.dtype;
  esz = dtype == SRT_F32 ? 4 : 2;
  const int B = cfg.max_batch, IMG = cfg.image;
  SRT_REQUIRE(B > 0 && IMG >= 32 && IMG % 32 == 0, "resnet: max_batch > 0 and image a multiple of 32 required");

  // ---- topology + parameter registry (torchvision names) ----
  stem.conv = make_conv("conv1", 3, 64, 7, 2, 3);
  stem.bn = make_bn("bn1", 64);
  stem.relu = 1;
  stem.H = stem.W = IMG;
  stem.P = stem.Q = IMG / 2;
  int H = IMG / 4, inC = 64;
  const int widths[4] = {64, 128, 256, 512};
  for (int l = 0; l < 4; ++l) {
    for (int b = 0; b < cfg.layers[l]; ++b) {
      const std::string pre = "layer" + std::to_string(l + 1) + "." + std::to_string(b);
      const int width = widths[l], outC = width * 4;
      const int stride = (b == 0 && l > 0) ? 2 : 1;
      Block blk;
      blk.u1.conv = make_conv(pre + ".conv1", inC, width, 1, 1, 0);
      blk.u1.bn = make_bn(pre + ".bn1", width);
      blk.u1.relu = 1; blk.u1.H = blk.u1.W = H; blk.u1.P = blk.u1.Q = H;
      blk.u2.conv = make_conv(pre + ".conv2", width, width, 3, stride, 1);
      blk.u2.bn = make_bn(pre + ".bn2", width);
      blk.u2.relu = 1; blk.u2.H = blk.u2.W = H; blk.u2.P = blk.u2.Q = H / stride;
      blk.u3.conv = make_conv(pre + ".conv3", width, outC, 1, 1, 0);
      blk.u3.bn = make_bn(pre + ".bn3", outC);
      blk.u3.relu = 1; blk.u3.H = blk.u3.W = H / stride; blk.u3.P = blk.u3.Q = H / stride;
      blk.has_ds = (b == 0);
      if (blk.has_ds) {
        blk.ds.conv = make_conv(pre + ".downsample.0", inC, outC, 1, stride, 0);
        blk.ds.bn = make_bn(pre + ".downsample.1", outC);
        blk.ds.relu = 0; blk.ds.H = blk.ds.W = H; blk.ds.P = blk.ds.Q = H / stride;
      }
      blocks.push_back(blk);
      inC = outC;
      H /= stride;
    }
  }
  feat_C = inC;
  final_HW = H * H;
  fc_w = add_param("fc.weight", SRT_PARAM_LINEAR, {cfg.num_classes, feat_C}, 0);
  fc_b = add_param("fc.bias", SRT_PARAM_VECTOR, {cfg.num_classes}, 0);
  const size_t fc_wt_off = n_wt;
  n_wt += align_up((size_t)cfg.num_classes * feat_C, 64);
  (void)fc_wt_off;
  SRT_REQUIRE(cfg.num_classes % 8 == 0, "resnet: num_classes must be a multiple of 8");

  // ---- device memory ----
  int rc;
  if ((rc = dalloc((void**)&P, n_flat * 4, true))) return rc;
  if ((rc = dalloc((void**)&G, n_flat * 4, true))) return rc;
  if ((rc = dalloc((void**)&M, n_flat * 4, true))) return rc;
  if ((rc = dalloc((void**)&ACC, n_flat * 4, true))) return rc;
  if ((rc = dalloc((void**)&BUF, n_buf * 4, true))) return rc;
  if (dtype == SRT_F32) Pw = P;
  else if ((rc = dalloc(&Pw, n_flat * 2, true))) return rc;
  if ((rc = dalloc(&WT, n_wt * esz, true))) return rc;

  size_t bn_elems = 0;
  auto count_bn = [&](BNL& b) { bn_elems += 4 * align_up(b.C, 64); };
  count_bn(stem.bn);
  for (auto& k : blocks) { count_bn(k.u1.bn); count_bn(k.u2.bn); count_bn(k.u3.bn); if (k.has_ds) count_bn(k.ds.bn); }
  if ((rc = dalloc((void**)&bn_vec, bn_elems * 4, true))) return rc;
  float* cur = bn_vec;
  auto place_bn = [&](BNL& b) {
    const size_t a = align_up(b.C, 64);
    b.mean = cur; b.invstd = cur + a; b.scale = cur + 2 * a; b.shift = cur + 3 * a;
    cur += 4 * a;
  };
  place_bn(stem.bn);
  for (auto& k : blocks) { place_bn(k.u1.bn); place_bn(k.u2.bn); place_bn(k.u3.bn); if (k.has_ds) place_bn(k.ds.bn); }

  if ((rc = dalloc(&avg, (size_t)B * feat_C * esz, false))) return rc;
  if ((rc = dalloc(&logits, (size_t)B * cfg.num_classes * esz, false))) return rc;
  if ((rc = dalloc(&dlogits, (size_t)B * cfg.num_classes * esz, false))) return rc;
  if ((rc = dalloc((void**)&row_loss, (size_t)B * 4, true))) return rc;
  if ((rc = dalloc((void**)&loss_acc, 256, true))) return rc;
  for (int i = 0; i < 2; ++i) {
    if ((rc = dalloc((void**)&stage_images_b[i], (size_t)B * 3 * IMG * IMG * 4, false))) return rc;
    if ((rc = dalloc((void**)&stage_labels_b[i], (size_t)B * 8, false))) return rc;
    SRT_CHECK_CUDA(cudaEventCreateWithFlags(&ev_up[i], cudaEventDisableTiming));
    SRT_CHECK_CUDA(cudaEventCreateWithFlags(&ev_used[i], cudaEventDisableTiming));
  }
  stage_images = stage_images_b[0];
  stage_labels = stage_labels_b[0];
  SRT_CHECK_CUDA(cudaStreamCreateWithFlags(&copy_stream, cudaStreamNonBlocking));

  if (pool_kind == SRT_POOL_INFER) {
    // the inference stand-in runs on the highest-priority stream so its blocks are scheduled ahead of
    // training blocks whenever an SM frees a slot
    int lo = 0, hi = 0;
    SRT_CHECK_CUDA(cudaDeviceGetStreamPriorityRange(&lo, &hi));
    SRT_CHECK_CUDA(cudaStreamCreateWithPriority(&stream, cudaStreamNonBlocking, hi));
  } else {
    SRT_CHECK_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
  }
  own_stream = true;
  home_stream = stream;
  if (pool_kind != SRT_POOL_INFER) {
    int lo = 0, hi = 0;
    SRT_CHECK_CUDA(cudaDeviceGetStreamPriorityRange(&lo, &hi));
    SRT_CHECK_CUDA(cudaStreamCreateWithPriority(&side, cudaStreamNonBlocking, lo));
    home_side = side;
    SRT_CHECK_CUDA(cudaEventCreateWithFlags(&ev_fork, cudaEventDisableTiming));
    SRT_CHECK_CUDA(cudaEventCreateWithFlags(&ev_join, cudaEventDisableTiming));
    for (auto& e : ev_read) SRT_CHECK_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  }
  SRT_CHECK_CUDA(cudaGetDevice(&cfg_device));
  if ((rc = alloc_activations(B))) return rc;

  // BN defaults (weight 1, bias 0, running_var 1); conv/fc weights are set by the caller.
  std::vector<float> ones;
  for (auto& r : params) {
    const bool bn_weight = r.kind == SRT_PARAM_VECTOR && r.name.size() > 7 &&
                           r.name.compare(r.name.size() - 7, 7, ".weight") == 0;
    const bool rvar = r.kind == SRT_PARAM_BUFFER && r.name.find("running_var") != std::string::npos;
    if (bn_weight || rvar) {
      ones.assign(r.count, 1.f);
      float* dst = rvar ? BUF + r.off : P + r.off;
      SRT_CHECK_CUDA(cudaMemcpy(dst, ones.data(), r.count * 4, cudaMemcpyHostToDevice));
    }
  }
  if ((rc = build_buckets((size_t)25 << 18))) return rc;  // 25 MiB of fp32 gradients per bucket, as c10d's default
  return refresh_working_copies();
}

int Step::build_buckets(size_t bucket_elems) {
  for (auto& b : buckets) if (b.ev) cudaEventDestroy(b.ev);
  buckets.clear();
  size_t end = n_flat;
  for (int i = (int)blocks.size() - 1; i >= 0; --i) {
    const size_t start = params[blocks[i].u1.conv.w].off;
    if (end - start >= bucket_elems && i > 0) {
      buckets.push_back({start, end - start, i, nullptr});
      end = start;
    }
  }
  // The last bucket is ready only when backward ends, so its exchange is the part that cannot hide behind compute:
  // keep it small. When "the rest" is large, cut it once more at the first block that starts at least 1 MiB into the
  // buffer (the stem, layer1 and the head of layer2 stay: a couple of megabytes whose all-reduce is latency-bound).
  constexpr size_t kTailElems = (size_t)1 << 18;
  if (end > 4 * kTailElems) {
    for (int i = 1; i < (int)blocks.size(); ++i) {
      const size_t start = params[blocks[i].u1.conv.w].off;
      if (start >= end) break;
      if (start >= kTailElems) {
        buckets.push_back({start, end - start, i, nullptr});
        end = start;
        break;
      }
    }
  }
  buckets.push_back({0, end, -1, nullptr});  // the rest, stem included: ready when backward is
  for (auto& b : buckets) SRT_CHECK_CUDA(cudaEventCreateWithFlags(&b.ev, cudaEventDisableTiming));
  return SRT_OK;
}

// Records bucket b's event behind the last kernel that writes into its range.
int Step::bucket_ready(int b, bool on_side) {
  if (on_side) {  // filter gradients come from the side stream, BatchNorm gradients from the main one
    SRT_CHECK_CUDA(cudaEventRecord(ev_fork, stream));
    SRT_CHECK_CUDA(cudaStreamWaitEvent(side, ev_fork, 0));
    SRT_CHECK_CUDA(cudaEventRecord(buckets[b].ev, side));
  } else {
    SRT_CHECK_CUDA(cudaEventRecord(buckets[b].ev, stream));
  }
  return SRT_OK;
}

// Activation set for micro-batches of up to B samples.
int Step::alloc_activations(int B) {
  SRT_REQUIRE(B > 0 && B <= cfg.max_batch, "activations: batch %d outside 1..%d", B, cfg.max_batch);
  if (act_batch == B) return SRT_OK;
  // the old set goes back to the allocator but its pages stay mapped: the new set lands on them again
  // and only the difference is mapped (growing) or left for the next empty-cache (shrinking)
  int rc = free_activation_blocks();
  if (rc) return rc;
  const int dtype = cfg.dtype, IMG = cfg.image;
  size_t max_act = 0, max_bn_scratch = 0, max_wg_scratch = 0;
  auto alloc_unit = [&](Unit& u, bool with_bits = false) -> int {
    const size_t elems = (size_t)B * u.P * u.Q * u.conv.K;
    if (elems > max_act) max_act = elems;
    int r;
    if ((r = aalloc(&u.z, elems * esz))) return r;
    if ((r = aalloc(&u.y, elems * esz))) return r;
    u.bits = nullptr;
    u.bits_valid = false;
    if (with_bits && relu_bits && dtype == SRT_BF16 && u.relu && (r = aalloc((void**)&u.bits, elems / 8))) return r;
    const size_t bs = bn_scratch_bytes((int64_t)B * u.P * u.Q, u.conv.K);
    if (bs > max_bn_scratch) max_bn_scratch = bs;
    srt_conv_desc d = {B, u.H, u.W, u.conv.C, u.conv.K, u.conv.R, u.conv.S, u.conv.stride, u.conv.pad, u.P, u.Q};
    const size_t ws = conv_wgrad_scratch_bytes(d, dtype, cfg.impl);
    if (ws > max_wg_scratch) max_wg_scratch = ws;
    if (conv_stats && conv_fprop_stats_supported(d, dtype, cfg.impl)) {
      const size_t cs = conv_fprop_stats_bytes(d);
      if (cs > max_bn_scratch) max_bn_scratch = cs;
    }
    return SRT_OK;
  };
  if ((rc = alloc_unit(stem))) return rc;
  for (auto& k : blocks) {
    if ((rc = alloc_unit(k.u1))) return rc;
    if ((rc = alloc_unit(k.u2))) return rc;
    if ((rc = alloc_unit(k.u3, true))) return rc;
    if (k.has_ds && (rc = alloc_unit(k.ds))) return rc;
  }
  {
    srt_conv_desc d = {B, 1, 1, feat_C, cfg.num_classes, 1, 1, 1, 0, 1, 1};
    const size_t ws = conv_wgrad_scratch_bytes(d, dtype, cfg.impl);
    if (ws > max_wg_scratch) max_wg_scratch = ws;
  }
  const size_t x0_elems = (size_t)B * IMG * IMG * kStemCpad;
  if (x0_elems > max_act) max_act = x0_elems;
  if ((rc = aalloc(&x0, x0_elems * esz))) return rc;
  const size_t pool_elems = (size_t)B * (IMG / 4) * (IMG / 4) * 64;
  if ((rc = aalloc(&pool_y, pool_elems * esz))) return rc;
  if ((rc = aalloc((void**)&pool_arg, pool_elems))) return rc;
  for (int i = 0; i < 6; ++i)
    if ((rc = aalloc(&T[i], max_act * esz))) return rc;
  scratch_bytes = max_bn_scratch > max_wg_scratch ? max_bn_scratch : max_wg_scratch;  // the fc wgrad uses it too
  if ((rc = aalloc(&scratch, scratch_bytes))) return rc;
  if ((rc = aalloc(&s2_tmp, max_act * esz))) return rc;
  scratch_wg_bytes = max_wg_scratch;
  if ((rc = aalloc(&scratch_wg, scratch_wg_bytes))) return rc;
  act_batch = B;
  return SRT_OK;
}

// Waits for the stream and hands every activation block back to its allocator (pages stay mapped).
int Step::free_activation_blocks() {
  if (stream && !act_blocks.empty()) SRT_CHECK_CUDA(cudaStreamSynchronize(stream));
  if (side && !act_blocks.empty()) SRT_CHECK_CUDA(cudaStreamSynchronize(side));  // an aborted backward never joined
  for (bool& b : read_pending) b = false;
  side_dirty = wt_dirty = false;
  for (void* p : act_blocks) {
    if (pool) {
      int rc = srt_pool_free(pool, pool_kind, p);
      if (rc) return rc;
    } else {
      cudaFree(p);
    }
  }
  act_blocks.clear();
  act_bytes = 0;
  act_batch = 0;
  return SRT_OK;
}

namespace {
struct PhaseTrace {  // SIRIUS_B200_TRACE=1 prints the phases of a release to stderr
  const char* what;
  bool on;
  std::chrono::steady_clock::time_point t[4];
  int n = 0;
  explicit PhaseTrace(const char* w) : what(w) {
    static const bool env = getenv("SIRIUS_B200_TRACE") != nullptr;
    on = env;
    mark();
  }
  void mark() { if (on && n < 4) t[n++] = std::chrono::steady_clock::now(); }
  void print(size_t freed) {
    if (!on) return;
    mark();
    auto ms = [&](int i) { return i + 1 < n ? std::chrono::duration<double, std::milli>(t[i + 1] - t[i]).count() : 0.0; };
    fprintf(stderr, "[sirius_b200] %s: free %.2f ms, regain %.2f ms, unmap %.2f ms, %zu MiB returned\n", what, ms(0), ms(1),
            ms(2), freed >> 20);
  }
};
}  // namespace

// Frees the activation set; with a pool attached, also returns every page that became empty.
int Step::release_activations(size_t* released_bytes) {
  if (released_bytes) *released_bytes = 0;
  if (act_blocks.empty()) { act_batch = 0; return SRT_OK; }
  PhaseTrace tr("release_activations");
  size_t freed = act_bytes;
  int rc = free_activation_blocks();
  if (rc) return rc;
  tr.mark();
  tr.mark();
  if (pool && (rc = srt_pool_empty_cache(pool, pool_kind, &freed))) return rc;
  tr.print(freed);
  if (released_bytes) *released_bytes = freed;
  return SRT_OK;
}

// Shrinks the activation set to micro-batches of B samples and returns the pages this frees. The smaller
// set is placed before anything is unmapped, so it reuses pages that are already mapped and the only
// driver work is unmapping the difference. B == 0 is release_activations.
int Step::shrink_activations(int B, size_t* released_bytes) {
  if (released_bytes) *released_bytes = 0;
  if (B <= 0) return release_activations(released_bytes);
  SRT_REQUIRE(B <= cfg.max_batch, "shrink_activations: batch %d above max_batch %d", B, cfg.max_batch);
  PhaseTrace tr("shrink_activations");
  const size_t before = act_bytes;
  int rc = free_activation_blocks();
  if (rc) return rc;
  tr.mark();
  if ((rc = alloc_activations(B))) return rc;
  tr.mark();
  size_t freed = before > act_bytes ? before - act_bytes : 0;
  if (pool && (rc = srt_pool_empty_cache(pool, pool_kind, &freed))) return rc;
  tr.print(freed);
  if (released_bytes) *released_bytes = freed;
  return SRT_OK;
}

// Parity sub-filters of a 3x3 stride-2 pad-1 filter from its transposed copy wt[c][rs][k]. Output row h = 2i + a
// receives tap r only when h + 1 - r is even: a = 0 takes r = 1 (input row i); a = 1 takes r = 2 (row i) and r = 0
// (row i + 1). Columns alike. Class (a, b) is stored as [c][tr][ts][k] in the order its stride-1 gather walks the taps.
namespace {
struct ParityTaps { int n; int r[2]; };
inline ParityTaps parity_taps(int a) { return a == 0 ? ParityTaps{1, {1, 0}} : ParityTaps{2, {2, 0}}; }
}  // namespace

int Step::build_subfilters(const ConvL& c, cudaStream_t st) {
  if (!s2_fast(c) || c.R != 3) return SRT_OK;
  size_t off = c.s2_off;
  for (int a = 0; a < 2; ++a)
    for (int b = 0; b < 2; ++b) {
      const ParityTaps ta = parity_taps(a), tb = parity_taps(b);
      int taps[4], n = 0;
      for (int i = 0; i < ta.n; ++i)
        for (int j = 0; j < tb.n; ++j) taps[n++] = ta.r[i] * 3 + tb.r[j];
      int rc = subfilter(cfg.dtype, wt(c), (char*)WT + off * esz, c.C, c.K, 9, taps, n, st);
      if (rc) return rc;
      off += (size_t)c.C * n * c.K;
    }
  return SRT_OK;
}

// Data gradient of a stride-2 convolution without multiplying the zeros a strided scatter is made of: each output
// parity class is a stride-1 gather GEMM over dy with its own taps (1, 2, 2, 4 of the 9; a 1x1 filter only has class
// (0, 0)), written compactly and interleaved (+ addend) by one pass.
int Step::dgrad_s2(const Unit& u, const void* dz, void* dx, const void* addend, int B) {
  const ConvL& c = u.conv;
  const int Hh = u.H / 2, Wh = u.W / 2;
  const size_t quarter = (size_t)B * Hh * Wh * c.C;
  const void* cls[4] = {nullptr, nullptr, nullptr, nullptr};
  size_t off = c.s2_off;
  int rc;
  for (int a = 0; a < 2; ++a)
    for (int b = 0; b < 2; ++b) {
      if (c.R == 1 && (a || b)) continue;
      const int nr = c.R == 1 ? 1 : parity_taps(a).n, ns = c.R == 1 ? 1 : parity_taps(b).n;
      GatherGeom g;
      g.n_img = B; g.src_h = u.P; g.src_w = u.Q; g.src_c = c.K;
      g.out_h = Hh; g.out_w = Wh;
      g.R = nr; g.S = ns; g.stride = 1; g.pad = 0; g.dgrad = 0;
      g.M = B * Hh * Wh; g.Kg = nr * ns * c.K; g.Nout = c.C;
      void* out = (char*)s2_tmp + (size_t)(a * 2 + b) * quarter * esz;
      const void* filt = c.R == 1 ? wt(c) : (const void*)((char*)WT + off * esz);
      if ((rc = conv_gather_gemm_tc(g, dz, filt, out, nullptr, stream))) return rc;
      cls[a * 2 + b] = out;
      off += (size_t)c.C * nr * ns * c.K;
    }
  return parity_interleave(cfg.dtype, cls[0], cls[1], cls[2], cls[3], addend, dx, B, u.H, u.W, c.C, stream);
}

// bf16 working copy of the parameters (bf16 mode) and transposed filters for dgrad.
int Step::refresh_working_copies() {
  int rc;
  if ((rc = join_side())) return rc;
  if (cfg.dtype == SRT_BF16 && (rc = cast_f32_to_bf16(P, Pw, (int64_t)n_flat, stream))) return rc;
  auto tr = [&](const ConvL& c) -> int {
    int r = filter_transpose(cfg.dtype, pw(c.w), wt(c), c.K, c.R * c.S, c.C, stream);
    return r ? r : build_subfilters(c, stream);
  };
  if ((rc = tr(stem.conv))) return rc;
  for (auto& k : blocks) {
    if ((rc = tr(k.u1.conv))) return rc;
    if ((rc = tr(k.u2.conv))) return rc;
    if ((rc = tr(k.u3.conv))) return rc;
    if (k.has_ds && (rc = tr(k.ds.conv))) return rc;
  }
  // fc: [classes][feat] -> [feat][classes], stored after the conv filters
  const size_t fc_wt_off = n_wt - align_up((size_t)cfg.num_classes * feat_C, 64);
  return filter_transpose(cfg.dtype, pw(fc_w), (char*)WT + fc_wt_off * esz, cfg.num_classes, 1, feat_C, stream);
}

int Step::forward(int B) {
  const int dt = cfg.dtype, impl = cfg.impl;
  int rc;
  if (side_dirty && (rc = join_side())) return rc;  // an aborted backward may have left filter-gradient kernels in flight
  auto run_unit = [&](Unit& u, const void* in, const void* residual) -> int {
    if (int c = checkpoint()) return c;
    srt_conv_desc d = {B, u.H, u.W, u.conv.C, u.conv.K, u.conv.R, u.conv.S, u.conv.stride, u.conv.pad, u.P, u.Q};
    int r;
    const int64_t rows = (int64_t)B * u.P * u.Q;
    const double flops = 2.0 * rows * u.conv.K * u.conv.R * u.conv.S * u.conv.C;
    const double abytes = (double)rows * u.bn.C * esz;
    uint8_t* bits = (residual && u.relu && !eval_mode) ? u.bits : nullptr;
    u.bits_valid = false;
    if (!eval_mode && conv_stats && conv_fprop_stats_supported(d, dt, impl)) {
      // the convolution's epilogue leaves the column sums of z; BatchNorm finalizes them and goes straight to apply
      int slabs = 0;
      if ((r = timed(SRT_PROF_CONV, flops, [&] {
            return conv_fprop_stats(d, dt, impl, in, pw(u.conv.w), u.z, nullptr, scratch, scratch_bytes, &slabs, stream); })))
        return r;
      if ((r = timed(SRT_PROF_NORM, 0.0, [&] {
            return bn_finalize(scratch, slabs, u.bn.C, rows, pf(u.bn.gamma), pf(u.bn.beta), cfg.bn_eps, cfg.bn_momentum,
                               bf_(u.bn.rmean), bf_(u.bn.rvar), u.bn.mean, u.bn.invstd, u.bn.scale, u.bn.shift, stream); })))
        return r;
      u.bits_valid = bits != nullptr;
      return timed(SRT_PROF_NORM, abytes * (residual ? 3 : 2) + (bits ? abytes / 16 : 0), [&] {
        return bn_apply(dt, u.z, residual, u.y, rows, u.bn.C, u.bn.scale, u.bn.shift, u.relu, stream, bits); });
    }
    if ((r = timed(SRT_PROF_CONV, flops, [&] { return conv_fprop(d, dt, impl, in, pw(u.conv.w), u.z, nullptr, stream); })))
      return r;
    if (eval_mode) {
      // inference: normalise with the running statistics (scale/shift prepared by bn_eval_params)
      if ((r = bn_eval_params(pf(u.bn.gamma), pf(u.bn.beta), bf_(u.bn.rmean), bf_(u.bn.rvar), cfg.bn_eps, u.bn.C,
                              u.bn.scale, u.bn.shift, stream)))
        return r;
    } else if (fused_bn && bn_fused_pays(dt, rows, u.bn.C, 0)) {
      // statistics, finalize and apply in one cooperative launch
      return timed(SRT_PROF_NORM, abytes * (residual ? 3 : 2), [&] {
        return bn_forward_fused(dt, u.z, residual, u.y, rows, u.bn.C, pf(u.bn.gamma), pf(u.bn.beta), cfg.bn_eps,
                                cfg.bn_momentum, bf_(u.bn.rmean), bf_(u.bn.rvar), u.bn.mean, u.bn.invstd, u.bn.scale,
                                u.bn.shift, u.relu, stream); });
    } else if ((r = timed(SRT_PROF_NORM, abytes, [&] {
          return bn_stats(dt, u.z, rows, u.bn.C, pf(u.bn.gamma), pf(u.bn.beta), cfg.bn_eps, cfg.bn_momentum,
                          bf_(u.bn.rmean), bf_(u.bn.rvar), u.bn.mean, u.bn.invstd, u.bn.scale, u.bn.shift,
                          scratch, scratch_bytes, stream); })))
      return r;
    u.bits_valid = bits != nullptr;
    return timed(SRT_PROF_NORM, abytes * (residual ? 3 : 2) + (bits ? abytes / 16 : 0), [&] {
      return bn_apply(dt, u.z, residual, u.y, rows, u.bn.C, u.bn.scale, u.bn.shift, u.relu, stream, bits); });
  };
  const double img_px = (double)B * cfg.image * cfg.image;
  if ((rc = timed(SRT_PROF_OTHER, img_px * (3 * 4 + kStemCpad * esz), [&] {
        return nchw_to_nhwc(dt, stage_images, x0, B, 3, cfg.image, cfg.image, kStemCpad, stream); })))
    return rc;
  if ((rc = run_unit(stem, x0, nullptr))) return rc;
  const double pool_in = (double)B * stem.P * stem.Q * 64 * esz;
  if ((rc = timed(SRT_PROF_OTHER, pool_in * 1.25 + pool_in / 4 / esz, [&] {
        return maxpool_fwd(dt, stem.y, pool_y, pool_arg, B, stem.P, stem.Q, 64, stream); })))
    return rc;
  const void* x = pool_y;
  for (auto& k : blocks) {
    if ((rc = run_unit(k.u1, x, nullptr))) return rc;
    if ((rc = run_unit(k.u2, k.u1.y, nullptr))) return rc;
    const void* identity = x;
    if (k.has_ds) {
      if ((rc = run_unit(k.ds, x, nullptr))) return rc;
      identity = k.ds.y;
    }
    if ((rc = run_unit(k.u3, k.u2.y, identity))) return rc;
    x = k.u3.y;
  }
  if ((rc = timed(SRT_PROF_OTHER, (double)B * (final_HW + 1) * feat_C * esz, [&] {
        return avgpool_fwd(dt, x, avg, B, final_HW, feat_C, stream); })))
    return rc;
  srt_conv_desc fd = {B, 1, 1, feat_C, cfg.num_classes, 1, 1, 1, 0, 1, 1};
  srt_conv_epilogue ep = {pf(fc_b), nullptr};
  return timed(SRT_PROF_CONV, 2.0 * B * feat_C * cfg.num_classes, [&] {
    return conv_fprop(fd, dt, impl, avg, pw(fc_w), logits, &ep, stream); });
}

int Step::backward(int B) {
  const int dt = cfg.dtype, impl = cfg.impl;
  int rc;
  if ((rc = join_side())) return rc;
  // fc
  srt_conv_desc fd = {B, 1, 1, feat_C, cfg.num_classes, 1, 1, 1, 0, 1, 1};
  const double fc_flops = 2.0 * B * feat_C * cfg.num_classes;
  if ((rc = timed(SRT_PROF_WGRAD, fc_flops, [&] {
        return conv_wgrad(fd, dt, impl, dlogits, avg, gf(fc_w), scratch, scratch_bytes, stream); })))
    return rc;
  if ((rc = timed(SRT_PROF_OTHER, (double)B * cfg.num_classes * esz, [&] {
        return colsum(dt, dlogits, B, cfg.num_classes, gf(fc_b), stream); })))
    return rc;
  const size_t fc_wt_off = n_wt - align_up((size_t)cfg.num_classes * feat_C, 64);
  if ((rc = timed(SRT_PROF_CONV, fc_flops, [&] {
        return conv_dgrad(fd, dt, impl, dlogits, (char*)WT + fc_wt_off * esz, T[1], nullptr, stream); })))
    return rc;
  if ((rc = timed(SRT_PROF_OTHER, (double)B * (final_HW + 1) * feat_C * esz, [&] {
        return avgpool_bwd(dt, T[1], T[0], B, final_HW, feat_C, stream); })))
    return rc;

  // gradient through conv+BN(+ReLU): dy (w.r.t. u.y) -> dz, filter gradient into G
  const bool fork = use_side();
  // res_unit: the unit's output had the residual added before its ReLU, so the mask cannot be recomputed from z:
  // it comes from the bits the forward pass left, or from the stored y. dres (optional) receives the masked gradient.
  auto unit_bwd = [&](Unit& u, const void* dy, const void* in, void* dz, void* dres, bool res_unit) -> int {
    if (int c = checkpoint()) return c;
    const int64_t rows = (int64_t)B * u.P * u.Q;
    int r;
    if ((r = before_write(dz))) return r;
    if (dres && (r = before_write(dres))) return r;
    const uint8_t* bits = res_unit && u.bits_valid ? u.bits : nullptr;
    const void* ymask = res_unit && !bits ? u.y : nullptr;
    // two passes over (dy, z[, y or its bits]) plus the dz (and masked-gradient) writes
    const double abytes = (double)rows * u.bn.C * esz;
    const double bn_bytes = abytes * ((2.0 + (ymask ? 1.0 : bits ? 1.0 / 16 : 0.0)) * 2 + 1 + (dres ? 1 : 0));
    if (fused_bn && bn_fused_pays(dt, rows, u.bn.C, 1)) {
      if ((r = timed(SRT_PROF_NORM, bn_bytes, [&] {
            return bn_backward_fused(dt, dy, ymask, u.z, rows, u.bn.C, pf(u.bn.gamma), u.bn.mean, u.bn.invstd,
                                     u.bn.scale, u.bn.shift, u.relu, dz, dres, gf(u.bn.gamma), gf(u.bn.beta), stream, bits); })))
        return r;
    } else if ((r = timed(SRT_PROF_NORM, bn_bytes, [&] {
          // units without a residual recompute the ReLU mask from z instead of reading y
          return bn_backward(dt, dy, ymask, u.z, rows, u.bn.C, pf(u.bn.gamma), u.bn.mean,
                             u.bn.invstd, u.bn.scale, u.bn.shift, u.relu, dz, dres, gf(u.bn.gamma),
                             gf(u.bn.beta), scratch, scratch_bytes, stream, bits); })))
      return r;
    srt_conv_desc d = {B, u.H, u.W, u.conv.C, u.conv.K, u.conv.R, u.conv.S, u.conv.stride, u.conv.pad, u.P, u.Q};
    const double flops = 2.0 * rows * u.conv.K * u.conv.R * u.conv.S * u.conv.C;
    if (!fork)
      return timed(SRT_PROF_WGRAD, flops, [&] {
        return conv_wgrad(d, dt, impl, dz, in, gf(u.conv.w), scratch_wg, scratch_wg_bytes, stream); });
    SRT_CHECK_CUDA(cudaEventRecord(ev_fork, stream));
    SRT_CHECK_CUDA(cudaStreamWaitEvent(side, ev_fork, 0));
    side_dirty = true;
    {
      PdlOff no_early_launch(true);
      r = conv_wgrad(d, dt, impl, dz, in, gf(u.conv.w), scratch_wg, scratch_wg_bytes, side);
    }
    if (r) return r;
    const int slot = t_slot(dz);
    if (slot >= 0) {
      SRT_CHECK_CUDA(cudaEventRecord(ev_read[slot], side));
      read_pending[slot] = true;
    }
    return SRT_OK;
  };
  auto unit_dgrad = [&](Unit& u, const void* dz, void* dx, const void* addend, const uint8_t* addend_bits = nullptr) -> int {
    srt_conv_desc d = {B, u.H, u.W, u.conv.C, u.conv.K, u.conv.R, u.conv.S, u.conv.stride, u.conv.pad, u.P, u.Q};
    srt_conv_epilogue ep = {nullptr, addend, addend_bits};
    const double flops = 2.0 * B * u.P * u.Q * u.conv.K * u.conv.R * u.conv.S * u.conv.C;
    if (int r = before_write(dx)) return r;
    if (s2_fast(u.conv) && u.H % 2 == 0 && u.W % 2 == 0)
      return timed(SRT_PROF_CONV, flops, [&] { return dgrad_s2(u, dz, dx, addend, B); });
    return timed(SRT_PROF_CONV, flops, [&] {
      return conv_dgrad(d, dt, impl, dz, wt(u.conv), dx, addend ? &ep : nullptr, stream); });
  };

  int flip = 0, next_bucket = 0;
  auto next_dz = [&]() -> void* { flip ^= 1; return flip ? T[1] : T[5]; };
  for (int i = (int)blocks.size() - 1; i >= 0; --i) {
    Block& k = blocks[i];
    const void* x_in = i == 0 ? pool_y : blocks[i - 1].u3.y;
    // T0 = dout. u3: dz3 -> D, masked dout -> T2
    void* D = next_dz();
    // With the mask bits of the block's output at hand (bf16), a block without a downsample branch needs no masked
    // copy of dout: the first convolution's data gradient adds dout under the bits in its epilogue.
    const bool masked_add = !k.has_ds && k.u3.bits_valid && !s2_fast(k.u1.conv);
    if ((rc = unit_bwd(k.u3, T[0], k.u2.y, D, masked_add ? nullptr : T[2], true))) return rc;
    if ((rc = unit_dgrad(k.u3, D, T[3], nullptr))) return rc;        // dy2 -> T3
    D = next_dz();
    if ((rc = unit_bwd(k.u2, T[3], k.u1.y, D, nullptr, false))) return rc;   // dz2 -> D
    if ((rc = unit_dgrad(k.u2, D, T[3], nullptr))) return rc;        // dy1 -> T3
    D = next_dz();
    if ((rc = unit_bwd(k.u1, T[3], x_in, D, nullptr, false))) return rc;     // dz1 -> D
    if (k.has_ds) {
      if ((rc = unit_bwd(k.ds, T[2], x_in, T[3], nullptr, false))) return rc;   // dz_ds -> T3
      if ((rc = unit_dgrad(k.ds, T[3], T[4], nullptr))) return rc;     // dx_ds -> T4
      if ((rc = unit_dgrad(k.u1, D, T[4], T[4]))) return rc;           // dx = dgrad(dz1) + dx_ds
    } else if (masked_add) {
      if ((rc = unit_dgrad(k.u1, D, T[4], T[0], k.u3.bits))) return rc;  // dx = dgrad(dz1) + dout under the ReLU mask
    } else {
      if ((rc = unit_dgrad(k.u1, D, T[4], T[2]))) return rc;           // dx = dgrad(dz1) + masked dout
    }
    void* t = T[0]; T[0] = T[4]; T[4] = t;
    if (next_bucket + 1 < (int)buckets.size() && buckets[next_bucket].first_block == i) {
      if ((rc = bucket_ready(next_bucket, fork))) return rc;
      ++next_bucket;
    }
  }
  // stem
  const double pool_in = (double)B * stem.P * stem.Q * 64 * esz;
  if ((rc = before_write(T[3]))) return rc;
  if ((rc = timed(SRT_PROF_OTHER, pool_in * 1.25 + pool_in / 4 / esz, [&] {
        return maxpool_bwd(dt, T[0], pool_arg, T[3], B, stem.P, stem.Q, 64, stream); })))
    return rc;
  if ((rc = unit_bwd(stem, T[3], x0, next_dz(), nullptr, false))) return rc;
  if ((rc = join_side())) return rc;
  return bucket_ready((int)buckets.size() - 1, false);
}

}  // namespace srt

using namespace srt;

extern "C" {

int srt_resnet_create(const srt_resnet_config* cfg, srt_step** out) {
  return srt_resnet_create_with_pool(cfg, nullptr, out);
}

int srt_resnet_create_with_pool(const srt_resnet_config* cfg, srt_pool* pool, srt_step** out) {
  return srt_resnet_create_on_allocator(cfg, pool, SRT_POOL_TRAIN, out);
}

int srt_resnet_create_on_allocator(const srt_resnet_config* cfg, srt_pool* pool, int pool_kind, srt_step** out) {
  SRT_REQUIRE(cfg && out, "resnet_create: null argument");
  SRT_REQUIRE(pool_kind == SRT_POOL_TRAIN || pool_kind == SRT_POOL_INFER, "resnet_create: unknown allocator %d", pool_kind);
  SRT_REQUIRE(cfg->dtype == SRT_F32 || cfg->dtype == SRT_BF16, "resnet_create: unknown dtype");
  Step* s = new Step();
  s->cfg = *cfg;
  s->pool = pool;
  s->pool_kind = pool_kind;
  int rc = s->build();
  if (rc == SRT_OK) rc = cudaStreamSynchronize(s->stream) == cudaSuccess ? SRT_OK : SRT_ERR_CUDA;
  if (rc != SRT_OK) { delete s; return rc; }
  *out = (srt_step*)s;
  return SRT_OK;
}

int srt_step_destroy(srt_step* h) {
  if (!h) return SRT_OK;
  Step* s = (Step*)h;
  cudaStreamSynchronize(s->stream);
  if (s->side) cudaStreamSynchronize(s->side);
  delete s;
  return SRT_OK;
}

int srt_step_num_params(srt_step* h) { return h ? (int)((Step*)h)->params.size() : -1; }

int srt_step_param_info(srt_step* h, int idx, char* name, int name_cap, int64_t shape[4], int* ndim,
                        int* kind) {
  Step* s = (Step*)h;
  SRT_REQUIRE(s && idx >= 0 && idx < (int)s->params.size(), "param_info: bad index");
  const ParamRec& r = s->params[idx];
  if (name && name_cap > 0) { strncpy(name, r.name.c_str(), name_cap - 1); name[name_cap - 1] = 0; }
  if (shape) for (int i = 0; i < 4; ++i) shape[i] = r.shape[i];
  if (ndim) *ndim = r.ndim;
  if (kind) *kind = r.kind;
  return SRT_OK;
}

// Host fp32 tensor in torch layout ([K,C,R,S] for conv) -> internal layout ([K,R,S,Cpad]).
int srt_step_set_param(srt_step* h, int idx, const float* host) {
  Step* s = (Step*)h;
  SRT_REQUIRE(s && host && idx >= 0 && idx < (int)s->params.size(), "set_param: bad argument");
  const ParamRec& r = s->params[idx];
  float* dst = r.kind == SRT_PARAM_BUFFER ? s->BUF + r.off : s->P + r.off;
  if (r.kind == SRT_PARAM_CONV) {
    const int K = (int)r.shape[0], C = (int)r.shape[1], R = (int)r.shape[2], S = (int)r.shape[3];
    std::vector<float> tmp((size_t)K * R * S * r.cpad, 0.f);
    for (int k = 0; k < K; ++k)
      for (int c = 0; c < C; ++c)
        for (int a = 0; a < R; ++a)
          for (int b = 0; b < S; ++b)
            tmp[(((size_t)k * R + a) * S + b) * r.cpad + c] = host[(((size_t)k * C + c) * R + a) * S + b];
    SRT_CHECK_CUDA(cudaMemcpy(dst, tmp.data(), tmp.size() * 4, cudaMemcpyHostToDevice));
  } else {
    SRT_CHECK_CUDA(cudaMemcpy(dst, host, r.count * 4, cudaMemcpyHostToDevice));
  }
  return SRT_OK;
}

int srt_step_set_state(srt_step* h, int idx, const float* host, int which) {
  Step* s = (Step*)h;
  SRT_REQUIRE(s && host && idx >= 0 && idx < (int)s->params.size(), "set_state: bad argument");
  SRT_REQUIRE(which == SRT_GET_VALUE || which == SRT_GET_MOMENTUM || which == SRT_GET_ACCUM,
              "set_state: only the value, the momentum and the accumulated gradient can be set");
  const ParamRec& r = s->params[idx];
  if (which == SRT_GET_VALUE || r.kind == SRT_PARAM_BUFFER) return srt_step_set_param(h, idx, host);
  float* dst = (which == SRT_GET_MOMENTUM ? s->M : s->ACC) + r.off;
  SRT_CHECK_CUDA(cudaStreamSynchronize(s->stream));
  if (r.kind == SRT_PARAM_CONV) {
    const int K = (int)r.shape[0], C = (int)r.shape[1], R = (int)r.shape[2], S = (int)r.shape[3];
    std::vector<float> tmp((size_t)K * R * S * r.cpad, 0.f);
    for (int k = 0; k < K; ++k)
      for (int c = 0; c < C; ++c)
        for (int a = 0; a < R; ++a)
          for (int b = 0; b < S; ++b)
            tmp[(((size_t)k * R + a) * S + b) * r.cpad + c] = host[(((size_t)k * C + c) * R + a) * S + b];
    SRT_CHECK_CUDA(cudaMemcpy(dst, tmp.data(), tmp.size() * 4, cudaMemcpyHostToDevice));
  } else {
    SRT_CHECK_CUDA(cudaMemcpy(dst, host, r.count * 4, cudaMemcpyHostToDevice));
  }
  // a loaded momentum continues a run: the next update is m = mu*m + g, not the first step's m = g
  if (which == SRT_GET_MOMENTUM && s->opt_steps == 0) s->opt_steps = 1;
  return SRT_OK;
}

int srt_step_get_param(srt_step* h, int idx, float* host, int which) {
  Step* s = (Step*)h;
  SRT_REQUIRE(s && host && idx >= 0 && idx < (int)s->params.size(), "get_param: bad argument");
  const ParamRec& r = s->params[idx];
  SRT_CHECK_CUDA(cudaStreamSynchronize(s->stream));
  const float* base = r.kind == SRT_PARAM_BUFFER ? s->BUF
                      : which == SRT_GET_GRAD     ? s->G
                      : which == SRT_GET_ACCUM    ? s->ACC
                      : which == SRT_GET_MOMENTUM ? s->M
                                                  : s->P;
  const float* src = base + r.off;
  if (r.kind == SRT_PARAM_CONV) {
    const int K = (int)r.shape[0], C = (int)r.shape[1], R = (int)r.shape[2], S = (int)r.shape[3];
    std::vector<float> tmp((size_t)K * R * S * r.cpad);
    SRT_CHECK_CUDA(cudaMemcpy(tmp.data(), src, tmp.size() * 4, cudaMemcpyDeviceToHost));
    for (int k = 0; k < K; ++k)
      for (int c = 0; c < C; ++c)
        for (int a = 0; a < R; ++a)
          for (int b = 0; b < S; ++b)
            host[(((size_t)k * C + c) * R + a) * S + b] = tmp[(((size_t)k * R + a) * S + b) * r.cpad + c];
  } else {
    SRT_CHECK_CUDA(cudaMemcpy(host, src, r.count * 4, cudaMemcpyDeviceToHost));
  }
  return SRT_OK;
}

int srt_step_commit_params(srt_step* h) {
  Step* s = (Step*)h;
  SRT_REQUIRE(s, "commit_params: null handle");
  int rc = s->refresh_working_copies();
  if (rc) return rc;
  SRT_CHECK_CUDA(cudaStreamSynchronize(s->stream));
  return SRT_OK;
}

void* srt_step_stream(srt_step* h) { return h ? (void*)((Step*)h)->stream : nullptr; }

int srt_step_upload_batch(srt_step* h, const float* host_images, const int64_t* host_labels, int B) {
  Step* s = (Step*)h;
  SRT_REQUIRE(s && host_images && host_labels && B > 0 && B <= s->cfg.max_batch, "upload_batch: bad argument");
  for (int i = 0; i < B; ++i)
    SRT_REQUIRE(host_labels[i] >= 0 && host_labels[i] < (int64_t)s->cfg.num_classes,
                "upload_batch: label %lld of sample %d is outside [0, %d)", (long long)host_labels[i], i, s->cfg.num_classes);
  const size_t img = (size_t)B * 3 * s->cfg.image * s->cfg.image * 4;
  const int idx = s->up_next;
  s->up_next ^= 1;
  if (s->used_pending[idx]) {  // the executor may still be reading this buffer
    SRT_CHECK_CUDA(cudaStreamWaitEvent(s->copy_stream, s->ev_used[idx], 0));
    s->used_pending[idx] = false;
  }
  SRT_CHECK_CUDA(cudaMemcpyAsync(s->stage_images_b[idx], host_images, img, cudaMemcpyHostToDevice, s->copy_stream));
  SRT_CHECK_CUDA(cudaMemcpyAsync(s->stage_labels_b[idx], host_labels, (size_t)B * 8, cudaMemcpyHostToDevice, s->copy_stream));
  SRT_CHECK_CUDA(cudaEventRecord(s->ev_up[idx], s->copy_stream));
  s->pending_up = idx;
  return SRT_OK;
}

int srt_step_set_batch_device(srt_step* h, const float* dev_images, const int64_t* dev_labels, int B) {
  Step* s = (Step*)h;
  SRT_REQUIRE(s && dev_images && dev_labels && B > 0 && B <= s->cfg.max_batch, "set_batch_device: bad argument");
  const size_t img = (size_t)B * 3 * s->cfg.image * s->cfg.image * 4;
  s->pending_up = -1;  // a device batch replaces whatever host batch was on its way
  SRT_CHECK_CUDA(cudaMemcpyAsync(s->stage_images, dev_images, img, cudaMemcpyDeviceToDevice, s->stream));
  SRT_CHECK_CUDA(cudaMemcpyAsync(s->stage_labels, dev_labels, (size_t)B * 8, cudaMemcpyDeviceToDevice, s->stream));
  return SRT_OK;
}

int srt_step_forward_backward(srt_step* h, int B, int global_batch) {
  Step* s = (Step*)h;
  SRT_REQUIRE(s && B > 0 && B <= s->cfg.max_batch && global_batch >= B, "forward_backward: bad batch sizes");
  Step::SmScope sm_scope(s);
  int rc;
  if ((rc = s->adopt_upload())) return rc;
  if (s->act_batch < B && (rc = s->alloc_activations(B))) return rc;  // regain after a release
  rc = s->forward(B);
  if (rc) return rc;
  const float scale = 1.f / (float)global_batch;
  if ((rc = softmax_ce(s->cfg.dtype, s->logits, s->stage_labels, B, s->cfg.num_classes, scale, s->row_loss,
                       s->dlogits, s->stream)))
    return rc;
  if ((rc = sum_f32(s->row_loss, B, s->loss_acc, 0, s->stream))) return rc;
  if ((rc = s->staging_consumed())) return rc;
  return s->backward(B);
}

int srt_step_forward_only(srt_step* h, int B) {
  Step* s = (Step*)h;
  SRT_REQUIRE(s && B > 0 && B <= s->cfg.max_batch, "forward_only: bad batch size");
  Step::SmScope sm_scope(s);
  int rc;
  if ((rc = s->adopt_upload())) return rc;
  if (s->act_batch < B && (rc = s->alloc_activations(B))) return rc;
  if ((rc = s->forward(B))) return rc;
  return s->staging_consumed();
}

int srt_step_forward_infer(srt_step* h, int B) {
  Step* s = (Step*)h;
  SRT_REQUIRE(s && B > 0 && B <= s->cfg.max_batch, "forward_infer: bad batch size");
  Step::SmScope sm_scope(s);
  int rc;
  if ((rc = s->adopt_upload())) return rc;
  if (s->act_batch < B && (rc = s->alloc_activations(B))) return rc;
  s->eval_mode = true;
  rc = s->forward(B);
  s->eval_mode = false;
  if (rc) return rc;
  return s->staging_consumed();
}

int srt_step_accumulate(srt_step* h) {
  Step* s = (Step*)h;
  SRT_REQUIRE(s, "accumulate: null handle");
  Step::SmScope sm_scope(s);
  s->accum_pending++;
  return grad_accumulate(s->ACC, s->G, (int64_t)s->n_flat, s->stream);
}

int srt_step_optimizer(srt_step* h) {
  Step* s = (Step*)h;
  SRT_REQUIRE(s, "optimizer: null handle");
  Step::SmScope sm_scope(s);
  if (int jr = s->join_side()) return jr;  // the parameters' working copy must not change under a reader
  const float* grad = s->accum_pending > 0 ? s->ACC : s->G;
  const bool bf = s->cfg.dtype == SRT_BF16;
  int rc = s->timed(SRT_PROF_OPTIM, (double)s->n_flat * (bf ? 22 : 20), [&] {
    return sgd_momentum(s->P, grad, s->M, bf ? s->Pw : nullptr, (int64_t)s->n_flat, s->cfg.lr, s->cfg.momentum,
                        s->cfg.weight_decay, s->opt_steps == 0, s->stream); });
  if (rc) return rc;
  if (s->accum_pending > 0) {
    SRT_CHECK_CUDA(cudaMemsetAsync(s->ACC, 0, s->n_flat * 4, s->stream));
    s->accum_pending = 0;
  }
  s->opt_steps++;
  // transposed filters follow the updated parameters (the bf16 copy was written by the optimizer). Only
  // the backward pass reads them, so they run on the side stream beside the next forward pass.
  cudaStream_t ts = s->stream;
  if (s->use_side()) {
    SRT_CHECK_CUDA(cudaEventRecord(s->ev_fork, s->stream));
    SRT_CHECK_CUDA(cudaStreamWaitEvent(s->side, s->ev_fork, 0));
    s->wt_dirty = true;
    ts = s->side;
  }
  PdlOff no_early_launch(ts != s->stream);
  auto tr = [&](const ConvL& c) -> int {
    int r;
    if (ts != s->stream) r = filter_transpose(s->cfg.dtype, s->pw(c.w), s->wt(c), c.K, c.R * c.S, c.C, ts);
    else r = s->timed(SRT_PROF_OPTIM, 2.0 * c.K * c.R * c.S * c.C * s->esz, [&] {
      return filter_transpose(s->cfg.dtype, s->pw(c.w), s->wt(c), c.K, c.R * c.S, c.C, s->stream); });
    return r ? r : s->build_subfilters(c, ts);
  };
  if ((rc = tr(s->stem.conv))) return rc;
  for (auto& k : s->blocks) {
    if ((rc = tr(k.u1.conv))) return rc;
    if ((rc = tr(k.u2.conv))) return rc;
    if ((rc = tr(k.u3.conv))) return rc;
    if (k.has_ds && (rc = tr(k.ds.conv))) return rc;
  }
  const size_t fc_wt_off = s->n_wt - align_up((size_t)s->cfg.num_classes * s->feat_C, 64);
  return filter_transpose(s->cfg.dtype, s->pw(s->fc_w), (char*)s->WT + fc_wt_off * s->esz, s->cfg.num_classes, 1,
                          s->feat_C, ts);
}

int srt_step_loss(srt_step* h, float* host_loss) {
  Step* s = (Step*)h;
  SRT_REQUIRE(s && host_loss, "loss: null argument");
  SRT_CHECK_CUDA(cudaMemcpyAsync(host_loss, s->loss_acc, 4, cudaMemcpyDeviceToHost, s->stream));
  SRT_CHECK_CUDA(cudaStreamSynchronize(s->stream));
  return SRT_OK;
}

int srt_step_follow_sm_mask(srt_step* h, int on) {
  Step* s = (Step*)h;
  SRT_REQUIRE(s, "follow_sm_mask: null handle");
  if (on) {
    cudaStream_t st;
    int sms;
    int rc = partition_stream(s->cfg_device, 1 << 30, &st, &sms);  // builds the ladder; fails where green contexts are missing
    if (rc) return rc;
    s->follow_mask = true;
    return SRT_OK;
  }
  s->follow_mask = false;
  if (s->stream != s->home_stream) {
    if (!s->switch_ev) SRT_CHECK_CUDA(cudaEventCreateWithFlags(&s->switch_ev, cudaEventDisableTiming));
    SRT_CHECK_CUDA(cudaEventRecord(s->switch_ev, s->stream));
    SRT_CHECK_CUDA(cudaStreamWaitEvent(s->home_stream, s->switch_ev, 0));
    if (s->side && s->home_side && s->side != s->home_side) {
      SRT_CHECK_CUDA(cudaEventRecord(s->switch_ev, s->side));
      SRT_CHECK_CUDA(cudaStreamWaitEvent(s->home_side, s->switch_ev, 0));
      s->side = s->home_side;
    }
    s->stream = s->home_stream;
    s->cur_sms = 0;
  }
  return SRT_OK;
}

int srt_step_follow_infer_tpc(srt_step* h, srt_comm* comm, int device, int min_train_tpc, int max_train_tpc) {
  Step* s = (Step*)h;
  SRT_REQUIRE(s, "follow_infer_tpc: null handle");
  if (!comm) { s->tpc_comm = nullptr; return srt_step_follow_sm_mask(h, 0); }
  s->tpc_comm = comm;
  s->tpc_device = device;
  s->tpc_min_train = min_train_tpc > 0 ? min_train_tpc : 1;
  s->tpc_max_train = max_train_tpc > 0 ? max_train_tpc : 1 << 20;
  return srt_step_follow_sm_mask(h, 1);
}

int srt_step_num_grad_buckets(srt_step* h) { return h ? (int)((Step*)h)->buckets.size() : -1; }

int srt_step_grad_bucket(srt_step* h, int i, int64_t* offset, int64_t* count) {
  Step* s = (Step*)h;
  SRT_REQUIRE(s && offset && count && i >= 0 && i < (int)s->buckets.size(), "grad_bucket: bad argument");
  *offset = (int64_t)s->buckets[i].off;
  *count = (int64_t)s->buckets[i].count;
  return SRT_OK;
}

int srt_step_wait_grad_bucket(srt_step* h, int i, void* stream) {
  Step* s = (Step*)h;
  SRT_REQUIRE(s && i >= 0 && i < (int)s->buckets.size(), "wait_grad_bucket: bad argument");
  SRT_CHECK_CUDA(cudaStreamWaitEvent((cudaStream_t)stream, s->buckets[i].ev, 0));
  return SRT_OK;
}

// accumulated = 0: the gradients of the backward pass just enqueued, bucket by bucket behind their ready events;
// accumulated = 1: the accumulated-gradient buffer (srt_step_accumulate) as one range behind the executor's stream,
// which is what ranks exchange when they ran different numbers of micro-batches.
int srt_step_allreduce_begin(srt_step* h, srt_ddp* c, int accumulated, int wire_dtype) {
  Step* s = (Step*)h;
  SRT_REQUIRE(s && c, "step_allreduce_begin: null argument");
  if (accumulated) {
    SRT_CHECK_CUDA(cudaEventRecord(s->ev_fork, s->stream));
    const int64_t off = 0, cnt = (int64_t)s->n_flat;
    const cudaEvent_t ev = s->ev_fork;
    return grad_exchange_begin((Comm*)c, s->ACC, 1, &off, &cnt, &ev, wire_dtype);
  }
  std::vector<int64_t> off, cnt;
  std::vector<cudaEvent_t> ev;
  for (auto& b : s->buckets) {
    off.push_back((int64_t)b.off);
    cnt.push_back((int64_t)b.count);
    ev.push_back(b.ev);
  }
  return grad_exchange_begin((Comm*)c, s->G, (int)off.size(), off.data(), cnt.data(), ev.data(), wire_dtype);
}

int srt_step_allreduce_wait(srt_step* h, srt_ddp* c) {
  Step* s = (Step*)h;
  SRT_REQUIRE(s && c, "step_allreduce_wait: null argument");
  return grad_exchange_wait((Comm*)c, s->stream);
}

int srt_step_wait_event(srt_step* h, void* event) {
  Step* s = (Step*)h;
  SRT_REQUIRE(s && event, "wait_event: null argument");
  SRT_CHECK_CUDA(cudaStreamWaitEvent(s->stream, (cudaEvent_t)event, 0));
  return SRT_OK;
}

int srt_step_overlap_wgrad(srt_step* h, int on) {
  Step* s = (Step*)h;
  SRT_REQUIRE(s, "overlap_wgrad: null handle");
  int rc = s->join_side();
  if (rc) return rc;
  s->overlap_wgrad = on != 0;
  return SRT_OK;
}

int srt_step_current_sms(srt_step* h, int* sms) {
  Step* s = (Step*)h;
  SRT_REQUIRE(s && sms, "current_sms: null argument");
  *sms = s->cur_sms > 0 ? s->cur_sms : Step::sm_count_device();
  return SRT_OK;
}

int srt_step_synchronize(srt_step* h) {
  Step* s = (Step*)h;
  SRT_REQUIRE(s, "synchronize: null handle");
  SRT_CHECK_CUDA(cudaStreamSynchronize(s->stream));
  if (s->side) SRT_CHECK_CUDA(cudaStreamSynchronize(s->side));
  return SRT_OK;
}

int srt_step_logits(srt_step* h, float* host, int B) {
  Step* s = (Step*)h;
  SRT_REQUIRE(s && host && B > 0 && B <= s->cfg.max_batch, "logits: bad argument");
  const size_t n = (size_t)B * s->cfg.num_classes;
  SRT_CHECK_CUDA(cudaStreamSynchronize(s->stream));
  if (s->cfg.dtype == SRT_F32) {
    SRT_CHECK_CUDA(cudaMemcpy(host, s->logits, n * 4, cudaMemcpyDeviceToHost));
  } else {
    std::vector<uint16_t> tmp(n);
    SRT_CHECK_CUDA(cudaMemcpy(tmp.data(), s->logits, n * 2, cudaMemcpyDeviceToHost));
    for (size_t i = 0; i < n; ++i) {
      uint32_t u = (uint32_t)tmp[i] << 16;
      memcpy(&host[i], &u, 4);
    }
  }
  return SRT_OK;
}

int srt_step_shrink_activations(srt_step* h, int B, size_t* released_bytes) {
  Step* s = (Step*)h;
  SRT_REQUIRE(s, "shrink_activations: null handle");
  return s->shrink_activations(B, released_bytes);
}

int srt_step_release_activations(srt_step* h, size_t* released_bytes) {
  Step* s = (Step*)h;
  SRT_REQUIRE(s, "release_activations: null handle");
  return s->release_activations(released_bytes);
}

int srt_step_reserve_activations(srt_step* h, int B) {
  Step* s = (Step*)h;
  SRT_REQUIRE(s, "reserve_activations: null handle");
  return s->alloc_activations(B);
}

int srt_step_request_abort(srt_step* h, int on) {
  Step* s = (Step*)h;
  SRT_REQUIRE(s, "request_abort: null handle");
  s->abort_flag.store(on ? 1 : 0, std::memory_order_release);
  return SRT_OK;
}

int srt_step_profile(srt_step* h, int enable) {
  Step* s = (Step*)h;
  SRT_REQUIRE(s, "profile: null handle");
  if (s->prof_on) s->prof_collect();
  s->prof_on = enable != 0;
  if (enable) {
    for (int i = 0; i < SRT_PROF_NCAT; ++i) { s->prof_ms[i] = 0; s->prof_work[i] = 0; s->prof_launches[i] = 0; }
  }
  return SRT_OK;
}

int srt_step_profile_read(srt_step* h, double ms[SRT_PROF_NCAT], double work[SRT_PROF_NCAT],
                          int64_t launches[SRT_PROF_NCAT]) {
  Step* s = (Step*)h;
  SRT_REQUIRE(s && ms && work && launches, "profile_read: null argument");
  s->prof_collect();
  for (int i = 0; i < SRT_PROF_NCAT; ++i) {
    ms[i] = s->prof_ms[i]; work[i] = s->prof_work[i]; launches[i] = s->prof_launches[i];
  }
  return SRT_OK;
}

int srt_step_grad_buffer(srt_step* h, int accumulated, void** ptr, int64_t* n) {
  Step* s = (Step*)h;
  SRT_REQUIRE(s && ptr && n, "grad_buffer: null argument");
  *ptr = accumulated ? (void*)s->ACC : (void*)s->G;
  *n = (int64_t)s->n_flat;
  return SRT_OK;
}

int64_t srt_step_memory_bytes(srt_step* h, int which) {
  Step* s = (Step*)h;
  if (!s) return -1;
  if (which == 0) return (int64_t)(s->n_flat * 16 + s->n_buf * 4);  // parameters + optimizer state
  return (int64_t)s->act_bytes;                                     // activations + gradient buffers
}

}  // extern "C"
