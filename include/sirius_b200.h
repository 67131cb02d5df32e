/*
 * sirius_b200 — C ABI of the B200-native colocated training step.
 *
 * Every entry point takes plain pointers and sizes, returns an int status (SRT_OK == 0) and never
 * throws. Device pointers are raw CUDA addresses; `stream` is a cudaStream_t passed as void*.
 * On failure srt_last_error() returns a thread-local description.
 *
 * Citations are paths inside the Sirius reference tree (file:line). The reference has no
 * arithmetic of its own: its training scripts call torchvision / HuggingFace modules
 * (train/resnet152.py:84-91, train/swin_b.py:83-95), so the compute entry points below replace
 * the PyTorch operator each one names; the runtime entry points replace the reference's C++.
 *
 * Tensor layouts: activations NHWC, filters KRSC, both densely packed. dtype SRT_F32 uses fp32
 * operands and fp32 accumulation on the CUDA cores; SRT_BF16 uses bf16 operands with fp32
 * accumulation on the tcgen05 tensor cores (accumulators in tensor memory).
 */
#ifndef SIRIUS_B200_H_
#define SIRIUS_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { SRT_OK = 0, SRT_ERR_INVALID = 1, SRT_ERR_CUDA = 2, SRT_ERR_UNSUPPORTED = 3,
       SRT_ERR_NOMEM = 4, SRT_ERR_TIMEOUT = 5, SRT_ERR_STATE = 6, SRT_ERR_ABORTED = 7 };
enum { SRT_F32 = 0, SRT_BF16 = 1 };
/* Which kernel family a convolution call uses. AUTO: tcgen05 for bf16, CUDA cores for fp32. */
enum { SRT_IMPL_AUTO = 0, SRT_IMPL_SIMT = 1, SRT_IMPL_TCGEN05 = 2 };

const char* srt_last_error(void);
const char* srt_version(void);

/* ---- convolution as implicit GEMM (replaces nn.Conv2d / nn.Linear inside model(images),
 *      train/resnet152.py:86; backward from scaler.scale(loss).backward(), :89) ------------- */
typedef struct srt_conv_desc {
  int N, H, W, C;   /* input  NHWC (C % 8 == 0) */
  int K, R, S;      /* filter KRSC              */
  int stride, pad;
  int P, Q;         /* output NPQK              */
} srt_conv_desc;

/* Fused epilogue of fprop/dgrad: y = acc (+ bias[k]) (+ addend[m][k]).  Null pointers disable a
 * term. addend may alias y. addend_bits (optional, with addend): one bit per element of addend, bit e of
 * byte i for element 8i + e in row-major order; an element whose bit is 0 is not added. This is how the
 * data gradient of the first convolution of a residual block receives the block's output gradient under
 * the ReLU mask of the block's output (srt_bn_apply_bits) without a masked copy of it in memory. */
typedef struct srt_conv_epilogue {
  const float* bias;     /* [K] fp32, or NULL            */
  const void*  addend;   /* same shape/dtype as y, or NULL */
  const unsigned char* addend_bits;  /* [M*K/8] or NULL */
} srt_conv_epilogue;

/* y[N,P,Q,K] = conv(x[N,H,W,C], w[K,R,S,C]). */
int srt_conv_fprop(const srt_conv_desc* d, int dtype, int impl, const void* x, const void* w,
                   void* y, const srt_conv_epilogue* ep, void* stream);
/* dx[N,H,W,C] = conv^T(dy[N,P,Q,K], wt[C,R,S,K]); wt comes from srt_conv_filter_transpose. */
int srt_conv_dgrad(const srt_conv_desc* d, int dtype, int impl, const void* dy, const void* wt,
                   void* dx, const srt_conv_epilogue* ep, void* stream);
/* dw[K,R,S,C] (fp32, overwritten) = sum over N,P,Q of dy x x. `scratch` holds split partial
 * sums; query its size with srt_conv_wgrad_scratch_bytes. */
int srt_conv_wgrad(const srt_conv_desc* d, int dtype, int impl, const void* dy, const void* x,
                   float* dw, void* scratch, size_t scratch_bytes, void* stream);
size_t srt_conv_wgrad_scratch_bytes(const srt_conv_desc* d, int dtype, int impl);
/* wt[C,R,S,K] = transpose of w[K,R,S,C] (same dtype). */
int srt_conv_filter_transpose(const srt_conv_desc* d, int dtype, const void* w, void* wt,
                              void* stream);

/* ---- BatchNorm2d in training mode over NHWC rows (replaces nn.BatchNorm2d + ReLU + residual
 *      add of torchvision Bottleneck, reached from train/resnet152.py:86,89) ---------------- */
/* Per-channel batch statistics of z[rows][C]; updates running stats in place
 * (momentum 0.1, unbiased running variance) and writes scale/shift so that
 * bn(z) = z*scale + shift, plus mean and invstd for the backward pass.
 * scratch: srt_bn_scratch_bytes(rows, C) bytes. */
int srt_bn_stats(int dtype, const void* z, int64_t rows, int C, const float* gamma,
                 const float* beta, float eps, float momentum, float* running_mean,
                 float* running_var, float* mean, float* invstd, float* scale, float* shift,
                 void* scratch, size_t scratch_bytes, void* stream);
size_t srt_bn_scratch_bytes(int64_t rows, int C);
/* srt_bn_stats without any allocation by anyone. This entry point has no counterpart in the
 * reference. It exists for callers that cannot obtain scratch memory: a colocated trainer that is
 * handing its memory pool over to the inference server has promised all free device memory to the
 * other process, so a cudaMalloc at that moment fails or takes what the server was told it may use;
 * and a control thread that must stay responsive cannot call cudaMalloc/cudaFree, which may
 * synchronise the device. The slab partial sums go into a fixed 4 MiB array inside the library
 * (every GPU that loads the library holds it until the process exits). The caller still passes
 * the input and all outputs. Limits and rules:
 *  - problems with srt_bn_scratch_bytes(rows, C) > SRT_BN_STATIC_SCRATCH_BYTES are rejected with
 *    SRT_ERR_INVALID and a message; use srt_bn_stats for those;
 *  - the array's device address is looked up once per device, with that device current: by
 *    srt_bn_static_prepare(), or else by the first srt_bn_stats_static call on the device. That first look-up
 *    is also when the CUDA runtime may load the module that holds the array (lazy module loading), so it can
 *    touch the driver's allocator: call srt_bn_static_prepare() at start-up, on every device to be used and
 *    before any stream capture is begun, and the later calls touch no allocator at all. Call it again after a
 *    cudaDeviceReset (an address looked up before the reset is stale);
 *  - all calls share the one array, which keeps whatever the previous call left in it (nothing in
 *    it needs clearing: each call writes every partial before reading it), so two calls whose
 *    kernels can overlap on the GPU (different streams, no ordering) race and must be serialised;
 *  - it calls neither cudaMalloc nor cudaFree nor any allocating library routine. */
#define SRT_BN_STATIC_SCRATCH_BYTES (4u << 20)
int srt_bn_static_prepare(void);
int srt_bn_stats_static(int dtype, const void* z, int64_t rows, int C, const float* gamma,
                        const float* beta, float eps, float momentum, float* running_mean,
                        float* running_var, float* mean, float* invstd, float* scale, float* shift,
                        void* stream);
/* Convolution followed by BatchNorm without the statistics pass over y (every conv + bn pair of
 * torchvision's Bottleneck, train/resnet152.py:86): the bf16 tensor-core fprop writes, besides
 * y, the sum and the sum of squares of the stored y values per 128-row tile and output channel
 * (`partial`, double2 [*slabs][K], srt_conv_fprop_bn_stats_bytes(d) bytes, 16-byte aligned), and
 * srt_bn_finalize turns partial sums of that layout into what srt_bn_stats returns. Only the
 * bf16 tensor-core path has this epilogue: srt_conv_fprop_bn_stats_supported says whether a
 * (dtype, impl) pair may use it; otherwise call srt_conv_fprop and srt_bn_stats. */
int srt_conv_fprop_bn_stats(const srt_conv_desc* d, int dtype, int impl, const void* x, const void* w,
                            void* y, const srt_conv_epilogue* ep, void* partial, size_t partial_bytes,
                            int* slabs, void* stream);
size_t srt_conv_fprop_bn_stats_bytes(const srt_conv_desc* d);
int srt_conv_fprop_bn_stats_supported(const srt_conv_desc* d, int dtype, int impl);
int srt_bn_finalize(const void* partial, int slabs, int C, int64_t rows, const float* gamma, const float* beta,
                    float eps, float momentum, float* running_mean, float* running_var, float* mean,
                    float* invstd, float* scale, float* shift, void* stream);
/* y = act(z*scale + shift (+ residual)); relu != 0 applies max(.,0). */
int srt_bn_apply(int dtype, const void* z, const void* residual, void* y, int64_t rows, int C,
                 const float* scale, const float* shift, int relu, void* stream);
/* Backward of y = act(bn(z) (+ residual)). dy is the gradient w.r.t. y. When relu != 0 the mask
 * comes from y; for units without a residual y may be NULL and the mask is recomputed from
 * z*scale + shift (saves one tensor read). Writes dz, dgamma, dbeta and, when dresidual != NULL,
 * the masked gradient that flows to the residual branch. */
int srt_bn_backward(int dtype, const void* dy, const void* y, const void* z, int64_t rows, int C,
                    const float* gamma, const float* mean, const float* invstd, const float* scale,
                    const float* shift, int relu, void* dz, void* dresidual, float* dgamma,
                    float* dbeta, void* scratch, size_t scratch_bytes, void* stream);
/* The ReLU mask of a bf16 unit as one bit per element instead of the stored output: srt_bn_apply_bits is
 * srt_bn_apply with relu = 1 that also writes relu_bits[rows*C/8] (bit e of byte i: element 8i + e of y is
 * positive); srt_bn_backward_bits is srt_bn_backward (one_launch = 0, needs scratch) or srt_bn_backward_fused
 * (one_launch = 1) reading those bits where the other two read y: a sixteenth of the bytes in both of their
 * passes. Together with srt_conv_epilogue.addend_bits a residual block's backward needs neither the stored
 * output nor a masked copy of its gradient. No counterpart in the reference (autograd keeps the output). */
int srt_bn_apply_bits(int dtype, const void* z, const void* residual, void* y, int64_t rows, int C,
                      const float* scale, const float* shift, unsigned char* relu_bits, void* stream);
int srt_bn_backward_bits(int dtype, const void* dy, const unsigned char* relu_bits, const void* z, int64_t rows, int C,
                         const float* gamma, const float* mean, const float* invstd, void* dz, void* dresidual,
                         float* dgamma, float* dbeta, void* scratch, size_t scratch_bytes, int one_launch, void* stream);
/* The same BatchNorm as ONE launch per direction: a cooperative grid of at most one block per SM sums its work
 * items, meets at a grid-wide barrier, finalizes the channels (dealt to the warps of the grid), meets again and
 * applies the coefficients to the same items. Pays where the three launches of the path above cost more than the
 * passes themselves (tensors that sit in L2). The split into work items depends on the shape only, so the result
 * has the same bits on any number of SMs. Partial sums and barrier words live in a 2.4 MB workspace that the
 * library keeps per (device, stream) and allocates on the first call on that stream; every barrier wait is
 * bounded and reports through srt_tc_status (code 0xB1). srt_bn_fused_fits tells whether a shape qualifies
 * (C a multiple of 16 bytes of elements, at most 75 776 channels). When dresidual is given, the masked
 * gradient is written there first and read back for dz (dresidual may alias dy). No counterpart in the
 * reference. */
int srt_bn_fused_fits(int dtype, int64_t rows, int C, int backward);
int srt_bn_forward_fused(int dtype, const void* z, const void* residual, void* y, int64_t rows, int C, const float* gamma,
                         const float* beta, float eps, float momentum, float* running_mean, float* running_var, float* mean,
                         float* invstd, float* scale, float* shift, int relu, void* stream);
int srt_bn_backward_fused(int dtype, const void* dy, const void* y, const void* z, int64_t rows, int C, const float* gamma,
                          const float* mean, const float* invstd, const float* scale, const float* shift, int relu, void* dz,
                          void* dresidual, float* dgamma, float* dbeta, void* stream);

/* ---- pooling (replaces nn.MaxPool2d(3,2,1) and nn.AdaptiveAvgPool2d(1) of torchvision
 *      ResNet) ------------------------------------------------------------------------------- */
int srt_maxpool3x3s2_fwd(int dtype, const void* x, void* y, uint8_t* argmax, int N, int H, int W,
                         int C, void* stream);
int srt_maxpool3x3s2_bwd(int dtype, const void* dy, const uint8_t* argmax, void* dx, int N, int H,
                         int W, int C, void* stream);
int srt_avgpool_fwd(int dtype, const void* x, void* y, int N, int HW, int C, void* stream);
int srt_avgpool_bwd(int dtype, const void* dy, void* dx, int N, int HW, int C, void* stream);

/* ---- loss (replaces nn.CrossEntropyLoss, train/resnet152.py:26,87, and the loss scaling of
 *      MicroBatchManager.scale_loss, pytorch/torch_col/dynamic_batch.py:112-120) -------------- */
/* row_loss[i] = CE(logits[i], labels[i]) * grad_scale ; dlogits = (softmax - onehot) * grad_scale.
 * With grad_scale = 1/global_batch the gradients of all micro-batches sum to the global mean.
 * row_loss and dlogits may each be NULL. */
int srt_softmax_ce(int dtype, const void* logits, const int64_t* labels, int B, int classes,
                   float grad_scale, float* row_loss, void* dlogits, void* stream);
/* out[0] = (accumulate ? out[0] : 0) + sum(v[0..n)), summed in a fixed order (loss.item() of
 * train/resnet152.py:88 reads this value). */
int srt_sum_f32(const float* v, int n, float* out, int accumulate, void* stream);
/* dbias[k] = sum over rows of dy[rows][K] (fp32 out). */
int srt_colsum(int dtype, const void* dy, int64_t rows, int K, float* out, void* stream);

/* ---- optimizer + gradient accumulation (replaces torch.optim.SGD, train/resnet152.py:27-28,
 *      and GradAccumulator, pytorch/torch_col/accumulate.py:7-49) ----------------------------- */
/* g += wd*p ; m = mu*m + g (m = g on the first step) ; p -= lr*m ; optional bf16 copy of p. */
int srt_sgd_momentum(float* p, const float* g, float* m, void* p_bf16, int64_t n, float lr,
                     float mu, float wd, int first_step, void* stream);
/* AdamW with fp32 state; step counts from 1. */
int srt_adamw(float* p, const float* g, float* m, float* v, void* p_bf16, int64_t n, float lr,
              float beta1, float beta2, float eps, float wd, int step, void* stream);
/* acc += g ; g = 0  (GradAccumulator.accumulate). */
int srt_grad_accumulate(float* acc, float* g, int64_t n, void* stream);

/* ---- layout / dtype helpers ---------------------------------------------------------------- */
/* NCHW fp32 (host convention of the reference's data path, pytorch/torch_col/dynamic_batch.py:
 * 438-459) -> NHWC of `dtype` with channels zero-padded to Cpad. */
int srt_nchw_to_nhwc(int dtype, const float* src, void* dst, int N, int C, int H, int W, int Cpad,
                     void* stream);
int srt_cast_f32_to_bf16(const float* src, void* dst, int64_t n, void* stream);
int srt_cast_bf16_to_f32(const void* src, float* dst, int64_t n, void* stream);

/* ---- SM partition seen by the kernels (replaces SMPartitioner::SetStreamTpcMask,
 *      common/sm_partition.cu:316-336: the reference pokes a TPC mask into the driver's stream
 *      struct; here every persistent kernel tests %smid against this mask and retires). ------- */
/* mask[0..2]: bit i set = SM i is available to training kernels. */
int srt_set_sm_mask(const uint64_t mask[3]);
int srt_get_sm_mask(uint64_t mask[3]);
/* Enforcement of the mask (SMPartitioner::SetStreamTpcMask, common/sm_partition.cu:316-336, pokes the
 * TPC mask into a private field of the stream). Here: CUDA green contexts. The SM resource of the device
 * is split once into a ladder of groups (whole device minus 16, 32, ... SMs; the driver rounds to its
 * granularity), each with a green context and a stream; kernels launched on such a stream run on the SMs
 * of its group only. srt_smp_partition_levels lists the SM counts of the ladder (widest first, starting
 * with the whole device); srt_smp_partition_stream returns the stream of the widest group with at most
 * allowed_sms SMs (NULL = whole device: use your own stream). SRT_ERR_UNSUPPORTED without green contexts.
 * The mask's population count is what is enforced; which SMs a group holds is the driver's choice. */
int srt_smp_partition_levels(int device, int* sms, int cap, int* n);
int srt_smp_partition_stream(int device, int allowed_sms, void** stream, int* sms);
/* Test aid: ORs the %smid of every block of a probe grid launched on `stream` into three device words. */
int srt_debug_smid_probe(void* device_mask3, void* stream);

/* ---- tcgen05 kernel status ------------------------------------------------------------------
 * Every wait inside the tensor-core kernels is bounded; a wait that gives up records a non-zero
 * code here instead of hanging the GPU. Synchronises the device, returns and clears the word. */
int srt_tc_status(int* status);
/* Plan override of the tensor-core fprop/dgrad kernel for tuning and for tests that must reach every
 * code path with small problems (process-wide; 0, 0, -1 restores the heuristics):
 *   gather  1 = fetch the A operand of 1x1 stride-1 problems with the gather threads instead of TMA
 *   tile_n  output-tile width: 64, 128 or 256 filters (0 = heuristic)
 *   pair    1 = two CTAs per 256-row tile (tcgen05 cta_group::2) wherever the output is wider than 64
 *           filters, 0 = always one CTA per 128-row tile, -1 = heuristic. */
int srt_conv_plan_override(int gather, int tile_n, int pair);
/* Process-wide: whether filter gradients may use the CTA-pair kernel (256 x 256 tiles, clusters of two) where the
 * shape allows, or always the single-CTA kernel. on = 1 / 0 sets it, -1 only reads; returns the previous setting.
 * srt_conv_wgrad_scratch_bytes covers both, so the switch may change between sizing and launch. Default 1; the
 * gradient exchange (srt_ddp_create) turns it off for data-parallel runs. */
int srt_conv_wgrad_pairs(int on);

/* ---- training-step executor (replaces the body of the reference's training loop:
 *      model(images) / criterion / backward / optimizer stage, train/resnet152.py:84-91, with
 *      the micro-batch semantics of pytorch/torch_col/dynamic_batch.py:112-153 and
 *      pytorch/torch_col/accumulate.py:7-49) ---------------------------------------------------- */
typedef struct srt_step srt_step;

typedef struct srt_resnet_config {
  int layers[4];      /* bottleneck blocks per stage: {3,8,36,3} = ResNet-152, {3,4,6,3} = ResNet-50 */
  int num_classes;    /* multiple of 8 */
  int max_batch;      /* largest micro-batch; buffers are sized for it */
  int image;          /* input height = width, multiple of 32 */
  int dtype;          /* SRT_F32 or SRT_BF16 */
  int impl;           /* SRT_IMPL_* for the convolutions */
  float lr, momentum, weight_decay;   /* torch.optim.SGD(lr, momentum, weight_decay) */
  float bn_eps, bn_momentum;          /* 1e-5, 0.1 */
} srt_resnet_config;

enum { SRT_PARAM_CONV = 0, SRT_PARAM_VECTOR = 1, SRT_PARAM_BUFFER = 2, SRT_PARAM_LINEAR = 3 };
enum { SRT_GET_VALUE = 0, SRT_GET_GRAD = 1, SRT_GET_ACCUM = 2, SRT_GET_MOMENTUM = 3 };

int srt_resnet_create(const srt_resnet_config* cfg, srt_step** out);
/* Same, with the releasable part of the step's memory (saved activations, gradient buffers, scratch)
 * taken from the training allocator of `pool` (sirius_pool.h), as the reference routes every tensor
 * of the step through CUDAColAllocator -> CUDAMemPool (torch_allocator_plugin.cc:108-139). */
struct srt_pool;
int srt_resnet_create_with_pool(const srt_resnet_config* cfg, struct srt_pool* pool, srt_step** out);
/* Same, choosing the allocator of the pool: 0 = training (caching), 1 = inference (direct; what the
 * stand-in inference worker uses, as the reference's server allocates with MemType::kInfer). */
int srt_resnet_create_on_allocator(const srt_resnet_config* cfg, struct srt_pool* pool, int pool_kind,
                                   srt_step** out);
/* Memory handover, training side (ColocateCtrl.adjust_l1, pytorch/torch_col/colocate_ctrl.py:413-445:
 * release_interm_memory + MemoryPool.empty_cache): synchronises the stream, frees the activation set
 * and returns the pages that became empty to the pool. *released_bytes = bytes of pages handed back
 * (bytes freed when no pool is attached). The next forward re-allocates for its batch size. */
int srt_step_release_activations(srt_step* s, size_t* released_bytes);
int srt_step_reserve_activations(srt_step* s, int B);
/* The same handover when the trainer already knows the batch size it continues with (the adjust command
 * carries it): frees the set, places the set for micro-batches of B samples on pages that are still
 * mapped, then returns only the pages that stayed empty. The outcome equals release + the re-allocation
 * the reference's next iteration would do, but nothing is unmapped and mapped again. B == 0 releases all. */
int srt_step_shrink_activations(srt_step* s, int B, size_t* released_bytes);
/* Kill batch (ColocateStub on kColocateAdjustL1, pytorch/torch_col/csrc/control_stub.cc:486-510; the
 * reference drops the launches still queued in xsched): any thread may raise the flag; forward and
 * backward test it between units and return SRT_ERR_ABORTED, and never run more than 8 units ahead of
 * the GPU, so the stream drains within a bounded time. Clear the flag before the next micro-batch. */
int srt_step_request_abort(srt_step* s, int on);
/* The pre-launch hook of the reference (pytorch/torch_col/csrc/init.cc:43-71) sets the TPC mask before
 * every kernel. With on != 0 the step does the equivalent between units: it reads the process-wide mask
 * (srt_set_sm_mask), and continues on the partition stream of the widest group that fits the mask's SM
 * count, ordered after its earlier work by an event; grids are sized for that width. srt_step_stream()
 * then returns the stream in use at the time of the call. Off by default. */
int srt_step_follow_sm_mask(srt_step* s, int on);
/* Backward runs the filter-gradient kernels on a second stream beside the data-gradient and BatchNorm
 * kernels of the following units (on by default; the result is bit-identical either way). Off while the
 * step follows an SM partition or is being profiled per kernel family. */
int srt_step_overlap_wgrad(srt_step* s, int on);
/* Data-parallel gradient exchange overlapped with backward (the c10d Reducer's buckets,
 * pytorch/torch_col/csrc/dist_ext.{h,cc}): the flat gradient buffer (srt_step_grad_buffer) is cut at block
 * boundaries into buckets of at least 25 MiB, numbered in the order backward completes them. After
 * srt_step_forward_backward has returned (everything is enqueued, little has run), make the communication
 * stream wait for bucket i with srt_step_wait_grad_bucket and enqueue the all-reduce of
 * [offset, offset + count) floats on it; when all are enqueued, record an event on that stream and pass it to
 * srt_step_wait_event so that the optimizer runs after the exchange. */
int srt_step_num_grad_buckets(srt_step* s);
int srt_step_grad_bucket(srt_step* s, int i, int64_t* offset, int64_t* count);
int srt_step_wait_grad_bucket(srt_step* s, int i, void* stream);
int srt_step_wait_event(srt_step* s, void* cuda_event);
/* ---- gradient exchange between data-parallel ranks (replaces the reference's c10d Reducer and ProcessGroupNCCL
 *      extension: pytorch/torch_col/csrc/dist_ext.h:109-243, dist_ext.cc:59-123; abort / restart of the communicator:
 *      dist_ext.cc:673-784 _set_nccl_comm_abort_flag, _restart_nccl_comm) ---------------------------------------
 * One NCCL communicator and one communication stream per rank, owned by the library (NCCL is loaded at run time;
 * srt_ddp_available() is 0 where it cannot be). Rank 0 obtains SRT_DDP_ID_BYTES of unique id and hands it to
 * the other ranks by any channel (the mailboxes of srt_dist_*, torch.distributed, a file); every rank then calls
 * srt_ddp_create with the same id, which blocks until all ranks have joined. max_ctas > 0 caps the CTAs NCCL's
 * kernels may occupy beside the training kernels (0 = NCCL's default). Creating a communicator of more than one
 * rank also switches the CTA-pair filter-gradient kernel off for the process (srt_conv_wgrad_pairs).
 *
 * srt_allreduce_begin enqueues, on the communication stream, one sum all-reduce per bucket
 * [offsets[i], offsets[i] + counts[i]) of the fp32 buffer `grad`, bucket i behind the CUDA event ready_events[i]
 * (NULL entries or a NULL array: no wait), and returns at once. wire_dtype SRT_F32 reduces the values in place;
 * SRT_BF16 rounds each bucket to bf16 into a staging buffer of the communicator (allocated at the first such call,
 * grown when a larger buffer comes), reduces half the bytes and widens the sums back into `grad` (bucket offsets
 * must then be multiples of 8). srt_allreduce_wait makes `stream` wait for the exchange begun last. The buffer
 * must not be written between begin and the moment the waiting stream proceeds.
 * srt_step_allreduce_begin / srt_gb_allreduce_begin take buckets and events from a step executor
 * (srt_step_num_grad_buckets ..., srt_<model>_grad_buckets); srt_step_allreduce_wait orders the ResNet executor's
 * stream behind the exchange (the transformer executors: srt_allreduce_wait on srt_<model>_stream).
 * srt_ddp_abort tears the communicator down without waiting for collectives in flight (after a killed batch left
 * ranks with different numbers of collectives issued); srt_ddp_restart joins a new communicator under a new id. */
typedef struct srt_ddp srt_ddp;
#define SRT_DDP_ID_BYTES 128
int srt_ddp_available(void);
int srt_ddp_nccl_version(int* version);
int srt_ddp_unique_id(void* id);
int srt_ddp_create(const void* id, int rank, int world, int device, int max_ctas, srt_ddp** out);
int srt_ddp_destroy(srt_ddp* c);
int srt_ddp_abort(srt_ddp* c);
int srt_ddp_restart(srt_ddp* c, const void* id);
void* srt_ddp_stream(srt_ddp* c);
int srt_ddp_stats(srt_ddp* c, int64_t* exchanges, int64_t* bytes_on_wire);
int srt_allreduce_begin(srt_ddp* c, float* grad, int nbuckets, const int64_t* offsets, const int64_t* counts,
                        void* const* ready_events, int wire_dtype);
int srt_allreduce_wait(srt_ddp* c, void* stream);
/* Plain in-place sum all-reduce of `count` elements on `stream` (accumulated gradients before an update, scalars). */
int srt_ddp_allreduce(srt_ddp* c, void* buf, int64_t count, int dtype, void* stream);
int srt_step_allreduce_begin(srt_step* s, srt_ddp* c, int accumulated, int wire_dtype);
int srt_step_allreduce_wait(srt_step* s, srt_ddp* c);
int srt_gb_allreduce_begin(void* buckets, float* grad, srt_ddp* c, int wire_dtype);
int srt_step_current_sms(srt_step* s, int* sms);
int srt_step_destroy(srt_step* s);
/* Parameter registry under torchvision state_dict names ("layer1.0.conv1.weight", ...). Shapes and
 * host data use the torch layout ([K,C,R,S] for convolutions); the device keeps [K,R,S,C]. */
int srt_step_num_params(srt_step* s);
int srt_step_param_info(srt_step* s, int idx, char* name, int name_cap, int64_t shape[4], int* ndim,
                        int* kind);
int srt_step_set_param(srt_step* s, int idx, const float* host);
int srt_step_get_param(srt_step* s, int idx, float* host, int which);
/* Resume support (what loading a torch.optim.SGD state_dict does, pytorch/torch_col/util.py:182-190 pre-allocates
 * the same buffers): sets the value (which = SRT_GET_VALUE), the momentum buffer (SRT_GET_MOMENTUM; the next
 * optimizer step then continues the run instead of initialising the momentum from the gradient) or the
 * accumulated gradient (SRT_GET_ACCUM) of one parameter from host data in the torch layout. */
int srt_step_set_state(srt_step* s, int idx, const float* host, int which);
/* Rebuild the derived copies (bf16 working weights, transposed filters) after set_param. */
int srt_step_commit_params(srt_step* s);
void* srt_step_stream(srt_step* s);
/* Stage one micro-batch: NCHW fp32 images and int64 labels, from (pinned) host memory
 * (DynamicBatchDataset._retrieve_batch, pytorch/torch_col/dynamic_batch.py:438-459) or from
 * device memory. Asynchronous on the step's stream. */
int srt_step_upload_batch(srt_step* s, const float* host_images, const int64_t* host_labels, int B);
int srt_step_set_batch_device(srt_step* s, const float* dev_images, const int64_t* dev_labels, int B);
/* Forward, loss and backward of one micro-batch of B samples out of a global batch; the loss is
 * scaled by B/global_batch (MicroBatchManager.scale_loss). Gradients overwrite the gradient
 * buffer. Asynchronous. */
int srt_step_forward_backward(srt_step* s, int B, int global_batch);
int srt_step_forward_only(srt_step* s, int B);
/* Inference-mode forward (BatchNorm uses its running statistics): the stand-in for the reference's
 * TVM graph executor run, server/model_store/infer_model.cc:656-686. Logits via srt_step_logits. */
int srt_step_forward_infer(srt_step* s, int B);
/* accumulated += grad ; grad = 0  (GradAccumulator.accumulate). */
int srt_step_accumulate(srt_step* s);
/* SGD-momentum update from the accumulated gradients (or the last micro-batch's if none were
 * accumulated), then refresh of the derived weight copies (GradAccumulator.step). */
int srt_step_optimizer(srt_step* s);
/* Scaled loss of the last micro-batch; synchronises the stream (loss.item()). */
int srt_step_loss(srt_step* s, float* host_loss);
int srt_step_logits(srt_step* s, float* host, int B);
int srt_step_synchronize(srt_step* s);
/* which = 0: parameter + optimizer-state bytes; 1: activation + gradient-buffer bytes. */
int64_t srt_step_memory_bytes(srt_step* s, int which);
/* Flat fp32 gradient buffer (last micro-batch, or the accumulated one): the operand of the data-
 * parallel gradient all-reduce (c10d Reducer buckets in pytorch/torch_col/csrc/dist_ext.cc:59-123). */
int srt_step_grad_buffer(srt_step* s, int accumulated, void** ptr, int64_t* n);
/* Per-category device timing: CUDA events on the step's stream around every launch while enabled
 * (counterpart of the reference's EventManager records, pytorch/torch_col/util.py:113-178, at kernel
 * granularity). work[] is algorithmic FLOPs (CONV, WGRAD) or bytes (others). */
enum { SRT_PROF_CONV = 0, SRT_PROF_WGRAD = 1, SRT_PROF_NORM = 2, SRT_PROF_OTHER = 3, SRT_PROF_OPTIM = 4,
       SRT_PROF_NCAT = 5 };
int srt_step_profile(srt_step* s, int enable);
int srt_step_profile_read(srt_step* s, double ms[SRT_PROF_NCAT], double work[SRT_PROF_NCAT],
                          int64_t launches[SRT_PROF_NCAT]);
/* Kernel launches issued by this library in this process so far. */
int64_t srt_launch_count(void);

/* ---- transformer step (GPT-2 layout) ---------------------------------------------------------------
 * The reference trains transformers.GPT2LMHeadModel with the same torch_col loop as the vision models
 * (train/gpt2.py:26,90-97: loss = model(ids, labels=ids).loss; backward; optimizer.step). There is no
 * reference C interface for the arithmetic (it is PyTorch's); these entry points are the compute boundary of
 * this library for that model, shaped like the srt_step_* calls above. Parameters carry the names and
 * shapes of the reference's state_dict (linear weights [in][out] as its Conv1D stores them). */
typedef struct srt_gpt2 srt_gpt2;
typedef struct srt_gpt2_config {
  int n_layer, n_head, d_model, vocab, ctx; /* GPT-2 small: 12, 12, 768, 50257, 1024 */
  int max_batch, seq;                       /* sequences per micro-batch, tokens per sequence (multiple of 8) */
  float lr, beta1, beta2, eps, weight_decay; /* AdamW (torch.optim.AdamW semantics) */
  float ln_eps;                             /* 1e-5 */
} srt_gpt2_config;
int srt_gpt2_create(const srt_gpt2_config* cfg, srt_gpt2** out);
/* Colocation hooks, as for srt_step_*: batch-sized buffers from the training allocator of a page pool
 * (sirius_pool.h), release / shrink for the memory handover (ColocateCtrl.adjust_l1), kill batch between layers
 * (at most 4 layers run ahead of the GPU), gradient accumulation over micro-batches (GradAccumulator). */
struct srt_pool;
int srt_gpt2_create_with_pool(const srt_gpt2_config* cfg, struct srt_pool* pool, srt_gpt2** out);
int srt_gpt2_release_activations(srt_gpt2* g, size_t* released_bytes);
int srt_gpt2_shrink_activations(srt_gpt2* g, int B, size_t* released_bytes);
int srt_gpt2_request_abort(srt_gpt2* g, int on);
int srt_gpt2_accumulate(srt_gpt2* g);
int srt_gpt2_destroy(srt_gpt2* g);
int srt_gpt2_num_params(srt_gpt2* g);
int srt_gpt2_param_info(srt_gpt2* g, int idx, char* name, int name_cap, int64_t shape[2], int* ndim);
int srt_gpt2_set_param(srt_gpt2* g, int idx, const float* host);
int srt_gpt2_get_param(srt_gpt2* g, int idx, float* host, int which /* SRT_GET_VALUE, _GRAD, _MOMENTUM */);
int srt_gpt2_commit_params(srt_gpt2* g);                 /* after set_param: bf16 copies, transposes */
/* ids: [B][seq] int32 host array; targets are the next token of the same sequence (labels = ids). */
int srt_gpt2_upload_tokens(srt_gpt2* g, const int32_t* host_ids, int B);
/* Forward, mean cross-entropy over the targets, backward. Gradients are scaled by B / global_batch
 * (MicroBatchManager.scale_loss, pytorch/torch_col/dynamic_batch.py:112-120). */
int srt_gpt2_forward_backward(srt_gpt2* g, int B, int global_batch);
int srt_gpt2_forward_only(srt_gpt2* g, int B);
int srt_gpt2_optimizer(srt_gpt2* g);
int srt_gpt2_loss(srt_gpt2* g, float* host_loss);        /* synchronises; loss of the last micro-batch */
int srt_gpt2_logits(srt_gpt2* g, float* host, int B);    /* [B*seq][vocab], after forward_only */
int srt_gpt2_synchronize(srt_gpt2* g);
int srt_gpt2_grad_buffer(srt_gpt2* g, void** ptr, int64_t* n); /* flat fp32 gradients, for the data-parallel all-reduce */
void* srt_gpt2_stream(srt_gpt2* g);
int64_t srt_gpt2_memory_bytes(srt_gpt2* g);
int64_t srt_gpt2_num_elements(srt_gpt2* g);

/* Single operators of the transformer step, for unit parity (bf16 device tensors, fp32 parameters). */
typedef struct srt_bgemm_desc { /* D[z][m][n] = alpha * sum_k A[z][m][k] B[z][n][k]; z = (z1, z2); strides in elements */
  int M, N, K, Z1, Z2;
  long long lda, a_s1, a_s2, ldb, b_s1, b_s2, ldd, d_s1, d_s2;
  float alpha;
  int causal;   /* skip output tiles wholly above the diagonal */
  int k_causal; /* 1: A is zero for k > m, 2: A is zero for k < m */
} srt_bgemm_desc;
int srt_bgemm(const srt_bgemm_desc* d, const void* A, const void* B, void* D, void* stream);
int srt_layernorm_fwd(const void* x, const float* gamma, const float* beta, void* y, float* mean, float* rstd,
                      int64_t rows, int C, float eps, void* stream);
size_t srt_layernorm_bwd_scratch_bytes(int C);
int srt_layernorm_bwd(const void* dy, const void* x, const float* gamma, const float* mean, const float* rstd,
                      const void* addend, void* dx, float* dgamma, float* dbeta, int64_t rows, int C, void* scratch,
                      size_t scratch_bytes, void* stream);
int srt_gelu_fwd(const void* x, void* y, int64_t n, void* stream);
int srt_gelu_bwd(const void* dy, const void* x, void* dx, int64_t n, void* stream);
int srt_causal_softmax_fwd(void* scores, int64_t Z, int S, void* stream);
int srt_causal_softmax_bwd(const void* P, void* dP, int64_t Z, int S, void* stream);
int srt_batched_transpose(const void* in, void* out, int R, int C, int64_t ld_in, int64_t s1, int64_t s2, int Z1,
                          int Z2, void* stream);
int srt_lm_cross_entropy(void* logits, const int32_t* labels, int64_t rows, int V, int ld, float grad_scale,
                         float* row_loss, void* stream);

/* ---- Swin transformer step -------------------------------------------------------------------------------
 * torchvision.models.swin_b as the reference trains it (train/swin_b.py:38,83-95; AdamW in the DDP config).
 * Parameters carry torchvision's state_dict names and shapes. Same call shape as the steps above. */
typedef struct srt_swin srt_swin;
typedef struct srt_swin_config {
  int image, patch, embed;      /* Swin-B: 224, 4, 128 */
  int depths[4], heads[4];      /* 2,2,18,2 and 4,8,16,32 */
  int window, num_classes;      /* 7, 1000 */
  int max_batch;
  float lr, beta1, beta2, eps, weight_decay; /* AdamW */
  float ln_eps;                 /* 1e-5 */
} srt_swin_config;
int srt_swin_create(const srt_swin_config* cfg, srt_swin** out);
int srt_swin_destroy(srt_swin* s);
int srt_swin_num_params(srt_swin* s);
int srt_swin_param_info(srt_swin* s, int idx, char* name, int name_cap, int64_t shape[4], int* ndim);
int srt_swin_set_param(srt_swin* s, int idx, const float* host);
int srt_swin_get_param(srt_swin* s, int idx, float* host, int which);
int srt_swin_commit_params(srt_swin* s);
int srt_swin_upload_batch(srt_swin* s, const float* host_images /* NCHW fp32 */, const int64_t* host_labels, int B);
int srt_swin_forward_backward(srt_swin* s, int B, int global_batch);
int srt_swin_forward_only(srt_swin* s, int B);
int srt_swin_optimizer(srt_swin* s);
int srt_swin_loss(srt_swin* s, float* host_loss);
int srt_swin_logits(srt_swin* s, float* host, int B);
int srt_swin_synchronize(srt_swin* s);
int srt_swin_grad_buffer(srt_swin* s, void** ptr, int64_t* n);
void* srt_swin_stream(srt_swin* s);
int64_t srt_swin_memory_bytes(srt_swin* s);

/* ---- Qwen2 style decoder step ---------------------------------------------------------------------------
 * transformers Qwen2ForCausalLM as the reference trains it (train/qwen.py:35-37,80-91): RMSNorm, rotary
 * embedding, grouped-query attention, SwiGLU, tied embeddings. Parameters carry the reference's state_dict
 * names and shapes (`lm_head.weight` is the tied token table). Same call shape as srt_gpt2_*. */
typedef struct srt_qwen2 srt_qwen2;
typedef struct srt_qwen2_config {
  int n_layer, n_head, n_kv_head, hidden, intermediate, vocab; /* Qwen2-0.5B: 24, 14, 2, 896, 4864, 151936 */
  int max_batch, seq;                                          /* seq a multiple of 128 */
  float rope_theta, rms_eps;                                   /* 1e6, 1e-6 */
  float lr, beta1, beta2, eps, weight_decay;                   /* AdamW */
} srt_qwen2_config;
int srt_qwen2_create(const srt_qwen2_config* cfg, srt_qwen2** out);
/* Colocation hooks, as srt_gpt2_*: activations from the pool's training allocator, kept for the largest batch run
 * so far; shrink keeps a set for batch B and returns the other pages; request_abort makes forward_backward return
 * SRT_ERR_ABORTED at the next layer boundary (kill batch); accumulate adds the micro-batch gradients to the
 * global-batch sum that the optimizer then consumes (pytorch/torch_col/accumulate.py:7-49). */
int srt_qwen2_create_with_pool(const srt_qwen2_config* cfg, struct srt_pool* pool, srt_qwen2** out);
int srt_qwen2_accumulate(srt_qwen2* g);
int srt_qwen2_release_activations(srt_qwen2* g, size_t* released_bytes);
int srt_qwen2_shrink_activations(srt_qwen2* g, int B, size_t* released_bytes);
int srt_qwen2_request_abort(srt_qwen2* g, int on);
int srt_qwen2_destroy(srt_qwen2* g);
int srt_qwen2_num_params(srt_qwen2* g);
int srt_qwen2_param_info(srt_qwen2* g, int idx, char* name, int name_cap, int64_t shape[2], int* ndim);
int srt_qwen2_set_param(srt_qwen2* g, int idx, const float* host);
int srt_qwen2_get_param(srt_qwen2* g, int idx, float* host, int which);
int srt_qwen2_commit_params(srt_qwen2* g);
int srt_qwen2_upload_tokens(srt_qwen2* g, const int32_t* host_ids, int B);
int srt_qwen2_forward_backward(srt_qwen2* g, int B, int global_batch);
int srt_qwen2_forward_only(srt_qwen2* g, int B);
int srt_qwen2_optimizer(srt_qwen2* g);
int srt_qwen2_loss(srt_qwen2* g, float* host_loss);
int srt_qwen2_logits(srt_qwen2* g, float* host, int B);
int srt_qwen2_synchronize(srt_qwen2* g);
int srt_qwen2_grad_buffer(srt_qwen2* g, void** ptr, int64_t* n);
void* srt_qwen2_stream(srt_qwen2* g);
int64_t srt_qwen2_memory_bytes(srt_qwen2* g);

/* ---- DistilBERT-style encoder, forward only: the second model of the stand-in inference worker (the reference
 *      serves "distilbert_base" through TVM, server/model_store/infer_model.cc:46-58,394-523; arithmetic of
 *      transformers.DistilBertModel: embeddings + LayerNorm, n_layer x [Q/K/V, bidirectional attention, out
 *      projection, residual + LayerNorm, erf-GELU MLP, residual + LayerNorm]). Parameters carry the state_dict
 *      names and shapes of DistilBertModel. With a pool, activations come from its INFERENCE allocator
 *      (MemType::kInfer): reserve maps them (after a handover from the trainer), release gives the pages back. */
typedef struct srt_bert srt_bert;
typedef struct srt_bert_config {
  int n_layer, n_head, dim, hidden_dim, vocab, max_pos; /* DistilBERT-base: 6, 12, 768, 3072, 30522, 512 */
  int max_batch, seq;                                   /* seq a multiple of 8 */
  float ln_eps;                                         /* 1e-12 */
} srt_bert_config;
int srt_bert_create(const srt_bert_config* cfg, struct srt_pool* pool /* may be NULL */, srt_bert** out);
int srt_bert_destroy(srt_bert* b);
int srt_bert_num_params(srt_bert* b);
int srt_bert_param_info(srt_bert* b, int idx, char* name, int name_cap, int64_t shape[2], int* ndim);
int srt_bert_set_param(srt_bert* b, int idx, const float* host);
int srt_bert_commit_params(srt_bert* b);
int srt_bert_upload_tokens(srt_bert* b, const int32_t* host_ids, int B);
int srt_bert_forward(srt_bert* b, int B);
int srt_bert_output(srt_bert* b, float* host /* [B][seq][dim] */, int B);
int srt_bert_synchronize(srt_bert* b);
int srt_bert_stream(srt_bert* b, void** stream);
int srt_bert_release_activations(srt_bert* b, size_t* released_bytes);
int srt_bert_reserve_activations(srt_bert* b);
int srt_bert_memory_bytes(srt_bert* b, size_t* weights, size_t* activations);

/* Gradient buckets of the transformer executors, for an all-reduce overlapped with backward (as srt_step_grad_bucket
 * and friends do for the ResNet executor): srt_<model>_grad_buckets returns the executor's bucket list; buckets are
 * ranges of its flat gradient buffer in the order backward completes them. After forward_backward has returned, make
 * the communication stream wait for bucket i (srt_gb_wait), enqueue its all-reduce there, and finally make the
 * executor's stream (srt_<model>_stream) wait for an event recorded behind the last one (srt_stream_wait_event). */
void* srt_gpt2_grad_buckets(srt_gpt2* g);
void* srt_swin_grad_buckets(srt_swin* s);
void* srt_qwen2_grad_buckets(srt_qwen2* g);
int srt_gb_count(void* buckets);
int srt_gb_get(void* buckets, int i, int64_t* offset, int64_t* count);
int srt_gb_wait(void* buckets, int i, void* stream);
int srt_stream_wait_event(void* stream, void* cuda_event);

#ifdef __cplusplus
}
#endif
#endif /* SIRIUS_B200_H_ */
