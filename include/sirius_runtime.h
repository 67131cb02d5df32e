/*
 * sirius_b200 — C ABI of the host-side runtime of the colocated training step: the training-side
 * half of Sirius's control plane, rebuilt on POSIX shared memory and pthreads (the reference builds
 * on Boost.Interprocess and glog). Same conventions as sirius_b200.h: int status, no exceptions,
 * srt_last_error() for the message. Citations are paths inside the Sirius reference tree.
 *
 * Shared-memory byte layouts are this library's own; compatibility with the reference is at the
 * level of names, message values and behaviour, not of segment bytes.
 */
#ifndef SIRIUS_RUNTIME_H_
#define SIRIUS_RUNTIME_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SRT_MAX_DEVICE_NUM 8 /* common/util.h:56 */

/* ---- inf_tra_comm: control messages and the shared information board ------------------------
 * (common/inf_tra_comm/message_queue.h:12-40,144-196; shared_info.h:16-35; communicator.cc:15-48) */
typedef struct srt_ctrl_msg {
  uint64_t id;
  int event;
  int value;
} srt_ctrl_msg;

/* CtrlEvent, same ordinals as common/inf_tra_comm/message_queue.h:18-40 */
enum {
  SRT_EV_TRAIN_START = 0, SRT_EV_TRAIN_END, SRT_EV_INTERRUPT_TRAIN_DONE, SRT_EV_RESUME_TRAIN_DONE,
  SRT_EV_COLOCATE_ADJUST_L1_DONE, SRT_EV_COLOCATE_ADJUST_L2_DONE, SRT_EV_REPORT_BATCH_SIZE,
  SRT_EV_INTERRUPT_TRAIN, SRT_EV_RESUME_TRAIN, SRT_EV_COLOCATE_ADJUST_L1, SRT_EV_COLOCATE_ADJUST_L2,
  SRT_EV_INFER_EXIT, SRT_EV_INFERENCE_WORKLOAD_DONE, SRT_EV_NUM_EVENT
};
enum { SRT_INF2TRA = 0, SRT_TRA2INF = 1 };

typedef struct srt_train_info { /* ctrl::TrainInfo */
  int train_pid;   /* -1 = invalid */
  int train_rank;
  int train_world_size;
  int init_batch_size;
  int current_batch_size;
  int target_batch_size;
  int target_batch_size_unpublished;
  char model_name[256];
  int first_epoch_done;
} srt_train_info;
enum { SRT_TI_PID = 0, SRT_TI_RANK, SRT_TI_WORLD_SIZE, SRT_TI_INIT_BS, SRT_TI_CURRENT_BS, SRT_TI_TARGET_BS,
       SRT_TI_TARGET_BS_UNPUBLISHED, SRT_TI_FIRST_EPOCH_DONE };

typedef struct srt_comm srt_comm;
/* name == NULL: "colserve_shm_<user>_p<SIRIUS_PORT>_inf_tra_comm" (common/util.h:113-132). The server
 * creates (cleanup != 0 removes a stale segment first); trainers open and wait up to timeout_ms. */
int srt_comm_open(const char* name, int is_server, int cleanup, int train_world_size, int timeout_ms,
                  srt_comm** out);
int srt_comm_close(srt_comm* c);
int srt_comm_world_size(srt_comm* c);
int srt_comm_put(srt_comm* c, const srt_ctrl_msg* msg, int direction, int rank);
/* n == 1: the same message to every rank; n == world size: msgs[i] to rank i (PutAll). */
int srt_comm_put_all(srt_comm* c, const srt_ctrl_msg* msgs, int n, int direction);
/* timeout_ms < 0 blocks, 0 polls. *got = 1 when a message was taken. */
int srt_comm_timed_get(srt_comm* c, int timeout_ms, int direction, int rank, srt_ctrl_msg* out, int* got);
int srt_comm_timed_get_from_any(srt_comm* c, int timeout_ms, int direction, int* rank, srt_ctrl_msg* out,
                                int* got);
int srt_comm_clear(srt_comm* c);
int srt_comm_set_train_info(srt_comm* c, int rank, const srt_train_info* info);
int srt_comm_get_train_info(srt_comm* c, int rank, srt_train_info* out);
int srt_comm_update_train_field(srt_comm* c, int rank, int field, int value);
int srt_comm_get_train_field(srt_comm* c, int rank, int field, int* out);
int srt_comm_invalidate_train_info(srt_comm* c, int rank);
/* InferInfo::tpc_datas[device].infer_required_tpc_num (common/sm_partition.cc:60-76): op 0 set, 1 add,
 * 2 subtract, 3 read; *out receives the value after the operation. */
int srt_comm_infer_tpc(srt_comm* c, int device, int op, int value, int* out);

/* ---- SM partition (common/sm_partition.cc:78-112) -------------------------------------------- */
/* Mask of TPCs DISABLED for training given how many the inference side asked for: the low
 * `n` TPCs, n clamped to [gpu_tpc - max_train, gpu_tpc - min_train] (0 required = no mask). */
uint64_t srt_smp_train_avail_tpc_mask(int infer_required_tpc, int gpu_tpc_num, int min_train_tpc,
                                      int max_train_tpc);
int srt_smp_train_avail_tpc_num(int infer_required_tpc, int gpu_tpc_num, int min_train_tpc, int max_train_tpc);
/* Wide form for GPUs with more than 64 TPCs/SMs: allowed_sm[3] gets one bit per SM that training may
 * use (TPC i = SMs 2i, 2i+1; training keeps the high-index TPCs as in the reference). */
int srt_smp_allowed_sm_mask(int infer_required_tpc, int gpu_sm_num, int min_train_tpc, int max_train_tpc,
                            uint64_t allowed_sm[3]);

/* The pre-launch hook (pytorch/torch_col/csrc/init.cc:56-62): between units the step reads
 * infer_required_tpc_num of `device` from the board, keeps srt_smp_train_avail_tpc_num() TPCs and moves to
 * the green-context partition that fits (sirius_b200.h: srt_step_follow_sm_mask). comm == NULL turns it off.
 * The comm handle must outlive the step or be detached first. */
struct srt_step;
int srt_step_follow_infer_tpc(struct srt_step* s, srt_comm* comm, int device, int min_train_tpc, int max_train_tpc);
/* The same hook for the transformer executors, checked between layers (GPT-2, Qwen2) or blocks (Swin): the
 * executor moves its main stream and the low-priority stream of its weight gradients to the partition that fits.
 * enable = 0 brings it back to its whole-device streams; enable = 1 with comm == NULL follows the process-wide
 * allowed-SM mask instead of a board. *_current_sms: SMs of the partition in use (the device's SM count when none is). */
struct srt_gpt2;
struct srt_qwen2;
struct srt_swin;
int srt_gpt2_follow_infer_tpc(struct srt_gpt2* g, srt_comm* comm, int device, int min_train_tpc, int max_train_tpc, int enable);
int srt_qwen2_follow_infer_tpc(struct srt_qwen2* g, srt_comm* comm, int device, int min_train_tpc, int max_train_tpc, int enable);
int srt_swin_follow_infer_tpc(struct srt_swin* g, srt_comm* comm, int device, int min_train_tpc, int max_train_tpc, int enable);
int srt_gpt2_current_sms(struct srt_gpt2* g);
int srt_qwen2_current_sms(struct srt_qwen2* g);
int srt_swin_current_sms(struct srt_swin* g);

/* ---- DistTrainSync, DynamicBatchDistirbutor, PerfModel ----------------------------------------
 * (pytorch/torch_col/csrc/dist_train_sync.{h,cc}, dynamic_batch.{h,cc}, perf_model.{h,cc}) */
typedef struct srt_dist srt_dist;
/* One segment per training job; rank 0 creates it, the others wait up to timeout_ms (the reference
 * waits 10 s, dist_train_sync.cc:109-116). name == NULL: default "<prefix>_dist_train_sync". */
int srt_dist_open(const char* name, int rank, int world_size, int timeout_ms, srt_dist** out);
int srt_dist_close(srt_dist* d);
int srt_dist_barrier(srt_dist* d, int timeout_ms);                       /* WaitBarrier */
int srt_dist_send(srt_dist* d, int dst, const char* data, int nbytes);    /* Send */
int srt_dist_recv(srt_dist* d, int src, char* buf, int cap, int timeout_ms, int* nbytes);
/* Task-switch flags shared by the ranks of a job (SwitchStub's shared data, control_stub.cc:186-200):
 * which 0 = global interrupt flag, 1 = a batch has been killed. set != 0 stores value; *out gets the flag. */
int srt_dist_switch_flag(srt_dist* d, int which, int set, int value, int* out);

enum { SRT_DBD_FIX = 0, SRT_DBD_SIMPLE = 1, SRT_DBD_BY_PERFORMANCE = 2 };
int srt_dbd_init(srt_dist* d, int dataset_size, int input_batch_size, int global_batch_size,
                 int lazy_distributing, int policy);
/* comm may be NULL (no colocated inference server): targets fall back to input_batch_size. */
int srt_dbd_distribute_batch(srt_dist* d, srt_comm* comm, int check_num_unproced_samples,
                             int distribute_to_all, int at_global_batch_begin);
/* ranges: pairs [first, second) of sample indices; *n_ranges pairs written; *last_micro_batch set. */
int srt_dbd_get_batch(srt_dist* d, int batch_size, int* ranges, int cap_pairs, int* n_ranges,
                      int* last_micro_batch);
int srt_dbd_query_next_batch_size(srt_dist* d, int batch_size, int* out);
int srt_dbd_finish_batch(srt_dist* d, const int* ranges, int n_ranges, int end_of_global_batch);
int srt_dbd_abort_batch(srt_dist* d, const int* ranges, int n_ranges, int end_of_global_batch);
/* *finished = 1 when every rank voted to finish, 0 when any rank aborted. */
int srt_dbd_vote_finish_last_micro_batch(srt_dist* d, int timeout_ms, int* finished);
int srt_dbd_vote_abort_last_micro_batch(srt_dist* d);
int srt_dbd_reset_last_micro_batch_finish_vote(srt_dist* d);
int srt_dbd_next_global_batch(srt_dist* d, srt_comm* comm, int timeout_ms);
int srt_dbd_next_epoch(srt_dist* d, int* epoch);
enum { SRT_DBD_GLOBAL_BATCH_SIZE = 0, SRT_DBD_NUM_GLOBAL_BATCH_PER_EPOCH, SRT_DBD_NUM_PROCED_GLOBAL_BATCH,
       SRT_DBD_NUM_UNPROC, SRT_DBD_NUM_PROCING, SRT_DBD_NUM_PROCED, SRT_DBD_RANK_UNPROC, SRT_DBD_RANK_PROCING,
       SRT_DBD_RANK_PROCED };
int srt_dbd_info(srt_dist* d, int which, int rank, int* out);

int srt_perf_record_thpt(srt_dist* d, int batch_size, double batch_time_ms);  /* PerfModel::RecordThpt */
int srt_perf_get_thpt(srt_dist* d, int batch_size, double* thpt);             /* PerfModel::GetThpt */

/* ---- TrainAdjuster (server/train_adjuster.{h,cc}) -------------------------------------------- */
typedef struct srt_adjuster srt_adjuster;
typedef struct srt_adjuster_config {
  double base_mb, slope_mb;         /* memory model mem = base + slope*batch; <= 0: table by model name */
  int batch_size_limit;             /* Config::train_adjust_batch_size_limit (0) */
  int enable_balance;               /* Config::enable_train_adjust_balance */
  double balance_threshold_mb;      /* Config::train_adjust_balance_threshold (1500) */
  int num_visible_gpu;
  int use_shared_tensor;
} srt_adjuster_config;
int srt_adjuster_create(srt_comm* comm, const srt_adjuster_config* cfg, srt_adjuster** out);
int srt_adjuster_destroy(srt_adjuster* a);
int srt_adjuster_load_train_info(srt_adjuster* a);
int srt_adjuster_reset_train_info(srt_adjuster* a);
/* GetModelMemParam (server/train_adjuster.cc:642-698): the reference's hand-fit constants for its PyTorch models. */
int srt_adjuster_model_mem_param(const char* model_name, double* base_mb, double* slope_mb);
/* The line measured for this library's executors on a B200; what the adjuster uses when the configuration gives no
 * slope, unless SIRIUS_B200_ADJUSTER_FIT=reference. */
int srt_adjuster_model_mem_param_measured(const char* model_name, double* base_mb, double* slope_mb);
int srt_adjuster_predict_train_mem_mb(srt_adjuster* a, int batch_size, double* mem_mb);
/* plan_bs[world]: target batch size per rank; *n = 0 when no adjustment is needed. Also writes
 * target_batch_size_unpublished of every rank (UpdateCachedTrainInfoByAdjustPlan).
 * train_avail_mb_minus_reserve[world] feeds the imbalance check (may be NULL when balance is off). */
int srt_adjuster_infer_require_plan(srt_adjuster* a, int device_id, double required_mem_mb,
                                    const double* train_avail_mb_minus_reserve, int* plan_bs, int* n);
int srt_adjuster_infer_release_plan(srt_adjuster* a, const double* train_avail_mb, const double* free_mb,
                                    const double* reserve_mb, int* plan_bs, int* n);

/* PredictTrainMemUsageMB (train_adjuster.cc:55-83): base + slope * the planned target batch of `device_id`. */
int srt_adjuster_predict_train_mem_usage_mb(srt_adjuster* a, int device_id, double* mem_mb);
/* The KV-cache pool's plans (train_adjuster.cc:343-520): the caller derives the memory figures from the page
 * pool (see srt_kvpool_*). *n = 0 when there is nothing to adjust. */
int srt_adjuster_llm_require_plan(srt_adjuster* a, int device_id, double required_mem_mb, double train_avail_mem_mb,
                                  const double* train_avail_mb_minus_reserve, int* plan_bs, int* n);
int srt_adjuster_llm_release_plan(srt_adjuster* a, const double* train_avail_mb, const double* free_mb, int* plan_bs,
                                  int* n);

/* ---- ColocateStub: the trainer's control thread (pytorch/torch_col/csrc/control_stub.{h,cc}) ------ */
typedef struct srt_stub srt_stub;
struct srt_step;
typedef struct srt_stub_config {
  int rank, world_size;
  int kill_batch_on_recv;   /* TorchColConfig::kill_batch_on_recv (hook mode xsched-sync2, config.cc:98-102) */
  int is_colocate_l1;
  int input_batch_size;     /* used when there is no inference server */
  int poll_ms;              /* timed get of the control thread; 0 = 1000 as in control_stub.cc:67-70 */
  int task_switch;          /* 1 = SwitchStub (kInterruptTrain / kResumeTrain), 0 = ColocateStub */
} srt_stub_config;
/* comm == NULL: no colocated inference server (no thread is started). step/dist may be NULL; with a
 * step the kill raises srt_step_request_abort, with a dist rank 0 redistributes on kInferExit. */
int srt_stub_create(srt_comm* comm, struct srt_step* step, srt_dist* dist, const srt_stub_config* cfg,
                    srt_stub** out);
/* Executors other than the ResNet one: what the kill means is fn(arg, 1) and clearing it fn(arg, 0), e.g.
 * (srt_gpt2_request_abort, handle). Set it right after srt_stub_create with step == NULL. */
int srt_stub_set_abort_target(srt_stub* s, int (*fn)(void*, int), void* arg);
int srt_stub_stop(srt_stub* s);       /* StubBase::Stop + destruction */
int srt_stub_cmd(srt_stub* s);        /* GetCmd: pending CtrlEvent or -1 */
int srt_stub_set_cmd(srt_stub* s, int cmd);
uint64_t srt_stub_cmd_id(srt_stub* s);
int srt_stub_train_start(srt_stub* s);
int srt_stub_train_end(srt_stub* s);
int srt_stub_report_batch_size(srt_stub* s, int batch_size);
int srt_stub_steps_no_interrupt_begin(srt_stub* s);
int srt_stub_steps_no_interrupt_end(srt_stub* s);
int srt_stub_adjust_l1_done(srt_stub* s);
int srt_stub_adjust_l2_done(srt_stub* s);
int srt_stub_target_batch_size(srt_stub* s, int unpublished, int* out);
int srt_stub_set_killed_batch_recover(srt_stub* s);     /* SetKilledBatchRecover: the next adjust may kill again */
int srt_stub_set_killed_batch_reconfiged(srt_stub* s);  /* SetKilledBatchReconfiged: redistribution after the kill is done */
int srt_stub_set_train_first_epoch_done(srt_stub* s);
int srt_stub_can_exit_after_infer_workload_done(srt_stub* s);
double srt_stub_passed_ms_from_set_cmd(srt_stub* s);
/* SwitchStub (task-switch mode, control_stub.cc:186-400). kInterruptTrain raises the global interrupt flag, kills the
 * batch in flight and becomes the pending command; the trainer releases its memory and calls
 * try_interrupt_train_done (replies kInterruptTrainDone once per command; *done = 1 when it replied). The trainer
 * then polls prepare_resume until kResumeTrain has arrived on every rank (two barriers over the shared flag; a new
 * interrupt in between is answered at once); the master replies kResumeTrainDone. switch_flag reads or writes the
 * shared flags (which as srt_dist_switch_flag). */
int srt_stub_try_interrupt_train_done(srt_stub* s, int barrier, int* done);
int srt_stub_prepare_resume(srt_stub* s, int* resumed);
int srt_stub_switch_flag(srt_stub* s, int which, int set, int value, int* out);
/* StubProfiler: microsecond unix timestamps of adjust requests / replies; returns how many exist. */
int srt_stub_adjust_timestamps(srt_stub* s, int done, int64_t* out, int cap);

#ifdef __cplusplus
}
#endif
#endif /* SIRIUS_RUNTIME_H_ */
