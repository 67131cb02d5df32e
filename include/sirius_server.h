/*
 * sirius_b200 — C ABI of the server side of the colocation protocol: what the inference server runs to talk to
 * the trainers (Controller), to decide how much memory it may take (ResourceManager, ColdModelCache), to start
 * a training job with the right environment (TrainLauncher), and to serve an LLM's KV cache from the page pool
 * while trading pages with training (KVCachePool).
 *
 * These replace, for the colocated training step, the corresponding classes of the reference's server
 * (server/control/controller.{h,cc}, server/resource_manager.{h,cc}, server/model_store/model_cache.{h,cc},
 * server/train_launcher.cc, server/llm/kv_cache_pool.{h,cc}). The model executors of that server (TVM graph
 * executor, vLLM) are outside this library; a server, or the stand-in inference workers of the benchmarks, call
 * this layer around their own model code. Every function returns a status (0 = ok) and leaves a message in
 * srt_last_error(); none aborts, and every wait takes a timeout in milliseconds (negative = no limit; the
 * reference's waits have none).
 */
#ifndef SIRIUS_SERVER_H_
#define SIRIUS_SERVER_H_

#include <stddef.h>
#include <stdint.h>

#include "sirius_pool.h"
#include "sirius_runtime.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---- Controller (server/control/controller.cc:84-445) ---------------------------------------------------
 * Owns the server end of the inf_tra_comm channel. A monitor thread (Controller::TrainMonitor) drains the
 * trainer-to-server queues: kTrainStart / kTrainEnd move the training status, kColocateAdjustL1/L2Done record
 * the command id a rank has acknowledged, kInterruptTrainDone / kResumeTrainDone drive the task-switch state,
 * kReportBatchSize records the batch size the trainer runs at. */
typedef struct srt_controller srt_controller;
enum { SRT_SERVE_NORMAL = 0, SRT_SERVE_TASKSWITCH_L1, SRT_SERVE_TASKSWITCH_L3, SRT_SERVE_COLOCATE_L1, SRT_SERVE_COLOCATE_L2 };
enum { SRT_TRAIN_IDLE = 0, SRT_TRAIN_RUNNING = 1, SRT_TRAIN_INTERRUPTED = 2 };
typedef struct srt_controller_config {
  int serve_mode;    /* SRT_SERVE_* (Config::serve_mode) */
  int dummy_adjust;  /* Config::dummy_adjust: InferenceWorkloadDone is not forwarded */
} srt_controller_config;
/* comm: the channel opened as server (srt_comm_open with is_server = 1). adjuster may be NULL; when given, its
 * train info is loaded on kTrainStart as TrainAdjuster::LoadTrainInfo does. */
int srt_controller_create(srt_comm* comm, srt_adjuster* adjuster, const srt_controller_config* cfg, srt_controller** out);
int srt_controller_destroy(srt_controller* c);
int srt_controller_train_status(srt_controller* c, int* status);
int srt_controller_cur_batch_size(srt_controller* c, int* batch_size);      /* last kReportBatchSize */
int srt_controller_set_train_pid(srt_controller* c, int pid);               /* task-switch L3 kills this process */
/* InterruptTrain / ResumeTrain: *cmd_id = 0 when nothing was sent (no training, or an interrupt without a resume
 * since the last one). */
int srt_controller_interrupt_train(srt_controller* c, uint64_t* cmd_id);
int srt_controller_resume_train(srt_controller* c, uint64_t* cmd_id);
/* ColocateAdjust (:203-262): lower every rank's target by batch_size unless an earlier plan already covers it
 * (no rank has unpublished < published target): *cmd_id = 0 then. */
int srt_controller_colocate_adjust(srt_controller* c, int device_id, int batch_size, uint64_t* cmd_id);
/* ColocateInferRequireAdjust / ColocateInferReleaseAdjust (:264-328): plan_bs[n] from the TrainAdjuster, one
 * kColocateAdjustL1/L2 (require) or kInferExit (release) message per rank carrying that rank's batch size. */
int srt_controller_infer_require_adjust(srt_controller* c, int device_id, const int* plan_bs, int n, uint64_t* cmd_id);
int srt_controller_infer_release_adjust(srt_controller* c, const int* plan_bs, int n, uint64_t* cmd_id);
int srt_controller_dummy_infer_exit(srt_controller* c, int device_id, int target_batch_size, uint64_t* cmd_id);
int srt_controller_inference_workload_done(srt_controller* c);
/* Waits (:330-376). SRT_ERR_TIMEOUT when the limit passes first; all return at once when training is idle. */
int srt_controller_wait_train_not_running(srt_controller* c, int timeout_ms);
int srt_controller_wait_task_switch_done(srt_controller* c, uint64_t cmd_id, int timeout_ms);
int srt_controller_wait_colocate_adjust_done(srt_controller* c, int device_id, uint64_t cmd_id, int timeout_ms);
int srt_controller_set_infer_status(srt_controller* c, int running);
int srt_controller_wait_infer_idle(srt_controller* c, int timeout_ms);
int srt_controller_has_flying_colocate_adjust(srt_controller* c, int* flying);

/* ---- ResourceManager (server/resource_manager.cc:22-104), shared-tensor mode: all figures from the page pool -- */
double srt_resmgr_infer_memory_mb(srt_pool* pool);
double srt_resmgr_train_memory_mb(srt_pool* pool);
/* pool size - inference usage - max(training usage, predicted training usage) - over_predict_mb */
int srt_resmgr_free_memory_mb(srt_pool* pool, srt_adjuster* adjuster, int device_id, double over_predict_mb, double* out);
/* pool size - inference usage - over_predict_mb */
int srt_resmgr_train_avail_memory_mb(srt_pool* pool, double over_predict_mb, double* out);

/* ---- ColdModelCache (server/model_store/model_cache.{h,cc}:93-270, 209-500): bookkeeping of the parameter
 * groups of cold models kept in GPU memory between requests, with a capacity that moves between a minimum and
 * a maximum; what capacity exceeds the cached bytes is the reserve training must not plan with. */
typedef struct srt_cold_cache srt_cold_cache;
typedef struct srt_cold_cache_config {
  size_t min_capacity_nbytes, max_capacity_nbytes;  /* Config::cold_cache_{min,max}_capacity_nbytes */
  double ratio;                                      /* Config::cold_cache_ratio: share of a model that may be cached */
} srt_cold_cache_config;
int srt_cold_cache_create(const srt_cold_cache_config* cfg, srt_cold_cache** out);
int srt_cold_cache_destroy(srt_cold_cache* c);
/* PushCacheItem: groups_nbytes[n_groups] of model `name` (hotness decides the eviction order: coldest first).
 * cached_groups[cap] receives the indices of the groups that stay cached (*n_cached of them); evicted (a
 * buffer of evicted_cap bytes) receives the names of the models evicted to make room, separated by '\n'.
 * *ok = 0 when the model is cached already. */
int srt_cold_cache_push(srt_cold_cache* c, const char* name, double hotness, const size_t* groups_nbytes, int n_groups,
                        int* cached_groups, int cap, int* n_cached, char* evicted, size_t evicted_cap, int* ok);
/* PopCacheItem: pop_to_inference != 0 also shrinks the capacity by what was cached (the model is being loaded). */
int srt_cold_cache_pop(srt_cold_cache* c, const char* name, int pop_to_inference, int* cached_groups, int cap, int* n_cached,
                       int* ok);
int srt_cold_cache_take_space(srt_cold_cache* c, size_t nbytes, int* ok);   /* TakeSpace */
int srt_cold_cache_set_capacity(srt_cold_cache* c, size_t nbytes);          /* SetNewCapacity */
int srt_cold_cache_info(srt_cold_cache* c, size_t* capacity_nbytes, size_t* cached_nbytes);
double srt_cold_cache_reserve_mb(srt_cold_cache* c);                        /* Get{Release,Adjust}ReserveMemoryMB */
double srt_cold_cache_releasable_mb(srt_cold_cache* c);                     /* GetColdCacheReleasableMemoryMBUnsafe */
double srt_cold_cache_buffer_mb(srt_cold_cache* c, double free_memory_mb);  /* GetBufferMBUnsafe */

/* ---- TrainLauncher (server/train_launcher.cc:88-311): the environment and command line of a training job ---- */
typedef struct srt_launcher_config {
  int serve_mode;                 /* SRT_SERVE_* */
  int use_xsched;                 /* COLTRAIN_USE_XSCHED, and the hook mode xsched-sync2 instead of sync */
  int use_shared_tensor_train;    /* COLTRAIN_USE_SHARED_TENSOR / COLTRAIN_HAS_SHARED_TENSOR_SERVER / ..._POOL_GB */
  double cuda_memory_pool_gb;
  const char* freelist_policy;    /* SHARED_TENSOR_POOL_FREELIST_POLICY (may be NULL) */
  const char* train_profile;      /* COLTRAIN_PROFILE_LOG_PATH (may be NULL or empty) */
  int skip_set_mps_thread_percent, dynamic_sm_partition, train_mps_thread_percent;
  int enable_train_adjust_balance;  /* COLTRAIN_BATCH_DISTRIBUTE_POLICY = BY_PERFORMANCE, else FIX */
} srt_launcher_config;
/* The variables LaunchTrain sets in the child, as "NAME=value" lines in buf. */
int srt_launcher_env(const srt_launcher_config* cfg, char* buf, size_t cap);
/* "batch-size=64, num-epoch=3" -> "python\n<script>\n--batch-size\n64\n--num-epoch\n3" (Train(), :110-128);
 * *batch_size gets the value of the argument whose name contains "batch-size" (0 if there is none). */
int srt_launcher_argv(const char* script, const char* args, char* buf, size_t cap, int* batch_size);
/* fork, set the environment, exec `interpreter` (NULL = "python") with that command line. log_path (may be
 * NULL) receives the child's stdout and stderr. */
int srt_launcher_launch(const srt_launcher_config* cfg, const char* interpreter, const char* script, const char* args,
                        const char* log_path, int* pid);
/* *exited = 1 with the wait status in *status once the child is gone; timeout_ms = 0 polls. */
int srt_launcher_wait(int pid, int timeout_ms, int* exited, int* status);
int srt_launcher_kill(int pid);
/* Supervision of a launched job (the tail of LaunchTrain, server/train_launcher.cc:335-381): waits up to timeout_ms
 * (-1 = for ever) for `pid`. When it has ended, the controller (may be NULL) forgets the pid and is told that training
 * has ended (Controller::TrainEnd, in case the trainer could not say so), *status gets the exit status (128 + signal
 * for a signalled child) and *outcome says what the end means:
 *   SRT_JOB_RUNNING   still running after timeout_ms
 *   SRT_JOB_FINISHED  it exited by itself
 *   SRT_JOB_KILLED    SIGKILL (task-switch l3's InterruptTrain, srt_launcher_kill, KillTrain): launch it again
 *   SRT_JOB_FAILED    any other signal: every rank on the board of `comm` (may be NULL) is killed and the call returns
 *                     SRT_ERR_STATE, srt_last_error() naming the signal and the batch sizes on the board (the
 *                     reference ends the server process at this point). */
enum { SRT_JOB_RUNNING = 0, SRT_JOB_FINISHED = 1, SRT_JOB_KILLED = 2, SRT_JOB_FAILED = 3 };
int srt_launcher_supervise(srt_controller* c, srt_comm* comm, int pid, int timeout_ms, int* outcome, int* status);
/* KillTrain (:410-427): SIGKILL to every rank whose TrainInfo on the board is valid; *killed (may be NULL) counts them. */
int srt_launcher_kill_train(srt_comm* comm, int* killed);
/* DummyAdjust (:383-408), the reference's fault injector for the adjust protocol (Config::dummy_adjust): blocks for
 * delay_ms (-1 = the reference's 60 s), then for duration_ms (0 = 60 s) or until training is idle repeats: ColocateAdjust
 * by one sample, wait for Done, DummyInferExit back to original_target_bs, sleep a uniform random min_gap_ms..max_gap_ms
 * (0 = 200..1000) drawn from std::mt19937(seed; 0 = 42). *rounds (may be NULL) counts the adjusts. The controller must
 * have been created with dummy_adjust = 1. Run it on a thread of its own. */
int srt_launcher_dummy_adjust(srt_controller* c, int original_target_bs, int delay_ms, int duration_ms, unsigned seed,
                              int min_gap_ms, int max_gap_ms, int* rounds);

/* ---- KVCachePool (server/llm/kv_cache_pool.cc:232-347): the LLM server's KV cache in pool pages ------------
 * KV-cache pages are blocks of page_nbytes from the pool's inference allocator. When the pool cannot supply a
 * request next to the memory training is predicted to need, training is asked to shrink first
 * (MaybeAdjustTrain: LLM require plan -> ColocateInferRequireAdjust -> wait for the Done replies); when pages come
 * back and at least reclaim_free_nbytes of the pool are free, training is told it may grow (ReclaimMemToTrain:
 * LLM release plan -> ColocateInferReleaseAdjust). */
typedef struct srt_kvpool srt_kvpool;
typedef struct srt_kvpool_config {
  int device_id;
  double train_memory_over_predict_mb;  /* Config::train_memory_over_predict_mb */
  size_t train_over_adjust_nbytes;      /* Config::train_over_adjust_nbytes */
  size_t min_adjust_nbytes;             /* 0 = 5 GiB: an adjust asks for at least this much */
  size_t reclaim_free_nbytes;           /* 0 = 6 GiB: free pool memory from which pages flow back to training */
  size_t reclaim_margin_nbytes;         /* 0 = 4 GiB: kept out of the release plan's free figure */
  int adjust_timeout_ms;                /* 0 = 60000 */
} srt_kvpool_config;
int srt_kvpool_create(srt_pool* pool, srt_controller* controller, srt_adjuster* adjuster, const srt_kvpool_config* cfg,
                      srt_kvpool** out);
int srt_kvpool_destroy(srt_kvpool* k);
/* MaybeSetKVCacheBlockNbytes: block_size tokens x num_heads x head_size per layer, block_nbytes per block over all layers. */
int srt_kvpool_set_block_shape(srt_kvpool* k, int64_t block_size, int64_t num_layers, int64_t num_heads, int64_t head_size,
                               size_t block_nbytes);
int64_t srt_kvpool_num_gpu_blocks(srt_kvpool* k);                          /* pool bytes / block bytes */
int srt_kvpool_shape(srt_kvpool* k, int64_t shape[3], int64_t stride[3]);   /* GetKVCacheShape / GetKVCacheStride */
int srt_kvpool_layer_block_info(srt_kvpool* k, int64_t* free_blocks, int64_t* used_blocks);
int srt_kvpool_update_free_layer_blocks(srt_kvpool* k, int64_t delta);
int srt_kvpool_update_free_layer_blocks_by_train_base(srt_kvpool* k, size_t train_base_nbytes);
/* AllocKVCachePage / FreeKVCachePage: n pages of page_nbytes; pages[] are device addresses. *adjusted = 1 when
 * training had to shrink first. */
int srt_kvpool_alloc_pages(srt_kvpool* k, size_t page_nbytes, int n, uint64_t* pages, int* adjusted);
int srt_kvpool_free_pages(srt_kvpool* k, const uint64_t* pages, int n, int* reclaimed_to_train);
double srt_kvpool_util(srt_kvpool* k);                                      /* GetKVCachePoolkUtil; NaN before the shape is set */

#ifdef __cplusplus
}
#endif
#endif /* SIRIUS_SERVER_H_ */
