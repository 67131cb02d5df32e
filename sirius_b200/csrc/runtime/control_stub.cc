// ColocateStub: the thread in every trainer that listens on the Inf2Tra queue and turns control
// messages into state the training loop polls (cmd), plus the status messages the trainer sends back.
//
// Follows pytorch/torch_col/csrc/control_stub.cc of the reference: the 1 s timed-get loop (:60-79),
// TrainStart/TrainEnd/ReportBatchSize (:97-128), the step mutex (:130-138), ColocateStub::
// ProcessCtrlMsg with kill-batch and the immediate-reply rule (:423-593), the Done replies (:595-629)
// and StubProfiler (:642-652). The reference kills a batch by rejecting CUDA calls and dropping the
// launches queued in its libcuda shim; here the step executor is told to stop between units
// (srt_step_request_abort), which bounds the drain to the units already in flight.
//
// With cfg.task_switch the same object is the SwitchStub (:186-400): kInterruptTrain / kResumeTrain, the
// interrupt flag shared by the ranks, TryInterruptTrainDone and PrepareResume.
#include <sys/time.h>

#include <atomic>
#include <chrono>
#include <mutex>
#include <thread>
#include <vector>

#include "../../../include/sirius_b200.h"
#include "../../../include/sirius_runtime.h"
#include "rt_common.h"

namespace srt {

static int64_t unix_us() {
  timeval tv;
  gettimeofday(&tv, nullptr);
  return (int64_t)tv.tv_sec * 1000000 + tv.tv_usec;
}

struct Stub {
  srt_comm* comm = nullptr;
  srt_step* step = nullptr;
  // what raising / clearing the kill flag means: by default the ResNet executor's call on `step`
  int (*abort_fn)(void*, int) = nullptr;
  void* abort_arg = nullptr;
  void request_abort(int on) {
    if (abort_fn) abort_fn(abort_arg, on);
    else if (step) srt_step_request_abort(step, on);
  }
  srt_dist* dist = nullptr;
  srt_stub_config cfg;
  std::thread th;
  std::atomic<bool> running{false};
  std::mutex mu, step_mu, prof_mu;
  std::atomic<int> cmd{-1};
  uint64_t cmd_id = 0;
  std::atomic<bool> has_killed_batch_recover{true}, will_killed_batch_reconfig{false};
  std::atomic<bool> exec_step{false};
  int64_t infer_workload_done_ms = 0;
  std::chrono::steady_clock::time_point set_cmd_time = std::chrono::steady_clock::now();
  std::vector<int64_t> req_us, done_us;
  int current_bs = 0;
  // task switch
  uint64_t last_reply_cmd_id = 0;
  int local_flag[2] = {0, 0};  // stand-in for the shared flags when there is no dist segment (one rank)

  int flag(int which, int set, int value) {
    int out = 0;
    if (dist) { srt_dist_switch_flag(dist, which, set, value, &out); return out; }
    if (set) local_flag[which] = value ? 1 : 0;
    return local_flag[which];
  }
  void barrier() { if (dist && cfg.world_size > 1) srt_dist_barrier(dist, 30000); }

  // caller holds mu
  bool try_interrupt_done_locked(bool with_barrier) {
    if (cmd_id > last_reply_cmd_id) {
      const uint64_t id = cmd_id;
      last_reply_cmd_id = cmd_id;
      cmd_id = 0;
      request_abort(0);
      if (with_barrier) barrier();
      if (cfg.rank == 0 && comm) put(id, SRT_EV_INTERRUPT_TRAIN_DONE, 0);
      return true;
    }
    return false;
  }

  void process_switch(const srt_ctrl_msg& msg) {
    std::unique_lock<std::mutex> lk(mu);
    SRT_LOG(LOG_CONTROL_STUB, "[SwitchStub] rank %d receives event %d (cmd_id %llu, value %d)", cfg.rank, msg.event,
            (unsigned long long)msg.id, msg.value);
    switch (msg.event) {
      case SRT_EV_INTERRUPT_TRAIN:
        if (cmd.load() == SRT_EV_INTERRUPT_TRAIN && cmd_id == 0) {
          // already interrupted and answered: the memory is free, reply at once
          last_reply_cmd_id = msg.id;
          if (cfg.rank == 0 && comm) put(msg.id, SRT_EV_INTERRUPT_TRAIN_DONE, 0);
          SRT_LOG(LOG_CONTROL_STUB, "[SwitchStub] already interrupted: InterruptTrainDone for cmd_id %llu sent at once",
                  (unsigned long long)msg.id);
        } else {
          if (cfg.rank == 0) { flag(0, 1, 1); flag(1, 1, 0); }
          if (cfg.kill_batch_on_recv && has_killed_batch_recover.load(std::memory_order_acquire)) {
            std::unique_lock<std::mutex> step_lock(step_mu);  // never inside the optimizer step
            request_abort(1);
            has_killed_batch_recover = false;
            SRT_LOG(LOG_CONTROL_STUB, "[SwitchStub] kill batch on InterruptTrain, cmd_id %llu", (unsigned long long)msg.id);
          }
          cmd_id = msg.id;
          cmd.store(SRT_EV_INTERRUPT_TRAIN);
          set_cmd_time = std::chrono::steady_clock::now();
          std::lock_guard<std::mutex> pl(prof_mu);
          req_us.push_back(unix_us());
        }
        break;
      case SRT_EV_RESUME_TRAIN:
        if (cmd.load() == SRT_EV_INTERRUPT_TRAIN && cmd_id == 0) {
          cmd.store(SRT_EV_RESUME_TRAIN);
          flag(0, 1, 0);
        }  // otherwise ignored, as in the reference: the interrupt has not been answered yet
        break;
      case SRT_EV_INFERENCE_WORKLOAD_DONE:
        infer_workload_done_ms = unix_us() / 1000;
        break;
      default:
        set_error("SwitchStub: unknown command %d", msg.event);
        break;
    }
  }

  void put(uint64_t id, int event, int value) {
    srt_ctrl_msg m = {id, event, value};
    srt_comm_put(comm, &m, SRT_TRA2INF, cfg.rank);
  }

  void process(const srt_ctrl_msg& msg) {
    if (cfg.task_switch) return process_switch(msg);
    std::unique_lock<std::mutex> lk(mu);
    SRT_LOG(LOG_CONTROL_STUB, "[ColocateStub] rank %d receives event %d (cmd_id %llu, value %d)", cfg.rank, msg.event,
            (unsigned long long)msg.id, msg.value);
    switch (msg.event) {
      case SRT_EV_COLOCATE_ADJUST_L1:
      case SRT_EV_COLOCATE_ADJUST_L2: {
        const bool should_kill = cfg.kill_batch_on_recv && msg.event == SRT_EV_COLOCATE_ADJUST_L1 &&
                                 cmd.load() != SRT_EV_COLOCATE_ADJUST_L1;
        if (should_kill && !has_killed_batch_recover.load(std::memory_order_acquire)) {
          // the previous killed batch has not been recovered yet: memory is already released
          put(msg.id, msg.event == SRT_EV_COLOCATE_ADJUST_L1 ? SRT_EV_COLOCATE_ADJUST_L1_DONE
                                                             : SRT_EV_COLOCATE_ADJUST_L2_DONE, 0);
          SRT_LOG(LOG_CONTROL_STUB, "[ColocateStub] killed batch not recovered yet: adjust cmd_id %llu answered at once",
                  (unsigned long long)msg.id);
          break;
        }
        has_killed_batch_recover = false;
        will_killed_batch_reconfig = true;
        if (should_kill) {
          std::unique_lock<std::mutex> step_lock(step_mu);  // never inside the optimizer step
          request_abort(1);
          SRT_LOG(LOG_CONTROL_STUB, "[ColocateStub] kill batch on adjust L1, cmd_id %llu, target batch size %d",
                  (unsigned long long)msg.id, msg.value);
        }
        cmd.store(msg.event);
        cmd_id = msg.id;
        set_cmd_time = std::chrono::steady_clock::now();
        std::lock_guard<std::mutex> pl(prof_mu);
        req_us.push_back(unix_us());
      } break;
      case SRT_EV_INFER_EXIT: {
        if (cfg.rank != 0) break;
        if (cfg.is_colocate_l1 && will_killed_batch_reconfig.load(std::memory_order_acquire)) {
          SRT_LOG(LOG_CONTROL_STUB, "[ColocateStub] InferExit: the killed batch is still being reconfigured, no redistribution");
          break;
        }
        bool all_same = true;
        for (int i = 0; i < cfg.world_size; ++i) {
          int t = 0, u = 0;
          if (srt_comm_get_train_field(comm, i, SRT_TI_TARGET_BS, &t) ||
              srt_comm_get_train_field(comm, i, SRT_TI_TARGET_BS_UNPUBLISHED, &u) || t != u) {
            all_same = false;
            break;
          }
        }
        SRT_LOG(LOG_CONTROL_STUB, "[ColocateStub] InferExit: %s", all_same ? "targets already published" : "redistribute the batch");
        if (!all_same && dist) srt_dbd_distribute_batch(dist, comm, 1, 0, 0);
      } break;
      case SRT_EV_INFERENCE_WORKLOAD_DONE:
        infer_workload_done_ms = unix_us() / 1000;
        break;
      default:
        set_error("ColocateStub: unknown command %d", msg.event);  // the reference aborts here
        break;
    }
  }

  void loop() {
    const int poll = cfg.poll_ms > 0 ? cfg.poll_ms : 1000;
    while (running.load()) {
      srt_ctrl_msg msg;
      int got = 0;
      if (srt_comm_timed_get(comm, poll, SRT_INF2TRA, cfg.rank, &msg, &got) == SRT_OK && got) process(msg);
    }
  }
};

}  // namespace srt

using namespace srt;

extern "C" {

int srt_stub_create(srt_comm* comm, srt_step* step, srt_dist* dist, const srt_stub_config* cfg, srt_stub** out) {
  SRT_REQUIRE(cfg && out, "stub_create: null argument");
  SRT_REQUIRE(cfg->rank >= 0 && cfg->rank < cfg->world_size && cfg->world_size <= SRT_MAX_DEVICE_NUM,
              "stub_create: bad rank/world");
  Stub* s = new Stub();
  s->comm = comm;
  s->step = step;
  s->dist = dist;
  s->cfg = *cfg;
  if (comm) {
    s->running = true;
    s->th = std::thread([s] { s->loop(); });
  }
  *out = (srt_stub*)s;
  return SRT_OK;
}

int srt_stub_stop(srt_stub* h) {
  Stub* s = (Stub*)h;
  if (!s) return SRT_OK;
  if (s->running.exchange(false) && s->th.joinable()) s->th.join();
  delete s;
  return SRT_OK;
}

int srt_stub_cmd(srt_stub* h) { return h ? ((Stub*)h)->cmd.load() : -1; }
uint64_t srt_stub_cmd_id(srt_stub* h) {
  Stub* s = (Stub*)h;
  if (!s) return 0;
  std::lock_guard<std::mutex> lk(s->mu);
  return s->cmd_id;
}
int srt_stub_set_cmd(srt_stub* h, int cmd) {
  Stub* s = (Stub*)h;
  SRT_REQUIRE(s, "stub: null handle");
  std::lock_guard<std::mutex> lk(s->mu);
  s->cmd.store(cmd);
  return SRT_OK;
}

int srt_stub_train_start(srt_stub* h) {
  Stub* s = (Stub*)h;
  SRT_REQUIRE(s, "stub: null handle");
  if (s->comm && s->cfg.rank == 0) s->put(0, SRT_EV_TRAIN_START, 0);
  return SRT_OK;
}
int srt_stub_train_end(srt_stub* h) {
  Stub* s = (Stub*)h;
  SRT_REQUIRE(s, "stub: null handle");
  if (s->comm && s->cfg.rank == 0) s->put(0, SRT_EV_TRAIN_END, 0);
  return SRT_OK;
}
int srt_stub_report_batch_size(srt_stub* h, int batch_size) {
  Stub* s = (Stub*)h;
  SRT_REQUIRE(s, "stub: null handle");
  s->current_bs = batch_size;
  if (s->comm) s->put(0, SRT_EV_REPORT_BATCH_SIZE, batch_size);
  return SRT_OK;
}
int srt_stub_set_abort_target(srt_stub* h, int (*fn)(void*, int), void* arg) {
  Stub* s = (Stub*)h;
  SRT_REQUIRE(s, "stub_set_abort_target: null handle");
  s->abort_fn = fn;
  s->abort_arg = arg;
  return SRT_OK;
}

int srt_stub_steps_no_interrupt_begin(srt_stub* h) {
  Stub* s = (Stub*)h;
  SRT_REQUIRE(s, "stub: null handle");
  s->step_mu.lock();
  s->exec_step = true;
  return SRT_OK;
}
int srt_stub_steps_no_interrupt_end(srt_stub* h) {
  Stub* s = (Stub*)h;
  SRT_REQUIRE(s, "stub: null handle");
  s->exec_step = false;
  s->step_mu.unlock();
  return SRT_OK;
}

static int adjust_done(Stub* s, int want_cmd, int done_event) {
  std::lock_guard<std::mutex> lk(s->mu);
  if (s->cmd.load() != want_cmd) return SRT_OK;
  if (s->comm) s->put(s->cmd_id, done_event, 0);
  SRT_LOG(LOG_CONTROL_STUB, "[ColocateStub] rank %d replies event %d for cmd_id %llu", s->cfg.rank, done_event,
          (unsigned long long)s->cmd_id);
  s->cmd.store(-1);
  s->cmd_id = 0;
  if (want_cmd == SRT_EV_COLOCATE_ADJUST_L1) s->request_abort(0);
  std::lock_guard<std::mutex> pl(s->prof_mu);
  s->done_us.push_back(unix_us());
  return SRT_OK;
}
int srt_stub_adjust_l1_done(srt_stub* h) {
  SRT_REQUIRE(h, "stub: null handle");
  return adjust_done((Stub*)h, SRT_EV_COLOCATE_ADJUST_L1, SRT_EV_COLOCATE_ADJUST_L1_DONE);
}
int srt_stub_adjust_l2_done(srt_stub* h) {
  SRT_REQUIRE(h, "stub: null handle");
  return adjust_done((Stub*)h, SRT_EV_COLOCATE_ADJUST_L2, SRT_EV_COLOCATE_ADJUST_L2_DONE);
}

int srt_stub_target_batch_size(srt_stub* h, int unpublished, int* out) {
  Stub* s = (Stub*)h;
  SRT_REQUIRE(s && out, "stub: null argument");
  std::lock_guard<std::mutex> lk(s->mu);
  if (!s->comm) { *out = s->cfg.input_batch_size; return SRT_OK; }
  return srt_comm_get_train_field(s->comm, s->cfg.rank, unpublished ? SRT_TI_TARGET_BS_UNPUBLISHED : SRT_TI_TARGET_BS,
                                  out);
}
int srt_stub_set_killed_batch_recover(srt_stub* h) {
  Stub* s = (Stub*)h;
  SRT_REQUIRE(s, "stub: null handle");
  s->has_killed_batch_recover.store(true, std::memory_order_release);
  return SRT_OK;
}

// ColocateStub::SetKilledBatchReconfiged (control_stub.h:114-116): rank 0 calls it once the remaining samples of
// the killed global batch have been redistributed. Until then a kInferExit must not redistribute concurrently
// (control_stub.cc:544), which is why this flag is separate from the "may be killed again" flag above.
int srt_stub_set_killed_batch_reconfiged(srt_stub* h) {
  Stub* s = (Stub*)h;
  SRT_REQUIRE(s, "stub: null handle");
  s->will_killed_batch_reconfig.store(false, std::memory_order_release);
  return SRT_OK;
}
int srt_stub_set_train_first_epoch_done(srt_stub* h) {
  Stub* s = (Stub*)h;
  SRT_REQUIRE(s, "stub: null handle");
  if (s->comm) return srt_comm_update_train_field(s->comm, s->cfg.rank, SRT_TI_FIRST_EPOCH_DONE, 1);
  return SRT_OK;
}
int srt_stub_can_exit_after_infer_workload_done(srt_stub* h) {
  Stub* s = (Stub*)h;
  if (!s) return 0;
  std::lock_guard<std::mutex> lk(s->mu);
  if (s->infer_workload_done_ms == 0) return 0;
  return unix_us() / 1000 - s->infer_workload_done_ms > 30 * 1000 ? 1 : 0;
}
int srt_stub_try_interrupt_train_done(srt_stub* h, int barrier, int* done) {
  Stub* s = (Stub*)h;
  SRT_REQUIRE(s, "stub: null handle");
  std::unique_lock<std::mutex> lk(s->mu);
  const bool ok = s->try_interrupt_done_locked(barrier != 0);
  if (ok) {
    std::lock_guard<std::mutex> pl(s->prof_mu);
    s->done_us.push_back(unix_us());
  }
  if (done) *done = ok ? 1 : 0;
  return SRT_OK;
}

// PrepareResume (control_stub.cc:339-392): every rank calls it in the same loop iteration.
int srt_stub_prepare_resume(srt_stub* h, int* resumed) {
  Stub* s = (Stub*)h;
  SRT_REQUIRE(s && resumed, "stub: null argument");
  std::unique_lock<std::mutex> lk(s->mu);
  if (s->cmd.load() == SRT_EV_INTERRUPT_TRAIN && s->cmd_id != 0) s->flag(0, 1, 1);  // a new interrupt came in
  s->barrier();
  const bool resume = s->flag(0, 0, 0) == 0;  // cleared by the master when kResumeTrain arrived
  s->barrier();
  if (!resume) {
    s->try_interrupt_done_locked(false);
    s->barrier();
    *resumed = 0;
    return SRT_OK;
  }
  s->cmd.store(SRT_EV_RESUME_TRAIN);
  s->has_killed_batch_recover = true;
  s->barrier();
  if (s->cfg.rank == 0 && s->comm) s->put(0, SRT_EV_RESUME_TRAIN_DONE, 0);
  *resumed = 1;
  return SRT_OK;
}

int srt_stub_switch_flag(srt_stub* h, int which, int set, int value, int* out) {
  Stub* s = (Stub*)h;
  SRT_REQUIRE(s && (which == 0 || which == 1), "stub_switch_flag: bad argument");
  const int v = s->flag(which, set, value);
  if (out) *out = v;
  return SRT_OK;
}

double srt_stub_passed_ms_from_set_cmd(srt_stub* h) {
  Stub* s = (Stub*)h;
  if (!s) return 0;
  std::lock_guard<std::mutex> lk(s->mu);
  return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - s->set_cmd_time).count();
}
int srt_stub_adjust_timestamps(srt_stub* h, int done, int64_t* out, int cap) {
  Stub* s = (Stub*)h;
  if (!s) return 0;
  std::lock_guard<std::mutex> pl(s->prof_mu);
  const std::vector<int64_t>& v = done ? s->done_us : s->req_us;
  for (int i = 0; i < (int)v.size() && i < cap && out; ++i) out[i] = v[i];
  return (int)v.size();
}

}  // extern "C"
