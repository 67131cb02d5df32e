// SM-partition following for the step executors: between layers an executor asks which share of the SMs training
// may use right now and continues on the green-context stream of that share (see sm_partition.cu), so that every
// kernel launched from then on runs inside the partition. The share comes from the inference side's required-TPC
// counter on the information board (what the reference's pre-launch hook reads: common/sm_partition.cc:219-261)
// or, without a board, from the process-wide allowed-SM mask.
#pragma once
#include "../../include/sirius_runtime.h"
#include "common.cuh"

namespace srt {

struct PartitionFollower {
  bool on = false;
  int device = 0;
  cudaStream_t home_stream = nullptr, home_side = nullptr;  // the whole-device streams the executor was created with
  int cur_sms = 0;                                          // 0 = whole device
  cudaEvent_t switch_ev = nullptr;
  srt_comm* tpc_comm = nullptr;
  int tpc_device = 0, tpc_min_train = 1, tpc_max_train = 1 << 20;

  ~PartitionFollower() {
    if (switch_ev) cudaEventDestroy(switch_ev);
  }
  static int device_sm_count() {
    const int lim = sm_limit();
    set_sm_limit(0);
    const int n = sm_count();
    set_sm_limit(lim);
    return n;
  }
  // Moves `stream` (and its low-priority companion `side`, when the executor has one) to `want` / `want_side`,
  // ordered behind everything queued so far.
  int move(cudaStream_t& stream, cudaStream_t& side, cudaStream_t want, cudaStream_t want_side, int sms) {
    if (want == stream) return SRT_OK;
    if (!switch_ev) SRT_CHECK_CUDA(cudaEventCreateWithFlags(&switch_ev, cudaEventDisableTiming));
    SRT_CHECK_CUDA(cudaEventRecord(switch_ev, stream));
    SRT_CHECK_CUDA(cudaStreamWaitEvent(want, switch_ev, 0));
    if (side && want_side && want_side != side) {
      SRT_CHECK_CUDA(cudaEventRecord(switch_ev, side));
      SRT_CHECK_CUDA(cudaStreamWaitEvent(want_side, switch_ev, 0));
      side = want_side;
    }
    stream = want;
    cur_sms = sms;
    return SRT_OK;
  }
  // Called between layers. Also sets the calling thread's grid-sizing limit to the partition's width.
  int follow(cudaStream_t& stream, cudaStream_t& side) {
    if (!on) return SRT_OK;
    const int total = device_sm_count();
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
    int rc = partition_streams(device, allowed, &want, &want_side, &sms);
    if (rc) return rc;
    if (!want) { want = home_stream; want_side = home_side; sms = 0; }
    rc = move(stream, side, want, want_side, sms);
    set_sm_limit(cur_sms);
    return rc;
  }
  // comm == nullptr turns following off and brings the executor back to its own streams.
  int configure(cudaStream_t& stream, cudaStream_t& side, srt_comm* comm, int dev, int min_train_tpc, int max_train_tpc,
                bool enable) {
    if (!home_stream) { home_stream = stream; home_side = side; }
    if (!enable) {
      on = false;
      tpc_comm = nullptr;
      return move(stream, side, home_stream, home_side, 0);
    }
    cudaStream_t st;
    int sms;
    int rc = partition_stream(device, 1 << 30, &st, &sms);  // builds the ladder; fails where green contexts are missing
    if (rc) return rc;
    tpc_comm = comm;
    tpc_device = dev;
    tpc_min_train = min_train_tpc > 0 ? min_train_tpc : 1;
    tpc_max_train = max_train_tpc > 0 ? max_train_tpc : 1 << 20;
    on = true;
    return SRT_OK;
  }
  // RAII for an executor's entry points: the thread's grid-sizing limit follows the partition while they run.
  struct Scope {
    int saved;
    explicit Scope(const PartitionFollower& f) : saved(sm_limit()) {
      if (f.on) set_sm_limit(f.cur_sms);
    }
    ~Scope() { set_sm_limit(saved); }
  };
};

}  // namespace srt
