// TrainAdjuster: turns "inference needs / releases this much memory" into per-rank target batch
// sizes with a linear memory model mem_MB = base + slope * batch_size.
//
// Follows server/train_adjuster.{h,cc} of the reference: PredictTargetBatchSize and
// GetDeltaBatchSize (:521-538), the require plan (:97-212), the release plan (:214-340), the
// imbalance check (:552-584) and the per-model constants (:642-698, hand-fit on V100/A100; callers
// on B200 pass their own base/slope, measured with srt_step_memory_bytes).
#include <math.h>
#include <stdlib.h>

#include <algorithm>
#include <limits>
#include <mutex>
#include <string>
#include <vector>

#include "../../../include/sirius_runtime.h"
#include "rt_common.h"

namespace srt {

struct Adjuster {
  srt_comm* comm = nullptr;
  srt_adjuster_config cfg;
  std::mutex mu;
  int cached_world = 0;
  int cached_target[SRT_MAX_DEVICE_NUM];
  double base = 0, slope = 1;
  bool have_param = false;

  int delta_bs(double mem_mb) const { return (int)std::ceil(mem_mb / slope); }
  double predict_mem(int bs) const { return bs <= 0 ? base : base + slope * bs; }
  int predict_target_bs(double mem_mb, int max_bs) const {
    int r = (int)((mem_mb - base) / slope);
    r = std::min(r, max_bs);
    return std::max(r, 0);
  }
  bool imbalance(int proposed_bs, const double* avail_minus_reserve) const {
    if (!cfg.enable_balance || !avail_minus_reserve) return false;
    double worst = 0;
    for (int r = 0; r < cached_world; ++r)
      worst = std::max(worst, std::max(0.0, avail_minus_reserve[r] - predict_mem(proposed_bs)));
    return worst > cfg.balance_threshold_mb;
  }
  int ensure_param() {
    if (have_param) return SRT_OK;
    if (cfg.slope_mb > 0) { base = cfg.base_mb; slope = cfg.slope_mb; have_param = true; return SRT_OK; }
    srt_train_info ti;
    int rc = srt_comm_get_train_info(comm, 0, &ti);
    if (rc) return rc;
    SRT_REQUIRE(ti.train_pid != -1, "train adjuster: train info of rank 0 is not valid");
    // the trainer is one of this library's executors unless told otherwise: use the line measured for it
    const char* fit = getenv("SIRIUS_B200_ADJUSTER_FIT");
    rc = (fit && std::string(fit) == "reference") ? srt_adjuster_model_mem_param(ti.model_name, &base, &slope)
                                                  : srt_adjuster_model_mem_param_measured(ti.model_name, &base, &slope);
    if (rc) return rc;
    have_param = true;
    return SRT_OK;
  }
  int publish(const int* plan) {  // UpdateCachedTrainInfoByAdjustPlan
    for (int r = 0; r < cached_world; ++r) {
      cached_target[r] = plan[r];
      int rc = srt_comm_update_train_field(comm, r, SRT_TI_TARGET_BS_UNPUBLISHED, plan[r]);
      if (rc) return rc;
    }
    return SRT_OK;
  }
};

}  // namespace srt

using namespace srt;

extern "C" {

int srt_adjuster_model_mem_param(const char* model_name, double* base_mb, double* slope_mb) {
  SRT_REQUIRE(model_name && base_mb && slope_mb, "model_mem_param: null argument");
  static const struct { const char* name; double base, slope; } kTable[] = {
      {"resnet152", 1150, 85}, {"swin_b", 1700, 145}, {"swin_b_ddp", 2560, 140}, {"gpt2", 2700, 490},
      {"qwen", 9000, 600}};
  for (const auto& e : kTable)
    if (std::string(model_name) == e.name) { *base_mb = e.base; *slope_mb = e.slope; return SRT_OK; }
  set_error("train adjuster: unsupported model '%s'", model_name);
  return SRT_ERR_UNSUPPORTED;
}

// The same line for this library's bf16 executors on a B200, measured with `python -m sirius_b200.mem_model`
// (device memory taken by the executor at two batch sizes; resnet152 at 224x224, gpt2 at 1024 tokens, qwen = the
// 0.5B shape at 2048 tokens). The swin_b_ddp entry adds the gradient buckets' bf16 wire buffer to swin_b.
int srt_adjuster_model_mem_param_measured(const char* model_name, double* base_mb, double* slope_mb) {
  SRT_REQUIRE(model_name && base_mb && slope_mb, "model_mem_param_measured: null argument");
  static const struct { const char* name; double base, slope; } kTable[] = {
      {"resnet152", 1475, 103}, {"swin_b", 1920, 143}, {"swin_b_ddp", 2090, 143}, {"gpt2", 3000, 737},
      {"qwen", 11530, 5453}};
  for (const auto& e : kTable)
    if (std::string(model_name) == e.name) { *base_mb = e.base; *slope_mb = e.slope; return SRT_OK; }
  set_error("train adjuster: no measured memory line for model '%s'", model_name);
  return SRT_ERR_UNSUPPORTED;
}

int srt_adjuster_create(srt_comm* comm, const srt_adjuster_config* cfg, srt_adjuster** out) {
  SRT_REQUIRE(comm && cfg && out, "adjuster_create: null argument");
  Adjuster* a = new Adjuster();
  a->comm = comm;
  a->cfg = *cfg;
  for (int& v : a->cached_target) v = std::numeric_limits<int>::min();
  *out = (srt_adjuster*)a;
  return SRT_OK;
}

int srt_adjuster_destroy(srt_adjuster* h) {
  delete (Adjuster*)h;
  return SRT_OK;
}

int srt_adjuster_load_train_info(srt_adjuster* h) {
  Adjuster* a = (Adjuster*)h;
  SRT_REQUIRE(a, "adjuster: null handle");
  std::lock_guard<std::mutex> lk(a->mu);
  a->cached_world = srt_comm_world_size(a->comm);
  SRT_REQUIRE(a->cached_world > 0, "adjuster: no trainer registered");
  for (int r = 0; r < a->cached_world; ++r) {
    int rc = srt_comm_get_train_field(a->comm, r, SRT_TI_TARGET_BS, &a->cached_target[r]);
    if (rc) return rc;
  }
  a->have_param = false;
  return a->ensure_param();
}

int srt_adjuster_reset_train_info(srt_adjuster* h) {
  Adjuster* a = (Adjuster*)h;
  SRT_REQUIRE(a, "adjuster: null handle");
  std::lock_guard<std::mutex> lk(a->mu);
  a->cached_world = 0;
  for (int& v : a->cached_target) v = std::numeric_limits<int>::min();
  return SRT_OK;
}

int srt_adjuster_predict_train_mem_mb(srt_adjuster* h, int batch_size, double* mem_mb) {
  Adjuster* a = (Adjuster*)h;
  SRT_REQUIRE(a && mem_mb, "adjuster: null argument");
  std::lock_guard<std::mutex> lk(a->mu);
  int rc = a->ensure_param();
  if (rc) return rc;
  *mem_mb = a->predict_mem(batch_size);
  return SRT_OK;
}

int srt_adjuster_infer_require_plan(srt_adjuster* h, int device_id, double required_mem_mb,
                                    const double* avail_minus_reserve, int* plan_bs, int* n) {
  Adjuster* a = (Adjuster*)h;
  SRT_REQUIRE(a && plan_bs && n, "adjuster: null argument");
  std::lock_guard<std::mutex> lk(a->mu);
  SRT_REQUIRE(a->cached_world > 0 && device_id >= 0 && device_id < a->cached_world,
              "adjuster: train info not loaded or bad device %d", device_id);
  int rc = a->ensure_param();
  if (rc) return rc;
  *n = 0;
  const int world = a->cached_world;
  const int cur = a->cached_target[device_id];
  const int min_bs = a->cfg.batch_size_limit;
  if (cur <= min_bs) return SRT_OK;
  if (required_mem_mb <= 0) return SRT_OK;
  int target = cur - a->delta_bs(required_mem_mb);
  if (a->cfg.num_visible_gpu > 1) target = std::max(target, min_bs);
  bool all_same = true;
  for (int r = 0; r < world; ++r)
    if (a->cached_target[r] != cur) all_same = false;
  auto fill_same = [&](int bs) { for (int r = 0; r < world; ++r) plan_bs[r] = bs; };
  auto fill_one = [&](int bs) { for (int r = 0; r < world; ++r) plan_bs[r] = r == device_id ? bs : a->cached_target[r]; };
  if (all_same) {
    // target > 0: never leave only part of the workers executing
    if (target > 0 && a->imbalance(target, avail_minus_reserve)) fill_one(target);
    else fill_same(target);
  } else {
    int mn = std::numeric_limits<int>::max();
    for (int r = 0; r < world; ++r) mn = std::min(mn, r == device_id ? target : a->cached_target[r]);
    if (mn > 0 && a->imbalance(mn, avail_minus_reserve)) fill_one(mn);
    else fill_same(target);
  }
  *n = world;
  return a->publish(plan_bs);
}

int srt_adjuster_infer_release_plan(srt_adjuster* h, const double* train_avail_mb, const double* free_mb,
                                    const double* reserve_mb, int* plan_bs, int* n) {
  Adjuster* a = (Adjuster*)h;
  SRT_REQUIRE(a && train_avail_mb && free_mb && reserve_mb && plan_bs && n, "adjuster: null argument");
  std::lock_guard<std::mutex> lk(a->mu);
  SRT_REQUIRE(a->cached_world > 0, "adjuster: train info not loaded");
  int rc = a->ensure_param();
  if (rc) return rc;
  const int world = a->cached_world;
  int init_bs = 0;
  rc = srt_comm_get_train_field(a->comm, 0, SRT_TI_INIT_BS, &init_bs);
  if (rc) return rc;
  std::vector<int> target(world);
  std::vector<double> avail_minus_reserve(world);
  for (int r = 0; r < world; ++r) {
    const double avail = std::max(train_avail_mb[r], 0.0), fre = std::max(free_mb[r], 0.0);
    const int cur = a->cached_target[r];
    avail_minus_reserve[r] = std::max(avail - reserve_mb[r], 0.0);
    if (a->cfg.use_shared_tensor) {
      const int by_avail = a->predict_target_bs(std::max(avail - reserve_mb[r], 0.0), init_bs);
      const int by_delta = cur + a->delta_bs(std::max(fre - reserve_mb[r], 0.0));
      target[r] = std::max(cur, std::min(by_avail, by_delta));
    } else {
      target[r] = std::max(cur, cur + a->delta_bs(fre));
    }
  }
  const int mn = *std::min_element(target.begin(), target.end());
  if (mn <= 0 || !a->imbalance(mn, avail_minus_reserve.data())) {
    for (int r = 0; r < world; ++r) plan_bs[r] = mn;
  } else {
    for (int r = 0; r < world; ++r) plan_bs[r] = target[r];
  }
  *n = world;
  return a->publish(plan_bs);
}

// TrainAdjuster::PredictTrainMemUsageMB (train_adjuster.cc:55-83): what the trainer on `device_id` will use once
// it runs at the target batch size the server has planned for it.
int srt_adjuster_predict_train_mem_usage_mb(srt_adjuster* h, int device_id, double* mem_mb) {
  Adjuster* a = (Adjuster*)h;
  SRT_REQUIRE(a && mem_mb, "adjuster: null argument");
  std::lock_guard<std::mutex> lk(a->mu);
  *mem_mb = 0.0;
  if (a->cached_world <= 0 || device_id < 0 || device_id >= a->cached_world) return SRT_OK;  // no trainer: no usage
  int rc = a->ensure_param();
  if (rc) return rc;
  const int bs = a->cached_target[device_id];
  *mem_mb = bs == std::numeric_limits<int>::min() ? 0.0 : a->predict_mem(bs);
  return SRT_OK;
}

// TrainAdjuster::GetLLMInferRequireMemAdjustPlan (train_adjuster.cc:436-520): the KV-cache pool needs
// required_mem_mb more; train_avail_mem_mb is what training could still use afterwards (free pages + its own
// pages - margin - the requirement), computed by the caller from the pool.
int srt_adjuster_llm_require_plan(srt_adjuster* h, int device_id, double required_mem_mb, double train_avail_mem_mb,
                                  const double* avail_minus_reserve, int* plan_bs, int* n) {
  Adjuster* a = (Adjuster*)h;
  SRT_REQUIRE(a && plan_bs && n, "adjuster: null argument");
  std::lock_guard<std::mutex> lk(a->mu);
  *n = 0;
  if (a->cached_world <= 0) return SRT_OK;  // no trainer to adjust
  SRT_REQUIRE(device_id >= 0 && device_id < a->cached_world, "adjuster: bad device %d", device_id);
  int rc = a->ensure_param();
  if (rc) return rc;
  const int world = a->cached_world, cur = a->cached_target[device_id];
  if (cur <= 0 || required_mem_mb <= 0) return SRT_OK;
  int init_bs = 0;
  rc = srt_comm_get_train_field(a->comm, 0, SRT_TI_INIT_BS, &init_bs);
  if (rc) return rc;
  const int by_avail = a->predict_target_bs(std::max(train_avail_mem_mb, 0.0), init_bs);
  const int by_required = cur - a->delta_bs(required_mem_mb);
  const int target = std::max(0, std::min(by_avail, by_required));
  for (int r = 0; r < world; ++r)
    SRT_REQUIRE(a->cached_target[r] == cur, "adjuster: ranks with different target batch sizes are not supported "
                "by the LLM require plan (as in the reference)");
  if (target > 0 && a->imbalance(target, avail_minus_reserve))
    for (int r = 0; r < world; ++r) plan_bs[r] = r == device_id ? target : a->cached_target[r];
  else
    for (int r = 0; r < world; ++r) plan_bs[r] = target;
  *n = world;
  return a->publish(plan_bs);
}

// TrainAdjuster::GetLLMInferReleaseMemAdjustPlan (train_adjuster.cc:343-434): the KV-cache pool gave pages back.
int srt_adjuster_llm_release_plan(srt_adjuster* h, const double* train_avail_mb, const double* free_mb, int* plan_bs,
                                  int* n) {
  Adjuster* a = (Adjuster*)h;
  SRT_REQUIRE(a && train_avail_mb && free_mb && plan_bs && n, "adjuster: null argument");
  std::lock_guard<std::mutex> lk(a->mu);
  *n = 0;
  if (a->cached_world <= 0) return SRT_OK;
  int rc = a->ensure_param();
  if (rc) return rc;
  const int world = a->cached_world;
  int init_bs = 0;
  rc = srt_comm_get_train_field(a->comm, 0, SRT_TI_INIT_BS, &init_bs);
  if (rc) return rc;
  std::vector<int> target(world);
  std::vector<double> avail(world);
  for (int r = 0; r < world; ++r) {
    const int cur = a->cached_target[r];
    avail[r] = std::max(train_avail_mb[r], 0.0);
    const int by_avail = a->predict_target_bs(avail[r], init_bs);
    const int by_delta = cur + a->delta_bs(std::max(free_mb[r], 0.0));
    target[r] = std::max(cur, std::min(by_avail, by_delta));
  }
  const int mn = *std::min_element(target.begin(), target.end());
  if (mn <= 0 || !a->imbalance(mn, avail.data())) {
    for (int r = 0; r < world; ++r) plan_bs[r] = mn;
  } else {
    for (int r = 0; r < world; ++r) plan_bs[r] = target[r];
  }
  *n = world;
  return a->publish(plan_bs);
}

}  // extern "C"
