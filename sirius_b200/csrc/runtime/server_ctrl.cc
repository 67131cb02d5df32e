// Server side of the colocation protocol: Controller, ResourceManager, ColdModelCache, TrainLauncher and
// KVCachePool behind a C ABI (include/sirius_server.h). Written from the behaviour of the reference's classes
// (server/control/controller.cc:84-445, server/resource_manager.cc:22-104, server/model_store/model_cache.cc:209-500,
// server/train_launcher.cc:88-311, server/llm/kv_cache_pool.cc:232-347): same messages, same decisions, same
// environment contract; errors are statuses instead of CHECK/LOG(FATAL), waits take time limits.
#include <fcntl.h>
#include <math.h>
#include <signal.h>
#include <string.h>
#include <sys/wait.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <map>
#include <mutex>
#include <random>
#include <sstream>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "../../../include/sirius_server.h"
#include "rt_common.h"

namespace srt {
namespace {

constexpr double kMB = 1024.0 * 1024.0;

template <typename Pred>
bool wait_for(std::condition_variable& cv, std::unique_lock<std::mutex>& lk, int timeout_ms, Pred pred) {
  if (timeout_ms < 0) { cv.wait(lk, pred); return true; }
  return cv.wait_for(lk, std::chrono::milliseconds(timeout_ms), pred);
}

}  // namespace

// ---------------------------------------------------------------------------------------------------------
struct Controller {
  srt_comm* comm = nullptr;
  srt_adjuster* adjuster = nullptr;
  srt_controller_config cfg{};
  int world = 1;
  std::thread monitor;
  std::atomic<bool> stop{false};

  std::mutex mu;  // status, done ids, flags
  std::condition_variable cv_train, cv_switch, cv_adjust, cv_infer;
  int train_status = SRT_TRAIN_IDLE;
  bool infer_running = false;
  uint64_t task_switch_done_id = 0;
  bool resumed_since_last_interrupt = true;
  uint64_t adjust_done_ids[SRT_MAX_DEVICE_NUM] = {0};
  int cur_batch_size = 0;
  int train_pid = -1;

  std::atomic<uint64_t> adjust_cmd_id{1}, interrupt_cmd_id{1}, resume_cmd_id{1}, dummy_exit_id{1}, workload_done_id{1};

  // Controller::TrainMonitor
  void run() {
    while (!stop.load(std::memory_order_acquire)) {
      int rank = -1, got = 0;
      srt_ctrl_msg m{};
      if (srt_comm_timed_get_from_any(comm, 50, SRT_TRA2INF, &rank, &m, &got) != SRT_OK || !got) continue;
      bool reload = false;
      {
        std::lock_guard<std::mutex> lk(mu);
        const int last = train_status;
        switch (m.event) {
          case SRT_EV_TRAIN_START:
            train_status = SRT_TRAIN_RUNNING;
            reload = true;
            break;
          case SRT_EV_INTERRUPT_TRAIN_DONE:
            train_status = SRT_TRAIN_INTERRUPTED;
            task_switch_done_id = m.id;
            cv_switch.notify_all();
            break;
          case SRT_EV_RESUME_TRAIN_DONE:
            train_status = SRT_TRAIN_RUNNING;
            break;
          case SRT_EV_COLOCATE_ADJUST_L1_DONE:
          case SRT_EV_COLOCATE_ADJUST_L2_DONE:
            if (rank >= 0 && rank < SRT_MAX_DEVICE_NUM) adjust_done_ids[rank] = m.id;
            cv_adjust.notify_all();
            break;
          case SRT_EV_TRAIN_END:
            train_status = SRT_TRAIN_IDLE;
            srt_comm_clear(comm);
            // nobody is left to acknowledge: waiters see "training idle" and return
            cv_adjust.notify_all();
            cv_switch.notify_all();
            break;
          case SRT_EV_REPORT_BATCH_SIZE:
            cur_batch_size = m.value;
            break;
          default:
            break;
        }
        if (last == SRT_TRAIN_RUNNING && train_status != SRT_TRAIN_RUNNING) cv_train.notify_all();
      }
      if (reload && adjuster) srt_adjuster_load_train_info(adjuster);
    }
  }
  bool idle() {
    std::lock_guard<std::mutex> lk(mu);
    return train_status == SRT_TRAIN_IDLE;
  }
  int adjust_event() const { return cfg.serve_mode == SRT_SERVE_COLOCATE_L1 ? SRT_EV_COLOCATE_ADJUST_L1 : SRT_EV_COLOCATE_ADJUST_L2; }
  bool colocate_mode() const { return cfg.serve_mode == SRT_SERVE_COLOCATE_L1 || cfg.serve_mode == SRT_SERVE_COLOCATE_L2; }
};

// ---------------------------------------------------------------------------------------------------------
struct ColdCache {
  struct Item { double hotness; std::vector<int> cached_groups; size_t cached_nbytes; };
  srt_cold_cache_config cfg{};
  std::mutex mu;
  size_t cached = 0, capacity = 0;
  std::unordered_map<std::string, Item> items;

  bool pop(const std::string& name, bool to_inference, std::vector<int>* groups) {
    auto it = items.find(name);
    if (it == items.end()) return false;
    if (groups) *groups = it->second.cached_groups;
    cached -= it->second.cached_nbytes;
    if (to_inference) capacity -= std::min(capacity, it->second.cached_nbytes);
    items.erase(it);
    return true;
  }
};

// ---------------------------------------------------------------------------------------------------------
struct KvPool {
  srt_pool* pool = nullptr;
  Controller* ctl = nullptr;
  srt_adjuster* adjuster = nullptr;
  srt_kvpool_config cfg{};
  std::mutex mu;
  int64_t block_size = 0, num_layers = 0, num_heads = 0, head_size = 0;
  size_t block_nbytes = 0;
  bool shape_set = false;
  int64_t free_layer_blocks = -1, used_layer_blocks = -1;
  std::map<uint64_t, size_t> pages;  // device address -> bytes
  size_t page_bytes() const { return (size_t)srt_pool_stat(pool, SRT_POOL_STAT_PAGE_NBYTES); }
  int64_t num_gpu_blocks() const { return block_nbytes ? (int64_t)((size_t)srt_pool_stat(pool, SRT_POOL_STAT_POOL_NBYTES) / block_nbytes) : 0; }
};

}  // namespace srt

using namespace srt;

extern "C" {

// ---- Controller -----------------------------------------------------------------------------------------
int srt_controller_create(srt_comm* comm, srt_adjuster* adjuster, const srt_controller_config* cfg, srt_controller** out) {
  SRT_REQUIRE(comm && cfg && out, "controller_create: null argument");
  SRT_REQUIRE(cfg->serve_mode >= SRT_SERVE_NORMAL && cfg->serve_mode <= SRT_SERVE_COLOCATE_L2, "controller_create: unknown serve mode %d",
              cfg->serve_mode);
  Controller* c = new Controller();
  c->comm = comm;
  c->adjuster = adjuster;
  c->cfg = *cfg;
  c->world = srt_comm_world_size(comm);
  c->monitor = std::thread([c] { c->run(); });
  *out = (srt_controller*)c;
  return SRT_OK;
}

int srt_controller_destroy(srt_controller* h) {
  Controller* c = (Controller*)h;
  if (!c) return SRT_OK;
  c->stop.store(true, std::memory_order_release);
  if (c->monitor.joinable()) c->monitor.join();
  delete c;
  return SRT_OK;
}

int srt_controller_train_status(srt_controller* h, int* status) {
  Controller* c = (Controller*)h;
  SRT_REQUIRE(c && status, "controller: null argument");
  std::lock_guard<std::mutex> lk(c->mu);
  *status = c->train_status;
  return SRT_OK;
}

int srt_controller_cur_batch_size(srt_controller* h, int* bs) {
  Controller* c = (Controller*)h;
  SRT_REQUIRE(c && bs, "controller: null argument");
  std::lock_guard<std::mutex> lk(c->mu);
  *bs = c->cur_batch_size;
  return SRT_OK;
}

int srt_controller_set_train_pid(srt_controller* h, int pid) {
  Controller* c = (Controller*)h;
  SRT_REQUIRE(c, "controller: null handle");
  std::lock_guard<std::mutex> lk(c->mu);
  c->train_pid = pid;
  return SRT_OK;
}

int srt_controller_interrupt_train(srt_controller* h, uint64_t* cmd_id) {
  Controller* c = (Controller*)h;
  SRT_REQUIRE(c && cmd_id, "controller: null argument");
  *cmd_id = 0;
  if (c->cfg.serve_mode == SRT_SERVE_TASKSWITCH_L1) {
    std::lock_guard<std::mutex> lk(c->mu);
    // a second interrupt before the resume of the first would let training re-allocate under the request
    if (c->train_status == SRT_TRAIN_IDLE || !c->resumed_since_last_interrupt) return SRT_OK;
    const uint64_t id = c->interrupt_cmd_id.fetch_add(1, std::memory_order_relaxed);
    srt_ctrl_msg m{id, SRT_EV_INTERRUPT_TRAIN, 0};
    int rc = srt_comm_put_all(c->comm, &m, 1, SRT_INF2TRA);
    if (rc) return rc;
    c->resumed_since_last_interrupt = false;
    *cmd_id = id;
    return SRT_OK;
  }
  if (c->cfg.serve_mode == SRT_SERVE_TASKSWITCH_L3) {
    int pid;
    { std::lock_guard<std::mutex> lk(c->mu); pid = c->train_pid; }
    if (pid > 0) {
      c->interrupt_cmd_id.fetch_add(1, std::memory_order_relaxed);
      SRT_REQUIRE(kill(pid, SIGKILL) == 0, "controller: cannot kill the training process %d", pid);
    }
    return SRT_OK;
  }
  set_error("controller: InterruptTrain needs a task-switch serve mode (have %d)", c->cfg.serve_mode);
  return SRT_ERR_STATE;
}

int srt_controller_resume_train(srt_controller* h, uint64_t* cmd_id) {
  Controller* c = (Controller*)h;
  SRT_REQUIRE(c && cmd_id, "controller: null argument");
  *cmd_id = c->resume_cmd_id.fetch_add(1, std::memory_order_relaxed);
  std::lock_guard<std::mutex> lk(c->mu);
  if (c->train_status == SRT_TRAIN_IDLE) return SRT_OK;
  srt_ctrl_msg m{*cmd_id, SRT_EV_RESUME_TRAIN, 0};
  int rc = srt_comm_put(c->comm, &m, SRT_INF2TRA, 0);  // rank 0 releases the others (kTraRank_0)
  if (rc) return rc;
  c->resumed_since_last_interrupt = true;
  return SRT_OK;
}

int srt_controller_colocate_adjust(srt_controller* h, int device_id, int batch_size, uint64_t* cmd_id) {
  Controller* c = (Controller*)h;
  SRT_REQUIRE(c && cmd_id, "controller: null argument");
  (void)device_id;
  *cmd_id = c->adjust_cmd_id.fetch_add(1, std::memory_order_relaxed);
  if (c->idle()) return SRT_OK;
  // 1. an earlier plan that training has not published yet may already cover this request
  bool skip = true;
  int target0 = 0;
  for (int r = 0; r < c->world; ++r) {
    int t = 0, u = 0;
    int rc = srt_comm_get_train_field(c->comm, r, SRT_TI_TARGET_BS, &t);
    if (!rc) rc = srt_comm_get_train_field(c->comm, r, SRT_TI_TARGET_BS_UNPUBLISHED, &u);
    if (rc) return rc;
    if (r == 0) target0 = u;
    if (u < t) { skip = false; }
  }
  if (skip) { *cmd_id = 0; return SRT_OK; }
  // 2. every rank runs on with batch_size fewer samples
  srt_ctrl_msg m{*cmd_id, c->adjust_event(), std::max(0, target0 - batch_size)};
  return srt_comm_put_all(c->comm, &m, 1, SRT_INF2TRA);
}

static int put_plan(Controller* c, int event, const int* plan_bs, int n, uint64_t id) {
  SRT_REQUIRE(plan_bs && n == c->world, "controller: an adjust plan has one batch size per training rank (%d given, %d ranks)", n,
              c->world);
  std::vector<srt_ctrl_msg> msgs((size_t)n);
  for (int i = 0; i < n; ++i) msgs[(size_t)i] = srt_ctrl_msg{id, event, plan_bs[i]};
  return srt_comm_put_all(c->comm, msgs.data(), n, SRT_INF2TRA);
}

int srt_controller_infer_require_adjust(srt_controller* h, int device_id, const int* plan_bs, int n, uint64_t* cmd_id) {
  Controller* c = (Controller*)h;
  SRT_REQUIRE(c && cmd_id, "controller: null argument");
  (void)device_id;
  *cmd_id = c->adjust_cmd_id.fetch_add(1, std::memory_order_relaxed);
  if (c->idle()) return SRT_OK;
  return put_plan(c, c->adjust_event(), plan_bs, n, *cmd_id);
}

int srt_controller_infer_release_adjust(srt_controller* h, const int* plan_bs, int n, uint64_t* cmd_id) {
  Controller* c = (Controller*)h;
  SRT_REQUIRE(c && cmd_id, "controller: null argument");
  *cmd_id = c->adjust_cmd_id.fetch_add(1, std::memory_order_relaxed);
  if (c->idle() || !c->colocate_mode()) return SRT_OK;
  return put_plan(c, SRT_EV_INFER_EXIT, plan_bs, n, *cmd_id);
}

int srt_controller_dummy_infer_exit(srt_controller* h, int device_id, int target_batch_size, uint64_t* cmd_id) {
  Controller* c = (Controller*)h;
  SRT_REQUIRE(c && cmd_id, "controller: null argument");
  SRT_REQUIRE(c->cfg.dummy_adjust, "controller: DummyInferExit is for dummy-adjust runs only");
  (void)device_id;
  *cmd_id = c->dummy_exit_id.fetch_add(1, std::memory_order_relaxed);
  if (c->idle()) return SRT_OK;
  srt_ctrl_msg m{*cmd_id, SRT_EV_INFER_EXIT, target_batch_size};
  return srt_comm_put_all(c->comm, &m, 1, SRT_INF2TRA);
}

int srt_controller_inference_workload_done(srt_controller* h) {
  Controller* c = (Controller*)h;
  SRT_REQUIRE(c, "controller: null handle");
  const uint64_t id = c->workload_done_id.fetch_add(1, std::memory_order_relaxed);
  if (c->cfg.dummy_adjust) return SRT_OK;
  srt_ctrl_msg m{id, SRT_EV_INFERENCE_WORKLOAD_DONE, 0};
  return srt_comm_put_all(c->comm, &m, 1, SRT_INF2TRA);
}

int srt_controller_wait_train_not_running(srt_controller* h, int timeout_ms) {
  Controller* c = (Controller*)h;
  SRT_REQUIRE(c, "controller: null handle");
  std::unique_lock<std::mutex> lk(c->mu);
  if (wait_for(c->cv_train, lk, timeout_ms, [&] { return c->train_status != SRT_TRAIN_RUNNING; })) return SRT_OK;
  set_error("controller: training still running after %d ms", timeout_ms);
  return SRT_ERR_TIMEOUT;
}

int srt_controller_wait_task_switch_done(srt_controller* h, uint64_t cmd_id, int timeout_ms) {
  Controller* c = (Controller*)h;
  SRT_REQUIRE(c, "controller: null handle");
  std::unique_lock<std::mutex> lk(c->mu);
  if (wait_for(c->cv_switch, lk, timeout_ms,
               [&] { return c->train_status == SRT_TRAIN_IDLE || c->task_switch_done_id >= cmd_id; }))
    return SRT_OK;
  set_error("controller: interrupt %llu not acknowledged after %d ms", (unsigned long long)cmd_id, timeout_ms);
  return SRT_ERR_TIMEOUT;
}

int srt_controller_wait_colocate_adjust_done(srt_controller* h, int device_id, uint64_t cmd_id, int timeout_ms) {
  Controller* c = (Controller*)h;
  SRT_REQUIRE(c && device_id >= 0 && device_id < SRT_MAX_DEVICE_NUM, "controller: bad argument");
  if (!c->colocate_mode()) return SRT_OK;
  std::unique_lock<std::mutex> lk(c->mu);
  if (wait_for(c->cv_adjust, lk, timeout_ms,
               [&] { return c->train_status == SRT_TRAIN_IDLE || c->adjust_done_ids[device_id] >= cmd_id; }))
    return SRT_OK;
  set_error("controller: adjust %llu not acknowledged by rank %d after %d ms", (unsigned long long)cmd_id, device_id, timeout_ms);
  return SRT_ERR_TIMEOUT;
}

int srt_controller_set_infer_status(srt_controller* h, int running) {
  Controller* c = (Controller*)h;
  SRT_REQUIRE(c, "controller: null handle");
  std::lock_guard<std::mutex> lk(c->mu);
  c->infer_running = running != 0;
  if (!c->infer_running) c->cv_infer.notify_all();
  return SRT_OK;
}

int srt_controller_wait_infer_idle(srt_controller* h, int timeout_ms) {
  Controller* c = (Controller*)h;
  SRT_REQUIRE(c, "controller: null handle");
  std::unique_lock<std::mutex> lk(c->mu);
  if (wait_for(c->cv_infer, lk, timeout_ms, [&] { return !c->infer_running; })) return SRT_OK;
  set_error("controller: inference still running after %d ms", timeout_ms);
  return SRT_ERR_TIMEOUT;
}

int srt_controller_has_flying_colocate_adjust(srt_controller* h, int* flying) {
  Controller* c = (Controller*)h;
  SRT_REQUIRE(c && flying, "controller: null argument");
  std::lock_guard<std::mutex> lk(c->mu);
  *flying = 0;
  const uint64_t next = c->adjust_cmd_id.load(std::memory_order_relaxed);
  for (int r = 0; r < c->world && r < SRT_MAX_DEVICE_NUM; ++r)
    if (c->adjust_done_ids[r] + 1 < next) *flying = 1;
  return SRT_OK;
}

// ---- ResourceManager ------------------------------------------------------------------------------------
double srt_resmgr_infer_memory_mb(srt_pool* pool) { return pool ? (double)srt_pool_stat(pool, SRT_POOL_STAT_INFER_USAGE) / kMB : 0.0; }
double srt_resmgr_train_memory_mb(srt_pool* pool) { return pool ? (double)srt_pool_stat(pool, SRT_POOL_STAT_TRAIN_ALL) / kMB : 0.0; }

int srt_resmgr_free_memory_mb(srt_pool* pool, srt_adjuster* adjuster, int device_id, double over_predict_mb, double* out) {
  SRT_REQUIRE(pool && out, "resmgr: null argument");
  double predict = 0.0;
  if (adjuster) {
    int rc = srt_adjuster_predict_train_mem_usage_mb(adjuster, device_id, &predict);
    if (rc) return rc;
  }
  *out = (double)srt_pool_stat(pool, SRT_POOL_STAT_POOL_NBYTES) / kMB - srt_resmgr_infer_memory_mb(pool) -
         std::max(srt_resmgr_train_memory_mb(pool), predict) - over_predict_mb;
  return SRT_OK;
}

int srt_resmgr_train_avail_memory_mb(srt_pool* pool, double over_predict_mb, double* out) {
  SRT_REQUIRE(pool && out, "resmgr: null argument");
  *out = (double)srt_pool_stat(pool, SRT_POOL_STAT_POOL_NBYTES) / kMB - srt_resmgr_infer_memory_mb(pool) - over_predict_mb;
  return SRT_OK;
}

// ---- ColdModelCache -------------------------------------------------------------------------------------
int srt_cold_cache_create(const srt_cold_cache_config* cfg, srt_cold_cache** out) {
  SRT_REQUIRE(cfg && out && cfg->max_capacity_nbytes >= cfg->min_capacity_nbytes && cfg->ratio >= 0 && cfg->ratio <= 1,
              "cold_cache_create: bad configuration");
  ColdCache* c = new ColdCache();
  c->cfg = *cfg;
  c->capacity = cfg->min_capacity_nbytes;
  *out = (srt_cold_cache*)c;
  return SRT_OK;
}
int srt_cold_cache_destroy(srt_cold_cache* h) { delete (ColdCache*)h; return SRT_OK; }

int srt_cold_cache_push(srt_cold_cache* h, const char* name, double hotness, const size_t* groups_nbytes, int n_groups,
                        int* cached_groups, int cap, int* n_cached, char* evicted, size_t evicted_cap, int* ok) {
  ColdCache* c = (ColdCache*)h;
  SRT_REQUIRE(c && name && groups_nbytes && n_groups > 0 && cached_groups && n_cached && ok, "cold_cache_push: bad argument");
  std::lock_guard<std::mutex> lk(c->mu);
  *ok = 0;
  *n_cached = 0;
  if (evicted && evicted_cap) evicted[0] = 0;
  if (c->items.count(name)) return SRT_OK;
  size_t total = 0;
  for (int k = 0; k < n_groups; ++k) total += groups_nbytes[k];
  const size_t model_max = c->cfg.max_capacity_nbytes > 0 ? (size_t)((double)total * c->cfg.ratio) : 0;
  // 1. which groups stay cached: the first, then as long as half of the next still fits the model's share
  ColdCache::Item item;
  item.hotness = hotness;
  item.cached_nbytes = 0;
  for (int k = 0; k < n_groups; ++k) {
    if (model_max > 0 && (k == 0 || item.cached_nbytes + groups_nbytes[k] / 2 <= model_max)) {
      item.cached_groups.push_back(k);
      item.cached_nbytes += groups_nbytes[k];
    } else {
      break;
    }
  }
  SRT_REQUIRE((int)item.cached_groups.size() <= cap, "cold_cache_push: %zu cached groups, room for %d", item.cached_groups.size(), cap);
  // 2. room for them
  std::string evicted_names;
  if (c->capacity + total <= c->cfg.max_capacity_nbytes) {
    c->capacity += total;  // the whole model is reserved, cached in part or not
    c->cached += item.cached_nbytes;
  } else {
    const size_t evict_to = (c->cfg.max_capacity_nbytes + c->cfg.min_capacity_nbytes) / 2;
    SRT_REQUIRE(evict_to >= item.cached_nbytes, "cold_cache_push: %zu bytes of %s do not fit the cache's stable point %zu",
                item.cached_nbytes, name, evict_to);
    std::vector<std::pair<double, std::string>> order;  // coldest first
    for (auto& kv : c->items) order.emplace_back(kv.second.hotness, kv.first);
    std::sort(order.begin(), order.end());
    for (auto& e : order) {
      if (c->cached <= evict_to) break;
      c->pop(e.second, false, nullptr);
      evicted_names += (evicted_names.empty() ? "" : "\n") + e.second;
    }
    SRT_REQUIRE(c->cached <= evict_to, "cold_cache_push: cannot evict down to %zu bytes", evict_to);
    c->capacity = c->cached + item.cached_nbytes;
    c->cached += item.cached_nbytes;
  }
  for (size_t i = 0; i < item.cached_groups.size(); ++i) cached_groups[i] = item.cached_groups[i];
  *n_cached = (int)item.cached_groups.size();
  if (evicted && evicted_cap) {
    SRT_REQUIRE(evicted_names.size() < evicted_cap, "cold_cache_push: the evicted names need %zu bytes", evicted_names.size() + 1);
    memcpy(evicted, evicted_names.c_str(), evicted_names.size() + 1);
  }
  c->items.emplace(name, std::move(item));
  *ok = 1;
  return SRT_OK;
}

int srt_cold_cache_pop(srt_cold_cache* h, const char* name, int pop_to_inference, int* cached_groups, int cap, int* n_cached,
                       int* ok) {
  ColdCache* c = (ColdCache*)h;
  SRT_REQUIRE(c && name && ok, "cold_cache_pop: bad argument");
  std::lock_guard<std::mutex> lk(c->mu);
  std::vector<int> groups;
  *ok = c->pop(name, pop_to_inference != 0, &groups) ? 1 : 0;
  if (n_cached) *n_cached = (int)groups.size();
  if (cached_groups)
    for (size_t i = 0; i < groups.size() && (int)i < cap; ++i) cached_groups[i] = groups[i];
  return SRT_OK;
}

int srt_cold_cache_take_space(srt_cold_cache* h, size_t nbytes, int* ok) {
  ColdCache* c = (ColdCache*)h;
  SRT_REQUIRE(c && ok, "cold_cache_take_space: bad argument");
  std::lock_guard<std::mutex> lk(c->mu);
  *ok = c->cached + nbytes <= c->capacity ? 1 : 0;
  if (*ok) c->capacity -= nbytes;
  return SRT_OK;
}

int srt_cold_cache_set_capacity(srt_cold_cache* h, size_t nbytes) {
  ColdCache* c = (ColdCache*)h;
  SRT_REQUIRE(c, "cold_cache_set_capacity: null handle");
  std::lock_guard<std::mutex> lk(c->mu);
  SRT_REQUIRE(nbytes >= c->cached, "cold_cache_set_capacity: %zu bytes are cached, capacity %zu is less", c->cached, nbytes);
  c->capacity = nbytes;
  return SRT_OK;
}

int srt_cold_cache_info(srt_cold_cache* h, size_t* capacity_nbytes, size_t* cached_nbytes) {
  ColdCache* c = (ColdCache*)h;
  SRT_REQUIRE(c, "cold_cache_info: null handle");
  std::lock_guard<std::mutex> lk(c->mu);
  if (capacity_nbytes) *capacity_nbytes = c->capacity;
  if (cached_nbytes) *cached_nbytes = c->cached;
  return SRT_OK;
}

double srt_cold_cache_reserve_mb(srt_cold_cache* h) {
  ColdCache* c = (ColdCache*)h;
  if (!c) return 0.0;
  std::lock_guard<std::mutex> lk(c->mu);
  return std::max(0.0, ((double)c->capacity - (double)c->cached) / kMB);
}

double srt_cold_cache_releasable_mb(srt_cold_cache* h) {
  ColdCache* c = (ColdCache*)h;
  if (!c) return 0.0;
  std::lock_guard<std::mutex> lk(c->mu);
  return c->cached > c->cfg.min_capacity_nbytes ? (double)(c->cached - c->cfg.min_capacity_nbytes) / kMB : 0.0;
}

double srt_cold_cache_buffer_mb(srt_cold_cache* h, double free_memory_mb) {
  ColdCache* c = (ColdCache*)h;
  if (!c) return 0.0;
  std::lock_guard<std::mutex> lk(c->mu);
  double buffer = free_memory_mb;
  if (c->cached > c->cfg.min_capacity_nbytes) buffer += (double)(c->cached - c->cfg.min_capacity_nbytes) / kMB;
  const double cur_max = (double)(c->cfg.max_capacity_nbytes - std::min(c->cfg.min_capacity_nbytes, c->cached)) / kMB;
  return std::max(0.0, std::min(buffer, cur_max));
}

// ---- TrainLauncher --------------------------------------------------------------------------------------
static std::vector<std::pair<std::string, std::string>> launcher_env(const srt_launcher_config& g) {
  std::vector<std::pair<std::string, std::string>> e;
  e.emplace_back("COLTRAIN_USE_XSCHED", g.use_xsched ? "1" : "0");
  e.emplace_back("COLTRAIN_HAS_INFER_SERVER", "1");
  if (g.use_shared_tensor_train) {
    e.emplace_back("COLTRAIN_USE_SHARED_TENSOR", "1");
    e.emplace_back("COLTRAIN_HAS_SHARED_TENSOR_SERVER", "1");
    std::ostringstream gb;
    gb << g.cuda_memory_pool_gb;
    e.emplace_back("COLTRAIN_SHARED_TENSOR_POOL_GB", gb.str());
    e.emplace_back("SHARED_TENSOR_POOL_FREELIST_POLICY", g.freelist_policy ? g.freelist_policy : "best-fit");
  } else {
    e.emplace_back("COLTRAIN_USE_SHARED_TENSOR", "0");
  }
  const bool l1 = g.serve_mode == SRT_SERVE_COLOCATE_L1 || g.serve_mode == SRT_SERVE_TASKSWITCH_L1;
  e.emplace_back("COLTRAIN_HOOK_MODE", l1 ? (g.use_xsched ? "xsched-sync2" : "sync") : "none");
  static const char* kModes[] = {"normal", "taskswitch-l1", "taskswitch-l3", "colocate-l1", "colocate-l2"};
  e.emplace_back("COLTRAIN_MODE", kModes[g.serve_mode]);
  if (g.train_profile && *g.train_profile) e.emplace_back("COLTRAIN_PROFILE_LOG_PATH", g.train_profile);
  if (g.skip_set_mps_thread_percent) {
    if (g.dynamic_sm_partition) e.emplace_back("COLTRAIN_DYNAMIC_SM_PARTITION", "1");
  } else if (g.train_mps_thread_percent >= 0 && g.train_mps_thread_percent <= 100) {
    e.emplace_back("CUDA_MPS_ACTIVE_THREAD_PERCENTAGE", std::to_string(g.train_mps_thread_percent));
  }
  e.emplace_back("COLTRAIN_BATCH_DISTRIBUTE_POLICY", g.enable_train_adjust_balance ? "BY_PERFORMANCE" : "FIX");
  return e;
}

// "k=v, k2=v2" or "k=v k2=v2" -> --k v --k2 v2
static std::vector<std::string> launcher_argv(const char* script, const char* args, int* batch_size) {
  std::vector<std::string> out = {"python", script};
  if (batch_size) *batch_size = 0;
  const std::string a = args ? args : "";
  size_t i = 0;
  while (i < a.size()) {
    while (i < a.size() && (a[i] == ' ' || a[i] == ',')) ++i;
    if (i >= a.size()) break;
    size_t j = i;
    while (j < a.size() && a[j] != '=' && a[j] != ' ' && a[j] != ',') ++j;
    const std::string key = a.substr(i, j - i);
    std::string val;
    if (j < a.size() && a[j] == '=') {
      size_t k = j + 1;
      while (k < a.size() && a[k] != ' ' && a[k] != ',') ++k;
      val = a.substr(j + 1, k - j - 1);
      j = k;
    }
    out.push_back("--" + key);
    if (!val.empty()) out.push_back(val);
    if (batch_size && key.find("batch-size") != std::string::npos && !val.empty()) *batch_size = atoi(val.c_str());
    i = j;
  }
  return out;
}

static int check_launcher_cfg(const srt_launcher_config* cfg) {
  SRT_REQUIRE(cfg && cfg->serve_mode >= SRT_SERVE_NORMAL && cfg->serve_mode <= SRT_SERVE_COLOCATE_L2, "launcher: bad serve mode");
  return SRT_OK;
}

int srt_launcher_env(const srt_launcher_config* cfg, char* buf, size_t cap) {
  if (int rc = check_launcher_cfg(cfg)) return rc;
  SRT_REQUIRE(buf && cap, "launcher_env: no buffer");
  std::string s;
  for (auto& kv : launcher_env(*cfg)) s += kv.first + "=" + kv.second + "\n";
  SRT_REQUIRE(s.size() < cap, "launcher_env: needs %zu bytes", s.size() + 1);
  memcpy(buf, s.c_str(), s.size() + 1);
  return SRT_OK;
}

int srt_launcher_argv(const char* script, const char* args, char* buf, size_t cap, int* batch_size) {
  SRT_REQUIRE(script && buf && cap, "launcher_argv: bad argument");
  std::string s;
  for (auto& a : launcher_argv(script, args, batch_size)) s += (s.empty() ? "" : "\n") + a;
  SRT_REQUIRE(s.size() < cap, "launcher_argv: needs %zu bytes", s.size() + 1);
  memcpy(buf, s.c_str(), s.size() + 1);
  return SRT_OK;
}

int srt_launcher_launch(const srt_launcher_config* cfg, const char* interpreter, const char* script, const char* args,
                        const char* log_path, int* pid) {
  if (int rc = check_launcher_cfg(cfg)) return rc;
  SRT_REQUIRE(script && pid, "launcher_launch: bad argument");
  std::vector<std::string> argv_s = launcher_argv(script, args, nullptr);
  if (interpreter && *interpreter) argv_s[0] = interpreter;
  const auto env = launcher_env(*cfg);
  std::vector<char*> argv;
  for (auto& s : argv_s) argv.push_back(const_cast<char*>(s.c_str()));
  argv.push_back(nullptr);
  const pid_t child = fork();
  SRT_REQUIRE(child >= 0, "launcher_launch: fork failed");
  if (child == 0) {
    for (auto& kv : env) setenv(kv.first.c_str(), kv.second.c_str(), 1);
    if (log_path && *log_path) {
      const int fd = open(log_path, O_WRONLY | O_CREAT | O_TRUNC, 0644);
      if (fd >= 0) { dup2(fd, STDOUT_FILENO); dup2(fd, STDERR_FILENO); close(fd); }
    }
    execvp(argv[0], argv.data());
    perror("execvp");
    _exit(127);
  }
  *pid = (int)child;
  return SRT_OK;
}

int srt_launcher_wait(int pid, int timeout_ms, int* exited, int* status) {
  SRT_REQUIRE(pid > 0 && exited, "launcher_wait: bad argument");
  *exited = 0;
  const auto give_up = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms < 0 ? 0 : timeout_ms);
  for (;;) {
    int st = 0;
    const pid_t r = waitpid(pid, &st, WNOHANG);
    if (r == pid) {
      *exited = 1;
      if (status) *status = WIFEXITED(st) ? WEXITSTATUS(st) : 128 + WTERMSIG(st);
      return SRT_OK;
    }
    SRT_REQUIRE(r == 0, "launcher_wait: %d is not a child of this process", pid);
    if (timeout_ms >= 0 && std::chrono::steady_clock::now() >= give_up) return SRT_OK;
    std::this_thread::sleep_for(std::chrono::milliseconds(5));
  }
}

int srt_launcher_kill(int pid) {
  SRT_REQUIRE(pid > 0, "launcher_kill: bad pid");
  if (kill(pid, SIGKILL) != 0 && errno != ESRCH) { set_error("launcher_kill: cannot signal %d", pid); return SRT_ERR_STATE; }
  return SRT_OK;
}

// What LaunchTrain does after the fork (server/train_launcher.cc:335-381): wait for the job, tell the controller that
// training has ended (the trainer may not have been able to), and decide what the end means.
int srt_launcher_supervise(srt_controller* ctl, srt_comm* comm, int pid, int timeout_ms, int* outcome, int* status) {
  SRT_REQUIRE(pid > 0 && outcome, "launcher_supervise: bad argument");
  *outcome = SRT_JOB_RUNNING;
  const auto give_up = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms < 0 ? 0 : timeout_ms);
  int st = 0;
  for (;;) {
    const pid_t r = waitpid(pid, &st, WNOHANG);
    if (r == pid) break;
    SRT_REQUIRE(r == 0, "launcher_supervise: %d is not a child of this process", pid);
    if (timeout_ms >= 0 && std::chrono::steady_clock::now() >= give_up) return SRT_OK;
    std::this_thread::sleep_for(std::chrono::milliseconds(5));
  }
  if (status) *status = WIFEXITED(st) ? WEXITSTATUS(st) : 128 + WTERMSIG(st);
  Controller* c = (Controller*)ctl;
  if (c) {
    { std::lock_guard<std::mutex> lk(c->mu); c->train_pid = -1; }
    srt_ctrl_msg end{0, SRT_EV_TRAIN_END, 0};  // Controller::TrainEnd: the monitor thread sees the trainer's own message
    srt_comm_put(c->comm, &end, SRT_TRA2INF, 0);
  }
  if (!WIFSIGNALED(st)) { *outcome = SRT_JOB_FINISHED; return SRT_OK; }
  const int sig = WTERMSIG(st);
  if (sig == SIGKILL) { *outcome = SRT_JOB_KILLED; return SRT_OK; }  // task-switch l3, KillTrain: start it again
  // Any other signal is a crash. The reference ends the server here (LOG(FATAL)) after killing every rank; this call
  // kills the ranks, records what the board says about the job and returns an error.
  *outcome = SRT_JOB_FAILED;
  int cur = -1, target = -1, unpub = -1, killed = 0;
  if (comm) {
    srt_comm_get_train_field(comm, 0, SRT_TI_CURRENT_BS, &cur);
    srt_comm_get_train_field(comm, 0, SRT_TI_TARGET_BS, &target);
    srt_comm_get_train_field(comm, 0, SRT_TI_TARGET_BS_UNPUBLISHED, &unpub);
    srt_launcher_kill_train(comm, &killed);
  }
  set_error("training job %d failed, signal is %s; batch size on the board: current %d, target %d, unpublished %d; "
            "%d other rank(s) killed", pid, strsignal(sig), cur, target, unpub, killed);
  return SRT_ERR_STATE;
}

// KillTrain (server/train_launcher.cc:410-427): every rank whose entry on the board is valid gets SIGKILL.
int srt_launcher_kill_train(srt_comm* comm, int* killed) {
  SRT_REQUIRE(comm, "launcher_kill_train: null channel");
  if (killed) *killed = 0;
  int pid0 = -1, world = 0;
  if (srt_comm_get_train_field(comm, 0, SRT_TI_PID, &pid0) != SRT_OK || pid0 == -1) return SRT_OK;  // no job on record
  if (srt_comm_get_train_field(comm, 0, SRT_TI_WORLD_SIZE, &world) != SRT_OK) return SRT_OK;
  for (int r = 0; r < world && r < SRT_MAX_DEVICE_NUM; ++r) {
    int pid = -1;
    if (srt_comm_get_train_field(comm, r, SRT_TI_PID, &pid) != SRT_OK || pid <= 0) continue;
    if (kill(pid, SIGKILL) == 0) { if (killed) ++*killed; }
    else SRT_REQUIRE(errno == ESRCH, "launcher_kill_train: cannot signal rank %d (pid %d)", r, pid);
  }
  return SRT_OK;
}

// DummyAdjust (server/train_launcher.cc:383-408): the reference's fault injector for the adjust protocol. After a delay
// it shrinks training by one sample, waits for Done and lets it grow back, at random intervals, while training runs.
int srt_launcher_dummy_adjust(srt_controller* ctl, int original_target_bs, int delay_ms, int duration_ms, unsigned seed,
                              int min_gap_ms, int max_gap_ms, int* rounds) {
  Controller* c = (Controller*)ctl;
  SRT_REQUIRE(c && c->cfg.dummy_adjust, "launcher_dummy_adjust: needs a controller created with dummy_adjust = 1");
  if (rounds) *rounds = 0;
  if (delay_ms < 0) delay_ms = 60000;
  if (duration_ms <= 0) duration_ms = 60000;
  if (min_gap_ms <= 0) min_gap_ms = 200;
  if (max_gap_ms < min_gap_ms) max_gap_ms = std::max(min_gap_ms, 1000);
  const auto t_wait = std::chrono::steady_clock::now() + std::chrono::milliseconds(delay_ms);
  while (c->idle() && std::chrono::steady_clock::now() < t_wait + std::chrono::milliseconds(duration_ms))
    std::this_thread::sleep_for(std::chrono::milliseconds(10));  // "while train_pid == -1"
  std::this_thread::sleep_until(t_wait);
  std::mt19937 gen(seed ? seed : 42);
  std::uniform_int_distribution<> gap(min_gap_ms, max_gap_ms);
  const auto t_end = std::chrono::steady_clock::now() + std::chrono::milliseconds(duration_ms);
  while (std::chrono::steady_clock::now() < t_end && !c->idle()) {
    uint64_t cid = 0, eid = 0;
    int rc = srt_controller_colocate_adjust(ctl, 0, 1, &cid);
    if (rc) return rc;
    if (cid) {
      rc = srt_controller_wait_colocate_adjust_done(ctl, 0, cid, 60000);
      if (rc) return rc;
    }
    rc = srt_controller_dummy_infer_exit(ctl, 0, original_target_bs, &eid);
    if (rc) return rc;
    if (rounds) ++*rounds;
    std::this_thread::sleep_for(std::chrono::milliseconds(gap(gen)));
  }
  return SRT_OK;
}

// ---- KVCachePool ----------------------------------------------------------------------------------------
int srt_kvpool_create(srt_pool* pool, srt_controller* controller, srt_adjuster* adjuster, const srt_kvpool_config* cfg,
                      srt_kvpool** out) {
  SRT_REQUIRE(pool && cfg && out, "kvpool_create: null argument");
  KvPool* k = new KvPool();
  k->pool = pool;
  k->ctl = (Controller*)controller;
  k->adjuster = adjuster;
  k->cfg = *cfg;
  if (!k->cfg.min_adjust_nbytes) k->cfg.min_adjust_nbytes = (size_t)5 << 30;
  if (!k->cfg.reclaim_free_nbytes) k->cfg.reclaim_free_nbytes = (size_t)6 << 30;
  if (!k->cfg.reclaim_margin_nbytes) k->cfg.reclaim_margin_nbytes = (size_t)4 << 30;
  if (!k->cfg.adjust_timeout_ms) k->cfg.adjust_timeout_ms = 60000;
  *out = (srt_kvpool*)k;
  return SRT_OK;
}

int srt_kvpool_destroy(srt_kvpool* h) {
  KvPool* k = (KvPool*)h;
  if (!k) return SRT_OK;
  for (auto& kv : k->pages) srt_pool_free(k->pool, SRT_POOL_INFER, (void*)(uintptr_t)kv.first);
  delete k;
  return SRT_OK;
}

int srt_kvpool_set_block_shape(srt_kvpool* h, int64_t block_size, int64_t num_layers, int64_t num_heads, int64_t head_size,
                               size_t block_nbytes) {
  KvPool* k = (KvPool*)h;
  SRT_REQUIRE(k && block_size > 0 && num_layers > 0 && num_heads > 0 && head_size > 0 && block_nbytes > 0, "kvpool_set_block_shape: bad argument");
  std::lock_guard<std::mutex> lk(k->mu);
  if (k->shape_set) {  // MaybeSet...: a second caller must agree
    SRT_REQUIRE(k->block_size == block_size && k->num_layers == num_layers && k->num_heads == num_heads && k->head_size == head_size &&
                    k->block_nbytes == block_nbytes,
                "kvpool_set_block_shape: the block shape was set differently before");
    return SRT_OK;
  }
  k->block_size = block_size; k->num_layers = num_layers; k->num_heads = num_heads; k->head_size = head_size;
  k->block_nbytes = block_nbytes;
  k->shape_set = true;
  return SRT_OK;
}

int64_t srt_kvpool_num_gpu_blocks(srt_kvpool* h) {
  KvPool* k = (KvPool*)h;
  if (!k) return -1;
  std::lock_guard<std::mutex> lk(k->mu);
  return k->shape_set ? k->num_gpu_blocks() : -1;
}

int srt_kvpool_shape(srt_kvpool* h, int64_t shape[3], int64_t stride[3]) {
  KvPool* k = (KvPool*)h;
  SRT_REQUIRE(k && shape && stride, "kvpool_shape: null argument");
  std::lock_guard<std::mutex> lk(k->mu);
  SRT_REQUIRE(k->shape_set, "kvpool_shape: the block shape is not set");
  const int64_t row = k->block_size * k->num_heads * k->head_size;
  shape[0] = 2; shape[1] = k->num_layers * k->num_gpu_blocks(); shape[2] = row;
  stride[0] = row; stride[1] = row * 2; stride[2] = 1;
  return SRT_OK;
}

static void init_layer_blocks(KvPool* k) {
  if (k->free_layer_blocks != -1) return;
  k->free_layer_blocks = k->num_gpu_blocks() * k->num_layers;
  k->used_layer_blocks = 0;
  if (const char* e = getenv("SIRIUS_VLLM_NUM_LAYER_BLOCK")) {
    const long long v = atoll(e);
    if (v > 0 && v <= k->free_layer_blocks) k->free_layer_blocks = v;
  }
}

int srt_kvpool_layer_block_info(srt_kvpool* h, int64_t* free_blocks, int64_t* used_blocks) {
  KvPool* k = (KvPool*)h;
  SRT_REQUIRE(k && free_blocks && used_blocks, "kvpool_layer_block_info: null argument");
  std::lock_guard<std::mutex> lk(k->mu);
  SRT_REQUIRE(k->shape_set, "kvpool_layer_block_info: the block shape is not set");
  init_layer_blocks(k);
  *free_blocks = k->free_layer_blocks;
  *used_blocks = k->used_layer_blocks;
  return SRT_OK;
}

int srt_kvpool_update_free_layer_blocks(srt_kvpool* h, int64_t delta) {
  KvPool* k = (KvPool*)h;
  SRT_REQUIRE(k, "kvpool: null handle");
  std::lock_guard<std::mutex> lk(k->mu);
  SRT_REQUIRE(k->shape_set, "kvpool: the block shape is not set");
  init_layer_blocks(k);
  SRT_REQUIRE(k->free_layer_blocks + delta >= 0, "kvpool: %lld free layer blocks, cannot take %lld", (long long)k->free_layer_blocks,
              (long long)-delta);
  k->free_layer_blocks += delta;
  k->used_layer_blocks -= delta;
  return SRT_OK;
}

int srt_kvpool_update_free_layer_blocks_by_train_base(srt_kvpool* h, size_t train_base_nbytes) {
  KvPool* k = (KvPool*)h;
  SRT_REQUIRE(k, "kvpool: null handle");
  std::lock_guard<std::mutex> lk(k->mu);
  SRT_REQUIRE(k->shape_set, "kvpool: the block shape is not set");
  init_layer_blocks(k);
  SRT_REQUIRE(k->used_layer_blocks == 0, "kvpool: blocks are in use; the training base has to be accounted for before serving starts");
  const int64_t taken = (int64_t)((train_base_nbytes + (size_t)(k->cfg.train_memory_over_predict_mb * kMB)) / k->block_nbytes);
  const int64_t blocks = k->num_gpu_blocks() - taken;
  SRT_REQUIRE(blocks >= 0, "kvpool: the training base does not fit the pool");
  k->free_layer_blocks = blocks * k->num_layers;
  return SRT_OK;
}

// MaybeAdjustTrain (kv_cache_pool.cc:288-332)
static int kv_adjust_train(KvPool* k, size_t need_nbytes, size_t min_nbytes, int* adjusted) {
  const size_t page = k->page_bytes();
  if (!k->ctl || !k->adjuster) {
    set_error("kvpool: %zu bytes are not available and no controller / adjuster was given to ask training for them", need_nbytes);
    return SRT_ERR_NOMEM;
  }
  const double require_mb = (double)(need_nbytes + k->cfg.train_over_adjust_nbytes) / kMB;
  const double free_b = (double)srt_pool_stat(k->pool, SRT_POOL_STAT_FREE_PAGES) * (double)page - k->cfg.train_memory_over_predict_mb * kMB;
  const double avail_mb = (free_b + (double)srt_pool_stat(k->pool, SRT_POOL_STAT_TRAIN_ALL)) / kMB - require_mb;
  int plan[SRT_MAX_DEVICE_NUM], n = 0;
  int rc = srt_adjuster_llm_require_plan(k->adjuster, k->cfg.device_id, require_mb, avail_mb, nullptr, plan, &n);
  if (rc) return rc;
  if (n > 0) {
    uint64_t id = 0;
    rc = srt_controller_infer_require_adjust((srt_controller*)k->ctl, k->cfg.device_id, plan, n, &id);
    if (rc) return rc;
    rc = srt_controller_wait_colocate_adjust_done((srt_controller*)k->ctl, k->cfg.device_id, id, k->cfg.adjust_timeout_ms);
    if (rc) return rc;
    if (adjusted) *adjusted = 1;
  }
  const size_t free_after = (size_t)srt_pool_stat(k->pool, SRT_POOL_STAT_FREE_PAGES) * page;
  SRT_REQUIRE(free_after >= min_nbytes, "kvpool: %zu bytes free after the adjust, %zu needed", free_after, min_nbytes);
  return SRT_OK;
}

int srt_kvpool_alloc_pages(srt_kvpool* h, size_t page_nbytes, int n, uint64_t* pages, int* adjusted) {
  KvPool* k = (KvPool*)h;
  SRT_REQUIRE(k && page_nbytes > 0 && n > 0 && pages, "kvpool_alloc_pages: bad argument");
  std::lock_guard<std::mutex> lk(k->mu);
  if (adjusted) *adjusted = 0;
  const size_t page = k->page_bytes();
  const size_t need = (size_t)n * page_nbytes;
  // what inference may take without pushing training below what it is predicted to need
  double predict_mb = 0.0;
  if (k->adjuster) {
    int rc = srt_adjuster_predict_train_mem_usage_mb(k->adjuster, k->cfg.device_id, &predict_mb);
    if (rc) return rc;
  }
  const double train_all = (double)srt_pool_stat(k->pool, SRT_POOL_STAT_TRAIN_ALL);
  const double train_mem = std::max(predict_mb * kMB, train_all);
  const double available = (double)srt_pool_stat(k->pool, SRT_POOL_STAT_FREE_PAGES) * (double)page + train_all - train_mem -
                           k->cfg.train_memory_over_predict_mb * kMB;
  if (available < (double)need) {
    const size_t ask = std::max(k->cfg.min_adjust_nbytes / page * page, (need + page - 1) / page * page);
    int rc = kv_adjust_train(k, ask, (need + page - 1) / page * page, adjusted);
    if (rc) return rc;
  }
  for (int i = 0; i < n; ++i) {
    void* p = nullptr;
    int rc = srt_pool_alloc(k->pool, SRT_POOL_INFER, page_nbytes, &p);
    if (rc) {
      for (int j = 0; j < i; ++j) {
        srt_pool_free(k->pool, SRT_POOL_INFER, (void*)(uintptr_t)pages[j]);
        k->pages.erase(pages[j]);
      }
      return rc;
    }
    pages[i] = (uint64_t)(uintptr_t)p;
    k->pages[pages[i]] = page_nbytes;
  }
  return SRT_OK;
}

int srt_kvpool_free_pages(srt_kvpool* h, const uint64_t* pages, int n, int* reclaimed_to_train) {
  KvPool* k = (KvPool*)h;
  SRT_REQUIRE(k && pages && n > 0, "kvpool_free_pages: bad argument");
  std::lock_guard<std::mutex> lk(k->mu);
  if (reclaimed_to_train) *reclaimed_to_train = 0;
  for (int i = 0; i < n; ++i) {
    auto it = k->pages.find(pages[i]);
    SRT_REQUIRE(it != k->pages.end(), "kvpool_free_pages: %#llx is not a KV-cache page", (unsigned long long)pages[i]);
    int rc = srt_pool_free(k->pool, SRT_POOL_INFER, (void*)(uintptr_t)pages[i]);
    if (rc) return rc;
    k->pages.erase(it);
  }
  size_t rel = 0;
  int rc = srt_pool_empty_cache(k->pool, SRT_POOL_INFER, &rel);
  if (rc) return rc;
  // ReclaimMemToTrain (kv_cache_pool.cc:334-342): enough of the pool is free again, training may grow
  const size_t page = k->page_bytes();
  const size_t free_b = (size_t)srt_pool_stat(k->pool, SRT_POOL_STAT_FREE_PAGES) * page;
  if (k->ctl && k->adjuster && !k->ctl->idle() && free_b >= k->cfg.reclaim_free_nbytes) {
    const int world = k->ctl->world;
    std::vector<double> avail((size_t)world), fre((size_t)world);
    const double f = (double)free_b - k->cfg.train_memory_over_predict_mb * kMB - (double)k->cfg.reclaim_margin_nbytes;
    for (int r = 0; r < world; ++r) {  // one pool per device; this one describes device_id, the others are taken to match
      fre[(size_t)r] = f / kMB;
      avail[(size_t)r] = (f + (double)srt_pool_stat(k->pool, SRT_POOL_STAT_TRAIN_ALL)) / kMB;
    }
    int plan[SRT_MAX_DEVICE_NUM], np = 0;
    rc = srt_adjuster_llm_release_plan(k->adjuster, avail.data(), fre.data(), plan, &np);
    if (rc) return rc;
    if (np > 0) {
      uint64_t id = 0;
      rc = srt_controller_infer_release_adjust((srt_controller*)k->ctl, plan, np, &id);
      if (rc) return rc;
      if (reclaimed_to_train) *reclaimed_to_train = 1;
    }
  }
  return SRT_OK;
}

double srt_kvpool_util(srt_kvpool* h) {
  KvPool* k = (KvPool*)h;
  if (!k) return NAN;
  std::lock_guard<std::mutex> lk(k->mu);
  if (!k->shape_set || k->used_layer_blocks < 0) return NAN;
  const double infer = (double)srt_pool_stat(k->pool, SRT_POOL_STAT_INFER_USAGE);
  if (infer <= 0) return NAN;
  return (double)k->used_layer_blocks * (double)k->block_nbytes / (double)k->num_layers / infer;
}

}  // extern "C"
