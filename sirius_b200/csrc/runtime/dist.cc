// DistTrainSync, DynamicBatchDistirbutor and PerfModel of the training job, in one shared-memory
// segment per job (rank 0 creates it).
//
// Follows pytorch/torch_col/csrc/dist_train_sync.{h,cc} (barrier, [src][dst] mailboxes),
// dynamic_batch.{h,cc} (ledger of sample-index ranges of the current global batch: unprocessed /
// processing / processed sets, per-rank counters, the finish/abort vote on the last micro-batch)
// and perf_model.{h,cc} (running mean throughput per batch size, linear interpolation). Every CHECK
// of the reference is kept as an error return. Sets are fixed-capacity sorted arrays.
#include <math.h>

#include <algorithm>
#include <string>
#include <vector>

#include "../../../include/sirius_runtime.h"
#include "rt_common.h"
#include "shm_util.h"

namespace srt {
namespace {

constexpr uint32_t kDistMagic = 0x53445432;  // "SDT2"
constexpr int kSetCap = 4096;
constexpr int kPerfCap = 1024;
constexpr int kMailBytes = 256 * 64;  // the reference moves strings in 256-byte chunks
constexpr int kAbortVote = INT32_MIN;

struct Range { int first, second; };
inline bool range_less(const Range& a, const Range& b) {
  return a.first != b.first ? a.first < b.first : a.second < b.second;
}

struct RangeSet {  // sorted, unique
  int n;
  Range v[kSetCap];
  void clear() { n = 0; }
  int lower(const Range& r) const { return (int)(std::lower_bound(v, v + n, r, range_less) - v); }
  int find(const Range& r) const {
    int i = lower(r);
    return (i < n && v[i].first == r.first && v[i].second == r.second) ? i : -1;
  }
  bool insert(const Range& r) {
    int i = lower(r);
    if (i < n && v[i].first == r.first && v[i].second == r.second) return true;
    if (n >= kSetCap) return false;
    memmove(&v[i + 1], &v[i], sizeof(Range) * (size_t)(n - i));
    v[i] = r;
    ++n;
    return true;
  }
  void erase_at(int i) {
    memmove(&v[i], &v[i + 1], sizeof(Range) * (size_t)(n - i - 1));
    --n;
  }
};

struct Mailbox {
  shm::Mutex mu;
  shm::Cond cond;
  int full;
  int nbytes;
  char data[kMailBytes];
};

struct PerfEntry { int bs; double thpt; int count; };

struct DistLayout {
  shm::SegHeader hdr;
  int world_size;
  // barrier
  shm::Mutex bar_mu;
  shm::Cond bar_cond;
  int bar_count;
  uint32_t bar_generation;
  // mailboxes [src][dst]
  Mailbox mail[SRT_MAX_DEVICE_NUM][SRT_MAX_DEVICE_NUM];
  // ledger of the current global batch (GlobalSharedData)
  shm::Mutex mu;
  shm::Cond vote_cv;
  std::atomic<int> vote_cnt;
  int unproc_per_train[SRT_MAX_DEVICE_NUM], procing_per_train[SRT_MAX_DEVICE_NUM],
      proced_per_train[SRT_MAX_DEVICE_NUM];
  int has_unproc_batches[SRT_MAX_DEVICE_NUM];
  int num_unproc, num_procing, num_proced;
  RangeSet unproc, procing, proced;
  // perf model
  shm::Mutex perf_mu;
  int perf_n;
  PerfEntry perf[kPerfCap];
  // task-switch flags shared by the ranks of one job (SwitchStub's "switch_stub" shared data,
  // pytorch/torch_col/csrc/control_stub.cc:186-200): [0] global interrupt flag, [1] has a batch been killed
  shm::Mutex sw_mu;
  int sw_flag[2];
};

}  // namespace

struct Dist {
  shm::Segment<DistLayout> seg;
  int rank = 0, world = 1;
  // per-process epoch bookkeeping, as in the reference (members of the distributor object)
  bool inited = false;
  bool lazy = false;
  int policy = SRT_DBD_SIMPLE;
  int dataset_size = 0, input_batch_size = 0, global_batch_size = 0;
  bool first_epoch_start = false;
  int num_proced_sample_of_epoch = 0, num_proced_global_batches = 0, next_epoch_idx = 0;
  int num_global_batches_per_epoch = 0;
  DistLayout* L() { return seg.get(); }
};

static double perf_get_locked(DistLayout* l, int bs) {
  if (l->perf_n == 0) return -1;
  if (bs <= 0) return 0;
  const PerfEntry* p = l->perf;
  const int n = l->perf_n;
  if (p[0].bs >= bs) return p[0].thpt / p[0].bs * bs;
  if (p[n - 1].bs <= bs) return p[n - 1].thpt / p[n - 1].bs * bs;
  int i = 0;
  while (p[i].bs < bs) ++i;  // lower_bound
  if (p[i].bs == bs) return p[i].thpt;
  return (p[i].thpt - p[i - 1].thpt) / (p[i].bs - p[i - 1].bs) * (bs - p[i - 1].bs) + p[i - 1].thpt;
}

static int barrier_wait(Dist* d, int timeout_ms) {
  DistLayout* l = d->L();
  shm::Guard g(l->bar_mu);
  const uint32_t gen = l->bar_generation;
  if (++l->bar_count == d->world) {
    l->bar_count = 0;
    l->bar_generation++;
    l->bar_cond.notify_all();
    return SRT_OK;
  }
  const timespec dl = shm::deadline_after_ms(timeout_ms < 0 ? 0 : timeout_ms);
  while (l->bar_generation == gen) {
    if (timeout_ms < 0) l->bar_cond.wait(l->bar_mu);
    else if (!l->bar_cond.wait_until(l->bar_mu, dl)) {
      if (l->bar_generation != gen) break;
      l->bar_count--;  // withdraw: the barrier stays usable for the others
      set_error("dist barrier: rank %d timed out after %d ms", d->rank, timeout_ms);
      return SRT_ERR_TIMEOUT;
    }
  }
  return SRT_OK;
}

// DistributeBatchImpl (dynamic_batch.cc:254-314)
static void distribute_impl(Dist* d, const std::vector<int>& workers, const std::vector<int>& target_bs,
                            int num_unproc) {
  DistLayout* l = d->L();
  const int nw = (int)workers.size();
  if (d->policy == SRT_DBD_FIX || d->policy == SRT_DBD_SIMPLE) {
    const int per = num_unproc / nw, rem = num_unproc % nw;
    for (int i = 0; i < nw; ++i) l->unproc_per_train[workers[i]] = per + (i < rem ? 1 : 0);
    return;
  }
  std::vector<double> perf(nw);
  double sum = 0;
  {
    shm::Guard g(l->perf_mu);
    for (int i = 0; i < nw; ++i) { perf[i] = perf_get_locked(l, target_bs[i]); sum += perf[i]; }
  }
  // Fewer samples left than ranks that could take them (the tail of a global batch after aborts): "at least one
  // each" cannot hold. The first num_unproc ranks get one sample, the others none and leave the distribution.
  if (num_unproc < nw) {
    for (int i = 0; i < nw; ++i) {
      l->unproc_per_train[workers[i]] = i < num_unproc ? 1 : 0;
      if (i >= num_unproc) l->has_unproc_batches[workers[i]] = 0;
    }
    return;
  }
  int distributed = 0;
  for (int i = 0; i < nw; ++i) {
    const double ratio = sum == 0 ? 1.0 / nw : perf[i] / sum;
    const int ns = std::max(1, (int)(num_unproc * ratio));
    l->unproc_per_train[workers[i]] = ns;
    distributed += ns;
  }
  // round-off: hand the difference out (or take it back, never below one sample) one by one; with
  // num_unproc >= nw this ends after at most |diff| + nw visits
  int diff = num_unproc - distributed;
  for (int i = 0, visits = 0; diff != 0 && visits < 4 * (nw + std::abs(num_unproc - distributed)); ++i, ++visits) {
    if (i >= nw) i = 0;
    int& v = l->unproc_per_train[workers[i]];
    if (diff > 0) { v += 1; diff--; }
    else if (v > 1) { v -= 1; diff++; }
  }
}

// DistributeBatchWithoutLock (dynamic_batch.cc:157-252)
static int distribute_locked(Dist* d, srt_comm* comm, bool check, bool to_all, bool at_begin) {
  DistLayout* l = d->L();
  std::vector<int> target_unpub(d->world, d->input_batch_size);
  if (comm) {
    for (int i = 0; i < d->world; ++i) {
      int rc = srt_comm_get_train_field(comm, i, SRT_TI_TARGET_BS_UNPUBLISHED, &target_unpub[i]);
      if (rc) return rc;
    }
  }
  const bool do_distribute = !(d->lazy || (!at_begin && d->policy == SRT_DBD_FIX));
  int num_unproc = l->num_unproc;
  if (check && do_distribute) {
    int s = 0;
    for (int i = 0; i < d->world; ++i) s += l->unproc_per_train[i];
    SRT_REQUIRE(s == l->num_unproc, "distribute_batch: per-rank unprocessed samples sum to %d, ledger has %d", s,
                l->num_unproc);
    num_unproc = s;
  }
  if (to_all)
    for (int i = 0; i < d->world; ++i) l->has_unproc_batches[i] = 1;
  if (do_distribute) {
    std::vector<int> workers, tbs;
    for (int i = 0; i < d->world; ++i)
      if (l->has_unproc_batches[i]) { workers.push_back(i); tbs.push_back(comm ? target_unpub[i] : d->input_batch_size); }
    if (!workers.empty()) distribute_impl(d, workers, tbs, num_unproc);
    else SRT_REQUIRE(num_unproc == 0, "distribute_batch: %d samples left but no rank can take them", num_unproc);
  }
  SRT_REQUIRE(num_unproc >= 0, "distribute_batch: negative unprocessed count");
  if (log_on(LOG_DYNAMIC_BATCH)) {
    std::string per, tgt;
    for (int i = 0; i < d->world; ++i) {
      per += (i ? " " : "") + std::to_string(l->unproc_per_train[i]);
      tgt += (i ? " " : "") + std::to_string(target_unpub[i]);
    }
    log_line(LOG_DYNAMIC_BATCH, "[DistributeBatch] %d unprocessed samples -> per rank [%s], target batch sizes [%s]%s",
             num_unproc, per.c_str(), tgt.c_str(), do_distribute ? "" : " (not redistributed)");
  }
  if (comm) {  // publish: target_batch_size := target_batch_size_unpublished
    for (int i = 0; i < d->world; ++i) {
      int rc = srt_comm_update_train_field(comm, i, SRT_TI_TARGET_BS, target_unpub[i]);
      if (rc) return rc;
    }
  }
  return SRT_OK;
}

}  // namespace srt

using namespace srt;

#define DIST_CHECK(h) SRT_REQUIRE((h) != nullptr && ((Dist*)(h))->L() != nullptr, "dist_train_sync: not open")
#define DBD_CHECK(h)  \
  DIST_CHECK(h);      \
  SRT_REQUIRE(((Dist*)(h))->inited, "dynamic batch distributor: srt_dbd_init has not been called")

extern "C" {

int srt_dist_open(const char* name, int rank, int world_size, int timeout_ms, srt_dist** out) {
  SRT_REQUIRE(out && world_size >= 1 && world_size <= SRT_MAX_DEVICE_NUM && rank >= 0 && rank < world_size,
              "dist_open: bad rank/world (%d/%d)", rank, world_size);
  Dist* d = new Dist();
  d->rank = rank;
  d->world = world_size;
  const std::string nm = name ? std::string(name) : default_shm_prefix() + "_dist_train_sync";
  std::string err;
  bool ok;
  if (rank == 0) {
    ok = d->seg.create(nm, kDistMagic, true, [&](DistLayout* l) {
      l->world_size = world_size;
      l->bar_mu.init(); l->bar_cond.init();
      for (int i = 0; i < SRT_MAX_DEVICE_NUM; ++i)
        for (int j = 0; j < SRT_MAX_DEVICE_NUM; ++j) { l->mail[i][j].mu.init(); l->mail[i][j].cond.init(); }
      l->mu.init(); l->vote_cv.init(); l->vote_cnt.store(0);
      l->perf_mu.init();
      l->sw_mu.init(); l->sw_flag[0] = l->sw_flag[1] = 0;
    }, &err);
  } else {
    ok = d->seg.open(nm, kDistMagic, timeout_ms, &err);
    if (ok && d->L()->world_size != world_size) { ok = false; err = "world size mismatch"; }
  }
  if (!ok) {
    set_error("dist_train_sync: %s", err.c_str());
    delete d;
    return SRT_ERR_STATE;
  }
  *out = (srt_dist*)d;
  return SRT_OK;
}

int srt_dist_close(srt_dist* h) {
  Dist* d = (Dist*)h;
  if (!d) return SRT_OK;
  if (d->rank == 0) d->seg.unlink();
  delete d;
  return SRT_OK;
}

int srt_dist_barrier(srt_dist* h, int timeout_ms) {
  DIST_CHECK(h);
  return barrier_wait((Dist*)h, timeout_ms);
}

int srt_dist_send(srt_dist* h, int dst, const char* data, int nbytes) {
  DIST_CHECK(h);
  Dist* d = (Dist*)h;
  SRT_REQUIRE(dst >= 0 && dst < d->world && data && nbytes >= 0 && nbytes <= kMailBytes, "dist_send: bad argument");
  Mailbox& m = d->L()->mail[d->rank][dst];
  shm::Guard g(m.mu);
  while (m.full) m.cond.wait(m.mu);
  memcpy(m.data, data, (size_t)nbytes);
  m.nbytes = nbytes;
  m.full = 1;
  m.cond.notify_all();
  return SRT_OK;
}

int srt_dist_recv(srt_dist* h, int src, char* buf, int cap, int timeout_ms, int* nbytes) {
  DIST_CHECK(h);
  Dist* d = (Dist*)h;
  SRT_REQUIRE(src >= 0 && src < d->world && buf && nbytes, "dist_recv: bad argument");
  Mailbox& m = d->L()->mail[src][d->rank];
  shm::Guard g(m.mu);
  const timespec dl = shm::deadline_after_ms(timeout_ms < 0 ? 0 : timeout_ms);
  while (!m.full) {
    if (timeout_ms < 0) m.cond.wait(m.mu);
    else if (!m.cond.wait_until(m.mu, dl) && !m.full) {
      set_error("dist_recv: nothing from rank %d within %d ms", src, timeout_ms);
      return SRT_ERR_TIMEOUT;
    }
  }
  SRT_REQUIRE(m.nbytes <= cap, "dist_recv: message of %d bytes does not fit %d", m.nbytes, cap);
  memcpy(buf, m.data, (size_t)m.nbytes);
  *nbytes = m.nbytes;
  m.full = 0;
  m.cond.notify_all();
  return SRT_OK;
}

int srt_dbd_init(srt_dist* h, int dataset_size, int input_batch_size, int global_batch_size,
                 int lazy_distributing, int policy) {
  DIST_CHECK(h);
  Dist* d = (Dist*)h;
  SRT_REQUIRE(!d->inited, "dynamic batch distributor: already initialised");
  SRT_REQUIRE(dataset_size > 0 && input_batch_size > 0 && global_batch_size > 0, "dbd_init: sizes must be positive");
  SRT_REQUIRE(policy >= SRT_DBD_FIX && policy <= SRT_DBD_BY_PERFORMANCE, "dbd_init: unknown policy %d", policy);
  d->dataset_size = dataset_size;
  d->input_batch_size = input_batch_size;
  d->global_batch_size = global_batch_size;
  d->lazy = lazy_distributing != 0;
  d->policy = policy;
  d->num_global_batches_per_epoch = (dataset_size + global_batch_size - 1) / global_batch_size;
  d->inited = true;
  if (d->lazy) {
    if (d->rank == 0) {
      DistLayout* l = d->L();
      shm::Guard g(l->mu);
      for (int i = 0; i < d->world; ++i) l->unproc_per_train[i] = l->procing_per_train[i] = l->proced_per_train[i] = -1;
    }
    return barrier_wait(d, 10000);
  }
  return SRT_OK;
}

int srt_dbd_distribute_batch(srt_dist* h, srt_comm* comm, int check, int to_all, int at_begin) {
  DBD_CHECK(h);
  Dist* d = (Dist*)h;
  shm::Guard g(d->L()->mu);
  return distribute_locked(d, comm, check != 0, to_all != 0, at_begin != 0);
}

int srt_dbd_get_batch(srt_dist* h, int batch_size_in, int* ranges, int cap_pairs, int* n_ranges,
                      int* last_micro_batch) {
  DBD_CHECK(h);
  Dist* d = (Dist*)h;
  SRT_REQUIRE(ranges && n_ranges && last_micro_batch && cap_pairs > 0, "dbd_get_batch: bad argument");
  DistLayout* l = d->L();
  shm::Guard g(l->mu);
  int batch_size = batch_size_in;
  bool last = false;
  if (d->lazy) {  // LazyDistributingGetBatchSize
    int ongoing = 0;
    for (int i = 0; i < d->world; ++i) ongoing += l->has_unproc_batches[i] ? 1 : 0;
    SRT_REQUIRE(ongoing > 0, "dbd_get_batch: no rank has batches left");
    const int max_bs = l->num_unproc - ongoing + 1;
    if (batch_size >= max_bs) { batch_size = max_bs; last = true; }
  } else {
    batch_size = std::min(batch_size, l->unproc_per_train[d->rank]);
  }
  int num = 0, n = 0, it = 0;
  while (num < batch_size) {
    SRT_REQUIRE(it < l->unproc.n, "dbd_get_batch: unprocessed queue exhausted (%d of %d samples)", num, batch_size);
    SRT_REQUIRE(n < cap_pairs, "dbd_get_batch: more than %d ranges", cap_pairs);
    const Range r = l->unproc.v[it];
    const int cur = r.second - r.first;
    if (cur + num <= batch_size) {
      num += cur;
      ranges[2 * n] = r.first; ranges[2 * n + 1] = r.second; ++n;
      SRT_REQUIRE(l->procing.insert(r), "dbd_get_batch: processing set is full");
      l->unproc.erase_at(it);  // `it` now names the next element
    } else {
      const Range slice = {r.first, r.first + (batch_size - num)}, rest = {r.first + (batch_size - num), r.second};
      num += slice.second - slice.first;
      ranges[2 * n] = slice.first; ranges[2 * n + 1] = slice.second; ++n;
      SRT_REQUIRE(l->procing.insert(slice), "dbd_get_batch: processing set is full");
      l->unproc.erase_at(it);
      SRT_REQUIRE(l->unproc.insert(rest), "dbd_get_batch: unprocessed set is full");
      it = l->unproc.find(rest);
    }
  }
  if (!d->lazy) {
    l->unproc_per_train[d->rank] -= num;
    l->procing_per_train[d->rank] += num;
    SRT_REQUIRE(l->unproc_per_train[d->rank] >= 0, "dbd_get_batch: negative per-rank unprocessed count");
    last = l->unproc_per_train[d->rank] == 0;
  }
  l->num_unproc -= num;
  l->num_procing += num;
  SRT_REQUIRE(l->num_unproc >= 0, "dbd_get_batch: negative unprocessed count");
  if (last) l->has_unproc_batches[d->rank] = 0;
  *n_ranges = n;
  *last_micro_batch = last ? 1 : 0;
  return SRT_OK;
}

int srt_dbd_query_next_batch_size(srt_dist* h, int batch_size, int* out) {
  DBD_CHECK(h);
  Dist* d = (Dist*)h;
  SRT_REQUIRE(out != nullptr, "dbd_query: null out");
  DistLayout* l = d->L();
  shm::Guard g(l->mu);
  const int mx = d->lazy ? l->num_unproc : l->unproc_per_train[d->rank];
  *out = std::min(mx, batch_size);
  return SRT_OK;
}

static int move_ranges(Dist* d, const int* ranges, int n, RangeSet& to, int* moved) {
  DistLayout* l = d->L();
  int num = 0;
  for (int i = 0; i < n; ++i) {
    const Range r = {ranges[2 * i], ranges[2 * i + 1]};
    SRT_REQUIRE(r.second > r.first, "range [%d,%d) is empty", r.first, r.second);
    const int at = l->procing.find(r);
    SRT_REQUIRE(at >= 0, "range [%d,%d) is not in the processing set", r.first, r.second);
    SRT_REQUIRE(to.insert(r), "ledger set is full");
    l->procing.erase_at(at);
    num += r.second - r.first;
  }
  *moved = num;
  return SRT_OK;
}

int srt_dbd_finish_batch(srt_dist* h, const int* ranges, int n_ranges, int end_of_global_batch) {
  DBD_CHECK(h);
  Dist* d = (Dist*)h;
  DistLayout* l = d->L();
  shm::Guard g(l->mu);
  int num = 0;
  int rc = move_ranges(d, ranges, n_ranges, l->proced, &num);
  if (rc) return rc;
  if (!d->lazy) { l->procing_per_train[d->rank] -= num; l->proced_per_train[d->rank] += num; }
  l->num_procing -= num;
  l->num_proced += num;
  SRT_LOG(LOG_DYNAMIC_BATCH, "[FinishBatch] rank %d finished %d samples%s: %d unprocessed, %d processing, %d processed",
          d->rank, num, end_of_global_batch ? " (end of global batch)" : "", l->num_unproc, l->num_procing, l->num_proced);
  if (end_of_global_batch) {
    SRT_REQUIRE(d->lazy || l->procing_per_train[d->rank] == 0,
                "finish_batch: end of global batch with %d samples still processing", l->procing_per_train[d->rank]);
    d->num_proced_global_batches++;
    d->num_proced_sample_of_epoch = std::min(d->num_proced_sample_of_epoch + d->global_batch_size, d->dataset_size);
  }
  return SRT_OK;
}

int srt_dbd_abort_batch(srt_dist* h, const int* ranges, int n_ranges, int /*end_of_global_batch*/) {
  DBD_CHECK(h);
  Dist* d = (Dist*)h;
  DistLayout* l = d->L();
  shm::Guard g(l->mu);
  int num = 0;
  int rc = move_ranges(d, ranges, n_ranges, l->unproc, &num);
  if (rc) return rc;
  if (!d->lazy) { l->procing_per_train[d->rank] -= num; l->unproc_per_train[d->rank] += num; }
  l->num_procing -= num;
  l->num_unproc += num;
  SRT_LOG(LOG_DYNAMIC_BATCH, "[AbortBatch] rank %d gives back %d samples: %d unprocessed, %d processing, %d processed",
          d->rank, num, l->num_unproc, l->num_procing, l->num_proced);
  return SRT_OK;
}

int srt_dbd_vote_finish_last_micro_batch(srt_dist* h, int timeout_ms, int* finished) {
  DBD_CHECK(h);
  Dist* d = (Dist*)h;
  SRT_REQUIRE(finished != nullptr, "vote_finish: null out");
  DistLayout* l = d->L();
  shm::Guard g(l->mu);
  const int before = l->vote_cnt.fetch_add(1, std::memory_order_relaxed);
  if (before + 1 == d->world) { l->vote_cv.notify_all(); *finished = 1; return SRT_OK; }
  if (before < 0) { *finished = 0; return SRT_OK; }
  const timespec dl = shm::deadline_after_ms(timeout_ms < 0 ? 0 : timeout_ms);
  for (;;) {
    const int v = l->vote_cnt.load(std::memory_order_relaxed);
    if (v == d->world) { *finished = 1; return SRT_OK; }
    if (v < 0) { *finished = 0; return SRT_OK; }
    if (timeout_ms < 0) l->vote_cv.wait(l->mu);
    else if (!l->vote_cv.wait_until(l->mu, dl)) {
      const int w = l->vote_cnt.load(std::memory_order_relaxed);
      if (w == d->world) { *finished = 1; return SRT_OK; }
      if (w < 0) { *finished = 0; return SRT_OK; }
      set_error("vote_finish: %d of %d ranks voted within %d ms", w, d->world, timeout_ms);
      return SRT_ERR_TIMEOUT;
    }
  }
}

int srt_dbd_vote_abort_last_micro_batch(srt_dist* h) {
  DBD_CHECK(h);
  DistLayout* l = ((Dist*)h)->L();
  shm::Guard g(l->mu);
  l->vote_cnt.store(kAbortVote, std::memory_order_relaxed);
  l->vote_cv.notify_all();
  SRT_LOG(LOG_DYNAMIC_BATCH, "[VoteAbortLastMicroBatch] rank %d", ((Dist*)h)->rank);
  return SRT_OK;
}

int srt_dbd_reset_last_micro_batch_finish_vote(srt_dist* h) {
  DBD_CHECK(h);
  DistLayout* l = ((Dist*)h)->L();
  shm::Guard g(l->mu);
  l->vote_cnt.store(0, std::memory_order_relaxed);
  return SRT_OK;
}

int srt_dbd_next_global_batch(srt_dist* h, srt_comm* comm, int timeout_ms) {
  DBD_CHECK(h);
  Dist* d = (Dist*)h;
  DistLayout* l = d->L();
  int rc = barrier_wait(d, timeout_ms);
  if (rc) return rc;
  int master_rc = SRT_OK;
  if (d->rank == 0) {
    shm::Guard g(l->mu);
    l->vote_cnt.store(0, std::memory_order_relaxed);
    const int cur = d->global_batch_size + d->num_proced_sample_of_epoch > d->dataset_size
                        ? d->dataset_size - d->num_proced_sample_of_epoch
                        : d->global_batch_size;
    if (cur < 0) {
      set_error("next_global_batch: negative global batch (%d processed of %d)", d->num_proced_sample_of_epoch,
                d->dataset_size);
      master_rc = SRT_ERR_STATE;
    } else {
      l->num_unproc = cur;
      l->num_procing = l->num_proced = 0;
      l->unproc.clear(); l->procing.clear(); l->proced.clear();
      if (cur > 0) {
        l->unproc.insert({d->num_proced_sample_of_epoch, d->num_proced_sample_of_epoch + cur});
        master_rc = distribute_locked(d, comm, false, true, true);
        if (!d->lazy)
          for (int i = 0; i < d->world; ++i) l->procing_per_train[i] = l->proced_per_train[i] = 0;
      } else if (!d->lazy) {
        for (int i = 0; i < d->world; ++i)
          l->unproc_per_train[i] = l->procing_per_train[i] = l->proced_per_train[i] = 0;
      }
    }
  }
  rc = barrier_wait(d, timeout_ms);
  return master_rc ? master_rc : rc;
}

int srt_dbd_next_epoch(srt_dist* h, int* epoch) {
  DBD_CHECK(h);
  Dist* d = (Dist*)h;
  SRT_REQUIRE(epoch != nullptr, "next_epoch: null out");
  if (d->first_epoch_start) {
    SRT_REQUIRE(d->num_proced_sample_of_epoch == d->dataset_size,
                "next_epoch: %d of %d samples processed", d->num_proced_sample_of_epoch, d->dataset_size);
    SRT_REQUIRE(d->num_proced_global_batches == d->num_global_batches_per_epoch,
                "next_epoch: %d of %d global batches processed", d->num_proced_global_batches,
                d->num_global_batches_per_epoch);
  } else {
    d->first_epoch_start = true;
  }
  *epoch = d->next_epoch_idx++;
  d->num_proced_global_batches = 0;
  d->num_proced_sample_of_epoch = 0;
  return SRT_OK;
}

int srt_dbd_info(srt_dist* h, int which, int rank, int* out) {
  DBD_CHECK(h);
  Dist* d = (Dist*)h;
  SRT_REQUIRE(out != nullptr && rank >= 0 && rank < SRT_MAX_DEVICE_NUM, "dbd_info: bad argument");
  DistLayout* l = d->L();
  shm::Guard g(l->mu);
  switch (which) {
    case SRT_DBD_GLOBAL_BATCH_SIZE: *out = d->global_batch_size; break;
    case SRT_DBD_NUM_GLOBAL_BATCH_PER_EPOCH: *out = d->num_global_batches_per_epoch; break;
    case SRT_DBD_NUM_PROCED_GLOBAL_BATCH: *out = d->num_proced_global_batches; break;
    case SRT_DBD_NUM_UNPROC: *out = l->num_unproc; break;
    case SRT_DBD_NUM_PROCING: *out = l->num_procing; break;
    case SRT_DBD_NUM_PROCED: *out = l->num_proced; break;
    case SRT_DBD_RANK_UNPROC: *out = l->unproc_per_train[rank]; break;
    case SRT_DBD_RANK_PROCING: *out = l->procing_per_train[rank]; break;
    case SRT_DBD_RANK_PROCED: *out = l->proced_per_train[rank]; break;
    default: set_error("dbd_info: unknown item %d", which); return SRT_ERR_INVALID;
  }
  return SRT_OK;
}

int srt_dist_switch_flag(srt_dist* h, int which, int set, int value, int* out) {
  DIST_CHECK(h);
  SRT_REQUIRE(which == 0 || which == 1, "dist_switch_flag: unknown flag %d", which);
  DistLayout* l = ((Dist*)h)->L();
  shm::Guard g(l->sw_mu);
  if (set) l->sw_flag[which] = value ? 1 : 0;
  if (out) *out = l->sw_flag[which];
  return SRT_OK;
}

int srt_perf_record_thpt(srt_dist* h, int batch_size, double batch_time_ms) {
  DIST_CHECK(h);
  SRT_REQUIRE(batch_size > 0 && batch_time_ms > 0, "perf_record: batch size and time must be positive");
  DistLayout* l = ((Dist*)h)->L();
  const double thpt = (double)batch_size / batch_time_ms;
  shm::Guard g(l->perf_mu);
  int i = 0;
  while (i < l->perf_n && l->perf[i].bs < batch_size) ++i;
  if (i < l->perf_n && l->perf[i].bs == batch_size) {
    PerfEntry& e = l->perf[i];
    e.thpt = (e.thpt * e.count + thpt) / (e.count + 1);
    e.count++;
    return SRT_OK;
  }
  SRT_REQUIRE(l->perf_n < kPerfCap, "perf_record: table is full");
  memmove(&l->perf[i + 1], &l->perf[i], sizeof(PerfEntry) * (size_t)(l->perf_n - i));
  l->perf[i] = {batch_size, thpt, 1};
  l->perf_n++;
  return SRT_OK;
}

int srt_perf_get_thpt(srt_dist* h, int batch_size, double* thpt) {
  DIST_CHECK(h);
  SRT_REQUIRE(thpt != nullptr, "perf_get: null out");
  DistLayout* l = ((Dist*)h)->L();
  if (batch_size <= 0) { *thpt = 0; return SRT_OK; }
  shm::Guard g(l->perf_mu);
  *thpt = perf_get_locked(l, batch_size);
  return SRT_OK;
}

}  // extern "C"
