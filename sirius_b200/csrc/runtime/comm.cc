// inf_tra_comm: the shared-memory channel between the inference server and the trainers, and the
// SM-partition arithmetic that reads its TPC counters.
//
// Follows common/inf_tra_comm/{communicator,message_queue,shared_info}.* and common/sm_partition.cc
// of the reference: one queue per direction and rank plus a group condition for "get from any",
// an information board with one TrainInfo per rank and one InferInfo. The containers are
// fixed-capacity rings in a plain struct instead of Boost.Interprocess deques.
#include <pwd.h>
#include <stdlib.h>

#include <algorithm>
#include <string>

#include "../../../include/sirius_b200.h"
#include "../../../include/sirius_runtime.h"
#include "rt_common.h"
#include "shm_util.h"

namespace srt {
namespace {

constexpr uint32_t kCommMagic = 0x53434d31;  // "SCM1"
constexpr int kRingCap = 512;

struct Ring {
  shm::Mutex mu;
  shm::Cond cond;
  uint32_t head, count;
  srt_ctrl_msg slot[kRingCap];
};
struct Group {
  shm::Mutex mu;
  shm::Cond cond;
};
struct TpcData {  // SMPartitioner::TpcData
  std::atomic<int> infer_required_tpc_num;
  uint64_t infer_tpc_mask;
};
struct CommLayout {
  shm::SegHeader hdr;
  std::atomic<int> world_size;  // read by every getter and putter while a registering rank may raise it
  shm::Mutex shm_mutex;
  Ring q[2][SRT_MAX_DEVICE_NUM];
  Group group[2];
  shm::Mutex infer_mu;
  TpcData tpc[SRT_MAX_DEVICE_NUM];
  shm::Mutex train_mu[SRT_MAX_DEVICE_NUM];
  srt_train_info train[SRT_MAX_DEVICE_NUM];
};

}  // namespace

std::string default_shm_prefix() {
  const char* port = getenv("SIRIUS_PORT");
  const char* user = getenv("USER");
  std::string u = user ? user : "";
  if (u.empty()) {
    passwd* pw = getpwuid(getuid());
    u = pw ? pw->pw_name : std::to_string(getuid());
  }
  return "colserve_shm_" + u + "_p" + (port ? port : "8080");
}

struct Comm {
  shm::Segment<CommLayout> seg;
  bool is_server = false;
  CommLayout* L() { return seg.get(); }
};

static bool ring_pop(Ring& r, srt_ctrl_msg* out) {
  if (r.count == 0) return false;
  *out = r.slot[r.head];
  r.head = (r.head + 1) % kRingCap;
  r.count--;
  return true;
}

}  // namespace srt

using namespace srt;

#define COMM_CHECK(c, rank)                                                                      \
  SRT_REQUIRE((c) != nullptr && ((Comm*)(c))->L() != nullptr, "inf_tra_comm: not open");         \
  SRT_REQUIRE((rank) >= 0 && (rank) < SRT_MAX_DEVICE_NUM, "inf_tra_comm: rank %d out of range", (int)(rank))

extern "C" {

int srt_comm_open(const char* name, int is_server, int cleanup, int train_world_size, int timeout_ms,
                  srt_comm** out) {
  SRT_REQUIRE(out != nullptr, "comm_open: null out");
  SRT_REQUIRE(train_world_size >= 0 && train_world_size <= SRT_MAX_DEVICE_NUM, "comm_open: world size %d",
              train_world_size);
  Comm* c = new Comm();
  c->is_server = is_server != 0;
  const std::string nm = name ? std::string(name) : default_shm_prefix() + "_inf_tra_comm";
  std::string err;
  bool ok;
  if (is_server) {
    ok = c->seg.create(nm, kCommMagic, cleanup != 0, [&](CommLayout* l) {
      l->world_size = train_world_size;
      l->shm_mutex.init();
      for (int d = 0; d < 2; ++d) {
        for (int i = 0; i < SRT_MAX_DEVICE_NUM; ++i) { l->q[d][i].mu.init(); l->q[d][i].cond.init(); }
        l->group[d].mu.init();
        l->group[d].cond.init();
      }
      l->infer_mu.init();
      for (int i = 0; i < SRT_MAX_DEVICE_NUM; ++i) {
        l->train_mu[i].init();
        l->train[i].train_pid = -1;
        l->tpc[i].infer_required_tpc_num.store(0);
      }
    }, &err);
  } else {
    ok = c->seg.open(nm, kCommMagic, timeout_ms, &err);
  }
  if (!ok) {
    set_error("inf_tra_comm: %s", err.c_str());
    delete c;
    return SRT_ERR_STATE;
  }
  if (!is_server && train_world_size > 0) {
    int none = 0;
    c->L()->world_size.compare_exchange_strong(none, train_world_size, std::memory_order_relaxed);
  }
  *out = (srt_comm*)c;
  return SRT_OK;
}

int srt_comm_close(srt_comm* h) {
  Comm* c = (Comm*)h;
  if (!c) return SRT_OK;
  if (c->is_server) c->seg.unlink();  // the reference's server removes the segment on exit
  delete c;
  return SRT_OK;
}

int srt_comm_world_size(srt_comm* h) {
  Comm* c = (Comm*)h;
  return c && c->L() ? c->L()->world_size.load(std::memory_order_relaxed) : -1;
}

int srt_comm_put(srt_comm* h, const srt_ctrl_msg* msg, int direction, int rank) {
  COMM_CHECK(h, rank);
  SRT_REQUIRE(msg && (direction == 0 || direction == 1), "comm_put: bad argument");
  CommLayout* l = ((Comm*)h)->L();
  Ring& r = l->q[direction][rank];
  {
    shm::Guard g(r.mu);
    SRT_REQUIRE(r.count < (uint32_t)kRingCap, "comm_put: queue %d/%d is full", direction, rank);
    r.slot[(r.head + r.count) % kRingCap] = *msg;
    r.count++;
    r.cond.notify_one();
  }
  shm::Guard gg(l->group[direction].mu);
  l->group[direction].cond.notify_all();
  return SRT_OK;
}

int srt_comm_put_all(srt_comm* h, const srt_ctrl_msg* msgs, int n, int direction) {
  COMM_CHECK(h, 0);
  CommLayout* l = ((Comm*)h)->L();
  const int world = l->world_size.load(std::memory_order_relaxed);
  SRT_REQUIRE(msgs && (n == 1 || n == world), "comm_put_all: need 1 or %d messages, got %d", world, n);
  for (int i = 0; i < world; ++i) {
    int rc = srt_comm_put(h, &msgs[n == 1 ? 0 : i], direction, i);
    if (rc) return rc;
  }
  return SRT_OK;
}

int srt_comm_timed_get(srt_comm* h, int timeout_ms, int direction, int rank, srt_ctrl_msg* out, int* got) {
  COMM_CHECK(h, rank);
  SRT_REQUIRE(out && got && (direction == 0 || direction == 1), "comm_get: bad argument");
  Ring& r = ((Comm*)h)->L()->q[direction][rank];
  shm::Guard g(r.mu);
  *got = 0;
  if (timeout_ms != 0 && r.count == 0) {
    if (timeout_ms < 0) {
      while (r.count == 0) r.cond.wait(r.mu);
    } else {
      const timespec dl = shm::deadline_after_ms(timeout_ms);
      while (r.count == 0)
        if (!r.cond.wait_until(r.mu, dl)) break;
    }
  }
  if (ring_pop(r, out)) *got = 1;
  return SRT_OK;
}

int srt_comm_timed_get_from_any(srt_comm* h, int timeout_ms, int direction, int* rank, srt_ctrl_msg* out,
                                int* got) {
  COMM_CHECK(h, 0);
  SRT_REQUIRE(rank && out && got && (direction == 0 || direction == 1), "comm_get_from_any: bad argument");
  CommLayout* l = ((Comm*)h)->L();
  *got = 0;
  const timespec dl = shm::deadline_after_ms(timeout_ms < 0 ? 0 : timeout_ms);
  Group& grp = l->group[direction];
  shm::Guard gg(grp.mu);
  for (;;) {
    const int world = l->world_size.load(std::memory_order_relaxed);
    for (int i = 0; i < world; ++i) {
      Ring& r = l->q[direction][i];
      shm::Guard g(r.mu);
      if (ring_pop(r, out)) { *rank = i; *got = 1; return SRT_OK; }
    }
    if (timeout_ms == 0) return SRT_OK;
    if (timeout_ms < 0) grp.cond.wait(grp.mu);
    else if (!grp.cond.wait_until(grp.mu, dl)) {
      // one last look: a put between the scan and the wait only signals the group condition
      for (int i = 0; i < l->world_size.load(std::memory_order_relaxed); ++i) {
        Ring& r = l->q[direction][i];
        shm::Guard g(r.mu);
        if (ring_pop(r, out)) { *rank = i; *got = 1; return SRT_OK; }
      }
      return SRT_OK;
    }
  }
}

int srt_comm_clear(srt_comm* h) {
  COMM_CHECK(h, 0);
  CommLayout* l = ((Comm*)h)->L();
  for (int d = 0; d < 2; ++d)
    for (int i = 0; i < SRT_MAX_DEVICE_NUM; ++i) {
      shm::Guard g(l->q[d][i].mu);
      l->q[d][i].head = l->q[d][i].count = 0;
    }
  return SRT_OK;
}

int srt_comm_set_train_info(srt_comm* h, int rank, const srt_train_info* info) {
  COMM_CHECK(h, rank);
  SRT_REQUIRE(info != nullptr, "set_train_info: null info");
  CommLayout* l = ((Comm*)h)->L();
  shm::Guard g(l->train_mu[rank]);
  l->train[rank] = *info;
  l->train[rank].model_name[255] = 0;
  int cur = l->world_size.load(std::memory_order_relaxed);   // only ever raised
  while (cur < info->train_world_size &&
         !l->world_size.compare_exchange_weak(cur, info->train_world_size, std::memory_order_relaxed)) {}
  return SRT_OK;
}

int srt_comm_get_train_info(srt_comm* h, int rank, srt_train_info* out) {
  COMM_CHECK(h, rank);
  SRT_REQUIRE(out != nullptr, "get_train_info: null out");
  CommLayout* l = ((Comm*)h)->L();
  shm::Guard g(l->train_mu[rank]);
  *out = l->train[rank];
  return SRT_OK;
}

static int* train_field(srt_train_info& t, int field) {
  switch (field) {
    case SRT_TI_PID: return &t.train_pid;
    case SRT_TI_RANK: return &t.train_rank;
    case SRT_TI_WORLD_SIZE: return &t.train_world_size;
    case SRT_TI_INIT_BS: return &t.init_batch_size;
    case SRT_TI_CURRENT_BS: return &t.current_batch_size;
    case SRT_TI_TARGET_BS: return &t.target_batch_size;
    case SRT_TI_TARGET_BS_UNPUBLISHED: return &t.target_batch_size_unpublished;
    case SRT_TI_FIRST_EPOCH_DONE: return &t.first_epoch_done;
    default: return nullptr;
  }
}

int srt_comm_update_train_field(srt_comm* h, int rank, int field, int value) {
  COMM_CHECK(h, rank);
  CommLayout* l = ((Comm*)h)->L();
  shm::Guard g(l->train_mu[rank]);
  int* p = train_field(l->train[rank], field);
  SRT_REQUIRE(p != nullptr, "update_train_field: unknown field %d", field);
  // the reference CHECKs validity before touching a field (shared_info.h:196-210)
  SRT_REQUIRE(field == SRT_TI_PID || l->train[rank].train_pid != -1, "train info of rank %d is not valid", rank);
  *p = value;
  return SRT_OK;
}

int srt_comm_get_train_field(srt_comm* h, int rank, int field, int* out) {
  COMM_CHECK(h, rank);
  SRT_REQUIRE(out != nullptr, "get_train_field: null out");
  CommLayout* l = ((Comm*)h)->L();
  shm::Guard g(l->train_mu[rank]);
  int* p = train_field(l->train[rank], field);
  SRT_REQUIRE(p != nullptr, "get_train_field: unknown field %d", field);
  SRT_REQUIRE(field == SRT_TI_PID || l->train[rank].train_pid != -1, "train info of rank %d is not valid", rank);
  *out = *p;
  return SRT_OK;
}

int srt_comm_invalidate_train_info(srt_comm* h, int rank) {
  COMM_CHECK(h, rank);
  CommLayout* l = ((Comm*)h)->L();
  shm::Guard g(l->train_mu[rank]);
  l->train[rank].train_pid = -1;
  return SRT_OK;
}

int srt_comm_infer_tpc(srt_comm* h, int device, int op, int value, int* out) {
  COMM_CHECK(h, device);
  std::atomic<int>& n = ((Comm*)h)->L()->tpc[device].infer_required_tpc_num;
  int v;
  switch (op) {
    case 0: n.store(value, std::memory_order_relaxed); v = value; break;
    case 1: v = n.fetch_add(value, std::memory_order_relaxed) + value; break;
    case 2: v = n.fetch_sub(value, std::memory_order_relaxed) - value; break;
    case 3: v = n.load(std::memory_order_relaxed); break;
    default: set_error("infer_tpc: unknown op %d", op); return SRT_ERR_INVALID;
  }
  if (out) *out = v;
  return SRT_OK;
}

// ---- SM partition arithmetic (SMPartitioner::GetTrainAvailTpcMask / GetTrainAvailTpcNum) ----
static int clamp_disabled(int required, int gpu_tpc, int min_train, int max_train) {
  if (min_train < 1) min_train = 1;
  if (max_train > gpu_tpc) max_train = gpu_tpc;
  int n = required;
  if (n <= 0) return 0;
  n = std::min(n, gpu_tpc - min_train);  // never starve training completely
  n = std::max(n, gpu_tpc - max_train);
  return n;
}

uint64_t srt_smp_train_avail_tpc_mask(int infer_required_tpc, int gpu_tpc_num, int min_train_tpc,
                                      int max_train_tpc) {
  const int n = clamp_disabled(infer_required_tpc, gpu_tpc_num, min_train_tpc, max_train_tpc);
  if (n <= 0) return 0;
  return n >= 64 ? ~0ull : ((1ull << n) - 1);  // set bit = TPC disabled; training keeps the high TPCs
}

int srt_smp_train_avail_tpc_num(int infer_required_tpc, int gpu_tpc_num, int min_train_tpc, int max_train_tpc) {
  if (min_train_tpc < 1) min_train_tpc = 1;
  if (max_train_tpc > gpu_tpc_num) max_train_tpc = gpu_tpc_num;
  int res = std::max(min_train_tpc, gpu_tpc_num - std::max(infer_required_tpc, 0));
  return std::min(res, max_train_tpc);
}

int srt_smp_allowed_sm_mask(int infer_required_tpc, int gpu_sm_num, int min_train_tpc, int max_train_tpc,
                            uint64_t allowed_sm[3]) {
  SRT_REQUIRE(allowed_sm != nullptr && gpu_sm_num > 0 && gpu_sm_num <= 192, "allowed_sm_mask: bad argument");
  const int gpu_tpc = gpu_sm_num / 2;
  const int n = clamp_disabled(infer_required_tpc, gpu_tpc, min_train_tpc, max_train_tpc);
  allowed_sm[0] = allowed_sm[1] = allowed_sm[2] = 0;
  for (int sm = 2 * n; sm < gpu_sm_num; ++sm) allowed_sm[sm >> 6] |= 1ull << (sm & 63);
  return SRT_OK;
}

}  // extern "C"
