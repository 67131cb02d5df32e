"""CPU restatement of the reference's integer / host arithmetic on the control path. TEST
INFRASTRUCTURE ONLY: never imported by the product.

Each function follows the cited reference code literally (plain Python ints / floats), so the C++
runtime can be compared with it on random inputs. The reference has no tests or golden vectors for
these functions, so PARITY IS UNPINNED here: the comparison is restatement against restatement
by independent code paths, anchored on the reference's source text only.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple


# ---- common/sm_partition.cc:78-112 -------------------------------------------------------------
def train_avail_tpc_mask(infer_required: int, gpu_tpc: int, min_train: int = 5, max_train: Optional[int] = None) -> int:
    max_train = gpu_tpc if max_train is None else min(max_train, gpu_tpc)
    min_train = max(min_train, 1)
    n = infer_required
    if n == 0:
        return 0
    n = min(n, gpu_tpc - min_train)
    n = max(n, gpu_tpc - max_train)
    return (1 << n) - 1 if n > 0 else 0


def train_avail_tpc_num(infer_required: int, gpu_tpc: int, min_train: int = 5, max_train: Optional[int] = None) -> int:
    max_train = gpu_tpc if max_train is None else min(max_train, gpu_tpc)
    min_train = max(min_train, 1)
    return min(max(min_train, gpu_tpc - infer_required), max_train)


# ---- pytorch/torch_col/csrc/perf_model.cc:25-95 -------------------------------------------------
class PerfModel:
    def __init__(self):
        self.table: Dict[int, Tuple[float, int]] = {}

    def record(self, bs: int, batch_time_ms: float):
        thpt = bs / batch_time_ms
        if bs not in self.table:
            self.table[bs] = (thpt, 1)
        else:
            t, c = self.table[bs]
            self.table[bs] = ((t * c + thpt) / (c + 1), c + 1)

    def get(self, bs: int) -> float:
        if bs <= 0:
            return 0
        if not self.table:
            return -1
        keys = sorted(self.table)
        lo, hi = keys[0], keys[-1]
        if lo >= bs:
            return self.table[lo][0] / lo * bs
        if hi <= bs:
            return self.table[hi][0] / hi * bs
        nxt = min(k for k in keys if k >= bs)
        if nxt == bs:
            return self.table[bs][0]
        prv = max(k for k in keys if k < bs)
        return (self.table[nxt][0] - self.table[prv][0]) / (nxt - prv) * (bs - prv) + self.table[prv][0]


# ---- pytorch/torch_col/csrc/dynamic_batch.cc:254-314 ---------------------------------------------
def distribute_batch(policy: str, num_unproc: int, perf: Optional[List[float]], n_workers: int) -> List[int]:
    if policy in ('fix', 'simple'):
        per, rem = divmod(num_unproc, n_workers)
        return [per + (1 if i < rem else 0) for i in range(n_workers)]
    s = sum(perf)
    out = []
    for i in range(n_workers):
        ratio = 1.0 / n_workers if s == 0 else perf[i] / s
        out.append(max(1, int(num_unproc * ratio)))
    diff = num_unproc - sum(out)
    i = 0
    while diff != 0:
        if i >= n_workers:
            i = 0
        if diff > 0:
            out[i] += 1
            diff -= 1
        elif out[i] > 1:
            out[i] -= 1
            diff += 1
        i += 1
    return out


# ---- server/train_adjuster.cc ------------------------------------------------------------------
MODEL_MEM_PARAM = {'resnet152': (1150, 85), 'swin_b': (1700, 145), 'swin_b_ddp': (2560, 140), 'gpt2': (2700, 490),
                   'qwen': (9000, 600)}  # :642-698


class TrainAdjuster:
    def __init__(self, base, slope, targets: List[int], init_bs: int, batch_size_limit=0, enable_balance=False,
                 balance_threshold=1500.0, num_visible_gpu=1, use_shared_tensor=True):
        self.base, self.slope = base, slope
        self.t = list(targets)
        self.init_bs = init_bs
        self.limit, self.balance, self.thr = batch_size_limit, enable_balance, balance_threshold
        self.ngpu, self.shared = num_visible_gpu, use_shared_tensor

    def predict_mem(self, bs): return self.base if bs <= 0 else self.base + self.slope * bs            # :83-96
    def predict_target_bs(self, mem): return max(min(int((mem - self.base) / self.slope), self.init_bs), 0)  # :521-533
    def delta_bs(self, mem): return int(math.ceil(mem / self.slope))                                    # :535-538

    def imbalance(self, bs, avail):                                                                       # :552-584
        if not self.balance or avail is None:
            return False
        return max(max(0.0, a - self.predict_mem(bs)) for a in avail) > self.thr

    def require(self, dev: int, required_mb: float, avail=None) -> List[int]:                             # :97-212
        cur = self.t[dev]
        if cur <= self.limit or required_mb <= 0:
            return []
        target = cur - self.delta_bs(required_mb)
        if self.ngpu > 1:
            target = max(target, self.limit)
        world = len(self.t)
        all_same = all(x == cur for x in self.t)
        one = lambda bs: [bs if r == dev else self.t[r] for r in range(world)]
        if all_same:
            plan = one(target) if target > 0 and self.imbalance(target, avail) else [target] * world
        else:
            mn = min(target if r == dev else self.t[r] for r in range(world))
            plan = one(mn) if mn > 0 and self.imbalance(mn, avail) else [target] * world
        self.t = list(plan)
        return plan

    def release(self, avail_mb, free_mb, reserve_mb) -> List[int]:                                        # :214-340
        world = len(self.t)
        targets, amr = [], []
        for r in range(world):
            a, f, cur = max(avail_mb[r], 0.0), max(free_mb[r], 0.0), self.t[r]
            amr.append(max(a - reserve_mb[r], 0.0))
            if self.shared:
                by_avail = self.predict_target_bs(max(a - reserve_mb[r], 0.0))
                by_delta = cur + self.delta_bs(max(f - reserve_mb[r], 0.0))
                targets.append(max(cur, min(by_avail, by_delta)))
            else:
                targets.append(max(cur, cur + self.delta_bs(f)))
        mn = min(targets)
        plan = [mn] * world if mn <= 0 or not self.imbalance(mn, amr) else targets
        self.t = list(plan)
        return plan

    # GetLLMInferRequireMemAdjustPlan (:435-519). train_avail_mb = what training could still use once the requirement
    # is met (free pages + its own pages - margin - requirement), as the function computes it from the pool.
    # With LLM serving the reference's CheckImbalance ends the server, so balance must be off.
    def llm_require(self, dev: int, required_mb: float, train_avail_mb: float) -> List[int]:
        cur = self.t[dev]
        if cur <= 0 or required_mb <= 0:
            return []
        by_avail = self.predict_target_bs(max(train_avail_mb, 0.0))
        by_required = cur - self.delta_bs(required_mb)
        target = max(0, min(by_avail, by_required))
        assert all(x == cur for x in self.t), "LOG(FATAL): Not supported"
        assert not self.balance, "LOG(FATAL): Not supported for LLM"
        self.t = [target] * len(self.t)
        return list(self.t)

    # GetLLMInferReleaseMemAdjustPlan (:342-433). free_mb / train_avail_mb per device as computed there from the pool.
    def llm_release(self, train_avail_mb, free_mb) -> List[int]:
        assert not self.balance, "LOG(FATAL): Not supported for LLM"
        targets = []
        for r, cur in enumerate(self.t):
            by_avail = self.predict_target_bs(max(train_avail_mb[r], 0.0))
            by_delta = cur + self.delta_bs(max(free_mb[r], 0.0))
            targets.append(max(cur, min(by_avail, by_delta)))
        self.t = [min(targets)] * len(self.t)
        return list(self.t)


# ---- pytorch/torch_col/csrc/dynamic_batch.cc:144-252, 316-573, 640-733 ---------------------------
class Ledger:
    """The DynamicBatchDistirbutor's shared state and the per-rank counters of every rank, in one object (the C++
    keeps the former in shared memory and the latter in each process). Sample ranges are half-open pairs kept in sets
    ordered by (first, second), as the reference's boost sets of pairs are. Every CHECK of the reference is an
    AssertionError here."""

    def __init__(self, world: int, dataset_size: int, input_batch_size: int, global_batch_size: int, lazy: bool,
                 policy: str, perf: Optional[PerfModel] = None):
        self.world, self.dataset_size, self.input_bs, self.gbs = world, dataset_size, input_batch_size, global_batch_size
        self.lazy, self.policy, self.perf = lazy, policy, perf or PerfModel()
        self.num_gb_per_epoch = (dataset_size + global_batch_size - 1) // global_batch_size       # :80-81
        init = -1 if lazy else 0                                                                    # :131-141
        self.unproc_per, self.procing_per, self.proced_per = [init] * world, [init] * world, [init] * world
        self.has_unproc = [False] * world
        self.unproc, self.procing, self.proced = [], [], []            # sorted lists of (first, second)
        self.n_unproc = self.n_procing = self.n_proced = 0
        # per-process members (:76-79), one entry per rank
        self.num_proced_gb = [0] * world
        self.num_proced_sample_of_epoch = [0] * world
        self.next_epoch_idx = [0] * world
        self.first_epoch_start = [False] * world

    @staticmethod
    def _n(r): return r[1] - r[0]

    # DistributeBatchWithoutLock (:157-252); target_unpub = the board's unpublished targets, None without a server
    def distribute(self, check: bool, to_all: bool, at_begin: bool, target_unpub: Optional[List[int]] = None):
        do = not (self.lazy or (not at_begin and self.policy == 'fix'))
        if check and do:
            n = sum(self.unproc_per)
            assert n == self.n_unproc, (self.unproc_per, self.n_unproc)
        else:
            n = self.n_unproc
        if to_all:
            self.has_unproc = [True] * self.world
        if do:
            workers = [i for i in range(self.world) if self.has_unproc[i]]
            if workers:
                tbs = [target_unpub[i] if target_unpub is not None else self.input_bs for i in workers]
                if self.policy == 'by_performance' and n < len(workers):
                    # the reference's round-off loop cannot end here (every worker holds the minimum of one sample);
                    # the library gives the first n workers one sample each and takes the others out
                    for k, w in enumerate(workers):
                        self.unproc_per[w] = 1 if k < n else 0
                        if k >= n:
                            self.has_unproc[w] = False
                else:
                    share = distribute_batch(self.policy, n, [self.perf.get(b) for b in tbs], len(workers))
                    for w, s in zip(workers, share):
                        self.unproc_per[w] = s
            else:
                assert n == 0
        assert n >= 0

    # NextGlobalBatchImpl (:640-716), the master's part; the ranks' counters are read from rank 0's members
    def next_global_batch(self, target_unpub: Optional[List[int]] = None):
        cur = self.gbs
        if self.gbs + self.num_proced_sample_of_epoch[0] > self.dataset_size:
            cur = self.dataset_size - self.num_proced_sample_of_epoch[0]
        assert cur >= 0
        self.n_unproc, self.n_procing, self.n_proced = cur, 0, 0
        self.unproc, self.procing, self.proced = [], [], []
        if cur > 0:
            first = self.num_proced_sample_of_epoch[0]
            self.unproc = [(first, first + cur)]
            self.distribute(False, True, True, target_unpub)
            if not self.lazy:
                self.procing_per, self.proced_per = [0] * self.world, [0] * self.world
        elif not self.lazy:
            self.unproc_per, self.procing_per, self.proced_per = [0] * self.world, [0] * self.world, [0] * self.world

    # LazyDistributingGetBatchSize (:414-436)
    def _lazy_size(self, batch_size: int):
        ongoing = sum(self.has_unproc)
        assert ongoing > 0
        mx = self.n_unproc - ongoing + 1
        return (mx, True) if batch_size >= mx else (batch_size, False)

    # GetBatch (:316-412)
    def get_batch(self, rank: int, batch_size: int):
        if self.lazy:
            size, last = self._lazy_size(batch_size)
        else:
            size, last = min(batch_size, self.unproc_per[rank]), None
        got, out, i = 0, [], 0
        while got < size:
            assert i < len(self.unproc)
            r = self.unproc[i]
            if self._n(r) + got <= size:
                got += self._n(r)
                out.append(r)
                self.procing.append(r)
                del self.unproc[i]                           # the iterator moves to the next range
            else:
                head, rest = (r[0], r[0] + size - got), (r[0] + size - got, r[1])      # SliceBatchRange
                got += self._n(head)
                out.append(head)
                self.procing.append(head)
                self.unproc[i] = rest
                self.unproc.sort()
                i = self.unproc.index(rest)
        self.procing.sort()
        if not self.lazy:
            self.unproc_per[rank] -= got
            self.procing_per[rank] += got
            assert self.unproc_per[rank] >= 0
        self.n_unproc -= got
        self.n_procing += got
        assert self.n_unproc >= 0
        if not self.lazy:
            last = self.unproc_per[rank] == 0
        if last:
            self.has_unproc[rank] = False
        return out, last

    # QueryNextBatchSize (:438-459)
    def query_next_batch_size(self, rank: int, batch_size: int) -> int:
        return min(self.n_unproc if self.lazy else self.unproc_per[rank], batch_size)

    def _move(self, ranges, dst):
        n = 0
        for r in ranges:
            r = tuple(r)
            assert r in self.procing, r
            self.procing.remove(r)
            dst.append(r)
            n += self._n(r)
        dst.sort()
        return n

    # FinishBatch (:461-530)
    def finish_batch(self, rank: int, ranges, end_of_global_batch: bool):
        n = self._move(ranges, self.proced)
        if not self.lazy:
            self.procing_per[rank] -= n
            self.proced_per[rank] += n
        self.n_procing -= n
        self.n_proced += n
        if end_of_global_batch:
            assert self.lazy or self.procing_per[rank] == 0
            self.num_proced_gb[rank] += 1
            self.num_proced_sample_of_epoch[rank] = min(self.num_proced_sample_of_epoch[rank] + self.gbs, self.dataset_size)

    # AbortBatch (:532-573)
    def abort_batch(self, rank: int, ranges):
        n = self._move(ranges, self.unproc)
        if not self.lazy:
            self.procing_per[rank] -= n
            self.unproc_per[rank] += n
        self.n_procing -= n
        self.n_unproc += n

    # NextEpoch (:718-733)
    def next_epoch(self, rank: int) -> int:
        if self.first_epoch_start[rank]:
            assert self.num_proced_sample_of_epoch[rank] == self.dataset_size
            assert self.num_proced_gb[rank] == self.num_gb_per_epoch
        else:
            self.first_epoch_start[rank] = True
        e = self.next_epoch_idx[rank]
        self.next_epoch_idx[rank] += 1
        self.num_proced_gb[rank] = 0
        self.num_proced_sample_of_epoch[rank] = 0
        return e
