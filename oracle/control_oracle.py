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
