#!/usr/bin/env python
"""Headline benchmark: ResNet-152 training step, bf16, batch 64 per GPU, 224x224 synthetic images.

    python bench.py [--gpus N] [--steps K] [--warmup W]            # this repo's CUDA step
    python bench.py --impl reference [--gpus N] [--steps K] ...    # the reference's CPU path

One JSON line on stdout (rank 0). `value` is samples/s with the batch already in HBM; `e2e` is the
same step driven through the public API from pinned host buffers (H2D of the batch and D2H of the
loss inside the timed region). Both are the median of three timed regions of exactly K steps each
(`timed_regions_ms`), CUDA events on the step's stream, max over ranks. `roofline` describes the
kernel family that takes the most device time, timed with CUDA events on the step's stream in a
separate profiled pass; its `traffic` is that family's DRAM bytes per kernel launch from an ncu
capture of a whole step. `kernel_families` carries the same for every family.

Additions to the line, run after the headline numbers exist and under a time budget
(`--extras-budget`; a leg that has not finished by then is left out and the line is printed anyway):
`handover.unmap_on_release` (release / regain of the activation pages with the reference's
unmap-at-release, beside the kept-mapping default), `workloads` (Swin-B batch 32 and GPT-2 small
8 x 1024 at the same number of GPUs), `colocated` (N = 1: training next to an inference server in a
second process, every request a memory handover and an SM-mask shrink for 30 s at 50 req/s, and the
same with pages kept until the server idles), `cpu_baseline` (the CPU oracle: stock torchvision /
PyTorch fp32, the reference's arithmetic path, timed on this box's host cores on a bounded sample).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

ARCH, BATCH, IMAGE, CLASSES = "resnet152", 64, 224, 1000
POOL_GB = 12.0            # COLTRAIN_SHARED_TENSOR_POOL_GB default of the reference (config.cc:57-69)
FLOP_PER_SAMPLE = 68.85e9  # forward + backward, 2 FLOP per MAC (torch.utils.flop_counter on the CPU model)
METRIC, UNIT = "train samples/s", "samples/s"
# DRAM bytes per launch by kernel family (dram__bytes_read.sum + dram__bytes_write.sum of every kernel of the family in
# one training step, divided by the family's launches): the one-pass ncu capture of a whole step summarised in
# profiles/resnet152_bf16_b64_step_launch_list.md. A benchmark run cannot be profiled while it is timed, so these are
# constants of that capture; they change when the kernels do.
DRAM_BYTES_PER_LAUNCH = {"batchnorm": 23500512, "conv_fprop_dgrad": 24757257, "conv_wgrad": 27412543,
                         "optimizer": 8842468, "other": 32372448}
KERNEL_LAUNCHES_PER_STEP = {"batchnorm": 609, "conv_fprop_dgrad": 310, "conv_wgrad": 266, "optimizer": 157, "other": 8}
REGIONS = 3               # timed regions per number; the median is reported
WORKLOAD = "ResNet-152 train step (fwd+bwd+SGD-momentum), bf16, batch 64 per GPU, 3x224x224 N(0,1)"


def load_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "tflops": float(p["bf16_tflops_sustained"]), "source": "measured"}
    except Exception:
        return {"hbm_gbs": 6650.0, "tflops": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        try:
            sm, mx, reasons = [], [], set()
            names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                sm.append(float(f[1])); mx.append(float(f[2]))
                for n, v in zip(names, f[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            if sm:
                sm.sort()
                out = {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                       "samples": len(sm)}
        except Exception:
            pass
        finally:
            try:
                os.unlink(self.path)
            except Exception:
                pass
        return out


def seeded_state(arch):
    """Random-init weights of the named architecture (seeded Kaiming init as torchvision does)."""
    import torch
    from torchvision.models.resnet import Bottleneck, ResNet
    from sirius_b200.step import RESNET_LAYERS
    torch.manual_seed(0)
    m = ResNet(Bottleneck, list(RESNET_LAYERS[arch]), num_classes=CLASSES)
    return {k: v for k, v in m.state_dict().items() if not k.endswith("num_batches_tracked")}


class _DevBuf:
    def __init__(self, ptr, n):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": "<f4", "data": (ptr, False), "version": 2}


def run_ours(args):
    import torch
    import torch.distributed as dist
    from sirius_b200 import _lib
    from sirius_b200.step import ResNetStep

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    # The headline part takes well under a minute. If it has not finished after fifteen, something on the device has
    # stopped making progress: every thread's stack goes to stderr and the process ends, which releases the device
    # (re-armed with the additions' own limit further down).
    import faulthandler
    faulthandler.dump_traceback_later(900.0, exit=True)
    torch.cuda.set_device(local)
    if world > 1:
        import datetime
        # a short collective timeout: a mismatch between ranks must fail in minutes, not hang the box
        dist.init_process_group("nccl", device_id=torch.device("cuda", local),
                                timeout=datetime.timedelta(seconds=120))

    # activations come from the training allocator of a page pool (CUDA VMM), as in the colocated setup
    from sirius_b200.pool import PagePool
    pool = PagePool(POOL_GB, device=local)
    step = ResNetStep(arch=ARCH, num_classes=CLASSES, max_batch=BATCH, image=IMAGE, dtype="bf16", pool=pool.handle)
    step.load_state_dict(seeded_state(ARCH))
    stream = torch.cuda.ExternalStream(step.stream)

    g = torch.Generator().manual_seed(1000 + rank)
    nbuf = 2  # distinct host batches, cycled
    host = [(torch.randn(BATCH, 3, IMAGE, IMAGE, generator=g).pin_memory(),
             torch.randint(0, CLASSES, (BATCH,), generator=g).pin_memory()) for _ in range(nbuf)]
    dev = [(im.cuda(), lb.cuda()) for im, lb in host]
    torch.cuda.synchronize()
    global_bs = BATCH * world

    # Gradient exchange overlapped with backward, inside the library: forward_backward returns once everything is
    # enqueued (the GPU is then still early in backward); begin() enqueues one NCCL all-reduce per gradient bucket
    # on the library's communication stream, each behind the event the executor records when that bucket's
    # gradients are final; wait() puts the optimizer behind the last one. bf16 on the wire (2 bytes per parameter).
    exchange = None
    if world > 1:
        from sirius_b200.ddp import GradExchange
        exchange = GradExchange(rank, world, device=local, wire=args.wire, max_ctas=args.nccl_max_ctas)
        step.forward_backward(BATCH, BATCH * world)   # communicator warm-up (pytorch/torch_col/__init__.py:61-64)
        exchange.allreduce(step)
        step.synchronize()

    def allreduce():
        if exchange is not None:
            exchange.begin(step)
            exchange.wait(step)

    def step_resident(i):
        im, lb = dev[i % nbuf]
        step.set_batch_device(im.data_ptr(), lb.data_ptr(), BATCH)
        step.forward_backward(BATCH, global_bs)
        allreduce()
        step.optimizer_step()

    def step_e2e(i):
        # the batch of this step was uploaded during the previous one (the loader's prefetch: pinned memory and an
        # asynchronous copy on the step's copy stream); every step issues exactly one upload, that of its successor
        step.forward_backward(BATCH, global_bs)
        im, lb = host[(i + 1) % nbuf]
        step.upload_batch(im, lb)
        allreduce()
        step.optimizer_step()
        return step.loss()  # D2H of the step's result, synchronises (loss.item() in the reference loop)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, k):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(k):
            fn(i)
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for i in range(max(args.warmup, 3)):
        step_resident(i)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    # Three timed regions of exactly `steps` steps each; the reported one is the median (a single region of a
    # few tenths of a second is at the mercy of one slow collective or one host hiccup).
    launches0 = _lib.lib().srt_launch_count()
    regions = [timed(step_resident, args.steps) for _ in range(REGIONS)]
    launches = (_lib.lib().srt_launch_count() - launches0) // REGIONS
    ms = sorted(regions)[REGIONS // 2]
    value = global_bs * args.steps / (ms / 1e3)

    step.upload_batch(*host[0])
    step_e2e(0)
    regions_e2e = [timed(step_e2e, args.steps) for _ in range(REGIONS)]
    clocks = sampler.stop() if rank == 0 else {}
    ms_e2e = sorted(regions_e2e)[REGIONS // 2]
    e2e = global_bs * args.steps / (ms_e2e / 1e3)

    # ---- per-kernel-family device time (separate profiled pass, not part of `value`) ----
    prof_steps = min(args.steps, 5)
    step.profile(True)
    for i in range(prof_steps):
        step_resident(i)
    prof = step.profile_read()
    step.profile(False)
    from sirius_b200 import ops
    status = ops.tc_status()

    # ---- memory handover: give the activation pages back to the pool, then regain them ----
    def time_handover(st, pl):
        rel_ms, regain_ms, nbytes = [], [], 0
        t_leg = time.perf_counter()
        for _ in range(3):
            if rel_ms and time.perf_counter() - t_leg > 20.0:
                break   # driver map/unmap calls occasionally take seconds each on a shared host: one sample is kept
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            nbytes = st.release_activations()      # sync + free blocks + pages marked FREE (unmapped in mpool mode)
            t1 = time.perf_counter()
            st.reserve_activations(BATCH)          # pages taken again for the same batch size
            t2 = time.perf_counter()
            rel_ms.append((t1 - t0) * 1e3)
            regain_ms.append((t2 - t1) * 1e3)
        torch.cuda.synchronize()
        gib = nbytes / 2 ** 30
        return {"released_gib": round(gib, 3), "release_ms": round(min(rel_ms), 3),
                "release_ms_median": round(sorted(rel_ms)[len(rel_ms) // 2], 3), "repeats": len(rel_ms),
                "release_ms_per_gib": round(min(rel_ms) / gib, 4), "regain_ms": round(min(regain_ms), 3),
                "page_mib": pl.stat("page_nbytes") >> 20}

    handover = None
    if rank == 0:
        handover = time_handover(step, pool)
        handover["what"] = ("srt_step_release_activations: stream sync, free of the activation set, every emptied page "
                            "marked FREE for the inference allocator; the pool keeps the old mapping of a released page "
                            "and reuses it, so no driver call is made")
    step.close()
    pool.close()

    peaks = load_peaks()
    fam = {}
    for name, d in prof.items():
        if d["launches"] == 0:
            continue
        sec = d["ms"] / 1e3
        tensor = name.startswith("conv")
        ach = d["work"] / sec / (1e12 if tensor else 1e9)
        peak = peaks["tflops"] if tensor else peaks["hbm_gbs"]
        fam[name] = {"bound": "tensor" if tensor else "hbm", "achieved": round(ach, 2), "peak": peak,
                     "unit": "TFLOP/s" if tensor else "GB/s", "frac": round(ach / peak, 4),
                     "ms_per_step": round(d["ms"] / prof_steps, 3), "launches_per_step": d["launches"] // prof_steps,
                     # per kernel launch of the family (an operator call of the profiled pass may be two or three
                     # kernels), so that both figures have the unit of the ncu capture
                     "algorithmic_per_launch": round(d["work"] / prof_steps / KERNEL_LAUNCHES_PER_STEP.get(name, d["launches"] // prof_steps)),
                     "traffic": DRAM_BYTES_PER_LAUNCH.get(name)}
    top = max(fam, key=lambda k: fam[k]["ms_per_step"]) if fam else None
    roofline = None
    if top:
        roofline = {k: fam[top][k] for k in ("bound", "achieved", "peak", "unit", "frac")}
        roofline.update({"kernel": top, "traffic": fam[top]["traffic"],
                         "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum per launch, whole-step capture "
                                           "(profiles/resnet152_bf16_b64_step_launch_list.md)",
                         "peak_source": f"of {peaks['source']}"})

    out = {
        "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(ms / args.steps, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "global_batch": global_bs, "per_gpu_batch": BATCH,
                   "parallelism": f"dp{world}", "optimizer": "SGD lr 0.1 momentum 0.9 wd 1e-4",
                   "init": "seeded Kaiming (no pretrained weights)",
                   "l2": "working set per step (activations of 64 images, several GB) exceeds the 126 MB L2"},
        "e2e": {"value": round(e2e, 2), "unit": UNIT,
                "h2d_bytes_per_step": BATCH * 3 * IMAGE * IMAGE * 4 + BATCH * 8, "d2h_bytes_per_step": 4,
                "ms_per_step": round(ms_e2e / args.steps, 3)},
        "gpu_launches": int(launches),
        "timed_regions_ms": {"resident": [round(x, 3) for x in regions], "e2e": [round(x, 3) for x in regions_e2e],
                             "reported": "median"},
        "clocks": clocks,
        "roofline": roofline,
        "kernel_families": fam,
        "model_flops_frac": round(value / world * FLOP_PER_SAMPLE / (peaks["tflops"] * 1e12), 4),
        "tc_status": status,
        "handover": handover,
    }
    # Everything below adds to the line and is not needed for the headline numbers: it runs in a worker thread under a
    # time budget, so that a slow leg (driver map/unmap calls on a shared host have been seen to take seconds each,
    # a colocation run spawns a second process) cannot keep the line from being printed.
    def extras():
        if rank == 0 and world == 1:
            # the same handover the way the reference's mpool does it: cuMemUnmap at release, cuMemMap at regain
            pool2 = PagePool(POOL_GB, device=local, unmap_on_release=True)
            step2 = ResNetStep(arch=ARCH, num_classes=CLASSES, max_batch=BATCH, image=IMAGE, dtype="bf16",
                               pool=pool2.handle)
            handover["unmap_on_release"] = time_handover(step2, pool2)
            step2.close()
            pool2.close()
        if args.other_workloads:
            # the other configurations the metric is defined on, at the same number of GPUs, a few steps each
            short = argparse.Namespace(**{**vars(args), "steps": max(3, min(args.steps, 10)), "warmup": 3})
            wl = {}
            out["workloads"] = wl
            for name, fn in (("swin_b", lambda: run_swin(short, embedded=True)),
                             ("gpt2", lambda: run_lm(short, "gpt2", embedded=True))):
                try:
                    wl[name] = fn()
                except Exception as e:  # noqa: BLE001  (the headline number stands on its own)
                    wl[name] = {"error": f"{type(e).__name__}: {e}"[:300]}
        if rank == 0 and world == 1 and args.colocate_seconds > 0:
            # Training next to an inference server in a second process that owns the page pool and the control
            # channel: request latency, training throughput, protocol-level handover latency per GiB. "per_request"
            # is the configuration as stated (every request triggers a memory handover and an SM-mask shrink,
            # continuous Poisson arrivals); "cold_request" keeps the pages until the server has been idle (the
            # reference server's own policy) and runs for a shorter window.
            from sirius_b200 import colocate_proc
            col = {}
            out["colocated"] = col
            for key, policy, secs in (("per_request", "per-request", args.colocate_seconds),
                                      ("cold_request", "cold-request", max(8.0, args.colocate_seconds / 3))):
                try:
                    # the multi-GiB handover rides on the second run only: the figures of the configuration as
                    # stated do not depend on it
                    col[key] = colocate_proc.run(duration_s=secs, policy=policy, multi_gib=(key == "cold_request"))
                except Exception as e:  # noqa: BLE001
                    col[key] = {"error": f"{type(e).__name__}: {e}"[:500]}
        if rank == 0 and world == 1 and not args.no_cpu_baseline:
            out["cpu_baseline"] = cpu_baseline(sample_batch=16, steps=3, warmup=1)

    failure = []

    def guarded():
        try:
            torch.cuda.set_device(local)   # the current device is per thread
            extras()
        except Exception as e:  # noqa: BLE001
            failure.append(f"{type(e).__name__}: {e}"[:300])
    if exchange is not None:
        exchange.close()     # the other workloads bring their own communicator
    # with several ranks the only additions are the two other workloads (tens of seconds): a shorter leash
    budget = args.extras_budget if world == 1 else min(args.extras_budget, 150.0)
    # shortly before the budget runs out, every thread's Python stack goes to stderr: says which leg and call is stuck
    faulthandler.dump_traceback_later(max(1.0, budget - 3.0), exit=False)
    worker = threading.Thread(target=guarded, daemon=True)
    worker.start()
    worker.join(budget)
    faulthandler.cancel_dump_traceback_later()
    unfinished = worker.is_alive()
    if unfinished:
        out["extras"] = f"stopped after {budget:.0f} s: the legs that had not finished are missing from this line"
    elif failure:
        out["extras"] = "failed: " + failure[0]
    if rank == 0:
        print(json.dumps(out, default=str), flush=True)
    if unfinished:
        # a leg is stuck in a call that cannot be interrupted: leave without waiting for it (children of the colocation
        # run are killed first)
        try:
            from sirius_b200 import colocate_proc
            colocate_proc.kill_children()
        except Exception:  # noqa: BLE001
            pass
        sys.stdout.flush()
        os._exit(0)
    if world > 1:
        # a rank whose additions ran out of time has left without this barrier: do not wait for it for ever
        leave = threading.Timer(30.0, lambda: os._exit(0))
        leave.daemon = True
        leave.start()
        dist.barrier()
        dist.destroy_process_group()
        leave.cancel()


def make_overlapped_allreduce(step, rank, world, local, args):
    """Gradient exchange of a transformer step through the library's NCCL communicator: one all-reduce per gradient
    bucket on the library's communication stream, each behind the bucket's ready event (recorded by the executor
    during backward); the executor's stream waits for the last one."""
    from sirius_b200.ddp import GradExchange
    ex = GradExchange(rank, world, device=local, wire=args.wire, max_ctas=args.nccl_max_ctas)

    def allreduce():
        ex.begin(step)
        ex.wait(step)
    return allreduce


# ---- second workload: GPT-2 small (batch 8 x 1024 tokens per GPU), selected with --workload gpt2 -----------------
GPT2 = dict(n_layer=12, n_head=12, d_model=768, vocab=50257, ctx=1024)
GPT2_BATCH, GPT2_SEQ = 8, 1024
GPT2_FLOP_PER_TOKEN = 0.854e9  # forward + backward (torch.utils.flop_counter on the CPU model, 2 FLOP per MAC)


QWEN2 = dict(n_layer=24, n_head=14, n_kv_head=2, hidden=896, intermediate=4864, vocab=151936)
QWEN2_BATCH, QWEN2_SEQ = 4, 2048
QWEN2_FLOP_PER_TOKEN = 2.964e9  # at 2048 tokens per sequence


def run_gpt2(args):
    return run_lm(args, "gpt2")


def compact(out):
    """The figures of a workload that the headline line carries for the other configurations."""
    return {"metric": out["metric"], "value": out["value"], "unit": out["unit"], "ms_per_step": out["ms_per_step"],
            "steps": out["steps"], "e2e": out["e2e"]["value"], "model_flops_frac": out["roofline"]["frac"],
            "workload": out["config"]["workload"], "global_batch": out["config"]["global_batch"],
            "gpu_launches": out["gpu_launches"], "clocks": out["clocks"], "tc_status": out["tc_status"]}


def run_lm(args, kind, embedded=False):
    """Causal-LM training step, bf16, AdamW lr 3e-4; tokens/s. kind: gpt2 (GPT-2 small, 8 x 1024 tokens per GPU) or
    qwen2 (Qwen2-0.5B shape, 4 x 2048 tokens per GPU)."""
    import torch
    import torch.distributed as dist
    from sirius_b200 import _lib, ops
    from sirius_b200.gpt2_step import Gpt2Step
    from sirius_b200.qwen2_step import Qwen2Step
    if kind == "qwen2":
        GPT2, GPT2_BATCH, GPT2_SEQ, GPT2_FLOP_PER_TOKEN = QWEN2, QWEN2_BATCH, QWEN2_SEQ, QWEN2_FLOP_PER_TOKEN
        title = "Qwen2-0.5B-shaped decoder train step (fwd+bwd+AdamW), bf16, batch 4 x 2048 tokens per GPU, token ids uniform in [0, 151936)"
    else:
        GPT2, GPT2_BATCH, GPT2_SEQ, GPT2_FLOP_PER_TOKEN = globals()["GPT2"], globals()["GPT2_BATCH"], globals()["GPT2_SEQ"], globals()["GPT2_FLOP_PER_TOKEN"]
        title = "GPT-2 small causal-LM train step (fwd+bwd+AdamW), bf16, batch 8 x 1024 tokens per GPU, token ids uniform in [0, 50257)"
    if args.lm_batch > 0:
        title = title.replace(f"batch {GPT2_BATCH} x", f"batch {args.lm_batch} x")
        GPT2_BATCH = args.lm_batch

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    if world > 1 and not embedded:
        import datetime
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=120))
    torch.manual_seed(0)
    if kind == "qwen2":
        from transformers import Qwen2Config, Qwen2ForCausalLM
        model = Qwen2ForCausalLM(Qwen2Config(vocab_size=GPT2["vocab"], hidden_size=GPT2["hidden"],
                                             intermediate_size=GPT2["intermediate"], num_hidden_layers=GPT2["n_layer"],
                                             num_attention_heads=GPT2["n_head"], num_key_value_heads=GPT2["n_kv_head"],
                                             max_position_embeddings=4096, rope_theta=1e6, rms_norm_eps=1e-6,
                                             tie_word_embeddings=True, use_sliding_window=False))
        sd = {k: v for k, v in model.state_dict().items() if k.startswith("model.")}
        del model
        step = Qwen2Step(**GPT2, max_batch=GPT2_BATCH, seq=GPT2_SEQ)
    else:
        from transformers import GPT2Config, GPT2LMHeadModel
        model = GPT2LMHeadModel(GPT2Config(vocab_size=GPT2["vocab"], n_positions=GPT2["ctx"], n_embd=GPT2["d_model"],
                                           n_layer=GPT2["n_layer"], n_head=GPT2["n_head"], resid_pdrop=0.0, embd_pdrop=0.0,
                                           attn_pdrop=0.0))
        sd = {k: v for k, v in model.state_dict().items() if k.startswith("transformer.") and not k.endswith(".attn.bias")
              and not k.endswith(".masked_bias")}
        del model
        step = Gpt2Step(**GPT2, max_batch=GPT2_BATCH, seq=GPT2_SEQ)
    step.load_state_dict(sd)
    stream = torch.cuda.ExternalStream(step.stream)
    g = torch.Generator().manual_seed(1000 + rank)
    host = [torch.randint(0, GPT2["vocab"], (GPT2_BATCH, GPT2_SEQ), generator=g, dtype=torch.int32) for _ in range(2)]
    global_bs = GPT2_BATCH * world
    allreduce = make_overlapped_allreduce(step, rank, world, local, args) if world > 1 else None

    def one(i, upload):
        if upload:
            step.upload_tokens(host[i % 2])
        step.forward_backward(global_bs)
        if allreduce is not None:
            allreduce()
        step.optimizer_step()
        return step.loss() if upload else None

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(upload, k):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(k):
            one(i, upload)
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    step.upload_tokens(host[0])
    for i in range(max(args.warmup, 3)):
        one(i, False)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = _lib.lib().srt_launch_count()
    ms = timed(False, args.steps)
    launches = _lib.lib().srt_launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else {}
    tokens = global_bs * GPT2_SEQ * args.steps
    value = tokens / (ms / 1e3)
    ms_e2e = timed(True, args.steps)
    e2e = tokens / (ms_e2e / 1e3)
    peaks = load_peaks()
    ach = value / world * GPT2_FLOP_PER_TOKEN / 1e12
    out = {
        "metric": "train tokens/s", "value": round(value, 1), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(ms / args.steps, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": title, "global_batch": global_bs, "seq_len": GPT2_SEQ,
                   "parallelism": f"dp{world}", "optimizer": "AdamW lr 3e-4 wd 0.01", "init": "seeded (no pretrained weights)",
                   "l2": "working set per step (GBs of activations and 0.8 GB of logits) exceeds the 126 MB L2"},
        "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": GPT2_BATCH * GPT2_SEQ * 4 * 4,
                "d2h_bytes_per_step": 4, "ms_per_step": round(ms_e2e / args.steps, 3)},
        "gpu_launches": int(launches), "clocks": clocks,
        "roofline": {"bound": "tensor", "achieved": round(ach, 2), "peak": peaks["tflops"], "unit": "TFLOP/s",
                     "frac": round(ach / peaks["tflops"], 4), "kernel": "whole step (model FLOPs of all GEMMs)",
                     "traffic": None, "peak_source": f"of {peaks['source']}"},
        "tc_status": ops.tc_status(), "memory_gib": round(step.memory_bytes() / 2 ** 30, 2),
    }
    if embedded:
        step.close()
        return compact(out)
    if rank == 0 and world == 1 and not args.no_cpu_baseline and kind == "gpt2":
        from oracle import gpt2_oracle as GO
        torch.set_num_threads(os.cpu_count() or 1)
        m = GO.build_model(**GPT2, seed=0)
        ids = GO.make_tokens(1, GPT2_SEQ, GPT2["vocab"], 2)
        opt = torch.optim.AdamW(m.parameters(), lr=3e-4)
        secs = []
        for b in ids:
            t0 = time.perf_counter()
            opt.zero_grad(set_to_none=True)
            m(b, labels=b).loss.backward()
            opt.step()
            secs.append(time.perf_counter() - t0)
        out["cpu_baseline"] = {"value": round(GPT2_SEQ / secs[-1], 1), "unit": "tokens/s", "cores": os.cpu_count(),
                               "kind": "port", "sample": "1 timed step after 1 warm-up of batch 1 x 1024 tokens (fp32, "
                               "same model and optimizer; the full workload is batch 8)", "sec_per_step": round(secs[-1], 3)}
    if rank == 0 and world == 1 and kind == "qwen2" and args.colocate_seconds > 0:
        # the same training step next to batch-1 DistilBERT-base requests on a bursty (gamma, CV 4) trace
        step.close()
        step = None
        from sirius_b200 import colocate_bench_lm
        out["colocated"] = colocate_bench_lm.run(duration_s=args.colocate_seconds)
    if rank == 0:
        print(json.dumps(out), flush=True)
    if step is not None:
        step.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# ---- third workload: Swin-B (batch 32 per GPU), selected with --workload swin_b ---------------------
SWIN_BATCH = 32
SWIN_FLOP_PER_SAMPLE = 92.55e9  # forward + backward (torch.utils.flop_counter on the CPU model)


def run_swin(args, embedded=False):
    """Swin-B training step, bf16, 32 images of 224 x 224 per GPU, AdamW lr 1e-3; samples/s."""
    import torch
    import torch.distributed as dist
    from sirius_b200 import _lib, ops
    from sirius_b200.swin_step import SWIN_B, SwinStep

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    if world > 1 and not embedded:
        import datetime
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=120))
    from torchvision.models.swin_transformer import SwinTransformer
    torch.manual_seed(0)
    model = SwinTransformer(patch_size=[4, 4], embed_dim=128, depths=[2, 2, 18, 2], num_heads=[4, 8, 16, 32],
                            window_size=[7, 7], stochastic_depth_prob=0.0, num_classes=1000)
    sd = {k: v for k, v in model.state_dict().items() if not k.endswith("relative_position_index")}
    del model
    step = SwinStep(**SWIN_B, max_batch=SWIN_BATCH)
    step.load_state_dict(sd)
    stream = torch.cuda.ExternalStream(step.stream)
    g = torch.Generator().manual_seed(1000 + rank)
    host = [(torch.randn(SWIN_BATCH, 3, 224, 224, generator=g).pin_memory(),
             torch.randint(0, 1000, (SWIN_BATCH,), generator=g).pin_memory()) for _ in range(2)]
    global_bs = SWIN_BATCH * world
    allreduce = make_overlapped_allreduce(step, rank, world, local, args) if world > 1 else None

    def one(i, upload):
        if upload:
            step.upload_batch(*host[i % 2])
        step.forward_backward(global_bs)
        if allreduce is not None:
            allreduce()
        step.optimizer_step()
        return step.loss() if upload else None

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(upload, k):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(k):
            one(i, upload)
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    step.upload_batch(*host[0])
    for i in range(max(args.warmup, 3)):
        one(i, False)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = _lib.lib().srt_launch_count()
    ms = timed(False, args.steps)
    launches = _lib.lib().srt_launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else {}
    value = global_bs * args.steps / (ms / 1e3)
    ms_e2e = timed(True, args.steps)
    e2e = global_bs * args.steps / (ms_e2e / 1e3)
    peaks = load_peaks()
    ach = value / world * SWIN_FLOP_PER_SAMPLE / 1e12
    out = {
        "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(ms / args.steps, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "Swin-B train step (fwd+bwd+AdamW), bf16, 32 images of 3x224x224 N(0,1) per GPU",
                   "global_batch": global_bs, "per_gpu_batch": SWIN_BATCH, "parallelism": f"dp{world}",
                   "optimizer": "AdamW lr 1e-3 wd 0.01", "init": "seeded (no pretrained weights)",
                   "l2": "working set per step (GBs of activations) exceeds the 126 MB L2"},
        "e2e": {"value": round(e2e, 1), "unit": UNIT, "h2d_bytes_per_step": SWIN_BATCH * 3 * 224 * 224 * 4 + SWIN_BATCH * 8,
                "d2h_bytes_per_step": 4, "ms_per_step": round(ms_e2e / args.steps, 3)},
        "gpu_launches": int(launches), "clocks": clocks,
        "roofline": {"bound": "tensor", "achieved": round(ach, 2), "peak": peaks["tflops"], "unit": "TFLOP/s",
                     "frac": round(ach / peaks["tflops"], 4), "kernel": "whole step (model FLOPs of all GEMMs)",
                     "traffic": None, "peak_source": f"of {peaks['source']}"},
        "tc_status": ops.tc_status(), "memory_gib": round(step.memory_bytes() / 2 ** 30, 2),
    }
    if embedded:
        step.close()
        return compact(out)
    if rank == 0:
        print(json.dumps(out), flush=True)
    step.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def cpu_baseline(sample_batch, steps, warmup):
    """The reference's arithmetic path (stock torchvision ResNet-152 + PyTorch CPU fp32, SGD) timed
    on this box's host cores on a bounded sample of the workload."""
    from oracle import resnet_oracle as O
    sec, threads = O.time_train_step(ARCH, batch=sample_batch, image=IMAGE, steps=steps, warmup=warmup)
    cpu_model = None
    try:
        with open("/proc/cpuinfo") as f:
            cpu_model = next((ln.split(":", 1)[1].strip() for ln in f if ln.startswith("model name")), None)
    except OSError:
        pass
    return {"value": round(sample_batch / sec, 3), "unit": UNIT, "cores": threads, "cpu_model": cpu_model, "kind": "port",
            "sample": f"{steps} timed step(s) after {warmup} warm-up of batch {sample_batch} (fp32, same model, "
                      f"optimizer and input distribution; the full workload is batch {BATCH})",
            "sec_per_step": round(sec, 3)}


def run_reference(args):
    """`--impl reference`: the reference's own CPU implementation of the path. The reference has no
    arithmetic of its own and its C++ runtime does not build here, so this is the CPU oracle: the
    torchvision/PyTorch calls of the reference's training script on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample = 8
    steps = max(1, min(args.steps, 4))
    warm = 1
    base = cpu_baseline(sample_batch=sample, steps=steps, warmup=warm)
    out = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warm, "ms_per_step": round(base["sec_per_step"] * 1e3, 1),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": base["sample"]},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--lm-batch", type=int, default=0,
                    help="sequences per GPU for the gpt2 / qwen2 workloads (0 = the configuration's own; smaller for profiling)")
    ap.add_argument("--workload", default="resnet152", choices=["resnet152", "gpt2", "swin_b", "qwen2"],
                    help="resnet152 (batch 64 per GPU) is the headline; swin_b, gpt2 and qwen2 time the other training workloads of the reference's evaluation")
    ap.add_argument("--wire", default="bf16", choices=["bf16", "f32"],
                    help="gradient format on NVLink for N > 1: bf16 (2 bytes per parameter) or f32")
    ap.add_argument("--nccl-max-ctas", type=int, default=0,
                    help="cap on the CTAs NCCL's kernels occupy beside the training kernels (0 = NCCL's default)")
    ap.add_argument("--colocate-seconds", type=float, default=30.0,
                    help="length of the colocated training+inference window at N=1 (0 = skip)")
    ap.add_argument("--extras-budget", type=float, default=300.0,
                    help="seconds the additions to the headline line (other workloads, colocation, reference-style handover, "
                         "CPU baseline) may take in total before the line is printed without the unfinished ones")
    ap.add_argument("--no-other-workloads", dest="other_workloads", action="store_false",
                    help="skip the compact Swin-B and GPT-2 results appended to the headline line")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "gpt2":
        run_gpt2(args)
    elif args.workload == "swin_b":
        run_swin(args)
    elif args.workload == "qwen2":
        run_lm(args, "qwen2")
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
