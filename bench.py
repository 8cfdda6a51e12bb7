#!/usr/bin/env python
"""Benchmark of the quantized-KV decode path on B200.

    python bench.py --gpus N --steps K --warmup W            # one rank per GPU under torchrun for N > 1
    python bench.py --impl reference --gpus N --steps K --warmup W

Workload (default ``serve``): the box-scale serving configuration -- 131,072 users over 8
GPUs, i.e. 16,384 users per GPU, each with a quantized cache of 32 kv heads x 2,048 keys x
128 dims (N(0,1) K/V through the codec), one bf16 query per user per step, 32 query heads.
Per-GPU work is fixed, so N GPUs serve N x 16,384 users per step (weak scaling) and N = 8 is
the configuration as stated.  A GPU keeps as many distinct users resident as fit in memory
(``config.resident_users``); logical user u reads slot u mod resident_users, so every step
still streams 16,384 x 9.18 MB from HBM (far larger than L2, no flush needed).

One JSON line is printed by rank 0.  ``value`` is users/s with the query already on the
device; ``e2e`` times the host-buffer C-ABI step (pinned host query in, pinned host result
out, copies inside the timed region).  ``roofline`` relates the algorithmic bytes of one
launch to the measured copy bandwidth in MEASURED_PEAKS.json.  ``cpu_baseline`` is the CPU
oracle (a port of the reference's torch path) timed on a few users of the same shape.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

USERS_PER_GPU = 131072 // 8
WORKLOADS = {
    # name: (description, Hq, Hkv, S, users per GPU)
    "serve": ("config4-box-serving-shard: 16384 users/GPU x 32 kv heads x 2048 keys, 1 bf16 query/user/step", 32, 32, 2048, USERS_PER_GPU),
    "decode64": ("config1: 64 users x 8 heads x 50 keys", 8, 8, 50, 64),
    "gqa": ("config2: 256 users, 32 q / 8 kv heads, context U[1024,8192], K/V N(0,1) with 4 channels x8 before the rotation", 32, 8, 8192, 256),
    # the reference's own headline benchmark shape (scripts/run_criteo_benchmark.py: 64 users per query, 32 q / 8 kv heads,
    # 50 keys, per-user LoRA query update on, V aliased to K's nibbles); published: 104,571.3 users/s on an A10
    "criteo": ("reference headline shape: 64 users/query, 32 q / 8 kv heads, 50 keys, LoRA-Q on, V = K nibbles", 32, 8, 50, 64),
    # the other codec kernels, one after the other (reporting only): rotation, dequantisation, fp32 quantize, calibration
    "codec": ("codec kernels: rotate / dequantize / quantize (fp32, rotated input) / Lloyd-Max fit, 2048 users x 8 heads x 256 tokens", 8, 8, 256, 2048),
    # grouped queries over several tokens (speculative decoding / short prefill; reporting only): 128 query columns per
    # kv head, the shape the tcgen05 kernel exists for
    "mtok": ("multi-token grouped queries: 64 users, 32 q / 8 kv heads, 32 query tokens, 2048 keys", 32, 8, 2048, 64),
    # quantize-append (reporting only): 8 kv heads, 256 new bf16 tokens per user, K and V
    "append": ("config3: 4096 users x 256 new tokens x 8 heads, bf16 K and V, N(0,1) with 1% x10", 8, 8, 256, 4096),
}
BYTES_PER_KEY = 64 + 8 + 4 + 64          # K nibbles + K sign bytes + K norm + V nibbles
FALLBACK_HBM_GBS = 6650.0
PAIR_V = True          # the resident cache keeps V's nibble rows pair-wise (--v-layout reference: one key per row)
# DRAM bytes per (user, kv head, key) of the decode kernel from its committed ncu capture summary;
# scaled to a full launch by the keys it processes.
NCU_DRAM_BYTES_PER_KEY = 150.0   # ncu capture of the decode kernel: (10.048 GB read + 0.020 GB written) / 67.1 M keys


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu), "-lms", "200"], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.thread.join(timeout=5)
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def build_resident_cache(dev, Hkv, S, n_res, seed, lens=None, outliers=False):
    """Fill a resident packed cache with N(0,1) K/V pushed through the library's own
    rotate+quantize kernel, chunk by chunk (set-up, untimed).  V's nibble rows are then put into the
    pair layout of a serving cache (every complete group of eight keys below the user's length)."""
    from omnistack_rs_b200.kernels.quantize import _quantize_into
    from omnistack_rs_b200.kernels.fused_attention import pair_v_rows
    gen = torch.Generator(device=dev).manual_seed(seed)
    cb = torch.tensor([-2.733, -2.069, -1.618, -1.256, -0.9424, -0.6568, -0.3881, -0.1284,
                       0.1284, 0.3881, 0.6568, 0.9424, 1.256, 1.618, 2.069, 2.733], device=dev)  # 16-level Lloyd-Max, unit Gaussian
    chans = None
    if outliers:
        # configuration 2: four channels (the same for every row) carry 8x the scale before the rotation; one
        # shared codebook fitted by the library's Lloyd-Max kernel on a million rotated samples
        from omnistack_rs_b200.kernels.hadamard import rotate_queries
        from omnistack_rs_b200.quantization import calibrate_codebook
        chans = torch.randperm(128, generator=torch.Generator().manual_seed(1))[:4].to(dev)
        x = torch.randn(64, Hkv, 16, 128, generator=torch.Generator(device=dev).manual_seed(seed + 7), device=dev)
        x[..., chans] *= 8.0
        cb = calibrate_codebook(rotate_queries(x).reshape(-1)[: 1 << 20].contiguous()).to(dev)
    k_nib = torch.empty(n_res, Hkv, S, 64, dtype=torch.uint8, device=dev)
    k_qjl = torch.empty(n_res, Hkv, S, 8, dtype=torch.uint8, device=dev)
    k_norms = torch.empty(n_res, Hkv, S, dtype=torch.float32, device=dev)
    v_nib = torch.empty(n_res, Hkv, S, 64, dtype=torch.uint8, device=dev)
    chunk = max(1, min(n_res, (1 << 28) // (Hkv * S * 128)))          # <= 512 MiB of bf16 per chunk
    sq = torch.empty(chunk, Hkv, S, 8, dtype=torch.uint8, device=dev)
    sn = torch.empty(chunk, Hkv, S, dtype=torch.float32, device=dev)
    for u0 in range(0, n_res, chunk):
        n = min(chunk, n_res - u0)
        x = torch.randn(n, Hkv, S, 128, generator=gen, device=dev, dtype=torch.bfloat16)
        if chans is not None:
            x[..., chans] *= 8.0
        _quantize_into(x, cb, 0, True, k_nib[u0:u0 + n], k_qjl[u0:u0 + n], k_norms[u0:u0 + n], Hkv * S, S, None, 0)
        x = torch.randn(n, Hkv, S, 128, generator=gen, device=dev, dtype=torch.bfloat16)
        if chans is not None:
            x[..., chans] *= 8.0
        _quantize_into(x, cb, 0, True, v_nib[u0:u0 + n], sq[:n], sn[:n], Hkv * S, S, None, 0)
    del sq, sn
    if PAIR_V:
        pair_v_rows(v_nib, 0, S if lens is None else lens.to(device=dev, dtype=torch.int64))
    torch.cuda.synchronize(dev)
    return k_nib, k_qjl, k_norms, v_nib, cb


def decode_launches_per_step(users, Hq, T, S, n_splits):
    """Kernels one decode call launches: the tensor-core kernel and its fp32 stand-by (or the lane-per-key kernel
    alone for small shapes), plus the split-K merge."""
    mma = S >= 128 or users * Hq * T >= 1024
    return (2 if mma else 1) + (1 if n_splits > 1 else 0)


def verify_against_oracle(dev, rank, world, users, Hq, q, out, k_nib, k_qjl, k_norms, v_nib, cb, slots, lens, n_check=4):
    """Scores gathered to rank 0 for verification (NCCL when there are several ranks): one checksum row per user
    and, for ``n_check`` sampled users of every rank, the full output rows together with the packed cache rows and
    the query they were computed from; rank 0 recomputes those users with the CPU oracle."""
    import torch.distributed as dist
    from omnistack_rs_b200.serving import gather_rows_to_rank0
    from omnistack_rs_b200.kernels.fused_attention import pair_v_rows
    t_start = time.perf_counter()
    g = torch.Generator().manual_seed(100 + rank)
    picks = sorted({0, users - 1, *torch.randint(0, users, (max(n_check - 2, 0),), generator=g).tolist()})
    while len(picks) < min(n_check, users):
        picks.append(next(u for u in range(users) if u not in picks))
    picks = sorted(picks)[:n_check]
    idx = torch.tensor(picks, device=dev)
    slot = idx if slots is None else slots[idx].long()
    S = k_nib.shape[2]
    sample_lens = lens[idx].to(torch.int32) if lens is not None else torch.full((len(picks),), S, dtype=torch.int32, device=dev)
    vn = v_nib[slot].contiguous()
    if PAIR_V:
        pair_v_rows(vn, 0, sample_lens.to(torch.int64))          # back to the reference layout the oracle reads
    sample = {"out": out[idx].float(), "q": q[idx], "kn": k_nib[slot], "kq": k_qjl[slot],
              "kr": k_norms[slot], "vn": vn, "len": sample_lens}
    checksum = out.float().sum(dim=(1, 2, 3)).unsqueeze(1)                      # one number per user
    if world > 1:
        sample = {k: gather_rows_to_rank0(v.contiguous(), len(picks) * world) for k, v in sample.items()}
        checksum = gather_rows_to_rank0(checksum.contiguous(), users * world)
    if rank != 0:
        return None
    import oracle as orc
    t_gathered = time.perf_counter()
    threads = use_all_host_threads()
    cbc = cb.cpu()
    sample = {k: v.cpu() for k, v in sample.items()}
    worst = 0.0
    for i in range(sample["out"].shape[0]):
        n = int(sample["len"][i])
        if n == 0:
            continue
        want = orc.decode_attention(sample["q"][i:i + 1], sample["kn"][i:i + 1, :, :n], sample["kq"][i:i + 1, :, :n],
                                    sample["kr"][i:i + 1, :, :n], sample["vn"][i:i + 1, :, :n], cbc, 0)
        worst = max(worst, float((sample["out"][i:i + 1] - want).abs().max()))
    return {"users_checked": int(sample["out"].shape[0]), "max_abs_err": worst, "tolerance": 3e-3,
            "seconds": {"gather": round(t_gathered - t_start, 2), "oracle": round(time.perf_counter() - t_gathered, 2)},
            "host_threads": threads,
            "ok": bool(worst <= 3e-3 and torch.isfinite(checksum).all()), "ranks": world,
            "checksum_rows_gathered": int(checksum.shape[0]), "transport": "nccl gather" if world > 1 else "local"}


def measure_decode(args, workload, dev, rank, world, local, steps, warmup, with_cpu, with_verify):
    """Times one decode workload on this rank's GPU; returns the fields of its JSON line (rank 0) or None."""
    import torch.distributed as dist
    from omnistack_rs_b200 import _lib
    from omnistack_rs_b200.kernels.fused_attention import _qattn, _auto_splits
    from omnistack_rs_b200.serving import HostDecodeStep

    desc, Hq, Hkv, S, users = WORKLOADS[workload]
    if args.users and workload == args.workload:
        users = args.users
    scale = 1.0 / math.sqrt(128)
    wall = {"start": time.perf_counter()}

    # ---- resident cache ------------------------------------------------------------
    bytes_per_user = Hkv * S * BYTES_PER_KEY
    free, _total = torch.cuda.mem_get_info(dev)
    budget = free - (20 << 30)
    n_res = (args.resident_users if workload == args.workload else None) or max(1, min(users, budget // bytes_per_user))
    n_res = min(n_res, users)
    lens = None
    if workload == "gqa":
        g = torch.Generator().manual_seed(1)
        lens = torch.randint(1024, 8193, (users,), generator=g).to(torch.int32)
    if lens is not None and n_res < users:
        raise SystemExit("ragged lengths need every user resident (the pair layout of V follows each user's length)")
    k_nib, k_qjl, k_norms, v_nib, cb = build_resident_cache(dev, Hkv, S, n_res, seed=1234 + rank, lens=lens,
                                                            outliers=(workload == "gqa"))
    slots = (torch.arange(users, dtype=torch.int32) % n_res).to(dev) if n_res < users else None
    lens_dev = None if lens is None else lens.to(dev)
    keys_per_step = int(lens.sum()) * Hkv if lens is not None else users * Hkv * S
    alg_bytes = keys_per_step * BYTES_PER_KEY + users * Hq * (256 + 512)

    n_q = 4
    qs = [torch.randn(users, Hq, 1, 128, device=dev, dtype=torch.bfloat16) for _ in range(n_q)]
    n_splits = (args.splits if workload == args.workload else None) or _auto_splits(users, Hq, Hkv, 1, S, lens is not None)

    def step(i):
        return _qattn(qs[i % n_q], k_nib, k_qjl, k_norms, v_nib, cb, 0, scale, True,
                      seq_lens=lens_dev, cache_slots=slots, n_splits=n_splits, v_paired=PAIR_V)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # A working set smaller than L2 (the 64-user configuration) is flushed between timed steps by writing a
    # buffer larger than L2; the larger workloads stream far more than L2 holds per step.
    small = alg_bytes < (256 << 20)
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=dev) if small else None

    # ---- device-resident timing ------------------------------------------------------
    torch.cuda.synchronize(dev)
    wall["cache_built"] = time.perf_counter()
    for i in range(warmup):
        step(i)
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    if small:
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        for i, (e0, e1) in enumerate(evs):
            flush.fill_(i & 1)
            e0.record()
            out = step(i)
            e1.record()
        barrier()
        ms_total = sum(e0.elapsed_time(e1) for e0, e1 in evs)
    else:
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for i in range(steps):
            out = step(i)
        ev1.record()
        barrier()
        ms_total = ev0.elapsed_time(ev1)
    clocks = sampler.stop()
    tmax = torch.tensor([ms_total], device=dev)
    if world > 1:
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    ms_step = float(tmax) / steps
    launches = decode_launches_per_step(users, Hq, 1, S, n_splits)
    checksum = float(out.float().abs().mean())

    # ---- end to end: host query in, host result out -----------------------------------
    wall["device_loop_done"] = time.perf_counter()
    host = HostDecodeStep(k_nib, k_qjl, k_norms, v_nib, cb, n_heads=Hq, batch=users, q_dtype=torch.bfloat16,
                          user_id=0, seq_lens=lens_dev, cache_slots=slots, scale=scale,
                          n_chunks=args.chunks if workload == args.workload else None, v_paired=PAIR_V)
    host.q_host.copy_(qs[0].cpu())
    for _ in range(max(1, min(warmup, 3))):
        host.step()
    barrier()
    e2e_steps = steps
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        if small:
            flush.fill_(1)
        res = host.step()
    torch.cuda.synchronize(dev)
    t1 = time.perf_counter()
    e2e_t = torch.tensor([t1 - t0], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(e2e_t, op=dist.ReduceOp.MAX)
    e2e_s_step = float(e2e_t) / e2e_steps
    ref_out = _qattn(qs[0], k_nib, k_qjl, k_norms, v_nib, cb, 0, scale, True,
                     seq_lens=lens_dev, cache_slots=slots, n_splits=1, v_paired=PAIR_V)
    e2e_ok = bool((res - ref_out.cpu()).abs().max() <= 1.5e-3)   # splits round their fp16 softmax weights against other maxima
    _lib.check_device_status(dev)

    wall["host_loop_done"] = time.perf_counter()
    verify = None
    if with_verify:
        verify = verify_against_oracle(dev, rank, world, users, Hq, qs[0], ref_out, k_nib, k_qjl, k_norms, v_nib, cb,
                                       slots, lens_dev, n_check=max(1, min(args.verify_users, users)))

    # ---- CPU baseline: the oracle on a few users of the same shape (rank 0, N = 1) ------
    cpu = None
    if with_cpu and rank == 0 and world == 1:
        cpu = cpu_baseline(Hq, Hkv, S, lens, budget_s=args.cpu_seconds)
    if rank != 0:
        return None
    peak, peak_kind = measured_peak()
    achieved = alg_bytes / (ms_step * 1e-3) / 1e9
    return {
        "metric": "users_per_sec_quantized_kv_decode", "value": users * world / (ms_step * 1e-3), "unit": "users/s",
        "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "dtype_note": "f16 tensor-core operands (s8 for the sign term), f32 accumulation and softmax", "data": "synthetic",
        "config": {"workload": desc, "users_per_gpu": users, "resident_users": n_res, "q_heads": Hq, "kv_heads": Hkv,
                   "keys": S, "head_dim": 128, "bytes_per_key": BYTES_PER_KEY, "splits": n_splits,
                   "v_layout": "pair" if PAIR_V else "reference",
                   "l2": ("L2 flushed between timed steps (a 192 MiB buffer is written before each)" if small else
                          "inputs larger than L2 (resident cache %.1f GB per GPU)" % (n_res * bytes_per_user / 1e9)),
                   "parallelism": f"users sharded over {world} GPU(s), no collective on the data path"},
        "kv_gb_per_s": achieved * world,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_source": peak_kind, "frac_of_8000_nominal": achieved / 8000.0,
                     "traffic": (NCU_DRAM_BYTES_PER_KEY * keys_per_step if NCU_DRAM_BYTES_PER_KEY else None),
                     "algorithmic_bytes_per_launch": alg_bytes, "kernel": "qattn decode", "launch_ms": ms_step},
        "cpu_baseline": cpu,
        "e2e": {"value": users * world / e2e_s_step, "unit": "users/s", "h2d_bytes_per_step": host.h2d_bytes,
                "d2h_bytes_per_step": host.d2h_bytes, "ms_per_step": e2e_s_step * 1e3, "chunks": host.n_chunks, "splits": host.n_splits,
                "transfer": ("kernels read q from and write rows to the page-locked host buffers (one launch)"
                             if host.mode == "direct" else "staged copies pipelined over user chunks"),
                "matches_device_path": e2e_ok},
        "verify": verify,
        "wall_seconds": {"cache_build": round(wall["cache_built"] - wall["start"], 2),
                         "device_loop": round(wall["device_loop_done"] - wall["cache_built"], 2),
                         "host_buffer_loop": round(wall["host_loop_done"] - wall["device_loop_done"], 2),
                         "verify_and_cpu": round(time.perf_counter() - wall["host_loop_done"], 2)},
        "gpu_launches": steps * launches,
        "clocks": clocks, "checksum": checksum,
    }


SECONDARY_KEYS = ("value", "unit", "ms_per_step", "steps", "e2e", "clocks", "config")


def run_ours(args):
    import torch.distributed as dist
    rank, world, local = dist_env()
    if args.gpus != world and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    line = measure_decode(args, args.workload, dev, rank, world, local, args.steps, args.warmup,
                          with_cpu=not args.no_cpu, with_verify=not args.no_verify)
    # The other benchmark configurations, measured in the same process once the headline cache is freed
    # (single-GPU runs of the default workload only; each is also a workload of its own via --workload).
    if world == 1 and args.workload == "serve" and not args.no_secondary:
        secondary = {}
        torch.cuda.empty_cache()
        for name, wl, st in (("config1_decode64", "decode64", 200), ("config2_gqa", "gqa", 50)):
            r = measure_decode(args, wl, dev, rank, world, local, st, 5, with_cpu=False, with_verify=True)
            torch.cuda.empty_cache()
            secondary[name] = {k: r[k] for k in SECONDARY_KEYS} | {"roofline": r["roofline"], "verify": r["verify"]}
        r = measure_append(args, dev, rank, world, local, 20, 5, with_cpu=False)
        secondary["config3_append"] = {k: r[k] for k in SECONDARY_KEYS} | {"roofline": r["roofline"]}
        line["secondary"] = secondary
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line))


def use_all_host_threads(peers_waiting=True):
    """torchrun exports OMP_NUM_THREADS=1; the CPU legs are meant to use every core they may.  With several ranks one
    core per rank is left alone: the ranks that wait for rank 0 spin on theirs, and an OpenMP team that shares a core
    with a spinning thread loses a scheduler quantum at every barrier (measured: 8 s instead of 0.1 s per user)."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1 and peers_waiting:
        n -= world
    torch.set_num_threads(max(1, n))
    return torch.get_num_threads()


def run_append(args):
    import torch.distributed as dist
    rank, world, local = dist_env()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    line = measure_append(args, dev, rank, world, local, args.steps, args.warmup, with_cpu=not args.no_cpu)
    if world > 1:
        dist.barrier(); dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line))


def measure_append(args, dev, rank, world, local, steps, warmup, with_cpu):
    """Quantize-append workload (benchmark configuration 3): every step rotates and quantizes 256 new
    bf16 K and V tokens per user into the users' packed caches.  Metric: tokens/s."""
    import torch.distributed as dist
    from omnistack_rs_b200.kernels.quantize import _quantize_into

    desc, _, H, T, users = WORKLOADS["append"]
    if args.users and args.workload == "append":
        users = args.users
    gen = torch.Generator(device=dev).manual_seed(99 + rank)

    def heavy_tail():
        x = torch.randn(users, H, T, 128, generator=gen, device=dev)
        return torch.where(torch.rand(users, H, T, 128, generator=gen, device=dev) < 0.01, x * 10, x).to(torch.bfloat16)

    xk, xv = heavy_tail(), heavy_tail()
    cb = torch.tensor([-2.733, -2.069, -1.618, -1.256, -0.9424, -0.6568, -0.3881, -0.1284,
                       0.1284, 0.3881, 0.6568, 0.9424, 1.256, 1.618, 2.069, 2.733], device=dev)
    ids = torch.arange(users, dtype=torch.int32, device=dev) + rank * users
    mk = lambda *shape, dt=torch.uint8: torch.empty(*shape, dtype=dt, device=dev)  # noqa: E731
    k_nib, k_qjl, k_nrm = mk(users, H, T, 64), mk(users, H, T, 8), mk(users, H, T, dt=torch.float32)
    v_nib, v_qjl, v_nrm = mk(users, H, T, 64), mk(users, H, T, 8), mk(users, H, T, dt=torch.float32)

    def step(src_k, src_v):
        _quantize_into(src_k, cb, ids, True, k_nib, k_qjl, k_nrm, H * T, T, None, 0)
        _quantize_into(src_v, cb, ids, True, v_nib, v_qjl, v_nrm, H * T, T, None, 0)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(warmup):
        step(xk, xv)
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(steps):
        step(xk, xv)
    ev1.record()
    barrier()
    clocks = sampler.stop()
    tmax = torch.tensor([ev0.elapsed_time(ev1)], device=dev)
    if world > 1:
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    ms_step = float(tmax) / steps
    # end to end: new tokens arrive in pinned host memory; a checksum of the norms goes back
    hk, hv = xk.cpu().pin_memory(), xv.cpu().pin_memory()
    dk, dv = torch.empty_like(xk), torch.empty_like(xv)
    e2e_steps = max(1, min(steps, 5))
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        dk.copy_(hk, non_blocking=True); dv.copy_(hv, non_blocking=True)
        step(dk, dv)
        chk = float(k_nrm.sum().cpu())
    torch.cuda.synchronize(dev)
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    e2e_t = torch.tensor([e2e_s], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(e2e_t, op=dist.ReduceOp.MAX)
    cpu = None
    if rank == 0 and world == 1 and with_cpu:
        import oracle as orc
        use_all_host_threads()
        n = 16
        xs = xk[:n].cpu()
        orc.rotate_quantize(xs[:2], cb.cpu(), 0)
        t0 = time.perf_counter()
        for u in range(n):
            orc.rotate_quantize(xs[u:u + 1], cb.cpu(), u)
        dt = time.perf_counter() - t0
        cpu = {"value": n * T / dt / 1.0, "unit": "tokens/s", "cores": torch.get_num_threads(), "host_cpus": os.cpu_count(),
               "kind": "port", "sample": f"{n} users x {H} heads x {T} tokens, K only, CPU oracle (rotate + quantize_heads)"}
        cpu["value"] = cpu["value"] / 2.0      # a token is a K row and a V row per head
    if rank != 0:
        return None
    peak, peak_kind = measured_peak()
    rows = 2 * users * H * T
    alg = rows * (256 + 76)
    achieved = alg / (ms_step * 1e-3) / 1e9
    return {
        "metric": "tokens_per_sec_quantize_append", "value": users * T * world / (ms_step * 1e-3), "unit": "tokens/s",
        "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "dtype_note": "f32 butterflies and centroid search, s8 tensor-core projections with an exact f64 fallback", "data": "synthetic",
        "config": {"workload": desc, "users_per_gpu": users, "kv_heads": H, "new_tokens": T, "rows_per_step": rows,
                   "l2": "inputs larger than L2" if alg > 2e8 else "inputs smaller than L2"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_source": peak_kind, "traffic": 321.0 * rows, "algorithmic_bytes_per_launch": alg / 2,
                     "kernel": "fast_quantize_kernel", "launch_ms": ms_step / 2},
        "cpu_baseline": cpu,
        "e2e": {"value": users * T * world / float(e2e_t), "unit": "tokens/s", "h2d_bytes_per_step": 2 * hk.numel() * 2,
                "d2h_bytes_per_step": 4, "ms_per_step": float(e2e_t) * 1e3},
        "gpu_launches": 2 * steps, "clocks": clocks, "checksum": chk,
    }


REFERENCE_A10_USERS_PER_S = 104571.3      # README.md:83-85 of the reference (A10, the shape of the "criteo" workload)


def run_criteo(args):
    """The reference's published benchmark shape, one query = 64 users (single GPU, reporting only)."""
    from omnistack_rs_b200 import _lib
    from omnistack_rs_b200.kernels.quantize import quantize_heads
    from omnistack_rs_b200.kernels.fused_attention import omni_attn
    rank, world, local = dist_env()
    if rank != 0:
        return
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    desc, Hq, Hkv, S, B = WORKLOADS["criteo"]
    gen = torch.Generator(device=dev).manual_seed(11)
    n_users = 256                                                   # the reference bakes 256 users and draws 64 per query
    kv = torch.randn(n_users, Hkv, S, 128, generator=gen, device=dev)
    cb = torch.sort(torch.randn(Hkv, 16, generator=gen, device=dev) * 1.2, dim=1).values
    nib, qjl, nrm = quantize_heads(kv, cb, 0, rotate=True)
    la = torch.randn(16, 16, 128, generator=gen, device=dev) * 0.25
    lb = torch.randn(16, Hq * 128, 16, generator=gen, device=dev) * 0.05
    batches = []
    for _ in range(8):
        pick = torch.randint(0, n_users, (B,), generator=gen, device=dev)
        batches.append(dict(q=torch.randn(B, Hq, 1, 128, generator=gen, device=dev, dtype=torch.bfloat16),
                            x=torch.randn(B, 1, 128, generator=gen, device=dev),
                            idx=torch.randint(-1, 16, (B,), generator=gen, device=dev, dtype=torch.int32),
                            kn=nib[pick].contiguous(), kq=qjl[pick].contiguous(), kr=nrm[pick].contiguous()))

    def query(bt):
        return omni_attn(bt["q"], bt["kn"], bt["kq"], bt["kr"], bt["kn"], cb, user_id=0, x=bt["x"], lora_a=la, lora_b=lb,
                         lora_indices=bt["idx"], lora_alpha=1.0 / 16)

    for i in range(args.warmup):
        query(batches[i % 8])
    torch.cuda.synchronize(dev)
    sampler = ClockSampler(local)
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for i in range(args.steps):
        out = query(batches[i % 8])
    ev1.record()
    torch.cuda.synchronize(dev)
    clocks = sampler.stop()
    ms = ev0.elapsed_time(ev1) / args.steps
    # end to end: query, hidden state and adapter indices arrive on the host; the scores go back
    hb = [dict((k, v.cpu().pin_memory()) for k, v in bt.items() if k in ("q", "x", "idx")) for bt in batches]
    t0 = time.perf_counter()
    for i in range(args.steps):
        bt = dict(batches[i % 8])
        for k in ("q", "x", "idx"):
            bt[k] = hb[i % 8][k].to(dev, non_blocking=True)
        res = query(bt).cpu()
    e2e = (time.perf_counter() - t0) / args.steps
    _lib.check_device_status(dev)
    # the same query replayed from a CUDA graph (fixed query / adapter-input buffers): one launch per query for the host
    from omnistack_rs_b200.serving import GraphedAttention
    bt = batches[0]
    graphed = GraphedAttention(tuple(bt["q"].shape), bt["q"].dtype, bt["kn"], bt["kq"], bt["kr"], bt["kn"], cb, user_id=0,
                               lora_a=la, lora_b=lb, lora_alpha=1.0 / 16)
    graphed(bt["q"], bt["x"], bt["idx"])
    torch.cuda.synchronize(dev)
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    g0.record()
    for i in range(args.steps):
        gout = graphed()
    g1.record()
    torch.cuda.synchronize(dev)
    graph_ms = g0.elapsed_time(g1) / args.steps
    graph_ok = bool(torch.equal(gout, query(bt)))
    peak, peak_kind = measured_peak()
    alg = B * Hkv * S * (64 + 8 + 4) + B * Hq * 768                # V aliases K's nibbles: they are read once
    print(json.dumps({
        "metric": "users_per_sec_quantized_kv_decode", "value": B / (ms * 1e-3), "unit": "users/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": B / (ms * 1e-3) / REFERENCE_A10_USERS_PER_S, "dtype": "f16", "dtype_note": "f16 tensor-core operands (s8 for the sign term), f32 accumulation and softmax", "data": "synthetic",
        "config": {"workload": desc, "users_per_query": B, "q_heads": Hq, "kv_heads": Hkv, "keys": S, "lora_rank": 16,
                   "l2": "launch-bound case: the 2 MB working set stays in L2 (as in the reference's own run)",
                   "baseline": "104,571.3 users/s on an NVIDIA A10 (reference README.md:83-85)"},
        "roofline": {"bound": "hbm", "achieved": alg / (ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                     "frac": alg / (ms * 1e-3) / 1e9 / peak, "peak_source": peak_kind, "traffic": None},
        "cpu_baseline": None,
        "e2e": {"value": B / e2e, "unit": "users/s", "h2d_bytes_per_step": B * (Hq * 128 * 2 + 128 * 4 + 4),
                "d2h_bytes_per_step": B * Hq * 128 * 4, "ms_per_step": e2e * 1e3},
        "cuda_graph": {"ms_per_step": graph_ms, "users_per_s": B / (graph_ms * 1e-3), "matches_eager_call": graph_ok},
        "gpu_launches": 2 * args.steps, "clocks": clocks, "checksum": float(res.abs().mean()),
    }))


def run_mtok(args):
    """Attention of 32 query tokens per user (128 query columns per kv head) over a 2,048-key packed cache: the
    tcgen05 kernel (default for 49 or more columns) and the warp-level kernel (eight columns per tile) on the same
    inputs.  Single GPU, reporting only."""
    from omnistack_rs_b200 import _lib
    from omnistack_rs_b200.kernels.fused_attention import omni_attn
    rank, world, local = dist_env()
    if rank != 0:
        return
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    desc, Hq, Hkv, S, users = WORKLOADS["mtok"]
    if args.users:
        users = args.users
    T = 32
    k_nib, k_qjl, k_norms, v_nib, cb = build_resident_cache(dev, Hkv, S, users, seed=77)
    q = torch.randn(users, Hq, T, 128, device=dev, dtype=torch.bfloat16)
    peak, peak_kind = measured_peak()
    alg = users * Hkv * S * BYTES_PER_KEY + users * Hq * T * 768
    sampler = ClockSampler(local)
    sampler.start()
    kernels = {}
    for name, env in (("tcgen05", None), ("warp_level_tiles", "mma")):
        if env is None:
            os.environ.pop("OMNI_QATTN_KERNEL", None)
        else:
            os.environ["OMNI_QATTN_KERNEL"] = env
        for _ in range(args.warmup):
            out = omni_attn(q, k_nib, k_qjl, k_norms, v_nib, cb, user_id=0, v_paired=PAIR_V)
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            out = omni_attn(q, k_nib, k_qjl, k_norms, v_nib, cb, user_id=0, v_paired=PAIR_V)
        e1.record()
        torch.cuda.synchronize(dev)
        ms = e0.elapsed_time(e1) / args.steps
        kernels[name] = {"ms": ms, "gb_per_s": alg / (ms * 1e-3) / 1e9, "checksum": float(out.abs().mean())}
    os.environ.pop("OMNI_QATTN_KERNEL", None)
    clocks = sampler.stop()
    _lib.check_device_status(dev)
    lead = kernels["tcgen05"]
    print(json.dumps({
        "metric": "query_tokens_per_sec_multi_token_attention", "value": users * T / (lead["ms"] * 1e-3), "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": lead["ms"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": desc, "users": users, "q_heads": Hq, "kv_heads": Hkv, "query_tokens": T, "keys": S,
                   "v_layout": "pair" if PAIR_V else "reference", "l2": "inputs larger than L2" if alg > 2e8 else "inputs smaller than L2"},
        "roofline": {"bound": "hbm", "achieved": lead["gb_per_s"], "peak": peak, "unit": "GB/s", "frac": lead["gb_per_s"] / peak,
                     "peak_source": peak_kind, "traffic": None, "kernel": "qattn_umma_kernel",
                     "note": "the kernel is bound by its serial softmax / dequantise phases, not by HBM"},
        "kernels": kernels, "speedup_over_warp_level_tiles": kernels["warp_level_tiles"]["ms"] / lead["ms"],
        "cpu_baseline": None, "e2e": None, "gpu_launches": 2 * args.steps, "clocks": clocks,
    }))


def run_codec(args):
    """Times the codec kernels that no serving workload exercises, each against its algorithmic bytes (single GPU)."""
    from omnistack_rs_b200 import _lib
    from omnistack_rs_b200.kernels.hadamard import rotate_queries
    from omnistack_rs_b200.kernels.quantize import quantize_heads, dequantize_heads
    from omnistack_rs_b200.quantization import calibrate_per_group
    rank, world, local = dist_env()
    if rank != 0:
        return
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    desc, _, H, T, users = WORKLOADS["codec"]
    if args.users:
        users = args.users
    rows = users * H * T
    gen = torch.Generator(device=dev).manual_seed(5)
    x32 = torch.randn(users, H, T, 128, generator=gen, device=dev)
    x16 = x32.to(torch.bfloat16)
    groups = [x32[:, h].reshape(-1)[: 1 << 20].contiguous() for h in range(H)]
    cb = calibrate_per_group(groups)
    nib, qjl, nrm = quantize_heads(x32, cb, 3)
    peak, peak_kind = measured_peak()
    sampler = ClockSampler(local)
    sampler.start()

    def timed(fn):
        for _ in range(max(args.warmup, 1)):
            fn()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize(dev)
        return e0.elapsed_time(e1) / args.steps

    cases = [
        ("rotate_bf16", lambda: rotate_queries(x16), rows * 512),
        ("rotate_f32", lambda: rotate_queries(x32), rows * 1024),
        ("dequantize_int4_qjl", lambda: dequantize_heads(nib, qjl, nrm, cb, 3, with_qjl=True), rows * (76 + 512)),
        ("dequantize_int4", lambda: dequantize_heads(nib, qjl, nrm, cb, 3, with_qjl=False), rows * (64 + 512)),
        ("quantize_f32_rotated_input", lambda: quantize_heads(x32, cb, 3), rows * (512 + 76)),
        ("lloyd_max_fit_8x1M", lambda: calibrate_per_group(groups), H * (1 << 20) * 12),
    ]
    kernels = {}
    for name, fn, nbytes in cases:
        ms = timed(fn)
        kernels[name] = {"ms": ms, "gb_per_s": nbytes / (ms * 1e-3) / 1e9, "frac": nbytes / (ms * 1e-3) / 1e9 / peak}
    clocks = sampler.stop()
    _lib.check_device_status(dev)
    lead = kernels["dequantize_int4_qjl"]
    print(json.dumps({
        "metric": "rows_per_sec_dequantize", "value": rows / (lead["ms"] * 1e-3), "unit": "rows/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": lead["ms"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": desc, "rows": rows, "l2": "inputs larger than L2 (%.1f GB of fp32 rows)" % (rows * 512 / 1e9),
                   "note": "timings include the output allocation of the Python API; the Lloyd-Max line includes the sort"},
        "roofline": {"bound": "hbm", "achieved": lead["gb_per_s"], "peak": peak, "unit": "GB/s", "frac": lead["frac"],
                     "peak_source": peak_kind, "traffic": None, "kernel": "dequantize_heads_kernel"},
        "kernels": kernels, "cpu_baseline": None, "e2e": None, "gpu_launches": args.steps, "clocks": clocks,
    }))


def cpu_baseline(Hq, Hkv, S, lens, budget_s=15.0, n_users=2):
    """Time the CPU oracle (port of the reference's torch path) on ``n_users`` users of the
    workload's shape; repeated until about ``budget_s`` seconds have been spent."""
    import oracle as orc
    use_all_host_threads()
    gen = torch.Generator().manual_seed(7)
    Su = S if lens is None else int(lens[:n_users].max())
    cb = orc.lloyd_max_fit(torch.randn(1 << 14, generator=gen), max_iters=20)
    kn, kq, kr = orc.quantize_heads(orc.wht128(torch.randn(n_users, Hkv, Su, 128, generator=gen)), cb, 0)
    vn, _, _ = orc.quantize_heads(orc.wht128(torch.randn(n_users, Hkv, Su, 128, generator=gen)), cb, 0)
    q = torch.randn(n_users, Hq, 1, 128, generator=gen).to(torch.bfloat16)
    orc.decode_attention(q, kn, kq, kr, vn, cb, 0)                      # warm-up
    best, spent, reps = float("inf"), 0.0, 0
    while spent < budget_s and reps < 50:
        t0 = time.perf_counter()
        orc.decode_attention(q, kn, kq, kr, vn, cb, 0)
        dt = time.perf_counter() - t0
        best, spent, reps = min(best, dt), spent + dt, reps + 1
    return {"value": n_users / best, "unit": "users/s", "cores": torch.get_num_threads(), "host_cpus": os.cpu_count(),
            "kind": "port", "sample": f"{n_users} users x {Hkv} kv heads x {Su} keys, best of {reps} calls of the CPU oracle"}


def run_reference(args):
    """Reference arm: the reference's CPU implementation of the path.  The reference is pure
    Python and cannot be shipped to the GPU box, so the oracle port (pinned against it by
    tests/golden) is what runs, with every host thread torch offers."""
    rank, world, _ = dist_env()
    if rank != 0:
        return
    import oracle as orc
    use_all_host_threads(peers_waiting=False)             # the other ranks have exited
    desc, Hq, Hkv, S, users = WORKLOADS[args.workload]
    n_users = args.ref_users
    gen = torch.Generator().manual_seed(7)
    cb = orc.lloyd_max_fit(torch.randn(1 << 14, generator=gen), max_iters=20)
    kn, kq, kr = orc.quantize_heads(orc.wht128(torch.randn(n_users, Hkv, S, 128, generator=gen)), cb, 0)
    vn, _, _ = orc.quantize_heads(orc.wht128(torch.randn(n_users, Hkv, S, 128, generator=gen)), cb, 0)
    q = torch.randn(n_users, Hq, 1, 128, generator=gen).to(torch.bfloat16)
    for _ in range(args.warmup):
        orc.decode_attention(q, kn, kq, kr, vn, cb, 0)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        orc.decode_attention(q, kn, kq, kr, vn, cb, 0)
    dt = (time.perf_counter() - t0) / args.steps
    value = n_users / dt
    sample = f"each step = {n_users} users x {Hkv} kv heads x {S} keys through the CPU oracle (dequantise + fp32 attention)"
    print(json.dumps({
        "impl": "reference", "metric": "users_per_sec_quantized_kv_decode", "value": value, "unit": "users/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": desc, "users_per_step": n_users, "q_heads": Hq, "kv_heads": Hkv, "keys": S, "head_dim": 128},
        "cpu_baseline": {"value": value, "unit": "users/s", "cores": torch.get_num_threads(), "host_cpus": os.cpu_count(),
                         "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "users/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="serve", choices=sorted(WORKLOADS))
    ap.add_argument("--users", type=int, default=None, help="users per GPU per step (default: the workload's)")
    ap.add_argument("--resident-users", type=int, default=None, help="distinct users held in HBM (default: as many as fit)")
    ap.add_argument("--splits", type=int, default=None, help="key-axis splits (default: chosen from the shape)")
    ap.add_argument("--chunks", type=int, default=None, help="user chunks of the pipelined host-buffer step (default: by batch)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-verify", action="store_true", help="skip the oracle check of gathered sample users")
    ap.add_argument("--verify-users", type=int, default=64, help="users per rank recomputed by the CPU oracle after the timed loops")
    ap.add_argument("--no-secondary", action="store_true", help="default workload only: skip the other configurations")
    ap.add_argument("--cpu-seconds", type=float, default=15.0)
    ap.add_argument("--ref-users", type=int, default=2, help="users per step of the reference arm")
    ap.add_argument("--v-layout", default="pair", choices=["pair", "reference"],
                    help="layout of V's nibble rows in the resident cache (pair: the serving cache's own format)")
    args = ap.parse_args()
    global PAIR_V
    PAIR_V = args.v_layout == "pair"
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "append":
        run_append(args)
    elif args.workload == "criteo":
        run_criteo(args)
    elif args.workload == "codec":
        run_codec(args)
    elif args.workload == "mtok":
        run_mtok(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
