#!/usr/bin/env python
"""Benchmark of the policy-rollout forward (env-steps/s), one JSON line on stdout.

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --steps K --warmup W    # CPU arm (host cores)

A step is one batched policy forward over `--envs` envs per GPU (default 262,144,
h256x2: the configuration the headline metric is quoted on) with synthetic records,
N(0,1) recurrent state and N(0,1/fan_in) weights.  `value` is timed with CUDA events
on the launching stream with inputs resident in HBM; `e2e` goes through
cfx_policy_forward_host with pinned host buffers (copies inside the timed region).
Under torchrun each rank drives its own GPU and its own contiguous slice of envs;
there is no data-path collective, only a barrier and a max over ranks of the timings.
The K-step region is timed several times (`timed_repetitions`, each bracketed by a barrier
and a synchronize, max over ranks per repetition, a short idle gap between repetitions) and the
median repetition is reported, so that a few milliseconds of work are not judged on one
sample; `sustained` is the same step run back to back for about a fifth of a second, where a
1 kW part meets its power cap (its clock record is reported with it).  At N = 1 the line also
carries the reference's own cuBLAS forward on the same GPU and inputs (`reference_cublas`,
from the library built out of the reference sources when it is present), whole rollouts of the
reference's `run` loop unmodified, with the forward swapped and with the record write swapped
too (`reference_rollout`; `--no-rollout` or `--no-reference-cublas` skip it), and the CPU arm
(`cpu_baseline`).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "craftax.cu_b200"))

A = 43
METRIC = "policy_fwd_env_steps_per_s"
UNIT = "env-steps/s"


def algorithmic_work(H, L):
    """Per env-step: FLOPs of the three GEMM stages and bytes that must cross HBM
    (record, state read+write, logits+value, action, logprob, env action, prev_terminal)."""
    flops = 2 * 843 * H + L * 2 * 3 * H * H + 2 * (A + 1) * H
    byts = 996 + L * H * 4 * 2 + (A + 1) * 4 + 4 + 4 + 4 + 4
    return flops, byts


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples the SM clock and the clock-event (throttle) reasons of one GPU every ~1 ms
    with NVML (read-only queries) while the timed region runs; falls back to nvidia-smi."""
    REASONS = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20,
               "hw_thermal_slowdown": 0x40}

    def __init__(self, index):
        self.index, self.mhz, self.bits, self.max_mhz = index, [], 0, None
        self._stop = threading.Event()
        self.active = threading.Event()   # samples are taken only while a timed region runs
        self.active.set()
        self.thread = None
        self._nvml = None
        try:   # NVML is brought up here, before the warm-up, so that start() costs nothing
            import pynvml
            pynvml.nvmlInit()
            self._h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
            self._nvml = pynvml
        except Exception as e:  # NVML missing: one nvidia-smi sample at stop()
            self.err = str(e)

    def _sample(self):
        nv, h = self._nvml, self._h
        self.mhz.append(float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)))
        try:
            self.bits |= int(nv.nvmlDeviceGetCurrentClocksEventReasons(h))
        except Exception:
            self.bits |= int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(h))

    def start(self):
        if self._nvml is None:
            return

        def loop():
            while not self._stop.is_set():
                if self.active.is_set():
                    self._sample()
                time.sleep(0.0005)
        self.thread = threading.Thread(target=loop, daemon=True)
        self.thread.start()

    def stop(self):
        if self.thread is not None:
            self._stop.set()
            self.thread.join(timeout=2)
            reasons = [k for k, b in self.REASONS.items() if self.bits & b]
            return {"sm_mhz": float(np.median(self.mhz)) if self.mhz else None,
                    "sm_max_mhz": self.max_mhz, "reasons": reasons, "samples": len(self.mhz)}
        try:
            out = subprocess.run(["nvidia-smi", "-i", str(self.index),
                                  "--query-gpu=clocks.sm,clocks.max.sm", "--format=csv,noheader,nounits"],
                                 capture_output=True, text=True, timeout=10).stdout.split(",")
            return {"sm_mhz": float(out[0]), "sm_max_mhz": float(out[1]), "reasons": [],
                    "samples": 1, "note": "nvidia-smi after the timed region (NVML unavailable)"}
        except Exception:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["clock query unavailable"]}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def run_cfx(args):
    import cfx
    rank, world, local = dist_env()
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = local
    from cfx.sharding import aggregate_throughput, env_slice, max_over_ranks
    # weak scaling: the job is world x --envs envs, this rank owns a contiguous slice of it
    env_begin, env_end = env_slice(rank, world, world * args.envs)
    n, H, L = env_end - env_begin, args.hidden, args.layers
    prec = args.precision
    rng = np.random.default_rng(4 + rank)
    from cfx.synth import synthetic_records, init_weights
    base = synthetic_records(min(n, 8192), seed=4 + rank)
    rec = np.tile(base, (n // base.shape[0] + 1, 1))[:n]
    rec = rec[rng.permutation(n)] if n <= 65536 else rec
    params = init_weights(H, L, A, seed=0)
    pol = cfx.Policy(n, H, L, A, prec, device=dev)
    pol.set_weights(params)
    state = rng.standard_normal((L, n, H), dtype=np.float32)
    pol.set_state(state)
    del state
    prev_t = (rng.random(n) < 1.0 / 265.0).astype(np.float32)
    d_rec = cfx.DeviceBuffer.from_host(rec, dev)
    d_pt = cfx.DeviceBuffer.from_host(prev_t, dev)
    d_env = cfx.DeviceBuffer((n,), np.float32, dev)
    d_act = cfx.DeviceBuffer((n,), np.int32, dev)
    d_lp = cfx.DeviceBuffer((n,), np.float32, dev)
    d_val = cfx.DeviceBuffer((n,), np.float32, dev)
    d_lav = cfx.DeviceBuffer((n, A + 1), np.float32, dev)
    stream = pol.stream

    def step():
        pol.forward_device(d_rec, d_pt, None, env_actions=d_env, actions=d_act, logprobs=d_lp,
                           values=d_val, logits_av=d_lav, seed=2, env_offset=env_begin,
                           bump_step=True, stream=stream)

    def barrier():
        if dist is not None:
            import torch
            dist.barrier()
            torch.cuda.synchronize()
        pol.sync()

    sampler = ClockSampler(dev)
    for _ in range(args.warmup):
        step()
    pol.sync()
    launches_per_step = pol.last_launches
    sampler.start()
    # The K-step region, repeated: one repetition of K = 20 steps is ~8 ms, too short for a
    # max over ranks; repetitions fill about `--min-timed-ms` of device time.
    t_probe = cfx.Timer(dev)
    t_probe.start(stream)
    step()
    t_probe.stop(stream)
    pol.sync()
    reps = int(np.clip(np.ceil(args.min_timed_ms / max(1e-3, t_probe.elapsed_ms() * args.steps)), 1, 50))
    if dist is not None:   # every rank must run the same number of repetitions
        import torch
        r = torch.tensor([reps], device="cuda")
        dist.all_reduce(r, op=dist.ReduceOp.MAX)
        reps = int(r.item())
    rep_ms, per_step = [], []
    for _ in range(reps):
        timers = [cfx.Timer(dev) for _ in range(args.steps)]
        sampler.active.clear()
        time.sleep(args.rep_gap_ms * 1e-3)   # repetitions are separate measurements, not one long run
        barrier()
        sampler.active.set()
        t_all = cfx.Timer(dev)
        t_all.start(stream)
        for t in timers:
            t.start(stream)
            step()
            t.stop(stream)
        t_all.stop(stream)
        barrier()
        rep_ms.append(t_all.elapsed_ms())
        per_step.extend(t.elapsed_ms() for t in timers)
    clocks = sampler.stop()   # sampled over the repetitions of the K-step region
    # the same step back to back for ~0.2 s: what a long rollout sees under the power cap
    sus_sampler = ClockSampler(dev)
    sus_steps = int(np.clip(args.sustained_ms / max(1e-3, float(np.median(per_step))), args.steps, 2000))
    barrier()
    sus_sampler.start()
    t_sus = cfx.Timer(dev)
    t_sus.start(stream)
    for _ in range(sus_steps):
        step()
    t_sus.stop(stream)
    barrier()
    sustained_ms = t_sus.elapsed_ms() / sus_steps
    sus_clocks = sus_sampler.stop()
    pol.check()

    # end to end through the host-buffer entry point, pinned buffers
    pin_rec = cfx.PinnedBuffer((n, 996), np.uint8)
    pin_rec.array[:] = rec
    pin_pt = cfx.PinnedBuffer((n,), np.float32)
    pin_pt.array[:] = prev_t
    outs = {k: cfx.PinnedBuffer((n,), dt) for k, dt in
            [("env_actions", np.float32), ("actions", np.int32), ("logprobs", np.float32),
             ("values", np.float32)]}
    out_arrays = {k: v.array for k, v in outs.items()}
    e2e_steps = max(2, min(args.steps, 10))
    for _ in range(2):
        pol.forward_host(pin_rec.array, pin_pt.array, None, seed=2, env_offset=env_begin,
                         bump_step=True, want_logits=False, out=out_arrays)
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        pol.forward_host(pin_rec.array, pin_pt.array, None, seed=2, env_offset=env_begin,
                         bump_step=True, want_logits=False, out=out_arrays)
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
    # where an end-to-end step goes: the same copies alone (CUDA events, all ranks at once)
    lib = cfx.lib()
    h2d = n * 996 + n * 4
    d2h = 4 * n * 4
    tc = cfx.Timer(dev)
    barrier()
    tc.start(stream)
    for _ in range(e2e_steps):
        cfx.check(lib.cfx_memcpy_h2d(dev, d_rec.ptr, pin_rec.ptr, n * 996, stream))
        cfx.check(lib.cfx_memcpy_h2d(dev, d_pt.ptr, pin_pt.ptr, n * 4, stream))
    tc.stop(stream)
    pol.sync()
    upload_ms = tc.elapsed_ms() / e2e_steps
    barrier()
    tc.start(stream)
    for _ in range(e2e_steps):
        for k, b in (("env_actions", d_env), ("actions", d_act), ("logprobs", d_lp), ("values", d_val)):
            cfx.check(lib.cfx_memcpy_d2h(dev, outs[k].ptr, b.ptr, n * 4, stream))
    tc.stop(stream)
    pol.sync()
    readback_ms = tc.elapsed_ms() / e2e_steps

    v = max_over_ranks(list(rep_ms) + [e2e_ms, upload_ms, readback_ms, sustained_ms], dist)
    rep_ms, (e2e_ms, upload_ms, readback_ms, sustained_ms) = np.array(v[:reps]), v[reps:]
    total_ms = float(np.median(rep_ms))
    # whole job: env-steps of all ranks over the slowest rank's time
    value, _ = aggregate_throughput(total_ms, n * args.steps, dist)
    ms_per_step = total_ms / args.steps
    flops, byts = algorithmic_work(H, L)
    peaks = load_peaks()
    kernel_ms = float(np.mean(per_step))
    tensor_peak = peaks["bf16_tflops"]
    t_hbm = n * byts / (peaks["hbm_gbs"] * 1e9)
    t_tensor = n * flops / (tensor_peak * 1e12)
    if prec == "fp32" or t_hbm >= t_tensor:
        roof = {"bound": "hbm", "achieved": n * byts / (kernel_ms * 1e-3) / 1e9,
                "peak": peaks["hbm_gbs"], "unit": "GB/s"}
    else:
        roof = {"bound": "tensor", "achieved": n * flops / (kernel_ms * 1e-3) / 1e12,
                "peak": tensor_peak, "unit": "TFLOP/s"}
    roof["frac"] = roof["achieved"] / roof["peak"]
    # DRAM bytes of one launch (dram__bytes_read.sum + dram__bytes_write.sum of the committed
    # ncu captures): hidden 256 was captured at this very size (262,144 envs); hidden 128 at
    # 131,072 envs and is scaled by envs.  Other shapes have no capture and report null.
    per_env = NCU_DRAM_BYTES_PER_ENV.get((H, L)) if prec in ("f16", "bf16") else None
    roof["traffic"] = per_env * n if per_env is not None else None
    roof["traffic_source"] = NCU_DRAM_SOURCE.get((H, L)) if per_env is not None else None
    roof["peak_source"] = peaks["source"]
    roof["fused_roofline_ms"] = max(t_hbm, t_tensor) * 1e3
    roof["fused_roofline_frac"] = max(t_hbm, t_tensor) * 1e3 / kernel_ms
    roof["kernel_ms"] = kernel_ms
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None,
        "dtype": {"fp32": "f32", "f16": "f16 operands, f32 accumulate",
                  "bf16": "bf16 operands, f32 accumulate"}[prec],
        "data": "synthetic",
        "config": {"workload": f"policy forward, {n} envs/GPU, h{H}x{L}, {A} actions, 996-B records",
                   "envs_per_gpu": n, "hidden": H, "layers": L, "precision": prec,
                   "sharding": f"contiguous env slices x{world}, no collective",
                   "l2": "inputs larger than L2 (records+state %.0f MB per GPU)"
                         % ((n * 996 + L * n * H * 4) / 1e6)},
        "roofline": roof,
        "e2e": {"value": world * n / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                # the step's copies timed alone (max over ranks, all ranks copying at once) and
                # what is left for the kernel that the sliced upload does not hide
                "upload_ms": upload_ms, "readback_ms": readback_ms,
                "exposed_kernel_ms": max(0.0, e2e_ms - upload_ms - readback_ms),
                "h2d_gbs_per_gpu": h2d / (upload_ms * 1e-3) / 1e9,
                "bound": "host-to-device link"},
        "gpu_launches": launches_per_step * args.steps * reps,
        "timed_repetitions": reps,
        "ms_per_step_repetitions": [float(x) / args.steps for x in rep_ms],
        "clocks": clocks,
        "sustained": {"ms_per_step": sustained_ms, "value": world * n / (sustained_ms * 1e-3), "steps": sus_steps,
                      "clocks": sus_clocks},
    }
    if rank == 0 and world == 1 and not args.no_reference_cublas:
        line["reference_cublas"] = reference_cublas_forward(args, d_rec, d_pt, kernel_ms)
    if rank == 0 and world == 1 and not args.no_rollout and not args.no_reference_cublas:
        line["reference_rollout"] = reference_rollout(args, prec)
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_forward_rate(H, L, budget_s=args.cpu_budget)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def reference_cublas_forward(args, d_rec, d_pt, kernel_ms):
    """The reference's own forward (k_expand_obs ... k_value_sample + k_bump_ctr with its cuBLAS
    GEMMs, CUDA-graph replay as in its `run` mode, craftax_full.cu:12142-12160) on the SAME
    device buffers, in this process, right after the product arm: its bf16 mode (its default on
    this GPU, :11325-11332) and its TF32 mode.  Needs the library built from the reference
    sources (oracle/_ref/); reported as unavailable where that is absent."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    try:
        import oracle as O
        L = args.layers
        if args.hidden != 256 or not O.RefCuda.available(L):
            return {"unavailable": f"oracle/_ref/libcfref_cuda_l{L}.so not built (reference sources absent)"}
        from cfx.synth import init_weights
        ref = O.RefCuda(args.envs, L)
        ref.set_weights(init_weights(256, L, A, seed=0))
        steps = max(10, min(args.steps, 50))
        out = {"steps": steps, "what": "reference kernels + cuBLAS, graph replay, same records and "
                                       "prev_terminals buffers, same process"}
        for name, mode in (("bf16", ref.BF16), ("tf32", ref.TF32)):
            ms = ref.time_forward(mode, d_rec.ptr, d_pt.ptr, warm=3, iters=steps, graph=1)
            out[f"{name}_ms"] = ms
            out[f"ratio_{name}"] = ms / kernel_ms
        ref.close()
        return out
    except Exception as e:   # a comparison arm must not take the product line down
        return {"unavailable": f"{type(e).__name__}: {e}"}


def reference_rollout(args, prec):
    """Whole rollouts of the reference's `run` loop on this GPU, in the same run, right after
    the product arm: unmodified (cu_rollout_step_plain with its cuBLAS policy), with the policy
    half swapped for cfx_policy_forward, and with the record write swapped for cfx_record_obs as
    well; plus the two record kernels timed alone.  CUDA-graph replay, CUDA events.  The two
    arms (`--impl ref-rollout`, `--impl record`) run as child processes with a time limit, so
    that a failure inside the library built from the reference sources (oracle/_ref/) cannot
    take the product line down."""
    import subprocess

    def child(impl, extra, limit):
        cmd = [sys.executable, os.path.abspath(__file__), "--impl", impl, "--envs", str(args.envs),
               "--layers", str(args.layers), "--hidden", str(args.hidden)] + extra
        env = dict(os.environ)
        for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE"):
            env.pop(k, None)
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True, timeout=limit, env=env)
        lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
        if r.returncode != 0 or not lines:
            raise RuntimeError(f"`bench.py --impl {impl}` exited with {r.returncode}")
        return json.loads(lines[-1])
    try:
        ro = child("ref-rollout", ["--steps", "20", "--precision", prec], 240)
        if "unavailable" in ro:
            return {"unavailable": ro["unavailable"]}
        out = {"unit": UNIT, "iters": ro["iters"],
               "what": "reference run loop (env kernels + policy), graph replay, same run and GPU",
               "reference": ro["reference_rollout"], "forward_swapped": ro.get("swapped_rollout"),
               "forward_and_record_swapped": ro.get("swapped_rollout_and_record"),
               "ratio_forward_swapped": ro.get("R3_swapped_over_reference"),
               "ratio_forward_and_record_swapped": ro.get("swapped_and_record_over_reference")}
        rec = child("record", [], 120)
        if "unavailable" not in rec:
            out["record_write"] = {k: rec[k] for k in ("reference_k_record_obs_ms", "cfx_record_obs_ms", "speedup",
                                                       "differing_bytes", "rows_compared")}
        # the classic game at its configuration's size: forward, and the reference's classic step
        # with the forward (and the record write) swapped
        try:
            cl = json.loads([ln for ln in subprocess.run(
                [sys.executable, os.path.abspath(__file__), "--impl", "classic", "--envs", "1048576", "--steps", "20",
                 "--warmup", "3", "--precision", prec], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
                timeout=240, env={k: v for k, v in os.environ.items() if k not in ("RANK", "LOCAL_RANK", "WORLD_SIZE")}
            ).stdout.splitlines() if ln.startswith("{")][-1])
            out["classic_game"] = {"envs": 1048576, "forward_ms": cl["ms_per_step"], "forward_env_steps_per_s": cl["value"],
                                   "forward_roofline_frac": cl["roofline"]["frac"],
                                   "rollout": cl.get("reference_classic_rollout")}
        except Exception as e:
            out["classic_game"] = {"unavailable": f"{type(e).__name__}: {e}"}
        return out
    except Exception as e:   # a comparison arm must not take the product line down
        return {"unavailable": f"{type(e).__name__}: {e}"}


def cpu_forward_rate(H, L, budget_s=15.0, steps=1, warmup=0, threads=0):
    """Times the CPU arm: the reference's C env (when its prebuilt producer is present)
    stepping a bounded sample of envs plus the oracle's fp32 host forward on all host
    threads.  Returns the cpu_baseline object."""
    # all host threads this process may use: torchrun exports OMP_NUM_THREADS=1 to its workers,
    # which would make the CPU arm single-threaded whenever it is launched for N > 1
    host = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    if not threads:
        os.environ["OMP_NUM_THREADS"] = str(host)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle as O
    if not threads:
        try:   # the OpenMP runtime may already be up: set its default team size as well
            import ctypes
            ctypes.CDLL("libgomp.so.1").omp_set_num_threads(host)
        except OSError:
            pass
    cores = threads or max(host, O.max_threads())
    params = O.init_weights(H, L, A, seed=0)
    probe = 64 * cores
    rec = O.synthetic_records(probe, seed=4)
    st = np.zeros((L, probe, H), np.float32)
    t0 = time.perf_counter()
    O.forward(params, rec, None, st, H, L, A, threads=cores)
    rate = probe / (time.perf_counter() - t0)
    per_step = max(32 * cores, int(rate * budget_s / max(1, steps + warmup)) // 32 * 32)
    use_env = O.RefEnv.available()
    env = O.RefEnv(per_step, 0) if use_env else None
    rec = env.records if use_env else O.synthetic_records(per_step, seed=4)
    st = np.zeros((L, per_step, H), np.float32)
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        lav = O.forward(params, rec, env.terminals if use_env else None, st, H, L, A, threads=cores)
        if use_env:
            env.step(np.argmax(lav[:, :A], 1).astype(np.float32))
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    if env:
        env.close()
    v = per_step / float(np.mean(times))
    return {"value": v, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"{per_step} envs x {steps} step(s): "
                      + ("reference C env (craftax_full.c, compact obs) stepping + " if use_env else "")
                      + "oracle fp32 scalar forward, OpenMP over envs",
            "ms_per_step": float(np.mean(times)) * 1e3, "envs_per_step": per_step}


def run_reference(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    H, L = args.hidden, args.layers
    total = max(1, args.steps + args.warmup)
    b = cpu_forward_rate(H, L, budget_s=min(120.0, 12.0 * total), steps=args.steps,
                         warmup=args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": b["value"], "unit": UNIT,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": b["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"policy forward, {args.envs} envs/GPU, h{H}x{L}, {A} actions, 996-B records",
                   "envs_per_gpu": args.envs, "hidden": H, "layers": L, "precision": "fp32",
                   "sharding": "rank 0 only, host cores",
                   "l2": "not applicable (CPU arm)",
                   "sample_envs": b["envs_per_step"],
                   "note": "CPU arm: every step is a bounded sample (sample_envs) of the workload"},
        "cpu_baseline": {k: b[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": b["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_ref_cublas(args):
    """The reference's own CUDA forward (its kernels + cuBLAS, built from its sources into
    oracle/_ref/) on one B200, forward-only, CUDA-graph replay as in its `run` mode."""
    rank, _, local = dist_env()
    if rank != 0:
        return
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import cfx
    import oracle as O
    n, L = args.envs, args.layers
    if cfx.device_count() < 1:
        print(json.dumps({"impl": "ref-cublas", "unavailable": "no CUDA device"}))
        return
    if args.hidden != 256 or not O.RefCuda.available(L):
        print(json.dumps({"impl": "ref-cublas", "unavailable":
                          f"oracle/_ref/libcfref_cuda_l{L}.so not built (reference sources absent)"}))
        return
    from cfx.synth import synthetic_records, init_weights
    ref = O.RefCuda(n, L)
    ref.set_weights(init_weights(256, L, A, seed=0))
    base = synthetic_records(min(n, 8192), seed=4)
    rec = np.tile(base, (n // base.shape[0] + 1, 1))[:n]
    d_rec = cfx.DeviceBuffer.from_host(rec, local)
    d_pt = cfx.DeviceBuffer.from_host((np.random.default_rng(4).random(n) < 1 / 265).astype(np.float32), local)
    mode = {"bf16": ref.BF16, "tf32": ref.TF32, "fp32": ref.FP32}[args.ref_mode]
    ms = ref.time_forward(mode, d_rec.ptr, d_pt.ptr, warm=max(3, args.warmup), iters=args.steps, graph=1)
    print(json.dumps({"impl": "ref-cublas", "metric": METRIC, "value": n / (ms * 1e-3), "unit": UNIT,
                      "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms,
                      "higher_is_better": True, "dtype": args.ref_mode, "data": "synthetic",
                      "config": {"workload": f"reference cuBLAS forward, {n} envs, h256x{L}, graph replay",
                                 "mode": args.ref_mode}}), flush=True)
    ref.close()


def run_sweep(args):
    """Synthetic fused-forward sweep: batch x hidden {128, 256} x MinGRU depth x operand type
    (the instantiations built), one JSON line per point with the fused-roofline fraction; hidden
    512 runs through the strict fp32 mode and is labelled so.  Under
    torchrun every rank sweeps its own GPU with its own env slice (`--envs`-independent: the batch
    sizes are per GPU) and a point's time is the max over ranks.  Points of the published sweep
    that are not built (hidden 512, tf32 operands) are listed once as unavailable, with the reason."""
    import cfx
    from cfx.synth import synthetic_records, init_weights
    from cfx.sharding import max_over_ranks
    rank, world, local = dist_env()
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    peaks = load_peaks()
    base = synthetic_records(8192, seed=4 + rank)
    for n in (8192, 65536, 262144, 1048576, 2097152):
        rec = np.tile(base, (n // 8192, 1))
        d_rec = cfx.DeviceBuffer.from_host(rec, local)
        del rec
        d_act = cfx.DeviceBuffer((n,), np.int32, local)
        d_lav = cfx.DeviceBuffer((n, A + 1), np.float32, local)
        # hidden 512 has no fused instantiation; its points run through the strict fp32 mode
        # (CUDA-core kernels in the reference's summation order) and say so
        fused_points = [(h, l, p) for h in (256, 128) for l in (2, 3) for p in ("f16", "bf16")]
        strict_points = [(512, l, "fp32") for l in (2, 3)]
        points = strict_points if args.sweep_hidden == 512 else fused_points + strict_points
        for H, L, prec in points:
            pol = cfx.Policy(n, H, L, A, prec, device=local)
            pol.set_weights(init_weights(H, L, A, seed=0))
            for _ in range(3):
                pol.forward_device(d_rec, None, None, actions=d_act, logits_av=d_lav, seed=1,
                                   env_offset=rank * n, bump_step=True)
            pol.check()
            steps = 20 if n <= 262144 else 8
            if prec == "fp32":
                steps = 4 if n <= 262144 else 2
            if dist is not None:
                import torch
                dist.barrier()
                torch.cuda.synchronize()
            t = cfx.Timer(local)
            t.start(pol.stream)
            for _ in range(steps):
                pol.forward_device(d_rec, None, None, actions=d_act, logits_av=d_lav, seed=1,
                                   env_offset=rank * n, bump_step=True)
            t.stop(pol.stream)
            pol.check()
            ms = max_over_ranks([t.elapsed_ms() / steps], dist)[0]
            flops, byts = algorithmic_work(H, L)
            t_roof = max(n * byts / (peaks["hbm_gbs"] * 1e9), n * flops / (peaks["bf16_tflops"] * 1e12))
            if rank == 0:
                print(json.dumps({"sweep": "fused forward" if prec != "fp32" else "strict fp32 forward (CUDA cores)",
                                  "n_gpus": world, "envs_per_gpu": n, "hidden": H,
                                  "layers": L, "operands": prec, "ms_per_step": ms,
                                  "env_steps_per_s": world * n / (ms * 1e-3),
                                  "fused_roofline_ms": t_roof * 1e3, "fused_roofline_frac": t_roof * 1e3 / ms,
                                  "peak_source": peaks["source"]}), flush=True)
            pol.close()
        d_rec.free(); d_act.free(); d_lav.free()
    if rank == 0:
        print(json.dumps({"sweep": "fused forward", "unavailable": {
            "hidden 512": "the 16-bit input and output of a 512-wide layer fill all 512 tensor-memory columns of a "
                          "128-env tile, leaving none for the accumulators; its points above are the strict fp32 mode",
            "tf32 operands": "fp32 activations of K = 256 take 256 tensor-memory columns per buffer; fp16 operands "
                             "carry the same 11-bit significand"}}), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def run_classic(args):
    """Classic game (148-byte records, 1345 features, 3 MinGRU layers, 17 actions): the fused
    forward on one GPU at --envs, its fused-roofline fraction, and beside it the reference's own
    classic kernels with cuBLAS TF32 products (record-driven encoder, its MinGRU epilogue and
    sampler kernels; built from its sources into oracle/_ref/) on the same inputs."""
    rank, _, local = dist_env()
    if rank != 0:
        return
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import cfx
    from cfx.synth import classic_synthetic_records, classic_init_weights
    n, H, L, AC = args.envs, 256, 3, 17
    prec = args.precision or DEFAULT_PRECISION
    params = classic_init_weights(H, L, AC, seed=0)
    rec = np.tile(classic_synthetic_records(8192, seed=4), (n // 8192 + 1, 1))[:n]
    pol = cfx.Policy(n, H, L, AC, prec, device=local, game="classic")
    pol.set_weights(params)
    rng = np.random.default_rng(4)
    pol.set_state(rng.standard_normal((L, n, H), dtype=np.float32))
    d_rec = cfx.DeviceBuffer.from_host(rec, local)
    d_pt = cfx.DeviceBuffer.from_host((rng.random(n) < 1 / 265).astype(np.float32), local)
    d_act = cfx.DeviceBuffer((n,), np.int32, local)
    d_lp = cfx.DeviceBuffer((n,), np.float32, local)
    d_val = cfx.DeviceBuffer((n,), np.float32, local)

    def step():
        pol.forward_device(d_rec, d_pt, None, actions=d_act, logprobs=d_lp, values=d_val, seed=2, bump_step=True)
    for _ in range(max(3, args.warmup)):
        step()
    pol.check()
    t = cfx.Timer(local)
    t.start(pol.stream)
    for _ in range(args.steps):
        step()
    t.stop(pol.stream)
    pol.check()
    ms = t.elapsed_ms() / args.steps
    flops = 2 * 1345 * H + L * 6 * H * H + 2 * (AC + 1) * H
    byts = 148 + L * H * 8 + 4 + 4 + 4 + 4
    peaks = load_peaks()
    t_hbm, t_tensor = n * byts / (peaks["hbm_gbs"] * 1e9), n * flops / (peaks["bf16_tflops"] * 1e12)
    line = {"impl": "classic", "metric": METRIC, "value": n / (ms * 1e-3), "unit": UNIT, "n_gpus": 1,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True,
            "dtype": f"{prec} operands, f32 accumulate", "data": "synthetic",
            "config": {"workload": f"classic policy forward, {n} envs, h{H}x{L}, {AC} actions, 148-B records"},
            "roofline": {"bound": "tensor" if t_tensor > t_hbm else "hbm",
                         "fused_roofline_ms": max(t_hbm, t_tensor) * 1e3, "frac": max(t_hbm, t_tensor) * 1e3 / ms,
                         "flops_per_env": flops, "bytes_per_env": byts, "peak_source": peaks["source"]},
            "gpu_launches": args.steps * pol.last_launches}
    try:
        import oracle as O
        if O.RefClassic.available():
            ref = O.RefClassic()
            d_par = cfx.DeviceBuffer.from_host(params, local)
            d_st = cfx.DeviceBuffer((L, n, H), np.float32, local, zero=True)
            d_done = cfx.DeviceBuffer((n,), np.int8, local, zero=True)
            rms = ref.time_forward(d_par.ptr, d_rec.ptr, d_done.ptr, d_st.ptr, n, 3, max(5, min(args.steps, 20)), 1)
            line["reference_classic_forward"] = {"ms_per_step": rms, "value": n / (rms * 1e-3),
                                                 "what": "reference classic kernels + cublasSgemm TF32, record-driven encoder"}
            # whole rollouts: the reference's classic step (main_classic.cu Rollout::step) from its
            # own kernels, with the forward taken from this library, and with the record write too
            if hasattr(ref.L, "refcl_rollout_sps"):
                pol.close()
                pol = None
                del d_par, d_st, d_done
                r = {m: ref.rollout_sps(n, max(5, min(args.steps, 20)), 3, params, m,
                                        {"f16": cfx.PREC_F16, "bf16": cfx.PREC_BF16, "fp32": cfx.PREC_FP32}[prec])
                     for m in (0, 1, 2)}
                line["reference_classic_rollout"] = {
                    "unit": UNIT, "reference": r[0], "forward_swapped": r[1], "forward_and_record_swapped": r[2],
                    "ratio_forward_swapped": r[1] / r[0], "ratio_forward_and_record_swapped": r[2] / r[0],
                    "what": "reference classic env + policy step (its kernels, cublasSgemm TF32), eager launches"}
    except Exception as e:   # the comparison is optional
        line["reference_classic_forward"] = {"unavailable": str(e)}
    print(json.dumps(line), flush=True)
    if pol is not None:
        pol.close()


def run_ref_rollout(args):
    """Whole rollouts on one B200: the reference's own `run` loop (env kernels + its cuBLAS
    policy, graph replay), its env kernels alone, and the same loop with the policy half
    swapped for this library's forward (the drop-in binding a maintainer would add).  The three
    ratios of the target sentence are printed: R1 forward-only vs forward-only comes from
    `--impl cfx` and `--impl ref-cublas`; R2 = this library's forward-only env-steps/s over the
    reference's full-rollout SPS; R3 = swapped rollout over reference rollout."""
    rank, _, local = dist_env()
    if rank != 0:
        return
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import ctypes as C
    import cfx
    import oracle as O
    n, L = args.envs, args.layers
    if cfx.device_count() < 1 or args.hidden != 256 or not O.RefCuda.available(L):
        print(json.dumps({"impl": "ref-rollout", "unavailable":
                          f"needs a GPU and oracle/_ref/libcfref_cuda_l{L}.so (reference sources absent)"}))
        return
    cfx.lib()   # libcfx.so first: the reference shim links against it
    lib = C.CDLL(O.RefCuda.path(L))
    for f in ("refcu_rollout_sps", "refcu_env_only_sps"):
        getattr(lib, f).restype = C.c_double
        getattr(lib, f).argtypes = [C.c_int, C.c_int, C.c_ulonglong, C.c_int]
    iters = max(20, args.steps)
    out = {"impl": "ref-rollout", "unit": "env-steps/s", "envs": n, "layers": L, "iters": iters,
           "reference_rollout": lib.refcu_rollout_sps(n, iters, 1, 1),
           "reference_env_only": lib.refcu_env_only_sps(n, iters, 1, 1)}
    if hasattr(lib, "refcu_rollout_swap_sps"):
        lib.refcu_rollout_swap_sps.restype = C.c_double
        lib.refcu_rollout_swap_sps.argtypes = [C.c_int, C.c_int, C.c_ulonglong, C.c_int, C.c_int]
        prec = {"f16": cfx.PREC_F16, "bf16": cfx.PREC_BF16, "fp32": cfx.PREC_FP32}[args.precision or DEFAULT_PRECISION]
        out["swapped_rollout"] = lib.refcu_rollout_swap_sps(n, iters, 1, 1, prec)
        out["R3_swapped_over_reference"] = out["swapped_rollout"] / out["reference_rollout"]
        out["amdahl_cap_env_only_over_reference"] = out["reference_env_only"] / out["reference_rollout"]
    if hasattr(lib, "refcu_rollout_swap2_sps"):
        # the record write swapped too (cfx_record_obs instead of k_record_obs)
        lib.refcu_rollout_swap2_sps.restype = C.c_double
        lib.refcu_rollout_swap2_sps.argtypes = [C.c_int, C.c_int, C.c_ulonglong, C.c_int, C.c_int, C.c_int]
        out["swapped_rollout_and_record"] = lib.refcu_rollout_swap2_sps(n, iters, 1, 1, prec, 1)
        out["swapped_and_record_over_reference"] = out["swapped_rollout_and_record"] / out["reference_rollout"]
    print(json.dumps(out), flush=True)


def run_record(args):
    """The record write alone: the reference's k_record_obs and this library's cfx_record_obs on
    the reference's CUDA env (a few steps of random play, then randomised state), bytes
    compared, both kernels timed with CUDA events (20 calls each)."""
    rank, _, local = dist_env()
    if rank != 0:
        return
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import cfx
    import oracle as O
    n = args.envs
    if cfx.device_count() < 1 or not O.RefCuda.available(2):
        print(json.dumps({"impl": "record", "unavailable":
                          "needs a GPU and oracle/_ref/libcfref_cuda_l2.so (reference sources absent)"}))
        return
    cfx.lib()
    r = O.RefCuda.record_parity(2, n, 4, 2, seed=1)
    # bytes the kernel must move per env: the record, the 3 x 99 map bytes, ~100 SoA words
    algo = 996 + 3 * 99 + 4 * 100
    peaks = load_peaks()
    out = {"impl": "record", "envs": n, "differing_bytes": r["differing_bytes"], "rows_compared": r["rows_compared"],
           "reference_k_record_obs_ms": r["reference_ms"], "cfx_record_obs_ms": r["cfx_ms"],
           "speedup": r["reference_ms"] / r["cfx_ms"],
           "roofline": {"bound": "hbm", "bytes_per_env": algo, "achieved": n * algo / (r["cfx_ms"] * 1e-3) / 1e9,
                        "peak": peaks["hbm_gbs"], "unit": "GB/s",
                        "frac": n * algo / (r["cfx_ms"] * 1e-3) / 1e9 / peaks["hbm_gbs"]}}
    print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="cfx", choices=["cfx", "reference", "ref-cublas", "ref-rollout", "sweep", "classic", "record"])
    ap.add_argument("--ref-mode", default="bf16", choices=["bf16", "tf32", "fp32"])
    ap.add_argument("--envs", type=int, default=262144, help="envs per GPU")
    ap.add_argument("--hidden", type=int, default=256)
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--precision", default=None, choices=["fp32", "f16", "bf16"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-reference-cublas", action="store_true")
    ap.add_argument("--no-rollout", action="store_true",
                    help="skip the whole-rollout comparison (reference run loop, swapped, record write)")
    ap.add_argument("--min-timed-ms", type=float, default=100.0,
                    help="device time to fill with repetitions of the K-step region")
    ap.add_argument("--rep-gap-ms", type=float, default=30.0, help="idle gap between repetitions")
    ap.add_argument("--sustained-ms", type=float, default=200.0,
                    help="length of the back-to-back run reported as `sustained`")
    ap.add_argument("--cpu-budget", type=float, default=15.0)
    ap.add_argument("--sweep-hidden", type=int, default=0, choices=[0, 512],
                    help="--impl sweep: 512 runs only the hidden-512 points (strict fp32 mode)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "cfx" else args.warmup
    if args.precision is None:
        args.precision = DEFAULT_PRECISION
    if args.impl == "reference":
        run_reference(args)
    elif args.impl == "ref-cublas":
        run_ref_cublas(args)
    elif args.impl == "ref-rollout":
        run_ref_rollout(args)
    elif args.impl == "sweep":
        run_sweep(args)
    elif args.impl == "classic":
        run_classic(args)
    elif args.impl == "record":
        run_record(args)
    else:
        run_cfx(args)


DEFAULT_PRECISION = "f16"
# dram__bytes_read.sum + dram__bytes_write.sum of one launch, per env (ncu captures in profiles/)
NCU_DRAM_BYTES_PER_ENV = {(256, 2): (824.78e6 + 531.57e6) / 262144, (128, 2): (265.90e6 + 111.43e6) / 131072}
NCU_DRAM_SOURCE = {(256, 2): "ncu capture of one launch at 262,144 envs",
                   (128, 2): "ncu capture at 131,072 envs, scaled by envs (part of the writes was still in L2)"}

if __name__ == "__main__":
    main()
