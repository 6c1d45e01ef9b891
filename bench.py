#!/usr/bin/env python
"""Benchmark of the spline-KV feature operator: forward + backward tokens/s at the d20 shape.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one forward and one backward of the feature operator over one batch of synthetic
pre-activations: N = 65536 tokens per GPU, h = 5120 keys, G = 20 (L = 22), r = 32, bf16, grid
[-5, 5], lambda = 1 (for more than one GPU: the token-sharded mode, lambda = 0.25 and wider
pre-activations, with the float32 dC all-reduce over NCCL).  Rank 0 prints one JSON line.

* ``value``: tokens/s of all ranks with inputs resident in HBM, CUDA-event timed, max over ranks.
* ``e2e``: the same through the public operator with HOST buffers: each step copies z and the
  upstream gradient from pinned host memory and copies f, dz and dC back, pipelined over sixteen
  token chunks on three streams so that copies in both directions overlap the kernels.  It is bound
  by the host link (PCIe and the host's memory), not by the kernels.
* ``roofline``: of forward and backward (the dz and dC kernels), the one furthest from its roofline, timed alone with
  CUDA events in a separate pass of the same length, against the measured dense bf16 peak.
* ``parity``: after the timed region, the operator against the CPU oracle on a token subset
  (knot-index mismatches, maxabs(diff)/maxabs(ref) and mean signed error of the float32 residual,
  dz and dC) and, on more than one GPU, the all-reduced dC against the float64 sum of the ranks'
  own float32 dC.
* ``extra``: short bounded measurements of the other configurations: the key-sharded mode at
  N = 131072 (partial residuals all-reduced), the rank/grid sweep (r = 16, 64, 128 at G = 20 and
  r = 32 at G = 40) and a stack of 7 layers with their W_in / W_out GEMMs.
* ``cpu_baseline``: the CPU oracle (a C/OpenMP port of the reference's algorithm) on a bounded
  token sample of the same workload, all host threads.

``--impl reference`` times that CPU port alone (rank 0 only) and prints the same line shape.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "spline-KV fwd+bwd tokens/s @ h=5120,G=20,r=32 bf16"
SHAPE = dict(N=65536, d=1280, h=5120, G=20, r=32, grid_lo=-5.0, grid_hi=5.0)
PARITY_TOKENS = 1024


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"],
                    bf16_tflops_sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while a region runs (read-only NVML queries
    from a thread every few milliseconds; nvidia-smi in a loop if the NVML binding is missing)."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")
    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, index: int):
        self.index, self.rows, self.proc, self.thread, self.stop_flag = index, [], None, None, False
        self.sm, self.smax, self.reasons = [], [], set()

    def _nvml_loop(self, nvml, handle):
        while not self.stop_flag:
            try:
                self.sm.append(float(nvml.nvmlDeviceGetClockInfo(handle, nvml.NVML_CLOCK_SM)))
                mask = int(nvml.nvmlDeviceGetCurrentClocksEventReasons(handle))
                for name, bit in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                break
            time.sleep(0.004)

    def start(self):
        try:
            import pynvml as nvml
            nvml.nvmlInit()
            # NVML orders devices by PCI bus id, as CUDA does when CUDA_VISIBLE_DEVICES is unset
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            idx = int(vis.split(",")[self.index]) if vis and vis.split(",")[self.index].isdigit() else self.index
            handle = nvml.nvmlDeviceGetHandleByIndex(idx)
            self.smax.append(float(nvml.nvmlDeviceGetMaxClockInfo(handle, nvml.NVML_CLOCK_SM)))
            self.thread = threading.Thread(target=self._nvml_loop, args=(nvml, handle), daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        self.stop_flag = True
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        if self.thread:
            self.thread.join(timeout=2)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                self.sm.append(float(r[0]))
                self.smax.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(names, r[4:8]):
                if val.lower().startswith("active"):
                    self.reasons.add(name)
        if not self.sm:
            return None
        return dict(sm_mhz=statistics.median(self.sm), sm_max_mhz=max(self.smax) if self.smax else None,
                    reasons=sorted(self.reasons), samples=len(self.sm))


def bind_to_gpu_numa_node(index: int):
    """Run this process on the host cores NVML reports as local to its GPU (a read-only query), so
    that the pinned host buffers of the end-to-end leg are allocated on that GPU's NUMA node.
    Returns the core list, or None when the query or the binding is not possible."""
    try:
        import pynvml as nvml
        nvml.nvmlInit()
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        idx = int(vis.split(",")[index]) if vis and vis.split(",")[index].isdigit() else index
        handle = nvml.nvmlDeviceGetHandleByIndex(idx)
        words = nvml.nvmlDeviceGetCpuAffinity(handle, (os.cpu_count() + 63) // 64)
        cores = {64 * w + b for w, word in enumerate(words) for b in range(64) if (int(word) >> b) & 1}
        cores &= os.sched_getaffinity(0)
        if not cores:
            return None
        os.sched_setaffinity(0, cores)
        return sorted(cores)
    except Exception:
        return None


def cpu_port_tokens_per_s(cfg, seed, target_seconds=12.0):
    """Forward + backward of the CPU oracle (C/OpenMP port) on a token sample of the workload, on
    every host core this process may run on (the thread count is set explicitly: a launcher such as
    torch.distributed.run exports OMP_NUM_THREADS=1)."""
    import numpy as np
    from oracle import c_binding as oc
    oc.build()
    oc.set_threads(len(os.sched_getaffinity(0)))
    h, r, G = cfg["h"], cfg["r"], cfg["G"]
    lo, hi, lam = cfg["grid_lo"], cfg["grid_hi"], cfg["lambda_scale"]
    rng = np.random.default_rng(seed)

    def run(n):
        z = (rng.standard_normal((n, h)) * cfg["z_std"]).astype(np.float32)
        C = (rng.standard_normal((h, G + 2, r)) * 0.02).astype(np.float32)
        go = rng.standard_normal((n, h + r)).astype(np.float32)
        t0 = time.perf_counter()
        oc.feature_forward(z, C, lo, hi, G, "relu_sq", lam)
        oc.feature_backward(z, C, go[:, h:], go[:, :h], lo, hi, G, "relu_sq", lam)
        return time.perf_counter() - t0

    run(64)
    probe_n = 256
    t = run(probe_n)
    n = int(max(256, min(cfg["N"], probe_n * target_seconds / max(t, 1e-6))))
    n = (n // 256) * 256
    t = run(n)
    return n / t, n, t, oc.num_threads()


def reference_arm(args, cfg):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    vals, n, threads = [], 0, 1
    per_step_target = max(2.0, min(20.0, 120.0 / max(1, args.steps + args.warmup)))
    for i in range(args.warmup + args.steps):
        v, n, t, threads = cpu_port_tokens_per_s(cfg, seed=i, target_seconds=per_step_target)
        if i >= args.warmup:
            vals.append((v, t))
    value = statistics.mean(v for v, _ in vals)
    ms = statistics.mean(t for _, t in vals) * 1e3
    sample = f"{n} of {cfg['N']} tokens per step at h={cfg['h']}, r={cfg['r']}, G={cfg['G']}; fwd+bwd, float64 accumulate"
    line = dict(impl="reference", metric=METRIC, value=value, unit="tokens/s", n_gpus=args.gpus, steps=args.steps,
                warmup=args.warmup, ms_per_step=ms, higher_is_better=True, scaling="weak", vs_baseline=None,
                dtype="f32", data="synthetic", config=cfg_json(cfg, args.gpus),
                cpu_baseline=dict(value=value, unit="tokens/s", cores=threads, kind="port", sample=sample),
                e2e=dict(value=value, unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0),
                gpu_launches=0)
    print(json.dumps(line), flush=True)


def cfg_json(cfg, gpus):
    return dict(workload=cfg["name"], tokens_per_gpu=cfg["N"], h=cfg["h"], G=cfg["G"], L=cfg["G"] + 2, r=cfg["r"],
                grid=[cfg["grid_lo"], cfg["grid_hi"]], lambda_scale=cfg["lambda_scale"], z_std=cfg["z_std"],
                sharding="none" if gpus == 1 else f"tokens x{gpus}, dC all-reduce (float32, NCCL)",
                l2="inputs larger than L2 (z is 671 MB per GPU)")


def make_cfg(gpus):
    cfg = dict(SHAPE)
    if gpus == 1:
        cfg.update(name="d20 production shape, single layer fwd+bwd (config 1)", lambda_scale=1.0, z_std=1.0)
    else:
        cfg.update(name="d20 shape token-sharded with dC all-reduce (config 2)", lambda_scale=0.25, z_std=2.0)
    return cfg


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=0, help="override tokens per GPU (profiling of small cases)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the parity and extra-configuration records")
    ap.add_argument("--fused-backward", action="store_true",
                    help="run dz and dC as one kernel where its plan fits (A/B against the default two kernels)")
    ap.add_argument("--only-readout", action="store_true",
                    help="print only the forward + read-out record (profiling of the read-out GEMM; one GPU)")
    ap.add_argument("--e2e-chunks", type=int, default=16, help="token chunks the end-to-end step is pipelined over")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    cfg = make_cfg(args.gpus)
    if args.tokens:
        cfg["N"] = args.tokens
        cfg["name"] += f" [reduced to {args.tokens} tokens]"
    if args.impl == "reference":
        reference_arm(args, cfg)
        return

    import torch
    import torch.distributed as dist
    from sparsespline_ffn_b200 import _lib, ops, sharded
    from sparsespline_ffn_b200 import flash_spline_feature

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    local_cores = bind_to_gpu_numa_node(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = _lib.load()
    _lib.check(lib.skv_device_ok())
    if args.fused_backward:
        lib.skv_debug_set(_lib.SKV_DEBUG_FUSED_BACKWARD, 1)

    if args.only_readout:
        def timed_1gpu(fn, steps):
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1)
        rec = extra_readout(torch, ops, cfg, rank, dev, timed_1gpu, steps=max(1, args.steps))
        ops.check_status(dev)
        print(json.dumps(dict(readout=rec, config=cfg_json(cfg, world))), flush=True)
        return

    N, d, h, G, r = cfg["N"], cfg["d"], cfg["h"], cfg["G"], cfg["r"]
    lo, hi, lam = cfg["grid_lo"], cfg["grid_hi"], cfg["lambda_scale"]
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    cgen = torch.Generator(device=dev).manual_seed(99)           # C is replicated: same seed on all ranks
    x = torch.randn(N, d, generator=gen, device=dev) * cfg["z_std"]
    W_in = torch.randn(d, h, generator=cgen, device=dev) * (1.0 / d) ** 0.5
    z = (x @ W_in).to(torch.bfloat16)
    del x, W_in
    C = (torch.randn(h, G + 2, r, generator=cgen, device=dev) * 0.02).to(torch.bfloat16)
    go = torch.randn(N, h + r, generator=gen, device=dev).to(torch.bfloat16)
    z.requires_grad_(True)
    C.requires_grad_(True)
    oor = float(((z.detach().float() < lo) | (z.detach().float() > hi)).float().mean().item())

    def step_device():
        z.grad = None
        C.grad = None
        if world == 1:
            f = flash_spline_feature(z, C, lo, hi, G, "relu_sq", lam, True)
        else:
            f = sharded.token_sharded_spline_feature(z, C, lo, hi, G, "relu_sq", lam)
        f.backward(go)
        return f

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        """K calls of fn bracketed by barrier + synchronize; ms of the whole region, max over ranks."""
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for _ in range(args.warmup):
        step_device()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = int(lib.skv_kernel_launches())
    total_ms = timed(step_device, args.steps)
    launches = int(lib.skv_kernel_launches()) - launches0
    clocks = sampler.stop() if rank == 0 else None
    ops.check_status(dev)
    ms_per_step = total_ms / args.steps
    value = world * N / (ms_per_step * 1e-3)

    # ---- per-kernel attribution: forward and backward each timed alone over the same number of steps;
    # the backward also as its two separate kernels (dz alone, dC alone), which is how it runs where the
    # fused kernel does not apply
    zd, Cd = z.detach(), C.detach()
    kern = {}
    kern["forward"] = timed(lambda: ops.feature_forward(zd, Cd, lo, hi, G, "relu_sq", lam), args.steps) / args.steps
    kern["backward"] = timed(lambda: ops.feature_backward(zd, Cd, go, lo, hi, G, "relu_sq", lam),
                             args.steps) / args.steps
    kern_split = {}
    kern_split["dz"] = timed(lambda: ops.feature_backward(zd, Cd, go, lo, hi, G, "relu_sq", lam, need_dC=False),
                             args.steps) / args.steps
    kern_split["dC"] = timed(lambda: ops.feature_backward(zd, Cd, go, lo, hi, G, "relu_sq", lam, need_dz=False),
                             args.steps) / args.steps
    impl = ops.resolve_impl(zd, Cd, lo, hi, G)
    peaks = measured_peaks()
    flops = 2.0 * N * h * (G + 2) * r                      # dense-equivalent FLOPs of one of the three GEMMs
    gemms = {"forward": 1, "backward": 2}                  # the backward is the dz and the dC contraction
    frac_of = {k: gemms[k] * flops / (kern[k] * 1e-3) / 1e12 / peaks["bf16_tflops"] for k in kern}
    dominant = min(frac_of, key=frac_of.get)               # the kernel furthest from its roofline
    achieved = gemms[dominant] * flops / (kern[dominant] * 1e-3) / 1e12
    traffic = None
    tpath = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(tpath):
        with open(tpath) as f:
            rec = json.load(f).get(f"{impl}:{dominant}")
        if rec and "bytes_per_token" in rec:
            # captured at two reduced token counts: the per-token part scales with N, the rest does not
            traffic = rec["bytes_per_token"] * N + rec["bytes_fixed"]
    step_tflops = 3 * flops / (ms_per_step * 1e-3) / 1e12
    roofline = dict(bound="tensor", kernel=f"{impl}:{dominant}", achieved=achieved, peak=peaks["bf16_tflops"],
                    unit="TFLOP/s", frac=achieved / peaks["bf16_tflops"], traffic=traffic,
                    peak_source=peaks["source"] + " burst bf16 (kernel timed alone)",
                    flops_per_launch=gemms[dominant] * flops,
                    kernel_ms={k: round(v, 4) for k, v in kern.items()},
                    kernel_ms_split_backward={k: round(v, 4) for k, v in kern_split.items()},
                    kernel_frac={k: round(v, 4) for k, v in frac_of.items()},
                    step_frac_of_burst_peak=step_tflops / peaks["bf16_tflops"],
                    step_frac_of_sustained_peak=step_tflops / peaks["bf16_tflops_sustained"])

    # ---- end to end through the public operator with host buffers
    e2e = None
    if not args.no_e2e:
        zh = z.detach().cpu().pin_memory()
        goh = go.cpu().pin_memory()
        fh = torch.empty((N, h + r), dtype=torch.bfloat16).pin_memory()
        dzh = torch.empty((N, h), dtype=torch.bfloat16).pin_memory()
        dCh = torch.empty((h, G + 2, r), dtype=torch.bfloat16).pin_memory()
        zdev = torch.empty_like(zh, device=dev)
        godev = torch.empty_like(goh, device=dev)

        # The step is pipelined over NCH token chunks on three streams: the host-to-device copies of
        # chunk i+1, the operator's forward+backward on chunk i and the device-to-host copies of chunk
        # i-1 overlap (PCIe is full duplex); dC is accumulated across the chunks on the device, as
        # autograd does for micro-batches, and copied back once.
        NCH = args.e2e_chunks if N % args.e2e_chunks == 0 and N >= 1024 * args.e2e_chunks else 1
        rows = N // NCH
        s_in, s_comp, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        state = dict(prev_comp=[None] * NCH)

        def step_e2e():
            cur = torch.cuda.current_stream()
            s_in.wait_stream(cur)
            s_comp.wait_stream(cur)
            s_out.wait_stream(cur)
            C.grad = None
            keep = []
            for c in range(NCH):
                sl = slice(c * rows, (c + 1) * rows)
                with torch.cuda.stream(s_in):
                    if state["prev_comp"][c] is not None:
                        s_in.wait_event(state["prev_comp"][c])     # chunk buffers still read by the last step
                    zdev[sl].copy_(zh[sl], non_blocking=True)
                    godev[sl].copy_(goh[sl], non_blocking=True)
                    ev_in = torch.cuda.Event()
                    ev_in.record(s_in)
                with torch.cuda.stream(s_comp):
                    s_comp.wait_event(ev_in)
                    zz = zdev[sl].detach().requires_grad_(True)
                    if world == 1:
                        f = flash_spline_feature(zz, C, lo, hi, G, "relu_sq", lam, True)
                    else:
                        f = sharded.token_sharded_spline_feature(zz, C, lo, hi, G, "relu_sq", lam)
                    f.backward(godev[sl])
                    ev_c = torch.cuda.Event()
                    ev_c.record(s_comp)
                    state["prev_comp"][c] = ev_c
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_c)
                    fh[sl].copy_(f.detach(), non_blocking=True)
                    dzh[sl].copy_(zz.grad, non_blocking=True)
                    f.record_stream(s_out)
                    zz.grad.record_stream(s_out)
                keep.append((f, zz))
            with torch.cuda.stream(s_out):
                s_out.wait_stream(s_comp)
                dCh.copy_(C.grad, non_blocking=True)
                C.grad.record_stream(s_out)
            cur.wait_stream(s_out)
            cur.wait_stream(s_comp)

        for _ in range(2):
            step_e2e()
        e2e_steps = max(2, min(args.steps, 5))
        e2e_ms = timed(step_e2e, e2e_steps) / e2e_steps
        h2d = zh.numel() * 2 + goh.numel() * 2
        d2h = fh.numel() * 2 + dzh.numel() * 2 + dCh.numel() * 2
        e2e = dict(value=world * N / (e2e_ms * 1e-3), unit="tokens/s", h2d_bytes_per_step=h2d,
                   d2h_bytes_per_step=d2h, ms_per_step=e2e_ms, token_chunks=NCH,
                   host_cores_local_to_gpu=(len(local_cores) if local_cores else 0),
                   bound="host link: every rank streams its inputs and outputs through the host's PCIe root and "
                         "memory, so this figure does not scale with the GPU count; `value` is the device-side one")
        ops.check_status(dev)
        del zh, goh, fh, dzh, dCh, zdev, godev

    parity, extra = None, None
    if not args.no_extra:
        parity = parity_record(torch, dist, ops, sharded, z, C, go, cfg, rank, world, dev)
        C.grad = None
        z.grad = None
        del go
        z = z.detach()
        torch.cuda.empty_cache()
        extra = dict(
            key_sharded=extra_key_sharded(torch, dist, ops, sharded, cfg, rank, world, dev, timed),
            sweep=extra_sweep(torch, ops, cfg, rank, dev, timed),
            readout=extra_readout(torch, ops, cfg, rank, dev, timed),
            stack7=extra_stack7(torch, dist, sharded, flash_spline_feature, cfg, kern, rank, world, dev, timed))
        ops.check_status(dev)

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        v, n, t, threads = cpu_port_tokens_per_s(cfg, seed=0)
        cpu_baseline = dict(value=v, unit="tokens/s", cores=threads, kind="port",
                            sample=f"{n} of {N} tokens, same h/r/G, fwd+bwd, {t:.1f} s")

    if rank == 0:
        line = dict(metric=METRIC, value=value, unit="tokens/s", n_gpus=world, steps=args.steps, warmup=args.warmup,
                    ms_per_step=ms_per_step, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="bf16",
                    data="synthetic", config=cfg_json(cfg, world), kernels=impl, out_of_grid_fraction=oor,
                    clocks=clocks, e2e=e2e, gpu_launches=launches, roofline=roofline, cpu_baseline=cpu_baseline,
                    parity=parity, extra=extra)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# -------------------------------------------------------------------------------------------------
# records taken after the timed region
# -------------------------------------------------------------------------------------------------
def _stats(test, ref):
    """maxabs(diff)/maxabs(ref), mean signed error, and the latter relative to max(1, maxabs(ref))."""
    import numpy as np
    t = np.asarray(test, dtype=np.float64)
    r = np.asarray(ref, dtype=np.float64)
    ref_max = float(np.abs(r).max())
    d = t - r
    bias = float(d.mean())
    return dict(rel=float(np.abs(d).max() / max(ref_max, 1e-30)), mean_signed=bias,
                mean_signed_rel=bias / max(1.0, ref_max), ref_max=ref_max)


def parity_record(torch, dist, ops, sharded, z, C, go, cfg, rank, world, dev):
    """The operator against the CPU oracle on the first PARITY_TOKENS tokens of this rank's batch;
    on more than one GPU also the collective: the all-reduced dC against the float64 sum of the
    all-gathered per-rank float32 dC.  Gates: 0 index mismatches, rel <= 1e-2, |mean signed| <= 5e-6
    (relative to maxabs(ref) where that exceeds 1)."""
    import numpy as np
    from oracle import c_binding as oc
    oc.build()
    oc.set_threads(len(os.sched_getaffinity(0)))
    h, G, r = cfg["h"], cfg["G"], cfg["r"]
    lo, hi, lam = cfg["grid_lo"], cfg["grid_hi"], cfg["lambda_scale"]
    n = min(PARITY_TOKENS, z.shape[0])
    zs, gos, Cd = z.detach()[:n], go[:n], C.detach()
    z32, C32, go32 = zs.float().cpu().numpy(), Cd.float().cpu().numpy(), gos.float().cpu().numpy()
    bins = ops.knot_index(zs, lo, hi, G).cpu().numpy()
    mism = int((bins != oc.knot_index(z32, lo, hi, G)).sum())
    _, d32 = ops.feature_forward(zs, Cd, lo, hi, G, "relu_sq", lam, delta_f32=True)
    dz, dC32, _ = ops.feature_backward(zs, Cd, gos, lo, hi, G, "relu_sq", lam)
    _, d_ref = oc.feature_forward(z32, C32, lo, hi, G, "relu_sq", lam)
    dz_ref, dC_ref = oc.feature_backward(z32, C32, go32[:, h:], go32[:, :h], lo, hi, G, "relu_sq", lam)
    rec = dict(tokens=n, knot_index_mismatches=mism, delta_f32=_stats(d32.cpu().numpy(), d_ref),
               dz=_stats(dz.float().cpu().numpy(), dz_ref), dC_f32=_stats(dC32.cpu().numpy(), dC_ref))
    ok = mism == 0 and all(rec[k]["rel"] <= 1e-2 for k in ("delta_f32", "dz", "dC_f32")) and all(
        abs(rec[k]["mean_signed_rel"]) <= 5e-6 for k in ("delta_f32", "dC_f32"))
    if world > 1:
        # every rank's own dC of its whole batch, gathered, summed in float64, against the operator's
        # all-reduced result
        _, mine, _ = ops.feature_backward(z.detach(), Cd, go, lo, hi, G, "relu_sq", lam, need_dz=False)
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)
        total = torch.zeros_like(mine, dtype=torch.float64)
        for p in parts:
            total += p.double()
        zz = z.detach().requires_grad_(False)
        Cg = Cd.clone().requires_grad_(True)
        f = sharded.token_sharded_spline_feature(zz, Cg, lo, hi, G, "relu_sq", lam)
        f.backward(go)
        diff = (Cg.grad.double() - total).abs().max().item()
        ref_max = total.abs().max().item()
        rec["allreduced_dC_vs_f64_sum_of_ranks"] = dict(rel=diff / max(ref_max, 1e-30), ref_max=ref_max,
                                                        ranks=world, rounding="result is bf16 (dtype of C)")
        ok = ok and diff <= 1e-2 * ref_max
        flag = torch.tensor([1 if ok else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        ok = bool(flag.item())
    rec["within_gates_on_all_ranks"] = ok
    return rec


def extra_key_sharded(torch, dist, ops, sharded, cfg, rank, world, dev, timed, N=131072, steps=5):
    """The key-sharded mode at the rank/grid sweep's token count: every rank holds all N tokens and
    h / P keys; the partial residuals are all-reduced in float32.  Timing of forward + backward, and
    the all-reduced residual against the unsharded operator on a replicated 2048-token subset."""
    h, G, r = cfg["h"], cfg["G"], cfg["r"]
    lo, hi, lam = cfg["grid_lo"], cfg["grid_hi"], cfg["lambda_scale"]
    ks = sharded.key_slice(h, world, rank, multiple=16)
    hl = ks.stop - ks.start
    cgen = torch.Generator(device=dev).manual_seed(4242)         # replicated tensors: same seed on all ranks
    C = (torch.randn(h, G + 2, r, generator=cgen, device=dev) * 0.02).to(torch.bfloat16)
    zsub = (torch.randn(2048, h, generator=cgen, device=dev) * cfg["z_std"]).to(torch.bfloat16)
    _, d_full = ops.feature_forward(zsub, C, lo, hi, G, "relu_sq", lam, delta_f32=True)
    _, d_sh = sharded.key_sharded_spline_feature(zsub[:, ks].contiguous(), C[ks].contiguous(), lo, hi, G, "relu_sq", lam)
    dmax = d_full.abs().max().item()
    rel = (d_sh.float() - d_full).abs().max().item() / max(dmax, 1e-30)
    gen = torch.Generator(device=dev).manual_seed(77 + rank)
    zl = (torch.randn(N, hl, generator=gen, device=dev) * cfg["z_std"]).to(torch.bfloat16).requires_grad_(True)
    Cl = C[ks].contiguous().requires_grad_(True)
    ga = torch.randn(N, hl, generator=gen, device=dev).to(torch.bfloat16)
    gd = torch.randn(N, r, generator=cgen, device=dev).to(torch.bfloat16)

    def step():
        zl.grad = None
        Cl.grad = None
        a, delta = sharded.key_sharded_spline_feature(zl, Cl, lo, hi, G, "relu_sq", lam)
        torch.autograd.backward([a, delta], [ga, gd])

    for _ in range(3):
        step()
    ms = timed(step, steps) / steps
    return dict(workload=f"key-sharded, N={N} tokens on every rank, {hl} of {h} keys per rank, r={r}, G={G} (config 4)",
                ms_per_step=ms, tokens_per_s=N / (ms * 1e-3), steps=steps,
                allreduced_delta_vs_unsharded=dict(rel=rel, ref_max=dmax, tokens=2048,
                                                   rounding="sharded result is bf16"),
                within_gate=rel <= 1e-2)


def extra_sweep(torch, ops, cfg, rank, dev, timed, N=131072, steps=5):
    """Kernel times of the rank/grid sweep at h = 5120, N = 131072 on this GPU: r = 16, 64, 128 at
    G = 20 and r = 32 at G = 40 (config 4; its token-sharded form is this on every rank), with the
    headline's r = 32, G = 20 beside them."""
    h = cfg["h"]
    lo, hi, lam = cfg["grid_lo"], cfg["grid_hi"], cfg["lambda_scale"]
    gen = torch.Generator(device=dev).manual_seed(555 + rank)
    z = (torch.randn(N, h, generator=gen, device=dev) * cfg["z_std"]).to(torch.bfloat16)
    out = []
    for r, G in ((16, 20), (32, 20), (64, 20), (128, 20), (32, 40)):
        C = (torch.randn(h, G + 2, r, generator=gen, device=dev) * 0.02).to(torch.bfloat16)
        go = torch.randn(N, h + r, generator=gen, device=dev).to(torch.bfloat16)
        fwd = lambda: ops.feature_forward(z, C, lo, hi, G, "relu_sq", lam)
        bwd = lambda: ops.feature_backward(z, C, go, lo, hi, G, "relu_sq", lam)
        for _ in range(2):
            fwd()
            bwd()
        f_ms = timed(fwd, steps) / steps
        b_ms = timed(bwd, steps) / steps
        flops = 2.0 * N * h * (G + 2) * r
        out.append(dict(r=r, G=G, N=N, forward_ms=round(f_ms, 4), backward_ms=round(b_ms, 4),
                        tokens_per_s=N / ((f_ms + b_ms) * 1e-3),
                        dense_equiv_tflops=round(3 * flops / ((f_ms + b_ms) * 1e-3) / 1e12, 1)))
        del C, go
    return out


def extra_readout(torch, ops, cfg, rank, dev, timed, steps=10):
    """Forward followed by the read-out projection y = f W_out^T at the d20 shape (d_out = h / 4) on
    this GPU: the fused entry point (delta-only feature kernels + this library's tcgen05 GEMM with the
    activation applied to the z tile in shared memory; f is never written) beside the two-step path
    (feature kernels + a torch matmul, i.e. the cuBLAS GEMM)."""
    N, h, r, G = cfg["N"], cfg["h"], cfg["r"], cfg["G"]
    lo, hi, lam = cfg["grid_lo"], cfg["grid_hi"], cfg["lambda_scale"]
    D = h // 4
    gen = torch.Generator(device=dev).manual_seed(777 + rank)
    z = (torch.randn(N, h, generator=gen, device=dev) * cfg["z_std"]).to(torch.bfloat16)
    C = (torch.randn(h, G + 2, r, generator=gen, device=dev) * 0.02).to(torch.bfloat16)
    W = (torch.randn(D, h + r, generator=gen, device=dev) * 0.02).to(torch.bfloat16)
    Wt = W.t()
    out = {}
    for act in ("relu_sq", "identity"):
        fused = lambda: ops.feature_readout_forward(z, C, W, lo, hi, G, act, lam)
        two_step = lambda: ops.feature_forward(z, C, lo, hi, G, act, lam) @ Wt
        delta_only = lambda: ops.feature_forward(z, C, lo, hi, G, act, lam, with_base=False)
        feature = lambda: ops.feature_forward(z, C, lo, hi, G, act, lam)
        ms = {}
        for name, fn in (("fused", fused), ("two_step", two_step), ("delta_only", delta_only), ("feature", feature)):
            for _ in range(3):
                fn()
            ms[name] = timed(fn, steps) / steps
        y1, y2 = fused().double(), two_step().double()
        flops = 2.0 * N * (h + r) * D
        gemm_ms = ms["fused"] - ms["delta_only"]
        out[act] = dict(N=N, d_out=D, fused_ms=round(ms["fused"], 4), two_step_ms=round(ms["two_step"], 4),
                        delta_only_ms=round(ms["delta_only"], 4), feature_ms=round(ms["feature"], 4),
                        readout_gemm_ms=round(gemm_ms, 4), library_gemm_ms=round(ms["two_step"] - ms["feature"], 4),
                        readout_gemm_tflops=round(flops / (gemm_ms * 1e-3) / 1e12, 1),
                        rel_norm_vs_two_step=float((y1 - y2).norm() / y2.norm()))
        del y1, y2
    return out


def extra_stack7(torch, dist, sharded, flash_spline_feature, cfg, kern, rank, world, dev, timed, layers=7, steps=3):
    """Seven consecutive layers x -> z = x W_in -> f = feature(z, C) -> y = f W_out^T, x <- x + y at
    the d20 shape (config 3), forward then backward through all of them, N = 65536 tokens per GPU;
    the GEMMs are torch (cuBLAS) bf16 matmuls, the operator is this library's; on more than one GPU
    every layer's dC is all-reduced by the token-sharded operator and the W gradients in one call."""
    N, d, h, G, r = cfg["N"], cfg["d"], cfg["h"], cfg["G"], cfg["r"]
    lo, hi, lam = cfg["grid_lo"], cfg["grid_hi"], cfg["lambda_scale"]
    wgen = torch.Generator(device=dev).manual_seed(31337)         # weights are replicated
    gen = torch.Generator(device=dev).manual_seed(9 + rank)
    bf = torch.bfloat16
    W_in = [(torch.randn(d, h, generator=wgen, device=dev) / d ** 0.5).to(bf).requires_grad_(True) for _ in range(layers)]
    # small read-out weights keep the residual stream (there is no normalisation in this stack) inside the grid
    W_out = [(torch.randn(h + r, d, generator=wgen, device=dev) * 0.05 / (h + r) ** 0.5).to(bf).requires_grad_(True)
             for _ in range(layers)]
    Cs = [(torch.randn(h, G + 2, r, generator=wgen, device=dev) * 0.02).to(bf).requires_grad_(True) for _ in range(layers)]
    x0 = (torch.randn(N, d, generator=gen, device=dev) * cfg["z_std"]).to(bf)
    gy = torch.randn(N, d, generator=gen, device=dev).to(bf)
    params = W_in + W_out + Cs

    def step():
        for p in params:
            p.grad = None
        x = x0
        for l in range(layers):
            z = x @ W_in[l]
            if world == 1:
                f = flash_spline_feature(z, Cs[l], lo, hi, G, "relu_sq", lam, True)
            else:
                f = sharded.token_sharded_spline_feature(z, Cs[l], lo, hi, G, "relu_sq", lam)
            x = x + f @ W_out[l]
        x.backward(gy)
        if world > 1:
            flat = torch.cat([w.grad.reshape(-1) for w in W_in + W_out]).float()
            dist.all_reduce(flat)

    for _ in range(2):
        step()
    ms = timed(step, steps) / steps
    op_ms = layers * (kern["forward"] + kern["backward"])
    return dict(workload=f"{layers} layers with W_in [d,h] and W_out [h+r,d] GEMMs, N={N} tokens per GPU (config 3)",
                ms_per_step=ms, tokens_per_s=world * N / (ms * 1e-3), steps=steps,
                operator_ms=round(op_ms, 3), operator_share=round(op_ms / ms, 3),
                note="operator_ms = layers x (forward + backward kernel time measured alone above)")


if __name__ == "__main__":
    main()
