#!/usr/bin/env python
"""Benchmark of the attention hot path.  One JSON line on stdout (rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

A step is one pass of the hot path over one batch of seeded synthetic input: Q/K preparation (RMSNorm +
rotation [+ e4m3 quantisation]) followed by the attention forward, on the 480p-like joint sequence
(49,384 tokens = 1,024 audio + 31x30x52 video, 40 heads, d = 128) unless --workload says otherwise.
`value` counts 4*Lq*Lk*d*H*density FLOPs per step; inputs are resident in HBM when the timed region
starts.  `e2e` is the same step driven from pinned HOST buffers (H2D of Q, K, V and D2H of the output
inside the timed region).  With N > 1 (launched by torchrun, one rank per GPU) the same total work is
split Ulysses-style: each rank holds L/N tokens, two all-to-all exchanges bracket the local attention.
`--impl reference` times the CPU oracle (the restatement of the reference's attention, all host threads)
on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (grid, n_audio, heads, mode, window, seed)
    "cfg1_dense": ((31, 30, 52), 1024, 40, "dense_bf16", None, 1001),
    "cfg2_fp8": ((31, 30, 52), 1024, 40, "fp8_qk", None, 1001),
    "cfg3_sparse": ((31, 48, 84), 1024, 40, "block_sparse", (2, 8, 8), 1003),
    "cfg3_sparse20": ((31, 48, 84), 1024, 40, "block_sparse", (3, 48, 84), 1003),
    "cfg0_dense": ((4, 32, 32), 0, 8, "dense_bf16", None, 1000),
    # config 4's cross-attention: the 49,384 joint tokens attend to 512 text tokens (already projected to 40 x 128)
    "cfg4_cross": ((31, 30, 52), 1024, 40, "cross_bf16", None, 1004),
    # small cases for profiler captures: inputs above the L2 size, a few ms per launch
    "prof_dense": ((15, 32, 32), 1024, 16, "dense_bf16", None, 2001),
    "prof_fp8": ((15, 32, 32), 1024, 16, "fp8_qk", None, 2001),
    "prof_sparse": ((31, 32, 32), 1024, 16, "block_sparse", (3, 32, 32), 2003),
}
# dram__bytes_read.sum + dram__bytes_write.sum of one attention-kernel launch, from the ncu captures summarised
# under profiles/ (None until a capture of that workload exists)
NCU_TRAFFIC_BYTES = {
    "prof_dense": 250.9e6,           # measured: the ncu capture of this workload summarised under profiles/
    "cfg1_dense": 250.9e6 * 7.535,   # the same capture scaled by the units per launch (L*H: 49,384*40 / 16,384*16)
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["bf16_tflops"]), float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "measured"
    return 1590.0, 1400.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons every 200 ms while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200", "-i", str(self.gpu)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def workload_dims(name):
    grid, n_audio, H, mode, window, seed = WORKLOADS[name]
    L = n_audio + grid[0] * grid[1] * grid[2]
    return grid, n_audio, L, H, mode, window, seed


# ------------------------------------------------------------------------------------------------ CPU oracle arm
def cpu_oracle_sample(name: str, target_seconds: float = 15.0, threads: int | None = None):
    """Time the CPU oracle (fp32, all host threads) on a bounded sample of query rows of the workload against
    the full key range.  Returns (tflops, cores, sample description, seconds)."""
    from oracle import oracle as O

    grid, n_audio, L, H, mode, window, seed = workload_dims(name)
    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    Hs = min(H, 4)  # heads in the sample (per-head work is identical)
    g = torch.Generator().manual_seed(seed)
    cross = mode == "cross_bf16"
    Lk = 512 if cross else L
    k = torch.randn(Lk, Hs, 128, generator=g)
    v = torch.randn(Lk, Hs, 128, generator=g)
    pos = O.make_positions(grid, n_audio)
    cos, sin = O.rope_table(pos)
    csr = None
    density = 1.0
    if mode == "block_sparse":
        import pika_h3_flex_b200 as h3

        bi = h3.build_block_index(grid, n_audio, window)  # host-only call
        csr = (bi.row_ptr.numpy(), bi.col_idx.numpy())
        density = bi.density

    def run(n_rows):
        rows = torch.linspace(0, L - 1, n_rows).long()
        q = torch.randn(L, Hs, 128, generator=torch.Generator().manual_seed(seed + 1))
        t0 = time.perf_counter()
        # preparation of the sampled rows and of all keys, then exact attention for the sampled rows
        if cross:
            qn, kn = O.rms_norm(q[rows]), O.rms_norm(k)
        else:
            qn = O.apply_rope(O.rms_norm(q[rows]), cos[rows], sin[rows])
            kn = O.apply_rope(O.rms_norm(k), cos, sin)
        if mode == "fp8_qk":
            kq, sk = O.quantize_e4m3_blocks(kn)
            kn = O.dequantize_blocks(kq, sk)
        if csr is None:
            O.attention(qn, kn, v, chunk=512)
        else:
            full_q = torch.zeros(L, Hs, 128)
            full_q[rows] = qn
            O.attention(full_q, kn, v, csr=csr, q_rows=rows, chunk=512)
        dt = time.perf_counter() - t0
        flops = 4.0 * n_rows * Lk * 128 * Hs
        return dt, flops

    run(64)  # warm-up (thread pool, allocator)
    dt, flops = run(256)
    n_rows = int(max(256, min(L, 256 * target_seconds / max(dt, 1e-3))))
    dt, flops = run(n_rows)
    # the masked oracle still evaluates full rows, so its useful FLOPs are scaled by the density
    tflops = flops * density / dt / 1e12
    return tflops, threads, f"{n_rows} query rows x {Hs} heads x all {Lk} keys of {name} (prep + exact softmax attention, fp32)", dt


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    name = args.workload
    grid, n_audio, L, H, mode, window, seed = workload_dims(name)
    Lk = 512 if mode == "cross_bf16" else L
    per_step = max(2.0, min(20.0, 90.0 / max(1, args.steps + args.warmup)))
    vals, times = [], []
    cores = os.cpu_count() or 1
    sample = ""
    for i in range(args.warmup + args.steps):
        tf, cores, sample, dt = cpu_oracle_sample(name, per_step)
        if i >= args.warmup:
            vals.append(tf)
            times.append(dt)
    value = sum(vals) / len(vals)
    line = {
        "impl": "reference", "metric": "attention_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * sum(times) / len(times),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": name, "L": L, "Lk": Lk, "H": H, "d": 128, "mode": mode,
                   "note": "CPU restatement of the reference attention (oracle); each step is a bounded sample"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------ GPU arm
def run_ours(args):
    import torch.distributed as dist

    import pika_h3_flex_b200 as h3
    from pika_h3_flex_b200 import _lib
    from pika_h3_flex_b200.ulysses import UlyssesAttention

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torchrun (one rank per GPU)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    torch.backends.cuda.matmul.allow_tf32 = False

    name = args.workload
    grid, n_audio, L, H, mode_name, window, seed = workload_dims(name)
    mode = {"dense_bf16": _lib.MODE_DENSE_BF16, "fp8_qk": _lib.MODE_FP8_QK, "block_sparse": _lib.MODE_BLOCK_SPARSE,
            "cross_bf16": _lib.MODE_DENSE_BF16}[mode_name]
    if L % world:
        raise SystemExit(f"sequence length {L} does not split over {world} ranks")
    Ls = L // world
    from pika_h3_flex_b200.layout import position_grid

    pos = position_grid(grid, n_audio)[rank * Ls : (rank + 1) * Ls]
    g = torch.Generator(device=dev).manual_seed(seed + rank)
    q = torch.randn(Ls, H, 128, device=dev, generator=g).bfloat16()
    k = torch.randn(Ls, H, 128, device=dev, generator=g).bfloat16()
    v = torch.randn(Ls, H, 128, device=dev, generator=g).bfloat16()
    rope = h3.rope_table(pos.to(dev))
    bi = None
    density = 1.0
    if mode == _lib.MODE_BLOCK_SPARSE:
        bi_host = h3.build_block_index(grid, n_audio, window)
        density = bi_host.density
        bi = bi_host.to(dev)
    cross = mode_name == "cross_bf16"
    Lk = 512 if cross else L
    if cross and world > 1:
        raise SystemExit("cross-attention needs no exchange: run it per rank with --gpus 1")
    flops = 4.0 * L * Lk * 128 * H * density
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    attn_events = []

    from pika_h3_flex_b200.ops import normed_logit_bound

    bound = 0.0 if args.online_max else normed_logit_bound(fp8=(mode == _lib.MODE_FP8_QK))  # unit-weight QK-RMSNorm
    if world == 1:
        out = torch.empty(L, H, 128, dtype=torch.bfloat16, device=dev)
        if bi is not None:
            ws = torch.empty((bi.nnz + (L + 255) // 256) * 4 + 16, dtype=torch.uint8, device=dev)
            split_bytes = 0
        else:  # optional scratch: the CTA pairs of the last, partly filled wave split the key range
            from pika_h3_flex_b200.ops import split_workspace_bytes
            split_bytes = split_workspace_bytes(L, Lk, H, mode, bound)
            ws = torch.empty(max(16, split_bytes), dtype=torch.uint8, device=dev)

        if cross:  # keys and values are the text tokens; QK-RMSNorm without rotation
            k = k[:Lk].contiguous()
            v = v[:Lk].contiguous()

        def step(record=False):
            qp, kp, qs, ks = h3.qk_prep(q, k, None if cross else rope, None if cross else rope, fp8=(mode == _lib.MODE_FP8_QK))
            if record:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            h3.attn_fwd(qp, kp, v, mode, qs, ks, bi, out=out, status_word=status, workspace=ws, logit_bound=bound)
            if record:
                e1.record()
                attn_events.append((e0, e1))
            return out

        # prep (2) + attention (1) [+ plan | + combine of the split last wave]; V is used where it lies
        launches_per_step = 3 + (1 if bi is not None else 0) + (1 if split_bytes else 0)
    else:
        ua = UlyssesAttention(None, mode, bi, head_groups=args.head_groups)

        def step(record=False):
            return ua(q, k, v, rope)

        # prep (2) + V head-major copy (1, torch) + attention (1) [+ plan]; only this library's kernels are counted
        launches_per_step = 3 + (1 if bi is not None else 0)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(3, args.warmup)):
        step()
    barrier()
    if h3.read_status(status) != 0:
        raise SystemExit(f"device wait gave up during warm-up: status 0x{h3.read_status(status):x}")

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    barrier()
    e_start, e_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e_start.record()
    for _ in range(args.steps):
        step(record=True)
    e_stop.record()
    barrier()
    elapsed_ms = e_start.elapsed_time(e_stop)
    if world > 1:
        t = torch.tensor([elapsed_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    ms_per_step = elapsed_ms / args.steps
    # nvidia-smi delivers a sample every 200 ms: a timed region shorter than about a second holds too few of them,
    # so the same steps keep running (untimed, every rank alike) until the record covers 1.5 s of this load
    extra_steps = 0
    if elapsed_ms < 1000.0:
        extra_steps = int(1500.0 / max(ms_per_step, 1e-3)) + 1
        for _ in range(extra_steps):
            step()
        barrier()
    clocks = sampler.stop() if rank == 0 else None
    if clocks is not None and extra_steps:
        clocks["note"] = f"timed region {elapsed_ms:.0f} ms: sampling continued over {extra_steps} identical untimed steps"
    value = flops / (ms_per_step * 1e-3) / 1e12
    if h3.read_status(status) != 0:
        raise SystemExit(f"device wait gave up: status 0x{h3.read_status(status):x}")

    # ---- dominant kernel, timed live with CUDA events on the launching stream
    roofline = None
    if attn_events:
        attn_ms = sum(a.elapsed_time(b) for a, b in attn_events) / len(attn_events)
        burst, sustained, src = measured_peaks()
        achieved = flops / (attn_ms * 1e-3) / 1e12
        # which kernel the library picks: CTA pairs with a logit bound, from 16 key tiles and (sparse) 12 % density up
        pair = (not args.online_max and os.environ.get("H3A_PAIR", "1")[:1] != "0" and (Lk + 127) // 128 >= 16
                and (mode_name != "block_sparse" or density >= 0.12))
        roofline = {"bound": "tensor", "kernel": "attn_fwd_pair_kernel" if pair else "attn_fwd_kernel", "achieved": achieved, "peak": burst, "unit": "TFLOP/s",
                    "frac": achieved / burst, "peak_source": f"bf16 burst, of {src}", "frac_of_sustained": achieved / sustained,
                    "frac_of_spec_2250": achieved / 2250.0, "kernel_ms": attn_ms, "traffic": NCU_TRAFFIC_BYTES.get(name)}

    # ---- end to end from host buffers through the public call
    e2e = None
    if world == 1 and cross:
        e2e = {"value": None, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
               "note": "host-buffer end-to-end is measured on the self-attention workloads"}
    elif world == 1:
        hq, hk, hv = (torch.empty(L, H, 128, dtype=torch.bfloat16).pin_memory() for _ in range(3))
        for dst, src_t in ((hq, q), (hk, k), (hv, v)):
            dst.copy_(src_t)
        ho = torch.empty(L, H, 128, dtype=torch.bfloat16).pin_memory()
        host_attn = h3.HostJointAttention(L, H, mode, bi)  # the public host-buffer call: pipelined over head groups
        torch.cuda.synchronize()

        def e2e_step():
            host_attn(hq, hk, hv, rope, ho)

        n_e2e = max(2, min(args.steps, 5))
        e2e_step()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n_e2e):
            e2e_step()
        b.record()
        torch.cuda.synchronize()
        e2e_ms = a.elapsed_time(b) / n_e2e
        nbytes = L * H * 128 * 2
        e2e = {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": 3 * nbytes,
               "d2h_bytes_per_step": nbytes, "ms_per_step": e2e_ms, "steps": n_e2e,
               "api": "HostJointAttention: H2D, prep+attention and D2H pipelined over head groups %s" % host_attn.groups}
    elif mode == _lib.MODE_FP8_QK or cross:
        e2e = {"value": None, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
               "note": "the multi-GPU host-buffer path covers the dense bf16 and block-sparse self-attention workloads"}
    else:
        try:
            # every rank's shard comes from its own pinned host buffers and goes back to one
            from pika_h3_flex_b200.host_path import HostUlyssesAttention

            hq, hk, hv = (torch.empty(Ls, H, 128, dtype=torch.bfloat16).pin_memory() for _ in range(3))
            for dst, src_t in ((hq, q), (hk, k), (hv, v)):
                dst.copy_(src_t)
            ho = torch.empty(Ls, H, 128, dtype=torch.bfloat16).pin_memory()
            host_attn = HostUlyssesAttention(Ls, H, mode, bi)
            barrier()
            n_e2e = max(2, min(args.steps, 5))
            for _ in range(2):
                host_attn(hq, hk, hv, rope, ho)
            barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(n_e2e):
                host_attn(hq, hk, hv, rope, ho)
            b.record()
            barrier()
            t = torch.tensor([a.elapsed_time(b) / n_e2e], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = float(t.item())
            nbytes = L * H * 128 * 2  # over all ranks
            e2e = {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": 3 * nbytes,
                   "d2h_bytes_per_step": nbytes, "ms_per_step": e2e_ms, "steps": n_e2e,
                   "api": "HostUlyssesAttention: per rank, H2D of its shard, prep, exchanges, attention and D2H pipelined over head-slot groups %s"
                          % host_attn.slot_groups}
            if h3.read_status(status) != 0:
                raise SystemExit(f"device wait gave up: status 0x{h3.read_status(status):x}")
        except (RuntimeError, ValueError, TypeError, AttributeError, NotImplementedError) as exc:  # keep the kernel-side line
            e2e = {"value": None, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                   "note": "multi-GPU host-buffer path failed: %r" % (exc,)}

    if world > 1:
        dist.barrier()
    if rank == 0:
        cpu_baseline = None
        if world == 1 and not args.no_cpu_baseline:
            tf, cores, sample, _ = cpu_oracle_sample(name, args.cpu_seconds)
            cpu_baseline = {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample}
        line = {
            "metric": "attention_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16" if mode != _lib.MODE_FP8_QK else "e4m3(QK)+bf16(PV)", "data": "synthetic",
            "config": {"workload": name, "L": L, "Lk": Lk, "H": H, "d": 128, "mode": mode_name, "density": density,
                       "flops_per_step": flops, "step": "qk_prep(RMSNorm+RoPE) + attention forward",
                       "softmax_reference": "running row maximum" if bound == 0.0 else "fixed logit bound %.2f from QK-RMSNorm" % bound,
                       "parallelism": "single GPU" if world == 1 else f"ulysses{world} (seq<->head all-to-all, NCCL)",
                       "l2": "inputs (Q,K,V = %.0f MB per rank) exceed the 126 MB L2; no flush" % (3 * Ls * H * 256 / 1e6)},
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e, "clocks": clocks,
            "gpu_launches": launches_per_step * args.steps,
            "attn_ms_per_dit_step_per_layer": ms_per_step,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------ projection workloads
# The Q/K/V projections feeding the attention (section "next" of the scope: LoRA-wrapped Linears with the
# preparation fused into the GEMM epilogue).  Not the headline metric: a side workload with its own roofline line.
PROJ_WORKLOADS = {
    # name: (tokens, model width, heads, LoRA rank)
    "cfg1_qkv_proj": (49384, 5120, 40, 128),
    "prof_qkv_proj": (8192, 5120, 40, 128),
}


def run_projection(args):
    import torch

    import pika_h3_flex_b200 as h3
    from oracle import oracle as O

    L, D, H, R = PROJ_WORKLOADS[args.workload]
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev).manual_seed(3001)
    x = torch.randn(L, D, device=dev, generator=g).bfloat16()
    ws = [(torch.randn(H * 128, D, device=dev, generator=g) / D ** 0.5).bfloat16() for _ in range(3)]
    las = [(torch.randn(R, D, device=dev, generator=g) / D ** 0.5).bfloat16() for _ in range(3)]
    lbs = [(0.5 * torch.randn(H * 128, R, device=dev, generator=g) / R ** 0.5).bfloat16() for _ in range(3)]
    # positions: config 1's grid when L is its length, otherwise frames of 8 x 8 tokens plus audio
    if L == 31 * 30 * 52 + 1024:
        pos = O.make_positions((31, 30, 52), 1024)
    else:
        frames = (L - 1024) // 64
        pos = O.make_positions((frames, 8, 8), L - frames * 64)
    rope = h3.rope_table(pos.to(dev))
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    events = []

    def step(record=False):
        outs = []
        for i in range(3):
            t = torch.nn.functional.linear(x, las[i])  # the thin LoRA product x A^T (torch / cuBLAS)
            if record:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            outs.append(h3.proj_fwd(x, ws[i], None, t, lbs[i], prep=(i < 2), rope=rope if i < 2 else None, status_word=status))
            if record:
                e1.record()
                events.append((e0, e1))
        return outs

    for _ in range(max(3, args.warmup)):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    sampler.start()
    e_start, e_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e_start.record()
    for _ in range(args.steps):
        step(record=True)
    e_stop.record()
    torch.cuda.synchronize()
    elapsed_ms = e_start.elapsed_time(e_stop)
    ms_per_step = elapsed_ms / args.steps
    extra = 0
    if elapsed_ms < 1000.0:
        extra = int(1500.0 / max(ms_per_step, 1e-3)) + 1
        for _ in range(extra):
            step()
        torch.cuda.synchronize()
    clocks = sampler.stop()
    if extra:
        clocks["note"] = f"timed region {elapsed_ms:.0f} ms: sampling continued over {extra} identical untimed steps"
    if h3.read_status(status) != 0:
        raise SystemExit(f"device wait gave up: status 0x{h3.read_status(status):x}")
    flops_kernel = 3 * 2.0 * L * (H * 128) * (D + R)       # the library's GEMMs (main + LoRA columns)
    flops_step = flops_kernel + 3 * 2.0 * L * D * R        # + the thin products done by torch
    kernel_ms = sum(a.elapsed_time(b) for a, b in events) / len(events)
    burst, sustained, src = measured_peaks()
    achieved = (flops_kernel / 3) / (kernel_ms * 1e-3) / 1e12
    # torch reference of the same step on the same box: Linear + LoRA update + the separate preparation kernel
    def torch_step():
        for i in range(3):
            y = torch.nn.functional.linear(x, ws[i]) + torch.nn.functional.linear(torch.nn.functional.linear(x, las[i]), lbs[i])
            y = y.view(L, H, 128)
            if i < 2:
                h3.qk_prep(y if i == 0 else None, y if i == 1 else None, rope if i == 0 else None, rope if i == 1 else None)
            else:
                y.permute(1, 0, 2).contiguous()
    for _ in range(3):
        torch_step()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(5):
        torch_step()
    t1.record()
    torch.cuda.synchronize()
    line = {
        "metric": "qkv_projection_tflops", "value": flops_step / (ms_per_step * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": args.workload, "L": L, "D": D, "H": H, "lora_rank": R,
                   "step": "to_q, to_k (LoRA + RMSNorm + RoPE in the epilogue) and to_v (LoRA, head-major store)",
                   "flops_per_step": flops_step, "l2": "X + W + out = %.0f MB per projection exceed the 126 MB L2; no flush" % ((2 * L * D * 2 + D * D * 2) / 1e6)},
        "roofline": {"bound": "tensor", "kernel": "qkv_proj_kernel", "achieved": achieved, "peak": burst, "unit": "TFLOP/s",
                     "frac": achieved / burst, "peak_source": f"bf16 burst, of {src}", "frac_of_sustained": achieved / sustained,
                     "kernel_ms": kernel_ms, "traffic": None},
        "torch_same_step_ms": t0.elapsed_time(t1) / 5, "cpu_baseline": None, "e2e": None, "clocks": clocks,
        "gpu_launches": 3 * args.steps,
    }
    print(json.dumps(line), flush=True)


def run_adaln(args):
    """Side workload: the pre-attention adaptive layer norm at the 480p-like length (HBM-bound)."""
    import torch

    import pika_h3_flex_b200 as h3

    L, D, T = 49384, 5120, 6
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev).manual_seed(3002)
    x = torch.randn(L, D, device=dev, generator=g).bfloat16()
    mod = (0.3 * torch.randn(T, 2 * D, device=dev, generator=g)).bfloat16()
    shift, scale = mod.chunk(2, dim=-1)
    idx = torch.randint(0, T, (L,), device=dev, generator=g)
    out = torch.empty_like(x)
    for _ in range(max(3, args.warmup)):
        h3.adaln_norm(x, scale, shift, idx, out=out)
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        h3.adaln_norm(x, scale, shift, idx, out=out)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    extra = int(1500.0 / max(ms, 1e-3)) + 1
    for _ in range(extra):
        h3.adaln_norm(x, scale, shift, idx, out=out)
    torch.cuda.synchronize()
    clocks = sampler.stop()
    clocks["note"] = f"timed region {ms * args.steps:.0f} ms: sampling continued over {extra} identical untimed steps"
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    hbm, src = 6650.0, "fallback"
    if os.path.exists(path):
        with open(path) as f:
            hbm, src = float(json.load(f)["hbm_gbs"]), "measured"
    algo_bytes = 4.0 * L * D  # one bf16 read and one bf16 write of every element; the tables stay in L2
    gbs = algo_bytes / (ms * 1e-3) / 1e9
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ref = lambda: torch.nn.functional.layer_norm(x, (D,), eps=1e-6) * (1.0 + scale.index_select(0, idx)) + shift.index_select(0, idx)
    for _ in range(3):
        ref()
    t0.record()
    for _ in range(5):
        ref()
    t1.record()
    torch.cuda.synchronize()
    print(json.dumps({
        "metric": "adaln_gbytes_per_s", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup),
        "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": args.workload, "L": L, "D": D, "timestep_rows": T, "step": "LayerNorm + per-token (1 + scale) / shift modulation",
                   "l2": "x and y are 506 MB each: above the 126 MB L2; no flush"},
        "roofline": {"bound": "hbm", "kernel": "adaln_norm_kernel", "achieved": gbs, "peak": hbm, "unit": "GB/s", "frac": gbs / hbm,
                     "peak_source": f"copy bandwidth, of {src}", "traffic": None},
        "torch_same_step_ms": t0.elapsed_time(t1) / 5, "cpu_baseline": None, "e2e": None, "clocks": clocks, "gpu_launches": args.steps,
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS) + sorted(PROJ_WORKLOADS) + ["cfg1_adaln"], default="cfg1_dense")
    ap.add_argument("--cpu-seconds", type=float, default=15.0, help="target CPU time of the cpu_baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--head-groups", type=int, default=2, help="N > 1: head groups the exchanges are pipelined over (1 = no overlap)")
    ap.add_argument("--online-max", action="store_true", help="use the running-maximum kernel instead of the fixed logit bound")
    args = ap.parse_args()
    if args.workload == "cfg1_adaln":
        if args.impl == "reference" or args.gpus != 1:
            raise SystemExit("the adaptive-layer-norm workload runs on one GPU with --impl ours")
        run_adaln(args)
    elif args.workload in PROJ_WORKLOADS:
        if args.impl == "reference" or args.gpus != 1:
            raise SystemExit("projection workloads run on one GPU with --impl ours")
        run_projection(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
