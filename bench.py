#!/usr/bin/env python
"""Benchmark of the attention hot path.  One JSON line on stdout (rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

A step is one pass of the hot path over one batch of seeded synthetic input: Q/K preparation (RMSNorm +
rotation [+ e4m3 quantisation]) followed by the attention forward, on the 480p-like joint sequence
(49,384 tokens = 1,024 audio + 31x30x52 video, 40 heads, d = 128) unless --workload says otherwise.
`value` counts 4*Lq*Lk*d*H*density FLOPs per step; inputs are resident in HBM when the timed region
starts.  `e2e` is the same step driven from pinned HOST buffers (H2D of Q, K, V and D2H of the output
inside the timed region).  With N > 1 (launched by torchrun, one rank per GPU) the same total work is
split Ulysses-style: each rank holds L/N tokens of one global seeded tensor, the operands are resharded
sequence -> heads before the local attention and the output heads -> sequence after it.

Besides the contract keys the line carries
  parity     sampled query rows of THIS run's outputs (every rank's own shard; device-resident path and
             host-buffer path) against the fp64 CPU oracle on the same global seeded tensors, computed outside the
             timed region, worst rank reported;
  roofline   the attention kernel alone (CUDA events around its launches, max over ranks);
  ms_per_step_sustained / ms_x_mhz   the same steps continued for about two seconds with the SM clock
             sampled over exactly that stretch (the part runs under a 1 kW power cap);
  also       (N = 1) short runs of the other configurations, each with its own kernel time and parity verdict.
`--impl reference` times the CPU oracle (the restatement of the reference's attention, all host threads)
on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
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
    "prof_sparse7": ((31, 48, 64), 1024, 8, "block_sparse", (2, 8, 8), 2003),  # 7.3 % of tiles: the single-CTA kernel
    "prof_cross": ((15, 32, 32), 1024, 16, "cross_bf16", None, 2004),
    # one rank's share of config 1 under 8-way sequence parallelism (5 of the 40 heads, all tokens): launches of 4.5 ms
    "prof_rank8": ((31, 30, 52), 1024, 5, "dense_bf16", None, 1001),
}
ALSO = ("cfg2_fp8", "cfg3_sparse", "cfg3_sparse20", "cfg4_cross")  # N = 1: short runs next to the headline workload

# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of ONE launch of the dominant kernel, from the ncu
# capture summarised in the named file under profiles/.  An entry is (kernel the capture is of, bytes per launch of
# the CAPTURED workload, L * H of the captured workload, file).  The figure is scaled to the benchmarked workload by
# the units per launch (L * H: traffic is Q, K, V, O once per head) and reported only when the kernel that ran is the
# captured one; otherwise `traffic` is null.
NCU_TRAFFIC = {
    "dense_bf16": ("attn_fwd_pair_kernel", 250.9e6, 16384 * 16, "profiles/attn_fwd_dense_bf16_prof_dense.md"),
    # without a logit bound: both launches of the two-launch online softmax together
    "dense_bf16_online": ("attn_fwd_pair_kernel (online softmax: per-row reference, then the running maximum where needed)", 250.4e6,
                          16384 * 16, "profiles/attn_fwd_pair_online_softmax_prof_dense.md"),
    "fp8_qk": ("attn_fwd_pair_kernel", 176.4e6, 16384 * 16, "profiles/attn_fwd_pair_fp8_prof_fp8.md"),
    "cross_bf16": ("attn_fwd_pair_kernel (persistent pairs, K/V resident)", 94.6e6, 16384 * 16, "profiles/attn_fwd_cross_attention_prof_cross.md"),
    # block-sparse: only the literal-rule mask at about 7 % density on the single-CTA kernel has a capture; a launch on
    # CTA pairs (denser masks) reports null
    "block_sparse": ("attn_fwd_kernel", 1113.8e6, 96256 * 8, "profiles/attn_fwd_block_sparse_7pct_prof_sparse7.md"),
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["bf16_tflops"]), float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "measured"
    return 1590.0, 1400.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons every 200 ms; `mark()` returns a position in the record so that
    a summary can cover one stretch of the run."""

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

    def mark(self) -> int:
        return len(self.lines)

    def stop(self):
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()

    def summary(self, lo: int = 0, hi: int | None = None):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines[lo:hi]:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
                pw.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "reasons": sorted(reasons), "samples": len(sm)}


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
    density = 1.0
    if mode == "block_sparse":
        import pika_h3_flex_b200 as h3

        density = h3.build_block_index(grid, n_audio, window).density
    line = {
        "impl": "reference", "metric": "attention_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * sum(times) / len(times),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": name, "L": L, "Lk": Lk, "H": H, "d": 128, "mode": mode, "density": density,
                   "flops_per_step": 4.0 * L * Lk * 128 * H * density,
                   "note": "CPU restatement of the reference attention (oracle); each step is a bounded sample of the workload "
                           "(ms_per_step is the sample's time, value its TFLOP/s)"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------ GPU arm
PARITY_HEADS = 2
BOUNDS = {"bf16": (2e-2, 2e-3, 1e-2), "fp8": (3e-2, 3e-3, 6e-2)}  # max-abs, mean-abs, rel-L2 (as in tests/test_gpu_parity.py)


class Case:
    """One workload on this rank: its shard of the global seeded operands on the device, what the oracle needs to
    rebuild sampled rows of the result on the host, and the step that runs it."""


def make_case(name, world, rank, dev, online_max=False):
    import pika_h3_flex_b200 as h3
    from pika_h3_flex_b200 import _lib
    from pika_h3_flex_b200.layout import position_grid
    from pika_h3_flex_b200.ops import normed_logit_bound

    c = Case()
    c.name = name
    grid, n_audio, L, H, mode_name, window, seed = workload_dims(name)
    c.grid, c.n_audio, c.L, c.H, c.mode_name, c.window = grid, n_audio, L, H, mode_name, window
    c.mode = {"dense_bf16": _lib.MODE_DENSE_BF16, "fp8_qk": _lib.MODE_FP8_QK, "block_sparse": _lib.MODE_BLOCK_SPARSE,
              "cross_bf16": _lib.MODE_DENSE_BF16}[mode_name]
    c.cross = mode_name == "cross_bf16"
    c.fp8 = c.mode == _lib.MODE_FP8_QK
    if L % world:
        raise SystemExit(f"sequence length {L} does not split over {world} ranks")
    c.Ls = Ls = L // world
    c.Lk = 512 if c.cross else L
    c.lo = rank * Ls
    c.heads = sorted({0, H - 1})[:PARITY_HEADS]
    # ONE global tensor per operand, the same on every rank (same seed, same generator, same draw order): a rank
    # keeps its token shard on the device and, for the parity check, the full keys / values of two heads on the host
    g = torch.Generator(device=dev).manual_seed(seed)
    shard = slice(c.lo, c.lo + Ls)
    full = torch.randn(L, H, 128, device=dev, generator=g).bfloat16()
    c.q = full[shard].clone()
    full = torch.randn(L, H, 128, device=dev, generator=g).bfloat16()
    c.k = full[: c.Lk].clone() if c.cross else full[shard].clone()
    c.k_host = full[: c.Lk][:, c.heads].cpu()
    full = torch.randn(L, H, 128, device=dev, generator=g).bfloat16()
    c.v = full[: c.Lk].clone() if c.cross else full[shard].clone()
    c.v_host = full[: c.Lk][:, c.heads].cpu()
    del full
    c.pos = position_grid(grid, n_audio)  # the whole sequence, fp32 on the host
    c.rope = None if c.cross else h3.rope_table(c.pos[shard].to(dev))
    c.bi = c.bi_host = None
    c.density = 1.0
    if c.mode == _lib.MODE_BLOCK_SPARSE:
        c.bi_host = h3.build_block_index(grid, n_audio, window)
        c.density = c.bi_host.density
        c.bi = c.bi_host.to(dev)
    c.flops = 4.0 * L * c.Lk * 128 * H * c.density
    c.bound = 0.0 if online_max else normed_logit_bound(fp8=c.fp8)  # unit-weight QK-RMSNorm
    return c


def kernel_name(c, online_max, world=1):
    """Which attention kernel the library launches for this case (asked of the library itself)."""
    from pika_h3_flex_b200.ops import kernel_choice, split_workspace_bytes

    nnz = 0 if c.bi_host is None else c.bi_host.nnz
    heads = max(1, c.H // world)
    ch = kernel_choice(c.L, c.Lk, heads, c.mode, c.bound, nnz, workspace_bytes=split_workspace_bytes(c.L, c.Lk, heads, c.mode, c.bound))
    if ch["fixed_reference"]:
        if ch.get("persistent"):
            return ch["kernel"] + (" (persistent pairs, K/V resident)" if ch["cta_pairs"] else " (persistent, one block per SM)")
        return ch["kernel"]
    return ch["kernel"] + (" (online softmax: per-row reference, then the running maximum where needed)" if ch["online_two_launch"] else " (online softmax)")


def single_gpu_step(c, status):
    """(step, events, launches per step) for one GPU: preparation + attention through the C ABI wrappers."""
    import pika_h3_flex_b200 as h3
    from pika_h3_flex_b200.ops import split_workspace_bytes

    dev = c.q.device
    out = torch.empty(c.L, c.H, 128, dtype=torch.bfloat16, device=dev)
    if c.bi is not None:
        ws = torch.empty((c.bi.nnz + (c.L + 255) // 256) * 4 + 16, dtype=torch.uint8, device=dev)
        split_bytes = 0
    else:  # optional scratch: the CTA pairs of the last, partly filled wave split the key range
        split_bytes = split_workspace_bytes(c.L, c.Lk, c.H, c.mode, c.bound)
        ws = torch.empty(max(16, split_bytes), dtype=torch.uint8, device=dev)
    events = {"prep": [], "attention": []}

    def step(record=False):
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)] if record else None
        if record:
            ev[0].record()
        qp, kp, qs, ks = h3.qk_prep(c.q, c.k, c.rope, c.rope, fp8=c.fp8)
        if record:
            ev[1].record()
        h3.attn_fwd(qp, kp, c.v, c.mode, qs, ks, c.bi, out=out, status_word=status, workspace=ws, logit_bound=c.bound)
        if record:
            ev[2].record()
            events["prep"].append((ev[0], ev[1]))
            events["attention"].append((ev[1], ev[2]))
        return out

    # prep (2) + attention (1) [+ plan | + combine of the split last wave]; V is used where it lies
    launches = 3 + (1 if c.bi is not None else 0) + (1 if split_bytes else 0)
    return step, events, launches


def sample_rows(c, n=40):
    """Global indices of the query rows of THIS rank's shard that the parity check looks at: evenly spread plus the
    shard's edges, the last (partial) tile and the audio / video border when the shard holds them."""
    lo, hi = c.lo, c.lo + c.Ls
    rows = set(torch.linspace(lo, hi - 1, n).long().tolist()) | {lo, hi - 1}
    for r in (c.L - 1, c.L - 104, c.L - 105, c.n_audio - 1, c.n_audio, 127, 128):
        if lo <= r < hi:
            rows.add(r)
    return torch.tensor(sorted(rows), dtype=torch.int64)


def parity_of(c, out_shard, world, dev):
    """Compare sampled rows of this rank's output shard (`out_shard [Ls, H, 128]`, device or pinned host) with the
    fp64 oracle evaluated on the global seeded operands of two heads; the worst rank's figures are returned."""
    import torch.distributed as dist

    from oracle import oracle as O

    rows = sample_rows(c)
    local = rows - c.lo
    hs = c.heads
    got = out_shard[local][:, hs].float().cpu()
    q = c.q[local][:, hs].cpu().double()
    k, v = c.k_host.double(), c.v_host.double()
    if c.cross:
        qn, kn = O.rms_norm(q), O.rms_norm(k)
        csr = None
    else:
        cos, sin = O.rope_table(c.pos.double())
        qn = O.apply_rope(O.rms_norm(q), cos[rows], sin[rows])
        kn = O.apply_rope(O.rms_norm(k), cos, sin)
        csr = None if c.bi_host is None else (c.bi_host.row_ptr.numpy(), c.bi_host.col_idx.numpy())
    if csr is None:
        ref = O.attention(qn, kn, v, chunk=64)
    else:  # the masked oracle looks the tile row up by the global row index
        full_q = torch.zeros(c.L, len(hs), 128, dtype=torch.float64)
        full_q[rows] = qn
        ref = O.attention(full_q, kn, v, csr=csr, q_rows=rows, chunk=64)
    st = O.error_stats(got, ref.float())
    finite = bool(torch.isfinite(got).all())
    mx, mean, rel = BOUNDS["fp8" if c.fp8 else "bf16"]
    ok = finite and st["max_abs"] <= mx and st["mean_abs"] <= mean and st["rel_l2"] <= rel
    t = torch.tensor([st["max_abs"], st["mean_abs"], st["rel_l2"], 0.0 if ok else 1.0], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return {"ok": bool(t[3].item() == 0.0), "max_abs": float(t[0]), "mean_abs": float(t[1]), "rel_l2": float(t[2]),
            "rows": int(rows.numel()) * world, "heads": hs, "bounds": {"max_abs": mx, "mean_abs": mean, "rel_l2": rel},
            "against": "fp64 CPU oracle (RMSNorm + rotation + exact softmax attention%s) on the same global seeded operands; worst rank"
                       % (", unquantised" if c.fp8 else "")}


def copy_floor(hq, hk, hv, ho, dev, barrier, rank_max):
    """What the host link allows: this rank's Q, K, V shards host -> device and an output shard device -> host with
    plain asynchronous copies, every rank copying at once.  Returns (ms with both directions together, H2D GB/s alone,
    D2H GB/s alone), each the slowest rank's."""
    dq, dk, dv, do = (torch.empty_like(t, device=dev) for t in (hq, hk, hv, ho))
    s1, s2 = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

    def run(h2d, d2h):
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        cur = torch.cuda.current_stream(dev)
        a.record(cur)
        s1.wait_stream(cur)
        s2.wait_stream(cur)
        if h2d:
            with torch.cuda.stream(s1):
                for d, h in ((dq, hq), (dk, hk), (dv, hv)):
                    d.copy_(h, non_blocking=True)
        if d2h:
            with torch.cuda.stream(s2):
                ho.copy_(do, non_blocking=True)
        cur.wait_stream(s1)
        cur.wait_stream(s2)
        b.record(cur)
        barrier()
        return rank_max(a.elapsed_time(b))

    run(True, True)
    both = min(run(True, True) for _ in range(3))
    t_in = min(run(True, False) for _ in range(2))
    t_out = min(run(False, True) for _ in range(2))
    nb = hq.numel() * 2
    return both, 3 * nb / (t_in * 1e-3) / 1e9, nb / (t_out * 1e-3) / 1e9


def mean_ms(pairs):
    return sum(a.elapsed_time(b) for a, b in pairs) / max(1, len(pairs))


def roofline_of(c, attn_ms, online_max, world=1):
    """Roofline entry of the attention kernel: `attn_ms` = its launches of one step on one GPU, which computes
    1/world of the step's FLOPs; `achieved` and the fractions are per GPU (fractions of ONE GPU's peak)."""
    burst, sustained, src = measured_peaks()
    achieved = c.flops / world / (attn_ms * 1e-3) / 1e12
    kern = kernel_name(c, online_max, world)
    traffic, traffic_src = None, None
    cap = NCU_TRAFFIC.get(c.mode_name + ("_online" if online_max else ""))
    if cap is not None and cap[0] == kern:  # only a capture of the kernel variant that ran counts
        traffic = cap[1] * (c.L * c.H / world) / cap[2]
        traffic_src = f"{cap[3]} (captured workload scaled by L*H per launch)"
    r = {"bound": "tensor", "kernel": kern, "achieved": achieved, "peak": burst, "unit": "TFLOP/s", "frac": achieved / burst,
         "peak_source": f"bf16 burst, of {src}", "frac_of_sustained": achieved / sustained, "frac_of_spec_2250": achieved / 2250.0,
         "kernel_ms": attn_ms, "traffic": traffic, "traffic_source": traffic_src}
    if world > 1:
        r["whole_job_tflops"] = achieved * world
        r["note"] = "per GPU: kernel_ms = attention launches of one step on one rank (max over ranks), 1/%d of the step's FLOPs" % world
    if c.fp8:
        r["frac_of_fp8_spec_4500"] = achieved / 4500.0
        r["frac_of_blended_3000"] = achieved / 3000.0
    return r


def ulysses_with_projections(c, ua, dev, world, rank, barrier, rank_max, steps=5):
    """N > 1: one attention block's Q/K/V projections (LoRA rank 128, model width H * 128) feeding the sequence-parallel
    attention.  Two forms of the same step: `fused_scatter` - the projection GEMM's epilogue normalises, rotates and
    stores every row straight at its head's owning rank (no separate outbound pass); `separate_scatter` - the same
    GEMMs store locally and the re-layout to the owners is a pass of its own.  Parity: sampled output rows against
    the fp64 oracle on operands projected in fp32 (torch on the GPU, TF32 off) for two heads."""
    import pika_h3_flex_b200 as h3
    from oracle import oracle as O

    H, Ls, L = c.H, c.Ls, c.L
    D, R = H * 128, 128
    g = torch.Generator(device=dev).manual_seed(3001)
    x_full = torch.randn(L, D, device=dev, generator=g).bfloat16()
    ws = [(torch.randn(D, D, device=dev, generator=g) / D ** 0.5).bfloat16() for _ in range(3)]
    las = [(torch.randn(R, D, device=dev, generator=g) / D ** 0.5).bfloat16() for _ in range(3)]
    lbs = [(0.5 * torch.randn(D, R, device=dev, generator=g) / R ** 0.5).bfloat16() for _ in range(3)]
    x = x_full[c.lo : c.lo + Ls].contiguous()
    status = ua.status.tensor(x)

    def proj(i, out_to=None):
        t = torch.nn.functional.linear(x, las[i])  # the thin LoRA product x A^T (torch / cuBLAS)
        return h3.proj_fwd(x, ws[i], None, t, lbs[i], prep=(i < 2), rope=c.rope if i < 2 else None, status_word=status, out_to=out_to)

    def fused():
        return ua.run_scattered(Ls, H, dev, lambda to: proj(0, to), lambda to: proj(1, to), lambda to: proj(2, to), c.bound)

    def separate():
        return ua.run(lambda: proj(0), lambda: proj(1), lambda: proj(2), None, logit_bound=c.bound, prepared=True)

    def time_of(fn):
        for _ in range(3):
            fn()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            out = fn()
        b.record()
        barrier()
        return rank_max(a.elapsed_time(b)) / steps, out

    ms_fused, out = time_of(fused)
    out = out.clone()
    ms_sep, _ = time_of(separate)
    # projections alone (local head-major store), for the split of the step
    def only_proj():
        for i in range(3):
            proj(i)
    ms_proj, _ = time_of(only_proj)
    ua.status.check("ulysses_with_projections")
    # parity: two heads, projections in fp32 on the GPU, the rest by the fp64 oracle
    hs = c.heads
    cols = torch.cat([torch.arange(h * 128, (h + 1) * 128) for h in hs]).to(dev)
    rows = sample_rows(c)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False

    def ref_proj(i, xr):
        y = xr.float() @ ws[i][cols].float().t() + (xr.float() @ las[i].float().t()).bfloat16().float() @ lbs[i][cols].float().t()
        return y.view(-1, len(hs), 128).cpu().double()

    q = ref_proj(0, x_full[rows.to(dev)])
    k, v = ref_proj(1, x_full), ref_proj(2, x_full)
    torch.backends.cuda.matmul.allow_tf32 = prev
    cos, sin = O.rope_table(c.pos.double())
    qn = O.apply_rope(O.rms_norm(q), cos[rows], sin[rows])
    kn = O.apply_rope(O.rms_norm(k), cos, sin)
    ref = O.attention(qn, kn, v.bfloat16().double(), chunk=64)
    st = O.error_stats(out[rows - c.lo][:, hs].float().cpu(), ref.float())
    ok = st["max_abs"] <= 2e-2 and st["mean_abs"] <= 2e-3 and st["rel_l2"] <= 2e-2
    t = torch.tensor([st["max_abs"], st["mean_abs"], st["rel_l2"], 0.0 if ok else 1.0], device=dev, dtype=torch.float64)
    import torch.distributed as dist

    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    flops = 3 * 2.0 * L * D * (D + R) + 3 * 2.0 * L * D * R + c.flops
    return {"workload": "ulysses_with_projections", "ms_per_step": ms_fused, "ms_separate_scatter": ms_sep, "projections_only_ms": ms_proj,
            "value": flops / (ms_fused * 1e-3) / 1e12, "unit": "TFLOP/s (projections + attention, whole job)", "steps": steps,
            "step": "to_q, to_k, to_v (LoRA rank 128; RMSNorm + rotation and the store at the head's owner in the GEMM epilogue), attention, output rows stored at the token's owner",
            "parity": {"ok": bool(t[3].item() == 0.0), "max_abs": float(t[0]), "mean_abs": float(t[1]), "rel_l2": float(t[2]), "rows": int(rows.numel()) * world,
                       "bounds": {"max_abs": 2e-2, "mean_abs": 2e-3, "rel_l2": 2e-2},
                       "against": "fp64 oracle attention on operands projected in fp32 (torch, TF32 off) for two heads; worst rank"}}


def torch_sdpa_comparison(c):
    """What a stock PyTorch build gives for the same attention on this GPU: ``scaled_dot_product_attention`` in bf16 on
    the already prepared operands of the headline workload (torch picks its own library kernel).  A comparison figure
    only: nothing of this library is involved and nothing of it is timed here."""
    import pika_h3_flex_b200 as h3

    qh, kh, _, _ = h3.qk_prep(c.q, c.k, c.rope, c.rope)  # prepared as the attention kernels take them: [L, H, 128] views of head-major memory
    q4, k4 = qh.permute(1, 0, 2)[None], kh.permute(1, 0, 2)[None]  # [1, H, L, 128], contiguous
    v4 = c.v.permute(1, 0, 2).contiguous()[None]
    f = torch.nn.functional.scaled_dot_product_attention
    n = 20  # as many launches as the headline's timed steps, so that the 1 kW power cap weighs on both alike
    for _ in range(3):
        f(q4, k4, v4)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(n):
        o = f(q4, k4, v4)
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / n
    del o, q4, k4, v4, qh, kh
    return {"workload": "cfg1_dense_torch_sdpa", "kernel": "torch.nn.functional.scaled_dot_product_attention (bf16, torch's choice of backend)",
            "kernel_ms": ms, "kernel_tflops": c.flops / (ms * 1e-3) / 1e12, "steps": n,
            "note": "stock PyTorch on the same prepared operands, attention only: a comparison figure, not this library"}


def run_also(name, dev, online_max=False):
    """A short run (3 warm-up + 5 timed steps) of another configuration on this GPU, with its parity verdict."""
    import pika_h3_flex_b200 as h3

    c = make_case(name, 1, 0, dev, online_max)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    step, events, _ = single_gpu_step(c, status)
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(5):
        out = step(record=True)
    b.record()
    torch.cuda.synchronize()
    if h3.read_status(status) != 0:
        return {"workload": name, "error": f"device status 0x{h3.read_status(status):x}"}
    ms = a.elapsed_time(b) / 5
    attn_ms = mean_ms(events["attention"])
    roof = roofline_of(c, attn_ms, online_max)
    par = parity_of(c, out, 1, dev)
    res = {"workload": name + ("_online_max" if online_max else ""), "value": c.flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
           "ms_per_step": ms, "kernel_ms": attn_ms, "kernel": roof["kernel"], "kernel_tflops": roof["achieved"], "frac": roof["frac"],
           "frac_of_spec_2250": roof["frac_of_spec_2250"], "density": c.density, "steps": 5,
           "parity": {k: par[k] for k in ("ok", "max_abs", "mean_abs", "rel_l2", "rows")}}
    if c.fp8:
        res["frac_of_fp8_spec_4500"] = roof["frac_of_fp8_spec_4500"]
        res["frac_of_blended_3000"] = roof["frac_of_blended_3000"]
    return res


def run_ours(args):
    import torch.distributed as dist

    import pika_h3_flex_b200 as h3
    from pika_h3_flex_b200 import _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torchrun (one rank per GPU)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import datetime

        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(minutes=10))
    torch.backends.cuda.matmul.allow_tf32 = False

    name = args.workload
    c = make_case(name, world, rank, dev, args.online_max)
    if c.cross and world > 1:
        raise SystemExit("cross-attention needs no exchange: run it per rank with --gpus 1")
    L, Ls, H = c.L, c.Ls, c.H
    status = h3.StatusWord(dev)
    ua = None
    if world == 1:
        step, events, launches_per_step = single_gpu_step(c, status.tensor())
    else:
        from pika_h3_flex_b200.ulysses import UlyssesAttention

        ua = UlyssesAttention(None, c.mode, c.bi, head_groups=args.head_groups, status=status, transport=args.transport)
        timeline = []

        def step(record=False):
            ua.timeline = timeline if record else None
            return ua(c.q, c.k, c.v, c.rope, logit_bound=c.bound)

        launches_per_step = ua.launches_per_step(Ls, H)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def rank_max(x):
        if world == 1:
            return float(x)
        t = torch.tensor([float(x)], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for _ in range(max(3, args.warmup)):
        step()
    barrier()
    status.check("warm-up")

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    barrier()
    m0 = sampler.mark()
    e_start, e_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e_start.record()
    for _ in range(args.steps):
        out = step(record=True)
    e_stop.record()
    barrier()
    m1 = sampler.mark()
    ms_per_step = rank_max(e_start.elapsed_time(e_stop)) / args.steps
    status.check("timed region")
    # ---- the same steps continued for about two seconds (every rank alike), timed again, with the clock record of
    #      exactly this stretch: nvidia-smi delivers a sample every 200 ms, and the power cap needs a second to bite
    n_sus = 0 if args.lean else max(args.steps, int(2000.0 / max(ms_per_step, 1e-3)) + 1)
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    m2 = sampler.mark()
    s0.record()
    for _ in range(n_sus):
        step()
    s1.record()
    barrier()
    m3 = sampler.mark()
    ms_sustained = rank_max(s0.elapsed_time(s1)) / n_sus if n_sus else None
    clocks = clocks_sus = None
    if rank == 0:
        sampler.stop()
        clocks = sampler.summary(m0, m1)
        clocks_sus = sampler.summary(m2, m3)
        if clocks["samples"] < 3 and n_sus:  # a short timed region holds too few samples: report the record of the whole run
            clocks = sampler.summary(m0, m3)
            clocks["note"] = f"timed region {ms_per_step * args.steps:.0f} ms: the record also covers the {n_sus} identical steps that followed"
    value = c.flops / (ms_per_step * 1e-3) / 1e12
    status.check("sustained stretch")

    # ---- dominant kernel and the token-local preparation, timed live with CUDA events on the launching stream
    if world == 1:
        attn_ms, prep_ms = mean_ms(events["attention"]), mean_ms(events["prep"])
    else:
        attn_ms = sum(sum(a.elapsed_time(b) for a, b in m["attention"]) for m in timeline) / max(1, len(timeline))
        prep_ms = sum(sum(a.elapsed_time(b) for a, b in m["prep"]) for m in timeline) / max(1, len(timeline))
    attn_ms, prep_ms = rank_max(attn_ms), rank_max(prep_ms)
    roofline = roofline_of(c, attn_ms, args.online_max, world)

    # ---- parity of this run's output (outside the timed region)
    parity = parity_of(c, out if world == 1 else out.contiguous(), world, dev)
    parity["path"] = "device-resident"

    # ---- end to end from host buffers through the public call
    e2e = None
    nbytes = L * H * 128 * 2  # over all ranks
    if c.cross or args.lean:
        e2e = {"value": None, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
               "note": "host-buffer end-to-end is measured on the self-attention workloads" if c.cross else "skipped (--lean)"}
    else:
        try:
            hq, hk, hv = (torch.empty(Ls, H, 128, dtype=torch.bfloat16).pin_memory() for _ in range(3))
            for dst, src_t in ((hq, c.q), (hk, c.k), (hv, c.v)):
                dst.copy_(src_t)
            ho = torch.empty(Ls, H, 128, dtype=torch.bfloat16).pin_memory()
            if world == 1:
                host_attn = h3.HostJointAttention(L, H, c.mode, c.bi, status=status)
                api = "HostJointAttention: H2D, prep+attention and D2H pipelined over head groups %s" % host_attn.groups
            else:
                from pika_h3_flex_b200.host_path import HostUlyssesAttention

                host_attn = HostUlyssesAttention(Ls, H, c.mode, c.bi, status=status, transport=args.transport)
                api = "HostUlyssesAttention: per rank, H2D of its shard, prep, reshard, attention, reshard and D2H pipelined over head-slot groups %s" % host_attn.slot_groups
            barrier()
            n_e2e = max(2, min(args.steps, 5))
            for _ in range(2):
                host_attn(hq, hk, hv, c.rope, ho)
            barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(n_e2e):
                host_attn(hq, hk, hv, c.rope, ho)
            b.record()
            barrier()
            e2e_ms = rank_max(a.elapsed_time(b)) / n_e2e
            status.check("host-buffer path")
            e2e = {"value": c.flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": 3 * nbytes,
                   "d2h_bytes_per_step": nbytes, "ms_per_step": e2e_ms, "steps": n_e2e, "api": api}
            pe = parity_of(c, ho, world, dev)
            e2e["parity"] = {k: pe[k] for k in ("ok", "max_abs", "mean_abs", "rel_l2", "rows")}
            floor_ms, h2d_gbs, d2h_gbs = copy_floor(hq, hk, hv, ho, dev, barrier, rank_max)
            e2e["copy_floor_ms"] = floor_ms
            e2e["copy_floor"] = ("plain asynchronous copies of the same shards, both directions at once, every rank at once (slowest rank); "
                                 "per rank H2D alone %.1f GB/s, D2H alone %.1f GB/s" % (h2d_gbs, d2h_gbs))
            e2e["ms_over_copy_floor"] = e2e_ms / floor_ms
            e2e["bound"] = "copy" if floor_ms >= ms_per_step else "compute"  # which of the two the call cannot beat: the plain copies or the resident step
            if hasattr(host_attn, "bound"):
                e2e["bound_estimated_from_shape"] = host_attn.bound
            stages = getattr(host_attn, "stage_ms", None)
            if stages is not None:
                e2e["stages_ms"] = stages()
            if hasattr(host_attn, "close"):
                host_attn.close()
            del host_attn
        except (RuntimeError, ValueError, TypeError, AttributeError, NotImplementedError) as exc:  # keep the kernel-side line
            e2e = {"value": None, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                   "note": "host-buffer path failed: %r" % (exc,)}
            parity["ok"] = False
            parity["note"] = "host-buffer path failed"
    if e2e is not None and e2e.get("parity") is not None:
        parity["ok"] = parity["ok"] and e2e["parity"]["ok"]

    also = None
    if world == 1 and name == "cfg1_dense" and not args.no_also and not args.online_max:
        also = []
        for other in ALSO:
            try:
                also.append(run_also(other, dev))
            except (RuntimeError, ValueError) as exc:
                also.append({"workload": other, "error": repr(exc)})
            torch.cuda.empty_cache()
        try:
            also.append(run_also("cfg1_dense", dev, online_max=True))
        except (RuntimeError, ValueError) as exc:
            also.append({"workload": "cfg1_dense_online_max", "error": repr(exc)})
        try:
            also.append(torch_sdpa_comparison(c))
        except (RuntimeError, ValueError, TypeError) as exc:
            also.append({"workload": "cfg1_dense_torch_sdpa", "error": repr(exc)})
        torch.cuda.empty_cache()

    if world > 1 and not args.no_also and name == "cfg1_dense" and ua.transport == "peer":
        try:
            also = [ulysses_with_projections(c, ua, dev, world, rank, barrier, rank_max)]
        except (RuntimeError, ValueError) as exc:
            also = [{"workload": "ulysses_with_projections", "error": repr(exc)}]
    if world > 1:
        dist.barrier()
    if rank == 0:
        cpu_baseline = None
        if not args.no_cpu_baseline:
            tf, cores, sample, _ = cpu_oracle_sample(name, args.cpu_seconds)
            cpu_baseline = {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample}
        sm = clocks_sus["sm_mhz"] if clocks_sus else None
        line = {
            "metric": "attention_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16" if not c.fp8 else "e4m3(QK)+bf16(PV)", "data": "synthetic",
            "config": {"workload": name, "L": L, "Lk": c.Lk, "H": H, "d": 128, "mode": c.mode_name, "density": c.density,
                       "flops_per_step": c.flops, "step": "qk_prep(RMSNorm+RoPE) + attention forward",
                       "softmax_reference": "running row maximum" if c.bound == 0.0 else "fixed logit bound %.2f from QK-RMSNorm" % c.bound,
                       "parallelism": "single GPU" if world == 1 else f"ulysses{world} (seq<->head reshard, transport: {ua.transport}"
                                      + (f"; peer memory unavailable: {ua.peer_unavailable}" if ua.peer_unavailable else "") + ")",
                       "l2": "inputs (Q,K,V = %.0f MB per rank) exceed the 126 MB L2; no flush" % (3 * Ls * H * 256 / 1e6)},
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e, "clocks": clocks, "parity": parity,
            "ms_per_step_sustained": ms_sustained, "sustained_steps": n_sus, "clocks_sustained": clocks_sus,
            "ms_x_mhz": None if not (sm and ms_sustained) else ms_sustained * sm,
            "prep_ms": prep_ms, "exchange_ms_exposed": None if world == 1 else ms_per_step - prep_ms - attn_ms,
            "gpu_launches": launches_per_step * args.steps,
            "attn_ms_per_dit_step_per_layer": ms_per_step,
        }
        if also is not None:
            line["also"] = also
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        if ua is not None:
            ua.close()
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
    from pika_h3_flex_b200.layout import position_grid

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
        pos = position_grid((31, 30, 52), 1024)
    else:
        frames = (L - 1024) // 64
        pos = position_grid((frames, 8, 8), L - frames * 64)
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
    sampler.stop()
    clocks = sampler.summary()
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
    # the same step with the LoRA update folded into a bf16 copy of each weight (the processor's merge_lora option):
    # one launch per projection, no thin product in front, no extra columns of the contraction
    merged = [torch.addmm(ws[i].float(), lbs[i].float(), las[i].float()).to(torch.bfloat16).contiguous() for i in range(3)]

    def merged_step():
        for i in range(3):
            h3.proj_fwd(x, merged[i], None, None, None, prep=(i < 2), rope=rope if i < 2 else None, status_word=status)
    for _ in range(3):
        merged_step()
    m0, m1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    m0.record()
    for _ in range(5):
        merged_step()
    m1.record()
    torch.cuda.synchronize()
    del merged
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
        "torch_same_step_ms": t0.elapsed_time(t1) / 5, "merged_lora_step_ms": m0.elapsed_time(m1) / 5, "cpu_baseline": None, "e2e": None,
        "clocks": clocks, "gpu_launches": 3 * args.steps,
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
    sampler.stop()
    clocks = sampler.summary()
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
    ap.add_argument("--no-also", action="store_true", help="N = 1: skip the short runs of the other configurations")
    ap.add_argument("--lean", action="store_true", help="for profiler captures: warm-up and timed steps only (no sustained stretch, host-buffer leg, "
                    "CPU baseline or other configurations)")
    ap.add_argument("--head-groups", type=int, default=2, help="N > 1: head groups the reshard is pipelined over (1 = no overlap)")
    ap.add_argument("--transport", choices=["auto", "peer", "nccl"], default="auto",
                    help="N > 1: how operands are resharded: direct stores into the owning rank's memory (peer) or NCCL all-to-all")
    ap.add_argument("--online-max", action="store_true", help="use the running-maximum kernel instead of the fixed logit bound")
    args = ap.parse_args()
    if args.lean:
        args.no_also = args.no_cpu_baseline = True
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
