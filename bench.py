#!/usr/bin/env python
"""Benchmark of the FP8 training hot path (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload ("fp8_linear_fwd_bwd_ffn"): one FP8 block-scaled Linear at DeepSeek-V3 FFN
width, forward + backward: x [16384, 7168] bf16 ~ N(0, 1), master weight
[18432, 7168] fp32 ~ N(0, 0.02), dy [16384, 18432] bf16 ~ N(0, 1).  A step is
FP8MatmulFunction forward + backward: quantise x (1x128) and W (128x128), forward GEMM,
quantise dy (1x128, and along tokens for the weight gradient), re-quantise x in blocks,
dgrad and wgrad GEMMs: 3 x 2*M*N*K = 12.99 TFLOP.  The dense path does not shard
("replicas only"): with N GPUs every rank runs its own replica and the value is the
aggregate (weak scaling).  Data is synthetic, seeded, and larger than L2.
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

M, K, N = 16384, 7168, 18432
FLOP_PER_STEP = 3 * 2.0 * M * N * K
WORKLOAD = "fp8_linear_fwd_bwd_ffn M=16384 K=7168 N=18432"
# DRAM bytes per GEMM launch: reduced-case ncu capture (8192 x 9216 x 7168: forward 363 MB, dgrad 389 MB, wgrad 600 MB
# read + written, for 276 / 259 / 398 MB of operands, scales and output) scaled to the full launch by the algorithmic
# bytes (854 / 669 / 947 MB), averaged over the three
GEMM_TRAFFIC_BYTES = (363.0e6 * 854 / 276 + 389.0e6 * 669 / 259 + 600.5e6 * 947 / 398) / 3


def bench_config(world: int) -> dict:
    """The ``config`` object of the JSON line: identical in both arms."""
    return {"workload": WORKLOAD, "parallelism": f"replicas x{world}" if world > 1 else "single GPU",
            "l2": f"inputs larger than L2 (x {M * K * 2 >> 20} MiB, W {N * K * 4 >> 20} MiB, dy {M * N * 2 >> 20} MiB)"}


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return json.load(f), "measured"
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


def measure_fp8_peak(dev, sustained=True):
    """Dense FP8 peak of this GPU as the library GEMM delivers it: e4m3 x e4m3 -> bf16, 8192^3, per-tensor scales,
    through ``torch._scaled_mm`` (cuBLASLt).  Best of 10 single launches after a pause (burst: the figure for a kernel
    timed alone) and back to back for about two seconds (sustained: the figure for a kernel inside a long step, where
    the part sits at its power cap).  None when the call is not available."""
    n = 8192
    try:
        g = torch.Generator(device=dev).manual_seed(7)
        a = torch.randn(n, n, generator=g, device=dev).to(torch.float8_e4m3fn)
        b = torch.randn(n, n, generator=g, device=dev).to(torch.float8_e4m3fn).t()          # column-major operand
        one = torch.ones((), device=dev)

        def f():
            return torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)

        for _ in range(3):
            f()
        torch.cuda.synchronize()
    except Exception as exc:                                    # noqa: BLE001
        return {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}
    flop = 2.0 * n ** 3
    time.sleep(1.0)
    best = float("inf")
    for _ in range(10):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        f()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    if not sustained:
        return {"fp8_tflops": flop / (best * 1e-3) / 1e12, "how": f"torch._scaled_mm e4m3 {n}^3 -> bf16, per-tensor scales: best of 10 launches"}
    reps = max(50, int(2000.0 / best))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        f()
    e1.record()
    torch.cuda.synchronize()
    sustained_ms = e0.elapsed_time(e1) / reps
    return {"fp8_tflops": flop / (best * 1e-3) / 1e12, "fp8_tflops_sustained": flop / (sustained_ms * 1e-3) / 1e12,
            "how": f"torch._scaled_mm e4m3 {n}^3 -> bf16, per-tensor scales: best of 10 launches; {reps} launches back to back"}


def load_reference_kernels():
    """The unmodified reference module (its Triton kernels) from the staged copy beside the repository, or
    (None, reason).  Used only to time the kernels this library replaces, next to it, on the same GPU."""
    path = os.path.join(ROOT, "baseline", "_ref", "src", "kernels.py")
    if not os.path.isfile(path):
        return None, "reference not staged (baseline/stage_reference.py)"
    try:
        import importlib.util
        import triton  # noqa: F401
        spec = importlib.util.spec_from_file_location("ref_kernels", path)
        mod = importlib.util.module_from_spec(spec)
        sys.modules["ref_kernels"] = mod
        spec.loader.exec_module(mod)
        return mod, None
    except Exception as exc:                                    # noqa: BLE001
        return None, f"{type(exc).__name__}: {exc}"[:200]


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.lines = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "20"], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def mark_begin(self):
        self.t_begin = time.time()

    def mark_end(self):
        self.t_end = time.time()

    def stop(self):
        """Median SM clock and the throttle reasons seen between mark_begin() and mark_end()."""
        import datetime
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, reasons, power, mask = [], None, set(), [], 0
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        # bits of clocks_event_reasons.active (NVML): what the part itself names as the reason for its clock
        bits = {0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x10: "sync_boost",
                0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown"}
        for ln in self.lines:
            p = [t.strip() for t in ln.split(",")]
            if len(p) < 9:
                continue
            try:
                ts = datetime.datetime.strptime(p[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                if not (self.t_begin - 0.005 <= ts <= self.t_end + 0.005):
                    continue
                sm.append(float(p[1]))
                smax = float(p[2])
            except ValueError:
                continue
            try:
                power.append(float(p[3]))
                mask |= int(p[4], 16)
            except ValueError:
                pass
            for name, val in zip(names, p[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        for bit, name in bits.items():
            if mask & bit:
                reasons.add(name)
        sm.sort()
        power.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": smax, "reasons": sorted(reasons),
                "samples": len(sm), "power_w": power[len(power) // 2] if power else None,
                "active_mask": hex(mask)}


def make_inputs(seed: int, pinned: bool):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g, dtype=torch.float32).to(torch.bfloat16)
    w = torch.randn(N, K, generator=g, dtype=torch.float32) * 0.02
    dy = torch.randn(M, N, generator=g, dtype=torch.float32).to(torch.bfloat16)
    if pinned:
        x, dy = x.pin_memory(), dy.pin_memory()
    return x, w, dy


# ---------------------------------------------------------------------------------------
# CPU arm: the reference's own CPU formulation of the path (its torch branches,
# src/kernels.py:753-756, 775-778, 789-792, restated in oracle/ because the reference's
# wrappers assert CUDA), on the host cores, on a bounded sample of the workload.
# ---------------------------------------------------------------------------------------
def cpu_step(sample_rows: int, w: torch.Tensor, x: torch.Tensor, dy: torch.Tensor):
    """One step of the reference's CPU formulation on ``sample_rows`` token rows.  Returns (seconds spent on the
    weight, which a full step pays once; seconds spent on the sampled rows, which grow with the row count)."""
    from oracle import fp8_oracle as O
    xs, dys = x[:sample_rows], dy[:sample_rows]
    t0 = time.perf_counter()
    w_q, w_s = O.quantize_blockwise(w, 128, 128)
    w_deq = O.dequantize_block(w_q, w_s, out_dtype=torch.float32)
    t1 = time.perf_counter()
    x_q, x_s = O.quantize_rowwise(xs, 128, False)
    x_deq = O.dequantize_rowwise(x_q, x_s)
    out = x_deq @ w_deq.t()                                       # forward  (:754-756)
    g_q, g_s = O.quantize_rowwise(dys, 128, False)
    g_deq = O.dequantize_rowwise(g_q, g_s)
    grad_x = g_deq @ w_deq                                        # dgrad    (:776-778)
    grad_w = g_deq.t() @ x_deq                                    # wgrad    (:790-792)
    t2 = time.perf_counter()
    assert torch.isfinite(out[0, 0] + grad_x[0, 0] + grad_w[0, 0])
    return t1 - t0, t2 - t1


def run_cpu_baseline(sample_rows: int, repeats: int, warmup: int = 0):
    """The oracle port timed on all host threads.  A sample of the token rows is run; the time of a full step is
    the weight's part (paid once per step) plus the rows' part scaled to all rows (it is linear in them)."""
    torch.set_num_threads(os.cpu_count() or 1)
    g = torch.Generator().manual_seed(1002)
    x = torch.randn(sample_rows, K, generator=g).to(torch.bfloat16)
    w = torch.randn(N, K, generator=g) * 0.02
    dy = torch.randn(sample_rows, N, generator=g).to(torch.bfloat16)
    for _ in range(warmup):
        cpu_step(sample_rows, w, x, dy)
    parts = [cpu_step(sample_rows, w, x, dy) for _ in range(repeats)]
    t_w = sum(p[0] for p in parts) / len(parts)
    t_rows = sum(p[1] for p in parts) / len(parts)
    step_s = t_w + t_rows * (M / sample_rows)
    return {"value": FLOP_PER_STEP / step_s / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{sample_rows} of {M} token rows, full K={K} N={N}, forward+dgrad+wgrad incl. quantisation, "
                      f"{len(parts)} run(s): weight quantise+dequantise {t_w:.2f} s (once per step), sampled rows "
                      f"{t_rows:.2f} s; full step extrapolated to {step_s:.1f} s"}, step_s


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rows = 256
    base, sec = run_cpu_baseline(rows, repeats=max(1, args.steps), warmup=min(args.warmup, 1))
    line = {
        "impl": "reference", "metric": "fp8_linear_fwd_bwd_tflops", "value": base["value"], "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "ms_per_step_extrapolated": True,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": bench_config(args.gpus),
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


# ---------------------------------------------------------------------------------------
# per-kernel figures: every kernel of the step alone, plus the other benchmark configurations
# ---------------------------------------------------------------------------------------
def _time_kernel(fn, iters=10, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def bench_kernels(Kmod, dev, x, w, dy, peaks, fp8_peak_burst=None):
    """Each kernel of the step on the FFN shapes (inputs larger than L2, so every launch streams from HBM),
    against the roof that bounds it: measured copy bandwidth for the quantisers, 2 x measured bf16 burst for
    the GEMMs (kernels timed alone).  Then the GEMM shapes of the other configurations (single Linear
    4096x512 -> 2048; MLA projections at 16384 tokens)."""
    hbm = float(peaks["hbm_gbs"])
    fp8_peak = fp8_peak_burst if fp8_peak_burst else 2.0 * float(peaks["bf16_tflops"])
    out = []

    def quant_line(name, fn, nbytes):
        ms = _time_kernel(fn)
        gbs = nbytes / (ms * 1e-3) / 1e9
        out.append({"kernel": name, "ms": ms, "bound": "hbm", "achieved": gbs, "peak": hbm, "unit": "GB/s", "frac": gbs / hbm})

    def gemm_line(name, fn, flop, nbytes=None):
        """``nbytes``: algorithmic HBM bytes (e4m3 operands + scales + output), so that shapes near the ridge show
        both bounds."""
        ms = _time_kernel(fn)
        tf = flop / (ms * 1e-3) / 1e12
        line = {"kernel": name, "ms": ms, "bound": "tensor", "achieved": tf, "peak": fp8_peak, "unit": "TFLOP/s",
                "frac": tf / fp8_peak, "frac_of_nominal_4500": tf / 4500.0}
        if nbytes is not None:
            gbs = nbytes / (ms * 1e-3) / 1e9
            line.update({"hbm_achieved_gbs": gbs, "hbm_frac": gbs / hbm, "flop_per_byte": flop / nbytes})
        out.append(line)

    xd, wd = x.detach(), w.detach()
    nkb, nnb = (K + 127) // 128, (N + 127) // 128
    quant_line("quant_row_vec x[16384,7168] bf16", lambda: Kmod.quantize_fp8_rowwise(xd), M * K * 3 + 4 * M * nkb)
    quant_line("quant_row + block re-quantisation x[16384,7168] bf16, one pass (forward of a trained Linear)",
               lambda: Kmod.quantize_fp8_rowwise_with_block(xd), M * K * 4 + 4 * M * nkb + 4 * (M // 128) * nkb)
    quant_line("quant_row_vec dy[16384,18432] bf16", lambda: Kmod.quantize_fp8_rowwise(dy), M * N * 3 + 4 * M * nnb)
    quant_line("quant_row_transposed dy^T (tiles along tokens)", lambda: Kmod.quantize_fp8_rowwise(dy.t()),
               M * N * 3 + 4 * N * (M // 128))
    quant_line("quant_row_dual dy (tiles along features + tiles along tokens, one pass)",
               lambda: Kmod.quantize_fp8_rowwise_dual(dy), M * N * 4 + 4 * (M * nnb + N * (M // 128)))
    quant_line("quant_block_vec W[18432,7168] fp32", lambda: Kmod.quantize_fp8_blockwise(wd), N * K * 5 + 4 * nnb * nkb)
    xq, xs = Kmod.quantize_fp8_rowwise(xd)
    quant_line("requant_row_to_block x e4m3", lambda: Kmod.requantize_rowwise_to_blockwise(xq, xs),
               M * K * 2 + 4 * M * nkb + 4 * (M // 128) * nkb)
    wq, ws = Kmod.quantize_fp8_blockwise(wd)
    dq, ds = Kmod.quantize_fp8_rowwise(dy)
    dtq, dts = Kmod.quantize_fp8_rowwise(dy.t())
    xbq, xbs = Kmod.requantize_rowwise_to_blockwise(xq, xs)
    flop = 2.0 * M * N * K
    gemm_line("gemm forward  16384x18432x7168 (B K-major, two-SM)", lambda: Kmod.fp8_matmul_dsv3(xq, wq.t(), xs, ws.t()), flop,
              M * K + N * K + 4 * (M * nkb + nnb * nkb) + 2 * M * N)
    wq_t = Kmod.transpose_fp8(wq)
    _, _, xbq_t, _ = Kmod.quantize_fp8_rowwise_with_block(xd, transpose_block=True)
    gemm_line("gemm dgrad    16384x7168x18432 (W^T copy, B K-major, two-SM)", lambda: Kmod.fp8_matmul_dsv3(dq, wq_t.t(), ds, ws), flop)
    gemm_line("gemm wgrad    18432x7168x16384 (x block copy transposed, B K-major, two-SM, fp32 out)",
              lambda: Kmod.fp8_matmul_dsv3(dtq, xbq_t.t(), dts, xbs, out_dtype=torch.float32), flop)
    gemm_line("gemm dgrad    16384x7168x18432 (B MN-major, one-SM)", lambda: Kmod.fp8_matmul_dsv3(dq, wq, ds, ws), flop)
    gemm_line("gemm wgrad    18432x7168x16384 (B MN-major, one-SM)", lambda: Kmod.fp8_matmul_dsv3(dtq, xbq, dts, xbs), flop)
    quant_line("quant_block_vec W[18432,7168] fp32 + transposed copy, one pass", lambda: Kmod.quantize_fp8_blockwise_t(wd),
               N * K * 6 + 4 * nnb * nkb)
    quant_line("quant_row + transposed block re-quantisation x[16384,7168] bf16, one pass",
               lambda: Kmod.quantize_fp8_rowwise_with_block(xd, transpose_block=True), M * K * 4 + 4 * M * nkb + 4 * (M // 128) * nkb)
    quant_line("transpose_fp8 W e4m3 [18432,7168]", lambda: Kmod.transpose_fp8(wq), 2 * N * K)
    del wq_t, xbq_t
    # the reference's own Triton kernels on the same GPU and the same operands: the kernels this library replaces
    ref, why = load_reference_kernels()
    if ref is None:
        out.append({"kernel": "reference Triton kernels", "unavailable": why})
    else:
        def versus(name, ours_fn, ref_fn, iters_ref=3, **extra):
            ours_ms = _time_kernel(ours_fn)
            ref_ms = _time_kernel(ref_fn, iters=iters_ref, warm=2)
            out.append(dict({"kernel": name, "ms": ours_ms, "reference_triton_ms": ref_ms,
                             "speedup_vs_reference_triton": ref_ms / ours_ms}, **extra))

        g1 = torch.Generator(device=dev).manual_seed(1001)
        x1 = torch.randn(4096, 512, generator=g1, device=dev).to(torch.bfloat16)
        w1 = (torch.randn(2048, 512, generator=g1, device=dev) * 0.02).to(torch.bfloat16)
        x1q, x1s = Kmod.quantize_fp8_rowwise(x1)
        w1q, w1s = Kmod.quantize_fp8_blockwise(w1)
        w1q_t, w1s_t = w1q.t().contiguous(), w1s.t().contiguous()            # what the reference's forward feeds its GEMM
        versus("fp8_matmul_dsv3 config 1 (4096x2048x512) vs reference fp8_gemm_kernel",
               lambda: Kmod.fp8_matmul_dsv3(x1q, w1q.t(), x1s, w1s.t()),
               lambda: ref.fp8_matmul_dsv3(x1q, w1q_t, x1s, w1s_t), iters_ref=10)
        wq_t_ref, ws_t_ref = wq.t().contiguous(), ws.t().contiguous()
        versus("fp8_matmul_dsv3 FFN forward (16384x18432x7168) vs reference fp8_gemm_kernel",
               lambda: Kmod.fp8_matmul_dsv3(xq, wq.t(), xs, ws.t()),
               lambda: ref.fp8_matmul_dsv3(xq, wq_t_ref, xs, ws_t_ref))
        out[-1]["tflops"] = flop / (out[-1]["ms"] * 1e-3) / 1e12
        out[-1]["reference_triton_tflops"] = flop / (out[-1]["reference_triton_ms"] * 1e-3) / 1e12
        del wq_t_ref, ws_t_ref
        versus("quantize_fp8_rowwise x[16384,7168] bf16 vs reference quantize_fp8_rowwise_kernel",
               lambda: Kmod.quantize_fp8_rowwise(xd), lambda: ref.quantize_fp8_rowwise(xd), iters_ref=10)
        versus("quantize_fp8_blockwise W[18432,7168] fp32 vs reference quantize_fp8_blockwise_kernel",
               lambda: Kmod.quantize_fp8_blockwise(wd), lambda: ref.quantize_fp8_blockwise(wd), iters_ref=10)
        # one 8-way expert-parallel rank's share of the MoE configuration: 32 experts x 1024 rows, 7168 -> 4096
        Eg, rows_e = 32, 1024
        xg_ = torch.randn(Eg * rows_e, MOE["d"], generator=g1, device=dev).to(torch.bfloat16)
        wg_ = (torch.randn(Eg, 2 * MOE["I"], MOE["d"], generator=g1, device=dev) * 0.02).to(torch.bfloat16)
        st_ = torch.arange(Eg, device=dev, dtype=torch.int64) * rows_e
        en_ = st_ + rows_e
        gflop = 2.0 * Eg * rows_e * MOE["d"] * 2 * MOE["I"]
        prec = Kmod.set_moe_grouped_precision("fp8") if hasattr(Kmod, "set_moe_grouped_precision") else None
        versus("moe_grouped_gemm 32 experts x 1024 rows, 7168->4096, bf16 in (e4m3 path, incl. quantising tokens + weights) "
               "vs reference grouped_gemm_kernel", lambda: Kmod.moe_grouped_gemm(xg_, wg_, st_, en_, rows_e),
               lambda: ref.moe_grouped_gemm(xg_, wg_, st_, en_, rows_e))
        if prec is not None:
            Kmod.set_moe_grouped_precision(prec)
        out[-1]["tflops"] = gflop / (out[-1]["ms"] * 1e-3) / 1e12
        out[-1]["reference_triton_tflops"] = gflop / (out[-1]["reference_triton_ms"] * 1e-3) / 1e12
        xgq, xgs = Kmod.quantize_fp8_rowwise(xg_)
        wgq, wgs = Kmod.quantize_expert_weights(wg_)
        versus("fp8_grouped_gemm (operands quantised beforehand, weights cached), same shape vs reference grouped_gemm_kernel",
               lambda: Kmod.fp8_grouped_gemm(xgq, xgs, wgq, wgs, st_, en_, out_dtype=torch.bfloat16),
               lambda: ref.moe_grouped_gemm(xg_, wg_, st_, en_, rows_e))
        out[-1]["tflops"] = gflop / (out[-1]["ms"] * 1e-3) / 1e12
        del xgq, xgs, wgq, wgs, x1, w1
        # forward + backward of that up-projection through the differentiable drop-in (the reference's has no backward):
        # token quantiser, grouped GEMM; output-gradient quantiser, grouped dgrad, weight gradients of all experts
        xg_t = xg_.clone().requires_grad_(True)
        wg_t = wg_.float().requires_grad_(True)
        go_ = torch.randn(Eg * rows_e, 2 * MOE["I"], generator=g1, device=dev).to(torch.bfloat16)

        def fwd_bwd():
            xg_t.grad = None
            wg_t.grad = None
            Kmod.moe_grouped_gemm(xg_t, wg_t, st_, en_, dtype=torch.bfloat16).backward(go_)

        ms_fb = _time_kernel(fwd_bwd, iters=5, warm=2)
        out.append({"kernel": "moe_grouped_gemm forward + backward, 32 experts x 1024 rows, 7168->4096 (e4m3; fp32 master weights, "
                              "cached as e4m3; weight gradients of all experts in one grouped-K GEMM writing 3.8 GB of fp32)", "ms": ms_fb, "bound": "tensor",
                    "achieved": 3 * gflop / (ms_fb * 1e-3) / 1e12, "peak": fp8_peak, "unit": "TFLOP/s",
                    "frac": 3 * gflop / (ms_fb * 1e-3) / 1e12 / fp8_peak})
        # the same with the expert weights (and so their gradients) in bf16: the grouped-K GEMM writes half the bytes
        wg_b = wg_.detach().clone().requires_grad_(True)

        def fwd_bwd_b():
            xg_t.grad = None
            wg_b.grad = None
            Kmod.moe_grouped_gemm(xg_t, wg_b, st_, en_, dtype=torch.bfloat16).backward(go_)

        ms_fb = _time_kernel(fwd_bwd_b, iters=5, warm=2)
        out.append({"kernel": "moe_grouped_gemm forward + backward, same shape, expert weights and their gradients in bf16",
                    "ms": ms_fb, "bound": "tensor", "achieved": 3 * gflop / (ms_fb * 1e-3) / 1e12, "peak": fp8_peak,
                    "unit": "TFLOP/s", "frac": 3 * gflop / (ms_fb * 1e-3) / 1e12 / fp8_peak})
        del xg_, wg_, xg_t, wg_t, wg_b, go_
    del dq, ds, dtq, dts, xbq, xbs, wq, ws
    # other configurations: (tokens, in, out)
    g = torch.Generator(device=dev).manual_seed(1003)
    for name, (m, k, n) in {"config 1 Linear 4096x512->2048": (4096, 512, 2048),
                            "MLA W_dq 7168->1536": (16384, 7168, 1536), "MLA W_dkv 7168->576": (16384, 7168, 576),
                            "MLA W_uq 1536->24576": (16384, 1536, 24576), "MLA W_uk/W_uv 512->16384": (16384, 512, 16384)}.items():
        a = torch.randn(m, k, generator=g, device=dev).to(torch.bfloat16)
        b = (torch.randn(n, k, generator=g, device=dev) * 0.02).to(torch.bfloat16)
        aq, as_ = Kmod.quantize_fp8_rowwise(a)
        bq, bs = Kmod.quantize_fp8_blockwise(b)
        gemm_line(f"gemm {name} ({m} tokens)", lambda: Kmod.fp8_matmul_dsv3(aq, bq.t(), as_, bs.t()), 2.0 * m * n * k,
                  m * k + n * k + 4 * (m * ((k + 127) // 128) + ((n + 127) // 128) * ((k + 127) // 128)) + 2 * m * n)
    del a, b, aq, as_, bq, bs
    # MoE plumbing at the C4 sizes (32768 tokens, top-8, d = 7168, I = 2048): HBM-bound passes
    T, E, k8, d, I = MOE["tokens"], MOE["E"], MOE["top_k"], MOE["d"], MOE["I"]
    logits = torch.randn(T, E, generator=g, device=dev)
    bias = torch.randn(E, generator=g, device=dev)
    quant_line("moe_route 32768 tokens x 256 experts, top-8 (3 launches)", lambda: Kmod.moe_route(logits, bias, k8),
               T * E * 4 + T * k8 * (4 + 4 + 8 + 4 + 8 + 8 + 4))
    r = Kmod.moe_route(logits, bias, k8)
    tq, ts = Kmod.quantize_fp8_rowwise(torch.randn(T, d, generator=g, device=dev).to(torch.bfloat16))
    quant_line("gather_rows e4m3 [262144,7168] + scales", lambda: Kmod.gather_quantized_rows(tq, ts, r["token_indices"]),
               T * k8 * (d + 4 * (d // 128)) * 2)
    del tq, ts
    h12 = torch.randn(T * k8 // 2, 2 * I, generator=g, device=dev).to(torch.bfloat16)
    quant_line("swiglu_quant_row h12[131072,4096] bf16", lambda: Kmod.swiglu_quantize_rowwise(h12),
               (T * k8 // 2) * (2 * I * 2 + I + 4 * (I // 128)))
    del h12
    rows = torch.randn(T * k8, d, generator=g, device=dev).to(torch.bfloat16)
    shared = torch.randn(T, d, generator=g, device=dev).to(torch.bfloat16)
    quant_line("moe_combine + shared [262144,7168] bf16 -> [32768,7168] fp32",
               lambda: Kmod.moe_combine(rows, r["pair_pos"], r["pair_gate"], shared), T * k8 * d * 2 + T * d * (2 + 4))
    del rows, shared, logits
    # sparse attention at the model's sizes (PoPE: 192-wide queries/keys, 64-wide values, 128 selected keys); the bound
    # is the L2 -> SM gather traffic, reported as such (no measured peak for it)
    Bs, Hs, Ls, Ks, Dq, Dvv = 32, 8, 1024, 128, 192, 64
    qa = torch.randn(Bs, Hs, Ls, Dq, generator=g, device=dev).to(torch.bfloat16).requires_grad_(True)
    ka = torch.randn(Bs, Hs, Ls, Dq, generator=g, device=dev).to(torch.bfloat16).requires_grad_(True)
    va = torch.randn(Bs, Hs, Ls, Dvv, generator=g, device=dev).to(torch.bfloat16).requires_grad_(True)
    pos = torch.arange(Ls, device=dev).view(1, Ls, 1)
    idx = (torch.rand(Bs, Ls, Ks, generator=g, device=dev) * (pos + 1)).long().clamp(max=Ls - 1)
    go = torch.randn(Bs, Hs, Ls, Dvv, generator=g, device=dev).to(torch.bfloat16)
    gathered = Bs * Hs * Ls * Ks * (Dq + Dvv) * 2

    def attn_fwd():
        with torch.no_grad():
            Kmod.sparse_attention(qa, ka, va, idx)

    def attn_fwd_bwd():
        o, _ = Kmod.sparse_attention(qa, ka, va, idx)
        o.backward(go)
        qa.grad = ka.grad = va.grad = None

    for name, fn, nbytes in (("sparse_attention forward B32 H8 L1024 K128 d192/64 bf16", attn_fwd, gathered),
                             ("sparse_attention forward+backward (same)", attn_fwd_bwd, 3 * gathered)):
        ms = _time_kernel(fn)
        out.append({"kernel": name, "ms": ms, "bound": "l2 gather", "achieved": nbytes / (ms * 1e-3) / 1e9, "peak": None,
                    "unit": "GB/s gathered", "frac": None})
    return out


def extras_small(Kmod, dev):
    """The MoE plumbing passes, the grouped weight gradient and sparse attention on a reduced case (8192 tokens,
    top-8, d = 7168; 8 experts x 1024 rows; attention B 8 x H 8 x L 1024 x K 128): inputs larger than L2 but at
    most about a GB each, for profiler captures.
    Runs every kernel three times and prints one line of CUDA-event timings; not a headline number."""
    g = torch.Generator(device=dev).manual_seed(77)
    T, E, k8, d, I = 8192, 256, 8, 7168, 2048
    logits = torch.randn(T, E, generator=g, device=dev)
    bias = torch.randn(E, generator=g, device=dev)
    tok = torch.randn(T, d, generator=g, device=dev).to(torch.bfloat16)
    h12 = torch.randn(T * k8 // 2, 2 * I, generator=g, device=dev).to(torch.bfloat16)
    rows = torch.randn(T * k8, d, generator=g, device=dev).to(torch.bfloat16)
    shared = torch.randn(T, d, generator=g, device=dev).to(torch.bfloat16)
    Bs, Hs, Ls, Ks, Dq, Dvv = 8, 8, 1024, 128, 192, 64
    qa = torch.randn(Bs, Hs, Ls, Dq, generator=g, device=dev).to(torch.bfloat16).requires_grad_(True)
    ka = torch.randn(Bs, Hs, Ls, Dq, generator=g, device=dev).to(torch.bfloat16).requires_grad_(True)
    va = torch.randn(Bs, Hs, Ls, Dvv, generator=g, device=dev).to(torch.bfloat16).requires_grad_(True)
    pos = torch.arange(Ls, device=dev).view(1, Ls, 1)
    idx = (torch.rand(Bs, Ls, Ks, generator=g, device=dev) * (pos + 1)).long().clamp(max=Ls - 1)
    go = torch.randn(Bs, Hs, Ls, Dvv, generator=g, device=dev).to(torch.bfloat16)
    tq, ts = Kmod.quantize_fp8_rowwise(tok)
    r = Kmod.moe_route(logits, bias, k8)

    def attn():
        o, _ = Kmod.sparse_attention(qa, ka, va, idx)
        o.backward(go)
        qa.grad = ka.grad = va.grad = None

    # backward of a grouped expert GEMM: 8 experts x 1024 rows, 7168 -> 4096 (a quarter of one 8-way rank's share)
    Eg, rows_e, d_out = 8, 1024, 4096
    xg = torch.randn(Eg * rows_e, d, generator=g, device=dev).to(torch.bfloat16)
    xgq, xgs = Kmod.quantize_fp8_rowwise(xg)
    gst = torch.arange(Eg, device=dev, dtype=torch.int64) * rows_e
    ggo = torch.randn(Eg * rows_e, d_out, generator=g, device=dev).to(torch.bfloat16)

    passes = {"grouped_wgrad": lambda: Kmod.fp8_grouped_wgrad(ggo, xgq, xgs, gst, gst + rows_e, Eg, d, d_out, torch.float32),
              "moe_route": lambda: Kmod.moe_route(logits, bias, k8),
              "gather_rows": lambda: Kmod.gather_quantized_rows(tq, ts, r["token_indices"]),
              "swiglu_quant": lambda: Kmod.swiglu_quantize_rowwise(h12),
              "moe_combine_add": lambda: Kmod.moe_combine(rows, r["pair_pos"], r["pair_gate"], shared),
              "sparse_attention_fwd_bwd": attn}
    out = {}
    for name, fn in passes.items():
        out[name + "_ms"] = round(_time_kernel(fn, iters=2, warm=1), 4)
    print(json.dumps({"extras_small": out}))


# ---------------------------------------------------------------------------------------
# MoE layer (expert parallel where N > 1): reported beside the dense line
# ---------------------------------------------------------------------------------------
MOE = dict(E=256, d=7168, I=2048, tokens=32768, top_k=8, shared_hidden=2048)


def bench_moe(Kmod, dev, rank, world, steps, warmup, bias_scale, label, chunks=1, exchange="nccl", splits=1, dispatch_sms=0):
    """256 routed experts (SwiGLU 7168 -> 2x2048 -> 7168) + 1 shared expert, 32768 tokens, top-8 with
    sigmoid scores + per-expert bias.  Strong scaling: tokens and experts are both split over the ranks.
    Returns a dict (rank 0) with whole-layer tokens/s, the per-phase times of the most loaded rank, the grouped-GEMM
    rate on the rows that rank really received, the load imbalance, and a parity check of sampled tokens against the
    same arithmetic done on one GPU with every expert's weights."""
    import torch.distributed as dist
    from cinnamon_b200 import moe
    c = MOE
    E_local, T_local = c["E"] // world, c["tokens"] // world
    g = torch.Generator(device=dev).manual_seed(1004)
    router = torch.randn(c["E"], c["d"], generator=g, device=dev) * 0.02
    bias = torch.randn(c["E"], generator=g, device=dev) * bias_scale
    gw = torch.Generator(device=dev).manual_seed(2004 + rank)
    w12 = (torch.randn(E_local, 2 * c["I"], c["d"], generator=gw, device=dev) * 0.02).to(torch.bfloat16)
    w3 = (torch.randn(E_local, c["d"], c["I"], generator=gw, device=dev) * 0.02).to(torch.bfloat16)
    x = torch.randn(T_local, c["d"], generator=gw, device=dev).to(torch.bfloat16)
    gs = torch.Generator(device=dev).manual_seed(3004)
    sw = [torch.randn(c["shared_hidden"], c["d"], generator=gs, device=dev) * 0.02,
          torch.randn(c["shared_hidden"], c["d"], generator=gs, device=dev) * 0.02,
          torch.randn(c["d"], c["shared_hidden"], generator=gs, device=dev) * 0.02]
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    # the layer as a user builds it: router + this rank's routed experts + the shared expert (round_scale on the
    # shared expert's input, as the reference's converted model has it)
    module = moe.ExpertParallelMoE(router, bias, w12, w3, c["top_k"], shared=moe.FP8SwiGLU(*sw, round_scale=True),
                                   n_chunks=chunks, exchange=exchange, max_tokens_per_rank=T_local, up_splits=splits, dispatch_sms=dispatch_sms)
    t1.record()
    torch.cuda.synchronize()
    wq_ms = t0.elapsed_time(t1)
    experts = module.experts
    del w12, w3, sw

    def layer():
        with torch.no_grad():
            return module(x)

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        layer()
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        y = layer()
    e1.record()
    sync()
    ms = torch.tensor([e0.elapsed_time(e1) / steps], device=dev, dtype=torch.float64)

    # ---- phases of one more call (CUDA events on the layer's main stream; outside the timed region)
    module.trace = []
    y = layer()
    sync()
    trace, module.trace = module.trace, None
    phases = [{"phase": name, "ms": round(trace[i - 1][1].elapsed_time(ev), 4)} for i, (name, ev) in enumerate(trace) if i > 0]

    # ---- the grouped GEMMs alone, on the quantised rows this rank really received in that call
    with torch.no_grad():
        logits = moe.router_logits(x, module._router_as(x.dtype))
        r = Kmod.moe_route(logits, bias, c["top_k"])
    if world > 1 and module.exchange in ("p2p", "p2p-fused") and module._peer_buffers is not None and module._peer_buffers.n_experts:
        pb = module._peer_buffers
        rows = int(pb._tables.total_rows)
        rq = pb.q.view(pb.capacity_rows, pb.d)[:rows].view(torch.float8_e4m3fn)
        rs = pb.s.view(pb.capacity_rows, pb.n_scales)[:rows]
        starts, ends = pb._tables.starts.clone(), pb._tables.ends.clone()
    else:
        plan = moe.make_plan(r["counts"]) if world == 1 else None
        xq_, xs_ = Kmod.quantize_fp8_rowwise(x)
        if world == 1:
            rq, rs = Kmod.gather_quantized_rows(xq_, xs_, r["token_indices"])
            starts, ends, rows = plan.starts, plan.ends, int(plan.ends[-1])
        else:                                        # all-to-all path: time the GEMMs on this rank's own pairs of its experts
            lo = rank * E_local
            cnt = r["counts"][lo:lo + E_local]
            ends = cnt.cumsum(0)
            starts = ends - cnt
            first = int(r["counts"][:lo].sum())
            rows = int(ends[-1])
            rq, rs = Kmod.gather_quantized_rows(xq_, xs_, r["token_indices"][first:first + rows])
        del xq_, xs_
    for _ in range(2):
        experts(rq, rs, starts, ends)
    sync()
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    g0.record()
    for _ in range(steps):
        experts(rq, rs, starts, ends)
    g1.record()
    sync()
    my_gms = g0.elapsed_time(g1) / steps
    my_flop = float(rows) * 2.0 * c["d"] * 3 * c["I"]

    # ---- parity: sampled tokens of this rank recomputed on this GPU alone with every expert's quantised weights
    parity = None
    n_s = 256
    with torch.no_grad():
        if world > 1:
            def gathered(t):
                out = torch.empty((world,) + tuple(t.shape), dtype=torch.uint8 if t.dtype == torch.float8_e4m3fn else t.dtype, device=dev)
                dist.all_gather_into_tensor(out, (t.view(torch.uint8) if t.dtype == torch.float8_e4m3fn else t).contiguous())
                out = out.view((world * t.shape[0],) + tuple(t.shape[1:]))
                return out.view(torch.float8_e4m3fn) if t.dtype == torch.float8_e4m3fn else out
            full = moe.FP8Experts.__new__(moe.FP8Experts)
            full.K, full.n_experts, full.d_model, full.hidden = Kmod, c["E"], c["d"], c["I"]
            full.w12_q, full.w12_s = gathered(experts.w12_q), gathered(experts.w12_s)
            full.w3_q, full.w3_s = gathered(experts.w3_q), gathered(experts.w3_s)
        else:
            full = experts
        idx = torch.randperm(T_local, generator=torch.Generator().manual_seed(9 + rank))[:n_s].sort().values.to(dev)
        x_s = x[idx].contiguous()
        r_s = Kmod.moe_route(logits[idx].contiguous(), bias, c["top_k"])
        cnt = r_s["counts"]
        ends_s = cnt.cumsum(0)
        starts_s = ends_s - cnt
        q_s, s_s = Kmod.quantize_fp8_rowwise(x_s)
        gq, gsc = Kmod.gather_quantized_rows(q_s, s_s, r_s["token_indices"])
        rows_out = full(gq, gsc, starts_s, ends_s)
        y_ref = Kmod.moe_combine(rows_out, r_s["pair_pos"], r_s["pair_gate"], module.shared(x_s))
        y_got = y.reshape(T_local, c["d"])[idx]
        err = float((y_got - y_ref).norm() / y_ref.norm())
        bit_equal = bool(torch.equal(y_got, y_ref))
        parity = {"sampled_tokens": n_s, "max_rel_err": err, "bit_equal_to_one_gpu_path": bit_equal}
        assert err < 1e-5, f"expert-parallel layer differs from the one-GPU arithmetic on sampled tokens: rel err {err}"
        del full, rows_out, gq, gsc

    load = torch.tensor([float(rows)], device=dev, dtype=torch.float64)
    total = load.clone()
    info = {"rank": rank, "rows": rows, "phases": phases, "grouped_gemm_ms": my_gms,
            "grouped_gemm_tflops": my_flop / (my_gms * 1e-3) / 1e12 if rows else 0.0, "parity": parity}
    infos = [info]
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        dist.all_reduce(load, op=dist.ReduceOp.MAX)
        dist.all_reduce(total, op=dist.ReduceOp.SUM)
        infos = [None] * world
        dist.all_gather_object(infos, info)
    busiest = max(infos, key=lambda i: i["rows"])
    active = int((r["counts"] > 0).sum())
    module_exchange = module.exchange              # "nccl" if symmetric memory was not available
    del experts, module, rq, rs
    torch.cuda.empty_cache()
    mean_rows = total.item() / world
    return {"workload": f"moe_layer E=256 d=7168 I=2048 tokens=32768 top8 {label}", "tokens_per_s": c["tokens"] / (ms.item() * 1e-3),
            "ms_per_layer": ms.item(), "expert_weight_quant_ms": wq_ms, "max_rank_rows": int(load.item()),
            "mean_rank_rows": mean_rows, "imbalance_bound_mean_over_max": mean_rows / max(1.0, load.item()),
            "most_loaded_rank": {"rank": busiest["rank"], "rows": busiest["rows"], "phases_ms": busiest["phases"],
                                 "grouped_gemm_ms": busiest["grouped_gemm_ms"], "grouped_gemm_tflops": busiest["grouped_gemm_tflops"],
                                 "grouped_gemm_note": "up-projection + SwiGLU/quantise + down-projection alone, on the e4m3 rows "
                                                      "this rank received in the traced call"},
            "parity": {"sampled_tokens_per_rank": n_s, "max_rel_err": max(i["parity"]["max_rel_err"] for i in infos),
                       "bit_equal_to_one_gpu_path": all(i["parity"]["bit_equal_to_one_gpu_path"] for i in infos),
                       "ranks_checked": len(infos)},
            "active_experts_rank0_view": active, "scaling": "strong", "n_gpus": world,
            "token_chunks": chunks if world > 1 else 1, "exchange": module_exchange if world > 1 else "none",
            "expert_ranges": splits if (world > 1 and module_exchange == "p2p-fused") else 1,
            "dispatch_sms": dispatch_sms if (world > 1 and module_exchange == "p2p-fused") else 0}


# ---------------------------------------------------------------------------------------
# End-to-end training step of the reference's model on the drop-in (data parallel where N > 1)
# ---------------------------------------------------------------------------------------
def bench_c5(dev, rank, world, steps=5, warmup=2, batch_size=32, seq_len=1024):
    """The reference's ``Cinnamon`` model (d_model 512, 8 layers, MLA, 16 routed experts top-2 + 1 shared expert,
    MTP depth 1, vocabulary 32000) with ``convert_to_fp8`` applied, on this library's ``kernels`` module: one
    training step = host batch -> device, forward + backward under bf16 autocast (src/train.py:338-376), gradient
    all-reduce (DistributedDataParallel over NCCL, as src/train.py:702), clip, AdamW.  Uniform random token ids,
    ``batch_size`` x ``seq_len`` per GPU; tokens/s is the whole job's.  ``torch.compile`` is off."""
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    from baseline import reference_model as RM
    if not RM.available():
        return {"workload": "config 5 end-to-end training step", "unavailable": "reference not staged (baseline/stage_reference.py)"}
    torch.manual_seed(1005)
    model, cfg, Kmod = RM.build_model(dev)
    n_fp8 = sum(1 for m in model.modules() if isinstance(m, Kmod.FP8Linear))
    model.train()
    net = model
    if world > 1:
        from torch.nn.parallel import DistributedDataParallel as DDP
        net = DDP(model, device_ids=[dev.index], find_unused_parameters=True)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4, weight_decay=0.1)
    g = torch.Generator().manual_seed(1005 + rank)
    host = torch.randint(0, cfg.vocab_size, (batch_size, seq_len + 1), generator=g).pin_memory()

    def step():
        return RM.train_step(net, host.to(dev, non_blocking=True), optimizer=opt)

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        loss = step()
    sync()
    launches0 = Kmod.launch_count
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        loss = step()
    e1.record()
    sync()
    ms = torch.tensor([e0.elapsed_time(e1) / steps], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    out = {"workload": "config 5: reference Cinnamon model + convert_to_fp8 on the drop-in kernels module, "
                       f"{batch_size} x {seq_len} tokens per GPU, forward + backward + AdamW",
           "tokens_per_s": world * batch_size * seq_len / (ms.item() * 1e-3), "ms_per_step": ms.item(), "n_gpus": world,
           "parallelism": f"DistributedDataParallel x{world} (NCCL all-reduce of the gradients)" if world > 1 else "single GPU",
           "scaling": "weak", "fp8_linear_layers": n_fp8, "library_launches_per_step": (Kmod.launch_count - launches0) / steps,
           "loss": float(loss), "torch_compile": False, "device_status": Kmod.device_status()}
    del net, model, opt
    torch.cuda.empty_cache()
    if world == 1:
        # the unmodified reference (its own Triton kernels) on the same GPU and batch, in a process of its own
        try:
            p = subprocess.run([sys.executable, os.path.join(ROOT, "baseline", "reference_model.py"), "--own-kernels", "--steps", "3",
                                "--batch", str(batch_size), "--seq", str(seq_len)], capture_output=True, text=True, timeout=900)
            lines = [ln for ln in p.stdout.splitlines() if ln.startswith("RESULT ")]
            if p.returncode == 0 and lines:
                ref = json.loads(lines[-1][len("RESULT "):])
                out["reference_triton"] = ref
                out["speedup_vs_reference_triton"] = ref["ms_per_step"] / out["ms_per_step"]
            else:
                out["reference_triton"] = {"unavailable": (p.stderr.strip().splitlines() or ["no output"])[-1][:300]}
        except Exception as exc:                                # noqa: BLE001
            out["reference_triton"] = {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}
    return out


def run_e2e(Kmod, dev, args, world, x_h, dy_h, w, barrier):
    """The step measured end to end: inputs start in pinned host memory, results end there, every step.
    Returns (ms per step, bytes host->device per step, bytes device->host per step)."""
    import torch.distributed as dist
    out_h = torch.empty(M, N, dtype=torch.bfloat16).pin_memory()
    gx_h = torch.empty(M, K, dtype=torch.bfloat16).pin_memory()
    gw_h = torch.empty(N, K, dtype=torch.float32).pin_memory()

    # Three streams, two sets of device buffers: while step i computes, step i+1's inputs come in over PCIe and
    # step i-1's results go out.  Every step still copies all of its inputs in and all of its results out.
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    s_cmp = torch.cuda.current_stream(dev)
    xd = [torch.empty(M, K, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    dyd = [torch.empty(M, N, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_free = [torch.cuda.Event() for _ in range(2)]
    ev_out = torch.cuda.Event()
    for e in ev_free:
        e.record(s_cmp)
    ev_out.record(s_out)

    def e2e_step(i):
        b = i & 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_free[b])                      # the step that last used these buffers has consumed them
            xd[b].copy_(x_h, non_blocking=True)
            dyd[b].copy_(dy_h, non_blocking=True)
            ev_in[b].record(s_in)
        s_cmp.wait_event(ev_in[b])
        xin = xd[b].detach().requires_grad_(True)
        w.grad = None
        out = Kmod.FP8MatmulFunction.apply(xin, w, False)
        out.backward(dyd[b])
        ev_free[b].record(s_cmp)
        done = torch.cuda.Event()
        done.record(s_cmp)
        results = (out.detach(), xin.grad, w.grad)
        with torch.cuda.stream(s_out):
            s_out.wait_event(done)
            for t, h in zip(results, (out_h, gx_h, gw_h)):
                t.record_stream(s_out)
                h.copy_(t, non_blocking=True)
            ev_out.record(s_out)

    e2e_steps = max(4, min(args.steps, 8))
    e2e_step(0)
    e2e_step(1)
    s_cmp.wait_event(ev_out)
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for i in range(e2e_steps):
        e2e_step(i)
    s_cmp.wait_event(ev_out)                                 # the last results have reached the host buffers
    f1.record()
    barrier()
    t2 = torch.tensor([f0.elapsed_time(f1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t2, op=dist.ReduceOp.MAX)
    e2e_ms = float(t2.item()) / e2e_steps
    h2d = x_h.numel() * 2 + dy_h.numel() * 2
    d2h = out_h.numel() * 2 + gx_h.numel() * 2 + gw_h.numel() * 4
    return e2e_ms, h2d, d2h


# ---------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------
_REAL_STDOUT = None


def _quiet_stdout():
    """Libraries (NCCL prints its version banner) write to file descriptor 1; the contract is ONE JSON
    line on stdout, so everything but that line is sent to stderr."""
    global _REAL_STDOUT
    sys.stdout.flush()
    _REAL_STDOUT = os.dup(1)
    os.dup2(2, 1)


def emit(line: dict) -> None:
    data = (json.dumps(line) + "\n").encode()
    if _REAL_STDOUT is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_REAL_STDOUT, data)


def main():
    _quiet_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-moe", action="store_true", help="skip the MoE layer measurements")
    ap.add_argument("--no-kernels", action="store_true", help="skip the per-kernel list (N = 1)")
    ap.add_argument("--no-c5", action="store_true", help="skip the end-to-end training step of the reference's model")
    ap.add_argument("--no-peak", action="store_true", help="skip the library FP8 GEMM peak measurement (roofline falls back to 2 x bf16)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-to-host leg (e2e is then null)")
    ap.add_argument("--moe-exchange", default="p2p-fused", choices=["nccl", "p2p", "p2p-fused"],
                    help="expert-parallel exchange (N > 1): all-to-all collectives, or peer stores into symmetric memory")
    ap.add_argument("--moe-chunks", type=int, default=1,
                    help="token chunks of the expert-parallel layer (N > 1): exchanges of one chunk run under the experts of another")
    ap.add_argument("--moe-splits", type=int, default=1, choices=[1, 2, 4],
                    help="peer-store exchange (N > 1): ranges of local experts dispatched and up-projected one after the other")
    ap.add_argument("--moe-dispatch-sms", type=int, default=32,
                    help="peer-store exchange (N > 1): SMs the dispatch stores come from while the shared expert runs on the rest (0 = dispatch on all SMs, shared expert after it; 32 measured best at 2 and 8 GPUs)")
    ap.add_argument("--shape", default=None, help="M,K,N of a smaller case (profiling captures); default is the FFN workload")
    ap.add_argument("--extras-small", action="store_true",
                    help="run only the MoE plumbing passes and sparse attention on a reduced case (profiling captures) and exit")
    args = ap.parse_args()
    if args.shape:
        global M, K, N, FLOP_PER_STEP, WORKLOAD
        M, K, N = (int(v) for v in args.shape.split(","))
        FLOP_PER_STEP = 3 * 2.0 * M * N * K
        WORKLOAD = f"fp8_linear_fwd_bwd M={M} K={K} N={N} (reduced case, not the headline workload)"
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    if args.impl == "reference":
        reference_arm(args)
        return

    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the FP8 kernels have no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from cinnamon_b200 import kernels as Kmod      # raises if the CUDA library is missing
    if args.extras_small:
        extras_small(Kmod, dev)
        return

    x_h, w_h, dy_h = make_inputs(1002 + rank, pinned=True)
    x = x_h.to(dev).requires_grad_(True)
    w = w_h.to(dev).requires_grad_(True)
    dy = dy_h.to(dev)

    def step():
        x.grad = None
        w.grad = None
        out = Kmod.FP8MatmulFunction.apply(x, w, False)
        out.backward(dy)
        return out

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()              # started early: nvidia-smi needs a moment before its first sample
    for _ in range(args.warmup):
        step()
    barrier()
    assert Kmod.device_status() == 0, "a kernel reported a device-side failure during warm-up"

    # ---- timed region: device-resident inputs ----
    Kmod.gemm_events = []
    launches0 = Kmod.launch_count
    barrier()
    sampler.mark_begin()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    sampler.mark_end()
    launches = Kmod.launch_count - launches0
    events, Kmod.gemm_events = Kmod.gemm_events, None
    clocks = sampler.stop() if rank == 0 else None
    ms = e0.elapsed_time(e1)
    gemm_ms = [a.elapsed_time(b) for a, b in events]
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = float(t.item())
    assert Kmod.device_status() == 0, "a kernel reported a device-side failure in the timed region"

    # ---- end to end: pinned host inputs in, host results out, every step ----
    e2e_ms, h2d, d2h = None, 0, 0
    out_h = gx_h = gw_h = None
    if not args.no_e2e:
        e2e_ms, h2d, d2h = run_e2e(Kmod, dev, args, world, x_h, dy_h, w, barrier)

    # dense FP8 peak of this GPU (library GEMM), measured here: the denominator of the roofline fractions
    # (the burst figure first and the per-kernel list right after it, while the part is cool; the two-second
    # sustained loop afterwards, followed by a pause before anything else is timed)
    kernel_lines = []
    if rank == 0 and world == 1 and not args.shape and not args.no_kernels:
        time.sleep(2.0)
        burst = measure_fp8_peak(dev, sustained=False)
        kernel_lines = bench_kernels(Kmod, dev, x, w, dy, measured_peaks()[0], (burst or {}).get("fp8_tflops"))
    fp8 = measure_fp8_peak(dev) if rank == 0 and not args.no_peak else None
    time.sleep(2.0)
    barrier()
    moe_lines = []
    if not args.no_moe and not args.shape:
        del x, w, dy
        torch.cuda.empty_cache()
        for scale, label in ((1.0, "bias~N(0,1) as specified"), (0.1, "mild skew: bias~N(0,0.1)")):
            moe_lines.append(bench_moe(Kmod, dev, rank, world, steps=5, warmup=3, bias_scale=scale, label=label,
                                       chunks=args.moe_chunks, exchange=args.moe_exchange, splits=args.moe_splits,
                                       dispatch_sms=args.moe_dispatch_sms))
        assert Kmod.device_status() == 0, "a kernel reported a device-side failure in the MoE layer"

    c5_line = None
    if not args.no_c5 and not args.shape:
        c5_line = bench_c5(dev, rank, world)

    if rank == 0:
        peaks, peak_kind = measured_peaks()
        ms_per_step = ms_max / args.steps
        value = world * FLOP_PER_STEP / (ms_per_step * 1e-3) / 1e12
        gemm_avg_ms = sum(gemm_ms) / max(1, len(gemm_ms))
        gemm_flop = 2.0 * M * N * K
        achieved = gemm_flop / (gemm_avg_ms * 1e-3) / 1e12 if gemm_ms else None
        if fp8 and "fp8_tflops_sustained" in fp8:
            fp8_peak = float(fp8["fp8_tflops_sustained"])
            peak_source = ("dense FP8 GEMM measured in this run, sustained (" + fp8["how"] + "); the GEMM launches are "
                           "timed inside a long step, where the part sits at its power cap")
        else:
            fp8_peak = 2.0 * float(peaks["bf16_tflops_sustained"])
            peak_source = (f"2 x bf16_tflops_sustained of {peak_kind} MEASURED_PEAKS (the FP8 library GEMM was not "
                           f"available: {(fp8 or {}).get('unavailable')})")
        line = {
            "metric": "fp8_linear_fwd_bwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3 (fp32 accumulate)", "data": "synthetic",
            "config": bench_config(world),
            "roofline": {"kernel": "fp8_gemm_kernel / fp8_gemm_pair_kernel (forward, dgrad, wgrad launches averaged)", "bound": "tensor", "achieved": achieved, "peak": fp8_peak,
                         "unit": "TFLOP/s", "frac": (achieved / fp8_peak) if achieved else None,
                         "peak_source": peak_source, "fp8_peak_measured": fp8,
                         "frac_of_2x_bf16_sustained": (achieved / (2.0 * float(peaks["bf16_tflops_sustained"]))) if achieved else None,
                         "frac_of_nominal_4500": (achieved / 4500.0) if achieved else None,
                         "launches_timed": len(gemm_ms), "avg_launch_ms": gemm_avg_ms,
                         "traffic": GEMM_TRAFFIC_BYTES if not args.shape else None,
                         "traffic_source": "ncu dram__bytes_read+write of the three GEMMs on a reduced case (8192x9216x7168), each "
                                           "scaled by the algorithmic bytes of its full launch, averaged"},
            "e2e": ({"value": world * FLOP_PER_STEP / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                     "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms} if e2e_ms else None),
            "gpu_launches": launches,
            "clocks": clocks,
        }
        if kernel_lines:
            line["kernels"] = kernel_lines
        if moe_lines:
            line["moe"] = moe_lines
        if c5_line:
            line["c5"] = c5_line
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"], _ = run_cpu_baseline(256, repeats=1)
        emit(line)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
