"""Device-timed comparison of the fused TP kernels with the NCCL + GEMM composition.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        -m easyllm_b200.parallel.bench_fused_tp [--model 7b] [--iters 20] [--json out.json]

Per shape: median over iterations of the CUDA-event time, maximum over ranks; an L2 flush
between iterations; a short device-side sleep precedes the first event so host launch work is not timed.  The roofline of a fused kernel is the slower of FLOPs at the measured
bf16 GEMM peak and the bytes that must cross NVLink at 770 GB/s per direction per GPU.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch
import torch.distributed as dist

from .. import ops
from ..ops import cuda as cu
from . import mappings as mp
from .grid import get_grid, initialize_distributed
from .symm import FusedTPWorkspace

LINK_GBS = 770.0
SHAPES = {  # name: (hidden, ffn, heads·d)
    "7b": (4096, 11008, 4096), "13b": (5120, 13824, 5120), "70b": (8192, 28672, 8192),
}


def _peak():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return json.load(f)["bf16_tflops"], "measured"
    return 1590.0, "fallback"


def timed(fn, iters, group, burst=1):
    """Median CUDA-event time of ``fn`` (max over ranks).  ``burst`` > 1 times that many back-to-back calls and
    divides: the ranks leave the barrier and the busy-wait below a few tens of microseconds apart (their clocks
    differ), and a single fused call charges that skew to whichever rank started first; in a burst the kernels'
    own handshakes keep the ranks in step, as the surrounding collectives do in a training step."""
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(3):
        fn()
    ts = []
    for _ in range(iters):
        flush.zero_()
        dist.barrier(group=group)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        # keep the device busy while the host prepares the launch (tensor maps, allocations), so the interval
        # between the two events is device time of the kernels only
        torch.cuda._sleep(400000 * burst)
        a.record()
        for _ in range(burst):
            fn()
        b.record()
        b.synchronize()
        ts.append(a.elapsed_time(b) / burst)
    t = torch.tensor([statistics.median(ts)], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="7b")
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--json", default=None)
    ap.add_argument("--burst", type=int, default=0, help="also time this many back-to-back calls per op (divided by "
                    "the count): free of the start skew between ranks, but the operands stay in L2")
    a = ap.parse_args()
    tp = int(os.environ.get("WORLD_SIZE", "1"))
    initialize_distributed(tp=tp, pp=1, backend="nccl")
    g = get_grid()
    H, F, QD = SHAPES[a.model]
    T = a.seq
    peak, src = _peak()
    ws = FusedTPWorkspace(T, H)
    rows = T // tp
    x_local = torch.randn(rows, H, device="cuda", dtype=torch.bfloat16)
    results = []

    def burst_of(fn):
        return timed(fn, max(4, a.iters // 2), g.tp_group, a.burst) if a.burst > 1 else None

    def report(name, kind, M, N, K, t_fused, t_comp, b_fused=None, b_comp=None):
        fl = 2.0 * M * N * K
        # bytes one GPU must receive: its peers' shards of the gathered operand (ag: rows of A, agk: rows of the
        # reduction operand), the peers' partials of its own rows (rs), or both phases of the two-shot all-reduce
        per_kind = {"ag": M * K, "agk": K * N, "rs": M * N, "ar": 2 * M * N}[kind]
        link_bytes = (tp - 1) / tp * per_kind * 2
        bound_ms = max(fl / (peak * 1e9), link_bytes / (LINK_GBS * 1e6))
        row = {"name": name, "kind": kind, "M": M, "N": N, "K": K, "tp": tp, "fused_ms": t_fused, "nccl_gemm_ms": t_comp,
               "speedup": t_comp / t_fused, "roofline_ms": bound_ms, "frac_of_roofline": bound_ms / t_fused,
               "tflops": fl / t_fused / 1e9}
        results.append(row)
        if g.rank == 0:
            print(f"{name:22s} tp{tp} {M}x{N}x{K}  fused {t_fused:7.3f} ms ({fl / t_fused / 1e9:6.0f} TF, "
                  f"{100 * row['frac_of_roofline']:5.1f}% of roofline [{src} peak])  nccl+gemm {t_comp:7.3f} ms  "
                  f"x{row['speedup']:.2f}", flush=True)
            if b_fused is not None:
                row["fused_burst_ms"], row["nccl_gemm_burst_ms"] = b_fused, b_comp
                print(f"{'':22s} burst of {a.burst} (no start skew, operands L2-warm): fused {b_fused:7.3f} ms "
                      f"({100 * bound_ms / b_fused:5.1f}% of roofline)  nccl+gemm {b_comp:7.3f} ms", flush=True)

    for name, N in (("qkv ag->gemm", 3 * QD // tp), ("gate_up ag->gemm", 2 * F // tp)):
        w = torch.randn(N, H, device="cuda", dtype=torch.bfloat16) * 0.02
        t_f = timed(lambda: ws.ag_gemm(x_local, w), a.iters, g.tp_group)

        def comp():
            xg = mp.gather_first_dim(x_local)
            return ops.matmul_nt(xg, w)
        report(name, "ag", T, N, H, t_f, timed(comp, a.iters, g.tp_group), burst_of(lambda: ws.ag_gemm(x_local, w)), burst_of(comp))
    for name, K in (("o_proj gemm->rs", QD // tp), ("down gemm->rs", F // tp)):
        K = (K + 7) // 8 * 8
        x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(H, K, device="cuda", dtype=torch.bfloat16) * 0.02
        t_f = timed(lambda: ws.gemm_rs(x, w), a.iters, g.tp_group)

        def comp():
            return mp.reduce_scatter_first_dim(ops.matmul_nt(x, w))
        report(name, "rs", T, H, K, t_f, timed(comp, a.iters, g.tp_group), burst_of(lambda: ws.gemm_rs(x, w)), burst_of(comp))
    # the backward and non-sequence-parallel forms, on the widest layer of the model
    K = (F // tp + 7) // 8 * 8
    x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(H, K, device="cuda", dtype=torch.bfloat16) * 0.02
    t_f = timed(lambda: ws.gemm_rs(x, w, all_reduce=True), a.iters, g.tp_group)

    def comp_ar():
        y = ops.matmul_nt(x, w)
        dist.all_reduce(y, group=g.tp_group)
        return y
    report("down gemm->allreduce", "ar", T, H, K, t_f, timed(comp_ar, a.iters, g.tp_group),
           burst_of(lambda: ws.gemm_rs(x, w, all_reduce=True)), burst_of(comp_ar))
    N = 2 * F // tp
    dy = torch.randn(T, N, device="cuda", dtype=torch.bfloat16)
    acc = torch.zeros(N, H, device="cuda")
    if ws._pair(rows, N):
        t_f = timed(lambda: ws.agk_wgrad(dy, x_local, acc), a.iters, g.tp_group)

        def comp_wg():
            xg = mp.gather_first_dim(x_local)
            return ops.matmul_tn_accum(dy, xg, acc)
        report("gate_up ag->wgrad", "agk", N, H, T, t_f, timed(comp_wg, a.iters, g.tp_group),
               burst_of(lambda: ws.agk_wgrad(dy, x_local, acc)), burst_of(comp_wg))
    torch.cuda.synchronize()
    cu.check_err_flag()
    if a.json and g.rank == 0:
        with open(a.json, "w") as f:
            json.dump({"peak_tflops": peak, "peak_source": src, "link_gbs": LINK_GBS, "rows": results}, f, indent=1)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
