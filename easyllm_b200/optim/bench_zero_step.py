"""Timing of the data-parallel optimizer step (ZeRO-1, fused kernels over symmetric memory) against the NCCL
composition, on the GPUs of one node:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m easyllm_b200.optim.bench_zero_step [--numel 268435456] [--iters 8] [--json out.json]

One step = reduce-scatter of the flat fp32 gradient buffer (1/dp folded in, sum of squares in the same pass),
gradient-norm all-reduce, clip, fused Adam on this rank's shard and the all-gather of the bf16 parameters.  The fused
path does the two collectives inside its own kernels (peer loads of the other ranks' gradient slices, peer stores of
the updated parameters); the composition calls NCCL ``reduce_scatter_tensor`` / ``all_gather_into_tensor`` around the
same Adam kernel (``EASYLLM_ZERO_FUSED=0``).  Times are CUDA events around ``optimizer.step()``, median over
iterations, maximum over ranks; the buffers (1.5 GiB + per 2^28 parameters) are far larger than L2.

Bytes over NVLink per rank and step: it reads (dp-1)/dp of its shard's fp32 gradients from the peers
(4 * numel * (dp-1) / dp) and writes its bf16 shard to dp-1 peers (2 * numel * (dp-1) / dp); the roofline is
those bytes over the measured per-direction peer bandwidth (reads and writes travel in opposite directions, so the
slower of the two bounds the step), or the HBM traffic of the Adam pass when that is larger.
"""
import argparse
import json
import os
import statistics

import torch
import torch.distributed as dist

LINK_GBS = 770.0     # measured peer-copy bandwidth per direction on this pool
HBM_GBS = 6536.0     # measured copy bandwidth


def build(numel, stage, fused):
    from ..optim import ZeroOptimizer
    os.environ["EASYLLM_ZERO_FUSED"] = "1" if fused else "0"
    torch.manual_seed(0)
    chunk = 1 << 24
    params = []
    for i in range(max(1, numel // chunk)):
        p = torch.nn.Parameter(torch.randn(chunk // 4096, 4096, device="cuda", dtype=torch.bfloat16) * 0.02)
        params.append((f"layer.{i}.weight", p))
    opt = ZeroOptimizer(params, lr=1e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, stage=stage, grad_clip=1.0)
    return opt, params


def time_steps(opt, iters, group):
    ts = []
    for it in range(iters + 2):
        opt.grad_buf.normal_(0.0, 1e-3)               # fresh gradients (also evicts whatever L2 held)
        dist.barrier(group=group)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        opt.step()
        b.record()
        b.synchronize()
        if it >= 2:
            ts.append(a.elapsed_time(b))
    t = torch.tensor([statistics.median(ts)], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--numel", type=int, default=1 << 28)
    ap.add_argument("--iters", type=int, default=8)
    ap.add_argument("--json", default=None)
    a = ap.parse_args()
    from ..parallel.grid import initialize_distributed, get_grid
    import easyllm_b200.ops.cuda as cu
    initialize_distributed(tp=1, pp=1, backend="nccl")
    g = get_grid()
    dp = g.dp
    rows = []
    for fused in (True, False):
        opt, params = build(a.numel, 1, fused)
        if fused and not opt.fused:
            raise SystemExit("fused ZeRO path unavailable (no symmetric memory)")
        ms = time_steps(opt, a.iters, g.dp_group)
        rows.append(ms)
        del opt, params
        torch.cuda.empty_cache()
    cu.check_err_flag()
    n = (a.numel // (1 << 24)) * (1 << 24)
    rd = 4.0 * n * (dp - 1) / dp / dp                 # peer reads of this rank's gradient shard from dp-1 ranks
    wr = 2.0 * n * (dp - 1) / dp                      # peer stores of this rank's parameter shard to dp-1 ranks
    hbm = (4 * n + 4 * n / dp) + (16 + 12 + 2) * n / dp   # gradient pass (read all, write shard) + Adam state traffic
    bound_ms = max(max(rd, wr) / (LINK_GBS * 1e6), hbm / (HBM_GBS * 1e6))
    out = {"numel": n, "dp": dp, "fused_ms": rows[0], "nccl_ms": rows[1], "speedup": rows[1] / rows[0],
           "nvlink_read_gb": rd / 1e9, "nvlink_write_gb": wr / 1e9, "roofline_ms": bound_ms,
           "frac_of_roofline": bound_ms / rows[0],
           "achieved_link_gbs": max(rd, wr) / rows[0] / 1e6}
    if g.rank == 0:
        print(f"ZeRO-1 step, {n / 2**20:.0f} Mi parameters over dp{dp}: fused {rows[0]:.2f} ms, NCCL composition "
              f"{rows[1]:.2f} ms (x{out['speedup']:.2f}); roofline {bound_ms:.2f} ms -> {100 * out['frac_of_roofline']:.0f}% "
              f"[of measured]; peer traffic {out['nvlink_read_gb']:.2f} GB read / {out['nvlink_write_gb']:.2f} GB written "
              f"per rank", flush=True)
        if a.json:
            with open(a.json, "w") as f:
                json.dump(out, f, indent=1)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
