"""Small fixed workloads for profiling one kernel at a time.

    python -m easyllm_b200.ops.profile_cases <case> [--iters 6]

Cases: gemm_nt, gemm_nt_n4096, gemm_dgrad, gemm_wgrad, gemm_ag, gemm_rs, gemm_ar (single-CTA kernel), the same with
the prefix gemm_pair_ (CTA-pair kernel) plus gemm_pair_agk (gather of the reduction rows into the weight-gradient
GEMM) and gemm_pair_ce (LM head with the cross-entropy epilogue), flash_fwd, flash_bwd, rmsnorm_fwd, rmsnorm_bwd,
swiglu, rope, adam, ce.
Inputs are larger than L2 (126 MB) where the op is memory-bound but hold well under a few GB,
so a full-section profiler capture of 1-3 launches ends by itself in a minute or two.
"""
from __future__ import annotations

import argparse

import torch

from . import cuda as cu


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case")
    ap.add_argument("--iters", type=int, default=6)
    a = ap.parse_args()
    cu.lib()
    bf = dict(device="cuda", dtype=torch.bfloat16)
    c = a.case
    if c.startswith("gemm_pair_"):          # same shapes as the single-CTA cases, through the CTA-pair kernel
        cu.set_gemm_pair(True)
        c = "gemm_" + c[len("gemm_pair_"):]
    elif c.startswith("gemm_"):
        cu.set_gemm_pair(False)
    if c == "gemm_nt":
        x = torch.randn(4096, 4096, **bf); w = torch.randn(12288, 4096, **bf)
        fn = lambda: cu.gemm(x, w)                                                   # noqa: E731
    elif c == "gemm_nt_n4096":      # few output tiles, long K: the o_proj / down_proj forward class
        x = torch.randn(4096, 11008, **bf); w = torch.randn(4096, 11008, **bf)
        fn = lambda: cu.gemm(x, w)                                                   # noqa: E731
    elif c == "gemm_nt_k2048":      # short reduction: the o_proj forward at tp 2 (epilogue-heavy: 32 k-blocks per tile)
        x = torch.randn(4096, 2048, **bf); w = torch.randn(4096, 2048, **bf)
        fn = lambda: cu.gemm(x, w)                                                   # noqa: E731
    elif c == "gemm_dgrad":
        x = torch.randn(4096, 11008, **bf); w = torch.randn(11008, 4096, **bf)
        fn = lambda: cu.gemm(x, w, b_mn=True)                                        # noqa: E731
    elif c == "gemm_wgrad":
        dy = torch.randn(4096, 11008, **bf); x = torch.randn(4096, 4096, **bf)
        acc = torch.zeros(11008, 4096, device="cuda")
        fn = lambda: cu.gemm(dy, x, out=acc, a_mn=True, b_mn=True, out_mode=1)        # noqa: E731
    elif c == "flash_fwd":
        qkv = torch.randn(4096, 3 * 32 * 128, **bf)
        q, k, v = (qkv[:, i * 4096:(i + 1) * 4096].view(4096, 32, 128) for i in range(3))
        rs = torch.zeros(4096, dtype=torch.int32, device="cuda")
        fn = lambda: cu.flash_attn_fwd(q, k, v, rs, 128 ** -0.5)                      # noqa: E731
    elif c == "flash_bwd":
        qkv = torch.randn(4096, 3 * 32 * 128, **bf)
        q, k, v = (qkv[:, i * 4096:(i + 1) * 4096].view(4096, 32, 128) for i in range(3))
        rs = torch.zeros(4096, dtype=torch.int32, device="cuda")
        out, lse = cu.flash_attn_fwd(q, k, v, rs, 128 ** -0.5)
        do = torch.randn_like(out)
        dqkv = torch.empty_like(qkv)
        dq, dk, dv = (dqkv[:, i * 4096:(i + 1) * 4096].view(4096, 32, 128) for i in range(3))
        fn = lambda: cu.flash_attn_bwd(do, q, k, v, out, lse, rs, 128 ** -0.5, dq, dk, dv)   # noqa: E731
    elif c == "gemm_ce":
        x = torch.randn(4096, 4096, **bf); w = torch.randn(32000, 4096, **bf) * 0.02
        t = torch.randint(0, 32000, (4096,), device="cuda")
        fn = lambda: cu.gemm_ce(x, w, t, 0, 32000)                                    # noqa: E731
    elif c in ("gemm_ag", "gemm_rs", "gemm_rs_k2048", "gemm_ar", "gemm_agk"):
        # the fused tensor-parallel kernels on a one-rank group: same kernel, flags and staging path, no peers
        import os
        import torch.distributed as dist
        from ..parallel import symm
        from ..parallel.grid import initialize_distributed
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1"); os.environ.setdefault("MASTER_PORT", "29655")
        os.environ.setdefault("RANK", "0"); os.environ.setdefault("WORLD_SIZE", "1"); os.environ.setdefault("LOCAL_RANK", "0")
        if not dist.is_initialized():
            initialize_distributed(tp=1, pp=1, backend="nccl", launcher="torch")
        ws = symm.FusedTPWorkspace(4096, 11008)
        if c == "gemm_ag":
            x = torch.randn(4096, 4096, **bf); w = torch.randn(22016, 4096, **bf)
            fn = lambda: ws.ag_gemm(x, w)                                             # noqa: E731
        elif c == "gemm_agk":
            dy = torch.randn(4096, 11008, **bf); x = torch.randn(4096, 4096, **bf)
            acc = torch.zeros(11008, 4096, device="cuda")
            fn = lambda: ws.agk_wgrad(dy, x, acc)                                     # noqa: E731
        else:
            k = 2048 if c.endswith("k2048") else 11008
            x = torch.randn(4096, k, **bf); w = torch.randn(4096, k, **bf)
            fn = lambda: ws.gemm_rs(x, w, all_reduce=(c == "gemm_ar"))                # noqa: E731
    elif c in ("rmsnorm_fwd", "rmsnorm_bwd"):
        x = torch.randn(16384, 4096, **bf); r = torch.randn_like(x); w = torch.ones(4096, **bf)
        y, h, rstd = cu.rmsnorm_fwd(x, r, w, 1e-5)
        fn = (lambda: cu.rmsnorm_fwd(x, r, w, 1e-5)) if c == "rmsnorm_fwd" else (lambda: cu.rmsnorm_bwd(y, h, w, rstd, r))
    elif c == "swiglu":
        gu = torch.randn(8192, 22016, **bf)
        fn = lambda: cu.swiglu_fwd(gu)                                                # noqa: E731
    elif c == "rope":
        qkv = torch.randn(8192, 12288, **bf)
        from .reference import rope_tables
        cos, sin = rope_tables(128, 8192, device="cuda")
        pos = torch.arange(8192, dtype=torch.int32, device="cuda")
        fn = lambda: cu.rope_(qkv, cos, sin, pos, 64, 128)                            # noqa: E731
    elif c == "adam":
        n = 1 << 27
        p = torch.randn(n, device="cuda"); g = torch.randn(n, device="cuda"); m = torch.zeros(n, device="cuda")
        v = torch.zeros(n, device="cuda"); low = torch.empty(n, **bf)
        fn = lambda: cu.adam(p, g, m, v, low, 1e-4, 0.9, 0.95, 1e-8, 0.1, 3)          # noqa: E731
    elif c == "ce":
        lg = torch.randn(4096, 32000, **bf); t = torch.randint(0, 32000, (4096,), device="cuda")
        fn = lambda: cu.ce_fwd(lg, t, 0, 32000)                                       # noqa: E731
    else:
        raise SystemExit(f"unknown case {c}")
    for _ in range(a.iters):
        fn()
    torch.cuda.synchronize()
    cu.check_err_flag()
    print(f"{a.case}: {a.iters} launches done")


if __name__ == "__main__":
    main()
