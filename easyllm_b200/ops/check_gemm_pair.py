"""Self-check of the CTA-pair GEMM (``csrc/gemm_pair.cu``) against fp32 matmul, then its device time beside the
single-CTA kernel (``csrc/gemm.cu``) on the Llama-2-7B GEMM shapes.

    python -m easyllm_b200.ops.check_gemm_pair [--iters 20] [--json out.json]

Numerics stop at the first failing case (error word set or difference above the rounding bound) and print the
worst difference per 128 x 128 quadrant of the first output tile, which tells the two CTAs' row halves and the
two B halves apart.  Timing: CUDA events around ``iters`` back-to-back launches after three warm-up launches, with
a device-side sleep before the first event so no host launch latency is inside the interval.
"""
from __future__ import annotations

import argparse
import json

import torch

from . import cuda as cu

CASES = [(256, 256, 64, {}), (256, 256, 512, {}), (512, 768, 512, {}), (2048, 1024, 1024, dict(bias=True)),
         (1024, 1024, 1024, dict(b_mn=True)), (1024, 1024, 1024, dict(a_mn=True, b_mn=True)),
         (1024, 1024, 1024, dict(a_mn=True, b_mn=True, out_mode=1)),
         (1024, 1024, 1024, dict(a_mn=True, b_mn=True, out_mode=2)),
         (1024, 1024, 1024, dict(out_mode=2)), (1024, 1024, 1024, dict(b_mn=True, out_mode=2)),
         (384, 320, 192, {}), (4096, 12288, 4096, {})]

BENCH = [("qkv fwd", 4096, 12288, 4096, {}), ("gate_up fwd", 4096, 22016, 4096, {}),
         ("down fwd", 4096, 4096, 11008, {}), ("o fwd", 4096, 4096, 4096, {}),
         ("gate_up dgrad", 4096, 4096, 22016, dict(b_mn=True)),
         ("gate_up wgrad", 22016, 4096, 4096, dict(a_mn=True, b_mn=True, out_mode=1)),
         ("8k cube", 8192, 8192, 8192, {})]


def _operands(M, N, K, a_mn, b_mn):
    dev = torch.device("cuda")
    a = (torch.randn(K, M, device=dev) if a_mn else torch.randn(M, K, device=dev)).bfloat16()
    b = (torch.randn(K, N, device=dev) if b_mn else torch.randn(N, K, device=dev)).bfloat16()
    return a, b


def check_case(M, N, K, a_mn=False, b_mn=False, out_mode=0, bias=False):
    a, b = _operands(M, N, K, a_mn, b_mn)
    bs = torch.randn(N, device="cuda").bfloat16() if bias else None
    ref = (a.float().t() if a_mn else a.float()) @ (b.float() if b_mn else b.float().t())
    if bias:
        ref = ref + bs.float()
    out = None
    if out_mode == 1:
        out = torch.ones(M, N, device="cuda", dtype=torch.float32)
        ref = ref + 1
    y = cu.gemm(a, b, out=out, bias=bs, a_mn=a_mn, b_mn=b_mn, out_mode=out_mode, pair=True)
    torch.cuda.synchronize()
    err = int(cu.err_flag().item())
    if err:
        cu.err_flag().zero_()
    d = (y.float() - ref).abs()
    tol = 0.02 * K ** 0.5 + (0.25 if out_mode == 0 else 0)
    quad = [[d[i:i + 128, j:j + 128].max().item() for j in (0, 128)] for i in (0, 128)]
    return err, d.max().item(), tol, quad


def time_case(M, N, K, pair, iters, a_mn=False, b_mn=False, out_mode=0):
    a, b = _operands(M, N, K, a_mn, b_mn)
    out = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16 if out_mode == 0 else torch.float32)

    def fn():
        cu.gemm(a, b, out=out, a_mn=a_mn, b_mn=b_mn, out_mode=out_mode, pair=pair)
    for _ in range(3):
        fn()
    s, t = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    torch.cuda._sleep(20_000_000)
    s.record()
    for _ in range(iters):
        fn()
    t.record()
    torch.cuda.synchronize()
    ms = s.elapsed_time(t) / iters
    return ms, 2.0 * M * N * K / ms / 1e9


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--json", default=None)
    args = ap.parse_args()
    torch.manual_seed(0)
    res = {"steps": [], "bench": []}
    ok = True
    for M, N, K, kw in CASES:
        err, diff, tol, quad = check_case(M, N, K, **kw)
        good = err == 0 and diff <= tol
        res["steps"].append({"shape": [M, N, K], "kw": kw, "err": err, "maxdiff": diff, "tol": tol, "ok": good})
        print(res["steps"][-1], flush=True)
        if not good:
            print("worst difference per quadrant of the first tile:", quad, flush=True)
            ok = False
            break
    res["numerics_ok"] = ok
    if ok:
        for name, M, N, K, kw in BENCH:
            one, two = time_case(M, N, K, False, args.iters, **kw), time_case(M, N, K, True, args.iters, **kw)
            res["bench"].append({"name": name, "shape": [M, N, K], "single_ms": one[0], "single_tflops": one[1],
                                 "pair_ms": two[0], "pair_tflops": two[1]})
            print(res["bench"][-1], flush=True)
        cu.check_err_flag()
    if args.json:
        with open(args.json, "w") as f:
            json.dump(res, f, indent=1)
    print("DONE", ok)
    raise SystemExit(0 if ok else 1)


if __name__ == "__main__":
    main()
