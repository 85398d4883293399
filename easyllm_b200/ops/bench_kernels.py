"""Device-timed micro-benchmarks of the sm_100a kernels at the flagship shapes.

    python -m easyllm_b200.ops.bench_kernels [--what gemm,norm,attn] [--iters 20] [--json out.json]

Timing: CUDA events on the launching stream, 3+ warm-ups, an L2 flush (a 256 MiB write)
between timed iterations, median of the iterations.  Fractions are "of measured" peaks read
from ``MEASURED_PEAKS.json`` (cuBLAS bf16 burst TFLOP/s, copy GB/s) when present.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch

from . import cuda as cu

_PEAKS = {"bf16_tflops": 1590.0, "hbm_gbs": 6650.0, "source": "fallback"}
_p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
if os.path.exists(_p):
    with open(_p) as f:
        d = json.load(f)
    _PEAKS = {"bf16_tflops": d["bf16_tflops"], "hbm_gbs": d["hbm_gbs"], "source": "measured"}


def timed(fn, iters=20, warmup=3):
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(iters):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda._sleep(300000)   # the device stays busy while the host prepares the launch: no host gap is timed
        a.record()
        fn()
        b.record()
        b.synchronize()
        ts.append(a.elapsed_time(b))
    return statistics.median(ts)


# Llama-2-7B per-rank GEMMs at seq 4096 (TP1 and TP2), then 13B TP4 and 70B-shape TP8 samples
GEMM_SHAPES = [
    ("7b qkv fwd", 4096, 12288, 4096, "nt"), ("7b o fwd", 4096, 4096, 4096, "nt"),
    ("7b gate_up fwd", 4096, 22016, 4096, "nt"), ("7b down fwd", 4096, 4096, 11008, "nt"),
    ("7b head fwd", 4096, 32000, 4096, "nt"),
    ("7b gate_up dgrad", 4096, 4096, 22016, "nn"), ("7b down dgrad", 4096, 11008, 4096, "nn"),
    ("7b gate_up wgrad", 22016, 4096, 4096, "tn"), ("7b down wgrad", 4096, 11008, 4096, "tn"),
    ("7b tp2 qkv fwd", 4096, 6144, 4096, "nt"), ("7b tp2 down fwd", 4096, 4096, 5504, "nt"),
    ("13b tp4 gate_up fwd", 4096, 6912, 5120, "nt"), ("70b tp8 gate_up fwd", 4096, 7168, 8192, "nt"),
]


def bench_gemm(iters):
    rows = []
    print(f"# CTA-pair kernel: {cu.lib().ell_gemm_pair_resident_clusters()} two-CTA clusters resident", flush=True)
    for name, M, N, K, lay in GEMM_SHAPES:
        if lay == "nt":
            a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16); b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
            mine = lambda: cu.gemm(a, b)                                       # noqa: E731
            lib = lambda: torch.matmul(a, b.t())                               # noqa: E731
        elif lay == "nn":
            a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16); b = torch.randn(K, N, device="cuda", dtype=torch.bfloat16)
            mine = lambda: cu.gemm(a, b, b_mn=True)                            # noqa: E731
            lib = lambda: torch.matmul(a, b)                                   # noqa: E731
        else:
            a = torch.randn(K, M, device="cuda", dtype=torch.bfloat16); b = torch.randn(K, N, device="cuda", dtype=torch.bfloat16)
            acc = torch.zeros(M, N, device="cuda")
            mine = lambda: cu.gemm(a, b, out=acc, a_mn=True, b_mn=True, out_mode=1)   # noqa: E731
            lib = lambda: torch.matmul(a.t(), b)                               # noqa: E731
        fl = 2.0 * M * N * K
        t_m, t_l = timed(mine, iters), timed(lib, iters)
        cu.set_gemm_pair(False)                      # the same call through the single-CTA kernel
        t_one = timed(mine, iters)
        cu.set_gemm_pair(True)
        rows.append({"name": name, "M": M, "N": N, "K": K, "layout": lay, "ms": t_m, "tflops": fl / t_m / 1e9,
                     "frac_of_peak": fl / t_m / 1e9 / _PEAKS["bf16_tflops"], "cublas_ms": t_l,
                     "cublas_tflops": fl / t_l / 1e9, "vs_cublas": t_l / t_m, "single_cta_ms": t_one})
        print(f"{name:24s} {M:6d}x{N:6d}x{K:6d} {lay}  {t_m:8.3f} ms {fl / t_m / 1e9:7.1f} TF "
              f"({100 * rows[-1]['frac_of_peak']:5.1f}% of {_PEAKS['source']})  cuBLAS {t_l:8.3f} ms "
              f"{fl / t_l / 1e9:7.1f} TF  ratio {t_l / t_m:5.2f}  single-CTA kernel {t_one:8.3f} ms", flush=True)
    cu.check_err_flag()
    return rows


def bench_norm(iters):
    rows = []
    for T, H in ((4096, 4096), (8192, 5120), (4096, 8192)):
        x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16); r = torch.randn_like(x)
        w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
        t = timed(lambda: cu.rmsnorm_fwd(x, r, w, 1e-5), iters)
        by = 4 * T * H * 2
        rows.append({"name": f"add_rmsnorm fwd {T}x{H}", "ms": t, "gbs": by / t / 1e6,
                     "frac_of_peak": by / t / 1e6 / _PEAKS["hbm_gbs"]})
        print(f"add_rmsnorm fwd {T}x{H}: {t:.4f} ms {by / t / 1e6:.0f} GB/s "
              f"({100 * rows[-1]['frac_of_peak']:.1f}% of {_PEAKS['source']} copy)", flush=True)
        y, h, rstd = cu.rmsnorm_fwd(x, r, w, 1e-5)
        t = timed(lambda: cu.rmsnorm_bwd(y, h, w, rstd, r), iters)
        rows.append({"name": f"add_rmsnorm bwd {T}x{H}", "ms": t, "gbs": by / t / 1e6,
                     "frac_of_peak": by / t / 1e6 / _PEAKS["hbm_gbs"]})
        print(f"add_rmsnorm bwd {T}x{H}: {t:.4f} ms {by / t / 1e6:.0f} GB/s "
              f"({100 * rows[-1]['frac_of_peak']:.1f}% of {_PEAKS['source']} copy)", flush=True)
        gu = torch.randn(T, 2 * 11008, device="cuda", dtype=torch.bfloat16)
        t = timed(lambda: cu.swiglu_fwd(gu), iters)
        by = 3 * T * 11008 * 2
        rows.append({"name": f"swiglu fwd {T}x11008", "ms": t, "gbs": by / t / 1e6,
                     "frac_of_peak": by / t / 1e6 / _PEAKS["hbm_gbs"]})
        print(f"swiglu fwd {T}x11008: {t:.4f} ms {by / t / 1e6:.0f} GB/s "
              f"({100 * rows[-1]['frac_of_peak']:.1f}%)", flush=True)
    n = 1 << 28
    p = torch.randn(n, device="cuda"); g = torch.randn(n, device="cuda"); m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda"); low = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    t = timed(lambda: cu.adam(p, g, m, v, low, 1e-4, 0.9, 0.95, 1e-8, 0.1, 3), max(3, iters // 4))
    by = n * (16 + 12 + 2)
    rows.append({"name": "adam 268M", "ms": t, "gbs": by / t / 1e6, "frac_of_peak": by / t / 1e6 / _PEAKS["hbm_gbs"]})
    print(f"adam 268M elems: {t:.3f} ms {by / t / 1e6:.0f} GB/s ({100 * rows[-1]['frac_of_peak']:.1f}%)", flush=True)
    return rows


def bench_attn(iters):
    from .. import ops
    rows = []
    for T, Hq, Hk in ((4096, 32, 32), (4096, 16, 16), (8192, 10, 10), (4096, 8, 1)):
        q = torch.randn(T, Hq, 128, device="cuda", dtype=torch.bfloat16)
        k = torch.randn(T, Hk, 128, device="cuda", dtype=torch.bfloat16); v = torch.randn_like(k)
        fl = 4.0 * T * T * 128 * Hq / 2
        res = {}
        for name in ("kernel", "library"):
            ops.set_attention_backend(name)
            try:
                t = timed(lambda: ops.flash_attention(q, k, v, None, T, True), iters)
                res[name] = t
            except Exception as e:  # kernel may not support a shape yet
                res[name] = None
                print(f"attn {name} T={T} H={Hq}/{Hk}: {type(e).__name__}: {e}")
        ops.set_attention_backend("auto")
        rows.append({"name": f"attn fwd causal T={T} H={Hq}/{Hk}", "kernel_ms": res["kernel"], "library_ms": res["library"],
                     "kernel_tflops": fl / res["kernel"] / 1e9 if res["kernel"] else None,
                     "library_tflops": fl / res["library"] / 1e9 if res["library"] else None})
        print(rows[-1], flush=True)
        # backward: the tcgen05 kernel against differentiating the library attention (its forward + backward)
        qkv = torch.randn(T, (Hq + 2 * Hk) * 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        do = torch.randn(T, Hq * 128, device="cuda", dtype=torch.bfloat16)
        o = ops.flash_attention_packed(qkv, Hq, Hk, 128, None, T)
        bres = {}
        for name in ("kernel", "library"):
            cu.set_attention_backward(name)
            bres[name] = timed(lambda: torch.autograd.grad(o, qkv, do, retain_graph=True), iters)
        cu.set_attention_backward("kernel")
        rows.append({"name": f"attn bwd causal T={T} H={Hq}/{Hk}", "kernel_ms": bres["kernel"],
                     "library_ms": bres["library"], "kernel_tflops": 2.5 * fl / bres["kernel"] / 1e9,
                     "library_tflops": 2.5 * fl / bres["library"] / 1e9})
        print(rows[-1], flush=True)
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", default="gemm,norm")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--json", default=None)
    a = ap.parse_args()
    cu.lib()
    out = {"peaks": _PEAKS}
    for w in a.what.split(","):
        out[w] = {"gemm": bench_gemm, "norm": bench_norm, "attn": bench_attn}[w](a.iters)
    if a.json:
        with open(a.json, "w") as f:
            json.dump(out, f, indent=1)


if __name__ == "__main__":
    main()
