"""Fused all-gather→GEMM and GEMM→reduce-scatter kernels on 2+ GPUs against the NCCL
composition (run as child processes, one per GPU; plain peer loads/stores, NVLS off)."""
import os
import subprocess
import sys
import tempfile

import pytest
import torch

pytestmark = pytest.mark.gpu

WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["ELL_ROOT"])
from easyllm_b200.parallel.grid import initialize_distributed, get_grid
from easyllm_b200.parallel import symm, tp_linear
from easyllm_b200 import ops
import easyllm_b200.ops.cuda as cu
tp = int(os.environ["WORLD_SIZE"])
initialize_distributed(tp=tp, pp=1, backend="nccl", launcher="torch", timeout_s=120)
g = get_grid()
torch.manual_seed(7)
T, H, F = 2048, 1024, 1536
ws = symm.FusedTPWorkspace(T, H)
full_x = (torch.randn(T, H, device="cuda") * 0.5).to(torch.bfloat16)          # same on every rank
w_col = (torch.randn(F // tp * 2, H, device="cuda") * 0.05).to(torch.bfloat16)  # per-rank weights differ by seed below
torch.manual_seed(100 + g.tp_rank)
w_col = (torch.randn(F // tp * 2, H, device="cuda") * 0.05).to(torch.bfloat16)
w_row = (torch.randn(H, F // tp, device="cuda") * 0.05).to(torch.bfloat16)
bias = torch.randn(w_col.shape[0], device="cuda").to(torch.bfloat16)
rows = T // tp
x_local = full_x[g.tp_rank * rows:(g.tp_rank + 1) * rows].contiguous()
worst = 0.0
for it in range(4):                                    # repeated calls exercise epoch / done handshakes
    y = ws.ag_gemm(x_local, w_col, bias if it % 2 else None)
    ref = torch.nn.functional.linear(full_x.float(), w_col.float(), bias.float() if it % 2 else None)
    worst = max(worst, (y.float() - ref).abs().max().item() / max(1.0, ref.abs().max().item()))
    a = (torch.randn(T, F // tp, device="cuda") * 0.5).to(torch.bfloat16)
    part = a.float() @ w_row.float().t()
    dist.all_reduce(part, group=g.tp_group)
    ref_rs = part[g.tp_rank * rows:(g.tp_rank + 1) * rows]
    y_rs = ws.gemm_rs(a, w_row)
    worst = max(worst, (y_rs.float() - ref_rs).abs().max().item() / max(1.0, ref_rs.abs().max().item()))
    # dgrad form: dy [T, N_local] · W [N_local, H] with W read as an MN-major operand
    dy = (torch.randn(T, w_col.shape[0], device="cuda") * 0.5).to(torch.bfloat16)
    part = dy.float() @ w_col.float()
    dist.all_reduce(part, group=g.tp_group)
    y_dg = ws.gemm_rs(dy, w_col, b_mn=True)
    ref_dg = part[g.tp_rank * rows:(g.tp_rank + 1) * rows]
    worst = max(worst, (y_dg.float() - ref_dg).abs().max().item() / max(1.0, ref_dg.abs().max().item()))
torch.cuda.synchronize()
cu.check_err_flag()
# the same ops through the autograd TP linears, fused vs NCCL composition
symm.install(T, H)
def run(fused):
    if not fused:
        tp_linear.set_fused_impl(None, None)
    xl = x_local.clone().requires_grad_()
    wc = w_col.clone().requires_grad_(); wr = w_row.clone().requires_grad_()
    h = tp_linear.column_parallel_linear(xl, wc, None, True)
    o = tp_linear.row_parallel_linear(h[:, :F // tp].contiguous(), wr, None, True)
    o.float().pow(2).mean().backward()
    return o.detach().float(), xl.grad.float(), wc.grad.float(), wr.grad.float()
a = run(True); b = run(False)
for u, v in zip(a, b):
    worst = max(worst, (u - v).abs().max().item() / max(1e-3, v.abs().max().item()))
torch.cuda.synchronize()
cu.check_err_flag()
print(f"RANK{g.rank} worst_rel_err={worst:.5f}", flush=True)
assert worst < 3e-2, worst
dist.barrier()
dist.destroy_process_group()
'''


def _run(nproc):
    if not torch.cuda.is_available() or torch.cuda.device_count() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path = os.path.join(tempfile.mkdtemp(prefix="ell_fused_tp_"), "worker.py")
    with open(path, "w") as f:
        f.write(WORKER)
    env = dict(os.environ, ELL_ROOT=root, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", "29611", path]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("worst_rel_err") == nproc


def test_fused_tp_2gpu():
    _run(2)


def test_fused_tp_4gpu():
    _run(4)
