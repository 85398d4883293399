"""sm_100a elementwise / reduction kernels against fp32 PyTorch statements of the same op."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cu():
    if not torch.cuda.is_available():
        pytest.skip("no GPU")
    import easyllm_b200.ops.cuda as cu
    cu.lib()
    return cu


def _close(a, b, atol, rtol):
    assert torch.allclose(a.float(), b.float(), atol=atol, rtol=rtol), (a.float() - b.float()).abs().max().item()


@pytest.mark.parametrize("rows,cols", [(7, 256), (300, 4096), (1024, 5120), (33, 8192)])
def test_rmsnorm_fwd_bwd(cu, rows, cols):
    from easyllm_b200.ops import reference as ref
    torch.manual_seed(0)
    x = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16)
    res = torch.randn_like(x)
    w = (1 + 0.1 * torch.randn(cols, device="cuda")).to(torch.bfloat16)
    y, _, rstd = cu.rmsnorm_fwd(x, None, w, 1e-5)
    _close(y, ref.rmsnorm(x.float(), w.float(), 1e-5), 2e-2, 2e-2)
    y2, h, rstd2 = cu.rmsnorm_fwd(x, res, w, 1e-5)
    hr = (x.float() + res.float()).to(torch.bfloat16)
    assert torch.equal(h, hr)
    _close(y2, ref.rmsnorm(hr.float(), w.float(), 1e-5), 2e-2, 2e-2)
    # backward vs autograd of the fp32 statement
    dy = torch.randn_like(x)
    dres = torch.randn_like(x)
    hf = hr.float().requires_grad_()
    wf = w.float().requires_grad_()
    ref.rmsnorm(hf, wf, 1e-5).backward(dy.float())
    dh, dw = cu.rmsnorm_bwd(dy, h, w, rstd2, dres)
    _close(dh, hf.grad + dres.float(), 3e-2, 3e-2)
    _close(dw, wf.grad, 5e-2 * max(1.0, wf.grad.abs().max().item()), 3e-2)
    # accumulate mode adds onto an existing fp32 buffer
    acc = torch.ones(cols, device="cuda")
    cu.rmsnorm_bwd(dy, h, w, rstd2, None, dw_out=acc, accumulate=True)
    _close(acc - 1, wf.grad, 5e-2 * max(1.0, wf.grad.abs().max().item()), 3e-2)


@pytest.mark.parametrize("T,hq,hk,D", [(64, 4, 4, 128), (257, 8, 2, 128), (33, 4, 1, 64)])
def test_rope_packed(cu, T, hq, hk, D):
    from easyllm_b200.ops import reference as ref
    torch.manual_seed(1)
    W = (hq + 2 * hk) * D
    qkv = torch.randn(T, W, device="cuda", dtype=torch.bfloat16)
    pos = torch.randint(0, 500, (T,), device="cuda", dtype=torch.int32)
    cos, sin = ref.rope_tables(D, 512, device="cuda")
    q = qkv[:, :hq * D].reshape(T, hq, D).float()
    k = qkv[:, hq * D:(hq + hk) * D].reshape(T, hk, D).float()
    rq, rk = ref.rope(q, k, cos, sin, pos.long())
    v_before = qkv[:, (hq + hk) * D:].clone()
    orig = qkv.clone()
    cu.rope_(qkv, cos, sin, pos, hq + hk, D)
    _close(qkv[:, :hq * D].reshape(T, hq, D), rq, 2e-2, 2e-2)
    _close(qkv[:, hq * D:(hq + hk) * D].reshape(T, hk, D), rk, 2e-2, 2e-2)
    assert torch.equal(qkv[:, (hq + hk) * D:], v_before)
    cu.rope_(qkv, cos, sin, pos, hq + hk, D, backward=True)   # inverse rotation
    _close(qkv, orig, 3e-2, 3e-2)


@pytest.mark.parametrize("T,F", [(5, 64), (300, 11008), (128, 3456)])
def test_swiglu(cu, T, F):
    torch.manual_seed(2)
    gu = torch.randn(T, 2 * F, device="cuda", dtype=torch.bfloat16)
    out = cu.swiglu_fwd(gu)
    g, u = gu[:, :F].float().requires_grad_(), gu[:, F:].float().requires_grad_()
    r = torch.nn.functional.silu(g) * u
    _close(out, r, 2e-2, 2e-2)
    d = torch.randn(T, F, device="cuda", dtype=torch.bfloat16)
    r.backward(d.float())
    dgu = cu.swiglu_bwd(d, gu)
    _close(dgu[:, :F], g.grad, 3e-2, 3e-2)
    _close(dgu[:, F:], u.grad, 3e-2, 3e-2)


@pytest.mark.parametrize("n", [1000, 1 << 20, (1 << 20) + 3])
def test_adam_and_sumsq(cu, n):
    from easyllm_b200.ops import reference as ref
    torch.manual_seed(3)
    p = torch.randn(n, device="cuda"); g = torch.randn(n, device="cuda")
    m = torch.rand(n, device="cuda") * 0.1; v = torch.rand(n, device="cuda") * 0.01
    pr, mr, vr = p.clone(), m.clone(), v.clone()
    low = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    scale = torch.tensor([0.5], device="cuda")
    cu.adam(p, g, m, v, low, 1e-3, 0.9, 0.95, 1e-8, 0.1, 7, True, 2.0, scale)
    ref.adam_step(pr, g, mr, vr, 1e-3, 0.9, 0.95, 1e-8, 0.1, 7, True, 1.0)
    _close(p, pr, 1e-6, 1e-5); _close(m, mr, 1e-6, 1e-5); _close(v, vr, 1e-7, 1e-5)
    assert torch.equal(low, p.to(torch.bfloat16))
    out = torch.zeros(1, device="cuda")
    cu.sumsq(g, out)
    _close(out, (g.double() ** 2).sum().float().view(1), 1e-2, 1e-4)


@pytest.mark.parametrize("T,V,valid", [(17, 1000, 1000), (256, 32000, 32000), (64, 38016, 38000)])
def test_cross_entropy(cu, T, V, valid):
    torch.manual_seed(4)
    logits = (3 * torch.randn(T, V, device="cuda")).to(torch.bfloat16)
    tgt = torch.randint(0, valid, (T,), device="cuda")
    parts = cu.ce_fwd(logits, tgt, 0, valid)
    lf = logits.float()[:, :valid].requires_grad_()
    ref_loss = torch.nn.functional.cross_entropy(lf, tgt, reduction="none")
    lse = torch.log(parts[:, 1]) + parts[:, 0]
    _close(lse - parts[:, 2], ref_loss, 2e-3, 2e-3)
    scale = torch.rand(T, device="cuda")
    (ref_loss * scale).sum().backward()
    work = logits.clone()
    cu.ce_bwd_(work, tgt, lse.contiguous(), scale, 0, valid)
    _close(work[:, :valid], lf.grad, 2e-3, 2e-2)
    if valid < V:
        assert work[:, valid:].abs().max().item() == 0
    # a shard that does not own the targets contributes target-logit 0
    parts2 = cu.ce_fwd(logits, tgt, V, valid)
    assert parts2[:, 2].abs().max().item() == 0


def test_accumulate_bf16_into_fp32(cu):
    x = torch.randn(100003, device="cuda").to(torch.bfloat16)
    acc = torch.ones(100003, device="cuda")
    cu.accum_bf16_to_f32(x, acc)
    _close(acc, 1 + x.float(), 1e-6, 1e-6)


def test_embedding_fwd_bwd(cu):
    from easyllm_b200 import ops
    torch.manual_seed(2)
    rows, h, T, start = 1000, 256, 4096, 3000
    w = torch.randn(rows, h, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    ids = torch.randint(start - 500, start + rows + 500, (4, T // 4), device="cuda")
    ids[0, :64] = start + 7                      # many duplicates: exercises the atomics
    out = ops.embedding(ids, w, start)
    mine = (ids >= start) & (ids < start + rows)
    want = torch.where(mine[..., None], w.detach()[(ids - start).clamp(0, rows - 1)], torch.zeros((), device="cuda", dtype=w.dtype))
    assert torch.equal(out, want)
    do = torch.randn_like(out)
    out.backward(do)
    ref = torch.zeros(rows, h, device="cuda")
    ref.index_add_(0, (ids - start)[mine], do.float()[mine])
    torch.testing.assert_close(w.grad.float(), ref, rtol=2e-2, atol=2e-2)
    # accumulation into an fp32 main_grad
    w2 = w.detach().clone().requires_grad_()
    w2.main_grad = torch.ones(rows, h, device="cuda")
    ops.embedding(ids, w2, start).backward(do)
    torch.testing.assert_close(w2.main_grad, ref + 1.0, rtol=1e-4, atol=1e-3)
    assert w2.grad is None
    torch.cuda.synchronize()
    cu.check_err_flag()


def test_bounded_wait_gives_up_and_reports(cu):
    """A wait on a flag that nothing sets (and on a barrier nobody arrives on) expires after its limit, the kernel
    returns with an error code the host reads, and the context stays usable."""
    import ctypes
    L = cu.lib()
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    waited = torch.zeros(1, dtype=torch.int64, device="cuda")
    err = cu.err_flag()
    rc = L.ell_bounded_wait_selftest(ctypes.c_void_p(flag.data_ptr()), ctypes.c_uint(1), ctypes.c_void_p(err.data_ptr()),
                                     ctypes.c_void_p(waited.data_ptr()), cu._stream())
    assert rc == 0
    torch.cuda.synchronize()
    assert 3.5e9 < int(waited) < 9e9, int(waited)          # two waits of 2 s each
    with pytest.raises(cu.KernelError):
        cu.check_err_flag()
    cu.check_err_flag()                                      # the error word was cleared by the read
    # the context is healthy: a tensor-core GEMM right after gives the right answer
    a = torch.randn(256, 128, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(256, 128, device="cuda", dtype=torch.bfloat16)
    torch.testing.assert_close(cu.gemm(a, b).float(), a.float() @ b.float().t(), rtol=2e-2, atol=2e-1)
    # success path: the flag is already at the wanted epoch, nothing is reported and nothing is waited for
    flag.fill_(7)
    rc = L.ell_bounded_wait_selftest(ctypes.c_void_p(flag.data_ptr()), ctypes.c_uint(7), ctypes.c_void_p(err.data_ptr()),
                                     ctypes.c_void_p(waited.data_ptr()), cu._stream())
    assert rc == 0
    torch.cuda.synchronize()
    assert int(waited) < 1e8
    cu.check_err_flag()


@pytest.mark.parametrize("rows,cols,res", [(64, 512, False), (300, 1024, True), (1000, 4096, True), (17, 8200, False)])
def test_layernorm_kernel_matches_fp32(cu, rows, cols, res):
    """Affine LayerNorm forward and backward (input, residual, weight and bias gradients) against F.layer_norm in
    fp32 on the same bf16 inputs."""
    from easyllm_b200 import ops
    torch.manual_seed(rows + cols)
    bf = dict(device="cuda", dtype=torch.bfloat16)
    x = (torch.randn(rows, cols, **bf) * 2 + 0.5).requires_grad_()
    r = torch.randn(rows, cols, **bf).requires_grad_() if res else None
    w = (1 + 0.1 * torch.randn(cols, **bf)).requires_grad_()
    b = (0.1 * torch.randn(cols, **bf)).requires_grad_()
    out = ops.layernorm(x, w, b, 1e-5, r)
    y, h = out if res else (out, None)
    dy = torch.randn_like(y)
    y.backward(dy)
    torch.cuda.synchronize()
    cu.check_err_flag()
    xf = x.detach().float().requires_grad_(); wf = w.detach().float().requires_grad_(); bf32 = b.detach().float().requires_grad_()
    rf = r.detach().float().requires_grad_() if res else None
    hf = (xf + rf).to(torch.bfloat16).float() if res else xf      # the kernel stores the sum in bf16 and normalises that
    yf = torch.nn.functional.layer_norm(hf, (cols,), wf, bf32, 1e-5)
    yf.backward(dy.float())
    assert (y.float() - yf).abs().max().item() < 4e-2
    assert (x.grad.float() - xf.grad).abs().max().item() < 4e-2 * max(1.0, xf.grad.abs().max().item())
    if res:
        assert torch.equal(x.grad, r.grad)
        assert (h.float() - (x.detach().float() + r.detach().float())).abs().max().item() < 4e-2
    for got, want in ((w.grad, wf.grad), (b.grad, bf32.grad)):
        assert ((got.float() - want).norm() / want.norm()).item() < 2e-2


def test_out_of_range_indices_are_reported_not_dereferenced(cu):
    """Bounds checks that are always on: a rotary position beyond the cos / sin tables and a token id beyond the
    embedding table set the device error word (the host raises at its next read) instead of reading past a buffer;
    the offending rows are left unrotated / zero."""
    from easyllm_b200.ops.reference import rope_tables
    torch.manual_seed(0)
    cos, sin = rope_tables(128, 64, device="cuda")                  # positions 0..63 only
    qkv = torch.randn(16, 3 * 128, device="cuda", dtype=torch.bfloat16)
    before = qkv.clone()
    pos = torch.arange(16, dtype=torch.int32, device="cuda")
    pos[5] = 4096                                                    # outside the tables
    cu.rope_(qkv, cos, sin, pos, 2, 128)
    torch.cuda.synchronize()
    with pytest.raises(cu.KernelError, match="code 32"):
        cu.check_err_flag()
    assert torch.equal(qkv[5], before[5]) and not torch.equal(qkv[4], before[4])
    w = torch.randn(100, 64, device="cuda", dtype=torch.bfloat16)
    ids = torch.tensor([1, 2, 250, 3], device="cuda")
    out = cu.embedding_fwd(ids, w, 0, 100)
    torch.cuda.synchronize()
    with pytest.raises(cu.KernelError, match="code 31"):
        cu.check_err_flag()
    assert torch.equal(out[2], torch.zeros_like(out[2])) and torch.equal(out[1], w[2])
    cu.check_err_flag()                                              # cleared
