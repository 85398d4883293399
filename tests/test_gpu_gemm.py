"""tcgen05 GEMM (all operand layouts and output modes) against fp32 matmul of the same bf16 inputs."""
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


def _check(out, ref, K):
    """Two bounds: the largest element error (catches a single bad element) and the relative Frobenius error (a
    dropped k-slice or a misplaced tile moves it far above bf16 rounding noise, which sits near 1e-3)."""
    err = (out.float() - ref).abs().max().item()
    tol = 2e-2 * max(1.0, ref.abs().max().item()) if out.dtype == torch.bfloat16 else 1e-3 * (K ** 0.5)
    assert err <= tol, (err, tol)
    rel = ((out.float() - ref).norm() / ref.norm().clamp_min(1e-12)).item()
    assert rel <= (4e-3 if out.dtype == torch.bfloat16 else 1e-4), rel


SHAPES = [(128, 256, 64), (128, 128, 128), (200, 136, 72), (512, 768, 512), (1000, 520, 264), (4096, 4096, 1024)]


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_gemm_nt(cu, M, N, K):
    torch.manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    out = cu.gemm(a, b)
    torch.cuda.synchronize()
    cu.check_err_flag()
    _check(out, a.float() @ b.float().t(), K)


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_gemm_nt_bias_and_bn128(cu, M, N, K):
    torch.manual_seed(1)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    ref = a.float() @ b.float().t()
    _check(cu.gemm(a, b, bias=bias), ref + bias.float(), K)
    _check(cu.gemm(a, b, bn=128), ref, K)
    cu.check_err_flag()


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_gemm_nn_dgrad_layout(cu, M, N, K):
    """dx = dy · W with W stored [K_red, N_out] (MN-major B)."""
    torch.manual_seed(2)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(K, N, device="cuda", dtype=torch.bfloat16)
    out = cu.gemm(a, b, b_mn=True)
    cu.check_err_flag()
    _check(out, a.float() @ b.float(), K)


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_gemm_tn_wgrad_layout(cu, M, N, K):
    """dW = dyᵀ · x with both operands stored [K_red, rows] (MN-major A and B), fp32 out."""
    torch.manual_seed(3)
    a = torch.randn(K, M, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(K, N, device="cuda", dtype=torch.bfloat16)
    ref = a.float().t() @ b.float()
    out = cu.gemm(a, b, a_mn=True, b_mn=True, out_mode=2)
    _check(out, ref, K)
    acc = torch.ones(M, N, device="cuda")
    cu.gemm(a, b, out=acc, a_mn=True, b_mn=True, out_mode=1)
    _check(acc - 1, ref, K)
    out16 = cu.gemm(a, b, a_mn=True, b_mn=True)
    _check(out16, ref, K)
    cu.check_err_flag()


# (256,256), (384,320), (1000,520): under half a wave of tiles, every tile runs as two half-width units;
# (2304,1280): 45 whole tiles; (4096,4096): 256 tiles, the last 34 of them cut in two; (4096,9472): 592 whole tiles
PAIR_SHAPES = [(256, 256, 64), (384, 320, 192), (1000, 520, 264), (2304, 1280, 328), (4096, 4096, 1024),
               (4096, 9472, 256)]


@pytest.mark.parametrize("M,N,K", PAIR_SHAPES)
def test_gemm_pair_kernel_all_layouts(cu, M, N, K):
    """The CTA-pair kernel (tcgen05.mma.cta_group::2, one 256 x 256 tile per two-CTA cluster) forced on, against
    fp32 matmul: K-major / MN-major operands, bias, fp32 store and fp32 accumulate, ragged edges in M, N and K."""
    torch.manual_seed(M + N + K)
    bf = dict(device="cuda", dtype=torch.bfloat16)
    a, b = torch.randn(M, K, **bf), torch.randn(N, K, **bf)
    bias = torch.randn(N, **bf)
    ref = a.float() @ b.float().t()
    _check(cu.gemm(a, b, pair=True), ref, K)
    _check(cu.gemm(a, b, bias=bias, pair=True), ref + bias.float(), K)
    _check(cu.gemm(a, b, out_mode=2, pair=True), ref, K)
    bt, at = b.t().contiguous(), a.t().contiguous()            # [K, N], [K, M]
    _check(cu.gemm(a, bt, b_mn=True, pair=True), ref, K)
    _check(cu.gemm(at, bt, a_mn=True, b_mn=True, pair=True), ref, K)
    _check(cu.gemm(at, bt, a_mn=True, b_mn=True, out_mode=2, pair=True), ref, K)
    acc = torch.ones(M, N, device="cuda")
    cu.gemm(at, bt, out=acc, a_mn=True, b_mn=True, out_mode=1, pair=True)
    cu.gemm(at, bt, out=acc, a_mn=True, b_mn=True, out_mode=1, pair=True)
    _check(acc - 1, 2 * ref, K)
    torch.cuda.synchronize()
    cu.check_err_flag()
    # and the two kernels agree with each other much more closely than either does with the rounding bound
    one, two = cu.gemm(a, b, out_mode=2, pair=False), cu.gemm(a, b, out_mode=2, pair=True)
    assert (one - two).abs().max().item() <= 1e-4 * (K ** 0.5)
    # whole tiles in the last wave (tail halving off) give the same numbers as the half-width units
    cu.lib().ell_gemm_set_tail_split(0)
    try:
        whole = cu.gemm(a, b, out_mode=2, pair=True)
        whole_t = cu.gemm(at, bt, a_mn=True, b_mn=True, out_mode=2, pair=True)
    finally:
        cu.lib().ell_gemm_set_tail_split(1)
    assert (whole - two).abs().max().item() <= 1e-4 * (K ** 0.5)
    _check(whole_t, ref, K)
    torch.cuda.synchronize()
    cu.check_err_flag()


def test_linear_autograd_matches_torch(cu):
    from easyllm_b200 import ops
    torch.manual_seed(5)
    x = torch.randn(384, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (0.05 * torch.randn(768, 512, device="cuda")).to(torch.bfloat16).requires_grad_()
    b = torch.randn(768, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    dy = torch.randn(384, 768, device="cuda", dtype=torch.bfloat16)
    ops.set_gemm_backend("tcgen05")
    y = ops.linear(x, w, b)
    y.backward(dy)
    xf, wf, bf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_(), b.detach().float().requires_grad_()
    yr = torch.nn.functional.linear(xf, wf, bf)
    yr.backward(dy.float())
    for got, want in ((y, yr), (x.grad, xf.grad), (w.grad, wf.grad), (b.grad, bf.grad)):
        assert (got.float() - want).abs().max().item() <= 3e-2 * max(1.0, want.abs().max().item())
    cu.check_err_flag()


@pytest.mark.parametrize("T,V,K,cut,start", [(256, 512, 256, 0, 0), (300, 1000, 128, 24, 0), (1024, 32000, 512, 0, 0),
                                             (128, 776, 64, 8, 776)])
def test_gemm_ce_epilogue_statistics(cu, T, V, K, cut, start):
    """LM-head GEMM with fused cross-entropy statistics against a plain fp32 log-softmax of the stored logits."""
    torch.manual_seed(T + V)
    x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(V, K, device="cuda") * 0.2).to(torch.bfloat16)
    valid = V - cut
    tgt = torch.randint(start, start + valid, (T,), device="cuda")
    tgt[::7] = start + V + 5                      # targets owned by another vocabulary shard
    logits, parts = cu.gemm_ce(x, w, tgt, start, valid)
    torch.cuda.synchronize()
    cu.check_err_flag()
    want_logits = x.float() @ w.float().t()
    assert (logits.float() - want_logits).abs().max().item() < 2e-2 * max(1.0, want_logits.abs().max().item())
    lf = logits.float()[:, :valid]
    mx = lf.max(1).values
    se = torch.exp(lf - mx[:, None]).sum(1)
    loc = tgt - start
    hit = (loc >= 0) & (loc < valid)
    tl = torch.where(hit, lf.gather(1, loc.clamp(0, valid - 1)[:, None]).squeeze(1), torch.zeros_like(mx))
    torch.testing.assert_close(parts[:, 0], mx, rtol=0, atol=0)
    torch.testing.assert_close(parts[:, 1], se, rtol=2e-3, atol=1e-3)
    torch.testing.assert_close(parts[:, 2], tl, rtol=0, atol=0)
    # and against the stand-alone statistics kernel on the same stored logits
    ref_parts = cu.ce_fwd(logits, tgt, start, valid)
    torch.testing.assert_close(parts, ref_parts, rtol=2e-3, atol=1e-3)


def test_lm_head_ce_autograd_matches_unfused(cu):
    from easyllm_b200 import ops
    torch.manual_seed(5)
    T, V, K = 512, 2048, 256
    x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(V, K, device="cuda") * 0.1).to(torch.bfloat16)
    tgt = torch.randint(0, V, (T,), device="cuda")
    outs = []
    for fused in (True, False):
        xx, ww = x.clone().requires_grad_(), w.clone().requires_grad_()
        if fused:
            loss = ops.lm_head_cross_entropy(xx, ww, tgt)
        else:
            loss = ops.vocab_parallel_cross_entropy(ops.linear(xx, ww), tgt, None, inplace_backward=True)
        loss.mean().backward()
        outs.append((loss.detach(), xx.grad.float(), ww.grad.float()))
    torch.cuda.synchronize()
    cu.check_err_flag()
    torch.testing.assert_close(outs[0][0], outs[1][0], rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(outs[0][1], outs[1][1], rtol=2e-2, atol=1e-5)
    torch.testing.assert_close(outs[0][2], outs[1][2], rtol=2e-2, atol=1e-5)
    ref_loss = torch.nn.functional.cross_entropy(x.float() @ w.float().t(), tgt, reduction="none")
    torch.testing.assert_close(outs[0][0], ref_loss, rtol=2e-2, atol=2e-2)
