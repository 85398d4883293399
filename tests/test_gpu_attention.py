"""tcgen05 flash attention (causal, GQA, packed documents) against fp32 exact attention."""
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


CASES = [  # T, Hq, Hk, cu_seqlens
    (128, 2, 2, None), (256, 4, 4, None), (300, 4, 2, None), (1024, 8, 1, None),
    (512, 4, 4, [0, 100, 101, 350, 512]), (777, 2, 1, [0, 128, 256, 640, 777]), (4096, 4, 4, None),
]


@pytest.mark.parametrize("T,Hq,Hk,cu_list", CASES)
def test_flash_fwd(cu, T, Hq, Hk, cu_list):
    from easyllm_b200.ops import reference as ref
    torch.manual_seed(T + Hq)
    W = (Hq + 2 * Hk) * 128
    qkv = torch.randn(T, W, device="cuda", dtype=torch.bfloat16)      # views into a packed buffer
    q = qkv[:, :Hq * 128].view(T, Hq, 128)
    k = qkv[:, Hq * 128:(Hq + Hk) * 128].view(T, Hk, 128)
    v = qkv[:, (Hq + Hk) * 128:].view(T, Hk, 128)
    cs = torch.tensor(cu_list, dtype=torch.int32, device="cuda") if cu_list else None
    rs = cu._row_start(cs, T, q.device)
    scale = 128 ** -0.5
    out, lse = cu.flash_attn_fwd(q, k, v, rs, scale)
    torch.cuda.synchronize()
    cu.check_err_flag()
    want = ref.attention_varlen(q.float(), k.float(), v.float(), cs, True, scale)
    err = (out.float() - want).abs().max().item()
    assert err < 2e-2, err
    # log-sum-exp of the first head against the exact one
    rep = Hq // Hk
    s = torch.einsum("td,sd->ts", q[:, 0].float(), k[:, 0].float()) * scale
    idx = torch.arange(T, device="cuda")
    mask = (idx[None, :] > idx[:, None]) | (idx[None, :] < rs[:, None])
    s = s.masked_fill(mask, float("-inf"))
    assert (torch.logsumexp(s, -1) - lse[0]).abs().max().item() < 2e-2


def test_flash_autograd_path(cu):
    from easyllm_b200 import ops
    from easyllm_b200.ops import reference as ref
    torch.manual_seed(0)
    T, H = 384, 2
    q = torch.randn(T, H, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(T, H, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(T, H, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    ops.set_attention_backend("kernel")
    try:
        o = ops.flash_attention(q, k, v, None, T, True)
        do = torch.randn_like(o)
        o.backward(do)
    finally:
        ops.set_attention_backend("auto")
    qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
    of = ref.attention_varlen(qf, kf, vf, None, True)
    of.backward(do.float())
    for a, b in ((q.grad, qf.grad), (k.grad, kf.grad), (v.grad, vf.grad)):
        assert (a.float() - b).abs().max().item() < 5e-2 * max(1.0, b.abs().max().item())


BWD_CASES = [  # T, Hq, Hk, cu_seqlens
    (128, 1, 1, None), (256, 2, 2, None), (300, 4, 2, None), (1024, 8, 2, None),
    (512, 4, 4, [0, 100, 101, 350, 512]), (777, 2, 1, [0, 128, 256, 640, 777]), (2048, 2, 2, None),
]


@pytest.mark.parametrize("T,Hq,Hk,cu_list", BWD_CASES)
def test_flash_bwd_packed(cu, T, Hq, Hk, cu_list):
    """Backward kernel on views of a packed buffer, gradients written into one packed dQKV."""
    from easyllm_b200.ops import reference as ref
    torch.manual_seed(T * 7 + Hq)
    W = (Hq + 2 * Hk) * 128
    qkv = torch.randn(T, W, device="cuda", dtype=torch.bfloat16)
    q, k, v = cu._split_packed(qkv, Hq, Hk, 128)
    cs = torch.tensor(cu_list, dtype=torch.int32, device="cuda") if cu_list else None
    rs = cu._row_start(cs, T, q.device)
    scale = 128 ** -0.5
    out, lse = cu.flash_attn_fwd(q, k, v, rs, scale)
    do = torch.randn(T, Hq, 128, device="cuda", dtype=torch.bfloat16)
    dqkv = torch.full_like(qkv, float("nan"))
    dq, dk, dv = cu._split_packed(dqkv, Hq, Hk, 128)
    cu.flash_attn_bwd(do, q, k, v, out, lse, rs, scale, dq, dk, dv)
    torch.cuda.synchronize()
    cu.check_err_flag()
    assert torch.isfinite(dqkv.float()).all()
    qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
    of = ref.attention_varlen(qf, kf, vf, cs, True, scale)
    of.backward(do.float())
    for name, a, b in (("dq", dq, qf.grad), ("dk", dk, kf.grad), ("dv", dv, vf.grad)):
        err = (a.float() - b).abs().max().item()
        tol = 3e-2 * max(1.0, b.abs().max().item())
        assert err < tol, (name, err, tol)


def test_flash_packed_autograd_matches_library(cu):
    from easyllm_b200 import ops
    torch.manual_seed(3)
    T, Hq, Hk = 640, 4, 2
    cs = torch.tensor([0, 200, 640], dtype=torch.int32, device="cuda")
    base = torch.randn(T, (Hq + 2 * Hk) * 128, device="cuda", dtype=torch.bfloat16)
    do = torch.randn(T, Hq * 128, device="cuda", dtype=torch.bfloat16)
    grads = {}
    for which in ("kernel", "library"):
        cu.set_attention_backward(which)
        try:
            x = base.clone().requires_grad_()
            o = ops.flash_attention_packed(x, Hq, Hk, 128, cs, 440)
            o.backward(do)
            grads[which] = x.grad.float()
        finally:
            cu.set_attention_backward("kernel")
    torch.cuda.synchronize()
    cu.check_err_flag()
    ref_max = grads["library"].abs().max().item()
    assert (grads["kernel"] - grads["library"]).abs().max().item() < 3e-2 * max(1.0, ref_max)


def test_packed_attention_with_rope_matches_reference(cu):
    """RoPE folded into the packed attention op (in-place rotate, packed un-rotated gradient)."""
    from easyllm_b200 import ops
    from easyllm_b200.ops import reference as ref
    torch.manual_seed(11)
    T, Hq, Hk, D = 384, 4, 2, 128
    cos, sin = ref.rope_tables(D, T, device="cuda")
    pos = torch.arange(T, device="cuda")
    base = torch.randn(T, (Hq + 2 * Hk) * D, device="cuda", dtype=torch.bfloat16)
    do = torch.randn(T, Hq * D, device="cuda", dtype=torch.bfloat16)
    x = base.clone().requires_grad_()
    o = ops.flash_attention_packed(x * 1, Hq, Hk, D, None, T, rope=(cos, sin, pos))
    o.backward(do)
    torch.cuda.synchronize()
    cu.check_err_flag()
    xf = base.float().requires_grad_()
    q = xf[:, :Hq * D].view(T, Hq, D)
    k = xf[:, Hq * D:(Hq + Hk) * D].view(T, Hk, D)
    v = xf[:, (Hq + Hk) * D:].view(T, Hk, D)
    qr, kr = ref.rope(q, k, cos.float(), sin.float(), pos)
    of = ref.attention_varlen(qr, kr, v, None, True).reshape(T, Hq * D)
    of.backward(do.float())
    assert (o.float() - of).abs().max().item() < 3e-2
    assert (x.grad.float() - xf.grad).abs().max().item() < 3e-2 * max(1.0, xf.grad.abs().max().item())


@pytest.mark.parametrize("T,Hq,Hk,D,cu_list", [(384, 4, 4, 128, None), (640, 8, 2, 128, [0, 130, 300, 640]),
                                               (300, 4, 4, 64, None), (512, 4, 2, 64, [0, 100, 512]),
                                               (256, 2, 2, 96, None)])
@pytest.mark.parametrize("alibi", [False, True])
def test_attention_kernel_with_alibi_and_small_heads(cu, T, Hq, Hk, D, cu_list, alibi):
    """ALiBi slopes (the bias slope · (key − query) inside the kernel's softmax, forward and backward) and head
    dimensions below 128 (zero-padded to the kernel's 128 columns), forced onto the kernel path, against the fp32
    statement of the same attention; forward output and all three gradients."""
    from easyllm_b200 import ops
    from easyllm_b200.models.layers import alibi_slopes
    from easyllm_b200.ops import reference as ref
    torch.manual_seed(T + D + Hq)
    q, k, v = (torch.randn(T, h, D, device="cuda", dtype=torch.bfloat16, requires_grad=True) for h in (Hq, Hk, Hk))
    cs = torch.tensor(cu_list, dtype=torch.int32, device="cuda") if cu_list else None
    slopes = torch.tensor(alibi_slopes(Hq), dtype=torch.float32, device="cuda") if alibi else None
    ops.set_attention_backend("kernel")
    ops.set_strict(True)
    try:
        o = ops.flash_attention(q, k, v, cs, T, True, alibi_slopes=slopes)
        do = torch.randn_like(o)
        o.backward(do)
    finally:
        ops.set_attention_backend("auto")
        ops.set_strict(False)
    torch.cuda.synchronize()
    cu.check_err_flag()
    qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
    of = ref.attention_varlen(qf, kf, vf, cs, True, None, slopes)
    of.backward(do.float())
    assert (o.float() - of).abs().max().item() < 2e-2
    for a, b in ((q.grad, qf.grad), (k.grad, kf.grad), (v.grad, vf.grad)):
        assert (a.float() - b).abs().max().item() < 5e-2 * max(1.0, b.abs().max().item())
        assert ((a.float() - b).norm() / b.norm()).item() < 2e-2


def test_attention_dropout_is_rejected_with_the_fused_kernels_and_applied_on_the_eager_path():
    from easyllm_b200.models.config import update_model_cfg
    base = dict(num_layers=1, hidden_size=128, num_attention_heads=2, vocab_size=256, seq_length=32)
    with pytest.raises(ValueError, match="attention_dropout"):
        update_model_cfg(dict(base, transformer_layer_params={"attention_dropout": 0.1}))
    args = update_model_cfg(dict(base, transformer_layer_params={"attention_dropout": 0.1, "use_flash_attn": False}))
    assert args.attention_dropout == 0.1 and not args.use_flash_attn
