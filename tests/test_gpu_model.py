"""Flagship model on the GPU: kernel path vs the PyTorch (library) path on the same weights,
and the smoke entry point."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _need_gpu():
    if not torch.cuda.is_available():
        pytest.skip("no GPU")


def _run(backend, gemm, sd=None):
    from easyllm_b200 import ops
    from easyllm_b200.models import llama_custom
    ops.set_backend(backend)
    ops.set_gemm_backend(gemm)
    torch.manual_seed(0)
    m = llama_custom(num_layers=2, hidden_size=512, num_attention_heads=4, num_kv_attention_heads=2,
                     intermediate_size=1408, vocab_size=32000, bf16=True, seq_length=256,
                     checkpoint_activations=False)
    if sd is not None:
        m.load_state_dict(sd)
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(0, 32000, (2, 256), generator=g).cuda()
    lab = torch.roll(tok, -1, 1)
    loss = m((tok, None, None), (lab, torch.ones_like(lab)))
    loss.backward()
    grads = {n: p.grad.float().clone() for n, p in m.named_parameters()}
    return loss.item(), grads, m.state_dict()


def test_kernel_path_matches_library_path():
    _need_gpu()
    from easyllm_b200 import ops
    try:
        l_ref, g_ref, sd = _run("torch", "cublas")
        l_k, g_k, _ = _run("b200", "tcgen05", sd)
    finally:
        ops.set_backend("b200"); ops.set_gemm_backend("tcgen05")
    assert abs(l_ref - l_k) < 3e-2, (l_ref, l_k)
    for n in g_ref:
        a, b = g_ref[n], g_k[n]
        denom = a.abs().max().item() + 1e-6
        assert (a - b).abs().max().item() / denom < 8e-2, n
    import easyllm_b200.ops.cuda as cu
    cu.check_err_flag()


def test_smoke_entry():
    _need_gpu()
    import __graft_entry__ as ge
    ge.smoke()


def test_hf_style_model_kernel_path_matches_library_path():
    """The generic HF-style decoder (llama / qwen-bias / GQA variants) through the sm_100a kernels vs the PyTorch path."""
    _need_gpu()
    from easyllm_b200 import ops
    from easyllm_b200.models.hf_models import CausalLM, HFArch
    import easyllm_b200.ops.cuda as cu
    for fam, extra in (("llama", {"num_key_value_heads": 2}), ("qwen", {})):
        torch.manual_seed(0)
        a = HFArch(family=fam, vocab_size=2048, hidden_size=512, intermediate_size=1408, num_hidden_layers=2,
                   num_attention_heads=4, qkv_bias=fam == "qwen", **extra)
        m = CausalLM(a, dtype=torch.bfloat16).cuda().train()
        ids = torch.randint(0, 2048, (2, 256), device="cuda")
        res = {}
        try:
            for backend, gemm in (("torch", "cublas"), ("b200", "tcgen05")):
                ops.set_backend(backend); ops.set_gemm_backend(gemm)
                m.zero_grad(set_to_none=True)
                out = m(input_ids=ids, labels=ids)
                out["loss"].backward()
                res[backend] = (float(out["loss"]), {n: p.grad.float().clone() for n, p in m.named_parameters()})
        finally:
            ops.set_backend("b200"); ops.set_gemm_backend("tcgen05")
        torch.cuda.synchronize()
        cu.check_err_flag()
        assert abs(res["torch"][0] - res["b200"][0]) < 3e-2, (fam, res["torch"][0], res["b200"][0])
        for n, g_ref in res["torch"][1].items():
            g_k = res["b200"][1][n]
            assert (g_ref - g_k).abs().max().item() / (g_ref.abs().max().item() + 1e-6) < 8e-2, (fam, n)
        # once the optimizer has moved the parameters into its flat buffer, q/k/v (and gate/up) are adjacent:
        # the fused projection aliases them and the wgrad GEMM accumulates into the adjacent fp32 main_grad views
        from easyllm_b200.optim import ZeroOptimizer
        opt = ZeroOptimizer(m.named_parameters(), lr=1e-4, stage=0)
        att = m.model.layers[0].self_attn if hasattr(m, "model") else None
        if att is not None:
            assert ops._adjacent_alias([att.q_proj.weight.detach(), att.k_proj.weight.detach(),
                                        att.v_proj.weight.detach()]) is not None
            assert ops._adjacent_alias([att.q_proj.weight.main_grad, att.k_proj.weight.main_grad,
                                        att.v_proj.weight.main_grad]) is not None
        opt.zero_grad()
        m(input_ids=ids, labels=ids)["loss"].backward()
        opt.accumulate_grads()
        torch.cuda.synchronize()
        cu.check_err_flag()
        for n, p in m.named_parameters():
            g_ref = res["torch"][1][n]
            assert (g_ref - p.main_grad.float()).abs().max().item() / (g_ref.abs().max().item() + 1e-6) < 8e-2, (fam, n)


def test_train_batch_refuses_a_step_after_a_kernel_gave_up_a_wait():
    """A fused kernel whose bounded wait expired writes the error word and leaves a partial result: the engine
    must raise before the optimizer update instead of training on it.  The word is set by hand here (no wait runs
    out, no kernel misbehaves)."""
    _need_gpu()
    from easyllm_b200.engine import PipelineEngine
    from easyllm_b200.models import llama_custom
    from easyllm_b200.optim import ZeroOptimizer
    from easyllm_b200.data.synthetic import synthetic_batches
    import easyllm_b200.ops.cuda as cu
    torch.manual_seed(0)
    m = llama_custom(num_layers=1, hidden_size=256, num_attention_heads=2, num_kv_attention_heads=2,
                     intermediate_size=512, vocab_size=1024, bf16=True, seq_length=128, checkpoint_activations=False)
    opt = ZeroOptimizer(m.named_parameters(), lr=1e-3, stage=1)
    eng = PipelineEngine(m, opt, None, {"train_micro_batch_size_per_gpu": 1, "gradient_accumulation_steps": 2,
                                        "bf16": {"enabled": True}})
    it = synthetic_batches(1024, 128, 1, seed=0)
    eng.train_batch(it)                                   # a clean step passes
    before = [p.detach().clone() for p in m.parameters()]
    cu.err_flag().fill_(5)                                # what a timed-out peer-flag wait would have written
    with pytest.raises(cu.KernelError):
        eng.train_batch(it)
    for p, q in zip(m.parameters(), before):              # the update was not applied
        assert torch.equal(p.detach(), q)
    opt.zero_grad()
    eng.train_batch(it)                                   # the word was cleared by the read: training goes on
    cu.check_err_flag()


def test_synchronizing_reads_do_not_grow_with_the_number_of_micro_batches():
    """A step may synchronise a few times (the gradient norm, the returned loss), but nothing per micro-batch: the
    batch is parsed on the host and the kernels range-check token ids themselves.  PyTorch's sync debug mode warns on
    every synchronising call; the count inside ``train_batch`` must be the same for 2 and for 6 micro-batches."""
    _need_gpu()
    import warnings
    from easyllm_b200.engine import PipelineEngine
    from easyllm_b200.models import llama_custom
    from easyllm_b200.optim import ZeroOptimizer
    from easyllm_b200.data.synthetic import synthetic_batches
    counts = []
    for accum in (2, 6):
        torch.manual_seed(0)
        m = llama_custom(num_layers=1, hidden_size=256, num_attention_heads=2, num_kv_attention_heads=2,
                         intermediate_size=512, vocab_size=1024, bf16=True, seq_length=128,
                         checkpoint_activations=False)
        opt = ZeroOptimizer(m.named_parameters(), lr=1e-3, stage=1, grad_clip=1.0)
        eng = PipelineEngine(m, opt, None, {"train_micro_batch_size_per_gpu": 1,
                                            "gradient_accumulation_steps": accum, "bf16": {"enabled": True}})
        it = synthetic_batches(1024, 128, 1, seed=0)
        eng.train_batch(it)                               # set-up work of the first step may synchronise
        torch.cuda.synchronize()
        torch.cuda.set_sync_debug_mode("warn")
        try:
            with warnings.catch_warnings(record=True) as seen:
                warnings.simplefilter("always")
                eng.train_batch(it)
        finally:
            torch.cuda.set_sync_debug_mode("default")
        counts.append(sum("synchroniz" in str(w.message).lower() for w in seen))
    assert counts[0] == counts[1], counts
