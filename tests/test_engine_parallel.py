"""Tiny Llama, fp32, CPU/gloo: DP=2, PP=2, TP=2(+SP) and ZeRO stages must reproduce the
single-process loss trajectory (4 steps, seq 128, micro-batch 2, Adam lr 1e-4)."""
import pytest
import torch

from dist_utils import run_ranks

TINY = dict(num_layers=2, hidden_size=256, num_attention_heads=4, intermediate_size=688, vocab_size=32000,
            layer_norm_params={"kwargs": {"eps": 1e-5}}, checkpoint_activations=False)
STEPS, SEQ, MBS, GBS = 4, 128, 2, 4


def _full_state(seed=0):
    """Reference weights built without any grid (TP=1) so every layout can slice them."""
    from easyllm_b200.models import llama_custom
    torch.manual_seed(seed)
    return llama_custom(**TINY).state_dict()


def _load_sliced(model, full):
    from easyllm_b200.parallel.grid import get_grid
    g = get_grid()
    sd = {}
    for k, v in model.state_dict().items():
        f = full[k]
        if v.shape != f.shape:
            dim = 0 if v.shape[0] != f.shape[0] else 1
            n = v.shape[dim]
            f = f.narrow(dim, g.tp_rank * n, n)
        sd[k] = f.clone()
    model.load_state_dict(sd)


def _train(rank, world, tp, pp, stage, sp, full, recompute=False, bucket_numel=1 << 27, clip=0.0, probe=None):
    from easyllm_b200.parallel.grid import initialize_model_parallel
    from easyllm_b200.models import llama_custom
    from easyllm_b200.optim import ZeroOptimizer
    from easyllm_b200.engine import PipelineEngine
    from easyllm_b200.data.synthetic import synthetic_batches
    g = initialize_model_parallel(tp, pp) if world > 1 else None
    from easyllm_b200.parallel.grid import get_grid
    g = get_grid()
    cfg = dict(TINY, sequence_parallel=sp, checkpoint_activations=recompute)
    model = llama_custom(**cfg)
    _load_sliced(model, full)
    opt = ZeroOptimizer(model.named_parameters(), lr=1e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0,
                        adamw=False, stage=stage, grad_clip=clip, bucket_numel=bucket_numel)
    eng = PipelineEngine(model, opt, None, {"train_micro_batch_size_per_gpu": MBS,
                                            "gradient_accumulation_steps": GBS // (MBS * g.dp)})
    it = synthetic_batches(32000, SEQ, MBS, seed=0)
    losses = [float(eng.train_batch(it)) for _ in range(STEPS)]
    if probe == "zero2":
        return losses, float(eng.get_global_grad_norm()), len(opt._buckets), opt.grad_buf is None, \
            not any(hasattr(p, "main_grad") for p in model.parameters()), opt._n_bufs
    if probe == "norm":
        return losses, float(eng.get_global_grad_norm())
    return losses


def _single(full):
    return _train(0, 1, 1, 1, 0, False, full)


@pytest.fixture(scope="module")
def baseline():
    full = _full_state()
    return full, _single(full)


def test_single_process_loss_is_sane(baseline):
    _, losses = baseline   # uniform random tokens: the loss sits near ln(32000) = 10.37
    assert all(abs(l - 10.4) < 0.3 for l in losses) and len(set(losses)) == STEPS


@pytest.mark.parametrize("tp,pp,stage,sp", [(1, 1, 0, False), (1, 1, 1, False), (1, 1, 2, False),
                                            (1, 2, 0, False), (2, 1, 0, False), (2, 1, 1, True)])
def test_two_ranks_match_single(baseline, tp, pp, stage, sp):
    full, ref = baseline
    outs = run_ranks(2, _train, tp, pp, stage, sp, full)
    for losses in outs:
        assert max(abs(a - b) for a, b in zip(losses, ref)) < 2e-5, (losses, ref)


def test_zero2_partitions_gradients_and_reduces_in_buckets(baseline):
    """ZeRO-2 over two DP ranks: no full gradient buffer and no ``main_grad`` views exist, the gradients travel in
    several buckets that are reduced from autograd hooks (a pool of at most three buffers), and losses, clipping
    and the global gradient norm match the single-process run; also with activation recompute."""
    full, _ = baseline
    ref_losses, ref_norm = _train(0, 1, 1, 1, 0, False, full, clip=0.3, probe="norm")
    for recompute in (False, True):
        outs = run_ranks(2, _train, 1, 1, 2, False, full, recompute, 200_000, 0.3, "zero2")
        for losses, norm, n_buckets, no_grad_buf, no_main_grad, n_bufs in outs:
            assert max(abs(a - b) for a, b in zip(losses, ref_losses)) < 2e-5, (losses, ref_losses)
            assert abs(norm - ref_norm) < 1e-4 * max(1.0, ref_norm)
            assert n_buckets >= 4 and no_grad_buf and no_main_grad and n_bufs <= 3


def test_zero2_with_tensor_and_sequence_parallelism(baseline):
    """tp2 x dp2, sequence parallel, ZeRO-2: the gradients of TP-replicated norm weights are summed over TP inside
    their bucket before the DP reduction."""
    full, ref = baseline
    outs = run_ranks(4, _train, 2, 1, 2, True, full, False, 200_000)
    for losses in outs:
        assert max(abs(a - b) for a, b in zip(losses, ref)) < 2e-5, (losses, ref)


def test_four_ranks_tp2_pp2_recompute(baseline):
    full, ref = baseline
    outs = run_ranks(4, _train, 2, 2, 0, True, full, True)
    for losses in outs:
        assert max(abs(a - b) for a, b in zip(losses, ref)) < 2e-5, (losses, ref)


def _train_adapter(rank, world, tp, pp, sp, full, native):
    """Adam with clipping at 0.5: natively on one process, or torch.optim.Adam through the adapter on a layout."""
    from easyllm_b200.parallel.grid import get_grid, initialize_model_parallel
    from easyllm_b200.models import llama_custom
    from easyllm_b200.optim import ZeroOptimizer
    from easyllm_b200.optim.torch_adapter import TorchOptimizerAdapter
    from easyllm_b200.engine import PipelineEngine
    from easyllm_b200.data.synthetic import synthetic_batches
    if world > 1:
        initialize_model_parallel(tp, pp)
    g = get_grid()
    model = llama_custom(**dict(TINY, sequence_parallel=sp))
    _load_sliced(model, full)
    if native:
        opt = ZeroOptimizer(model.named_parameters(), lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0,
                            adamw=False, stage=0, grad_clip=0.5)
    else:
        inner = torch.optim.Adam([p for p in model.parameters() if p.requires_grad], lr=1e-3, betas=(0.9, 0.999), eps=1e-8)
        opt = TorchOptimizerAdapter(inner, model.named_parameters(), grad_clip=0.5)
    eng = PipelineEngine(model, opt, None, {"train_micro_batch_size_per_gpu": MBS,
                                            "gradient_accumulation_steps": GBS // (MBS * g.dp)})
    it = synthetic_batches(32000, SEQ, MBS, seed=0)
    losses = [float(eng.train_batch(it)) for _ in range(3)]
    return losses, eng.get_global_grad_norm()


def test_optimizer_adapter_matches_the_native_path_on_every_layout(baseline):
    """The adapter's gradient plumbing (fp32 accumulation, DP averaging, TP sum of sequence-parallel norm weights,
    global norm with replicated parameters counted once, clipping) reproduces the native optimizer's trajectory."""
    full, _ = baseline
    ref_losses, ref_norm = _train_adapter(0, 1, 1, 1, False, full, True)
    one_losses, one_norm = _train_adapter(0, 1, 1, 1, False, full, False)
    assert max(abs(a - b) for a, b in zip(one_losses, ref_losses)) < 2e-5 and abs(one_norm - ref_norm) < 1e-4 * ref_norm
    for tp, pp, sp in ((2, 1, True), (1, 2, False), (1, 1, False)):
        for losses, norm in run_ranks(2, _train_adapter, tp, pp, sp, full, False):
            assert max(abs(a - b) for a, b in zip(losses, ref_losses)) < 5e-5, (tp, pp, sp, losses, ref_losses)
            assert abs(norm - ref_norm) < 1e-3 * ref_norm, (tp, pp, sp, norm, ref_norm)



def _packed_batches(seq, dp_rank, dp_size, min_len=16):
    """Micro-batches of one packed sequence each; tokens AND document layout are functions of the global sample
    index, so every parallel layout trains on the same stream (sample i goes to DP rank i mod dp)."""
    from easyllm_b200.data.synthetic import SyntheticTokenDataset
    ds = SyntheticTokenDataset(32000, seq, seed=0)
    step = 0
    while True:
        idx = step * dp_size + dp_rank
        step += 1
        row = ds[idx]
        gen = torch.Generator().manual_seed(1000 + idx)
        cu, at = [0], 0
        pos = torch.empty(1, seq, dtype=torch.int64)
        mask = torch.ones(1, seq, dtype=torch.int64)
        while at < seq:
            n = min(int(torch.randint(min_len, seq + 1, (1,), generator=gen)), seq - at)
            pos[0, at:at + n] = torch.arange(n)
            mask[0, at + n - 1] = 0
            at += n
            cu.append(at)
        yield (row["input_ids"][None], pos, None, torch.tensor(cu, dtype=torch.int32)), (row["labels"][None], mask)


def _train_packed(rank, world, tp, stage, sp, full, size_map):
    """ZeRO stage `stage`, packed variable-length documents, Dynamic Checkpoint chosen from each micro-batch's tokens."""
    from easyllm_b200.parallel.grid import get_grid, initialize_model_parallel
    from easyllm_b200.models import llama_custom
    from easyllm_b200.optim import ZeroOptimizer
    from easyllm_b200.engine import PipelineEngine
    if world > 1:
        initialize_model_parallel(tp, 1)
    g = get_grid()
    dc = {"enabled": True, "size_map": size_map} if size_map else None
    model = llama_custom(**dict(TINY, sequence_parallel=sp, dynamic_checkpoint=dc))
    _load_sliced(model, full)
    opt = ZeroOptimizer(model.named_parameters(), lr=1e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0,
                        adamw=False, stage=stage, grad_clip=0.5, bucket_numel=200_000)
    eng = PipelineEngine(model, opt, None, {"train_micro_batch_size_per_gpu": 1,
                                            "gradient_accumulation_steps": 4 // g.dp})
    it = _packed_batches(SEQ, g.dp_rank, g.dp)
    losses = [float(eng.train_batch(it)) for _ in range(3)]
    plan = model.recompute_plan(SEQ) if size_map else None      # what a micro-batch of SEQ tokens recomputes
    return losses, float(eng.get_global_grad_norm()), plan


def test_packed_documents_zero2_tp_sp_and_dynamic_checkpoint_match_single_process(baseline):
    """The ingredients of the Qwen-14B benchmark config in miniature (tp2 x dp2, sequence parallel, ZeRO-2, packed
    variable-length documents with cu_seqlens, recompute chosen per micro-batch from its token count): losses and the
    gradient norm match one process that trains on the same stream without recompute."""
    full, _ = baseline
    ref_losses, ref_norm, _ = _train_packed(0, 1, 1, 0, False, full, None)
    assert len(set(ref_losses)) == 3
    for losses, norm, plan in run_ranks(4, _train_packed, 2, 2, True, full, {64: 0, 128: 1}):
        assert max(abs(a - b) for a, b in zip(losses, ref_losses)) < 3e-5, (losses, ref_losses)
        assert abs(norm - ref_norm) < 2e-4 * max(1.0, ref_norm)
        assert plan == [True, False]                 # 128 tokens: the first of the two layers is recomputed


def _alternating_batches(dp_rank, dp_size):
    """Micro-batches whose token count changes from one to the next (128, 64, 128, ...)."""
    from easyllm_b200.data.synthetic import SyntheticTokenDataset
    ds = SyntheticTokenDataset(32000, SEQ, seed=0)
    step = 0
    while True:
        idx = step * dp_size + dp_rank
        n = SEQ if idx % 2 == 0 else SEQ // 2
        step += 1
        row = ds[idx]
        pos = torch.arange(n, dtype=torch.int64)[None]
        yield (row["input_ids"][None, :n], pos, None), (row["labels"][None, :n], torch.ones(1, n, dtype=torch.int64))


def _train_alternating(rank, world, tp, pp, sp, full, dynamic):
    from easyllm_b200.parallel.grid import get_grid, initialize_model_parallel
    from easyllm_b200.models import llama_custom
    from easyllm_b200.optim import ZeroOptimizer
    from easyllm_b200.engine import PipelineEngine
    if world > 1:
        initialize_model_parallel(tp, pp)
    g = get_grid()
    model = llama_custom(**dict(TINY, sequence_parallel=sp))
    _load_sliced(model, full)
    opt = ZeroOptimizer(model.named_parameters(), lr=1e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0,
                        adamw=False, stage=0)
    eng = PipelineEngine(model, opt, None, {"train_micro_batch_size_per_gpu": 1, "gradient_accumulation_steps": 4 // g.dp})
    it = _alternating_batches(g.dp_rank, g.dp)
    return [float(eng.train_batch(it, dynamic=dynamic)) for _ in range(3)]


def test_pipeline_links_follow_micro_batches_of_changing_length(baseline):
    """1F1B over two stages with micro-batches of 128 and 64 tokens in turn: the shape header that travels with every
    activation (dynamic mode) keeps the stages in step, with and without tensor + sequence parallelism inside a
    stage; the losses are those of one process on the same stream."""
    full, _ = baseline
    ref = _train_alternating(0, 1, 1, 1, False, full, True)
    for losses in run_ranks(2, _train_alternating, 1, 2, False, full, True):
        assert max(abs(a - b) for a, b in zip(losses, ref)) < 2e-5, (losses, ref)
    for losses in run_ranks(4, _train_alternating, 2, 2, True, full, True):
        assert max(abs(a - b) for a, b in zip(losses, ref)) < 3e-5, (losses, ref)
