"""Headline benchmark: Llama-2-7B 3D-parallel bf16 pre-training throughput (tokens/s).

    python bench.py --gpus 1 --steps 3 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Config (weak scaling): Llama-2-7B shape (32 layers, hidden 4096, 32 heads, FFN 11008, vocab
32000), seq 4096, micro-batch 1, 32 sequences per GPU per step (256 at 8 GPUs), bf16 compute
with fp32 master weights, fused Adam (weight decay 0.1, clip 1.0), ZeRO-1, TP = min(2, N)
with sequence parallelism, DP = N / TP.  Synthetic uniform-random token ids, random-init
weights.  The working set (≥ 13 GB of weights per rank) is far larger than L2, so no flush
is needed between steps.

Two measurements per run, both of K steps after W warm-ups, both bracketed by a barrier and
``torch.cuda.synchronize()`` and timed with CUDA events (max over ranks):
  value — inputs pre-staged on the device, loss left on the device;
  e2e   — ``engine.train_batch`` fed from pinned host memory (H2D copy of every micro-batch)
          and the loss read back to the host every step.

``--impl reference`` is the reference arm: the unmodified reference cannot be imported here
(its modules import a DeepSpeed fork that is not shipped, and apex / peft), so it prints an
``unavailable`` line.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PUBLISHED_TOK_S_GPU = 4304.0   # docs/benchmark.md:10 — 7B, seq 4096, ZeRO-1, 8 x 80 GB GPUs (nearest published row)

MODELS = {
    "llama2_7b": dict(num_layers=32, hidden_size=4096, num_attention_heads=32, num_kv_attention_heads=32,
                      intermediate_size=11008),
    "llama2_13b": dict(num_layers=40, hidden_size=5120, num_attention_heads=40, num_kv_attention_heads=40,
                       intermediate_size=13824),
    "llama2_7b_4l": dict(num_layers=4, hidden_size=4096, num_attention_heads=32, num_kv_attention_heads=32,
                         intermediate_size=11008),
    # BASELINE config shapes beyond the headline: Qwen-14B (QKV bias, 152k vocabulary) and the Llama-2-70B layer
    # shape truncated to 40 layers (GQA 64/8)
    "qwen_14b": dict(num_layers=40, hidden_size=5120, num_attention_heads=40, num_kv_attention_heads=40,
                     intermediate_size=13696, vocab_size=152064,
                     transformer_layer_params={"attention_qkv_bias": True}),
    "llama2_70b_40l": dict(num_layers=40, hidden_size=8192, num_attention_heads=64, num_kv_attention_heads=8,
                           intermediate_size=28672),
    "dev_1b": dict(num_layers=8, hidden_size=2048, num_attention_heads=16, num_kv_attention_heads=16,
                   intermediate_size=5632),
}


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons every 200 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu, self.rows, self.proc = gpu_index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except Exception:
                continue
            for n, v in zip(names, r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def _pair_on(ops):
    """Whether plain GEMMs run on the CTA-pair (tcgen05.mma.cta_group::2) kernel in this run."""
    if ops.get_backend() != "b200" or ops.get_gemm_backend() != "tcgen05":
        return False
    import easyllm_b200.ops.cuda as cu
    return bool(cu._GEMM_PAIR)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama2_7b", choices=sorted(MODELS))
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--seqs-per-gpu", type=int, default=32, help="sequences per GPU per step (weak scaling)")
    ap.add_argument("--tp", type=int, default=0, help="tensor-parallel size (default min(2, gpus))")
    ap.add_argument("--pp", type=int, default=1)
    ap.add_argument("--zero", type=int, default=1)
    ap.add_argument("--gemm", default=None, choices=[None, "tcgen05", "cublas"])
    ap.add_argument("--ops", default=None, choices=[None, "b200", "torch"])
    ap.add_argument("--recompute-layers", type=int, default=0, help="leading layers per stage to recompute")
    ap.add_argument("--dc-map", default="", help="Dynamic Checkpoint size map 'tokens:layers,...': a micro-batch with at "
                    "most that many tokens recomputes that many leading layers per stage (chosen per micro-batch)")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--runner", default="megatron", choices=["megatron", "hf"],
                    help="megatron: 3D-parallel LlamaModelPipe + PipelineEngine; hf: HF-style decoder + ZeRO data-parallel engine")
    ap.add_argument("--varlen", action="store_true",
                    help="packed variable-length documents (lengths uniform in [256, seq]) with cu_seqlens")
    ap.add_argument("--no-fused-tp", action="store_true", help="use the NCCL + GEMM composition for TP linears")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "reference imports a DeepSpeed fork that is not shipped (plus apex/peft, not installed); "
                          "`import llm` fails, and its pip wheel installs no modules"}))
        return 0

    import torch
    import torch.distributed as dist
    from easyllm_b200 import ops
    from easyllm_b200.parallel.grid import initialize_distributed, get_grid
    from easyllm_b200.models import llama_custom
    from easyllm_b200.optim import ZeroOptimizer
    from easyllm_b200.engine import PipelineEngine
    from easyllm_b200.data.synthetic import synthetic_batches
    import easyllm_b200.ops.cuda as cu

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    tp = args.tp or min(2, world)
    if world > 1:
        initialize_distributed(tp=tp, pp=args.pp, backend="nccl", launcher="torch")
    else:
        torch.cuda.set_device(0)
    g = get_grid()
    if args.gemm:
        ops.set_gemm_backend(args.gemm)
    if args.ops:
        ops.set_backend(args.ops)
    # a call that cannot run on the sm_100a kernels raises instead of quietly taking a library path
    ops.set_strict(ops.get_backend() == "b200" and ops.get_gemm_backend() == "tcgen05")
    cu.lib()
    torch.manual_seed(1234 + g.rank)

    shape = dict(MODELS[args.model])
    vocab = shape.pop("vocab_size", 32000)
    dc = None
    if args.recompute_layers:
        dc = {"enabled": True, "size_map": {1 << 30: args.recompute_layers}}
    if args.dc_map:
        dc = {"enabled": True, "size_map": {int(k): int(v) for k, v in (kv.split(":") for kv in args.dc_map.split(","))}}
    if args.runner == "hf":
        if g.tp > 1 or g.pp > 1:
            raise SystemExit("--runner hf is data-parallel only: pass --tp 1 --pp 1")
        from easyllm_b200.models.hf_models import CausalLM, HFArch
        arch = HFArch(family="qwen" if (shape.get("transformer_layer_params") or {}).get("attention_qkv_bias") else "llama",
                      vocab_size=vocab, hidden_size=shape["hidden_size"], intermediate_size=shape["intermediate_size"],
                      num_hidden_layers=shape["num_layers"], num_attention_heads=shape["num_attention_heads"],
                      num_key_value_heads=shape["num_kv_attention_heads"], max_position_embeddings=args.seq,
                      qkv_bias=bool((shape.get("transformer_layer_params") or {}).get("attention_qkv_bias")))
        with torch.device(torch.device("cuda", torch.cuda.current_device())):
            model = CausalLM(arch, dtype=torch.bfloat16).train()
    else:
        model = llama_custom(vocab_size=vocab, seq_length=args.seq, bf16=True, sequence_parallel=g.tp > 1,
                             checkpoint_activations=False, dynamic_checkpoint=dc, pp_partition_method="parameters",
                             **shape)
    fused_tp = False
    if g.tp > 1 and not args.no_fused_tp and ops.get_backend() == "b200":
        from easyllm_b200.parallel import symm
        symm.install(args.seq, shape["hidden_size"])
        fused_tp = True
    opt = ZeroOptimizer(model.named_parameters(), lr=1e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1,
                        stage=args.zero, grad_clip=1.0)
    n_micro = args.seqs_per_gpu * g.tp * g.pp          # per DP rank: global / dp
    global_batch = args.seqs_per_gpu * world
    tokens_per_step = global_batch * args.seq
    dev = torch.device("cuda", torch.cuda.current_device())
    if args.runner == "hf":
        from easyllm_b200.engine.zero_dp import ZeroDPEngine
        dp_eng = ZeroDPEngine(model, opt, None, {"gradient_accumulation_steps": n_micro, "bf16": {"enabled": True}})

        class _HFSteps:
            """One optimizer step of the HF runner's loop (model call, engine.backward, engine.step per micro-batch)."""

            def train_batch(self, it):
                total = None
                for _ in range(n_micro):
                    inp, _ = next(it)
                    tok = inp[0].to(dev, non_blocking=True)
                    pos = inp[1].to(dev, non_blocking=True)
                    cu = inp[3].to(dev, non_blocking=True) if len(inp) > 3 and inp[3] is not None else None
                    # HF convention: the model shifts the labels itself
                    out = model(input_ids=tok, labels=tok, position_ids=pos, cu_seqlens=cu)
                    dp_eng.backward(out["loss"])
                    dp_eng.step()
                    total = out["loss"].detach() if total is None else total + out["loss"].detach()
                return total / n_micro
        eng = _HFSteps()
    else:
        eng = PipelineEngine(model, opt, None, {"train_micro_batch_size_per_gpu": 1,
                                                "gradient_accumulation_steps": n_micro, "bf16": {"enabled": True}})

    host_iter = synthetic_batches(vocab, args.seq, 1, seed=0, pin=True, packed_varlen=args.varlen)

    def device_iter():
        """Micro-batches made on the device: fresh uniform-random token ids for every micro-batch of every step (the
        model never sees a batch twice), labels = ids shifted by one.  Fixed-length batches share one position /
        document layout; ``--varlen`` cycles through 64 packings drawn on the host."""
        from easyllm_b200.models.llama import StageIO
        gen = torch.Generator(device=dev).manual_seed(4321 + g.dp_rank)
        layouts = []
        if args.varlen:
            src = synthetic_batches(vocab, args.seq, 1, seed=1, packed_varlen=True)
            for _ in range(64):
                inp, (_, msk) = next(src)
                layouts.append((inp[1].to(dev), inp[3].to(dev), msk.to(dev), inp[3]))
        else:
            pos = torch.arange(args.seq, dtype=torch.int64, device=dev).unsqueeze(0)
            layouts.append((pos, None, torch.ones(1, args.seq, dtype=torch.int64, device=dev), None))
        parsed = []
        if args.runner != "hf":
            dummy = torch.zeros(1, args.seq, dtype=torch.int64)
            for pos, cu_d, msk, cu_h in layouts:          # parse every layout once, on the host
                io = model.parse_batch((dummy, pos.cpu(), None) + ((cu_h,) if cu_h is not None else ()), device=dev)
                parsed.append(io)
        i = 0
        while True:
            ids = torch.randint(0, vocab, (1, args.seq + 1), generator=gen, device=dev)
            tok, lab = ids[:, :-1], ids[:, 1:]
            pos, cu_d, msk, _ = layouts[i % len(layouts)]
            if args.runner == "hf":
                yield (tok, pos, None, cu_d), (lab, msk)
            else:
                p = parsed[i % len(parsed)]
                io = StageIO(None, p.position_ids, p.cu_seqlens, 1, args.seq, p.max_seqlen, p.max_position,
                             p.row_start, tok.reshape(-1))
                yield io, (lab, msk)
            i += 1

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(it, steps, read_loss):
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        last = None
        for _ in range(steps):
            loss = eng.train_batch(it)
            last = float(loss) if read_loss else loss
        b.record()
        barrier()
        ms = torch.tensor([a.elapsed_time(b)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms), float(last)

    dit = device_iter()
    for _ in range(args.warmup):
        eng.train_batch(dit)
    sampler = ClockSampler(torch.cuda.current_device())
    if g.rank == 0:
        sampler.start()
    l0 = cu.LAUNCHES
    ms, loss = timed(dit, args.steps, read_loss=False)
    launches = cu.LAUNCHES - l0
    clocks = sampler.stop() if g.rank == 0 else None
    cu.check_err_flag()
    value = tokens_per_step * args.steps / (ms / 1e3)

    e2e = None
    if not args.skip_e2e:
        for _ in range(1):
            eng.train_batch(host_iter)
        ms_e, loss_e = timed(host_iter, args.steps, read_loss=True)
        # bytes per step over PCIe: every DP rank copies tokens, positions, labels, mask (int64) per micro-batch
        h2d = 4 * args.seq * 8 * n_micro * g.dp * (g.tp if g.tp > 1 else 1)
        e2e = {"value": tokens_per_step * args.steps / (ms_e / 1e3), "unit": "tokens/s",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * world, "ms_per_step": ms_e / args.steps,
               "loss": loss_e}

    if g.rank == 0:
        out = {"metric": ("tokens/sec, whole job (tokens/sec/GPU in tokens_per_s_per_gpu), "
                          + ("Llama-2-7B" if args.model == "llama2_7b" else args.model) + " 3D-parallel bf16 train"),
               "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
               "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
               "vs_baseline": (value / world) / PUBLISHED_TOK_S_GPU, "dtype": "bf16", "data": "synthetic",
               "tokens_per_s_per_gpu": value / world, "loss": loss, "impl": "ours",
               "config": {"model": args.model, "global_batch": global_batch, "seq_len": args.seq,
                          "parallelism": f"tp{g.tp}pp{g.pp}dp{g.dp}-zero{args.zero}" + ("-sp" if g.tp > 1 else ""),
                          "packing": "variable-length documents, cu_seqlens" if args.varlen else "fixed length",
                          "runner": args.runner,
                          "micro_batch": 1, "grad_accum": n_micro, "optimizer": "fused Adam wd 0.1 clip 1.0",
                          "gemm": ops.get_gemm_backend(), "gemm_cta_pair": _pair_on(ops), "ops": ops.get_backend(), "fused_tp": fused_tp,
                          "recompute_layers": args.recompute_layers, "dynamic_checkpoint_map": args.dc_map or None,
                          "l2": "inputs (weights+activations) far larger than L2; no flush",
                          "vs_baseline_note": "per-GPU tokens/s over the published 4304 tok/s/GPU "
                                              "(7B seq 4096 ZeRO-1 row, other hardware)"},
               "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "kernel_fallbacks": len(ops.fallbacks()),
               "peak_mem_gb": torch.cuda.max_memory_allocated() / 2 ** 30}
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
