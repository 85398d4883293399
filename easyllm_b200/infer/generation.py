"""Text generation and log-prob scoring under TP × PP.

Parity: llm/models/mg_models/base_modules/post_process/text_generation.py:9-182 and
text_generation_utils.py:7-170 (interactive REPL with ``quit`` / ``system`` / ``clean``,
eval loop, temperature / top-k / top-p multinomial or greedy sampling, token broadcast from
the last to the first pipeline stage, done flag over the pipe), and ``infer_logp``
(llm/runners/base_llm_runner.py:367-410).

Difference by design: decoding uses a per-layer KV cache (one-token forwards after the
prompt) instead of recomputing the full prefix for every generated token; ``--recompute``
restores the reference behaviour.
"""
from __future__ import annotations

import json

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..parallel import mappings as mp
from ..parallel.grid import get_grid
from ..utils.log import default_logger as logger


def top_k_logits(logits, top_k=0, top_p=0.0, filter_value=-float("inf")):
    """Mask logits outside the top-k set and outside the smallest set with mass ≥ top_p."""
    if top_k > 0:
        kth = torch.topk(logits, min(top_k, logits.size(-1)))[0][..., -1, None]
        logits = logits.masked_fill(logits < kth, filter_value)
    if top_p > 0.0:
        sorted_logits, idx = torch.sort(logits, descending=True, dim=-1)
        cum = torch.cumsum(F.softmax(sorted_logits, dim=-1), dim=-1)
        remove = cum > top_p
        remove[..., 1:] = remove[..., :-1].clone()
        remove[..., 0] = False
        mask = torch.zeros_like(remove).scatter(-1, idx, remove)
        logits = logits.masked_fill(mask, filter_value)
    return logits


def sample_next(logits, temperature=1.0, top_k=0, top_p=0.0, greedy=False, generator=None):
    if greedy:
        return torch.argmax(logits, dim=-1)
    logits = top_k_logits(logits.float() / max(temperature, 1e-6), top_k, top_p)
    return torch.multinomial(F.softmax(logits, dim=-1), 1, generator=generator).squeeze(-1)


class Generator:
    def __init__(self, engine, tokenizer, seed=1234):
        self.engine, self.model, self.tok = engine, engine.module, tokenizer
        self.g = get_grid()
        self.dev = next(self.model.parameters()).device
        self.rng = torch.Generator(device=self.dev).manual_seed(seed)

    def _logits_last(self, tokens, pos0, use_cache):
        """Pipeline forward of ``tokens [b, s]`` at positions ``pos0 …``; full-vocab logits of the
        last position on the last stage, None elsewhere."""
        b, s = tokens.shape
        pos = (torch.arange(s, device=self.dev) + pos0).unsqueeze(0).expand(b, s)
        out = self.engine.forward_tokens(tokens, pos)
        if out is None:
            return None
        last = out[:, -1, :]
        if self.g.tp > 1 and self.model.parallel_output:
            last = mp.gather_last_dim(last.contiguous())
        return last[:, :self.model.args.unpad_vocab_size or last.shape[-1]]

    @torch.no_grad()
    def generate(self, contexts, max_new_tokens=128, temperature=1.0, top_k=0, top_p=0.0, greedy=False,
                 eos_id=None, recompute=False, stream=False):
        """``contexts``: list of token-id lists (same length or left-padded by the caller to a
        common length).  Returns the full sequences as lists of ids."""
        g = self.g
        eos = self.tok.eos_token_id if eos_id is None else eos_id
        self.model.eval()
        toks = torch.tensor(contexts, dtype=torch.long, device=self.dev)
        b, ctx = toks.shape
        if not recompute:
            self.model.allocate_kv_cache(b, ctx + max_new_tokens)
        done = torch.zeros(b, dtype=torch.bool, device=self.dev)
        try:
            for step in range(max_new_tokens):
                if recompute:
                    logits = self._logits_last(toks, 0, False)
                else:
                    inp = toks if step == 0 else toks[:, -1:]
                    logits = self._logits_last(inp, 0 if step == 0 else toks.shape[1] - 1, True)
                nxt = torch.zeros(b, dtype=torch.long, device=self.dev)
                if logits is not None:
                    nxt = sample_next(logits, temperature, top_k, top_p, greedy, self.rng)
                    if g.tp > 1:                       # identical sampling is not guaranteed across TP ranks
                        dist.broadcast(nxt, g.tp_src_rank(), group=g.tp_group)
                if g.pp > 1:
                    dist.broadcast(nxt, g.last_stage_rank(), group=g.pp_group)
                nxt = torch.where(done, torch.full_like(nxt, eos), nxt)
                toks = torch.cat((toks, nxt.unsqueeze(1)), dim=1)
                done |= nxt == eos
                if stream:
                    yield toks
                if bool(done.all()):
                    break
        finally:
            self.model.free_kv_cache()
        if not stream:
            yield toks

    def generate_once(self, contexts, **kw):
        out = None
        for out in self.generate(contexts, **kw):
            pass
        return out.tolist()

    @torch.no_grad()
    def token_logps(self, tokens, labels):
        """log p(label_t | tokens_≤t) for one sample, from vocab-parallel logits; ignored labels → 0."""
        from ..models.losses import label_logps
        b, s = tokens.shape
        pos = torch.arange(s, device=self.dev).unsqueeze(0).expand(b, s)
        out = self.engine.forward_tokens(tokens, pos)
        res = torch.zeros(b, s, device=self.dev)
        if out is not None:
            lp, _ = label_logps(out, labels)
            res = lp
        if self.g.pp > 1:
            dist.broadcast(res, self.g.last_stage_rank(), group=self.g.pp_group)
        return res


def generate_samples_interactive(args, config, engine, tokenizer, force_eos_id=None, input_fn=input):
    """REPL on (tp 0, first stage); every other rank follows through broadcasts."""
    from ..data.parsers import build_augmentation
    g = get_grid()
    cfg_tok = config["infer_tokenization"]
    tokenization = build_augmentation([cfg_tok], tokenizer).transforms[0]
    tokenization.parser.inference_mode = True
    gen = Generator(engine, tokenizer)
    dev = gen.dev
    history, system_next = [], False
    leader = g.tp_rank == 0 and g.is_first_stage() and g.dp_rank == 0
    while True:
        terminate = cont = 0
        ctx, text = [], ""
        if leader:
            logger.info("Input your questions (quit to exit) >>> ")
            text = input_fn()
            if system_next:
                history.append({"role": "system", "content": text})
                system_next, cont = False, 1
            elif not text.strip():
                logger.info("Input questions must not be empty!")
                cont = 1
            elif text == "quit":
                terminate = 1
            elif text == "system":
                system_next, cont = True, 1
            elif text == "clean":
                logger.info("Clean dialog, the conversation will restart from scratch...")
                history, cont = [], 1
            else:
                parser = tokenization.parser
                if hasattr(parser, "build_inference_meta"):
                    ctx, _ = tokenization(parser.build_inference_meta(text, history))
                else:
                    ctx, _ = tokenization({"text": text, "dialog_history": history})
        info = torch.tensor([terminate, len(ctx), cont], dtype=torch.long, device=dev)
        if dist.is_initialized() and g.world > 1:
            dist.all_reduce(info)
        terminate, n_ctx, cont = (int(x) for x in info)
        if terminate:
            return
        if cont:
            continue
        ctx_t = torch.tensor(ctx if leader else [0] * n_ctx, dtype=torch.long, device=dev)
        if dist.is_initialized() and g.world > 1:
            dist.all_reduce(ctx_t)        # only the leader holds non-zero ids: the sum is a broadcast
        out = gen.generate_once([ctx_t.tolist()], max_new_tokens=args.out_seq_length, temperature=args.temperature,
                                top_k=args.top_k, top_p=args.top_p, greedy=args.greedy, eos_id=force_eos_id,
                                recompute=getattr(args, "recompute", False))
        if leader:
            reply = tokenizer.decode(out[0][n_ctx:], skip_special_tokens=True)
            logger.info(f"\nContext: {text}")
            logger.info(f"\nEasyLLM: {reply}")
            history += [{"role": "user", "content": text}, {"role": "assistant", "content": reply}]


def generate_samples_eval(args, context_tokens, engine, tokenizer, force_eos_id=None, generator=None):
    gen = generator or Generator(engine, tokenizer)
    out = gen.generate_once([context_tokens], max_new_tokens=args.out_seq_length, temperature=args.temperature,
                            top_k=args.top_k, top_p=args.top_p, greedy=args.greedy, eos_id=force_eos_id,
                            recompute=getattr(args, "recompute", False))
    ids = out[0][len(context_tokens):]
    eos = tokenizer.eos_token_id if force_eos_id is None else force_eos_id
    if eos in ids:
        ids = ids[:ids.index(eos)]
    return tokenizer.decode(ids, skip_special_tokens=True)


def infer_logp(engine, tokenizer, data_iter, batch_fn, out_file, num_samples):
    """Per-token label log-probs of every sample → jsonl (offline reference log-probs for DPO).

    One value per input position that holds a real token, i.e. per token of the sample after the first (the
    collator feeds ``ids[:-1]`` and asks for ``ids[1:]``); positions whose label is ignored give 0.  This is the
    ``yw_logp`` / ``yl_logp`` list the ``combine_dpo_general_chat`` parser multiplies with its label mask."""
    g = get_grid()
    gen = Generator(engine, tokenizer)
    pad = len(tokenizer) - 1
    f = open(out_file, "w") if g.rank == 0 else None
    for i in range(num_samples):
        batch = next(data_iter)
        (tokens, _pos, *_), (labels, _mask, *_) = batch_fn(batch)
        lp = gen.token_logps(tokens.to(gen.dev), labels.to(gen.dev))
        if f is not None:
            n_real = int((tokens[0] != pad).sum())          # alignment padding is not part of the sample
            f.write(json.dumps({"id": i, "logp": lp[0][:n_real].tolist()}) + "\n")
    if f is not None:
        f.close()
