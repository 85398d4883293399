"""Adam with 8-bit optimizer state (block-wise quantisation).

The reference's optimizer builder offers bitsandbytes ``Adam8bit`` (llm/utils/model/optimizer_helper.py:70-98) for
the single-axis runners; this is a self-contained PyTorch version of the same idea: both moments are kept as one
byte per element plus one fp32 scale per block of ``block_size`` elements, and are de-quantised, updated and
re-quantised block by block on every step.

* first moment  — signed, quantised on a square-root grid: ``q = round(127 · sign(m) · sqrt(|m| / absmax))``,
  so small entries keep relative precision;
* second moment — non-negative, quantised on a fourth-root grid ``q = round(255 · (v / max) ** 0.25)``, which gives
  the update's denominator ``sqrt(v)`` the same square-root spacing.

Tensors smaller than ``min_8bit_size`` keep fp32 state (as bitsandbytes does).  Parameters are updated in fp32 and
written back in their own dtype; ``weight_decay`` is decoupled when ``adamw`` is set.
"""
from __future__ import annotations

import torch
from torch.optim.optimizer import Optimizer


def _blocks(t, block):
    flat = t.reshape(-1)
    pad = (-flat.numel()) % block
    if pad:
        flat = torch.cat((flat, flat.new_zeros(pad)))
    return flat.view(-1, block)


def quantize_signed(x, block):
    b = _blocks(x.float(), block)
    scale = b.abs().amax(dim=1, keepdim=True).clamp_min(1e-30)
    q = torch.round(127.0 * torch.sign(b) * torch.sqrt(b.abs() / scale)).to(torch.int8)
    return q, scale


def dequantize_signed(q, scale, numel, shape):
    f = q.float() / 127.0
    return (torch.sign(f) * f * f * scale).reshape(-1)[:numel].view(shape)


def quantize_unsigned(x, block):
    b = _blocks(x.float(), block)
    scale = b.amax(dim=1, keepdim=True).clamp_min(1e-30)
    q = torch.round(255.0 * (b / scale) ** 0.25).to(torch.uint8)
    return q, scale


def dequantize_unsigned(q, scale, numel, shape):
    f = q.float() / 255.0
    return ((f * f) ** 2 * scale).reshape(-1)[:numel].view(shape)


class Adam8bit(Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, adamw=False,
                 block_size=2048, min_8bit_size=4096, **_):
        if lr < 0 or not 0 <= betas[0] < 1 or not 0 <= betas[1] < 1:
            raise ValueError("invalid Adam8bit hyper-parameters")
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, adamw=adamw))
        self.block_size, self.min_8bit_size = int(block_size), int(min_8bit_size)

    def state_bytes(self):
        """Bytes held by the optimizer state (for reports and tests)."""
        n = 0
        for st in self.state.values():
            n += sum(v.numel() * v.element_size() for v in st.values() if torch.is_tensor(v))
        return n

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        blk = self.block_size
        for group in self.param_groups:
            b1, b2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                g = p.grad.float()
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["eight_bit"] = p.numel() >= self.min_8bit_size
                    if st["eight_bit"]:
                        st["m_q"], st["m_s"] = quantize_signed(torch.zeros_like(g), blk)
                        st["v_q"], st["v_s"] = quantize_unsigned(torch.zeros_like(g), blk)
                    else:
                        st["m"], st["v"] = torch.zeros_like(g), torch.zeros_like(g)
                st["step"] += 1
                t = st["step"]
                w = p.float()
                if group["weight_decay"] and not group["adamw"]:
                    g = g + group["weight_decay"] * w
                if st["eight_bit"]:
                    m = dequantize_signed(st["m_q"], st["m_s"], g.numel(), g.shape)
                    v = dequantize_unsigned(st["v_q"], st["v_s"], g.numel(), g.shape)
                else:
                    m, v = st["m"], st["v"]
                m = m.mul(b1).add_(g, alpha=1 - b1)
                v = v.mul(b2).addcmul_(g, g, value=1 - b2)
                if st["eight_bit"]:
                    st["m_q"], st["m_s"] = quantize_signed(m, blk)
                    st["v_q"], st["v_s"] = quantize_unsigned(v, blk)
                else:
                    st["m"], st["v"] = m, v
                c1, c2 = 1 - b1 ** t, 1 - b2 ** t
                if group["weight_decay"] and group["adamw"]:
                    w = w * (1 - group["lr"] * group["weight_decay"])
                w = w - group["lr"] / c1 * m / ((v / c2).sqrt() + group["eps"])
                p.copy_(w.to(p.dtype))
        return loss
