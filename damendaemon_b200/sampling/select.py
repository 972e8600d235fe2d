"""Choose one token per logits row with the CUDA sampling kernels."""
from __future__ import annotations

import torch

from .. import kernels


class NonFiniteLogits(RuntimeError):
    pass


def sample_rows(logits, samplers):
    """logits: float32 [rows, vocab] on the device; samplers: one Sampler per row. Returns a list
    of token ids. Greedy rows take the first maximum; sampled rows consume one draw of their
    sampler's stream. A row without a finite maximum raises (the reference fails closed in the
    same way, damendaemon/sampling.py:136-139)."""
    rows = logits.shape[0]
    if rows != len(samplers) or logits.dim() != 2 or logits.shape[1] == 0:
        raise RuntimeError("invalid sampling logit batch")
    device = logits.device
    options = [s.options for s in samplers]
    if any(o.has_adjustments for o in options):
        logits = logits.clone()
        item_row, item_token, item_count, item_bias, item_seen = [], [], [], [], []
        for r, s in enumerate(samplers):
            for token, count, bias, seen in s.adjustments():
                item_row.append(r); item_token.append(token); item_count.append(count)
                item_bias.append(bias); item_seen.append(seen)
        if item_row:
            f = lambda v, dt: torch.tensor(v, dtype=dt, device=device)
            kernels.adjust_logits(logits, f(item_row, torch.int32), f(item_token, torch.int32),
                                  f(item_count, torch.float32), f(item_bias, torch.float32), f(item_seen, torch.int32),
                                  f([o.repetition_penalty for o in options], torch.float32),
                                  f([o.frequency_penalty for o in options], torch.float32),
                                  f([o.presence_penalty for o in options], torch.float32))
    if all(o.greedy for o in options):
        ids = kernels.sample(logits)
    else:
        temperature = torch.tensor([float(o.temperature) for o in options], dtype=torch.float32, device=device)
        uniform = torch.tensor([s.draw() if not o.greedy else 0.0 for s, o in zip(samplers, options)],
                               dtype=torch.float64, device=device)
        top_k = top_p = None
        if any(o.top_k for o in options):
            top_k = torch.tensor([o.top_k for o in options], dtype=torch.int32, device=device)
        if any(o.top_p < 1 for o in options):
            top_p = torch.tensor([float(o.top_p) for o in options], dtype=torch.float32, device=device)
        ids = kernels.sample(logits, temperature, uniform, top_k, top_p)
    tokens = ids.tolist()
    if any(t < 0 for t in tokens):
        raise NonFiniteLogits("cannot sample non-finite model logits")
    return tokens
