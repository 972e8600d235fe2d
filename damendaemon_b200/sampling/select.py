"""Choose one token per logits row with the CUDA sampling kernels."""
from __future__ import annotations

import torch

from .. import kernels


class NonFiniteLogits(RuntimeError):
    pass


class DeviceStepError(RuntimeError):
    """A kernel of the step whose tokens are being read set an error bit; the tokens are not to be trusted."""


class PendingTokens:
    """Sampled token ids that the host has not read yet: ``ids`` int32 [rows] on the device (what the
    next step can take as its ``device_ids``), and their copy into pinned host memory, in flight.
    The kernels' error word of the device travels in the same pinned buffer, behind the ids, under the
    same event: reading the tokens also tells whether a kernel up to this step reported a missing page,
    a bad token or a wait that ran out, without another synchronisation."""
    __slots__ = ("ids", "host", "event", "rows")

    def __init__(self, ids):
        self.ids = ids
        self.rows = ids.numel()
        self.host = torch.empty(self.rows + 1, dtype=torch.int32, pin_memory=True)
        self.host[:self.rows].copy_(ids.reshape(-1), non_blocking=True)
        self.host[self.rows:].copy_(kernels.error_flag(ids.device), non_blocking=True)
        self.event = torch.cuda.Event()
        self.event.record()


def launch_sample_rows(logits, samplers):
    """logits: float32 [rows, vocab] on the device; samplers: one Sampler per row. Launches the sampling
    kernels and the copy of the ids to the host and returns a PendingTokens without waiting for either.
    Greedy rows take the first maximum; sampled rows consume one draw of their sampler's stream."""
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
    return PendingTokens(ids)


def read_sampled(pending):
    """Wait for the ids of launch_sample_rows (not for anything launched after it) and return them as
    a list. A row without a finite maximum raises (the reference fails closed in the same way,
    damendaemon/sampling.py:136-139); so does an error bit that a kernel of this step, or of one before it
    that nobody has read, left in the device's error word (the word is cleared)."""
    pending.event.synchronize()
    *tokens, bits = pending.host.tolist()
    if bits:
        # in stream order this clears the word after every step launched so far, the one launched ahead included
        kernels.clear_after_error(pending.ids.device, bits)
        raise DeviceStepError(f"a kernel reported error bits {bits:#x} (1 bad token/position, 2 bad page on write, "
                              "4 bad page on read, 8 wait timed out)")
    if any(t < 0 for t in tokens):
        raise NonFiniteLogits("cannot sample non-finite model logits")
    return tokens


def sample_rows(logits, samplers):
    """Sample one token per row and return the ids as a list; see launch_sample_rows and read_sampled,
    which are also reachable as ``sample_rows.launch`` and ``sample_rows.read`` (the scheduler uses
    them to launch the next decode step before it reads this one's tokens)."""
    return read_sampled(launch_sample_rows(logits, samplers))


sample_rows.launch = launch_sample_rows
sample_rows.read = read_sampled
