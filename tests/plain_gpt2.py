"""A plain, slow GPT-2: whole sequences, no cache, one function per part.

It shares no code with the product path: it reads config.json and model.safetensors
itself and computes with ordinary tensor arithmetic (float64 by default, so that it is
the more exact side of every comparison) on whatever device its weights lie: the CPU
for the small models, a GPU for a model of the benchmark's full size. Each function cites the
reference lines its formula comes from. The reference's own model code was run once
on the CPU against this file (tests/golden/make_golden.py). The two options the
reference rejects (damendaemon/config.py:301-303) are held in other ways: scaling by
inverse layer index against the reference run on weights whose queries carry the
factor (the "Bscaled" case of make_golden.py), the exact-erf gelu against torch's own
function in float64 (tests/test_plain_against_golden.py).
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

_NP = {"F32": np.float32, "F64": np.float64, "F16": np.float16, "I32": np.int32, "I64": np.int64}


def read_folder(folder, dtype=torch.float64):
    """(config dict, {name without 'transformer.': tensor of dtype})."""
    folder = Path(folder)
    config = json.loads((folder / "config.json").read_text())
    raw = (folder / "model.safetensors").read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    tensors = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        b, e = meta["data_offsets"]
        chunk = raw[8 + n + b:8 + n + e]
        if meta["dtype"] == "BF16":
            # bfloat16 is the upper half of a float32
            u16 = np.frombuffer(chunk, dtype=np.uint16).astype(np.uint32) << 16
            arr = u16.view(np.float32)
        else:
            arr = np.frombuffer(chunk, dtype=_NP[meta["dtype"]])
        t = torch.from_numpy(arr.copy()).reshape(meta["shape"])
        tensors[name.removeprefix("transformer.")] = t.to(dtype) if t.is_floating_point() else t
    return config, tensors


def embed(ids, wte, wpe):
    """x[t] = wte[ids[t]] + wpe[t]  (damendaemon/gpt2.py:46; positions are arange, damendaemon/qwen2.py:866)."""
    return wte[ids] + wpe[torch.arange(len(ids), device=wte.device)]


def layer_norm(x, gamma, beta, eps):
    """(x - mean) / sqrt(biased var + eps) * gamma + beta  (damendaemon/starcoder.py:53-55)."""
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * gamma + beta


def conv1d(x, weight_in_out, bias):
    """y = x @ W + b with W stored [in, out]  (damendaemon/gpt2.py:32-37,48)."""
    return x @ weight_in_out + bias


def causal_attention(q, k, v, scale, window=None):
    """softmax(q k^T * scale, keys j <= i [and j > i - window]) v, per head.

    q, k, v: [T, H, d]. Scale d^-0.5 and the causal rule are damendaemon/kernels.py:147,263
    and damendaemon/qwen2.py:769-770; softmax with the maximum subtracted,
    damendaemon/kernels.py:168-178.
    """
    T = q.shape[0]
    scores = torch.einsum("ihd,jhd->hij", q, k) * scale
    i = torch.arange(T, device=q.device)[:, None]
    j = torch.arange(T, device=q.device)[None, :]
    visible = j <= i
    if window is not None:
        visible = visible & (j > i - window)
    scores = scores.masked_fill(~visible, float("-inf"))
    scores = scores - scores.max(-1, keepdim=True).values
    p = torch.exp(scores)
    p = p / p.sum(-1, keepdim=True)
    return torch.einsum("hij,jhd->ihd", p, v)


def gelu_new(u):
    """0.5 u (1 + tanh(sqrt(2/pi) (u + 0.044715 u^3)))  (damendaemon/gpt2.py:63, approximate='tanh')."""
    return 0.5 * u * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (u + 0.044715 * u ** 3)))


def gelu_erf(u):
    """0.5 u (1 + erf(u / sqrt 2)): the exact form, which the reference rejects (damendaemon/config.py:301)."""
    return 0.5 * u * (1.0 + torch.erf(u / math.sqrt(2.0)))


def attention_block(x, w, prefix, n_head, scale):
    """c_attn, split in thirds, heads, attention, c_proj  (damendaemon/gpt2.py:48-61)."""
    T, h = x.shape
    qkv = conv1d(x, w[prefix + "attn.c_attn.weight"], w[prefix + "attn.c_attn.bias"])
    q, k, v = (part.reshape(T, n_head, h // n_head) for part in qkv.split(h, dim=-1))
    o = causal_attention(q, k, v, scale).reshape(T, h)
    return conv1d(o, w[prefix + "attn.c_proj.weight"], w[prefix + "attn.c_proj.bias"])


def mlp_block(x, w, prefix, activation):
    """c_fc, activation, c_proj  (damendaemon/gpt2.py:62-64)."""
    u = conv1d(x, w[prefix + "mlp.c_fc.weight"], w[prefix + "mlp.c_fc.bias"])
    g = gelu_new(u) if activation == "gelu_new" else gelu_erf(u)
    return conv1d(g, w[prefix + "mlp.c_proj.weight"], w[prefix + "mlp.c_proj.bias"])


def logits_of(config, w, ids, rounded=None, rows=None):
    """Logits at every position of one whole sequence, [T, vocab]  (damendaemon/gpt2.py:42-66).

    ``rounded``: a dtype (torch.bfloat16) to which the activations that a reduced-precision engine
    stores between kernels are rounded (norm outputs, q/k/v, attended values, the activated MLP
    hidden); the residual stream and all arithmetic stay wide. It shows how far rounding alone
    moves the logits of a given model, which is what a bfloat16 tolerance has to allow for.
    """
    keep = (lambda t: t) if rounded is None else (lambda t: t.to(rounded).to(t.dtype))
    ids = torch.as_tensor(ids, dtype=torch.long, device=w["wte.weight"].device)
    h, H = config["n_embd"], config["n_head"]
    T = len(ids)
    eps = config.get("layer_norm_epsilon", 1e-5)
    activation = config.get("activation_function", "gelu_new")
    x = embed(ids, w["wte.weight"], w["wpe.weight"])
    for i in range(config["n_layer"]):
        p = f"h.{i}."
        scale = (h // H) ** -0.5
        if config.get("scale_attn_by_inverse_layer_idx", False):
            scale = scale / (i + 1)
        y = keep(layer_norm(x, w[p + "ln_1.weight"], w[p + "ln_1.bias"], eps))
        qkv = keep(conv1d(y, w[p + "attn.c_attn.weight"], w[p + "attn.c_attn.bias"]))
        q, k, v = (part.reshape(T, H, h // H) for part in qkv.split(h, dim=-1))
        o = keep(causal_attention(q, k, v, scale).reshape(T, h))
        x = x + conv1d(o, w[p + "attn.c_proj.weight"], w[p + "attn.c_proj.bias"])
        y = keep(layer_norm(x, w[p + "ln_2.weight"], w[p + "ln_2.bias"], eps))
        u = conv1d(y, w[p + "mlp.c_fc.weight"], w[p + "mlp.c_fc.bias"])
        g = keep(gelu_new(u) if activation == "gelu_new" else gelu_erf(u))
        x = x + conv1d(g, w[p + "mlp.c_proj.weight"], w[p + "mlp.c_proj.bias"])
    if rows is not None:
        x = x[torch.as_tensor(rows, dtype=torch.long, device=x.device)]       # the head only where it is asked for (damendaemon/gpt2.py:65)
    x = keep(layer_norm(x, w["ln_f.weight"], w["ln_f.bias"], eps))
    return x @ w["wte.weight"].t()          # tied head, no bias (damendaemon/gpt2.py:18,66)


class PlainGpt2:
    def __init__(self, folder, dtype=torch.float64):
        self.config, self.w = read_folder(folder, dtype)

    def logits(self, ids, rounded=None, rows=None):
        return logits_of(self.config, self.w, ids, rounded, rows)

    def greedy(self, prompt, n_new):
        ids = list(prompt)
        for _ in range(n_new):
            if len(ids) >= self.config["n_positions"]:
                break
            ids.append(int(self.logits(ids)[-1].argmax()))
        return ids[len(prompt):]


def sample_token(logits_row, temperature, u, top_k=0, top_p=1.0):
    """The engine's sampling rule, restated: greedy = first maximum; else inverse CDF.

    Keep the top_k largest logits (ties with the k-th stay), p = softmax(logits / T) over them,
    keep the most probable tokens until their mass reaches top_p (the crossing token and its
    ties stay), then with c the cumulative sum in token-id order the token is the first index
    whose c exceeds u * c[-1] (the reference draws u from a per-request random.Random and
    searches the normalised CDF, damendaemon/sampling.py:140-177).
    """
    row = torch.as_tensor(logits_row, dtype=torch.float64)
    if not temperature:
        return int(row.argmax())
    keep = torch.ones_like(row, dtype=torch.bool)
    if top_k and top_k < len(row):
        keep &= row >= row.topk(top_k).values[-1]
    e = torch.where(keep, torch.exp((row - row.max()) / temperature), torch.zeros_like(row))
    if top_p < 1:
        order = torch.argsort(row, descending=True, stable=True)
        mass = e[order].cumsum(0)
        crossing = int(torch.searchsorted(mass, torch.tensor(top_p * float(mass[-1]), dtype=torch.float64)))
        keep &= row >= row[order[min(crossing, len(row) - 1)]]
        e = torch.where(keep, e, torch.zeros_like(e))
    c = e.cumsum(0)
    return int(min(torch.searchsorted(c, torch.tensor(u * float(c[-1]), dtype=torch.float64), right=True), len(row) - 1))


def adjust_logits(logits_row, prompt, generated, repetition=1.0, frequency=0.0, presence=0.0, bias=None):
    """Penalties and bias as the reference applies them (damendaemon/sampling.py:86-104): divide or
    multiply the logits of seen tokens by the repetition penalty, subtract count * frequency +
    presence for generated tokens, add the bias."""
    row = torch.as_tensor(logits_row, dtype=torch.float64).clone()
    from collections import Counter
    counts = Counter(generated)
    if repetition != 1:
        for t in set(prompt) | set(counts):
            row[t] = row[t] / repetition if row[t] > 0 else row[t] * repetition
    for t, n in counts.items():
        row[t] -= n * frequency + presence
    for t, b in (bias or {}).items():
        row[t] += b
    return row
