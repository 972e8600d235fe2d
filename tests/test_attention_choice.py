"""Which attention kernel a step takes (parts/paged_attention.py), decided on the CPU against a stand-in for the
kernels module that only records what was asked of it: decode-only steps by (token, head) pairs and context, mixed
steps split into single tokens (a decode kernel) and portions (a prompt kernel), the cache write fused or not."""
import types

import pytest
import torch

from damendaemon_b200.engine.context import StepContext
from damendaemon_b200.parts import paged_attention as pa


class Recorder:
    """The functions of the kernels module that paged_attention calls; every call is noted, nothing runs."""
    ATTENTION_PREFILL_TCGEN05_KEY_BLOCK = 128

    def __init__(self, head_dims_decode=(64, 128), tcgen05=True, mma=True, pages=True):
        self.calls = []
        self.head_dims_decode, self.tcgen05, self.mma, self.pages = head_dims_decode, tcgen05, mma, pages

    def attention_decode_supported(self, n_heads, kv_heads, head_dim, dtype):
        return dtype == torch.bfloat16 and n_heads == kv_heads and head_dim in self.head_dims_decode

    def attention_decode_pages_supported(self, n_heads, kv_heads, head_dim, page_size, dtype):
        return self.pages and dtype == torch.bfloat16 and n_heads == kv_heads and head_dim == 64

    def attention_prefill_tcgen05_supported(self, n_heads, kv_heads, head_dim, page_size, dtype):
        return self.tcgen05 and dtype == torch.bfloat16 and head_dim == 64

    def attention_prefill_supported(self, n_heads, kv_heads, head_dim, dtype):
        return self.mma and dtype == torch.bfloat16

    def attention_decode_pages_splits(self, n_tokens, n_heads, page_size, context, device):
        return 4

    def attention_decode(self, q, kv, token_entry, positions, table, n_heads, scale, window, n_splits=1, out=None,
                         k_new=None, v_new=None, kernel="rows"):
        self.calls.append(("decode-" + kernel, q.shape[0], token_entry is None, k_new is not None))
        return out if out is not None else q

    def attention_prefill(self, q, kv, entry_start, entry_pos0, table, n_heads, scale, window=None, out=None, kernel="mma",
                          k_new=None, v_new=None, store_new=False):
        self.calls.append(("prefill-" + kernel, entry_pos0.numel(), bool(store_new), table.shape[0]))
        return out if out is not None else q

    def attention_rows(self, q, kv, token_entry, positions, table, n_heads, scale, window=None, n_splits=1, out=None):
        self.calls.append(("rows", q.shape[0], n_splits))
        return q

    def kv_store(self, k, v, token_entry, positions, table, kv):
        self.calls.append(("kv_store", k.shape[0]))


def step(n_single, portions, heads=25, head_dim=64, dtype=torch.bfloat16, context=768, aligned=False, attention="auto",
         writable=True, page=16):
    """A context of n_single single-token entries followed by portions (a list of lengths), and its q, k, v and cache."""
    lengths = [1] * n_single + list(portions)
    n, e = sum(lengths), len(lengths)
    start = torch.tensor([sum(lengths[:i]) for i in range(e + 1)], dtype=torch.int32)
    group = types.SimpleNamespace(name="all")
    runtime = types.SimpleNamespace(attention=attention, attention_tuning=pa.AttentionTuning())
    ctx = StepContext(n_tokens=n, n_entries=e, n_wanted=1, token_ids=torch.zeros(n, dtype=torch.int32),
                      positions=torch.zeros(n, dtype=torch.int32), token_entry=torch.zeros(n, dtype=torch.int32),
                      want_rows=torch.zeros(1, dtype=torch.int32), entry_slot=torch.zeros(e, dtype=torch.int32),
                      entry_start=start, entry_pos0=torch.zeros(e, dtype=torch.int32),
                      block_tables={"all": torch.zeros((e, 64), dtype=torch.int32)}, decode_only=not portions,
                      split_context=context, aligned_starts=aligned, runtime=runtime, n_single=n_single)
    qkv = torch.zeros((n, 3 * heads * head_dim), dtype=dtype)
    q, k, v = qkv.split(heads * head_dim, dim=1)
    cache = types.SimpleNamespace(kv=torch.zeros((4, 2, heads, page, head_dim), dtype=dtype), group=group, writable=writable)
    return ctx, q, k, v, cache


@pytest.fixture
def recorder(monkeypatch):
    r = Recorder()
    monkeypatch.setattr(pa, "kernels", r)
    return r


def run(recorder, *args, **kwargs):
    ctx, q, k, v, cache = step(*args, **kwargs)
    heads = cache.kv.shape[2]
    pa.paged_attention(ctx, q, k, v, cache, heads, 0.125)
    return recorder.calls


def test_decode_steps_by_pairs_and_context(recorder):
    assert run(recorder, 8, [])[-1] == ("decode-pages", 8, True, True)          # 200 pairs: whole pages by TMA
    assert run(recorder, 4, [])[-1] == ("decode-rows", 4, True, True)           # 100 pairs at 768 keys: rows
    assert run(recorder, 1, [], context=16384)[-1][0] == "decode-pages"         # one long request: pages again
    assert run(recorder, 1, [], context=4096)[-1][0] == "decode-rows"
    assert run(recorder, 2, [], context=4096)[-1][0] == "decode-pages"
    assert run(recorder, 8, [], writable=False)[-1] == ("decode-pages", 8, True, False)   # another layer's cache: nothing to write
    assert run(recorder, 8, [], attention="rows")[-1][0] == "rows"              # the general kernel on request
    assert run(recorder, 8, [], dtype=torch.float32)[-1][0] == "rows"           # the float32 path


def test_mixed_steps_are_split(recorder):
    calls = run(recorder, 56, [249] * 8, aligned=True)
    assert calls == [("decode-pages", 56, True, True), ("prefill-tcgen05", 8, True, 8)]      # fused cache write for the portions
    recorder.calls.clear()
    calls = run(recorder, 3, [100, 7])
    assert calls == [("decode-rows", 3, True, True), ("kv_store", 107), ("prefill-tcgen05", 2, False, 2)]
    recorder.calls.clear()
    calls = run(recorder, 0, [128, 128], aligned=True)
    assert calls == [("prefill-tcgen05", 2, True, 2)]
    recorder.calls.clear()
    calls = run(recorder, 5, [64], head_dim=128)                # head size 128: mma.sync prompt kernel, row decode kernel
    assert calls == [("decode-rows", 5, True, True), ("kv_store", 64), ("prefill-mma", 1, False, 1)]


def test_without_a_decode_kernel_the_prompt_kernel_takes_everything(monkeypatch):
    r = Recorder(head_dims_decode=())
    monkeypatch.setattr(pa, "kernels", r)
    ctx, q, k, v, cache = step(6, [128], aligned=True)
    pa.paged_attention(ctx, q, k, v, cache, 25, 0.125)
    # the single tokens may start anywhere, so the prompt kernel may not write the cache itself
    assert r.calls == [("kv_store", 134), ("prefill-tcgen05", 7, False, 7)]


def test_no_tensor_core_prompt_kernel_means_the_general_kernel(monkeypatch):
    r = Recorder(tcgen05=False, mma=False)
    monkeypatch.setattr(pa, "kernels", r)
    ctx, q, k, v, cache = step(2, [40])
    pa.paged_attention(ctx, q, k, v, cache, 25, 0.125)
    assert r.calls == [("kv_store", 42), ("rows", 42, 1)]
