"""Paged causal attention of a step's tokens: the cache write and the choice of kernel.

Five kernels can serve (csrc/attention_*.cu): the general one (any sizes, both dtypes: the float32 path, the
fallback and the reference of the others), two bfloat16 decode kernels (rows by cp.async; whole pages of a group of
heads by TMA) and two bfloat16 prompt kernels (mma.sync; tcgen05). Which one a step takes depends on the step
(decode only or not, how many (token, head) pairs), on what each kernel supports (head size, page size, groups) and
on thresholds that were measured, which are data: ``AttentionTuning``, a field of the runtime, not constants of a
model. A mixer calls ``paged_attention`` through ``ctx.attend``.
"""
from __future__ import annotations

from dataclasses import dataclass

from .. import kernels


@dataclass(frozen=True)
class AttentionTuning:
    """Thresholds of the kernel choice. The defaults were measured on a B200 with 25 heads of 64 and 768 keys per
    request: the page-streaming decode kernel wins from 8 requests on (11.6 against 14.0 us; 54 against 68 us at 64
    requests) and loses at 4 and below (11.0 against 9.8 us; 9.1 against 5.5 us at one request)."""
    pages_from_pairs: int = 150           # decode steps with at least this many (token, head) pairs stream whole pages
    pages_per_block: int = 128            # a block of the page-streaming kernel holds the ids of this many pages
    row_keys_per_block: int = 128         # key split of the row decode kernel: keys per block ...
    row_blocks_per_sm: int = 2            # ... and blocks wanted per SM


def prompt_key_block(n_heads, kv_heads, head_dim, page_size, dtype):
    """Where the tcgen05 prompt kernel likes prompts to be cut, or 1 if it does not take these sizes: a portion that
    starts on a key block lets the kernel write the cache itself and read whole blocks."""
    if kernels.attention_prefill_tcgen05_supported(n_heads, kv_heads, head_dim, page_size, dtype):
        return kernels.ATTENTION_PREFILL_TCGEN05_KEY_BLOCK
    return 1


def paged_attention(ctx, q, k, v, cache, n_heads, scale, window=None):
    runtime = ctx.runtime
    tune = runtime.attention_tuning
    if not (q.stride(0) == k.stride(0) == v.stride(0)) or q.stride(1) != 1 or k.stride(1) != 1 or v.stride(1) != 1:
        # the kernels read q, k and v as row views of one buffer (what a fused projection leaves); a part that made
        # new tensors of some of them (a position encoding that does not rotate in place) gets them packed again
        import torch
        widths = (q.shape[1], k.shape[1], v.shape[1])
        q, k, v = torch.cat([q, k, v], dim=1).split(widths, dim=1)
    kv, table = cache.kv, ctx.block_table(cache.group)
    kv_heads, page_size, head_dim = kv.shape[2], kv.shape[3], kv.shape[4]
    k_new, v_new = (k, v) if cache.writable else (None, None)
    fast = runtime.attention != "rows"
    tensor = fast and runtime.attention != "mma"
    if ctx.decode_only and tensor and ctx.n_tokens * n_heads >= tune.pages_from_pairs and \
            kernels.attention_decode_pages_supported(n_heads, kv_heads, head_dim, page_size, q.dtype):
        # whole pages of a group of heads by TMA; it takes the new keys and values from the projection and writes them
        splits = kernels.attention_decode_pages_splits(ctx.n_tokens, n_heads, page_size, ctx.split_context, q.device)
        splits = max(splits, -(-table.shape[1] // tune.pages_per_block))
        # (decode only: token t is entry t, so the kernels are spared the look-up)
        return kernels.attention_decode(q, kv, None, ctx.positions, table, n_heads, scale, window,
                                        n_splits=splits, k_new=k_new, v_new=v_new, kernel="pages")
    if ctx.decode_only and fast and kernels.attention_decode_supported(n_heads, kv_heads, head_dim, q.dtype):
        # the decode kernel takes the new keys and values from the projection and writes them itself
        splits = ctx.key_splits(n_heads, keys_per_block=tune.row_keys_per_block, blocks_per_sm=tune.row_blocks_per_sm)
        return kernels.attention_decode(q, kv, None, ctx.positions, table, n_heads, scale, window,
                                        n_splits=splits, k_new=k_new, v_new=v_new)
    tcgen05 = not ctx.decode_only and tensor and \
        kernels.attention_prefill_tcgen05_supported(n_heads, kv_heads, head_dim, page_size, q.dtype)
    # the tcgen05 prompt kernel writes the cache itself when no key block mixes cached and new keys
    fused_store = tcgen05 and cache.writable and ctx.aligned_starts
    if cache.writable and not fused_store:
        kernels.kv_store(k, v, ctx.token_entry, ctx.positions, table, kv)
    if tcgen05:
        return kernels.attention_prefill(q, kv, ctx.entry_start, ctx.entry_pos0, table, n_heads, scale, window,
                                         kernel="tcgen05", k_new=k_new, v_new=v_new, store_new=fused_store)
    if not ctx.decode_only and fast and kernels.attention_prefill_supported(n_heads, kv_heads, head_dim, q.dtype):
        return kernels.attention_prefill(q, kv, ctx.entry_start, ctx.entry_pos0, table, n_heads, scale, window)
    return kernels.attention_rows(q, kv, ctx.token_entry, ctx.positions, table, n_heads, scale, window,
                                  n_splits=ctx.key_splits(n_heads))
