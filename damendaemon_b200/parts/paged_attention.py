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
    pages_from_pairs: int = 150           # decode steps with at least this many (token, head) pairs stream whole pages,
    pages_from_pair_keys: int = 200_000   # ... or with this many pairs x keys of context (one request of 16,384 keys:
                                          # 36 us in pages, 45 us in rows; two of 4,096: 25 us either way; one: 22 / 15)
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
    def wants_pages(n_tokens):
        pairs = n_tokens * n_heads
        return pairs >= tune.pages_from_pairs or pairs * ctx.split_context >= tune.pages_from_pair_keys
    if ctx.decode_only and tensor and wants_pages(ctx.n_tokens) and \
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
    mma = not tcgen05 and not ctx.decode_only and fast and kernels.attention_prefill_supported(n_heads, kv_heads, head_dim, q.dtype)
    # A step that mixes portions with single tokens: the single tokens come first (ctx.n_single) and go to a decode
    # kernel, the portions to a prompt kernel. A prompt kernel spends a tile of 64 or 128 query rows and a walk over all
    # key blocks on a single token (measured with 56 decoding requests beside 8 portions of 249 tokens, 36 layers:
    # 8.3 ms a step through the prompt kernel alone, against 4.5 ms for 2,048 prompt tokens).
    n1 = ctx.n_single if (tcgen05 or mma) and fast and kernels.attention_decode_supported(n_heads, kv_heads, head_dim, q.dtype) else 0
    out = None
    if n1:
        import torch
        out = torch.empty((q.shape[0], n_heads * head_dim), dtype=q.dtype, device=q.device)
        pages = tensor and wants_pages(n1) and \
            kernels.attention_decode_pages_supported(n_heads, kv_heads, head_dim, page_size, q.dtype)
        if pages:
            splits = kernels.attention_decode_pages_splits(n1, n_heads, page_size, ctx.split_context, q.device)
            splits = max(splits, -(-table.shape[1] // tune.pages_per_block))
        else:
            splits = ctx.key_splits(n_heads, keys_per_block=tune.row_keys_per_block, blocks_per_sm=tune.row_blocks_per_sm,
                                    n_tokens=n1)
        kernels.attention_decode(q[:n1], kv, None, ctx.positions[:n1], table, n_heads, scale, window, n_splits=splits,
                                 out=out[:n1], k_new=None if k_new is None else k_new[:n1],
                                 v_new=None if v_new is None else v_new[:n1], kernel="pages" if pages else "rows")
        if n1 == ctx.n_entries:
            return out
    # the tcgen05 prompt kernel writes the cache itself when no key block of its entries mixes cached and new keys
    fused_store = tcgen05 and cache.writable and ctx.aligned_starts and n1 == ctx.n_single
    if cache.writable and not fused_store:
        kernels.kv_store(k[n1:], v[n1:], ctx.token_entry[n1:], ctx.positions[n1:], table, kv)
    if tcgen05:
        return kernels.attention_prefill(q, kv, ctx.entry_start[n1:], ctx.entry_pos0[n1:], table[n1:], n_heads, scale, window,
                                         out=out, kernel="tcgen05", k_new=k_new, v_new=v_new, store_new=fused_store)
    if mma:
        return kernels.attention_prefill(q, kv, ctx.entry_start[n1:], ctx.entry_pos0[n1:], table[n1:], n_heads, scale, window,
                                         out=out)
    return kernels.attention_rows(q, kv, ctx.token_entry, ctx.positions, table, n_heads, scale, window,
                                  n_splits=ctx.key_splits(n_heads))
