"""The description of one step as the kernels see it: flattened tokens with per-token
position and entry, per-entry bookkeeping, the rows whose logits are wanted, and the
block tables of the entries, all int32 on the device (one host-to-device copy a step)."""
from __future__ import annotations

from dataclasses import dataclass, field

from .. import kernels


@dataclass
class StepContext:
    n_tokens: int
    n_entries: int
    n_wanted: int
    token_ids: object          # int32 [N]
    positions: object          # int32 [N]   absolute position of each token in its request
    token_entry: object        # int32 [N]   which entry (row of the block tables) a token belongs to
    want_rows: object          # int32 [M]   flattened token indices whose logits are wanted
    entry_slot: object         # int32 [E]   the request's state slot
    entry_start: object        # int32 [E+1] first flattened token of each entry
    entry_pos0: object         # int32 [E]   tokens the request held before this step
    block_tables: dict         # cache group name -> int32 [E, max_blocks]
    host: dict = field(default_factory=dict)   # the same lists on the host, for parts that plan there
    decode_only: bool = False
    split_context: int = 0     # context length the key splits are planned for
    aligned_starts: bool = False   # every entry starts at a multiple of the prompt attention's key block
    runtime: object = None
    sm_count: int = 148

    def block_table(self, group):
        return self.block_tables[group.name]

    def key_splits(self, n_heads, keys_per_block=64, blocks_per_sm=16):
        """How many pieces each row's keys are cut into so that a decode-only step fills the GPU."""
        if not self.decode_only:
            return 1
        want = -(-(self.sm_count * blocks_per_sm) // max(1, self.n_tokens * n_heads))
        return max(1, min(want, (self.split_context + keys_per_block - 1) // keys_per_block, 32))

    def attend(self, q, k, v, cache, n_heads, scale, window=None):
        """Put this step's keys and values into the layer's cache pages (unless the cache is another
        stop's, ``cache.writable == False``) and run paged causal attention of the step's tokens.
        q, k, v: row views [N, heads * head_dim] of one buffer (the fused projection's output)."""
        kv, table = cache.kv, self.block_table(cache.group)
        kv_heads, head_dim = kv.shape[2], kv.shape[4]
        fast = self.runtime.attention != "rows"
        if self.decode_only and fast and self.runtime.attention != "mma" and self.n_tokens * n_heads >= 150 and \
                kernels.attention_decode_pages_supported(n_heads, kv_heads, head_dim, kv.shape[3], q.dtype):
            # whole pages of a group of heads by TMA; it too takes the new keys and values from the projection. Measured
            # with 25 heads and 768 keys: faster than the row kernel from 8 tokens on (11.6 against 14.0 us; 54 against 68
            # at 64), slower at 4 and below (11.0 against 9.8 us; 9.1 against 5.5 at one token), hence the threshold
            splits = kernels.attention_decode_pages_splits(self.n_tokens, n_heads, kv.shape[3], self.split_context, q.device)
            splits = max(splits, -(-table.shape[1] // 128))          # a block holds the ids of at most 128 pages
            return kernels.attention_decode(q, kv, self.token_entry, self.positions, table, n_heads, scale, window,
                                            n_splits=splits, k_new=k if cache.writable else None,
                                            v_new=v if cache.writable else None, kernel="pages")
        if self.decode_only and fast and kernels.attention_decode_supported(n_heads, kv_heads, head_dim, q.dtype):
            # the decode kernel takes the new keys and values from the projection and writes them itself
            return kernels.attention_decode(q, kv, self.token_entry, self.positions, table, n_heads, scale, window,
                                            n_splits=self.key_splits(n_heads, keys_per_block=128, blocks_per_sm=2),
                                            k_new=k if cache.writable else None, v_new=v if cache.writable else None)
        tcgen05 = not self.decode_only and fast and self.runtime.attention != "mma" and \
            kernels.attention_prefill_tcgen05_supported(n_heads, kv_heads, head_dim, kv.shape[3], q.dtype)
        # the tcgen05 prompt kernel writes the cache itself when no key block mixes cached and new keys
        fused_store = tcgen05 and cache.writable and self.aligned_starts
        if cache.writable and not fused_store:
            kernels.kv_store(k, v, self.token_entry, self.positions, table, kv)
        if tcgen05:
            return kernels.attention_prefill(q, kv, self.entry_start, self.entry_pos0, table, n_heads, scale, window,
                                             kernel="tcgen05", k_new=k if cache.writable else None,
                                             v_new=v if cache.writable else None, store_new=fused_store)
        if not self.decode_only and fast and kernels.attention_prefill_supported(n_heads, kv_heads, head_dim, q.dtype):
            return kernels.attention_prefill(q, kv, self.entry_start, self.entry_pos0, table, n_heads, scale, window)
        return kernels.attention_rows(q, kv, self.token_entry, self.positions, table, n_heads, scale, window,
                                      n_splits=self.key_splits(n_heads))
