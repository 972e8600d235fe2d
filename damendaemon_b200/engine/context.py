"""The description of one step as the kernels see it: flattened tokens with per-token
position and entry, per-entry bookkeeping, the rows whose logits are wanted, and the
block tables of the entries, all int32 on the device (one host-to-device copy a step)."""
from __future__ import annotations

from dataclasses import dataclass, field



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
    decode_only: bool = False  # every entry brings exactly one token: token t belongs to entry t
    split_context: int = 0     # context length the key splits are planned for
    n_single: int = 0          # the first n_single entries bring exactly one token each (token t is entry t there);
                               # the engine lays single-token entries out first
    aligned_starts: bool = False   # every entry after the first n_single starts at a multiple of the model's portion
                                   # multiple (the key block of its prompt attention kernel), so no key block of theirs
                                   # mixes cached and new keys
    runtime: object = None
    sm_count: int = 148

    def block_table(self, group):
        return self.block_tables[group.name]

    def key_splits(self, n_heads, keys_per_block=64, blocks_per_sm=16, n_tokens=None):
        """How many pieces each row's keys are cut into so that a decode-only step (or, with n_tokens given, the
        single tokens of a mixed step) fills the GPU."""
        if n_tokens is None:
            if not self.decode_only:
                return 1
            n_tokens = self.n_tokens
        want = -(-(self.sm_count * blocks_per_sm) // max(1, n_tokens * n_heads))
        return max(1, min(want, (self.split_context + keys_per_block - 1) // keys_per_block, 32))

    def attend(self, q, k, v, cache, n_heads, scale, window=None):
        """Put this step's keys and values into the layer's cache pages (unless the cache is another
        stop's, ``cache.writable == False``) and run paged causal attention of the step's tokens.
        q, k, v: row views [N, heads * head_dim] of one buffer (the fused projection's output).
        Which kernel runs is decided in parts/paged_attention.py from the sizes and the runtime's tuning."""
        from ..parts.paged_attention import paged_attention
        return paged_attention(self, q, k, v, cache, n_heads, scale, window)
