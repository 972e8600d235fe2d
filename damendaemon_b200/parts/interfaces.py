"""What a part must look like. Parts are chosen by the spec's ``kind`` and built as
``cls(spec, weights, runtime)``; none of them knows which model it is in.

``weights``  {checkpoint name: device tensor}, already checked and placed.
``runtime``  a ``Runtime`` (below): engine dtype, device and kernel choices.
``ctx``      the step's ``StepContext`` (engine/context.py): flattened token metadata
             on the device, block tables per cache group, and ``ctx.attend(q, k, v, cache,
             heads, scale, window)``: cache write plus paged causal attention with the best
             kernel for the step.
``cache``    a ``LayerCache`` (cache/manager.py): ``kv`` pages of this layer
             [pages, 2, kv_heads, page_size, head_dim], ``group`` (its block table is
             ``ctx.block_table(cache.group)``), ``state`` rows [max_requests, ...],
             ``writable`` (False when the stop reads another stop's cache).

Embedding         tensor_decls(spec); forward(ctx, position) -> float32 residual stream [N,width]
Head              tensor_decls(spec); forward(x, ctx) -> float32 logits [ctx.n_wanted, vocab] at rows ctx.want_rows
Norm              tensor_decls(spec); forward(x_f32 [N,width], row_index=None) -> [N,width] engine dtype
PositionEncoding  tensor_decls(spec); embedding_table() -> table or None (added to the token
                  embedding by the fused embedding kernel); on_embedding(x, ctx) -> x for
                  encodings that act there without a table; on_query_key(q, k, ctx) -> (q, k)
                  for encodings that rotate or bias inside the mixer
Mixer             tensor_decls(spec); cache_needs(spec) -> [a paged need (cache/manager.py: PagedKeyValues, or any
                  PagedNeed of the mixer's own) | RequestState]; forward(y, residual, ctx, cache, position) ->
                  residual + mix(y)   (float32 [N,width]); optionally portion_multiple: where the mixer likes a
                  prompt to be cut (the engine passes the largest one on to the scheduler)
FeedForward       tensor_decls(spec); forward(y, residual, ctx) -> residual + ff(y)
Arrangement       cls(layer_spec, norms, mixer, feed_forward), norms being the built norms of layer_spec.norms in
                  order; forward(x, ctx, cache, position) -> x

``residual`` is the float32 residual stream; a part returns the updated stream and may
write it in place (the GEMM epilogues add into it).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from .paged_attention import AttentionTuning


@dataclass
class Runtime:
    dtype: torch.dtype            # engine dtype: torch.bfloat16 or torch.float32
    device: torch.device
    gemm: str = "auto"            # 'auto' | 'simt' | 'tcgen05'
    attention: str = "auto"       # 'auto' | 'mma' (no tcgen05 prompt kernel) | 'rows' (the general kernel only)
    attention_tuning: AttentionTuning = field(default_factory=AttentionTuning)   # measured thresholds of the kernel choice
    page_size: int = 16           # tokens per cache page (mixers ask their kernels what they support at this size)


class Part:
    @staticmethod
    def tensor_decls(spec):
        return []


class Mixer(Part):
    # True if forward() launches the same kernels with the same arguments whenever the step's
    # counts are the same (everything that varies is read from device memory), so that a
    # decode step may be replayed from a CUDA graph. Parts that plan on the host say False.
    graph_safe = False

    @staticmethod
    def cache_needs(spec):
        return []

    def forward(self, y, residual, ctx, cache, position):
        raise NotImplementedError


class FeedForward(Part):
    graph_safe = False

    def forward(self, y, residual, ctx):
        raise NotImplementedError


class Norm(Part):
    def forward(self, x, row_index=None):
        raise NotImplementedError


class Embedding(Part):
    def forward(self, ctx, position):
        raise NotImplementedError


class Head(Part):
    def forward(self, x, ctx):
        raise NotImplementedError


class PositionEncoding(Part):
    def embedding_table(self):
        return None

    def on_embedding(self, x, ctx):
        return x

    def on_query_key(self, q, k, ctx):
        return q, k
