"""The engine: a model, its cache, and ONE step function.

``step(entries)`` takes a batch of (request, its next tokens, where logits are wanted):
portions of prompts beside single decoded tokens, cut anywhere. It runs only the tokens
it is given, as one flattened batch, against the cache earlier steps left, and returns
float32 logits at the wanted places. The reference has three separate calls that are never
mixed in one forward (prefill_batch / prefill_chunk / decode_batch, damendaemon/paged.py:133-177);
validation before any state change follows damendaemon/paged.py:144-147.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, Sequence

import numpy as np
import torch

from .. import kernels
from ..cache import CacheManager, PageCapacityError
from ..parts import DecoderModel, Runtime, cache_needs, tensor_decls
from ..registry import load_config
from ..weights.loader import DictSource, check_and_place, load_weights
from .context import StepContext

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
          torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


@dataclass
class StepEntry:
    request: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=tuple)   # places among ``tokens`` whose logits are wanted


class StepError(ValueError):
    """The step was refused before anything changed."""


def require_cuda(device):
    if not torch.cuda.is_available():
        raise kernels.KernelError("no CUDA device: this engine runs on an NVIDIA B200 only (no CPU fallback)")
    device = torch.device(device)
    if device.type != "cuda":
        raise kernels.KernelError(f"device {device} is not a CUDA device")
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    return device


class Engine:
    def __init__(self, model_dir=None, *, config=None, tensors=None, dtype="bfloat16", kv_tokens=None,
                 page_size=16, max_requests=64, device="cuda:0", gemm="auto", check_device_errors=True,
                 use_graph=False):
        """Either ``model_dir`` (config.json + model.safetensors) or ``config`` (the raw
        config.json dict) with ``tensors`` ({checkpoint name: tensor})."""
        self.device = require_cuda(device)
        torch.cuda.set_device(self.device)
        self.dtype = DTYPES[dtype]
        if model_dir is not None:
            self.architecture, self.config = load_config(model_dir)
        else:
            from ..registry import architecture_of
            self.architecture = architecture_of(config)
            self.config = self.architecture.parse_config(config)
        self.spec = self.architecture.build_spec(self.config)
        decls = tensor_decls(self.spec)
        if model_dir is not None:
            weights = load_weights(model_dir, self.spec, decls, self.dtype, self.device)
        else:
            weights = check_and_place(DictSource(tensors), self.spec, decls, self.dtype, self.device)
        self.runtime = Runtime(dtype=self.dtype, device=self.device, gemm=gemm, page_size=page_size)
        kernels.library("core")
        if self.dtype == torch.bfloat16 and gemm != "simt":
            kernels.library("tensor")
        self.model = DecoderModel(self.spec, weights, self.runtime)
        self.weight_bytes = sum(t.numel() * t.element_size() for t in weights.values())
        self.page_size = page_size
        self.max_context = self.spec.max_positions
        # where a scheduler should cut a prompt that it has to cut: where the model's mixers like it (a key block of a
        # prompt attention kernel), 1 if they do not care
        self.portion_multiple = self.model.portion_multiple
        if kv_tokens is None:
            kv_tokens = max_requests * self.max_context
        kv_tokens = (kv_tokens + page_size - 1) // page_size * page_size
        self.kv_tokens = kv_tokens
        self.cache = CacheManager(cache_needs(self.spec), kv_tokens, page_size, max_requests, self.max_context)
        self._admit_memory()
        self.cache.allocate(self.device, self.dtype)
        self._caches = [self.cache.layer_view(i) if e.cache_of is None else self.cache.layer_view(e.cache_of, writable=False)
                        for i, e in enumerate(self.spec.run_order)]
        self.check_device_errors = check_device_errors
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.use_graph = use_graph and self.model.graph_safe
        self._graphs, self._seen = {}, {}
        self.graph_replays = 0                          # steps that ran as a replay of a captured graph
        self.graph_captures = 0
        # A capture costs about ten eager steps' worth of host time, so a shape must come back before it is captured:
        # decode-only shapes (which then recur for hundreds of steps) at their second appearance, shapes with prompt
        # portions (whose token counts seldom repeat exactly) at their fourth.
        self.capture_after = {True: 1, False: 3}        # decode only? -> appearances before the capturing one
        self.max_graphs = 48                            # replayable step shapes kept; the least recently used goes first
        # programmatic dependent launch: a gain for the bfloat16 kernels, a loss for the float32 ones (kernels.pdl_scope)
        self.early_launch = self.dtype == torch.bfloat16
        self.max_graph_tokens = 4096                    # larger steps run eagerly (a graph keeps its activations)
        kernels.error_flag(self.device)                 # allocated before any graph capture
        if self.dtype == torch.bfloat16 and gemm != "simt":
            heads = max((getattr(l.mixer, "n_heads", 1) for l in self.spec.layers), default=1)
            kernels._tile_counters(self.device, max(8192, max_requests * heads))
        self._meta_dev = None
        self._meta_host = []
        self._meta_events = []
        self._meta_numpy = []
        self._meta_recorded = [False, False]
        self._arange = np.arange(max_requests + 2, dtype=np.int32)
        self._turn = 0
        self.steps = 0
        self.tokens_run = 0

    HEADROOM_BYTES = 512 << 20

    def _admit_memory(self):
        """Weights are on the device already; the cache, the activations of the largest step and 512 MiB of
        headroom must fit into what is free now, else MemoryError before anything more is allocated
        (damendaemon/qwen2.py:551-553: weights + cache + workspace + 512 MiB against free memory)."""
        element = 2 if self.dtype == torch.bfloat16 else 4
        cache_bytes = self.cache.bytes_needed(element)
        widest = max((getattr(l.feed_forward, "inner", 0) for l in self.spec.layers), default=0)
        per_token = 4 * self.spec.width * 4 + (3 * self.spec.width + widest) * element
        workspace = min(self.max_context * self.cache.max_requests, 8192) * per_token + self.cache.max_requests * self.spec.vocab_size * 4
        free, total = torch.cuda.mem_get_info(self.device)
        need = cache_bytes + workspace + self.HEADROOM_BYTES
        if need > free:
            gib = lambda b: f"{b / 2 ** 30:.2f} GiB"
            raise MemoryError(f"the cache needs {gib(cache_bytes)} ({self.kv_tokens} tokens), a step's activations about "
                              f"{gib(workspace)}, plus {gib(self.HEADROOM_BYTES)} of headroom: {gib(need)} in all, but only "
                              f"{gib(free)} of {gib(total)} are free beside {gib(self.weight_bytes)} of weights; "
                              f"ask for fewer cache tokens (kv_tokens / --kv-cache-tokens)")

    # ------------------------------------------------------------------ requests
    def live_requests(self):
        return list(self.cache.slot_of)

    def length(self, request) -> int:
        return self.cache.length.get(request, 0)

    def finish(self, request):
        """Give back everything the request holds."""
        self.cache.release(request)

    def reserve(self, request, total_tokens, max_step_tokens):
        """Admit a request and promise it pages for total_tokens (see CacheManager.reserve)."""
        fresh = request not in self.cache.slot_of
        if fresh:
            self.cache.admit(request)
        try:
            self.cache.reserve(request, total_tokens, max_step_tokens)
        except Exception:
            if fresh:
                self.cache.release(request)
            raise

    # ------------------------------------------------------------------ the step
    def _validate(self, entries):
        if not entries:
            raise StepError("a step needs at least one entry")
        seen = set()
        vocab = self.spec.vocab_size
        for e in entries:
            if e.request in seen:
                raise StepError(f"request {e.request!r} appears twice in one step")
            seen.add(e.request)
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"request {e.request!r} brings no tokens")
            for t in e.tokens:
                if type(t) is not int or not 0 <= t < vocab:
                    raise StepError(f"request {e.request!r}: token {t!r} is outside the vocabulary of {vocab}")
            if self.length(e.request) + n > self.max_context:
                raise StepError(f"request {e.request!r}: {self.length(e.request)} + {n} tokens exceed the "
                                f"model's {self.max_context} positions")
            for w in e.want:
                if type(w) is not int or not 0 <= w < n:
                    raise StepError(f"request {e.request!r}: wanted place {w!r} is not among its {n} tokens")
            if len(set(e.want)) != len(e.want):
                raise StepError(f"request {e.request!r}: a wanted place is named twice")

    def _meta_buffers(self, n_ints):
        if self._meta_dev is None or self._meta_dev.numel() < n_ints:
            cap = max(1 << 16, 1 << (n_ints - 1).bit_length())
            torch.cuda.current_stream().synchronize()
            self._meta_dev = torch.empty(cap, dtype=torch.int32, device=self.device)
            self._meta_host = [torch.empty(cap, dtype=torch.int32, pin_memory=True) for _ in range(2)]
            self._meta_numpy = [h.numpy() for h in self._meta_host]
            self._meta_events = [torch.cuda.Event(), torch.cuda.Event()]
            self._meta_recorded = [False, False]
            self._graphs.clear()                 # graphs hold views of the old buffer
        self._turn ^= 1
        if self._meta_recorded[self._turn]:
            self._meta_events[self._turn].synchronize()      # the copy out of this host buffer two steps ago is done
        return self._meta_host[self._turn]

    def _layout(self, N, E, M):
        """Offsets of the step's int32 arrays in the metadata buffer; a function of the counts only."""
        MB, o, at = self.cache.max_blocks, 0, {}
        for name, n in (("ids", N), ("pos", N), ("ent", N), ("want", M), ("slot", E), ("start", E + 1), ("pos0", E)):
            at[name] = (o, o + n)
            o += n
        for g in self.cache.groups:
            at["table:" + g.name] = (o, o + E * MB)
            o += E * MB
        at["total"] = o
        return at

    def _fill(self, entries, lengths, at, arr, order=None):
        """Write the step's arrays. order: the entries' indices in the order they are laid out in (None: as given);
        the wanted rows keep the order of the entries as given. Returns slots and first positions in layout order."""
        N, E = sum(lengths), len(entries)
        MB = self.cache.max_blocks
        ids, pos, ent = (arr[at[k][0]:at[k][1]] for k in ("ids", "pos", "ent"))
        want, slot, start, pos0 = (arr[at[k][0]:at[k][1]] for k in ("want", "slot", "start", "pos0"))
        if N == E:
            # one token per entry (a decode step): whole arrays at once instead of an entry at a time
            cache = self.cache
            p0s = [cache.length[e.request] for e in entries]
            slots = [cache.slot_of[e.request] for e in entries]
            ids[:] = [e.tokens[0] for e in entries]
            pos[:] = p0s
            pos0[:] = p0s
            ent[:] = self._arange[:E]
            start[:] = self._arange[:E + 1]
            slot[:] = slots
            wi = 0
            for i, e in enumerate(entries):
                if e.want:                      # [0] or nothing
                    want[wi] = i
                    wi += 1
            for g in cache.groups:
                a, b = at["table:" + g.name]
                arr[a:b].reshape(E, MB)[:] = g.table_array[slots]
            return slots, p0s
        cursor, slots, first_row = 0, [], [0] * E
        for j, i in enumerate(range(E) if order is None else order):
            e, n = entries[i], lengths[i]
            p0 = self.cache.length[e.request]
            ids[cursor:cursor + n] = e.tokens
            pos[cursor:cursor + n] = np.arange(p0, p0 + n, dtype=np.int32)
            ent[cursor:cursor + n] = j
            s = self.cache.slot_of[e.request]
            slots.append(s)
            slot[j], start[j], pos0[j] = s, cursor, p0
            first_row[i] = cursor
            cursor += n
        start[E] = cursor
        wi = 0
        for i, e in enumerate(entries):
            for w in e.want:
                want[wi] = first_row[i] + w
                wi += 1
        for g in self.cache.groups:
            a, b = at["table:" + g.name]
            arr[a:b].reshape(E, MB)[:] = g.table_array[slots]
        return slots, [int(x) for x in pos0]

    def _context(self, N, E, M, at, decode_only, split_context, host=None, aligned=False, n_single=0):
        dev, MB = self._meta_dev, self.cache.max_blocks
        view = lambda k: dev[at[k][0]:at[k][1]]
        return StepContext(
            n_tokens=N, n_entries=E, n_wanted=M, token_ids=view("ids"), positions=view("pos"),
            token_entry=view("ent"), want_rows=view("want"), entry_slot=view("slot"), entry_start=view("start"),
            entry_pos0=view("pos0"),
            block_tables={g.name: view("table:" + g.name).view(E, MB) for g in self.cache.groups},
            host=host or {}, decode_only=decode_only, split_context=split_context, runtime=self.runtime,
            sm_count=self.sm_count, aligned_starts=aligned, n_single=n_single)

    def _upload(self, entries, lengths, at, order=None):
        host = self._meta_buffers(at["total"])
        slots, pos0 = self._fill(entries, lengths, at, self._meta_numpy[self._turn], order)
        kernels.copy_to_device(self._meta_dev, host, at["total"] * 4)
        self.last_h2d_bytes = at["total"] * 4
        self._meta_events[self._turn].record()
        self._meta_recorded[self._turn] = True
        return slots, pos0

    def _run(self, entries, device_ids=None):
        lengths = [len(e.tokens) for e in entries]
        N, E, M = sum(lengths), len(entries), sum(len(e.want) for e in entries)
        at = self._layout(N, E, M)
        decode_only = N == E
        # Entries of a single token are laid out first (a mixer can then give them to a decode kernel as one run of
        # rows and the rest to a prompt kernel); the logits keep the order of the entries as given. Token ids that
        # come from the device are in the given order, so then nothing moves and only the leading singles count.
        order, n_single = None, E
        if not decode_only:
            singles = [i for i, n in enumerate(lengths) if n == 1]
            n_single = len(singles)
            if device_ids is not None or singles == list(range(n_single)):
                n_single = next((i for i, n in enumerate(lengths) if n != 1), E)
            else:
                order = singles + [i for i, n in enumerate(lengths) if n != 1]
                lengths = [lengths[i] for i in order]
        slots, pos0 = self._upload(entries, [len(e.tokens) for e in entries], at, order)
        if device_ids is not None:
            a, b = at["ids"]
            self._meta_dev[a:b].copy_(device_ids.reshape(-1), non_blocking=True)
        host = {"lengths": lengths, "pos0": pos0, "slots": slots}            # in layout order, like the device arrays
        block = self.portion_multiple
        aligned = n_single < E and block > 1 and all(p % block == 0 for p in pos0[n_single:])
        if self.use_graph and M > 0 and N <= self.max_graph_tokens:
            # Every kernel reads lengths, positions and page tables from the metadata buffer, and launch shapes
            # depend only on the counts, so a step of counts seen before can be replayed whatever the lengths are.
            key = (N, E, M, n_single, aligned)
            graph = self._graphs.get(key)
            if graph is None and self._seen.get(key, 0) >= self.capture_after[decode_only]:
                # this shape has come back often enough: capture it (its first run was eager and warmed everything up)
                ctx = self._context(N, E, M, at, decode_only, self.max_context, aligned=aligned, n_single=n_single)
                graph = torch.cuda.CUDAGraph()
                torch.cuda.current_stream().synchronize()
                with torch.cuda.graph(graph), kernels.stream_scope(), kernels.pdl_scope(self.early_launch):
                    static_logits = self.model.forward(ctx, self._caches)
                while len(self._graphs) >= self.max_graphs:
                    self._graphs.pop(next(iter(self._graphs)))
                self._graphs[key] = graph = (graph, static_logits)
                self.graph_captures += 1
            if graph is not None:
                self._graphs[key] = self._graphs.pop(key)        # most recently used last
                graph[0].replay()
                self.graph_replays += 1
                return graph[1]             # valid until the next step of this shape
            self._seen[key] = self._seen.get(key, 0) + 1
            if len(self._seen) > 4096:                   # shapes that never came back
                self._seen = {k: n for k, n in self._seen.items() if n > 1}
        ctx = self._context(N, E, M, at, decode_only, max(p + n for p, n in zip(pos0, lengths)), host, aligned, n_single)
        with kernels.stream_scope(), kernels.pdl_scope(self.early_launch):
            return self.model.forward(ctx, self._caches)

    accepts_device_ids = True          # step() can take the token ids of a decode step from a device tensor

    @torch.no_grad()
    def step(self, entries, end=(), device_ids=None):
        """Run one batch. Returns float32 logits [number of wanted places, vocab] in the order of
        the entries and of each entry's ``want`` (an empty [0, vocab] tensor if none are wanted).
        ``end``: requests that are finished after this step; what they hold is given back.
        ``device_ids``: an int32 tensor on the device with one id per token of the step, in the order of
        the entries, taken instead of the entries' own token values (which then only give the counts):
        the sampler's output of the step before, so that this step can be launched before the host has
        read those tokens. An id outside the vocabulary (the sampler's -1 for a row without a finite
        maximum) sets error bit 1 on the device and its row computes nothing worth having.
        Raises StepError (bad batch) or PageCapacityError (no pages) with nothing changed.
        With CUDA graphs on, the logits of a step whose counts (tokens, entries, wanted places) were
        seen before live in a buffer that the next step of the same counts overwrites."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        self._validate(entries)
        if device_ids is not None and (not torch.is_tensor(device_ids) or device_ids.dtype != torch.int32
                                       or device_ids.numel() != sum(len(e.tokens) for e in entries)
                                       or device_ids.device != self.device):
            raise StepError("device_ids must be an int32 tensor on the engine's device with one id per token")
        fresh = [e.request for e in entries if e.request not in self.cache.slot_of]
        try:
            for r in fresh:
                self.cache.admit(r)
            self.cache.extend([(e.request, self.cache.length[e.request] + len(e.tokens)) for e in entries])
        except Exception:
            for r in fresh:
                self.cache.release(r)
            raise
        logits = self._run(entries, device_ids)
        for e in entries:
            self.cache.advance(e.request, self.cache.length[e.request] + len(e.tokens))
        for r in end:
            self.finish(r)
        self.steps += 1
        self.tokens_run += sum(len(e.tokens) for e in entries)
        if logits is None:
            logits = torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.device)
        if self.check_device_errors:
            self.raise_device_errors()
        return logits

    def raise_device_errors(self):
        """Read the kernels' error word (synchronises). Bits: 1 token or position out of range,
        2 page missing on a cache write, 4 page missing on a cache read, 8 a bounded wait ran out."""
        flag = kernels.read_error_flag(self.device)
        if flag:
            raise RuntimeError(f"a kernel reported error bits {flag:#x} (1 bad token/position, 2 bad page on write, "
                               "4 bad page on read, 8 wait timed out)")
