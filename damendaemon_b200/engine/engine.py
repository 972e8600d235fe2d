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
    return device


class Engine:
    def __init__(self, model_dir=None, *, config=None, tensors=None, dtype="bfloat16", kv_tokens=None,
                 page_size=16, max_requests=64, device="cuda:0", gemm="auto", check_device_errors=True):
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
        self.runtime = Runtime(dtype=self.dtype, device=self.device, gemm=gemm)
        kernels.library("core")
        if self.dtype == torch.bfloat16 and gemm != "simt":
            kernels.library("tensor")
        self.model = DecoderModel(self.spec, weights, self.runtime)
        self.weight_bytes = sum(t.numel() * t.element_size() for t in weights.values())
        self.page_size = page_size
        self.max_context = self.spec.max_positions
        if kv_tokens is None:
            kv_tokens = max_requests * self.max_context
        kv_tokens = (kv_tokens + page_size - 1) // page_size * page_size
        self.cache = CacheManager(cache_needs(self.spec), kv_tokens, page_size, max_requests, self.max_context)
        self.cache.allocate(self.device, self.dtype)
        self._caches = [self.cache.layer_view(i) for i in range(len(self.spec.layers))]
        self.check_device_errors = check_device_errors
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self._meta_dev = None
        self._meta_host = []
        self._meta_events = []
        self._turn = 0
        self.steps = 0
        self.tokens_run = 0

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

    def _meta_buffers(self, n_ints):
        if self._meta_dev is None or self._meta_dev.numel() < n_ints:
            cap = max(4096, 1 << (n_ints - 1).bit_length())
            torch.cuda.current_stream().synchronize()
            self._meta_dev = torch.empty(cap, dtype=torch.int32, device=self.device)
            self._meta_host = [torch.empty(cap, dtype=torch.int32, pin_memory=True) for _ in range(2)]
            self._meta_events = [None, None]
        self._turn ^= 1
        if self._meta_events[self._turn] is not None:
            self._meta_events[self._turn].synchronize()
        return self._meta_host[self._turn]

    def _build_context(self, entries):
        lengths = [len(e.tokens) for e in entries]
        N, E, M = sum(lengths), len(entries), sum(len(e.want) for e in entries)
        MB = self.cache.max_blocks
        groups = self.cache.groups
        total = 3 * N + M + E + (E + 1) + E + len(groups) * E * MB
        host = self._meta_buffers(total)
        arr = host.numpy()
        ids, pos, ent = arr[0:N], arr[N:2 * N], arr[2 * N:3 * N]
        o = 3 * N
        want = arr[o:o + M]; o += M
        slot = arr[o:o + E]; o += E
        start = arr[o:o + E + 1]; o += E + 1
        pos0 = arr[o:o + E]; o += E
        tables = []
        for _ in groups:
            tables.append(arr[o:o + E * MB].reshape(E, MB)); o += E * MB
        cursor, wi = 0, 0
        slots = []
        for i, e in enumerate(entries):
            n = lengths[i]
            p0 = self.cache.length[e.request]
            ids[cursor:cursor + n] = e.tokens
            pos[cursor:cursor + n] = np.arange(p0, p0 + n, dtype=np.int32)
            ent[cursor:cursor + n] = i
            for w in e.want:
                want[wi] = cursor + w
                wi += 1
            s = self.cache.slot_of[e.request]
            slots.append(s)
            slot[i], start[i], pos0[i] = s, cursor, p0
            cursor += n
        start[E] = cursor
        for g, table in zip(groups, tables):
            table[:] = g.table_array[slots]
        dev = self._meta_dev
        dev[:total].copy_(host[:total], non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        self._meta_events[self._turn] = event
        o = 3 * N
        views = {}
        views["want"] = dev[o:o + M]; o += M
        views["slot"] = dev[o:o + E]; o += E
        views["start"] = dev[o:o + E + 1]; o += E + 1
        views["pos0"] = dev[o:o + E]; o += E
        block_tables = {}
        for g in groups:
            block_tables[g.name] = dev[o:o + E * MB].view(E, MB); o += E * MB
        decode_only = all(n == 1 for n in lengths)
        return StepContext(
            n_tokens=N, n_entries=E, n_wanted=M, token_ids=dev[0:N], positions=dev[N:2 * N],
            token_entry=dev[2 * N:3 * N], want_rows=views["want"], entry_slot=views["slot"],
            entry_start=views["start"], entry_pos0=views["pos0"], block_tables=block_tables,
            host={"lengths": lengths, "pos0": [int(x) for x in pos0], "slots": slots},
            decode_only=decode_only, split_context=int(max(p + n for p, n in zip(pos0, lengths))),
            runtime=self.runtime, sm_count=self.sm_count)

    @torch.no_grad()
    def step(self, entries, end=()):
        """Run one batch. Returns float32 logits [number of wanted places, vocab] in the order of
        the entries and of each entry's ``want`` (an empty [0, vocab] tensor if none are wanted).
        ``end``: requests that are finished after this step; what they hold is given back.
        Raises StepError (bad batch) or PageCapacityError (no pages) with nothing changed."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        self._validate(entries)
        fresh = [e.request for e in entries if e.request not in self.cache.slot_of]
        try:
            for r in fresh:
                self.cache.admit(r)
            self.cache.extend([(e.request, self.cache.length[e.request] + len(e.tokens)) for e in entries])
        except Exception:
            for r in fresh:
                self.cache.release(r)
            raise
        ctx = self._build_context(entries)
        logits = self.model.forward(ctx, self._caches)
        for e in entries:
            self.cache.advance(e.request, self.cache.length[e.request] + len(e.tokens))
        for r in end:
            self.finish(r)
        self.steps += 1
        self.tokens_run += ctx.n_tokens
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
