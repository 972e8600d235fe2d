"""The Python entry point: a ``Runtime`` with ``generate`` in the reference's manner
(damendaemon/runtime.py:514-623): a generator of ``{"token", "text"}`` events and one
terminal ``{"finish_reason", "usage", "timing"}`` event. Prompts are token ids, or text when
the model folder has a ``tokenizer.json`` (the reference requires one, damendaemon/qwen2.py:147;
here it is optional because random-weight folders have none).
"""
from __future__ import annotations

import time
from pathlib import Path

from .engine import Engine
from .engine.scheduler import Request, Scheduler
from .sampling import Sampling
from .text_stream import TextStream, checked_stops


class Runtime:
    def __init__(self, model, context=None, *, dtype="bfloat16", kv_cache_tokens=None, max_batch=16, page_size=16,
                 device="cuda:0", use_graph=True, prefill_chunk_size=0, token_budget=4096, config=None, tensors=None,
                 run_ahead=True, queue_timeout=None):
        """model: a folder with config.json and model.safetensors (or None with config= and tensors=).
        context: most tokens a request may hold (default: the model's positions).
        kv_cache_tokens: size of the shared page pool in tokens (default: max_batch * context).
        prefill_chunk_size: largest prompt portion per step, 0 = up to the token budget.
        run_ahead: launch the next decode step before this step's tokens are read (see the scheduler).
        queue_timeout: seconds a request may wait for cache pages before it fails (None: no limit)."""
        self.engine = Engine(model, config=config, tensors=tensors, dtype=dtype, page_size=page_size,
                             max_requests=max_batch, device=device,
                             kv_tokens=kv_cache_tokens or max_batch * min(context or 10 ** 9, _positions(model, config)),
                             check_device_errors=False, use_graph=use_graph)
        self.context = min(context or self.engine.max_context, self.engine.max_context)
        self.prefill_chunk_size = prefill_chunk_size
        self.token_budget = token_budget
        self.run_ahead = run_ahead
        self.queue_timeout = queue_timeout
        self.tokenizer = _load_tokenizer(model)

    # ------------------------------------------------------------------ helpers
    def _prompt_ids(self, raw_prompt):
        if isinstance(raw_prompt, str):
            if self.tokenizer is None:
                raise ValueError("a text prompt needs tokenizer.json in the model folder; pass token ids instead")
            return self.tokenizer.encode(raw_prompt).ids
        if isinstance(raw_prompt, list) and raw_prompt and all(type(t) is int and t >= 0 for t in raw_prompt):
            return list(raw_prompt)
        raise ValueError("prompt must be text or a nonempty list of token IDs")

    def _scheduler(self, length_policy="reject"):
        return Scheduler(self.engine, token_budget=self.token_budget, chunk_size=self.prefill_chunk_size,
                         length_policy=length_policy, run_ahead=self.run_ahead, max_context=self.context,
                         queue_timeout=self.queue_timeout)

    def _text(self, tokens):
        return self.tokenizer.decode(tokens) if self.tokenizer is not None else ""

    # ------------------------------------------------------------------ one request, streamed
    def generate(self, raw_prompt, max_tokens=128, ignore_eos=False, temperature=0, top_p=1, top_k=0, seed=None,
                 presence_penalty=0, frequency_penalty=0, repetition_penalty=1, logit_bias=None, stop=None):
        """Yield ``{"token": id, "text": delta}`` per generated token, then the terminal event. ``text`` is what has
        become certain with this token (an unfinished UTF-8 sequence or the beginning of a stop string is held back).
        ``stop``: one to four strings; generation ends ('stop') where the text first holds one of them, and neither it
        nor anything after it is handed out (damendaemon/stopping.py:4-41). Stop strings need the folder's tokenizer."""
        if type(max_tokens) is not int or max_tokens <= 0:
            raise ValueError("max_tokens must be a positive integer")
        if max_tokens > self.context:
            raise ValueError("max_tokens exceeds configured context")
        sampling = Sampling(temperature, top_p, top_k, seed, presence_penalty, frequency_penalty, repetition_penalty,
                            logit_bias)
        stops = checked_stops(stop)
        if stops and self.tokenizer is None:
            raise ValueError("stop strings need tokenizer.json in the model folder")
        prompt = self._prompt_ids(raw_prompt)
        if len(prompt) + max_tokens > self.context:
            raise ValueError("prompt plus max_tokens exceeds configured context")
        start = time.perf_counter()
        scheduler = self._scheduler()
        request = scheduler.submit(Request(prompt, max_tokens, sampling, ignore_eos))
        stream, first, stopped_at = TextStream(stops), None, None
        try:
            for event in scheduler.run():
                if event.token is None:
                    if request.finish_reason == "cancelled":
                        break                               # withdrawn below, after a stop string
                    raise RuntimeError(request.error)
                if stopped_at is not None:
                    continue                                # a token of a step that was in flight when the text stopped
                if first is None:
                    first = time.perf_counter() - start
                delta, stopped = stream.push(self._text(request.output), final=event.finished)
                if stopped:
                    stopped_at = len(request.output)
                    scheduler.cancel(request)               # pages back at the next step; no further token is handed out
                yield {"token": event.token, "text": delta}
        finally:
            self.engine.finish(request.id)
        elapsed = time.perf_counter() - start
        n = stopped_at if stopped_at is not None else len(request.output)
        yield {"finish_reason": "stop" if stopped_at is not None else request.finish_reason,
               "usage": {"prompt_tokens": len(prompt), "completion_tokens": n, "total_tokens": len(prompt) + n},
               "timing": {"kernel_backend": "cuda-sm100a", "compute_dtype": str(self.engine.dtype).removeprefix("torch."),
                          "first_token_seconds": first, "total_seconds": elapsed,
                          "decode_tokens_per_second": (n - 1) / (elapsed - first) if n > 1 and elapsed > first else None}}

    # ------------------------------------------------------------------ many requests, batched
    def generate_batch(self, prompts, max_tokens=128, ignore_eos=False, temperature=0, top_p=1, top_k=0, seed=None,
                       length_policy="reject", **penalties):
        """Generate for a list of prompts with continuous batching; returns one list of new token
        ids per prompt, in order. ``seed`` may be one integer (request i uses seed + i) or a list."""
        scheduler = self._scheduler(length_policy)
        requests = []
        for i, p in enumerate(prompts):
            s = seed[i] if isinstance(seed, (list, tuple)) else (None if seed is None else seed + i)
            n = max_tokens[i] if isinstance(max_tokens, (list, tuple)) else max_tokens
            requests.append(scheduler.submit(Request(self._prompt_ids(p), n,
                                                     Sampling(temperature, top_p, top_k, s, **penalties), ignore_eos)))
        try:
            for _ in scheduler.run():
                pass
        finally:
            for r in requests:
                self.engine.finish(r.id)
        failed = [r for r in requests if r.finish_reason == "error"]
        if failed:
            raise RuntimeError(f"{len(failed)} request(s) failed: {failed[0].error}")
        self.last_scheduler = scheduler
        return [list(r.output) for r in requests]


def _positions(model, config):
    from .registry import architecture_of, load_config
    if config is not None:
        arch = architecture_of(config)
        typed = arch.parse_config(config)
    else:
        arch, typed = load_config(model)
    return arch.build_spec(typed).max_positions


def _load_tokenizer(model):
    if model is None or not (Path(model) / "tokenizer.json").is_file():
        return None
    try:
        from tokenizers import Tokenizer
    except ImportError:
        return None
    return Tokenizer.from_file(str(Path(model) / "tokenizer.json"))


def generate(model, prompts, max_new_tokens=128, *, temperature=0, seed=None, ignore_eos=True, dtype="bfloat16",
             page_size=16, kv_tokens=None, **options):
    """One call from a model folder to new token ids: ``generate(dir, [[ids], ...], 16)``."""
    runtime = Runtime(model, dtype=dtype, page_size=page_size, kv_cache_tokens=kv_tokens,
                      max_batch=max(1, min(64, len(prompts))))
    return runtime.generate_batch(prompts, max_new_tokens, ignore_eos=ignore_eos, temperature=temperature, seed=seed,
                                  **options)
