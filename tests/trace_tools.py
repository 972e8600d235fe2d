"""Helpers for the replay tests: build traces, run bin/trace_run, read its output."""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent


def run_trace(model_dir, dtype, steps, out_dir, max_tokens, page_size=16, timeout=900):
    """steps: list of dicts as trace_run reads them. Returns {step: float32 array [wanted, vocab]}."""
    out_dir = Path(out_dir)
    text = "".join(json.dumps(s) + "\n" for s in steps)
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype,
                           "--out", str(out_dir), "--max-tokens", str(max_tokens), "--page-size", str(page_size)],
                          input=text, capture_output=True, text=True, timeout=timeout)
    assert proc.returncode == 0, f"trace_run failed ({proc.returncode}):\n{proc.stdout[-2000:]}\n{proc.stderr[-4000:]}"
    done = [line for line in proc.stdout.splitlines() if line.startswith("done ")]
    assert [d.split()[1] for d in done] == [str(s["step"]) for s in steps], proc.stdout[-2000:]
    vocab = json.loads((Path(model_dir) / "config.json").read_text())["vocab_size"]
    result = {}
    for s in steps:
        wanted = sum(len(e.get("want", ())) for e in s["entries"])
        path = out_dir / f"{s['step']}.f32"
        if wanted:
            result[s["step"]] = np.fromfile(path, dtype="<f4").reshape(wanted, vocab)
        else:
            assert not path.exists()
    return result


class TraceBuilder:
    """Collects steps and remembers which (request, position) each wanted row is."""

    def __init__(self, wanted=None):
        """wanted: {request: positions whose logits are asked for}; None = every position."""
        self.steps = []
        self.where = {}       # step -> [(request, position)]
        self.fed = {}         # request -> tokens fed so far
        self.wanted = wanted

    def step(self, parts, end=()):
        """parts: [(request, tokens, want: bool)]; where ``wanted`` was given, a part that wants logits
        asks for those of its positions that are in its request's set."""
        number = len(self.steps)
        entries, where = [], []
        for request, tokens, want_all in parts:
            start = self.fed.get(request, 0)
            want = list(range(len(tokens))) if want_all else []
            if self.wanted is not None:
                want = [i for i in want if start + i in self.wanted[request]]
            entries.append({"id": request, "tokens": list(tokens), "want": want})
            where += [(request, start + w) for w in want]
            self.fed[request] = start + len(tokens)
        self.steps.append({"step": number, "entries": entries, "end": list(end)})
        self.where[number] = where
        for r in end:
            self.fed.pop(r, None)
        return number

    def collect(self, outputs):
        """{request: {position: logits row}} from run_trace's result."""
        got = {}
        for number, rows in outputs.items():
            for (request, position), row in zip(self.where[number], rows):
                got.setdefault(request, {})[position] = row
        return got


def round64(n):
    return (n + 63) // 64 * 64


def whole_steps(requests, wanted=None):
    """Each request alone and whole, every position wanted."""
    b = TraceBuilder(wanted)
    for r, tokens in requests.items():
        b.step([(r, tokens, True)], end=[r])
    return b


def tail_steps(requests, tail=32, wanted=None):
    """Most of a request in one step, its last `tail` tokens one by one."""
    b = TraceBuilder(wanted)
    for r, tokens in requests.items():
        head = max(1, len(tokens) - tail)
        b.step([(r, tokens[:head], True)])
        for i in range(head, len(tokens)):
            b.step([(r, tokens[i:i + 1], True)], end=[r] if i == len(tokens) - 1 else [])
        if head == len(tokens):
            b.step([], end=[r])
    return b


def portion_steps(requests, sizes=(7, 2, 16, 3, 2, 33, 5, 2, 64, 1), wanted=None):
    """Portions of changing size, down to two tokens (and one)."""
    b = TraceBuilder(wanted)
    for r, tokens in requests.items():
        at, i = 0, 0
        while at < len(tokens):
            n = min(sizes[i % len(sizes)], len(tokens) - at)
            b.step([(r, tokens[at:at + n], True)], end=[r] if at + n == len(tokens) else [])
            at, i = at + n, i + 1
    return b


def mixed_steps(requests, seed=0, max_live=4, prompt_share=0.6, wanted=None, portions=(2, 3, 5, 8, 13, 17, 32)):
    """Up to max_live requests at a time: portions of some beside decoded tokens of others,
    requests now and then left out of a step. Returns (builder, most tokens held at once, each
    request's count rounded up to 64)."""
    import random
    rng = random.Random(seed)
    b = TraceBuilder(wanted)
    waiting = list(requests)
    live, at = [], {}
    peak = 0
    while waiting or live:
        while waiting and len(live) < max_live:
            r = waiting.pop(0)
            live.append(r)
            at[r] = 0
        parts, ended = [], []
        for r in list(live):
            tokens = requests[r]
            if len(live) > 1 and rng.random() < 0.15:
                continue
            left = len(tokens) - at[r]
            if at[r] < int(prompt_share * len(tokens)):
                n = min(left, rng.choice(portions))
            else:
                n = 1
            parts.append((r, tokens[at[r]:at[r] + n], True))
            at[r] += n
            if at[r] == len(tokens):
                ended.append(r)
        peak = max(peak, sum(round64(at[r]) for r in live))
        if parts:
            b.step(parts, end=ended)
        for r in ended:
            live.remove(r)
    return b, peak
