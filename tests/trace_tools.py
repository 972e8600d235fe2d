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

    def __init__(self):
        self.steps = []
        self.where = {}       # step -> [(request, position)]
        self.fed = {}         # request -> tokens fed so far

    def step(self, parts, end=()):
        """parts: [(request, tokens, want_all: bool)]"""
        number = len(self.steps)
        entries, where = [], []
        for request, tokens, want_all in parts:
            start = self.fed.get(request, 0)
            want = list(range(len(tokens))) if want_all else []
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
