#!/usr/bin/env python3
"""The reference arm of bench.py: the UNMODIFIED reference (installed under baseline/_ref) on the
same metric and configuration, through its own public API and stock code path.

GPT-2 XL shape, seeded random weights written to a temporary model folder (config.json,
model.safetensors, a two-word tokenizer.json the reference insists on), then
``damendaemon.scheduler.BatchedRuntime`` with ``batch_size`` concurrent ``generate`` calls, the way
its server drives it: 512-token raw prompts, greedy, W + K + 1 new tokens each. Decode tokens
per second are counted from the moment every request has its first token. The reference runs
GPT-2 in float32 only (damendaemon/qwen2.py:401-405), with fixed per-slot caches and batch <= 16.
None of this repository's model, engine or kernel code is on this path; only its random-weight
writer prepares the folder.

Runs in a process of its own because the reference wants CUDA_VISIBLE_DEVICES to be one GPU UUID
before torch is imported (damendaemon/runtime.py:41-59).
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def gpu_uuid():
    out = subprocess.run(["nvidia-smi", "-L"], capture_output=True, text=True, timeout=60).stdout
    for line in out.splitlines():
        if "UUID:" in line:
            return line.split("UUID:")[1].strip().rstrip(")").strip()
    raise RuntimeError("no GPU UUID from nvidia-smi -L")


def write_folder(folder, config):
    sys.path.insert(0, str(ROOT))
    from damendaemon_b200.weights import write_random_model
    write_random_model(folder, {**config, "eos_token_id": config["vocab_size"] - 1}, seed=0, dtype="bfloat16",
                       name_prefix="transformer.")
    (Path(folder) / "tokenizer.json").write_text(json.dumps({
        "version": "1.0", "truncation": None, "padding": None, "added_tokens": [], "normalizer": None,
        "pre_tokenizer": {"type": "Whitespace"}, "post_processor": None, "decoder": None,
        "model": {"type": "WordLevel", "vocab": {"a": 0, "b": 1}, "unk_token": "a"}}))
    (Path(folder) / "tokenizer_config.json").write_text("{}")


def child(args):
    os.environ["CUDA_VISIBLE_DEVICES"] = gpu_uuid()
    os.environ.setdefault("HF_HUB_OFFLINE", "1")
    sys.path.insert(0, str(ROOT / "baseline" / "_ref"))
    config = json.loads(args.config)
    prompt_len, batch, new_tokens = args.prompt, args.batch, args.warmup + args.steps + 1
    with tempfile.TemporaryDirectory() as tmp:
        folder = Path(tmp) / "model"
        write_folder(folder, config)
        import torch
        from damendaemon.scheduler import BatchedRuntime
        runtime = BatchedRuntime({"model": str(folder)}, batch_size=batch, queue_size=max(8, batch), context=config["n_positions"],
                                 use_graph=True)
        g = torch.Generator().manual_seed(100)
        prompts = [torch.randint(0, config["vocab_size"] - 1, (prompt_len,), generator=g).tolist() for _ in range(batch)]
        first, done, counts, errors = [None] * batch, [None] * batch, [0] * batch, []

        def run(i):
            try:
                for event in runtime.generate("model", None, max_tokens=new_tokens, raw_prompt=prompts[i]):
                    if "token" in event:
                        counts[i] += 1
                        if first[i] is None:
                            first[i] = time.perf_counter()
                done[i] = time.perf_counter()
            except Exception as error:      # noqa: BLE001
                errors.append(f"{type(error).__name__}: {error}")

        def round_trip():
            for i in range(batch):
                first[i], done[i], counts[i] = None, None, 0
            threads = [threading.Thread(target=run, args=(i,)) for i in range(batch)]
            for t in threads:
                t.start()
            for t in threads:
                t.join()

        round_trip()                     # loads the model, compiles kernels, captures graphs
        if not errors:
            round_trip()
        if errors:
            print(json.dumps({"impl": "reference", "unavailable": "the reference failed on this box: " + errors[0][:300]}))
            return 0
        start = max(first)
        tokens = sum(counts) - batch
        elapsed = max(done) - start
        value = tokens / elapsed if elapsed > 0 and tokens > 0 else None
        print(json.dumps({
            "impl": "reference", "metric": f"decode tok/s at batch {batch} (GPT-2 XL shape, prompts of {prompt_len}, timed steps at context "
                                           f"{prompt_len + 2}->{prompt_len + new_tokens})",
            "value": None if value is None else round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": None if value is None else round(1000.0 * batch / value, 4),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
            "e2e": {"value": None if value is None else round(value, 1), "unit": "tokens/s"},
            "config": {"model": "gpt2-xl-shape", "n_layer": config["n_layer"], "global_batch": batch, "seq_len": 1024,
                       "prompt_len": prompt_len, "tokens_generated": sum(counts), "expected": batch * new_tokens,
                       "path": "BatchedRuntime.generate, fixed slots, CUDA graphs, float32 (its only GPT-2 mode)",
                       "timing": "wall clock from every request's first token to the last request's end"}}))
    return 0


def run(args, config, prompt_len):
    """Called by bench.py: run this file in a fresh process and hand back its JSON line."""
    cmd = [sys.executable, str(Path(__file__).resolve()), "--child", "--config", json.dumps(config), "--prompt", str(prompt_len),
           "--steps", str(min(args.steps, config["n_positions"] - prompt_len - args.warmup - 1)), "--warmup", str(args.warmup),
           "--batch", str(args.batch)]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=1500)
    lines = [l for l in proc.stdout.splitlines() if l.startswith("{")]
    if proc.returncode or not lines:
        tail = (proc.stderr or proc.stdout).strip().splitlines()[-1:] or ["no output"]
        return {"impl": "reference", "unavailable": f"the reference process exited {proc.returncode}: {tail[0][:300]}"}
    return json.loads(lines[-1])


if __name__ == "__main__":
    parser = argparse.ArgumentParser()
    parser.add_argument("--child", action="store_true")
    parser.add_argument("--config")
    parser.add_argument("--prompt", type=int, default=512)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--batch", type=int, default=8)
    sys.exit(child(parser.parse_args()))
