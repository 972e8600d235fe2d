#!/usr/bin/env python3
"""Headline benchmark: GPT-2 XL shape, random bfloat16 weights, one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--layers N]

A "step" is one decode step of the whole batch. Default run: batch 8, every request a
512-token prompt, then W untimed and K timed decode steps (context 512 -> 1024). ``value`` is
decoded tokens a second timed on the device with CUDA events (tokens known in advance, the
argmax kernel included, nothing read back); ``e2e`` is the same through the Python entry
point's scheduler: host token ids in (pinned metadata copy every step), sampled ids out
(device-to-host read every step). Also on the line: a 2,048-token prefill (2 prompts of
1,024), decode at batch 1 and 64, the HBM roofline of the decode step, clocks sampled
during the timed region, and the number of kernels launched.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

XL = {"architectures": ["GPT2LMHeadModel"], "model_type": "gpt2", "n_layer": 48, "n_embd": 1600, "n_head": 25,
      "n_inner": 6400, "vocab_size": 50257, "n_positions": 1024, "layer_norm_epsilon": 1e-5,
      "activation_function": "gelu_new"}
PROMPT = 512
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            raw = json.loads(path.read_text())
            return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"])}, "measured"
        except (KeyError, ValueError, TypeError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self):
        self.lines, self.proc = [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.thread.join(timeout=5)

    def summary(self):
        sm, top, reasons = [], 0, set()
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) != 6 or not parts[0].isdigit():
                continue
            sm.append(int(parts[0]))
            top = max(top, int(parts[1]) if parts[1].isdigit() else 0)
            reasons |= {n for n, v in zip(self.NAMES, parts[2:]) if v.lower().startswith("active")}
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": top or None, "reasons": sorted(reasons),
                "samples": len(sm)}


def make_runtime(config, batch, use_graph=True, seed=0, dtype="bfloat16"):
    import torch
    from damendaemon_b200.registry import architecture_of
    from damendaemon_b200.runtime import Runtime
    arch = architecture_of(config)
    typed = arch.parse_config(config)
    tensors = arch.random_tensors(typed, seed, torch.bfloat16, device="cuda")
    slots = max(batch, 2)           # the prefill of two prompts runs on the same engine
    runtime = Runtime(None, config=config, tensors=tensors, dtype=dtype, max_batch=slots,
                      kv_cache_tokens=slots * config["n_positions"], use_graph=use_graph, token_budget=4096)
    del tensors
    torch.cuda.empty_cache()
    return runtime


def random_ids(n, vocab, seed):
    import torch
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def prefill_all(engine, prompts, budget=4096):
    from damendaemon_b200.engine import StepEntry
    names = list(prompts)
    per = max(1, budget // max(len(p) for p in prompts.values()))
    for i in range(0, len(names), per):
        engine.step([StepEntry(r, prompts[r], []) for r in names[i:i + per]])


def decode_device_timed(engine, batch, warmup, steps, vocab, prompt_len=PROMPT):
    """K decode steps with tokens known in advance, timed on the device. Returns (ms per step, bytes per step, launches per step)."""
    import torch
    from damendaemon_b200 import kernels
    from damendaemon_b200.engine import StepEntry
    prompts = {f"d{i}": random_ids(prompt_len, vocab, 100 + i) for i in range(batch)}
    prefill_all(engine, prompts)
    feed = [random_ids(batch, vocab, 1000 + s) for s in range(warmup + steps)]

    def one(s):
        logits = engine.step([StepEntry(r, [feed[s][i]], [0]) for i, r in enumerate(prompts)])
        return kernels.sample(logits)
    # one eager step counts the kernels of a step (graph replays launch the same ones)
    before = kernels.launches
    one(0)
    per_step = kernels.launches - before
    for s in range(1, warmup):
        one(s)
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for s in range(warmup, warmup + steps):
        one(s)
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / steps
    kv_per_token = engine.cache.bytes_per_token(2)
    contexts = [prompt_len + s + 1 for s in range(warmup, warmup + steps)]
    position_table = engine.spec.max_positions * engine.spec.width * 2
    bytes_per_step = engine.weight_bytes - position_table + batch * kv_per_token * statistics.mean(contexts)
    for r in prompts:
        engine.finish(r)
    return ms, bytes_per_step, per_step


def decode_end_to_end(runtime, batch, warmup, steps, vocab):
    """The same through the scheduler: host tokens in, sampled tokens out, every step."""
    import torch
    from damendaemon_b200.engine.scheduler import Request, Scheduler
    scheduler = Scheduler(runtime.engine, token_budget=4096)
    for i in range(batch):
        # a few tokens beyond the timed steps: no request ends inside them, so the scheduler keeps one step in flight
        # at both ends of the timed region, which then holds `steps` forward passes launched and waited for
        scheduler.submit(Request(random_ids(PROMPT, vocab, 100 + i), max_tokens=warmup + steps + 4, ignore_eos=True))
    while scheduler.waiting or scheduler.prefilling:
        scheduler.step()
    for _ in range(warmup):
        scheduler.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    produced = 0
    for _ in range(steps):
        produced += len(scheduler.step())
    stop.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    h2d = runtime.engine.last_h2d_bytes
    for r in scheduler.live():
        runtime.engine.finish(r.id)
    return produced / wall, h2d, (batch + 1) * 4     # the sampled ids and the kernels' error word


def prefill_timed(engine, vocab, repeats=5, prompts=2, length=1024):
    import torch
    from damendaemon_b200.engine import StepEntry
    times = []
    for rep in range(2 + repeats):
        entries = [StepEntry(f"p{rep}-{i}", random_ids(length, vocab, 7 + i + 10 * rep), [length - 1]) for i in range(prompts)]
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        engine.step(entries, end=[e.request for e in entries])
        stop.record()
        torch.cuda.synchronize()
        if rep >= 2:
            times.append(start.elapsed_time(stop))
    return statistics.median(times)


def prefill_flops(c, layers, tokens_per_prompt=1024, prompts=2):
    h, inner = c["n_embd"], c["n_inner"]
    matrices = layers * (3 * h * h + h * h + 2 * h * inner)
    gemm = 2 * matrices * tokens_per_prompt * prompts + 2 * prompts * c["vocab_size"] * h
    attention = prompts * layers * 4 * (tokens_per_prompt * (tokens_per_prompt + 1) // 2) * h
    return gemm + attention


WORKLOADS = {
    # GPT-2 medium shape: 32 requests, prompt lengths uniform in [16, 768], 128 new tokens each at temperature 1.0,
    # admitted continuously
    "medium": {"config": {**XL, "n_layer": 24, "n_embd": 1024, "n_head": 16, "n_inner": 4096}, "max_live": 32},
    # GPT-2 large shape: 8 prompts of 1,000 tokens in portions of 256 beside 56 requests that decode from contexts
    # spread over 1..1000, greedy
    "large": {"config": {**XL, "n_layer": 36, "n_embd": 1280, "n_head": 20, "n_inner": 5120}, "max_live": 64},
}


def run_workload(name, dtype="bfloat16"):
    """The scheduler under a mixed load (continuous batching): total generated tokens per second and the step mix."""
    import random
    import torch
    from damendaemon_b200.engine.scheduler import Request, Scheduler
    from damendaemon_b200.sampling import Sampling
    spec = WORKLOADS[name]
    config = spec["config"]
    vocab = config["vocab_size"]
    runtime = make_runtime(config, spec["max_live"], dtype=dtype)
    def make_requests():
        rng = random.Random(0)
        if name == "medium":
            return [Request(random_ids(rng.randint(16, 768), vocab, 10 + i), 128, Sampling(temperature=1.0, seed=i), True)
                    for i in range(32)]
        requests = [Request(random_ids(1 + (i * 999) // 55, vocab, 10 + i), 24, Sampling(), True) for i in range(56)]
        return requests + [Request(random_ids(1000, vocab, 100 + i), 24, Sampling(), True) for i in range(8)]

    def one_pass():
        if name == "medium":
            scheduler = Scheduler(runtime.engine, token_budget=2048, chunk_size=512, max_live=32)
        else:
            scheduler = Scheduler(runtime.engine, token_budget=2048, chunk_size=256, max_live=64, length_policy="clamp")
        requests = make_requests()
        for r in requests:
            scheduler.submit(r)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in scheduler.run():
            pass
        torch.cuda.synchronize()
        return scheduler, requests, time.perf_counter() - t0
    # the first pass meets every step shape for the first time; later passes over the same requests replay what has
    # been captured meanwhile: what a server that has been up for a while does
    _, first_requests, cold = one_pass()
    cold_value = sum(len(r.output) for r in first_requests) / cold
    for _ in range(3):                                   # shapes that keep coming back are captured on the way
        one_pass()
    scheduler, requests, wall = one_pass()
    generated = sum(len(r.output) for r in requests)
    prompt_tokens = sum(len(r.prompt) for r in requests)
    mixed = sum(1 for p, d in scheduler.step_log if p and d)
    run_workload.outputs = [list(r.output) for r in requests]
    return {"workload": name, "metric": "generated tokens/s through the scheduler", "value": round(generated / wall, 1),
            "unit": "tokens/s", "requests": len(requests), "prompt_tokens": prompt_tokens, "generated_tokens": generated,
            "prompt_tokens_per_s": round(prompt_tokens / wall, 1), "seconds": round(wall, 3), "steps": scheduler.steps,
            "steps_mixing_prompt_and_decode": mixed, "failed": sum(1 for r in requests if r.finish_reason == "error"),
            "first_pass_value": round(cold_value, 1), "graph_replays": runtime.engine.graph_replays,
            "graph_captures": runtime.engine.graph_captures,
            "config": {"n_layer": config["n_layer"], "n_embd": config["n_embd"], "n_head": config["n_head"], "dtype": dtype,
                       "note": "value: the fifth pass over the same requests (step shapes that keep coming back are replayed from "
                               "graphs); first_pass_value: the first, in which every step shape is new"}}


def parity(layers):
    """The float32 engine beside the bfloat16 one on the benchmark's own model (seeded random weights): two requests,
    a 512-token prompt and 32 teacher-forced decode steps each. Reports the largest difference of the float32
    logits from the plain float64 implementation (tests/plain_gpt2.py, run on the GPU) and of the bfloat16 logits from
    the float32 ones, and how often the greedy tokens agree."""
    import torch
    from damendaemon_b200.engine import Engine, StepEntry
    from damendaemon_b200.registry import architecture_of
    sys.path.insert(0, str(ROOT / "tests"))
    import plain_gpt2
    config = {**XL, "n_layer": layers}
    arch = architecture_of(config)
    tensors = arch.random_tensors(arch.parse_config(config), 0, torch.float32, device="cuda")
    for name, t in tensors.items():
        if t.dim() == 2:
            tensors[name] = t.to(torch.bfloat16).float()        # both engines and the plain side read the same numbers
    requests = {f"p{i}": random_ids(PROMPT + 32, config["vocab_size"], 40 + i) for i in range(2)}
    rows = list(range(PROMPT - 1, PROMPT + 32))
    w = {k: v.double() for k, v in tensors.items()}
    want = {r: plain_gpt2.logits_of(config, w, ids, rows=rows).float() for r, ids in requests.items()}
    del w
    torch.cuda.empty_cache()
    got = {}
    for dtype in ("float32", "bfloat16"):
        engine = Engine(config=config, tensors=tensors, dtype=dtype, kv_tokens=2 * 1024, page_size=16, max_requests=2,
                        use_graph=True)
        out = {r: [] for r in requests}
        first = engine.step([StepEntry(r, ids[:PROMPT], [PROMPT - 1]) for r, ids in requests.items()])
        for i, r in enumerate(requests):
            out[r].append(first[i].clone())
        for s in range(32):
            logits = engine.step([StepEntry(r, [ids[PROMPT + s]], [0]) for r, ids in requests.items()])
            for i, r in enumerate(requests):
                out[r].append(logits[i].clone())
        got[dtype] = {r: torch.stack(v) for r, v in out.items()}
        del engine
        torch.cuda.empty_cache()
    worst = lambda a, b: max(float((a[r] - b[r]).abs().max()) for r in requests)
    same = lambda a, b: sum(int((a[r].argmax(-1) == b[r].argmax(-1)).sum()) for r in requests)
    total = 33 * len(requests)

    def widest_flipped_margin(a, b):
        """Among rows whose greedy tokens differ: the largest gap between the reference's best and second-best logit
        (a flip is a near tie if this is below the logit difference between the two engines)."""
        gap = 0.0
        for r in requests:
            flipped = a[r].argmax(-1) != b[r].argmax(-1)
            if bool(flipped.any()):
                top = b[r][flipped].topk(2, dim=-1).values
                gap = max(gap, float((top[:, 0] - top[:, 1]).max()))
        return gap
    return {"parity": "GPT-2 XL shape, seeded random weights, 2 requests x (512-token prompt + 32 forced decode steps)",
            "n_layer_run": layers, "rows_compared": total,
            "float32_vs_plain_float64": {"max_abs_logit_diff": worst(got["float32"], want), "same_greedy": same(got["float32"], want)},
            "bfloat16_vs_float32": {"max_abs_logit_diff": worst(got["bfloat16"], got["float32"]),
                                    "same_greedy": same(got["bfloat16"], got["float32"]),
                                    "widest_top2_gap_where_greedy_differs": widest_flipped_margin(got["bfloat16"], got["float32"])},
            "logit_scale": float(max(v.abs().max() for v in want.values()))}


def line_config(layers, batch, cuda_graph=True):
    """What both arms run, in the same words (the `config` of the bench line, flat): every size of the model, the batch,
    the lengths. What only one arm can say of itself (page size, timing method) is under `engine`."""
    return {"model": "gpt2-xl-shape", "n_layer": XL["n_layer"], "n_layer_run": layers, "n_embd": XL["n_embd"], "n_head": XL["n_head"],
            "head_dim": XL["n_embd"] // XL["n_head"], "n_inner": XL["n_inner"], "vocab_size": XL["vocab_size"],
            "n_positions": XL["n_positions"], "global_batch": batch, "seq_len": XL["n_positions"], "prompt_len": PROMPT,
            "activation": XL["activation_function"], "parallelism": "single-gpu",
            "l2": "inputs>L2 (every weight is read once a step)", "cuda_graph": cuda_graph}


def reference_arm(args):
    """The unmodified reference through its own public API, if it is installed under baseline/_ref."""
    ref = ROOT / "baseline" / "_ref"
    note = (ROOT / "baseline" / "UNAVAILABLE.txt")
    why = note.read_text().strip() if note.is_file() else None
    if why is None and not (ref / "damendaemon").is_dir():
        why = "the reference is not installed under baseline/_ref"
    if why is None:
        try:
            sys.path.insert(0, str(ROOT / "baseline"))
            import run_reference
            config = dict(XL)
            if args.layers:
                config["n_layer"] = args.layers
            line = run_reference.run(args, config, PROMPT)
            if "config" in line:
                line["engine"] = line.pop("config")
                line["config"] = line_config(config["n_layer"], args.batch)
            print(json.dumps(line), flush=True)
            return 0
        except Exception as error:      # noqa: BLE001
            why = f"the reference arm failed: {type(error).__name__}: {str(error)[:200]}"
    print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
    return 0


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=480)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=0, help="run fewer layers than the configuration has (named in config)")
    parser.add_argument("--no-points", action="store_true", help="skip the batch-1 and batch-64 points")
    parser.add_argument("--no-graph", action="store_true", help="launch every decode kernel eagerly (for profilers)")
    parser.add_argument("--kernel-case", help="time one kernel alone at XL shape (see bench_kernel_cases.py)")
    parser.add_argument("--case-iters", type=int, default=50)
    parser.add_argument("--case-graph", action="store_true", help="time the kernel case as launches replayed from one CUDA graph")
    parser.add_argument("--workload", choices=sorted(WORKLOADS), help="run a scheduler workload instead of the headline bench")
    parser.add_argument("--parity", action="store_true", help="the float32 engine beside the bfloat16 one: on the benchmark's model "
                        "(logit differences, greedy agreement), or with --workload on that workload (the same requests in both)")
    args = parser.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.impl == "reference":
        return reference_arm(args)
    if args.workload:
        result = run_workload(args.workload)
        if args.parity:
            # the same requests through the float32 engine: greedy tokens agree until rounding flips a near tie
            half = run_workload.outputs
            result["float32"] = {k: v for k, v in run_workload(args.workload, dtype="float32").items()
                                 if k in ("value", "seconds", "steps", "failed")}
            full = run_workload.outputs
            common = [next((i for i, (a, b) in enumerate(zip(x, y)) if a != b), min(len(x), len(y))) for x, y in zip(half, full)]
            result["parity"] = {"requests_with_the_same_first_token": sum(1 for n in common if n >= 1), "requests": len(common),
                                "mean_common_prefix": round(sum(common) / len(common), 2),
                                "note": "sampled at a temperature (medium): equal draws, so tokens agree until rounding moves one across a boundary"
                                if args.workload == "medium" else "greedy: tokens agree until rounding flips a near tie"}
        print(json.dumps(result), flush=True)
        return 0
    if args.parity:
        print(json.dumps(parity(args.layers or XL["n_layer"])), flush=True)
        return 0
    if args.kernel_case:
        from bench_kernel_cases import time_case
        print(json.dumps(time_case(args.kernel_case, args.case_iters, graph=args.case_graph)), flush=True)
        return 0
    if args.warmup < 3:
        args.warmup = 3
    if PROMPT + args.warmup + args.steps + 4 > XL["n_positions"]:
        args.steps = XL["n_positions"] - PROMPT - args.warmup - 4
    import torch
    config = dict(XL)
    layers = args.layers or XL["n_layer"]
    config["n_layer"] = layers
    vocab = config["vocab_size"]
    peak, peak_source = peaks()

    runtime = make_runtime(config, args.batch, use_graph=not args.no_graph)
    engine = runtime.engine
    with ClockSampler() as clocks:
        ms, step_bytes, launches_per_step = decode_device_timed(engine, args.batch, args.warmup, args.steps, vocab)
    clock_summary = clocks.summary()
    e2e_value, h2d, d2h = decode_end_to_end(runtime, args.batch, args.warmup, args.steps, vocab)
    prefill_ms = prefill_timed(engine, vocab)
    flops = prefill_flops(config, layers)
    del runtime, engine
    torch.cuda.empty_cache()

    points = {}
    if not args.no_points:
        for batch in (1, 64):
            rt = make_runtime(config, batch, use_graph=not args.no_graph)
            steps = min(args.steps, 128)
            point_ms, _, _ = decode_device_timed(rt.engine, batch, args.warmup, steps, vocab)
            points[f"decode_b{batch}"] = round(batch * 1000.0 / point_ms, 1)
            if batch == 64:
                # the cache-dominated end: 64 requests at context 1,000 -> 1,020
                for r in list(rt.engine.live_requests()):
                    rt.engine.finish(r)
                long_ms, long_bytes, _ = decode_device_timed(rt.engine, batch, 3, 16, vocab, prompt_len=1000)
                points["decode_b64_ctx1000"] = round(batch * 1000.0 / long_ms, 1)
                points["decode_b64_ctx1000_hbm_frac"] = round(long_bytes / (long_ms * 1e-3) / 1e9 / peak["hbm_gbs"], 4)
            del rt
            torch.cuda.empty_cache()
        # a longer prefill than the model's own positions allow: the same layers with a position table of 4,096 rows
        # (a bench-only configuration), four prompts of 4,096 tokens in one step
        long_config = {**config, "n_positions": 4096}
        rt = make_runtime(long_config, 4, use_graph=False)
        long_ms = prefill_timed(rt.engine, vocab, repeats=3, prompts=4, length=4096)
        points["prefill_4x4096"] = round(4 * 4096 * 1000.0 / long_ms, 1)
        points["prefill_4x4096_frac"] = round(prefill_flops(long_config, layers, 4096, 4) / (long_ms * 1e-3) / (peak["bf16_tflops"] * 1e12), 4)
        del rt
        torch.cuda.empty_cache()
        # the same decode step in true 32-bit (float32 weights and cache, CUDA-core products): the reference's only mode
        rt = make_runtime(config, args.batch, dtype="float32")
        f32_ms, _, _ = decode_device_timed(rt.engine, args.batch, 3, 10, vocab)
        points[f"decode_b{args.batch}_float32"] = round(args.batch * 1000.0 / f32_ms, 1)
        del rt
        torch.cuda.empty_cache()
        if layers == XL["n_layer"]:
            for name in sorted(WORKLOADS):          # the scheduler under mixed loads (generated tokens a second)
                points[f"workload_{name}"] = run_workload(name)["value"]
                torch.cuda.empty_cache()

    achieved = step_bytes / (ms * 1e-3) / 1e9
    line = {
        "metric": f"decode tok/s at batch {args.batch} (GPT-2 XL shape, prompts of {PROMPT}, timed steps at context "
                  f"{PROMPT + args.warmup + 1}->{PROMPT + args.warmup + args.steps})",
        "value": round(args.batch * 1000.0 / ms, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": line_config(layers, args.batch, not args.no_graph),
        "engine": {"page_size": 16, "weights": "random bf16", "cache": "bf16", "peaks": peak_source,
                   "context_timed": f"{PROMPT + args.warmup + 1}-{PROMPT + args.warmup + args.steps}",
                   "bytes_per_step": int(step_bytes), "path": "Engine.step replayed from a CUDA graph; e2e through the scheduler"},
        "prefill": {"value": round(2048 * 1000.0 / prefill_ms, 1), "tokens": 2048, "ms": round(prefill_ms, 3),
                    "frac": round(flops / (prefill_ms * 1e-3) / (peak["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peak["hbm_gbs"], 4)},
        "points": points,
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clock_summary,
    }
    print(json.dumps(line), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
