"""Single kernels at GPT-2 XL shapes, for timing and for profiler captures.

``python bench.py --kernel-case NAME [--case-iters N]`` builds the inputs of one case, runs the
kernel N times back to back (rotating through enough copies of the big operand that the 126 MB
L2 cannot hold them) and prints the time per launch from CUDA events. A profiler is pointed at
the same command with a small N.
"""
from __future__ import annotations

import torch

from damendaemon_b200 import kernels as K

H, D, PAGE = 25, 64, 16
SHAPES = {"qkv": (4800, 1600, "bias"), "proj": (1600, 1600, "residual"), "fc": (6400, 1600, "gelu"),
          "fc2": (1600, 6400, "residual"), "head": (50257, 1600, "none")}


def _gemm_case(name, tokens, dev):
    features, reduction, epilogue = SHAPES[name]
    copies = max(2, min(24, (300 << 20) // (features * reduction * 2)))
    weights = [torch.randn(features, reduction, device=dev).mul_(0.02).to(torch.bfloat16) for _ in range(copies)]
    bias = torch.randn(features, device=dev)
    x = torch.randn(tokens, reduction, device=dev).to(torch.bfloat16)
    stream = torch.zeros(tokens, features, device=dev)
    out16 = torch.empty(tokens, features, device=dev, dtype=torch.bfloat16)

    def run(i):
        w = weights[i % copies]
        if epilogue == "bias":
            K.gemm_tcgen05(x, w, bias, out=out16)
        elif epilogue == "gelu":
            K.gemm_tcgen05(x, w, bias, activation="gelu_new", out=out16)
        elif epilogue == "residual":
            K.gemm_tcgen05(x, w, bias, residual=stream, out_dtype=torch.float32, out=stream)
        else:
            K.gemm_tcgen05(x, w, out_dtype=torch.float32, out=stream)
    work = {"bytes": features * reduction * 2, "flops": 2 * tokens * features * reduction}
    return run, work


def _gemm32_case(name, tokens, dev):
    """The same products in true 32-bit on the CUDA cores (float32 weights, activations and stream)."""
    features, reduction, epilogue = SHAPES[name]
    copies = max(2, min(12, (300 << 20) // (features * reduction * 4)))
    weights = [torch.randn(features, reduction, device=dev).mul_(0.02) for _ in range(copies)]
    bias = torch.randn(features, device=dev)
    x = torch.randn(tokens, reduction, device=dev)
    stream = torch.zeros(tokens, features, device=dev)
    out = torch.empty(tokens, features, device=dev)

    def run(i):
        w = weights[i % copies]
        if epilogue == "residual":
            K.gemm_simt(x, w, bias, residual=stream, out=stream)
        else:
            K.gemm_simt(x, w, bias if epilogue != "none" else None, activation="gelu_new" if epilogue == "gelu" else None, out=out)
    return run, {"bytes": features * reduction * 4, "flops": 2 * tokens * features * reduction}


def _layernorm_case(rows, dev):
    """LayerNorm of `rows` rows of the float32 stream (width 1600) into bfloat16, as before every projection."""
    width = H * D
    copies = max(2, min(24, (300 << 20) // (rows * width * 4)))
    xs = [torch.randn(rows, width, device=dev) for _ in range(copies)]
    gamma, beta = torch.ones(width, device=dev), torch.zeros(width, device=dev)
    out = torch.empty(rows, width, device=dev, dtype=torch.bfloat16)
    run = lambda i: K.layernorm(xs[i % copies], gamma, beta, 1e-5, torch.bfloat16, out=out)
    return run, {"bytes": rows * width * 6, "flops": 8 * rows * width}


def _cache_case(batch, context, dev, copies):
    n_pages = batch * ((context + PAGE - 1) // PAGE)
    caches = [torch.randn(n_pages, 2, H, PAGE, D, device=dev).to(torch.bfloat16) for _ in range(copies)]
    table = torch.arange(n_pages, dtype=torch.int32, device=dev).view(batch, -1)
    return caches, table


def _decode_case(batch, context, dev, kernel="pages"):
    copies = max(2, min(12, (300 << 20) // (batch * context * H * D * 4)))
    caches, table = _cache_case(batch, context, dev, copies)
    ent = torch.arange(batch, dtype=torch.int32, device=dev)
    pos = torch.full((batch,), context - 1, dtype=torch.int32, device=dev)
    q = torch.randn(batch, H * D, device=dev).to(torch.bfloat16)
    if kernel == "pages":
        splits = K.attention_decode_pages_splits(batch, H, PAGE, context, dev)
    else:
        splits = max(1, min(-(-(K.sm_count(dev) * 2) // (batch * H)), (context + 127) // 128, 32))
    run = lambda i: K.attention_decode(q, caches[i % copies], ent, pos, table, H, D ** -0.5, None, n_splits=splits, kernel=kernel)
    return run, {"bytes": batch * context * H * D * 4, "flops": 4 * batch * context * H * D}


def _prefill_case(prompts, length, dev, kernel="tcgen05", store=False):
    caches, table = _cache_case(prompts, length, dev, 4)
    start = torch.arange(prompts + 1, dtype=torch.int32, device=dev) * length
    pos0 = torch.zeros(prompts, dtype=torch.int32, device=dev)
    qkv = torch.randn(prompts * length, 3 * H * D, device=dev).to(torch.bfloat16)      # as the fused projection leaves them
    q, k, v = qkv[:, :H * D], qkv[:, H * D:2 * H * D], qkv[:, 2 * H * D:]
    new = {"k_new": k, "v_new": v, "store_new": store} if kernel == "tcgen05" else {}
    run = lambda i: K.attention_prefill(q, caches[i % 4], start, pos0, table, H, D ** -0.5, None, kernel=kernel, **new)
    return run, {"bytes": prompts * length * H * D * 6, "flops": prompts * 4 * (length * (length + 1) // 2) * H * D}


def build(name, device="cuda:0"):
    """name: gemm_<qkv|proj|fc|fc2|head>_m<tokens> | gemm32_<...>_m<tokens> (float32, CUDA cores) | attn_decode_b<batch>[_c<context>] (page streaming) | attn_decode_rows_b<batch>[_c<context>] | attn_prefill_p<prompts>_t<tokens> | attn_prefill | attn_prefill_store (the kernel writes the cache too) | attn_prefill_mma |
    attn_prefill_long (one prompt of 4,096 tokens) | layernorm_m<rows>"""
    K.library("core"), K.library("tensor")
    parts = name.split("_")
    if parts[0] == "gemm" and len(parts) == 3 and parts[1] in SHAPES and parts[2][0] == "m":
        return _gemm_case(parts[1], int(parts[2][1:]), device)
    if parts[0] == "gemm32" and len(parts) == 3 and parts[1] in SHAPES and parts[2][0] == "m":
        return _gemm32_case(parts[1], int(parts[2][1:]), device)
    if name.startswith("layernorm_m"):
        return _layernorm_case(int(name[len("layernorm_m"):]), device)
    if name.startswith("attn_decode_rows_b") or name.startswith("attn_decode_b"):
        # attn_decode[_rows]_b<batch>[_c<context>]: the context is 768 keys unless it is given
        rows = name.startswith("attn_decode_rows_b")
        numbers = name[len("attn_decode_rows_b" if rows else "attn_decode_b"):].split("_c")
        return _decode_case(int(numbers[0]), int(numbers[1]) if len(numbers) > 1 else 768, device, kernel="rows" if rows else "pages")
    if name.startswith("attn_prefill_p"):
        # attn_prefill_p<prompts>_t<tokens>: whole prompts of that many tokens
        prompts, tokens = name[len("attn_prefill_p"):].split("_t")
        return _prefill_case(int(prompts), int(tokens), device)
    if name == "attn_prefill":
        return _prefill_case(2, 1024, device)
    if name == "attn_prefill_store":
        return _prefill_case(2, 1024, device, store=True)
    if name == "attn_prefill_mma":
        return _prefill_case(2, 1024, device, kernel="mma")
    if name == "attn_prefill_long":
        return _prefill_case(1, 4096, device)
    if name == "attn_prefill_long_mma":
        return _prefill_case(1, 4096, device, kernel="mma")
    raise ValueError(f"unknown kernel case {name!r}")


def time_case(name, iters=50, device="cuda:0", graph=False):
    """graph: the launches are captured into one CUDA graph and replayed, so that the host's time per launch (a
    few microseconds of Python) does not stand between two kernels, as it does not in a captured decode step."""
    run, work = build(name, device)
    for i in range(3):
        run(i)
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if graph:
        captured = torch.cuda.CUDAGraph()
        with torch.cuda.graph(captured):
            for i in range(iters):
                run(i)
        captured.replay()
        torch.cuda.synchronize()
        start.record()
        captured.replay()
        stop.record()
    else:
        start.record()
        for i in range(iters):
            run(i)
        stop.record()
    torch.cuda.synchronize()
    us = start.elapsed_time(stop) * 1000.0 / iters
    return {"case": name, "us_per_launch": round(us, 2), "GB_per_s": round(work["bytes"] / us / 1e3, 1),
            "TFLOP_per_s": round(work["flops"] / us / 1e6, 1), "iters": iters, "graph": bool(graph)}
