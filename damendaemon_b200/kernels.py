"""Python face of the hand-written CUDA kernels (ctypes over the extern "C" launchers).

Every function takes CUDA tensors and launches on the current stream. There is no CPU
path and no library stand-in: a tensor that is not on a CUDA device, or a library that
cannot be built or loaded, raises ``KernelError``.
"""
from __future__ import annotations

import ctypes
import threading

import torch

from .csrc import build

F32, BF16 = 0, 1
ACTIVATIONS = {None: 0, "none": 0, "gelu_new": 1, "gelu": 2}

_c_int, _c_float, _c_void = ctypes.c_int, ctypes.c_float, ctypes.c_void_p


class KernelError(RuntimeError):
    pass


_SIGNATURES = {
    "core": {
        "dd_device_arch": [],
        "dd_copy_to_device": [_c_void, _c_void, ctypes.c_longlong, _c_void],
        "dd_embed": [_c_void] * 5 + [_c_int] * 5 + [_c_void, _c_void],
        "dd_layernorm": [_c_void] * 5 + [_c_int, _c_int, _c_float, _c_int, _c_void],
        "dd_gemm_simt": [_c_void, _c_int, _c_void, _c_int, _c_void, _c_void, _c_int, _c_void, _c_int] + [_c_int] * 6 + [_c_void],
        "dd_kv_store": [_c_void, _c_void, _c_int, _c_void, _c_void, _c_void, _c_int, _c_void] + [_c_int] * 6 + [_c_void, _c_void],
        "dd_attention_rows": [_c_void, _c_int, _c_void, _c_void, _c_void, _c_void, _c_int, _c_void, _c_int, _c_void, _c_void]
                             + [_c_int] * 7 + [_c_float, _c_int, _c_int, _c_void, _c_void],
        "dd_sample": [_c_void, _c_int, _c_int, _c_int] + [_c_void] * 6,
        "dd_adjust_logits": [_c_void, _c_int, _c_int] + [_c_void] * 8 + [_c_int, _c_void],
    },
    "tensor": {
        "dd_gemm_tcgen05_plan": [_c_int, _c_int, _c_int, _c_int, _c_void, _c_void],
        "dd_wait_probe": [ctypes.c_ulonglong, _c_void, _c_void, _c_void],
        "dd_attention_decode_supported": [_c_int] * 4,
        "dd_attention_prefill_supported": [_c_int] * 4,
        "dd_attention_prefill": [_c_void, _c_int, _c_void, _c_void, _c_void, _c_int, _c_int, _c_void, _c_int, _c_void, _c_int]
                                + [_c_int] * 6 + [_c_float, _c_void, _c_void],
        "dd_attention_prefill_tcgen05_supported": [_c_int] * 5,
        "dd_attention_prefill_tcgen05": [_c_void, _c_int, _c_void, _c_void, _c_int, _c_void, _c_void, _c_void, _c_int, _c_int, _c_void, _c_int, _c_void, _c_int]
                                        + [_c_int] * 6 + [_c_float, _c_void, _c_void],
        "dd_attention_decode_pages_supported": [_c_int] * 5,
        "dd_attention_decode_pages_splits": [_c_int] * 5,
        "dd_attention_decode_pages": [_c_void, _c_int, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_void, _c_int,
                                      _c_void, _c_void, _c_void] + [_c_int] * 7 + [_c_float, _c_int, _c_void, _c_void],
        "dd_attention_decode": [_c_void, _c_int, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_void, _c_int,
                                _c_void, _c_void, _c_void] + [_c_int] * 7 + [_c_float, _c_int, _c_void, _c_void],
        "dd_gemm_tcgen05": [_c_void, _c_int, _c_void, _c_int, _c_void, _c_void, _c_int, _c_void, _c_int] + [_c_int] * 8
                           + [_c_void, _c_void, _c_int, _c_void, ctypes.c_longlong, _c_void, _c_void],
    },
}

_libs, _lock = {}, threading.Lock()


def library(name):
    """Load (building first if needed) one of the kernel libraries."""
    lib = _libs.get(name)
    if lib is not None:
        return lib
    with _lock:
        if name in _libs:
            return _libs[name]
        try:
            path = build.build_library(name)
            lib = ctypes.CDLL(str(path))
        except (build.BuildError, OSError) as error:
            raise KernelError(f"the '{name}' CUDA kernels are not available ({error}); "
                              "this engine has no CPU or library fallback") from error
        lib.dd_last_error.restype = ctypes.c_char_p
        lib.dd_set_pdl.argtypes, lib.dd_set_pdl.restype = [_c_int], _c_int
        lib.dd_set_pdl(1 if _pdl else 0)
        for fn, args in _SIGNATURES[name].items():
            f = getattr(lib, fn)
            f.argtypes, f.restype = args, _c_int
        _libs[name] = lib
        return lib


launches = 0          # kernels launched through this module (what the bench reports as gpu_launches)


def set_pdl(enabled):
    """Programmatic dependent launch for every kernel of both libraries (on by default)."""
    for name in list(_libs):
        _libs[name].dd_set_pdl(1 if enabled else 0)
    global _pdl
    _pdl = bool(enabled)


_pdl = True


class pdl_scope:
    """Kernels launched inside run with programmatic dependent launch on or off; the setting that was in force comes
    back afterwards. The float32 engine turns it off: its kernels (hundreds of blocks of CUDA-core work, no prologue
    worth starting early) were measured to run a decode step of 12 GPT-2 XL layers in 2.2 ms without it and in 2.6
    to 4.3 ms with it, while the bfloat16 kernels gain from it everywhere (1.78 against 2.34 ms for 48 layers)."""

    def __init__(self, enabled):
        self.enabled = bool(enabled)

    def __enter__(self):
        self.before = _pdl
        if self.enabled != self.before:
            set_pdl(self.enabled)

    def __exit__(self, *exc):
        if _pdl != self.before:
            set_pdl(self.before)
        return False


def _call(lib, fn, *args, n_kernels=1):
    global launches
    launches += n_kernels
    code = getattr(lib, fn)(*args)
    if code:
        raise KernelError(lib.dd_last_error().decode())


_scoped_stream = None


def _stream():
    return _scoped_stream if _scoped_stream is not None else torch.cuda.current_stream().cuda_stream


class stream_scope:
    """Every kernel launched inside the scope goes to the stream that was current when the scope was entered, looked
    up once: asking torch for the current stream costs a few microseconds, and a step launches hundreds of kernels.
    (Enter it inside a graph capture, not around it: the capture switches streams.)"""

    def __enter__(self):
        global _scoped_stream
        self.outer, _scoped_stream = _scoped_stream, torch.cuda.current_stream().cuda_stream
        return self

    def __exit__(self, *exc):
        global _scoped_stream
        _scoped_stream = self.outer
        return False


def _dt(t):
    if t is torch.float32 or t == torch.float32:
        return F32
    if t == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported element type {t}")


def _ptr(t, name="tensor", dtype=None):
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError(f"{name} is on {t.device}; the kernels run on CUDA only (no CPU fallback)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, is {t.dtype}")
    return t.data_ptr()


def _rows(t, name):
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{name} must be 2-D with contiguous rows, has shape {tuple(t.shape)} strides {t.stride()}")
    return t


_error_flags = {}


def error_flag(device):
    """One int32 per device that kernels OR error bits into (1 bad token/position, 2 bad page
    on store, 4 bad page on read, 8 a bounded wait ran out)."""
    key = torch.device(device).index or 0
    if key not in _error_flags:
        _error_flags[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _error_flags[key]


def copy_to_device(dst, src, n_bytes):
    """One asynchronous host-to-device copy on the current stream, from pinned memory (src) into dst: the step's
    metadata. Not counted as a kernel launch."""
    global launches
    _call(library("core"), "dd_copy_to_device", dst.data_ptr(), src.data_ptr(), int(n_bytes), _stream(), n_kernels=0)


def read_error_flag(device):
    flag = error_flag(device)
    value = int(flag.item())
    if value:
        clear_after_error(device, value)
    return value


def clear_after_error(device, bits):
    """Zero the device's error word (in stream order) and, after a wait that ran out (bit 8), the split counters:
    a kernel that gave up may have left one short of its reset."""
    error_flag(device).zero_()
    key = torch.device(device).index or 0
    if bits & 8 and key in _counters:
        _counters[key].zero_()


def wait_probe(limit_ns, device):
    """Launch the block whose barrier nobody arrives at (csrc/wait_probe.cu) with a wait limit of limit_ns and
    return how long its two waiting warps waited, in ns. The device's error word then has bit 8 set, as after a
    wait that ran out in a pipelined kernel; read_error_flag reads and clears it."""
    waited = torch.zeros(2, dtype=torch.int64, device=device)
    _call(library("tensor"), "dd_wait_probe", int(limit_ns), _ptr(error_flag(device)), waited.data_ptr(), _stream())
    return waited.tolist()


# ---------------------------------------------------------------- kernels

def embed(ids, positions, token_table, position_table=None, out=None):
    n, width = ids.numel(), token_table.shape[1]
    if out is None:
        out = torch.empty((n, width), dtype=torch.float32, device=ids.device)
    if position_table is not None and position_table.dtype != token_table.dtype:
        raise KernelError("token and position tables must have one dtype")
    _call(library("core"), "dd_embed", _ptr(ids, "ids", torch.int32), _ptr(positions, "positions", torch.int32),
          _ptr(token_table, "token table"), _ptr(position_table, "position table"), _ptr(out, "out", torch.float32),
          n, width, token_table.shape[0], 0 if position_table is None else position_table.shape[0],
          _dt(token_table.dtype), _ptr(error_flag(ids.device)), _stream())
    return out


def layernorm(x, gamma, beta, eps, out_dtype, row_index=None, out=None):
    _rows(x, "x")
    rows = x.shape[0] if row_index is None else row_index.numel()
    width = x.shape[1]
    if not x.is_contiguous():
        raise KernelError("layernorm input must be contiguous")
    if out is None:
        out = torch.empty((rows, width), dtype=out_dtype, device=x.device)
    _call(library("core"), "dd_layernorm", _ptr(x, "x", torch.float32), _ptr(row_index, "row_index", torch.int32),
          _ptr(gamma, "gamma", torch.float32), _ptr(beta, "beta", torch.float32), _ptr(out, "out", out_dtype),
          rows, width, float(eps), _dt(out_dtype), _stream())
    return out


def gemm_simt(a, w, bias=None, residual=None, activation=None, out_dtype=None, out=None):
    """act(a @ w.T + bias) (+ residual) with CUDA-core float32 multiply-add. a [M,K], w [N,K]."""
    _rows(a, "a"), _rows(w, "w")
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or a.dtype != w.dtype:
        raise KernelError(f"gemm: a {tuple(a.shape)} {a.dtype} does not fit w {tuple(w.shape)} {w.dtype}")
    out_dtype = out_dtype or a.dtype
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    _rows(out, "out")
    if residual is not None:
        _rows(residual, "residual")
    _call(library("core"), "dd_gemm_simt", _ptr(a, "a"), a.stride(0), _ptr(w, "w"), w.stride(0),
          _ptr(bias, "bias", torch.float32), _ptr(residual, "residual", torch.float32),
          0 if residual is None else residual.stride(0), _ptr(out, "out", out_dtype), out.stride(0),
          M, N, K, ACTIVATIONS[activation], _dt(a.dtype), _dt(out_dtype), _stream())
    return out


def kv_store(k, v, token_entry, positions, block_table, cache, n_tokens=None):
    """k, v: [N, kv_heads*head_dim] views (row stride free); cache [pages, 2, kv_heads, page, head_dim]."""
    n_pages, _, kv_heads, page_size, head_dim = cache.shape
    if k.stride(0) != v.stride(0) or k.stride(1) != 1 or v.stride(1) != 1 or k.dtype != cache.dtype:
        raise KernelError("kv_store: k and v must be row views of one buffer in the cache dtype")
    if k.shape[1] != kv_heads * head_dim or not cache.is_contiguous():
        raise KernelError("kv_store: shapes do not fit the cache")
    _call(library("core"), "dd_kv_store", _ptr(k, "k"), _ptr(v, "v"), k.stride(0),
          _ptr(token_entry, "token_entry", torch.int32), _ptr(positions, "positions", torch.int32),
          _ptr(block_table, "block_table", torch.int32), block_table.shape[1], _ptr(cache, "cache"),
          n_pages, kv_heads, page_size, head_dim, k.shape[0] if n_tokens is None else n_tokens, _dt(cache.dtype),
          _ptr(error_flag(k.device)), _stream())


def attention_rows(q, cache, token_entry, positions, block_table, n_heads, scale, window=None, n_splits=1, out=None):
    """General paged causal attention. q: [N, n_heads*head_dim] view; returns [N, n_heads*head_dim]."""
    n_pages, _, kv_heads, page_size, head_dim = cache.shape
    n = q.shape[0]
    if q.shape[1] != n_heads * head_dim or q.stride(1) != 1 or q.dtype != cache.dtype or not cache.is_contiguous():
        raise KernelError("attention: q does not fit the cache")
    if out is None:
        out = torch.empty((n, n_heads * head_dim), dtype=q.dtype, device=q.device)
    part_o = part_ml = None
    if n_splits > 1:
        part_o = torch.empty((n * n_heads * n_splits * head_dim,), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n * n_heads * n_splits * 2,), dtype=torch.float32, device=q.device)
    _call(library("core"), "dd_attention_rows", _ptr(q, "q"), q.stride(0), _ptr(cache, "cache"),
          _ptr(token_entry, "token_entry", torch.int32), _ptr(positions, "positions", torch.int32),
          _ptr(block_table, "block_table", torch.int32), block_table.shape[1], _ptr(out, "out"), out.stride(0),
          _ptr(part_o), _ptr(part_ml), n, n_heads, kv_heads, head_dim, page_size, n_pages,
          0 if window is None else int(window), float(scale), int(n_splits), _dt(q.dtype),
          _ptr(error_flag(q.device)), _stream(), n_kernels=2 if n_splits > 1 else 1)
    return out


def sample(logits, temperature=None, uniform=None, top_k=None, top_p=None, out=None):
    """Row-wise token choice: argmax where temperature is 0 (or None), else an inverse-CDF draw
    with the given uniform numbers over the tokens that top_k and top_p keep. Returns int32 ids,
    -1 for rows without a finite maximum."""
    _rows(logits, "logits")
    rows, vocab = logits.shape
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    if temperature is not None and uniform is None:
        raise KernelError("sampling with a temperature needs uniform draws")
    _call(library("core"), "dd_sample", _ptr(logits, "logits", torch.float32), logits.stride(0), rows, vocab,
          _ptr(temperature, "temperature", torch.float32), _ptr(top_k, "top_k", torch.int32),
          _ptr(top_p, "top_p", torch.float32), _ptr(uniform, "uniform", torch.float64),
          _ptr(out, "out", torch.int32), _stream())
    return out


def adjust_logits(logits, item_row, item_token, item_count, item_bias, item_seen, repetition, frequency, presence):
    """In place: penalties and bias on the listed (row, token) pairs (each pair listed once)."""
    _rows(logits, "logits")
    _call(library("core"), "dd_adjust_logits", _ptr(logits, "logits", torch.float32), logits.stride(0), logits.shape[1],
          _ptr(item_row, "item_row", torch.int32), _ptr(item_token, "item_token", torch.int32),
          _ptr(item_count, "item_count", torch.float32), _ptr(item_bias, "item_bias", torch.float32),
          _ptr(item_seen, "item_seen", torch.int32), _ptr(repetition, "repetition", torch.float32),
          _ptr(frequency, "frequency", torch.float32), _ptr(presence, "presence", torch.float32),
          item_row.numel(), _stream())
    return logits


_counters = {}
_sm_count = {}


def _tile_counters(device, n):
    key = torch.device(device).index or 0
    if key not in _counters or _counters[key].numel() < n:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError(f"{n} split counters are needed during a graph capture; size them before (kernels._tile_counters)")
        _counters[key] = torch.zeros(max(n, 8192), dtype=torch.int32, device=device)
    return _counters[key]


def sm_count(device):
    key = torch.device(device).index or 0
    if key not in _sm_count:
        _sm_count[key] = torch.cuda.get_device_properties(device).multi_processor_count
    return _sm_count[key]


_plans = {}


def gemm_tcgen05(a, w, bias=None, residual=None, activation=None, out_dtype=None, out=None, splits=None, token_tile=None,
                 cluster=None, prefetch=None):
    """act(a @ w.T + bias) (+ residual) on the tcgen05 tensor cores. a [M,K] and w [N,K] bfloat16,
    bias/residual float32, out bfloat16 or float32. K and the row strides must be multiples of 8.
    splits/token_tile/cluster override the kernel's own plan (cluster 1: reduce the K splits inside a
    thread-block cluster instead of through a workspace; 3: the same with rings of 10 stages, one block per SM,
    token tiles of 16 only; 2: two SMs on a tile of 256 tokens). prefetch: a tensor that a later kernel will
    stream (the next weight matrix of a decode step); this kernel asks L2 to fetch it meanwhile."""
    _rows(a, "a"), _rows(w, "w")
    M, K = a.shape
    N = w.shape[0]
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != K:
        raise KernelError(f"gemm_tcgen05: needs bfloat16 a [M,K] and w [N,K]; got {tuple(a.shape)} {a.dtype}, {tuple(w.shape)} {w.dtype}")
    out_dtype = out_dtype or torch.bfloat16
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    _rows(out, "out")
    lib = library("tensor")
    plan = _plans.get((M, N, K))
    if plan is None:
        tile, mode = ctypes.c_int(0), ctypes.c_int(0)
        planned = lib.dd_gemm_tcgen05_plan(M, N, K, sm_count(a.device), ctypes.byref(tile), ctypes.byref(mode))
        plan = _plans[(M, N, K)] = (planned, tile.value, mode.value)
    if splits is not None and cluster is None:
        cluster = 0
    splits = plan[0] if splits is None else splits
    token_tile = plan[1] if token_tile is None else token_tile
    cluster = plan[2] if cluster is None else int(cluster)
    workspace = counters = None
    n_counters = 0
    if splits > 1 and not cluster:
        workspace = torch.empty((splits * M * N,), dtype=torch.float32, device=a.device)
        n_counters = ((N + 127) // 128) * ((M + token_tile - 1) // token_tile)
        counters = _tile_counters(a.device, n_counters)
    _call(lib, "dd_gemm_tcgen05", _ptr(a, "a"), a.stride(0), _ptr(w, "w"), w.stride(0),
          _ptr(bias, "bias", torch.float32), _ptr(residual, "residual", torch.float32),
          0 if residual is None else residual.stride(0), _ptr(out, "out", out_dtype), out.stride(0), M, N, K,
          ACTIVATIONS[activation], _dt(out_dtype), splits, token_tile, cluster, _ptr(workspace), _ptr(counters), n_counters,
          None if prefetch is None else prefetch.data_ptr(),
          0 if prefetch is None else prefetch.numel() * prefetch.element_size(), _ptr(error_flag(a.device)), _stream())
    return out


def attention_decode_supported(n_heads, kv_heads, head_dim, dtype):
    return dtype == torch.bfloat16 and bool(library("tensor").dd_attention_decode_supported(n_heads, kv_heads, head_dim, BF16))


def attention_decode_pages_supported(n_heads, kv_heads, head_dim, page_size, dtype):
    return dtype == torch.bfloat16 and bool(
        library("tensor").dd_attention_decode_pages_supported(n_heads, kv_heads, head_dim, page_size, BF16))


def attention_decode_pages_splits(n_tokens, n_heads, page_size, context, device):
    """The key split count the page-streaming decode kernel wants for this many tokens and this longest context."""
    return int(library("tensor").dd_attention_decode_pages_splits(n_tokens, n_heads, page_size, context, sm_count(device)))


def attention_decode(q, cache, token_entry, positions, block_table, n_heads, scale, window=None, n_splits=1, out=None,
                     k_new=None, v_new=None, kernel="rows"):
    """Decode attention (one query per token) over a bfloat16 cache. kernel 'rows': a warp copies key rows 16 bytes
    at a time (see attention_decode_supported); 'pages': whole pages of a group of heads by TMA (see
    attention_decode_pages_supported). With k_new/v_new (row views of the buffer q lives in) the step's own keys and
    values are used from there and written into the cache by this kernel; otherwise they must be in the cache already.
    token_entry None: token t belongs to entry t (a step of single tokens in entry order). n_splits: into how many
    pieces a token's keys are cut; for 'pages' the most a token may get (the kernel deals them out by context length)."""
    if kernel not in ("rows", "pages"):
        raise KernelError(f"attention_decode: unknown kernel {kernel!r}")
    n_pages, _, kv_heads, page_size, head_dim = cache.shape
    n = q.shape[0]
    if q.shape[1] != n_heads * head_dim or q.stride(1) != 1 or q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 \
            or not cache.is_contiguous():
        raise KernelError("attention_decode: q does not fit the cache")
    if (k_new is None) != (v_new is None):
        raise KernelError("attention_decode: k_new and v_new come together")
    if k_new is not None and (k_new.stride(0) != q.stride(0) or v_new.stride(0) != q.stride(0) or k_new.stride(1) != 1
                              or v_new.stride(1) != 1 or k_new.dtype != q.dtype or k_new.shape != q.shape):
        raise KernelError("attention_decode: k_new and v_new must be row views like q")
    if out is None:
        out = torch.empty((n, n_heads * head_dim), dtype=q.dtype, device=q.device)
    part_o = part_ml = counters = None
    if n_splits > 1:
        part_o = torch.empty((n * n_heads * n_splits * head_dim,), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n * n_heads * n_splits * 2,), dtype=torch.float32, device=q.device)
        counters = _tile_counters(q.device, n * n_heads)
    _call(library("tensor"), "dd_attention_decode" + ("_pages" if kernel == "pages" else ""), _ptr(q, "q"), q.stride(0),
          _ptr(k_new, "k_new"), _ptr(v_new, "v_new"),
          _ptr(cache, "cache"), _ptr(token_entry, "token_entry", torch.int32), _ptr(positions, "positions", torch.int32),
          _ptr(block_table, "block_table", torch.int32), block_table.shape[1], _ptr(out, "out"), out.stride(0),
          _ptr(part_o), _ptr(part_ml), _ptr(counters), n, n_heads, kv_heads, head_dim, page_size, n_pages,
          0 if window is None else int(window), float(scale), int(n_splits), _ptr(error_flag(q.device)), _stream())
    return out


def attention_prefill_supported(n_heads, kv_heads, head_dim, dtype):
    return dtype == torch.bfloat16 and bool(library("tensor").dd_attention_prefill_supported(n_heads, kv_heads, head_dim, BF16))


def attention_prefill_tcgen05_supported(n_heads, kv_heads, head_dim, page_size, dtype):
    return dtype == torch.bfloat16 and bool(
        library("tensor").dd_attention_prefill_tcgen05_supported(n_heads, kv_heads, head_dim, page_size, BF16))


ATTENTION_PREFILL_TCGEN05_KEY_BLOCK = 128       # keys per block of the tcgen05 prompt attention


def attention_prefill(q, cache, entry_start, entry_pos0, block_table, n_heads, scale, window=None, out=None, kernel="mma",
                      k_new=None, v_new=None, store_new=False):
    """Tensor-core attention for runs of consecutive tokens (prompt portions; a decoded token is a run of one)
    over a bfloat16 cache. entry_start: int32 [E+1], entry_pos0: int32 [E]. kernel: 'mma' (mma.sync tiles of 64
    queries, see attention_prefill_supported) or 'tcgen05' (tiles of 128 queries with TMA and TMEM accumulators,
    see attention_prefill_tcgen05_supported). The cache must hold this step's keys and values already; k_new/v_new
    (row views of the buffer q lives in, the same values) let the tcgen05 kernel read the key blocks that lie wholly
    in this step from there, in one piece per block instead of page by page. store_new: the tcgen05 kernel writes
    k_new/v_new into the cache itself (no kv_store before it); only for steps whose entries all start at a position
    that is a multiple of ATTENTION_PREFILL_TCGEN05_KEY_BLOCK (an entry that does not sets error bit 2)."""
    n_pages, _, kv_heads, page_size, head_dim = cache.shape
    n, n_entries = q.shape[0], entry_pos0.numel()
    if q.shape[1] != n_heads * head_dim or q.stride(1) != 1 or q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 \
            or not cache.is_contiguous() or entry_start.numel() != n_entries + 1:
        raise KernelError("attention_prefill: q or the entry arrays do not fit the cache")
    if out is None:
        out = torch.empty((n, n_heads * head_dim), dtype=q.dtype, device=q.device)
    if kernel not in ("mma", "tcgen05"):
        raise KernelError(f"attention_prefill: unknown kernel {kernel!r}")
    if (k_new is None) != (v_new is None) or (k_new is not None and (
            kernel != "tcgen05" or k_new.stride(0) != q.stride(0) or v_new.stride(0) != q.stride(0) or k_new.stride(1) != 1
            or v_new.stride(1) != 1 or k_new.dtype != q.dtype or v_new.dtype != q.dtype
            or k_new.shape != (n, kv_heads * head_dim) or v_new.shape != k_new.shape)):
        raise KernelError("attention_prefill: k_new and v_new come together, as row views like q, for the tcgen05 kernel")
    if store_new and k_new is None:
        raise KernelError("attention_prefill: store_new needs k_new and v_new")
    new_rows = (_ptr(k_new, "k_new"), _ptr(v_new, "v_new"), int(bool(store_new))) if kernel == "tcgen05" else ()
    _call(library("tensor"), "dd_attention_prefill" + ("_tcgen05" if kernel == "tcgen05" else ""), _ptr(q, "q"), q.stride(0), *new_rows,
          _ptr(cache, "cache"),
          _ptr(entry_start, "entry_start", torch.int32), _ptr(entry_pos0, "entry_pos0", torch.int32), n_entries, n,
          _ptr(block_table, "block_table", torch.int32), block_table.shape[1], _ptr(out, "out"), out.stride(0),
          n_heads, kv_heads, head_dim, page_size, n_pages, 0 if window is None else int(window), float(scale),
          _ptr(error_flag(q.device)), _stream())
    return out
