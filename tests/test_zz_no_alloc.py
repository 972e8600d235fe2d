"""dd_attention_rows_static, the attention entry point that allocates nothing (csrc/no_alloc.h).

Some hosts of these kernels cannot call cudaMalloc when they need attention: they run inside a
fixed memory plan, or in a loop that must not take the allocator's lock. This file calls the
entry point the way such a host does, through the exported C symbol, and holds its output to
the ordinary entry point's (which takes caller-allocated scratch), on two calls in a row with
different inputs, so that what the first call left in the shared scratch cannot leak into the
second. pytest collects this file last (by name), so a run that stops at the first failure has
already run every other test.
"""
import ctypes

import pytest
import torch

from test_gpu_kernels import paged_case

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SCRATCH_BYTES = 8 << 20


@pytest.fixture(scope="module")
def entry():
    from damendaemon_b200 import kernels
    lib = kernels.library("core")
    fn = lib.dd_attention_rows_static
    v, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [v, i, v, v, v, v, i, v, i] + [i] * 7 + [f, i, i, v, v]
    fn.restype = i
    return kernels, lib, fn


def call_static(kernels, lib, fn, c, heads, n_splits, window=None):
    q, cache = c["q"], c["cache"]
    n_pages, _, kv_heads, page, d = cache.shape
    out = torch.empty((q.shape[0], heads * d), dtype=q.dtype, device=q.device)
    code = fn(q.data_ptr(), q.stride(0), cache.data_ptr(), c["ent"].data_ptr(), c["pos"].data_ptr(), c["table"].data_ptr(),
              c["table"].shape[1], out.data_ptr(), out.stride(0), q.shape[0], heads, kv_heads, d, page, n_pages,
              0 if window is None else window, float(c["scale"]), n_splits, kernels._dt(q.dtype),
              kernels.error_flag(q.device).data_ptr(), torch.cuda.current_stream().cuda_stream)
    return code, out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_two_calls_in_a_row_match_the_allocating_entry_point(entry, dtype):
    kernels, lib, fn = entry
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    first = paged_case(kernels, dtype, 4, 2, 64, 16, lengths=[300, 33, 1, 700], new=[1, 1, 1, 1], window=None, n_splits=5, seed=1)
    second = paged_case(kernels, dtype, 6, 3, 48, 8, lengths=[90, 257], new=[2, 1], window=40, n_splits=3, seed=2)
    for case, heads, splits, window in ((first, 4, 5, None), (second, 6, 3, 40)):
        want = kernels.attention_rows(case["q"], case["cache"], case["ent"], case["pos"], case["table"], heads,
                                      case["scale"], window, n_splits=splits)
        code, got = call_static(kernels, lib, fn, case, heads, splits, window)
        assert code == 0, lib.dd_last_error().decode()
        torch.cuda.synchronize()
        assert kernels.read_error_flag(DEV) == 0
        assert (got.float() - want.float()).abs().max().item() <= tol
        assert (got.double().cpu() - case["ref"]).abs().max().item() < tol


def test_refuses_more_than_its_scratch_and_allocates_nothing(entry):
    kernels, lib, fn = entry
    case = paged_case(kernels, torch.float32, 4, 2, 64, 16, lengths=[40], new=[1], window=None, n_splits=2, seed=3)
    call_static(kernels, lib, fn, case, 4, 2)             # the first call on the device has done its set-up
    torch.cuda.synchronize()
    before = torch.cuda.mem_get_info()[0]
    code, _ = call_static(kernels, lib, fn, case, 4, 2)
    torch.cuda.synchronize()
    assert code == 0 and torch.cuda.mem_get_info()[0] == before, "the call changed the device's free memory"
    # 1 token x 4 heads x n_splits x 66 floats: beyond 8 MiB from 7,944 splits on
    too_many = SCRATCH_BYTES // (4 * 66 * 4) + 1
    code, _ = call_static(kernels, lib, fn, case, 4, too_many)
    assert code != 0
    message = lib.dd_last_error().decode()
    assert "scratch" in message and str(SCRATCH_BYTES) in message
    code, _ = call_static(kernels, lib, fn, case, 4, 1)    # without splits no scratch is touched
    assert code == 0
