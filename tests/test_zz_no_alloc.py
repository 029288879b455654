"""The allocation-free column sum, called through its exported C symbol.

``csb_colsum_noalloc`` serves callers that cannot call cudaMalloc (allocator callbacks, frozen memory
pools, fixed-footprint host processes): it keeps its partial-sum scratch in a fixed device array inside
the library.  The test loads the shared library with ctypes, calls the symbol directly twice in a row on
different inputs (the scratch keeps the first call's contents, which must not leak into the second
result) and compares with the regular ``csb_colsum`` entry point, whose scratch the caller allocates.
It also checks that a width beyond the built-in scratch is refused.  The file name sorts last so that a
run stopping at the first failure has already executed every other test.
"""

import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_H = 8192


def _lib():
    from cornstarch_b200.ops import _native as nat

    raw = C.CDLL(str(nat.lib_path()))
    raw.csb_colsum_noalloc.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
    raw.csb_colsum_noalloc.restype = C.c_int
    raw.csb_colsum.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
    raw.csb_colsum.restype = C.c_int
    raw.csb_colsum_parts.argtypes = [C.c_int]
    raw.csb_colsum_parts.restype = C.c_int
    return raw


def _existing(lib, x, out_dtype, accumulate, init):
    rows, H = x.shape
    parts = lib.csb_colsum_parts(rows)
    scratch = torch.empty(parts * H, dtype=torch.float32, device=x.device)
    out = init.clone()
    rc = lib.csb_colsum(x.data_ptr(), scratch.data_ptr(), out.data_ptr(), int(out_dtype == torch.float32), int(accumulate),
                        rows, H, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    return out


def _noalloc(lib, x, out_dtype, accumulate, init):
    rows, H = x.shape
    out = init.clone()
    rc = lib.csb_colsum_noalloc(x.data_ptr(), out.data_ptr(), int(out_dtype == torch.float32), int(accumulate), rows, H,
                                torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    return out


def test_noalloc_colsum_matches_existing_entry_point_twice_in_a_row():
    lib = _lib()
    torch.manual_seed(0)
    cases = [((3000, 4096), torch.float32, False), ((517, 1152), torch.bfloat16, True)]
    for (rows, H), dt, acc in cases:  # two different calls back to back share the built-in scratch
        x = torch.randn(rows, H, device="cuda").bfloat16()
        init = torch.randn(H, device="cuda").to(dt)
        want = _existing(lib, x, dt, acc, init)
        got = _noalloc(lib, x, dt, acc, init)
        torch.cuda.synchronize()
        ref = x.float().sum(0) + (init.float() if acc else 0)
        tol = 2e-2 * max(1.0, ref.abs().max().item())
        assert (got.float() - want.float()).abs().max().item() <= tol
        assert (got.float() - ref).abs().max().item() <= tol
    # the same input again: identical result although the scratch now holds the previous call's partials
    x = torch.randn(64, 256, device="cuda").bfloat16()
    zero = torch.zeros(256, device="cuda")
    a = _noalloc(lib, x, torch.float32, False, zero)
    b = _noalloc(lib, x, torch.float32, False, zero)
    torch.cuda.synchronize()
    assert torch.equal(a, b)


def test_noalloc_colsum_refuses_oversized_width():
    lib = _lib()
    H = MAX_H + 8
    x = torch.zeros(4, H, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(H, device="cuda")
    rc = lib.csb_colsum_noalloc(x.data_ptr(), out.data_ptr(), 1, 0, 4, H, torch.cuda.current_stream().cuda_stream)
    assert rc == -4
    torch.cuda.synchronize()


def test_noalloc_colsum_refuses_misaligned_input():
    """x is read in 16-byte pieces: a pointer off that boundary (a sliced view handed over as a raw address) is
    refused with CSB_ERR_BAD_ARG before anything is launched, instead of faulting on the GPU."""
    lib = _lib()
    H = 256
    buf = torch.zeros(4 * H + 8, device="cuda", dtype=torch.bfloat16)
    out = torch.full((H,), 7.0, device="cuda")
    rc = lib.csb_colsum_noalloc(buf.data_ptr() + 2, out.data_ptr(), 1, 0, 4, H, torch.cuda.current_stream().cuda_stream)
    assert rc == -1
    rc = lib.csb_colsum_noalloc(buf.data_ptr(), out.data_ptr() + 2, 1, 0, 4, H, torch.cuda.current_stream().cuda_stream)
    assert rc == -1
    torch.cuda.synchronize()
    assert bool((out == 7.0).all())  # nothing ran
