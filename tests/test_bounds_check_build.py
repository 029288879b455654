"""The bounds-checked debug build of the native library (``python -m cornstarch_b200.csrc.build --bounds-check``):
kernels that take an index from DATA (embedding ids / feature rows of the merge kernels, rotary positions, source rows
of the expert dispatch) compare it with the extent their entry point was given, record a code and skip the access.

The test loads the debug library next to the release one, runs small valid cases (no record), then hands each kernel
one out-of-range index: the record names the kind of violation, the output row of the bad index is left untouched and
the device keeps working.  Nothing faults: the bad index never reaches memory.  The check that the loaded library
really is the checked build comes first (an unchecked build would make the bad index a real out-of-bounds access, so
those cases are skipped instead)."""

import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

vp, i32, i64, f32 = C.c_void_p, C.c_int, C.c_long, C.c_float


def _dbg():
    from cornstarch_b200.csrc.build import DEBUG_LIB_PATH

    if not DEBUG_LIB_PATH.exists():
        pytest.skip("debug library not built (python -m cornstarch_b200.csrc.build --bounds-check)")
    lib = C.CDLL(str(DEBUG_LIB_PATH))
    lib.csb_gather_merge.argtypes = [vp, vp, vp, vp, i64, i32, i64, i64, vp]
    lib.csb_rope.argtypes = [vp, vp, vp, vp, i64, i32, i32, i32, i32, i32, f32, i32, vp]
    lib.csb_moe_push.argtypes = [vp, vp, i64, i32, vp, vp, i32, i64, vp]
    for name in ("csb_gather_merge", "csb_rope", "csb_moe_push", "csb_bounds_status", "csb_bounds_check_enabled"):
        getattr(lib, name).restype = C.c_int
    if lib.csb_bounds_check_enabled() != 1:
        pytest.skip("the library at the debug path was built without -DCSB_BOUNDS_CHECK")
    return lib


def _stream():
    return torch.cuda.current_stream().cuda_stream


def test_valid_indices_leave_no_record_and_match_the_release_build():
    from cornstarch_b200.ops import elementwise as E

    lib = _dbg()
    emb = torch.randn(50, 64, device="cuda").bfloat16()
    feats = torch.randn(7, 64, device="cuda").bfloat16()
    src = torch.tensor([0, 49, -1, -7, 3, 3], dtype=torch.int32, device="cuda")
    out = torch.empty(6, 64, device="cuda", dtype=torch.bfloat16)
    assert lib.csb_gather_merge(emb.data_ptr(), feats.data_ptr(), src.data_ptr(), out.data_ptr(), 6, 64, 50, 7, _stream()) == 0
    assert lib.csb_bounds_status() == 0
    want = E.embed_merge(emb, src, feats)  # the release build through the package
    assert torch.equal(out, want)


def test_out_of_range_indices_are_recorded_and_skipped():
    lib = _dbg()
    emb = torch.randn(50, 64, device="cuda").bfloat16()
    feats = torch.randn(7, 64, device="cuda").bfloat16()
    # embedding id beyond the table, then a feature row beyond the feature matrix
    for bad, code in ((50, 101), (-8, 102)):
        src = torch.tensor([1, bad, 2], dtype=torch.int32, device="cuda")
        out = torch.full((3, 64), 9.0, device="cuda", dtype=torch.bfloat16)
        assert lib.csb_gather_merge(emb.data_ptr(), feats.data_ptr(), src.data_ptr(), out.data_ptr(), 3, 64, 50, 7, _stream()) == 0
        assert lib.csb_bounds_status() == code
        assert lib.csb_bounds_status() == 0  # reading clears the record
        assert torch.equal(out[0], emb[1]) and torch.equal(out[2], emb[2]) and bool((out[1] == 9.0).all())
    # rotary position beyond the cos / sin tables
    D, rows = 32, 16
    cos = torch.ones(rows, D // 2, device="cuda")
    sin = torch.zeros(rows, D // 2, device="cuda")
    buf = torch.randn(1, 4, D, device="cuda").bfloat16()
    before = buf.clone()
    pos = torch.tensor([0, 5, 16, 3], dtype=torch.int32, device="cuda")
    assert lib.csb_rope(buf.data_ptr(), cos.data_ptr(), sin.data_ptr(), pos.data_ptr(), 4, 4, D, 1, D, D, 1.0, rows, _stream()) == 0
    assert lib.csb_bounds_status() == 103
    assert torch.equal(buf, before)  # cos 1 / sin 0 leaves valid rows as they were; the bad row was not touched either
    # expert dispatch: a source row beyond the token matrix
    x = torch.randn(10, 64, device="cuda").bfloat16()
    idx = torch.tensor([0, 10, 9], dtype=torch.int32, device="cuda")
    dst = torch.zeros(3, 64, device="cuda", dtype=torch.bfloat16)
    seg = (i32 * 9)(0, 3, 3, 3, 3, 3, 3, 3, 3)
    dsts = (vp * 1)(dst.data_ptr())
    assert lib.csb_moe_push(x.data_ptr(), idx.data_ptr(), 3, 64, C.cast(seg, vp), C.cast(dsts, vp), 1, 10, _stream()) == 0
    assert lib.csb_bounds_status() == 104
    assert torch.equal(dst[0], x[0]) and torch.equal(dst[2], x[9]) and bool((dst[1] == 0).all())
    # the device is intact
    assert float((torch.ones(8, device="cuda") * 2).sum()) == 16.0
