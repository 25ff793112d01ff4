"""The allocation-free planning entry point against the regular one.

msc_moe_plan_noalloc exists for hosts that must not allocate device memory when they plan a
batch (a frozen memory pool, a framework that owns every allocation); it keeps its ticket
counter in an array built into the library instead of taking scratch from the caller.  This
file is collected last on purpose: if it fails under `-x`, everything else has already run.
Both entry points are called through the C ABI on two different batches in a row and must
agree exactly (they produce integers)."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _plan(lib, fn_name, ids, first, local, scratch=None):
    from mosaicist_b200 import _lib

    entries = ids.numel()
    rank = torch.full((entries,), -9, dtype=torch.int32, device="cuda")
    rows = torch.full((local,), -9, dtype=torch.int32, device="cuda")
    offs = torch.full((local,), -9, dtype=torch.int32, device="cuda")
    tot = torch.full((1,), -9, dtype=torch.int32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    args = [ids.data_ptr(), entries, first, local, rank.data_ptr(), rows.data_ptr(), offs.data_ptr(),
            tot.data_ptr()]
    if scratch is not None:
        args.append(scratch.data_ptr())
    _lib.check(getattr(lib, fn_name)(*args, st))
    torch.cuda.synchronize()
    return [t.cpu().numpy() for t in (rank, rows, offs, tot)]


def test_noalloc_plan_matches_regular_plan_twice_in_a_row():
    from mosaicist_b200 import _lib

    lib = _lib.load()
    scratch = torch.zeros(4, dtype=torch.int32, device="cuda")
    for call, (tokens, experts, k, first, local) in enumerate([(500, 64, 4, 16, 32), (123, 256, 8, 0, 256)]):
        g = torch.Generator(device="cuda").manual_seed(call)
        ids = torch.randint(0, experts, (tokens * k,), dtype=torch.int32, device="cuda", generator=g)
        want = _plan(lib, "msc_moe_plan", ids, first, local, scratch)
        got = _plan(lib, "msc_moe_plan_noalloc", ids, first, local)
        for a, b in zip(got, want):
            assert np.array_equal(a, b)
        assert want[1].sum() > 0 and want[3][0] % 128 == 0        # the comparison is not vacuous
        # counts and total may stay inside the library: NULL outputs are accepted
        rank = torch.empty(ids.numel(), dtype=torch.int32, device="cuda")
        offs = torch.empty(local, dtype=torch.int32, device="cuda")
        _lib.check(lib.msc_moe_plan_noalloc(ids.data_ptr(), ids.numel(), first, local, rank.data_ptr(),
                                            None, offs.data_ptr(), None,
                                            torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        assert np.array_equal(offs.cpu().numpy(), want[2])


def test_noalloc_plan_rejects_more_experts_than_the_builtin_area_holds():
    from mosaicist_b200 import _lib

    lib = _lib.load()
    ids = torch.zeros(8, dtype=torch.int32, device="cuda")
    out = torch.zeros(2048, dtype=torch.int32, device="cuda")
    rc = lib.msc_moe_plan_noalloc(ids.data_ptr(), 8, 0, 1025, out.data_ptr(), out.data_ptr(),
                                  out.data_ptr(), out.data_ptr(), None)
    assert rc == _lib.ERR_BAD_ARG and b"1024" in lib.msc_last_error()
