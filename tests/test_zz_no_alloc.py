"""The scratch-free top-1 entry point against the regular one.

ts_top_1_static exists for hosts that cannot give a kernel scratch memory (a runtime whose device
buffers were all fixed at plan time, a process with no memory budget left): it keeps its scratch
inside the library.  Its ids are integers and must equal ts_top_k's (k = 1) and the CPU checker's exactly.  Two calls in a
row share that built-in scratch, so the second must not be disturbed by what the first left there.
This file sorts last on purpose: a run that stops at the first failure has then already run
everything else.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _static_top1(x: torch.Tensor) -> np.ndarray:
    from tessera_b200 import _lib
    rows, width = x.shape
    ids = torch.empty(rows, dtype=torch.int32, device=x.device)
    code = _lib.TS_F32 if x.dtype == torch.float32 else _lib.TS_BF16
    _lib.check(_lib.lib.ts_top_1_static(C.c_void_p(x.data_ptr()), code, C.c_void_p(ids.data_ptr()), rows, width,
                                        C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    torch.cuda.synchronize()
    return ids.cpu().numpy().view(np.uint32)


def _regular_top1(x: torch.Tensor) -> np.ndarray:
    from tessera_b200 import ops
    ids = ops.top_k(x, 1)
    torch.cuda.synchronize()
    return ids.cpu().numpy().view(np.uint32).reshape(-1)


def test_two_calls_in_a_row_match_the_workspace_entry_point():
    rng = np.random.default_rng(31)
    # first call: many rows over the vocabulary; second: fewer rows and a narrower width, so stale
    # pairs from the first call sit in the scratch beside the ones the second call writes
    first = torch.from_numpy(rng.standard_normal((64, 151936), dtype=np.float32)).cuda()
    first[5, 100] = first[5, 140000] = 50.0   # a tie across parts: the lower index wins
    first[9, :] = float("-inf")               # nothing ranks: the spare value is the width
    second = torch.from_numpy(rng.standard_normal((7, 20000), dtype=np.float32)).cuda().to(torch.bfloat16)
    got_first = _static_top1(first)
    got_second = _static_top1(second)
    assert np.array_equal(got_first, _regular_top1(first))
    assert np.array_equal(got_second, _regular_top1(second))
    assert got_first[5] == 100 and got_first[9] == 151936
    import oracle as O
    assert np.array_equal(got_first, O.top_k(first.cpu().numpy(), 1).reshape(-1))
    assert np.array_equal(got_second, O.top_k(second.float().cpu().numpy(), 1).reshape(-1))


def test_narrow_rows_and_dependent_launch():
    # widths below the 64 parts a row is cut into (most parts empty), and a call with programmatic dependent
    # launch switched on: both must still equal the workspace entry point and the checker
    import oracle as O
    from tessera_b200 import ops
    rng = np.random.default_rng(32)
    for width, pdl in ((5, False), (63, False), (40, True), (3000, True)):
        x = torch.from_numpy(rng.standard_normal((9, width), dtype=np.float32)).cuda()
        x[2, :] = 1.5                               # a whole row of ties: index 0 wins
        ops.set_pdl(pdl)
        try:
            got = _static_top1(x)
            again = _static_top1(x)
        finally:
            ops.set_pdl(False)
        assert np.array_equal(got, again) and got[2] == 0
        assert np.array_equal(got, _regular_top1(x))
        assert np.array_equal(got, O.top_k(x.cpu().numpy(), 1).reshape(-1))


def test_too_many_rows_are_refused():
    from tessera_b200 import TesseraError
    x = torch.zeros((1025, 64), dtype=torch.float32, device="cuda")
    with pytest.raises(TesseraError) as e:
        _static_top1(x)
    assert e.value.code == 3 and "1024" in str(e.value)
