"""ne_exl3_linear_static, the EXL3 Linear for callers that cannot allocate (allocator hooks, fixed-budget serving
loops, GPUs whose remaining memory belongs to another runtime): its scratch is an array built into the library, so it
must give exactly what ne_exl3_linear gives, call after call, on the shared area. Collected last on purpose: a run
that stops at the first failure has then already run every other test."""
import ctypes as C

import numpy as np
import pytest

from ijah_b200 import packgen

pytestmark = pytest.mark.gpu


def test_static_scratch_linear_matches_the_arena_version_twice():
    import torch
    from ijah_b200 import engine as E
    assert torch.cuda.is_available()
    eng = E.Engine()
    rng = np.random.default_rng(42)
    cap = eng.lib.ne_exl3_linear_static_capacity()
    assert cap == 8 << 20
    # everything that may allocate happens first: weights, inputs, outputs, the arena calls that give the expected results
    # (the arena grows to its final size here), one static call (resolves the array's address)
    cases = []
    for n_in, n_out, K, rows in ((2048, 768, 5, 4), (768, 2048, 6, 16)):
        tr, su, sv = packgen.exl3_linear(rng, n_in, n_out, K)
        lin = E.Exl3Linear(eng, tr, su, sv)
        x = torch.from_numpy(rng.standard_normal((rows, n_in)).astype(np.float16).astype(np.float32)).cuda()
        cases.append((lin, x, lin(x), torch.empty((rows, n_out), device="cuda")))
    lin, x, want, got = cases[0]
    call = lambda lin, x, got: eng.lib.ne_exl3_linear_static(C.byref(lin.c), C.c_void_p(x.data_ptr()), x.shape[0],
                                                             C.c_void_p(got.data_ptr()), None)
    assert call(lin, x, got) == 0, eng.last_error()
    torch.cuda.synchronize()
    # two different shapes back to back on the one shared area, twice each: the second call finds the first call's
    # leftovers. The device's free memory must not move across these calls: the entry point allocates nothing.
    free0 = torch.cuda.mem_get_info()[0]
    for lin, x, want, got in cases + cases:
        got.zero_()
        assert call(lin, x, got) == 0, eng.last_error()
        torch.cuda.synchronize()
        assert torch.equal(got, want)  # same kernels, same plan: bit-identical (the tolerance the other tests use for two runs)
    assert eng.lib.ne_device_wait_status() == 0  # the word the static launches report into
    assert torch.cuda.mem_get_info()[0] == free0, "ne_exl3_linear_static changed the amount of free device memory"
    # a request beyond the built-in area is refused with both sizes in the message, nothing is launched
    tr, su, sv = packgen.exl3_linear(rng, 4096, 4096, 4)
    big = E.Exl3Linear(eng, tr, su, sv)
    x = torch.zeros((64, 4096), device="cuda")
    y = torch.zeros((64, 4096), device="cuda")
    rc = eng.lib.ne_exl3_linear_static(C.byref(big.c), C.c_void_p(x.data_ptr()), 64, C.c_void_p(y.data_ptr()), None)
    assert rc == -1
    assert "built-in area holds" in eng.last_error() and str(cap) in eng.last_error()
    assert eng.lib.ne_device_wait_status() == 0
