"""The gemv entry point that allocates nothing, against the ordinary one.

`qb200_gemv_blocks_noalloc` serves hosts that own all device memory themselves (an allocation by the
library would bypass their pool and stall the device) by keeping its scratch in an array compiled into
the library.  It must give the bits `qb200_gemv_blocks` gives, call after call, since every call reuses
that one array; and it must refuse, loudly, an x wider than the array holds.

Collected last on purpose: a failure here cannot hide the other tests from a run that stops early.
"""
import ctypes as C

import numpy as np
import pytest

from qiyas_b200 import blocks as B

pytestmark = pytest.mark.gpu


def _run(lib, fn_name, fmt_a, a_dev, x_dev, rows, cols):
    import torch
    y = torch.full((rows,), float("nan"), dtype=torch.float32, device="cuda:0")
    rc = getattr(lib, fn_name)(fmt_a, B.F32, a_dev.data_ptr(), x_dev.data_ptr(), y.data_ptr(), rows, cols, None)
    assert rc == 0, lib.qb200_last_error().decode()
    torch.cuda.synchronize()
    return y.cpu().numpy()


@pytest.mark.parametrize("fmt_a,rows,cols", [(B.Q4_0, 1031, 8192), (B.Q8_0, 517, 4064), (B.Q4_K, 300, 4096), (B.Q6_K, 129, 2304)])
def test_same_bits_as_the_allocating_entry_point_twice_in_a_row(fmt_a, rows, cols):
    import torch
    from qiyas_b200 import _lib
    lib = _lib.load()
    assert lib.qb200_init(0) == 0                      # the ordinary entry point needs it; the new one does not
    a = torch.from_numpy(B.make_weights(fmt_a, rows, cols, 11)).cuda()
    for call, seed in enumerate((12, 13)):             # a second call finds the first call's x in the scratch array
        x = torch.from_numpy(B.make_activations(cols, seed)).cuda()
        want = _run(lib, "qb200_gemv_blocks", fmt_a, a, x, rows, cols)
        got = _run(lib, "qb200_gemv_blocks_noalloc", fmt_a, a, x, rows, cols)
        assert np.isfinite(want).all()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), f"call {call}"
        status = C.c_int(-1)
        assert lib.qb200_gemv_noalloc_status(C.byref(status)) == 0 and status.value == 0


def test_refuses_what_the_static_scratch_cannot_hold():
    import torch
    from qiyas_b200 import _lib
    lib = _lib.load()
    cols = 16384 + 32
    a = torch.zeros(B.nbytes(B.Q8_0, 2 * cols), dtype=torch.uint8, device="cuda:0")
    x = torch.zeros(cols, dtype=torch.float32, device="cuda:0")
    y = torch.zeros(2, dtype=torch.float32, device="cuda:0")
    rc = lib.qb200_gemv_blocks_noalloc(B.Q8_0, B.F32, a.data_ptr(), x.data_ptr(), y.data_ptr(), 2, cols, None)
    assert rc == -6
    assert b"16384" in lib.qb200_last_error()
    # the widest x it does hold goes through
    cols = 16384
    rc = lib.qb200_gemv_blocks_noalloc(B.Q8_0, B.F32, a.data_ptr(), x.data_ptr(), y.data_ptr(), 2, cols, None)
    assert rc == 0, lib.qb200_last_error().decode()
    torch.cuda.synchronize()
    assert np.array_equal(y.cpu().numpy(), np.zeros(2, np.float32))
