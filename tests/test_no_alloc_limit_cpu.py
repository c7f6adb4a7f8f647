"""Size limit of the allocation-free batch-norm entry point, checked where there is no GPU.

The refusal of an oversized problem is the only thing between such a call and kernels that would write past the
library's fixed scratch array, so it must come before the entry point touches CUDA at all.  On a machine without a
GPU any CUDA call fails with its own error (code -7); getting the size message (code -2) with null data pointers
therefore shows that nothing was looked up, copied or launched first."""
import ctypes
import os

import pytest

LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "tips_b200", "lib",
                   "libtips_kernels.so")


def test_oversized_problem_is_refused_before_any_cuda_call():
    import torch
    if torch.cuda.is_available():
        pytest.skip("meaningful only where CUDA calls cannot succeed")
    if not os.path.exists(LIB):
        from tips_b200 import build
        build.build_kernels()
    lib = ctypes.CDLL(LIB)
    P, L, I, F = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float
    lib.tipsk_bn_fwd_train_noalloc.restype = I
    lib.tipsk_bn_fwd_train_noalloc.argtypes = [P, P, P, P, P, P, P, P, P, L, I, F, F, I, I, P]
    lib.tipsk_bn_partials.restype = I
    lib.tipsk_bn_partials.argtypes = [L, I]
    lib.tipsk_last_error.restype = ctypes.c_char_p
    c, m = 200704, 256
    assert 2 * c * lib.tipsk_bn_partials(m, c) > 768 * 1024
    rc = lib.tipsk_bn_fwd_train_noalloc(None, None, None, None, None, None, None, None, None, m, c, 1e-5, 0.1, 0, 6, None)
    assert rc == -2 and b"scratch floats" in lib.tipsk_last_error()
    # a problem that fits goes on to the device lookup, which cannot succeed here: a CUDA error, not the size message
    rc = lib.tipsk_bn_fwd_train_noalloc(None, None, None, None, None, None, None, None, None, 64, 64, 1e-5, 0.1, 0, 6, None)
    assert rc == -7 and b"scratch floats" not in lib.tipsk_last_error()
