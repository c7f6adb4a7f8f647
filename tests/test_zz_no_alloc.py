"""The allocation-free batch-norm entry point, called through its exported C symbol, must give the
same result as the regular entry point (which takes a caller-provided workspace) on two calls in a row.

It is for callers that cannot allocate device memory (a fixed memory budget, a thread that must stay off
the framework's allocator, a fully committed device): its scratch is a fixed array inside the library.
This file is collected last on purpose, so a failure here cannot hide any other test.
"""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "tips_b200", "lib",
                   "libtips_kernels.so")


def _load():
    lib = ctypes.CDLL(LIB)
    P, L, I, F = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float
    lib.tipsk_bn_fwd_train_noalloc.restype = I
    lib.tipsk_bn_fwd_train_noalloc.argtypes = [P, P, P, P, P, P, P, P, P, L, I, F, F, I, I, P]
    lib.tipsk_bn_fwd_train.restype = I
    lib.tipsk_bn_fwd_train.argtypes = [P, P, P, P, P, P, P, P, P, P, L, I, F, F, I, I, P]
    lib.tipsk_bn_partials.restype = I
    lib.tipsk_bn_partials.argtypes = [L, I]
    lib.tipsk_last_error.restype = ctypes.c_char_p
    return lib


def _run(lib, noalloc, x, res, gamma, beta, relu):
    c = x.shape[1]
    m = x.numel() // c
    y = torch.empty_like(x)
    rm, rv = torch.zeros(c, device=x.device), torch.ones(c, device=x.device)
    sm, si = torch.empty(c, device=x.device), torch.empty(c, device=x.device)
    stream = torch.cuda.current_stream().cuda_stream
    if noalloc:
        rc = lib.tipsk_bn_fwd_train_noalloc(x.data_ptr(), res.data_ptr(), y.data_ptr(), gamma.data_ptr(),
                                            beta.data_ptr(), rm.data_ptr(), rv.data_ptr(), sm.data_ptr(),
                                            si.data_ptr(), m, c, 1e-5, 0.1, relu, 6, stream)
    else:
        ws = torch.empty(2 * c * lib.tipsk_bn_partials(m, c), dtype=torch.float32, device=x.device)
        rc = lib.tipsk_bn_fwd_train(x.data_ptr(), res.data_ptr(), y.data_ptr(), gamma.data_ptr(), beta.data_ptr(),
                                    rm.data_ptr(), rv.data_ptr(), sm.data_ptr(), si.data_ptr(), ws.data_ptr(), m, c,
                                    1e-5, 0.1, relu, 6, stream)
    assert rc == 0, lib.tipsk_last_error().decode()
    torch.cuda.synchronize()
    return y, rm, rv, sm, si


def test_noalloc_matches_regular_entry_point_twice():
    lib = _load()
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    for shape in [(16, 64, 28, 28), (8, 256, 14, 14)]:     # two calls in a row, different shapes share the scratch
        x = torch.randn(shape, device=dev).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        res = torch.randn_like(x)
        gamma = torch.rand(shape[1], device=dev) + 0.5
        beta = torch.randn(shape[1], device=dev)
        got = _run(lib, True, x, res, gamma, beta, 1)
        ref = _run(lib, False, x, res, gamma, beta, 1)
        for g, r in zip(got, ref):
            assert torch.allclose(g.float(), r.float(), atol=1e-5, rtol=1e-5)
        # and against plain PyTorch fp32 within the tolerance the other batch-norm tests use
        yr = torch.relu(torch.nn.functional.batch_norm(x.float(), None, None, gamma, beta, True, 0.1, 1e-5) + res.float())
        assert torch.allclose(got[0].float(), yr, atol=6e-2, rtol=6e-2)


def test_noalloc_rejects_oversized_problem():
    """A shape whose partial sums do not fit the built-in array is refused before anything is launched.
    The size check on the host is the only guard: x and y below have the right size, but the scratch is the fixed
    786432-float array and this shape needs 1204224 floats, so kernels launched for it would write past the
    array.  tests/test_no_alloc_limit_cpu.py checks on a machine without a GPU that the refusal comes before any
    CUDA call."""
    lib = _load()
    dev = torch.device("cuda", 0)
    c, m = 200704, 256     # 784 column tiles -> 2 partial rows + 1 -> 1204224 scratch floats > 786432
    assert 2 * c * lib.tipsk_bn_partials(m, c) > 768 * 1024
    x = torch.randn(m, c, device=dev).to(torch.bfloat16)
    y = torch.empty_like(x)
    gamma, beta = torch.ones(c, device=dev), torch.zeros(c, device=dev)
    sm, si = torch.empty(c, device=dev), torch.empty(c, device=dev)
    rc = lib.tipsk_bn_fwd_train_noalloc(x.data_ptr(), None, y.data_ptr(), gamma.data_ptr(), beta.data_ptr(), None, None,
                                        sm.data_ptr(), si.data_ptr(), m, c, 1e-5, 0.1, 0, 6,
                                        torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc < 0 and b"scratch floats" in lib.tipsk_last_error()
