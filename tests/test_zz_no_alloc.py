"""The allocation-free SYRK entry point, called the way a C host would call it.

Some hosts own the GPU's memory budget themselves (a server that pre-carved the device into its
own arena, a plug-in contract that forbids allocator calls) and therefore cannot let the library
allocate the split-K scratch buffer.  ``asdl_b200_syrk_bf16_noalloc`` keeps that scratch in a
static device array inside the shared object.  Here it is resolved through its exported C symbol
with ctypes and compared with the regular (allocating) entry point on two consecutive calls,
which also shows that nothing left in the shared scratch by the first call leaks into the second.

This file sorts last on purpose: if it fails, a run that stops at the first failure has already
executed every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _entry_point():
    from asdl_b200.ops import _build
    _build.load()  # makes sure the shared object exists and libtorch is loaded first
    lib = ctypes.CDLL(_build._so_path())
    fn = lib.asdl_b200_syrk_bf16_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_longlong,
                   ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_float, ctypes.c_int,
                   ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int]
    return fn


def _status(lib_fn=None):
    """The entry point's own status word (read and cleared through its exported C symbol)."""
    from asdl_b200.ops import _build
    lib = ctypes.CDLL(_build._so_path())
    fn = lib.asdl_b200_noalloc_status
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.POINTER(ctypes.c_int)]
    code = ctypes.c_int(-1)
    rc = fn(ctypes.byref(code))
    assert rc == 0, f'asdl_b200_noalloc_status failed with {rc}'
    return code.value


def _call(fn, x, c, alpha, beta, nsplit):
    err = ctypes.create_string_buffer(256)
    stream = torch.cuda.current_stream().cuda_stream
    rc = fn(x.data_ptr(), x.shape[0], x.shape[1], x.stride(0), c.data_ptr(), c.stride(0),
            alpha, beta, nsplit, stream, err, len(err))
    return rc, err.value.decode()


def test_noalloc_entry_matches_regular_entry_twice():
    from asdl_b200 import ops
    ext = ops.extension()
    fn = _entry_point()
    torch.manual_seed(7)
    for rows, n, nsplit, beta in [(4096, 320, 4, 0.0), (6000, 192, 0, 0.9)]:
        x = torch.randn(rows, n, device='cuda').to(torch.bfloat16)
        c0 = torch.randn(n, n, device='cuda')
        c0 = c0 + c0.T
        want = c0.clone()
        ext.umma_gemm([x], [x], False, False, want, 1.0 / rows, beta, True, None, None, nsplit)
        got = c0.clone()
        rc, msg = _call(fn, x, got, 1.0 / rows, beta, nsplit)
        assert rc == 0, msg
        torch.cuda.synchronize()
        torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-6)
        ref = (x.double().T @ x.double() / rows + beta * c0.double()).float()
        torch.testing.assert_close(got, ref, rtol=1e-4, atol=1e-4)
        assert torch.equal(got, got.T)
        assert _status() == 0
    ops.check_status()


def test_noalloc_entry_rejects_oversized_request():
    fn = _entry_point()
    n = 4096  # 528 lower tiles x 64 KiB = 33 MiB per split: two splits exceed the 32 MiB buffer
    x = torch.zeros(2048, n, device='cuda', dtype=torch.bfloat16)
    c = torch.zeros(n, n, device='cuda')
    rc, msg = _call(fn, x, c, 1.0, 0.0, 2)
    assert rc != 0 and 'scratch' in msg
    rc, msg = _call(fn, x[:, :100], c, 1.0, 0.0, 1)  # n = 100 with ldx = 4096 is fine
    assert rc == 0, msg
    bad = torch.zeros(64, 12, device='cuda', dtype=torch.bfloat16)
    rc, msg = _call(fn, bad, c, 1.0, 0.0, 1)  # row pitch of 12 elements is not TMA-legal
    assert rc != 0 and 'ldx' in msg
    # a C pointer that is not 16-byte aligned with a row pitch that makes the kernel use 16-byte accesses:
    # refused on the host, nothing is launched
    flat = torch.zeros(128 * 128 + 4, device='cuda')
    x_ok = torch.zeros(256, 128, device='cuda', dtype=torch.bfloat16)
    err = ctypes.create_string_buffer(256)
    rc = fn(x_ok.data_ptr(), 256, 128, 128, flat.data_ptr() + 4, 128, 1.0, 0.0, 1,
            torch.cuda.current_stream().cuda_stream, err, len(err))
    assert rc != 0 and 'aligned' in err.value.decode()
    # row counts beyond the 32-bit range are refused before anything touches x
    rc = fn(x_ok.data_ptr(), 1 << 31, 128, 128, flat.data_ptr(), 128, 1.0, 0.0, 1,
            torch.cuda.current_stream().cuda_stream, err, len(err))
    assert rc != 0 and 'rows' in err.value.decode()
    torch.cuda.synchronize()
    assert _status() == 0
