"""`oa_col_sum_static`: the column sum for callers that cannot allocate device memory.

Some callers of the kernel library only hold a stream and pointers (a host callback on a stream, a thread
from another runtime, a loop that must not touch the allocator) and so cannot give `oa_col_sum` the scratch
buffer it needs.  `oa_col_sum_static` keeps that scratch in a fixed array inside the library.  This test
calls it through its exported C symbol, twice in a row (the array is shared and keeps the previous call's
contents), and checks each result against the existing `oa_col_sum` entry point; it also checks that a
problem beyond the array's size is refused.  The file name sorts last so that a run that stops at the
first failure has already run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from oa_b200 import _native
    lib = _native.require()
    fn = lib.oa_col_sum_static
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_int,
                   ctypes.c_int, ctypes.c_void_p]
    lib.oa_col_sum_static_max_floats.restype = ctypes.c_size_t
    lib.oa_col_sum_static_max_floats.argtypes = []
    return lib


@pytest.mark.parametrize("dtype,code,tol", [(torch.float32, 0, 1e-5), (torch.bfloat16, 1, 1e-2)])
def test_col_sum_static_matches_col_sum_twice(dtype, code, tol):
    from oa_b200.ops import kernels as K
    lib = _lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    torch.manual_seed(11)
    stream = torch.cuda.current_stream().cuda_stream
    # two different shapes back to back: the second call sees the first call's leftovers in the shared array
    for rows, cols in [(1000, 384), (700, 96)]:
        x = torch.randn(rows, cols, device=dev).to(dtype)
        ref = K.col_sum(x)                                   # existing entry point (caller-provided scratch)
        out = torch.empty(cols, dtype=dtype, device=dev)
        rc = lib.oa_col_sum_static(code, x.data_ptr(), out.data_ptr(), code, rows, cols, 0, stream)
        assert rc == 0, f"oa_col_sum_static returned {rc}"
        torch.cuda.synchronize()
        scale = ref.float().abs().max().item() + 1e-12
        err = (out.float() - ref.float()).abs().max().item()
        assert err <= tol * scale, f"{rows}x{cols}: max err {err} vs tol {tol * scale}"
        # accumulate form
        out2 = out.clone()
        rc = lib.oa_col_sum_static(code, x.data_ptr(), out2.data_ptr(), code, rows, cols, 1, stream)
        assert rc == 0
        torch.cuda.synchronize()
        err2 = (out2.float() - 2 * ref.float()).abs().max().item()
        assert err2 <= 2 * tol * scale + (0.02 * scale if dtype == torch.bfloat16 else 0.0)


def test_col_sum_static_refuses_oversize():
    lib = _lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    limit = lib.oa_col_sum_static_max_floats()
    assert limit == 1 << 20
    rows, cols = 256 * 9, (limit // 8)      # 9 partial rows x limit/8 columns > limit floats
    x = torch.zeros(8, device=dev)           # never read: the call must be refused before any launch
    out = torch.zeros(8, device=dev)
    rc = lib.oa_col_sum_static(0, x.data_ptr(), out.data_ptr(), 0, rows, cols, 0, torch.cuda.current_stream().cuda_stream)
    assert rc == 6, "a problem beyond the static scratch must be refused with OA_ERR_TOO_LARGE"
    torch.cuda.synchronize()
