"""The allocation-free sum-of-squares entry point, called the way a C program would call it.

Some users of the native library cannot allocate device memory where they need this reduction (a latency-critical
loop, under somebody else's memory pool, from plain C without a caching allocator).  ``kf_sumsq_noalloc``
keeps its scratch in a device array inside the library; this test calls the exported symbol directly through
ctypes and checks it against the regular entry point (which takes a caller-allocated scratch buffer), twice in
a row because the scratch array is shared between calls and keeps the previous call's contents.

Runs last (file name) so that a failure here cannot hide results of the other GPU tests.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _load():
    from kempnerforge_b200.ops.build import build

    lib = ctypes.CDLL(str(build()))
    lib.kf_sumsq_noalloc.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p,
                                     ctypes.c_int, ctypes.c_void_p]
    lib.kf_sumsq_noalloc.restype = ctypes.c_int
    lib.kf_sumsq.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                             ctypes.c_int, ctypes.c_void_p]
    lib.kf_sumsq.restype = ctypes.c_int
    return lib


def _reference(lib, x, dt):
    partial = torch.empty(1024, dtype=torch.float32, device=x.device)
    out = torch.zeros(1, dtype=torch.float32, device=x.device)
    rc = lib.kf_sumsq(x.data_ptr(), x.numel(), dt, partial.data_ptr(), out.data_ptr(), 0, None)
    assert rc == 0
    return out


@pytest.mark.parametrize("dtype,dt", [(torch.bfloat16, 0), (torch.float32, 1)])
def test_noalloc_sumsq_matches_regular_entry_point_twice(dtype, dt):
    lib = _load()
    torch.manual_seed(0)
    dev = torch.device("cuda", torch.cuda.current_device())
    torch.cuda.synchronize()
    # first call: large input (uses all 1024 scratch slots); second call: small input (uses a few slots while the
    # rest still hold the first call's partial sums)
    for n in (3_000_001, 4_099):
        x = torch.randn(n, device=dev, dtype=torch.float32).to(dtype)
        want = _reference(lib, x, dt)
        got = torch.full((1,), -1.0, dtype=torch.float32, device=dev)
        stream = torch.cuda.current_stream().cuda_stream
        rc = lib.kf_sumsq_noalloc(x.data_ptr(), x.numel(), dt, got.data_ptr(), 0, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.allclose(got, want, rtol=1e-6, atol=0.0), (got.item(), want.item())
        exact = (x.double() ** 2).sum().item()
        assert abs(got.item() - exact) <= 1e-4 * exact
        # accumulate mode adds to what is already there
        rc = lib.kf_sumsq_noalloc(x.data_ptr(), x.numel(), dt, got.data_ptr(), 1, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert abs(got.item() - 2 * want.item()) <= 1e-5 * abs(want.item())


def test_noalloc_sumsq_unaligned_bf16_view_and_empty_input():
    """A bf16 view that starts one element into its allocation is only 2-byte aligned (the scalar path of the
    kernel); a length that is not a multiple of 8 exercises the tail; an empty input must give 0."""
    lib = _load()
    dev = torch.device("cuda", torch.cuda.current_device())
    torch.manual_seed(1)
    stream = torch.cuda.current_stream().cuda_stream
    base = torch.randn(70_003, device=dev, dtype=torch.float32).to(torch.bfloat16)
    for _ in range(2):
        x = base[1:]                                        # odd element offset, n % 8 != 0
        assert x.data_ptr() % 16 != 0 and x.numel() % 8 != 0
        got = torch.full((1,), -1.0, dtype=torch.float32, device=dev)
        assert lib.kf_sumsq_noalloc(x.data_ptr(), x.numel(), 0, got.data_ptr(), 0, stream) == 0
        want = _reference(lib, x, 0)
        torch.cuda.synchronize()
        exact = (x.double() ** 2).sum().item()
        assert torch.allclose(got, want, rtol=1e-6, atol=0.0) and abs(got.item() - exact) <= 1e-4 * exact
        empty = torch.full((1,), 5.0, dtype=torch.float32, device=dev)
        assert lib.kf_sumsq_noalloc(x.data_ptr(), 0, 0, empty.data_ptr(), 0, stream) == 0
        torch.cuda.synchronize()
        assert empty.item() == 0.0


def test_noalloc_sumsq_rejects_oversize_and_bad_dtype():
    lib = _load()
    out = torch.zeros(1, dtype=torch.float32, device="cuda")
    x = torch.zeros(8, dtype=torch.float32, device="cuda")
    assert lib.kf_sumsq_noalloc(x.data_ptr(), (1 << 34) + 1, 1, out.data_ptr(), 0, None) == 3
    assert lib.kf_sumsq_noalloc(x.data_ptr(), -1, 1, out.data_ptr(), 0, None) == 3
    assert lib.kf_sumsq_noalloc(x.data_ptr(), 8, 7, out.data_ptr(), 0, None) == 4
