"""The allocation-free CEMA entry point, called through its exported C symbol
the way a caller without a tensor library would (ctypes, raw device pointers),
must reproduce the regular entry point.  It is meant for callers that cannot
allocate device memory while running - e.g. a latency-critical loop that may
not enter the allocator, or a C host with a fixed memory budget - so the test
hands it only inputs and outputs and checks two consecutive calls, since both
share the library's built-in scratch array."""
import ctypes
import glob
import math
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _lib():
    import megalodon_b200._C  # noqa: F401  (makes sure libtorch / cudart are loaded first)
    path = glob.glob(os.path.join(ROOT, "megalodon_b200", "_C*.so"))[0]
    lib = ctypes.CDLL(path)
    lib.mb_cema_fwd_noalloc.restype = ctypes.c_int
    lib.mb_cema_fwd_noalloc.argtypes = [ctypes.c_void_p] * 8 + [ctypes.c_int] * 5 + [ctypes.c_void_p]
    lib.mb_cema_noalloc_scratch_needed.restype = ctypes.c_ulonglong
    lib.mb_cema_noalloc_scratch_needed.argtypes = [ctypes.c_int] * 4
    return lib


def _coeffs(D, N, dev):
    alpha = torch.sigmoid(torch.randn(D, N, device=dev))
    delta = torch.sigmoid(torch.randn(D, N, device=dev))
    theta = torch.sigmoid(torch.randn(D, 1, device=dev)) * (2 * math.pi / N) * torch.arange(1, N + 1, device=dev)
    p = alpha.contiguous()
    q = torch.view_as_real(torch.polar(1.0 - alpha * delta, theta)).contiguous()
    gamma = (torch.randn(D, N, 2, device=dev) * math.sqrt(1.0 / N)).contiguous()
    omega = (torch.randn(D, device=dev) * 0.3).contiguous()
    return p, q, gamma, omega


def test_noalloc_cema_matches_regular_entry_point_twice():
    from megalodon_b200 import ops
    lib = _lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    torch.manual_seed(11)
    B, L, D, N = 2, 700, 96, 16          # 6 segments -> the scratch array is really used
    assert 0 < lib.mb_cema_noalloc_scratch_needed(B, L, D, N) <= (32 << 20)
    p, q, gamma, omega = _coeffs(D, N, dev)
    stream = torch.cuda.current_stream().cuda_stream
    for trial, dtype in enumerate((torch.bfloat16, torch.float32)):
        x = torch.randn(B, L, D, device=dev).to(dtype)
        hx = torch.randn(B, D, N, 2, device=dev)
        y_ref, h_ref = ops.cema(x, p.unsqueeze(-1), torch.view_as_complex(q).unsqueeze(-1),
                                torch.view_as_complex(gamma), omega.unsqueeze(-1),
                                torch.view_as_complex(hx), True)
        y = torch.empty_like(x)
        h_last = torch.empty(B, D, N, 2, device=dev)
        before = torch.cuda.memory_allocated(dev)
        rc = lib.mb_cema_fwd_noalloc(x.data_ptr(), p.data_ptr(), q.data_ptr(), gamma.data_ptr(), omega.data_ptr(),
                                     hx.data_ptr(), y.data_ptr(), h_last.data_ptr(), B, L, D, N,
                                     1 if dtype == torch.bfloat16 else 0, stream)
        assert rc == 0, f"call {trial} returned {rc}"
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated(dev) == before
        atol, rtol = (4e-2, 4e-2) if dtype == torch.bfloat16 else (1e-4, 1e-3)
        assert torch.allclose(y.float(), y_ref.float(), atol=atol, rtol=rtol), (y.float() - y_ref.float()).abs().max()
        assert torch.allclose(h_last, torch.view_as_real(h_ref), atol=1e-3, rtol=1e-2)


def test_noalloc_cema_rejects_oversized_problem():
    lib = _lib()
    dev = torch.device("cuda", 0)
    B, L, D, N = 4, 8192, 4096, 16        # needs 1 GiB of scratch
    assert lib.mb_cema_noalloc_scratch_needed(B, L, D, N) > (32 << 20)
    dummy = torch.zeros(8, device=dev)
    rc = lib.mb_cema_fwd_noalloc(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
                                 dummy.data_ptr(), None, dummy.data_ptr(), None, B, L, D, N, 1,
                                 torch.cuda.current_stream().cuda_stream)
    assert rc == 1      # MB_NOALLOC_TOO_LARGE: nothing was launched
    assert lib.mb_cema_fwd_noalloc(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
                                   dummy.data_ptr(), None, dummy.data_ptr(), None, 1, 64, 8, 3, 1,
                                   torch.cuda.current_stream().cuda_stream) == 2   # N = 3 unsupported
