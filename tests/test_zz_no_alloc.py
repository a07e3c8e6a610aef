"""The allocation-free GEMM entry point, called through its exported C symbol.

Some hosts of the library cannot allocate device memory while they call it (a serving process
whose pool already owns the GPU, start-up-only allocation policies, bare C callers), so
``oxb_gemm_bf16_noalloc`` keeps the split-K scratch in a fixed device array inside the library.
It must agree with the ordinary entry point, also when called twice in a row on the shared array.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / (b.norm() + 1e-12))


@pytest.mark.parametrize("T,N,K", [(64, 1280, 8192), (7, 200, 1000), (256, 512, 2048)])
def test_noalloc_gemm_matches_regular_entry_point(T, N, K):
    from oxidize_b200.ops import cuda as C

    L = C.lib()
    fn = L.oxb_gemm_bf16_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int] * 4 + [ctypes.c_void_p]
    torch.manual_seed(T + N)
    stream = torch.cuda.current_stream().cuda_stream
    for rep in range(2):  # two calls in a row share the static scratch
        x = (torch.randn(T, K, device="cuda") * 0.5).to(torch.bfloat16)
        w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
        bias = torch.randn(N, device="cuda") if rep else None
        want = C.gemm_bf16(x, w, bias=bias)
        got = torch.empty(T, N, dtype=torch.bfloat16, device="cuda")
        rc = fn(x.data_ptr(), w.data_ptr(), got.data_ptr(), None if bias is None else bias.data_ptr(), T, N, K, N, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert _rel_err(got, want) < 6e-3
        assert _rel_err(got, x.float() @ w.float().t() + (0 if bias is None else bias)) < 6e-3
    assert C.status()[0] == 0


def test_noalloc_gemm_rejects_oversize():
    from oxidize_b200.ops import cuda as C

    L = C.lib()
    fn = L.oxb_gemm_bf16_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int] * 4 + [ctypes.c_void_p]
    x = torch.zeros(300, 64, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(128, 64, dtype=torch.bfloat16, device="cuda")
    y = torch.zeros(300, 128, dtype=torch.bfloat16, device="cuda")
    assert fn(x.data_ptr(), w.data_ptr(), y.data_ptr(), None, 300, 128, 64, 128, None) == -1
    assert fn(x.data_ptr(), w.data_ptr(), y.data_ptr(), None, 16, 128, 63, 128, None) == -2
