"""The engine's token-block product against torch fp32 / float64 on its own: every kernel it can pick (rows, tiled,
tensor-core), shapes with ragged edges (K not a multiple of the 64-wide K block, few features, token tails)."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lib():
    from kuiperllama_b200 import build
    L = ctypes.CDLL(str(build.build_seq()))
    L.kllm_seq_gemm.restype = ctypes.c_int
    L.kllm_seq_gemm.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                                ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    return L


SHAPES = [(1, 72, 230), (3, 256, 77), (8, 40, 16), (5, 33, 9), (64, 64, 8), (120, 72, 230), (120, 240, 72), (65, 200, 129),
          (300, 256, 512), (257, 1000, 300), (1113, 384, 256), (90, 50, 70)]


@pytest.mark.parametrize("T,K,N", SHAPES)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gemm_against_torch(lib, T, K, N, dtype):
    g = torch.Generator().manual_seed(T * 7 + K)
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    a = torch.randn(T, K, generator=g).to(td).cuda()
    w = torch.randn(N, K, generator=g).to(td).cuda()
    out = torch.full((T, N), float("nan"), device="cuda")
    rc = lib.kllm_seq_gemm(0 if dtype == "float32" else 1, a.data_ptr(), w.data_ptr(), out.data_ptr(), T, K, N, None)
    assert rc == 0
    torch.cuda.synchronize()
    ref = a.double() @ w.double().T
    err = (out.double() - ref).abs().max().item()
    assert err < 2e-5 * K ** 0.5 * 4, f"max abs error {err}"
