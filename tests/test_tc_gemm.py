"""GPU parity test of the tcgen05/TMEM batched projection kernel against a float64 matmul of the
same BF16 values (products of BF16 numbers are exact in f32; only the f32 accumulation order
differs, so the tolerance is a few f32 ulps of the row's magnitude)."""
import ctypes as C

import numpy as np
import pytest

from util import pkg, syn

pytestmark = pytest.mark.gpu


def run(N, K, B, seed=0):
    rng = np.random.default_rng(seed)
    w = syn.f32_to_bf16_bits((rng.standard_normal((N, K)) * 0.05).astype(np.float32)).reshape(N, K)
    x = syn.f32_to_bf16_bits(rng.standard_normal((B, K)).astype(np.float32)).reshape(B, K)
    out = np.zeros((B, N), dtype=np.float32)
    ms = C.c_float(0)
    lib = pkg._native.lib()
    pkg._native.check(lib.oxg4_debug_tc_gemm(w.ctypes.data_as(C.c_void_p), x.ctypes.data_as(C.c_void_p), N, K, B,
                                             out.ctypes.data_as(C.c_void_p), C.byref(ms)))
    ref = syn.bf16_bits_to_f32(x).reshape(B, K).astype(np.float64) @ syn.bf16_bits_to_f32(w).reshape(N, K).astype(np.float64).T
    return out, ref, ms.value


@pytest.mark.parametrize("N,K,B", [(128, 64, 16), (256, 256, 16), (384, 2560, 16), (1000, 1152, 9), (4096, 2560, 32),
                                   (2560, 10240, 64), (200, 136, 33),
                                   # prompt chunks: blocks of 128 / 256 activation rows (UMMA N = 128 / 256)
                                   (384, 256, 100), (1000, 1152, 128), (4096, 2560, 200), (2560, 10240, 256),
                                   (300, 136, 255)])
def test_tc_gemm_matches_float64(N, K, B):
    out, ref, ms = run(N, K, B)
    scale = np.abs(ref).max()
    assert np.isfinite(out).all()
    assert np.abs(out - ref).max() <= 2e-5 * max(1.0, scale), (np.abs(out - ref).max(), scale)
