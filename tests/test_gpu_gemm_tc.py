"""Parity of the tcgen05 skinny GEMM (9..64 activation rows) against the CPU oracle's f32 x bf16
matmul, through the C ABI.  The kernel splits each f32 activation into three bf16 terms, so the
only differences from the oracle are f32 summation order and the 2^-24 tail of the split."""
import numpy as np
import pytest

from homura_b200 import synth

pytestmark = pytest.mark.gpu

SWEEP = [(896, 1152), (896, 9728), (4864, 896), (1536, 17920), (8960, 1536), (1024, 151936 // 16)]


def rel_err(got, want):
    return float(np.abs(got - want).max() / (np.abs(want).max() + 1e-30))


def host_pack_tc(w):
    """numpy restatement of the tile layout: [nb][kb][128][64], 16-byte chunks XOR-swizzled by row."""
    K, N = w.shape
    nb, kb = (N + 127) // 128, (K + 63) // 64
    pad = np.zeros((kb * 64, nb * 128), np.uint16)
    pad[:K, :N] = w
    t = pad.T.reshape(nb, 128, kb, 8, 8).transpose(0, 2, 1, 3, 4)  # [nb][kb][row][chunk][e]
    out = np.empty_like(t)
    rows = np.arange(128)
    for c in range(8):
        out[:, :, rows, c ^ (rows & 7), :] = t[:, :, rows, c, :]
    return np.ascontiguousarray(out).reshape(-1)


def test_pack_tc_layout(hm):
    rng = np.random.default_rng(3)
    for (K, N) in [(64, 128), (200, 136), (896, 1152)]:
        w = rng.integers(0, 65536, (K, N), dtype=np.uint16)
        np.testing.assert_array_equal(hm.pack_bf16_tc(w), host_pack_tc(w))


@pytest.mark.parametrize("K,N", SWEEP)
@pytest.mark.parametrize("M", [16, 64])
def test_gemm_tc_matches_oracle(hm, oracle, K, N, M):
    rng = np.random.default_rng(K * 31 + N + M)
    w = synth.f32_to_bf16_rne(rng.standard_normal((K, N), dtype=np.float32) * np.float32(0.02))
    x = rng.standard_normal((M, K), dtype=np.float32)
    want = oracle.matmul_bf16(x, w)
    wt = hm.pack_bf16_tc(w)
    got = hm.gemm_bf16_tc(x, wt, N)
    assert rel_err(got, want) < 2e-5
    # deterministic: fixed-order cluster reduction
    np.testing.assert_array_equal(got, hm.gemm_bf16_tc(x, wt, N))
    # every split factor computes the same product
    for ks in (1, 2, 4, 8, 12, 16):
        assert rel_err(hm.gemm_bf16_tc(x, wt, N, ksplit=ks), want) < 2e-5


def test_gemm_tc_ragged_and_limits(hm, oracle):
    for (M, K, N) in [(1, 64, 128), (9, 200, 136), (33, 1000, 1000), (64, 48, 8), (17, 96, 264)]:
        rng = np.random.default_rng(M + K + N)
        w = synth.f32_to_bf16_rne(rng.standard_normal((K, N), dtype=np.float32))
        x = rng.standard_normal((M, K), dtype=np.float32)
        assert rel_err(hm.gemm_bf16_tc(x, hm.pack_bf16_tc(w), N), oracle.matmul_bf16(x, w)) < 2e-5
    w = hm.pack_bf16_tc(np.ones((64, 128), np.uint16))
    with pytest.raises(hm.HomuraError):
        hm.gemm_bf16_tc(np.ones((65, 64), np.float32), w, 128)  # M > 64
    with pytest.raises(hm.HomuraError):
        hm.gemm_bf16_tc(np.ones((4, 64), np.float32), w, 128, ksplit=17)


def test_gemm_tc_keeps_f32_activation_precision(hm, oracle):
    # activations with bits far below bf16 resolution: a bf16-only path would lose them
    K, N, M = 512, 256, 32
    rng = np.random.default_rng(11)
    w = synth.f32_to_bf16_rne(rng.standard_normal((K, N), dtype=np.float32))
    base = rng.standard_normal((M, K), dtype=np.float32)
    x = base * np.float32(1.0 + 2.0 ** -12)
    want = oracle.matmul_bf16(x, w)
    got = hm.gemm_bf16_tc(x, hm.pack_bf16_tc(w), N)
    assert rel_err(got, want) < 2e-6
