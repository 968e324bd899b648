"""Int4GemvA8Multi (W4A8 group-128 GEMV for 1..8 activation rows, weights streamed once through a
ring of bulk copies, dp4a) against the CPU oracle's one-row GEMV: every batch entry bit for bit,
for the sweep's shapes, ragged row counts, odd tile counts per block and extreme values."""
import numpy as np
import pytest

import oracle_lib as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    from ainfer_b200 import cuda_abi
    d = cuda_abi.Device(0)
    yield d
    d.close()


def run(dev, P, S, xq, sq, N, K, M, groups=None):
    dY = dev.upload(np.full((M, N), 7.0, np.float32))
    tiles = -(-N // (256 // (K // 128)))
    groups = groups or min(tiles, dev.info().sm_count * 2)
    dev.kernel("Int4GemvA8Multi")(groups, dev.upload(P), dev.upload(S), dev.upload(xq), dev.upload(sq), dY, N, K, M, N)
    dev.sync()
    return dev.download(dY, M * N, np.float32).reshape(M, N)


@pytest.mark.parametrize("N,K,M,groups", [(136, 2048, 1, None), (136, 2048, 8, None), (512, 2048, 2, None), (512, 2048, 4, 3),
                                          (2048, 512, 8, None), (300, 128, 3, None), (1000, 1024, 5, 7), (4096, 2048, 8, None),
                                          (640, 4096, 7, None), (33, 256, 2, 1), (8192, 2048, 4, 296)])
def test_gemv_multi_bit_exact(dev, N, K, M, groups):
    rng = np.random.default_rng(N * 7 + K + M)
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    P, S = O.quantize_int4(w)
    x = rng.standard_normal((M, K)).astype(np.float32) * 2
    q = [O.aquant(x[m]) for m in range(M)]
    xq = np.stack([a for a, _ in q]); sq = np.stack([b for _, b in q])
    want = np.stack([O.gemv_a8(P, S, xq[m], sq[m]) for m in range(M)])
    got = run(dev, P, S, xq, sq, N, K, M, groups)
    assert np.array_equal(got, want)


def test_gemv_multi_extreme_values(dev):
    rng = np.random.default_rng(3)
    N, K, M = 1300, 2048, 8
    w = np.where(rng.random((N, K)) < 0.5, -0.08, 0.07).astype(np.float32)
    P, S = O.quantize_int4(w)
    x = np.where(rng.random((M, K)) < 0.5, -1.0, 1.0).astype(np.float32)
    q = [O.aquant(x[m]) for m in range(M)]
    xq = np.stack([a for a, _ in q]); sq = np.stack([b for _, b in q])
    want = np.stack([O.gemv_a8(P, S, xq[m], sq[m]) for m in range(M)])
    assert np.array_equal(run(dev, P, S, xq, sq, N, K, M, groups=2), want)
