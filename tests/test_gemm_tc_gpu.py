"""Int4GemmA8Tc (W4A8 group-128 GEMM on tcgen05 tensor cores, accumulators in tensor memory,
weights streamed once for the whole batch) against the CPU oracle's one-row GEMV: every batch
entry bit for bit, for the batch widths and shapes of the operator sweep, ragged row counts and
several row tiles per block."""
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


def run_tc(dev, P, S, xq, sq, N, K, M, groups=None):
    dY = dev.zeros(M * N * 4)
    ntiles = (N + 127) // 128
    groups = groups or min(ntiles, dev.info().sm_count * 2)
    dev.kernel("Int4GemmA8Tc")(groups, dev.upload(P), dev.upload(S), dev.upload(xq), dev.upload(sq), dY, N, K, M, N)
    dev.sync()
    return dev.download(dY, M * N, np.float32).reshape(M, N)


@pytest.mark.parametrize("N,K,M", [(136, 2048, 1), (136, 2048, 8), (512, 2048, 2), (512, 2048, 4), (2048, 512, 8),
                                   (300, 128, 3), (1000, 1024, 16), (4096, 2048, 64), (2048, 512, 64), (640, 4096, 37)])
def test_gemm_a8_tc_bit_exact(dev, N, K, M):
    rng = np.random.default_rng(N * 7 + K + M)
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    P, S = O.quantize_int4(w)
    x = rng.standard_normal((M, K)).astype(np.float32) * 2
    q = [O.aquant(x[m]) for m in range(M)]
    xq = np.stack([a for a, _ in q]); sq = np.stack([b for _, b in q])
    want = np.stack([O.gemv_a8(P, S, xq[m], sq[m]) for m in range(M)])
    got = run_tc(dev, P, S, xq, sq, N, K, M)
    assert np.array_equal(got, want)


def test_gemm_a8_tc_several_tiles_per_block_and_extreme_values(dev):
    """Two blocks walk 11 row tiles; activations at +-127 and weights at -8 / 7 (the largest group sums)."""
    rng = np.random.default_rng(3)
    N, K, M = 1300, 2048, 8
    w = np.where(rng.random((N, K)) < 0.5, -0.08, 0.07).astype(np.float32)
    P, S = O.quantize_int4(w)
    x = np.where(rng.random((M, K)) < 0.5, -1.0, 1.0).astype(np.float32)
    q = [O.aquant(x[m]) for m in range(M)]
    xq = np.stack([a for a, _ in q]); sq = np.stack([b for _, b in q])
    want = np.stack([O.gemv_a8(P, S, xq[m], sq[m]) for m in range(M)])
    got = run_tc(dev, P, S, xq, sq, N, K, M, groups=2)
    assert np.array_equal(got, want)


TC_GROUP = np.dtype([("P", "<u8"), ("S", "<u8"), ("x_row0", "<i4"), ("M", "<i4"), ("y_col", "<i4"), ("pad", "<i4")])


@pytest.mark.parametrize("N,K,blocks", [(512, 2048, 7), (2048, 512, 296), (300, 1024, 3)])
def test_grouped_gemm_a8_tc_bit_exact(dev, N, K, blocks):
    """A list of problems (own weights, own range of activation rows, own output column) in one
    launch, the list and its length in device memory: every row equals the one-row GEMV; rows no
    problem covers stay untouched; a second launch with an empty list writes nothing."""
    rng = np.random.default_rng(N + K)
    Ms = [1, 64, 3, 8, 17, 2, 40]
    rows = sum(Ms) + 5
    x = rng.standard_normal((rows, K)).astype(np.float32) * 2
    q = [O.aquant(x[m]) for m in range(rows)]
    xq = np.stack([a for a, _ in q]); sq = np.stack([b for _, b in q])
    ldy = 2 * N + 8
    want = np.full((rows, ldy), 7.0, np.float32)
    tab = np.zeros(len(Ms), TC_GROUP)
    keep = []
    row0 = 2
    for i, M in enumerate(Ms):
        w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
        P, S = O.quantize_int4(w)
        dP, dS = dev.upload(P), dev.upload(S)
        keep.append((dP, dS))
        col = (i % 2) * N + 4 * (i % 2)
        tab[i] = (dP, dS, row0, M, col, 0)
        for m in range(M):
            want[row0 + m, col:col + N] = O.gemv_a8(P, S, xq[row0 + m], sq[row0 + m])
        row0 += M
    order = rng.permutation(len(Ms))          # the list need not be in row order
    dTab, dN = dev.upload(tab[order].view(np.uint8)), dev.upload(np.array([len(Ms)], np.int32))
    dY = dev.upload(np.full((rows, ldy), 7.0, np.float32))
    k = dev.kernel("Int4GemmA8TcGrouped")
    k(blocks, dTab, dN, dev.upload(xq), dev.upload(sq), dY, N, K, 64, ldy)
    dev.sync()
    got = dev.download(dY, rows * ldy, np.float32).reshape(rows, ldy)
    assert np.array_equal(got, want)
    dev.write(dN, np.zeros(1, np.int32))
    dev.write(dY, np.full((rows, ldy), 3.0, np.float32))
    k(blocks, dTab, dN, dev.upload(xq), dev.upload(sq), dY, N, K, 64, ldy)
    dev.sync()
    assert np.all(dev.download(dY, rows * ldy, np.float32) == 3.0)
