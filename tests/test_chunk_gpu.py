"""Chunk path of the Gated DeltaNet layer (ChunkConvSilu, ChunkDeltaNet: M tokens per launch with
conv history and recurrent state carried on the chip) against the CPU oracle's sequential
recurrence, bit for bit: outputs of every row and the state left behind, for chunk sizes around
the 64-row staging block, with the state carried across launches, and the check that a later
chunk run alone (from a zero state) gives something else."""
import numpy as np
import pytest

import oracle_lib as O

pytestmark = pytest.mark.gpu
D = 128


@pytest.fixture(scope="module")
def dev():
    from ainfer_b200 import cuda_abi
    d = cuda_abi.Device(0)
    yield d
    d.close()


def oracle_rows(mx, S, bt, gt, nK, nV, states=None):
    """Sequential recurrence over the rows of mx [M][C]; S [nV][D*D] updated in place; states
    (optional list) receives a copy of S after every row."""
    L = O.lib()
    M = mx.shape[0]
    out = np.zeros((M, nV, D), np.float32)
    ratio = nV // nK
    for m in range(M):
        for h in range(nV):
            kh = h // ratio
            q = np.zeros(D, np.float32); k = np.zeros(D, np.float32)
            L.orc_l2norm(np.ascontiguousarray(mx[m, kh * D:(kh + 1) * D]), D, np.float32(0.0883883476), q)
            L.orc_l2norm(np.ascontiguousarray(mx[m, (nK + kh) * D:(nK + kh + 1) * D]), D, np.float32(1.0), k)
            v = np.ascontiguousarray(mx[m, (2 * nK + h) * D:(2 * nK + h + 1) * D])
            L.orc_deltanet_head(S[h], q, k, v, float(bt[m, h]), float(gt[m, h]), D, out[m, h])
        if states is not None:
            states.append(S.copy())
    return out


@pytest.mark.parametrize("nK,nV,chunks", [(2, 4, [1]), (2, 4, [17, 64]), (4, 8, [65, 3]), (16, 32, [64]), (2, 4, [130])])
def test_chunk_deltanet_equals_sequential_recurrence(dev, nK, nV, chunks):
    rng = np.random.default_rng(nV * 100 + sum(chunks))
    C = (2 * nK + nV) * D
    M = sum(chunks)
    mx = rng.standard_normal((M, C)).astype(np.float32)
    bt = rng.uniform(0.1, 0.9, (M, nV)).astype(np.float32)
    gt = (-rng.uniform(0.001, 0.5, (M, nV))).astype(np.float32)
    S0 = (rng.standard_normal((nV, D * D)) * 0.1).astype(np.float32)
    S_ref = S0.copy()
    want = oracle_rows(mx, S_ref, bt, gt, nK, nV)
    dS = dev.upload(S0)
    k = dev.kernel("ChunkDeltaNet")
    got, m0 = [], 0
    for n in chunks:                                   # state carried across the launches
        dOut = dev.zeros(n * nV * D * 4)
        k(nV * 4, dOut, dev.upload(mx[m0:m0 + n]), dS, dev.upload(bt[m0:m0 + n]), dev.upload(gt[m0:m0 + n]), nK, nV, n, 0, 0)
        dev.sync()
        got.append(dev.download(dOut, (n, nV, D), np.float32))
        m0 += n
    got = np.concatenate(got, 0)
    assert np.array_equal(got, want)
    assert np.array_equal(dev.download(dS, (nV, D * D), np.float32), S_ref)
    if len(chunks) > 1:
        # the last chunk alone, from a zero state, must differ: the carried state matters
        n = chunks[-1]
        dZ, dOut = dev.zeros(nV * D * D * 4), dev.zeros(n * nV * D * 4)
        k(nV * 4, dOut, dev.upload(mx[M - n:]), dZ, dev.upload(bt[M - n:]), dev.upload(gt[M - n:]), nK, nV, n, 0, 0)
        dev.sync()
        assert not np.array_equal(dev.download(dOut, (n, nV, D), np.float32), want[M - n:])
    # the decode kernel, one row at a time, gives the same rows (chunk == M decode steps)
    if M <= 20:
        dS2, dO2 = dev.upload(S0), dev.zeros(nV * D * 4)
        step = dev.kernel("DeltaNetStep")
        for m in range(M):
            step(nV * 4, dO2, dev.upload(mx[m]), dS2, dev.upload(bt[m]), dev.upload(gt[m]), nK, nV)
            dev.sync()
            assert np.array_equal(dev.download(dO2, (nV, D), np.float32), want[m])


@pytest.mark.parametrize("C,chunks", [(300, [1, 5]), (8192, [64, 64, 7])])
def test_chunk_conv_silu_equals_sequential(dev, C, chunks):
    L = O.lib()
    rng = np.random.default_rng(C)
    M = sum(chunks)
    x = rng.standard_normal((M, C)).astype(np.float32)
    cw = (rng.standard_normal((C, 4)) * 0.5).astype(np.float32)
    cs0 = rng.standard_normal((C, 3)).astype(np.float32)
    cs = cs0.copy().reshape(-1)
    want = np.zeros((M, C), np.float32)
    for m in range(M):
        L.orc_conv_silu(np.ascontiguousarray(x[m]), cs, cw.reshape(-1), C, want[m])
    dCS, dCW = dev.upload(cs0), dev.upload(cw)
    k = dev.kernel("ChunkConvSilu")
    m0 = 0
    for n in chunks:
        dMx = dev.zeros(n * C * 4)
        k((C + 255) // 256, dMx, dev.upload(x[m0:m0 + n]), dCS, dCW, C, n, 0, 0)
        dev.sync()
        assert np.array_equal(dev.download(dMx, (n, C), np.float32), want[m0:m0 + n])
        m0 += n
    assert np.array_equal(dev.download(dCS, C * 3, np.float32), cs)


def test_chunk_snapshots_hold_the_state_after_every_row(dev):
    """Speculative rows: with a snapshot buffer the kernels also keep the state after each row, so a
    caller can roll back to any of them."""
    L = O.lib()
    nK, nV, M = 2, 4, 4
    rng = np.random.default_rng(9)
    C = (2 * nK + nV) * D
    mx = rng.standard_normal((M, C)).astype(np.float32)
    bt = rng.uniform(0.1, 0.9, (M, nV)).astype(np.float32)
    gt = (-rng.uniform(0.001, 0.5, (M, nV))).astype(np.float32)
    S0 = (rng.standard_normal((nV, D * D)) * 0.1).astype(np.float32)
    states = []
    oracle_rows(mx, S0.copy(), bt, gt, nK, nV, states)
    stride = nV * D * D + 64                      # rows of the snapshot buffer need not be packed
    dSnap, dS, dOut = dev.zeros(M * stride * 4), dev.upload(S0), dev.zeros(M * nV * D * 4)
    dev.kernel("ChunkDeltaNet")(nV * 4, dOut, dev.upload(mx), dS, dev.upload(bt), dev.upload(gt), nK, nV, M, dSnap, stride)
    dev.sync()
    snap = dev.download(dSnap, (M, stride), np.float32)
    for m in range(M):
        assert np.array_equal(snap[m, :nV * D * D].reshape(nV, D * D), states[m]), m
    # conv history snapshots
    Cc = 300
    x = rng.standard_normal((M, Cc)).astype(np.float32)
    cw = (rng.standard_normal((Cc, 4)) * 0.5).astype(np.float32)
    cs = rng.standard_normal((Cc, 3)).astype(np.float32)
    ref = cs.copy().reshape(-1)
    hist = []
    for m in range(M):
        L.orc_conv_silu(np.ascontiguousarray(x[m]), ref, cw.reshape(-1), Cc, np.zeros(Cc, np.float32))
        hist.append(ref.copy())
    dSn = dev.zeros(M * Cc * 3 * 4)
    dev.kernel("ChunkConvSilu")((Cc + 255) // 256, dev.zeros(M * Cc * 4), dev.upload(x), dev.upload(cs), dev.upload(cw), Cc, M, dSn, Cc * 3)
    dev.sync()
    got = dev.download(dSn, (M, Cc * 3), np.float32)
    for m in range(M):
        assert np.array_equal(got[m], hist[m]), m
