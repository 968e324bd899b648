"""ainfer_router_topk_static: the router + top-k step with its scratch in a fixed device array.

Collected last (file name) and self-contained: it opens its own device handle, so it passes alone
and after every other GPU test. It calls the C-ABI entry point twice in a row and compares each
result, bit for bit, with the existing "RouterTopK" kernel entry driven through the generic
kernel-by-name calls on caller-provided scratch, and with the CPU oracle's router arithmetic.
"""
import ctypes as C

import numpy as np
import pytest

import oracle_lib as O
from oracle_lib import bf16_bits

pytestmark = pytest.mark.gpu


@pytest.fixture()
def dev():
    from ainfer_b200 import cuda_abi
    d = cuda_abi.Device(0)
    yield d
    d.close()


def run_generic(dev, dWr, dWsg, dHn, E, H, k):
    dLog, dCnt = dev.zeros((E + 1) * 4), dev.zeros(4)
    dI, dW, dG = dev.zeros((k + 1) * 4), dev.zeros((k + 1) * 4), dev.zeros(4)
    dev.kernel("RouterTopK")((E + 8) // 8, dWr, dWsg, dHn, dLog, dCnt, dI, dW, dG, E, H, k, 0, 0)
    dev.sync()
    return (dev.download(dI, k + 1, np.int32), dev.download(dW, k + 1, np.uint32), dev.download(dG, 1, np.uint32))


def run_static(dev, dWr, dWsg, dHn, E, H, k):
    dI, dW, dG = dev.zeros((k + 1) * 4), dev.zeros((k + 1) * 4), dev.zeros(4)
    dev.check(dev.L.ainfer_router_topk_static(dev.h, dWr, dWsg, dHn, dI, dW, dG, E, H, k))
    dev.sync()
    return (dev.download(dI, k + 1, np.int32), dev.download(dW, k + 1, np.uint32), dev.download(dG, 1, np.uint32))


@pytest.mark.parametrize("E,k,H,shared", [(64, 4, 1024, True), (512, 10, 2048, True), (1024, 8, 256, False)])
def test_static_scratch_router_matches_generic_entry_twice(dev, E, k, H, shared):
    rng = np.random.default_rng(1000 + E)
    wr_bits = bf16_bits((rng.standard_normal((E, H)) * 0.05).astype(np.float32))
    dWr = dev.upload(wr_bits)
    dWsg = dev.upload(bf16_bits((rng.standard_normal(H) * 0.05).astype(np.float32))) if shared else None
    for call in range(2):  # two calls in a row share the fixed array: the second must not see the first
        hn = rng.standard_normal(H).astype(np.float32)
        dHn = dev.upload(hn)
        want = run_generic(dev, dWr, dWsg, dHn, E, H, k)
        got = run_static(dev, dWr, dWsg, dHn, E, H, k)
        for g, w in zip(got, want):
            assert np.array_equal(g, w), f"call {call}"
        assert got[0][k] == E
        # and the oracle: logits by its bf16 row dot, then its softmax / top-k / renormalisation
        L = O.lib()
        logits = np.array([L.orc_dot_bf16(np.ascontiguousarray(wr_bits[e]), hn, H) for e in range(E)], np.float32)
        idx, wt, gap = np.zeros(k, np.int32), np.zeros(k, np.float32), np.zeros(1, np.float32)
        L.orc_router_topk(logits, E, k, idx, wt, gap.ctypes.data_as(C.POINTER(C.c_float)))
        assert got[0][:k].tolist() == idx.tolist(), f"call {call}"
        assert np.array_equal(got[1][:k], wt.view(np.uint32)), f"call {call}"
        assert np.array_equal(got[2], gap.view(np.uint32)), f"call {call}"


def test_static_scratch_router_rejects_sizes_beyond_the_array(dev):
    from ainfer_b200 import cuda_abi
    d = dev.zeros(64)
    st = dev.L.ainfer_router_topk_static(dev.h, d, None, d, d, d, d, 1025, 256, 4)
    assert st == 1  # AINFER_ERR_INVALID
    msg = (dev.L.ainfer_last_error(dev.h) or b"").decode()
    assert "1025" in msg and "1024" in msg
    with pytest.raises(cuda_abi.AinferError):
        dev.check(dev.L.ainfer_router_topk_static(dev.h, d, None, d, d, d, d, 64, 256, 40))
