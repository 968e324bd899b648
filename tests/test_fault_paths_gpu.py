"""The error paths that bounded waits and the weight-stream checks rely on, exercised without
any faulting access: a wait that runs out, a weight pointer that cannot be bulk-copied, and a
sync with a timeout. The library's fault word is sticky for the life of a process, so every case
runs in a process of its own; the GPU stays usable throughout (each script keeps using it after
the reported error)."""
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu


def run(script):
    r = subprocess.run([sys.executable, "-c", textwrap.dedent(script)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    return r.stdout


PRELUDE = """
    import os, sys
    sys.path.insert(0, os.getcwd()); sys.path.insert(0, os.path.join(os.getcwd(), "tests"))
    import numpy as np
    from ainfer_b200 import cuda_abi
    dev = cuda_abi.Device(0)
    def sync(tag):
        try:
            dev.sync(); print(tag, "OK")
        except cuda_abi.AinferError as e:
            print(tag, "FAIL", e.status, str(e))
"""


def test_a_bounded_wait_that_runs_out_is_reported_and_sticky():
    out = run(PRELUDE + """
    res = dev.zeros(16)
    sync("before")
    dev.kernel("BoundedWaitProbe")(1, res)
    sync("after")
    print("RESULT", int(dev.download(res, 1, np.int32)[0]))
    sync("later")
    """)
    assert "before OK" in out
    assert "after FAIL 3" in out and "bounded wait" in out          # AINFER_ERR_DEVICE with the reason
    assert "RESULT 2" in out                                          # the kernel ended by itself and said why
    assert "later FAIL 3" in out                                      # sticky: the process must not go on computing


def test_a_weight_pointer_off_by_8_bytes_is_reported_and_nothing_faults():
    out = run(PRELUDE + """
    import oracle_lib as O
    from test_kernels_gpu import GEMV_MAT, rnd_weights
    rng = np.random.default_rng(5)
    N, K = 64, 2048
    P, S = rnd_weights(rng, N + 1, K)
    xq, sq = O.aquant(rng.standard_normal(K).astype(np.float32))
    dP, dY = dev.upload(P), dev.zeros(N * 4)
    tab = np.zeros(1, GEMV_MAT)
    tab[0]["P"], tab[0]["S"], tab[0]["Y"], tab[0]["N"], tab[0]["ldy"] = dP + 8, dev.upload(S), dY, N, N
    dev.kernel("Int4GemvA8")(4, dev.upload(tab.view(np.uint8)), 1, N, dev.upload(xq), dev.upload(sq), K, 1)
    sync("after")
    # the device still answers: memory traffic and another (well-formed) launch work
    tab[0]["P"] = dP
    dev.kernel("Int4GemvA8")(4, dev.upload(tab.view(np.uint8)), 1, N, dev.upload(xq), dev.upload(sq), K, 1)
    try:
        dev.L.ainfer_sync(dev.h, 2**64 - 1)
    except Exception:
        pass
    got = dev.download(dY, N, np.float32)
    print("SECOND", bool(np.array_equal(got, O.gemv_a8(P[:N], S[:N], xq, sq))))
    """)
    assert "after FAIL 3" in out and "16-byte aligned" in out
    assert "SECOND True" in out


def test_sync_with_a_timeout_returns_timeout_and_a_later_sync_succeeds():
    out = run(PRELUDE + """
    ctrl, ids = dev.zeros(16), dev.zeros(64)
    k = dev.kernel("ControlAdvance")
    k.set_args(ctrl, ids, 16)
    cl = dev.new_list()
    for _ in range(20000):
        cl.append(k, 1)
    cl.close()
    cl.execute(); cl.execute(); cl.execute()
    st = dev.L.ainfer_sync(dev.h, 0)
    print("TIMED", st, (dev.L.ainfer_last_error(dev.h) or b"").decode())
    sync("blocking")
    print("POS", int(dev.download(ctrl, 4, np.int32)[1]))
    """)
    assert "TIMED 5 sync timed out" in out                           # AINFER_ERR_TIMEOUT
    assert "blocking OK" in out and "POS 60000" in out
