"""Device-side sampler (kernel SampleToken, ainfer_session_sample) against the contracts of the
reference's host sampler (the checks of tools/sample/validate_t71.cpp:24-186, restated here for
the device: greedy fixtures, determinism by seed, top-k and top-p support, chi-square match with
the softmax, temperature limits, repetition penalty) and against this library's host sampler on
the same logits and RNG state (same token except where a draw lands within rounding of a CDF step)."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    from ainfer_b200 import cuda_abi
    d = cuda_abi.Device(0)
    yield d
    d.close()


class DevSampler:
    def __init__(self, dev, V):
        self.dev, self.V = dev, V
        self.k = dev.kernel("SampleToken")
        self.dL, self.dW, self.dM = dev.zeros(V * 4), dev.zeros(V * 8), dev.zeros(V)
        self.dSeen, self.dRng, self.dOut, self.dP = dev.zeros(4096 * 4), dev.zeros(8), dev.zeros(4), dev.zeros(V * 4)

    def set_logits(self, lg):
        self.dev.write(self.dL, np.ascontiguousarray(lg, np.float32))

    def draw(self, rng, temp=0.0, top_k=0, top_p=1.0, rep=1.0, seen=(), probs=False):
        seen = np.ascontiguousarray(seen, np.int32)
        if seen.size:
            self.dev.write(self.dSeen, np.pad(seen, (0, 4096 - seen.size)))
        self.dev.write(self.dRng, np.array([rng], np.uint64))
        self.k(1, self.dL, self.dSeen, self.dW, self.dM, self.dRng, self.dOut, self.dP if probs else 0, 0, self.V, int(seen.size),
               float(temp), int(top_k), float(top_p), float(rep))
        self.dev.sync()
        tok = int(self.dev.download(self.dOut, 1, np.int32)[0])
        new = int(self.dev.download(self.dRng, 1, np.uint64)[0])
        return (tok, new, self.dev.download(self.dP, self.V, np.float32)) if probs else (tok, new)


def test_greedy_fixtures(dev):
    V = 151936
    s = DevSampler(dev, V)
    lg = np.zeros(V, np.float32); lg[12345] = 9.0
    s.set_logits(lg); assert s.draw(1)[0] == 12345
    lg = np.full(V, -1.0, np.float32); lg[0] = 0.5
    s.set_logits(lg); assert s.draw(1)[0] == 0
    lg = np.full(V, -1.0, np.float32); lg[V - 1] = 0.5
    s.set_logits(lg); assert s.draw(1)[0] == V - 1
    s.set_logits(np.zeros(V, np.float32)); assert s.draw(1)[0] == 0                       # all equal: first
    lg = np.zeros(V, np.float32); lg[100] = lg[5000] = lg[90000] = 3.0
    s.set_logits(lg); assert s.draw(1)[0] == 100                                          # first maximum wins
    tok, rng = s.draw(77)
    assert rng == 77                                                                      # greedy consumes no randomness


def test_determinism_support_and_limits(dev):
    V = 4096
    s = DevSampler(dev, V)
    g = np.random.default_rng(0)
    lg = (g.standard_normal(V) * 2).astype(np.float32)
    s.set_logits(lg)
    def stream(seed, n=64, **kw):
        out, r = [], seed
        for _ in range(n):
            t, r = s.draw(r, **kw)
            out.append(t)
        return out
    assert stream(42, temp=0.8, top_k=50, top_p=0.9) == stream(42, temp=0.8, top_k=50, top_p=0.9)
    assert stream(42, temp=0.8, top_k=50, top_p=0.9) != stream(43, temp=0.8, top_k=50, top_p=0.9)
    top10 = set(np.argsort(-lg, kind="stable")[:10].tolist())
    assert set(stream(5, n=300, temp=1.5, top_k=10)) <= top10                              # top-k support
    # top-p nucleus: {3, 9} hold 0.88 + 0.12 of the mass: p = 0.95 needs both and nothing else
    lg2 = np.full(V, -30.0, np.float32); lg2[3] = 5.0; lg2[9] = 3.0
    s.set_logits(lg2)
    assert set(stream(9, n=300, temp=1.0, top_p=0.95)) == {3, 9}
    tok, _, probs = s.draw(9, temp=1.0, top_p=0.95, probs=True)
    assert abs(probs.sum() - 1.0) < 1e-5 and np.count_nonzero(probs) == 2
    assert set(stream(9, n=100, temp=1.0, top_p=0.5)) == {3}                               # the first entry alone reaches 0.5
    # temperature limits: tiny -> argmax; huge -> close to uniform over a small vocabulary
    s.set_logits(lg)
    assert set(stream(3, n=50, temp=1e-4)) == {int(np.argmax(lg))}


def test_chi_square_matches_softmax(dev):
    V = 8
    s = DevSampler(dev, V)
    lg = np.array([0.1, 1.2, -0.7, 2.0, 0.0, 0.9, -1.5, 0.4], np.float32)
    s.set_logits(lg)
    for temp in (1.0, 0.5):
        p = np.exp((lg - lg.max()).astype(np.float64) / temp); p /= p.sum()
        n, r, counts = 6000, 1234, np.zeros(V)
        for _ in range(n):
            t, r = s.draw(r, temp=temp)
            counts[t] += 1
        chi2 = float(((counts - n * p) ** 2 / (n * p)).sum())
        assert chi2 < 24.32, (temp, chi2)                                                  # df = 7, p = 0.001
    n, r, counts = 4000, 99, np.zeros(V)
    for _ in range(n):
        t, r = s.draw(r, temp=1e4)
        counts[t] += 1
    assert float(((counts - n / V) ** 2 / (n / V)).sum()) < 24.32                          # huge temperature: uniform


def test_repetition_penalty(dev):
    V = 64
    s = DevSampler(dev, V)
    lg = np.linspace(-2, 2, V).astype(np.float32)
    s.set_logits(lg)
    _, _, base = s.draw(1, temp=1.0, probs=True)
    _, _, pen = s.draw(1, temp=1.0, rep=1.5, seen=[5, 60, 5, 60], probs=True)              # duplicates penalise once
    assert pen[60] < base[60] and pen[5] < base[5] and pen[30] > base[30]
    want = lg.copy(); want[5] *= 1.5; want[60] /= 1.5
    p = np.exp((want - want.max()).astype(np.float64)); p /= p.sum()
    assert np.allclose(pen, p, rtol=1e-5, atol=1e-9)
    _, _, same = s.draw(1, temp=1.0, rep=1.0, seen=[5, 60], probs=True)
    assert np.array_equal(same, base)                                                     # penalty 1: identity


def test_agrees_with_the_host_sampler(dev):
    from ainfer_b200 import runtime
    V = 32000
    s = DevSampler(dev, V)
    g = np.random.default_rng(3)
    same = total = 0
    for case in range(12):
        lg = (g.standard_normal(V) * 3).astype(np.float32)
        s.set_logits(lg)
        kw = [dict(temp=1.0), dict(temp=0.7, top_k=40), dict(temp=1.2, top_p=0.9), dict(temp=0.9, top_k=100, top_p=0.8)][case % 4]
        r = 1000 + case
        for _ in range(10):
            t_dev, r_dev = s.draw(r, **kw)
            t_host, r_host, _ = runtime.sample_token(lg, rng=r, **kw)
            assert r_dev == r_host                                                         # the same stream of uniforms
            same += t_dev == t_host
            total += 1
            r = r_host
    assert same >= total - 1, (same, total)


def test_session_sampling(dev):
    from ainfer_b200 import runtime
    model = runtime.Model(dev, "synth:tiny:seed=1")
    sess = runtime.Session(model, 64)
    sess.step(5, 0)
    lg = sess.logits()
    t_dev, r_dev = sess.sample(0.8, top_k=20, top_p=0.95, rep_penalty=1.2, seen=[5, 7], rng=11)
    lgp = runtime.apply_rep_penalty(lg, [5, 7], 1.2)
    t_host, r_host, _ = runtime.sample_token(lgp, temp=0.8, top_k=20, top_p=0.95, rng=11)
    assert (t_dev, r_dev) == (t_host, r_host)
    assert sess.sample(0.0)[0] == int(np.argmax(lg))
    sess.close(); model.close()
