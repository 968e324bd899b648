"""Chunked prefill (ainfer_session_prefill: up to 64 prompt rows per pass through row-batched
kernels: tensor-core GEMMs, DeltaNet chunk kernels, per-row attention, the batched MoE block)
against token-by-token decoding of the same prompt: the tokens generated afterwards and the whole
session state (DeltaNet state, conv history, INT8 KV cache and its scales) must be bit-identical."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

STATE = (("S", np.float32), ("conv", np.float32), ("Kc", np.int8), ("Vc", np.int8), ("Ks", np.uint16), ("Vs", np.uint16))


@pytest.fixture(scope="module")
def dev():
    from ainfer_b200 import cuda_abi
    d = cuda_abi.Device(0)
    yield d
    d.close()


@pytest.mark.parametrize("preset,P,splits,flags", [("tiny", 150, [149], 0), ("mini", 131, [64, 1, 65], 0),
                                                   ("mini", 70, [69], 16), ("small", 100, [99], 16)])
def test_prefill_equals_token_by_token_decode(dev, preset, P, splits, flags):
    from ainfer_b200 import runtime
    model = runtime.Model(dev, f"synth:{preset}:seed=4")
    V = model.config["vocab"]
    prompt = np.random.default_rng(P).integers(0, V, P).astype(np.int32)
    G = 8
    a = runtime.Session(model, P + G + 8, flags)
    want = a.generate(prompt, G)
    b = runtime.Session(model, P + G + 8, flags)
    pos = 0
    for n in splits:                      # several calls: the state carries over, chunks of 64 inside a call
        b.prefill(prompt[pos:pos + n], start_pos=pos)
        pos += n
    assert pos == P - 1
    # the state after the prompt's first P - 1 tokens equals a decode session's at the same point
    c = runtime.Session(model, P + G + 8, flags)
    for i in range(P - 1):
        c.step(int(prompt[i]), i)
    for name, dt in STATE:
        assert np.array_equal(b.read(name, dt), c.read(name, dt)), name
    got = b.generate(prompt[P - 1:], G, start_pos=P - 1)
    assert got.tolist() == want.tolist()
    for name, dt in STATE:
        assert np.array_equal(a.read(name, dt), b.read(name, dt)), name
    a.close(); b.close(); c.close(); model.close()


def test_prefill_rejects_context_overflow(dev):
    from ainfer_b200 import runtime
    model = runtime.Model(dev, "synth:tiny:seed=0")
    s = runtime.Session(model, 32)
    with pytest.raises(Exception) as e:
        s.prefill(np.zeros(40, np.int32))
    assert "context overflow" in str(e.value)
    s.close(); model.close()
