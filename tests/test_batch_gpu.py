"""Batched decode (ainfer_batch_*): several sequences with different prompts and lengths advance
together, one token each per step, every sequence with its own DeltaNet state, conv history and
INT8 KV cache. Each sequence must produce exactly the tokens and logits it produces when decoded
alone by a session, and leave the same state."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    from ainfer_b200 import cuda_abi
    d = cuda_abi.Device(0)
    yield d
    d.close()


@pytest.mark.parametrize("preset,B", [("tiny", 3), ("mini", 5), ("small", 64)])
def test_batch_equals_sequences_decoded_alone(dev, preset, B):
    from ainfer_b200 import runtime
    model = runtime.Model(dev, f"synth:{preset}:seed=6")
    cfg = model.config
    V = cfg["vocab"]
    rng = np.random.default_rng(B)
    steps = 12 if B <= 8 else 6
    max_ctx = 40
    # sequence b starts at its own position p0[b] (as if it had a history of that length: the
    # caches below that position are zero on both sides) and is fed its own token stream
    feed = rng.integers(0, V, (B, 4)).astype(np.int32)      # the first 4 inputs are forced, then greedy
    bd = runtime.BatchDecode(model, B, max_ctx)
    tok = feed[:, 0].copy()
    pos = np.zeros(B, np.int32)
    got = np.zeros((B, steps), np.int32)
    logits_last = None
    for i in range(steps):
        if i < 4:
            bd.set_inputs(feed[:, i], pos)      # forced input; afterwards the device-advanced block feeds the greedy token
        bd.step()
        got[:, i] = bd.tokens()
        pos += 1
    logits_last = bd.read("logits", np.float32).reshape(B, V)
    check = range(B) if B <= 8 else (0, 17, 63)
    H = cfg["hidden"]
    for b in check:
        s = runtime.Session(model, max_ctx)
        t = None
        for i in range(steps):
            t = s.step(int(feed[b, i]) if i < 4 else int(t), i)
            assert t == got[b, i], (b, i)
        assert np.array_equal(s.logits(), logits_last[b]), b
        for name, dt in (("S", np.float32), ("conv", np.float32), ("Kc", np.int8), ("Ks", np.uint16), ("Vc", np.int8), ("Vs", np.uint16)):
            mine = bd.read(name, dt).reshape(B, -1)[b]
            alone = s.read(name, dt)
            if name in ("Kc", "Vc", "Ks", "Vs"):
                # the session's cache may hold one more slot (an MTP head's); compare the trunk's layers
                n_attn = cfg["layer_types"].count("A")
                alone = alone.reshape(-1, alone.size // (n_attn + cfg["mtp_layers"]))[:n_attn].reshape(-1)
            assert np.array_equal(mine, alone), (name, b)
        s.close()
    bd.close(); model.close()
