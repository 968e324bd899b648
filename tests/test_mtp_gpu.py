"""MTP head on the GPU against the CPU oracle: single drafts (token and logits, bit for bit),
chained drafts, and the draft/verify generation loop (tokens identical to plain greedy decoding,
statistics identical to the same loop run on the oracle; the trunk verifies a round's rows in one
batched pass and rolls its recurrent state back to the last accepted row)."""
import ctypes as C

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


@pytest.fixture(scope="module", params=["tiny", "mini-mtp"])
def mtp_file(request, tmp_path_factory):
    from ainfer_b200 import runtime
    p = str(tmp_path_factory.mktemp("mtp") / f"{request.param}.binfer")
    runtime.synth_write(p, request.param, seed=3)
    return p


def oracle_mtp(osess, tok, pos, h, V):
    logits = np.zeros(V, np.float32)
    d = O.lib().orc_mtp_step(osess.h, int(tok), int(pos), h, logits)
    return d, logits


def test_mtp_drafts_match_oracle(dev, mtp_file):
    from ainfer_b200 import runtime
    model = runtime.Model(dev, mtp_file)
    V = model.config["vocab"]
    sess = runtime.Session(model, 64)
    om = O.Model(path=mtp_file)
    osess = O.Session(om, 64)
    prompt = [5, 77, 300 % V, 12]
    y = yo = -1
    for i, t in enumerate(prompt):
        y = sess.step(t, i)
        yo = osess.step(t, i)
    assert y == yo
    p = len(prompt) - 1
    h = osess.buf("hidden").copy()          # the oracle's final residual of the last trunk step
    inp = y
    for i in range(3):                       # a chain of three drafts
        d = sess.mtp_draft(inp, p + 1 + i, from_trunk=(i == 0))
        do, lo = oracle_mtp(osess, inp, p + 1 + i, h, V)   # h is updated in place (chained)
        assert d == do, f"draft {i}"
        assert np.array_equal(sess.mtp_logits(), lo), f"draft {i} logits"
        assert np.array_equal(sess.read("mtp_hidden", np.float32), h), f"draft {i} hidden"
        inp = d
    # the trunk is untouched by drafting: its next step still matches the oracle
    assert sess.step(y, p + 1) == osess.step(y, p + 1)
    sess.close(); model.close(); osess.close(); om.close()


def test_generate_mtp_equals_greedy_and_oracle_loop(dev, mtp_file):
    from ainfer_b200 import runtime
    model = runtime.Model(dev, mtp_file)
    V = model.config["vocab"]
    prompt = np.array([9, 41, 7, 300 % V, 2], np.int32)
    G, K = 24, 3
    plain = runtime.Session(model, 64)
    want = plain.generate(prompt, G)
    plain.close()
    sess = runtime.Session(model, 64)
    got, st = sess.generate_mtp(prompt, G, draft_k=K)
    assert got.tolist() == want.tolist()
    # the same loop on the oracle: the head runs after every trunk step on (next token, h), so
    # that its own cache holds a true row for every position
    om = O.Model(path=mtp_file)
    osess = O.Session(om, 64)
    y = d = -1
    for i, t in enumerate(prompt):
        y = osess.step(int(t), i)
        h = osess.buf("hidden").copy()
        d, _ = oracle_mtp(osess, int(prompt[i + 1]) if i + 1 < len(prompt) else y, i + 1, h, V)
    p, out = len(prompt) - 1, [y]
    rounds = drafted = accepted = 0
    while len(out) < G:
        # a round: the accepted token and up to K drafts are verified together; the oracle (which
        # never speculates) feeds the same rows one by one and stops at the first rejected draft
        rows = min(K + 1, G - len(out))
        feed = [y] + ([d] if rows > 1 else [])
        for i in range(2, rows):
            dd, _ = oracle_mtp(osess, feed[i - 1], p + i, h, V)   # h: the head's own chained state
            feed.append(dd)
        rounds += 1
        drafted += rows - 1
        preds, j = [], 0
        for i in range(rows):
            t = osess.step(feed[i], p + 1 + i)
            preds.append((t, osess.buf("hidden").copy()))
            if i < rows - 1 and feed[i + 1] == t:
                j += 1
            else:
                break
        accepted += j
        for i in range(j + 1):
            h = preds[i][1].copy()
            d, _ = oracle_mtp(osess, preds[i][0], p + 2 + i, h, V)
            out.append(preds[i][0])
        p += j + 1
        y = preds[j][0]
    assert out == got.tolist()
    assert st == {"rounds": rounds, "drafted": drafted, "accepted": accepted}
    # the head's own KV slot (the last one): every row up to the last position it ran at is a
    # true row, non-empty and equal to the oracle's
    cfg = model.config
    n_slots = cfg["layer_types"].count("A") + cfg["mtp_layers"]
    for name, dt in (("Kc", np.int8), ("Vc", np.int8), ("Ks", np.uint16), ("Vs", np.uint16)):
        a = sess.read(name, dt).reshape(n_slots, 64, -1)[-1]
        b = osess.buf(name).reshape(n_slots, 64, -1)[-1]
        assert np.array_equal(a[:p + 2], b[:p + 2]), name
        if name in ("Kc", "Vc"):
            assert all(np.any(a[r] != 0) for r in range(1, p + 2)), f"{name}: empty row in the head's cache"
    sess.close(); model.close(); osess.close(); om.close()


def test_mtp_calls_fail_cleanly_without_a_head(dev, tmp_path):
    from ainfer_b200 import runtime
    model = runtime.Model(dev, "synth:mini:seed=0")   # mini has no MTP head
    sess = runtime.Session(model, 32)
    sess.step(1, 0)
    with pytest.raises(Exception) as e:
        sess.mtp_draft(1, 1)
    assert "no MTP head" in str(e.value)
    sess.close(); model.close()
