"""Chunked prefill (ainfer_session_prefill: up to 192 prompt rows per pass through row-batched
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
                                                   ("mini", 70, [69], 16), ("small", 100, [99], 16),
                                                   ("mini", 461, [460], 0), ("small", 300, [299], 16)])   # passes of 192 rows and a ragged last one
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


def _ep_rank_main(rank, world, conn, q, preset, P):
    import os
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    from ainfer_b200 import cuda_abi, runtime
    dev = cuda_abi.Device(rank)
    if rank == 0:
        nid = runtime.ep_unique_id()
        for c in conn:
            c.send_bytes(nid)
    else:
        nid = conn[0].recv_bytes()
    model = runtime.Model(dev, f"synth:{preset}:seed=4")       # replicated weights: same seed on every rank
    V = model.config["vocab"]
    prompt = np.random.default_rng(100 + rank).integers(0, V, P).astype(np.int32)   # every rank its own sequence
    G = 6
    alone = runtime.Session(model, P + G + 8)
    alone.prefill(prompt[:P - 1])
    ep = runtime.Session(model, P + G + 8)
    ep.prefill_ep(rank, world, nid)
    ep.prefill(prompt[:P - 1])              # passes of 64 / world rows, the MoE block exchanged between the ranks
    same = all(np.array_equal(alone.read(name, dt), ep.read(name, dt)) for name, dt in STATE)
    t_alone = alone.generate(prompt[P - 1:], G, start_pos=P - 1)
    t_ep = ep.generate(prompt[P - 1:], G, start_pos=P - 1)
    q.put((rank, bool(same), t_alone.tolist(), t_ep.tolist()))
    ep.close(); alone.close(); model.close(); dev.close()


@pytest.mark.parametrize("preset,P", [("mini", 101), ("small", 70)])
def test_prefill_with_two_expert_parallel_ranks_equals_one_gpu(preset, P):
    """ainfer_session_prefill_ep: two NCCL ranks prefill their own prompts with the experts split
    between them; each rank's state and the tokens it then generates must be bit-identical to its
    own one-GPU prefill."""
    from ainfer_b200 import cuda_abi
    if cuda_abi.device_count() < 2:
        pytest.skip("needs two GPUs")
    import multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    a, b = ctx.Pipe()
    procs = [ctx.Process(target=_ep_rank_main, args=(0, 2, [a], q, preset, P)),
             ctx.Process(target=_ep_rank_main, args=(1, 2, [b], q, preset, P))]
    for p in procs:
        p.start()
    got = {}
    for _ in procs:
        r, same, t_alone, t_ep = q.get(timeout=600)
        got[r] = (same, t_alone, t_ep)
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    for r in (0, 1):
        assert got[r][0], f"rank {r}: state differs"
        assert got[r][1] == got[r][2], f"rank {r}: tokens differ"
    assert got[0][1] != got[1][1]           # the two ranks really ran different sequences


def test_prefill_ep_usage_errors(dev):
    from ainfer_b200 import runtime
    model = runtime.Model(dev, "synth:tiny:seed=4")
    s = runtime.Session(model, 32)
    for kw in (dict(rank=0, world=3), dict(rank=2, world=2), dict(rank=0, world=2)):   # 64 % world, rank range, no id
        with pytest.raises(RuntimeError) as e:
            s.prefill_ep(kw["rank"], kw["world"], None)
        assert "usage" in str(e.value)
    s.prefill_ep(0, 1, None)                # one rank: the plain prefill
    s.prefill(np.array([1, 2, 3], np.int32))
    s.close(); model.close()
