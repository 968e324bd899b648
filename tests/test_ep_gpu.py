"""Expert-parallel MoE block of the runtime (ainfer_ep_*: batched router, device permute, grouped
tensor-core expert GEMMs, un-permute, slot-ordered combine; NCCL send/recv between ranks) against
the CPU oracle's single-token MoE block: every row of the batch bit for bit, with one rank and,
when two GPUs are visible, with two NCCL ranks that each hold half of the experts."""
import os
import socket

import numpy as np
import pytest

import oracle_lib as O

pytestmark = pytest.mark.gpu


def _oracle_rows(preset, seed, layer, res):
    """x[t] = res[t] + MoE(rmsnorm(res[t])) and the routed experts, by the oracle, per row."""
    import json
    cfg = json.loads(O.preset_json(preset))
    H, k = cfg["hidden"], cfg["top_k"]
    om = O.Model(arch_json=O.preset_json(preset), synth_seed=seed)
    pfx = f"model.language_model.layers.{layer}."
    w = O.bf16_to_f32(om.tensor(pfx + "post_attention_layernorm.weight")["data"].view(np.uint16))
    out = np.zeros_like(res)
    routed = np.zeros((res.shape[0], k), np.int32)
    for t in range(res.shape[0]):
        hn, y, gap = np.zeros(H, np.float32), np.zeros(H, np.float32), np.zeros(1, np.float32)
        O.lib().orc_rmsnorm(np.ascontiguousarray(res[t]), np.ascontiguousarray(w), H, float(cfg["rms_eps"]), hn)
        O.lib().orc_moe_block(om.h, pfx.encode(), hn, y, routed[t], gap)
        out[t] = res[t] + y
    om.close()
    return out, routed


def _batch(H, n, seed=5):
    return np.random.default_rng(seed).standard_normal((n, H)).astype(np.float32)


@pytest.mark.parametrize("preset,batch,layer", [("mini", 8, 1), ("mini", 64, 0), ("tiny", 3, 1), ("small", 64, 2)])
def test_one_rank_equals_oracle(preset, batch, layer):
    from ainfer_b200 import cuda_abi, runtime
    dev = cuda_abi.Device(0)
    model = runtime.Model(dev, f"synth:{preset}:seed=2")
    H, k = model.config["hidden"], model.config["top_k"]
    ep = runtime.EpMoe(model, batch)
    res = _batch(H, batch)
    got = ep.layer(layer, res)
    want, routed = _oracle_rows(preset, 2, layer, res)
    assert np.array_equal(ep.read("sel_idx", np.int32).reshape(batch, k + 1)[:, :k], routed)
    assert np.array_equal(got, want)
    counts = ep.read("counts", np.int32)
    n_down = counts[2] + counts[4]                       # experts with few rows + experts with many
    assert counts[0] == batch * k and counts[1] + counts[3] == 2 * n_down
    assert 1 <= n_down <= min(model.config["experts"], batch * k) + 1   # + the shared expert
    # a second layer through the same object, chained (res <- x), equals two oracle layers
    if model.config["text_layers"] > layer + 1:
        ep.write("res", res)
        ep.stack(layer, 2)
        dev.sync()
        want2, _ = _oracle_rows(preset, 2, layer + 1, want)
        assert np.array_equal(ep.read("x", np.float32).reshape(batch, H), want2)
    ep.close(); model.close(); dev.close()


def test_usage_errors():
    from ainfer_b200 import cuda_abi, runtime
    dev = cuda_abi.Device(0)
    model = runtime.Model(dev, "synth:tiny:seed=0")
    for kw in (dict(batch=3, world=2), dict(batch=4096), dict(batch=4, world=2, rank=0)):   # ragged split, too many (row, expert) items, no id
        with pytest.raises(Exception) as e:
            runtime.EpMoe(model, **kw)
        assert "usage" in str(e.value)
    model.close(); dev.close()


def _rank_main(rank, world, conn, q, preset, batch, layer):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    from ainfer_b200 import cuda_abi, runtime
    dev = cuda_abi.Device(rank)
    if rank == 0:
        nid = runtime.ep_unique_id()
        for c in conn:
            c.send_bytes(nid)
    else:
        nid = conn[0].recv_bytes()
    model = runtime.Model(dev, f"synth:{preset}:seed=2")       # replicated weights: same seed on every rank
    H = model.config["hidden"]
    ep = runtime.EpMoe(model, batch, rank=rank, world=world, nccl_id=nid)
    n = batch // world
    res = _batch(H, batch)[rank * n:(rank + 1) * n]
    out = ep.layer(layer, res)
    seg = ep.stack(layer, 1, segments=True)
    q.put((rank, out, ep.read("counts", np.int32), seg))
    ep.close(); model.close(); dev.close()


@pytest.mark.parametrize("preset,batch,layer", [("mini", 16, 1), ("small", 64, 1)])
def test_two_nccl_ranks_equal_oracle(preset, batch, layer):
    from ainfer_b200 import cuda_abi
    if cuda_abi.device_count() < 2:
        pytest.skip("needs two GPUs")
    import multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    a, b = ctx.Pipe()
    procs = [ctx.Process(target=_rank_main, args=(0, 2, [a], q, preset, batch, layer)),
             ctx.Process(target=_rank_main, args=(1, 2, [b], q, preset, batch, layer))]
    for p in procs:
        p.start()
    got = {}
    for _ in procs:
        r, out, counts, seg = q.get(timeout=600)
        got[r] = (out, counts, seg)
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    import json
    H = json.loads(O.preset_json(preset))["hidden"]
    k = json.loads(O.preset_json(preset))["top_k"]
    want, _ = _oracle_rows(preset, 2, layer, _batch(H, batch))
    n = batch // 2
    assert np.array_equal(got[0][0], want[:n]) and np.array_equal(got[1][0], want[n:])
    assert got[0][1][0] + got[1][1][0] == batch * k          # every (token, slot) item computed exactly once
    print(json.dumps({"ep_two_ranks": {"preset": preset, "batch": batch, "items": [int(got[0][1][0]), int(got[1][1][0])],
                                       "segments_ms_rank0": [round(x, 4) for x in got[0][2]]}}))
