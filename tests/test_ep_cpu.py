"""Expert-parallel MoE block, host logic: two gloo ranks on the CPU (arithmetic by the oracle)
must reproduce, bit for bit, the block computed by one rank that holds every expert; plus unit
checks of ownership and the dispatch plan (ragged and empty cases)."""
import os
import socket
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(__file__))

import ep_harness as ep


def test_ownership_and_plan_edges():
    assert [ep.owned_range(5, r, 2) for r in range(2)] == [(0, 3), (3, 5)]
    assert [ep.owned_range(1, r, 4) for r in range(4)] == [(0, 1), (1, 1), (1, 1), (1, 1)]   # ranks without tokens
    assert [ep.expert_owner(e, 8, 4) for e in range(8)] == [0, 0, 1, 1, 2, 2, 3, 3]
    sel = np.array([[7, 0], [1, 6], [3, 2]], np.int32)
    plans = ep.plan_dispatch(sel, token0=10, experts=8, world=2)
    assert [tuple(x) for x in plans[0][["token", "slot", "expert"]]] == [(10, 1, 0), (11, 0, 1), (12, 0, 3), (12, 1, 2)]
    assert [tuple(x) for x in plans[1][["token", "slot", "expert"]]] == [(10, 0, 7), (11, 1, 6)]
    empty = ep.plan_dispatch(np.zeros((0, 2), np.int32), 0, 8, 2)
    assert all(len(p) == 0 for p in empty)


def _rank_main(rank, world, port, batch, q):
    import torch.distributed as dist
    from ep_oracle_backend import OracleMoeBackend
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        b = OracleMoeBackend(256, 8, 2, 128, seed=7)
        res = np.random.default_rng(99).standard_normal((batch, 256)).astype(np.float32)
        blk = ep.EpMoeBlock(b, ep.TorchComm())
        out = blk.forward(res)
        lo = 8 // world * rank
        routed_here = [e for e in b.calls if e < 8]
        assert all(lo <= e < lo + 8 // world for e in routed_here), "an expert of another rank's shard was computed here"
        q.put((rank, out, blk.stats))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("batch", [5, 1])
def test_two_gloo_ranks_equal_one_rank(batch):
    import torch.multiprocessing as mp
    from ep_oracle_backend import OracleMoeBackend
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, batch, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict()
    for _ in procs:
        r, out, stats = q.get(timeout=240)
        got[r] = (out, stats)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    # one rank holding every expert
    b = OracleMoeBackend(256, 8, 2, 128, seed=7)
    res = np.random.default_rng(99).standard_normal((batch, 256)).astype(np.float32)
    want = ep.EpMoeBlock(b, ep.LocalComm()).forward(res)
    assert np.array_equal(got[0][0], want) and np.array_equal(got[1][0], want)
    assert got[0][1]["owned_tokens"] + got[1][1]["owned_tokens"] == batch
    assert got[0][1]["items_computed"] + got[1][1]["items_computed"] == batch * 2   # every (token, slot) exactly once
