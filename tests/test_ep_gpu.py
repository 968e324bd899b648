"""Expert-parallel MoE block on GPUs: the per-item decomposition (route, one expert at a time,
slot-ordered combine) must equal the fused single-GPU kernels bit for bit, and two NCCL ranks
(when two GPUs are visible) must reproduce it for a whole batch."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _batch(H, n, seed=5):
    return np.random.default_rng(seed).standard_normal((n, H)).astype(np.float32)


def test_single_gpu_decomposition_equals_fused_kernels():
    from ainfer_b200 import cuda_abi, ep, runtime
    dev = cuda_abi.Device(0)
    model = runtime.Model(dev, "synth:mini:seed=2")
    b = ep.GpuMoeBackend(dev, model, layer=1)
    res = _batch(b.hidden, 6)
    got = ep.EpMoeBlock(b, ep.LocalComm()).forward(res)
    for t in range(res.shape[0]):
        assert np.array_equal(got[t], b.fused_reference(res[t])), f"token {t}"
    model.close(); dev.close()


def _rank_main(rank, world, port, q):
    import torch
    import torch.distributed as dist
    from ainfer_b200 import cuda_abi, ep, runtime
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        dev = cuda_abi.Device(rank)
        model = runtime.Model(dev, "synth:mini:seed=2")       # replicated weights: same seed on every rank
        b = ep.GpuMoeBackend(dev, model, layer=1)
        res = _batch(b.hidden, 8)
        blk = ep.EpMoeBlock(b, ep.TorchComm(device=torch.device("cuda", rank)))
        out = blk.forward(res)
        want = np.stack([b.fused_reference(res[t]) for t in range(res.shape[0])]) if rank == 0 else None
        q.put((rank, out, want, blk.stats))
        model.close(); dev.close()
    finally:
        dist.destroy_process_group()


def test_two_nccl_ranks_equal_single_gpu():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = {}
    for _ in procs:
        r, out, want, stats = q.get(timeout=600)
        got[r] = (out, want, stats)
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    want = got[0][1]
    assert np.array_equal(got[0][0], want) and np.array_equal(got[1][0], want)
    assert got[0][2]["items_computed"] + got[1][2]["items_computed"] == 8 * 4
