#!/usr/bin/env python
"""Decode benchmark of the B200 hot path.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (ours): the 80B-A3B-shaped INT4 model filled with seeded synthetic weights directly
in HBM, a seeded random prompt of --prompt-len tokens processed by loop-decode, then greedy
decode at batch 1. A step is one decoded token. The timed region decodes K tokens in at least
five windows that all start at position prompt-len (the DeltaNet state carries over, the KV
window is rewritten), so that the context stays the one the configuration names; every window
is timed with device events on the launching stream. Prints ONE JSON line on rank 0.

--impl reference times the CPU restatement of the reference's operator path (oracle/, kind
"port": the reference's device code needs icpx / Level Zero and its Python paths need an absent
checkpoint) on the host cores, on the same model shape and context. It loads nothing of the
product: the model shape comes from oracle/presets.json, the weights from the oracle's own
generator.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

METRIC = "decode_tokens_per_s_batch1"
UNIT = "tokens/s"
WINDOW = 256
STATE = (("S", np.float32), ("conv", np.float32), ("Kc", np.int8), ("Vc", np.int8), ("Ks", np.uint16), ("Vs", np.uint16))


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs, burst copy)"
        except Exception:
            pass
    return 6650.0, "fallback (6.65 TB/s)"


def prompt_ids(vocab, n, seed=0):
    """Seeded prompt (counter-based draws of the synthetic generator, stream "input.prompt")."""
    M = (1 << 64) - 1

    def mix(z):
        z = (z + 0x9E3779B97F4A7C15) & M
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M
        return z ^ (z >> 31)
    h = 0xCBF29CE484222325
    for b in b"input.prompt":
        h = ((h ^ b) * 0x100000001B3) & M
    key = mix((seed & M) ^ mix(h))
    return np.array([(mix((key + i) & M) >> 32) % vocab for i in range(n)], np.int32)


class ClockSampler:
    """nvidia-smi samples during the timed region (reads only; never changes a GPU setting)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                       "-lms", "50", "-i", str(gpu_index)], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.p = None

    def stop(self):
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except Exception:
            self.p.kill()
        self.f.flush()
        rows = [r.strip().split(", ") for r in open(self.f.name).read().strip().splitlines() if r.strip()]
        os.unlink(self.f.name)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
                for n, v in zip(names, r[5:9]):
                    if v.strip().lower().startswith("active"):
                        reasons.add(n)
            except Exception:
                continue
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def model_bytes_per_token(cfg, ctx):
    """Algorithmic HBM bytes of one batch-1 decode step (INT4 weight = 0.5 B + 2 B / 128)."""
    w = 0.515625
    H, I, V = cfg["hidden"], cfg["expert_intermediate"], cfg["vocab"]
    D, nQ, nKV = cfg["head_dim"], cfg["q_heads"], cfg["kv_heads"]
    nK, nV = cfg["lin_k_heads"], cfg["lin_v_heads"]
    n_lin, n_attn = cfg["layer_types"].count("L"), cfg["layer_types"].count("A")
    C = (2 * nK + nV) * 128
    lin = (C * H + nV * 128 * H + 2 * nV * H + H * nV * 128) * w
    att = (nQ * 2 * D * H + 2 * nKV * D * H + H * nQ * D) * w
    expert = 3 * I * H * w
    router = (cfg["experts"] + 1) * H * 2
    slots = cfg["top_k"] + cfg["shared_experts"]
    state = n_lin * nV * 128 * 128 * 4 * 2
    kv = n_attn * 2 * nKV * (D + 2) * ctx
    return n_lin * lin + n_attn * att + (n_lin + n_attn) * (slots * expert + router) + V * H * w + H * 2 + state + kv


def synthetic_state(osess, cfg, ctx, seed=7):
    """Seeded decode state at context `ctx` for the CPU arm: DeltaNet S ~ N(0, 0.1), conv history
    ~ N(0, 1), INT8 K/V rows uniform in [-127, 127] with fp16 scales near 1/64 (what quantised
    N(0, 1) vectors look like). Timing does not depend on the values."""
    rng = np.random.default_rng(seed)
    nKV, D = cfg["kv_heads"], cfg["head_dim"]
    n_kv = cfg["layer_types"].count("A") + cfg["mtp_layers"]
    S = osess.buf("S"); S[:] = rng.standard_normal(S.size, dtype=np.float32) * 0.1
    cv = osess.buf("conv"); cv[:] = rng.standard_normal(cv.size, dtype=np.float32)
    max_ctx = osess.buf("Ks").size // (n_kv * nKV)
    for name in ("Kc", "Vc"):
        b = osess.buf(name).reshape(n_kv, max_ctx, nKV, D)
        b[:, :ctx] = rng.integers(-127, 128, size=(n_kv, ctx, nKV, D), dtype=np.int8)
    for name in ("Ks", "Vs"):
        b = osess.buf(name).reshape(n_kv, max_ctx, nKV)
        b[:, :ctx] = np.float16(1.0 / 64.0).view(np.uint16)


def run_reference(args):
    """CPU arm: the oracle (port of the reference's host operator math) on all host threads.
    One step = one batch-1 decode token of the same model shape at the same context. The weights
    are the oracle's own lazily generated ones (80 G draws for the whole model is minutes of host
    time), so every step replays the SAME token from the SAME saved state: an untimed first pass
    generates the 3.3 G weights that token touches, the timed passes stream them (2.1 GB per
    step, far more than the host caches hold)."""
    rank, _, world = dist_env()
    if rank != 0:
        return 0
    import oracle_lib as O
    arch = O.preset_json(args.model)
    cfg = json.loads(arch)
    P = args.prompt_len
    t0 = time.time()
    om = O.Model(arch_json=arch, synth_seed=0)
    sess = O.Session(om, P + 8)
    synthetic_state(sess, cfg, P)
    saved = {n: sess.buf(n).copy() for n, _ in STATE}
    tok = int(prompt_ids(cfg["vocab"], 1, seed=5)[0])

    def one():
        for n, _ in STATE:
            sess.buf(n)[:] = saved[n]
        t = time.time()
        sess.step(tok, P, True)
        return time.time() - t
    one()                                   # generates the weights the token touches (not timed)
    t_setup = time.time() - t0
    for _ in range(args.warmup):
        one()
    times = [one() for _ in range(args.steps)]
    dt = float(np.sum(times))
    v = args.steps / dt
    cores = O.lib().orc_threads()
    sample = (f"one batch-1 decode token of the {args.model} model at context {P} (seeded synthetic INT8 KV cache and "
              f"DeltaNet state), replayed {args.steps} times from the same state after {args.warmup} warm-up replays; "
              f"weights from the oracle's own generator, generated in an untimed first pass ({t_setup:.0f} s)")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1000.0 / v, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int4xint8->int32, fp32 rescale", "data": "synthetic",
        "config": workload_config(args.model, P, cfg),
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "repeats": {"n": len(times), "median_ms": float(np.median(times)) * 1e3, "min_ms": float(np.min(times)) * 1e3,
                    "max_ms": float(np.max(times)) * 1e3},
        "gpu_launches": 0}))
    return 0


def workload_config(model, P, cfg):
    if model == "full":
        w = ("full (80B-A3B-shaped INT4 g128, 48 layers 3:1 DeltaNet:GQA, 512 experts top-10 + shared, vocab 151936) "
             f"batch-1 greedy decode at context {P}")
    else:
        w = f"{model} model batch-1 greedy decode at context {P}"
    return {"workload": w, "context": P, "kv_cache": "int8 + fp16 per-token-per-head scales"}


def gemv_probe(dev, N, K, reps=20):
    """Isolated Int4GemvA8 launches on seeded device-generated weights: mean ms per launch of a recorded
    list of `reps` launches rotating over more than 256 MB of distinct weight buffers (cold L2, no host
    launch latency in the figure); thread groups sized by the runtime's own rule."""
    from ainfer_b200 import opbench
    return opbench.gemv_once(dev, N, K, 1, reps)["ms"]


def step_traffic_note():
    """DRAM bytes and algorithmic bytes of one launch of the persistent step as an ncu capture on a
    smaller preset measured them (a data file beside the package; the capture's command is in it)."""
    p = os.path.join(ROOT, "ainfer_b200", "step_traffic.json")
    try:
        j = json.load(open(p))
        return float(j["dram_bytes_per_launch"]), float(j["algorithmic_bytes_per_launch"]), f"ncu capture on the {j['preset']} preset"
    except Exception:
        pass
    return None


def zipf_router_bias(experts, s=1.1, seed=0):
    """log of a Zipf(s) popularity over a seeded permutation of the experts: added to the router
    logits, it skews which experts the top-k picks the way a Zipf(s) load does."""
    rng = np.random.default_rng(seed)
    rank_of = rng.permutation(experts)
    p = 1.0 / np.power(np.arange(1, experts + 1, dtype=np.float64), s)
    p /= p.sum()
    return np.log(p[rank_of]).astype(np.float32)


def run_ep(args, dev, model, rank, world, dist):
    """Batched decode of the MoE layers with the experts sharded over the ranks (expert parallelism):
    a batch of EP_BATCH rows through the MoE block of every layer of the model (post-attention
    norm, router with a Zipf(1.1) bias, top-k, dispatch all-to-all, grouped expert GEMMs, return
    all-to-all, shared expert, combine), each layer feeding the next. Every rank owns batch/world
    rows and experts/world experts. The timed region holds the whole stack, exchanges included;
    device events, max over ranks."""
    from ainfer_b200 import runtime
    cfg = model.config
    B, L = args.ep_batch, cfg["text_layers"]
    if B % world or cfg["experts"] % world:
        return {"skipped": f"batch {B} or {cfg['experts']} experts do not divide over {world} ranks"}
    nid = None
    if world > 1:
        import torch
        t = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            t = torch.frombuffer(bytearray(runtime.ep_unique_id()), dtype=torch.uint8).cuda()
        dist.broadcast(t, 0)
        nid = bytes(t.cpu().numpy().tobytes())
    ep = runtime.EpMoe(model, B, rank=rank, world=world, nccl_id=nid, flags=runtime.EpMoe.ROUTER_BIAS)
    ep.write("router_bias", zipf_router_bias(cfg["experts"]))
    n, H = B // world, cfg["hidden"]
    rows = np.random.default_rng(1234).standard_normal((B, H)).astype(np.float32)[rank * n:(rank + 1) * n]
    ep.write("res", rows)
    for _ in range(max(1, args.ep_warmup)):
        ep.stack(0, L)
    dev.sync()
    if dist is not None:
        dist.barrier()
    passes, ms = [], 0.0
    for _ in range(args.ep_steps):
        e0, e1 = dev.event(), dev.event()
        e0.record()
        ep.stack(0, L)
        e1.record()
        dev.sync()
        passes.append(e0.elapsed_ms(e1))
    items = int(ep.read("counts", np.int32)[0])
    seg = ep.stack(0, L, segments=True)
    if dist is not None:
        import torch
        t = torch.tensor(passes + [float(items)], device="cuda", dtype=torch.float64)
        tmax = t.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        passes, items_max, items_sum = [float(x) for x in tmax[:-1]], float(tmax[-1]), float(t[-1])
    else:
        items_max = items_sum = float(items)
    ep.close()
    # The exchange an all-reduce form of the block would need instead of the two all-to-alls: one
    # fp32 sum of the batch's partial outputs [B][H] over the ranks per layer (the library's
    # collective on the framework's communicator; device events, max over ranks). Not the product
    # path: its sum order is the collective's, not the slot order the parity contract fixes.
    allreduce_us = None
    if dist is not None:
        import torch
        buf = torch.zeros(B * H, device="cuda", dtype=torch.float32)
        for _ in range(10):
            dist.all_reduce(buf)
        torch.cuda.synchronize()
        dist.barrier()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        for _ in range(100):
            dist.all_reduce(buf)
        a1.record()
        torch.cuda.synchronize()
        tt = torch.tensor([a0.elapsed_time(a1) * 10.0], device="cuda", dtype=torch.float64)   # us per call
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        allreduce_us = float(tt[0])
    med = float(np.median(passes))
    I, k = cfg["expert_intermediate"], cfg["top_k"]
    return {"workload": f"batch {B} through the MoE block of {L} layers, experts sharded over {world} rank(s), Zipf(1.1) router bias",
            "tokens_per_s": B / (med / 1000.0), "ms_per_stack": med, "us_per_layer": med * 1000.0 / L,
            "passes_ms": {"n": len(passes), "min": min(passes), "max": max(passes)},
            "scaling": "strong", "batch": B, "layers": L, "world": world,
            "exchange": "NCCL send/recv all-to-all, fixed-size slots" if world > 1 else "none (one rank)",
            "segments_us_per_layer_rank0": dict(zip(("route_pack", "dispatch", "experts", "return", "shared_combine"),
                                                    [round(x * 1000.0 / L, 2) for x in seg])),
            "allreduce_variant_exchange_us_per_layer": allreduce_us,
            "last_layer_items": {"max_rank": items_max, "mean_rank": items_sum / world, "total": B * k},
            "expert_bytes_per_layer_all_ranks_upper": cfg["experts"] * 3 * H * I * (0.5 + 2.0 / 128)}


def run_mtp(args, dev, model, ms_plain):
    """MTP draft / batched-verify rounds (config 3's speculative loop) next to plain greedy decoding:
    same tokens, the cost of a round (draft_k drafts + one pass of draft_k + 1 rows through the trunk +
    rollback) against the same number of plain steps, and the acceptance needed to break even. With
    seeded random weights no draft is ever accepted, so the headline stays the plain loop."""
    from ainfer_b200 import runtime
    cfg = model.config
    if not cfg.get("mtp_layers"):
        return {"skipped": "the model has no MTP head"}
    K, P, G = 3, 64, 33
    prompt = prompt_ids(cfg["vocab"], P, seed=5)
    s = runtime.Session(model, P + 2 * G + 32, runtime.Session.PERSISTENT)
    want = s.generate(prompt, G)
    s.reset()
    s.generate_mtp(prompt, 2 * K + 4, draft_k=K)          # creates the verifier and records its lists (untimed)
    s.reset(); dev.sync()
    t0 = time.time(); s.generate_mtp(prompt, 1, draft_k=K); t_prompt = time.time() - t0
    s.reset(); dev.sync()
    t0 = time.time(); got, st = s.generate_mtp(prompt, G, draft_k=K); t_all = time.time() - t0
    s.close()
    round_ms = (t_all - t_prompt) * 1000.0 / max(st["rounds"], 1)
    return {"draft_k": K, "rows_per_verify_pass": K + 1, "generated": G, "tokens_equal_plain_greedy": got.tolist() == want.tolist(),
            "stats": st, "round_ms": round_ms, "plain_ms_for_the_same_rows": ms_plain * (K + 1),
            "tokens_per_round_to_break_even": round_ms / ms_plain,
            "note": "seeded random weights: no draft is accepted, every round yields one token"}


def run_batch(args, dev, model, rank, world, dist):
    """Batched decode (the metric's batch-64 half): BATCH sequences, each at a long context with an
    INT8 KV cache, advance one greedy token per step. Sequences are split over the ranks (state and
    caches live with their owner); the MoE layers run expert-parallel with a Zipf(1.1) router bias.
    The caches are filled with a seeded pattern (no 32 k-token prompt is decoded for each of 64
    sequences); the timed region is whole steps: mixers, exchanges, LM head, argmax; device
    events, max over ranks."""
    from ainfer_b200 import runtime
    cfg = model.config
    B, ctx = args.batch, args.batch_ctx
    if B % world or cfg["experts"] % world:
        return {"skipped": f"batch {B} or {cfg['experts']} experts do not divide over {world} ranks"}
    nid = None
    if world > 1:
        import torch
        t = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            t = torch.frombuffer(bytearray(runtime.ep_unique_id()), dtype=torch.uint8).cuda()
        dist.broadcast(t, 0)
        nid = bytes(t.cpu().numpy().tobytes())
    steps, warm = args.batch_steps, max(1, args.batch_warmup)
    max_ctx = ctx + steps + warm + 8
    try:
        bd = runtime.BatchDecode(model, B, max_ctx, rank=rank, world=world, nccl_id=nid, flags=runtime.BatchDecode.ROUTER_BIAS)
    except Exception as e:
        return {"skipped": f"cannot create the batch engine: {str(e)[:200]}"}
    n = B // world
    bd.write("router_bias", zipf_router_bias(cfg["experts"]))
    rng = np.random.default_rng(4321 + rank)
    # seeded cache contents: a 32 MB block of INT8 values, and fp16 scales near 0.02, repeated
    block = rng.integers(-127, 128, 32 << 20, dtype=np.int8)
    sblock = (0x2000 + rng.integers(0, 0x400, 1 << 20)).astype(np.uint16)     # fp16 in [0.0078, 0.0156)
    for name, src in (("Kc", block), ("Vc", block[::-1].copy()), ("Ks", sblock), ("Vs", sblock[::-1].copy())):
        p, nb = bd.buffer(name)
        raw = src.view(np.uint8)
        d0 = dev.upload(raw)
        off = 0
        while off < nb:
            m = min(raw.nbytes, nb - off)
            dev.copy_d2d(p + off, d0, m)
            off += m
        dev.free(d0)
    bd.write("S", (rng.standard_normal(bd.buffer("S")[1] // 4) * 0.1).astype(np.float32))
    bd.set_inputs(rng.integers(0, cfg["vocab"], n), np.full(n, ctx, np.int32))
    for _ in range(warm):
        bd.step()
    dev.sync()
    if dist is not None:
        dist.barrier()
    passes = []
    for _ in range(steps):
        e0, e1 = dev.event(), dev.event()
        e0.record()
        bd.step()
        e1.record()
        dev.sync()
        passes.append(e0.elapsed_ms(e1))
    toks = bd.tokens()
    total_ms = float(sum(passes))
    if dist is not None:
        import torch
        t = torch.tensor([total_ms] + passes, device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, passes = float(t[0]), [float(x) for x in t[1:]]
    bd.close()
    nkv, D = cfg["kv_heads"], cfg["head_dim"]
    n_attn = cfg["layer_types"].count("A")
    kv_bytes = B * n_attn * ctx * nkv * (2 * D + 4)
    return {"workload": f"batch {B} greedy decode, every sequence at context {ctx} (INT8 KV), sequences and experts split over {world} rank(s), Zipf(1.1) router bias",
            "tokens_per_s": B * steps / (total_ms / 1000.0), "ms_per_step": total_ms / steps,
            "passes_ms": {"n": len(passes), "median": float(np.median(passes)), "min": min(passes), "max": max(passes)},
            "scaling": "strong", "batch": B, "context": ctx, "world": world, "steps": steps, "warmup": warm,
            "kv_bytes_per_step_all_ranks": kv_bytes, "first_tokens_rank0": [int(x) for x in toks[:4]],
            "cache_fill": "seeded INT8 pattern and fp16 scales (not decoded prompts)"}


def run_prefill_ep(args, dev, model, rank, world, dist):
    """Prefill with expert parallelism (N > 1): every rank prefills its own seeded prompt of the same
    length, passes of 64 / N rows, the MoE block of each pass exchanged between the ranks (NCCL
    all-to-all inside the timed region). Wall clock around the call after a device sync, max over ranks."""
    from ainfer_b200 import runtime
    if world == 1 or 64 % world or model.config["experts"] % world:
        return None
    import torch
    t = torch.zeros(128, dtype=torch.uint8, device="cuda")
    if rank == 0:
        t = torch.frombuffer(bytearray(runtime.ep_unique_id()), dtype=torch.uint8).cuda()
    dist.broadcast(t, 0)
    nid = bytes(t.cpu().numpy().tobytes())
    n_tok = args.prefill_ep_tokens
    try:
        sess = runtime.Session(model, n_tok + 16)
        sess.prefill_ep(rank, world, nid)
        prompt = prompt_ids(model.config["vocab"], n_tok, seed=100 + rank)
        sess.prefill(prompt[:64])     # creates the row buffers and the communicator, records the MoE lists
        sess.reset()
        dev.sync()
        dist.barrier()
        t0 = time.time()
        sess.prefill(prompt)
        dev.sync()
        sec = time.time() - t0
    except Exception as e:
        return {"skipped": f"expert-parallel prefill failed: {str(e)[:200]}"}
    tt = torch.tensor([sec], device="cuda", dtype=torch.float64)
    dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    sec = float(tt[0])
    sess.close()
    most = max(1, 2048 // (model.config["top_k"] * world))
    rows_pp = min(192, most // 8 * 8 if most >= 8 else most)     # the runtime's default
    return {"workload": f"prefill of {n_tok} seeded tokens on each of {world} ranks (one sequence per rank), passes of {rows_pp} rows, experts split over the ranks",
            "tokens_per_s": world * n_tok / sec, "seconds": sec, "prompt_tokens_per_rank": n_tok, "world": world,
            "rows_per_pass": rows_pp, "scaling": "weak"}


def run_ours(args):
    rank, local_rank, world = dist_env()
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        import datetime
        # a short timeout: a rank that leaves early must end the others' next collective, not hang them
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank),
                                timeout=datetime.timedelta(seconds=180))
    from ainfer_b200 import cuda_abi, runtime
    dev = cuda_abi.Device(local_rank)
    t_load = time.time()
    model = runtime.Model(dev, f"synth:{args.model}:seed=0")   # same weights on every rank (the experts are sharded below)
    cfg = model.config
    t_load = time.time() - t_load
    P = args.prompt_len
    max_ctx = P + WINDOW + 8
    persistent = not args.list
    sess = runtime.Session(model, max_ctx, runtime.Session.PERSISTENT if persistent else runtime.Session.MULTI_KERNEL)
    prompt = prompt_ids(cfg["vocab"], P, seed=rank)

    def barrier():
        dev.sync()
        if dist is not None:
            dist.barrier()

    t_prompt_only = 0.0
    t_prompt = time.time()
    if args.loop_prompt:
        last = int(sess.generate(prompt, 1)[0])      # whole prompt token by token + first token
    else:
        sess.prefill(prompt[:2])                     # creates the row buffers and records the MoE lists (untimed)
        sess.reset()
        dev.sync()
        t_pf = time.time()
        sess.prefill(prompt[:-1])                    # chunked prefill (state identical to token-by-token decoding)
        t_prompt_only = time.time() - t_pf
        last = int(sess.generate(prompt[-1:], 1, start_pos=P - 1)[0])
    t_prompt = time.time() - t_prompt
    if args.warmup > 0:
        sess.generate(np.array([last], np.int32), args.warmup, start_pos=P)
    # ---- timed: K steps in >= 5 windows that start at position P, each timed with device events ----
    nwin = max(5, -(-args.steps // WINDOW))
    sizes = [args.steps // nwin + (1 if i < args.steps % nwin else 0) for i in range(nwin)]
    sizes = [n for n in sizes if n > 0]
    barrier()
    clocks = ClockSampler(local_rank) if rank == 0 else None
    gen_ms, toks0, win_ms = 0.0, None, []
    t_wall = time.time()
    for n in sizes:
        toks, ms = sess.generate(np.array([last], np.int32), n, start_pos=P, timed=True)
        if toks0 is None:
            toks0 = toks.copy()
        gen_ms += ms
        win_ms.append(ms / n)
    barrier()
    t_wall = time.time() - t_wall
    clk = clocks.stop() if clocks else None
    # ---- e2e: one public-API call per token, host control write + token readback every step ----
    barrier()
    n_e2e = min(args.steps, WINDOW)
    tok, t_e2e = last, time.time()
    for i in range(n_e2e):
        tok = sess.step(tok, P + i)
    dev.sync()
    t_e2e = time.time() - t_e2e
    if dist is not None:
        import torch
        t = torch.tensor([gen_ms, t_e2e], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        gen_ms, t_e2e = float(t[0]), float(t[1])
    ep_line = None if args.no_ep else run_ep(args, dev, model, rank, world, dist)
    batch_line = None if args.no_batch else run_batch(args, dev, model, rank, world, dist)
    prefill_ep_line = None if (args.no_batch or world == 1) else run_prefill_ep(args, dev, model, rank, world, dist)
    mtp_line = None
    if rank == 0 and not args.no_mtp:
        try:
            mtp_line = run_mtp(args, dev, model, gen_ms / args.steps)
        except Exception as e:
            mtp_line = {"error": str(e)[:200]}
    if rank != 0:
        model.close(); dev.close()
        dist.destroy_process_group()
        return 0
    value = world * args.steps / (gen_ms / 1000.0)
    e2e_value = world * n_e2e / t_e2e
    ms_step = gen_ms / args.steps
    bytes_tok = model_bytes_per_token(cfg, P)
    peak, peak_src = measured_peak()
    launches = int(sess.launches_per_token())
    # ---- roofline of the kernel that dominates the step ----
    # Persistent step: the timed region is one DecodeStep launch per token, so that kernel IS the
    # step; its launch duration is the event time per step and its algorithmic bytes are the token's.
    if persistent:
        roof = {"bound": "hbm", "kernel": "DecodeStep (one persistent launch per token: all layers, LM head, argmax)",
                "share_of_step": 1.0, "achieved": bytes_tok / ms_step / 1e6, "peak": peak, "unit": "GB/s",
                "frac": bytes_tok / ms_step / 1e6 / peak, "peak_source": peak_src,
                "algorithmic_bytes_per_launch": bytes_tok, "launch_ms": ms_step, "traffic": None}
        tr = step_traffic_note()
        if tr:
            # measured on a smaller model; DRAM traffic of this kernel grows with the bytes it must read
            roof["traffic"] = tr[0] / tr[1] * bytes_tok
            roof["traffic_source"] = f"{tr[2]}: dram bytes / algorithmic bytes = {tr[0] / tr[1]:.3f} on the small model, scaled"
    else:
        roof = {"bound": "hbm", "kernel": "whole recorded list (several hundred launches per token)", "achieved": bytes_tok / ms_step / 1e6,
                "peak": peak, "unit": "GB/s", "frac": bytes_tok / ms_step / 1e6 / peak, "peak_source": peak_src,
                "algorithmic_bytes_per_launch": bytes_tok / max(launches, 1), "traffic": None}
    sweep = []
    if not args.no_sweep:
        try:
            for (N, K) in [(cfg["vocab"], cfg["hidden"]), (8192, 2048), (4096, 2048), (512, 2048), (2048, 512)]:
                ms = gemv_probe(dev, N, K)
                b = N * K * 0.515625 + K * 1 + (K // 128) * 4 + N * 4
                sweep.append({"kernel": "Int4GemvA8", "N": N, "K": K, "M": 1, "ms": ms, "gbs": b / ms / 1e6, "frac": b / ms / 1e6 / peak})
        except Exception as e:     # the probe must never take the decode number down with it
            sweep = [{"error": str(e)[:200]}]
    # ---- CPU baseline: the oracle on the host cores, on the SAME weights (copied from the device
    # ---- once) and from the GPU session's state at position P; also a token-by-token parity check ----
    cpu = None
    parity = None
    if not args.no_cpu:
        try:
            import oracle_lib as O
            t0 = time.time()
            om = O.model_from_device(dev, model)
            t_copy = time.time() - t0
            osess = O.Session(om, max_ctx)
            sess.reset()
            sess.prefill(prompt[:-1])
            first = int(sess.generate(prompt[-1:], 1, start_pos=P - 1)[0])
            state = {n: sess.read(n, dt) for n, dt in STATE}
            n_cpu = args.cpu_steps
            gpu_toks = sess.generate(np.array([first], np.int32), n_cpu, start_pos=P)
            for n, _ in STATE:
                osess.buf(n)[:] = state[n]
            osess.step(first, P, True)          # untimed warm-up token
            for n, _ in STATE:
                osess.buf(n)[:] = state[n]
            t0 = time.time()
            cpu_toks, tok = [], first
            for i in range(n_cpu):
                tok = osess.step(tok, P + i, True)
                cpu_toks.append(tok)
            dt_cpu = time.time() - t0
            cpu = {"value": n_cpu / dt_cpu, "unit": UNIT, "cores": O.lib().orc_threads(), "kind": "port",
                   "sample": f"{n_cpu} greedy decode tokens of the {args.model} model at context {P}, from the GPU "
                             f"session's state after the {P}-token prompt, on host copies of the device's weight "
                             f"arenas (copied in {t_copy:.0f} s, not timed); one untimed warm-up token"}
            parity = {"tokens_compared": n_cpu, "tokens_match": [int(t) for t in gpu_toks] == cpu_toks}
            osess.close(); om.close()
        except Exception as e:
            cpu = {"value": None, "unit": UNIT, "cores": None, "kind": "port", "sample": f"failed: {str(e)[:300]}"}
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int4xint8->int32, fp32 rescale", "data": "synthetic",
        "config": dict(workload_config(args.model, P, cfg),
                       mtp="off in the timed steps (measured separately in `mtp`)", step=("one persistent cooperative launch per token (DecodeStep)" if persistent else
                                        "one recorded list of stand-alone launches chained by programmatic dependencies"),
                       parallelism=("batch-1 steps: one independent replica per GPU (the batch-1 path has no exchange); "
                                    "the `ep` object times the sharded MoE layers") if world > 1 else "single GPU",
                       l2="inputs larger than L2: about 2.1 GB of weights and state streamed per step",
                       launches_per_token=launches),
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": 16, "d2h_bytes_per_step": 4,
                "steps": n_e2e, "api": "ainfer_session_step (control write + replay + token readback)"},
        "gpu_launches": launches * args.steps,
        "repeats": {"windows": len(win_ms), "ms_per_step_median": float(np.median(win_ms)), "ms_per_step_min": float(np.min(win_ms)),
                    "ms_per_step_max": float(np.max(win_ms))},
        "clocks": clk, "roofline": roof, "gemv_sweep": sweep,
        "cpu_baseline": cpu, "parity": parity, "ep": ep_line, "batch_decode": batch_line, "mtp": mtp_line,
        "prefill_ep": prefill_ep_line,
        "prefill": None if args.loop_prompt else {"prompt_tokens": P - 1, "seconds": t_prompt_only, "tokens_per_s": (P - 1) / max(t_prompt_only, 1e-9),
                                                  "how": "chunked prefill, up to 192 rows per pass, one sequence (wall clock around the call, this rank)"},
        "timing": {"model_fill_s": t_load, "prompt_s": t_prompt, "prompt_by": "token-by-token decode" if args.loop_prompt else "chunked prefill (up to 192 rows per pass)", "timed_wall_s": t_wall, "first_tokens": [int(t) for t in toks0[:8]]},
    }
    print(json.dumps(line))
    sess.close(); model.close(); dev.close()
    if dist is not None:
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1024)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="full")
    ap.add_argument("--prompt-len", type=int, default=4096)
    ap.add_argument("--cpu-steps", type=int, default=16)
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-sweep", action="store_true", help="skip the isolated GEMV probes")
    ap.add_argument("--loop-prompt", action="store_true", help="run the prompt token by token instead of by chunked prefill")
    ap.add_argument("--no-mtp", action="store_true", help="skip the MTP round measurement")
    ap.add_argument("--no-batch", action="store_true", help="skip the batched decode measurement")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--batch-ctx", type=int, default=32768)
    ap.add_argument("--batch-steps", type=int, default=8)
    ap.add_argument("--batch-warmup", type=int, default=2)
    ap.add_argument("--prefill-ep-tokens", type=int, default=1024, help="prompt length per rank of the expert-parallel prefill (N > 1)")
    ap.add_argument("--no-ep", action="store_true", help="skip the expert-parallel MoE stack")
    ap.add_argument("--ep-batch", type=int, default=64)
    ap.add_argument("--ep-steps", type=int, default=5)
    ap.add_argument("--ep-warmup", type=int, default=2)
    ap.add_argument("--list", action="store_true", help="time the recorded list of stand-alone launches instead of the persistent step")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        if args.steps > 64:
            args.steps = 64      # every step is the same replayed token; more of them add nothing
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
