#!/usr/bin/env python
"""Decode benchmark of the B200 hot path.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (ours): the 80B-A3B-shaped INT4 model filled with seeded synthetic
weights directly in HBM, a seeded random prompt of --prompt-len tokens
processed by loop-decode, then greedy decode at batch 1. A step is one decoded
token. The timed region decodes K tokens in windows of 256 that all start at
position prompt-len (the DeltaNet state carries over, the KV window is
rewritten), so that the context stays the one the configuration names.
Prints ONE JSON line on rank 0.

--impl reference times the CPU restatement of the reference's operator path
(oracle/, kind "port": the reference's device code needs icpx/Level Zero and
its Python paths need an absent checkpoint) on the host cores.
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


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        except Exception:
            pass
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


def seeded_prompt(vocab, n, seed=0):
    import oracle_lib as O
    L = O.lib()
    return np.array([L.orc_draw_u32(b"input.prompt", seed, i) % vocab for i in range(n)], np.int32)


def prompt_ids(vocab, n, seed=0):
    """Seeded prompt without the oracle library (product path): same counter-based draws."""
    from ainfer_b200 import _mix64, synth_key
    key = synth_key(seed, "input.prompt")
    return np.array([(_mix64((key + i) & ((1 << 64) - 1)) >> 32) % vocab for i in range(n)], np.int32)


class ClockSampler:
    """nvidia-smi samples during the timed region (never changes any GPU setting)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                       "-lms", "100", "-i", str(gpu_index)], stdout=self.f, stderr=subprocess.DEVNULL)
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
    total = n_lin * lin + n_attn * att + (n_lin + n_attn) * (slots * expert + router) + V * H * w + H * 2 + state + kv
    return total


def run_reference(args):
    """CPU arm: the oracle (port of the reference's host operator math) on the host cores."""
    rank, _, world = dist_env()
    if rank != 0:
        return 0
    import oracle_lib as O
    from ainfer_b200 import runtime
    arch = runtime.preset_config_json(args.model)
    cfg = json.loads(arch)
    t0 = time.time()
    om = O.Model(arch_json=arch, synth_seed=0)
    P = 8
    sess = O.Session(om, P + args.warmup + args.steps + 8)
    prompt = seeded_prompt(cfg["vocab"], P)
    tok = None
    pos = 0
    for i in range(P):                       # prompt (also generates the non-expert weights lazily)
        tok = sess.step(int(prompt[i]), pos, i == P - 1)
        pos += 1
    for _ in range(args.warmup):
        tok = sess.step(tok, pos, True); pos += 1
    done, t1 = 0, time.time()
    budget = args.cpu_budget
    while done < args.steps:
        tok = sess.step(tok, pos, True); pos += 1; done += 1
        if time.time() - t1 > budget:
            break
    dt = time.time() - t1
    v = done / dt
    cores = O.lib().orc_threads()
    sample = (f"{done} greedy decode tokens after an {P}-token prompt and {args.warmup} warm-up tokens, "
              f"{args.model} model with lazily generated seeded weights, context < {pos + 1}; "
              f"set-up {t1 - t0:.0f} s not timed")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": done,
        "warmup": args.warmup, "ms_per_step": 1000.0 / v, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int4xint8->int32, fp32 rescale", "data": "synthetic",
        "config": {"workload": f"{args.model} model batch-1 greedy decode (CPU oracle port)", "context": pos},
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}))
    return 0


def gemv_probe(dev, N, K, reps=20):
    """Isolated Int4GemvA8 launches on seeded device-generated weights: mean ms per launch of a recorded
    list of `reps` launches rotating over more than 256 MB of distinct weight buffers (cold L2, no host
    launch latency in the figure); thread groups sized by the runtime's own rule."""
    from ainfer_b200 import opbench
    return opbench.gemv_once(dev, N, K, 1, reps)["ms"]


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
    model = runtime.Model(dev, f"synth:{args.model}:seed={rank}")
    cfg = model.config
    t_load = time.time() - t_load
    P = args.prompt_len
    max_ctx = P + WINDOW + 8
    sess = runtime.Session(model, max_ctx, runtime.Session.PERSISTENT if args.persistent else 0)
    prompt = prompt_ids(cfg["vocab"], P, seed=rank)

    def barrier():
        dev.sync()
        if dist is not None:
            dist.barrier()

    t_prompt = time.time()
    last = int(sess.generate(prompt, 1)[0])          # whole prompt by loop-decode + first token
    t_prompt = time.time() - t_prompt
    # untimed warm-up steps
    if args.warmup > 0:
        sess.generate(np.array([last], np.int32), args.warmup, start_pos=P)
    # ---- timed: K steps in windows that start at position P ----
    barrier()
    clocks = ClockSampler(local_rank) if rank == 0 else None
    left, gen_ms, toks0 = args.steps, 0.0, None
    t_wall = time.time()
    while left > 0:
        n = min(WINDOW, left)
        toks, ms = sess.generate(np.array([last], np.int32), n, start_pos=P, timed=True)
        if toks0 is None:
            toks0 = toks.copy()
        gen_ms += ms
        left -= n
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
    # Expert-parallel MoE block over all ranks (only when there is more than one): a decode batch of
    # 64 token rows through layer 0's MoE with experts sharded E/N per rank, NCCL all-to-all for
    # dispatch and combine. Functional probe (host-staged exchange, one expert item at a time):
    # it reports what moved and that every replica ended up with the same rows, not a speed.
    ep_probe = None
    if world > 1:
        try:
            import torch
            from ainfer_b200 import ep
            be = ep.GpuMoeBackend(dev, model, layer=0)
            blk = ep.EpMoeBlock(be, ep.TorchComm(device=torch.device("cuda", local_rank)))
            rows = np.random.default_rng(1234).standard_normal((64, cfg["hidden"])).astype(np.float32)
            out = blk.forward(rows)
            chk = torch.tensor([float(np.abs(out).sum())], dtype=torch.float64, device=torch.device("cuda", local_rank))
            lo_, hi_ = chk.clone(), chk.clone()
            dist.all_reduce(lo_, op=dist.ReduceOp.MIN); dist.all_reduce(hi_, op=dist.ReduceOp.MAX)
            st = torch.tensor([blk.stats["items_computed"], blk.stats["dispatch_bytes"], blk.stats["combine_bytes"]],
                              dtype=torch.int64, device=torch.device("cuda", local_rank))
            dist.all_reduce(st)
            ep_probe = {"ranks": world, "batch": 64, "layer": 0, "experts_per_rank": cfg["experts"] // world,
                        "items": int(st[0]), "dispatch_bytes": int(st[1]), "combine_bytes": int(st[2]),
                        "replicas_identical": bool(lo_.item() == hi_.item()), "collective": "nccl all_to_all_single"}
        except Exception as e:
            ep_probe = {"error": str(e)[:200]}
    if rank != 0:
        model.close(); dev.close()
        dist.destroy_process_group()
        return 0
    value = world * args.steps / (gen_ms / 1000.0)
    e2e_value = world * n_e2e / t_e2e
    ctx = P + WINDOW // 2
    bytes_tok = model_bytes_per_token(cfg, ctx)
    peak, peak_src = measured_peak()
    # ---- roofline of the dominant kernel, measured live: the LM-head launch of Int4GemvA8 ----
    roof = None
    sweep = []
    try:
        for (N, K) in [(cfg["vocab"], cfg["hidden"]), (8192, 2048), (4096, 2048), (512, 2048), (2048, 512)]:
            ms = gemv_probe(dev, N, K)
            b = N * K * 0.515625 + K * 1 + (K // 128) * 4 + N * 4
            sweep.append({"N": N, "K": K, "M": 1, "ms": ms, "gbs": b / ms / 1e6, "frac": b / ms / 1e6 / peak})
        top = sweep[0]
        roof = {"bound": "hbm", "kernel": f"Int4GemvA8 lm_head [{top['N']}x{top['K']}] M=1",
                "achieved": top["gbs"], "peak": peak, "unit": "GB/s", "frac": top["frac"],
                "peak_source": peak_src,
                # DRAM bytes of one launch of this kernel at this shape from the ncu capture summarised in
                # profiles/int4_gemv_a8_lm_head_151936x2048.md (dram__bytes_read.sum + dram__bytes_write.sum)
                "traffic": 164.45e6 if (top["N"], top["K"]) == (151936, 2048) else None,
                "algorithmic_bytes_per_launch": top["N"] * top["K"] * 0.515625 + top["K"] + top["K"] // 128 * 4 + top["N"] * 4}
    except Exception as e:     # the probe must never take the decode number down with it
        roof = {"bound": "hbm", "error": str(e)}
    token_roof = {"bytes_per_token": bytes_tok, "achieved_gbs": bytes_tok / (gen_ms / args.steps) / 1e6,
                  "frac_of_measured_peak": bytes_tok / (gen_ms / args.steps) / 1e6 / peak,
                  "frac_of_nominal_8tbs": bytes_tok / (gen_ms / args.steps) / 1e6 / 8000.0}
    # ---- CPU baseline: the oracle on the host cores, from the GPU session's state at position P ----
    cpu = None
    parity = None
    if not args.no_cpu:
        try:
            import oracle_lib as O
            om = O.Model(arch_json=model.config_json, synth_seed=0)
            osess = O.Session(om, max_ctx)
            # state at position P: run the prompt again on the GPU from a clean session
            sess.reset()
            first = int(sess.generate(prompt, 1)[0])
            names = (("S", np.float32), ("conv", np.float32), ("Kc", np.int8), ("Vc", np.int8),
                     ("Ks", np.uint16), ("Vs", np.uint16))
            state = {n: sess.read(n, dt) for n, dt in names}
            n_cpu = args.cpu_steps
            gpu_toks = sess.generate(np.array([first], np.int32), n_cpu, start_pos=P)
            for n, _ in names:
                osess.buf(n)[:] = state[n]
            osess.step(first, P, True)          # untimed warm-up: also generates the weights it touches
            for n, _ in names:
                osess.buf(n)[:] = state[n]
            t0 = time.time()
            cpu_toks, tok = [], first
            for i in range(n_cpu):
                tok = osess.step(tok, P + i, True)
                cpu_toks.append(tok)
            dt_cpu = time.time() - t0
            cpu = {"value": n_cpu / dt_cpu, "unit": UNIT, "cores": O.lib().orc_threads(), "kind": "port",
                   "sample": f"{n_cpu} greedy decode tokens of the {args.model} model at context {P}, starting "
                             f"from the GPU session's state after the {P}-token prompt; weights generated by the "
                             f"oracle's own generator; one untimed warm-up token"}
            parity = {"tokens_compared": n_cpu, "tokens_match": [int(t) for t in gpu_toks] == cpu_toks}
        except Exception as e:
            cpu = {"value": None, "unit": UNIT, "cores": None, "kind": "port", "sample": f"failed: {e}"}
    # MTP draft-3 / verify loop on a short run of its own (separate session: the timed decode above is
    # plain greedy). With seeded random weights the head agrees with the trunk about as often as
    # chance, so this reports the mechanism and its cost, not a speed-up.
    mtp = None
    if rank == 0 and cfg.get("mtp_layers", 0) and not args.no_mtp:
        try:
            ms_ = runtime.Session(model, 96)
            t0 = time.time()
            mt, st = ms_.generate_mtp(prompt_ids(cfg["vocab"], 8, seed=11), 32, draft_k=3)
            dt = time.time() - t0
            pl = runtime.Session(model, 96)
            same = [int(t) for t in pl.generate(prompt_ids(cfg["vocab"], 8, seed=11), 32)] == [int(t) for t in mt]
            pl.close(); ms_.close()
            mtp = {"draft": 3, "tokens": 32, "rounds": st["rounds"], "drafted": st["drafted"], "accepted": st["accepted"],
                   "tokens_equal_plain_greedy": same, "tokens_per_s_sequential_verify": 32 / dt,
                   "note": "verification is one trunk step per token; batched verification is not built"}
        except Exception as e:
            mtp = {"error": str(e)}
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": gen_ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int4xint8->int32, fp32 rescale", "data": "synthetic",
        "config": {"workload": f"{args.model} (80B-A3B-shaped INT4 g128, 48 layers 3:1 DeltaNet:GQA, 512 experts "
                               f"top-10 + shared, vocab 151936) batch-1 greedy decode after a {P}-token seeded prompt"
                   if args.model == "full" else f"{args.model} model batch-1 greedy decode after a {P}-token prompt",
                   "context": f"{P}..{P + WINDOW}", "kv_cache": "int8 + fp16 per-token-per-head scales",
                   "mtp": "off in the timed decode (see mtp_probe)", "step": "one persistent cooperative launch" if args.persistent else "one recorded list of stand-alone launches chained by programmatic dependencies", "parallelism": "replicas" if world > 1 else "single GPU",
                   "l2": "inputs larger than L2: about 2.1 GB of weights and state streamed per step",
                   "launches_per_token": sess.launches_per_token()},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": 16, "d2h_bytes_per_step": 4,
                "steps": n_e2e, "api": "ainfer_session_step (control write + replay + token readback)"},
        "gpu_launches": int(sess.launches_per_token() * args.steps),
        "clocks": clk, "roofline": roof, "token_roofline": token_roof, "gemv_sweep": sweep,
        "cpu_baseline": cpu, "parity": parity, "mtp_probe": mtp, "ep_probe": ep_probe,
        "timing": {"model_fill_s": t_load, "prompt_s": t_prompt, "timed_wall_s": t_wall, "first_tokens": [int(t) for t in toks0[:8]]},
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
    ap.add_argument("--cpu-steps", type=int, default=4)
    ap.add_argument("--cpu-budget", type=float, default=150.0, help="seconds of timed CPU work in the reference arm")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-mtp", action="store_true", help="skip the short MTP draft/verify probe")
    ap.add_argument("--persistent", action="store_true", help="one persistent cooperative launch per token instead of the recorded list")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
