"""Operator and short-decode microbenchmarks of the B200 decode path.

  python -m ainfer_b200.opbench gemv [--m 1] [--n 151936] [--k 2048] [--reps 20] [--sweep]
      INT4 g128 GEMV (Int4GemvA8) on seeded device-generated weights: ms and GB/s
      of algorithmic bytes per launch, cold L2 (launches of a recorded list rotate over
      more than 256 MB of distinct weight buffers; --flush: single launches, each after a
      256 MB rewrite). --sweep runs the operator sweep shapes
      M in {1,2,4,8} x (N,K) in {(512,2048),(4096,2048),(8192,2048),(151936,2048),(2048,512)}.
      --a16 runs the bf16-activation operator Int4GemmA16 instead (sweep: M in {1,2,4,8,64}).
  python -m ainfer_b200.opbench decode [--model small] [--prompt 4] [--steps 8]
      A short greedy decode of a synthetic model preset through the runtime
      (small enough to sit under a profiler).

Prints one JSON object per line. Timing uses device timestamps on the
execution queue.
"""
import argparse
import ctypes as C
import json
import sys

import numpy as np

from . import cuda_abi, runtime, synth_key

GEMV_MAT = np.dtype([("P", "<u8"), ("S", "<u8"), ("Y", "<u8"), ("e0", "<u8"), ("e1", "<u8"), ("e2", "<u8"),
                     ("row_start", "<i4"), ("N", "<i4"), ("epi", "<i4"), ("ldy", "<i4")])
KERNEL_BY_M = {1: "Int4GemvA8", 2: "Int4GemvA8M2", 4: "Int4GemvA8M4", 8: "Int4GemvA8M8"}


def gemv_bytes(N, K, M):
    """Algorithmic bytes of one launch: packed nibbles + bf16 scales, INT8 activations + fp32 group
    scales, fp32 outputs."""
    return N * K * 0.515625 + M * (K + (K // 128) * 4) + M * N * 4


def stream_groups(rows, K, sm_count):
    """Thread groups of a weight-streaming launch: at least one 16 KB tile (32768/K rows) per group,
    at most two groups per SM (the runtime's rule)."""
    rpt = 32768 // K
    return max(1, min(-(-rows // rpt), 2 * sm_count))


def gemv_once(dev, N, K, M=1, reps=20, flush=False, groups=None):
    """Times one GEMV shape. Default: a recorded command list of `reps` launches that rotate over
    enough distinct weight buffers to exceed L2 (>= 256 MB in total), timed as a whole on the device,
    so neither host launch latency nor L2 hits enter the figure. flush=True instead times single
    launches, each after a 256 MB rewrite."""
    wbytes = N * K // 2 + N * K // 128 * 2
    nbuf = 1 if flush else max(1, min(64, -(-(256 << 20) // wbytes)))
    sm = dev.info().sm_count
    rng = np.random.default_rng(0)
    xq = dev.upload(rng.integers(-127, 128, (M, K), dtype=np.int8))
    sq = dev.upload(np.full((M, K // 128), 0.01, np.float32))
    if not groups:
        groups = stream_groups(N, K, sm)
    bufs, kernels = [], []
    for b in range(nbuf):
        dP, dS, dY = dev.alloc(N * K // 2), dev.alloc(N * K // 128 * 2), dev.zeros(M * N * 4)
        k = dev.kernel("SynthInt4")
        k.set_arg(0, dP); k.set_arg(1, dS); k.set_arg(2, synth_key(b, f"opbench.{N}.{K}"), "u64")
        k.set_arg(3, N * K // 128, "u64"); k.set_arg(4, 0.02)
        k.launch(sm * 8)
        tab = np.zeros(1, GEMV_MAT)
        tab[0]["P"], tab[0]["S"], tab[0]["Y"], tab[0]["N"], tab[0]["ldy"] = dP, dS, dY, N, N
        g = dev.kernel(KERNEL_BY_M[M])
        g.set_args(dev.upload(tab.view(np.uint8)), 1, N, xq, sq, K, M)
        bufs.append((dP, dS, dY)); kernels.append(g)
    e0, e1 = dev.event(), dev.event()
    for i in range(3):
        kernels[i % nbuf].launch(groups)
    if flush:
        total = 0.0
        for _ in range(reps):
            dev.flush_l2()
            e0.record(); kernels[0].launch(groups); e1.record()
            total += e0.elapsed_ms(e1)
        ms = total / reps
    else:
        cl = dev.new_list()
        for i in range(reps):
            cl.append(kernels[i % nbuf], groups)
        cl.close()
        cl.execute()
        e0.record(); cl.execute(); e1.record()
        ms = e0.elapsed_ms(e1) / reps
        cl.destroy()
    dev.sync()
    for t in bufs:
        for p in t:
            dev.free(p)
    b = gemv_bytes(N, K, M)
    return {"op": "int4_gemv_a8", "M": M, "N": N, "K": K, "ms": ms, "gbs": b / ms / 1e6, "bytes": b,
            "groups": groups, "buffers": nbuf, "mode": "flush" if flush else "list",
            "flops": 2.0 * M * N * K, "tflops": 2.0 * M * N * K / ms / 1e9}


def gemm_a16_once(dev, N, K, M, reps=20):
    """Int4GemmA16 (bf16 activations, 1 <= M <= 64) on one shape: recorded list rotating over enough
    weight buffers to exceed L2, timed as a whole on the device."""
    wbytes = N * K // 2 + N * K // 128 * 2
    nbuf = max(1, min(64, -(-(256 << 20) // wbytes)))
    rng = np.random.default_rng(0)
    xb = rng.standard_normal((M, K)).astype(np.float32).view(np.uint32)
    xb = ((xb + 0x7FFF + ((xb >> 16) & 1)) >> 16).astype(np.uint16)
    dX = dev.upload(xb)
    kernels, bufs = [], []
    for b in range(nbuf):
        dP, dS, dY = dev.alloc(N * K // 2), dev.alloc(N * K // 128 * 2), dev.zeros(M * N * 4)
        k = dev.kernel("SynthInt4")
        k.set_arg(0, dP); k.set_arg(1, dS); k.set_arg(2, synth_key(b, f"opbench.a16.{N}.{K}"), "u64")
        k.set_arg(3, N * K // 128, "u64"); k.set_arg(4, 0.02)
        k.launch(dev.info().sm_count * 8)
        g = dev.kernel("Int4GemmA16")
        g.set_args(dP, dS, dX, dY, N, K, M)
        kernels.append(g); bufs.append((dP, dS, dY))
    groups = (N + 127) // 128
    for i in range(3):
        kernels[i % nbuf].launch(groups)
    cl = dev.new_list()
    for i in range(reps):
        cl.append(kernels[i % nbuf], groups)
    cl.close()
    e0, e1 = dev.event(), dev.event()
    cl.execute()
    e0.record(); cl.execute(); e1.record()
    ms = e0.elapsed_ms(e1) / reps
    cl.destroy()
    dev.sync()
    for t in bufs:
        for p in t:
            dev.free(p)
    b = N * K * 0.515625 + M * K * 2 + M * N * 4
    return {"op": "int4_gemm_a16", "M": M, "N": N, "K": K, "ms": ms, "gbs": b / ms / 1e6, "bytes": b,
            "groups": groups, "buffers": nbuf, "flops": 2.0 * M * N * K, "tflops": 2.0 * M * N * K / ms / 1e9}


def gemv_multi_once(dev, N, K, M, reps=20, groups=0):
    """Int4GemvA8Multi (W4A8, 1 <= M <= 8, weights streamed once, dp4a) on one shape; same protocol as gemm_tc_once."""
    return gemm_tc_once(dev, N, K, M, reps, groups, kernel="Int4GemvA8Multi")


def gemm_tc_once(dev, N, K, M, reps=20, groups=0, kernel="Int4GemmA8Tc"):
    """Int4GemmA8Tc (W4A8 on tcgen05, 1 <= M <= 64, weights streamed once) on one shape: recorded list
    rotating over enough weight buffers to exceed L2, timed as a whole on the device."""
    wbytes = N * K // 2 + N * K // 128 * 2
    nbuf = max(1, min(64, -(-(256 << 20) // wbytes)))
    rng = np.random.default_rng(0)
    xq = dev.upload(rng.integers(-127, 128, (M, K), dtype=np.int8))
    sq = dev.upload(np.full((M, K // 128), 0.01, np.float32))
    kernels, bufs = [], []
    for b in range(nbuf):
        dP, dS, dY = dev.alloc(N * K // 2), dev.alloc(N * K // 128 * 2), dev.zeros(M * N * 4)
        k = dev.kernel("SynthInt4")
        k.set_arg(0, dP); k.set_arg(1, dS); k.set_arg(2, synth_key(b, f"opbench.tc.{N}.{K}"), "u64")
        k.set_arg(3, N * K // 128, "u64"); k.set_arg(4, 0.02)
        k.launch(dev.info().sm_count * 8)
        g = dev.kernel(kernel)
        g.set_args(dP, dS, xq, sq, dY, N, K, M, N)
        kernels.append(g); bufs.append((dP, dS, dY))
    if kernel == "Int4GemvA8Multi":
        groups = groups or min(-(-N // (256 // (K // 128))), dev.info().sm_count * 2)
    groups = groups or min((N + 127) // 128, dev.info().sm_count * 2)
    for i in range(3):
        kernels[i % nbuf].launch(groups)
    cl = dev.new_list()
    for i in range(reps):
        cl.append(kernels[i % nbuf], groups)
    cl.close()
    e0, e1 = dev.event(), dev.event()
    cl.execute()
    e0.record(); cl.execute(); e1.record()
    ms = e0.elapsed_ms(e1) / reps
    cl.destroy()
    dev.sync()
    for t in bufs:
        for p in t:
            dev.free(p)
    b = gemv_bytes(N, K, M)
    return {"op": "int4_gemm_a8_tc" if kernel == "Int4GemmA8Tc" else "int4_gemv_a8_multi", "M": M, "N": N, "K": K, "ms": ms, "gbs": b / ms / 1e6, "bytes": b,
            "groups": groups, "buffers": nbuf, "flops": 2.0 * M * N * K, "tflops": 2.0 * M * N * K / ms / 1e9}


def token_kernel_names(cfg):
    """Kernel names of one token step of the recorded list, in launch order."""
    lin = ["RmsNormQuant:in", "Int4GemvA8:in_proj", "DeltaNetStep", "GatedNormQuant", "Int4GemvA8:out_proj"]
    att = ["RmsNormQuant:in", "Int4GemvA8:qkv", "AttnPrep", "AttnSplit", "AttnCombine", "Int4GemvA8:o_proj"]
    moe = ["RmsNormQuant:post", "RouterTopK", "ExpertGateUp", "ExpertDownCombine"]
    names = ["EmbedRow"]
    for t in cfg["layer_types"]:
        names += (att if t == "A" else lin) + moe
    return names + ["RmsNormQuant:final", "Int4GemvA8:lm_head", "ArgmaxStage1", "ArgmaxStage2"]


def timeline(dev, model, sess, prompt, steps):
    """Cost of every kernel on the dependency chain of the recorded token step: the time from
    the moment its dependency wait returned (its predecessor is complete) to the moment its
    successor's wait returned, from global-timer stamps that block 0 of each kernel takes."""
    lib = cuda_abi.load()
    if not hasattr(lib, "ainfer_timeline_read"):
        raise SystemExit("this library was not built with AINFER_TIMELINE=1")
    rd = lib.ainfer_timeline_read
    rd.argtypes = [C.c_int, C.c_void_p, C.c_size_t, C.POINTER(C.c_size_t), C.c_int]
    names = token_kernel_names(model.config)
    sess.generate(prompt, 2)                      # prompt steps + warm-up, stamps discarded below
    cap = 1 << 18
    buf = np.zeros((cap, 2), np.uint64)
    n = C.c_size_t()
    assert rd(0, buf.ctypes.data, cap, C.byref(n), 1) == 0
    toks, ms = sess.generate(np.array([int(prompt[0])], np.int32), steps, start_pos=len(prompt) + 2, timed=True)
    assert rd(0, buf.ctypes.data, cap, C.byref(n), 1) == 0
    raw = buf[:n.value]
    is_mark = (raw[:, 0] >> np.uint64(63)) != 0
    # marks inside kernels (timeline builds may carry some): offset from the go of the kernel they follow
    kernel_index = np.cumsum(~is_mark) - 1
    marks_raw = [(int(kernel_index[i]), int(raw[i, 0] & np.uint64(0xFFFF)), int(raw[i, 1])) for i in np.nonzero(is_mark)[0]]
    n_kernels = int((~is_mark).sum())
    ev = raw[~is_mark].astype(np.int64)
    per = len(names)
    usable = (len(ev) // per) * per
    ev = ev[len(ev) - usable:]                    # whole token steps, counted from the end
    go = ev[:, 1]
    cost = np.diff(go, append=go[-1]).reshape(-1, per)[:-1] / 1000.0   # us; the last step has no successor
    early = ((ev[:, 1] - ev[:, 0]).reshape(-1, per)[:-1]) / 1000.0      # how long block 0 sat in its wait
    agg = {}
    for i, nm in enumerate(names):
        a = agg.setdefault(nm, [0, 0.0, 0.0])
        a[0] += 1; a[1] += float(cost[:, i].mean()); a[2] += float(early[:, i].mean())
    total = sum(a[1] for a in agg.values())
    rows = [{"kernel": k, "per_token": a[0], "us_per_token": round(a[1], 1), "share": round(a[1] / total, 4),
             "mean_us": round(a[1] / a[0], 2), "mean_wait_us": round(a[2] / a[0], 2)}
            for k, a in sorted(agg.items(), key=lambda kv: -kv[1][1])]
    marks = {}
    first = n_kernels - usable
    for (ki, mid, t) in marks_raw:
        if ki < first:
            continue
        pos = ki - first
        a = marks.setdefault(f"{names[pos % per]}#{mid}", [0, 0.0])
        a[0] += 1; a[1] += (t - int(go[pos])) / 1000.0
    print(json.dumps({"op": "timeline", "tokens": int(cost.shape[0]), "launches_per_token": per,
                      "chain_us_per_token": round(total, 1), "ms_per_token_events": ms / steps,
                      "kernels": rows,
                      "marks_us_after_go": {k: round(v[1] / v[0], 2) for k, v in sorted(marks.items())}}), flush=True)


def main(argv=None):
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("gemv")
    g.add_argument("--m", type=int, default=1)
    g.add_argument("--n", type=int, default=151936)
    g.add_argument("--k", type=int, default=2048)
    g.add_argument("--reps", type=int, default=20)
    g.add_argument("--sweep", action="store_true")
    g.add_argument("--a16", action="store_true", help="bf16 activations (Int4GemmA16, M up to 64) instead of W4A8")
    g.add_argument("--multi", action="store_true", help="W4A8 for M up to 8 with the weights streamed once (Int4GemvA8Multi, dp4a)")
    g.add_argument("--tc", action="store_true", help="W4A8 on the tcgen05 tensor cores (Int4GemmA8Tc, M up to 64)")
    g.add_argument("--groups", type=int, default=0, help="thread groups per launch (default: by shape)")
    g.add_argument("--flush", action="store_true", help="time single launches after an L2 rewrite")
    ll = sub.add_parser("listlat", help="device time per node of a recorded list of tiny dependent launches")
    ll.add_argument("--n", type=int, default=400)
    pl = sub.add_parser("pairlat", help="device time per (norm, GEMV) pair of a recorded list")
    pl.add_argument("--n", type=int, default=200)
    pl.add_argument("--rows", type=int, default=8192)
    d = sub.add_parser("decode")
    d.add_argument("--model", default="small")
    d.add_argument("--prompt", type=int, default=4)
    d.add_argument("--steps", type=int, default=8)
    d.add_argument("--per-layer", action="store_true")
    d.add_argument("--multi-kernel", action="store_true")
    d.add_argument("--persistent", action="store_true", help="one cooperative launch per token")
    d.add_argument("--stage-clock", action="store_true", help="print the time between grid barriers of the last token")
    d.add_argument("--timeline", action="store_true",
                   help="per-kernel cost on the dependency chain, measured inside the recorded list "
                        "(needs a library built with AINFER_TIMELINE=1)")
    pf = sub.add_parser("prefill", help="chunked prefill of a seeded prompt against token-by-token decoding of it")
    pf.add_argument("--model", default="small")
    pf.add_argument("--prompt", type=int, default=512)
    pf.add_argument("--steps", type=int, default=8)
    pf.add_argument("--no-loop", action="store_true", help="skip the token-by-token run (no comparison)")
    mt = sub.add_parser("mtp", help="draft / batched-verify rounds against plain greedy decoding")
    mt.add_argument("--model", default="mini-mtp")
    mt.add_argument("--prompt", type=int, default=32)
    mt.add_argument("--gen", type=int, default=32)
    mt.add_argument("--draft-k", type=int, default=3)
    args = ap.parse_args(argv)
    dev = cuda_abi.Device(0)
    if args.cmd == "mtp":
        import time
        model = runtime.Model(dev, f"synth:{args.model}:seed=0")
        V, P, G = model.config["vocab"], args.prompt, args.gen
        prompt = np.random.default_rng(11).integers(0, V, P).astype(np.int32)
        a = runtime.Session(model, P + G + 16, runtime.Session.PERSISTENT)
        a.generate(prompt, 2)
        a.reset(); dev.sync()
        t0 = time.time(); want = a.generate(prompt, G); t_plain = time.time() - t0
        t0 = time.time(); a.reset(); a.generate(prompt, 1); t_prompt = time.time() - t0
        b = runtime.Session(model, P + G + 16, runtime.Session.PERSISTENT)
        b.generate_mtp(prompt, 2 * args.draft_k + 4, draft_k=args.draft_k)   # creates the verifier and records its lists (untimed)
        b.reset(); dev.sync()
        t0 = time.time(); got, st = b.generate_mtp(prompt, G, draft_k=args.draft_k); t_mtp = time.time() - t0
        t0 = time.time(); b.reset(); b.generate_mtp(prompt, 1, draft_k=args.draft_k); t_mprompt = time.time() - t0
        gen_plain, gen_mtp = t_plain - t_prompt, t_mtp - t_mprompt
        print(json.dumps({"op": "mtp", "model": args.model, "prompt": P, "generated": G, "draft_k": args.draft_k,
                          "same_tokens": got.tolist() == want.tolist(), "stats": st,
                          "plain_ms_per_token": gen_plain * 1000 / max(G - 1, 1),
                          "round_ms": gen_mtp * 1000 / max(st["rounds"], 1),
                          "rows_per_round": args.draft_k + 1,
                          "plain_ms_for_the_same_rows": gen_plain * 1000 / max(G - 1, 1) * (args.draft_k + 1),
                          "mtp_tokens_per_s": (G - 1) / gen_mtp, "plain_tokens_per_s": (G - 1) / gen_plain}), flush=True)
        a.close(); b.close(); model.close()
    elif args.cmd == "prefill":
        import time
        model = runtime.Model(dev, f"synth:{args.model}:seed=0")
        V, P = model.config["vocab"], args.prompt
        prompt = np.random.default_rng(7).integers(0, V, P).astype(np.int32)
        b = runtime.Session(model, P + args.steps + 8, runtime.Session.PERSISTENT)
        b.prefill(prompt[:2])                       # creates the row buffers and records the MoE lists (untimed)
        b.reset()
        dev.sync()
        t0 = time.time()
        b.prefill(prompt[:P - 1])
        t_pf = time.time() - t0
        got = b.generate(prompt[P - 1:], args.steps, start_pos=P - 1)
        out = {"op": "prefill", "model": args.model, "prompt": P, "prefill_s": t_pf, "prompt_tokens_per_s": (P - 1) / t_pf,
               "tokens": [int(t) for t in got]}
        if not args.no_loop:
            a = runtime.Session(model, P + args.steps + 8, runtime.Session.PERSISTENT)
            dev.sync()
            t0 = time.time()
            want = a.generate(prompt, args.steps)
            t_loop = time.time() - t0
            out.update({"loop_decode_s": t_loop, "same_tokens": got.tolist() == want.tolist()})
            a.close()
        print(json.dumps(out), flush=True)
        b.close(); model.close()
    elif args.cmd == "gemv":
        ms_ = (1, 2, 4, 8, 64) if (args.a16 or args.tc) else (1, 2, 4, 8)
        if args.multi and not args.sweep and args.m > 8:
            raise SystemExit("--multi takes M up to 8")
        shapes = ([(m, n, k) for (n, k) in [(512, 2048), (4096, 2048), (8192, 2048), (151936, 2048), (2048, 512)]
                   for m in ms_] if args.sweep else [(args.m, args.n, args.k)])
        for (m, n, k) in shapes:
            if args.tc:
                r = gemm_tc_once(dev, n, k, m, args.reps, args.groups)
            elif args.multi:
                r = gemv_multi_once(dev, n, k, m, args.reps, args.groups)
            elif args.a16:
                r = gemm_a16_once(dev, n, k, m, args.reps)
            else:
                r = gemv_once(dev, n, k, m, args.reps, args.flush, args.groups)
            print(json.dumps(r), flush=True)
    elif args.cmd == "pairlat":
        # a recorded list of (RmsNormQuant, Int4GemvA8 on a small matrix) pairs: the dependency chain
        # of a decode layer in miniature; run with and without AINFER_NO_EARLY_LAUNCH=1
        K, N = 2048, args.rows
        rng = np.random.default_rng(0)
        dX = dev.upload(rng.standard_normal(K).astype(np.float32)); dW = dev.zeros(K * 4)
        dQ8, dSQ = dev.zeros(K), dev.zeros(K // 128 * 4)
        dP, dS, dY = dev.alloc(N * K // 2), dev.alloc(N * K // 128 * 2), dev.zeros(N * 4)
        k = dev.kernel("SynthInt4")
        k.set_arg(0, dP); k.set_arg(1, dS); k.set_arg(2, synth_key(0, "pairlat"), "u64")
        k.set_arg(3, N * K // 128, "u64"); k.set_arg(4, 0.02)
        k.launch(dev.info().sm_count * 8)
        tab = np.zeros(1, GEMV_MAT)
        tab[0]["P"], tab[0]["S"], tab[0]["Y"], tab[0]["N"], tab[0]["ldy"] = dP, dS, dY, N, N
        norm, gemv = dev.kernel("RmsNormQuant"), dev.kernel("Int4GemvA8")
        norm.set_args(dX, 0, 0, dW, 0, dQ8, dSQ, K, 1e-6)
        gemv.set_args(dev.upload(tab.view(np.uint8)), 1, N, dQ8, dSQ, K, 1)
        groups = stream_groups(N, K, dev.info().sm_count)
        cl = dev.new_list()
        for _ in range(args.n):
            cl.append(norm, 1)
            cl.append(gemv, groups)
        cl.close()
        e0, e1 = dev.event(), dev.event()
        cl.execute()
        e0.record(); cl.execute(); e1.record()
        dev.sync()
        print(json.dumps({"op": "pairlat", "pairs": args.n, "rows": N, "groups": groups,
                          "us_per_pair": e0.elapsed_ms(e1) * 1000.0 / args.n}), flush=True)
        cl.destroy()
    elif args.cmd == "listlat":
        ctrl = dev.zeros(16); ids = dev.zeros(64)
        k = dev.kernel("ControlAdvance")
        k.set_args(ctrl, ids, 16)
        cl = dev.new_list()
        for _ in range(args.n):
            cl.append(k, 1)
        cl.close()
        e0, e1 = dev.event(), dev.event()
        cl.execute()
        e0.record(); cl.execute(); e1.record()
        dev.sync()
        print(json.dumps({"op": "listlat", "nodes": args.n, "us_per_node": e0.elapsed_ms(e1) * 1000.0 / args.n}), flush=True)
        cl.destroy()
    else:
        model = runtime.Model(dev, f"synth:{args.model}:seed=0")
        sess = runtime.Session(model, args.prompt + args.steps + 16,
                               runtime.Session.PER_LAYER_LISTS if args.per_layer else
                               (runtime.Session.MULTI_KERNEL if args.multi_kernel else
                                runtime.Session.PERSISTENT if args.persistent else
                                (runtime.Session.STAGE_CLOCK if args.stage_clock else 0)))
        prompt = (np.arange(args.prompt, dtype=np.int32) * 7919 + 13) % model.config["vocab"]
        if args.timeline:
            timeline(dev, model, sess, prompt, args.steps)
            sess.close(); model.close(); dev.close()
            return 0
        toks, ms = sess.generate(prompt, args.steps, timed=True)
        print(json.dumps({"op": "decode", "model": args.model, "prompt": args.prompt, "steps": args.steps,
                          "ms_per_token": ms / args.steps, "launches_per_token": sess.launches_per_token(),
                          "tokens": [int(t) for t in toks]}), flush=True)
        if args.stage_clock:
            # block 0's records of the last token: [id, microseconds since the previous record]; the
            # consumers' list (id 1 = a grid barrier was passed) and the producer warp's list
            st = sess.read("stage_stamps", np.uint64)
            half = len(st) // 2
            mask = (1 << 48) - 1
            nz = st[st != 0]
            origin = int(min(int(t) & mask for t in nz)) if len(nz) else 0   # both lists on one time axis
            for name, part in (("consumer", st[:half]), ("producer", st[half:])):
                part = part[part != 0]
                ev = [(int(t) >> 48, int(t) & mask) for t in part]
                out, prev = [], ev[0][1] if ev else 0
                for (i, t) in ev:
                    out.append([i, round((t - prev) / 1000.0, 2)])
                    prev = t
                print(json.dumps({"op": "stage_clock", "who": name, "unit": "us", "events": out,
                                  "at_us": [round((t - origin) / 1000.0, 2) for (_, t) in ev]}), flush=True)
        sess.close(); model.close()
    dev.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
