"""Regenerates the committed golden fixtures from the reference checkout.

Run where the reference checkout is at $REFERENCE (default: a directory named
"reference" beside this repository):   python tests/golden/make_golden.py

Outputs (committed, small):
  ref_vectors.npz   vectors extracted from the reference's own fixture files
                    (reference/lin_block_L0.json, attn_block_L3.json,
                    rope_applied.json, rope_pos4.json, operators_t14.npz)
  quant_golden.npz  outputs of the reference's quantize_int4_sym /
                    dequantize_int4_sym / f32_to_bf16_bits (tools/binfer.py:65-102)
                    on seeded inputs, obtained by importing that module
  sampler_golden.json  outputs of the reference's host sampler
                    (tools/sample/sampler.h) through oracle/_ref/libref_sampler.so
"""
import ctypes as C
import importlib.util
import json
import os
import subprocess
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get("REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference")


def ref_vectors():
    out = {}
    lin = json.load(open(os.path.join(REF, "reference", "lin_block_L0.json")))
    for k in ["decode_q_full", "decode_k_full", "decode_v_full", "decode_z_full", "decode_g_full",
              "decode_beta_full", "decode_S_final_head0", "decode_q_h0", "decode_k_h0",
              "decode_v_h0", "decode_g48", "decode_beta48", "S_head0", "decode_core_h0_full"]:
        out["lin_" + k] = np.array(lin[k], dtype=np.float32)
    out["lin_chunk_vs_recurrent_maxdiff"] = np.float64(lin["chunk_vs_recurrent_maxdiff"])
    att = json.load(open(os.path.join(REF, "reference", "attn_block_L3.json")))
    for k in ["decode_q", "decode_gate", "decode_K5", "decode_V5", "decode_attn_weights_head0"]:
        out["attn_" + k] = np.array(att[k], dtype=np.float32)
    ra = json.load(open(os.path.join(REF, "reference", "rope_applied.json")))
    for k in ["q", "k", "cos", "sin", "q_applied", "k_applied"]:
        out["rope_" + k] = np.array(ra[k], dtype=np.float32)
    rp = json.load(open(os.path.join(REF, "reference", "rope_pos4.json")))
    out["rope_pos4_cos"] = np.array(rp["cos"], dtype=np.float64)
    out["rope_pos4_sin"] = np.array(rp["sin"], dtype=np.float64)
    ops = np.load(os.path.join(REF, "reference", "operators_t14.npz"))
    for k in ops.files:
        out["ops_" + k] = ops[k]
    np.savez_compressed(os.path.join(HERE, "ref_vectors.npz"), **out)
    print("ref_vectors.npz", len(out), "arrays")


def quant_golden():
    import torch
    spec = importlib.util.spec_from_file_location("ref_binfer", os.path.join(REF, "tools", "binfer.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    rng = np.random.default_rng(0)
    w = (rng.standard_normal((24, 512)) * 0.02).astype(np.float32)
    w[3, 128:256] = 0.0          # an all-zero group (scale -> 1.0)
    w[5, 0] = 0.14               # an outlier group
    w[7, :128] = np.linspace(-0.07, 0.07, 128, dtype=np.float32)  # includes exact .5 ties
    packed, scales, mx, mean = mod.quantize_int4_sym(torch.from_numpy(w))
    deq = mod.dequantize_int4_sym(packed, scales, w.size)
    bf = mod.f32_to_bf16_bits(w.reshape(-1))
    np.savez_compressed(os.path.join(HERE, "quant_golden.npz"), w=w,
                        packed=np.frombuffer(packed, np.uint8), scales=np.frombuffer(scales, np.uint16),
                        dequant=deq.astype(np.float32), bf16_bits=bf,
                        max_err=np.float64(mx), mean_err=np.float64(mean))
    print("quant_golden.npz ok")


def sampler_golden():
    subprocess.run(["make", "-C", os.path.join(ROOT, "oracle"), "ref", f"REFERENCE={REF}"], check=True)
    L = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libref_sampler.so"))
    f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
    L.ref_sample_token.restype = C.c_int
    L.ref_sample_token.argtypes = [f32p, C.c_int, C.c_float, C.c_int, C.c_float, C.c_float,
                                   C.c_uint64, C.POINTER(C.c_uint64), f32p]
    L.ref_apply_rep_penalty.argtypes = [f32p, C.c_int, np.ctypeslib.ndpointer(np.int32), C.c_int, C.c_float]
    L.ref_xrs64.restype = C.c_uint64
    L.ref_xrs64.argtypes = [C.POINTER(C.c_uint64)]
    rng = np.random.default_rng(1)
    V = 97
    logits = (rng.standard_normal(V) * 2.0).astype(np.float32)
    logits[11] = logits[40] = logits.max() + 0.5   # planted tie: first max wins
    cases = []
    for (temp, top_k, top_p, rep, seed) in [(0.0, 0, 1.0, 1.0, 0), (1.0, 0, 1.0, 1.0, 7),
                                            (0.7, 5, 1.0, 1.0, 123), (1.3, 0, 0.8, 1.0, 99),
                                            (0.9, 12, 0.6, 1.3, 2024)]:
        lg = logits.copy()
        seen = np.array([11, 3, 40, 96, 3], dtype=np.int32)
        if rep > 1.0:
            L.ref_apply_rep_penalty(lg, V, seen, len(seen), rep)
        state = C.c_uint64(seed if seed else 0x9E3779B97F4A7C15)
        probs = np.zeros(V, np.float32)
        draws = []
        for _ in range(16):
            draws.append(int(L.ref_sample_token(lg, V, temp, top_k, top_p, rep, seed, C.byref(state), probs)))
        cases.append(dict(temp=temp, top_k=top_k, top_p=top_p, rep_penalty=rep, seed=seed,
                          rng_init=(seed if seed else 0x9E3779B97F4A7C15), seen=seen.tolist(),
                          penalised_logits=[float(x) for x in lg], tokens=draws,
                          probs=[float(x) for x in probs], rng_final=int(state.value)))
    st = C.c_uint64(0x1234567)
    xs = [int(L.ref_xrs64(C.byref(st))) for _ in range(8)]
    json.dump(dict(V=V, logits=[float(x) for x in logits], cases=cases, xrs64_from_0x1234567=xs),
              open(os.path.join(HERE, "sampler_golden.json"), "w"))
    print("sampler_golden.json ok")


if __name__ == "__main__":
    if not os.path.isdir(REF):
        sys.exit(f"reference checkout not found at {REF}")
    ref_vectors()
    quant_golden()
    sampler_golden()
