"""Pins the CPU oracle against the reference's own golden vectors.

Fixtures under tests/golden/ were extracted from the reference's fixture files
and from its importable Python/C++ code by tests/golden/make_golden.py.
Tolerances are the reference's own bars for each operator class
(tools/cmdlist/*_replay.cpp headers): attention 1e-5, recurrence 1e-4,
RoPE 1e-6; integer/byte work is bit-exact.
"""
import ctypes as C
import os

import numpy as np
import pytest

import oracle_lib as O

G = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def ref():
    return np.load(os.path.join(G, "ref_vectors.npz"))


def test_quantizer_bit_exact_vs_reference_binfer():
    g = np.load(os.path.join(G, "quant_golden.npz"))
    packed, scales = O.quantize_int4(g["w"])
    assert np.array_equal(packed.reshape(-1), g["packed"])
    assert np.array_equal(scales.reshape(-1), g["scales"])
    assert np.array_equal(O.bf16_bits(g["w"].reshape(-1)), g["bf16_bits"])
    L = O.lib()
    for v in g["w"].reshape(-1)[:64]:
        assert L.orc_f32_to_bf16(float(v)) == int(O.bf16_bits(np.array([v]))[0])
    # dequant rule: nibble * bf16 scale, two's complement, low nibble = even k
    nib = np.empty(g["packed"].size * 2, np.int8)
    nib[0::2] = g["packed"] & 0xF
    nib[1::2] = g["packed"] >> 4
    nib[nib >= 8] -= 16
    deq = nib.astype(np.float32) * np.repeat(O.bf16_to_f32(g["scales"]), 128)
    assert np.array_equal(deq, g["dequant"])


def test_deltanet_recurrence_vs_hf_fixture(ref):
    """Zero-state decode step and non-zero-state head-0 step of HF layer 0
    (reference/lin_block_L0.json); tol 1e-4 as tools/cmdlist/ssm_replay.cpp."""
    L = O.lib()
    D = 128
    q = np.ascontiguousarray(ref["lin_decode_q_full"].reshape(48, D))
    k = np.ascontiguousarray(ref["lin_decode_k_full"].reshape(48, D))
    v = np.ascontiguousarray(ref["lin_decode_v_full"].reshape(48, D))
    qn = np.zeros(D, np.float32)
    kn = np.zeros(D, np.float32)
    L.orc_l2norm(q[0], D, np.float32(1.0 / np.sqrt(D)), qn)
    L.orc_l2norm(k[0], D, np.float32(1.0), kn)
    S = np.zeros((D, D), np.float32)
    o = np.zeros(D, np.float32)
    L.orc_deltanet_head(S.reshape(-1), qn, kn, v[0], float(ref["lin_decode_beta_full"][0]),
                        float(ref["lin_decode_g_full"][0]), D, o)
    assert np.abs(S - ref["lin_decode_S_final_head0"]).max() < 1e-6
    # step from the recorded non-zero state (fixture q/k are pre-l2norm there too)
    S = np.ascontiguousarray(ref["lin_S_head0"]).copy()
    L.orc_l2norm(np.ascontiguousarray(ref["lin_decode_q_h0"]), D, np.float32(1.0 / np.sqrt(D)), qn)
    L.orc_l2norm(np.ascontiguousarray(ref["lin_decode_k_h0"]), D, np.float32(1.0), kn)
    L.orc_deltanet_head(S.reshape(-1), qn, kn,
                        np.ascontiguousarray(ref["lin_decode_v_h0"]),
                        float(ref["lin_decode_beta48"][0]), float(ref["lin_decode_g48"][0]), D, o)
    assert np.abs(o - ref["lin_decode_core_h0_full"]).max() < 1e-4 * np.abs(o).max()


def test_attention_weights_vs_hf_fixture(ref):
    """softmax(q.k/16) of head 0 over 5 cached tokens (reference/attn_block_L3.json)."""
    L = O.lib()
    q = np.ascontiguousarray(ref["attn_decode_q"].reshape(24, 256))
    gate = np.ascontiguousarray(ref["attn_decode_gate"].reshape(24, 256))
    K5 = ref["attn_decode_K5"]          # [4][5][256] -> token-major [5][4][256]
    V5 = ref["attn_decode_V5"]
    Kc = O.bf16_bits(np.ascontiguousarray(K5.transpose(1, 0, 2)).reshape(-1))
    Vc = O.bf16_bits(np.ascontiguousarray(V5.transpose(1, 0, 2)).reshape(-1))
    out = np.zeros((24, 256), np.float32)
    wts = np.zeros((24, 5), np.float32)
    L.orc_attn_bf16kv(q, Kc, Vc, gate, 24, 4, 256, 5, out, wts.ctypes.data)
    # the cache is BF16-rounded; the fixture is fp32: bf16 relative step 2^-8
    assert np.abs(wts[0] - ref["attn_decode_attn_weights_head0"]).max() < 5e-3
    # exact-input check of the softmax itself (fp32 K, no rounding), tol 1e-5
    s = (K5[0] @ q[0]) / 16.0
    w = np.array([L.orc_expf(float(x - s.max())) for x in s], np.float32)
    w /= w.sum()
    assert np.abs(w - ref["attn_decode_attn_weights_head0"]).max() < 1e-5
    # gate and weighted V against an fp64 evaluation on the same rounded cache
    Kf = O.bf16_to_f32(Kc).reshape(5, 4, 256).astype(np.float64)
    Vf = O.bf16_to_f32(Vc).reshape(5, 4, 256).astype(np.float64)
    for h in (0, 7, 23):
        kv = h // 6
        sc = Kf[:, kv, :] @ q[h].astype(np.float64) / 16.0
        p = np.exp(sc - sc.max())
        p /= p.sum()
        want = (p @ Vf[:, kv, :]) / (1.0 + np.exp(-gate[h].astype(np.float64)))
        assert np.abs(out[h] - want).max() < 1e-5 * max(1.0, np.abs(want).max())


def test_int8kv_attention_close_to_fp32(ref):
    """The INT8-KV split attention stays within quantisation error of the fp32 path."""
    L = O.lib()
    rng = np.random.default_rng(3)
    nQ, nKV, D, T = 8, 2, 256, 150
    q = rng.standard_normal((nQ, D)).astype(np.float32)
    gate = rng.standard_normal((nQ, D)).astype(np.float32)
    K = rng.standard_normal((T, nKV, D)).astype(np.float32)
    V = rng.standard_normal((T, nKV, D)).astype(np.float32)
    Kc = np.zeros((T, nKV, D), np.int8); Vc = np.zeros((T, nKV, D), np.int8)
    Ks = np.zeros((T, nKV), np.uint16); Vs = np.zeros((T, nKV), np.uint16)
    for t in range(T):
        for h in range(nKV):
            L.orc_kv_quant_row(K[t, h], D, Kc[t, h], Ks[t, h:h + 1])
            L.orc_kv_quant_row(V[t, h], D, Vc[t, h], Vs[t, h:h + 1])
    out = np.zeros((nQ, D), np.float32)
    L.orc_attn_int8kv(q, Kc.reshape(-1), Ks.reshape(-1), Vc.reshape(-1), Vs.reshape(-1), gate,
                      nQ, nKV, D, T, out)
    Kd = Kc.astype(np.float64) * np.array([[L.orc_f16_to_f32(int(s)) for s in r] for r in Ks])[:, :, None]
    Vd = Vc.astype(np.float64) * np.array([[L.orc_f16_to_f32(int(s)) for s in r] for r in Vs])[:, :, None]
    for h in range(nQ):
        kv = h // (nQ // nKV)
        sc = Kd[:, kv, :] @ q[h].astype(np.float64) / 16.0
        p = np.exp(sc - sc.max()); p /= p.sum()
        want = (p @ Vd[:, kv, :]) / (1.0 + np.exp(-gate[h].astype(np.float64)))
        assert np.abs(out[h] - want).max() < 2e-5
    assert np.abs(Kd - K).max() < np.abs(K).max() / 127 * 0.51 + 1e-3


def test_rope_vs_hf_fixture(ref):
    L = O.lib()
    q, qa = ref["rope_q"], ref["rope_q_applied"]          # [1][2][4][256]
    cos, sin = ref["rope_cos"][0], ref["rope_sin"][0]      # [4][64]
    for h in range(q.shape[1]):
        for t in range(q.shape[2]):
            x = np.ascontiguousarray(q[0, h, t]).copy()
            L.orc_rope_apply(x, 64, np.ascontiguousarray(cos[t]), np.ascontiguousarray(sin[t]))
            assert np.abs(x - qa[0, h, t]).max() < 1e-6
            assert np.array_equal(x[64:], q[0, h, t, 64:])
    cs = np.zeros(64, np.float32); sn = np.zeros(64, np.float32)
    L.orc_rope_table(4, 64, 1e7, cs, sn)
    assert np.abs(cs - ref["rope_pos4_cos"]).max() < 1e-6
    assert np.abs(sn - ref["rope_pos4_sin"]).max() < 1e-6


def test_float64_operator_fixtures(ref):
    """reference/operators_t14.npz: silu-gate and the (plain-w) rmsnorm fixture.
    The fixture's rmsnorm multiplies by w, the decode path by (1+w): feed w-1."""
    L = O.lib()
    g, u, want = ref["ops_g"], ref["ops_u"], ref["ops_silu_gate_out"]
    got = np.array([[(gg / (1.0 + L.orc_expf(float(-gg)))) * uu for gg, uu in zip(gr, ur)]
                    for gr, ur in zip(g.astype(np.float32), u.astype(np.float32))])
    assert np.abs(got - want).max() < 1e-6
    x, w, y = ref["ops_rmsnorm_in"], ref["ops_rmsnorm_w"], ref["ops_rmsnorm_out"]
    for r in range(x.shape[0]):
        out = np.zeros(64, np.float32)
        L.orc_rmsnorm(x[r].astype(np.float32), (w - 1.0).astype(np.float32), 64, 1e-6, out)
        assert np.abs(out - y[r]).max() < 2e-6 * max(1.0, np.abs(y[r]).max())


def test_det_math_accuracy():
    L = O.lib()
    xs = np.concatenate([np.linspace(-85, 85, 4001), np.linspace(-1, 1, 2001)]).astype(np.float32)
    for x in xs:
        got, want = L.orc_expf(float(x)), np.exp(np.float64(x))
        assert abs(got - want) <= 2.5e-7 * want
    for x in np.concatenate([np.logspace(-30, 30, 3001), np.linspace(0.5, 2.0, 2001)]).astype(np.float32):
        got, want = L.orc_logf(float(x)), np.log(np.float64(x))
        assert abs(got - want) <= 2.5e-7 * max(1.0, abs(want))
    assert L.orc_expf(-200.0) == 0.0
    # fp16 round trip agrees with numpy's IEEE half
    vals = np.concatenate([np.logspace(-9, 5, 5000), -np.logspace(-9, 5, 200), [0.0, 65504.0, 65520.0, 1e-8]])
    for v in vals.astype(np.float32):
        h = L.orc_f32_to_f16(float(v))
        assert h == int(np.float16(v).view(np.uint16)), v
        if np.isfinite(np.float16(v)):
            assert L.orc_f16_to_f32(h) == float(np.float16(v))


def test_synthetic_normal_distribution():
    from scipy import stats
    z = O.synth_normal("model.test.weight", 0, 400000, 1.0)
    assert abs(z.mean()) < 0.01 and abs(z.std() - 1.0) < 0.01
    assert stats.kstest(z[:100000], "norm").pvalue > 1e-3
    # inverse CDF accuracy against scipy on a grid of draws
    L = O.lib()
    for r in np.linspace(0, 2**32 - 1, 2001).astype(np.uint64):
        k = int(r) >> 9
        p = (k + 0.5) / 2**23
        assert abs(L.orc_normal_from_u32(int(r)) - stats.norm.ppf(p)) < 3e-4 * max(1.0, abs(stats.norm.ppf(p)))
    # streams are independent of each other and reproducible
    a = O.synth_normal("a", 0, 1000, 1.0); b = O.synth_normal("b", 0, 1000, 1.0)
    assert abs(np.corrcoef(a, b)[0, 1]) < 0.1
    assert np.array_equal(a[10:20], O.synth_normal("a", 0, 10, 1.0, first=10))


def test_gemv_policies_agree():
    """W4A8 integer path vs the float-activation host reference (tools/gemv/gemv.cpp:480-501)
    on LCG weights as tools/cmdlist/gemv_replay.cpp:159-163; bar: its 0.02 mean-rel."""
    s = 0x9E3779B9
    N, K = 64, 512
    vals = np.zeros(N * K + K, np.float32)
    for i in range(vals.size):
        s = (s * 6364136223846793005 + 1442695040888963407) & (2**64 - 1)
        vals[i] = np.float32((((s >> 33) & 0xFFFF) - 32768)) * np.float32(0.02 / 32768.0)
    P, S = O.quantize_int4(vals[:N * K].reshape(N, K))
    x = O.bf16_to_f32(O.bf16_bits(vals[N * K:] * 50.0))
    xq, sq = O.aquant(x)
    y8 = O.gemv_a8(P, S, xq, sq)
    y16 = O.gemv_a16(P, S, x[None, :])[0]
    assert np.abs(y8 - y16).mean() / np.abs(y16).mean() < 0.02
    # integer identity: the group sums are exact, so an fp64 evaluation of the same
    # quantised operands matches to fp32 rounding of 4 additions
    nib = np.empty((N, K), np.int32)
    nib[:, 0::2] = P & 0xF; nib[:, 1::2] = P >> 4
    nib[nib >= 8] -= 16
    ref = np.zeros(N)
    for g in range(K // 128):
        gs = (nib[:, g * 128:(g + 1) * 128] * xq[g * 128:(g + 1) * 128].astype(np.int32)).sum(1)
        ref += gs * O.bf16_to_f32(S[:, g]).astype(np.float64) * np.float64(sq[g])
    assert np.abs(y8 - ref).max() <= 1e-6 * np.abs(ref).max()


def test_router_topk_ties_and_gap():
    L = O.lib()
    logits = np.array([0.5, 2.0, 2.0, -1.0, 1.0, 2.0, 0.0, 0.25], np.float32)
    idx = np.zeros(3, np.int32); wt = np.zeros(3, np.float32); gap = C.c_float()
    L.orc_router_topk(logits, 8, 3, idx, wt, C.byref(gap))
    assert idx.tolist() == [1, 2, 5]            # equal values: lowest index first
    assert abs(wt.sum() - 1.0) < 1e-6 and np.allclose(wt, 1 / 3, atol=1e-6)
    assert gap.value > 0.5
    logits[4] = np.float32(2.0)                 # k-th and (k+1)-th tie -> near-tie flagged
    L.orc_router_topk(logits, 8, 3, idx, wt, C.byref(gap))
    assert idx.tolist() == [1, 2, 4] and gap.value < 1e-5
    assert L.orc_argmax(np.array([1, 5, 5, 2], np.float32), 4) == 1
