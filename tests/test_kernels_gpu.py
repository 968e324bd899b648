"""Kernel-level parity: every decode kernel, called through the device C ABI,
against the CPU oracle on the same seeded inputs. Bit-exact (floats compared
by value, so that +0 == -0), as the arithmetic contract fixes the order of
every floating-point operation."""
import ctypes as C

import numpy as np
import pytest

import oracle_lib as O

pytestmark = pytest.mark.gpu

GEMV_MAT = np.dtype([("P", "<u8"), ("S", "<u8"), ("Y", "<u8"), ("e0", "<u8"), ("e1", "<u8"),
                     ("e2", "<u8"), ("row_start", "<i4"), ("N", "<i4"), ("epi", "<i4"), ("ldy", "<i4")])
EXPERT_W = np.dtype([("gP", "<u8"), ("gS", "<u8"), ("uP", "<u8"), ("uS", "<u8"), ("dP", "<u8"),
                     ("dS", "<u8")])
EPI_STORE, EPI_RESADD, EPI_CONV, EPI_BETA, EPI_GDECAY = range(5)


@pytest.fixture(scope="module")
def dev():
    from ainfer_b200 import cuda_abi
    d = cuda_abi.Device(0)
    yield d
    d.close()


def rnd_weights(rng, N, K, std=0.02):
    w = (rng.standard_normal((N, K)) * std).astype(np.float32)
    return O.quantize_int4(w)


def gemv_groups(dev, rows):
    return max(1, min((rows + 15) // 16, dev.info().sm_count * 4))


def run_gemv(dev, mats, xq, sq, K, M=1):
    """mats: list of dict(P,S,N,epi,e0,e1,e2,ldy) with numpy arrays -> list of outputs (and e1)."""
    tab = np.zeros(len(mats), GEMV_MAT)
    outs, e1s = [], []
    row = 0
    for i, m in enumerate(mats):
        N = m["N"]
        ylen = M * N
        y = dev.zeros(ylen * 4)
        tab[i]["P"], tab[i]["S"], tab[i]["Y"] = dev.upload(m["P"]), dev.upload(m["S"]), y
        tab[i]["e0"] = dev.upload(m["e0"]) if m.get("e0") is not None else 0
        e1 = dev.upload(m["e1"]) if m.get("e1") is not None else 0
        tab[i]["e1"] = e1
        tab[i]["e2"] = dev.upload(m["e2"]) if m.get("e2") is not None else 0
        tab[i]["row_start"], tab[i]["N"], tab[i]["epi"], tab[i]["ldy"] = row, N, m.get("epi", 0), N
        row += N
        outs.append((y, ylen))
        e1s.append((e1, m["e1"].size if m.get("e1") is not None else 0))
    name = {1: "Int4GemvA8", 2: "Int4GemvA8M2", 4: "Int4GemvA8M4", 8: "Int4GemvA8M8"}[M]
    k = dev.kernel(name)
    k(gemv_groups(dev, row), dev.upload(tab.view(np.uint8)), len(mats), row, dev.upload(xq),
      dev.upload(sq), K, M)
    dev.sync()
    return ([dev.download(p, n, np.float32) for p, n in outs],
            [dev.download(p, n, np.float32) if n else None for p, n in e1s])


@pytest.mark.parametrize("K", [128, 256, 512, 1024, 2048, 4096, 8192])
def test_gemv_a8_bit_exact_all_k(dev, K):
    rng = np.random.default_rng(K)
    N = 200 if K < 4096 else 72        # not a multiple of the warp tile on purpose
    P, S = rnd_weights(rng, N, K)
    x = rng.standard_normal(K).astype(np.float32) * 3
    xq, sq = O.aquant(x)
    want = O.gemv_a8(P, S, xq, sq)
    (got,), _ = run_gemv(dev, [dict(P=P, S=S, N=N)], xq, sq, K)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("N,K,groups", [(3000, 2048, 1), (3000, 2048, 2), (3000, 2048, 5), (4100, 512, 3),
                                        (1030, 4096, 1), (777, 128, 2), (1, 2048, 1), (5, 256, 4)])
def test_gemv_a8_streams_many_sub_blocks(dev, N, K, groups):
    """Few thread groups over many rows: every group walks several sub-blocks, so its weight ring
    runs on from one segment list into the next (and wraps many times); plus single-row and
    fewer-rows-than-groups cases."""
    rng = np.random.default_rng(N * 7 + K)
    P, S = rnd_weights(rng, N, K)
    x = rng.standard_normal(K).astype(np.float32) * 2
    xq, sq = O.aquant(x)
    want = O.gemv_a8(P, S, xq, sq)
    dY = dev.zeros(N * 4)
    tab = np.zeros(1, GEMV_MAT)
    tab[0]["P"], tab[0]["S"], tab[0]["Y"], tab[0]["N"], tab[0]["ldy"] = dev.upload(P), dev.upload(S), dY, N, N
    dev.kernel("Int4GemvA8")(groups, dev.upload(tab.view(np.uint8)), 1, N, dev.upload(xq), dev.upload(sq), K, 1)
    dev.sync()
    assert np.array_equal(dev.download(dY, N, np.float32), want)


@pytest.mark.parametrize("M", [2, 4, 8])
def test_gemv_a8_batched(dev, M):
    rng = np.random.default_rng(M)
    N, K = 136, 2048
    P, S = rnd_weights(rng, N, K)
    x = rng.standard_normal((M, K)).astype(np.float32)
    q = [O.aquant(x[m]) for m in range(M)]
    xq = np.stack([a for a, _ in q]); sq = np.stack([b for _, b in q])
    want = np.stack([O.gemv_a8(P, S, xq[m], sq[m]) for m in range(M)])
    (got,), _ = run_gemv(dev, [dict(P=P, S=S, N=N)], xq, sq, K, M)
    assert np.array_equal(got.reshape(M, N), want)


def test_gemv_multi_matrix_epilogues(dev):
    """qkv (conv+SiLU epilogue), z (store), b (sigmoid), a (decay) in one launch; then a
    residual-add launch: the reference's SsmConv / BetaG / ResAddF fused behind Int4Gemv."""
    L = O.lib()
    rng = np.random.default_rng(7)
    K, C_, NZ, NH = 1024, 300, 130, 18
    x = rng.standard_normal(K).astype(np.float32)
    xq, sq = O.aquant(x)
    Pq, Sq = rnd_weights(rng, C_, K); Pz, Sz = rnd_weights(rng, NZ, K)
    Pb, Sb = rnd_weights(rng, NH, K, 0.2); Pa, Sa = rnd_weights(rng, NH, K, 0.5)
    cw = (rng.standard_normal((C_, 4)) * 0.5).astype(np.float32)
    cs = rng.standard_normal((C_, 3)).astype(np.float32)
    al = (rng.standard_normal(NH) * 0.05).astype(np.float32)
    dt = (rng.standard_normal(NH) * 0.05).astype(np.float32)
    dt[0] = 30.0   # softplus pass-through branch
    (mx, z, bt, g), e1 = run_gemv(dev, [
        dict(P=Pq, S=Sq, N=C_, epi=EPI_CONV, e0=cw, e1=cs),
        dict(P=Pz, S=Sz, N=NZ, epi=EPI_STORE),
        dict(P=Pb, S=Sb, N=NH, epi=EPI_BETA),
        dict(P=Pa, S=Sa, N=NH, epi=EPI_GDECAY, e0=al, e2=dt)], xq, sq, K)
    qkv = O.gemv_a8(Pq, Sq, xq, sq)
    cs_ref = cs.copy().reshape(-1); mx_ref = np.zeros(C_, np.float32)
    L.orc_conv_silu(qkv, cs_ref, cw.reshape(-1), C_, mx_ref)
    assert np.array_equal(mx, mx_ref) and np.array_equal(e1[0], cs_ref)
    assert np.array_equal(z, O.gemv_a8(Pz, Sz, xq, sq))
    b = O.gemv_a8(Pb, Sb, xq, sq); a = O.gemv_a8(Pa, Sa, xq, sq)
    assert np.array_equal(bt, np.array([L.orc_dn_beta(float(v)) for v in b], np.float32))
    assert np.array_equal(g, np.array([L.orc_dn_gdecay(float(v), float(al[i]), float(dt[i]))
                                       for i, v in enumerate(a)], np.float32))
    res = rng.standard_normal(NZ).astype(np.float32)
    (y,), _ = run_gemv(dev, [dict(P=Pz, S=Sz, N=NZ, epi=EPI_RESADD, e0=res)], xq, sq, K)
    assert np.array_equal(y, res + O.gemv_a8(Pz, Sz, xq, sq))


@pytest.mark.parametrize("N,with_add", [(1024, False), (2048, True), (4096, True)])
def test_rmsnorm_quant(dev, N, with_add):
    L = O.lib()
    rng = np.random.default_rng(N)
    rows = 3
    a = rng.standard_normal((rows, N)).astype(np.float32)
    b = rng.standard_normal((rows, N)).astype(np.float32) if with_add else None
    a[1, 128:256] = 0.0
    if b is not None:
        b[1, 128:256] = 0.0     # an all-zero group: scale must become 1
    w = (rng.standard_normal(N) * 0.1).astype(np.float32)
    dA = dev.upload(a); dB = dev.upload(b) if with_add else 0
    dSum, dHn = dev.zeros(rows * N * 4), dev.zeros(rows * N * 4)
    dQ, dS = dev.zeros(rows * N), dev.zeros(rows * (N // 128) * 4)
    dev.kernel("RmsNormQuant")(rows, dA, dB, dSum, dev.upload(w), dHn, dQ, dS, N, 1e-6)
    dev.sync()
    x = a + b if with_add else a
    for r in range(rows):
        want = np.zeros(N, np.float32)
        L.orc_rmsnorm(np.ascontiguousarray(x[r]), w, N, 1e-6, want)
        q, s = O.aquant(want)
        assert np.array_equal(dev.download(dHn + r * N * 4, N, np.float32), want)
        assert np.array_equal(dev.download(dQ + r * N, N, np.int8), q)
        assert np.array_equal(dev.download(dS + r * (N // 128) * 4, N // 128, np.float32), s)
        assert np.array_equal(dev.download(dSum + r * N * 4, N, np.float32), x[r])


def test_embed_row(dev):
    rng = np.random.default_rng(1)
    V, H = 500, 1024
    emb = O.bf16_bits(rng.standard_normal((V, H)).astype(np.float32))
    ctrl = np.array([[123, 0, 1, -1], [499, 0, 1, -1]], np.int32)
    dX = dev.zeros(2 * H * 4)
    k = dev.kernel("EmbedRow")
    k.set_args(dX, dev.upload(emb), dev.upload(ctrl), H, V, 4)
    k.launch(2)   # one group per batch row
    dev.sync()
    got = dev.download(dX, (2, H), np.float32)
    assert np.array_equal(got[0], O.bf16_to_f32(emb[123]))
    assert np.array_equal(got[1], O.bf16_to_f32(emb[499]))


@pytest.mark.parametrize("nK,nV", [(8, 16), (16, 32), (16, 48)])
def test_deltanet_step_and_gated_norm(dev, nK, nV):
    L = O.lib()
    rng = np.random.default_rng(nV)
    D = 128
    mx = rng.standard_normal((2 * nK + nV) * D).astype(np.float32)
    S = (rng.standard_normal((nV, D, D)) * 0.1).astype(np.float32)
    bt = rng.uniform(0.1, 0.9, nV).astype(np.float32)
    gt = (-rng.uniform(0.001, 0.5, nV)).astype(np.float32)
    z = rng.standard_normal((nV, D)).astype(np.float32)
    w = (1.0 + rng.standard_normal(D) * 0.1).astype(np.float32)
    dS, dOut = dev.upload(S), dev.zeros(nV * D * 4)
    dev.kernel("DeltaNetStep")(nV * 4, dOut, dev.upload(mx), dS, dev.upload(bt), dev.upload(gt), nK, nV)
    dQ, dSQ, dY = dev.zeros(nV * D), dev.zeros(nV * 4), dev.zeros(nV * D * 4)
    dev.kernel("GatedNormQuant")((nV + 3) // 4, dOut, dev.upload(z), dev.upload(w), dQ, dSQ, dY, nV, 1e-6)
    dev.sync()
    got_o = dev.download(dOut, (nV, D), np.float32)
    got_S = dev.download(dS, (nV, D, D), np.float32)
    got_y = dev.download(dY, (nV, D), np.float32)
    ratio = nV // nK
    y_ref = np.zeros((nV, D), np.float32)
    for h in range(nV):
        kh = h // ratio
        q = np.zeros(D, np.float32); k = np.zeros(D, np.float32); o = np.zeros(D, np.float32)
        L.orc_l2norm(np.ascontiguousarray(mx[kh * D:(kh + 1) * D]), D, np.float32(0.0883883476), q)
        L.orc_l2norm(np.ascontiguousarray(mx[(nK + kh) * D:(nK + kh + 1) * D]), D, np.float32(1.0), k)
        v = np.ascontiguousarray(mx[(2 * nK + h) * D:(2 * nK + h + 1) * D])
        Sh = S[h].copy().reshape(-1)
        L.orc_deltanet_head(Sh, q, k, v, float(bt[h]), float(gt[h]), D, o)
        assert np.array_equal(got_o[h], o), h
        assert np.array_equal(got_S[h].reshape(-1), Sh), h
        L.orc_gated_norm(o, np.ascontiguousarray(z[h]), w, D, y_ref[h])
    assert np.array_equal(got_y, y_ref)
    q8, sq = O.aquant(y_ref.reshape(-1))
    assert np.array_equal(dev.download(dQ, nV * D, np.int8), q8)
    assert np.array_equal(dev.download(dSQ, nV, np.float32), sq)


@pytest.mark.parametrize("nQ,nKV,T", [(8, 2, 1), (8, 2, 64), (8, 2, 65), (16, 2, 512), (16, 2, 1500)])
def test_attention_decode_int8kv(dev, nQ, nKV, T):
    """AttnPrep + AttnSplit + AttnCombine vs the oracle's attention mixer pieces, with the new
    token appended at position T-1 of a cache holding T-1 seeded prior tokens."""
    L = O.lib()
    rng = np.random.default_rng(T + nQ)
    D, rot, max_ctx = 256, 64, T + 7
    pos = T - 1
    q16 = rng.standard_normal((nQ, 2 * D)).astype(np.float32)
    k16 = rng.standard_normal((nKV, D)).astype(np.float32)
    v16 = rng.standard_normal((nKV, D)).astype(np.float32)
    qnw = (rng.standard_normal(D) * 0.1).astype(np.float32)
    knw = (rng.standard_normal(D) * 0.1).astype(np.float32)
    Kc = np.zeros((max_ctx, nKV, D), np.int8); Vc = np.zeros((max_ctx, nKV, D), np.int8)
    Ks = np.zeros((max_ctx, nKV), np.uint16); Vs = np.zeros((max_ctx, nKV), np.uint16)
    prior = rng.standard_normal((2, max_ctx, nKV, D)).astype(np.float32)
    for t in range(pos):
        for h in range(nKV):
            L.orc_kv_quant_row(prior[0, t, h], D, Kc[t, h], Ks[t, h:h + 1])
            L.orc_kv_quant_row(prior[1, t, h], D, Vc[t, h], Vs[t, h:h + 1])
    cos = np.zeros((max_ctx, rot), np.float32); sin = np.zeros((max_ctx, rot), np.float32)
    for t in range(max_ctx):
        L.orc_rope_table(t, rot, 1e7, cos[t], sin[t])
    # oracle
    qn = np.zeros((nQ, D), np.float32)
    for h in range(nQ):
        L.orc_headnorm(np.ascontiguousarray(q16[h, :D]), qnw, D, 1e-6, qn[h])
        L.orc_rope_apply(qn[h], rot, cos[pos], sin[pos])
    Kr, Vr, Ksr, Vsr = Kc.copy(), Vc.copy(), Ks.copy(), Vs.copy()
    for h in range(nKV):
        kn = np.zeros(D, np.float32)
        L.orc_headnorm(np.ascontiguousarray(k16[h]), knw, D, 1e-6, kn)
        L.orc_rope_apply(kn, rot, cos[pos], sin[pos])
        L.orc_kv_quant_row(kn, D, Kr[pos, h], Ksr[pos, h:h + 1])
        L.orc_kv_quant_row(np.ascontiguousarray(v16[h]), D, Vr[pos, h], Vsr[pos, h:h + 1])
    gate = np.ascontiguousarray(q16[:, D:])
    want = np.zeros((nQ, D), np.float32)
    L.orc_attn_int8kv(qn, Kr.reshape(-1), Ksr.reshape(-1), Vr.reshape(-1), Vsr.reshape(-1), gate,
                      nQ, nKV, D, T, want)
    # device
    ctrl = np.array([0, pos, T, -1], np.int32)
    dCtrl = dev.upload(ctrl)
    dQ16, dQn = dev.upload(q16), dev.zeros(nQ * D * 4)
    dKc, dVc, dKs, dVs = dev.upload(Kc), dev.upload(Vc), dev.upload(Ks), dev.upload(Vs)
    dev.kernel("AttnPrep")((nQ + 2 * nKV + 7) // 8, dQ16, dev.upload(k16), dev.upload(v16),
                           dev.upload(qnw), dev.upload(knw), dev.upload(cos), dev.upload(sin), dCtrl,
                           dQn, dKc, dVc, dKs, dVs, nQ, nKV, rot, max_ctx, 1e-6)
    nch = (max_ctx + 63) // 64
    dPm, dPse, dPacc = dev.zeros(nQ * nch * 4), dev.zeros(nQ * nch * 4), dev.zeros(nQ * nch * D * 4)
    dev.kernel("AttnSplit")(((T + 63) // 64) * nKV, dQn, dKc, dVc, dKs, dVs, dCtrl, dPm, dPse, dPacc,
                            nQ, nKV, max_ctx, nch)
    dQ8, dSQ, dAtt = dev.zeros(nQ * D), dev.zeros(nQ * 2 * 4), dev.zeros(nQ * D * 4)
    dev.kernel("AttnCombine")(nQ, dPm, dPse, dPacc, dQ16, dCtrl, dQ8, dSQ, dAtt, nQ, max_ctx, nch)
    dev.sync()
    assert np.array_equal(dev.download(dQn, (nQ, D), np.float32), qn)
    assert np.array_equal(dev.download(dKc, Kc.shape, np.int8), Kr)
    assert np.array_equal(dev.download(dVc, Vc.shape, np.int8), Vr)
    assert np.array_equal(dev.download(dKs, Ks.shape, np.uint16), Ksr)
    assert np.array_equal(dev.download(dVs, Vs.shape, np.uint16), Vsr)
    assert np.array_equal(dev.download(dAtt, (nQ, D), np.float32), want)
    q8, sq = O.aquant(want.reshape(-1))
    assert np.array_equal(dev.download(dQ8, nQ * D, np.int8), q8)
    assert np.array_equal(dev.download(dSQ, nQ * 2, np.float32), sq)


@pytest.mark.parametrize("nQ,nKV", [(16, 2), (8, 2)])
def test_batch_attention_both_forms(dev, nQ, nKV):
    """BatchAttnSplit over rows that share one INT8 cache and end at their own lengths (the prefill
    layout). The long rows make the launch hold more than 2048 (chunk, KV head) items, so they take
    the one-warp-per-item form; the short rows take the one-block-per-item form. Every row, merged by
    AttnCombine, must equal the oracle's attention bit for bit."""
    L = O.lib()
    rng = np.random.default_rng(nQ)
    D, max_ctx = 256, 2200
    Ts = [2049 + 4 * b for b in range(32)] + [1, 64, 65, 700]
    B = len(Ts)
    nch = (max_ctx + 63) // 64
    assert B * ((2049 + 63) // 64) * nKV >= 2048 and B * ((700 + 63) // 64) * nKV < 2048
    Kc = np.zeros((max_ctx, nKV, D), np.int8); Vc = np.zeros((max_ctx, nKV, D), np.int8)
    Ks = np.zeros((max_ctx, nKV), np.uint16); Vs = np.zeros((max_ctx, nKV), np.uint16)
    prior = rng.standard_normal((2, max_ctx, nKV, D)).astype(np.float32)
    prior[1] *= rng.uniform(0.2, 3.0, (max_ctx, nKV, 1)).astype(np.float32)   # value scales that differ by token
    for t in range(max_ctx):
        for h in range(nKV):
            L.orc_kv_quant_row(prior[0, t, h], D, Kc[t, h], Ks[t, h:h + 1])
            L.orc_kv_quant_row(prior[1, t, h], D, Vc[t, h], Vs[t, h:h + 1])
    qn = rng.standard_normal((B, nQ, D)).astype(np.float32)
    q16 = np.zeros((B, nQ, 2 * D), np.float32)
    q16[:, :, D:] = rng.standard_normal((B, nQ, D)).astype(np.float32)   # the gates
    ctrl = np.array([[0, T - 1, T, -1] for T in Ts], np.int32)
    dCtrl, dQ16, dQn = dev.upload(ctrl), dev.upload(q16), dev.upload(qn)
    dKc, dVc, dKs, dVs = dev.upload(Kc), dev.upload(Vc), dev.upload(Ks), dev.upload(Vs)
    dPm, dPse, dPacc = dev.zeros(B * nQ * nch * 4), dev.zeros(B * nQ * nch * 4), dev.zeros(B * nQ * nch * D * 4)
    dQ8, dSQ = dev.zeros(B * nQ * D), dev.zeros(B * nQ * 2 * 4)
    groups = (dev.info().sm_count * 8 + B - 1) // B
    dev.kernel("BatchAttnSplit")(B * groups, 0, 0, 0, 0, 0, 0, 0, dCtrl, dQn, dKc, dVc, dKs, dVs, dPm, dPse, dPacc, dQ8, dSQ,
                                 nQ, nKV, 64, max_ctx, nch, B, groups, 1e-6, 0)
    dAtt = dev.zeros(nQ * D * 4)
    d8, dS = dev.zeros(nQ * D), dev.zeros(nQ * 2 * 4)
    comb = dev.kernel("AttnCombine")
    for b, T in enumerate(Ts):
        comb(nQ, dPm + b * nQ * nch * 4, dPse + b * nQ * nch * 4, dPacc + b * nQ * nch * D * 4, dQ16 + b * nQ * 2 * D * 4,
             dCtrl + 16 * b, d8, dS, dAtt, nQ, max_ctx, nch)
        dev.sync()
        want = np.zeros((nQ, D), np.float32)
        L.orc_attn_int8kv(qn[b], Kc.reshape(-1), Ks.reshape(-1), Vc.reshape(-1), Vs.reshape(-1),
                          np.ascontiguousarray(q16[b, :, D:]), nQ, nKV, D, T, want)
        assert np.array_equal(dev.download(dAtt, (nQ, D), np.float32), want), (b, T)


@pytest.mark.parametrize("E,k,H,I", [(32, 2, 256, 128), (64, 4, 1024, 256), (512, 10, 2048, 512)])
def test_moe_block(dev, E, k, H, I):
    """RouterTopK + ExpertGateUp + ExpertDownCombine vs the oracle's MoE arithmetic."""
    L = O.lib()
    rng = np.random.default_rng(E)
    hn = rng.standard_normal(H).astype(np.float32)
    hq, hs = O.aquant(hn)
    Wr = O.bf16_bits((rng.standard_normal((E, H)) * 0.05).astype(np.float32))
    Wsg = O.bf16_bits((rng.standard_normal(H) * 0.05).astype(np.float32))
    logits = np.array([L.orc_dot_bf16(np.ascontiguousarray(Wr[e]), hn, H) for e in range(E)], np.float32)
    idx = np.zeros(k, np.int32); wt = np.zeros(k, np.float32); gap = C.c_float()
    L.orc_router_topk(logits, E, k, idx, wt, C.byref(gap))
    sg = np.float32(1.0) / (np.float32(1.0) + np.float32(L.orc_expf(-L.orc_dot_bf16(Wsg, hn, H))))
    # weights only for the experts that can be selected plus a few decoys (memory)
    need = sorted(set(idx.tolist()) | set(range(0, E, max(1, E // 8))))
    tab = np.zeros(E + 1, EXPERT_W)
    host = {}
    for e in need + [E]:
        g = rnd_weights(rng, I, H); u = rnd_weights(rng, I, H); d = rnd_weights(rng, H, I)
        host[e] = (g, u, d)
        tab[e] = tuple(dev.upload(a) for a in (g[0], g[1], u[0], u[1], d[0], d[1]))
    for e in range(E):
        if e not in host:
            tab[e] = tab[need[0]]
    dLog, dCnt = dev.zeros((E + 1) * 4), dev.zeros(4)
    dSelI, dSelW, dGap = dev.zeros((k + 1) * 4), dev.zeros((k + 1) * 4), dev.zeros(4)
    dHn = dev.upload(hn)
    dTab = dev.upload(tab.view(np.uint8))
    dRows = dev.zeros((k + 1) * EXPERT_W.itemsize)   # the selected experts' records, slot order
    router = dev.kernel("RouterTopK")
    for _ in range(2):   # twice: the arrival counter must be left at zero
        router((E + 8) // 8, dev.upload(Wr), dev.upload(Wsg), dHn, dLog, dCnt, dSelI, dSelW, dGap, E, H, k, dTab, dRows)
    dev.sync()
    assert np.array_equal(dev.download(dLog, E, np.float32), logits)
    selI = dev.download(dSelI, k + 1, np.int32); selW = dev.download(dSelW, k + 1, np.float32)
    assert selI[:k].tolist() == idx.tolist() and selI[k] == E
    assert np.array_equal(selW[:k], wt) and selW[k] == sg
    assert dev.download(dGap, 1, np.float32)[0] == np.float32(gap.value)
    slots = k + 1
    rows = dev.download(dRows, k + 1, EXPERT_W)
    assert all(rows[s_] == tab[int(selI[s_])] for s_ in range(k + 1))
    dAct = dev.zeros(slots * I * 4)
    # gate/up through the index list; down through the records the router published (null index list)
    dev.kernel("ExpertGateUp")(dev.info().sm_count * 2, dTab, dSelI, dev.upload(hq), dev.upload(hs), dAct,
                               slots, I, H, 0, 1)
    res = rng.standard_normal(H).astype(np.float32)
    dX, dMoe = dev.zeros(H * 4), dev.zeros(H * 4)
    dev.kernel("ExpertDownCombine")(dev.info().sm_count, dRows, 0, dSelW, dAct, dev.upload(res), dX, dMoe,
                                    slots, I, H)
    dev.sync()
    act_ref = np.zeros((slots, I), np.float32); y = np.zeros((slots, H), np.float32)
    for s in range(slots):
        g, u, d = host[int(selI[s])]
        gg = O.gemv_a8(g[0], g[1], hq, hs); uu = O.gemv_a8(u[0], u[1], hq, hs)
        act_ref[s] = np.array([(a / (np.float32(1.0) + np.float32(L.orc_expf(float(-a))))) * b
                               for a, b in zip(gg, uu)], np.float32)
        aq, asq = O.aquant(act_ref[s])
        y[s] = O.gemv_a8(d[0], d[1], aq, asq)
    assert np.array_equal(dev.download(dAct, (slots, I), np.float32), act_ref)
    acc = np.zeros(H, np.float32)
    for s in range(slots):
        acc = acc + selW[s] * y[s]
    assert np.array_equal(dev.download(dMoe, H, np.float32), acc)
    assert np.array_equal(dev.download(dX, H, np.float32), res + acc)


def test_argmax_first_max_wins_and_advance(dev):
    rng = np.random.default_rng(5)
    V = 151936
    lg = rng.standard_normal(V).astype(np.float32)
    lg[[777, 90000, 150000]] = lg.max() + 1.0   # planted three-way tie: lowest index wins
    parts = 64
    dPV, dPI, dOut = dev.zeros(parts * 4), dev.zeros(parts * 4), dev.zeros(4)
    ctrl = np.array([5, 10, 11, -1], np.int32)
    dCtrl, dHist = dev.upload(ctrl), dev.zeros(16 * 4)
    dev.kernel("ArgmaxStage1")(parts, dev.upload(lg), dPV, dPI, V)
    dev.kernel("ArgmaxStage2")(1, dPV, dPI, dOut, dCtrl, dHist, parts, 1, 16)
    dev.sync()
    assert dev.download(dOut, 1, np.int32)[0] == 777 == O.lib().orc_argmax(lg, V)
    assert dev.download(dCtrl, 4, np.int32).tolist() == [777, 11, 12, 777]
    assert dev.download(dHist, 16, np.int32)[10] == 777


def test_synth_kernels_match_oracle_generator(dev):
    from ainfer_b200 import synth_key
    name, seed, N, K = "model.language_model.layers.0.mlp.experts.3.up_proj.weight", 0, 64, 512
    w = O.synth_normal(name, seed, N * K, 0.02).reshape(N, K)
    P, S = O.quantize_int4(w)
    dP, dS = dev.zeros(N * K // 2), dev.zeros(N * K // 128 * 2)
    k = dev.kernel("SynthInt4")
    k.set_arg(0, dP); k.set_arg(1, dS); k.set_arg(2, synth_key(seed, name), "u64")
    k.set_arg(3, N * K // 128, "u64"); k.set_arg(4, 0.02)
    k.launch(8)
    dB = dev.zeros(N * K * 2)
    k2 = dev.kernel("SynthBf16")
    k2.set_arg(0, dB); k2.set_arg(1, synth_key(seed, name), "u64"); k2.set_arg(2, N * K, "u64")
    k2.set_arg(3, 0.02); k2.set_arg(4, 0.0)
    k2.launch(8)
    dev.sync()
    assert np.array_equal(dev.download(dP, P.shape, np.uint8), P)
    assert np.array_equal(dev.download(dS, S.shape, np.uint16), S)
    assert np.array_equal(dev.download(dB, N * K, np.uint16), O.bf16_bits(w.reshape(-1)))


def test_command_list_replay_is_deterministic(dev):
    """Record once, replay: outputs bitwise identical (the reference's replay-determinism
    check, tools/cmdlist/gemv_replay.cpp)."""
    rng = np.random.default_rng(11)
    N, K = 512, 2048
    P, S = rnd_weights(rng, N, K)
    xq, sq = O.aquant(rng.standard_normal(K).astype(np.float32))
    tab = np.zeros(1, GEMV_MAT)
    dY = dev.zeros(N * 4)
    tab[0]["P"], tab[0]["S"], tab[0]["Y"], tab[0]["N"], tab[0]["ldy"] = dev.upload(P), dev.upload(S), dY, N, N
    k = dev.kernel("Int4GemvA8")
    k.set_args(dev.upload(tab.view(np.uint8)), 1, N, dev.upload(xq), dev.upload(sq), K, 1)
    lst = dev.new_list()
    lst.append(k, 32)
    lst.close()
    outs = []
    for _ in range(3):
        dev.fill(dY, 0xFF, N * 4)     # NaN-poison: proves the kernel wrote every row
        lst.execute()
        dev.sync()
        outs.append(dev.download(dY, N, np.float32))
    lst.destroy()
    assert np.array_equal(outs[0], O.gemv_a8(P, S, xq, sq))
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[1], outs[2])


@pytest.mark.parametrize("N,K,M", [(512, 2048, 1), (512, 2048, 5), (4096, 2048, 64), (1000, 512, 3),
                                   (2048, 512, 8), (130, 256, 64)])
def test_gemm_a16_within_reference_tolerance(dev, N, K, M):
    """Int4GemmA16 (bf16 activations, tensor-core products) vs the double-precision host form of the
    float-activation policy. Tolerance: rel 2e-2 / abs 1e-2, the bar of the reference's own GEMV test."""
    rng = np.random.default_rng(N + K + M)
    P, S = rnd_weights(rng, N, K)
    xb = O.bf16_bits(rng.standard_normal((M, K)).astype(np.float32))
    want = O.gemv_a16(P, S, O.bf16_to_f32(xb))
    dY = dev.zeros(M * N * 4)
    dev.kernel("Int4GemmA16")((N + 127) // 128, dev.upload(P), dev.upload(S), dev.upload(xb), dY, N, K, M)
    dev.sync()
    got = dev.download(dY, (M, N), np.float32)
    err = np.abs(got - want)
    assert np.all(err <= 1e-2 + 2e-2 * np.abs(want)), float(err.max())
    # far inside the bar in practice: fp32 accumulation of exact bf16 products
    assert float(err.max()) <= 1e-4 * max(1.0, float(np.abs(want).max()))
