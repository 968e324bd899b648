"""MoE-block arithmetic on the CPU oracle, in the shape ep_harness.EpMoeBlock expects from a
backend. Test infrastructure: lets the expert-parallel host logic (ownership, dispatch plan,
exchange, slot-ordered combine, gather) run as gloo ranks without a GPU."""
import ctypes as C

import numpy as np

import oracle_lib as O


class OracleMoeBackend:
    def __init__(self, hidden, experts, top_k, inter, seed=0, shared=True, eps=1e-6):
        self.hidden, self.experts, self.top_k, self.inter, self.shared, self.eps = hidden, experts, top_k, inter, shared, eps
        rng = np.random.default_rng(seed)
        H, E, I = hidden, experts, inter
        self.norm_w = (rng.standard_normal(H) * 0.05).astype(np.float32)
        self.router = O.bf16_bits((rng.standard_normal((E, H)) * 0.05).astype(np.float32))
        self.sgate = O.bf16_bits((rng.standard_normal(H) * 0.05).astype(np.float32))
        q = lambda n, k: O.quantize_int4((rng.standard_normal((n, k)) * 0.02).astype(np.float32))
        self.w = [(q(I, H), q(I, H), q(H, I)) for _ in range(E + 1)]
        self.calls = []

    def route(self, res_row):
        L, H, E, k = O.lib(), self.hidden, self.experts, self.top_k
        hn = np.zeros(H, np.float32)
        L.orc_rmsnorm(np.ascontiguousarray(res_row, np.float32), self.norm_w, H, C.c_float(self.eps), hn)
        hq, hs = O.aquant(hn)
        logits = np.array([L.orc_dot_bf16(np.ascontiguousarray(self.router[e]), hn, H) for e in range(E)], np.float32)
        idx = np.zeros(k, np.int32); wt = np.zeros(k, np.float32); gap = C.c_float()
        L.orc_router_topk(logits, E, k, idx, wt, C.byref(gap))
        sg = np.float32(1.0) / (np.float32(1.0) + np.float32(L.orc_expf(-L.orc_dot_bf16(self.sgate, hn, H))))
        return hq, hs, idx, np.concatenate([wt, [sg]]).astype(np.float32)

    def expert(self, e, hq, hs):
        L = O.lib()
        self.calls.append(int(e))
        g, u, d = self.w[e]
        hq = np.ascontiguousarray(hq, np.int8); hs = np.ascontiguousarray(hs, np.float32)
        gg, uu = O.gemv_a8(g[0], g[1], hq, hs), O.gemv_a8(u[0], u[1], hq, hs)
        act = np.array([(a / (np.float32(1.0) + np.float32(L.orc_expf(float(-a))))) * b for a, b in zip(gg, uu)], np.float32)
        aq, asq = O.aquant(act)
        return O.gemv_a8(d[0], d[1], aq, asq)

    def combine(self, res_row, ys, w):
        acc = np.zeros(self.hidden, np.float32)
        for s in range(ys.shape[0]):
            acc = acc + np.float32(w[s]) * ys[s]
        return (np.asarray(res_row, np.float32) + acc).astype(np.float32)
