"""Expert-parallel MoE block for a decode batch (the one place the decode path shards across GPUs).

Experts are split evenly over the ranks (contiguous ids, E/R per rank); router, shared expert and
everything outside the MoE block are replicated. Rank r OWNS tokens [r*B/R, (r+1)*B/R) of the batch:

  1. owner: post-attention RMSNorm + activation quantiser, router, top-k (its own tokens only);
  2. dispatch: every (token, slot) item goes to the rank that holds the slot's expert, as the
     token's quantised hidden vector (H int8 + H/128 fp32 scales, not the fp32 vector) plus
     (token, slot, expert) metadata: one all-to-all of item counts, one of payload bytes;
  3. expert owner: gate/up + SiLU-mul + down projection of each received item, unweighted;
  4. combine: the fp32 outputs travel back with a second all-to-all; the token's owner adds them
     in slot order (routed ranks first, shared expert last) to the residual, the same additions
     in the same order as the single-GPU kernel, so the result is bit-identical to it;
  5. all-gather of the owners' rows, so that every replica holds the whole batch again.

The exchange runs on torch.distributed (NCCL on GPUs, gloo in the CPU tests); the arithmetic is a
backend object (`GpuMoeBackend` drives this package's kernels; the tests also plug in the CPU
oracle to check the host logic without a GPU). Shapes follow the reference's conventions: one
hidden row per token, experts addressed by global id.
"""
import numpy as np

ITEM_META = np.dtype([("token", "<i4"), ("slot", "<i4"), ("expert", "<i4"), ("pad", "<i4")])


def owned_range(batch, rank, world):
    per = (batch + world - 1) // world
    lo = min(batch, rank * per)
    return lo, min(batch, lo + per)


def expert_owner(expert, experts, world):
    """Rank that holds a routed expert (contiguous shards of experts/world ids)."""
    return int(expert) // (experts // world)


def plan_dispatch(sel_idx, token0, experts, world):
    """sel_idx: [n_owned][k] routed expert ids of this rank's tokens (rank order). Returns, per
    destination rank, an ITEM_META array of the items to send there, ordered by (token, slot)."""
    out = [[] for _ in range(world)]
    for t in range(sel_idx.shape[0]):
        for j in range(sel_idx.shape[1]):
            e = int(sel_idx[t, j])
            out[expert_owner(e, experts, world)].append((token0 + t, j, e, 0))
    return [np.array(v, ITEM_META) if v else np.zeros(0, ITEM_META) for v in out]


class TorchComm:
    """All-to-all / all-gather of byte buffers over a torch.distributed group (nccl or gloo)."""

    def __init__(self, group=None, device=None):
        import torch
        import torch.distributed as dist
        self.torch, self.dist, self.group = torch, dist, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.device = device if device is not None else torch.device("cpu")

    def _t(self, a):
        return self.torch.from_numpy(np.ascontiguousarray(a)).to(self.device)

    def exchange(self, send):
        """send: list (per destination rank) of uint8 arrays. Returns the list (per source rank)
        of uint8 arrays received."""
        torch, dist = self.torch, self.dist
        counts = torch.tensor([len(b) for b in send], dtype=torch.int64, device=self.device)
        rcounts = torch.zeros_like(counts)
        dist.all_to_all_single(rcounts, counts, group=self.group)
        rc = [int(x) for x in rcounts.cpu()]
        sc = [len(b) for b in send]
        sbuf = self._t(np.concatenate([np.asarray(b, np.uint8) for b in send]) if sum(sc) else np.zeros(0, np.uint8))
        rbuf = torch.zeros(sum(rc), dtype=torch.uint8, device=self.device)
        dist.all_to_all_single(rbuf, sbuf, output_split_sizes=rc, input_split_sizes=sc, group=self.group)
        flat = rbuf.cpu().numpy()
        out, o = [], 0
        for n in rc:
            out.append(flat[o:o + n].copy())
            o += n
        return out

    def all_gather_rows(self, rows, batch):
        """rows: this rank's owned rows [n_owned][H] fp32; returns the whole batch [batch][H]."""
        torch, dist = self.torch, self.dist
        H = rows.shape[1]
        per = (batch + self.world - 1) // self.world
        pad = np.zeros((per, H), np.float32)
        pad[:rows.shape[0]] = rows
        mine = self._t(pad)
        parts = [torch.zeros_like(mine) for _ in range(self.world)]
        dist.all_gather(parts, mine, group=self.group)
        full = np.concatenate([p.cpu().numpy() for p in parts], 0)
        return full[:batch]


class LocalComm:
    """World of one rank (no exchange): the single-GPU decomposition of the same block."""
    rank, world = 0, 1

    def exchange(self, send):
        return [np.asarray(send[0], np.uint8)]

    def all_gather_rows(self, rows, batch):
        return rows[:batch]


class EpMoeBlock:
    """x = res + MoE(norm(res)) for a batch of token rows, experts sharded over comm.world ranks.

    backend must provide:
      hidden, experts, top_k, shared (bool)
      route(res_row) -> (hq int8[H], hs f32[H/128], sel_idx int32[k], sel_w f32[k+1])
      expert(expert_id, hq, hs) -> y f32[H]          (unweighted down-projection output)
      combine(res_row, ys f32[slots][H], w f32[slots]) -> x_row f32[H]
    """

    def __init__(self, backend, comm):
        self.b, self.comm = backend, comm
        if backend.experts % comm.world:
            raise ValueError("experts must divide evenly over the ranks")
        self.stats = {}

    def forward(self, res):
        b, comm = self.b, self.comm
        B, H = res.shape
        k, G = b.top_k, H // 128
        lo, hi = owned_range(B, comm.rank, comm.world)
        item_bytes = H + G * 4
        # 1. route the owned tokens
        routed = [b.route(res[t]) for t in range(lo, hi)]
        sel = np.array([r[2] for r in routed], np.int32).reshape(hi - lo, k)
        # 2. dispatch
        plans = plan_dispatch(sel, lo, b.experts, comm.world)
        send = []
        for p in plans:
            payload = np.zeros((len(p), item_bytes), np.uint8)
            for i, it in enumerate(p):
                hq, hs = routed[it["token"] - lo][0], routed[it["token"] - lo][1]
                payload[i, :H] = hq.view(np.uint8)
                payload[i, H:] = hs.view(np.uint8)
            send.append(np.concatenate([p.view(np.uint8).reshape(-1), payload.reshape(-1)]))
        recv = comm.exchange(send)
        # 3. experts of this rank
        back = []
        n_items = 0
        for src, raw in enumerate(recv):
            n = len(raw) // (ITEM_META.itemsize + item_bytes)
            meta = raw[:n * ITEM_META.itemsize].view(ITEM_META)
            pay = raw[n * ITEM_META.itemsize:].reshape(n, item_bytes)
            ys = np.zeros((n, H), np.float32)
            for i in range(n):
                hq = pay[i, :H].view(np.int8)
                hs = pay[i, H:].view(np.float32)
                ys[i] = b.expert(int(meta[i]["expert"]), hq, hs)
            n_items += n
            back.append(np.concatenate([meta.view(np.uint8).reshape(-1), ys.view(np.uint8).reshape(-1)]))
        # 4. combine on the owners
        got = comm.exchange(back)
        slots = k + (1 if b.shared else 0)
        ys_all = np.zeros((hi - lo, slots, H), np.float32)
        for raw in got:
            n = len(raw) // (ITEM_META.itemsize + H * 4)
            meta = raw[:n * ITEM_META.itemsize].view(ITEM_META)
            ys = raw[n * ITEM_META.itemsize:].view(np.float32).reshape(n, H)
            for i in range(n):
                ys_all[meta[i]["token"] - lo, meta[i]["slot"]] = ys[i]
        out = np.zeros((hi - lo, H), np.float32)
        for t in range(hi - lo):
            hq, hs, _, w = routed[t]
            if b.shared:  # replicated: computed by the owner itself
                ys_all[t, k] = b.expert(b.experts, hq, hs)
            out[t] = b.combine(res[lo + t], ys_all[t], np.ascontiguousarray(w[:slots]))
        self.stats = {"owned_tokens": hi - lo, "items_sent": int(sum(len(p) for p in plans)),
                      "items_computed": n_items,
                      "dispatch_bytes": int(sum(len(p) for p in plans)) * (item_bytes + ITEM_META.itemsize),
                      "combine_bytes": n_items * (H * 4 + ITEM_META.itemsize)}
        # 5. every replica gets the whole batch back
        return comm.all_gather_rows(out, B)


EXPERT_W = np.dtype([("gP", "<u8"), ("gS", "<u8"), ("uP", "<u8"), ("uS", "<u8"), ("dP", "<u8"), ("dS", "<u8")])


def _bf16_to_f32(u16):
    return (u16.astype(np.uint32) << 16).view(np.float32)


class GpuMoeBackend:
    """The MoE block of one layer of a loaded model, run with this package's kernels through the
    C-ABI. Only the experts of this rank's shard are ever touched by `expert` calls that the
    dispatch plan routes here (plus the replicated shared expert)."""

    def __init__(self, dev, model, layer):
        cfg = model.config
        self.dev, self.hidden, self.experts = dev, cfg["hidden"], cfg["experts"]
        self.top_k, self.shared, self.inter = cfg["top_k"], bool(cfg["shared_experts"]), cfg["expert_intermediate"]
        self.eps = float(cfg["rms_eps"])
        H, E, I, k = self.hidden, self.experts, self.inter, self.top_k
        p = f"model.language_model.layers.{layer}."
        t = model.tensor
        self.router = t(p + "mlp.gate.weight").data
        self.sgate = t(p + "mlp.shared_expert_gate.weight").data if self.shared else 0
        nw = t(p + "post_attention_layernorm.weight")
        self.norm_w = dev.upload(_bf16_to_f32(dev.download(nw.data, H, np.uint16)))
        tab = np.zeros(E + 1, EXPERT_W)
        for e in range(E + 1):
            q = p + (f"mlp.experts.{e}." if e < E else "mlp.shared.")
            if e == E and not self.shared:
                continue
            g, u, d = t(q + "gate_proj.weight"), t(q + "up_proj.weight"), t(q + "down_proj.weight")
            tab[e] = (g.data, g.scales, u.data, u.scales, d.data, d.scales)
        self.tab = dev.upload(tab.view(np.uint8))
        # scratch (allocated once)
        z = dev.zeros
        self.dRes, self.dHn, self.dQ8, self.dSQ = z(H * 4), z(H * 4), z(H), z(H // 128 * 4)
        self.dLog, self.dCnt = z((E + 1) * 4), z(4)
        self.dSelI, self.dSelW, self.dGap = z((k + 1) * 4), z((k + 1) * 4), z(4)
        self.dOne, self.dAct, self.dY, self.dX = dev.upload(np.ones(1, np.float32)), z(I * 4), z(H * 4), z(H * 4)
        self.dZero, self.dE1 = z(H * 4), z(4)
        self.dYs, self.dW = z((k + 1) * H * 4), z((k + 1) * 4)
        self.sm = dev.info().sm_count
        self.k_norm, self.k_router = dev.kernel("RmsNormQuant"), dev.kernel("RouterTopK")
        self.k_up, self.k_down, self.k_comb = dev.kernel("ExpertGateUp"), dev.kernel("ExpertDownCombine"), dev.kernel("CombineSlots")

    def route(self, res_row):
        d, H, E, k = self.dev, self.hidden, self.experts, self.top_k
        d.write(self.dRes, np.ascontiguousarray(res_row, np.float32))
        self.k_norm(1, self.dRes, 0, 0, self.norm_w, self.dHn, self.dQ8, self.dSQ, H, self.eps)
        self.k_router((E + 8) // 8, self.router, self.sgate, self.dHn, self.dLog, self.dCnt, self.dSelI, self.dSelW,
                      self.dGap, E, H, k, 0, 0)
        d.sync()
        return (d.download(self.dQ8, H, np.int8), d.download(self.dSQ, H // 128, np.float32),
                d.download(self.dSelI, k, np.int32), d.download(self.dSelW, k + 1, np.float32))

    def expert(self, e, hq, hs):
        d, H, I = self.dev, self.hidden, self.inter
        d.write(self.dQ8, np.ascontiguousarray(hq)); d.write(self.dSQ, np.ascontiguousarray(hs))
        d.write(self.dE1, np.array([e], np.int32))
        self.k_up(min(2 * self.sm, max(1, 2 * I * H // 32768)), self.tab, self.dE1, self.dQ8, self.dSQ, self.dAct, 1, I, H, 0, 0)
        self.k_down(min(2 * self.sm, max(1, H // 8)), self.tab, self.dE1, self.dOne, self.dAct, self.dZero, self.dX, self.dY, 1, I, H)
        d.sync()
        return d.download(self.dY, H, np.float32)

    def combine(self, res_row, ys, w):
        d, H = self.dev, self.hidden
        slots = ys.shape[0]
        d.write(self.dRes, np.ascontiguousarray(res_row, np.float32))
        d.write(self.dYs, np.ascontiguousarray(ys)); d.write(self.dW, np.ascontiguousarray(w, np.float32))
        self.k_comb(max(1, H // 256), self.dYs, self.dW, self.dRes, self.dX, slots, H)
        d.sync()
        return d.download(self.dX, H, np.float32)

    def fused_reference(self, res_row):
        """The same block through the single-GPU kernels (all slots in one launch each)."""
        d, H, E, I, k = self.dev, self.hidden, self.experts, self.inter, self.top_k
        slots = k + (1 if self.shared else 0)
        self.route(res_row)
        dAct = d.zeros(slots * I * 4)
        self.k_up(2 * self.sm, self.tab, self.dSelI, self.dQ8, self.dSQ, dAct, slots, I, H, 0, 0)
        self.k_down(self.sm, self.tab, self.dSelI, self.dSelW, dAct, self.dRes, self.dX, 0, slots, I, H)
        d.sync()
        out = d.download(self.dX, H, np.float32)
        d.free(dAct)
        return out
