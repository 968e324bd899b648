"""Host-side model of the expert-parallel MoE block's protocol (test infrastructure): ownership,
dispatch plan, exchange and slot-ordered combine in numpy over torch.distributed, with the
arithmetic supplied by a backend (the CPU oracle in the tests). The runtime's own implementation
is csrc/runtime/ep.cpp with the kernels of csrc/kernels/k_ep.cu; this model states the same
protocol in a form that runs as gloo ranks without a GPU.

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

The exchange runs on torch.distributed (gloo in the CPU tests); the arithmetic is a backend
object (the tests plug in the CPU oracle). Shapes follow the reference's conventions: one
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
