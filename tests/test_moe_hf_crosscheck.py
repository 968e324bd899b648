"""Third-party cross-check of the oracle's MoE block (router softmax, top-k, renormalised
weights, shared-expert gate, expert MLP, combine) against Hugging Face transformers'
Qwen3NextSparseMoeBlock, which is CALLED here, not restated.

The reference has no MoE code, so nothing of its own pins this part of the oracle. HF's block
computes in fp32 on the dequantised weights; the oracle quantises activations to INT8 per group
of 128 (the decode policy), so routing must agree exactly away from near-ties, routing weights
and the shared gate to fp32 rounding, and the block output to the activation-quantisation error.
"""
import ctypes as C
import json

import numpy as np
import pytest

import oracle_lib as O

torch = pytest.importorskip("torch")
hf = pytest.importorskip("transformers.models.qwen3_next.modeling_qwen3_next")
hfc = pytest.importorskip("transformers.models.qwen3_next.configuration_qwen3_next")


def dequant(t):
    """fp32 matrix of an INT4 g128 tensor of the oracle model (low nibble = even k)."""
    rows, cols = t["shape"]
    b = t["data"].reshape(rows, cols // 2)
    lo = (b & 0xF).astype(np.int8)
    hi = (b >> 4).astype(np.int8)
    lo = np.where(lo >= 8, lo - 16, lo)
    hi = np.where(hi >= 8, hi - 16, hi)
    q = np.empty((rows, cols), np.float32)
    q[:, 0::2] = lo
    q[:, 1::2] = hi
    sc = O.bf16_to_f32(t["scales"]).reshape(rows, cols // 128)
    return q * np.repeat(sc, 128, axis=1)


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_oracle_moe_block_agrees_with_hf_qwen3_next(seed):
    H, E, k, I = 256, 32, 4, 128
    arch = dict(arch="qwen3_5_moe", text_layers=1, layer_types="L", hidden=H, vocab=512, q_heads=2, kv_heads=1,
                head_dim=256, rotary_dim=64, rope_theta=1e7, lin_k_heads=2, lin_v_heads=4, lin_head_dim=128,
                conv_kernel=4, experts=E, top_k=k, shared_experts=1, expert_intermediate=I, mtp_layers=0,
                rms_eps=1e-6)
    om = O.Model(arch_json=json.dumps(arch, separators=(",", ":")), synth_seed=seed)
    pfx = "model.language_model.layers.0."
    cfg = hfc.Qwen3NextConfig(hidden_size=H, num_experts=E, num_experts_per_tok=k, moe_intermediate_size=I,
                              shared_expert_intermediate_size=I, norm_topk_prob=True, hidden_act="silu")
    blk = hf.Qwen3NextSparseMoeBlock(cfg).float().eval()
    with torch.no_grad():
        router = O.bf16_to_f32(om.tensor(pfx + "mlp.gate.weight")["data"].view(np.uint16)).reshape(E, H)
        blk.gate.weight.copy_(torch.from_numpy(router))
        sg = O.bf16_to_f32(om.tensor(pfx + "mlp.shared_expert_gate.weight")["data"].view(np.uint16)).reshape(1, H)
        blk.shared_expert_gate.weight.copy_(torch.from_numpy(sg))
        for e in range(E):
            ep = f"{pfx}mlp.experts.{e}."
            g, u, d = (dequant(om.tensor(ep + n + ".weight")) for n in ("gate_proj", "up_proj", "down_proj"))
            blk.experts.gate_up_proj[e].copy_(torch.from_numpy(np.concatenate([g, u], 0)))
            blk.experts.down_proj[e].copy_(torch.from_numpy(d))
        for n in ("gate_proj", "up_proj", "down_proj"):
            getattr(blk.shared_expert, n).weight.copy_(torch.from_numpy(dequant(om.tensor(f"{pfx}mlp.shared.{n}.weight"))))
    hn = O.synth_normal("crosscheck.hn", seed, H, 1.0)
    out = np.zeros(H, np.float32)
    routed = np.zeros(k, np.int32)
    gap = np.zeros(1, np.float32)
    O.lib().orc_moe_block(om.h, pfx.encode(), hn, out, routed, gap)
    with torch.no_grad():
        x = torch.from_numpy(hn).view(1, 1, H)
        want = blk(x).view(H).numpy()
        _, w_hf, idx_hf = blk.gate(x.view(1, H))
        sg_hf = torch.sigmoid(blk.shared_expert_gate(x.view(1, H))).item()
    # routing: same experts in the same rank order (this draw is not a near-tie)
    assert gap[0] > 1e-5
    assert routed.tolist() == idx_hf.view(-1).tolist()
    # routing weights and shared gate: the oracle's own arithmetic on the same logits
    logits = np.array([O.lib().orc_dot_bf16(np.ascontiguousarray(router_row), hn, H) for router_row in
                       om.tensor(pfx + "mlp.gate.weight")["data"].view(np.uint16).reshape(E, H)], np.float32)
    idx = np.zeros(k, np.int32); wt = np.zeros(k, np.float32); g2 = np.zeros(1, np.float32)
    O.lib().orc_router_topk(logits, E, k, idx, wt, g2.ctypes.data_as(C.POINTER(C.c_float)))
    assert idx.tolist() == routed.tolist()
    assert np.allclose(wt, w_hf.view(-1).numpy(), rtol=2e-5, atol=1e-7)
    sg_row = om.tensor(pfx + "mlp.shared_expert_gate.weight")["data"].view(np.uint16)
    sg_orc = 1.0 / (1.0 + np.exp(-np.float64(O.lib().orc_dot_bf16(np.ascontiguousarray(sg_row), hn, H))))
    assert abs(sg_orc - sg_hf) < 1e-5
    # block output: INT8 activations against fp32 activations
    err = np.abs(out - want).max()
    assert err <= 2e-2 * np.abs(want).max() + 1e-4, (err, np.abs(want).max())
    om.close()
