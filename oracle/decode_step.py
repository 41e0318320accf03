"""Oracle for one whole decode / speculative-verify step: the per-layer flow of the reference's layer node
(kb34/qwen36_layer/layer.py:486-531: token mixer -> prepare_mlp (deferred projection + residual add + Gemma norm,
proj.py:84-112) -> sparse MoE -> combine + next layer's input norm, qk_route.cu:779-819) and of its LM-head node
(qwen36_lmhead8/node.py:136-151) composed from the pieces of this package, at the target formats (fp8
block-scaled projections and experts, e4m3 KV pages, explicit fp32 GDN state, greedy argmax).

Test infrastructure only (see oracle/__init__.py).  PARITY UNPINNED as a whole: the reference runs this flow only
inside a serving engine on a GPU; every piece carries its own pin or its own "unpinned" note.

A model is a dict of numpy arrays: `layers` (list of per-layer dicts with the keys used below), `first_norm`,
`lm_w`, `lm_s`, `cos_sin`, `positions`, `seqlens`, `accepted`; bf16 tensors as fp32 values, e4m3 tensors as uint8
codes.
"""
from __future__ import annotations

import numpy as np

from . import attn_lmhead as al
from . import attn_verify as av
from . import gdn as ogdn
from . import moe as omoe
from . import router as orouter
from .numerics import F32

GDN_SPLIT = (8192, 4096, 32, 32)   # q | k | v, z, b, a (dense8.py:64-68)
TOP_K = 10


def mixer_gdn(L, h, accepted):
    """in_proj -> GDN verify -> out_proj (layer.py:294-371; gdn_fused.py:37-57).  Returns (proj, state', conv_state')."""
    p = al.dense_fp8(h, L["in_w"], L["in_s"])
    o0, o1, o2 = GDN_SPLIT[0], GDN_SPLIT[0] + GDN_SPLIT[1], GDN_SPLIT[0] + GDN_SPLIT[1] + GDN_SPLIT[2]
    mixed, z, b, a = p[:, :o0], p[:, o0:o1], p[:, o1:o2], p[:, o2:]
    core, state, conv = ogdn.gdn_verify(mixed, z, a, b, L["conv_state"], L["conv_w"], L["a_log"], L["dt_bias"], L["state"],
                                        accepted, L["gdn_norm"], 1e-6)
    return al.dense_fp8(core, L["out_w"], L["out_s"]), state, conv


def mixer_attn(L, h, positions, cos_sin, seqlens):
    """fused projection front -> attention verify core -> o_proj (attn_fused.py:213-275).  Returns (proj, kcache', vcache')."""
    q, gate, k, v = al.attn_front(h, L["qkv_w"], L["qkv_s"], L["q_norm"], L["k_norm"], positions, cos_sin, 1e-6, True)
    core, kc, vc = av.attn_verify(q, gate, k, v, L["kcache"], L["vcache"], L["page_table"], seqlens)
    return al.dense_fp8(core, L["o_w"], L["o_s"]), kc, vc


def route(L, h2):
    """(logits, ids, weights) of the layer's router over all experts."""
    logits = orouter.gate_logits(h2, L["wr"])
    ids, wts = orouter.topk_softmax(logits, TOP_K)
    return logits, ids, wts


def moe(L, h2, ids, wts):
    """Routed + shared fp8 experts and the combine (without the next layer's norm); returns (out, debug dict)."""
    return omoe.moe_fp8(h2, ids, wts, L["w13"], L["s13"], L["w2"], L["s2"], L["sh13"], L["shs13"], L["sh2"], L["shs2"],
                        L["gate_w"], want_debug=True)


def layer(L, h, residual, model, ids=None, wts=None):
    """One decoder layer.  h = normed input rows, residual = the running residual (both bf16 values [T, 2048]).
    `ids` / `wts` override the router's picks (a test that found a near tie hands the other side's picks in).
    Returns a dict: proj, h2, residual_mid, logits, ids, wts, moe_out, h_out, residual_out and the updated state
    (state / conv_state or kcache / vcache)."""
    out = {}
    if L["attn"]:
        proj, out["kcache"], out["vcache"] = mixer_attn(L, h, model["positions"], model["cos_sin"], model["seqlens"])
    else:
        proj, out["state"], out["conv_state"] = mixer_gdn(L, h, model["accepted"])
    h2, r_mid = al.add_rmsnorm(proj, residual, L["post_norm"])
    logits, rid, rwt = route(L, h2)
    if ids is None:
        ids, wts = rid, rwt
    moe_out, dbg = moe(L, h2, ids, wts)
    h_out, r_out = al.add_rmsnorm(moe_out, r_mid, L["next_norm"])
    out.update(proj=proj, h2=h2, residual_mid=r_mid, logits=logits, ids=ids, wts=wts, router_ids=rid, moe_out=moe_out,
               cache=dbg["cache"], h_out=h_out, residual_out=r_out)
    return out


def lm_tokens(model, h, world=1):
    """Greedy token per row: per vocabulary shard (max, argmax), then the merge (largest value, lower id on ties).
    Returns (tokens int32 [T], logits fp32 [T, V])."""
    logits = al.lmhead_logits(h, model["lm_w"], model["lm_s"])
    V = logits.shape[1]
    mx, ix = [], []
    for lo, hi in al.vocab_shards(V, world):
        m, i = al.shard_argmax(logits[:, lo:hi], lo)
        mx.append(m)
        ix.append(i)
    return al.merge_argmax(np.stack(mx), np.stack(ix)), logits


def decode_step(model, x):
    """The whole step, free running: x bf16 values [T, 2048] -> (tokens, final hidden, per-layer outputs)."""
    residual = np.zeros_like(np.asarray(x, dtype=F32))
    h, residual = al.add_rmsnorm(x, residual, model["first_norm"])
    outs = []
    for L in model["layers"]:
        o = layer(L, h, residual, model)
        h, residual = o["h_out"], o["residual_out"]
        outs.append(o)
    tokens, _ = lm_tokens(model, h)
    return tokens, h, outs
