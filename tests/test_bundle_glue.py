"""The bundle's two ops behind the reference's plugin interface (prepare / forward), driven by
stand-ins for the engine's objects.  CPU part: manifest and the error behaviour of prepare."""
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BUNDLE = os.path.join(ROOT, "bundles_b200", "bundle")
if BUNDLE not in sys.path:
    sys.path.insert(0, BUNDLE)          # the engine imports `qwen36_layer.layer` relative to the bundle root

from qwen36_layer import layer as qlayer          # noqa: E402
from qwen36_lmhead8 import node as qnode          # noqa: E402

from tests.fake_engine import (FakeDecoderLayer, FakeHybridLayer, FakeLogitsProcessor, FakeMode, FakeMoe,   # noqa: E402
                               fake_attn_backend, fake_gdn_backend)


def test_manifest_has_the_reference_ops():
    import tomllib
    m = tomllib.load(open(os.path.join(BUNDLE, "manifest.toml"), "rb"))
    assert m["abi_version"] == "cacheon-op-abi-v0"
    slots = {op["slot"]: op for op in m["ops"]}
    assert set(slots) == {"model.layers.*", "logits_processor"}
    for op in m["ops"]:
        assert op["entry"] == "forward" and op["prepare"] == "prepare" and op["dtypes"] == ["bfloat16"]
        assert op["architectures"] == ["sm100"]
        assert os.path.exists(os.path.join(BUNDLE, op["source"]))
    for src in slots["model.layers.*"]["cuda_sources"]:
        assert os.path.exists(os.path.join(BUNDLE, src)), src


@pytest.mark.parametrize("kw,msg", [(dict(tp_size=2), "tensor-parallel"), (dict(scoring="sigmoid"), "softmax"),
                                    (dict(renorm=False), "renormalised")])
def test_prepare_rejects_unsupported_configs(kw, msg):
    moe = FakeMoe(64, 256, 128, 4, "cpu", **kw)
    with pytest.raises(qlayer.UnsupportedLayer, match=msg):
        qlayer.prepare(FakeDecoderLayer(moe))


def test_prepare_rejects_bad_shapes_and_cpu_weights():
    with pytest.raises(qlayer.UnsupportedLayer, match="multiple of 256"):
        qlayer.prepare(FakeDecoderLayer(FakeMoe(64, 192, 128, 4, "cpu")))
    with pytest.raises(qlayer.UnsupportedLayer, match="no CPU path"):
        qlayer.prepare(FakeDecoderLayer(FakeMoe(64, 256, 128, 4, "cpu")))
    with pytest.raises(qlayer.UnsupportedLayer, match="no sparse-MoE"):
        qlayer.prepare(torch.nn.Linear(4, 4))
    lp = FakeLogitsProcessor(1024)
    lp.do_tensor_parallel_all_gather = True
    with pytest.raises(qnode.UnsupportedHead):
        qnode.prepare(lp)


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["w8a8", "fp8"])
def test_layer_forward_matches_oracle(fmt, monkeypatch):
    from oracle import moe as omoe
    from oracle import router as orouter
    from bundles_b200 import synth
    from tests.util import bf16_to_np, close_bf16
    monkeypatch.setattr(qlayer, "EXPERT_FORMAT", fmt)
    dev = torch.device("cuda", 0)
    E, H, I, K, T = 64, 2048, 512, 10, 24
    moe = FakeMoe(E, H, I, K, dev, seed=3)
    stock = FakeDecoderLayer(moe)
    before = moe.experts.w13_weight.clone()
    prepared = qlayer.prepare(stock)
    g = torch.Generator().manual_seed(5)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).to(dev)
    res = torch.randn(T, H, generator=g).to(torch.bfloat16).to(dev)
    pos = torch.arange(1, T + 1, device=dev)
    pos[7] = 0                                            # a graph-padding row
    fb = type("FB", (), {"positions": pos})()
    out, residual = qlayer.forward(prepared, pos, x, fb, res)
    torch.cuda.synchronize()
    assert torch.equal(moe.experts.w13_weight, before)    # stock weights are read-only
    assert torch.equal(residual, x + res)
    assert not out[7].any()
    # oracle on the same private-copy arithmetic
    xin = bf16_to_np(residual)
    wr = moe.gate.weight.float().cpu().numpy()
    _, ids, wts = orouter.route(xin, wr, K)
    q = synth.quant_int8_rows if fmt == "w8a8" else synth.quant_fp8_blocks
    n = {}
    for name, t in (("w13", moe.experts.w13_weight), ("w2", moe.experts.w2_weight),
                    ("sh13", moe.shared_expert.gate_up_proj.weight), ("sh2", moe.shared_expert.down_proj.weight)):
        a, b = q(t.cpu())
        n[name], n["s" + name] = a.numpy(), b.numpy()
    fn = omoe.moe_int8 if fmt == "w8a8" else omoe.moe_fp8
    ref = fn(xin, ids, wts, n["w13"], n["sw13"], n["w2"], n["sw2"], n["sh13"], n["ssh13"], n["sh2"], n["ssh2"],
             bf16_to_np(moe.shared_expert_gate.weight.reshape(-1)), (pos != 0).cpu().numpy())
    ok, err, nbad = close_bf16(bf16_to_np(out), ref)
    assert ok, (err, nbad)
    assert qlayer.prepare(stock) is prepared              # a second prepare reuses the private copy


@pytest.mark.gpu
def test_logits_node_matches_oracle():
    from oracle import attn_lmhead as olm
    from bundles_b200 import synth
    from tests.util import bf16_to_np, close_bf16
    dev = torch.device("cuda", 0)
    V, H, T = 128 * 9, 2048, 70                           # more than 64 rows: two GEMM calls
    g = torch.Generator().manual_seed(8)
    w = (torch.randn(V, H, generator=g) * 0.02).to(torch.bfloat16).to(dev)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).to(dev)
    lm_head = type("Head", (), {"weight": w})()
    node = qnode.prepare(FakeLogitsProcessor(V))
    out = qnode.forward(node, None, x, lm_head, None)
    torch.cuda.synchronize()
    codes, scales = synth.quant_fp8_blocks(w.float().cpu())
    ref = olm.lmhead_logits(bf16_to_np(x), codes.numpy(), scales.numpy())
    ok, err, nbad = close_bf16(out.next_token_logits.cpu().numpy(), ref)
    assert ok, (err, nbad)
    got = out.next_token_ids.cpu().numpy()
    want = np.argmax(ref, axis=1)
    for t in np.nonzero(got != want)[0]:
        assert abs(ref[t, got[t]] - ref[t, want[t]]) <= 2e-4 * max(1.0, abs(ref[t, want[t]]))


def ops_status(status):
    from bundles_b200 import ops
    return ops.read_status(status)


def _private_fp8(w):
    from bundles_b200 import prepare
    n = w.shape[0]
    pad = (-n) % 128
    wf = w.float().cpu()
    if pad:
        wf = torch.cat([wf, torch.zeros(pad, wf.shape[1])])
    c, sc = prepare.quant_fp8_blocks(wf)
    return c[:n].numpy(), sc.numpy()


def _moe_ref(moe, h2, K):
    """The oracle's fp8 MoE block on the private-copy arithmetic of `qlayer._quantise`."""
    from oracle import moe as omoe
    from oracle import router as orouter
    from bundles_b200 import prepare
    from tests.util import bf16_to_np
    _, ids, wts = orouter.route(h2, moe.gate.weight.float().cpu().numpy(), K)
    n = {}
    for name, t in (("w13", moe.experts.w13_weight), ("w2", moe.experts.w2_weight),
                    ("sh13", moe.shared_expert.gate_up_proj.weight), ("sh2", moe.shared_expert.down_proj.weight)):
        a, b = prepare.quant_fp8_blocks(t.cpu())
        n[name], n["s" + name] = a.numpy(), b.numpy()
    return omoe.moe_fp8(h2, ids, wts, n["w13"], n["sw13"], n["w2"], n["sw2"], n["sh13"], n["ssh13"], n["sh2"], n["ssh2"],
                        bf16_to_np(moe.shared_expert_gate.weight.reshape(-1)))


@pytest.mark.gpu
def test_recurrent_layer_verify_branch_and_handoff(monkeypatch):
    """A target-verify batch through two prepared layers behind the stock layer loop: in_proj + verify kernel on the
    engine's pool tensors + deferred out_proj / add / norm + MoE, the first layer's combine handing the second layer
    its normed rows; every stage against the oracle on the GPU's own input of that stage.  A decode batch goes to the
    stock recurrent block."""
    from oracle import attn_lmhead as al
    from oracle import gdn as ogdn
    from bundles_b200 import synth
    from tests.util import bf16_to_np, close_bf16
    monkeypatch.setattr(qlayer, "EXPERT_FORMAT", "fp8")
    dev = torch.device("cuda", 0)
    B, K = 3, 10
    T = 4 * B
    cfg = synth.gdn_replay(seed=51, B=B, extra_slots=2)
    backend, pool = fake_gdn_backend(cfg, dev)
    layers = [FakeHybridLayer(i, FakeMoe(64, 2048, 512, K, dev, seed=60 + i), dev, "gdn", cfg) for i in (10, 11)]
    prepared = [qlayer.prepare(l) for l in layers]
    g = torch.Generator().manual_seed(52)
    x = torch.randn(T, 2048, generator=g).to(torch.bfloat16).to(dev)
    res = torch.randn(T, 2048, generator=g).to(torch.bfloat16).to(dev)
    fb = type("FB", (), dict(forward_mode=FakeMode("target_verify"), positions=torch.arange(1, T + 1, device=dev),
                             req_pool_indices=pool["ring_idx"], spec_info=type("S", (), dict(draft_token_num=4))(),
                             attn_backend=backend))()
    before = {k: pool[k].clone() for k in ("conv_state", "checkpoint", "d_ring", "k_ring", "g_ring")}
    L = layers[0]
    tr = prepared[0].state.trace = {}
    out, residual = qlayer.forward(prepared[0], fb.positions, x, fb, res)
    torch.cuda.synchronize()
    f = lambda t: bf16_to_np(t) if t.dtype == torch.bfloat16 else t.cpu().numpy()  # noqa: E731
    # mixer: input norm (stock) -> in_proj -> verify kernel on the pool tensors -> out_proj
    h1_t, r1_t = L.input_layernorm(x, res)
    assert torch.equal(tr["h1"], h1_t)
    r1 = f(r1_t)
    w_in = torch.cat([L.linear_attn.in_proj_qkvz.weight, L.linear_attn.in_proj_ba.weight])
    p = al.dense_fp8(f(tr["h1"]), *_private_fp8(w_in))
    for name, lo, hi in (("mixed", 0, 8192), ("z", 8192, 12288), ("b", 12288, 12320), ("a", 12320, 12352)):
        ok, err, nbad = close_bf16(f(tr[name]), p[:, lo:hi])
        assert ok, ("in_proj " + name, err, nbad)
    ref = ogdn.gdn_verify_replay(f(tr["mixed"]), f(tr["z"]), f(tr["a"]), f(tr["b"]), f(before["conv_state"]),
                                 f(cfg["conv_w"]), f(cfg["a_log"]), f(cfg["dt_bias"]), f(before["checkpoint"]),
                                 f(before["d_ring"]), f(before["k_ring"]), f(before["g_ring"]), f(cfg["state_idx"]),
                                 f(cfg["ring_idx"]), f(cfg["write_pos"]), f(cfg["cache_base"]), f(cfg["norm_w"]), 1e-6)
    ok, err, nbad = close_bf16(f(tr["core"]), ref["out"])
    assert ok, ("verify kernel output", err, nbad)
    ok, err, nbad = close_bf16(f(tr["proj"]), al.dense_fp8(f(tr["core"]), *_private_fp8(L.linear_attn.out_proj.weight)))
    assert ok, ("out_proj", err, nbad)
    h2, r2 = al.add_rmsnorm(f(tr["proj"]), r1, f(L.post_attention_layernorm.weight))
    assert np.array_equal(f(tr["residual_mid"]), r2)
    ok, err, nbad = close_bf16(f(tr["h2"]), h2)
    assert ok, ("post-attention norm", err, nbad)
    assert torch.equal(pool["checkpoint"], before["checkpoint"]), "the checkpoint is read-only"
    assert not torch.equal(pool["conv_state"], before["conv_state"]), "the conv state is rolled in the pool"
    assert L.linear_attn.out_proj.calls == 0, "the stock out_proj must not run for a row batch"
    # MoE on the rows the GPU fed it, and the hand-off: residual <- out + residual, normed rows for layer 11
    ok, err, nbad = close_bf16(f(out), _moe_ref(L.mlp, f(tr["h2"]), K))
    assert ok, ("moe out", err, nbad)
    normed_ref, r_next = al.add_rmsnorm(f(out), r2, f(layers[1].input_layernorm.weight))
    assert np.array_equal(f(residual), r_next)
    ok, err, nbad = close_bf16(f(tr["normed"]), normed_ref)
    assert ok, ("handed-off rows", err, nbad)
    assert 11 in qlayer._handoff
    calls = []
    orig = layers[1].input_layernorm.forward
    layers[1].input_layernorm.forward = lambda *a, **k: (calls.append(1), orig(*a, **k))[1]
    out2, residual2 = qlayer.forward(prepared[1], fb.positions, out, fb, residual)
    torch.cuda.synchronize()
    assert not calls and 11 not in qlayer._handoff, "layer 11 takes the handed-off rows instead of running its input norm"
    assert residual2.data_ptr() == residual.data_ptr()
    assert out2.shape == out.shape and torch.isfinite(out2.float()).all()
    for st in (prepared[0].state, prepared[1].state):
        assert ops_status(st.status) == 0
    from bundles_b200 import evidence
    paths = {k[2] for k in evidence.seen()}
    assert {"gdn_verify", "proj_add_norm", "moe_combine_norm_handoff"} <= paths      # one line per path, not per layer
    # a decode batch runs the stock recurrent block
    fb_dec = type("FB", (), dict(forward_mode=FakeMode("decode"), positions=fb.positions, attn_backend=backend,
                                 req_pool_indices=pool["ring_idx"]))()
    qlayer._handoff.clear()
    qlayer.forward(prepared[0], fb.positions, x, fb_dec, res.clone())
    assert L.linear_attn.stock_calls == 1


@pytest.mark.gpu
def test_attention_layer_verify_branch(monkeypatch):
    """Projection front + verify core over the engine's paged KV pool + deferred o_proj / add / norm, against the
    oracle; an extend batch goes to the stock attention."""
    from oracle import attn_lmhead as al
    from oracle import attn_verify as oav
    from bundles_b200 import synth
    from tests.util import bf16_to_np, close_bf16
    monkeypatch.setattr(qlayer, "EXPERT_FORMAT", "fp8")
    dev = torch.device("cuda", 0)
    B, K, ctx = 2, 10, 300
    T = 4 * B
    av = synth.attn_verify(seed=71, B=B, ctx=ctx)
    backend, pool = fake_attn_backend(av, dev)
    L = FakeHybridLayer(23, FakeMoe(64, 2048, 512, K, dev, seed=72), dev, "attention")
    prepared = qlayer.prepare(L)
    g = torch.Generator().manual_seed(73)
    x = torch.randn(T, 2048, generator=g).to(torch.bfloat16).to(dev)
    res = torch.randn(T, 2048, generator=g).to(torch.bfloat16).to(dev)
    positions = (torch.arange(ctx - 4, ctx)[None, :].repeat(B, 1)).reshape(-1).to(dev)
    fb = type("FB", (), dict(forward_mode=FakeMode("target_verify"), positions=positions,
                             spec_info=type("S", (), dict(draft_token_num=4))(), attn_backend=backend))()
    kc0, vc0 = av["kcache"].numpy().copy(), av["vcache"].numpy().copy()
    tr = prepared.state.trace = {}
    out, residual = qlayer.forward(prepared, positions, x, fb, res.clone())
    torch.cuda.synchronize()
    f = lambda t: bf16_to_np(t) if t.dtype == torch.bfloat16 else t.cpu().numpy()  # noqa: E731
    h1_t, r1_t = L.input_layernorm(x, res)
    assert torch.equal(tr["h1"], h1_t)
    q, gate, k, v = al.attn_front(f(tr["h1"]), *_private_fp8(L.qkv_proj.weight), f(L.q_norm.weight), f(L.k_norm.weight),
                                  positions.cpu().numpy(), L.rotary_emb.cos_sin_cache.cpu().numpy(), 1e-6, True)
    from oracle.numerics import e4m3_decode
    for name, want in (("q", q), ("k", k), ("v", v)):
        ok, err, nbad = close_bf16(e4m3_decode(f(tr[name])), e4m3_decode(want), rtol=7e-2, atol=2e-2)   # one e4m3 step
        assert ok, ("front " + name, err, nbad)
    ok, err, nbad = close_bf16(f(tr["gate"]), gate)
    assert ok, ("front gate", err, nbad)
    core, kc, vc = oav.attn_verify(f(tr["q"]), f(tr["gate"]), f(tr["k"]), f(tr["v"]), kc0, vc0, av["page_table"].numpy(),
                                   av["seqlens"].numpy(), 256 ** -0.5)
    ok, err, nbad = close_bf16(f(tr["core"]), core)
    assert ok, ("verify core", err, nbad)
    assert np.array_equal(pool["kcache"].cpu().numpy(), kc) and np.array_equal(pool["vcache"].cpu().numpy(), vc), "appended rows"
    ok, err, nbad = close_bf16(f(tr["proj"]), al.dense_fp8(f(tr["core"]), *_private_fp8(L.o_proj.weight)))
    assert ok, ("o_proj", err, nbad)
    h2, r2 = al.add_rmsnorm(f(tr["proj"]), f(r1_t), f(L.post_attention_layernorm.weight))
    assert np.array_equal(f(residual), r2)
    assert L.o_proj.calls == 0
    ok, err, nbad = close_bf16(f(out), _moe_ref(L.mlp, f(tr["h2"]), K))
    assert ok, ("moe out", err, nbad)
    fb_ext = type("FB", (), dict(forward_mode=FakeMode("extend"), positions=positions, attn_backend=backend))()
    qlayer.forward(prepared, positions, x, fb_ext, res.clone())
    assert L.stock_attention_calls == 1 and L.o_proj.calls == 1


@pytest.mark.gpu
def test_attention_layer_rejects_a_foreign_kv_layout(monkeypatch):
    from bundles_b200 import synth
    dev = torch.device("cuda", 0)
    av = synth.attn_verify(seed=74, B=1, ctx=200)
    backend, pool = fake_attn_backend(av, dev)
    one_token_pages = torch.zeros(512, 2, 256, dtype=torch.uint8, device=dev)
    backend.full_attn_backend.token_to_kv_pool.get_kv_buffer = lambda layer_id: (one_token_pages, one_token_pages)
    L = FakeHybridLayer(31, FakeMoe(64, 2048, 512, 10, dev, seed=75), dev, "attention")
    prepared = qlayer.prepare(L)
    x = torch.zeros(4, 2048, dtype=torch.bfloat16, device=dev)
    fb = type("FB", (), dict(forward_mode=FakeMode("target_verify"), positions=torch.arange(196, 200, device=dev),
                             spec_info=type("S", (), dict(draft_token_num=4))(), attn_backend=backend))()
    with pytest.raises(qlayer.UnsupportedLayer, match="128-token pages"):
        qlayer.forward(prepared, fb.positions, x, fb, x.clone())


@pytest.mark.gpu
def test_moe_block_memory_stays_flat_over_many_batch_sizes():
    """Prefill batches of many different lengths and one above the chunk size: buffer sets and graphs are bounded."""
    from bundles_b200 import moe_block, ops, synth
    dev = torch.device("cuda", 0)
    cfg = synth.moe_w8a8(seed=81, T=8, E=64, zipf_s=0.0, device=dev)
    w = ops.MoeW8A8Weights(cfg["w13"], cfg["s13"], cfg["w2"], cfg["s2"], cfg["sh13"], cfg["shs13"], cfg["sh2"], cfg["shs2"])
    block = moe_block.MoeBlockW8A8(cfg["wr"], w, cfg["gate_w"], 10)
    g = torch.Generator(device=dev).manual_seed(82)
    big = torch.randn(5000, 2048, generator=g, device=dev).to(torch.bfloat16)
    out = block(big)                                   # 5000 rows: three chunks, no routing-list overflow
    assert out.shape == big.shape
    ref = torch.cat([block(big[:2048]).clone(), block(big[2048:4096]).clone(), block(big[4096:]).clone()])
    assert torch.equal(out, ref)
    torch.cuda.synchronize()
    base = None
    for i, T in enumerate(range(300, 350)):            # 50 distinct lengths
        block(big[:T])
        if i == 9:
            torch.cuda.synchronize()
            base = torch.cuda.memory_allocated(dev)
    torch.cuda.synchronize()
    assert len(block._ws) <= block.MAX_CACHED and len(block._graphs) <= block.MAX_CACHED
    assert torch.cuda.memory_allocated(dev) <= base * 1.05 + (8 << 20)


@pytest.mark.gpu
def test_moe_block_through_the_op_registry_equals_the_python_operators():
    """router -> build_lists -> moe_fp8 -> moe_combine composed through torch.ops.b200nodes give the bits of the
    same chain through bundles_b200.ops."""
    import bundles_b200.torch_ops  # noqa: F401
    from bundles_b200 import ops, synth
    dev = torch.device("cuda", 0)
    cfg = synth.moe_fp8(seed=91, T=20, E=64)
    d = {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in cfg.items()}
    K = 10
    t = torch.ops.b200nodes
    ids, wts = t.router(d["x"], d["wr"], None, K, False)
    li, lf = t.build_lists(ids, wts, None, 0, 64, 32, True)
    cache = t.moe_fp8(d["x"], d["w13"], d["s13"], d["w2"], d["s2"], d["sh13"], d["shs13"], d["sh2"], d["shs2"], li, lf, K, 32)
    out = t.moe_combine(cache, d["x"], d["gate_w"], K, None)
    _, ids2, wts2 = ops.router(d["x"], d["wr"], K, want_logits=False)
    lists = ops.RoutingLists(20, K, 64, 32, dev)
    ops.build_lists(ids2, wts2, lists)
    w = ops.MoeW8A8Weights(d["w13"], d["s13"], d["w2"], d["s2"], d["sh13"], d["shs13"], d["sh2"], d["shs2"])
    want = ops.moe_combine(ops.moe_fp8(d["x"], w, lists), d["x"], d["gate_w"], K)
    torch.cuda.synchronize()
    assert torch.equal(ids, ids2) and torch.equal(out, want)
    y = t.dense_fp8(d["x"], d["sh13"], d["shs13"])
    assert torch.equal(y, ops.dense_fp8(d["x"], d["sh13"], d["shs13"]))


def test_torch_ops_are_registered_for_cuda_only():
    # hosts that dispatch by op name find every operator of the path under torch.ops.b200nodes; there is no CPU kernel
    import bundles_b200.torch_ops  # noqa: F401
    names = ["router", "gdn_verify", "gdn_verify_replay", "attn_front", "attn_verify", "lmhead_argmax", "moe_combine",
             "moe_combine_norm", "build_lists", "moe_w8a8", "moe_fp8", "dense_fp8", "add_rmsnorm", "argmax_merge",
             "gdn_ring_fold"]
    for n in names:
        assert hasattr(torch.ops.b200nodes, n), n
    x = torch.zeros(4, 2048, dtype=torch.bfloat16)
    with pytest.raises((NotImplementedError, RuntimeError)):
        torch.ops.b200nodes.router(x, torch.zeros(64, 2048), None, 10, False)
