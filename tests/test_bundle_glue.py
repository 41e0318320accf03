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

from tests.fake_engine import FakeDecoderLayer, FakeLogitsProcessor, FakeMoe   # noqa: E402


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
    with pytest.raises(qlayer.UnsupportedLayer, match="multiples of 128"):
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


def test_torch_ops_are_registered_for_cuda_only():
    # hosts that dispatch by op name find every operator of the path under torch.ops.b200nodes; there is no CPU kernel
    import bundles_b200.torch_ops  # noqa: F401
    names = ["router", "gdn_verify", "gdn_verify_replay", "attn_front", "attn_verify", "lmhead_argmax", "moe_combine"]
    for n in names:
        assert hasattr(torch.ops.b200nodes, n), n
    x = torch.zeros(4, 2048, dtype=torch.bfloat16)
    with pytest.raises((NotImplementedError, RuntimeError)):
        torch.ops.b200nodes.router(x, torch.zeros(64, 2048), None, 10, False)
