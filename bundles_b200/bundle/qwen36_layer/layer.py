"""`model.layers.*` op: prepare(module) / forward(prepared, *args, **kwargs).

Same contract as the reference's qwen36_layer/layer.py (prepare :486-531, forward :762-764):
`prepare` makes a shallow replica of the stock decoder layer, reads the stock weights WITHOUT
modifying them (layer.py:16-17), builds private quantised copies and routes the replica's
per-token (decode / target-verify) work through the B200 kernels; `forward` calls the stock
layer's own forward on the replica and returns exactly what it returns
(`(hidden_states, residual)`).  Unsupported configurations raise at `prepare` or on the first
call, as the reference's do (layer.py:394-415, gdn_fused.py:19-34, attn_fused.py:48-60); there is
no fallback path for the work this module takes over, and everything it does not take over
(prefill / extend batches of the mixers, idle batches) goes to the stock methods untouched.

What is installed on the replica (reference lines in brackets):
  * sparse-MoE block -> router, routing lists, expert GEMMs, combine              [layer.py:387-483]
  * out_proj / o_proj of a row batch is deferred into `prepare_mlp`, which runs the fp8 projection
    and the fused residual add + Gemma norm                                        [layer.py:192-265, proj.py:84-112]
  * Gated DeltaNet block, target-verify branch: one fp8 in_proj whose outputs land split
    (q k v | z | b | a), then the verify kernel on the engine's own pool tensors   [layer.py:294-371, gdn_fused.py:37-57]
  * gated attention, target-verify branch: fused projection front (q/k norm + RoPE, e4m3 q k v)
    and the verify core over the paged e4m3 KV cache                               [attn_fused.py:110-124,213-275]
  * the combine of layer i writes layer i + 1's residual and normed input rows; layer i + 1's
    `prepare_attn` takes them instead of running its input norm                    [layer.py:534-566, qk_route.cu:779-819]

Host objects read (the reference reads the same ones, layer.py:125,199-209,246-292,392-415,495-500;
gdn_fused.py:42-57; attn_fused.py:63-69,115-124):
  module.layer_id, module.mlp.{gate.weight, topk.topk_config, experts.{w13_weight, w2_weight},
  shared_expert.{gate_up_proj, down_proj}.weight, shared_expert_gate.weight, tp_size},
  module.{input_layernorm, post_attention_layernorm}.{weight, variance_epsilon},
  module.layer_communicator.{prepare_attn, prepare_mlp},
  module.linear_attn.{in_proj_qkvz, in_proj_ba, out_proj}.weight, .attn.{conv_weights, A_log, dt_bias, bias,
  activation, head_k_dim, layer_id}, .norm.{weight, eps, norm_before_gate, activation}  (recurrent layers),
  module.{qkv_proj, o_proj}.weight, .{q_norm, k_norm}.{weight, variance_epsilon}, .rotary_emb.{cos_sin_cache,
  rotary_dim}, .attn.{layer_id, scaling}, .num_heads, .num_kv_heads, .head_dim  (attention layers),
  forward_batch.{forward_mode, positions, req_pool_indices, spec_info.draft_token_num, attn_backend}.
The attention backends come from `forward_batch.attn_backend` when the batch carries them, else from the
engine's forward context (as gdn_fused.py:12,42 does).
"""
from __future__ import annotations

import copy

import torch

from bundles_b200 import moe_block, ops
from bundles_b200 import prepare as prepare_q
from bundles_b200.evidence import note

EXPERT_FORMAT = "w8a8"      # "w8a8": int8 per-output-channel; "fp8": e4m3 with 128 x 128 block scales
HIDDEN, PROJ_IN = 2048, 4096
GDN_SPLIT = (8192, 4096, 32, 32)            # q k v | z | b | a (dense8.py:64-68)
HEADS, KV_HEADS, HEAD_DIM, ROTARY, DRAFT, RING = 16, 2, 256, 64, 4, 16
MAX_ROWS = 1024             # rows of a decode / verify batch served here; larger batches go to the stock path
_prepared = {}              # id(module) -> prepared callable, so that a second prepare reuses the private copies
_by_id = {}                 # layer_id -> replica (for the combine -> next input norm hand-off)
_handoff = {}               # layer_id -> dict(out, residual, normed) left by the previous layer's combine


class UnsupportedLayer(RuntimeError):
    pass


def _row_batch(forward_batch):
    """The engine's per-token calls: plain decode and target-verify (layer.py:174-189)."""
    mode = forward_batch.forward_mode
    return mode.is_decode() or mode.is_target_verify()


def _decode_rows(forward_batch, x):
    return (forward_batch is not None and _row_batch(forward_batch) and 0 < x.shape[0] <= MAX_ROWS
            and x.dtype == torch.bfloat16)


def _backends(forward_batch):
    be = getattr(forward_batch, "attn_backend", None)
    if be is None:
        try:
            from sglang.srt.model_executor.forward_context import get_attn_backend
        except ImportError as exc:
            raise UnsupportedLayer("qwen36_layer: the batch carries no attention backends and the engine's forward "
                                   "context is not importable") from exc
        be = get_attn_backend()
    return be


def _fp8_copy(weight):
    """Private e4m3 copy with 128 x 128 block scales of a [N, K] projection weight (rows padded to a block)."""
    n = weight.shape[0]
    pad = (-n) % 128
    w = weight.float()
    if pad:
        w = torch.cat([w, torch.zeros(pad, w.shape[1], device=w.device)])
    codes, scales = prepare_q.quant_fp8_blocks(w)
    return codes[:n].contiguous(), scales.contiguous()


# ---------------------------------------------------------------------------------------------------
# sparse MoE
# ---------------------------------------------------------------------------------------------------
def _check_moe(mlp):
    cfg = mlp.topk.topk_config
    if getattr(mlp, "tp_size", 1) != 1:
        raise UnsupportedLayer("qwen36_layer: the MoE block must not be tensor-parallel (tp_size == 1)")
    if not getattr(cfg, "renormalize", True):
        raise UnsupportedLayer("qwen36_layer: top-k weights must be renormalised")
    if getattr(cfg, "scoring_func", "softmax") != "softmax":
        raise UnsupportedLayer("qwen36_layer: only softmax routing is supported")
    w13, w2 = mlp.experts.w13_weight, mlp.experts.w2_weight
    E, twoI, H = w13.shape
    if w2.shape != (E, H, twoI // 2) or mlp.gate.weight.shape != (E, H):
        raise UnsupportedLayer(f"qwen36_layer: unexpected expert shapes {tuple(w13.shape)} / {tuple(w2.shape)}")
    if H % 256 or (twoI // 2) % 128 or E % 64 or E > 1024:
        raise UnsupportedLayer(f"qwen36_layer: need H a multiple of 256, I of 128 and E of 64 (H={H} I={twoI // 2} E={E})")
    if cfg.top_k > 32 or cfg.top_k > E:
        raise UnsupportedLayer(f"qwen36_layer: top_k {cfg.top_k} is not supported")
    return E, twoI // 2, H, cfg.top_k


def _quantise(mlp, fmt):
    """Private quantised copy of the experts (the stock bf16 weights stay untouched)."""
    q = prepare_q.quant_int8_rows if fmt == "w8a8" else prepare_q.quant_fp8_blocks
    E = mlp.experts.w13_weight.shape[0]
    parts13, parts2 = [], []
    for e0 in range(0, E, 32):          # in slices: the fp32 staging copy stays small
        parts13.append(q(mlp.experts.w13_weight[e0:e0 + 32]))
        parts2.append(q(mlp.experts.w2_weight[e0:e0 + 32]))
    w13 = torch.cat([p[0] for p in parts13])
    s13 = torch.cat([p[1] for p in parts13])
    w2 = torch.cat([p[0] for p in parts2])
    s2 = torch.cat([p[1] for p in parts2])
    sh13 = shs13 = sh2 = shs2 = None
    if getattr(mlp, "shared_expert", None) is not None:
        sh13, shs13 = q(mlp.shared_expert.gate_up_proj.weight)
        sh2, shs2 = q(mlp.shared_expert.down_proj.weight)
    return ops.MoeW8A8Weights(w13.contiguous(), s13.contiguous(), w2.contiguous(), s2.contiguous(), sh13, shs13, sh2,
                              shs2)


class _MoeOverride(torch.nn.Module):
    """Drop-in for the stock sparse-MoE block's forward(hidden_states, forward_batch=None, ...)."""

    def __init__(self, mlp, fmt, owner=None):
        super().__init__()
        E, I, H, K = _check_moe(mlp)
        if not mlp.gate.weight.is_cuda:
            raise UnsupportedLayer("qwen36_layer: weights must live on a CUDA device (there is no CPU path)")
        weights = _quantise(mlp, fmt)
        gate_w = None
        if getattr(mlp, "shared_expert_gate", None) is not None:
            gate_w = mlp.shared_expert_gate.weight.reshape(-1).to(torch.bfloat16).contiguous()
        bias = getattr(mlp.topk.topk_config, "correction_bias", None)
        wr = mlp.gate.weight.float().contiguous()          # the router runs on an fp32 copy of the gate weight
        cls = moe_block.MoeBlockW8A8 if fmt == "w8a8" else moe_block.MoeBlockFp8
        self.block = cls(wr, weights, gate_w, K, bias=None if bias is None else bias.float())
        self.hidden, self.top_k, self.gate_w = H, K, gate_w
        self.owner = owner          # the layer's hand-off state (residual seen by prepare_mlp, next layer's norm)

    def forward(self, hidden_states, forward_batch=None, *args, **kwargs):
        shape = hidden_states.shape
        x = hidden_states.reshape(-1, self.hidden)
        pos = getattr(forward_batch, "positions", None) if forward_batch is not None else None
        if pos is not None and pos.dtype != torch.int64:
            pos = pos.to(torch.int64)
        nxt = self.owner.next_norm(forward_batch, x) if self.owner is not None else None
        if nxt is not None:
            # the combine also writes the next layer's residual and normed rows (qk_route.cu:779-819); that layer's
            # prepare_attn picks them up instead of running its input norm (layer.py:555-566)
            residual, norm_w, eps, key = nxt
            note("moe_combine_norm_handoff", x.shape[0])
            out, normed = self.block.forward_combine_norm(x, pos, residual, norm_w, eps)
            _handoff[key] = dict(out=out, residual=residual, normed=normed)
            if self.owner.trace is not None:
                self.owner.trace.update(normed=normed.clone())
            return out.reshape(shape)
        # rows whose position is 0 are graph padding and come back as zeros (layer.py:476-477)
        note("moe_block", x.shape[0])
        return self.block(x, pos).reshape(shape).clone()


# ---------------------------------------------------------------------------------------------------
# deferred output projection + residual add + norm, and the input-norm hand-off
# ---------------------------------------------------------------------------------------------------
class _Deferred:
    """Projection input held until the layer's post-attention norm consumes it (layer.py:167-171)."""

    def __init__(self, x):
        self.x = x


class _LayerState:
    """Per-layer glue state shared by the installed pieces."""

    def __init__(self, layer, replica):
        self.layer, self.replica = layer, replica
        self.layer_id = int(getattr(layer, "layer_id", -1))
        self.batch = None           # the forward batch of the call in flight (set by prepare_attn)
        self.residual = None        # the residual prepare_mlp produced, for the combine's hand-off
        self.status = ops.new_status(layer.post_attention_layernorm.weight.device)
        self.trace = None           # set to a dict to keep copies of the stage outputs (tests)

    def next_norm(self, forward_batch, x):
        """(residual, weight, eps, key) of the next layer's input norm if that layer takes the hand-off."""
        nxt = _by_id.get(self.layer_id + 1)
        if (nxt is None or self.residual is None or forward_batch is None or not _decode_rows(forward_batch, x)
                or self.residual.shape != x.shape or not getattr(nxt, "_b200_takes_handoff", False)):
            return None
        norm = nxt.input_layernorm
        return self.residual, norm.weight, norm.variance_epsilon, self.layer_id + 1


def _install_projection(layer, replica, state, owner, owner_name, projection, proj_name):
    """Defer the row-batch output projection into the fused add-and-norm (layer.py:192-265)."""
    norm = layer.post_attention_layernorm
    if (tuple(projection.weight.shape) != (HIDDEN, PROJ_IN) or projection.weight.dtype != torch.bfloat16
            or getattr(projection, "bias", None) is not None or tuple(norm.weight.shape) != (HIDDEN,)):
        raise UnsupportedLayer(f"qwen36_layer: {proj_name} or its norm is not the BF16 [2048, 4096] / [2048] shape: "
                               f"{tuple(projection.weight.shape)} {projection.weight.dtype} norm {tuple(norm.weight.shape)}")
    codes, scales = _fp8_copy(projection.weight)
    norm_w, eps = norm.weight, norm.variance_epsilon

    def project(x, *args, **kwargs):
        if (not args and not kwargs and x.ndim == 2 and x.shape[1] == PROJ_IN and x.is_contiguous()
                and _decode_rows(state.batch, x)):
            return _Deferred(x), None
        return projection.forward(x, *args, **kwargs)

    private = copy.copy(projection)
    private.forward = project
    if owner_name is None:
        replica._modules[proj_name] = private
        owner_replica = replica
    else:
        owner_replica = copy.copy(owner)
        owner_replica._modules = dict(owner._modules)
        owner_replica._modules[proj_name] = private
        replica._modules[owner_name] = owner_replica
    communicator = copy.copy(layer.layer_communicator)
    stock_prepare_mlp = type(communicator).prepare_mlp
    stock_prepare_attn = type(communicator).prepare_attn

    def prepare_mlp(hidden_states, residual, forward_batch, *args, **kwargs):
        if isinstance(hidden_states, _Deferred):
            x = hidden_states.x
            if (residual is None or residual.shape != (x.shape[0], HIDDEN) or residual.dtype != torch.bfloat16
                    or not residual.is_contiguous()):
                hidden_states, _ = projection.forward(x)
                return stock_prepare_mlp(communicator, hidden_states, residual, forward_batch, *args, **kwargs)
            note("proj_add_norm", x.shape[0])
            proj = torch.empty_like(residual) if state.trace is not None else None
            # split-K fp8 projection, then one kernel: residual <- proj + residual (in place) and the norm
            out = ops.dense_fp8_add_rmsnorm(x, codes, scales, residual, norm_w, eps, proj_out=proj, status=state.status)
            state.residual = residual
            if state.trace is not None:
                state.trace.update(core=x.clone(), proj=proj, h2=out.clone(), residual_mid=residual.clone())
            return out, residual
        state.residual = None
        return stock_prepare_mlp(communicator, hidden_states, residual, forward_batch, *args, **kwargs)

    def prepare_attn(hidden_states, residual, forward_batch, *args, **kwargs):
        state.batch = forward_batch
        state.residual = None
        pending = _handoff.pop(state.layer_id, None)
        if pending is not None:
            if (pending["out"].data_ptr() == hidden_states.data_ptr() and residual is not None
                    and pending["residual"].data_ptr() == residual.data_ptr()):
                return pending["normed"].reshape(hidden_states.shape), residual
            raise RuntimeError(f"qwen36_layer: layer {state.layer_id} was handed rows normed by the previous layer's combine "
                               "but was called with other tensors; the residual already holds the sum")
        return stock_prepare_attn(communicator, hidden_states, residual, forward_batch, *args, **kwargs)

    communicator.prepare_mlp = prepare_mlp
    communicator.prepare_attn = prepare_attn
    replica.layer_communicator = communicator       # a plain attribute, not a registered submodule
    replica._b200_takes_handoff = True
    return owner_replica


# ---------------------------------------------------------------------------------------------------
# Gated DeltaNet block: target-verify branch
# ---------------------------------------------------------------------------------------------------
def _require_gdn_layout(lin, attn, norm, params, pool, draft):
    """The layout the verify kernel serves (gdn_fused.py:19-34)."""
    if (getattr(params, "replayssm_d", None) is None or getattr(pool, "replayssm_cache_base", None) is None
            or params.replayssm_rawv is None or params.replayssm_rawk is None or params.replayssm_d.shape[-2] != RING):
        raise UnsupportedLayer("qwen36_layer: the verify kernel serves the 16-entry circular (d, k, g) ring only")
    if draft != DRAFT:
        raise UnsupportedLayer(f"qwen36_layer: the verify kernel serves {DRAFT}-token drafts, not {draft}")
    if getattr(attn, "bias", None) is not None or getattr(attn, "activation", "silu") not in ("silu", "swish"):
        raise UnsupportedLayer("qwen36_layer: the verify kernel serves a bias-free SiLU conv only")
    if (getattr(norm, "norm_before_gate", True) is not True or getattr(norm, "activation", "silu") not in ("silu", "swish")
            or getattr(norm, "bias", None) is not None or tuple(norm.weight.shape) != (128,)):
        raise UnsupportedLayer("qwen36_layer: the verify kernel serves the swish-gated RMSNorm over 128 channels only")


def _install_gdn(gdn, gdn_replica, state):
    """in_proj + verify kernel for a target-verify batch; every other mode runs the stock block (layer.py:294-371)."""
    w_qkvz, w_ba = gdn.in_proj_qkvz.weight, gdn.in_proj_ba.weight
    if (tuple(w_qkvz.shape) != (GDN_SPLIT[0] + GDN_SPLIT[1], HIDDEN) or tuple(w_ba.shape) != (64, HIDDEN)
            or getattr(gdn.in_proj_qkvz, "bias", None) is not None or getattr(gdn.in_proj_ba, "bias", None) is not None):
        raise UnsupportedLayer("qwen36_layer: the recurrent block is not the [12288 | 64, 2048] in_proj shape")
    codes, scales = _fp8_copy(torch.cat([w_qkvz, w_ba]))       # one GEMM: [q k v | z | b | a] = 12352 rows
    stock_forward = type(gdn).forward
    checked = [False]
    bufs = {}

    def forward(hidden_states, forward_batch, *args, **kwargs):
        mode = forward_batch.forward_mode
        x = hidden_states
        if (not isinstance(x, torch.Tensor) or not mode.is_target_verify() or x.shape[0] == 0 or x.shape[0] > MAX_ROWS
                or x.shape[0] % DRAFT or x.dtype != torch.bfloat16 or not x.is_contiguous()):
            return stock_forward(gdn_replica, hidden_states, forward_batch, *args, **kwargs)
        lin = _backends(forward_batch).linear_attn_backend
        fm = lin.forward_metadata
        attn, norm = gdn_replica.attn, gdn_replica.norm
        params = lin.req_to_token_pool.mamba2_layer_cache(attn.layer_id)
        pool = lin.req_to_token_pool.mamba_pool
        if not checked[0]:
            _require_gdn_layout(lin, attn, norm, params, pool, forward_batch.spec_info.draft_token_num)
            checked[0] = True
        T = x.shape[0]
        note("gdn_verify", T)
        outs = bufs.get(T)
        if outs is None:
            outs = bufs[T] = [torch.empty(T, wd, dtype=torch.bfloat16, device=x.device) for wd in GDN_SPLIT]
        mixed, z, b, a = ops.dense_fp8_split(x, codes, scales, GDN_SPLIT, outs=outs, status=state.status)
        if state.trace is not None:
            state.trace.update(h1=x.clone(), mixed=mixed.clone(), z=z.clone(), b=b.clone(), a=a.clone())
        i32 = lambda t: t if t.dtype == torch.int32 else t.to(torch.int32)  # noqa: E731
        core = ops.gdn_verify_replay(
            mixed, z, a, b, params.conv[0], attn.conv_weights, params.intermediate_conv_window[0].view(-1, 8192, 6),
            attn.A_log, attn.dt_bias, params.temporal, params.replayssm_d, params.replayssm_rawv, params.replayssm_k,
            params.replayssm_rawk, params.replayssm_g, i32(fm.mamba_cache_indices), i32(forward_batch.req_pool_indices),
            i32(lin.verify_intermediate_state_indices), pool.replayssm_spec_write_pos, pool.replayssm_cache_base,
            norm.weight, norm.eps, status=state.status)
        output, _ = gdn_replica.out_proj(core)      # deferred into prepare_mlp for a row batch
        return output

    gdn_replica.forward = forward


# ---------------------------------------------------------------------------------------------------
# gated attention: target-verify branch
# ---------------------------------------------------------------------------------------------------
def _require_attn_layout(layer, backend, k_cache, v_cache):
    """The layout the fused attention serves (attn_fused.py:48-60), with this library's page layout."""
    if (layer.num_heads != HEADS or layer.num_kv_heads != KV_HEADS or layer.head_dim != HEAD_DIM
            or layer.rotary_emb.rotary_dim != ROTARY or not getattr(layer, "attn_output_gate", True)):
        raise UnsupportedLayer("qwen36_layer: the fused attention serves 16 x 256 query heads over 2 KV heads with a gate")
    if layer.q_norm.variance_epsilon != layer.k_norm.variance_epsilon:
        raise UnsupportedLayer("qwen36_layer: the fused attention assumes one q/k norm epsilon")
    if getattr(layer.attn, "k_scale", None) is not None or getattr(layer.attn, "v_scale", None) is not None:
        raise UnsupportedLayer("qwen36_layer: the fused attention serves an unscaled E4M3 KV cache only")
    ok = (k_cache.dim() == 4 and v_cache.dim() == 4 and tuple(k_cache.shape[1:]) == (KV_HEADS, 128, HEAD_DIM)
          and tuple(v_cache.shape[1:]) == (KV_HEADS, HEAD_DIM, 128) and k_cache.element_size() == 1
          and getattr(backend, "page_size", 128) == 128)
    if not ok:
        raise UnsupportedLayer("qwen36_layer: the verify attention reads a paged E4M3 KV pool of 128-token pages, K "
                               "[pages, 2, 128, 256] and V [pages, 2, 256, 128] (dim-major); the engine's pool is "
                               f"{tuple(k_cache.shape)} / {tuple(v_cache.shape)}")


def _install_attention(module, replica, state):
    """Projection front + verify core for a target-verify batch (attn_fused.py:213-275); other modes run stock."""
    w = module.qkv_proj.weight
    if tuple(w.shape) != (9216, HIDDEN) or w.dtype != torch.bfloat16 or getattr(module.qkv_proj, "bias", None) is not None:
        raise UnsupportedLayer("qwen36_layer: qkv_proj is not the BF16 [9216, 2048] weight")
    codes, scales = _fp8_copy(w)
    stock = type(module).self_attention
    checked = [False]
    cos_sin = [None]

    def self_attention(positions, hidden_states, forward_batch, *args, **kwargs):
        x = hidden_states
        if (not forward_batch.forward_mode.is_target_verify() or x.shape[0] == 0 or x.shape[0] > MAX_ROWS
                or x.shape[0] % DRAFT or x.dtype != torch.bfloat16 or not x.is_contiguous()):
            return stock(replica, positions, hidden_states, forward_batch, *args, **kwargs)
        backend = _backends(forward_batch).full_attn_backend
        k_cache, v_cache = backend.token_to_kv_pool.get_kv_buffer(module.attn.layer_id)
        if not checked[0]:
            _require_attn_layout(module, backend, k_cache, v_cache)
            if forward_batch.spec_info.draft_token_num != DRAFT:
                raise UnsupportedLayer(f"qwen36_layer: the fused verify attention serves {DRAFT}-token drafts")
            cs = module.rotary_emb.cos_sin_cache
            cos_sin[0] = cs.float().contiguous()           # [max_pos, 64] = [cos 32 | sin 32]
            checked[0] = True
        md = backend.forward_metadata
        note("attn_verify", x.shape[0])
        pos = positions if positions.dtype == torch.int64 else positions.to(torch.int64)
        q, gate, k, v = ops.attn_front(x, codes, scales, module.q_norm.weight, module.k_norm.weight, pos.contiguous(),
                                       cos_sin[0], module.q_norm.variance_epsilon, True, status=state.status)
        as_u8 = lambda t: t if t.dtype == torch.uint8 else t.view(torch.uint8)  # noqa: E731
        if state.trace is not None:
            state.trace.update(h1=x.clone(), q=q.clone(), gate=gate.clone(), k=k.clone(), v=v.clone())
        core = ops.attn_verify(q, gate, k, v, as_u8(k_cache), as_u8(v_cache), md.page_table, md.cache_seqlens_int32,
                               scale=float(module.attn.scaling), status=state.status)
        output, _ = replica.o_proj(core)            # deferred into prepare_mlp for a row batch
        return output

    replica.self_attention = self_attention


# ---------------------------------------------------------------------------------------------------
def prepare(module):
    """Once per decoder layer (reference: layer.py:486-531).  Returns the callable the engine stores."""
    key = id(module)
    if key in _prepared:
        return _prepared[key]
    if not hasattr(module, "mlp") or not hasattr(module.mlp, "experts"):
        raise UnsupportedLayer("qwen36_layer: the layer has no sparse-MoE block (`mlp.experts`)")
    replica = copy.copy(module)                        # shallow: shares the stock weights, read-only
    replica._modules = dict(module._modules)
    state = None
    full = hasattr(module, "layer_communicator") and hasattr(module, "post_attention_layernorm")
    if full:        # the whole layer: mixers, deferred projection, hand-off
        state = _LayerState(module, replica)
        if hasattr(module, "linear_attn"):
            gdn = module.linear_attn
            gdn_replica = _install_projection(module, replica, state, gdn, "linear_attn", gdn.out_proj, "out_proj")
            _install_gdn(gdn, gdn_replica, state)
        elif hasattr(module, "qkv_proj") and hasattr(module, "o_proj"):
            _install_projection(module, replica, state, module, None, module.o_proj, "o_proj")
            _install_attention(module, replica, state)
        else:
            raise UnsupportedLayer("qwen36_layer: the layer has neither a recurrent block nor attention projections")
        if state.layer_id >= 0:
            _by_id[state.layer_id] = replica
    replica._modules["mlp"] = _MoeOverride(module.mlp, EXPERT_FORMAT, state)

    def layer(*args, **kwargs):
        return type(module).forward(replica, *args, **kwargs)

    layer.replica = replica
    layer.state = state
    _prepared[key] = layer
    return layer


def forward(prepared, *args, **kwargs):
    return prepared(*args, **kwargs)
