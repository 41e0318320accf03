"""One decode / speculative-verify step through a whole stack of layers, built from the operators of this package.

The host-side loop a serving engine runs per step for the Qwen3.6-35B-A3B layout of the reference bundle
(`layer.py:486-531`: every layer = token mixer + sparse MoE; full attention every fourth layer, Gated DeltaNet
otherwise; `node.py:136-151`: LM head at the end), at the target formats: fp8 block-scaled projections and
experts, e4m3 KV pages, explicit fp32 GDN state, greedy token from the fused LM-head argmax.  Weights are
random-initialised on the device from a seed (there are no checkpoints here); every layer owns its own weights,
state and KV pages, so a step streams what a real model would stream.

Per layer, for this rank's rows (4 drafts x its sequences):
    GDN layer:        in_proj (dense fp8, outputs split into q k v | z | b | a) -> gdn_verify;
                      with `gdn_layout="ring"` the state is the engine's read-only checkpoint + 16-entry (d, k, g)
                      ring and the step appends to the ring
    attention layer:  attn_front (projection + q/k norm + RoPE, e4m3 q/k/v) -> attn_verify
    then              out_proj / o_proj (split-K fp8) fused with the residual add + RMSNorm -> router -> lists -> fp8 experts -> combine fused with the next
                      layer's residual add + input RMSNorm
and after the last layer the vocabulary argmax.

On several GPUs (`ep` = an expert-parallel group) the sequences are split over the ranks (state and KV pages never
move), the routed experts are split over the ranks (expert e lives on rank e // (E / world)) and so is the
vocabulary (128-row scale-block boundaries).  Per layer every rank routes its own rows, stores them and their
routing into every rank's gathered buffers (peer stores), barrier, builds the lists of ITS experts over the
gathered rows and runs them; the down GEMM's epilogue stores each weighted row straight into its home rank's cache
(peer stores), barrier, and the home rank combines.  The shared expert runs on the home rank.  For the LM head the
final hidden rows are gathered the same way, every rank takes (max, argmax) over its vocabulary shard, the pairs are
gathered and merged.  No NCCL call, no TMA on peer memory and no multicast in the step.  All of it yields the same
bits as the single-GPU step: every row's arithmetic is independent of which other rows share its GEMM tile.
"""
from __future__ import annotations

import os

import math
import zlib

import torch

from . import ops
from .parallel import run_lockstep, vocab_shards
from .prepare import quant_fp8_blocks

H, I, E, K = 2048, 512, 512, 10
GDN_SPLIT = (8192, 4096, 32, 32)    # q | k | v, z, b, a   (dense8.py:64-68)
GDN_PROJ = sum(GDN_SPLIT)


class DecodeStep:
    """`layers` layers (layer i is full attention iff i % 4 == 3), `B` sequences with `ctx` tokens of context each.
    `ep`: None (one GPU), a `parallel.EpGroup` (one process per GPU) or a view of a `parallel.VirtualEpGroup`; the
    rank then owns sequences [rank * B / world, ...), experts [rank * E / world, ...) and one vocabulary shard.
    Every rank draws the same model from `seed` and keeps its part.  `gate`: an optional `parallel.StepGate`."""

    def __init__(self, layers=48, B=8, ctx=8192, vocab=151936, experts=E, seed=1005, device="cuda", gdn_layout="explicit",
                 ring_fill=0, ep=None, gate=None, attn_splits=None):
        if gdn_layout not in ("explicit", "ring"):
            raise ValueError("gdn_layout is 'explicit' or 'ring'")
        self.gdn_layout = gdn_layout
        self.ep = ep
        self.gate = gate        # optional parallel.StepGate: host-side roll call of the ranks before every step
        # CTAs per (request, kv head) of the attention core; None lets the kernel fill the GPU for this rank's
        # batch.  The split count sets the order in which partial sums are merged, so two forms of the step give
        # the same bits only with the same count.
        self.attn_splits = attn_splits
        self.world = 1 if ep is None else ep.world
        self.rank = 0 if ep is None else ep.rank
        if B % self.world or experts % self.world:
            raise ValueError(f"{B} sequences / {experts} experts do not split evenly over {self.world} ranks")
        dev = torch.device(device)
        self.dev, self.seed = dev, seed
        bf = torch.bfloat16
        W, R = self.world, self.rank
        self.B_all, self.B = B, B // W
        self.T, self.T_all = 4 * self.B, 4 * B
        self.ctx, self.n_layers, self.E, self.vocab = ctx, layers, experts, vocab
        self.E_local, self.e_lo = experts // W, R * (experts // W)
        b0, b1 = R * self.B, (R + 1) * self.B
        self.status = ops.new_status(dev)
        Bl = self.B
        self.layers = []
        per = (ctx + 127) // 128
        for i in range(layers):
            L = dict(attn=(i % 4 == 3))
            rn = lambda tag, *s, std=1.0, i=i: torch.randn(*s, generator=self._gen(i, tag), device=dev) * std  # noqa: E731
            if L["attn"]:
                L["qkv_w"], L["qkv_s"] = self._fp8_matrix((i, "qkv"), 9216, H)
                L["q_norm"], L["k_norm"] = rn("qn", 256, std=0.1).to(bf), rn("kn", 256, std=0.1).to(bf)
                L["o_w"], L["o_s"] = self._fp8_matrix((i, "o"), H, 4096)
                # every sequence owns `per` pages of a pool with one spare page; the page ids are a seeded permutation
                # (this rank's part of it renumbered into a pool of its own), the contents are drawn per sequence,
                # so a sequence has the same bytes whichever rank holds it
                P_all = B * per + 1
                perm = torch.randperm(P_all, generator=self._gen(i, "pages"), device=dev)[:B * per].reshape(B, per)
                table = perm[b0:b1].reshape(-1).argsort().argsort().reshape(Bl, per)
                P = Bl * per + 1
                kc = torch.zeros(P, 2, 128, 256, dtype=torch.uint8, device=dev)
                vc = torch.zeros(P, 2, 256, 128, dtype=torch.uint8, device=dev)
                for b in range(Bl):
                    gk = self._gen(i, "kv", b0 + b)
                    kc[table[b]] = torch.randn(per, 2, 128, 256, generator=gk, device=dev).to(
                        torch.float8_e4m3fn).view(torch.uint8)
                    vc[table[b]] = torch.randn(per, 2, 256, 128, generator=gk, device=dev).to(
                        torch.float8_e4m3fn).view(torch.uint8)
                L["kcache"], L["vcache"] = kc, vc
                L["page_table"] = table.to(torch.int32).contiguous()
            else:
                L["in_w"], L["in_s"] = self._fp8_matrix((i, "in"), GDN_PROJ, H)
                L["out_w"], L["out_s"] = self._fp8_matrix((i, "out"), H, 4096)
                L["conv_state"] = rn("conv_state", B, 8192, 3)[b0:b1].to(bf).contiguous()
                L["conv_w"] = rn("conv_w", 8192, 4, std=0.5).to(bf)
                L["a_log"] = torch.rand(32, generator=self._gen(i, "a_log"), device=dev) * math.log(16.0)
                L["dt_bias"] = rn("dt_bias", 32)
                st = torch.empty(Bl, 32, 128, 128, device=dev)
                for b in range(Bl):
                    st[b] = torch.randn(32, 128, 128, generator=self._gen(i, "state", b0 + b), device=dev) * 0.1
                L["state"] = st
                L["gdn_norm"] = rn("gdn_norm", 128, std=0.1).to(bf)
                if gdn_layout == "ring":   # pools of B slots, request b in slot b; `ring_fill` committed entries
                    gr = self._gen(i, "ring")
                    L["window"] = torch.zeros(Bl, 8192, 6, dtype=bf, device=dev)
                    L["d_ring"] = (torch.randn(B, 32, 16, 128, generator=gr, device=dev) * 0.3)[b0:b1].to(bf).contiguous()
                    L["dlo_ring"] = torch.zeros(Bl, 32, 16, 128, dtype=bf, device=dev)
                    L["k_ring"] = torch.nn.functional.normalize(torch.randn(B, 16, 16, 128, generator=gr, device=dev),
                                                                dim=-1)[b0:b1].to(bf).contiguous()
                    L["klo_ring"] = torch.zeros(Bl, 16, 16, 128, dtype=bf, device=dev)
                    L["g_ring"] = (-torch.rand(B, 32, 16, generator=gr, device=dev) * 0.5)[b0:b1].contiguous()
            L["post_norm"] = rn("post_norm", H, std=0.1).to(bf)     # norm between the mixer and the MoE
            L["next_norm"] = rn("next_norm", H, std=0.1).to(bf)     # input norm of the next layer (final norm after the last)
            L["wr"] = rn("wr", experts, H, std=0.02)
            L["gate_w"] = rn("gate_w", H, std=0.02).to(bf)
            w13, s13 = self._fp8_experts((i, "w13"), 2 * I, H)
            w2, s2 = self._fp8_experts((i, "w2"), H, I)
            sh13, shs13 = self._fp8_matrix((i, "sh13"), 2 * I, H)
            sh2, shs2 = self._fp8_matrix((i, "sh2"), H, I)
            L["w"] = ops.MoeW8A8Weights(w13, s13, w2, s2, sh13, shs13, sh2, shs2)
            self.layers.append(L)
        # LM head: this rank's vocabulary shard (the whole vocabulary on one GPU)
        self.shard_lo, self.shard_hi = vocab_shards(vocab, W)[R]
        self.lm_w, self.lm_s = self._fp8_rows(("lm",), vocab, H, self.shard_lo, self.shard_hi)
        self.first_norm = (torch.randn(H, generator=self._gen("first_norm"), device=dev) * 0.1).to(bf)
        half = 32
        inv = torch.pow(torch.tensor(1e7, dtype=torch.float64), -2.0 * torch.arange(half, dtype=torch.float64) / 64)
        ang = torch.arange(ctx + 8, dtype=torch.float64)[:, None] * inv[None, :]
        self.cos_sin = torch.cat([ang.cos(), ang.sin()], 1).float().to(dev)
        self.seqlens = torch.full((Bl,), ctx, dtype=torch.int32, device=dev)
        self.positions = (torch.arange(Bl, device=dev)[:, None] * 0 + torch.arange(ctx - 4, ctx, device=dev)[None, :]
                          ).reshape(-1).to(torch.int64).contiguous()
        self.accepted = torch.randint(0, 5, (B,), generator=self._gen("accepted"), device=dev, dtype=torch.int32)[b0:b1].contiguous()
        self.slots = torch.arange(Bl, dtype=torch.int32, device=dev)
        self.write_pos = torch.full((Bl,), int(ring_fill), dtype=torch.int32, device=dev)
        self.cache_base = torch.zeros(Bl, dtype=torch.int32, device=dev)
        # buffers reused by every layer
        T, Ta = self.T, self.T_all
        Tm = Ta if ep is not None else T                      # rows the expert GEMMs of this rank see
        self.lists = ops.RoutingLists(Tm, K, self.E_local, 32, dev)   # the fp8 expert GEMMs take blocks of <= 32 rows
        self.moe_ws = ops.moe_fp8_workspace(Tm, H, I, K, dev)
        self.scratch = ops.router_scratch(T, H, experts, dev)
        self.ids = torch.empty(T, K, dtype=torch.int32, device=dev)
        self.wts = torch.empty(T, K, dtype=torch.float32, device=dev)
        self.gdn_ws = ops.gdn_workspace(Bl, dev)
        self.dense_ws = ops.dense_fp8_workspace(T, 4096, dev)
        self.hq = torch.empty(T, H, dtype=torch.uint8, device=dev)          # a layer's input rows as e4m3 + scales,
        self.hs = torch.empty(T, H // 128, dtype=torch.float32, device=dev)  # left by the previous layer's combine + norm
        self.proj_ws = ops.dense_fp8_add_rmsnorm_workspace(T, 4096, H, dev)
        self.gdn_in = [torch.empty(T, wd, dtype=bf, device=dev) for wd in GDN_SPLIT]
        self.lm_ws = ops.lmhead_workspace(Ta if ep is not None else T, H, self.shard_hi - self.shard_lo, dev)
        if ep is None:
            self.cache = torch.zeros(T * (K + 1), H, dtype=bf, device=dev)
        else:
            self.cache, self.peer_cache = ep.shared((T * (K + 1), H), bf)
            self.x_all, self.peer_x = ep.shared((Ta, H), bf)
            self.ids_all, self.peer_ids = ep.shared((Ta, K), torch.int32)
            self.wts_all, self.peer_wts = ep.shared((Ta, K), torch.float32)
            self.h_all, self.peer_h = ep.shared((Ta, H), bf)
            self.max_all, self.peer_max = ep.shared((W, Ta), torch.float32)
            self.idx_all, self.peer_idx = ep.shared((W, Ta), torch.int32)
        self.launches = 0
        self.trace = None       # set to a list to record per-layer intermediates (tests)

    # ---- seeded model parts -----------------------------------------------------------------------------
    def _gen(self, *tag):
        """A generator whose seed depends on `seed` and the tag only, so that a rank can draw just its own part."""
        g = torch.Generator(device=self.dev)
        g.manual_seed((self.seed * 1000003 + zlib.crc32(repr(tag).encode())) & 0x7fffffffffffffff)
        return g

    def _fp8_matrix(self, tag, rows, cols, std=0.02):
        """Random weight [rows, cols] -> (e4m3 codes, 128 x 128 block scales); a ragged last block row is quantised
        as if padded with zeros."""
        rp = (rows + 127) // 128 * 128
        w = torch.zeros(rp, cols, device=self.dev)
        w[:rows] = torch.randn(rows, cols, generator=self._gen(*tag), device=self.dev) * std
        q, s = quant_fp8_blocks(w)
        return q[:rows].contiguous(), s

    def _fp8_rows(self, tag, rows, cols, lo, hi, std=0.02, chunk=128 * 64):
        """Rows [lo, hi) (lo on a 128-row boundary) of a random [rows, cols] weight drawn in fixed row chunks."""
        n = hi - lo
        q = torch.empty(n, cols, dtype=torch.uint8, device=self.dev)
        s = torch.empty((n + 127) // 128, cols // 128, dtype=torch.float32, device=self.dev)
        for c0 in range(0, rows, chunk):
            c1 = min(rows, c0 + chunk)
            if c1 <= lo or c0 >= hi:
                continue
            cp = (c1 - c0 + 127) // 128 * 128
            w = torch.zeros(cp, cols, device=self.dev)
            w[:c1 - c0] = torch.randn(c1 - c0, cols, generator=self._gen(*tag, c0), device=self.dev) * std
            qc, sc = quant_fp8_blocks(w)
            a, b = max(lo, c0), min(hi, c1)
            q[a - lo:b - lo] = qc[a - c0:b - c0]
            s[(a - lo) // 128:(b - lo + 127) // 128] = sc[(a - c0) // 128:(b - c0 + 127) // 128]
        return q, s

    def _fp8_experts(self, tag, rows, cols, std=0.02):
        """This rank's experts of a random [E, rows, cols] weight, drawn in chunks of E / 8 experts."""
        chunk = max(1, self.E // 8)
        n = self.E_local
        q = torch.empty(n, rows, cols, dtype=torch.uint8, device=self.dev)
        s = torch.empty(n, rows // 128, cols // 128, dtype=torch.float32, device=self.dev)
        for e0 in range(0, self.E, chunk):
            m = min(chunk, self.E - e0)
            if e0 + m <= self.e_lo or e0 >= self.e_lo + n:
                continue
            qc, sc = quant_fp8_blocks(torch.randn(m, rows, cols, generator=self._gen(*tag, e0), device=self.dev) * std)
            a, b = max(self.e_lo, e0), min(self.e_lo + n, e0 + m)
            q[a - self.e_lo:b - self.e_lo] = qc[a - e0:b - e0]
            s[a - self.e_lo:b - self.e_lo] = sc[a - e0:b - e0]
        return q, s

    # ---- the step ----------------------------------------------------------------------------------------------
    def _mixer(self, L, h, hq=None):
        """`hq`: the rows of `h` in e4m3 + scales when the kernel that made `h` left them (one launch less)."""
        st = self.status
        nq = 0 if hq is not None else 1
        if L["attn"]:
            q, gate, k, v = ops.attn_front(h, L["qkv_w"], L["qkv_s"], L["q_norm"], L["k_norm"], self.positions,
                                           self.cos_sin, 1e-6, True, status=st, quantised=hq)
            core = ops.attn_verify(q, gate, k, v, L["kcache"], L["vcache"], L["page_table"], self.seqlens,
                                   splits=self.attn_splits, status=st)
            return core, L["o_w"], L["o_s"], 1 + nq + 3
        mixed, z, b, a = ops.dense_fp8_split(h, L["in_w"], L["in_s"], GDN_SPLIT, outs=self.gdn_in, ws=self.dense_ws, status=st,
                                             quantised=hq)
        if self.gdn_layout == "ring":
            core = ops.gdn_verify_replay(mixed, z, a, b, L["conv_state"], L["conv_w"], L["window"], L["a_log"],
                                         L["dt_bias"], L["state"], L["d_ring"], L["dlo_ring"], L["k_ring"],
                                         L["klo_ring"], L["g_ring"], self.slots, self.slots, self.slots,
                                         self.write_pos, self.cache_base, L["gdn_norm"], 1e-6, status=st,
                                         ws=self.gdn_ws)
        else:
            core = ops.gdn_verify(mixed, z, a, b, L["conv_state"], L["conv_w"], L["a_log"], L["dt_bias"], L["state"],
                                  self.accepted, L["gdn_norm"], 1e-6, status=st, ws=self.gdn_ws)
        return core, L["out_w"], L["out_s"], 1 + nq + 2

    def run(self, x: torch.Tensor):
        """Generator form of `step`: yields the barrier channel at every point where the ranks of an expert-parallel
        group must meet (the caller runs the barrier, or advances the other virtual ranks); returns the tokens."""
        st, ep = self.status, self.ep
        T, R = self.T, self.rank
        self._chunks = 1          # the dense projections take any number of rows in one launch
        residual = torch.zeros_like(x)
        h = ops.add_rmsnorm(x, residual, self.first_norm)          # residual <- x, h = norm(x)
        n = 1
        hq = None
        for li, L in enumerate(self.layers):
            rec = None if self.trace is None else dict(h_in=h.clone(), residual_in=residual.clone())
            core, ow, osc, nl = self._mixer(L, h, hq)
            # output projection (split-K) + residual add + post-attention norm
            proj = torch.empty_like(residual) if rec is not None else None
            h2 = ops.dense_fp8_add_rmsnorm(core, ow, osc, residual, L["post_norm"], 1e-6, proj_out=proj, ws=self.proj_ws, status=st)
            ops.router(h2, L["wr"], K, None, scratch=self.scratch, want_logits=False, ids=self.ids, wts=self.wts)
            n += nl + 3 + 2
            if ep is None:
                ops.build_lists(self.ids, self.wts, self.lists)
                ops.moe_fp8(h2, L["w"], self.lists, cache=self.cache, ws=self.moe_ws, status=st)
                n += 1 + 4
            else:
                ops.ep_push(h2, self.ids, self.wts, R, self.peer_x, self.peer_ids, self.peer_wts)
                yield 0                                            # every rank's rows and routing have landed
                ops.build_lists(self.ids_all, self.wts_all, self.lists, None, e_lo=self.e_lo, shared_range=(R * T, T))
                ops.moe_fp8_ep(self.x_all, L["w"], self.lists, self.peer_cache, R, T, ws=self.moe_ws, status=st)
                yield 1                                            # every rank's rows for my tokens have landed
                n += 1 + 1 + 1 + 4 + 1
            if rec is not None:
                rec.update(core=core.clone(), proj=proj, h2=h2.clone(), ids=self.ids.clone(), wts=self.wts.clone(),
                           cache=self.cache.clone(), residual_mid=residual.clone())
            hq = (self.hq, self.hs)   # the next layer's projection reads these instead of quantising h again
            out, h = ops.moe_combine_norm(self.cache, h2, L["gate_w"], K, residual, L["next_norm"], quantised=hq)
            n += 1
            if rec is not None:
                rec.update(moe_out=out.clone(), h_out=h.clone(), residual_out=residual.clone())
                self.trace.append(rec)
        self.final_hidden = h
        if ep is None:
            _, idx, _ = ops.lmhead_argmax(h, self.lm_w, self.lm_s, 0, ws=self.lm_ws, status=st)
            self.launches = n + 3 * self._chunks
            return idx
        Ta = self.T_all
        ops.ep_put(h, R * T * H * 2, self.peer_h)
        yield 2
        mx, idx, _ = ops.lmhead_argmax(self.h_all, self.lm_w, self.lm_s, self.shard_lo, ws=self.lm_ws, status=st)
        ops.ep_put(mx, R * Ta * 4, self.peer_max)
        ops.ep_put(idx, R * Ta * 4, self.peer_idx)
        yield 3
        tokens = ops.argmax_merge(self.max_all, self.idx_all)      # the tokens of ALL sequences, on every rank
        self.launches = n + 1 + 1 + 3 + 2 + 1 + 1
        return tokens

    def step(self, x: torch.Tensor) -> torch.Tensor:
        """x bf16 [T, 2048] (this rank's embedded draft tokens) -> greedy next-token ids int32: [T] on one GPU, the
        ids of all ranks' rows [T_all] (rank-major) under expert parallelism."""
        if self.gate is not None:
            self.gate.sync()    # raises parallel.RankLost before anything is launched
        gen = self.run(x)
        try:
            while True:
                channel = next(gen)
                self.ep.barrier(channel, self.status)
        except StopIteration as stop:
            return stop.value


def step_virtual(steps, xs):
    """One step of every virtual rank of a `parallel.VirtualEpGroup` in lockstep; returns each rank's tokens."""
    return run_lockstep([s.run(x) for s, x in zip(steps, xs)])
