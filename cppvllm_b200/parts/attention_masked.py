"""Grouped-query attention whose mask and score terms are switched on by parameters (mixer ``masked_attention``):

    [q | k | v] = x W^T                       no biases; keys of `dim`, values of `vdim` elements per head
    q, k <- RMSNorm over dim * w              per head, one weight vector for all heads (``qk_norm``), in float
    q, k <- turned by the position            optional (``position``: a rotary part; its first rotary_dim elements in pairs)
    v    <- (1 - lam) v + lam v_first         ``v_mix = "mix"``: v_first is the same token's value in the model's first layer
                                              with ``v_mix = "first"`` (that layer keeps its values for the step); the mixed
                                              value is what the cache holds
    s_ij = scale q_i . k_j;  s <- c tanh(s / c) (``softcap`` = c);  s <- s - r1_h ln(1 + r2_h (i - j)) (``distance_bias``)
    visible: j <= i and  same chunk of ``chunk`` positions  |  i - j < ``window``  |  all;  with ``pool`` = P beside a window
             also one key and value per block of P positions that lies wholly before the window (the means of the block's
             cached keys and values), in the same softmax
    softmax, with exp(sink_h) added to the denominator (``sink``);  o_h <- o_h sigmoid((Wg x)_h) (``head_gate``);  y = Wo o

The cache holds, per token and kv head, the key and behind it the value; with pooled blocks a second plane of the same pages
holds the blocks' means at the place of position b (pages [plane, kv head, slot, dim + vdim]), written by the step that
brings a block's last token.  float32 and any sizes run on the general kernel; bf16 with sizes the tensor-core kernel takes
runs there (csrc/attention_masked.cu).
"""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import CacheSpec, Mixer, WeightSpec, register_part


@register_part("mixer", "masked_attention")
class MaskedAttention(Mixer):
    def __init__(self, runtime, prefix="", names=None, *, hidden_size: int, num_heads: int, num_kv_heads: int, dim: int, vdim: int,
                 scale: float, eps: float, qk_norm: bool = True, position=None, chunk: int = 0, window: int = 0, pool: int = 0,
                 softcap: float = 0.0, distance_bias: bool = False, sink: bool = False, head_gate: bool = False,
                 v_mix: str = "none", force_general: bool = False):
        super().__init__(runtime, prefix, names)
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads are not a multiple of {num_kv_heads} key/value heads")
        if v_mix not in ("none", "first", "mix"):
            raise ValueError(f"v_mix is 'none', 'first' or 'mix', got {v_mix!r}")
        if min(chunk, window, pool) < 0 or (pool and not window):
            raise ValueError("chunk, window and pool are not negative, and pooled blocks stand beside a window")
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.dim, self.vdim, self.scale, self.eps = int(dim), int(vdim), float(scale), float(eps)
        self.qk_norm, self.position = bool(qk_norm), position
        self.chunk, self.window, self.pool, self.softcap = int(chunk), int(window), int(pool), float(softcap or 0.0)
        self.distance_bias, self.sink, self.head_gate, self.v_mix = bool(distance_bias), bool(sink), bool(head_gate), v_mix
        self.force_general = bool(force_general) or runtime.plain_kernels
        self.planes = 2 if self.pool else 1
        self.rot = position.rotary_dim if position is not None else 0
        if self.rot > self.dim:
            raise ValueError(f"{self.rot} turned elements in a head of {self.dim}")
        self.w_in = self.w_o = self.q_norm = self.k_norm = self.r1 = self.r2 = self.sinks = self.lam = None

    def cache_spec(self) -> CacheSpec:
        if self.planes == 2:
            return CacheSpec((2, self.num_kv_heads, self.dim + self.vdim), token_axis=2)
        return CacheSpec((self.num_kv_heads, self.dim + self.vdim), token_axis=1)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        D, H, G, dk, dv = self.hidden_size, self.num_heads, self.num_kv_heads, self.dim, self.vdim
        f = self.full_name
        specs = {f("q"): WeightSpec((H * dk, D)), f("k"): WeightSpec((G * dk, D)), f("v"): WeightSpec((G * dv, D)),
                 f("o"): WeightSpec((D, H * dv))}
        if self.qk_norm:
            specs[f("q.norm")] = WeightSpec((dk,), role="vector", init="norm")
            specs[f("k.norm")] = WeightSpec((dk,), role="vector", init="norm")
        if self.v_mix != "none":            # the first mixing layer stores the number too and does not use it
            specs[f("vmix")] = WeightSpec((), role="vector", init="normal")
        if self.distance_bias:
            specs[f("r1")] = WeightSpec((H,), role="vector", init="norm")
            specs[f("r2")] = WeightSpec((H,), role="vector", init="norm")
        if self.sink:
            specs[f("sink")] = WeightSpec((H,), role="vector", init="normal")
        if self.head_gate:
            specs[f("g")] = WeightSpec((H, D))
        return specs

    def bind(self, tensors) -> None:
        t = lambda n: tensors[self.full_name(n)]          # noqa: E731
        rows = [t("q"), t("k"), t("v")] + ([t("g")] if self.head_gate else [])
        if len({r.dtype for r in rows}) > 1:
            rows = [r.float() for r in rows]
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.w_o = t("o")
        if self.qk_norm:
            self.q_norm, self.k_norm = t("q.norm"), t("k.norm")
        if self.v_mix == "mix":
            self.lam = t("vmix").reshape(1).contiguous()
        if self.distance_bias:
            self.r1, self.r2 = t("r1"), t("r2")
        if self.sink:
            self.sinks = t("sink")

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_o))

    def _project(self, x, w, out, rows):
        return ops.linear(x, w, out=out) if self.rt.plain_kernels else ops.project_rows(x, w, out, rows)

    def forward(self, x, ctx, cache, state):
        T = x.shape[0]
        H, G, dk, dv = self.num_heads, self.num_kv_heads, self.dim, self.vdim
        ws = self.rt.workspace
        g = ctx.groups[cache.group]
        packed = self._project(x, self.w_in, ws.rows("attn_qkv", T, self.w_in.shape[0], x.dtype), T)
        q = ws.rows("attn_q", T, H * dk, x.dtype)
        v_first_out = v_first_in = None
        if self.v_mix == "first":
            v_first_out = ws.rows("attn_v_first", T, G * dv, x.dtype)
            ctx.extras["v_first"] = v_first_out
        elif self.v_mix == "mix":
            v_first_in = ctx.extras.get("v_first")
            if v_first_in is None or v_first_in.shape[1] != G * dv:
                raise ValueError("values are mixed with those of an earlier layer of the same value size, which this step has not run")
        pos = self.position
        ops.masked_qkv_prep(q, packed, H, G, dk, dv, self.eps, q_weight=self.q_norm, k_weight=self.k_norm,
                            cos=pos.cos if pos is not None else None, sin=pos.sin if pos is not None else None, rot=self.rot,
                            interleaved=pos.interleaved if pos is not None else True, positions=ctx.positions,
                            pages=cache.pages if cache.writes else None, slots=g.slot_mapping if cache.writes else None,
                            page_size=g.page_size, planes=self.planes, v_first_out=v_first_out, v_first_in=v_first_in, lam=self.lam)
        if self.pool and cache.writes:
            ops.pool_entries(cache.pages, g.block_tables, ctx.seq_of_token, ctx.positions, T, G, dk + dv, self.pool, g.page_size)
        att = ws.rows("attn_out", T, H * dv, x.dtype)
        gate = packed[:, H * dk + G * (dk + dv):] if self.head_gate else None
        self.attend(att, q, gate, ctx, cache, g)
        return self._project(att, self.w_o, ws.rows("attn_proj", T, self.hidden_size, x.dtype), T)

    def attend(self, att, q, gate, ctx, cache, g):
        H, G, dk, dv = self.num_heads, self.num_kv_heads, self.dim, self.vdim
        if not self.force_general and ops.attn_masked_supported(q.dtype, H, G, dk, dv):
            q_lens = ctx.q_lens if ctx.q_lens is not None else [1] * ctx.num_seqs
            single = ctx.all_decode and ctx.num_tokens == ctx.num_seqs and H // G <= 16
            splits, scratch = 1, None
            if single:
                # what a decoded token can see at most: its chunk, or its window and the pooled blocks before it
                seen = ctx.max_kv_len
                if self.chunk:
                    seen = min(seen, self.chunk)
                if self.window:
                    seen = min(seen, self.window + (ctx.max_kv_len // self.pool if self.pool else 0))
                splits = ops.attn_masked_decode_splits(ctx.num_seqs, G, seen)
                if splits > 1:
                    most = ops.attn_keys_scratch_floats(self.rt.workspace.max_seqs, G, dv, 8)
                    scratch = self.rt.workspace.flat(f"attn_masked_parts_{G}_{dv}", most, torch.float32)
            ops.attn_masked_bf16(att, q, cache.pages, g.block_tables, ctx.cu_seqlens, ctx.positions, ctx.num_seqs,
                                 ops.attn_keys_tiles(q_lens, H, G), H, G, dk, dv, g.page_size, self.scale, planes=self.planes,
                                 chunk=self.chunk, window=self.window, pool=self.pool, softcap=self.softcap, r1=self.r1, r2=self.r2,
                                 sink=self.sinks, gate=gate, all_single=single, splits=splits, scratch=scratch)
            return
        ops.attn_masked_general(att, q, cache.pages, g.block_tables, ctx.seq_of_token, ctx.positions, ctx.num_tokens, H, G, dk, dv,
                                g.page_size, self.scale, planes=self.planes, chunk=self.chunk, window=self.window, pool=self.pool,
                                softcap=self.softcap, r1=self.r1, r2=self.r2, sink=self.sinks, gate=gate)
