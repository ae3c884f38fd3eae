"""Grouped-query attention without rotation, whose positions enter through a learned bias per head and distance and through
a temperature on the queries:

    [q | k | v] = x W^T                    no biases; keys of `dim`, values of `vdim` elements per head (they may differ)
    q <- RMSNorm(q) * wq,  k <- RMSNorm(k) * wk     ONE norm over the whole projection (all heads at once), plain weights
    q_p <- q_p * (1 + coef * ln(floor((p + 1) / every) + 1))      at position p (every = 0: no temperature)
    s_pj = scale * q_p . k_j + R[bucket(p - j), head]              over j <= p;  softmax;  y = Wo concat_h(sum_j a_pj v_j)
    bucket(n) = n                                                            for n < B/2
              = min(B - 1, B/2 + floor(ln(n / (B/2)) / ln(far / (B/2)) * (B - B/2)))   else       (B = rows of R)

Every distance of `far` and more falls into the last bucket, so the bias is a table [H, far + 1] by distance, made once at
load time; the kernels look up min(p - j, far).  The cache holds, per token and kv head, the normed key and behind it the
value (pages [page, kv head, slot, dim + vdim]).  A mixer with ``reads_other_cache`` has no key and value projections and
reads the entries another layer wrote, with its own queries, bias table and output projection.  bf16 with sizes the
tensor-core kernel takes runs there (csrc/attention_bias.cu); float32 and other shapes take the general kernel
(csrc/attention_general.cu).
"""
from __future__ import annotations

import math
from typing import Dict

import torch

from ..csrc import ops
from .base import CacheSpec, Mixer, WeightSpec, register_part


def distance_buckets(rows: int, far: int):
    """bucket(n) for n = 0..far; every larger distance shares the last entry."""
    half = rows // 2
    if half < 1 or far <= half:
        raise ValueError(f"a distance table of {rows} rows needs a largest distance above {half}, got {far}")
    out = []
    for n in range(far + 1):
        if n < half:
            out.append(n)
        else:
            out.append(min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half)))))
    return out


@register_part("mixer", "biased_attention")
class BiasedAttention(Mixer):
    def __init__(self, runtime, prefix="", names=None, *, hidden_size: int, num_heads: int, num_kv_heads: int, dim: int, vdim: int,
                 scale: float, eps: float, bias_max: int, bias_rows: int = -1, temp_coef: float = 0.0, temp_every: int = 0,
                 reads_other_cache: bool = False, force_general: bool = False):
        super().__init__(runtime, prefix, names)
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads are not a multiple of {num_kv_heads} key/value heads")
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.dim, self.vdim, self.scale, self.eps = int(dim), int(vdim), float(scale), float(eps)
        self.bias_max, self.bias_rows = int(bias_max), int(bias_rows) if bias_rows else -1
        self.temp_coef, self.temp_every = float(temp_coef), int(temp_every)
        if self.temp_every < 0 or self.bias_max < 1:
            raise ValueError("temp_every cannot be negative and bias_max is at least 1")
        self.reads_other_cache = bool(reads_other_cache)
        self.force_general = bool(force_general) or runtime.plain_kernels
        self.w_in = self.w_o = self.q_norm = self.k_norm = self.bias_table = None

    def cache_spec(self) -> CacheSpec:
        return CacheSpec((self.num_kv_heads, self.dim + self.vdim), token_axis=1)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        D, H, G, dk, dv = self.hidden_size, self.num_heads, self.num_kv_heads, self.dim, self.vdim
        f = self.full_name
        specs = {f("q"): WeightSpec((H * dk, D)), f("q.norm"): WeightSpec((H * dk,), role="vector", init="norm"),
                 f("rel"): WeightSpec((self.bias_rows, H), role="vector"), f("o"): WeightSpec((D, H * dv))}
        if not self.reads_other_cache:
            specs.update({f("k"): WeightSpec((G * dk, D)), f("v"): WeightSpec((G * dv, D)),
                          f("k.norm"): WeightSpec((G * dk,), role="vector", init="norm")})
        return specs

    def bind(self, tensors) -> None:
        t = lambda n: tensors[self.full_name(n)]          # noqa: E731
        rows = [t("q")] if self.reads_other_cache else [t("q"), t("k"), t("v")]
        if len({r.dtype for r in rows}) > 1:
            rows = [r.float() for r in rows]
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.w_o, self.q_norm = t("o"), t("q.norm")
        self.k_norm = None if self.reads_other_cache else t("k.norm")
        rel = t("rel").float()
        self.bias_rows = rel.shape[0]
        buckets = torch.tensor(distance_buckets(self.bias_rows, self.bias_max), dtype=torch.long, device=rel.device)
        self.bias_table = rel[buckets].t().contiguous()                 # [H, far + 1]

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
        writes = cache.writes and not self.reads_other_cache
        ops.wide_qk_prep(q, packed, self.q_norm, ctx.positions, self.eps, self.temp_coef, self.temp_every, G, dk, dv,
                         pages=cache.pages if writes else None, k_weight=self.k_norm, slots=g.slot_mapping if writes else None,
                         page_size=g.page_size)
        att = ws.rows("attn_out", T, H * dv, x.dtype)
        self.attend(att, q, ctx, cache, g)
        return self._project(att, self.w_o, ws.rows("attn_proj", T, self.hidden_size, x.dtype), T)

    def attend(self, att, q, ctx, cache, g):
        H, G, dk, dv = self.num_heads, self.num_kv_heads, self.dim, self.vdim
        if not self.force_general and ops.attn_bias_supported(q.dtype, H, G, dk, dv):
            q_lens = ctx.q_lens if ctx.q_lens is not None else [1] * ctx.num_seqs
            single = ctx.all_decode and ctx.num_tokens == ctx.num_seqs
            splits, scratch = 1, None
            if single:
                splits = ops.attn_keys_decode_splits(ctx.num_seqs, G, ctx.max_kv_len)
                if splits > 1:
                    most = ops.attn_keys_scratch_floats(self.rt.workspace.max_seqs, G, dv, 8)
                    scratch = self.rt.workspace.flat(f"attn_bias_parts_{G}_{dv}", most, torch.float32)
            ops.attn_bias_bf16(att, q, cache.pages, g.block_tables, ctx.cu_seqlens, ctx.positions, ctx.num_seqs,
                               ops.attn_keys_tiles(q_lens, H, G), H, G, dk, dv, g.page_size, self.scale, self.bias_table,
                               all_single=single, splits=splits, scratch=scratch)
            return
        ops.paged_attention_entries(att, q, cache.pages, g.block_tables, ctx.seq_of_token, ctx.positions, H, G, dk, dv, g.page_size,
                                    self.scale, bias=self.bias_table, num_tokens=ctx.num_tokens)
