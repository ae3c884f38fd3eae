"""Attention whose keys and values are up-projections of one small latent vector per token, so that only the latent
(and one positional key part that all heads share) is cached:

    [a | b | r | z] = x Wdown^T         Wdown = rows(dq) over rows(dkv) over rows(g); a: q_rank, b: kv_rank, r: rot_dim, z: H
    cq = RMSNorm(a) * w_q;   q = Wuq cq, per head [nope_dim | rot_dim]
    c  = RMSNorm(b) * w_kv;  kr = rot_p(r);   the cache entry of the token is [c | kr]
    k_h = Wuk_h c,  v_h = Wuv_h c;   s_ij = scale * (q_nope_i . k_h,j + rot_i(q_rot_i) . kr_j),  j <= i;  softmax over j
    y = Wo concat_h( sigmoid(z_h) * sum_j a_ij v_h,j )

The up-projections are taken to the query's and the output's side, so that attention runs over the cached entries
themselves and no key or value is ever rebuilt:  q_nope . (Wuk_h c) = (Wuk_h^T q_nope) . c,  and
sum_j a_ij Wuv_h c_j = Wuv_h (sum_j a_ij c_j).  Every head then reads the same entries: keys of kv_rank + rot_dim elements
whose first kv_rank elements are also the value: one kv head and a value narrower than the key, on the tensor cores
(csrc/attention_keys.cu) for bf16 entries of up to 128 elements in steps of 16, else in csrc/attention_general.cu.  The two per-head products are batched library products.  The rotation turns the first ``rot`` elements of the
positional parts in pairs (2i, 2i+1); the rest pass.  ``reads_other_cache``: the layer has no dkv projection and reads the
entries another layer wrote (the run list names the unit), with its own up-projections, queries and gate.
``q_rank = 0``: the queries have no latent of their own, q = Wq x (tensor ``q``).  ``gate = "element"``: the gate has one number
per element of the concatenated heads (Wg is [H * value_dim, D]): y = Wo (concat_h(o_h) * sigmoid(Wg x)).
"""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import CacheSpec, Mixer, WeightSpec, register_part


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    def __init__(self, runtime, prefix="", names=None, *, hidden_size: int, num_heads: int, nope_dim: int, rot_dim: int,
                 value_dim: int, q_rank: int = 0, kv_rank: int, scale: float, eps: float, position, rot: int = -1,
                 reads_other_cache: bool = False, gate: str = "head"):
        super().__init__(runtime, prefix, names)
        self.hidden_size, self.num_heads, self.nope_dim, self.rot_dim = int(hidden_size), int(num_heads), int(nope_dim), int(rot_dim)
        self.value_dim, self.q_rank, self.kv_rank = int(value_dim), int(q_rank), int(kv_rank)
        self.scale, self.eps = float(scale), float(eps)
        self.position = position
        self.rot = int(rot) if rot >= 0 else position.rotary_dim
        if self.rot > self.rot_dim or self.rot != position.rotary_dim or not position.interleaved:
            raise ValueError("the positional part is turned in pairs (2i, 2i+1) over at most its own width")
        self.own_cache = not reads_other_cache
        if gate not in ("head", "element"):
            raise ValueError(f"gate is 'head' or 'element', got {gate!r}")
        self.gate_cols = self.num_heads if gate == "head" else self.num_heads * self.value_dim
        self.w_down = self.w_uq = self.w_uk = self.w_uv = self.w_o = self.w_qnorm = self.w_kvnorm = None

    def cache_spec(self) -> CacheSpec:
        return CacheSpec((self.kv_rank + self.rot_dim,), token_axis=0)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        D, H = self.hidden_size, self.num_heads
        specs = {
            self.full_name("uk"): WeightSpec((H * self.nope_dim, self.kv_rank)),
            self.full_name("uv"): WeightSpec((H * self.value_dim, self.kv_rank)),
            self.full_name("g"): WeightSpec((self.gate_cols, D)),
            self.full_name("o"): WeightSpec((D, H * self.value_dim)),
        }
        if self.q_rank:
            specs[self.full_name("dq")] = WeightSpec((self.q_rank, D))
            specs[self.full_name("dq.norm")] = WeightSpec((self.q_rank,), role="vector", init="norm")
            specs[self.full_name("uq")] = WeightSpec((H * (self.nope_dim + self.rot_dim), self.q_rank))
        else:
            specs[self.full_name("q")] = WeightSpec((H * (self.nope_dim + self.rot_dim), D))
        if self.own_cache:
            specs[self.full_name("dkv")] = WeightSpec((self.kv_rank + self.rot_dim, D))
            specs[self.full_name("dkv.norm")] = WeightSpec((self.kv_rank,), role="vector", init="norm")
        return specs

    def bind(self, tensors) -> None:
        t = lambda n: tensors[self.full_name(n)]          # noqa: E731
        rows = ([t("dq")] if self.q_rank else []) + ([t("dkv")] if self.own_cache else []) + [t("g")]
        if len({r.dtype for r in rows}) > 1:
            rows = [r.float() for r in rows]
        self.w_down = torch.cat(rows, dim=0).contiguous()
        self.kv_off = self.q_rank
        self.g_off = self.q_rank + (self.kv_rank + self.rot_dim if self.own_cache else 0)
        self.w_qnorm = t("dq.norm") if self.q_rank else None
        self.w_kvnorm = t("dkv.norm") if self.own_cache else None
        self.w_uq, self.w_o = (t("uq") if self.q_rank else t("q")), t("o")
        H = self.num_heads
        self.w_uk = t("uk").view(H, self.nope_dim, self.kv_rank)                        # q_abs_h = q_nope_h @ Wuk_h
        self.w_uv = t("uv").view(H, self.value_dim, self.kv_rank).transpose(1, 2)       # o_h = o_lat_h @ Wuv_h^T

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_down, self.w_uq, self.w_uk, self.w_uv, self.w_o))

    def _project(self, x, w, out, rows):
        return ops.linear(x, w, out=out) if self.rt.plain_kernels else ops.project_rows(x, w, out, rows)

    def forward(self, x, ctx, cache, state):
        T = x.shape[0]
        H, dn, dr, dv, R = self.num_heads, self.nope_dim, self.rot_dim, self.value_dim, self.kv_rank
        ws = self.rt.workspace
        g = ctx.groups[cache.group]
        pos = self.position
        packed = self._project(x, self.w_down, ws.rows("lat_down", T, self.w_down.shape[0], x.dtype), T)
        cq = ws.rows("lat_cq", T, self.q_rank, x.dtype) if self.q_rank else None
        writes = self.own_cache and cache.writes
        ops.latent_prep(packed, cq, 0, self.q_rank, self.w_qnorm, cache.pages if writes else None, self.kv_off, R, dr, self.rot,
                        self.w_kvnorm, pos.cos, pos.sin, ctx.positions, g.slot_mapping if writes else None, self.eps)
        q = self._project(cq if self.q_rank else x, self.w_uq, ws.rows("lat_q", T, H * (dn + dr), x.dtype), T)
        q_abs = ws.rows("lat_qabs", T, H * R, x.dtype).view(H, T, R)
        torch.bmm(q.view(T, H, dn + dr)[:, :, :dn].transpose(0, 1), self.w_uk, out=q_abs)
        q_att = ops.latent_q_assemble(ws.rows("lat_qatt", T, H * (R + dr), x.dtype), q_abs, q, H, dn, R, dr, self.rot, pos.cos,
                                      pos.sin, ctx.positions)
        o_lat = ws.rows("lat_o", T, H * R, x.dtype)
        self.attend(o_lat, q_att, ctx, cache, g)
        o_heads = ws.rows("lat_ov", T, H * dv, x.dtype).view(H, T, dv)
        torch.bmm(o_lat.view(T, H, R).transpose(0, 1), self.w_uv, out=o_heads)
        att = ops.head_gate(ws.rows("attn_out", T, H * dv, x.dtype), o_heads, packed[:, self.g_off:self.g_off + self.gate_cols], H, dv,
                            per_element=self.gate_cols != H)
        return self._project(att, self.w_o, ws.rows("attn_proj", T, self.hidden_size, x.dtype), T)

    def attend(self, o_lat, q_att, ctx, cache, g):
        H, HD, R = self.num_heads, self.kv_rank + self.rot_dim, self.kv_rank
        if not self.rt.plain_kernels and R % 16 == 0 and ops.attn_keys_supported(q_att.dtype, H, 1, HD, q_att.shape[1]):
            # bf16, sizes in steps of 16 up to 128: the tensor-core kernel over keys that are values, with a narrower value
            q_lens = ctx.q_lens if ctx.q_lens is not None else [1] * ctx.num_seqs
            if ctx.all_decode and ctx.num_tokens == ctx.num_seqs:
                # one token per request: the heads go in groups of at most 16 (a slab of the decode kernel), all on the one entry
                groups = min(n for n in range(1, H + 1) if H % n == 0 and H // n <= 16)
                splits, scratch = ops.attn_keys_decode_splits(ctx.num_seqs, groups, ctx.max_kv_len), None
                if splits > 1:
                    most = ops.attn_keys_scratch_floats(self.rt.workspace.max_seqs, groups, HD, 8)
                    scratch = self.rt.workspace.flat(f"attn_keys_parts_{groups}_{HD}", most, torch.float32)
                ops.attn_keys_bf16(o_lat, q_att, cache.pages, g.block_tables, ctx.cu_seqlens, ctx.positions, ctx.num_seqs,
                                   ctx.num_seqs, H, groups, HD, g.page_size, self.scale, all_single=True, splits=splits,
                                   scratch=scratch, value_dim=R, kv_heads_in_pages=1)
                return
            ops.attn_keys_bf16(o_lat, q_att, cache.pages, g.block_tables, ctx.cu_seqlens, ctx.positions, ctx.num_seqs,
                               ops.attn_keys_tiles(q_lens, H, 1), H, 1, HD, g.page_size, self.scale, value_dim=R)
            return
        ops.paged_attention_general(o_lat, q_att, cache.pages, g.block_tables, ctx.seq_of_token, ctx.positions, self.num_heads, 1,
                                    self.kv_rank + self.rot_dim, g.page_size, self.scale, num_tokens=ctx.num_tokens,
                                    keys_are_values=True, value_dim=self.kv_rank)
