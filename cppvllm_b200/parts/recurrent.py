"""Mixers that carry a matrix per request and head from token to token (fixed-size state in the request's state slot, float32,
zero at admission) instead of a cache that grows with the sequence.  The recurrences run in float32 whatever the activations'
type; only the projections around them are products in the activations' type.

* ``lightning``: q = silu(Wq x), k = silu(Wk x), v = silu(Wv x), heads side by side;  S <- decay_h S + k v^T;  o = S^T q;
  y = Wo (RMSNorm(concat_h o) * w * sigmoid(Wg x)).  State per request: [H, dim, vdim].
* ``channel_delta``: q = Wq x, k = Wk x (kv_heads x dim), v = Wv x (heads x vdim), each through a short causal convolution
  over time per channel (weights [channels, taps], last tap on the current token) and silu; q and k unit vectors per head
  (x / sqrt(sum x^2 + 1e-6)), q also times dim^-1/2; b = sigmoid(Wb x) per head; g = exp(-exp(A_h) * softplus(Wa2 Wa1 x + dt))
  per head and key channel;  S <- diag(g) S;  u = b (v - S^T k);  S <- S + k u^T;  o = S^T q (head h reads q/k head
  h / (heads / kv_heads));  y = Wo concat_h(RMSNorm(o_h) * w * sigmoid(Wg2 Wg1 x)_h), w shared by the heads.  State per request:
  [H, dim, vdim] and behind it the last taps - 1 inputs of the convolutions [taps - 1, channels].  The inner sizes of the
  two low-rank projections are whatever the checkpoint holds.
* ``head_delta``: the same rule with ONE decay per head and token, g = exp(-exp(A_h) * softplus(Wa x + dt_h)), S <- g S, full-rank
  projections for the decay (Wa [H, D]) and the output gate (Wg [H * vdim, D]), and the gate through silu instead of the
  logistic function: y = Wo concat_h(RMSNorm(o_h) * w * silu(Wg x)_h).
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch

from ..csrc import ops
from .base import Mixer, StateSpec, WeightSpec, register_part


def _project(rt, x, w, out, rows):
    return ops.linear(x, w, out=out) if rt.plain_kernels else ops.project_rows(x, w, out, rows)


def _cat_rows(rows):
    if len({r.dtype for r in rows}) > 1:
        rows = [r.float() for r in rows]
    return torch.cat(rows, dim=0).contiguous()


@register_part("mixer", "lightning")
class LightningMixer(Mixer):
    def __init__(self, runtime, prefix="", names=None, *, hidden_size: int, num_heads: int, dim: int, vdim: int,
                 decay: Sequence[float], eps: float):
        super().__init__(runtime, prefix, names)
        self.hidden_size, self.num_heads, self.dim, self.vdim, self.eps = int(hidden_size), int(num_heads), int(dim), int(vdim), float(eps)
        if len(decay) != self.num_heads:
            raise ValueError(f"{len(decay)} decays for {self.num_heads} heads")
        if self.dim > 256:
            raise ValueError("the scan kernel keeps at most 256 key channels per head")
        self.decay = torch.tensor([float(d) for d in decay], dtype=torch.float32, device=runtime.device)
        self.w_in = self.w_o = self.w_norm = None

    def state_spec(self) -> StateSpec:
        return StateSpec((self.num_heads * self.dim * self.vdim,), torch.float32)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        D, H, dk, dv = self.hidden_size, self.num_heads, self.dim, self.vdim
        return {self.full_name("q"): WeightSpec((H * dk, D)), self.full_name("k"): WeightSpec((H * dk, D)),
                self.full_name("v"): WeightSpec((H * dv, D)), self.full_name("g"): WeightSpec((H * dv, D)),
                self.full_name("o"): WeightSpec((D, H * dv)),
                self.full_name("norm"): WeightSpec((H * dv,), role="vector", init="norm")}

    def bind(self, tensors) -> None:
        t = lambda n: tensors[self.full_name(n)]          # noqa: E731
        self.w_in = _cat_rows([t("q"), t("k"), t("v"), t("g")])
        self.w_o, self.w_norm = t("o"), t("norm")

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_o))

    def forward(self, x, ctx, cache, state):
        T = x.shape[0]
        H, dk, dv = self.num_heads, self.dim, self.vdim
        ws = self.rt.workspace
        packed = _project(self.rt, x, self.w_in, ws.rows("rec_in", T, self.w_in.shape[0], x.dtype), T)
        f32 = torch.float32
        qf, kf, vf = ws.rows("delta_q", T, H * dk, f32), ws.rows("delta_k", T, H * dk, f32), ws.rows("delta_v", T, H * dv, f32)
        ops.lightning_prep(qf, kf, vf, packed, 0, H * dk, 2 * H * dk)
        o = ws.rows("rec_o", T, H * dv, f32)
        ops.lightning_scan(o, qf, kf, vf, state, self.decay, ctx.cu_seqlens, ctx.state_slots, ctx.num_seqs, H, dk, dv)
        g_off = 2 * H * dk + H * dv
        y = ops.gated_norm(ws.rows("rec_y", T, H * dv, x.dtype), o, packed[:, g_off:g_off + H * dv], self.w_norm, 1, self.eps)
        return _project(self.rt, y, self.w_o, ws.rows("attn_proj", T, self.hidden_size, x.dtype), T)


@register_part("mixer", "channel_delta")
class ChannelDeltaMixer(Mixer):
    def __init__(self, runtime, prefix="", names=None, *, hidden_size: int, num_heads: int, num_kv_heads: int, dim: int, vdim: int,
                 taps: int, eps: float, decay_rank: Optional[int] = None, gate_rank: Optional[int] = None):
        super().__init__(runtime, prefix, names)
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.dim, self.vdim, self.taps, self.eps = int(dim), int(vdim), int(taps), float(eps)
        if self.num_heads % self.num_kv_heads:
            raise ValueError(f"{self.num_heads} heads are not a multiple of {self.num_kv_heads} query/key heads")
        if self.taps < 1:
            raise ValueError("a convolution has at least one tap")
        if self.dim > 256:
            raise ValueError("the scan kernel keeps at most 256 key channels per head")
        self.decay_rank = int(decay_rank) if decay_rank else -1
        self.gate_rank = int(gate_rank) if gate_rank else -1
        self.channels = 2 * self.num_kv_heads * self.dim + self.num_heads * self.vdim
        self.matrix_floats = self.num_heads * self.dim * self.vdim

    def state_spec(self) -> StateSpec:
        return StateSpec((self.matrix_floats + (self.taps - 1) * self.channels,), torch.float32)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        D, H, G, dk, dv, K = self.hidden_size, self.num_heads, self.num_kv_heads, self.dim, self.vdim, self.taps
        f = self.full_name
        return {f("q"): WeightSpec((G * dk, D)), f("q.conv"): WeightSpec((G * dk, K), role="vector"),
                f("k"): WeightSpec((G * dk, D)), f("k.conv"): WeightSpec((G * dk, K), role="vector"),
                f("v"): WeightSpec((H * dv, D)), f("v.conv"): WeightSpec((H * dv, K), role="vector"),
                f("b"): WeightSpec((H, D)), f("A_log"): WeightSpec((H,), role="vector"),
                f("norm"): WeightSpec((dv,), role="vector", init="norm"),
                f("a1"): WeightSpec((self.decay_rank, D)), f("a2"): WeightSpec((H * dk, self.decay_rank)),
                f("dt_bias"): WeightSpec((H * dk,), role="vector"),
                f("g1"): WeightSpec((self.gate_rank, D)), f("g2"): WeightSpec((H * dv, self.gate_rank)),
                f("o"): WeightSpec((D, H * dv))}

    def bind(self, tensors) -> None:
        t = lambda n: tensors[self.full_name(n)]          # noqa: E731
        self.decay_rank, self.gate_rank = t("a1").shape[0], t("g1").shape[0]
        if t("a2").shape[1] != self.decay_rank or t("g2").shape[1] != self.gate_rank:
            raise ValueError(f"{self.prefix}: the two halves of a low-rank projection disagree about its inner size")
        self.w_in = _cat_rows([t("q"), t("k"), t("v"), t("g1"), t("a1")])
        self.g_off = self.channels
        self.a_off = self.channels + self.gate_rank
        self.w_b, self.w_a2, self.w_g2, self.w_o = t("b"), t("a2"), t("g2"), t("o")
        self.conv_w = torch.cat([t("q.conv"), t("k.conv"), t("v.conv")], dim=0).contiguous()
        self.dt_bias, self.a_log, self.w_norm = t("dt_bias"), t("A_log"), t("norm")

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_b, self.w_a2, self.w_g2, self.w_o))

    def forward(self, x, ctx, cache, state):
        T, S = x.shape[0], ctx.num_seqs
        H, G, dk, dv = self.num_heads, self.num_kv_heads, self.dim, self.vdim
        ws = self.rt.workspace
        f32 = torch.float32
        packed = _project(self.rt, x, self.w_in, ws.rows("rec_in", T, self.w_in.shape[0], x.dtype), T)
        # what enters the recurrence leaves its product unrounded
        b = ops.linear(x, self.w_b, out=ws.rows("delta_b", T, H, f32), out_dtype=f32)
        a = ops.linear(packed[:, self.a_off:self.a_off + self.decay_rank], self.w_a2, out=ws.rows("delta_a", T, H * dk, f32), out_dtype=f32)
        gate = ops.linear(packed[:, self.g_off:self.g_off + self.gate_rank], self.w_g2, out=ws.rows("delta_gate", T, H * dv, x.dtype))
        qn, kn = ws.rows("delta_q", T, G * dk, f32), ws.rows("delta_k", T, G * dk, f32)
        vv, gg, bb = ws.rows("delta_v", T, H * dv, f32), ws.rows("delta_g", T, H * dk, f32), ws.rows("delta_beta", T, H, f32)
        ops.delta_prep(qn, kn, vv, gg, bb, packed, 0, self.conv_w, a, self.dt_bias, self.a_log, b, state, self.matrix_floats,
                       ctx.seq_of_token, ctx.cu_seqlens, ctx.state_slots, H, G, dk, dv)
        ops.conv_history(state, self.matrix_floats, packed, 0, self.channels, self.taps, ctx.cu_seqlens, ctx.state_slots, S)
        o = ws.rows("rec_o", T, H * dv, f32)
        ops.delta_scan(o, qn, kn, vv, gg, bb, state, ctx.cu_seqlens, ctx.state_slots, S, H, G, dk, dv)
        y = ops.gated_norm(ws.rows("rec_y", T, H * dv, x.dtype), o, gate, self.w_norm, H, self.eps)
        return _project(self.rt, y, self.w_o, ws.rows("attn_proj", T, self.hidden_size, x.dtype), T)


@register_part("mixer", "head_delta")
class HeadDeltaMixer(Mixer):
    def __init__(self, runtime, prefix="", names=None, *, hidden_size: int, num_heads: int, num_kv_heads: int, dim: int, vdim: int,
                 taps: int, eps: float):
        super().__init__(runtime, prefix, names)
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.dim, self.vdim, self.taps, self.eps = int(dim), int(vdim), int(taps), float(eps)
        if self.num_heads % self.num_kv_heads:
            raise ValueError(f"{self.num_heads} heads are not a multiple of {self.num_kv_heads} query/key heads")
        if self.taps < 1:
            raise ValueError("a convolution has at least one tap")
        if self.dim > 256:
            raise ValueError("the scan kernel keeps at most 256 key channels per head")
        self.channels = 2 * self.num_kv_heads * self.dim + self.num_heads * self.vdim
        self.matrix_floats = self.num_heads * self.dim * self.vdim

    def state_spec(self) -> StateSpec:
        return StateSpec((self.matrix_floats + (self.taps - 1) * self.channels,), torch.float32)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        D, H, G, dk, dv, K = self.hidden_size, self.num_heads, self.num_kv_heads, self.dim, self.vdim, self.taps
        f = self.full_name
        return {f("q"): WeightSpec((G * dk, D)), f("q.conv"): WeightSpec((G * dk, K), role="vector"),
                f("k"): WeightSpec((G * dk, D)), f("k.conv"): WeightSpec((G * dk, K), role="vector"),
                f("v"): WeightSpec((H * dv, D)), f("v.conv"): WeightSpec((H * dv, K), role="vector"),
                f("b"): WeightSpec((H, D)), f("a"): WeightSpec((H, D)), f("A_log"): WeightSpec((H,), role="vector"),
                f("dt_bias"): WeightSpec((H,), role="vector"), f("norm"): WeightSpec((dv,), role="vector", init="norm"),
                f("g"): WeightSpec((H * dv, D)), f("o"): WeightSpec((D, H * dv))}

    def bind(self, tensors) -> None:
        t = lambda n: tensors[self.full_name(n)]          # noqa: E731
        self.w_in = _cat_rows([t("q"), t("k"), t("v"), t("g")])
        self.g_off = self.channels
        self.w_b, self.w_a, self.w_o = t("b"), t("a"), t("o")
        self.conv_w = torch.cat([t("q.conv"), t("k.conv"), t("v.conv")], dim=0).contiguous()
        self.dt_bias, self.a_log, self.w_norm = t("dt_bias"), t("A_log"), t("norm")

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_b, self.w_a, self.w_o))

    def forward(self, x, ctx, cache, state):
        T, S = x.shape[0], ctx.num_seqs
        H, G, dk, dv = self.num_heads, self.num_kv_heads, self.dim, self.vdim
        ws = self.rt.workspace
        f32 = torch.float32
        packed = _project(self.rt, x, self.w_in, ws.rows("rec_in", T, self.w_in.shape[0], x.dtype), T)
        # what enters the recurrence leaves its product unrounded
        b = ops.linear(x, self.w_b, out=ws.rows("delta_b", T, H, f32), out_dtype=f32)
        a = ops.linear(x, self.w_a, out=ws.rows("delta_a1", T, H, f32), out_dtype=f32)
        qn, kn = ws.rows("delta_q", T, G * dk, f32), ws.rows("delta_k", T, G * dk, f32)
        vv, gg, bb = ws.rows("delta_v", T, H * dv, f32), ws.rows("delta_g1", T, H, f32), ws.rows("delta_beta", T, H, f32)
        ops.delta_prep(qn, kn, vv, gg, bb, packed, 0, self.conv_w, a, self.dt_bias, self.a_log, b, state, self.matrix_floats,
                       ctx.seq_of_token, ctx.cu_seqlens, ctx.state_slots, H, G, dk, dv, decay_dim=1)
        ops.conv_history(state, self.matrix_floats, packed, 0, self.channels, self.taps, ctx.cu_seqlens, ctx.state_slots, S)
        o = ws.rows("rec_o", T, H * dv, f32)
        ops.delta_scan(o, qn, kn, vv, gg, bb, state, ctx.cu_seqlens, ctx.state_slots, S, H, G, dk, dv, decay_dim=1)
        y = ops.gated_norm(ws.rows("rec_y", T, H * dv, x.dtype), o, packed[:, self.g_off:self.g_off + H * dv], self.w_norm, H, self.eps,
                           gate_act="silu")
        return _project(self.rt, y, self.w_o, ws.rows("attn_proj", T, self.hidden_size, x.dtype), T)
