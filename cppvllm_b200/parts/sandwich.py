"""Block ``sandwich``: every sublayer stands between two norms, reads its input through a short convolution over time and
leaves through a learned gate.  On a residual stream x kept in float32, per sublayer f (the mixer, then the feed-forward if
the layer has one):

    a = norm_in(x)                                   RMS norm, weights as the norm parts store them
    h = a + conv(a)                                  conv(a)_t = sum_j c[:, j] a_(t - K + 1 + j): causal, per channel, no bias
    r = f(h) * sigmoid(Wr a + br)                    the gate reads a, not h
    x <- x + norm_out(r)

The last K - 1 rows of `a` are part of a request's state, for both sublayers of every layer: the block asks for K - 1 rows
per sublayer behind the mixer's own state in the run entry's state row (float32, zero at admission), so portions of a
prompt cut anywhere continue where the history stands.  Kernels (csrc/sandwich.cu): the convolution; and ONE kernel for
the gate, the norm behind the sublayer, the sum into the stream, the history's update and the norm in front of the NEXT
sublayer (the new row of the stream never leaves the chip in between).  The block hands the already normed input of the
next layer on as its pending value, so a layer costs two such kernels, two convolutions and two gate products besides its
sublayers.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import ops
from .base import Block, StateSpec, WeightSpec, register_part


class NormedAhead:
    """What a sandwich block leaves as `pending`: the next norm's output, already computed by the kernel that closed the
    block, together with the weight it was made with (a following block of another kind, or the final norm, ignores it
    unless the weight is its own)."""

    def __init__(self, rows: torch.Tensor, weight: torch.Tensor):
        self.rows, self.weight = rows, weight


@register_part("block", "sandwich")
class SandwichBlock(Block):
    accepts_normed_ahead = True       # forward() takes a NormedAhead made with its first norm's weight as `pending`

    def __init__(self, runtime, prefix="", names=None, *, mixer, ffn, mixer_norm, ffn_norm=None, hidden_size: int, taps: int, eps: float,
                 out_offset: float = 1.0):
        super().__init__(runtime, prefix, names)
        if (ffn is None) != (ffn_norm is None):
            raise ValueError("a feed-forward and the norm in front of it come together")
        if int(taps) < 1:
            raise ValueError("a convolution has at least one tap")
        self.mixer, self.ffn, self.mixer_norm, self.ffn_norm = mixer, ffn, mixer_norm, ffn_norm
        self.hidden_size, self.taps, self.eps, self.out_offset = int(hidden_size), int(taps), float(eps), float(out_offset)
        ms = mixer.state_spec()
        if ms is not None and (ms.dtype != torch.float32 or len(ms.shape) != 1):
            raise ValueError("the mixer's state must be one float32 row: the block's histories lie behind it")
        self.mixer_floats = int(ms.shape[0]) if ms is not None else 0
        self.taps1 = self.taps2 = self.w_g1 = self.w_g2 = self.b_g1 = self.b_g2 = self.w_out1 = self.w_out2 = None

    def parts(self):
        return tuple(p for p in (self, self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if p is not None)

    def state_spec(self) -> StateSpec:
        subs = 2 if self.ffn is not None else 1
        return StateSpec((self.mixer_floats + subs * (self.taps - 1) * self.hidden_size,), torch.float32)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        D, K = self.hidden_size, self.taps
        f = self.full_name
        specs = {}
        for n in ("1", "2") if self.ffn is not None else ("1",):
            specs[f("norm" + n + "b")] = WeightSpec((D,), role="vector", init="normal" if self.out_offset else "norm")
            specs[f("canon" + n)] = WeightSpec((D, K), role="vector")
            specs[f("rg" + n)] = WeightSpec((D, D))
            specs[f("rg" + n + ".b")] = WeightSpec((D,), role="vector")
        return specs

    def bind(self, tensors) -> None:
        t = lambda n: tensors[self.full_name(n)]          # noqa: E731
        # the convolution's weights by tap ([taps, D], oldest first): a tap's weights of neighbouring channels lie side by side
        self.taps1, self.w_g1, self.b_g1 = t("canon1").float().t().contiguous(), t("rg1"), t("rg1.b")
        self.w_out1 = (t("norm1b") + self.out_offset).contiguous()
        if self.ffn is not None:
            self.taps2, self.w_g2, self.b_g2 = t("canon2").float().t().contiguous(), t("rg2"), t("rg2.b")
            self.w_out2 = (t("norm2b") + self.out_offset).contiguous()

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_g1, self.w_g2) if w is not None)

    def _project(self, x, w, out, rows):
        return ops.linear(x, w, out=out) if self.rt.plain_kernels else ops.project_rows(x, w, out, rows)

    def _sublayer(self, h, a, f, taps, w_gate, b_gate, w_out, hist_off, ctx, state, nxt):
        """One sublayer on the stream h, given its normed input a.  `nxt` = (weight, eps) of the norm that follows (or None);
        returns that norm's output."""
        T, D = h.shape
        ws = self.rt.workspace
        x = ops.input_conv(ws.rows("sand_in", T, D, a.dtype), a, taps, state, hist_off, ctx.seq_of_token, ctx.cu_seqlens, ctx.state_slots)
        y = f(x)
        z = self._project(a, w_gate, ws.rows("sand_gate", T, D, a.dtype), T)
        out = ws.other_of_pair("normed", a, T, D, a.dtype) if nxt is not None else None
        ops.gated_norm_add(h, y, w_out, self.eps, gate=z, gate_bias=b_gate, next_weight=nxt[0] if nxt else None,
                           next_eps=nxt[1] if nxt else 0.0, next_out=out,
                           history=(a, self.taps, state, hist_off, ctx.seq_of_token, ctx.cu_seqlens, ctx.state_slots))
        return out

    def forward(self, h, pending, ctx, cache, state):
        T, D = h.shape
        if isinstance(pending, NormedAhead) and pending.weight is self.mixer_norm.weight:
            a = pending.rows
        else:
            if pending is not None and not isinstance(pending, NormedAhead):
                ops.resid_update(h, tuple(pending) if isinstance(pending, (tuple, list)) else (pending,))
            a = self.mixer_norm.forward(h, out=self.rt.workspace.rows("normed", T, D, self.rt.dtype))
        off1 = self.mixer_floats
        ahead = ctx.extras.get("norm_ahead")          # the norm that follows this block, if the model named one
        after = (ahead.weight, ahead.eps) if getattr(ahead, "plain_rms", False) and ahead.size == D else None
        if self.ffn is None:
            a = self._sublayer(h, a, lambda x: self.mixer.forward(x, ctx, cache, state), self.taps1, self.w_g1, self.b_g1,
                               self.w_out1, off1, ctx, state, after)
        else:
            a = self._sublayer(h, a, lambda x: self.mixer.forward(x, ctx, cache, state), self.taps1, self.w_g1, self.b_g1,
                               self.w_out1, off1, ctx, state, (self.ffn_norm.weight, self.ffn_norm.eps))
            a = self._sublayer(h, a, lambda x: self.ffn.forward(x, ctx), self.taps2, self.w_g2, self.b_g2, self.w_out2,
                               off1 + (self.taps - 1) * D, ctx, state, after)
        return h, (NormedAhead(a, after[0]) if after is not None else None)
