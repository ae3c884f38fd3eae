"""Parts that work on a residual stream kept in float32 under activations of any element type
(``ModelSpec.residual_dtype = "float32"``): the stream is summed in 32-bit and rounded to the activations' type only
where a norm hands it to a matrix product.

* embedding ``scaled_positions``: h = table[token] * scale + pos_table[position] (a learned vector per position; the
  position table is optional, the scale defaults to 1).
* norm ``rmsnorm_wide``: y = T(x / sqrt(mean(x^2) + eps) * w), one rounding, at the store.  ``add_forward`` takes one
  delta or a tuple of two, adds them to the stream in float (h + (d1 + d2)) and norms the sum, one kernel.
  With ``offset`` the stored weight is a distance from it (w_used = offset + w_stored; 1 for weights stored around zero).
  ``add_normed`` is the norm behind a sublayer: h <- h + norm(y [+ bias]); only the normed output joins the stream.
* embedding ``normed_tokens``: h = norm(table[token]), a norm of the embedding's own on the gathered rows.
* block ``outnorm``: h <- h + norm_m(mixer(h));  h <- h + norm_f(ffn(h)).  The sublayers read the stream itself (rounded once
  to the activations' type where that is narrower); the norms stand behind them.  A layer may have no feed-forward.
* block ``parallel``: x = norm(h);  h <- h + (mixer(x) + ffn(x)).  One norm; both sublayers read its output; a layer may
  have no feed-forward.  The two outputs leave the block as pending deltas, so that the next block's norm (or the final
  norm) adds them: a layer costs one elementwise kernel.
* input ``pass_input``: in front of pass number t of a repeated run of layers, h <- (h + embedded) + step[t] (the
  embedding output only from the second pass on); pending deltas are folded in by the same kernel.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import ops
from .base import Block, Norm, Part, StreamInput, WeightSpec, register_part


def stream_as_activations(rt, h, ctx):
    """The residual stream in the element type that matrix products read.  The kernels that change the stream leave such a
    copy beside it (see ``WideRMSNorm.add_normed``); without one it is made here."""
    if h.dtype == rt.dtype:
        return h
    have = ctx.extras.get("stream_copy")
    if have is not None and have[0] == h.data_ptr() and have[1].shape == h.shape:
        return have[1]
    out = rt.workspace.rows("stream_copy", h.shape[0], h.shape[1], rt.dtype)
    out.copy_(h)
    ctx.extras["stream_copy"] = (h.data_ptr(), out)
    return out


def _as_tuple(pending):
    if pending is None:
        return ()
    return tuple(pending) if isinstance(pending, (tuple, list)) else (pending,)


@register_part("embedding", "scaled_positions")
class ScaledPositionEmbedding(Part):
    category = "embedding"

    def __init__(self, runtime, prefix="", names=None, *, vocab_size: int, hidden_size: int, scale: float = 1.0,
                 max_positions: int = 0):
        super().__init__(runtime, prefix, names)
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.scale, self.max_positions = float(scale), int(max_positions)
        self.table = self.pos_table = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs = {self.full_name("embed"): WeightSpec((self.vocab_size, self.hidden_size))}
        if self.max_positions > 0:
            specs[self.full_name("pos")] = WeightSpec((self.max_positions, self.hidden_size))
        return specs

    def bind(self, tensors) -> None:
        self.table = tensors[self.full_name("embed")]
        if self.max_positions > 0:
            self.pos_table = tensors[self.full_name("pos")]
            if self.pos_table.dtype != self.table.dtype:
                self.table, self.pos_table = self.table.float(), self.pos_table.float()

    def forward_step(self, ctx, keep: bool = False):
        """Returns (residual stream, embedding output).  With `keep` the two are different buffers, so that the
        embedding output survives the layers."""
        T = ctx.num_tokens
        ws = self.rt.workspace
        out = ws.rows("residual", T, self.hidden_size, torch.float32)
        kept = ws.rows("embedded", T, self.hidden_size, torch.float32) if keep else None
        ops.embed_positions(out, self.table, ctx.tokens[:T], ctx.positions[:T], self.scale, self.pos_table, kept)
        return out, (kept if keep else out)


@register_part("norm", "rmsnorm_wide")
class WideRMSNorm(Norm):
    plain_rms = True          # y = x / rms(x) * self.weight with self.eps: a kernel that holds the row may apply it ahead of time

    def __init__(self, runtime, prefix="", names=None, *, size: int, eps: float, buffer: str = "normed",
                 weight_name: str = "weight", offset: float = 0.0):
        super().__init__(runtime, prefix, names)
        self.size, self.eps, self.buffer, self.weight_name = int(size), float(eps), buffer, weight_name
        self.offset = float(offset)
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.full_name(self.weight_name): WeightSpec((self.size,), role="vector", init="normal" if self.offset else "norm")}

    def bind(self, tensors) -> None:
        self.weight = tensors[self.full_name(self.weight_name)]
        if self.offset:
            self.weight = (self.weight + self.offset).contiguous()

    def add_normed(self, h, y, ctx, bias=None):
        """h <- h + norm(y + bias) * w, in place; returns the new stream in the activations' type."""
        T, D = h.shape
        copy = self.rt.workspace.rows("stream_copy", T, D, self.rt.dtype) if h.dtype != self.rt.dtype else None
        ops.norm_add(h, y, self.weight, self.eps, bias=bias, accumulate=True, copy=copy)
        if copy is None:
            return h
        ctx.extras["stream_copy"] = (h.data_ptr(), copy)
        return copy

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def _out(self, x, out):
        return out if out is not None else self.rt.workspace.rows(self.buffer, x.shape[0], self.size, self.rt.dtype)

    def forward(self, x, out=None):
        return ops.resid_update(x, (), norm_weight=self.weight, eps=self.eps, out=self._out(x, out))

    def add_forward(self, residual, delta, out=None):
        return ops.resid_update(residual, _as_tuple(delta), norm_weight=self.weight, eps=self.eps, out=self._out(residual, out))


@register_part("embedding", "normed_tokens")
class NormedTokenEmbedding(Part):
    category = "embedding"

    def __init__(self, runtime, prefix="", names=None, *, vocab_size: int, hidden_size: int, eps: float, offset: float = 0.0,
                 table_name: str = "embed", norm_name: str = "embed.norm"):
        super().__init__(runtime, prefix, names)
        self.vocab_size, self.hidden_size, self.eps, self.offset = int(vocab_size), int(hidden_size), float(eps), float(offset)
        self.table_name, self.norm_name = table_name, norm_name
        self.table = self.weight = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.full_name(self.table_name): WeightSpec((self.vocab_size, self.hidden_size)),
                self.full_name(self.norm_name): WeightSpec((self.hidden_size,), role="vector", init="normal" if self.offset else "norm")}

    def bind(self, tensors) -> None:
        self.table = tensors[self.full_name(self.table_name)]
        self._gather_table = self.table if self.table.dtype == self.rt.dtype else self.table.to(self.rt.dtype)
        self.weight = (tensors[self.full_name(self.norm_name)] + self.offset).contiguous()

    def forward_step(self, ctx, keep: bool = False):
        T, D = ctx.num_tokens, self.hidden_size
        ws = self.rt.workspace
        rows = ops.embed(ws.rows("embed_rows", T, D, self.rt.dtype), self._gather_table, ctx.tokens[:T])
        h = ws.rows("residual", T, D, torch.float32)
        copy = ws.rows("stream_copy", T, D, self.rt.dtype) if self.rt.dtype != torch.float32 else None
        ops.norm_add(h, rows, self.weight, self.eps, accumulate=False, copy=copy)
        if copy is not None:
            ctx.extras["stream_copy"] = (h.data_ptr(), copy)
        kept = h
        if keep:
            kept = ws.rows("embedded", T, D, torch.float32)
            kept.copy_(h)
        return h, kept


@register_part("block", "outnorm")
class OutNormBlock(Block):
    def __init__(self, runtime, prefix="", names=None, *, mixer, ffn, mixer_norm, ffn_norm=None):
        super().__init__(runtime, prefix, names)
        if (ffn is None) != (ffn_norm is None):
            raise ValueError("a feed-forward and the norm behind it come together")
        for n in (mixer_norm, ffn_norm):
            if n is not None and not hasattr(n, "add_normed"):
                raise ValueError("the norms of this block stand behind the sublayers: they need add_normed")
        self.mixer, self.ffn, self.mixer_norm, self.ffn_norm = mixer, ffn, mixer_norm, ffn_norm

    def parts(self):
        return tuple(p for p in (self.mixer, self.mixer_norm, self.ffn, self.ffn_norm) if p is not None)

    def forward(self, h, pending, ctx, cache, state):
        if pending is not None:
            ops.resid_update(h, _as_tuple(pending))
            ctx.extras.pop("stream_copy", None)
        x = stream_as_activations(self.rt, h, ctx)
        x = self.mixer_norm.add_normed(h, self.mixer.forward(x, ctx, cache, state), ctx)
        if self.ffn is not None:
            split = getattr(self.ffn, "forward_unbiased", None)       # the output bias rides along into the norm's kernel
            y, bias = split(x, ctx) if split is not None else (self.ffn.forward(x, ctx), None)
            self.ffn_norm.add_normed(h, y, ctx, bias=bias)
        return h, None


@register_part("block", "parallel")
class ParallelBlock(Block):
    def __init__(self, runtime, prefix="", names=None, *, mixer, ffn, mixer_norm, ffn_norm=None):
        super().__init__(runtime, prefix, names)
        if ffn_norm is not None:
            raise ValueError("a parallel block has one norm; its sublayers share it")
        self.mixer, self.ffn, self.norm = mixer, ffn, mixer_norm

    def parts(self):
        return tuple(p for p in (self.norm, self.mixer, self.ffn) if p is not None)

    def forward(self, h, pending, ctx, cache, state):
        x = self.norm.forward(h) if pending is None else self.norm.add_forward(h, pending)
        a = self.mixer.forward(x, ctx, cache, state)
        if self.ffn is None:
            return h, a
        return h, (a, self.ffn.forward(x, ctx))


@register_part("input", "pass_input")
class PassInput(StreamInput):
    def __init__(self, runtime, prefix="", names=None, *, hidden_size: int, times: int, weight_name: str = "step",
                 embedding_from: int = 1):
        super().__init__(runtime, prefix, names)
        self.hidden_size, self.times, self.weight_name = int(hidden_size), int(times), weight_name
        self.embedding_from = int(embedding_from)         # the embedding output is added from this pass on
        self.steps: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.full_name(self.weight_name): WeightSpec((self.times, self.hidden_size), role="vector")}

    def bind(self, tensors) -> None:
        self.steps = tensors[self.full_name(self.weight_name)]

    def weight_bytes(self) -> int:
        return self.hidden_size * self.steps.element_size()

    def forward(self, h, pending, embedded, index: int):
        if not (0 <= index < self.times):
            raise ValueError(f"pass {index} of {self.times}")
        rows = embedded if index >= self.embedding_from else None
        if rows is not None and rows.data_ptr() == h.data_ptr():
            raise ValueError("the embedding output was not kept apart from the residual stream")
        ops.resid_update(h, _as_tuple(pending), rows=rows, vector=self.steps[index])
        return h, None
