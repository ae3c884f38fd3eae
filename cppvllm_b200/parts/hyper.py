"""Parts of a model whose residual stream is several copies ("streams", hyper-connections) in float32:

    X = [x_1 .. x_S], every x_s = table[token] at the start.  A sublayer f with learned numbers a[S] (read), M[S, S] (from, to)
    and b[S] (write) and an RMS norm with ONE weight g:
        u = sum_s a_s x_s;   y = f(g * u / sqrt(mean(u^2) + eps));   x_t <- sum_s M[s, t] x_s + b_t y     (all t from the old X)
    At the end the streams are added up and normed once more.

* embedding ``token_streams``: the stream tensor [T, S * D] (stream s of a token in columns s D .. s D + D - 1).
* norm ``rmsnorm_scalar``: the norm with one weight (a tensor with a single element).  Called on the stream tensor it reads
  with a = 1: the sum of the streams, normed (the model's last norm).
* block ``hyper``: a layer = the mixer's sublayer, then the feed-forward's (a layer may have none).  A sublayer's write and the
  next sublayer's read and norm are ONE kernel (csrc/hyper.cu): the block hands its last write on as ``pending`` when the next
  block is of this kind, so a layer costs two passes over the streams.  With ``streams`` = 1 and ``learned = False`` the numbers
  are a = M = b = 1: the plain pre-norm residual sum in float32.

Every number is a parameter or a tensor; S is bounded by the kernel (8).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch

from ..csrc import ops
from .base import Block, Norm, Part, WeightSpec, register_part


@dataclass
class StreamWrite:
    """A sublayer's output (a tensor, or two that are to be added) that has not been written into the streams yet."""
    y: object
    mix: torch.Tensor
    out: torch.Tensor
    streams: int


@register_part("embedding", "token_streams")
class TokenStreams(Part):
    category = "embedding"

    def __init__(self, runtime, prefix="", names=None, *, vocab_size: int, hidden_size: int, streams: int = 1, table_name: str = "embed"):
        super().__init__(runtime, prefix, names)
        self.vocab_size, self.hidden_size, self.streams, self.table_name = int(vocab_size), int(hidden_size), int(streams), table_name
        self.table = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.full_name(self.table_name): WeightSpec((self.vocab_size, self.hidden_size))}

    def bind(self, tensors) -> None:
        self.table = tensors[self.full_name(self.table_name)]

    def forward_step(self, ctx, keep: bool = False):
        T = ctx.num_tokens
        X = self.rt.workspace.rows("residual", T, self.streams * self.hidden_size, torch.float32)
        ops.stream_embed(X, self.table, ctx.tokens[:T], self.streams)
        return X, X


@register_part("norm", "rmsnorm_scalar")
class ScalarRMSNorm(Norm):
    def __init__(self, runtime, prefix="", names=None, *, size: int, eps: float, streams: int = 1, buffer: str = "normed",
                 weight_name: str = "weight"):
        super().__init__(runtime, prefix, names)
        self.size, self.eps, self.streams, self.buffer, self.weight_name = int(size), float(eps), int(streams), buffer, weight_name
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.full_name(self.weight_name): WeightSpec((), role="vector", init="norm")}

    def bind(self, tensors) -> None:
        self.weight = tensors[self.full_name(self.weight_name)].reshape(1).contiguous()

    def weight_bytes(self) -> int:
        return 4

    def forward(self, x, out=None):
        """x: the stream tensor [T, S * D]; out [T, D] = the norm of the sum of the streams."""
        if out is None:
            out = self.rt.workspace.rows(self.buffer, x.shape[0], self.size, self.rt.dtype)
        return ops.stream_step(x, self.streams, read=(None, self.weight), eps=self.eps, out=out)

    def add_forward(self, residual, delta, out=None):
        raise NotImplementedError("a sublayer's output joins the streams through the block's own weights, not through this norm")


@register_part("block", "hyper")
class HyperBlock(Block):
    accepts_normed_ahead = True         # the model then names this block's first norm to the block in front of it

    def __init__(self, runtime, prefix="", names=None, *, mixer, ffn, mixer_norm, ffn_norm=None, hidden_size: int, streams: int = 1,
                 learned: bool = True, mixer_name: str = "hc1.", ffn_name: str = "hc2."):
        super().__init__(runtime, prefix, names)
        if (ffn is None) != (ffn_norm is None):
            raise ValueError("a feed-forward and the norm in front of it come together")
        for n in (mixer_norm, ffn_norm):
            if n is not None and not isinstance(n, ScalarRMSNorm):
                raise ValueError("the sublayers of this block read the streams through a norm with one weight (rmsnorm_scalar)")
        self.mixer, self.ffn, self.mixer_norm, self.ffn_norm = mixer, ffn, mixer_norm, ffn_norm
        self.hidden_size, self.streams, self.learned = int(hidden_size), int(streams), bool(learned)
        if not self.learned and self.streams != 1:
            raise ValueError("several streams need learned weights")
        self.mixer_name, self.ffn_name = mixer_name, ffn_name
        self.mixer_norm.first_of_hyper_block = True
        self.w = {}

    def parts(self):
        return tuple(p for p in (self, self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if p is not None)

    def _sub_names(self):
        return [self.mixer_name] + ([self.ffn_name] if self.ffn is not None else [])

    def weight_specs(self) -> Dict[str, WeightSpec]:
        if not self.learned:
            return {}
        S, specs = self.streams, {}
        for sub in self._sub_names():
            specs[self.full_name(sub + "in")] = WeightSpec((S,), role="vector", init="norm")
            specs[self.full_name(sub + "out")] = WeightSpec((S,), role="vector", init="norm")
            specs[self.full_name(sub + "mix")] = WeightSpec((S, S), role="vector", init="eye")
        return specs

    def bind(self, tensors) -> None:
        for sub in self._sub_names():
            if self.learned:
                self.w[sub] = tuple(tensors[self.full_name(sub + k)].contiguous() for k in ("in", "mix", "out"))
            else:
                one = torch.ones(1, dtype=torch.float32, device=self.rt.device)
                self.w[sub] = (one, one, one)

    def weight_bytes(self) -> int:
        return sum(t.numel() * 4 for ws in self.w.values() for t in ws) if self.learned else 0

    def forward(self, X, pending, ctx, cache, state):
        T, D, S = ctx.num_tokens, self.hidden_size, self.streams
        ws = self.rt.workspace
        if pending is not None and not isinstance(pending, StreamWrite):
            raise ValueError("a block in front of this one left a delta that only its own kind of stream can take")
        a1, m1, b1 = self.w[self.mixer_name]
        x = ws.rows(self.mixer_norm.buffer, T, D, self.rt.dtype)
        ops.stream_step(X, S, write=(pending.y, pending.mix, pending.out) if pending is not None else None,
                        read=(a1, self.mixer_norm.weight), eps=self.mixer_norm.eps, out=x)
        y = self.mixer.forward(x, ctx, cache, state)
        last = StreamWrite(y, m1, b1, S)
        if self.ffn is not None:
            a2, m2, b2 = self.w[self.ffn_name]
            x = ws.rows(self.ffn_norm.buffer, T, D, self.rt.dtype)
            ops.stream_step(X, S, write=(y, m1, b1), read=(a2, self.ffn_norm.weight), eps=self.ffn_norm.eps, out=x)
            ctx.extras["takes_two_outputs"] = True      # a feed-forward may hand back (routed, shared): added in float by the write
            last = StreamWrite(self.ffn.forward(x, ctx), m2, b2, S)
            ctx.extras.pop("takes_two_outputs", None)
        ahead = ctx.extras.get("norm_ahead")
        if ahead is not None and getattr(ahead, "first_of_hyper_block", False) and getattr(ahead, "streams", S) == S:
            return X, last                              # the next block's first kernel does the write
        ops.stream_step(X, S, write=(last.y, last.mix, last.out))
        return X, None
