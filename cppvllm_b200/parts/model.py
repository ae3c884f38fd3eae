"""The generic causal language model: an embedding, a run list of blocks, a final norm and an output head,
all built from a ``ModelSpec`` through the part registry.  It holds no architecture-specific code; an
architecture contributes only its spec (see models/qwen3.py).

``forward(ctx, caches, states)`` runs exactly the tokens of the step, reading and writing the cache units it is
given, and returns float32 logits for the rows listed in ``ctx.logit_rows`` (any tokens of the step, not only
last ones; the reference computes one row per sequence whether it samples or not, model_architecture.cpp:232-235).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..csrc import ops
from .base import CacheSpec, Runtime, StateSpec, WeightSpec, build_part, part_class
from .spec import ModelSpec, RunEntry


class CausalLM:
    def __init__(self, spec: ModelSpec, runtime: Runtime):
        self.spec, self.rt = spec, runtime
        self.hidden_size, self.vocab_size = spec.hidden_size, spec.vocab_size
        self.positions = {name: build_part("position", ps, runtime) for name, ps in spec.positions.items()}
        self.embedding = build_part("embedding", spec.embedding, runtime)
        self.blocks = []
        for ls in spec.layers:
            mixer_extra = {}
            mparams = dict(ls.mixer.params)
            pos_name = mparams.pop("position", None)
            mixer_cls = part_class("mixer", ls.mixer.kind)
            if pos_name is not None:
                if pos_name not in self.positions:
                    raise ValueError(f"mixer names position encoding '{pos_name}', which the spec does not define")
                mixer_extra["position"] = self.positions[pos_name]
            mixer = mixer_cls(runtime, prefix=ls.mixer.prefix, names=dict(ls.mixer.names), **mparams, **mixer_extra)
            ffn = build_part("ffn", ls.ffn, runtime) if ls.ffn is not None else None
            mixer_norm = build_part("norm", ls.mixer_norm, runtime)
            ffn_norm = build_part("norm", ls.ffn_norm, runtime) if ls.ffn_norm is not None else None
            block_cls = part_class("block", ls.block)
            self.blocks.append(block_cls(runtime, mixer=mixer, ffn=ffn, mixer_norm=mixer_norm, ffn_norm=ffn_norm,
                                         **ls.block_params))
        self.inputs = {name: build_part("input", ps, runtime) for name, ps in spec.inputs.items()}
        self.final_norm = build_part("norm", spec.final_norm, runtime)
        self.head = build_part("head", spec.lm_head, runtime)
        self.run_order: List[RunEntry] = spec.resolved_run_order()
        self._check_shared_caches()

    @property
    def capturable(self) -> bool:
        return all(p.capturable for p in self.all_parts())

    # ---- what the model keeps between steps ------------------------------------------------------------
    def cache_units(self) -> Dict[int, CacheSpec]:
        """cache unit id -> spec, taken from the mixer of the entry that writes the unit."""
        units = {}
        for e in self.run_order:
            cs = self.blocks[e.layer].mixer.cache_spec()
            if cs is not None and e.writes_cache:
                units[e.cache] = cs
        return units

    def state_specs(self) -> List[Optional[StateSpec]]:
        """One entry per item of the run list: the fixed-size per-request state its mixer wants, or None.  A block that keeps
        state of its own (``state_spec()`` on the block) answers for its mixer too."""
        out = []
        for e in self.run_order:
            b = self.blocks[e.layer]
            own = getattr(b, "state_spec", None)
            out.append(own() if own is not None else b.mixer.state_spec())
        return out

    def _check_shared_caches(self) -> None:
        units = self.cache_units()
        for e in self.run_order:
            cs = self.blocks[e.layer].mixer.cache_spec()
            if cs is None or e.writes_cache:
                continue
            w = units.get(e.cache)
            if w is None or (w.entry_shape, w.token_axis) != (cs.entry_shape, cs.token_axis):
                raise ValueError(f"layer {e.layer} reads cache unit {e.cache}, whose entries have another shape")

    # ---- weights -------------------------------------------------------------------------------------
    def all_parts(self):
        yield self.embedding
        for b in self.blocks:
            yield from b.parts()
        yield self.final_norm
        yield self.head
        yield from self.positions.values()
        yield from self.inputs.values()

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs: Dict[str, WeightSpec] = {}
        for p in self.all_parts():
            for name, ws in p.weight_specs().items():
                if name in specs and specs[name].shape != ws.shape:
                    raise ValueError(f"tensor '{name}' is declared with shapes {specs[name].shape} and {ws.shape}")
                specs.setdefault(name, ws)
        return specs

    def ignorable_weights(self):
        """Tensors a checkpoint may hold although the model does not read them: the head's own table when
        the head is tied to the embedding."""
        own = self.spec.lm_head.prefix + "weight"
        return [own] if self.head.full_name("weight") != own else []

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self.all_parts():
            p.bind(tensors)

    def decode_weight_bytes(self) -> int:
        """Bytes of weights one decode step reads: every run entry's layer once (a layer run twice is read
        twice), the final norm and the head; the embedding table only as the head when tied."""
        total = 0
        for e in self.run_order:
            total += sum(p.weight_bytes() for p in self.blocks[e.layer].parts())
            if e.input is not None:
                total += self.inputs[e.input].weight_bytes()
        return total + self.final_norm.weight_bytes() + self.head.weight_bytes()

    # ---- step ----------------------------------------------------------------------------------------
    def forward_hidden(self, ctx, caches, states):
        positioned = getattr(self.embedding, "forward_step", None)     # an embedding that also reads the positions
        if positioned is not None:
            h, embedded = positioned(ctx, keep=bool(self.inputs))
        else:
            h = embedded = self.embedding.forward(ctx.tokens, ctx.num_tokens)
        pending = None
        last = len(self.run_order) - 1
        for i, e in enumerate(self.run_order):
            if e.input is not None:
                h, pending = self.inputs[e.input].forward(h, pending, embedded, e.input_index)
            # the norm that reads the stream next: a block that holds the new row on the chip may apply it ahead of time
            if i == last:
                ctx.extras["norm_ahead"] = self.final_norm
            else:
                nxt = self.run_order[i + 1]
                nb = self.blocks[nxt.layer]
                takes = nxt.input is None and getattr(nb, "accepts_normed_ahead", False)
                ctx.extras["norm_ahead"] = nb.mixer_norm if takes else None
            h, pending = self.blocks[e.layer].forward(h, pending, ctx, caches.get(i), states.get(i))
        return h, pending

    def forward(self, ctx, caches, states, logits_out: torch.Tensor) -> torch.Tensor:
        h, pending = self.forward_hidden(ctx, caches, states)
        R = ctx.num_logit_rows
        ws = self.rt.workspace
        normed = ws.rows("head_normed", R, self.hidden_size, self.rt.dtype)
        if getattr(pending, "weight", None) is not None and pending.weight is getattr(self.final_norm, "weight", None):
            # the last block has applied the final norm already: only the wanted rows are picked
            return self.head.forward(ops.gather_rows(normed, pending.rows, ctx.logit_rows), logits_out[:R])
        rows_h = ops.gather_rows(ws.rows("head_rows", R, h.shape[1], h.dtype), h, ctx.logit_rows)     # several streams: a wider row
        if isinstance(pending, tuple):               # several deltas (a block whose sublayers run side by side)
            rows_p = tuple(ops.gather_rows(ws.rows(f"head_pending{i}", R, self.hidden_size, p.dtype), p, ctx.logit_rows)
                           for i, p in enumerate(pending))
            self.final_norm.add_forward(rows_h, rows_p, out=normed)
        elif pending is not None:
            rows_p = ops.gather_rows(ws.rows("head_pending", R, self.hidden_size, pending.dtype), pending, ctx.logit_rows)
            self.final_norm.add_forward(rows_h, rows_p, out=normed)
        else:
            self.final_norm.forward(rows_h, out=normed)
        return self.head.forward(normed, logits_out[:R])
