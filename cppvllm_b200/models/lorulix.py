"""Lorulix as data: the typed configuration becomes a ``ModelSpec``.

A decoder-only model with a residual stream summed in 32-bit.  The embedding row and a learned position vector are added.
Every sublayer stands between two RMS norms whose weights are stored around zero (1 + w is used), reads its input through a
short causal convolution (block ``sandwich``) and leaves through a learned gate.  Layers come in any order with one of two
mixers: grouped-query attention without rotation (a norm over the whole query and key projections, a temperature on the
queries that grows with the position, a learned bias per head and distance bucket; optionally reading the keys and values
of an earlier layer), or a gated delta rule with one decay per head and short convolutions.  The feed-forward is absent, dense
(gated, with clamps) or a mixture of squared-relu experts with an optional shared expert.  Tensor names: ``embed``, ``pos``,
``l<i>.norm1|norm1b|norm2|norm2b``, ``l<i>.canon1|canon2``, ``l<i>.rg1|rg2`` (+ ``.b``), ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``,
``head``.
"""
from __future__ import annotations

from ..config.lorulix_config import LorulixConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry


def build_lorulix_spec(cfg: LorulixConfig) -> ModelSpec:
    D, eps = cfg.width, cfg.norm_eps
    layers, order = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        entry = RunEntry(i)
        if layer.type == "attention":
            mixer = PartSpec("biased_attention", dict(
                hidden_size=D, num_heads=m.heads, num_kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim, scale=m.scale, eps=eps,
                bias_max=m.bias_max, bias_rows=m.bias_rows or -1, temp_coef=m.temp_coef, temp_every=m.temp_every,
                reads_other_cache=m.kv_from is not None), prefix=p + "mix.")
            # cache units are numbered by the layer that writes them
            entry = RunEntry(i, cache=i if m.kv_from is None else m.kv_from, writes_cache=m.kv_from is None)
        else:
            mixer = PartSpec("head_delta", dict(hidden_size=D, num_heads=m.heads, num_kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim,
                                                taps=m.conv, eps=eps), prefix=p + "mix.")
        ffn = ffn_norm = None
        f = layer.mlp
        if f is not None:
            if f.kind == "dense":
                ffn = PartSpec("clamped_glu", dict(hidden_size=D, intermediate_size=f.ff, limit=f.limit), prefix=p + "mlp.")
            else:
                ffn = PartSpec("routed_act", dict(hidden_size=D, intermediate_size=f.ff, num_experts=f.experts, top=f.top,
                                                  scale=f.scale, activation="relu2", shared_size=f.shared_ff), prefix=p + "mlp.")
            ffn_norm = PartSpec("rmsnorm_wide", dict(size=D, eps=eps, weight_name="norm2", offset=1.0), prefix=p)
        layers.append(LayerSpec(mixer=mixer, ffn=ffn,
                                mixer_norm=PartSpec("rmsnorm_wide", dict(size=D, eps=eps, weight_name="norm1", offset=1.0), prefix=p),
                                ffn_norm=ffn_norm, block="sandwich",
                                block_params=dict(prefix=p, hidden_size=D, taps=cfg.taps, eps=eps, out_offset=1.0)))
        order.append(entry)
    return ModelSpec(
        architecture=cfg.architecture,
        hidden_size=D,
        vocab_size=cfg.vocab,
        embedding=PartSpec("scaled_positions", dict(vocab_size=cfg.vocab, hidden_size=D, scale=1.0, max_positions=cfg.max_positions)),
        layers=layers,
        final_norm=PartSpec("rmsnorm_wide", dict(size=D, eps=eps, buffer="head_normed", weight_name="norm", offset=1.0), prefix="final."),
        lm_head=PartSpec("lm_head", dict(vocab_size=cfg.vocab, hidden_size=D), names={"weight": "head"}),
        run_order=order,
        max_positions=cfg.max_positions,
        eos_token_ids=tuple(cfg.eos_token_ids),
        residual_dtype="float32",
    )


register_architecture("Lorulix", LorulixConfig.from_dict, build_lorulix_spec, model_types=("lorulix",), replace=True, builtin=True)
