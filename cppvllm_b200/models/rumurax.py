"""Rumurax as data: the typed configuration becomes a ``ModelSpec``.

A decoder-only model whose residual stream is several copies in 32-bit that every sublayer reads through learned weights and
writes back through a learned matrix (block ``hyper``, parts/hyper.py), with norms of ONE weight.  Layers come in any order
with one of three mixers: grouped-query attention without rotation inside chunks of positions, with capped scores, a
logarithmic distance term, a sink in the softmax and a gate per head; grouped-query attention with a rotation behind a
sliding window with pooled blocks of older tokens (both: mixer ``masked_attention``; both may mix their values with those of
the first such layer); and attention over a cached latent with queries of their own and a gate per element (mixer
``latent_attention``).  The feed-forward is absent or a mixture of gated experts with logistic scores that multiply the experts'
inputs, plus an optional shared expert (``routed_glu``).  Tensor names: ``embed``, ``l<i>.norm1|norm2``, ``l<i>.hc1|hc2.in|out|mix``,
``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.rumurax_config import LatentAttentionConfig, RumuraxConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec


def build_rumurax_spec(cfg: RumuraxConfig) -> ModelSpec:
    D, eps = cfg.width, cfg.norm_eps
    S = max(1, cfg.streams)
    layers, positions = [], {}

    def rotation(dims: int, base: float):
        if not dims:
            return None
        name = f"rot{dims}_{base!r}"
        positions.setdefault(name, PartSpec("rotary", dict(rotary_dim=dims, theta=base, max_positions=0, pairing="interleaved")))
        return name

    mixes_seen = False
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        if isinstance(m, LatentAttentionConfig):
            params = dict(hidden_size=D, num_heads=m.heads, nope_dim=m.dim, rot_dim=m.rot_dim, value_dim=m.vdim, q_rank=0,
                          kv_rank=m.kv_rank, scale=m.scale, eps=eps, gate="element", position=rotation(m.rot_dims, m.rot_base))
            if params["position"] is None:      # nothing turns: tables of no width would not do, so a rotation by base 1 of 0 elements is left out
                raise ValueError(f"layer {i}: latent attention needs rot.dims > 0")
            mixer = PartSpec("latent_attention", params, prefix=p + "mix.")
        else:
            gated = layer.type == "attention"
            params = dict(hidden_size=D, num_heads=m.heads, num_kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim, scale=m.scale, eps=eps,
                          chunk=m.chunk, window=m.window, pool=m.pool, softcap=m.softcap, distance_bias=gated, sink=gated,
                          head_gate=gated, v_mix="none" if not m.v_mix else ("mix" if mixes_seen else "first"))
            pos = rotation(m.rot_dims, m.rot_base)
            if pos is not None:
                params["position"] = pos
            mixes_seen = mixes_seen or m.v_mix
            mixer = PartSpec("masked_attention", params, prefix=p + "mix.")
        ffn = ffn_norm = None
        f = layer.mlp
        if f is not None:
            ffn = PartSpec("routed_glu", dict(hidden_size=D, intermediate_size=f.ff, num_experts=f.experts, top=f.top, score="sigmoid",
                                              weight_on_input=True, router_bias=False, shared_size=f.shared_ff), prefix=p + "mlp.")
            ffn_norm = PartSpec("rmsnorm_scalar", dict(size=D, eps=eps, streams=S, weight_name="norm2"), prefix=p)
        layers.append(LayerSpec(mixer=mixer, ffn=ffn,
                                mixer_norm=PartSpec("rmsnorm_scalar", dict(size=D, eps=eps, streams=S, weight_name="norm1"), prefix=p),
                                ffn_norm=ffn_norm, block="hyper",
                                block_params=dict(prefix=p, hidden_size=D, streams=S, learned=cfg.streams > 0)))
    return ModelSpec(
        architecture=cfg.architecture,
        hidden_size=D,
        vocab_size=cfg.vocab,
        embedding=PartSpec("token_streams", dict(vocab_size=cfg.vocab, hidden_size=D, streams=S)),
        layers=layers,
        final_norm=PartSpec("rmsnorm_scalar", dict(size=D, eps=eps, streams=S, buffer="head_normed", weight_name="norm"), prefix="final."),
        lm_head=PartSpec("lm_head", dict(vocab_size=cfg.vocab, hidden_size=D), names={"weight": "head"}),
        positions=positions,
        eos_token_ids=tuple(cfg.eos_token_ids),
        residual_dtype="float32",
    )


register_architecture("Rumurax", RumuraxConfig.from_dict, build_rumurax_spec, model_types=("rumurax",), replace=True, builtin=True)
