"""Typed configuration of the Lorulix decoder, read from its ``config.json``.

Top level: ``vocab``, ``width``, ``max_positions`` (rows of the learned position table), ``norm.eps``, ``canon.taps`` (taps of the
convolution in front of every sublayer) and ``layers``, a list with one entry per layer: ``type`` (which mixer: ``attention`` or
``delta``), ``mixer`` (its sizes and constants) and ``mlp`` (``null``, a dense one with ``ff`` and ``limit``, or a mixture of
experts with ``expert.ff``, ``router.experts``, ``router.top``, ``router.scale`` and optionally ``shared.ff``).  Layers need not be
alike and come in any order.  An attention mixer may name ``kv_from``: an earlier attention layer with key and value
projections of its own whose cache entries it reads.  Every size and constant is taken from the file; a missing required
key, an unknown kind or sizes that contradict one another raise ``ConfigError``.  Optional keys that only the random-weights
writer needs: ``mixer.bias_rows`` of an attention mixer (the rows of its distance table, which a checkpoint's tensor fixes
otherwise) and ``eos_token_id``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple, Union

from .givirax_config import _get
from .model_config import ConfigError


@dataclass(frozen=True)
class BiasedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    bias_max: int
    temp_coef: float = 0.0
    temp_every: int = 0           # 0: no query temperature
    kv_from: Optional[int] = None
    bias_rows: Optional[int] = None


@dataclass(frozen=True)
class HeadDeltaConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int


@dataclass(frozen=True)
class LorulixMlpConfig:
    kind: str                     # "dense" | "moe"
    ff: int
    limit: float = 0.0            # dense: the clamp
    experts: int = 0
    top: int = 0
    scale: float = 1.0
    shared_ff: int = 0            # 0: no shared expert


@dataclass(frozen=True)
class LorulixLayerConfig:
    type: str
    mixer: Union[BiasedAttentionConfig, HeadDeltaConfig]
    mlp: Optional[LorulixMlpConfig]


@dataclass(frozen=True)
class LorulixConfig:
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    taps: int
    layers: Tuple[LorulixLayerConfig, ...]
    eos_token_ids: tuple = ()
    architecture: str = "Lorulix"

    @staticmethod
    def from_dict(d: Mapping[str, Any]) -> "LorulixConfig":
        layers = d.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        parsed = []
        for i, entry in enumerate(layers):
            where = f"layers[{i}]."
            kind = _get(entry, "type", str, where)
            m = entry.get("mixer")
            if not isinstance(m, Mapping):
                raise ConfigError(f"config.json: required key '{where}mixer' is missing")
            w = where + "mixer."
            heads = _get(m, "heads", int, w)
            kv_heads = _get(m, "kv_heads", int, w, heads, required=False)
            dim = _get(m, "dim", int, w)
            vdim = _get(m, "vdim", int, w, dim, required=False)
            if min(heads, kv_heads, dim, vdim) <= 0 or heads % kv_heads:
                raise ConfigError(f"config.json: {w}: {heads} heads over {kv_heads} key heads, sizes {dim} and {vdim}")
            if kind == "attention":
                qt = m.get("q_temp") or {}
                mixer = BiasedAttentionConfig(
                    heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=_get(m, "scale", float, w),
                    bias_max=_get(m, "bias_max", int, w),
                    temp_coef=_get(qt, "coef", float, w + "q_temp.", 0.0, required=bool(qt)),
                    temp_every=_get(qt, "every", int, w + "q_temp.", 0, required=bool(qt)),
                    kv_from=_get(m, "kv_from", int, w, None, required=False),
                    bias_rows=_get(m, "bias_rows", int, w, None, required=False))
                if mixer.bias_max < 1 or (qt and mixer.temp_every < 1):
                    raise ConfigError(f"config.json: {w}: bias_max {mixer.bias_max}, q_temp.every {mixer.temp_every}")
                if mixer.kv_from is not None:
                    j = mixer.kv_from
                    src = parsed[j].mixer if 0 <= j < i else None
                    if not isinstance(src, BiasedAttentionConfig) or src.kv_from is not None:
                        raise ConfigError(f"config.json: {w}kv_from = {j} must name an earlier attention layer that has key and "
                                          "value projections of its own")
                    if (src.kv_heads, src.dim, src.vdim) != (kv_heads, dim, vdim):
                        raise ConfigError(f"config.json: {w}kv_from = {j}: kv_heads, dim and vdim must equal that layer's")
            elif kind == "delta":
                mixer = HeadDeltaConfig(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=_get(m, "conv", int, w))
                if mixer.conv <= 0:
                    raise ConfigError(f"config.json: {w}conv: a convolution has at least one tap")
            else:
                raise ConfigError(f"config.json: {where}type '{kind}' is not a mixer of this design; known: attention, delta")
            f = entry.get("mlp")
            mlp = None
            if f is not None:
                fw = where + "mlp."
                fk = _get(f, "kind", str, fw)
                if fk == "dense":
                    mlp = LorulixMlpConfig("dense", _get(f, "ff", int, fw), limit=_get(f, "limit", float, fw))
                    if mlp.limit <= 0:
                        raise ConfigError(f"config.json: {fw}limit must be positive")
                elif fk == "moe":
                    r = f.get("router")
                    sh = f.get("shared")
                    mlp = LorulixMlpConfig("moe", _get(f.get("expert"), "ff", int, fw + "expert."),
                                           experts=_get(r, "experts", int, fw + "router."), top=_get(r, "top", int, fw + "router."),
                                           scale=_get(r, "scale", float, fw + "router.", 1.0, required=False),
                                           shared_ff=_get(sh, "ff", int, fw + "shared.") if sh is not None else 0)
                    if not (0 < mlp.top <= mlp.experts) or mlp.shared_ff < 0:
                        raise ConfigError(f"config.json: {fw}: top {mlp.top} of {mlp.experts} experts, shared size {mlp.shared_ff}")
                else:
                    raise ConfigError(f"config.json: {fw}kind '{fk}' is unknown; known: dense, moe")
                if mlp.ff <= 0:
                    raise ConfigError(f"config.json: {fw}: inner size must be positive")
            parsed.append(LorulixLayerConfig(kind, mixer, mlp))
        eos = d.get("eos_token_id")
        eos = tuple(int(x) for x in eos) if isinstance(eos, (list, tuple)) else ((int(eos),) if eos is not None else ())
        cfg = LorulixConfig(vocab=_get(d, "vocab", int, ""), width=_get(d, "width", int, ""),
                            max_positions=_get(d, "max_positions", int, ""),
                            norm_eps=_get(d.get("norm") or {}, "eps", float, "norm."),
                            taps=_get(d.get("canon") or {}, "taps", int, "canon."), layers=tuple(parsed), eos_token_ids=eos)
        if cfg.vocab <= 0 or cfg.width <= 0 or cfg.max_positions <= 0 or cfg.taps <= 0:
            raise ConfigError("config.json: vocab, width, max_positions and canon.taps must be positive")
        return cfg
