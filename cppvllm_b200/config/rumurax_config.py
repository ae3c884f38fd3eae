"""Typed configuration of the Rumurax decoder, read from its ``config.json``.

Top level: ``vocab``, ``width``, ``norm.eps``, ``streams`` (copies of the residual stream; absent: one plain stream without
learned stream weights) and ``layers``, a list with one entry per layer: ``type`` (which mixer: ``attention``, ``attention_2`` or
``latent_attention``), ``mixer`` (its sizes and constants) and ``mlp`` (``null``, or a mixture of experts with ``expert.ff``,
``router.experts``, ``router.top`` and optionally ``shared.ff``).  Layers need not be alike and come in any order.

* ``attention``: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``mask.size`` (positions per chunk), ``softcap``, ``v_mix``.
* ``attention_2``: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``mask.size`` (the window), ``mask.pool`` (positions per pooled
  block), ``rot.dims``, ``rot.base``, ``v_mix``.
* ``latent_attention``: ``heads``, ``dim`` (unrotated), ``rot_dim``, ``vdim``, ``kv_rank``, ``scale``, ``rot.dims``, ``rot.base``.

Optional keys (``softcap``, ``mask``, ``mask.pool``, ``rot``, ``v_mix``, ``shared``) switch their mechanism off when absent.  Every
size and constant is taken from the file; a missing required key, an unknown kind or sizes that contradict one another raise
``ConfigError``.  ``eos_token_id`` is optional.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple, Union

from .givirax_config import _get
from .model_config import ConfigError


@dataclass(frozen=True)
class MaskedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    chunk: int = 0                # "attention": positions per chunk (0: all earlier positions)
    window: int = 0               # "attention_2": the window (0: all earlier positions)
    pool: int = 0                 # "attention_2": positions per pooled block behind the window (0: none)
    softcap: float = 0.0          # 0: no cap
    rot_dims: int = 0             # 0: no rotation
    rot_base: float = 10000.0
    v_mix: bool = False


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_dims: int
    rot_base: float


@dataclass(frozen=True)
class RumuraxMlpConfig:
    ff: int
    experts: int
    top: int
    shared_ff: int = 0            # 0: no shared expert


@dataclass(frozen=True)
class RumuraxLayerConfig:
    type: str
    mixer: Union[MaskedAttentionConfig, LatentAttentionConfig]
    mlp: Optional[RumuraxMlpConfig]


def _rotation(m: Mapping[str, Any], where: str, limit: int):
    rot = m.get("rot")
    if rot is None:
        return 0, 10000.0
    dims = _get(rot, "dims", int, where + "rot.")
    base = _get(rot, "base", float, where + "rot.")
    if dims < 0 or dims % 2 or dims > limit or base <= 0:
        raise ConfigError(f"config.json: {where}rot: {dims} turned elements of {limit}, base {base}")
    return dims, base


@dataclass(frozen=True)
class RumuraxConfig:
    vocab: int
    width: int
    norm_eps: float
    streams: int                  # 0: the key is absent (one stream, no learned stream weights)
    layers: Tuple[RumuraxLayerConfig, ...]
    eos_token_ids: tuple = ()
    architecture: str = "Rumurax"

    @staticmethod
    def from_dict(d: Mapping[str, Any]) -> "RumuraxConfig":
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
            dim = _get(m, "dim", int, w)
            vdim = _get(m, "vdim", int, w, dim, required=False)
            scale = _get(m, "scale", float, w)
            if kind in ("attention", "attention_2"):
                kv_heads = _get(m, "kv_heads", int, w, heads, required=False)
                if min(heads, kv_heads, dim, vdim) <= 0 or heads % kv_heads:
                    raise ConfigError(f"config.json: {w}: {heads} heads over {kv_heads} key heads, sizes {dim} and {vdim}")
                mask = m.get("mask") or {}
                size = _get(mask, "size", int, w + "mask.", 0, required=False)
                pool = _get(mask, "pool", int, w + "mask.", 0, required=False)
                rot_dims, rot_base = _rotation(m, w, dim) if kind == "attention_2" else (0, 10000.0)
                if size < 0 or pool < 0 or (pool and not size):
                    raise ConfigError(f"config.json: {w}mask: size {size}, pool {pool}")
                mixer = MaskedAttentionConfig(
                    heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale,
                    chunk=size if kind == "attention" else 0, window=size if kind == "attention_2" else 0,
                    pool=pool if kind == "attention_2" else 0,
                    softcap=_get(m, "softcap", float, w, 0.0, required=False) if kind == "attention" else 0.0,
                    rot_dims=rot_dims, rot_base=rot_base, v_mix=bool(m.get("v_mix", False)))
                if mixer.softcap < 0:
                    raise ConfigError(f"config.json: {w}softcap cannot be negative")
            elif kind == "latent_attention":
                rot_dim = _get(m, "rot_dim", int, w)
                kv_rank = _get(m, "kv_rank", int, w)
                if min(heads, dim, vdim, kv_rank) <= 0 or rot_dim < 0:
                    raise ConfigError(f"config.json: {w}: {heads} heads, sizes {dim}, {rot_dim}, {vdim}, latent {kv_rank}")
                rot_dims, rot_base = _rotation(m, w, rot_dim)
                mixer = LatentAttentionConfig(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, scale=scale,
                                              rot_dims=rot_dims, rot_base=rot_base)
            else:
                raise ConfigError(f"config.json: {where}type '{kind}' is not a mixer of this design; known: attention, "
                                  "attention_2, latent_attention")
            f = entry.get("mlp")
            mlp = None
            if f is not None:
                fw = where + "mlp."
                fk = _get(f, "kind", str, fw, "moe", required=False)
                if fk != "moe":
                    raise ConfigError(f"config.json: {fw}kind '{fk}' is unknown; known: moe")
                r, sh = f.get("router"), f.get("shared")
                mlp = RumuraxMlpConfig(ff=_get(f.get("expert"), "ff", int, fw + "expert."),
                                       experts=_get(r, "experts", int, fw + "router."), top=_get(r, "top", int, fw + "router."),
                                       shared_ff=_get(sh, "ff", int, fw + "shared.") if sh is not None else 0)
                if mlp.ff <= 0 or not (0 < mlp.top <= mlp.experts) or mlp.shared_ff < 0:
                    raise ConfigError(f"config.json: {fw}: inner size {mlp.ff}, top {mlp.top} of {mlp.experts} experts, "
                                      f"shared size {mlp.shared_ff}")
            parsed.append(RumuraxLayerConfig(kind, mixer, mlp))
        mixing = [l.mixer for l in parsed if isinstance(l.mixer, MaskedAttentionConfig) and l.mixer.v_mix]
        if len({(x.kv_heads, x.vdim) for x in mixing}) > 1:
            raise ConfigError("config.json: layers that mix their values with the first such layer's need its kv_heads and vdim")
        eos = d.get("eos_token_id")
        eos = tuple(int(x) for x in eos) if isinstance(eos, (list, tuple)) else ((int(eos),) if eos is not None else ())
        cfg = RumuraxConfig(vocab=_get(d, "vocab", int, ""), width=_get(d, "width", int, ""),
                            norm_eps=_get(d.get("norm") or {}, "eps", float, "norm."),
                            streams=_get(d, "streams", int, "", 0, required=False), layers=tuple(parsed), eos_token_ids=eos)
        if cfg.vocab <= 0 or cfg.width <= 0 or cfg.streams < 0 or cfg.streams > 8:
            raise ConfigError("config.json: vocab and width must be positive, streams between 1 and 8")
        return cfg
