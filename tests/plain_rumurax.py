"""Plain, slow implementation of the Rumurax decoder: whole sequences, no cache, no batching, one function per mechanism,
float64 on the CPU.  It shares no code with the package under test: its own config.json reading, its own safetensors
reading and its own arithmetic.  In this file's notation (rms_e(x) = sqrt(mean(x^2) + e), sg = logistic function,
n(x; w) = x / rms_e(x) * w, positions i, j count from 0):

    streams   : X = [x_1 .. x_S], all equal to E[token] at the start.  A sublayer f with numbers (a[S], M[S, S], b[S], g):
                u = sum_s a_s x_s;  y = f(g * u / rms_e(u));  x_t <- sum_s M[s, t] x_s + b_t y  (all t from the old X)
                a layer = the mixer's sublayer, then the feed-forward's (if the layer has one); at the end x = sum_s x_s
    chunked   : q, k, v = W. h;  q, k <- n(.; w) per head over dim;  v <- (1 - lam) v + lam v_first (not in the first mixing
                layer);  s_ij = cap tanh(scale q_i . k_j / cap) - r1 ln(1 + r2 (i - j))  for j <= i in i's chunk of C positions;
                a_ij = exp(s_ij) / (exp(sink) + sum_j exp(s_ij));  o_i = sum_j a_ij v_j;  y = Wo concat_h(sg(Wg h)_h o_h)
    windowed  : q, k as above, then turned: pairs (2m, 2m + 1), m < dims / 2, by the angle i base^(-2m / dims);  v mixed as
                above;  i sees j with 0 <= i - j < W, and block b (positions bP .. bP + P - 1) once bP + P - 1 <= i - W,
                through the means of the block's (turned) keys and (mixed) values;  one softmax;  y = Wo concat_h(o_h)
    latent    : q = Wq h per head [dim | rot_dim];  [c' | r] = Wdkv h;  c = n(c'; w);  k_h = Wuk_h c,  v_h = Wuv_h c;
                s_ij = scale (q_nope_i . k_h,j + turn_i(q_rot_i) . turn_j(r_j)),  j <= i;  softmax;
                y = Wo (concat_h(o_h) * sg(Wg h))
    experts   : s = sg(Wr h);  C = the `top` largest;  y = sum_{e in C} ex_e(s_e h) + ex_shared(h),
                ex(z) = Wd (silu(Wg z) * (Wu z))
    logits    = Wh n(x; g_final)

`rnd` (default: the identity) is applied where an engine with 16-bit activations rounds: operands and results of matrix
products; with it the file predicts the size of that engine's rounding error.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np
import torch

F = torch.float64


def identity(x):
    return x


def to_bf16(x):
    return x.to(torch.float32).to(torch.bfloat16).to(F)


def read_config(model_dir: str) -> dict:
    with open(os.path.join(model_dir, "config.json")) as f:
        return json.load(f)


def read_weights(model_dir: str) -> dict:
    """Own reader of the container: 8 bytes of header length, a JSON header, raw little-endian data."""
    out = {}
    with open(os.path.join(model_dir, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        raw = data[meta["data_offsets"][0]:meta["data_offsets"][1]]
        shape = tuple(meta["shape"])
        if meta["dtype"] == "BF16":
            a = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            t = torch.from_numpy(a.view(np.float32).copy()).to(F)
        elif meta["dtype"] == "F32":
            t = torch.from_numpy(np.frombuffer(raw, dtype="<f4").copy()).to(F)
        elif meta["dtype"] == "I32":
            t = torch.from_numpy(np.frombuffer(raw, dtype="<i4").copy())
        else:
            raise ValueError(f"{name}: element type {meta['dtype']}")
        out[name] = t.reshape(shape)
    return out


# ---- mechanisms ----------------------------------------------------------------------------------------------------------

def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def turn_pairs(x, positions, dims, base):
    """x [T, ..., d]: the first `dims` elements turn in pairs (2m, 2m + 1) by the angle position * base^(-2m / dims)."""
    if not dims:
        return x
    m = torch.arange(dims // 2, dtype=F)
    angle = positions.to(F)[:, None] * base ** (-2.0 * m / dims)                 # [T, dims / 2]
    while angle.dim() < x.dim():
        angle = angle.unsqueeze(1)
    c, s = angle.cos(), angle.sin()
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def mix_values(v, v_first, lam):
    return v if v_first is None else (1.0 - lam) * v + lam * v_first


def chunk_visible(T, size):
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & (i // size == j // size)


def window_visible(T, size):
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & (i - j < size)


def blocks_visible(T, size, pool):
    """[T, T // pool]: block b is seen from i once its last position has left the window."""
    i = torch.arange(T)[:, None]
    b = torch.arange(T // pool)[None, :]
    return b * pool + pool - 1 <= i - size


def chunked_attention(h, w, p, m, eps, v_first, rnd=identity):
    """Returns (output, the values that were cached).  `m` is the layer's 'mixer' dictionary, `p` the tensor-name prefix."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rnd(h @ w[p + "q"].T).view(T, H, dk)
    k = rnd(h @ w[p + "k"].T).view(T, G, dk)
    v = rnd(h @ w[p + "v"].T).view(T, G, dv)
    q = rnd(unit_rms(q, eps) * w[p + "q.norm"])
    k = rnd(unit_rms(k, eps) * w[p + "k.norm"])
    if m.get("v_mix"):
        v = rnd(mix_values(v, v_first, w[p + "vmix"]))
    vis = chunk_visible(T, m["mask"]["size"])
    dist = (torch.arange(T)[:, None] - torch.arange(T)[None, :]).clamp(min=0).to(F)
    gate = torch.sigmoid(h @ w[p + "g"].T) if (p + "g") in w else None         # [T, H]
    out = torch.zeros(T, H, dv, dtype=F)
    for hh in range(H):
        g = hh // (H // G)
        s = (q[:, hh] @ k[:, g].T) * m["scale"]
        cap = m.get("softcap")
        if cap:
            s = cap * torch.tanh(s / cap)
        if (p + "r1") in w:
            s = s - w[p + "r1"][hh] * torch.log(1.0 + w[p + "r2"][hh] * dist)
        s = s.masked_fill(~vis, -math.inf)
        top = s.max(dim=1, keepdim=True).values
        e = torch.exp(s - top)
        den = e.sum(dim=1, keepdim=True)
        if (p + "sink") in w:
            den = den + torch.exp(w[p + "sink"][hh] - top)
        out[:, hh] = (e / den) @ v[:, g]
        if gate is not None:
            out[:, hh] = out[:, hh] * gate[:, hh:hh + 1]
    return rnd(rnd(out.reshape(T, H * dv)) @ w[p + "o"].T), v


def windowed_attention(h, w, p, m, eps, v_first, rnd=identity):
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = rnd(h @ w[p + "q"].T).view(T, H, dk)
    k = rnd(h @ w[p + "k"].T).view(T, G, dk)
    v = rnd(h @ w[p + "v"].T).view(T, G, dv)
    q = unit_rms(q, eps) * w[p + "q.norm"]
    k = unit_rms(k, eps) * w[p + "k.norm"]
    rot = m.get("rot") or {}
    q = rnd(turn_pairs(q, pos, rot.get("dims", 0), rot.get("base", 1.0)))
    k = rnd(turn_pairs(k, pos, rot.get("dims", 0), rot.get("base", 1.0)))
    if m.get("v_mix"):
        v = rnd(mix_values(v, v_first, w[p + "vmix"]))
    size, pool = m["mask"]["size"], m["mask"].get("pool", 0)
    vis = window_visible(T, size)
    nb = T // pool if pool else 0
    if nb:
        kb = rnd(k[:nb * pool].view(nb, pool, G, dk).mean(dim=1))
        vb = rnd(v[:nb * pool].view(nb, pool, G, dv).mean(dim=1))
        bvis = blocks_visible(T, size, pool)
    out = torch.zeros(T, H, dv, dtype=F)
    for hh in range(H):
        g = hh // (H // G)
        s = ((q[:, hh] @ k[:, g].T) * m["scale"]).masked_fill(~vis, -math.inf)
        vals = v[:, g]
        if nb:
            sb = ((q[:, hh] @ kb[:, g].T) * m["scale"]).masked_fill(~bvis, -math.inf)
            s = torch.cat([sb, s], dim=1)
            vals = torch.cat([vb[:, g], vals], dim=0)
        out[:, hh] = torch.softmax(s, dim=1) @ vals
    return rnd(rnd(out.reshape(T, H * dv)) @ w[p + "o"].T), v


def latent_attention(h, w, p, m, eps, rnd=identity):
    T = h.shape[0]
    H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    rot = m.get("rot") or {}
    q = rnd(h @ w[p + "q"].T).view(T, H, dn + dr)
    low = rnd(h @ w[p + "dkv"].T)
    c = rnd(unit_rms(low[:, :R], eps) * w[p + "dkv.norm"])
    kr = rnd(turn_pairs(low[:, R:], pos, rot.get("dims", 0), rot.get("base", 1.0)))              # [T, dr], one for all heads
    qr = rnd(turn_pairs(q[:, :, dn:], pos, rot.get("dims", 0), rot.get("base", 1.0)))
    kn = rnd(c @ w[p + "uk"].T).view(T, H, dn)
    vv = rnd(c @ w[p + "uv"].T).view(T, H, dv)
    causal = torch.arange(T)[None, :] <= torch.arange(T)[:, None]
    out = torch.zeros(T, H, dv, dtype=F)
    for hh in range(H):
        s = (q[:, hh, :dn] @ kn[:, hh].T + qr[:, hh] @ kr.T) * m["scale"]
        out[:, hh] = torch.softmax(s.masked_fill(~causal, -math.inf), dim=1) @ vv[:, hh]
    gated = out.reshape(T, H * dv) * torch.sigmoid(h @ w[p + "g"].T)
    return rnd(rnd(gated) @ w[p + "o"].T)


def expert(z, w, p, rnd=identity):
    a = rnd(silu(rnd(z @ w[p + "gate"].T)) * rnd(z @ w[p + "up"].T))
    return rnd(a @ w[p + "down"].T)


def routed_experts(h, w, p, f, rnd=identity, margins=None):
    """`margins` (a list) receives, per token, how far the last chosen expert's router logit lies above the first one left out."""
    T = h.shape[0]
    E, top = f["router"]["experts"], f["router"]["top"]
    z = h @ w[p + "router"].T
    s = torch.sigmoid(z)                                                        # [T, E]
    best = torch.topk(s, top, dim=1)
    if margins is not None:
        ordered = torch.sort(z, dim=1, descending=True).values
        margins.append(ordered[:, top - 1] - ordered[:, top] if top < E else torch.full((T,), math.inf, dtype=F))
    y = torch.zeros_like(h)
    for c in range(top):                                                       # the tokens whose c-th choice is expert e, together
        for e in range(E):
            rows = (best.indices[:, c] == e).nonzero().flatten()
            if len(rows):
                y[rows] += expert(rnd(s[rows, e:e + 1] * h[rows]), w, f"{p}e{e}.", rnd)
    if f.get("shared") is not None:
        y = y + expert(h, w, p + "shared.", rnd)
    return y


def stream_sublayer(X, w, p, norm_weight, eps, fn, rnd=identity):
    """X [T, S, D]; `p` the prefix of the sublayer's three stream tensors."""
    u = torch.einsum("s,tsd->td", w[p + "in"], X)
    y = fn(rnd(unit_rms(u, eps) * norm_weight))
    return torch.einsum("sr,tsd->trd", w[p + "mix"], X) + w[p + "out"][None, :, None] * y[:, None, :]


def forward(model_dir: str, tokens, rnd=identity, return_layers: bool = False):
    """Logits [T, vocab] of one whole sequence (float64); with `return_layers` also the summed streams after every layer."""
    cfg, w = read_config(model_dir), read_weights(model_dir)
    return forward_loaded(cfg, w, tokens, rnd, return_layers)


def forward_loaded(cfg, w, tokens, rnd=identity, return_layers: bool = False, router_margins=None):
    eps, S = cfg["norm"]["eps"], cfg.get("streams", 1)
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    X = w["embed"][tokens][:, None, :].repeat(1, S, 1)                          # [T, S, D]
    v_first = None
    seen = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        kept = {}

        def mixer(h, m=m, p=p, kind=layer["type"], kept=kept):
            if kind == "attention":
                y, kept["v"] = chunked_attention(h, w, p + "mix.", m, eps, v_first, rnd)
            elif kind == "attention_2":
                y, kept["v"] = windowed_attention(h, w, p + "mix.", m, eps, v_first, rnd)
            elif kind == "latent_attention":
                y = latent_attention(h, w, p + "mix.", m, eps, rnd)
            else:
                raise ValueError(f"layer {i}: mixer '{kind}'")
            return y

        if S > 1 or (p + "hc1.in") in w:
            X = stream_sublayer(X, w, p + "hc1.", w[p + "norm1"], eps, mixer, rnd)
        else:
            X = X + mixer(rnd(unit_rms(X[:, 0], eps) * w[p + "norm1"]))[:, None, :]
        if m.get("v_mix") and v_first is None:
            v_first = kept["v"]
        f = layer.get("mlp")
        if f is not None:
            ff = lambda h, f=f, p=p: routed_experts(h, w, p + "mlp.", f, rnd, router_margins)   # noqa: E731
            if S > 1 or (p + "hc2.in") in w:
                X = stream_sublayer(X, w, p + "hc2.", w[p + "norm2"], eps, ff, rnd)
            else:
                X = X + ff(rnd(unit_rms(X[:, 0], eps) * w[p + "norm2"]))[:, None, :]
        seen.append(X.sum(dim=1))
    x = X.sum(dim=1)
    logits = rnd(unit_rms(x, eps) * w["final.norm"]) @ w["head"].T
    return (logits, torch.stack(seen)) if return_layers else logits
