"""Plain, slow implementation of the Lorulix decoder: whole sequences, no cache, no batching, one function per mechanism,
float64 on the CPU.  It shares no code with the package under test: its own config.json reading, its own safetensors
reading and its own arithmetic.  In this file's notation (rms_e(x) = sqrt(mean(x^2) + e), n(x; w) = x / rms_e(x) * w,
sg = logistic function, cv(h; c)_t = sum_j c[:, j] h_(t - taps + 1 + j)):

    x_0       = E[token] + P[position]
    sublayer  : a = n(x; 1 + w_in);  r = f(a + cv(a; c)) * sg(Wr a + br);  x <- x + n(r; 1 + w_out)
                (f = the mixer with c = canon1, then f = the feed-forward with c = canon2)
    attention : q = Wq h, k = Wk h, v = Wv h;  q <- n(q; wq) and k <- n(k; wk) over the whole projection;
                q_i <- q_i (1 + coef ln(floor((i + 1) / every) + 1));  s_ij = scale q_i . k_j + R[bucket(i - j), head], j <= i;
                softmax over j;  y = Wo concat_h(sum_j a_ij v_j).  A layer with kv_from = j reads layer j's (k, v).
    bucket    : n for n < B/2, else min(B - 1, B/2 + floor(ln(n / (B/2)) / ln(D / (B/2)) (B - B/2)))
    delta     : q, k, v = silu(cv(W. h));  q, k <- unit vectors per head (q also / sqrt(dim));  b = sg(Wb h);
                g = exp(-exp(A_h) softplus(Wa h + dt)) per head;  S <- g S;  u = b (v - S^T k);  S <- S + k u^T;  o = S^T q;
                y = Wo concat_h(n(o_h; w) * silu(Wg h)_h)
    dense ff  : g = min(Wg h, L), u = clamp(Wu h, -L, L);  y = Wd (g sg(1.702 g) (u + 1))
    experts   : s = softmax(Wr h);  C = the `top` largest;  y = sum_{e in C} scale s_e Wd_e relu(Wu_e h)^2
                + sg(w_sg . h) Wd_s relu(Wu_s h)^2
    logits    = Wh n(x; 1 + w_final)

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
        if meta["dtype"] == "BF16":
            bits = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            t = torch.from_numpy(bits.view(np.float32).copy())
        elif meta["dtype"] == "F32":
            t = torch.from_numpy(np.frombuffer(raw, dtype="<f4").copy())
        elif meta["dtype"] == "I32":
            t = torch.from_numpy(np.frombuffer(raw, dtype="<i4").copy())
        else:
            raise ValueError(f"{name}: element type {meta['dtype']}")
        t = t.reshape(meta["shape"])
        out[name] = t.to(F) if t.dtype.is_floating_point else t
    return out


# ---- small pieces --------------------------------------------------------------------------------------------------

def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_around_zero(x, w, eps):
    return unit_rms(x, eps) * (1.0 + w)


def logistic(x):
    return 1.0 / (1.0 + torch.exp(-x))


def silu(x):
    return x * logistic(x)


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def causal_conv(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """x [T, C], taps [C, K]; the last column multiplies the current token, zeros stand before the sequence."""
    T, C = x.shape
    K = taps.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=x.dtype), x], dim=0)
    out = torch.zeros_like(x)
    for j in range(K):
        out = out + padded[j:j + T] * taps[:, j]
    return out


def with_input_conv(h, taps):
    return h + causal_conv(h, taps)


# ---- attention -------------------------------------------------------------------------------------------------------

def distance_bucket(n: int, rows: int, far: float) -> int:
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def query_temperature(T: int, coef: float, every: int) -> torch.Tensor:
    return torch.tensor([1.0 + coef * math.log((p + 1) // every + 1) for p in range(T)], dtype=F)


def attention_keys_values(h, w, pre, m, eps, rnd):
    k = rnd(h @ w[pre + "k"].T)
    v = rnd(h @ w[pre + "v"].T)
    k = rnd(unit_rms(k, eps) * w[pre + "k.norm"])
    return k, v


def biased_attention(h, w, pre, m, eps, kv, rnd):
    """kv: this layer's own keys and values, or those of the layer it reads."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rnd(h @ w[pre + "q"].T)
    q = unit_rms(q, eps) * w[pre + "q.norm"]
    q = rnd(q * query_temperature(T, m["q_temp"]["coef"], m["q_temp"]["every"])[:, None]).reshape(T, H, dk)
    k, v = kv
    k, v = k.reshape(T, G, dk), v.reshape(T, G, dv)
    rel = w[pre + "rel"]
    rows = rel.shape[0]
    dist = torch.tensor([[distance_bucket(i - j, rows, m["bias_max"]) if j <= i else 0 for j in range(T)] for i in range(T)])
    visible = torch.tril(torch.ones(T, T, dtype=torch.bool))
    out = torch.zeros(T, H, dv, dtype=F)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * m["scale"] + rel[:, head][dist]
        s = s.masked_fill(~visible, -math.inf)
        a = torch.softmax(s, dim=-1)
        out[:, head] = a @ v[:, g]
    return rnd(rnd(out.reshape(T, H * dv)) @ w[pre + "o"].T)


# ---- the gated delta rule ------------------------------------------------------------------------------------------------

def unit_vectors(x):
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + 1e-6)


def delta_rule(q, k, v, beta, g):
    """q, k [T, H, dk], v [T, H, dv], beta, g [T, H]; returns o [T, H, dv]."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    S = torch.zeros(H, dk, dv, dtype=F)
    o = torch.zeros(T, H, dv, dtype=F)
    for t in range(T):
        S = S * g[t][:, None, None]
        u = beta[t][:, None] * (v[t] - torch.einsum("hkv,hk->hv", S, k[t]))
        S = S + torch.einsum("hk,hv->hkv", k[t], u)
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return o


def delta_mixer(h, w, pre, m, eps, rnd):
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rnd(silu(causal_conv(rnd(h @ w[pre + "q"].T), w[pre + "q.conv"]))).reshape(T, G, dk)
    k = rnd(silu(causal_conv(rnd(h @ w[pre + "k"].T), w[pre + "k.conv"]))).reshape(T, G, dk)
    v = rnd(silu(causal_conv(rnd(h @ w[pre + "v"].T), w[pre + "v.conv"]))).reshape(T, H, dv)
    q = unit_vectors(q) * dk ** -0.5
    k = unit_vectors(k)
    share = H // G
    q, k = q.repeat_interleave(share, dim=1), k.repeat_interleave(share, dim=1)
    beta = logistic(h @ w[pre + "b"].T)
    g = torch.exp(-torch.exp(w[pre + "A_log"]) * softplus(h @ w[pre + "a"].T + w[pre + "dt_bias"]))
    o = delta_rule(q, k, v, beta, g)
    gate = silu(rnd(h @ w[pre + "g"].T)).reshape(T, H, dv)
    y = unit_rms(o, eps) * w[pre + "norm"] * gate
    return rnd(rnd(y.reshape(T, H * dv)) @ w[pre + "o"].T)


# ---- feed-forwards -------------------------------------------------------------------------------------------------------

def clamped_glu(h, w, pre, f, rnd):
    L = f["limit"]
    g = torch.clamp(rnd(h @ w[pre + "gate"].T), max=L)
    u = torch.clamp(rnd(h @ w[pre + "up"].T), min=-L, max=L)
    return rnd(rnd(g * logistic(1.702 * g) * (u + 1.0)) @ w[pre + "down"].T)


def relu2_expert(h, up, down, rnd):
    return rnd(rnd(torch.relu(rnd(h @ up.T)) ** 2) @ down.T)


def routed_experts(h, w, pre, f, rnd, margins=None):
    """`margins` (a list) receives, per token, how far the last chosen expert's logit lies above the first one left out."""
    E, top, scale = f["router"]["experts"], f["router"]["top"], f["router"]["scale"]
    z = h @ w[pre + "router"].T
    if margins is not None:
        ranked = torch.sort(z, dim=-1, descending=True).values
        margins.append(ranked[:, top - 1] - ranked[:, top] if top < E else torch.full((h.shape[0],), math.inf, dtype=F))
    s = torch.softmax(z, dim=-1)
    chosen = torch.topk(s, top, dim=-1).indices
    y = torch.zeros(h.shape[0], w[pre + "e0.down"].shape[0], dtype=F)
    for e in range(E):
        mine = (chosen == e).any(dim=-1)
        if mine.any():
            y[mine] += (scale * s[mine, e])[:, None] * relu2_expert(h[mine], w[pre + f"e{e}.up"], w[pre + f"e{e}.down"], rnd)
    if f.get("shared"):
        y = y + logistic(h @ w[pre + "shared.sg"].T) * relu2_expert(h, w[pre + "shared.up"], w[pre + "shared.down"], rnd)
    return y


# ---- the model ---------------------------------------------------------------------------------------------------------

def forward(cfg: dict, w: dict, tokens, rnd=identity, layer_outputs=None, router_margins=None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence; `layer_outputs` (a list) receives the stream after every layer,
    `router_margins` (a list) one tensor [T] per routed feed-forward (see routed_experts)."""
    eps = cfg["norm"]["eps"]
    T = len(tokens)
    x = w["embed"][torch.tensor(tokens)] + w["pos"][:T]
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        a = rnd(norm_around_zero(x, w[p + "norm1"], eps))
        h = rnd(with_input_conv(a, w[p + "canon1"]))
        if layer["type"] == "attention":
            if m.get("kv_from") is None:
                kept[i] = attention_keys_values(h, w, p + "mix.", m, eps, rnd)
            y = biased_attention(h, w, p + "mix.", m, eps, kept[m["kv_from"] if m.get("kv_from") is not None else i], rnd)
        elif layer["type"] == "delta":
            y = delta_mixer(h, w, p + "mix.", m, eps, rnd)
        else:
            raise ValueError(layer["type"])
        y = y * logistic(rnd(a @ w[p + "rg1"].T) + w[p + "rg1.b"])
        x = x + norm_around_zero(y, w[p + "norm1b"], eps)
        f = layer.get("mlp")
        if f is not None:
            a = rnd(norm_around_zero(x, w[p + "norm2"], eps))
            h = rnd(with_input_conv(a, w[p + "canon2"]))
            y = clamped_glu(h, w, p + "mlp.", f, rnd) if f["kind"] == "dense" else routed_experts(h, w, p + "mlp.", f, rnd, router_margins)
            y = y * logistic(rnd(a @ w[p + "rg2"].T) + w[p + "rg2.b"])
            x = x + norm_around_zero(y, w[p + "norm2b"], eps)
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    return rnd(norm_around_zero(x, w["final.norm"], eps)) @ w["head"].T
