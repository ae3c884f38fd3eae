"""Small Lorulix configurations that differ from one another in every size and option, and a writer of their folders.

          width vocab taps  layers (mixer; feed-forward)
    lx_a    48    97    3   attention 3/1 heads, 16/24, 8 rows to 20, temperature .4 every 5; dense 40 limit .7
                            delta 4/2 heads, 12/20, 2 taps; 5 experts, 2 per token, 24 wide, shared 16
                            attention reading layer 0's keys and values; no feed-forward
                            delta 2/2 heads, 8/8, 4 taps; dense 56 limit 3
    lx_b    80   131    1   delta 3/1 heads, 40/33, 1 tap; 3 experts, 1 per token, no shared expert
                            attention 4/4 heads, 24/16, 6 rows to 9, temperature every token; no feed-forward
                            attention 2/1 heads, 40/40, 16 rows to 300, no temperature (coef 0); 2 experts, both, shared 8
    lx_c    96   150    4   attention 6/2 heads, 64/64, 32 rows to 100; 4 experts, 4 per token, shared 32
                            attention reading layer 0's; dense 128
                            delta 2/2 heads, 64/64, 3 taps; dense 64
                            attention 4/2 heads, 32/64, 12 rows to 50; dense 64
                            attention reading layer 3's; 4 experts, 2 per token
    lx_d    50    61    2   attention 5/5 heads, 10/6, 4 rows to 3; 6 experts, 3 per token, 12 wide, shared 12
                            delta 1/1 head, 5/3, 6 taps; none
Widths 50 and rows of 10 or 6 elements fit no vector width; lx_b has no history in front of its sublayers (one tap) and
starts with a recurrent layer; lx_c has the head sizes tensor-core kernels take, key and value sizes that differ and two
pairs of layers that share a cache; in lx_d the distance table is as small as it can be, so nearly every key lies in the
last bucket; scales, eps, limits, router scales all differ (one is 1)."""
import json
import os

import torch


def _attn(heads, kv, dim, vdim, rows, far, coef, every, scale, kv_from=None):
    m = {"dim": dim, "heads": heads, "kv_heads": kv, "vdim": vdim, "scale": scale, "bias_max": far, "bias_rows": rows,
         "q_temp": {"coef": coef, "every": every}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m}


def _delta(heads, kv, dim, vdim, conv):
    return {"type": "delta", "mixer": {"dim": dim, "heads": heads, "kv_heads": kv, "vdim": vdim, "conv": conv}}


def _dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def _moe(experts, top, ff, scale, shared=0):
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}
    if shared:
        f["shared"] = {"ff": shared}
    return f


def _layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


LX_A = {"architecture": "Lorulix", "vocab": 97, "width": 48, "max_positions": 160, "norm": {"eps": 1e-5}, "canon": {"taps": 3},
        "layers": [_layer(_attn(3, 1, 16, 24, 8, 20, 0.4, 5, 0.3), _dense(40, 0.7)),
                   _layer(_delta(4, 2, 12, 20, 2), _moe(5, 2, 24, 2.0, shared=16)),
                   _layer(_attn(3, 1, 16, 24, 8, 20, 0.4, 5, 0.3, kv_from=0), None),
                   _layer(_delta(2, 2, 8, 8, 4), _dense(56, 3.0))]}
LX_B = {"architecture": "Lorulix", "vocab": 131, "width": 80, "max_positions": 200, "norm": {"eps": 1e-6}, "canon": {"taps": 1},
        "layers": [_layer(_delta(3, 1, 40, 33, 1), _moe(3, 1, 16, 1.0)),
                   _layer(_attn(4, 4, 24, 16, 6, 9, 0.25, 1, 0.2), None),
                   _layer(_attn(2, 1, 40, 40, 16, 300, 0.0, 7, 0.15), _moe(2, 2, 16, 0.5, shared=8))]}
LX_C = {"architecture": "Lorulix", "vocab": 150, "width": 96, "max_positions": 400, "norm": {"eps": 1e-5}, "canon": {"taps": 4},
        "layers": [_layer(_attn(6, 2, 64, 64, 32, 100, 0.3, 16, 0.125), _moe(4, 4, 32, 1.5, shared=32)),
                   _layer(_attn(6, 2, 64, 64, 32, 100, 0.3, 16, 0.125, kv_from=0), _dense(128, 1.0)),
                   _layer(_delta(2, 2, 64, 64, 3), _dense(64, 1.5)),
                   _layer(_attn(4, 2, 32, 64, 12, 50, 0.1, 64, 0.18), _dense(64, 0.5)),
                   _layer(_attn(4, 2, 32, 64, 12, 50, 0.1, 64, 0.18, kv_from=3), _moe(4, 2, 32, 3.0))]}
LX_D = {"architecture": "Lorulix", "vocab": 61, "width": 50, "max_positions": 120, "norm": {"eps": 1e-4}, "canon": {"taps": 2},
        "layers": [_layer(_attn(5, 5, 10, 6, 4, 3, 1.0, 3, 0.4), _moe(6, 3, 12, 2.5, shared=12)),
                   _layer(_delta(1, 1, 5, 3, 6), None)]}

# name -> (config, seed, page size)
SETUPS = {"lx_a": (LX_A, 21, 16), "lx_b": (LX_B, 22, 32), "lx_c": (LX_C, 23, 16), "lx_d": (LX_D, 24, 64)}


def write_model(path, cfg, seed, sharpen=4.0):
    """Random weights through the package's random-weights writer (tensor names and shapes come from the architecture),
    then made sharp: query weights of attention layers are scaled up so that attention concentrates on few keys, the
    distance table is made large so that a bucket that is one off shows, routers are scaled so that experts are chosen with
    clear margins, the decays' logarithms are moved down so that the recurrent state remembers hundreds of tokens, and the
    embedding and position tables are made large."""
    from cppvllm_b200.weights.random_init import random_tensors
    from cppvllm_b200.weights.safetensors_io import save_safetensors
    import cppvllm_b200.models  # noqa: F401
    os.makedirs(path, exist_ok=True)
    tensors = random_tensors(cfg, seed, std=0.08, norm_spread=0.3)
    kinds = [l["type"] for l in cfg["layers"]]
    for k in list(tensors):
        t = tensors[k].float()
        layer = int(k[1:k.index(".")]) if k.startswith("l") and k[1].isdigit() else -1
        if k.endswith(".mix.q") and kinds[layer] == "attention":
            t = t * sharpen
        elif k.endswith(".mix.rel"):
            t = t * 12.0
        elif k.endswith(".router"):
            t = t * 3.0
        elif k.endswith(".mix.A_log"):
            t = t - 3.0
        elif k.endswith(".conv") or ".canon" in k:
            t = t * 5.0
        elif k.endswith(".rg1.b") or k.endswith(".rg2.b"):
            t = t * 10.0
        elif k in ("embed", "pos"):
            t = t * 4.0
        tensors[k] = t.to(torch.bfloat16)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_safetensors(os.path.join(path, "model.safetensors"), tensors)
    return path


def random_config(seed, tensor_core=False):
    """A configuration drawn at random: 2 to 6 layers of both kinds in any order, with no, a dense or a routed feed-forward;
    sizes odd, prime, 1 or large; layers that read an earlier layer's keys and values.  With `tensor_core` the key and value
    sizes of attention are multiples of 16, the sizes its tensor-core kernels take."""
    import random
    r = random.Random(1000 + seed)
    width = r.choice([32, 40, 50, 64, 72, 100, 128])
    layers, writers = [], []
    for i in range(r.randint(2, 6)):
        if r.random() < 0.6:
            if writers and r.random() < 0.4:
                j = r.choice(writers)
                m = dict(layers[j]["mixer"], kv_from=j, scale=r.choice([0.1, 0.2, 0.35]), bias_max=r.randint(layers[j]["mixer"]["bias_rows"] // 2 + 1, 260))
                m["q_temp"] = {"coef": r.choice([0.0, 0.2, 0.7]), "every": r.choice([1, 3, 16, 50])}
                layer = {"type": "attention", "mixer": m}
            else:
                kv, group = r.choice([1, 2, 3]), r.choice([1, 2, 4, 5] if not tensor_core else [1, 2, 4, 8])
                sizes = [16, 32, 48, 64, 96, 128] if tensor_core else [6, 8, 10, 16, 24, 40, 64]
                rows = r.choice([4, 6, 8, 12, 20, 32])
                layer = _attn(kv * group, kv, r.choice(sizes), r.choice(sizes), rows, r.randint(rows // 2 + 1, 260),
                              r.choice([0.0, 0.2, 0.7]), r.choice([1, 3, 16, 50]), r.choice([0.1, 0.2, 0.35]))
                writers.append(i)
        else:
            kv, group = r.choice([1, 2]), r.choice([1, 2, 3])
            layer = _delta(kv * group, kv, r.choice([3, 8, 16, 33, 64]), r.choice([5, 8, 16, 40, 64]), r.randint(1, 5))
        kind = r.random()
        if kind < 0.2:
            mlp = None
        elif kind < 0.55:
            mlp = _dense(r.choice([24, 50, 64, 128]), r.choice([0.5, 1.0, 2.5, 7.0]))
        else:
            experts = r.randint(2, 9)
            mlp = _moe(experts, r.randint(1, experts), r.choice([8, 20, 32, 64]), r.choice([0.5, 1.0, 2.0, 3.5]),
                       shared=r.choice([0, 8, 24, 48]))
        layers.append(_layer(layer, mlp))
    return {"architecture": "Lorulix", "vocab": r.randint(40, 300), "width": width, "max_positions": 256,
            "norm": {"eps": r.choice([1e-6, 1e-5, 1e-4])}, "canon": {"taps": r.randint(1, 5)}, "layers": layers}


def write_all(base):
    return {name: write_model(os.path.join(base, name), cfg, seed) for name, (cfg, seed, _) in SETUPS.items()}


def page_size(name):
    return SETUPS[name][2]


def config(name):
    return SETUPS[name][0]


def random_tokens(vocab, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


_CLEAR = {}


def clear_tokens(model_dir, n, seed, margin=0.3):
    """Random tokens among which no routed feed-forward has a close call: where the last chosen expert's router logit lies
    less than `margin` above the first one left out (in the plain implementation, exact or with 16-bit rounding), the
    token is drawn again.  A model is causal, so a token changes nothing before it and the walk goes from left to right.
    With a norm behind every sublayer another expert changes a token's stream by its whole size, and the keys made from it
    carry that to every later token, so a close call would bury the errors the tests look for."""
    import plain_lorulix as plain
    key = (model_dir, n, seed)
    if key in _CLEAR:
        return list(_CLEAR[key])
    cfg, w = plain.read_config(model_dir), plain.read_weights(model_dir)
    toks = random_tokens(cfg["vocab"], n, seed)
    if not any(l.get("mlp") and l["mlp"]["kind"] == "moe" for l in cfg["layers"]):
        _CLEAR[key] = toks
        return list(toks)

    def smallest(tokens):
        out = None
        for rnd in (plain.identity, plain.to_bf16):
            m = []
            plain.forward(cfg, w, tokens, rnd=rnd, router_margins=m)
            m = torch.stack(m).min(dim=0).values
            out = m if out is None else torch.minimum(out, m)
        return out

    g = torch.Generator().manual_seed(seed + 7919)
    at = 0
    while at < n:
        m = smallest(toks)
        bad = [i for i in range(at, n) if float(m[i]) < margin]
        if not bad:
            break
        at = bad[0]
        for _ in range(200):
            toks[at] = int(torch.randint(0, cfg["vocab"], (1,), generator=g))
            if float(smallest(toks[:at + 1])[at]) >= margin:
                break
        else:
            raise AssertionError(f"no token with a clear routing at position {at}")
        at += 1
    _CLEAR[key] = toks
    return list(toks)


def reference(model_dir, tokens, layer_outputs=None):
    """Logits of one whole sequence from the plain implementation, which reads the folder with its own readers."""
    import plain_lorulix as plain
    return plain.forward(plain.read_config(model_dir), plain.read_weights(model_dir), tokens, layer_outputs=layer_outputs)
