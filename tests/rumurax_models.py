"""Small Rumurax configurations that differ from one another in every size and option, and a writer of their folders.

          width vocab streams  layers (mixer; feed-forward)
    rx_a    48    97     3     windowed 4/2 heads, 16 (8 turned)/24, window 20, blocks of 4, mixing; 5 experts, 2 per token, 24 wide, shared 16
                               chunked 4/2 heads, 16/24, chunks of 16, cap 5, mixing; none
                               latent 3 heads, 8 + 6 (6 turned), values 10, latent 20; 3 experts, 1 per token, 16 wide
                               windowed 2/2 heads, 12 (12 turned)/24, window 7, blocks of 3, mixing; 2 experts, both, shared 8
    rx_b    80   131     1     chunked 6/3 heads, 24/16, chunks of 33, no cap, mixing (the first); 4 experts, 4 per token
                               windowed 3/3 heads, 10 (4 turned)/16, window 50, no blocks, mixing; none
                               latent 2 heads, 16 + 8 (4 turned), values 24, latent 40; 3 experts, 2 per token, shared 24
    rx_c    96   150     2     windowed 6/2 heads, 64 (32 turned)/64, window 40, blocks of 8, mixing; 4 experts, 2 per token, 32 wide, shared 32
                               chunked 4/2 heads, 32/64, chunks of 48, cap 12, mixing; 4 experts, 1 per token
                               latent 4 heads, 32 + 16 (16 turned), values 32, latent 64; none
                               windowed 4/2 heads, 80 (80 turned)/64, window 70, blocks of 16, mixing; 2 experts, 1 per token
                               chunked 2/1 heads, 64/64, chunks of 100, cap 30, no mixing; 3 experts, 3 per token, shared 16
    rx_e    64    83     6     windowed 32/1 heads, 16 (16 turned)/16, window 30, blocks of 5; 3 experts, 2 per token, 16 wide, shared 8
                               chunked 2/1 heads, 160/144, chunks of 40, cap 8; none
                               latent 2 heads, 24 + 8 (8 turned), values 40, latent 200; 9 experts, 1 per token, 8 wide
    rx_d    50    61  (none)   chunked 5/5 heads, 10/6, chunks of 5, cap 2; 6 experts, 3 per token, 12 wide, shared 12
                               windowed 1/1 head, 6 (4 turned)/3, window 3, blocks of 2; none
Widths of 50 and rows of 10, 6 or 3 elements fit no vector width; rx_b has one stream with learned weights, rx_d none at all
(no 'streams' key: a plain residual sum); rx_b starts with a chunked layer and has a window without blocks; rx_c has the
sizes the tensor-core kernels take, keys and values of different sizes and a layer that mixes no values among layers that do;
in rx_d windows and chunks are a handful of tokens; rx_e has six streams (beyond the stream kernel's vector forms), 32 query heads
on one kv head (beyond the 16 rows of the form for decoded tokens), heads of 160 and 144 elements and a latent of 200 (beyond
what the tensor-core kernels take, in bfloat16 too).  Scales, eps, caps and bases all differ."""
import json
import os

import torch


def _windowed(heads, kv, dim, vdim, window, pool, rot, base, scale, v_mix=True):
    m = {"dim": dim, "heads": heads, "kv_heads": kv, "vdim": vdim, "scale": scale, "mask": {"size": window},
         "rot": {"dims": rot, "base": base}}
    if pool:
        m["mask"]["pool"] = pool
    if v_mix:
        m["v_mix"] = True
    return {"type": "attention_2", "mixer": m}


def _chunked(heads, kv, dim, vdim, chunk, cap, scale, v_mix=True):
    m = {"dim": dim, "heads": heads, "kv_heads": kv, "vdim": vdim, "scale": scale, "mask": {"size": chunk}}
    if cap:
        m["softcap"] = cap
    if v_mix:
        m["v_mix"] = True
    return {"type": "attention", "mixer": m}


def _latent(heads, dim, rot_dim, vdim, rank, rot, base, scale):
    return {"type": "latent_attention", "mixer": {"dim": dim, "heads": heads, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank,
                                                  "scale": scale, "rot": {"dims": rot, "base": base}}}


def _moe(experts, top, ff, shared=0):
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        f["shared"] = {"ff": shared}
    return f


def _layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


RX_A = {"architecture": "Rumurax", "vocab": 97, "width": 48, "streams": 3, "norm": {"eps": 1e-5},
        "layers": [_layer(_windowed(4, 2, 16, 24, 20, 4, 8, 100.0, 0.3), _moe(5, 2, 24, shared=16)),
                   _layer(_chunked(4, 2, 16, 24, 16, 5.0, 0.35), None),
                   _layer(_latent(3, 8, 6, 10, 20, 6, 50.0, 0.3), _moe(3, 1, 16)),
                   _layer(_windowed(2, 2, 12, 24, 7, 3, 12, 1000.0, 0.25), _moe(2, 2, 8, shared=8))]}
RX_B = {"architecture": "Rumurax", "vocab": 131, "width": 80, "streams": 1, "norm": {"eps": 1e-6},
        "layers": [_layer(_chunked(6, 3, 24, 16, 33, 0.0, 0.2), _moe(4, 4, 16)),
                   _layer(_windowed(3, 3, 10, 16, 50, 0, 4, 10000.0, 0.3), None),
                   _layer(_latent(2, 16, 8, 24, 40, 4, 250000.0, 0.2), _moe(3, 2, 24, shared=24))]}
RX_C = {"architecture": "Rumurax", "vocab": 150, "width": 96, "streams": 2, "norm": {"eps": 1e-5},
        "layers": [_layer(_windowed(6, 2, 64, 64, 40, 8, 32, 10000.0, 0.125), _moe(4, 2, 32, shared=32)),
                   _layer(_chunked(4, 2, 32, 64, 48, 12.0, 0.18), _moe(4, 1, 32)),
                   _layer(_latent(4, 32, 16, 32, 64, 16, 500000.0, 0.15), None),
                   _layer(_windowed(4, 2, 80, 64, 70, 16, 80, 300.0, 0.11), _moe(2, 1, 64)),
                   _layer(_chunked(2, 1, 64, 64, 100, 30.0, 0.125, v_mix=False), _moe(3, 3, 16, shared=16))]}
RX_D = {"architecture": "Rumurax", "vocab": 61, "width": 50, "norm": {"eps": 1e-4},
        "layers": [_layer(_chunked(5, 5, 10, 6, 5, 2.0, 0.4, v_mix=False), _moe(6, 3, 12, shared=12)),
                   _layer(_windowed(1, 1, 6, 3, 3, 2, 4, 20.0, 0.5, v_mix=False), None)]}

RX_E = {"architecture": "Rumurax", "vocab": 83, "width": 64, "streams": 6, "norm": {"eps": 1e-5},
        "layers": [_layer(_windowed(32, 1, 16, 16, 30, 5, 16, 5000.0, 0.25, v_mix=False), _moe(3, 2, 16, shared=8)),
                   _layer(_chunked(2, 1, 160, 144, 40, 8.0, 0.08, v_mix=False), None),
                   _layer(_latent(2, 24, 8, 40, 200, 8, 1000.0, 0.18), _moe(9, 1, 8))]}

# name -> (config, seed, page size)
SETUPS = {"rx_a": (RX_A, 31, 16), "rx_b": (RX_B, 32, 32), "rx_c": (RX_C, 33, 16), "rx_d": (RX_D, 34, 64), "rx_e": (RX_E, 35, 32)}


def write_model(path, cfg, seed, sharpen=4.0):
    """Random weights through the package's random-weights writer (tensor names and shapes come from the architecture),
    then made sharp: query weights are scaled up so that attention concentrates on few keys (a mask that is one token off
    then shows), sinks and the distance term are made large, the mixing weights of values are moved away from 0, routers are
    scaled so that experts are chosen with clear margins, and the embedding table is made large."""
    from cppvllm_b200.weights.random_init import random_tensors
    from cppvllm_b200.weights.safetensors_io import save_safetensors
    import cppvllm_b200.models  # noqa: F401
    os.makedirs(path, exist_ok=True)
    tensors = random_tensors(cfg, seed, std=0.08, norm_spread=0.3)
    for k in list(tensors):
        t = tensors[k].float()
        if k.endswith(".mix.q"):
            t = t * sharpen
        elif k.endswith(".mix.sink"):
            t = t * 25.0
        elif k.endswith(".mix.vmix"):
            t = t + 0.35
        elif k.endswith(".mix.r2"):
            t = t * 0.5
        elif k.endswith(".mix.g"):
            t = t * 6.0
        elif k.endswith(".router"):
            t = t * 3.0
        elif k == "embed":
            t = t * 4.0
        tensors[k] = t.to(torch.bfloat16)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_safetensors(os.path.join(path, "model.safetensors"), tensors)
    return path


def random_config(seed, tensor_core=False):
    """A configuration drawn at random: 2 to 6 layers of the three kinds in any order, with or without experts; sizes odd,
    prime, 1 or large; windows, chunks and blocks from 1 token to more than a prompt; 1 to 4 streams or none.  With
    `tensor_core` the key and value sizes are multiples of 16, the sizes the tensor-core kernels take."""
    import random
    r = random.Random(2000 + seed)
    width = r.choice([32, 40, 50, 64, 72, 100, 128])
    sizes = [16, 32, 48, 64, 96, 128] if tensor_core else [2, 6, 8, 10, 16, 24, 40, 64]
    kv, group = r.choice([1, 2, 3]), r.choice([1, 2, 4] if tensor_core else [1, 2, 3, 5])
    vdim = r.choice(sizes)                               # layers that mix values share their kv heads and value size
    layers = []
    for i in range(r.randint(2, 6)):
        kind = r.random()
        if kind < 0.4:
            dim = r.choice(sizes)
            window = r.choice([1, 2, 5, 17, 64, 100, 500])
            layer = _windowed(kv * group, kv, dim, vdim, window, r.choice([0, 1, 2, 3, 8, 16]), r.choice([x for x in (2, 4, 8, 16, dim) if x <= dim and x % 2 == 0]),
                              r.choice([10.0, 1000.0, 250000.0]), r.choice([0.1, 0.2, 0.35]), v_mix=r.random() < 0.7)
        elif kind < 0.75:
            layer = _chunked(kv * group, kv, r.choice(sizes), vdim, r.choice([1, 2, 7, 32, 64, 300]), r.choice([0.0, 3.0, 20.0]),
                             r.choice([0.1, 0.2, 0.35]), v_mix=r.random() < 0.7)
        else:
            rank = r.choice([16, 32, 48] if tensor_core else [5, 12, 20, 64])
            rot_dim = r.choice([16, 32] if tensor_core else [2, 4, 6, 16])
            layer = _latent(r.choice([1, 2, 3, 4]), r.choice([4, 8, 16, 32] if tensor_core else [3, 8, 16]), rot_dim, r.choice(sizes), rank,
                            r.choice([x for x in (2, 4, rot_dim) if x <= rot_dim]), r.choice([100.0, 500000.0]), r.choice([0.1, 0.2, 0.3]))
        if r.random() < 0.25:
            mlp = None
        else:
            experts = r.randint(1, 9)
            mlp = _moe(experts, r.randint(1, experts), r.choice([8, 20, 32, 64]), shared=r.choice([0, 8, 24, 48]))
        layers.append(_layer(layer, mlp))
    cfg = {"architecture": "Rumurax", "vocab": r.randint(40, 300), "width": width, "norm": {"eps": r.choice([1e-6, 1e-5, 1e-4])},
           "layers": layers}
    streams = r.choice([0, 1, 2, 3, 4])
    if streams:
        cfg["streams"] = streams
    return cfg


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
_REFERENCE = {}


def clear_tokens(model_dir, n, seed, margin=0.3):
    """Random tokens among which no routed feed-forward has a close call: where the last chosen expert's router logit lies
    less than `margin` above the first one left out (in the plain implementation, exact or with 16-bit rounding), the token
    is drawn again.  A model is causal, so a token changes nothing before it and the walk goes from left to right.  Another
    expert changes a token's streams by a large step, and the keys made from them carry that to later tokens, so a close
    call would bury the errors the tests look for."""
    import plain_rumurax as plain
    key = (model_dir, n, seed)
    if key in _CLEAR:
        return list(_CLEAR[key])
    cfg, w = plain.read_config(model_dir), plain.read_weights(model_dir)
    toks = random_tokens(cfg["vocab"], n, seed)
    if not any(l.get("mlp") and l["mlp"]["router"]["top"] < l["mlp"]["router"]["experts"] for l in cfg["layers"]):
        _CLEAR[key] = toks
        return list(toks)

    def smallest(tokens):
        out = None
        for rnd in (plain.identity, plain.to_bf16):
            m = []
            plain.forward_loaded(cfg, w, tokens, rnd=rnd, router_margins=m)
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
    import plain_rumurax as plain
    if layer_outputs is None:
        key = (model_dir, tuple(tokens))
        if key not in _REFERENCE:
            _REFERENCE[key] = plain.forward(model_dir, tokens)
        return _REFERENCE[key]
    logits, layers = plain.forward(model_dir, tokens, return_layers=True)
    layer_outputs.extend(layers)
    return logits
