"""A design beside Qwen3 at equal layer sizes (Givirax, below; Dugulorn, at the end of this text), random weights, bf16: prefill and decode throughput of whole models through
the step function, and every kernel of the Givirax parts beside the like kernel of the Qwen3 parts, each with its
fraction of its own roofline (bytes it must move over the measured copy bandwidth, or flops over the measured bf16 peak).

    python bench.py --design givirax            (or: python -m cppvllm_b200.design_bench)

Sizes: "small" has Qwen3-0.6B's layer sizes (width 1,024, 16 query and 8 kv heads of 128, inner size 3,072), "large"
Qwen3-8B's (4,096, 32 and 8 heads of 128, 12,288), a few layers each.  The Givirax model of a size has the same width,
heads and head size, a window of 1,024 positions with 4 kept first tokens, and alternates a dense tanh-GELU feed-forward
of the same inner size with 8 gated experts, 2 per token, of half that inner size each (the same flops per token as the
dense gated feed-forward of Qwen3).  Timing: CUDA events around steps that are already warm, buffers rotated or larger
than the L2 for single kernels.

    python bench.py --design dugulorn

The Dugulorn model of a size has the same width and inner size; its layers repeat the pattern [latent attention with a
feed-forward, lightning, latent attention reading the first one's cache with a feed-forward, channel delta]: as many heads as
Qwen3's query heads, latent entries of 96 + 32 elements (the largest the tensor-core kernel takes), matrices of dim x dim per
head in the two recurrent mixers.  Its kernels are timed beside the Qwen3 kernels that do the like job: latent attention
beside grouped-query attention (prompt and decode), the two scans beside prompt attention (both are the mixer's core over
2,048 tokens) and, for decoded tokens, as bytes of state over the copy bandwidth, the norm behind a sublayer beside the
fused add-and-norm, bias and squared relu beside SwiGLU.

    python bench.py --design lorulix

The Lorulix model of a size has the same width, heads and head size; its layers repeat the pattern [attention with a dense
clamped feed-forward, head delta with experts, attention reading the first one's cache with experts, head delta with a dense
feed-forward]: a distance table of 32 rows up to distance 1,024, a query temperature, input convolutions of 4 taps, 8
squared-relu experts of half the inner size, 2 per token, with a shared expert.  Whole models stand beside Givirax (the closest
existing model: a float32 stream, attention over cache entries, routed experts) and Qwen3; its kernels beside the like kernels of
Givirax (attention, experts), Dugulorn (the delta rule, the norm behind a sublayer) and Qwen3 (the projection's epilogue, the
activation).
    python bench.py --design rumurax

The Rumurax model of a size has the same width, heads and head size; two residual streams; its layers repeat the pattern
[attention with a rotation behind a window of 1,024 tokens and pooled blocks of 64, chunked attention (chunks of 1,024, capped
scores, distance term, sink, gate per head), attention over a latent of 96 + 32 elements, chunked attention], every layer with 8
gated experts, 2 per token, of half the inner size, whose logistic scores multiply their inputs, and a shared expert of the same
size.  Whole models stand beside Givirax (the closest existing model: a float32 stream, attention over cache entries behind a
window, routed gated experts) and Qwen3; its kernels beside the like kernels of Lorulix (attention over entries of a key and its
value), Givirax (the stream update, the router, the experts), Qwen3 (the projection's epilogue) and Dugulorn (the gate).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import shutil
import sys
import tempfile
import time

import torch

SIZES = {
    "small": dict(width=1024, heads=16, kv_heads=8, dim=128, ff=3072, layers=8, vocab=32000),
    "large": dict(width=4096, heads=32, kv_heads=8, dim=128, ff=12288, layers=4, vocab=32000),
}
WINDOW, KEEP, EXPERTS, TOP = 1024, 4, 8, 2
BIAS_ROWS, BIAS_FAR = 32, 1024


def givirax_config(s, max_positions):
    mixer = {"dim": s["dim"], "heads": s["heads"], "kv_heads": s["kv_heads"], "vdim": s["dim"], "scale": 1.0 / math.sqrt(s["dim"]),
             "mask": {"size": WINDOW, "keep_first": KEEP}}
    dense = {"kind": "dense", "ff": s["ff"]}
    moe = {"kind": "moe", "expert": {"ff": s["ff"] // 2}, "router": {"experts": EXPERTS, "top": TOP}}
    layers = [{"type": "attention", "mixer": mixer, "mlp": dense if i % 2 == 0 else moe} for i in range(s["layers"])]
    return {"architecture": "Givirax", "vocab": s["vocab"], "width": s["width"], "max_positions": max_positions,
            "embedding": {"scale": math.sqrt(s["width"])}, "norm": {"eps": 1e-5}, "layers": layers}


def dugulorn_config(s, max_positions):
    D, H, hd = s["width"], s["heads"], s["dim"]
    rot = {"dims": 32, "base": 1.0e6, "scaling": {"factor": 8.0, "original": 4096, "fast": 16.0, "slow": 2.0}}

    def latent(src=None):
        m = {"heads": H, "dim": hd, "rot_dim": 32, "vdim": hd, "q_rank": 3 * D // 8, "kv_rank": 96, "scale": 1.0 / math.sqrt(hd + 32), "rot": rot}
        if src is not None:
            m["kv_from"] = src
        return {"type": "latent_attention", "mixer": m, "mlp": {"kind": "dense", "ff": s["ff"]}}
    layers = []
    for i in range(0, s["layers"], 4):
        layers += [latent(),
                   {"type": "lightning", "mixer": {"heads": H, "dim": hd, "vdim": hd, "decay": [1.0 - 2.0 ** -(2 + 6 * h / H) for h in range(H)]}, "mlp": None},
                   latent(i),
                   {"type": "channel_delta", "mixer": {"heads": H, "kv_heads": s["kv_heads"], "dim": hd, "vdim": hd, "conv": 4, "a_rank": 64, "g_rank": 64},
                    "mlp": None}]
    return {"architecture": "Dugulorn", "vocab": s["vocab"], "width": D, "max_positions": max_positions, "norm": {"eps": 1e-5},
            "layers": layers[:s["layers"]]}


def lorulix_config(s, max_positions):
    H, KV, hd, I = s["heads"], s["kv_heads"], s["dim"], s["ff"]

    def attention(src=None):
        m = {"dim": hd, "heads": H, "kv_heads": KV, "vdim": hd, "scale": 1.0 / math.sqrt(hd), "bias_max": BIAS_FAR, "bias_rows": BIAS_ROWS,
             "q_temp": {"coef": 0.25, "every": 128}}
        if src is not None:
            m["kv_from"] = src
        return m
    delta = {"dim": hd, "heads": H, "kv_heads": KV, "vdim": hd, "conv": 4}
    dense = {"kind": "dense", "ff": I, "limit": 7.0}
    moe = {"kind": "moe", "expert": {"ff": I // 2}, "router": {"experts": EXPERTS, "top": TOP, "scale": 1.0}, "shared": {"ff": I // 2}}
    layers = []
    for i in range(s["layers"]):
        k = i % 4
        if k == 0:
            layers.append({"type": "attention", "mixer": attention(), "mlp": dense})
        elif k == 2:
            layers.append({"type": "attention", "mixer": attention(i - 2), "mlp": moe})
        else:
            layers.append({"type": "delta", "mixer": delta, "mlp": moe if k == 1 else dense})
    return {"architecture": "Lorulix", "vocab": s["vocab"], "width": s["width"], "max_positions": max_positions,
            "norm": {"eps": 1e-5}, "canon": {"taps": 4}, "layers": layers}


RX_WINDOW, RX_POOL, RX_CHUNK = 1024, 64, 1024


def rumurax_config(s, max_positions):
    H, KV, hd, I = s["heads"], s["kv_heads"], s["dim"], s["ff"]
    windowed = {"type": "attention_2", "mixer": {"dim": hd, "heads": H, "kv_heads": KV, "vdim": hd, "scale": 1.0 / math.sqrt(hd),
                                                 "mask": {"size": RX_WINDOW, "pool": RX_POOL}, "rot": {"dims": hd, "base": 1.0e6}, "v_mix": True}}
    chunked = {"type": "attention", "mixer": {"dim": hd, "heads": H, "kv_heads": KV, "vdim": hd, "scale": 1.0 / math.sqrt(hd),
                                              "mask": {"size": RX_CHUNK}, "softcap": 30.0, "v_mix": True}}
    latent = {"type": "latent_attention", "mixer": {"heads": H, "dim": hd, "rot_dim": 32, "vdim": hd, "kv_rank": 96,
                                                    "scale": 1.0 / math.sqrt(hd + 32), "rot": {"dims": 32, "base": 1.0e6}}}
    moe = {"kind": "moe", "expert": {"ff": I // 2}, "router": {"experts": EXPERTS, "top": TOP}, "shared": {"ff": I // 2}}
    pattern = [windowed, chunked, latent, chunked]
    return {"architecture": "Rumurax", "vocab": s["vocab"], "width": s["width"], "streams": 2, "norm": {"eps": 1e-5},
            "layers": [dict(pattern[i % 4], mlp=moe) for i in range(s["layers"])]}


def qwen3_config(s, max_positions):
    return dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=s["width"], num_hidden_layers=s["layers"],
                num_attention_heads=s["heads"], num_key_value_heads=s["kv_heads"], head_dim=s["dim"], intermediate_size=s["ff"],
                vocab_size=s["vocab"], rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False,
                max_position_embeddings=max_positions)


def peaks():
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    try:
        with open(os.path.join(here, "MEASURED_PEAKS.json")) as f:
            j = json.load(f)
        return {"hbm_gbs": float(j["hbm_gbs"]), "bf16_tflops": float(j["bf16_tflops"]), "source": "measured"}
    except (OSError, KeyError, ValueError):
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def _events():
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def model_points(cfg, prefill_tokens, batch, context, steps):
    """(prefill tokens/s, decode tokens/s at `batch` requests of `context` tokens, decode tokens/s at batch 1)."""
    from .engine.runner import ModelRunner, StepEntry
    from .weights.random_init import write_random_model
    tmp = tempfile.mkdtemp(prefix="cppvllm_b200_design_")
    try:
        d = write_random_model(os.path.join(tmp, "m"), cfg, seed=0, std=0.02, norm_spread=0.0)
        page = 32
        max_len = max(prefill_tokens, context + 8)
        r = ModelRunner(d, dtype=torch.bfloat16, page_size=page, num_pages=(batch + 1) * ((max_len + page - 1) // page) + 8,
                        max_step_tokens=8192, max_seqs=max(batch, 8), max_model_len=max_len)
        gen = torch.Generator().manual_seed(0)
        vocab = r.vocab_size
        best = float("inf")
        for it in range(4):
            toks = torch.randint(0, vocab, (prefill_tokens,), generator=gen).tolist()
            r.cache.admit("p"); r.cache.reserve("p", prefill_tokens)
            torch.cuda.synchronize()
            e0, e1 = _events()
            e0.record()
            r.step([StepEntry("p", toks, 0, [prefill_tokens - 1])])
            e1.record()
            torch.cuda.synchronize()
            if it:
                best = min(best, e0.elapsed_time(e1))
            r.cache.release("p")
        out = {"prefill_tok_s": round(prefill_tokens / (best / 1e3), 1), "prefill_ms": round(best, 3)}
        for b in (batch, 1):
            ids = [f"d{i}" for i in range(b)]
            ctx0 = context - steps - 8
            for i in ids:
                r.cache.admit(i); r.cache.reserve(i, context + 1)
            fed, per = 0, max(1, 8192 // b)
            while fed < ctx0:
                n = min(per, ctx0 - fed)
                r.step([StepEntry(i, torch.randint(0, vocab, (n,), generator=gen).tolist(), fed, []) for i in ids])
                fed += n
            pos = ctx0
            e0, e1 = _events()
            for s in range(8 + steps):
                if s == 8:
                    torch.cuda.synchronize()
                    e0.record()
                r.step([StepEntry(i, [1 + (s + k) % 100], pos, [0]) for k, i in enumerate(ids)])
                pos += 1
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / steps
            r.check_errors()
            nbytes = r.model.decode_weight_bytes() + sum(
                b * min(context, (cs.window + cs.keep_first) if cs.window else context) * cs.elements_per_token() * 2 * len(m)
                for cs, m in r.group_specs)
            nbytes += sum(b * st[0].numel() * st.element_size() * 2 for st in r.states.values())      # per-request state: read and written
            out[f"decode_b{b}_tok_s"] = round(b / (ms / 1e3), 1)
            out[f"decode_b{b}_ms"] = round(ms, 4)
            out[f"decode_b{b}_hbm_frac"] = round(nbytes / (ms / 1e3) / 1e9 / peaks()["hbm_gbs"], 4)
            for i in ids:
                r.cache.release(i)
        del r
        torch.cuda.empty_cache()
        return out
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


# ---- single kernels, in pairs ------------------------------------------------------------------------------------------

def _us(fn, iters=20):
    from .kernel_bench import _time
    return _time(fn, iters)


def kernel_pairs(s, pk):
    """Each kernel of the Givirax parts beside the like kernel of the Qwen3 parts at the same sizes: microseconds and the
    fraction of its roofline, and how much further from its roofline the new one is (`gap`, 1 = equally far)."""
    from .csrc import ops
    d = torch.device("cuda:0")
    g = torch.Generator(device="cuda").manual_seed(0)
    bf = torch.bfloat16
    D, H, KV, hd, I = s["width"], s["heads"], s["kv_heads"], s["dim"], s["ff"]
    F = I // 2
    page, out = 32, {}

    def rnd(*shape, scale=1.0):
        return (torch.randn(*shape, generator=g, device=d, dtype=torch.float32) * scale).to(bf)

    def pair(name, new_us, new_work, like_us, like_work, unit):
        peak = pk["hbm_gbs"] * 1e9 if unit == "bytes" else pk["bf16_tflops"] * 1e12
        fn, fl = new_work / (new_us * 1e-6) / peak, like_work / (like_us * 1e-6) / peak
        out[name] = {"new_us": round(new_us, 2), "new_frac": round(fn, 4), "like_us": round(like_us, 2), "like_frac": round(fl, 4),
                     "gap": round(fl / fn, 2), "roofline": "copy bandwidth" if unit == "bytes" else "bf16 peak"}

    # -- attention of a prompt of 2,048 tokens behind the window ---------------------------------------------------------
    T = 2048
    n_pages = T // page
    visible = sum(min(p + 1, WINDOW) + (min(KEEP, max(0, p - WINDOW + 1))) for p in range(T))
    flops = 4.0 * H * hd * visible
    tables = torch.arange(n_pages, dtype=torch.int32, device=d).view(1, n_pages)
    cu = torch.tensor([0, T], dtype=torch.int32, device=d)
    pos = torch.arange(T, dtype=torch.int32, device=d)
    keys_pages = rnd(n_pages + 1, KV, page, hd)
    qk = rnd(T, (H + KV) * hd)
    att = torch.empty(T, H * hd, dtype=bf, device=d)
    scale = 1 / math.sqrt(hd)
    tiles = ops.attn_keys_tiles([T], H, KV)
    new = _us(lambda i: ops.attn_keys_bf16(att, qk, keys_pages, tables, cu, pos, 1, tiles, H, KV, hd, page, scale, WINDOW, KEEP))
    kv_pages = rnd(n_pages + 1, 2, KV, page, hd)
    q = rnd(T, H * hd)
    tiles_tc = ops.prefill_tiles_tcgen05([T], H, KV)
    like = _us(lambda i: ops.attn_prefill_tcgen05(att, q, kv_pages, tables, cu, pos, 1, tiles_tc, H, KV, hd, page, scale, window=WINDOW))
    flops_like = 4.0 * H * hd * sum(min(p + 1, WINDOW) for p in range(T))
    pair("attention_prefill_2048", new, flops, like, flops_like, "flops")

    # -- attention of decoded tokens: batch 8 at 4,096 tokens, a window of 1,024 ------------------------------------------
    B, ctx = 8, 4096
    pps = ctx // page
    copies = 8
    tabs = [torch.randperm(B * pps, generator=g, device=d).to(torch.int32).view(B, pps).contiguous() for _ in range(copies)]
    keys_big = [rnd(B * pps + 1, KV, page, hd) for _ in range(copies)]
    kv_big = [rnd(B * pps + 1, 2, KV, page, hd) for _ in range(copies)]
    cu_b = torch.arange(0, B + 1, dtype=torch.int32, device=d)
    pos_b = torch.full((B,), ctx - 1, dtype=torch.int32, device=d)
    qk_b, q_b = rnd(B, (H + KV) * hd), rnd(B, H * hd)
    att_b = torch.empty(B, H * hd, dtype=bf, device=d)
    z = ops.attn_keys_decode_splits(B, KV, WINDOW + KEEP)
    parts = torch.empty(ops.attn_keys_scratch_floats(B, KV, hd, z), dtype=torch.float32, device=d)
    new = _us(lambda i: ops.attn_keys_bf16(att_b, qk_b, keys_big[i % copies], tabs[i % copies], cu_b, pos_b, B, B, H, KV, hd, page,
                                           scale, WINDOW, KEEP, all_single=True, splits=z, scratch=parts))
    splits = 4
    scratch = torch.empty(max(1, ops.attn_decode_scratch_floats(B, KV, hd, splits)), dtype=torch.float32, device=d)
    like = _us(lambda i: ops.attn_decode_bf16(att_b, q_b, kv_big[i % copies], tabs[i % copies], cu_b, pos_b, B, H, KV, hd, page, scale,
                                              splits, scratch, window=WINDOW))
    pair("attention_decode_b8_window_1024", new, B * (WINDOW + KEEP) * KV * hd * 2.0, like, B * WINDOW * KV * hd * 4.0, "bytes")
    del keys_big, kv_big

    # -- the feed-forward of 2,048 tokens: grouped experts beside the dense gated product ---------------------------------
    x = rnd(T, D)
    w_router = torch.randn(EXPERTS, D, generator=g, device=d)
    b_router = torch.zeros(EXPERTS, device=d)
    ids = torch.empty(T, TOP, dtype=torch.int32, device=d)
    wts = torch.empty(T, TOP, dtype=torch.float32, device=d)
    ops.route_topk(ids, wts, x, w_router, b_router)
    wgu, wd = rnd(EXPERTS, 2 * F, D, scale=0.02), rnd(EXPERTS, D, F, scale=0.02)
    y = torch.empty(T, D, dtype=bf, device=d)
    R = ops.grouped_rows_tcgen05(T, TOP, EXPERTS)
    scr2 = dict(tile_expert=torch.empty(R, dtype=torch.int32, device=d), row_token=torch.empty(R, dtype=torch.int32, device=d),
                slot_of=torch.empty(T * TOP, dtype=torch.int32, device=d), xs=torch.empty(R, D, dtype=bf, device=d), hid=torch.empty(R, F, dtype=bf, device=d),
                rows=torch.empty(R, D, dtype=bf, device=d))
    new = _us(lambda i: ops.experts_grouped_tcgen05(y, x, ids, wts, wgu, wd, **scr2))
    w_gate_up, w_down = rnd(2 * I, D, scale=0.02), rnd(D, I, scale=0.02)
    act = torch.empty(T, I, dtype=bf, device=d)
    gu = torch.empty(T, 2 * I, dtype=bf, device=d)

    def dense(i):
        if ops.gated_product_fused(bf, w_gate_up, T):
            ops.gemm_bf16_tcgen05(act, x, w_gate_up, swiglu=True)
        else:
            ops.linear(x, w_gate_up, out=gu)
            ops.swiglu(act, gu)
        ops.linear(act, w_down, out=y)
    like = _us(dense)
    pair("feed_forward_2048_tokens", new, 2.0 * T * TOP * 3 * D * F, like, 2.0 * T * 3 * D * I, "flops")
    new = _us(lambda i: ops.route_topk(ids, wts, x, w_router, b_router))
    out["router_2048_tokens"] = {"new_us": round(new, 2), "note": "no like kernel in the closest model"}

    # -- the feed-forward of 8 decoded tokens --------------------------------------------------------------------------------
    copies = max(2, int(300e6 // (wgu.numel() * 2 + wd.numel() * 2)) + 1)
    wgus, wds = [wgu] + [rnd(EXPERTS, 2 * F, D, scale=0.02) for _ in range(copies - 1)], [wd] + [rnd(EXPERTS, D, F, scale=0.02) for _ in range(copies - 1)]
    x8, y8 = x[:8].contiguous(), torch.empty(8, D, dtype=bf, device=d)
    ids8, wts8 = ids[:8].contiguous(), wts[:8].contiguous()
    hid8 = torch.empty(8 * TOP, F, dtype=bf, device=d)
    rows_us = _us(lambda i: ops.expert_rows(y8, hid8, x8, ids8, wts8, wgus[i % copies], wds[i % copies]))
    from .parts.base import Workspace
    ws8 = Workspace(d, 8)
    new = _us(lambda i: ops.routed_experts(y8, x8, ids8, wts8, wgus[i % copies], wds[i % copies], workspace=ws8))
    used = len(set(ids8.flatten().tolist()))
    dense_copies = max(2, int(300e6 // (w_gate_up.numel() * 2 + w_down.numel() * 2)) + 1)
    wgs = [w_gate_up] + [rnd(2 * I, D, scale=0.02) for _ in range(dense_copies - 1)]
    wdn = [w_down] + [rnd(D, I, scale=0.02) for _ in range(dense_copies - 1)]
    act8, gu8 = torch.empty(8, I, dtype=bf, device=d), torch.empty(8, 2 * I, dtype=bf, device=d)

    def dense8(i):
        ops.project_rows(x8, wgs[i % dense_copies], gu8, 8)
        ops.swiglu(act8, gu8)
        ops.project_rows(act8, wdn[i % dense_copies], y8, 8)
    dense8(0)
    like = _us(dense8)
    pair("feed_forward_8_decoded_tokens", new, used * 3.0 * D * F * 2, like, 3.0 * D * I * 2, "bytes")
    out["feed_forward_8_decoded_tokens"]["pair_by_pair_us"] = round(rows_us, 2)
    out["feed_forward_8_decoded_tokens"]["experts_in_use"] = used
    del wgus, wds, wgs, wdn

    # -- the residual update with its norm, and the activation, 2,048 tokens ---------------------------------------------------
    h32 = torch.randn(T, D, generator=g, device=d)
    d1, d2, normed = rnd(T, D), rnd(T, D), torch.empty(T, D, dtype=bf, device=d)
    w = torch.ones(D, device=d)
    new = _us(lambda i: ops.resid_update(h32, (d1, d2), norm_weight=w, eps=1e-5, out=normed))
    h16 = rnd(T, D)
    like = _us(lambda i: ops.add_rmsnorm(normed, h16, d1, w, 1e-6))
    pair("residual_add_and_norm_2048_tokens", new, T * D * (4 + 4 + 2 + 2 + 2.0), like, T * D * (2 + 2 + 2 + 2.0), "bytes")
    up = rnd(T, I)
    new = _us(lambda i: ops.gelu_tanh(up, up))
    gu_t = rnd(T, 2 * I)
    like = _us(lambda i: ops.swiglu(act, gu_t))
    pair("activation_2048_tokens", new, T * I * 4.0, like, T * I * 6.0, "bytes")
    return out


def dugulorn_kernel_pairs(s, pk):
    """The kernels that the Dugulorn parts brought, each beside the Qwen3 kernel that does the like job at the same sizes."""
    from .csrc import ops
    d = torch.device("cuda:0")
    g = torch.Generator(device="cuda").manual_seed(0)
    bf, f32 = torch.bfloat16, torch.float32
    D, H, KV, hd, I = s["width"], s["heads"], s["kv_heads"], s["dim"], s["ff"]
    R, dr = 96, 32
    HD = R + dr
    page, out = 32, {}

    def rnd(*shape, scale=1.0, dtype=bf):
        return (torch.randn(*shape, generator=g, device=d, dtype=f32) * scale).to(dtype)

    def pair(name, new_us, new_work, like_us, like_work, unit, note=None):
        peak = pk["hbm_gbs"] * 1e9 if unit == "bytes" else pk["bf16_tflops"] * 1e12
        fn, fl = new_work / (new_us * 1e-6) / peak, like_work / (like_us * 1e-6) / peak
        out[name] = {"new_us": round(new_us, 2), "new_frac": round(fn, 4), "like_us": round(like_us, 2), "like_frac": round(fl, 4),
                     "gap": round(fl / fn, 2), "roofline": "copy bandwidth" if unit == "bytes" else "bf16 peak"}
        if note:
            out[name]["note"] = note

    # -- attention of a prompt of 2,048 tokens ---------------------------------------------------------------------------
    T = 2048
    n_pages = T // page
    pairs_seen = T * (T + 1) / 2
    tables = torch.arange(n_pages, dtype=torch.int32, device=d).view(1, n_pages)
    cu = torch.tensor([0, T], dtype=torch.int32, device=d)
    pos = torch.arange(T, dtype=torch.int32, device=d)
    lat_pages = rnd(n_pages + 1, page, HD)
    q_lat = rnd(T, H * HD)
    o_lat = torch.empty(T, H * R, dtype=bf, device=d)
    tiles = ops.attn_keys_tiles([T], H, 1)
    new = _us(lambda i: ops.attn_keys_bf16(o_lat, q_lat, lat_pages, tables, cu, pos, 1, tiles, H, 1, HD, page, 0.09, value_dim=R))
    kv_pages = rnd(n_pages + 1, 2, KV, page, hd)
    q = rnd(T, H * hd)
    att = torch.empty(T, H * hd, dtype=bf, device=d)
    tiles_tc = ops.prefill_tiles_tcgen05([T], H, KV)
    like = _us(lambda i: ops.attn_prefill_tcgen05(att, q, kv_pages, tables, cu, pos, 1, tiles_tc, H, KV, hd, page, 0.09))
    pair("attention_prefill_2048", new, 2.0 * H * (HD + R) * pairs_seen, like, 4.0 * H * hd * pairs_seen, "flops")

    # -- attention of decoded tokens: batch 8 at 4,096 tokens --------------------------------------------------------------
    B, ctx = 8, 4096
    pps = ctx // page
    copies = 8
    tabs = [torch.randperm(B * pps, generator=g, device=d).to(torch.int32).view(B, pps).contiguous() for _ in range(copies)]
    lat_big = [rnd(B * pps + 1, page, HD) for _ in range(copies)]
    kv_big = [rnd(B * pps + 1, 2, KV, page, hd) for _ in range(copies)]
    cu_b = torch.arange(0, B + 1, dtype=torch.int32, device=d)
    pos_b = torch.full((B,), ctx - 1, dtype=torch.int32, device=d)
    ql_b, q_b = rnd(B, H * HD), rnd(B, H * hd)
    ol_b, att_b = torch.empty(B, H * R, dtype=bf, device=d), torch.empty(B, H * hd, dtype=bf, device=d)
    groups = min(n for n in range(1, H + 1) if H % n == 0 and H // n <= 16)      # heads in slabs of at most 16, as the part does
    z = ops.attn_keys_decode_splits(B, groups, ctx)
    parts = torch.empty(max(1, ops.attn_keys_scratch_floats(B, groups, HD, z)), dtype=f32, device=d)
    new = _us(lambda i: ops.attn_keys_bf16(ol_b, ql_b, lat_big[i % copies], tabs[i % copies], cu_b, pos_b, B, B, H, groups, HD, page, 0.09,
                                           all_single=True, splits=z, scratch=parts if z > 1 else None, value_dim=R, kv_heads_in_pages=1))
    splits = 4
    scratch = torch.empty(max(1, ops.attn_decode_scratch_floats(B, KV, hd, splits)), dtype=f32, device=d)
    like = _us(lambda i: ops.attn_decode_bf16(att_b, q_b, kv_big[i % copies], tabs[i % copies], cu_b, pos_b, B, H, KV, hd, page, 0.09,
                                              splits, scratch))
    pair("attention_decode_b8_ctx_4096", new, B * ctx * HD * 2.0, like, B * ctx * KV * hd * 4.0, "bytes")
    del lat_big, kv_big

    # -- the two scans over a prompt of 2,048 tokens, beside prompt attention (the mixer's core in both designs) -----------
    slots = torch.zeros(1, dtype=torch.int32, device=d)
    state = torch.zeros(2, H * hd * hd + 3 * (2 * KV * hd + H * hd), dtype=f32, device=d)
    packed = rnd(T, 4 * H * hd)
    o32 = torch.empty(T, H * hd, dtype=f32, device=d)
    decay = torch.full((H,), 0.99, dtype=f32, device=d)
    qf, kf, vf = (torch.empty(T, H * hd, dtype=f32, device=d) for _ in range(3))
    prep_us = _us(lambda i: ops.lightning_prep(qf, kf, vf, packed, 0, H * hd, 2 * H * hd))
    out["lightning_prep_2048"] = {"new_us": round(prep_us, 2), "new_frac": round(T * 3 * H * hd * 6.0 / (prep_us * 1e-6) / (pk["hbm_gbs"] * 1e9), 4),
                                  "roofline": "copy bandwidth", "note": "no like kernel in the closest model"}
    new = _us(lambda i: ops.lightning_scan(o32, qf, kf, vf, state, decay, cu, slots, 1, H, hd, hd))
    attn_us = out["attention_prefill_2048"]["like_us"]
    out["lightning_prefill_2048"] = {"new_us": round(new, 2), "new_frac": round(4.0 * H * hd * hd * T / (new * 1e-6) / (pk["bf16_tflops"] * 1e12), 5),
                                     "like_us": attn_us, "like_frac": out["attention_prefill_2048"]["like_frac"],
                                     "roofline": "bf16 peak (a token-by-token scan on the float units cannot come near it)"}
    qn, kn = rnd(T, KV * hd, dtype=f32), rnd(T, KV * hd, dtype=f32)
    vv, gg, bb = rnd(T, H * hd, dtype=f32), torch.rand(T, H * hd, generator=g, device=d), torch.rand(T, H, generator=g, device=d)
    new = _us(lambda i: ops.delta_scan(o32, qn, kn, vv, gg, bb, state, cu, slots, 1, H, KV, hd, hd))
    out["delta_prefill_2048"] = {"new_us": round(new, 2), "new_frac": round(6.0 * H * hd * hd * T / (new * 1e-6) / (pk["bf16_tflops"] * 1e12), 5),
                                 "like_us": attn_us, "like_frac": out["attention_prefill_2048"]["like_frac"],
                                 "roofline": "bf16 peak (a token-by-token scan on the float units cannot come near it)"}
    C = 2 * KV * hd + H * hd
    raw, conv_w = rnd(T, C), rnd(C, 4, dtype=f32)
    a32, b32 = rnd(T, H * hd, dtype=f32), rnd(T, H, dtype=f32)
    dt, alog = rnd(H * hd, dtype=f32), rnd(H, dtype=f32)
    seq_of = torch.zeros(T, dtype=torch.int32, device=d)
    new = _us(lambda i: ops.delta_prep(qn, kn, vv, gg, bb, raw, 0, conv_w, a32, dt, alog, b32, state, H * hd * hd, seq_of, cu, slots, H, KV, hd, hd))
    out["delta_prep_2048"] = {"new_us": round(new, 2), "new_frac": round(T * (C * 2 + H * hd * 4 + (2 * KV * hd + 2 * H * hd) * 4.0) / (new * 1e-6) / (pk["hbm_gbs"] * 1e9), 4),
                              "roofline": "copy bandwidth", "note": "no like kernel in the closest model"}

    # -- the scans of 8 decoded tokens: the state is read and written once -------------------------------------------------
    Bs = 8
    n_copy = max(2, int(300e6 // (Bs * H * hd * hd * 4)) + 1)
    states = [torch.zeros(Bs + 1, H * hd * hd, dtype=f32, device=d) for _ in range(n_copy)]
    cu8, slots8 = torch.arange(0, Bs + 1, dtype=torch.int32, device=d), torch.arange(0, Bs, dtype=torch.int32, device=d)
    new = _us(lambda i: ops.lightning_scan(o32[:Bs], qf[:Bs], kf[:Bs], vf[:Bs], states[i % n_copy], decay, cu8, slots8, Bs, H, hd, hd))
    like_d = out["attention_decode_b8_ctx_4096"]
    out["lightning_decode_b8"] = {"new_us": round(new, 2), "new_frac": round(Bs * H * hd * hd * 8.0 / (new * 1e-6) / (pk["hbm_gbs"] * 1e9), 4),
                                  "like_us": like_d["like_us"], "like_frac": like_d["like_frac"], "roofline": "copy bandwidth"}
    new = _us(lambda i: ops.delta_scan(o32[:Bs], qn[:Bs], kn[:Bs], vv[:Bs], gg[:Bs], bb[:Bs], states[i % n_copy], cu8, slots8, Bs, H, KV, hd, hd))
    out["delta_decode_b8"] = {"new_us": round(new, 2), "new_frac": round(Bs * H * hd * hd * 8.0 / (new * 1e-6) / (pk["hbm_gbs"] * 1e9), 4),
                              "like_us": like_d["like_us"], "like_frac": like_d["like_frac"], "roofline": "copy bandwidth"}
    for k in ("lightning_decode_b8", "delta_decode_b8"):
        out[k]["gap"] = round(out[k]["like_frac"] / out[k]["new_frac"], 2)
    del states

    # -- elementwise kernels, 2,048 tokens -------------------------------------------------------------------------------------
    h32 = torch.randn(T, D, generator=g, device=d)
    y, copy = rnd(T, D), torch.empty(T, D, dtype=bf, device=d)
    w, bias = torch.ones(D, device=d), torch.zeros(D, device=d)
    new = _us(lambda i: ops.norm_add(h32, y, w, 1e-5, bias=bias, copy=copy))
    h16, normed = rnd(T, D), torch.empty(T, D, dtype=bf, device=d)
    like = _us(lambda i: ops.add_rmsnorm(normed, h16, y, w, 1e-6))
    pair("norm_behind_sublayer_2048_tokens", new, T * D * (4 + 4 + 2 + 2.0), like, T * D * (2 + 2 + 2 + 2.0), "bytes")
    up, bup = rnd(T, I), torch.zeros(I, device=d)
    new = _us(lambda i: ops.bias_act(up, up, bup, "relu2"))
    gu_t, act = rnd(T, 2 * I), torch.empty(T, I, dtype=bf, device=d)
    like = _us(lambda i: ops.swiglu(act, gu_t))
    pair("activation_2048_tokens", new, T * I * 4.0, like, T * I * 6.0, "bytes")
    o_rows, gate = torch.randn(T, H * hd, generator=g, device=d), rnd(T, H * hd)
    yy = torch.empty(T, H * hd, dtype=bf, device=d)
    wn = torch.ones(hd, device=d)
    new = _us(lambda i: ops.gated_norm(yy, o_rows, gate, wn, H, 1e-5))
    out["gated_norm_2048_tokens"] = {"new_us": round(new, 2), "new_frac": round(T * H * hd * 8.0 / (new * 1e-6) / (pk["hbm_gbs"] * 1e9), 4),
                                     "roofline": "copy bandwidth", "note": "no like kernel in the closest model"}
    return out


def lorulix_kernel_pairs(s, pk):
    """The kernels that the Lorulix parts brought, each beside the like kernel of an existing model at the same sizes (`like`
    names it)."""
    from .csrc import ops
    d = torch.device("cuda:0")
    g = torch.Generator(device="cuda").manual_seed(0)
    bf, f32, i32 = torch.bfloat16, torch.float32, torch.int32
    D, H, KV, hd, I = s["width"], s["heads"], s["kv_heads"], s["dim"], s["ff"]
    F = I // 2
    page, out = 32, {}
    hbm, flop = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12

    def rnd(*shape, scale=1.0, dtype=bf):
        return (torch.randn(*shape, generator=g, device=d, dtype=f32) * scale).to(dtype)

    def pair(name, new_us, new_work, like_us, like_work, unit, like, note=None):
        peak = hbm if unit == "bytes" else flop
        fn, fl = new_work / (new_us * 1e-6) / peak, like_work / (like_us * 1e-6) / peak
        out[name] = {"new_us": round(new_us, 2), "new_frac": round(fn, 4), "like_us": round(like_us, 2), "like_frac": round(fl, 4),
                     "gap": round(fl / fn, 2), "roofline": "copy bandwidth" if unit == "bytes" else "bf16 peak", "like": like}
        if note:
            out[name]["note"] = note

    def alone(name, new_us, work, note="no like kernel in an existing model"):
        out[name] = {"new_us": round(new_us, 2), "new_frac": round(work / (new_us * 1e-6) / hbm, 4), "roofline": "copy bandwidth", "note": note}

    # -- attention of a prompt of 2,048 tokens ---------------------------------------------------------------------------
    T = 2048
    n_pages = T // page
    flops = 4.0 * H * hd * T * (T + 1) / 2
    tables = torch.arange(n_pages, dtype=i32, device=d).view(1, n_pages)
    cu = torch.tensor([0, T], dtype=i32, device=d)
    pos = torch.arange(T, dtype=i32, device=d)
    seq_of = torch.zeros(T, dtype=i32, device=d)
    scale = 1 / math.sqrt(hd)
    entries = rnd(n_pages + 1, KV, page, 2 * hd)
    q = rnd(T, H * hd)
    att = torch.empty(T, H * hd, dtype=bf, device=d)
    bias = rnd(H, BIAS_FAR + 1, dtype=f32)
    tiles = ops.attn_keys_tiles([T], H, KV)
    new = _us(lambda i: ops.attn_bias_bf16(att, q, entries, tables, cu, pos, 1, tiles, H, KV, hd, hd, page, scale, bias))
    keys_pages = rnd(n_pages + 1, KV, page, hd)
    qk = rnd(T, (H + KV) * hd)
    like = _us(lambda i: ops.attn_keys_bf16(att, qk, keys_pages, tables, cu, pos, 1, tiles, H, KV, hd, page, scale))
    pair("attention_prefill_2048", new, flops, like, flops, "flops", "Givirax attn_keys_kernel, no window")
    kv_pages = rnd(n_pages + 1, 2, KV, page, hd)
    tiles_tc = ops.prefill_tiles_tcgen05([T], H, KV)
    like_tc = _us(lambda i: ops.attn_prefill_tcgen05(att, q, kv_pages, tables, cu, pos, 1, tiles_tc, H, KV, hd, page, scale))
    out["attention_prefill_2048"]["qwen3_tcgen05_us"] = round(like_tc, 2)
    out["attention_prefill_2048"]["qwen3_tcgen05_frac"] = round(flops / (like_tc * 1e-6) / flop, 4)

    # -- attention of decoded tokens: batch 8 at 4,096 tokens ---------------------------------------------------------------
    B, ctx = 8, 4096
    pps = ctx // page
    copies = 4
    tabs = [torch.randperm(B * pps, generator=g, device=d).to(i32).view(B, pps).contiguous() for _ in range(copies)]
    ent_big = [rnd(B * pps + 1, KV, page, 2 * hd) for _ in range(copies)]
    keys_big = [rnd(B * pps + 1, KV, page, hd) for _ in range(copies)]
    kv_big = [rnd(B * pps + 1, 2, KV, page, hd) for _ in range(copies)]
    cu_b = torch.arange(0, B + 1, dtype=i32, device=d)
    pos_b = torch.full((B,), ctx - 1, dtype=i32, device=d)
    q_b, qk_b = rnd(B, H * hd), rnd(B, (H + KV) * hd)
    att_b = torch.empty(B, H * hd, dtype=bf, device=d)
    z = ops.attn_keys_decode_splits(B, KV, ctx)
    parts = torch.empty(max(1, ops.attn_keys_scratch_floats(B, KV, hd, z)), dtype=f32, device=d)
    new = _us(lambda i: ops.attn_bias_bf16(att_b, q_b, ent_big[i % copies], tabs[i % copies], cu_b, pos_b, B, B, H, KV, hd, hd, page, scale,
                                           bias, all_single=True, splits=z, scratch=parts))
    like = _us(lambda i: ops.attn_keys_bf16(att_b, qk_b, keys_big[i % copies], tabs[i % copies], cu_b, pos_b, B, B, H, KV, hd, page, scale,
                                            all_single=True, splits=z, scratch=parts))
    pair("attention_decode_b8_ctx_4096", new, B * ctx * KV * hd * 4.0, like, B * ctx * KV * hd * 2.0, "bytes", "Givirax attn_keys_decode_kernel, no window")
    splits = 4
    scratch = torch.empty(max(1, ops.attn_decode_scratch_floats(B, KV, hd, splits)), dtype=f32, device=d)
    like_q = _us(lambda i: ops.attn_decode_bf16(att_b, q_b, kv_big[i % copies], tabs[i % copies], cu_b, pos_b, B, H, KV, hd, page, scale,
                                                splits, scratch))
    out["attention_decode_b8_ctx_4096"]["qwen3_us"] = round(like_q, 2)
    out["attention_decode_b8_ctx_4096"]["qwen3_frac"] = round(B * ctx * KV * hd * 4.0 / (like_q * 1e-6) / hbm, 4)
    del ent_big, keys_big, kv_big

    # -- the projection's epilogue, 2,048 tokens: norms over the whole projections, temperature, cache write ------------------
    packed = rnd(T, (H + 2 * KV) * hd)
    q_out = torch.empty(T, H * hd, dtype=bf, device=d)
    wq, wk = torch.ones(H * hd, device=d), torch.ones(KV * hd, device=d)
    slots_t = torch.arange(T, dtype=i32, device=d)
    new = _us(lambda i: ops.wide_qk_prep(q_out, packed, wq, pos, 1e-5, 0.25, 128, KV, hd, hd, pages=entries, k_weight=wk, slots=slots_t, page_size=page))
    cos, sin = torch.rand(T, hd // 2, generator=g, device=d), torch.rand(T, hd // 2, generator=g, device=d)
    w1 = torch.ones(hd, device=d)
    like = _us(lambda i: ops.qk_norm_rope_kv(q_out, packed, w1, w1, cos, sin, pos, slots_t, kv_pages, H, KV, hd, page, 1e-6))
    moved = T * (H + 2 * KV) * hd * 4.0
    pair("projection_epilogue_2048_tokens", new, moved, like, moved, "bytes", "Qwen3 qk_norm_rope_kv")

    # -- the delta rule with one decay per head: 2,048 tokens of one request, and 8 decoded tokens ----------------------------
    C = 2 * KV * hd + H * hd
    slots1 = torch.zeros(1, dtype=i32, device=d)
    state = torch.zeros(2, H * hd * hd + 3 * C, dtype=f32, device=d)
    o32 = torch.empty(T, H * hd, dtype=f32, device=d)
    qn, kn, vv = rnd(T, KV * hd, dtype=f32, scale=0.05), rnd(T, KV * hd, dtype=f32, scale=0.05), rnd(T, H * hd, dtype=f32)
    g1, gd, bb = torch.rand(T, H, generator=g, device=d), torch.rand(T, H * hd, generator=g, device=d), torch.rand(T, H, generator=g, device=d)
    new = _us(lambda i: ops.delta_scan(o32, qn, kn, vv, g1, bb, state, cu, slots1, 1, H, KV, hd, hd, decay_dim=1))
    like = _us(lambda i: ops.delta_scan(o32, qn, kn, vv, gd, bb, state, cu, slots1, 1, H, KV, hd, hd))
    work = 6.0 * H * hd * hd * T
    pair("delta_prefill_2048", new, work, like, work, "flops", "Dugulorn delta_scan with a decay per key channel",
         note="a token-by-token scan on the float units; neither comes near the tensor peak")
    raw, conv_w = rnd(T, C), rnd(C, 4, dtype=f32)
    a1, ad, b32 = rnd(T, H, dtype=f32), rnd(T, H * hd, dtype=f32), rnd(T, H, dtype=f32)
    dt1, dtd, alog = rnd(H, dtype=f32), rnd(H * hd, dtype=f32), rnd(H, dtype=f32)
    new = _us(lambda i: ops.delta_prep(qn, kn, vv, g1, bb, raw, 0, conv_w, a1, dt1, alog, b32, state, H * hd * hd, seq_of, cu, slots1, H, KV, hd, hd, decay_dim=1))
    like = _us(lambda i: ops.delta_prep(qn, kn, vv, gd, bb, raw, 0, conv_w, ad, dtd, alog, b32, state, H * hd * hd, seq_of, cu, slots1, H, KV, hd, hd))
    pair("delta_prep_2048", new, T * (C * 2 + (2 * KV * hd + H * hd) * 4.0 + H * 16.0), like, T * (C * 2 + H * hd * 4 + (2 * KV * hd + 2 * H * hd) * 4.0),
         "bytes", "Dugulorn delta_prep with a decay per key channel")
    Bs = 8
    n_copy = max(2, int(300e6 // (Bs * H * hd * hd * 4)) + 1)
    states = [torch.zeros(Bs + 1, H * hd * hd, dtype=f32, device=d) for _ in range(n_copy)]
    cu8, slots8 = torch.arange(0, Bs + 1, dtype=i32, device=d), torch.arange(0, Bs, dtype=i32, device=d)
    new = _us(lambda i: ops.delta_scan(o32[:Bs], qn[:Bs], kn[:Bs], vv[:Bs], g1[:Bs], bb[:Bs], states[i % n_copy], cu8, slots8, Bs, H, KV, hd, hd, decay_dim=1))
    like = _us(lambda i: ops.delta_scan(o32[:Bs], qn[:Bs], kn[:Bs], vv[:Bs], gd[:Bs], bb[:Bs], states[i % n_copy], cu8, slots8, Bs, H, KV, hd, hd))
    work = Bs * H * hd * hd * 8.0
    pair("delta_decode_b8", new, work, like, work, "bytes", "Dugulorn delta_scan with a decay per key channel")
    del states
    gate16, y16, wn = rnd(T, H * hd), torch.empty(T, H * hd, dtype=bf, device=d), torch.ones(hd, device=d)
    new = _us(lambda i: ops.gated_norm(y16, o32, gate16, wn, H, 1e-5, gate_act="silu"))
    like = _us(lambda i: ops.gated_norm(y16, o32, gate16, wn, H, 1e-5))
    pair("gated_norm_2048_tokens", new, T * H * hd * 8.0, like, T * H * hd * 8.0, "bytes", "Dugulorn gated_norm with the logistic gate")

    # -- the block: input convolution, and the kernel that closes a sublayer ---------------------------------------------------
    a16, x16, yy, zz, nxt = rnd(T, D), torch.empty(T, D, dtype=bf, device=d), rnd(T, D), rnd(T, D), torch.empty(T, D, dtype=bf, device=d)
    h32 = torch.randn(T, D, generator=g, device=d)
    taps = rnd(4, D, dtype=f32)
    hist = torch.zeros(2, 3 * D, dtype=f32, device=d)
    new = _us(lambda i: ops.input_conv(x16, a16, taps, hist, 0, seq_of, cu, slots1))
    alone("input_convolution_2048_tokens", new, T * D * 4.0)
    w, bz = torch.ones(D, device=d), torch.zeros(D, device=d)
    new = _us(lambda i: ops.gated_norm_add(h32, yy, w, 1e-5, gate=zz, gate_bias=bz, next_weight=w, next_eps=1e-5, next_out=nxt,
                                           history=(a16, 4, hist, 0, seq_of, cu, slots1)))
    copy = torch.empty(T, D, dtype=bf, device=d)
    like = _us(lambda i: ops.norm_add(h32, yy, w, 1e-5, bias=bz, copy=copy))
    pair("sublayer_close_2048_tokens", new, T * D * (4 + 4 + 2 + 2 + 2.0), like, T * D * (4 + 4 + 2 + 2.0), "bytes", "Dugulorn norm_add",
         note="also the gate, the next sublayer's norm and the convolution's history")
    h16, normed = rnd(T, D), torch.empty(T, D, dtype=bf, device=d)
    like_q = _us(lambda i: ops.add_rmsnorm(normed, h16, yy, w, 1e-6))
    out["sublayer_close_2048_tokens"]["qwen3_add_rmsnorm_us"] = round(like_q, 2)
    out["sublayer_close_2048_tokens"]["qwen3_add_rmsnorm_frac"] = round(T * D * 8.0 / (like_q * 1e-6) / hbm, 4)

    # -- feed-forwards ---------------------------------------------------------------------------------------------------------
    gu_t, act = rnd(T, 2 * I), torch.empty(T, I, dtype=bf, device=d)
    new = _us(lambda i: ops.glu_clamped(act, gu_t, 7.0, 1.702))
    like = _us(lambda i: ops.swiglu(act, gu_t))
    pair("activation_2048_tokens", new, T * I * 6.0, like, T * I * 6.0, "bytes", "Qwen3 swiglu")
    x = rnd(T, D)
    w_router = torch.randn(EXPERTS + 1, D, generator=g, device=d)
    ids, wts = torch.empty(T, TOP, dtype=i32, device=d), torch.empty(T, TOP, dtype=f32, device=d)
    sg = torch.empty(T, 1, dtype=f32, device=d)
    new = _us(lambda i: ops.route_topk(ids, wts, x, w_router, None, over_all=True, scale=1.0, extra_out=sg))
    w_r8, b_r8 = w_router[:EXPERTS].contiguous(), torch.zeros(EXPERTS, device=d)
    ids2, wts2 = torch.empty(T, TOP, dtype=i32, device=d), torch.empty(T, TOP, dtype=f32, device=d)
    like = _us(lambda i: ops.route_topk(ids2, wts2, x, w_r8, b_r8))
    pair("router_2048_tokens", new, T * D * 2.0, like, T * D * 2.0, "bytes", "Givirax route_topk")
    from .parts.base import Workspace
    ws = Workspace(d, T)
    w_up, w_dn = rnd(EXPERTS, F, D, scale=0.02), rnd(EXPERTS, D, F, scale=0.02)
    w_gu = rnd(EXPERTS, 2 * F, D, scale=0.02)
    y = torch.empty(T, D, dtype=bf, device=d)
    new = _us(lambda i: ops.routed_experts(y, x, ids, wts, w_up, w_dn, workspace=ws, gated=False))
    like = _us(lambda i: ops.routed_experts(y, x, ids2, wts2, w_gu, w_dn, workspace=ws))
    pair("experts_2048_tokens", new, 2.0 * T * TOP * 2 * D * F, like, 2.0 * T * TOP * 3 * D * F, "flops", "Givirax gated experts")
    ws8 = Workspace(d, 8)
    copies = max(2, int(300e6 // (w_gu.numel() * 2 + w_dn.numel() * 2)) + 1)
    ups = [w_up] + [rnd(EXPERTS, F, D, scale=0.02) for _ in range(copies - 1)]
    gus = [w_gu] + [rnd(EXPERTS, 2 * F, D, scale=0.02) for _ in range(copies - 1)]
    dns = [w_dn] + [rnd(EXPERTS, D, F, scale=0.02) for _ in range(copies - 1)]
    x8, y8 = x[:8].contiguous(), torch.empty(8, D, dtype=bf, device=d)
    ids8, wts8, ids28, wts28 = ids[:8].contiguous(), wts[:8].contiguous(), ids2[:8].contiguous(), wts2[:8].contiguous()
    new = _us(lambda i: ops.routed_experts(y8, x8, ids8, wts8, ups[i % copies], dns[i % copies], workspace=ws8, gated=False))
    like = _us(lambda i: ops.routed_experts(y8, x8, ids28, wts28, gus[i % copies], dns[i % copies], workspace=ws8))
    used, used2 = len(set(ids8.flatten().tolist())), len(set(ids28.flatten().tolist()))
    pair("experts_8_decoded_tokens", new, used * 2.0 * D * F * 2, like, used2 * 3.0 * D * F * 2, "bytes", "Givirax gated experts")
    s16, zt = rnd(T, D), torch.rand(T, generator=g, device=d)
    new = _us(lambda i: ops.add_gated_rows(y, s16, zt))
    alone("shared_expert_sum_2048_tokens", new, T * D * 6.0)
    return out


def rumurax_kernel_pairs(s, pk):
    """The kernels that the Rumurax parts brought, each beside the like kernel of an existing model at the same sizes (`like`
    names it)."""
    from .csrc import ops
    from .parts.base import Workspace
    d = torch.device("cuda:0")
    g = torch.Generator(device="cuda").manual_seed(0)
    bf, f32, i32 = torch.bfloat16, torch.float32, torch.int32
    D, H, KV, hd, I = s["width"], s["heads"], s["kv_heads"], s["dim"], s["ff"]
    F = I // 2
    page, out = 32, {}
    hbm, flop = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12

    def rnd(*shape, scale=1.0, dtype=bf):
        return (torch.randn(*shape, generator=g, device=d, dtype=f32) * scale).to(dtype)

    def pair(name, new_us, new_work, like_us, like_work, unit, like, note=None):
        peak = hbm if unit == "bytes" else flop
        fn, fl = new_work / (new_us * 1e-6) / peak, like_work / (like_us * 1e-6) / peak
        out[name] = {"new_us": round(new_us, 2), "new_frac": round(fn, 4), "like_us": round(like_us, 2), "like_frac": round(fl, 4),
                     "gap": round(fl / fn, 2), "roofline": "copy bandwidth" if unit == "bytes" else "bf16 peak", "like": like}
        if note:
            out[name]["note"] = note

    # -- attention of a prompt of 2,048 tokens ---------------------------------------------------------------------------
    T = 2048
    n_pages = T // page
    tables = torch.arange(n_pages, dtype=i32, device=d).view(1, n_pages)
    cu = torch.tensor([0, T], dtype=i32, device=d)
    pos = torch.arange(T, dtype=i32, device=d)
    scale = 1 / math.sqrt(hd)
    q = rnd(T, H * hd)
    att = torch.empty(T, H * hd, dtype=bf, device=d)
    tiles = ops.attn_keys_tiles([T], H, KV)
    r1, r2, sink = torch.rand(H, device=d), torch.rand(H, device=d), torch.randn(H, device=d)
    gate = rnd(T, H)
    ent1 = rnd(n_pages + 1, KV, page, 2 * hd)
    ent2 = rnd(n_pages + 1, 2, KV, page, 2 * hd)
    bias = rnd(H, BIAS_FAR + 1, dtype=f32)
    like = _us(lambda i: ops.attn_bias_bf16(att, q, ent1, tables, cu, pos, 1, tiles, H, KV, hd, hd, page, scale, bias))
    like_flops = 4.0 * H * hd * T * (T + 1) / 2
    seen = sum(p % RX_CHUNK + 1 for p in range(T))
    new = _us(lambda i: ops.attn_masked_bf16(att, q, ent1, tables, cu, pos, 1, tiles, H, KV, hd, hd, page, scale, chunk=RX_CHUNK, softcap=30.0,
                                             r1=r1, r2=r2, sink=sink, gate=gate))
    pair("attention_chunked_prefill_2048", new, 4.0 * H * hd * seen, like, like_flops, "flops", "Lorulix attn_bias_kernel, all earlier keys",
         note="chunks of 1,024: half the keys of the like kernel; cap, distance term, sink and gate on the score fragments")
    seen = sum(min(p + 1, RX_WINDOW) + max(0, (p - RX_WINDOW + 1) // RX_POOL) for p in range(T))
    new = _us(lambda i: ops.attn_masked_bf16(att, q, ent2, tables, cu, pos, 1, tiles, H, KV, hd, hd, page, scale, planes=2, window=RX_WINDOW,
                                             pool=RX_POOL))
    pair("attention_windowed_prefill_2048", new, 4.0 * H * hd * seen, like, like_flops, "flops", "Lorulix attn_bias_kernel, all earlier keys",
         note="a window of 1,024 and the pooled blocks before it")
    kv_pages = rnd(n_pages + 1, 2, KV, page, hd)
    tiles_tc = ops.prefill_tiles_tcgen05([T], H, KV)
    like_tc = _us(lambda i: ops.attn_prefill_tcgen05(att, q, kv_pages, tables, cu, pos, 1, tiles_tc, H, KV, hd, page, scale))
    out["attention_chunked_prefill_2048"]["qwen3_tcgen05_us"] = round(like_tc, 2)
    out["attention_chunked_prefill_2048"]["qwen3_tcgen05_frac"] = round(like_flops / (like_tc * 1e-6) / flop, 4)

    # -- attention of decoded tokens: batch 8 at 4,096 tokens ---------------------------------------------------------------
    B, ctx = 8, 4096
    pps = ctx // page
    copies = 4
    tabs = [torch.randperm(B * pps, generator=g, device=d).to(i32).view(B, pps).contiguous() for _ in range(copies)]
    e1_big = [rnd(B * pps + 1, KV, page, 2 * hd) for _ in range(copies)]
    e2_big = [rnd(B * pps + 1, 2, KV, page, 2 * hd) for _ in range(copies)]
    cu_b = torch.arange(0, B + 1, dtype=i32, device=d)
    pos_b = torch.full((B,), ctx - 1, dtype=i32, device=d)
    q_b, gate_b = rnd(B, H * hd), rnd(B, H)
    att_b = torch.empty(B, H * hd, dtype=bf, device=d)
    z = ops.attn_keys_decode_splits(B, KV, ctx)
    parts = torch.empty(max(1, ops.attn_keys_scratch_floats(B, KV, hd, z)), dtype=f32, device=d)
    like = _us(lambda i: ops.attn_bias_bf16(att_b, q_b, e1_big[i % copies], tabs[i % copies], cu_b, pos_b, B, B, H, KV, hd, hd, page, scale,
                                            bias, all_single=True, splits=z, scratch=parts))
    like_bytes = B * ctx * KV * hd * 4.0
    zm = ops.attn_masked_decode_splits(B, KV, RX_CHUNK)
    new = _us(lambda i: ops.attn_masked_bf16(att_b, q_b, e1_big[i % copies], tabs[i % copies], cu_b, pos_b, B, B, H, KV, hd, hd, page, scale,
                                             chunk=RX_CHUNK, softcap=30.0, r1=r1, r2=r2, sink=sink, gate=gate_b, all_single=True, splits=zm,
                                             scratch=parts))
    pair("attention_chunked_decode_b8_ctx_4096", new, B * RX_CHUNK * KV * hd * 4.0, like, like_bytes, "bytes",
         "Lorulix attn_bias_decode_kernel, 4,096 keys", note="the last token of a chunk: 1,024 keys")
    nb = (ctx - RX_WINDOW) // RX_POOL
    new = _us(lambda i: ops.attn_masked_bf16(att_b, q_b, e2_big[i % copies], tabs[i % copies], cu_b, pos_b, B, B, H, KV, hd, hd, page, scale,
                                             planes=2, window=RX_WINDOW, pool=RX_POOL, all_single=True, splits=zm, scratch=parts))
    pair("attention_windowed_decode_b8_ctx_4096", new, B * (RX_WINDOW + nb) * KV * hd * 4.0, like, like_bytes, "bytes",
         "Lorulix attn_bias_decode_kernel, 4,096 keys", note="1,024 keys and 48 pooled blocks")
    del e1_big, e2_big

    # -- the projection's epilogue, 2,048 tokens: per-head norms, rotation, value mixing, cache write, pooled blocks -----------
    packed = rnd(T, (H + 2 * KV) * hd)
    q_out = torch.empty(T, H * hd, dtype=bf, device=d)
    w1 = torch.ones(hd, device=d)
    slots_t = torch.arange(T, dtype=i32, device=d)
    cos, sin = torch.rand(T, hd // 2, generator=g, device=d), torch.rand(T, hd // 2, generator=g, device=d)
    vf, lam = rnd(T, KV * hd), torch.tensor([0.3], device=d)
    seq_of = torch.zeros(T, dtype=i32, device=d)
    new = _us(lambda i: ops.masked_qkv_prep(q_out, packed, H, KV, hd, hd, 1e-5, q_weight=w1, k_weight=w1, cos=cos, sin=sin, rot=hd, positions=pos,
                                            pages=ent2, slots=slots_t, page_size=page, planes=2, v_first_in=vf, lam=lam))
    like = _us(lambda i: ops.qk_norm_rope_kv(q_out, packed, w1, w1, cos, sin, pos, slots_t, kv_pages, H, KV, hd, page, 1e-6))
    moved = T * (H + 2 * KV) * hd * 4.0
    pair("projection_epilogue_2048_tokens", new, moved + T * KV * hd * 2.0, like, moved, "bytes", "Qwen3 qk_norm_rope_kv", note="also mixes the values")
    new = _us(lambda i: ops.pool_entries(ent2, tables, seq_of, pos, T, KV, 2 * hd, RX_POOL, page))
    out["pooled_blocks_2048_tokens"] = {"new_us": round(new, 2), "new_frac": round(T * KV * 2 * hd * 2.0 * (1 + 1 / RX_POOL) / (new * 1e-6) / hbm, 4),
                                        "roofline": "copy bandwidth", "note": "no like kernel in an existing model"}

    # -- the streams: a sublayer's write and the next one's read and norm, beside the float32 stream update --------------------
    S = 2
    X = torch.randn(T, S * D, generator=g, device=d)
    yy, nxt = rnd(T, D), torch.empty(T, D, dtype=bf, device=d)
    mix, a, b, gw = torch.eye(S, device=d).contiguous(), torch.ones(S, device=d), torch.ones(S, device=d), torch.ones(1, device=d)
    new = _us(lambda i: ops.stream_step(X, S, write=(yy, mix, b), read=(a, gw), eps=1e-5, out=nxt))
    h32, w = torch.randn(T, D, generator=g, device=d), torch.ones(D, device=d)
    like = _us(lambda i: ops.resid_update(h32, (yy,), norm_weight=w, eps=1e-5, out=nxt))
    pair("stream_step_2048_tokens", new, T * D * (S * 8 + 4.0), like, T * D * (8 + 4.0), "bytes", "Givirax resid_update", note="two streams")

    # -- feed-forwards ---------------------------------------------------------------------------------------------------------
    x = rnd(T, D)
    w_router = torch.randn(EXPERTS, D, generator=g, device=d)
    ids, wts = torch.empty(T, TOP, dtype=i32, device=d), torch.empty(T, TOP, dtype=f32, device=d)
    new = _us(lambda i: ops.route_topk(ids, wts, x, w_router, None, logistic=True))
    b_r8 = torch.zeros(EXPERTS, device=d)
    ids2, wts2 = torch.empty(T, TOP, dtype=i32, device=d), torch.empty(T, TOP, dtype=f32, device=d)
    like = _us(lambda i: ops.route_topk(ids2, wts2, x, w_router, b_r8))
    pair("router_2048_tokens", new, T * D * 2.0, like, T * D * 2.0, "bytes", "Givirax route_topk")
    ws = Workspace(d, T)
    w_gu, w_dn = rnd(EXPERTS, 2 * F, D, scale=0.02), rnd(EXPERTS, D, F, scale=0.02)
    y = torch.empty(T, D, dtype=bf, device=d)
    new = _us(lambda i: ops.routed_experts(y, x, ids, wts, w_gu, w_dn, workspace=ws, weight_on_input=True))
    like = _us(lambda i: ops.routed_experts(y, x, ids2, wts2, w_gu, w_dn, workspace=ws))
    work = 2.0 * T * TOP * 3 * D * F
    pair("experts_2048_tokens", new, work, like, work, "flops", "Givirax gated experts", note="the weight scales the rows on their way into the grouped product")
    ws8 = Workspace(d, 8)
    copies = max(2, int(300e6 // (w_gu.numel() * 2 + w_dn.numel() * 2)) + 1)
    gus = [w_gu] + [rnd(EXPERTS, 2 * F, D, scale=0.02) for _ in range(copies - 1)]
    dns = [w_dn] + [rnd(EXPERTS, D, F, scale=0.02) for _ in range(copies - 1)]
    x8, y8 = x[:8].contiguous(), torch.empty(8, D, dtype=bf, device=d)
    ids8, wts8, ids28, wts28 = ids[:8].contiguous(), wts[:8].contiguous(), ids2[:8].contiguous(), wts2[:8].contiguous()
    new = _us(lambda i: ops.routed_experts(y8, x8, ids8, wts8, gus[i % copies], dns[i % copies], workspace=ws8, weight_on_input=True))
    like = _us(lambda i: ops.routed_experts(y8, x8, ids28, wts28, gus[i % copies], dns[i % copies], workspace=ws8))
    used, used2 = len(set(ids8.flatten().tolist())), len(set(ids28.flatten().tolist()))
    pair("experts_8_decoded_tokens", new, used * 3.0 * D * F * 2, like, used2 * 3.0 * D * F * 2, "bytes", "Givirax gated experts")

    # -- the gate per element behind latent attention, beside the gate per head ---------------------------------------------------
    o_h, g_el, g_hd = rnd(H, T, hd), rnd(T, H * hd), rnd(T, H)
    new = _us(lambda i: ops.head_gate(att, o_h, g_el, H, hd, per_element=True))
    like = _us(lambda i: ops.head_gate(att, o_h, g_hd, H, hd))
    pair("gate_2048_tokens", new, T * H * hd * 6.0, like, T * H * hd * 4.0, "bytes", "Dugulorn head_gate, one number per head")
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="design_bench", description=__doc__.split("\n\n")[0])
    ap.add_argument("--design", default="givirax", choices=["givirax", "dugulorn", "lorulix", "rumurax"])
    ap.add_argument("--sizes", default="small,large")
    ap.add_argument("--steps", type=int, default=48)
    ap.add_argument("--no-kernels", action="store_true", help="whole models only")
    ap.add_argument("--no-models", action="store_true", help="single kernels only")
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("design_bench: needs a CUDA device", file=sys.stderr)
        return 2
    from .csrc import ops
    ops.configure_library_matmul()
    pk = peaks()
    result = {"design": a.design, "closest": "Qwen3ForCausalLM", "dtype": "bf16", "data": "synthetic, random weights", "peaks": pk, "sizes": {}}
    if a.design == "givirax":
        result.update(window=WINDOW, keep_first=KEEP, experts=EXPERTS, top=TOP)
    if a.design == "lorulix":
        result.update(closest="Givirax", bias_rows=BIAS_ROWS, bias_far=BIAS_FAR, experts=EXPERTS, top=TOP)
    if a.design == "rumurax":
        result.update(closest="Givirax", window=RX_WINDOW, pool=RX_POOL, chunk=RX_CHUNK, streams=2, experts=EXPERTS, top=TOP)
    for name in a.sizes.split(","):
        s = SIZES[name]
        entry = {"shape": s}
        if not a.no_models:
            t0 = time.time()
            design_config = {"givirax": givirax_config, "dugulorn": dugulorn_config, "lorulix": lorulix_config, "rumurax": rumurax_config}[a.design]
            entry[a.design] = model_points(design_config(s, 4160), 2048, 8, 4096, a.steps)
            if a.design in ("lorulix", "rumurax"):
                entry["givirax"] = model_points(givirax_config(s, 4160), 2048, 8, 4096, a.steps)
            entry["qwen3"] = model_points(qwen3_config(s, 4160), 2048, 8, 4096, a.steps)
            entry["seconds"] = round(time.time() - t0, 1)
        if not a.no_kernels:
            entry["kernels"] = {"givirax": kernel_pairs, "dugulorn": dugulorn_kernel_pairs, "lorulix": lorulix_kernel_pairs,
                                "rumurax": rumurax_kernel_pairs}[a.design](s, pk)
        result["sizes"][name] = entry
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
