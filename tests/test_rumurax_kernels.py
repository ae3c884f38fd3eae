"""The kernels that came with Rumurax, each alone against float64 arithmetic written here or in tests/plain_rumurax.py: the
pass over several residual streams, the projection's epilogue with value mixing and the pooled blocks, attention with chunks,
windows, pooled blocks, cap, distance term, sink and gate (the general kernel in both element types and the tensor-core
form), the logistic router, experts that weigh their input, and the gate per element.  Attention is tested with ONE key
made to dominate (its key aligned with the query, its value large), placed just inside and just outside every edge."""
import math

import numpy as np
import pytest
import torch

import plain_rumurax as plain

pytestmark = pytest.mark.gpu

F = torch.float64
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 2e-5, "bfloat16": 2e-2}


def dev():
    return torch.device("cuda:0")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("S,D", [(1, 64), (2, 50), (3, 352), (4, 96), (8, 40)])
def test_stream_step(dtype, S, D):
    from cppvllm_b200.csrc import ops
    g = torch.Generator().manual_seed(S * 100 + D)
    T, dt = 7, DT[dtype]
    X = torch.randn(T, S, D, generator=g, dtype=F)
    y = torch.randn(T, D, generator=g, dtype=F).to(dt)
    mix = torch.eye(S, dtype=F) + 0.3 * torch.randn(S, S, generator=g, dtype=F)
    b, a = torch.randn(S, generator=g, dtype=F), torch.randn(S, generator=g, dtype=F)
    gw = torch.tensor([1.7], dtype=F)
    Xd = X.float().reshape(T, S * D).to(dev()).contiguous()
    X = Xd.cpu().double().view(T, S, D)
    tab = torch.randn(11, D, generator=g).to(dt)
    toks = torch.randint(0, 11, (T,), generator=g, dtype=torch.int32)
    E = torch.empty(T, S * D, dtype=torch.float32, device=dev())
    ops.stream_embed(E, tab.to(dev()), toks.to(dev()), S)
    assert torch.equal(E.cpu().view(T, S, D), tab[toks.long()].float()[:, None, :].expand(T, S, D))
    out = torch.empty(T, D, dtype=dt, device=dev())
    ops.stream_step(Xd, S, write=(y.to(dev()), mix.float().to(dev()).contiguous(), b.float().to(dev())),
                    read=(a.float().to(dev()), gw.float().to(dev())), eps=1e-5, out=out)
    newX = torch.einsum("sr,tsd->trd", mix.float().double(), X) + b.float().double()[None, :, None] * y.double()[:, None, :]
    u = torch.einsum("s,tsd->td", a.float().double(), newX)
    want = plain.unit_rms(u, 1e-5) * 1.7
    assert float((Xd.cpu().double().view(T, S, D) - newX).abs().max()) < 1e-5 * float(newX.abs().max())
    assert float((out.cpu().double() - want).abs().max()) < TOL[dtype] * float(want.abs().max())
    ops.stream_step(Xd, S, read=(None, None), eps=0.0, out=out)          # the sum of the streams, normed, no weight
    want = plain.unit_rms(Xd.cpu().double().view(T, S, D).sum(1), 0.0)
    assert float((out.cpu().double() - want).abs().max()) < TOL[dtype] * float(want.abs().max())


class Cache:
    """One request of L tokens in shuffled pages; pages nobody owns and the slots behind the request's last token hold NaN."""

    def __init__(self, L, G, E, page, planes, dtype, seed):
        g = torch.Generator().manual_seed(seed)
        self.L, self.page, self.planes = L, page, planes
        n = (L + page - 1) // page
        total = n + 3
        order = torch.randperm(total, generator=g)[:n]
        shape = (total, planes, G, page, E) if planes == 2 else (total, G, page, E)
        self.pages = torch.full(shape, float("nan"), dtype=dtype, device=dev())
        self.table = torch.full((1, n + 2), -1, dtype=torch.int32)
        self.table[0, :n] = order.to(torch.int32)
        pos = torch.arange(L)
        self.slots = (order[pos // page] * page + pos % page).to(torch.int32).to(dev())
        self.table = self.table.to(dev())

    def entries(self, plane=0):
        """[positions, G, E] in float64, in order of position."""
        n = (self.L + self.page - 1) // self.page
        pg = self.pages[self.table[0, :n].long()]
        pg = pg[:, plane] if self.planes == 2 else pg
        return pg.permute(0, 2, 1, 3).reshape(n * self.page, pg.shape[1], -1)[:self.L].double().cpu()


def reference_attention(q, ent, ent_blocks, pos, H, G, dk, dv, scale, chunk, window, pool, cap, r1, r2, sink, gate):
    """q [n, H, dk] float64 for tokens at positions `pos`; ent [L, G, dk + dv]; ent_blocks [L // pool, G, dk + dv] or None."""
    L = ent.shape[0]
    i = torch.tensor(pos)[:, None]
    j = torch.arange(L)[None, :]
    vis = j <= i
    if chunk:
        vis = vis & (j // chunk == i // chunk)
    if window:
        vis = vis & (i - j < window)
    out = torch.zeros(len(pos), H, dv, dtype=F)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ ent[:, g, :dk].T) * scale
        if cap:
            s = cap * torch.tanh(s / cap)
        if r1 is not None:
            s = s - r1[h].double() * torch.log(1.0 + r2[h].double() * (i - j).clamp(min=0).double())
        s = s.masked_fill(~vis, -math.inf)
        vals = ent[:, g, dk:]
        if pool and window:
            nb = ent_blocks.shape[0]
            sb = (q[:, h] @ ent_blocks[:, g, :dk].T) * scale
            sb = sb.masked_fill(~(torch.arange(nb)[None, :] < ((i - window + 1) // pool).clamp(min=0)), -math.inf)
            s = torch.cat([s, sb], dim=1)
            vals = torch.cat([vals, ent_blocks[:, g, dk:]], dim=0)
        top = s.max(dim=1, keepdim=True).values
        if sink is not None:
            top = torch.maximum(top, sink[h].double().expand_as(top))
        e = torch.exp(s - top)
        den = e.sum(dim=1, keepdim=True) + (torch.exp(sink[h].double() - top) if sink is not None else 0.0)
        o = (e / den) @ torch.nan_to_num(vals)
        if gate is not None:
            o = o * torch.sigmoid(gate[:, h:h + 1])
        out[:, h] = o
    return out


CASES = [
    # name, H, G, dk, dv, chunk, window, pool, cap, bias, sink, gate, rot, page, L
    ("chunked", 4, 2, 16, 32, 24, 0, 0, 30.0, True, True, True, 0, 16, 150),
    ("chunk_is_page", 2, 1, 32, 32, 32, 0, 0, 0.0, True, False, False, 0, 32, 100),
    ("windowed_blocks", 4, 2, 32, 48, 0, 40, 8, 0.0, False, False, False, 16, 16, 200),
    ("window_of_one", 2, 2, 16, 16, 0, 1, 1, 0.0, False, False, False, 16, 16, 70),
    ("blocks_wider_than_pages", 8, 2, 64, 64, 0, 20, 24, 0.0, False, True, False, 32, 16, 300),
    ("plain_causal", 3, 1, 128, 128, 0, 0, 0, 0.0, False, False, True, 0, 64, 130),
    ("odd_sizes", 5, 5, 10, 6, 7, 0, 0, 4.0, True, True, True, 0, 16, 60),
    ("odd_windowed", 3, 1, 6, 3, 0, 5, 3, 0.0, False, False, False, 4, 32, 75),
    ("wide_entries_long_blocks", 2, 1, 320, 256, 0, 10, 150, 0.0, False, False, False, 8, 32, 400),
]


@pytest.mark.parametrize("kernel,dtype", [("general", "float32"), ("general", "bfloat16"), ("tensor", "bfloat16")])
@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
@pytest.mark.parametrize("step", ["decoded", "portion_end", "portion_middle"])
def test_masked_attention_with_a_dominating_key_at_every_edge(case, kernel, dtype, step):
    from cppvllm_b200.csrc import ops
    name, H, G, dk, dv, chunk, window, pool, cap, bias, sink, gate, rot, page, L = case
    dt = DT[dtype]
    if kernel == "tensor" and not ops.attn_masked_supported(dt, H, G, dk, dv):
        pytest.skip("sizes the tensor-core kernel does not take")
    planes = 2 if pool else 1
    E = dk + dv
    # the step: the request's last n tokens (one decoded token, a portion that ends the request, or a portion in the
    # middle of what the pages hold: later tokens are in the cache already, as after a preemption, and must not be seen)
    n = {"decoded": 1, "portion_end": 37, "portion_middle": 23}[step]
    end = L if step != "portion_middle" else L - 19
    first = end - n
    last = end - 1
    # keys to make dominant for the step's LAST token: around every edge it has
    lo = 0
    if chunk:
        lo = last // chunk * chunk
    if window:
        lo = max(lo, last - window + 1)
    targets = {last, lo, max(lo - 1, 0), 0, min(lo + 1, last)}
    targets |= {j for j in (page - 1, page, 2 * page - 1, 2 * page) if j <= last}
    if pool and window:
        nb = max(0, (last - window + 1) // pool)
        targets |= {j for j in (nb * pool - 1, nb * pool, nb * pool + pool - 1, (nb - 1) * pool) if 0 <= j <= last}
    worst = 0.0
    for tj, target in enumerate(sorted(targets)):
        g = torch.Generator().manual_seed(1000 * tj + L)
        packed = torch.randn(L, H * dk + G * E + (H if gate else 0), generator=g)
        u = torch.randn(dk, generator=g)
        for h in range(H):
            packed[last, h * dk:(h + 1) * dk] = u
        for kv in range(G):
            packed[target, H * dk + kv * dk: H * dk + (kv + 1) * dk] = u
            packed[target, H * dk + G * dk + kv * dv: H * dk + G * dk + (kv + 1) * dv] = 40.0
        packed = packed.to(dt).to(dev())
        qw, kw = (1 + 0.2 * torch.randn(dk, generator=g)).to(dev()), (1 + 0.2 * torch.randn(dk, generator=g)).to(dev())
        cos = sin = None
        if rot:
            ang = torch.outer(torch.arange(L, dtype=F), 100.0 ** (-torch.arange(0, rot, 2, dtype=F) / rot)) * 0.05
            cos, sin = ang.cos().float().to(dev()).contiguous(), ang.sin().float().to(dev()).contiguous()
        c = Cache(L, G, E, page, planes, dt, seed=tj)
        pos_all = torch.arange(L, dtype=torch.int32, device=dev())
        q_all = torch.empty(L, H * dk, dtype=dt, device=dev())
        ops.masked_qkv_prep(q_all, packed, H, G, dk, dv, 1e-5, q_weight=qw, k_weight=kw, cos=cos, sin=sin, rot=rot, positions=pos_all,
                            pages=c.pages, slots=c.slots, page_size=page, planes=planes)
        seq0 = torch.zeros(L, dtype=torch.int32, device=dev())
        if pool:
            ops.pool_entries(c.pages, c.table, seq0, pos_all, L, G, E, pool, page)
        ent = c.entries(0)
        blocks = None
        if pool:
            blocks = c.entries(1)[:L // pool]
            means = ent[:L // pool * pool].view(L // pool, pool, G, E).mean(1)
            assert float((blocks - means).abs().max()) <= (1e-6 if dtype == "float32" else 8e-3) * max(1.0, float(means.abs().max()))
        # the epilogue itself: norm, rotation, layout
        pk = packed.double().cpu()
        kn = plain.unit_rms(pk[:, H * dk:H * dk + G * dk].view(L, G, dk), 1e-5) * kw.double().cpu()
        if rot:
            a, b = kn[..., 0:rot:2].clone(), kn[..., 1:rot:2].clone()
            cc, ss = cos.double().cpu()[:, None, :], sin.double().cpu()[:, None, :]
            kn[..., 0:rot:2], kn[..., 1:rot:2] = a * cc - b * ss, b * cc + a * ss
        assert float((ent[..., :dk] - kn).abs().max()) < TOL[dtype] * float(kn.abs().max())
        assert float((ent[..., dk:] - pk[:, H * dk + G * dk:H * dk + G * E].view(L, G, dv)).abs().max()) == 0.0
        q = q_all[first:end].contiguous()
        pos = torch.arange(first, end, dtype=torch.int32, device=dev())
        r1 = (0.5 + torch.rand(H, generator=g)).to(dev()) if bias else None
        r2 = (0.2 + torch.rand(H, generator=g)).to(dev()) if bias else None
        sk = (3.0 * torch.randn(H, generator=g)).to(dev()) if sink else None
        gt = packed[first:end, H * dk + G * E:] if gate else None
        out = torch.empty(n, H * dv, dtype=dt, device=dev())
        if kernel == "general":
            ops.attn_masked_general(out, q, c.pages, c.table, seq0[:n], pos, n, H, G, dk, dv, page, 0.25, planes=planes, chunk=chunk,
                                    window=window, pool=pool, softcap=cap, r1=r1, r2=r2, sink=sk, gate=gt)
        else:
            cu = torch.tensor([0, n], dtype=torch.int32, device=dev())
            ops.attn_masked_bf16(out, q, c.pages, c.table, cu, pos, 1, ops.attn_keys_tiles([n], H, G), H, G, dk, dv, page, 0.25,
                                 planes=planes, chunk=chunk, window=window, pool=pool, softcap=cap, r1=r1, r2=r2, sink=sk, gate=gt)
        ops.check_device_errors(dev())
        want = reference_attention(q.double().cpu().view(n, H, dk), ent, blocks, list(range(first, end)), H, G, dk, dv, 0.25, chunk, window,
                                   pool, cap, r1.cpu() if bias else None, r2.cpu() if bias else None, sk.cpu() if sink else None,
                                   gt.double().cpu() if gate else None)
        got = out.double().cpu().view(n, H, dv)
        assert torch.isfinite(got).all()
        err = float((got - want).abs().max()) / max(1.0, float(want.abs().max()))
        worst = max(worst, err)
        assert err < TOL[dtype], f"{name}, key {target} of {last} ({step}): {err:.2e}"
    print(f"{name} {kernel} {dtype} {step}: worst {worst:.2e} over {len(targets)} dominant keys")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_value_mixing_and_kept_values(dtype):
    from cppvllm_b200.csrc import ops
    dt = DT[dtype]
    g = torch.Generator().manual_seed(5)
    T, H, G, dk, dv, page = 20, 2, 2, 8, 6, 16
    packed = torch.randn(T, H * dk + G * (dk + dv), generator=g).to(dt).to(dev())
    c = Cache(T, G, dk + dv, page, 1, dt, 3)
    kept = torch.empty(T, G * dv, dtype=dt, device=dev())
    q = torch.empty(T, H * dk, dtype=dt, device=dev())
    ops.masked_qkv_prep(q, packed, H, G, dk, dv, 1e-5, pages=c.pages, slots=c.slots, page_size=page, v_first_out=kept)
    assert torch.equal(kept, packed[:, H * dk + G * dk:])
    assert torch.equal(q, packed[:, :H * dk])                      # no norm weights, no rotation: the queries pass
    other = torch.randn(T, H * dk + G * (dk + dv), generator=g).to(dt).to(dev())
    lam = torch.tensor([0.3], device=dev())
    ops.masked_qkv_prep(q, other, H, G, dk, dv, 1e-5, pages=c.pages, slots=c.slots, page_size=page, v_first_in=kept, lam=lam)
    want = 0.7 * other[:, H * dk + G * dk:].double().cpu() + 0.3 * kept.double().cpu()
    got = c.entries()[..., dk:].reshape(T, G * dv)
    assert float((got - want).abs().max()) < TOL[dtype] * float(want.abs().max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,D,E,top,I,shared,kernel", [(1, 64, 4, 2, 32, 16, ""), (9, 50, 5, 5, 12, 0, "rows"), (70, 128, 8, 3, 64, 32, "tcgen05"),
                                                        (300, 256, 6, 2, 48, 96, ""), (5, 96, 1, 1, 24, 8, "")])
def test_logistic_router_and_experts_that_weigh_their_input(dtype, T, D, E, top, I, shared, kernel):
    from cppvllm_b200.csrc import ops
    dt = DT[dtype]
    g = torch.Generator().manual_seed(T + D)
    w = {"router": (torch.randn(E, D, generator=g) * 0.5).to(torch.bfloat16).double()}
    for e in list(range(E)):
        for nme, shape in (("gate", (I, D)), ("up", (I, D)), ("down", (D, I))):
            w[f"e{e}.{nme}"] = (torch.randn(shape, generator=g) * 0.15).to(torch.bfloat16).double()
    x = torch.randn(T, D, generator=g).to(dt)
    z = x.double() @ w["router"].T
    srt = torch.sort(z, dim=1, descending=True).values
    if top < E:                                                  # no close calls: nudge the tokens that have one
        close = (srt[:, top - 1] - srt[:, top]) < 0.05
        x[close] = x[close] * 1.5
        z = x.double() @ w["router"].T
    xd = x.to(dev())
    ids = torch.empty(T, top, dtype=torch.int32, device=dev())
    wts = torch.empty(T, top, dtype=torch.float32, device=dev())
    ops.route_topk(ids, wts, xd, w["router"].float().to(dev()), None, logistic=True)
    best = torch.topk(z, top, dim=1)
    assert torch.equal(ids.cpu().long(), best.indices)
    assert float((wts.cpu().double() - torch.sigmoid(best.values)).abs().max()) < 1e-5
    gu = torch.stack([torch.cat([w[f"e{e}.gate"], w[f"e{e}.up"]]) for e in range(E)]).to(dt).to(dev())
    dn = torch.stack([w[f"e{e}.down"] for e in range(E)]).to(dt).to(dev())
    y = torch.empty(T, D, dtype=dt, device=dev())
    if kernel == "tcgen05" and dtype != "bfloat16":
        kernel = "rows"
    ops.routed_experts(y, xd, ids, wts, gu, dn, kernel=kernel, weight_on_input=True)
    ops.check_device_errors(dev())
    want = plain.routed_experts(x.double(), w, "", {"router": {"experts": E, "top": top}}, rnd=plain.to_bf16 if dtype == "bfloat16" else plain.identity)
    err = float((y.cpu().double() - want).abs().max()) / float(want.abs().max())
    assert err < (3e-5 if dtype == "float32" else 3e-2), err


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gate_per_element(dtype):
    from cppvllm_b200.csrc import ops
    dt = DT[dtype]
    g = torch.Generator().manual_seed(9)
    T, H, dv = 6, 3, 10
    o = torch.randn(H, T, dv, generator=g).to(dt).to(dev())
    packed = torch.randn(T, 7 + H * dv, generator=g).to(dt).to(dev())
    out = torch.empty(T, H * dv, dtype=dt, device=dev())
    ops.head_gate(out, o, packed[:, 7:], H, dv, per_element=True)
    want = o.double().cpu().permute(1, 0, 2).reshape(T, H * dv) * torch.sigmoid(packed[:, 7:].double().cpu())
    assert float((out.double().cpu() - want).abs().max()) < TOL[dtype] * float(want.abs().max())


@pytest.mark.parametrize("splits", [1, 2, 4])
@pytest.mark.parametrize("page", [16, 32])
@pytest.mark.parametrize("kind", ["chunked", "windowed", "causal"])
def test_decoded_tokens_of_several_requests(kind, page, splits):
    """The form for steps of one token per request (tiles shared out among warps and blocks, parts merged, the sink and the gate
    joined once at the merge) against the general kernel, over requests of unequal lengths in shuffled pages."""
    from cppvllm_b200.csrc import ops
    g = torch.Generator().manual_seed(11)
    H, G, dk, dv = 6, 3, 32, 48                     # pages of 32 tokens hold a tile of the decode form whole: one page lookup per tile
    chunk, window, pool, cap = (80, 0, 0, 15.0) if kind == "chunked" else ((0, 100, 10, 0.0) if kind == "windowed" else (0, 0, 0, 0.0))
    planes = 2 if pool else 1
    lens = [1, 17, 64, 65, 300, 777, 128, 137]
    B, E = len(lens), dk + dv
    per = [(n + page - 1) // page for n in lens]
    total = sum(per) + 2
    order = torch.randperm(total, generator=g)
    shape = (total, planes, G, page, E) if planes == 2 else (total, G, page, E)
    pages = torch.randn(shape, generator=g).to(torch.bfloat16)
    table = torch.full((B, max(per)), -1, dtype=torch.int32)
    at = 0
    owned = torch.zeros(total, dtype=torch.bool)
    for b, n in enumerate(per):
        table[b, :n] = order[at:at + n].to(torch.int32)
        owned[order[at:at + n]] = True
        last = lens[b] % page
        if last:                                           # NaN behind the request's last token
            pg = int(order[at + n - 1])
            if planes == 2:
                pages[pg, 0, :, last:] = float("nan")
            else:
                pages[pg, :, last:] = float("nan")
        at += n
    pages[~owned] = float("nan")
    pages, table = pages.to(dev()), table.to(dev())
    q = torch.randn(B, H * dk, generator=g).to(torch.bfloat16).to(dev())
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=dev())
    cu = torch.arange(B + 1, dtype=torch.int32, device=dev())
    seq = torch.arange(B, dtype=torch.int32, device=dev())
    r1 = r2 = sk = gt = None
    if kind == "chunked":
        r1, r2 = (0.5 + torch.rand(H, generator=g)).to(dev()), (0.2 + torch.rand(H, generator=g)).to(dev())
        sk = (2.0 * torch.randn(H, generator=g)).to(dev())
        gt = torch.randn(B, H, generator=g).to(torch.bfloat16).to(dev())
    kw = dict(planes=planes, chunk=chunk, window=window, pool=pool, softcap=cap, r1=r1, r2=r2, sink=sk, gate=gt)
    want = torch.empty(B, H * dv, dtype=torch.bfloat16, device=dev())
    ops.attn_masked_general(want, q, pages, table, seq, pos, B, H, G, dk, dv, page, 0.2, **kw)
    got = torch.empty_like(want)
    scratch = torch.empty(ops.attn_keys_scratch_floats(B, G, dv, splits), dtype=torch.float32, device=dev())
    ops.attn_masked_bf16(got, q, pages, table, cu, pos, B, B, H, G, dk, dv, page, 0.2, all_single=True, splits=splits, scratch=scratch, **kw)
    ops.check_device_errors(dev())
    assert torch.isfinite(got.float()).all()
    assert float((got.float() - want.float()).abs().max()) < 2e-2 * max(1.0, float(want.float().abs().max()))
