"""The kernels that Lorulix brought, each alone against the plain functions of tests/plain_lorulix.py (float64): the
convolution in front of a sublayer and the kernel that closes one (gate, norm, sum into the stream, history, the next
norm), continued across portions of every size through state slots that held something else before; the clamped gated
activation; the norm over a whole projection with the query temperature and the cache write; attention with a bias per
head and distance bucket (one key made to dominate: far away, on both sides of a bucket's edge, at page borders, the token's
own, read by a decoded token, by the last token of a portion and from the middle of one); the delta rule with one decay per
head; the router over all experts and ungated squared-relu experts with a gated shared expert."""
import math

import pytest
import torch

import plain_lorulix as plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
F64 = torch.float64


def _ops():
    from cppvllm_b200.csrc import ops
    return ops


def _rand(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float32) * scale


def _dev(t, dtype=None):
    return t.to(DEV, dtype if dtype is not None else t.dtype).contiguous()


def _i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def _close(got, ref, tol):
    got, ref = got.detach().cpu().to(F64), ref.to(F64)
    err = float((got - ref).abs().max()) / max(1.0, float(ref.abs().max()))
    assert err <= tol, f"error {err:.3e} of scale beyond {tol:.1e}"


TOLS = {torch.float32: 3e-6, torch.bfloat16: 1.2e-2}
CUTS = [[1], [2], [5, 1, 1], [17, 2, 16, 1, 33], [70], [1, 1, 1, 1, 2, 3]]


def _steps(lengths_per_request):
    n = max(len(c) for c in lengths_per_request)
    return [[(r, c[i]) for r, c in enumerate(lengths_per_request) if i < len(c)] for i in range(n)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D,K", [(50, 3), (256, 4), (96, 1), (1030, 2), (64, 6)])
def test_a_sublayer_between_its_convolution_and_its_closing_kernel(dtype, D, K):
    """Per request: a_t given; x = a + conv(a); y = 2 x (a stand-in for the sublayer); h += norm(y * sigmoid(z + b)) * w;
    next = norm(h) * w2.  Portions of every size, four requests side by side, then two more in slots the first have left."""
    ops = _ops()
    eps = 1e-5
    taps, w_out, w_next, bias = _rand(D, K, seed=1, scale=0.8), _rand(D, seed=2) * 0.2 + 1, _rand(D, seed=3) * 0.2 + 1, _rand(D, seed=4)
    reqs = [(_rand(sum(c), D, seed=10 + i).to(dtype), _rand(sum(c), D, seed=20 + i).to(dtype), _rand(sum(c), D, seed=30 + i, scale=3.0))
            for i, c in enumerate(CUTS)]                                                   # a, the gate's product, the stream
    front = 7                                                                              # floats of a mixer's state in front
    state = torch.full((4, front + (K - 1) * D + 3), 7.0, dtype=torch.float32, device=DEV)
    slot_of = [2, 0, 3, 1, 2, 0]
    got_x, got_h, got_n = ([[] for _ in CUTS] for _ in range(3))
    at = [0] * len(CUTS)
    for group in ([0, 1, 2, 3], [4, 5]):
        for r in group:
            state[slot_of[r], front:front + (K - 1) * D].zero_()
        for step in _steps([CUTS[r] for r in group]):
            a_rows, z_rows, h_rows, cu, slots, seq_of = [], [], [], [0], [], []
            for i, (gi, n) in enumerate(step):
                r = group[gi]
                a, z, h = reqs[r]
                a_rows.append(a[at[r]:at[r] + n]); z_rows.append(z[at[r]:at[r] + n]); h_rows.append(h[at[r]:at[r] + n]); at[r] += n
                cu.append(cu[-1] + n); slots.append(slot_of[r]); seq_of += [i] * n
            a, z, h = _dev(torch.cat(a_rows)), _dev(torch.cat(z_rows)), _dev(torch.cat(h_rows))
            x = ops.input_conv(torch.empty_like(a), a, _dev(taps.t().contiguous()), state, front, _i32(seq_of), _i32(cu), _i32(slots))
            y = (x.float() * 2).to(dtype)
            nxt = torch.empty_like(a)
            ops.gated_norm_add(h, y, _dev(w_out), eps, gate=z, gate_bias=_dev(bias), next_weight=_dev(w_next), next_eps=eps, next_out=nxt,
                               history=(a, K, state, front, _i32(seq_of), _i32(cu), _i32(slots)))
            for i, (gi, n) in enumerate(step):
                r = group[gi]
                got_x[r].append(x[cu[i]:cu[i + 1]].cpu()); got_h[r].append(h[cu[i]:cu[i + 1]].cpu()); got_n[r].append(nxt[cu[i]:cu[i + 1]].cpu())
    ops.check_device_errors(torch.device(DEV))
    tol = TOLS[dtype]
    for r, (a, z, h) in enumerate(reqs):
        a64 = a.to(F64)
        x = plain.with_input_conv(a64, taps.to(F64))
        _close(torch.cat(got_x[r]), x, tol)
        y = torch.cat(got_x[r]).float().mul(2).to(dtype).to(F64)                           # the stand-in, as the kernel received it
        hh = h.to(F64) + plain.unit_rms(y * plain.logistic(z.to(F64) + bias.to(F64)), eps) * w_out.to(F64)
        _close(torch.cat(got_h[r]), hh, 3e-6)
        _close(torch.cat(got_n[r]), plain.unit_rms(hh, eps) * w_next.to(F64), tol)
    assert float(state[:, :front].min()) == 7.0 and float(state[:, front + (K - 1) * D:].min()) == 7.0      # nothing around the history was touched


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,I,limit", [(5, 40, 0.7), (33, 256, 1.0), (2, 1030, 3.0)])
def test_clamped_gated_activation_and_a_gated_sum(dtype, T, I, limit):
    ops = _ops()
    gu = _rand(T, 2 * I, seed=5, scale=2.0).to(dtype)
    got = ops.glu_clamped(torch.empty(T, I, dtype=dtype, device=DEV), _dev(gu), limit, 1.702)
    g = torch.clamp(gu[:, :I].to(F64), max=limit)
    u = torch.clamp(gu[:, I:].to(F64), min=-limit, max=limit)
    _close(got, g * plain.logistic(1.702 * g) * (u + 1), TOLS[dtype])
    y, s, z = _rand(T, I, seed=6).to(dtype), _rand(T, I, seed=7).to(dtype), _rand(T, 3, seed=8, scale=2.0)
    zz = _dev(z)
    got = ops.add_gated_rows(_dev(y), _dev(s), zz[:, 1])                                    # a column of a wider tensor
    _close(got, y.to(F64) + plain.logistic(z[:, 1:2].to(F64)) * s.to(F64), TOLS[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dk,dv,page,coef,every", [(3, 1, 16, 24, 16, 0.4, 5), (6, 2, 64, 64, 16, 0.3, 16), (5, 5, 10, 6, 64, 1.0, 1),
                                                       (4, 2, 32, 64, 32, 0.0, 7), (2, 1, 40, 40, 32, 0.5, 0)])
def test_norm_over_a_whole_projection_temperature_and_cache_write(dtype, H, G, dk, dv, page, coef, every):
    ops = _ops()
    T, eps = 23, 1e-5
    nq, nk, nv = H * dk, G * dk, G * dv
    packed = _rand(T, nq + nk + nv, seed=40, scale=2.0).to(dtype)
    wq, wk = _rand(nq, seed=41) * 0.3 + 1, _rand(nk, seed=42) * 0.3 + 1
    positions = [3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 0, 1, 2, 60, 61, 62, 63, 64, 65, 14, 15, 16, 119]
    num_pages = 6
    slots = torch.randperm(num_pages * page, generator=torch.Generator().manual_seed(1))[:T].tolist()
    pages = torch.full((num_pages, G, page, dk + dv), 7.0, dtype=dtype, device=DEV)
    q = ops.wide_qk_prep(torch.empty(T, nq, dtype=dtype, device=DEV), _dev(packed), _dev(wq), _i32(positions), eps, coef, every, G, dk, dv,
                         pages=pages, k_weight=_dev(wk), slots=_i32(slots), page_size=page)
    ops.check_device_errors(torch.device(DEV))
    p64 = packed.to(F64)
    temp = torch.tensor([1.0 + coef * math.log((p + 1) // every + 1) if every else 1.0 for p in positions], dtype=F64)
    _close(q, plain.unit_rms(p64[:, :nq], eps) * wq.to(F64) * temp[:, None], TOLS[dtype])
    k_ref = (plain.unit_rms(p64[:, nq:nq + nk], eps) * wk.to(F64)).reshape(T, G, dk)
    v_ref = p64[:, nq + nk:].reshape(T, G, dv)
    flat = pages.permute(0, 2, 1, 3).reshape(num_pages * page, G, dk + dv)                  # [slot, kv head, entry]
    _close(flat[slots][:, :, :dk], k_ref, TOLS[dtype])
    _close(flat[slots][:, :, dk:], v_ref, 0.0 if dtype == torch.float32 else 1e-9)
    untouched = torch.ones(num_pages * page, dtype=torch.bool)
    untouched[slots] = False
    assert float(flat[untouched].float().min()) == 7.0
    # a layer that reads another's cache writes nothing
    q2 = ops.wide_qk_prep(torch.empty(T, nq, dtype=dtype, device=DEV), _dev(packed[:, :nq]), _dev(wq), _i32(positions), eps, coef, every, G, dk, dv)
    assert torch.equal(q2, q)


def _biased_attention_case(dtype, H, G, dk, dv, page, rows, far, kernel, seed, splits=1):
    """Three requests in one step: a decoded token at position 299, a portion of 40 tokens that ends a context of 200, and a
    portion of 9 tokens in the middle of what its pages hold (the keys behind it must stay unseen).  Every probed token's
    query points at ONE key: the first key, the token's own, its neighbour, both sides of the edge between the exact buckets
    and the logarithmic ones, both sides of a later bucket's edge, the last distance of the table and the ones around it,
    and keys on both sides of page borders; the table's entries are large, so a distance in the wrong bucket shows as well."""
    ops = _ops()
    share, scale = H // G, 0.21
    half = rows // 2
    rel = _rand(rows, H, seed=seed + 1, scale=2.0)
    table = [plain.distance_bucket(n, rows, far) for n in range(far + 1)]
    edge = next(n for n in range(half + 1, far + 1) if table[n] != table[n - 1])             # first distance of a later bucket
    wanted = [0, 1, half - 1, half, half + 1, edge - 1, edge, far - 1, far, far + 1, 2 * far + 3]
    contexts, portions_ = [300, 200, 150], [1, 40, 9]
    held = [300, 200, 170]                                                                   # request 2's pages hold 20 later keys
    n_pages = sum((n + page - 1) // page for n in held) + 2
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    pages = torch.full((n_pages, G, page, dk + dv), float("nan"), dtype=dtype)
    width = max((n + page - 1) // page for n in held)
    tables = torch.full((3, width), -1, dtype=torch.int32)
    keys, values, q_rows, seq_of, positions = [], [], [], [], []
    for s, (ctx_len, n) in enumerate(zip(contexts, portions_)):
        k = _rand(held[s], G, dk, seed=seed + 10 + s).to(dtype)
        v = _rand(held[s], G, dv, seed=seed + 20 + s).to(dtype)
        keys.append(k); values.append(v)
        for b in range((held[s] + page - 1) // page):
            tables[s, b] = perm.pop()
            m = min(page, held[s] - b * page)
            pages[tables[s, b], :, :m, :dk] = k[b * page:b * page + m].transpose(0, 1)
            pages[tables[s, b], :, :m, dk:] = v[b * page:b * page + m].transpose(0, 1)
        q = _rand(n, H, dk, seed=seed + 30 + s, scale=0.3)
        for i in range(n):
            p = ctx_len - n + i
            borders = [p - (p // page) * page, p - (p // page) * page + 1, p]                # the page's first key, the one before it, key 0
            dist = (wanted + borders)[(i + 3 * s) % (len(wanted) + 3)]
            j = p - min(dist, p)
            for h in range(H):
                kt = k[j, h // share].float()
                q[i, h] += 14.0 * kt / (kt @ kt) / scale * (1.0 if h % 2 == 0 else 0.6)
            seq_of.append(s); positions.append(p)
        q_rows.append(q.to(dtype))
    q_all = torch.cat(q_rows).reshape(-1, H * dk)
    T = q_all.shape[0]
    bias = rel[torch.tensor(table)].t().contiguous()                                         # [H, far + 1]
    out = torch.full((T, H * dv), 5.0, dtype=dtype, device=DEV)
    if kernel == "general":
        ops.paged_attention_entries(out, _dev(q_all), _dev(pages), _dev(tables), _i32(seq_of), _i32(positions), H, G, dk, dv, page, scale,
                                    bias=_dev(bias))
    else:
        cu = [0, 1, 41, 50]
        single = kernel == "decode"
        if single:                                                                           # the decode form: one token per request
            keep = [0, 40, 49]
            q_all, seq_of, positions, cu, T = q_all[keep], [0, 1, 2], [positions[i] for i in keep], [0, 1, 2, 3], 3
            out = out[:3]
        ops.attn_bias_bf16(out, _dev(q_all), _dev(pages), _dev(tables), _i32(cu), _i32(positions), 3,
                           ops.attn_keys_tiles([1, 1, 1] if single else portions_, H, G), H, G, dk, dv, page, scale, _dev(bias),
                           all_single=single, splits=splits,
                           scratch=torch.empty(ops.attn_keys_scratch_floats(3, G, dv, splits), dtype=torch.float32, device=DEV) if splits > 1 else None)
    ops.check_device_errors(torch.device(DEV))
    ref = torch.zeros(T, H, dv, dtype=F64)
    qq = q_all.to(F64).reshape(T, H, dk)
    for t in range(T):
        s, p = seq_of[t], positions[t]
        k, v = keys[s].to(F64), values[s].to(F64)
        buckets = torch.tensor([plain.distance_bucket(p - j, rows, far) for j in range(p + 1)])
        for h in range(H):
            sc = (k[:p + 1, h // share] @ qq[t, h]) * scale + rel.to(F64)[buckets, h]
            ref[t, h] = torch.softmax(sc, 0) @ v[:p + 1, h // share]
    _close(out.reshape(T, H, dv), ref, 2e-5 if dtype == torch.float32 else 2.5e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dk,dv,page,rows,far", [(3, 1, 16, 24, 16, 8, 20), (6, 2, 64, 64, 16, 32, 100), (5, 5, 10, 6, 64, 4, 3),
                                                     (4, 2, 32, 64, 32, 12, 50), (2, 1, 40, 40, 32, 16, 290)])
def test_attention_with_a_bias_per_distance_bucket_general(dtype, H, G, dk, dv, page, rows, far):
    _biased_attention_case(dtype, H, G, dk, dv, page, rows, far, "general", seed=600)


CASES_TC = [(6, 2, 64, 64, 16, 32, 100), (4, 2, 32, 64, 32, 12, 50), (8, 4, 96, 80, 64, 24, 200), (3, 1, 16, 48, 16, 8, 20),
            (16, 1, 128, 128, 64, 16, 290), (4, 4, 64, 32, 16, 4, 3)]


@pytest.mark.parametrize("H,G,dk,dv,page,rows,far", CASES_TC)
def test_attention_with_a_bias_per_distance_bucket_tensor_cores(H, G, dk, dv, page, rows, far):
    assert _ops().attn_bias_supported(torch.bfloat16, H, G, dk, dv)
    _biased_attention_case(torch.bfloat16, H, G, dk, dv, page, rows, far, "portions", seed=700)


@pytest.mark.parametrize("splits", [1, 4])
@pytest.mark.parametrize("H,G,dk,dv,page,rows,far", CASES_TC)
def test_attention_with_a_bias_tensor_core_decode_form(H, G, dk, dv, page, rows, far, splits):
    """One token per request; with `splits` several blocks share a request's keys and a second kernel merges their parts."""
    _biased_attention_case(torch.bfloat16, H, G, dk, dv, page, rows, far, "decode", seed=800, splits=splits)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dk,dv,taps", [(4, 2, 12, 20, 2), (2, 2, 64, 64, 3), (3, 1, 40, 33, 1), (1, 1, 5, 3, 6), (4, 2, 32, 64, 3), (2, 1, 128, 16, 4)])
def test_delta_rule_with_one_decay_per_head_continues_across_portions_and_slots(dtype, H, G, dk, dv, taps):
    """The decays' logarithms are low (a state that remembers the whole sequence), so a state that is lost, scaled by the
    wrong head's decay or continued from another request's slot shows in every later token."""
    ops = _ops()
    C = 2 * G * dk + H * dv
    mat = H * dk * dv
    conv_w = _rand(C, taps, seed=500, scale=0.6)
    dt_bias, a_log = _rand(H, seed=501), _rand(H, seed=502) - 3.0
    reqs = [(_rand(sum(c), 2 + C, seed=510 + i).to(dtype), _rand(sum(c), H, seed=520 + i), _rand(sum(c), H, seed=530 + i))
            for i, c in enumerate(CUTS)]
    state = torch.full((4, mat + (taps - 1) * C + 2), 7.0, dtype=torch.float32, device=DEV)
    slot_of = [2, 0, 3, 1, 2, 0]
    got = [[] for _ in CUTS]
    at = [0] * len(CUTS)
    f32 = dict(dtype=torch.float32, device=DEV)
    for group in ([0, 1, 2, 3], [4, 5]):
        for r in group:
            state[slot_of[r], :mat + (taps - 1) * C].zero_()
        for step in _steps([CUTS[r] for r in group]):
            rows, arows, brows, cu, slots, seq_of = [], [], [], [0], [], []
            for i, (gi, n) in enumerate(step):
                r = group[gi]
                x, a, b = reqs[r]
                rows.append(x[at[r]:at[r] + n]); arows.append(a[at[r]:at[r] + n]); brows.append(b[at[r]:at[r] + n]); at[r] += n
                cu.append(cu[-1] + n); slots.append(slot_of[r]); seq_of += [i] * n
            packed, T = _dev(torch.cat(rows)), cu[-1]
            qn, kn = torch.empty(T, G * dk, **f32), torch.empty(T, G * dk, **f32)
            vv, gg, bb = torch.empty(T, H * dv, **f32), torch.empty(T, H, **f32), torch.empty(T, H, **f32)
            ops.delta_prep(qn, kn, vv, gg, bb, packed, 2, _dev(conv_w), _dev(torch.cat(arows)), _dev(dt_bias), _dev(a_log),
                           _dev(torch.cat(brows)), state, mat, _i32(seq_of), _i32(cu), _i32(slots), H, G, dk, dv, decay_dim=1)
            ops.conv_history(state, mat, packed, 2, C, taps, _i32(cu), _i32(slots), len(step))
            out = torch.empty(T, H * dv, **f32)
            ops.delta_scan(out, qn, kn, vv, gg, bb, state, _i32(cu), _i32(slots), len(step), H, G, dk, dv, decay_dim=1)
            for i, (gi, n) in enumerate(step):
                got[group[gi]].append(out[cu[i]:cu[i + 1]].cpu())
    ops.check_device_errors(torch.device(DEV))
    share = H // G
    for r, (x, a, b) in enumerate(reqs):
        T = x.shape[0]
        y = plain.silu(plain.causal_conv(x[:, 2:].to(F64), conv_w.to(F64)))
        q = plain.unit_vectors(y[:, :G * dk].reshape(T, G, dk)) * dk ** -0.5
        k = plain.unit_vectors(y[:, G * dk:2 * G * dk].reshape(T, G, dk))
        v = y[:, 2 * G * dk:].reshape(T, H, dv)
        g = torch.exp(-torch.exp(a_log.to(F64)) * plain.softplus(a.to(F64) + dt_bias.to(F64)))
        ref = plain.delta_rule(q.repeat_interleave(share, dim=1), k.repeat_interleave(share, dim=1), v, plain.logistic(b.to(F64)), g)
        _close(torch.cat(got[r]).reshape(T, H, dv), ref, 3e-5)
    assert float(state[:, mat + (taps - 1) * C:].min()) == 7.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,dv", [(4, 20), (2, 64), (3, 33)])
def test_head_norm_with_a_silu_gate(dtype, H, dv):
    ops = _ops()
    T, eps = 19, 1e-5
    o, w = _rand(T, H * dv, seed=60, scale=3.0), _rand(dv, seed=61) * 0.3 + 1
    wide = _rand(T, 5 + H * dv, seed=62, scale=2.0).to(dtype)                                # the gate inside a wider row
    gate = _dev(wide)[:, 5:]
    got = ops.gated_norm(torch.empty(T, H * dv, dtype=dtype, device=DEV), _dev(o), gate, _dev(w), H, eps, gate_act="silu")
    ref = plain.unit_rms(o.to(F64).reshape(T, H, dv), eps) * w.to(F64) * plain.silu(wide[:, 5:].to(F64)).reshape(T, H, dv)
    _close(got.reshape(T, H, dv), ref, TOLS[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,D,E,top,I,shared,scale", [(1, 48, 5, 2, 24, 16, 2.0), (2, 80, 3, 1, 16, 0, 1.0), (37, 96, 4, 4, 32, 32, 1.5),
                                                      (70, 50, 6, 3, 12, 12, 2.5), (300, 192, 10, 3, 80, 48, 2.0)])
def test_router_over_all_experts_and_squared_relu_experts_with_a_gated_shared_one(dtype, T, D, E, top, I, shared, scale):
    """Through the part itself (what the model calls), with the simple kernels and with the ones a step of that size takes."""
    from cppvllm_b200.parts.base import Runtime, Workspace
    from cppvllm_b200.parts.moe import RoutedAct
    dev = torch.device(DEV)
    w = {"f.router": _rand(E, D, seed=70, scale=0.5)}
    for e in range(E):
        w[f"f.e{e}.up"] = _rand(I, D, seed=71 + e, scale=0.2).to(dtype).float()
        w[f"f.e{e}.down"] = _rand(D, I, seed=91 + e, scale=0.2).to(dtype).float()
    if shared:
        w.update({"f.shared.up": _rand(shared, D, seed=111, scale=0.2).to(dtype).float(), "f.shared.down": _rand(D, shared, seed=112, scale=0.2).to(dtype).float(),
                  "f.shared.sg": _rand(1, D, seed=113, scale=0.3)})
    x = _rand(T, D, seed=114).to(dtype)
    cfg = {"router": {"experts": E, "top": top, "scale": scale}, "shared": {"ff": shared} if shared else None}
    ref = plain.routed_experts(x.to(F64), {k: v.to(F64) for k, v in w.items()}, "f.", cfg, plain.identity)
    for plain_kernels in (True, False):
        rt = Runtime(dev, dtype, Workspace(dev, max(T, 8)), plain_kernels=plain_kernels)
        part = RoutedAct(rt, prefix="f.", hidden_size=D, intermediate_size=I, num_experts=E, top=top, scale=scale, shared_size=shared)
        part.bind({k: _dev(v, torch.float32 if ("router" in k or k.endswith(".sg")) else dtype) for k, v in w.items()})
        got = part.forward(_dev(x), None)
        _ops().check_device_errors(dev)
        _close(got, ref, 2e-5 if dtype == torch.float32 else 3e-2)
