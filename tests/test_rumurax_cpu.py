"""The plain Rumurax implementation against closed forms, the test models against the faults they are made to show, and the
configuration reader's refusals.  No GPU."""
import copy
import math

import pytest
import torch

import plain_rumurax as plain
import rumurax_models as rm

F = torch.float64


@pytest.fixture(scope="module")
def rx_dirs(tmp_path_factory):
    return rm.write_all(str(tmp_path_factory.mktemp("rumurax_cpu")))


def test_visibility_of_chunks_windows_and_blocks():
    c = plain.chunk_visible(12, 5)
    assert c[4, 0] and c[4, 4] and not c[5, 4] and c[5, 5] and c[9, 5] and not c[10, 9] and not c[3, 4]
    w = plain.window_visible(20, 4)
    assert w[7, 4] and not w[7, 3] and w[7, 7] and not w[7, 8] and w[2, 0]
    b = plain.blocks_visible(20, 4, 3)              # block b = positions 3b .. 3b + 2, seen once 3b + 2 <= i - 4
    assert not b[5, 0] and b[6, 0] and not b[8, 1] and b[9, 1] and b.shape == (20, 6)
    # a token that has left the window and whose block is not yet seen is not seen at all
    i = 7
    seen_tokens = {j for j in range(20) if w[i, j]}
    seen_through_blocks = {3 * blk + k for blk in range(6) if b[i, blk] for k in range(3)}
    assert seen_tokens == {4, 5, 6, 7} and seen_through_blocks == {0, 1, 2} and 3 not in seen_tokens | seen_through_blocks


def test_rotation_depends_on_the_distance_only_and_leaves_the_rest():
    g = torch.Generator().manual_seed(1)
    q, k = torch.randn(1, 10, generator=g, dtype=F), torch.randn(1, 10, generator=g, dtype=F)
    def score(i, j):
        a = plain.turn_pairs(q, torch.tensor([i]), 6, 50.0)
        b = plain.turn_pairs(k, torch.tensor([j]), 6, 50.0)
        assert torch.equal(a[:, 6:], q[:, 6:])
        return float((a * b).sum())
    assert abs(score(9, 4) - score(105, 100)) < 1e-9 and abs(score(9, 4) - score(9, 5)) > 1e-3
    one = plain.turn_pairs(torch.tensor([[1.0, 0.0, 1.0, 0.0]], dtype=F), torch.tensor([3]), 4, 100.0)
    assert torch.allclose(one, torch.tensor([[math.cos(3.0), math.sin(3.0), math.cos(0.3), math.sin(0.3)]], dtype=F))


def _one_head(sink=None, cap=None, r=None, chunk=100):
    """A chunked layer of one head whose projections are identities on a width of 2."""
    eye = torch.eye(2, dtype=F)
    w = {"q": eye, "k": eye, "v": eye, "o": eye, "q.norm": torch.ones(2, dtype=F), "k.norm": torch.ones(2, dtype=F)}
    m = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 2, "scale": 1.0, "mask": {"size": chunk}}
    if sink is not None:
        w["sink"] = torch.tensor([sink], dtype=F)
    if r is not None:
        w["r1"], w["r2"] = torch.tensor([r[0]], dtype=F), torch.tensor([r[1]], dtype=F)
    if cap:
        m["softcap"] = cap
    return w, m


def test_sink_cap_and_distance_term_in_closed_form():
    h = torch.tensor([[1.0, 0.0], [1.0, 0.0]], dtype=F)          # unit rms makes q = k = (sqrt 2, 0): every score is 2
    w, m = _one_head(sink=2.0)
    y, _ = plain.chunked_attention(h, w, "", m, 0.0, None)
    assert torch.allclose(y[0], h[0] / 2) and torch.allclose(y[1], h[1] * 2 / 3)        # the sink counts once, with weight e^2
    w, m = _one_head(cap=1.0, sink=math.tanh(2.0))
    y, _ = plain.chunked_attention(h, w, "", m, 0.0, None)
    assert torch.allclose(y[0], h[0] / 2)                         # the capped score is tanh(2); the sink is not capped
    w, m = _one_head(r=(1.0, 3.0))
    hv = torch.tensor([[1.0, 0.0], [0.0, 1.0]], dtype=F)
    y, _ = plain.chunked_attention(hv, w, "", m, 0.0, None)
    # token 1: scores 0 - ln(1 + 3) for key 0 and 2 for its own key: weights 1/4 and e^2, over their sum
    a = 0.25 / (0.25 + math.exp(2.0))
    assert torch.allclose(y[1], a * math.sqrt(2) * hv[0] / math.sqrt(2) + (1 - a) * hv[1])
    w, m = _one_head(chunk=1)
    y, _ = plain.chunked_attention(h, w, "", m, 0.0, None)
    assert torch.allclose(y, h)                                   # chunks of one token: every token sees itself only


def test_streams_with_unit_weights_are_the_plain_residual_sum():
    g = torch.Generator().manual_seed(2)
    X = torch.randn(5, 1, 8, generator=g, dtype=F)
    w = {"in": torch.ones(1, dtype=F), "mix": torch.ones(1, 1, dtype=F), "out": torch.ones(1, dtype=F)}
    out = plain.stream_sublayer(X, w, "", torch.tensor(2.0, dtype=F), 1e-5, lambda h: 3 * h)
    assert torch.allclose(out[:, 0], X[:, 0] + 6 * plain.unit_rms(X[:, 0], 1e-5))
    # two streams: the matrix is indexed [from, to]
    X = torch.randn(3, 2, 4, generator=g, dtype=F)
    w = {"in": torch.tensor([1.0, 0.0], dtype=F), "mix": torch.tensor([[0.0, 1.0], [0.0, 0.0]], dtype=F), "out": torch.zeros(2, dtype=F)}
    out = plain.stream_sublayer(X, w, "", torch.tensor(1.0, dtype=F), 0.0, lambda h: h)
    assert torch.equal(out[:, 1], X[:, 0]) and torch.equal(out[:, 0], torch.zeros(3, 4, dtype=F))


def test_experts_weigh_their_input():
    g = torch.Generator().manual_seed(3)
    D, I = 6, 4
    w = {"router": torch.tensor([[10.0] + [0.0] * (D - 1), [-10.0] + [0.0] * (D - 1)], dtype=F)}
    for e in range(2):
        for n, shape in (("gate", (I, D)), ("up", (I, D)), ("down", (D, I))):
            w[f"e{e}.{n}"] = torch.randn(shape, generator=g, dtype=F)
    h = torch.randn(3, D, generator=g, dtype=F)
    h[:, 0] = torch.tensor([0.1, -0.2, 0.05])
    y = plain.routed_experts(h, w, "", {"router": {"experts": 2, "top": 1}})
    for t in range(3):
        e = 0 if h[t, 0] > 0 else 1
        s = torch.sigmoid(w["router"][e] @ h[t])
        z = s * h[t]
        want = w[f"e{e}.down"] @ (plain.silu(w[f"e{e}.gate"] @ z) * (w[f"e{e}.up"] @ z))
        assert torch.allclose(y[t], want)
        on_output = s * (w[f"e{e}.down"] @ (plain.silu(w[f"e{e}.gate"] @ h[t]) * (w[f"e{e}.up"] @ h[t])))
        assert not torch.allclose(y[t], on_output, rtol=1e-3)


def _faulty(monkeypatch, name, fn):
    monkeypatch.setattr(plain, name, fn)


@pytest.mark.parametrize("fault", ["window", "chunk", "blocks", "mix", "sink", "streams", "weights_on_output"])
def test_the_test_models_show_the_faults_they_are_made_for(rx_dirs, monkeypatch, fault):
    """A mask that is one token off, a block seen one token early, values left unmixed, a sink left out, a stream matrix read
    the wrong way round, router weights on the experts' outputs: each moves the logits by far more than the tolerance."""
    name = {"chunk": "rx_a", "sink": "rx_a", "mix": "rx_a"}.get(fault, "rx_a")
    d = rx_dirs[name]
    toks = rm.clear_tokens(d, 90, 1)
    good = plain.forward(d, toks)
    cfg, w = plain.read_config(d), plain.read_weights(d)
    if fault == "window":
        orig = plain.window_visible
        _faulty(monkeypatch, "window_visible", lambda T, size: orig(T, size + 1))
    elif fault == "chunk":
        _faulty(monkeypatch, "chunk_visible", lambda T, size: (torch.arange(T)[None, :] <= torch.arange(T)[:, None])
                & ((torch.arange(T)[:, None] + 1) // size == (torch.arange(T)[None, :] + 1) // size))
    elif fault == "blocks":
        orig = plain.blocks_visible
        _faulty(monkeypatch, "blocks_visible", lambda T, size, pool: orig(T, size - 1, pool))
    elif fault == "mix":
        _faulty(monkeypatch, "mix_values", lambda v, v_first, lam: v)
    elif fault == "sink":
        w = {k: v for k, v in w.items() if not k.endswith(".sink")}
    elif fault == "streams":
        w = {k: (v.T.contiguous() if k.endswith(".mix") and v.dim() == 2 else v) for k, v in w.items()}
    elif fault == "weights_on_output":
        orig = plain.expert
        def on_output(z, ww, p, rnd=plain.identity):
            return orig(z, ww, p, rnd)
        def routed(h, ww, p, f, rnd=plain.identity, margins=None):
            s = torch.sigmoid(h @ ww[p + "router"].T)
            best = torch.topk(s, f["router"]["top"], dim=1)
            y = torch.zeros_like(h)
            for t in range(h.shape[0]):
                for c in range(f["router"]["top"]):
                    e = int(best.indices[t, c])
                    y[t] += s[t, e] * orig(h[t:t + 1], ww, f"{p}e{e}.", rnd)[0]
            return y + (orig(h, ww, p + "shared.", rnd) if f.get("shared") is not None else 0)
        _faulty(monkeypatch, "routed_experts", routed)
    bad = plain.forward_loaded(cfg, w, toks)
    moved = float((bad - good).abs().max()) / float(good.abs().max())
    assert moved > 3e-3, f"{fault}: the logits moved by {moved:.2e} of their size only"


def test_configuration_reader():
    from cppvllm_b200.config.model_config import ConfigError
    from cppvllm_b200.config.rumurax_config import RumuraxConfig
    from cppvllm_b200.config.registry import resolve_architecture
    cfg = RumuraxConfig.from_dict(rm.RX_A)
    assert cfg.streams == 3 and cfg.layers[0].mixer.pool == 4 and cfg.layers[0].mixer.window == 20 and cfg.layers[1].mixer.chunk == 16
    assert cfg.layers[1].mixer.softcap == 5.0 and cfg.layers[2].mixer.kv_rank == 20 and cfg.layers[1].mlp is None
    assert RumuraxConfig.from_dict(rm.RX_D).streams == 0 and RumuraxConfig.from_dict(rm.RX_B).layers[1].mixer.pool == 0
    assert resolve_architecture(rm.RX_A).name == "Rumurax"
    def broken(change):
        d = copy.deepcopy(rm.RX_A)
        change(d)
        with pytest.raises(ConfigError):
            RumuraxConfig.from_dict(d)
    broken(lambda d: d["layers"][0].update(type="attention_3"))
    broken(lambda d: d["layers"][0]["mixer"].pop("scale"))
    broken(lambda d: d["layers"][0]["mixer"].update(heads=3))
    broken(lambda d: d["layers"][0]["mixer"]["rot"].update(dims=5))
    broken(lambda d: d["layers"][0]["mixer"]["mask"].pop("size"))          # blocks without a window
    broken(lambda d: d["layers"][0]["mlp"]["router"].update(top=9))
    broken(lambda d: d["layers"][1]["mixer"].update(vdim=8))               # mixing layers share their value size
    broken(lambda d: d.update(streams=9))
    broken(lambda d: d.pop("width"))


def test_the_model_as_data_names_every_tensor():
    """The spec built from a configuration declares the tensors by the names and shapes the design gives them."""
    from cppvllm_b200.weights.random_init import random_tensors
    t = random_tensors(rm.RX_A, 1)
    assert t["l0.norm1"].shape == () and t["final.norm"].shape == () and t["l0.hc1.mix"].shape == (3, 3) and t["l0.hc2.in"].shape == (3,)
    assert t["l0.mix.q"].shape == (64, 48) and t["l0.mix.k"].shape == (32, 48) and t["l0.mix.v"].shape == (48, 48)
    assert t["l0.mix.vmix"].shape == () and "l0.mix.sink" not in t and "l0.mix.g" not in t
    assert t["l1.mix.sink"].shape == (4,) and t["l1.mix.r1"].shape == (4,) and t["l1.mix.g"].shape == (4, 48) and "l1.hc2.in" not in t
    assert t["l2.mix.q"].shape == (3 * 14, 48) and t["l2.mix.dkv"].shape == (26, 48) and t["l2.mix.dkv.norm"].shape == (20,)
    assert t["l2.mix.uk"].shape == (24, 20) and t["l2.mix.uv"].shape == (30, 20) and t["l2.mix.g"].shape == (30, 48)
    assert t["l0.mlp.router"].shape == (5, 48) and t["l0.mlp.shared.gate"].shape == (16, 48) and "l2.mlp.shared.up" not in t
    d = random_tensors(rm.RX_D, 1)
    assert not any(".hc" in k for k in d) and "l0.mix.vmix" not in d
