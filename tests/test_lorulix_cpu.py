"""Lorulix without a GPU: the configuration reader and its refusals, the model as data (run list, shared caches, state rows,
tensor names), the table of distance buckets, the plain implementation's mechanisms one by one, and that the test models
are sharp enough for a fault of each mechanism to show."""
import copy
import math

import pytest
import torch

import lorulix_models as lm
import plain_lorulix as plain
from cppvllm_b200.config.lorulix_config import LorulixConfig
from cppvllm_b200.config.model_config import ConfigError
from cppvllm_b200.config.registry import resolve_architecture
from cppvllm_b200.parts.attention_bias import distance_buckets
from cppvllm_b200.parts.base import Runtime, Workspace
from cppvllm_b200.parts.model import CausalLM

F = torch.float64


def build(cfg):
    arch = resolve_architecture(cfg)
    spec = arch.build_spec(arch.parse_config(cfg))
    cpu = torch.device("cpu")
    return spec, CausalLM(spec, Runtime(cpu, torch.float32, Workspace(cpu, 0)))


def test_configuration_is_read_from_the_file_alone():
    c = LorulixConfig.from_dict(lm.LX_A)
    assert (c.vocab, c.width, c.max_positions, c.norm_eps, c.taps) == (97, 48, 160, 1e-5, 3)
    assert [l.type for l in c.layers] == ["attention", "delta", "attention", "delta"]
    assert [l.mlp.kind if l.mlp else None for l in c.layers] == ["dense", "moe", None, "dense"]
    m = c.layers[0].mixer
    assert (m.heads, m.kv_heads, m.dim, m.vdim, m.scale, m.bias_max, m.temp_coef, m.temp_every, m.kv_from) == (3, 1, 16, 24, 0.3, 20, 0.4, 5, None)
    assert c.layers[2].mixer.kv_from == 0
    d = c.layers[1].mixer
    assert (d.heads, d.kv_heads, d.dim, d.vdim, d.conv) == (4, 2, 12, 20, 2)
    f = c.layers[1].mlp
    assert (f.experts, f.top, f.ff, f.scale, f.shared_ff) == (5, 2, 24, 2.0, 16) and c.layers[0].mlp.limit == 0.7
    assert LorulixConfig.from_dict(lm.LX_B).layers[0].mlp.shared_ff == 0
    assert resolve_architecture(lm.LX_B).name == "Lorulix"
    for breaker in (lambda d: d.pop("vocab"), lambda d: d["layers"][0].update(type="conv"), lambda d: d["canon"].pop("taps"),
                    lambda d: d["layers"][1]["mlp"].update(kind="glu"), lambda d: d["layers"][0]["mixer"].update(kv_heads=2),
                    lambda d: d["layers"][2]["mixer"].update(kv_from=1),        # a recurrent layer has no keys to lend
                    lambda d: d["layers"][2]["mixer"].update(kv_from=2),        # nor has the layer itself
                    lambda d: d["layers"][2]["mixer"].update(vdim=8),           # other sizes than the layer it reads
                    lambda d: d["layers"][1]["mlp"]["router"].update(top=6), lambda d: d["norm"].pop("eps"),
                    lambda d: d["layers"][0]["mlp"].pop("limit"), lambda d: d["layers"][1]["mixer"].pop("conv"),
                    lambda d: d["layers"][0]["mixer"].pop("scale")):
        bad = copy.deepcopy(lm.LX_A)
        breaker(bad)
        with pytest.raises(ConfigError):
            LorulixConfig.from_dict(bad)


def test_run_list_caches_states_and_tensor_names():
    spec, model = build(lm.LX_C)
    assert spec.residual_dtype == "float32"
    order = [(e.layer, e.cache, e.writes_cache) for e in model.run_order]
    assert [o for o in order if o[0] != 2] == [(0, 0, True), (1, 0, False), (3, 3, True), (4, 3, False)]      # readers share the writer's unit
    units = model.cache_units()
    assert set(units) == {0, 3} and units[0].entry_shape == (2, 128) and units[3].entry_shape == (2, 96)      # a key and its value behind it
    states = [s.shape[0] for s in model.state_specs()]
    D, K = 96, 4
    conv_rows = (3 - 1) * (2 * 2 * 64 + 2 * 64)
    assert states == [2 * (K - 1) * D, 2 * (K - 1) * D, 2 * 64 * 64 + conv_rows + 2 * (K - 1) * D, 2 * (K - 1) * D, 2 * (K - 1) * D]
    names = set(model.weight_specs())
    assert {"embed", "pos", "l0.norm1", "l0.norm1b", "l0.norm2", "l0.norm2b", "l0.canon1", "l0.canon2", "l0.rg1", "l0.rg1.b", "l0.rg2.b",
            "l0.mix.q", "l0.mix.k", "l0.mix.v", "l0.mix.q.norm", "l0.mix.k.norm", "l0.mix.rel", "l0.mix.o", "l0.mlp.router",
            "l0.mlp.e3.up", "l0.mlp.e0.down", "l0.mlp.shared.up", "l0.mlp.shared.down", "l0.mlp.shared.sg", "l1.mlp.gate", "l1.mlp.up",
            "l1.mlp.down", "l2.mix.q.conv", "l2.mix.k.conv", "l2.mix.v.conv", "l2.mix.b", "l2.mix.a", "l2.mix.A_log", "l2.mix.dt_bias",
            "l2.mix.norm", "l2.mix.g", "l2.mix.o", "final.norm", "head"} <= names
    # a layer that reads another's cache has no key or value tensors; a layer without a feed-forward has nothing of one
    assert not any(n.startswith(("l1.mix.k", "l1.mix.v", "l4.mix.k", "l4.mix.v", "l4.mlp.shared")) for n in names)
    specs = model.weight_specs()
    assert specs["l0.mix.rel"].shape == (32, 6) and specs["l3.mix.q"].shape == (4 * 32, 96) and specs["l3.mix.o"].shape == (96, 4 * 64)
    assert specs["l2.mix.norm"].shape == (64,) and specs["l0.mlp.shared.sg"].shape == (1, 96) and specs["l0.canon1"].shape == (96, 4)
    _, model_a = build(lm.LX_A)
    assert not any(n.startswith("l2.mlp") or n.startswith("l2.norm2") or n.startswith("l2.canon2") or n.startswith("l2.rg2")
                   for n in model_a.weight_specs())
    _, model_b = build(lm.LX_B)                          # one tap: no history in front of the sublayers
    assert [s.shape[0] for s in model_b.state_specs()] == [3 * 40 * 33, 0, 0]


def test_distance_buckets():
    for rows, far in ((32, 384), (8, 20), (6, 9), (4, 3), (12, 50), (16, 300), (64, 4096)):
        table = distance_buckets(rows, far)
        assert table == [plain.distance_bucket(n, rows, far) for n in range(far + 1)]
        half = rows // 2
        assert table[:half] == list(range(half)) and table[half] == half and table[-1] == rows - 1
        assert all(b >= a for a, b in zip(table, table[1:]))
        assert all(plain.distance_bucket(n, rows, far) == rows - 1 for n in (far, far + 1, 10 * far))
    # a bucket's first distance by the closed form: the smallest n with half * (far / half)^((b - half) / (rows - half)) <= n
    table = distance_buckets(32, 384)
    for b in range(17, 32):
        edge = 16 * (384 / 16) ** ((b - 16) / 16)
        first = table.index(b) if b in table else None
        assert first is None or first == math.ceil(edge - 1e-9)
    with pytest.raises(ValueError):
        distance_buckets(8, 4)


def test_plain_mechanisms_one_by_one():
    torch.manual_seed(0)
    x = torch.randn(5, 8, dtype=F)
    w = torch.randn(8, dtype=F) * 0.1
    n = plain.norm_around_zero(x, w, 1e-3)
    assert torch.allclose(n / (1 + w) * torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-3), x)
    # the convolution: the last column is the current token's, zeros stand before the start
    taps = torch.tensor([[1.0, 10.0, 100.0]], dtype=F)
    assert plain.causal_conv(torch.tensor([[1.0], [2.0], [3.0], [4.0]], dtype=F), taps).flatten().tolist() == [100.0, 210.0, 321.0, 432.0]
    assert plain.query_temperature(7, 0.5, 3).tolist() == [1 + 0.5 * math.log(k + 1) for k in (0, 0, 1, 1, 1, 2, 2)]
    # the delta rule with beta = 1, no decay and orthonormal keys stores every value under its key and reads it back
    k = torch.eye(4, dtype=F).reshape(4, 1, 4)
    v = torch.randn(4, 1, 3, dtype=F)
    o = plain.delta_rule(k, k, v, torch.ones(4, 1, dtype=F), torch.ones(4, 1, dtype=F))
    assert torch.allclose(o, v)
    # writing under the same key again replaces the value (u = v - S^T k); a decay of one half halves what was stored before
    k2 = torch.tensor([[[1.0, 0.0]], [[1.0, 0.0]]], dtype=F)
    v2 = torch.tensor([[[3.0]], [[5.0]]], dtype=F)
    assert plain.delta_rule(k2, k2, v2, torch.ones(2, 1, dtype=F), torch.ones(2, 1, dtype=F)).flatten().tolist() == [3.0, 5.0]
    half = plain.delta_rule(k2, k2, v2, torch.full((2, 1), 0.5, dtype=F), torch.full((2, 1), 0.5, dtype=F))
    assert half.flatten().tolist() == [1.5, 0.75 + 0.5 * (5.0 - 0.75)]
    # the dense feed-forward's clamps
    ws = {"f.gate": torch.eye(2, dtype=F), "f.up": torch.eye(2, dtype=F), "f.down": torch.eye(2, dtype=F)}
    y = plain.clamped_glu(torch.tensor([[5.0, -5.0]], dtype=F), ws, "f.", {"limit": 2.0}, plain.identity)
    g = torch.tensor([2.0, -5.0], dtype=F)
    assert torch.allclose(y[0], g * plain.logistic(1.702 * g) * (torch.tensor([2.0, -2.0], dtype=F) + 1))
    # routed experts: the chosen experts' shares of the softmax over all, times the scale, not renormalised
    E, D = 3, 2
    ws = {"f.router": torch.tensor([[2.0, 0.0], [1.0, 0.0], [0.0, 0.0]], dtype=F)}
    for e in range(E):
        ws[f"f.e{e}.up"] = torch.eye(D, dtype=F) * (e + 1)
        ws[f"f.e{e}.down"] = torch.eye(D, dtype=F)
    h = torch.tensor([[1.0, -1.0]], dtype=F)
    s = torch.softmax(torch.tensor([2.0, 1.0, 0.0], dtype=F), 0)
    y = plain.routed_experts(h, ws, "f.", {"router": {"experts": 3, "top": 2, "scale": 4.0}}, plain.identity)
    assert torch.allclose(y[0], 4.0 * (s[0] * torch.tensor([1.0, 0.0], dtype=F) + s[1] * torch.tensor([4.0, 0.0], dtype=F)))


@pytest.mark.parametrize("name", ["lx_a", "lx_c"])
def test_the_test_models_show_a_fault_of_every_mechanism(tmp_path, name):
    """With the sharpened weights the logits move by a fiftieth of their size or more when a distance falls into the
    neighbouring bucket, the temperature's step comes one token late, a convolution loses its oldest tap, the recurrent state
    forgets, a clamp or a router's scale is off: hundreds of times the float32 tolerance of the engine tests."""
    cfg = lm.config(name)
    d = lm.write_model(str(tmp_path / name), cfg, lm.SETUPS[name][1])
    toks = lm.random_tokens(cfg["vocab"], 100, 1)
    w = plain.read_weights(d)
    ref = plain.forward(cfg, w, toks)
    scale = float(ref.abs().max())

    def moved(other_cfg=None, other_w=None):
        return float((plain.forward(other_cfg or cfg, other_w or w, toks) - ref).abs().max()) / scale

    def with_mixers(change, kind):
        other = copy.deepcopy(cfg)
        for layer in other["layers"]:
            if layer["type"] == kind:
                change(layer["mixer"])
        return other

    assert moved(with_mixers(lambda m: m.update(bias_max=m["bias_max"] + 7), "attention")) > 0.02
    assert moved(with_mixers(lambda m: m["q_temp"].update(every=m["q_temp"]["every"] + 1), "attention")) > 0.02
    assert moved(with_mixers(lambda m: m.update(scale=m["scale"] * 1.1), "attention")) > 0.02
    shifted = dict(w)
    for k in w:
        if k.endswith(".mix.rel"):
            shifted[k] = torch.roll(w[k], 1, dims=0)              # every distance one bucket off
    assert moved(other_w=shifted) > 0.02
    for pattern in (".canon1", ".canon2", ".v.conv"):
        lost = dict(w)
        for k in w:
            if k.endswith(pattern):
                lost[k] = w[k].clone()
                lost[k][:, 0] = 0.0                                # the oldest tap: a history that is one row short
        assert moved(other_w=lost) > 0.02, pattern
    forgot = dict(w)
    for k in w:
        if k.endswith(".A_log"):
            forgot[k] = w[k] + 3.0                                 # a state that decays within a few tokens
    assert moved(other_w=forgot) > 0.02
    other = copy.deepcopy(cfg)
    for layer in other["layers"]:
        f = layer["mlp"]
        if f and f["kind"] == "dense":
            f["limit"] *= 2
        elif f:
            f["router"]["scale"] *= 1.2
    assert moved(other) > 0.02
