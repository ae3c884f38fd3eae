"""Rumurax through the engine against the plain implementation (tests/plain_rumurax.py): whole prompts, the last tokens
one by one, portions down to two tokens, the first tokens alone, unequal requests in one batch, pools so small that pages
and slots are used again, long decoding past windows, chunks and pooled blocks, the streams after every layer, greedy
generation through the public entry point and the trace replay as a process.  Weights are sharpened
(tests/rumurax_models.py), so a wrong key, a mask that is one token off, a lost sink or unmixed values show."""
import numpy as np
import pytest
import torch

import rumurax_models as rm
from trace_util import TraceBuilder, needed_max_tokens, portions, rows_by_position, run_trace, run_trace_in_process, tail_one_by_one, whole

pytestmark = pytest.mark.gpu

TOL = {"float32": 3e-5, "bfloat16": 5e-2}        # of the largest logit; a fault of a mechanism moves logits by tenths of it
NAMES = ["rx_a", "rx_b", "rx_c", "rx_d", "rx_e"]


@pytest.fixture(scope="module")
def rx_dirs(tmp_path_factory):
    return rm.write_all(str(tmp_path_factory.mktemp("rumurax")))


def make_runner(d, name, dtype, pages=24, **kw):
    from cppvllm_b200.engine.runner import ModelRunner
    args = dict(dtype=torch.float32 if dtype == "float32" else torch.bfloat16, page_size=rm.page_size(name), num_pages=pages,
                max_step_tokens=256, max_seqs=8, max_model_len=256)
    args.update(kw)
    return ModelRunner(d, **args)


def check(rows, refs, dtype):
    """float32: every row within the tolerance.  bfloat16: the sharpened models amplify rounding (a peaked softmax moves its
    weight), so a twentieth of the rows may lie beyond the tolerance; a fault of a mechanism moves most rows and fails both."""
    errs = []
    for (rid, pos), row in rows.items():
        ref = refs[rid.split("#")[0]]
        scale = max(1.0, float(ref.abs().max()))
        errs.append((float(np.abs(row - ref[pos].numpy()).max()) / scale, rid, pos))
    worst, rid, pos = max(errs)
    over = sum(1 for e in errs if e[0] > TOL[dtype])
    allowed = 0 if dtype == "float32" else max(1, len(errs) // 20)
    assert over <= allowed, f"{over} of {len(errs)} rows beyond {TOL[dtype]:.1e}; worst {worst:.3e} at request {rid} position {pos}"
    print(f"worst error {worst:.3e} of scale, {over} rows beyond the tolerance ({dtype})")
    return worst


def refs_of(d, toks):
    return {k: rm.reference(d, v).float() for k, v in toks.items()}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", NAMES)
def test_whole_tail_and_portions_match_the_plain_implementation(rx_dirs, name, dtype):
    d = rx_dirs[name]
    toks = {"w": rm.clear_tokens(d, 110, 1), "t": rm.clear_tokens(d, 101, 2), "p": rm.clear_tokens(d, 110, 1),
            "s": rm.clear_tokens(d, 1, 3), "q": rm.clear_tokens(d, 3, 4)}
    tb = TraceBuilder()
    whole(tb, "w", toks["w"])
    tail_one_by_one(tb, "t", toks["t"], tail=85)       # decoded tokens pass windows, chunk edges, new blocks and page borders
    portions(tb, "p", toks["p"])
    whole(tb, "s", toks["s"])                          # the first token alone
    tb.add([("q", toks["q"][:1], [0])])                # the first tokens one by one
    tb.add([("q", toks["q"][1:2], [0])])
    tb.add([("q", toks["q"][2:3], [0])], end=["q"])
    runner = make_runner(d, name, dtype, pages=(128 // rm.page_size(name)))
    rows = rows_by_position(tb.steps, run_trace_in_process(runner, tb.steps))
    assert len(rows) == 110 + 101 + 110 + 1 + 3
    check(rows, refs_of(d, toks), dtype)
    apart = sum(1 for pos in range(110)               # cut differently, equal beyond rounding
                if np.abs(rows[("w", pos)] - rows[("p", pos)]).max() > TOL[dtype] * max(1.0, np.abs(rows[("w", pos)]).max()))
    assert apart <= (0 if dtype == "float32" else 5)
    runner.cache.check_invariants()
    assert all(runner.cache.num_free_pages(g) == 128 // rm.page_size(name) for g in range(len(runner.group_specs)))


@pytest.mark.parametrize("seed,dtype", [(s, "float32") for s in range(6)] + [(s, "bfloat16") for s in range(20, 24)])
def test_configurations_drawn_at_random(tmp_path, seed, dtype):
    """Layers of the three kinds in any order and size (tests/rumurax_models.py: random_config): a whole prompt, a tail decoded
    token by token, portions down to two tokens and three unequal requests in one batch.  In float32 nothing but the order of
    sums may differ; in bfloat16 the sizes are the ones the tensor-core kernels take."""
    import random
    cfg = rm.random_config(seed, tensor_core=dtype == "bfloat16")
    d = rm.write_model(str(tmp_path / "m"), cfg, seed)
    toks = {"w": rm.clear_tokens(d, 150, 1), "t": rm.clear_tokens(d, 140, 2), "p": rm.clear_tokens(d, 150, 1),
            "x": rm.clear_tokens(d, 70, 5), "y": rm.clear_tokens(d, 33, 6), "z": rm.clear_tokens(d, 2, 7)}
    tb = TraceBuilder()
    whole(tb, "w", toks["w"])
    tail_one_by_one(tb, "t", toks["t"], tail=40)
    portions(tb, "p", toks["p"])
    tb.add([("x", toks["x"][:37], range(37)), ("y", toks["y"][:32], range(32)), ("z", toks["z"][:1], [0])])
    tb.add([("x", toks["x"][37:39], range(2)), ("y", toks["y"][32:], [0]), ("z", toks["z"][1:], [0])], end=["y", "z"])
    tb.add([("x", toks["x"][39:], range(31))], end=["x"])
    from cppvllm_b200.engine.runner import ModelRunner
    page = random.Random(seed).choice([16, 32, 64])
    runner = ModelRunner(d, dtype=torch.float32 if dtype == "float32" else torch.bfloat16, page_size=page, num_pages=256 // page,
                         max_step_tokens=256, max_seqs=4, max_model_len=256, num_state_slots=3)
    rows = rows_by_position(tb.steps, run_trace_in_process(runner, tb.steps))
    assert len(rows) == 150 + 140 + 150 + 70 + 33 + 2
    check(rows, refs_of(d, toks), dtype)


@pytest.mark.parametrize("dtype,eager", [("float32", False), ("bfloat16", False), ("float32", True)])
@pytest.mark.parametrize("name", ["rx_a", "rx_b", "rx_c"])
def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again(rx_dirs, name, dtype, eager):
    """Up to four live requests: portions of some beside single tokens of others, in a pool of 384 tokens (the requests
    need 704) and four slots, so that every page serves several requests; every logit is compared with the request run
    alone in the plain implementation."""
    d = rx_dirs[name]
    lens = {"a": 97, "b": 64, "c": 33, "d": 120, "e": 2, "f": 71, "g": 65}
    toks = {k: rm.clear_tokens(d, n, 30 + n) for k, n in lens.items()}
    cuts = {"a": [2, 31, 1, 1, 1, 29, 32], "b": [64], "c": [16, 15, 1, 1], "d": [3, 2, 59, 1, 1, 1, 53], "e": [1, 1],
            "f": [40, 2, 29], "g": [63, 1, 1]}
    waiting = ["a", "b", "c", "d", "e", "f", "g"]
    live, at, part = [], {k: 0 for k in lens}, {k: 0 for k in lens}
    tb = TraceBuilder()
    while waiting or live:
        while waiting and len(live) < 4 and sum((lens[k] + 63) // 64 * 64 for k in live + [waiting[0]]) <= 384:
            live.append(waiting.pop(0))
        entries, end = [], []
        for k in list(live):
            n = cuts[k][part[k]]
            entries.append((k, toks[k][at[k]:at[k] + n], range(n)))
            at[k] += n
            part[k] += 1
            if at[k] == lens[k]:
                end.append(k)
                live.remove(k)
        tb.add(entries, end=end)
    assert needed_max_tokens(tb.steps) <= 384 and max(len(st["entries"]) for st in tb.steps) == 4
    runner = make_runner(d, name, dtype, pages=384 // rm.page_size(name), num_state_slots=4, enforce_eager=eager)
    rows = rows_by_position(tb.steps, run_trace_in_process(runner, tb.steps))
    assert len(rows) == sum(lens.values())
    check(rows, refs_of(d, toks), dtype)
    runner.cache.check_invariants()
    # the same trace once more on the same runner: every page has had another owner by now
    again = rows_by_position(tb.steps, run_trace_in_process(runner, tb.steps))
    for key, row in rows.items():                      # the same steps, the same kernels: the same bits
        assert np.array_equal(again[key], row)


@pytest.mark.parametrize("name", ["rx_a", "rx_c", "rx_d"])
@pytest.mark.parametrize("use_ref_kernels", [False, True])
def test_streams_after_every_layer(rx_dirs, name, use_ref_kernels):
    """The sum of the streams after each layer equals the plain implementation's, with the fused kernels and the simple ones."""
    d = rx_dirs[name]
    toks = rm.clear_tokens(d, 37, 5)
    runner = make_runner(d, name, "float32", enforce_eager=True, use_ref_kernels=use_ref_kernels)
    seen = []
    for b in runner.model.blocks:
        def wrapped(h, pending, ctx, cache, state, f=b.forward, S=b.streams):
            h2, p2 = f(h, pending, ctx, cache, state)
            X = h2.double().view(ctx.num_tokens, S, -1)
            if p2 is not None:                         # the last write of the layer is still to come: apply it here
                y = sum(part.double() for part in p2.y) if isinstance(p2.y, (tuple, list)) else p2.y.double()
                X = torch.einsum("sr,tsd->trd", p2.mix.double().view(S, S), X) + p2.out.double()[None, :, None] * y[:, None, :]
            seen.append(X.sum(1).cpu())
            return h2, p2
        b.forward = wrapped
    tb = TraceBuilder()
    whole(tb, "x", toks)
    run_trace_in_process(runner, tb.steps)
    runs = []
    rm.reference(d, toks, layer_outputs=runs)
    assert len(seen) == len(runs) == len(rm.config(name)["layers"])
    for got, ref in zip(seen, runs):
        assert float((got - ref).abs().max()) <= 3e-5 * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["rx_a", "rx_c"])
def test_long_decoding(rx_dirs, name, dtype):
    """A short prompt and 190 tokens decoded one by one through the captured graphs: windows pass over decoded tokens, chunks
    begin and end, pooled blocks are closed and become visible, pages fill."""
    d, ps = rx_dirs[name], rm.page_size(name)
    toks = rm.clear_tokens(d, 200, 9)
    tb = TraceBuilder()
    tb.add([("z", toks[:10], range(10))])
    for i in range(10, 200):
        tb.add([("z", toks[i:i + 1], [0])], end=["z"] if i == 199 else [])
    runner = make_runner(d, name, dtype, pages=(200 + ps - 1) // ps + 1)
    rows = rows_by_position(tb.steps, run_trace_in_process(runner, tb.steps))
    check(rows, {"z": rm.reference(d, toks).float()}, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(rx_dirs, dtype):
    from cppvllm_b200 import LLM, SamplingParams
    d = rx_dirs["rx_b"]
    prompts = [rm.clear_tokens(d, n, 70 + n) for n in (1, 6, 40, 75)]
    llm = LLM(d, dtype=dtype, block_size=32, num_kv_blocks=12, max_num_batched_tokens=48, max_num_seqs=4, max_chunk_tokens=20,
              max_model_len=200)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o.prompt_ids == p and len(o.token_ids) == 10
        ref = rm.reference(d, (p + o.token_ids)[:-1])
        for i, tok in enumerate(o.token_ids):
            row = ref[len(p) - 1 + i]
            slack = (1e-4 if dtype == "float32" else 0.05) * max(1.0, float(row.abs().max()))
            assert row[tok] >= row.max() - slack
    llm.runner.check_errors()
    llm.runner.cache.check_invariants()


def test_trace_replay_command_line(rx_dirs, tmp_path):
    d = rx_dirs["rx_d"]
    toks = rm.clear_tokens(d, 70, 8)
    tb = TraceBuilder()
    portions(tb, "r", toks, sizes=(2, 5, 2, 31))
    out = run_trace(d, "float32", tb.steps, 128, str(tmp_path / "o"), ["--block-size", "64"])
    check(rows_by_position(tb.steps, out), {"r": rm.reference(d, toks).float()}, "float32")


def test_the_example_command_line(rx_dirs):
    """`example <model_dir>`: the registry picks the design by config.json, the pool is sized from what the device has left
    after the weights, and every generated token is the plain implementation's best one."""
    import ast
    import os
    import subprocess
    import sys
    d = rx_dirs["rx_a"]
    prompt = rm.clear_tokens(d, 9, 77)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "example"), d, "--dtype", "float32", "--prompt", ",".join(map(str, prompt)),
                        "--temperature", "0", "--max-tokens", "5", "--ignore-eos", "--max-num-seqs", "4", "--max-model-len", "64",
                        "--max-num-batched-tokens", "64", "--block-size", "16"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("Completion:")][0]
    got = ast.literal_eval(line[len("Completion:"):].strip())
    assert len(got) == 5
    ref = rm.reference(d, (prompt + got)[:-1])
    for i, tok in enumerate(got):
        row = ref[len(prompt) - 1 + i]
        assert row[tok] >= row.max() - 1e-4 * max(1.0, float(row.abs().max()))
