"""The Rogosun design in the engine against the plain implementation (tests/plain_rogosun.py).

Every test makes its own small configuration and weights (tests/rogosun_util.py).  The CPU tests put the
plain PyTorch stand-ins of the kernels (tests/kernel_refs.py) under the engine, so they test what is host
logic: configuration, registry, tensor names and free ranks, caches and states per layer and branch,
batching.  The GPU tests run the same traces on the kernels, in float32 and bfloat16: whole prompts,
prompts followed by token-by-token decoding (from CUDA graphs), portions down to one and two tokens, mixed
batches of unequal requests with pages and state slots that are used again, long prompts whose attention
is peaky (a far key, a key at a page's edge or a stale page would show) and whose recurrences forget
slowly, the first tokens of a sequence where the sink carries most of the softmax, and greedy generation
through ``Engine.generate``.
"""
import copy
import io
import json
import os
import subprocess
import sys
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_rogosun as P
import replay_util as ru
import rogosun_util as U

DEV = "cuda:0"
# float32: the engine against 64-bit arithmetic, both from the same bfloat16-representable weights, relative to a
# row's largest logit.  bfloat16: products and activations are rounded to 8 bits of mantissa between kernels, and
# the tests' peaky attention (so that a lost key shows) multiplies the rounding of q and k by the scores' spread.
# The float32 runs go through the same kernels and are the sharp test of every index and edge.
TOL = {torch.float32: dict(rtol=5e-5, atol=1e-6), torch.bfloat16: dict(rtol=8e-2, atol=4e-3)}


def make_runner(tmp_path, cfg, weights, dtype, device, **kw):
    from zinfer_b200.engine import ModelRunner

    d = U.write_model(str(tmp_path / f"m{abs(hash(json.dumps(cfg, sort_keys=True))) % 10**8}"), cfg, weights)
    kw.setdefault("page_size", 8)
    kw.setdefault("max_requests", 4)
    return ModelRunner.from_model_dir(d, dtype=dtype, device=device, **kw)


# ============================================================================ CPU
def test_config_is_read_and_registered():
    from zinfer_b200.config import ConfigError, RogosunConfig, family_for, rogosun_model_spec
    from zinfer_b200.engine.model import declared_tensors

    raw = U.CONFIGS["mix"]
    fam = family_for(raw)
    assert fam.name == "Rogosun" and fam.config_class is RogosunConfig
    cfg = RogosunConfig.from_dict(raw)
    assert RogosunConfig.from_dict(cfg.to_dict()) == cfg                      # survives a round trip
    for name, other in {**U.CONFIGS, **U.MECHANISMS}.items():
        got = declared_tensors(rogosun_model_spec(RogosunConfig.from_dict(other)))
        want = U.tensor_shapes(other, rank=5, gate_rank=9)
        assert set(got) == set(want), name
        # every size but the low-rank pairs' ranks is fixed by the configuration; the ranks are the file's
        assert all(got[k].fits(want[k]) for k in got), name
        free = {k for k, v in got.items() if -1 in v.shape}
        assert free == {k for k in want if k.endswith((".a1", ".a2", ".g1", ".g2"))}, name
    for path, value, match in ((("layers", 0, "type"), "convolution", "unknown mixer"),
                               (("layers", 1, "mixer", "left", "rot", "dims"), 18, "rot.dims"),
                               (("layers", 1, "mixer", "right", "kv_heads"), 3, "kv heads"),
                               (("layers", 1, "mlp", "router", "groups", "keep"), 4, "groups"),
                               (("layers", 1, "mlp", "router", "top"), 5, "more experts"),
                               (("layers", 0, "mlp", "kind"), "sparse", "feed-forward")):
        bad = copy.deepcopy(raw)
        node = bad
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        with pytest.raises(ConfigError, match=match):
            RogosunConfig.from_dict(bad)
    bad = copy.deepcopy(raw)
    del bad["layers"][0]["mixer"]["tau"]
    with pytest.raises(ConfigError, match="tau"):
        RogosunConfig.from_dict(bad)


def test_weights_with_ranks_of_their_own_load_and_wrong_shapes_do_not(tmp_path):
    from zinfer_b200.config import load_config
    from zinfer_b200.engine.model import DecoderModel
    from zinfer_b200.weights import load_tensors
    from zinfer_b200.weights.loader import WeightsError

    cfg = U.CONFIGS["alt"]
    w = U.make_weights(cfg, seed=2, rank=3, gate_rank=7)
    d = U.write_model(str(tmp_path / "m"), cfg, w)
    fam, typed = load_config(d)
    model = DecoderModel(fam.model_spec(typed), torch.float32, "cpu")
    model.bind(load_tensors(d, model.tensor_specs(), torch.float32, "cpu"))
    assert model.blocks[1].mixer.rank == 3 and model.blocks[0].mixer.right.gate_rank == 7
    w["l1.mix.q"] = w["l1.mix.q"][:-1]                              # a fixed size that is wrong is still refused
    d = U.write_model(str(tmp_path / "bad"), cfg, w)
    with pytest.raises(WeightsError, match="l1.mix.q"):
        load_tensors(d, model.tensor_specs(), torch.float32, "cpu")
    w = U.make_weights(cfg, seed=2)
    w["l1.mix.a2"] = torch.zeros(5 * 40, 9, dtype=torch.bfloat16)   # a pair that does not share its rank
    d = U.write_model(str(tmp_path / "pair"), cfg, w)
    with pytest.raises(ValueError, match="rank"):
        model.bind(load_tensors(d, model.tensor_specs(), torch.float32, "cpu"))


def test_caches_and_states_per_layer_and_branch():
    from zinfer_b200.config import RogosunConfig, rogosun_model_spec
    from zinfer_b200.engine import DecoderModel

    model = DecoderModel(rogosun_model_spec(RogosunConfig.from_dict(U.CONFIGS["mix"])), torch.float32, "cpu")
    kv, state = model.cache_needs()
    # layers: gla, parallel, gla, parallel: two key/value caches (the attentions), four states
    assert sorted(kv) == ["run1.left", "run3.left"] and sorted(state) == ["run0", "run1.right", "run2", "run3.right"]
    assert all(n.num_kv_heads == 2 and n.head_dim == 16 and n.values and n.window is None for n in kv.values())
    assert state["run0"].shape == (3, 24, 16)
    # S of four heads [24, 16], then three carried inputs of 2*2*24 + 4*16 convolved channels
    assert state["run1.right"].shape == (4 * 24 * 16 + 3 * (96 + 64),)
    assert all(n.dtype == torch.float32 for n in state.values())


def test_command_line_inspects_the_model(tmp_path):
    from zinfer_b200 import cli

    d = U.write_model(str(tmp_path / "m"), U.CONFIGS["mix"], U.make_weights(U.CONFIGS["mix"], seed=1))
    out = io.StringIO()
    assert cli.run(["inspect-config", d], out) == 0
    text = out.getvalue()
    assert "architecture: Rogosun" in text and "layer 0: gla" in text and "layer 1: parallel" in text
    assert "moe experts=6 top=2 groups=3 keep=2 ff=40 shared ff=24" in text
    out = io.StringIO()
    assert cli.run(["inspect-weights", d], out) == 0 and "tensor_count:" in out.getvalue()


@pytest.mark.parametrize("name", ["mix", "alt", "odd"])
def test_engine_host_logic_on_stand_ins(cpu_kernels, tmp_path, name):
    cfg = U.CONFIGS[name]
    weights = U.make_weights(cfg, seed=3)
    runner = make_runner(tmp_path, cfg, weights, torch.float32, "cpu", max_tokens=192, max_requests=3, cuda_graphs=False)
    reqs = U.clear_requests(cfg, weights, [23, 1, 40, 9, 17], seed=4, margin=1e-3)
    plain = U.plain_logits(cfg, weights, reqs)
    for mode, trace in (("whole", ru.trace_whole(reqs)), ("tail", ru.trace_tail_decode(reqs, 6)),
                        ("portions", ru.trace_portions(reqs, 2)), ("mixed", ru.trace_mixed(reqs, 5, max_live=3, tail=4))):
        got = ru.run_in_process(runner, trace)
        ru.assert_close(got, plain, what=f"{name}/{mode}", argmax_frac=0.0, rtol=2e-4, atol=1e-5)
        assert not runner.manager.requests
    assert runner.manager.slots.reused > 0        # three slots served five requests, four times over


def test_plain_model_pieces():
    """The plain implementation against numbers worked out by hand."""
    F = torch.float64
    # convolution: kernel [1, 2, 3] on inputs 1, 10, 100 after a carried 5, 7: 5+14+3=22 -> silu, ...
    y, tail = P.short_conv(torch.tensor([[1.0], [10.0], [100.0]], dtype=F), torch.tensor([[1.0, 2.0, 3.0]], dtype=F),
                           torch.tensor([[5.0], [7.0]], dtype=F))
    want = torch.tensor([22.0, 7 + 2 + 30.0, 1 + 20 + 300.0], dtype=F)
    assert torch.allclose(y.reshape(-1), want * torch.sigmoid(want)) and tail.reshape(-1).tolist() == [10.0, 100.0]
    # a rotation at position 2 with base 1 and factor 4: angle 0.5 for the one pair; the third value passes
    r = P.rotate(torch.tensor([[[1.0, 0.0, 7.0]]], dtype=F), torch.tensor([2]), 2, 1.0, 4.0)
    assert torch.allclose(r, torch.tensor([[[np.cos(0.5), np.sin(0.5), 7.0]]], dtype=F))
    # routing: groups (0.9, 0.1), (0.5, 0.45), (0.6, 0.2) score 1.0, 0.95, 0.8; two groups kept; the best three of
    # their four experts are 0, 2, 3: expert 4 (0.6) is larger than 3 (0.45) but its group is out
    chosen = P.route(torch.tensor([0.9, 0.1, 0.5, 0.45, 0.6, 0.2], dtype=F), 3, 3, 2)
    assert sorted(chosen.tolist()) == [0, 2, 3]
    # one step of the delta rule from S = 0 with k a unit vector: S = k (beta v)^T, o = (k.q) beta v
    one = lambda *v: torch.tensor(v, dtype=F)
    S = torch.zeros(2, 2, dtype=F)
    k, q, v, beta, g = one(1.0, 0.0), one(0.5, 0.5), one(2.0, 4.0), 0.5, one(0.9, 0.8)
    Sh = g.unsqueeze(-1) * S
    u = beta * (v - Sh.T @ k)
    Sh = Sh + k.unsqueeze(-1) * u.unsqueeze(0)
    assert torch.allclose(Sh.T @ q, 0.5 * beta * v)
    # the sink: a single key of score 0 gets weight 1/2
    assert P.SINK == 1.0


# ============================================================================ GPU
gpu = pytest.mark.gpu


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", list(U.MECHANISMS))
def test_each_mechanism_alone(tmp_path, name, dtype):
    cfg = U.MECHANISMS[name]
    weights = U.make_weights(cfg, seed=11)
    reqs = U.clear_requests(cfg, weights, [37, 1, 20], seed=12, margin=0.05)
    plain = U.plain_logits(cfg, weights, reqs)
    runner = make_runner(tmp_path, cfg, weights, dtype, DEV, max_tokens=128, max_requests=2)
    for mode, trace in (("whole", ru.trace_whole(reqs)), ("tail", ru.trace_tail_decode(reqs, 12)),
                        ("portions", ru.trace_portions(reqs, 7, sizes=(2, 1, 5, 2, 3, 9, 2)))):
        got = ru.run_in_process(runner, trace)
        ru.assert_close(got, plain, what=f"{name}/{mode}", argmax_frac=0.0, **TOL[dtype])
    runner.manager.check()


@pytest.fixture(scope="module")
def models():
    """Per configuration: weights, requests with clear choices of experts, the plain model's logits."""
    out = {}
    for name, cfg in U.CONFIGS.items():
        weights = U.make_weights(cfg, seed=21 + len(name))
        reqs = U.clear_requests(cfg, weights, [45, 3, 70, 18, 1, 33], seed=5, margin=0.04)
        out[name] = (cfg, weights, reqs, U.plain_logits(cfg, weights, reqs))
    return out


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", list(U.CONFIGS))
def test_whole_decode_portions_mixed(tmp_path, models, name, dtype):
    cfg, weights, reqs, plain = models[name]
    # pool: the three longest requests rounded up to pages, so pages and the three slots are used again
    runner = make_runner(tmp_path, cfg, weights, dtype, DEV, max_tokens=176, max_requests=3)
    for mode, trace in (("whole", ru.trace_whole(reqs)), ("tail", ru.trace_tail_decode(reqs, 24)),
                        ("portions", ru.trace_portions(reqs, 9)), ("mixed", ru.trace_mixed(reqs, 13, max_live=3, tail=10))):
        got = ru.run_in_process(runner, trace)
        ru.assert_close(got, plain, what=f"{name}/{mode}", argmax_frac=0.0, **TOL[dtype])
        assert not runner.manager.requests
    assert runner.graphs is not None and runner.graphs.replays > 0         # single tokens came from CUDA graphs
    assert runner.manager.slots.reused > 0 and sum(g.pool.reused for g in runner.manager.groups) > 0
    runner.manager.check()


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_batch_against_each_alone(tmp_path, models, dtype):
    """Unequal requests in one batch give the rows they give alone: in float32 to the last bits (every kernel visits
    a request's data in an order that depends on the request alone)."""
    from zinfer_b200.engine import StepEntry

    cfg, weights, reqs, _ = models["mix"]
    runner = make_runner(tmp_path, cfg, weights, dtype, DEV, max_tokens=256, max_requests=4)
    ids = ["r0", "r2", "r3", "r4"]
    alone = {}
    for rid in ids:
        alone[rid] = runner.step([StepEntry(rid, reqs[rid], list(range(len(reqs[rid]))))]).clone()
        runner.end_request(rid)
    # together: the first request has half of its tokens in the cache already, the others come whole
    half = len(reqs["r0"]) // 2
    runner.step([StepEntry("r0", reqs["r0"][:half], [])])
    entries = [StepEntry("r0", reqs["r0"][half:], list(range(len(reqs["r0"]) - half)))] + \
        [StepEntry(rid, reqs[rid], list(range(len(reqs[rid])))) for rid in ids[1:]]
    got = runner.step(entries)
    row = 0
    for e in entries:
        want = alone[e.request_id][-len(e.want):]
        part = got[row:row + len(e.want)]
        row += len(e.want)
        tol = 2e-6 if dtype == torch.float32 else 2e-2
        assert (part - want).abs().max() <= tol * want.abs().max(), e.request_id


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_far_keys_page_edges_and_long_memory(tmp_path, dtype):
    """Prompts of several hundred tokens whose attention is peaky and whose two recurrences forget slowly: whole,
    against portions that end on, one before and one after page edges, against long token-by-token decoding, with
    pages poisoned when they are given back."""
    cfg = U.config(131, 64, [
        U.layer(U.par(U.att(4, 2, 16, 2.0, 12, base=2000.0, factor=2.0), U.delta(2, 1, 16, 24, 4), 0.8, 0.6), U.dense(64)),
        U.layer(U.gla(2, 32, 16, 16.0), None),
        U.layer(U.par(U.att(4, 2, 16, 2.0, 12, base=2000.0, factor=2.0), U.delta(2, 1, 16, 24, 4), 0.8, 0.6), None),
    ])
    weights = U.make_weights(cfg, seed=31, slow_decay=True)
    reqs = ru.make_requests(cfg["vocab"], [300, 203], seed=6)
    plain = U.plain_logits(cfg, weights, reqs)
    runner = make_runner(tmp_path, cfg, weights, dtype, DEV, page_size=16, max_tokens=320, max_requests=2,
                         poison_freed_pages=True)
    edges = (16, 15, 1, 17, 31, 2, 30, 33, 47, 64, 1, 1, 14)      # cumulative ends: 16, 31, 32, 49, 80, 82, 112, ...
    for mode, trace in (("whole", ru.trace_whole(reqs)), ("edges", ru.trace_portions(reqs, 0, sizes=edges)),
                        ("long decode", ru.trace_tail_decode(reqs, 90))):
        got = ru.run_in_process(runner, trace)
        ru.assert_close(got, plain, what=f"far/{mode}", argmax_frac=0.0, **TOL[dtype])
    runner.manager.check()


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dim,heads,kv_heads", [(64, 4, 2), (128, 3, 1)])
def test_attention_heads_the_tensor_core_kernels_take(tmp_path, dtype, dim, heads, kv_heads):
    """Heads of 64 and 128: in bfloat16 the attention with its sink runs on the tensor-core kernels (prompt portions and
    single tokens, the latter replayed from CUDA graphs with key splits), in float32 on the exact kernel; both against
    the plain model, over prompts of hundreds of tokens, portions across page edges and long decoding."""
    cfg = U.config(151, 96, [
        U.layer(U.par(U.att(heads, kv_heads, dim, 0.4, dim // 2, base=5000.0, factor=2.0), U.delta(2, 1, 16, 24, 4), 0.9, 0.4), U.dense(64)),
        U.layer(U.gla(2, 32, 16, 16.0), None),
        U.layer(U.par(U.att(heads, kv_heads, dim, 0.4, dim // 2, base=5000.0, factor=2.0), U.delta(2, 1, 16, 24, 4), 0.9, 0.4), None),
    ])
    weights = U.make_weights(cfg, seed=71)
    reqs = ru.make_requests(cfg["vocab"], [290, 150, 1], seed=10)
    plain = U.plain_logits(cfg, weights, reqs)
    runner = make_runner(tmp_path, cfg, weights, dtype, DEV, page_size=16, max_tokens=512, max_requests=3, poison_freed_pages=True)
    edges = (16, 15, 1, 17, 31, 2, 130, 33, 47, 64, 1, 1, 14)
    for mode, trace in (("whole", ru.trace_whole(reqs)), ("edges", ru.trace_portions(reqs, 0, sizes=edges)),
                        ("long decode", ru.trace_tail_decode(reqs, 70)), ("mixed", ru.trace_mixed(reqs, 3, max_live=3, tail=20))):
        got = ru.run_in_process(runner, trace)
        ru.assert_close(got, plain, what=f"heads of {dim}/{mode}", argmax_frac=0.0, **TOL[dtype])
    assert runner.graphs is not None and runner.graphs.replays > 60
    runner.manager.check()


@gpu
def test_long_memory_is_real_and_a_lost_state_would_show(tmp_path):
    """With slowly forgetting recurrences the first token still moves the logits 200 tokens later by a hundred times
    the float32 tolerance (so a state that is lost, reset or taken from another slot cannot pass), and the engine
    agrees with the plain model there."""
    cfg = U.config(67, 32, [U.layer(U.gla(2, 16, 8, 64.0), None), U.layer(
        U.par(U.att(1, 1, 8, 1.0, 8), U.delta(2, 2, 8, 8, 3), 1e-3, 1.0), None)])
    weights = U.make_weights(cfg, seed=51, slow_decay=True)
    toks = ru.make_requests(cfg["vocab"], [220], seed=8)["r0"]
    plain = U.plain_logits(cfg, weights, {"r0": toks})
    other = U.plain_logits(cfg, weights, {"r0": [(toks[0] + 1) % cfg["vocab"]] + toks[1:]})
    assert np.abs(plain["r0"][-1] - other["r0"][-1]).max() > 0.005 * np.abs(plain["r0"][-1]).max()
    for dtype in (torch.float32, torch.bfloat16):
        runner = make_runner(tmp_path, cfg, weights, dtype, DEV, page_size=16, max_tokens=256, max_requests=1)
        for trace in (ru.trace_whole({"r0": toks}), ru.trace_tail_decode({"r0": toks}, 40),
                      ru.trace_portions({"r0": toks}, 1, sizes=(2, 9, 64, 3, 2))):
            ru.assert_close(ru.run_in_process(runner, trace), plain, what="long memory", argmax_frac=0.0, **TOL[dtype])


@gpu
def test_a_single_far_key_decides(tmp_path):
    """One key 250 tokens back carries much of the last query's softmax: among all tokens that could stand at
    position 19, the test takes the one whose presence moves the last position's logits most in the plain model, and
    requires that move to be large; an engine that lost that key could not match."""
    cfg = U.config(67, 32, [U.layer(U.par(U.att(2, 1, 8, 1.5, 4), U.delta(1, 1, 8, 8, 2), 1.0, 1e-3), None)])
    weights = U.make_weights(cfg, seed=41)
    toks = ru.make_requests(cfg["vocab"], [270], seed=7)["r0"]
    without = toks[:19] + [toks[18]] + toks[20:]
    lost = U.plain_logits(cfg, weights, {"r0": without})
    move = {c: np.abs(U.plain_logits(cfg, weights, {"r0": toks[:19] + [c] + toks[20:]})["r0"][-1] - lost["r0"][-1]).max()
            for c in range(0, cfg["vocab"], 3)}
    toks[19] = max(move, key=move.get)
    plain = U.plain_logits(cfg, weights, {"r0": toks})
    assert np.abs(plain["r0"][-1] - lost["r0"][-1]).max() > 0.03 * np.abs(plain["r0"][-1]).max()     # the far key matters
    for dtype in (torch.float32, torch.bfloat16):
        runner = make_runner(tmp_path, cfg, weights, dtype, DEV, page_size=16, max_tokens=288, max_requests=1)
        for trace in (ru.trace_whole({"r0": toks}), ru.trace_tail_decode({"r0": toks}, 5)):
            ru.assert_close(ru.run_in_process(runner, trace), plain, what="one far key", argmax_frac=0.0, **TOL[dtype])


@gpu
def test_the_sink_carries_the_first_tokens(tmp_path):
    """At a sequence's first tokens the sink holds a large share of the softmax's denominator: the plain model
    without it gives other logits by far, and the engine matches the one with it, in prompts and in decoding."""
    cfg = U.MECHANISMS["attention_only_matters"]
    weights = U.make_weights(cfg, seed=61)
    reqs = ru.make_requests(cfg["vocab"], [12, 2, 1], seed=9)
    plain = U.plain_logits(cfg, weights, reqs)
    P.SINK = 0.0
    try:
        no_sink = U.plain_logits(cfg, weights, reqs)
    finally:
        P.SINK = 1.0
    assert all(np.abs(plain[r][:3] - no_sink[r][:3]).max() > 0.05 * np.abs(plain[r][:3]).max() for r in reqs)
    for dtype in (torch.float32, torch.bfloat16):
        runner = make_runner(tmp_path, cfg, weights, dtype, DEV, max_tokens=64, max_requests=2)
        for trace in (ru.trace_whole(reqs), ru.trace_tail_decode(reqs, 11), ru.trace_portions(reqs, 3, sizes=(2, 1, 2, 3))):
            ru.assert_close(ru.run_in_process(runner, trace), plain, what="sink", argmax_frac=0.0, **TOL[dtype])


@gpu
def test_greedy_generation_through_the_engine(tmp_path, models):
    from zinfer_b200.engine.api import Engine
    from zinfer_b200.sampling import SamplingParams

    cfg, weights, reqs, _ = models["alt"]
    d = U.write_model(str(tmp_path / "gen"), cfg, weights)
    prompts = [reqs["r1"], reqs["r3"], reqs["r0"][:30]]
    eng = Engine(d, dtype="float32", device=DEV, page_size=8, kv_cache_tokens=192, max_batched_tokens=16, max_requests=3)
    got = eng.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=6, ignore_eos=True))
    for p, r in zip(prompts, got):
        assert len(r.token_ids) == 6
        logits = P.PlainRogosun(cfg, weights).forward(p + r.token_ids).numpy()
        for i, t in enumerate(r.token_ids):      # the best token given the same history, or tied with it to rounding
            row = logits[len(p) - 1 + i]
            assert row[t] >= row.max() - 1e-4 * np.abs(row).max()


@gpu
def test_command_line_makes_a_random_model_and_generates(tmp_path):
    """bin/zinfer: a model folder of random weights made from a Rogosun config.json (the low-rank pairs get the ranks
    the parts propose), then tokens from it, greedy and sampled."""
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(U.CONFIGS["odd"]))
    d = str(tmp_path / "random")
    tool = os.path.join(ru.REPO, "bin", "zinfer")
    r = subprocess.run([sys.executable, tool, "random-model", d, str(cfg_path), "7"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    r = subprocess.run([sys.executable, tool, "generate-token-ids", d, "5,17,3,60,2", "6", "--dtype", "float32"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "tokens: [5, 17, 3, 60, 2, " in r.stdout, r.stderr[-2000:]
    r = subprocess.run([sys.executable, tool, "generate-token-ids", d, "5,17,3,60,2", "6", "--temperature", "0.8", "--top-k", "10",
                        "--seed", "3"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "tokens: [5, 17, 3, 60, 2, " in r.stdout, r.stderr[-2000:]


@gpu
def test_replay_program(tmp_path, models):
    """bin/trace_run as a user runs it: the model class comes from config.json, four state slots."""
    cfg, weights, reqs, plain = models["odd"]
    d = U.write_model(str(tmp_path / "tool"), cfg, weights)
    trace = ru.trace_mixed(reqs, 3, max_live=4, tail=8)
    info = {}
    got = ru.run_trace_tool(d, "float32", trace, str(tmp_path / "out"), ru.max_live_tokens(trace), cfg["vocab"], info=info)
    ru.assert_close(got, plain, what="trace_run", argmax_frac=0.0, **TOL[torch.float32])
    assert info["pages_reused"] and info["pages_reused"] > 0


def _step(q_lens, slots):
    cu = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
    return SimpleNamespace(cu_q=torch.tensor(cu, device=DEV), state_slots=torch.tensor(slots, dtype=torch.int32, device=DEV),
                           n_seqs=len(q_lens))


@gpu
@pytest.mark.parametrize("D,V,heads,key_heads", [(16, 8, 2, 2), (24, 40, 4, 2), (80, 33, 3, 1), (130, 64, 2, 2)])
@pytest.mark.parametrize("delta", [False, True])
def test_recurrence_kernel_against_the_loop(D, V, heads, key_heads, delta):
    """The recurrence as a kernel against the loop of tests/kernel_refs.py, from a state that is not zero, for
    requests of unequal length in slots out of order, and again cut in two steps (the same bits)."""
    import kernel_refs as ref
    from zinfer_b200 import ops

    gen = torch.Generator().manual_seed(D * 7 + V)
    q_lens, slots = [5, 1, 19], [2, 0, 3]
    T = sum(q_lens)
    r = lambda *s: torch.randn(s, generator=gen)
    q, k, v = r(T, key_heads * D), r(T, key_heads * D) / D ** 0.5, r(T, heads * V)
    decay = torch.sigmoid(2.0 + r(T, heads * D))
    beta = torch.sigmoid(r(T, heads)) if delta else None
    state0 = 0.3 * r(5, heads, D, V)
    want_state = state0.clone()
    cpu_step = SimpleNamespace(cu_q=torch.tensor(np.concatenate([[0], np.cumsum(q_lens)])), state_slots=torch.tensor(slots), n_seqs=3)
    want = ref.linear_recurrence(q, k, v, decay, beta, 0.5, want_state, heads, key_heads, D, V, cpu_step)
    dev = lambda t: None if t is None else t.to(DEV)
    state = state0.to(DEV)
    got = ops.linear_recurrence(dev(q), dev(k), dev(v), dev(decay), dev(beta), 0.5, state, heads, key_heads, D, V, _step(q_lens, slots))
    assert torch.allclose(got.cpu(), want, rtol=2e-5, atol=2e-5)
    assert torch.allclose(state.cpu(), want_state, rtol=2e-5, atol=2e-5)
    assert torch.equal(state[1].cpu(), state0[1]) and torch.equal(state[4].cpu(), state0[4])      # other slots untouched
    # the same requests cut in two steps give the same bits
    state2 = state0.to(DEV)
    first, second = [2, 1, 7], [3, 12]
    rows1 = [0, 1, 5, 6, 7, 8, 9, 10, 11, 12]
    rows2 = [2, 3, 4] + list(range(13, 25))
    pick = lambda t, rows: None if t is None else t[rows].to(DEV)
    o1 = ops.linear_recurrence(pick(q, rows1), pick(k, rows1), pick(v, rows1), pick(decay, rows1), pick(beta, rows1), 0.5, state2,
                               heads, key_heads, D, V, _step(first, slots))
    o2 = ops.linear_recurrence(pick(q, rows2), pick(k, rows2), pick(v, rows2), pick(decay, rows2), pick(beta, rows2), 0.5, state2,
                               heads, key_heads, D, V, _step(second, [2, 3]))
    assert torch.equal(o1, got[rows1]) and torch.equal(o2, got[rows2]) and torch.equal(state2, state)


@gpu
def test_small_kernels_against_plain_formulas():
    """Routing over groups, the short convolution with its carried inputs, the decays, the gated head norm, the norm
    of a sublayer's output and the partly rotated keys, each against a few lines of plain arithmetic."""
    import kernel_refs as ref
    from zinfer_b200 import ops

    gen = torch.Generator().manual_seed(5)
    r = lambda *s: torch.randn(s, generator=gen)
    # routing: 12 experts in 4 groups of which 3 are kept, sigmoid scores, weights times 2.5
    logits = 2.0 * r(50, 12)
    for score, groups, keep, top in (("sigmoid", 4, 3, 4), ("sigmoid", 12, 5, 3), ("softmax", 1, 1, 2), ("sigmoid", 3, 1, 4)):
        c, w = ops.moe_route_grouped(logits.to(DEV), top, score, groups, keep, 2.5)
        rc, rw = ref.moe_route_grouped(logits, top, score, groups, keep, 2.5)
        assert torch.equal(c.cpu().sort(-1).values, rc.sort(-1).values) and torch.allclose(w.cpu().sort(-1).values, rw.sort(-1).values, rtol=1e-5)
    # convolution: three requests in slots 1, 0, 2, one of them shorter than the taps
    for taps in (4, 2, 1):
        C, q_lens, slots = 10, [2, 7, 1], [1, 0, 2]
        x, kern, tail = r(10, 16)[:, 3:13], r(C, taps), r(4, max(taps - 1, 0), C)
        cpu_step = SimpleNamespace(cu_q=torch.tensor([0, 2, 9, 10]), state_slots=torch.tensor(slots), n_seqs=3)
        want, want_tail = ref.short_conv(x, kern, tail, cpu_step), tail.clone()
        ref.short_conv_carry(x, taps, want_tail, cpu_step)
        x_dev, tail_dev = x.to(DEV), tail.to(DEV)
        got = ops.short_conv(x_dev, kern.to(DEV), tail_dev, _step(q_lens, slots))
        ops.short_conv_carry(x_dev, taps, tail_dev, _step(q_lens, slots))
        assert torch.allclose(got.cpu(), want, rtol=1e-5, atol=1e-6) and torch.allclose(tail_dev.cpu(), want_tail)
    # decays
    z, bias, a_log = r(9, 24), r(24), 0.3 * r(3)
    assert torch.allclose(ops.decay_sigmoid_root_(z.to(DEV), bias.to(DEV), 16.0).cpu(), torch.sigmoid(z + bias) ** (1 / 16.0), rtol=1e-5)
    want = torch.exp(-torch.exp(a_log).repeat_interleave(8) * torch.nn.functional.softplus(z + bias))
    assert torch.allclose(ops.decay_exp_softplus_(z.to(DEV), bias.to(DEV), a_log.to(DEV), 8).cpu(), want, rtol=1e-5)
    # unit norm of part of a row, gated head norm
    x = r(7, 40)
    got = ops.unit_norm_(x.to(DEV)[:, :30], 3, 10, 1e-6, 0.25).cpu()
    v = x[:, :30].reshape(7, 3, 10)
    assert torch.allclose(got, (0.25 * v / torch.sqrt((v * v).sum(-1, keepdim=True) + 1e-6)).reshape(7, 30), rtol=1e-5)
    o, wt, gate = r(7, 36), 1 + 0.1 * r(12), r(7, 36)
    for kind in ("silu", "sigmoid"):
        want = ref.head_norm_gate(o, wt, 1e-5, gate, kind, 3, 12, torch.float32)
        assert torch.allclose(ops.head_norm_gate(o.to(DEV), wt.to(DEV), 1e-5, gate.to(DEV), kind, 3, 12, torch.float32).cpu(), want, rtol=1e-5, atol=1e-6)
    # the norm of two scaled updates, added into the stream
    h, a, b, wt = r(6, 44), r(6, 44), r(6, 44), 1 + 0.1 * r(44)
    want_h = h.clone()
    ref.norm_residual(want_h, ref.Scaled(a, 0.7), wt, 1e-5, torch.float32, b=ref.Scaled(b, 1.3))
    h_dev = h.to(DEV)
    x = ops.norm_residual(h_dev, ops.Scaled(a.to(DEV), 0.7), wt.to(DEV), 1e-5, torch.bfloat16, b=ops.Scaled(b.to(DEV), 1.3))
    assert torch.allclose(h_dev.cpu(), want_h, rtol=1e-5, atol=1e-6) and torch.equal(x.cpu(), h_dev.cpu().to(torch.bfloat16))
    # the same in its other forms: many rows (16-byte accesses; widths that do not allow them), updates in bfloat16,
    # updates as split-K partial sums over few rows, one update only; relu^2 with and without 16-byte accesses
    for T, H, parts in ((600, 48, 0), (600, 43, 0), (5, 4100, 3), (520, 36, 2), (3, 52, 0)):
        h, wt = r(T, H), 1 + 0.1 * r(H)
        a = r(parts, T, H) if parts else r(T, H).to(torch.bfloat16)
        for b in (None, r(T, H)):
            want_h = h.clone()
            ref.norm_residual(want_h, ref.Scaled(a.sum(0) if parts else a, 0.7), wt, 1e-5, torch.float32,
                              b=None if b is None else ref.Scaled(b, 1.3))
            h_dev = h.to(DEV)
            x = ops.norm_residual(h_dev, ops.Scaled(ops.Partials(a.to(DEV)) if parts else a.to(DEV), 0.7), wt.to(DEV), 1e-5,
                                  torch.bfloat16, b=None if b is None else ops.Scaled(b.to(DEV), 1.3))
            assert torch.allclose(h_dev.cpu(), want_h, rtol=1e-5, atol=2e-6), (T, H, parts, b is None)
            assert torch.equal(x.cpu(), h_dev.cpu().to(torch.bfloat16))
    for n, dt in ((4096, torch.bfloat16), (37, torch.float32), (1028, torch.float32)):
        v = r(n).to(dt)
        assert torch.equal(ops.relu2_(v.to(DEV)).cpu(), (torch.relu(v.float()) ** 2).to(dt))
    # keys: norm, rotation of the first 6 of 10 dimensions with scaled positions, raw keys as values
    nq, nkv, d, rot, page = 4, 2, 10, 6, 4
    qkv = r(5, (nq + nkv) * d)
    cos, sin = ops.rope_table(16, rot, 100.0, DEV, 2.0)
    rc, rs = ref.rope_table(16, rot, 100.0, "cpu", 2.0)
    assert torch.allclose(cos.cpu(), rc, atol=1e-6) and torch.allclose(sin.cpu(), rs, atol=1e-6)
    pos, slots = torch.tensor([3, 4, 5, 0, 9], dtype=torch.int32), torch.tensor([7, 8, 9, 0, -1], dtype=torch.int32)
    qw, kw = 1 + 0.1 * r(d), 1 + 0.1 * r(d)
    kc, vc = torch.zeros(3, nkv, page, d), torch.zeros(3, nkv, page, d)
    want = ref.qk_prepare(qkv.clone(), nq, nkv, d, rot, qw, kw, 1e-5, rc, rs, pos, kc, vc, slots, page, values_from_keys=True)
    kd, vd = torch.zeros(3, nkv, page, d, device=DEV), torch.zeros(3, nkv, page, d, device=DEV)
    got = ops.qk_prepare(qkv.to(DEV), nq, nkv, d, rot, qw.to(DEV), kw.to(DEV), 1e-5, cos, sin, pos.to(DEV), kd, vd, slots.to(DEV),
                         page, values_from_keys=True)
    assert torch.allclose(got.cpu()[:, :nq * d], want[:, :nq * d], rtol=1e-5, atol=1e-6)
    assert torch.allclose(kd.cpu(), kc, rtol=1e-5, atol=1e-6) and torch.allclose(vd.cpu(), vc)
    assert torch.equal(vd.cpu()[1, :, 3], qkv[0, nq * d:].reshape(nkv, d))          # slot 7: the key as projected
