"""The Luvavik design in the engine against the plain implementation (tests/plain_luvavik.py).

Every test makes its own small configuration and weights (tests/luvavik_util.py).  The CPU tests put
the plain PyTorch stand-ins of the kernels (tests/kernel_refs.py) under the engine, so they test what
is host logic: configuration, registry, tensor names, the schedule of looped layers, caches and state
slots per pass, batching.  The GPU tests run the same traces on the kernels, in float32 and bfloat16:
whole prompts, prompts followed by token-by-token decoding (from CUDA graphs), portions down to one and
two tokens, mixed batches of unequal requests with pages and state slots that are used again, long
prompts whose attention is peaky (a far key, a key at a page's edge or a stale page would show), a
recurrence that remembers for dozens of tokens, and greedy generation through ``Engine.generate``.
"""
import copy
import json

import numpy as np
import pytest
import torch

import luvavik_util as U
import plain_luvavik as P
import replay_util as ru

DEV = "cuda:0"
# float32: the engine against 64-bit arithmetic, both from the same bfloat16-representable weights;
# relative to a row's largest logit.  bfloat16: products and activations are rounded to 8 bits of
# mantissa between kernels, over up to eight layer runs, and the tests' peaky attention (scores spread
# over tens of units, so that a lost key shows) multiplies the rounding of q and k by that spread.  The
# float32 runs go through the same kernels and are the sharp test of every index and edge.
TOL = {torch.float32: dict(rtol=5e-5, atol=1e-6), torch.bfloat16: dict(rtol=8e-2, atol=4e-3)}


def plain_logits(cfg, weights, reqs):
    w64 = U.f64(weights)
    return {rid: P.forward(cfg, w64, toks).numpy() for rid, toks in reqs.items()}


def make_runner(tmp_path, cfg, weights, dtype, device, **kw):
    from zinfer_b200.engine import ModelRunner

    d = U.write_model(str(tmp_path / f"m{abs(hash(json.dumps(cfg, sort_keys=True))) % 10**8}"), cfg, weights)
    kw.setdefault("page_size", 8)
    kw.setdefault("max_requests", 4)
    return ModelRunner.from_model_dir(d, dtype=dtype, device=device, **kw)


# ============================================================================ CPU
def test_config_is_read_and_registered():
    from zinfer_b200.config import ConfigError, LuvavikConfig, family_for, luvavik_model_spec
    from zinfer_b200.engine.model import declared_tensors

    raw = U.CONFIGS["mix"]
    fam = family_for(raw)
    assert fam.name == "Luvavik" and fam.config_class is LuvavikConfig
    cfg = LuvavikConfig.from_dict(raw)
    assert LuvavikConfig.from_dict(cfg.to_dict()) == cfg                      # survives a round trip
    spec = luvavik_model_spec(cfg)
    # the tensors the model asks for are exactly the design's names and shapes
    want = U.tensor_shapes(raw)
    got = {k: tuple(v.shape) for k, v in declared_tensors(spec).items()}
    assert got == want
    # layers 1..2 run twice, every run with a cache of its own, and a vector is added before each pass
    assert [(e.layer, e.pre_add) for e in spec.schedule] == [
        (0, None), (1, ("loop.step", 0)), (2, None), (1, ("loop.step", 1)), (2, None), (3, None)]
    assert all(e.cache is None for e in spec.schedule)
    for name, other in U.CONFIGS.items():
        assert {k: tuple(v.shape) for k, v in declared_tensors(luvavik_model_spec(LuvavikConfig.from_dict(other))).items()} \
            == U.tensor_shapes(other), name
    bad = copy.deepcopy(raw)
    bad["layers"][0]["type"] = "convolution"
    with pytest.raises(ConfigError, match="unknown mixer"):
        LuvavikConfig.from_dict(bad)
    bad = copy.deepcopy(raw)
    bad["loop"]["stop"] = 9
    with pytest.raises(ConfigError, match="loop"):
        LuvavikConfig.from_dict(bad)
    bad = copy.deepcopy(raw)
    del bad["layers"][1]["mixer"]["blocks"]
    with pytest.raises(ConfigError, match="blocks"):
        LuvavikConfig.from_dict(bad)


def test_command_line_inspects_the_model(tmp_path):
    import io

    from zinfer_b200 import cli

    d = U.write_model(str(tmp_path / "m"), U.CONFIGS["alt"], U.make_weights(U.CONFIGS["alt"], seed=1))
    out = io.StringIO()
    assert cli.run(["inspect-config", d], out) == 0
    text = out.getvalue()
    assert "architecture: Luvavik" in text and "loop: layers 0..1 run 1 times" in text
    assert "layer 1: latent_attention" in text and "moe experts=4 top=1 identity=0 ff=56" in text
    out = io.StringIO()
    assert cli.run(["inspect-weights", d], out) == 0 and "tensor_count:" in out.getvalue()


def test_caches_and_states_per_pass():
    from zinfer_b200.config import LuvavikConfig, luvavik_model_spec
    from zinfer_b200.engine import DecoderModel

    model = DecoderModel(luvavik_model_spec(LuvavikConfig.from_dict(U.CONFIGS["mix"])), torch.float32, "cpu")
    kv, state = model.cache_needs()
    # runs: attention, (recurrent, attention) x 2, recurrent: three latent caches, three states
    assert len(kv) == 3 and len(state) == 3
    assert all(n.num_kv_heads == 1 and n.head_dim == 32 + 8 and not n.values for n in kv.values())
    assert all(n.shape == (4, 48) and n.dtype == torch.float32 for n in state.values())


@pytest.mark.parametrize("name", ["mix", "alt", "flat"])
def test_engine_host_logic_on_stand_ins(cpu_kernels, tmp_path, name):
    cfg = U.CONFIGS[name]
    weights = U.make_weights(cfg, seed=3)
    runner = make_runner(tmp_path, cfg, weights, torch.float32, "cpu", max_tokens=192, max_requests=3, cuda_graphs=False)
    reqs = ru.make_requests(cfg["vocab"], [23, 1, 40, 9, 17], seed=4)
    plain = plain_logits(cfg, weights, reqs)
    for mode, trace in (("whole", ru.trace_whole(reqs)), ("tail", ru.trace_tail_decode(reqs, 6)),
                        ("portions", ru.trace_portions(reqs, 2)), ("mixed", ru.trace_mixed(reqs, 5, max_live=3, tail=4))):
        got = ru.run_in_process(runner, trace)
        ru.assert_close(got, plain, what=f"{name}/{mode}", argmax_frac=0.0, rtol=2e-4, atol=1e-5)
        assert not runner.manager.requests
    assert runner.manager.slots.reused > 0        # three slots served five requests, four times over


def test_plain_model_pieces():
    """The plain implementation against numbers worked out by hand."""
    F = torch.float64
    # convolution: kernel [1, 2, 3] on inputs 1, 10, 100 gives 3, 32, 321 (the last column meets the current token)
    out = P.causal_conv(torch.tensor([[1.0], [10.0], [100.0]], dtype=F), torch.tensor([[1.0, 2.0, 3.0]], dtype=F),
                        torch.zeros(1, dtype=F))
    assert out.reshape(-1).tolist() == [3.0, 32.0, 321.0]
    # a quarter turn at position 1 with base 1: (u, v) = (1, 0) -> (cos 1, sin 1); the rest passes
    r = P.rotate_half(torch.tensor([[1.0, 0.0, 7.0]], dtype=F), torch.tensor([1]), 2, 1.0)
    assert torch.allclose(r, torch.tensor([[np.cos(1.0), np.sin(1.0), 7.0]], dtype=F))
    # routing: scores 0.5, 0.3, 0.2; the correction lifts the last above the second; weights stay scores
    w = {"r.router": torch.log(torch.tensor([[0.5], [0.3], [0.2]], dtype=F)), "r.correction": torch.tensor([0.0, 0.0, 0.2], dtype=F)}
    chosen, weight = P.route(torch.ones(1, 1, dtype=F), w, "r.", {"top": 2})
    assert chosen.tolist() == [[0, 2]] and torch.allclose(weight, torch.tensor([[0.5, 0.2]], dtype=F))
    assert abs(P.gelu_tanh(torch.tensor(1.0, dtype=F)).item() - 0.8411919906082768) < 1e-12


# ============================================================================ GPU
gpu = pytest.mark.gpu


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", list(U.MECHANISMS))
def test_each_mechanism_alone(tmp_path, name, dtype):
    cfg = U.MECHANISMS[name]
    weights = U.make_weights(cfg, seed=11)
    w64 = U.f64(weights)
    reqs = U.clear_requests(cfg, w64, [37, 1, 20], seed=12, margin=0.05)
    plain = plain_logits(cfg, weights, reqs)
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
        reqs = U.clear_requests(cfg, U.f64(weights), [45, 3, 70, 18, 1, 33], seed=5, margin=0.04)
        out[name] = (cfg, weights, reqs, plain_logits(cfg, weights, reqs))
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
    """Unequal requests in one batch give the rows they give alone, to the last bits in float32 (a request
    that brings one token takes the fused single-token kernels when it is alone, so not bit for bit)."""
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
        if dtype == torch.float32:
            assert (part - want).abs().max() <= 2e-6 * want.abs().max(), e.request_id
        else:
            assert (part - want).abs().max() <= 2e-2 * want.abs().max(), e.request_id


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_far_keys_page_edges_and_long_memory(tmp_path, dtype):
    """Prompts of several hundred tokens whose attention is peaky (scores spread over tens of units) and
    whose recurrence forgets slowly: whole, against portions that end on, one before and one after page
    edges, against long token-by-token decoding, with pages poisoned when they are given back."""
    cfg = U.config(131, 64, [
        U.layer(U.attn(4, 16, 8, 16, 24, 2.5), U.dense(64)),
        U.layer(U.rec(64, 2, 4), None),
        U.layer(U.attn(4, 16, 8, 16, 24, 2.5), None),
    ], loop=(1, 3, 2), residual_mult=0.5, logit_scale=1.0)
    weights = U.make_weights(cfg, seed=31, slow_decay=True)
    reqs = ru.make_requests(cfg["vocab"], [300, 203], seed=6)
    plain = plain_logits(cfg, weights, reqs)
    # the peaks are real: in the plain model the last token's attention puts most of its weight on few keys
    runner = make_runner(tmp_path, cfg, weights, dtype, DEV, page_size=16, max_tokens=320, max_requests=2,
                         poison_freed_pages=True)
    edges = (16, 15, 1, 17, 31, 2, 30, 33, 47, 64, 1, 1, 14)      # cumulative ends: 16, 31, 32, 49, 80, 82, 112, ...
    for mode, trace in (("whole", ru.trace_whole(reqs)), ("edges", ru.trace_portions(reqs, 0, sizes=edges)),
                        ("long decode", ru.trace_tail_decode(reqs, 90))):
        got = ru.run_in_process(runner, trace)
        ru.assert_close(got, plain, what=f"far/{mode}", argmax_frac=0.0, **TOL[dtype])
    runner.manager.check()


@gpu
def test_a_single_far_key_decides(tmp_path):
    """One key 250 tokens back carries much of the last query's softmax: among all tokens that could stand
    at position 19, the test takes the one whose presence moves the last position's logits most in the plain
    model, and requires that move to be large; an engine that lost that key could not match."""
    cfg = U.config(67, 32, [U.layer(U.attn(2, 8, 8, 8, 16, 1.5), None)])
    weights = U.make_weights(cfg, seed=41)
    w64 = U.f64(weights)
    toks = ru.make_requests(cfg["vocab"], [270], seed=7)["r0"]
    without = toks[:19] + [toks[18]] + toks[20:]
    lost = plain_logits(cfg, weights, {"r0": without})
    move = {c: np.abs(P.forward(cfg, w64, toks[:19] + [c] + toks[20:]).numpy()[-1] - lost["r0"][-1]).max()
            for c in range(cfg["vocab"])}
    toks[19] = max(move, key=move.get)
    plain = plain_logits(cfg, weights, {"r0": toks})
    assert np.abs(plain["r0"][-1] - lost["r0"][-1]).max() > 0.05 * np.abs(plain["r0"][-1]).max()     # the far key matters
    for dtype in (torch.float32, torch.bfloat16):
        runner = make_runner(tmp_path, cfg, weights, dtype, DEV, page_size=16, max_tokens=288, max_requests=1)
        for trace in (ru.trace_whole({"r0": toks}), ru.trace_tail_decode({"r0": toks}, 5)):
            ru.assert_close(ru.run_in_process(runner, trace), plain, what="one far key", argmax_frac=0.0, **TOL[dtype])


@gpu
def test_greedy_generation_through_the_engine(tmp_path, models):
    from zinfer_b200.engine.api import Engine
    from zinfer_b200.sampling import SamplingParams

    cfg, weights, reqs, _ = models["alt"]
    d = U.write_model(str(tmp_path / "gen"), cfg, weights)
    w64 = U.f64(weights)
    prompts = [reqs["r1"], reqs["r3"], reqs["r0"][:30]]
    eng = Engine(d, dtype="float32", device=DEV, page_size=8, kv_cache_tokens=192, max_batched_tokens=16, max_requests=3)
    got = eng.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=6, ignore_eos=True))
    for p, r in zip(prompts, got):
        assert len(r.token_ids) == 6
        logits = P.forward(cfg, w64, p + r.token_ids).numpy()
        for i, t in enumerate(r.token_ids):      # the best token given the same history, or tied with it to rounding
            row = logits[len(p) - 1 + i]
            assert row[t] >= row.max() - 1e-4 * np.abs(row).max()


@gpu
def test_command_line_generates(tmp_path):
    """bin/zinfer: a model folder of random weights made from a Luvavik config.json, greedy tokens in float32 as the
    plain model gives them, and sampled tokens with the reference's options (the sampling kernel on this vocabulary)."""
    import os
    import subprocess
    import sys

    cfg = U.CONFIGS["flat"]
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(cfg))
    d = str(tmp_path / "random")
    tool = os.path.join(ru.REPO, "bin", "zinfer")
    r = subprocess.run([sys.executable, tool, "random-model", d, str(cfg_path), "7"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    pcfg, w = P.load_model(d)
    r = subprocess.run([sys.executable, tool, "generate-token-ids", d, "5,17,3,60,2", "6", "--dtype", "float32"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    want = [5, 17, 3, 60, 2] + P.greedy(pcfg, w, [5, 17, 3, 60, 2], 6)
    assert "tokens: [" + ", ".join(map(str, want)) + "]" in r.stdout
    r = subprocess.run([sys.executable, tool, "generate-token-ids", d, "5,17,3,60,2", "6", "--temperature", "0.8", "--top-k", "10",
                        "--seed", "3"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "tokens: [5, 17, 3, 60, 2, " in r.stdout, r.stderr[-2000:]


@gpu
def test_replay_program(tmp_path, models):
    """bin/trace_run as a user runs it: the model class comes from config.json, four state slots."""
    cfg, weights, reqs, plain = models["flat"]
    d = U.write_model(str(tmp_path / "tool"), cfg, weights)
    trace = ru.trace_mixed(reqs, 3, max_live=4, tail=8)
    info = {}
    got = ru.run_trace_tool(d, "float32", trace, str(tmp_path / "out"), ru.max_live_tokens(trace), cfg["vocab"], info=info)
    ru.assert_close(got, plain, what="trace_run", argmax_frac=0.0, **TOL[torch.float32])
    assert info["pages_reused"] and info["pages_reused"] > 0


@gpu
def test_kernels_of_the_new_parts_against_plain_formulas():
    """Routing and the recurrence as kernels, each against a few lines of 64-bit arithmetic."""
    from types import SimpleNamespace

    from zinfer_b200 import ops

    gen = torch.Generator().manual_seed(2)
    # routing: 37 tokens, 11 outputs, 3 chosen, with ties made on purpose (equal logits): the lower index wins
    logits = torch.randn(37, 11, generator=gen)
    logits[5, 3] = logits[5, 7] = 4.0
    corr = 0.1 * torch.randn(11, generator=gen)
    corr[3] = corr[7] = 0.0
    chosen, weight = ops.moe_route(logits.to(DEV), corr.to(DEV), 3)
    s = torch.softmax(logits.double(), dim=-1)
    want = torch.topk(s + corr.double(), 3, dim=-1).indices
    assert sorted(chosen[5].tolist())[:2].count(3) == 1 and 7 in chosen[5].tolist()
    assert (chosen.cpu().sort(dim=1).values == want.sort(dim=1).values.int()).all()
    assert torch.allclose(weight.cpu().double(), torch.gather(s, 1, chosen.cpu().long()), rtol=1e-5, atol=1e-7)
    # the pairs laid out by expert: every real pair has a row of its expert's tiles, identity pairs none
    row_token, row_self, pair_row, tile_expert, n_tiles = ops.moe_align(chosen, 9, 16)
    pr, rt, te = pair_row.cpu().tolist(), row_token.cpu().tolist(), tile_expert.cpu().tolist()
    flat = chosen.cpu().reshape(-1).tolist()
    for p, e in enumerate(flat):
        if e >= 9:
            assert pr[p] == -1
        else:
            assert rt[pr[p]] == p // 3 and te[pr[p] // 16] == e
    assert len({r for r in pr if r >= 0}) == sum(e < 9 for e in flat)
    # the router's product and the choice in one kernel against the product followed by the choice
    xr, wr = torch.randn(37, 52, generator=gen).to(torch.bfloat16).to(DEV), torch.randn(11, 52, generator=gen).to(torch.bfloat16).to(DEV)
    c2, w2 = ops.moe_router(xr, wr, corr.to(DEV), 3)
    c1, w1 = ops.moe_route(ops.linear_cuda_cores(xr, wr, out_dtype=torch.float32), corr.to(DEV), 3)
    assert torch.equal(c1, c2) and torch.allclose(w1, w2, rtol=1e-5, atol=1e-7)
    # few rows per expert: the memory-bound grouped product against the general one, on the same layout
    for dt in (torch.float32, torch.bfloat16):
        xe = torch.randn(37, 40, generator=gen).to(dt).to(DEV)
        we = torch.randn(9, 28, 40, generator=gen).to(dt).to(DEV)
        a = torch.zeros((row_token.numel(), 28), dtype=torch.float32, device=DEV)
        b = torch.zeros_like(a)
        ops.linear_grouped(xe, we, a, row_token, tile_expert, n_tiles, 16, relu2=True)
        assert ops.linear_few_rows_ok(xe, we)
        ops.linear_few_rows(xe, we, b, row_token, tile_expert, n_tiles, relu2=True)
        torch.testing.assert_close(b, a, rtol=1e-5, atol=1e-5)
    # recurrence: two requests of 9 and 4 tokens continue from given states; 5 channels in one block, 3 taps
    T, C, taps = 13, 5, 3
    step = SimpleNamespace(cu_q=torch.tensor([0, 9, 13], dtype=torch.int32, device=DEV),
                           state_slots=torch.tensor([2, 0], dtype=torch.int32, device=DEV), n_seqs=2)
    x, y = torch.randn(T, C, generator=gen), torch.randn(T, C, generator=gen)
    xb, yb, cb = (0.3 * torch.randn(C, generator=gen) for _ in range(3))
    kern, lam = torch.randn(C, taps, generator=gen), torch.randn(C, generator=gen) - 2.0
    gates, rb, ib = torch.randn(T, 1, 2, C, generator=gen), torch.randn(C, generator=gen), torch.randn(C, generator=gen)
    state = torch.randn(3, taps, C, generator=gen)
    dev = lambda t: t.to(DEV).contiguous()
    st = dev(state)
    u = ops.causal_conv(dev(x), dev(xb), dev(kern), dev(cb), st, step)
    out = ops.rglru_scan(u, dev(gates), C, dev(rb), dev(ib), dev(lam), 8.0, dev(y), dev(yb), dev(x), dev(xb), st, step)
    for (lo, hi), slot in (((0, 9), 2), ((9, 13), 0)):
        seq = torch.cat([state[slot, :taps - 1], x[lo:hi] + xb]).double()
        S = state[slot, taps - 1].double()
        for t in range(hi - lo):
            uu = cb.double() + (kern.double() * seq[t:t + taps].T).sum(dim=1)
            assert torch.allclose(u[lo + t].cpu().double(), uu, rtol=1e-5, atol=1e-6)
            r, i = torch.sigmoid(gates[lo + t, 0, 0].double() + rb), torch.sigmoid(gates[lo + t, 0, 1].double() + ib)
            a = torch.exp(-8.0 * r * torch.nn.functional.softplus(lam.double()))
            S = a * S + torch.sqrt(1 - a * a) * i * uu
            assert torch.allclose(out[lo + t].cpu().double(), S * P.gelu_tanh(y[lo + t].double() + yb), rtol=2e-5, atol=1e-6)
        assert torch.allclose(st[slot, taps - 1].cpu().double(), S, rtol=2e-5, atol=1e-6)
        assert torch.allclose(st[slot, :taps - 1].cpu().double(), seq[-(taps - 1):], rtol=1e-6, atol=1e-7)
    assert torch.equal(st[1].cpu(), state[1])          # a slot of no request in the step is left alone
    # one token per request: the fused kernel against the three kernels it stands for
    n, B, bw = 3, 2, 6
    C = B * bw
    step1 = SimpleNamespace(cu_q=torch.arange(n + 1, dtype=torch.int32, device=DEV), n_seqs=n,
                            state_slots=torch.tensor([1, 3, 0], dtype=torch.int32, device=DEV))
    yx = dev(torch.randn(n, 2 * C, generator=gen))
    yb, xb, cb, rb, ib = (dev(0.3 * torch.randn(C, generator=gen)) for _ in range(5))
    kern, lam = dev(torch.randn(C, taps, generator=gen)), dev(torch.randn(C, generator=gen) - 2.0)
    wg = dev(torch.randn(B, 2 * bw, bw, generator=gen))
    state0 = torch.randn(4, taps, C, generator=gen)
    sa, sb = dev(state0), dev(state0)
    u = ops.causal_conv(yx[:, C:], xb, kern, cb, sa, step1)
    gates = torch.empty((n, B, 2 * bw), dtype=torch.float32, device=DEV)
    ops.linear_batched(u.view(n, B, bw).transpose(0, 1), wg, gates.transpose(0, 1))
    want = ops.rglru_scan(u, gates, bw, rb, ib, lam, 8.0, yx[:, :C], yb, yx[:, C:], xb, sa, step1)
    got = ops.rglru_decode(yx, yb, xb, kern, cb, wg, rb, ib, lam, 8.0, sb, step1)
    torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(sb, sa, rtol=1e-5, atol=1e-6)


@gpu
def test_recurrence_in_chunks_against_the_walk():
    """Three requests of 70, 1 and 89 tokens in one bfloat16 step (the recurrence runs in chunks of the flat
    batch, across the requests' borders) against the same step in float32 (token by token)."""
    from types import SimpleNamespace

    from zinfer_b200 import ops

    gen = torch.Generator().manual_seed(9)
    T, B, bw, taps = 160, 2, 20, 4
    C = B * bw
    step = SimpleNamespace(cu_q=torch.tensor([0, 70, 71, 160], dtype=torch.int32, device=DEV), n_seqs=3,
                           state_slots=torch.tensor([2, 0, 3], dtype=torch.int32, device=DEV))
    dev = lambda t: t.to(DEV).contiguous()
    yx = torch.randn(T, 2 * C, generator=gen).to(torch.bfloat16)
    yb, xb, rb, ib = (dev(0.3 * torch.randn(C, generator=gen)) for _ in range(4))
    lam = dev(torch.randn(C, generator=gen) - 3.0)                      # slow decay: chunks feed one another
    u, gates = dev(torch.randn(T, C, generator=gen)), dev(torch.randn(T, B, 2 * bw, generator=gen))
    state0 = torch.randn(4, taps, C, generator=gen)
    outs, states = [], []
    for dtype in (torch.float32, torch.bfloat16):
        st, v = dev(state0), dev(yx.to(dtype))
        outs.append(ops.rglru_scan(u, gates, bw, rb, ib, lam, 8.0, v[:, :C], yb, v[:, C:], xb, st, step).float())
        states.append(st)
    torch.testing.assert_close(outs[1], outs[0], rtol=1e-2, atol=1e-2)          # the result's own rounding to bfloat16
    torch.testing.assert_close(states[1], states[0], rtol=1e-5, atol=1e-6)      # the carried state is 32-bit in both
    assert torch.equal(states[1][1].cpu(), state0[1])


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,D,rank,page", [(6, 40, 32, 8), (20, 24, 16, 4), (16, 576, 512, 16), (3, 200, 136, 16)])
def test_latent_attention_kernels_agree(dtype, heads, D, rank, page):
    """Single tokens through the split-key kernel (1, 3 and many splits; 1 to 700 keys, tile edges at 31/32/33) and,
    in bfloat16, a portion through the tensor-core products, each against the exact kernel on the same pages."""
    from types import SimpleNamespace

    from zinfer_b200 import ops

    gen = torch.Generator().manual_seed(heads * D)
    kv_lens = [1, 31, 32, 33, 700, 64, 257]
    n = len(kv_lens)
    blocks = [-(-k // page) for k in kv_lens]
    n_pages = sum(blocks) + 5
    perm = torch.randperm(n_pages, generator=gen).tolist()
    bt = -torch.ones((n, max(blocks)), dtype=torch.int32)
    at = 0
    for i, b in enumerate(blocks):
        bt[i, :b] = torch.tensor(perm[at:at + b], dtype=torch.int32)
        at += b
    cache = torch.randn(n_pages, 1, page, D, generator=gen).to(dtype).to(DEV)
    q = (torch.randn(n, heads * D, generator=gen) * (3.0 / D ** 0.5)).to(dtype).to(DEV)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    step = SimpleNamespace(cu_q=i32(list(range(n + 1))), kv_lens=i32(kv_lens), tile_seq=i32(list(range(n))), tile_q0=i32([0] * n),
                           dec_seq=i32(list(range(n))), n_dec=n, n_seqs=n, q_lens=[1] * n, ctx_lens=[k - 1 for k in kv_lens],
                           max_kv_len=max(kv_lens))
    bt = bt.to(DEV)
    before = ops.ATTENTION_BACKEND
    try:
        ops.ATTENTION_BACKEND = "generic"
        want = ops.latent_attention(q, cache, bt, step, heads, rank, page, None, 1.0)
    finally:
        ops.ATTENTION_BACKEND = before
    tol = dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    for max_kv in (40, 300, 5000):          # 1, a few and 32 splits in bfloat16; always 8 in float32
        step.max_kv_len = max_kv
        got = ops.latent_attention(q, cache, bt, step, heads, rank, page, None, 1.0)
        torch.testing.assert_close(got.float(), want.float(), **tol)
    if dtype == torch.bfloat16 and D % 8 == 0 and rank % 8 == 0:
        # a portion of 600 tokens that follows 100 cached ones, on the tensor cores (two blocks of queries)
        n_q, kv = 600, 700
        pages = torch.tensor(perm[:-(-kv // page)], dtype=torch.int32, device=DEV).reshape(1, -1).contiguous()
        qp = (torch.randn(n_q, heads * D, generator=gen) * (3.0 / D ** 0.5)).to(dtype).to(DEV)
        tr = ops.attention_tile_rows()
        tiles = -(-n_q // tr)
        pstep = SimpleNamespace(cu_q=i32([0, n_q]), kv_lens=i32([kv]), tile_seq=i32([0] * tiles), tile_q0=i32([t * tr for t in range(tiles)]),
                                dec_seq=i32([0]), n_dec=0, n_seqs=1, q_lens=[n_q], ctx_lens=[100], max_kv_len=kv)
        try:
            ops.ATTENTION_BACKEND = "generic"
            want = ops.latent_attention(qp, cache, pages, pstep, heads, rank, page, None, 1.0)
        finally:
            ops.ATTENTION_BACKEND = before
        got = ops.latent_attention(qp, cache, pages, pstep, heads, rank, page, None, 1.0)
        torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2)


@gpu
@pytest.mark.parametrize("T,H,K,N,pitch", [(300, 5, 72, 40, 96), (2048, 16, 128, 512, 192), (129, 3, 512, 128, 512), (200, 1, 64, 24, 80)])
def test_one_product_per_head_in_one_launch(T, H, K, N, pitch):
    """The tensor-core kernel's per-head form (heads side by side in their rows, also with columns between them and
    with K no multiple of the kernel's 64-column blocks) against one 64-bit product per head."""
    from zinfer_b200 import ops

    gen = torch.Generator().manual_seed(T + H)
    rows = torch.randn(T, H * pitch + 16, generator=gen).to(torch.bfloat16).to(DEV)
    x = rows[:, :H * pitch].view(T, H, pitch)[:, :, :K]
    w = (torch.randn(H, N, K, generator=gen) / K ** 0.5).to(torch.bfloat16).to(DEV)
    wide = torch.zeros(T, H * (N + 8), dtype=torch.bfloat16, device=DEV)
    out = wide.view(T, H, N + 8)[:, :, :N]
    assert ops.linear_heads_ok(x, w, out)
    ops.linear_heads(x, w, out)
    want = torch.einsum("thk,hnk->thn", x.double(), w.double())
    torch.testing.assert_close(out.double(), want, rtol=1e-2, atol=1e-2)
    assert wide.view(T, H, N + 8)[:, :, N:].abs().max() == 0          # nothing is written between the heads' results
    ops.require_kernel_status_ok("per-head product")
