"""Small Rogosun configurations and weights for the tests, made here from seeds.

The configurations differ from one another in every size and option: heads and groups of heads on both
sides of the parallel mixer, head sizes that are no multiples of the kernels' tiles, rotations of part of
a head, scaled and unscaled positions, taps of the short convolutions, experts in groups of several, of
one, or in one group, routers with and without a scale, layers without a feed-forward, any order of layers.
"""
from __future__ import annotations

import copy
import json
import os

import torch

import plain_rogosun as P


def gla(heads, dim, vdim, tau):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}}


def par(left, right, left_scale, right_scale):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}}


def att(heads, kv_heads, dim, scale, rot_dims, base=10000.0, factor=None):
    rot = {"base": base, "dims": rot_dims}
    if factor is not None:
        rot["scaling"] = {"factor": factor}
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale, "rot": rot}


def delta(heads, kv_heads, dim, vdim, taps):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": taps}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top, groups=None, scale=None, shared=None):
    router = {"experts": experts, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    if scale is not None:
        router["scale"] = scale
    out = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


def layer(mixer, mlp):
    out = copy.deepcopy(mixer)
    out["mlp"] = copy.deepcopy(mlp)
    return out


def config(vocab, width, layers, eps=1e-5):
    return {"architecture": "Rogosun", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps}}


# attention scores are made peaky (scale well above 1/sqrt(size)) so that a key that is lost, far away or at
# a page's edge changes the result by much more than any tolerance
CONFIGS = {
    # every mechanism; groups of two query heads on the left, of two value heads on the right; half of the head rotates
    "mix": config(211, 64, [
        layer(gla(3, 24, 16, 8.0), dense(96)),
        layer(par(att(4, 2, 16, 0.9, 8, factor=2.0), delta(4, 2, 24, 16, 4), 0.7, 1.3), moe(40, 6, 2, groups=(3, 2), scale=1.5, shared=24)),
        layer(gla(3, 24, 16, 8.0), moe(40, 6, 2, groups=(3, 2), scale=1.5, shared=24)),
        layer(par(att(4, 2, 16, 0.9, 8, factor=2.0), delta(4, 2, 24, 16, 4), 0.7, 1.3), None),
    ]),
    # parallel first; one head each; the whole head rotates, no scaling; two taps; groups of one expert; no shared expert
    "alt": config(157, 96, [
        layer(par(att(1, 1, 32, 0.6, 32, base=300.0), delta(1, 1, 40, 48, 2), 1.0, 1.0), moe(56, 4, 2, groups=(4, 3))),
        layer(gla(5, 40, 8, 2.0), None),
        layer(gla(2, 72, 36, 30.0), dense(72)),
    ], eps=3e-6),
    # sizes that are multiples of nothing: every product falls to the CUDA-core kernels; no groups, no scale, one tap
    "odd": config(97, 44, [
        layer(gla(3, 10, 6, 4.0), moe(18, 3, 2, shared=10)),
        layer(par(att(3, 1, 10, 1.1, 6, base=50.0, factor=1.5), delta(6, 3, 10, 14, 1), 0.4, 2.0), dense(30)),
    ]),
}
MECHANISMS = {
    "gla_alone": config(61, 32, [layer(gla(2, 16, 8, 4.0), None)]),
    "gla_wide_state": config(61, 32, [layer(gla(2, 80, 40, 16.0), None)]),       # more key channels than one part of the kernel
    "parallel_alone": config(61, 32, [layer(par(att(2, 1, 8, 1.2, 8), delta(2, 2, 8, 12, 3), 0.8, 0.5), None)]),
    "attention_only_matters": config(61, 32, [layer(par(att(4, 2, 8, 1.2, 4, factor=3.0), delta(2, 1, 8, 12, 3), 1.0, 1e-3), None)]),
    "delta_only_matters": config(61, 32, [layer(par(att(2, 1, 8, 1.2, 8), delta(4, 2, 16, 8, 5), 1e-3, 1.0), None)]),
    "dense_ff": config(61, 32, [layer(gla(2, 16, 8, 4.0), dense(40))]),
    "experts": config(61, 32, [layer(gla(2, 16, 8, 4.0), moe(20, 8, 3, groups=(4, 2), scale=2.5, shared=12))]),
    "experts_one_group": config(61, 32, [layer(gla(2, 16, 8, 4.0), moe(20, 5, 1))]),
}


def tensor_shapes(cfg, rank=8, gate_rank=12):
    """Names and shapes of a configuration's tensors, from the design's naming (no engine code)."""
    W = cfg["width"]
    out = {"embed": (cfg["vocab"], W), "head": (cfg["vocab"], W), "final.norm": (W,)}
    for i, lay in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lay["mixer"]
        out[p + "norm1"] = (W,)
        if lay["type"] == "gla":
            H, D, V = m["heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": (H * D, W), p + "mix.k": (H * D, W), p + "mix.v": (H * V, W), p + "mix.g": (H * V, W),
                        p + "mix.o": (W, H * V), p + "mix.norm": (V,), p + "mix.a1": (rank, W), p + "mix.a2": (H * D, rank),
                        p + "mix.a2.b": (H * D,)})
        else:
            a, d = m["left"], m["right"]
            q = p + "mix.left."
            out.update({q + "q": (a["heads"] * a["dim"], W), q + "k": (a["kv_heads"] * a["dim"], W), q + "q.norm": (a["dim"],),
                        q + "k.norm": (a["dim"],), q + "o": (W, a["heads"] * a["dim"])})
            q = p + "mix.right."
            H, G, D, V, taps = d["heads"], d["kv_heads"], d["dim"], d["vdim"], d["conv"]
            out.update({q + "q": (G * D, W), q + "q.conv": (G * D, taps), q + "k": (G * D, W), q + "k.conv": (G * D, taps),
                        q + "v": (H * V, W), q + "v.conv": (H * V, taps), q + "b": (H, W), q + "A_log": (H,), q + "norm": (V,),
                        q + "a1": (rank, W), q + "a2": (H * D, rank), q + "dt_bias": (H * D,), q + "g1": (gate_rank, W),
                        q + "g2": (H * V, gate_rank), q + "o": (W, H * V)})
        mlp = lay["mlp"]
        if mlp is None:
            continue
        out[p + "norm2"] = (W,)
        if mlp["kind"] == "dense":
            out.update({p + "mlp.up": (mlp["ff"], W), p + "mlp.down": (W, mlp["ff"])})
        else:
            ff = mlp["expert"]["ff"]
            for e in range(mlp["router"]["experts"]):
                out.update({f"{p}mlp.e{e}.gate": (ff, W), f"{p}mlp.e{e}.up": (ff, W), f"{p}mlp.e{e}.down": (W, ff)})
            out[p + "mlp.router"] = (mlp["router"]["experts"], W)
            if mlp.get("shared"):
                sf = mlp["shared"]["ff"]
                out.update({p + "mlp.shared.gate": (sf, W), p + "mlp.shared.up": (sf, W), p + "mlp.shared.down": (W, sf)})
    return out


def make_weights(cfg, seed, slow_decay=False, rank=8, gate_rank=12):
    """bfloat16-representable weights: matrices with unit-sized outputs, norms near 1, router matrices large (clear
    choices), biases that matter.  ``slow_decay`` makes both recurrences remember for hundreds of tokens (a lost or
    stale state then shows long after)."""
    gen = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tensor_shapes(cfg, rank, gate_rank).items():
        r = lambda *sh: torch.randn(sh or shape, generator=gen)
        if name.endswith(("norm", "norm1", "norm2")):
            t = 1.0 + 0.2 * (torch.rand(shape, generator=gen) - 0.5)
        elif name.endswith("a2.b"):                   # sigmoid(z)^(1/tau): z around 2 (or 6: a slow decay)
            t = (6.0 if slow_decay else 2.0) + 0.5 * r()
        elif name.endswith("dt_bias"):                # softplus(x) small: a slow decay
            t = (-5.0 if slow_decay else -1.0) + 0.5 * r()
        elif name.endswith("A_log"):
            t = 0.3 * r()
        elif name.endswith("router"):
            t = 6.0 * r() / shape[-1] ** 0.5
        elif name.endswith("conv"):
            t = r() / shape[-1] ** 0.5 + 0.5
        elif name == "embed":
            t = r()
        elif name.endswith((".a2", ".g2")):
            t = 2.0 * r() / shape[-1] ** 0.5
        else:
            t = r() / shape[-1] ** 0.5
        w[name] = t.to(torch.bfloat16)
    return w


def write_model(path, cfg, weights):
    from zinfer_b200.weights import write_safetensors

    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(path, "model.safetensors"), {k: v.contiguous() for k, v in weights.items()})
    return path


def plain_logits(cfg, weights, reqs):
    return {rid: P.PlainRogosun(cfg, weights).forward(toks).numpy() for rid, toks in reqs.items()}


def _margin(scores, top, groups, keep):
    """How far the score of the last chosen expert lies above the first one left out, and how far the last kept
    group lies above the first dropped one (the smaller of both)."""
    per = scores.numel() // groups
    gscore = scores.view(groups, per).topk(min(2, per), dim=-1).values.sum(-1)
    gs = gscore.sort(descending=True).values
    gm = float(gs[keep - 1] - gs[keep]) if keep < groups else float("inf")
    allowed = torch.zeros(groups, dtype=torch.bool)
    allowed[gscore.topk(keep).indices] = True
    cand = scores[allowed.repeat_interleave(per)].sort(descending=True).values
    em = float(cand[top - 1] - cand[top]) if top < cand.numel() else float("inf")
    return min(gm, em)


def clear_requests(cfg, weights, lengths, seed, margin):
    """Requests whose every choice of experts and of groups is clear by ``margin`` in the plain model: a choice that
    bfloat16 cannot tell apart would be no fault of the engine's.  Built token by token: the plain model carries its
    states, a candidate token is fed, and if one of its choices is unclear the states are put back and another is tried."""
    import random
    rng = random.Random(seed)
    has_moe = any(lay["mlp"] and lay["mlp"]["kind"] == "moe" for lay in cfg["layers"])
    margins = []
    orig = P.route

    def spy(scores, top, groups, keep):
        margins.append(_margin(scores, top, groups, keep))
        return orig(scores, top, groups, keep)

    reqs = {}
    P.route = spy
    try:
        for r, n in enumerate(lengths):
            model, toks = P.PlainRogosun(cfg, weights), []
            while len(toks) < n:
                for _ in range(300):
                    cand = rng.randrange(cfg["vocab"])
                    if not has_moe:
                        break
                    saved = (list(model.states), model.pos)
                    del margins[:]
                    model.forward([cand])
                    if min(margins) >= margin:
                        break
                    model.states, model.pos = saved
                else:
                    raise AssertionError("no candidate token with clear choices of experts")
                toks.append(cand)
            reqs[f"r{r}"] = toks
    finally:
        P.route = orig
    return reqs
