"""Small Luvavik configurations and weights for the tests, made here from seeds.

The configurations differ from one another in every size and option: heads, head sizes that
differ between keys and values, latent and rotary sizes, blocks and taps of the recurrent mixer,
experts chosen and identity experts, layers without a feed-forward, loops over different spans
(also from layer 0, also a single pass), multipliers of 1 and not 1.
"""
from __future__ import annotations

import copy
import json
import os
import random

import torch

import plain_luvavik as P


def attn(heads, dim, rot_dim, vdim, rank, scale, base=10000.0, rot_dims=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
                      "rot": {"base": base, "dims": rot_dims or rot_dim}}}


def rec(width, blocks, taps):
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": taps}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top, identity):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "identity": identity}}


def layer(mixer, mlp):
    out = copy.deepcopy(mixer)
    out["mlp"] = copy.deepcopy(mlp)
    return out


def config(vocab, width, layers, loop=None, residual_mult=1.0, logit_scale=1.0, eps=1e-5):
    cfg = {"architecture": "Luvavik", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps},
           "residual_mult": residual_mult, "logit_scale": logit_scale}
    if loop is not None:
        cfg["loop"] = dict(zip(("start", "stop", "times"), loop))
    return cfg


# scores are made peaky (scale well above 1/sqrt(size)) so that a key that is lost, far away or at a
# page's edge, changes the result by much more than any tolerance
CONFIGS = {
    # every mechanism, a loop over the middle, both multipliers away from 1
    "mix": config(211, 64, [
        layer(attn(3, 16, 8, 24, 32, 1.5), dense(96)),
        layer(rec(48, 3, 4), moe(40, 5, 2, 1)),
        layer(attn(3, 16, 8, 24, 32, 1.5), moe(40, 5, 2, 1)),
        layer(rec(48, 3, 4), None),
    ], loop=(1, 3, 2), residual_mult=0.4, logit_scale=1.7),
    # a loop from layer 0 with a single pass, one block, two taps, one expert chosen, no identity experts
    "alt": config(157, 96, [
        layer(rec(64, 1, 2), dense(72)),
        layer(attn(5, 24, 16, 8, 40, 2.0, base=300.0), moe(56, 4, 1, 0)),
        layer(attn(2, 8, 4, 32, 24, 2.5, base=5000.0), None),
    ], loop=(0, 2, 1), residual_mult=1.0, logit_scale=1.0, eps=3e-6),
    # no loop at all, three chosen of which any may be the identity
    "flat": config(97, 48, [
        layer(attn(1, 32, 32, 16, 16, 1.0), moe(24, 3, 3, 2)),
        layer(rec(80, 5, 3), dense(64)),
    ], residual_mult=0.7, logit_scale=0.5),
}
MECHANISMS = {
    "recurrent_alone": config(61, 32, [layer(rec(40, 2, 3), None)]),
    "attention_alone": config(61, 32, [layer(attn(2, 8, 8, 12, 16, 2.0), None)]),
    "dense_ff": config(61, 32, [layer(attn(2, 8, 8, 12, 16, 2.0), dense(40))], residual_mult=0.5),
    "experts": config(61, 32, [layer(attn(2, 8, 8, 12, 16, 2.0), moe(20, 4, 2, 1))], residual_mult=0.5),
    "loop": config(61, 32, [layer(rec(40, 2, 3), None), layer(attn(2, 8, 8, 12, 16, 2.0), None)], loop=(0, 2, 3)),
    # of the 8 rotated values only the first 4 turn; a convolution of one tap (nothing is carried but S)
    "partial_rotation": config(61, 32, [layer(attn(2, 8, 8, 12, 16, 2.0, rot_dims=4), None)]),
    "one_tap": config(61, 32, [layer(rec(40, 2, 1), dense(24))]),
    # sizes that are multiples of nothing: every product falls to the CUDA-core kernels, rows of 20 values
    "odd_sizes": config(53, 44, [layer(attn(3, 10, 6, 14, 14, 1.5), moe(18, 3, 2, 1)), layer(rec(20, 5, 2), dense(30))],
                        residual_mult=0.6, logit_scale=1.3),
}


def tensor_shapes(cfg):
    """Names and shapes of a configuration's tensors, from the design's naming (no engine code)."""
    W = cfg["width"]
    out = {"embed": (cfg["vocab"], W), "head": (cfg["vocab"], W), "final.norm": (W,)}
    if cfg.get("loop"):
        out["loop.step"] = (cfg["loop"]["times"], W)
    for i, lay in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lay["mixer"]
        out[p + "norm1"] = (W,)
        if lay["type"] == "rglru":
            C, B = m["width"], m["blocks"]
            out.update({p + "mix.y": (C, W), p + "mix.y.b": (C,), p + "mix.x": (C, W), p + "mix.x.b": (C,),
                        p + "mix.conv": (C, m["conv"]), p + "mix.conv.b": (C,), p + "mix.ra": (B, C // B, C // B),
                        p + "mix.ra.b": (B, C // B), p + "mix.ri": (B, C // B, C // B), p + "mix.ri.b": (B, C // B),
                        p + "mix.lam": (C,), p + "mix.o": (W, C)})
        else:
            H, D = m["heads"], m["kv_rank"] + m["rot_dim"]
            out.update({p + "mix.q": (H * (m["dim"] + m["rot_dim"]), W), p + "mix.dkv": (D, W),
                        p + "mix.dkv.norm": (m["kv_rank"],), p + "mix.uk": (H * m["dim"], m["kv_rank"]),
                        p + "mix.uv": (H * m["vdim"], m["kv_rank"]), p + "mix.g": (H * m["vdim"], W),
                        p + "mix.o": (W, H * m["vdim"])})
        mlp = lay["mlp"]
        if mlp is None:
            continue
        out[p + "norm2"] = (W,)
        if mlp["kind"] == "dense":
            out.update({p + "mlp.gate": (mlp["ff"], W), p + "mlp.up": (mlp["ff"], W), p + "mlp.down": (W, mlp["ff"])})
        else:
            r = mlp["router"]
            for e in range(r["experts"]):
                out[f"{p}mlp.e{e}.up"] = (mlp["expert"]["ff"], W)
                out[f"{p}mlp.e{e}.down"] = (W, mlp["expert"]["ff"])
            out[p + "mlp.router"] = (r["experts"] + r["identity"], W)
            out[p + "mlp.correction"] = (r["experts"] + r["identity"],)
    return out


def make_weights(cfg, seed, slow_decay=False):
    """bfloat16-representable weights: matrices with unit-sized outputs, norms near 1, router matrices large
    (clear choices), biases that matter.  ``slow_decay`` makes the recurrence remember for dozens of
    tokens (a lost or stale state then shows long after)."""
    gen = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        if name.endswith(("norm", "norm1", "norm2")):
            t = 1.0 + 0.2 * (torch.rand(shape, generator=gen) - 0.5)
        elif name.endswith(".lam"):
            t = (-4.0 + torch.rand(shape, generator=gen)) if slow_decay else torch.randn(shape, generator=gen)
        elif name.endswith("correction"):
            t = 0.05 * torch.randn(shape, generator=gen)
        elif name.endswith(".b") or name == "loop.step":
            t = 0.3 * torch.randn(shape, generator=gen)
        elif name.endswith("router"):
            t = 6.0 * torch.randn(shape, generator=gen) / shape[-1] ** 0.5
        elif name.endswith("conv"):
            t = torch.randn(shape, generator=gen) / shape[-1] ** 0.5
        elif name in ("embed",):
            t = torch.randn(shape, generator=gen)
        else:
            t = torch.randn(shape, generator=gen) / shape[-1] ** 0.5
        w[name] = t.to(torch.bfloat16)
    return w


def write_model(path, cfg, weights):
    from zinfer_b200.weights import write_safetensors

    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(path, "model.safetensors"), {k: v.contiguous() for k, v in weights.items()})
    return path


def f64(weights):
    return {k: v.to(torch.float64) for k, v in weights.items()}


def clear_requests(cfg, w64, lengths, seed, margin):
    """Requests whose every token's choice of experts is clear by ``margin`` in the plain model (the
    score of the last chosen over the first left out), built token by token from random candidates: a
    choice that bfloat16 cannot tell apart would be no fault of the engine's."""
    rng = random.Random(seed)
    has_moe = any(lay["mlp"] and lay["mlp"]["kind"] == "moe" for lay in cfg["layers"])
    reqs = {}
    for r, n in enumerate(lengths):
        toks = []
        while len(toks) < n:
            for _ in range(200):
                cand = rng.randrange(cfg["vocab"])
                if not has_moe:
                    break
                margins = []
                P.forward(cfg, w64, toks + [cand], margins=margins, last_only_margins=True)
                if min(margins) >= margin:
                    break
            else:
                raise AssertionError("no candidate token with a clear choice of experts")
            toks.append(cand)
        reqs[f"r{r}"] = toks
    return reqs
