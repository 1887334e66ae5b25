"""A plain, slow implementation of the Luvavik design, one function per mechanism, in
64-bit floats on whole sequences.  It is the oracle of the tests: it shares no code with
the engine, has no cache and no batching, and is written from the design's equations.

Notation: ``h`` [S, width] is a mixer's or feed-forward's input, ``w`` a dictionary from
tensor name to a float64 tensor, ``p`` the prefix of the part's tensors (``l3.mix.``).
Linear weights are stored [out, in].
"""
from __future__ import annotations

import json
import math
import os

import torch

F64 = torch.float64


# ------------------------------------------------------------------ small pieces
def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms_unit(x, eps):
    """x divided by its root mean square over the last axis (eps inside the root)."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rmsnorm(x, weight, eps):
    return rms_unit(x, eps) * weight


def rotate_half(x, positions, dims, base):
    """Rotary positions on the first ``dims`` entries of the last axis: entry i is paired with
    entry i + dims/2, the pair (u, v) at position p turns by the angle p * base^(-2i/dims).
    ``x`` is [S, ..., n] with n >= dims; ``positions`` [S]."""
    half = dims // 2
    i = torch.arange(half, dtype=F64)
    freq = base ** (-2.0 * i / dims)
    ang = positions.to(F64)[:, None] * freq[None, :]
    while ang.dim() < x.dim():
        ang = ang.unsqueeze(1)
    c, s = torch.cos(ang), torch.sin(ang)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


# ------------------------------------------------------------------------ mixers
def causal_conv(x, kernel, bias):
    """Per-channel causal convolution: x [S, C], kernel [C, taps] whose last column meets the
    current token, zeros before the start."""
    S, C = x.shape
    taps = kernel.shape[1]
    out = torch.zeros_like(x)
    for t in range(S):
        for j in range(taps):
            src = t - (taps - 1 - j)
            if src >= 0:
                out[t] += kernel[:, j] * x[src]
    return out + bias


def rglru_mixer(h, w, p, mixer):
    """Recurrent block: a gated branch y and a branch u that passes a short convolution and
    the real-gated linear recurrence S_t = a_t S_{t-1} + sqrt(1 - a_t^2) i_t u_t, a_t =
    exp(-8 r_t softplus(lam)); the gates r and i are block-diagonal in the channels."""
    width, blocks = mixer["width"], mixer["blocks"]
    y = gelu_tanh(h @ w[p + "y"].T + w[p + "y.b"])
    u = causal_conv(h @ w[p + "x"].T + w[p + "x.b"], w[p + "conv"], w[p + "conv.b"])
    bw = width // blocks
    ub = u.reshape(-1, blocks, bw)
    r = torch.sigmoid(torch.einsum("sbi,boi->sbo", ub, w[p + "ra"]) + w[p + "ra.b"]).reshape(-1, width)
    i = torch.sigmoid(torch.einsum("sbi,boi->sbo", ub, w[p + "ri"]) + w[p + "ri.b"]).reshape(-1, width)
    log_a = -8.0 * r * torch.nn.functional.softplus(w[p + "lam"])
    a = torch.exp(log_a)
    drive = torch.sqrt(1.0 - a * a) * i * u
    state = torch.zeros(width, dtype=F64)
    out = []
    for t in range(h.shape[0]):
        state = a[t] * state + drive[t]
        out.append(state)
    return (torch.stack(out) * y) @ w[p + "o"].T


def latent_attention_mixer(h, w, p, mixer, eps):
    """Attention whose keys and values are made from a small latent per token: c = norm(first
    kv_rank rows of W_dkv h), a rotated key part shared by all heads (the last rot_dim rows),
    per head k = [W_uk c | rotated part], v = W_uv c; q per head is [dim plain | rot_dim
    rotated]; causal softmax; the heads are gated by sigmoid(W_g h) before W_o."""
    S = h.shape[0]
    H, dim, rd, vd, rank = mixer["heads"], mixer["dim"], mixer["rot_dim"], mixer["vdim"], mixer["kv_rank"]
    rot = mixer["rot"]
    pos = torch.arange(S)
    q = (h @ w[p + "q"].T).reshape(S, H, dim + rd)
    q_plain, q_rot = q[..., :dim], rotate_half(q[..., dim:], pos, rot["dims"], rot["base"])
    dkv = h @ w[p + "dkv"].T
    c = rmsnorm(dkv[:, :rank], w[p + "dkv.norm"], eps)
    k_rot = rotate_half(dkv[:, rank:], pos, rot["dims"], rot["base"])
    k_plain = (c @ w[p + "uk"].T).reshape(S, H, dim)
    v = (c @ w[p + "uv"].T).reshape(S, H, vd)
    score = (torch.einsum("shd,thd->hst", q_plain, k_plain) + torch.einsum("shd,td->hst", q_rot, k_rot)) * mixer["scale"]
    visible = pos[None, :] <= pos[:, None]
    score = score.masked_fill(~visible[None], float("-inf"))
    weight = torch.softmax(score, dim=-1)
    heads = torch.einsum("hst,thd->shd", weight, v).reshape(S, H * vd)
    return (heads * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


# ----------------------------------------------------------------- feed-forwards
def dense_ff(h, w, p):
    return (gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(h, w, p, router):
    """Chosen experts [S, top] and their weights: softmax over all router outputs; the choice
    adds the correction, the weight does not, and the weights are not renormalized."""
    s = torch.softmax(h @ w[p + "router"].T, dim=-1)
    chosen = torch.topk(s + w[p + "correction"], router["top"], dim=-1).indices
    return chosen, torch.gather(s, 1, chosen)


def moe_ff(h, w, p, mlp, margins=None, last_only=False):
    """Mixture of experts: expert e is W_down relu(W_up h)^2; the last ``identity`` router
    outputs stand for experts that return h itself."""
    router = mlp["router"]
    E = router["experts"]
    chosen, weight = route(h, w, p, router)
    if margins is not None:   # how clearly the chosen set beat the best expert left out
        s = torch.softmax(h @ w[p + "router"].T, dim=-1) + w[p + "correction"]
        if router["top"] < s.shape[-1]:
            top = torch.topk(s, router["top"] + 1, dim=-1).values
            gap = top[:, -2] - top[:, -1]
            margins.append((gap[-1] if last_only else gap.min()).item())
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t].tolist(), weight[t]):
            if e >= E:
                out[t] += g * h[t]
            else:
                mid = torch.relu(w[f"{p}e{e}.up"] @ h[t]) ** 2
                out[t] += g * (w[f"{p}e{e}.down"] @ mid)
    return out


# ------------------------------------------------------------------------- model
def layer_runs(cfg):
    """(layer, pass number or None) in the order the layers run: layers start..stop-1 run
    ``times`` times in a row, the rest once."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    runs = [(i, None, False) for i in range(loop["start"])]
    for t in range(loop["times"]):
        for i in range(loop["start"], loop["stop"]):
            runs.append((i, t, i == loop["start"]))
    runs += [(i, None, False) for i in range(loop["stop"], n)]
    return runs


def forward(cfg, w, tokens, residuals=None, margins=None, last_only_margins=False):
    """Logits [S, vocab] of a whole sequence.  ``residuals`` (a list) receives the residual
    stream after every layer run; ``margins`` (a list) how clearly each routed layer run chose
    (over all positions, or the last one only)."""
    eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
    x = w["embed"][torch.as_tensor(tokens)]
    for i, t, first in layer_runs(cfg):
        layer, p = cfg["layers"][i], f"l{i}."
        if first:
            x = x + w["loop.step"][t]
        hin = rmsnorm(x, w[p + "norm1"], eps)
        if layer["type"] == "rglru":
            mixed = rglru_mixer(hin, w, p + "mix.", layer["mixer"])
        elif layer["type"] == "latent_attention":
            mixed = latent_attention_mixer(hin, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(f"unknown mixer {layer['type']!r}")
        x = x + m * mixed
        mlp = layer.get("mlp")
        if mlp is not None:
            hin = rmsnorm(x, w[p + "norm2"], eps)
            ff = dense_ff(hin, w, p + "mlp.") if mlp["kind"] == "dense" else \
                moe_ff(hin, w, p + "mlp.", mlp, margins, last_only_margins)
            x = x + m * ff
        if residuals is not None:
            residuals.append(x.clone())
    return (rmsnorm(x, w["final.norm"], eps) @ w["head"].T) * cfg["logit_scale"]


def greedy(cfg, w, prompt, n_new):
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(torch.argmax(forward(cfg, w, toks)[-1])))
    return toks[len(prompt):]


def load_model(model_dir):
    """(config dictionary, float64 tensors) of a model folder, read with a reader of its own."""
    import struct

    import numpy as np

    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    with open(os.path.join(model_dir, "model.safetensors"), "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        header = json.loads(f.read(n))
        data = f.read()
    w = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        raw = data[a:b]
        if info["dtype"] == "BF16":
            u16 = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            arr = u16.view(np.float32).astype(np.float64)
        elif info["dtype"] == "F32":
            arr = np.frombuffer(raw, dtype="<f4").astype(np.float64)
        elif info["dtype"] == "I32":
            arr = np.frombuffer(raw, dtype="<i4").astype(np.int64)
        else:
            raise ValueError(f"{name}: dtype {info['dtype']}")
        w[name] = torch.from_numpy(arr.copy()).reshape(info["shape"])
    return cfg, w
