"""A plain, slow implementation of the Rogosun design in 64-bit arithmetic: the oracle of the tests.

One function per mechanism, written from the design's equations with loops over tokens; it shares
no code with the engine.  Weights come as a dictionary name -> tensor (any floating type; they are
widened to float64), the configuration as the dictionary of config.json.

Notation: ``h`` [T, W] is a sublayer's input (the residual stream itself: this design norms a
sublayer's OUTPUT, x <- x + norm(sublayer(x))).  States are returned so that a caller can run a
sequence in pieces.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64
SINK = 1.0      # the attention's softmax counts this much beside the keys' exponentials (a test sets 0 to show it matters)


def _w(t):
    return t.to(F64)


def rms_norm(x, weight, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * _w(weight)


def silu(z):
    return z * torch.sigmoid(z)


# --------------------------------------------------------------------------- gated linear attention
def gla_mixer(h, p, m, eps, state=None):
    """``p``: the mixer's tensors by short name (q, k, v, g, o, norm, a1, a2, a2.b); ``m``: its sizes.
    State: S [heads, dim, vdim].  Returns (output [T, W], state)."""
    T = h.shape[0]
    H, D, V, tau = m["heads"], m["dim"], m["vdim"], float(m["tau"])
    q = (h @ _w(p["q"]).T).view(T, H, D) * D ** -0.5
    k = (h @ _w(p["k"]).T).view(T, H, D)
    v = (h @ _w(p["v"]).T).view(T, H, V)
    z = (h @ _w(p["a1"]).T) @ _w(p["a2"]).T + _w(p["a2.b"])
    alpha = torch.sigmoid(z).pow(1.0 / tau).view(T, H, D)
    S = torch.zeros(H, D, V, dtype=F64) if state is None else state.clone()
    o = torch.zeros(T, H, V, dtype=F64)
    for t in range(T):
        S = alpha[t].unsqueeze(-1) * S + k[t].unsqueeze(-1) * v[t].unsqueeze(-2)
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms_norm(o, p["norm"], eps).reshape(T, H * V)
    o = o * silu(h @ _w(p["g"]).T)
    return o @ _w(p["o"]).T, S


# ------------------------------------------------------- attention with a sink, values = raw keys
def rotate(x, positions, dims, base, factor):
    """x [T, heads, d]: the first ``dims`` dimensions in pairs (i, i + dims/2)."""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) / factor for i in range(half)], dtype=F64)
    a = positions.to(F64).unsqueeze(-1) * f                       # [T, half]
    c, s = torch.cos(a).unsqueeze(1), torch.sin(a).unsqueeze(1)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def sink_attention(h, p, m, eps, pos0=0, cache=None):
    """``cache``: (keys [n, G, d] normed and rotated, values [n, G, d] = keys as projected) of the tokens before.
    Returns (output, cache)."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    rot = m["rot"]
    q = (h @ _w(p["q"]).T).view(T, H, D)
    k_raw = (h @ _w(p["k"]).T).view(T, G, D)
    pos = torch.arange(pos0, pos0 + T)
    factor = float(rot.get("scaling", {}).get("factor", 1.0)) if rot.get("scaling") else 1.0
    qn = rotate(rms_norm(q, p["q.norm"], eps), pos, rot["dims"], float(rot["base"]), factor)
    kn = rotate(rms_norm(k_raw, p["k.norm"], eps), pos, rot["dims"], float(rot["base"]), factor)
    if cache is not None:
        keys, vals = torch.cat([cache[0], kn]), torch.cat([cache[1], k_raw])
    else:
        keys, vals = kn, k_raw
    out = torch.zeros(T, H, D, dtype=F64)
    for t in range(T):
        n = pos0 + t + 1
        for hd in range(H):
            g = hd // (H // G)
            s = (keys[:n, g] @ qn[t, hd]) * float(m["scale"])
            e = torch.exp(s)
            w = e / (SINK + e.sum())                # the sink: score 0, no value
            out[t, hd] = w @ vals[:n, g]
    return out.reshape(T, H * D) @ _w(p["o"]).T, (keys, vals)


# -------------------------------------------------------------------------------- gated delta rule
def short_conv(x, kernel, tail):
    """x [T, C]; kernel [C, taps] (last column: the current token); tail [taps-1, C]: the inputs before.
    Returns (silu(conv) [T, C], new tail)."""
    taps = kernel.shape[1]
    full = torch.cat([tail, x])                     # [taps-1+T, C]
    kt = _w(kernel)
    y = torch.zeros_like(x)
    for t in range(x.shape[0]):
        y[t] = (full[t:t + taps] * kt.T).sum(0)
    return silu(y), full[full.shape[0] - (taps - 1):]


def delta_mixer(h, p, m, eps, state=None):
    """State: (S [heads, dim, vdim], tails of q, k, v).  Returns (output, state)."""
    T = h.shape[0]
    H, G, D, V, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
    if state is None:
        state = (torch.zeros(H, D, V, dtype=F64), torch.zeros(taps - 1, G * D, dtype=F64),
                 torch.zeros(taps - 1, G * D, dtype=F64), torch.zeros(taps - 1, H * V, dtype=F64))
    S, tq, tk, tv = state
    S = S.clone()
    q, tq = short_conv(h @ _w(p["q"]).T, p["q.conv"], tq)
    k, tk = short_conv(h @ _w(p["k"]).T, p["k.conv"], tk)
    v, tv = short_conv(h @ _w(p["v"]).T, p["v.conv"], tv)
    q, k, v = q.view(T, G, D), k.view(T, G, D), v.view(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ _w(p["b"]).T)                                         # [T, H]
    x = (h @ _w(p["a1"]).T) @ _w(p["a2"]).T + _w(p["dt_bias"])
    g = torch.exp(-torch.exp(_w(p["A_log"])).view(1, H, 1) * torch.nn.functional.softplus(x).view(T, H, D))
    o = torch.zeros(T, H, V, dtype=F64)
    rep = H // G
    for t in range(T):
        for hd in range(H):
            kk, qq = k[t, hd // rep], q[t, hd // rep]
            Sh = g[t, hd].unsqueeze(-1) * S[hd]
            u = beta[t, hd] * (v[t, hd] - Sh.T @ kk)
            Sh = Sh + kk.unsqueeze(-1) * u.unsqueeze(0)
            S[hd] = Sh
            o[t, hd] = Sh.T @ qq
    o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps) * _w(p["norm"])
    gate = torch.sigmoid((h @ _w(p["g1"]).T) @ _w(p["g2"]).T).view(T, H, V)
    return (o * gate).reshape(T, H * V) @ _w(p["o"]).T, (S, tq, tk, tv)


def parallel_mixer(h, p, m, eps, pos0=0, state=None):
    left = {k[5:]: v for k, v in p.items() if k.startswith("left.")}
    right = {k[6:]: v for k, v in p.items() if k.startswith("right.")}
    state = state or (None, None)
    lo, cache = sink_attention(h, left, m["left"], eps, pos0, state[0])
    ro, rs = delta_mixer(h, right, m["right"], eps, state[1])
    return float(m["left_scale"]) * lo + float(m["right_scale"]) * ro, (cache, rs)


# ------------------------------------------------------------------------------------ feed-forward
def dense_ff(h, p):
    return torch.relu(h @ _w(p["up"]).T) ** 2 @ _w(p["down"]).T


def gated_expert(h, p, prefix):
    return (silu(h @ _w(p[prefix + "gate"]).T) * (h @ _w(p[prefix + "up"]).T)) @ _w(p[prefix + "down"]).T


def route(scores, top, groups, keep):
    """scores [E] -> the chosen experts' indices: only experts of the ``keep`` groups whose two largest
    scores sum highest can be chosen."""
    E = scores.numel()
    per = E // groups
    gs = scores.view(groups, per)
    gscore = gs.topk(min(2, per), dim=-1).values.sum(-1)
    best = gscore.topk(keep).indices
    allowed = torch.zeros(groups, dtype=torch.bool)
    allowed[best] = True
    masked = torch.where(allowed.repeat_interleave(per), scores, torch.full_like(scores, -math.inf))
    return masked.topk(top).indices


def moe_ff(h, p, mlp):
    r = mlp["router"]
    E, top = r["experts"], r["top"]
    groups, keep = (r["groups"]["count"], r["groups"]["keep"]) if r.get("groups") else (1, 1)
    s = torch.sigmoid(h @ _w(p["router"]).T)
    out = torch.zeros(h.shape[0], _w(p["e0.down"]).shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for e in route(s[t], top, groups, keep).tolist():
            out[t] += s[t, e] * float(r.get("scale", 1.0)) * gated_expert(h[t:t + 1], p, f"e{e}.")[0]
    if mlp.get("shared"):
        out = out + gated_expert(h, p, "shared.")
    return out


# ------------------------------------------------------------------------------------- whole model
def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


class PlainRogosun:
    """Runs token ids through the model; ``forward`` may be called piece by piece (the states carry on)."""

    def __init__(self, config: dict, tensors: dict):
        self.cfg, self.t = config, tensors
        self.eps = float(config["norm"]["eps"])
        self.states = [None] * len(config["layers"])
        self.pos = 0

    def forward(self, tokens, keep_layers=False):
        cfg, t, eps = self.cfg, self.t, self.eps
        x = _w(t["embed"])[torch.as_tensor(tokens, dtype=torch.long)]
        layers = []
        for i, layer in enumerate(cfg["layers"]):
            p = sub(t, f"l{i}.")
            mix = sub(p, "mix.")
            if layer["type"] == "gla":
                y, self.states[i] = gla_mixer(x, mix, layer["mixer"], eps, self.states[i])
            elif layer["type"] == "parallel":
                y, self.states[i] = parallel_mixer(x, mix, layer["mixer"], eps, self.pos, self.states[i])
            else:
                raise ValueError(layer["type"])
            x = x + rms_norm(y, p["norm1"], eps)
            mlp = layer.get("mlp")
            if mlp is not None:
                f = dense_ff(x, sub(p, "mlp.")) if mlp["kind"] == "dense" else moe_ff(x, sub(p, "mlp."), mlp)
                x = x + rms_norm(f, p["norm2"], eps)
            if keep_layers:
                layers.append(x.clone())
        self.pos += len(tokens)
        logits = rms_norm(x, t["final.norm"], eps) @ _w(t["head"]).T
        return (logits, torch.stack(layers)) if keep_layers else logits
