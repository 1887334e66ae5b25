"""Mixers that keep a matrix-valued state per head instead of keys: linear attention with a decay per key
channel, in two forms.

Both carry, per request and head, S [dim key channels, vdim value channels] in 32-bit and update it token by token:

    S <- diag(g_t) S ;  u_t = v_t  or  beta_t (v_t - S^T k_t) ;  S <- S + k_t u_t^T ;  o_t = S^T q_t

(the read-out sees the current token's write).  Each head's o is divided by its root mean square over vdim
(eps inside the root), multiplied by a weight [vdim] shared by the heads and by a gate, and projected by W_o.

:class:`GatedLinearAttention` (the plain form; "Gated Linear Attention Transformers with Hardware-Efficient
Training", Yang et al., 2023, is the family): q = W_q h * dim^(-1/2), k = W_k h, v = W_v h,
g = sigmoid(W_a2 (W_a1 h) + b)^(1/tau), gate silu(W_g h).

:class:`GatedDeltaRule` (the delta-rule form; "Gated Delta Networks: Improving Mamba2 with Delta Rule",
Yang et al., 2024, is the family): q, k (``kv_heads`` heads, shared by groups of value heads) and v each pass a short
causal convolution per channel and silu; q and k are made unit vectors per head (x / sqrt(sum x^2 + 1e-6)), q also
times dim^(-1/2); beta = sigmoid(W_b h); g = exp(-exp(A_log_h) * softplus(W_a2 (W_a1 h) + dt_bias)) per head and key
channel; gate sigmoid(W_g2 (W_g1 h)).  The convolutions' last taps-1 inputs are state too.

Decays, beta, unit norms, the recurrence, the state and the head norm are 32-bit; the projections run in the
model's dtype.  The ranks of the low-rank pairs (a1/a2, g1/g2) are read from the tensors.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import Mixer, StateNeed, TensorSpec


def _cat(tensors):
    if len({t.dtype for t in tensors}) > 1:
        tensors = [t.to(torch.float32) for t in tensors]
    return torch.cat(tensors, dim=0).contiguous()


class GatedLinearAttention(Mixer):
    graph_safe = True   # kernels on the step's device arrays only

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden = int(params["hidden_size"])
        self.heads = int(params["num_heads"])
        self.dim = int(params["dim"])
        self.vdim = int(params["vdim"])
        self.tau = float(params["tau"])
        self.eps = float(params["norm_eps"])
        self.rank_hint = int(params.get("decay_rank", 16))
        if not self.tau > 0.0:
            raise ValueError(f"tau must be positive, got {self.tau}")
        if min(self.heads, self.dim, self.vdim) <= 0:
            raise ValueError("heads, dim and vdim must be positive")

    def tensor_specs(self):
        qk, hv, hid = self.heads * self.dim, self.heads * self.vdim, self.hidden
        return {
            "q": TensorSpec((qk, hid)), "k": TensorSpec((qk, hid)), "v": TensorSpec((hv, hid)), "g": TensorSpec((hv, hid)),
            "o": TensorSpec((hid, hv)), "norm": TensorSpec((self.vdim,), init="norm"),
            "a1": TensorSpec((-1, hid), free=self.rank_hint), "a2": TensorSpec((qk, -1), free=self.rank_hint),
            "a2.b": TensorSpec((qk,), init="zeros"),
        }

    def bind(self, tensors):
        if tensors["a1"].shape[0] != tensors["a2"].shape[1]:
            raise ValueError(f"a1 {list(tensors['a1'].shape)} and a2 {list(tensors['a2'].shape)} do not share a rank")
        self.rank = tensors["a1"].shape[0]
        self.w_in = _cat([tensors[n] for n in ("q", "k", "v", "g", "a1")])     # one product feeds all five
        self.w_a2 = tensors["a2"].contiguous()
        self.a_bias = tensors["a2.b"].to(torch.float32).contiguous()
        self.norm = tensors["norm"].to(torch.float32).contiguous()
        self.w_o = tensors["o"].contiguous()

    def cache_need(self):
        return StateNeed((self.heads, self.dim, self.vdim), torch.float32)

    def forward(self, x, step, cache):
        qk, hv = self.heads * self.dim, self.heads * self.vdim
        proj = ops.linear(x, self.w_in, out_dtype=self.ctx.dtype)
        q, k, v, g = proj[:, :qk], proj[:, qk:2 * qk], proj[:, 2 * qk:2 * qk + hv], proj[:, 2 * qk + hv:2 * qk + 2 * hv]
        z = ops.linear(proj[:, 2 * qk + 2 * hv:], self.w_a2, out_dtype=torch.float32)
        decay = ops.decay_sigmoid_root_(z, self.a_bias, self.tau)
        o = ops.linear_recurrence(q, k, v, decay, None, self.dim ** -0.5, cache.state, self.heads, self.heads, self.dim,
                                  self.vdim, step)
        y = ops.head_norm_gate(o, self.norm, self.eps, g, "silu", self.heads, self.vdim, self.ctx.dtype)
        return ops.linear(y, self.w_o, out_dtype=self.ctx.dtype, allow_partials=True)


class GatedDeltaRule(Mixer):
    graph_safe = True
    UNIT_EPS = 1e-6      # inside the root of the unit norms of q and k

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden = int(params["hidden_size"])
        self.heads = int(params["num_heads"])
        self.kv_heads = int(params["num_kv_heads"])
        self.dim = int(params["dim"])
        self.vdim = int(params["vdim"])
        self.taps = int(params["conv_taps"])
        self.eps = float(params["norm_eps"])
        self.decay_rank_hint = int(params.get("decay_rank", 16))
        self.gate_rank_hint = int(params.get("gate_rank", 16))
        if self.kv_heads <= 0 or self.heads % self.kv_heads:
            raise ValueError(f"{self.heads} heads do not divide into {self.kv_heads} query/key heads")
        if not 1 <= self.taps <= 64:
            raise ValueError(f"the convolution has 1 to 64 taps, got {self.taps}")
        self.qk = self.kv_heads * self.dim
        self.hv = self.heads * self.vdim
        self.channels = 2 * self.qk + self.hv            # the convolved channels: q, k, v side by side
        self.s_size = self.heads * self.dim * self.vdim

    def tensor_specs(self):
        hid, hd = self.hidden, self.heads * self.dim
        return {
            "q": TensorSpec((self.qk, hid)), "q.conv": TensorSpec((self.qk, self.taps)),
            "k": TensorSpec((self.qk, hid)), "k.conv": TensorSpec((self.qk, self.taps)),
            "v": TensorSpec((self.hv, hid)), "v.conv": TensorSpec((self.hv, self.taps)),
            "b": TensorSpec((self.heads, hid)), "A_log": TensorSpec((self.heads,), init="zeros"),
            "norm": TensorSpec((self.vdim,), init="norm"),
            "a1": TensorSpec((-1, hid), free=self.decay_rank_hint), "a2": TensorSpec((hd, -1), free=self.decay_rank_hint),
            "dt_bias": TensorSpec((hd,), init="zeros"),
            "g1": TensorSpec((-1, hid), free=self.gate_rank_hint), "g2": TensorSpec((self.hv, -1), free=self.gate_rank_hint),
            "o": TensorSpec((hid, self.hv)),
        }

    def bind(self, tensors):
        for a, b in (("a1", "a2"), ("g1", "g2")):
            if tensors[a].shape[0] != tensors[b].shape[1]:
                raise ValueError(f"{a} {list(tensors[a].shape)} and {b} {list(tensors[b].shape)} do not share a rank")
        self.decay_rank, self.gate_rank = tensors["a1"].shape[0], tensors["g1"].shape[0]
        self.w_in = _cat([tensors[n] for n in ("q", "k", "v", "b", "a1", "g1")])      # one product feeds all six
        f32 = lambda name: tensors[name].to(torch.float32).contiguous()
        self.conv = torch.cat([f32("q.conv"), f32("k.conv"), f32("v.conv")], dim=0).contiguous()   # [channels, taps]
        self.a_log, self.dt_bias, self.norm = f32("A_log"), f32("dt_bias"), f32("norm")
        self.w_a2, self.w_g2 = tensors["a2"].contiguous(), tensors["g2"].contiguous()
        self.w_o = tensors["o"].contiguous()

    def cache_need(self):
        # one slot per request: S of every head, then the convolutions' last taps-1 inputs [taps-1, channels]
        return StateNeed((self.s_size + (self.taps - 1) * self.channels,), torch.float32)

    def forward(self, x, step, cache):
        C, H, qk = self.channels, self.heads, self.qk
        proj = ops.linear(x, self.w_in, out_dtype=self.ctx.dtype)
        state = cache.state
        s_view = state[:, :self.s_size]
        tail = state[:, self.s_size:].view(state.shape[0], self.taps - 1, C)
        raw = proj[:, :C]
        qkv = ops.short_conv(raw, self.conv, tail, step, "silu")                   # float32 [T, C]
        ops.short_conv_carry(raw, self.taps, tail, step)
        q, k, v = qkv[:, :qk], qkv[:, qk:2 * qk], qkv[:, 2 * qk:]
        ops.unit_norm_(q, self.kv_heads, self.dim, self.UNIT_EPS)
        ops.unit_norm_(k, self.kv_heads, self.dim, self.UNIT_EPS)
        beta = ops.sigmoid_rows(proj[:, C:C + H])
        a0 = C + H
        z = ops.linear(proj[:, a0:a0 + self.decay_rank], self.w_a2, out_dtype=torch.float32)
        decay = ops.decay_exp_softplus_(z, self.dt_bias, self.a_log, self.dim)
        o = ops.linear_recurrence(q, k, v, decay, beta, self.dim ** -0.5, s_view, H, self.kv_heads, self.dim, self.vdim, step)
        gate = ops.linear(proj[:, a0 + self.decay_rank:], self.w_g2, out_dtype=self.ctx.dtype)
        y = ops.head_norm_gate(o, self.norm, self.eps, gate, "sigmoid", H, self.vdim, self.ctx.dtype)
        return ops.linear(y, self.w_o, out_dtype=self.ctx.dtype, allow_partials=True)


class ParallelMixer(Mixer):
    """Two mixers side by side on the same input: ``left_scale * left(h) + right_scale * right(h)``.  Each keeps its
    own cache or state (``cache_need`` gives both by name).  ``forward`` hands back the two scaled updates as a pair;
    the block adds them (inside its norm's kernel)."""

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        from .base import make_part
        self.left = make_part(params["left"], ctx)
        self.right = make_part(params["right"], ctx)
        self.left_scale = float(params.get("left_scale", 1.0))
        self.right_scale = float(params.get("right_scale", 1.0))
        self.names = (params.get("left_name", "left."), params.get("right_name", "right."))
        self.graph_safe = bool(getattr(self.left, "graph_safe", False) and getattr(self.right, "graph_safe", False))

    def tensor_specs(self):
        from .base import prefixed
        out = prefixed(self.names[0], self.left.tensor_specs())
        out.update(prefixed(self.names[1], self.right.tensor_specs()))
        return out

    def bind(self, tensors):
        from .base import take
        self.left.bind(take(tensors, self.names[0]))
        self.right.bind(take(tensors, self.names[1]))

    def cache_need(self):
        needs = {"left": self.left.cache_need(), "right": self.right.cache_need()}
        return {k: v for k, v in needs.items() if v is not None}

    def max_positions(self):
        limits = [m.max_positions() for m in (self.left, self.right) if hasattr(m, "max_positions")]
        limits = [v for v in limits if v is not None]
        return min(limits) if limits else None

    def forward(self, x, step, cache):
        left = self.left.forward(x, step, cache.get("left"))
        right = self.right.forward(x, step, cache.get("right"))
        return ops.Scaled(left, self.left_scale), ops.Scaled(right, self.right_scale)
