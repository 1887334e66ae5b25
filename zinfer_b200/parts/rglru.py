"""Recurrent block with a real-gated linear recurrent unit (the recurrent block of
"Griffin: Mixing Gated Linear Recurrences with Local Attention for Efficient Language Models",
De et al., 2024).

Two branches of ``width`` channels from the input h:  y = gelu_tanh(W_y h + b_y)  and
u = conv(W_x h + b_x), a causal convolution per channel over the last ``taps`` tokens.  The
channels are cut into ``blocks`` equal parts; in part b the gates are
r = sigmoid(A_b u_b + a_b) and i = sigmoid(I_b u_b + i_b).  With
a = exp(-decay_scale * r * softplus(lam)) the state follows
S_t = a_t S_(t-1) + sqrt(1 - a_t^2) * i_t * u_t  from S = 0, and the output is W_o (S * y).

Per request the mixer keeps S and the convolution's last taps-1 inputs in one state slot
(float32 [taps, width]: the inputs oldest first, then S), so a request may be cut into steps
anywhere.  The convolution's output, the gates, the decay and the state are 32-bit; the two
branch products and the output product run in the model's dtype.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import Mixer, StateNeed, TensorSpec


class RGLRUMixer(Mixer):
    graph_safe = True   # kernels on the step's device arrays only

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden = int(params["hidden_size"])
        self.width = int(params["width"])
        self.blocks = int(params["blocks"])
        self.taps = int(params["conv_taps"])
        self.decay_scale = float(params.get("decay_scale", 8.0))
        if self.blocks <= 0 or self.width % self.blocks:
            raise ValueError(f"{self.width} channels do not divide into {self.blocks} blocks")
        if not 1 <= self.taps <= 9:
            raise ValueError(f"the convolution has 1 to 9 taps, got {self.taps}")
        self.bw = self.width // self.blocks

    def tensor_specs(self):
        W, B, bw = self.width, self.blocks, self.bw
        return {
            "y": TensorSpec((W, self.hidden)), "y.b": TensorSpec((W,), init="zeros"),
            "x": TensorSpec((W, self.hidden)), "x.b": TensorSpec((W,), init="zeros"),
            "conv": TensorSpec((W, self.taps)), "conv.b": TensorSpec((W,), init="zeros"),
            "ra": TensorSpec((B, bw, bw)), "ra.b": TensorSpec((B, bw), init="zeros"),
            "ri": TensorSpec((B, bw, bw)), "ri.b": TensorSpec((B, bw), init="zeros"),
            "lam": TensorSpec((W,), init="norm"),
            "o": TensorSpec((self.hidden, W)),
        }

    def bind(self, tensors):
        f32 = lambda name: tensors[name].to(torch.float32).contiguous()
        wy, wx = tensors["y"], tensors["x"]
        if wy.dtype != wx.dtype:
            wy, wx = wy.to(torch.float32), wx.to(torch.float32)
        self.w_yx = torch.cat([wy, wx], dim=0).contiguous()            # one product feeds both branches
        self.y_bias, self.x_bias = f32("y.b"), f32("x.b")
        self.conv, self.conv_bias = f32("conv"), f32("conv.b")
        # per block the recurrence gate's matrix above the input gate's: [blocks, 2 bw, bw]
        ra, ri = tensors["ra"], tensors["ri"]
        if ra.dtype != ri.dtype:
            ra, ri = ra.to(torch.float32), ri.to(torch.float32)
        self.w_gates = torch.cat([ra, ri], dim=1).contiguous()
        self.r_bias, self.i_bias = f32("ra.b").reshape(-1), f32("ri.b").reshape(-1)
        self.lam = f32("lam")
        self.w_o = tensors["o"].contiguous()

    def cache_need(self):
        return StateNeed((self.taps, self.width), torch.float32)

    def forward(self, x, step, cache):
        T, W, B, bw = x.shape[0], self.width, self.blocks, self.bw
        yx = ops.linear(x, self.w_yx, out_dtype=self.ctx.dtype)         # [T, 2W]: y branch, then x branch
        if step.all_decode and step.n_seqs == T:
            # one token per request: convolution, gates and recurrence are one kernel
            mixed = ops.rglru_decode(yx, self.y_bias, self.x_bias, self.conv, self.conv_bias, self.w_gates, self.r_bias,
                                     self.i_bias, self.lam, self.decay_scale, cache.state, step)
            return ops.linear(mixed, self.w_o, out_dtype=self.ctx.dtype, allow_partials=True)
        y, xb = yx[:, :W], yx[:, W:]
        u = ops.causal_conv(xb, self.x_bias, self.conv, self.conv_bias, cache.state, step)     # float32 [T, W]
        gates = torch.empty((T, B, 2 * bw), dtype=torch.float32, device=x.device)
        ops.linear_batched(u.view(T, B, bw).transpose(0, 1), self.w_gates, gates.transpose(0, 1))
        mixed = ops.rglru_scan(u, gates, bw, self.r_bias, self.i_bias, self.lam, self.decay_scale, y, self.y_bias,
                               xb, self.x_bias, cache.state, step)
        return ops.linear(mixed, self.w_o, out_dtype=self.ctx.dtype, allow_partials=True)
