"""State-space mixer with a scalar decay per head (the "state-space duality" form) and a short causal
convolution in front of it.

Per row h_t, with ``heads`` heads of size P, state size N, ``groups`` groups of B/C, inner = heads * P:
    [z | x | B | C | dt] = W_in h_t                  (inner, inner, groups*N, groups*N, heads)
    [x | B | C] <- silu(conv([x | B | C]))           per channel, ``taps`` taps, the last one the current token's
    dt <- softplus(dt + dt_bias)                     no clamp
    S_t = exp(-exp(A_log_h) dt) S_{t-1} + dt B_t x_t^T        per head, S is N x P, fp32, zero at the sequence's start
    y_t = S_t^T C_t + D_h x_t
    g = y * silu(z);   out = W_o (norm_parts(g) * w)          RMS norm over ``norm_groups`` equal parts of the row
Head h reads the B and C of group ``h // (heads / groups)``.

A request's state is one fp32 vector per slot, ``[S: heads*Npad*P | last taps-1 conv inputs: (taps-1) * channels]``
(Npad: N rounded up to what the scan kernel's threads hold);
the kernels start a portion from it and leave the next portion's behind (``csrc/ssm.cu``), so prompts can be cut
anywhere and decoding is the same path with one row. Step size, decay, state, the gate and the norm are fp32 in both
precisions.

Tensor names below the part's prefix: in, conv, conv.b, dt_bias, A_log, D, norm, o.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Mixer, StateNeed, register_mixer
from .linear import linear


class StateSpace(Mixer):
    capturable = True

    def __init__(self, params, dtype, device, position=None):
        super().__init__(params, dtype, device, position)
        g = params
        self.hidden = int(g["hidden_size"])
        self.heads = int(g["num_heads"])
        self.P = int(g["head_dim"])
        self.N = int(g["state_size"])
        self.groups = int(g["groups"])
        self.taps = int(g["conv_taps"])
        self.norm_groups = int(g.get("norm_groups", 1))
        self.eps = float(g["eps"])
        self.inner = self.heads * self.P
        self.channels = self.inner + 2 * self.groups * self.N
        if self.heads % self.groups:
            raise ValueError(f"state_space: {self.heads} heads are not a multiple of {self.groups} groups")
        if self.inner % self.norm_groups:
            raise ValueError(f"state_space: inner size {self.inner} does not split into {self.norm_groups} norm groups")
        if not 1 <= self.taps <= 17:
            raise ValueError(f"state_space: {self.taps} convolution taps are not supported (1 to 17)")
        self.conv_off = self.heads * ops.ssm_padded_state(self.N, self.P) * self.P      # the scan's part of the slot
        self.w_in = self.w_o = None
        self.conv_w = self.conv_b = self.dt_bias = self.a_log = self.d_skip = self.norm_w = None

    def weight_shapes(self):
        h = self.heads
        return {"in": (2 * self.inner + 2 * self.groups * self.N + h, self.hidden),
                "conv": (self.channels, self.taps), "conv.b": (self.channels,),
                "dt_bias": (h,), "A_log": (h,), "D": (h,), "norm": (self.inner,),
                "o": (self.hidden, self.inner)}

    def keeps_dtype(self, name):
        return name in ("conv", "conv.b", "dt_bias", "A_log", "D", "norm")

    def norm_like(self, name):
        return name in ("norm", "D")

    def load_weights(self, t):
        self.w_in = t["in"].contiguous()
        self.w_o = t["o"].contiguous()
        f32 = lambda n: t[n].float().contiguous()      # what enters the recurrence is 32-bit in both precisions
        self.conv_w, self.conv_b = f32("conv"), f32("conv.b")
        self.dt_bias, self.a_log, self.d_skip, self.norm_w = f32("dt_bias"), f32("A_log"), f32("D"), f32("norm")

    def state_need(self):
        return StateNeed((self.conv_off + (self.taps - 1) * self.channels,), torch.float32)

    def streams_first(self, rows):
        return self.w_in if self.dtype == torch.bfloat16 and rows <= ops.SKINNY_MAX_ROWS else None

    def kernel_files(self, page_size):
        return ("ssm",) + (("gemm_f32",) if self.dtype == torch.float32 else ("gemm_skinny", "gemm_rows", "gemm_tc05"))

    def forward(self, x, ctx, cache):
        T = x.shape[0]
        inner, C = self.inner, self.channels
        u = ctx.buf("ssm_in", (T, self.w_in.shape[0]), self.dtype)
        linear(x, self.w_in, u, ctx.status)
        state = cache.state
        xbc = ctx.buf("ssm_xbc", (T, C), torch.float32)
        ops.causal_conv(u[:, inner:inner + C], self.conv_w, self.conv_b, state, self.conv_off, xbc, ctx.positions,
                        ctx.row_seq, ctx.q_start, ctx.ctx_len, ctx.slots, ctx.seq_slots, status=ctx.status)
        y = ctx.buf("ssm_y", (T, inner), torch.float32)
        ops.ssm_scan(xbc, u[:, inner + C:], self.dt_bias, self.a_log, self.d_skip, state, y, ctx.q_start, ctx.ctx_len,
                     ctx.slots, ctx.seq_slots, self.heads, self.groups, self.N, self.P)
        g = ctx.buf("ssm_gated", (T, inner), self.dtype)
        ops.gated_part_norm(y, u[:, :inner], self.norm_w, g, self.norm_groups, self.eps)
        out = ctx.buf("delta", (T, self.hidden), self.dtype)
        linear(g, self.w_o, out, ctx.status)
        return out


register_mixer("state_space", StateSpace)
