"""Gated delta rule mixer: linear attention whose state, a matrix per head, forgets by a scalar decay and is corrected
by each token's prediction error, behind short causal convolutions.

Per row x, with H heads of value size dv and G query/key heads of size dk (head h reads q/k head h // (H / G)):
    q = W_q x [G, dk],  k = W_k x [G, dk],  v = W_v x [H, dv]
    q, k, v <- silu(conv(.))                 per channel, ``conv_taps`` taps, the last one the current token's, no bias
    q <- q / sqrt(sum(q^2) + 1e-6) * dk^-1/2;   k <- k / sqrt(sum(k^2) + 1e-6)            per head
    beta = sigmoid(W_b x)_h;   g = exp(-exp(A_log_h) * softplus((W_a x)_h + dt_bias_h))
    S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q                          S is dk x dv, fp32, zero at the start
    o <- norm_w * o * rsqrt(mean(o^2) + eps) * silu(W_g x)_h                               per head, norm_w of size dv shared
    out = W_o concat_h o
A request's state is one fp32 vector per slot: ``[S, head by head in the scan kernel's layout | the
convolution's last taps - 1 inputs]``; kernels start
a portion from it and leave the next portion's behind, so prompts can be cut anywhere and decoding is the same path with
one row. Norms of q and k, beta, the decay, the state, the sums, the read-out's norm and its gate are fp32 in both
precisions; the convolution's result stays fp32 on its way into the recurrence.

Tensor names below the part's prefix: q, k, v, q.conv, k.conv, v.conv, b, a, A_log, dt_bias, g, norm, o.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Mixer, StateNeed, register_mixer
from .linear import linear


class GatedDeltaRule(Mixer):
    capturable = True

    def __init__(self, params, dtype, device, position=None):
        super().__init__(params, dtype, device, position)
        p = params
        self.hidden = int(p["hidden_size"])
        self.H = int(p["num_heads"])
        self.G = int(p["num_kv_heads"])
        self.dk = int(p["head_dim"])
        self.dv = int(p["value_dim"])
        self.taps = int(p["conv_taps"])
        self.eps = float(p["eps"])
        if self.H % self.G:
            raise ValueError(f"gated_delta: {self.H} heads are not a multiple of {self.G} query/key heads")
        if not 1 <= self.taps <= 17:
            raise ValueError(f"gated_delta: {self.taps} convolution taps are not supported (1 to 17)")
        if self.dk > 512:
            raise ValueError("gated_delta: key sizes above 512 are not supported")
        self.nqk, self.nv = self.G * self.dk, self.H * self.dv
        self.channels = 2 * self.nqk + self.nv                     # what the convolution runs over: [q | k | v]
        self.g_off = self.channels
        self.b_off = self.g_off + self.nv
        self.a_off = self.b_off + self.H
        self.proj_rows = -(-(self.a_off + self.H) // 8) * 8
        self.conv_off = self.H * ops.delta_state_floats(self.dk, self.dv)        # the scan's part of the slot
        self.w_in = self.w_o = self.conv_w = self.conv_b = self.a_log = self.dt_bias = self.norm_w = None

    def weight_shapes(self):
        d, t = self.hidden, self.taps
        return {"q": (self.nqk, d), "k": (self.nqk, d), "v": (self.nv, d), "g": (self.nv, d), "b": (self.H, d),
                "a": (self.H, d), "q.conv": (self.nqk, t), "k.conv": (self.nqk, t), "v.conv": (self.nv, t),
                "A_log": (self.H,), "dt_bias": (self.H,), "norm": (self.dv,), "o": (d, self.nv)}

    def keeps_dtype(self, name):
        return name in ("q.conv", "k.conv", "v.conv", "A_log", "dt_bias", "norm")

    def norm_like(self, name):
        return name == "norm"

    def load_weights(self, t):
        parts = [t["q"], t["k"], t["v"], t["g"], t["b"], t["a"]]
        rows = sum(p.shape[0] for p in parts)
        if rows < self.proj_rows:
            parts.append(torch.zeros(self.proj_rows - rows, self.hidden, dtype=parts[0].dtype, device=parts[0].device))
        self.w_in = torch.cat(parts, 0).contiguous()
        self.w_o = t["o"].contiguous()
        f32 = lambda n: t[n].float().contiguous()                    # what enters the recurrence is 32-bit in both precisions
        self.conv_w = torch.cat([f32("q.conv"), f32("k.conv"), f32("v.conv")], 0).contiguous()
        self.conv_b = torch.zeros(self.channels, dtype=torch.float32, device=self.conv_w.device)
        self.a_log, self.dt_bias, self.norm_w = f32("A_log"), f32("dt_bias"), f32("norm")

    def state_need(self):
        return StateNeed((self.conv_off + (self.taps - 1) * self.channels,), torch.float32)

    def streams_first(self, rows):
        return self.w_in if self.dtype == torch.bfloat16 and rows <= ops.SKINNY_MAX_ROWS else None

    def kernel_files(self, page_size):
        return ("ssm", "delta_rule") + (("gemm_f32",) if self.dtype == torch.float32 else ("gemm_skinny", "gemm_rows", "gemm_tc05"))

    def forward(self, x, ctx, cache):
        T = x.shape[0]
        H, G, dk, dv, C = self.H, self.G, self.dk, self.dv, self.channels
        u = ctx.buf("delta_proj", (T, self.proj_rows), self.dtype)
        linear(x, self.w_in, u, ctx.status)
        state = cache.state
        xc = ctx.buf("delta_conv", (T, C), torch.float32)
        ops.causal_conv(u[:, :C], self.conv_w, self.conv_b, state, self.conv_off, xc, ctx.positions, ctx.row_seq,
                        ctx.q_start, ctx.ctx_len, ctx.slots, ctx.seq_slots, status=ctx.status)
        bg = ctx.buf("delta_bg", (T, 2 * H + G), torch.float32)
        ops.delta_prepare(xc, u, self.b_off, self.a_off, self.a_log, self.dt_bias, bg, G, H, dk, dk ** -0.5)
        y = ctx.buf("delta_y", (T, self.nv), torch.float32)
        ops.delta_scan(xc, bg, state, y, ctx.q_start, ctx.ctx_len, ctx.slots, ctx.seq_slots, G, H, dk, dv)
        gated = ctx.buf("delta_gated", (T, self.nv), self.dtype)
        ops.head_norm_gate(y, u[:, self.g_off:self.g_off + self.nv], self.norm_w, gated, H, dv, self.eps)
        out = ctx.buf("delta", (T, self.hidden), self.dtype)
        linear(gated, self.w_o, out, ctx.status)
        return out


register_mixer("gated_delta", GatedDeltaRule)
