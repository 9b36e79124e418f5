"""Differential attention mixer: every head runs two softmax attentions ("maps") with queries and keys of their own
over the same values and takes their difference.

Per row x, with H heads, G key/value heads (head h reads key/value head h // (H / G)), key size dk, value size dv:
    q = W_q x  [H, 2, dk],  k = W_k x  [G, 2, dk],  v = W_v x  [G, dv]          laid out head by head as [map 1, map 2]
    q, k <- rms_norm(q or k, shared weight of size dk), then the first ``rot_dims`` entries rotated by position
            (neighbouring pairs (2i, 2i + 1) when ``rot_interleaved``, else (i, i + rot_dims / 2))
    s_m = softcap * tanh(scale * q_m . k_m / softcap)   over the keys j with 0 <= i - j < window  (softcap 0: none)
    a_m = softmax(s_m) v                                 m = 1, 2
    lam = exp(lq1 . lk1) - exp(lq2 . lk2) + diff         one number for the layer
    o   = rms_norm(a_1 - lam a_2) (1 - diff)             over the head's dv values, no weight
    o  <- o sigmoid(W_g x)_h                             one gate per head (``gate``: True)
    out = W_o concat_h o
The cache keeps 2 G key heads of dk and G value heads of dv per token (``CacheNeed.num_value_heads``): both maps of a
head read one value head. Scores, softmax, the difference, the norm and the gate are fp32 in both precisions; the
maps' results stay fp32 until they are combined.

Tensor names below the part's prefix (``names`` overrides): q, k, v, g, o, q.norm, k.norm, lq1, lk1, lq2, lk2.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import CacheNeed, Mixer, register_mixer
from . import flex_plan
from .linear import linear

MAPS = 2
USE_TENSOR_CORES = True      # bf16 only; False sends bf16 through the plain kernel as well


class DiffAttention(Mixer):
    capturable = True

    def __init__(self, params, dtype, device, position=None):
        super().__init__(params, dtype, device, position)
        p = params
        self.hidden = int(p["hidden_size"])
        self.H = int(p["num_heads"])
        self.G = int(p["num_kv_heads"])
        self.dk = int(p["head_dim"])
        self.dv = int(p.get("value_dim") or self.dk)
        self.scale = float(p["scale"])
        self.softcap = float(p.get("softcap") or 0.0)
        self.window = p.get("window") or None
        self.diff = float(p["diff"])
        self.eps = float(p["eps"])
        self.gate = bool(p.get("gate", True))
        self.rot_interleaved = bool(p.get("rot_interleaved", True))
        if self.H % self.G:
            raise ValueError(f"diff_attention: {self.H} heads are not a multiple of {self.G} kv heads")
        if self.dk > 640 or self.dv > 640:
            raise ValueError("diff_attention: key and value sizes above 640 are not supported")
        rot = position.rotary() if position is not None else None
        if position is not None and rot is None:
            raise ValueError("diff_attention: the position encoding must give rotary frequencies")
        self.inv_freq, self.rot_dims = rot if rot is not None else (None, 0)
        self.names = {n: n for n in ("q", "k", "v", "g", "o", "q.norm", "k.norm", "lq1", "lk1", "lq2", "lk2")}
        self.names.update(p.get("names") or {})
        self.nq, self.nk = self.H * MAPS * self.dk, self.G * MAPS * self.dk
        self.gate_off = self.nq + self.nk + self.G * self.dv
        self.proj_rows = -(-(self.gate_off + (self.H if self.gate else 0)) // 8) * 8      # rows of 16-byte multiples
        self.w_in = self.w_o = self.q_norm = self.k_norm = None
        self.lam = 0.0

    def weight_shapes(self):
        n = self.names
        s = {n["q"]: (self.nq, self.hidden), n["k"]: (self.nk, self.hidden), n["v"]: (self.G * self.dv, self.hidden),
             n["o"]: (self.hidden, self.H * self.dv), n["q.norm"]: (self.dk,), n["k.norm"]: (self.dk,),
             n["lq1"]: (self.dk,), n["lk1"]: (self.dk,), n["lq2"]: (self.dk,), n["lk2"]: (self.dk,)}
        if self.gate:
            s[n["g"]] = (self.H, self.hidden)
        return s

    def keeps_dtype(self, name):
        n = self.names
        return name in (n["q.norm"], n["k.norm"], n["lq1"], n["lk1"], n["lq2"], n["lk2"])

    def norm_like(self, name):
        return name in (self.names["q.norm"], self.names["k.norm"])

    def load_weights(self, t):
        n = self.names
        parts = [t[n["q"]], t[n["k"]], t[n["v"]]] + ([t[n["g"]]] if self.gate else [])
        rows = sum(p.shape[0] for p in parts)
        if rows < self.proj_rows:
            parts.append(torch.zeros(self.proj_rows - rows, self.hidden, dtype=parts[0].dtype, device=parts[0].device))
        self.w_in = torch.cat(parts, 0).contiguous()
        self.w_o = t[n["o"]].contiguous()
        self.q_norm = t[n["q.norm"]].float().contiguous()
        self.k_norm = t[n["k.norm"]].float().contiguous()
        f = lambda a, b: torch.exp((t[n[a]].float() * t[n[b]].float()).sum())
        self.lam = float((f("lq1", "lk1") - f("lq2", "lk2")).item()) + self.diff

    def cache_need(self):
        return CacheNeed(self.G * MAPS, self.dk, self.window, self.dv, self.G)

    def streams_first(self, rows):
        return self.w_in if self.dtype == torch.bfloat16 and rows <= ops.SKINNY_MAX_ROWS else None

    def kernel_files(self, page_size):
        if self.dtype == torch.float32:
            return ("qk_prepare", "attention_general", "gemm_f32")
        return ("qk_prepare", "attention_flex" if self.uses_flex() else "attention_general", "gemm_skinny", "gemm_rows", "gemm_tc05")

    def uses_flex(self) -> bool:
        """The maps on the tensor cores: bfloat16 and sizes in multiples of 8."""
        return (self.dtype == torch.bfloat16 and USE_TENSOR_CORES
                and ops.attn_flex_ok(self.H * MAPS, self.G * MAPS, self.dk, self.dv, True))

    def prepare(self, ctx, cache):
        if self.uses_flex() and cache.k is not None:
            flex_plan.plan(ctx, self.device, self.H * MAPS, self.G * MAPS, self.dk, self.dv, True, self.window)

    def forward(self, x, ctx, cache):
        T = x.shape[0]
        H, G, dk, dv = self.H, self.G, self.dk, self.dv
        u = ctx.buf("dattn_proj", (T, self.proj_rows), self.dtype)
        linear(x, self.w_in, u, ctx.status)
        writes = cache.writes
        # queries in the order [key head][map][head of the group]: map m of a head then reads key head (g, m) as
        # query head i of any grouped attention reads key head i // (heads a key head)
        q = ctx.buf("dattn_q", (T, self.nq), self.dtype)
        ops.qk_prepare(u, self.q_norm, self.k_norm, self.eps, self.inv_freq, self.rot_dims, self.rot_interleaved,
                       ctx.positions, ctx.row_seq, cache.block_table, cache.k if writes else None,
                       cache.v if writes else None, cache.page_size, ctx.seq_slots, H * MAPS, G * MAPS, G, dk, dv,
                       status=ctx.status, q_out=q, maps=MAPS)
        maps = ctx.buf("dattn_maps", (T, H * MAPS * dv), torch.float32)
        self.attend(q, cache, ctx, maps)
        o = ctx.buf("attn_out", (T, H * dv), self.dtype)
        gate = u[:, self.gate_off:self.gate_off + H] if self.gate else None
        ops.diff_combine(maps, gate, o, H, dv, H // G, self.lam, self.eps, 1.0 - self.diff)
        out = ctx.buf("delta", (T, self.hidden), self.dtype)
        linear(o, self.w_o, out, ctx.status)
        return out

    def attend(self, q, cache, ctx, maps):
        """Both maps of every head as 2 H query heads over 2 G key heads; neighbouring key heads share a value head."""
        if self.uses_flex():
            H, G = self.H * MAPS, self.G * MAPS
            flex_plan.attend(flex_plan.plan(ctx, self.device, H, G, self.dk, self.dv, True, self.window), q, cache.k, cache.v,
                             cache.block_table, maps, cache.page_size, ctx.seq_slots, H, G, self.dk, self.dv, self.scale,
                             self.window, status=ctx.status, softcap=self.softcap, v_share=MAPS)
            return
        ops.attention_general(q, cache.k, cache.v, cache.block_table, ctx.row_seq, ctx.positions, maps, cache.page_size,
                              ctx.seq_slots, self.H * MAPS, self.G * MAPS, self.dk, self.dv, self.scale, self.window or 0,
                              status=ctx.status, softcap=self.softcap, v_share=MAPS)


register_mixer("diff_attention", DiffAttention)
