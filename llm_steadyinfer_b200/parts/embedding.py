"""Embedders: the step's tokens into rows of the fp32 residual stream.

``table``        ``x = scale * table[token]`` (``scale`` 1 unless given): the reference's embedding
                 (src/source/op/kernels/cuda/emb_kernel.cu:3-21) has no scale.
``table_pair``   ``x = table[token] + pair[r]`` with a hashed embedding of the pair (previous token, token):
                 ``r = (previous * mul_prev + token * mul_cur) mod buckets``; the first token of a sequence takes
                 the pair table's extra last row, number ``buckets``. The previous token of a portion's first row is
                 per-request state (one int32 per slot), kept and renewed on the device, so a sequence may be cut
                 anywhere and a token sampled on the device needs no trip to the host.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Embedder, StateNeed, register_embedder


class TableEmbedder(Embedder):
    capturable = True

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.name = params.get("name", "weight")
        self.scale = float(params.get("scale", 1.0))

    def weight_shapes(self):
        return {self.name: (self.vocab, self.hidden)}

    def load_weights(self, tensors):
        self.table = tensors[self.name].contiguous()

    def kernel_files(self, page_size):
        return ("embedding",)

    def forward(self, ctx, out, state):
        ops.embedding_gather(ctx.tokens, self.table, out, status=ctx.status, scale=self.scale)


class TablePairEmbedder(TableEmbedder):
    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.buckets = int(params["buckets"])
        self.mul_prev = int(params["mul_prev"])
        self.mul_cur = int(params["mul_cur"])
        self.pair_name = params.get("pair_name", "pair")
        if self.scale != 1.0:
            raise ValueError("table_pair: a scale on the embedding is not supported")
        if self.buckets <= 0 or self.mul_prev < 0 or self.mul_cur < 0:
            raise ValueError("table_pair: buckets must be positive and the multipliers not negative")
        self.pair = None

    def weight_shapes(self):
        return {self.name: (self.vocab, self.hidden), self.pair_name: (self.buckets + 1, self.hidden)}

    def load_weights(self, tensors):
        super().load_weights(tensors)
        self.pair = tensors[self.pair_name].contiguous()

    def state_need(self):
        return StateNeed((1,), torch.int32)            # the request's latest token

    def forward(self, ctx, out, state):
        ops.embedding_pair(ctx.tokens, ctx.positions, ctx.row_seq, ctx.q_start, ctx.slots, state.view(-1), self.table,
                           self.pair, out, self.buckets, self.mul_prev, self.mul_cur, ctx.seq_slots, status=ctx.status)


register_embedder("table", TableEmbedder)
register_embedder("table_pair", TablePairEmbedder)
