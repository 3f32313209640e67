"""What enters the residual stream for every token, where it is more than the token's row of the table."""
from __future__ import annotations

import numpy as np
import torch

from ..cache import StateSpec
from ..csrc import ops
from .base import ParamSpec, Part, register


class SummedEmbedding(Part):
    """Token row + hashed bigram row + sinusoidal position vector (each of the two optional).  The bigram row of a
    token is (previous * mul_prev + token * mul_cur) mod buckets, the sequence's first token reads row ``buckets``.
    The token before a step's first one belongs to the sequence's state: one int32 per slot (token + 1; zero in a
    fresh slot), read and left by the kernel itself, so a step that takes its tokens from the device needs no host.
    Position vector: entry 2i = sin(p f_i), entry 2i + 1 = cos(p f_i), f_i = base^(-2i / width); the frequencies are
    made once in 64-bit and rounded, the angle is a 32-bit product."""

    graph_safe = True

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        self.bigram = self.freq = None

    def param_specs(self):
        b = self.spec.bigram
        return [ParamSpec(b.weight, (b.buckets + 1, self.spec.width), "matrix")] if b is not None else []

    def allocate_with(self, stored, rt, table_dtype):
        """The model calls this from its own ``allocate``: the bigram table is kept in the token table's dtype (the
        kernel reads both with one type)."""
        b = self.spec.bigram
        if b is None:
            return {}
        self.bigram = torch.empty((b.buckets + 1, self.spec.width), dtype=table_dtype, device=rt.device)
        return {b.weight: self.bigram}

    def finalize(self):
        if self.freq is None and self.spec.sinusoid_base is not None and self.rt.device is not None:
            i = np.arange((self.spec.width + 1) // 2, dtype=np.float64)
            f = np.power(float(self.spec.sinusoid_base), -2.0 * i / self.spec.width)
            self.freq = torch.from_numpy(f.astype(np.float32)).to(self.rt.device)

    def state_spec(self):
        return StateSpec((), torch.int32) if self.spec.bigram is not None else None

    def forward(self, table, ctx, x, state, scale: float = 1.0):
        b = self.spec.bigram
        ops.embed_sum(table, self.bigram, self.freq, ctx.tok_ids, ctx.tok_seq, ctx.tok_pos, ctx.seq_start, ctx.seq_slot, state,
                      x, self.rt.status, buckets=b.buckets if b else 0, mul_prev=b.mul_prev if b else 0,
                      mul_cur=b.mul_cur if b else 0, scale=scale)


register("embedding", "summed", SummedEmbedding)
