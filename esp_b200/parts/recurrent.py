"""Mixers with a recurrent state of fixed size per sequence: two forms of the gated outer-product recurrence
S_t = diag(d_t) S_(t-1) + k_t v_t^T per head.  A head's matrix S is float32 and belongs to the sequence: it sits in
the cache's per-slot state rows, is zeroed when the slot is opened, and every step continues from what the step before
left there, whatever run of tokens it brings.  Both run on ``ops.gated_scan``, which makes the gates from the projections' raw outputs."""
from __future__ import annotations

import numpy as np
import torch

from ..cache import StateSpec
from ..csrc import ops
from ..errors import Unsupported
from .base import ParamSpec, Part, register
from .linear import SKINNY_ROWS, linear


# Steps with more rows than this per sequence make the gates in a parallel pass ahead of the recurrence; shorter
# ones (decoding) let the recurrence make them as it stages its rows.  Both give the same bits.
GATES_AHEAD_ROWS = 8


def _check_dims(kind, key_dim):
    if key_dim > ops.SCAN_MAX_KEY_DIM:
        raise Unsupported(kind + ".dim", f"{key_dim}; the recurrence kernel takes up to {ops.SCAN_MAX_KEY_DIM} key "
                                         f"channels per head")


class LowerBoundRecurrence(Part):
    """q = silu(W_q h), v = W_v h, f = lower + (1 - lower) sigmoid(W_f h + b_f) per head and key channel;
    S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T; o_t = S_t^T q_t; every head's o RMS-normed over its value channels
    with one weight vector for all heads; then W_o.  The three projections are one packed product."""

    graph_safe = True

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        _check_dims(spec.kind, spec.key_dim)
        self.kw = spec.num_heads * spec.key_dim
        self.vw = spec.num_heads * spec.value_dim
        self.w_qfv = self.w_o = self.f_bias = self.lower = self.norm_w = None

    def _n(self, which):
        return self.spec.prefix + getattr(self.spec.names, which)

    def param_specs(self):
        s = self.spec
        return [ParamSpec(self._n("q"), (self.kw, s.hidden), "matrix"),
                ParamSpec(self._n("forget"), (self.kw, s.hidden), "matrix"),
                ParamSpec(self._n("forget") + ".b", (self.kw,), "bias"),
                ParamSpec(self._n("lower"), (self.kw,), "gate_floor", init=(0.3, 0.1)),
                ParamSpec(self._n("v"), (self.vw, s.hidden), "matrix"),
                ParamSpec(self._n("norm"), (s.value_dim,), "norm_scale"),
                ParamSpec(self._n("o"), (s.hidden, self.vw), "matrix")]

    def allocate(self, stored, rt):
        s, dev = self.spec, rt.device
        names = [self._n("q"), self._n("forget"), self._n("v")]
        self.w_qfv = torch.empty((2 * self.kw + self.vw, s.hidden), dtype=rt.matrix_dtype([stored[n] for n in names]), device=dev)
        self.w_o = torch.empty((s.hidden, self.vw), dtype=rt.matrix_dtype([stored[self._n("o")]]), device=dev)
        self.f_bias = torch.empty(self.kw, dtype=torch.float32, device=dev)
        self.lower = torch.empty(self.kw, dtype=torch.float32, device=dev)
        self.norm_w = torch.empty(s.value_dim, dtype=torch.float32, device=dev)
        return {names[0]: self.w_qfv[:self.kw], names[1]: self.w_qfv[self.kw:2 * self.kw], names[2]: self.w_qfv[2 * self.kw:],
                self._n("o"): self.w_o, self._n("forget") + ".b": self.f_bias, self._n("lower"): self.lower,
                self._n("norm"): self.norm_w}

    def kv_layout(self):
        return None

    def state_spec(self):
        return StateSpec((self.spec.num_heads * self.spec.value_dim * self.spec.key_dim,), torch.float32)

    def forward(self, h, ctx, layer):
        s, rt = self.spec, self.rt
        n = h.shape[0]
        proj = rt.ws.get("rec_proj", (n, 2 * self.kw + self.vw), torch.float32)
        linear(rt, h, self.w_qfv, proj)
        o = rt.ws.get("rec_out", (n, self.vw), torch.float32)
        q, f, v = proj[:, :self.kw], proj[:, self.kw:2 * self.kw], proj[:, 2 * self.kw:]
        if n > GATES_AHEAD_ROWS * ctx.n_seqs:
            gates = rt.ws.get("rec_gates", (3, n, self.kw), torch.float32)
            ops.gate_prepare(ops.SCAN_LOWER_SIGMOID, q, f, self.f_bias, self.lower, gates[0], gates[1], gates[2])
            ops.gated_scan(ops.SCAN_LOWER_SIGMOID, gates[0], gates[1], gates[2], v, None, None, None, layer.state,
                           ctx.seq_start, ctx.seq_slot, o, ctx.n_seqs, s.num_heads, s.key_dim, s.value_dim, ready=True)
        else:
            ops.gated_scan(ops.SCAN_LOWER_SIGMOID, q, None, f, v, self.f_bias, self.lower, None, layer.state, ctx.seq_start,
                           ctx.seq_slot, o, ctx.n_seqs, s.num_heads, s.key_dim, s.value_dim)
        y = rt.ws.get("rec_normed", (n, self.vw), rt.dtype)
        ops.head_rmsnorm_gate(o, self.norm_w, 0, None, y, s.num_heads, s.value_dim, s.eps)
        out = rt.ws.get("mixer_out", (n, s.hidden), torch.float32)
        linear(rt, y, self.w_o, out)
        return out


SHIFTS = ("r", "k", "v", "g", "w")


class DecayBonusRecurrence(Part):
    """Each of r, k, v, g, w reads its own mix h + (h' - h) mu of a row and the row before it (h' is part of the
    state); r, k, v are projections of their mixes, gate = silu(W_g mix_g), the decay per head and key channel
    w = exp(-exp(W_w2 tanh(W_w1 mix_w) + w0)); o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t, then
    S_t = diag(w_t) S_(t-1) + k_t v_t^T; every head's o is scaled to unit root mean square, multiplied by a
    weight per channel and by the gate; then W_o."""

    graph_safe = True

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        _check_dims(spec.kind, spec.head_dim)
        self.kw = spec.num_heads * spec.head_dim
        self.state_words = spec.num_heads * spec.head_dim * spec.head_dim
        self.mu = self.w = self.w1 = self.w2 = self.w0 = self.u = self.norm_w = self.w_o = None

    def _n(self, which):
        return self.spec.prefix + getattr(self.spec.names, which)

    def param_specs(self):
        s, nm = self.spec, self.spec.names
        specs = [ParamSpec(self._n("shift") + t, (s.hidden,), "shift_mix", init=(0.5, 0.2)) for t in SHIFTS]
        specs += [ParamSpec(self._n(t), (self.kw, s.hidden), "matrix") for t in ("receptance", "k", "v", "gate")]
        specs += [ParamSpec(self._n("decay_in"), (s.decay_rank, s.hidden), "matrix"),
                  ParamSpec(self._n("decay_out"), (self.kw, s.decay_rank), "matrix"),
                  ParamSpec(self._n("decay_bias"), (self.kw,), "decay_bias", init=(-1.0, 0.7)),
                  ParamSpec(self._n("bonus"), (s.num_heads, s.head_dim), "bonus", init=(0.3, 0.3)),
                  ParamSpec(self._n("norm"), (self.kw,), "norm_scale"),
                  ParamSpec(self._n("o"), (s.hidden, self.kw), "matrix")]
        return specs

    def allocate(self, stored, rt):
        s, dev = self.spec, rt.device
        f32 = lambda *shape: torch.empty(shape, dtype=torch.float32, device=dev)
        self.mu = f32(len(SHIFTS), s.hidden)
        proj = [self._n(t) for t in ("receptance", "k", "v", "gate")]
        self.w = torch.empty((4, self.kw, s.hidden), dtype=rt.matrix_dtype([stored[n] for n in proj]), device=dev)
        self.w1 = torch.empty((s.decay_rank, s.hidden), dtype=rt.matrix_dtype([stored[self._n("decay_in")]]), device=dev)
        self.w2 = torch.empty((self.kw, s.decay_rank), dtype=rt.matrix_dtype([stored[self._n("decay_out")]]), device=dev)
        self.w_o = torch.empty((s.hidden, self.kw), dtype=rt.matrix_dtype([stored[self._n("o")]]), device=dev)
        self.w0, self.u, self.norm_w = f32(self.kw), f32(s.num_heads, s.head_dim), f32(self.kw)
        views = {self._n("shift") + t: self.mu[i] for i, t in enumerate(SHIFTS)}
        views.update({n: self.w[i] for i, n in enumerate(proj)})
        views.update({self._n("decay_in"): self.w1, self._n("decay_out"): self.w2, self._n("decay_bias"): self.w0,
                      self._n("bonus"): self.u, self._n("norm"): self.norm_w, self._n("o"): self.w_o})
        return views

    def kv_layout(self):
        return None

    # the four projections of a short step are one grouped weight-streaming product: rows [mix, token], one group a mix
    def step_arrays_key(self):
        return ("token_shift_groups",)

    def step_arrays(self, step):
        return {"token_shift.group_offsets4": np.arange(5, dtype=np.int32) * step.n_tokens}

    def state_spec(self):
        # the heads' matrices, then the row before the sequence's next token
        return StateSpec((self.state_words + self.spec.hidden,), torch.float32)

    def forward(self, h, ctx, layer):
        s, rt = self.spec, self.rt
        n = h.shape[0]
        prev = layer.state[:, self.state_words:]
        mixed = rt.ws.get("wkv_mixed", (len(SHIFTS), n, s.hidden), rt.dtype)
        ops.token_shift_mix(h, prev, ctx.tok_seq, ctx.seq_start, ctx.seq_slot, self.mu, mixed)
        ops.token_shift_keep(h, prev, ctx.seq_start, ctx.seq_slot, ctx.n_seqs)
        proj = rt.ws.get("wkv_proj", (5, n, self.kw), torch.float32)      # r, k, v, gate, raw decay
        offsets = ctx.arrays.get("token_shift.group_offsets4")
        if (offsets is not None and n <= SKINNY_ROWS and mixed.dtype == torch.bfloat16 and self.w.dtype == torch.bfloat16
                and ops.skinny_fits(s.hidden)):
            ops.gemm_skinny(mixed.view(len(SHIFTS) * n, s.hidden), self.w, proj.view(5 * n, self.kw), group_offsets=offsets,
                            rows=4 * n, max_rows=n)
        else:
            for i in range(4):
                linear(rt, mixed[i], self.w[i], proj[i])
        inner = rt.ws.get("wkv_decay_inner", (n, s.decay_rank), torch.float32)
        linear(rt, mixed[4], self.w1, inner)
        inner_act = rt.ws.get("wkv_decay_act", (n, s.decay_rank), rt.dtype)
        ops.tanh(inner, inner_act)
        linear(rt, inner_act, self.w2, proj[4])
        o = rt.ws.get("rec_out", (n, self.kw), torch.float32)
        decay, ready = proj[4], False
        if n > GATES_AHEAD_ROWS * ctx.n_seqs:
            decay, ready = rt.ws.get("rec_gates", (1, n, self.kw), torch.float32)[0], True
            ops.gate_prepare(ops.SCAN_DECAY_BONUS, None, proj[4], self.w0, None, None, None, decay)
        ops.gated_scan(ops.SCAN_DECAY_BONUS, proj[0], proj[1], decay, proj[2], None if ready else self.w0, None, self.u.view(-1),
                       layer.state, ctx.seq_start, ctx.seq_slot, o, ctx.n_seqs, s.num_heads, s.head_dim, s.head_dim, ready=ready)
        y = rt.ws.get("rec_normed", (n, self.kw), rt.dtype)
        ops.head_rmsnorm_gate(o, self.norm_w, s.head_dim, proj[3], y, s.num_heads, s.head_dim, s.eps)
        out = rt.ws.get("mixer_out", (n, s.hidden), torch.float32)
        linear(rt, y, self.w_o, out)
        return out


register("mixer", "hgrn2", LowerBoundRecurrence)
register("mixer", "wkv", DecayBonusRecurrence)
