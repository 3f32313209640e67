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


class MatrixMemory(Part):
    """Matrix memory with exponential gating (see ``MatrixMemorySpec``).  One packed product makes q, k, v, the output
    gate and the two gate scalars per head; a short kernel turns the scalars into the running maximum m, the decay
    exp(f + m' - m) and the input weight exp(i - m) (32-bit, a chain over the tokens); the shared recurrence kernel
    takes the decay as one number per head and token and the input weight as a factor on the values; the normaliser n
    rides along as one more value column whose value is always one.  Per
    slot the state holds S and n as [heads, value columns, key channels] floats and then m per head."""

    graph_safe = True
    FLOOR = 1e-6                 # added to the denominator max(|n . q|, exp(-m))

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        _check_dims(spec.kind, spec.key_dim)
        s = spec
        self.kw, self.vw = s.num_heads * s.key_dim, s.num_heads * s.value_dim
        self.cols = (s.value_dim + 1 + 3) // 4 * 4          # value columns of the recurrence: v, the one, zeros up to a multiple of 4
        self.state_words = s.num_heads * self.cols * s.key_dim
        self.proj_width = 2 * self.kw + 2 * self.vw + 2 * s.num_heads
        self.w_in = self.w_o = self.gate_bias = self.norm_w = None

    def _n(self, which):
        return self.spec.prefix + getattr(self.spec.names, which)

    def param_specs(self):
        s = self.spec
        return [ParamSpec(self._n("q"), (self.kw, s.hidden), "matrix"), ParamSpec(self._n("k"), (self.kw, s.hidden), "matrix"),
                ParamSpec(self._n("v"), (self.vw, s.hidden), "matrix"), ParamSpec(self._n("gate"), (self.vw, s.hidden), "matrix"),
                ParamSpec(self._n("input_gate"), (s.num_heads, s.hidden), "matrix"),
                ParamSpec(self._n("input_gate") + ".b", (s.num_heads,), "bias"),
                ParamSpec(self._n("forget_gate"), (s.num_heads, s.hidden), "matrix"),
                ParamSpec(self._n("forget_gate") + ".b", (s.num_heads,), "forget_bias", init=(2.0, 1.0)),
                ParamSpec(self._n("norm"), (self.vw,), "norm_scale"),
                ParamSpec(self._n("o"), (s.hidden, self.vw), "matrix")]

    def allocate(self, stored, rt):
        s, dev = self.spec, rt.device
        order = ["q", "k", "v", "gate", "input_gate", "forget_gate"]
        names = [self._n(t) for t in order]
        sizes = [self.kw, self.kw, self.vw, self.vw, s.num_heads, s.num_heads]
        self.w_in = torch.empty((self.proj_width, s.hidden), dtype=rt.matrix_dtype([stored[n] for n in names]), device=dev)
        self.w_o = torch.empty((s.hidden, self.vw), dtype=rt.matrix_dtype([stored[self._n("o")]]), device=dev)
        self.gate_bias = torch.empty((2, s.num_heads), dtype=torch.float32, device=dev)
        self.norm_w = torch.empty(self.vw, dtype=torch.float32, device=dev)
        views, at = {}, 0
        self.cols_at = {}
        for t, n, size in zip(order, names, sizes):
            views[n] = self.w_in[at:at + size]
            self.cols_at[t] = (at, at + size)
            at += size
        views.update({self._n("input_gate") + ".b": self.gate_bias[0], self._n("forget_gate") + ".b": self.gate_bias[1],
                      self._n("norm"): self.norm_w, self._n("o"): self.w_o})
        return views

    def kv_layout(self):
        return None

    def state_spec(self):
        return StateSpec((self.state_words + self.spec.num_heads,), torch.float32)

    def forward(self, h, ctx, layer):
        s, rt = self.spec, self.rt
        n, H = h.shape[0], s.num_heads
        proj = rt.ws.get("mm_proj", (n, self.proj_width), torch.float32)
        linear(rt, h, self.w_in, proj)
        part = lambda t: proj[:, self.cols_at[t][0]:self.cols_at[t][1]]
        v1 = rt.ws.get("mm_values", (n, H * self.cols), torch.float32)
        ktm = rt.ws.get("mm_keep_take_max", (3, n, H), torch.float32)
        ops.matrix_memory_prepare(part("v"), part("input_gate"), part("forget_gate"), self.proj_width, self.gate_bias[0],
                                  self.gate_bias[1], s.gate_cap, layer.state[:, self.state_words:], ctx.seq_start, ctx.seq_slot,
                                  v1, ktm, ctx.n_seqs, H, s.value_dim, self.cols)
        o = rt.ws.get("rec_out", (n, H * self.cols), torch.float32)
        # queries and keys go in as projected: the input weight rides on the values, the queries' scale on the result
        ops.gated_scan(ops.SCAN_SCALAR_DECAY, part("q"), part("k"), ktm[0], v1, None, None, None, layer.state, ctx.seq_start,
                       ctx.seq_slot, o, ctx.n_seqs, H, s.key_dim, self.cols, ready=True)
        y = rt.ws.get("rec_normed", (n, self.vw), rt.dtype)
        ops.matrix_memory_finish(o, ktm[2], self.norm_w, part("gate"), y, H, s.value_dim, self.cols, s.eps, self.FLOOR,
                                 q_scale=s.key_dim ** -0.5)
        out = rt.ws.get("mixer_out", (n, s.hidden), torch.float32)
        linear(rt, y, self.w_o, out)
        return out


class GatedDiagonalRecurrence(Part):
    """Recurrent block with a real-gated diagonal recurrence (see ``GatedDiagonalSpec``).  One packed product makes
    both branches; a kernel applies GELU to the gate branch and the causal convolution to the other (the last taps - 1
    inputs of a sequence are state); the recurrence and input gates are block-diagonal projections of the
    convolution's output (one per-block product for both); a scan kernel makes the decay and walks the tokens.  Per
    slot the state holds S [channels] and then the convolution's inputs [taps - 1, channels], all floats."""

    graph_safe = True

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        s = spec
        if s.channels % s.blocks:
            raise Unsupported(s.kind + ".blocks", f"{s.blocks} does not divide {s.channels} channels")
        if s.taps > ops.CONV_MAX_TAPS:
            raise Unsupported(s.kind + ".conv", f"{s.taps} taps; the convolution kernel takes up to {ops.CONV_MAX_TAPS}")
        self.cb = s.channels // s.blocks
        if self.cb * 8 * 4 > 48 * 1024:
            raise Unsupported(s.kind + ".blocks", f"blocks of {self.cb} channels are beyond what the per-block product takes")
        self.w_in = self.b_in = self.conv_w = self.conv_b = self.w_gates = self.b_gates = self.lam = self.w_o = None

    def _n(self, which):
        return self.spec.prefix + getattr(self.spec.names, which)

    def param_specs(self):
        s, C, B, cb = self.spec, self.spec.channels, self.spec.blocks, self.cb
        return [ParamSpec(self._n("gate_branch"), (C, s.hidden), "matrix"), ParamSpec(self._n("gate_branch") + ".b", (C,), "bias"),
                ParamSpec(self._n("in_branch"), (C, s.hidden), "matrix"), ParamSpec(self._n("in_branch") + ".b", (C,), "bias"),
                ParamSpec(self._n("conv"), (C, s.taps), "conv_taps", init=(0.0, 0.5)),
                ParamSpec(self._n("conv") + ".b", (C,), "bias"),
                ParamSpec(self._n("recurrence_gate"), (B, cb, cb), "gate_matrix", init=(0.0, 0.2)),
                ParamSpec(self._n("recurrence_gate") + ".b", (B, cb), "bias"),
                ParamSpec(self._n("input_gate"), (B, cb, cb), "gate_matrix", init=(0.0, 0.2)),
                ParamSpec(self._n("input_gate") + ".b", (B, cb), "bias"),
                ParamSpec(self._n("decay"), (C,), "decay_rate", init=(-1.0, 1.0)),
                ParamSpec(self._n("o"), (s.hidden, C), "matrix")]

    def allocate(self, stored, rt):
        s, dev, C, B, cb = self.spec, rt.device, self.spec.channels, self.spec.blocks, self.cb
        f32 = lambda *shape: torch.empty(shape, dtype=torch.float32, device=dev)
        ny, nx = self._n("gate_branch"), self._n("in_branch")
        self.w_in = torch.empty((2 * C, s.hidden), dtype=rt.matrix_dtype([stored[ny], stored[nx]]), device=dev)
        self.b_in = f32(2, C)
        self.conv_w, self.conv_b = f32(C, s.taps), f32(C)
        nr, ni = self._n("recurrence_gate"), self._n("input_gate")
        # a block's two gate matrices stacked: one per-block product makes [r | i] of the block
        self.w_gates = torch.empty((B, 2 * cb, cb), dtype=rt.matrix_dtype([stored[nr], stored[ni]]), device=dev)
        self.b_gates = f32(2, C)
        self.lam = f32(C)
        self.w_o = torch.empty((s.hidden, C), dtype=rt.matrix_dtype([stored[self._n("o")]]), device=dev)
        return {ny: self.w_in[:C], nx: self.w_in[C:], ny + ".b": self.b_in[0], nx + ".b": self.b_in[1],
                self._n("conv"): self.conv_w, self._n("conv") + ".b": self.conv_b, nr: self.w_gates[:, :cb], ni: self.w_gates[:, cb:],
                nr + ".b": self.b_gates[0].view(B, cb), ni + ".b": self.b_gates[1].view(B, cb), self._n("decay"): self.lam,
                self._n("o"): self.w_o}

    def kv_layout(self):
        return None

    def state_spec(self):
        return StateSpec((self.spec.taps * self.spec.channels,), torch.float32)

    def forward(self, h, ctx, layer):
        s, rt, C = self.spec, self.rt, self.spec.channels
        n = h.shape[0]
        proj = rt.ws.get("diag_proj", (n, 2 * C), torch.float32)
        linear(rt, h, self.w_in, proj)
        branch = rt.ws.get("diag_branch", (2, n, C), torch.float32)        # the gate branch, the convolution's output
        u_act = rt.ws.get("diag_u", (n, C), rt.dtype)
        ops.conv_branches(proj, self.b_in[0], self.b_in[1], self.conv_w, self.conv_b, layer.state[:, C:], ctx.tok_seq,
                          ctx.seq_start, ctx.seq_slot, branch[0], branch[1], u_act, ctx.n_seqs, C, s.taps)
        gates = rt.ws.get("diag_gates", (n, 2 * C), torch.float32)
        ops.per_head_linear(u_act, C, self.cb, self.w_gates, gates, 2 * C, 2 * self.cb, n, s.blocks, self.cb, 2 * self.cb)
        y = rt.ws.get("rec_normed", (n, C), rt.dtype)
        ops.diag_scan(gates, self.b_gates[0], self.b_gates[1], self.lam, s.decay_scale, branch[1], branch[0], layer.state,
                      ctx.seq_start, ctx.seq_slot, y, ctx.n_seqs, C, s.blocks)
        out = rt.ws.get("mixer_out", (n, s.hidden), torch.float32)
        linear(rt, y, self.w_o, out)
        return out


register("mixer", "hgrn2", LowerBoundRecurrence)
register("mixer", "mlstm", MatrixMemory)
register("mixer", "rglru", GatedDiagonalRecurrence)
register("mixer", "wkv", DecayBonusRecurrence)
