"""How the parts of one layer are arranged."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import ParamSpec, Part, build, plain_delta, register
from .norm import DeferredPostNorm


class PreNormResidualBlock(Part):
    """x += mixer(norm(x)); x += ffn(norm(x))
    (crates/esp/src/infer/decoder/layer.rs:115-153).  The residual adds are
    folded into the norm that follows them: a part's output travels as
    ``pending`` until the next norm adds it to the 32-bit residual stream."""

    graph_safe = True

    def __init__(self, spec, rt):
        self.spec = spec
        self.rt = rt
        self.mixer_norm = build("norm", spec.mixer_norm, rt)
        self.mixer = build("mixer", spec.mixer, rt)
        self.ffn_norm = build("norm", spec.ffn_norm, rt)
        self.ffn = build("ffn", spec.ffn, rt)

    def children(self):
        return [self.mixer_norm, self.mixer, self.ffn_norm, self.ffn]

    def forward(self, x, pending, ctx, layer):
        rt = self.rt
        h = rt.ws.get("block_h", tuple(x.shape), rt.dtype)
        self.mixer_norm.forward(x, plain_delta(self.mixer_norm, pending), h)
        delta = self.mixer.forward(h, ctx, layer)
        h32 = None
        if rt.dtype != torch.float32 and getattr(self.ffn, "wants_f32_input", False):
            h32 = rt.ws.get("block_h32", tuple(x.shape), torch.float32)
        self.ffn_norm.forward(x, plain_delta(self.ffn_norm, delta), h, h32=h32)
        return self.ffn.forward(h, ctx, h32=h32)


class ScaledDepthMixBlock(Part):
    """x <- x + m s1 * mixer(norm1(x)); x <- x + m s2 * ffn(norm2(x)) with s1, s2 a scale per channel and m the
    residual multiplier; the result X_(i+1) of layer i is kept, and what the next layer (or the model's end) reads is
    sum_j w[j] X_j over the embedding output X_0 and every result so far.  The first add is folded into the second
    norm; the second add, the bookkeeping of X and the weighted sum are one kernel.  A layer without a feed-forward
    has no second norm and no second scale."""

    graph_safe = True

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        self.mixer_norm = build("norm", spec.mixer_norm, rt)
        self.mixer = build("mixer", spec.mixer, rt)
        self.ffn_norm = build("norm", spec.ffn_norm, rt)
        self.ffn = build("ffn", spec.ffn, rt)
        self.scale1 = self.scale2 = self.weights = None
        self._folded = False

    def children(self):
        return [p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if p is not None]

    def param_specs(self):
        s = self.spec
        specs = [ParamSpec(s.mixer_scale, (s.hidden,), "norm_scale"),
                 ParamSpec(s.depth_weights, (s.index + 2,), "depth_weights", init=(1.0 / (s.index + 2), 0.2 / (s.index + 2)))]
        if s.ffn_scale is not None:
            specs.append(ParamSpec(s.ffn_scale, (s.hidden,), "norm_scale"))
        return specs

    def allocate(self, stored, rt):
        s = self.spec
        f32 = lambda n: torch.empty(n, dtype=torch.float32, device=rt.device)
        self.scale1, self.weights = f32(s.hidden), f32(s.index + 2)
        views = {s.mixer_scale: self.scale1, s.depth_weights: self.weights}
        if s.ffn_scale is not None:
            self.scale2 = f32(s.hidden)
            views[s.ffn_scale] = self.scale2
        return views

    def finalize(self):
        if not self._folded:                      # the residual multiplier goes into the scales once
            self._folded = True
            self.scale1.mul_(self.spec.residual_mult)
            if self.scale2 is not None:
                self.scale2.mul_(self.spec.residual_mult)

    def forward(self, x, pending, ctx, layer):
        rt, s = self.rt, self.spec
        n = x.shape[0]
        history = rt.ws.get("depth_history", (s.depth + 1, n, s.hidden), torch.float32)
        h = rt.ws.get("block_h", tuple(x.shape), rt.dtype)
        self.mixer_norm.forward(x, plain_delta(self.mixer_norm, pending), h)
        if s.index == 0:
            history[0].copy_(x)                   # X_0: what the embedding (and anything before this stack) left
        delta = self.mixer.forward(h, ctx, layer)
        if self.ffn is None:
            ops.depth_mix(x, delta, self.scale1, history, self.weights, s.index)
            self._trace(x, ctx)
            return None
        self.ffn_norm.forward(x, delta, h, delta_scale=self.scale1)
        delta = self.ffn.forward(h, ctx)
        ops.depth_mix(x, plain_delta(None, delta), self.scale2, history, self.weights, s.index)
        self._trace(x, ctx)
        return None

    @staticmethod
    def _trace(x, ctx):
        """Debugging aid: a caller that passes ``aux={"residual_trace": []}`` to the step gets a copy of the
        residual stream behind every layer (such a step is never replayed from a captured graph)."""
        if "residual_trace" in ctx.aux:
            ctx.aux["residual_trace"].append(x.clone())


class SandwichBlock(Part):
    """x += post1(mixer(pre1(x))); x += post2(ffn(pre2(x))): a norm before and a norm after every sublayer.  A
    sublayer's result travels as a ``DeferredPostNorm`` until the next norm that reads x (this block's, the next
    block's or the model's last) normalises it, adds it and normalises x, all in one launch."""

    graph_safe = True

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        self.mixer_norm = build("norm", spec.mixer_norm, rt)
        self.mixer_post = build("norm", spec.mixer_post_norm, rt)
        self.mixer = build("mixer", spec.mixer, rt)
        self.ffn_norm = build("norm", spec.ffn_norm, rt)
        self.ffn_post = build("norm", spec.ffn_post_norm, rt)
        self.ffn = build("ffn", spec.ffn, rt)

    def children(self):
        return [p for p in (self.mixer_norm, self.mixer, self.mixer_post, self.ffn_norm, self.ffn, self.ffn_post)
                if p is not None]

    def forward(self, x, pending, ctx, layer):
        rt = self.rt
        h = rt.ws.get("block_h", tuple(x.shape), rt.dtype)
        self.mixer_norm.forward(x, plain_delta(self.mixer_norm, pending), h)
        pending = DeferredPostNorm(rt, self.mixer.forward(h, ctx, layer), self.mixer_post)
        if self.ffn is not None:
            h32 = None
            if rt.dtype != torch.float32 and getattr(self.ffn, "wants_f32_input", False):
                h32 = rt.ws.get("block_h32", tuple(x.shape), torch.float32)
            self.ffn_norm.forward(x, plain_delta(self.ffn_norm, pending), h, h32=h32)
            pending = DeferredPostNorm(rt, plain_delta(None, self.ffn.forward(h, ctx, h32=h32)), self.ffn_post)
        if "residual_trace" in ctx.aux:
            # debugging aid (see ScaledDepthMixBlock._trace): the add is done here so that x is the layer's result
            pending.add_to(x)
            ctx.aux["residual_trace"].append(x.clone())
            return None
        return pending


register("block", "prenorm_residual", PreNormResidualBlock)
register("block", "sandwich_residual", SandwichBlock)
register("block", "prenorm_scaled_depthmix", ScaledDepthMixBlock)
