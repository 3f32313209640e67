"""Configuration of the Zusepel decoder: a stack of layers, each with one of three token mixers (a gated linear
recurrence with a lower-bounded forget gate, a time-mixing recurrence with token shift and data-dependent
decay, attention through a cached low-rank latent with a sliding window), an optional dense feed-forward, a
scale per channel on both results and a weighted average over the depth behind every layer.

config.json names every size; this class reads it, refuses what the parts cannot run, and turns it into the
architecture-neutral plan.  Keys:

    architecture: "Zusepel";  vocab, width;  norm.eps;  residual_mult;
    layers: [{type: "hgrn2" | "wkv" | "latent_attention", mixer: {...}, mlp: {kind: "dense", ff} | null}, ...]
    mixer (hgrn2):  heads, dim, vdim
    mixer (wkv):    heads, dim                       (the decay's inner width is the stored tensor's)
    mixer (latent_attention): heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, mask.size,
                    rot {base, dims, scaling {factor, original, fast, slow} | null}, kv_from (optional)

Tensor names: ``embed``, ``head``, ``final.norm``, and per layer i ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.ls1``,
``l<i>.ls2``, ``l<i>.dwa``, ``l<i>.mix.*``, ``l<i>.mlp.*``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional

from ..errors import InvalidConfig, Unsupported
from .plan import (DecayBonusRecurrenceSpec, DepthMixBlockSpec, LatentAttentionSpec, LowerBoundRecurrenceSpec, ModelPlan,
                   NormSpec, ScaledRopeSpec, ScheduleEntry, XieluFfnSpec)
from .registry import register_architecture

ARCHITECTURE = "Zusepel"
MODEL_TYPE = "zusepel"
MIXERS = ("hgrn2", "wkv", "latent_attention")
# The design names no longest position.  Positions are 32-bit floats in the rotation, exact up to 2^24; the cache
# book wants a bound, and this is it.
POSITION_BOUND = 1 << 20


def _int(d, key, where, minimum=1):
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v < minimum:
        raise InvalidConfig(f"{where}.{key} must be an integer >= {minimum}, got {v!r}")
    return v


def _num(d, key, where):
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v):
        raise InvalidConfig(f"{where}.{key} must be a finite number, got {v!r}")
    return float(v)


@dataclass
class ZusepelConfig:
    vocab: int
    width: int
    eps: float
    residual_mult: float
    layers: list = field(default_factory=list)       # the config's entries, checked
    decay_ranks: dict = field(default_factory=dict)  # layer -> inner width of a wkv layer's decay projection

    # the inner width of a wkv layer's decay is not in config.json: a model folder gives it by the tensor's shape
    # (``bind_shapes``), a configuration without a folder uses this
    DEFAULT_DECAY_RANK = 16

    @classmethod
    def from_dict(cls, raw: dict) -> "ZusepelConfig":
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise InvalidConfig("norm must be an object with eps")
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise InvalidConfig("layers must be a non-empty list")
        layers = [dict(l, mixer=dict(l["mixer"])) if isinstance(l, dict) and isinstance(l.get("mixer"), dict) else l
                  for l in layers]
        if not all(isinstance(l, dict) for l in layers):
            raise InvalidConfig("every entry of layers must be an object")
        for i, layer in enumerate(layers):
            mix = layer.get("mixer")
            if not isinstance(mix, dict):
                continue
            if "vdim" not in mix and "dim" in mix and layer.get("type") in ("hgrn2", "latent_attention"):
                mix["vdim"] = mix["dim"]                   # value channels default to the key channels
            src = mix.get("kv_from")
            if layer.get("type") == "latent_attention" and isinstance(src, int) and not isinstance(src, bool) and 0 <= src < i:
                owner = layers[src].get("mixer")
                if isinstance(owner, dict):                # what a reader must share with the cache's owner may be left out
                    for key in ("kv_rank", "rot_dim", "rot"):
                        if key not in mix and key in owner:
                            mix[key] = owner[key]
        cfg = cls(vocab=_int(raw, "vocab", "config"), width=_int(raw, "width", "config"), eps=_num(norm, "eps", "norm"),
                  residual_mult=_num(raw, "residual_mult", "config") if "residual_mult" in raw else 1.0, layers=layers,
                  decay_ranks={int(k): int(v) for k, v in (raw.get("decay_ranks") or {}).items()})
        cfg.validate()
        return cfg

    # ---- checks -----------------------------------------------------------------
    def validate(self) -> None:
        if not self.eps > 0:
            raise InvalidConfig("norm.eps must be positive")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            kind = layer.get("type")
            if kind not in MIXERS:
                raise Unsupported("layers.type", f"{kind!r} in {where}; this design has {', '.join(MIXERS)}")
            mix = layer.get("mixer")
            if not isinstance(mix, dict):
                raise InvalidConfig(f"{where}.mixer must be an object")
            _int(mix, "heads", where + ".mixer")
            _int(mix, "dim", where + ".mixer")
            if kind == "hgrn2":
                _int(mix, "vdim", where + ".mixer")
            if kind == "latent_attention":
                self._check_latent(i, mix, where + ".mixer")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise Unsupported("layers.mlp.kind", f"{mlp!r} in {where}; this design has dense feed-forwards")
                _int(mlp, "ff", where + ".mlp")

    def _check_latent(self, i, mix, where):
        for key in ("rot_dim", "vdim", "q_rank", "kv_rank"):
            _int(mix, key, where)
        _num(mix, "scale", where)
        rot = mix.get("rot")
        if not isinstance(rot, dict):
            raise InvalidConfig(f"{where}.rot must be an object")
        dims = _int(rot, "dims", where + ".rot", 2)
        if dims % 2 or dims > mix["rot_dim"]:
            raise InvalidConfig(f"{where}.rot.dims must be even and at most rot_dim, got {dims}")
        if not _num(rot, "base", where + ".rot") > 0:
            raise InvalidConfig(f"{where}.rot.base must be positive")
        sc = rot.get("scaling")
        if sc is not None:
            for key in ("factor", "original", "fast", "slow"):
                if not _num(sc, key, where + ".rot.scaling") > 0:
                    raise InvalidConfig(f"{where}.rot.scaling.{key} must be positive")
        mask = mix.get("mask")
        if mask is not None:
            _int(mask, "size", where + ".mask")
        src = mix.get("kv_from")
        if src is not None:
            ok = isinstance(src, int) and not isinstance(src, bool) and 0 <= src < i
            other = self.layers[src] if ok else None
            if not ok or other.get("type") != "latent_attention" or other["mixer"].get("kv_from") is not None:
                raise InvalidConfig(f"{where}.kv_from must name an earlier latent_attention layer with a cache of its own")
            for key in ("kv_rank", "rot_dim", "rot"):
                if other["mixer"].get(key) != mix.get(key):
                    raise InvalidConfig(f"{where}.{key} differs from layer {src}'s, whose cache it reads")

    # ---- shapes that only the checkpoint knows --------------------------------------
    def bind_shapes(self, shapes: dict) -> None:
        """``shapes``: tensor name -> shape of a checkpoint.  Takes from it what config.json leaves to the tensors."""
        for i, layer in enumerate(self.layers):
            name = f"l{i}.mix.w1"
            if layer["type"] == "wkv" and name in shapes and len(shapes[name]) == 2:
                self.decay_ranks[i] = int(shapes[name][0])

    # ---- writing ------------------------------------------------------------------
    def to_dict(self) -> dict:
        d = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
             "residual_mult": self.residual_mult, "layers": self.layers}
        if self.decay_ranks:
            d["decay_ranks"] = {str(k): v for k, v in sorted(self.decay_ranks.items())}
        return d

    # ---- the plan -------------------------------------------------------------------
    def _keep_window(self, owner: int) -> Optional[int]:
        """How far back layer ``owner``'s cache must reach: the widest window among the layers that read it."""
        sizes = []
        for i, layer in enumerate(self.layers):
            if layer["type"] == "latent_attention" and (i == owner or layer["mixer"].get("kv_from") == owner):
                mask = layer["mixer"].get("mask")
                if mask is None:
                    return None
                sizes.append(mask["size"])
        return max(sizes)

    def _mixer_spec(self, i: int, layer: dict):
        mix, p = layer["mixer"], f"l{i}.mix."
        if layer["type"] == "hgrn2":
            return LowerBoundRecurrenceSpec(self.width, mix["heads"], mix["dim"], mix["vdim"], self.eps, p)
        if layer["type"] == "wkv":
            return DecayBonusRecurrenceSpec(self.width, mix["heads"], mix["dim"],
                                            self.decay_ranks.get(i, self.DEFAULT_DECAY_RANK), self.eps, p)
        rot, sc = mix["rot"], mix["rot"].get("scaling")
        pos = ScaledRopeSpec(rot["dims"], float(rot["base"]), *((float(sc["factor"]), float(sc["original"]), float(sc["fast"]),
                                                                  float(sc["slow"])) if sc else ()))
        owner = mix.get("kv_from")
        mask = mix.get("mask")
        return LatentAttentionSpec(self.width, mix["heads"], mix["dim"], mix["rot_dim"], mix["vdim"], mix["q_rank"],
                                   mix["kv_rank"], float(mix["scale"]), mask["size"] if mask else None,
                                   self._keep_window(i if owner is None else owner), self.eps, pos, owner is None, p)

    def plan(self) -> ModelPlan:
        blocks, schedule = [], []
        depth = len(self.layers)
        for i, layer in enumerate(self.layers):
            mlp = layer.get("mlp")
            ffn = XieluFfnSpec(self.width, mlp["ff"], f"l{i}.mlp.") if mlp is not None else None
            blocks.append(DepthMixBlockSpec(
                self._mixer_spec(i, layer), ffn, NormSpec("rmsnorm", self.width, self.eps, f"l{i}.norm1"),
                NormSpec("rmsnorm", self.width, self.eps, f"l{i}.norm2") if ffn is not None else None,
                self.residual_mult, f"l{i}.ls1", f"l{i}.ls2" if ffn is not None else None, f"l{i}.dwa", i, depth, self.width))
            schedule.append(ScheduleEntry(i, layer["mixer"].get("kv_from") if layer["type"] == "latent_attention" else None))
        return ModelPlan(architecture=ARCHITECTURE, hidden=self.width, vocab=self.vocab, max_positions=POSITION_BOUND,
                         blocks=blocks, schedule=schedule,
                         final_norm=NormSpec("rmsnorm", self.width, self.eps, "final.norm"),
                         embed_weight="embed", head_weight="head")


register_architecture(ARCHITECTURE, MODEL_TYPE, ZusepelConfig)
