"""Configuration of the Vumedra decoder: token, hashed-bigram and sinusoidal embeddings summed; a stack of layers,
each with one of three token mixers (softmax attention with normed queries and keys and a sink in the denominator,
a matrix memory with exponential gating, a gated diagonal recurrence behind a short convolution) and an optional
feed-forward (dense SwiGLU, or routed experts with a sigmoid router and a shared expert); every sublayer's result
passes a norm of its own before it joins the residual stream; norms carry one learned number.

config.json names every size and every constant that may differ between models; this class reads it, refuses what
the parts cannot run, and turns it into the architecture-neutral plan.  Keys:

    architecture: "Vumedra";  vocab, width;  norm.eps;  embedding.bigram {buckets, mul_prev, mul_cur}
    layers: [{type: "attention" | "mlstm" | "rglru", mixer: {...}, mlp: {...} | null}, ...]
    mixer (attention): heads, kv_heads, dim, vdim, scale, q_temp {coef, every}
    mixer (mlstm):     heads, dim, vdim, gate_cap
    mixer (rglru):     width, blocks, conv
    mlp: {kind: "dense", ff} | {kind: "moe", router {experts, top}, expert {ff}, shared {ff}}

Tensor names: ``embed``, ``bigram``, ``head``, ``final.norm``, and per layer i ``l<i>.norm1``, ``l<i>.norm1b``,
``l<i>.norm2``, ``l<i>.norm2b``, ``l<i>.mix.*``, ``l<i>.mlp.*``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

from ..errors import InvalidConfig, Unsupported
from .plan import (DenseFfnSpec, GatedDiagonalSpec, HashedBigramSpec, MatrixMemorySpec, ModelPlan, NormedAttentionSpec,
                   NormSpec, QueryTemperature, SandwichBlockSpec, ScaledInputMoeSpec, ScheduleEntry, SummedEmbeddingSpec,
                   SwiGluNames)
from .registry import register_architecture

ARCHITECTURE = "Vumedra"
MODEL_TYPE = "vumedra"
MIXERS = ("attention", "mlstm", "rglru")
# The design names no longest position; positions are exact as 32-bit floats up to 2^24, and the cache book wants a bound.
POSITION_BOUND = 1 << 20
# Fixed by the design: the base of the sinusoidal positions and the factor in the diagonal recurrence's decay.
SINUSOID_BASE = 10000.0
DECAY_SCALE = 8.0


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


def _obj(d, key, where):
    v = d.get(key)
    if not isinstance(v, dict):
        raise InvalidConfig(f"{where}.{key} must be an object")
    return v


@dataclass
class VumedraConfig:
    vocab: int
    width: int
    eps: float
    bigram: dict
    layers: list = field(default_factory=list)       # the config's entries, checked

    @classmethod
    def from_dict(cls, raw: dict) -> "VumedraConfig":
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers or not all(isinstance(l, dict) for l in layers):
            raise InvalidConfig("layers must be a non-empty list of objects")
        layers = [dict(l, mixer=dict(l["mixer"])) if isinstance(l.get("mixer"), dict) else dict(l) for l in layers]
        for layer in layers:
            mix = layer.get("mixer")
            if isinstance(mix, dict) and layer.get("type") in ("attention", "mlstm"):
                if "vdim" not in mix and "dim" in mix:
                    mix["vdim"] = mix["dim"]               # value channels default to the key channels
                if layer["type"] == "attention" and "kv_heads" not in mix and "heads" in mix:
                    mix["kv_heads"] = mix["heads"]
        cfg = cls(vocab=_int(raw, "vocab", "config"), width=_int(raw, "width", "config"),
                  eps=_num(_obj(raw, "norm", "config"), "eps", "norm"),
                  bigram=dict(_obj(_obj(raw, "embedding", "config"), "bigram", "embedding")), layers=layers)
        cfg.validate()
        return cfg

    # ---- checks -----------------------------------------------------------------
    def validate(self) -> None:
        if not self.eps > 0:
            raise InvalidConfig("norm.eps must be positive")
        _int(self.bigram, "buckets", "embedding.bigram")
        _int(self.bigram, "mul_prev", "embedding.bigram", 0)
        _int(self.bigram, "mul_cur", "embedding.bigram", 0)
        # the hash is taken in 64-bit integers on the device
        if max(self.bigram["mul_prev"], self.bigram["mul_cur"]) * self.vocab >= 1 << 62:
            raise InvalidConfig("embedding.bigram: multiplier times vocabulary passes 62 bits")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            kind = layer.get("type")
            if kind not in MIXERS:
                raise Unsupported("layers.type", f"{kind!r} in {where}; this design has {', '.join(MIXERS)}")
            mix = _obj(layer, "mixer", where)
            w = where + ".mixer"
            if kind == "attention":
                for key in ("heads", "kv_heads", "dim", "vdim"):
                    _int(mix, key, w)
                if mix["heads"] % mix["kv_heads"]:
                    raise InvalidConfig(f"{w}.kv_heads must divide heads")
                _num(mix, "scale", w)
                temp = mix.get("q_temp")
                if temp is not None:
                    _num(_obj(mix, "q_temp", w), "coef", w + ".q_temp")
                    _int(temp, "every", w + ".q_temp")
            elif kind == "mlstm":
                for key in ("heads", "dim", "vdim"):
                    _int(mix, key, w)
                if not _num(mix, "gate_cap", w) > 0:
                    raise InvalidConfig(f"{w}.gate_cap must be positive")
            else:
                for key in ("width", "blocks", "conv"):
                    _int(mix, key, w)
                if mix["width"] % mix["blocks"]:
                    raise InvalidConfig(f"{w}.blocks must divide width")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
                raise Unsupported("layers.mlp.kind", f"{mlp!r} in {where}; this design has dense and moe feed-forwards")
            w = where + ".mlp"
            if mlp["kind"] == "dense":
                _int(mlp, "ff", w)
            else:
                router = _obj(mlp, "router", w)
                if _int(router, "top", w + ".router") > _int(router, "experts", w + ".router"):
                    raise InvalidConfig(f"{w}.router.top exceeds the number of experts")
                _int(_obj(mlp, "expert", w), "ff", w + ".expert")
                if mlp.get("shared") is not None:
                    _int(_obj(mlp, "shared", w), "ff", w + ".shared")

    # ---- writing ------------------------------------------------------------------
    def to_dict(self) -> dict:
        return {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
                "embedding": {"bigram": dict(self.bigram)}, "layers": self.layers}

    # ---- the plan -------------------------------------------------------------------
    def _mixer_spec(self, i: int, layer: dict):
        mix, p = layer["mixer"], f"l{i}.mix."
        if layer["type"] == "attention":
            temp = mix.get("q_temp")
            return NormedAttentionSpec(self.width, mix["heads"], mix["kv_heads"], mix["dim"], mix["vdim"], float(mix["scale"]),
                                       self.eps, True, True,
                                       QueryTemperature(float(temp["coef"]), int(temp["every"])) if temp else None, None, p)
        if layer["type"] == "mlstm":
            return MatrixMemorySpec(self.width, mix["heads"], mix["dim"], mix["vdim"], float(mix["gate_cap"]), self.eps, p)
        return GatedDiagonalSpec(self.width, mix["width"], mix["blocks"], mix["conv"], DECAY_SCALE, p)

    def _ffn_spec(self, i: int, mlp):
        p = f"l{i}.mlp."
        if mlp["kind"] == "dense":
            return DenseFfnSpec(self.width, mlp["ff"], p, names=SwiGluNames("gate", "up", "down"))
        shared = mlp.get("shared")
        return ScaledInputMoeSpec(self.width, mlp["router"]["experts"], mlp["router"]["top"], mlp["expert"]["ff"],
                                  shared["ff"] if shared is not None else None, p)

    def plan(self) -> ModelPlan:
        norm = lambda name: NormSpec("rmsnorm_scalar", self.width, self.eps, name)
        blocks, schedule = [], []
        for i, layer in enumerate(self.layers):
            mlp = layer.get("mlp")
            ffn = self._ffn_spec(i, mlp) if mlp is not None else None
            blocks.append(SandwichBlockSpec(self._mixer_spec(i, layer), ffn, norm(f"l{i}.norm1"), norm(f"l{i}.norm1b"),
                                            norm(f"l{i}.norm2") if ffn is not None else None,
                                            norm(f"l{i}.norm2b") if ffn is not None else None))
            schedule.append(ScheduleEntry(i))
        b = self.bigram
        return ModelPlan(architecture=ARCHITECTURE, hidden=self.width, vocab=self.vocab, max_positions=POSITION_BOUND,
                         blocks=blocks, schedule=schedule, final_norm=norm("final.norm"), embed_weight="embed",
                         head_weight="head",
                         # a layer without feed-forward has no second pair of norms; a checkpoint that stores them all
                         # the same is read without them
                         tolerated_suffixes=(".norm2", ".norm2b"),
                         embedding=SummedEmbeddingSpec(self.width, HashedBigramSpec(b["buckets"], b["mul_prev"], b["mul_cur"],
                                                                                    "bigram"), SINUSOID_BASE))


register_architecture(ARCHITECTURE, MODEL_TYPE, VumedraConfig)
