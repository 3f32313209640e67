"""Vumedra configurations drawn at random (sizes, head counts, order of the layers, constants, seeds), each run whole,
as a prompt followed by single tokens and as one unequal batch, in both dtypes, against the plain restatement."""
import json

import numpy as np
import pytest
import torch

import plain_vumedra as plain
from gpu_util import run_steps, steps_batches, steps_tail, steps_whole
from test_gpu_vumedra import BOUND, Choices
from vumedra_cases import random_weights

from esp_b200.engine import Engine
from esp_b200.weights import write_safetensors

pytestmark = pytest.mark.gpu


def draw(rng):
    pick = lambda *xs: xs[int(rng.integers(0, len(xs)))]
    width = pick(64, 72, 100, 128, 160, 256)
    layers = []
    for _ in range(int(rng.integers(2, 6))):
        kind = pick("attention", "mlstm", "rglru")
        if kind == "attention":
            heads = pick(1, 2, 3, 4, 6, 8)
            dim = pick(8, 16, 20, 24, 32, 64, 64, 128)
            mixer = {"heads": heads, "kv_heads": pick(*[g for g in range(1, heads + 1) if heads % g == 0]), "dim": dim,
                     "vdim": pick(dim, dim, 8, 16, 40, 64, 72), "scale": float(rng.uniform(0.05, 0.4))}
            if rng.integers(0, 4) > 0:
                mixer["q_temp"] = {"coef": float(rng.uniform(0.1, 1.0)), "every": pick(1, 3, 16, 64, 100)}
        elif kind == "mlstm":
            mixer = {"heads": pick(1, 2, 3, 4), "dim": pick(8, 16, 24, 32, 64), "vdim": pick(8, 12, 16, 31, 48),
                     "gate_cap": float(rng.uniform(5.0, 20.0))}
        else:
            blocks = pick(1, 2, 4, 5)
            mixer = {"width": blocks * pick(8, 12, 16, 40), "blocks": blocks, "conv": pick(1, 2, 3, 4, 5)}
        which = int(rng.integers(0, 5))
        if which == 0:
            mlp = None
        elif which < 3:
            mlp = {"kind": "dense", "ff": pick(16, 40, 64, 136)}
        else:
            experts = pick(2, 3, 4, 8, 16)
            mlp = {"kind": "moe", "router": {"experts": experts, "top": int(rng.integers(1, min(experts, 4) + 1))},
                   "expert": {"ff": pick(8, 16, 24, 32, 64)}, "shared": None if rng.integers(0, 3) == 0 else {"ff": pick(8, 16, 48)}}
        layers.append({"type": kind, "mixer": mixer, "mlp": mlp})
    return {"architecture": "Vumedra", "vocab": pick(97, 256, 301, 513), "width": width, "norm": {"eps": pick(1e-6, 1e-5)},
            "embedding": {"bigram": {"buckets": pick(31, 257, 4099), "mul_prev": int(rng.integers(0, 1 << 20)),
                                     "mul_cur": int(rng.integers(0, 1 << 20))}}, "layers": layers}


def relative_error(got, ref):
    d = got - ref
    d = d - d.mean(1, keepdims=True)
    return np.sqrt((d ** 2).mean(1)) / np.sqrt((ref ** 2).mean())


@pytest.mark.parametrize("seed", list(range(10)))
def test_random_configuration(tmp_path, seed):
    rng = np.random.default_rng(2000 + seed)
    lengths = (1, 70, 133)
    # a draw whose 32-bit arithmetic is ill conditioned by itself (the matrix memory's quotient by a sum that nearly
    # cancels: the plain restatement in 32-bit then misses its own 64-bit run) says nothing about the engine: draw again
    for attempt in range(20):
        raw = draw(rng)
        stored = random_weights(raw, 50 + seed + 100 * attempt)
        w = {k: v.double() for k, v in stored.items()}
        reqs = {f"r{i}": [int(t) for t in rng.integers(0, raw["vocab"], n)] for i, n in enumerate(lengths)}
        own = max(float(relative_error(plain.forward(raw, w, t, dtype=torch.float32).double().numpy(),
                                       plain.forward(raw, w, t).numpy()).max()) for t in reqs.values())
        if own < 4e-6:
            break
    else:
        pytest.fail("no well-conditioned draw")
    (tmp_path / "config.json").write_text(json.dumps(raw))
    write_safetensors(tmp_path / "model.safetensors", stored)
    ids = list(reqs)
    for dtype in ("float32", "bfloat16"):
        eng = Engine.from_folder(tmp_path, dtype=dtype, max_tokens=1024)
        eng.rt.record_routing = True
        for what, steps in (("whole", steps_whole(reqs)), ("prompt + single tokens", steps_tail(reqs, tail=40)),
                            ("one batch", steps_batches(reqs, [ids], {rid: max(1, len(t) - 25) for rid, t in reqs.items()}))):
            rec = Choices(raw["vocab"])
            run_steps(eng, steps, rec)
            for rid, toks in reqs.items():
                chosen = rec.chosen(rid, len(toks))
                ref = plain.forward(raw, w, toks, choices=chosen or None).numpy()
                err = relative_error(rec.logits_of(rid, list(range(len(toks)))), ref)
                assert err.max() <= BOUND[dtype], (f"seed {seed}, {dtype}, {what}, request {rid}: position {int(err.argmax())} "
                                                   f"is off by {err.max():.3e}; configuration {json.dumps(raw)}")
        del eng
