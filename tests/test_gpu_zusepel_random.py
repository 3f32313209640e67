"""Zusepel configurations drawn at random (sizes, head counts, order of the layers, windows, constants, seeds), each
run whole and as a prompt followed by single tokens in both dtypes against the plain restatement."""
import json

import numpy as np
import pytest

import plain_zusepel as plain
from gpu_util import Recorder, run_steps, steps_tail, steps_whole

from esp_b200.engine import Engine
from esp_b200.weights import write_safetensors

pytestmark = pytest.mark.gpu
BOUND = {"float32": 2e-5, "bfloat16": 4e-2}


def draw(rng):
    pick = lambda *xs: xs[int(rng.integers(0, len(xs)))]
    width = pick(64, 72, 100, 128, 160)
    n_layers = int(rng.integers(2, 6))
    layers, owners = [], []
    for i in range(n_layers):
        kind = pick("hgrn2", "wkv", "latent_attention", "latent_attention")
        if kind == "hgrn2":
            mixer = {"heads": pick(1, 2, 3, 4), "dim": pick(8, 16, 20, 32, 48, 64), "vdim": pick(8, 12, 16, 40, 64)}
        elif kind == "wkv":
            mixer = {"heads": pick(1, 2, 3), "dim": pick(8, 16, 24, 32, 64)}
        else:
            rot_dim = pick(4, 8, 16, 32)
            scaling = None if rng.integers(0, 3) == 0 else {"factor": float(pick(2.0, 8.0, 32.0)), "original": pick(32, 256, 4096),
                                                            "fast": float(pick(4.0, 32.0)), "slow": float(pick(0.5, 1.0, 2.0))}
            mixer = {"heads": pick(1, 2, 3, 4, 5, 8), "dim": pick(8, 16, 24, 32), "rot_dim": rot_dim, "vdim": pick(8, 16, 24, 40),
                     "q_rank": pick(8, 16, 24, 40), "kv_rank": pick(8, 16, 24, 32, 40, 48, 64), "scale": float(rng.uniform(0.05, 0.4)),
                     "rot": {"base": float(pick(100.0, 10000.0, 1e6)), "dims": rot_dim, "scaling": scaling}}
            if rng.integers(0, 5) > 0:
                mixer["mask"] = {"size": pick(1, 2, 3, 17, 64, 65, 100, 1000)}
            if owners and rng.integers(0, 2) == 0:
                src = pick(*owners)
                for key in ("kv_rank", "rot_dim", "rot"):
                    mixer[key] = layers[src]["mixer"][key]
                mixer["kv_from"] = src
            else:
                owners.append(i)
        mlp = None if rng.integers(0, 4) == 0 else {"kind": "dense", "ff": pick(16, 40, 64, 136)}
        layers.append({"type": kind, "mixer": mixer, "mlp": mlp})
    raw = {"architecture": "Zusepel", "vocab": pick(97, 256, 301), "width": width, "norm": {"eps": pick(1e-6, 1e-5)},
           "residual_mult": float(rng.uniform(0.3, 1.5)), "layers": layers}
    return raw, pick(4, 8, 12, 16, 20)


@pytest.mark.parametrize("seed", list(range(10)))
def test_random_configuration(tmp_path, seed):
    rng = np.random.default_rng(1000 + seed)
    raw, rank = draw(rng)
    weights = plain.random_weights(raw, 50 + seed, decay_rank=rank)
    (tmp_path / "config.json").write_text(json.dumps(raw))
    write_safetensors(tmp_path / "model.safetensors", weights)
    reqs = {f"r{i}": [int(t) for t in rng.integers(0, raw["vocab"], n)] for i, n in enumerate((1, 70, 133))}
    refs = {rid: plain.forward(raw, weights, toks).numpy() for rid, toks in reqs.items()}
    for dtype in ("float32", "bfloat16"):
        eng = Engine.from_folder(tmp_path, dtype=dtype, max_tokens=1024)
        for what, steps in (("whole", steps_whole(reqs)), ("prompt + single tokens", steps_tail(reqs, tail=70))):
            rec = Recorder(raw["vocab"])
            run_steps(eng, steps, rec)
            for rid, toks in reqs.items():
                d = rec.logits_of(rid, list(range(len(toks)))) - refs[rid]
                d = d - d.mean(1, keepdims=True)
                err = np.sqrt((d ** 2).mean(1)) / np.sqrt((refs[rid] ** 2).mean())
                assert err.max() <= BOUND[dtype], (f"seed {seed}, {dtype}, {what}, request {rid}: position {int(err.argmax())} is "
                                                   f"off by {err.max():.3e}; configuration {json.dumps(raw)}")
        del eng
