"""Small configurations of the Vumedra design for the tests.  They differ from one another in every size, in the
order of the layers and in which options are present; none has a size equal to another size by accident."""
import copy

import torch

import plain_vumedra as plain

# every mixer and both feed-forwards; two key/value heads under six query heads; values wider than keys; three
# experts a token; a temperature step every 7 positions, so that short tests pass many steps; three blocks; four taps
CASE_A = {
    "architecture": "Vumedra", "vocab": 211, "width": 96, "norm": {"eps": 1e-5},
    "embedding": {"bigram": {"buckets": 97, "mul_prev": 13, "mul_cur": 5}},
    "layers": [
        {"type": "rglru", "mixer": {"width": 72, "blocks": 3, "conv": 4}, "mlp": {"kind": "dense", "ff": 136}},
        {"type": "attention", "mixer": {"heads": 6, "kv_heads": 2, "dim": 16, "vdim": 40, "scale": 0.3,
                                        "q_temp": {"coef": 0.4, "every": 7}},
         "mlp": {"kind": "moe", "router": {"experts": 6, "top": 3}, "expert": {"ff": 24}, "shared": {"ff": 40}}},
        {"type": "mlstm", "mixer": {"heads": 3, "dim": 24, "vdim": 16, "gate_cap": 9.0}, "mlp": None},
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 72, "vdim": 8, "scale": 0.08,
                                        "q_temp": {"coef": 0.9, "every": 50}},
         "mlp": {"kind": "dense", "ff": 64}},
    ],
}

# attention first; a width that is no multiple of 8; one head; head sizes that the tensor-core attention does not take
# (20) and that it pads (24 / 104); one block; one tap (no convolution state); every expert chosen; no shared expert;
# no temperature; key and value sizes equal; 2 taps; a matrix memory with one head of 40 x 12
CASE_B = {
    "architecture": "Vumedra", "vocab": 97, "width": 100, "norm": {"eps": 1e-6},
    "embedding": {"bigram": {"buckets": 1000, "mul_prev": 1, "mul_cur": 99991}},
    "layers": [
        {"type": "attention", "mixer": {"heads": 1, "kv_heads": 1, "dim": 20, "vdim": 20, "scale": 0.5}, "mlp": None},
        {"type": "mlstm", "mixer": {"heads": 1, "dim": 40, "vdim": 12, "gate_cap": 15.0},
         "mlp": {"kind": "moe", "router": {"experts": 3, "top": 3}, "expert": {"ff": 16}, "shared": None}},
        {"type": "rglru", "mixer": {"width": 56, "blocks": 1, "conv": 1}, "mlp": None},
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 1, "dim": 24, "vdim": 104, "scale": 0.2,
                                        "q_temp": {"coef": 0.25, "every": 1}},
         "mlp": {"kind": "moe", "router": {"experts": 5, "top": 1}, "expert": {"ff": 8}, "shared": {"ff": 8}}},
        {"type": "rglru", "mixer": {"width": 64, "blocks": 8, "conv": 2}, "mlp": {"kind": "dense", "ff": 48}},
        {"type": "mlstm", "mixer": {"heads": 5, "dim": 8, "vdim": 24, "gate_cap": 6.0}, "mlp": {"kind": "dense", "ff": 32}},
    ],
}

CASES = {"A": CASE_A, "B": CASE_B}


def case(name):
    return copy.deepcopy(CASES[name])


def one_layer(layer, width=64, vocab=131):
    """A model of a single layer: one mechanism alone between the embeddings and the head."""
    return {"architecture": "Vumedra", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
            "embedding": {"bigram": {"buckets": 53, "mul_prev": 3, "mul_cur": 11}}, "layers": [copy.deepcopy(layer)]}


def random_weights(cfg, seed, dtype=torch.bfloat16):
    """Weights that make every mechanism matter: gates that open and close, decays on both sides, biases, norm
    weights away from one.  Returned as stored (``dtype``)."""
    g = torch.Generator().manual_seed(seed)
    rnd = lambda shape, std, mean=0.0: torch.randn(shape, generator=g) * std + mean
    out = {}
    for name, shape in plain.tensor_shapes(cfg).items():
        leaf = name.split(".", 1)[1] if name[0] == "l" and "." in name else name
        if shape == ():
            t = rnd((), 0.15, 1.0)
        elif leaf in ("mix.q.norm", "mix.k.norm", "mix.norm"):
            t = rnd(shape, 0.2, 1.0)
        elif leaf == "mix.f.b":
            t = rnd(shape, 1.5, 2.0)
        elif leaf == "mix.i.b":
            t = rnd(shape, 1.0, -3.0)
        elif leaf in ("mix.i", "mix.f"):
            t = rnd(shape, 0.2)
        elif leaf == "mix.lam":
            t = rnd(shape, 1.5, -1.0)
        elif leaf == "mix.conv":
            t = rnd(shape, 0.5)
        elif leaf in ("mix.ra", "mix.ri"):
            t = rnd(shape, 2.0 / shape[-1] ** 0.5)
        elif leaf.endswith(".b"):
            t = rnd(shape, 0.3)
        elif leaf.endswith("router"):
            t = rnd(shape, 0.5)
        elif name in ("embed", "bigram"):
            t = rnd(shape, 0.7)
        else:
            t = rnd(shape, 1.2 / shape[-1] ** 0.5)
        out[name] = t.to(dtype)
    # A matrix memory divides by max(|n . q|, exp(-m)): with keys unrelated to queries that sum of products often nearly
    # cancels and magnifies the rounding of 32-bit terms a hundredfold, in any implementation.  Keys that lean towards
    # the queries, as trained ones do, keep the quotient well conditioned.
    for i, layer in enumerate(cfg["layers"]):
        if layer["type"] == "mlstm":
            q, k = out[f"l{i}.mix.q"].float(), out[f"l{i}.mix.k"].float()
            out[f"l{i}.mix.k"] = (0.8 * q + 0.6 * k).to(dtype)
    return out
