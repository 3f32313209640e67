"""Small configurations of the Zusepel design for the tests.  They differ from one another in every size, in the
order of the layers, and in which options are present."""
import copy

ROT_A = {"base": 10000.0, "dims": 16, "scaling": {"factor": 4.0, "fast": 16.0, "original": 64, "slow": 2.0}}
ROT_B = {"base": 500.0, "dims": 8, "scaling": None}

# every mixer once, unequal key and value sizes, head counts that are no power of two, a reader of another layer's
# cache with a wider window than the owner's, a layer without feed-forward
CASE_A = {
    "architecture": "Zusepel", "vocab": 301, "width": 96, "norm": {"eps": 1e-5}, "residual_mult": 0.6,
    "layers": [
        {"type": "wkv", "mixer": {"heads": 2, "dim": 48}, "mlp": {"kind": "dense", "ff": 80}},
        {"type": "latent_attention", "mixer": {"heads": 6, "dim": 40, "rot_dim": 16, "vdim": 24, "q_rank": 40, "kv_rank": 48,
                                               "scale": 0.17, "mask": {"size": 37}, "rot": ROT_A}, "mlp": None},
        {"type": "hgrn2", "mixer": {"heads": 3, "dim": 24, "vdim": 40}, "mlp": {"kind": "dense", "ff": 136}},
        {"type": "latent_attention", "mixer": {"heads": 3, "dim": 24, "rot_dim": 16, "vdim": 56, "q_rank": 32, "kv_rank": 48,
                                               "scale": 0.11, "mask": {"size": 70}, "rot": ROT_A, "kv_from": 1},
         "mlp": {"kind": "dense", "ff": 64}},
    ],
}
DECAY_A = 12

# attention first, a width that is no multiple of 8, one head, a window of one position (the query alone), a
# window longer than any test sequence, plain rotary frequencies, large heads in the recurrences
CASE_B = {
    "architecture": "Zusepel", "vocab": 97, "width": 100, "norm": {"eps": 1e-6}, "residual_mult": 1.3,
    "layers": [
        {"type": "latent_attention", "mixer": {"heads": 1, "dim": 16, "rot_dim": 8, "vdim": 16, "q_rank": 24, "kv_rank": 24,
                                               "scale": 0.3, "mask": {"size": 1000}, "rot": ROT_B},
         "mlp": {"kind": "dense", "ff": 44}},
        {"type": "hgrn2", "mixer": {"heads": 1, "dim": 128, "vdim": 72}, "mlp": None},
        {"type": "latent_attention", "mixer": {"heads": 5, "dim": 8, "rot_dim": 8, "vdim": 8, "q_rank": 16, "kv_rank": 24,
                                               "scale": 0.5, "mask": {"size": 1}, "rot": ROT_B, "kv_from": 0},
         "mlp": {"kind": "dense", "ff": 32}},
        {"type": "wkv", "mixer": {"heads": 1, "dim": 128}, "mlp": {"kind": "dense", "ff": 60}},
        {"type": "latent_attention", "mixer": {"heads": 2, "dim": 32, "rot_dim": 32, "vdim": 48, "q_rank": 8, "kv_rank": 136,
                                               "scale": 0.2, "mask": {"size": 64},
                                               "rot": {"base": 10000.0, "dims": 32,
                                                       "scaling": {"factor": 16.0, "fast": 8.0, "original": 256, "slow": 0.5}}},
         "mlp": None},
    ],
}
DECAY_B = 5

CASES = {"A": (CASE_A, DECAY_A), "B": (CASE_B, DECAY_B)}


def case(name):
    cfg, rank = CASES[name]
    return copy.deepcopy(cfg), rank
