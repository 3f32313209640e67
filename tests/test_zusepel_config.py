"""Configuration of the Zusepel design, its plan and its tensor list, without a GPU; and the plain restatement
against itself (a whole sequence against the same sequence with a token appended)."""
import copy
import json

import numpy as np
import pytest
import torch

import plain_zusepel as plain
from zusepel_cases import CASE_A, CASE_B, case

from esp_b200.config import config_from_dict, config_from_json
from esp_b200.config.zusepel import ZusepelConfig
from esp_b200.errors import InvalidConfig, Unsupported
from esp_b200.parts import Runtime
from esp_b200.parts.position import RopeScaled
from esp_b200.weights import write_safetensors
from esp_b200.weights.random_init import parameter_specs, write_model_folder


def test_registry_finds_the_design_by_its_one_architecture_string():
    cfg = config_from_dict(case("A")[0])
    assert isinstance(cfg, ZusepelConfig)
    assert config_from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()


@pytest.mark.parametrize("name", ["A", "B"])
def test_tensor_names_and_shapes_are_the_designs(name):
    raw, rank = case(name)
    cfg = config_from_dict(raw)
    cfg.decay_ranks = {i: rank for i, l in enumerate(raw["layers"]) if l["type"] == "wkv"}
    mine = {s.name: tuple(s.shape) for s in parameter_specs(cfg)}
    assert mine == plain.tensor_shapes(raw, rank)


def test_decay_width_comes_from_the_stored_tensor(tmp_path):
    raw, rank = case("A")
    w = plain.random_weights(raw, 3, decay_rank=rank)
    (tmp_path / "config.json").write_text(json.dumps(raw))
    write_safetensors(tmp_path / "model.safetensors", w)
    cfg = config_from_json(tmp_path)
    from esp_b200.weights.loader import FolderSource
    src = FolderSource(tmp_path)
    cfg.bind_shapes({n: src.shape(n) for n in src.names()})
    assert cfg.plan().blocks[0].mixer.decay_rank == rank


def test_plan_shares_caches_and_keeps_the_widest_window():
    plan = config_from_dict(case("A")[0]).plan()
    assert [e.cache_of for e in plan.schedule] == [None, None, None, 1]
    owner, reader = plan.blocks[1].mixer, plan.blocks[3].mixer
    assert (owner.window, reader.window) == (37, 70)
    assert owner.keep_window == reader.keep_window == 70          # the owner's cache must reach as far as its reader looks
    assert owner.own_kv and not reader.own_kv
    assert plan.blocks[1].ffn is None and plan.blocks[1].ffn_norm is None
    plan_b = config_from_dict(case("B")[0]).plan()
    assert plan_b.blocks[0].mixer.keep_window == 1000 and plan_b.blocks[2].mixer.window == 1
    assert plan_b.blocks[0].mixer.position.factor is None


def _broken(change):
    raw = copy.deepcopy(CASE_A)
    change(raw)
    return raw


@pytest.mark.parametrize("change,error", [
    (lambda r: r["layers"][0].update(type="conv"), Unsupported),
    (lambda r: r["layers"][0]["mlp"].update(kind="routed"), Unsupported),
    (lambda r: r["layers"][3]["mixer"].update(kv_from=2), InvalidConfig),        # not an attention layer
    (lambda r: r["layers"][3]["mixer"].update(kv_from=3), InvalidConfig),        # not an earlier layer
    (lambda r: r["layers"][3]["mixer"].update(kv_rank=40), InvalidConfig),       # differs from the owner's
    (lambda r: r["layers"][1]["mixer"]["rot"].update(dims=18), InvalidConfig),   # more than rot_dim
    (lambda r: r["layers"][1]["mixer"].pop("scale"), InvalidConfig),
    (lambda r: r.pop("norm"), InvalidConfig),
    (lambda r: r.update(width=0), InvalidConfig),
    (lambda r: r["layers"][2]["mixer"].pop("dim"), InvalidConfig),
])
def test_refusals(change, error):
    with pytest.raises(error):
        config_from_dict(_broken(change))


@pytest.mark.parametrize("rot", [CASE_A["layers"][1]["mixer"]["rot"], CASE_B["layers"][0]["mixer"]["rot"],
                                 CASE_B["layers"][4]["mixer"]["rot"],
                                 {"base": 1e6, "dims": 64, "scaling": {"factor": 40.0, "fast": 32.0, "original": 4096, "slow": 1.0}}])
def test_interpolated_frequencies_match_the_plain_formula(rot):
    from esp_b200.config.plan import ScaledRopeSpec
    sc = rot.get("scaling")
    spec = ScaledRopeSpec(rot["dims"], rot["base"], *((sc["factor"], sc["original"], sc["fast"], sc["slow"]) if sc else ()))
    f, mag = RopeScaled(spec, Runtime(None, torch.float32)).frequencies()
    pos = torch.tensor([1.0])
    cos, sin = plain.rotary_tables(rot, pos, torch.float64)
    want_mag = float(torch.sqrt(cos[0, 0] ** 2 + sin[0, 0] ** 2))
    assert abs(mag - want_mag) < 1e-12
    np.testing.assert_allclose(np.cos(f.astype(np.float64)) * mag, cos[0].numpy(), rtol=0, atol=1e-12)
    # the ramp really has a flat start, a slope and a flat end where the constants allow it
    if sc and rot["dims"] >= 32:
        plainf = rot["base"] ** (-2.0 * np.arange(rot["dims"] // 2) / rot["dims"])
        ratio = f / plainf
        assert ratio[0] == pytest.approx(1.0) and ratio[-1] == pytest.approx(1.0 / sc["factor"])


def test_random_model_folder_round_trip(tmp_path):
    raw, _ = case("B")
    cfg = config_from_dict(raw)
    folder = write_model_folder(cfg, 5, tmp_path / "m", "bfloat16")
    again = config_from_json(folder)
    assert again.to_dict()["layers"] == cfg.to_dict()["layers"]
    from esp_b200.weights.loader import FolderSource
    src = FolderSource(folder)
    lower = src.metas["l1.mix.lower"]
    from esp_b200.weights.safetensors_io import read_tensor
    t = read_tensor(lower).float()
    assert 0.0 < float(t.mean()) < 1.0          # the role's own initialisation, not a matrix's


def test_plain_prefix_property():
    """Appending a token changes no earlier row (causality of every mixer in the plain restatement)."""
    raw, rank = case("A")
    w = plain.random_weights(raw, 11, decay_rank=rank)
    toks = list(np.random.default_rng(0).integers(0, raw["vocab"], 50))
    a = plain.forward(raw, w, toks)
    b = plain.forward(raw, w, toks[:-7])
    assert float((a[:-7] - b).abs().max()) < 1e-10      # sums of other lengths may differ in their last bits


def test_a_reader_may_leave_out_what_it_shares_with_the_owner():
    raw = copy.deepcopy(CASE_A)
    for key in ("kv_rank", "rot_dim", "rot"):
        raw["layers"][3]["mixer"].pop(key)
    raw.pop("residual_mult")
    cfg = config_from_dict(raw)
    full = config_from_dict(copy.deepcopy(CASE_A))
    assert cfg.plan().blocks[3].mixer == full.plan().blocks[3].mixer
    assert cfg.residual_mult == 1.0
