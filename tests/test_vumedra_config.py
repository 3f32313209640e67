"""Configuration of the Vumedra design, its plan and its tensor list, without a GPU; and the plain restatement against
itself (a whole sequence against the same sequence with a token appended; scaled expert inputs against scaled
outputs)."""
import copy
import json

import pytest
import torch

import plain_vumedra as plain
from vumedra_cases import case, random_weights

from esp_b200.cache import KvLayout
from esp_b200.config import config_from_dict, config_from_json
from esp_b200.config.vumedra import VumedraConfig
from esp_b200.errors import InvalidConfig, Unsupported
from esp_b200.weights.random_init import parameter_specs, write_model_folder


def test_registry_finds_the_design_by_its_one_architecture_string():
    cfg = config_from_dict(case("A"))
    assert isinstance(cfg, VumedraConfig)
    assert config_from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()


@pytest.mark.parametrize("name", ["A", "B"])
def test_tensor_names_and_shapes_are_the_designs(name):
    raw = case(name)
    mine = {s.name: tuple(s.shape) for s in parameter_specs(config_from_dict(raw))}
    assert mine == plain.tensor_shapes(raw)


def test_plan_takes_every_size_and_constant_from_the_configuration():
    raw = case("A")
    plan = config_from_dict(raw).plan()
    assert plan.embedding.bigram.buckets == 97 and (plan.embedding.bigram.mul_prev, plan.embedding.bigram.mul_cur) == (13, 5)
    diag, attn, mem, attn2 = (b.mixer for b in plan.blocks)
    assert (diag.channels, diag.blocks, diag.taps) == (72, 3, 4)
    assert (attn.num_heads, attn.num_kv_heads, attn.key_dim, attn.value_dim, attn.scale) == (6, 2, 16, 40, 0.3)
    assert (attn.q_temp.coef, attn.q_temp.every) == (0.4, 7) and attn.sink and attn.qkv_bias
    assert (mem.num_heads, mem.key_dim, mem.value_dim, mem.gate_cap) == (3, 24, 16, 9.0)
    assert attn2.q_temp.every == 50
    moe = plan.blocks[1].ffn
    assert (moe.num_experts, moe.top_k, moe.expert_intermediate, moe.shared_intermediate) == (6, 3, 24, 40)
    assert plan.blocks[2].ffn is None and plan.blocks[2].ffn_norm is None and plan.blocks[2].ffn_post_norm is None
    assert all(b.mixer_norm.eps == 1e-5 and b.mixer_post_norm.kind == "rmsnorm_scalar" for b in plan.blocks)
    b = config_from_dict(case("B")).plan()
    assert b.blocks[0].mixer.q_temp is None and b.blocks[1].ffn.shared_intermediate is None


def test_defaults():
    raw = case("B")
    del raw["layers"][0]["mixer"]["vdim"], raw["layers"][0]["mixer"]["kv_heads"]
    mix = config_from_dict(raw).plan().blocks[0].mixer
    assert (mix.value_dim, mix.num_kv_heads) == (mix.key_dim, mix.num_heads)


def test_keys_and_values_of_different_sizes_in_the_cache_layout():
    lay = KvLayout(2, 16, None, value_dim=40)
    assert lay.row_elements == 2 * (16 + 40)
    assert KvLayout(2, 16).row_elements == 2 * 32 and KvLayout(1, 24, values=False).row_elements == 24


@pytest.mark.parametrize("change, error", [
    (lambda c: c["layers"][0].update(type="conv"), Unsupported),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=4), InvalidConfig),
    (lambda c: c["layers"][0]["mixer"].update(blocks=5), InvalidConfig),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=7), InvalidConfig),
    (lambda c: c["layers"][2]["mixer"].update(gate_cap=0), InvalidConfig),
    (lambda c: c["layers"][0]["mlp"].update(kind="glu"), Unsupported),
    (lambda c: c.pop("embedding"), InvalidConfig),
    (lambda c: c["norm"].update(eps=0), InvalidConfig),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), InvalidConfig),
])
def test_refusals(change, error):
    raw = case("A")
    change(raw)
    with pytest.raises(error):
        config_from_dict(raw)


def test_norms_of_a_missing_feed_forward_may_be_stored():
    from esp_b200.weights.loader import check_names_and_shapes

    class Names:
        def __init__(self, shapes):
            self.shapes = shapes

        def names(self):
            return list(self.shapes)

        def shape(self, n):
            return self.shapes[n]

        def dtype(self, n):
            return torch.bfloat16

    raw = case("A")
    cfg = config_from_dict(raw)
    specs = parameter_specs(cfg)
    shapes = dict(plain.tensor_shapes(raw))
    shapes.update({"l2.norm2": (), "l2.norm2b": ()})          # layer 2 has no feed-forward
    check_names_and_shapes(specs, Names(shapes), cfg.plan().tolerated_suffixes)
    shapes["l2.norm3"] = ()
    from esp_b200.errors import InvalidWeights
    with pytest.raises(InvalidWeights):
        check_names_and_shapes(specs, Names(shapes), cfg.plan().tolerated_suffixes)


def test_random_model_folder_round_trips(tmp_path):
    cfg = config_from_dict(case("B"))
    write_model_folder(cfg, 5, tmp_path)
    again = config_from_json(tmp_path)
    assert again.to_dict() == cfg.to_dict()
    from esp_b200.weights.loader import FolderSource
    src = FolderSource(tmp_path)
    assert {n: src.shape(n) for n in src.names()} == plain.tensor_shapes(case("B"))


@pytest.mark.parametrize("name", ["A", "B"])
def test_plain_restatement_is_causal_and_finite(name):
    raw = case(name)
    w = {k: v.double() for k, v in random_weights(raw, 11).items()}
    toks = [int(t) for t in torch.randint(0, raw["vocab"], (30,), generator=torch.Generator().manual_seed(1))]
    a = plain.forward(raw, w, toks)
    b = plain.forward(raw, w, toks + [3])
    assert torch.isfinite(a).all() and torch.allclose(a, b[:-1], atol=1e-12)


def test_scaling_an_experts_input_is_scaling_its_output_by_the_square():
    raw = case("A")
    w = {k: v.double() for k, v in random_weights(raw, 4).items()}
    h = torch.randn(5, raw["width"], dtype=torch.float64, generator=torch.Generator().manual_seed(2))
    mlp = copy.deepcopy(raw["layers"][1]["mlp"])
    out, chosen = plain.moe_ffn(h, w, "l1.mlp.", mlp)
    s = torch.sigmoid(h @ w["l1.mlp.router"].T)
    want = plain.relu2_expert(h, w, "l1.mlp.shared.")
    for t in range(5):
        assert len(set(chosen[t].tolist())) == 3
        assert min(s[t, chosen[t]]) >= max(s[t, [e for e in range(6) if e not in chosen[t].tolist()]])
        for e in chosen[t].tolist():
            want[t] += s[t, e] ** 2 * plain.relu2_expert(h[t], w, f"l1.mlp.e{e}.")
    assert torch.allclose(out, want, atol=1e-10)
