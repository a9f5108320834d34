"""Host-side pieces of the Bizurax design: its configuration and registry entry, the order in which looped layers run,
the tensors it declares, what its layers ask of the cache manager (pages for the two attentions, a state slot for
retention, one of each per pass of a loop), and two identities of the plain implementation: retention's recurrence
against its sum over all earlier tokens, and the rotation of neighbour pairs against the rotation of halves on
reordered elements."""

from __future__ import annotations

import copy

import pytest
import torch

import plain_bizurax as plain
from mini_engine_b200.cache.storage import plan_groups
from mini_engine_b200.config import BizuraxConfig, load_model_config
from mini_engine_b200.config.qwen3 import ConfigError
from mini_engine_b200.config.registry import architecture_for
from mini_engine_b200.parts.base import PagedCacheSpec, StateSpec
from mini_engine_b200.parts.model import DecoderModel, declared_weights
from mini_engine_b200.weights import write_random_model


def raw_config():
    return copy.deepcopy({
        "architecture": "Bizurax", "vocab": 90, "width": 48, "norm": {"eps": 2e-5}, "residual_mult": 0.7, "streams": 3,
        "loop": {"start": 1, "stop": 3, "times": 2},
        "layers": [
            {"type": "latent_attention", "mlp": {"kind": "dense", "ff": 40},
             "mixer": {"heads": 3, "dim": 16, "rot_dim": 8, "vdim": 24, "kv_rank": 20, "scale": 0.2, "rot": {"base": 300.0, "dims": 8}}},
            {"type": "retention", "mlp": {"kind": "moe", "expert": {"ff": 16}, "router": {"experts": 5, "top": 2}, "shared": {"ff": 24}},
             "mixer": {"heads": 3, "dim": 16, "vdim": 24, "decay": [0.9, 0.99, 1.0], "rot": {"base": 1000.0, "dims": 8}}},
            {"type": "attention", "mlp": None,
             "mixer": {"heads": 6, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 4.0, "softcap": 3.0,
                       "rot": {"base": 500.0, "dims": 12, "scaling": {"factor": 2.0}}}},
            {"type": "attention", "mlp": {"kind": "moe", "expert": {"ff": 24}, "router": {"experts": 4, "top": 1}},
             "mixer": {"heads": 2, "kv_heads": 2, "dim": 24, "vdim": 8, "scale": 6.0, "rot": {"base": 10000.0, "dims": 24}}},
        ],
    })  # fmt: skip


def test_config_round_trip_and_registry(tmp_path):
    cfg = BizuraxConfig.from_dict(raw_config())
    assert BizuraxConfig.from_dict(cfg.to_dict()) == cfg and cfg.to_dict() == raw_config()
    assert cfg.layer_order() == [0, 1, 2, 1, 2, 3] == plain.layer_order(raw_config())
    assert cfg.layers[2].mixer.rot.factor == 2.0 and cfg.layers[1].mixer.rot.factor == 1.0 and cfg.layers[3].mixer.softcap is None
    assert cfg.layers[1].mlp.shared_ff == 24 and cfg.layers[3].mlp.shared_ff == 0 and cfg.layers[2].mlp is None
    assert cfg.layers[1].mixer.decay == (0.9, 0.99, 1.0) and cfg.streams == 3 and cfg.residual_mult == 0.7
    write_random_model(tmp_path, cfg, seed=1)
    arch, loaded = load_model_config(tmp_path)
    assert arch.name == "Bizurax" and loaded == cfg


@pytest.mark.parametrize(
    "path,value,message",
    [
        (("layers", 0, "type"), "conv", "not a mixer"),
        (("layers", 2, "mixer", "heads"), 5, "multiple of kv_heads"),
        (("layers", 0, "mixer", "rot", "dims"), 10, "dims"),
        (("layers", 2, "mixer", "rot", "dims"), 3, "dims"),
        (("layers", 2, "mixer", "rot", "scaling"), {"factor": 0}, "positive"),
        (("layers", 0, "mixer", "kv_rank"), 0, "positive"),
        (("layers", 1, "mixer", "decay"), [0.9, 0.99], "one number"),
        (("layers", 1, "mixer", "decay"), [0.9, 0.99, 1.5], "one number"),
        (("layers", 1, "mlp", "router", "top"), 6, "router.top"),
        (("layers", 0, "mlp", "kind"), "gated", "not a feed-forward"),
        (("layers", 2, "mixer", "softcap"), -1.0, "softcap"),
        (("loop",), {"start": 2, "stop": 2, "times": 2}, "loop"),
        (("loop",), {"start": 0, "stop": 5, "times": 2}, "loop"),
        (("streams",), 0, "streams"),
        (("norm",), None, "lacks the key"),
    ],
)
def test_config_errors_name_the_key(path, value, message):
    raw = raw_config()
    at = raw
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    with pytest.raises(ConfigError, match=message):
        BizuraxConfig.from_dict(raw)


def test_optional_keys_may_be_absent():
    raw = raw_config()
    del raw["loop"], raw["streams"], raw["residual_mult"]
    cfg = BizuraxConfig.from_dict(raw)
    assert cfg.loop is None and cfg.streams is None and cfg.residual_mult == 1.0 and cfg.layer_order() == [0, 1, 2, 3]
    spec = architecture_for("Bizurax").build_spec(cfg)
    assert [layer.block for layer in spec.layers] == ["prenorm", "prenorm", "prenorm_mixer_only", "prenorm"]
    assert not any(".hc" in s.name for s in declared_weights(spec))


def test_a_checkpoint_may_carry_the_tensors_of_a_feed_forward_that_a_layer_does_not_have(tmp_path):
    from mini_engine_b200.weights.loader import check_specs
    from mini_engine_b200.weights.safetensors_io import SafetensorsFile, write_safetensors

    cfg = BizuraxConfig.from_dict(raw_config())
    write_random_model(tmp_path, cfg, seed=1)
    stored = SafetensorsFile(tmp_path / "model.safetensors")
    assert "l2.norm2" not in stored.entries
    tensors = {name: stored.tensor(name).clone() for name in stored.entries}
    tensors.update({"l2.norm2": torch.ones(48, dtype=torch.bfloat16), "l2.hc2.in": torch.ones(3, dtype=torch.bfloat16),
                    "l2.hc2.out": torch.ones(3, dtype=torch.bfloat16), "l2.hc2.mix": torch.eye(3, dtype=torch.bfloat16)})  # fmt: skip
    write_safetensors(tmp_path / "more.safetensors", tensors)
    specs = declared_weights(architecture_for("Bizurax").build_spec(cfg))
    check_specs(specs, SafetensorsFile(tmp_path / "more.safetensors").entries)  # nothing is unexpected
    check_specs(specs, stored.entries)  # and nothing is missing without them


def test_declared_tensors():
    spec = architecture_for("Bizurax").build_spec(BizuraxConfig.from_dict(raw_config()))
    declared = {s.name: s for s in declared_weights(spec)}
    assert declared["embed"].shape == (90, 48) and declared["head"].shape == (90, 48) and declared["head"].alias_of is None
    assert declared["final.norm"].shape == (48,) and declared["l1.norm2"].shape == (48,) and not declared["l1.norm2"].optional
    for sub in ("hc1", "hc2"):
        assert declared[f"l0.{sub}.in"].shape == (3,) and declared[f"l0.{sub}.out"].shape == (3,) and declared[f"l0.{sub}.mix"].shape == (3, 3)
        assert declared[f"l0.{sub}.mix"].role == "vector"
    # a layer without feed-forward has one set; a checkpoint may carry the other set and its norm all the same
    assert "l2.hc1.in" in declared and all(declared[f"l2.{name}"].optional for name in ("norm2", "hc2.in", "hc2.mix", "hc2.out"))
    assert declared["l0.mix.q"].shape == (72, 48) and declared["l0.mix.dkv"].shape == (28, 48) and declared["l0.mix.dkv.norm"].shape == (20,)
    assert declared["l0.mix.uk"].shape == (48, 20) and declared["l0.mix.uv"].shape == (72, 20) and "l0.mix.dq" not in declared
    assert declared["l1.mix.q"].shape == (48, 48) and declared["l1.mix.v"].shape == (72, 48) and declared["l1.mix.g"].shape == (72, 48)
    assert declared["l1.mix.o"].shape == (48, 72) and "l1.mix.q.b" not in declared
    assert declared["l2.mix.q.b"].shape == (96,) and declared["l2.mix.k.b"].shape == (32,) and declared["l2.mix.v.b"].shape == (48,)
    assert declared["l2.mix.sink"].shape == (6,) and declared["l2.mix.sink"].role == "vector" and declared["l2.mix.o"].shape == (48, 144)
    assert declared["l0.mlp.up"].shape == (40, 48) and declared["l0.mlp.down"].shape == (48, 40) and "l0.mlp.gate" not in declared
    assert declared["l1.mlp.router"].shape == (5, 48) and declared["l1.mlp.router"].role == "vector" and declared["l1.mlp.router.b"].shape == (5,)
    assert declared["l1.mlp.e4.gate"].shape == (16, 48) and declared["l1.mlp.e0.down"].shape == (48, 16) and "l1.mlp.e5.up" not in declared
    assert declared["l1.mlp.shared.up"].shape == (24, 48) and declared["l1.mlp.shared.down"].shape == (48, 24)
    assert "l3.mlp.shared.up" not in declared and declared["l3.mlp.e3.up"].shape == (24, 48)
    assert [(entry.layer, entry.cache_of) for entry in spec.order] == [(0, None), (1, None), (2, None), (1, None), (2, None), (3, None)]


def test_every_pass_of_a_loop_has_a_cache_or_a_state_of_its_own():
    model = DecoderModel(architecture_for("Bizurax").build_spec(BizuraxConfig.from_dict(raw_config())))
    needs = model.cache_needs()
    assert needs[0] == (PagedCacheSpec(1, 28, None, 0, 0), None, None)
    assert needs[1] == needs[3] == (None, StateSpec((3, 16, 24), torch.float32), None)
    assert needs[2] == needs[4] == (PagedCacheSpec(2, 16, None, 24, 0), None, None)
    assert needs[5][0] == PagedCacheSpec(2, 24, None, 8, 0)
    specs, group_of = plan_groups(needs)
    assert group_of[2] == group_of[4] and len({group_of[0], group_of[2], group_of[5]}) == 3 and group_of[1] is None
    assert model.embedding_state() is None and model.capturable


def test_plain_retention_equals_the_sum_over_earlier_tokens():
    """o_t = sum_(j <= t) a^(t - j) (q_t . k_j) v_j: the recurrence is linear attention with a decaying weight."""
    torch.manual_seed(0)
    m = {"heads": 2, "dim": 6, "vdim": 5, "decay": [0.9, 0.5], "rot": {"base": 100.0, "dims": 4, "scaling": {"factor": 2.0}}}
    hidden, tokens, eps = 10, 17, 1e-5
    w = {"m." + k: torch.randn(s, dtype=torch.float64) for k, s in {"q": (12, hidden), "k": (12, hidden), "v": (10, hidden), "g": (10, hidden), "o": (hidden, 10)}.items()}
    h = torch.randn(tokens, hidden, dtype=torch.float64)
    want, state = plain.retention(h, w, "m.", m, eps)
    positions = torch.arange(tokens)
    q = plain.rotate((h @ w["m.q"].T).view(tokens, 2, 6), positions, m["rot"], False)
    k = plain.rotate((h @ w["m.k"].T).view(tokens, 2, 6), positions, m["rot"], False) * 6**-0.5
    v = (h @ w["m.v"].T).view(tokens, 2, 5)
    distance = (positions.view(-1, 1) - positions.view(1, -1)).clamp(min=0).double()
    weight = torch.tensor(m["decay"]).double().view(2, 1, 1) ** distance * plain.causal(tokens)
    o = torch.einsum("hij,jhe->ihe", torch.einsum("ihd,jhd->hij", q, k) * weight, v)
    gate = h @ w["m.g"].T
    out = (plain.rms_norm(o, None, eps).reshape(tokens, 10) * gate * torch.sigmoid(gate)) @ w["m.o"].T
    assert torch.allclose(out, want, atol=1e-10)
    # in two portions, from the carried state
    first, held = plain.retention(h[:7], w, "m.", m, eps)
    second, last = plain.retention(h[7:], w, "m.", m, eps, state=held, start=7)
    assert torch.allclose(torch.cat((first, second)), want, atol=1e-12) and torch.allclose(last, state, atol=1e-12)


def test_neighbour_pairs_are_halves_of_reordered_elements():
    """Rotating pairs (2 i, 2 i + 1) of q and k equals rotating halves of the same elements reordered to [even | odd]:
    the scores, which is all that the rotated parts enter, are the same."""
    torch.manual_seed(1)
    rotation = {"base": 50.0, "dims": 8}
    q, k = torch.randn(9, 3, 8, dtype=torch.float64), torch.randn(9, 8, dtype=torch.float64)
    positions = torch.arange(9)
    order = torch.cat((torch.arange(0, 8, 2), torch.arange(1, 8, 2)))
    pairs = torch.einsum("ihd,jd->hij", plain.rotate(q, positions, rotation, True), plain.rotate(k, positions, rotation, True))
    halves = torch.einsum("ihd,jd->hij", plain.rotate(q[..., order], positions, rotation, False), plain.rotate(k[..., order], positions, rotation, False))
    assert torch.allclose(pairs, halves, atol=1e-12)
