"""Host-side pieces of the Bevadra design: its configuration and registry entry, the tensors it declares, the cache
groups its layers ask for (a latent layer keeps one row per token that is key and value at once), the block that
hands on an output bias, and the plain implementation's two ways of writing the latent layer."""

from __future__ import annotations

import copy

import pytest
import torch

import plain_bevadra as plain
from mini_engine_b200.cache.storage import bytes_per_token, plan_groups
from mini_engine_b200.config import BevadraConfig, load_model_config
from mini_engine_b200.config.qwen3 import ConfigError
from mini_engine_b200.parts.base import PagedCacheSpec
from mini_engine_b200.parts.model import DecoderModel, declared_weights
from mini_engine_b200.weights import write_random_model


def attention(window=20, kv_from=None, heads=6, kv_heads=2, dim=16, vdim=24):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": 0.2, "mask": {"size": window}}
    if kv_from is not None:
        out["kv_from"] = kv_from
    return out


def latent(window=19):
    return {"heads": 3, "dim": 16, "rot_dim": 8, "vdim": 24, "kv_rank": 20, "q_rank": 28, "scale": 0.2,
            "mask": {"size": window}, "rot": {"base": 300.0, "dims": 8}}  # fmt: skip


def raw_config():
    return copy.deepcopy({
        "architecture": "Bevadra", "vocab": 90, "width": 48, "norm": {"eps": 2e-5}, "logit_softcap": 6.0,
        "layers": [
            {"type": "latent_attention", "mixer": latent(), "mlp": {"kind": "dense", "ff": 40}},
            {"type": "attention", "mixer": attention(), "mlp": {"kind": "dense", "ff": 24}},
            {"type": "attention", "mixer": attention(window=33, kv_from=1), "mlp": None},
            {"type": "latent_attention", "mixer": latent(), "mlp": None},
        ],
    })  # fmt: skip


def test_config_round_trip_and_registry(tmp_path):
    cfg = BevadraConfig.from_dict(raw_config())
    assert BevadraConfig.from_dict(cfg.to_dict()) == cfg and cfg.to_dict() == raw_config()
    assert cfg.layers[2].mixer.kv_from == 1 and cfg.layers[2].mlp is None and cfg.layers[0].mixer.kv_rank == 20
    assert cfg.layers[0].mixer.rot_dims == 8 and cfg.logit_softcap == 6.0 and cfg.layers[1].mlp.ff == 24
    write_random_model(tmp_path, cfg, seed=1)
    arch, loaded = load_model_config(tmp_path)
    assert arch.name == "Bevadra" and loaded == cfg


@pytest.mark.parametrize(
    "path,value,message",
    [
        (("layers", 0, "type"), "conv", "not a mixer"),
        (("layers", 2, "mixer", "kv_from"), 0, "earlier attention layer"),
        (("layers", 2, "mixer", "kv_from"), 2, "earlier attention layer"),
        (("layers", 2, "mixer", "dim"), 32, "do not fit"),
        (("layers", 1, "mixer", "heads"), 5, "multiple of kv_heads"),
        (("layers", 0, "mixer", "rot", "dims"), 10, "rot.dims"),
        (("layers", 0, "mixer", "rot", "dims"), 3, "rot.dims"),
        (("layers", 0, "mixer", "kv_rank"), 0, "positive"),
        (("layers", 0, "mixer", "q_rank"), None, "lacks the key"),
        (("layers", 0, "mlp", "kind"), "moe", "not a feed-forward"),
        (("layers", 1, "mixer", "mask", "size"), 0, "positive"),
        (("logit_softcap",), -1.0, "logit_softcap"),
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
        BevadraConfig.from_dict(raw)


def test_optional_keys_may_be_absent():
    raw = raw_config()
    del raw["logit_softcap"], raw["layers"][1]["mixer"]["mask"], raw["layers"][3]["mixer"]["mask"]
    cfg = BevadraConfig.from_dict(raw)
    assert cfg.logit_softcap is None and cfg.layers[1].mixer.window is None and cfg.layers[3].mixer.window is None
    assert "logit_softcap" not in cfg.to_dict()


def test_declared_tensors():
    from mini_engine_b200.config.registry import architecture_for

    spec = architecture_for("Bevadra").build_spec(BevadraConfig.from_dict(raw_config()))
    declared = {s.name: s for s in declared_weights(spec)}
    assert declared["embed"].shape == (90, 48) and declared["head.tied"].alias_of == "embed"
    assert declared["l1.norm1"].shape == (48,) and declared["l1.norm1.b"].role == "vector" and "l1.norm2" not in declared
    assert declared["final.norm.b"].shape == (48,)
    assert declared["l1.mix.q.b"].shape == (96,) and declared["l1.mix.k.b"].shape == (32,) and declared["l1.mix.v.b"].shape == (48,)
    assert declared["l1.mix.g"].shape == (144, 48) and declared["l1.mix.o"].shape == (48, 144) and declared["l1.mix.o.b"].shape == (48,)
    assert declared["l1.mix.sink"].shape == (6,) and declared["l1.mix.sink"].role == "vector"
    # a layer that reads another layer's keys and values has none of their tensors
    assert "l2.mix.q" in declared and not any(name in declared for name in ("l2.mix.k", "l2.mix.v", "l2.mix.k.b", "l2.mix.v.b"))
    assert "l2.mlp.gate" not in declared and declared["l1.mlp.down"].shape == (48, 24)
    assert declared["l0.mix.dq"].shape == (28, 48) and declared["l0.mix.dq.norm"].shape == (28,) and declared["l0.mix.uq"].shape == (72, 28)
    assert declared["l0.mix.dkv"].shape == (28, 48) and declared["l0.mix.dkv.norm"].shape == (20,)
    assert declared["l0.mix.uk"].shape == (48, 20) and declared["l0.mix.uv"].shape == (72, 20)
    assert declared["l0.mix.g"].shape == (3, 48) and declared["l0.mix.o"].shape == (48, 72) and "l0.mix.o.b" not in declared
    assert spec.order[2].cache_of == 1 and spec.order[3].cache_of is None


def test_cache_groups_latent_rows_and_a_reader_with_a_wider_window():
    from mini_engine_b200.config.registry import architecture_for

    model = DecoderModel(architecture_for("Bevadra").build_spec(BevadraConfig.from_dict(raw_config())))
    needs = model.cache_needs()
    # one row of kv_rank + rot_dim per token, which is key and value at once: no value pages
    assert needs[0][0] == PagedCacheSpec(1, 28, 19, 0, 0) and needs[0][0].v_dim == 0 and needs[0][1] is None
    assert needs[1][0] == PagedCacheSpec(2, 16, 20, 24, 0) and needs[2][0].window == 33 and needs[2][2] == 1
    specs, group_of = plan_groups(needs)
    # layer 1 keeps its pages for the wider window of its reader; the two latent layers share a group
    assert group_of == [0, 1, 1, 0] and specs[1].window == 33 and specs[0].window == 19
    assert bytes_per_token(needs, torch.bfloat16) == 2 * (2 * 28 + 2 * (16 + 24))
    assert model.embedding_state() is None and model.capturable and model.programmatic_launch


def test_an_output_bias_needs_a_block_that_adds_it():
    from mini_engine_b200.config.model_spec import LayerSpec, PartSpec
    from mini_engine_b200.parts.model import build_block
    from types import SimpleNamespace

    mixer = PartSpec("gqa_attention", {"num_heads": 2, "kv_heads": 1, "head_dim": 16, "position_encoding": None, "o_bias": True})
    norm = PartSpec("rmsnorm", {"name": "n", "eps": 1e-5})
    layer = LayerSpec(prefix="l0.", block="prenorm", mixer=mixer, feed_forward=PartSpec("gated_mlp", {"intermediate_size": 8}),
                      mixer_norm=norm, feed_forward_norm=norm)  # fmt: skip
    with pytest.raises(ValueError, match="does not add the bias"):
        build_block(SimpleNamespace(layers=[layer], hidden_size=32), 0)
    layer = LayerSpec(prefix="l0.", block="parallel", mixer=mixer, feed_forward=None, mixer_norm=PartSpec("layernorm", {"name": "n", "eps": 1e-5}))
    block = build_block(SimpleNamespace(layers=[layer], hidden_size=32), 0)
    assert {s.name for s in block.weight_specs()} >= {"l0.o_proj.bias", "l0.n", "l0.n.b"}


def test_plain_latent_layer_equals_its_form_with_the_maps_on_the_query_side():
    """The plain layer expands keys and values per head; the engine applies the two maps to the query and to the
    averaged latent instead.  Both are the same function."""
    torch.manual_seed(0)
    m = {"heads": 3, "dim": 6, "rot_dim": 4, "vdim": 5, "kv_rank": 7, "q_rank": 9, "scale": 0.3, "mask": {"size": 11}, "rot": {"base": 100.0, "dims": 4}}
    hidden, T, eps = 10, 30, 1e-5
    shapes = {"dq": (9, hidden), "dq.norm": (9,), "uq": (30, 9), "dkv": (11, hidden), "dkv.norm": (7,), "uk": (18, 7), "uv": (15, 7),
              "g": (3, hidden), "o": (hidden, 15)}  # fmt: skip
    w = {"m." + k: torch.randn(s, dtype=torch.float64) for k, s in shapes.items()}
    h = torch.randn(T, hidden, dtype=torch.float64)
    want = plain.latent_attention(h, w, "m.", m, eps)
    positions = torch.arange(T)
    q = (plain.rms_norm(h @ w["m.dq"].T, w["m.dq.norm"], eps) @ w["m.uq"].T).view(T, 3, 10)
    down = h @ w["m.dkv"].T
    row = torch.cat((plain.rms_norm(down[:, :7], w["m.dkv.norm"], eps), plain.rotate_half(down[:, 7:], positions, 100.0, 4)), dim=-1)
    mapped = torch.cat((torch.einsum("thd,hdr->thr", q[..., :6], w["m.uk"].view(3, 6, 7)), plain.rotate_half(q[..., 6:], positions, 100.0, 4)), dim=-1)
    scores = torch.einsum("ihk,jk->hij", mapped, row) * 0.3
    weights = plain.softmax_with_extra(scores, plain.window_mask(T, 11, h))
    mean = torch.einsum("hij,jr->ihr", weights, row[:, :7]) * torch.sigmoid(h @ w["m.g"].T).unsqueeze(-1)
    out = torch.einsum("ihr,hvr->ihv", mean, w["m.uv"].view(3, 5, 7)).reshape(T, 15) @ w["m.o"].T
    assert torch.allclose(out, want, atol=1e-10)
