"""The Lodalix configuration reader, its model description, its tensor names and the rotary
frequencies of its position encoding (no GPU)."""

import copy
import math

import pytest
import torch

import plain_lodalix as plain
from cloud_inference_from_scratch_b200 import models, parts  # noqa: F401  (registries)
from cloud_inference_from_scratch_b200.config import ConfigError, LodalixConfig, resolve_config
from cloud_inference_from_scratch_b200.models import DecoderModel


def raw_config():
    rot1 = dict(base=50000.0, dims=4)
    rot2 = dict(base=3000.0, dims=8, scaling=dict(factor=4.0, original=64, fast=8.0, slow=0.5))
    first = dict(heads=3, dim=8, rot_dim=4, vdim=10, kv_rank=24, q_rank=12, scale=0.3, rot=rot1)
    second = dict(heads=2, dim=4, rot_dim=8, vdim=6, kv_rank=16, q_rank=20, scale=0.25, rot=rot2)
    mlp = dict(kind="dense", ff=14, limit=2.5)
    return dict(architecture="Lodalix", vocab=50, width=24, norm=dict(eps=1e-5),
                layers=[dict(type="general_delta", mixer=dict(heads=2, dim=6, decay_rank=5), mlp=mlp),
                        dict(type="latent_attention_2", mixer=second, mlp=None),
                        dict(type="latent_attention", mixer=first, mlp=mlp),
                        dict(type="latent_attention_2", mixer=dict(second, heads=5, vdim=3, kv_from=1), mlp=mlp)])


def test_reads_back_what_it_wrote_and_is_found_by_its_name():
    arch, config, spec = resolve_config(raw_config())
    assert arch.name == "Lodalix" and isinstance(config, LodalixConfig)
    assert LodalixConfig.from_dict(config.to_dict()) == config
    assert [(entry.layer, entry.reads_cache_of) for entry in spec.schedule] == [(0, None), (1, None), (2, None), (3, 1)]
    assert spec.residual_streams == 1 and spec.position_tensor is None


def test_tensor_names_shapes_and_caches():
    _, _, spec = resolve_config(raw_config())
    model = DecoderModel(spec)
    table = model.tensor_table()
    assert table["embed"].shape == (50, 24) and table["head"].shape == (50, 24) and table["final.norm"].shape == (24,)
    assert table["l0.norm1"].shape == (24,) and "l0.norm2" not in table
    for name in "rkvga":
        assert table[f"l0.mix.{name}"].shape == (12, 24)
    assert table["l0.mix.a.b"].shape == (12,) and table["l0.mix.w0"].shape == (12,) and table["l0.mix.norm"].shape == (12,)
    assert table["l0.mix.w1"].shape == (5, 24) and table["l0.mix.w2"].shape == (12, 5) and table["l0.mix.o"].shape == (24, 12)
    assert table["l0.mlp.gate"].shape == (14, 24) and table["l0.mlp.up.b"].shape == (14,) and table["l0.mlp.down.b"].shape == (24,)
    assert not any(name.startswith("l1.mlp") for name in table)
    assert table["l1.mix.dq"].shape == (20, 24) and table["l1.mix.dq.norm"].shape == (20,) and table["l1.mix.uq"].shape == (24, 20)
    assert table["l1.mix.dkv"].shape == (24, 24) and table["l1.mix.dkv.norm"].shape == (16,)
    assert table["l1.mix.uk"].shape == (8, 16) and table["l1.mix.uv"].shape == (12, 16)
    assert table["l1.mix.g"].shape == (12, 24) and table["l1.mix.o"].shape == (24, 12) and "l1.mix.sink" not in table
    assert table["l2.mix.sink"].shape == (3,) and "l2.mix.g" not in table and table["l2.mix.uq"].shape == (36, 12)
    assert table["l2.mix.dkv"].shape == (28, 24) and table["l2.mix.uv"].shape == (30, 24)
    # the layer that reads another layer's latent has neither the down projection nor its norm
    assert "l3.mix.dkv" not in table and "l3.mix.dkv.norm" not in table
    assert table["l3.mix.uk"].shape == (20, 16) and table["l3.mix.uv"].shape == (15, 16) and table["l3.mix.g"].shape == (15, 24)
    needs = model.cache_needs()
    assert [need.owner for need in needs] == [0, 1, 2, 1]
    assert needs[0].pages is None and needs[0].state.shape == (2, 6, 6)
    assert (needs[1].pages.kv_heads, needs[1].pages.head_dim, needs[1].pages.value_size, needs[1].pages.window) == (1, 16, 8, 0)
    assert needs[2].pages.head_dim == 24 and needs[2].pages.value_size == 4 and needs[3].pages == needs[1].pages


def test_the_decay_width_may_be_left_to_the_file():
    from cloud_inference_from_scratch_b200.weights.loader import check_tensors
    from cloud_inference_from_scratch_b200.weights.source import RandomSource, WeightsError

    raw = raw_config()
    full = DecoderModel(resolve_config(raw)[2]).tensor_table()
    del raw["layers"][0]["mixer"]["decay_rank"]
    table = DecoderModel(resolve_config(raw)[2]).tensor_table()
    assert table["l0.mix.w1"].shape == (-1, 24) and table["l0.mix.w2"].shape == (12, -1)
    check_tensors(RandomSource(full, 1), table)                        # any width fits
    with pytest.raises(WeightsError, match="leaves a size open"):
        RandomSource(table, 1).get("l0.mix.w1")


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="conv"), "mixer type"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=2), "kv_from"),          # another kind of layer
    (lambda c: c["layers"][3]["mixer"].update(kv_rank=8), "kv_from"),          # another latent size
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=6), "exceeds"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=3), "even"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "not built"),
    (lambda c: c["layers"][0]["mlp"].update(limit=0), "positive"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["layers"][1]["mixer"].pop("q_rank"), "q_rank"),
])
def test_refusals(change, message):
    raw = copy.deepcopy(raw_config())
    change(raw)
    with pytest.raises(ConfigError, match=message):
        LodalixConfig.from_dict(raw)


def test_pools_group_layers_by_what_a_token_leaves():
    from cloud_inference_from_scratch_b200.cache.pools import plan_groups

    raw = raw_config()
    raw["layers"].append(copy.deepcopy(raw["layers"][1]))        # a second owner with rows of the same sizes
    groups, place = plan_groups(DecoderModel(resolve_config(raw)[2]).cache_needs(), 2)
    assert len(groups) == 2 and sorted(place) == [1, 2, 4] and place[1][0] == place[4][0] != place[2][0]
    assert groups[place[1][0]].bytes_per_token == (16 + 8) * 2 * 2 and groups[place[2][0]].bytes_per_token == (24 + 4) * 2


@pytest.mark.parametrize("rot", [
    dict(base=10000.0, dims=16),
    dict(base=10000.0, dims=64, scaling=dict(factor=8.0, original=512, fast=32.0, slow=1.0)),
    dict(base=500.0, dims=6, scaling=dict(factor=1.5, original=30, fast=2.0, slow=1.9)),      # a ramp of no width
    dict(base=1e6, dims=32, scaling=dict(factor=40.0, original=4096, fast=4000.0, slow=1e-4)),  # both ends clamped
])
def test_rotary_frequencies_and_magnitude(rot):
    from cloud_inference_from_scratch_b200.config import PartSpec
    from cloud_inference_from_scratch_b200.parts import build_part

    scaling = rot.get("scaling")
    ramp = tuple(scaling[key] for key in ("factor", "original", "fast", "slow")) if scaling else None
    part = build_part("position", PartSpec("rope_neox", dict(head_dim=rot["dims"], rotary_dim=rot["dims"], theta=rot["base"],
                                                             max_positions=100, ramp=ramp)))
    want, magnitude = plain.rotary_frequencies(rot)
    assert torch.allclose(torch.tensor(part.frequencies(), dtype=torch.float64), want, rtol=1e-12, atol=0)
    assert math.isclose(part.magnitude, magnitude, rel_tol=1e-12)
    if scaling:
        plainly = plain.rotary_frequencies(dict(base=rot["base"], dims=rot["dims"]))[0]
        assert (want <= plainly * (1 + 1e-12)).all() and (want >= plainly / scaling["factor"] * (1 - 1e-12)).all()
