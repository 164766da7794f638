"""Configuration, plan, weights and cache bookkeeping of the Bofusun decoder (no GPU)."""

import json

import pytest
import torch

import plain_bofusun as plain
from bofusun_tiny import TINY, make_folder


def test_config_round_trip_and_plan():
    from socrates_b200.config import BofusunConfig, ConfigError, config_from_dict
    cfg_dict, _ = TINY["P"]
    cfg = config_from_dict(cfg_dict)
    assert isinstance(cfg, BofusunConfig) and cfg.loop == (0, 2, 3) and cfg.width == 48
    assert config_from_dict(json.loads(json.dumps(cfg.to_dict()))) == cfg
    plan = cfg.plan()
    # three passes over layers 0 and 1, then layer 2; every pass starts with its own injection
    assert [e.layer for e in plan.order] == [0, 1, 0, 1, 0, 1, 2]
    starts = [(i, e.before.params["index"], e.before.params["add_embedding"])
              for i, e in enumerate(plan.order) if e.before is not None]
    assert starts == [(0, 0, False), (2, 1, True), (4, 2, True)]
    assert [(i, s) for i, s in plain.run_order(cfg_dict)] == \
        [(e.layer, e.before.params["index"] if e.before else None) for e in plan.order]
    assert plan.layers[1].feed_forward is None and len(plan.layers[1].norms) == 2
    assert plan.layers[0].feed_forward.kind == "dense_act" and len(plan.layers[0].norms) == 4
    # a loop of one pass, and no loop at all
    assert [e.before is not None for e in config_from_dict(TINY["R"][0]).plan().order] == [False, True, False]
    assert all(e.before is None for e in config_from_dict(TINY["Q"][0]).plan().order)
    bad = json.loads(json.dumps(cfg_dict))
    bad["layers"][0]["type"] = "convolution"
    with pytest.raises(ConfigError):
        config_from_dict(bad)
    bad = json.loads(json.dumps(cfg_dict))
    bad["layers"][0]["mlp"]["kind"] = "routed"
    with pytest.raises(ConfigError):
        config_from_dict(bad)
    bad = json.loads(json.dumps(cfg_dict))
    bad["loop"]["stop"] = 9
    with pytest.raises(ConfigError):
        config_from_dict(bad)


def test_tensor_names_and_cache_needs():
    from socrates_b200.config import config_from_dict
    from socrates_b200.engine.model import Model
    model = Model(config_from_dict(TINY["R"][0]).plan())
    names = model.parameters()
    for n in ("embed", "embed.norm", "loop.step", "final.norm", "head", "l0.norm1", "l0.norm1b", "l1.norm2b",
              "l0.mix.left.q.b", "l0.mix.left.k.conv", "l0.mix.left.rel", "l0.mix.left.out", "l0.mix.right.A_log",
              "l0.mix.right.conv.b", "l0.mix.right.dt.b", "l1.mix.g", "l1.mlp.up.b", "l2.mlp.down"):
        assert n in names, n
    assert "l0.norm2" not in names and "l0.mlp.up" not in names
    assert names["l0.mix.left.rel"].shape == (-1, 6) and names["l0.mix.left.rel"].matches((20, 6))
    assert names["loop.step"].shape == (1, 40)
    assert names["l0.mix.left.v"].shape == (16, 40) and names["l0.mix.left.k"].shape == (8, 40)
    needs = model.cache_needs()
    assert needs[0].paged.window == 16 and needs[0].paged.value_dim == 16 and needs[0].paged.head_dim == 8
    assert set(needs[0].state_specs()) == {"left.conv", "right.ssm", "right.conv"}
    assert needs[0].state_specs()["left.conv"].shape == (2, 6 * 8 + 8 + 16)
    assert needs[1].paged is None and needs[1].state_specs()[""].shape == (5, 8, 8)
    # one tap on the right: no convolution state there
    assert set(needs[2].state_specs()) == {"left.conv", "right.ssm"} and needs[2].paged.window == 50


@pytest.mark.parametrize("rows,far", [(32, 240), (9, 64), (12, 20), (20, 100), (16, 128), (8, 1000), (2, 5)])
def test_distance_table_agrees_with_the_bucket_formula(rows, far):
    from socrates_b200.parts.window_attention import bias_by_distance
    rel = torch.randn(rows, 3)
    for window in (None, 7, far + 40):
        table = bias_by_distance(rel, float(far), window)
        assert table.shape[0] == 3 and table.shape[1] == (min(window, far + 1) if window else far + 1)
        for n in range(table.shape[1]):
            assert torch.equal(table[:, n], rel[plain.distance_bucket(n, rows, far)]), n
        # past the table's end the bucket no longer changes
        for n in (far + 1, far * 3):
            if not window or n < window:
                assert plain.distance_bucket(n, rows, far) == plain.distance_bucket(table.shape[1] - 1, rows, far)
    assert plain.distance_bucket(far, rows, far) == rows - 1


def test_folder_loads_with_a_table_length_from_the_file(tmp_path):
    from socrates_b200.config import load_config
    from socrates_b200.engine.model import Model
    from socrates_b200.weights import WeightsError, load_weights
    from safetensors.torch import load_file, save_file
    folder, cfg, w = make_folder(tmp_path, "Q")
    model = Model(load_config(folder).plan())
    t = load_weights(folder, model.parameters(), torch.float32, "cpu")
    assert t["l0.mix.left.rel"].shape == (9, 2) and t["l0.mix.left.rel"].dtype == torch.float32
    assert t["l0.mix.left.q"].dtype == torch.float32 and t["l0.norm1"].dtype == torch.float32
    raw = load_file(str(folder / "model.safetensors"))
    raw["l0.mix.left.rel"] = raw["l0.mix.left.rel"][:, :1].contiguous()       # a head is missing
    del raw["l1.mix.g"]
    save_file(raw, str(folder / "model.safetensors"))
    with pytest.raises(WeightsError) as e:
        load_weights(folder, model.parameters(), torch.float32, "cpu")
    assert e.value.missing == ["l1.mix.g"] and len(e.value.wrong_shape) == 1


def test_cache_rows_with_named_states_and_unequal_key_value_sizes():
    from socrates_b200.cache import CacheManager, CacheNeeds, PagedKVSpec, StateSpec
    needs = [CacheNeeds(paged=PagedKVSpec(2, 8, 5, 24), state={"a": StateSpec((3,)), "b.c": StateSpec((2, 2))}),
             CacheNeeds(state=StateSpec((4,)))]
    cache = CacheManager(needs, max_rows=3, max_len=64, page_size=4, num_pages=10, dtype=torch.float32, device="cpu")
    k, v = cache.pools(0)
    assert k.shape == (11, 2, 4, 8) and v.shape == (11, 2, 4, 24)
    assert CacheManager.bytes_per_page(needs, 4, torch.float32) == 2 * 4 * (8 + 24) * 4
    cache.assign(1)
    cache.state(0, "a")[1] += 1.0
    cache.state(0, "b.c")[1] += 2.0
    cache.state(1)[1] += 3.0
    assert cache.reserve(1, 9) and cache.free_pages() == [7]
    cache.commit(1, 9)                      # a window of 5: the first block went back
    assert cache.free_pages() == [8]
    cache.move_row(1, 2)
    assert float(cache.state(0, "b.c")[2].sum()) == 8.0 and float(cache.state(1)[2].sum()) == 12.0
    cache.release(2)
    cache.assign(2)                         # a slot that is used again starts from zero
    assert float(cache.state(0, "a")[2].abs().sum()) == 0.0 and float(cache.state(1)[2].abs().sum()) == 0.0
    assert cache.free_pages() == [10]
    cache.check()
