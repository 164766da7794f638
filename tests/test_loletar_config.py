"""The Loletar configuration: reading, refusing, the plan it makes, tensor names, cache needs (CPU)."""

import json

import pytest
import torch

import plain_loletar as plain
from loletar_tiny import TINY, make_weights


def test_registry_and_round_trip():
    from socrates_b200.config import LoletarConfig, config_from_dict, known_architectures
    assert "Loletar" in known_architectures()
    for name, d in TINY.items():
        cfg = config_from_dict(d)
        assert isinstance(cfg, LoletarConfig)
        again = config_from_dict(json.loads(json.dumps(cfg.to_dict())))
        assert again == cfg, name
    assert config_from_dict(TINY["A"]).embedding_scale == 3.0


def test_plan_order_parts_and_borrowed_caches():
    from socrates_b200.config import config_from_dict
    plan = config_from_dict(TINY["A"]).plan()
    assert [e.layer for e in plan.order] == [0, 1, 2, 3]
    assert [e.reads_cache_of for e in plan.order] == [None, None, 1, None]
    assert [l.mixer.kind for l in plan.layers] == ["gated_delta_rule"] + ["gated_sink_attention"] * 3
    assert [l.feed_forward.kind if l.feed_forward else None for l in plan.layers] == \
        ["routed_experts", "swiglu", None, "routed_experts"]
    assert all(l.arrangement == "branch_norm" for l in plan.layers)
    assert [len(l.norms) for l in plan.layers] == [2, 2, 1, 2]
    att = plan.layers[1].mixer.params
    assert att["sink"] == 0.0 and att["gate"] == "dim" and att["own_kv"] and not plan.layers[2].mixer.params["own_kv"]
    assert att["position"].params["pairing"] == "neighbours" and att["position"].params["rotary_dim"] == 6
    assert plan.layers[0].mixer.params["query_scale"] == 16 ** -0.5
    planB = config_from_dict(TINY["B"]).plan()
    assert [e.reads_cache_of for e in planB.order] == [None, None, None, 0]
    assert planB.layers[0].mixer.params["position"].kind == "none"
    r = plan.layers[0].feed_forward.params
    assert (r["num_experts"], r["num_identity"], r["top"], r["groups"], r["keep_groups"]) == (5, 1, 2, 3, 2)
    r = plan.layers[3].feed_forward.params
    assert (r["num_identity"], r["groups"], r["keep_groups"]) == (0, 1, 1)


def test_tensor_names_and_cache_needs():
    from socrates_b200.cache.manager import PagedKVSpec
    from socrates_b200.config import config_from_dict
    from socrates_b200.engine.model import Model
    m = Model(config_from_dict(TINY["A"]).plan())
    p = m.parameters()
    for n in ("embed", "head", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.q.conv", "l0.mix.A_log", "l0.mix.dt_bias",
              "l0.mix.a", "l0.mix.b", "l0.mix.norm", "l0.mlp.router", "l0.mlp.correction", "l0.mlp.e4.down",
              "l1.mix.q.norm", "l1.mix.k.norm", "l1.mix.g", "l1.mlp.gate", "l2.mix.q", "l2.mix.q.norm", "l2.mix.o"):
        assert n in p, n
    for n in ("l2.mix.k", "l2.mix.v", "l2.mix.k.norm", "l2.norm2", "l0.mlp.e5.gate"):
        assert n not in p, n
    assert p["l0.mlp.router"].shape == (6, 48) and p["l0.mix.q.conv"].shape == (32, 2)
    assert p["l3.mix.v"].shape == (24, 48) and p["l3.mix.g"].shape == (48, 48) and p["l1.mix.g"].shape == (48, 48)
    needs = m.cache_needs()
    assert needs[2] is None
    assert needs[1].paged == PagedKVSpec(2, 16, None, 8) and needs[3].paged == PagedKVSpec(1, 8, None, 24)
    assert needs[0].paged is None and needs[0].state["S"].shape == (4, 16, 8) and needs[0].state["conv"].shape == (1, 96)
    mB = Model(config_from_dict(TINY["B"]).plan())
    assert "conv" not in mB.cache_needs()[1].state            # one tap: no inputs to remember
    assert all(n.paged is None for n in Model(config_from_dict(TINY["C"]).plan()).cache_needs())


@pytest.mark.parametrize("change,text", [
    (lambda d: d["layers"][0].update(type="scan"), "known mixer"),
    (lambda d: d["layers"][1]["mixer"].update(kv_heads=4), "multiple"),
    (lambda d: d["layers"][2]["mixer"].update(kv_from=0), "kv_from"),
    (lambda d: d["layers"][2]["mixer"].update(kv_from=2), "kv_from"),
    (lambda d: d["layers"][2]["mixer"].update(vdim=16), "differs"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=5), "rot.dims"),
    (lambda d: d["layers"][0]["mlp"]["router"].update(top=5), "top"),
    (lambda d: d["layers"][0]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda d: d["layers"][1]["mlp"].update(kind="sparse"), "kind"),
    (lambda d: d["norm"].pop("eps"), "eps"),
])
def test_refusals(change, text):
    from socrates_b200.config import ConfigError, config_from_dict
    d = json.loads(json.dumps(TINY["A"]))
    change(d)
    with pytest.raises(ConfigError) as e:
        config_from_dict(d)
    assert text in str(e.value)


def test_plain_statement_on_itself():
    """The plain statement's own pieces agree: token-by-token recurrence carries its state, the sink only
    ever lowers the weights, rotation keeps norms and depends on the distance alone."""
    g = torch.Generator().manual_seed(0)
    T, H, G, D, Dv = 9, 4, 2, 6, 5
    q, k = plain.unit(torch.randn(T, G, D, generator=g).double()), plain.unit(torch.randn(T, G, D, generator=g).double())
    v = torch.randn(T, H, Dv, generator=g).double()
    beta, decay = torch.rand(T, H, generator=g).double(), torch.rand(T, H, generator=g).double()
    whole, S = plain.delta_recurrence(q, k, v, beta, decay)
    a, Sa = plain.delta_recurrence(q[:4], k[:4], v[:4], beta[:4], decay[:4])
    b, Sb = plain.delta_recurrence(q[4:], k[4:], v[4:], beta[4:], decay[4:], Sa)
    assert torch.allclose(torch.cat([a, b]), whole) and torch.allclose(S, Sb)
    qq, kk = torch.randn(T, H, D, generator=g).double(), torch.randn(T, G, D, generator=g).double()
    vv = torch.ones(T, G, Dv).double()
    with_sink, without = plain.sink_attention(qq, kk, vv, 0.7), plain.sink_attention(qq, kk, vv, 0.7, sink=False)
    assert torch.allclose(without, torch.ones_like(without)) and bool((with_sink < 1.0).all())
    x = torch.randn(1, 1, 8, generator=g).double().expand(T, 1, 8)
    r0 = plain.rotate_pairs(x, torch.arange(T), 6, 50.0)
    r5 = plain.rotate_pairs(x, torch.arange(T) + 5, 6, 50.0)
    assert torch.allclose(r0.norm(dim=-1), x.norm(dim=-1)) and torch.equal(r0[..., 6:], x[..., 6:])
    assert torch.allclose(r0[2, 0] @ r0[7, 0], r5[2, 0] @ r5[7, 0])
    z = torch.tensor([[0.0, 3.0, 2.9, 0.0, 0.0, 1.0]]).double()
    r = {"experts": 4, "identity": 2, "top": 2, "groups": {"count": 3, "keep": 2}}
    ids, wts = plain.route(z, torch.zeros(6).double(), r)
    assert ids.tolist() == [[1, 2]]
    ids, wts = plain.route(z, torch.tensor([0.0, 0.0, 0.0, 0.0, 0.0, 2.0]).double(), r)
    assert ids.tolist() == [[5, 1]] and torch.allclose(wts, torch.softmax(z, -1)[0, [5, 1]][None])   # weights without the correction
    ids, _ = plain.route(z, torch.tensor([0.0, 0.0, 0.0, 0.1, 0.0, 0.12]).double(), {**r, "groups": {"count": 3, "keep": 1}})
    assert ids.tolist() == [[1, 0]]                            # only the best group is open, although 2, 3 and 5 score higher than 0


def test_random_weights_cover_every_tensor():
    w = make_weights(TINY["B"], 1)
    assert w["l1.mix.A_log"].shape == (1,) and w["l0.mlp.correction"].shape == (8,)
    assert all(t.dtype == torch.bfloat16 for t in w.values())
