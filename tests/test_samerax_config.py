"""The Samerax configuration: reading, refusing, the plan it makes, tensor names, cache needs; the cache
manager's bookkeeping of a window that keeps the first keys; the plain statement checked on itself (CPU)."""

import json
import math

import pytest
import torch

import plain_samerax as plain
from samerax_tiny import TINY, make_weights


def test_registry_and_round_trip():
    from socrates_b200.config import SameraxConfig, config_from_dict, known_architectures
    assert "Samerax" in known_architectures()
    for name, d in TINY.items():
        cfg = config_from_dict(d)
        assert isinstance(cfg, SameraxConfig)
        again = config_from_dict(json.loads(json.dumps(cfg.to_dict())))
        assert again == cfg, name
    a, b = config_from_dict(TINY["A"]), config_from_dict(TINY["B"])
    assert a.embedding_scale == 2.5 and a.logit_softcap == 20.0
    assert b.embedding_scale == 1.0 and b.logit_softcap is None


def test_plan_order_parts_and_shared_weights():
    from socrates_b200.config import config_from_dict
    plan = config_from_dict(TINY["A"]).plan()
    assert len(plan.layers) == 3                                    # layers 0, 1 and 4 own tensors
    assert [e.layer for e in plan.order] == [0, 1, 0, 1, 2, 0]
    assert all(e.reads_cache_of is None for e in plan.order)        # the same weights, a cache of its own each time
    assert [l.prefix for l in plan.layers] == ["l0.", "l1.", "l4."]
    assert [l.mixer.kind for l in plan.layers] == ["differential_attention"] * 3
    assert [l.feed_forward.kind if l.feed_forward else None for l in plan.layers] == ["swiglu", "routed_experts", None]
    assert [l.arrangement for l in plan.layers] == ["pre_norm", "pre_norm", "pre_norm_mixer"]
    m = plan.layers[0].mixer.params
    assert (m["num_heads"], m["num_kv_heads"], m["map_dim"], m["value_dim"]) == (6, 2, 8, 24)
    assert (m["window"], m["keep_first"], m["diff"], m["scale"]) == (37, 5, 0.3, 0.4)
    pos = m["position"].params
    assert pos["pairing"] == "halves" and pos["rotary_dim"] == 6 and pos["scaling"]["factor"] == 4.0
    assert plan.layers[1].mixer.params["position"].kind == "none"
    assert plan.layers[2].mixer.params["window"] is None and plan.layers[2].mixer.params["keep_first"] == 0
    r = plan.layers[1].feed_forward.params
    assert (r["router"], r["num_experts"], r["top"], r["vocab_size"], r["num_identity"]) == ("table", 5, 2, 101, 0)
    assert plan.head.params["softcap"] == 20.0 and plan.embedding.params["scale"] == 2.5
    assert config_from_dict(TINY["B"]).plan().head.params["softcap"] is None
    # an entry that names another layer's weights but other constants is a layer of its own with the same tensors
    d = json.loads(json.dumps(TINY["A"]))      # (layers share their dictionaries: a plain deepcopy would keep that)
    d["layers"][2]["mixer"]["mask"]["size"] = 11
    plan2 = config_from_dict(d).plan()
    assert [e.layer for e in plan2.order] == [0, 1, 2, 1, 3, 0] and plan2.layers[2].prefix == "l0."
    assert plan2.layers[2].mixer.params["window"] == 11


def test_tensor_names_and_cache_needs():
    from socrates_b200.cache.manager import PagedKVSpec
    from socrates_b200.config import config_from_dict
    from socrates_b200.engine.model import Model
    m = Model(config_from_dict(TINY["A"]).plan())
    p = m.parameters()
    for n in ("embed", "head", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.q", "l0.mix.q.b", "l0.mix.k.b", "l0.mix.v.b",
              "l0.mix.lq1", "l0.mix.lk2", "l0.mix.o", "l0.mlp.gate", "l1.mlp.table", "l1.mlp.e4.down", "l4.mix.v", "l4.norm1"):
        assert n in p, n
    for n in ("l2.mix.q", "l3.mlp.table", "l5.norm1", "l4.norm2", "l1.mlp.e5.gate", "l1.mlp.router", "l0.mix.o.b"):
        assert n not in p, n
    assert p["l0.mix.q"].shape == (6 * 2 * 8, 48) and p["l0.mix.k"].shape == (2 * 2 * 8, 48)
    assert p["l0.mix.v"].shape == (2 * 24, 48) and p["l0.mix.o"].shape == (48, 6 * 24) and p["l0.mix.lq1"].shape == (8,)
    assert p["l1.mlp.table"].shape == (101, 2) and p["l1.mlp.table"].role == "int"
    needs = m.cache_needs()
    assert len(needs) == 6 and all(n is not None for n in needs)
    assert needs[0].paged == PagedKVSpec(2, 16, 37, 24, keep_first=5) == needs[2].paged == needs[5].paged
    assert needs[1].paged == PagedKVSpec(1, 32, 20, 8, keep_first=0)
    assert needs[4].paged == PagedKVSpec(3, 24, None, 40, keep_first=0)
    w = make_weights(TINY["A"], 1)
    t = w["l1.mlp.table"]
    assert t.dtype == torch.int32 and int(t.min()) >= 0 and int(t.max()) < 5 and bool((t[:, 0] != t[:, 1]).all())


@pytest.mark.parametrize("change,words", [
    (lambda d: d["layers"][0].__setitem__("type", "delta"), "not a known mixer"),
    (lambda d: d["layers"][0]["mixer"].__setitem__("heads", 5), "no multiple"),
    (lambda d: d["layers"][0]["mixer"].pop("diff"), "diff"),
    (lambda d: d["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "even"),
    (lambda d: d["layers"][0]["mixer"]["rot"]["scaling"].pop("slow"), "slow"),
    (lambda d: d["layers"][0]["mixer"]["mask"].__setitem__("size", 0), "mask"),
    (lambda d: d["layers"][1]["mlp"]["router"].__setitem__("top", 6), "top"),
    (lambda d: d["layers"][1]["mlp"].__setitem__("kind", "sparse"), "not supported"),
    (lambda d: d["layers"][2].__setitem__("weights_of", 3), "earlier layer"),
    (lambda d: d["layers"][3].__setitem__("weights_of", 2), "earlier layer"),
    (lambda d: d["layers"][5].__setitem__("weights_of", 4), "feed-forward"),
    (lambda d: d.__setitem__("logit_softcap", -1.0), "logit_softcap"),
    (lambda d: d.pop("norm"), "norm"),
])
def test_refusals(change, words):
    from socrates_b200.config import ConfigError, config_from_dict
    d = json.loads(json.dumps(TINY["A"]))      # (layers share their dictionaries: a plain deepcopy would keep that)
    change(d)
    with pytest.raises(ConfigError, match=words):
        config_from_dict(d)


def test_stretched_frequencies_of_the_position_part():
    """The position part's table against the plain formula, with and without stretching."""
    from socrates_b200.config.plan import PartSpec
    from socrates_b200.parts.base import build_part
    for dims, base, sc in ((6, 100.0, (4.0, 32, 8.0, 1.0)), (32, 50000.0, (8.0, 64, 4.0, 0.5)), (24, 500.0, None),
                           (16, 1e6, (2.0, 2048, 32.0, 1.0)), (10, 10.0, (3.0, 7, 100.0, 0.001))):
        rot = {"dims": dims, "base": base}
        if sc:
            rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), sc))
        part = build_part("position", PartSpec("rotary", {"head_dim": dims + 2, "rotary_dim": dims, "theta": base,
                                                          "table_precision": "float64", "scaling": rot.get("scaling")}), "")
        table, r = part.tables("cpu")
        f, mag = plain.yarn_frequencies(rot)
        assert r == dims and torch.equal(table, f.float())
        assert part.magnitude == pytest.approx(mag) and (mag == 1.0) == (sc is None)
    # stretched: the fastest dims keep their frequency, the slowest are divided by the factor
    f, _ = plain.yarn_frequencies({"dims": 64, "base": 10000.0, "scaling": {"factor": 4.0, "original": 1024, "fast": 32.0, "slow": 1.0}})
    plain_f = 10000.0 ** (-torch.arange(32, dtype=torch.float64) / 32)
    assert f[0] == plain_f[0] and f[-1] == pytest.approx(float(plain_f[-1]) / 4.0)
    assert bool((f <= plain_f).all()) and bool((f >= plain_f / 4.0 - 1e-18).all())


def test_plain_statement_on_itself():
    # the mask: a window, the first keys beside it, nothing from the future
    v = plain.visible(12, 4, 2)
    assert v[11].tolist() == [True, True] + [False] * 6 + [True] * 4
    assert v[3].tolist() == [True] * 4 + [False] * 8 and v[5].tolist() == [True, True, True, True, True, True] + [False] * 6
    assert bool(plain.visible(7, None, 0).equal(torch.ones(7, 7).tril().bool()))
    assert plain.visible(9, 3, 0)[8].tolist() == [False] * 6 + [True] * 3
    # rotation: scores depend on the distance only; dims past rot.dims pass unchanged
    rot = {"dims": 6, "base": 100.0, "scaling": {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}}
    g = torch.Generator().manual_seed(0)
    q, k = torch.randn(1, 1, 10, generator=g, dtype=torch.float64), torch.randn(1, 1, 10, generator=g, dtype=torch.float64)
    s = lambda i, j: float((plain.rotate(q, torch.tensor([i]), rot) * plain.rotate(k, torch.tensor([j]), rot)).sum())
    assert s(9, 4) == pytest.approx(s(105, 100)) and abs(s(9, 4) - s(9, 5)) > 1e-3
    assert torch.equal(plain.rotate(q, torch.tensor([77]), rot)[..., 6:], q[..., 6:])
    mag = 0.1 * math.log(4.0) + 1.0
    assert float(plain.rotate(q, torch.tensor([0]), rot)[0, 0, 0]) == pytest.approx(float(q[0, 0, 0]) * mag)
    # a layer that runs another layer's weights gives what the owner gives on the same input
    cfg = TINY["B"]
    w = {k: (t if t.dtype == torch.int32 else t.double()) for k, t in make_weights(cfg, 2).items()}
    ids = torch.randint(0, cfg["vocab"], (30,), generator=g).tolist()
    z, streams = plain.forward(cfg, w, ids, True)
    assert streams.shape == (3, 30, cfg["width"]) and z.shape == (30, cfg["vocab"])
    # experts by table: top = every expert is the mean of all experts
    h = torch.randn(4, cfg["width"], generator=g, dtype=torch.float64)
    both = plain.table_experts(h, torch.tensor([1, 2, 3, 4]), w, "l1.mlp.", 2)
    mean = 0.5 * (plain.gated_ff(h, w, "l1.mlp.e0.") + plain.gated_ff(h, w, "l1.mlp.e1."))
    assert torch.allclose(both, mean)
    # the cap bends large logits and leaves small ones
    capped = plain.forward(TINY["C"], {k: (t if t.dtype == torch.int32 else t.double()) for k, t in make_weights(TINY["C"], 2).items()},
                           ids[:9])
    assert float(capped.abs().max()) < 8.0


def test_cache_bookkeeping_of_a_window_that_keeps_the_first_keys():
    from socrates_b200.cache.manager import CacheManager, CacheNeeds, PagedKVSpec
    page = 4
    needs = [CacheNeeds(paged=PagedKVSpec(1, 8, window=6, keep_first=5)), CacheNeeds(paged=PagedKVSpec(1, 8, window=6)),
             CacheNeeds(paged=PagedKVSpec(1, 8))]
    cm = CacheManager(needs, max_rows=2, max_len=64, page_size=page, num_pages=24, dtype=torch.float32, device="cpu")
    kept, plain_window, full = cm.groups
    assert kept.kept_blocks() == 2 and plain_window.kept_blocks() == 0 and full.kept_blocks() == 0
    cm.assign(0)
    length = 0
    for step in (3, 1, 9, 1, 1, 2, 17, 1):
        assert cm.reserve(0, length + step)
        length += step
        cm.commit(0, length)
        cm.check()
        first = max(0, length - 6 + 1) // page
        last = -(-length // page)
        held = lambda g: [b for b, p in enumerate(g.row_pages[0]) if p != 0]
        assert held(full) == list(range(last))
        assert held(plain_window) == list(range(first, last))
        assert held(kept) == sorted(set(range(min(2, last))) | set(range(first, last)))
    # a second row: the pages the window gave back are handed out again; the kept blocks never were
    cm.assign(1)
    assert cm.reserve(1, 30)
    cm.commit(1, 30)
    cm.check()
    assert set(kept.owned(0)).isdisjoint(kept.owned(1))
    cm.release(0)
    cm.release(1)
    assert cm.free_pages() == [24, 24, 24]
    # a long first portion far past the window: everything it writes is held while the step runs, then given back
    cm.assign(0)
    assert cm.pages_needed(0, 41) == [11, 11, 11]
    assert cm.reserve(0, 41)
    cm.commit(0, 41)
    assert [b for b, p in enumerate(kept.row_pages[0]) if p != 0] == [0, 1, 9, 10]
    assert cm.pages_needed(0, 45) == [1, 1, 1]
    cm.check()
