"""The Magedra configuration, its plan, tensor names and cache needs; the plain statement checked on itself.
Nothing here needs a GPU."""

import json
import math

import pytest
import torch

import plain_magedra as plain
from magedra_tiny import TINY, make_weights
from socrates_b200.config import ConfigError, MagedraConfig, config_from_dict, known_architectures
from socrates_b200.engine.model import Model

F64 = torch.float64


def test_registry_and_round_trip():
    assert "Magedra" in known_architectures()
    for name, cfg in TINY.items():
        c = config_from_dict(cfg)
        assert isinstance(c, MagedraConfig)
        again = config_from_dict(json.loads(json.dumps(c.to_dict())))
        assert again == c, name
    c = config_from_dict(TINY["C"])
    assert c.streams == 0 and c.logit_scale == 0.25 and c.residual_mult == 0.5
    assert config_from_dict(TINY["B"]).logit_scale == 1.0


def test_plan_order_parts_and_shared_weights():
    plan = config_from_dict(TINY["A"]).plan()
    assert [e.layer for e in plan.order] == [0, 1, 1, 2, 0, 2]          # runs 2, 4 and 5 are earlier layers again
    assert [l.mixer.kind for l in plan.layers] == ["min_gru", "scaled_sum", "latent_attention"]
    assert all(l.arrangement == "hyper_connections" and l.params["streams"] == 3 for l in plan.layers)
    assert plan.layers[2].feed_forward is None and len(plan.layers[2].norms) == 1
    assert plan.embedding.kind == "normed_embedding" and plan.final_norm.kind == "layernorm"
    inner = plan.layers[1].mixer.params["branches"]
    assert [b.kind for b in inner] == ["talking_attention", "gated_linear_attention"]
    assert plan.layers[1].mixer.params["scales"] == (1.3, 0.8)
    assert plan.head.params["scale"] == 1.5


def test_tensor_names_and_cache_needs():
    m = Model(config_from_dict(TINY["A"]).plan())
    names = set(m.parameters())
    for n in ("embed", "embed.norm", "final.norm", "head", "l0.mix.z", "l0.mix.z.b", "l0.mix.x.b", "l0.mix.g", "l0.mix.o",
              "l0.hc1.in", "l0.hc1.out", "l0.hc1.mix", "l0.hc2.mix", "l0.mlp.gate.b", "l0.mlp.up", "l0.mlp.down.b",
              "l1.mix.left.q", "l1.mix.left.talk", "l1.mix.left.g", "l1.mix.right.f.b", "l1.mix.right.lower",
              "l1.mix.right.norm", "l3.mix.dq.norm", "l3.mix.uq", "l3.mix.dkv", "l3.mix.uk", "l3.mix.uv", "l3.norm1"):
        assert n in names, n
    assert not any(n.startswith(("l2.", "l4.", "l5.")) for n in names)      # they run other layers' weights
    assert "l3.norm2" not in names and "l3.hc2.in" not in names             # no feed-forward there
    p = m.parameters()
    assert p["l1.mix.left.talk"].shape == (4, 4) and p["l0.hc1.mix"].shape == (3, 3)
    assert p["l3.mix.dkv"].shape == (20 + 4, 40) and p["l3.mix.uq"].shape == (3 * 12, 16)
    needs = m.cache_needs()
    assert len(needs) == 6 and all(n is not None for n in needs)            # every run has a cache or state of its own
    assert needs[0].paged is None and needs[0].state_specs()["S"].shape == (24,)
    assert needs[1].paged.num_kv_heads == 2 and needs[1].paged.head_dim == 16 and needs[1].paged.value_dim == 8
    assert needs[1].state_specs()["right.S"].shape == (2, 12, 20)
    assert needs[3].paged.num_kv_heads == 1 and needs[3].paged.head_dim == 24 and needs[3].paged.value_dim == 20
    # without streams there are no stream tensors
    assert not any(".hc" in n for n in Model(config_from_dict(TINY["C"]).plan()).parameters())


def test_refusals():
    def broken(change):
        cfg = json.loads(json.dumps(TINY["A"]))
        change(cfg)
        return cfg
    for change in (lambda c: c["layers"][0].update(type="lstm"),
                   lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=3),
                   lambda c: c["layers"][3]["mixer"].update(rot_dim=3),
                   lambda c: c["layers"][2].update(weights_of=2),
                   lambda c: c["layers"][0]["mlp"].update(kind="moe"),
                   lambda c: c.update(streams=9),
                   lambda c: c["layers"][0]["mlp"].pop("limit"),
                   lambda c: c["norm"].pop("eps")):
        with pytest.raises(ConfigError):
            config_from_dict(broken(change))


def test_plain_statement_on_itself():
    g = torch.Generator().manual_seed(3)
    # layer norm: zero mean, unit variance, then the gain
    x = torch.randn(5, 12, generator=g, dtype=F64) * 3 + 2
    y = plain.layer_norm(x, torch.ones(12, dtype=F64), 0.0)
    assert float(y.mean(-1).abs().max()) < 1e-12 and float(((y * y).mean(-1) - 1).abs().max()) < 1e-9
    # rotations depend on the distance only, in both pairings, and leave the dims past rot.dims alone
    rot = {"dims": 6, "base": 100.0}
    q, k = torch.randn(1, 1, 10, generator=g, dtype=F64), torch.randn(1, 1, 10, generator=g, dtype=F64)
    for turn in (plain.rotate_halves, plain.rotate_pairs):
        a = (turn(q, torch.tensor([7]), rot) * turn(k, torch.tensor([3]), rot)).sum()
        b = (turn(q, torch.tensor([104]), rot) * turn(k, torch.tensor([100]), rot)).sum()
        assert abs(float(a - b)) < 1e-9
        assert torch.equal(turn(q, torch.tensor([9]), rot)[..., 6:], q[..., 6:])
    assert not torch.allclose(plain.rotate_halves(q, torch.tensor([5]), rot), plain.rotate_pairs(q, torch.tensor([5]), rot))
    # the candidate of the minGRU is continuous at zero and positive
    u = torch.tensor([-1e-9, 0.0, 1e-9], dtype=F64)
    c = torch.where(u >= 0, u + 0.5, plain.sigmoid(u))
    assert float((c - 0.5).abs().max()) < 1e-8
    # a recurrence continued from its state equals the recurrence over the whole sequence
    cfg = TINY["A"]
    w = {k: v.double() for k, v in make_weights(cfg, 2).items()}
    h = torch.randn(30, cfg["width"], generator=g, dtype=F64)
    whole, _ = plain.min_gru(h, w, "l0.mix.")
    first, S = plain.min_gru(h[:11], w, "l0.mix.")
    rest, _ = plain.min_gru(h[11:], w, "l0.mix.", S)
    assert torch.allclose(torch.cat([first, rest]), whole, atol=1e-12)
    m = cfg["layers"][1]["mixer"]["right"]
    whole, _ = plain.gated_linear_attention(h, w, "l1.mix.right.", m, 1e-6)
    first, S = plain.gated_linear_attention(h[:11], w, "l1.mix.right.", m, 1e-6)
    rest, _ = plain.gated_linear_attention(h[11:], w, "l1.mix.right.", m, 1e-6, S)
    assert torch.allclose(torch.cat([first, rest]), whole, atol=1e-12)
    # mixing the heads with the identity is ordinary attention; the forget gate never falls below its bound
    w2 = dict(w)
    w2["l1.mix.left.talk"] = torch.eye(4, dtype=F64)
    ml = cfg["layers"][1]["mixer"]["left"]
    pos = torch.arange(30)
    a = plain.talking_attention(h, w2, "l1.mix.left.", ml, pos)
    w3 = dict(w2)
    w3["l1.mix.left.talk"] = torch.eye(4, dtype=F64)[[1, 0, 2, 3]]          # heads 0 and 1 trade scores
    assert not torch.allclose(a, plain.talking_attention(h, w3, "l1.mix.left.", ml, pos))
    # latent attention written with keys and values equals the form that keeps only the latent
    ml = cfg["layers"][3]["mixer"]
    p = "l3.mix."
    a = plain.latent_attention(h, w, p, ml, 1e-6, pos)
    H, dn, dr, dv, rank = 3, 8, 4, 12, 20
    rot = {"dims": dr, "base": ml["rot"]["base"]}
    cq = plain.rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], 1e-6)
    q = (cq @ w[p + "uq"].T).view(30, H, dn + dr)
    down = h @ w[p + "dkv"].T
    c = plain.rms_norm(down[:, :rank], w[p + "dkv.norm"], 1e-6)
    kr = plain.rotate_pairs(down[:, rank:].view(30, 1, dr), pos, rot)[:, 0]
    q_lat = torch.einsum("ihd,hdr->ihr", q[..., :dn], w[p + "uk"].view(H, dn, rank))
    s = (torch.einsum("ihr,jr->hij", q_lat, c) + torch.einsum("ihd,jd->hij", plain.rotate_pairs(q[..., dn:], pos, rot), kr)) * ml["scale"]
    o_lat = torch.einsum("hij,jr->ihr", plain.causal_softmax(s), c)
    b = torch.einsum("ihr,her->ihe", o_lat, w[p + "uv"].view(H, dv, rank)).reshape(30, H * dv) @ w[p + "o"].T
    assert torch.allclose(a, b, atol=1e-10)


def test_streams_that_start_equal_and_one_stream():
    """With one stream whose reading, mixing and writing weights are all one the block is the ordinary
    residual sum; several streams start as copies of the embedding's output."""
    cfg = json.loads(json.dumps(TINY["B"]))
    w = {k: v.double() for k, v in make_weights(cfg, 4).items()}
    for k in list(w):
        if ".hc" in k:
            w[k] = torch.ones_like(w[k])
    ids = [3, 9, 27, 40, 5, 5, 61]
    a = plain.forward(cfg, w, ids)
    plain_cfg = {k: v for k, v in cfg.items() if k != "streams"}
    assert torch.allclose(a, plain.forward(plain_cfg, w, ids), atol=1e-10)
    assert math.isfinite(float(a.abs().max()))
