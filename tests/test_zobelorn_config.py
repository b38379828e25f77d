"""The Zobelorn configuration on the CPU: what it reads, what it refuses, the tensors it declares, which
layers share a cache and what that cache may give back, the rotation's scaled frequencies, and the plain
restatement's own mechanisms on cases small enough to do by hand."""
import copy
import math

import pytest
import torch

import plain_zobelorn as plain
from tiny_zobelorn import TINY, chunked, config, dense, moe, windowed
from tokenizer_b200.cache.manager import CachePlan
from tokenizer_b200.config import ConfigError, ZobelornConfig, config_from_dict
from tokenizer_b200.parts.model import declared_tensors


def test_the_registry_finds_the_design_by_its_name():
    cfg, _, _ = TINY["a"]()
    again = config_from_dict(cfg.to_dict())
    assert isinstance(again, ZobelornConfig) and again.to_dict() == cfg.to_dict()
    assert config_from_dict(dict(cfg.to_dict(), architectures=["Zobelorn"])).to_dict() == cfg.to_dict()


def test_declared_tensors_follow_the_sizes():
    cfg, _, _ = TINY["a"]()
    shapes = {t.name: tuple(t.shape) for t in declared_tensors(cfg.model_spec())}
    assert shapes["embed"] == (301, 96) and shapes["head"] == (301, 96) and shapes["final.norm"] == (96,)
    assert shapes["l0.mix.q"] == (6 * 16, 96) and shapes["l0.mix.k"] == (3 * 16, 96) and shapes["l0.mix.v"] == (3 * 32, 96)
    assert shapes["l0.mix.o"] == (96, 6 * 32) and shapes["l0.mix.g"] == (6 * 32, 96)
    assert shapes["l0.mix.q.norm"] == (96,) and shapes["l0.mix.k.norm"] == (48,)
    assert all(shapes[f"l0.{n}"] == (96,) for n in ("norm1", "norm1b", "norm2", "norm2b"))
    assert shapes["l1.mix.k"] == (2 * 24, 96) and "l1.mix.g" not in shapes and "l1.mix.q.norm" not in shapes
    assert shapes["l1.mlp.e5.down"] == (96, 40) and shapes["l1.mlp.router"] == (6, 96) and shapes["l1.mlp.shared.up"] == (56, 96)
    assert "l1.mlp.shared.sg" not in shapes and "l1.mlp.correction" not in shapes
    # a layer that borrows keys and values has queries and an output projection only, and here no feed-forward
    assert sorted(n for n in shapes if n.startswith("l2.")) == ["l2.mix.o", "l2.mix.q", "l2.norm1", "l2.norm1b"]
    assert not any(name.endswith(".b") and ".mix." in name for name in shapes)          # no biases


@pytest.mark.parametrize("change,word", [
    (lambda r: r["layers"][0].update(type="other"), "unknown type"),
    (lambda r: r["layers"][0]["mixer"].update(kv_heads=4), "do not divide"),
    (lambda r: r["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda r: r["layers"][0]["mixer"].update(mask={"size": 0}), "size"),
    (lambda r: r["layers"][0]["mixer"].update(softcap=0.0), "softcap"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda r: r["layers"][0]["mixer"].update(kv_from=0), "attention_2"),
    (lambda r: r["layers"][1]["mixer"]["rot"]["scaling"].pop("low"), "low"),
    (lambda r: r["layers"][2]["mixer"].update(kv_from=2), "does not run before"),
    (lambda r: r["layers"][2]["mixer"].update(kv_from=0), "keys of its own"),
    (lambda r: r["layers"][2]["mixer"].update(kv_heads=1), "not this layer's"),
    (lambda r: r["layers"][1]["mlp"]["router"].update(top=7), "experts"),
    (lambda r: r["layers"][1]["mlp"].update(kind="sparse"), "dense or moe"),
    (lambda r: r.pop("norm"), "norm"),
    (lambda r: r.update(layers=[]), "layers"),
])
def test_what_the_configuration_refuses(change, word):
    raw = copy.deepcopy(TINY["a"]()[0].to_dict())
    change(raw)
    with pytest.raises(ConfigError, match=word):
        ZobelornConfig.from_dict(raw)


def test_constants_that_a_file_leaves_out_are_neutral():
    raw = copy.deepcopy(TINY["c"]()[0].to_dict())
    raw.pop("embedding")
    raw.pop("residual_mult")
    cfg = ZobelornConfig.from_dict(raw)
    spec = cfg.model_spec()
    assert spec.embedding.params["scale"] == 1.0 and "gain_scale" not in spec.layers[0].parts["mixer_post_norm"].params


def needs_of(cfg):
    """What every call keeps per request, from the model's description alone (the parts are not built); None
    where a call reads an earlier call's cache."""
    from tokenizer_b200.parts.base import CacheNeed, KVNeed
    spec = cfg.model_spec()
    out = []
    for call in spec.order:
        p = spec.layers[call.layer].parts["mixer"].params
        row = -(-max(p["dim"], p["vdim"]) // 16) * 16
        out.append(None if call.cache is not None else
                   CacheNeed(kv=KVNeed(p["kv_heads"], row, p["window"], chunk=p.get("cache_chunk", p["chunk"]))))
    return out


def test_a_borrowed_cache_keeps_what_every_reader_can_still_see():
    cfg, _, page = TINY["a"]()
    spec = cfg.model_spec()
    assert [c.cache for c in spec.order] == [None, None, 1]
    # chunks of 20 and, in the borrower, of 10: pages go back by chunks of 20
    assert spec.layers[1].parts["mixer"].params["cache_chunk"] == 20 and spec.layers[1].parts["mixer"].params["chunk"] == 20
    assert spec.layers[2].parts["mixer"].params["chunk"] == 10 and not spec.layers[2].parts["mixer"].params["own_kv"]
    plan = CachePlan(needs_of(cfg), num_pages=32, page_size=page, max_requests=3)
    assert [(g.window, g.chunk, g.calls) for g in plan.groups] == [(23, None, [0]), (None, 20, [1])]
    cache = plan.open("r")
    plan.reserve(cache, 45)
    plan.commit(cache, 45)             # next position 45: the window reaches back to 22, the chunk began at 40
    assert [p >= 0 for p in cache.tables[0]] == [False, False, True, True, True, True]
    assert [p >= 0 for p in cache.tables[1]] == [False, False, False, False, False, True]
    plan.check()
    plan.close(cache)
    assert all(a.available == 32 for a in plan.allocators)
    # chunks of 21 and 7 read together with a layer that sees every key: nothing goes back
    cfg, _, _ = TINY["d"]()
    spec = cfg.model_spec()
    assert [c.cache for c in spec.order] == [None, 0, None, 0, None]
    assert spec.layers[0].parts["mixer"].params["cache_chunk"] is None
    # unlike chunk sizes without a common multiple below their product
    cfg = config([chunked(2, 1, 8, 8, 0.3, size=6, mlp=dense(8)), chunked(2, 1, 8, 8, 0.3, size=4, kv_from=0)],
                 vocab=20, width=16, eps=1e-6, scale=1.0, mult=1.0)
    assert cfg.model_spec().layers[0].parts["mixer"].params["cache_chunk"] == 12


def test_the_model_spec_names_parts_that_other_designs_can_use():
    cfg, _, _ = TINY["d"]()
    spec = cfg.model_spec()
    assert [l.block for l in spec.layers] == ["sandwich_norm_residual"] * 2 + ["sandwich_norm_mixer_only"] + \
        ["sandwich_norm_residual"] * 2
    assert all(l.parts["mixer"].kind == "gqa_rotary" for l in spec.layers)
    assert all(l.parts["mixer_norm"].kind == "rms_norm" and l.parts["mixer_norm"].params["one_plus"] for l in spec.layers)
    assert spec.layers[0].parts["mixer_post_norm"].params["gain_scale"] == 0.35
    assert "gain_scale" not in spec.layers[0].parts["mixer_norm"].params and "gain_scale" not in spec.final_norm.params
    routed = spec.layers[1].parts["feed_forward"].params
    assert (routed["score"], routed["share_on"], routed["shared_gate"], routed["top"]) == ("sigmoid", "input", False, 3)
    w = spec.layers[2].parts["mixer"].params
    assert (w["window"], w["chunk"], w["softcap"], w["output_gate"], w["qk_norm"]) == (49, None, 50.0, True, True)
    assert w["position"].kind == "rope_half" and w["position"].params["scaling"] == {"kind": "linear", "factor": 1.5}
    c = spec.layers[0].parts["mixer"].params
    assert (c["window"], c["chunk"], c["head_norm"], c.get("softcap")) == (None, 21, True, None)
    assert c["position"].kind == "rope_interleaved" and c["position"].params["scaling"]["kind"] == "bands"


def test_scaled_frequencies_of_the_rotation_parts():
    from tokenizer_b200.parts.position import scaled_frequencies
    base, dims = 300.0, 16
    freq = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    assert scaled_frequencies(freq, None) == freq
    assert scaled_frequencies(freq, {"kind": "linear", "factor": 4.0}) == [f / 4.0 for f in freq]
    got = scaled_frequencies(freq, {"kind": "bands", "factor": 16.0, "low": 2.0, "high": 8.0, "original": 128})
    want = plain.banded_frequencies(base, dims, 16.0, 2.0, 8.0, 128)
    assert got == pytest.approx(want, rel=1e-15)
    kinds = [("kept" if g == f else "divided" if g == pytest.approx(f / 16.0) else "blended") for g, f in zip(got, freq)]
    assert kinds[0] == "kept" and kinds[-1] == "divided" and "blended" in kinds      # all three bands occur
    with pytest.raises(ConfigError):
        scaled_frequencies(freq, {"kind": "other", "factor": 2.0})


# ---- the plain restatement, by hand ---------------------------------------------------------------------
def test_plain_windows_and_chunks_count_as_the_design_says():
    w = plain.visible_window(6, 3)
    assert w[4].tolist() == [False, False, True, True, True, False]        # itself and the two before it
    assert plain.visible_window(3, 1).tolist() == [[True, False, False], [False, True, False], [False, False, True]]
    c = plain.visible_chunk(7, 3)
    assert c[4].tolist() == [False, False, False, True, True, False, False]    # chunks 0-2 | 3-5 | 6
    assert c[6].tolist() == [False] * 6 + [True]


def test_plain_rotation_layouts_pair_lanes_differently():
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0]]], dtype=torch.float64)
    pos = torch.tensor([1])
    a, b = 0.5, 0.25
    half = plain.rotate(x, pos, [a, b], "half")[0, 0]
    inter = plain.rotate(x, pos, [a, b], "interleaved")[0, 0]
    assert half.tolist() == pytest.approx([math.cos(a) - 3 * math.sin(a), 2 * math.cos(b) - 4 * math.sin(b),
                                           3 * math.cos(a) + math.sin(a), 4 * math.cos(b) + 2 * math.sin(b), 5.0])
    assert inter.tolist() == pytest.approx([math.cos(a) - 2 * math.sin(a), 2 * math.cos(a) + math.sin(a),
                                            3 * math.cos(b) - 4 * math.sin(b), 4 * math.cos(b) + 3 * math.sin(b), 5.0])


def test_plain_cap_bounds_a_score_and_leaves_small_ones():
    q = torch.tensor([[[100.0]], [[100.0]]], dtype=torch.float64)
    k = torch.tensor([[[100.0]], [[0.01]]], dtype=torch.float64)
    v = torch.tensor([[[1.0]], [[0.0]]], dtype=torch.float64)
    out = plain.attend(q, k, v, plain.visible_window(2, 2), 1.0, softcap=2.0)
    # scores 10000 and 1: capped to 2 tanh(5000) = 2 and 2 tanh(0.5)
    a, b = 2.0, 2.0 * math.tanh(0.5)
    assert float(out[1, 0]) == pytest.approx(math.exp(a) / (math.exp(a) + math.exp(b)))


def test_plain_experts_weigh_their_input():
    torch.manual_seed(0)
    h = torch.randn(1, 4, dtype=torch.float64)
    w = {"m.router": torch.zeros(3, 4, dtype=torch.float64)}
    w["m.router"][1] = h[0] / (h[0] @ h[0])                       # logit 1 for expert 1, 0 for the others
    for e in range(3):
        for n, shape in (("gate", (5, 4)), ("up", (5, 4)), ("down", (4, 5))):
            w[f"m.e{e}.{n}"] = torch.randn(*shape, dtype=torch.float64)
    out = plain.routed_feed_forward(h, w, "m", {"router": {"experts": 3, "top": 2}})
    s1, s0 = 1.0 / (1.0 + math.exp(-1.0)), 0.5                      # ties among the zeros go to the lower index
    want = plain.gated_feed_forward(s1 * h, w, "m.e1") + plain.gated_feed_forward(s0 * h, w, "m.e0")
    assert torch.allclose(out, want)
    assert not torch.allclose(out, s1 * plain.gated_feed_forward(h, w, "m.e1") + s0 * plain.gated_feed_forward(h, w, "m.e0"))
