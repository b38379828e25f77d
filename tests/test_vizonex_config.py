"""The Vizonex configuration on the CPU: what it reads, what it refuses, the tensors it declares, what every
layer keeps per request, and the plain restatement's own mechanisms on cases small enough to do by hand."""
import copy
import math

import pytest
import torch

import plain_vizonex as plain
from tiny_vizonex import TINY, attention, config, dense, mamba2, moe
from tokenizer_b200.cache.manager import CachePlan
from tokenizer_b200.config import ConfigError, VizonexConfig, config_from_dict
from tokenizer_b200.parts.model import declared_tensors


def test_the_registry_finds_the_design_by_its_name():
    cfg, _, _ = TINY["a"]()
    again = config_from_dict(cfg.to_dict())
    assert isinstance(again, VizonexConfig) and again.to_dict() == cfg.to_dict()
    assert config_from_dict(dict(cfg.to_dict(), architectures=["Vizonex"])).to_dict() == cfg.to_dict()


def test_declared_tensors_follow_the_sizes():
    cfg, _, _ = TINY["a"]()
    shapes = {t.name: tuple(t.shape) for t in declared_tensors(cfg.model_spec())}
    assert shapes["embed"] == (301, 96) and shapes["pos"] == (512, 96) and shapes["head"] == (301, 96)
    assert shapes["l0.mix.q"] == (6 * 16, 96) and shapes["l0.mix.k"] == (3 * 16, 96) and shapes["l0.mix.v"] == (3 * 32, 96)
    assert shapes["l0.mix.o"] == (96, 6 * 32) and shapes["l0.mix.q.norm"] == (96,) and shapes["l0.mix.k.norm"] == (48,)
    assert shapes["l0.mix.temp"] == (6,) and shapes["l0.mix.sink"] == (6,)
    assert shapes["l0.canon1"] == (96, 3) and shapes["l0.ls1"] == (96,) and shapes["l0.ls2"] == (96,)
    assert shapes["l0.mlp.gate"] == (136, 96) and shapes["l0.mlp.down"] == (96, 136)
    inner, channels = 4 * 24, 4 * 24 + 2 * 2 * 16
    assert shapes["l1.mix.in"] == (2 * inner + 2 * 2 * 16 + 4, 96) and shapes["l1.mix.conv"] == (channels, 4)
    assert shapes["l1.mix.conv.b"] == (channels,) and shapes["l1.mix.norm"] == (inner,) and shapes["l1.mix.o"] == (96, inner)
    assert shapes["l1.mix.A_log"] == shapes["l1.mix.D"] == shapes["l1.mix.dt_bias"] == (4,)
    assert shapes["l1.mlp.e5.down"] == (96, 40) and shapes["l1.mlp.router"] == (6, 96) and shapes["l1.mlp.correction"] == (6,)
    assert shapes["l1.mlp.shared.gate"] == (56, 96) and "l1.mlp.shared.sg" not in shapes
    assert not any(name.startswith("l2.mlp") or name == "l2.ls2" for name in shapes) and "l2.ls1" in shapes
    assert not any(name.endswith(".b") and ".mix.q" in name for name in shapes)       # no biases
    cfg, _, _ = TINY["b"]()
    shapes = {t.name: tuple(t.shape) for t in declared_tensors(cfg.model_spec())}
    assert not any("shared" in name for name in shapes)                                 # an experts' layer without one


@pytest.mark.parametrize("change,word", [
    (lambda r: r["layers"][0].update(type="other"), "unknown type"),
    (lambda r: r["layers"][0]["mixer"].update(kv_heads=4), "do not divide"),
    (lambda r: r["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda r: r["layers"][0]["mixer"].update(mask={"size": 0}), "size"),
    (lambda r: r["layers"][1]["mixer"].update(groups=3), "do not divide"),
    (lambda r: r["layers"][1]["mixer"].update(norm_groups=7), "norm_groups"),
    (lambda r: r["layers"][1]["mlp"]["router"].update(top=7), "experts"),
    (lambda r: r["layers"][1]["mlp"]["router"]["groups"].update(keep=1, count=6), "groups"),
    (lambda r: r["layers"][1]["mlp"].update(kind="sparse"), "dense or moe"),
    (lambda r: r.pop("norm"), "norm"),
    (lambda r: r["canon"].update(taps=0), "taps"),
    (lambda r: r.update(layers=[]), "layers"),
])
def test_what_the_configuration_refuses(change, word):
    raw = copy.deepcopy(TINY["a"]()[0].to_dict())
    change(raw)
    with pytest.raises(ConfigError, match=word):
        VizonexConfig.from_dict(raw)


def needs_of(cfg):
    """What every layer keeps per request, from the configuration alone (the parts are not built)."""
    from tokenizer_b200.parts.base import CacheNeed, KVNeed, StateNeed
    out = []
    for layer in cfg.layers:
        m = layer["mixer"]
        side = StateNeed(((cfg.taps - 1) * cfg.width,)) if cfg.taps > 1 else None
        if layer["type"] == "attention":
            row = -(-max(m["dim"], m["vdim"]) // 16) * 16
            out.append(CacheNeed(kv=KVNeed(m["kv_heads"], row, None, chunk=m["mask"]["size"] if m.get("mask") else None),
                                 side_state=side))
        else:
            floats = m["heads"] * m["vdim"] * m["state"] + (m["conv"] - 1) * (m["heads"] * m["vdim"] + 2 * m["groups"] * m["state"])
            out.append(CacheNeed(state=StateNeed((floats,)), side_state=side))
    return out


def test_layers_of_unlike_chunks_and_rows_keep_their_keys_apart_and_every_layer_keeps_inputs():
    cfg, _, page = TINY["d"]()
    plan = CachePlan(needs_of(cfg), num_pages=32, page_size=page, max_requests=3)
    assert [(g.chunk, g.calls) for g in plan.groups] == [(7, [1]), (50, [2])]
    assert plan.state_calls == [0, 3] and plan.side_state_calls == [0, 1, 2, 3] and not plan.share_prefixes
    cache = plan.open("r")
    plan.reserve(cache, 60)
    plan.commit(cache, 60)              # next position 60: the chunk of 7 starts at 56, the chunk of 50 at 50
    assert [p >= 0 for p in cache.tables[0]] == [False, False, False, True]
    assert [p >= 0 for p in cache.tables[1]] == [False, False, False, True]
    plan.check()
    plan.close(cache)
    assert all(a.available == 32 for a in plan.allocators)


def test_a_model_of_recurrences_alone_has_no_pages_and_one_tap_keeps_nothing():
    cfg = config([mamba2(2, 8, 4, 1, 2, 1, dense(16)), mamba2(2, 8, 4, 2, 3, 2)], vocab=40, width=16, eps=1e-6, taps=1)
    plan = CachePlan(needs_of(cfg), num_pages=4, page_size=16, max_requests=2)
    assert plan.groups == [] and plan.state_calls == [0, 1] and plan.side_state_calls == []
    a, b = plan.open("a"), plan.open("b")
    plan.reserve(a, 1000)
    plan.commit(a, 1000)                # tokens without keys need no pages
    assert a.state_slot != b.state_slot
    plan.close(a)
    plan.close(b)
    plan.check()


def test_the_model_spec_names_parts_that_other_designs_can_use():
    cfg, _, _ = TINY["d"]()
    spec = cfg.model_spec()
    assert [l.block for l in spec.layers] == ["parallel_residual"] * 4
    assert [l.parts["mixer"].kind for l in spec.layers] == ["mamba2", "gqa_rotary", "gqa_rotary", "mamba2"]
    routed = spec.layers[0].parts["feed_forward"].params
    assert (routed["score"], routed["groups"], routed["group_keep"], routed["route_scale"]) == ("sigmoid", 4, 2, 0.8)
    assert (routed["limit"], routed["shared_limit"], routed["alpha"]) == (1.5, 2.5, 1.702)
    attn = spec.layers[1].parts["mixer"].params
    assert attn["chunk"] == 7 and attn["position"] is None and attn["sink"] and attn["qk_norm"] and not attn["bias"]
    cfg, _, _ = TINY["a"]()
    spec = cfg.model_spec()
    assert spec.layers[2].block == "parallel_residual_mixer_only" and spec.layers[2].parts["mixer"].params["chunk"] is None


# ---- the plain restatement, by hand ---------------------------------------------------------------------
def test_plain_convolution_puts_the_last_tap_on_the_current_token():
    x = torch.tensor([[1.0], [10.0], [100.0], [1000.0]], dtype=torch.float64)
    taps = torch.tensor([[3.0, 2.0, 1.0]], dtype=torch.float64)
    out = plain.causal_convolution(x, taps)
    assert out[:, 0].tolist() == [1.0, 12.0, 123.0, 1230.0]


def test_plain_attention_counts_chunks_from_zero_and_the_sink_once():
    q = torch.zeros(5, 1, 2, dtype=torch.float64)               # every score 0: weights are counts
    k = torch.zeros(5, 1, 2, dtype=torch.float64)
    v = torch.arange(1.0, 6.0, dtype=torch.float64).view(5, 1, 1)
    out = plain.sink_chunk_attention(q, k, v, 1.0, torch.ones(1, dtype=torch.float64), torch.zeros(1, dtype=torch.float64), 3)
    # positions 0 1 2 | 3 4: sums of the chunk's values so far over (keys so far + 1 for the sink)
    assert torch.allclose(out[:, 0, 0], torch.tensor([1 / 2, 3 / 3, 6 / 4, 4 / 2, 9 / 3], dtype=torch.float64))


def test_plain_recurrence_by_hand():
    x = torch.tensor([[2.0], [0.0]], dtype=torch.float64)
    B = torch.tensor([[1.0, 0.0], [0.0, 0.0]], dtype=torch.float64)
    C = torch.tensor([[1.0, 0.0], [1.0, 0.0]], dtype=torch.float64)
    dt = torch.tensor([0.5, 2.0], dtype=torch.float64)
    y = plain.selective_state_space(x, B, C, dt, torch.tensor(1.0, dtype=torch.float64), torch.tensor(3.0, dtype=torch.float64))
    # token 0 writes 0.5 * 2 along the first lane and reads it, plus 3 * 2; token 1 reads it decayed by exp(-2)
    assert torch.allclose(y[:, 0], torch.tensor([1.0 + 6.0, math.exp(-2.0)], dtype=torch.float64))


def test_plain_router_keeps_the_groups_whose_two_best_add_up_to_the_most():
    h = torch.eye(1, 4, dtype=torch.float64)
    z = torch.tensor([[4.0, -4.0, 1.0, 1.2, 0.9, -9.0]], dtype=torch.float64)
    w = {"router": torch.zeros(6, 4, dtype=torch.float64), "correction": torch.zeros(6, dtype=torch.float64)}
    w["router"][:, 0] = z[0]
    r = {"experts": 6, "top": 2, "scale": 2.0, "groups": {"count": 3, "keep": 1}}
    chosen, weights = plain.route(h, w, "", r)
    # groups (0, 1), (2, 3), (4, 5): the single best expert is in the first, the best pair in the second
    assert sorted(chosen[0].tolist()) == [2, 3]
    assert torch.allclose(weights[0].sort().values, 2.0 * plain.sigmoid(torch.tensor([1.0, 1.2], dtype=torch.float64)))
    w["correction"][1] = 9.0                                     # the correction moves the choice, not the weights
    chosen, weights = plain.route(h, w, "", r)
    assert sorted(chosen[0].tolist()) == [0, 1]
    assert torch.allclose(weights[0].sort().values, 2.0 * plain.sigmoid(torch.tensor([-4.0, 4.0], dtype=torch.float64)))
