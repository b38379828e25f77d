"""Small Vizonex configurations for the tests.  They differ from one another in every size, in the
order and kinds of the layers, in which layers have a feed-forward and of which kind, in chunk sizes,
taps, groups of experts and constants."""
import os

import torch

import plain_vizonex as plain
from tokenizer_b200 import write_random_model
from tokenizer_b200.config import VizonexConfig


def attention(heads, kv_heads, dim, vdim, scale, size=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if size is not None:
        m["mask"] = {"size": size}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def mamba2(heads, vdim, state, groups, conv, norm_groups, mlp=None):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups}, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, limit, scale, groups=None, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top, "scale": scale}}
    if groups is not None:
        m["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
    if shared is not None:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
    return m


def config(layers, vocab, width, eps, taps, positions=512):
    return VizonexConfig.from_dict({"architecture": "Vizonex", "vocab": vocab, "width": width, "max_positions": positions,
                                    "norm": {"eps": eps}, "canon": {"taps": taps}, "layers": layers})


# name -> (configuration, seed, page size)
def tiny_a():
    """Chunks of 24 on pages of 8, value heads twice as wide as key heads, three taps in front of the mixers,
    experts in three groups of which two are kept, a shared expert with a limit of its own, a layer of plain
    causal attention without a feed-forward."""
    return config([attention(6, 3, 16, 32, 0.9, size=24, mlp=dense(136)),
                   mamba2(4, 24, 16, 2, 4, 1, moe(6, 2, 40, 2.0, 1.5, groups=(3, 2), shared=(56, 1.0))),
                   attention(2, 1, 32, 16, 0.6)], vocab=301, width=96, eps=1e-5, taps=3), 3, 8


def tiny_b():
    """Sizes the tensor-core kernels take (cache rows of 64 and 128 lanes), chunks of 100 that do not fit the pages
    and of 256, a state of 128 lanes in one group, one expert a token without groups or a shared one."""
    return config([attention(4, 2, 64, 64, 0.5, size=100, mlp=moe(4, 1, 64, 3.0, 1.0)),
                   mamba2(8, 64, 128, 1, 4, 4, dense(256)),
                   attention(2, 2, 128, 96, 0.35, size=256, mlp=dense(128))], vocab=1000, width=128, eps=1e-6, taps=4), 4, 16


def tiny_c():
    """Sizes that no vector load fits (a width of 50, a vocabulary of 77, heads of 10, 6 and 5 lanes), one tap in
    front of the mixers (nothing kept) and a recurrence with one tap too, chunks of one position (a token sees
    itself and the sink alone), every expert chosen, as many norm parts and groups as heads, pages of 32."""
    return config([attention(3, 3, 10, 20, 1.2, size=1, mlp=dense(30)),
                   mamba2(3, 10, 6, 3, 1, 3, moe(3, 3, 14, 0.7, 2.5, groups=(1, 1), shared=(10, 0.5))),
                   mamba2(2, 5, 40, 1, 5, 2)], vocab=77, width=50, eps=3e-6, taps=1), 5, 32


def tiny_d():
    """The recurrence first, with a state of 256 lanes and heads of 40 (more than a block's columns); chunks of 7
    (shorter than a page) and of 50 in two cache groups of unlike rows, keys wider than values, five taps, eight
    experts in four groups of which two are kept."""
    return config([mamba2(2, 40, 256, 2, 2, 2, moe(8, 3, 16, 1.5, 0.8, groups=(4, 2), shared=(24, 2.5))),
                   attention(2, 1, 48, 16, 0.4, size=7, mlp=dense(72)),
                   attention(6, 3, 16, 32, 0.8, size=50, mlp=moe(4, 2, 24, 1.0, 1.0, groups=(2, 2))),
                   mamba2(4, 16, 32, 4, 3, 1, dense(40))], vocab=120, width=64, eps=2e-6, taps=5), 6, 16


TINY = {"a": tiny_a, "b": tiny_b, "c": tiny_c, "d": tiny_d}
# logits of a size against which a tolerance means something, router logits that differ from token to token
SHARPEN = {r"^head$": 10.0, r"\.router$": 5.0}


def settle_routing(folder, cfg):
    """Make every token's CHOICE of experts safe from rounding, so that bfloat16 runs can be compared (where two
    choice scores nearly tie, rounding anywhere upstream decides, and the outputs differ by an expert): the
    correction of `top` favoured experts, taken group by group from as many groups as are kept, is lifted by 3,
    far above what a score in (0, 1) can make up.  The weights, which leave the correction out, still vary from
    token to token.  Which experts a token chooses varies in the runs without this (float32)."""
    from tokenizer_b200.weights.safetensors_io import read_safetensors, write_safetensors
    path = os.path.join(folder, "model.safetensors")
    tensors = dict(read_safetensors(path))
    for index, layer in enumerate(cfg.layers):
        mlp = layer.get("mlp")
        if not mlp or mlp["kind"] != "moe":
            continue
        router = mlp["router"]
        experts, top = router["experts"], router["top"]
        groups = router.get("groups") or {"count": 1, "keep": 1}
        size = experts // groups["count"]
        first = (index + 1) % groups["count"]
        favoured = []
        for k in range(groups["keep"]):
            g = (first + k) % groups["count"]
            favoured += [g * size + (index + j) % size for j in range(size)]
        # one expert of every kept group first, so that every kept group is safely among the best
        order = sorted(range(len(favoured)), key=lambda i: (i % size, i // size))
        favoured = [favoured[i] for i in order][:top]
        correction = tensors[f"l{index}.mlp.correction"].clone()
        correction[favoured] += 3.0
        tensors[f"l{index}.mlp.correction"] = correction
    write_safetensors(path, tensors)


def make_folder(tmp_path_factory, name, scale=SHARPEN, settled=True):
    cfg, seed, page = TINY[name]()
    folder = str(tmp_path_factory.mktemp(f"vizonex_{name}"))
    write_random_model(folder, cfg, seed, scale=scale)
    if settled:
        settle_routing(folder, cfg)
    return folder, cfg, page


def reference_logits(folder, requests):
    """{request: array [len, vocab]} from the plain implementation (float64, kept as float32)."""
    cfg, weights = plain.load_folder(folder)
    return {name: plain.forward(cfg, weights, ids).to(torch.float32).numpy() for name, ids in requests.items()}
