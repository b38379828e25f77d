"""Small Zobelorn configurations for the tests.  They differ from one another in every size, in the order
and kinds of the layers, in which layers have a feed-forward and of which kind, in windows, chunks, rotated
lanes, the scaling of the rotation, which layers borrow keys and values, and in the constants."""
import torch

import plain_zobelorn as plain
from tokenizer_b200 import write_random_model
from tokenizer_b200.config import ZobelornConfig


def windowed(heads, kv_heads, dim, vdim, scale, size=None, rot=None, softcap=None, mlp=None):
    """type "attention"; rot = (base, dims, factor or None)."""
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if size is not None:
        m["mask"] = {"size": size}
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
        if rot[2] is not None:
            m["rot"]["scaling"] = {"factor": rot[2]}
    if softcap is not None:
        m["softcap"] = softcap
    return {"type": "attention", "mixer": m, "mlp": mlp}


def chunked(heads, kv_heads, dim, vdim, scale, size=None, rot=None, kv_from=None, mlp=None):
    """type "attention_2"; rot = (base, dims, (factor, low, high, original) or None)."""
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if size is not None:
        m["mask"] = {"size": size}
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
        if rot[2] is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), rot[2]))
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention_2", "mixer": m, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


def config(layers, vocab, width, eps, scale, mult):
    return ZobelornConfig.from_dict({"architecture": "Zobelorn", "vocab": vocab, "width": width, "norm": {"eps": eps},
                                     "embedding": {"scale": scale}, "residual_mult": mult, "layers": layers})


# name -> (configuration, seed, page size)
def tiny_a():
    """A window of 24 on pages of 8 with half of every head rotated and value heads twice the keys'; chunks of
    20 whose keys a later layer of chunks of 10 borrows (the cache keeps what both can read); two of six
    experts with a shared one; a layer without a feed-forward."""
    bands = (4.0, 1.0, 3.0, 64)
    return config([windowed(6, 3, 16, 32, 0.3, size=24, rot=(10000.0, 8, 2.0), softcap=5.0, mlp=dense(136)),
                   chunked(4, 2, 24, 8, 0.21, size=20, rot=(500.0, 24, bands), mlp=moe(6, 2, 40, shared=56)),
                   chunked(4, 2, 24, 8, 0.21, size=10, rot=(500.0, 24, bands), kv_from=1)],
                  vocab=301, width=96, eps=1e-5, scale=3.0, mult=0.5), 3, 8


def tiny_b():
    """Sizes the tensor-core kernels take (cache rows of 64 and 128 lanes): chunks of 100 that do not fit the
    pages, a window of 130 with whole heads rotated and no scaling, a layer that borrows keys two layers back,
    one expert a token and no shared one, no multiplier on the residual."""
    return config([chunked(4, 2, 64, 64, 0.125, size=100, rot=(5000.0, 64, (6.0, 1.0, 3.0, 256)), mlp=moe(4, 1, 64)),
                   windowed(2, 2, 128, 96, 0.09, size=130, rot=(800000.0, 128, None), softcap=20.0, mlp=dense(256)),
                   chunked(4, 2, 64, 64, 0.11, size=100, rot=(5000.0, 64, (6.0, 1.0, 3.0, 256)), kv_from=0, mlp=dense(128))],
                  vocab=1000, width=128, eps=1e-6, scale=1.0, mult=1.0), 4, 16


def tiny_c():
    """Sizes that no vector load fits (a width of 50, a vocabulary of 77, heads of 10 and 6 lanes), a window of
    one key (a token sees itself alone), chunks of one position, no rotation in one layer and two rotated lanes
    in another, no cap, every expert chosen, pages of 32."""
    return config([windowed(3, 3, 10, 20, 0.3, size=1, rot=(100.0, 2, 4.0), mlp=dense(30)),
                   chunked(2, 1, 6, 10, 0.4, size=1, mlp=moe(3, 3, 14, shared=10)),
                   windowed(5, 1, 6, 6, 0.5, softcap=2.0, mlp=moe(5, 2, 8))],
                  vocab=77, width=50, eps=3e-6, scale=0.5, mult=0.8), 5, 32


def tiny_d():
    """Borrowing first thing: layers 1 and 3 read layer 0's keys, one with chunks of 7 (shorter than a page) and
    one seeing every key, so the cache keeps all; a window of 50 and keys wider than values; a window wider than
    any prompt; three of eight experts."""
    bands = (16.0, 2.0, 8.0, 32)
    return config([chunked(2, 1, 48, 16, 0.14, size=21, rot=(300.0, 16, bands), mlp=dense(72)),
                   chunked(4, 1, 48, 16, 0.1, size=7, rot=(300.0, 16, bands), kv_from=0, mlp=moe(8, 3, 16, shared=24)),
                   windowed(6, 3, 16, 32, 0.25, size=50, rot=(50.0, 16, 1.5), softcap=50.0),
                   chunked(2, 1, 48, 16, 0.2, rot=(300.0, 16, bands), kv_from=0, mlp=dense(40)),
                   windowed(2, 2, 32, 32, 0.18, size=4096, rot=(10000.0, 32, 8.0), mlp=dense(64))],
                  vocab=120, width=64, eps=2e-6, scale=4.0, mult=0.35), 6, 16


TINY = {"a": tiny_a, "b": tiny_b, "c": tiny_c, "d": tiny_d}
# logits of a size against which a tolerance means something, router logits that differ from token to token,
# attention that is sharp enough for a wrong key to show
SHARPEN = {r"^head$": 10.0, r"\.router$": 5.0, r"\.mix\.(q|k)$": 4.0}


def make_folder(tmp_path_factory, name, scale=SHARPEN):
    cfg, seed, page = TINY[name]()
    folder = str(tmp_path_factory.mktemp(f"zobelorn_{name}"))
    write_random_model(folder, cfg, seed, scale=scale)
    return folder, cfg, page


def reference_logits(folder, requests):
    """{request: array [len, vocab]} from the plain implementation (float64, kept as float32)."""
    cfg, weights = plain.load_folder(folder)
    return {name: plain.forward(cfg, weights, ids).to(torch.float32).numpy() for name, ids in requests.items()}
