"""A plain, slow restatement of the Zobelorn decoder on the CPU, one function per mechanism.  It
reads config.json and the weight file itself and shares nothing with the engine: it is what the
engine is compared with.

Everything is computed in float64 unless `dtype` says otherwise, so that it stands between the
engine's two precisions as the exact answer.  A sequence is always run whole, from position 0.
"""
import json
import math
import os

import torch


def load_folder(folder, dtype=torch.float64):
    from safetensors.torch import load_file
    with open(os.path.join(folder, "config.json")) as fh:
        cfg = json.load(fh)
    weights = {k: (v.to(dtype) if v.is_floating_point() else v)
               for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    return cfg, weights


# ---- mechanisms ---------------------------------------------------------------------------
def linear(x, w):
    return x @ w.t()


def sigmoid(x):
    return 1.0 / (1.0 + torch.exp(-x))


def silu(x):
    return x * sigmoid(x)


def root_mean_square_norm(x, eps, gain=None):
    """x / sqrt(mean(x^2) + eps) over the last axis, times `gain` where there is one."""
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if gain is None else y * gain


def layer_norm_one_plus(x, w, eps):
    """The layers' norm: the gain is one plus the tensor."""
    return root_mean_square_norm(x, eps, 1.0 + w)


def linear_frequencies(base, dims, factor):
    """f_i = base^(-2i / dims) / factor, i < dims / 2."""
    return [base ** (-2.0 * i / dims) / factor for i in range(dims // 2)]


def banded_frequencies(base, dims, factor, low, high, original):
    """f_i = base^(-2i / dims), left alone where its wavelength is shorter than original / high, divided
    by `factor` where it is longer than original / low, and blended in between."""
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        wavelength = 2.0 * math.pi / f
        if wavelength < original / high:
            out.append(f)
        elif wavelength > original / low:
            out.append(f / factor)
        else:
            s = (original / wavelength - low) / (high - low)
            out.append((1.0 - s) * f / factor + s * f)
    return out


def rotate(x, positions, freqs, layout):
    """x [T, heads, dim]; the first 2 * len(freqs) lanes of every head are rotated by the angle position *
    f_i.  `layout` "half": lane i pairs with lane i + len(freqs); "interleaved": lane 2i with 2i + 1."""
    n = len(freqs)
    if n == 0:
        return x
    angle = positions.to(x.dtype)[:, None] * torch.tensor(freqs, dtype=x.dtype)[None, :]     # [T, n]
    c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    out = x.clone()
    if layout == "half":
        u, v = x[..., :n], x[..., n:2 * n]
        out[..., :n], out[..., n:2 * n] = u * c - v * s, v * c + u * s
    else:
        u, v = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
        out[..., 0:2 * n:2], out[..., 1:2 * n:2] = u * c - v * s, v * c + u * s
    return out


def visible_window(n, size):
    """[n, n] booleans: query i sees key j when 0 <= i - j < size."""
    i, j = torch.arange(n)[:, None], torch.arange(n)[None, :]
    return (j <= i) & (i - j < size)


def visible_chunk(n, size):
    """[n, n] booleans: query i sees key j <= i of its own chunk of `size` positions counted from 0."""
    i, j = torch.arange(n)[:, None], torch.arange(n)[None, :]
    return (j <= i) & (i // size == j // size)


def attend(q, k, v, visible, scale, softcap=None):
    """q [T, H, dim], k [T, G, dim], v [T, G, vdim]; query head h reads key/value head h // (H / G).
    Scores q . k * scale, through softcap * tanh(. / softcap) where there is one; softmax over the
    visible keys.  Returns [T, H * vdim]."""
    T, H, _ = q.shape
    G = k.shape[1]
    rows = []
    for h in range(H):
        g = h // (H // G)
        score = (q[:, h] @ k[:, g].t()) * scale
        if softcap is not None:
            score = softcap * torch.tanh(score / softcap)
        score = score.masked_fill(~visible, float("-inf"))
        rows.append(torch.softmax(score, dim=-1) @ v[:, g])
    return torch.stack(rows, dim=1).reshape(T, -1)


def windowed_attention(h, w, prefix, m, eps, positions):
    """Mixer "attention": norms over the whole q and k projections, the half layout of the rotation
    with every frequency divided by a factor, capped scores, a sliding window, a sigmoid gate on the
    heads' outputs.  Returns the mixer's output and (keys, values) as a cache would hold them."""
    T = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = root_mean_square_norm(linear(h, w[prefix + ".q"]), eps, w[prefix + ".q.norm"])
    k = root_mean_square_norm(linear(h, w[prefix + ".k"]), eps, w[prefix + ".k.norm"])
    v = linear(h, w[prefix + ".v"]).view(T, G, vdim)
    rot = m.get("rot")
    freqs = []
    if rot is not None:
        factor = (rot.get("scaling") or {}).get("factor", 1.0)
        freqs = linear_frequencies(rot["base"], rot["dims"], factor)
    q = rotate(q.view(T, H, dim), positions, freqs, "half")
    k = rotate(k.view(T, G, dim), positions, freqs, "half")
    size = m["mask"]["size"] if m.get("mask") is not None else T + 1
    mixed = attend(q, k, v, visible_window(T, size), m["scale"], m.get("softcap"))
    mixed = mixed * sigmoid(linear(h, w[prefix + ".g"]))
    return linear(mixed, w[prefix + ".o"]), (k, v)


def chunked_attention(h, w, prefix, m, eps, positions, borrowed=None):
    """Mixer "attention_2": the interleaved layout of the rotation with frequencies scaled by bands,
    queries and keys divided by their root mean square a head after the rotation, keys seen inside
    chunks.  With `borrowed` (keys, values) of an earlier layer it projects queries only."""
    T = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot = m.get("rot")
    freqs = []
    if rot is not None:
        s = rot.get("scaling")
        if s is None:
            freqs = linear_frequencies(rot["base"], rot["dims"], 1.0)
        else:
            freqs = banded_frequencies(rot["base"], rot["dims"], s["factor"], s["low"], s["high"], s["original"])
    q = linear(h, w[prefix + ".q"]).view(T, H, dim)
    q = root_mean_square_norm(rotate(q, positions, freqs, "interleaved"), eps)
    if borrowed is None:
        k = linear(h, w[prefix + ".k"]).view(T, G, dim)
        k = root_mean_square_norm(rotate(k, positions, freqs, "interleaved"), eps)
        v = linear(h, w[prefix + ".v"]).view(T, G, vdim)
    else:
        k, v = borrowed
    size = m["mask"]["size"] if m.get("mask") is not None else None
    visible = visible_chunk(T, size) if size is not None else visible_window(T, T + 1)
    return linear(attend(q, k, v, visible, m["scale"]), w[prefix + ".o"]), (k, v)


def gated_feed_forward(h, w, prefix):
    return linear(silu(linear(h, w[prefix + ".gate"])) * linear(h, w[prefix + ".up"]), w[prefix + ".down"])


def routed_feed_forward(h, w, prefix, mlp):
    """Scores sigmoid(W_router h); the `top` largest choose the experts (ties: the lower index); an
    expert's score multiplies its INPUT; a shared expert, where there is one, counts for every token."""
    experts, top = mlp["router"]["experts"], mlp["router"]["top"]
    score = sigmoid(linear(h, w[prefix + ".router"]))                # [T, experts]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        order = sorted(range(experts), key=lambda e: (-float(score[t, e]), e))[:top]
        for e in order:
            out[t] = out[t] + gated_feed_forward(score[t, e] * h[t:t + 1], w, f"{prefix}.e{e}")[0]
    if mlp.get("shared") is not None:
        out = out + gated_feed_forward(h, w, prefix + ".shared")
    return out


def feed_forward(h, w, prefix, mlp):
    if mlp["kind"] == "dense":
        return gated_feed_forward(h, w, prefix)
    return routed_feed_forward(h, w, prefix, mlp)


# ---- the model ----------------------------------------------------------------------------
def forward(cfg, w, tokens, layers_out=None):
    """Logits [T, vocab] of a whole sequence from position 0.  `layers_out`: a list that receives
    the residual stream after every layer."""
    dtype = w["embed"].dtype
    eps, mult = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    ids = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(len(tokens))
    x = w["embed"][ids] * (cfg.get("embedding") or {}).get("scale", 1.0)
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}", layer["mixer"]
        h = layer_norm_one_plus(x, w[p + ".norm1"], eps)
        if layer["type"] == "attention":
            y, kept[i] = windowed_attention(h, w, p + ".mix", m, eps, positions)
        elif layer["type"] == "attention_2":
            source = m.get("kv_from")
            y, kv = chunked_attention(h, w, p + ".mix", m, eps, positions, None if source is None else kept[source])
            if source is None:
                kept[i] = kv
        else:
            raise ValueError(layer["type"])
        x = x + mult * layer_norm_one_plus(y, w[p + ".norm1b"], eps)
        if layer.get("mlp") is not None:
            h = layer_norm_one_plus(x, w[p + ".norm2"], eps)
            x = x + mult * layer_norm_one_plus(feed_forward(h, w, p + ".mlp", layer["mlp"]), w[p + ".norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return linear(layer_norm_one_plus(x, w["final.norm"], eps), w["head"]).to(dtype)
