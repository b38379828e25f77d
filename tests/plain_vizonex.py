"""A plain, slow restatement of the Vizonex decoder on the CPU, one function per mechanism,
token by token where a mechanism is a recurrence.  It reads config.json and the weight file
itself and shares nothing with the engine: it is what the engine is compared with.

Everything is computed in float64, so that it stands between the engine's two precisions as the
exact answer.
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


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def causal_convolution(x, taps, bias=None):
    """Over time, channel by channel, from a sequence's start.  x [T, C], taps [C, n]: column n - 1
    weighs the current token, column 0 the token n - 1 back; zeros before the start."""
    T, n = x.shape[0], taps.shape[1]
    full = torch.cat([torch.zeros(n - 1, x.shape[1], dtype=x.dtype), x], dim=0)
    out = torch.zeros_like(x)
    for j in range(n):
        out = out + full[j:j + T] * taps[:, j]
    return out if bias is None else out + bias


def sink_chunk_attention(q, k, v, scale, temp, sink, chunk):
    """q [T, H, d], k [T, G, d], v [T, G, dv]; query head h reads key/value head h // (H / G).
    Position i sees j <= i inside its own chunk of `chunk` positions counted from 0 (None: every
    j <= i).  Weights exp(score) / (sum of exp(score) + exp(sink_h)), score = q . k * scale * temp_h."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            first = 0 if chunk is None else i - i % chunk
            s = (k[first:i + 1, g] @ q[i, h]) * scale * temp[h]
            top = torch.maximum(s.max(), sink[h])
            e = torch.exp(s - top)
            out[i, h] = (e[:, None] * v[first:i + 1, g]).sum(dim=0) / (e.sum() + torch.exp(sink[h] - top))
    return out


def attention_mixer(h, w, p, m, eps):
    heads, groups, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = rms(linear(h, w[p + "q"]), eps) * w[p + "q.norm"]          # over the whole projection
    k = rms(linear(h, w[p + "k"]), eps) * w[p + "k.norm"]
    v = linear(h, w[p + "v"])
    chunk = m["mask"]["size"] if m.get("mask") else None
    o = sink_chunk_attention(q.view(T, heads, dim), k.view(T, groups, dim), v.view(T, groups, vdim),
                             m["scale"], w[p + "temp"], w[p + "sink"], chunk)
    return linear(o.reshape(T, heads * vdim), w[p + "o"])


def selective_state_space(x, B, C, dt, a, d):
    """One head.  x [T, P], B and C [T, N], dt [T] (after softplus), a = exp(A_log), d the skip.
    S_t = exp(-a dt_t) S_(t-1) + dt_t B_t x_t^T (N x P, from zero); y_t = S_t^T C_t + d x_t."""
    S = torch.zeros(B.shape[1], x.shape[1], dtype=x.dtype)
    rows = []
    for t in range(x.shape[0]):
        S = torch.exp(-a * dt[t]) * S + dt[t] * torch.outer(B[t], x[t])
        rows.append(S.t() @ C[t] + d * x[t])
    return torch.stack(rows)


def mamba2_mixer(h, w, p, m, eps):
    heads, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner, T = heads * P, h.shape[0]
    z, xbc, dt = torch.split(linear(h, w[p + "in"]), [inner, inner + 2 * G * N, heads], dim=1)
    xbc = silu(causal_convolution(xbc, w[p + "conv"], w[p + "conv.b"]))
    x, B, C = torch.split(xbc, [inner, G * N, G * N], dim=1)
    x, B, C = x.view(T, heads, P), B.view(T, G, N), C.view(T, G, N)
    dt = softplus(dt + w[p + "dt_bias"])
    ys = []
    for head in range(heads):
        g = head // (heads // G)
        ys.append(selective_state_space(x[:, head], B[:, g], C[:, g], dt[:, head], torch.exp(w[p + "A_log"][head]),
                                        w[p + "D"][head]))
    y = torch.cat(ys, dim=1) * silu(z)                                 # the gate comes before the norm
    parts = m["norm_groups"]
    y = rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"]
    return linear(y, w[p + "o"])


def clamped_expert(h, w, p, limit):
    g = torch.clamp(linear(h, w[p + "gate"]), max=limit)
    u = torch.clamp(linear(h, w[p + "up"]), min=-limit, max=limit)
    return linear(g * sigmoid(1.702 * g) * (u + 1.0), w[p + "down"])


def route(h, w, p, r):
    """Per token the chosen experts and their weights: scores sigmoid(W_router h); the choice is made
    on scores + correction, among the experts of the `keep` groups (of `count` equal groups of
    neighbours) whose two largest choice scores add up to the most; weights are the plain scores
    times `scale`."""
    s = sigmoid(linear(h, w[p + "router"]))
    choice = s + w[p + "correction"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    E, count, keep = r["experts"], groups["count"], groups["keep"]
    grouped = choice.view(-1, count, E // count)
    group_score = grouped.topk(min(2, E // count), dim=-1).values.sum(dim=-1)
    kept = group_score.topk(keep, dim=-1).indices
    allowed = torch.zeros_like(group_score, dtype=torch.bool).scatter(1, kept, True)
    masked = torch.where(allowed[:, :, None].expand_as(grouped), grouped, torch.full_like(grouped, -math.inf))
    chosen = masked.reshape(-1, E).topk(r["top"], dim=-1).indices
    return chosen, s.gather(1, chosen) * r["scale"]


def feed_forward(h, w, p, mlp):
    if mlp["kind"] == "dense":
        return linear(gelu_tanh(linear(h, w[p + "gate"])) * linear(h, w[p + "up"]), w[p + "down"])
    chosen, weights = route(h, w, p, mlp["router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, share in zip(chosen[t].tolist(), weights[t]):
            out[t] = out[t] + share * clamped_expert(h[t:t + 1], w, f"{p}e{e}.", mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        out = out + clamped_expert(h, w, p + "shared.", mlp["shared"]["limit"])
    return out


def layer(x, w, i, spec, cfg):
    eps = cfg["norm"]["eps"]
    h = rms(x, eps) * w[f"l{i}.norm1"]
    read = h + causal_convolution(h, w[f"l{i}.canon1"])
    mixer = attention_mixer if spec["type"] == "attention" else mamba2_mixer
    x = x + w[f"l{i}.ls1"] * mixer(read, w, f"l{i}.mix.", spec["mixer"], eps)
    if spec.get("mlp") is not None:
        x = x + w[f"l{i}.ls2"] * feed_forward(h, w, f"l{i}.mlp.", spec["mlp"])
    return x


def forward(cfg, w, tokens, keep_layers=False):
    """Logits [T, vocab] of a whole sequence from its start (and the stream after every layer)."""
    ids = torch.tensor(tokens, dtype=torch.long)
    x = w["embed"][ids] + w["pos"][:len(tokens)]
    kept = []
    for i, spec in enumerate(cfg["layers"]):
        x = layer(x, w, i, spec, cfg)
        kept.append(x)
    logits = linear(rms(x, cfg["norm"]["eps"]) * w["final.norm"], w["head"])
    return (logits, torch.stack(kept)) if keep_layers else logits
