"""Gated feed-forward: down(act(gate(x)) * up(x)), no biases; the gate and up
products are one stacked product (reference: qwen-infer/src/model.rs:226-250,
silu(z) = z * sigmoid(z)).  The activation is a parameter of the part and of the kernels
behind it (`ops.ACTIVATIONS`); the architecture served asks for silu."""
from __future__ import annotations

import os

import torch

from ..config.spec import ConfigError
from ..kernels import ops
from ..weights.store import TensorSpec
from .base import register_part
from .linear import Linear
from .recurrent import SideProjection


# TOKB200_FFN=separate runs the feed-forward of few rows as norm, gate/up and down kernels
_FUSED_STEP = os.environ.get("TOKB200_FFN", "fused") != "separate"
# Where the one-kernel feed-forward leads the separate kernels (norm, gate/up with activation, down),
# measured: up to 8 rows of a narrow stream (hidden 896: 0.69 against 0.74 ms a decoding step of 24
# layers).  With 9 to 16 rows it trails (0.91 against 0.86 ms), and so it does on a wider stream,
# where every block's own norm of all rows costs more than a launch (hidden 1,536, 32 requests with
# portions of 512 tokens: 0.63 against 0.56 s).
FUSED_ROWS = 8
FUSED_HIDDEN = 1024


def _names(spec):
    """The three matrices' names behind the prefix: `params["names"]` = (gate, up, down) where the
    file names them otherwise than `.gate_proj.weight`, `.up_proj.weight`, `.down_proj.weight`."""
    return tuple(spec.params.get("names") or (".gate_proj.weight", ".up_proj.weight", ".down_proj.weight"))


class GatedMLP:
    @staticmethod
    def tensors(spec):
        p, x = spec.params, spec.prefix
        gate, up, down = _names(spec)
        return [
            TensorSpec(x + gate, (p["intermediate_size"], p["hidden_size"])),
            TensorSpec(x + up, (p["intermediate_size"], p["hidden_size"])),
            TensorSpec(x + down, (p["hidden_size"], p["intermediate_size"])),
        ]

    def __init__(self, spec, store, runtime):
        p, x = spec.params, spec.prefix
        if p["activation"] not in ops.ACTIVATIONS:
            raise ConfigError(f"gated feed-forward knows the activations {', '.join(ops.ACTIVATIONS)}; "
                              f"found {p['activation']}")
        self.activation = p["activation"]
        self.runtime = runtime
        self.inner = int(p["intermediate_size"])
        gate_name, up_name, down_name = _names(spec)
        gate, up = store.get(x + gate_name), store.get(x + up_name)
        hidden = int(p["hidden_size"])
        # bfloat16 with sizes the gated kernels take: the activation is folded into the
        # product's epilogue and the stacked weight is laid out for that
        self.fused = runtime.dtype == torch.bfloat16 and self.inner % 128 == 0 and \
            ops.gated_linear_supported(hidden, 2 * self.inner)
        if self.fused:
            self.gate_up_weight = ops.interleave_gate_up(runtime.matrix(gate), runtime.matrix(up))
        else:
            self.gate_up = Linear(runtime.matrix(torch.cat([gate, up], dim=0)))
        self.down = Linear(runtime.matrix(store.get(x + down_name)))

    def fused_step(self, stream, norm) -> bool:
        """For few rows in bfloat16: residual add, norm, both products and the activation
        in one kernel, straight from the stream (the norm must be one that can be folded:
        it offers `folded() -> (gain, eps)` of an RMS norm).  True when it was done; the
        stream then holds the new sum and this part's output as pending partial sums."""
        fold = getattr(norm, "folded", None)
        if not (_FUSED_STEP and self.fused and fold is not None):
            return False
        x = stream.x
        rows, hidden = x.shape
        if rows > FUSED_ROWS or hidden > FUSED_HIDDEN:
            return False
        splits = ops.ffn_small_m_splits(rows, hidden, self.inner)
        if splits == 0:
            return False
        gain, eps = fold()
        delta, stream.pending = stream.pending, None
        x_out = torch.empty_like(x)
        out = torch.empty((splits, rows, hidden), dtype=torch.float32, device=x.device)
        ops.ffn_small_m(x, x_out, delta, gain, eps, self.gate_up_weight, self.down.weight, out,
                        self.activation)
        stream.x, stream.pending = x_out, out
        return True

    def gated_operands(self):
        """(gate/up weight in the gated kernels' interleaved row order, down weight, activation)
        for a kernel that computes this feed-forward inside a larger fusion; None when the sizes
        or the precision have no such layout."""
        if not (_FUSED_STEP and self.fused):
            return None
        return self.gate_up_weight, self.down.weight, self.activation

    def streamed_weights(self):
        """What a second stream may bring into L2 ahead of a step of few rows: nothing when
        the fused kernel runs, which streams its weights itself from its first cycle."""
        if _FUSED_STEP and self.fused:
            return []
        return [self.gate_up_weight if self.fused else self.gate_up.weight, self.down.weight]

    def forward(self, h):
        act = self.runtime.empty(h.shape[0], self.inner)
        if self.fused:
            ops.gated_linear(h, self.gate_up_weight, act, self.activation)
        else:
            ops.silu_gate(self.gate_up.forward(h), act, self.activation)
        return self.down.forward(act, partials_ok=True)


class PolyNormMLP(SideProjection):
    """Dense feed-forward down(act(up(h) + b_up)) + b_down with the PolyNorm activation: for a
    token's vector z, a N(z) + b N(z^2) + c N(z^3) + e, powers taken element by element and
    N(v) = v / sqrt(mean(v^2) + eps) over the vector; the four numbers are a tensor of the model.
    The mean squares and the sum are 32-bit (`csrc/activation.cu`).  With a side projection taken
    (`take_side`), the down product's bias is left to the consumer (`deferred_bias`), so that the
    product may come as partial sums."""

    @staticmethod
    def tensors(spec):
        p, x = spec.params, spec.prefix
        return [TensorSpec(x + ".up", (p["inner_size"], p["hidden_size"])), TensorSpec(x + ".up.b", (p["inner_size"],)),
                TensorSpec(x + ".down", (p["hidden_size"], p["inner_size"])),
                TensorSpec(x + ".down.b", (p["hidden_size"],)), TensorSpec(x + ".act", (4,), "normal", 0.5)]

    def __init__(self, spec, store, runtime):
        p, x = spec.params, spec.prefix
        self.runtime = runtime
        self.inner, self.eps = int(p["inner_size"]), float(p["eps"])
        self._own = ([store.get(x + ".up")], [store.get(x + ".up.b")])
        self.up = self._stack(runtime, list(self._own[0]), list(self._own[1]), None)
        self.down = Linear(runtime.matrix(store.get(x + ".down")), runtime.vector(store.get(x + ".down.b")))
        self.coeff = runtime.vector(store.get(x + ".act"))
        self.deferred_bias = None

    def take_side(self, weight, bias):
        self.up = self._stack(self.runtime, list(self._own[0]), list(self._own[1]), (weight, bias))
        self.deferred_bias = self.down.bias

    def streamed_weights(self):
        return [self.up.weight, self.down.weight]

    def forward(self, h):
        z = self.up.forward(h, out_dtype=torch.float32)
        act = self.runtime.empty(h.shape[0], self.inner)
        ops.poly_norm(z[:, :self.inner], self.coeff, self.eps, act,
                      bias=self.stack_bias[:self.inner] if self.stack_bias is not None else None)
        self._keep_side(z)
        if self.deferred_bias is not None:
            return self.down.forward(act, use_bias=False, partials_ok=True)
        return self.down.forward(act)


class RoutedMLP:
    """A feed-forward of `experts` small gated feed-forwards (`<prefix>.e<i>.gate`, `.up`, `.down`,
    inner size `expert_inner`, no biases), of which every token uses the `top` with the largest
    router logits z = W_router h (32-bit sums), weighed by the softmax over those logits alone; and,
    with `shared_inner`, one more of that form (`<prefix>.shared.*`) that every token uses, scaled by
    sigmoid(W_sg h) (`.shared.sg`, one row).

    How it is computed: as ONE gated feed-forward whose inner lanes are all experts' lanes side by
    side, the shared expert's behind them.  The gate/up product is one stacked product; every inner
    lane is then scaled by its expert's share for the token, zero for an expert the token did not
    choose (`csrc/moe.cu`); the down product over all lanes is the weighted sum of the chosen
    experts' outputs.  Nothing depends on values read back to the host, so a step can be captured.
    It costs experts / top times the routed experts' arithmetic: what a model of few experts pays
    for products of full size instead of a product per expert over gathered rows.

    Parameters beyond the sizes: `score` ("softmax_of_chosen" as above; "sigmoid": scores
    s = sigmoid(z), the choice made on s + `<prefix>.correction` (with `correction`) among the experts
    of the `group_keep` best of `groups` equal groups of neighbours, a group's worth the sum of its two
    largest choice scores, weights s * `route_scale`, not renormalized); `shared_gate` (False: the shared
    expert counts fully and `.shared.sg` does not exist); `activation` (one of `ops.MOE_ACTIVATIONS`;
    "clamped_swish" with `limit`, `shared_limit` and `alpha`: g = min(gate, limit), u = clamp(up, -limit,
    limit), g sigmoid(alpha g) (u + 1)); `share_on` ("output": an expert's output is multiplied by its weight;
    "input": its input is, expert(w h), which for products without biases is act(w gate) * (w up) on its inner
    lanes and an unweighted sum behind the down product)."""

    @staticmethod
    def tensors(spec):
        p, x = spec.params, spec.prefix
        hidden, inner = p["hidden_size"], p["expert_inner"]
        out = []
        for e in range(p["experts"]):
            out += [TensorSpec(f"{x}.e{e}.gate", (inner, hidden)), TensorSpec(f"{x}.e{e}.up", (inner, hidden)),
                    TensorSpec(f"{x}.e{e}.down", (hidden, inner))]
        out.append(TensorSpec(x + ".router", (p["experts"], hidden)))
        if p.get("shared_inner"):
            s = p["shared_inner"]
            out += [TensorSpec(x + ".shared.gate", (s, hidden)), TensorSpec(x + ".shared.up", (s, hidden)),
                    TensorSpec(x + ".shared.down", (hidden, s))]
            if p.get("shared_gate", True):
                out.append(TensorSpec(x + ".shared.sg", (1, hidden)))
        if p.get("correction"):
            out.append(TensorSpec(x + ".correction", (p["experts"],), "normal", 0.1))
        return out

    def __init__(self, spec, store, runtime):
        p, x = spec.params, spec.prefix
        self.runtime = runtime
        self.experts, self.top, self.ff = int(p["experts"]), int(p["top"]), int(p["expert_inner"])
        self.shared = int(p.get("shared_inner") or 0)
        self.activation = p.get("activation", "silu")
        if self.activation not in ops.MOE_ACTIVATIONS:
            raise ConfigError(f"routed feed-forward knows the activations {', '.join(ops.MOE_ACTIVATIONS)}; "
                              f"found {self.activation}")
        if not 1 <= self.top <= self.experts or self.experts > 1024:
            raise ConfigError(f"a token uses 1 .. experts of at most 1024 experts; found top {self.top} of {self.experts}")
        self.score = p.get("score", "softmax_of_chosen")
        self.groups, self.group_keep = int(p.get("groups", 1)), int(p.get("group_keep", 1))
        self.route_scale = float(p.get("route_scale", 1.0))
        self.limit, self.shared_limit = float(p.get("limit", 0.0)), float(p.get("shared_limit", 0.0))
        self.alpha = float(p.get("alpha", 1.0))
        self.share_on = p.get("share_on", "output")
        if self.share_on not in ("output", "input"):
            raise ConfigError(f"an expert's weight multiplies its output or its input; found {self.share_on}")
        if self.score not in ops.MOE_SCORES:
            raise ConfigError(f"a router scores by one of {', '.join(ops.MOE_SCORES)}; found {self.score}")
        if self.groups < 1 or self.experts % self.groups or not 1 <= self.group_keep <= self.groups or \
                self.group_keep * (self.experts // self.groups) < self.top:
            raise ConfigError(f"{self.experts} experts in {self.groups} equal groups of which {self.group_keep} are kept "
                              f"cannot give a token {self.top} experts")
        self.shared_mode = None if not self.shared else "gated" if p.get("shared_gate", True) else "one"
        self.correction = runtime.vector(store.get(x + ".correction")) if p.get("correction") else None
        names = [f"{x}.e{e}" for e in range(self.experts)] + ([x + ".shared"] if self.shared else [])
        self.inner = self.experts * self.ff + self.shared
        gates = torch.cat([store.get(n + ".gate") for n in names], dim=0)
        ups = torch.cat([store.get(n + ".up") for n in names], dim=0)
        self.gate_up = Linear(runtime.matrix(torch.cat([gates, ups], dim=0)))
        self.down = Linear(runtime.matrix(torch.cat([store.get(n + ".down") for n in names], dim=1)))
        rows = [store.get(x + ".router")] + ([store.get(x + ".shared.sg")] if self.shared_mode == "gated" else [])
        self.router = runtime.vector(torch.cat(rows, dim=0))       # float32: the logits are 32-bit

    def streamed_weights(self):
        return [self.gate_up.weight, self.down.weight]

    def forward(self, h):
        n = h.shape[0]
        share = torch.empty((n, self.experts + (1 if self.shared else 0)), dtype=torch.float32, device=h.device)
        ops.moe_route(h, self.router, self.experts, self.top, self.shared_mode, share, score=self.score,
                      correction=self.correction, groups=self.groups, keep=self.group_keep, scale=self.route_scale)
        act = self.runtime.empty(n, self.inner)
        ops.moe_gate(self.gate_up.forward(h), share, act, self.experts, self.ff, bool(self.shared), self.activation,
                     limit=self.limit, shared_limit=self.shared_limit, alpha=self.alpha,
                     on_input=self.share_on == "input")
        return self.down.forward(act, partials_ok=True)


register_part("feed_forward", "gated_mlp", GatedMLP)
register_part("feed_forward", "routed_mlp", RoutedMLP)
register_part("feed_forward", "poly_norm_mlp", PolyNormMLP)
