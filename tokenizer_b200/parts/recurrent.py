"""Recurrent mixers: minGRU and the gated delta rule (`GatedDeltaNet`, below).

minGRU: a gated recurrence whose gates read only the current token.

For a token's input h: z = sigmoid(Wz h + bz), u = Wx h + bx, candidate = u + 1/2 where u >= 0 and
sigmoid(u) below, state S_t = (1 - z) S_(t-1) + z candidate element by element, output
Wo (S_t * silu(Wg h)).  The state has `width` lanes, starts at zero, is float32 and lives in the
request's state slot.  The three input projections are one stacked product (a fourth may ride
along, see `take_side`); gates, candidate, recurrence and the product with silu are one kernel
(`csrc/recurrence.cu`), 32-bit whatever the products' precision.
"""
from __future__ import annotations

import os

import torch

from ..config.spec import ConfigError
from ..kernels import ops
from ..weights.store import TensorSpec
from .base import CacheNeed, StateNeed, register_part
from .linear import Linear


class SideProjection:
    """Mixers and feed-forwards whose first step is a product of their input may carry one more
    projection of the same input in that product (`take_side(weight, bias)`, CPU tensors as
    stored): its result of the last `forward` is `side_pre` [T, rows of weight], float32, still
    lacking `side_bias`.  The arrangement of a layer uses it for a gate on the sublayer's output.
    The stacked product is computed WITHOUT its biases: `stack_bias` (float32, one a column, or
    None) is added by the kernels that consume the columns, which spares a pass over the product."""

    side_rows = 0
    side_pre = None
    side_bias = None
    stack_bias = None

    def _stack(self, runtime, weights, biases, side):
        """One Linear over `weights` stacked row-wise (+ the side projection); `biases` are
        per-weight float tensors or None (zeros)."""
        self.side_rows = 0
        if side is not None:
            weights, biases = weights + [side[0]], biases + [side[1]]
            self.side_rows = side[0].shape[0]
        self.own_rows = sum(w.shape[0] for w in weights) - self.side_rows
        self.stack_bias = self.side_bias = None
        if any(b is not None for b in biases):
            bias = torch.cat([torch.zeros(w.shape[0], dtype=torch.float32, device=w.device) if b is None
                              else b.to(torch.float32) for w, b in zip(weights, biases)])
            self.stack_bias = runtime.vector(bias)
            if self.side_rows and biases[-1] is not None:
                self.side_bias = self.stack_bias[self.own_rows:]
        return Linear(runtime.matrix(torch.cat(weights, dim=0)))

    def _keep_side(self, product):
        self.side_pre = product[:, self.own_rows:] if self.side_rows else None


class MinGRU(SideProjection):
    graph_safe = True    # launches depend on device-side metadata alone

    @staticmethod
    def tensors(spec):
        p, x = spec.params, spec.prefix
        hidden, width = p["hidden_size"], p["width"]
        return [TensorSpec(x + ".z", (width, hidden)), TensorSpec(x + ".z.b", (width,)),
                TensorSpec(x + ".x", (width, hidden)), TensorSpec(x + ".x.b", (width,)),
                TensorSpec(x + ".g", (width, hidden)), TensorSpec(x + ".o", (hidden, width))]

    def __init__(self, spec, store, runtime):
        p, x = spec.params, spec.prefix
        self.runtime = runtime
        self.hidden, self.width = int(p["hidden_size"]), int(p["width"])
        self._own = ([store.get(x + ".z"), store.get(x + ".x"), store.get(x + ".g")],
                     [store.get(x + ".z.b"), store.get(x + ".x.b"), None])
        self.inputs = self._stack(runtime, list(self._own[0]), list(self._own[1]), None)
        self.out = Linear(runtime.matrix(store.get(x + ".o")))

    def take_side(self, weight, bias):
        self.inputs = self._stack(self.runtime, list(self._own[0]), list(self._own[1]), (weight, bias))

    def cache_need(self):
        return CacheNeed(state=StateNeed((self.width,)))

    def shape_key(self, q_lens):
        return "scan1" if max(q_lens) == 1 else "scan"

    def streamed_weights(self):
        return [self.inputs.weight, self.out.weight]

    def forward(self, h, ctx, cache):
        w = self.width
        product = self.inputs.forward(h, out_dtype=torch.float32)
        y = self.runtime.empty(ctx.n_tokens, w)
        ops.min_gru_scan(product, 0, w, 2 * w, w, cache.state, ctx.q_start, ctx.state_slot,
                         max(ctx.max_q_len, 1), y, bias=self.stack_bias)
        self._keep_side(product)
        return self.out.forward(y, partials_ok=True)


# TOKB200_GDN_STEP=separate runs a step of single tokens through the kernels for portions too
_ONE_KERNEL_STEP = os.environ.get("TOKB200_GDN_STEP", "fused") != "separate"


def stacked_rows(weights, multiple: int = 8):
    """The matrices one under the other, with zero rows behind them up to a whole `multiple` of rows
    (rows of the float32 product then start on 32 bytes)."""
    rows = sum(w.shape[0] for w in weights)
    spare = -rows % multiple
    if spare:
        weights = list(weights) + [torch.zeros((spare, weights[0].shape[1]), dtype=weights[0].dtype)]
    return torch.cat(weights, dim=0)


class GatedDeltaNet:
    """The gated delta rule: per head a matrix state S (dim x vdim, float32) that every token
    decays, corrects along its key and reads along its query:
        S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q.
    From the mixer's input h: q = Wq h and k = Wk h (kv_heads x dim; value head i uses q/k head
    i // (heads / kv_heads)), v = Wv h (heads x vdim); each of the three passes a short causal
    convolution over time, channel by channel (`<tensor>.conv` [channels, taps], the last tap on the
    current token, zeros before a sequence's start), and silu; q and k become unit vectors per head
    (x / sqrt(sum x^2 + 1e-6)), q also times dim^(-1/2); beta = sigmoid(Wb h) and the decay
    g = exp(-exp(A_log) softplus(Wa h + dt_bias)), one a head; every head's o is divided by its root
    mean square over vdim, scaled by the gain `norm` (vdim lanes, shared by the heads) and by
    silu(Wg h); then Wo.  Everything behind the six input products (one stacked product, written
    in float32) is 32-bit (`csrc/delta_rule.cu`).

    Per request it keeps, in one state slot: the heads' matrices and the convolution's last
    taps - 1 inputs.  `input_stack` / `forward_projected`: a mixer that runs beside another one on
    the same input may have its input products computed in one product with the other's."""

    graph_safe = True    # launches depend on device-side metadata alone

    @staticmethod
    def tensors(spec):
        p, x = spec.params, spec.prefix
        hidden, heads, groups, dim, vdim, taps = (p["hidden_size"], p["heads"], p["kv_heads"], p["dim"], p["vdim"],
                                                  p["conv"])
        return [TensorSpec(x + ".q", (groups * dim, hidden)), TensorSpec(x + ".q.conv", (groups * dim, taps), "normal", 0.5),
                TensorSpec(x + ".k", (groups * dim, hidden)), TensorSpec(x + ".k.conv", (groups * dim, taps), "normal", 0.5),
                TensorSpec(x + ".v", (heads * vdim, hidden)), TensorSpec(x + ".v.conv", (heads * vdim, taps), "normal", 0.5),
                TensorSpec(x + ".b", (heads, hidden)), TensorSpec(x + ".A_log", (heads,), "normal", 0.5),
                TensorSpec(x + ".norm", (vdim,), "one_plus_normal"), TensorSpec(x + ".a", (heads, hidden)),
                TensorSpec(x + ".dt_bias", (heads,), "normal", 0.5), TensorSpec(x + ".g", (heads * vdim, hidden)),
                TensorSpec(x + ".o", (hidden, heads * vdim))]

    def __init__(self, spec, store, runtime):
        p, x = spec.params, spec.prefix
        self.runtime = runtime
        self.hidden = int(p["hidden_size"])
        self.heads, self.groups = int(p["heads"]), int(p["kv_heads"])
        self.dim, self.vdim, self.taps = int(p["dim"]), int(p["vdim"]), int(p["conv"])
        self.eps = float(p["eps"])
        if self.groups <= 0 or self.heads % self.groups:
            raise ConfigError(f"{self.heads} value heads do not divide into {self.groups} query/key heads")
        self.dim_padded = ops.gdn_padded_dim(self.dim)
        if not self.dim_padded or not 1 <= self.taps <= 16:
            raise ConfigError(f"the delta rule takes heads of up to 1024 lanes and convolutions of up to 16 taps; "
                              f"found {self.dim} and {self.taps}")
        self.channels = 2 * self.groups * self.dim + self.heads * self.vdim
        self._stack = [store.get(x + "." + n) for n in ("q", "k", "v", "b", "a", "g")]
        self.conv_w = runtime.vector(torch.cat([store.get(x + f".{n}.conv").to(torch.float32) for n in "qkv"], dim=0))
        self.a_log = runtime.vector(store.get(x + ".A_log"))
        self.dt_bias = runtime.vector(store.get(x + ".dt_bias"))
        self.gain = runtime.vector(store.get(x + ".norm"))
        self.out = Linear(runtime.matrix(store.get(x + ".o")))
        self.inputs = None                      # built at first use: a mixer beside this one may carry the product
        # a slot: [heads, vdim, dim_padded] and behind it [taps - 1, channels], in whole 4s of floats
        self.conv_off = self.heads * self.vdim * self.dim_padded
        self.state_floats = -(-(self.conv_off + (self.taps - 1) * self.channels) // 4) * 4

    def shape_key(self, q_lens):
        longest = max(q_lens)
        return "delta1" if longest == 1 else "delta" if longest < 32 else "delta32"      # the kernels' choices

    def input_stack(self):
        """(the six input matrices one under the other, as stored; their bias: none)."""
        return torch.cat(self._stack, dim=0), None

    def cache_need(self):
        return CacheNeed(state=StateNeed((self.state_floats,)))

    def streamed_weights(self):
        return [self.out.weight] if self.inputs is None else [self.inputs.weight, self.out.weight]

    def forward_projected(self, proj, at, ctx, cache, out_scale: float = 1.0):
        """From the stacked product `proj` (float32 or the compute type), this mixer's columns
        starting at `at`; the output is scaled by `out_scale` (in float32, before it is rounded for
        the output projection)."""
        n, c, h = ctx.n_tokens, self.channels, self.heads
        if ctx.max_q_len == 1 and _ONE_KERNEL_STEP and ops.gdn_step_supported(self.dim, self.vdim):
            # every request brings one token: one kernel a mixer instead of four (a decoding step is bound
            # by its launches)
            y = self.runtime.empty(n, h * self.vdim)
            ops.gdn_step(proj, at, at + c, at + c + h, at + c + 2 * h, self.groups, h, self.dim, self.vdim, self.taps,
                         self.conv_w, self.a_log, self.dt_bias, self.gain, out_scale, self.eps, cache.state,
                         self.conv_off, ctx.row_req, ctx.q_start, ctx.state_slot, y)
            return self.out.forward(y, partials_ok=True)
        qkv = torch.empty((n, c), dtype=torch.float32, device=proj.device)
        bg = torch.empty((n, 2 * h + self.groups), dtype=torch.float32, device=proj.device)
        ops.gdn_prepare(proj, at, at + c, at + c + h, self.groups, h, self.dim, self.vdim, self.taps, self.conv_w,
                        self.a_log, self.dt_bias, cache.state, self.conv_off, ctx.row_req, ctx.q_start,
                        ctx.state_slot, qkv, bg)
        o = torch.empty((n, h * self.vdim), dtype=torch.float32, device=proj.device)
        ops.gdn_scan(qkv, bg, self.groups, h, self.dim, self.vdim, cache.state, ctx.q_start, ctx.state_slot, o,
                     longest=ctx.max_q_len)
        y = self.runtime.empty(n, h * self.vdim)
        ops.gdn_out_norm(o, proj, at + c + 2 * h, self.gain, out_scale, self.eps, y, h, self.vdim, ctx.row_req)
        return self.out.forward(y, partials_ok=True)

    def forward(self, h, ctx, cache):
        if self.inputs is None:
            self.inputs = Linear(self.runtime.matrix(stacked_rows([self.input_stack()[0]])))
        return self.forward_projected(self.inputs.forward(h, out_dtype=torch.float32), 0, ctx, cache)


class Mamba2:
    """The selective state-space mixer with a scalar decay a head (Mamba-2).  With inner = heads * vdim,
    N = `state` lanes and G = `groups`: the input product W_in h is [z: inner | x: inner | B: G N | C: G N |
    dt: heads].  x, B and C together pass a short causal convolution over time, channel by channel
    (`.conv` [channels, taps], bias `.conv.b`, the last tap on the current token, zeros before a sequence's
    start), and silu.  dt = softplus(dt + `.dt_bias`).  Per head (head h reads the B and C of group
    h // (heads / G)) a matrix S (N x vdim) from zero:
        S <- exp(-exp(A_log) dt) S + dt B x^T;   y = S^T C + D x.
    y, heads side by side, times silu(z), is divided by its root mean square inside each of `norm_groups`
    equal parts of the row (`eps` inside the root), multiplied by `.norm` and goes through `.o`.

    The input product is written in float32; the convolution, dt, the decay, the recurrence, its state, the
    gate and the norm are 32-bit whatever the products' precision (`csrc/short_conv.cu`, `csrc/mamba2.cu`).
    Per request it keeps, in one state slot, the heads' matrices ([heads, vdim, N]) and behind them the
    convolution's last taps - 1 inputs."""

    graph_safe = True    # launches depend on device-side metadata alone

    @staticmethod
    def tensors(spec):
        p, x = spec.params, spec.prefix
        hidden, heads, vdim, n, groups, taps = p["hidden_size"], p["heads"], p["vdim"], p["state"], p["groups"], p["conv"]
        inner, channels = heads * vdim, heads * vdim + 2 * groups * n
        return [TensorSpec(x + ".in", (2 * inner + 2 * groups * n + heads, hidden)),
                TensorSpec(x + ".conv", (channels, taps), "normal", 0.5), TensorSpec(x + ".conv.b", (channels,), "normal", 0.1),
                TensorSpec(x + ".dt_bias", (heads,), "normal", 0.5), TensorSpec(x + ".A_log", (heads,), "normal", 0.5),
                TensorSpec(x + ".D", (heads,), "one_plus_normal", 0.2), TensorSpec(x + ".norm", (inner,), "one_plus_normal"),
                TensorSpec(x + ".o", (hidden, inner))]

    def __init__(self, spec, store, runtime):
        p, x = spec.params, spec.prefix
        self.runtime = runtime
        self.hidden = int(p["hidden_size"])
        self.heads, self.vdim, self.n, self.groups = int(p["heads"]), int(p["vdim"]), int(p["state"]), int(p["groups"])
        self.taps, self.norm_groups, self.eps = int(p["conv"]), int(p["norm_groups"]), float(p["eps"])
        self.inner = self.heads * self.vdim
        self.channels = self.inner + 2 * self.groups * self.n
        if self.groups <= 0 or self.heads % self.groups:
            raise ConfigError(f"{self.heads} heads do not divide into {self.groups} groups")
        if self.norm_groups <= 0 or self.inner % self.norm_groups:
            raise ConfigError(f"{self.inner} lanes do not divide into {self.norm_groups} parts for the norm")
        if not 1 <= self.n <= ops.MAMBA2_MAX_STATE or not 1 <= self.taps <= 16:
            raise ConfigError(f"the state-space recurrence takes states of up to {ops.MAMBA2_MAX_STATE} lanes and "
                              f"convolutions of up to 16 taps; found {self.n} and {self.taps}")
        self.inputs = Linear(runtime.matrix(stacked_rows([store.get(x + ".in")])))
        self.conv_w = runtime.vector(store.get(x + ".conv"))
        self.conv_b = runtime.vector(store.get(x + ".conv.b"))
        self.dt_bias = runtime.vector(store.get(x + ".dt_bias"))
        self.a_log = runtime.vector(store.get(x + ".A_log"))
        self.skip = runtime.vector(store.get(x + ".D"))
        self.gain = runtime.vector(store.get(x + ".norm"))
        self.out = Linear(runtime.matrix(store.get(x + ".o")))
        # a slot: [heads, vdim, N] and behind it [taps - 1, channels], in whole 4s of floats
        self.conv_off = self.heads * self.vdim * self.n
        self.state_floats = -(-(self.conv_off + (self.taps - 1) * self.channels) // 4) * 4

    def cache_need(self):
        return CacheNeed(state=StateNeed((self.state_floats,)))

    def shape_key(self, q_lens):
        return "ssm1" if max(q_lens) == 1 else "ssm"

    def streamed_weights(self):
        return [self.inputs.weight, self.out.weight]

    def forward(self, h, ctx, cache):
        n = ctx.n_tokens
        proj = self.inputs.forward(h, out_dtype=torch.float32)
        xbc = torch.empty((n, self.channels), dtype=torch.float32, device=proj.device)
        single = ctx.max_q_len == 1          # a step of single tokens: the kept inputs move on in the same launch
        ops.short_conv(proj, self.inner, self.channels, self.conv_w, self.conv_b, cache.state, self.conv_off, ctx.row_req,
                       ctx.q_start, ctx.state_slot, xbc, activation="silu", shift=single)
        if not single:
            ops.short_conv_state(proj, self.inner, self.channels, self.taps, cache.state, self.conv_off, ctx.q_start,
                                 ctx.state_slot)
        y = torch.empty((n, self.inner), dtype=torch.float32, device=proj.device)
        ops.mamba2_scan(xbc, proj, self.inner + self.channels, self.dt_bias, self.a_log, self.skip, self.heads,
                        self.groups, self.vdim, self.n, cache.state, ctx.q_start, ctx.state_slot, y)
        gated = self.runtime.empty(n, self.inner)
        ops.mamba2_out_norm(y, proj, 0, self.gain, self.eps, self.norm_groups, ctx.row_req, gated)
        return self.out.forward(gated, partials_ok=True)


register_part("mixer", "mamba2", Mamba2)
register_part("mixer", "min_gru", MinGRU)
register_part("mixer", "gated_delta_net", GatedDeltaNet)
