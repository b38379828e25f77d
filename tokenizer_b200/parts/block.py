"""Arrangement of a layer's parts.  Pre-norm residual: x += mixer(norm(x));
x += feed_forward(norm(x)) (reference: qwen-infer/src/model.rs:603-623).  The
adds are left pending on the stream so the next norm performs them."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.store import TensorSpec
from .base import GatedDelta, register_part
from .linear import Linear


class PreNormResidual:
    # the parts this arrangement wants, by name, and the category each is built from; the
    # model builds them from the layer's spec and hands them over as keyword arguments
    PARTS = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm",
             "feed_forward_norm": "norm"}

    def __init__(self, mixer, feed_forward, mixer_norm, feed_forward_norm):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm

    def streamed_weights(self):
        """The matrices a step with few rows reads once, in the order it reads them."""
        out = []
        for part in (self.mixer, self.feed_forward):
            out += list(getattr(part, "streamed_weights", lambda: [])())
        return out

    def layer_start_operands(self):
        """What this layer's kernels read first (the mixer's first weight, the first norm's
        gain, the mixer's bias), for the layer before to bring into L2; None when the parts
        have no such operands."""
        start = getattr(self.mixer, "start_operands", None)
        fold = getattr(self.mixer_norm, "folded", None)
        if start is None or fold is None:
            return None
        weight, bias = start()
        return weight, fold()[0], bias

    def forward(self, stream, ctx, cache):
        # a mixer may take the whole layer (both norms, itself, the feed-forward) into one kernel
        whole = getattr(self.mixer, "fused_layer", None)
        if whole is not None and whole(stream, self.mixer_norm, ctx, cache, self.feed_forward,
                                       self.feed_forward_norm):
            return
        # a mixer may take the stream as it is and fold the norm into its own kernel
        fused = getattr(self.mixer, "fused_step", None)
        delta = fused(stream, self.mixer_norm, ctx, cache) if fused is not None else None
        if delta is None:
            delta = self.mixer.forward(stream.normed(self.mixer_norm), ctx, cache)
        stream.add(delta)
        # a feed-forward may take the stream as it is and fold the norm into its own kernel
        fused = getattr(self.feed_forward, "fused_step", None)
        if fused is None or not fused(stream, self.feed_forward_norm):
            stream.add(self.feed_forward.forward(stream.normed(self.feed_forward_norm)))


register_part("block", "pre_norm_residual", PreNormResidual)


class ResidualGate:
    """A gate on a sublayer's output: sigmoid(W h + b) of the sublayer's own input h, element by
    element.  Tensors `<prefix>` (the matrix) and `<prefix>.b`.  A sublayer that can carry the
    product in its own first product takes it over (`take_side`); else `forward` computes it."""

    @staticmethod
    def tensors(spec):
        n = spec.params["hidden_size"]
        return [TensorSpec(spec.prefix, (n, n)), TensorSpec(spec.prefix + ".b", (n,))]

    def __init__(self, spec, store, runtime):
        self.stored = (store.get(spec.prefix), store.get(spec.prefix + ".b"))
        self.runtime = runtime
        self.proj = None

    def forward(self, h):
        """The gate's pre-activation, float32 [T, hidden]."""
        if self.proj is None:
            self.proj = Linear(self.runtime.matrix(self.stored[0]), self.runtime.vector(self.stored[1]))
        return self.proj.forward(h, out_dtype=torch.float32)


class GatedPreNormResidual:
    """x += mixer(norm1(x)) * gate1(norm1(x)); x += feed_forward(norm2(x)) * gate2(norm2(x)).  The
    gates' products ride in the sublayers' first products where those offer it; the gated outputs
    stay pending on the stream with their gates unapplied, so that the next norm applies the gate,
    adds and norms in one kernel."""

    PARTS = {"mixer": "mixer", "mixer_norm": "norm", "mixer_gate": "gate",
             "feed_forward": "feed_forward", "feed_forward_norm": "norm", "feed_forward_gate": "gate"}

    def __init__(self, mixer, mixer_norm, mixer_gate, feed_forward=None, feed_forward_norm=None,
                 feed_forward_gate=None):
        self.mixer, self.mixer_norm, self.mixer_gate = mixer, mixer_norm, mixer_gate
        self.feed_forward, self.feed_forward_norm = feed_forward, feed_forward_norm
        self.feed_forward_gate = feed_forward_gate
        self._carried = {}
        for part, gate in ((mixer, mixer_gate), (feed_forward, feed_forward_gate)):
            take = getattr(part, "take_side", None)
            if part is not None and take is not None:
                take(*gate.stored)
                self._carried[id(part)] = True

    def streamed_weights(self):
        out = []
        for part in (self.mixer, self.feed_forward):
            out += list(getattr(part, "streamed_weights", lambda: [])())
        return out

    def _gated(self, stream, part, gate, h, y):
        carried = id(part) in self._carried
        pre = part.side_pre if carried else gate.forward(h)
        stream.add_gated(GatedDelta(y, getattr(part, "deferred_bias", None), pre,
                                    part.side_bias if carried else None))

    def forward(self, stream, ctx, cache):
        h = stream.normed(self.mixer_norm)
        self._gated(stream, self.mixer, self.mixer_gate, h, self.mixer.forward(h, ctx, cache))
        if self.feed_forward is not None:
            h = stream.normed(self.feed_forward_norm)
            self._gated(stream, self.feed_forward, self.feed_forward_gate, h, self.feed_forward.forward(h))


class GatedPreNormMixerOnly(GatedPreNormResidual):
    """The same arrangement for a layer without a feed-forward."""

    PARTS = {"mixer": "mixer", "mixer_norm": "norm", "mixer_gate": "gate"}


register_part("block", "gated_pre_norm_residual", GatedPreNormResidual)
register_part("block", "gated_pre_norm_mixer_only", GatedPreNormMixerOnly)
register_part("gate", "residual_gate", ResidualGate)


class SandwichNormResidual:
    """A norm in front of AND behind every sublayer: x += post1(mixer(norm1(x)));
    x += post2(feed_forward(norm2(x))).  A sublayer's output stays pending on the stream together
    with the norm that follows it, so that this norm, the add and the norm in front of the next
    sublayer (of this layer or of the next) are one kernel.  A mixer may hand back a sum of scaled
    terms (`ScaledTerms`); the norm behind it sums them."""

    PARTS = {"mixer": "mixer", "mixer_norm": "norm", "mixer_post_norm": "norm",
             "feed_forward": "feed_forward", "feed_forward_norm": "norm", "feed_forward_post_norm": "norm"}

    def __init__(self, mixer, mixer_norm, mixer_post_norm, feed_forward=None, feed_forward_norm=None,
                 feed_forward_post_norm=None):
        self.mixer, self.mixer_norm, self.mixer_post_norm = mixer, mixer_norm, mixer_post_norm
        self.feed_forward, self.feed_forward_norm = feed_forward, feed_forward_norm
        self.feed_forward_post_norm = feed_forward_post_norm

    def streamed_weights(self):
        out = []
        for part in (self.mixer, self.feed_forward):
            out += list(getattr(part, "streamed_weights", lambda: [])())
        return out

    def forward(self, stream, ctx, cache):
        stream.add_normed(self.mixer.forward(stream.normed(self.mixer_norm), ctx, cache), self.mixer_post_norm)
        if self.feed_forward is not None:
            stream.add_normed(self.feed_forward.forward(stream.normed(self.feed_forward_norm)),
                              self.feed_forward_post_norm)


class SandwichNormMixerOnly(SandwichNormResidual):
    """The same arrangement for a layer without a feed-forward."""

    PARTS = {"mixer": "mixer", "mixer_norm": "norm", "mixer_post_norm": "norm"}


class PassEntry:
    """What a pass of a looped stack of layers adds to the stream right before its first layer:
    the embedding's output (`add_embedding`: every pass but the first) and row `index` of a
    tensor [passes, hidden] (`tensor`)."""

    @staticmethod
    def tensors(spec):
        return [TensorSpec(spec.params["tensor"], (spec.params["passes"], spec.params["hidden_size"]))]

    def __init__(self, spec, store, runtime):
        p = spec.params
        if not 0 <= int(p["index"]) < int(p["passes"]):
            raise ValueError(f"pass {p['index']} of {p['passes']}")
        self.needs_embedding = bool(p.get("add_embedding"))
        self.vector = runtime.vector(store.get(p["tensor"])[int(p["index"])])

    def forward(self, stream, embedded):
        ops.stream_inject(stream.flush(), embedded if self.needs_embedding else None, self.vector)


register_part("block", "sandwich_norm_residual", SandwichNormResidual)
register_part("block", "sandwich_norm_mixer_only", SandwichNormMixerOnly)
register_part("injection", "pass_entry", PassEntry)


class LayerScale:
    """A learned vector over the width that multiplies a sublayer's output, element by element, before it
    is added to the stream.  One tensor [hidden], named outright (`tensor`)."""

    @staticmethod
    def tensors(spec):
        return [TensorSpec(spec.params["tensor"], (spec.params["hidden_size"],), "one_plus_normal")]

    def __init__(self, spec, store, runtime):
        self.vector = runtime.vector(store.get(spec.params["tensor"]))


class CausalConvResidual:
    """What a sublayer reads instead of the normed stream h: h + conv(h), a causal convolution over time
    on each channel, conv(h)_t = sum_j w[:, j] h_(t - taps + 1 + j) with zeros before a sequence's start
    (tensor `tensor` [hidden, taps], no bias).  The last taps - 1 inputs of every request are kept between
    steps (`state_need`), so a prompt cut anywhere gives what the whole prompt gives."""

    @staticmethod
    def tensors(spec):
        return [TensorSpec(spec.params["tensor"], (spec.params["hidden_size"], spec.params["taps"]), "normal", 0.3)]

    def __init__(self, spec, store, runtime):
        self.runtime = runtime
        self.hidden, self.taps = int(spec.params["hidden_size"]), int(spec.params["taps"])
        if not 1 <= self.taps <= 16:
            raise ValueError(f"a short convolution has 1 to 16 taps, found {self.taps}")
        self.weight = runtime.vector(store.get(spec.params["tensor"]))

    def state_need(self):
        from .base import StateNeed
        return StateNeed(((self.taps - 1) * self.hidden,)) if self.taps > 1 else None

    def shape_key(self, q_lens):
        return "conv1" if max(q_lens) == 1 else "conv"

    def forward(self, h, ctx, state):
        out = self.runtime.empty(h.shape[0], self.hidden)
        single = ctx.max_q_len == 1          # a step of single tokens: the kept inputs move on in the same launch
        ops.short_conv(h, 0, self.hidden, self.weight, None, state, 0, ctx.row_req, ctx.q_start, ctx.state_slot, out,
                       residual=True, shift=single)
        if not single:
            ops.short_conv_state(h, 0, self.hidden, self.taps, state, 0, ctx.q_start, ctx.state_slot)
        return out


class ParallelResidual:
    """Both sublayers on ONE norm: with h = norm(x), x += s1 * mixer(filter(h)) + s2 * feed_forward(h), s1
    and s2 learned vectors over the width (`LayerScale`), `filter` what stands between the norm and the
    mixer (`CausalConvResidual`; the feed-forward reads h as it is).  The two outputs stay pending on the
    stream with their vectors, so that the next norm scales, adds and norms in one kernel.  The filter's
    kept inputs are this arrangement's own state beside the mixer's (`CacheNeed.side_state`)."""

    PARTS = {"mixer": "mixer", "mixer_norm": "norm", "mixer_filter": "filter", "mixer_scale": "scale",
             "feed_forward": "feed_forward", "feed_forward_scale": "scale"}

    def __init__(self, mixer, mixer_norm, mixer_filter, mixer_scale, feed_forward=None, feed_forward_scale=None):
        self.mixer, self.mixer_norm, self.mixer_filter, self.mixer_scale = mixer, mixer_norm, mixer_filter, mixer_scale
        self.feed_forward, self.feed_forward_scale = feed_forward, feed_forward_scale

    def cache_need(self):
        from .base import CacheNeed
        need = self.mixer.cache_need()
        return CacheNeed(kv=need.kv, state=need.state, side_state=self.mixer_filter.state_need())

    def streamed_weights(self):
        out = []
        for part in (self.mixer, self.feed_forward):
            out += list(getattr(part, "streamed_weights", lambda: [])())
        return out

    def forward(self, stream, ctx, cache):
        from .base import VectorScaledTerms
        h = stream.normed(self.mixer_norm)
        terms = [(self.mixer.forward(self.mixer_filter.forward(h, ctx, cache.side_state), ctx, cache),
                  self.mixer_scale.vector)]
        if self.feed_forward is not None:
            terms.append((self.feed_forward.forward(h), self.feed_forward_scale.vector))
        stream.add_scaled(VectorScaledTerms(terms))


class ParallelResidualMixerOnly(ParallelResidual):
    """The same arrangement for a layer without a feed-forward."""

    PARTS = {"mixer": "mixer", "mixer_norm": "norm", "mixer_filter": "filter", "mixer_scale": "scale"}


register_part("scale", "layer_scale", LayerScale)
register_part("filter", "causal_conv_residual", CausalConvResidual)
register_part("block", "parallel_residual", ParallelResidual)
register_part("block", "parallel_residual_mixer_only", ParallelResidualMixerOnly)
