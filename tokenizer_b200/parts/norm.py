"""RMSNorm: y = x / sqrt(mean(x^2) + eps) * gain, statistics in float32
(reference: qwen-infer/src/model.rs:594-599, 616, 749); and the layer norm with gain and bias."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.store import TensorSpec
from .base import register_part


def tensor_name(spec) -> str:
    """Where a part with one tensor finds it: `params["tensor"]` where the file names it
    outright, else `<prefix>.weight`."""
    return spec.params.get("tensor") or spec.prefix + ".weight"


class RMSNorm:
    """`gain_scale` (optional): a constant folded into the gain in float32, for a model whose
    logits are the head's product times a constant (the final norm carries it), or whose sublayer
    outputs are normed and multiplied by a constant before they are added (the norm behind the
    sublayer carries it).  `one_plus` (optional): the tensor holds the gain's offset from one; the gain is
    1 + w, taken in float32.  As the norm on a sublayer's OUTPUT it offers `add_to`, like the layer
    norm: x += norm(sum of the output's scaled terms), and the next norm of the new x in the same
    kernel (`csrc/layer_norm.cu`, the RMS form)."""

    @staticmethod
    def tensors(spec):
        if spec.params.get("one_plus"):
            return [TensorSpec(tensor_name(spec), (spec.params["size"],), "normal", 0.1)]
        return [TensorSpec(tensor_name(spec), (spec.params["size"],), "one_plus_normal")]

    def __init__(self, spec, store, runtime):
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.runtime = runtime
        self.gain = runtime.vector(store.get(tensor_name(spec)))
        if spec.params.get("one_plus"):
            self.gain = (self.gain + 1.0).contiguous()
        if spec.params.get("gain_scale") is not None:
            self.gain = (self.gain * float(spec.params["gain_scale"])).contiguous()

    def folded(self):
        """(gain, eps) for a consumer that computes this norm inside its own kernel."""
        return self.gain, self.eps

    def add_to(self, x, terms, then=None):
        """x += this norm of the summed terms, in place; with `then` (the norm in front of the next
        sublayer), returns that norm of the new x: one kernel where `then` can be folded (an RMS norm
        with `folded`, or a layer norm with `affine`)."""
        if then is None:
            ops.post_norm_add(x, terms, self.gain, None, self.eps, rms=True)
            return None
        fold, affine = getattr(then, "folded", None), getattr(then, "affine", None)
        if fold is None and affine is None:
            ops.post_norm_add(x, terms, self.gain, None, self.eps, rms=True)
            return then.forward(x)
        out = self.runtime.empty(x.shape[0], self.size)
        if fold is not None:
            gain, eps = fold()
            ops.post_norm_add(x, terms, self.gain, None, self.eps, gain, None, eps, out, rms=True, next_rms=True)
        else:
            gain, bias, eps = affine()
            ops.post_norm_add(x, terms, self.gain, None, self.eps, gain, bias, eps, out, rms=True)
        return out

    def forward_gated(self, x, gated):
        """x += (y + bias) * sigmoid(pre + pre_bias), then the norm of the new x: one kernel."""
        out = self.runtime.empty(x.shape[0], self.size)
        ops.gated_add_rms_norm(x, gated.y, gated.bias, gated.pre, gated.pre_bias, self.gain, self.eps, out)
        return out

    def forward_scaled(self, x, scaled):
        """x += sum of vector * output over `scaled.terms`, then the norm of the new x: one kernel."""
        out = self.runtime.empty(x.shape[0], self.size)
        ops.scaled_add_norm(x, scaled.terms, self.gain, self.eps, out)
        return out

    def forward(self, x, delta=None, rows=None):
        n = x.shape[0] if rows is None else rows.shape[0]
        out = self.runtime.empty(n, self.size)
        ops.rms_norm(x, self.gain, self.eps, out, delta=delta, rows=rows)
        return out


class LayerNorm:
    """(x - mean) / sqrt(var + eps) * gain + bias, var the mean of the squared deviations; the
    bias is the tensor of the gain's name with `.b` added.  Statistics in float32, two passes.
    As the norm on a sublayer's OUTPUT it offers `add_to`: x += norm(sum of the output's scaled
    terms), and, where the next norm is of this kind too, that norm of the new x in the same
    kernel (`csrc/layer_norm.cu`)."""

    @staticmethod
    def tensors(spec):
        name = tensor_name(spec)
        return [TensorSpec(name, (spec.params["size"],), "one_plus_normal"),
                TensorSpec(name + ".b", (spec.params["size"],), "normal")]

    def __init__(self, spec, store, runtime):
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.runtime = runtime
        name = tensor_name(spec)
        self.gain = runtime.vector(store.get(name))
        self.bias = runtime.vector(store.get(name + ".b"))

    def affine(self):
        """(gain, bias, eps) for a kernel that computes this norm behind its own work."""
        return self.gain, self.bias, self.eps

    def add_to(self, x, terms, then=None):
        """x += this norm of the summed terms, in place; with `then` (the norm in front of the next
        sublayer), returns that norm of the new x."""
        following = getattr(then, "affine", None)
        if then is None or following is None:
            ops.post_norm_add(x, terms, self.gain, self.bias, self.eps)
            return None if then is None else then.forward(x)
        gain, bias, eps = following()
        out = self.runtime.empty(x.shape[0], self.size)
        ops.post_norm_add(x, terms, self.gain, self.bias, self.eps, gain, bias, eps, out)
        return out

    def forward(self, x, delta=None, rows=None):
        if delta is not None:
            ops.residual_add(x, delta)
        n = x.shape[0] if rows is None else rows.shape[0]
        out = self.runtime.empty(n, self.size)
        ops.layer_norm(x, self.gain, self.bias, self.eps, out, rows=rows)
        return out


register_part("norm", "rms_norm", RMSNorm)
register_part("norm", "layer_norm", LayerNorm)
