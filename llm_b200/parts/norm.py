"""Norms: RMSNorm, and the element-wise tanh norm."""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import ParamSpec
from .base import Norm, register_norm, to_float32


class RmsNorm(Norm):
    """x / sqrt(mean(x^2) + eps) * weight, the norm of MythEclipse/llm
    (apps/engine/src/ops.rs:4-12). The weight is held in 32-bit. A spec with `unit_offset`
    stores its weight around zero: the gain is then 1 + weight (added in 32-bit at bind)."""
    graph_safe = True
    libraries = ("elementwise",)
    #: y = x / sqrt(mean(x^2) + eps) * gain: a part behind this norm may fold it (Part.fold_input_norm)
    foldable = True

    def __init__(self, spec):
        self.spec = spec
        self.gain = None

    def parameters(self):
        role = "gain_offset" if getattr(self.spec, "unit_offset", False) else "gain"
        return {self.spec.weight: ParamSpec((self.spec.size,), role)}

    def bind(self, tensors, dtype, device):
        self.gain = to_float32(tensors[self.spec.weight], device)
        if getattr(self.spec, "unit_offset", False):
            self.gain = (self.gain + 1.0).contiguous()

    def replay_key(self, step):
        return ()

    def forward(self, x, out_dtype, rows=None, out=None):
        return ops.rmsnorm(x, self.gain, self.spec.eps, out_dtype, rows, out=out)


register_norm("rmsnorm", RmsNorm)


class TanhNorm(Norm):
    """y = tanh(alpha x) * weight + bias with one learned number alpha (Zhu et al., "Transformers
    without Normalization"): no mean and no variance of the row enters, so nothing of it can be
    folded into a product behind it. alpha, weight and bias are held in 32-bit."""
    graph_safe = True
    libraries = ("elementwise",)
    foldable = False

    def __init__(self, spec):
        self.spec = spec
        self.alpha = 0.0
        self.gain = self.bias = None

    def parameters(self):
        s = self.spec
        return {s.weight: ParamSpec((s.size,), "gain"), s.bias: ParamSpec((s.size,), "bias"),
                s.alpha: ParamSpec((), "gate_scalar")}

    def bind(self, tensors, dtype, device):
        self.gain = to_float32(tensors[self.spec.weight], device)
        self.bias = to_float32(tensors[self.spec.bias], device)
        self.alpha = float(tensors[self.spec.alpha].to(torch.float32).reshape(()).cpu())

    def weights(self):
        return [self.gain, self.bias]

    def replay_key(self, step):
        return ()

    def forward(self, x, out_dtype, rows=None, out=None):
        return ops.tanh_norm(x, self.alpha, self.gain, self.bias, out_dtype, rows, out=out)

    def forward_with(self, other, x, out_dtype, out=None, out_other=None):
        """This norm and `other` (a TanhNorm too) of the same x in one launch: x is read once."""
        if out_other is None:
            out_other = torch.empty(tuple(x.shape), dtype=out_dtype, device=x.device)
        first = ops.tanh_norm(x, self.alpha, self.gain, self.bias, out_dtype, out=out,
                              second=(other.alpha, other.gain, other.bias, out_other))
        return first, out_other


register_norm("tanh_norm", TanhNorm)
