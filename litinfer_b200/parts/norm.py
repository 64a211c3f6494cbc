"""RMSNorm: y_j = w_j * x_j / sqrt(mean(x^2) + eps), per token
(src/ops/rms_norm/op.cpp:13-24).  Sum, reciprocal root and products in
float32 on the float32 residual stream; one rounding of y to the run dtype.
``gain`` (a parameter of the spec, default 1) is a constant factor on the result, multiplied into the
weight once when it is bound: a block that adds ``gain * norm(y)`` to the stream.  ``offset`` (default 0) is added to
the stored weight when it is bound: a weight that is stored around zero and applied as ``offset + w``.  Kind ``identity``
is no norm at all: the stream as it is, in the run dtype, for a sublayer that reads the stream itself.  Kind
``channel_scale`` is no norm either: a learned factor per channel (stored as it is applied), for an arrangement that
multiplies a sublayer's output by one before it joins the stream."""

from __future__ import annotations

import os
from typing import Dict, List

import torch

from .. import kernels as K
from ..weights.loader import ParamSpec
from .base import NORMS, Deferred, Norm

DEFER_UP_TO = int(os.environ.get("LITINFER_B200_DEFER_UP_TO", "32"))


def defers(tokens: int) -> bool:
    """Whether the norm between two products rides on them for a step of this many tokens.  Measured (1.5B shape, a
    context of 2,048): it saves two kernels a layer and 4-9 % of the step up to 32 tokens (24 tokens 2.12 -> 2.03 ms, 32
    tokens 2.12 -> 2.04 ms); at 64 tokens the epilogues of the weight-streaming products carry too much (2.54 -> 2.78
    ms).  (Tried in the tensor-memory GEMM of prefill too: there the residual stream read and written by the epilogue's
    threads, a row each, cost more than the norm kernels it replaced.)"""
    return 0 < tokens <= DEFER_UP_TO


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    def __init__(self, spec, prefix, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.tensor = self.prefix + str(spec.get("tensor", "weight"))      # the weight's name below the prefix
        self.gain = float(spec.get("gain", 1.0))
        self.offset = float(spec.get("offset", 0.0))
        self.weight = None

    def params(self) -> List[ParamSpec]:
        # (a weight that is applied as offset + w is stored around 1 - offset)
        if self.offset:
            return [ParamSpec(self.tensor, (self.size,), role="vector", mean=1.0 - self.offset, std=0.1)]
        return [ParamSpec(self.tensor, (self.size,), role="vector", init="ones_normal")]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors.pop(self.tensor)
        if self.offset:
            self.weight = (self.weight + self.offset).contiguous()
        if self.gain != 1.0:
            self.weight = (self.weight * self.gain).contiguous()

    def fused_decode(self):
        return {"weight": self.weight, "eps": self.eps, "size": self.size} if type(self) is RMSNorm and self.weight is not None else None

    def statistics(self):
        """(weight, centered, eps) as :func:`litinfer_b200.kernels.norm_add_norm` takes a norm: not centered."""
        return (self.weight, False, self.eps)

    def forward(self, x32):
        out = torch.empty(x32.shape, dtype=self.dtype, device=x32.device)
        K.rmsnorm(x32, self.weight, self.eps, out)
        return out

    def add_forward(self, x32, delta):
        out = torch.empty(x32.shape, dtype=self.dtype, device=x32.device)
        K.add_rmsnorm(x32, delta, self.weight, self.eps, out)
        return out

    def after_linear(self, linear, a, x32, defer=False):
        # bfloat16 and a consumer that applies the reciprocal root itself: the product adds to the stream and leaves
        # weight * x with the sums of squares, all in its epilogue; this norm has no kernel of its own.
        if defer and self.dtype == torch.bfloat16 and not isinstance(a, Deferred) and defers(a.shape[0]):
            h = torch.empty(x32.shape, dtype=self.dtype, device=x32.device)
            parts = K.linear_add_scaled_parts(a, linear.weight, x32, h)
            if parts:
                ssq = torch.empty((x32.shape[0], parts), dtype=torch.float32, device=x32.device)
                K.linear_add_scaled(a, linear.weight, linear.bias, x32, self.weight, h, ssq)
                return Deferred(h, ssq, self.size, self.eps)
        return self.add_forward(x32, linear(a))

    def streams_forward(self, xs, read, rows=None):
        out = torch.empty((xs.shape[0] if rows is None else rows.shape[0], xs.shape[2]), dtype=self.dtype, device=xs.device)
        K.hc_read_norm(xs, read, rows, self.weight, self.eps, out)
        return out

    def streams_update_forward(self, xs, y, mix, write, read):
        out = torch.empty((xs.shape[0], xs.shape[2]), dtype=self.dtype, device=xs.device)
        K.hc_update(xs, y, mix, write, read, self.weight, self.eps, out)
        return out

    def gather_forward(self, x32, rows):
        out = torch.empty((rows.shape[0], x32.shape[1]), dtype=self.dtype, device=x32.device)
        K.gather_rmsnorm(x32, rows, self.weight, self.eps, out)
        return out


@NORMS.register("layernorm")
class LayerNorm(Norm):
    """Layer norm with a weight and no bias: ``y = (x - mean(x)) / sqrt(var(x) + eps) * w`` with the variance the mean of
    the squared deviations; mean, variance and products in float32, one rounding to the run dtype.  Every form is the one
    kernel that also serves an arrangement with norms on both sides of a sublayer (``kernels.norm_add_norm``)."""

    def __init__(self, spec, prefix, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.tensor = self.prefix + str(spec.get("tensor", "weight"))
        self.weight = None

    def params(self) -> List[ParamSpec]:
        return [ParamSpec(self.tensor, (self.size,), role="vector", init="ones_normal")]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors.pop(self.tensor)

    def statistics(self):
        return (self.weight, True, self.eps)

    def forward(self, x32):
        out = torch.empty(x32.shape, dtype=self.dtype, device=x32.device)
        K.norm_add_norm(x32, None, None, self.statistics(), out)
        return out

    def add_forward(self, x32, delta):
        out = torch.empty(x32.shape, dtype=self.dtype, device=x32.device)
        K.norm_add_norm(x32, delta, None, self.statistics(), out)
        return out

    def gather_forward(self, x32, rows):
        out = torch.empty((rows.shape[0], x32.shape[1]), dtype=self.dtype, device=x32.device)
        K.norm_add_norm(x32, None, None, self.statistics(), out, rows=rows)
        return out


@NORMS.register("identity")
class NoNorm(Norm):
    """No norm: the residual stream as it is, rounded once to the run dtype.  It stands where an arrangement expects the
    norm before a sublayer and the design has the sublayer read the stream itself; it has no tensor.  ``statistics()``
    says so with a weight of None, which :func:`litinfer_b200.kernels.norm_add_norm` takes as "the row as it is"."""

    def __init__(self, spec, prefix, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        self.size = int(spec["size"])

    def statistics(self):
        return (None, False, 0.0)

    def forward(self, x32):
        out = torch.empty(x32.shape, dtype=self.dtype, device=x32.device)
        K.norm_add_norm(x32, None, None, self.statistics(), out)
        return out

    def add_forward(self, x32, delta):
        out = torch.empty(x32.shape, dtype=self.dtype, device=x32.device)
        K.norm_add_norm(x32, delta, None, self.statistics(), out)
        return out

    def gather_forward(self, x32, rows):
        out = torch.empty((rows.shape[0], x32.shape[1]), dtype=self.dtype, device=x32.device)
        K.norm_add_norm(x32, None, None, self.statistics(), out, rows=rows)
        return out


@NORMS.register("channel_scale")
class ChannelScale(Norm):
    """A learned factor per channel and nothing else: ``y = x * w``.  It stands where an arrangement expects the norm behind
    a sublayer (``sandwich``: ``x += post(sublayer(pre(x)))``) and the design multiplies the sublayer's output by a vector
    before it joins the stream.  ``statistics()`` says so with the mode :data:`litinfer_b200.kernels.SCALE_ONLY`, which the
    pass over the stream takes as "the row times the weight"."""

    def __init__(self, spec, prefix, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        self.size = int(spec["size"])
        self.tensor = self.prefix + str(spec.get("tensor", "weight"))
        self.weight = None

    def params(self) -> List[ParamSpec]:
        return [ParamSpec(self.tensor, (self.size,), role="vector", mean=float(self.spec.get("mean", 1.0)), std=float(self.spec.get("std", 0.1)))]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors.pop(self.tensor)

    def statistics(self):
        return (self.weight, K.SCALE_ONLY, 0.0)

    def forward(self, x32):
        out = torch.empty(x32.shape, dtype=self.dtype, device=x32.device)
        K.norm_add_norm(x32, None, None, self.statistics(), out)
        return out

    def add_forward(self, x32, delta):
        out = torch.empty(x32.shape, dtype=self.dtype, device=x32.device)
        K.norm_add_norm(x32, delta, None, self.statistics(), out)
        return out

    def gather_forward(self, x32, rows):
        out = torch.empty((rows.shape[0], x32.shape[1]), dtype=self.dtype, device=x32.device)
        K.norm_add_norm(x32, None, None, self.statistics(), out, rows=rows)
        return out
