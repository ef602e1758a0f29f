"""Norms with the residual add fused in front of them: RMS norm, and layer norm with weight and bias.

``v = x + pending branch`` (written back to the 32-bit residual), ``y = (rsqrt(mean(v^2) + eps) * v) * w`` with the
sum of squares, the scale and both products in 32-bit - the reference's ``nbq_add_rms_q8`` (``kindi/nbq.cu:412-432``)
and, for the final norm on the rows whose logits are wanted, ``nbq_add_rms`` (``kindi/nbq.cu:435-453``). The weight
multiplies as stored (no ``1 + w``) unless the part's ``one_plus`` is set: the stored weight then lies around zero and
the gain is ``1 + w``, made once in 32-bit when the part is built. ``eps`` is a parameter of the part.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..config.registry import register_part
from ..config.spec import PartSpec
from ..kernels import lib as K
from .base import Branch, Norm, StepContext, WeightView


class RMSNorm(Norm):
    """``eps``, the gain's suffix (``weight``, default "weight") and ``one_plus`` (the gain is 1 + the stored weight)
    are parameters of the part"""

    @classmethod
    def tensor_shapes(cls, spec: PartSpec, width: int) -> Dict[str, Tuple[int, ...]]:
        return {spec.get("weight", "weight"): (width,)}

    @classmethod
    def tensor_init(cls, spec: PartSpec, width: int) -> Dict[str, str]:
        # (a weight stored around zero is drawn like any other tensor)
        return {} if spec.get("one_plus") else {spec.get("weight", "weight"): "gain"}

    def __init__(self, spec, width, weights: WeightView, *, dtype, device):
        super().__init__(spec, width, weights, dtype=dtype, device=device)
        self.eps = float(spec["eps"])
        self.weight = weights(spec.get("weight", "weight"))
        if spec.get("one_plus"):
            self.weight = (1.0 + self.weight.to(torch.float32)).contiguous()

    def add_norm(self, ctx: StepContext, x, pending: Optional[Branch], rows=None):
        n_out = x.shape[0] if rows is None else rows.numel()
        y = torch.empty((n_out, self.width), dtype=self.dtype, device=x.device)
        scale = None if pending is None else pending.scale
        if scale is not None and scale.dtype != self.weight.dtype:
            scale = scale.to(self.weight.dtype)
        K.add_rmsnorm(x, None if pending is None else pending.parts, self.weight, self.eps, y, rows,
                      write_back=rows is None and pending is not None, status=ctx.status, branch_scale=scale)
        return y

    def bytes_read(self) -> int:
        return self.weight.numel() * self.weight.element_size()


class LayerNorm(Norm):
    """``v = x + pending branch`` (written back), ``y = (v - mean(v)) / sqrt(var(v) + eps) * w + b`` with the variance
    the mean of the squared deviations, all in 32-bit. ``eps`` and the tensors' suffixes (``weight``, ``bias``) are
    parameters of the part."""

    @classmethod
    def _names(cls, spec: PartSpec):
        return spec.get("weight", "weight"), spec.get("bias", "bias")

    @classmethod
    def tensor_shapes(cls, spec: PartSpec, width: int) -> Dict[str, Tuple[int, ...]]:
        w, b = cls._names(spec)
        return {w: (width,), b: (width,)}

    @classmethod
    def tensor_init(cls, spec: PartSpec, width: int) -> Dict[str, str]:
        w, b = cls._names(spec)
        return {w: "gain", b: "zero"}

    def __init__(self, spec, width, weights: WeightView, *, dtype, device):
        super().__init__(spec, width, weights, dtype=dtype, device=device)
        self.eps = float(spec["eps"])
        w, b = self._names(spec)
        self.weight, self.bias = weights(w), weights(b)
        if self.weight.dtype != self.bias.dtype:
            raise ValueError("weight and bias of the norm %s are stored in different dtypes" % weights.prefix)

    def add_norm(self, ctx: StepContext, x, pending: Optional[Branch], rows=None):
        n_out = x.shape[0] if rows is None else rows.numel()
        if pending is not None and pending.scale is not None:
            raise NotImplementedError("the layer norm kernel adds a branch as it is; a scaled branch needs the RMS norm")
        y = torch.empty((n_out, self.width), dtype=self.dtype, device=x.device)
        K.add_layernorm(x, None if pending is None else pending.parts, self.weight, self.bias, self.eps, y, rows,
                        write_back=rows is None and pending is not None, status=ctx.status)
        return y

    def bytes_read(self) -> int:
        return 2 * self.weight.numel() * self.weight.element_size()


register_part("norm", "rmsnorm", RMSNorm)
register_part("norm", "layernorm", LayerNorm)
