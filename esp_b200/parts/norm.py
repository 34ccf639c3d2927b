"""RMSNorm fused with the residual add that precedes it."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import ParamSpec, Part, register


class RmsNorm(Part):
    """h = (x + delta) * rsqrt(mean((x + delta)^2) + eps) * weight, in 32-bit
    (crates/esp/src/infer/decoder/layer.rs:27-33)."""

    graph_safe = True
    takes_deferred = True      # a deferred expert sum is added and normalised here in one launch

    def __init__(self, spec, rt):
        self.spec = spec
        self.rt = rt
        self.weight = None

    def param_specs(self):
        return [ParamSpec(self.spec.weight, (self.spec.width,), "norm_scale")]

    def allocate(self, stored, rt):
        self.weight = torch.empty(self.spec.width, dtype=torch.float32, device=rt.device)
        return {self.spec.weight: self.weight}

    def forward(self, x, delta, h, rows=None, write_x=True, h32=None, delta_scale=None):
        """``delta_scale`` (float32 [width]): delta is multiplied by it channel by channel as it is added."""
        if hasattr(delta, "fused_add_rmsnorm") and delta_scale is not None:
            delta = delta.materialize()
        if hasattr(delta, "fused_add_rmsnorm"):
            # the producer left its last step (an ordered sum) to be done here, in the same launch
            delta.fused_add_rmsnorm(x, self.weight, h, self.spec.eps, rows, write_x, h32)
            return h
        ops.add_rmsnorm(x, delta, self.weight, h, self.spec.eps, rows=rows, write_x=write_x, h32=h32,
                        yscale=delta_scale if delta is not None else None)
        return h


class ScalarRmsNorm(RmsNorm):
    """RMS norm whose weight is one number for all channels (a tensor without dimensions in the checkpoint).  The
    number is spread over a vector once the weights are in, so the kernels of the vector form run it."""

    def param_specs(self):
        return [ParamSpec(self.spec.weight, (), "norm_scale")]

    def allocate(self, stored, rt):
        self.weight = torch.empty(self.spec.width, dtype=torch.float32, device=rt.device)
        return {self.spec.weight: self.weight[0]}        # the loader fills the first entry; finalize copies it to all

    def finalize(self):
        if self.weight is not None:
            self.weight.copy_(self.weight[0].clone().expand(self.spec.width))


class OffsetRmsNorm(RmsNorm):
    """RMS norm whose tensor holds the scale minus one: h = x * rsqrt(mean(x^2) + eps) * (1 + w).  The one is added once
    the weights are in (in 32-bit), so the kernels of the plain form run it."""

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self._offset_done = False

    def param_specs(self):
        return [ParamSpec(self.spec.weight, (self.spec.width,), "norm_offset", init=(0.0, 0.1))]

    def finalize(self):
        if self.weight is not None and not self._offset_done:
            self._offset_done = True
            self.weight.add_(1.0)


class DeferredPostNorm:
    """A sublayer's result on its way into the residual stream through a norm of its own: x += norm(y).  The norm that
    reads x next does that add and its own normalisation in one launch (``fused_add_rmsnorm``); anything else gets the
    normed rows from ``materialize()``."""

    def __init__(self, rt, y, norm):
        self.rt, self.y, self.norm = rt, y, norm

    def materialize(self):
        out = self.rt.ws.get("post_normed", tuple(self.y.shape), torch.float32)
        ops.norm_add_rmsnorm(None, self.y, self.norm.weight, self.norm.spec.eps, None, None, 0.0, h32=out)
        return out

    def fused_add_rmsnorm(self, x, gamma, h, eps, rows, write_x, h32):
        ops.norm_add_rmsnorm(x, self.y, self.norm.weight, self.norm.spec.eps, gamma, h, eps, rows=rows, write_x=write_x,
                             h32=h32)

    def add_to(self, x):
        """x += norm(y), nothing else."""
        ops.norm_add_rmsnorm(x, self.y, self.norm.weight, self.norm.spec.eps, None, None, 0.0)


register("norm", "rmsnorm", RmsNorm)
register("norm", "rmsnorm_scalar", ScalarRmsNorm)
register("norm", "rmsnorm_offset", OffsetRmsNorm)
