"""The selective scan: a mixer whose per-sequence state is a diagonal recurrence per channel and state entry, with step
size, input and read-out vectors made from the token.  The state is float32 and belongs to the sequence: it sits in the
cache's per-slot state rows (the recurrence's entries, then the convolution's last inputs), is zeroed when the slot is
opened, and every step continues from what the step before left there, whatever run of tokens it brings.  Everything
between the projections and the output product is 32-bit."""
from __future__ import annotations

import torch

from ..cache import StateSpec
from ..csrc import ops
from ..errors import Unsupported
from .base import ParamSpec, Part, register
from .linear import SKINNY_ROWS, linear


class SelectiveScan(Part):
    """See ``SelectiveScanSpec``.  One product makes [x | z]; a kernel runs the causal convolution with bias and SiLU
    over x (the last taps - 1 inputs of a sequence are state); a product of the rounded x makes [dt_low | B | C] in
    32-bit; the step size's projection of dt_low runs as a true 32-bit product with its bias; the recurrence walks
    the tokens and multiplies its result by silu(z); then W_o.  Per slot the state holds S as [inner, state] floats
    and then the convolution's inputs [taps - 1, inner]."""

    graph_safe = True

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        s = spec
        if s.state > ops.SELECTIVE_MAX_STATE:
            raise Unsupported(s.kind + ".state", f"{s.state}; the recurrence kernel takes up to {ops.SELECTIVE_MAX_STATE} entries a channel")
        if s.taps > ops.CONV_MAX_TAPS or s.taps < 1:
            raise Unsupported(s.kind + ".conv", f"{s.taps} taps; the convolution kernel takes 1 to {ops.CONV_MAX_TAPS}")
        self.state_words = s.inner * s.state
        self.low_width = s.dt_rank + 2 * s.state
        self.w_in = self.w_x = self.w_dt = self.w_o = self.conv_w = self.conv_b = self.dt_b = self.a_log = self.skip = None

    def _n(self, which):
        return self.spec.prefix + getattr(self.spec.names, which)

    def param_specs(self):
        s = self.spec
        return [ParamSpec(self._n("in_proj"), (2 * s.inner, s.hidden), "matrix"),
                ParamSpec(self._n("conv"), (s.inner, s.taps), "conv_taps", init=(0.0, 0.5)),
                ParamSpec(self._n("conv_bias"), (s.inner,), "conv_bias", init=(0.0, 0.1)),
                ParamSpec(self._n("x_proj"), (self.low_width, s.inner), "matrix"),
                ParamSpec(self._n("dt_proj"), (s.inner, s.dt_rank), "step_matrix", init=(0.0, s.dt_rank ** -0.5)),
                ParamSpec(self._n("dt_bias"), (s.inner,), "step_bias", init=(-2.0, 0.7)),
                ParamSpec(self._n("a_log"), (s.inner, s.state), "decay_rate", init=(1.0, 0.8)),
                ParamSpec(self._n("skip"), (s.inner,), "norm_scale"),
                ParamSpec(self._n("o"), (s.hidden, s.inner), "matrix")]

    def allocate(self, stored, rt):
        s, dev = self.spec, rt.device
        mat = lambda which, *shape: torch.empty(shape, dtype=rt.matrix_dtype([stored[self._n(which)]]), device=dev)
        f32 = lambda *shape: torch.empty(shape, dtype=torch.float32, device=dev)
        self.w_in = mat("in_proj", 2 * s.inner, s.hidden)
        self.w_x = mat("x_proj", self.low_width, s.inner)
        self.w_dt = f32(s.inner, s.dt_rank)          # widened exactly: the step size's projection is always 32-bit
        self.w_o = mat("o", s.hidden, s.inner)
        self.conv_w, self.conv_b, self.dt_b = f32(s.inner, s.taps), f32(s.inner), f32(s.inner)
        self.a_log, self.skip = f32(s.inner, s.state), f32(s.inner)
        return {self._n("in_proj"): self.w_in, self._n("x_proj"): self.w_x, self._n("dt_proj"): self.w_dt, self._n("o"): self.w_o,
                self._n("conv"): self.conv_w, self._n("conv_bias"): self.conv_b, self._n("dt_bias"): self.dt_b,
                self._n("a_log"): self.a_log, self._n("skip"): self.skip}

    def kv_layout(self):
        return None

    def state_spec(self):
        return StateSpec((self.state_words + (self.spec.taps - 1) * self.spec.inner,), torch.float32)

    def forward(self, h, ctx, layer):
        s, rt = self.spec, self.rt
        n, C = h.shape[0], s.inner
        xz = rt.ws.get("sel_xz", (n, 2 * C), torch.float32)
        linear(rt, h, self.w_in, xz)
        x = rt.ws.get("sel_x", (n, C), torch.float32)
        ops.causal_conv(xz[:, :C], self.conv_w, layer.state[:, self.state_words:] if s.taps > 1 else None, ctx.tok_seq,
                        ctx.seq_start, ctx.seq_slot, x, ctx.n_seqs, s.taps, silu=True, bias=self.conv_b)
        xa = x
        if rt.dtype != torch.float32:
            xa = rt.ws.get("sel_x_act", (n, C), rt.dtype)
            ops.cast_cols(x, xa)
        low = rt.ws.get("sel_low", (n, self.low_width), torch.float32)          # dt_low | B | C
        linear(rt, xa, self.w_x, low)
        dt_raw = rt.ws.get("sel_dt", (n, C), torch.float32)
        # the step size enters the recurrence: its projection is a true 32-bit product, whatever the engine's dtype.  The
        # 32-bit engine keeps the kernel with the fixed order of sums for every step; the bfloat16 engine hands steps of
        # many rows to the library's 32-bit product (no reduced-precision matrix mode), as it does with its other products.
        if rt.dtype == torch.float32 or n <= SKINNY_ROWS or torch.backends.cuda.matmul.allow_tf32:
            ops.gemm_simt(low[:, :s.dt_rank], self.w_dt, dt_raw, bias=self.dt_b)
        else:
            torch.addmm(self.dt_b, low[:, :s.dt_rank], self.w_dt.t(), out=dt_raw)
        y = rt.ws.get("sel_y", (n, C), rt.dtype)
        ops.selective_scan(x, dt_raw, low[:, s.dt_rank:], xz[:, C:], self.a_log, self.skip, layer.state, ctx.seq_start,
                           ctx.seq_slot, y, ctx.n_seqs, C, s.state)
        out = rt.ws.get("mixer_out", (n, s.hidden), torch.float32)
        linear(rt, y, self.w_o, out)
        return out


register("mixer", "selective_scan", SelectiveScan)
