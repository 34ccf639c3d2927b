"""Position encodings: they act on the new queries and keys between the
projection and the cache write."""
from __future__ import annotations

import numpy as np
import torch

from ..csrc import ops
from .base import Part, register


class RopeSplitHalf(Part):
    """Rotary encoding over the first ``rotary_dim`` columns of each head, pairs
    (i, i + rotary_dim/2).  Frequencies 1/theta^(2i/d) and angles p*f are taken
    in 32-bit on the host once (crates/esp/src/infer/decoder/attention.rs:58-95)
    and kept as cos/sin tables [max_positions, rotary_dim/2]."""

    graph_safe = True

    def __init__(self, spec, rt):
        self.spec = spec
        self.rt = rt
        self.cos = self.sin = None

    def finalize(self):
        if self.cos is not None:
            return
        spec, rt = self.spec, self.rt
        half = spec.rotary_dim // 2
        i = np.arange(half, dtype=np.float32)
        freq = (np.float32(1.0) / np.power(np.float32(spec.theta), (np.float32(2.0) * i) / np.float32(spec.rotary_dim)))
        ang = np.arange(spec.max_positions, dtype=np.float32)[:, None] * freq.astype(np.float32)[None, :]
        self.cos = torch.from_numpy(np.cos(ang).astype(np.float32)).to(rt.device).contiguous()
        self.sin = torch.from_numpy(np.sin(ang).astype(np.float32)).to(rt.device).contiguous()

    def rotate_and_store(self, qkv, bias, ctx, q_out, layer, nh, nkv, hd, status):
        table = ctx.block_tables[layer.group] if layer.group is not None else None
        ops.rope_kvwrite(qkv, bias, ctx.tok_seq, ctx.tok_pos, self.cos, self.sin, self.spec.rotary_dim, q_out,
                         layer.k, layer.v, table, layer.page, nh, nkv, hd, layer.writes, status)

    def project_rotate_store(self, h, w_qkv, bias, ctx, q_out, layer, nh, nkv, hd, status) -> bool:
        """Optional short cut of a position part: the packed projection, this encoding and the cache write
        in one kernel.  False: not for these sizes; the caller projects and calls ``rotate_and_store``."""
        if (h.dtype != torch.bfloat16 or w_qkv.dtype != torch.bfloat16 or self.spec.rotary_dim != hd
                or layer.group is None or not ops.qkv_rope_skinny_fits(h.shape[0], h.shape[1], hd)):
            return False
        ops.qkv_rope_skinny(h, w_qkv, bias, ctx.tok_seq, ctx.tok_pos, self.cos, self.sin, q_out, layer.k, layer.v,
                            ctx.block_tables[layer.group], layer.page, nh, nkv, hd, layer.writes, status)
        return True


class NoPosition(Part):
    """No encoding: queries and keys are stored as projected."""

    graph_safe = True

    def __init__(self, spec, rt):
        self.spec = spec

    def rotate_and_store(self, qkv, bias, ctx, q_out, layer, nh, nkv, hd, status):
        table = ctx.block_tables[layer.group] if layer.group is not None else None
        ops.rope_kvwrite(qkv, bias, ctx.tok_seq, ctx.tok_pos, None, None, 0, q_out, layer.k, layer.v, table,
                         layer.page, nh, nkv, hd, layer.writes, status)


class RopeScaled(Part):
    """Split-half rotary encoding with interpolated slow frequencies (see ``ScaledRopeSpec``).  It keeps one
    frequency per pair and the magnitude factor; kernels take the angle position * frequency in 32-bit where they
    rotate, so no table bounds the positions.  With d = rotary_dim, base b and i = 0 .. d/2 - 1:
        f_i = b^(-2i/d);  corr(t) = d ln(original / (2 pi t)) / (2 ln b)
        lo = max(floor(corr(fast)), 0), hi = min(ceil(corr(slow)), d - 1), ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)
        frequency_i = f_i / factor * ramp_i + f_i (1 - ramp_i);  magnitude = 0.1 ln(factor) + 1."""

    graph_safe = True

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        self.inv_freq = None
        self.magnitude = 1.0

    def frequencies(self):
        """(float32 [rotary_dim / 2], magnitude), on the host."""
        sp = self.spec
        i = np.arange(sp.rotary_dim // 2, dtype=np.float64)
        f = np.power(float(sp.theta), -2.0 * i / sp.rotary_dim)
        mag = 1.0
        if sp.factor is not None:
            def corr(turns):
                return sp.rotary_dim * np.log(sp.original / (2.0 * np.pi * turns)) / (2.0 * np.log(sp.theta))
            lo = max(int(np.floor(corr(sp.fast))), 0)
            hi = min(int(np.ceil(corr(sp.slow))), sp.rotary_dim - 1)
            ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            f = f / sp.factor * ramp + f * (1.0 - ramp)
            mag = 0.1 * float(np.log(sp.factor)) + 1.0
        return f.astype(np.float32), float(mag)

    def finalize(self):
        if self.inv_freq is None:
            f, self.magnitude = self.frequencies()
            self.inv_freq = torch.from_numpy(f).to(self.rt.device).contiguous()


register("position", "rope_split_half", RopeSplitHalf)
register("position", "rope_split_half_scaled", RopeScaled)
register("position", "rope_neighbour_pairs", RopeScaled)     # the same frequencies; which channels form a pair is the kernel's business
register("position", "none", NoPosition)
