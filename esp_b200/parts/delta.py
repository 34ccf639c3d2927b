"""Mixers whose per-sequence state is a matrix per head with a decay per key channel: the delta rule behind short
convolutions, and gated linear attention.  A head's matrix is float32 and belongs to the sequence: it sits in the
cache's per-slot state rows, is zeroed when the slot is opened, and every step continues from what the step before
left there, whatever run of tokens it brings.  Everything between the projections and the output product is 32-bit."""
from __future__ import annotations

import torch

from ..cache import StateSpec
from ..csrc import ops
from ..errors import Unsupported
from .base import ParamSpec, Part, register
from .linear import linear


def _check_key_dim(kind, key_dim):
    if key_dim > ops.SCAN_MAX_KEY_DIM:
        raise Unsupported(kind + ".dim", f"{key_dim}; the recurrence kernels take up to {ops.SCAN_MAX_KEY_DIM} key "
                                         f"channels per head")


class GatedDelta(Part):
    """The delta rule with a decay per head and key channel (see ``GatedDeltaSpec``).  One packed product makes, from
    the layer's input, q, k, v, the raw beta and the inner rows of the two low-rank projections; a kernel runs the causal
    convolution with SiLU over q, k, v (the last taps - 1 inputs of a sequence are state); a second small product makes
    the raw decay and the raw output gate from the inner rows; a kernel makes unit vectors, decay and beta; the
    recurrence walks the tokens; a kernel norms every head's output and multiplies by the sigmoid gate; then W_o.  Per
    slot the state holds S as [heads, value columns, key channels] floats and then the convolution's inputs
    [taps - 1, channels]."""

    graph_safe = True

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        s = spec
        _check_key_dim(s.kind, s.key_dim)
        if s.num_heads % s.num_kv_heads:
            raise Unsupported(s.kind + ".kv_heads", f"{s.num_kv_heads} does not divide {s.num_heads} heads")
        if s.taps > ops.CONV_MAX_TAPS or s.taps < 1:
            raise Unsupported(s.kind + ".conv", f"{s.taps} taps; the convolution kernel takes 1 to {ops.CONV_MAX_TAPS}")
        self.kw = s.num_kv_heads * s.key_dim          # width of q, and of k
        self.vw = s.num_heads * s.value_dim
        self.dw = s.num_heads * s.key_dim             # width of the decay
        self.conv_channels = 2 * self.kw + self.vw
        self.state_words = s.num_heads * s.value_dim * s.key_dim
        # columns of the packed product: q, k, v (what the convolution reads), beta, inner decay, inner gate
        self.at_beta = self.conv_channels
        self.at_inner = self.at_beta + s.num_heads
        self.proj_width = self.at_inner + s.decay_rank + s.gate_rank
        self.w_in = self.w_low = self.w_o = self.conv_w = self.dt_bias = self.a_log = self.norm_w = None

    def _n(self, which):
        return self.spec.prefix + getattr(self.spec.names, which)

    def param_specs(self):
        s, nm = self.spec, self.spec.names
        conv = lambda t, width: ParamSpec(self._n(t) + nm.conv, (width, s.taps), "conv_taps", init=(0.0, 0.5))
        return [ParamSpec(self._n("q"), (self.kw, s.hidden), "matrix"), conv("q", self.kw),
                ParamSpec(self._n("k"), (self.kw, s.hidden), "matrix"), conv("k", self.kw),
                ParamSpec(self._n("v"), (self.vw, s.hidden), "matrix"), conv("v", self.vw),
                ParamSpec(self._n("beta"), (s.num_heads, s.hidden), "matrix"),
                ParamSpec(self._n("decay_log"), (s.num_heads,), "decay_rate", init=(-0.5, 0.7)),
                ParamSpec(self._n("norm"), (s.value_dim,), "norm_scale"),
                ParamSpec(self._n("decay_in"), (s.decay_rank, s.hidden), "matrix"),
                ParamSpec(self._n("decay_out"), (self.dw, s.decay_rank), "matrix"),
                ParamSpec(self._n("decay_bias"), (self.dw,), "decay_bias", init=(-1.0, 1.0)),
                ParamSpec(self._n("gate_in"), (s.gate_rank, s.hidden), "matrix"),
                ParamSpec(self._n("gate_out"), (self.vw, s.gate_rank), "matrix"),
                ParamSpec(self._n("o"), (s.hidden, self.vw), "matrix")]

    def allocate(self, stored, rt):
        s, nm, dev = self.spec, self.spec.names, rt.device
        f32 = lambda *shape: torch.empty(shape, dtype=torch.float32, device=dev)
        order = ["q", "k", "v", "beta", "decay_in", "gate_in"]
        sizes = [self.kw, self.kw, self.vw, s.num_heads, s.decay_rank, s.gate_rank]
        names = [self._n(t) for t in order]
        self.w_in = torch.empty((self.proj_width, s.hidden), dtype=rt.matrix_dtype([stored[n] for n in names]), device=dev)
        views, at = {}, 0
        for n, size in zip(names, sizes):
            views[n] = self.w_in[at:at + size]
            at += size
        # the two second halves of the low-rank projections as one block-diagonal product over [inner decay | inner gate]
        low = [self._n("decay_out"), self._n("gate_out")]
        self.w_low = torch.zeros((self.dw + self.vw, s.decay_rank + s.gate_rank), dtype=rt.matrix_dtype([stored[n] for n in low]),
                                 device=dev)
        views[low[0]] = self.w_low[:self.dw, :s.decay_rank]
        views[low[1]] = self.w_low[self.dw:, s.decay_rank:]
        self.w_o = torch.empty((s.hidden, self.vw), dtype=rt.matrix_dtype([stored[self._n("o")]]), device=dev)
        self.conv_w = f32(self.conv_channels, s.taps)
        self.dt_bias, self.a_log, self.norm_w = f32(self.dw), f32(s.num_heads), f32(s.value_dim)
        views.update({self._n("q") + nm.conv: self.conv_w[:self.kw], self._n("k") + nm.conv: self.conv_w[self.kw:2 * self.kw],
                      self._n("v") + nm.conv: self.conv_w[2 * self.kw:], self._n("decay_bias"): self.dt_bias,
                      self._n("decay_log"): self.a_log, self._n("norm"): self.norm_w, self._n("o"): self.w_o})
        return views

    def kv_layout(self):
        return None

    def state_spec(self):
        return StateSpec((self.state_words + (self.spec.taps - 1) * self.conv_channels,), torch.float32)

    def forward(self, h, ctx, layer):
        s, rt = self.spec, self.rt
        n, H = h.shape[0], s.num_heads
        proj = rt.ws.get("delta_proj", (n, self.proj_width), torch.float32)
        linear(rt, h, self.w_in, proj)
        qkv = rt.ws.get("delta_qkv", (n, self.conv_channels), torch.float32)
        ops.causal_conv(proj[:, :self.conv_channels], self.conv_w, layer.state[:, self.state_words:] if s.taps > 1 else None,
                        ctx.tok_seq, ctx.seq_start, ctx.seq_slot, qkv, ctx.n_seqs, s.taps, silu=True)
        inner = rt.ws.get("delta_inner", (n, s.decay_rank + s.gate_rank), rt.dtype)
        ops.cast_cols(proj[:, self.at_inner:], inner)
        low = rt.ws.get("delta_low", (n, self.dw + self.vw), torch.float32)       # raw decay, raw output gate
        linear(rt, inner, self.w_low, low)
        decay = rt.ws.get("delta_decay", (n, self.dw), torch.float32)
        beta = rt.ws.get("delta_beta", (n, H), torch.float32)
        ops.delta_prepare(qkv[:, :2 * self.kw], s.num_kv_heads, s.key_dim, s.unit_eps, s.key_dim ** -0.5, low[:, :self.dw],
                          decay, self.dt_bias, self.a_log, proj[:, self.at_beta:self.at_beta + H], beta, H)
        o = rt.ws.get("rec_out", (n, self.vw), torch.float32)
        ops.delta_scan(qkv[:, :self.kw], qkv[:, self.kw:2 * self.kw], decay, qkv[:, 2 * self.kw:], beta, layer.state,
                       ctx.seq_start, ctx.seq_slot, o, ctx.n_seqs, H, s.num_kv_heads, s.key_dim, s.value_dim)
        y = rt.ws.get("rec_normed", (n, self.vw), rt.dtype)
        ops.head_rmsnorm_gate(o, self.norm_w, 0, low[:, self.dw:], y, H, s.value_dim, s.eps, gate_sigmoid=True)
        out = rt.ws.get("delta_out", (n, s.hidden), torch.float32)
        linear(rt, y, self.w_o, out)
        return out


class ChannelDecayAttention(Part):
    """Gated linear attention (see ``ChannelDecayAttentionSpec``).  One packed product makes q, k, v, the output gate and
    the inner rows of the decay's low-rank projection; a second makes the raw decay; a kernel turns it into
    sigmoid(.)^(1/tau) and scales the queries; the shared recurrence kernel walks the tokens (the read-out sees the
    token's own write); every head's output is RMS-normed and multiplied by the SiLU gate; then W_o."""

    graph_safe = True

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        s = spec
        _check_key_dim(s.kind, s.key_dim)
        self.kw, self.vw = s.num_heads * s.key_dim, s.num_heads * s.value_dim
        self.at_v, self.at_gate = 2 * self.kw, 2 * self.kw + self.vw
        self.at_inner = self.at_gate + self.vw
        self.proj_width = self.at_inner + s.decay_rank
        self.w_in = self.w_a2 = self.w_o = self.bias = self.norm_w = None

    def _n(self, which):
        return self.spec.prefix + getattr(self.spec.names, which)

    def param_specs(self):
        s = self.spec
        return [ParamSpec(self._n("q"), (self.kw, s.hidden), "matrix"), ParamSpec(self._n("k"), (self.kw, s.hidden), "matrix"),
                ParamSpec(self._n("v"), (self.vw, s.hidden), "matrix"), ParamSpec(self._n("gate"), (self.vw, s.hidden), "matrix"),
                ParamSpec(self._n("o"), (s.hidden, self.vw), "matrix"), ParamSpec(self._n("norm"), (s.value_dim,), "norm_scale"),
                ParamSpec(self._n("decay_in"), (s.decay_rank, s.hidden), "matrix"),
                ParamSpec(self._n("decay_out"), (self.kw, s.decay_rank), "matrix"),
                ParamSpec(self._n("decay_bias"), (self.kw,), "decay_bias", init=(2.0, 1.5))]

    def allocate(self, stored, rt):
        s, dev = self.spec, rt.device
        order = ["q", "k", "v", "gate", "decay_in"]
        sizes = [self.kw, self.kw, self.vw, self.vw, s.decay_rank]
        names = [self._n(t) for t in order]
        self.w_in = torch.empty((self.proj_width, s.hidden), dtype=rt.matrix_dtype([stored[n] for n in names]), device=dev)
        views, at = {}, 0
        for n, size in zip(names, sizes):
            views[n] = self.w_in[at:at + size]
            at += size
        self.w_a2 = torch.empty((self.kw, s.decay_rank), dtype=rt.matrix_dtype([stored[self._n("decay_out")]]), device=dev)
        self.w_o = torch.empty((s.hidden, self.vw), dtype=rt.matrix_dtype([stored[self._n("o")]]), device=dev)
        self.bias = torch.empty(self.kw, dtype=torch.float32, device=dev)
        self.norm_w = torch.empty(s.value_dim, dtype=torch.float32, device=dev)
        views.update({self._n("decay_out"): self.w_a2, self._n("o"): self.w_o, self._n("decay_bias"): self.bias,
                      self._n("norm"): self.norm_w})
        return views

    def kv_layout(self):
        return None

    def state_spec(self):
        return StateSpec((self.spec.num_heads * self.spec.value_dim * self.spec.key_dim,), torch.float32)

    def forward(self, h, ctx, layer):
        s, rt = self.spec, self.rt
        n = h.shape[0]
        proj = rt.ws.get("gla_proj", (n, self.proj_width), torch.float32)
        linear(rt, h, self.w_in, proj)
        inner = rt.ws.get("gla_inner", (n, s.decay_rank), rt.dtype)
        ops.cast_cols(proj[:, self.at_inner:], inner)
        decay = rt.ws.get("gla_decay", (n, self.kw), torch.float32)
        linear(rt, inner, self.w_a2, decay)
        q = rt.ws.get("gla_q", (n, self.kw), torch.float32)
        ops.channel_decay_prepare(decay, self.bias, s.tau, proj[:, :self.kw], s.key_dim ** -0.5, q)
        o = rt.ws.get("rec_out", (n, self.vw), torch.float32)
        ops.gated_scan(ops.SCAN_LOWER_SIGMOID, q, proj[:, self.kw:2 * self.kw], decay, proj[:, self.at_v:self.at_gate], None, None,
                       None, layer.state, ctx.seq_start, ctx.seq_slot, o, ctx.n_seqs, s.num_heads, s.key_dim, s.value_dim,
                       ready=True)
        y = rt.ws.get("rec_normed", (n, self.vw), rt.dtype)
        ops.head_rmsnorm_gate(o, self.norm_w, 0, proj[:, self.at_gate:self.at_inner], y, s.num_heads, s.value_dim, s.eps)
        out = rt.ws.get("mixer_out", (n, s.hidden), torch.float32)
        linear(rt, y, self.w_o, out)
        return out


register("mixer", "gated_delta", GatedDelta)
register("mixer", "gla", ChannelDecayAttention)
