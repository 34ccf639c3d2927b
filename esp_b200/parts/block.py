"""How the parts of one layer are arranged."""
from __future__ import annotations

import torch

from ..csrc import ops
from ..errors import Backend, Unsupported
from .base import ParamSpec, Part, build, plain_delta, register
from .norm import DeferredPostNorm


class PreNormResidualBlock(Part):
    """x += mixer(norm(x)); x += ffn(norm(x))
    (crates/esp/src/infer/decoder/layer.rs:115-153).  The residual adds are
    folded into the norm that follows them: a part's output travels as
    ``pending`` until the next norm adds it to the 32-bit residual stream."""

    graph_safe = True

    def __init__(self, spec, rt):
        self.spec = spec
        self.rt = rt
        self.mixer_norm = build("norm", spec.mixer_norm, rt)
        self.mixer = build("mixer", spec.mixer, rt)
        self.ffn_norm = build("norm", spec.ffn_norm, rt)
        self.ffn = build("ffn", spec.ffn, rt)

    def children(self):
        return [p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if p is not None]

    def forward(self, x, pending, ctx, layer):
        rt = self.rt
        h = rt.ws.get("block_h", tuple(x.shape), rt.dtype)
        self.mixer_norm.forward(x, plain_delta(self.mixer_norm, pending), h)
        delta = self.mixer.forward(h, ctx, layer)
        if self.ffn is not None:                 # a layer may be a mixer alone
            h32 = None
            if rt.dtype != torch.float32 and getattr(self.ffn, "wants_f32_input", False):
                h32 = rt.ws.get("block_h32", tuple(x.shape), torch.float32)
            self.ffn_norm.forward(x, plain_delta(self.ffn_norm, delta), h, h32=h32)
            delta = self.ffn.forward(h, ctx, h32=h32)
        if "residual_trace" in ctx.aux:
            # debugging aid (see ScaledDepthMixBlock._trace): the add is done here so that x is the layer's result
            x.add_(plain_delta(None, delta))
            ctx.aux["residual_trace"].append(x.clone())
            return None
        return delta


class ScaledDepthMixBlock(Part):
    """x <- x + m s1 * mixer(norm1(x)); x <- x + m s2 * ffn(norm2(x)) with s1, s2 a scale per channel and m the
    residual multiplier; the result X_(i+1) of layer i is kept, and what the next layer (or the model's end) reads is
    sum_j w[j] X_j over the embedding output X_0 and every result so far.  The first add is folded into the second
    norm; the second add, the bookkeeping of X and the weighted sum are one kernel.  A layer without a feed-forward
    has no second norm and no second scale."""

    graph_safe = True

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        self.mixer_norm = build("norm", spec.mixer_norm, rt)
        self.mixer = build("mixer", spec.mixer, rt)
        self.ffn_norm = build("norm", spec.ffn_norm, rt)
        self.ffn = build("ffn", spec.ffn, rt)
        self.scale1 = self.scale2 = self.weights = None
        self._folded = False

    def children(self):
        return [p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if p is not None]

    def param_specs(self):
        s = self.spec
        specs = [ParamSpec(s.mixer_scale, (s.hidden,), "norm_scale"),
                 ParamSpec(s.depth_weights, (s.index + 2,), "depth_weights", init=(1.0 / (s.index + 2), 0.2 / (s.index + 2)))]
        if s.ffn_scale is not None:
            specs.append(ParamSpec(s.ffn_scale, (s.hidden,), "norm_scale"))
        return specs

    def allocate(self, stored, rt):
        s = self.spec
        f32 = lambda n: torch.empty(n, dtype=torch.float32, device=rt.device)
        self.scale1, self.weights = f32(s.hidden), f32(s.index + 2)
        views = {s.mixer_scale: self.scale1, s.depth_weights: self.weights}
        if s.ffn_scale is not None:
            self.scale2 = f32(s.hidden)
            views[s.ffn_scale] = self.scale2
        return views

    def finalize(self):
        if not self._folded:                      # the residual multiplier goes into the scales once
            self._folded = True
            self.scale1.mul_(self.spec.residual_mult)
            if self.scale2 is not None:
                self.scale2.mul_(self.spec.residual_mult)

    def forward(self, x, pending, ctx, layer):
        rt, s = self.rt, self.spec
        n = x.shape[0]
        history = rt.ws.get("depth_history", (s.depth + 1, n, s.hidden), torch.float32)
        h = rt.ws.get("block_h", tuple(x.shape), rt.dtype)
        self.mixer_norm.forward(x, plain_delta(self.mixer_norm, pending), h)
        if s.index == 0:
            history[0].copy_(x)                   # X_0: what the embedding (and anything before this stack) left
        delta = self.mixer.forward(h, ctx, layer)
        if self.ffn is None:
            ops.depth_mix(x, delta, self.scale1, history, self.weights, s.index)
            self._trace(x, ctx)
            return None
        self.ffn_norm.forward(x, delta, h, delta_scale=self.scale1)
        delta = self.ffn.forward(h, ctx)
        ops.depth_mix(x, plain_delta(None, delta), self.scale2, history, self.weights, s.index)
        self._trace(x, ctx)
        return None

    @staticmethod
    def _trace(x, ctx):
        """Debugging aid: a caller that passes ``aux={"residual_trace": []}`` to the step gets a copy of the
        residual stream behind every layer (such a step is never replayed from a captured graph)."""
        if "residual_trace" in ctx.aux:
            ctx.aux["residual_trace"].append(x.clone())


class SandwichBlock(Part):
    """x += post1(mixer(pre1(x))); x += post2(ffn(pre2(x))): a norm before and a norm after every sublayer.  A
    sublayer's result travels as a ``DeferredPostNorm`` until the next norm that reads x (this block's, the next
    block's or the model's last) normalises it, adds it and normalises x, all in one launch."""

    graph_safe = True

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        self.mixer_norm = build("norm", spec.mixer_norm, rt)
        self.mixer_post = build("norm", spec.mixer_post_norm, rt)
        self.mixer = build("mixer", spec.mixer, rt)
        self.ffn_norm = build("norm", spec.ffn_norm, rt)
        self.ffn_post = build("norm", spec.ffn_post_norm, rt)
        self.ffn = build("ffn", spec.ffn, rt)

    def children(self):
        return [p for p in (self.mixer_norm, self.mixer, self.mixer_post, self.ffn_norm, self.ffn, self.ffn_post)
                if p is not None]

    def forward(self, x, pending, ctx, layer):
        rt = self.rt
        h = rt.ws.get("block_h", tuple(x.shape), rt.dtype)
        self.mixer_norm.forward(x, plain_delta(self.mixer_norm, pending), h)
        pending = DeferredPostNorm(rt, self.mixer.forward(h, ctx, layer), self.mixer_post)
        if self.ffn is not None:
            h32 = None
            if rt.dtype != torch.float32 and getattr(self.ffn, "wants_f32_input", False):
                h32 = rt.ws.get("block_h32", tuple(x.shape), torch.float32)
            self.ffn_norm.forward(x, plain_delta(self.ffn_norm, pending), h, h32=h32)
            pending = DeferredPostNorm(rt, plain_delta(None, self.ffn.forward(h, ctx, h32=h32)), self.ffn_post)
        if "residual_trace" in ctx.aux:
            # debugging aid (see ScaledDepthMixBlock._trace): the add is done here so that x is the layer's result
            pending.add_to(x)
            ctx.aux["residual_trace"].append(x.clone())
            return None
        return pending


class DeferredStreamWrite:
    """The write of a sublayer into the copies of the residual stream, on its way to whoever reads them next: the
    next layer's first read, or the model's last norm (which then sees the sum of the copies).  Either does the
    write and its own read in one launch."""

    def __init__(self, rt, streams, x, y, mix, out_w):
        self.rt, self.streams, self.x, self.y, self.mix, self.out_w = rt, streams, x, y, mix, out_w

    def apply(self, h, gamma, eps, read_w=None, rows=None, u_out=None, write_streams=True):
        ops.hc_step(self.streams, h, gamma, eps, y=self.y, mix=self.mix, out_w=self.out_w, read_w=read_w, rows=rows,
                    u_out=u_out, write_streams=write_streams)

    def materialize(self):
        """Does the write, leaves the sum of the copies in the model's residual rows; nothing is left to add."""
        self.apply(None, None, 0.0, u_out=self.x)
        return None

    def fused_add_rmsnorm(self, x, gamma, h, eps, rows, write_x, h32):
        if h32 is not None:
            self.materialize()
            ops.add_rmsnorm(x, None, gamma, h, eps, rows=rows, write_x=False, h32=h32)
            return
        self.apply(h, gamma, eps, rows=rows, u_out=x if write_x else None, write_streams=write_x)


class HyperConnectionBlock(Part):
    """A pre-norm layer over several copies of the residual stream (see ``HyperConnectionBlockSpec``).  The copies
    are float32 [streams, rows, width].  What lies between two sublayers is one launch: the write of the one that
    ran (all copies at once from the old ones), the weighted read of the next and its RMS norm.  The stack's first
    layer fills the copies from the rows it is given; the last layer's second write travels on to the model's last
    norm, which reads the plain sum of the copies."""

    graph_safe = True

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        if spec.streams > ops.HC_MAX_STREAMS or spec.streams < 1:
            raise Unsupported("streams", f"{spec.streams}; the kernel takes 1 to {ops.HC_MAX_STREAMS} copies of the residual stream")
        self.mixer_norm = build("norm", spec.mixer_norm, rt)
        self.mixer = build("mixer", spec.mixer, rt)
        self.ffn_norm = build("norm", spec.ffn_norm, rt)
        self.ffn = build("ffn", spec.ffn, rt)
        self.weights = {}

    def children(self):
        return [p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if p is not None]

    def _prefixes(self):
        s = self.spec
        return [s.mixer_prefix] + ([s.ffn_prefix] if s.ffn is not None else [])

    def param_specs(self):
        s, nm, S = self.spec, self.spec.names, self.spec.streams
        specs = []
        for p in self._prefixes():
            specs += [ParamSpec(p + nm.read, (S,), "stream_read", init=(1.0 / S, 0.3 / S)),
                      ParamSpec(p + nm.write, (S,), "stream_write", init=(1.0, 0.3)),
                      ParamSpec(p + nm.mix, (S, S), "stream_mix", init=(0.0, 0.2))]
        return specs

    def allocate(self, stored, rt):
        nm, S = self.spec.names, self.spec.streams
        views = {}
        for p in self._prefixes():
            block = torch.empty(S * S + 2 * S, dtype=torch.float32, device=rt.device)
            w = {"mix": block[:S * S].view(S, S), "read": block[S * S:S * S + S], "write": block[S * S + S:]}
            self.weights[p] = w
            views.update({p + nm.mix: w["mix"], p + nm.read: w["read"], p + nm.write: w["write"]})
        return views

    def forward(self, x, pending, ctx, layer):
        rt, s = self.rt, self.spec
        n = x.shape[0]
        streams = rt.ws.get("residual_streams", (s.streams, n, s.hidden), torch.float32)
        h = rt.ws.get("block_h", tuple(x.shape), rt.dtype)
        w1 = self.weights[s.mixer_prefix]
        gamma1, eps = self.mixer_norm.weight, s.mixer_norm.eps
        if isinstance(pending, DeferredStreamWrite) and pending.streams.data_ptr() == streams.data_ptr() and s.index > 0:
            pending.apply(h, gamma1, eps, read_w=w1["read"])
        elif s.index == 0:
            before = plain_delta(None, pending)
            if before is not None:
                x.add_(before)
            ops.hc_step(streams, h, gamma1, eps, x0=x, read_w=w1["read"])          # every copy starts as x
        else:
            if pending is not None:
                raise Backend("a layer over several residual streams was handed a result that is not a write into them")
            ops.hc_step(streams, h, gamma1, eps, read_w=w1["read"], write_streams=False)
        y = plain_delta(None, self.mixer.forward(h, ctx, layer))
        last = w1
        if self.ffn is not None:
            w2 = self.weights[s.ffn_prefix]
            ops.hc_step(streams, h, self.ffn_norm.weight, s.ffn_norm.eps, y=y, mix=w1["mix"], out_w=w1["write"], read_w=w2["read"])
            y = plain_delta(None, self.ffn.forward(h, ctx))
            last = w2
        pending = DeferredStreamWrite(rt, streams, x, y, last["mix"], last["write"])
        if "residual_trace" in ctx.aux:
            # debugging aid (see ScaledDepthMixBlock._trace): the write is done here so that x is the layer's result
            pending.materialize()
            ctx.aux["residual_trace"].append(x.clone())
            return None
        return pending


register("block", "prenorm_residual", PreNormResidualBlock)
register("block", "hyper_connections", HyperConnectionBlock)
register("block", "sandwich_residual", SandwichBlock)
register("block", "prenorm_scaled_depthmix", ScaledDepthMixBlock)
