"""Feed-forward parts: a dense SwiGLU MLP and the sparse block with routed
experts and a gated shared expert."""
from __future__ import annotations

import torch

from ..csrc import ops
from ..errors import Unsupported
from .base import ParamSpec, Part, register
from .linear import grouped_linear, grouped_swiglu_linear, grouped_uses_tc05, linear, relu2_linear, swiglu_linear, xielu_linear


class DeferredMoeCombine:
    """What a sparse block hands on instead of its output when nothing has to see that output by itself:
    the pieces of the combine.  A norm that knows the fused kernel adds and normalises in one launch
    (``fused_add_rmsnorm``); anything else calls ``materialize()`` and gets the plain tensor."""

    def __init__(self, rt, expert_out, ids, inverse, gate, shared, width, passing=None):
        self.rt, self.expert_out, self.ids, self.inverse, self.gate, self.shared = rt, expert_out, ids, inverse, gate, shared
        self.width = width
        self.passing = passing      # (weights, the block's input rows in 32-bit, first id without weights) or None

    def materialize(self):
        y = self.rt.ws.get("ffn_out", (self.ids.shape[0], self.width), torch.float32)
        ops.moe_combine(self.expert_out, self.ids, self.inverse, self.gate, self.shared, y, passing=self.passing)
        return y

    def fused_add_rmsnorm(self, x, gamma, h, eps, rows, write_x, h32):
        ops.moe_combine_add_rmsnorm(self.expert_out, self.ids, self.inverse, self.gate, self.shared, x, gamma, h, eps,
                                    rows=rows, write_x=write_x, h32=h32, passing=self.passing)


# Steps with at least AHEAD_ROWS rows start the shared expert's first product on a second stream before the
# router, on all SMs but ROUTING_SMS: the router and the permutation are a chain of short launches that leaves
# the device idle, and they find room on the SMs left over (2,048 tokens, 24 layers: 12.7 -> 12.2 ms; with 4 or 16
# SMs left over 12.6 and 12.5 ms).  Below about 768 rows it does not pay (one prompt of 400 tokens: 7.4 -> 7.7 ms;
# 768: even; 1,024: 8.9 -> 8.3 ms).
AHEAD_ROWS = 768
EARLY_SECOND_PRODUCT_ROWS = 16
ROUTING_SMS = 8
SIDE_STREAM_ROWS = 64      # steps with at most this many rows run the shared expert on a second stream


def _swiglu_mlp(rt, h, w_gate_up, w_down, out, tag):
    """out = down(silu(gate h) * (up h)); w_gate_up is [2I, H], gate rows first."""
    n = h.shape[0]
    inter = w_gate_up.shape[0] // 2
    act = rt.ws.get(tag + "_act", (n, inter), rt.dtype)
    swiglu_linear(rt, h, w_gate_up, act, tag)
    linear(rt, act, w_down, out)
    return out


class DenseSwiGlu(Part):
    """y = W_d(silu(W_g h) * (W_u h)), no biases
    (crates/esp/src/infer/decoder/moe.rs:87-89, :143-148)."""

    graph_safe = True

    def __init__(self, spec, rt):
        self.spec = spec
        self.rt = rt
        self.w_gate_up = self.w_down = None

    def param_specs(self):
        s, p, n = self.spec, self.spec.prefix, self.spec.names
        return [ParamSpec(p + n.gate, (s.intermediate, s.hidden), "matrix"),
                ParamSpec(p + n.up, (s.intermediate, s.hidden), "matrix"),
                ParamSpec(p + n.down, (s.hidden, s.intermediate), "matrix")]

    def allocate(self, stored, rt):
        s, p, n = self.spec, self.spec.prefix, self.spec.names
        dt = rt.matrix_dtype([stored[p + n.gate], stored[p + n.up]])
        self.w_gate_up = torch.empty((2 * s.intermediate, s.hidden), dtype=dt, device=rt.device)
        self.w_down = torch.empty((s.hidden, s.intermediate), dtype=rt.matrix_dtype([stored[p + n.down]]),
                                  device=rt.device)
        return {p + n.gate: self.w_gate_up[:s.intermediate], p + n.up: self.w_gate_up[s.intermediate:],
                p + n.down: self.w_down}

    def forward(self, h, ctx, h32=None):
        rt = self.rt
        n = h.shape[0]
        y = rt.ws.get("ffn_out", (n, self.spec.hidden), torch.float32)
        step = rt.ffn_chunk_tokens
        for a in range(0, n, step):
            b = min(n, a + step)
            _swiglu_mlp(rt, h[a:b], self.w_gate_up, self.w_down, y[a:b], "dense")
        return y


class DenseXielu(Part):
    """y = W_down xIELU(W_up h): for z > 0 softplus(p) z^2 + z/2, else (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2,
    p and q being the two numbers of the activation's tensor."""

    graph_safe = True

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        self.w_up = self.w_down = self.pq = None

    def param_specs(self):
        s, p = self.spec, self.spec.prefix
        return [ParamSpec(p + s.up, (s.intermediate, s.hidden), "matrix"),
                ParamSpec(p + s.down, (s.hidden, s.intermediate), "matrix"),
                ParamSpec(p + s.act, (2,), "activation", init=(0.5, 0.3))]

    def allocate(self, stored, rt):
        s, p = self.spec, self.spec.prefix
        self.w_up = torch.empty((s.intermediate, s.hidden), dtype=rt.matrix_dtype([stored[p + s.up]]), device=rt.device)
        self.w_down = torch.empty((s.hidden, s.intermediate), dtype=rt.matrix_dtype([stored[p + s.down]]), device=rt.device)
        self.pq = torch.empty(2, dtype=torch.float32, device=rt.device)
        return {p + s.up: self.w_up, p + s.down: self.w_down, p + s.act: self.pq}

    def forward(self, h, ctx, h32=None):
        rt, s = self.rt, self.spec
        n = h.shape[0]
        y = rt.ws.get("ffn_out", (n, s.hidden), torch.float32)
        step = rt.ffn_chunk_tokens
        for a in range(0, n, step):
            b = min(n, a + step)
            act = rt.ws.get("xielu_act", (b - a, s.intermediate), rt.dtype)
            xielu_linear(rt, h[a:b], self.w_up, self.pq, act, "xielu")
            linear(rt, act, self.w_down, y[a:b])
        return y


def glu_clamped_linear(rt, a, w_gate_up, act, spec, tag):
    """act = g sigmoid(alpha g) (u + shift), g = min(a @ w_gate.T, limit), u = clamp(a @ w_up.T, -limit, limit), in the
    activation dtype; w_gate_up is [2I, K] with the gate rows first."""
    gu = rt.ws.get(tag + "_gu", (a.shape[0], w_gate_up.shape[0]), torch.float32)
    linear(rt, a, w_gate_up, gu)
    ops.glu_clamped(gu, act, spec.limit, spec.alpha, spec.up_shift)
    return act


class ClampedGlu(Part):
    """y = W_d(g sigmoid(alpha g) (u + shift)) with g = min(W_g h, limit) and u = clamp(W_u h, -limit, limit), no biases:
    a gated unit whose two branches are bounded before they meet."""

    graph_safe = True

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        self.w_gate_up = self.w_down = None

    def param_specs(self):
        s, p, n = self.spec, self.spec.prefix, self.spec.names
        return [ParamSpec(p + n.gate, (s.intermediate, s.hidden), "matrix"),
                ParamSpec(p + n.up, (s.intermediate, s.hidden), "matrix"),
                ParamSpec(p + n.down, (s.hidden, s.intermediate), "matrix")]

    def allocate(self, stored, rt):
        s, p, n = self.spec, self.spec.prefix, self.spec.names
        dt = rt.matrix_dtype([stored[p + n.gate], stored[p + n.up]])
        self.w_gate_up = torch.empty((2 * s.intermediate, s.hidden), dtype=dt, device=rt.device)
        self.w_down = torch.empty((s.hidden, s.intermediate), dtype=rt.matrix_dtype([stored[p + n.down]]), device=rt.device)
        return {p + n.gate: self.w_gate_up[:s.intermediate], p + n.up: self.w_gate_up[s.intermediate:], p + n.down: self.w_down}

    def forward(self, h, ctx, h32=None):
        rt, s = self.rt, self.spec
        n = h.shape[0]
        y = rt.ws.get("ffn_out", (n, s.hidden), torch.float32)
        step = rt.ffn_chunk_tokens
        for a in range(0, n, step):
            b = min(n, a + step)
            act = rt.ws.get("glu_act", (b - a, s.intermediate), rt.dtype)
            glu_clamped_linear(rt, h[a:b], self.w_gate_up, act, s, "glu")
            linear(rt, act, self.w_down, y[a:b])
        return y


class MoeSwiGluShared(Part):
    """Router (32-bit softmax over all experts, top-k, ties to the lower id,
    optional renormalisation), routed SwiGLU experts whose outputs are scaled
    by their routing weight and summed in ascending expert id, plus a shared
    SwiGLU expert scaled by sigmoid(h . w_shared_gate)
    (crates/esp/src/infer/decoder/moe.rs:135-256).  Options of the spec: router outputs without an expert behind
    them (a chosen one returns the block's input times its weight), a correction per output that counts for the
    choice only, a choice limited to the best groups of neighbouring outputs, no shared expert."""

    graph_safe = True

    def __init__(self, spec, rt):
        self.spec = spec
        self.rt = rt
        self.n_outputs = spec.num_experts + spec.identity_experts      # what the router scores
        if spec.groups > 1:
            if spec.groups > 32 or self.n_outputs % spec.groups or not 1 <= spec.keep_groups <= spec.groups:
                raise Unsupported("router.groups", f"{spec.groups} groups (keep {spec.keep_groups}) over {self.n_outputs} router "
                                                   f"outputs; the groups are equal and at most 32")
            if spec.keep_groups * (self.n_outputs // spec.groups) < spec.top_k:
                raise Unsupported("router.groups", "the kept groups hold fewer experts than are chosen")
        self.correction = None
        self.w_router = self.w_shared_gate = None
        self.w_gate_up = self.w_down = None            # [E, 2Im, H], [E, H, Im]
        self.w_shared_gate_up = self.w_shared_down = None
        # experts with at least one token, summed over this block's calls (a device counter; nothing waits for it)
        self.expert_reads = rt.new_counter("expert_reads")

    def _names(self):
        """(router, shared gate, shared (gate, up, down), [per expert (gate, up, down)])"""
        s, p, n = self.spec, self.spec.prefix, self.spec.names
        mlp = lambda q: (q + n.mlp.gate, q + n.mlp.up, q + n.mlp.down)
        return (p + n.router, p + n.shared_gate, mlp(p + n.shared),
                [mlp(p + n.expert.format(e=e)) for e in range(s.num_experts)])

    def param_specs(self):
        s = self.spec
        router, shared_gate, shared, experts = self._names()
        specs = [ParamSpec(router, (self.n_outputs, s.hidden), "matrix")]
        if s.shared_intermediate is not None:
            specs += [ParamSpec(shared_gate, (1, s.hidden), "matrix"),
                      ParamSpec(shared[0], (s.shared_intermediate, s.hidden), "matrix"),
                      ParamSpec(shared[1], (s.shared_intermediate, s.hidden), "matrix"),
                      ParamSpec(shared[2], (s.hidden, s.shared_intermediate), "matrix")]
        if s.correction is not None:
            specs.append(ParamSpec(s.prefix + s.correction, (self.n_outputs,), "router_correction", init=(0.0, 0.02)))
        for gate, up, down in experts:
            specs += [ParamSpec(gate, (s.expert_intermediate, s.hidden), "matrix"),
                      ParamSpec(up, (s.expert_intermediate, s.hidden), "matrix"),
                      ParamSpec(down, (s.hidden, s.expert_intermediate), "matrix")]
        return specs

    def allocate(self, stored, rt):
        s = self.spec
        dev = rt.device
        E, Im, Is, H = s.num_experts, s.expert_intermediate, s.shared_intermediate, s.hidden
        router, shared_gate, shared, experts = self._names()
        has_shared = Is is not None
        rdt = rt.matrix_dtype([stored[router]] + ([stored[shared_gate]] if has_shared else []))
        self.w_router = torch.empty((self.n_outputs, H), dtype=rdt, device=dev)
        gu_dt = rt.matrix_dtype([stored[n] for g, u, _d in experts for n in (g, u)])
        self.w_gate_up = torch.empty((E, 2 * Im, H), dtype=gu_dt, device=dev)
        self.w_down = torch.empty((E, H, Im), dtype=rt.matrix_dtype([stored[d] for _g, _u, d in experts]), device=dev)
        views = {router: self.w_router}
        if has_shared:
            self.w_shared_gate = torch.empty((1, H), dtype=rdt, device=dev)
            sdt = rt.matrix_dtype([stored[shared[0]], stored[shared[1]]])
            self.w_shared_gate_up = torch.empty((2 * Is, H), dtype=sdt, device=dev)
            self.w_shared_down = torch.empty((H, Is), dtype=rt.matrix_dtype([stored[shared[2]]]), device=dev)
            views.update({shared_gate: self.w_shared_gate, shared[0]: self.w_shared_gate_up[:Is],
                          shared[1]: self.w_shared_gate_up[Is:], shared[2]: self.w_shared_down})
        if s.correction is not None:
            self.correction = torch.empty(self.n_outputs, dtype=torch.float32, device=dev)
            views[s.prefix + s.correction] = self.correction
        for e, (gate, up, down) in enumerate(experts):
            views[gate] = self.w_gate_up[e, :Im]
            views[up] = self.w_gate_up[e, Im:]
            views[down] = self.w_down[e]
        return views

    wants_f32_input = True      # the router works from unrounded rows

    def forward(self, h, ctx, h32=None):
        rt = self.rt
        n = h.shape[0]
        step = rt.ffn_chunk_tokens
        if n <= step and self.spec.hidden % 4 == 0 and self.spec.hidden <= 16384:
            # one chunk: leave the combine to the norm that follows (one launch for combine, add and norm)
            return self._forward_rows(h, None, ctx, 0, h32 if h32 is not None else h)
        y = rt.ws.get("ffn_out", (n, self.spec.hidden), torch.float32)
        for a in range(0, n, step):
            b = min(n, a + step)
            self._forward_rows(h[a:b], y[a:b], ctx, a, h32[a:b] if h32 is not None else h[a:b])
        return y

    def _forward_rows(self, h, y, ctx, row0, router_in):
        s, rt = self.spec, self.rt
        n, k, E, Im, H = h.shape[0], s.top_k, s.num_experts, s.expert_intermediate, s.hidden
        R = self.n_outputs                       # router outputs: experts with weights, then those without
        has_shared = s.shared_intermediate is not None
        choice = (self.correction, s.groups, s.keep_groups) if (self.correction is not None or s.groups > 1) else None
        ws = rt.ws
        ids = ws.get("moe_ids", (n, k), torch.int32)
        wts = ws.get("moe_w", (n, k), torch.float32)
        gate = ws.get("moe_gate", (n,), torch.float32) if has_shared else None
        probs = None
        if rt.record_routing:
            probs = torch.empty((n, R), dtype=torch.float32, device=rt.device)
        offsets = ws.get("moe_offsets", (R + 1,), torch.int32)
        passing = None
        if R > E:
            ident = router_in
            if ident.dtype != torch.float32:     # a caller without unrounded rows: the rounded ones, widened
                ident = ws.get("moe_ident", tuple(h.shape), torch.float32)
                ident.copy_(router_in)
            passing = (wts, ident, E)

        perm_token = ws.get("moe_perm_token", (n * k,), torch.int32)
        perm_weight = ws.get("moe_perm_weight", (n * k,), torch.float32)
        inverse = ws.get("moe_inverse", (n, k), torch.int32)
        tiles = None
        shared = ws.get("moe_shared_out", (n, H), torch.float32) if has_shared else None
        beside = has_shared and n <= SIDE_STREAM_ROWS and rt.side_stream is not None
        ahead = has_shared and not beside and n >= AHEAD_ROWS and rt.side_stream is not None and rt.dtype == torch.bfloat16
        if ahead:
            main = torch.cuda.current_stream()
            rt.side_stream.wait_stream(main)
            act_s = ws.get("moe_shared_act", (n, s.shared_intermediate), rt.dtype)
            with torch.cuda.stream(rt.side_stream):
                swiglu_linear(rt, h, self.w_shared_gate_up, act_s, "moe_shared", max_ctas=max(2, rt.sm_count - ROUTING_SMS))
        if beside:
            # few rows: the shared expert depends neither on the router nor on the routing, so it runs beside
            # them and the routed experts on a second stream (in a captured step: a parallel branch of the graph)
            main = torch.cuda.current_stream()
            rt.side_stream.wait_stream(main)
            with torch.cuda.stream(rt.side_stream):
                _swiglu_mlp(rt, h, self.w_shared_gate_up, self.w_shared_down, shared, "moe_shared")
        uses_tc05 = grouped_uses_tc05(h, self.w_gate_up, n * k, n) and Im % 8 == 0
        if uses_tc05 and R > E:
            perm_token.zero_()                   # the gather reads n * k rows; those behind the last expert's are never placed
        if uses_tc05:
            max_tiles = (n * k + ops.TC05_TILE_ROWS - 1) // ops.TC05_TILE_ROWS + E
            tiles = (ws.get("moe_tile_group", (max_tiles,), torch.int32),
                     ws.get("moe_tile_row0", (max_tiles,), torch.int32),
                     ws.get("moe_tile_count", (max_tiles,), torch.int32), ws.get("moe_n_tiles", (1,), torch.int32))
        if n <= ops.ROUTE_SMALL_TOKENS and ops.route_small_fits(H, R):
            # few tokens: router and permutation (and the tile list, when the tensor-core products follow) in two
            # short launches
            logits = ws.get("moe_logits", (n, R + 1), torch.float32)
            ops.route_small(router_in, self.w_router, self.w_shared_gate, logits, ids, wts, gate, k, s.norm_topk,
                            offsets, perm_token, perm_weight, inverse, rt.status, probs, distinct=self.expert_reads,
                            tiles=tiles, choice=choice, n_real=E)
        else:
            ops.router_topk(router_in, self.w_router, self.w_shared_gate, ids, wts, gate, k, s.norm_topk, rt.status,
                            probs, logits=ws.get("moe_logits", (n, R + 1), torch.float32), choice=choice)
            ops.moe_permute(ids, wts, E, offsets, perm_token, perm_weight, inverse, rt.status, tiles=tiles,
                            distinct=self.expert_reads, n_ids=R)
        if rt.record_routing:
            ctx.aux.setdefault("routing", []).append((s.prefix, row0, ids.clone(), wts.clone(), probs))
        if ahead:
            main.wait_stream(rt.side_stream)
        expert_out = self.experts(h, offsets, perm_token, perm_weight, n * k, n, tiles)
        if beside:
            main.wait_stream(rt.side_stream)
        elif ahead:
            linear(rt, act_s, self.w_shared_down, shared)
        elif has_shared:
            _swiglu_mlp(rt, h, self.w_shared_gate_up, self.w_shared_down, shared, "moe_shared")
        if y is None:
            return DeferredMoeCombine(rt, expert_out, ids, inverse, gate, shared, H, passing)
        ops.moe_combine(expert_out, ids, inverse, gate, shared, y, passing=passing)
        return y

    def experts(self, h, offsets, perm_token, perm_weight, rows, max_rows, tiles=None):
        """expert_out[r] = weight[r] * down_e(silu(gate_e x) * (up_e x)) for every
        permuted row r, x = h[perm_token[r]], e the expert whose range holds r.
        ``max_rows``: no expert has more rows than this (a token names an expert once)."""
        s, rt = self.spec, self.rt
        act = rt.ws.get("moe_act", (rows, s.expert_intermediate), rt.dtype)
        grouped_swiglu_linear(rt, h, self.w_gate_up, act, offsets, perm_token, rows, max_rows, "moe", tiles)
        out = rt.ws.get("moe_expert_out", (rows, s.hidden), torch.float32)
        # the routing was complete before the first product started: the second may look its groups up and ask for
        # its weights while the first still runs.  Only for few rows, where the first product is one wave of
        # blocks and the second's blocks take no room from blocks yet to start (batch 1 +1.2 %, batch 4 +1.5 %,
        # batch 8 -0.3 %).
        grouped_linear(rt, act, self.w_down, out, offsets, perm_weight, rows, max_rows, tiles,
                       offsets_ready=rows <= EARLY_SECOND_PRODUCT_ROWS)
        return out


def _relu2_mlp(rt, h, w_up, w_down, out, tag):
    """out = down(relu(up h)^2)."""
    act = rt.ws.get(tag + "_act", (h.shape[0], w_up.shape[0]), rt.dtype)
    relu2_linear(rt, h, w_up, act, tag)
    linear(rt, act, w_down, out)
    return out


class DenseRelu2(Part):
    """y = W_down relu(W_up h)^2, no biases."""

    graph_safe = True

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        self.w_up = self.w_down = None

    def param_specs(self):
        s, p = self.spec, self.spec.prefix
        return [ParamSpec(p + s.up, (s.intermediate, s.hidden), "matrix"),
                ParamSpec(p + s.down, (s.hidden, s.intermediate), "matrix")]

    def allocate(self, stored, rt):
        s, p = self.spec, self.spec.prefix
        self.w_up = torch.empty((s.intermediate, s.hidden), dtype=rt.matrix_dtype([stored[p + s.up]]), device=rt.device)
        self.w_down = torch.empty((s.hidden, s.intermediate), dtype=rt.matrix_dtype([stored[p + s.down]]), device=rt.device)
        return {p + s.up: self.w_up, p + s.down: self.w_down}

    def forward(self, h, ctx, h32=None):
        rt, s = self.rt, self.spec
        n = h.shape[0]
        y = rt.ws.get("ffn_out", (n, s.hidden), torch.float32)
        step = rt.ffn_chunk_tokens
        for a in range(0, n, step):
            b = min(n, a + step)
            _relu2_mlp(rt, h[a:b], self.w_up, self.w_down, y[a:b], "relu2")
        return y


class ScaledInputMoe(Part):
    """Router with sigmoid scores (32-bit), the top-k experts by score (ties to the lower id), weights = the chosen
    scores as they are; a chosen expert works on weight * h: down_e(relu(up_e (w h))^2), which is computed as
    relu(w (up_e h))^2 with the weight applied to the up-projection's 32-bit result; outputs are summed in ascending
    expert id; a shared expert of the same form takes every token with weight one."""

    graph_safe = True
    wants_f32_input = True      # the router works from unrounded rows

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        if spec.activation != "relu2":
            raise Unsupported("mlp.activation", f"{spec.activation!r}; experts of this kind square a relu")
        self.w_router = self.w_up = self.w_down = self.w_shared_up = self.w_shared_down = None
        self.expert_reads = rt.new_counter("expert_reads")

    def _names(self):
        s, p = self.spec, self.spec.prefix
        experts = [(p + s.expert.format(e=e) + s.up, p + s.expert.format(e=e) + s.down) for e in range(s.num_experts)]
        return p + s.router, (p + s.shared + s.up, p + s.shared + s.down), experts

    def param_specs(self):
        s = self.spec
        router, shared, experts = self._names()
        specs = [ParamSpec(router, (s.num_experts, s.hidden), "matrix")]
        if s.shared_intermediate is not None:
            specs += [ParamSpec(shared[0], (s.shared_intermediate, s.hidden), "matrix"),
                      ParamSpec(shared[1], (s.hidden, s.shared_intermediate), "matrix")]
        for up, down in experts:
            specs += [ParamSpec(up, (s.expert_intermediate, s.hidden), "matrix"),
                      ParamSpec(down, (s.hidden, s.expert_intermediate), "matrix")]
        return specs

    def allocate(self, stored, rt):
        s, dev = self.spec, rt.device
        E, Im, H = s.num_experts, s.expert_intermediate, s.hidden
        router, shared, experts = self._names()
        self.w_router = torch.empty((E, H), dtype=rt.matrix_dtype([stored[router]]), device=dev)
        self.w_up = torch.empty((E, Im, H), dtype=rt.matrix_dtype([stored[u] for u, _d in experts]), device=dev)
        self.w_down = torch.empty((E, H, Im), dtype=rt.matrix_dtype([stored[d] for _u, d in experts]), device=dev)
        views = {router: self.w_router}
        if s.shared_intermediate is not None:
            self.w_shared_up = torch.empty((s.shared_intermediate, H), dtype=rt.matrix_dtype([stored[shared[0]]]), device=dev)
            self.w_shared_down = torch.empty((H, s.shared_intermediate), dtype=rt.matrix_dtype([stored[shared[1]]]), device=dev)
            views.update({shared[0]: self.w_shared_up, shared[1]: self.w_shared_down})
        for e, (up, down) in enumerate(experts):
            views[up] = self.w_up[e]
            views[down] = self.w_down[e]
        return views

    def forward(self, h, ctx, h32=None):
        rt = self.rt
        n = h.shape[0]
        y = rt.ws.get("ffn_out", (n, self.spec.hidden), torch.float32)
        step = rt.ffn_chunk_tokens
        for a in range(0, n, step):
            b = min(n, a + step)
            self._forward_rows(h[a:b], y[a:b], ctx, a, h32[a:b] if h32 is not None else h[a:b])
        return y

    def _forward_rows(self, h, y, ctx, row0, router_in):
        s, rt = self.spec, self.rt
        n, k, E, Im, H = h.shape[0], s.top_k, s.num_experts, s.expert_intermediate, s.hidden
        ws = rt.ws
        ids = ws.get("moe_ids", (n, k), torch.int32)
        wts = ws.get("moe_w", (n, k), torch.float32)
        probs = torch.empty((n, E), dtype=torch.float32, device=rt.device) if rt.record_routing else None
        offsets = ws.get("moe_offsets", (E + 1,), torch.int32)
        perm_token = ws.get("moe_perm_token", (n * k,), torch.int32)
        perm_weight = ws.get("moe_perm_weight", (n * k,), torch.float32)
        inverse = ws.get("moe_inverse", (n, k), torch.int32)
        rows = n * k
        tiles = None
        if grouped_uses_tc05(h, self.w_up, rows, n) and Im % 16 == 0 and H % 16 == 0:
            max_tiles = (rows + ops.TC05_TILE_ROWS - 1) // ops.TC05_TILE_ROWS + E
            tiles = (ws.get("moe_tile_group", (max_tiles,), torch.int32), ws.get("moe_tile_row0", (max_tiles,), torch.int32),
                     ws.get("moe_tile_count", (max_tiles,), torch.int32), ws.get("moe_n_tiles", (1,), torch.int32))
        shared = None
        beside = self.w_shared_up is not None and n <= SIDE_STREAM_ROWS and rt.side_stream is not None
        if beside:
            # few rows: the shared expert needs nothing of the routing and runs beside it on a second stream
            shared = ws.get("moe_shared_out", (n, H), torch.float32)
            main = torch.cuda.current_stream()
            rt.side_stream.wait_stream(main)
            with torch.cuda.stream(rt.side_stream):
                _relu2_mlp(rt, h, self.w_shared_up, self.w_shared_down, shared, "moe_shared")
        if n <= ops.ROUTE_SMALL_TOKENS and ops.route_small_fits(H, E):
            logits = ws.get("moe_logits", (n, E + 1), torch.float32)
            ops.route_small(router_in, self.w_router, None, logits, ids, wts, None, k, False, offsets, perm_token, perm_weight,
                            inverse, rt.status, probs, distinct=self.expert_reads, tiles=tiles, sigmoid=True)
        else:
            ops.router_topk(router_in, self.w_router, None, ids, wts, None, k, False, rt.status, probs,
                            logits=ws.get("moe_logits", (n, E + 1), torch.float32), sigmoid=True)
            ops.moe_permute(ids, wts, E, offsets, perm_token, perm_weight, inverse, rt.status, tiles=tiles,
                            distinct=self.expert_reads)
        if rt.record_routing:
            ctx.aux.setdefault("routing", []).append((s.prefix, row0, ids.clone(), wts.clone(), probs))
        # routed experts: z = up_e h (32-bit result), act = relu(w z)^2, out = down_e act
        z = ws.get("moe_z", (rows, Im), torch.float32)
        act = ws.get("moe_act", (rows, Im), rt.dtype)
        out = ws.get("moe_expert_out", (rows, H), torch.float32)
        if tiles is not None:
            gathered = ws.get("moe_gathered", (rows, H), torch.bfloat16)
            ops.gather_rows(h, perm_token, gathered)
            ops.gemm_tc05(gathered, self.w_up, z, rt.status, row_scale=perm_weight, tiles=tiles)
            ops.relu2(z, act)
            ops.gemm_tc05(act, self.w_down, out, rt.status, tiles=tiles)
        elif h.dtype == torch.bfloat16 and self.w_up.dtype == torch.bfloat16 and self.w_down.dtype == torch.bfloat16 \
                and ops.skinny_fits(H) and ops.skinny_fits(Im):
            # the weight and the activation are the first product's epilogue
            ops.gemm_skinny(h, self.w_up, act, a_rows=perm_token, row_scale=perm_weight, group_offsets=offsets, rows=rows,
                            max_rows=n, relu2=True)
            ops.gemm_skinny(act, self.w_down, out, group_offsets=offsets, rows=rows, max_rows=n)
        else:
            ops.gemm_simt(h, self.w_up, z, a_rows=perm_token, row_scale=perm_weight, group_offsets=offsets, rows=rows)
            ops.relu2(z, act)
            ops.gemm_simt(act, self.w_down, out, group_offsets=offsets, rows=rows)
        if self.w_shared_up is not None:
            if beside:
                main.wait_stream(rt.side_stream)
            else:
                shared = ws.get("moe_shared_out", (n, H), torch.float32)
                _relu2_mlp(rt, h, self.w_shared_up, self.w_shared_down, shared, "moe_shared")
        ops.moe_combine(out, ids, inverse, None, shared, y)
        return y


register("ffn", "swiglu", DenseSwiGlu)
register("ffn", "glu_clamped", ClampedGlu)
register("ffn", "moe_sigmoid_scaled_input", ScaledInputMoe)
register("ffn", "xielu", DenseXielu)
register("ffn", "relu2", DenseRelu2)
register("ffn", "moe_swiglu_shared", MoeSwiGluShared)
