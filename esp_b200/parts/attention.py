"""Softmax attention over the paged cache with grouped query heads."""
from __future__ import annotations

import numpy as np
import torch

from ..cache import KvLayout
from ..cache.book import PAGE
from ..csrc import ops
from ..errors import Unsupported
from .base import ParamSpec, Part, build, register
from .linear import linear
from .position import NoPosition


DECODE_ROWS = 128      # steps with at most this many token rows use the split-key kernel


# ---- attention with the scores' scale given, keys and values of different sizes, a sink, a window or a mask of blocks:
# which kernel a step of n token rows gets, the index lists it needs, and the launch.  Shared by the parts below.
def scaled_kernel_for(rt, key_dim: int, value_dim: int, scale: float, n: int, page: int = PAGE) -> str:
    if rt.dtype == torch.bfloat16 and page == PAGE:
        same = key_dim == value_dim and scale > 0
        if same and key_dim in (64, 128, 192, 256) and n <= DECODE_ROWS:
            return "split"         # few rows: the keys are split over blocks
        if same and ops.attn_prefill_tc05_fits(key_dim, page):
            return "tc05"          # many rows: scores and weighted values in tensor memory
        if ops.attn_flash_fits(key_dim, value_dim):
            return "flash"         # keys and values of different sizes, any multiples of 8 up to 128
    return "plain"


def scaled_tiles(kind: str, step) -> dict:
    """Tiles of new tokens for the two tensor-core kernels of many rows: (sequence, first new token) per tile; for
    the tensor-memory kernel the tiles that see the most keys come first (its blocks take them in order)."""
    if kind == "tc05":
        rows = ops.ATTN_TC05_TILE_ROWS
        tiles = sorted(((i, f) for i, t in enumerate(step.news) for f in range(0, t, rows)),
                       key=lambda sf: -(step.pasts[sf[0]] + min(sf[1] + rows, step.news[sf[0]])))
    elif kind == "flash":
        rows = 64
        tiles = [(i, f) for i, t in enumerate(step.news) for f in range(0, t, rows)]
    else:
        return {}
    return {f"attention.tiles{rows}.seq": np.asarray([t[0] for t in tiles], dtype=np.int32),
            f"attention.tiles{rows}.first": np.asarray([t[1] for t in tiles], dtype=np.int32)}


def scaled_attend(rt, kind, q, o, ctx, layer, num_heads, num_kv_heads, key_dim, value_dim, scale, sink, window=None, chunk=None):
    """``sink``: False, True (a term exp(0)) or a float32 tensor with a number per head (a term exp(sink_h))."""
    n = q.shape[0]
    table = ctx.block_tables[layer.group]
    tile_seq = tile_first = None
    if kind in ("tc05", "flash"):
        rows = ops.ATTN_TC05_TILE_ROWS if kind == "tc05" else 64
        tile_seq, tile_first = ctx.arrays.get(f"attention.tiles{rows}.seq"), ctx.arrays.get(f"attention.tiles{rows}.first")
        if tile_seq is None:
            kind = "plain"         # a step made without this part's lists
    if kind == "split":
        positions = table.shape[1] * layer.page
        group = num_heads // num_kv_heads
        kv_blocks = num_kv_heads * ((group + 15) // 16)
        # a layer with a window or a mask of blocks reads at most that many keys (+ a page) of each row
        seen = window or chunk
        span = min(positions, seen + layer.page) if seen else positions
        split = ops.attn_decode_split(n, kv_blocks, span, key_dim, rt.sm_count)
        n_splits = (positions + split - 1) // split
        part_o = rt.ws.get("attn_part_o", (n, num_heads, n_splits, key_dim), torch.float32)
        part_ml = rt.ws.get("attn_part_ml", (n, num_heads, n_splits, 2), torch.float32)
        if getattr(rt, "attn_counters", None) is None:
            rt.attn_counters = torch.zeros(ops.ATTN_DECODE_COUNTERS, dtype=torch.int32, device=rt.device)
        ops.attn_decode(q, layer.k, layer.v, o, part_o, part_ml, rt.attn_counters, ctx.tok_seq, ctx.tok_pos, table, layer.page,
                        num_heads, num_kv_heads, key_dim, window, split, n_splits, rt.status,
                        seq_past=ctx.seq_past if layer.writes else None, scale=scale, sink=sink, chunk=chunk)
    elif kind == "tc05":
        ops.attn_prefill_tc05(q, layer.k, layer.v, o, tile_seq, tile_first, ctx.seq_start, ctx.seq_past, table, layer.page,
                              num_heads, num_kv_heads, key_dim, window, rt.status, scale=scale, sink=sink, chunk=chunk)
    elif kind == "flash":
        ops.attn_prefill(q, layer.k, layer.v, o, tile_seq, tile_first, ctx.seq_start, ctx.seq_past, table, layer.page,
                         num_heads, num_kv_heads, key_dim, window, rt.status, vd=value_dim, scale=scale, sink=sink, chunk=chunk)
    else:
        ops.attn_simt(q, layer.k, layer.v, o, ctx.tok_seq, ctx.tok_pos, table, layer.page, num_heads, num_kv_heads,
                      key_dim, window, rt.status, vd=value_dim, scale=scale, sink=sink, chunk=chunk)


class Attention(Part):
    """q/k/v projection (+bias), position encoding of q and k, cache write,
    causal (optionally windowed) softmax attention, output projection
    (crates/esp/src/infer/decoder/attention.rs:292-404).  Query head i reads
    key/value head i // (num_heads / num_kv_heads)."""

    graph_safe = True

    def __init__(self, spec, rt):
        self.spec = spec
        self.rt = rt
        s = spec
        if s.head_dim % 8 != 0 or s.head_dim > 256:
            raise Unsupported("head_dim", f"{s.head_dim}; the attention kernels take head sizes that are multiples "
                                          f"of 8 up to 256")
        if s.num_heads % s.num_kv_heads != 0:
            raise Unsupported("num_key_value_heads", f"{s.num_kv_heads} does not divide {s.num_heads} heads")
        self.q_width = s.num_heads * s.head_dim
        self.kv_width = s.num_kv_heads * s.head_dim
        self.qkv_width = self.q_width + 2 * self.kv_width
        # layers with the same encoding share one part (and its tables)
        key = ("position", s.position)
        if key not in rt.shared_parts:
            rt.shared_parts[key] = build("position", s.position, rt) if s.position is not None else NoPosition(None, rt)
        self.position = rt.shared_parts[key]
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = None

    def children(self):
        return [self.position]

    # -- parameters ----------------------------------------------------------
    def _name(self, which: str, bias: bool = False) -> str:
        n = self.spec.names
        return self.spec.prefix + getattr(n, which) + (n.bias if bias else n.weight)

    def param_specs(self):
        s = self.spec
        specs = [ParamSpec(self._name("q"), (self.q_width, s.hidden), "matrix"),
                 ParamSpec(self._name("k"), (self.kv_width, s.hidden), "matrix"),
                 ParamSpec(self._name("v"), (self.kv_width, s.hidden), "matrix"),
                 ParamSpec(self._name("o"), (s.hidden, self.q_width), "matrix")]
        if s.qkv_bias:
            specs += [ParamSpec(self._name("q", True), (self.q_width,), "bias"),
                      ParamSpec(self._name("k", True), (self.kv_width,), "bias"),
                      ParamSpec(self._name("v", True), (self.kv_width,), "bias")]
        if s.out_bias:
            specs.append(ParamSpec(self._name("o", True), (s.hidden,), "bias"))
        return specs

    def allocate(self, stored, rt):
        s = self.spec
        names = [self._name("q"), self._name("k"), self._name("v")]
        dt = rt.matrix_dtype([stored[n] for n in names])
        self.w_qkv = torch.empty((self.qkv_width, s.hidden), dtype=dt, device=rt.device)
        self.w_o = torch.empty((s.hidden, self.q_width), dtype=rt.matrix_dtype([stored[self._name("o")]]),
                               device=rt.device)
        a, b = self.q_width, self.q_width + self.kv_width
        views = {names[0]: self.w_qkv[:a], names[1]: self.w_qkv[a:b], names[2]: self.w_qkv[b:],
                 self._name("o"): self.w_o}
        if s.qkv_bias:
            self.b_qkv = torch.empty(self.qkv_width, dtype=torch.float32, device=rt.device)
            views.update({self._name("q", True): self.b_qkv[:a], self._name("k", True): self.b_qkv[a:b],
                          self._name("v", True): self.b_qkv[b:]})
        if s.out_bias:
            self.b_o = torch.empty(s.hidden, dtype=torch.float32, device=rt.device)
            views[self._name("o", True)] = self.b_o
        return views

    # -- which kernel a step of n token rows gets, and the index lists it needs ----------
    def kernel_for(self, n: int, page: int = PAGE) -> str:
        s, rt = self.spec, self.rt
        if rt.dtype == torch.bfloat16:
            if s.head_dim in (64, 128, 192, 256) and n <= DECODE_ROWS and page == PAGE:
                return "split"         # few rows: split the keys over blocks so that the cache streams at full width
            if ops.attn_prefill_tc05_fits(s.head_dim, page):
                return "tc05"          # many rows, head size 64 or 128: scores and weighted values in tensor memory
            if s.head_dim <= 128 and page == 64:
                return "flash"
        return "plain"

    def step_arrays_key(self):
        return ("attention", self.rt.dtype, self.spec.head_dim)

    def step_arrays(self, step):
        """Tiles of new tokens for the two prefill kernels: (sequence, first new token) per tile; for the
        tensor-memory kernel the tiles that see the most keys come first (its blocks take them in order)."""
        kind = self.kernel_for(step.n_tokens)
        if kind == "tc05":
            rows = ops.ATTN_TC05_TILE_ROWS
            tiles = sorted(((i, f) for i, t in enumerate(step.news) for f in range(0, t, rows)),
                           key=lambda sf: -(step.pasts[sf[0]] + min(sf[1] + rows, step.news[sf[0]])))
        elif kind == "flash":
            rows = 64
            tiles = [(i, f) for i, t in enumerate(step.news) for f in range(0, t, rows)]
        else:
            return {}
        return {f"attention.tiles{rows}.seq": np.asarray([t[0] for t in tiles], dtype=np.int32),
                f"attention.tiles{rows}.first": np.asarray([t[1] for t in tiles], dtype=np.int32)}

    # -- what it keeps per sequence ------------------------------------------------
    def kv_layout(self):
        return KvLayout(self.spec.num_kv_heads, self.spec.head_dim, self.spec.window)

    def state_spec(self):
        return None

    # -- running ---------------------------------------------------------------
    def forward(self, h, ctx, layer):
        s, rt = self.spec, self.rt
        n = h.shape[0]
        q = rt.ws.get("attn_q", (n, self.q_width), rt.dtype)
        fused = getattr(self.position, "project_rotate_store", None)
        if fused is None or not fused(h, self.w_qkv, self.b_qkv, ctx, q, layer, s.num_heads, s.num_kv_heads, s.head_dim,
                                      rt.status):
            qkv = rt.ws.get("attn_qkv", (n, self.qkv_width), torch.float32)
            linear(rt, h, self.w_qkv, qkv)
            self.position.rotate_and_store(qkv, self.b_qkv, ctx, q, layer, s.num_heads, s.num_kv_heads, s.head_dim,
                                           rt.status)
        o = rt.ws.get("attn_o", (n, self.q_width), rt.dtype)
        self.attend(q, o, ctx, layer)
        y = rt.ws.get("mixer_out", (n, s.hidden), torch.float32)
        linear(rt, o, self.w_o, y)
        if self.b_o is not None:
            y.add_(self.b_o)
        return y

    def attend(self, q, o, ctx, layer):
        s, rt = self.spec, self.rt
        table = ctx.block_tables[layer.group]
        n = q.shape[0]
        kind = self.kernel_for(n, layer.page)
        if kind in ("tc05", "flash"):
            rows = ops.ATTN_TC05_TILE_ROWS if kind == "tc05" else 64
            tile_seq, tile_first = ctx.arrays.get(f"attention.tiles{rows}.seq"), ctx.arrays.get(f"attention.tiles{rows}.first")
            if tile_seq is None:
                kind = "plain"         # a step made without this part's lists (a caller that built its own context)
        if kind == "split":
            positions = table.shape[1] * layer.page
            group = s.num_heads // s.num_kv_heads
            kv_blocks = s.num_kv_heads * ((group + 15) // 16)
            # a windowed layer reads at most window + a page of each row, wherever in the table that lies
            span = min(positions, s.window + layer.page) if s.window else positions
            split = ops.attn_decode_split(n, kv_blocks, span, s.head_dim, rt.sm_count)
            n_splits = (positions + split - 1) // split
            part_o = rt.ws.get("attn_part_o", (n, s.num_heads, n_splits, s.head_dim), torch.float32)
            part_ml = rt.ws.get("attn_part_ml", (n, s.num_heads, n_splits, 2), torch.float32)
            if getattr(rt, "attn_counters", None) is None:
                rt.attn_counters = torch.zeros(ops.ATTN_DECODE_COUNTERS, dtype=torch.int32, device=rt.device)
            ops.attn_decode(q, layer.k, layer.v, o, part_o, part_ml, rt.attn_counters, ctx.tok_seq, ctx.tok_pos, table, layer.page,
                            s.num_heads, s.num_kv_heads, s.head_dim, s.window, split, n_splits, rt.status,
                            seq_past=ctx.seq_past if layer.writes else None)
        elif kind == "tc05":
            ops.attn_prefill_tc05(q, layer.k, layer.v, o, tile_seq, tile_first, ctx.seq_start, ctx.seq_past,
                                  table, layer.page, s.num_heads, s.num_kv_heads, s.head_dim, s.window, rt.status)
        elif kind == "flash":
            ops.attn_prefill(q, layer.k, layer.v, o, tile_seq, tile_first, ctx.seq_start, ctx.seq_past,
                             table, layer.page, s.num_heads, s.num_kv_heads, s.head_dim, s.window, rt.status)
        else:
            ops.attn_simt(q, layer.k, layer.v, o, ctx.tok_seq, ctx.tok_pos, table, layer.page, s.num_heads,
                          s.num_kv_heads, s.head_dim, s.window, rt.status)


class NormedAttention(Part):
    """Causal softmax attention without rotation over the paged cache: packed q/k/v projection (+bias), an RMS norm
    per query and key head (one weight vector for all heads of a side), a factor on the queries that grows with the
    logarithm of the position in steps, keys and values of different sizes, scores times the spec's scale, and
    (``sink``) one more term exp(0) in the softmax's denominator.  Keys are cached after their norm.  Query head i
    reads key/value head i // (num_heads / num_kv_heads)."""

    graph_safe = True

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        s = spec
        if s.key_dim > 256 or s.value_dim > 256:
            raise Unsupported("dim", f"{s.key_dim} / {s.value_dim}; the attention kernels take head sizes up to 256")
        if s.num_heads % s.num_kv_heads != 0:
            raise Unsupported("kv_heads", f"{s.num_kv_heads} does not divide {s.num_heads} heads")
        self.q_width = s.num_heads * s.key_dim
        self.k_width = s.num_kv_heads * s.key_dim
        self.v_width = s.num_kv_heads * s.value_dim
        self.o_width = s.num_heads * s.value_dim
        self.qkv_width = self.q_width + self.k_width + self.v_width
        self.w_qkv = self.b_qkv = self.w_o = self.q_norm = self.k_norm = None

    def _n(self, which, bias=False):
        n = self.spec.names
        return self.spec.prefix + getattr(n, which) + (n.bias if bias else "")

    def param_specs(self):
        s = self.spec
        specs = [ParamSpec(self._n("q"), (self.q_width, s.hidden), "matrix"),
                 ParamSpec(self._n("k"), (self.k_width, s.hidden), "matrix"),
                 ParamSpec(self._n("v"), (self.v_width, s.hidden), "matrix"),
                 ParamSpec(self._n("o"), (s.hidden, self.o_width), "matrix"),
                 ParamSpec(self._n("q_norm"), (s.key_dim,), "norm_scale"),
                 ParamSpec(self._n("k_norm"), (s.key_dim,), "norm_scale")]
        if s.qkv_bias:
            specs += [ParamSpec(self._n("q", True), (self.q_width,), "bias"),
                      ParamSpec(self._n("k", True), (self.k_width,), "bias"),
                      ParamSpec(self._n("v", True), (self.v_width,), "bias")]
        return specs

    def allocate(self, stored, rt):
        s, dev = self.spec, rt.device
        names = [self._n("q"), self._n("k"), self._n("v")]
        self.w_qkv = torch.empty((self.qkv_width, s.hidden), dtype=rt.matrix_dtype([stored[n] for n in names]), device=dev)
        self.w_o = torch.empty((s.hidden, self.o_width), dtype=rt.matrix_dtype([stored[self._n("o")]]), device=dev)
        self.q_norm = torch.empty(s.key_dim, dtype=torch.float32, device=dev)
        self.k_norm = torch.empty(s.key_dim, dtype=torch.float32, device=dev)
        a, b = self.q_width, self.q_width + self.k_width
        views = {names[0]: self.w_qkv[:a], names[1]: self.w_qkv[a:b], names[2]: self.w_qkv[b:], self._n("o"): self.w_o,
                 self._n("q_norm"): self.q_norm, self._n("k_norm"): self.k_norm}
        if s.qkv_bias:
            self.b_qkv = torch.empty(self.qkv_width, dtype=torch.float32, device=dev)
            views.update({self._n("q", True): self.b_qkv[:a], self._n("k", True): self.b_qkv[a:b],
                          self._n("v", True): self.b_qkv[b:]})
        return views

    def kv_layout(self):
        s = self.spec
        return KvLayout(s.num_kv_heads, s.key_dim, s.window, value_dim=s.value_dim if s.value_dim != s.key_dim else None)

    def state_spec(self):
        return None

    # -- which kernel a step of n token rows gets, and the index lists it needs ----------
    def kernel_for(self, n: int, page: int = PAGE) -> str:
        s = self.spec
        return scaled_kernel_for(self.rt, s.key_dim, s.value_dim, s.scale, n, page)

    def step_arrays_key(self):
        s = self.spec
        return ("attention_qknorm", self.rt.dtype, s.key_dim, s.value_dim, s.scale > 0)

    def step_arrays(self, step):
        return scaled_tiles(self.kernel_for(step.n_tokens), step)

    def forward(self, h, ctx, layer):
        s, rt = self.spec, self.rt
        n = h.shape[0]
        table = ctx.block_tables[layer.group]
        qkv = rt.ws.get("attn_qkv", (n, self.qkv_width), torch.float32)
        linear(rt, h, self.w_qkv, qkv)
        q = rt.ws.get("attn_q", (n, self.q_width), rt.dtype)
        temp = s.q_temp
        ops.qknorm_kvwrite(qkv, self.b_qkv, self.q_norm, self.k_norm, s.eps, temp.coef if temp else 0.0,
                           temp.every if temp else 0, ctx.tok_seq, ctx.tok_pos, q, layer.k, layer.v, table, layer.page,
                           s.num_heads, s.num_kv_heads, s.key_dim, s.value_dim, layer.writes, rt.status)
        o = rt.ws.get("attn_o", (n, self.o_width), rt.dtype)
        scaled_attend(rt, self.kernel_for(n, layer.page), q, o, ctx, layer, s.num_heads, s.num_kv_heads, s.key_dim, s.value_dim,
                      s.scale, s.sink, window=s.window)
        y = rt.ws.get("mixer_out", (n, s.hidden), torch.float32)
        linear(rt, o, self.w_o, y)
        return y


class WideNormAttention(Part):
    """Causal softmax attention over the paged cache whose query and key norms run over the whole projection (see
    ``WideNormAttentionSpec``): packed q/k/v projection; one kernel norms queries and keys over all their heads at
    once, rotates the first channels of every head and stores keys (normed and rotated) and values in the cache;
    the attention kernels take the scores' scale as given, a mask of blocks counted from the sequence's start
    (``chunk``) or a window, and a learned sink per head.  Query head i reads key/value head
    i // (num_heads / num_kv_heads)."""

    graph_safe = True

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        s = spec
        if s.key_dim > 256 or s.value_dim > 256:
            raise Unsupported("dim", f"{s.key_dim} / {s.value_dim}; the attention kernels take head sizes up to 256")
        if s.num_heads % s.num_kv_heads != 0:
            raise Unsupported("kv_heads", f"{s.num_kv_heads} does not divide {s.num_heads} heads")
        if s.window is not None and s.chunk is not None:
            raise Unsupported("mask", "a window and a mask of blocks on the same layer")
        self.q_width = s.num_heads * s.key_dim
        self.k_width = s.num_kv_heads * s.key_dim
        self.v_width = s.num_kv_heads * s.value_dim
        self.o_width = s.num_heads * s.value_dim
        self.qkv_width = self.q_width + self.k_width + self.v_width
        self.position = None
        if s.position is not None:
            if getattr(s.position, "factor", None) is not None:
                raise Unsupported("rot", "interpolated frequencies on an attention layer with norms over the whole projection")
            key = ("position", s.position)            # layers with the same encoding share one part (and its frequencies)
            if key not in rt.shared_parts:
                rt.shared_parts[key] = build("position", s.position, rt)
            self.position = rt.shared_parts[key]
        self.w_qkv = self.w_o = self.q_norm = self.k_norm = self.sink = None

    def children(self):
        return [self.position] if self.position is not None else []

    def _n(self, which):
        return self.spec.prefix + getattr(self.spec.names, which)

    def param_specs(self):
        s = self.spec
        specs = [ParamSpec(self._n("q"), (self.q_width, s.hidden), "matrix"),
                 ParamSpec(self._n("k"), (self.k_width, s.hidden), "matrix"),
                 ParamSpec(self._n("v"), (self.v_width, s.hidden), "matrix"),
                 ParamSpec(self._n("o"), (s.hidden, self.o_width), "matrix"),
                 ParamSpec(self._n("q_norm"), (self.q_width,), "norm_scale"),
                 ParamSpec(self._n("k_norm"), (self.k_width,), "norm_scale")]
        if s.learned_sink:
            specs.append(ParamSpec(self._n("sink"), (s.num_heads,), "attention_sink", init=(0.0, 1.0)))
        return specs

    def allocate(self, stored, rt):
        s, dev = self.spec, rt.device
        names = [self._n("q"), self._n("k"), self._n("v")]
        self.w_qkv = torch.empty((self.qkv_width, s.hidden), dtype=rt.matrix_dtype([stored[n] for n in names]), device=dev)
        self.w_o = torch.empty((s.hidden, self.o_width), dtype=rt.matrix_dtype([stored[self._n("o")]]), device=dev)
        self.q_norm = torch.empty(self.q_width, dtype=torch.float32, device=dev)
        self.k_norm = torch.empty(self.k_width, dtype=torch.float32, device=dev)
        a, b = self.q_width, self.q_width + self.k_width
        views = {names[0]: self.w_qkv[:a], names[1]: self.w_qkv[a:b], names[2]: self.w_qkv[b:], self._n("o"): self.w_o,
                 self._n("q_norm"): self.q_norm, self._n("k_norm"): self.k_norm}
        if s.learned_sink:
            self.sink = torch.empty(s.num_heads, dtype=torch.float32, device=dev)
            views[self._n("sink")] = self.sink
        return views

    def kv_layout(self):
        s = self.spec
        return KvLayout(s.num_kv_heads, s.key_dim, s.window, value_dim=s.value_dim if s.value_dim != s.key_dim else None,
                        chunk=s.chunk)

    def state_spec(self):
        return None

    # -- which kernel a step of n token rows gets, and the index lists it needs ----------
    def kernel_for(self, n: int, page: int = PAGE) -> str:
        s = self.spec
        return scaled_kernel_for(self.rt, s.key_dim, s.value_dim, s.scale, n, page)

    def step_arrays_key(self):
        s = self.spec
        return ("attention_widenorm", self.rt.dtype, s.key_dim, s.value_dim, s.scale > 0)

    def step_arrays(self, step):
        return scaled_tiles(self.kernel_for(step.n_tokens), step)

    def forward(self, h, ctx, layer):
        s, rt = self.spec, self.rt
        n = h.shape[0]
        table = ctx.block_tables[layer.group]
        qkv = rt.ws.get("attn_qkv", (n, self.qkv_width), torch.float32)
        linear(rt, h, self.w_qkv, qkv)
        q = rt.ws.get("attn_q", (n, self.q_width), rt.dtype)
        pos = self.position
        ops.widenorm_rope_kvwrite(qkv, self.q_norm, self.k_norm, s.eps, pos.inv_freq if pos is not None else None,
                                  pos.spec.rotary_dim if pos is not None else 0, 1.0, ctx.tok_seq, ctx.tok_pos, q, layer.k,
                                  layer.v, table, layer.page, s.num_heads, s.num_kv_heads, s.key_dim, s.value_dim, layer.writes,
                                  rt.status)
        o = rt.ws.get("attn_o", (n, self.o_width), rt.dtype)
        scaled_attend(rt, self.kernel_for(n, layer.page), q, o, ctx, layer, s.num_heads, s.num_kv_heads, s.key_dim, s.value_dim,
                      s.scale, self.sink if s.learned_sink else False, window=s.window, chunk=s.chunk)
        y = rt.ws.get("mixer_out", (n, s.hidden), torch.float32)
        linear(rt, o, self.w_o, y)
        return y


class UnitNormAttention(Part):
    """Causal softmax attention over the paged cache with unit heads (see ``UnitNormAttentionSpec``): one packed q/k/v
    product; one kernel adds the biases, rotates neighbouring channel pairs of the first channels of every head,
    divides every query and key head by its root mean square, blends the values with those that the first blending
    layer made for the same tokens, and stores keys (rotated, normed) and values (blended) in the cache; the
    attention kernels take the scores' scale as given, a window and a learned sink per head.  The first blending
    layer leaves its values of the step's tokens (32-bit, unrounded) in a workspace buffer that the later ones read.
    Query head i reads key/value head i // (num_heads / num_kv_heads)."""

    graph_safe = True

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        s = spec
        if s.key_dim > 256 or s.value_dim > 256:
            raise Unsupported("dim", f"{s.key_dim} / {s.value_dim}; the attention kernels take head sizes up to 256")
        if s.num_heads % s.num_kv_heads != 0:
            raise Unsupported("kv_heads", f"{s.num_kv_heads} does not divide {s.num_heads} heads")
        if s.value_blend not in (None, "first", "blend"):
            raise Unsupported("v_mix", f"{s.value_blend!r}")
        self.q_width = s.num_heads * s.key_dim
        self.k_width = s.num_kv_heads * s.key_dim
        self.v_width = s.num_kv_heads * s.value_dim
        self.o_width = s.num_heads * s.value_dim
        self.qkv_width = self.q_width + self.k_width + self.v_width
        self.position = None
        if s.position is not None:
            if s.position.rotary_dim % 2 or s.position.rotary_dim > s.key_dim:
                raise Unsupported("rot.dims", f"{s.position.rotary_dim}; an even number of channels of a head of {s.key_dim}")
            key = ("position", s.position)            # layers with the same encoding share one part (and its frequencies)
            if key not in rt.shared_parts:
                rt.shared_parts[key] = build("position", s.position, rt)
            self.position = rt.shared_parts[key]
        self.w_qkv = self.b_qkv = self.w_o = self.sink = self.blend = None

    def children(self):
        return [self.position] if self.position is not None else []

    def _n(self, which, bias=False):
        n = self.spec.names
        return self.spec.prefix + getattr(n, which) + (n.bias if bias else "")

    def param_specs(self):
        s = self.spec
        specs = [ParamSpec(self._n("q"), (self.q_width, s.hidden), "matrix"),
                 ParamSpec(self._n("k"), (self.k_width, s.hidden), "matrix"),
                 ParamSpec(self._n("v"), (self.v_width, s.hidden), "matrix"),
                 ParamSpec(self._n("o"), (s.hidden, self.o_width), "matrix")]
        if s.qkv_bias:
            specs += [ParamSpec(self._n("q", True), (self.q_width,), "bias"),
                      ParamSpec(self._n("k", True), (self.k_width,), "bias"),
                      ParamSpec(self._n("v", True), (self.v_width,), "bias")]
        if s.learned_sink:
            specs.append(ParamSpec(self._n("sink"), (s.num_heads,), "attention_sink", init=(0.0, 1.0)))
        if s.value_blend is not None:
            specs.append(ParamSpec(self._n("value_blend"), (), "value_blend", init=(0.5, 0.1)))
        return specs

    def allocate(self, stored, rt):
        s, dev = self.spec, rt.device
        names = [self._n("q"), self._n("k"), self._n("v")]
        self.w_qkv = torch.empty((self.qkv_width, s.hidden), dtype=rt.matrix_dtype([stored[n] for n in names]), device=dev)
        self.w_o = torch.empty((s.hidden, self.o_width), dtype=rt.matrix_dtype([stored[self._n("o")]]), device=dev)
        a, b = self.q_width, self.q_width + self.k_width
        views = {names[0]: self.w_qkv[:a], names[1]: self.w_qkv[a:b], names[2]: self.w_qkv[b:], self._n("o"): self.w_o}
        if s.qkv_bias:
            self.b_qkv = torch.empty(self.qkv_width, dtype=torch.float32, device=dev)
            views.update({self._n("q", True): self.b_qkv[:a], self._n("k", True): self.b_qkv[a:b],
                          self._n("v", True): self.b_qkv[b:]})
        if s.learned_sink:
            self.sink = torch.empty(s.num_heads, dtype=torch.float32, device=dev)
            views[self._n("sink")] = self.sink
        if s.value_blend is not None:
            self.blend = torch.empty(1, dtype=torch.float32, device=dev)
            views[self._n("value_blend")] = self.blend[0]
        return views

    def kv_layout(self):
        s = self.spec
        return KvLayout(s.num_kv_heads, s.key_dim, s.window, value_dim=s.value_dim if s.value_dim != s.key_dim else None)

    def state_spec(self):
        return None

    # -- which kernel a step of n token rows gets, and the index lists it needs ----------
    def kernel_for(self, n: int, page: int = PAGE) -> str:
        s = self.spec
        return scaled_kernel_for(self.rt, s.key_dim, s.value_dim, s.scale, n, page)

    def step_arrays_key(self):
        s = self.spec
        return ("attention_unitnorm", self.rt.dtype, s.key_dim, s.value_dim, s.scale > 0)

    def step_arrays(self, step):
        return scaled_tiles(self.kernel_for(step.n_tokens), step)

    def forward(self, h, ctx, layer):
        s, rt = self.spec, self.rt
        n = h.shape[0]
        table = ctx.block_tables[layer.group]
        qkv = rt.ws.get("attn_qkv", (n, self.qkv_width), torch.float32)
        linear(rt, h, self.w_qkv, qkv)
        q = rt.ws.get("attn_q", (n, self.q_width), rt.dtype)
        pos = self.position
        shared_v = None
        if s.value_blend is not None:
            # the first blending layer's values of this step's tokens, for every later one of the same width
            shared_v = rt.ws.get(f"attn_first_values_{self.v_width}", (n, self.v_width), torch.float32)
        ops.pair_rope_unitnorm_kvwrite(qkv, self.b_qkv, pos.inv_freq if pos is not None else None,
                                       pos.spec.rotary_dim if pos is not None else 0, s.eps, s.unit_heads, shared_v,
                                       {None: 0, "first": 1, "blend": 2}[s.value_blend], self.blend, ctx.tok_seq, ctx.tok_pos, q,
                                       layer.k, layer.v, table, layer.page, s.num_heads, s.num_kv_heads, s.key_dim, s.value_dim,
                                       layer.writes, rt.status)
        o = rt.ws.get("attn_o", (n, self.o_width), rt.dtype)
        scaled_attend(rt, self.kernel_for(n, layer.page), q, o, ctx, layer, s.num_heads, s.num_kv_heads, s.key_dim, s.value_dim,
                      s.scale, self.sink if s.learned_sink else False, window=s.window)
        y = rt.ws.get("mixer_out", (n, s.hidden), torch.float32)
        linear(rt, o, self.w_o, y)
        return y


register("mixer", "attention", Attention)
register("mixer", "attention_qknorm", NormedAttention)
register("mixer", "attention_widenorm", WideNormAttention)
register("mixer", "attention_unitnorm", UnitNormAttention)
