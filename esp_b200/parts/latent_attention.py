"""Attention through a cached low-rank latent, with a sliding window and one rotated key part for all heads."""
from __future__ import annotations

import numpy as np
import torch

from ..cache import KvLayout
from ..cache.book import PAGE
from ..csrc import ops
from ..errors import Unsupported
from .attention import scaled_tiles
from .base import ParamSpec, Part, build, register
from .linear import linear

# a step of whole prompts takes the unfolded form when its longest prompt has at least this many tokens (the folded
# form's cost grows with rank x tokens squared: 2,048 tokens at rank 512 took 495 us against about 100 unfolded)
UNFOLD_ROWS = 512


class LatentAttention(Part):
    """c_q = norm(W_dq h), q = W_uq c_q laid out per head as [nope | rot]; W_dkv h gives the latent c (its first
    kv_rank rows, normed) and one rotated key part for all heads; per head the unrotated key is W_uk c and the value
    W_uv c; score = (q_nope . k_nope + q_rot . k_rot) * scale over the window; softmax; W_o on the heads.

    The cache holds one row [c | k_rot] per position and nothing per head.  The keys' up-projection is
    folded into the query (q_lat = W_uk^T q_nope per head) and the values' up-projection is applied to the
    weighted sum of latents, so every head attends to the cached rows themselves.  A layer without a
    down-projection of its own (``own_kv`` False) reads the rows another layer cached, with its own window.

    A step that brings whole prompts (nothing cached before) of which one is long may take the unfolded form instead,
    where the sizes allow it (bfloat16, no rotated part, no window, keys and values of one size that the tensor-memory
    attention takes): every head's keys and values are made from the step's latents with one dense product, written
    to pages of their own, and the tensor-memory attention of the other attention parts runs over them; the folded
    form pays rank multiply-adds a score where this pays the head size.  The cache still gets the latents."""

    graph_safe = True

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        self.position = None
        if spec.position is not None:
            key = ("position", spec.position)
            if key not in rt.shared_parts:
                rt.shared_parts[key] = build("position", spec.position, rt)
            self.position = rt.shared_parts[key]
        elif spec.rot_dim:
            raise Unsupported("rot", "a rotated key part without a position encoding")
        if spec.kv_rank > 512:
            raise Unsupported("kv_rank", f"{spec.kv_rank}; the latent attention kernels take up to 512 value channels a row")
        self.w_q = None                          # full-rank queries (q_rank None): [queries; head gates] x hidden
        self.w_ukv = None                        # [keys of every head; values of every head] x rank, for the unfolded form
        self.row = spec.kv_rank + spec.rot_dim
        self.q_head = spec.nope_dim + spec.rot_dim
        self.w_dq = self.dq_norm = self.w_uq = self.w_dkv = self.dkv_norm = self.w_uk = self.w_uv = self.w_o = self.w_gate = None
        self.w_uk_t = None

    def children(self):
        return [self.position] if self.position is not None else []

    def _n(self, which):
        return self.spec.prefix + getattr(self.spec.names, which)

    def param_specs(self):
        s = self.spec
        if s.q_rank is not None:
            specs = [ParamSpec(self._n("q_down"), (s.q_rank, s.hidden), "matrix"),
                     ParamSpec(self._n("q_norm"), (s.q_rank,), "norm_scale"),
                     ParamSpec(self._n("q_up"), (s.num_heads * self.q_head, s.q_rank), "matrix")]
        else:
            specs = [ParamSpec(self._n("q"), (s.num_heads * self.q_head, s.hidden), "matrix")]
        if s.head_gate:
            specs.append(ParamSpec(self._n("head_gate"), (s.num_heads, s.hidden), "matrix"))
        specs += [ParamSpec(self._n("k_up"), (s.num_heads * s.nope_dim, s.kv_rank), "matrix"),
                 ParamSpec(self._n("v_up"), (s.num_heads * s.value_dim, s.kv_rank), "matrix"),
                 ParamSpec(self._n("o"), (s.hidden, s.num_heads * s.value_dim), "matrix")]
        if s.own_kv:
            specs += [ParamSpec(self._n("kv_down"), (self.row, s.hidden), "matrix"),
                      ParamSpec(self._n("kv_norm"), (s.kv_rank,), "norm_scale")]
        return specs

    def allocate(self, stored, rt):
        s, dev = self.spec, rt.device
        mat = lambda which, *shape: torch.empty(shape, dtype=rt.matrix_dtype([stored[self._n(which)]]), device=dev)
        self.w_uk = mat("k_up", s.num_heads * s.nope_dim, s.kv_rank)
        self.w_uv = mat("v_up", s.num_heads * s.value_dim, s.kv_rank)
        self.w_o = mat("o", s.hidden, s.num_heads * s.value_dim)
        views = {self._n("k_up"): self.w_uk, self._n("v_up"): self.w_uv, self._n("o"): self.w_o}
        qw = s.num_heads * self.q_head
        if s.q_rank is not None:
            self.w_dq = mat("q_down", s.q_rank, s.hidden)
            self.w_uq = mat("q_up", qw, s.q_rank)
            self.dq_norm = torch.empty(s.q_rank, dtype=torch.float32, device=dev)
            views.update({self._n("q_down"): self.w_dq, self._n("q_up"): self.w_uq, self._n("q_norm"): self.dq_norm})
            if s.head_gate:
                self.w_gate = mat("head_gate", s.num_heads, s.hidden)
                views[self._n("head_gate")] = self.w_gate
        else:
            # the queries and the heads' gates are one product of the layer's input
            names = [self._n("q")] + ([self._n("head_gate")] if s.head_gate else [])
            self.w_q = torch.empty((qw + (s.num_heads if s.head_gate else 0), s.hidden),
                                   dtype=rt.matrix_dtype([stored[n] for n in names]), device=dev)
            views[names[0]] = self.w_q[:qw]
            if s.head_gate:
                views[names[1]] = self.w_q[qw:]
        if s.own_kv:
            self.w_dkv = mat("kv_down", self.row, s.hidden)
            self.dkv_norm = torch.empty(s.kv_rank, dtype=torch.float32, device=dev)
            views.update({self._n("kv_down"): self.w_dkv, self._n("kv_norm"): self.dkv_norm})
        return views

    def finalize(self):
        s = self.spec
        if self.w_uk is not None and self.w_ukv is None and self._unfolded_fits():
            self.w_ukv = torch.cat([self.w_uk, self.w_uv]).contiguous()
        if self.w_uk is not None and self.w_uk_t is None:
            # per head [kv_rank, nope]: the product that folds the keys' up-projection into the query reads it row by row
            self.w_uk_t = self.w_uk.view(s.num_heads, s.nope_dim, s.kv_rank).transpose(1, 2).contiguous()
            self.w_uk = None

    # -- what it keeps per sequence ------------------------------------------------
    def kv_layout(self):
        # one row per position for all heads, no separate values: they are the row's first kv_rank channels
        return KvLayout(1, self.row, self.spec.keep_window, values=False)

    def state_spec(self):
        return None

    # -- which attention kernel a step gets, and the index lists it needs --------------
    def _tensor_cores(self, page: int = PAGE) -> bool:
        return self.rt.dtype == torch.bfloat16 and ops.attn_latent_mma_fits(self.row, self.spec.kv_rank, page)

    def _unfolded_fits(self) -> bool:
        s = self.spec
        return (self.rt.dtype == torch.bfloat16 and s.own_kv and s.rot_dim == 0 and s.window is None and s.scale > 0
                and s.nope_dim == s.value_dim and ops.attn_prefill_tc05_fits(s.nope_dim, PAGE) and s.kv_rank % 8 == 0
                and self.w_uk is not None and self.w_uk.dtype == torch.bfloat16 and self.w_uv.dtype == torch.bfloat16)

    def step_arrays_key(self):
        if not self._tensor_cores() and self.w_ukv is None:
            return None
        return ("latent_attention", self.rt.dtype, ops.attn_latent_mma_heads(self.spec.num_heads), self._tensor_cores(),
                self.w_ukv is not None)

    def step_arrays(self, step):
        """Tiles of new tokens of one sequence for the tensor-core kernel: (sequence, first new token) per tile.  For a
        step of whole prompts with a long one, where the unfolded form runs: the pages of the step's own keys and
        values (sequence after sequence) and the tiles of the tensor-memory attention."""
        out = {}
        if self.w_ukv is not None and max(step.news) >= UNFOLD_ROWS and not any(step.pasts):
            pages = [(t + PAGE - 1) // PAGE for t in step.news]
            table = np.full((len(pages), max(pages)), -1, dtype=np.int32)
            at = 0
            for i, n in enumerate(pages):
                table[i, :n] = np.arange(at, at + n, dtype=np.int32)
                at += n
            out["latent.unfolded.table"] = table
            out.update(scaled_tiles("tc05", step))
            return out
        if self._tensor_cores():
            tq = ops.ATTN_LATENT_MMA_ROWS // ops.attn_latent_mma_heads(self.spec.num_heads)
            tiles = [(i, f) for i, t in enumerate(step.news) for f in range(0, t, tq)]
            out[f"latent.tiles{tq}.seq"] = np.asarray([t[0] for t in tiles], dtype=np.int32)
            out[f"latent.tiles{tq}.first"] = np.asarray([t[1] for t in tiles], dtype=np.int32)
        return out

    def attend(self, qx, o_lat, ctx, layer, table):
        s, rt = self.spec, self.rt
        H = s.num_heads
        hg = ops.attn_latent_mma_heads(H)
        tq = ops.ATTN_LATENT_MMA_ROWS // hg
        tile_seq = ctx.arrays.get(f"latent.tiles{tq}.seq") if self._tensor_cores(layer.page) else None
        if tile_seq is None:
            ops.attn_latent(qx, layer.k, o_lat, ctx.tok_seq, ctx.tok_pos, table, layer.page, H, self.row, s.kv_rank, s.window,
                            s.scale, rt.status)
            return
        tile_first = ctx.arrays[f"latent.tiles{tq}.first"]
        # few blocks and many pages: deal every tile's pages to several blocks (about one block an SM in all), so that
        # the cache streams at full width; every split costs a partial result of float values, so no more than that
        n = qx.shape[0]
        blocks = tile_seq.shape[0] * ((H + hg - 1) // hg)
        positions = table.shape[1] * layer.page
        span = min(positions, s.window + tq + layer.page) if s.window else positions
        pages = (span + layer.page - 1) // layer.page
        n_splits = max(1, min(pages, rt.sm_count // max(1, blocks)))
        part_o = part_ml = None
        per = 0
        if n_splits > 1:
            per = (pages + n_splits - 1) // n_splits
            n_splits = (pages + per - 1) // per
            part_o = rt.ws.get("la_part_o", (n, H, n_splits, s.kv_rank), torch.float32)
            part_ml = rt.ws.get("la_part_ml", (n, H, n_splits, 2), torch.float32)
        ops.attn_latent_mma(qx, layer.k, o_lat, tile_seq, tile_first, ctx.seq_start, ctx.seq_past, table, layer.page, H, self.row,
                            s.kv_rank, s.window, s.scale, rt.status, n_splits, per, part_o, part_ml)

    def _attend_unfolded(self, q, d, gate, ctx, table):
        """Whole prompts: keys and values of every head from the step's own latents, then the tensor-memory attention.
        q float32 [n, H * K] (a view), d float32 [n, rank] the down-projection's output, gate float32 [n, H] or None."""
        s, rt = self.spec, self.rt
        n, H, K = q.shape[0], s.num_heads, s.nope_dim
        c = rt.ws.get("la_c_act", (n, s.kv_rank), rt.dtype)
        ops.add_rmsnorm(d, None, self.dkv_norm, c, s.eps, write_x=False)          # the rows the cache got, as a matrix
        kv = rt.ws.get("la_kv", (n, 2 * H * K), torch.float32)
        linear(rt, c, self.w_ukv, kv)
        n_pages = int(table.shape[0]) * int(table.shape[1])
        k_pool = rt.ws.get("la_k_pages", (n_pages, H, PAGE, K), rt.dtype)
        v_pool = rt.ws.get("la_v_pages", (n_pages, H, PAGE, K), rt.dtype)
        # what lies behind a prompt's last token in its last page is masked, but a weight of zero times a value that is
        # no number is no number: the pages start from zeros, as the cache's own pools do
        k_pool.zero_()
        v_pool.zero_()
        ops.heads_to_pages(kv[:, :H * K], kv[:, H * K:], ctx.tok_seq, ctx.tok_pos, table, k_pool, v_pool, PAGE, H, K, K, rt.status)
        qa = rt.ws.get("la_q_act", (n, H * K), rt.dtype)
        ops.cast_cols(q, qa)
        o = rt.ws.get("la_o", (n, H * K), rt.dtype)
        rows = ops.ATTN_TC05_TILE_ROWS
        ops.attn_prefill_tc05(qa, k_pool, v_pool, o, ctx.arrays[f"attention.tiles{rows}.seq"],
                              ctx.arrays[f"attention.tiles{rows}.first"], ctx.seq_start, ctx.seq_past, table, PAGE, H, H, K,
                              None, rt.status, scale=s.scale)
        if gate is not None:
            ops.head_scalar_gate(o, gate, o, H, K)
        return o

    def forward(self, h, ctx, layer):
        s, rt, pos = self.spec, self.rt, self.position
        n, H = h.shape[0], s.num_heads
        table = ctx.block_tables[layer.group]
        qw = H * self.q_head
        gate = None                              # float32 [n, H] (a view with its row stride): one number per token and head
        if s.q_rank is not None:
            dq = rt.ws.get("la_dq", (n, s.q_rank), torch.float32)
            linear(rt, h, self.w_dq, dq)
            cq = rt.ws.get("la_cq", (n, s.q_rank), rt.dtype)
            ops.add_rmsnorm(dq, None, self.dq_norm, cq, s.eps, write_x=False)
            q = rt.ws.get("la_q", (n, qw), torch.float32)
            linear(rt, cq, self.w_uq, q)
            if s.head_gate:
                gate = rt.ws.get("la_gate", (n, H), torch.float32)
                linear(rt, h, self.w_gate, gate)
        else:
            qg = rt.ws.get("la_q", (n, self.w_q.shape[0]), torch.float32)
            linear(rt, h, self.w_q, qg)
            q = qg[:, :qw]
            if s.head_gate:
                gate = qg[:, qw:]
        inv_freq = pos.inv_freq if pos is not None else None
        magnitude = pos.magnitude if pos is not None else 1.0
        rot_dims = pos.spec.rotary_dim if pos is not None else 0
        if layer.writes:
            d = rt.ws.get("la_dkv", (n, self.row), torch.float32)
            linear(rt, h, self.w_dkv, d)
            ops.latent_kv_store(d, self.dkv_norm, inv_freq, magnitude, rot_dims, ctx.tok_seq, ctx.tok_pos,
                                table, layer.k, layer.page, s.kv_rank, s.rot_dim, s.eps, rt.status)
        unfolded = ctx.arrays.get("latent.unfolded.table") if (self.w_ukv is not None and layer.writes) else None
        if unfolded is not None:
            o = self._attend_unfolded(q, d, gate, ctx, unfolded)
            y = rt.ws.get("mixer_out", (n, s.hidden), torch.float32)
            linear(rt, o, self.w_o, y)
            return y
        qx = rt.ws.get("la_qx", (n, H * self.row), rt.dtype)
        if s.rot_dim:
            ops.latent_q_rotate(q, inv_freq, magnitude, rot_dims, ctx.tok_pos, qx, H, s.nope_dim, s.rot_dim, s.kv_rank)
        ops.per_head_linear(q, q.stride(0), self.q_head, self.w_uk_t, qx, H * self.row, self.row, n, H, s.nope_dim,
                            s.kv_rank)
        o_lat = rt.ws.get("la_olat", (n, H * s.kv_rank), rt.dtype)
        self.attend(qx, o_lat, ctx, layer, table)
        o = rt.ws.get("la_o", (n, H * s.value_dim), rt.dtype)
        if gate is None:
            ops.per_head_linear(o_lat, H * s.kv_rank, s.kv_rank, self.w_uv.view(H, s.value_dim, s.kv_rank), o, H * s.value_dim,
                                s.value_dim, n, H, s.kv_rank, s.value_dim)
        else:
            o32 = rt.ws.get("la_o32", (n, H * s.value_dim), torch.float32)
            ops.per_head_linear(o_lat, H * s.kv_rank, s.kv_rank, self.w_uv.view(H, s.value_dim, s.kv_rank), o32, H * s.value_dim,
                                s.value_dim, n, H, s.kv_rank, s.value_dim)
            ops.head_scalar_gate(o32, gate, o, H, s.value_dim)
        y = rt.ws.get("mixer_out", (n, s.hidden), torch.float32)
        linear(rt, o, self.w_o, y)
        return y


register("mixer", "latent_attention", LatentAttention)
