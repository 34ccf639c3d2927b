"""Several mixers side by side on the same input."""
from __future__ import annotations

import dataclasses

import torch

from ..cache import StateSpec
from ..csrc import ops
from ..errors import Unsupported
from .base import Part, build, register


class ParallelMixer(Part):
    """out = sum_i scales[i] * branch_i(h), added in the order of the branches.  At most one branch may keep keys and
    values in the paged cache (the layer's pages are its own); the branches' states of fixed size lie one behind the
    other in the layer's state row, each branch seeing its own part."""

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        if not 1 <= len(spec.branches) <= 4 or len(spec.scales) != len(spec.branches):
            raise Unsupported("parallel_sum.branches", "one to four branches with a scale each")
        self.branches = [build("mixer", b, rt) for b in spec.branches]
        self.graph_safe = all(getattr(b, "graph_safe", False) for b in self.branches)
        with_kv = [b for b in self.branches if b.kv_layout() is not None]
        if len(with_kv) > 1:
            raise Unsupported("parallel_sum.branches", "more than one branch with cached keys and values in one layer")
        self._kv_branch = with_kv[0] if with_kv else None
        self._ranges, at = [], 0
        for b in self.branches:
            st = b.state_spec()
            if st is None:
                self._ranges.append(None)
                continue
            if st.dtype != torch.float32 or len(st.shape) != 1:
                raise Unsupported("parallel_sum.branches", "a branch whose state is not one row of 32-bit floats")
            self._ranges.append((at, at + st.shape[0]))
            at += st.shape[0]
        self._state_words = at
        self._views: dict = {}

    def children(self):
        return list(self.branches)

    def kv_layout(self):
        return self._kv_branch.kv_layout() if self._kv_branch is not None else None

    def state_spec(self):
        return StateSpec((self._state_words,), torch.float32) if self._state_words else None

    def _layer_for(self, i, layer):
        """What branch i sees of the layer's cache: the pages if it is the branch that has some, and its part of the state."""
        key = (i, id(layer))
        seen = self._views.get(key)
        if seen is not None and seen[0] is layer:
            return seen[1]
        rng = self._ranges[i]
        state = layer.state[:, rng[0]:rng[1]] if rng is not None else None
        if self.branches[i] is self._kv_branch:
            view = dataclasses.replace(layer, state=state)
        else:
            view = dataclasses.replace(layer, k=None, v=None, group=None, writes=False, state=state)
        self._views[key] = (layer, view)
        return view

    def forward(self, h, ctx, layer):
        rt = self.rt
        out = rt.ws.get("parallel_out", (h.shape[0], self.spec.hidden), torch.float32)
        for i, (branch, scale) in enumerate(zip(self.branches, self.spec.scales)):
            y = branch.forward(h, ctx, self._layer_for(i, layer))
            if i == 0:
                ops.weighted_sum(out, [y], [scale])
            else:
                ops.weighted_sum(out, [out, y], [1.0, scale])
        return out


register("mixer", "parallel_sum", ParallelMixer)
