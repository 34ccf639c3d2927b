"""Configuration of the Migosun decoder: a scaled token embedding; a stack of pre-norm layers over several copies
of the residual stream (hyper-connections: every sublayer reads a weighted sum of the copies and writes back
through a small mixing matrix), each layer with one of two token mixers and an optional feed-forward; the copies
are summed behind the last layer; the head is the embedding table.

The mixers: ``parallel`` runs two mixers on the same input and adds their results with a weight each: on the left
softmax attention with norms over the whole query and key projections, rotation of the first channels of every
head, a mask of chunks counted from the sequence's start and a learned sink per head; on the right the delta rule
with a decay per key channel behind short convolutions.  ``gla`` is gated linear attention with a decay per key
channel.  The feed-forward is a gated unit with clamped branches.

config.json names every size and every constant that may differ between models; this class reads it, refuses what
the parts cannot run, and turns it into the architecture-neutral plan.  Keys:

    architecture: "Migosun";  vocab, width;  norm.eps;  embedding.scale;  streams (absent: one plain residual stream)
    layers: [{type: "parallel" | "gla", mixer: {...}, mlp: {kind: "dense", ff, limit} | null}, ...]
    mixer (parallel): left {heads, kv_heads, dim, vdim, scale, rot {dims, base}, mask {size}},
                      right {heads, kv_heads, dim, vdim, conv}, left_scale, right_scale
    mixer (gla):      heads, dim, vdim, tau

Tensor names: ``embed``, ``final.norm``, and per layer i ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.hc1.*``,
``l<i>.hc2.*``, ``l<i>.mix.*``, ``l<i>.mlp.*``.  The inner widths of the low-rank projections (decay, output gate)
are not in config.json; they are the stored tensors' (``bind_shapes``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

from ..errors import InvalidConfig, Unsupported
from .plan import (BlockSpec, ChannelDecayAttentionSpec, ClampedGluFfnSpec, GatedDeltaSpec, HyperConnectionBlockSpec,
                   ModelPlan, NormSpec, ParallelMixerSpec, ScaledRopeSpec, ScheduleEntry, WideNormAttentionSpec)
from .registry import register_architecture
from .vumedra import _int, _num, _obj

ARCHITECTURE = "Migosun"
MODEL_TYPE = "migosun"
MIXERS = ("parallel", "gla")
# The design names no longest position; positions are exact as 32-bit floats up to 2^24, and the cache book wants a bound.
POSITION_BOUND = 1 << 20
# Fixed by the design: the feed-forward's sigmoid slope and the shift of its linear branch.
GLU_ALPHA = 1.702
GLU_UP_SHIFT = 1.0
DEFAULT_RANK = 32        # inner width of the low-rank projections of a configuration that comes without tensors


@dataclass
class MigosunConfig:
    vocab: int
    width: int
    eps: float
    embed_scale: float
    streams: Optional[int]
    layers: list = field(default_factory=list)       # the config's entries, checked
    # (layer, tensor) -> inner width of a low-rank projection; filled from a folder's tensors, or given as "ranks"
    ranks: dict = field(default_factory=dict)

    @classmethod
    def from_dict(cls, raw: dict) -> "MigosunConfig":
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers or not all(isinstance(l, dict) for l in layers):
            raise InvalidConfig("layers must be a non-empty list of objects")
        emb = raw.get("embedding")
        streams = raw.get("streams")
        if streams is not None:
            streams = _int(raw, "streams", "config")
        ranks = {}
        for key, v in (raw.get("ranks") or {}).items():
            layer, _, name = key.partition(":")
            ranks[(int(layer), name)] = int(v)
        cfg = cls(vocab=_int(raw, "vocab", "config"), width=_int(raw, "width", "config"),
                  eps=_num(_obj(raw, "norm", "config"), "eps", "norm"),
                  embed_scale=_num(emb, "scale", "embedding") if isinstance(emb, dict) and "scale" in emb else 1.0,
                  streams=streams, layers=[dict(l) for l in layers], ranks=ranks)
        cfg.validate()
        return cfg

    # ---- checks -----------------------------------------------------------------
    def validate(self) -> None:
        if not self.eps > 0:
            raise InvalidConfig("norm.eps must be positive")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            kind = layer.get("type")
            if kind not in MIXERS:
                raise Unsupported("layers.type", f"{kind!r} in {where}; this design has {', '.join(MIXERS)}")
            mix = _obj(layer, "mixer", where)
            w = where + ".mixer"
            if kind == "parallel":
                left, right = _obj(mix, "left", w), _obj(mix, "right", w)
                _num(mix, "left_scale", w)
                _num(mix, "right_scale", w)
                wl = w + ".left"
                for key in ("heads", "kv_heads", "dim", "vdim"):
                    _int(left, key, wl)
                if left["heads"] % left["kv_heads"]:
                    raise InvalidConfig(f"{wl}.kv_heads must divide heads")
                _num(left, "scale", wl)
                if left.get("rot") is not None:
                    rot = _obj(left, "rot", wl)
                    if _int(rot, "dims", wl + ".rot", 2) % 2 or rot["dims"] > left["dim"]:
                        raise InvalidConfig(f"{wl}.rot.dims must be even and at most dim")
                    if not _num(rot, "base", wl + ".rot") > 0:
                        raise InvalidConfig(f"{wl}.rot.base must be positive")
                if left.get("mask") is not None:
                    _int(_obj(left, "mask", wl), "size", wl + ".mask")
                wr = w + ".right"
                for key in ("heads", "kv_heads", "dim", "vdim", "conv"):
                    _int(right, key, wr)
                if right["heads"] % right["kv_heads"]:
                    raise InvalidConfig(f"{wr}.kv_heads must divide heads")
            else:
                for key in ("heads", "dim", "vdim"):
                    _int(mix, key, w)
                if not _num(mix, "tau", w) > 0:
                    raise InvalidConfig(f"{w}.tau must be positive")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                raise Unsupported("layers.mlp.kind", f"{mlp!r} in {where}; this design has dense feed-forwards")
            _int(mlp, "ff", where + ".mlp")
            if not _num(mlp, "limit", where + ".mlp") > 0:
                raise InvalidConfig(f"{where}.mlp.limit must be positive")

    # ---- sizes that only the tensors give ------------------------------------------
    def _rank_tensors(self, i: int, layer: dict) -> list:
        if layer["type"] == "parallel":
            return [f"l{i}.mix.right.a1", f"l{i}.mix.right.g1"]
        return [f"l{i}.mix.a1"]

    def bind_shapes(self, shapes: dict) -> None:
        """``shapes``: tensor name -> shape of a model folder's tensors."""
        for i, layer in enumerate(self.layers):
            for name in self._rank_tensors(i, layer):
                if name in shapes and len(shapes[name]) == 2:
                    self.ranks[(i, name.rsplit(".", 1)[1])] = int(shapes[name][0])

    def _rank(self, i: int, name: str) -> int:
        return self.ranks.get((i, name), DEFAULT_RANK)

    # ---- writing ------------------------------------------------------------------
    def to_dict(self) -> dict:
        d = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
             "embedding": {"scale": self.embed_scale}, "layers": self.layers}
        if self.streams is not None:
            d["streams"] = self.streams
        if self.ranks:
            d["ranks"] = {f"{i}:{name}": v for (i, name), v in sorted(self.ranks.items())}
        return d

    # ---- the plan -------------------------------------------------------------------
    def _mixer_spec(self, i: int, layer: dict):
        mix, p = layer["mixer"], f"l{i}.mix."
        if layer["type"] == "gla":
            return ChannelDecayAttentionSpec(self.width, mix["heads"], mix["dim"], mix["vdim"], float(mix["tau"]),
                                             self._rank(i, "a1"), self.eps, p)
        a, b = mix["left"], mix["right"]
        rot, mask = a.get("rot"), a.get("mask")
        left = WideNormAttentionSpec(self.width, a["heads"], a["kv_heads"], a["dim"], a["vdim"], float(a["scale"]), self.eps,
                                     True, None, mask["size"] if mask else None,
                                     ScaledRopeSpec(rot["dims"], float(rot["base"])) if rot else None, p + "left.")
        right = GatedDeltaSpec(self.width, b["heads"], b["kv_heads"], b["dim"], b["vdim"], b["conv"], self._rank(i, "a1"),
                               self._rank(i, "g1"), self.eps, p + "right.")
        return ParallelMixerSpec(self.width, (left, right), (float(mix["left_scale"]), float(mix["right_scale"])))

    def plan(self) -> ModelPlan:
        norm = lambda name: NormSpec("rmsnorm", self.width, self.eps, name)
        blocks, schedule = [], []
        depth = len(self.layers)
        for i, layer in enumerate(self.layers):
            mlp = layer.get("mlp")
            ffn = ClampedGluFfnSpec(self.width, mlp["ff"], float(mlp["limit"]), f"l{i}.mlp.", GLU_ALPHA, GLU_UP_SHIFT) \
                if mlp is not None else None
            mixer = self._mixer_spec(i, layer)
            if self.streams is None:
                if ffn is None:
                    raise Unsupported("layers.mlp", f"null in layers[{i}]; a layer without hyper-connections needs a feed-forward")
                blocks.append(BlockSpec(mixer, ffn, norm(f"l{i}.norm1"), norm(f"l{i}.norm2")))
            else:
                blocks.append(HyperConnectionBlockSpec(mixer, ffn, norm(f"l{i}.norm1"), norm(f"l{i}.norm2") if ffn is not None else None,
                                                       self.streams, f"l{i}.hc1.", f"l{i}.hc2." if ffn is not None else None,
                                                       i, depth, self.width))
            schedule.append(ScheduleEntry(i))
        return ModelPlan(architecture=ARCHITECTURE, hidden=self.width, vocab=self.vocab, max_positions=POSITION_BOUND,
                         blocks=blocks, schedule=schedule, final_norm=norm("final.norm"), embed_weight="embed",
                         head_weight=None, embed_scale=self.embed_scale,
                         # a layer without feed-forward has no second norm and no second set of connection weights; a
                         # checkpoint that stores them all the same is read without them
                         tolerated_suffixes=(".norm2", ".hc2.in", ".hc2.out", ".hc2.mix"))


register_architecture(ARCHITECTURE, MODEL_TYPE, MigosunConfig)
