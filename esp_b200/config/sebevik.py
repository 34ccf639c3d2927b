"""Configuration of the Sebevik decoder: a pre-norm stack whose norm weights are offsets from one; each layer has
one of three token mixers (attention through a cached latent without positions and with a sigmoid gate per head;
grouped attention with biases, neighbour-pair rotation, unit heads, a sliding window, a learned sink per head and values
blended with the first such layer's; the selective scan behind a short convolution) and an optional feed-forward (dense
with a squared ReLU, or routed gated experts with a corrected, group-limited choice, router outputs that pass the
input through, and a gated shared expert); the head is the token table.

config.json names every size and every constant that may differ between models; this class reads it, refuses what
the parts cannot run, and turns it into the architecture-neutral plan.  Keys:

    architecture: "Sebevik";  vocab, width;  norm.eps
    layers: [{type: "latent_attention" | "attention" | "mamba1", mixer: {...}, mlp: {...} | null}, ...]
    mixer (latent_attention): heads, dim, vdim, kv_rank, scale
    mixer (attention):        heads, kv_heads, dim, vdim, scale, rot {dims, base}, mask {size}, v_mix
    mixer (mamba1):           inner, state, dt_rank, conv
    mlp: {kind: "dense", ff} | {kind: "moe", router {experts, top, identity, groups {count, keep}}, expert {ff}, shared {ff}}

Tensor names: ``embed``, ``final.norm``, and per layer i ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

from ..errors import InvalidConfig, Unsupported
from .plan import (BlockSpec, LatentAttentionSpec, ModelPlan, MoeFfnSpec, MoeNames, NeighbourRopeSpec, NormSpec, Relu2FfnSpec,
                   ScheduleEntry, SelectiveScanSpec, SwiGluNames, UnitNormAttentionSpec)
from .registry import register_architecture

ARCHITECTURE = "Sebevik"
MODEL_TYPE = "sebevik"
MIXERS = ("latent_attention", "attention", "mamba1")
# The design names no longest position; positions are exact as 32-bit floats up to 2^24, and the cache book wants a bound.
POSITION_BOUND = 1 << 20


def _int(d, key, where, minimum=1):
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v < minimum:
        raise InvalidConfig(f"{where}.{key} must be an integer >= {minimum}, got {v!r}")
    return v


def _num(d, key, where):
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v):
        raise InvalidConfig(f"{where}.{key} must be a finite number, got {v!r}")
    return float(v)


def _obj(d, key, where):
    v = d.get(key)
    if not isinstance(v, dict):
        raise InvalidConfig(f"{where}.{key} must be an object")
    return v


@dataclass
class SebevikConfig:
    vocab: int
    width: int
    eps: float
    layers: list = field(default_factory=list)       # the config's entries, checked

    @classmethod
    def from_dict(cls, raw: dict) -> "SebevikConfig":
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers or not all(isinstance(l, dict) for l in layers):
            raise InvalidConfig("layers must be a non-empty list of objects")
        layers = [dict(l, mixer=dict(l["mixer"])) if isinstance(l.get("mixer"), dict) else dict(l) for l in layers]
        for layer in layers:
            mix = layer.get("mixer")
            if isinstance(mix, dict) and layer.get("type") in ("latent_attention", "attention"):
                if "vdim" not in mix and "dim" in mix:
                    mix["vdim"] = mix["dim"]               # value channels default to the key channels
                if layer["type"] == "attention" and "kv_heads" not in mix and "heads" in mix:
                    mix["kv_heads"] = mix["heads"]
        cfg = cls(vocab=_int(raw, "vocab", "config"), width=_int(raw, "width", "config"),
                  eps=_num(_obj(raw, "norm", "config"), "eps", "norm"), layers=layers)
        cfg.validate()
        return cfg

    # ---- checks -----------------------------------------------------------------
    def validate(self) -> None:
        if not self.eps > 0:
            raise InvalidConfig("norm.eps must be positive")
        blend_width = None
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            kind = layer.get("type")
            if kind not in MIXERS:
                raise Unsupported("layers.type", f"{kind!r} in {where}; this design has {', '.join(MIXERS)}")
            mix = _obj(layer, "mixer", where)
            w = where + ".mixer"
            if kind == "latent_attention":
                for key in ("heads", "dim", "vdim", "kv_rank"):
                    _int(mix, key, w)
                _num(mix, "scale", w)
            elif kind == "attention":
                for key in ("heads", "kv_heads", "dim", "vdim"):
                    _int(mix, key, w)
                if mix["heads"] % mix["kv_heads"]:
                    raise InvalidConfig(f"{w}.kv_heads must divide heads")
                _num(mix, "scale", w)
                if mix.get("rot") is not None:
                    rot = _obj(mix, "rot", w)
                    if _int(rot, "dims", w + ".rot", 2) % 2 or rot["dims"] > mix["dim"]:
                        raise InvalidConfig(f"{w}.rot.dims must be an even number of at most dim channels")
                    if not _num(rot, "base", w + ".rot") > 0:
                        raise InvalidConfig(f"{w}.rot.base must be positive")
                if mix.get("mask") is not None:
                    _int(_obj(mix, "mask", w), "size", w + ".mask")
                if mix.get("v_mix") not in (None, True, False):
                    raise InvalidConfig(f"{w}.v_mix must be true or false")
                if mix.get("v_mix"):
                    if blend_width not in (None, (mix["kv_heads"], mix["vdim"])):
                        raise InvalidConfig(f"{w}: layers that blend their values must agree in kv_heads and vdim")
                    blend_width = (mix["kv_heads"], mix["vdim"])
            else:
                for key in ("inner", "state", "dt_rank", "conv"):
                    _int(mix, key, w)
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
                raise Unsupported("layers.mlp.kind", f"{mlp!r} in {where}; this design has dense and moe feed-forwards")
            w = where + ".mlp"
            if mlp["kind"] == "dense":
                _int(mlp, "ff", w)
                continue
            router = _obj(mlp, "router", w)
            experts, top = _int(router, "experts", w + ".router"), _int(router, "top", w + ".router")
            identity = _int(router, "identity", w + ".router", 0) if router.get("identity") is not None else 0
            total = experts + identity
            if top > total:
                raise InvalidConfig(f"{w}.router.top exceeds the number of router outputs")
            if router.get("groups") is not None:
                groups = _obj(router, "groups", w + ".router")
                count, keep = _int(groups, "count", w + ".router.groups"), _int(groups, "keep", w + ".router.groups")
                if total % count or keep > count:
                    raise InvalidConfig(f"{w}.router.groups: count must divide the {total} router outputs and keep <= count")
                if keep * (total // count) < top:
                    raise InvalidConfig(f"{w}.router.groups: the kept groups hold fewer experts than top")
            _int(_obj(mlp, "expert", w), "ff", w + ".expert")
            if mlp.get("shared") is not None:
                _int(_obj(mlp, "shared", w), "ff", w + ".shared")

    # ---- writing ------------------------------------------------------------------
    def to_dict(self) -> dict:
        return {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
                "layers": self.layers}

    # ---- the plan -------------------------------------------------------------------
    def _mixer_spec(self, i: int, layer: dict, first_blend: bool):
        mix, p = layer["mixer"], f"l{i}.mix."
        if layer["type"] == "latent_attention":
            return LatentAttentionSpec(hidden=self.width, num_heads=mix["heads"], nope_dim=mix["dim"], rot_dim=0,
                                       value_dim=mix["vdim"], q_rank=None, kv_rank=mix["kv_rank"], scale=float(mix["scale"]),
                                       window=None, keep_window=None, eps=self.eps, position=None, own_kv=True, prefix=p,
                                       head_gate=True)
        if layer["type"] == "attention":
            rot, mask = mix.get("rot"), mix.get("mask")
            blend = None
            if mix.get("v_mix"):
                blend = "first" if first_blend else "blend"
            return UnitNormAttentionSpec(hidden=self.width, num_heads=mix["heads"], num_kv_heads=mix["kv_heads"],
                                         key_dim=mix["dim"], value_dim=mix["vdim"], scale=float(mix["scale"]), eps=self.eps,
                                         qkv_bias=True, unit_heads=True, learned_sink=True,
                                         window=int(mask["size"]) if mask else None,
                                         position=NeighbourRopeSpec(int(rot["dims"]), float(rot["base"])) if rot else None,
                                         value_blend=blend, prefix=p)
        return SelectiveScanSpec(self.width, mix["inner"], mix["state"], mix["dt_rank"], mix["conv"], p)

    def _ffn_spec(self, i: int, mlp):
        p = f"l{i}.mlp."
        if mlp["kind"] == "dense":
            return Relu2FfnSpec(self.width, mlp["ff"], p)
        router, shared, groups = mlp["router"], mlp.get("shared"), mlp["router"].get("groups")
        names = MoeNames(router="router", shared_gate="shared.sg", shared="shared.", expert="e{e}.",
                         mlp=SwiGluNames("gate", "up", "down"))
        return MoeFfnSpec(hidden=self.width, num_experts=router["experts"], top_k=router["top"], norm_topk=False,
                          expert_intermediate=mlp["expert"]["ff"], shared_intermediate=shared["ff"] if shared else None,
                          prefix=p, names=names, identity_experts=router.get("identity") or 0, correction="correction",
                          groups=groups["count"] if groups else 0, keep_groups=groups["keep"] if groups else 0)

    def plan(self) -> ModelPlan:
        norm = lambda name: NormSpec("rmsnorm_offset", self.width, self.eps, name)
        blocks, schedule = [], []
        seen_blend = False
        for i, layer in enumerate(self.layers):
            mlp = layer.get("mlp")
            ffn = self._ffn_spec(i, mlp) if mlp is not None else None
            blends = layer["type"] == "attention" and bool(layer["mixer"].get("v_mix"))
            blocks.append(BlockSpec(self._mixer_spec(i, layer, blends and not seen_blend), ffn, norm(f"l{i}.norm1"),
                                    norm(f"l{i}.norm2") if ffn is not None else None))
            seen_blend = seen_blend or blends
            schedule.append(ScheduleEntry(i))
        return ModelPlan(architecture=ARCHITECTURE, hidden=self.width, vocab=self.vocab, max_positions=POSITION_BOUND,
                         blocks=blocks, schedule=schedule, final_norm=norm("final.norm"), embed_weight="embed",
                         head_weight=None,
                         # a layer without feed-forward has no second norm and an attention layer that blends nothing
                         # has no blend weight; a checkpoint that stores them all the same is read without them
                         tolerated_suffixes=(".norm2", ".mix.vmix"))


register_architecture(ARCHITECTURE, MODEL_TYPE, SebevikConfig)
