"""Small configurations of the Sebevik design for the tests.  They differ from one another in every size, in the order
of the layers, and in which options are present."""
import copy


def _moe(experts, top, identity, groups, ff, shared):
    router = {"experts": experts, "top": top, "identity": identity}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    out = {"kind": "moe", "router": router, "expert": {"ff": ff}}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


# the selective scan first; windows of 37 positions (no multiple of a page) and of 70 (longer than a page); key and value
# heads of different sizes, six query heads on two key heads; head size 64 with the whole head rotated (the tensor-core
# kernels in bfloat16); a layer without feed-forward; a latent of rank 48 under three heads; three groups of which two
# are kept; a state of 24 entries (two lanes a channel, the second half used); three taps
CASE_A = {
    "architecture": "Sebevik", "vocab": 211, "width": 96, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "mamba1", "mixer": {"inner": 80, "state": 24, "dt_rank": 5, "conv": 3},
         "mlp": {"kind": "dense", "ff": 72}},
        {"type": "attention", "mixer": {"heads": 6, "kv_heads": 2, "dim": 40, "vdim": 24, "scale": 0.21, "v_mix": True,
                                        "rot": {"dims": 16, "base": 500.0}, "mask": {"size": 37}},
         "mlp": _moe(7, 2, 2, (3, 2), 40, 56)},
        {"type": "latent_attention", "mixer": {"heads": 3, "dim": 24, "vdim": 40, "kv_rank": 48, "scale": 0.19}, "mlp": None},
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 64, "vdim": 64, "scale": 0.13,
                                        "rot": {"dims": 64, "base": 10000.0}, "mask": {"size": 70}},
         "mlp": _moe(4, 1, 0, None, 24, None)},
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.3, "v_mix": True,
                                        "rot": {"dims": 2, "base": 77.0}, "mask": {"size": 64}},
         "mlp": {"kind": "dense", "ff": 40}},
    ],
}

# a width that is no multiple of 8; one head; a window of one position (the query alone, beside the sink); a window
# longer than any test sequence; no window at all; no rotation at all; a convolution of one tap (no inputs kept) and one
# of five; head size 128; one state entry; every router output chosen in both sparse layers (no choice can flip under
# rounding); one group (no limit); one expert with weights beside three outputs without; a single blending layer (nothing to blend with)
CASE_B = {
    "architecture": "Sebevik", "vocab": 97, "width": 100, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention", "mixer": {"heads": 1, "kv_heads": 1, "dim": 16, "vdim": 16, "scale": 0.4,
                                        "rot": {"dims": 8, "base": 100.0}, "mask": {"size": 1}},
         "mlp": _moe(1, 4, 3, (1, 1), 36, 20)},
        {"type": "mamba1", "mixer": {"inner": 52, "state": 1, "dt_rank": 1, "conv": 1}, "mlp": None},
        {"type": "latent_attention", "mixer": {"heads": 1, "dim": 72, "vdim": 8, "kv_rank": 20, "scale": 0.1},
         "mlp": _moe(3, 3, 0, None, 28, 12)},
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 1, "dim": 128, "vdim": 128, "scale": 0.08, "v_mix": True,
                                        "rot": {"dims": 2, "base": 10000.0}, "mask": {"size": 1000}},
         "mlp": {"kind": "dense", "ff": 44}},
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 24, "vdim": 8, "scale": 0.25}, "mlp": None},
        {"type": "mamba1", "mixer": {"inner": 24, "state": 40, "dt_rank": 7, "conv": 5}, "mlp": {"kind": "dense", "ff": 32}},
    ],
}

# latent attention first, with a rank of 128 on the tensor-core kernel; a window of exactly one page and one of two
# pages; three blending layers; sixteen router outputs in four groups of which one is kept; a state of 16 entries (one
# lane a channel); two taps; a dt_rank as large as the state
CASE_C = {
    "architecture": "Sebevik", "vocab": 150, "width": 64, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "latent_attention", "mixer": {"heads": 5, "dim": 32, "vdim": 16, "kv_rank": 128, "scale": 0.15},
         "mlp": _moe(13, 4, 3, (4, 1), 32, 48)},
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 128, "vdim": 32, "scale": 0.09, "v_mix": True,
                                        "rot": {"dims": 32, "base": 1000.0}, "mask": {"size": 64}},
         "mlp": {"kind": "dense", "ff": 72}},
        {"type": "mamba1", "mixer": {"inner": 128, "state": 16, "dt_rank": 16, "conv": 2},
         "mlp": _moe(6, 2, 2, (2, 1), 16, None)},
        {"type": "attention", "mixer": {"heads": 3, "kv_heads": 1, "dim": 32, "vdim": 32, "scale": 0.18, "v_mix": True,
                                        "rot": {"dims": 8, "base": 50.0}, "mask": {"size": 128}},
         "mlp": {"kind": "dense", "ff": 48}},
        {"type": "attention", "mixer": {"heads": 1, "kv_heads": 1, "dim": 8, "vdim": 32, "scale": 0.5, "v_mix": True,
                                        "rot": {"dims": 4, "base": 9.0}, "mask": {"size": 5}},
         "mlp": None},
    ],
}

CASES = {"A": CASE_A, "B": CASE_B, "C": CASE_C}


def case(name):
    return copy.deepcopy(CASES[name])
