"""Small configurations of the Migosun design for the tests.  They differ from one another in every size, in the
order of the layers, and in which options are present."""
import copy

# gated linear attention first; chunks of 37 positions (no multiple of a page) and of 70 (longer than a page); key and
# value heads of different sizes, six query heads on two key heads; head size 64 with the whole head rotated (the
# tensor-core kernels in bfloat16); a layer without feed-forward; unequal inner widths of the low-rank projections
CASE_A = {
    "architecture": "Migosun", "vocab": 211, "width": 96, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.7}, "streams": 2,
    "layers": [
        {"type": "gla", "mixer": {"heads": 3, "dim": 24, "vdim": 40, "tau": 4.0}, "mlp": {"kind": "dense", "ff": 80, "limit": 2.0}},
        {"type": "parallel", "mixer": {
            "left": {"heads": 6, "kv_heads": 2, "dim": 40, "vdim": 24, "scale": 0.2, "rot": {"dims": 16, "base": 500.0},
                     "mask": {"size": 37}},
            "right": {"heads": 4, "kv_heads": 2, "dim": 24, "vdim": 40, "conv": 4},
            "left_scale": 0.7, "right_scale": 1.3}, "mlp": None},
        {"type": "parallel", "mixer": {
            "left": {"heads": 2, "kv_heads": 2, "dim": 64, "vdim": 64, "scale": 0.11, "rot": {"dims": 64, "base": 10000.0},
                     "mask": {"size": 70}},
            "right": {"heads": 2, "kv_heads": 1, "dim": 32, "vdim": 16, "conv": 2},
            "left_scale": 1.0, "right_scale": 0.4}, "mlp": {"kind": "dense", "ff": 136, "limit": 0.8}},
        {"type": "gla", "mixer": {"heads": 1, "dim": 64, "vdim": 16, "tau": 1.0}, "mlp": None},
    ],
}
RANKS_A = (12, 20)

# one residual stream under the connection weights; a width that is no multiple of 8; one head; a chunk of one position
# (the query alone, beside the sink); a chunk longer than any test sequence; a convolution of one tap (no inputs kept)
# and one of five; head size 128 with two rotated channels; large heads in the recurrences
CASE_B = {
    "architecture": "Migosun", "vocab": 97, "width": 100, "norm": {"eps": 1e-6}, "embedding": {"scale": 0.6}, "streams": 1,
    "layers": [
        {"type": "parallel", "mixer": {
            "left": {"heads": 1, "kv_heads": 1, "dim": 16, "vdim": 16, "scale": 0.3, "rot": {"dims": 8, "base": 100.0},
                     "mask": {"size": 1}},
            "right": {"heads": 1, "kv_heads": 1, "dim": 128, "vdim": 72, "conv": 1},
            "left_scale": 1.0, "right_scale": 1.0}, "mlp": {"kind": "dense", "ff": 44, "limit": 1.0}},
        {"type": "gla", "mixer": {"heads": 5, "dim": 8, "vdim": 8, "tau": 16.0}, "mlp": None},
        {"type": "parallel", "mixer": {
            "left": {"heads": 4, "kv_heads": 1, "dim": 128, "vdim": 128, "scale": 0.07, "rot": {"dims": 2, "base": 10000.0},
                     "mask": {"size": 1000}},
            "right": {"heads": 3, "kv_heads": 3, "dim": 16, "vdim": 24, "conv": 5},
            "left_scale": 0.5, "right_scale": 2.0}, "mlp": {"kind": "dense", "ff": 32, "limit": 3.0}},
    ],
}
RANKS_B = (5, 5)

# four streams; a chunk of exactly one page and one of two pages; unequal key and value sizes with head size 128 for
# the keys; every layer with a feed-forward
CASE_C = {
    "architecture": "Migosun", "vocab": 150, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0}, "streams": 4,
    "layers": [
        {"type": "parallel", "mixer": {
            "left": {"heads": 2, "kv_heads": 1, "dim": 128, "vdim": 32, "scale": 0.09, "rot": {"dims": 32, "base": 1000.0},
                     "mask": {"size": 64}},
            "right": {"heads": 2, "kv_heads": 2, "dim": 40, "vdim": 8, "conv": 3},
            "left_scale": 1.1, "right_scale": 0.9}, "mlp": {"kind": "dense", "ff": 72, "limit": 1.2}},
        {"type": "parallel", "mixer": {
            "left": {"heads": 3, "kv_heads": 3, "dim": 32, "vdim": 48, "scale": 0.18, "rot": {"dims": 8, "base": 50.0},
                     "mask": {"size": 128}},
            "right": {"heads": 6, "kv_heads": 2, "dim": 8, "vdim": 16, "conv": 2},
            "left_scale": 0.3, "right_scale": 1.5}, "mlp": {"kind": "dense", "ff": 48, "limit": 6.0}},
        {"type": "gla", "mixer": {"heads": 2, "dim": 16, "vdim": 32, "tau": 8.0}, "mlp": {"kind": "dense", "ff": 40, "limit": 0.5}},
    ],
}
RANKS_C = (16, 4)

CASES = {"A": (CASE_A, RANKS_A), "B": (CASE_B, RANKS_B), "C": (CASE_C, RANKS_C)}


def case(name):
    cfg, ranks = CASES[name]
    return copy.deepcopy(cfg), ranks
