"""Sebevik configurations drawn at random (sizes, head counts, order of the layers, windows, constants, seeds), each run
whole, as a prompt followed by single tokens and as one unequal batch, in both dtypes, against the plain restatement."""
import json

import numpy as np
import pytest
import torch

import plain_sebevik as plain
from gpu_util import run_steps, steps_batches, steps_tail, steps_whole
from test_gpu_sebevik import BOUND, Rec

from esp_b200.engine import Engine
from esp_b200.weights import write_safetensors

pytestmark = pytest.mark.gpu


def draw(rng):
    pick = lambda *xs: xs[int(rng.integers(0, len(xs)))]
    width = pick(64, 72, 100, 128, 160, 256)
    layers = []
    blend = None                        # (key heads, value size) that blending layers share
    for _ in range(int(rng.integers(2, 7))):
        kind = pick("latent_attention", "attention", "attention", "mamba1")
        if kind == "latent_attention":
            mixer = {"heads": pick(1, 2, 3, 4, 6, 8), "dim": pick(8, 16, 24, 32, 64), "vdim": pick(8, 16, 24, 40, 64),
                     "kv_rank": pick(8, 20, 32, 48, 64, 96, 128), "scale": float(rng.uniform(0.05, 0.3))}
        elif kind == "attention":
            heads = pick(1, 2, 3, 4, 6, 8)
            dim = pick(8, 16, 20, 24, 32, 64, 64, 128)
            mixer = {"heads": heads, "kv_heads": pick(*[g for g in range(1, heads + 1) if heads % g == 0]), "dim": dim,
                     "vdim": pick(dim, dim, 8, 16, 40, 64, 72), "scale": float(rng.uniform(0.05, 0.4))}
            if rng.integers(0, 5) > 0:
                mixer["rot"] = {"dims": 2 * int(rng.integers(1, dim // 2 + 1)), "base": pick(50.0, 1000.0, 10000.0, 500000.0)}
            if rng.integers(0, 6) > 0:
                mixer["mask"] = {"size": pick(1, 3, 17, 41, 63, 64, 65, 100, 128, 500)}
            if rng.integers(0, 2):
                if blend is None:
                    blend = (mixer["kv_heads"], mixer["vdim"])
                if heads % blend[0] == 0:
                    mixer["kv_heads"], mixer["vdim"] = blend
                    mixer["v_mix"] = True
        else:
            mixer = {"inner": pick(24, 52, 64, 96, 128, 200), "state": pick(1, 4, 8, 16, 16, 24, 32, 64), "dt_rank": pick(1, 3, 4, 8, 12, 16),
                     "conv": pick(1, 2, 3, 4, 4, 5)}
        which = int(rng.integers(0, 6))
        if which == 0:
            mlp = None
        elif which < 3:
            mlp = {"kind": "dense", "ff": pick(16, 40, 64, 136)}
        else:
            count = pick(1, 1, 2, 3, 4)
            per = pick(1, 2, 3, 4, 5)
            total = count * per
            identity = int(rng.integers(0, total))
            keep = int(rng.integers(1, count + 1))
            router = {"experts": total - identity, "identity": identity, "top": int(rng.integers(1, min(keep * per, 4) + 1))}
            if count > 1 or rng.integers(0, 2):
                router["groups"] = {"count": count, "keep": keep}
            mlp = {"kind": "moe", "router": router, "expert": {"ff": pick(8, 16, 24, 32, 64)}}
            if rng.integers(0, 3):
                mlp["shared"] = {"ff": pick(8, 16, 48)}
        layers.append({"type": kind, "mixer": mixer, "mlp": mlp})
    return {"architecture": "Sebevik", "vocab": pick(97, 256, 301, 513), "width": width, "norm": {"eps": pick(1e-6, 1e-5)},
            "layers": layers}


LENGTHS = (1, 70, 133)


def relative_error(got, ref):
    d = got - ref
    d = d - d.mean(1, keepdims=True)
    return np.sqrt((d ** 2).mean(1)) / np.sqrt((ref ** 2).mean())


@pytest.mark.parametrize("seed", list(range(10)))
def test_random_configuration(tmp_path, seed):
    rng = np.random.default_rng(3000 + seed)
    lengths = LENGTHS
    raw = draw(rng)
    stored = plain.random_weights(raw, 50 + seed)
    reqs = {f"r{i}": [int(t) for t in rng.integers(0, raw["vocab"], n)] for i, n in enumerate(lengths)}
    (tmp_path / "config.json").write_text(json.dumps(raw))
    write_safetensors(tmp_path / "model.safetensors", stored)
    ids = list(reqs)
    for dtype in ("float32", "bfloat16"):
        eng = Engine.from_folder(tmp_path, dtype=dtype, max_tokens=1024)
        eng.rt.record_routing = True
        for what, steps in (("whole", steps_whole(reqs)), ("prompt + single tokens", steps_tail(reqs, tail=40)),
                            ("one batch", steps_batches(reqs, [ids], {rid: max(1, len(t) - 25) for rid, t in reqs.items()}))):
            rec = Rec(raw["vocab"])
            run_steps(eng, steps, rec)
            for rid, toks in reqs.items():
                forced = {layer: torch.from_numpy(chosen.astype(np.int64)) for layer, chosen in rec.forced(rid, len(toks)).items()}
                ref = plain.forward(raw, stored, toks, forced_routing=forced or None).numpy()
                err = relative_error(rec.logits_of(rid, list(range(len(toks)))), ref)
                assert err.max() <= BOUND[dtype], (f"seed {seed}, {dtype}, {what}, request {rid}: position {int(err.argmax())} "
                                                   f"is off by {err.max():.3e}; configuration {json.dumps(raw)}")
                if dtype == "float32" and forced:
                    # in 32-bit the engine's choices are the restatement's own, but for scores within rounding of each other
                    own = plain.forward(raw, stored, toks).numpy()
                    assert relative_error(rec.logits_of(rid, list(range(len(toks)))), own).max() <= 1e-2
        del eng
