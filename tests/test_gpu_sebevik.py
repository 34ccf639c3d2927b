"""The Sebevik design in the engine against its plain restatement: each mechanism alone in a model of one layer, whole
prompts, prompts followed by single tokens, portions of many sizes, unequal batches, caches so small that slots, pages
and state rows are used again, long decoding past window edges and page borders, greedy generation through the entry
point, and the replay program."""
import functools
import json
import os
import re
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_sebevik as plain
from gpu_util import Recorder, run_steps, steps_batches, steps_tail, steps_whole
from tiny import repo_root
from sebevik_cases import case

from esp_b200.engine import Engine, StepEntry
from esp_b200.weights import write_safetensors

pytestmark = pytest.mark.gpu

# root mean square of (engine - plain) over a row of logits, mean taken off, over the root mean square of the
# request's plain logits.  float32: only the order of sums differs.  bfloat16: activations and cached rows are
# rounded to 8 bits a few times per layer; the recurrence itself stays 32-bit.
BOUND = {"float32": 2e-5, "bfloat16": 4e-2}

# one layer each: the mechanisms alone (sizes unlike the three cases')
SINGLE = {
    "latent": {"type": "latent_attention", "mixer": {"heads": 2, "dim": 16, "vdim": 24, "kv_rank": 32, "scale": 0.3}, "mlp": None},
    "window": {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 32, "vdim": 32, "scale": 0.17, "v_mix": True,
                                              "rot": {"dims": 12, "base": 40.0}, "mask": {"size": 9}}, "mlp": None},
    "scan": {"type": "mamba1", "mixer": {"inner": 48, "state": 12, "dt_rank": 3, "conv": 4}, "mlp": None},
    "dense": {"type": "mamba1", "mixer": {"inner": 8, "state": 2, "dt_rank": 2, "conv": 2}, "mlp": {"kind": "dense", "ff": 56}},
    "experts": {"type": "mamba1", "mixer": {"inner": 8, "state": 2, "dt_rank": 2, "conv": 2},
                "mlp": {"kind": "moe", "router": {"experts": 5, "top": 3, "identity": 3, "groups": {"count": 4, "keep": 2}},
                        "expert": {"ff": 24}, "shared": {"ff": 40}}},
}


def single_config(which):
    return {"architecture": "Sebevik", "vocab": 83, "width": 72, "norm": {"eps": 1e-5}, "layers": [dict(SINGLE[which])]}


@functools.lru_cache(maxsize=None)
def model(name, seed=7):
    raw = single_config(name[1:]) if name.startswith("+") else case(name)
    return raw, plain.random_weights(raw, seed)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name in ["A", "B", "C"] + ["+" + k for k in SINGLE]:
        raw, w = model(name)
        d = tmp_path_factory.mktemp(f"sebevik_{name.strip('+')}")
        (d / "config.json").write_text(json.dumps(raw))
        write_safetensors(d / "model.safetensors", w)
        out[name] = d
    return out


_engines = {}


def engine_for(folder, dtype, max_tokens=2048, record=None, **kw):
    """bfloat16 engines note their expert choices (the restatement is then given them, so that no bound has to absorb
    a flipped expert); float32 engines do not, so that their decode steps replay captured graphs."""
    record = (dtype == "bfloat16") if record is None else record
    key = (str(folder), dtype, max_tokens, record, tuple(sorted(kw.items())))
    if key not in _engines:
        eng = Engine.from_folder(folder, dtype=dtype, max_tokens=max_tokens, **kw)
        eng.rt.record_routing = record
        _engines[key] = eng
    return _engines[key]


class Rec(Recorder):
    """The shared recorder, reading the layer out of this design's tensor prefixes."""

    def take(self, entries, ids_of, logits, aux):
        routing = aux.pop("routing", []) if aux else []
        super().take(entries, ids_of, logits, {})
        for prefix, row0, ids, _w, _p in routing:
            layer = int(re.match(r"l(\d+)\.mlp\.", prefix).group(1))
            ids = ids.cpu().numpy()
            start = 0
            for rid, first, n, _want in entries:
                lo, hi = max(start, row0), min(start + n, row0 + ids.shape[0])
                for r in range(lo, hi):
                    self.routing.setdefault(rid, {}).setdefault(layer, {})[first + (r - start)] = ids[r - row0]
                start += n


def requests_for(name, lengths, seed=3):
    rng = np.random.default_rng(seed)
    vocab = model(name)[0]["vocab"]
    return {f"r{i}": [int(t) for t in rng.integers(0, vocab, n)] for i, n in enumerate(lengths)}


def check(name, dtype, requests, rec, what, positions=None):
    raw, w = model(name)
    for rid, toks in requests.items():
        forced = None
        if dtype == "bfloat16":
            forced = {layer: torch.from_numpy(ids.astype(np.int64)) for layer, ids in rec.forced(rid, len(toks)).items()}
            sparse = [i for i, l in enumerate(raw["layers"]) if l.get("mlp") and l["mlp"]["kind"] == "moe"]
            assert sorted(forced) == sparse
        ref = plain.forward(raw, w, toks, forced_routing=forced).numpy()
        at = list(range(len(toks))) if positions is None else list(positions[rid])
        got = rec.logits_of(rid, at)
        d = got - ref[at]
        d = d - d.mean(1, keepdims=True)
        err = np.sqrt((d ** 2).mean(1)) / np.sqrt((ref ** 2).mean())
        worst = int(np.argmax(err))
        assert err[worst] <= BOUND[dtype], (f"{what}, case {name}, {dtype}, request {rid} ({len(toks)} tokens): position "
                                            f"{at[worst]} is off by {err[worst]:.3e} (bound {BOUND[dtype]:.1e}); first "
                                            f"position over its bound: {at[int(np.argmax(err > BOUND[dtype]))]}")
        if forced:
            # the engine's choices are the restatement's own but for scores within rounding of one another
            for layer, mine in forced.items():
                h_ids = route_of(name, tuple(toks), layer)
                differ = sum(set(a.tolist()) != set(b.tolist()) for a, b in zip(mine, h_ids))
                assert differ <= max(1, len(toks) // 10), (layer, differ)


@functools.lru_cache(maxsize=None)
def route_of(name, toks, layer):
    """The restatement's own expert choices in ``layer`` for the whole sequence."""
    raw, w = model(name)
    seen = {}
    real_route = plain.route

    def spy(h, ww, pre, router):
        out = real_route(h, ww, pre, router)
        seen[pre] = out[0]
        return out

    plain.route = spy
    try:
        plain.forward(raw, w, list(toks))
    finally:
        plain.route = real_route
    return seen[f"l{layer}.mlp."]


def steps_portions(requests, sizes):
    """Each request alone, cut into portions whose sizes cycle through ``sizes``."""
    steps = []
    for rid, toks in requests.items():
        at, i = 0, 0
        while at < len(toks):
            n = min(sizes[i % len(sizes)], len(toks) - at)
            steps.append(([(rid, toks[at:at + n], list(range(n)))], [rid] if at + n == len(toks) else []))
            at += n
            i += 1
    return steps


LENGTHS = {"A": (1, 9, 83, 150), "B": (2, 40, 77, 131), "C": (3, 64, 129, 200)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", list(SINGLE))
def test_each_mechanism_alone(folders, which, dtype):
    """A model of one layer: whole, then cut into a prompt and single tokens, then in portions of two and three."""
    name = "+" + which
    reqs = requests_for(name, (1, 30, 75))
    eng = engine_for(folders[name], dtype)
    for steps, what in ((steps_whole(reqs), "whole"), (steps_tail(reqs, tail=25), "tail"), (steps_portions(reqs, [2, 3]), "portions")):
        rec = Rec(model(name)[0]["vocab"])
        run_steps(eng, steps, rec)
        check(name, dtype, reqs, rec, f"{which} alone, {what}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_prompts(folders, name, dtype):
    reqs = requests_for(name, LENGTHS[name])
    eng = engine_for(folders[name], dtype)
    rec = Rec(model(name)[0]["vocab"])
    run_steps(eng, steps_whole(reqs), rec)
    check(name, dtype, reqs, rec, "whole prompts")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_prefill_then_token_by_token(folders, name, dtype):
    """The last 80 tokens one by one: the windows of 5, 37, 64, 70 and 128 positions pass over decoded tokens, page
    borders lie at 64 and 128, and the first requests are decoded from their second token on."""
    reqs = requests_for(name, LENGTHS[name])
    eng = engine_for(folders[name], dtype)
    rec = Rec(model(name)[0]["vocab"])
    run_steps(eng, steps_tail(reqs, tail=80), rec)
    check(name, dtype, reqs, rec, "prompt, then single tokens")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_portions_of_many_sizes(folders, name, dtype):
    reqs = requests_for(name, LENGTHS[name][1:], seed=5)
    eng = engine_for(folders[name], dtype)
    rec = Rec(model(name)[0]["vocab"])
    run_steps(eng, steps_portions(reqs, [2, 31, 3, 64, 17, 2, 2]), rec)
    check(name, dtype, reqs, rec, "portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_unequal_batches_in_a_cache_that_is_used_again(folders, name, dtype):
    """Two batches, one after the other, in a cache that holds one of them: every slot, page and state row of the
    second batch was used by the first.  A state that is not cleared, or a page table that keeps an old page, shows."""
    lengths = (70, 5, 140, 33, 129, 64, 2, 100)
    reqs = requests_for(name, lengths, seed=9)
    ids = list(reqs)
    batches = [ids[:4], ids[4:]]
    prompt = {rid: max(1, len(reqs[rid]) - 40 + 7 * i) for i, rid in enumerate(ids)}
    prompt = {rid: min(n, len(reqs[rid])) for rid, n in prompt.items()}
    eng = engine_for(folders[name], dtype, max_tokens=7 * 64, max_slots=4)
    rec = Rec(model(name)[0]["vocab"])
    run_steps(eng, steps_batches(reqs, batches, prompt), rec)
    check(name, dtype, reqs, rec, "unequal batches")
    assert eng.cache.book.slots.available == 4
    assert all(g.pool.available == g.pool.n for g in eng.cache.book.groups)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_cuttings_agree_bit_for_bit_in_float32(folders, name):
    """No sum's order depends on how a sequence is cut or what it is batched with; decode steps replay captured graphs."""
    reqs = requests_for(name, (3, 90, 150), seed=13)
    eng = engine_for(folders[name], "float32")
    outs = []
    ids = list(reqs)
    for steps in (steps_whole(reqs), steps_tail(reqs, tail=40), steps_portions(reqs, [2, 5, 64]),
                  steps_batches(reqs, [ids], {rid: max(1, len(t) - 30) for rid, t in reqs.items()})):
        rec = Rec(model(name)[0]["vocab"])
        run_steps(eng, steps, rec)
        outs.append(rec)
    assert eng.graph_replays > 0
    for rid, toks in reqs.items():
        at = list(range(len(toks)))
        first = outs[0].logits_of(rid, at)
        for other in outs[1:]:
            assert np.array_equal(first, other.logits_of(rid, at))


@pytest.mark.parametrize("heads, dim, rank", [(3, 64, 48), (2, 128, 32)])
def test_whole_long_prompts_take_the_unfolded_latent_attention(tmp_path, heads, dim, rank):
    """A step of whole prompts of which one has 600 tokens, in bfloat16 at head sizes 64 and 128: every head's keys and
    values are made from the step's latents and the tensor-memory attention runs over them; the tokens decoded afterwards
    read the latents that the same step cached.  The same requests in portions (the folded form) agree within the bound."""
    from esp_b200.csrc import ops
    raw = {"architecture": "Sebevik", "vocab": 91, "width": 64, "norm": {"eps": 1e-5}, "layers": [
        {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "vdim": dim, "kv_rank": rank, "scale": 0.11},
         "mlp": {"kind": "dense", "ff": 48}},
        {"type": "latent_attention", "mixer": {"heads": 2, "dim": 24, "vdim": 24, "kv_rank": 32, "scale": 0.2}, "mlp": None}]}
    w = plain.random_weights(raw, 11)
    (tmp_path / "config.json").write_text(json.dumps(raw))
    write_safetensors(tmp_path / "model.safetensors", w)
    rng = np.random.default_rng(4)
    reqs = {f"r{i}": [int(t) for t in rng.integers(0, raw["vocab"], n)] for i, n in enumerate((620, 75, 130))}
    eng = Engine.from_folder(tmp_path, dtype="bfloat16", max_tokens=2048)
    # scratch that held values that are no numbers: what lies behind a prompt's end in its last page must not count
    for name in ("la_k_pages", "la_v_pages"):
        eng.rt.ws.get(name, (64, heads, 64, dim), torch.bfloat16).fill_(float("nan"))
    calls = []
    real = ops.heads_to_pages
    ops.heads_to_pages = lambda *a, **k: (calls.append(1), real(*a, **k))[1]
    try:
        ids = list(reqs)
        rec = Recorder(raw["vocab"])
        run_steps(eng, steps_batches(reqs, [ids], {rid: len(t) - 12 for rid, t in reqs.items()}), rec)
        assert len(calls) == 1                  # the first layer, in the step of the prompts; the second one's sizes do not fit
        rec2 = Recorder(raw["vocab"])
        run_steps(eng, steps_portions(reqs, [300, 7, 64]), rec2)
        assert len(calls) == 1
    finally:
        ops.heads_to_pages = real
    for rid, toks in reqs.items():
        ref = plain.forward(raw, w, toks).numpy()
        for r in (rec, rec2):
            d = r.logits_of(rid, list(range(len(toks)))) - ref
            d = d - d.mean(1, keepdims=True)
            err = np.sqrt((d ** 2).mean(1)) / np.sqrt((ref ** 2).mean())
            assert err.max() <= BOUND["bfloat16"], (rid, int(err.argmax()), float(err.max()))


def test_long_decoding_in_a_small_cache(folders):
    """300 single tokens after a prompt of 3 in a cache of 6 pages: the windowed layers give their old pages back and
    get them again, the layer that sees everything keeps its five, the recurrent state carries the rest."""
    name = "A"
    reqs = requests_for(name, (303,), seed=21)
    for dtype in ("float32", "bfloat16"):
        eng = engine_for(folders[name], dtype, max_tokens=6 * 64)
        rec = Rec(model(name)[0]["vocab"])
        run_steps(eng, steps_tail(reqs, tail=300), rec)
        check(name, dtype, reqs, rec, "long decoding")


def test_residual_stream_behind_every_layer(folders):
    for name in ("A", "B"):
        raw, w = model(name)
        toks = requests_for(name, (45,), seed=2)["r0"]
        layers = []
        plain.forward(raw, w, toks, trace=layers)
        eng = engine_for(folders[name], "float32")
        slot = eng.open()
        aux = {"residual_trace": []}
        eng.step([StepEntry(slot, toks, [0])], aux)
        eng.close(slot)
        assert len(aux["residual_trace"]) == len(layers)
        for i, (got, want) in enumerate(zip(aux["residual_trace"], layers)):
            err = float((got.cpu().double() - want).abs().max() / want.abs().max())
            assert err < 1e-5, f"case {name}, layer {i}: {err:.2e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(folders, dtype):
    from esp_b200.provider import DecoderProvider, GenerationRequest
    name = "C"
    raw, w = model(name)
    prompts = list(requests_for(name, (4, 19, 70), seed=31).values())
    prov = DecoderProvider.load(folders[name], dtype=dtype, max_batch=2, max_tokens=1024)
    outs = prov.generate([GenerationRequest(prompt_ids=p, max_tokens=12) for p in prompts])
    for p, out in zip(prompts, outs):
        assert len(out.token_ids) == 12 and out.finish_reason == "length"
        # every token the engine chose is, for the plain restatement given the same prefix, the best token or
        # within rounding of it
        seq = list(p)
        for tok in out.token_ids:
            ref = plain.forward(raw, w, seq)[-1]
            slack = (1e-4 if dtype == "float32" else 0.12) * float(ref.abs().max())
            assert float(ref.max() - ref[tok]) <= slack
            seq.append(tok)


def test_the_command_line_generates(folders):
    env = dict(os.environ)
    proc = subprocess.run([sys.executable, "-m", "esp_b200", "generate", "--model", str(folders["A"]), "--dtype", "float32",
                           "--prompt-ids", "5,17,3", "--prompt-ids", "9 8 7 6 5 4", "--max-tokens", "5"],
                          capture_output=True, text=True, env=env, cwd=str(repo_root()), timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    lines = [json.loads(l) for l in proc.stdout.splitlines() if l.startswith("{")]
    assert [len(l["token_ids"]) for l in lines] == [5, 5]
    raw, w = model("A")
    want, margins = plain.greedy(raw, w, [5, 17, 3], 5)
    if min(margins) > 1e-3:
        assert lines[0]["token_ids"] == want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_program(folders, tmp_path, dtype):
    """Case B: every router output is chosen in its sparse layers, so no choice can flip under bfloat16 rounding and
    every row is held against the restatement's own run."""
    name = "B"
    reqs = requests_for(name, (1, 60, 141), seed=17)
    ids = list(reqs)
    steps = steps_tail(reqs, tail=20) + steps_batches({k + "x": v for k, v in reqs.items()}, [[i + "x" for i in ids]],
                                                      {i + "x": max(1, len(reqs[i]) - 9) for i in ids})
    lines, wanted = [], []
    for i, (entries, end) in enumerate(steps):
        lines.append(json.dumps({"step": i, "entries": [{"id": rid, "tokens": t, "want": wnt} for rid, t, wnt in entries],
                                 "end": end}))
        wanted.append(sum(len(wnt) for _, _, wnt in entries))
    proc = subprocess.run([sys.executable, str(repo_root() / "bin" / "trace_run"), "--model", str(folders[name]), "--dtype",
                           dtype, "--out", str(tmp_path), "--max-tokens", "404"], input="\n".join(lines) + "\n",
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert proc.stdout.split("\n")[:len(steps)] == [f"done {i}" for i in range(len(steps))]
    raw, w = model(name)
    vocab = raw["vocab"]
    got, pos = {}, {}
    for i, (entries, _end) in enumerate(steps):
        data = np.fromfile(tmp_path / f"{i}.f32", dtype="<f4").reshape(wanted[i], vocab)
        r = 0
        for rid, toks, want in entries:
            for wnt in want:
                got.setdefault(rid, {})[pos.get(rid, 0) + wnt] = data[r]
                r += 1
            pos[rid] = pos.get(rid, 0) + len(toks)
    for rid, toks in reqs.items():
        ref = plain.forward(raw, w, toks).numpy()
        for key in (rid, rid + "x"):
            rows = np.stack([got[key][p] for p in range(len(toks))])
            d = rows - ref
            d = d - d.mean(1, keepdims=True)
            err = np.sqrt((d ** 2).mean(1)) / np.sqrt((ref ** 2).mean())
            assert err.max() <= BOUND[dtype], (key, float(err.max()))
