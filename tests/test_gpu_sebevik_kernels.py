"""The kernels behind the Sebevik design, each alone against a float64 statement of the same mechanism, at sizes the
model tests do not have, with inputs made so that a fault shows: one key whose score stands out just inside and just
outside the window, at a page's border and at the first positions; a selective scan that keeps a value over hundreds
of tokens, cut into calls in the middle; corrected scores that are all negative; groups that shut out the best expert;
router outputs without an expert behind them."""
import math

import numpy as np
import pytest
import torch

import plain_sebevik as plain

from esp_b200.csrc import ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
PAGE = 64


def dev(t, dtype=None):
    return t.to(DEV, dtype if dtype is not None else t.dtype).contiguous()


def i32(values):
    return torch.tensor(np.asarray(values), dtype=torch.int32, device=DEV)


def status():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


def paged(rows, table, n_pages, dtype):
    """rows [T, G, W] of one sequence -> pool [n_pages, G, PAGE, W] with position p in page table[p // PAGE]."""
    T, G, W = rows.shape
    pool = torch.zeros(n_pages, G, PAGE, W, dtype=dtype)
    for p in range(T):
        pool[table[p // PAGE], :, p % PAGE] = rows[p].to(dtype)
    return pool


# ------------------------------------------------------------------------------------------------ attention
KERNELS = ["plain32", "plain16", "tensor16", "tmem16", "split16"]


def takes(kernel, K, V):
    return kernel in ("plain32", "plain16", "tensor16") or (K == V and K in (64, 128))


def run_attention(kernel, q, k_pool, v_pool, out, table, first, new, H, G, K, V, scale, sink, window):
    st = status()
    args = (q, k_pool, v_pool, out)
    tables = i32([table])
    if kernel == "tensor16":
        firsts = list(range(0, new, 64))
        ops.attn_prefill(*args, i32([0] * len(firsts)), i32(firsts), i32([0, new]), i32([first]), tables, PAGE, H, G, K, window,
                         st, vd=V, scale=scale, sink=sink)
    elif kernel == "tmem16":
        firsts = list(range(0, new, ops.ATTN_TC05_TILE_ROWS))
        ops.attn_prefill_tc05(*args, i32([0] * len(firsts)), i32(firsts), i32([0, new]), i32([first]), tables, PAGE, H, G, K,
                              window, st, scale=scale, sink=sink)
    elif kernel == "split16":
        split = 128
        n_splits = (len(table) * PAGE + split - 1) // split
        part_o = torch.zeros(new, H, n_splits, K, device=DEV)
        part_ml = torch.zeros(new, H, n_splits, 2, device=DEV)
        counters = torch.zeros(ops.ATTN_DECODE_COUNTERS, dtype=torch.int32, device=DEV)
        ops.attn_decode(*args, part_o, part_ml, counters, i32([0] * new), i32(list(range(first, first + new))), tables, PAGE, H, G,
                        K, window, split, n_splits, st, scale=scale, sink=sink)
        assert int(counters.abs().sum().item()) == 0
    else:
        ops.attn_simt(*args, i32([0] * new), i32(list(range(first, first + new))), tables, PAGE, H, G, K, window, st, vd=V,
                      scale=scale, sink=sink)
    assert int(st.item()) == 0


def windowed(q, k, v, scale, first, window, sink):
    """float64: new rows first .. of one sequence against all of k, v; a row sees itself and window - 1 keys before it."""
    Tq, H, _ = q.shape
    T, G = k.shape[0], k.shape[1]
    qp, kp = torch.arange(first, first + Tq)[:, None], torch.arange(T)[None, :]
    visible = (kp <= qp) & (qp - kp < window)
    out = torch.zeros(Tq, H, v.shape[2], dtype=torch.float64)
    for h in range(H):
        s = (q[:, h] @ k[:, h // (H // G)].T) * scale
        s = s.masked_fill(~visible, -math.inf)
        m = torch.maximum(s.max(-1, keepdim=True).values, sink[h])
        e = torch.exp(s - m)
        out[:, h] = (e / (e.sum(-1, keepdim=True) + torch.exp(sink[h] - m))) @ v[:, h // (H // G)]
    return out


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("H, G, K, V, window", [(4, 2, 16, 40, 37), (3, 1, 56, 88, 100), (2, 2, 128, 128, 70), (8, 2, 64, 64, 64),
                                                (2, 1, 64, 64, 129), (2, 1, 24, 24, 1), (2, 2, 64, 64, 400)])
@pytest.mark.parametrize("new", [200, 3])
def test_window_edges_with_a_sink_from_prompt_rows_and_from_single_rows(kernel, H, G, K, V, window, new):
    """460 cached positions in pages handed out in no order; the new tokens are the last 200 (a prompt's portion) or the
    last 3 (decoding).  For probed queries one key gets a large score: the oldest position the window holds (just inside),
    the one before it (just outside: it must not count), the query itself, its predecessor, a page's first position."""
    if not takes(kernel, K, V):
        pytest.skip("this kernel wants keys and values of one size, 64 or 128")
    dtype = torch.float32 if kernel == "plain32" else torch.bfloat16
    g = torch.Generator().manual_seed(window * 7 + new)
    T = 460
    q = torch.randn(new, H, K, generator=g) * 0.3
    k = torch.randn(T, G, K, generator=g) * 0.3
    v = torch.randn(T, G, V, generator=g)
    first = T - new
    used, kinds = set(), set()
    for n, row in enumerate(sorted(set([0, 1, 2, new - 1, new // 2, new // 3, new // 4, new // 5, new - 2, new // 7]))):
        pos = first + row
        key = [pos - window + 1, pos - window, pos, pos - 1, pos - pos % PAGE][n % 5]
        if key < 0 or key > pos or key in used:
            continue
        used.add(key)
        kinds.add(n % 5)
        head = row % H
        direction = torch.randn(K, generator=g)
        direction /= direction.norm()
        k[key, head // (H // G)] = direction * 6
        q[row, head] = direction * 6
    q, k, v = (t.to(dtype).double() for t in (q, k, v))
    sink = torch.randn(H, generator=g).double()
    scale = 0.9
    want = windowed(q, k, v, scale, first, window, sink)
    # the probes tell a window that is one position off: too long sees the key just outside, too short loses the one just inside
    if 1 in kinds:
        assert (windowed(q, k, v, scale, first, window + 1, sink) - want).abs().max() > 0.3
    if 0 in kinds and window > 1:
        assert (windowed(q, k, v, scale, first, window - 1, sink) - want).abs().max() > 0.3
    first_needed = max(0, first - window + 1)
    order = [7, 2, 11, 0, 5, 13, 1, 9]
    table = [order[i] if (i + 1) * PAGE > first_needed else -1 for i in range((T + PAGE - 1) // PAGE)]
    k_pool, v_pool = paged(k, [max(t, 0) for t in table], 16, dtype), paged(v, [max(t, 0) for t in table], 16, dtype)
    out = torch.zeros(new, H * V, dtype=dtype, device=DEV)
    run_attention(kernel, dev(q.reshape(new, H * K), dtype), dev(k_pool), dev(v_pool), out, table, first, new, H, G, K, V, scale,
                  dev(sink.float()), window)
    err = (out.double().cpu().view(new, H, V) - want).abs()
    worst = int(err.amax((1, 2)).argmax())
    assert err.max() < (1e-5 if dtype == torch.float32 else 5e-2), (first + worst, float(err.max()))


# --------------------------------------------------------------- neighbour-pair rotation, unit heads, blended values
@pytest.mark.parametrize("H, G, K, V, rot", [(3, 1, 24, 40, 8), (2, 2, 64, 64, 64), (4, 2, 16, 8, 2), (1, 1, 128, 128, 0),
                                             (2, 1, 256, 16, 100), (5, 5, 10, 12, 10)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("blend_mode", [0, 1, 2])
def test_rotation_of_neighbours_then_unit_heads_and_blended_values(H, G, K, V, rot, dtype, blend_mode):
    g = torch.Generator().manual_seed(K + rot)
    positions = [0, 1, 63, 64, 65, 1000, 99999, 1048575][:6 if dtype == torch.bfloat16 else 8]
    n = len(positions)
    width = H * K + G * K + G * V
    qkv = torch.randn(n, width, generator=g)
    qkv[:, :K] *= 100.0                              # a norm over all heads at once would crush the others
    bias = torch.randn(width, generator=g) * 0.3
    eps, base, lam = 1e-5, 300.0, 0.3125
    inv_freq = torch.tensor([base ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float32) if rot else None
    pos = torch.tensor(positions)
    x = qkv.double() + bias.double()
    qs, ks, vs = x[:, :H * K].view(n, H, K), x[:, H * K:(H + G) * K].view(n, G, K), x[:, (H + G) * K:].view(n, G, V)

    def turn(t):
        if not rot:
            return t
        ang = (pos.float()[:, None] * inv_freq[None, :]).double()      # the angle as the kernel takes it: a 32-bit product
        c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        out = t.clone()
        a, b = t[..., 0:rot:2], t[..., 1:rot:2]
        out[..., 0:rot:2] = a * c - b * s
        out[..., 1:rot:2] = b * c + a * s
        return out

    q_want, k_want = plain.unit_rms(turn(qs), eps), plain.unit_rms(turn(ks), eps)
    if rot:
        small = pos < 2000      # there the 32-bit angle and the exact one agree to 1e-4: the design's own formula
        ref = plain.unit_rms(plain.rotate_neighbours(qs, pos, rot, base), eps)
        assert (ref[small] - q_want[small]).abs().max() < 2e-2
    shared_before = torch.randn(n, G * V, generator=g)
    v_want = vs.reshape(n, G * V)
    if blend_mode == 2:
        v_want = (1 - lam) * v_want + lam * shared_before.double()
    pages_per = (max(positions) // PAGE) + 1
    n_pages = 24
    table = torch.full((n, pages_per), -1, dtype=torch.int32)
    for i, p in enumerate(positions):
        table[i, p // PAGE] = n_pages - 1 - 2 * i
    k_cache = torch.zeros(n_pages, G, PAGE, K, dtype=dtype, device=DEV)
    v_cache = torch.zeros(n_pages, G, PAGE, V, dtype=dtype, device=DEV)
    q_out = torch.zeros(n, H * K, dtype=dtype, device=DEV)
    shared = dev(shared_before)
    st = status()
    ops.pair_rope_unitnorm_kvwrite(dev(qkv), dev(bias), dev(inv_freq) if rot else None, rot, eps, True,
                                   shared if blend_mode else None, blend_mode, dev(torch.tensor([lam])) if blend_mode == 2 else None,
                                   i32(list(range(n))), i32(positions), q_out, k_cache, v_cache, dev(table), PAGE, H, G, K, V, True, st)
    assert int(st.item()) == 0
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert (q_out.double().cpu().view(n, H, K) - q_want).abs().max() < tol
    for i, p in enumerate(positions):
        page = n_pages - 1 - 2 * i
        assert (k_cache[page, :, p % PAGE].double().cpu() - k_want[i]).abs().max() < tol
        assert (v_cache[page, :, p % PAGE].double().cpu().reshape(-1) - v_want[i]).abs().max() < (1e-5 if dtype == torch.float32 else 5e-2)
    if blend_mode == 1:       # the first blending layer leaves its values, unrounded, for the later ones
        assert (shared.double().cpu() - vs.reshape(n, G * V)).abs().max() < 1e-5
    else:
        assert torch.equal(shared.cpu(), shared_before)
    # everything else of the cache is untouched
    assert int((k_cache != 0).any(-1).sum().item()) <= n * G and int((v_cache != 0).any(-1).sum().item()) <= n * G


# ------------------------------------------------------------------------------------------------ selective scan
def scan_inputs(rows, C, N, g, slow=False):
    x = torch.randn(rows, C, generator=g)
    dt_raw = torch.randn(rows, C, generator=g) - 1.0
    bc = torch.randn(rows, 2 * N, generator=g)
    z = torch.randn(rows, C, generator=g)
    a_log = torch.log(0.05 + 4 * torch.rand(C, N, generator=g))
    if slow:
        a_log = a_log - 12.0                    # decays of nearly one: what is written stays
    skip = torch.randn(C, generator=g)
    return x, dt_raw, bc, z, a_log, skip


def scan_want(x, dt_raw, bc, z, a_log, skip, runs, state0=None):
    """float64, run by run from ``state0`` [runs, C, N] (zeros); returns (y, final states)."""
    N = a_log.shape[1]
    ys, finals, at = [], [], 0
    for i, n in enumerate(runs):
        sl = slice(at, at + n)
        xs, dts = x[sl].double(), plain.softplus(dt_raw[sl].double())
        A = -torch.exp(a_log.double())
        S = torch.zeros_like(A) if state0 is None else state0[i].clone()
        for t in range(n):
            S = torch.exp(dts[t][:, None] * A) * S + (dts[t] * xs[t])[:, None] * bc[sl][t, :N].double()[None, :]
            ys.append((S @ bc[sl][t, N:].double() + skip.double() * xs[t]) * plain.silu(z[sl][t].double()))
        finals.append(S)
        at += n
    return torch.stack(ys), torch.stack(finals)


@pytest.mark.parametrize("C, N", [(40, 1), (96, 16), (33, 24), (128, 40), (20, 130), (260, 8), (12, 300)])
def test_selective_scan_over_unequal_runs_from_and_to_the_state(C, N):
    g = torch.Generator().manual_seed(C + N)
    runs = [37, 1, 70, 2]
    rows = sum(runs)
    x, dt_raw, bc, z, a_log, skip = scan_inputs(rows, C, N, g)
    want, finals = scan_want(x, dt_raw, bc, z, a_log, skip, runs)
    slots = [5, 0, 3, 6]
    pad = 7                                       # the state rows are longer than the recurrence's part
    state = torch.full((8, C * N + pad), 0.0, device=DEV)
    state[:, C * N:] = 9.0
    state[1, :C * N] = 4.0                        # a slot of nobody
    starts = i32(np.concatenate([[0], np.cumsum(runs)]))
    y = torch.zeros(rows, C, device=DEV)
    wide = torch.zeros(rows, 2 * C + 3, device=DEV)           # x and z as parts of wider rows
    wide[:, :C], wide[:, C + 3:] = dev(x), dev(z)
    low = torch.zeros(rows, 5 + 2 * N, device=DEV)
    low[:, 5:] = dev(bc)
    ops.selective_scan(wide[:, :C], dev(dt_raw), low[:, 5:], wide[:, C + 3:], dev(a_log), dev(skip), state, starts, i32(slots), y,
                       len(runs), C, N)
    assert (y.double().cpu() - want).abs().max() < 2e-4 * max(1.0, float(want.abs().max()))
    for i, s in enumerate(slots):
        assert (state[s, :C * N].double().cpu().view(C, N) - finals[i]).abs().max() < 1e-4 * max(1.0, float(finals[i].abs().max()))
    assert torch.all(state[:, C * N:] == 9.0) and torch.all(state[1, :C * N] == 4.0)
    # the same rows cut into calls of 5, 1 and the rest: equal bits
    state2 = torch.zeros_like(state)
    y2 = torch.zeros_like(y)
    at = 0
    for i, n in enumerate(runs):
        for a, b in ((0, min(5, n)), (min(5, n), min(6, n)), (min(6, n), n)):
            if b > a:
                sl = slice(at + a, at + b)
                ops.selective_scan(wide[sl, :C], dev(dt_raw)[sl], low[sl, 5:], wide[sl, C + 3:], dev(a_log), dev(skip), state2,
                                   i32([0, b - a]), i32([slots[i]]), y2[sl], 1, C, N)
        at += n
    assert torch.equal(y, y2)
    for s in slots:
        assert torch.equal(state[s, :C * N], state2[s, :C * N])
    # bfloat16 output (the bfloat16 engine's form: its exponentials come from the special-function unit, the 32-bit
    # engine's from multiply-adds): the same values up to that and one rounding
    y16 = torch.zeros(rows, C, device=DEV, dtype=torch.bfloat16)
    ops.selective_scan(wide[:, :C], dev(dt_raw), low[:, 5:], wide[:, C + 3:], dev(a_log), dev(skip), torch.zeros_like(state), starts,
                       i32(slots), y16, len(runs), C, N)
    assert ((y16.float() - y).abs() <= 2.0 ** -7 * y.abs() + 1e-4 * float(y.abs().max())).all()
    assert (y16.double().cpu() - want).abs().max() < 1e-2 * max(1.0, float(want.abs().max()))


def test_selective_scan_keeps_what_it_wrote_for_hundreds_of_tokens():
    """Decays of nearly one and a read-out vector that is zero but at the end: what the first token wrote is read back by
    the last one, 600 tokens later, through three calls."""
    C, N, rows = 8, 16, 600
    g = torch.Generator().manual_seed(4)
    x, dt_raw, bc, z, a_log, skip = scan_inputs(rows, C, N, g, slow=True)
    x[1:] = 0.0
    x[0] = 3.0
    bc[:, N:] = 0.0
    bc[-1, N:] = 1.0
    skip[:] = 0.0
    z[:] = 5.0
    want, _ = scan_want(x, dt_raw, bc, z, a_log, skip, [rows])
    assert float(want[-1].abs().min()) > 1e-3 and float(want[:-1].abs().max()) == 0.0
    state = torch.zeros(2, C * N, device=DEV)
    y = torch.zeros(rows, C, device=DEV)
    for a, b in ((0, 1), (1, 300), (300, rows)):
        sl = slice(a, b)
        ops.selective_scan(dev(x)[sl], dev(dt_raw)[sl], dev(bc)[sl], dev(z)[sl], dev(a_log), dev(skip), state, i32([0, b - a]), i32([1]),
                           y[sl], 1, C, N)
    assert (y.double().cpu() - want).abs().max() < 1e-4 * float(want.abs().max())


@pytest.mark.parametrize("C, taps", [(64, 4), (36, 2), (50, 5), (17, 1)])
def test_convolution_with_a_bias(C, taps):
    g = torch.Generator().manual_seed(taps)
    runs = [6, 1, 2, 9]
    rows = sum(runs)
    x = torch.randn(rows, C, generator=g)
    w = torch.randn(C, taps, generator=g)
    b = torch.randn(C, generator=g)
    want, at = [], 0
    for n in runs:
        want.append(plain.silu(plain.short_conv(x[at:at + n].double(), w.double(), b.double())))
        at += n
    want = torch.cat(want)
    state = torch.zeros(4, 3 + (taps - 1) * C, device=DEV)
    seq = sum(([i] * n for i, n in enumerate(runs)), [])
    y = torch.zeros(rows, C, device=DEV)
    ops.causal_conv(dev(x), dev(w), state[:, 3:] if taps > 1 else None, i32(seq), i32(np.concatenate([[0], np.cumsum(runs)])),
                    i32([2, 0, 3, 1]), y, len(runs), taps, silu=True, bias=dev(b))
    assert (y.double().cpu() - want).abs().max() < 1e-5


# ------------------------------------------------------------------------------------------------ router
def route_want(h, w_router, correction, top, groups, keep):
    w = {"router": w_router.double(), "correction": correction.double()}
    spec = {"experts": w_router.shape[0], "top": top}
    if groups:
        spec["groups"] = {"count": groups, "keep": keep}
    return plain.route(h.double(), w, "", spec)


@pytest.mark.parametrize("n, width, wdtype", [(5, 96, torch.float32), (40, 128, torch.bfloat16), (100, 96, torch.float32),
                                              (300, 256, torch.bfloat16), (70, 100, torch.bfloat16)])
@pytest.mark.parametrize("outputs, real, top, groups, keep", [(18, 14, 4, 3, 1), (9, 7, 2, 3, 2), (6, 6, 6, 0, 0), (12, 5, 4, 4, 2),
                                                              (40, 33, 8, 1, 1)])
def test_corrected_group_limited_choice_and_outputs_without_an_expert(n, width, wdtype, outputs, real, top, groups, keep):
    """Every path of the router (two launches for few tokens; a block per few tokens; logits on the tensor cores for many
    tokens and bfloat16 weights) against the float64 choice.  The corrections make every corrected score negative, so a
    shut-out group counted as zero would win."""
    g = torch.Generator().manual_seed(n + outputs)
    h = torch.randn(n, width, generator=g)
    w_router = (torch.randn(outputs, width, generator=g) * (3.0 / math.sqrt(width))).to(wdtype).float()
    correction = torch.randn(outputs, generator=g) * 0.05 - 1.5
    ids_want, wts_want, s = route_want(h, w_router, correction, top, groups, keep)
    ids = torch.zeros(n, top, dtype=torch.int32, device=DEV)
    wts = torch.zeros(n, top, device=DEV)
    offsets = torch.zeros(outputs + 1, dtype=torch.int32, device=DEV)
    perm_token = torch.zeros(n * top, dtype=torch.int32, device=DEV)
    perm_weight = torch.zeros(n * top, device=DEV)
    inverse = torch.zeros(n, top, dtype=torch.int32, device=DEV)
    logits = torch.zeros(n, outputs + 1, device=DEV)
    st = status()
    choice = (dev(correction), groups, keep)
    hd, wd = dev(h), dev(w_router, wdtype)
    if n <= ops.ROUTE_SMALL_TOKENS:
        ops.route_small(hd, wd, None, logits, ids, wts, None, top, False, offsets, perm_token, perm_weight, inverse, st,
                        choice=choice, n_real=real)
    else:
        ops.router_topk(hd, wd, None, ids, wts, None, top, False, st, logits=logits, choice=choice)
        ops.moe_permute(ids, wts, real, offsets, perm_token, perm_weight, inverse, st, n_ids=outputs)
    assert int(st.item()) == 0
    got_ids, got_w = ids.cpu().long(), wts.cpu().double()
    choice_scores = s + correction.double()
    for t in range(n):
        mine, want = set(got_ids[t].tolist()), set(ids_want[t].tolist())
        if mine != want:       # only between scores that 32-bit rounding cannot tell apart
            for e in mine ^ want:
                kth = choice_scores[t, ids_want[t]].min()
                assert abs(float(choice_scores[t, e] - kth)) < 1e-5, (t, e)
        assert len(mine) == top
        assert (got_w[t] - s[t, got_ids[t]]).abs().max() < 1e-5
    # the permutation: rows of the experts with weights, in expert order; the other choices have no row
    off, inv, ptok = offsets.cpu().long(), inverse.cpu().long(), perm_token.cpu().long()
    counts = torch.bincount(got_ids[got_ids < real].flatten(), minlength=real)
    assert off[:real + 1].tolist() == [0] + torch.cumsum(counts, 0).tolist()
    for t in range(n):
        for j in range(top):
            e, row = int(got_ids[t, j]), int(inv[t, j])
            if e >= real:
                assert row == -1
            else:
                assert off[e] <= row < off[e + 1] and int(ptok[row]) == t and float(perm_weight[row]) == float(wts[t, j])
    # the ordered sum: experts in ascending id, the outputs without an expert add weight times the input at their place
    width_out = 64
    rows_real = int(off[real])
    expert_out = torch.randn(max(rows_real, 1), width_out, generator=g)
    ident = torch.randn(n, width_out, generator=g)
    shared = torch.randn(n, width_out, generator=g)
    gate = torch.rand(n, generator=g)
    want = torch.zeros(n, width_out, dtype=torch.float64)
    for t in range(n):
        for e, j in sorted((int(got_ids[t, j]), j) for j in range(top)):
            want[t] += expert_out[inv[t, j]].double() if e < real else got_w[t, j] * ident[t].double()
        want[t] += gate[t].double() * shared[t].double()
    y = torch.zeros(n, width_out, device=DEV)
    passing = (wts, dev(ident), real)
    ops.moe_combine(dev(expert_out), ids, inverse, dev(gate), dev(shared), y, passing=passing)
    assert (y.double().cpu() - want).abs().max() < 1e-5
    # the same sum in the launch that also adds it to the residual stream and norms: equal bits with the two kernels
    x = torch.randn(n, width_out, generator=g)
    gamma = torch.rand(width_out, generator=g) + 0.5
    x1, x2 = dev(x), dev(x)
    h1 = torch.zeros(n, width_out, device=DEV)
    h2 = torch.zeros(n, width_out, device=DEV)
    ops.moe_combine_add_rmsnorm(dev(expert_out), ids, inverse, dev(gate), dev(shared), x1, dev(gamma), h1, 1e-5, passing=passing)
    ops.add_rmsnorm(x2, y, dev(gamma), h2, 1e-5)
    assert torch.equal(x1, x2) and torch.equal(h1, h2)


def test_a_gate_per_head_scales_the_heads_whole_output():
    g = torch.Generator().manual_seed(2)
    n, H, V = 37, 5, 24
    o = torch.randn(n, H * V, generator=g)
    wide = torch.randn(n, H + 9, generator=g)
    wd = dev(wide)
    for dtype in (torch.float32, torch.bfloat16):
        y = torch.zeros(n, H * V, dtype=dtype, device=DEV)
        ops.head_scalar_gate(dev(o), wd[:, 9:], y, H, V)
        want = o.double().view(n, H, V) * plain.sigmoid(wide[:, 9:].double())[:, :, None]
        assert (y.double().cpu().view(n, H, V) - want).abs().max() < (1e-6 if dtype == torch.float32 else 2e-2)


def test_the_gate_takes_rounded_input_in_place():
    g = torch.Generator().manual_seed(3)
    n, H, V = 21, 3, 64
    o = torch.randn(n, H * V, generator=g).to(torch.bfloat16)
    gate = torch.randn(n, H, generator=g)
    y = dev(o)
    ops.head_scalar_gate(y, dev(gate), y, H, V)
    want = o.double().view(n, H, V) * plain.sigmoid(gate.double())[:, :, None]
    assert (y.double().cpu().view(n, H, V) - want).abs().max() < 2e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_keys_and_values_of_every_head_into_pages_of_their_own(dtype):
    g = torch.Generator().manual_seed(5)
    H, K = 3, 64
    runs = [70, 1, 130]
    rows = sum(runs)
    kv = torch.randn(rows, 2 * H * K, generator=g)
    table = torch.full((3, 3), -1, dtype=torch.int32)
    table[0, :2] = torch.tensor([4, 1])
    table[1, :1] = torch.tensor([0])
    table[2, :3] = torch.tensor([5, 2, 3])
    seq = sum(([i] * n for i, n in enumerate(runs)), [])
    pos = sum((list(range(n)) for n in runs), [])
    k_pool = torch.zeros(6, H, PAGE, K, dtype=dtype, device=DEV)
    v_pool = torch.zeros(6, H, PAGE, K, dtype=dtype, device=DEV)
    kvd = dev(kv)
    st = status()
    ops.heads_to_pages(kvd[:, :H * K], kvd[:, H * K:], i32(seq), i32(pos), dev(table), k_pool, v_pool, PAGE, H, K, K, st)
    assert int(st.item()) == 0
    for r in range(rows):
        page = int(table[seq[r], pos[r] // PAGE])
        assert torch.equal(k_pool[page, :, pos[r] % PAGE].cpu(), kv[r, :H * K].view(H, K).to(dtype))
        assert torch.equal(v_pool[page, :, pos[r] % PAGE].cpu(), kv[r, H * K:].view(H, K).to(dtype))
    assert int((k_pool != 0).any(-1).sum().item()) == rows * H
