"""The kernels behind the Migosun design, each alone against the plain restatement's function of the same mechanism,
at sizes the model tests do not have, with inputs made so that a fault shows: one key whose score stands out just
inside and just outside a chunk's edge, at a page's border, far back and at the sequence's first positions; scores so
low that only the learned sink is left; a convolution cut in the middle of its reach; a delta rule that overwrites a
key's value; decays of exactly one over hundreds of tokens."""
import math

import numpy as np
import pytest
import torch

import plain_migosun as plain

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


def run_attention(kernel, q, k_pool, v_pool, out, table, first, new, H, G, K, V, scale, sink, chunk):
    """The new tokens are positions first .. first + new - 1 of one sequence whose pages ``table`` lists (-1: none)."""
    st = status()
    args = (q, k_pool, v_pool, out)
    tables = i32([table])
    if kernel == "tensor16":              # mma.sync, tiles of 64 rows
        firsts = list(range(0, new, 64))
        ops.attn_prefill(*args, i32([0] * len(firsts)), i32(firsts), i32([0, new]), i32([first]), tables, PAGE, H, G, K, None,
                         st, vd=V, scale=scale, sink=sink, chunk=chunk)
    elif kernel == "tmem16":              # tcgen05, tiles of 128 rows
        firsts = list(range(0, new, ops.ATTN_TC05_TILE_ROWS))
        ops.attn_prefill_tc05(*args, i32([0] * len(firsts)), i32(firsts), i32([0, new]), i32([first]), tables, PAGE, H, G, K,
                              None, st, scale=scale, sink=sink, chunk=chunk)
    elif kernel == "split16":             # keys split over blocks, for few rows
        split = 128
        n_splits = (len(table) * PAGE + split - 1) // split
        part_o = torch.zeros(new, H, n_splits, K, device=DEV)
        part_ml = torch.zeros(new, H, n_splits, 2, device=DEV)
        counters = torch.zeros(ops.ATTN_DECODE_COUNTERS, dtype=torch.int32, device=DEV)
        ops.attn_decode(*args, part_o, part_ml, counters, i32([0] * new), i32(list(range(first, first + new))), tables, PAGE, H, G,
                        K, None, split, n_splits, st, scale=scale, sink=sink, chunk=chunk)
        assert int(counters.abs().sum().item()) == 0
    else:
        ops.attn_simt(*args, i32([0] * new), i32(list(range(first, first + new))), tables, PAGE, H, G, K, None, st, vd=V,
                      scale=scale, sink=sink, chunk=chunk)
    assert int(st.item()) == 0


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("H, G, K, V, chunk", [(4, 2, 16, 40, 37), (3, 1, 56, 88, 100), (2, 2, 128, 128, 70), (8, 2, 64, 64, 64),
                                               (2, 1, 64, 64, 129), (2, 1, 24, 24, 1)])
@pytest.mark.parametrize("new", [200, 3])
def test_chunk_edges_seen_from_prompt_rows_and_from_single_rows(kernel, H, G, K, V, chunk, new):
    """460 cached positions in pages handed out in no order; the new tokens are the last 200 (rows of a prompt's
    portion) or the last 3 (decoding).  For probed queries one key gets a large score: the chunk's first position (just
    inside), the position before it (just outside: it must not be seen, so the result is the plain average with the sink),
    the query itself, the key before the query, and the far end of a long chunk."""
    if not takes(kernel, K, V):
        pytest.skip("this kernel wants keys and values of one size, 64 or 128")
    dtype = torch.float32 if kernel == "plain32" else torch.bfloat16
    g = torch.Generator().manual_seed(chunk * 7 + new)
    T = 460
    q = torch.randn(new, H, K, generator=g) * 0.3
    k = torch.randn(T, G, K, generator=g) * 0.3
    v = torch.randn(T, G, V, generator=g)
    first = T - new
    rows = sorted(set([0, 1, new - 1, new // 2] + [r for r in range(new) if (first + r) % chunk in (0, 1, chunk - 1)][:12]))
    used = set()
    for n, row in enumerate(rows):
        pos = first + row
        start = pos - pos % chunk
        key = [start, start - 1, pos, pos - 1, start + 1][n % 5]
        if key < 0 or key > pos + 0 and key != pos or key in used:
            continue
        used.add(key)
        head = row % H
        direction = torch.randn(K, generator=g)
        direction /= direction.norm()
        k[key, head // (H // G)] = direction * 6
        q[row, head] = direction * 6
    q, k, v = (t.to(dtype).double() for t in (q, k, v))
    sink = torch.randn(H, generator=g)
    scale = 0.9
    pos = torch.arange(T)
    want = plain.attend_learned_sink(q, k, v, scale, plain.chunk_visible(pos[first:], pos, chunk), sink.double())
    if chunk > 1:     # the probes tell a mask that is one position off either way
        for off in (chunk - 1, 1):
            shifted = plain.chunk_visible(pos[first:] + off, pos + off, chunk)
            other = plain.attend_learned_sink(q, k, v, scale, shifted, sink.double())
            assert (other - want).abs().max() > 0.3
    # pages behind the first chunk that any new token sees are not held any more
    first_needed = first - first % chunk
    order = [7, 2, 11, 0, 5, 13, 1, 9]
    table = [order[i] if (i + 1) * PAGE > first_needed else -1 for i in range((T + PAGE - 1) // PAGE)]
    k_pool, v_pool = paged(k, [max(t, 0) for t in table], 16, dtype), paged(v, [max(t, 0) for t in table], 16, dtype)
    out = torch.zeros(new, H * V, dtype=dtype, device=DEV)
    run_attention(kernel, dev(q.reshape(new, H * K), dtype), dev(k_pool), dev(v_pool), out, table, first, new, H, G, K, V, scale,
                  dev(sink.float()), chunk)
    err = (out.double().cpu().view(new, H, V) - want).abs()
    worst = int(err.amax((1, 2)).argmax())
    assert err.max() < (1e-5 if dtype == torch.float32 else 5e-2), (first + worst, float(err.max()))


@pytest.mark.parametrize("K, V", [(32, 16), (64, 64), (128, 128)])
@pytest.mark.parametrize("kernel", ["plain32", "tensor16", "tmem16", "split16"])
def test_the_learned_sink_is_one_unscaled_term_per_head(kernel, K, V):
    """Every score equals s: a row that sees n keys gives n e^s / (n e^s + e^sink) of the values' mean, whatever the
    scale.  Head 0 has a sink far above the scores (the output is nearly nothing), head 1 one of the scores' size (the
    output is a known fraction), head 2 one far below (the plain mean)."""
    if not takes(kernel, K, V):
        pytest.skip("this kernel wants keys and values of one size, 64 or 128")
    dtype = torch.float32 if kernel == "plain32" else torch.bfloat16
    H, chunk = 3, 50
    T = 120 if kernel == "split16" else 130
    g = torch.Generator().manual_seed(8)
    direction = torch.randn(K, generator=g)
    direction /= direction.norm()
    q = (direction * 2).repeat(T, H, 1)
    k = (direction * 2).repeat(T, 1, 1)
    v = torch.ones(T, 1, V) * 2.0
    q, k, v = (t.to(dtype).double() for t in (q, k, v))
    scale = 0.25
    s = float((q[0, 0] * k[0, 0]).sum()) * scale
    sink = torch.tensor([s + 12.0, s + 0.5, s - 30.0])
    table = [2, 0, 1]
    out = torch.zeros(T, H * V, dtype=dtype, device=DEV)
    run_attention(kernel, dev(q.reshape(T, H * K), dtype), dev(paged(k, table, 3, dtype)), dev(paged(v, table, 3, dtype)), out,
                  table, 0, T, H, 1, K, V, scale, dev(sink.float()), chunk)
    got = out.double().cpu().view(T, H, V)
    seen = (torch.arange(T) % chunk + 1).double()
    for head in range(H):
        want = 2.0 * seen / (seen + torch.exp(sink[head].double() - s))
        assert (got[:, head] - want[:, None]).abs().max() < (1e-5 if dtype == torch.float32 else 3e-2), head
    assert got[:, 0].abs().max() < 1e-2 and (got[:, 2] - 2.0).abs().max() < 2e-2
    assert 0.5 < got[0, 1, 0] < 1.0                   # one key beside the sink: 2 / (1 + e^0.5)


# ------------------------------------------------------------------------------ norms over the projection, rotation
@pytest.mark.parametrize("H, G, K, V, rot", [(3, 1, 24, 40, 8), (2, 2, 64, 64, 64), (4, 2, 16, 8, 2), (1, 1, 128, 128, 0)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_over_the_whole_projection_then_rotation_of_the_first_channels(H, G, K, V, rot, dtype):
    """One head of the queries is made a hundred times larger than the others: a norm per head would hide that, the norm
    over the whole projection keeps it.  Positions up to a million: the angles are 32-bit products of exact positions."""
    g = torch.Generator().manual_seed(K + rot)
    positions = [0, 1, 63, 64, 65, 1000, 99999, 1048575][:6 if dtype == torch.bfloat16 else 8]
    n = len(positions)
    qkv = torch.randn(n, H * K + G * K + G * V, generator=g)
    qkv[:, :K] *= 100.0
    q_w, k_w = torch.rand(H * K, generator=g) + 0.5, torch.rand(G * K, generator=g) + 0.5
    eps, base = 1e-5, 300.0
    inv_freq = torch.tensor([base ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float32) if rot else None
    pos = torch.tensor(positions)
    q_want = plain.rms(qkv[:, :H * K].double(), eps) * q_w.double()
    k_want = plain.rms(qkv[:, H * K:H * K + G * K].double(), eps) * k_w.double()
    if rot:
        # the frequencies as the kernel gets them (32-bit), the angle in 32-bit too: compare with that angle exactly
        ang = (pos.float()[:, None] * inv_freq[None, :]).double()
        def turn(x, heads):
            x = x.view(n, heads, K)
            a, b = x[..., :rot // 2], x[..., rot // 2:rot]
            c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
            return torch.cat([a * c - b * s, b * c + a * s, x[..., rot:]], -1)
        q_want, k_want = turn(q_want, H), turn(k_want, G)
        small = pos < 2000      # there the 32-bit angle and the exact one agree to 1e-4: the design's own formula
        ref = plain.rotate_half_layout((plain.rms(qkv[:, :H * K].double(), eps) * q_w.double()).view(n, H, K), pos, rot, base)
        assert (ref[small] - q_want.view(n, H, K)[small]).abs().max() < 2e-2
    q_want, k_want = q_want.reshape(n, H, K), k_want.reshape(n, G, K)
    # every position in a sequence of its own, at that position, in pages handed out backwards
    pages_per = (max(positions) // PAGE) + 1
    n_pages = 24
    table = torch.full((n, pages_per), -1, dtype=torch.int32)
    for i, p in enumerate(positions):
        table[i, p // PAGE] = n_pages - 1 - i
    k_pool = torch.zeros(n_pages, G, PAGE, K, dtype=dtype, device=DEV)
    v_pool = torch.zeros(n_pages, G, PAGE, V, dtype=dtype, device=DEV)
    q_out = torch.zeros(n, H * K, dtype=dtype, device=DEV)
    st = status()
    ops.widenorm_rope_kvwrite(dev(qkv), dev(q_w), dev(k_w), eps, dev(inv_freq) if rot else None, rot, 1.0, i32(list(range(n))),
                              i32(positions), q_out, k_pool, v_pool, table.to(DEV), PAGE, H, G, K, V, True, st)
    assert int(st.item()) == 0
    tol = 1e-4 if dtype == torch.float32 else 4e-2
    scale = float(q_want.abs().max())
    assert (q_out.double().cpu().view(n, H, K) - q_want).abs().max() < tol * scale
    for i, p in enumerate(positions):
        got_k = k_pool[n_pages - 1 - i, :, p % PAGE].double().cpu()
        got_v = v_pool[n_pages - 1 - i, :, p % PAGE].double().cpu()
        assert (got_k - k_want[i]).abs().max() < tol * float(k_want.abs().max())
        assert (got_v - qkv[i, H * K + G * K:].double().view(G, V)).abs().max() < tol * 4
    if rot and rot < K:         # the channels behind the rotated ones are the normed ones themselves
        plain_q = (plain.rms(qkv[:, :H * K].double(), eps) * q_w.double()).view(n, H, K)
        assert (q_out.double().cpu().view(n, H, K)[..., rot:] - plain_q[..., rot:]).abs().max() < tol * scale


# ------------------------------------------------------------------------------------------ short convolution
@pytest.mark.parametrize("C,lead,pad", [(37, 11, 9), (40, 12, 12)])
@pytest.mark.parametrize("taps", [1, 2, 3, 4, 7])
def test_convolution_cut_in_the_middle_of_its_reach(taps, C, lead, pad):
    """Three sequences in slots 5, 0, 2, cut into steps of 1, 2, 3 and more rows so that a cut falls inside the reach of
    the taps again and again; the kept inputs move from step to step.  One sequence is shorter than the taps.  With 40
    channels and aligned rows a short reach takes the kernel that walks tiles of rows (a run may begin inside a tile),
    otherwise the kernel of single rows."""
    g = torch.Generator().manual_seed(taps)
    w = torch.randn(C, taps, generator=g)
    lengths, slots = [45, taps - 1 if taps > 1 else 1, 12], [5, 0, 2]
    xs = [torch.randn(L, C, generator=g) for L in lengths]
    want = [plain.silu(plain.causal_conv(x.double(), w.double())) for x in xs]
    state = torch.full((6, lead + (taps - 1) * C), 7.0, device=DEV)        # other state ahead of the kept inputs
    conv_state = state[:, lead:] if taps > 1 else None
    if taps > 1:
        state[:, lead:] = 0.0                                                # what opening a slot does
    got = [torch.zeros(L, C) for L in lengths]
    at = [0, 0, 0]
    cuts = [1, 2, 3, 1, 5, 2, 64]
    step = 0
    while any(a < L for a, L in zip(at, lengths)):
        live = [i for i in range(3) if at[i] < lengths[i]]
        take = [min(cuts[(step + i) % len(cuts)], lengths[i] - at[i]) for i in live]
        x = torch.cat([xs[i][at[i]:at[i] + t] for i, t in zip(live, take)])
        wide = torch.zeros(x.shape[0], C + pad)                              # rows that are parts of wider rows
        wide[:, 4:4 + C] = x
        wide = dev(wide)
        y = torch.zeros(x.shape[0], C, device=DEV)
        starts = np.concatenate([[0], np.cumsum(take)])
        tok_seq = np.repeat(np.arange(len(live)), take)
        ops.causal_conv(wide[:, 4:4 + C], dev(w), conv_state, i32(tok_seq), i32(starts), i32([slots[i] for i in live]), y, len(live),
                        taps, silu=True)
        y = y.cpu()
        for j, (i, t) in enumerate(zip(live, take)):
            got[i][at[i]:at[i] + t] = y[starts[j]:starts[j] + t]
            at[i] += t
        step += 1
    for i in range(3):
        assert (got[i].double() - want[i]).abs().max() < 1e-5, i
    assert float(state[:, :lead].min()) == 7.0                               # the kernel keeps to its part of the state rows
    if taps > 1:
        kept = state[5, lead:].view(taps - 1, C).cpu()
        assert torch.equal(kept, xs[0][-(taps - 1):])


# -------------------------------------------------------------------------------------------------- delta rule
def delta_inputs(T, H, G, K, V, g):
    q = plain.unit_vectors(torch.randn(T, G, K, generator=g).double()) * K ** -0.5
    k = plain.unit_vectors(torch.randn(T, G, K, generator=g).double())
    v = torch.randn(T, H, V, generator=g).double()
    decay = torch.sigmoid(torch.randn(T, H, K, generator=g) * 2 + 3).double()
    beta = torch.sigmoid(torch.randn(T, H, generator=g)).double()
    return q, k, v, decay, beta


def run_delta(q, k, v, decay, beta, state, slot, H, G, K, V, cuts):
    T = q.shape[0]
    out = torch.zeros(T, H * V)
    at, i = 0, 0
    f = lambda t: dev(t.reshape(t.shape[0], -1).float())
    while at < T:
        n = min(cuts[i % len(cuts)], T - at)
        o = torch.zeros(n, H * V, device=DEV)
        ops.delta_scan(f(q[at:at + n]), f(k[at:at + n]), f(decay[at:at + n]), f(v[at:at + n]), f(beta[at:at + n]), state,
                       i32([0, n]), i32([slot]), o, 1, H, G, K, V)
        out[at:at + n] = o.cpu()
        at += n
        i += 1
    return out.view(T, H, V)


@pytest.mark.parametrize("H, G, K, V", [(4, 2, 24, 40), (1, 1, 128, 72), (6, 2, 8, 16), (2, 2, 64, 5), (3, 3, 200, 33)])
def test_delta_rule_in_runs_of_every_size_from_a_state_used_before(H, G, K, V):
    g = torch.Generator().manual_seed(H * K + V)
    T = 150
    q, k, v, decay, beta = delta_inputs(T, H, G, K, V, g)
    want, S_want = plain.delta_rule(q, k, v, decay, beta, torch.zeros(H, K, V, dtype=torch.float64))
    state = torch.randn(3, H * V * K + 13, device=DEV)                     # a slot that another sequence left
    state[1, :H * V * K] = 0.0                                             # opened: the matrices are zero
    whole = run_delta(q, k, v, decay, beta, state, 1, H, G, K, V, [T])
    assert (whole.double() - want).abs().max() < 2e-5 * max(1.0, float(want.abs().max()))
    S_got = state[1, :H * V * K].view(H, V, K).transpose(1, 2).double().cpu()
    assert (S_got - S_want).abs().max() < 2e-5 * max(1.0, float(S_want.abs().max()))
    state[1, :H * V * K] = 0.0
    cut = run_delta(q, k, v, decay, beta, state, 1, H, G, K, V, [1, 2, 1, 16, 17, 3, 33])
    assert torch.equal(cut, whole)                                         # no sum's order depends on the cutting


def test_delta_rule_overwrites_a_keys_value():
    """With beta 1 and no decay a second write under the same unit key replaces the first: reading with that key gives
    the second value alone, where a plain sum of outer products would give both.  Keys at right angles stay."""
    H, G, K, V, T = 2, 1, 32, 8, 40
    k = torch.zeros(T, G, K, dtype=torch.float64)
    k[:, 0, 3] = 1.0                     # filler tokens write under channel 3 ...
    k[5, 0] = 0.0
    k[5, 0, 0] = 1.0                     # token 5 and token 20 under channel 0
    k[20, 0] = 0.0
    k[20, 0, 0] = 1.0
    k[9, 0] = 0.0
    k[9, 0, 1] = 1.0                     # token 9 under channel 1
    v = torch.randn(T, H, V, generator=torch.Generator().manual_seed(1)).double()
    q = torch.zeros(T, G, K, dtype=torch.float64)
    q[:, 0, 0] = 1.0                     # every token reads channel 0
    q[30:, 0, 0] = 0.0
    q[30:, 0, 1] = 1.0                   # the last ones read channel 1
    decay, beta = torch.ones(T, H, K, dtype=torch.float64), torch.ones(T, H, dtype=torch.float64)
    state = torch.zeros(1, H * V * K, device=DEV)
    out = run_delta(q, k, v, decay, beta, state, 0, H, G, K, V, [7, 1, 1, 30]).double()
    assert out[:5].abs().max() == 0
    assert (out[5:20] - v[5][None]).abs().max() < 1e-6
    assert (out[20:30] - v[20][None]).abs().max() < 1e-6                   # not v[5] + v[20]
    assert (out[30:] - v[9][None]).abs().max() < 1e-6
    want, _ = plain.delta_rule(q, k, v, decay, beta, torch.zeros(H, K, V, dtype=torch.float64))
    assert (out - want).abs().max() < 1e-6


@pytest.mark.parametrize("H, G, K", [(4, 2, 24), (3, 3, 128), (2, 1, 7)])
def test_unit_vectors_decay_and_step_size_of_the_delta_rule(H, G, K):
    g = torch.Generator().manual_seed(K)
    n = 19
    qk = torch.randn(n, 2 * G * K + 3, generator=g) * 3
    qk[2] = 0.0                                                            # a row of zeros: the small constant keeps it finite
    qk[3] *= 1e-3
    raw = torch.randn(n, H * K + 5, generator=g) * 4
    raw[0, :4] = torch.tensor([-60.0, 60.0, 25.0, 0.0])
    dt_bias, a_log = torch.randn(H * K, generator=g), torch.randn(H, generator=g)
    b_raw = torch.randn(n, H + 2, generator=g) * 5
    want_q = plain.unit_vectors(qk[:, :G * K].double().view(n, G, K)) * K ** -0.5
    want_k = plain.unit_vectors(qk[:, G * K:2 * G * K].double().view(n, G, K))
    want_d = plain.delta_decay(raw[:, :H * K].double().view(n, H, K), a_log.double(), dt_bias.double().view(H, K))
    want_b = plain.sigmoid(b_raw[:, 1:1 + H].double())
    qk_d, raw_d, b_d = dev(qk), dev(raw), dev(b_raw)
    decay, beta = torch.zeros(n, H * K, device=DEV), torch.zeros(n, H, device=DEV)
    ops.delta_prepare(qk_d[:, :2 * G * K], G, K, 1e-6, K ** -0.5, raw_d[:, :H * K], decay, dev(dt_bias), dev(a_log), b_d[:, 1:1 + H],
                      beta, H)
    assert (qk_d[:, :G * K].double().cpu().view(n, G, K) - want_q).abs().max() < 1e-6
    assert (qk_d[:, G * K:2 * G * K].double().cpu().view(n, G, K) - want_k).abs().max() < 1e-6
    assert torch.equal(qk_d[:, 2 * G * K:].cpu(), qk[:, 2 * G * K:])
    assert (decay.double().cpu().view(n, H, K) - want_d).abs().max() < 1e-6
    assert (beta.double().cpu() - want_b).abs().max() < 1e-6


# ------------------------------------------------------------------------------------- gated linear attention
@pytest.mark.parametrize("tau", [1.0, 16.0, 2.5])
def test_decay_of_gated_linear_attention(tau):
    g = torch.Generator().manual_seed(3)
    n, W = 11, 40
    z = torch.randn(n, W, generator=g) * 6
    z[0, :3] = torch.tensor([-80.0, 80.0, 0.0])
    bias = torch.randn(W, generator=g)
    q = torch.randn(n, W + 8, generator=g)
    want = plain.channel_decay(z.double() + bias.double(), tau)
    z_d, q_out = dev(z), torch.zeros(n, W, device=DEV)
    ops.channel_decay_prepare(z_d, dev(bias), tau, dev(q)[:, 8:], 0.125, q_out)
    assert (z_d.double().cpu() - want).abs().max() < 1e-6
    assert (q_out.cpu() - q[:, 8:] * 0.125).abs().max() < 1e-7


@pytest.mark.parametrize("H, K, V", [(3, 24, 40), (1, 64, 16), (5, 8, 8), (2, 128, 128)])
def test_decays_of_exactly_one_keep_a_write_over_hundreds_of_tokens(H, K, V):
    """Token 0 writes value w under key channel 1 and nothing else ever writes there; channel 1 never decays, the
    others lose a tenth per token.  500 tokens later a query on channel 1 still reads w exactly; the read-out of a
    token sees the token's own write.  Cut into runs, from a slot's state."""
    g = torch.Generator().manual_seed(V)
    T = 520
    q = torch.randn(T, H, K, generator=g).double() * 0.1
    k = torch.randn(T, H, K, generator=g).double()
    k[:, :, 1] = 0.0
    k[0, :, 1] = 1.0
    v = torch.randn(T, H, V, generator=g).double()
    alpha = torch.full((T, H, K), 0.9, dtype=torch.float64)
    alpha[:, :, 1] = 1.0
    q[T - 1] = 0.0
    q[T - 1, :, 1] = 1.0
    want, S_want = plain.decayed_outer_products(q, k, v, alpha, torch.zeros(H, K, V, dtype=torch.float64))
    state = torch.zeros(2, H * V * K, device=DEV)
    f = lambda t: dev(t.reshape(t.shape[0], -1).float())
    out = torch.zeros(T, H * V)
    at = 0
    for n in [1, 1, 2, 60, 300, 156]:
        o = torch.zeros(n, H * V, device=DEV)
        ops.gated_scan(ops.SCAN_LOWER_SIGMOID, f(q[at:at + n]), f(k[at:at + n]), f(alpha[at:at + n]), f(v[at:at + n]), None, None,
                       None, state, i32([0, n]), i32([1]), o, 1, H, K, V, ready=True)
        out[at:at + n] = o.cpu()
        at += n
    out = out.view(T, H, V).double()
    assert (out[T - 1] - v[0]).abs().max() < 1e-5                          # the far write, untouched
    assert (out[0] - torch.einsum("hk,hk->h", q[0], k[0])[:, None] * v[0]).abs().max() < 1e-5   # a token sees its own write
    assert (out - want).abs().max() < 1e-4 * max(1.0, float(want.abs().max()))
    assert float(state[0].abs().max()) == 0.0


@pytest.mark.parametrize("sigmoid_gate", [False, True])
@pytest.mark.parametrize("H, V", [(3, 40), (1, 128), (6, 8)])
def test_norm_of_every_head_with_one_weight_for_all_heads_and_a_gate(H, V, sigmoid_gate):
    g = torch.Generator().manual_seed(V)
    n, eps = 9, 1e-5
    o = torch.randn(n, H * V, generator=g) * torch.logspace(-3, 3, n)[:, None]
    o[1] = 0.0
    w = torch.rand(V, generator=g) + 0.5
    gate = torch.randn(n, H * V + 6, generator=g) * 3
    want = plain.rms(o.double().view(n, H, V), eps) * w.double()
    act = plain.sigmoid(gate[:, 6:].double()) if sigmoid_gate else plain.silu(gate[:, 6:].double())
    want = want.reshape(n, H * V) * act
    y = torch.zeros(n, H * V, device=DEV)
    ops.head_rmsnorm_gate(dev(o), dev(w), 0, dev(gate)[:, 6:], y, H, V, eps, gate_sigmoid=sigmoid_gate)
    assert (y.double().cpu() - want).abs().max() < 1e-5 * max(1.0, float(want.abs().max()))


# -------------------------------------------------------------------------------- feed-forward, residual streams
@pytest.mark.parametrize("n_parts", [1, 2, 4])
@pytest.mark.parametrize("count", [3 * 52, 3 * 53])
def test_branches_side_by_side_are_added_with_a_weight_each(n_parts, count):
    g = torch.Generator().manual_seed(count + n_parts)
    parts = [torch.randn(3, count // 3, generator=g) for _ in range(n_parts)]
    scales = [0.5, -1.25, 2.0, 0.125][:n_parts]
    out = torch.zeros(3, count // 3, device=DEV)
    ops.weighted_sum(out, [dev(p) for p in parts], scales)
    want = sum(s * p.double() for s, p in zip(scales, parts))
    assert (out.double().cpu() - want).abs().max() < 1e-5


@pytest.mark.parametrize("I", [50, 52])
@pytest.mark.parametrize("limit", [0.5, 7.0])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_unit_with_clamped_branches(limit, dtype, I):
    """The gate is cut from above only (a very negative gate stays and gives nearly nothing), the linear branch on both
    sides, before one is added to it."""
    gu = torch.randn(13, 2 * I, generator=torch.Generator().manual_seed(5)) * 4
    gu[0, :4] = torch.tensor([-30.0, 30.0, limit, -limit])
    gu[0, I:I + 4] = torch.tensor([30.0, -30.0, -limit - 0.1, limit + 0.1])
    want = plain.clamped_glu(gu[:, :I].double(), gu[:, I:].double(), limit)
    assert abs(float(want[0, 1]) - limit / (1 + math.exp(-1.702 * limit)) * (1 - limit)) < 1e-9
    act = torch.zeros(13, I, dtype=dtype, device=DEV)
    ops.glu_clamped(dev(gu), act, limit, 1.702, 1.0)
    assert (act.double().cpu() - want).abs().max() < (1e-5 if dtype == torch.float32 else 2e-2) * float(want.abs().max())


@pytest.mark.parametrize("D", [52, 50, 1028])
@pytest.mark.parametrize("S", [1, 2, 3, 4, 5])
def test_write_to_all_copies_of_the_residual_stream_then_read(S, D):
    """The mixing matrix is far from symmetric, so [from, to] and [to, from] differ; all copies are written from the old
    ones at once.  Widths of whole pieces of four channels with few copies take the kernel of 16-byte accesses, the
    others the kernel of single channels."""
    g = torch.Generator().manual_seed(S)
    n, eps = 7, 1e-5
    streams = torch.randn(S, n, D, generator=g)
    y = torch.randn(n, D, generator=g)
    mix = torch.triu(torch.randn(S, S, generator=g)) + torch.eye(S)
    out_w, read_w, gamma = torch.randn(S, generator=g), torch.randn(S, generator=g), torch.rand(D, generator=g) + 0.5
    new = plain.hyper_write(streams.double(), mix.double(), out_w.double(), y.double())
    u = plain.hyper_read(new, read_w.double())
    h_want = plain.rms(u, eps) * gamma.double()
    st = dev(streams)
    h, u_out = torch.zeros(n, D, device=DEV), torch.zeros(n, D, device=DEV)
    ops.hc_step(st, h, dev(gamma), eps, y=dev(y), mix=dev(mix), out_w=dev(out_w), read_w=dev(read_w), u_out=u_out)
    assert (st.double().cpu() - new).abs().max() < 1e-5
    assert (u_out.double().cpu() - u).abs().max() < 1e-5
    assert (h.double().cpu() - h_want).abs().max() < 1e-5
    if S > 1:
        other = plain.hyper_write(streams.double(), mix.double().T, out_w.double(), y.double())
        assert (other - new).abs().max() > 0.1
    # the first write of a model: all copies equal the embedding output
    x0 = torch.randn(n, D, generator=g)
    st = torch.zeros(S, n, D, device=DEV)
    ops.hc_step(st, h, dev(gamma), eps, x0=dev(x0), y=dev(y), mix=dev(mix), out_w=dev(out_w), read_w=None, u_out=u_out)
    first = plain.hyper_write(x0.double()[None].repeat(S, 1, 1), mix.double(), out_w.double(), y.double())
    assert (st.double().cpu() - first).abs().max() < 1e-5
    assert (u_out.double().cpu() - first.sum(0)).abs().max() < 1e-5        # without read weights: the plain sum
