"""A plain, slow restatement of the Migosun decoder, one function per mechanism.

It shares no code with the library: tensors come in as a dict name -> torch
tensor, the configuration as the parsed config.json, and everything runs on the
CPU in one dtype (float64 by default), token by token where the design has a
recurrence.  ``forward`` returns logits for a whole sequence and, optionally,
the residual stream (the sum of the streams) after every layer.

Notation: T tokens, D width, H heads, G key/value heads, K key channels per
head, V value channels per head, S residual streams.
"""
from __future__ import annotations

import contextlib
import math

import torch


_round_norms_to = None


def rms(x, eps):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if _round_norms_to is None else y.to(_round_norms_to).to(x.dtype)


@contextlib.contextmanager
def norms_rounded_to(dtype):
    """Inside, every norm's result is rounded to ``dtype`` (and nothing else is): how far the logits of a position move
    under that tells how well conditioned the position is for an engine that keeps activations in that type."""
    global _round_norms_to
    _round_norms_to = dtype
    try:
        yield
    finally:
        _round_norms_to = None


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def sigmoid(z):
    return 1 / (1 + torch.exp(-z))


def silu(z):
    return z * sigmoid(z)


# ---------------------------------------------------------------------------------------------------------
def rotate_half_layout(x, positions, dims, base):
    """x [T, heads, K]: the first ``dims`` channels of every head are rotated, channel i with channel i + dims/2."""
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    freq = float(base) ** (-2.0 * i / dims)
    ang = positions.to(torch.float64)[:, None] * freq[None, :]
    cos, sin = torch.cos(ang).to(x.dtype)[:, None, :], torch.sin(ang).to(x.dtype)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, x[..., dims:]], dim=-1)


def chunk_visible(q_pos, k_pos, size):
    """[Tq, Tk] bool: key j is seen from position i if j <= i and both lie in the same chunk of ``size`` positions
    counted from the start of the sequence."""
    qi, kj = q_pos[:, None], k_pos[None, :]
    return (kj <= qi) & (torch.div(qi, size, rounding_mode="floor") == torch.div(kj, size, rounding_mode="floor"))


def attend_learned_sink(q, k, v, scale, visible, sink):
    """q [Tq, H, K], k [Tk, G, K], v [Tk, G, V], sink [H]: softmax whose denominator holds exp(sink_h) besides the
    visible keys' terms.  Returns [Tq, H, V]."""
    H, G = q.shape[1], k.shape[1]
    out = torch.zeros(q.shape[0], H, v.shape[2], dtype=q.dtype)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * scale
        s = s.masked_fill(~visible, float("-inf"))
        m = torch.maximum(s.max(-1, keepdim=True).values, sink[head].to(q.dtype))
        e = torch.exp(s - m)
        p = e / (e.sum(-1, keepdim=True) + torch.exp(sink[head].to(q.dtype) - m))
        out[:, head] = p @ v[:, g]
    return out


def chunked_sink_attention(h, w, pre, mix, eps, positions):
    """The 'left' mixer: norms over the whole query and key projections, partial rotation, chunked mask, sink."""
    H, G, K, V = mix["heads"], mix["kv_heads"], mix["dim"], mix["vdim"]
    T = h.shape[0]
    q = rms(h @ w[pre + "q"].T, eps) * w[pre + "q.norm"]
    k = rms(h @ w[pre + "k"].T, eps) * w[pre + "k.norm"]
    v = (h @ w[pre + "v"].T).view(T, G, V)
    q = rotate_half_layout(q.view(T, H, K), positions, mix["rot"]["dims"], mix["rot"]["base"])
    k = rotate_half_layout(k.view(T, G, K), positions, mix["rot"]["dims"], mix["rot"]["base"])
    o = attend_learned_sink(q, k, v, mix["scale"], chunk_visible(positions, positions, mix["mask"]["size"]), w[pre + "sink"])
    return o.reshape(T, H * V) @ w[pre + "o"].T


# ---------------------------------------------------------------------------------------------------------
def causal_conv(x, taps_w, before=None):
    """x [T, C], taps_w [C, taps]: y_t = sum_j taps_w[:, taps - 1 - j] x_(t - j).  ``before`` [taps - 1, C]: the inputs
    ahead of x's first row (oldest first); zeros at the start of a sequence."""
    T, C = x.shape
    taps = taps_w.shape[1]
    if before is None:
        before = torch.zeros(taps - 1, C, dtype=x.dtype)
    full = torch.cat([before.to(x.dtype), x], 0)
    y = torch.zeros_like(x)
    for j in range(taps):
        y += full[taps - 1 - j:taps - 1 - j + T] * taps_w[:, taps - 1 - j]
    return y


def unit_vectors(x, eps=1e-6):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + eps)


def delta_decay(raw, a_log, dt_bias):
    """raw [T, H, K], a_log [H], dt_bias [H, K] -> exp(-exp(a_log_h) softplus(raw + dt_bias))."""
    return torch.exp(-torch.exp(a_log)[None, :, None] * softplus(raw + dt_bias[None]))


def delta_rule(q, k, v, decay, beta, S):
    """Token by token, per head: S <- diag(decay) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q.
    q, k [T, G, K]; v [T, H, V]; decay [T, H, K]; beta [T, H]; S [H, K, V].  Returns (o [T, H, V], S)."""
    T, H = v.shape[0], v.shape[1]
    G = q.shape[1]
    S = S.clone()
    o = torch.zeros_like(v)
    for t in range(T):
        for head in range(H):
            g = head // (H // G)
            S[head] = decay[t, head][:, None] * S[head]
            u = beta[t, head] * (v[t, head] - S[head].T @ k[t, g])
            S[head] = S[head] + torch.outer(k[t, g], u)
            o[t, head] = S[head].T @ q[t, g]
    return o, S


def gated_delta(h, w, pre, mix, eps):
    """The 'right' mixer: the delta rule with a decay per key channel behind short convolutions."""
    H, G, K, V = mix["heads"], mix["kv_heads"], mix["dim"], mix["vdim"]
    T = h.shape[0]
    conv = lambda name: silu(causal_conv(h @ w[pre + name].T, w[pre + name + ".conv"].to(h.dtype)))
    q, k, v = conv("q").view(T, G, K), conv("k").view(T, G, K), conv("v").view(T, H, V)
    q, k = unit_vectors(q) * K ** -0.5, unit_vectors(k)
    beta = sigmoid(h @ w[pre + "b"].T)                                                     # [T, H]
    raw = ((h @ w[pre + "a1"].T) @ w[pre + "a2"].T).view(T, H, K)
    decay = delta_decay(raw, w[pre + "A_log"].to(h.dtype), w[pre + "dt_bias"].view(H, K))
    gate = sigmoid((h @ w[pre + "g1"].T) @ w[pre + "g2"].T).view(T, H, V)
    o, _ = delta_rule(q, k, v, decay, beta, torch.zeros(H, K, V, dtype=h.dtype))
    y = rms(o, eps) * w[pre + "norm"] * gate
    return y.reshape(T, H * V) @ w[pre + "o"].T


def parallel_mixer(h, w, pre, mix, eps, positions):
    left = chunked_sink_attention(h, w, pre + "left.", mix["left"], eps, positions)
    right = gated_delta(h, w, pre + "right.", mix["right"], eps)
    return mix["left_scale"] * left + mix["right_scale"] * right


# ---------------------------------------------------------------------------------------------------------
def channel_decay(z, tau):
    """sigmoid(z)^(1/tau), through the logarithm."""
    return torch.exp(-softplus(-z) / tau)


def decayed_outer_products(q, k, v, alpha, S):
    """Token by token: S <- diag(alpha_t) S + k_t v_t^T; o_t = S^T q_t.  q, k, alpha [T, H, K]; v [T, H, V]; S [H, K, V]."""
    S = S.clone()
    o = torch.zeros_like(v)
    for t in range(q.shape[0]):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return o, S


def gla(h, w, pre, mix, eps):
    """Gated linear attention: a decay per key channel, the read-out after the write."""
    H, K, V = mix["heads"], mix["dim"], mix["vdim"]
    T = h.shape[0]
    q = (h @ w[pre + "q"].T).view(T, H, K) * K ** -0.5
    k = (h @ w[pre + "k"].T).view(T, H, K)
    v = (h @ w[pre + "v"].T).view(T, H, V)
    z = (h @ w[pre + "a1"].T) @ w[pre + "a2"].T + w[pre + "a2.b"]
    o, _ = decayed_outer_products(q, k, v, channel_decay(z, mix["tau"]).view(T, H, K), torch.zeros(H, K, V, dtype=h.dtype))
    y = (rms(o, eps) * w[pre + "norm"]).reshape(T, H * V) * silu(h @ w[pre + "g"].T)
    return y @ w[pre + "o"].T


# ---------------------------------------------------------------------------------------------------------
def clamped_glu(g, u, lim):
    g = torch.clamp(g, max=lim)
    u = torch.clamp(u, min=-lim, max=lim)
    return g * sigmoid(1.702 * g) * (u + 1)


def clamped_glu_ffn(h, w, pre, mlp):
    return clamped_glu(h @ w[pre + "gate"].T, h @ w[pre + "up"].T, mlp["limit"]) @ w[pre + "down"].T


# ---------------------------------------------------------------------------------------------------------
def hyper_read(streams, read_w):
    return torch.einsum("s,std->td", read_w, streams)


def hyper_write(streams, mix, out_w, y):
    """x_t <- sum_s mix[s, t] x_s + out[t] y for all t at once (mix is indexed [from, to])."""
    return torch.einsum("sr,std->rtd", mix, streams) + out_w[:, None, None] * y[None]


def hyper_sublayer(streams, w, pre, fn, norm_w, eps):
    """streams [S, T, D] -> new streams: read the sublayer's input, run it on the norm, write back."""
    y = fn(rms(hyper_read(streams, w[pre + "in"]), eps) * norm_w)
    return hyper_write(streams, w[pre + "mix"], w[pre + "out"], y)


def forward(cfg, weights, tokens, dtype=torch.float64, trace=None):
    """Logits [T, vocab] of one sequence from its first token.  ``trace``: a list that receives the sum of the
    streams after every layer."""
    w = {n: (t.to(dtype) if t.is_floating_point() else t) for n, t in weights.items()}
    eps = cfg["norm"]["eps"]
    T = len(tokens)
    positions = torch.arange(T)
    x = w["embed"][torch.as_tensor(tokens)] * cfg["embedding"]["scale"]
    S = cfg.get("streams")
    streams = x[None].repeat(S, 1, 1) if S else None
    for i, layer in enumerate(cfg["layers"]):
        pre, mix = f"l{i}.mix.", layer["mixer"]
        if layer["type"] == "parallel":
            mixer = lambda hh: parallel_mixer(hh, w, pre, mix, eps, positions)
        elif layer["type"] == "gla":
            mixer = lambda hh: gla(hh, w, pre, mix, eps)
        else:
            raise ValueError(layer["type"])
        mlp = layer.get("mlp")
        ffn = (lambda hh: clamped_glu_ffn(hh, w, f"l{i}.mlp.", mlp)) if mlp is not None else None
        if S:
            streams = hyper_sublayer(streams, w, f"l{i}.hc1.", mixer, w[f"l{i}.norm1"], eps)
            if ffn is not None:
                streams = hyper_sublayer(streams, w, f"l{i}.hc2.", ffn, w[f"l{i}.norm2"], eps)
            x = streams.sum(0)
        else:
            x = x + mixer(rms(x, eps) * w[f"l{i}.norm1"])
            if ffn is not None:
                x = x + ffn(rms(x, eps) * w[f"l{i}.norm2"])
        if trace is not None:
            trace.append(x.clone())
    return (rms(x, eps) * w["final.norm"]) @ w["embed"].T


# ---------------------------------------------------------------------------------------------------------
def tensor_shapes(cfg, decay_rank=8, gate_rank=8):
    """name -> shape of every tensor of a model of this configuration, from the design.  The inner widths of the
    low-rank projections are not part of the configuration."""
    D, out = cfg["width"], {}
    out["embed"] = (cfg["vocab"], D)
    out["final.norm"] = (D,)
    S = cfg.get("streams")
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        out[p + "norm1"] = (D,)
        if S:
            out.update({p + "hc1.in": (S,), p + "hc1.out": (S,), p + "hc1.mix": (S, S)})
        if layer["type"] == "parallel":
            a, b = m["left"], m["right"]
            q = p + "mix.left."
            out.update({q + "q": (a["heads"] * a["dim"], D), q + "k": (a["kv_heads"] * a["dim"], D),
                        q + "v": (a["kv_heads"] * a["vdim"], D), q + "q.norm": (a["heads"] * a["dim"],),
                        q + "k.norm": (a["kv_heads"] * a["dim"],), q + "sink": (a["heads"],),
                        q + "o": (D, a["heads"] * a["vdim"])})
            q = p + "mix.right."
            kw, vw, r, rg = b["kv_heads"] * b["dim"], b["heads"] * b["vdim"], decay_rank, gate_rank
            out.update({q + "q": (kw, D), q + "q.conv": (kw, b["conv"]), q + "k": (kw, D), q + "k.conv": (kw, b["conv"]),
                        q + "v": (vw, D), q + "v.conv": (vw, b["conv"]), q + "b": (b["heads"], D), q + "A_log": (b["heads"],),
                        q + "norm": (b["vdim"],), q + "a1": (r, D), q + "a2": (b["heads"] * b["dim"], r),
                        q + "dt_bias": (b["heads"] * b["dim"],), q + "g1": (rg, D), q + "g2": (vw, rg), q + "o": (D, vw)})
        else:
            q = p + "mix."
            kw, vw, r = m["heads"] * m["dim"], m["heads"] * m["vdim"], decay_rank
            out.update({q + "q": (kw, D), q + "k": (kw, D), q + "v": (vw, D), q + "g": (vw, D), q + "o": (D, vw),
                        q + "norm": (m["vdim"],), q + "a1": (r, D), q + "a2": (kw, r), q + "a2.b": (kw,)})
        mlp = layer.get("mlp")
        if mlp is not None:
            out[p + "norm2"] = (D,)
            if S:
                out.update({p + "hc2.in": (S,), p + "hc2.out": (S,), p + "hc2.mix": (S, S)})
            out.update({p + "mlp.gate": (mlp["ff"], D), p + "mlp.up": (mlp["ff"], D), p + "mlp.down": (D, mlp["ff"])})
    return out


def random_weights(cfg, seed, decay_rank=8, gate_rank=8, gain=1.0):
    """name -> bfloat16 tensor (what a model folder stores).  The ranges are chosen so that every mechanism matters:
    decays between about 0.3 and nearly 1, sinks of the order of the scores, connection weights that mix the streams."""
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g)
    ru = lambda *s: torch.rand(*s, generator=g)
    S = cfg.get("streams")
    out = {}
    for name, shape in tensor_shapes(cfg, decay_rank, gate_rank).items():
        leaf = name.rsplit(".", 1)[-1]
        if name == "embed":
            t = rn(*shape) * 0.5
        elif name.endswith(".conv"):
            t = rn(*shape) * 0.6
        elif name.endswith(".q.norm") or name.endswith(".k.norm") or leaf in ("norm", "norm1", "norm2"):
            t = 1 + 0.2 * rn(*shape)
        elif leaf == "sink":
            t = rn(*shape) * 1.5
        elif leaf == "A_log":
            t = rn(*shape) * 0.7 - 0.5
        elif leaf == "dt_bias":
            t = rn(*shape) - 1.0
        elif name.endswith(".a2.b"):
            t = rn(*shape) * 1.5 + 2.0
        elif ".hc" in name and leaf == "in":
            t = (0.5 + ru(*shape)) / S
        elif ".hc" in name and leaf == "out":
            t = 0.5 + ru(*shape)
        elif ".hc" in name and leaf == "mix":
            t = torch.eye(S) * 0.8 + 0.3 * ru(*shape) / S + 0.1 * rn(*shape)
        elif len(shape) == 2:
            t = rn(*shape) * (gain / math.sqrt(shape[1]))
        else:
            raise ValueError(name)
        out[name] = t.to(torch.bfloat16)
    return out


def greedy(cfg, weights, prompt, count):
    """Greedy continuation by running the whole sequence anew for every token; returns (tokens, the margin between
    the best and the second logit at every choice)."""
    tokens, margins = list(prompt), []
    for _ in range(count):
        top = torch.topk(forward(cfg, weights, tokens)[-1], 2)
        margins.append(float(top.values[0] - top.values[1]))
        tokens.append(int(top.indices[0]))
    return tokens[len(prompt):], margins
