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

import math

import torch


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


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
def causal_conv(x, taps_w):
    """x [T, C], taps_w [C, taps]: y_t = sum_j taps_w[:, taps - 1 - j] x_(t - j), zeros before the start."""
    T, C = x.shape
    taps = taps_w.shape[1]
    y = torch.zeros_like(x)
    for j in range(taps):
        if j < T:
            y[j:] += x[:T - j] * taps_w[:, taps - 1 - j]
    return y


def gated_delta(h, w, pre, mix, eps):
    """The 'right' mixer: the delta rule with a decay per key channel, token by token."""
    H, G, K, V = mix["heads"], mix["kv_heads"], mix["dim"], mix["vdim"]
    T = h.shape[0]
    conv = lambda name: silu(causal_conv(h @ w[pre + name].T, w[pre + name + ".conv"].to(h.dtype)))
    q, k, v = conv("q").view(T, G, K), conv("k").view(T, G, K), conv("v").view(T, H, V)
    unit = lambda x: x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)
    q, k = unit(q) * K ** -0.5, unit(k)
    beta = sigmoid(h @ w[pre + "b"].T)                                                     # [T, H]
    raw = (h @ w[pre + "a1"].T) @ w[pre + "a2"].T + w[pre + "dt_bias"]
    decay = torch.exp(-torch.exp(w[pre + "A_log"].to(h.dtype))[None, :, None] * softplus(raw).view(T, H, K))
    gate = sigmoid((h @ w[pre + "g1"].T) @ w[pre + "g2"].T).view(T, H, V)
    S = torch.zeros(H, K, V, dtype=h.dtype)
    o = torch.zeros(T, H, V, dtype=h.dtype)
    for t in range(T):
        for head in range(H):
            g = head // (H // G)
            S[head] = decay[t, head][:, None] * S[head]
            u = beta[t, head] * (v[t, head] - S[head].T @ k[t, g])
            S[head] = S[head] + torch.outer(k[t, g], u)
            o[t, head] = S[head].T @ q[t, g]
    y = rms(o, eps) * w[pre + "norm"] * gate
    return y.reshape(T, H * V) @ w[pre + "o"].T


def parallel_mixer(h, w, pre, mix, eps, positions):
    left = chunked_sink_attention(h, w, pre + "left.", mix["left"], eps, positions)
    right = gated_delta(h, w, pre + "right.", mix["right"], eps)
    return mix["left_scale"] * left + mix["right_scale"] * right


# ---------------------------------------------------------------------------------------------------------
def gla(h, w, pre, mix, eps):
    """Gated linear attention: a decay per key channel, the read-out after the write."""
    H, K, V = mix["heads"], mix["dim"], mix["vdim"]
    T = h.shape[0]
    q = (h @ w[pre + "q"].T).view(T, H, K) * K ** -0.5
    k = (h @ w[pre + "k"].T).view(T, H, K)
    v = (h @ w[pre + "v"].T).view(T, H, V)
    z = (h @ w[pre + "a1"].T) @ w[pre + "a2"].T + w[pre + "a2.b"]
    alpha = torch.exp(-softplus(-z) / mix["tau"]).view(T, H, K)                            # sigmoid(z)^(1/tau)
    S = torch.zeros(H, K, V, dtype=h.dtype)
    o = torch.zeros(T, H, V, dtype=h.dtype)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    y = (rms(o, eps) * w[pre + "norm"]).reshape(T, H * V) * silu(h @ w[pre + "g"].T)
    return y @ w[pre + "o"].T


# ---------------------------------------------------------------------------------------------------------
def clamped_glu_ffn(h, w, pre, mlp):
    lim = mlp["limit"]
    g = torch.clamp(h @ w[pre + "gate"].T, max=lim)
    u = torch.clamp(h @ w[pre + "up"].T, min=-lim, max=lim)
    return (g * sigmoid(1.702 * g) * (u + 1)) @ w[pre + "down"].T


# ---------------------------------------------------------------------------------------------------------
def hyper_sublayer(streams, w, pre, fn, norm_w, eps):
    """streams [S, T, D] -> new streams: read u = sum_s in[s] x_s, run the sublayer on its norm, then
    x_t <- sum_s mix[s, t] x_s + out[t] y for all t at once."""
    u = torch.einsum("s,std->td", w[pre + "in"], streams)
    y = fn(rms(u, eps) * norm_w)
    return torch.einsum("sr,std->rtd", w[pre + "mix"], streams) + w[pre + "out"][:, None, None] * y[None]


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
def tensor_shapes(cfg):
    """name -> shape of every tensor of a model of this configuration, from the design."""
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
            kw, vw, r = b["kv_heads"] * b["dim"], b["heads"] * b["vdim"], b.get("rank", 8)
            out.update({q + "q": (kw, D), q + "q.conv": (kw, b["conv"]), q + "k": (kw, D), q + "k.conv": (kw, b["conv"]),
                        q + "v": (vw, D), q + "v.conv": (vw, b["conv"]), q + "b": (b["heads"], D), q + "A_log": (b["heads"],),
                        q + "norm": (b["vdim"],), q + "a1": (r, D), q + "a2": (b["heads"] * b["dim"], r),
                        q + "dt_bias": (b["heads"] * b["dim"],), q + "g1": (r, D), q + "g2": (vw, r), q + "o": (D, vw)})
        else:
            q = p + "mix."
            kw, vw, r = m["heads"] * m["dim"], m["heads"] * m["vdim"], m.get("rank", 8)
            out.update({q + "q": (kw, D), q + "k": (kw, D), q + "v": (vw, D), q + "g": (vw, D), q + "o": (D, vw),
                        q + "norm": (m["vdim"],), q + "a1": (r, D), q + "a2": (kw, r), q + "a2.b": (kw,)})
        mlp = layer.get("mlp")
        if mlp is not None:
            out[p + "norm2"] = (D,)
            if S:
                out.update({p + "hc2.in": (S,), p + "hc2.out": (S,), p + "hc2.mix": (S, S)})
            out.update({p + "mlp.gate": (mlp["ff"], D), p + "mlp.up": (mlp["ff"], D), p + "mlp.down": (D, mlp["ff"])})
    return out


def greedy(cfg, weights, prompt, count):
    tokens = list(prompt)
    for _ in range(count):
        tokens.append(int(forward(cfg, weights, tokens)[-1].argmax()))
    return tokens[len(prompt):]
