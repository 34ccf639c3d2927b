"""A plain, slow restatement of the Sebevik decoder, one function per mechanism.

It shares no code with the library: tensors come in as a dict name -> torch
tensor, the configuration as the parsed config.json, and everything runs on the
CPU in one dtype (float64 by default), token by token where the design has a
recurrence.  ``forward`` returns logits for a whole sequence and, optionally,
the residual stream after every layer.

Notation: T tokens, D width, H heads, G key/value heads, K key channels per
head, V value channels per head, R latent rank, C inner channels, N state size,
E experts with weights, I identity experts.
"""
from __future__ import annotations

import math

import torch


def sigmoid(z):
    return 1 / (1 + torch.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_norm(x, w, eps):
    """RMS norm whose tensor w holds the scale minus one."""
    return unit_rms(x, eps) * (1 + w)


# ---------------------------------------------------------------------------------------------------------
def causal_softmax_rows(scores, visible, extra=None):
    """scores [H, T, T]; visible [T, T] bool; ``extra`` [H]: one more term exp(extra_h) in every row's denominator."""
    s = scores.masked_fill(~visible[None], -math.inf)
    m = s.max(-1, keepdim=True).values
    if extra is not None:
        m = torch.maximum(m, extra[:, None, None])
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if extra is not None:
        den = den + torch.exp(extra[:, None, None] - m)
    return e / den


def latent_attention(h, w, pre, mix, eps):
    """Queries of full rank; one normed latent per position from which every head's keys and values are made; no
    positions; every earlier key is seen; each head's output times a sigmoid gate made from the layer's input."""
    T = h.shape[0]
    H, K, V = mix["heads"], mix["dim"], mix["vdim"]
    q = (h @ w[pre + "q"].T).view(T, H, K)
    c = unit_rms(h @ w[pre + "dkv"].T, eps) * w[pre + "dkv.norm"]
    k = (c @ w[pre + "uk"].T).view(T, H, K)
    v = (c @ w[pre + "uv"].T).view(T, H, V)
    scores = torch.einsum("thk,shk->hts", q, k) * mix["scale"]
    t = torch.arange(T)
    p = causal_softmax_rows(scores, t[None, :] <= t[:, None])
    o = torch.einsum("hts,shv->thv", p, v)
    o = o * sigmoid(h @ w[pre + "g"].T)[:, :, None]
    return o.reshape(T, H * V) @ w[pre + "o"].T


def rotate_neighbours(x, positions, dims, base):
    """x [T, heads, K]: of the first ``dims`` channels of every head, channel 2i is rotated with channel 2i + 1."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    ang = positions.to(torch.float64)[:, None] * (float(base) ** (-2.0 * i / dims))[None, :]
    cos, sin = torch.cos(ang).to(x.dtype)[:, None, :], torch.sin(ang).to(x.dtype)[:, None, :]
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = a * cos - b * sin
    out[..., 1:dims:2] = b * cos + a * sin
    return out


def window_sink_attention(h, w, pre, mix, eps, positions, first_values):
    """Grouped heads with biases, neighbour-pair rotation of the first channels, q and k divided by their root mean
    square per head, a sliding window, a learned term per head in the softmax's denominator, and values blended
    with those of the first blending layer.  Returns (output, this layer's values before any blend)."""
    T = h.shape[0]
    H, G, K, V = mix["heads"], mix["kv_heads"], mix["dim"], mix["vdim"]
    q = (h @ w[pre + "q"].T + w[pre + "q.b"]).view(T, H, K)
    k = (h @ w[pre + "k"].T + w[pre + "k.b"]).view(T, G, K)
    v = (h @ w[pre + "v"].T + w[pre + "v.b"]).view(T, G, V)
    rot = mix.get("rot")
    if rot:
        q, k = rotate_neighbours(q, positions, rot["dims"], rot["base"]), rotate_neighbours(k, positions, rot["dims"], rot["base"])
    q, k = unit_rms(q, eps), unit_rms(k, eps)
    own = v
    if mix.get("v_mix") and first_values is not None:
        lam = w[pre + "vmix"]
        v = (1 - lam) * v + lam * first_values
    rep = H // G
    scores = torch.einsum("thk,shk->hts", q, k.repeat_interleave(rep, dim=1)) * mix["scale"]
    t = torch.arange(T)
    dist = t[:, None] - t[None, :]
    visible = dist >= 0
    if mix.get("mask"):
        visible = visible & (dist < mix["mask"]["size"])
    p = causal_softmax_rows(scores, visible, extra=w[pre + "sink"].to(h.dtype))
    o = torch.einsum("hts,shv->thv", p, v.repeat_interleave(rep, dim=1))
    return o.reshape(T, H * V) @ w[pre + "o"].T, own


def short_conv(x, taps_w, bias):
    """x [T, C]; taps_w [C, taps] with the last column the current token's; zeros before the start."""
    T, C = x.shape
    taps = taps_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x])
    y = torch.zeros_like(x)
    for j in range(taps):
        y = y + padded[j:j + T] * taps_w[:, j]
    return y + bias


def selective_scan(x, dt, A, B, Cm, D):
    """x, dt [T, C]; A [C, N]; B, Cm [T, N]: S <- exp(dt A) S + dt x B; y = S Cm + D x, token by token from zero."""
    T, C = x.shape
    S = torch.zeros(C, A.shape[1], dtype=x.dtype)
    ys = []
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        ys.append(S @ Cm[t] + D * x[t])
    return torch.stack(ys)


def mamba(h, w, pre, mix):
    C, N, R = mix["inner"], mix["state"], mix["dt_rank"]
    xz = h @ w[pre + "in"].T
    x, z = xz[:, :C], xz[:, C:]
    x = silu(short_conv(x, w[pre + "conv"], w[pre + "conv.b"]))
    low = x @ w[pre + "x"].T
    dt = softplus(low[:, :R] @ w[pre + "dt"].T + w[pre + "dt.b"])
    y = selective_scan(x, dt, -torch.exp(w[pre + "A_log"]), low[:, R:R + N], low[:, R + N:], w[pre + "D"])
    return (y * silu(z)) @ w[pre + "o"].T


# ---------------------------------------------------------------------------------------------------------
def relu2_ffn(h, w, pre):
    return torch.relu(h @ w[pre + "up"].T) ** 2 @ w[pre + "down"].T


def gated_expert(h, w, pre):
    return (silu(h @ w[pre + "gate"].T) * (h @ w[pre + "up"].T)) @ w[pre + "down"].T


def route(h, w, pre, router):
    """(chosen ids [T, top], weights [T, top], scores [T, E + I]) by the corrected, group-limited choice."""
    s = torch.softmax(h @ w[pre + "router"].T, dim=-1)
    choice = s + w[pre + "correction"]
    groups = router.get("groups")
    if groups and groups["count"] > 1:
        T, n = choice.shape
        per = n // groups["count"]
        best = choice.view(T, groups["count"], per).max(-1).values
        keep = torch.topk(best, groups["keep"], dim=-1).indices
        allowed = torch.zeros(T, groups["count"], dtype=torch.bool)
        allowed.scatter_(1, keep, True)
        choice = choice.masked_fill(~allowed.repeat_interleave(per, dim=1), -math.inf)
    ids = torch.topk(choice, router["top"], dim=-1).indices
    return ids, torch.gather(s, 1, ids), s


def moe_ffn(h, w, pre, mlp, forced=None):
    """``forced`` (ids [T, top]): use these experts instead of the router's choice (the weights stay the scores)."""
    router = mlp["router"]
    E = router["experts"]
    ids, wts, s = route(h, w, pre, router)
    if forced is not None:
        ids = forced
        wts = torch.gather(s, 1, ids)
    y = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(ids.shape[1]):
            e = int(ids[t, j])
            out = gated_expert(h[t], w, f"{pre}e{e}.") if e < E else h[t]
            y[t] = y[t] + wts[t, j] * out
    if mlp.get("shared"):
        y = y + sigmoid(h @ w[pre + "shared.sg"].T) * gated_expert(h, w, pre + "shared.")
    return y


# ---------------------------------------------------------------------------------------------------------
def forward(cfg, weights, tokens, dtype=torch.float64, trace=None, forced_routing=None):
    """Logits [T, vocab].  ``trace``: a list that receives the residual stream behind every layer.
    ``forced_routing``: {layer index: ids [T, top]}."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    T = len(tokens)
    positions = torch.arange(T)
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    first_values = None
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = offset_norm(x, w[p + "norm1"], eps)
        mix = layer["mixer"]
        if layer["type"] == "latent_attention":
            y = latent_attention(h, w, p + "mix.", mix, eps)
        elif layer["type"] == "attention":
            y, own = window_sink_attention(h, w, p + "mix.", mix, eps, positions, first_values)
            if mix.get("v_mix") and first_values is None:
                first_values = own
        else:
            y = mamba(h, w, p + "mix.", mix)
        x = x + y
        mlp = layer.get("mlp")
        if mlp is not None:
            h = offset_norm(x, w[p + "norm2"], eps)
            if mlp["kind"] == "dense":
                x = x + relu2_ffn(h, w, p + "mlp.")
            else:
                x = x + moe_ffn(h, w, p + "mlp.", mlp, None if forced_routing is None else forced_routing.get(i))
        if trace is not None:
            trace.append(x.clone())
    return offset_norm(x, w["final.norm"], eps) @ w["embed"].T


def tensor_shapes(cfg):
    """name -> shape of every tensor a model folder of this design holds."""
    D = cfg["width"]
    out = {"embed": (cfg["vocab"], D), "final.norm": (D,)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        q = p + "mix."
        out[p + "norm1"] = (D,)
        if layer["type"] == "latent_attention":
            H, K, V, R = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
            out.update({q + "q": (H * K, D), q + "dkv": (R, D), q + "dkv.norm": (R,), q + "uk": (H * K, R), q + "uv": (H * V, R),
                        q + "g": (H, D), q + "o": (D, H * V)})
        elif layer["type"] == "attention":
            H, G, K, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({q + "q": (H * K, D), q + "q.b": (H * K,), q + "k": (G * K, D), q + "k.b": (G * K,), q + "v": (G * V, D),
                        q + "v.b": (G * V,), q + "sink": (H,), q + "o": (D, H * V)})
            if m.get("v_mix"):
                out[q + "vmix"] = ()
        else:
            C, N, R, taps = m["inner"], m["state"], m["dt_rank"], m["conv"]
            out.update({q + "in": (2 * C, D), q + "conv": (C, taps), q + "conv.b": (C,), q + "x": (R + 2 * N, C), q + "dt": (C, R),
                        q + "dt.b": (C,), q + "A_log": (C, N), q + "D": (C,), q + "o": (D, C)})
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        out[p + "norm2"] = (D,)
        f = p + "mlp."
        if mlp["kind"] == "dense":
            out.update({f + "up": (mlp["ff"], D), f + "down": (D, mlp["ff"])})
            continue
        r = mlp["router"]
        for e in range(r["experts"]):
            ff = mlp["expert"]["ff"]
            out.update({f"{f}e{e}.gate": (ff, D), f"{f}e{e}.up": (ff, D), f"{f}e{e}.down": (D, ff)})
        total = r["experts"] + r.get("identity", 0)
        out.update({f + "router": (total, D), f + "correction": (total,)})
        if mlp.get("shared"):
            ff = mlp["shared"]["ff"]
            out.update({f + "shared.gate": (ff, D), f + "shared.up": (ff, D), f + "shared.down": (D, ff), f + "shared.sg": (1, D)})
    return out


def random_weights(cfg, seed, gain=1.0):
    """name -> bfloat16 tensor (what a model folder stores), in ranges where every mechanism matters: sinks of the
    order of the scores, corrections of the order of the scores' spread, step sizes from about 0.01 to 1."""
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(tuple(s), generator=g)
    ru = lambda *s: torch.rand(tuple(s), generator=g)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.rsplit(".", 1)[-1]
        if name == "embed":
            t = rn(*shape) * 0.7
        elif leaf in ("norm1", "norm2") or name == "final.norm":
            t = 0.15 * rn(*shape)
        elif name.endswith("dkv.norm"):
            t = 1 + 0.2 * rn(*shape)
        elif leaf == "sink":
            t = rn(*shape) * 1.5
        elif leaf == "vmix":
            t = 0.2 + 0.6 * ru(*shape)
        elif leaf == "conv":
            t = rn(*shape) * 0.5
        elif leaf == "b":
            t = rn(*shape) * (0.7 if name.endswith("dt.b") else 0.3) - (2.0 if name.endswith("dt.b") else 0.0)
        elif leaf == "A_log":
            t = torch.log(1 + 15 * ru(*shape))
        elif leaf == "D":
            t = 1 + 0.3 * rn(*shape)
        elif leaf == "correction":
            t = rn(*shape) * 0.05
        elif leaf == "router":
            t = rn(*shape) * (2.0 / math.sqrt(shape[1]))
        elif leaf == "dt" and len(shape) == 2:
            t = rn(*shape) * (1.0 / math.sqrt(shape[1]))
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
