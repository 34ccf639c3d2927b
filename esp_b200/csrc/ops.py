"""Python faces of the compiled kernels.

Every function here checks what it is given (device, dtype, contiguity, the
sizes the kernel takes), launches on torch's current stream and raises
``Backend`` if the launch is refused.  There is no other implementation behind
these functions: without the compiled library they raise.
"""
from __future__ import annotations

import ctypes
import functools
import os
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p

import torch

from ..errors import Backend
from .build import load_library

P = c_void_p

_SIGNATURES = {
    "esp_embed_gather": [P, c_int, P, P, c_int, c_int, c_int, c_float, P, P],
    "esp_softcap": [P, c_longlong, c_float, P],
    "esp_feed_tokens": [P, P, P, c_int, P],
    "esp_add_rmsnorm": [P, P, P, P, P, P, c_int, P, c_int, c_int, c_float, c_int, P],
    "esp_depth_mix": [P, P, P, P, P, c_int, c_int, c_int, P],
    "esp_xielu": [P, P, P, c_int, c_longlong, P],
    "esp_tanh": [P, P, c_int, c_longlong, P],
    "esp_token_shift_mix": [P, c_int, P, c_longlong, P, P, P, P, P, c_int, c_int, c_int, P],
    "esp_token_shift_keep": [P, c_int, P, c_longlong, P, P, c_int, c_int, P],
    "esp_gate_prepare": [c_int, P, c_longlong, P, c_longlong, P, P, P, P, P, c_longlong, c_int, P],
    "esp_gated_scan": [c_int, c_int, P, c_longlong, P, c_longlong, P, c_longlong, P, c_longlong, P, P, P, P, c_longlong, P, P, P,
                       c_int, c_int, c_int, c_int, P],
    "esp_head_rmsnorm_gate": [P, P, c_int, P, c_longlong, P, c_int, c_int, c_int, c_int, c_float, c_int, P],
    "esp_latent_kv_store": [P, P, P, c_float, c_int, P, P, P, c_int, c_int, c_int, P, c_int, c_int, c_int, c_int, c_float, P,
                            P],
    "esp_latent_q_rotate": [P, P, c_float, c_int, P, P, c_int, c_int, c_int, c_int, c_int, c_int, P],
    "esp_per_head_linear": [P, c_int, c_longlong, c_int, P, c_int, P, c_int, c_longlong, c_int, c_int, c_int, c_int, c_int, P],
    "esp_attn_latent_mma": [P, P, P, P, P, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                            c_float, c_int, c_int, P, P, P, P],
    "esp_attn_latent": [P, P, P, c_int, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, P, P],
    "esp_swiglu": [P, P, c_int, c_longlong, c_int, P],
    "esp_finite_check": [P, c_int, c_longlong, P, c_int, P],
    "esp_normal_fill": [P, c_int, c_longlong, c_ulonglong, c_float, c_float, P],
    "esp_gemm_simt": [P, c_int, P, P, c_int, P, P, P, c_int, P, c_int, c_int, c_int, c_int, c_longlong, c_longlong, P],
    "esp_rope_kvwrite": [P, P, P, P, P, P, c_int, c_int, P, P, P, c_int, P, c_int, c_int, c_int, c_int, c_int, c_int,
                         c_int, c_int, P, P],
    "esp_attn_simt": [P, P, P, P, c_int, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, P,
                      c_int, c_int, P, P],
    "esp_embed_sum": [P, P, c_int, P, P, P, P, P, P, P, P, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_float, P, P],
    "esp_norm_add_rmsnorm": [P, P, P, c_float, P, P, P, c_int, P, c_int, c_int, c_float, c_int, P],
    "esp_relu2": [P, P, P, c_int, c_longlong, c_int, P],
    "esp_qknorm_kvwrite": [P, P, P, P, c_float, c_float, c_int, P, P, P, P, P, c_int, P, c_int, c_int, c_int, c_int, c_int,
                           c_int, c_int, c_int, c_int, P, P],
    "esp_matrix_memory_prepare": [P, P, P, c_longlong, P, P, c_float, P, c_longlong, P, P, P, P, c_int, c_int, c_int, c_int,
                                  c_int, P],
    "esp_matrix_memory_finish": [P, P, P, P, c_longlong, P, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_float, P],
    "esp_conv_branches": [P, P, P, P, P, P, c_longlong, P, P, P, P, P, P, c_int, c_int, c_int, c_int, c_int, P],
    "esp_diag_scan": [P, P, P, P, c_float, P, P, P, c_longlong, P, P, P, c_int, c_int, c_int, c_int, c_int, P],
    "esp_hc_step": [P, P, P, P, P, P, P, P, P, c_int, P, c_int, c_longlong, c_int, c_int, c_float, c_int, P],
    "esp_glu_clamped": [P, P, c_int, c_longlong, c_int, c_float, c_float, c_float, P],
    "esp_weighted_sum": [P, P, P, P, P, c_float, c_float, c_float, c_float, c_longlong, P],
    "esp_cast_cols": [P, c_longlong, P, c_int, c_longlong, c_int, P],
    "esp_widenorm_rope_kvwrite": [P, P, P, c_float, P, c_int, c_float, P, P, P, P, P, c_int, P, c_int, c_int, c_int, c_int,
                                  c_int, c_int, c_int, c_int, c_int, P, P],
    "esp_delta_scan": [P, c_longlong, P, c_longlong, P, c_longlong, P, c_longlong, P, P, c_longlong, P, P, P, c_int, c_int,
                       c_int, c_int, c_int, P],
    "esp_delta_prepare": [P, c_longlong, c_int, c_int, c_float, c_float, P, c_longlong, P, P, P, P, c_longlong, P, c_int, c_int, P],
    "esp_channel_decay_prepare": [P, P, c_float, P, c_longlong, c_float, P, c_longlong, c_int, P],
    "esp_selective_scan": [P, c_longlong, P, c_longlong, P, c_longlong, P, c_longlong, P, P, P, c_longlong, P, P, P, c_int, c_int,
                           c_int, c_int, P],
    "esp_head_scalar_gate": [P, c_int, P, c_longlong, P, c_int, c_int, c_int, c_int, P],
    "esp_heads_to_pages": [P, c_longlong, P, c_longlong, P, P, P, c_int, c_int, c_int, P, P, c_int, c_int, c_int, c_int, c_int, P, P],
    "esp_pair_rope_unitnorm_kvwrite": [P, P, P, c_int, c_float, c_int, P, c_int, P, P, P, P, P, P, c_int, P, c_int, c_int, c_int,
                                       c_int, c_int, c_int, c_int, c_int, c_int, P, P],
    "esp_causal_conv": [P, c_longlong, P, P, P, c_longlong, P, P, P, P, c_int, c_int, c_int, c_int, c_int, P],
    "esp_router_topk": [P, c_int, P, P, c_int, P, P, P, P, P, c_int, c_int, c_int, c_int, c_int, P, c_int, c_int, P, P],
    "esp_moe_permute": [P, P, c_int, c_int, c_int, P, P, P, P, P, P, P, P, c_int, c_int, P, P, c_int, P],
    "esp_gather_rows": [P, P, P, c_int, c_int, P],
    "esp_route_small": [P, c_int, P, P, c_int, P, P, P, P, P, c_int, c_int, c_int, c_int, c_int, P, P, P, P, P, P, P, P, P, P,
                        c_int, P, c_int, c_int, c_int, P],
    "esp_gemm_tc05": [P, c_longlong, P, c_int, c_int, P, P, c_longlong, P, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int,
                      c_int, c_int, P, P],
    "esp_wait_probe": [c_int, P, P],
    "esp_moe_combine": [P, P, P, P, P, P, c_int, c_int, c_int, P, P, c_int, P],
    "esp_pick_tokens": [P, c_int, c_int, P, P, P, P, P, P],
    "esp_moe_combine_add_rmsnorm": [P, P, P, P, P, P, P, P, P, c_int, P, c_int, c_int, c_int, c_float, c_int, P, P, c_int, P],
    "esp_gemm_skinny": [P, c_longlong, P, P, c_longlong, P, P, c_int, c_longlong, P, c_int, c_int, c_int, c_int, c_int,
                        c_int, c_int, P, P],
    "esp_qkv_rope_skinny": [P, c_longlong, P, P, P, P, P, P, c_int, P, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int,
                            c_int, c_int, c_int, P, P],
    "esp_attn_prefill": [P, P, P, P, P, P, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                         P, c_int, c_int, P, P],
    "esp_attn_prefill_tc05": [P, c_longlong, P, P, P, P, P, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                              c_int, P, c_int, c_int, P, P],
    "esp_attn_decode": [P, P, P, P, P, P, P, P, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                        c_int, c_float, c_int, P, c_int, P, P],
}

_bound: dict = {}


def _fn(library: str, name: str):
    f = _bound.get(name)
    if f is None:
        lib = load_library(library)
        try:
            f = getattr(lib, name)
        except AttributeError:
            raise Backend(f"the compiled library '{library}' has no entry point {name}") from None
        f.argtypes = _SIGNATURES[name]
        f.restype = c_int
        _bound[name] = f
    return f


_device_index = None


def _stream() -> int:
    """The current stream's handle.  Asked for at every launch, so it takes the short way (the full
    ``torch.cuda.current_stream()`` costs several microseconds a call, a quarter of an eager step's host time)."""
    global _device_index
    if _device_index is None:
        _device_index = torch.cuda.current_device()
    raw = getattr(torch._C, "_cuda_getCurrentRawStream", None)
    if raw is not None:
        return raw(_device_index)
    return torch.cuda.current_stream().cuda_stream


_launches = 0


def launch_count() -> int:
    """Kernel launches made through this module since the process started."""
    return _launches


def add_launches(count: int) -> None:
    """Accounts for kernels that ran through the replay of a captured graph."""
    global _launches
    _launches += count


class LaunchProfile:
    """Device time by kind of kernel.  While one is active (``with LaunchProfile() as prof``) every launch made
    through this module on the current stream is followed by a CUDA event; the time between two events is
    charged to the later launch (so a launch's share holds the gap before it as well).  Meant for steps that
    run eagerly on one stream: no captured graphs, nothing on a second stream."""

    active = None

    def __init__(self):
        self.marks = []                      # (what, event)

    def __enter__(self):
        first = torch.cuda.Event(enable_timing=True)
        first.record()
        self.marks = [("start", first)]
        LaunchProfile.active = self
        return self

    def __exit__(self, *exc):
        LaunchProfile.active = None

    def note(self, what: str) -> None:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self.marks.append((what, ev))

    def rows(self) -> list:
        """[(kind, launches, microseconds)], the largest first."""
        torch.cuda.synchronize()
        total: dict = {}
        for (_w0, e0), (what, e1) in zip(self.marks, self.marks[1:]):
            n, us = total.get(what, (0, 0.0))
            total[what] = (n + 1, us + e0.elapsed_time(e1) * 1e3)
        return sorted(((w, n, us) for w, (n, us) in total.items()), key=lambda r: -r[2])

    def table(self) -> str:
        rows = self.rows()
        whole = sum(us for _w, _n, us in rows) or 1.0
        lines = [f"{'kernel':<28}{'launches':>9}{'us':>12}{'share':>8}"]
        lines += [f"{w:<28}{n:>9}{us:>12.1f}{us / whole:>8.1%}" for w, n, us in rows]
        lines.append(f"{'all':<28}{sum(n for _w, n, _u in rows):>9}{whole:>12.1f}{1:>8.0%}")
        return "\n".join(lines)


def _check(code: int, what: str) -> None:
    global _launches
    _launches += 1
    if LaunchProfile.active is not None:
        LaunchProfile.active.note(what)
    if code != 0:
        raise Backend(f"{what}: the launch was refused with CUDA error {code} "
                      f"(invalid value means a size this kernel does not take)")


def _ptr(t, dtype=None, what="tensor"):
    if t is None:
        return None
    if not t.is_cuda:
        raise Backend(f"{what} must live on the GPU; this library has no CPU path")
    if not t.is_contiguous():
        raise Backend(f"{what} must be contiguous")
    if dtype is not None and t.dtype not in (dtype if isinstance(dtype, tuple) else (dtype,)):
        raise Backend(f"{what} has dtype {t.dtype}, expected {dtype}")
    return t.data_ptr()


FLOATS = (torch.float32, torch.bfloat16)


def _is_bf16(t) -> int:
    return 1 if t.dtype == torch.bfloat16 else 0


# ---------------------------------------------------------------------------

def embed_gather(table, ids, x, status, scale: float = 1.0):
    """x[n] = scale * float(table[ids[n]]); ids int32 [N], x float32 [N, H]."""
    n, width = x.shape
    _check(_fn("core", "esp_embed_gather")(
        _ptr(table, FLOATS, "embedding table"), _is_bf16(table), _ptr(ids, torch.int32, "ids"),
        _ptr(x, torch.float32, "x"), n, width, table.shape[0], float(scale), _ptr(status, torch.int32), _stream()),
        "embed_gather")


def softcap(values, cap: float):
    """values = cap * tanh(values / cap), in place (float32)."""
    if not cap > 0:
        raise Backend(f"softcap: the cap must be positive, got {cap}")
    _check(_fn("core", "esp_softcap")(_ptr(values, torch.float32, "values"), values.numel(), float(cap), _stream()),
           "softcap")


def feed_tokens(ids, picks, src):
    """ids[j] = picks[src[j]] where src[j] >= 0 (all int32 on the device)."""
    _check(_fn("core", "esp_feed_tokens")(_ptr(ids, torch.int32, "ids"), _ptr(picks, torch.int32, "picks"),
                                           _ptr(src, torch.int32, "src"), ids.shape[0], _stream()), "feed_tokens")


def add_rmsnorm(x, y, gamma, h, eps, rows=None, write_x=True, h32=None, yscale=None):
    """h = rmsnorm(x + y) * gamma with x (+= y when write_x) float32, gamma
    float32, h float32 or bfloat16.  ``rows`` (int32) selects source rows;
    ``h32`` (float32, same shape as h) receives the unrounded rows; ``yscale``
    (float32 [width]) multiplies y channel by channel before it is added."""
    n_rows = h.shape[0]
    width = h.shape[1]
    if x.shape[1] != width or gamma.shape[0] != width:
        raise Backend("add_rmsnorm: widths disagree")
    _check(_fn("core", "esp_add_rmsnorm")(
        _ptr(x, torch.float32, "x"), _ptr(y, torch.float32, "y"), _ptr(yscale, torch.float32, "yscale"),
        _ptr(gamma, torch.float32, "gamma"),
        _ptr(rows, torch.int32, "rows"), _ptr(h, FLOATS, "h"), _is_bf16(h), _ptr(h32, torch.float32, "h32"), n_rows,
        width, float(eps),
        1 if write_x else 0, _stream()), "add_rmsnorm")


def depth_mix(x, y, yscale, history, weights, index: int):
    """Ends layer ``index`` of a model that averages over depth: history[index + 1] = x + y * yscale (y may be
    None), then x = sum_j weights[j] * history[j] over j = 0 .. index + 1.  All float32; history
    [depth, rows, width]."""
    n, width = x.shape
    if history.shape[0] < index + 2 or tuple(history.shape[1:]) != (n, width) or weights.shape[0] < index + 2:
        raise Backend("depth_mix: the history or the weights are too short for this layer")
    _check(_fn("core", "esp_depth_mix")(
        _ptr(x, torch.float32, "x"), _ptr(y, torch.float32, "y"), _ptr(yscale, torch.float32, "yscale"),
        _ptr(history, torch.float32, "history"), _ptr(weights, torch.float32, "weights"), int(index), n, width, _stream()),
        "depth_mix")


def xielu(z, pq, act):
    """act = xIELU(z) with the two raw numbers ``pq`` (float32 [2] on the device); z float32, act float32 or bfloat16."""
    if act.shape != z.shape:
        raise Backend("xielu: shapes disagree")
    _check(_fn("core", "esp_xielu")(_ptr(z, torch.float32, "z"), _ptr(pq, torch.float32, "pq"), _ptr(act, FLOATS, "act"),
                                    _is_bf16(act), z.numel(), _stream()), "xielu")


def tanh(z, out):
    _check(_fn("core", "esp_tanh")(_ptr(z, torch.float32, "z"), _ptr(out, FLOATS, "out"), _is_bf16(out), z.numel(),
                                   _stream()), "tanh")


def swiglu(gu, act):
    """act[m, i] = silu(gu[m, i]) * gu[m, I + i]; gu float32 [M, 2I]."""
    rows, inter = act.shape
    if gu.shape[0] < rows or gu.shape[1] != 2 * inter:
        raise Backend("swiglu: gu must be [rows, 2 * intermediate]")
    _check(_fn("core", "esp_swiglu")(_ptr(gu, torch.float32, "gu"), _ptr(act, FLOATS, "act"), _is_bf16(act), rows,
                                     inter, _stream()), "swiglu")


STATUS_LOGITS_NONFINITE = 2


def finite_check(values, status, bit: int = STATUS_LOGITS_NONFINITE):
    """ORs ``bit`` into status[0] if ``values`` (float32 or bfloat16, contiguous) hold a NaN or an infinity."""
    _check(_fn("core", "esp_finite_check")(_ptr(values, FLOATS, "values"), _is_bf16(values), values.numel(),
                                           _ptr(status, torch.int32), int(bit), _stream()), "finite_check")


def normal_fill(out, key: int, mean: float, std: float):
    """out[i] = mean + std * z(key, i), z standard normal, counter-based."""
    _check(_fn("core", "esp_normal_fill")(_ptr(out, FLOATS, "out"), _is_bf16(out), out.numel(),
                                          key & 0xFFFFFFFFFFFFFFFF, float(mean), float(std), _stream()), "normal_fill")


def gemm_simt(a, w, c, bias=None, row_scale=None, a_rows=None, group_offsets=None, rows=None):
    """c[m, :] = (a[a_rows[m] or m, :] @ w[g].T + bias) * row_scale[m] with true
    32-bit multiply-adds.  ``w`` is [N, K] or, grouped, [G, N, K] with
    ``group_offsets`` int32 [G+1] over the rows.  ``rows``: how many rows of c to
    compute (default: all of c)."""
    grouped = group_offsets is not None
    if grouped:
        groups, n, k = w.shape
    else:
        groups = 1
        n, k = w.shape
    m = c.shape[0] if rows is None else rows
    if a.shape[-1] != k or c.shape[-1] != n:
        raise Backend(f"gemm: shapes disagree: a {tuple(a.shape)}, w {tuple(w.shape)}, c {tuple(c.shape)}")
    if a.stride(-1) != 1 or c.stride(-1) != 1 or not w.is_contiguous():
        raise Backend("gemm: operands must be row-major")
    code = _fn("core", "esp_gemm_simt")(
        a.data_ptr(), _is_bf16(a), _ptr(a_rows, torch.int32, "a_rows"), w.data_ptr(), _is_bf16(w),
        _ptr(bias, torch.float32, "bias"), _ptr(row_scale, torch.float32, "row_scale"), c.data_ptr(), _is_bf16(c),
        _ptr(group_offsets, torch.int32, "group_offsets"), groups, m, n, k, a.stride(0), c.stride(0), _stream())
    _check(code, "gemm_simt")


def rope_kvwrite(qkv, bias, tok_seq, tok_pos, cos, sin, rot, q_out, k_cache, v_cache, block_table, page, nh, nkv, hd,
                 write_kv, status):
    """Add the bias, rotate queries and keys (split-half, 32-bit) and store keys
    and values in the paged cache.  k_cache/v_cache: [pages, nkv, page, hd]."""
    n = qkv.shape[0]
    if qkv.shape[1] != (nh + 2 * nkv) * hd:
        raise Backend("rope_kvwrite: qkv width disagrees with the head counts")
    n_pages = k_cache.shape[0] if k_cache is not None else 0
    _check(_fn("core", "esp_rope_kvwrite")(
        _ptr(qkv, torch.float32, "qkv"), _ptr(bias, torch.float32, "bias"), _ptr(tok_seq, torch.int32),
        _ptr(tok_pos, torch.int32), _ptr(cos, torch.float32), _ptr(sin, torch.float32), rot, cos.shape[0] if cos is not None else (1 << 30),
        _ptr(q_out, FLOATS, "q_out"), _ptr(k_cache, FLOATS), _ptr(v_cache, FLOATS), _is_bf16(q_out),
        _ptr(block_table, torch.int32), block_table.shape[1] if block_table is not None else 0, n_pages, page, n,
        nh, nkv, hd, 1 if write_kv else 0, _ptr(status, torch.int32), _stream()), "rope_kvwrite")


def _sink_args(sink, nh):
    """(flag, pointer) of a sink: True is one more term exp(0) in the softmax's denominator, a float32 tensor [heads]
    the term exp(sink[head])."""
    if isinstance(sink, torch.Tensor):
        if sink.dtype != torch.float32 or sink.numel() != nh:
            raise Backend("attention: the sinks must be one float32 number per query head")
        return 1, _ptr(sink, torch.float32, "sink")
    return (1 if sink else 0), None


def attn_simt(q, k_cache, v_cache, out, tok_seq, tok_pos, block_table, page, nh, nkv, hd, window, status, vd=None,
              scale=0.0, sink=False, chunk=None):
    """Attention of every token over its sequence's cached keys (32-bit arithmetic).  ``vd``: size of a value head
    (default: the key size); ``scale`` > 0 multiplies the scores instead of the division by sqrt(hd); ``sink``: the
    softmax's denominator holds one more term exp(0), or exp(sink[head]) when a tensor is given; ``chunk``: a query
    sees the keys of its own block of that many positions only."""
    sink_flag, sink_ptr = _sink_args(sink, nh)
    vd = hd if vd is None else vd
    if hd > 256 or vd > 256:
        raise Backend(f"attention: head sizes {hd} / {vd} are beyond the 256 this kernel takes")
    _check(_fn("core", "esp_attn_simt")(
        _ptr(q, FLOATS, "q"), _ptr(k_cache, FLOATS), _ptr(v_cache, FLOATS), _ptr(out, FLOATS), _is_bf16(q),
        _ptr(tok_seq, torch.int32), _ptr(tok_pos, torch.int32), _ptr(block_table, torch.int32), block_table.shape[1],
        k_cache.shape[0], page, q.shape[0], nh, nkv, hd, vd, float(scale), sink_flag, sink_ptr, int(window or 0),
        int(chunk or 0), _ptr(status, torch.int32), _stream()), "attn_simt")


def _choice_args(choice, n_experts):
    """(correction pointer, groups, kept groups) of a ``choice`` = (correction float32 [experts] or None, groups, keep)."""
    if choice is None:
        return None, 0, 0
    correction, groups, keep = choice
    if correction is not None and correction.shape[0] != n_experts:
        raise Backend("router: the correction has another length than the router has outputs")
    if groups and groups > 1 and (groups > 32 or n_experts % groups or not 1 <= keep <= groups):
        raise Backend(f"router: {groups} groups (keep {keep}) over {n_experts} experts are not taken")
    return _ptr(correction, torch.float32, "correction"), int(groups or 0), int(keep or 0)


def router_topk(h, w_router, w_gate, topk_ids, topk_w, gate, top_k, norm_topk, status, probs_out=None, logits=None,
                sigmoid=False, choice=None):
    """``choice``: None, or (correction, groups, keep): a number per expert added to its score for the choice only, and
    a limit of the choice to the best ``keep`` of ``groups`` equal groups of neighbouring experts.  ``logits``: optional float32 scratch [n, experts + 1]; with it, 32-bit activations and bfloat16 weights
    the logits of a step of many tokens are made on the tensor cores (three bfloat16 parts of every
    activation: products exact, sums in float)."""
    n, width = h.shape
    n_experts = w_router.shape[0]
    if top_k > 32:
        raise Backend(f"router: top-k {top_k} is beyond the 32 this kernel takes")
    if (width + 2 * n_experts) * 4 > 200 * 1024:
        raise Backend(f"router: width {width} + experts {n_experts} do not fit the kernel's shared memory")
    pc, groups, keep = _choice_args(choice, n_experts)
    if w_gate is not None and w_gate.dtype != w_router.dtype:
        raise Backend("router: router and shared-gate weights must share a dtype")
    if logits is not None and logits.numel() < n * (n_experts + 1):
        raise Backend("router: the logits scratch is smaller than [tokens, experts + 1]")
    _check(_fn("core", "esp_router_topk")(
        _ptr(h, FLOATS, "h"), _is_bf16(h), _ptr(w_router, FLOATS), _ptr(w_gate, FLOATS), _is_bf16(w_router),
        _ptr(topk_ids, torch.int32), _ptr(topk_w, torch.float32), _ptr(gate, torch.float32),
        _ptr(probs_out, torch.float32), _ptr(logits, torch.float32), n, width, n_experts, top_k,
        (1 if norm_topk else 0) | (2 if sigmoid else 0), pc, groups, keep, _ptr(status, torch.int32), _stream()), "router_topk")


ROUTE_SMALL_TOKENS = 64


def route_small_fits(width: int, n_experts: int) -> bool:
    # the second kernel's shared memory: probabilities of eight tokens, counts and cursors, and the step's pairs
    return width * 4 <= 48 * 1024 and (16 * n_experts) * 4 + (2 * n_experts + 1) * 4 + ROUTE_SMALL_TOKENS * 32 * 8 <= 48 * 1024


def route_small(h, w_router, w_gate, logits, topk_ids, topk_w, gate, top_k, norm_topk, offsets, perm_token,
                perm_weight, inverse, status, probs_out=None, distinct=None, tiles=None, sigmoid=False, choice=None,
                n_real=None):
    """``choice``: as for router_topk.  ``n_real``: experts from this id on have no rows (their pairs get inverse -1).
    Router and permutation for at most ROUTE_SMALL_TOKENS tokens: logits over many blocks, then one
    block for softmax, top-k and the permutation.  ``logits``: float32 scratch [N, E + 1].  ``distinct``:
    an int64 tensor of one element to which the number of experts with at least one token is added.
    ``tiles``: as for moe_permute (the row tiles of the grouped tensor-core products; one per expert with rows)."""
    n, width = h.shape
    n_experts = w_router.shape[0]
    if n > ROUTE_SMALL_TOKENS or top_k > 32 or not route_small_fits(width, n_experts):
        raise Backend("route_small: too many tokens or experts for this kernel")
    pc, groups, keep = _choice_args(choice, n_experts)
    _check(_fn("core", "esp_route_small")(
        _ptr(h, FLOATS, "h"), _is_bf16(h), _ptr(w_router, FLOATS), _ptr(w_gate, FLOATS), _is_bf16(w_router),
        _ptr(logits, torch.float32), _ptr(topk_ids, torch.int32), _ptr(topk_w, torch.float32),
        _ptr(gate, torch.float32), _ptr(probs_out, torch.float32), n, width, n_experts, top_k,
        (1 if norm_topk else 0) | (2 if sigmoid else 0), _ptr(offsets, torch.int32), _ptr(perm_token, torch.int32), _ptr(perm_weight, torch.float32),
        _ptr(inverse, torch.int32), _ptr(status, torch.int32), _ptr(distinct, torch.int64),
        _ptr(tiles[0], torch.int32) if tiles else None, _ptr(tiles[1], torch.int32) if tiles else None,
        _ptr(tiles[2], torch.int32) if tiles else None, _ptr(tiles[3], torch.int32) if tiles else None,
        tiles[0].shape[0] if tiles else 0, pc, groups, keep, int(n_real if n_real is not None else n_experts), _stream()),
        "route_small")


def moe_permute(topk_ids, topk_w, n_experts, offsets, perm_token, perm_weight, inverse, status, tiles=None,
                distinct=None, n_ids=None):
    """``n_ids``: ids from n_experts up to this name experts without rows (their pairs get inverse -1).  ``distinct``: as for route_small.  ``tiles``: optional (tile_group, tile_row0, tile_count, n_tiles) int32 tensors that receive the
    list of row tiles (of at most TC05_TILE_ROWS rows) for the grouped tensor-core products."""
    n, top_k = topk_ids.shape
    if (2 * n_experts + 1) * 4 > 48 * 1024:
        raise Backend(f"moe_permute: {n_experts} experts are beyond what this kernel takes")
    _check(_fn("core", "esp_moe_permute")(
        _ptr(topk_ids, torch.int32), _ptr(topk_w, torch.float32), n, top_k, n_experts, _ptr(offsets, torch.int32),
        _ptr(perm_token, torch.int32), _ptr(perm_weight, torch.float32), _ptr(inverse, torch.int32),
        _ptr(tiles[0], torch.int32) if tiles else None, _ptr(tiles[1], torch.int32) if tiles else None,
        _ptr(tiles[2], torch.int32) if tiles else None, _ptr(tiles[3], torch.int32) if tiles else None,
        TC05_TILE_ROWS if tiles else 0, tiles[0].shape[0] if tiles else 0, _ptr(status, torch.int32),
        _ptr(distinct, torch.int64), int(n_ids if n_ids is not None else n_experts), _stream()), "moe_permute")


def moe_combine(expert_out, topk_ids, inverse, gate, shared, y, passing=None):
    """``passing``: None, or (topk_w, ident float32 [tokens, width], n_real): a chosen id from n_real on adds its weight
    times the token's row of ``ident`` instead of an expert's row."""
    n, width = y.shape
    pw, pi, pn = (_ptr(passing[0], torch.float32), _ptr(passing[1], torch.float32, "ident"), int(passing[2])) if passing else (None, None, 0)
    _check(_fn("core", "esp_moe_combine")(
        _ptr(expert_out, torch.float32), _ptr(topk_ids, torch.int32), _ptr(inverse, torch.int32),
        _ptr(gate, torch.float32), _ptr(shared, torch.float32), _ptr(y, torch.float32), n, width, topk_ids.shape[1],
        pw, pi, pn, _stream()), "moe_combine")


def moe_combine_add_rmsnorm(expert_out, topk_ids, inverse, gate, shared, x, gamma, h, eps, rows=None, write_x=True,
                            h32=None, passing=None):
    """moe_combine followed by add_rmsnorm in one kernel (same operations in the same order): x (+)= combined
    expert outputs, h = rmsnorm(x) * gamma.  Width a multiple of 4, at most 16384.  ``passing``: as for moe_combine."""
    n_rows, width = h.shape
    pw, pi, pn = (_ptr(passing[0], torch.float32), _ptr(passing[1], torch.float32, "ident"), int(passing[2])) if passing else (None, None, 0)
    if width % 4 != 0 or width > 16384:
        raise Backend(f"moe_combine_add_rmsnorm: width {width} not taken")
    _check(_fn("core", "esp_moe_combine_add_rmsnorm")(
        _ptr(expert_out, torch.float32), _ptr(topk_ids, torch.int32), _ptr(inverse, torch.int32),
        _ptr(gate, torch.float32), _ptr(shared, torch.float32), _ptr(x, torch.float32), _ptr(gamma, torch.float32),
        _ptr(rows, torch.int32), _ptr(h, FLOATS, "h"), _is_bf16(h), _ptr(h32, torch.float32), n_rows, width,
        topk_ids.shape[1], float(eps), 1 if write_x else 0, pw, pi, pn, _stream()), "moe_combine_add_rmsnorm")


def pick_tokens(logits, temperature, top_p, rng_state, row_slot, tokens):
    """tokens[r] = arg-max of row r when temperature[r] == 0 (or temperature is
    None), else a draw from the row's own splitmix64 stream rng_state[row_slot[r]]
    (int64 storage read as unsigned)."""
    n, vocab = logits.shape
    _check(_fn("core", "esp_pick_tokens")(
        _ptr(logits, torch.float32, "logits"), n, vocab, _ptr(temperature, torch.float32), _ptr(top_p, torch.float32),
        _ptr(rng_state, torch.int64), _ptr(row_slot, torch.int32), _ptr(tokens, torch.int32), _stream()), "pick_tokens")


# ---------------------------------------------------------------------------
# bfloat16 kernels (library "bf16")
# ---------------------------------------------------------------------------
SKINNY_MAX_SMEM = 227 * 1024


def skinny_fits(k: int) -> bool:
    """Whether gemm_skinny can stage eight activation rows of width k."""
    return k % 8 == 0 and 8 * (k + 32) * 2 + 8 * 512 <= SKINNY_MAX_SMEM


def gemm_skinny(a, w, c, swiglu=False, row_scale=None, a_rows=None, group_offsets=None, rows=None, max_rows=None,
                offsets_ready=False, xielu_pq=None, relu2=False):
    """Weight-streaming product for few rows; bfloat16 a and w.  Plain: c[m] =
    scale[m] * a[row(m)] @ w[g].T with w [N,K] or [G,N,K].  swiglu: w holds
    [gate rows; up rows] ([2I,K] or [G,2I,K]) and c[m, j] = silu(gate_j) * up_j
    ([rows, I]).  ``max_rows``: upper bound of the rows of one group.  ``offsets_ready``: the group offsets (and
    ``row_scale``) were complete before the kernel that runs right before this one started, so this one may
    find its group and ask for its weights while that kernel still runs (only ``a`` is waited for).  ``xielu_pq`` (plain
    form; float32 [2] on the device): every output passes through the xIELU with these two raw numbers.  ``relu2`` (plain
    form): every output, after its row's scale, becomes max(v, 0)^2."""
    if relu2 and (swiglu or xielu_pq is not None):
        raise Backend("gemm_skinny: one activation at a time")
    grouped = group_offsets is not None
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise Backend("gemm_skinny takes bfloat16 operands")
    if grouped:
        groups, wn, k = w.shape
    else:
        groups = 1
        wn, k = w.shape
    n = wn // 2 if swiglu else wn
    m = c.shape[0] if rows is None else rows
    if a.shape[-1] != k or c.shape[-1] != n or a.stride(-1) != 1 or c.stride(-1) != 1 or not w.is_contiguous():
        raise Backend(f"gemm_skinny: shapes disagree: a {tuple(a.shape)}, w {tuple(w.shape)}, c {tuple(c.shape)}")
    if k % 8 != 0 or a.stride(0) % 8 != 0 or a.data_ptr() % 16 != 0:
        raise Backend(f"gemm_skinny: width {k} (and the row stride) must be a multiple of 8")
    if max_rows is None:
        max_rows = m
    code = _fn("bf16", "esp_gemm_skinny")(
        a.data_ptr(), a.stride(0), _ptr(a_rows, torch.int32, "a_rows"), w.data_ptr(), wn * k,
        _ptr(row_scale, torch.float32, "row_scale"), c.data_ptr(), _is_bf16(c), c.stride(0),
        _ptr(group_offsets, torch.int32, "group_offsets"), groups, m, n, k, max_rows, 2 if relu2 else 1 if swiglu else 0,
        1 if offsets_ready else 0, _ptr(xielu_pq, torch.float32, "xielu_pq"), _stream())
    _check(code, "gemm_skinny")


def qkv_rope_skinny_fits(rows: int, k: int, hd: int) -> bool:
    return rows <= 16 and hd % 16 == 0 and skinny_fits(k)


def qkv_rope_skinny(a, w_qkv, bias, tok_seq, tok_pos, cos, sin, q_out, k_cache, v_cache, block_table, page, nh, nkv, hd,
                    write_kv, status):
    """The packed q/k/v projection of at most 16 rows with bias, full split-half rotation of queries and keys
    and the cache write in one kernel (bfloat16): what gemm_skinny followed by rope_kvwrite computes."""
    m, k = a.shape
    if w_qkv.shape != ((nh + 2 * nkv) * hd, k) or not qkv_rope_skinny_fits(m, k, hd):
        raise Backend(f"qkv_rope_skinny: sizes not taken: a {tuple(a.shape)}, w {tuple(w_qkv.shape)}, head size {hd}")
    if cos.shape[1] != hd // 2:
        raise Backend("qkv_rope_skinny rotates the whole head: the tables must be [positions, head size / 2]")
    if a.stride(-1) != 1 or a.stride(0) % 8 != 0 or a.data_ptr() % 16 != 0:
        raise Backend("qkv_rope_skinny: the rows must be 16-byte aligned")
    _check(_fn("bf16", "esp_qkv_rope_skinny")(
        _ptr(a, torch.bfloat16, "a") if a.is_contiguous() else a.data_ptr(), a.stride(0), _ptr(w_qkv, torch.bfloat16, "w_qkv"),
        _ptr(bias, torch.float32, "bias"), _ptr(tok_seq, torch.int32), _ptr(tok_pos, torch.int32),
        _ptr(cos, torch.float32, "cos"), _ptr(sin, torch.float32, "sin"), cos.shape[0], _ptr(q_out, torch.bfloat16, "q_out"),
        _ptr(k_cache, torch.bfloat16), _ptr(v_cache, torch.bfloat16), _ptr(block_table, torch.int32),
        block_table.shape[1], k_cache.shape[0], page, m, k, nh, nkv, hd, 1 if write_kv else 0,
        _ptr(status, torch.int32), _stream()), "qkv_rope_skinny")


# blocks of the split-key kernel that one SM holds at a time, by head size (registers: 72 / 122 / 160 / 162 a thread)
ATTN_DECODE_BLOCKS_PER_SM = {64: 7, 128: 4, 192: 3, 256: 3}


@functools.lru_cache(maxsize=4096)
def attn_decode_split(n_rows: int, nkv_blocks: int, positions: int, head_dim: int = 128, sm_count: int = 148) -> int:
    """Key positions per block (whole pages of 64), the same for every row of the step: the length with the least
    estimated time.  The estimate, fitted to steps of 1 to 64 rows with 16 key/value heads of 128 at 4,096
    positions and checked at 8,000 to 32,000 positions with 4: the device holds ``room`` blocks at once and needs
    three quarters of that many to draw the full memory rate; blocks start as others end, so the time is that of
    all blocks' pages at the full rate, plus what the last, partly filled round lacks of three quarters, plus one
    page's time a block for its start, its partial result and its share of the combine.  It gives one round of
    short blocks to a few rows (128 positions at batch 1, 256 at batch 2, 1,024 at batch 8), whole rows to 32 or
    64 rows, and thirds or quarters of a row where whole rows would leave a round nearly empty (batch 24, 40, 48).
    Against the earlier choice among 128, 256 and 512 under a limit of 1,024 blocks: batch 2 +3.5 %, 5 +6 %, 6 +5 %,
    8 +1.5 %, 16 +4 %, 32 +4 %, 48 +2 %, 64 +4.5 %; batch 8 at 8,000 positions +5 %.  At least 128 positions, 256 beyond
    4,096 (at batch 1, 128 gains 1 % at 4,096 positions and loses 7 % at 8,192 with 4 key/value heads)."""
    room = sm_count * ATTN_DECODE_BLOCKS_PER_SM.get(head_dim, 3)
    full_rate = 0.75 * room
    pairs = max(1, n_rows * nkv_blocks)
    pages = max(1, (positions + 63) // 64)
    shortest = min(pages, 2 if positions <= 4096 else 4)
    best, best_cost = pages, None
    for length in range(pages, shortest - 1, -1):          # longest first: it wins a tie
        blocks = pairs * ((pages + length - 1) // length)
        last = blocks % room
        cost = (blocks + (full_rate - last if 0 < last < full_rate else 0.0)) * (length + 1.0)
        if best_cost is None or cost < best_cost:
            best, best_cost = length, cost
    return 64 * best


ATTN_DECODE_COUNTERS = 65536


def attn_decode(q, k_cache, v_cache, out, part_o, part_ml, counters, tok_seq, tok_pos, block_table, page, nh, nkv, hd,
                window, split, n_splits, status, seq_past=None, scale=0.0, sink=False, chunk=None):
    """Split-key attention for few token rows (bfloat16; head sizes 64, 128, 192, 256).  ``split``: key
    positions per block (a multiple of 64); n_splits >= ceil(positions / split).  part_o float32
    [N, nh, n_splits, hd] and part_ml float32 [N, nh, n_splits, 2] are scratch; ``counters``: int32, at least
    N * nh words, all zero (the kernel leaves them zero).  ``seq_past`` (int32 per sequence of the step: the
    positions cached before it): blocks whose keys are all older then load them without waiting for the
    kernel before this one, which writes the step's new keys and values.  ``scale`` > 0 multiplies the scores instead
    of the division by sqrt(hd); ``sink``: the softmax's denominator holds one more term exp(0), or exp(sink[head]) when
    a float32 tensor is given; ``chunk``: a query sees the keys of its own block of that many positions only."""
    sink_flag, sink_ptr = _sink_args(sink, nh)
    if counters.numel() < q.shape[0] * nh:
        raise Backend("attn_decode: too few counters for this many rows and heads")
    if split < 64 or split % 64:
        raise Backend(f"attn_decode: split {split} is not a multiple of 64")
    if hd not in (64, 128, 192, 256):
        raise Backend(f"attn_decode: head size {hd} is not one of 64, 128, 192, 256")
    n = q.shape[0]
    if part_o.numel() < n * nh * n_splits * hd or part_ml.numel() < n * nh * n_splits * 2:
        raise Backend("attn_decode: scratch is too small")
    _check(_fn("bf16", "esp_attn_decode")(
        _ptr(q, torch.bfloat16, "q"), _ptr(k_cache, torch.bfloat16), _ptr(v_cache, torch.bfloat16),
        _ptr(out, torch.bfloat16), _ptr(part_o, torch.float32), _ptr(part_ml, torch.float32),
        _ptr(counters, torch.int32), _ptr(tok_seq, torch.int32), _ptr(tok_pos, torch.int32), _ptr(seq_past, torch.int32),
        _ptr(block_table, torch.int32), block_table.shape[1],
        k_cache.shape[0], page, n, nh, nkv, hd, int(window or 0), split, n_splits, float(scale), sink_flag, sink_ptr,
        int(chunk or 0), _ptr(status, torch.int32), _stream()), "attn_decode")


def attn_flash_fits(hd, vd=None, page=64) -> bool:
    """Head sizes (keys, values) and page size that ``attn_prefill`` takes."""
    vd = hd if vd is None else vd
    return hd % 8 == 0 and vd % 8 == 0 and 0 < hd <= 128 and 0 < vd <= 128 and page == 64


def attn_prefill(q, k_cache, v_cache, out, tile_seq, tile_first, seq_start, seq_past, block_table, page, nh, nkv, hd,
                 window, status, vd=None, scale=0.0, sink=False, chunk=None):
    """Flash-style attention for runs of new tokens (bfloat16; head sizes that are multiples of 8 up to
    128; pages of 64 positions).  tile_seq / tile_first describe the tiles of 64 new tokens.  ``vd``: size of a
    value head (default: the key size); ``scale`` > 0 multiplies the scores instead of the division by sqrt(hd);
    ``sink``: the softmax's denominator holds one more term exp(0), or exp(sink[head]) when a float32 tensor is given;
    ``chunk``: a query sees the keys of its own block of that many positions only."""
    sink_flag, sink_ptr = _sink_args(sink, nh)
    vd = hd if vd is None else vd
    if not attn_flash_fits(hd, vd, page):
        raise Backend(f"attn_prefill: head sizes {hd} / {vd} / page {page} not taken (multiples of 8 up to 128; page 64)")
    _check(_fn("bf16", "esp_attn_prefill")(
        _ptr(q, torch.bfloat16, "q"), _ptr(k_cache, torch.bfloat16), _ptr(v_cache, torch.bfloat16),
        _ptr(out, torch.bfloat16), _ptr(tile_seq, torch.int32), _ptr(tile_first, torch.int32),
        _ptr(seq_start, torch.int32), _ptr(seq_past, torch.int32), _ptr(block_table, torch.int32),
        block_table.shape[1], k_cache.shape[0], page, tile_seq.shape[0], nh, nkv, hd, vd, float(scale), sink_flag, sink_ptr,
        int(window or 0), int(chunk or 0), _ptr(status, torch.int32), _stream()), "attn_prefill")


ATTN_TC05_TILE_ROWS = 128      # new tokens of a sequence to a tile of attn_prefill_tc05


def attn_prefill_tc05_fits(hd, page) -> bool:
    """Head sizes and page size that the tensor-memory prefill attention takes."""
    return hd in (64, 128) and page == 64


def attn_prefill_tc05(q, k_cache, v_cache, out, tile_seq, tile_first, seq_start, seq_past, block_table, page, nh, nkv, hd,
                      window, status, scale=0.0, sink=False, chunk=None):
    """Prefill attention on tcgen05 with accumulators in tensor memory (bfloat16; head size 64 or 128; pages
    of 64 positions).  Same arguments as attn_prefill, but tile_seq / tile_first list tiles of
    ATTN_TC05_TILE_ROWS new tokens, best with the tiles that see the most keys first (the order only matters
    for the balance).  ``scale`` > 0 multiplies the scores instead of the division by sqrt(hd); ``sink``: the softmax's
    denominator holds one more term exp(0), or exp(sink[head]) when a float32 tensor is given; ``chunk``: a query sees the
    keys of its own block of that many positions only."""
    sink_flag, sink_ptr = _sink_args(sink, nh)
    if not attn_prefill_tc05_fits(hd, page):
        raise Backend(f"attn_prefill_tc05: head size {hd} / page {page} not taken (64 or 128; page 64)")
    if not q.is_contiguous() or q.numel() != q.shape[0] * nh * hd:
        raise Backend("attn_prefill_tc05 takes contiguous queries [tokens, heads * head size]")
    _check(_fn("tc05", "esp_attn_prefill_tc05")(
        _ptr(q, torch.bfloat16, "q"), q.shape[0], _ptr(k_cache, torch.bfloat16), _ptr(v_cache, torch.bfloat16),
        _ptr(out, torch.bfloat16), _ptr(tile_seq, torch.int32), _ptr(tile_first, torch.int32),
        _ptr(seq_start, torch.int32), _ptr(seq_past, torch.int32), _ptr(block_table, torch.int32),
        block_table.shape[1], k_cache.shape[0], page, tile_seq.shape[0], nh, nkv, hd, float(scale), sink_flag, sink_ptr,
        int(window or 0), int(chunk or 0), _ptr(status, torch.int32), _stream()), "attn_prefill_tc05")


def gather_rows(src, rows, out):
    """out[r] = src[rows[r]] for bfloat16 rows (width a multiple of 8)."""
    _check(_fn("core", "esp_gather_rows")(_ptr(src, torch.bfloat16, "src"), _ptr(rows, torch.int32, "rows"),
                                          _ptr(out, torch.bfloat16, "out"), out.shape[0], src.shape[1], _stream()),
           "gather_rows")


TC05_TILE_ROWS = 256


# Which tensor-memory products run on pairs of CTAs (tcgen05 cta_group::2: one MMA of 256 weight rows, each CTA of
# the pair loads its own 128 and half of the token rows): "0" none, "grouped", "dense" or "all".  Measured at the
# A2.7B sizes, 2,048 tokens: grouped gate/up 143.5 -> 133.8 us, grouped down 86.9 -> 82.8 us, dense fused SwiGLU
# 78.4 -> 74.7 us, dense plain 42.3 -> 43.9 us; results are equal bit for bit.
TC05_PAIR = os.environ.get("ESP_B200_TC05_PAIR", "all")
TC05_PAIR_ROWS_PER_GROUP = 32          # grouped products with fewer rows per group than this run on single CTAs


def gemm_tc05(a, w, c, status, swiglu=False, row_scale=None, tiles=None, rows=None, tile_rows=None, pair=None,
              max_ctas=0):
    """TMA + tcgen05 product for many rows.  a [rows, K] bfloat16 contiguous; w [N, K] or [G, N, K]
    bfloat16.  Plain: c float32 [rows, N] = scale * a @ w[g].T.  swiglu: w rows are [gate; up] and c is
    bfloat16 [rows, I].  Grouped: ``tiles`` = (tile_group, tile_row0, tile_count, n_tiles) from moe_permute,
    ``tile_rows`` the most rows a tile has (128 or 256; TC05_TILE_ROWS when not given).  ``max_ctas`` > 0:
    the kernel takes at most that many SMs, so that kernels of another stream find room beside it."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not a.is_contiguous() or not w.is_contiguous():
        raise Backend("gemm_tc05 takes contiguous bfloat16 operands")
    if w.dim() == 3:
        groups, wn, k = w.shape
    else:
        groups = 1
        wn, k = w.shape
    n = wn // 2 if swiglu else wn
    m = a.shape[0] if rows is None else rows
    if a.shape[1] != k or c.shape[1] != n or k % 8 != 0 or c.stride(1) != 1:
        raise Backend(f"gemm_tc05: shapes disagree or K is no multiple of 8: a {tuple(a.shape)}, w {tuple(w.shape)}, "
                      f"c {tuple(c.shape)}")
    if c.dtype != (torch.bfloat16 if swiglu else torch.float32):
        raise Backend("gemm_tc05: the plain product writes float32, the SwiGLU product bfloat16")
    grouped = tiles is not None
    tile_rows = TC05_TILE_ROWS if tile_rows is None else tile_rows
    if pair is None:
        pair = TC05_PAIR == "all" or TC05_PAIR == ("grouped" if grouped else "dense")
        # narrow token tiles gain nothing from sharing them between two CTAs, and one MMA thread per CTA issues
        # more per SM than one per pair: a prompt of 256 tokens (17 rows an expert) 7.45 -> 6.91 ms on single
        # CTAs, one of 1,024 tokens (68 rows an expert) 8.11 -> 8.55 ms
        if grouped and m < TC05_PAIR_ROWS_PER_GROUP * groups:
            pair = False
    code = _fn("tc05", "esp_gemm_tc05")(
        a.data_ptr(), m, w.data_ptr(), groups, wn, _ptr(row_scale, torch.float32, "row_scale"), c.data_ptr(),
        c.stride(0), _ptr(tiles[0], torch.int32) if grouped else None,
        _ptr(tiles[1], torch.int32) if grouped else None, _ptr(tiles[2], torch.int32) if grouped else None,
        _ptr(tiles[3], torch.int32) if grouped else None, tiles[0].shape[0] if grouped else 0,
        tile_rows if grouped else 0, m, n, k,
        1 if swiglu else 0, 1 if pair else 0, int(max_ctas), _ptr(status, torch.int32), _stream())
    _check(code, "gemm_tc05")


def wait_probe(polls: int, status):
    """Runs the library's bounded wait on a barrier that nothing completes: after ``polls`` tries the
    kernel sets the wait-expired bit of ``status`` and returns."""
    _check(_fn("tc05", "esp_wait_probe")(int(polls), _ptr(status, torch.int32, "status"), _stream()), "wait_probe")


# ---------------------------------------------------------------------------
# recurrent layers and latent attention (library "mixers")
# ---------------------------------------------------------------------------
def _rows_ld(t, what):
    """(pointer, row stride) of a float32 matrix whose rows may be parts of wider rows."""
    if t is None:
        return None, 0
    if not t.is_cuda or t.dtype != torch.float32 or t.dim() != 2 or t.stride(1) != 1:
        raise Backend(f"{what} must be a float32 matrix on the GPU with unit column stride")
    return t.data_ptr(), t.stride(0)


def token_shift_mix(h, prev_state, tok_seq, seq_start, seq_slot, mu, out):
    """out[m, n] = h[n] + (prev(n) - h[n]) * mu[m]: prev(n) is the row before n in its sequence, or, for the
    first row of the sequence in this step, the sequence's row of ``prev_state`` (float32 [slots, width], rows
    may be parts of wider rows)."""
    n, width = h.shape
    if tuple(out.shape) != (mu.shape[0], n, width) or prev_state.shape[1] != width or prev_state.stride(1) != 1:
        raise Backend("token_shift_mix: shapes disagree")
    _check(_fn("mixers", "esp_token_shift_mix")(
        _ptr(h, FLOATS, "h"), _is_bf16(h), prev_state.data_ptr(), prev_state.stride(0), _ptr(tok_seq, torch.int32),
        _ptr(seq_start, torch.int32), _ptr(seq_slot, torch.int32), _ptr(mu, torch.float32, "mu"), _ptr(out, h.dtype, "out"),
        mu.shape[0], n, width, _stream()), "token_shift_mix")


def token_shift_keep(h, prev_state, seq_start, seq_slot, n_seqs: int):
    """prev_state[slot of sequence b] = the last row that b brings in this step."""
    width = h.shape[1]
    if prev_state.shape[1] != width or prev_state.stride(1) != 1 or prev_state.dtype != torch.float32:
        raise Backend("token_shift_keep: the state rows must be float32 of the rows' width")
    _check(_fn("mixers", "esp_token_shift_keep")(
        _ptr(h, FLOATS, "h"), _is_bf16(h), prev_state.data_ptr(), prev_state.stride(0), _ptr(seq_start, torch.int32),
        _ptr(seq_slot, torch.int32), int(n_seqs), width, _stream()), "token_shift_keep")


SCAN_DECAY_BONUS = 0          # d = exp(-exp(g + bias)), the current token weighted by ``bonus``, output before the update
SCAN_LOWER_SIGMOID = 1        # d = lower + (1 - lower) sigmoid(g + bias), k = 1 - d, q = silu(q), output after the update
SCAN_SCALAR_DECAY = 2         # with ready=True: g holds one ready-made decay per head and token [rows, heads]; output after the update
SCAN_MAX_KEY_DIM = 256


def gate_prepare(mode, q, g, gate_bias, lower, q_out, k_out, d_out):
    """The gates of many rows ahead of ``gated_scan(..., ready=True)``: d_out (and for SCAN_LOWER_SIGMOID q_out = silu(q)
    and k_out = 1 - d), float32 [rows, heads * key_dim], from the projections' raw outputs.  The same operations as
    the recurrence applies when it makes the gates itself: equal bits."""
    (pq, ldq), (pg, ldg) = _rows_ld(q, "q"), _rows_ld(g, "g")
    _check(_fn("mixers", "esp_gate_prepare")(
        int(mode), pq, ldq, pg, ldg, _ptr(gate_bias, torch.float32, "gate_bias"), _ptr(lower, torch.float32, "lower"),
        _ptr(q_out, torch.float32, "q_out"), _ptr(k_out, torch.float32, "k_out"), _ptr(d_out, torch.float32, "d_out"),
        g.shape[0], g.shape[1], _stream()), "gate_prepare")


def gated_scan(mode, q, k, g, v, gate_bias, lower, bonus, state, seq_start, seq_slot, out, n_seqs, heads, key_dim, value_dim,
               ready=False):
    """The gated outer-product recurrence S_t = diag(d_t) S_(t-1) + k_t v_t^T per head with its output, over the
    runs of rows that the sequences bring (seq_start), from and to ``state`` (float32 [slots, >= heads * value_dim *
    key_dim], a head's block laid out [value_dim, key_dim]).  q, k, g: float32 [rows, heads * key_dim]; v: float32
    [rows, heads * value_dim]; out: float32 [rows, heads * value_dim].  All 32-bit.  ``ready``: q, k and g hold the
    query, the written key and the decay themselves (``gate_prepare`` made them)."""
    if key_dim > SCAN_MAX_KEY_DIM:
        raise Backend(f"gated_scan: {key_dim} key channels per head are beyond the {SCAN_MAX_KEY_DIM} this kernel takes")
    if state.dtype != torch.float32 or state.stride(1) != 1 or state.shape[1] < heads * key_dim * value_dim:
        raise Backend("gated_scan: the state rows are too short or not float32")
    (pq, ldq), (pk, ldk), (pg, ldg), (pv, ldv) = (_rows_ld(t, n) for t, n in ((q, "q"), (k, "k"), (g, "g"), (v, "v")))
    _check(_fn("mixers", "esp_gated_scan")(
        int(mode), 1 if ready else 0, pq, ldq, pk, ldk, pg, ldg, pv, ldv, _ptr(gate_bias, torch.float32, "gate_bias"),
        _ptr(lower, torch.float32, "lower"), _ptr(bonus, torch.float32, "bonus"), state.data_ptr(), state.stride(0),
        _ptr(seq_start, torch.int32), _ptr(seq_slot, torch.int32), _ptr(out, torch.float32, "out"), int(n_seqs), heads,
        key_dim, value_dim, _stream()), "gated_scan")


def head_rmsnorm_gate(o, weight, weight_head_stride, gate, y, heads, value_dim, eps, gate_sigmoid=False):
    """y[n, h] = o[n, h] / rms(o[n, h]) * weight[h * weight_head_stride + :] (* silu(gate[n, h]), or its sigmoid with
    ``gate_sigmoid``); o float32 [rows, heads * value_dim], gate float32 or None, y float32 or bfloat16."""
    pg, ldg = _rows_ld(gate, "gate")
    _check(_fn("mixers", "esp_head_rmsnorm_gate")(
        _ptr(o, torch.float32, "o"), _ptr(weight, torch.float32, "weight"), int(weight_head_stride), pg, ldg,
        _ptr(y, FLOATS, "y"), _is_bf16(y), o.shape[0], heads, value_dim, float(eps), 1 if gate_sigmoid else 0, _stream()),
        "head_rmsnorm_gate")


def latent_kv_store(d, norm_w, inv_freq, magnitude, rot_dims, tok_seq, tok_pos, block_table, pool, page, rank, rot, eps, status):
    """Rows of the latent cache from the down-projection's output d (float32 [rows, rank + rot]): the first
    ``rank`` channels RMS-normed times norm_w, the last ``rot`` rotated (the first rot_dims of them, in pairs
    (i, i + rot_dims/2), angle position * inv_freq[i], cos and sin times ``magnitude``).  pool: [pages, 1, page,
    rank + rot]."""
    if d.shape[1] != rank + rot or pool.shape[-1] != rank + rot:
        raise Backend("latent_kv_store: widths disagree")
    _check(_fn("mixers", "esp_latent_kv_store")(
        _ptr(d, torch.float32, "d"), _ptr(norm_w, torch.float32, "norm_w"), _ptr(inv_freq, torch.float32, "inv_freq"),
        float(magnitude), int(rot_dims), _ptr(tok_seq, torch.int32), _ptr(tok_pos, torch.int32),
        _ptr(block_table, torch.int32), block_table.shape[1], pool.shape[0], page, _ptr(pool, FLOATS, "pool"), _is_bf16(pool),
        d.shape[0], rank, rot, float(eps), _ptr(status, torch.int32), _stream()), "latent_kv_store")


def latent_q_rotate(q, inv_freq, magnitude, rot_dims, tok_pos, qx, heads, nope, rot, rank):
    """qx[n, h, rank:] = rotation of q[n, h, nope:] (q float32 [rows, heads * (nope + rot)]; qx [rows, heads *
    (rank + rot)])."""
    _check(_fn("mixers", "esp_latent_q_rotate")(
        _ptr(q, torch.float32, "q"), _ptr(inv_freq, torch.float32, "inv_freq"), float(magnitude), int(rot_dims),
        _ptr(tok_pos, torch.int32), _ptr(qx, FLOATS, "qx"), _is_bf16(qx), q.shape[0], heads, nope, rot, rank, _stream()),
        "latent_q_rotate")


def per_head_linear(a, lda, a_head, w, out, ldo, o_head, n_rows, heads, kin, nout):
    """out[n, h, :nout] = w[h] @ a[n, h, :kin] with w [heads, nout, kin]; element (n, h, i) of a lies at
    n * lda + h * a_head + i (out likewise), so both may be parts of wider rows."""
    if tuple(w.shape) != (heads, nout, kin) or kin * 8 * 4 > 48 * 1024:
        raise Backend(f"per_head_linear: weights {tuple(w.shape)} do not fit heads {heads}, {nout} x {kin}")
    code = {torch.float32: 0, torch.bfloat16: 1}
    # ``a`` may be a view of the leading columns of wider rows (its row stride is lda)
    if not a.is_cuda or a.dtype not in FLOATS or a.stride(-1) != 1 or (a.dim() == 2 and a.shape[0] > 1 and a.stride(0) != lda):
        raise Backend("per_head_linear: a must be rows of unit column stride whose row stride is lda")
    pa = a.data_ptr()
    _check(_fn("mixers", "esp_per_head_linear")(
        pa, code[a.dtype], int(lda), int(a_head), _ptr(w, FLOATS, "w"), code[w.dtype],
        _ptr(out, FLOATS, "out"), code[out.dtype], int(ldo), int(o_head), int(n_rows), heads, kin, nout, _stream()),
        "per_head_linear")


def attn_latent(qx, pool, out, tok_seq, tok_pos, block_table, page, heads, key_dim, value_dim, window, scale, status):
    """Attention of every head of every token over its sequence's cached rows (one row per position, shared by
    the heads): scores from the whole row (key_dim), values the row's first value_dim channels.  32-bit
    arithmetic; qx, pool and out share a dtype."""
    if pool.shape[-1] != key_dim or value_dim > 512:
        raise Backend(f"attn_latent: rows of {pool.shape[-1]} / values of {value_dim} channels not taken")
    _check(_fn("mixers", "esp_attn_latent")(
        _ptr(qx, FLOATS, "qx"), _ptr(pool, qx.dtype, "pool"), _ptr(out, qx.dtype, "out"), _is_bf16(qx),
        _ptr(tok_seq, torch.int32), _ptr(tok_pos, torch.int32), _ptr(block_table, torch.int32), block_table.shape[1],
        pool.shape[0], page, qx.shape[0], heads, key_dim, value_dim, int(window or 0), float(scale),
        _ptr(status, torch.int32), _stream()), "attn_latent")


ATTN_LATENT_MMA_ROWS = 32        # (token, head) rows of a tile of attn_latent_mma


def attn_latent_mma_heads(heads: int) -> int:
    """Heads of a tile: the power of two that holds all heads, at most the tile's rows."""
    hg = 1
    while hg < heads and hg < ATTN_LATENT_MMA_ROWS:
        hg *= 2
    return hg


def attn_latent_mma_fits(key_dim: int, value_dim: int, page: int) -> bool:
    smem = (2 * 64 + 32) * (key_dim + 8) * 2 + 32 * 72 * 2 + 8 * 32 * 4
    return page == 64 and key_dim % 16 == 0 and value_dim % 16 == 0 and value_dim <= min(512, key_dim) and smem <= 227 * 1024


def attn_latent_mma(qx, pool, out, tile_seq, tile_first, seq_start, seq_past, block_table, page, heads, key_dim, value_dim,
                    window, scale, status, n_splits=1, pages_per_split=0, part_o=None, part_ml=None):
    """attn_latent on the tensor cores (bfloat16).  tile_seq / tile_first list tiles of 32 / attn_latent_mma_heads(heads)
    new tokens of one sequence each.  n_splits > 1: the pages a tile sees are dealt to that many blocks,
    pages_per_split each, through the float32 scratch part_o [rows, heads, n_splits, value_dim] and part_ml [rows, heads,
    n_splits, 2]."""
    if not attn_latent_mma_fits(key_dim, value_dim, page) or pool.shape[-1] != key_dim:
        raise Backend(f"attn_latent_mma: rows of {key_dim} / values of {value_dim} channels / pages of {page} not taken")
    n = qx.shape[0]
    if n_splits > 1 and (part_o.numel() < n * heads * n_splits * value_dim or part_ml.numel() < n * heads * n_splits * 2):
        raise Backend("attn_latent_mma: scratch is too small")
    _check(_fn("bf16", "esp_attn_latent_mma")(
        _ptr(qx, torch.bfloat16, "qx"), _ptr(pool, torch.bfloat16, "pool"), _ptr(out, torch.bfloat16, "out"),
        _ptr(tile_seq, torch.int32), _ptr(tile_first, torch.int32), _ptr(seq_start, torch.int32), _ptr(seq_past, torch.int32),
        _ptr(block_table, torch.int32), block_table.shape[1], pool.shape[0], page, tile_seq.shape[0], n, heads,
        attn_latent_mma_heads(heads), key_dim, value_dim, int(window or 0), float(scale), int(n_splits), int(pages_per_split),
        _ptr(part_o, torch.float32), _ptr(part_ml, torch.float32), _ptr(status, torch.int32), _stream()), "attn_latent_mma")


# ---------------------------------------------------------------------------
# summed embeddings, norms around a sublayer, squared ReLU

def embed_sum(table, bigram, freq, ids, tok_seq, tok_pos, seq_start, seq_slot, prev_state, x, status, buckets=0, mul_prev=0,
              mul_cur=0, scale: float = 1.0):
    """x[n] = scale * table[ids[n]] + bigram[hash(previous token, token)] + sinusoid(position).  ``bigram``
    [buckets + 1, width] and ``freq`` (float32 [ceil(width / 2)]) may be None.  ``prev_state`` (int32 [slots]) holds
    every sequence's last token + 1 (0: none yet); it is read for a run's first token and left at the run's last."""
    n, width = x.shape
    if bigram is not None and (bigram.dtype != table.dtype or bigram.shape != (buckets + 1, width)):
        raise Backend("embed_sum: the bigram table must be [buckets + 1, width] in the token table's dtype")
    if freq is not None and freq.shape[0] * 2 < width:
        raise Backend("embed_sum: too few frequencies for the width")
    _check(_fn("core", "esp_embed_sum")(
        _ptr(table, FLOATS, "embedding table"), _ptr(bigram, FLOATS, "bigram table"), _is_bf16(table),
        _ptr(freq, torch.float32, "freq"), _ptr(ids, torch.int32, "ids"), _ptr(tok_seq, torch.int32), _ptr(tok_pos, torch.int32),
        _ptr(seq_start, torch.int32), _ptr(seq_slot, torch.int32), _ptr(prev_state, torch.int32, "prev_state"),
        _ptr(x, torch.float32, "x"), n, width, table.shape[0], int(buckets), int(mul_prev), int(mul_cur), float(scale),
        _ptr(status, torch.int32), _stream()), "embed_sum")


def norm_add_rmsnorm(x, y, gamma_y, eps_y, gamma, h, eps, rows=None, write_x=True, h32=None):
    """x (+)= rmsnorm(y) * gamma_y, then h = rmsnorm(x) * gamma, in one launch; all float32 but h.  ``h`` None: the
    add alone.  ``x`` None: h32 = rmsnorm(y) * gamma_y and nothing else."""
    width = y.shape[1]
    if x is None:
        n_rows = h32.shape[0]
    else:
        n_rows = h.shape[0] if h is not None else x.shape[0]
    _check(_fn("core", "esp_norm_add_rmsnorm")(
        _ptr(x, torch.float32, "x"), _ptr(y, torch.float32, "y"), _ptr(gamma_y, torch.float32, "gamma_y"), float(eps_y),
        _ptr(gamma, torch.float32, "gamma"), _ptr(rows, torch.int32, "rows"), _ptr(h, FLOATS, "h"),
        _is_bf16(h) if h is not None else 0, _ptr(h32, torch.float32, "h32"), n_rows, width, float(eps),
        1 if write_x else 0, _stream()), "norm_add_rmsnorm")


def relu2(z, act, row_scale=None):
    """act[m, :] = max(z[m, :] * row_scale[m], 0)^2; z float32 [M, W], act float32 or bfloat16."""
    rows, width = act.shape
    if z.shape[0] < rows or z.shape[1] != width:
        raise Backend("relu2: shapes disagree")
    _check(_fn("core", "esp_relu2")(_ptr(z, torch.float32, "z"), _ptr(row_scale, torch.float32, "row_scale"),
                                    _ptr(act, FLOATS, "act"), _is_bf16(act), rows, width, _stream()), "relu2")


def qknorm_kvwrite(qkv, bias, q_w, k_w, eps, temp_coef, temp_every, tok_seq, tok_pos, q_out, k_cache, v_cache, block_table,
                   page, nh, nkv, hd, vd, write_kv, status):
    """Bias, RMS norm per query and key head (weights q_w, k_w of hd numbers, None: no norm), the queries' factor
    1 + temp_coef ln(floor((p + 1) / temp_every) + 1) (temp_every 0: none), and the write of keys [pages, nkv, page,
    hd] and values [pages, nkv, page, vd] into the paged cache.  qkv float32 [N, nh*hd + nkv*hd + nkv*vd]."""
    n = qkv.shape[0]
    if qkv.shape[1] != (nh + nkv) * hd + nkv * vd:
        raise Backend("qknorm_kvwrite: qkv width disagrees with the head counts")
    _check(_fn("core", "esp_qknorm_kvwrite")(
        _ptr(qkv, torch.float32, "qkv"), _ptr(bias, torch.float32, "bias"), _ptr(q_w, torch.float32), _ptr(k_w, torch.float32),
        float(eps), float(temp_coef), int(temp_every), _ptr(tok_seq, torch.int32), _ptr(tok_pos, torch.int32),
        _ptr(q_out, FLOATS, "q_out"), _ptr(k_cache, q_out.dtype), _ptr(v_cache, q_out.dtype), _is_bf16(q_out),
        _ptr(block_table, torch.int32), block_table.shape[1], k_cache.shape[0], page, n, nh, nkv, hd, vd,
        1 if write_kv else 0, _ptr(status, torch.int32), _stream()), "qknorm_kvwrite")


# ---------------------------------------------------------------------------
# matrix memory and gated diagonal recurrence (library ``mixers``)

def matrix_memory_prepare(v, gi, gf, ld, bias_i, bias_f, cap, m_state, seq_start, seq_slot, v_out, keep_take_m, n_seqs, heads,
                          value_dim, value_cols):
    """Gates of a matrix memory with exponential gating: v, gi, gf are views into one float32 projection with row
    stride ``ld``; m_state float32 [slots, heads] (a view with its slot stride).  keep_take_m float32 [3, N, heads]
    receives the decay exp(f + m' - m), the input weight exp(i - m) and the running maximum m of every token and head
    (``gated_scan(SCAN_SCALAR_DECAY, ...)`` takes the first as its decays, ``matrix_memory_finish`` reads the last);
    v_out float32 [N, heads * value_cols] = input weight * [v, 1, 0 ...]."""
    for t in (v, gi, gf):
        if t.dtype != torch.float32 or t.stride(-1) != 1 or t.stride(0) != ld:
            raise Backend("matrix_memory_prepare: the projections must be float32 views of rows with stride ld")
    if tuple(keep_take_m.shape) != (3, v.shape[0], heads):
        raise Backend("matrix_memory_prepare: keep_take_m must be [3, rows, heads]")
    _check(_fn("mixers", "esp_matrix_memory_prepare")(
        v.data_ptr(), gi.data_ptr(), gf.data_ptr(), int(ld), _ptr(bias_i, torch.float32), _ptr(bias_f, torch.float32),
        float(cap), m_state.data_ptr(), m_state.stride(0), _ptr(seq_start, torch.int32), _ptr(seq_slot, torch.int32),
        _ptr(v_out, torch.float32), _ptr(keep_take_m, torch.float32), v.shape[0], n_seqs, heads, value_dim, value_cols,
        _stream()), "matrix_memory_prepare")


def matrix_memory_finish(o, m, w, gate, y, heads, value_dim, value_cols, eps, floor_eps, q_scale=1.0):
    """y[n, h, :] = unit-rms(q_scale o[n, h, :value_dim] / (max(|q_scale o[n, h, value_dim]|, exp(-m[n, h])) + floor_eps))
    * w[h] * sigmoid(gate[n, h, :]); o float32 [N, heads*value_cols], gate a float32 view [N, heads*value_dim] or None."""
    n = o.shape[0]
    if gate is not None and (gate.dtype != torch.float32 or gate.stride(-1) != 1):
        raise Backend("matrix_memory_finish: the gate must be a float32 view with unit column stride")
    _check(_fn("mixers", "esp_matrix_memory_finish")(
        _ptr(o, torch.float32, "o"), _ptr(m, torch.float32, "m"), _ptr(w, torch.float32, "w"),
        gate.data_ptr() if gate is not None else None, gate.stride(0) if gate is not None else 0, _ptr(y, FLOATS, "y"),
        _is_bf16(y), n, heads, value_dim, value_cols, float(eps), float(floor_eps), float(q_scale), _stream()),
        "matrix_memory_finish")


CONV_MAX_TAPS = 16


def conv_branches(proj, bias_y, bias_x, conv_w, conv_b, conv_state, tok_seq, seq_start, seq_slot, gate_out, u32, u_act,
                  n_seqs, channels, taps):
    """proj float32 [N, 2C] (gate branch, then input branch).  gate_out = gelu_tanh(proj_y + bias_y); u = causal
    convolution of (proj_x + bias_x) over ``taps`` positions per channel (conv_w [C, taps], last column the token's
    own; conv_state float32 [slots, (taps - 1) * C] (a view with its slot stride) holds a sequence's last taps - 1
    inputs and is brought up to date); u32 float32, u_act in the activation dtype."""
    if taps > CONV_MAX_TAPS:
        raise Backend(f"conv_branches: {taps} taps are beyond the {CONV_MAX_TAPS} this kernel takes")
    _check(_fn("mixers", "esp_conv_branches")(
        _ptr(proj, torch.float32, "proj"), _ptr(bias_y, torch.float32), _ptr(bias_x, torch.float32),
        _ptr(conv_w, torch.float32), _ptr(conv_b, torch.float32), conv_state.data_ptr(), conv_state.stride(0),
        _ptr(tok_seq, torch.int32), _ptr(seq_start, torch.int32), _ptr(seq_slot, torch.int32),
        _ptr(gate_out, torch.float32), _ptr(u32, torch.float32), _ptr(u_act, FLOATS), _is_bf16(u_act), proj.shape[0],
        n_seqs, channels, taps, _stream()), "conv_branches")


def diag_scan(gates, bias_r, bias_i, lam, decay_scale, u, gate, state, seq_start, seq_slot, out, n_seqs, channels, blocks):
    """S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t, a_t = exp(-decay_scale sigmoid(raw_r + bias_r) softplus(lam)),
    i_t = sigmoid(raw_i + bias_i); out = S_t * gate.  gates float32 [N, blocks, 2, C / blocks] (overwritten with the
    recurrence's coefficients); state float32 [slots, C] (a view with its slot stride)."""
    _check(_fn("mixers", "esp_diag_scan")(
        _ptr(gates, torch.float32, "gates"), _ptr(bias_r, torch.float32), _ptr(bias_i, torch.float32),
        _ptr(lam, torch.float32), float(decay_scale), _ptr(u, torch.float32), _ptr(gate, torch.float32), state.data_ptr(),
        state.stride(0), _ptr(seq_start, torch.int32), _ptr(seq_slot, torch.int32), _ptr(out, FLOATS), _is_bf16(out),
        gates.shape[0], n_seqs, channels, blocks, _stream()), "diag_scan")


# ---------------------------------------------------------------------------
HC_MAX_STREAMS = 8


def hc_step(streams, h, gamma, eps, x0=None, y=None, mix=None, out_w=None, read_w=None, rows=None, u_out=None,
            write_streams=True):
    """What lies between two sublayers of a layer over several copies of the residual stream (``streams`` float32
    [S, rows, width]): with ``y`` the write of the sublayer that ran, new_t = sum_s mix[s, t] old_s + out_w[t] y (the old
    copies all equal ``x0`` when that is given); then the read of the next one, u = sum_s read_w[s] new_s (the plain sum
    without ``read_w``), ``h`` = rmsnorm(u) * gamma in its dtype (None: no norm), ``u_out`` = u.  ``rows`` (int32)
    selects rows; h has one row per selected row."""
    n_streams, n_total, width = streams.shape
    if n_streams > HC_MAX_STREAMS:
        raise Backend(f"hc_step: {n_streams} streams are beyond the {HC_MAX_STREAMS} this kernel takes")
    n_rows = rows.shape[0] if rows is not None else n_total
    if h is not None and (h.shape[0] != n_rows or h.shape[1] != width):
        raise Backend("hc_step: h does not fit the rows")
    _check(_fn("core", "esp_hc_step")(
        _ptr(streams, torch.float32, "streams"), _ptr(x0, torch.float32, "x0"), _ptr(y, torch.float32, "y"),
        _ptr(mix, torch.float32, "mix"), _ptr(out_w, torch.float32, "out_w"), _ptr(read_w, torch.float32, "read_w"),
        _ptr(gamma, torch.float32, "gamma"), _ptr(rows, torch.int32, "rows"), _ptr(h, FLOATS, "h"),
        _is_bf16(h) if h is not None else 0, _ptr(u_out, torch.float32, "u_out"), n_streams, n_total * width, n_rows, width,
        float(eps), 1 if write_streams else 0, _stream()), "hc_step")


def glu_clamped(gu, act, limit, alpha, shift):
    """act = g sigmoid(alpha g) (u + shift), g = min(gu[:, :I], limit), u = clamp(gu[:, I:], -limit, limit); gu float32
    [rows, 2I], act float32 or bfloat16 [rows, I]."""
    rows, inter = act.shape
    if tuple(gu.shape) != (rows, 2 * inter):
        raise Backend("glu_clamped: shapes disagree")
    _check(_fn("core", "esp_glu_clamped")(_ptr(gu, torch.float32, "gu"), _ptr(act, FLOATS, "act"), _is_bf16(act), rows, inter,
                                           float(limit), float(alpha), float(shift), _stream()), "glu_clamped")


def weighted_sum(out, parts, scales):
    """out = sum_i scales[i] * parts[i] over up to four float32 tensors of out's size, added in the order given."""
    if not 1 <= len(parts) <= 4 or len(scales) != len(parts):
        raise Backend("weighted_sum: one to four parts with a scale each")
    ptrs = [_ptr(p, torch.float32, "part") for p in parts] + [None] * (4 - len(parts))
    sc = [float(v) for v in scales] + [0.0] * (4 - len(parts))
    if any(p.numel() != out.numel() for p in parts):
        raise Backend("weighted_sum: sizes disagree")
    _check(_fn("core", "esp_weighted_sum")(_ptr(out, torch.float32, "out"), *ptrs, *sc, out.numel(), _stream()), "weighted_sum")


def cast_cols(src, dst):
    """dst = src in dst's dtype; src float32 rows that may be parts of wider rows."""
    p, ld = _rows_ld(src, "src")
    if tuple(dst.shape) != tuple(src.shape):
        raise Backend("cast_cols: shapes disagree")
    _check(_fn("core", "esp_cast_cols")(p, ld, _ptr(dst, FLOATS, "dst"), _is_bf16(dst), src.shape[0], src.shape[1], _stream()),
           "cast_cols")


def widenorm_rope_kvwrite(qkv, q_w, k_w, eps, inv_freq, rot, v_scale, tok_seq, tok_pos, q_out, k_cache, v_cache, block_table,
                          page, nh, nkv, hd, vd, write_kv, status):
    """Queries and keys normed over their whole projection (weights q_w [nh * hd], k_w [nkv * hd]), the first ``rot``
    channels of every head rotated by position * inv_freq, values times v_scale; queries to q_out, keys and values to the
    paged cache.  qkv float32 [rows, nh * hd + nkv * hd + nkv * vd]."""
    if qkv.shape[1] != nh * hd + nkv * hd + nkv * vd:
        raise Backend("widenorm_rope_kvwrite: the projection's width does not fit the head sizes")
    if rot and (inv_freq is None or inv_freq.shape[0] < rot // 2):
        raise Backend("widenorm_rope_kvwrite: too few frequencies")
    _check(_fn("core", "esp_widenorm_rope_kvwrite")(
        _ptr(qkv, torch.float32, "qkv"), _ptr(q_w, torch.float32, "q_w"), _ptr(k_w, torch.float32, "k_w"), float(eps),
        _ptr(inv_freq, torch.float32, "inv_freq"), int(rot), float(v_scale), _ptr(tok_seq, torch.int32),
        _ptr(tok_pos, torch.int32), _ptr(q_out, FLOATS, "q_out"), _ptr(k_cache, q_out.dtype, "k_cache"),
        _ptr(v_cache, q_out.dtype, "v_cache"), _is_bf16(q_out), _ptr(block_table, torch.int32), block_table.shape[1],
        k_cache.shape[0], page, qkv.shape[0], nh, nkv, hd, vd, 1 if write_kv else 0, _ptr(status, torch.int32), _stream()),
        "widenorm_rope_kvwrite")


def delta_scan(q, k, d, v, beta, state, seq_start, seq_slot, out, n_seqs, heads, kv_heads, key_dim, value_dim):
    """The delta rule with a decay per key channel over the runs of rows that the sequences bring, from and to ``state``
    (float32 [slots, >= heads * value_dim * key_dim], a head's block laid out [value_dim, key_dim]): S <- diag(d) S;
    u = beta (v - S^T k); S <- S + k u^T; o = S^T q.  q, k: float32 [rows, kv_heads * key_dim]; d: [rows, heads * key_dim];
    v, out: [rows, heads * value_dim]; beta: [rows, heads].  All 32-bit."""
    if key_dim > SCAN_MAX_KEY_DIM:
        raise Backend(f"delta_scan: {key_dim} key channels per head are beyond the {SCAN_MAX_KEY_DIM} this kernel takes")
    if state.dtype != torch.float32 or state.stride(1) != 1 or state.shape[1] < heads * key_dim * value_dim:
        raise Backend("delta_scan: the state rows are too short or not float32")
    (pq, ldq), (pk, ldk), (pd, ldd), (pv, ldv) = (_rows_ld(t, n) for t, n in ((q, "q"), (k, "k"), (d, "d"), (v, "v")))
    _check(_fn("mixers", "esp_delta_scan")(
        pq, ldq, pk, ldk, pd, ldd, pv, ldv, _ptr(beta, torch.float32, "beta"), state.data_ptr(), state.stride(0),
        _ptr(seq_start, torch.int32), _ptr(seq_slot, torch.int32), _ptr(out, torch.float32, "out"), int(n_seqs), heads,
        kv_heads, key_dim, value_dim, _stream()), "delta_scan")


def delta_prepare(qk, kv_heads, key_dim, unit_eps, q_scale, raw, decay, dt_bias, a_log, b_raw, beta, heads):
    """The kv_heads query heads at column 0 of ``qk`` and the key heads behind them become unit vectors in place
    (queries times q_scale); decay = exp(-exp(a_log[h]) softplus(raw + dt_bias)) (float32 [rows, heads * key_dim], raw
    rows that may be parts of wider rows); beta = sigmoid(b_raw)."""
    (pqk, ldqk), (pb, ldb), (praw, ldraw) = _rows_ld(qk, "qk"), _rows_ld(b_raw, "b_raw"), _rows_ld(raw, "raw")
    _check(_fn("mixers", "esp_delta_prepare")(
        pqk, ldqk, kv_heads, key_dim, float(unit_eps), float(q_scale), praw, ldraw, _ptr(decay, torch.float32, "decay"),
        _ptr(dt_bias, torch.float32, "dt_bias"), _ptr(a_log, torch.float32, "a_log"), pb, ldb,
        _ptr(beta, torch.float32, "beta"), heads, qk.shape[0], _stream()), "delta_prepare")


def channel_decay_prepare(z, bias, tau, q, q_scale, q_out):
    """In place z = sigmoid(z + bias)^(1 / tau); q_out = q * q_scale (q float32 rows that may be parts of wider rows)."""
    pq, ldq = _rows_ld(q, "q")
    _check(_fn("mixers", "esp_channel_decay_prepare")(
        _ptr(z, torch.float32, "z"), _ptr(bias, torch.float32, "bias"), float(tau), pq, ldq, float(q_scale),
        _ptr(q_out, torch.float32, "q_out"), z.shape[0], z.shape[1], _stream()), "channel_decay_prepare")


def causal_conv(x, w, conv_state, tok_seq, seq_start, seq_slot, y, n_seqs, taps, silu=True, bias=None):
    """y = act(causal convolution of x over ``taps`` positions per channel (+ bias float32 [C])) within every sequence (w float32 [C, taps],
    last column the token's own); conv_state float32 [slots, (taps - 1) * C] (a view with its slot stride) holds a
    sequence's last taps - 1 inputs and is brought up to date.  x float32 rows that may be parts of wider rows."""
    if taps > CONV_MAX_TAPS:
        raise Backend(f"causal_conv: {taps} taps are beyond the {CONV_MAX_TAPS} this kernel takes")
    px, ldx = _rows_ld(x, "x")
    channels = x.shape[1]
    if tuple(y.shape) != tuple(x.shape) or tuple(w.shape) != (channels, taps):
        raise Backend("causal_conv: shapes disagree")
    _check(_fn("mixers", "esp_causal_conv")(
        px, ldx, _ptr(w, torch.float32, "w"), _ptr(bias, torch.float32, "bias"),
        conv_state.data_ptr() if conv_state is not None else None,
        conv_state.stride(0) if conv_state is not None else 0, _ptr(tok_seq, torch.int32), _ptr(seq_start, torch.int32),
        _ptr(seq_slot, torch.int32), _ptr(y, torch.float32, "y"), x.shape[0], int(n_seqs), channels, taps, 1 if silu else 0,
        _stream()), "causal_conv")


# ---------------------------------------------------------------------------
# selective scan, a scalar gate per head, neighbour-pair rotation with unit heads and blended values

SELECTIVE_MAX_STATE = 512


def selective_scan(x, dt_raw, bc, z, a_log, d_skip, state, seq_start, seq_slot, y, n_seqs, channels, n_state):
    """The selective scan over the runs of rows that the sequences bring, from and to ``state`` (float32 [slots, >=
    channels * n_state], a channel's entries side by side): dt = softplus(dt_raw); S <- exp(-dt exp(a_log)) S + dt x B;
    y = (S . C + d_skip x) silu(z).  x, dt_raw, z: float32 [rows, channels] (may be parts of wider rows); bc: float32
    [rows, 2 * n_state], B then C; y: [rows, channels] float32 or bfloat16.  All arithmetic 32-bit."""
    if n_state > SELECTIVE_MAX_STATE:
        raise Backend(f"selective_scan: {n_state} state entries a channel are beyond the {SELECTIVE_MAX_STATE} this kernel takes")
    if state.dtype != torch.float32 or state.stride(1) != 1 or state.shape[1] < channels * n_state:
        raise Backend("selective_scan: the state rows are too short or not float32")
    if tuple(a_log.shape) != (channels, n_state) or bc.shape[1] != 2 * n_state or tuple(y.shape) != (x.shape[0], channels):
        raise Backend("selective_scan: shapes disagree")
    (px, ldx), (pdt, lddt), (pbc, ldbc), (pz, ldz) = (_rows_ld(t, n) for t, n in ((x, "x"), (dt_raw, "dt_raw"), (bc, "bc"), (z, "z")))
    _check(_fn("mixers", "esp_selective_scan")(
        px, ldx, pdt, lddt, pbc, ldbc, pz, ldz, _ptr(a_log, torch.float32, "a_log"), _ptr(d_skip, torch.float32, "d_skip"),
        state.data_ptr(), state.stride(0), _ptr(seq_start, torch.int32), _ptr(seq_slot, torch.int32), _ptr(y, FLOATS, "y"),
        _is_bf16(y), int(n_seqs), int(channels), int(n_state), _stream()), "selective_scan")


def head_scalar_gate(o, gate, y, heads, value_dim):
    """y[n, h, :] = o[n, h, :] * sigmoid(gate[n, h]); o float32 or bfloat16 [rows, heads * value_dim], gate float32
    [rows, heads] (may be part of wider rows), y float32 or bfloat16."""
    pg, ldg = _rows_ld(gate, "gate")
    if tuple(y.shape) != tuple(o.shape) or o.shape[1] != heads * value_dim:
        raise Backend("head_scalar_gate: shapes disagree")
    _check(_fn("mixers", "esp_head_scalar_gate")(
        _ptr(o, FLOATS, "o"), _is_bf16(o), pg, ldg, _ptr(y, FLOATS, "y"), _is_bf16(y), o.shape[0], heads, value_dim, _stream()),
        "head_scalar_gate")


def heads_to_pages(k, v, tok_seq, tok_pos, table, k_pool, v_pool, page, heads, key_dim, value_dim, status):
    """Keys float32 [rows, heads * key_dim] and values float32 [rows, heads * value_dim] (may be parts of wider rows) into
    the pools k_pool [pages, heads, page, key_dim] and v_pool [pages, heads, page, value_dim] at every token's place
    (``table`` int32 [sequences, stride]: the pages of each sequence).  Sizes are multiples of four."""
    (pk, ldk), (pv, ldv) = _rows_ld(k, "k"), _rows_ld(v, "v")
    if k.shape[1] != heads * key_dim or v.shape[1] != heads * value_dim or k_pool.dtype != v_pool.dtype:
        raise Backend("heads_to_pages: shapes disagree")
    _check(_fn("mixers", "esp_heads_to_pages")(
        pk, ldk, pv, ldv, _ptr(tok_seq, torch.int32), _ptr(tok_pos, torch.int32), _ptr(table, torch.int32), table.shape[1],
        k_pool.shape[0], page, _ptr(k_pool, FLOATS, "k_pool"), _ptr(v_pool, FLOATS, "v_pool"), _is_bf16(k_pool), k.shape[0],
        heads, key_dim, value_dim, _ptr(status, torch.int32), _stream()), "heads_to_pages")


def pair_rope_unitnorm_kvwrite(qkv, bias, inv_freq, rot, eps, unit_norm, v_shared, blend_mode, blend, tok_seq, tok_pos, q_out,
                               k_cache, v_cache, block_table, page, nh, nkv, hd, vd, write_kv, status):
    """Bias, rotation of neighbouring channel pairs (2i with 2i + 1) of the first ``rot`` channels of every query and key
    head by position * inv_freq[i], every head then divided by its root mean square (``unit_norm``), values copied to
    (blend_mode 1) or blended with (blend_mode 2: (1 - blend) v + blend v_shared, ``blend`` a float32 tensor of one
    element on the device) the float32 rows v_shared [rows, nkv * vd]; queries to q_out, keys and values to the paged
    cache.  qkv float32 [rows, nh * hd + nkv * hd + nkv * vd]."""
    if qkv.shape[1] != nh * hd + nkv * hd + nkv * vd:
        raise Backend("pair_rope_unitnorm_kvwrite: the projection's width does not fit the head sizes")
    if rot and (inv_freq is None or inv_freq.shape[0] < rot // 2):
        raise Backend("pair_rope_unitnorm_kvwrite: too few frequencies")
    if blend_mode and (v_shared is None or v_shared.numel() < qkv.shape[0] * nkv * vd):
        raise Backend("pair_rope_unitnorm_kvwrite: the shared value rows are missing or too small")
    _check(_fn("core", "esp_pair_rope_unitnorm_kvwrite")(
        _ptr(qkv, torch.float32, "qkv"), _ptr(bias, torch.float32, "bias"), _ptr(inv_freq, torch.float32, "inv_freq"), int(rot),
        float(eps), 1 if unit_norm else 0, _ptr(v_shared, torch.float32, "v_shared"), int(blend_mode),
        _ptr(blend, torch.float32, "blend"), _ptr(tok_seq, torch.int32), _ptr(tok_pos, torch.int32), _ptr(q_out, FLOATS, "q_out"),
        _ptr(k_cache, q_out.dtype, "k_cache"), _ptr(v_cache, q_out.dtype, "v_cache"), _is_bf16(q_out),
        _ptr(block_table, torch.int32), block_table.shape[1], k_cache.shape[0], page, qkv.shape[0], nh, nkv, hd, vd,
        1 if write_kv else 0, _ptr(status, torch.int32), _stream()), "pair_rope_unitnorm_kvwrite")
