"""Python face of the sm_100a kernels: argument checks, then the launch.

Every function takes torch tensors that live on the CUDA device, checks types,
shapes and contiguity on the host, and launches on torch's current stream, so
the launches can be captured into a CUDA graph with everything else.  There is
no CPU implementation and no library fallback behind these calls; a tensor on
another device is an error.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_double, c_float, c_int, c_longlong, c_ulonglong, c_void_p
from typing import Optional

import torch

from . import csrc

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}


class KernelError(RuntimeError):
    """A launcher refused its arguments or the launch failed."""


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DT[dt]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16, not {dt}") from None


def _ptr(t: Optional[torch.Tensor]) -> int:
    """The address for a ``c_void_p`` parameter (ctypes takes the integer as it is; None is NULL)."""
    return 0 if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    """The current stream's handle on the current device.  (Asked of torch's C layer directly: a
    launcher is called hundreds of times a step, and ``torch.cuda.current_stream()`` builds a
    Python object each time.)"""
    if _raw_stream is None or _raw_device is None:
        return torch.cuda.current_stream().cuda_stream
    return _raw_stream(_raw_device())


def _need(t: torch.Tensor, what: str, dtype=None, ndim=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{what} must be on the CUDA device (it is on {t.device}); there is no CPU path")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{what} must be {dtype}, not {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise KernelError(f"{what} must have {ndim} dimensions, not {t.dim()}")


def _rows_contiguous(t: torch.Tensor, what: str) -> int:
    """Row stride of a 2-D tensor whose rows are dense."""
    if t.dim() != 2 or t.stride(1) != 1 or t.stride(0) < t.shape[1]:
        raise KernelError(f"{what} must be 2-D with dense rows (shape {tuple(t.shape)}, strides {t.stride()})")
    return t.stride(0)


_prototyped = set()


class KernelTimes:
    """Device time of every launcher of this package by kernel class, for as long as the context
    lasts: a CUDA event before and one after each call (the launches then run one after the other
    as usual, but a kernel that would overlap the one ahead of it through programmatic dependent
    launch is still charged its whole length: the figures are shares, not a step's time; captured
    graphs hide their kernels, so the runner steps eagerly meanwhile).

        with ops.KernelTimes() as kt:
            runner.step(...)
        kt.totals()        # {"gemm_tcgen05": microseconds, ...}
    """

    active: Optional["KernelTimes"] = None

    def __init__(self):
        self.records = []          # (name, start event, end event)

    def __enter__(self):
        if KernelTimes.active is not None:
            raise KernelError("KernelTimes does not nest")
        KernelTimes.active = self
        return self

    def __exit__(self, *exc):
        KernelTimes.active = None
        torch.cuda.synchronize()
        return False

    def totals(self) -> dict:
        """Microseconds per launcher name, and the number of calls under "<name> calls"."""
        torch.cuda.synchronize()
        out = {}
        for name, a, b in self.records:
            out[name] = out.get(name, 0.0) + a.elapsed_time(b) * 1e3
            out[name + " calls"] = out.get(name + " calls", 0) + 1
        return out


class _Timed:
    """A launcher that, while a ``KernelTimes`` is open, brackets its call with two events."""

    def __init__(self, fn, name: str):
        self.fn, self.name = fn, name

    def __call__(self, *args):
        kt = KernelTimes.active
        if kt is None:
            return self.fn(*args)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        rc = self.fn(*args)
        b.record()
        kt.records.append((self.name, a, b))
        return rc


_wrapped = {}


def _fn(lib_name: str, fn_name: str, argtypes):
    key = (lib_name, fn_name)
    got = _wrapped.get(key)
    if got is not None:
        return got
    lib = csrc.load(lib_name)
    fn = getattr(lib, fn_name)
    if key not in _prototyped:
        fn.argtypes = argtypes
        fn.restype = c_int
        err = getattr(lib, f"lgml_{lib_name}_last_error")
        err.restype = ctypes.c_char_p
        _prototyped.add(key)
        _wrapped[key] = _Timed(fn, fn_name[len("lgml_"):] if fn_name.startswith("lgml_") else fn_name)
    return _wrapped[key]


_launches = 0


def launch_count() -> int:
    """How many kernel launchers of this package have been called (a launcher starts one
    kernel; split-KV attention starts two).  Launches replayed by a CUDA graph are not
    counted here; the runner knows how many a graph holds."""
    return _launches


def _check(lib_name: str, rc: int, what: str) -> None:
    global _launches
    _launches += 1
    if rc != 0:
        err = getattr(csrc.load(lib_name), f"lgml_{lib_name}_last_error")
        err.restype = ctypes.c_char_p
        raise KernelError(f"{what}: {err().decode('utf-8', 'replace')} (code {rc})")


# ----------------------------------------------------------------------------------------
# elementwise
# ----------------------------------------------------------------------------------------

def embed_rows(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, status: torch.Tensor) -> torch.Tensor:
    """out[t] = table[ids[t]] as float32."""
    _need(table, "embedding table", ndim=2)
    _need(ids, "token ids", torch.int32, 1)
    _need(out, "embedding output", torch.float32, 2)
    if not table.is_contiguous() or not out.is_contiguous():
        raise KernelError("embedding table and output must be contiguous")
    n, width = out.shape
    if ids.numel() != n or table.shape[1] != width:
        raise KernelError(f"embed_rows: shapes disagree: table {tuple(table.shape)}, ids {tuple(ids.shape)}, out {tuple(out.shape)}")
    fn = _fn("elementwise", "lgml_embed_rows", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p])
    _check("elementwise", fn(_ptr(table), dtype_code(table.dtype), _ptr(ids), _ptr(out), n, width, table.shape[0], _ptr(status), _stream()), "embed_rows")
    return out


class Partials:
    """The float32 partial sums of a matrix product cut along K: ``data`` is
    [n_parts, rows, width]; the kernel that reads them adds the parts in order and then
    ``bias`` (per column) if there is one."""

    def __init__(self, data: torch.Tensor, bias: Optional[torch.Tensor] = None):
        self.data, self.bias = data, bias

    @property
    def shape(self):
        return self.data.shape[1:]

    def sum(self) -> torch.Tensor:
        """The product itself (for a part that does not read partial sums)."""
        y = self.data.sum(dim=0)
        return y if self.bias is None else y + self.bias


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, delta=None,
            rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = rmsnorm(x [+ delta]) * weight.  With ``delta`` (a tensor, or ``Partials``) and
    no ``rows`` the sum is written back to x (the residual add); with ``rows`` output row r
    reads x[rows[r]]."""
    _need(x, "norm input", torch.float32, 2)
    _need(weight, "norm weight", torch.float32, 1)
    _need(out, "norm output", ndim=2)
    width = x.shape[1]
    n_rows = out.shape[0]
    if not x.is_contiguous() or not out.is_contiguous() or out.shape[1] != width or weight.numel() != width:
        raise KernelError(f"rmsnorm: shapes disagree: x {tuple(x.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    if rows is None and n_rows != x.shape[0]:
        raise KernelError("rmsnorm: without a row list the output has the input's rows")
    if rows is not None:
        _need(rows, "row list", torch.int32, 1)
        if rows.numel() != n_rows:
            raise KernelError("rmsnorm: one output row per listed row")
    ddt, n_parts, stride, dbias, dptr = F32, 1, 0, None, None
    if isinstance(delta, Partials):
        d = delta.data
        _need(d, "residual delta parts", torch.float32, 3)
        if tuple(d.shape[1:]) != tuple(x.shape) or not d.is_contiguous():
            raise KernelError("rmsnorm: delta parts must be [parts, rows, width] and contiguous")
        n_parts, stride, dbias, dptr = d.shape[0], d.shape[1] * d.shape[2], delta.bias, d
    elif delta is not None:
        _need(delta, "residual delta", ndim=2)
        if delta.shape != x.shape or not delta.is_contiguous():
            raise KernelError("rmsnorm: delta must have the input's shape and be contiguous")
        ddt, dptr = dtype_code(delta.dtype), delta
    fn = _fn("elementwise", "lgml_rmsnorm", [c_void_p, c_void_p, c_int, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                             c_int, c_int, c_float, c_void_p])
    _check("elementwise", fn(_ptr(x), _ptr(dptr), ddt, n_parts, stride, _ptr(dbias), _ptr(weight), _ptr(rows), _ptr(out),
                             dtype_code(out.dtype), n_rows, width, float(eps), _stream()), "rmsnorm")
    return out


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, paired: bool = False) -> torch.Tensor:
    """out[t, f] = silu(gate[t, f]) * up[t, f]; gate|up are the two halves of a row, or, with
    ``paired``, neighbours (gate at 2f, up at 2f + 1)."""
    _need(gate_up, "gate|up", ndim=2)
    _need(out, "activation", gate_up.dtype, 2)
    n, two_f = gate_up.shape
    if two_f != 2 * out.shape[1] or out.shape[0] != n or not gate_up.is_contiguous() or not out.is_contiguous():
        raise KernelError(f"silu_mul: shapes disagree: gate|up {tuple(gate_up.shape)}, out {tuple(out.shape)}")
    fn = _fn("elementwise", "lgml_silu_mul", [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check("elementwise", fn(_ptr(gate_up), _ptr(out), dtype_code(out.dtype), n, out.shape[1], 1 if paired else 0, _stream()), "silu_mul")
    return out


def residual_add(x: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    """x += delta, the sum in float32."""
    _need(x, "residual stream", torch.float32)
    _need(delta, "residual delta")
    if x.shape != delta.shape or not x.is_contiguous() or not delta.is_contiguous():
        raise KernelError("residual_add: shapes disagree or not contiguous")
    fn = _fn("elementwise", "lgml_residual_add", [c_void_p, c_void_p, c_int, c_longlong, c_void_p])
    _check("elementwise", fn(_ptr(x), _ptr(delta), dtype_code(delta.dtype), x.numel(), _stream()), "residual_add")
    return x


def scale_cap(x: torch.Tensor, scale: float = 1.0, cap: float = 0.0) -> torch.Tensor:
    """In place on float32: x *= scale, then x = cap * tanh(x / cap) when cap > 0."""
    _need(x, "tensor to scale", torch.float32)
    if not x.is_contiguous():
        raise KernelError("scale_cap: tensor must be contiguous")
    fn = _fn("elementwise", "lgml_scale_cap", [c_void_p, c_longlong, c_float, c_float, c_void_p])
    _check("elementwise", fn(_ptr(x), x.numel(), float(scale), float(cap or 0.0), _stream()), "scale_cap")
    return x


def l2_ahead(t: torch.Tensor, n_bytes: Optional[int] = None, keep: bool = True) -> None:
    """Ask L2 for the first ``n_bytes`` of ``t`` (all of it when None); returns at once."""
    if not t.is_contiguous():
        raise KernelError("l2_ahead: tensor must be contiguous")
    total = t.numel() * t.element_size()
    n = total if n_bytes is None else min(int(n_bytes), total)
    fn = _fn("elementwise", "lgml_l2_ahead", [c_void_p, c_longlong, c_int, c_void_p])
    _check("elementwise", fn(_ptr(t), n, 1 if keep else 0, _stream()), "l2_ahead")


def fill_normal(out: torch.Tensor, mean: float, sd: float, seed: int) -> torch.Tensor:
    """Seeded N(mean, sd^2) fill on the device."""
    _need(out, "tensor to fill")
    if not out.is_contiguous():
        raise KernelError("fill_normal: tensor must be contiguous")
    fn = _fn("elementwise", "lgml_fill_normal", [c_void_p, c_int, c_longlong, c_float, c_float, c_ulonglong, c_void_p])
    _check("elementwise", fn(_ptr(out), dtype_code(out.dtype), out.numel(), float(mean), float(sd), seed & 0xFFFFFFFFFFFFFFFF, _stream()), "fill_normal")
    return out


# ----------------------------------------------------------------------------------------
# matrix products
# ----------------------------------------------------------------------------------------

def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[M,N] = a[M,K] . w[N,K]^T (+ bias), true float32 with a fixed summation order."""
    _need(a, "gemm input", torch.float32, 2)
    _need(w, "gemm weight", torch.float32, 2)
    _need(out, "gemm output", ndim=2)
    lda, ldw, ldc = _rows_contiguous(a, "gemm input"), _rows_contiguous(w, "gemm weight"), _rows_contiguous(out, "gemm output")
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"gemm_f32: shapes disagree: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if bias is not None:
        _need(bias, "gemm bias", torch.float32, 1)
        if bias.numel() != N:
            raise KernelError("gemm_f32: bias length is not N")
    fn = _fn("gemm_f32", "lgml_gemm_f32", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check("gemm_f32", fn(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), dtype_code(out.dtype), M, N, K, lda, ldw, ldc, _stream()), "gemm_f32")
    return out


# ----------------------------------------------------------------------------------------
# position encoding + cache write, attention
# ----------------------------------------------------------------------------------------

PAIRING = {"half": 0, "adjacent": 1}


def rope_kv_write(qkv, positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor,
                  inv_freq: torch.Tensor, n_rot: int, pairing: str, k_pages: torch.Tensor, v_pages: torch.Tensor, n_heads: int,
                  n_kv_heads: int, head_dim: int, status: torch.Tensor, write_kv: bool = True,
                  q_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rotate the first ``n_rot`` dimensions of q and k by the positions and store k and v in
    their cells (``write_kv`` False: q only, for a layer that reads another layer's cache).
    ``qkv`` is [tokens, (H + 2 Hkv) D] in the cache's type (q is then rotated in place unless
    ``q_out`` is given), or ``Partials`` of a projection cut along K (``q_out`` is then made
    if absent).  ``inv_freq``: float32 [n_rot / 2], or [2, n_rot / 2] with the part of each
    frequency that float32 lost in the second row (angles at positions in the thousands are
    then as exact as at the first ones).  Returns the rotated q as [tokens, H D] (a view of qkv when in place)."""
    _need(k_pages, "key pages", ndim=4)
    _need(v_pages, "value pages", k_pages.dtype, 4)
    cache_dt = k_pages.dtype
    width = (n_heads + 2 * n_kv_heads) * head_dim
    bias = None
    if isinstance(qkv, Partials):
        src = qkv.data
        _need(src, "qkv parts", torch.float32, 3)
        if not src.is_contiguous() or src.shape[2] != width:
            raise KernelError("rope_kv_write: parts must be [parts, tokens, (H + 2 Hkv) D] and contiguous")
        n_parts, n, lds, stride, bias = src.shape[0], src.shape[1], width, src.shape[1] * width, qkv.bias
        if q_out is None:
            q_out = torch.empty((n, n_heads * head_dim), dtype=cache_dt, device=src.device)
    else:
        src = qkv
        _need(src, "qkv", ndim=2)
        lds = _rows_contiguous(src, "qkv")
        n_parts, n, stride = 1, src.shape[0], 0
        if src.shape[1] != width:
            raise KernelError("rope_kv_write: qkv width is not (H + 2 Hkv) D")
        if q_out is None:
            if src.dtype != cache_dt:
                raise KernelError(f"rope_kv_write: qkv is {src.dtype} but the cache is {cache_dt}; give q_out")
            q_out = src[:, : n_heads * head_dim]
    _need(q_out, "rotated q", cache_dt, 2)
    ldq = _rows_contiguous(q_out, "rotated q")
    _need(positions, "positions", torch.int32, 1)
    _need(seq_of_token, "request index of tokens", torch.int32, 1)
    _need(block_table, "block table", torch.int32, 2)
    freq_lo = None
    if inv_freq.dim() == 2:          # [2, n_rot / 2]: the frequencies, and what float32 lost of each
        if inv_freq.shape[0] != 2 or not inv_freq.is_contiguous():
            raise KernelError("rope_kv_write: frequencies with low parts are a contiguous [2, n_rot / 2]")
        inv_freq, freq_lo = inv_freq[0], inv_freq[1]
    _need(inv_freq, "rotary frequencies", torch.float32, 1)
    if positions.numel() != n or seq_of_token.numel() != n or q_out.shape != (n, n_heads * head_dim):
        raise KernelError("rope_kv_write: one position, one request index and one q row per token")
    n_pages, hkv, page, d = k_pages.shape
    if (hkv, d) != (n_kv_heads, head_dim) or v_pages.shape != k_pages.shape or not k_pages.is_contiguous() or not v_pages.is_contiguous():
        raise KernelError(f"rope_kv_write: pages {tuple(k_pages.shape)} do not fit {n_kv_heads} KV heads of {head_dim}")
    if not block_table.is_contiguous():
        raise KernelError("rope_kv_write: the block table is not contiguous")
    if n_rot % 2 or n_rot > head_dim or inv_freq.numel() < max(n_rot // 2, 1):
        raise KernelError(f"rope_kv_write: n_rot {n_rot} must be even, at most head_dim, and have n_rot / 2 frequencies")
    fn = _fn("rope_cache", "lgml_rope_kv_write", [c_void_p, c_int, c_int, c_int, c_longlong, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                                   c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                                   c_int, c_int, c_void_p, c_void_p])
    _check("rope_cache", fn(_ptr(src), dtype_code(src.dtype), lds, n_parts, stride, _ptr(bias), _ptr(q_out), dtype_code(cache_dt), ldq,
                            _ptr(positions), _ptr(seq_of_token), _ptr(block_table), block_table.shape[1], _ptr(inv_freq), _ptr(freq_lo), n_rot,
                            PAIRING[pairing], _ptr(k_pages), _ptr(v_pages), n_pages, page, n, n_heads, n_kv_heads, head_dim,
                            1 if write_kv else 0, _ptr(status), _stream()), "rope_kv_write")
    return q_out


def paged_attention_ref(q: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor,
                        k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor, n_heads: int, scale: float, window: int,
                        status: torch.Tensor, softcap: float = 0.0) -> torch.Tensor:
    """out[t, h] = attention of query (t, h) over its request's cached keys at positions
    <= its own (the last ``window`` of them if window > 0).  ``q`` may be a column slice
    of a wider buffer.  ``softcap`` > 0 caps the scaled scores: s -> softcap * tanh(s / softcap)."""
    _need(q, "queries", ndim=2)
    _need(out, "attention output", q.dtype, 2)
    ldq, ldo = _rows_contiguous(q, "queries"), _rows_contiguous(out, "attention output")
    n = q.shape[0]
    n_pages, hkv, page, d = k_pages.shape
    _need(k_pages, "key pages", q.dtype, 4)
    _need(v_pages, "value pages", q.dtype, 4)
    _need(positions, "positions", torch.int32, 1)
    _need(seq_of_token, "request index of tokens", torch.int32, 1)
    _need(block_table, "block table", torch.int32, 2)
    if q.shape[1] != n_heads * d or out.shape != (n, n_heads * d):
        raise KernelError(f"paged_attention: q {tuple(q.shape)} / out {tuple(out.shape)} do not fit {n_heads} heads of {d}")
    if not k_pages.is_contiguous() or not v_pages.is_contiguous() or not block_table.is_contiguous():
        raise KernelError("paged_attention: pages and block table must be contiguous")
    fn = _fn("attention_ref", "lgml_paged_attention_ref", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                                           c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_float, c_void_p, c_void_p])
    _check("attention_ref", fn(_ptr(q), dtype_code(q.dtype), ldq, _ptr(positions), _ptr(seq_of_token), _ptr(block_table), block_table.shape[1],
                               _ptr(k_pages), _ptr(v_pages), n_pages, page, _ptr(out), ldo, n, n_heads, hkv, d, float(scale), int(window or 0),
                               float(softcap or 0.0), _ptr(status), _stream()), "paged_attention_ref")
    return out


# ----------------------------------------------------------------------------------------
# sampling
# ----------------------------------------------------------------------------------------

def argmax_rows(logits: torch.Tensor, out: torch.Tensor, scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[r] = index of the largest logit of row r; the lowest index wins a tie."""
    _need(logits, "logits", torch.float32, 2)
    _need(out, "token output", torch.int32, 1)
    ld = _rows_contiguous(logits, "logits")
    n = logits.shape[0]
    if out.numel() != n:
        raise KernelError("argmax_rows: one output per row")
    if scratch is None:
        scratch = torch.empty(max(64 * n, 1), dtype=torch.int32, device=logits.device)
    if scratch.numel() < 64 * n or scratch.element_size() != 4:
        raise KernelError("argmax_rows: scratch needs 64 32-bit words per row")
    fn = _fn("sampling", "lgml_argmax_rows", [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p])
    _check("sampling", fn(_ptr(logits), ld, n, logits.shape[1], _ptr(out), _ptr(scratch), _stream()), "argmax_rows")
    return out


TOPK_MAX = 128


def topk_rows(logits: torch.Tensor, k: int, out_vals: Optional[torch.Tensor] = None, out_ids: Optional[torch.Tensor] = None):
    """The k best candidates of every row, ordered by (logit descending, id ascending), as the
    sampler's top_k leaves them: (values float32 [rows, k], ids int32 [rows, k])."""
    _need(logits, "logits", torch.float32, 2)
    ld = _rows_contiguous(logits, "logits")
    n, v = logits.shape
    if not 1 <= k <= min(v, TOPK_MAX):
        raise KernelError(f"topk_rows: k = {k} must be between 1 and min(vocabulary {v}, {TOPK_MAX})")
    if out_vals is None:
        out_vals = torch.empty((n, k), dtype=torch.float32, device=logits.device)
    if out_ids is None:
        out_ids = torch.empty((n, k), dtype=torch.int32, device=logits.device)
    _need(out_vals, "top-k values", torch.float32, 2)
    _need(out_ids, "top-k ids", torch.int32, 2)
    if tuple(out_vals.shape) != (n, k) or tuple(out_ids.shape) != (n, k) or not out_vals.is_contiguous() or not out_ids.is_contiguous():
        raise KernelError("topk_rows: outputs must be contiguous [rows, k]")
    fn = _fn("sampling", "lgml_topk_rows", [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p])
    _check("sampling", fn(_ptr(logits), ld, n, v, int(k), _ptr(out_vals), _ptr(out_ids), _stream()), "topk_rows")
    return out_vals, out_ids


def sample_candidates(vals: torch.Tensor, ids: torch.Tensor, params: torch.Tensor, uniform: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """The chain after top_k on its candidates (``topk_rows``): top_p, min_p, temperature, draw.
    ``params`` float32 [rows, 3]: top_p, ln(min_p) or -inf, temperature > 0; ``uniform`` float64
    [rows]; ``out`` int32 [rows]."""
    _need(vals, "candidate values", torch.float32, 2)
    _need(ids, "candidate ids", torch.int32, 2)
    _need(params, "chain parameters", torch.float32, 2)
    _need(uniform, "uniform numbers", torch.float64, 1)
    _need(out, "token output", torch.int32, 1)
    n, k = vals.shape
    if tuple(ids.shape) != (n, k) or tuple(params.shape) != (n, 3) or uniform.numel() != n or out.numel() != n \
            or not (vals.is_contiguous() and ids.is_contiguous() and params.is_contiguous()):
        raise KernelError("sample_candidates: shapes disagree")
    fn = _fn("sampling", "lgml_sample_candidates", [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _check("sampling", fn(_ptr(vals), _ptr(ids), n, k, _ptr(params), _ptr(uniform), _ptr(out), _stream()), "sample_candidates")
    return out


def sampler_edits(logits: torch.Tensor, edits: torch.Tensor, params: torch.Tensor) -> torch.Tensor:
    """In place on the rows of ``logits``: the sampler's logit bias, then its history penalties.
    ``edits`` int32 [rows, stride]: per row (n_bias, n_hist, n_bias x (id, float bits of the
    bias), n_hist x (id, count)); ``params`` float32 [rows, 3]: repeat, frequency, presence."""
    _need(logits, "logits", torch.float32, 2)
    _need(edits, "sampler edits", torch.int32, 2)
    _need(params, "penalty parameters", torch.float32, 2)
    ld = _rows_contiguous(logits, "logits")
    n, v = logits.shape
    if edits.shape[0] != n or tuple(params.shape) != (n, 3) or not edits.is_contiguous() or not params.is_contiguous():
        raise KernelError("sampler_edits: one row of edits and of parameters per row of logits")
    fn = _fn("sampling", "lgml_sampler_edits", [c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p])
    _check("sampling", fn(_ptr(logits), ld, n, v, _ptr(edits), edits.shape[1], _ptr(params), _stream()), "sampler_edits")
    return logits


def sample_rows(logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """Row r: argmax if temperature[r] <= 0, else the inverse-CDF draw of
    softmax(logits[r] / temperature[r]) at uniform[r]."""
    _need(logits, "logits", torch.float32, 2)
    _need(temperature, "temperatures", torch.float32, 1)
    _need(uniform, "uniform numbers", torch.float64, 1)
    _need(out, "token output", torch.int32, 1)
    ld = _rows_contiguous(logits, "logits")
    r = logits.shape[0]
    if temperature.numel() != r or uniform.numel() != r or out.numel() != r:
        raise KernelError("sample_rows: one temperature, uniform number and output per row")
    fn = _fn("sampling", "lgml_sample_rows", [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _check("sampling", fn(_ptr(logits), ld, r, logits.shape[1], _ptr(temperature), _ptr(uniform), _ptr(out), _stream()), "sample_rows")
    return out


# ----------------------------------------------------------------------------------------
# bfloat16 matrix products and the fast attention paths
# ----------------------------------------------------------------------------------------

def tcgen05_supports(x: torch.Tensor, w: torch.Tensor) -> bool:
    """TMA wants 16-byte aligned operands whose row strides are multiples of 16 bytes."""
    return (x.stride(1) == 1 and w.stride(1) == 1 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


_splits_memo = {}


def tcgen05_splits(M: int, N: int, K: int) -> int:
    """K ranges of a product (remembered per shape: a step asks for the same few shapes again and again)."""
    key = (M, N, K)
    got = _splits_memo.get(key)
    if got is None:
        got = _splits_memo[key] = _tcgen05_splits(M, N, K)
    return got


def _tcgen05_splits(M: int, N: int, K: int) -> int:
    """K ranges for a product with few tokens: enough CTAs to cover the SMs about twice (once
    from 65 tokens on: every range writes and the next kernel reads M x N float32 partial sums,
    which with many tokens is no longer small beside the weights; at 64 tokens nine ranges of
    the output projection still win 0.9 us over five and cost the norm behind them 0.6), each
    with at least four 64-wide K blocks."""
    if M > 64:
        fn = getattr(csrc.load("gemm_tcgen05"), "lgml_gemm_tcgen05_pair_ranges", None)
        if fn is not None:
            fn.argtypes, fn.restype = [c_int, c_int, c_int], c_int
            ranges = fn(M, N, K)
            if ranges:          # on pairs of CTAs: the kernel library knows how it would cut K
                return ranges
    if M > 256:
        return 1
    tiles = -(-N // 128)
    k_blocks = -(-K // 64)
    cover = (2 * sm_count()) // tiles if M <= 64 else -(-sm_count() // tiles)
    splits = max(1, min(cover, k_blocks // 4, 16))
    # no range without K blocks: 64 blocks in 9 ranges of 8 would leave the ninth empty
    return -(-k_blocks // -(-k_blocks // splits))


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor], bias: Optional[torch.Tensor], status: torch.Tensor,
                 n_splits: Optional[int] = None, scratch: Optional[torch.Tensor] = None, swiglu: bool = False,
                 partials_ok: bool = False, checked: bool = False):
    """out[M,N] = x[M,K] . w[N,K]^T (+ bias) on tcgen05 tensor cores; bfloat16 in, float32
    accumulation, out bfloat16 or float32.  ``swiglu``: the rows of w (and bias) come in
    (gate, up) pairs and out[M, N/2] = silu(gate) * up.  ``partials_ok``: when K is cut, return
    ``Partials`` (the float32 partial sums and the bias) instead of adding them up here.
    ``checked``: the caller (``gemm_bf16``) has checked x and w and chosen ``n_splits`` by
    ``tcgen05_splits``."""
    if not checked:
        _need(x, "gemm input", torch.bfloat16, 2)
        _need(w, "gemm weight", torch.bfloat16, 2)
    ldx, ldw = _rows_contiguous(x, "gemm input"), _rows_contiguous(w, "gemm weight")
    M, K = x.shape
    N = w.shape[0]
    n_out = N // 2 if swiglu else N
    if w.shape[1] != K:
        raise KernelError(f"gemm_tcgen05: shapes disagree: x {tuple(x.shape)}, w {tuple(w.shape)}")
    if bias is not None:
        _need(bias, "gemm bias", torch.float32, 1)
        if bias.numel() != N:
            raise KernelError("gemm_tcgen05: bias length is not N")
    if n_splits is None:
        n_splits = 1 if swiglu else tcgen05_splits(M, N, K)
    elif checked:
        pass
    elif M > 64 and n_splits > 1 and tcgen05_splits(M, N, K) and os.environ.get("LGML_GEMM_PAIR") != "0":
        # on pairs of CTAs a K range is a whole number of 128-element stages, and none may be empty
        stages = -(-K // 128)
        n_splits = -(-stages // -(-stages // min(n_splits, stages)))
    n_splits = max(1, min(n_splits, -(-K // 64)))
    if swiglu and n_splits != 1:
        raise KernelError("gemm_tcgen05: the gated epilogue takes no K split")
    raw = partials_ok and n_splits > 1
    if n_splits > 1:
        need = n_splits * M * N
        if scratch is None:
            scratch = torch.empty(need, dtype=torch.float32, device=x.device)
        if scratch.numel() < need or scratch.dtype != torch.float32:
            raise KernelError(f"gemm_tcgen05: scratch of {scratch.numel()} floats, {need} needed")
    ldy, y_f32 = n_out, 0
    if not raw:
        _need(out, "gemm output", ndim=2)
        ldy = _rows_contiguous(out, "gemm output")
        if out.shape != (M, n_out) or out.dtype not in (torch.bfloat16, torch.float32):
            raise KernelError(f"gemm_tcgen05: output {tuple(out.shape)} {out.dtype} does not fit [{M}, {n_out}]")
        y_f32 = 1 if out.dtype == torch.float32 else 0
    fn = _fn("gemm_tcgen05", "lgml_gemm_tcgen05", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                                   c_int, c_void_p, c_int, c_int, c_void_p, c_void_p])
    _check("gemm_tcgen05", fn(_ptr(x), _ptr(w), _ptr(bias), _ptr(None if raw else out), y_f32, M, N, K, ldx, ldw, ldy,
                              n_splits, _ptr(scratch if n_splits > 1 else None), 1 if swiglu else 0, 0 if raw else 1, _ptr(status),
                              _stream()), "gemm_tcgen05")
    if raw:
        return Partials(scratch[: n_splits * M * N].view(n_splits, M, N), bias)
    return out


def gemm_cublas(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The library product (the reference engine's matrix products are a library's too)."""
    if bias is None and out_dtype == torch.bfloat16:
        return torch.mm(x, w.t())
    y = torch.mm(x, w.t(), out_dtype=torch.float32)
    if bias is not None:
        y += bias
    return y if out_dtype == torch.float32 else y.to(out_dtype)


def gemm_bf16(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, bias: Optional[torch.Tensor] = None,
              backend: str = "auto", status: Optional[torch.Tensor] = None, partials_ok: bool = False):
    """y[M,N] = x[M,K] . w[N,K]^T (+ bias) with bfloat16 operands and float32 accumulation;
    y is bfloat16 or float32.  ``backend``: "tcgen05" is the hand-written tensor-core kernel,
    "cublas" the library product; "auto" takes tcgen05 whenever its operands fit TMA's
    alignment rules.  With ``partials_ok`` the result may be ``Partials``."""
    _need(x, "gemm input", torch.bfloat16, 2)
    _need(w, "gemm weight", torch.bfloat16, 2)
    if x.shape[1] != w.shape[1]:
        raise KernelError(f"gemm_bf16: shapes disagree: x {tuple(x.shape)}, w {tuple(w.shape)}")
    if x.shape[0] == 0:
        return torch.empty((0, w.shape[0]), dtype=out_dtype, device=x.device)
    if backend == "cublas" or (backend == "auto" and not tcgen05_supports(x, w)):
        return gemm_cublas(x, w, out_dtype, bias)
    if backend not in ("auto", "tcgen05"):
        raise KernelError(f"unknown gemm backend '{backend}'")
    if status is None:
        raise KernelError("gemm_bf16: the tcgen05 kernel needs the status word")
    n_splits = tcgen05_splits(x.shape[0], w.shape[0], x.shape[1])
    if partials_ok and n_splits > 1:          # the partial sums are the result: no output to make
        return gemm_tcgen05(x, w, None, bias, status, n_splits=n_splits, partials_ok=True, checked=True)
    out = torch.empty((x.shape[0], w.shape[0]), dtype=out_dtype, device=x.device)
    return gemm_tcgen05(x, w, out, bias, status, n_splits=n_splits, checked=True)


def gemm_bf16_swiglu(x: torch.Tensor, w_pairs: torch.Tensor, bias_pairs: Optional[torch.Tensor], status: torch.Tensor) -> torch.Tensor:
    """act[M, F] = silu(x . gate^T) * (x . up^T) in one kernel; ``w_pairs`` [2F, K] holds the
    gate and up rows of each feature next to each other (gate first)."""
    out = torch.empty((x.shape[0], w_pairs.shape[0] // 2), dtype=torch.bfloat16, device=x.device)
    if x.shape[0] == 0:
        return out
    return gemm_tcgen05(x, w_pairs, out, bias_pairs, status, swiglu=True)


_sm_count = None


def sm_count() -> int:
    """Streaming multiprocessors of the current device (148 on a B200)."""
    global _sm_count
    if _sm_count is None:
        _sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count if torch.cuda.is_available() else 148
    return _sm_count


def decode_splits(n_tokens: int, n_kv_heads: int, group: int, max_kv_len: int, page: int = 64) -> int:
    """How many ranges the keys of a token are cut into.  A range costs its CTA's start and its
    share of the merge whatever its length, so: at least four pages a range; as many CTAs as fill
    the SMs twice over, or once over while there are few of them to begin with and the context is
    short (one or two requests up to 4,096 tokens: the step waits for the slowest CTA, not for
    bandwidth); and no more than 16 ranges, or a 16th of the pages where that is more (the merge
    reads every range of a head).  Measured with `kernel_bench decode_attention`, 32 heads on 8 KV
    heads of 128, merge included: one request at 2,176 tokens 10.2 us with 9 ranges, 8.6 with 16,
    9.6 with 18; at 8,192 tokens 13.8 us with 16, 15.7 with 37; at 32,768 tokens 38.3 us with 16,
    31.7 with 37; two requests at 2,176 tokens 9.7 us with 9, 11.1 with 16, at 8,192 tokens 18.6 us
    with 16, 21.1 with 9 or 18; eight requests 18.4 us
    with 4 ranges, 21.8 with 3, 23.4 with 5."""
    ctas = max(n_tokens * n_kv_heads * ((group + 7) // 8), 1)
    pages = max(1, -(-max_kv_len // page))
    per_sm = 1 if ctas <= 16 and pages <= 64 else 2
    return max(1, min(-(-pages // 4), (per_sm * sm_count()) // ctas, max(16, pages // 16), 512))


def decode_attention(q: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor,
                     k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor, n_heads: int, scale: float, window: int,
                     status: torch.Tensor, n_splits: int, scratch: Optional[torch.Tensor] = None, max_new_tokens: int = 16) -> torch.Tensor:
    """bfloat16 split-KV attention: each token over its request's cells.  Scratch (float32,
    ``decode_attention_scratch_floats`` elements) is needed when n_splits > 1.
    ``max_new_tokens``: the most tokens one request brings in this step (the kernel starts
    fetching older pages before the kernels ahead of it have finished)."""
    _need(q, "queries", torch.bfloat16, 2)
    _need(out, "attention output", torch.bfloat16, 2)
    ldq, ldo = _rows_contiguous(q, "queries"), _rows_contiguous(out, "attention output")
    n = q.shape[0]
    _need(k_pages, "key pages", torch.bfloat16, 4)
    _need(v_pages, "value pages", torch.bfloat16, 4)
    n_pages, hkv, page, d = k_pages.shape
    _need(positions, "positions", torch.int32, 1)
    _need(seq_of_token, "request index of tokens", torch.int32, 1)
    _need(block_table, "block table", torch.int32, 2)
    if q.shape[1] != n_heads * d or out.shape != (n, n_heads * d):
        raise KernelError(f"decode_attention: q {tuple(q.shape)} / out {tuple(out.shape)} do not fit {n_heads} heads of {d}")
    if not k_pages.is_contiguous() or not v_pages.is_contiguous() or not block_table.is_contiguous() or v_pages.shape != k_pages.shape:
        raise KernelError("decode_attention: pages and block table must be contiguous")
    if n_splits > 1:
        need = n * n_heads * n_splits * (d + 2)
        if scratch is None:
            scratch = torch.empty(need, dtype=torch.float32, device=q.device)
        _need(scratch, "scratch", torch.float32, 1)
        if scratch.numel() < need:
            raise KernelError(f"decode_attention: scratch of {scratch.numel()} floats, {need} needed")
    fn = _fn("attention_decode", "lgml_decode_attention", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                                                           c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p])
    _check("attention_decode", fn(_ptr(q), ldq, _ptr(positions), _ptr(seq_of_token), _ptr(block_table), block_table.shape[1], _ptr(k_pages),
                                  _ptr(v_pages), n_pages, page, _ptr(out), ldo, _ptr(scratch if n_splits > 1 else None), n_splits, n, n_heads, hkv, d,
                                  float(scale), int(window or 0), int(max_new_tokens), _ptr(status), _stream()), "decode_attention")
    return out


def prefill_tile_tokens(n_heads: int, n_kv_heads: int) -> int:
    """Tokens per tile of the prefill attention kernel for this grouping of heads."""
    hpc = min(n_heads // n_kv_heads, 8)
    return 16 * (8 // hpc)


def _prefill_attention_call(library: str, symbol: str, label: str, q, positions, tiles, block_table, k_pages, v_pages, out, n_heads, scale,
                            window, status) -> torch.Tensor:
    """The checks and the call that the three prefill attention kernels share (one signature)."""
    _need(q, "queries", torch.bfloat16, 2)
    _need(out, "attention output", torch.bfloat16, 2)
    ldq, ldo = _rows_contiguous(q, "queries"), _rows_contiguous(out, "attention output")
    n = q.shape[0]
    _need(k_pages, "key pages", torch.bfloat16, 4)
    _need(v_pages, "value pages", torch.bfloat16, 4)
    n_pages, hkv, page, d = k_pages.shape
    _need(positions, "positions", torch.int32, 1)
    _need(tiles, "tiles", torch.int32, 2)
    _need(block_table, "block table", torch.int32, 2)
    if q.shape[1] != n_heads * d or out.shape != (n, n_heads * d) or tiles.shape[1] != 4:
        raise KernelError(f"{label}: q {tuple(q.shape)} / out {tuple(out.shape)} / tiles {tuple(tiles.shape)} do not fit")
    if not k_pages.is_contiguous() or not v_pages.is_contiguous() or not block_table.is_contiguous() or not tiles.is_contiguous():
        raise KernelError(f"{label}: pages, block table and tiles must be contiguous")
    fn = _fn(library, symbol, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
                               c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p])
    _check(library, fn(_ptr(q), ldq, _ptr(positions), _ptr(tiles), tiles.shape[0], _ptr(block_table), block_table.shape[1],
                       _ptr(k_pages), _ptr(v_pages), n_pages, page, _ptr(out), ldo, n_heads, hkv, d, float(scale),
                       int(window or 0), _ptr(status), _stream()), label)
    return out


def prefill_attention(q: torch.Tensor, positions: torch.Tensor, tiles: torch.Tensor, block_table: torch.Tensor,
                      k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor, n_heads: int, scale: float, window: int,
                      status: torch.Tensor) -> torch.Tensor:
    """bfloat16 tensor-core attention for prompts and portions (``mma.sync``).  ``tiles`` is int32
    [n_tiles, 4]: (request row, first token row, tokens, 0), each tile within one request
    and at most ``prefill_tile_tokens`` long."""
    return _prefill_attention_call("attention_prefill", "lgml_prefill_attention", "prefill_attention", q, positions, tiles, block_table,
                                   k_pages, v_pages, out, n_heads, scale, window, status)


def prefill_tc_tile_tokens(n_heads: int, n_kv_heads: int) -> int:
    """Tokens per tile of the tcgen05 prefill attention kernel: 128 rows / heads per CTA."""
    return 128 // min(n_heads // n_kv_heads, 8)


def prefill_attention_tc(q: torch.Tensor, positions: torch.Tensor, tiles: torch.Tensor, block_table: torch.Tensor,
                         k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor, n_heads: int, scale: float, window: int,
                         status: torch.Tensor) -> torch.Tensor:
    """bfloat16 attention for prompts and portions on tcgen05 tensor cores (S and the page's
    output in tensor memory), one tile of 128 rows per CTA.  ``tiles`` as for
    ``prefill_attention``, each at most ``prefill_tc_tile_tokens`` long."""
    return _prefill_attention_call("attention_prefill_tc", "lgml_prefill_attention_tc", "prefill_attention_tc", q, positions, tiles,
                                   block_table, k_pages, v_pages, out, n_heads, scale, window, status)


def prefill_twin_tile_tokens(n_heads: int, n_kv_heads: int) -> int:
    """Tokens per CTA of the two-tile tcgen05 prefill attention kernel: 2 x (128 rows / heads per CTA)."""
    return 2 * (128 // min(n_heads // n_kv_heads, 8))


def prefill_attention_twin(q: torch.Tensor, positions: torch.Tensor, tiles: torch.Tensor, block_table: torch.Tensor,
                           k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor, n_heads: int, scale: float, window: int,
                           status: torch.Tensor) -> torch.Tensor:
    """bfloat16 attention for prompts and portions on tcgen05 tensor cores, two tiles of 128
    rows per CTA (scores, P and the output in tensor memory), for head sizes 64 and 128.
    ``tiles`` as for ``prefill_attention``, each at most ``prefill_twin_tile_tokens`` long."""
    return _prefill_attention_call("attention_prefill_twin", "lgml_prefill_attention_twin", "prefill_attention_twin", q, positions, tiles,
                                   block_table, k_pages, v_pages, out, n_heads, scale, window, status)


def prefill_tc_supports(q: torch.Tensor, out: torch.Tensor) -> bool:
    """The tcgen05 kernel reads q and writes out in 16-byte pieces."""
    return q.stride(0) % 8 == 0 and out.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0


# which kernel runs prompts and portions: "tcgen05" (default: two tiles per CTA for head sizes 64
# and 128, one tile otherwise), "single" (one tile per CTA for every head size) or "mma" (the
# mma.sync kernel)
PREFILL_ATTENTION = os.environ.get("LGML_PREFILL_ATTENTION", "tcgen05")

# a portion of at most this many tokens per request is run by the decode kernel
DECODE_MAX_Q = 8


def paged_attention(q, batch, cache, out, n_heads: int, scale: float, window: int, status: torch.Tensor) -> torch.Tensor:
    """bfloat16 attention over the paged cache; picks the kernel by the batch's shape: the
    split-KV kernel when every request brings a few tokens, the tensor-core kernel for
    prompts and portions (head sizes up to 128), the general kernel otherwise."""
    d = cache.k.shape[3]
    hkv = cache.k.shape[1]
    if cache.k.shape[2] == 64 and d % 16 == 0:
        if batch.max_q_len <= DECODE_MAX_Q:
            n_splits = batch.decode_splits if getattr(batch, "decode_splits", None) else decode_splits(q.shape[0], hkv, n_heads // hkv, batch.max_kv_len)
            return decode_attention(q, batch.positions, batch.seq_of_token, cache.block_table, cache.k, cache.v, out, n_heads, scale,
                                    window, status, n_splits, max_new_tokens=batch.max_q_len)
        if d in (64, 128) and PREFILL_ATTENTION == "tcgen05" and prefill_tc_supports(q, out):
            tiles = batch.attention_tiles(prefill_twin_tile_tokens(n_heads, hkv))
            return prefill_attention_twin(q, batch.positions, tiles, cache.block_table, cache.k, cache.v, out, n_heads, scale, window, status)
        if d <= 128 and PREFILL_ATTENTION in ("tcgen05", "single") and prefill_tc_supports(q, out):
            tiles = batch.attention_tiles(prefill_tc_tile_tokens(n_heads, hkv))
            return prefill_attention_tc(q, batch.positions, tiles, cache.block_table, cache.k, cache.v, out, n_heads, scale, window, status)
        if d <= 128:
            tiles = batch.attention_tiles(prefill_tile_tokens(n_heads, hkv))
            return prefill_attention(q, batch.positions, tiles, cache.block_table, cache.k, cache.v, out, n_heads, scale, window, status)
    return paged_attention_ref(q, batch.positions, batch.seq_of_token, cache.block_table, cache.k, cache.v, out, n_heads,
                               scale, window, status)
