"""Python faces of the CUDA launchers: argument checks, pointer passing, status codes turned into errors.

Every function works on CUDA tensors only and launches on the current stream of PyTorch, so the launches
are ordered with PyTorch's own work and are captured by ``torch.cuda.graph``.  There is no CPU path: a
tensor that is not on a CUDA device, or a missing compiler, raises.
"""
from __future__ import annotations

import ctypes
import math
import os
import sys
from ctypes import c_int, c_int64, c_float, c_void_p
from typing import Dict, Optional

import torch

from .build import load_library

_ERRORS = {
    -1: "element type must be float32 or bfloat16",
    -2: "a size is zero, negative or beyond what the kernel takes",
    -3: "a pointer or a row length breaks the kernel's alignment rule",
    -4: "sizes are inconsistent with one another",
    -5: "this specialised kernel does not cover the configuration",
    -6: "scratch memory is missing or too small",
}

DEVICE_ERRORS = {
    1: "a token id lies outside the embedding table",
    2: "a cache slot lies outside the page pool",
    3: "a position lies outside the position tables (beyond the model's maximum position)",
    4: "attention needed a key whose page is missing from the block table",
    5: "a bounded wait in a kernel ran out",
    6: "a kernel found its shared memory misaligned for swizzled tiles",
    7: "a routed feed-forward met an expert index outside its experts",
}


class KernelError(RuntimeError):
    pass


LAUNCHES = 0      # kernels of this package launched (or recorded into a graph being captured) so far


def launches() -> int:
    return LAUNCHES


def _check(status: int, what: str, kernels: int = 1) -> None:
    global LAUNCHES
    if status == 0:
        LAUNCHES += kernels
        return
    if status < 0:
        raise KernelError(f"{what}: refused: {_ERRORS.get(status, f'code {status}')}")
    raise KernelError(f"{what}: CUDA launch failed with cudaError {status}")


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return 0
    if dt == torch.bfloat16:
        return 1
    raise KernelError(f"element type must be float32 or bfloat16, got {dt}")


def _cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("the kernels run on CUDA tensors only; got a tensor on " + str(t.device))


def _contig(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_contiguous():
            raise KernelError("kernel arguments must be contiguous")


def _ptr(t: Optional[torch.Tensor]):
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


_device_index = None


def _stream():
    """The current CUDA stream's handle.  Asked of torch's C layer directly: `torch.cuda.current_stream()` builds a
    Python object at every call and costs about 15 us, which a step of a few hundred launches feels."""
    global _device_index
    if _device_index is None:
        _device_index = torch.cuda.current_device()
    return c_void_p(torch._C._cuda_getCurrentRawStream(_device_index))


_core = None


def core():
    global _core
    if _core is None:
        lib = load_library("core")
        for name in ("cvb_embed", "cvb_rmsnorm", "cvb_add_rmsnorm", "cvb_add", "cvb_swiglu", "cvb_gather_rows",
                     "cvb_qk_norm_rope_kv", "cvb_paged_attention_general", "cvb_paged_attention_entries", "cvb_sample", "cvb_sample_chunked",
                     "cvb_feed_tokens"):
            getattr(lib, name).restype = c_int
        _core = lib
    return _core


_err_flags = {}


def error_flag(device) -> torch.Tensor:
    """One int32 per device that kernels set when they meet an index they refuse to follow."""
    device = torch.device(device)
    key = device.index if device.index is not None else torch.cuda.current_device()
    f = _err_flags.get(key)
    if f is None:
        f = torch.zeros(1, dtype=torch.int32, device=device)
        _err_flags[key] = f
    return f


def check_device_errors(device) -> None:
    """Read the device error flag (synchronises) and raise if a kernel recorded a refused index."""
    f = error_flag(device)
    v = int(f.item())
    if v != 0:
        f.zero_()
        raise KernelError(f"a kernel reported: {DEVICE_ERRORS.get(v, f'error {v}')}")


def selftest_wait_runs_out(limit_cycles: int = 2_000_000) -> int:
    """Launches a block that waits on a barrier nothing arrives on, with a limit of `limit_cycles` clock cycles (about a
    millisecond by default).  Returns 1 if the wait gave up and the kernel ran to its end; the device error word then
    holds 5 (check_device_errors raises "a bounded wait in a kernel ran out")."""
    lib = core()
    lib.cvb_selftest_wait_runs_out.restype = c_int
    dev = torch.device("cuda", torch.cuda.current_device())
    finished = torch.zeros(1, dtype=torch.int32, device=dev)
    _check(lib.cvb_selftest_wait_runs_out(_ptr(error_flag(dev)), _ptr(finished), ctypes.c_longlong(limit_cycles), _stream()),
           "selftest_wait_runs_out")
    return int(finished.item())


# ---- elementwise ------------------------------------------------------------------------------------------

def embed(out: torch.Tensor, table: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
    _cuda(out, table, tokens); _contig(out, table, tokens)
    T, D = out.shape
    if tokens.dtype != torch.int32 or tokens.numel() != T or table.shape[1] != D or table.dtype != out.dtype:
        raise KernelError("embed: tokens must be int32 [T]; table [V, D] and out [T, D] of one element type")
    _check(core().cvb_embed(_ptr(out), _ptr(table), _ptr(tokens), c_int(T), c_int(D), c_int(table.shape[0]),
                            c_int(dtype_code(out.dtype)), _ptr(error_flag(out.device)), _stream()), "embed")
    return out


def rmsnorm(out: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    _cuda(out, x, weight); _contig(out, x, weight)
    T, D = x.shape
    if weight.dtype != torch.float32 or weight.numel() != D or out.shape != x.shape or out.dtype != x.dtype:
        raise KernelError("rmsnorm: weight must be float32 [D]; out like x")
    _check(core().cvb_rmsnorm(_ptr(out), _ptr(x), _ptr(weight), c_int(T), c_int(D), c_float(eps),
                              c_int(dtype_code(x.dtype)), _stream()), "rmsnorm")
    return out


def add_rmsnorm(out: torch.Tensor, resid: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """resid <- T(resid + x) in place; out <- rmsnorm(resid)."""
    _cuda(out, resid, x, weight); _contig(out, resid, x, weight)
    T, D = x.shape
    if (weight.dtype != torch.float32 or weight.numel() != D or out.shape != x.shape or resid.shape != x.shape
            or out.dtype != x.dtype or resid.dtype != x.dtype):
        raise KernelError("add_rmsnorm: weight must be float32 [D]; out, resid like x")
    _check(core().cvb_add_rmsnorm(_ptr(out), _ptr(resid), _ptr(x), _ptr(weight), c_int(T), c_int(D), c_float(eps),
                                  c_int(dtype_code(x.dtype)), _stream()), "add_rmsnorm")
    return out


def add_(resid: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    _cuda(resid, x); _contig(resid, x)
    if resid.shape != x.shape or resid.dtype != x.dtype:
        raise KernelError("add_: operands must match")
    _check(core().cvb_add(_ptr(resid), _ptr(x), c_int64(x.numel()), c_int(dtype_code(x.dtype)), _stream()), "add_")
    return resid


def swiglu(out: torch.Tensor, gate_up: torch.Tensor) -> torch.Tensor:
    _cuda(out, gate_up); _contig(out, gate_up)
    T, I = out.shape
    if gate_up.shape != (T, 2 * I) or gate_up.dtype != out.dtype:
        raise KernelError("swiglu: gate_up must be [T, 2I] for out [T, I]")
    _check(core().cvb_swiglu(_ptr(out), _ptr(gate_up), c_int(T), c_int(I), c_int(dtype_code(out.dtype)), _stream()),
           "swiglu")
    return out


def gather_rows(out: torch.Tensor, src: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    _cuda(out, src, rows); _contig(out, src, rows)
    R, D = out.shape
    if rows.dtype != torch.int32 or rows.numel() < R or src.shape[1] != D or src.dtype != out.dtype:
        raise KernelError("gather_rows: rows must be int32 [R]; src [N, D], out [R, D] of one element type")
    _check(core().cvb_gather_rows(_ptr(out), _ptr(src), _ptr(rows), c_int(R), c_int(D), c_int(src.shape[0]),
                                  c_int(dtype_code(out.dtype)), _stream()), "gather_rows")
    return out


# ---- a residual stream in float under activations of any element type ----------------------------------------

_resid32 = None


def _resid32_lib():
    global _resid32
    if _resid32 is None:
        lib = load_library("resid32")
        for name in ("cvb_embed_positions", "cvb_resid_update", "cvb_gelu_tanh", "cvb_write_rows", "cvb_norm_add", "cvb_bias_act",
                     "cvb_gated_norm"):
            getattr(lib, name).restype = c_int
        _resid32 = lib
    return _resid32


def embed_positions(out: torch.Tensor, table: torch.Tensor, tokens: torch.Tensor, positions: torch.Tensor, scale: float = 1.0,
                    pos_table: Optional[torch.Tensor] = None, out2: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t] = float(table[tokens[t]]) * scale + float(pos_table[positions[t]]); `out2` receives a second copy."""
    _cuda(out, table, tokens, positions, pos_table, out2); _contig(out, table, tokens, positions, pos_table, out2)
    T, D = out.shape
    if (out.dtype != torch.float32 or tokens.dtype != torch.int32 or positions.dtype != torch.int32 or tokens.numel() < T
            or positions.numel() < T or table.shape[1] != D
            or (pos_table is not None and (pos_table.dtype != table.dtype or pos_table.shape[1] != D))
            or (out2 is not None and (out2.dtype != torch.float32 or out2.shape != out.shape))):
        raise KernelError("embed_positions: out float32 [T, D]; tokens, positions int32 [T]; table [V, D] and pos_table [P, D] of "
                          "one element type")
    _check(_resid32_lib().cvb_embed_positions(
        _ptr(out), _ptr(out2), _ptr(table), _ptr(pos_table), _ptr(tokens), _ptr(positions), c_int(T), c_int(D),
        c_int(table.shape[0]), c_int(pos_table.shape[0] if pos_table is not None else 0), c_float(scale),
        c_int(dtype_code(table.dtype)), _ptr(error_flag(out.device)), _stream()), "embed_positions")
    return out


def resid_update(h: torch.Tensor, deltas=(), rows: Optional[torch.Tensor] = None, vector: Optional[torch.Tensor] = None,
                 norm_weight: Optional[torch.Tensor] = None, eps: float = 0.0, out: Optional[torch.Tensor] = None):
    """h (float32 [T, D], in place) <- ((h + (deltas[0] + deltas[1])) + rows) + vector, each addend optional: up to two
    deltas of the activations' element type [T, D], float32 rows [T, D], a float32 vector [D].  With `norm_weight`
    (float32 [D]) also out <- RMSNorm(h) * norm_weight, rounded once, in out's element type.  Returns out (or h)."""
    deltas = tuple(d for d in deltas if d is not None)
    if len(deltas) > 2:
        raise KernelError("resid_update: at most two deltas")
    d1 = deltas[0] if deltas else None
    d2 = deltas[1] if len(deltas) > 1 else None
    _cuda(h, d1, d2, rows, vector, norm_weight, out); _contig(h, d1, d2, rows, vector, norm_weight, out)
    T, D = h.shape
    act = out.dtype if out is not None else (d1.dtype if d1 is not None else torch.float32)
    if h.dtype != torch.float32:
        raise KernelError("resid_update: the residual stream must be float32")
    for d in deltas:
        if d.shape != h.shape or d.dtype != act:
            raise KernelError("resid_update: deltas must be shaped like h and share the output's element type")
    if rows is not None and (rows.dtype != torch.float32 or rows.shape != h.shape):
        raise KernelError("resid_update: rows must be float32, shaped like h")
    if vector is not None and (vector.dtype != torch.float32 or vector.numel() != D):
        raise KernelError("resid_update: vector must be float32 [D]")
    if norm_weight is not None and (out is None or norm_weight.dtype != torch.float32 or norm_weight.numel() != D
                                    or out.shape != h.shape):
        raise KernelError("resid_update: the norm needs a float32 weight [D] and an out shaped like h")
    _check(_resid32_lib().cvb_resid_update(_ptr(h), _ptr(d1), _ptr(d2), _ptr(rows), _ptr(vector), _ptr(norm_weight), _ptr(out),
                                           c_int(T), c_int(D), c_float(eps), c_int(dtype_code(act)), _stream()), "resid_update")
    return out if out is not None else h


def gelu_tanh(out: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    _cuda(out, x); _contig(out, x)
    if out.shape != x.shape or out.dtype != x.dtype:
        raise KernelError("gelu_tanh: out must match x")
    _check(_resid32_lib().cvb_gelu_tanh(_ptr(out), _ptr(x), c_int64(x.numel()), c_int(dtype_code(x.dtype)), _stream()), "gelu_tanh")
    return out


def write_rows(pages: torch.Tensor, src: torch.Tensor, slots: torch.Tensor, col0: int, heads: int, width: int,
               page_size: int) -> torch.Tensor:
    """pages[slot // page_size, head, slot % page_size, :] = src[t, col0 + head * width : ...] for every row t of src."""
    _cuda(pages, src, slots); _contig(pages, src, slots)
    T = src.shape[0]
    if pages.dtype != src.dtype or slots.dtype != torch.int32 or slots.numel() < T or src.dim() != 2:
        raise KernelError("write_rows: pages and src of one element type, slots int32 [T]")
    _check(_resid32_lib().cvb_write_rows(_ptr(pages), _ptr(src), _ptr(slots), c_int(T), c_int(src.shape[1]), c_int(col0),
                                         c_int(heads), c_int(width), c_int(page_size), c_int64(pages.numel()),
                                         c_int(dtype_code(src.dtype)), _ptr(error_flag(src.device)), _stream()), "write_rows")
    return pages


def norm_add(h: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float, bias: Optional[torch.Tensor] = None,
             accumulate: bool = True, copy: Optional[torch.Tensor] = None) -> torch.Tensor:
    """h (float32 [T, D]) <- [h +] RMSNorm(y + bias) * weight: the norm behind a sublayer, whose result alone joins the stream
    (`accumulate=False`: h is set, not added to).  `copy` (the activations' type, shaped like h) receives the new stream
    rounded once."""
    _cuda(h, y, weight, bias, copy); _contig(h, y, weight, bias, copy)
    T, D = h.shape
    if (h.dtype != torch.float32 or y.shape != h.shape or weight.dtype != torch.float32 or weight.numel() != D
            or (bias is not None and (bias.dtype != torch.float32 or bias.numel() != D))
            or (copy is not None and (copy.shape != h.shape or copy.dtype != y.dtype))):
        raise KernelError("norm_add: h float32 [T, D]; y [T, D]; weight and bias float32 [D]; copy like y")
    _check(_resid32_lib().cvb_norm_add(_ptr(h), _ptr(y), _ptr(bias), _ptr(weight), _ptr(copy), c_int(T), c_int(D), c_float(eps),
                                       c_int(1 if accumulate else 0), c_int(dtype_code(y.dtype)), _stream()), "norm_add")
    return h


ACTIVATIONS = {"none": 0, "relu2": 1, "gelu_tanh": 2}


def bias_act(out: torch.Tensor, x: torch.Tensor, bias: Optional[torch.Tensor], activation: str) -> torch.Tensor:
    """out = act(x + bias) over rows of bias.numel() elements; act = none | relu2 (the square of relu) | gelu_tanh."""
    _cuda(out, x, bias); _contig(out, x, bias)
    if activation not in ACTIVATIONS:
        raise KernelError(f"bias_act: activation '{activation}' is not built; built: {sorted(ACTIVATIONS)}")
    D = x.shape[-1]
    if out.shape != x.shape or out.dtype != x.dtype or (bias is not None and (bias.dtype != torch.float32 or bias.numel() != D)):
        raise KernelError("bias_act: out like x; bias float32 [D]")
    _check(_resid32_lib().cvb_bias_act(_ptr(out), _ptr(x), _ptr(bias), c_int64(x.numel()), c_int(D), c_int(ACTIVATIONS[activation]),
                                       c_int(dtype_code(x.dtype)), _stream()), "bias_act")
    return out


def gated_norm(out: torch.Tensor, o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, groups: int, eps: float,
               gate_act: str = "sigmoid") -> torch.Tensor:
    """out[t, g, :] = RMSNorm(o[t, g, :]) * weight * sigmoid(gate[t, g, :]) (or * silu(gate): `gate_act` = "silu") over `groups` groups of weight.numel() elements;
    o float32 [T, groups * G]; gate a view of [T, groups * G] columns inside rows of gate.stride(0) elements."""
    _cuda(out, o, gate, weight); _contig(out, o, weight)
    T = o.shape[0]
    G = weight.numel()
    if gate_act not in ("sigmoid", "silu"):
        raise KernelError("gated_norm: gate_act is sigmoid or silu")
    if (o.dtype != torch.float32 or o.shape[1] != groups * G or out.shape != o.shape or gate.dtype != out.dtype or gate.dim() != 2
            or gate.shape != o.shape or gate.stride(1) != 1 or weight.dtype != torch.float32):
        raise KernelError("gated_norm: o float32 [T, groups * G]; out and gate [T, groups * G] of the activations' type; weight float32 [G]")
    _check(_resid32_lib().cvb_gated_norm(_ptr(out), _ptr(o), _ptr(gate), c_int(gate.stride(0)), _ptr(weight), c_int(T), c_int(groups),
                                         c_int(G), c_float(eps), c_int(1 if gate_act == "silu" else 0), c_int(dtype_code(out.dtype)), _stream()), "gated_norm")
    return out


# ---- sublayers wrapped twice, read through a convolution and left through a gate; attention with whole-projection norms ----

_sandwich = None


def _sandwich_lib():
    global _sandwich
    if _sandwich is None:
        lib = load_library("sandwich")
        for name in ("cvb_input_conv", "cvb_gated_norm_add", "cvb_glu_clamped", "cvb_add_gated_rows", "cvb_wide_qk_prep"):
            getattr(lib, name).restype = c_int
        _sandwich = lib
    return _sandwich


def input_conv(out: torch.Tensor, a: torch.Tensor, taps: torch.Tensor, state: torch.Tensor, hist_off: int, seq_of_token, cu_seqlens,
               state_slots) -> torch.Tensor:
    """out[t, c] = a[t, c] + sum_j taps[j, c] * a[t - K + 1 + j, c]: a causal convolution over time per channel, added to its
    input; `taps` holds one row of D weights per tap, the oldest tap first.  What lies before the step's portion comes from the request's history: K - 1 rows of D floats from `hist_off` on in
    the request's state row (oldest first)."""
    _cuda(out, a, taps, state, seq_of_token, cu_seqlens, state_slots); _contig(out, a, taps, seq_of_token, cu_seqlens, state_slots)
    sp, sf, n_slots = _state_args(state)
    T, D = a.shape
    if out.shape != a.shape or out.dtype != a.dtype or taps.dtype != torch.float32 or taps.dim() != 2 or taps.shape[1] != D:
        raise KernelError("input_conv: out like a [T, D]; taps float32 [K, D]")
    _check(_sandwich_lib().cvb_input_conv(_ptr(out), _ptr(a), _ptr(taps), c_int(T), c_int(D), c_int(taps.shape[0]), sp, sf,
                                          c_int64(hist_off), _ptr(seq_of_token), _ptr(cu_seqlens), _ptr(state_slots), c_int(n_slots),
                                          c_int(dtype_code(a.dtype)), _ptr(error_flag(a.device)), _stream()), "input_conv")
    return out


def gated_norm_add(h: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float, gate: Optional[torch.Tensor] = None,
                   gate_bias: Optional[torch.Tensor] = None, next_weight: Optional[torch.Tensor] = None, next_eps: float = 0.0,
                   next_out: Optional[torch.Tensor] = None, history=None) -> torch.Tensor:
    """h (float32 [T, D]) += RMSNorm(y * sigmoid(gate + gate_bias)) * weight.  With `next_weight` also next_out = RMSNorm(h) *
    next_weight (the activations' type).  `history` = (a, taps, state, hist_off, seq_of_token, cu_seqlens, state_slots): the
    last taps - 1 rows of `a` of every request's portion (older ones from the old history) become its convolution history;
    `next_out` must not be `a` then."""
    _cuda(h, y, weight, gate, gate_bias, next_weight, next_out); _contig(h, y, weight, gate, gate_bias, next_weight, next_out)
    T, D = h.shape
    if (h.dtype != torch.float32 or y.shape != h.shape or weight.dtype != torch.float32 or weight.numel() != D
            or (gate is not None and (gate.shape != h.shape or gate.dtype != y.dtype))
            or (gate_bias is not None and (gate_bias.dtype != torch.float32 or gate_bias.numel() != D))
            or (next_weight is not None and (next_out is None or next_out.shape != h.shape or next_out.dtype != y.dtype
                                             or next_weight.dtype != torch.float32 or next_weight.numel() != D))):
        raise KernelError("gated_norm_add: h float32 [T, D]; y, gate, next_out [T, D] of the activations' type; weights float32 [D]")
    a = st = sot = cu = slots = None
    sf, n_slots, hist_off, taps = c_int64(0), 0, 0, 0
    if history is not None:
        a, taps, state, hist_off, sot, cu, slots = history
        _cuda(a, state, sot, cu, slots); _contig(a, sot, cu, slots)
        st, sf, n_slots = _state_args(state)
        if a.shape != h.shape or a.dtype != y.dtype or (next_out is not None and next_out.data_ptr() == a.data_ptr()):
            raise KernelError("gated_norm_add: the history's rows are [T, D] of the activations' type, apart from next_out")
    _check(_sandwich_lib().cvb_gated_norm_add(
        _ptr(h), _ptr(y), _ptr(gate), _ptr(gate_bias), _ptr(weight), c_float(eps), _ptr(next_weight), c_float(next_eps), _ptr(next_out),
        c_int(T), c_int(D), _ptr(a), st if st is not None else _ptr(None), sf, c_int64(hist_off), c_int(int(taps)), _ptr(sot), _ptr(cu),
        _ptr(slots), c_int(n_slots), c_int(dtype_code(y.dtype)), _stream()), "gated_norm_add")
    return h


def glu_clamped(out: torch.Tensor, gate_up: torch.Tensor, limit: float, alpha: float) -> torch.Tensor:
    """out = g * sigmoid(alpha * g) * (u + 1), g = min(gate, limit), u = clamp(up, -limit, limit); gate_up [T, 2 I] (gate columns, then up)."""
    _cuda(out, gate_up); _contig(out, gate_up)
    T, I = out.shape
    if gate_up.shape != (T, 2 * I) or gate_up.dtype != out.dtype:
        raise KernelError("glu_clamped: gate_up must be [T, 2I] for out [T, I]")
    _check(_sandwich_lib().cvb_glu_clamped(_ptr(out), _ptr(gate_up), c_int(T), c_int(I), c_float(limit), c_float(alpha),
                                           c_int(dtype_code(out.dtype)), _stream()), "glu_clamped")
    return out


def add_gated_rows(y: torch.Tensor, s: torch.Tensor, z: torch.Tensor) -> torch.Tensor:
    """y[t, :] += sigmoid(z[t]) * s[t, :]; z float32, one element per row (a column of a wider float32 tensor will do)."""
    _cuda(y, s, z); _contig(y, s)
    T, D = y.shape
    if s.shape != y.shape or s.dtype != y.dtype or z.dtype != torch.float32 or z.dim() != 1 or z.shape[0] != T:
        raise KernelError("add_gated_rows: s like y [T, D]; z float32 [T]")
    _check(_sandwich_lib().cvb_add_gated_rows(_ptr(y), _ptr(s), _ptr(z), c_int(z.stride(0) if T > 0 else 1), c_int(T), c_int(D),
                                              c_int(dtype_code(y.dtype)), _stream()), "add_gated_rows")
    return y


def wide_qk_prep(q_out: torch.Tensor, packed: torch.Tensor, q_weight: torch.Tensor, positions: torch.Tensor, eps: float,
                 temp_coef: float, temp_every: int, num_kv_heads: int, dim: int, vdim: int, pages: Optional[torch.Tensor] = None,
                 k_weight: Optional[torch.Tensor] = None, slots: Optional[torch.Tensor] = None, page_size: int = 1) -> torch.Tensor:
    """q_out = RMSNorm over the WHOLE query projection (the first q_out.shape[1] columns of `packed`) * q_weight * (1 + temp_coef *
    ln(floor((p + 1) / temp_every) + 1)) (temp_every = 0: no temperature).  With `pages`: the key projection behind the queries
    is normed the same way with k_weight and written, with the value projection behind it, into pages [page, kv head, slot,
    dim + vdim] at `slots`."""
    _cuda(q_out, packed, q_weight, positions, pages, k_weight, slots); _contig(q_out, packed, q_weight, positions, pages, k_weight, slots)
    T, nq = q_out.shape
    write = pages is not None
    if (q_out.dtype != packed.dtype or packed.shape[0] != T or q_weight.dtype != torch.float32 or q_weight.numel() != nq
            or positions.dtype != torch.int32
            or (write and (pages.dtype != packed.dtype or k_weight is None or k_weight.dtype != torch.float32
                           or k_weight.numel() != num_kv_heads * dim or slots is None or slots.dtype != torch.int32))):
        raise KernelError("wide_qk_prep: q_out [T, nq] and pages like packed; weights float32; positions, slots int32")
    num_pages = pages.numel() // (num_kv_heads * page_size * (dim + vdim)) if write else 0
    _check(_sandwich_lib().cvb_wide_qk_prep(
        _ptr(q_out), _ptr(pages), _ptr(packed), c_int(T), c_int(packed.shape[1]), _ptr(q_weight), _ptr(k_weight), _ptr(positions),
        _ptr(slots), c_int(nq), c_int(num_kv_heads), c_int(dim), c_int(vdim), c_int(page_size), c_int64(num_pages), c_float(eps),
        c_float(temp_coef), c_int(temp_every), c_int(1 if write else 0), c_int(dtype_code(packed.dtype)),
        _ptr(error_flag(packed.device)), _stream()), "wide_qk_prep")
    return q_out


_attn_bias = None


def _attn_bias_lib():
    global _attn_bias
    if _attn_bias is None:
        lib = load_library("attn_bias")
        lib.cvb_attn_bias_bf16.restype = c_int
        _attn_bias = lib
    return _attn_bias


def attn_bias_supported(dtype: torch.dtype, num_heads: int, num_kv_heads: int, dim: int, vdim: int) -> bool:
    """Whether the tensor-core kernel takes the shape (csrc/attention_bias.cu): bf16, key and value sizes 16 to 128 in steps
    of 16, up to 64 query heads per kv head."""
    return (dtype == torch.bfloat16 and dim % 16 == 0 and 16 <= dim <= 128 and vdim % 16 == 0 and 16 <= vdim <= 128
            and num_kv_heads > 0 and num_heads % num_kv_heads == 0 and num_heads // num_kv_heads <= 64)


def attn_bias_bf16(out: torch.Tensor, q: torch.Tensor, pages: torch.Tensor, block_tables: torch.Tensor, cu_seqlens: torch.Tensor,
                   positions: torch.Tensor, num_seqs: int, num_tiles: int, num_heads: int, num_kv_heads: int, dim: int, vdim: int,
                   page_size: int, scale: float, bias: torch.Tensor, all_single: bool = False, splits: int = 1,
                   scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of prompt portions and decoded tokens over pages [kv head, slot, dim + vdim] whose entries hold a key and,
    behind it, its value; the score of key j for the token at position p receives bias[h, min(p - j, L - 1)] (float32 [H, L])
    after the scale.  `num_tiles` as attn_keys_tiles gives it.  `all_single`: every request brings exactly one token; with
    `splits` > 1 that many blocks share a (request, kv head), through `scratch` (float32, attn_keys_scratch_floats with vdim
    as the head size) and a merge kernel."""
    _cuda(out, q, pages, block_tables, cu_seqlens, positions, bias); _contig(out, q, pages, block_tables, cu_seqlens, positions, bias)
    if q.dtype != torch.bfloat16 or pages.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("attn_bias_bf16 takes bf16 queries, pages and output")
    if block_tables.dtype != torch.int32 or block_tables.dim() != 2 or cu_seqlens.dtype != torch.int32 or positions.dtype != torch.int32:
        raise KernelError("attn_bias_bf16: block_tables [S, W], cu_seqlens and positions must be int32")
    if bias.dtype != torch.float32 or bias.dim() != 2 or bias.shape[0] != num_heads:
        raise KernelError("attn_bias_bf16: bias is float32 [H, L]")
    num_pages = pages.numel() // (num_kv_heads * page_size * (dim + vdim))
    if splits > 1 and (scratch is None or scratch.dtype != torch.float32 or not scratch.is_cuda or not scratch.is_contiguous()):
        raise KernelError("attn_bias_bf16: splits need a contiguous float32 CUDA scratch")
    _check(_attn_bias_lib().cvb_attn_bias_bf16(
        _ptr(out), _ptr(q), c_int(q.shape[1]), _ptr(pages), _ptr(block_tables), c_int(block_tables.shape[1]), _ptr(cu_seqlens),
        _ptr(positions), c_int(num_seqs), c_int(num_tiles), c_int(num_heads), c_int(num_kv_heads), c_int(dim), c_int(vdim),
        c_int(page_size), c_float(scale), _ptr(bias), c_int(bias.shape[1]), c_int(num_pages), c_int(1 if all_single else 0),
        c_int(splits), _ptr(scratch), c_int64(scratch.numel() if scratch is not None else 0),
        _ptr(error_flag(q.device)), _stream()), "attn_bias_bf16", kernels=2 if all_single and splits > 1 else 1)
    return out


def paged_attention_entries(out: torch.Tensor, q: torch.Tensor, pages: torch.Tensor, block_tables: torch.Tensor,
                            seq_of_token: torch.Tensor, positions: torch.Tensor, num_heads: int, num_kv_heads: int, dim: int,
                            vdim: int, page_size: int, scale: float, bias: Optional[torch.Tensor] = None, window: int = 0,
                            num_tokens: Optional[int] = None) -> torch.Tensor:
    """The general attention kernel (one block per token and query head, any sizes, float32 or bf16) over pages [page, kv head,
    slot, dim + vdim] whose entries hold a key and, behind it, its value.  `bias` float32 [H, L]: the score of key j for the
    token at position p receives bias[h, min(p - j, L - 1)] after the scale."""
    _cuda(out, q, pages, block_tables, seq_of_token, positions, bias); _contig(out, q, pages, block_tables, seq_of_token, positions, bias)
    T = q.shape[0] if num_tokens is None else num_tokens
    if q.dtype != pages.dtype or out.dtype != q.dtype:
        raise KernelError("paged_attention_entries: q, out and the cache pages must share one element type")
    if block_tables.dtype != torch.int32 or block_tables.dim() != 2 or seq_of_token.dtype != torch.int32 or positions.dtype != torch.int32:
        raise KernelError("paged_attention_entries: block_tables int32 [S, W]; seq_of_token and positions int32")
    if num_heads % num_kv_heads or out.numel() < T * num_heads * vdim:
        raise KernelError("paged_attention_entries: head counts or the size of out do not fit")
    if bias is not None and (bias.dtype != torch.float32 or bias.dim() != 2 or bias.shape[0] != num_heads):
        raise KernelError("paged_attention_entries: bias is float32 [H, L]")
    num_pages = pages.numel() // (num_kv_heads * page_size * (dim + vdim))
    _check(core().cvb_paged_attention_entries(
        _ptr(out), _ptr(q), _ptr(pages), _ptr(block_tables), c_int(block_tables.shape[1]), _ptr(seq_of_token), _ptr(positions),
        c_int(T), c_int(num_heads), c_int(num_kv_heads), c_int(dim), c_int(vdim), c_int(page_size), c_int(window),
        c_int(q.shape[1]), c_float(scale), c_int(num_pages), _ptr(bias), c_int(bias.shape[1] if bias is not None else 0),
        c_int(dtype_code(q.dtype)), _ptr(error_flag(q.device)), _stream()), "paged_attention_entries")
    return out


# ---- attention over a cache of latent vectors: what stands around the attention kernel ------------------------------

_latent = None


def _latent_lib():
    global _latent
    if _latent is None:
        lib = load_library("latent")
        for name in ("cvb_latent_prep", "cvb_latent_q_assemble", "cvb_head_gate"):
            getattr(lib, name).restype = c_int
        _latent = lib
    return _latent


def latent_prep(packed: torch.Tensor, cq_out: Optional[torch.Tensor], q_off: int, q_rank: int, q_weight: Optional[torch.Tensor],
                pages: Optional[torch.Tensor], kv_off: int, rank: int, rot_width: int, rot: int, kv_weight: Optional[torch.Tensor],
                cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], positions: torch.Tensor, slots: Optional[torch.Tensor],
                eps: float) -> None:
    """Per row of `packed`: cq_out = RMSNorm(packed[q_off : q_off + q_rank]) * q_weight, and into the row's cache slot
    [RMSNorm(packed[kv_off : kv_off + rank]) * kv_weight | rotation of the rot_width elements behind them] (their first `rot`
    elements turn in pairs (2i, 2i+1) by cos/sin[position]).  `cq_out` or `pages` may be None."""
    _cuda(packed, cq_out, q_weight, pages, kv_weight, cos, sin, positions, slots)
    _contig(packed, cq_out, q_weight, pages, kv_weight, cos, sin, positions, slots)
    T = packed.shape[0]
    for t in (cq_out, pages):
        if t is not None and t.dtype != packed.dtype:
            raise KernelError("latent_prep: outputs share the packed rows' element type")
    for t in (q_weight, kv_weight, cos, sin):
        if t is not None and t.dtype != torch.float32:
            raise KernelError("latent_prep: norm weights and angle tables are float32")
    if positions.dtype != torch.int32 or (slots is not None and slots.dtype != torch.int32):
        raise KernelError("latent_prep: positions and slots are int32")
    if pages is not None and (slots is None or (rot > 0 and (cos is None or cos.shape[1] != rot // 2))):
        raise KernelError("latent_prep: a cache write needs slots and angle tables [positions, rot / 2]")
    total_slots = pages.numel() // (rank + rot_width) if pages is not None else 0
    _check(_latent_lib().cvb_latent_prep(
        _ptr(cq_out), _ptr(pages), _ptr(packed), c_int(T), c_int(packed.shape[1]), c_int(q_off), c_int(q_rank), _ptr(q_weight),
        c_int(kv_off), c_int(rank), c_int(rot_width), c_int(rot), _ptr(kv_weight), _ptr(cos), _ptr(sin),
        c_int(cos.shape[0] if cos is not None else 1), _ptr(positions), _ptr(slots), c_int64(total_slots), c_float(eps),
        c_int(dtype_code(packed.dtype)), _ptr(error_flag(packed.device)), _stream()), "latent_prep")


def latent_q_assemble(q_out: torch.Tensor, q_abs: torch.Tensor, q: torch.Tensor, num_heads: int, nope: int, rank: int, rot_width: int,
                      rot: int, cos: torch.Tensor, sin: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
    """q_out[t, h] = [q_abs[h, t, :rank] | rotation of q[t, h, nope : nope + rot_width]]."""
    _cuda(q_out, q_abs, q, cos, sin, positions); _contig(q_out, q_abs, q, cos, sin, positions)
    T = q.shape[0]
    if (q_out.dtype != q.dtype or q_abs.dtype != q.dtype or cos.dtype != torch.float32 or sin.dtype != torch.float32
            or positions.dtype != torch.int32 or q_out.numel() != T * num_heads * (rank + rot_width)
            or q_abs.numel() != T * num_heads * rank or (rot > 0 and cos.shape[1] != rot // 2)):
        raise KernelError("latent_q_assemble: q [T, H * (nope + rot_width)], q_abs [H, T, rank], q_out [T, H, rank + rot_width]")
    _check(_latent_lib().cvb_latent_q_assemble(
        _ptr(q_out), _ptr(q_abs), _ptr(q), c_int(T), c_int(q.shape[1]), c_int(num_heads), c_int(nope), c_int(rank), c_int(rot_width),
        c_int(rot), _ptr(cos), _ptr(sin), c_int(cos.shape[0]), _ptr(positions), c_int(dtype_code(q.dtype)),
        _ptr(error_flag(q.device)), _stream()), "latent_q_assemble")
    return q_out


def head_gate(out: torch.Tensor, o: torch.Tensor, gate: torch.Tensor, num_heads: int, vdim: int, per_element: bool = False) -> torch.Tensor:
    """out[t, h * vdim + j] = o[h, t, j] * sigmoid(gate[t, h]); gate is a view of H columns inside rows of gate.stride(0).
    `per_element`: the gate has H * vdim columns, one per element: out[t, i] = o[..] * sigmoid(gate[t, i])."""
    _cuda(out, o, gate); _contig(out, o)
    T = out.shape[0]
    cols = num_heads * vdim if per_element else num_heads
    if (out.dtype != o.dtype or gate.dtype != o.dtype or out.shape[1] != num_heads * vdim or o.numel() != T * num_heads * vdim
            or gate.shape != (T, cols) or gate.stride(1) != 1):
        raise KernelError("head_gate: o [H, T, vdim], out [T, H * vdim], gate [T, H] (or [T, H * vdim]) of one element type")
    _check(_latent_lib().cvb_head_gate(_ptr(out), _ptr(o), _ptr(gate), c_int(T), c_int(gate.stride(0)), c_int(num_heads), c_int(vdim),
                                       c_int(1 if per_element else 0), c_int(dtype_code(o.dtype)), _stream()), "head_gate")
    return out


# ---- mixers with a matrix of fixed size per request and head -------------------------------------------------------------

_recurrent = None


def _recurrent_lib():
    global _recurrent
    if _recurrent is None:
        lib = load_library("recurrent")
        for name in ("cvb_lightning_prep", "cvb_lightning_scan", "cvb_delta_prep", "cvb_conv_history", "cvb_delta_scan"):
            getattr(lib, name).restype = c_int
        _recurrent = lib
    return _recurrent


def _state_args(state: torch.Tensor):
    if state.dtype != torch.float32 or not state.is_contiguous() or state.dim() != 2:
        raise KernelError("a recurrent state is float32 [slots, floats]")
    return _ptr(state), c_int64(state.shape[1]), state.shape[0]


def lightning_prep(qf: torch.Tensor, kf: torch.Tensor, vf: torch.Tensor, packed: torch.Tensor, q_off: int, k_off: int, v_off: int) -> None:
    """qf, kf [T, H * dim] and vf [T, H * vdim] (float32) = silu of the packed projection's column ranges from q_off, k_off, v_off."""
    _cuda(qf, kf, vf, packed); _contig(qf, kf, vf, packed)
    T = packed.shape[0]
    if (qf.dtype != torch.float32 or kf.dtype != torch.float32 or vf.dtype != torch.float32 or qf.shape != kf.shape
            or qf.shape[0] != T or vf.shape[0] != T):
        raise KernelError("lightning_prep: qf, kf [T, H * dim] and vf [T, H * vdim] are float32")
    _check(_recurrent_lib().cvb_lightning_prep(_ptr(qf), _ptr(kf), _ptr(vf), _ptr(packed), c_int(T), c_int(packed.shape[1]), c_int(q_off),
                                               c_int(k_off), c_int(v_off), c_int(qf.shape[1]), c_int(vf.shape[1]),
                                               c_int(dtype_code(packed.dtype)), _stream()), "lightning_prep")


def lightning_scan(out: torch.Tensor, qf: torch.Tensor, kf: torch.Tensor, vf: torch.Tensor, state: torch.Tensor, decay: torch.Tensor,
                   cu_seqlens: torch.Tensor, state_slots: torch.Tensor, num_seqs: int, num_heads: int, dim: int, vdim: int) -> torch.Tensor:
    """Per request and head, over the request's tokens of this step: S <- decay_h S + k v^T, out = S^T q; q, k [T, H * dim] and
    v [T, H * vdim] float32; S [dim, vdim] float32 at the front of the request's state row.  out float32 [T, H * vdim]."""
    _cuda(out, qf, kf, vf, state, decay, cu_seqlens, state_slots); _contig(out, qf, kf, vf, decay, cu_seqlens, state_slots)
    sp, sf, n_slots = _state_args(state)
    T = qf.shape[0]
    if (out.dtype != torch.float32 or out.shape != (T, num_heads * vdim) or decay.dtype != torch.float32 or decay.numel() != num_heads
            or cu_seqlens.dtype != torch.int32 or state_slots.dtype != torch.int32 or qf.dtype != torch.float32
            or kf.dtype != torch.float32 or vf.dtype != torch.float32 or qf.shape != (T, num_heads * dim) or kf.shape != qf.shape
            or vf.shape != out.shape):
        raise KernelError("lightning_scan: q, k float32 [T, H * dim]; v, out float32 [T, H * vdim]; decay float32 [H]; cu_seqlens, "
                          "state_slots int32")
    _check(_recurrent_lib().cvb_lightning_scan(
        _ptr(out), _ptr(qf), _ptr(kf), _ptr(vf), sp, sf, _ptr(decay), _ptr(cu_seqlens), _ptr(state_slots), c_int(n_slots), c_int(num_seqs),
        c_int(num_heads), c_int(dim), c_int(vdim), _ptr(error_flag(out.device)), _stream()), "lightning_scan")
    return out


def delta_prep(qn, kn, vv, gg, bb, packed: torch.Tensor, qkv_off: int, conv_w: torch.Tensor, a: torch.Tensor, dt_bias: torch.Tensor,
               a_log: torch.Tensor, b: torch.Tensor, state: torch.Tensor, conv_off: int, seq_of_token, cu_seqlens, state_slots,
               num_heads: int, num_kv_heads: int, dim: int, vdim: int, decay_dim: Optional[int] = None) -> None:
    """Per token: convolutions with silu, unit q and k, sigmoid(b), the decay; all outputs float32 (see csrc/recurrent.cu).
    `decay_dim`: decays per head, `dim` (one per key channel, the default) or 1 (one per head)."""
    _cuda(qn, kn, vv, gg, bb, packed, conv_w, a, dt_bias, a_log, b, state, seq_of_token, cu_seqlens, state_slots)
    _contig(qn, kn, vv, gg, bb, packed, conv_w, a, dt_bias, a_log, b, seq_of_token, cu_seqlens, state_slots)
    sp, sf, n_slots = _state_args(state)
    T = packed.shape[0]
    H, G = num_heads, num_kv_heads
    C = 2 * G * dim + H * vdim
    gd = dim if decay_dim is None else int(decay_dim)
    for t_, n_ in ((qn, T * G * dim), (kn, T * G * dim), (vv, T * H * vdim), (gg, T * H * gd), (bb, T * H), (a, T * H * gd), (b, T * H),
                   (dt_bias, H * gd), (a_log, H)):
        if t_.dtype != torch.float32 or t_.numel() != n_:
            raise KernelError("delta_prep: float32 buffers of the sizes the head counts give")
    if conv_w.dtype != torch.float32 or conv_w.dim() != 2 or conv_w.shape[0] != C:
        raise KernelError("delta_prep: conv_w float32 [channels, taps]")
    _check(_recurrent_lib().cvb_delta_prep(
        _ptr(qn), _ptr(kn), _ptr(vv), _ptr(gg), _ptr(bb), _ptr(packed), c_int(T), c_int(packed.shape[1]), c_int(qkv_off), _ptr(conv_w),
        c_int(conv_w.shape[1]), _ptr(a), _ptr(dt_bias), _ptr(a_log), _ptr(b), sp, sf, c_int64(conv_off), _ptr(seq_of_token),
        _ptr(cu_seqlens), _ptr(state_slots), c_int(n_slots), c_int(H), c_int(G), c_int(dim), c_int(vdim), c_int(gd), c_int(dtype_code(packed.dtype)),
        _ptr(error_flag(packed.device)), _stream()), "delta_prep")


def conv_history(state: torch.Tensor, conv_off: int, packed: torch.Tensor, qkv_off: int, channels: int, taps: int, cu_seqlens,
                 state_slots, num_seqs: int) -> None:
    """The last taps - 1 raw inputs of every request's portion (older ones from the old history) become its history."""
    _cuda(state, packed, cu_seqlens, state_slots); _contig(packed, cu_seqlens, state_slots)
    sp, sf, n_slots = _state_args(state)
    _check(_recurrent_lib().cvb_conv_history(sp, sf, c_int64(conv_off), _ptr(packed), c_int(packed.shape[1]), c_int(qkv_off), c_int(channels),
                                             c_int(taps), _ptr(cu_seqlens), _ptr(state_slots), c_int(n_slots), c_int(num_seqs),
                                             c_int(dtype_code(packed.dtype)), _stream()), "conv_history", kernels=1 if taps > 1 else 0)


def delta_scan(out, qn, kn, vv, gg, bb, state: torch.Tensor, cu_seqlens, state_slots, num_seqs: int, num_heads: int, num_kv_heads: int,
               dim: int, vdim: int, decay_dim: Optional[int] = None) -> torch.Tensor:
    """Per request and head: S <- diag(g) S; u = b (v - S^T k); S <- S + k u^T; out = S^T q.  out float32 [T, H * vdim].
    gg is [T, H * dim], or [T, H] with `decay_dim` = 1 (one decay per head: S <- g S)."""
    _cuda(out, qn, kn, vv, gg, bb, state, cu_seqlens, state_slots); _contig(out, qn, kn, vv, gg, bb, cu_seqlens, state_slots)
    sp, sf, n_slots = _state_args(state)
    if out.dtype != torch.float32:
        raise KernelError("delta_scan: out is float32")
    _check(_recurrent_lib().cvb_delta_scan(_ptr(out), _ptr(qn), _ptr(kn), _ptr(vv), _ptr(gg), _ptr(bb), sp, sf, _ptr(cu_seqlens),
                                           _ptr(state_slots), c_int(n_slots), c_int(num_seqs), c_int(num_heads), c_int(num_kv_heads),
                                           c_int(dim), c_int(vdim), c_int(dim if decay_dim is None else int(decay_dim)),
                                           _ptr(error_flag(out.device)), _stream()), "delta_scan")
    return out


# ---- attention over keys that are also the values ------------------------------------------------------------------

_attn_keys = None


def _attn_keys_lib():
    global _attn_keys
    if _attn_keys is None:
        lib = load_library("attn_keys")
        lib.cvb_attn_keys_bf16.restype = c_int
        lib.cvb_attn_keys_supported.restype = c_int
        _attn_keys = lib
    return _attn_keys


def attn_keys_supported(dtype: torch.dtype, num_heads: int, num_kv_heads: int, head_dim: int, q_stride: int) -> bool:
    """The tensor-core kernel covers bf16, head sizes 16 to 128 in steps of 16, up to 64 query heads per kv head, and query
    rows that start on 16-byte boundaries."""
    return (dtype == torch.bfloat16 and q_stride % 8 == 0 and head_dim % 16 == 0 and 16 <= head_dim <= 128
            and num_kv_heads > 0 and num_heads % num_kv_heads == 0 and num_heads // num_kv_heads <= 64)


def attn_keys_scratch_floats(num_seqs: int, num_kv_heads: int, head_dim: int, splits: int) -> int:
    return num_seqs * num_kv_heads * splits * 16 * (head_dim + 2)


def attn_keys_decode_splits(num_seqs: int, num_kv_heads: int, visible_keys: int, sms: int = 148) -> int:
    """Blocks per (request, kv head) of a decode step: enough to give every SM a block while a warp keeps a tile of 32 keys
    or more (eight warps per block), at most 8."""
    pairs = max(1, num_seqs * num_kv_heads)
    tiles = max(1, (visible_keys + 31) // 32)
    splits = 1
    while splits < 8 and pairs * splits * 2 <= 2 * sms and tiles >= 8 * splits * 2:
        splits *= 2
    return splits


def attn_keys_tiles(q_lens, num_heads: int, num_kv_heads: int) -> int:
    """Blocks per kv head: per request ceil(tokens / (64 // group))."""
    tpt = 64 // (num_heads // num_kv_heads)
    return sum((n + tpt - 1) // tpt for n in q_lens)


def attn_keys_bf16(out: torch.Tensor, q: torch.Tensor, pages: torch.Tensor, block_tables: torch.Tensor, cu_seqlens: torch.Tensor,
                   positions: torch.Tensor, num_seqs: int, num_tiles: int, num_heads: int, num_kv_heads: int, head_dim: int,
                   page_size: int, scale: float, window: int = 0, keep_first: int = 0, all_single: bool = False, splits: int = 1,
                   scratch: Optional[torch.Tensor] = None, value_dim: Optional[int] = None, kv_heads_in_pages: int = 0) -> torch.Tensor:
    """Attention of prompt portions and decoded tokens over pages [kv head, slot, head_dim] whose keys are also the
    values; `q` may be the packed output of a projection (rows of q.shape[1] elements, queries first).  `all_single`:
    every request brings exactly one token (a decode step): a block per (request, kv head) whose warps share out the key
    tiles among themselves; with `splits` > 1 that many blocks share them, through `scratch` (float32,
    attn_keys_scratch_floats elements) and a merge kernel.  `value_dim` (a multiple of 16): only the first value_dim elements
    of a key are its value; out is [T, H * value_dim].  `kv_heads_in_pages` (a divisor of num_kv_heads): the pages hold fewer
    kv heads than the grid walks, the query heads of one stored head being dealt with as several groups (a decode step of more
    than 16 query heads per stored head)."""
    _cuda(out, q, pages, block_tables, cu_seqlens, positions); _contig(out, q, pages, block_tables, cu_seqlens, positions)
    if q.dtype != torch.bfloat16 or pages.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("attn_keys_bf16 takes bf16 queries, pages and output")
    if block_tables.dtype != torch.int32 or block_tables.dim() != 2 or cu_seqlens.dtype != torch.int32 or positions.dtype != torch.int32:
        raise KernelError("attn_keys_bf16: block_tables [S, W], cu_seqlens and positions must be int32")
    num_pages = pages.numel() // ((kv_heads_in_pages or num_kv_heads) * page_size * head_dim)
    if splits > 1 and (scratch is None or scratch.dtype != torch.float32 or not scratch.is_cuda or not scratch.is_contiguous()):
        raise KernelError("attn_keys_bf16: splits need a contiguous float32 CUDA scratch")
    _check(_attn_keys_lib().cvb_attn_keys_bf16(
        _ptr(out), _ptr(q), c_int(q.shape[1]), _ptr(pages), _ptr(block_tables), c_int(block_tables.shape[1]), _ptr(cu_seqlens),
        _ptr(positions), c_int(num_seqs), c_int(num_tiles), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim),
        c_int(head_dim if value_dim is None else value_dim), c_int(page_size), c_int(window), c_int(keep_first), c_float(scale),
        c_int(num_pages), c_int(1 if all_single else 0),
        c_int(splits), _ptr(scratch), c_int64(scratch.numel() if scratch is not None else 0), c_int(kv_heads_in_pages),
        _ptr(error_flag(q.device)), _stream()), "attn_keys_bf16", kernels=2 if all_single and splits > 1 else 1)
    return out


# ---- routed feed-forward ---------------------------------------------------------------------------------------

_moe = None


def _moe_lib():
    global _moe
    if _moe is None:
        lib = load_library("moe")
        for name in ("cvb_route_topk", "cvb_expert_rows", "cvb_sort_pairs_padded", "cvb_combine_pairs_bf16"):
            getattr(lib, name).restype = c_int
        _moe = lib
    return _moe


def route_topk(ids: torch.Tensor, weights: torch.Tensor, x: torch.Tensor, router: torch.Tensor,
               bias: Optional[torch.Tensor], over_all: bool = False, scale: float = 1.0,
               extra_out: Optional[torch.Tensor] = None, logistic: bool = False) -> None:
    """ids, weights [T, top]: the `top` largest of x @ router^T + bias (float32 arithmetic) and the softmax over them; with
    `over_all` the weights are `scale` times the winners' shares of the softmax over ALL experts instead.  `extra_out`
    float32 [T, n]: the last n rows of `router` are not experts, their products with x leave there unchanged.  `logistic`: the
    weights are `scale` times the winners' own sigmoid(z), with no sum over experts."""
    _cuda(ids, weights, x, router, bias, extra_out); _contig(ids, weights, x, router, bias, extra_out)
    T, D = x.shape
    extra = 0 if extra_out is None else extra_out.shape[1]
    E = router.shape[0] - extra
    top = ids.shape[1]
    if extra_out is not None and (extra_out.dtype != torch.float32 or extra_out.shape[0] != T or E <= 0):
        raise KernelError("route_topk: extra_out float32 [T, n] with n below the router's rows")
    if (ids.dtype != torch.int32 or weights.dtype != torch.float32 or router.dtype != torch.float32 or router.shape[1] != D
            or ids.shape != (T, top) or weights.shape != (T, top) or (bias is not None and (bias.dtype != torch.float32 or bias.numel() != E))):
        raise KernelError("route_topk: ids int32 and weights float32 [T, top]; router float32 [E, D]; bias float32 [E]")
    _check(_moe_lib().cvb_route_topk(_ptr(ids), _ptr(weights), _ptr(x), _ptr(router), _ptr(bias), c_int(T), c_int(D), c_int(E),
                                     c_int(top), c_int(2 if logistic else (1 if over_all else 0)), c_float(scale), c_int(extra), _ptr(extra_out),
                                     c_int(dtype_code(x.dtype)), _stream()), "route_topk")


def expert_rows(y: torch.Tensor, hid: torch.Tensor, x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor,
                w_gate_up: torch.Tensor, w_down: torch.Tensor, gated: bool = True, weight_on_input: bool = False) -> torch.Tensor:
    """y[t] = sum_k weights[t, k] * down_e(silu(gate_e x) * up_e x), e = ids[t, k]; w_gate_up [E, 2 ff, D], w_down [E, D, ff];
    with `weight_on_input` y[t] = sum_k expert_e(weights[t, k] * x) instead;
    `hid` [T * top, ff] is scratch.  Two kernels that read only the chosen experts' weights: for a few tokens, and for
    float32.  `gated=False`: an expert is down_e(relu(up_e x)^2) and w_gate_up holds [E, ff, D]."""
    _cuda(y, hid, x, ids, weights, w_gate_up, w_down); _contig(y, hid, x, ids, weights, w_gate_up, w_down)
    T, D = x.shape
    E, F2, _ = w_gate_up.shape
    F = F2 // 2 if gated else F2
    top = ids.shape[1]
    if (y.shape != x.shape or y.dtype != x.dtype or w_gate_up.dtype != x.dtype or w_down.dtype != x.dtype or hid.dtype != x.dtype
            or w_gate_up.shape != (E, (2 if gated else 1) * F, D) or w_down.shape != (E, D, F) or ids.dtype != torch.int32 or hid.numel() < T * top * F
            or weights.dtype != torch.float32 or ids.shape != weights.shape or ids.shape[0] != T):
        raise KernelError("expert_rows: x, y [T, D], hid [T * top, ff], w_gate_up [E, 2 ff, D] and w_down [E, D, ff] of one element "
                          "type; ids int32 and weights float32 [T, top]")
    _check(_moe_lib().cvb_expert_rows(_ptr(y), _ptr(hid), _ptr(x), _ptr(ids), _ptr(weights), _ptr(w_gate_up), _ptr(w_down), c_int(T),
                                      c_int(D), c_int(F), c_int(E), c_int(top), c_int(1 if gated else 0), c_int(1 if weight_on_input else 0),
                                      c_int(dtype_code(x.dtype)), _ptr(error_flag(x.device)), _stream()), "expert_rows", kernels=2)
    return y


def experts_grouped_supported(x_dtype: torch.dtype, D: int, F: int) -> bool:
    """The grouped tensor-core products take bf16 and sizes that are multiples of 8."""
    return x_dtype == torch.bfloat16 and D % 8 == 0 and F % 8 == 0


def grouped_rows_tcgen05(num_tokens: int, top: int, num_experts: int) -> int:
    """Rows of scratch the tcgen05 grouped path needs: every expert's segment starts on a multiple of 128 rows."""
    return ((num_tokens * top + 127) // 128 + num_experts) * 128


def experts_grouped_tcgen05(y, x, ids, weights, w_gate_up, w_down, tile_expert, row_token, slot_of, xs, hid, rows,
                            gated: bool = True, weight_on_input: bool = False) -> torch.Tensor:
    """More tokens on the tcgen05 tensor cores: the pairs are sorted by expert into segments that start on multiples of
    128 rows (device side), the tokens' rows are gathered into that order, and two grouped products (the first with the
    gated activation as its epilogue) run on csrc/gemm_tcgen05.cu's kernel; the last kernel adds a token's expert outputs
    up with its weights.  Scratch: R = grouped_rows_tcgen05(T, top, E) rows: tile_expert int32 [R / 128], row_token int32 [R],
    slot_of int32 [T * top], xs bf16 [R, D], hid bf16 [R, ff], rows bf16 [R, D]."""
    global _gemm
    _cuda(y, x, ids, weights, w_gate_up, w_down, tile_expert, row_token, slot_of, xs, hid, rows)
    _contig(y, x, ids, weights, w_gate_up, w_down, tile_expert, row_token, slot_of, xs, hid, rows)
    T, D = x.shape
    E, F2, _ = w_gate_up.shape
    F, top = (F2 // 2 if gated else F2), ids.shape[1]
    R = grouped_rows_tcgen05(T, top, E)
    bf = torch.bfloat16
    if (any(t.dtype != bf for t in (y, x, w_gate_up, w_down, xs, hid, rows)) or y.shape != x.shape or w_gate_up.shape != (E, F2, D)
            or w_down.shape != (E, D, F) or ids.dtype != torch.int32 or weights.dtype != torch.float32 or ids.shape != weights.shape
            or any(t.dtype != torch.int32 for t in (tile_expert, row_token, slot_of)) or tile_expert.numel() < R // 128
            or row_token.numel() < R or slot_of.numel() < T * top or xs.numel() < R * D or hid.numel() < R * F or rows.numel() < R * D):
        raise KernelError("experts_grouped_tcgen05: bf16 x, y, weights and scratch of the documented sizes; int32 index scratch")
    if _gemm is None:
        lib = load_library("gemm_bf16")
        lib.cvb_gemm_bf16_tcgen05.restype = c_int
        _gemm = lib
    _gemm.cvb_gemm_grouped_bf16_tcgen05.restype = c_int
    err = _ptr(error_flag(x.device))
    _check(_moe_lib().cvb_sort_pairs_padded(_ptr(tile_expert), _ptr(row_token), _ptr(slot_of), _ptr(ids), c_int(T), c_int(E), c_int(top),
                                            c_int(R // 128), err, _stream()), "sort_pairs_padded")
    xs2, hid2, rows2 = xs.view(-1)[:R * D].view(R, D), hid.view(-1)[:R * F].view(R, F), rows.view(-1)[:R * D].view(R, D)
    if weight_on_input:     # a pair's weight scales its row on the way in; the rows behind a segment keep what they held (finite)
        _moe_lib().cvb_scatter_pairs_scaled_bf16.restype = c_int
        _check(_moe_lib().cvb_scatter_pairs_scaled_bf16(_ptr(xs2), _ptr(x), _ptr(slot_of), _ptr(weights), c_int(T), c_int(D), c_int(top),
                                                        _stream()), "scatter_pairs_scaled")
    else:
        gather_rows(xs2, x, row_token.view(-1)[:R])
    if gated:
        _check(_gemm.cvb_gemm_grouped_bf16_tcgen05(_ptr(hid2), _ptr(xs2), _ptr(w_gate_up), _ptr(tile_expert), c_int(R), c_int(2 * F), c_int(E),
                                                   c_int(D), c_int(1), c_int(256), err, _stream()), "gemm_grouped_bf16_tcgen05")
    else:           # the squared relu is the epilogue
        up_256 = (T * top // 128 + 1) * ((F + 255) // 256)
        _check(_gemm.cvb_gemm_grouped_bf16_tcgen05(_ptr(hid2), _ptr(xs2), _ptr(w_gate_up), _ptr(tile_expert), c_int(R), c_int(F), c_int(E),
                                                   c_int(D), c_int(3), c_int(256 if up_256 >= 120 else 128), err, _stream()),
               "gemm_grouped_bf16_tcgen05")
    tiles_256 = (T * top // 128 + 1) * ((D + 255) // 256)
    _check(_gemm.cvb_gemm_grouped_bf16_tcgen05(_ptr(rows2), _ptr(hid2), _ptr(w_down), _ptr(tile_expert), c_int(R), c_int(D), c_int(E),
                                               c_int(F), c_int(0), c_int(256 if tiles_256 >= 120 else 128), err, _stream()),
           "gemm_grouped_bf16_tcgen05")
    _check(_moe_lib().cvb_combine_pairs_bf16(_ptr(y), _ptr(rows2), _ptr(slot_of), _ptr(None if weight_on_input else weights), c_int(T),
                                             c_int(D), c_int(top), _stream()),
           "combine_pairs")
    return y


def grouped_experts_preferred(num_pairs: int, num_experts: int, expert_bytes: int) -> bool:
    """Whether a step's (token, expert) pairs go through the grouped tcgen05 products rather than pair by pair.  Pair by pair
    reads an expert once per pair (the L2 absorbs repeats only for small experts) and costs two launches; grouped reads
    every chosen expert once and costs five.  Measured on a B200 (8 experts of 9 MB, 2 per token: 4 tokens 28 against 34 us,
    8 tokens 48 against 35; 8 experts of 151 MB: 1 token 92 against 110 us, 2 tokens 171 against 122, 8 tokens 623 against
    218; 64 experts of 9 MB, 4 per token: 8 tokens 94 against 94 us, 16 tokens 169 against 111)."""
    return (num_pairs >= 48 or num_pairs >= 2 * min(num_pairs, num_experts)
            or (num_pairs >= 3 and expert_bytes >= (64 << 20)))


def routed_experts(y, x, ids, weights, w_gate_up, w_down, workspace=None, kernel: str = "", gated: bool = True,
                   weight_on_input: bool = False) -> torch.Tensor:
    """The experts' outputs added up with the router's weights, by the kernels that suit the step: one or two tokens (and
    float32, and sizes that are no multiples of 8) read the chosen experts' weights pair by pair; more go through the
    grouped tcgen05 products (see grouped_experts_preferred).  `workspace` (parts.base.Workspace) lends the scratch;
    without it the scratch is allocated.  `kernel` = "rows" | "tcgen05" fixes the choice (where the shape allows it)."""
    T, D = x.shape
    E, F2, _ = w_gate_up.shape
    F, top = (F2 // 2 if gated else F2), ids.shape[1]
    expert_bytes = (3 if gated else 2) * D * F * x.element_size()
    grouped = kernel == "tcgen05" or (kernel == "" and grouped_experts_preferred(T * top, E, expert_bytes))
    if grouped and experts_grouped_supported(x.dtype, D, F):
        R = grouped_rows_tcgen05(T, top, E)

        def buf(name, n, dtype):
            if workspace is not None:
                # sized once for the largest step (the address must not move: captured graphs hold it)
                return workspace.flat(f"{name}_{E}_{top}", grouped_rows_tcgen05(workspace.max_tokens, top, E) * (n // R), dtype, zero=True)
            return torch.zeros(n, dtype=dtype, device=x.device)
        slot_of = workspace.rows("moe_slot_of", T, top, torch.int32) if workspace is not None else torch.empty(T * top, dtype=torch.int32, device=x.device)
        return experts_grouped_tcgen05(y, x, ids, weights, w_gate_up, w_down, buf("moe_tile_expert", R, torch.int32),
                                       buf("moe_row_token", R, torch.int32), slot_of, buf(f"moe_xs{D}", R * D, x.dtype),
                                       buf(f"moe_hid{F}", R * F, x.dtype), buf(f"moe_rows{D}", R * D, x.dtype), gated=gated,
                                       weight_on_input=weight_on_input)
    if workspace is not None:
        hid = workspace.rows("moe_hidden", T, top * F, x.dtype)
    else:
        hid = torch.empty((T, top * F), dtype=x.dtype, device=x.device)
    return expert_rows(y, hid, x, ids, weights, w_gate_up, w_down, gated=gated, weight_on_input=weight_on_input)


# ---- several residual streams read and written through learned weights (csrc/hyper.cu) ------------------------------------

_hyper = None


def _hyper_lib():
    global _hyper
    if _hyper is None:
        lib = load_library("hyper")
        for name in ("cvb_stream_embed", "cvb_stream_step"):
            getattr(lib, name).restype = c_int
        _hyper = lib
    return _hyper


def stream_embed(X: torch.Tensor, table: torch.Tensor, tokens: torch.Tensor, streams: int) -> torch.Tensor:
    """X (float32 [T, streams * D]): every stream of a token starts as its row of `table` [vocab, D]."""
    _cuda(X, table, tokens); _contig(X, table, tokens)
    T = X.shape[0]
    V, D = table.shape
    if X.dtype != torch.float32 or X.shape[1] != streams * D or tokens.dtype != torch.int32 or tokens.numel() < T:
        raise KernelError("stream_embed: X float32 [T, streams * D], tokens int32 [T]")
    _check(_hyper_lib().cvb_stream_embed(_ptr(X), _ptr(table), _ptr(tokens), c_int(T), c_int(streams), c_int(D), c_int(V),
                                         c_int(dtype_code(table.dtype)), _ptr(error_flag(X.device)), _stream()), "stream_embed")
    return X


def stream_step(X: torch.Tensor, streams: int, write=None, read=None, eps: float = 0.0, out: Optional[torch.Tensor] = None):
    """One pass over the streams X (float32 [T, streams * D], in place).  `write` = (y [T, D], mix float32 [S, S] (from, to),
    b float32 [S]): x_t <- sum_s mix[s, t] x_s + b_t y; y may be a pair of tensors, which are added in float.  `read` = (a float32 [S] or None for ones, g float32 with one element
    or None for 1) with `out` [T, D]: out = T(u / sqrt(mean(u^2) + eps) * g), u = sum_s a_s x_s, of the streams after the write."""
    T = X.shape[0]
    S = int(streams)
    D = X.shape[1] // S
    y = mix = b = a = g = None
    y2 = None
    if write is not None:
        y, mix, b = write
        if isinstance(y, (tuple, list)):
            y, y2 = (y[0], y[1]) if len(y) > 1 else (y[0], None)
    if read is not None:
        a, g = read
        if out is None:
            raise KernelError("stream_step: a read needs an output")
    _cuda(X, y, y2, mix, b, a, g, out); _contig(X, y, y2, mix, b, a, g, out)
    act = out.dtype if out is not None else y.dtype
    if X.dtype != torch.float32 or X.shape[1] != S * D:
        raise KernelError("stream_step: the streams are float32 [T, S * D]")
    if y2 is not None and (y2.shape != y.shape or y2.dtype != y.dtype):
        raise KernelError("stream_step: the two addends of a write are alike")
    if y is not None and (y.shape != (T, D) or y.dtype != act or mix.dtype != torch.float32 or mix.numel() != S * S
                          or b.dtype != torch.float32 or b.numel() != S):
        raise KernelError("stream_step: write = (y [T, D], mix float32 [S, S], b float32 [S])")
    if out is not None and (out.shape != (T, D) or (a is not None and (a.dtype != torch.float32 or a.numel() != S))
                            or (g is not None and (g.dtype != torch.float32 or g.numel() != 1))):
        raise KernelError("stream_step: read = (a float32 [S], g float32 [1]) into out [T, D]")
    _check(_hyper_lib().cvb_stream_step(_ptr(X), _ptr(y), _ptr(y2), _ptr(mix), _ptr(b), _ptr(a), _ptr(g), c_float(eps), _ptr(out), c_int(T),
                                        c_int(S), c_int(D), c_int(dtype_code(act)), _stream()), "stream_step")
    return out if out is not None else X


# ---- attention over entries of a key and its value with chunk, window, pooled blocks, cap, distance term and sink ----------

_attn_masked = None


def _attn_masked_lib():
    global _attn_masked
    if _attn_masked is None:
        lib = load_library("attn_masked")
        for name in ("cvb_masked_qkv_prep", "cvb_pool_entries", "cvb_attn_masked_general", "cvb_attn_masked_bf16"):
            getattr(lib, name).restype = c_int
        _attn_masked = lib
    return _attn_masked


def masked_qkv_prep(q_out: torch.Tensor, packed: torch.Tensor, num_heads: int, num_kv_heads: int, dim: int, vdim: int, eps: float,
                    q_weight: Optional[torch.Tensor] = None, k_weight: Optional[torch.Tensor] = None,
                    cos: Optional[torch.Tensor] = None, sin: Optional[torch.Tensor] = None, rot: int = 0, interleaved: bool = True,
                    positions: Optional[torch.Tensor] = None, pages: Optional[torch.Tensor] = None,
                    slots: Optional[torch.Tensor] = None, page_size: int = 1, planes: int = 1,
                    v_first_out: Optional[torch.Tensor] = None, v_first_in: Optional[torch.Tensor] = None,
                    lam: Optional[torch.Tensor] = None) -> torch.Tensor:
    """From rows [q: H dim | k: G dim | v: G vdim] of `packed`: q_out [T, H, dim] = turn(norm(q)); the entry [turn(norm(k)) | v']
    of every kv head into the token's cache slot of `pages` ([page, planes, G, slot, dim + vdim], plane 0), with
    v' = (1 - lam) v + lam v_first_in (v itself without v_first_in); `v_first_out` [T, G * vdim] receives v as projected."""
    _cuda(q_out, packed, q_weight, k_weight, cos, sin, positions, pages, slots, v_first_out, v_first_in, lam)
    _contig(q_out, packed, q_weight, k_weight, cos, sin, positions, pages, slots, v_first_out, v_first_in, lam)
    T = packed.shape[0]
    H, G = num_heads, num_kv_heads
    if q_out.dtype != packed.dtype or q_out.numel() != T * H * dim or packed.shape[1] < H * dim + G * (dim + vdim):
        raise KernelError("masked_qkv_prep: packed [T, H dim + G (dim + vdim)] and q_out [T, H, dim] of one element type")
    for w in (q_weight, k_weight):
        if w is not None and (w.dtype != torch.float32 or w.numel() != dim):
            raise KernelError("masked_qkv_prep: norm weights are float32 [dim]")
    max_pos = 0
    if rot:
        if cos is None or sin is None or cos.dtype != torch.float32 or sin.shape != cos.shape or cos.shape[1] != rot // 2 or positions is None:
            raise KernelError("masked_qkv_prep: a rotation needs float32 tables [positions, rot / 2] and the positions")
        max_pos = cos.shape[0]
    for t in (pages, v_first_out, v_first_in):
        if t is not None and t.dtype != packed.dtype:
            raise KernelError("masked_qkv_prep: pages and kept values share the rows' element type")
    for t in (v_first_out, v_first_in):
        if t is not None and t.numel() < T * G * vdim:
            raise KernelError("masked_qkv_prep: kept values are [T, G * vdim]")
    if v_first_in is not None and (lam is None or lam.dtype != torch.float32 or lam.numel() != 1):
        raise KernelError("masked_qkv_prep: mixing needs a float32 weight of one element")
    for t in (positions, slots):
        if t is not None and (t.dtype != torch.int32 or t.numel() < T):
            raise KernelError("masked_qkv_prep: positions and slots are int32 [T]")
    total_slots = pages.numel() // (planes * G * (dim + vdim)) if pages is not None else 0
    _check(_attn_masked_lib().cvb_masked_qkv_prep(
        _ptr(q_out), _ptr(packed), c_int(T), c_int(packed.shape[1]), _ptr(q_weight), _ptr(k_weight), _ptr(cos if rot else None),
        _ptr(sin if rot else None), _ptr(positions), _ptr(slots), _ptr(pages), _ptr(v_first_out), _ptr(v_first_in), _ptr(lam),
        c_int(H), c_int(G), c_int(dim), c_int(vdim), c_int(rot), c_int(1 if interleaved else 0), c_int(planes), c_int(page_size),
        c_int(max_pos), c_float(eps), c_int64(total_slots), c_int(dtype_code(packed.dtype)), _ptr(error_flag(packed.device)),
        _stream()), "masked_qkv_prep")
    return q_out


def pool_entries(pages: torch.Tensor, block_tables: torch.Tensor, seq_of_token: torch.Tensor, positions: torch.Tensor,
                 num_tokens: int, num_kv_heads: int, entry_width: int, pool: int, page_size: int) -> None:
    """Tokens of the step whose position closes a block of `pool` positions write the mean of the block's entries (plane 0 of
    `pages` [page, 2, G, slot, entry_width]) into plane 1 at the place of position (p + 1) / pool - 1."""
    _cuda(pages, block_tables, seq_of_token, positions); _contig(pages, block_tables, seq_of_token, positions)
    if block_tables.dtype != torch.int32 or seq_of_token.dtype != torch.int32 or positions.dtype != torch.int32:
        raise KernelError("pool_entries: index tensors are int32")
    num_pages = pages.numel() // (2 * num_kv_heads * page_size * entry_width)
    _check(_attn_masked_lib().cvb_pool_entries(_ptr(pages), _ptr(block_tables), c_int(block_tables.shape[1]), _ptr(seq_of_token),
                                               _ptr(positions), c_int(num_tokens), c_int(num_kv_heads), c_int(entry_width), c_int(pool),
                                               c_int(page_size), c_int(num_pages), c_int(dtype_code(pages.dtype)),
                                               _ptr(error_flag(pages.device)), _stream()), "pool_entries")


def attn_masked_general(out: torch.Tensor, q: torch.Tensor, pages: torch.Tensor, block_tables: torch.Tensor,
                        seq_of_token: torch.Tensor, positions: torch.Tensor, num_tokens: int, num_heads: int, num_kv_heads: int,
                        dim: int, vdim: int, page_size: int, scale: float, planes: int = 1, chunk: int = 0, window: int = 0,
                        pool: int = 0, softcap: float = 0.0, r1: Optional[torch.Tensor] = None, r2: Optional[torch.Tensor] = None,
                        sink: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out [T, H, vdim]: one block per (token, query head), any sizes, float32 or bf16 (see csrc/attention_masked.cu).
    `gate` [T, H] (a view with unit column stride): the head's output is multiplied by sigmoid(gate[t, h])."""
    _cuda(out, q, pages, block_tables, seq_of_token, positions, r1, r2, sink, gate)
    _contig(out, q, pages, block_tables, seq_of_token, positions, r1, r2, sink)
    T, H, G = num_tokens, num_heads, num_kv_heads
    if q.dtype != pages.dtype or out.dtype != q.dtype or q.numel() < T * H * dim or out.numel() < T * H * vdim:
        raise KernelError("attn_masked: q [T, H, dim], out [T, H, vdim] and the pages share one element type")
    if block_tables.dtype != torch.int32 or block_tables.dim() != 2 or seq_of_token.dtype != torch.int32 or positions.dtype != torch.int32:
        raise KernelError("attn_masked: block_tables int32 [S, W]; seq_of_token and positions int32")
    for t in (r1, r2, sink):
        if t is not None and (t.dtype != torch.float32 or t.numel() != H):
            raise KernelError("attn_masked: r1, r2 and sink are float32 [H]")
    if gate is not None and (gate.dtype != q.dtype or gate.shape[1] != H or gate.stride(1) != 1 or gate.shape[0] < T):
        raise KernelError("attn_masked: gate [T, H] of the queries' element type")
    num_pages = pages.numel() // (planes * G * page_size * (dim + vdim))
    _check(_attn_masked_lib().cvb_attn_masked_general(
        _ptr(out), _ptr(q), _ptr(pages), _ptr(block_tables), c_int(block_tables.shape[1]), _ptr(seq_of_token), _ptr(positions),
        c_int(T), c_int(H), c_int(G), c_int(dim), c_int(vdim), c_int(page_size), c_int(planes), c_int(chunk), c_int(window),
        c_int(pool), c_float(scale), c_float(softcap), _ptr(r1), _ptr(r2), _ptr(sink), _ptr(gate),
        c_int(gate.stride(0) if gate is not None else 0), c_int(num_pages), c_int(dtype_code(q.dtype)),
        _ptr(error_flag(q.device)), _stream()), "attn_masked_general")
    return out



def attn_masked_supported(dtype: torch.dtype, num_heads: int, num_kv_heads: int, dim: int, vdim: int) -> bool:
    """Whether the tensor-core kernel takes the shape (csrc/attention_masked.cu): bf16, key and value sizes 16 to 128 in steps
    of 16, up to 64 query heads per kv head."""
    return (dtype == torch.bfloat16 and dim % 16 == 0 and 16 <= dim <= 128 and vdim % 16 == 0 and 16 <= vdim <= 128
            and num_kv_heads > 0 and num_heads % num_kv_heads == 0 and num_heads // num_kv_heads <= 64)


def attn_masked_decode_splits(num_seqs: int, num_kv_heads: int, visible_keys: int, sms: int = 148) -> int:
    """Blocks per (request, kv head) of a decode step over entries of a key and its value: a block's warps keep two stages of
    32 entries each, which at 128 + 128 elements fills an SM's shared memory, so the blocks of a step should be one wave: the
    largest power of two (at most 8) that keeps them within the SMs and leaves every block four tiles or more."""
    pairs = max(1, num_seqs * num_kv_heads)
    tiles = max(1, (visible_keys + 31) // 32)
    splits = 1
    while splits < 8 and pairs * splits * 2 <= sms and tiles >= 4 * splits * 2:
        splits *= 2
    return splits


def attn_masked_bf16(out: torch.Tensor, q: torch.Tensor, pages: torch.Tensor, block_tables: torch.Tensor, cu_seqlens: torch.Tensor,
                     positions: torch.Tensor, num_seqs: int, num_tiles: int, num_heads: int, num_kv_heads: int, dim: int, vdim: int,
                     page_size: int, scale: float, planes: int = 1, chunk: int = 0, window: int = 0, pool: int = 0,
                     softcap: float = 0.0, r1: Optional[torch.Tensor] = None, r2: Optional[torch.Tensor] = None,
                     sink: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None, all_single: bool = False,
                     splits: int = 1, scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The tensor-core form of attn_masked_general for prompt portions and decoded tokens alike; `num_tiles` as
    attn_keys_tiles gives it (blocks of 64 // group tokens of one request).  `all_single`: every request brings exactly one
    token (the form for decoded tokens, up to 16 query heads per kv head); with `splits` > 1 that many blocks share a
    (request, kv head), through `scratch` (float32, attn_keys_scratch_floats with vdim as the head size) and a merge kernel."""
    _cuda(out, q, pages, block_tables, cu_seqlens, positions, r1, r2, sink, gate)
    _contig(out, q, pages, block_tables, cu_seqlens, positions, r1, r2, sink)
    H = num_heads
    if q.dtype != torch.bfloat16 or pages.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("attn_masked_bf16 takes bf16 queries, pages and output")
    if block_tables.dtype != torch.int32 or block_tables.dim() != 2 or cu_seqlens.dtype != torch.int32 or positions.dtype != torch.int32:
        raise KernelError("attn_masked_bf16: block_tables [S, W], cu_seqlens and positions must be int32")
    for t in (r1, r2, sink):
        if t is not None and (t.dtype != torch.float32 or t.numel() != H):
            raise KernelError("attn_masked_bf16: r1, r2 and sink are float32 [H]")
    if gate is not None and (gate.dtype != torch.bfloat16 or gate.shape[1] != H or gate.stride(1) != 1):
        raise KernelError("attn_masked_bf16: gate bf16 [T, H]")
    num_pages = pages.numel() // (planes * num_kv_heads * page_size * (dim + vdim))
    if splits > 1 and (scratch is None or scratch.dtype != torch.float32 or not scratch.is_cuda or not scratch.is_contiguous()):
        raise KernelError("attn_masked_bf16: splits need a contiguous float32 CUDA scratch")
    _check(_attn_masked_lib().cvb_attn_masked_bf16(
        _ptr(out), _ptr(q), _ptr(pages), _ptr(block_tables), c_int(block_tables.shape[1]), _ptr(cu_seqlens), _ptr(positions),
        c_int(num_seqs), c_int(num_tiles), c_int(H), c_int(num_kv_heads), c_int(dim), c_int(vdim), c_int(page_size), c_int(planes),
        c_int(chunk), c_int(window), c_int(pool), c_float(scale), c_float(softcap), _ptr(r1), _ptr(r2), _ptr(sink), _ptr(gate),
        c_int(gate.stride(0) if gate is not None else 0), c_int(num_pages), c_int(1 if all_single else 0), c_int(splits), _ptr(scratch),
        c_int64(scratch.numel() if scratch is not None else 0), _ptr(error_flag(q.device)), _stream()), "attn_masked_bf16",
        kernels=2 if all_single and splits > 1 else 1)
    return out


# ---- projection epilogue: per-head norm, rotary, cache write --------------------------------------------------

def qk_norm_rope_kv(q_out: torch.Tensor, qkv: torch.Tensor, q_weight: Optional[torch.Tensor],
                    k_weight: Optional[torch.Tensor], cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                    positions: Optional[torch.Tensor], slots: Optional[torch.Tensor],
                    cache: Optional[torch.Tensor], num_heads: int, num_kv_heads: int, head_dim: int,
                    page_size: int, eps: float, rotary_dim: Optional[int] = None, interleaved: bool = False) -> torch.Tensor:
    """q_out[T, H, hd] <- rotate(norm(q)); k -> rotate(norm(k)) and v into `cache` [pages, 2, KV, page, hd]."""
    _cuda(q_out, qkv, q_weight, k_weight, cos, sin, positions, slots, cache)
    _contig(q_out, qkv, q_weight, k_weight, cos, sin, positions, slots, cache)
    T = qkv.shape[0]
    H, KV, hd = num_heads, num_kv_heads, head_dim
    if qkv.shape[1] != (H + 2 * KV) * hd or q_out.numel() != T * H * hd or q_out.dtype != qkv.dtype:
        raise KernelError("qk_norm_rope_kv: qkv must be [T, (H + 2 KV) hd] and q_out [T, H, hd]")
    for w in (q_weight, k_weight):
        if w is not None and (w.dtype != torch.float32 or w.numel() != hd):
            raise KernelError("qk_norm_rope_kv: per-head norm weights must be float32 [hd]")
    rot = head_dim if rotary_dim is None else int(rotary_dim)
    max_pos = 0
    if cos is not None:
        if cos.dtype != torch.float32 or sin is None or sin.shape != cos.shape or cos.shape[1] != rot // 2:
            raise KernelError("qk_norm_rope_kv: cos/sin tables must be float32 [max_pos, rotary_dim / 2]")
        max_pos = cos.shape[0]
        if positions is None or positions.dtype != torch.int32 or positions.numel() < T:
            raise KernelError("qk_norm_rope_kv: positions must be int32 [T]")
    if slots is not None and (slots.dtype != torch.int32 or slots.numel() < T):
        raise KernelError("qk_norm_rope_kv: slots must be int32 [T]")
    cache_elems = 0
    if cache is not None:
        if cache.dtype != qkv.dtype:
            raise KernelError("qk_norm_rope_kv: cache pages must have the activations' element type")
        cache_elems = cache.numel()
    _check(core().cvb_qk_norm_rope_kv(
        _ptr(q_out), _ptr(qkv), _ptr(q_weight), _ptr(k_weight), _ptr(cos), _ptr(sin), _ptr(positions), _ptr(slots),
        _ptr(cache), c_int(T), c_int(H), c_int(KV), c_int(hd), c_int(rot), c_int(1 if interleaved else 0),
        c_int(page_size), c_int(max_pos), c_float(eps), c_int64(cache_elems), c_int(dtype_code(qkv.dtype)),
        _ptr(error_flag(qkv.device)), _stream()), "qk_norm_rope_kv")
    return q_out


# ---- attention ---------------------------------------------------------------------------------------------

def paged_attention_general(out: torch.Tensor, q: torch.Tensor, cache: torch.Tensor, block_tables: torch.Tensor,
                            seq_of_token: torch.Tensor, positions: torch.Tensor, num_heads: int, num_kv_heads: int,
                            head_dim: int, page_size: int, scale: float, window: int = 0,
                            num_tokens: Optional[int] = None, keep_first: int = 0, keys_are_values: bool = False,
                            value_dim: Optional[int] = None) -> torch.Tensor:
    """One block per (token, query head); any head size.  `keep_first`: positions 0..keep_first-1 stay visible behind the
    window.  `keys_are_values`: pages are [kv head, slot, head_dim] and a key is also its value (else [K|V, kv head, slot,
    head_dim]).  `q` may be the packed output of a projection: rows of q.shape[1] elements whose first H * head_dim are
    the queries.  `value_dim` (with keys_are_values): only the first value_dim elements of a key are its value; out is
    [T, H, value_dim]."""
    _cuda(out, q, cache, block_tables, seq_of_token, positions)
    _contig(out, q, cache, block_tables, seq_of_token, positions)
    T = q.shape[0] if num_tokens is None else num_tokens
    if q.dtype != cache.dtype or out.dtype != q.dtype:
        raise KernelError("paged_attention: q, out and the cache pages must share one element type")
    if block_tables.dtype != torch.int32 or block_tables.dim() != 2:
        raise KernelError("paged_attention: block_tables must be int32 [S, W]")
    if seq_of_token.dtype != torch.int32 or positions.dtype != torch.int32:
        raise KernelError("paged_attention: seq_of_token and positions must be int32")
    if num_heads % num_kv_heads:
        raise KernelError(f"paged_attention: {num_heads} query heads are not a multiple of {num_kv_heads} kv heads")
    planes = 1 if keys_are_values else 2
    vd = head_dim if value_dim is None else int(value_dim)
    if vd != head_dim and not keys_are_values:
        raise KernelError("paged_attention: a value narrower than the key needs keys that are the values")
    if out.numel() < T * num_heads * vd:
        raise KernelError("paged_attention: out is too small")
    page_elems = planes * num_kv_heads * page_size * head_dim
    num_pages = cache.numel() // page_elems
    q_stride = q.shape[1] if q.dim() == 2 else num_heads * head_dim
    _check(core().cvb_paged_attention_general(
        _ptr(out), _ptr(q), _ptr(cache), _ptr(block_tables), c_int(block_tables.shape[1]), _ptr(seq_of_token),
        _ptr(positions), c_int(T), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(vd), c_int(page_size),
        c_int(window), c_int(keep_first), c_int(planes), c_int(q_stride), c_float(scale), c_int(num_pages),
        c_int(dtype_code(q.dtype)),
        _ptr(error_flag(q.device)), _stream()), "paged_attention_general")
    return out


_attn = None


def attn_bf16():
    global _attn
    if _attn is None:
        lib = load_library("attn_bf16")
        lib.cvb_attn_prefill_bf16.restype = c_int
        lib.cvb_attn_decode_bf16.restype = c_int
        lib.cvb_attn_decode_scratch_floats.restype = c_int64
        _attn = lib
    return _attn


def fast_attention_supported(dtype: torch.dtype, num_heads: int, num_kv_heads: int, head_dim: int,
                             page_size: int = 16) -> bool:
    """The tensor-core kernels cover bf16, head sizes 64 and 128, up to 16 query heads per kv head and pages of
    16, 32, 64, ... tokens (a power of two)."""
    return (dtype == torch.bfloat16 and head_dim in (64, 128) and num_heads % num_kv_heads == 0
            and num_heads // num_kv_heads <= 16 and page_size >= 16 and page_size & (page_size - 1) == 0)


def prefill_tiles(q_lens, num_heads: int, num_kv_heads: int, skip_single: bool = True) -> int:
    """Tiles the prefill kernel's grid needs: per request ceil(tokens / (64 / group))."""
    tpt = 64 // (num_heads // num_kv_heads)
    return sum((n + tpt - 1) // tpt for n in q_lens if not (skip_single and n == 1))


def _attn_common_checks(out, q, cache, block_tables, cu_seqlens, positions):
    _cuda(out, q, cache, block_tables, cu_seqlens, positions)
    _contig(out, q, cache, block_tables, cu_seqlens, positions)
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("tensor-core attention takes bf16 queries, pages and output")
    if block_tables.dtype != torch.int32 or block_tables.dim() != 2 or cu_seqlens.dtype != torch.int32 \
            or positions.dtype != torch.int32:
        raise KernelError("tensor-core attention: block_tables [S, W], cu_seqlens and positions must be int32")


def attn_prefill_bf16(out, q, cache, block_tables, cu_seqlens, positions, num_seqs: int, num_tiles: int,
                      num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, scale: float,
                      window: int = 0, skip_single: bool = True):
    _attn_common_checks(out, q, cache, block_tables, cu_seqlens, positions)
    num_pages = cache.numel() // (2 * num_kv_heads * page_size * head_dim)
    _check(attn_bf16().cvb_attn_prefill_bf16(
        _ptr(out), _ptr(q), _ptr(cache), _ptr(block_tables), c_int(block_tables.shape[1]), _ptr(cu_seqlens),
        _ptr(positions), c_int(num_seqs), c_int(num_tiles), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim),
        c_int(page_size), c_int(window), c_float(scale), c_int(num_pages), c_int(1 if skip_single else 0),
        _ptr(error_flag(q.device)), _stream()), "attn_prefill_bf16")
    return out


_attn_tc = None


def prefill_tiles_tcgen05(q_lens, num_heads: int, num_kv_heads: int, skip_single: bool = True) -> int:
    """Blocks the tcgen05 prefill kernel's grid needs: per request ceil(tokens / (2 * (128 // group)))."""
    tpt = (128 // (num_heads // num_kv_heads)) * 2
    return sum((n + tpt - 1) // tpt for n in q_lens if not (skip_single and n == 1))


def _attn_tc_lib():
    global _attn_tc
    if _attn_tc is None:
        lib = load_library("attn_tcgen05")
        lib.cvb_attn_prefill_tcgen05.restype = c_int
        lib.cvb_attn_prefill_tcgen05_scratch_floats.restype = c_int64
        _attn_tc = lib
    return _attn_tc


# The tcgen05 prefill kernel shares the key tiles of a long query block out among several blocks when its grid leaves
# most SMs idle: a portion of 512 tokens behind 8,192 cached ones is 32 blocks (8 kv heads) of 68 key tiles each, 128 us
# as they are and 52 us in four pieces.  Pieces are taken only while all blocks can run at once (a second wave costs
# what the cut saves), and a piece has at least PREFILL_MIN_ROUNDS tiles: what a block costs outside its tiles, and
# adding the shares up, is worth about six tiles.
PREFILL_SMS = 148
PREFILL_MAX_PIECES = 8
PREFILL_MIN_ROUNDS = 8


def prefill_pieces_tcgen05(num_tiles: int, num_kv_heads: int, max_kv_len: int = 1 << 30) -> int:
    """Into how many pieces the kernel may cut a query block's keys; 1 if no request of the step is long enough for two
    pieces (the kernel that adds the shares up is then not launched)."""
    if max_kv_len < 2 * PREFILL_MIN_ROUNDS * 128:
        return 1
    blocks = max(1, num_tiles * num_kv_heads)
    return max(1, min(PREFILL_MAX_PIECES, PREFILL_SMS // blocks))


def attn_prefill_tcgen05_scratch_floats(num_tiles: int, num_kv_heads: int, head_dim: int, pieces: int) -> int:
    return int(_attn_tc_lib().cvb_attn_prefill_tcgen05_scratch_floats(c_int(num_tiles), c_int(num_kv_heads), c_int(head_dim),
                                                                      c_int(pieces)))


def attn_prefill_tcgen05(out, q, cache, block_tables, cu_seqlens, positions, num_seqs: int, num_tiles: int,
                         num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, scale: float,
                         window: int = 0, skip_single: bool = True, pieces: int = 1, min_rounds: int = PREFILL_MIN_ROUNDS,
                         scratch=None, piece_counts=None):
    """Flash attention of prompt portions on the tcgen05 tensor cores (same contract as attn_prefill_bf16).
    ``pieces`` > 1: a query block with at least 2 * min_rounds key tiles is worked on by up to ``pieces`` blocks;
    ``scratch`` (float32, attn_prefill_tcgen05_scratch_floats elements) and ``piece_counts`` (int32, num_tiles * kv heads)
    are then required, and a second kernel adds the pieces' shares up."""
    lib = _attn_tc_lib()
    _attn_common_checks(out, q, cache, block_tables, cu_seqlens, positions)
    num_pages = cache.numel() // (2 * num_kv_heads * page_size * head_dim)
    if pieces > 1:
        if scratch is None or piece_counts is None:
            raise ValueError("attn_prefill_tcgen05 with pieces > 1 needs scratch and piece_counts")
        if scratch.dtype != torch.float32 or piece_counts.dtype != torch.int32 or piece_counts.numel() < num_tiles * num_kv_heads:
            raise ValueError("attn_prefill_tcgen05: scratch must be float32 and piece_counts int32 with one entry per "
                             "(query block, kv head)")
    _check(lib.cvb_attn_prefill_tcgen05(
        _ptr(out), _ptr(q), _ptr(cache), _ptr(block_tables), c_int(block_tables.shape[1]), _ptr(cu_seqlens),
        _ptr(positions), c_int(num_seqs), c_int(num_tiles), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim),
        c_int(page_size), c_int(window), c_float(scale), c_int(num_pages), c_int(1 if skip_single else 0),
        c_int(pieces), c_int(min_rounds), _ptr(scratch), c_int64(scratch.numel() if scratch is not None else 0), _ptr(piece_counts),
        _ptr(error_flag(q.device)), _stream()), "attn_prefill_tcgen05", kernels=2 if pieces > 1 else 1)
    return out


def attn_decode_scratch_floats(num_seqs: int, num_kv_heads: int, head_dim: int, splits: int) -> int:
    return int(attn_bf16().cvb_attn_decode_scratch_floats(c_int(num_seqs), c_int(num_kv_heads), c_int(head_dim), c_int(splits)))


def attn_decode_bf16(out, q, cache, block_tables, cu_seqlens, positions, num_seqs: int, num_heads: int,
                     num_kv_heads: int, head_dim: int, page_size: int, scale: float, splits: int,
                     scratch: Optional[torch.Tensor], window: int = 0, cluster_merge: bool = True):
    """Split-KV attention of single decoded tokens.  With `cluster_merge` (and up to 16 splits) the splits of a request
    and kv head run as one thread-block cluster and merge their parts through distributed shared memory; otherwise the
    parts go through `scratch` and a second kernel merges them."""
    _attn_common_checks(out, q, cache, block_tables, cu_seqlens, positions)
    if scratch is not None and (scratch.dtype != torch.float32 or not scratch.is_cuda or not scratch.is_contiguous()):
        raise KernelError("attn_decode_bf16: scratch must be a contiguous float32 CUDA tensor")
    num_pages = cache.numel() // (2 * num_kv_heads * page_size * head_dim)
    _check(attn_bf16().cvb_attn_decode_bf16(
        _ptr(out), _ptr(q), _ptr(cache), _ptr(block_tables), c_int(block_tables.shape[1]), _ptr(cu_seqlens),
        _ptr(positions), c_int(num_seqs), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(page_size),
        c_int(window), c_float(scale), c_int(num_pages), c_int(splits), _ptr(scratch),
        c_int64(scratch.numel() if scratch is not None else 0), c_int(1 if cluster_merge else 0),
        _ptr(error_flag(q.device)), _stream()), "attn_decode_bf16",
        kernels=2 if splits > 1 and not (cluster_merge and splits <= 16) else 1)
    return out


DECODE_CLUSTER_SPLITS = 16      # up to this many splits merge inside a thread-block cluster and need no scratch


def attn_decode_fused_bf16(out, qkv, cache, block_tables, cu_seqlens, positions, slots, num_seqs: int, num_heads: int,
                           num_kv_heads: int, head_dim: int, page_size: int, scale: float, splits: int,
                           scratch: Optional[torch.Tensor], q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
                           qk_eps: float, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], window: int = 0):
    """Attention of single decoded tokens from the projection's raw output qkv [T, (H + 2 KV) hd]: per-head norm and
    rotation of queries and of the new key, the cache write of the new key and value, and the attention, one kernel."""
    _attn_common_checks(out, qkv, cache, block_tables, cu_seqlens, positions)
    _cuda(slots, q_weight, k_weight, cos, sin, scratch)
    _contig(slots, q_weight, k_weight, cos, sin, scratch)
    T = qkv.shape[0]
    if T != num_seqs:
        raise KernelError("attn_decode_fused_bf16: every request brings exactly one token (qkv has one row per request)")
    if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim or out.shape != (T, num_heads * head_dim):
        raise KernelError("attn_decode_fused_bf16: qkv must be [T, (H + 2 KV) hd] and out [T, H hd]")
    if slots.dtype != torch.int32 or slots.numel() < T:
        raise KernelError("attn_decode_fused_bf16: slots must be int32 [T]")
    for w in (q_weight, k_weight):
        if w is not None and (w.dtype != torch.float32 or w.numel() != head_dim):
            raise KernelError("attn_decode_fused_bf16: norm weights must be float32 [head_dim]")
    max_pos = 0
    if cos is not None:
        if sin is None or cos.dtype != torch.float32 or sin.dtype != torch.float32 or cos.shape != sin.shape \
                or cos.dim() != 2 or cos.shape[1] != head_dim // 2:
            raise KernelError("attn_decode_fused_bf16: cos and sin must be float32 [max_pos, head_dim / 2]")
        max_pos = cos.shape[0]
    if scratch is not None and scratch.dtype != torch.float32:
        raise KernelError("attn_decode_fused_bf16: scratch must be float32")
    num_pages = cache.numel() // (2 * num_kv_heads * page_size * head_dim)
    lib = attn_bf16()
    lib.cvb_attn_decode_fused_bf16.restype = c_int
    _check(lib.cvb_attn_decode_fused_bf16(
        _ptr(out), _ptr(qkv), _ptr(cache), _ptr(block_tables), c_int(block_tables.shape[1]), _ptr(cu_seqlens),
        _ptr(positions), _ptr(slots), c_int(num_seqs), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim),
        c_int(page_size), c_int(window), c_float(scale), c_int(num_pages), c_int(splits), _ptr(scratch),
        c_int64(scratch.numel() if scratch is not None else 0), _ptr(q_weight), _ptr(k_weight), c_float(qk_eps),
        _ptr(cos), _ptr(sin), c_int(max_pos), _ptr(error_flag(qkv.device)), _stream()), "attn_decode_fused_bf16",
        kernels=2 if splits > 16 else 1)
    return out


_gemv = None

SPLITK_MIN_BYTES = 16 << 20
GEMV_MAX_ROWS = 16           # the weight-streaming product: one or two groups of eight activation rows
SPLITK_MAX_ROWS = 8          # its split-K form: one group


def gemv_supported(x_dtype: torch.dtype, weight: torch.Tensor, rows: int) -> bool:
    """The weight-streaming product covers bf16 operands, up to 16 rows, and inner sizes that are multiples of 8 and whose
    staged rows (8 or 16 of them) fit into shared memory.  More than 8 rows against a large weight are left to the
    library: the split-K form takes 8 rows, and the plain form is slower than the library there."""
    staged = 8 if rows <= 8 else 16
    return (x_dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and 0 < rows <= GEMV_MAX_ROWS
            and weight.shape[1] % 8 == 0 and weight.shape[1] * staged * 2 + 32 * 1024 <= 200 * 1024
            and (rows <= 8 or weight.numel() * 2 < SPLITK_MIN_BYTES))


def gemv_bf16(out: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, rows: int, norm_weight: Optional[torch.Tensor] = None,
              eps: float = 0.0, delta: Optional[torch.Tensor] = None, resid_out: Optional[torch.Tensor] = None,
              swiglu: bool = False) -> torch.Tensor:
    """out[:rows] = x[:rows] @ weight^T for a few rows.  With `norm_weight`, x is the residual stream: `delta` (if given)
    is added first and the sum written to `resid_out`, then the RMSNorm with `norm_weight` is applied before the
    product.  With `swiglu`, weight holds gate rows over up rows and out receives silu(gate) * up."""
    _gemv_lib()
    _cuda(out, x, weight, norm_weight, delta, resid_out)
    _contig(out, x, weight, norm_weight, delta, resid_out)
    N, K = weight.shape
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or x.shape[1] != K:
        raise KernelError("gemv_bf16: x [M, K], weight [N, K] and out must be bf16")
    if out.shape[1] != (N // 2 if swiglu else N) or out.shape[0] < rows or x.shape[0] < rows:
        raise KernelError("gemv_bf16: out must be [M, N] (or [M, N / 2] with swiglu)")
    if swiglu and norm_weight is None:
        raise KernelError("gemv_bf16: the SwiGLU form comes with the norm prologue")
    if norm_weight is not None and (norm_weight.dtype != torch.float32 or norm_weight.numel() != K):
        raise KernelError("gemv_bf16: norm_weight must be float32 [K]")
    if delta is not None and (norm_weight is None or resid_out is None or delta.dtype != torch.bfloat16
                              or resid_out.dtype != torch.bfloat16 or resid_out.data_ptr() == x.data_ptr()):
        raise KernelError("gemv_bf16: delta needs the norm prologue and a resid_out buffer other than x")
    mode = 0 if norm_weight is None else (2 if swiglu else 1)
    _check(_gemv.cvb_gemv_bf16(_ptr(out), _ptr(x), _ptr(delta), _ptr(resid_out), _ptr(norm_weight), _ptr(weight), c_int(rows),
                               c_int(N), c_int(K), c_float(eps), c_int(mode), _stream()), "gemv_bf16")
    return out


def _gemv_lib():
    global _gemv
    if _gemv is None:
        lib = load_library("gemv_bf16")
        for name in ("cvb_gemv_bf16", "cvb_gemv_splitk_bf16", "cvb_gemv_splitk_counters", "cvb_gemv_stream_bf16",
                     "cvb_gemv_stream_supported", "cvb_gemv_ring_bf16"):
            getattr(lib, name).restype = c_int
        lib.cvb_gemv_splitk_scratch_floats.restype = c_int64
        _gemv = lib
    return _gemv


STREAM_MAX_ROWS = 16
_stream_ok: Dict[tuple, bool] = {}


def gemv_stream_supported(x_dtype: torch.dtype, weight: torch.Tensor, rows: int, swiglu: bool = False) -> bool:
    """The product that runs one block per SM and fetches the block's whole share of the weight ahead of its dependency
    covers bf16 operands, up to 16 rows, and weights whose share per SM (rows / #SMs, whole rows) fits into about half an
    SM's shared memory beside the staged activations (all of it from nine rows on): matrices of a few megabytes."""
    if not (x_dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.dim() == 2 and 0 < rows <= STREAM_MAX_ROWS):
        return False
    key = (weight.shape[0], weight.shape[1], swiglu, rows > 8)
    ok = _stream_ok.get(key)
    if ok is None:
        ok = bool(_gemv_lib().cvb_gemv_stream_supported(c_int(key[0]), c_int(key[1]), c_int(2 if swiglu else 0), c_int(rows)))
        _stream_ok[key] = ok
    return ok


def gemv_stream_bf16(out: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, rows: int, norm_weight: Optional[torch.Tensor] = None,
                     eps: float = 0.0, delta: Optional[torch.Tensor] = None, resid_out: Optional[torch.Tensor] = None,
                     swiglu: bool = False, prefetch: Optional[torch.Tensor] = None, late_trigger: bool = False,
                     dependent: bool = True, add_to: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Same contract as gemv_bf16 for shapes that gemv_stream_supported accepts.  `prefetch`: a tensor that a later kernel
    will stream (asked into the L2 by this kernel).  `late_trigger`: the next kernel on the stream may start only when
    this one's products are done (for successors whose blocks should find the SMs free).  `dependent=False` launches
    without the programmatic-dependent-launch attribute.  `add_to` (plain form only): out = rnd(add_to + rnd(x @ weight^T)),
    the residual sum folded into the product's store; `add_to` may be `out` itself."""
    lib = _gemv_lib()
    _cuda(out, x, weight, norm_weight, delta, resid_out, prefetch, add_to)
    _contig(out, x, weight, norm_weight, delta, resid_out, prefetch, add_to)
    if add_to is not None and (norm_weight is not None or add_to.dtype != torch.bfloat16 or add_to.shape != out.shape):
        raise KernelError("gemv_stream_bf16: add_to goes with the plain form and must be bf16, shaped like out")
    N, K = weight.shape
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or x.shape[1] != K:
        raise KernelError("gemv_stream_bf16: x [M, K], weight [N, K] and out must be bf16")
    if out.shape[1] != (N // 2 if swiglu else N) or out.shape[0] < rows or x.shape[0] < rows:
        raise KernelError("gemv_stream_bf16: out must be [M, N] (or [M, N / 2] with swiglu)")
    if swiglu and norm_weight is None:
        raise KernelError("gemv_stream_bf16: the SwiGLU form comes with the norm prologue")
    if norm_weight is not None and (norm_weight.dtype != torch.float32 or norm_weight.numel() != K):
        raise KernelError("gemv_stream_bf16: norm_weight must be float32 [K]")
    if delta is not None and (norm_weight is None or resid_out is None or delta.dtype != torch.bfloat16
                              or resid_out.dtype != torch.bfloat16 or resid_out.data_ptr() == x.data_ptr()):
        raise KernelError("gemv_stream_bf16: delta needs the norm prologue and a resid_out buffer other than x")
    mode = 0 if norm_weight is None else (2 if swiglu else 1)
    _check(lib.cvb_gemv_stream_bf16(_ptr(out), _ptr(x), _ptr(delta), _ptr(resid_out), _ptr(norm_weight), _ptr(weight), c_int(rows),
                                    c_int(N), c_int(K), c_float(eps), c_int(mode), _ptr(add_to), _ptr(prefetch),
                                    ctypes.c_longlong(prefetch.numel() * prefetch.element_size() if prefetch is not None else 0),
                                    c_int(1 if late_trigger else 0), c_int(1 if dependent else 0),
                                    _ptr(error_flag(x.device)), _stream()), "gemv_stream_bf16")
    return out


_splitk_buffers: Dict[int, list] = {}


def gemv_splitk_preferred(x_dtype: torch.dtype, weight: torch.Tensor, rows: int) -> bool:
    """Weights of 16 MB and more go through the kernel that splits the inner dimension over blocks as well."""
    return (x_dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and 0 < rows <= SPLITK_MAX_ROWS
            and weight.dim() == 2 and weight.shape[1] % 8 == 0 and weight.numel() * 2 >= SPLITK_MIN_BYTES)


def gemv_splitk_bf16(out: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, rows: int) -> torch.Tensor:
    """out[:rows] = x[:rows] @ weight^T for up to 8 rows and a large weight.  The scratch for the partial sums and the
    counters belong to the device and grow with the largest weight seen; they are made at the first call with a weight
    (a warm-up before any graph capture, as the runner does, sizes them)."""
    _gemv_lib()
    _cuda(out, x, weight)
    _contig(out, x, weight)
    N, K = weight.shape
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or x.shape[1] != K:
        raise KernelError("gemv_splitk_bf16: x [M, K], weight [N, K] and out must be bf16")
    if out.shape[1] != N or out.shape[0] < rows or x.shape[0] < rows:
        raise KernelError("gemv_splitk_bf16: out must be [M, N]")
    need_f = int(_gemv.cvb_gemv_splitk_scratch_floats(c_int(N), c_int(K)))
    need_c = int(_gemv.cvb_gemv_splitk_counters(c_int(N)))
    idx = x.device.index if x.device.index is not None else torch.cuda.current_device()
    buf = _splitk_buffers.get(idx)
    if buf is None or buf[0].numel() < need_f or buf[1].numel() < need_c:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("gemv_splitk_bf16: its scratch has to grow; run the shape once before capturing it")
        buf = [torch.empty(max(need_f, buf[0].numel() if buf else 0), dtype=torch.float32, device=x.device),
               torch.zeros(max(need_c, buf[1].numel() if buf else 0, 1024), dtype=torch.int32, device=x.device)]
        _splitk_buffers[idx] = buf
    _check(_gemv.cvb_gemv_splitk_bf16(_ptr(out), _ptr(x), _ptr(weight), c_int(rows), c_int(N), c_int(K), _ptr(buf[0]),
                                      c_int64(buf[0].numel()), _ptr(buf[1]), _stream()), "gemv_splitk_bf16")
    return out


RING_MAX_ROWS = 8


def gemv_ring_supported(x_dtype: torch.dtype, weight: torch.Tensor, rows: int) -> bool:
    """The ring-buffered streaming product covers bf16 operands, up to 8 rows, any weight whose rows are multiples of 16
    bytes; it is meant for weights too large for the decode chain's product."""
    return (x_dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.dim() == 2 and 0 < rows <= RING_MAX_ROWS
            and weight.shape[1] % 8 == 0)


def gemv_ring_bf16(out: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, rows: int, dependent: bool = False) -> torch.Tensor:
    """out[:rows] = x[:rows] @ weight^T for up to 8 rows: one block per SM streams its share of the weight's rows through a
    ring of shared-memory stages filled by bulk copies."""
    lib = _gemv_lib()
    _cuda(out, x, weight)
    _contig(out, x, weight)
    N, K = weight.shape
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or x.shape[1] != K:
        raise KernelError("gemv_ring_bf16: x [M, K], weight [N, K] and out must be bf16")
    if out.shape[1] != N or out.shape[0] < rows or x.shape[0] < rows:
        raise KernelError("gemv_ring_bf16: out must be [M, N]")
    _check(lib.cvb_gemv_ring_bf16(_ptr(out), _ptr(x), _ptr(weight), c_int(rows), c_int(N), c_int(K), c_int(1 if dependent else 0),
                                  _ptr(error_flag(x.device)), _stream()), "gemv_ring_bf16")
    return out


_project_choice: Dict[tuple, str] = {}
_flush_buffers: Dict[int, torch.Tensor] = {}


def _project_candidates(x: torch.Tensor, weight: torch.Tensor, rows: int):
    names = []
    if gemv_supported(x.dtype, weight, rows):
        names.append("gemv")
    if (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and 0 < rows <= SPLITK_MAX_ROWS and weight.dim() == 2
            and weight.shape[1] % 8 == 0 and weight.numel() * 2 >= (1 << 20)):
        names.append("splitk")
    if gemv_ring_supported(x.dtype, weight, rows) and weight.numel() * 2 >= (1 << 20):
        names.append("ring")
    names.append("library")
    return names


def _project_with(name: str, x, weight, out, rows, dependent: bool = False):
    if name == "gemv":
        return gemv_bf16(out, x, weight, rows)
    if name == "splitk":
        return gemv_splitk_bf16(out, x, weight, rows)
    if name == "ring":
        return gemv_ring_bf16(out, x, weight, rows, dependent=dependent)
    return linear(x, weight, out=out)


def _measure_projection(name: str, x, weight, out, rows) -> float:
    """Microseconds of four calls, each with the weight out of the L2 (a buffer larger than the L2 is written before every
    call), replayed from a captured graph so that the host's launch cost does not blur the comparison.  The writes of
    the buffer take the same time for every candidate."""
    idx = x.device.index if x.device.index is not None else torch.cuda.current_device()
    flush = _flush_buffers.get(idx)
    if flush is None:
        flush = torch.empty(256 << 20, dtype=torch.int8, device=x.device)
        _flush_buffers[idx] = flush
    _project_with(name, x, weight, out, rows)                 # sizes its scratch, loads its code
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(4):
            flush.zero_()
            _project_with(name, x, weight, out, rows)
    graph.replay()
    best = float("inf")
    for _ in range(3):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) * 1e3)
    return best


def project_rows(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, rows: int, dependent: bool = True) -> torch.Tensor:
    """out = x @ weight^T by the kernel that suits the step.  A weight whose share per SM fits into shared memory goes
    through the product made for chains of dependent launches (`dependent=False` keeps that kernel behind its
    predecessor's end instead of letting it start early and fetch its weights meanwhile).  Otherwise the candidates for a
    few bf16 rows (the weight-streaming product, its split-K form, the ring-buffered product, the library's product) are timed once per shape, with
    the weight out of the L2, the first time the shape is seen outside a graph capture, and the fastest is kept; during
    a capture an unseen shape takes the split-K form for large weights, the weight-streaming product for small ones.
    CVB_PROJECT=gemv|splitk|ring|library in the environment fixes the choice."""
    if gemv_stream_supported(x.dtype, weight, rows):
        return gemv_stream_bf16(out, x, weight, rows, dependent=dependent)
    if rows > GEMV_MAX_ROWS or x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        return linear(x, weight, out=out)
    key = (weight.shape[0], weight.shape[1], rows if rows <= 2 else (8 if rows <= 8 else 16))
    choice = _project_choice.get(key)
    if choice is None:
        names = _project_candidates(x, weight, rows)
        forced = os.environ.get("CVB_PROJECT")
        if forced in names:
            choice = forced
        elif len(names) == 1:
            choice = names[0]
        elif torch.cuda.is_current_stream_capturing():
            fallback = "splitk" if gemv_splitk_preferred(x.dtype, weight, rows) else ("gemv" if "gemv" in names else "library")
            return _project_with(fallback, x, weight, out, rows)
        else:
            timed = {n: _measure_projection(n, x, weight, out, rows) for n in names}
            choice = min(timed, key=timed.get)
            if os.environ.get("CVB_PROJECT_VERBOSE"):
                print(f"[cppvllm_b200] projection {key}: " + ", ".join(f"{n} {t:.1f} us" for n, t in timed.items()) + f" -> {choice}",
                      file=sys.stderr, flush=True)
        _project_choice[key] = choice
    return _project_with(choice, x, weight, out, rows, dependent)


_gemm = None


def gemm_tcgen05_supported(x_dtype: torch.dtype, weight: torch.Tensor, swiglu: bool = False) -> bool:
    """The tcgen05 product covers bf16 operands with inner sizes that are multiples of 8 and output widths that are
    multiples of 8."""
    n_out = weight.shape[0] // 2 if swiglu else weight.shape[0]
    return (x_dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.shape[1] % 8 == 0 and n_out % 8 == 0
            and (not swiglu or weight.shape[0] % 2 == 0))


def gemm_bf16_tcgen05(out: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, swiglu: bool = False, tile_n: int = 0,
                      resid: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = x @ weight^T on the tcgen05 tensor cores; with `swiglu`, weight holds gate rows over up rows and
    out = silu(x @ gate^T) * (x @ up^T); with `resid` (which may be `out`), out = round(x @ weight^T) + resid.
    `tile_n` (128 or 256) picks the tile width; 0 chooses by the number of tiles it gives."""
    global _gemm
    if _gemm is None:
        lib = load_library("gemm_bf16")
        lib.cvb_gemm_bf16_tcgen05.restype = c_int
        _gemm = lib
    _cuda(out, x, weight, resid); _contig(out, x, weight, resid)
    M, K = x.shape
    N = weight.shape[0]
    n_out = N // 2 if swiglu else N
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or weight.shape[1] != K \
            or out.shape != (M, n_out) or (swiglu and resid is not None) \
            or (resid is not None and (resid.dtype != torch.bfloat16 or resid.shape != out.shape)):
        raise KernelError("gemm_bf16_tcgen05: x [M, K], weight [N, K], out [M, N] (or [M, N / 2] with swiglu), resid like out, "
                          "all bf16")
    if tile_n == 0:
        # tiles of 256 columns halve the traffic of A; take them when they still fill the SMs
        tiles_256 = ((M + 127) // 128) * ((N + 255) // 256)
        tile_n = 256 if tiles_256 >= 120 else 128
    mode = 1 if swiglu else (2 if resid is not None else 0)
    _check(_gemm.cvb_gemm_bf16_tcgen05(_ptr(out), _ptr(x), _ptr(weight), _ptr(resid), c_int(M), c_int(N), c_int(K), c_int(mode),
                                       c_int(tile_n), _ptr(error_flag(x.device)), _stream()), "gemm_bf16_tcgen05")
    return out


GATED_MIN_ROWS = 1024
GATED_SMS = 148


def gated_product_fused(x_dtype: torch.dtype, weight: torch.Tensor, rows: int) -> bool:
    """Whether the gate/up product of `rows` tokens goes through the tcgen05 kernel with the SwiGLU epilogue instead of the
    library's product followed by the SwiGLU kernel.  The fused kernel wins where its tiles of 128 rows by 128 outputs
    fill the SMs at least twice over with little left over in the last round (measured on a B200, against the library
    product plus the SwiGLU kernel: 2,048 x 6,144 x 1,024: 25 us against 30; 4,096 rows: 43 against 57; 2,048 x 24,576 x
    4,096: 281 against 302; 1,024 rows or fewer: the library wins by 2 to 35 %).  CVB_GATED=fused|library fixes it."""
    forced = os.environ.get("CVB_GATED", "")
    ok = (x_dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.dim() == 2 and weight.shape[1] % 8 == 0
          and weight.shape[0] % 16 == 0)
    if not ok or forced == "library":
        return False
    if forced == "fused":
        return True
    if rows < GATED_MIN_ROWS:
        return False
    tiles = ((rows + 127) // 128) * ((weight.shape[0] // 2 + 127) // 128)
    rounds = tiles / GATED_SMS
    return rounds >= 2 and rounds / math.ceil(rounds) >= 0.8


# ---- sampling ----------------------------------------------------------------------------------------------

def sample(out: torch.Tensor, logits: torch.Tensor, rows: Optional[torch.Tensor], temps: torch.Tensor,
           seeds: torch.Tensor, out_positions: torch.Tensor, num_rows: Optional[int] = None,
           scratch: Optional[torch.Tensor] = None, chunks: int = 0) -> torch.Tensor:
    """With `scratch` (any dtype, at least rows * chunks * 8 bytes) and `chunks` > 1 the vocabulary of every row is
    searched by `chunks` blocks in parallel; the token is the same as with one block per row."""
    _cuda(out, logits, rows, temps, seeds, out_positions); _contig(out, logits, rows, temps, seeds, out_positions)
    R = out.numel() if num_rows is None else num_rows
    if (logits.dtype != torch.float32 or logits.dim() != 2 or out.dtype != torch.int32 or temps.dtype != torch.float32
            or seeds.dtype != torch.int64 or out_positions.dtype != torch.int32
            or (rows is not None and rows.dtype != torch.int32)):
        raise KernelError("sample: logits float32 [N, V]; out, rows, out_positions int32; temps float32; seeds int64")
    if scratch is not None and chunks > 1:
        _cuda(scratch); _contig(scratch)
        _check(core().cvb_sample_chunked(_ptr(out), _ptr(logits), _ptr(rows), _ptr(temps), _ptr(seeds), _ptr(out_positions),
                                         c_int(R), c_int(logits.shape[1]), c_int(logits.shape[0]), c_int(chunks), _ptr(scratch),
                                         c_int64(scratch.numel() * scratch.element_size()), _stream()), "sample", kernels=2)
        return out
    _check(core().cvb_sample(_ptr(out), _ptr(logits), _ptr(rows), _ptr(temps), _ptr(seeds), _ptr(out_positions),
                             c_int(R), c_int(logits.shape[1]), c_int(logits.shape[0]), _stream()), "sample")
    return out


def feed_tokens(tokens: torch.Tensor, src: torch.Tensor, sampled: torch.Tensor, n: int) -> torch.Tensor:
    _cuda(tokens, src, sampled); _contig(tokens, src, sampled)
    if tokens.dtype != torch.int32 or src.dtype != torch.int32 or sampled.dtype != torch.int32:
        raise KernelError("feed_tokens: all arguments must be int32")
    _check(core().cvb_feed_tokens(_ptr(tokens), _ptr(src), _ptr(sampled), c_int(n), c_int(sampled.numel()), _stream()),
           "feed_tokens")
    return tokens


# ---- library matrix products ---------------------------------------------------------------------------------

def linear(x: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """y = x @ weight^T through cuBLAS, as the reference does with at::linear (model_architecture.cpp:155,178,
    182,185,224).  float32 operands use full float32 arithmetic (no TF32); bf16 operands accumulate in
    float32.  `out_dtype=torch.float32` with bf16 operands returns the float32 accumulators unrounded."""
    _cuda(x, weight)
    if x.dtype != weight.dtype:
        if weight.dtype == torch.float32 and x.dtype == torch.bfloat16:
            # a weight stored in 32-bit stays so: the product runs in float32 and is rounded once at the end
            y = torch.mm(x.float(), weight.t())
            want = out_dtype or x.dtype
            if out is not None:
                out.copy_(y)
                return out
            return y.to(want)
        raise KernelError(f"linear: activations are {x.dtype} but the weight is {weight.dtype}")
    if out_dtype is not None and out_dtype != x.dtype:
        if out is not None:
            return torch.mm(x, weight.t(), out_dtype=out_dtype, out=out)
        return torch.mm(x, weight.t(), out_dtype=out_dtype)
    if out is not None:
        return torch.mm(x, weight.t(), out=out)
    return torch.mm(x, weight.t())


def configure_library_matmul() -> None:
    """Pin cuBLAS to exact modes: float32 products in true float32 (no TF32), bf16 products with float32
    accumulation and no reduced-precision split-K reduction."""
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    try:
        torch.backends.cuda.matmul.fp32_precision = "ieee"
    except (AttributeError, RuntimeError):
        torch.backends.cuda.matmul.allow_tf32 = False
