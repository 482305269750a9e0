"""Row-wise kernels around a residual stream kept in 32-bit floats: the RMS norm of a scaled sum,
the per-head RMS norm with gain and gate that closes a linear-attention mixer, and xIELU.
Every operand is float32 or bfloat16 on its own; the arithmetic is 32-bit."""
from __future__ import annotations

import torch

from dispec_b200.ops import library as L


def _rows2d(t: torch.Tensor, what: str) -> None:
    if not (t.is_cuda and t.dim() == 2 and t.stride(1) == 1):
        raise L.KernelError(f"{what}: a CUDA matrix with unit column stride is needed (there is no CPU path)")


def sum_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, delta: torch.Tensor | None = None,
             alpha: float = 1.0, rows: torch.Tensor | None = None, out32: torch.Tensor | None = None,
             out_dtype: torch.dtype | None = None, want32: bool = True):
    """y = weight * s / sqrt(mean(s^2) + eps) with s = alpha * x + delta, per row, in 32-bit.

    Returns (y as float32 or None, y rounded to ``out_dtype`` or None).  ``out32`` may be ``x``
    itself.  ``rows`` (int32) gathers input rows; the outputs are dense."""
    _rows2d(x, "sum_norm")
    assert weight.dtype == torch.float32 and weight.is_contiguous() and weight.shape == (x.shape[1],)
    if delta is not None:
        _rows2d(delta, "sum_norm")
        assert delta.shape == x.shape
    n = x.shape[0] if rows is None else rows.shape[0]
    width = x.shape[1]
    if rows is not None:
        assert rows.dtype == torch.int32 and rows.is_contiguous()
    y32 = out32
    if y32 is None and want32:
        y32 = torch.empty((n, width), dtype=torch.float32, device=x.device)
    y16 = None
    if out_dtype is not None and not (out_dtype == torch.float32 and y32 is not None):
        y16 = torch.empty((n, width), dtype=out_dtype, device=x.device)
    L.check(L.core().dsp_sum_norm(
        L.ptr(x), L.dtype_code(x.dtype), L.i64(x.stride(0)), L.ptr(delta),
        L.dtype_code(delta.dtype) if delta is not None else 0, L.i64(delta.stride(0) if delta is not None else 0),
        L.ptr(weight), L.f32(alpha), L.f32(eps), L.ptr(rows), L.ptr(y32), L.i64(y32.stride(0) if y32 is not None else 0),
        L.ptr(y16), L.dtype_code(y16.dtype) if y16 is not None else 0, L.i64(y16.stride(0) if y16 is not None else 0),
        n, width, L.stream_handle()))
    if out_dtype == torch.float32 and y16 is None:
        y16 = y32
    return y32, y16


def head_norm_gate(o: torch.Tensor, num_heads: int, eps: float, out_dtype: torch.dtype,
                   gain: torch.Tensor | None = None, gate: torch.Tensor | None = None) -> torch.Tensor:
    """o float32 [T, H * dv]: every head's dv values divided by their root mean square (eps inside
    the root), times ``gain`` [dv] (optional) and silu(gate[t, h * dv + j]) (optional)."""
    _rows2d(o, "head_norm_gate")
    assert o.dtype == torch.float32 and o.shape[1] % num_heads == 0
    T, dv = o.shape[0], o.shape[1] // num_heads
    if gain is not None:
        assert gain.dtype == torch.float32 and gain.shape == (dv,) and gain.is_contiguous()
    if gate is not None:
        _rows2d(gate, "head_norm_gate")
        assert gate.shape == o.shape
    y = torch.empty((T, o.shape[1]), dtype=out_dtype, device=o.device)
    L.check(L.core().dsp_head_norm_gate(
        L.ptr(o), L.i64(o.stride(0)), L.ptr(gain), L.ptr(gate), L.dtype_code(gate.dtype) if gate is not None else 0,
        L.i64(gate.stride(0) if gate is not None else 0), L.ptr(y), L.dtype_code(out_dtype), L.i64(y.stride(0)),
        T, num_heads, dv, L.f32(eps), L.stream_handle()))
    return y


def xielu(z: torch.Tensor, params: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """xIELU of every element: softplus(p) z^2 + z/2 for z > 0, (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2
    otherwise; ``params`` = (p, q) as a float32 device tensor."""
    _rows2d(z, "xielu")
    assert params.dtype == torch.float32 and params.numel() == 2 and params.is_cuda
    y = torch.empty(z.shape, dtype=out_dtype, device=z.device)
    L.check(L.core().dsp_xielu(L.ptr(z), L.dtype_code(z.dtype), L.i64(z.stride(0)), L.ptr(params), L.ptr(y),
                               L.dtype_code(out_dtype), L.i64(y.stride(0)), L.i64(z.shape[0]), z.shape[1],
                               L.stream_handle()))
    return y
