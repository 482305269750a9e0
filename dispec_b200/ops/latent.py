"""Attention over a cached latent (one shared key/value row per token): the store of a token's
normalised latent and rotated key part into the pages, and the attention itself in 32-bit.
See ``csrc/attn_latent.cu``."""
from __future__ import annotations

import torch

from dispec_b200.ops import library as L


def latent_store(down: torch.Tensor, c_off: int, r_off: int, gain: torch.Tensor, eps: float,
                 inv_freq: torch.Tensor | None, rot: int, positions: torch.Tensor, seq_of_token: torch.Tensor,
                 page_table: torch.Tensor, c_pool: torch.Tensor, r_pool: torch.Tensor) -> None:
    """``down`` [T, columns]: rows of the down projection; columns c_off.. hold the R latent values
    (RMS-normed here with ``gain``), columns r_off.. the r values of the shared key part (pairs
    (2i, 2i+1) of its first ``rot`` values turned by position * inv_freq[i]).  Pools:
    [num_pages, 1, page_size, R] and [num_pages, 1, page_size, r]."""
    if not (down.is_cuda and c_pool.is_cuda):
        raise L.KernelError("latent_store: CUDA tensors only (there is no CPU path)")
    assert down.dim() == 2 and down.stride(1) == 1
    num_pages, one, page_size, R = c_pool.shape
    r = r_pool.shape[3]
    assert one == 1 and r_pool.shape[:3] == (num_pages, 1, page_size) and r_pool.dtype == c_pool.dtype
    assert c_pool.is_contiguous() and r_pool.is_contiguous()
    assert gain.dtype == torch.float32 and gain.shape == (R,) and gain.is_contiguous()
    assert positions.dtype == torch.int32 and seq_of_token.dtype == torch.int32
    assert page_table.dtype == torch.int32 and page_table.dim() == 2 and page_table.stride(1) == 1
    if rot:
        assert inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.shape[0] >= rot // 2
    lib = L.mixer_library("attn_latent")
    L.check(lib.dsp_latent_store(
        L.ptr(down), L.dtype_code(down.dtype), L.i64(down.stride(0)), c_off, r_off, L.ptr(gain), L.f32(eps),
        L.ptr(inv_freq), rot, L.ptr(positions), L.ptr(seq_of_token), L.ptr(page_table), page_table.stride(0),
        L.ptr(c_pool), L.ptr(r_pool), L.dtype_code(c_pool.dtype), down.shape[0], R, r, page_size, num_pages,
        L.stream_handle()))


def latent_attention(q_absorbed: torch.Tensor, q: torch.Tensor, q_head_stride: int, qr_off: int,
                     inv_freq: torch.Tensor | None, rot: int, c_pool: torch.Tensor, r_pool: torch.Tensor,
                     page_table: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor,
                     num_heads: int, scale: float, out_dtype: torch.dtype) -> torch.Tensor:
    """``q_absorbed`` float32 [T, H * R]: every head's query with the key map folded in.  ``q``
    [T, columns]: the projected queries; head h's part to be rotated starts at column
    h * q_head_stride + qr_off and has r values.  Returns sum_j softmax_j c_j per head as
    [T, H * R] of ``out_dtype``; the query at position p sees every cached j <= p."""
    if not (q_absorbed.is_cuda and c_pool.is_cuda):
        raise L.KernelError("latent_attention: CUDA tensors only (there is no CPU path)")
    num_pages, _, page_size, R = c_pool.shape
    r = r_pool.shape[3]
    T = positions.shape[0]
    assert q_absorbed.dtype == torch.float32 and q_absorbed.shape == (T, num_heads * R) and q_absorbed.stride(1) == 1
    assert q.dim() == 2 and q.stride(1) == 1 and q.shape[0] == T
    assert c_pool.is_contiguous() and r_pool.is_contiguous() and r_pool.dtype == c_pool.dtype
    assert page_table.dtype == torch.int32 and page_table.stride(1) == 1
    assert positions.dtype == torch.int32 and seq_of_token.dtype == torch.int32
    out = torch.empty((T, num_heads * R), dtype=out_dtype, device=q.device)
    lib = L.mixer_library("attn_latent")
    L.check(lib.dsp_attn_latent(
        L.ptr(q_absorbed), L.i64(q_absorbed.stride(0)), L.ptr(q), L.dtype_code(q.dtype), L.i64(q.stride(0)),
        q_head_stride, qr_off, L.ptr(inv_freq), rot, L.ptr(c_pool), L.ptr(r_pool), L.dtype_code(c_pool.dtype),
        L.ptr(page_table), page_table.stride(0), L.ptr(positions), L.ptr(seq_of_token), L.ptr(out),
        L.dtype_code(out_dtype), L.i64(out.stride(0)), T, num_heads, R, r, page_size, num_pages, L.f32(scale),
        L.stream_handle()))
    return out
