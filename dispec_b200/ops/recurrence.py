"""Linear attention as a recurrence over a per-request matrix state (32-bit, FMA units):
S_t = diag(a_t) S_(t-1) + b_t v_t^T,  o_t = S_t^T q_t.  See ``csrc/linear_recurrence.cu``."""
from __future__ import annotations

import torch

from dispec_b200.ops import library as L

FIXED_DECAY, FORGET_GATE = 0, 1


def linear_recurrence(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, mode: int, num_heads: int,
                      dim: int, vdim: int, state: torch.Tensor, state_slot: torch.Tensor,
                      q_start: torch.Tensor, positions: torch.Tensor, *, decay: torch.Tensor | None = None,
                      inv_freq: torch.Tensor | None = None, rot: int = 0, key_scale: float = 1.0,
                      gate_bias: torch.Tensor | None = None, lower: torch.Tensor | None = None,
                      silu_inputs: bool = False) -> torch.Tensor:
    """``proj`` [T, columns]: the raw rows of the mixer's fused projection (query columns from
    ``q_off``, key or forget-gate columns from ``k_off``, value columns from ``v_off``, each head by
    head).  ``state`` float32 [slots, H, dim, vdim] is read and left updated for the sequences of the
    step (``q_start`` [S + 1], ``state_slot`` [S]); a sequence whose first position is negative is
    skipped.  ``silu_inputs`` (fixed decay only): the raw query, key and value columns pass through
    silu before anything else.  Returns o as float32 [T, H * vdim]."""
    if not (proj.is_cuda and state.is_cuda):
        raise L.KernelError("linear_recurrence: CUDA tensors only (there is no CPU path)")
    assert proj.dim() == 2 and proj.stride(1) == 1
    assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (num_heads, dim, vdim)
    for t in (state_slot, q_start, positions):
        assert t.dtype == torch.int32 and t.is_contiguous()
    for t in (decay, inv_freq, gate_bias, lower):
        assert t is None or (t.dtype == torch.float32 and t.is_contiguous() and t.is_cuda)
    S = state_slot.shape[0]
    assert q_start.shape[0] == S + 1
    T = proj.shape[0]
    out = torch.empty((T, num_heads * vdim), dtype=torch.float32, device=proj.device)
    lib = L.mixer_library("linear_recurrence")
    # portions of prompts: a first, parallel kernel writes q_t, b_t (a_t) of every token as floats and
    # the sequential kernel streams them; steps of (nearly) single tokens transform while staging
    scratch = None
    if T > 2 * S:
        planes = 3 if mode == FORGET_GATE else 2
        scratch = torch.empty((T, planes, num_heads * dim), dtype=torch.float32, device=proj.device)
    L.check(lib.dsp_linear_recurrence(
        L.ptr(proj), L.dtype_code(proj.dtype), L.i64(proj.stride(0)), q_off, k_off, v_off, mode, num_heads, dim,
        vdim, L.ptr(decay), L.ptr(inv_freq), rot, L.f32(key_scale), int(silu_inputs), L.ptr(gate_bias), L.ptr(lower), L.ptr(state),
        L.ptr(state_slot), L.ptr(q_start), L.ptr(positions), L.ptr(out), L.i64(out.stride(0)), S, T,
        L.ptr(scratch), L.stream_handle()))
    return out
