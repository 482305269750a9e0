"""Linear-attention mixers whose memory is a matrix state per head and request, carried from
token to token in the request's state slot (32-bit floats, zero at admission):

    S_t = diag(a_t) S_(t-1) + b_t v_t^T,      o_t = S_t^T q_t        (S: [dim, vdim])

``retention``: a fixed decay per head, a_t = decay_h; q and k are turned by a rotary encoding
(pairs (i, i + rot/2)), k scaled by dim^(-1/2) afterwards, b_t = k_t; every head's o is divided
by its root mean square (no gain), the heads are multiplied by silu(W_g h) and projected.

``hgrn2``: the forget gate also decides what is written: f_t = lower + (1 - lower) *
sigmoid(W_f h + bias), a_t = f_t, b_t = 1 - f_t, q_t = silu(W_q h); every head's o is RMS-normed
with one gain of size vdim shared by the heads, then projected.

``lightning``: a fixed decay per head, q, k and v all pass through silu, a_t = decay_h, b_t = k_t,
no other scale; the concatenated heads are RMS-normed together with one gain over all of them,
multiplied by sigmoid(W_g h) and projected.

All run one fused projection, the recurrence kernel (which forms a_t, b_t, q_t from the raw
projection rows in 32-bit), the per-head norm kernel and the output projection.
"""
from __future__ import annotations

import torch

from dispec_b200 import ops
from dispec_b200.ops import norm32 as norm32_ops
from dispec_b200.ops import recurrence as rec_ops
from dispec_b200.parts.base import Mixer, StateNeed, TensorSpec
from dispec_b200.registry import register_part


class _MatrixStateMixer(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, dim: int, vdim: int, eps: float):
        if min(hidden_size, num_heads, dim, vdim) <= 0:
            raise ValueError("sizes of a linear-attention mixer must be positive")
        self.hidden_size, self.num_heads, self.dim, self.vdim = hidden_size, num_heads, dim, vdim
        self.eps = float(eps)
        self.w_in = self.w_o = None

    def state_need(self):
        return StateNeed((self.num_heads, self.dim, self.vdim), "float32")


@register_part("mixer", "retention")
class Retention(_MatrixStateMixer):
    def __init__(self, hidden_size: int, num_heads: int, dim: int, vdim: int, decay, eps: float,
                 position_encoding):
        super().__init__(hidden_size, num_heads, dim, vdim, eps)
        decay = [float(v) for v in decay]
        if len(decay) != num_heads:
            raise ValueError(f"retention: {len(decay)} decays for {num_heads} heads")
        self.decay_values = decay
        self.position_encoding = position_encoding
        self.decay = None

    def tensor_specs(self):
        h, H, d, dv = self.hidden_size, self.num_heads, self.dim, self.vdim
        return {"q.weight": TensorSpec((H * d, h)), "k.weight": TensorSpec((H * d, h)),
                "v.weight": TensorSpec((H * dv, h)), "g.weight": TensorSpec((H * dv, h)),
                "o.weight": TensorSpec((h, H * dv))}

    def load(self, tensors):
        self.w_in = torch.cat([tensors["q.weight"], tensors["k.weight"], tensors["v.weight"],
                               tensors["g.weight"]], dim=0).contiguous()
        self.w_o = tensors["o.weight"]
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=self.w_o.device)

    def forward(self, ctx, x, cache, state):
        H, d, dv = self.num_heads, self.dim, self.vdim
        proj = ops.linear(x, self.w_in, out_dtype=torch.float32)  # [T, q | k | v | g]
        rot = self.position_encoding.rotation()
        if rot is not None and rot.layout != "halves":
            raise ValueError(f"retention turns pairs (i, i + rot/2) only, not the {rot.layout!r} layout")
        o = rec_ops.linear_recurrence(
            proj, 0, H * d, 2 * H * d, rec_ops.FIXED_DECAY, H, d, dv, state.buffer, state.slots, ctx.q_start,
            ctx.positions, decay=self.decay, inv_freq=rot.inv_freq if rot is not None else None,
            rot=rot.rotary_dim if rot is not None else 0, key_scale=d ** -0.5)
        gated = norm32_ops.head_norm_gate(o, H, self.eps, x.dtype, gate=proj[:, 2 * H * d + H * dv:])
        return ops.linear(gated, self.w_o, out_dtype=torch.float32)


@register_part("mixer", "hgrn2")
class HGRN2(_MatrixStateMixer):
    def tensor_specs(self):
        h, H, d, dv = self.hidden_size, self.num_heads, self.dim, self.vdim
        return {"q.weight": TensorSpec((H * d, h)), "f.weight": TensorSpec((H * d, h)),
                "f.bias": TensorSpec((H * d,), dtype="float32", init="zeros"),
                "lower": TensorSpec((H * d,), dtype="float32", init="zeros"),
                "v.weight": TensorSpec((H * dv, h)),
                "norm.weight": TensorSpec((dv,), dtype="float32", init="one_plus_normal"),
                "o.weight": TensorSpec((h, H * dv))}

    def load(self, tensors):
        self.w_in = torch.cat([tensors["q.weight"], tensors["f.weight"], tensors["v.weight"]], dim=0).contiguous()
        self.f_bias, self.lower, self.gain = tensors["f.bias"], tensors["lower"], tensors["norm.weight"]
        self.w_o = tensors["o.weight"]

    def forward(self, ctx, x, cache, state):
        H, d, dv = self.num_heads, self.dim, self.vdim
        proj = ops.linear(x, self.w_in, out_dtype=torch.float32)  # [T, q | f | v]
        o = rec_ops.linear_recurrence(
            proj, 0, H * d, 2 * H * d, rec_ops.FORGET_GATE, H, d, dv, state.buffer, state.slots, ctx.q_start,
            ctx.positions, gate_bias=self.f_bias, lower=self.lower)
        normed = norm32_ops.head_norm_gate(o, H, self.eps, x.dtype, gain=self.gain)
        return ops.linear(normed, self.w_o, out_dtype=torch.float32)


@register_part("mixer", "lightning")
class Lightning(_MatrixStateMixer):
    def __init__(self, hidden_size: int, num_heads: int, dim: int, vdim: int, decay, eps: float):
        super().__init__(hidden_size, num_heads, dim, vdim, eps)
        decay = [float(v) for v in decay]
        if len(decay) != num_heads:
            raise ValueError(f"lightning: {len(decay)} decays for {num_heads} heads")
        self.decay_values = decay
        self.decay = self.gain = None

    def tensor_specs(self):
        h, H, d, dv = self.hidden_size, self.num_heads, self.dim, self.vdim
        return {"q.weight": TensorSpec((H * d, h)), "k.weight": TensorSpec((H * d, h)),
                "v.weight": TensorSpec((H * dv, h)), "g.weight": TensorSpec((H * dv, h)),
                "norm.weight": TensorSpec((H * dv,), dtype="float32", init="one_plus_normal"),
                "o.weight": TensorSpec((h, H * dv))}

    def load(self, tensors):
        self.w_in = torch.cat([tensors["q.weight"], tensors["k.weight"], tensors["v.weight"],
                               tensors["g.weight"]], dim=0).contiguous()
        self.w_o, self.gain = tensors["o.weight"], tensors["norm.weight"]
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=self.w_o.device)

    def forward(self, ctx, x, cache, state):
        H, d, dv = self.num_heads, self.dim, self.vdim
        proj = ops.linear(x, self.w_in, out_dtype=torch.float32)  # [T, q | k | v | g]
        o = rec_ops.linear_recurrence(
            proj, 0, H * d, 2 * H * d, rec_ops.FIXED_DECAY, H, d, dv, state.buffer, state.slots, ctx.q_start,
            ctx.positions, decay=self.decay, silu_inputs=True)
        gated = norm32_ops.head_norm_gate(o, 1, self.eps, x.dtype, gain=self.gain,
                                          gate=proj[:, 2 * H * d + H * dv:], gate_kind="sigmoid")
        return ops.linear(gated, self.w_o, out_dtype=torch.float32)
