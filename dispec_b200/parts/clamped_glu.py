"""Gated feed-forwards beside SwiGLU.

``clamped_glu``: g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit);
y = g * sigmoid(alpha * g) * (u + 1); output W_down y.  No biases; the activation is 32-bit on the
32-bit rows of the fused gate/up product.

``token_table_input``: a per-token addend for a residual stream, from a table row of the token:
e = table[token][offset : offset + dim]; y = W_proj (gelu_tanh(W_gate x) * e).  The block that
uses it norms y (``norm_weight``, ``eps``: an RMS norm with a plain gain) and adds it.
"""
from __future__ import annotations

import torch

from dispec_b200 import ops
from dispec_b200.ops import norm32 as norm32_ops
from dispec_b200.parts.base import FeedForward, TensorSpec
from dispec_b200.registry import register_part


@register_part("feed_forward", "clamped_glu")
class ClampedGLU(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int, limit: float, alpha: float = 1.702):
        if not limit > 0:
            raise ValueError(f"clamped_glu: the limit must be positive, got {limit}")
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.limit, self.alpha = float(limit), float(alpha)

    def tensor_specs(self):
        h, i = self.hidden_size, self.intermediate_size
        return {"gate.weight": TensorSpec((i, h)), "up.weight": TensorSpec((i, h)), "down.weight": TensorSpec((h, i))}

    def load(self, tensors):
        self.w_gate_up = torch.cat([tensors["gate.weight"], tensors["up.weight"]], dim=0).contiguous()
        self.w_down = tensors["down.weight"]

    def forward(self, ctx, x):
        z = ops.linear(x, self.w_gate_up, out_dtype=torch.float32)
        return ops.linear(norm32_ops.clamped_glu(z, self.limit, self.alpha, x.dtype), self.w_down,
                          out_dtype=torch.float32)


@register_part("feed_forward", "token_table_input")
class TokenTableInput(FeedForward):
    def __init__(self, hidden_size: int, vocab_size: int, table_width: int, offset: int, dim: int, eps: float):
        if not 0 <= offset <= offset + dim <= table_width:
            raise ValueError(f"token_table_input: columns [{offset}, {offset + dim}) outside a table of {table_width}")
        self.hidden_size, self.vocab_size, self.table_width = hidden_size, vocab_size, table_width
        self.offset, self.dim, self.eps = offset, dim, float(eps)
        self.norm_weight = None

    def tensor_specs(self):
        return {"table": TensorSpec((self.vocab_size, self.table_width)),
                "gate.weight": TensorSpec((self.dim, self.hidden_size)),
                "proj.weight": TensorSpec((self.hidden_size, self.dim)),
                "norm.weight": TensorSpec((self.hidden_size,), dtype="float32", init="one_plus_normal")}

    def load(self, tensors):
        self.table, self.w_gate, self.w_proj = tensors["table"], tensors["gate.weight"], tensors["proj.weight"]
        self.norm_weight = tensors["norm.weight"]

    def forward(self, ctx, x):
        z = ops.linear(x, self.w_gate, out_dtype=torch.float32)
        g = norm32_ops.gelu_table_gate(z, self.table, self.offset, ctx.token_ids, x.dtype)
        return ops.linear(g, self.w_proj, out_dtype=torch.float32)
