"""Dense feed-forward with the xIELU activation: down(act(up h)), no gate, no biases;

    act(z) = softplus(p) z^2 + z / 2                            for z > 0
           = (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2       otherwise

with the layer's two learned numbers (p, q)."""
from __future__ import annotations

import torch

from dispec_b200 import ops
from dispec_b200.ops import norm32 as norm32_ops
from dispec_b200.parts.base import FeedForward, TensorSpec
from dispec_b200.registry import register_part


@register_part("feed_forward", "xielu")
class XIELUFeedForward(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int):
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size

    def tensor_specs(self):
        h, i = self.hidden_size, self.intermediate_size
        return {"up.weight": TensorSpec((i, h)), "down.weight": TensorSpec((h, i)),
                "act": TensorSpec((2,), dtype="float32")}

    def load(self, tensors):
        self.w_up, self.w_down, self.act = tensors["up.weight"], tensors["down.weight"], tensors["act"]

    def forward(self, ctx, x):
        z = ops.linear(x, self.w_up, out_dtype=torch.float32)
        return ops.linear(norm32_ops.xielu(z, self.act, x.dtype), self.w_down, out_dtype=torch.float32)
