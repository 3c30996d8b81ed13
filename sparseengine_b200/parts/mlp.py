"""An ungated feed-forward: ``down(act(up(x)))``.

The two products are library GEMMs (or this library's few-row kernel) through
:func:`parts.linear.linear`; the activation runs in place between them in 32-bit arithmetic
(kernel: csrc/stream32.cu).
"""
from __future__ import annotations

from ..config.specs import ParamSpec
from ..csrc import ops
from .base import FeedForward, register_feed_forward
from .linear import linear


class PlainMLP(FeedForward):
    graph_safe = True

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        if spec.activation not in ops.ACTIVATIONS:
            raise ValueError(f"activation {spec.activation!r} is not supported; known: {sorted(ops.ACTIVATIONS)}")
        if spec.hidden_size <= 0 or spec.intermediate_size <= 0:
            raise ValueError("hidden_size and intermediate_size must be positive")

    def parameters(self):
        s = self.spec
        return {"up": ParamSpec((s.intermediate_size, s.hidden_size)),
                "down": ParamSpec((s.hidden_size, s.intermediate_size))}

    def forward(self, x, step):
        h = linear(x, self.up)
        ops.activation_(h, self.spec.activation)
        return linear(h, self.down)


register_feed_forward("plain_mlp", PlainMLP)
