"""SiLU-gated feed-forward: `down(silu(gate(x)) * up(x))`, no bias
(src/minillm/runtime.cpp:323-335; src/minillm/cuda/layer.cpp:65-70).

The gate and up matrices are stacked into one operand at bind time, so one product
yields both, and the gate is applied by that product's epilogue or by the kernel that
reads its result; how the rows are stacked is the runtime's business
(`Runtime.stack_gate_up`), which may round the inner width up (the extra activations
are zero, and "down" gets zero columns for them).  Parameters: hidden_size,
intermediate_size.  Weights: "gate", "up" [I, width], "down" [width, I].
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..config.registry import register_part
from ..ops import functions as F
from ..weights.loader import WeightSpec
from .base import FeedForward, StepContext


class SwiGLU(FeedForward):
    def __init__(self, spec):
        super().__init__(spec)
        self.width = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.w_gate_up = None
        self.w_down = None

    def weight_specs(self) -> List[WeightSpec]:
        w = self.spec.weights
        return [WeightSpec(w["gate"], (self.inter, self.width)), WeightSpec(w["up"], (self.inter, self.width)),
                WeightSpec(w["down"], (self.width, self.inter))]

    def kernel_modules(self, dtype) -> List[str]:
        return ["elementwise"] + F.product_modules(dtype)

    def bind(self, tensors: Dict[str, torch.Tensor], rt) -> None:
        w = self.spec.weights
        self.w_gate_up, inner = rt.stack_gate_up(tensors[w["gate"]], tensors[w["up"]])
        self.w_down = rt.matrix(tensors[w["down"]])
        if inner != self.inter:
            padded = torch.zeros((self.width, inner), dtype=self.w_down.dtype, device=self.w_down.device)
            padded[:, :self.inter] = self.w_down
            self.w_down = padded

    def emit(self, b, x):
        act = b.rt.gated_linear(b, x, self.w_gate_up)
        return b.rt.linear_delta(b, act, self.w_down, into=b.residual)


register_part("feed_forward", "swiglu", SwiGLU)


class GatedBiasFeedForward(FeedForward):
    """Gated feed-forward whose three projections have biases: `down(act(gate x + b_g) * (up x + b_u)) + b_d`,
    act = SiLU or the tanh form of GELU.  Gate and up are one stacked product; a row-wise kernel adds their
    biases and gates; the last bias travels with the result (`Buf.bias`) to whoever adds it into the stream.
    A third activation, "swish", is `g * sigmoid(alpha * g) * (u + up_offset)` with g = gate x + b_g and u = up x + b_u, after
    g <- min(g, limit) and u <- clamp(u, -limit, limit) where a limit is given.
    Parameters: hidden_size, intermediate_size, activation ("silu" | "gelu_tanh" | "swish"), and for "swish" alpha (default 1),
    limit (default none), up_offset (default 0).  Weights: "gate", "up" [I, width], "down" [width, I], "gate_bias", "up_bias" [I],
    "down_bias" [width]."""
    ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "swish": 2}

    def __init__(self, spec):
        super().__init__(spec)
        self.width = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.activation = self.ACTIVATIONS[spec.params.get("activation", "silu")]
        self.alpha, self.limit = float(spec.params.get("alpha", 1.0)), float(spec.params.get("limit") or 0.0)
        self.up_offset = float(spec.params.get("up_offset", 0.0))
        if self.activation != 2 and (self.alpha != 1.0 or self.limit or self.up_offset):
            raise ValueError("alpha, limit and up_offset belong to the activation 'swish'")
        self.w_gate_up = self.w_down = self.b_gate = self.b_up = self.b_down = None

    def weight_specs(self) -> List[WeightSpec]:
        w = self.spec.weights
        return [WeightSpec(w["gate"], (self.inter, self.width)), WeightSpec(w["up"], (self.inter, self.width)),
                WeightSpec(w["down"], (self.width, self.inter)),
                WeightSpec(w["gate_bias"], (self.inter,), "vector", ("normal", 0.02)),
                WeightSpec(w["up_bias"], (self.inter,), "vector", ("normal", 0.02)),
                WeightSpec(w["down_bias"], (self.width,), "vector", ("normal", 0.02))]

    def kernel_modules(self, dtype) -> List[str]:
        return ["elementwise"] + F.product_modules(dtype)

    def bind(self, tensors: Dict[str, torch.Tensor], rt) -> None:
        w = self.spec.weights
        self.w_gate_up = torch.cat([rt.matrix(tensors[w["gate"]]), rt.matrix(tensors[w["up"]])], dim=0).contiguous()
        self.w_down = rt.matrix(tensors[w["down"]])
        self.b_gate, self.b_up, self.b_down = (rt.vector(tensors[w[r]]).float() for r in ("gate_bias", "up_bias", "down_bias"))

    def emit(self, b, x):
        rt = b.rt
        both = rt.linear(b, x, self.w_gate_up, activation=True)
        act = b.temp(x.rows, self.inter, rt.dtype)
        b.launch("elementwise", "mlr_gated_bias_shaped", both.ptr, both.ld, self.b_gate.data_ptr(), self.b_up.data_ptr(), act.ptr, act.ld,
                 act.is_bf16, x.rows, self.inter, self.activation, self.alpha, self.limit, self.up_offset, b.stream)
        out = rt.linear(b, act, self.w_down, out_dtype=torch.float32)
        out.bias = self.b_down
        return out


register_part("feed_forward", "gated_bias", GatedBiasFeedForward)


class PlainFeedForward(FeedForward):
    """Feed-forward without a gate: `down(act(up(x)))`, no biases; act is the square of relu ("relu2"), the tanh form of
    GELU ("gelu_tanh") or SiLU ("silu"), applied in the first product's epilogue where its kernel has one
    (`Runtime.activated_linear`) and by a row-wise kernel between the two products otherwise.
    Parameters: hidden_size, intermediate_size, activation.  Weights: "up" [I, width], "down" [width, I]."""
    ACTIVATIONS = {"relu2": 0, "gelu_tanh": 1, "silu": 2}

    def __init__(self, spec):
        super().__init__(spec)
        self.width = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.activation = self.ACTIVATIONS[spec.params["activation"]]
        self.w_up = self.w_down = None

    def weight_specs(self) -> List[WeightSpec]:
        w = self.spec.weights
        return [WeightSpec(w["up"], (self.inter, self.width)), WeightSpec(w["down"], (self.width, self.inter))]

    def kernel_modules(self, dtype) -> List[str]:
        return ["elementwise"] + F.product_modules(dtype)

    def bind(self, tensors: Dict[str, torch.Tensor], rt) -> None:
        w = self.spec.weights
        self.w_up, self.w_down = rt.matrix(tensors[w["up"]]), rt.matrix(tensors[w["down"]])

    def emit(self, b, x):
        rt = b.rt
        up = rt.activated_linear(b, x, self.w_up, self.spec.params["activation"])
        if b.residual is not None:
            return rt.linear_delta(b, up, self.w_down, into=b.residual)
        return rt.linear(b, up, self.w_down, out_dtype=torch.float32)      # a block whose norm stands behind wants the plain result


register_part("feed_forward", "plain", PlainFeedForward)
