"""RMS norm, fused with the residual add that precedes it.

`(x * 1/sqrt(mean(x^2) + eps)) * w` over the full width, in float32
(src/minillm/kernels.cpp:209-216; GPU twin src/minillm/cuda/ops.cu:87-126).
Parameters: width, eps.  Weights: "weight" [width].
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.registry import register_part
from ..engine.builder import Buf
from ..ops import native
from ..weights.loader import WeightSpec
from .base import Norm, StepContext


class RmsNorm(Norm):
    def __init__(self, spec):
        super().__init__(spec)
        self.width = int(spec.params["width"])
        self.eps = float(spec.params["eps"])
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.spec.weights["weight"], (self.width,), "vector", ("one_plus_normal", 0.01))]

    def kernel_modules(self, dtype) -> List[str]:
        return ["elementwise"]

    def bind(self, tensors: Dict[str, torch.Tensor], rt) -> None:
        self.weight = rt.vector(tensors[self.spec.weights["weight"]])

    def foldable(self):
        return ("rms", self.weight, self.eps, self.width)

    def emit(self, b, h, delta, wanted_only: bool = False):
        """out[r] = rmsnorm(h[row] + delta[row]) * weight, row = the r-th wanted row or r; unless only
        the wanted rows are normed, the sum is stored back to h, which moves the residual stream on.
        `delta` may be partial sums [S, M, width], which are added in order first."""
        if delta is not None and getattr(delta, "bias", None) is not None:
            raise native.KernelError("this norm cannot add the bias its contribution carries")
        count = b.want if wanted_only else h.rows
        prepared, b.prepared = b.prepared, None
        if delta is None and b.rt.norm_can_wait(b, count, self.width):
            # The product that reads this norm's result will norm its own input (a few-row product
            # streams the weights once and has the rows in shared memory anyway): nothing to launch here.
            # The product that last added into the stream may have left this norm half done.
            if prepared is not None and (wanted_only or prepared["stream"] != h.ptr or prepared["weight"] is not self.weight):
                prepared = None
            return Buf(None, count, self.width, b.rt.dtype, self.width, norm=(h, self.weight, self.eps, wanted_only, prepared))
        out = b.temp(count, self.width, b.rt.dtype)
        slices, stride = (delta.slices or 1, delta.slice_stride) if delta is not None else (1, 0)
        b.launch("elementwise", "mlr_rmsnorm", h.ptr, delta.ptr if delta is not None else None, slices, stride,
                 self.weight.data_ptr(), native.is_bf16(self.weight), out.ptr, out.is_bf16,
                 b.meta("want_rows") if wanted_only else None, count, self.width, self.eps, int(not wanted_only), b.stream,
                 need="want" if wanted_only else None)
        return out


register_part("norm", "rmsnorm", RmsNorm)


class GroupRmsNorm(Norm):
    """RMS norm in groups: the vector in `groups` equal consecutive parts, each over its own root mean
    square, the whole times a weight.  groups = 1 is `rmsnorm` computed by the same kernel.

    Besides the interface of every norm (`emit`: add a pending contribution as it is, then norm) it can
    stand BEHIND a sub-layer: `emit_residual` adds norm(contribution [+ bias]) * weight into the stream,
    and in the same launch applies the norm that reads the stream next (`then`), if one is named: a grouped norm of the
    same shape, or no norm at all (`identity`: the sub-layers of such a model read the stream as it is).
    With `offset` the stored weight is the distance from that number: the norm multiplies by offset + weight.
    Parameters: width, groups, eps, offset (default 0).  Weights: "weight" [width]."""

    def __init__(self, spec):
        super().__init__(spec)
        self.width = int(spec.params["width"])
        self.groups = int(spec.params.get("groups", 1))
        self.eps = float(spec.params["eps"])
        self.offset = float(spec.params.get("offset") or 0.0)
        if self.groups < 1 or self.width % self.groups:
            raise ValueError(f"a norm over {self.width} values cannot have {self.groups} equal groups")
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        init = ("normal", 0.05) if self.offset else ("one_plus_normal", 0.01)
        return [WeightSpec(self.spec.weights["weight"], (self.width,), "vector", init)]

    def kernel_modules(self, dtype) -> List[str]:
        return ["norm_grouped"]

    def bind(self, tensors: Dict[str, torch.Tensor], rt) -> None:
        self.weight = rt.vector(tensors[self.spec.weights["weight"]]).float()
        if self.offset:
            self.weight = (self.weight + self.offset).contiguous()       # float32: 1 + w keeps what bfloat16 would drop

    def foldable(self):
        """The block before may apply this norm in the launch that ends it (`emit_residual(then=...)`) and leave the
        result on the builder (`prepared`)."""
        return ("group_rms", self)

    def emit(self, b, h, delta, wanted_only: bool = False):
        if delta is not None and (delta.slices or wanted_only):
            raise native.KernelError("the grouped norm adds a plain [rows, width] contribution for all rows only")
        prepared, b.prepared = b.prepared, None
        if (delta is None and not wanted_only and isinstance(prepared, dict) and prepared.get("group_rms") is self
                and prepared.get("stream") is h):
            return prepared["out"]          # the launch that ended the block before has applied this norm already
        count = b.want if wanted_only else h.rows
        out = b.temp(count, self.width, b.rt.dtype)
        bias = getattr(delta, "bias", None) if delta is not None else None
        b.launch("norm_grouped", "mlr_group_rmsnorm", h.ptr, delta.ptr if delta is not None else None,
                 delta.ld if delta is not None else 0, bias.data_ptr() if bias is not None else None, None,
                 self.weight.data_ptr(), out.ptr, out.ld, out.is_bf16, b.meta("want_rows") if wanted_only else None, count,
                 self.width, self.groups, self.eps, 0, b.stream, need="want" if wanted_only else None)
        return out

    def same_shape(self, other) -> bool:
        if isinstance(other, IdentityNorm):
            return other.width == self.width
        return isinstance(other, GroupRmsNorm) and (other.width, other.groups, other.eps) == (self.width, self.groups, self.eps)

    takes_pieces = True      # `emit_residual` adds up a contribution that routed experts left in pieces (`Buf.pieces`)

    def emit_residual(self, b, h, delta, then: Optional[Norm] = None):
        """h += norm(delta + its bias) * weight; returns then(h) in the activation dtype, or None."""
        if delta.slices:
            raise native.KernelError("the grouped norm takes a plain [rows, width] contribution")
        plain = isinstance(then, IdentityNorm)
        if plain and then.reads_stream(b, h):
            then = None                 # the reader takes the float32 stream itself: nothing to write for it
        if then is not None and not self.same_shape(then):
            out = None
        else:
            out = b.temp(h.rows, self.width, b.rt.dtype) if then is not None else None
        bias = getattr(delta, "bias", None)
        w_pre = then.weight.data_ptr() if out is not None and not plain else None
        if delta.pieces is not None:
            y, row_of_pair, weights, top, shared, gate = delta.pieces
            if bias is not None or y.dtype is not torch.float32 or (shared is not None and shared.dtype is not torch.float32):
                raise native.KernelError("the grouped norm adds up float32 pieces without a bias")
            b.launch("norm_grouped", "mlr_group_rmsnorm_pieces", h.ptr, y.ptr, self.width, row_of_pair.ptr, weights.ptr, top,
                     shared.ptr if shared is not None else None, shared.ld if shared is not None else 0, gate.ptr if gate is not None else None,
                     self.weight.data_ptr(), w_pre, out.ptr if out is not None else None, out.ld if out is not None else 0,
                     int(b.rt.is_bf16), h.rows, self.width, self.groups, self.eps, 1 | (2 if plain else 0), b.stream)
        else:
            b.launch("norm_grouped", "mlr_group_rmsnorm", h.ptr, delta.ptr, delta.ld, bias.data_ptr() if bias is not None else None,
                     self.weight.data_ptr(), w_pre, out.ptr if out is not None else None, out.ld if out is not None else 0,
                     int(b.rt.is_bf16), None, h.rows, self.width, self.groups, self.eps, 1 | (2 if plain else 0), b.stream)
        if plain and then is None:
            return h
        if then is not None and out is None:
            return then.emit(b, h, None)
        return out


register_part("norm", "group_rmsnorm", GroupRmsNorm)


class IdentityNorm(Norm):
    """No norm: the reader takes the residual stream as it is, in the activation dtype.  It stands where a block expects a
    norm in front of a sub-layer in designs whose norms stand behind their sub-layers only.  On the 32-bit path the result
    IS the stream (no launch, no copy); in bfloat16 it is the stream's rounding, written by the launch that last added into
    the stream (`GroupRmsNorm.emit_residual(then=...)`) or by a launch of its own.  Parameters: width.  No weights."""

    def __init__(self, spec):
        super().__init__(spec)
        self.width = int(spec.params["width"])
        self.weight = None

    def kernel_modules(self, dtype) -> List[str]:
        return ["norm_grouped"]

    def foldable(self):
        return ("group_rms", self)

    def reads_stream(self, b, h) -> bool:
        return b.rt.dtype is torch.float32 and h.dtype is torch.float32 and h.ld == h.width == self.width

    def emit(self, b, h, delta, wanted_only: bool = False):
        if delta is not None and (delta.slices or wanted_only or getattr(delta, "norm", None) is not None):
            raise native.KernelError("this part adds a plain [rows, width] contribution for all rows only")
        prepared, b.prepared = b.prepared, None
        if (delta is None and not wanted_only and isinstance(prepared, dict) and prepared.get("group_rms") is self
                and prepared.get("stream") is h):
            return prepared["out"]          # the launch that ended the block before has written the copy already
        if delta is None and not wanted_only and self.reads_stream(b, h):
            return h
        count = b.want if wanted_only else h.rows
        out = b.temp(count, self.width, b.rt.dtype)
        bias = getattr(delta, "bias", None) if delta is not None else None
        b.launch("norm_grouped", "mlr_group_rmsnorm", h.ptr, delta.ptr if delta is not None else None,
                 delta.ld if delta is not None else 0, bias.data_ptr() if bias is not None else None, None, None, out.ptr, out.ld,
                 out.is_bf16, b.meta("want_rows") if wanted_only else None, count, self.width, 1, 0.0, 2, b.stream,
                 need="want" if wanted_only else None)
        return out


register_part("norm", "identity", IdentityNorm)


class LayerNorm(Norm):
    """Layer norm with weight and bias: `(x - mean) / sqrt(var + eps) * w + b`, the variance as the mean of the squared
    deviations, all float32 (`mlr_depth_norm` of `layernorm.cu`, which a block may also hand the sub-layers' results
    and the stream's earlier states: `parts/block.py`).  Parameters: width, eps.  Weights: "weight", "bias" [width]."""

    def __init__(self, spec):
        super().__init__(spec)
        self.width = int(spec.params["width"])
        self.eps = float(spec.params["eps"])
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.spec.weights["weight"], (self.width,), "vector", ("one_plus_normal", 0.01)),
                WeightSpec(self.spec.weights["bias"], (self.width,), "vector", ("normal", 0.02))]

    def kernel_modules(self, dtype) -> List[str]:
        return ["layernorm"]

    def bind(self, tensors: Dict[str, torch.Tensor], rt) -> None:
        self.weight = rt.vector(tensors[self.spec.weights["weight"]]).float().contiguous()
        self.bias = rt.vector(tensors[self.spec.weights["bias"]]).float().contiguous()

    def foldable(self):
        """The block before may apply this norm in the launch that ends it and leave the result on the builder (`prepared`)."""
        return ("layernorm", self)

    def same_shape(self, other) -> bool:
        return isinstance(other, LayerNorm) and other.width == self.width

    def emit(self, b, h, delta, wanted_only: bool = False):
        if delta is not None and (delta.slices or delta.norm is not None or delta.dtype is not torch.float32 or wanted_only):
            raise native.KernelError("the layer norm adds a plain float32 [rows, width] contribution, for all rows only")
        prepared, b.prepared = b.prepared, None
        if (delta is None and not wanted_only and isinstance(prepared, dict) and prepared.get("layernorm") is self
                and prepared.get("stream") is h):
            return prepared["out"]          # the launch that ended the block before has applied this norm already
        count = b.want if wanted_only else h.rows
        out = b.temp(count, self.width, b.rt.dtype)
        bias = getattr(delta, "bias", None) if delta is not None else None
        b.launch("layernorm", "mlr_depth_norm", h.ptr, delta.ptr if delta is not None else None, delta.ld if delta is not None else 0,
                 None, 0, bias.data_ptr() if bias is not None else None, None, 0, 0, None, self.weight.data_ptr(), self.bias.data_ptr(),
                 self.eps, out.ptr, out.ld, out.is_bf16, b.meta("want_rows") if wanted_only else None, count, self.width,
                 int(delta is not None), b.stream, need="want" if wanted_only else None)
        return out


register_part("norm", "layernorm", LayerNorm)
