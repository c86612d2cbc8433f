"""Pre-norm residual block: `h += mixer(norm(h))`, then `h += feed_forward(norm(h))`
(src/minillm/runtime.cpp:245-337; src/minillm/cuda/layer.cpp:42-70).

Each residual add is folded into a neighbouring kernel: either the sub-layer's last
product adds its result into `h` itself (it finds `h` in `step.residual` and returns
None), or its output is handed on as `pending` and added to `h` by the next norm's
kernel.  Either way the residual stream is read and written once per sub-layer.  Norm
slots: "pre_mixer", "pre_feed_forward".
"""
from __future__ import annotations

from typing import List

import torch

from ..config.registry import register_part
from ..ops import native
from ..weights.loader import WeightSpec
from .base import Block


class PreNormBlock(Block):
    def forward(self, h, pending, step, run):
        step.residual = h
        x = self.norms["pre_mixer"].forward(h, pending, step)
        mixed = self.mixer.forward(x, step, run)
        x = self.norms["pre_feed_forward"].forward(h, mixed, step)
        return self.feed_forward.forward(x, step)

    def first_norm(self):
        return self.norms["pre_mixer"]

    def emit(self, b, h, pending, run):
        b.residual = h
        after = b.norm_after_block
        x = self.norms["pre_mixer"].emit(b, h, pending)
        # Whoever adds into the stream is told which norm reads it next (a few-row product can leave it half done).
        b.norm_ahead = self.norms["pre_feed_forward"].foldable()
        mixed = self.mixer.emit(b, x, run)
        x = self.norms["pre_feed_forward"].emit(b, h, mixed)
        b.norm_ahead = after
        out = self.feed_forward.emit(b, x)
        b.norm_ahead = None
        return out


register_part("block", "pre_norm", PreNormBlock)


class SandwichBlock(Block):
    """Norms on both sides of each sub-layer: `h += post(mixer(pre(h)))`, then
    `h += post(feed_forward(pre(h)))`; a layer without a feed-forward has only the first.

    The sub-layers' results are contributions that a norm stands behind, so they are not added into the
    stream by their last product; the norm behind a sub-layer adds it and applies the norm before the
    next sub-layer in the same launch.  Norm slots: "pre_mixer", "post_mixer", "pre_feed_forward",
    "post_feed_forward"; the norms must offer `emit_residual` (the grouped RMS norm does)."""

    def forward(self, h, pending, step, run):
        from ..engine.builder import EagerBuilder
        b = EagerBuilder(step)
        out = self.emit(b, b.wrap(h), b.wrap(pending), run)
        return out.tensor if out is not None else None

    def first_norm(self):
        return self.norms["pre_mixer"]

    def emit(self, b, h, pending, run):
        b.residual = None            # nothing of this block is added into the stream by a product
        b.norm_ahead = None
        x = self.norms["pre_mixer"].emit(b, h, pending)
        mixed = self.mixer.emit(b, x, run)
        # The norm behind the block's last sub-layer also applies the first norm of the block that follows (the model
        # names it in `norm_after_block`), whose `emit` then finds the result in `prepared` and launches nothing.
        after = b.norm_after_block
        following = after[1] if after is not None and after[0] == "group_rms" else None
        last = "post_mixer" if self.feed_forward is None else "post_feed_forward"
        if following is not None and not self.norms[last].same_shape(following):
            following = None
        if self.feed_forward is None:
            ahead = self.norms["post_mixer"].emit_residual(b, h, mixed, then=following)
        else:
            x = self.norms["post_mixer"].emit_residual(b, h, mixed, then=self.norms["pre_feed_forward"])
            # A feed-forward of routed experts may leave its result in pieces for the norm behind it to add up.
            b.accepts_pieces = bool(getattr(self.norms["post_feed_forward"], "takes_pieces", False))
            try:
                out = self.feed_forward.emit(b, x)
            finally:
                b.accepts_pieces = False
            ahead = self.norms["post_feed_forward"].emit_residual(b, h, out, then=following)
        b.prepared = {"group_rms": following, "stream": h, "out": ahead} if following is not None else None
        return None


register_part("block", "sandwich", SandwichBlock)


class ParallelResidualBlock(Block):
    """Both sub-layers read ONE norm of the stream and their results are added together:
    `h += mixer(norm(h)) + feed_forward(norm(h))` (a layer without a feed-forward adds the mixer's result only).

    With `states` the block also averages over depth: the stream's earlier states of the step are kept (`X_0` what the
    embedding made, `X_j` what block j - 1 computed), this block's result `h` is stored as `X_states`, and what goes on to
    the next block is `sum_j depth[j] * X_j` over j = 0..states.  `states` is how many states exist before this block's
    (its index in the model plus one) and `total_states` how many the model keeps in all; the block with `states` = 1
    stores the embedding's output itself.

    The add of both results, the average and the norm that reads the stream next (this kind of block's, or a model's last
    layer norm is not: that one norms wanted rows only) are one launch, `mlr_depth_norm`; the block leaves the next block's
    input on the builder (`prepared`) like the other blocks that do this.  Sub-layers hand over plain float32 results; no
    product adds into the stream.  Parameters: width, states (None: no averaging), total_states.  Weights: "depth"
    [states + 1] with averaging.  Norm slot: "pre" (a `layernorm`)."""

    def __init__(self, spec, mixer, feed_forward, norms):
        super().__init__(spec, mixer, feed_forward, norms)
        self.width = int(spec.params["width"])
        states = spec.params.get("states")
        self.states = int(states) if states is not None else None
        self.total_states = int(spec.params.get("total_states") or 0)
        if self.states is not None and not 1 <= self.states < self.total_states:
            raise ValueError(f"a block after {self.states} states in a model that keeps {self.total_states}")
        self.depth = None
        self._one = None

    def weight_specs(self) -> List[WeightSpec]:
        if self.states is None:
            return []
        return [WeightSpec(self.spec.weights["depth"], (self.states + 1,), "vector", ("normal", 0.4))]

    def kernel_modules(self, dtype) -> List[str]:
        return ["layernorm"]

    def bind(self, tensors, rt) -> None:
        if self.states is not None:
            self.depth = rt.vector(tensors[self.spec.weights["depth"]]).to(device=rt.device, dtype=torch.float32).contiguous()
            self._one = torch.ones(1, dtype=torch.float32, device=rt.device)

    def first_norm(self):
        return self.norms["pre"]

    def forward(self, h, pending, step, run):
        from ..engine.builder import EagerBuilder
        b = EagerBuilder(step)
        self.emit(b, b.wrap(h), b.wrap(pending), run)
        return None

    def _history(self, b, h):
        if self.states is None:
            return None
        return b.kept("depth_states", h.rows, self.width, torch.float32, slices=self.total_states)

    def emit(self, b, h, pending, run):
        if pending is not None:
            raise native.KernelError("a parallel block takes no pending contribution: the block before it must add its own")
        if h.width != self.width or h.ld != self.width:
            raise native.KernelError("a parallel block works on a plain [rows, width] stream")
        b.residual = None            # nothing of this block is added into the stream by a product
        b.norm_ahead = None
        norm = self.norms["pre"]
        history = self._history(b, h)
        prepared = b.prepared
        if isinstance(prepared, dict) and prepared.get("layernorm") is norm and prepared.get("stream") is h:
            b.prepared = None
            x = prepared["out"]      # the launch that ended the block before has applied this block's norm already
        elif self.states == 1:
            # The first of the averaging blocks: its norm's launch also stores the stream as state 0.
            b.prepared = None
            x = b.temp(h.rows, self.width, b.rt.dtype)
            b.launch("layernorm", "mlr_depth_norm", h.ptr, None, 0, None, 0, None, history.ptr, history.slice_stride, 0, self._one.data_ptr(),
                     norm.weight.data_ptr(), norm.bias.data_ptr(), norm.eps, x.ptr, x.ld, x.is_bf16, None, h.rows, self.width, 0, b.stream)
        else:
            x = norm.emit(b, h, None)
        after = b.norm_after_block
        mixed = self.mixer.emit(b, x, run)
        out = self.feed_forward.emit(b, x) if self.feed_forward is not None else None
        for y in (mixed, out):
            if y is not None and (y.slices or y.norm is not None or y.dtype is not torch.float32):
                raise native.KernelError("a sub-layer of a parallel block hands over a plain float32 [rows, width] result")
        biases = [y.bias for y in (mixed, out) if y is not None and y.bias is not None]
        if len(biases) > 1:
            raise native.KernelError("a parallel block adds one bias vector with its sub-layers' results")
        following = after[1] if after is not None and after[0] == "layernorm" and after[1].width == self.width else None
        ahead = b.temp(h.rows, self.width, b.rt.dtype) if following is not None else None
        b.launch("layernorm", "mlr_depth_norm", h.ptr, mixed.ptr if mixed is not None else None, mixed.ld if mixed is not None else 0,
                 out.ptr if out is not None else None, out.ld if out is not None else 0, biases[0].data_ptr() if biases else None,
                 history.ptr if history is not None else None, history.slice_stride if history is not None else 0,
                 self.states or 0, self.depth.data_ptr() if history is not None else None,
                 following.weight.data_ptr() if following is not None else None, following.bias.data_ptr() if following is not None else None,
                 float(following.eps) if following is not None else 0.0, ahead.ptr if ahead is not None else None,
                 ahead.ld if ahead is not None else 0, int(b.rt.is_bf16), None, h.rows, self.width, 1, b.stream)
        b.prepared = {"layernorm": following, "stream": h, "out": ahead} if following is not None else None
        return None


register_part("block", "parallel_residual", ParallelResidualBlock)
