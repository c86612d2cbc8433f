"""Grouped-query attention over the paged cache with the choices that differ between designs as
parameters: which earlier keys a query sees (all, a window, its own chunk of positions), keys and
values of different sizes, rotation of only the first values of a head with or without linear
position scaling, a sink in the softmax, and a gate on the output.

    q, k, v, g = x [Wq; Wk; Wv; Wg]^T             one stacked product
    k <- rotate(k, position); cache <- k, v       `mlr_kv_rope_cache`
    o_h = sum_j p_j v_j,  p_j = exp(s_j) / (sink + sum exp(s_j)),  s_j = (rotate(q_h) . k_j) * scale
          over the keys j <= position that the window and the chunk allow;  sink = 1 (a key of score 0
          without a value) or 0                    `mlr_attention_masked`
    o <- o * sigmoid(g)  (or silu, or no gate), times a constant
    result = o Wo^T                               float32, not added into the stream

Parameters: hidden_size, num_heads, num_kv_heads, head_dim, value_dim, scale, window (None or n), chunk
(None or n), sink (bool), gate (None | "sigmoid" | "silu"), position (name of a `rotary_frequencies`
encoding of the plan, or None).  Weights: "q" [H D, W], "k" [G D, W], "v" [G Dv, W], "g" [H Dv, W] (with a
gate), "o" [W, H Dv].

Further parameters, all off unless named (with any of the first four the step's q, k and v go through
`mlr_qkv_prepare_cache` instead of `mlr_kv_rope_cache`):
    bias        q, k and v have biases: weights "q_bias" [H D], "k_bias" [G D], "v_bias" [G Dv]
    unit_qk     each head of q and of k is divided by its root mean square (eps `eps`, no weight)
    unit_v      each head of v likewise; the cache holds the divided values
    value_mix   "first": this layer's values (after the division) are kept for the step;  "later": v <- (1 - l) v + l v_first with
                v_first what the "first" layer kept for the same token and l the weight "vmix" (a single number); the mixed values are
                cached.  Both kinds name the weight (a checkpoint stores it for the first layer too, which does not read it).
    keep_first  with a window: the first keep_first positions of a sequence stay visible (the cache then keeps every page)
    softcap     score <- softcap * tanh(score / softcap)
    slopes      one number per head: score -= slope_h * (query position - key position)
    sink        "learned": the sink's score is a weight per head ("sink" [H]) instead of 0
    gate        "sigmoid_head": one gate value per head ("g" [H, W])
    qk_norm     a weighted RMS norm of q and k (eps `eps`) before rotation: "head": every head over its own root mean square,
                times one weight for all heads ("q_norm", "k_norm" [D]); "whole": the whole projection (all heads at once) over
                its root mean square, times a weight of its size ("q_norm" [H D], "k_norm" [G D])
    own_kv      False: the layer reads the keys and values that the run named by its `Run.kv_from` cached (as that cache holds
                them: normed, rotated) and has no "k", "v", "k_norm" and no biases but "q_bias"
    dense_kernels   True: where the layer is plain causal (or windowed) attention after its preparation (keys and values of one size
                up to 256; no chunk, sink, gate, cap, slopes, kept tokens, value mixing), `mlr_qkv_prepare_cache` also rotates the
                queries and writes the cache as the kernels of the `attention` part read it, and those run: tcgen05 flash attention
                for prompt portions, split-KV for decoded tokens (`ops/attention.py`).  Asked for where it does not fit, it is ignored.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..config.base import ConfigError
from ..config.registry import register_part
from ..ops import attention as A
from ..ops import functions as F
from ..ops import native
from ..ops.specs import GATES, QK_NORMS, MaskedAttentionSpec, address
from .base import CacheNeed, RunContext, SequenceCore, columns_of


class MaskedAttentionMixer(SequenceCore):
    FINER = 4       # how much finer than the step's plan the row kernel cuts long contexts (see emit_core)

    def __init__(self, spec):
        super().__init__(spec)
        p = spec.params
        self.width = int(p["hidden_size"])
        self.heads, self.kv_heads = int(p["num_heads"]), int(p["num_kv_heads"])
        self.dim, self.vdim = int(p["head_dim"]), int(p.get("value_dim") or p["head_dim"])
        self.scale = float(p["scale"])
        self.window, self.chunk = p.get("window"), p.get("chunk")
        self.sink = bool(p.get("sink", False))
        self.learned_sink = p.get("sink") == "learned"
        self.gate = p.get("gate")
        self.bias, self.unit_qk, self.unit_v = bool(p.get("bias", False)), bool(p.get("unit_qk", False)), bool(p.get("unit_v", False))
        self.eps = float(p.get("eps", 0.0))
        self.value_mix = p.get("value_mix")
        self.keep_first = int(p.get("keep_first") or 0)
        self.softcap = float(p.get("softcap") or 0.0)
        self.slopes = [float(v) for v in p["slopes"]] if p.get("slopes") is not None else None
        self.qk_norm = p.get("qk_norm")
        self.own_kv = bool(p.get("own_kv", True))
        if self.qk_norm not in QK_NORMS:
            raise ConfigError(f"unknown norm of q and k {self.qk_norm!r}")
        if self.qk_norm is not None and (self.unit_qk or self.eps <= 0):
            raise ConfigError("a weighted norm of q and k needs a positive eps and stands instead of the division of heads")
        if not self.own_kv and (self.unit_v or p.get("value_mix") is not None):
            raise ConfigError("a layer that reads another layer's keys and values changes no values")
        if self.value_mix not in (None, "first", "later"):
            raise ConfigError(f"unknown value mixing {self.value_mix!r}")
        if self.keep_first and (self.window is None or self.chunk is not None):
            raise ConfigError("kept first tokens go with a window and without chunks")
        if self.slopes is not None and len(self.slopes) != self.heads:
            raise ConfigError(f"{len(self.slopes)} distance slopes for {self.heads} heads")
        if (self.unit_qk or self.unit_v) and self.eps <= 0:
            raise ConfigError("dividing heads by their root mean square needs a positive eps")
        self.position_name = p.get("position")
        self.position = None
        self.dense = (bool(p.get("dense_kernels")) and self.dim == self.vdim and self.dim <= 256 and self.chunk is None and not self.sink
                      and self.gate is None and not self.softcap and self.slopes is None and not self.keep_first
                      and self.value_mix is None and not self.unit_v)
        if self.heads % self.kv_heads:
            raise ConfigError(f"{self.heads} query heads cannot share {self.kv_heads} kv heads")
        if self.gate not in GATES:
            raise ConfigError(f"unknown output gate {self.gate!r}")
        if not (1 <= self.dim <= 1024 and 1 <= self.vdim <= 1024):
            raise ConfigError(f"key size {self.dim} / value size {self.vdim} is outside what the masked attention kernel takes (1024 / 1024)")
        if (self.window is not None and self.window <= 0) or (self.chunk is not None and self.chunk <= 0):
            raise ConfigError("a window or chunk must be positive")
        self.desc: Optional[MaskedAttentionSpec] = None

    def attach_positions(self, positions) -> None:
        if self.position_name is not None:
            self.position = positions[self.position_name]
            if getattr(self.position, "interleaved", False):
                raise ConfigError("the masked attention kernels pair value i with value i + dims / 2; an interleaved rotation is not built there")
            if self.position.dims > self.dim:
                raise ConfigError(f"{self.position.dims} rotated values do not fit a head of {self.dim}")

    def cache_need(self) -> CacheNeed:
        # Kept first tokens lie before the window: such a cache gives no pages back (the window is then a mask only).
        if self.dense:
            return CacheNeed(self.window, self.kv_heads, self.dim)      # the pool of the plain attention kernels
        return CacheNeed(None if self.keep_first else self.window, self.kv_heads, self.dim, self.vdim)

    def in_roles(self) -> List[Tuple[str, int]]:
        roles = [("q", self.heads * self.dim)]
        if self.own_kv:
            roles += [("k", self.kv_heads * self.dim), ("v", self.kv_heads * self.vdim)]
        if self.gate:
            roles.append(("g", self.heads if self.gate == "sigmoid_head" else self.heads * self.vdim))
        return roles

    def extra_weight_specs(self):
        from ..weights.loader import WeightSpec
        w, specs = self.spec.weights, []
        if self.bias:
            specs.append(WeightSpec(w["q_bias"], (self.heads * self.dim,), "vector", ("normal", 0.02)))
            if self.own_kv:
                specs += [WeightSpec(w["k_bias"], (self.kv_heads * self.dim,), "vector", ("normal", 0.02)),
                          WeightSpec(w["v_bias"], (self.kv_heads * self.vdim,), "vector", ("normal", 0.02))]
        if self.qk_norm is not None:
            whole = self.qk_norm == "whole"
            specs.append(WeightSpec(w["q_norm"], (self.heads * self.dim if whole else self.dim,), "vector", ("one_plus_normal", 0.05)))
            if self.own_kv:
                specs.append(WeightSpec(w["k_norm"], (self.kv_heads * self.dim if whole else self.dim,), "vector", ("one_plus_normal", 0.05)))
        if self.value_mix is not None:
            specs.append(WeightSpec(w["vmix"], (), "vector", ("normal", 0.3)))
        if self.learned_sink:
            specs.append(WeightSpec(w["sink"], (self.heads,), "vector", ("normal", 0.5)))
        return specs

    @property
    def _prepares(self) -> bool:
        return self.bias or self.unit_qk or self.unit_v or self.value_mix is not None or self.qk_norm is not None or self.dense

    def core_width(self) -> int:
        return self.heads * self.vdim

    def kernel_modules(self, dtype) -> List[str]:
        return ["attention_masked"] + (A.modules_for(dtype, self.dim) if self.dense else []) + F.product_modules(dtype)

    def bind_core(self, tensors, rt, out_scale: float) -> None:
        freq = self.position.frequencies() if self.position is not None else None
        self._freq = freq
        w = self.spec.weights
        f32 = lambda t: t.to(device=rt.device, dtype=torch.float32).contiguous()
        self._sinks = f32(rt.vector(tensors[w["sink"]])) if self.learned_sink else None
        self._slopes = torch.tensor(self.slopes, dtype=torch.float32, device=rt.device) if self.slopes is not None else None
        self._biases = [f32(rt.vector(tensors[w[r]])) if self.bias and (self.own_kv or r == "q_bias") else None
                        for r in ("q_bias", "k_bias", "v_bias")]
        self._q_weight = f32(rt.vector(tensors[w["q_norm"]])) if self.qk_norm is not None else None
        self._k_weight = f32(rt.vector(tensors[w["k_norm"]])) if self.qk_norm is not None and self.own_kv else None
        self._lambda = float(tensors[w["vmix"]].float().item()) if self.value_mix == "later" else 0.0
        self.desc = MaskedAttentionSpec(
            freq=freq.data_ptr() if freq is not None and freq.numel() else None,
            sinks=self._sinks.data_ptr() if self._sinks is not None else None,
            slopes=self._slopes.data_ptr() if self._slopes is not None else None,
            q_weight=self._q_weight.data_ptr() if self._q_weight is not None else None,
            k_weight=self._k_weight.data_ptr() if self._k_weight is not None else None, qk_norm=QK_NORMS[self.qk_norm],
            heads=self.heads, kv_heads=self.kv_heads, dim=self.dim,
            vdim=self.vdim, rot_dims=self.position.dims if self.position is not None else 0, window=self.window or 0,
            chunk=self.chunk or 0, sink=int(self.sink), gate_kind=GATES[self.gate], keep_first=self.keep_first, scale=self.scale,
            out_scale=float(out_scale), softcap=self.softcap, dense_cache=int(self.dense))
        if self.dense and out_scale != 1.0:
            raise ConfigError("the plain attention kernels scale no result; this mixer stands alone")

    def emit_core(self, b, proj, act, run: RunContext) -> None:
        if run.cache is None or run.cache.dtype is not proj.dtype:
            raise native.KernelError("masked attention: the cache must have the activations' precision")
        at = self.in_columns()
        if self.own_kv != bool(run.write_cache):
            raise native.KernelError("masked attention: a layer writes the cache exactly when it makes keys and values of its own")
        k = columns_of(proj, at["k"], self.kv_heads * self.dim) if self.own_kv else None
        v = columns_of(proj, at["v"], self.kv_heads * self.vdim) if self.own_kv else None
        gate = columns_of(proj, at["g"], self.heads if self.gate == "sigmoid_head" else self.heads * self.vdim) if self.gate else None
        table, stride = b.table(run.group), b.table_stride(run.group)
        if self._prepares and not self.own_kv:
            # Queries only: biases and the norm in place; the attention kernels rotate them as they load them.
            b.launch("attention_masked", "mlr_qkv_prepare_cache", address(self.desc), proj.ptr, proj.ld, None, 0, None, 0, proj.is_bf16,
                     self._biases[0].data_ptr() if self._biases[0] is not None else None, None, None, int(self.unit_qk), 0, self.eps,
                     None, 0, 0, 0.0, None, 0, b.meta("positions"), b.meta("segment_of_row"), None, 0, b.page_size, proj.rows,
                     b.status, b.stream)
        elif self._prepares:
            first = None
            if self.value_mix is not None:
                first = b.kept(("value_mix", self.kv_heads, self.vdim), proj.rows, self.kv_heads * self.vdim, torch.float32)
            ptr = lambda t: t.data_ptr() if t is not None else None
            b.launch("attention_masked", "mlr_qkv_prepare_cache", address(self.desc), proj.ptr, proj.ld, k.ptr, k.ld, v.ptr, v.ld, proj.is_bf16,
                     ptr(self._biases[0]), ptr(self._biases[1]), ptr(self._biases[2]), int(self.unit_qk), int(self.unit_v), self.eps,
                     first.ptr if first is not None else None, first.ld if first is not None else 0,
                     {None: 0, "first": 1, "later": 2}[self.value_mix], self._lambda, run.cache.data_ptr(), run.cache.shape[0],
                     b.meta("positions"), b.meta("segment_of_row"), table, stride, b.page_size, proj.rows, b.status, b.stream)
        elif run.write_cache:
            b.launch("attention_masked", "mlr_kv_rope_cache", address(self.desc), k.ptr, k.ld, v.ptr, v.ld, proj.is_bf16,
                     run.cache.data_ptr(), run.cache.shape[0], b.meta("positions"), b.meta("segment_of_row"), table, stride,
                     b.page_size, proj.rows, b.status, b.stream)
        if self.dense:
            if act.ld != self.heads * self.vdim:
                raise native.KernelError("masked attention: the plain attention kernels write a result of its own width")
            A.paged_attention(b, proj, act, run.cache, run.group, self.heads, self.kv_heads, self.dim, self.window or 0, self.scale)
            return
        emit_masked_attention(b, self.desc, proj, gate, act, run, self.FINER)


def emit_masked_attention(b, desc: MaskedAttentionSpec, q, gate, act, run: RunContext, finer: int = 4) -> None:
    """The attention launches of a step for the description `desc`: queries from `q` (head h at column h * dim), the gate's
    columns or None, the result into `act`, keys and values from the run's cache."""
    heads, kv_heads, dim, vdim = desc.heads, desc.kv_heads, desc.dim, desc.vdim
    proj = q
    table, stride = b.table(run.group), b.table_stride(run.group)
    args = (address(desc), proj.ptr, proj.ld, gate.ptr if gate else None, gate.ld if gate else 0, act.ptr, act.ld)
    where = (run.cache.data_ptr(), run.cache.shape[0])
    tiled = (proj.dtype is torch.bfloat16 and native.module("attention_masked").mlr_attention_masked_tiles_fit(dim, vdim)
             and act.ld % 2 == 0 and act.ptr % 4 == 0)
    if not tiled:
        # One block per (row, head): the float32 path, and sizes the tiled kernel does not take.
        b.launch("attention_masked", "mlr_attention_masked", *args, proj.is_bf16, *where, b.meta("positions"),
                 b.meta("segment_of_row"), table, stride, b.page_size, proj.rows, None, 0, None, 0, 1, 1, None, b.status, b.stream)
        return
    # The step's launch plan (made by the native executor from the step's segments, shared by all layers):
    # segments of few rows (a decoded token, a short portion) go to the row kernel, prompt portions in tiles of 64
    # rows to the tensor-core kernel.
    # The row kernel cuts long contexts into key ranges that run as blocks of their own (the plan's split of the keys and
    # its scratch for the ranges' partial results: 16 rows x kv heads x splits x (head size + 2) floats per segment).
    # The planner sizes the scratch by the head size it is told: FINER times the room of a range's (value size + 2)
    # floats lets the kernel cut every planned range into FINER (its blocks wait for memory most of the time, and
    # more of them in flight is what makes a long context fast; the planner's own split is tuned for a kernel that
    # copies keys in bulk).
    # Where more than 16 query heads share a kv head (latent attention: all of them), the few-row kernel takes them 16 at a
    # time in blocks of their own: the planner is told of that many more kv heads, each shared by 16 (a few-row segment is then
    # ONE row, a decoded token), and sizes the ranges' scratch for them.
    group = heads // kv_heads
    chunks = (group + 15) // 16
    plan = b.plan((min(group, 16), kv_heads * chunks, 0, 0, finer * (max(dim, vdim) + 2), 1))
    info = b.meta("segment_info")
    split = (plan.chunk, plan.max_splits, finer, plan.scratch)
    b.launch("attention_masked", "mlr_attention_masked", *args, 1, *where, b.meta("positions"), b.meta("segment_of_row"), table,
             stride, b.page_size, 0, plan.items, plan.n_items, info, *split, b.status, b.stream, need=plan.n_items)
    b.launch("attention_masked", "mlr_attention_masked_tiles", *args, *where, plan.tiles, plan.n_tiles, info, table, stride,
             b.page_size, b.status, b.stream, need=plan.n_tiles)


register_part("mixer", "masked_attention", MaskedAttentionMixer)
