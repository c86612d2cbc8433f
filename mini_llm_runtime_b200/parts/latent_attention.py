"""Latent attention: keys and values of all heads are projections of one small vector per token, and only
that vector is cached.

    q = Wq x  [H, D];   c = rmsnorm(Wdkv x) * w  [R]  (the latent; cached);   k_h = Uk_h c,  v_h = Uv_h c
    o_h = softmax over j <= i of (q_h . k_hj) * scale, applied to v_hj;   result = o Wo^T        (no positions)

Because q_h . (Uk_h c) = (Uk_h^T q_h) . c  and  sum_j p_j Uv_h c_j = Uv_h sum_j p_j c_j,  the queries go through
Uk_h^T first (`mlr_head_project`), attention then runs on the cached latents themselves, as keys and as values
of one kv head shared by all query heads (`mlr_attention_masked` with shared_kv: a page holds one vector per
token), and its result goes through Uv_h (`mlr_head_project` again) before the output projection.  A mixer
without a latent of its own (`own_latent` False) has no Wdkv: its run reads the cache of the run the plan names
(`Run.kv_from`), with its own Uk, Uv and queries.

Parameters: hidden_size, num_heads, head_dim, value_dim, rank, scale, eps (of the latent's norm), own_latent.
Weights: "q" [H D, W], "dkv" [R, W], "dkv_norm" [R] (both only with a latent of its own), "uk" [H D, R],
"uv" [H Dv, R], "o" [W, H Dv].

Further parameters, all off unless named:
    rot_dim, position   a rotated part of P values beside the latent: a head of q is [D plain | P rotated] ("q" is [H (D + P), W]), the down
                projection has R + P rows of which the last P (not normed) are ONE rotated key part for all heads, and the score is
                (q_plain . k_plain + q_rot . k_rot) * scale.  The cached vector of a token is [latent | rotated key part]: a key of R + P
                values whose first R are the value.  `position` names a `rotary_frequencies` encoding (pairs side by side or halves)
                that turns the first `dims` of the P values (`mlr_latent_rot_cache`).
    window      a query sees itself and the window - 1 tokens before it (the cache gives older pages back)
    sink        "learned": exp(sink_h) in the softmax's denominator, weight "sink" [H]
    gate        "sigmoid_head": head h's result times sigmoid((Wg x)_h), weight "g" [H, W], stacked into the first product
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.base import ConfigError
from ..config.registry import register_part
from ..ops import functions as F
from ..ops import native
from ..ops.specs import GATES, MaskedAttentionSpec
from ..weights.loader import WeightSpec
from .base import CacheNeed, Mixer, RunContext, columns_of, pad_rows
from .masked_attention import emit_masked_attention


class LatentAttentionMixer(Mixer):
    def __init__(self, spec):
        super().__init__(spec)
        p = spec.params
        self.width = int(p["hidden_size"])
        self.heads, self.dim, self.vdim, self.rank = int(p["num_heads"]), int(p["head_dim"]), int(p["value_dim"]), int(p["rank"])
        self.scale, self.eps = float(p["scale"]), float(p["eps"])
        self.own_latent = bool(p.get("own_latent", True))
        self.rot = int(p.get("rot_dim") or 0)
        self.position_name = p.get("position")
        self.position = None
        self.window = p.get("window")
        self.sink, self.gate = p.get("sink"), p.get("gate")
        if not 1 <= self.rank <= 1024 or self.rank + self.rot > 1024:
            raise ConfigError(f"a latent of {self.rank} values (+ {self.rot} rotated) is outside what the attention kernel takes as a key and value (1 to 1024)")
        if self.sink not in (None, "learned") or self.gate not in (None, "sigmoid_head"):
            raise ConfigError(f"latent attention has sink None | 'learned' and gate None | 'sigmoid_head', not {self.sink!r} / {self.gate!r}")
        if (self.rot > 0) != (self.position_name is not None):
            raise ConfigError("a rotated part needs a position encoding, and the other way round")
        if self.window is not None and self.window <= 0:
            raise ConfigError("a window must be positive")
        self.desc: Optional[MaskedAttentionSpec] = None

    def attach_positions(self, positions) -> None:
        if self.position_name is not None:
            self.position = positions[self.position_name]
            if self.position.dims > self.rot:
                raise ConfigError(f"{self.position.dims} rotated values do not fit a rotated part of {self.rot}")

    def cache_need(self) -> CacheNeed:
        # One kv head whose keys are the latents (with their rotated part); value size 0: the values are the keys' first `rank`
        # values and take no room of their own.
        return CacheNeed(self.window, 1, self.rank + self.rot, 0)

    def weight_specs(self) -> List[WeightSpec]:
        w = self.spec.weights
        specs = [WeightSpec(w["q"], (self.heads * (self.dim + self.rot), self.width)), WeightSpec(w["uk"], (self.heads * self.dim, self.rank)),
                 WeightSpec(w["uv"], (self.heads * self.vdim, self.rank)), WeightSpec(w["o"], (self.width, self.heads * self.vdim))]
        if self.own_latent:
            specs += [WeightSpec(w["dkv"], (self.rank + self.rot, self.width)),
                      WeightSpec(w["dkv_norm"], (self.rank,), "vector", ("one_plus_normal", 0.01))]
        if self.sink:
            specs.append(WeightSpec(w["sink"], (self.heads,), "vector", ("normal", 0.5)))
        if self.gate:
            specs.append(WeightSpec(w["g"], (self.heads, self.width)))
        return specs

    def kernel_modules(self, dtype) -> List[str]:
        return ["latent", "attention_masked"] + (["experts"] if dtype is torch.bfloat16 else []) + F.product_modules(dtype)

    def _per_head(self, b, x, w, w_t, y, inputs: int, outputs: int, x_step: int, y_step: int) -> None:
        """y[m, h * y_step + :outputs] = x[m, h * x_step + :inputs] W_h: on the tensor cores (the batched product of `experts.cu`) for
        bfloat16 rows on 16-byte borders, else on the CUDA cores."""
        if b.rt.is_bf16 and native.module("experts").mlr_experts_tensor_cores(inputs, x.ld) and x.ptr % 16 == 0 and x_step % 8 == 0:
            b.launch("experts", "mlr_batched_product_bf16_strided", x.ptr, x.ld, x_step, w_t.data_ptr(), y.ptr, y.ld, y_step, x.rows, self.heads,
                     outputs, inputs, b.stream)
        else:
            b.launch("latent", "mlr_head_project_strided", x.ptr, x.ld, x_step, w.data_ptr(), y.ptr, y.ld, y_step, x.is_bf16, x.rows, self.heads,
                     inputs, outputs, b.stream)

    def bind(self, tensors: Dict[str, torch.Tensor], rt) -> None:
        w = self.spec.weights
        stacked = [rt.matrix(tensors[w["q"]])] + ([rt.matrix(tensors[w["dkv"]])] if self.own_latent else [])
        self._down_at = self.heads * (self.dim + self.rot)
        self._gate_at = self._down_at + (self.rank + self.rot if self.own_latent else 0)
        if self.gate:
            stacked.append(rt.matrix(tensors[w["g"]]))
        self.w_in = pad_rows(torch.cat(stacked, dim=0), 8)
        self.w_out = rt.matrix(tensors[w["o"]])
        # [heads, D, R] as stored; [heads, R, Dv] transposed, so that both per-head products read rows of their matrix.
        self.w_uk = rt.matrix(tensors[w["uk"]]).view(self.heads, self.dim, self.rank).contiguous()
        self.w_uv = rt.matrix(tensors[w["uv"]]).view(self.heads, self.vdim, self.rank).transpose(1, 2).contiguous()
        # The same two as [heads, outputs, inputs], the operand layout of the tensor-core product (bfloat16 only).
        self.w_uk_t = self.w_uk.transpose(1, 2).contiguous() if rt.is_bf16 else None
        self.w_uv_t = self.w_uv.transpose(1, 2).contiguous() if rt.is_bf16 else None
        self.latent_weight = rt.vector(tensors[w["dkv_norm"]]).float().contiguous() if self.own_latent else None
        self._sinks = rt.vector(tensors[w["sink"]]).to(device=rt.device, dtype=torch.float32).contiguous() if self.sink else None
        self._freq = self.position.frequencies() if self.position is not None else None
        # The rotation is done before attention (`mlr_latent_rot_cache`), so the attention kernels rotate nothing.
        self.desc = MaskedAttentionSpec(freq=None, sinks=self._sinks.data_ptr() if self.sink else None, slopes=None, heads=self.heads, kv_heads=1,
                                        dim=self.rank + self.rot, vdim=self.rank, rot_dims=0, window=self.window or 0, chunk=0,
                                        sink=int(bool(self.sink)), gate_kind=GATES[self.gate], shared_kv=1, keep_first=0, scale=self.scale,
                                        out_scale=1.0, softcap=0.0)

    def emit(self, b, x, run: RunContext):
        rt = b.rt
        if run.cache is None or run.cache.dtype is not rt.dtype:
            raise native.KernelError("latent attention: the cache must have the activations' precision")
        if run.write_cache != self.own_latent:
            raise native.KernelError("latent attention: a mixer with a latent of its own writes its cache, one without reads another's")
        proj = rt.linear(b, x, self.w_in, activation=True)
        rows = proj.rows
        key = self.rank + self.rot
        q = b.temp(rows, self.heads * key, rt.dtype)
        if self.rot:
            # The latent and the rotated key part into the cache; the queries' rotated parts behind the places of their projected plain parts.
            down = columns_of(proj, self._down_at, key) if self.own_latent else None
            b.launch("latent", "mlr_latent_rot_cache", down.ptr if down else None, down.ld if down else 0, proj.is_bf16,
                     self.latent_weight.data_ptr() if self.own_latent else None, self.eps, self.rank, self.rot, self.position.dims,
                     int(self.position.interleaved), self._freq.data_ptr() if self._freq.numel() else None, proj.ptr, proj.ld, self.dim,
                     self.dim + self.rot, self.heads, q.ptr, q.ld, self.rank, key, run.cache.data_ptr(), run.cache.shape[0],
                     b.meta("positions"), b.meta("segment_of_row"), b.table(run.group), b.table_stride(run.group), b.page_size,
                     int(self.own_latent), rows, b.status, b.stream)
        elif self.own_latent:
            down = columns_of(proj, self._down_at, self.rank)
            b.launch("latent", "mlr_latent_cache", down.ptr, down.ld, proj.is_bf16, self.latent_weight.data_ptr(), 1, self.eps, self.rank,
                     run.cache.data_ptr(), run.cache.shape[0], b.meta("positions"), b.meta("segment_of_row"), b.table(run.group),
                     b.table_stride(run.group), b.page_size, rows, b.status, b.stream)
        self._per_head(b, proj, self.w_uk, self.w_uk_t, q, self.dim, self.rank, self.dim + self.rot, key)
        mixed = b.temp(rows, self.heads * self.rank, rt.dtype)
        gate = columns_of(proj, self._gate_at, self.heads) if self.gate else None
        emit_masked_attention(b, self.desc, q, gate, mixed, run)
        act = b.temp(rows, self.heads * self.vdim, rt.dtype)
        self._per_head(b, mixed, self.w_uv, self.w_uv_t, act, self.rank, self.vdim, self.rank, self.vdim)
        return rt.linear(b, act, self.w_out, out_dtype=torch.float32)


register_part("mixer", "latent_attention", LatentAttentionMixer)
