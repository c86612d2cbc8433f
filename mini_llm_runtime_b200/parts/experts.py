"""Routed experts: many small SiLU-gated feed-forwards of which every token uses `top`, chosen by a router,
beside an optional shared one that every token uses.

    s = sigmoid(R x)  (float32);  choice = s + correction;  experts form `groups` equal groups of neighbours, a group's
    score is the sum of its two largest choices, and only experts of the `keep` best groups can be chosen; the `top`
    largest choices are taken;  weight_e = s_e / (sum of the chosen s + 1e-20)
    result = sum_e weight_e expert_e(x)  +  sigmoid(g . x) * shared(x)          expert(x) = Wd (silu(Wg x) .* (Wu x))

Launches: route (also counts every expert's tokens) -> arrange (rows in the order by expert, the products' row tiles)
-> the gate/up product with the gate in its epilogue, over rows gathered from the tokens -> the down product
-> combine (weights, the shared expert and its gate; a block whose norm stands behind the sub-layer takes the pieces and
combines them in that norm's launch: `Buf.pieces`).  The shared expert is the package's dense gated feed-forward.
The products over the experts' rows read their row ranges from the device, so a step needs no answer from the GPU.

Two choices differ between designs and are parameters.  `router`: "sigmoid_groups" is the rule above; "softmax_of_chosen"
takes z = R x + bias (float32), chooses the `top` largest z and weighs them by the softmax over the chosen z alone (weight
"router_bias" [E] instead of "correction"; no groups).  `activation`: "silu" is the expert above; "swish" is
Wd (g sigmoid(alpha g) (u + up_offset)) with g = min(Wg x, limit), u = clamp(Wu x, -limit, limit) where a limit is given
(the shared expert has a limit of its own, `shared_limit`).

Parameters: hidden_size, intermediate_size, experts, top, groups, keep, shared_intermediate_size (None: no shared expert),
router, activation, alpha, limit, up_offset, shared_limit.
Weights: "router" [E, W], "correction" or "router_bias" [E], "e<i>.gate", "e<i>.up" [I, W], "e<i>.down" [W, I], "shared.gate",
"shared.up" [Is, W], "shared.down" [W, Is], "shared.sg" [1, W].
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..config.base import ConfigError
from ..config.registry import register_part
from ..ops import functions as F
from ..ops import native
from ..weights.loader import WeightSpec
from .base import FeedForward


class RoutedExperts(FeedForward):
    def __init__(self, spec):
        super().__init__(spec)
        p = spec.params
        self.width, self.inter = int(p["hidden_size"]), int(p["intermediate_size"])
        self.experts, self.top = int(p["experts"]), int(p["top"])
        self.groups, self.keep = int(p.get("groups", 1)), int(p.get("keep", 1))
        self.shared_inter = int(p["shared_intermediate_size"]) if p.get("shared_intermediate_size") else 0
        self.router_kind = {"sigmoid_groups": 0, "softmax_of_chosen": 1}.get(p.get("router", "sigmoid_groups"))
        self.gate_kind = {"silu": 1, "swish": 2}.get(p.get("activation", "silu"))
        if self.router_kind is None or self.gate_kind is None:
            raise ConfigError(f"unknown router {p.get('router')!r} or expert activation {p.get('activation')!r}")
        self.alpha, self.up_offset = float(p.get("alpha", 1.0)), float(p.get("up_offset", 0.0))
        self.limit, self.shared_limit = float(p.get("limit") or 0.0), float(p.get("shared_limit") or 0.0)
        if self.gate_kind == 1 and (self.alpha != 1.0 or self.up_offset or self.limit or self.shared_limit):
            raise ConfigError("alpha, limit and up_offset belong to the expert activation 'swish'")
        if self.router_kind == 1 and self.groups != 1:
            raise ConfigError("a router that takes the softmax of the chosen logits has no groups")
        self._bias_role = "router_bias" if self.router_kind == 1 else "correction"
        if not (1 <= self.top <= min(32, self.experts) and self.experts <= 1024):
            raise ConfigError(f"{self.top} of {self.experts} experts is outside what the router kernel takes (32 of 1024)")
        if self.experts % self.groups or not 1 <= self.keep <= self.groups or self.top > self.keep * (self.experts // self.groups):
            raise ConfigError(f"{self.experts} experts in {self.groups} groups of which {self.keep} are kept cannot give {self.top}")

    def weight_specs(self) -> List[WeightSpec]:
        w = self.spec.weights
        specs = [WeightSpec(w["router"], (self.experts, self.width)), WeightSpec(w[self._bias_role], (self.experts,), "vector", ("normal", 0.1))]
        for i in range(self.experts):
            specs += [WeightSpec(w[f"e{i}.gate"], (self.inter, self.width)), WeightSpec(w[f"e{i}.up"], (self.inter, self.width)),
                      WeightSpec(w[f"e{i}.down"], (self.width, self.inter))]
        if self.shared_inter:
            specs += [WeightSpec(w["shared.gate"], (self.shared_inter, self.width)), WeightSpec(w["shared.up"], (self.shared_inter, self.width)),
                      WeightSpec(w["shared.down"], (self.width, self.shared_inter)), WeightSpec(w["shared.sg"], (1, self.width))]
        return specs

    def kernel_modules(self, dtype) -> List[str]:
        return ["experts", "elementwise"] + F.product_modules(dtype)

    def bind(self, tensors: Dict[str, torch.Tensor], rt) -> None:
        w = self.spec.weights
        f32 = lambda t: rt.matrix(t).to(torch.float32)
        rows = [f32(tensors[w["router"]])] + ([f32(tensors[w["shared.sg"]]).view(1, self.width)] if self.shared_inter else [])
        self.router = torch.cat(rows, dim=0).contiguous()          # float32: the router's products are 32-bit in both paths
        self.correction = rt.vector(tensors[w[self._bias_role]]).to(torch.float32).contiguous()
        stack = lambda role: torch.stack([rt.matrix(tensors[w[f"e{i}.{role}"]]) for i in range(self.experts)], dim=0).contiguous()
        self.w_gate, self.w_up, self.w_down = stack("gate"), stack("up"), stack("down")
        self.counts = torch.zeros(self.experts, dtype=torch.int32, device=rt.device)    # zero between steps (arrange leaves them so)
        if self.shared_inter and self.gate_kind == 2:
            # The clamped gate is a row-wise kernel behind the stacked product: all gate rows, then all up rows.
            self.shared_gate_up = torch.cat([rt.matrix(tensors[w["shared.gate"]]), rt.matrix(tensors[w["shared.up"]])], dim=0).contiguous()
            self.shared_down = rt.matrix(tensors[w["shared.down"]])
        elif self.shared_inter:
            self.shared_gate_up, inner = rt.stack_gate_up(tensors[w["shared.gate"]], tensors[w["shared.up"]])
            self.shared_down = rt.matrix(tensors[w["shared.down"]])
            if inner != self.shared_inter:
                padded = torch.zeros((self.width, inner), dtype=self.shared_down.dtype, device=self.shared_down.device)
                padded[:, :self.shared_inter] = self.shared_down
                self.shared_down = padded

    def emit(self, b, x):
        rt = b.rt
        x = rt.materialize(b, x)
        rows, top, E = x.rows, self.top, self.experts
        i32, f32 = torch.int32, torch.float32
        chosen, place, weights = b.temp(rows, top, i32), b.temp(rows, top, i32), b.temp(rows, top, f32)
        row_of_pair, pair_of_row = b.temp(rows, top, i32), b.temp(rows, top, i32)
        gate = b.temp(rows, 1, f32) if self.shared_inter else None
        first_row = b.temp(E + 1, 1, i32)
        max_tiles = b.bound(rows) * top // 32 + E
        tiles, n_tiles = b.temp(3 * max_tiles, 1, i32), b.temp(1, 1, i32)
        b.launch("experts", "mlr_experts_route", x.ptr, x.ld, x.is_bf16, self.router.data_ptr(), self.correction.data_ptr(), rows,
                 self.width, E, self.groups, self.keep, top, int(bool(self.shared_inter)), chosen.ptr, weights.ptr, place.ptr,
                 self.counts.data_ptr(), gate.ptr if gate else None, self.router_kind, b.stream)
        # Tiles of 64 rows for the tensor-core products once an expert gets that many rows on average; 32 otherwise (a decode
        # step's few rows per expert, the float32 path, rows that do not start on 16-byte borders).
        lib = native.module("experts")
        both = rt.is_bf16 and lib.mlr_experts_tensor_cores(self.width, x.ld) and lib.mlr_experts_tensor_cores(self.inter, self.inter)
        tile_rows = 64 if both and b.ge(rows, max(1, 64 * E // top)) else 32
        b.launch("experts", "mlr_experts_arrange", self.counts.data_ptr(), chosen.ptr, place.ptr, E, rows, top, tile_rows, first_row.ptr,
                 tiles.ptr, n_tiles.ptr, row_of_pair.ptr, pair_of_row.ptr, b.stream)
        act = b.temp(rows, top * self.inter, rt.dtype)             # [rows * top, inter], rows in the order by expert
        b.launch("experts", "mlr_experts_product", x.ptr, x.ld, x.is_bf16, pair_of_row.ptr, top, self.w_gate.data_ptr(),
                 self.w_up.data_ptr(), self.gate_kind, self.inter, self.width, act.ptr, self.inter, int(not rt.is_bf16), tiles.ptr, n_tiles.ptr,
                 rows, top, E, tile_rows, self.alpha, self.limit, self.up_offset, b.stream)
        y = b.temp(rows, top * self.width, f32)
        b.launch("experts", "mlr_experts_product", act.ptr, self.inter, x.is_bf16, None, 1, self.w_down.data_ptr(), None, 0, self.width,
                 self.inter, y.ptr, self.width, 1, tiles.ptr, n_tiles.ptr, rows, top, E, tile_rows, 0.0, 0.0, 0.0, b.stream)
        shared = None
        if self.shared_inter and self.gate_kind == 2:
            both = rt.linear(b, x, self.shared_gate_up, activation=True)
            hidden = b.temp(rows, self.shared_inter, rt.dtype)
            b.launch("elementwise", "mlr_gated_bias_shaped", both.ptr, both.ld, None, None, hidden.ptr, hidden.ld, hidden.is_bf16, rows,
                     self.shared_inter, 2, self.alpha, self.shared_limit, self.up_offset, b.stream)
            shared = rt.linear(b, hidden, self.shared_down, out_dtype=f32)
        elif self.shared_inter:
            hidden = rt.gated_linear(b, x, self.shared_gate_up)
            shared = rt.linear(b, hidden, self.shared_down, out_dtype=f32)
        if getattr(b, "accepts_pieces", False):
            # Whoever adds this result into the stream adds the pieces up itself (the norm behind the sub-layer): no launch here.
            from ..engine.builder import Buf
            return Buf(None, rows, self.width, f32, self.width, pieces=(y, row_of_pair, weights, top, shared, gate))
        out = b.temp(rows, self.width, f32)
        b.launch("experts", "mlr_experts_combine", y.ptr, self.width, row_of_pair.ptr, weights.ptr, top, shared.ptr if shared else None,
                 shared.ld if shared else 0, 0, gate.ptr if gate else None, out.ptr, out.ld, rows, self.width, b.stream)
        return out


register_part("feed_forward", "routed_experts", RoutedExperts)
