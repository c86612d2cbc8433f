"""Descriptions that some kernels read from host memory: the constants of a mixer, gathered once
when the part is bound, so that a launch names the description and the step's buffers only.

Each class mirrors a struct of the same name in the kernel module (`csrc/kernels/attention_masked.cu`,
`csrc/kernels/recurrence.cu`): pointers first, then 32-bit integers, then floats.  The part keeps the
object (and the device tensors it points to) alive for as long as programs name its address.
"""
from __future__ import annotations

import ctypes

GATES = {None: 0, "sigmoid": 1, "silu": 2, "sigmoid_head": 3}      # "sigmoid_head": one gate value per head, not per value
QK_NORMS = {None: 0, "head": 1, "whole": 2}                        # a weighted RMS norm of q and k: per head, or over all heads at once


class MaskedAttentionSpec(ctypes.Structure):
    _fields_ = [("freq", ctypes.c_void_p), ("sinks", ctypes.c_void_p), ("slopes", ctypes.c_void_p), ("q_weight", ctypes.c_void_p),
                ("k_weight", ctypes.c_void_p),
                ("heads", ctypes.c_int32), ("kv_heads", ctypes.c_int32), ("dim", ctypes.c_int32), ("vdim", ctypes.c_int32),
                ("rot_dims", ctypes.c_int32), ("window", ctypes.c_int32), ("chunk", ctypes.c_int32), ("sink", ctypes.c_int32),
                ("gate_kind", ctypes.c_int32), ("shared_kv", ctypes.c_int32), ("keep_first", ctypes.c_int32), ("qk_norm", ctypes.c_int32),
                ("dense_cache", ctypes.c_int32),
                ("scale", ctypes.c_float), ("out_scale", ctypes.c_float), ("softcap", ctypes.c_float)]


class RecurrenceSpec(ctypes.Structure):
    PREP = {None: 0, "rotate": 1, "unit": 2}
    RULE = {"decay": 0, "delta": 1}
    IN_ACT = {None: 0, "silu": 1}
    _fields_ = [("freq", ctypes.c_void_p), ("decay", ctypes.c_void_p), ("a_log", ctypes.c_void_p), ("dt_bias", ctypes.c_void_p),
                ("out_weight", ctypes.c_void_p),
                ("heads", ctypes.c_int32), ("qk_heads", ctypes.c_int32), ("dim", ctypes.c_int32), ("vdim", ctypes.c_int32),
                ("prep", ctypes.c_int32), ("rot_dims", ctypes.c_int32), ("rule", ctypes.c_int32), ("gate_kind", ctypes.c_int32),
                ("col_q", ctypes.c_int32), ("col_k", ctypes.c_int32), ("col_v", ctypes.c_int32), ("col_a", ctypes.c_int32),
                ("col_b", ctypes.c_int32), ("col_gate", ctypes.c_int32), ("in_act", ctypes.c_int32), ("norm_all", ctypes.c_int32),
                ("q_mult", ctypes.c_float), ("k_mult", ctypes.c_float), ("unit_eps", ctypes.c_float), ("eps", ctypes.c_float),
                ("out_scale", ctypes.c_float)]


def address(spec: ctypes.Structure) -> int:
    return ctypes.addressof(spec)
