"""sym (Q6_K-style: block 16, super-block 16; 6 or 8 bit) quantized linear.

Same contract as the reference's ``SymQuantLinear`` / ``SymQuantLinearFused``
(backends/metal/quant_linear_sym.py:372-574), including the numpy-only
``from_buffers`` constructor (:392-405) and ``_dequant_w`` whose fp32 result
equals ``codec.dequant_sym`` bit for bit (:433-452).
"""
from __future__ import annotations

import numpy as np
import torch

from .quant_linear_gw import _FusedBase, _QuantLinearBase
from ...formats.container import QuantizedTensor


class SymQuantLinear(_QuantLinearBase):
    kind = "sym"

    def __init__(self, qt, device="cuda"):
        super().__init__(qt, device)
        assert self.dq.gs == 16 and self.dq.sb == 16, "sym layout is block 16 / super-block 16"

    @classmethod
    def from_buffers(cls, *, shape, bits, qs, d, codes=None, codes_packed=None,
                     qh=None, qh2=None, device="cuda"):
        t = lambda a: None if a is None else torch.from_numpy(np.ascontiguousarray(a))
        qt = QuantizedTensor(key="", group="", bits=int(bits), shape=tuple(shape), gw_mode="sym",
                             gw_gs=16, gw_sb=16, codes=t(codes), codes_packed=t(codes_packed),
                             gw_qh=t(qh), gw_qh2=t(qh2), gw_qs=t(qs), gw_d=t(d))
        return cls(qt, device)

    def can_fuse_with(self, other) -> bool:
        return (isinstance(other, SymQuantLinear) and other.bits == self.bits
                and other.in_features == self.in_features
                and other.out_features == self.out_features)


class SymQuantLinearFused(_FusedBase):
    pass
