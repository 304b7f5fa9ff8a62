"""sb6 (block 32, super-block 8; int4 / int5 / int6) quantized linear.

Same contract as the reference's ``GwQuantLinear`` / ``GwQuantLinearFused``
(backends/metal/quant_linear_gw.py:747-1020): built from a QuantizedTensor,
``__call__(x[..., IN]) -> [..., OUT]`` fp32 for any leading shape.  The weights
stay in the file layout on the device; no K3-style interleave is made.
"""
from __future__ import annotations

import torch

from . import ops
from ... import _lib

# N at or above which the dequant + tensor-core GEMM path takes over from the
# weight-streaming GEMV (the reference's crossover constant, quant_linear_gw.py:153)
GEMM_MIN_BATCH_NB = 128
# N up to which every column gets its own exact single-vector launch (results independent of
# the batch they were computed in); between the two the weights-once small-batch kernel runs
GEMV_MAX_BATCH = 2


class _QuantLinearBase:
    kind = None

    def __init__(self, qt, device="cuda"):
        self.dq = qt if isinstance(qt, ops.DeviceQT) else ops.DeviceQT(qt, device)
        if self.kind is not None and self.dq.kind != self.kind:
            raise AssertionError(f"{type(self).__name__} needs a {self.kind!r} tensor, "
                                 f"got {self.dq.kind!r}")
        self.out_features, self.in_features = self.dq.rows, self.dq.cols
        self.bits = self.dq.bits

    def __call__(self, x: torch.Tensor, epilogue: int = _lib.EPI_NONE, resid=None) -> torch.Tensor:
        x2, lead = ops.as_rows(x, self.in_features)
        if resid is not None:
            resid = resid.reshape(-1, self.out_features).contiguous()
        if x2.shape[0] >= GEMM_MIN_BATCH_NB and self.dq.kind in ("sb6", "sym"):
            # the reference's crossover (quant_linear_gw.py:846-849, quant_linear_sym.py:481-484):
            # its dequant + fp16 matmul; here the dequantisation is fused into the tensor-core GEMM
            y = ops.gemm(self.dq, x2.float(), epilogue, resid)
        elif x2.shape[0] > GEMV_MAX_BATCH and ops.has_batch_layout(self.dq):
            # the reference decodes each weight once per chunk of 4 columns (_gemv_nb,
            # quant_linear_gw.py:850-905); here once per 64 columns
            y = ops.gemv_batch(self.dq, x2, epilogue, resid)
        else:
            y = self.dq.gemv(x2, epilogue, resid)
        return y.reshape(*lead, self.out_features)

    def _dequant_w(self, dtype=torch.float32) -> torch.Tensor:
        """Dense [OUT, IN]; the fp32 result equals the numpy codec bit for bit."""
        return self.dq.dequant(dtype, False)

    def weight_nbytes(self) -> int:
        return self.dq.nbytes()


class GwQuantLinear(_QuantLinearBase):
    kind = "sb6"

    @property
    def has_qh(self) -> bool:
        return self.bits >= 5


class _FusedBase:
    """K same-shape matrices with K different inputs in one launch; results are
    bit-identical to K separate single-vector calls."""

    def __init__(self, lins):
        shapes = {(l.in_features, l.out_features, l.bits, l.dq.kind) for l in lins}
        if len(shapes) != 1:
            raise AssertionError(f"fused projections need one shape and layout, got {shapes}")
        self.lins = list(lins)
        self.in_features = lins[0].in_features
        self.out_per = lins[0].out_features

    def __call__(self, xstack: torch.Tensor) -> torch.Tensor:
        k = len(self.lins)
        x2 = xstack.reshape(k, self.in_features)
        if x2.dtype not in _lib.DTYPE_CODE:
            x2 = x2.float()
        return ops.gemv_fused([l.dq for l in self.lins], x2.contiguous())


class GwQuantLinearFused(_FusedBase):
    pass
