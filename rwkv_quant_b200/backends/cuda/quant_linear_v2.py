"""Per-row (rtn) quantized linear and the dense fallback.

``QuantLinearV2`` has the contract of the reference class of the same name
(backends/metal/quant_linear_v2.py:279-351): int8 codes with an fp16 scale per
output row, or biased split nibbles at <= 4 bits.  ``DenseLinear`` serves
tensors stored as bf16 (bits >= 16) and `asym` tensors met in linear position
(quant_model.py:245-262 falls back to a dense matmul there too).
"""
from __future__ import annotations

from .quant_linear_gw import _QuantLinearBase


class QuantLinearV2(_QuantLinearBase):
    kind = "rtn"


class DenseLinear(_QuantLinearBase):
    kind = None
