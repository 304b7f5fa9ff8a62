"""CUDA (sm_100a) backend with the reference backend's operator surface."""
from .ops import DeviceQT  # noqa: F401
from .quant_linear_gw import GwQuantLinear, GwQuantLinearFused  # noqa: F401
from .quant_linear_sym import SymQuantLinear, SymQuantLinearFused  # noqa: F401
from .quant_linear_v2 import DenseLinear, QuantLinearV2  # noqa: F401
from .fused_tail import can_fuse_tail, wkv_tail  # noqa: F401
from .wkv7 import wkv7_infer, wkv7_train  # noqa: F401
from .quant_model import Decoder, QuantRWKV7  # noqa: F401


def linear_for(qt, device="cuda"):
    """Dispatch on the tensor's layout (the reference's ``_linear``,
    backends/metal/quant_model.py:245-262)."""
    mode = getattr(qt, "gw_mode", "") or ""
    if qt.bits < 16:
        if mode == "sb6":
            return GwQuantLinear(qt, device)
        if mode == "sym":
            return SymQuantLinear(qt, device)
        if mode == "asym":
            return DenseLinear(qt, device)
        return QuantLinearV2(qt, device)
    return DenseLinear(qt, device)
