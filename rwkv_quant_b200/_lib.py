"""ctypes binding of ``librwkvq_b200.so`` (declared in ``include/rwkvq_b200.h``).

There is no CPU or PyTorch fallback: if the library is missing or the device is
not a B200-class GPU, loading fails with an error that says how to build it.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "librwkvq_b200.so")

F32, F16, BF16 = 0, 1, 2
KIND = {"dense": 0, "sb6": 1, "sym": 2, "asym": 3, "rtn": 4}
EPI_NONE, EPI_RELU2, EPI_ADD = 0, 1, 2
E_SHAPE, E_ALIGN, E_DTYPE, E_ARCH, E_LAUNCH, E_TIMEOUT, E_NULL, E_LIMIT, E_FORMAT = -1, -2, -3, -4, -5, -6, -7, -8, -9
DTYPE_CODE = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}


class QTensorStruct(C.Structure):
    """``rwkvq_qtensor`` of the header."""
    _fields_ = [("kind", C.c_int32), ("bits", C.c_int32), ("rows", C.c_int32),
                ("cols", C.c_int32), ("gs", C.c_int32), ("sb", C.c_int32),
                ("codes", C.c_void_p), ("qh", C.c_void_p), ("qh2", C.c_void_p),
                ("qsqm", C.c_void_p), ("qs", C.c_void_p), ("d", C.c_void_p),
                ("dm", C.c_void_p), ("scale", C.c_void_p), ("mn", C.c_void_p),
                ("dev_meta", C.c_void_p), ("dev_planes", C.c_void_p)]


_FP = C.c_void_p


class LayerStruct(C.Structure):
    """``rwkvq_layer`` of the header."""
    _fields_ = ([(n, _FP) for n in ("ln1_w", "ln1_b", "ln2_w", "ln2_b", "x_mix", "w0", "a0", "v0",
                                    "k_k", "k_a", "r_k", "lnx_w", "lnx_b", "ffn_x_k")]
                + [(n, QTensorStruct) for n in ("w1", "w2", "a1", "a2", "v1", "v2", "g1", "g2",
                                                "Wr", "Wk", "Wv", "Wo", "Wfk", "Wfv")])


class ModelStruct(C.Structure):
    """``rwkvq_model`` of the header."""
    _fields_ = ([(n, C.c_int32) for n in ("n_layer", "n_embd", "head_size", "vocab_size", "ffn_dim",
                                          "max_rank")]
                + [("emb", QTensorStruct), ("head", QTensorStruct)]
                + [(n, _FP) for n in ("ln0_w", "ln0_b", "lnout_w", "lnout_b")]
                + [("layers", C.POINTER(LayerStruct))])


class RwkvqError(RuntimeError):
    def __init__(self, code: int, name: str, detail: str):
        super().__init__(f"{name} failed: {code} ({detail})")
        self.code = code


_lib = None

# name -> (restype, argtypes); every symbol the header declares
_PROTOS = {
    "rwkvq_strerror": (C.c_char_p, [C.c_int]),
    "rwkvq_last_error_detail": (C.c_char_p, []),
    "rwkvq_check_device": (C.c_int, []),
    "rwkvq_abi_version": (C.c_int, []),
    "rwkvq_dequant": (C.c_int, [C.POINTER(QTensorStruct), C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "rwkvq_gemv": (C.c_int, [C.POINTER(QTensorStruct), C.c_void_p, C.c_int, C.c_int, C.c_int64,
                             C.c_void_p, C.c_int64, C.c_int, C.c_void_p, C.c_void_p]),
    "rwkvq_outlier_tail": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int64,
                                     C.c_void_p, C.c_int64, C.c_int, C.c_void_p, C.c_void_p]),
    "rwkvq_quantize_sb6": (C.c_int, [C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                     C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "rwkvq_quantize_sym": (C.c_int, [C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p,
                                     C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "rwkvq_gemv_batch_workspace_bytes": (C.c_size_t, [C.c_int]),
    "rwkvq_gemv_batch": (C.c_int, [C.POINTER(QTensorStruct), C.c_void_p, C.c_int, C.c_int64, C.c_void_p, C.c_int64,
                                   C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "rwkvq_gemm_workspace_bytes": (C.c_size_t, [C.c_int]),
    "rwkvq_gemm_workspace_bytes_for": (C.c_size_t, [C.c_int, C.c_int]),
    "rwkvq_gemm": (C.c_int, [C.POINTER(QTensorStruct), C.c_void_p, C.c_int, C.c_int64, C.c_void_p, C.c_int64,
                             C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "rwkvq_gemv_fused": (C.c_int, [C.POINTER(QTensorStruct), C.c_int, C.c_void_p, C.c_int,
                                   C.c_void_p, C.c_void_p]),
    "rwkvq_wkv7": (C.c_int, [C.c_void_p] * 9 + [C.c_int] * 4 + [C.c_void_p]),
    "rwkvq_wkv_tail": (C.c_int, [C.c_void_p] * 9 + [C.c_int] * 3 + [C.c_float, C.c_void_p]),
    "rwkvq_decode_workspace_bytes": (C.c_size_t, [C.POINTER(ModelStruct), C.c_int]),
    "rwkvq_decode_step": (C.c_int, [C.POINTER(ModelStruct), C.c_int, C.c_void_p,
                                    C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.POINTER(C.c_void_p),
                                    C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p]),
    "rwkvq_relayout_meta": (C.c_int, [C.POINTER(QTensorStruct), C.c_void_p, C.c_void_p]),
    "rwkvq_relayout_planes": (C.c_int, [C.POINTER(QTensorStruct), C.c_void_p, C.c_void_p]),
    "rwkvq_gemv_t": (C.c_int, [C.POINTER(QTensorStruct), C.c_void_p, C.c_int, C.c_int64,
                               C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_void_p]),
    "rwkvq_lora_pair_workspace_bytes": (C.c_size_t, [C.c_int, C.c_int]),
    "rwkvq_lora_pair": (C.c_int, [C.POINTER(QTensorStruct), C.POINTER(QTensorStruct), C.c_int, C.POINTER(C.c_void_p),
                                  C.POINTER(C.c_void_p), C.POINTER(C.c_int), C.c_int, C.c_int, C.c_void_p, C.c_size_t,
                                  C.c_void_p]),
    "rwkvq_gemv_static": (C.c_int, [C.POINTER(QTensorStruct), C.c_void_p, C.c_int, C.c_void_p,
                                    C.c_int, C.c_void_p, C.c_void_p]),
    "rwkvq_seq_ln_shift_mix": (C.c_int, [C.c_void_p] * 5 + [C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                         C.c_void_p]),
    "rwkvq_seq_embed_ln0": (C.c_int, [C.POINTER(QTensorStruct), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                      C.c_int, C.c_void_p]),
    "rwkvq_seq_layer_norm": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_void_p]),
    "rwkvq_split_fp16": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_void_p]),
    "rwkvq_file_open": (C.c_int, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "rwkvq_file_close": (None, [C.c_void_p]),
    "rwkvq_file_get_info": (C.c_int, [C.c_void_p, C.c_void_p]),
    "rwkvq_file_tensor_key": (C.c_char_p, [C.c_void_p, C.c_int]),
    "rwkvq_file_tensor": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(QTensorStruct), C.POINTER(C.c_int32),
                                    C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.POINTER(C.c_int64)]),
    "rwkvq_file_upload": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(QTensorStruct), C.POINTER(C.c_void_p), C.c_void_p]),
    "rwkvq_file_free_slab": (C.c_int, [C.c_void_p]),
    "rwkvq_gemm_x16_pitch": (C.c_size_t, [C.c_int]),
    "rwkvq_gemm_x16": (C.c_int, [C.POINTER(QTensorStruct), C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int64,
                                 C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "rwkvq_seq_ln_shift_mix_prep": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,
                                              C.POINTER(C.c_int), C.POINTER(C.c_void_p), C.POINTER(C.c_void_p),
                                              C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_void_p,
                                              C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "rwkvq_seq_tmix_pre": (C.c_int, [C.c_void_p] * 16 + [C.c_int64, C.c_int, C.c_void_p]),
    "rwkvq_tp_alloc": (C.c_int, [C.c_size_t, C.POINTER(C.c_void_p)]),
    "rwkvq_tp_free": (C.c_int, [C.c_void_p]),
    "rwkvq_ipc_export": (C.c_int, [C.c_void_p, C.c_void_p]),
    "rwkvq_ipc_open": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "rwkvq_ipc_close": (C.c_int, [C.c_void_p]),
    "rwkvq_tp_allgather_store": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p),
                                           C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_longlong, C.c_void_p]),
}


def exported_symbols():
    """Names the header declares (and the library must export)."""
    return sorted(_PROTOS)


def load(check_device: bool = False) -> C.CDLL:
    """Load the library (once).  ``check_device`` additionally requires sm_100."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m rwkv_quant_b200.build` "
                f"(nvcc, sm_100a). There is no CPU fallback.")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in _PROTOS.items():
            fn = getattr(lib, name)         # AttributeError if the symbol is absent
            fn.restype, fn.argtypes = res, args
        _lib = lib
    if check_device:
        check(_lib.rwkvq_check_device(), "rwkvq_check_device")
    return _lib


def check(code: int, name: str) -> None:
    if code != 0:
        lib = load()
        detail = lib.rwkvq_last_error_detail().decode() or lib.rwkvq_strerror(code).decode()
        raise RwkvqError(code, name, detail)


def last_error() -> str:
    """Detail text of the calling thread's last failed library call."""
    return load().rwkvq_last_error_detail().decode()


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream
