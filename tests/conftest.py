import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")
REFERENCE = os.environ.get("RWKVQ_REFERENCE", os.path.join(os.path.dirname(ROOT), "reference"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) GPU and the built CUDA library")


def have_reference() -> bool:
    return os.path.isdir(os.path.join(REFERENCE, "rwkv_quant"))


@pytest.fixture(scope="session")
def reference():
    """The reference project, importable; tests using it are skipped where it is absent."""
    if not have_reference():
        pytest.skip("reference project not present on this machine")
    if REFERENCE not in sys.path:
        sys.path.insert(0, REFERENCE)
    import rwkv_quant  # noqa: F401
    return REFERENCE


@pytest.fixture(scope="session")
def codec_cases():
    """{name: (meta, {field: ndarray}, sample)} from tests/golden/codec_cases.npz."""
    z = np.load(os.path.join(GOLDEN, "codec_cases.npz"))
    meta = json.loads(bytes(z["__meta__"]).decode())
    out = {}
    for name, m in meta.items():
        out[name] = (m, {f: z[f"{name}::{f}"] for f in m["fields"]}, z[f"{name}::sample"])
    return out


@pytest.fixture(scope="session")
def config1_case():
    """(meta, {field: ndarray}, x fp16 [1, 2048], y fp32 [1, 8192]) of tests/golden/config1_gemv.npz:
    the single-GEMV benchmark tensor as packed by the reference's search packer."""
    z = np.load(os.path.join(GOLDEN, "config1_gemv.npz"))
    meta = json.loads(bytes(z["__meta__"]).decode())["config1"]
    return meta, {f: z[f"config1::{f}"] for f in meta["fields"]}, z["x"], z["y"]


@pytest.fixture(scope="session")
def cuda_lib():
    """The loaded C-ABI library on a B200; GPU tests fail (not skip) if it is missing."""
    import torch
    from rwkv_quant_b200 import _lib
    assert torch.cuda.is_available(), "GPU test selected but no CUDA device is visible"
    return _lib.load(check_device=True)
