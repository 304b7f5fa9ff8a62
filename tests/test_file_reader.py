"""The C reader of the .rwkvq container (rwkvq_file_*) against the Python reader and the
reference-written fixtures: same manifest facts, same bytes behind every descriptor pointer,
same refusals (formats/codec.py:462-511, formats/reader.py:42-93).  Host code only."""
import ctypes as C
import json
import os

import numpy as np
import pytest

from conftest import GOLDEN
from rwkv_quant_b200 import _lib
from rwkv_quant_b200.formats import container
from test_container import _rewrite_manifest

FIXTURES = ["toy_compression", "toy_reduction", "toy_custom_int8", "toy_custom_compression", "toy_custom_d128_int8"]


class Info(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("format_version", "naming", "n_layer", "n_embd", "head_size",
                                         "vocab_size", "n_tensors")]


def _open(lib, path):
    h = C.c_void_p()
    rc = lib.rwkvq_file_open(path.encode(), C.byref(h))
    return rc, h


# descriptor member -> file field, per layout kind (include/rwkvq_b200.h)
MEMBERS = {
    "dense": {"codes": "dense"},
    "sb6": {"codes": "codes_packed", "qh": "gw_qh", "qh2": "gw_qh2", "qsqm": "gw_qsqm", "d": "gw_d", "dm": "gw_dm"},
    "sym": {"codes": ("codes", "codes_packed"), "qh": "gw_qh", "qh2": "gw_qh2", "qs": "gw_qs", "d": "gw_d"},
    "asym": {"codes": "codes", "scale": "gw_scale", "mn": "gw_min"},
    "rtn": {"codes": ("codes", "codes_packed"), "scale": "scale"},
}


@pytest.mark.parametrize("name", FIXTURES)
def test_c_reader_equals_python_reader(name):
    lib = _lib.load()
    path = os.path.join(GOLDEN, name + ".rwkvq")
    man, arrays, _ = container.open_rwkvq(path)
    rc, h = _open(lib, path)
    assert rc == 0, _lib.last_error()
    try:
        info = Info()
        assert lib.rwkvq_file_get_info(h, C.byref(info)) == 0
        assert info.format_version == man["format_version"] and info.naming == (man["naming"] == "custom")
        assert (info.n_layer, info.n_embd, info.head_size, info.vocab_size) == \
            (man["n_layer"], man["n_embd"], man["head_size"], man["vocab_size"])
        keys = [lib.rwkvq_file_tensor_key(h, i).decode() for i in range(info.n_tensors)]
        assert keys == list(man["tensors"].keys())
        assert lib.rwkvq_file_tensor_key(h, info.n_tensors) is None
        n_out = 0
        for key, t in man["tensors"].items():
            v = _lib.QTensorStruct()
            tr, oi, ov, no = C.c_int32(-1), C.c_void_p(), C.c_void_p(), C.c_int64(-1)
            assert lib.rwkvq_file_tensor(h, key.encode(), C.byref(v), C.byref(tr), C.byref(oi), C.byref(ov),
                                         C.byref(no)) == 0, _lib.last_error()
            shape = t["shape"]
            assert v.kind == _lib.KIND[t["kind"]] and v.bits == t["bits"]
            assert v.cols == shape[-1] and v.rows == int(np.prod(shape[:-1], dtype=np.int64))
            assert (v.gs, v.sb) == (t["gw_gs"], t["gw_sb"])
            assert bool(tr.value) == bool(t["transposed"])
            for member, field in MEMBERS[t["kind"]].items():
                fields = field if isinstance(field, tuple) else (field,)
                present = [f for f in fields if f in t["fields"]]
                ptr = getattr(v, member)
                if not present:
                    assert ptr is None, (key, member)
                    continue
                a = arrays[f"{key}::{present[0]}"]
                assert C.string_at(ptr, a.nbytes) == a.tobytes(), (key, member)
            if "outlier_indices" in t["fields"] and arrays[f"{key}::outlier_values"].size:
                a_i, a_v = arrays[f"{key}::outlier_indices"], arrays[f"{key}::outlier_values"]
                assert no.value == a_v.size
                assert C.string_at(oi.value, a_i.nbytes) == a_i.tobytes()
                assert C.string_at(ov.value, a_v.nbytes) == a_v.tobytes()
                n_out += 1
            else:
                assert no.value == 0 and oi.value is None
        assert (n_out > 0) == ("int8" in name)
        v = _lib.QTensorStruct()
        assert lib.rwkvq_file_tensor(h, b"no.such.tensor", C.byref(v), None, None, None, None) == _lib.E_FORMAT
    finally:
        lib.rwkvq_file_close(h)


def test_c_reader_refusals(tmp_path):
    lib = _lib.load()
    src = os.path.join(GOLDEN, "toy_compression.rwkvq")
    p = str(tmp_path / "x.rwkvq")

    def refused():
        rc, h = _open(lib, p)
        assert h.value is None
        return rc == _lib.E_FORMAT

    _rewrite_manifest(src, p, lambda m, h: m.__setitem__("format_version", 3))
    assert refused() and "newer" in _lib.last_error()
    _rewrite_manifest(src, p, lambda m, h: m.__setitem__("format", "gguf"))
    assert refused()
    _rewrite_manifest(src, p, lambda m, h: None, drop=True)
    assert refused() and "manifest" in _lib.last_error()
    open(p, "wb").write(b"PK\x03\x04" + b"\0" * 64)
    assert refused() and "pickle" in _lib.last_error()
    open(p, "wb").write(b"\x01\x02")
    assert refused()
    open(p, "wb").write((1 << 40).to_bytes(8, "little") + b"{}")
    assert refused()
    open(p, "wb").write((9).to_bytes(8, "little") + b'{"a": [1,')
    assert refused()
    assert _open(lib, str(tmp_path / "missing.rwkvq"))[0] == _lib.E_FORMAT
    # a buffer that points outside the file
    def beyond(m, h):
        k = next(k for k in h if k.endswith("::codes_packed"))
        h[k]["data_offsets"] = [h[k]["data_offsets"][0], 1 << 40]
    _rewrite_manifest(src, p, beyond)
    assert refused() and "outside" in _lib.last_error()
    # a dtype / shape that disagrees with the byte count
    def wrong_shape(m, h):
        k = next(k for k in h if k.endswith("::codes_packed"))
        h[k]["shape"] = [h[k]["shape"][0], h[k]["shape"][1] + 1]
    _rewrite_manifest(src, p, wrong_shape)
    assert refused()
    # version-1 manifests (no `transposed`) stay readable, orientation from the key
    def v1(m, h):
        m["format_version"] = 1
        for t in m["tensors"].values():
            t.pop("transposed", None)
            t.pop("n_blocks", None)
    _rewrite_manifest(src, p, v1)
    rc, h = _open(lib, p)
    assert rc == 0
    v, tr = _lib.QTensorStruct(), C.c_int32()
    lib.rwkvq_file_tensor(h, b"blocks.0.att.w1", C.byref(v), C.byref(tr), None, None, None)
    assert tr.value == 1
    lib.rwkvq_file_tensor(h, b"head.weight", C.byref(v), C.byref(tr), None, None, None)
    assert tr.value == 0
    lib.rwkvq_file_close(h)


def test_c_reader_refuses_buffers_that_do_not_fit_the_shape(tmp_path):
    """The descriptor has no buffer sizes: a manifest shape larger than its buffers, a missing
    plane, or a sparse override outside the tensor is refused when the descriptor is made."""
    import torch
    from rwkv_quant_b200 import synth
    lib = _lib.load()
    src = os.path.join(GOLDEN, "toy_compression.rwkvq")
    p = str(tmp_path / "x.rwkvq")

    def tensor_rc(key):
        rc, h = _open(lib, p)
        assert rc == 0, _lib.last_error()
        v = _lib.QTensorStruct()
        rc = lib.rwkvq_file_tensor(h, key.encode(), C.byref(v), None, None, None, None)
        slab, dv = C.c_void_p(), _lib.QTensorStruct()
        rc_up = lib.rwkvq_file_upload(h, key.encode(), C.byref(dv), C.byref(slab), None)   # refused before any CUDA call
        lib.rwkvq_file_close(h)
        assert rc_up == rc and slab.value is None
        return rc

    def grow_rows(m, h):
        m["tensors"]["blocks.0.ffn.key.weight"]["shape"][0] += 16
    _rewrite_manifest(src, p, grow_rows)
    assert tensor_rc("blocks.0.ffn.key.weight") == _lib.E_FORMAT and "codes_packed" in _lib.last_error()
    def drop_plane(m, h):
        t = m["tensors"]["blocks.0.att.key.weight"]
        t["fields"] = [f for f in t["fields"] if f != "gw_qh"]
    _rewrite_manifest(src, p, drop_plane)
    assert tensor_rc("blocks.0.att.key.weight") == _lib.E_FORMAT and "gw_qh" in _lib.last_error()
    def grow_lora(m, h):
        m["tensors"]["blocks.1.att.w1"]["shape"][1] += 64
    _rewrite_manifest(src, p, grow_lora)
    assert tensor_rc("blocks.1.att.w1") == _lib.E_FORMAT
    # an override that points outside its tensor
    ck = synth.build_checkpoint("toy", "compression", seed=1)
    qt = ck.tensors["blocks.0.att.g1"]
    qt.outlier_indices = torch.tensor([[0, 1], [qt.shape[0], 0]], dtype=torch.int32)
    qt.outlier_values = torch.zeros(2, dtype=torch.bfloat16)
    container.save_rwkvq(ck, p)
    rc, h = _open(lib, p)
    assert rc == 0
    v = _lib.QTensorStruct()
    assert lib.rwkvq_file_tensor(h, b"blocks.0.att.g1", C.byref(v), None, None, None, None) == _lib.E_FORMAT
    assert "outside" in _lib.last_error()
    lib.rwkvq_file_close(h)
    with pytest.raises(ValueError, match="outside"):
        container.load_raw(p)


def test_json_strings_with_escapes(tmp_path):
    """config_repr and tokenizer may carry quotes, backslashes and non-ASCII text."""
    lib = _lib.load()
    src = os.path.join(GOLDEN, "toy_reduction.rwkvq")
    p = str(tmp_path / "x.rwkvq")
    _rewrite_manifest(src, p, lambda m, h: m.update(config_repr='q"uo\\te\né中\U0001f600', tokenizer=None))
    rc, h = _open(lib, p)
    assert rc == 0, _lib.last_error()
    info = Info()
    lib.rwkvq_file_get_info(h, C.byref(info))
    assert info.n_tensors == len(json.loads(json.dumps(container.open_rwkvq(p)[0]))["tensors"])
    lib.rwkvq_file_close(h)
