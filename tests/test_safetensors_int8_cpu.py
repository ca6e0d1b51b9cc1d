"""CPU tests of the int8 on-disk format: bit-for-bit round trips, the container's byte layout
(checked against a hand-assembled file), F32-only files as the reference's own writer lays them
out (src/io/safetensors.rs:12-51), and the errors for foreign dtypes and damaged files."""
import json
import struct
import types

import numpy as np
import pytest

import oracle


def fake_qlinear(seed, n, k, bias=True):
    w = oracle.normal(seed, 0, (n, k), 0.0, 0.02)
    q, s = oracle.quantize_rows(w)
    b = oracle.normal(seed, 1, (n,), 0.0, 0.1) if bias else None
    return types.SimpleNamespace(qweight=q.reshape(-1), scales=s, bias=b, in_features=k, out_features=n)


def test_round_trip_bit_for_bit(nne, tmp_path):
    st = nne.safetensors_int8
    layers = {"model.layers.0.q_proj": fake_qlinear(1, 96, 160), "model.layers.0.down_proj": fake_qlinear(2, 33, 7, bias=False)}
    path = str(tmp_path / "q.safetensors")
    st.save_qlinears(layers, path)
    for name, ql in layers.items():
        q, s, b = st.load_qlinear_fields(path, name)
        assert q.dtype == np.int8 and np.array_equal(q.reshape(-1), ql.qweight)
        assert np.array_equal(s.view(np.uint32), ql.scales.view(np.uint32))
        assert (b is None) == (ql.bias is None)
        if b is not None:
            assert np.array_equal(b.view(np.uint32), ql.bias.view(np.uint32))
    with pytest.raises(st.SerializationError):
        st.load_qlinear_fields(path, "model.layers.1.q_proj")


def test_container_layout_matches_a_hand_built_file(nne, tmp_path):
    st = nne.safetensors_int8
    q = np.array([[1, -2, 3], [-128, 127, 0]], dtype=np.int8)
    s = np.array([0.5, 0.25], dtype=np.float32)
    path = str(tmp_path / "a.safetensors")
    st.save_tensors({"l.qweight": q, "l.scales": s}, path)
    raw = open(path, "rb").read()
    (hlen,) = struct.unpack("<Q", raw[:8])
    assert hlen % 8 == 0
    header = json.loads(raw[8:8 + hlen])
    assert header == {"l.qweight": {"dtype": "I8", "shape": [2, 3], "data_offsets": [0, 6]},
                      "l.scales": {"dtype": "F32", "shape": [2], "data_offsets": [6, 14]}}
    assert raw[8 + hlen:] == q.tobytes() + s.astype("<f4").tobytes()
    # and a file assembled by hand, header unpadded, loads
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 16]},
                      "__metadata__": {"who": "test"}}).encode()
    w = np.arange(4, dtype="<f4").reshape(2, 2)
    p2 = str(tmp_path / "b.safetensors")
    open(p2, "wb").write(struct.pack("<Q", len(hdr)) + hdr + w.tobytes())
    assert np.array_equal(st.load_tensors(p2)["w"], w)


def test_foreign_dtypes_and_damaged_files_are_errors(nne, tmp_path):
    st = nne.safetensors_int8
    def write(header, data):
        h = json.dumps(header).encode()
        p = str(tmp_path / "x.safetensors")
        open(p, "wb").write(struct.pack("<Q", len(h)) + h + data)
        return p
    with pytest.raises(st.SerializationError, match="Unsupported SafeTensors dtype F16"):
        st.load_tensors(write({"t": {"dtype": "F16", "shape": [2], "data_offsets": [0, 4]}}, b"\0" * 4))
    with pytest.raises(st.SerializationError, match="do not match shape"):
        st.load_tensors(write({"t": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}, b"\0" * 8))
    with pytest.raises(st.SerializationError, match="outside the file"):
        st.load_tensors(write({"t": {"dtype": "I8", "shape": [9], "data_offsets": [0, 9]}}, b"\0" * 4))
    with pytest.raises(st.SerializationError, match="not contiguous"):
        st.load_tensors(write({"t": {"dtype": "I8", "shape": [2], "data_offsets": [2, 4]}}, b"\0" * 4))
    p = str(tmp_path / "short.safetensors")
    open(p, "wb").write(b"\1\2\3")
    with pytest.raises(st.SerializationError):
        st.load_tensors(p)
    with pytest.raises(st.SerializationError, match="F32 and I8 only"):
        st.save_tensors({"t": np.zeros(2, dtype=np.float64)}, str(tmp_path / "y.safetensors"))
    with pytest.raises(st.SerializationError):
        st.load_tensors(str(tmp_path / "missing.safetensors"))
