"""Checkpoint formats of src/serialize.rs: the library's host-side reader / writer (C ABI, no GPU needed) against
the numpy restatement in oracle/serialize.py, replaying the reference's tests/serialize_test.rs, and — where the
`safetensors` Python package is installed — against that independent implementation of the published format."""
import os
import struct

import numpy as np
import pytest

from oracle import serialize as ref


@pytest.fixture(scope="module")
def ser(nrs_lib):
    from neuralrs_b200.cuda import serialize
    return serialize


def test_format_f32_is_rust_display():
    # Rust's `{}` for f32: shortest digits that round-trip, positional, no exponent, no trailing ".0"
    cases = [(1.5, "1.5"), (-2.25, "-2.25"), (0.0, "0"), (3.75, "3.75"), (0.125, "0.125"), (1.0, "1"), (-0.0, "-0"),
             (1e-7, "0.0000001"), (0.1, "0.1"), (16777216.0, "16777216"), (1e10, "10000000000"),
             (3.4028235e38, "340282350000000000000000000000000000000")]
    for v, want in cases:
        assert ref.format_f32(v) == want
    assert ref.format_f32(float("inf")) == "inf" and ref.format_f32(float("nan")) == "NaN"


def test_text_roundtrip_reference_cases(ser, tmp_path):
    # tests/serialize_test.rs:31-43 (save_load_tensors_roundtrip) and :66-75 (text through the unified API)
    a, b = np.array([1.5, -2.25, 0.0, 3.75], np.float32), np.full(7, 0.125, np.float32)
    path = str(tmp_path / "test_tensors.txt")
    ser.save([("x", [4], a), ("y", [7], b)], path)
    raw = open(path, "rb").read()
    assert raw == ref.text_bytes([("x", [4], a), ("y", [7], b)])
    assert raw.startswith(b"tensors 2\nlen 4\n1.5\n-2.25\n0\n3.75\nlen 7\n0.125\n")
    assert not os.path.exists(path + ".tmp")                 # written to <path>.tmp, then renamed
    got = ser.load(path)
    assert [g[0] for g in got] == ["tensor_0", "tensor_1"]   # the text format drops names ...
    assert [g[1] for g in got] == [[4], [7]]                 # ... and shapes
    assert np.array_equal(got[0][2], a) and np.array_equal(got[1][2], b)


def test_text_is_lossless_for_awkward_values(ser, tmp_path):
    rng = np.random.default_rng(3)
    bits = rng.integers(0, 2 ** 32, 4000, dtype=np.uint64).astype(np.uint32)
    vals = bits.view(np.float32)
    vals = vals[np.isfinite(vals)]
    vals = np.concatenate([vals, np.array([0.0, -0.0, 1e-45, 1.17549435e-38, 3.4028235e38, np.inf, -np.inf], np.float32)])
    path = str(tmp_path / "awkward.txt")
    ser.save([("v", [vals.size], vals)], path)
    assert open(path, "rb").read() == ref.text_bytes([("v", [vals.size], vals)])     # same digits as the restatement
    got = ser.load(path)[0][2]
    assert np.array_equal(got.view(np.uint32), vals.view(np.uint32))                 # bit-exact, signed zero included
    assert all(np.array_equal(x[2].view(np.uint32), vals.view(np.uint32)) for x in ref.load_bytes(open(path, "rb").read(), path))


def test_safetensors_roundtrip_reference_case(ser, tmp_path):
    # tests/serialize_test.rs:45-64: saved weight-then-bias, loaded back name-sorted with shapes
    a = np.array([1.5, -2.25, 0.0, 3.75, 0.125, -1.0], np.float32)
    b = np.full(12, 0.5, np.float32)
    path = str(tmp_path / "test_roundtrip.safetensors")
    tensors = [("layer.weight", [2, 3], a), ("layer.bias", [12], b)]
    ser.save(tensors, path)
    raw = open(path, "rb").read()
    assert raw == ref.safetensors_bytes(tensors)
    (n,) = struct.unpack("<Q", raw[:8])
    assert n % 8 == 0 and raw[8:8 + n].rstrip(b" ") == (
        b'{"layer.bias":{"dtype":"F32","shape":[12],"data_offsets":[0,48]},'
        b'"layer.weight":{"dtype":"F32","shape":[2,3],"data_offsets":[48,72]}}')
    got = ser.load(path)
    assert [(g[0], g[1]) for g in got] == [("layer.bias", [12]), ("layer.weight", [2, 3])]
    assert np.array_equal(got[0][2], b) and np.array_equal(got[1][2], a)
    want = ref.load_bytes(raw, path)
    assert all(g[0] == w[0] and g[1] == w[1] and np.array_equal(g[2], w[2]) for g, w in zip(got, want))


def test_safetensors_against_the_python_package(ser, tmp_path):
    st = pytest.importorskip("safetensors.numpy")
    rng = np.random.default_rng(5)
    tensors = [("conv1.weight", [4, 3, 3, 3], rng.normal(size=108).astype(np.float32)), ("conv1.bias", [4], rng.normal(size=4).astype(np.float32)),
               ("optim.t", [1], np.array([17.0], np.float32)), ("empty", [0], np.zeros(0, np.float32)),
               ('odd "name"\\x', [2], np.array([1.0, 2.0], np.float32))]
    path = str(tmp_path / "ours.safetensors")
    ser.save(tensors, path)
    theirs = st.load_file(path)                                # the package reads what the library wrote
    assert set(theirs) == {t[0] for t in tensors}
    for name, shape, data in tensors:
        assert list(theirs[name].shape) == shape and np.array_equal(theirs[name].ravel(), data)
    path2 = str(tmp_path / "theirs.safetensors")
    st.save_file({name: data.reshape(shape) for name, shape, data in tensors}, path2, metadata={"format": "np"})
    got = ser.load(path2)                                      # the library reads what the package wrote (metadata skipped)
    assert [g[0] for g in got] == sorted(t[0] for t in tensors)
    by = {t[0]: t for t in tensors}
    assert all(g[1] == by[g[0]][1] and np.array_equal(g[2], by[g[0]][2]) for g in got)


def test_load_rejects_malformed_files(ser, tmp_path):
    from neuralrs_b200._lib import NrsError
    cases = {"short.safetensors": b"\x01\x02", "hdrlen.safetensors": struct.pack("<Q", 1 << 40) + b"{}",
             "json.safetensors": struct.pack("<Q", 8) + b"{\"a\": [ ",
             "dtype.safetensors": ref.safetensors_bytes([("a", [1], [1.0])]).replace(b"F32", b"F16"),
             "offsets.safetensors": ref.safetensors_bytes([("a", [2], [1.0, 2.0])]).replace(b"[0,8]", b"[0,4]"),
             "trunc.txt": b"tensors 2\nlen 2\n1\n", "value.txt": b"tensors 1\nlen 1\nabc\n", "header.txt": b"nonsense\n"}
    for name, blob in cases.items():
        p = tmp_path / name
        p.write_bytes(blob)
        with pytest.raises(NrsError):
            ser.load(str(p))
    with pytest.raises(NrsError):
        ser.load(str(tmp_path / "missing.safetensors"))
    with pytest.raises(ValueError):                            # shape that does not match the data
        ser.save([("a", [3], np.zeros(2, np.float32))], str(tmp_path / "bad.safetensors"))
    # an interrupted or failed save leaves an existing checkpoint alone
    good = str(tmp_path / "keep.safetensors")
    ser.save([("a", [2], np.array([1.0, 2.0], np.float32))], good)
    before = open(good, "rb").read()
    with pytest.raises(NrsError):
        ser.save([("a", [2], np.zeros(2, np.float32)), ("a", [2], np.zeros(2, np.float32))], good)   # duplicate name
    assert open(good, "rb").read() == before
