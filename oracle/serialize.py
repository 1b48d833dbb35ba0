"""The reference's checkpoint formats restated in numpy (TEST INFRASTRUCTURE ONLY, like the rest of oracle/).

* text: src/serialize.rs:81-136 (`save_tensors` / `load_tensors`): "tensors N", per tensor "len L" and one value
  per line in Rust's `{}` form — the shortest decimal that reads back to the same f32, positional, no exponent.
* safetensors: src/serialize.rs:197-238 through the `safetensors` crate (0.8.0 in the reference's Cargo.lock).
  The crate is not vendored in the reference; its published layout is: u64 little-endian header length, a
  compact JSON header {"name":{"dtype":"F32","shape":[..],"data_offsets":[b,e]},..} with the tensors in name
  order (all F32 here) padded with spaces to a multiple of 8 bytes, then the little-endian data back to back.
* `load` returns safetensors tensors sorted by name (:235); text tensors as tensor_{i} with a flat shape (:188-194).
"""
import json
import struct

import numpy as np


def format_f32(v) -> str:
    v = np.float32(v)
    if np.isnan(v):
        return "NaN"
    if np.isinf(v):
        return "-inf" if v < 0 else "inf"
    return np.format_float_positional(v, unique=True, trim="-")


def text_bytes(tensors) -> bytes:
    lines = [f"tensors {len(tensors)}"]
    for _, _, data in tensors:
        data = np.asarray(data, np.float32).ravel()
        lines.append(f"len {data.size}")
        lines += [format_f32(v) for v in data]
    return ("\n".join(lines) + "\n").encode()


def safetensors_bytes(tensors) -> bytes:
    order = sorted(tensors, key=lambda t: t[0])
    header, blobs, off = {}, [], 0
    for name, shape, data in order:
        raw = np.asarray(data, "<f4").ravel().tobytes()
        header[name] = {"dtype": "F32", "shape": [int(s) for s in shape], "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    h = json.dumps(header, separators=(",", ":"), ensure_ascii=False).encode()
    h += b" " * (-len(h) % 8)
    return struct.pack("<Q", len(h)) + h + b"".join(blobs)


def save_bytes(tensors, path: str) -> bytes:
    return safetensors_bytes(tensors) if path.endswith(".safetensors") else text_bytes(tensors)


def load_bytes(buf: bytes, path: str):
    if path.endswith(".safetensors"):
        (n,) = struct.unpack("<Q", buf[:8])
        header = json.loads(buf[8:8 + n])
        data = buf[8 + n:]
        out = []
        for name, info in header.items():
            if name == "__metadata__":
                continue
            assert info["dtype"] == "F32"
            b, e = info["data_offsets"]
            out.append((name, list(info["shape"]), np.frombuffer(data[b:e], "<f4").copy()))
        return sorted(out, key=lambda t: t[0])
    lines = buf.decode().split("\n")
    n = int(lines[0].split()[1])
    out, at = [], 1
    for i in range(n):
        ln = int(lines[at].split()[1])
        vals = np.array([np.float32(x) for x in lines[at + 1:at + 1 + ln]], np.float32)
        out.append((f"tensor_{i}", [ln], vals))
        at += 1 + ln
    return out
