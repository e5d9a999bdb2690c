"""The reference's checkpoint formats for `Tensor` and `Adam`: JSON and the `TS_B` binary container.

A run trained with the reference on the CPU can be resumed here and the other way round: files written here follow
the reference's writer, and everything its writer can produce is accepted by the reader here.  Host-side byte work
only; tensors reach the device through `Tensor.from_slice` / `copy_from_host`.

Format, as the reference defines it (paths inside ewhinery8/train-station):
  * serialization/binary/header.rs:20-60 — 24-byte header: magic 0x54535F42 ("TS_B"), version 1, a checksum word that
    the writer leaves 0 and the reader ignores, the length of what follows (u64) and an object type (always 0x1001,
    serialization/binary/structs.rs:8-21); little endian throughout (writer.rs:98-260).
  * structs.rs:8-140 — the body: field count (u64), then per field a name (u32 length + UTF-8) and a tagged value:
    0 bool, 1..4 i8..i64, 5..8 u8..u64, 9 usize (u64), 10 f32, 11 f64, 12 string, 13 bytes (u64 length), 14 JSON
    object (string), 15 binary object (bytes), 16 array (u64 count + values), 17 optional (bool + value), 18 object
    (u64 count + name/value pairs), 19 enum (variant string, bool, value).
  * serialization/json/structs.rs:5-110 — JSON: numbers; f32/f64 with a trailing ".0" when integral; enum as
    {"variant": ..., "data": ...}; optional as the value or null; nested serializable objects embedded as JSON.
  * tensor/core/serialization.rs:472-552 — Tensor: fields data (array of f32), shape {dims, size, strides, layout},
    device {type, index}, requires_grad.
  * optimizers/adam/serialization.rs:180-260, 524-600, 692-752 — Adam: config {learning_rate, beta1, beta2, eps,
    weight_decay, amsgrad}, states {"<id>": {m, v, v_hat_max, step}} (tensors embedded as JSON objects), step_count,
    insertion_order; `relink_parameters` (optimizers/adam/mod.rs:396-458) maps saved states to new tensors by position.
The reference builds its objects from hash maps, so the order of fields inside an object differs from file to file
even there; readers on both sides look fields up by name.
"""
from __future__ import annotations

import json
import struct
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np

MAGIC = 0x54535F42
VERSION = 1
OBJECT_TYPE = 0x1001      # ObjectType::Tensor: what to_binary_internal writes for every struct
HEADER_BYTES = 24


class SerializationError(ValueError):
    pass


# ----------------------------------------------------------------------------- field values
# A field value is a pair (tag, payload) with the reference's tag names.
class FV:
    __slots__ = ("tag", "v")

    def __init__(self, tag: str, v: Any):
        self.tag, self.v = tag, v

    def __repr__(self):
        return f"FV({self.tag}, {self.v!r})"


def fv_bool(b): return FV("Bool", bool(b))
def fv_usize(n): return FV("Usize", int(n))
def fv_f32(x): return FV("F32", np.float32(x))
def fv_string(s): return FV("String", str(s))
def fv_array(items): return FV("Array", list(items))
def fv_object(d): return FV("Object", dict(d))
def fv_enum_unit(variant): return FV("Enum", (str(variant), None))
def fv_optional(inner): return FV("Optional", inner)
def fv_json_object(text): return FV("JsonObject", str(text))


_TAGS = ["Bool", "I8", "I16", "I32", "I64", "U8", "U16", "U32", "U64", "Usize", "F32", "F64", "String", "Bytes", "JsonObject",
         "BinaryObject", "Array", "Optional", "Object", "Enum"]
_INT_FMT = {"I8": "<b", "I16": "<h", "I32": "<i", "I64": "<q", "U8": "<B", "U16": "<H", "U32": "<I", "U64": "<Q", "Usize": "<Q"}


# ----------------------------------------------------------------------------- binary
def _w_string(out: bytearray, s: str):
    b = s.encode("utf-8")
    out += struct.pack("<I", len(b)) + b


def _w_value(out: bytearray, fv: FV):
    tag = _TAGS.index(fv.tag)
    out.append(tag)
    t, v = fv.tag, fv.v
    if t == "Bool":
        out.append(1 if v else 0)
    elif t in _INT_FMT:
        out += struct.pack(_INT_FMT[t], v)
    elif t == "F32":
        out += struct.pack("<f", float(v))
    elif t == "F64":
        out += struct.pack("<d", float(v))
    elif t in ("String", "JsonObject"):
        _w_string(out, v)
    elif t in ("Bytes", "BinaryObject"):
        out += struct.pack("<Q", len(v)) + bytes(v)
    elif t == "Array":
        out += struct.pack("<Q", len(v))
        if isinstance(v, np.ndarray):                      # the tensor payload: one tag byte (10, f32) + four data bytes per element
            a = np.empty(v.size, dtype=[("t", "u1"), ("x", "<f4")])
            a["t"] = 10
            a["x"] = v.reshape(-1)
            out += a.tobytes()
        else:
            for e in v:
                _w_value(out, e)
    elif t == "Optional":
        out.append(1 if v is not None else 0)
        if v is not None:
            _w_value(out, v)
    elif t == "Object":
        out += struct.pack("<Q", len(v))
        for k, e in v.items():
            _w_string(out, k)
            _w_value(out, e)
    elif t == "Enum":
        variant, data = v
        _w_string(out, variant)
        out.append(1 if data is not None else 0)
        if data is not None:
            _w_value(out, data)
    else:
        raise SerializationError(f"unknown field tag {t}")


def fields_to_binary(fields: Sequence[Tuple[str, FV]]) -> bytes:
    body = bytearray(struct.pack("<Q", len(fields)))
    for name, fv in fields:
        _w_string(body, name)
        _w_value(body, fv)
    header = struct.pack("<IIIQI", MAGIC, VERSION, 0, len(body), OBJECT_TYPE)
    return bytes(header) + bytes(body)


class _Reader:
    def __init__(self, data: bytes):
        self.d, self.p = memoryview(data), 0

    def take(self, n: int) -> memoryview:
        if self.p + n > len(self.d):
            raise SerializationError(f"unexpected end of data at byte {self.p} (wanted {n} more)")
        r = self.d[self.p:self.p + n]
        self.p += n
        return r

    def unpack(self, fmt: str):
        return struct.unpack(fmt, self.take(struct.calcsize(fmt)))[0]

    def string(self) -> str:
        n = self.unpack("<I")
        if n > 1_000_000:      # reader.rs:265-270
            raise SerializationError(f"String length {n} exceeds maximum allowed")
        return bytes(self.take(n)).decode("utf-8")


def _r_value(r: _Reader) -> Any:
    """Decodes one tagged value into plain Python: numbers, str, bytes, list, dict; an enum becomes
    {"variant": ..., "data": ...}; a JSON object field is parsed; a float array comes back as a float32 ndarray."""
    tag = r.unpack("<B")
    if tag >= len(_TAGS):
        raise SerializationError(f"Unknown field type tag: {tag}")
    t = _TAGS[tag]
    if t == "Bool":
        return r.unpack("<B") != 0
    if t in _INT_FMT:
        return r.unpack(_INT_FMT[t])
    if t == "F32":
        return np.float32(r.unpack("<f"))
    if t == "F64":
        return r.unpack("<d")
    if t == "String":
        return r.string()
    if t == "JsonObject":
        return _json_loads(r.string())
    if t in ("Bytes", "BinaryObject"):
        return bytes(r.take(r.unpack("<Q")))
    if t == "Array":
        n = r.unpack("<Q")
        if n and r.p + 5 * n <= len(r.d):
            blob = np.frombuffer(r.d[r.p:r.p + 5 * n], dtype=[("t", "u1"), ("x", "<f4")])
            if np.all(blob["t"] == 10):                    # an array of f32: the tensor payload
                r.p += 5 * n
                return blob["x"].astype(np.float32)
        return [_r_value(r) for _ in range(n)]
    if t == "Optional":
        return _r_value(r) if r.unpack("<B") else None
    if t == "Object":
        return {r.string(): _r_value(r) for _ in range(r.unpack("<Q"))}
    variant = r.string()
    data = _r_value(r) if r.unpack("<B") else None
    return {"variant": variant, "data": data}


def binary_to_fields(data: bytes) -> Dict[str, Any]:
    if len(data) < HEADER_BYTES:
        raise SerializationError("binary data shorter than the 24-byte header")
    magic, version, _checksum, length, otype = struct.unpack("<IIIQI", data[:HEADER_BYTES])
    if magic != MAGIC:
        raise SerializationError(f"Invalid magic number: expected 0x{MAGIC:08X}, found 0x{magic:08X}")      # header.rs:80-85
    if version != VERSION:
        raise SerializationError(f"Version mismatch: expected {VERSION}, found {version}")                  # header.rs:88-93
    if otype != OBJECT_TYPE:
        raise SerializationError(f"Object type mismatch: expected 0x{OBJECT_TYPE:04X}, found 0x{otype:04X}")
    if HEADER_BYTES + length > len(data):
        raise SerializationError("data length in the header exceeds the buffer")
    r = _Reader(data[HEADER_BYTES:HEADER_BYTES + length])
    return {r.string(): _r_value(r) for _ in range(r.unpack("<Q"))}


# ----------------------------------------------------------------------------- JSON
def _f32_text(x) -> str:
    """Rust's Display for f32 (shortest digits that read back to the same f32, never an exponent), with the ".0" the
    reference appends to integral values (json/structs.rs:25-31)."""
    x = np.float32(x)
    if np.isnan(x):
        return "NaN"
    if np.isinf(x):
        return "inf" if x > 0 else "-inf"
    s = np.format_float_positional(x, unique=True, trim="-")
    return s + ".0" if float(x).is_integer() else s


_ESC = {'"': '\\"', "\\": "\\\\", "\n": "\\n", "\r": "\\r", "\t": "\\t", "\b": "\\b", "\f": "\\f"}


def _escape(s: str) -> str:
    return "".join(_ESC.get(ch, ch if ord(ch) >= 0x20 else f"\\u{ord(ch):04x}") for ch in s)


def _j_value(fv: FV) -> str:
    t, v = fv.tag, fv.v
    if t == "Bool":
        return "true" if v else "false"
    if t in _INT_FMT:
        return str(int(v))
    if t == "F32":
        return _f32_text(v)
    if t == "F64":
        return repr(float(v)) if not float(v).is_integer() else f"{int(v)}.0"
    if t == "String":
        return f'"{_escape(v)}"'
    if t in ("Bytes", "BinaryObject"):
        return '"' + bytes(v).hex() + '"'
    if t == "JsonObject":
        return v
    if t == "Array":
        if isinstance(v, np.ndarray):
            return "[" + ",".join(_f32_text(x) for x in v.reshape(-1)) + "]"
        return "[" + ",".join(_j_value(e) for e in v) + "]"
    if t == "Optional":
        return "null" if v is None else _j_value(v)
    if t == "Object":
        return "{" + ",".join(f'"{_escape(k)}":{_j_value(e)}' for k, e in v.items()) + "}"
    variant, data = v
    return f'{{"variant":"{_escape(variant)}","data":{"null" if data is None else _j_value(data)}}}'


def fields_to_json(fields: Sequence[Tuple[str, FV]]) -> str:
    return "{" + ",".join(f'"{name}":{_j_value(fv)}' for name, fv in fields) + "}"


def _json_loads(text: str) -> Any:
    try:
        return json.loads(text, parse_constant=float)     # NaN / Infinity; Rust's bare "inf" is not JSON and is refused
    except json.JSONDecodeError as e:
        raise SerializationError(f"JSON parse error: {e}") from None


def json_to_fields(text: str) -> Dict[str, Any]:
    d = _json_loads(text)
    if not isinstance(d, dict):
        raise SerializationError("Expected JSON object at root")       # json/structs.rs:113-116
    return d


# ----------------------------------------------------------------------------- typed access, as the reference's from_field_value
def _need(d: Dict[str, Any], key: str, what: str) -> Any:
    if not isinstance(d, dict) or key not in d:
        raise SerializationError(f"Missing field '{key}' in {what}")
    return d[key]


def _as_usize(v: Any, what: str) -> int:
    if isinstance(v, bool) or not isinstance(v, (int, np.integer, float, np.floating)) or float(v) != int(v) or v < 0:
        raise SerializationError(f"Expected an unsigned integer for {what}, got {v!r}")
    return int(v)


def _as_f32(v: Any, what: str) -> np.float32:
    if isinstance(v, bool) or not isinstance(v, (int, float, np.integer, np.floating)):
        raise SerializationError(f"Expected a number for {what}, got {v!r}")
    return np.float32(v)


def _variant(v: Any, what: str) -> str:
    if isinstance(v, dict) and "variant" in v:
        return str(v["variant"])
    if isinstance(v, str):
        return v
    raise SerializationError(f"Expected an enum for {what}, got {v!r}")


# ----------------------------------------------------------------------------- Tensor
def contiguous_strides(dims: Sequence[int]) -> List[int]:
    s, acc = [], 1
    for d in reversed(dims):
        s.append(acc)
        acc *= int(d)
    return list(reversed(s))


def tensor_fields(data: np.ndarray, dims: Sequence[int], requires_grad: bool, device: str = "Cpu", index: int = 0):
    """The four fields of tensor/core/serialization.rs:483-492 for a contiguous tensor."""
    data = np.ascontiguousarray(data, np.float32).reshape(-1)
    dims = [int(d) for d in dims]
    shape = fv_object({"dims": fv_array(fv_usize(d) for d in dims), "size": fv_usize(data.size),
                       "strides": fv_array(fv_usize(s) for s in contiguous_strides(dims)), "layout": fv_enum_unit("Contiguous")})
    dev = fv_object({"type": fv_enum_unit(device), "index": fv_usize(index)})
    # the data array is kept as one ndarray (an Array of F32 values in the reference's terms) so that large tensors stay cheap
    return [("data", FV("Array", data)), ("shape", shape), ("device", dev), ("requires_grad", fv_bool(requires_grad))]


def tensor_from_fields(f: Dict[str, Any]):
    """-> (float32 array with the tensor's dims, requires_grad, device type, device index); validation as in
    tensor/core/serialization.rs:386-466, 506-550."""
    data = _need(f, "data", "tensor")
    shape = _need(f, "shape", "tensor")
    dev = _need(f, "device", "tensor")
    rg = _need(f, "requires_grad", "tensor")
    if not isinstance(rg, bool):
        raise SerializationError("Expected bool for requires_grad")
    if isinstance(data, np.ndarray):
        arr = data.astype(np.float32, copy=False)
    elif isinstance(data, list):
        arr = np.array([_as_f32(x, "data") for x in data], np.float32) if data else np.zeros(0, np.float32)
    else:
        raise SerializationError("Expected an array of numbers for data")
    dims = [_as_usize(d, "shape.dims") for d in _need(shape, "dims", "shape")]
    size = _as_usize(_need(shape, "size", "shape"), "shape.size")
    strides = [_as_usize(s, "shape.strides") for s in _need(shape, "strides", "shape")]
    layout = _variant(_need(shape, "layout", "shape"), "shape.layout")
    if layout not in ("Contiguous", "Strided", "View"):
        raise SerializationError(f"Unknown memory layout: {layout}")
    expected = int(np.prod(dims, dtype=np.int64)) if dims else 1
    if size != expected:
        raise SerializationError(f"Shape size {size} doesn't match computed size {expected}")
    if len(dims) != len(strides):
        raise SerializationError("Dimensions and strides must have same length")
    if arr.size != size:
        raise SerializationError(f"Data length {arr.size} doesn't match shape size {size}")
    if strides != contiguous_strides(dims):
        # the reference rebuilds a fresh contiguous tensor and refuses a file whose strides differ (serialization.rs:539-549)
        raise SerializationError("Reconstructed tensor shape doesn't match serialized shape")
    dtype = _variant(_need(dev, "type", "device"), "device.type")
    if dtype not in ("Cpu", "Cuda"):
        raise SerializationError(f"Unknown device type: {dtype}")
    return arr.reshape(dims), rg, dtype, _as_usize(_need(dev, "index", "device"), "device.index")


# ----------------------------------------------------------------------------- Adam
def adam_fields(config: Dict[str, Any], states: Dict[int, Dict[str, Any]], step_count: int, insertion_order: Sequence[int]):
    """config: the six AdamConfig values; states: id -> {m, v, v_hat_max (or None), step, dims} with host arrays."""
    cfg = fv_object({"learning_rate": fv_f32(config["learning_rate"]), "beta1": fv_f32(config["beta1"]), "beta2": fv_f32(config["beta2"]),
                     "eps": fv_f32(config["eps"]), "weight_decay": fv_f32(config["weight_decay"]), "amsgrad": fv_bool(config["amsgrad"])})

    def embedded(a, dims):
        return fv_json_object(fields_to_json(tensor_fields(a, dims, False)))

    st = {}
    for pid, s in states.items():
        vmax = s.get("v_hat_max")
        st[str(int(pid))] = fv_object({"m": embedded(s["m"], s["dims"]), "v": embedded(s["v"], s["dims"]),
                                       "v_hat_max": fv_optional(embedded(vmax, s["dims"]) if vmax is not None else None),
                                       "step": fv_usize(s["step"])})
    return [("config", cfg), ("states", fv_object(st)), ("step_count", fv_usize(step_count)),
            ("insertion_order", fv_array(fv_usize(i) for i in insertion_order))]


def adam_from_fields(f: Dict[str, Any]):
    cfg = _need(f, "config", "Adam")
    config = {k: float(_as_f32(_need(cfg, k, "config"), k)) for k in ("learning_rate", "beta1", "beta2", "eps", "weight_decay")}
    ams = _need(cfg, "amsgrad", "config")
    if not isinstance(ams, bool):
        raise SerializationError("Expected bool for amsgrad")
    config["amsgrad"] = ams
    states = {}
    for key, s in _need(f, "states", "Adam").items():
        try:
            pid = int(key)
        except ValueError:
            raise SerializationError(f"Invalid parameter id '{key}' in states") from None

        def tensor_of(name):
            v = _need(s, name, "parameter state")
            if isinstance(v, str):            # a JSON object stored as text
                v = _json_loads(v)
            return tensor_from_fields(v)[0]

        vmax = s.get("v_hat_max")
        if isinstance(vmax, str):
            vmax = _json_loads(vmax)
        m = tensor_of("m")
        states[pid] = {"m": m, "v": tensor_of("v"), "v_hat_max": tensor_from_fields(vmax)[0] if vmax is not None else None,
                       "step": _as_usize(_need(s, "step", "parameter state"), "step"), "dims": list(m.shape)}
    order = [_as_usize(i, "insertion_order") for i in _need(f, "insertion_order", "Adam")]
    return config, states, _as_usize(_need(f, "step_count", "Adam"), "step_count"), order
