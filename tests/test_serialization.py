"""CPU: the codec of the reference's checkpoint formats (train-station_b200/serialization.py) against byte strings and
JSON text assembled here by hand from the reference's format definition (serialization/binary/{header,structs,writer}.rs,
serialization/json/structs.rs, tensor/core/serialization.rs:472-552, optimizers/adam/serialization.rs).  No device is
involved.  The reference cannot be run in this environment, so no file produced by it is available: the format is
pinned by its source, and the reader is exercised on every encoding its writer can choose (field order inside objects
is arbitrary there, since it iterates hash maps)."""
import json
import struct

import numpy as np
import pytest


@pytest.fixture(scope="module")
def S(ts):
    return ts.serialization


def s_(text):      # string: u32 length + UTF-8 (writer.rs:286-292)
    b = text.encode()
    return struct.pack("<I", len(b)) + b


def usize(n):      # tag 9 + u64
    return b"\x09" + struct.pack("<Q", n)


def f32(x):        # tag 10 + f32
    return b"\x0a" + struct.pack("<f", x)


def enum_unit(v):  # tag 19 + variant + has_data = 0
    return b"\x13" + s_(v) + b"\x00"


def hand_built_tensor_bytes(order=("dims", "size", "strides", "layout"), dev_order=("type", "index")):
    """Tensor [[1.5, -2.0, 0.25]] (dims [1, 3]), requires_grad = true, device Cpu:0."""
    shape_fields = {"dims": b"\x10" + struct.pack("<Q", 2) + usize(1) + usize(3), "size": usize(3),
                    "strides": b"\x10" + struct.pack("<Q", 2) + usize(3) + usize(1), "layout": enum_unit("Contiguous")}
    dev_fields = {"type": enum_unit("Cpu"), "index": usize(0)}
    body = struct.pack("<Q", 4)
    body += s_("data") + b"\x10" + struct.pack("<Q", 3) + f32(1.5) + f32(-2.0) + f32(0.25)
    body += s_("shape") + b"\x12" + struct.pack("<Q", 4) + b"".join(s_(k) + shape_fields[k] for k in order)
    body += s_("device") + b"\x12" + struct.pack("<Q", 2) + b"".join(s_(k) + dev_fields[k] for k in dev_order)
    body += s_("requires_grad") + b"\x00\x01"
    header = struct.pack("<I", 0x54535F42) + struct.pack("<I", 1) + struct.pack("<I", 0) + struct.pack("<Q", len(body)) + struct.pack("<I", 0x1001)
    return header + body


def test_binary_writer_matches_hand_built_bytes(S):
    x = np.array([[1.5, -2.0, 0.25]], np.float32)
    got = S.fields_to_binary(S.tensor_fields(x, [1, 3], True))
    assert got == hand_built_tensor_bytes()
    assert got[:4] == b"B_ST"                          # 0x54535F42 little endian: "TS_B" read as a big-endian word
    assert len(got) == 24 + struct.unpack("<Q", got[12:20])[0]


def test_binary_reader_accepts_any_field_order(S):
    for order in (("dims", "size", "strides", "layout"), ("layout", "strides", "size", "dims"), ("size", "layout", "dims", "strides")):
        for dev_order in (("type", "index"), ("index", "type")):
            arr, rg, dev, idx = S.tensor_from_fields(S.binary_to_fields(hand_built_tensor_bytes(order, dev_order)))
            assert arr.tolist() == [[1.5, -2.0, 0.25]] and rg is True and dev == "Cpu" and idx == 0


def test_json_writer_text(S):
    x = np.array([[1.5, -2.0, 0.25]], np.float32)
    text = S.fields_to_json(S.tensor_fields(x, [1, 3], True))
    assert text == ('{"data":[1.5,-2.0,0.25],"shape":{"dims":[1,3],"size":3,"strides":[3,1],"layout":{"variant":"Contiguous","data":null}},'
                    '"device":{"type":{"variant":"Cpu","data":null},"index":0},"requires_grad":true}')
    arr, rg, dev, idx = S.tensor_from_fields(S.json_to_fields(text))
    assert arr.tolist() == [[1.5, -2.0, 0.25]] and rg and dev == "Cpu"
    # whitespace and reordered keys, as another writer might produce
    loose = json.dumps({"requires_grad": False, "device": {"index": 1, "type": {"variant": "Cuda", "data": None}},
                        "shape": {"layout": {"variant": "Contiguous", "data": None}, "size": 2, "dims": [2], "strides": [1]}, "data": [1, 2.5]}, indent=2)
    arr, rg, dev, idx = S.tensor_from_fields(S.json_to_fields(loose))
    assert arr.tolist() == [1.0, 2.5] and rg is False and dev == "Cuda" and idx == 1


def test_f32_text_is_rusts_display(S):
    """Display for f32: shortest digits that read back, no exponent; the reference appends ".0" to integral values."""
    cases = {3.0: "3.0", -0.0: "-0.0", 0.1: "0.1", 1e-8: "0.00000001", 1e20: "100000000000000000000.0", 16777216.0: "16777216.0",
             0.3333333432674408: "0.33333334", 1.17549435e-38: "0.000000000000000000000000000000000000011754944"}
    for x, want in cases.items():
        assert S._f32_text(np.float32(x)) == want, x
    for x in np.random.default_rng(0).standard_normal(2000).astype(np.float32):
        assert np.float32(float(S._f32_text(x))) == x        # reads back to the same f32


def test_round_trips_preserve_every_bit(S):
    rng = np.random.default_rng(1)
    x = rng.standard_normal((7, 5, 3)).astype(np.float32)
    x.reshape(-1)[:6] = [0.0, -0.0, 1e-45, -3.4e38, 1.17549435e-38, 16777217.0]
    for enc, dec in ((S.fields_to_binary, S.binary_to_fields), (S.fields_to_json, S.json_to_fields)):
        arr, rg, _, _ = S.tensor_from_fields(dec(enc(S.tensor_fields(x, list(x.shape), False))))
        assert arr.shape == x.shape and rg is False
        assert np.array_equal(arr.view(np.uint32), x.view(np.uint32))
    e = np.zeros((0, 4), np.float32)
    arr, _, _, _ = S.tensor_from_fields(S.binary_to_fields(S.fields_to_binary(S.tensor_fields(e, [0, 4], False))))
    assert arr.shape == (0, 4)


def test_reader_refuses_what_the_reference_refuses(S):
    good = hand_built_tensor_bytes()
    E = S.SerializationError
    with pytest.raises(E, match="Invalid magic"):                      # header.rs:80-85
        S.binary_to_fields(b"\x00" + good[1:])
    with pytest.raises(E, match="Version mismatch"):                   # header.rs:88-93
        S.binary_to_fields(good[:4] + struct.pack("<I", 2) + good[8:])
    with pytest.raises(E, match="Object type mismatch"):
        S.binary_to_fields(good[:20] + struct.pack("<I", 0x1002) + good[24:])
    with pytest.raises(E):
        S.binary_to_fields(good[:-3])                                   # truncated
    with pytest.raises(E, match="Expected JSON object at root"):
        S.json_to_fields("[1, 2]")
    base = {"data": [1, 2, 3, 4, 5, 6], "shape": {"dims": [2, 3], "size": 6, "strides": [3, 1], "layout": {"variant": "Contiguous", "data": None}},
            "device": {"type": {"variant": "Cpu", "data": None}, "index": 0}, "requires_grad": False}

    def broken(path, value):
        d = json.loads(json.dumps(base))
        t = d
        for k in path[:-1]:
            t = t[k]
        t[path[-1]] = value
        return d

    with pytest.raises(E, match="doesn't match computed size"):        # tensor/core/serialization.rs:443-452 (size 10 for dims [2,3])
        S.tensor_from_fields(broken(("shape", "size"), 10))
    with pytest.raises(E, match="same length"):                        # :454-459
        S.tensor_from_fields(broken(("shape", "strides"), [3]))
    with pytest.raises(E, match="Data length"):                        # :513-523
        S.tensor_from_fields(broken(("data",), [1, 2, 3]))
    with pytest.raises(E, match="Unknown memory layout"):
        S.tensor_from_fields(broken(("shape", "layout"), {"variant": "Tiled", "data": None}))
    with pytest.raises(E, match="Unknown device type"):
        S.tensor_from_fields(broken(("device", "type"), {"variant": "Tpu", "data": None}))
    with pytest.raises(E, match="doesn't match serialized shape"):     # :539-549: strides of a non-contiguous view
        S.tensor_from_fields(broken(("shape", "strides"), [1, 2]))
    with pytest.raises(E, match="Missing field"):
        S.tensor_from_fields({k: v for k, v in base.items() if k != "device"})


def test_adam_fields_round_trip(S):
    rng = np.random.default_rng(2)
    states = {41: {"m": rng.standard_normal((3, 2)).astype(np.float32), "v": rng.random((3, 2)).astype(np.float32), "v_hat_max": None, "step": 7, "dims": [3, 2]},
              17: {"m": rng.standard_normal(4).astype(np.float32), "v": rng.random(4).astype(np.float32),
                   "v_hat_max": rng.random(4).astype(np.float32), "step": 7, "dims": [4]}}
    cfg = {"learning_rate": 1e-3, "beta1": 0.9, "beta2": 0.999, "eps": 1e-8, "weight_decay": 0.01, "amsgrad": True}
    fields = S.adam_fields(cfg, states, 7, [41, 17])
    for enc, dec in ((S.fields_to_binary, S.binary_to_fields), (S.fields_to_json, S.json_to_fields)):
        config, st, step_count, order = S.adam_from_fields(dec(enc(fields)))
        assert step_count == 7 and order == [41, 17] and config["amsgrad"] is True
        assert np.float32(config["learning_rate"]) == np.float32(1e-3) and np.float32(config["weight_decay"]) == np.float32(0.01)
        for pid in (41, 17):
            for k in ("m", "v"):
                assert np.array_equal(st[pid][k], states[pid][k]) and st[pid][k].shape == states[pid][k].shape
            assert st[pid]["step"] == 7
        assert st[41]["v_hat_max"] is None and np.array_equal(st[17]["v_hat_max"], states[17]["v_hat_max"])
    # the layout of the JSON form (optimizers/adam/serialization.rs:702-717): tensors embedded as objects, ids as keys
    d = json.loads(S.fields_to_json(fields))
    assert set(d) == {"config", "states", "step_count", "insertion_order"} and set(d["states"]) == {"41", "17"}
    assert d["states"]["41"]["v_hat_max"] is None and d["states"]["17"]["m"]["shape"]["dims"] == [4]
    assert d["config"]["learning_rate"] == pytest.approx(1e-3) and d["insertion_order"] == [41, 17]
    # in the binary form a state's tensors are JSON-object fields (tag 14), as core/impls.rs:416-427 makes them
    assert b"\x0e" + struct.pack("<I", len(S.fields_to_json(S.tensor_fields(states[17]["m"], [4], False)))) in S.fields_to_binary(fields)


def test_literals_the_reference_own_tests_hold(S):
    """What the reference's serialization unit tests write out literally, replayed through this codec: the only
    reference-held vectors there are for the format (no file written by the reference can be produced here).
    JSON field text: serialization/json/structs.rs:457-472 (every scalar kind this codec writes) and :487-490 (string
    escapes); compact object text: serialization/json/formatter.rs:336.  Binary primitives: an empty string is four zero
    bytes and an absent optional one zero byte (binary/reader.rs:741-750), the magic number's first byte on disk is
    0x42 (binary/header.rs:493, little endian) and the header is 24 bytes (binary/header.rs:519-523)."""
    text = S.fields_to_json([("bool_field", S.fv_bool(True)), ("usize_field", S.fv_usize(42)), ("f32_field", S.fv_f32(np.float32(np.pi))),
                             ("string_field", S.fv_string("Hello, World!")), ("json_field", S.fv_string('{"nested": "value"}'))])
    for want in ('"bool_field":true', '"usize_field":42', '"f32_field":3.1415927', '"string_field":"Hello, World!"',
                 '"json_field":"{\\"nested\\": \\"value\\"}"'):
        assert want in text, want
    text = S.fields_to_json([("quotes", S.fv_string('Hello "World"')), ("newlines", S.fv_string("Line1\nLine2")),
                             ("tabs", S.fv_string("Tab\there")), ("backslashes", S.fv_string("Path\\to\\file"))])
    for want in ('"quotes":"Hello \\"World\\""', '"newlines":"Line1\\nLine2"', '"tabs":"Tab\\there"', '"backslashes":"Path\\\\to\\\\file"'):
        assert want in text, want
    assert S.fields_to_json([("name", S.fv_string("test")), ("value", S.fv_usize(42))]) == '{"name":"test","value":42}'
    # and read back to the same values
    back = S.json_to_fields(text)
    assert back["quotes"] == 'Hello "World"' and back["newlines"] == "Line1\nLine2" and back["backslashes"] == "Path\\to\\file"
    # binary primitives
    blob = S.fields_to_binary([("s", S.fv_string("")), ("o", S.fv_optional(None))])
    assert len(blob) - 24 == struct.unpack("<Q", blob[12:20])[0] and blob[:4] == bytes([0x42, 0x5F, 0x53, 0x54])
    body = blob[24:]
    assert body == struct.pack("<Q", 2) + s_("s") + b"\x0c" + b"\x00\x00\x00\x00" + s_("o") + b"\x11" + b"\x00"
    got = S.binary_to_fields(blob)
    assert got["s"] == "" and got["o"] is None
