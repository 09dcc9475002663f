"""GGUF reader (C++ behind include/strix_gguf.h) on CPU: the reference's own parser tests
(crates/strix-models/src/gguf.rs:381-452) replayed, then the edge cases its parser code handles:
every truncation is an error and never a read past the buffer, versions, alignment, typed metadata
and its widening rules, arrays, refused inputs."""
import struct

import numpy as np
import pytest


@pytest.fixture(scope="module")
def gguf(pkg):
    from strix_rs_b200 import gguf as g
    return g


def ref_test_file(gguf):
    # gguf.rs:385-430: one string, one u32, one F16 tensor [1.5, -0.5]
    raw = np.array([1.5, -0.5], dtype=np.float16).tobytes()
    return gguf.gguf_bytes({"general.architecture": "test", "test.block_count": gguf.Typed(4, 7)},
                           [("w", [2], gguf.GGML_F16, raw)]), raw


def test_ref_parses_metadata_and_tensor(gguf, tmp_path):
    b, raw = ref_test_file(gguf)
    # the byte string is what the reference's test builds by hand: check the fixed prefix
    assert b[:24] == struct.pack("<IIQQ", 0x46554747, 3, 1, 2)
    assert len(b) % 32 == 0 and b[160:164] == raw        # header padded to 32, then the tensor data (padded too)
    p = tmp_path / "t.gguf"
    p.write_bytes(b)
    for g in (gguf.GgufFile(path=p), gguf.GgufFile(data=b)):
        assert g.architecture() == "test"
        assert g.meta_u64("test.block_count") == 7
        (info,) = g.tensors()
        assert info["name"] == "w" and info["dims"] == [2] and info["ggml_type"] == gguf.GGML_F16
        got = g.tensor_bytes("w").tobytes()
        assert np.frombuffer(got, dtype=np.float16).astype(np.float32).tolist() == [1.5, -0.5]
        g.close()


def test_ref_bad_magic_errors(gguf, tmp_path):
    p = tmp_path / "bad.gguf"
    p.write_bytes(bytes(64))
    with pytest.raises(gguf.GgufError, match="not a GGUF file"):
        gguf.GgufFile(path=p)
    with pytest.raises(gguf.GgufError):
        gguf.GgufFile(path=tmp_path / "missing.gguf")


def test_every_truncation_is_an_error(gguf):
    b, _ = ref_test_file(gguf)
    g = gguf.GgufFile(data=b)
    header_end = g.data_offset
    g.close()
    for n in range(0, header_end):
        with pytest.raises(gguf.GgufError):
            gguf.GgufFile(data=b[:n])
    # header complete, tensor data short: the file opens, the tensor's bytes are refused (gguf.rs:224-230)
    g = gguf.GgufFile(data=b[:header_end + 2])
    with pytest.raises(gguf.GgufError, match="past EOF"):
        g.tensor_bytes("w")
    with pytest.raises(gguf.GgufError, match="not found"):
        g.tensor_bytes("nope")
    assert g.tensor_info("nope") is None


def test_versions_and_alignment(gguf):
    raw = bytes(range(36))
    for version in (2, 3):
        assert gguf.GgufFile(data=gguf.gguf_bytes({}, [("t", [32], gguf.GGML_Q8_0, raw[:34])], version=version)).version == version
    for version in (1, 4):
        with pytest.raises(gguf.GgufError, match="GGUF version %d" % version):
            gguf.GgufFile(data=gguf.gguf_bytes({}, [], version=version))
    for align in (8, 64, 4096):
        t = [("a", [32], gguf.GGML_Q8_0, raw[:34]), ("b", [32], gguf.GGML_Q4_0, raw[:18])]
        g = gguf.GgufFile(data=gguf.gguf_bytes({"k": 1}, t, alignment=align))
        assert g.alignment == align and g.data_offset % align == 0
        assert g.tensor_info("b")["offset"] % align == 0
        assert g.tensor_bytes("a").tobytes() == raw[:34] and g.tensor_bytes("b").tobytes() == raw[:18]
    # no general.alignment: 32 (gguf.rs:20, 163-167)
    assert gguf.GgufFile(data=gguf.gguf_bytes({}, [])).alignment == 32


def test_metadata_kinds_and_widening(gguf):
    T = gguf.Typed
    meta = {"u8": T(0, 200), "i8": T(1, -3), "i8p": T(1, 5), "u16": T(2, 60000), "i16": T(3, -2), "u32": T(4, 4000000000),
            "i32": T(5, 9), "f32": T(6, 1e-6), "bool": T(7, 1), "str": T(8, "héllo"), "u64": T(10, 2 ** 40),
            "i64": T(11, -(2 ** 40)), "f64": T(12, 0.25), "strs": T(9, ["a", "bc", ""], elem_type=8),
            "ints": T(9, [1, 2, 3], elem_type=5), "empty": T(9, [], elem_type=6)}
    g = gguf.GgufFile(data=gguf.gguf_bytes(meta, []))
    assert [k for k, _ in g.meta_keys()] == list(meta)
    # as_u64: unsigned kinds, signed kinds only when non-negative, nothing else (gguf.rs:43-56)
    assert g.meta_u64("u8") == 200 and g.meta_u64("u16") == 60000 and g.meta_u64("u32") == 4000000000
    assert g.meta_u64("u64") == 2 ** 40 and g.meta_u64("i8p") == 5 and g.meta_u64("i32") == 9
    for k in ("i8", "i16", "i64", "f32", "bool", "str", "strs", "missing"):
        assert g.meta_u64(k) is None, k
    # as_f32: f32, f64, or whatever as_u64 accepts (gguf.rs:59-65)
    assert g.meta_f32("f32") == np.float32(1e-6) and g.meta_f32("f64") == 0.25 and g.meta_f32("u8") == 200.0
    assert g.meta_f32("i8") is None and g.meta_f32("str") is None
    assert g.meta_str("str") == "héllo" and g.meta_str("u8") is None
    assert g.meta_array_len("strs") == (3, 8) and g.meta_array_len("ints") == (3, 5) and g.meta_array_len("empty") == (0, 6)
    assert g.meta_array_len("u8") is None


def test_refused_inputs(gguf):
    T = gguf.Typed
    nested = T(9, [T(9, [1], elem_type=4)], elem_type=9)
    with pytest.raises(gguf.GgufError, match="nested arrays"):
        gguf.GgufFile(data=gguf.gguf_bytes({"n": nested}, []))
    # an unknown metadata value type
    b = struct.pack("<IIQQ", 0x46554747, 3, 0, 1) + struct.pack("<Q", 1) + b"k" + struct.pack("<I", 13) + bytes(8)
    with pytest.raises(gguf.GgufError, match="value type 13"):
        gguf.GgufFile(data=b)
    # an unknown tensor type (IQ / TQ ids), as GgmlType::from_u32 refuses (ggml_quant.rs:41-64)
    with pytest.raises(gguf.GgufError, match="type id 16"):
        gguf.GgufFile(data=gguf.gguf_bytes({}, [("t", [256], 16, bytes(64))]))
    # a string length that runs past the file
    b = struct.pack("<IIQQ", 0x46554747, 3, 0, 1) + struct.pack("<Q", 2 ** 60) + b"k"
    with pytest.raises(gguf.GgufError, match="EOF"):
        gguf.GgufFile(data=b)
    # an array count that runs past the file
    b = struct.pack("<IIQQ", 0x46554747, 3, 0, 1) + struct.pack("<Q", 1) + b"k" + struct.pack("<IIQ", 9, 4, 2 ** 61)
    with pytest.raises(gguf.GgufError, match="EOF"):
        gguf.GgufFile(data=b)
    # alignment larger than the file: data offset past EOF (gguf.rs:169-171)
    with pytest.raises(gguf.GgufError, match="past EOF"):
        gguf.GgufFile(data=gguf.gguf_bytes({"general.alignment": T(4, 1 << 20)}, [])[:100])


def test_sizes_that_wrap_are_parse_errors(gguf):
    """Sizes in a file are untrusted: an element count whose product wraps, an offset near 2^64, a tensor that is
    not whole blocks and an alignment that overflows the data offset are errors, never a view whose dims and bytes
    disagree."""
    hdr = lambda n_t, n_kv: struct.pack("<IIQQ", 0x46554747, 3, n_t, n_kv)  # noqa: E731
    name = struct.pack("<Q", 1) + b"t"
    # dims 2^33 x 2^33: the product wraps to 0
    b = hdr(1, 0) + name + struct.pack("<I", 2) + struct.pack("<QQ", 1 << 33, 1 << 33) + struct.pack("<IQ", 0, 0) + bytes(64)
    with pytest.raises(gguf.GgufError, match="overflows"):
        gguf.GgufFile(data=b)
    # offset close to 2^64: data_offset + offset wraps
    b = hdr(1, 0) + name + struct.pack("<I", 1) + struct.pack("<Q", 32) + struct.pack("<IQ", 0, (1 << 64) - 8) + bytes(256)
    with pytest.raises(gguf.GgufError, match="overflows|past EOF"):
        gguf.GgufFile(data=b).tensor_bytes("t")
    # 40 elements of a 32-element block type
    b = hdr(1, 0) + name + struct.pack("<I", 1) + struct.pack("<Q", 40) + struct.pack("<IQ", 2, 0) + bytes(256)
    with pytest.raises(gguf.GgufError, match="whole blocks"):
        gguf.GgufFile(data=b).tensor_bytes("t")
    # general.alignment = 2^63 - 1 (the largest the reference's widening admits): the data offset lands past the file
    T = gguf.Typed
    with pytest.raises(gguf.GgufError, match="overflows|past EOF"):
        gguf.GgufFile(data=gguf.gguf_bytes({"general.alignment": T(10, (1 << 63) - 1)}, []))


def test_block_geometry_table(gguf, orc):
    # ggml_quant.rs:88-124
    want = {0: (1, 4), 1: (1, 2), 2: (32, 18), 3: (32, 20), 6: (32, 22), 7: (32, 24), 8: (32, 34), 9: (32, 36),
            10: (256, 84), 11: (256, 110), 12: (256, 144), 13: (256, 176), 14: (256, 210), 15: (256, 292)}
    for ty in range(0, 40):
        assert (gguf.block_elems(ty), gguf.block_bytes(ty)) == want.get(ty, (0, 0))


def test_tensor_bytes_feed_the_oracle(gguf, orc, synth, tmp_path):
    """A synthetic model file: tensor bytes read back through the map dequantise to what went in."""
    in_dim, out_dim = 256, 24
    ts, raws = [], {}
    for name, ty in (("blk.0.attn_q.weight", synth.Q4_0), ("blk.0.ffn_down.weight", synth.Q8_0), ("output.weight", synth.Q6_K)):
        raws[name] = synth.quant(ty, 3, name, out_dim, in_dim)
        ts.append((name, [in_dim, out_dim], ty, raws[name].tobytes()))
    norm = synth.norm_weight(3, "n", in_dim)
    ts.append(("output_norm.weight", [in_dim], gguf.GGML_F32, norm.tobytes()))
    p = tmp_path / "m.gguf"
    gguf.write_gguf(p, {"general.architecture": "qwen3", "qwen3.block_count": 1, "qwen3.attention.layer_norm_rms_epsilon": 1e-6}, ts)
    with gguf.GgufFile(path=p) as g:
        assert g.architecture() == "qwen3" and g.meta_u64("qwen3.block_count") == 1
        assert g.meta_f32("qwen3.attention.layer_norm_rms_epsilon") == np.float32(1e-6)
        for name, ty in (("blk.0.attn_q.weight", synth.Q4_0), ("blk.0.ffn_down.weight", synth.Q8_0), ("output.weight", synth.Q6_K)):
            info = g.tensor_info(name)
            assert info["dims"] == [in_dim, out_dim] and info["ggml_type"] == ty
            b = g.tensor_bytes(name)
            np.testing.assert_array_equal(b, raws[name].reshape(-1))
            np.testing.assert_array_equal(orc.dequantize(ty, b, in_dim * out_dim), orc.dequantize(ty, raws[name], in_dim * out_dim))
        np.testing.assert_array_equal(np.frombuffer(g.tensor_bytes("output_norm.weight").tobytes(), np.float32), norm)
        g.advise_dontneed("output.weight")          # whole pages only; the bytes re-fault from the file
        np.testing.assert_array_equal(g.tensor_bytes("output.weight"), raws["output.weight"].reshape(-1))
