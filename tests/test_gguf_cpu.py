"""The GGUF reader and the host-side loader pieces, without a GPU.

The cases follow the reference's reader tests (src/loader/gguf.rs:694-980): a small file the test writes itself
(no model files exist here), aligned tensor data read back without reordering, expert shapes, untagged files,
skipped arrays, and the rejections (magic, truncation, alignment, block size, unknown type, overlap, ranges).
Q3_K rewritten as Q6_K keeps every value (src/hybrid/iq_tests.rs:1502-1527); the Q8_0 row quantiser follows
`quantize_row` (src/hybrid/weights.rs:1397-1415).
"""
import os
import struct

import numpy as np
import pytest

from ferrum_b200 import _lib
from oracle import ref

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def S():
    if not os.path.exists(_lib.LIB_PATH):
        from ferrum_b200 import build
        build.build()
    from ferrum_b200 import surface
    return surface


def gstr(s: str) -> bytes:
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def meta_u32(key, v):
    return gstr(key) + struct.pack("<II", 4, v)


def meta_str(key, v):
    return gstr(key) + struct.pack("<I", 8) + gstr(v)


def meta_str_array(key, items):
    return gstr(key) + struct.pack("<IIQ", 9, 8, len(items)) + b"".join(gstr(i) for i in items)


def meta_i32_array(key, items):
    return gstr(key) + struct.pack("<IIQ", 9, 5, len(items)) + b"".join(struct.pack("<i", i) for i in items)


def gguf_bytes(tensors, metadata=None, alignment=32, version=3, architecture=True, quant_version=True, payload_fill=None):
    """`tensors`: list of (name, dims, type_id, offset, payload bytes or None)."""
    md = list(metadata or [])
    if architecture:
        md.insert(0, meta_str("general.architecture", "test"))
    if quant_version:
        md.append(meta_u32("general.quantization_version", 2))
    if alignment != 32:
        md.append(meta_u32("general.alignment", alignment))
    out = b"GGUF" + struct.pack("<IQQ", version, len(tensors), len(md)) + b"".join(md)
    for name, dims, type_id, offset, _ in tensors:
        out += gstr(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", type_id, offset)
    out += b"\0" * ((-len(out)) % alignment)
    data = bytearray()
    for name, dims, type_id, offset, payload in tensors:
        if payload is None:
            continue
        if len(data) < offset + len(payload):
            data += b"\0" * (offset + len(payload) - len(data))
        data[offset:offset + len(payload)] = payload
    return out + bytes(data)


def write(tmp_path, name, data):
    p = tmp_path / name
    p.write_bytes(data)
    return str(p)


def test_reads_aligned_q8_0_tensor_without_reordering_payload(S, tmp_path):
    payload = bytes([1]) * 68
    f = S.GgufFile(write(tmp_path, "a.gguf", gguf_bytes([("w", [32, 2], 8, 0, payload)])))
    t = f.tensor("w")
    assert t["type_id"] == 8 and t["byte_len"] == 68 and t["dimensions"] == [32, 2]
    assert f.version == 3 and f.alignment == 32 and f.tensor_data_offset % 32 == 0
    assert bytes(f.read_tensor("w")) == payload
    assert f.metadata_string("general.architecture") == "test"
    assert f.metadata_u64("general.quantization_version") == 2
    with pytest.raises(S.GgufError, match="missing tensor"):
        f.tensor("nope")


def test_tensors_are_listed_in_name_order_and_offsets_are_relative_to_the_data_section(S, tmp_path):
    a, b = bytes(range(144)), bytes(reversed(range(210)))
    data = gguf_bytes([("zeta.weight", [256, 1], 12, 0, a), ("alpha.weight", [256, 1], 14, 160, b)])
    f = S.GgufFile(write(tmp_path, "b.gguf", data))
    assert [t["name"] for t in f.tensors()] == ["alpha.weight", "zeta.weight"]
    assert bytes(f.read_tensor("zeta.weight")) == a and bytes(f.read_tensor("alpha.weight")) == b
    assert f.file_len == len(data)


def test_expert_tensor_shape_is_gguf_order(S, tmp_path):
    # dims [cols, rows, experts]; 2048 x 4 x 2 of Q4_K = 8 * 2 * 8 blocks
    payload = bytes(144 * 64)
    f = S.GgufFile(write(tmp_path, "e.gguf", gguf_bytes([("blk.0.ffn_gate_exps.weight", [2048, 4, 2], 12, 0, payload)])))
    t = f.tensor("blk.0.ffn_gate_exps.weight")
    assert t["dimensions"] == [2048, 4, 2] and t["byte_len"] == 144 * 64


def test_an_untagged_file_opens_only_on_request(S, tmp_path):
    name = "model.diffusion_model.blocks.0." + "x" * 60 + ".weight"
    assert len(name) > 64
    data = gguf_bytes([(name, [32, 1], 0, 0, bytes(128))], architecture=False, quant_version=False)
    path = write(tmp_path, "u.gguf", data)
    with pytest.raises(S.GgufError):
        S.GgufFile(path)
    f = S.GgufFile(path, require_architecture=False)
    assert f.tensor(name)["dimensions"] == [32, 1]


def test_skipping_arrays_keeps_everything_else(S, tmp_path):
    md = [meta_str_array("tokenizer.ggml.tokens", ["a", "bc", "def"]), meta_i32_array("tokenizer.ggml.token_type", [1, 2, 3]),
          meta_u32("test.block_count", 7)]
    path = write(tmp_path, "s.gguf", gguf_bytes([("w", [32, 1], 0, 0, bytes([7]) * 128)], metadata=md, quant_version=False))
    full, skim = S.GgufFile(path), S.GgufFile(path, skip_arrays_over=2)
    assert full.metadata_array("tokenizer.ggml.tokens") == (8, 3, 3)
    assert skim.metadata_array("tokenizer.ggml.tokens") == (8, 3, 0)
    assert skim.metadata_array("tokenizer.ggml.token_type") == (5, 3, 0)
    assert skim.metadata_u64("test.block_count") == 7
    assert skim.tensor("w") == full.tensor("w")
    assert bytes(skim.read_tensor("w")) == bytes([7]) * 128


def test_rejects_bad_magic_and_truncated_header(S, tmp_path):
    good = gguf_bytes([("w", [32, 1], 8, 0, bytes(34))])
    with pytest.raises(S.GgufError, match="magic"):
        S.GgufFile(write(tmp_path, "m.gguf", b"GGML" + good[4:]))
    with pytest.raises(S.GgufError):
        S.GgufFile(write(tmp_path, "t.gguf", b"GGUF\x03\0"))
    with pytest.raises(S.GgufError, match="version"):
        S.GgufFile(write(tmp_path, "v.gguf", b"GGUF" + struct.pack("<I", 1) + good[8:]))


def test_rejects_unaligned_offsets_and_non_block_dimensions(S, tmp_path):
    with pytest.raises(S.GgufError, match="not aligned"):
        S.GgufFile(write(tmp_path, "o.gguf", gguf_bytes([("w", [32, 1], 8, 8, bytes(34))])))
    with pytest.raises(S.GgufError, match="block size"):
        S.GgufFile(write(tmp_path, "d.gguf", gguf_bytes([("w", [48, 1], 8, 0, bytes(51))])))


def test_rejects_unknown_types_overlaps_and_ranges_past_the_file(S, tmp_path):
    with pytest.raises(S.GgufError, match="unsupported GGML tensor type 99"):
        S.GgufFile(write(tmp_path, "q.gguf", gguf_bytes([("w", [32, 1], 99, 0, bytes(34))])))
    two = [("a", [32, 2], 8, 0, bytes(68)), ("b", [32, 1], 8, 32, bytes(34))]
    with pytest.raises(S.GgufError, match="ranges overlap"):
        S.GgufFile(write(tmp_path, "l.gguf", gguf_bytes(two)))
    whole = gguf_bytes([("w", [256, 4], 12, 0, bytes(576))])
    with pytest.raises(S.GgufError, match="exceeds file length"):
        S.GgufFile(write(tmp_path, "r.gguf", whole[:-100]))  # a truncated tensor
    with pytest.raises(S.GgufError, match="quantization_version"):
        S.GgufFile(write(tmp_path, "n.gguf", gguf_bytes([("w", [32, 1], 8, 0, bytes(34))], quant_version=False)))
    with pytest.raises(S.GgufError, match="duplicate tensor name"):
        S.GgufFile(write(tmp_path, "p.gguf", gguf_bytes([("w", [32, 1], 8, 0, bytes(34)), ("w", [32, 1], 8, 64, bytes(34))])))


def test_block_sizes_match_the_ggml_layouts(S):
    L = _lib.load()
    import ctypes as C
    want = {0: (1, 4), 1: (1, 2), 2: (32, 18), 8: (32, 34), 10: (256, 84), 11: (256, 110), 12: (256, 144), 13: (256, 176),
            14: (256, 210), 15: (256, 292), 21: (256, 110), 23: (256, 136), 30: (1, 2), 42: (64, 18)}
    for type_id, (el, by) in want.items():
        e, b = C.c_uint32(), C.c_uint32()
        assert L.fq_block_layout(type_id, C.byref(e), C.byref(b)) == _lib.OK
        assert (e.value, b.value) == (el, by), type_id
    assert L.fq_block_layout(4, C.byref(e), C.byref(b)) == _lib.ERR_GGUF  # a removed encoding


def test_q3_k_rewritten_as_q6_k_keeps_every_value(S):
    blocks = 64
    q3 = ref.random_blocks(ref.Q3_K, blocks, seed=5)
    q6 = S.q3k_to_q6k(q3)
    a, b = ref.dequant(ref.Q3_K, q3), ref.dequant(ref.Q6_K, q6)
    assert (a != 0).any()
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_q8_0_row_quantiser_follows_ggml(S):
    rng = np.random.default_rng(3)
    x = np.concatenate([rng.standard_normal(32 * 50).astype(np.float32) * 3, np.zeros(32, dtype=np.float32),
                        np.array([0.5, -0.5, 1.5, 2.5] * 8, dtype=np.float32)])
    got = S.quantize_q8_0(x).reshape(-1, 34)
    xb = x.reshape(-1, 32)
    amax = np.abs(xb).max(axis=1)
    d = (amax / np.float32(127.0)).astype(np.float32)
    inv = np.where(d != 0, np.float32(1.0) / np.where(d != 0, d, np.float32(1)), np.float32(0)).astype(np.float32)
    scaled = (xb * inv[:, None]).astype(np.float32)
    q = np.where(scaled >= 0, np.floor(scaled + np.float32(0.5)), np.ceil(scaled - np.float32(0.5))).astype(np.int8)  # f32::round: ties away
    assert np.array_equal(got[:, :2].copy().view(np.float16).ravel(), d.astype(np.float16))
    assert np.array_equal(got[:, 2:].view(np.int8), q)
    # the blocks pass the loader's payload check and decode back close to the input
    assert ref.validate(ref.Q8_0, got.ravel()) == 0
    back = ref.dequant(ref.Q8_0, got.ravel()).reshape(-1, 32)
    assert np.abs(back - xb).max() <= (amax / 127.0).max() * 0.51 + 1e-3


@pytest.mark.parametrize("rows,cols", [(5, 512), (9, 1024)])
def test_q5k_decoder_matches_closed_form(rows, cols):
    got = ref.dequant(ref.Q5_K, ref.qk_q5k_packed(rows, cols)).reshape(rows, cols)
    want = np.array([[ref.qk_q5k_value(r, c) for c in range(cols)] for r in range(rows)], dtype=np.float32)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
