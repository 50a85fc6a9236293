"""The CPU oracle against the reference's own known-answer material (no GPU).

The reference stores no golden outputs for this path; its tests compute expectations from closed-form
per-element formulas (src/ops/transformer.rs:2920-2956, 4153-4169, 1707-1710).  Those formulas are
restated in ``oracle/ref.py`` independently of the block decoders in ``oracle/fq_ref.c``; demanding
bit-equality between the two pins the decoders' bit layout, value order and operation order.
"""
import json
import os

import numpy as np
import pytest

from oracle import ref

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def test_f16_conversions_match_ieee():
    allh = np.arange(65536, dtype=np.uint16)
    got = np.array([ref.lib().fqo_f16_to_f32(int(h)) for h in allh], dtype=np.float32)
    want = allh.view(np.float16).astype(np.float32)
    ok = ~np.isnan(want)
    assert np.array_equal(bits(got)[ok], bits(want)[ok])
    assert np.isnan(got[~ok]).all()
    rng = np.random.default_rng(1)
    xs = np.concatenate([rng.standard_normal(4000).astype(np.float32) * s for s in (1e-8, 1e-5, 1e-3, 1, 100, 7e4)]
                        + [np.array([65504, 65519.9, 65520, 65536, 1e-30, 2 ** -25, 2 ** -24, 6.1e-5, np.inf, -np.inf, 0, -0.0],
                                    dtype=np.float32)])
    got = np.array([ref.lib().fqo_f32_to_f16(float(v)) for v in xs], dtype=np.uint16)
    with np.errstate(over="ignore"):
        want = xs.astype(np.float16).view(np.uint16)
    assert np.array_equal(got, want)


def test_bf16_rounding_is_rne_with_quiet_nan():
    # src/hybrid/draft/gguf.rs:362-369
    vals = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.3895314e38, 1e-40], dtype=np.float32)
    got = np.array([ref.lib().fqo_f32_to_bf16(float(v)) for v in vals], dtype=np.uint16)
    assert np.array_equal(got, ref.to_bf16(vals))
    assert got[0] == 0x3F80 and got[1] == 0x3F80 and got[2] == 0x3F82  # ties to even, both directions
    nan = np.frombuffer(np.uint32(0x7F800001).tobytes(), dtype=np.float32)[0]
    assert ref.lib().fqo_f32_to_bf16(float(nan)) & 0x7FC0 == 0x7FC0


@pytest.mark.parametrize("rows,cols", [(5, 512), (65, 512)])
def test_q4k_decoder_matches_closed_form(rows, cols):
    got = ref.dequant(ref.Q4_K, ref.qk_q4k_packed(rows, cols)).reshape(rows, cols)
    want = np.array([[ref.qk_q4k_value(r, c) for c in range(cols)] for r in range(rows)], dtype=np.float32)
    assert np.array_equal(bits(got), bits(want))


def test_q6k_decoder_matches_both_closed_forms():
    got = ref.dequant(ref.Q6_K, ref.qk_q6k_packed(5, 512)).reshape(5, 512)
    want = np.array([[ref.qk_q6k_value(r, c) for c in range(512)] for r in range(5)], dtype=np.float32)
    assert np.array_equal(bits(got), bits(want))
    got = ref.dequant(ref.Q6_K, ref.q6_packed(6, 768)).reshape(6, 768)
    want = np.array([[ref.q6_value(r, c) for c in range(768)] for r in range(6)], dtype=np.float32)
    assert np.array_equal(bits(got), bits(want))


def test_q8_0_decoder_matches_closed_form():
    got = ref.dequant(ref.Q8_0, ref.q8_packed(7, 128)).reshape(7, 128)
    want = np.array([[ref.q8_value(r, c) for c in range(128)] for r in range(7)], dtype=np.float32)
    assert np.array_equal(bits(got), bits(want))


def test_legacy_expected_values_match_f32_sequential_matmul():
    # `expected` of src/ops/transformer.rs:2964-2980 on the (5, 512) fixture, M = 1, 2, 3, 4, 5, 7.
    packed = ref.qk_q4k_packed(5, 512)
    for m in (1, 2, 3, 4, 5, 7):
        x = ref.qk_input(m, 512)
        got = ref.matmul(ref.Q4_K, packed, 5, 512, x, m, mode=1)
        want = ref.closed_form_expected(ref.qk_q4k_value, x, m, 5, 512)
        assert np.array_equal(bits(got), bits(want))
    x = ref.q6_input(1, 768)
    got = ref.matmul(ref.Q6_K, ref.q6_packed(6, 768), 6, 768, x, 1, mode=1)
    assert np.array_equal(bits(got), bits(ref.closed_form_expected(ref.q6_value, x, 1, 6, 768)))
    x = ref.q8_input(2, 128)
    got = ref.matmul(ref.Q8_0, ref.q8_packed(7, 128), 7, 128, x, 2, mode=1)
    assert np.array_equal(bits(got), bits(ref.closed_form_expected(ref.q8_value, x, 2, 7, 128)))


def test_golden_vectors():
    """Committed known-answer vectors (tests/golden/make_golden.py): closed-form weights and the
    f32-sequential outputs of the reference's fixtures, computed without the C oracle."""
    with open(os.path.join(GOLDEN, "closed_form.json")) as f:
        g = json.load(f)
    for case in g["cases"]:
        fmt = {"q4_k": ref.Q4_K, "q5_k": ref.Q5_K, "q6_k": ref.Q6_K, "q8_0": ref.Q8_0}[case["format"]]
        packed = np.array(case["packed_u8"], dtype=np.uint8)
        rows, cols, m = case["rows"], case["cols"], case["m"]
        dense = ref.dequant(fmt, packed)
        assert np.array_equal(bits(dense), np.array(case["dense_bits"], dtype=np.uint32))
        x = np.array(case["x_bits"], dtype=np.uint32).view(np.float32)
        y = ref.matmul(fmt, packed, rows, cols, x, m, mode=1)
        assert np.array_equal(bits(y).ravel(), np.array(case["y_f32seq_bits"], dtype=np.uint32))


def test_xorshift_generators_follow_the_reference():
    # src/diffusion/tests.rs:770-794: scales land in [0.002, 0.004] and everything is finite.
    for fmt in (ref.Q4_K, ref.Q6_K):
        b = ref.xorshift_kquant_blocks(fmt, 8)
        assert ref.validate(fmt, b) == 0
        dense = ref.dequant(fmt, b)
        assert np.isfinite(dense).all() and np.abs(dense).max() > 0
    x = ref.xorshift_f32(1000, 31)
    assert x.min() >= -1 and x.max() < 1 and abs(float(x.mean())) < 0.1


def test_payload_validation_follows_the_loader():
    # src/quantization.rs:212-261
    b = ref.random_matrix(ref.Q4_K, 2, 256).copy()
    assert ref.validate(ref.Q4_K, b) == 0
    assert ref.validate(ref.Q4_K, b[:-1]) == 1
    bad = b.copy(); bad[0:2] = np.frombuffer(np.float16(np.inf).tobytes(), dtype=np.uint8)
    assert ref.validate(ref.Q4_K, bad) == 2
    q8 = ref.random_matrix(ref.Q8_0, 2, 64).copy()
    assert ref.validate(ref.Q8_0, q8) == 0
    bad = q8.copy(); bad[5] = 0x80
    assert ref.validate(ref.Q8_0, bad) == 3
    bad = q8.copy(); bad[0:2] = np.frombuffer(np.float16(-1.0).tobytes(), dtype=np.uint8)
    assert ref.validate(ref.Q8_0, bad) == 2
    q6 = ref.random_matrix(ref.Q6_K, 1, 256).copy()
    bad = q6.copy(); bad[208:210] = np.frombuffer(np.float16(np.nan).tobytes(), dtype=np.uint8)
    assert ref.validate(ref.Q6_K, bad) == 2


def test_routing_oracle_matches_a_stable_sort():
    # src/hybrid/engine.rs:4947-5041: 256 experts, top-6, 3 tokens, logits 3 * U(-1, 1).
    experts, used, hidden, m = 256, 6, 2048, 3
    logits = ref.xorshift_f32(m * experts, 21) * np.float32(3.0)
    x = ref.xorshift_f32(m * hidden, 22)
    sw = ref.xorshift_f32(hidden, 23)
    for sigmoid, norm, gate in [(True, True, False), (False, True, True), (True, False, True)]:
        ids, w, g = ref.moe_route(logits, x, sw, experts, used, hidden, m, sigmoid, norm, gate)
        for t in range(m):
            row = logits[t * experts:(t + 1) * experts].astype(np.float64)
            scores = 1 / (1 + np.exp(-row)) if sigmoid else np.exp(row - row.max()) / np.exp(row - row.max()).sum()
            order = sorted(range(experts), key=lambda i: (-scores[i], i))[:used]
            assert list(ids[t * used:(t + 1) * used]) == order
            want = scores[order] / scores[order].sum() if norm else scores[order]
            assert np.abs(w[t * used:(t + 1) * used] - want).max() < 1e-5
            if gate:
                dot = float(np.dot(x[t * hidden:(t + 1) * hidden].astype(np.float64), sw.astype(np.float64)))
                assert abs(g[t] - 1 / (1 + np.exp(-dot))) < 1e-4
            else:
                assert g[t] == 1.0


def test_map_gather_combine_oracles():
    ids = np.array([2, 0, 1, 1, 2, 0, 0, 2], dtype=np.uint32)
    offsets, sorted_, position = ref.moe_map(ids, 3)
    assert list(offsets) == [0, 3, 5, 8]
    assert list(sorted_) == [1, 5, 6, 2, 3, 0, 4, 7]
    assert all(sorted_[position[r]] == r for r in range(8))
    x = np.arange(4 * 6, dtype=np.float32).reshape(4, 6)
    xg = ref.moe_gather(x, sorted_, 6, 2)
    assert np.array_equal(xg, x[sorted_ // 2])
    down = np.random.default_rng(0).standard_normal((8, 6)).astype(np.float32)
    w = np.random.default_rng(1).random(8).astype(np.float32)
    shared = np.ones((4, 6), dtype=np.float32)
    gate = np.full(4, 0.5, dtype=np.float32)
    out = ref.moe_combine(down, w, position, shared, gate, 6, 2, 4, identity=False)
    want = np.stack([w[2 * t] * down[position[2 * t]] + w[2 * t + 1] * down[position[2 * t + 1]] + 0.5 for t in range(4)])
    assert np.allclose(out, want, atol=1e-6)


def test_threaded_gemv_agrees_with_the_parity_oracle():
    for fmt in (ref.Q4_K, ref.Q6_K, ref.Q8_0):
        packed = ref.random_matrix(fmt, 37, 512, seed=3)
        x = np.random.default_rng(4).standard_normal((3, 512)).astype(np.float32)
        want = ref.matmul(fmt, packed, 37, 512, x, 3, mode=0)
        got = ref.gemv_threads(fmt, packed, 37, 512, x, 3, threads=3)
        assert ref.rel_err(got, want) < 1e-5


@pytest.mark.parametrize("fmt", [ref.IQ4_NL, ref.IQ4_XS])
def test_iq4_decoders_match_the_format_definition(fmt):
    """IQ4_NL (`dequant_iq4_nl`, src/hybrid/iq_tests.rs:1606-1618) and IQ4_XS (`dequantize_iq4_xs`,
    src/metal/shaders/hybrid.metal:580-596): the C block loops against an array restatement, bit for bit, on
    random blocks and on a block that walks the codebook and every 6-bit scale."""
    packed = ref.random_blocks(fmt, 64, seed=5)
    assert np.array_equal(ref.dequant(fmt, packed).view(np.uint32), ref.iq4_closed_form(fmt, packed).view(np.uint32))
    el, bb = ref.LAYOUT[fmt]
    if fmt == ref.IQ4_NL:
        blk = np.zeros(bb, dtype=np.uint8)
        blk[0:2] = np.array([0.5], dtype=np.float16).view(np.uint8)
        blk[2:18] = np.arange(16, dtype=np.uint8) | (np.arange(15, -1, -1, dtype=np.uint8) << 4)
        got = ref.dequant(fmt, blk)
        assert np.array_equal(got[:16], 0.5 * ref.IQ4_VALUES) and np.array_equal(got[16:], 0.5 * ref.IQ4_VALUES[::-1])
    else:
        blk = np.zeros(bb, dtype=np.uint8)
        blk[0:2] = np.array([0.25], dtype=np.float16).view(np.uint8)
        ls = np.array([0, 63, 32, 33, 17, 48, 5, 60])  # sub-block scales
        blk[2:4] = np.array([sum(int(v >> 4) << (2 * i) for i, v in enumerate(ls))], dtype=np.uint16).view(np.uint8)
        for i in range(4):
            blk[4 + i] = (ls[2 * i] & 15) | ((ls[2 * i + 1] & 15) << 4)
        blk[8:136] = np.tile(np.arange(16, dtype=np.uint8) | (np.arange(15, -1, -1, dtype=np.uint8) << 4), 8)
        got = ref.dequant(fmt, blk).reshape(8, 32)
        for ib in range(8):
            want = np.float32(0.25) * np.float32(ls[ib] - 32)
            assert np.array_equal(got[ib, :16], want * ref.IQ4_VALUES) and np.array_equal(got[ib, 16:], want * ref.IQ4_VALUES[::-1])
