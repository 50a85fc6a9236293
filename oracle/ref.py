"""ctypes front end of the CPU oracle (``fq_ref.c``) plus the seeded input generators.

TEST INFRASTRUCTURE ONLY.  The shipped package (``ferrum_b200``) never imports this module;
the test-suite, the smoke check and the benchmark's CPU-baseline leg do.

The generators reproduce (a) the benchmark's block distributions (numpy ``default_rng(seed)``:
``d``/``dmin`` = fp16(|N(0,1)| * 1e-2), scale bytes and quant bytes uniform), (b) the reference's
xorshift random blocks (src/diffusion/tests.rs:770-794, src/hybrid/iq_tests.rs:1235-1262) and
(c) the reference's closed-form fixtures (src/ops/transformer.rs:2833-2903, 4102-4151, 1683-1705).
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

Q8_0, Q3_K, Q4_K, Q5_K, Q6_K, IQ4_NL, IQ4_XS = 8, 11, 12, 13, 14, 20, 23
LAYOUT = {Q8_0: (32, 34), Q3_K: (256, 110), Q4_K: (256, 144), Q5_K: (256, 176), Q6_K: (256, 210), IQ4_NL: (32, 18), IQ4_XS: (256, 136)}  # format -> (elements, bytes)
NAME = {Q8_0: "q8_0", Q3_K: "q3_k", Q4_K: "q4_k", Q5_K: "q5_k", Q6_K: "q6_k", IQ4_NL: "iq4_nl", IQ4_XS: "iq4_xs"}

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libfq_ref.so")


def build(force: bool = False) -> str:
    """Compile ``fq_ref.c`` with the Makefile beside it (gcc, -ffp-contract=off)."""
    src = os.path.join(_HERE, "fq_ref.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libfq_ref.so"], stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        L = ctypes.CDLL(build())
        c = ctypes
        u8p, f32p, u32p = c.c_void_p, c.c_void_p, c.c_void_p
        L.fqo_f16_to_f32.restype = c.c_float
        L.fqo_f16_to_f32.argtypes = [c.c_uint16]
        L.fqo_f32_to_f16.restype = c.c_uint16
        L.fqo_f32_to_f16.argtypes = [c.c_float]
        L.fqo_f32_to_bf16.restype = c.c_uint16
        L.fqo_f32_to_bf16.argtypes = [c.c_float]
        L.fqo_validate.argtypes = [c.c_int, u8p, c.c_size_t]
        L.fqo_dequant.argtypes = [c.c_int, u8p, c.c_size_t, f32p]
        L.fqo_matmul_dense.argtypes = [f32p, c.c_size_t, c.c_size_t, f32p, c.c_size_t, c.c_int, f32p]
        L.fqo_matmul_dense.restype = None
        L.fqo_matmul.argtypes = [c.c_int, u8p, c.c_size_t, c.c_size_t, f32p, c.c_size_t, c.c_int, f32p]
        L.fqo_matmul_id.argtypes = [c.c_int, u8p, c.c_size_t, c.c_size_t, f32p, u32p, c.c_size_t,
                                    c.c_size_t, c.c_int, f32p]
        L.fqo_matmul_grouped.argtypes = [c.c_int, u8p, c.c_size_t, c.c_size_t, f32p, u32p, u32p,
                                         c.c_size_t, c.c_int, f32p]
        L.fqo_moe_route.argtypes = [f32p, f32p, f32p] + [c.c_int] * 7 + [u32p, f32p, f32p]
        L.fqo_moe_route.restype = None
        L.fqo_moe_map.argtypes = [u32p, c.c_int, c.c_int, u32p, u32p, u32p]
        L.fqo_moe_map.restype = None
        L.fqo_moe_gather.argtypes = [f32p, u32p, c.c_int, c.c_int, c.c_int, f32p]
        L.fqo_moe_gather.restype = None
        L.fqo_moe_combine.argtypes = [f32p, f32p, u32p, f32p, f32p] + [c.c_int] * 4 + [f32p]
        L.fqo_moe_combine.restype = None
        L.fqo_swiglu.argtypes = [f32p, f32p, c.c_size_t, f32p]
        L.fqo_swiglu.restype = None
        L.fqo_gemv_threads.argtypes = [c.c_int, u8p, c.c_size_t, c.c_size_t, f32p, c.c_size_t,
                                       c.c_int, f32p]
        _lib = L
    return _lib


def _p(a: np.ndarray) -> int:
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data


def _u8(b) -> np.ndarray:
    return np.ascontiguousarray(np.frombuffer(b, dtype=np.uint8) if not isinstance(b, np.ndarray) else b,
                                dtype=np.uint8)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _u32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint32)


# ------------------------------------------------------------------ oracle calls

def row_bytes(fmt: int, cols: int) -> int:
    el, bb = LAYOUT[fmt]
    assert cols % el == 0
    return cols // el * bb


def validate(fmt: int, packed) -> int:
    p = _u8(packed)
    return lib().fqo_validate(fmt, _p(p), p.size)


def dequant(fmt: int, packed) -> np.ndarray:
    """All blocks of ``packed`` decoded to fp32, in block order."""
    p = _u8(packed)
    el, bb = LAYOUT[fmt]
    assert p.size % bb == 0
    out = np.empty(p.size // bb * el, dtype=np.float32)
    assert lib().fqo_dequant(fmt, _p(p), p.size // bb, _p(out)) == 0
    return out


def matmul(fmt: int, packed, rows: int, cols: int, x, m: int, mode: int = 0) -> np.ndarray:
    """``y[m, rows]``; mode 0 = f64 accumulate, 1 = f32 sequential, 2 = bf16 operands and result."""
    p, x = _u8(packed), _f32(x)
    assert p.size == rows * row_bytes(fmt, cols) and x.size == m * cols
    y = np.empty((m, rows), dtype=np.float32)
    assert lib().fqo_matmul(fmt, _p(p), rows, cols, _p(x), m, mode, _p(y)) == 0
    return y


def matmul_id(fmt, packed, rows_e, cols, x, ids, x_div=1, mode=0) -> np.ndarray:
    p, x, ids = _u8(packed), _f32(x), _u32(ids)
    y = np.empty((ids.size, rows_e), dtype=np.float32)
    assert lib().fqo_matmul_id(fmt, _p(p), rows_e, cols, _p(x), _p(ids), ids.size, x_div, mode, _p(y)) == 0
    return y


def matmul_grouped(fmt, packed, rows_e, cols, x, offsets, slots=None, mode=0) -> np.ndarray:
    p, x, offsets = _u8(packed), _f32(x), _u32(offsets)
    groups = offsets.size - 1
    sl = _u32(slots) if slots is not None else None
    y = np.zeros((int(offsets[-1]), rows_e), dtype=np.float32)
    assert lib().fqo_matmul_grouped(fmt, _p(p), rows_e, cols, _p(x), _p(offsets),
                                    _p(sl) if sl is not None else None, groups, mode, _p(y)) == 0
    return y


def moe_route(logits, x, shared_w, experts, used, hidden, tokens, sigmoid, norm, shared_gate):
    logits, x, shared_w = _f32(logits), _f32(x), _f32(shared_w)
    ids = np.empty(tokens * used, dtype=np.uint32)
    w = np.empty(tokens * used, dtype=np.float32)
    g = np.empty(tokens, dtype=np.float32)
    lib().fqo_moe_route(_p(logits), _p(x), _p(shared_w), experts, used, hidden, tokens,
                        int(sigmoid), int(norm), int(shared_gate), _p(ids), _p(w), _p(g))
    return ids, w, g


def moe_map(ids, experts):
    ids = _u32(ids)
    offsets = np.empty(experts + 1, dtype=np.uint32)
    sorted_ = np.empty(ids.size, dtype=np.uint32)
    position = np.empty(ids.size, dtype=np.uint32)
    lib().fqo_moe_map(_p(ids), experts, ids.size, _p(offsets), _p(sorted_), _p(position))
    return offsets, sorted_, position


def moe_gather(x, sorted_, hidden, used):
    x, sorted_ = _f32(x), _u32(sorted_)
    xg = np.empty((sorted_.size, hidden), dtype=np.float32)
    lib().fqo_moe_gather(_p(x), _p(sorted_), hidden, used, sorted_.size, _p(xg))
    return xg


def moe_combine(down, weights, position, shared, gate, hidden, used, tokens, identity):
    down, weights, shared, gate = _f32(down), _f32(weights), _f32(shared), _f32(gate)
    position = _u32(position)
    out = np.empty((tokens, hidden), dtype=np.float32)
    lib().fqo_moe_combine(_p(down), _p(weights), _p(position), _p(shared), _p(gate), hidden, used,
                          tokens, int(identity), _p(out))
    return out


def swiglu(g, u):
    g, u = _f32(g), _f32(u)
    y = np.empty_like(g)
    lib().fqo_swiglu(_p(g), _p(u), g.size, _p(y))
    return y


def rmsnorm(x, w, eps) -> np.ndarray:
    """`reference::rmsnorm` (src/reference.rs:23-36): f64 sum of squares, 1 / sqrt(mean + eps), x * inv * w in f64,
    cast to f32.  `x` is [rows, n]."""
    x64, w64 = np.asarray(x, dtype=np.float64), np.asarray(w, dtype=np.float64)
    inv = 1.0 / np.sqrt((x64 ** 2).sum(axis=-1, keepdims=True) / w64.size + np.float64(np.float32(eps)))
    return (x64 * inv * w64).astype(np.float32)


def argmax_first(x) -> np.ndarray:
    """`h_argmax` (src/metal/shaders/hybrid.metal:2214-2243): the index of the first maximum of each row."""
    return np.argmax(np.asarray(x, dtype=np.float32), axis=-1).astype(np.uint32)


def topk_blocks(x) -> tuple:
    """`h_topk_blocks` (hybrid.metal:3616-3657): per 1024-value block of each row the 32 largest values in
    descending order with their indices, ties to the lower index; blocks past the row's end pad with -inf."""
    x = np.asarray(x, dtype=np.float32)
    rows, n = x.shape
    blocks = (n + 1023) // 1024
    vals = np.full((rows, blocks, 32), -np.inf, dtype=np.float32)
    idx = np.zeros((rows, blocks, 32), dtype=np.uint32)
    for r in range(rows):
        for b in range(blocks):
            seg = x[r, b * 1024:(b + 1) * 1024]
            order = np.lexsort((np.arange(seg.size), -seg.astype(np.float64)))[:32]  # value descending, then index ascending
            vals[r, b, :order.size] = seg[order]
            idx[r, b, :order.size] = order + b * 1024
    return vals, idx


def gemv_threads(fmt, packed, rows, cols, x, m, threads) -> np.ndarray:
    p, x = _u8(packed), _f32(x)
    y = np.empty((m, rows), dtype=np.float32)
    assert lib().fqo_gemv_threads(fmt, _p(p), rows, cols, _p(x), m, threads, _p(y)) == 0
    return y


def to_bf16(a) -> np.ndarray:
    """fp32 -> bf16 bits (RNE, NaN quieted), vectorised restatement of ``fqo_f32_to_bf16``."""
    a = _f32(a)
    bits = a.view(np.uint32)
    r = ((bits.astype(np.uint64) + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)
    nan = np.isnan(a)
    r[nan] = ((bits[nan] >> 16) | 0x40).astype(np.uint16)
    return r


def from_bf16(b) -> np.ndarray:
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def round_bf16(a) -> np.ndarray:
    return from_bf16(to_bf16(a)).reshape(np.shape(a))


def rel_err(got, want) -> float:
    """max|got - want| / max|want| (src/hybrid/bench.rs:56-69)."""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    scale = np.abs(want).max()
    return float(np.abs(got - want).max() / scale) if scale > 0 else float(np.abs(got).max())


# ------------------------------------------------------------------ benchmark-distribution blocks

def random_blocks(fmt: int, blocks: int, seed: int = 0) -> np.ndarray:
    """Packed blocks with the benchmark's distributions; draw order d -> dmin -> scales -> quants,
    each as one array over all blocks."""
    rng = np.random.default_rng(seed)
    el, bb = LAYOUT[fmt]
    out = np.empty((blocks, bb), dtype=np.uint8)
    half = lambda: (np.abs(rng.standard_normal(blocks)) * 1e-2).astype(np.float16).view(np.uint16)
    if fmt == Q4_K:
        d, dmin = half(), half()
        out[:, 0:2] = d.view(np.uint8).reshape(blocks, 2)
        out[:, 2:4] = dmin.view(np.uint8).reshape(blocks, 2)
        out[:, 4:16] = rng.integers(0, 256, size=(blocks, 12), dtype=np.uint8)
        out[:, 16:144] = rng.integers(0, 256, size=(blocks, 128), dtype=np.uint8)
    elif fmt == Q5_K:  # as Q4_K, the 32 bytes of fifth bits drawn after the scales
        d, dmin = half(), half()
        out[:, 0:2] = d.view(np.uint8).reshape(blocks, 2)
        out[:, 2:4] = dmin.view(np.uint8).reshape(blocks, 2)
        out[:, 4:16] = rng.integers(0, 256, size=(blocks, 12), dtype=np.uint8)
        out[:, 16:48] = rng.integers(0, 256, size=(blocks, 32), dtype=np.uint8)
        out[:, 48:176] = rng.integers(0, 256, size=(blocks, 128), dtype=np.uint8)
    elif fmt == Q3_K:  # hmask, qs and the packed scales uniform; d last (src/hybrid/iq_tests.rs:1502-1508)
        out[:, 0:108] = rng.integers(0, 256, size=(blocks, 108), dtype=np.uint8)
        out[:, 108:110] = half().view(np.uint8).reshape(blocks, 2)
    elif fmt == Q6_K:
        d = half()
        out[:, 208:210] = d.view(np.uint8).reshape(blocks, 2)
        out[:, 192:208] = rng.integers(-128, 128, size=(blocks, 16), dtype=np.int8).view(np.uint8)
        out[:, 0:192] = rng.integers(0, 256, size=(blocks, 192), dtype=np.uint8)
    elif fmt == Q8_0:
        d = half()
        out[:, 0:2] = d.view(np.uint8).reshape(blocks, 2)
        out[:, 2:34] = rng.integers(-127, 128, size=(blocks, 32), dtype=np.int8).view(np.uint8)
    elif fmt == IQ4_NL:  # d, then the nibbles
        out[:, 0:2] = half().view(np.uint8).reshape(blocks, 2)
        out[:, 2:18] = rng.integers(0, 256, size=(blocks, 16), dtype=np.uint8)
    elif fmt == IQ4_XS:  # d, then scales_h | scales_l, then the nibbles
        out[:, 0:2] = half().view(np.uint8).reshape(blocks, 2)
        out[:, 2:8] = rng.integers(0, 256, size=(blocks, 6), dtype=np.uint8)
        out[:, 8:136] = rng.integers(0, 256, size=(blocks, 128), dtype=np.uint8)
    else:
        raise ValueError(fmt)
    return out.reshape(-1)


IQ4_VALUES = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], dtype=np.float32)


def iq4_closed_form(fmt: int, packed: np.ndarray) -> np.ndarray:
    """The IQ4 decoders written from the format definition with array operations, independently of the C loops
    (IQ4_NL: src/hybrid/iq_tests.rs:1606-1618; IQ4_XS: src/metal/shaders/hybrid.metal:580-596)."""
    el, bb = LAYOUT[fmt]
    b = np.ascontiguousarray(packed, dtype=np.uint8).reshape(-1, bb)
    d = b[:, 0:2].copy().view(np.float16).astype(np.float32)  # [blocks, 1]
    if fmt == IQ4_NL:
        q = b[:, 2:18]
        vals = np.concatenate([IQ4_VALUES[q & 15], IQ4_VALUES[q >> 4]], axis=1)
        return (d * vals).astype(np.float32).reshape(-1)
    sh = b[:, 2].astype(np.uint32) | (b[:, 3].astype(np.uint32) << 8)
    out = np.empty((b.shape[0], 256), dtype=np.float32)
    for ib in range(8):
        ls = ((b[:, 4 + ib // 2] >> (4 * (ib % 2))) & 15).astype(np.int32) | (((sh >> (2 * ib)) & 3) << 4).astype(np.int32)
        dl = (d[:, 0] * (ls - 32).astype(np.float32)).astype(np.float32)[:, None]
        q = b[:, 8 + 16 * ib:24 + 16 * ib]
        out[:, 32 * ib:32 * ib + 16] = dl * IQ4_VALUES[q & 15]
        out[:, 32 * ib + 16:32 * ib + 32] = dl * IQ4_VALUES[q >> 4]
    return out.reshape(-1)


def random_matrix(fmt: int, rows: int, cols: int, seed: int = 0) -> np.ndarray:
    return random_blocks(fmt, rows * cols // LAYOUT[fmt][0], seed)


# ------------------------------------------------------------------ the reference's xorshift blocks

def _xorshift_bytes(state: int, n: int) -> np.ndarray:
    mask = (1 << 64) - 1
    out = np.empty(n, dtype=np.uint8)
    x = state
    for i in range(n):
        x ^= (x << 13) & mask
        x ^= x >> 7
        x ^= (x << 17) & mask
        out[i] = (x >> 32) & 0xFF
    return out


def xorshift_kquant_blocks(fmt: int, count: int) -> np.ndarray:
    """``kquant::blocks`` of src/diffusion/tests.rs:770-794: xorshift bytes seeded by the block
    size, with the f16 scales overwritten by small finite values taken from bytes 4 and 5."""
    el, bb = LAYOUT[fmt]
    state = ((bb * 0x9E3779B97F4A7C15) & ((1 << 64) - 1)) | 1
    b = _xorshift_bytes(state, count * bb).reshape(count, bb)
    scale = lambda v: (np.float32(0.002) + np.float32(0.002) * v.astype(np.float32) / np.float32(255.0)
                       ).astype(np.float16).view(np.uint16)
    s0, s1 = scale(b[:, 4]), scale(b[:, 5])
    if fmt == Q6_K:
        b[:, 208:210] = s0.view(np.uint8).reshape(count, 2)
    else:
        b[:, 0:2] = s0.view(np.uint8).reshape(count, 2)
        b[:, 2:4] = s1.view(np.uint8).reshape(count, 2)
    return b.reshape(-1)


def xorshift_f32(n: int, seed: int) -> np.ndarray:
    """``random`` of src/hybrid/iq_tests.rs:1252-1262: values in [-1, 1)."""
    mask = (1 << 64) - 1
    x = ((seed * 0x2545F4914F6CDD1D) & mask) | 1
    out = np.empty(n, dtype=np.float32)
    for i in range(n):
        x ^= (x << 13) & mask
        x ^= x >> 7
        x ^= (x << 17) & mask
        out[i] = np.float32(np.float32(x >> 40) / np.float32(1 << 24)) * np.float32(2.0) - np.float32(1.0)
    return out


# ------------------------------------------------------------------ the reference's closed-form fixtures
# src/ops/transformer.rs: `qk_tests` (:2833-2962), `q6_k_tests` (:4102-4175), `q8_0_tests` (:1683-1716).
# Each has a byte generator (here: *_packed) and an independent per-element formula (here: *_value);
# the tests pin the oracle's block decoders by demanding decode(packed) == value, bit for bit.

def qk_scales(row, block):
    return np.array([(row * 47 + block * 31 + i * 53 + 0x9D) & 255 for i in range(12)], dtype=np.uint8)


def qk_qbyte(row, block, index):
    return (row * 17 + block * 43 + index * 29 + 0x6B) & 255


def qk_parameters(row, block):
    return np.float32(0.00390625) + np.float32(row) * np.float32(0.00048828125), np.float32(0.015625)


def qk_q4k_packed(rows: int, cols: int) -> np.ndarray:
    out = bytearray()
    for row in range(rows):
        for blk in range(cols // 256):
            d, dmin = qk_parameters(row, blk)
            out += np.float16(d).tobytes() + np.float16(dmin).tobytes()
            out += qk_scales(row, blk).tobytes()
            out += bytes(qk_qbyte(row, blk, i) for i in range(128))
    return np.frombuffer(bytes(out), dtype=np.uint8).copy()


def qk5_parameters(row, block):
    """`parameters` for Q5_K (src/ops/transformer.rs:2845-2851)."""
    return np.float32(0.001953125) + np.float32(block) / np.float32(4096.0), np.float32(0.0078125)


def qk_q5k_packed(rows: int, cols: int) -> np.ndarray:
    """The Q5_K branch of `qk_tests::packed` (src/ops/transformer.rs:2879-2896)."""
    out = bytearray()
    for row in range(rows):
        for blk in range(cols // 256):
            d, dmin = qk5_parameters(row, blk)
            out += np.float16(d).tobytes() + np.float16(dmin).tobytes()
            out += qk_scales(row, blk).tobytes()
            out += bytes(qk_qbyte(row + 7, blk, i) for i in range(32))
            out += bytes(qk_qbyte(row, blk, i) for i in range(128))
    return np.frombuffer(bytes(out), dtype=np.uint8).copy()


def qk_q5k_value(row: int, column: int) -> np.float32:
    """`qk_value` for Q5_K (src/ops/transformer.rs:2939-2956)."""
    blk, within = divmod(column, 256)
    group, lane = divmod(within, 32)
    chunk = within // 64
    packed = qk_qbyte(row, blk, chunk * 32 + lane)
    nibble = packed & 15 if group % 2 == 0 else packed >> 4
    high = (qk_qbyte(row + 7, blk, lane) >> group) & 1
    d, dmin = qk5_parameters(row, blk)
    d = np.float32(np.float16(d))  # what the block stores
    scale, minimum = _unpack_scale_min(qk_scales(row, blk), group)
    return np.float32(np.float32(np.float32(d * np.float32(scale)) * np.float32(nibble | (high << 4)))
                      - np.float32(dmin * np.float32(minimum)))


def qk_q6k_packed(rows: int, cols: int) -> np.ndarray:
    """The Q6_K branch of `qk_tests::packed` (src/ops/transformer.rs:2864-2877)."""
    out = bytearray()
    for row in range(rows):
        for blk in range(cols // 256):
            out += bytes(qk_qbyte(row, blk, i) for i in range(128))
            out += bytes(qk_qbyte(row + 5, blk, i) for i in range(64))
            out += bytes((((row * 7 + blk * 3 + i * 5) % 15) - 7) & 255 for i in range(16))
            out += np.float16(np.float32(0.015625) + np.float32(row) / np.float32(4096.0)).tobytes()
    return np.frombuffer(bytes(out), dtype=np.uint8).copy()


def _unpack_scale_min(sc, group):
    if group < 4:
        return int(sc[group] & 63), int(sc[group + 4] & 63)
    return (int(sc[group + 4] & 15) | (int(sc[group - 4] >> 6) << 4),
            int(sc[group + 4] >> 4) | (int(sc[group] >> 6) << 4))


def qk_q4k_value(row: int, column: int) -> np.float32:
    """`qk_value` for Q4_K (src/ops/transformer.rs:2920-2956)."""
    blk, within = divmod(column, 256)
    group, lane = divmod(within, 32)
    chunk = within // 64
    packed = qk_qbyte(row, blk, chunk * 32 + lane)
    nibble = packed & 15 if group % 2 == 0 else packed >> 4
    d, dmin = qk_parameters(row, blk)
    # the fixture's d and dmin are exactly representable in f16
    scale, minimum = _unpack_scale_min(qk_scales(row, blk), group)
    return np.float32(np.float32(np.float32(d * np.float32(scale)) * np.float32(nibble))
                      - np.float32(dmin * np.float32(minimum)))


def qk_q6k_value(row: int, column: int) -> np.float32:
    """`qk_value` for Q6_K (src/ops/transformer.rs:2925-2938)."""
    blk, within = divmod(column, 256)
    group, lane = divmod(within, 32)
    half_block, slice_ = divmod(group, 4)
    packed = qk_qbyte(row, blk, half_block * 64 + (slice_ & 1) * 32 + lane)
    low = packed & 15 if slice_ < 2 else packed >> 4
    high = (qk_qbyte(row + 5, blk, half_block * 32 + lane) >> (slice_ * 2)) & 3
    q = (low | (high << 4)) - 32
    scale_index = half_block * 8 + slice_ * 2 + lane // 16
    scale = ((row * 7 + blk * 3 + scale_index * 5) % 15) - 7
    d = np.float32(np.float16(np.float32(0.015625) + np.float32(row) / np.float32(4096.0)))
    return np.float32(np.float32(d * np.float32(scale)) * np.float32(q))


def qk_input(rows: int, cols: int) -> np.ndarray:
    i = np.arange(rows * cols, dtype=np.int64)
    return (((i * 41 + 11) % 127).astype(np.float32) / np.float32(113.0) - np.float32(0.55)).astype(np.float32)


def q6_packed_byte(row, block, index):
    return (row * 13 + block * 7 + index * 17 + 3) & 255


def q6_scale_byte(row, block, index):
    return ((row * 3 + block * 5 + index * 7) % 9) - 4


def q6_block_scale(row, block):
    return np.float32(0.125) if (row + block) % 2 == 0 else np.float32(-0.0625)


def q6_packed(rows: int, cols: int) -> np.ndarray:
    out = bytearray()
    for row in range(rows):
        for blk in range(cols // 256):
            out += bytes(q6_packed_byte(row, blk, i) for i in range(128))
            out += bytes(q6_packed_byte(row + 11, blk, i) for i in range(64))
            out += bytes(q6_scale_byte(row, blk, i) & 255 for i in range(16))
            out += np.float16(q6_block_scale(row, blk)).tobytes()
    return np.frombuffer(bytes(out), dtype=np.uint8).copy()


def q6_value(row: int, column: int) -> np.float32:
    """`q6_value` (src/ops/transformer.rs:4153-4169)."""
    blk, within = divmod(column, 256)
    group, lane = divmod(within, 32)
    half_block, slice_ = divmod(group, 4)
    ql = q6_packed_byte(row, blk, half_block * 64 + (slice_ % 2) * 32 + lane)
    ql_bits = ql & 15 if slice_ < 2 else ql >> 4
    qh = q6_packed_byte(row + 11, blk, half_block * 32 + lane)
    high = (qh >> (slice_ * 2)) & 3
    quant = (ql_bits | (high << 4)) - 32
    scale = np.float32(q6_scale_byte(row, blk, half_block * 8 + slice_ * 2 + lane // 16))
    return np.float32(np.float32(q6_block_scale(row, blk) * scale) * np.float32(quant))


def q6_input(rows: int, cols: int) -> np.ndarray:
    i = np.arange(rows * cols, dtype=np.int64)
    return (((i * 19 + 7) % 127).astype(np.float32) / np.float32(113.0) - np.float32(0.56)).astype(np.float32)


def q8_packed(rows: int, cols: int) -> np.ndarray:
    out = bytearray()
    for row in range(rows):
        for _ in range(cols // 32):
            out += np.float16(0.03125).tobytes()
            out += bytes((((row * 11 + c * 7) % 25) - 12) & 255 for c in range(32))
    return np.frombuffer(bytes(out), dtype=np.uint8).copy()


def q8_value(row: int, column: int) -> np.float32:
    q = ((row * 11 + (column % 32) * 7) % 25) - 12
    return np.float32(np.float32(0.03125) * np.float32(q))


def q8_input(rows: int, cols: int) -> np.ndarray:
    i = np.arange(rows * cols, dtype=np.int64)
    return (((i * 29 + 3) % 101).astype(np.float32) / np.float32(73.0) - np.float32(0.65)).astype(np.float32)


def closed_form_expected(value_fn, x: np.ndarray, m: int, n: int, k: int) -> np.ndarray:
    """`expected` of the legacy tests: f32 left-to-right sum of x * value (src/ops/transformer.rs:2964-2980)."""
    w = np.array([[value_fn(r, c) for c in range(k)] for r in range(n)], dtype=np.float32)
    x = x.reshape(m, k)
    y = np.zeros((m, n), dtype=np.float32)
    for c in range(k):
        y = (y + x[:, c:c + 1] * w[None, :, c]).astype(np.float32)
    return y
