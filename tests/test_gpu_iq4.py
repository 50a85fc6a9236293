"""IQ4_NL and IQ4_XS on the op surface (the reference's `Format::Iq4Nl` / `Iq4Xs`, src/hybrid/weights.rs:38-103;
kernels `dequantize_iq4_xs`, `h_mv_iq4_xs`, `h_get_rows_iq4_xs`, src/metal/shaders/hybrid.metal:580-596, 900-1000,
1541): every projection path against the CPU oracle at the widths the reference tests its formats at
(M = 1, 3, 16 and 64, src/hybrid/iq_tests.rs:1686-1700), the expert paths with the reference's ids / offsets /
slot tables, and the bit-exact embedding lookup."""
import numpy as np
import pytest
import torch

from oracle import ref

pytestmark = pytest.mark.gpu

TOL_F32 = 1e-3
FORMATS = [ref.IQ4_NL, ref.IQ4_XS]


def S():
    from ferrum_b200 import surface
    return surface


def dev_f32(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()


def dev_u32(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.uint32).view(np.int32)).cuda()


def host(t):
    return t.detach().float().cpu().numpy()


@pytest.mark.parametrize("fmt", FORMATS)
def test_get_rows_is_bit_exact(device, fmt):
    s = S()
    rows, cols = 37, 768
    packed = ref.random_blocks(fmt, rows * cols // ref.LAYOUT[fmt][0], seed=3)
    dense = ref.dequant(fmt, packed).reshape(rows, cols)
    w = s.Matrix.from_packed(device, rows, cols, 1, fmt, packed)
    ids = np.array([36, 0, 5, 5, 17], dtype=np.uint32)
    y = torch.zeros(len(ids) * cols, dtype=torch.float32, device="cuda")
    s.get_rows(device, w, dev_u32(ids), y)
    device.synchronize()
    assert np.array_equal(host(y).reshape(len(ids), cols).view(np.uint32), dense[ids].view(np.uint32))


@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("m", [1, 3, 16, 64])
def test_project_matches_the_oracle(device, fmt, m):
    s = S()
    rows, cols = 70, 1024
    packed = ref.random_blocks(fmt, rows * cols // ref.LAYOUT[fmt][0], seed=11 + m)
    w = s.Matrix.from_packed(device, rows, cols, 1, fmt, packed)
    x = ref.xorshift_f32(m * cols, 21 + m)
    y = torch.zeros(m * rows, dtype=torch.float32, device="cuda")
    s.project(device, w, dev_f32(x), m, y)
    device.synchronize()
    want = ref.matmul(fmt, packed, rows, cols, x, m)
    assert ref.rel_err(host(y).reshape(m, rows), want) <= TOL_F32


@pytest.mark.parametrize("fmt", FORMATS)
def test_expert_paths(device, fmt):
    s = S()
    experts, rows, cols = 3, 13, 1024
    packed = ref.random_blocks(fmt, experts * rows * cols // ref.LAYOUT[fmt][0], seed=7)
    w = s.Matrix.from_packed(device, rows, cols, experts, fmt, packed)
    ids = np.array([2, 0, 1, 1, 2], dtype=np.uint32)  # src/hybrid/iq_tests.rs:1403
    x = ref.xorshift_f32(len(ids) * cols, 11)
    y = torch.zeros(len(ids) * rows, dtype=torch.float32, device="cuda")
    s.project_id(device, w, dev_f32(x), dev_u32(ids), len(ids), 1, y)
    device.synchronize()
    assert ref.rel_err(host(y).reshape(-1, rows), ref.matmul_id(fmt, packed, rows, cols, x, ids, 1)) <= TOL_F32
    offsets = np.array([0, 2, 2, 7], dtype=np.uint32)  # src/hybrid/iq_tests.rs:1766
    x7 = ref.xorshift_f32(7 * cols, 12)
    y7 = torch.zeros(7 * rows, dtype=torch.float32, device="cuda")
    s.project_mm_id(device, w, dev_f32(x7), dev_u32(offsets), 7, y7)
    device.synchronize()
    assert ref.rel_err(host(y7).reshape(-1, rows), ref.matmul_grouped(fmt, packed, rows, cols, x7, offsets)) <= TOL_F32
    table, offs = np.array([2, 0], dtype=np.uint32), np.array([0, 3, 5], dtype=np.uint32)  # src/hybrid/iq_tests.rs:1782
    x5 = ref.xorshift_f32(5 * cols, 13)
    y5 = torch.zeros(5 * rows, dtype=torch.float32, device="cuda")
    s.project_mm_id_in(device, w, dev_f32(x5), dev_u32(offs), (dev_u32(table), 2), 5, y5)
    device.synchronize()
    assert ref.rel_err(host(y5).reshape(-1, rows), ref.matmul_grouped(fmt, packed, rows, cols, x5, offs, table)) <= TOL_F32


@pytest.mark.parametrize("fmt", FORMATS)
def test_non_finite_scale_is_refused(device, fmt):
    s = S()
    packed = ref.random_blocks(fmt, 4 * 256 // ref.LAYOUT[fmt][0], seed=1).copy()
    packed[0:2] = np.array([np.inf], dtype=np.float16).view(np.uint8)
    with pytest.raises(s.WeightError):
        s.Matrix.from_packed(device, 4, 256, 1, fmt, packed)


def _dense_ffn(fmt, g, u, d, x, m, hidden, ef):
    gg = ref.matmul(fmt, g, ef, hidden, x, m)
    uu = ref.matmul(fmt, u, ef, hidden, x, m)
    return ref.matmul(fmt, d, hidden, ef, ref.swiglu(gg, uu), m)


@pytest.mark.parametrize("m", [2, 40])
def test_moe_block_with_iq4_xs_experts(device, m):
    """`moe_ffn` with every expert matrix in IQ4_XS (the encoding of the validated 35B-A3B file's experts): the
    per-route path (m * used <= 32) and the expert-sorted path against the oracle composition."""
    s = S()
    fmt = ref.IQ4_XS
    experts, used, hidden, ef = 16, 4, 512, 256
    rng = np.random.default_rng(m)
    router = ref.random_matrix(ref.Q8_0, experts, hidden, 10)
    gate_e, up_e = ref.random_matrix(fmt, experts * ef, hidden, 11), ref.random_matrix(fmt, experts * ef, hidden, 12)
    down_e = ref.random_matrix(fmt, experts * hidden, ef, 13)
    sg, su, sd = ref.random_matrix(fmt, ef, hidden, 14), ref.random_matrix(fmt, ef, hidden, 15), ref.random_matrix(fmt, hidden, ef, 16)
    x = (rng.standard_normal((m, hidden)) * 0.12).astype(np.float32)
    M = s.Matrix.from_packed
    f = s.MoeFfn(M(device, experts, hidden, 1, ref.Q8_0, router), M(device, ef, hidden, experts, fmt, gate_e),
                 M(device, ef, hidden, experts, fmt, up_e), M(device, hidden, ef, experts, fmt, down_e),
                 M(device, ef, hidden, 1, fmt, sg), M(device, ef, hidden, 1, fmt, su), M(device, hidden, ef, 1, fmt, sd),
                 None, experts, used, hidden, ef, ef, False, True)
    scratch = torch.zeros(s.moe_ffn_scratch_elems(device, f, m), dtype=torch.float32, device="cuda")
    out = torch.zeros(m * hidden, dtype=torch.float32, device="cuda")
    s.moe_ffn(device, f, dev_f32(x), m, scratch, out)
    device.synchronize()
    logits = ref.matmul(ref.Q8_0, router, experts, hidden, x, m)
    ids, wts, gate = ref.moe_route(logits, x, x[0], experts, used, hidden, m, False, True, False)
    shared = _dense_ffn(fmt, sg, su, sd, x, m, hidden, ef)
    g = ref.matmul_id(fmt, gate_e, ef, hidden, x, ids, used)
    u = ref.matmul_id(fmt, up_e, ef, hidden, x, ids, used)
    dn = ref.matmul_id(fmt, down_e, hidden, ef, ref.swiglu(g, u), ids, 1)
    want = ref.moe_combine(dn, wts, ids, shared, gate, hidden, used, m, identity=True)
    assert ref.rel_err(host(out).reshape(m, hidden), want) <= 3 * TOL_F32
