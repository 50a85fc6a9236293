"""Parity of the CUDA path (through the C ABI) with the CPU oracle on identical seeded inputs.

Shapes, id vectors and tolerances follow the reference's kernel tests (src/hybrid/iq_tests.rs:1301-1439,
1686-1814; src/ops/transformer.rs:2982-3200, 4176-4296; src/diffusion/tests.rs:716-760).  Bars:
decoded weights bit-exact; fp32 projections max|d|/max|y| <= 1e-3; bf16 projections <= 2e-2.
"""
import numpy as np
import pytest
import torch

from oracle import ref

pytestmark = pytest.mark.gpu

TOL_F32 = 1e-3   # fp32 GEMV / GEMM outputs, relative to max|y|
TOL_BF16 = 2e-2  # bf16 in / bf16 out

FORMATS = [ref.Q4_K, ref.Q5_K, ref.Q6_K, ref.Q8_0]


def S():
    from ferrum_b200 import surface
    return surface


def dev_f32(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()


def dev_u32(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.uint32).view(np.int32)).cuda()


def host(t):
    return t.detach().float().cpu().numpy()


def blocks_for(fmt, rows, cols, kind, seed=0):
    n = rows * cols // ref.LAYOUT[fmt][0]
    if kind == "random":
        return ref.random_blocks(fmt, n, seed)
    if kind == "xorshift":
        if fmt == ref.Q8_0:
            return ref.random_blocks(fmt, n, seed + 100)
        return ref.xorshift_kquant_blocks(fmt, n)
    if kind == "closed":
        return {ref.Q4_K: ref.qk_q4k_packed, ref.Q5_K: ref.qk_q5k_packed, ref.Q6_K: ref.q6_packed, ref.Q8_0: ref.q8_packed}[fmt](rows, cols)
    raise ValueError(kind)


# ------------------------------------------------------------------ decoded weights: bit-exact

@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("kind", ["closed", "xorshift", "random"])
def test_get_rows_is_bit_exact(device, fmt, kind):
    s = S()
    rows, cols = 37, 768 if fmt != ref.Q8_0 else 832
    packed = blocks_for(fmt, rows, cols, kind, seed=3)
    dense = ref.dequant(fmt, packed).reshape(rows, cols)
    w = s.Matrix.from_packed(device, rows, cols, 1, fmt, packed)
    ids = np.array([36, 0, 17, 17], dtype=np.uint32)  # src/hybrid/iq_tests.rs:1803
    y = torch.zeros(len(ids) * cols, dtype=torch.float32, device="cuda")
    s.get_rows(device, w, dev_u32(ids), y)
    device.synchronize()
    assert np.array_equal(host(y).view(np.uint32), dense[ids].ravel().view(np.uint32))
    # legacy embedding gather: bf16(decode), exactly (src/ops/transformer.rs:3308-3329)
    yb = torch.zeros(len(ids) * cols, dtype=torch.bfloat16, device="cuda")
    s.get_rows(device, w, dev_u32(ids), yb)
    device.synchronize()
    assert np.array_equal(yb.view(torch.int16).cpu().numpy().view(np.uint16), ref.to_bf16(dense[ids].ravel()))


def test_get_rows_whole_matrix_config0_sample(device):
    """Every row of a (512, 4096) Q4_K slice of the config-0 distribution decodes bit-exactly."""
    s = S()
    rows, cols = 512, 4096
    packed = ref.random_matrix(ref.Q4_K, rows, cols, seed=0)
    w = s.Matrix.from_packed(device, rows, cols, 1, ref.Q4_K, packed)
    y = torch.zeros(rows * cols, dtype=torch.float32, device="cuda")
    s.get_rows(device, w, dev_u32(np.arange(rows)), y)
    device.synchronize()
    assert np.array_equal(host(y).view(np.uint32), ref.dequant(ref.Q4_K, packed).view(np.uint32))


# ------------------------------------------------------------------ dense projections

def run_project(device, fmt, packed, rows, cols, x, m, dtype=torch.float32):
    s = S()
    w = s.Matrix.from_packed(device, rows, cols, 1, fmt, packed)
    xt = dev_f32(x).to(dtype).contiguous()
    y = torch.full((m * rows,), float("nan"), dtype=dtype, device="cuda")
    s.project(device, w, xt, m, y)
    device.synchronize()
    return host(y).reshape(m, rows)


CASES = [
    # (rows, cols, ms, kind) -- tails of rows, blocks and batch from the reference's tests
    (5, 512, (1, 2, 3, 4, 5, 7), "closed"),
    (133, 2560, (1,), "closed"),
    (6, 4864, (1,), "closed"),
    (65, 512, (4, 8, 15, 16), "closed"),
    (13, 1024, (1, 3, 16), "xorshift"),
    (100, 512, (9,), "xorshift"),
]


@pytest.mark.parametrize("exact", [False, True])
@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("rows,cols,ms,kind", CASES)
def test_project_matches_the_cpu_dequant(device, fmt, rows, cols, ms, kind, exact):
    if fmt == ref.Q8_0 and cols == 4864:
        cols = 896  # a Q8_0 width that is not a multiple of 256 (Qwen2.5 lm_head)
    packed = blocks_for(fmt, rows, cols, kind)
    device.set_exact(exact)
    try:
        for m in ms:
            x = ref.xorshift_f32(m * cols, m) if kind == "xorshift" else ref.qk_input(m, cols)
            want = ref.matmul(fmt, packed, rows, cols, x, m, mode=0)
            got = run_project(device, fmt, packed, rows, cols, x, m)
            assert np.abs(want).max() > 1e-2, "reference is vacuous"
            err = ref.rel_err(got, want)
            assert err <= TOL_F32, f"fmt {fmt} ({rows},{cols}) m={m} exact={exact}: {err:.3e}"
    finally:
        device.set_exact(False)


@pytest.mark.parametrize("fmt", FORMATS)
def test_project_m64_and_bf16(device, fmt):
    rows, cols = 65, 512
    packed = blocks_for(fmt, rows, cols, "random", seed=5)
    x = np.random.default_rng(6).standard_normal((64, cols)).astype(np.float32)
    want64 = ref.matmul(fmt, packed, rows, cols, x, 64, mode=0)
    # F32 in / F32 out wider than the verify widths: tensor cores with both operands split in two bf16 terms
    got = run_project(device, fmt, packed, rows, cols, x, 64)
    assert ref.rel_err(got, want64) <= 1e-4
    # ... m = 17 is the narrowest such call
    got = run_project(device, fmt, packed, rows, cols, x[:17], 17)
    assert ref.rel_err(got, want64[:17]) <= 1e-4
    # ... and the exact kernels agree
    device.set_exact(True)
    try:
        got = run_project(device, fmt, packed, rows, cols, x, 64)
    finally:
        device.set_exact(False)
    assert ref.rel_err(got, want64) <= TOL_F32
    # bf16 in / bf16 out, M = 35 (src/ops/transformer.rs:3116-3160): operands rounded to bf16.
    xb = ref.round_bf16(x[:35])
    want = ref.matmul(fmt, packed, rows, cols, xb, 35, mode=0)
    got = run_project(device, fmt, packed, rows, cols, xb, 35, dtype=torch.bfloat16)
    assert ref.rel_err(got, want) <= TOL_BF16


def test_wide_f32_projection_in_slices(device):
    """F32 in / F32 out at a width whose split copy of X exceeds the scratch half: the call runs in slices of
    activation rows (5120 -> 17408-wide input, 600 rows)."""
    rows, cols, m = 256, 17408, 600
    packed = ref.random_matrix(ref.Q6_K, rows, cols, seed=21)
    x = np.random.default_rng(22).standard_normal((m, cols)).astype(np.float32)
    dense = ref.dequant(ref.Q6_K, packed).reshape(rows, cols)
    want = x.astype(np.float64) @ dense.astype(np.float64).T
    got = run_project(device, ref.Q6_K, packed, rows, cols, x, m)
    assert np.abs(got - want).max() / np.abs(want).max() <= 1e-4


def test_config0_gemv(device):
    """Benchmark configuration 0: Q4_K 4096 x 4096, seed 0, x ~ N(0,1), M = 1."""
    rows = cols = 4096
    packed = ref.random_matrix(ref.Q4_K, rows, cols, seed=0)
    x = np.random.default_rng(0).standard_normal(cols).astype(np.float32)
    want = ref.matmul(ref.Q4_K, packed, rows, cols, x, 1, mode=0)
    got = run_project(device, ref.Q4_K, packed, rows, cols, x, 1)
    err = ref.rel_err(got, want)
    assert err <= TOL_F32, err
    again = run_project(device, ref.Q4_K, packed, rows, cols, x, 1)
    assert np.array_equal(got.view(np.uint32), again.view(np.uint32)), "projection is not deterministic"


def test_activation_magnitudes_do_not_matter(device):
    """The f16 tensor-core operands are rescaled per superblock, so huge and tiny activations keep
    the same relative accuracy."""
    rows, cols = 48, 1024
    packed = ref.random_matrix(ref.Q4_K, rows, cols, seed=9)
    base = np.random.default_rng(10).standard_normal((4, cols)).astype(np.float32)
    for scale in (1e-6, 1.0, 3e4, 1e9):
        x = (base * np.float32(scale)).astype(np.float32)
        x[0, 5] *= 1000  # an outlier inside one superblock
        want = ref.matmul(ref.Q4_K, packed, rows, cols, x, 4, mode=0)
        got = run_project(device, ref.Q4_K, packed, rows, cols, x, 4)
        assert ref.rel_err(got, want) <= TOL_F32, scale
    zero = run_project(device, ref.Q4_K, packed, rows, cols, np.zeros((2, cols), np.float32), 2)
    assert not zero.any()


# ------------------------------------------------------------------ expert projections

@pytest.mark.parametrize("exact", [False, True])
@pytest.mark.parametrize("fmt", FORMATS)
def test_project_id_and_grouped(device, fmt, exact):
    s = S()
    experts, rows, cols = 3, 13, 1024
    packed = blocks_for(fmt, experts * rows, cols, "random", seed=7 + fmt)
    w = s.Matrix.from_packed(device, rows, cols, experts, fmt, packed)
    assert (w.rows, w.experts, w.expert_rows()) == (experts * rows, experts, rows)
    device.set_exact(exact)
    try:
        ids = np.array([2, 0, 1, 1, 2], dtype=np.uint32)  # src/hybrid/iq_tests.rs:1403
        x = ref.xorshift_f32(len(ids) * cols, 11)
        y = torch.zeros(len(ids) * rows, dtype=torch.float32, device="cuda")
        s.project_id(device, w, dev_f32(x), dev_u32(ids), len(ids), 1, y)
        device.synchronize()
        want = ref.matmul_id(fmt, packed, rows, cols, x, ids, 1)
        assert ref.rel_err(host(y).reshape(-1, rows), want) <= TOL_F32
        # several routes share one activation row (gate / up of a token's experts)
        ids6 = np.array([0, 2, 1, 0, 2, 2], dtype=np.uint32)
        x3 = ref.xorshift_f32(3 * cols, 14)
        y6 = torch.zeros(6 * rows, dtype=torch.float32, device="cuda")
        s.project_id(device, w, dev_f32(x3), dev_u32(ids6), 6, 2, y6)
        device.synchronize()
        assert ref.rel_err(host(y6).reshape(-1, rows), ref.matmul_id(fmt, packed, rows, cols, x3, ids6, 2)) <= TOL_F32
        # expert-sorted rows: 0..2 expert 0, none of expert 1, 2..7 expert 2 (src/hybrid/iq_tests.rs:1766)
        offsets = np.array([0, 2, 2, 7], dtype=np.uint32)
        x7 = ref.xorshift_f32(7 * cols, 12)
        y7 = torch.zeros(7 * rows, dtype=torch.float32, device="cuda")
        s.project_mm_id(device, w, dev_f32(x7), dev_u32(offsets), 7, y7)
        device.synchronize()
        # the expert-sorted GEMM is a bf16 tensor-core path (bar 2e-2; the reference's own F16-tile kernel is
        # checked at 5e-3, src/hybrid/iq_tests.rs:1289-1299); exact mode keeps fp32
        tol_g = TOL_F32 if exact else TOL_BF16
        assert ref.rel_err(host(y7).reshape(-1, rows), ref.matmul_grouped(fmt, packed, rows, cols, x7, offsets)) <= tol_g
        # arena slots: group z is stored at table[z] (src/hybrid/iq_tests.rs:1782)
        table, offs = np.array([2, 0], dtype=np.uint32), np.array([0, 3, 5], dtype=np.uint32)
        x5 = ref.xorshift_f32(5 * cols, 13)
        y5 = torch.zeros(5 * rows, dtype=torch.float32, device="cuda")
        s.project_mm_id_in(device, w, dev_f32(x5), dev_u32(offs), (dev_u32(table), 2), 5, y5)
        device.synchronize()
        assert ref.rel_err(host(y5).reshape(-1, rows), ref.matmul_grouped(fmt, packed, rows, cols, x5, offs, table)) <= tol_g
    finally:
        device.set_exact(False)


# ------------------------------------------------------------------ MoE glue

def near_tie(scores, used):
    """True when the k-th and (k+1)-th scores are within 4 ulp: the device's exp may order them
    differently from libm's, as the reference's own GPU-vs-CPU test accepts."""
    top = np.sort(scores)[::-1]
    return bool(np.abs(top[:used + 1][:-1] - top[1:used + 1]).min() <= 4 * np.spacing(top[0]))


@pytest.mark.parametrize("sigmoid,norm,shared_gate", [(True, True, False), (False, True, True), (True, False, True)])
def test_moe_route(device, sigmoid, norm, shared_gate):
    s = S()
    experts, used, hidden, m = 256, 6, 2048, 3  # src/hybrid/engine.rs:4951
    logits = ref.xorshift_f32(m * experts, 21) * np.float32(3.0)
    x = ref.xorshift_f32(m * hidden, 22)
    sw = ref.xorshift_f32(hidden, 23)
    ids = torch.zeros(m * used, dtype=torch.int32, device="cuda")
    wts = torch.zeros(m * used, dtype=torch.float32, device="cuda")
    gate = torch.zeros(m, dtype=torch.float32, device="cuda")
    s.moe_route(device, dev_f32(logits), dev_f32(x), dev_f32(sw), experts, used, hidden, m, sigmoid, norm, shared_gate,
                ids, wts, gate)
    device.synchronize()
    want_ids, want_w, want_g = ref.moe_route(logits, x, sw, experts, used, hidden, m, sigmoid, norm, shared_gate)
    assert np.array_equal(ids.cpu().numpy().view(np.uint32), want_ids)
    assert np.abs(host(wts) - want_w).max() < 1e-5
    assert np.abs(host(gate) - want_g).max() < 1e-4


def test_moe_route_top8_of_256_for_1024_tokens(device):
    """Config 3's router: softmax -> top-8 -> renormalise, T = 1024, logits ~ N(0,1)."""
    s = S()
    experts, used, hidden, m = 256, 8, 2048, 1024
    rng = np.random.default_rng(3)
    logits = rng.standard_normal((m, experts)).astype(np.float32)
    x = rng.standard_normal((m, hidden)).astype(np.float32)
    ids = torch.zeros(m * used, dtype=torch.int32, device="cuda")
    wts = torch.zeros(m * used, dtype=torch.float32, device="cuda")
    gate = torch.zeros(m, dtype=torch.float32, device="cuda")
    s.moe_route(device, dev_f32(logits), dev_f32(x), dev_f32(x[0]), experts, used, hidden, m, False, True, False, ids, wts, gate)
    device.synchronize()
    want_ids, want_w, _ = ref.moe_route(logits, x, x[0], experts, used, hidden, m, False, True, False)
    got_ids = ids.cpu().numpy().view(np.uint32).reshape(m, used)
    bad = [t for t in range(m) if not np.array_equal(got_ids[t], want_ids.reshape(m, used)[t])]
    for t in bad:  # only exact ties of rounded scores may differ
        e = np.exp(logits[t] - logits[t].max())
        assert near_tie((e / e.sum()).astype(np.float32), used), t
    assert len(bad) <= 2
    keep = np.setdiff1d(np.arange(m), bad)
    assert np.abs(host(wts).reshape(m, used)[keep] - want_w.reshape(m, used)[keep]).max() < 1e-5
    assert np.allclose(host(wts).reshape(m, used).sum(1), 1.0, atol=1e-5)


@pytest.mark.parametrize("routes", [24, 40, 3000, 6000, 66000])
def test_moe_map_with_ids_that_name_no_expert(device, routes):
    """Routes whose id is not an expert belong to no row: position 0, and the rows past the last expert's point at
    route 0 (one warp, one block and the cluster of blocks)."""
    s = S()
    experts = 19
    rng = np.random.default_rng(routes)
    ids = rng.integers(0, experts, routes).astype(np.uint32)
    bad = rng.choice(routes, max(1, routes // 7), replace=False)
    ids[bad] = rng.integers(experts, 2**32 - 1, bad.size, dtype=np.uint64).astype(np.uint32)
    offsets = torch.full((experts + 1,), -1, dtype=torch.int32, device="cuda")
    sorted_ = torch.full((routes,), -1, dtype=torch.int32, device="cuda")
    position = torch.full((routes,), -1, dtype=torch.int32, device="cuda")
    s.moe_map(device, dev_u32(ids), experts, routes, offsets, sorted_, position)
    device.synchronize()
    valid = ids < experts
    order = np.argsort(ids[valid], kind="stable")
    want_sorted = np.flatnonzero(valid)[order].astype(np.uint32)
    got_o, got_s, got_p = (t.cpu().numpy().view(np.uint32) for t in (offsets, sorted_, position))
    assert np.array_equal(got_o, np.concatenate([[0], np.cumsum(np.bincount(ids[valid], minlength=experts))]).astype(np.uint32))
    assert np.array_equal(got_s[:want_sorted.size], want_sorted)
    assert not got_s[want_sorted.size:].any()
    assert np.array_equal(got_p[want_sorted], np.arange(want_sorted.size, dtype=np.uint32))
    assert not got_p[~valid].any()


@pytest.mark.parametrize("experts,routes", [(3, 8), (256, 8), (1000, 32), (7, 5), (256, 8192), (256, 40), (1000, 777), (256, 4096),
                                            (1000, 5000), (37, 70001), (5, 300000)])
def test_moe_map_gather_combine(device, experts, routes):
    s = S()
    rng = np.random.default_rng(routes)
    used = 8 if routes % 8 == 0 else 1
    tokens = routes // used
    ids = rng.integers(0, experts, routes).astype(np.uint32)
    offsets = torch.zeros(experts + 1, dtype=torch.int32, device="cuda")
    sorted_ = torch.zeros(routes, dtype=torch.int32, device="cuda")
    position = torch.zeros(routes, dtype=torch.int32, device="cuda")
    s.moe_map(device, dev_u32(ids), experts, routes, offsets, sorted_, position)
    device.synchronize()
    wo, ws, wp = ref.moe_map(ids, experts)
    assert np.array_equal(offsets.cpu().numpy().view(np.uint32), wo)
    assert np.array_equal(sorted_.cpu().numpy().view(np.uint32), ws)
    assert np.array_equal(position.cpu().numpy().view(np.uint32), wp)
    hidden = 96
    x = rng.standard_normal((tokens, hidden)).astype(np.float32)
    xg = torch.zeros(routes * hidden, dtype=torch.float32, device="cuda")
    s.moe_gather(device, dev_f32(x), sorted_, hidden, used, routes, xg)
    device.synchronize()
    assert np.array_equal(host(xg).reshape(routes, hidden), ref.moe_gather(x, ws, hidden, used))
    down = rng.standard_normal((routes, hidden)).astype(np.float32)
    wts = rng.random(routes).astype(np.float32)
    shared = rng.standard_normal((tokens, hidden)).astype(np.float32)
    gate = rng.random(tokens).astype(np.float32)
    out = torch.zeros(tokens * hidden, dtype=torch.float32, device="cuda")
    for identity in (False, True):
        s.moe_combine(device, dev_f32(down), dev_f32(wts), position, dev_f32(shared), dev_f32(gate), hidden, used, tokens,
                      identity, out)
        device.synchronize()
        want = ref.moe_combine(down, wts, wp, shared, gate, hidden, used, tokens, identity)
        assert np.abs(host(out).reshape(tokens, hidden) - want).max() <= 1e-5 * max(1.0, np.abs(want).max())


def test_glu(device):
    s = S()
    rng = np.random.default_rng(2)
    g = (rng.standard_normal(5000) * 4).astype(np.float32)
    u = rng.standard_normal(5000).astype(np.float32)
    out = torch.zeros(5000, dtype=torch.float32, device="cuda")
    s.glu(device, dev_f32(g), dev_f32(u), out)
    device.synchronize()
    assert np.abs(host(out) - ref.swiglu(g, u)).max() <= 1e-5 * np.abs(ref.swiglu(g, u)).max()


# ------------------------------------------------------------------ feed-forward blocks

def oracle_dense_ffn(gate, up, down, x, m, hidden, width):
    g = ref.matmul(ref.Q4_K, gate, width, hidden, x, m)
    u = ref.matmul(ref.Q4_K, up, width, hidden, x, m)
    return ref.matmul(ref.Q6_K, down, hidden, width, ref.swiglu(g, u), m)


def test_dense_ffn(device):
    s = S()
    hidden, width, m = 512, 768, 3
    gate, up = ref.random_matrix(ref.Q4_K, width, hidden, 1), ref.random_matrix(ref.Q4_K, width, hidden, 2)
    down = ref.random_matrix(ref.Q6_K, hidden, width, 3)
    x = np.random.default_rng(4).standard_normal((m, hidden)).astype(np.float32)
    mats = [s.Matrix.from_packed(device, width, hidden, 1, ref.Q4_K, gate), s.Matrix.from_packed(device, width, hidden, 1, ref.Q4_K, up),
            s.Matrix.from_packed(device, hidden, width, 1, ref.Q6_K, down)]
    scratch = torch.zeros(3 * m * width, dtype=torch.float32, device="cuda")
    out = torch.zeros(m * hidden, dtype=torch.float32, device="cuda")
    s.dense_ffn(device, *mats, dev_f32(x), m, scratch, out)
    device.synchronize()
    want = oracle_dense_ffn(gate, up, down, x, m, hidden, width)
    assert ref.rel_err(host(out).reshape(m, hidden), want) <= 2 * TOL_F32  # three chained projections


@pytest.mark.parametrize("m", [1, 3, 40])
def test_moe_ffn(device, m):
    """`moe_ffn` end to end: m * used <= 32 takes the per-route GEMVs, m = 40 the expert-sorted GEMM."""
    s = S()
    experts, used, hidden, ef = 16, 4, 512, 256
    rng = np.random.default_rng(m)
    router = ref.random_matrix(ref.Q8_0, experts, hidden, 10)
    gate_e = ref.random_matrix(ref.Q4_K, experts * ef, hidden, 11)
    up_e = ref.random_matrix(ref.Q4_K, experts * ef, hidden, 12)
    down_e = ref.random_matrix(ref.Q6_K, experts * hidden, ef, 13)
    sg, su = ref.random_matrix(ref.Q4_K, ef, hidden, 14), ref.random_matrix(ref.Q4_K, ef, hidden, 15)
    sd = ref.random_matrix(ref.Q6_K, hidden, ef, 16)
    x = (rng.standard_normal((m, hidden)) * 0.12).astype(np.float32)  # router logits of spread ~2
    M = s.Matrix.from_packed
    f = s.MoeFfn(M(device, experts, hidden, 1, ref.Q8_0, router), M(device, ef, hidden, experts, ref.Q4_K, gate_e),
                 M(device, ef, hidden, experts, ref.Q4_K, up_e), M(device, hidden, ef, experts, ref.Q6_K, down_e),
                 M(device, ef, hidden, 1, ref.Q4_K, sg), M(device, ef, hidden, 1, ref.Q4_K, su), M(device, hidden, ef, 1, ref.Q6_K, sd),
                 None, experts, used, hidden, ef, ef, False, True)
    scratch = torch.zeros(s.moe_ffn_scratch_elems(device, f, m), dtype=torch.float32, device="cuda")
    out = torch.zeros(m * hidden, dtype=torch.float32, device="cuda")
    s.moe_ffn(device, f, dev_f32(x), m, scratch, out)
    device.synchronize()
    # oracle composition
    logits = ref.matmul(ref.Q8_0, router, experts, hidden, x, m)
    ids, wts, gate = ref.moe_route(logits, x, x[0], experts, used, hidden, m, False, True, False)
    shared = oracle_dense_ffn(sg, su, sd, x, m, hidden, ef)
    g = ref.matmul_id(ref.Q4_K, gate_e, ef, hidden, x, ids, used)
    u = ref.matmul_id(ref.Q4_K, up_e, ef, hidden, x, ids, used)
    dn = ref.matmul_id(ref.Q6_K, down_e, hidden, ef, ref.swiglu(g, u), ids, 1)
    want = ref.moe_combine(dn, wts, ids, shared, gate, hidden, used, m, identity=True)
    # m = 40 runs three chained bf16 expert GEMMs; the smaller cases stay on the fp32-accurate GEMVs
    assert ref.rel_err(host(out).reshape(m, hidden), want) <= (3 * TOL_F32 if m * used <= 32 else TOL_BF16)


@pytest.mark.parametrize("m", [2, 40])
def test_moe_ffn_expert_parallel_on_one_rank_is_bit_identical(device, m):
    """`moe_ffn_ep` with a communicator of one rank: the expert-sorted order it always works in (gathered rows,
    local expert ids, position-indexed combine) gives the bits of `moe_ffn`."""
    s = S()
    experts, used, hidden, ef = 16, 4, 512, 256
    M = s.Matrix.from_packed
    f = s.MoeFfn(M(device, experts, hidden, 1, ref.Q8_0, ref.random_matrix(ref.Q8_0, experts, hidden, 10)),
                 M(device, ef, hidden, experts, ref.Q4_K, ref.random_matrix(ref.Q4_K, experts * ef, hidden, 11)),
                 M(device, ef, hidden, experts, ref.Q4_K, ref.random_matrix(ref.Q4_K, experts * ef, hidden, 12)),
                 M(device, hidden, ef, experts, ref.Q6_K, ref.random_matrix(ref.Q6_K, experts * hidden, ef, 13)),
                 M(device, ef, hidden, 1, ref.Q4_K, ref.random_matrix(ref.Q4_K, ef, hidden, 14)),
                 M(device, ef, hidden, 1, ref.Q4_K, ref.random_matrix(ref.Q4_K, ef, hidden, 15)),
                 M(device, hidden, ef, 1, ref.Q6_K, ref.random_matrix(ref.Q6_K, hidden, ef, 16)),
                 None, experts, used, hidden, ef, ef, False, True)
    x = dev_f32((np.random.default_rng(m).standard_normal((m, hidden)) * 0.12).astype(np.float32))
    n = s.moe_ffn_scratch_elems(device, f, m)
    out1 = torch.zeros(m * hidden, dtype=torch.float32, device="cuda")
    s.moe_ffn(device, f, x, m, torch.zeros(n, dtype=torch.float32, device="cuda"), out1)
    comm = s.Comm(device, 0, 1, 4096 + m * used * hidden * 4)
    out2 = torch.zeros(m * hidden, dtype=torch.float32, device="cuda")
    s.moe_ffn_ep(device, comm, 4096, f, 0, x, m, torch.zeros(n, dtype=torch.float32, device="cuda"), out2)
    device.synchronize()
    assert torch.equal(out1, out2)
    comm.close()


# ------------------------------------------------------------------ error behaviour and the boundary

def test_errors_follow_the_reference(device):
    s = S()
    packed = ref.random_matrix(ref.Q4_K, 16, 512, 1)
    w = s.Matrix.from_packed(device, 16, 512, 1, ref.Q4_K, packed)
    x = torch.zeros(2 * 512, dtype=torch.float32, device="cuda")
    y = torch.zeros(2 * 16, dtype=torch.float32, device="cuda")
    with pytest.raises(s.ShapeError):   # Error::Shape, src/hybrid/engine.rs:3414-3421
        s.project(device, w, x, 3, y)
    with pytest.raises(s.ShapeError):
        s.project(device, w, x, 2, y[:-1].contiguous())
    big = torch.zeros(4096, dtype=torch.float32, device="cuda")
    with pytest.raises(s.AliasError):   # Error::Dispatch(alias), src/metal/mod.rs:880-896
        s.project(device, w, big[:1024], 2, big[512:544])
    with pytest.raises(s.RangeError):   # misaligned binding
        s.project(device, w, big[1:1025], 2, y)
    with pytest.raises(s.WeightError):  # src/hybrid/weights.rs:702-722
        s.Matrix.from_packed(device, 16, 512, 1, ref.Q4_K, packed[:-1])
    with pytest.raises(s.WeightError):
        s.Matrix.from_packed(device, 16, 320, 1, ref.Q4_K, packed[: 16 * 144])
    bad = packed.copy()
    bad[0:2] = np.frombuffer(np.float16(np.inf).tobytes(), dtype=np.uint8)
    with pytest.raises(s.WeightError):  # src/quantization.rs:236-240
        s.Matrix.from_packed(device, 16, 512, 1, ref.Q4_K, bad)
    with pytest.raises(s.WeightError):
        s.Matrix.from_packed(device, 16, 512, 1, 11, packed)  # Q3_K: no kernel (the loader rewrites it as Q6_K)
    s.project(device, w, x, 2, y)  # the handle still works
    device.synchronize()


def test_injected_failures_poison_and_recover(device):
    """`fail_after` / `fail_completion` (src/metal/mod.rs:1196-1303), injected on the host."""
    s = S()
    w = s.Matrix.from_packed(device, 16, 512, 1, ref.Q4_K, ref.random_matrix(ref.Q4_K, 16, 512, 1))
    x = torch.ones(512, dtype=torch.float32, device="cuda")
    y = torch.zeros(16, dtype=torch.float32, device="cuda")
    device.fail_after(1)
    s.project(device, w, x, 1, y)
    with pytest.raises(s.SynchronizationError):
        s.project(device, w, x, 1, y)
    with pytest.raises(s.SynchronizationError):  # refused until recovered
        s.project(device, w, x, 1, y)
    device.recover()
    s.project(device, w, x, 1, y)
    device.fail_completion()
    with pytest.raises(s.SynchronizationError):
        device.synchronize()
    device.recover()
    device.synchronize()


class _Owned:
    """A buffer the device handle allocated (`fq_buffer_alloc`), viewed as a torch tensor of floats."""

    def __init__(self, device, floats):
        import ctypes as C
        self.device, self.ptr = device, C.c_void_p()
        device.check(device._L.fq_buffer_alloc(device.handle, floats * 4, C.byref(self.ptr)))
        self.__cuda_array_interface__ = {"shape": (floats,), "typestr": "<f4", "data": (self.ptr.value, False), "version": 3}
        self.tensor = torch.as_tensor(self, device="cuda")

    def free(self):
        self.device.check(self.device._L.fq_buffer_free(self.device.handle, self.ptr))


def test_outputs_of_a_failed_submission_are_refused_as_inputs(device):
    """What a failed submission wrote into a buffer of the handle may not feed a later dispatch until it has been
    written again by a submission that completed (`Completion::Failed`, src/metal/mod.rs:865-873); other buffers are
    unaffected, and so is memory the caller owns."""
    s = S()
    w1 = s.Matrix.from_packed(device, 512, 512, 1, ref.Q4_K, ref.random_matrix(ref.Q4_K, 512, 512, 1))
    packed2 = ref.random_matrix(ref.Q4_K, 16, 512, 2)
    w2 = s.Matrix.from_packed(device, 16, 512, 1, ref.Q4_K, packed2)
    x = torch.ones(512, dtype=torch.float32, device="cuda")
    hb = _Owned(device, 512)
    h = hb.tensor
    y = torch.zeros(16, dtype=torch.float32, device="cuda")
    try:
        s.project(device, w1, x, 1, h)
        device.fail_completion()
        with pytest.raises(s.SynchronizationError):
            device.synchronize()
        device.recover()
        with pytest.raises(s.SynchronizationError):   # h belongs to the failed submission
            s.project(device, w2, h, 1, y)
        s.project(device, w2, x, 1, y)                # x does not
        s.project(device, w1, x, 1, h)                # written again ...
        device.synchronize()                          # ... by a submission that completed
        s.project(device, w2, h, 1, y)
        device.synchronize()
        want = ref.matmul(ref.Q4_K, packed2, 16, 512, host(h), 1)
        assert ref.rel_err(host(y).reshape(1, 16), want) <= TOL_F32
    finally:
        hb.free()


def test_host_buffer_entry_points_match_the_device_path(device):
    s = S()
    rows, cols, m = 96, 1024, 5
    packed = ref.random_matrix(ref.Q4_K, rows, cols, 21)
    w = s.Matrix.from_packed(device, rows, cols, 1, ref.Q4_K, packed)
    w2 = s.Matrix.from_packed(device, 32, cols, 1, ref.Q4_K, ref.random_matrix(ref.Q4_K, 32, cols, 22))
    x = np.random.default_rng(23).standard_normal((m, cols)).astype(np.float32)
    y = np.zeros((m, rows), dtype=np.float32)
    before = device.counters()
    s.project_host(device, w, x, m, y)
    after = device.counters()
    assert after.bytes_uploaded - before.bytes_uploaded == x.nbytes
    assert after.bytes_downloaded - before.bytes_downloaded == y.nbytes
    assert after.dispatches > before.dispatches
    yd = torch.zeros(m * rows, dtype=torch.float32, device="cuda")
    s.project(device, w, dev_f32(x), m, yd)
    device.synchronize()
    assert np.array_equal(y.view(np.uint32), host(yd).reshape(m, rows).view(np.uint32))
    ya, yb = np.zeros((m, rows), np.float32), np.zeros((m, 32), np.float32)
    s.project_many_host(device, [w, w2], x, m, [ya, yb])
    assert np.array_equal(ya, y)
    assert ref.rel_err(yb, ref.matmul(ref.Q4_K, ref.random_matrix(ref.Q4_K, 32, cols, 22), 32, cols, x, m)) <= TOL_F32


# ------------------------------------------------------------------ full-size shapes (config 1)

@pytest.mark.parametrize("fmt,rows,cols", [(ref.Q4_K, 6144, 5120), (ref.Q4_K, 1024, 5120), (ref.Q6_K, 5120, 17408)])
@pytest.mark.parametrize("m", [1, 8, 16])
def test_full_size_projection_rows_and_self_consistency(device, fmt, rows, cols, m):
    """27B-class shapes: a random subset of output rows against the oracle, and the default path
    against the exact-decode path over all rows (`max|batched - single| / max|single|`,
    src/hybrid/bench.rs:56-69)."""
    s = S()
    packed = ref.random_matrix(fmt, rows, cols, seed=rows % 97)
    x = np.random.default_rng(m).standard_normal((m, cols)).astype(np.float32)
    got = run_project(device, fmt, packed, rows, cols, x, m)
    rb = ref.row_bytes(fmt, cols)
    pick = np.sort(np.random.default_rng(5).choice(rows, 24, replace=False))
    sub = np.concatenate([packed[r * rb:(r + 1) * rb] for r in pick])
    want = ref.matmul(fmt, sub, len(pick), cols, x, m, mode=0)
    scale = np.abs(got).max()
    assert np.abs(got[:, pick] - want).max() / scale <= TOL_F32
    device.set_exact(True)
    try:
        exact = run_project(device, fmt, packed, rows, cols, x, m)
    finally:
        device.set_exact(False)
    assert ref.rel_err(got, exact) <= TOL_F32


# ------------------------------------------------------------------ fused launches and batched submission

@pytest.mark.parametrize("fmt", [ref.Q4_K, ref.Q6_K])
@pytest.mark.parametrize("m", [1, 3, 5, 16])
def test_project_many_is_bit_identical_to_separate_projections(device, fmt, m):
    """q|k|v-style fusion: one launch over several matrices gives each matrix exactly what its own
    projection gives (same kernel, same per-row summation order)."""
    s = S()
    cols, rows = 1024, (96, 40, 17)
    packed = [ref.random_matrix(fmt, r, cols, seed=30 + i) for i, r in enumerate(rows)]
    ws = [s.Matrix.from_packed(device, r, cols, 1, fmt, p) for r, p in zip(rows, packed)]
    x = np.random.default_rng(m).standard_normal((m, cols)).astype(np.float32)
    xt = dev_f32(x)
    fused = [torch.zeros(m * r, dtype=torch.float32, device="cuda") for r in rows]
    s.project_many(device, ws, xt, m, fused)
    device.synchronize()
    for w, r, p, yf in zip(ws, rows, packed, fused):
        ys = torch.zeros(m * r, dtype=torch.float32, device="cuda")
        s.project(device, w, xt, m, ys)
        device.synchronize()
        assert np.array_equal(host(yf).view(np.uint32), host(ys).view(np.uint32))
        assert ref.rel_err(host(yf).reshape(m, r), ref.matmul(fmt, p, r, cols, x, m)) <= TOL_F32
    # mixed formats fall back to one projection each, with the same results
    mixed = [ws[0], s.Matrix.from_packed(device, 24, cols, 1, ref.Q8_0, ref.random_matrix(ref.Q8_0, 24, cols, 40))]
    outs = [torch.zeros(m * 96, dtype=torch.float32, device="cuda"), torch.zeros(m * 24, dtype=torch.float32, device="cuda")]
    s.project_many(device, mixed, xt, m, outs)
    device.synchronize()
    assert np.array_equal(host(outs[0]).view(np.uint32), host(fused[0]).view(np.uint32))
    assert ref.rel_err(host(outs[1]).reshape(m, 24), ref.matmul(ref.Q8_0, ref.random_matrix(ref.Q8_0, 24, cols, 40), 24, cols, x, m)) <= TOL_F32


def test_captured_graph_replays_a_layer(device):
    """A recorded batch (the counterpart of one command epoch) replays with new inputs in place."""
    s = S()
    d2 = s.Device(0, use_torch_stream=False)
    hidden, width = 512, 768
    gate, up = ref.random_matrix(ref.Q4_K, width, hidden, 1), ref.random_matrix(ref.Q4_K, width, hidden, 2)
    down = ref.random_matrix(ref.Q6_K, hidden, width, 3)
    mats = [s.Matrix.from_packed(d2, width, hidden, 1, ref.Q4_K, gate), s.Matrix.from_packed(d2, width, hidden, 1, ref.Q4_K, up),
            s.Matrix.from_packed(d2, hidden, width, 1, ref.Q6_K, down)]
    m = 2
    x = torch.zeros(m * hidden, dtype=torch.float32, device="cuda")
    scratch = torch.zeros(3 * m * width, dtype=torch.float32, device="cuda")
    out = torch.zeros(m * hidden, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    with pytest.raises(s.ParameterError):
        d2.capture_end()
    d2.capture_begin()
    s.dense_ffn(d2, *mats, x, m, scratch, out)
    with pytest.raises(s.ParameterError):
        d2.synchronize()  # refused while recording
    graph = d2.capture_end()
    before = d2.counters().dispatches
    for seed in (4, 5):
        xv = np.random.default_rng(seed).standard_normal((m, hidden)).astype(np.float32)
        d2.upload(x, xv)
        graph.launch()
        d2.synchronize()
        want = oracle_dense_ffn(gate, up, down, xv, m, hidden, width)
        assert ref.rel_err(host(out).reshape(m, hidden), want) <= 2 * TOL_F32
    # gate|up and down with the gated unit inside down's activation preparation: (prep + gemv) x 2 per replay,
    # or two kernels with the staged GEMV
    assert d2.counters().dispatches - before in (2 * 4, 2 * 2)
    graph.close()
    d2.close()


# ------------------------------------------------------------------ prefill dequant-GEMM (tensor memory path)

def run_project_bf16(device, fmt, packed, rows, cols, xb, m):
    s = S()
    w = s.Matrix.from_packed(device, rows, cols, 1, fmt, packed)
    xt = dev_f32(xb).to(torch.bfloat16).contiguous()
    y = torch.full((m * rows,), float("nan"), dtype=torch.bfloat16, device="cuda")
    s.project(device, w, xt, m, y)
    device.synchronize()
    return y


@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("m,cols,rows", [(200, 512, 100), (35, 512, 65), (1025, 256, 65), (512, 1024, 384), (300, 2048, 129)])
def test_bf16_gemm_matches_the_cpu_dequant(device, fmt, m, cols, rows):
    """bf16 x bf16-rounded weights, fp32 accumulate, bf16 out (src/ops/transformer.rs:3116-3160,
    src/diffusion/tests.rs:716-760): token and output counts that are not whole tiles."""
    packed = blocks_for(fmt, rows, cols, "random", seed=m)
    xb = ref.round_bf16(np.random.default_rng(m + 1).standard_normal((m, cols)).astype(np.float32))
    dense_b = ref.round_bf16(ref.dequant(fmt, packed)).reshape(rows, cols)
    want = xb.astype(np.float64) @ dense_b.astype(np.float64).T
    got = run_project_bf16(device, fmt, packed, rows, cols, xb, m).float().cpu().numpy().reshape(m, rows)
    assert np.abs(want).max() > 0.1
    err = np.abs(got - want).max() / np.abs(want).max()
    assert err <= TOL_BF16, err
    # fp32 accumulation of bf16 operands leaves only the final bf16 rounding: far inside the bar
    assert err <= 6e-3, err


@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("m,cols,rows", [(2048, 512, 10240), (1100, 768, 5000), (600, 256, 19200)])
def test_bf16_gemm_whole_waves_plus_split_tail(device, fmt, m, cols, rows):
    """More tiles than SMs but not whole waves: the tiles of the last, partly filled wave are split along K and
    summed by the fix-up kernel; the others are computed whole."""
    packed = ref.random_matrix(fmt, rows, cols, seed=m)
    xb = ref.round_bf16(np.random.default_rng(m + 1).standard_normal((m, cols)).astype(np.float32))
    dense_b = ref.round_bf16(ref.dequant(fmt, packed)).reshape(rows, cols)
    want = xb @ dense_b.T
    got = run_project_bf16(device, fmt, packed, rows, cols, xb, m).float().cpu().numpy().reshape(m, rows)
    assert np.isfinite(got).all()
    err = np.abs(got - want).max() / np.abs(want).max()
    assert err <= 6e-3, err
    # the same call again gives the same bits (fixed summation order)
    again = run_project_bf16(device, fmt, packed, rows, cols, xb, m).float().cpu().numpy().reshape(m, rows)
    assert np.array_equal(got, again)


@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("m", [100, 700])
def test_bf16_project_many_is_one_launch_with_the_same_bits(device, fmt, m):
    """q|k|v-like matrices sharing X at a prefill width: one tensor-core launch over all their row tiles returns
    what the separate projections return, bit for bit (whole tiles and K-split tail tiles alike)."""
    s = S()
    cols, rows = 1024, (300, 65, 128)
    xb = ref.round_bf16(np.random.default_rng(m).standard_normal((m, cols)).astype(np.float32))
    xt = dev_f32(xb).to(torch.bfloat16).contiguous()
    packed = [ref.random_matrix(fmt, r, cols, seed=50 + i) for i, r in enumerate(rows)]
    ws = [s.Matrix.from_packed(device, r, cols, 1, fmt, p) for r, p in zip(rows, packed)]
    alone = [torch.full((m * r,), float("nan"), dtype=torch.bfloat16, device="cuda") for r in rows]
    for w, y in zip(ws, alone):
        s.project(device, w, xt, m, y)
    fused = [torch.full((m * r,), float("nan"), dtype=torch.bfloat16, device="cuda") for r in rows]
    before = device.counters().dispatches
    s.project_many(device, ws, xt, m, fused)
    device.synchronize()
    for a, f, r, p in zip(alone, fused, rows, packed):
        assert torch.equal(a.view(torch.int16), f.view(torch.int16))
        want = xb.astype(np.float64) @ ref.round_bf16(ref.dequant(fmt, p)).reshape(r, cols).astype(np.float64).T
        assert np.abs(f.float().cpu().numpy().reshape(m, r) - want).max() / np.abs(want).max() <= 6e-3


@pytest.mark.parametrize("fmt", FORMATS)
def test_bf16_gemm_weight_tiles_are_bit_exact(device, fmt):
    """X = identity makes Y the weight tile itself: it must equal bf16_rne(exact fp32 decode) bit for bit."""
    rows, cols = 200, 512
    packed = blocks_for(fmt, rows, cols, "random", seed=77)
    eye = np.eye(cols, dtype=np.float32)
    y = run_project_bf16(device, fmt, packed, rows, cols, eye, cols)
    got = y.view(torch.int16).cpu().numpy().view(np.uint16).reshape(cols, rows)
    want = ref.to_bf16(ref.dequant(fmt, packed)).reshape(rows, cols).T
    # An accumulated sum cannot keep the sign of a zero weight (-0 + 0 = +0); everything else is bit-equal.
    zero = (want & 0x7FFF) == 0
    assert np.array_equal(got[~zero], want[~zero]) and not (got[zero] & 0x7FFF).any()


@pytest.mark.parametrize("fmt,rows,cols", [(ref.Q4_K, 6144, 5120), (ref.Q6_K, 5120, 17408)])
def test_full_size_prefill_rows(device, fmt, rows, cols):
    """Config 2 shapes at M = 512: a random subset of output rows against the oracle."""
    m = 512
    packed = ref.random_matrix(fmt, rows, cols, seed=11)
    xb = ref.round_bf16(np.random.default_rng(12).standard_normal((m, cols)).astype(np.float32))
    got = run_project_bf16(device, fmt, packed, rows, cols, xb, m).float().cpu().numpy().reshape(m, rows)
    rb = ref.row_bytes(fmt, cols)
    pick = np.sort(np.random.default_rng(5).choice(rows, 16, replace=False))
    sub = np.concatenate([packed[r * rb:(r + 1) * rb] for r in pick])
    dense_b = ref.round_bf16(ref.dequant(fmt, sub)).reshape(len(pick), cols)
    want = xb.astype(np.float64) @ dense_b.astype(np.float64).T
    assert np.abs(got[:, pick] - want).max() / np.abs(got).max() <= TOL_BF16
    assert np.isfinite(got).all()


def test_grouped_expert_gemm_config3_shape(device):
    """Config 3 geometry, scaled to 32 experts: gate 512 x 2048 Q4_K per expert, 1024 routes sorted by expert
    with uneven group sizes (some empty), F32 in / F32 out through the tensor-memory path."""
    s = S()
    experts, rows_e, cols, routes = 32, 512, 2048, 1024
    packed = ref.random_matrix(ref.Q4_K, experts * rows_e, cols, seed=61)
    w = s.Matrix.from_packed(device, rows_e, cols, experts, ref.Q4_K, packed)
    rng = np.random.default_rng(62)
    ids = np.sort(rng.integers(0, experts, routes)).astype(np.uint32)
    ids[ids == 7] = 8  # an expert nobody picked
    counts = np.bincount(ids, minlength=experts)
    offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.uint32)
    x = rng.standard_normal((routes, cols)).astype(np.float32)
    y = torch.full((routes * rows_e,), float("nan"), dtype=torch.float32, device="cuda")
    s.project_mm_id(device, w, dev_f32(x), dev_u32(offsets), int(counts.max()), y)
    device.synchronize()
    got = host(y).reshape(routes, rows_e)
    assert np.isfinite(got).all()
    pick = rng.choice(routes, 24, replace=False)
    rb = ref.row_bytes(ref.Q4_K, cols)
    for r in pick:
        e = int(ids[r])
        want = ref.matmul(ref.Q4_K, packed[e * rows_e * rb:(e + 1) * rows_e * rb], rows_e, cols, x[r], 1)[0]
        assert np.abs(got[r] - want).max() / np.abs(got).max() <= TOL_BF16
