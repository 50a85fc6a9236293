"""Parity at the sizes the benchmark configurations state, and the failure paths that need a GPU but no fault.

Config 1: the o and gate/up shapes at decode and verify widths.  Config 2: M = 2048 on gate and down.  Config 3:
the whole MoE block with 256 experts, top-8, T = 1 and 1024 (sampled tokens against the oracle composition; the
reference's expert-path tests are src/hybrid/iq_tests.rs:1686-1814).  Failure paths: a device-side wait that
runs out (the counterpart of src/metal/mod.rs:1196-1303) and a router row without a ranking
(src/nn/moe.rs:392-397).
"""
import numpy as np
import pytest
import torch

from oracle import ref

pytestmark = pytest.mark.gpu

TOL_F32 = 1e-3
TOL_BF16 = 2e-2


def S():
    from ferrum_b200 import surface
    return surface


def dev_f32(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()


def host(t):
    return t.detach().float().cpu().numpy()


def dev_u32(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.uint32).view(np.int32)).cuda()


def rows_of(packed, fmt, cols, pick):
    rb = ref.row_bytes(fmt, cols)
    return np.concatenate([packed[r * rb:(r + 1) * rb] for r in pick])


@pytest.mark.parametrize("rows,cols", [(5120, 6144), (17408, 5120)])
@pytest.mark.parametrize("m", [1, 8, 16])
def test_config1_o_and_gate_shapes(device, rows, cols, m):
    s = S()
    fmt = ref.Q4_K
    packed = ref.random_matrix(fmt, rows, cols, seed=rows % 89)
    x = np.random.default_rng(m + 3).standard_normal((m, cols)).astype(np.float32)
    w = s.Matrix.from_packed(device, rows, cols, 1, fmt, packed)
    y = torch.full((m * rows,), float("nan"), dtype=torch.float32, device="cuda")
    s.project(device, w, dev_f32(x), m, y)
    device.synchronize()
    got = host(y).reshape(m, rows)
    assert np.isfinite(got).all()
    pick = np.sort(np.random.default_rng(6).choice(rows, 24, replace=False))
    want = ref.matmul(fmt, rows_of(packed, fmt, cols, pick), len(pick), cols, x, m, mode=0)
    assert np.abs(got[:, pick] - want).max() / np.abs(got).max() <= TOL_F32


@pytest.mark.parametrize("fmt,rows,cols", [(ref.Q4_K, 17408, 5120), (ref.Q6_K, 5120, 17408)])
def test_config2_m2048_rows(device, fmt, rows, cols):
    s = S()
    m = 2048
    packed = ref.random_matrix(fmt, rows, cols, seed=21)
    xb = ref.round_bf16(np.random.default_rng(22).standard_normal((m, cols)).astype(np.float32))
    w = s.Matrix.from_packed(device, rows, cols, 1, fmt, packed)
    y = torch.zeros(m * rows, dtype=torch.bfloat16, device="cuda")
    s.project(device, w, torch.from_numpy(xb).cuda().to(torch.bfloat16), m, y)
    device.synchronize()
    got = y.float().cpu().numpy().reshape(m, rows)
    assert np.isfinite(got).all()
    pick = np.sort(np.random.default_rng(7).choice(rows, 12, replace=False))
    dense_b = ref.round_bf16(ref.dequant(fmt, rows_of(packed, fmt, cols, pick))).reshape(len(pick), cols)
    want = xb.astype(np.float64) @ dense_b.astype(np.float64).T
    assert np.abs(got[:, pick] - want).max() / np.abs(got).max() <= TOL_BF16


def expert_rows(packed, fmt, rows_e, cols, e):
    rb = ref.row_bytes(fmt, cols)
    return packed[e * rows_e * rb:(e + 1) * rows_e * rb]


@pytest.fixture(scope="module")
def config3():
    experts, used, hidden, ef = 256, 8, 2048, 512
    mats = dict(router=ref.random_matrix(ref.Q8_0, experts, hidden, 70),
                gate=ref.random_matrix(ref.Q4_K, experts * ef, hidden, 71), up=ref.random_matrix(ref.Q4_K, experts * ef, hidden, 72),
                down=ref.random_matrix(ref.Q6_K, experts * hidden, ef, 73),
                sg=ref.random_matrix(ref.Q4_K, ef, hidden, 74), su=ref.random_matrix(ref.Q4_K, ef, hidden, 75),
                sd=ref.random_matrix(ref.Q6_K, hidden, ef, 76))
    return experts, used, hidden, ef, mats


@pytest.mark.parametrize("tokens", [1, 384, 1024, 2048])
def test_config3_moe_block(device, config3, tokens):
    """35B-A3B-class block: 256 experts + shared, top-8, hidden 2048, expert width 512.  T = 1 takes the per-route
    projections, T = 384 (12 rows per expert) the integer grouped kernel over expert-sorted rows, T = 1024 the fp16
    tensor-core grouped kernel, T = 2048 the same in two launches (the fp16 copy of the 16384 gathered rows does not
    fit the activation scratch at once); sampled tokens against the oracle."""
    s = S()
    experts, used, hidden, ef, mats = config3
    M = s.Matrix.from_packed
    f = s.MoeFfn(M(device, experts, hidden, 1, ref.Q8_0, mats["router"]), M(device, ef, hidden, experts, ref.Q4_K, mats["gate"]),
                 M(device, ef, hidden, experts, ref.Q4_K, mats["up"]), M(device, hidden, ef, experts, ref.Q6_K, mats["down"]),
                 M(device, ef, hidden, 1, ref.Q4_K, mats["sg"]), M(device, ef, hidden, 1, ref.Q4_K, mats["su"]),
                 M(device, hidden, ef, 1, ref.Q6_K, mats["sd"]), None, experts, used, hidden, ef, ef, False, True)
    x = (np.random.default_rng(tokens).standard_normal((tokens, hidden)) * 0.06).astype(np.float32)
    scratch = torch.zeros(s.moe_ffn_scratch_elems(device, f, tokens), dtype=torch.float32, device="cuda")
    out = torch.full((tokens * hidden,), float("nan"), dtype=torch.float32, device="cuda")
    s.moe_ffn(device, f, dev_f32(x), tokens, scratch, out)
    device.synchronize()
    got = host(out).reshape(tokens, hidden)
    assert np.isfinite(got).all()
    checked = 0
    for t in np.random.default_rng(9).permutation(tokens)[:12]:
        xt = x[t:t + 1]
        logits = ref.matmul(ref.Q8_0, mats["router"], experts, hidden, xt, 1)
        p = np.sort(np.exp(logits[0] - logits[0].max()))[::-1]
        if (p[used - 1] - p[used]) < 1e-3 * p[used - 1]:
            continue  # the eighth and ninth expert are too close for a 16-bit-activation router to be held to
        ids, wts, gate = ref.moe_route(logits, xt, xt[0], experts, used, hidden, 1, False, True, False)
        g = np.stack([ref.matmul(ref.Q4_K, expert_rows(mats["gate"], ref.Q4_K, ef, hidden, int(e)), ef, hidden, xt, 1)[0] for e in ids.ravel()])
        u = np.stack([ref.matmul(ref.Q4_K, expert_rows(mats["up"], ref.Q4_K, ef, hidden, int(e)), ef, hidden, xt, 1)[0] for e in ids.ravel()])
        act = ref.swiglu(g, u)
        dn = np.stack([ref.matmul(ref.Q6_K, expert_rows(mats["down"], ref.Q6_K, hidden, ef, int(e)), hidden, ef, act[i:i + 1], 1)[0]
                       for i, e in enumerate(ids.ravel())])
        gs = ref.matmul(ref.Q4_K, mats["sg"], ef, hidden, xt, 1)
        us = ref.matmul(ref.Q4_K, mats["su"], ef, hidden, xt, 1)
        shared = ref.matmul(ref.Q6_K, mats["sd"], hidden, ef, ref.swiglu(gs, us), 1)
        want = ref.moe_combine(dn, wts, ids, shared, gate, hidden, used, 1, identity=True)[0]
        assert np.abs(got[t] - want).max() / np.abs(want).max() <= 3 * TOL_F32, f"token {t}"
        checked += 1
        if checked == 4:
            break
    assert checked >= 1


def test_a_wait_for_an_absent_peer_runs_out(device):
    """A communicator of two ranks whose peer is a buffer nothing writes: the exchange kernels give up after the
    (shortened) wall-time limit, `synchronize` reports a timeout, and after `recover` the handle works again."""
    s = S()
    rows, cols = 256, 1024
    packed = ref.random_matrix(ref.Q4_K, rows, cols, seed=3)
    w = s.Matrix.from_packed(device, rows, cols, 1, ref.Q4_K, packed)
    x = np.random.default_rng(1).standard_normal((1, cols)).astype(np.float32)
    xd = dev_f32(x)
    comm = s.Comm(device, 0, 2, 1 << 16, local_peer=True)
    comm.set_wait_ns(2_000_000)  # 2 ms
    # The copy-kernel exchange.
    comm.all_gather(0, 1024)
    with pytest.raises(s.TimeoutError_):
        device.synchronize()
    device.recover()
    # The exchange fused into the projection kernel, at one and at four activation rows.
    for m, region in ((1, 8192), (4, 16384)):
        xm = dev_f32(np.repeat(x, m, axis=0))
        y = comm.view(region, m * rows)
        s.project_many_gather(device, comm, region, m * rows * 4, [w], xm, m, [y])
        with pytest.raises(s.TimeoutError_):
            device.synchronize()
        with pytest.raises(s.SynchronizationError):
            s.project(device, w, xd, 1, torch.zeros(rows, dtype=torch.float32, device="cuda"))  # a failed handle refuses work
        device.recover()
        # the local slice was computed all the same
        want = ref.matmul(ref.Q4_K, packed, rows, cols, np.repeat(x, m, axis=0), m)
        assert ref.rel_err(host(y).reshape(m, rows), want) <= TOL_F32
    # Reusing the region of the exchange before is refused up front.
    with pytest.raises(s.ParameterError):
        comm.all_gather(16384, 1024)
    comm.close()
    out = torch.zeros(rows, dtype=torch.float32, device="cuda")
    s.project(device, w, xd, 1, out)
    device.synchronize()
    assert ref.rel_err(host(out).reshape(1, rows), ref.matmul(ref.Q4_K, packed, rows, cols, x, 1)) <= TOL_F32


def test_router_refuses_logits_without_a_ranking(device):
    """A NaN or an infinity among the logits: the token gets in-range experts with zero weight, nothing reads out
    of range, and `synchronize` reports the row as the reference's router does."""
    s = S()
    experts, used, hidden, tokens = 64, 8, 128, 5
    rng = np.random.default_rng(2)
    logits = rng.standard_normal((tokens, experts)).astype(np.float32)
    logits[1, 7] = np.nan
    logits[3, 0] = np.inf
    x = rng.standard_normal((tokens, hidden)).astype(np.float32)
    ids = torch.full((tokens * used,), -1, dtype=torch.int32, device="cuda")
    wts = torch.full((tokens * used,), float("nan"), dtype=torch.float32, device="cuda")
    gate = torch.zeros(tokens, dtype=torch.float32, device="cuda")
    s.moe_route(device, dev_f32(logits), dev_f32(x), dev_f32(x[0]), experts, used, hidden, tokens, False, True, False, ids, wts, gate)
    with pytest.raises(s.WeightError):
        device.synchronize()
    device.recover()
    got_ids = ids.cpu().numpy().view(np.uint32).reshape(tokens, used)
    assert (got_ids < experts).all()
    assert (wts.cpu().numpy().reshape(tokens, used)[[1, 3]] == 0).all()
    want_ids, want_w, _ = ref.moe_route(logits[[0, 2, 4]], x[[0, 2, 4]], x[0], experts, used, hidden, 3, False, True, False)
    assert np.array_equal(got_ids[[0, 2, 4]], want_ids.reshape(3, used))


def test_matrices_load_from_a_gguf_file(device, tmp_path):
    """A GGUF file the test writes itself (Q4_K dense, Q5_K dense, Q6_K experts, Q3_K dense): `from_gguf` checks the
    geometry, reads the payload, rewrites Q3_K as Q6_K, and the projections match the oracle on the stored bytes
    (src/hybrid/weights.rs:671-736; src/hybrid/iq_tests.rs:1529-1560 for the Q3_K case)."""
    import struct
    s = S()

    def gstr(t):
        b = t.encode()
        return struct.pack("<Q", len(b)) + b
    rows, cols, experts = 48, 1024, 3
    payloads = {"blk.0.attn_q.weight": (ref.Q4_K, [cols, rows], ref.random_matrix(ref.Q4_K, rows, cols, 1)),
                "blk.0.attn_k.weight": (ref.Q5_K, [cols, rows], ref.random_matrix(ref.Q5_K, rows, cols, 2)),
                "blk.0.ffn_down_exps.weight": (ref.Q6_K, [cols, rows, experts], ref.random_matrix(ref.Q6_K, experts * rows, cols, 3)),
                "mtp.ffn_up.weight": (ref.Q3_K, [cols, rows], ref.random_matrix(ref.Q3_K, rows, cols, 4))}
    md = [gstr("general.architecture") + struct.pack("<I", 8) + gstr("test"), gstr("general.quantization_version") + struct.pack("<II", 4, 2)]
    head = b"GGUF" + struct.pack("<IQQ", 3, len(payloads), len(md)) + b"".join(md)
    data, offsets = bytearray(), {}
    for name, (fmt, dims, packed) in payloads.items():
        data += b"\0" * ((-len(data)) % 32)
        offsets[name] = len(data)
        data += packed.tobytes()
    for name, (fmt, dims, packed) in payloads.items():
        head += gstr(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", fmt, offsets[name])
    head += b"\0" * ((-len(head)) % 32)
    path = tmp_path / "model.gguf"
    path.write_bytes(head + bytes(data))
    f = s.GgufFile(str(path))
    x = np.random.default_rng(5).standard_normal((2, cols)).astype(np.float32)
    for name, fmt in (("blk.0.attn_q.weight", ref.Q4_K), ("blk.0.attn_k.weight", ref.Q5_K)):
        w = s.Matrix.from_gguf(device, f, name, 1, rows, cols)
        assert (w.rows, w.cols, w.format) == (rows, cols, fmt)
        y = torch.zeros(2 * rows, dtype=torch.float32, device="cuda")
        s.project(device, w, dev_f32(x), 2, y)
        device.synchronize()
        assert ref.rel_err(host(y).reshape(2, rows), ref.matmul(fmt, payloads[name][2], rows, cols, x, 2)) <= TOL_F32
    # experts: [experts, rows, cols] stacked
    we = s.Matrix.from_gguf(device, f, "blk.0.ffn_down_exps.weight", experts, rows, cols)
    assert (we.rows, we.experts) == (experts * rows, experts)
    ids = torch.tensor([2, 0], dtype=torch.int32, device="cuda")
    y = torch.zeros(2 * rows, dtype=torch.float32, device="cuda")
    s.project_id(device, we, dev_f32(x), ids, 2, 1, y)
    device.synchronize()
    want = ref.matmul_id(ref.Q6_K, payloads["blk.0.ffn_down_exps.weight"][2], rows, cols, x, np.array([2, 0], dtype=np.uint32), 1)
    assert ref.rel_err(host(y).reshape(2, rows), want) <= TOL_F32
    # Q3_K: refused as it is, loaded as Q6_K on request, equal to the Q3_K CPU dequant
    with pytest.raises(s.WeightError, match="no kernel"):
        s.Matrix.from_gguf(device, f, "mtp.ffn_up.weight", 1, rows, cols)
    w3 = s.Matrix.from_gguf(device, f, "mtp.ffn_up.weight", 1, rows, cols, q3k_as_q6k=True)
    assert w3.format == ref.Q6_K
    y = torch.zeros(2 * rows, dtype=torch.float32, device="cuda")
    s.project(device, w3, dev_f32(x), 2, y)
    device.synchronize()
    assert ref.rel_err(host(y).reshape(2, rows), ref.matmul(ref.Q3_K, payloads["mtp.ffn_up.weight"][2], rows, cols, x, 2)) <= TOL_F32
    # geometry the caller expects must be the file's
    with pytest.raises(s.WeightError, match="expected GGUF dims"):
        s.Matrix.from_gguf(device, f, "blk.0.attn_q.weight", 1, rows + 1, cols)
    with pytest.raises(s.GgufError, match="missing tensor"):
        s.Matrix.from_gguf(device, f, "blk.9.attn_q.weight", 1, rows, cols)


@pytest.mark.parametrize("rows,n", [(1, 5120), (3, 2048), (40, 1024)])
def test_rmsnorm_and_add_rmsnorm(device, rows, n):
    """`h_rmsnorm` / `h_add_rmsnorm` against the reference's CPU rmsnorm (f64), src/reference.rs:23-36."""
    s = S()
    rng = np.random.default_rng(rows)
    x = rng.standard_normal((rows, n)).astype(np.float32) * 3
    r = rng.standard_normal((rows, n)).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(n)).astype(np.float32)
    eps = 1e-6
    y = torch.zeros(rows * n, dtype=torch.float32, device="cuda")
    s.rmsnorm(device, dev_f32(x), dev_f32(w), eps, rows, y)
    device.synchronize()
    want = ref.rmsnorm(x, w, eps)
    assert np.abs(host(y).reshape(rows, n) - want).max() <= 2e-6 * np.abs(want).max()
    h = torch.zeros(rows * n, dtype=torch.float32, device="cuda")
    y2 = torch.zeros(rows * n, dtype=torch.float32, device="cuda")
    s.add_rmsnorm(device, dev_f32(x), dev_f32(r), dev_f32(w), eps, rows, h, y2)
    device.synchronize()
    assert np.array_equal(host(h).reshape(rows, n), x + r)
    want2 = ref.rmsnorm(x + r, w, eps)
    assert np.abs(host(y2).reshape(rows, n) - want2).max() <= 2e-6 * np.abs(want2).max()


@pytest.mark.parametrize("fmt", [ref.Q4_K, ref.Q6_K])
@pytest.mark.parametrize("m", [1, 5, 16, 40])
def test_rmsnorm_folded_into_the_projection(device, fmt, m):
    """rmsnorm inside the activation preparation (m <= 16) gives the bits of rmsnorm followed by the projections,
    and both match the oracle; m = 40 takes the two-step route of the same call."""
    s = S()
    cols, rows = 2048, (96, 40)
    packed = [ref.random_matrix(fmt, r, cols, seed=50 + i) for i, r in enumerate(rows)]
    ws = [s.Matrix.from_packed(device, r, cols, 1, fmt, p) for r, p in zip(rows, packed)]
    rng = np.random.default_rng(m)
    x = (rng.standard_normal((m, cols)) * 2).astype(np.float32)
    nw = (1 + 0.1 * rng.standard_normal(cols)).astype(np.float32)
    eps = 1e-5
    xd, nwd = dev_f32(x), dev_f32(nw)
    fused = [torch.zeros(m * r, dtype=torch.float32, device="cuda") for r in rows]
    scratch = torch.zeros(m * cols, dtype=torch.float32, device="cuda")
    s.rmsnorm_project_many(device, ws, xd, nwd, eps, m, fused, scratch)
    device.synchronize()
    normed = torch.zeros(m * cols, dtype=torch.float32, device="cuda")
    s.rmsnorm(device, xd, nwd, eps, m, normed)
    two = [torch.zeros(m * r, dtype=torch.float32, device="cuda") for r in rows]
    s.project_many(device, ws, normed, m, two)
    device.synchronize()
    xn = ref.rmsnorm(x, nw, eps)
    for yf, yt, p, r in zip(fused, two, packed, rows):
        assert torch.equal(yf, yt)
        tol = TOL_F32 if m <= 16 else 1e-3
        assert ref.rel_err(host(yf).reshape(m, r), ref.matmul(fmt, p, r, cols, xn, m)) <= tol


def test_argmax_and_topk_blocks(device):
    """`h_argmax` and `h_topk_blocks`: exact indices, ties to the lower index."""
    s = S()
    rng = np.random.default_rng(8)
    rows, n = 3, 5000
    x = rng.standard_normal((rows, n)).astype(np.float32)
    x[0, 77] = x[0, 4000] = 9.5       # a tie for the maximum: the first wins
    x[1, 1024:1060] = 3.25            # ties inside a block
    x[2, :] = -np.inf                 # nothing to rank: index 0
    out = torch.zeros(rows, dtype=torch.int32, device="cuda")
    s.argmax(device, dev_f32(x), n, rows, out)
    blocks = (n + 1023) // 1024
    top = torch.zeros(rows * blocks * 32 * 2, dtype=torch.float32, device="cuda")
    s.topk_blocks(device, dev_f32(x), n, rows, top)
    device.synchronize()
    assert np.array_equal(out.cpu().numpy().view(np.uint32), ref.argmax_first(x))
    got = top.cpu().numpy().reshape(rows, blocks, 32, 2)
    vals, idx = ref.topk_blocks(x)
    assert np.array_equal(got[..., 0].view(np.uint32)[:2], vals.view(np.uint32)[:2])
    assert np.array_equal(np.ascontiguousarray(got[..., 1]).view(np.uint32)[:2], idx[:2])
    # the head of the vocabulary for a 65,536-row logit vector, one row
    big = rng.standard_normal((1, 65536)).astype(np.float32)
    out1 = torch.zeros(1, dtype=torch.int32, device="cuda")
    s.argmax(device, dev_f32(big), 65536, 1, out1)
    device.synchronize()
    assert int(out1.item()) == int(np.argmax(big))


def test_profile_table_names_times_and_clears(device):
    """`set_profiling` / `take_profile` (src/metal/mod.rs:636-676): per-operation calls and device times keyed by
    name; taking the table clears it; switching profiling off stops the recording."""
    s = S()
    rows, cols = 2048, 2048
    w = s.Matrix.from_packed(device, rows, cols, 1, ref.Q4_K, ref.random_matrix(ref.Q4_K, rows, cols, seed=41))
    x1 = dev_f32(np.random.default_rng(5).standard_normal(cols))
    x8 = dev_f32(np.random.default_rng(6).standard_normal((8, cols)))
    y1 = torch.zeros(rows, dtype=torch.float32, device="cuda")
    y8 = torch.zeros(8 * rows, dtype=torch.float32, device="cuda")
    device.set_profiling(True)
    for _ in range(3):
        s.project(device, w, x1, 1, y1)
    s.project(device, w, x8, 8, y8)
    s.rmsnorm(device, x8, x1, 1e-6, 8, y8[:8 * cols])
    table = device.take_profile()
    assert list(table) == sorted(table)
    assert table["gemv_i8s"]["calls"] == 3 and table["gemv_i8s"]["gpu_samples"] == 3 and table["gemv_i8s"]["kernels"] == 3
    assert table["gemv_nt"]["calls"] == 1 and table["gemv_nt"]["kernels"] == 2
    assert table["rmsnorm"]["calls"] == 1
    for e in table.values():
        assert e["gpu_ns"] > 0 and e["wall_ns"] > 0
        assert e["gpu_ns"] < 50_000_000  # milliseconds at most for these launches
    assert device.take_profile() == {}
    device.set_profiling(False)
    s.project(device, w, x1, 1, y1)
    assert device.take_profile() == {}
    # inside a capture an enqueue is counted but has no device time of its own
    device.set_profiling(True)
    device.capture_begin()
    s.project(device, w, x1, 1, y1)
    g = device.capture_end()
    g.launch()
    table = device.take_profile()
    assert table["gemv_i8s"]["calls"] == 1 and table["gemv_i8s"]["gpu_samples"] == 0
    device.set_profiling(False)
    device.synchronize()


@pytest.mark.parametrize("fmt,rows_e,cols", [(ref.Q4_K, 512, 2048), (ref.Q6_K, 2048, 512), (ref.Q4_K, 200, 768), (ref.Q6_K, 136, 256)])
def test_grouped_rows_at_about_thirty_to_an_expert(device, fmt, rows_e, cols):
    """`project_mm_id` with about 30 rows per expert (config 3's grouped widths): the fp16 tensor-core kernel
    (weights within 2^-11 of their value, activations to 22 bits) where the weight-row count is a multiple of 16,
    the integer kernel (exact integer products with 16-bit activations) elsewhere; the fp32 GEMV bar applies to
    both.  Uneven groups, an empty expert, a group of more than 32 rows, weight-row counts that are not a
    multiple of 16 x 8."""
    s = S()
    experts, routes = 24, 24 * 30
    packed = ref.random_matrix(fmt, experts * rows_e, cols, seed=71)
    w = s.Matrix.from_packed(device, rows_e, cols, experts, fmt, packed)
    rng = np.random.default_rng(72)
    ids = np.sort(rng.integers(0, experts, routes)).astype(np.uint32)
    ids[ids == 5] = 6   # an expert nobody picked, and one with about twice the rows
    counts = np.bincount(ids, minlength=experts)
    offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.uint32)
    x = rng.standard_normal((routes, cols)).astype(np.float32)
    y = torch.full((routes * rows_e,), float("nan"), dtype=torch.float32, device="cuda")
    s.project_mm_id(device, w, dev_f32(x), dev_u32(offsets), int(counts.max()), y)
    device.synchronize()
    got = host(y).reshape(routes, rows_e)
    assert np.isfinite(got).all()
    rb = ref.row_bytes(fmt, cols)
    worst = 0.0
    for r in rng.choice(routes, 40, replace=False):
        e = int(ids[r])
        want = ref.matmul(fmt, packed[e * rows_e * rb:(e + 1) * rows_e * rb], rows_e, cols, x[r], 1)[0]
        worst = max(worst, np.abs(got[r] - want).max() / np.abs(want).max())
    assert worst <= TOL_F32, worst


@pytest.mark.parametrize("fmt,rows_e,cols", [(ref.Q4_K, 512, 2048), (ref.Q6_K, 208, 512), (ref.Q4_K, 400, 256)])
def test_grouped_rows_on_the_fp16_kernel(device, fmt, rows_e, cols):
    """`project_mm_id` at about 70 rows per expert: groups of more than 64 rows (two activation tiles), of exactly
    64, of one row, an empty one; weight-row counts that end inside a 256-row tile; expert slots.  fp32 GEMV bar."""
    s = S()
    experts = 12
    counts = np.array([70, 0, 150, 64, 1, 65, 33, 128, 90, 17, 100, 122], dtype=np.int64)
    routes = int(counts.sum())
    packed = ref.random_matrix(fmt, experts * rows_e, cols, seed=81)
    w = s.Matrix.from_packed(device, rows_e, cols, experts, fmt, packed)
    rng = np.random.default_rng(82)
    slots = rng.permutation(experts).astype(np.uint32)   # group z is served by expert slots[z]
    offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.uint32)
    group_of = np.repeat(np.arange(experts), counts)
    x = (rng.standard_normal((routes, cols)) * np.exp(rng.uniform(-6, 6, (routes, 1)))).astype(np.float32)  # rows of very different scale
    y = torch.full((routes * rows_e,), float("nan"), dtype=torch.float32, device="cuda")
    s.project_mm_id_in(device, w, dev_f32(x), dev_u32(offsets), (dev_u32(slots), experts), int(counts.max()), y)
    device.synchronize()
    got = host(y).reshape(routes, rows_e)
    assert np.isfinite(got).all()
    rb = ref.row_bytes(fmt, cols)
    worst = 0.0
    picks = list(rng.choice(routes, 30, replace=False)) + [int(offsets[2]), int(offsets[3]) - 1, int(offsets[4]), routes - 1]
    for r in picks:
        e = int(slots[group_of[r]])
        want = ref.matmul(fmt, packed[e * rows_e * rb:(e + 1) * rows_e * rb], rows_e, cols, x[r], 1)[0]
        worst = max(worst, np.abs(got[r] - want).max() / np.abs(want).max())
    assert worst <= TOL_F32, worst
