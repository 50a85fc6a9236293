"""The allocation-free decode projection, `fq_gemv_q4k_static`, against `fq_project`.

Some users of this library cannot allocate device memory when they call it: an inference server whose
memory pool has already claimed the whole GPU, a plugin loaded into a host process that owns the
allocator, a real-time section where a cudaMalloc would stall every stream.  They cannot create a
device handle or a matrix handle (both allocate), so they call this entry point with raw device
pointers; its scratch is a fixed array inside the library.  The test drives it through the C ABI on
buffers the caller (here: torch) already owns, twice in a row with different activations, because the
second call reuses the array the first one filled.

This file sorts last on purpose: a run that stops at the first failure has then run everything else.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import ref

pytestmark = pytest.mark.gpu

TOL_F32 = 1e-3  # the bar of the other fp32 projection tests


def call_static(lib, w_dev, rows, cols, x_dev, m, y_dev, stream):
    err = C.create_string_buffer(256)
    rc = lib.fq_gemv_q4k_static(C.c_void_p(w_dev.data_ptr()), rows, cols, C.c_void_p(x_dev.data_ptr()), m,
                                C.c_void_p(y_dev.data_ptr()), C.c_void_p(stream), err, len(err))
    return rc, err.value.decode()


@pytest.mark.parametrize("m", [1, 2, 3, 4])
def test_static_entry_point_matches_project(m):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from ferrum_b200 import _lib, surface as S
    lib = _lib.load()
    rows, cols = 200, 2048
    packed = ref.random_matrix(ref.Q4_K, rows, cols, seed=41)
    torch.cuda.set_device(0)
    w_dev = torch.from_numpy(packed).cuda()      # the caller's own copy of the GGUF bytes
    x_dev = torch.zeros(m * cols, dtype=torch.float32, device="cuda")
    y_dev = torch.full((m * rows,), float("nan"), dtype=torch.float32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    d = S.Device(0)                               # the existing path, for comparison
    w = S.Matrix.from_packed(d, rows, cols, 1, ref.Q4_K, packed)
    y_ref = torch.zeros(m * rows, dtype=torch.float32, device="cuda")
    for call in range(2):                         # the second call reuses the library's fixed scratch
        x = (np.random.default_rng(100 + call).standard_normal((m, cols)) * (1.0 + 50 * call)).astype(np.float32)
        x_dev.copy_(torch.from_numpy(x).reshape(-1))
        y_dev.fill_(float("nan"))
        rc, msg = call_static(lib, w_dev, rows, cols, x_dev, m, y_dev, stream)
        assert rc == _lib.OK, msg
        S.project(d, w, x_dev, m, y_ref)
        d.synchronize()
        torch.cuda.synchronize()
        got, want = y_dev.cpu().numpy().reshape(m, rows), y_ref.cpu().numpy().reshape(m, rows)
        assert np.isfinite(got).all()
        assert ref.rel_err(got, want) <= TOL_F32
        assert ref.rel_err(got, ref.matmul(ref.Q4_K, packed, rows, cols, x, m)) <= TOL_F32


def test_static_entry_point_rejects_what_does_not_fit():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from ferrum_b200 import _lib
    lib = _lib.load()
    torch.cuda.set_device(0)
    buf = torch.zeros(4096, dtype=torch.float32, device="cuda")
    rc, msg = call_static(lib, buf, 16, 65536, buf, 4, buf, 0)  # 4 rows x 65536 activations: beyond the fixed scratch
    assert rc == _lib.ERR_SHAPE and "fixed scratch" in msg
    rc, msg = call_static(lib, buf, 16, 512, buf, 5, buf, 0)    # more activation rows than it serves
    assert rc == _lib.ERR_SHAPE and "activation rows" in msg
    rc, msg = call_static(lib, buf, 16, 300, buf, 1, buf, 0)    # not whole superblocks
    assert rc == _lib.ERR_SHAPE
    w = torch.zeros(16 * 288, dtype=torch.uint8, device="cuda")  # 16 rows of 512 Q4_K weights
    rc, msg = call_static(lib, w, 16, 512, buf, 1, buf[256:], 0)  # the output lies inside the activations
    assert rc == _lib.ERR_ALIAS and "overlaps" in msg
