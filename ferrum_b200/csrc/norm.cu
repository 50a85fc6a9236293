// The steps on either side of a projection: the row normalisation that produces its input and the reductions
// that consume the output head's logits.  Counterparts of `h_rmsnorm` / `h_add_rmsnorm`
// (src/metal/shaders/hybrid.metal:1563-1595; `HybridModel::rmsnorm` / `add_rmsnorm`, src/hybrid/engine.rs:3301-3345),
// `h_argmax` (:2214-2243) and `h_topk_blocks` (:3616-3657).  The normalisation is also available inside the
// activation preparation of the decode / verify projections (ProjectArgs::norm_w), with the same arithmetic.
#include "gemv_common.cuh"
#include "internal.h"

namespace {
using namespace fqk;

// One warp per row.
__global__ void __launch_bounds__(128)
k_rmsnorm(const float *__restrict__ x, const float *__restrict__ r, const float *__restrict__ w, uint32_t n, float eps, uint32_t rows,
          float *__restrict__ h, float *__restrict__ y) {
    const uint32_t row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float *xr = x + (size_t)row * n;
    if (r) { // h = x + r first; the norm is taken of h
        const float *rr = r + (size_t)row * n;
        float *hr = h + (size_t)row * n;
        for (uint32_t i = lane; i < n / 4; i += 32) {
            const float4 a = reinterpret_cast<const float4 *>(xr)[i], b = reinterpret_cast<const float4 *>(rr)[i];
            reinterpret_cast<float4 *>(hr)[i] = make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
        }
        __syncwarp();
        xr = hr;
    }
    const float scale = row_inv_rms(xr, n, eps, lane);
    float *yr = y + (size_t)row * n;
    for (uint32_t i = lane; i < n / 4; i += 32) {
        const float4 v = reinterpret_cast<const float4 *>(xr)[i], g = reinterpret_cast<const float4 *>(w)[i];
        reinterpret_cast<float4 *>(yr)[i] = make_float4(v.x * scale * g.x, v.y * scale * g.y, v.z * scale * g.z, v.w * scale * g.w);
    }
}

__device__ __forceinline__ void better(float &bv, uint32_t &bi, float ov, uint32_t oi) {
    if (ov > bv || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
    }
}

// One block of 1024 threads per row: the index of the first maximum.
__global__ void __launch_bounds__(1024)
k_argmax(const float *__restrict__ x, uint32_t n, uint32_t *__restrict__ out) {
    __shared__ float best_v[32];
    __shared__ uint32_t best_i[32];
    const uint32_t tid = threadIdx.x;
    x += (size_t)blockIdx.x * n;
    float bv = -INFINITY;
    uint32_t bi = 0;
    for (uint32_t i = tid; i < n; i += 1024) {
        const float v = x[i];
        if (v > bv) {
            bv = v;
            bi = i;
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) better(bv, bi, __shfl_down_sync(0xffffffffu, bv, off), __shfl_down_sync(0xffffffffu, bi, off));
    if ((tid & 31) == 0) {
        best_v[tid >> 5] = bv;
        best_i[tid >> 5] = bi;
    }
    __syncthreads();
    if (tid < 32) {
        bv = best_v[tid];
        bi = best_i[tid];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) better(bv, bi, __shfl_down_sync(0xffffffffu, bv, off), __shfl_down_sync(0xffffffffu, bi, off));
        if (tid == 0) out[blockIdx.x] = bi;
    }
}

// grid (ceil(n / 1024), rows), 256 threads: per 1024-value block the 32 largest (value, index) pairs in descending
// order, ties to the lower index; out[(row * blocks + block) * 32 + k] = {value, index bits}.
__global__ void __launch_bounds__(256)
k_topk_blocks(const float *__restrict__ x, uint32_t n, float2 *__restrict__ out) {
    __shared__ float sv[8];
    __shared__ uint32_t si[8];
    const uint32_t tid = threadIdx.x, block = blockIdx.x;
    x += (size_t)blockIdx.y * n;
    out += (size_t)blockIdx.y * ((n + 1023) / 1024) * 32;
    float v[4];
    uint32_t idx[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        idx[j] = block * 1024 + j * 256 + tid;
        v[j] = idx[j] < n ? x[idx[j]] : -INFINITY;
    }
    for (int k = 0; k < 32; k++) {
        float best = v[0];
        uint32_t bidx = idx[0];
        int slot = 0;
#pragma unroll
        for (int j = 1; j < 4; j++)
            if (v[j] > best || (v[j] == best && idx[j] < bidx)) {
                best = v[j];
                bidx = idx[j];
                slot = j;
            }
        float wv = best;
        uint32_t wi = bidx;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) better(wv, wi, __shfl_down_sync(0xffffffffu, wv, off), __shfl_down_sync(0xffffffffu, wi, off));
        if ((tid & 31) == 0) {
            sv[tid >> 5] = wv;
            si[tid >> 5] = wi;
        }
        __syncthreads();
        float gv = sv[0];
        uint32_t gi = si[0];
#pragma unroll
        for (int s = 1; s < 8; s++) better(gv, gi, sv[s], si[s]);
        __syncthreads();
        if (tid == 0) out[block * 32 + k] = make_float2(gv, __uint_as_float(gi));
        if (bidx == gi && best == gv) v[slot] = -INFINITY;
    }
}

int check_norm(fq_device *dev, const float *x, const float *w, uint32_t n, uint32_t rows, const float *y) {
    if (n == 0 || n % 4 || rows == 0) return fq_fail(dev, FQ_ERR_SHAPE, "normalisation of %u rows of %u values (a multiple of 4)", rows, n);
    if (int rc = fq_check_binding(dev, x, (size_t)rows * n * 4, "x")) return rc;
    if (int rc = fq_check_binding(dev, w, (size_t)n * 4, "w")) return rc;
    return fq_check_binding(dev, y, (size_t)rows * n * 4, "y");
}

} // namespace

extern "C" int fq_rmsnorm(fq_device *dev, const float *x, const float *w, uint32_t n, float eps, uint32_t rows, float *y) {
    if (int rc = fq_begin_enqueue(dev)) return rc;
    if (int rc = check_norm(dev, x, w, n, rows, y)) return rc;
    k_rmsnorm<<<(rows + 3) / 4, 128, 0, dev->stream>>>(x, nullptr, w, n, eps, rows, nullptr, y);
    return fq_end_enqueue(dev, "rmsnorm", 1);
}

extern "C" int fq_add_rmsnorm(fq_device *dev, const float *x, const float *r, const float *w, uint32_t n, float eps, uint32_t rows, float *h,
                              float *y) {
    if (int rc = fq_begin_enqueue(dev)) return rc;
    if (int rc = check_norm(dev, x, w, n, rows, y)) return rc;
    if (int rc = fq_check_binding(dev, r, (size_t)rows * n * 4, "r")) return rc;
    if (int rc = fq_check_binding(dev, h, (size_t)rows * n * 4, "h")) return rc;
    if (int rc = fq_check_no_alias(dev, y, (size_t)rows * n * 4, h, (size_t)rows * n * 4, "y")) return rc;
    k_rmsnorm<<<(rows + 3) / 4, 128, 0, dev->stream>>>(x, r, w, n, eps, rows, h, y);
    return fq_end_enqueue(dev, "add_rmsnorm", 1);
}

extern "C" int fq_argmax(fq_device *dev, const float *x, uint32_t n, uint32_t rows, uint32_t *out) {
    if (int rc = fq_begin_enqueue(dev)) return rc;
    if (n == 0 || rows == 0) return fq_fail(dev, FQ_ERR_SHAPE, "argmax of %u rows of %u values", rows, n);
    if (int rc = fq_check_binding(dev, x, (size_t)rows * n * 4, "x")) return rc;
    if (int rc = fq_check_binding(dev, out, (size_t)rows * 4, "out")) return rc;
    k_argmax<<<rows, 1024, 0, dev->stream>>>(x, n, out);
    return fq_end_enqueue(dev, "argmax", 1);
}

extern "C" int fq_topk_blocks(fq_device *dev, const float *x, uint32_t n, uint32_t rows, float *out) {
    if (int rc = fq_begin_enqueue(dev)) return rc;
    if (n == 0 || rows == 0) return fq_fail(dev, FQ_ERR_SHAPE, "top-k of %u rows of %u values", rows, n);
    const uint32_t blocks = (n + 1023) / 1024;
    if (int rc = fq_check_binding(dev, x, (size_t)rows * n * 4, "x")) return rc;
    if (int rc = fq_check_binding(dev, out, (size_t)rows * blocks * 32 * 8, "out")) return rc;
    k_topk_blocks<<<dim3(blocks, rows), 256, 0, dev->stream>>>(x, n, reinterpret_cast<float2 *>(out));
    return fq_end_enqueue(dev, "topk_blocks", 1);
}
