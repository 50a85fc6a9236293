/*
 * ferrum_b200 — C ABI of the B200 (sm_100a) K-quant dequantize-and-multiply library.
 *
 * This is the boundary a Ferrum build binds in place of `MetalDevice::dispatch_hybrid` for the
 * quantized-linear op surface.  Each entry point names the reference interface it replaces
 * (paths are relative to the reference crate).  Conventions shared by all of them:
 *
 *   - every call returns an `fq_status`; nothing aborts; `fq_last_error` gives the message;
 *   - work is ENQUEUED on the device handle's CUDA stream and runs asynchronously, like the
 *     reference's command epochs (src/metal/mod.rs:456, 563-633); `fq_synchronize` is the only
 *     blocking call and the place where asynchronous failures surface;
 *   - weights are immutable packed GGUF blocks owned by the library behind `fq_matrix`
 *     (src/tensor/mod.rs:336-385); activations and outputs are caller-owned DEVICE pointers,
 *     16-byte aligned, that must not overlap one another (src/metal/mod.rs:854-896);
 *   - nothing allocates device memory after `fq_device_create` / `fq_matrix_create`
 *     (the reference: "nothing allocates after load");
 *   - handles are not thread-safe: one host thread per device handle
 *     (the reference's handles are `Rc`, `!Send`, `!Sync`).
 */
#ifndef FERRUM_B200_H
#define FERRUM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct fq_device fq_device;
typedef struct fq_matrix fq_matrix;

/* src/error.rs: Shape, Range, DeviceMismatch, Dispatch("alias"), Weight, Synchronization, Gguf. */
typedef enum fq_status {
    FQ_OK = 0,
    FQ_ERR_SHAPE = 1,       /* element counts do not match the matrix geometry */
    FQ_ERR_RANGE = 2,       /* a binding is null, misaligned or outside its allocation */
    FQ_ERR_DEVICE = 3,      /* a handle or pointer belongs to another device */
    FQ_ERR_ALIAS = 4,       /* an output overlaps an input or another output */
    FQ_ERR_WEIGHT = 5,      /* packed payload rejected (length, block count, non-finite scale) */
    FQ_ERR_SYNC = 6,        /* asynchronous failure reported at enqueue or synchronize */
    FQ_ERR_TIMEOUT = 7,     /* a bounded device-side wait gave up */
    FQ_ERR_CUDA = 8,        /* CUDA runtime error */
    FQ_ERR_PARAM = 9,       /* invalid argument */
    FQ_ERR_UNSUPPORTED = 10,/* format / dtype combination without a kernel */
    FQ_ERR_GGUF = 11        /* a GGUF file is malformed, truncated or lacks what was asked for */
} fq_status;

/* GGML type ids, as in `Format::from_type` (src/hybrid/weights.rs:47-66) and
 * `QuantizationFormat` (src/quantization.rs:24-73).  Q8_0, Q4_K, Q5_K and Q6_K have kernels at every width.
 * IQ4_NL and IQ4_XS decode exactly everywhere (embedding lookup, every projection entry point) but have a tuned
 * kernel only for one activation row; at other widths they run on the exact fp32 kernels. */
typedef enum fq_format { FQ_Q8_0 = 8, FQ_Q4_K = 12, FQ_Q5_K = 13, FQ_Q6_K = 14, FQ_IQ4_NL = 20, FQ_IQ4_XS = 23 } fq_format;

/* Activation / output element types (GGML ids of F32 and BF16). */
typedef enum fq_dtype { FQ_F32 = 0, FQ_BF16 = 30 } fq_dtype;

/* `Matrix{rows, cols, experts, format, row_bytes}` (src/hybrid/weights.rs:107-115).
 * `rows` counts all experts' rows (rows_per_expert * experts). */
typedef struct fq_matrix_info {
    uint64_t rows, cols, experts, row_bytes, byte_size;
    int32_t format;
} fq_matrix_info;

/* `Counters` (src/metal/mod.rs:209-228): kernels enqueued and synchronisations since creation. */
typedef struct fq_counters {
    uint64_t dispatches, synchronizes, bytes_uploaded, bytes_downloaded;
} fq_counters;

/* ---- device, stream, errors ------------------------------------------------------------ */

/* `MetalDevice::new` (src/metal/mod.rs:480-560).  Creates the stream and the fixed scratch. */
int fq_device_create(int ordinal, fq_device **out);
int fq_device_destroy(fq_device *dev);
/* Enqueue on a caller-provided `cudaStream_t` (NULL restores the handle's own stream). */
int fq_device_set_stream(fq_device *dev, void *cuda_stream);
void *fq_device_stream(fq_device *dev);
/* `MetalDevice::synchronize` (src/metal/mod.rs:633): blocks; reports asynchronous errors as
 * FQ_ERR_SYNC and leaves the handle refusing further enqueues until `fq_device_recover`. */
int fq_synchronize(fq_device *dev);
int fq_device_recover(fq_device *dev);
const char *fq_last_error(fq_device *dev);
const char *fq_status_name(int status);
int fq_get_counters(fq_device *dev, fq_counters *out);
/* `FERRUM_HYBRID_EXACT` (src/hybrid/engine.rs:3435-3461, 3532-3563): when on, every projection
 * runs the fp32 GEMV that decodes weights with the exact per-value formula, at any M. */
int fq_set_exact(fq_device *dev, int on);
/* Test-only host-side fault injection, the counterpart of `fail_after` / `fail_completion`
 * (src/metal/mod.rs:368-371, 617-620, 846-853): the n-th enqueue from now fails with
 * FQ_ERR_SYNC before anything is launched (n < 0 disarms); `fq_test_fail_completion` makes the
 * next `fq_synchronize` report a failure.  No GPU fault is produced. */
int fq_test_fail_after(fq_device *dev, int n);
int fq_test_fail_completion(fq_device *dev);

/* Opt-in per-operation measurements, the counterpart of `set_profiling` / `take_profile` / `ProfileEntry`
 * (src/metal/mod.rs:636-676, 231-242).  While profiling is on every enqueue is bracketed by a pair of CUDA
 * events on its stream (outside graph capture; a captured enqueue is counted without a device time) and keyed
 * by the operation's name ("gemv_i8s", "gemv_nt", "gemm_tc", "moe_route", ...).  `fq_set_profiling` switches it
 * and clears the table.  `fq_take_profile` waits for the stream, resolves the events, writes up to `capacity`
 * entries in name order, stores the number of entries the table holds in `*count`, and clears the table when
 * all of them fitted.  `wall_ns` is host time spent enqueueing, `gpu_ns` the sum over the `gpu_samples` timed
 * calls of the device time between the operation's first and last kernel (operations of one stream run in
 * order, so this includes waiting behind the operation before it). */
typedef struct fq_profile_entry {
    char name[48];
    uint64_t calls, kernels, wall_ns, gpu_ns, gpu_samples;
} fq_profile_entry;
int fq_set_profiling(fq_device *dev, int on);
int fq_take_profile(fq_device *dev, fq_profile_entry *out, size_t capacity, size_t *count);

/* Diagnostic: enqueues a kernel that only READS `bytes` bytes at `data` (16 bytes per thread and step, the
 * weight-streaming loads of the projection kernels, `blocks_per_sm` blocks of 256 threads per SM): timed by the
 * caller it gives the read-only streaming ceiling of the device, the counterpart of the reference's `h_bw_read`
 * probe (src/hybrid/bench.rs:140-167). */
int fq_probe_read_stream(fq_device *dev, const void *data, size_t bytes, uint32_t blocks_per_sm);

/* ---- batched submission ------------------------------------------------------------------- */

/* The reference batches the dispatches of a forward pass into one command epoch
 * (`execution_with_shared_encoder`, src/metal/mod.rs:563-633) because a 27B decode step is ~930
 * small dispatches.  The CUDA counterpart is a captured graph: every enqueue between
 * `fq_capture_begin` and `fq_capture_end` is recorded instead of run (on the handle's OWN stream; a
 * caller-provided stream must be restored first), and `fq_graph_launch` replays the whole batch with
 * one submission.  Pointers and shapes are baked in; `fq_synchronize` is refused while capturing. */
typedef struct fq_graph fq_graph;
int fq_capture_begin(fq_device *dev);
int fq_capture_end(fq_device *dev, fq_graph **out);
int fq_graph_launch(fq_device *dev, fq_graph *graph);
int fq_graph_destroy(fq_graph *graph);

/* ---- caller-visible device buffers (src/metal/mod.rs:700-760 `buffer`, Tensor::from_f32) ---
 * For buffers allocated here the handle remembers what each submission writes: when a completion point
 * (`fq_synchronize`, `fq_download`) fails, the ranges written since the last one are refused as inputs
 * (FQ_ERR_SYNC) until a later submission that writes them again has completed -- src/metal/mod.rs:865-873.
 * Memory allocated elsewhere is accepted everywhere but is not tracked. */
int fq_buffer_alloc(fq_device *dev, size_t bytes, void **device_ptr);
int fq_buffer_free(fq_device *dev, void *device_ptr);
int fq_upload(fq_device *dev, void *device_ptr, const void *host, size_t bytes);
/* `fq_download` waits for the data (a read of results is a completion point, as `Tensor::to_f32`
 * is in the reference); `fq_download_async` only enqueues the copy -- `host` should be pinned -- and
 * the data is valid after the next `fq_synchronize`. */
int fq_download(fq_device *dev, void *host, const void *device_ptr, size_t bytes);
int fq_download_async(fq_device *dev, void *host, const void *device_ptr, size_t bytes);

/* ---- weights ----------------------------------------------------------------------------- */

/* `Matrix::from_packed` / `gguf_matrix` (src/hybrid/weights.rs:671-736, 1301-1330) with the
 * payload checks of `validate_gguf_quantized_payload` (src/quantization.rs:212-261).
 * `packed` is HOST memory holding `experts` stacked slices of `rows` rows, each row
 * cols/block_elements GGUF blocks; `len` must equal the geometry.  `cols` must be a whole number
 * of blocks and a multiple of 64 (`PROJECTION_K_STEP`). */
int fq_matrix_create(fq_device *dev, int format, uint64_t rows, uint64_t cols, uint64_t experts,
                     const void *packed, size_t len, fq_matrix **out);
int fq_matrix_destroy(fq_matrix *w);
int fq_matrix_get_info(const fq_matrix *w, fq_matrix_info *out);

/* ---- GGUF files ------------------------------------------------------------------------------ */

/* `GgufReader` (src/loader/gguf.rs:162-530): a bounds-checked index of a GGUF v2 / v3 file -- header, metadata,
 * tensor descriptors with the block layouts of `block_layout` (:87-121), alignment (`general.alignment`,
 * default 32), every tensor range inside the file and no two overlapping -- and tensor payloads read on demand.
 * `require_architecture` = 0 is `open_untagged` (tensor-only files: no `general.architecture`, names up to 256
 * bytes); `skip_arrays_over` > 0 is `from_reader_skipping_arrays` (longer metadata arrays are skipped and read
 * back empty).  On failure the message goes to `err` (may be NULL) and the status is FQ_ERR_GGUF. */
typedef struct fq_gguf fq_gguf;
typedef struct fq_gguf_tensor {
    char name[260];
    uint32_t n_dims;
    uint64_t dims[4];  /* GGUF order: dims[0] is the contiguous dimension */
    uint32_t type_id;
    uint64_t offset;   /* relative to the tensor-data section */
    uint64_t byte_len;
} fq_gguf_tensor;
typedef struct fq_gguf_info_t {
    uint32_t version, alignment;
    uint64_t file_len, tensor_data_offset, tensor_count, metadata_count;
} fq_gguf_info_t;
int fq_gguf_open(const char *path, int require_architecture, uint64_t skip_arrays_over, fq_gguf **out, char *err, size_t err_len);
int fq_gguf_close(fq_gguf *file);
const char *fq_gguf_last_error(const fq_gguf *file);
int fq_gguf_info(const fq_gguf *file, fq_gguf_info_t *out);
int fq_gguf_tensor_by_name(fq_gguf *file, const char *name, fq_gguf_tensor *out);
int fq_gguf_tensor_by_index(fq_gguf *file, uint64_t index, fq_gguf_tensor *out); /* in name order */
/* `read_tensor_into` (src/loader/gguf.rs:474-495): `len` must be the tensor's byte length. */
int fq_gguf_read_tensor(fq_gguf *file, const char *name, void *dst, size_t len);
int fq_gguf_metadata_u64(fq_gguf *file, const char *key, uint64_t *out);
int fq_gguf_metadata_f64(fq_gguf *file, const char *key, double *out);
int fq_gguf_metadata_string(fq_gguf *file, const char *key, char *out, size_t len);
int fq_gguf_metadata_array(fq_gguf *file, const char *key, uint32_t *element_type, uint64_t *count, uint64_t *kept);
/* `block_layout` (src/loader/gguf.rs:87-121): elements and bytes of one block of a GGML type. */
int fq_block_layout(uint32_t type_id, uint32_t *elements, uint32_t *bytes);
/* `gguf_matrix` (src/hybrid/weights.rs:671-736): tensor `name` as `experts` stacked [rows, cols] slices
 * (GGUF dims [cols, rows] or [cols, rows, experts], else FQ_ERR_WEIGHT), in its stored encoding, or -- with
 * `q3k_as_q6k` -- Q3_K rewritten as Q6_K; then the checks and the upload of `fq_matrix_create`. */
int fq_matrix_from_gguf(fq_device *dev, fq_gguf *file, const char *name, uint64_t experts, uint64_t rows, uint64_t cols,
                        int q3k_as_q6k, fq_matrix **out);
/* `q3k_to_q6k` (src/hybrid/weights.rs:761-805): `blocks` Q3_K blocks (110 bytes) as Q6_K blocks (210 bytes)
 * that decode to exactly the same values.  Host memory. */
int fq_q3k_to_q6k(const void *src, size_t blocks, void *dst);
/* ggml's reference Q8_0 row quantisation as the loader applies it to unquantised tensors
 * (`quantize_row`, src/hybrid/weights.rs:1397-1415): n floats (a multiple of 32) to n / 32 blocks.  Host memory. */
int fq_quantize_q8_0(const float *x, size_t n, void *out);

/* ---- the op surface ------------------------------------------------------------------------ */

/* `HybridModel::project(d, w, x, m, y)` (src/hybrid/engine.rs:3407-3500):
 * y[m][rows] = x[m][cols] . W^T.  x_elems must be m*cols and y_elems m*rows (else FQ_ERR_SHAPE).
 * F32 in / F32 out is the hybrid engine's contract; BF16 in / BF16 out (fp32 accumulate, RNE
 * store) is the legacy `project_quantized` tensor path (src/ops/transformer.rs:96-297). */
int fq_project(fq_device *dev, const fq_matrix *w, const void *x, int x_dtype, size_t x_elems,
               size_t m, void *y, int y_dtype, size_t y_elems);

/* `count` projections that share x and m, as the reference issues back to back for q|k|v
 * (src/hybrid/engine.rs:2265-2267) and gate|up (:3239-3240).  y[i] receives m * rows_i values.
 * Matrices of one format and width run as ONE launch over all their rows; otherwise this is
 * `fq_project` in a loop.  Same checks and errors as `fq_project`. */
int fq_project_many(fq_device *dev, const fq_matrix *const *w, size_t count, const void *x, int x_dtype,
                    size_t x_elems, size_t m, void *const *y, int y_dtype);

/* ---- either side of a projection ------------------------------------------------------------ */

/* `HybridModel::rmsnorm` = `h_rmsnorm` (src/hybrid/engine.rs:3301-3320; hybrid.metal:1563-1575):
 * y[r][i] = x[r][i] * rsqrt(mean_i x[r][i]^2 + eps) * w[i] for `rows` rows of n values (n a multiple of 4). */
int fq_rmsnorm(fq_device *dev, const float *x, const float *w, uint32_t n, float eps, uint32_t rows, float *y);
/* `HybridModel::add_rmsnorm` = `h_add_rmsnorm` (src/hybrid/engine.rs:3322-3345; hybrid.metal:1577-1595):
 * h = x + r (written to h), y = rmsnorm(h) * w. */
int fq_add_rmsnorm(fq_device *dev, const float *x, const float *r, const float *w, uint32_t n, float eps, uint32_t rows,
                   float *h, float *y);
/* `fq_project_many` on rmsnorm(x) * norm_w: the normalisation that produces a projection's input, folded into
 * the projection.  At 1..16 activation rows on Q4_K / Q5_K / Q6_K matrices of one format it is computed inside
 * the activation preparation (no launch of its own, no round trip of the normalised row, and bit for bit what
 * `fq_rmsnorm` followed by `fq_project_many` gives); otherwise `scratch` (m * cols floats, may be NULL when the
 * fused case is certain) receives the normalised rows first.  F32 in and out. */
int fq_rmsnorm_project_many(fq_device *dev, const fq_matrix *const *w, size_t count, const float *x, const float *norm_w,
                            float eps, size_t x_elems, size_t m, float *scratch, void *const *y);
/* `h_argmax` (hybrid.metal:2214-2243): out[r] = index of the first maximum of row r of n values (the consumer of
 * the output head's logits under greedy sampling). */
int fq_argmax(fq_device *dev, const float *x, uint32_t n, uint32_t rows, uint32_t *out);
/* `h_topk_blocks` (hybrid.metal:3616-3657): per block of 1024 values of each row, the 32 largest (value, index)
 * pairs in descending order, ties to the lower index; out[(r * ceil(n / 1024) + block) * 32 + k] = {value, index
 * as the bits of a float}. */
int fq_topk_blocks(fq_device *dev, const float *x, uint32_t n, uint32_t rows, float *out);

/* `HybridModel::project_id(d, w, x, ids, routes, x_div, y)` (src/hybrid/engine.rs:3114-3147):
 * route r multiplies activation row r / x_div by the rows of expert ids[r]; F32 in and out. */
int fq_project_id(fq_device *dev, const fq_matrix *w, const float *x, size_t x_elems,
                  const uint32_t *ids, size_t routes, size_t x_div, float *y, size_t y_elems);

/* `HybridModel::project_mm_id_in(d, w, x, offsets, slots, max_rows, y)`
 * (src/hybrid/engine.rs:3164-3224): rows offsets[z]..offsets[z+1] of x and y belong to group z,
 * which uses the expert stored at slots[z] (slots == NULL: expert z).  `groups` is the number of
 * groups (w.experts without a slot table); `max_rows` bounds any group's row count.  `offsets` and `slots`
 * are read one 32-bit value at a time: 4-byte alignment is enough for them (a rank's window into a larger
 * table of expert offsets starts wherever its first expert falls).  F32 callers get fp32-level results at every
 * width (the integer kernel below about 16 rows per group on average; from there on fp16 tensor-core products of
 * weights rounded to fp16 and activations carried to 22 bits: within 1e-3 of the largest output, 4e-4 measured);
 * BF16 callers the bf16 contract of the prefill GEMM. */
int fq_project_mm_id(fq_device *dev, const fq_matrix *w, const void *x, int x_dtype, size_t x_elems,
                     const uint32_t *offsets, const uint32_t *slots, size_t groups, size_t max_rows,
                     void *y, int y_dtype, size_t y_elems);

/* `HybridModel::get_rows(d, w, ids, y)` (src/hybrid/engine.rs:3274-3300): y[t][:] = the exact
 * fp32 decode of row ids[t] (BF16 output = that value rounded, the legacy
 * `embedding_gather_quantized`, src/ops/transformer.rs:299). */
int fq_get_rows(fq_device *dev, const fq_matrix *w, const uint32_t *ids, size_t tokens, void *y,
                int y_dtype, size_t y_elems);

/* `h_moe_route` via `moe_ffn` (src/hybrid/engine.rs:2907-2924; hybrid.metal:2252-2319). */
int fq_moe_route(fq_device *dev, const float *logits, const float *x, const float *shared_w,
                 uint32_t experts, uint32_t used, uint32_t hidden, uint32_t tokens, int sigmoid,
                 int norm, int shared_gate, uint32_t *ids, float *weights, float *gate);
/* `h_moe_map` (src/hybrid/engine.rs:3043-3051; hybrid.metal:2321-2358). */
int fq_moe_map(fq_device *dev, const uint32_t *ids, uint32_t experts, uint32_t routes,
               uint32_t *offsets, uint32_t *sorted, uint32_t *position);
/* `h_moe_gather` (src/hybrid/engine.rs:3052-3060; hybrid.metal:2360-2369). */
int fq_moe_gather(fq_device *dev, const float *x, const uint32_t *sorted, uint32_t hidden,
                  uint32_t used, uint32_t routes, float *xg);
/* `h_moe_combine` (src/hybrid/engine.rs:3068-3091; hybrid.metal:2371-2388). */
int fq_moe_combine(fq_device *dev, const float *down, const float *weights, const uint32_t *position,
                   const float *shared, const float *gate, uint32_t hidden, uint32_t used,
                   uint32_t tokens, int identity, float *out);
/* `HybridModel::glu` with SiLU = `h_swiglu` (src/hybrid/engine.rs:3094-3110; hybrid.metal:1606). */
int fq_glu(fq_device *dev, const float *gate, const float *up, size_t n, float *out);

/* `HybridModel::dense_ffn` (src/hybrid/engine.rs:3226-3243): out = down(silu(gate x) * up x).
 * `scratch` holds 3 * m * gate.rows floats (the reference's ffn_gate / ffn_up / ffn_act). */
int fq_dense_ffn(fq_device *dev, const fq_matrix *gate, const fq_matrix *up, const fq_matrix *down,
                 const float *x, size_t m, float *scratch, size_t scratch_elems, float *out);

/* Geometry and weights of one MoE FFN (`MoeFfn`, src/hybrid/engine.rs:2881-2906). */
typedef struct fq_moe_ffn_desc {
    const fq_matrix *router;      /* [experts, hidden] */
    const fq_matrix *gate_exps;   /* experts x [expert_ffn, hidden] */
    const fq_matrix *up_exps;     /* experts x [expert_ffn, hidden] */
    const fq_matrix *down_exps;   /* experts x [hidden, expert_ffn] */
    const fq_matrix *shared_gate; /* shared expert, [shared_ffn, hidden] */
    const fq_matrix *shared_up;
    const fq_matrix *shared_down; /* [hidden, shared_ffn] */
    const float *shared_gate_inp; /* [hidden] or NULL */
    uint32_t experts, used, hidden, expert_ffn, shared_ffn;
    int32_t sigmoid, norm_weights;
} fq_moe_ffn_desc;

/* Floats of scratch `fq_moe_ffn` needs for m tokens. */
size_t fq_moe_ffn_scratch_elems(const fq_moe_ffn_desc *f, size_t m);
/* `HybridModel::moe_ffn` (src/hybrid/engine.rs:2881-3092): router projection, routing, shared
 * expert, per-route expert GEMVs when m*used <= 32 (`MV_ID_MAX_ROUTES`) or the handle is exact,
 * else map + gather + grouped expert GEMMs, then combine. */
int fq_moe_ffn(fq_device *dev, const fq_moe_ffn_desc *f, const float *x, size_t m, float *scratch,
               size_t scratch_elems, float *out);

/* ---- host-buffer entry points (what a caller without device pointers uses) ----------------- */

/* `project` for HOST x / y: copies x to the device, runs `fq_project` (F32), copies y back and
 * waits.  The staging buffers are the handle's fixed scratch (m * (cols + rows) floats must fit
 * `FQ_HOST_STAGING_BYTES`). */
#define FQ_HOST_STAGING_BYTES (64u << 20)
int fq_project_host(fq_device *dev, const fq_matrix *w, const float *x_host, size_t m, float *y_host);
/* The same for several matrices that share x (q|k|v, gate|up): one upload, `count` projections,
 * one wait.  y_host[i] receives m * rows_i floats. */
int fq_project_many_host(fq_device *dev, const fq_matrix *const *w, size_t count, const float *x_host,
                         size_t m, float *const *y_host);

/* ---- tensor-parallel exchange (no counterpart in the single-GPU reference) -------------------- */

/* Row-sharded projections: rank r holds rows [r N / g, (r + 1) N / g) of every matrix and computes its
 * slice of the output; the slices are gathered over NVLink peer memory.  One process per GPU.
 *   fq_comm_create   allocates this rank's symmetric buffer (`bytes` of payload, a multiple of 256), its flag
 *                    words and a mirror area of 2 x `bytes` for the fused exchange of `fq_project_many_gather`;
 *   fq_comm_handle   writes the 64-byte CUDA IPC handle of that buffer, to be exchanged out of band
 *                    (e.g. one torch.distributed all_gather of 64 bytes);
 *   fq_comm_open     maps every peer's buffer from the `world` x 64 handle bytes, ordered by rank;
 *   fq_comm_buffer   the local buffer: projections write their outputs into it;
 *   fq_comm_all_gather  for the region [offset, offset + world * shard_bytes): this rank's slice
 *                    [offset + rank * shard_bytes, + shard_bytes) must have been written by work enqueued
 *                    before the call; after it (in stream order) the region holds every rank's slice.  All
 *                    ranks must enqueue the same sequence of gathers.  A peer that never arrives makes the
 *                    kernel give up after a bounded wait; `fq_synchronize` then returns FQ_ERR_TIMEOUT. */
typedef struct fq_comm fq_comm;
int fq_comm_create(fq_device *dev, int rank, int world, size_t bytes, fq_comm **out);
int fq_comm_handle(fq_comm *comm, void *out64);
int fq_comm_open(fq_comm *comm, const void *handles);
void *fq_comm_buffer(fq_comm *comm);
int fq_comm_all_gather(fq_device *dev, fq_comm *comm, size_t region_offset, size_t shard_bytes);
/* The same exchange for runs of rows of unequal length: the region is `total_rows` rows of `row_bytes`
 * bytes (a multiple of 16) from `region_offset`; rank r owns rows bounds[r * stride] .. bounds[(r + 1) * stride].
 * `bounds` is DEVICE memory (world * stride + 1 words) that work enqueued earlier may still be writing --
 * e.g. the expert offsets of `fq_moe_map`, with stride = experts per rank. */
int fq_comm_all_gather_rows(fq_device *dev, fq_comm *comm, size_t region_offset, size_t row_bytes, const uint32_t *bounds,
                            uint32_t stride, size_t total_rows);
int fq_comm_destroy(fq_comm *comm);
/* Wall-time limit (nanoseconds, default 2 s) of every device-side wait of this communicator's exchanges: a
 * kernel that has waited this long for a peer records FQ_ERR_TIMEOUT and returns; `fq_synchronize` reports it
 * and `fq_device_recover` makes the handle usable again.  The counterpart of the reference's failed command
 * epoch (src/metal/mod.rs:598-625) for a peer that never arrives. */
int fq_comm_set_wait_ns(fq_comm *comm, uint64_t ns);
/* Test-only, in place of `fq_comm_open` on a communicator of two ranks: the "peer" is a second buffer on
 * this GPU that nothing ever writes, so every wait for the peer runs out -- the give-up path can be tested on
 * one GPU without a second process and without a fault (the reference's failure tests,
 * src/metal/mod.rs:1196-1303, inject on the host as well). */
int fq_comm_open_local(fq_comm *comm);
/* Exchange regions: consecutive exchanges of one communicator (`fq_comm_all_gather`, `fq_comm_all_gather_rows`,
 * `fq_project_many_gather`, `fq_moe_ffn_ep`, and the first exchange of a replayed graph against what ran before
 * it) must use regions that do not overlap.  A rank that runs ahead writes its peers' copy of the region it is
 * exchanging; if that region were the one of the exchange before, a slower peer might still be reading it.
 * With another exchange in between the writer cannot be that far ahead.  A reuse is refused with FQ_ERR_PARAM. */
/* `fq_project_many` on row shards with the exchange included: every y[i] (F32) must lie in this rank's
 * slice [region_offset + rank * shard_bytes, + shard_bytes) of a gathered region of the symmetric buffer,
 * y[0] at the start of the slice and every y[i + 1] directly after y[i] (FQ_ERR_RANGE otherwise; what is left
 * of the slice after the last output is padding that is neither sent nor waited for);
 * when the call's work has run, the region holds every rank's slice, as after `fq_comm_all_gather`.  At
 * decode and verify widths (m <= 16, Q4_K / Q6_K) there is ONE launch for compute and exchange and no fence: the
 * projection kernel stores every output value, paired with the exchange's sequence number in one 8-byte
 * store, into a mirror area of every peer's buffer, and before it ends its blocks collect the values the
 * peers sent (polling each slot, bounded, for the current sequence number).  Other shapes project, then
 * gather the region with the copy kernel.  The buffer `fq_comm_create` allocates is three times `bytes`
 * plus the flag words (payload, flags, mirror). */
int fq_project_many_gather(fq_device *dev, fq_comm *comm, size_t region_offset, size_t shard_bytes, const fq_matrix *const *w,
                           size_t count, const void *x, int x_dtype, size_t x_elems, size_t m, void *const *y, int y_dtype);

/* ---- expert-parallel MoE block (no counterpart in the single-GPU reference) -------------------- */

/* `fq_moe_ffn` with the experts sharded over the ranks of `comm`: rank r stores experts
 * [r E / g, (r + 1) E / g) -- the expert matrices of `f` hold only those (`f->experts` stays E), and
 * `expert_first` = r E / g.  x, the router and the shared expert are replicated.  Every rank routes all
 * tokens and computes the expert-sorted rows of its own experts into the symmetric buffer at `region_offset`.
 * With more than 32 routes the exchange is an all-to-all: a row goes only to the rank that owns its token
 * (tokens are split evenly, ceil(m / g) rounded up to a multiple of 4 to a rank), the owner combines its tokens,
 * and the combined outputs are gathered; the buffer must hold, from `region_offset`, m * used * hidden floats
 * (rounded up to 256 bytes) and then g * tokens-per-rank * hidden floats.  With 32 routes or fewer every row is
 * gathered on every rank (`fq_comm_all_gather_rows`) and every rank combines.  Either way `out` is complete on
 * every rank and equals `fq_moe_ffn` on one GPU bit for bit.  All ranks must make the same calls in the same
 * order.  Scratch as for `fq_moe_ffn`. */
int fq_moe_ffn_ep(fq_device *dev, fq_comm *comm, size_t region_offset, const fq_moe_ffn_desc *f, uint32_t expert_first,
                  const float *x, size_t m, float *scratch, size_t scratch_elems, float *out);

/* ---- allocation-free decode projection ------------------------------------------------------- */

/* No counterpart in the reference (its backend allocates its buffers at load and has no notion of a
 * caller that may not).  For callers that cannot allocate device memory at all -- code running after a
 * memory pool has taken every byte, a plugin inside a process whose allocator belongs to someone else,
 * a latency-critical section where cudaMalloc would serialise the device -- and so cannot use
 * `fq_device_create` / `fq_matrix_create`, which both allocate.
 *
 *   y[m][rows] = x[m][cols] . W^T,  W = `rows` rows of cols / 256 Q4_K blocks (GGUF bytes), 1 <= m <= 4.
 *
 * All pointers are DEVICE pointers, 16-byte aligned, on the current device; the work is enqueued on
 * `cuda_stream` and is complete when that stream reaches it.  The arithmetic is that of `fq_project` on a
 * Q4_K matrix (integer dot products against activations rounded to 16 bits); the summation order over K
 * differs, so results agree with it to that accuracy (about 1e-5 of the largest output), not bit for bit.
 * x, y and the weights may not overlap (FQ_ERR_ALIAS).  The status covers this call's own launch only: an
 * error left pending on the calling thread by earlier CUDA calls is cleared, not reported.  The prepared
 * activations live in a fixed array inside the library
 * image (FQ_STATIC_SCRATCH_BYTES per GPU that loads the library, held until the process exits);
 * m * (about 2.4 * cols) bytes must fit, otherwise the call returns FQ_ERR_SHAPE and says so in `err`.
 * The call itself uses no cudaMalloc, cudaFree or other allocating routine.  The first call on each
 * device also looks up the array's device address (first calls from several threads are safe): make that
 * call before any stream capture.  Every
 * call on a device shares the one array (each call rewrites all of it that it reads, so nothing is
 * carried over), hence two calls whose kernels may overlap on the GPU -- different streams, no
 * ordering -- race; calls on one stream, or ordered by events, are safe.  `err` (may be NULL) receives
 * a message when the status is not FQ_OK. */
#define FQ_STATIC_SCRATCH_BYTES (256u << 10)
int fq_gemv_q4k_static(const void *w_packed, uint64_t rows, uint64_t cols, const float *x, uint32_t m, float *y,
                       void *cuda_stream, char *err, size_t err_len);

#ifdef __cplusplus
}
#endif
#endif /* FERRUM_B200_H */
