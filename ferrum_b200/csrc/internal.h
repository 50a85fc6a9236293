// Shared declarations of the library's translation units (host side).
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>

#include <cstdint>
#include <cstdio>
#include <map>
#include <string>
#include <utility>
#include <vector>

#include "../../include/ferrum_b200.h"

// Largest activation-row count the decode/verify GEMV handles with weights streamed once.
constexpr int FQ_GEMV_MAX_M = 16;
// Widest projection input the activation-preparation scratch is sized for.
constexpr size_t FQ_MAX_COLS = 65536;

struct fq_device {
    int ordinal = 0;
    int sm_count = 0;
    cudaStream_t own_stream = nullptr;
    cudaStream_t stream = nullptr;
    // A second stream with its own small activation scratch, for a branch of work that is independent of what
    // runs on `stream` (the shared expert beside the routed experts at decode widths); joined back by events.
    cudaStream_t side_stream = nullptr;
    cudaEvent_t fork_event = nullptr, join_event = nullptr;
    void *side_xprep = nullptr;
    size_t side_xprep_bytes = 0;
    std::string error;
    bool failed = false;          // an asynchronous failure was reported; enqueues are refused
    bool exact = false;
    int fail_after = -1;          // test hook: enqueues left before an injected failure
    bool fail_completion = false; // test hook: next synchronize reports failure
    fq_counters counters{};
    // Output ranges enqueued since the last completion point, and the ranges a failed submission wrote: an input
    // that overlaps one of the latter is refused until a later submission that rewrites it has completed
    // (`Completion::Failed`, src/metal/mod.rs:865-873).
    std::vector<std::pair<uintptr_t, uintptr_t>> pending_writes, failed_writes;
    // Opt-in per-operation measurements (`fq_set_profiling` / `fq_take_profile`): a pair of events around every
    // enqueue outside graph capture, resolved into the table when it is taken.
    struct ProfileSample { const char *name; cudaEvent_t start, stop; };
    struct ProfileTotals { uint64_t calls = 0, kernels = 0, wall_ns = 0, gpu_ns = 0, gpu_samples = 0; };
    bool profiling = false, profile_open = false, profile_auto = false;
    cudaEvent_t profile_start = nullptr;
    uint64_t profile_t0 = 0;
    std::vector<ProfileSample> profile_samples;
    std::vector<cudaEvent_t> profile_free; // events ready for reuse
    std::map<std::string, ProfileTotals> profile;
    bool capturing = false;       // between fq_capture_begin and fq_capture_end
    const struct TpPush *tp_push = nullptr; // set while a projection that exchanges its own output is enqueued
    bool tp_pushed = false;                 // the kernel that was launched took tp_push
    uint64_t captured_kernels = 0;
    // Exchanges recorded by the open capture: their communicator, and the first and the last region.
    struct fq_comm *cap_comm = nullptr;
    size_t cap_first_off = 0, cap_first_bytes = 0, cap_last_off = 0, cap_last_bytes = 0;
    std::map<uintptr_t, size_t> allocations; // buffers handed out by fq_buffer_alloc
    // Fixed scratch, allocated once at creation.
    void *xprep = nullptr;        // prepared activations of the tensor-core GEMV
    size_t xprep_bytes = 0;
    uint32_t xprep_turn = 0;      // successive projections alternate between the two halves of xprep
    void *staging_dev = nullptr;  // device side of the host-buffer entry points
    void *staging_host = nullptr; // pinned host side
    // K-slice workspace of the verify-width GEMV (partial sums and one arrival counter per 16-row tile); the side
    // stream has its own.
    void *nt_ws = nullptr, *side_nt_ws = nullptr;
    size_t nt_ws_bytes = 0, side_nt_ws_bytes = 0;
    uint32_t *nt_counters = nullptr, *side_nt_counters = nullptr;
    uint32_t *combine_counters = nullptr; // FQ_COMBINE_COUNTERS words, zero between launches
    uint32_t nt_counter_count = 0, side_nt_counter_count = 0;
    // Split-K workspace of the prefill GEMM: partial fp32 tiles and one arrival counter per tile.
    float *gemm_ws = nullptr;
    size_t gemm_ws_bytes = 0;
    // One word in mapped pinned host memory that kernels set when a bounded wait gives up.
    volatile int *status_host = nullptr;
    int *status_dev = nullptr;
};

struct fq_graph {
    fq_device *dev = nullptr;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    uint64_t kernels = 0;
    struct fq_comm *comm = nullptr; // set when the graph holds exchanges
    size_t first_off = 0, first_bytes = 0, last_off = 0, last_bytes = 0;
};

struct fq_matrix {
    fq_device *dev = nullptr;
    int format = 0;
    uint64_t rows = 0, cols = 0, experts = 1, row_bytes = 0, byte_size = 0;
    uint64_t pitch = 0; // bytes between rows of the device layout (see fq_row_pitch)
    uint32_t block_elems = 0, block_bytes = 0;
    uint8_t *data = nullptr; // device copy of the blocks in the device layout
    uint64_t expert_rows() const { return rows / experts; }
};

int fq_fail(fq_device *dev, int status, const char *fmt, ...);
int fq_check_cuda(fq_device *dev, cudaError_t e, const char *what);
// Common prologue of every enqueue: refuses a failed handle, runs the injected-failure hook,
// makes the device current.
int fq_begin_enqueue(fq_device *dev);
int fq_end_enqueue(fq_device *dev, const char *what, int kernels);
// Binding checks shared by the op surface (null, alignment, ownership range, overlap).
void fq_note_write(fq_device *dev, const void *out, size_t bytes); // an enqueue writes [out, out + bytes)
int fq_check_binding(fq_device *dev, const void *p, size_t bytes, const char *name, uint32_t align = 16);
int fq_check_no_alias(fq_device *dev, const void *out, size_t out_bytes, const void *in,
                      size_t in_bytes, const char *name);

inline size_t fq_dtype_size(int dtype) { return dtype == FQ_BF16 ? 2 : 4; }

// Kernel launchers (one per translation unit); all enqueue on dev->stream and return a status.
// `h_moe_combine` (src/metal/shaders/hybrid.metal:2371-2388) carried out by the down projection of per-route
// experts: the last of a token's `used` route blocks to finish a 16-row tile adds the routes' rows in route order.
constexpr uint32_t FQ_COMBINE_COUNTERS = 8192;
struct CombineTail {
    const float *weights, *shared, *gate; // [tokens][used], [tokens][hidden], [tokens]
    float *out;                           // [tokens][hidden]
    uint32_t *counters;                   // [tokens][tiles]: arrivals, back at zero when the kernel ends; null = no tail
    uint32_t used;
};

struct ProjectArgs {
    const uint8_t *w;
    uint32_t format, rows, cols, row_bytes; // rows = rows of one expert slice; row_bytes = device row pitch
    const void *x;
    const float *x_up = nullptr; // decode kernels only: the activations are silu(x) * x_up (the gated unit, fused into their preparation)
    // Per-route expert projections over a permutation of the routes (an expert-parallel rank's expert-sorted rows):
    // output row r takes the expert ids[route_map[r]] - id_base (a value outside the matrix's experts: the row is
    // another rank's and is skipped) and, with map_x, the activation row route_map[r] / x_div (else r / x_div).
    const uint32_t *route_map = nullptr;
    uint32_t id_base = 0;
    bool map_x = false;
    const float *norm_w = nullptr; // decode kernels only: the activations are rmsnorm(x) * norm_w (fused into their preparation)
    float norm_eps = 0.f;
    void *y;
    int x_dtype, y_dtype;
    uint32_t m;        // activation rows (project) / routes (project_id) / 0 (grouped)
    // expert addressing
    const uint32_t *ids = nullptr;     // project_id: expert of each route
    uint32_t x_div = 1;
    const uint32_t *offsets = nullptr; // grouped: row ranges
    const uint32_t *slots = nullptr;
    uint32_t groups = 0, max_rows = 0;
    uint32_t experts = 1;              // expert slices stored in w
    const CombineTail *combine = nullptr; // project_id of one target, one activation row per route (x_div = 1)
};
int fq_launch_project_exact(fq_device *dev, const ProjectArgs &a);
int fq_launch_project_id_exact(fq_device *dev, const ProjectArgs &a);
int fq_launch_project_grouped_exact(fq_device *dev, const ProjectArgs &a);
int fq_launch_get_rows(fq_device *dev, const fq_matrix *w, const uint32_t *ids, uint32_t tokens,
                       void *y, int y_dtype);
// Bytes of the per-handle activation scratch (two halves used alternately).
constexpr size_t FQ_GEMV_SCRATCH_BYTES = (size_t)96 << 20;
// Kernel launchers return FQ_ERR_UNSUPPORTED when the shape has no fast kernel, so that the caller can fall
// back to the exact one.
// Integer tensor-core decode GEMV for one activation row and for per-route expert projections; several
// matrices of one format and width sharing x in one launch.
int fq_launch_gemv_i8_many(fq_device *dev, const ProjectArgs *a, uint32_t count);
// The same for 2..16 activation rows (activation rows on the MMA's N side).
int fq_launch_gemv_nt_many(fq_device *dev, const ProjectArgs *a, uint32_t count);
// Grouped expert projection over expert-sorted rows (a[i].offsets / slots / groups) for one or two expert stacks
// of one shape (F32 in and out); row r of the sorted set is row src[r] / src_div of x (src null: row r).
int fq_launch_gemv_iq4(fq_device *dev, const ProjectArgs &a);
int fq_launch_gemv_nt_grouped(fq_device *dev, const ProjectArgs *a, uint32_t count, uint32_t total_rows, const uint32_t *src, uint32_t src_div);
// tcgen05 dequant-GEMM (BF16 in/out); same fallback contract.
// Q8_0 integer-dot GEMV (M <= FQ_GEMV_MAX_M, F32 in/out, no routes); FQ_ERR_UNSUPPORTED otherwise.
int fq_launch_gemv_q8(fq_device *dev, const ProjectArgs &a);
int fq_launch_gemm_tc(fq_device *dev, const ProjectArgs &a);
// 2..4 matrices of one format and width sharing X (BF16 in/out, wider than the verify widths) in one launch.
int fq_launch_gemm_tc_many(fq_device *dev, const ProjectArgs *a, uint32_t count);
// The same over expert-sorted activation rows (a.offsets / a.slots / a.groups / a.max_rows); F32 or BF16.
int fq_launch_gemm_tc_grouped(fq_device *dev, const ProjectArgs &a, uint32_t total_rows);
// The same rows on fp16 products with fp32-level activations (F32 in and out); arguments as fq_launch_gemv_nt_grouped.
int fq_launch_gemm_f16_grouped(fq_device *dev, const ProjectArgs *a, uint32_t count, uint32_t total_rows, const uint32_t *src, uint32_t src_div);
// Expert-sorted activations and the gated unit with bf16 results (inputs of the grouped tensor-core GEMM).
// `range` (may be null) limits the work to rows [range[0], range[stride]): the experts one rank owns.
int fq_launch_moe_gather_bf16(fq_device *dev, const float *x, const uint32_t *sorted, uint32_t hidden, uint32_t used, uint32_t routes,
                              const uint32_t *range, uint32_t stride, void *xg);
// Routing and, with `offsets`, the expert-major map of the routes (fq_moe_map's outputs); one launch at decode widths.
int fq_moe_route_map(fq_device *dev, const float *logits, const float *x, const float *shared_w, uint32_t experts, uint32_t used,
                     uint32_t hidden, uint32_t tokens, int sigmoid, int norm, int shared_gate, uint32_t *ids, float *weights, float *gate,
                     uint32_t *offsets, uint32_t *sorted, uint32_t *position);
int fq_launch_glu_bf16(fq_device *dev, const float *gate, const float *up, size_t n, const uint32_t *range, uint32_t stride, uint32_t width,
                       void *out);
// out[row] = expert of expert-sorted row `row` minus `first`, or an id that names no expert when it is not one
// of the `count` experts from `first`.
int fq_launch_moe_local_ids(fq_device *dev, const uint32_t *ids, const uint32_t *sorted, uint32_t routes, uint32_t first, uint32_t count,
                            uint32_t *out);
// Fused exchange of a row-sharded projection (comm.cu, gemv_i8.cu), without fences or a separate copy: next to
// its payload every symmetric buffer has a mirror of 8-byte slots {value, sequence number}, one per payload
// float.  The kernel that computes this rank's output rows stores each value into its own payload slice and,
// paired with the exchange's sequence number in ONE 8-byte peer store over NVLink, into the mirror of every
// peer (a value and its tag arrive together, so no ordering between stores is needed).  Before it ends, every
// block takes a share of the slots the peers send to this rank, polls each -- bounded -- until its tag is the
// current sequence number, and moves the value into the payload; when the kernel has ended every rank's rows
// are in local memory.  The sequence number counts the communicator's fused exchanges in device memory (the
// last block to finish advances it; all ranks make the same calls, so it is the same everywhere and never
// repeats for a slot), so a captured graph can replay the exchange.  world <= 1 turns it off.
struct TpPush {
    uint8_t *peer[8];    // symmetric buffers by rank (peer[rank] is the local one)
    uint32_t world, rank, slot, pad;
    uint32_t *epoch;     // local: number of fused exchanges this communicator has completed (the same on every rank)
    uint32_t *counter;   // local: blocks of this launch that have finished
    size_t mirror_off;   // the mirror starts here in every buffer: payload float at byte o <-> slot at mirror_off + 2 o
    size_t slice_off, slice_bytes; // this rank's slice of the gathered region; rank p's is (p - rank) slices away
    size_t covered_bytes;          // leading bytes of every slice that the projection outputs fill (the rest is padding)
    uint64_t wait_ns;              // wall-time limit of a block's wait for incoming values
    int *status;
};
struct fq_comm;
// Fills `out` for the next exchange of `c` (takes a flag slot); FQ_ERR_RANGE unless [y, y + bytes) lies in
// the local symmetric buffer.
int fq_comm_begin_push(fq_comm *c, const void *y, size_t bytes, TpPush *out);
// Bookkeeping of exchange regions (consecutive exchanges must use disjoint regions): before every exchange is
// enqueued, and before a graph that holds exchanges is replayed.  FQ_ERR_PARAM on a reuse.
int fq_comm_note_region(fq_device *dev, fq_comm *c, size_t off, size_t bytes);
int fq_comm_note_graph(fq_device *dev, const struct fq_graph *g);
fq_device *fq_comm_device(const fq_comm *c);
int fq_comm_all_gather_unchecked(fq_device *dev, fq_comm *c, size_t region_offset, size_t shard_bytes);
// The dispatch half of an all-to-all over expert-sorted rows: row p of this rank's run (bounds / stride as in
// fq_comm_all_gather_rows) goes only to the rank that owns token sorted[p] / used, token t belonging to rank
// min(t / tokens_per_rank, world - 1).
int fq_comm_dispatch_rows(fq_device *dev, fq_comm *c, size_t region_offset, size_t row_bytes, const uint32_t *bounds, uint32_t stride,
                          const uint32_t *sorted, uint32_t used, uint32_t tokens_per_rank, size_t total_rows);
// `fq_moe_combine` for tokens [token0, token0 + tokens) of a block (internal buffers: no binding checks).
int fq_launch_moe_combine_range(fq_device *dev, const float *down, const float *weights, const uint32_t *position, const float *shared,
                                const float *gate, uint32_t hidden, uint32_t used, uint32_t token0, uint32_t tokens, float *out);
// The symmetric buffer of a communicator and its geometry (comm.cu).
struct fq_comm;
uint8_t *fq_comm_local(fq_comm *c);
size_t fq_comm_bytes(const fq_comm *c);
int fq_comm_rank(const fq_comm *c);
int fq_comm_world(const fq_comm *c);
