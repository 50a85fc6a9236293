// The C ABI: device handles, buffers, weight matrices, binding checks and the dispatch policy of
// the quantized-linear op surface (the counterpart of src/hybrid/engine.rs:3407-3500 and of the
// checks in src/metal/mod.rs:838-897).
#include <cstdarg>
#include <cstdlib>
#include <algorithm>
#include <ctime>
#include <cstring>
#include <utility>
#include <vector>

#include "blocks.cuh"
#include "internal.h"

// ------------------------------------------------------------------ errors

int fq_fail(fq_device *dev, int status, const char *fmt, ...) {
    if (dev) {
        char buf[512];
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(buf, sizeof buf, fmt, ap);
        va_end(ap);
        dev->error = buf;
    }
    return status;
}

int fq_check_cuda(fq_device *dev, cudaError_t e, const char *what) {
    if (e == cudaSuccess) return FQ_OK;
    return fq_fail(dev, FQ_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

extern "C" const char *fq_status_name(int status) {
    switch (status) {
    case FQ_OK: return "ok";
    case FQ_ERR_SHAPE: return "shape";
    case FQ_ERR_RANGE: return "range";
    case FQ_ERR_DEVICE: return "device mismatch";
    case FQ_ERR_ALIAS: return "alias";
    case FQ_ERR_WEIGHT: return "weight";
    case FQ_ERR_SYNC: return "synchronization";
    case FQ_ERR_TIMEOUT: return "timeout";
    case FQ_ERR_CUDA: return "cuda";
    case FQ_ERR_PARAM: return "parameter";
    case FQ_ERR_UNSUPPORTED: return "unsupported";
    case FQ_ERR_GGUF: return "gguf";
    default: return "unknown";
    }
}

extern "C" const char *fq_last_error(fq_device *dev) { return dev ? dev->error.c_str() : "null device handle"; }

// ------------------------------------------------------------------ enqueue bookkeeping

static uint64_t host_ns() {
    timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (uint64_t)ts.tv_sec * 1000000000ull + (uint64_t)ts.tv_nsec;
}

static cudaEvent_t profile_event(fq_device *dev) {
    if (!dev->profile_free.empty()) {
        cudaEvent_t e = dev->profile_free.back();
        dev->profile_free.pop_back();
        return e;
    }
    cudaEvent_t e = nullptr;
    if (cudaEventCreate(&e) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return e;
}

constexpr size_t PROFILE_MAX_PENDING = 1u << 16; // samples kept between two `fq_take_profile`; later calls are counted without a device time

int fq_begin_enqueue(fq_device *dev) {
    if (!dev) return FQ_ERR_PARAM;
    if (dev->failed) return fq_fail(dev, FQ_ERR_SYNC, "device handle holds a failed submission; call fq_device_recover");
    if (dev->fail_after >= 0) {
        if (dev->fail_after == 0) {
            dev->fail_after = -1;
            dev->failed = true;
            return fq_fail(dev, FQ_ERR_SYNC, "injected enqueue failure");
        }
        dev->fail_after--;
    }
    if (int rc = fq_check_cuda(dev, cudaSetDevice(dev->ordinal), "cudaSetDevice")) return rc;
    if (dev->profiling && (!dev->profile_open || dev->profile_auto)) {
        // The operation's start: one enqueue may pass here several times (checks, then launchers) before it ends.
        // A start that the previous operation's end left behind (for launchers that end several operations after
        // one begin) is replaced, so the host's time between two calls is not charged to the second.
        if (dev->profile_open && dev->profile_start) dev->profile_free.push_back(dev->profile_start);
        dev->profile_open = true;
        dev->profile_auto = false;
        dev->profile_t0 = host_ns();
        dev->profile_start = nullptr;
        if (!dev->capturing && dev->profile_samples.size() < PROFILE_MAX_PENDING && (dev->profile_start = profile_event(dev)))
            if (cudaEventRecord(dev->profile_start, dev->stream) != cudaSuccess) {
                cudaGetLastError();
                dev->profile_free.push_back(dev->profile_start);
                dev->profile_start = nullptr;
            }
    }
    return FQ_OK;
}

int fq_end_enqueue(fq_device *dev, const char *what, int kernels) {
    cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) {
        cudaGetLastError();
        dev->profile_open = false;
        return fq_fail(dev, FQ_ERR_CUDA, "%s: launch failed: %s", what, cudaGetErrorString(e));
    }
    if (dev->capturing) dev->captured_kernels += (uint64_t)kernels;
    else dev->counters.dispatches += (uint64_t)kernels;
    if (dev->profiling && dev->profile_open) {
        dev->profile_open = false;
        fq_device::ProfileTotals &t = dev->profile[what];
        t.calls++;
        t.kernels += (uint64_t)kernels;
        t.wall_ns += host_ns() - dev->profile_t0;
        if (dev->profile_start) {
            cudaEvent_t stop = profile_event(dev);
            if (stop && cudaEventRecord(stop, dev->stream) == cudaSuccess) {
                dev->profile_samples.push_back({what, dev->profile_start, stop});
            } else {
                cudaGetLastError();
                dev->profile_free.push_back(dev->profile_start);
                if (stop) dev->profile_free.push_back(stop);
            }
            dev->profile_start = nullptr;
        }
        // What is enqueued next without a begin of its own starts here.
        dev->profile_open = dev->profile_auto = true;
        dev->profile_t0 = host_ns();
        if (!dev->capturing && dev->profile_samples.size() < PROFILE_MAX_PENDING && (dev->profile_start = profile_event(dev)))
            if (cudaEventRecord(dev->profile_start, dev->stream) != cudaSuccess) {
                cudaGetLastError();
                dev->profile_free.push_back(dev->profile_start);
                dev->profile_start = nullptr;
            }
    }
    return FQ_OK;
}

// `MetalDevice::set_profiling` (src/metal/mod.rs:636-639): switches the per-operation table on or off and clears it.
extern "C" int fq_set_profiling(fq_device *dev, int on) {
    if (!dev) return FQ_ERR_PARAM;
    if (dev->capturing) return fq_fail(dev, FQ_ERR_PARAM, "profiling cannot be switched inside a graph capture");
    for (auto &smp : dev->profile_samples) {
        dev->profile_free.push_back(smp.start);
        dev->profile_free.push_back(smp.stop);
    }
    dev->profile_samples.clear();
    dev->profile.clear();
    if (dev->profile_open && dev->profile_start) dev->profile_free.push_back(dev->profile_start);
    dev->profile_start = nullptr;
    dev->profile_open = dev->profile_auto = false;
    dev->profiling = on != 0;
    return FQ_OK;
}

// `MetalDevice::take_profile` (src/metal/mod.rs:649-651): waits for the stream, resolves the pending event pairs
// into device times, copies the table (in name order, like the reference's BTreeMap) and clears it.
extern "C" int fq_take_profile(fq_device *dev, fq_profile_entry *out, size_t capacity, size_t *count) {
    if (!dev || !count || (capacity && !out)) return FQ_ERR_PARAM;
    if (dev->capturing) return fq_fail(dev, FQ_ERR_PARAM, "the profile cannot be taken inside a graph capture");
    if (int rc = fq_synchronize(dev)) return rc;
    if (dev->side_stream) cudaStreamSynchronize(dev->side_stream);
    for (auto &smp : dev->profile_samples) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, smp.start, smp.stop) == cudaSuccess) {
            fq_device::ProfileTotals &t = dev->profile[smp.name];
            t.gpu_ns += (uint64_t)((double)ms * 1e6);
            t.gpu_samples++;
        } else {
            cudaGetLastError();
        }
        dev->profile_free.push_back(smp.start);
        dev->profile_free.push_back(smp.stop);
    }
    dev->profile_samples.clear();
    *count = dev->profile.size();
    size_t i = 0;
    for (const auto &kv : dev->profile) {
        if (i >= capacity) break;
        fq_profile_entry &e = out[i++];
        memset(&e, 0, sizeof e);
        snprintf(e.name, sizeof e.name, "%s", kv.first.c_str());
        e.calls = kv.second.calls;
        e.kernels = kv.second.kernels;
        e.wall_ns = kv.second.wall_ns;
        e.gpu_ns = kv.second.gpu_ns;
        e.gpu_samples = kv.second.gpu_samples;
    }
    if (capacity >= dev->profile.size()) dev->profile.clear();
    return FQ_OK;
}

// `align`: 16 for everything kernels read or write in 16-byte pieces; 4 for arrays of 32-bit indices, which are
// read one at a time (a rank's slice of the expert offsets starts wherever its first expert falls).
int fq_check_binding(fq_device *dev, const void *p, size_t bytes, const char *name, uint32_t align) {
    if (!p) return fq_fail(dev, FQ_ERR_RANGE, "%s: null binding", name);
    const uintptr_t a = (uintptr_t)p;
    if (a & (uintptr_t)(align - 1)) return fq_fail(dev, FQ_ERR_RANGE, "%s: binding %p is not %u-byte aligned", name, p, align);
    // A pointer inside a buffer this handle allocated must stay inside it.
    auto it = dev->allocations.upper_bound(a);
    if (it != dev->allocations.begin()) {
        --it;
        if (a < it->first + it->second && a + bytes > it->first + it->second)
            return fq_fail(dev, FQ_ERR_RANGE, "%s: %zu bytes at %p run past the end of their allocation", name, bytes, p);
    }
    return FQ_OK;
}

int fq_check_no_alias(fq_device *dev, const void *out, size_t out_bytes, const void *in, size_t in_bytes,
                      const char *name) {
    const uintptr_t o = (uintptr_t)out, i = (uintptr_t)in;
    if (!out || !in) return FQ_OK;
    if (o < i + in_bytes && i < o + out_bytes) return fq_fail(dev, FQ_ERR_ALIAS, "%s: output overlaps an input", name);
    // What a failed submission wrote is not an input until it has been written again.  Only buffers the handle
    // allocated itself are tracked (`fq_buffer_alloc`, the counterpart of the reference's device buffers): memory the
    // caller owns is recycled and rewritten by the caller's allocator without the library seeing it.
    for (const auto &f : dev->failed_writes)
        if (i < f.second && f.first < i + in_bytes) return fq_fail(dev, FQ_ERR_SYNC, "%s: input range belongs to a failed submission", name);
    fq_note_write(dev, out, out_bytes);
    return FQ_OK;
}

void fq_note_write(fq_device *dev, const void *out, size_t bytes) {
    if (dev->capturing || dev->allocations.empty()) return;
    const uintptr_t o = (uintptr_t)out;
    auto it = dev->allocations.upper_bound(o);
    if (it == dev->allocations.begin()) return;
    --it;
    if (o >= it->first + it->second) return; // not inside a buffer of the handle
    if ((dev->pending_writes.empty() || dev->pending_writes.back() != std::make_pair(o, o + bytes)) && dev->pending_writes.size() < 4096)
        dev->pending_writes.emplace_back(o, o + bytes);
}

// A completion point: a failed one poisons what the submission wrote; a good one clears what it rewrote.
static void settle_writes(fq_device *dev, bool ok) {
    if (ok) {
        for (const auto &w : dev->pending_writes)
            dev->failed_writes.erase(std::remove_if(dev->failed_writes.begin(), dev->failed_writes.end(),
                                                    [&](const std::pair<uintptr_t, uintptr_t> &f) { return w.first <= f.first && f.second <= w.second; }),
                                     dev->failed_writes.end());
    } else {
        dev->failed_writes.insert(dev->failed_writes.end(), dev->pending_writes.begin(), dev->pending_writes.end());
        if (dev->failed_writes.size() > 8192) dev->failed_writes.erase(dev->failed_writes.begin(), dev->failed_writes.begin() + 4096);
    }
    dev->pending_writes.clear();
}

// ------------------------------------------------------------------ device

extern "C" int fq_device_create(int ordinal, fq_device **out) {
    if (!out) return FQ_ERR_PARAM;
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || ordinal < 0 || ordinal >= count) return FQ_ERR_DEVICE;
    fq_device *dev = new fq_device();
    dev->ordinal = ordinal;
    auto bail = [&](cudaError_t err, const char *what) {
        fprintf(stderr, "ferrum_b200: %s: %s\n", what, cudaGetErrorString(err));
        fq_device_destroy(dev);
        return FQ_ERR_CUDA;
    };
    if ((e = cudaSetDevice(ordinal)) != cudaSuccess) return bail(e, "cudaSetDevice");
    cudaDeviceProp prop;
    if ((e = cudaGetDeviceProperties(&prop, ordinal)) != cudaSuccess) return bail(e, "cudaGetDeviceProperties");
    if (prop.major != 10) {
        fprintf(stderr, "ferrum_b200: device %d is sm_%d%d; this library is built for sm_100a only\n", ordinal,
                prop.major, prop.minor);
        delete dev;
        return FQ_ERR_DEVICE;
    }
    dev->sm_count = prop.multiProcessorCount;
    if ((e = cudaStreamCreateWithFlags(&dev->own_stream, cudaStreamNonBlocking)) != cudaSuccess) return bail(e, "cudaStreamCreate");
    dev->stream = dev->own_stream;
    if ((e = cudaStreamCreateWithFlags(&dev->side_stream, cudaStreamNonBlocking)) != cudaSuccess) return bail(e, "cudaStreamCreate");
    if ((e = cudaEventCreateWithFlags(&dev->fork_event, cudaEventDisableTiming)) != cudaSuccess) return bail(e, "cudaEventCreate");
    if ((e = cudaEventCreateWithFlags(&dev->join_event, cudaEventDisableTiming)) != cudaSuccess) return bail(e, "cudaEventCreate");
    dev->side_xprep_bytes = (size_t)64 << 20;
    if ((e = cudaMalloc(&dev->side_xprep, dev->side_xprep_bytes)) != cudaSuccess) return bail(e, "activation scratch");
    dev->xprep_bytes = FQ_GEMV_SCRATCH_BYTES;
    if ((e = cudaMalloc(&dev->xprep, dev->xprep_bytes)) != cudaSuccess) return bail(e, "activation scratch");
    dev->nt_ws_bytes = (size_t)48 << 20;
    dev->nt_counter_count = 1u << 18;
    dev->side_nt_ws_bytes = (size_t)4 << 20;
    dev->side_nt_counter_count = 1u << 14;
    if ((e = cudaMalloc(&dev->nt_ws, dev->nt_ws_bytes)) != cudaSuccess) return bail(e, "slice workspace");
    if ((e = cudaMalloc(&dev->side_nt_ws, dev->side_nt_ws_bytes)) != cudaSuccess) return bail(e, "slice workspace");
    if ((e = cudaMalloc((void **)&dev->nt_counters, (size_t)dev->nt_counter_count * 4)) != cudaSuccess) return bail(e, "slice counters");
    if ((e = cudaMalloc((void **)&dev->side_nt_counters, (size_t)dev->side_nt_counter_count * 4)) != cudaSuccess) return bail(e, "slice counters");
    if ((e = cudaMemset(dev->nt_counters, 0, (size_t)dev->nt_counter_count * 4)) != cudaSuccess) return bail(e, "slice counters");
    if ((e = cudaMemset(dev->side_nt_counters, 0, (size_t)dev->side_nt_counter_count * 4)) != cudaSuccess) return bail(e, "slice counters");
    if ((e = cudaMalloc((void **)&dev->combine_counters, (size_t)FQ_COMBINE_COUNTERS * 4)) != cudaSuccess) return bail(e, "combine counters");
    if ((e = cudaMemset(dev->combine_counters, 0, (size_t)FQ_COMBINE_COUNTERS * 4)) != cudaSuccess) return bail(e, "combine counters");
    if ((e = cudaMalloc(&dev->staging_dev, FQ_HOST_STAGING_BYTES)) != cudaSuccess) return bail(e, "device staging");
    if ((e = cudaMallocHost(&dev->staging_host, FQ_HOST_STAGING_BYTES)) != cudaSuccess) return bail(e, "pinned staging");
    dev->gemm_ws_bytes = (size_t)96 << 20;
    if ((e = cudaMalloc((void **)&dev->gemm_ws, dev->gemm_ws_bytes)) != cudaSuccess) return bail(e, "gemm workspace");
    void *status = nullptr;
    if ((e = cudaHostAlloc(&status, 64, cudaHostAllocMapped)) != cudaSuccess) return bail(e, "status word");
    dev->status_host = (volatile int *)status;
    *dev->status_host = 0;
    if ((e = cudaHostGetDevicePointer((void **)&dev->status_dev, status, 0)) != cudaSuccess) return bail(e, "status word mapping");
    *out = dev;
    return FQ_OK;
}

extern "C" int fq_device_destroy(fq_device *dev) {
    if (!dev) return FQ_ERR_PARAM;
    cudaSetDevice(dev->ordinal);
    if (dev->own_stream) cudaStreamSynchronize(dev->own_stream);
    for (auto &kv : dev->allocations) cudaFree((void *)kv.first);
    if (dev->xprep) cudaFree(dev->xprep);
    if (dev->side_xprep) cudaFree(dev->side_xprep);
    if (dev->nt_ws) cudaFree(dev->nt_ws);
    if (dev->side_nt_ws) cudaFree(dev->side_nt_ws);
    if (dev->nt_counters) cudaFree(dev->nt_counters);
    if (dev->side_nt_counters) cudaFree(dev->side_nt_counters);
    if (dev->combine_counters) cudaFree(dev->combine_counters);
    if (dev->side_stream) {
        cudaStreamSynchronize(dev->side_stream);
        cudaStreamDestroy(dev->side_stream);
    }
    for (auto &smp : dev->profile_samples) {
        cudaEventDestroy(smp.start);
        cudaEventDestroy(smp.stop);
    }
    if (dev->profile_start) cudaEventDestroy(dev->profile_start);
    for (cudaEvent_t e : dev->profile_free) cudaEventDestroy(e);
    if (dev->fork_event) cudaEventDestroy(dev->fork_event);
    if (dev->join_event) cudaEventDestroy(dev->join_event);
    if (dev->staging_dev) cudaFree(dev->staging_dev);
    if (dev->gemm_ws) cudaFree(dev->gemm_ws);
    if (dev->staging_host) cudaFreeHost(dev->staging_host);
    if (dev->status_host) cudaFreeHost((void *)dev->status_host);
    if (dev->own_stream) cudaStreamDestroy(dev->own_stream);
    delete dev;
    return FQ_OK;
}

extern "C" int fq_device_set_stream(fq_device *dev, void *cuda_stream) {
    if (!dev) return FQ_ERR_PARAM;
    dev->stream = cuda_stream ? (cudaStream_t)cuda_stream : dev->own_stream;
    return FQ_OK;
}

extern "C" void *fq_device_stream(fq_device *dev) { return dev ? (void *)dev->stream : nullptr; }

extern "C" int fq_synchronize(fq_device *dev) {
    if (!dev) return FQ_ERR_PARAM;
    if (dev->capturing) return fq_fail(dev, FQ_ERR_PARAM, "fq_synchronize inside a capture");
    cudaSetDevice(dev->ordinal);
    dev->counters.synchronizes++;
    cudaError_t e = cudaStreamSynchronize(dev->stream);
    if (dev->fail_completion) {
        dev->fail_completion = false;
        dev->failed = true;
        settle_writes(dev, false);
        return fq_fail(dev, FQ_ERR_SYNC, "injected completion failure");
    }
    if (e != cudaSuccess) {
        dev->failed = true;
        settle_writes(dev, false);
        return fq_fail(dev, FQ_ERR_SYNC, "stream failed: %s", cudaGetErrorString(e));
    }
    if (dev->status_host && *dev->status_host != 0) {
        const int st = *dev->status_host;
        *dev->status_host = 0;
        dev->failed = true;
        settle_writes(dev, false);
        if (st == FQ_ERR_WEIGHT) return fq_fail(dev, FQ_ERR_WEIGHT, "router produced invalid logits");
        return fq_fail(dev, st == FQ_ERR_TIMEOUT ? FQ_ERR_TIMEOUT : FQ_ERR_SYNC, "a kernel gave up a bounded wait (status %d)", st);
    }
    if (dev->failed) return fq_fail(dev, FQ_ERR_SYNC, "device handle holds a failed submission");
    settle_writes(dev, true);
    return FQ_OK;
}

extern "C" int fq_device_recover(fq_device *dev) {
    if (!dev) return FQ_ERR_PARAM;
    cudaSetDevice(dev->ordinal);
    cudaError_t e = cudaStreamSynchronize(dev->stream);
    if (e != cudaSuccess) return fq_fail(dev, FQ_ERR_SYNC, "stream is still failing: %s", cudaGetErrorString(e));
    // A kernel that gave up a wait may have left arrival counters behind.
    if (cudaMemset(dev->combine_counters, 0, (size_t)FQ_COMBINE_COUNTERS * 4) != cudaSuccess) cudaGetLastError();
    dev->failed = false;
    dev->error.clear();
    return FQ_OK;
}

extern "C" int fq_get_counters(fq_device *dev, fq_counters *out) {
    if (!dev || !out) return FQ_ERR_PARAM;
    *out = dev->counters;
    return FQ_OK;
}

extern "C" int fq_set_exact(fq_device *dev, int on) {
    if (!dev) return FQ_ERR_PARAM;
    dev->exact = on != 0;
    return FQ_OK;
}

extern "C" int fq_test_fail_after(fq_device *dev, int n) {
    if (!dev) return FQ_ERR_PARAM;
    dev->fail_after = n;
    return FQ_OK;
}

extern "C" int fq_test_fail_completion(fq_device *dev) {
    if (!dev) return FQ_ERR_PARAM;
    dev->fail_completion = true;
    return FQ_OK;
}

// ------------------------------------------------------------------ batched submission

extern "C" int fq_capture_begin(fq_device *dev) {
    if (int rc = fq_begin_enqueue(dev)) return rc;
    if (dev->capturing) return fq_fail(dev, FQ_ERR_PARAM, "a capture is already open");
    if (dev->stream != dev->own_stream) return fq_fail(dev, FQ_ERR_PARAM, "capture runs on the handle's own stream; restore it first");
    if (int rc = fq_check_cuda(dev, cudaStreamBeginCapture(dev->stream, cudaStreamCaptureModeThreadLocal), "begin capture")) return rc;
    dev->capturing = true;
    dev->captured_kernels = 0;
    dev->cap_comm = nullptr;
    return FQ_OK;
}

extern "C" int fq_capture_end(fq_device *dev, fq_graph **out) {
    if (!dev || !out) return FQ_ERR_PARAM;
    *out = nullptr;
    if (!dev->capturing) return fq_fail(dev, FQ_ERR_PARAM, "no capture is open");
    dev->capturing = false;
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamEndCapture(dev->stream, &graph);
    if (e != cudaSuccess || !graph) {
        cudaGetLastError();
        return fq_fail(dev, FQ_ERR_CUDA, "end capture: %s", cudaGetErrorString(e));
    }
    cudaGraphExec_t exec = nullptr;
    e = cudaGraphInstantiate(&exec, graph, 0);
    if (e != cudaSuccess) {
        cudaGraphDestroy(graph);
        return fq_check_cuda(dev, e, "graph instantiate");
    }
    fq_graph *g = new fq_graph();
    g->dev = dev;
    g->graph = graph;
    g->exec = exec;
    g->kernels = dev->captured_kernels;
    g->comm = dev->cap_comm;
    g->first_off = dev->cap_first_off;
    g->first_bytes = dev->cap_first_bytes;
    g->last_off = dev->cap_last_off;
    g->last_bytes = dev->cap_last_bytes;
    *out = g;
    return FQ_OK;
}

extern "C" int fq_graph_launch(fq_device *dev, fq_graph *graph) {
    if (int rc = fq_begin_enqueue(dev)) return rc;
    if (!graph || graph->dev != dev) return fq_fail(dev, FQ_ERR_DEVICE, "graph belongs to another device handle");
    if (dev->capturing) return fq_fail(dev, FQ_ERR_PARAM, "graph launch inside a capture");
    if (int rc = fq_comm_note_graph(dev, graph)) return rc;
    if (int rc = fq_check_cuda(dev, cudaGraphLaunch(graph->exec, dev->stream), "graph launch")) return rc;
    dev->counters.dispatches += graph->kernels;
    return FQ_OK;
}

extern "C" int fq_graph_destroy(fq_graph *graph) {
    if (!graph) return FQ_ERR_PARAM;
    cudaSetDevice(graph->dev->ordinal);
    cudaStreamSynchronize(graph->dev->stream);
    if (graph->exec) cudaGraphExecDestroy(graph->exec);
    if (graph->graph) cudaGraphDestroy(graph->graph);
    delete graph;
    return FQ_OK;
}

// ------------------------------------------------------------------ buffers

extern "C" int fq_buffer_alloc(fq_device *dev, size_t bytes, void **device_ptr) {
    if (!dev || !device_ptr || bytes == 0) return fq_fail(dev, FQ_ERR_PARAM, "buffer of %zu bytes", bytes);
    cudaSetDevice(dev->ordinal);
    void *p = nullptr;
    if (int rc = fq_check_cuda(dev, cudaMalloc(&p, bytes), "cudaMalloc")) return rc;
    dev->allocations[(uintptr_t)p] = bytes;
    *device_ptr = p;
    return FQ_OK;
}

extern "C" int fq_buffer_free(fq_device *dev, void *device_ptr) {
    if (!dev) return FQ_ERR_PARAM;
    auto it = dev->allocations.find((uintptr_t)device_ptr);
    if (it == dev->allocations.end()) return fq_fail(dev, FQ_ERR_RANGE, "%p was not allocated by this handle", device_ptr);
    cudaSetDevice(dev->ordinal);
    cudaStreamSynchronize(dev->stream);
    // Nothing is remembered about a buffer that is gone.
    const uintptr_t lo = it->first, hi = it->first + it->second;
    auto inside = [&](const std::pair<uintptr_t, uintptr_t> &r) { return r.first >= lo && r.second <= hi; };
    dev->failed_writes.erase(std::remove_if(dev->failed_writes.begin(), dev->failed_writes.end(), inside), dev->failed_writes.end());
    dev->pending_writes.erase(std::remove_if(dev->pending_writes.begin(), dev->pending_writes.end(), inside), dev->pending_writes.end());
    dev->allocations.erase(it);
    return fq_check_cuda(dev, cudaFree(device_ptr), "cudaFree");
}

extern "C" int fq_upload(fq_device *dev, void *device_ptr, const void *host, size_t bytes) {
    if (!dev || !host) return fq_fail(dev, FQ_ERR_PARAM, "upload arguments");
    if (int rc = fq_begin_enqueue(dev)) return rc;
    if (int rc = fq_check_binding(dev, device_ptr, bytes, "upload destination")) return rc;
    dev->counters.bytes_uploaded += bytes;
    fq_note_write(dev, device_ptr, bytes);
    return fq_check_cuda(dev, cudaMemcpyAsync(device_ptr, host, bytes, cudaMemcpyHostToDevice, dev->stream), "upload");
}

extern "C" int fq_download_async(fq_device *dev, void *host, const void *device_ptr, size_t bytes) {
    if (!dev || !host) return fq_fail(dev, FQ_ERR_PARAM, "download arguments");
    if (int rc = fq_begin_enqueue(dev)) return rc;
    if (int rc = fq_check_binding(dev, device_ptr, bytes, "download source")) return rc;
    dev->counters.bytes_downloaded += bytes;
    return fq_check_cuda(dev, cudaMemcpyAsync(host, device_ptr, bytes, cudaMemcpyDeviceToHost, dev->stream), "download");
}

extern "C" int fq_download(fq_device *dev, void *host, const void *device_ptr, size_t bytes) {
    if (int rc = fq_download_async(dev, host, device_ptr, bytes)) return rc;
    // A read of results is a completion point, as `Tensor::to_f32` is in the reference.
    return fq_synchronize(dev);
}

// ------------------------------------------------------------------ matrices

static float half_bits_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 31) bits = sign | 0x7F800000u | (man << 13);
    else if (exp == 0) {
        // Only finiteness and sign matter here; a subnormal is finite.
        bits = sign | (man ? 0x33800000u : 0u);
    } else bits = sign | ((exp + 112) << 23) | (man << 13);
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

// `validate_gguf_quantized_payload` (src/quantization.rs:212-261).
static int validate_payload(fq_device *dev, int format, const uint8_t *p, size_t len, uint32_t bb) {
    auto finite = [](float v) { return v == v && v - v == 0.0f; };
    for (size_t o = 0; o < len; o += bb) {
        const uint8_t *b = p + o;
        auto half_at = [&](int at) { return half_bits_to_float((uint16_t)(b[at] | (b[at + 1] << 8))); };
        if (format == FQ_Q4_K || format == FQ_Q5_K) {
            if (!finite(half_at(0)) || !finite(half_at(2)))
                return fq_fail(dev, FQ_ERR_WEIGHT, "%s scale must be finite (block %zu)", format == FQ_Q4_K ? "Q4_K" : "Q5_K", o / bb);
        } else if (format == FQ_Q6_K) {
            if (!finite(half_at(208))) return fq_fail(dev, FQ_ERR_WEIGHT, "Q6_K scale must be finite (block %zu)", o / bb);
        } else if (format == FQ_IQ4_NL || format == FQ_IQ4_XS) {
            if (!finite(half_at(0))) return fq_fail(dev, FQ_ERR_WEIGHT, "%s scale must be finite (block %zu)", format == FQ_IQ4_NL ? "IQ4_NL" : "IQ4_XS", o / bb);
        } else {
            const float s = half_at(0);
            if (!finite(s) || s < 0.0f) return fq_fail(dev, FQ_ERR_WEIGHT, "Q8_0 scale must be finite (block %zu)", o / bb);
            for (int i = 2; i < 34; i++)
                if (b[i] == 0x80) return fq_fail(dev, FQ_ERR_WEIGHT, "Q8_0 value -128 is outside the GGML range (block %zu)", o / bb);
        }
    }
    return FQ_OK;
}

extern "C" int fq_matrix_create(fq_device *dev, int format, uint64_t rows, uint64_t cols, uint64_t experts,
                                const void *packed, size_t len, fq_matrix **out) {
    if (!dev || !out) return FQ_ERR_PARAM;
    *out = nullptr;
    uint32_t el, bb;
    switch (format) {
    case FQ_Q4_K: el = 256; bb = 144; break;
    case FQ_Q5_K: el = 256; bb = 176; break;
    case FQ_Q6_K: el = 256; bb = 210; break;
    case FQ_Q8_0: el = 32; bb = 34; break;
    case FQ_IQ4_NL: el = 32; bb = 18; break;
    case FQ_IQ4_XS: el = 256; bb = 136; break;
    default: return fq_fail(dev, FQ_ERR_WEIGHT, "GGML type %d has no kernel", format);
    }
    if (!packed) return fq_fail(dev, FQ_ERR_PARAM, "null payload");
    if (rows == 0 || cols == 0 || experts == 0) return fq_fail(dev, FQ_ERR_SHAPE, "empty matrix geometry");
    if (cols % el || cols % 64) return fq_fail(dev, FQ_ERR_WEIGHT, "row width is not a whole number of blocks");
    if (cols > FQ_MAX_COLS || rows * experts > 0x7fffffffull) return fq_fail(dev, FQ_ERR_SHAPE, "matrix geometry is out of range");
    const uint64_t row_bytes = cols / el * bb;
    if (row_bytes * rows * experts != len) return fq_fail(dev, FQ_ERR_WEIGHT, "byte length differs from geometry");
    if (int rc = validate_payload(dev, format, (const uint8_t *)packed, len, bb)) return rc;
    if (int rc = fq_check_cuda(dev, cudaSetDevice(dev->ordinal), "cudaSetDevice")) return rc;
    fq_matrix *w = new fq_matrix();
    w->dev = dev;
    w->format = format;
    w->rows = rows * experts;
    w->cols = cols;
    w->experts = experts;
    w->row_bytes = row_bytes;
    w->byte_size = len;
    w->block_elems = el;
    w->block_bytes = bb;
    w->pitch = fq_row_pitch(format, (uint32_t)cols);
    const size_t dev_len = (size_t)w->pitch * w->rows;
    // Q6_K and Q8_0 are regrouped by field on the host (see blocks.cuh); Q4_K uploads as it is.
    std::vector<uint8_t> regrouped;
    const uint8_t *upload = (const uint8_t *)packed;
    if (format == FQ_Q6_K) {
        regrouped.assign(dev_len, 0);
        const size_t nb = cols / 256;
        for (size_t r = 0; r < w->rows; r++) {
            const uint8_t *src = (const uint8_t *)packed + r * row_bytes;
            uint8_t *dst = regrouped.data() + r * w->pitch;
            for (size_t b = 0; b < nb; b++, src += 210) {
                memcpy(dst + 128 * b, src, 128);
                memcpy(dst + 128 * nb + 64 * b, src + 128, 64);
                memcpy(dst + 192 * nb + 16 * b, src + 192, 16);
                memcpy(dst + 208 * nb + 2 * b, src + 208, 2);
            }
        }
        upload = regrouped.data();
    } else if (format == FQ_Q8_0) {
        regrouped.assign(dev_len, 0);
        const size_t nb = cols / 32;
        for (size_t r = 0; r < w->rows; r++) {
            const uint8_t *src = (const uint8_t *)packed + r * row_bytes;
            uint8_t *dst = regrouped.data() + r * w->pitch;
            for (size_t b = 0; b < nb; b++, src += 34) {
                memcpy(dst + 32 * nb + 2 * b, src, 2);
                memcpy(dst + 32 * b, src + 2, 32);
            }
        }
        upload = regrouped.data();
    } else if (format == FQ_IQ4_NL || format == FQ_IQ4_XS) {
        // nibbles of all blocks first, then the rest of each block (IQ4_NL: d; IQ4_XS: d | scales_h | scales_l)
        regrouped.assign(dev_len, 0);
        const size_t nb = cols / el, qb = el / 2, hb = bb - qb;
        for (size_t r = 0; r < w->rows; r++) {
            const uint8_t *src = (const uint8_t *)packed + r * row_bytes;
            uint8_t *dst = regrouped.data() + r * w->pitch;
            for (size_t b = 0; b < nb; b++, src += bb) {
                memcpy(dst + qb * nb + hb * b, src, hb);
                memcpy(dst + qb * b, src + hb, qb);
            }
        }
        upload = regrouped.data();
    }
    // 256 spare bytes let kernels read whole 16-byte words around the last block.
    cudaError_t e = cudaMalloc((void **)&w->data, dev_len + 256);
    if (e == cudaSuccess) e = cudaMemsetAsync(w->data + dev_len, 0, 256, dev->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(w->data, upload, dev_len, cudaMemcpyHostToDevice, dev->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(dev->stream);
    if (e != cudaSuccess) {
        if (w->data) cudaFree(w->data);
        delete w;
        return fq_check_cuda(dev, e, "weight upload");
    }
    dev->counters.bytes_uploaded += len;
    *out = w;
    return FQ_OK;
}

extern "C" int fq_matrix_destroy(fq_matrix *w) {
    if (!w) return FQ_ERR_PARAM;
    cudaSetDevice(w->dev->ordinal);
    cudaStreamSynchronize(w->dev->stream);
    cudaFree(w->data);
    delete w;
    return FQ_OK;
}

extern "C" int fq_matrix_get_info(const fq_matrix *w, fq_matrix_info *out) {
    if (!w || !out) return FQ_ERR_PARAM;
    out->rows = w->rows;
    out->cols = w->cols;
    out->experts = w->experts;
    out->row_bytes = w->row_bytes;
    out->byte_size = w->byte_size;
    out->format = w->format;
    return FQ_OK;
}

// ------------------------------------------------------------------ op surface

static ProjectArgs base_args(const fq_matrix *w, const void *x, int xd, void *y, int yd) {
    ProjectArgs a{};
    a.w = w->data;
    a.format = (uint32_t)w->format;
    a.rows = (uint32_t)w->expert_rows();
    a.cols = (uint32_t)w->cols;
    a.row_bytes = (uint32_t)w->pitch;
    a.x = x;
    a.y = y;
    a.x_dtype = xd;
    a.y_dtype = yd;
    a.experts = (uint32_t)w->experts;
    return a;
}

static int check_dtype(fq_device *dev, int dt) {
    return (dt == FQ_F32 || dt == FQ_BF16) ? FQ_OK : fq_fail(dev, FQ_ERR_UNSUPPORTED, "element type %d", dt);
}

// Decode / verify widths (F32 in and out): Q8_0 on the integer-dot kernel, Q4_K / Q6_K on the integer tensor
// path -- one activation row (and per-route expert projections) in gemv_i8.cu, 2..16 rows in gemv_nt.cu.
static int launch_decode(fq_device *dev, const ProjectArgs *a, uint32_t count) {
    if (count == 1 && a[0].format == FQ_Q8_0) {
        int rc = fq_launch_gemv_q8(dev, a[0]);
        if (rc != FQ_ERR_UNSUPPORTED) return rc;
    }
    if (count == 1 && (a[0].m == 1 || a[0].ids) && (a[0].format == FQ_IQ4_NL || a[0].format == FQ_IQ4_XS)) { // dense with more rows: the exact kernel measured faster
        int rc = fq_launch_gemv_iq4(dev, a[0]);
        if (rc != FQ_ERR_UNSUPPORTED) return rc;
    }
    if (a[0].m == 1 || a[0].ids) return fq_launch_gemv_i8_many(dev, a, count);
    return fq_launch_gemv_nt_many(dev, a, count);
}

extern "C" int fq_project(fq_device *dev, const fq_matrix *w, const void *x, int x_dtype, size_t x_elems, size_t m,
                          void *y, int y_dtype, size_t y_elems) {
    if (int rc = fq_begin_enqueue(dev)) return rc;
    if (!w) return fq_fail(dev, FQ_ERR_PARAM, "null matrix");
    if (w->dev != dev) return fq_fail(dev, FQ_ERR_DEVICE, "matrix belongs to another device handle");
    if (int rc = check_dtype(dev, x_dtype)) return rc;
    if (int rc = check_dtype(dev, y_dtype)) return rc;
    if (m == 0 || x_elems != m * w->cols || y_elems != m * w->rows)
        return fq_fail(dev, FQ_ERR_SHAPE, "projection [%zu, %llu] x [%llu, %llu]^T into %zu values", m,
                       (unsigned long long)w->cols, (unsigned long long)w->rows, (unsigned long long)w->cols, y_elems);
    if (m > 0x7fffffffu / 8) return fq_fail(dev, FQ_ERR_SHAPE, "too many activation rows");
    const size_t xb = x_elems * fq_dtype_size(x_dtype), yb = y_elems * fq_dtype_size(y_dtype);
    if (int rc = fq_check_binding(dev, x, xb, "x")) return rc;
    if (int rc = fq_check_binding(dev, y, yb, "y")) return rc;
    if (int rc = fq_check_no_alias(dev, y, yb, x, xb, "y")) return rc;
    ProjectArgs a = base_args(w, x, x_dtype, y, y_dtype);
    a.rows = (uint32_t)w->rows; // a plain projection spans every stacked row
    a.m = (uint32_t)m;
    if (!dev->exact) {
        int rc = FQ_ERR_UNSUPPORTED;
        if (m <= (size_t)FQ_GEMV_MAX_M && x_dtype == FQ_F32 && y_dtype == FQ_F32) rc = launch_decode(dev, &a, 1);
        else if (x_dtype == y_dtype) rc = fq_launch_gemm_tc(dev, a);
        if (rc != FQ_ERR_UNSUPPORTED) return rc;
    }
    if (int rc = fq_launch_project_exact(dev, a)) return rc;
    return fq_end_enqueue(dev, "project", 1);
}

extern "C" int fq_project_many(fq_device *dev, const fq_matrix *const *w, size_t count, const void *x, int x_dtype,
                               size_t x_elems, size_t m, void *const *y, int y_dtype) {
    if (int rc = fq_begin_enqueue(dev)) return rc;
    if (!w || !y || count == 0) return fq_fail(dev, FQ_ERR_PARAM, "projection list");
    if (int rc = check_dtype(dev, x_dtype)) return rc;
    if (int rc = check_dtype(dev, y_dtype)) return rc;
    constexpr size_t MAX = 8;
    if (count > MAX) return fq_fail(dev, FQ_ERR_PARAM, "at most %zu projections share an input", MAX);
    ProjectArgs args[MAX];
    for (size_t i = 0; i < count; i++) {
        if (!w[i]) return fq_fail(dev, FQ_ERR_PARAM, "null matrix");
        if (w[i]->dev != dev) return fq_fail(dev, FQ_ERR_DEVICE, "matrix belongs to another device handle");
        if (m == 0 || x_elems != m * w[i]->cols)
            return fq_fail(dev, FQ_ERR_SHAPE, "projection [%zu, %llu] from %zu values", m, (unsigned long long)w[i]->cols, x_elems);
        const size_t xb = x_elems * fq_dtype_size(x_dtype), yb = m * w[i]->rows * fq_dtype_size(y_dtype);
        if (int rc = fq_check_binding(dev, x, xb, "x")) return rc;
        if (int rc = fq_check_binding(dev, y[i], yb, "y")) return rc;
        if (int rc = fq_check_no_alias(dev, y[i], yb, x, xb, "y")) return rc;
        for (size_t j = 0; j < i; j++)
            if (int rc = fq_check_no_alias(dev, y[i], yb, y[j], m * w[j]->rows * fq_dtype_size(y_dtype), "y")) return rc;
        args[i] = base_args(w[i], x, x_dtype, y[i], y_dtype);
        args[i].rows = (uint32_t)w[i]->rows;
        args[i].m = (uint32_t)m;
    }
    if (!dev->exact && count <= 4) {
        int rc = m <= (size_t)FQ_GEMV_MAX_M ? launch_decode(dev, args, (uint32_t)count) : fq_launch_gemm_tc_many(dev, args, (uint32_t)count);
        if (rc != FQ_ERR_UNSUPPORTED) return rc;
    }
    dev->tp_push = nullptr; // separate launches cannot share one fused exchange
    for (size_t i = 0; i < count; i++)
        if (int rc = fq_project(dev, w[i], x, x_dtype, x_elems, m, y[i], y_dtype, m * w[i]->rows)) return rc;
    return FQ_OK;
}

// `fq_project_many` on rmsnorm(x) * norm_w (F32 in and out): at decode and verify widths on the K-quant formats the
// normalisation happens inside the projections' activation preparation; otherwise `fq_rmsnorm` into `scratch`
// (m * cols floats), then the projections.
extern "C" int fq_rmsnorm_project_many(fq_device *dev, const fq_matrix *const *w, size_t count, const float *x, const float *norm_w, float eps,
                                       size_t x_elems, size_t m, float *scratch, void *const *y) {
    if (int rc = fq_begin_enqueue(dev)) return rc;
    if (!w || !y || count == 0 || !w[0]) return fq_fail(dev, FQ_ERR_PARAM, "projection list");
    const size_t cols = w[0]->cols;
    if (m == 0 || x_elems != m * cols || cols % 4) return fq_fail(dev, FQ_ERR_SHAPE, "normalised projection [%zu, %zu] from %zu values", m, cols, x_elems);
    if (int rc = fq_check_binding(dev, x, x_elems * 4, "x")) return rc;
    if (int rc = fq_check_binding(dev, norm_w, cols * 4, "norm_w")) return rc;
    bool fused = !dev->exact && m <= (size_t)FQ_GEMV_MAX_M && count <= 4;
    ProjectArgs args[4];
    for (size_t i = 0; i < count && fused; i++) {
        if (!w[i] || w[i]->dev != dev) return fq_fail(dev, FQ_ERR_DEVICE, "matrix belongs to another device handle");
        fused = w[i]->cols == cols && w[i]->format == w[0]->format && (w[i]->format == FQ_Q4_K || w[i]->format == FQ_Q5_K || w[i]->format == FQ_Q6_K);
        if (!fused) break;
        const size_t yb = m * w[i]->rows * 4;
        if (int rc = fq_check_binding(dev, y[i], yb, "y")) return rc;
        if (int rc = fq_check_no_alias(dev, y[i], yb, x, x_elems * 4, "y")) return rc;
        args[i] = base_args(w[i], x, FQ_F32, y[i], FQ_F32);
        args[i].rows = (uint32_t)w[i]->rows;
        args[i].m = (uint32_t)m;
        args[i].norm_w = norm_w;
        args[i].norm_eps = eps;
    }
    if (fused) {
        const int rc = launch_decode(dev, args, (uint32_t)count);
        if (rc != FQ_ERR_UNSUPPORTED) return rc;
    }
    if (!scratch) return fq_fail(dev, FQ_ERR_RANGE, "scratch: these projections need the normalised activations in memory");
    if (int rc = fq_rmsnorm(dev, x, norm_w, (uint32_t)cols, eps, (uint32_t)m, scratch)) return rc;
    return fq_project_many(dev, w, count, scratch, FQ_F32, x_elems, m, y, FQ_F32);
}

// Row-sharded `fq_project_many`: every y[i] lies in this rank's slice [region_offset + rank * shard_bytes,
// + shard_bytes) of a gathered region of the communicator's symmetric buffer.  Decode widths on the integer
// kernel exchange inside the projection kernel; anything else projects first and gathers the region with
// the copy kernel.
extern "C" int fq_project_many_gather(fq_device *dev, fq_comm *comm, size_t region_offset, size_t shard_bytes, const fq_matrix *const *w,
                                      size_t count, const void *x, int x_dtype, size_t x_elems, size_t m, void *const *y, int y_dtype) {
    if (!dev || !comm || !w || !y || count == 0) return fq_fail(dev, FQ_ERR_PARAM, "projection list");
    if (fq_comm_device(comm) != dev) return fq_fail(dev, FQ_ERR_DEVICE, "communicator belongs to another device handle");
    const int world = fq_comm_world(comm), rank = fq_comm_rank(comm);
    if (y_dtype != FQ_F32) return fq_fail(dev, FQ_ERR_UNSUPPORTED, "gathered projections are F32");
    if (shard_bytes == 0 || shard_bytes % 16 || region_offset % 16 || region_offset + shard_bytes * world > fq_comm_bytes(comm))
        return fq_fail(dev, FQ_ERR_RANGE, "gather of %zu bytes per rank at offset %zu does not fit the symmetric buffer", shard_bytes, region_offset);
    // The outputs tile this rank's slice from its start, in order, without gaps (what follows them is padding
    // that no rank sends or waits for).
    const uint8_t *mine = fq_comm_local(comm) + region_offset + (size_t)rank * shard_bytes;
    size_t covered = 0;
    for (size_t i = 0; i < count; i++) {
        if (!w[i]) return fq_fail(dev, FQ_ERR_PARAM, "null matrix");
        if ((const uint8_t *)y[i] != mine + covered)
            return fq_fail(dev, FQ_ERR_RANGE, "output %zu does not follow the output before it from the start of this rank's slice", i);
        covered += m * w[i]->rows * 4;
    }
    if (covered > shard_bytes) return fq_fail(dev, FQ_ERR_RANGE, "%zu bytes of outputs exceed the slice of %zu bytes", covered, shard_bytes);
    if (world == 1) return fq_project_many(dev, w, count, x, x_dtype, x_elems, m, y, y_dtype);
    if (int rc = fq_begin_enqueue(dev)) return rc;
    if (int rc = fq_comm_note_region(dev, comm, region_offset, shard_bytes * world)) return rc;
    TpPush push{};
    if (int rc = fq_comm_begin_push(comm, mine, shard_bytes, &push)) return fq_fail(dev, rc, "communicator peers are not opened");
    push.covered_bytes = covered;
    dev->tp_push = &push;
    dev->tp_pushed = false;
    const int rc = fq_project_many(dev, w, count, x, x_dtype, x_elems, m, y, y_dtype);
    dev->tp_push = nullptr;
    if (rc) return rc;
    if (dev->tp_pushed) return FQ_OK;
    return fq_comm_all_gather_unchecked(dev, comm, region_offset, shard_bytes);
}

extern "C" int fq_project_id(fq_device *dev, const fq_matrix *w, const float *x, size_t x_elems, const uint32_t *ids,
                             size_t routes, size_t x_div, float *y, size_t y_elems) {
    if (int rc = fq_begin_enqueue(dev)) return rc;
    if (!w) return fq_fail(dev, FQ_ERR_PARAM, "null matrix");
    if (w->dev != dev) return fq_fail(dev, FQ_ERR_DEVICE, "matrix belongs to another device handle");
    const size_t rows_e = w->expert_rows();
    if (routes == 0 || x_div == 0 || y_elems != routes * rows_e || x_elems * x_div != routes * w->cols)
        return fq_fail(dev, FQ_ERR_SHAPE, "expert projection geometry");
    if (int rc = fq_check_binding(dev, x, x_elems * 4, "x")) return rc;
    if (int rc = fq_check_binding(dev, ids, routes * 4, "ids")) return rc;
    if (int rc = fq_check_binding(dev, y, y_elems * 4, "y")) return rc;
    if (int rc = fq_check_no_alias(dev, y, y_elems * 4, x, x_elems * 4, "y")) return rc;
    if (int rc = fq_check_no_alias(dev, y, y_elems * 4, ids, routes * 4, "y")) return rc;
    ProjectArgs a = base_args(w, x, FQ_F32, y, FQ_F32);
    a.m = (uint32_t)routes;
    a.ids = ids;
    a.x_div = (uint32_t)x_div;
    if (!dev->exact) {
        int rc = launch_decode(dev, &a, 1);
        if (rc != FQ_ERR_UNSUPPORTED) return rc;
    }
    if (int rc = fq_launch_project_id_exact(dev, a)) return rc;
    return fq_end_enqueue(dev, "project_id", 1);
}

// Grouped F32 projections by average rows per expert: below GROUPED_F16_MIN_AVG_ROWS the integer kernel of
// gemv_nt.cu (the work is streaming weights; its per-row arithmetic is still small), from there on the fp16
// tensor-core kernel k_gemm_f16g, which decodes every weight once per 64 rows (measured on the 35B-A3B-class
// block, integer against fp16 kernel: 378 / 385 us at 14 rows per expert, 406 / 384 at 16, 425 / 394 at 20,
// 446 / 421 at 24, 538 / 452 at 32, 702 / 578 at 48).  Formats the fp16 kernel does not serve stay on the integer
// kernel up to GROUPED_NT_MAX_AVG_ROWS.
constexpr size_t GROUPED_F16_MIN_AVG_ROWS = 16;
constexpr size_t GROUPED_NT_MAX_AVG_ROWS = 48;

// Arguments as fq_launch_gemv_nt_grouped, and `group_rows`: how many of the rows the groups in `a` cover (all of
// them, or a rank's expected share); FQ_ERR_UNSUPPORTED when neither kernel serves the shape.
static int launch_grouped_f32(fq_device *dev, const ProjectArgs *a, uint32_t count, uint32_t total_rows, size_t group_rows, const uint32_t *src,
                              uint32_t src_div) {
    int rc = FQ_ERR_UNSUPPORTED;
    if (group_rows >= GROUPED_F16_MIN_AVG_ROWS * a[0].groups) rc = fq_launch_gemm_f16_grouped(dev, a, count, total_rows, src, src_div);
    if (rc == FQ_ERR_UNSUPPORTED && group_rows <= GROUPED_NT_MAX_AVG_ROWS * a[0].groups)
        rc = fq_launch_gemv_nt_grouped(dev, a, count, total_rows, src, src_div);
    return rc;
}

extern "C" int fq_project_mm_id(fq_device *dev, const fq_matrix *w, const void *x, int x_dtype, size_t x_elems,
                                const uint32_t *offsets, const uint32_t *slots, size_t groups, size_t max_rows,
                                void *y, int y_dtype, size_t y_elems) {
    if (int rc = fq_begin_enqueue(dev)) return rc;
    if (!w) return fq_fail(dev, FQ_ERR_PARAM, "null matrix");
    if (w->dev != dev) return fq_fail(dev, FQ_ERR_DEVICE, "matrix belongs to another device handle");
    if (int rc = check_dtype(dev, x_dtype)) return rc;
    if (int rc = check_dtype(dev, y_dtype)) return rc;
    const size_t rows_e = w->expert_rows();
    if (groups == 0 || max_rows == 0 || x_elems % w->cols || y_elems % rows_e || x_elems / w->cols != y_elems / rows_e ||
        (!slots && groups != w->experts))
        return fq_fail(dev, FQ_ERR_SHAPE, "grouped expert projection geometry");
    const size_t xb = x_elems * fq_dtype_size(x_dtype), yb = y_elems * fq_dtype_size(y_dtype);
    if (int rc = fq_check_binding(dev, x, xb, "x")) return rc;
    if (int rc = fq_check_binding(dev, offsets, (groups + 1) * 4, "offsets", 4)) return rc;
    if (slots)
        if (int rc = fq_check_binding(dev, slots, groups * 4, "slots", 4)) return rc;
    if (int rc = fq_check_binding(dev, y, yb, "y")) return rc;
    if (int rc = fq_check_no_alias(dev, y, yb, x, xb, "y")) return rc;
    ProjectArgs a = base_args(w, x, x_dtype, y, y_dtype);
    a.offsets = offsets;
    a.slots = slots;
    a.groups = (uint32_t)groups;
    a.max_rows = (uint32_t)max_rows;
    if (!dev->exact) {
        const uint32_t total_rows = (uint32_t)(x_elems / w->cols);
        int rc = FQ_ERR_UNSUPPORTED;
        // F32 callers: the integer kernel or the fp16 tensor-core kernel, by rows per expert; what neither serves
        // (and BF16 callers) takes the bf16 tcgen05 GEMM.
        if (x_dtype == FQ_F32 && y_dtype == FQ_F32) rc = launch_grouped_f32(dev, &a, 1, total_rows, total_rows, nullptr, 1);
        if (rc == FQ_ERR_UNSUPPORTED) rc = fq_launch_gemm_tc_grouped(dev, a, total_rows);
        if (rc != FQ_ERR_UNSUPPORTED) return rc;
    }
    if (int rc = fq_launch_project_grouped_exact(dev, a)) return rc;
    return fq_end_enqueue(dev, "project_mm_id", 1);
}

extern "C" int fq_get_rows(fq_device *dev, const fq_matrix *w, const uint32_t *ids, size_t tokens, void *y, int y_dtype,
                           size_t y_elems) {
    if (int rc = fq_begin_enqueue(dev)) return rc;
    if (!w) return fq_fail(dev, FQ_ERR_PARAM, "null matrix");
    if (w->dev != dev) return fq_fail(dev, FQ_ERR_DEVICE, "matrix belongs to another device handle");
    if (int rc = check_dtype(dev, y_dtype)) return rc;
    if (tokens == 0 || y_elems != tokens * w->cols) return fq_fail(dev, FQ_ERR_SHAPE, "embedding lookup geometry");
    if (int rc = fq_check_binding(dev, ids, tokens * 4, "ids")) return rc;
    if (int rc = fq_check_binding(dev, y, y_elems * fq_dtype_size(y_dtype), "y")) return rc;
    if (int rc = fq_check_no_alias(dev, y, y_elems * fq_dtype_size(y_dtype), ids, tokens * 4, "y")) return rc;
    if (int rc = fq_launch_get_rows(dev, w, ids, (uint32_t)tokens, y, y_dtype)) return rc;
    return fq_end_enqueue(dev, "get_rows", 1);
}

// ------------------------------------------------------------------ feed-forward blocks

// A branch of independent work on the side stream: everything enqueued between side_begin and side_end runs
// after what `stream` held at side_begin and concurrently with what `stream` gets until side_end, after which
// `stream` waits for the branch.  Works the same while `stream` is being captured (fork / join by events).
struct SideBranch {
    fq_device *dev;
    cudaStream_t main;
    void *xprep;
    size_t xprep_bytes;
    bool on;
};
// The scratch areas kernels of the two streams must not share.
static void swap_side_scratch(fq_device *dev) {
    std::swap(dev->xprep, dev->side_xprep);
    std::swap(dev->xprep_bytes, dev->side_xprep_bytes);
    std::swap(dev->nt_ws, dev->side_nt_ws);
    std::swap(dev->nt_ws_bytes, dev->side_nt_ws_bytes);
    std::swap(dev->nt_counters, dev->side_nt_counters);
    std::swap(dev->nt_counter_count, dev->side_nt_counter_count);
}
static SideBranch side_begin(fq_device *dev) {
    SideBranch b{dev, dev->stream, dev->xprep, dev->xprep_bytes, false};
    if (!dev->side_stream) return b;
    if (cudaEventRecord(dev->fork_event, dev->stream) != cudaSuccess || cudaStreamWaitEvent(dev->side_stream, dev->fork_event, 0) != cudaSuccess) {
        cudaGetLastError();
        return b;
    }
    dev->stream = dev->side_stream;
    swap_side_scratch(dev);
    b.on = true;
    return b;
}
// End of the branch's enqueues: later calls go to `stream` again (and run beside the branch).
static int side_detach(SideBranch &b) {
    if (!b.on) return FQ_OK;
    fq_device *dev = b.dev;
    const cudaError_t e = cudaEventRecord(dev->join_event, dev->side_stream);
    dev->stream = b.main;
    swap_side_scratch(dev);
    return fq_check_cuda(dev, e, "side stream event");
}
// `stream` waits for the branch.
static int side_join(SideBranch &b) {
    if (!b.on) return FQ_OK;
    b.on = false;
    return fq_check_cuda(b.dev, cudaStreamWaitEvent(b.dev->stream, b.dev->join_event, 0), "joining the side stream");
}

// y = W . (silu(g) * u): at decode widths the gated unit is computed inside the projection's activation
// preparation (no separate launch, no round trip of `act`); otherwise `fq_glu` into `act`, then the projection.
// With `ids` (routes, one activation row each) W is an expert stack.
// `combine` (routes only): the projection also carries out the weighted sum over each token's routes; `*combined`
// tells whether it did (else the caller combines).
// `route_map` (with `ids`; may be null): output row r takes the expert ids[route_map[r]] - id_base, rows whose expert
// the matrix does not hold are skipped; only the decode kernel does that (FQ_ERR_UNSUPPORTED otherwise, nothing
// enqueued).
static int project_gated(fq_device *dev, const fq_matrix *w, const float *g, const float *u, float *act, size_t rows_x, const uint32_t *ids,
                         float *y, const CombineTail *combine = nullptr, bool *combined = nullptr, const uint32_t *route_map = nullptr,
                         uint32_t id_base = 0) {
    const size_t width = w->cols, rows_e = w->expert_rows();
    if (combined) *combined = false;
    if (route_map && (dev->exact || !ids)) return FQ_ERR_UNSUPPORTED;
    if (!dev->exact) {
        if (int rc = fq_begin_enqueue(dev)) return rc;
        if (int rc = fq_check_binding(dev, g, rows_x * width * 4, "gate")) return rc;
        if (int rc = fq_check_binding(dev, u, rows_x * width * 4, "up")) return rc;
        if (int rc = fq_check_binding(dev, y, rows_x * rows_e * 4, "y")) return rc;
        ProjectArgs a = base_args(w, g, FQ_F32, y, FQ_F32);
        a.x_up = u;
        a.m = (uint32_t)rows_x;
        if (ids) {
            a.ids = ids;
            a.x_div = 1;
            a.route_map = route_map;
            a.id_base = id_base;
        } else {
            a.rows = (uint32_t)w->rows;
        }
        if (route_map) return fq_launch_gemv_i8_many(dev, &a, 1);
        if (ids && combine) {
            a.combine = combine;
            const int rc = fq_launch_gemv_i8_many(dev, &a, 1);
            if (rc != FQ_ERR_UNSUPPORTED) {
                if (combined) *combined = rc == FQ_OK;
                return rc;
            }
            a.combine = nullptr;
        }
        const int rc = (ids || rows_x == 1) ? fq_launch_gemv_i8_many(dev, &a, 1) : fq_launch_gemv_nt_many(dev, &a, 1);
        if (rc != FQ_ERR_UNSUPPORTED) return rc;
    }
    if (int rc = fq_glu(dev, g, u, rows_x * width, act)) return rc;
    if (ids) return fq_project_id(dev, w, act, rows_x * width, ids, rows_x, 1, y, rows_x * rows_e);
    return fq_project(dev, w, act, FQ_F32, rows_x * width, rows_x, y, FQ_F32, rows_x * rows_e);
}

// Two expert stacks of one shape (gate and up) on the same routes: one launch at decode widths.
// `route_map` (may be null): output row r takes route route_map[r] -- its activation row route_map[r] / x_div and
// the expert ids[route_map[r]] - id_base; rows whose expert the matrices do not hold are skipped.  Only the decode
// kernel does that (FQ_ERR_UNSUPPORTED otherwise, nothing enqueued).
static int project_id_pair(fq_device *dev, const fq_matrix *w0, const fq_matrix *w1, const float *x, size_t x_elems, const uint32_t *ids,
                           size_t routes, size_t x_div, float *y0, float *y1, const uint32_t *route_map = nullptr, uint32_t id_base = 0) {
    const bool alike = w0->format == w1->format && w0->cols == w1->cols && w0->expert_rows() == w1->expert_rows() && w0->experts == w1->experts;
    if (route_map && (dev->exact || !alike)) return FQ_ERR_UNSUPPORTED;
    if (!dev->exact && alike) {
        if (int rc = fq_begin_enqueue(dev)) return rc;
        ProjectArgs a[2] = {base_args(w0, x, FQ_F32, y0, FQ_F32), base_args(w1, x, FQ_F32, y1, FQ_F32)};
        for (ProjectArgs &p : a) {
            p.m = (uint32_t)routes;
            p.ids = ids;
            p.x_div = (uint32_t)x_div;
            p.route_map = route_map;
            p.id_base = id_base;
            p.map_x = route_map != nullptr;
        }
        if (int rc = fq_check_binding(dev, x, x_elems * 4, "x")) return rc;
        if (int rc = fq_check_binding(dev, ids, routes * 4, "ids")) return rc;
        if (int rc = fq_check_binding(dev, y0, routes * w0->expert_rows() * 4, "y")) return rc;
        if (int rc = fq_check_binding(dev, y1, routes * w1->expert_rows() * 4, "y")) return rc;
        const int rc = fq_launch_gemv_i8_many(dev, a, 2);
        if (rc != FQ_ERR_UNSUPPORTED || route_map) return rc;
    }
    if (int rc = fq_project_id(dev, w0, x, x_elems, ids, routes, x_div, y0, routes * w0->expert_rows())) return rc;
    return fq_project_id(dev, w1, x, x_elems, ids, routes, x_div, y1, routes * w1->expert_rows());
}

extern "C" int fq_dense_ffn(fq_device *dev, const fq_matrix *gate, const fq_matrix *up, const fq_matrix *down,
                            const float *x, size_t m, float *scratch, size_t scratch_elems, float *out) {
    if (!dev || !gate || !up || !down) return fq_fail(dev, FQ_ERR_PARAM, "null matrix");
    const size_t width = gate->rows;
    if (up->rows != width || up->cols != gate->cols || down->cols != width)
        return fq_fail(dev, FQ_ERR_SHAPE, "feed-forward matrices do not chain");
    if (scratch_elems < 3 * m * width) return fq_fail(dev, FQ_ERR_SHAPE, "feed-forward scratch holds %zu of %zu floats", scratch_elems, 3 * m * width);
    float *g = scratch, *u = scratch + m * width, *act = scratch + 2 * m * width;
    const fq_matrix *pair[2] = {gate, up};
    void *outs[2] = {g, u};
    if (int rc = fq_project_many(dev, pair, 2, x, FQ_F32, m * gate->cols, m, outs, FQ_F32)) return rc;
    return project_gated(dev, down, g, u, act, m, nullptr, out);
}

// Expert routes at or below which experts use per-route GEMVs (`MV_ID_MAX_ROUTES`,
// src/hybrid/engine.rs:3586).
constexpr size_t MV_ID_MAX_ROUTES = 32;

static size_t align4(size_t n) { return (n + 3) & ~(size_t)3; }

struct MoeScratch {
    float *logits, *weights, *gate, *shared, *shared_tmp, *g, *u, *act, *down, *xg;
    uint32_t *ids, *offsets, *sorted, *position;
    size_t total;
};

static MoeScratch moe_layout(const fq_moe_ffn_desc *f, size_t m, float *base) {
    MoeScratch s{};
    const size_t routes = m * f->used;
    size_t at = 0;
    auto take = [&](size_t n) { float *p = base ? base + at : nullptr; at += align4(n); return p; };
    s.logits = take(m * f->experts);
    s.weights = take(routes);
    s.gate = take(m);
    s.shared = take(m * f->hidden);
    s.shared_tmp = take(3 * m * f->shared_ffn);
    s.g = take(routes * f->expert_ffn);
    s.u = take(routes * f->expert_ffn);
    s.act = take(routes * f->expert_ffn);
    s.down = take(routes * f->hidden);
    s.xg = take(routes * f->hidden);
    s.ids = (uint32_t *)take(routes);
    s.offsets = (uint32_t *)take(f->experts + 1);
    s.sorted = (uint32_t *)take(routes);
    s.position = (uint32_t *)take(routes);
    s.total = at;
    return s;
}

// Routed experts over expert-sorted rows, F32 throughout (the integer kernel or the fp16 tensor-core kernel, by
// rows per expert): gate and up as two targets of one launch that gathers the rows itself (row r of the sorted set
// is token sorted[r] / used), then the down projection whose activation preparation computes the gated unit.  `offsets[0 .. groups]` bound the rows of the experts the
// matrices hold.  FQ_ERR_UNSUPPORTED when the shapes have no such kernel (nothing is enqueued then).
static int moe_experts_f32(fq_device *dev, const fq_moe_ffn_desc *f, const float *x, const MoeScratch &s, const uint32_t *offsets, uint32_t groups,
                          size_t routes, float *down) {
    if (int rc = fq_begin_enqueue(dev)) return rc;
    ProjectArgs gu[2] = {base_args(f->gate_exps, x, FQ_F32, s.g, FQ_F32), base_args(f->up_exps, x, FQ_F32, s.u, FQ_F32)};
    for (ProjectArgs &p : gu) {
        p.offsets = offsets;
        p.groups = groups;
    }
    ProjectArgs dn = base_args(f->down_exps, s.g, FQ_F32, down, FQ_F32);
    dn.x_up = s.u;
    dn.offsets = offsets;
    dn.groups = groups;
    const size_t share = routes * groups / f->experts; // the rows these groups are expected to hold
    if (int rc = launch_grouped_f32(dev, gu, 2, (uint32_t)routes, share, s.sorted, f->used)) return rc;
    return launch_grouped_f32(dev, &dn, 1, (uint32_t)routes, share, nullptr, 1);
}

extern "C" size_t fq_moe_ffn_scratch_elems(const fq_moe_ffn_desc *f, size_t m) {
    return f ? moe_layout(f, m, nullptr).total : 0;
}

extern "C" int fq_moe_ffn(fq_device *dev, const fq_moe_ffn_desc *f, const float *x, size_t m, float *scratch,
                          size_t scratch_elems, float *out) {
    if (!dev || !f || !f->router || !f->gate_exps || !f->up_exps || !f->down_exps || !f->shared_gate || !f->shared_up ||
        !f->shared_down)
        return fq_fail(dev, FQ_ERR_PARAM, "incomplete MoE description");
    const size_t experts = f->experts, used = f->used, hidden = f->hidden, ef = f->expert_ffn;
    if (f->router->rows != experts || f->router->cols != hidden || f->gate_exps->experts != experts ||
        f->gate_exps->expert_rows() != ef || f->gate_exps->cols != hidden || f->up_exps->experts != experts ||
        f->up_exps->expert_rows() != ef || f->down_exps->experts != experts || f->down_exps->expert_rows() != hidden ||
        f->down_exps->cols != ef || f->shared_gate->rows != f->shared_ffn || f->shared_down->rows != hidden)
        return fq_fail(dev, FQ_ERR_SHAPE, "MoE matrices do not match the description");
    MoeScratch s = moe_layout(f, m, scratch);
    if (scratch_elems < s.total) return fq_fail(dev, FQ_ERR_SHAPE, "MoE scratch holds %zu of %zu floats", scratch_elems, s.total);
    const size_t routes = m * used;
    const bool identity = routes <= MV_ID_MAX_ROUTES || dev->exact;
    // The shared expert depends on x only and runs on the side stream beside the routed chain: at decode widths
    // (small kernels, latency-bound) from the start; at wide inputs after the router, whose GEMM shares the
    // split-K workspace with the shared expert's (the routing, map and grouped expert kernels use none of it).
    SideBranch side{dev, dev->stream, dev->xprep, dev->xprep_bytes, false};
    int rc = FQ_OK;
    auto shared_expert = [&]() {
        if (!dev->exact) side = side_begin(dev);
        const int r = fq_dense_ffn(dev, f->shared_gate, f->shared_up, f->shared_down, x, m, s.shared_tmp, 3 * m * f->shared_ffn, s.shared);
        const int r2 = side_detach(side);
        return r ? r : r2;
    };
    if (identity) rc = shared_expert();
    const float *shared_w = f->shared_gate_inp ? f->shared_gate_inp : x;
    if (!rc) rc = fq_project(dev, f->router, x, FQ_F32, m * hidden, m, s.logits, FQ_F32, m * experts);
    if (!identity) {
        const int r = shared_expert(); // also after an error: the branch must be detached exactly once
        rc = rc ? rc : r;
    }
    if (!rc)
        rc = fq_moe_route(dev, s.logits, x, shared_w, (uint32_t)experts, (uint32_t)used, (uint32_t)hidden, (uint32_t)m, f->sigmoid,
                          f->norm_weights, f->shared_gate_inp != nullptr, s.ids, s.weights, s.gate);
    bool combined = false;
    if (!rc && identity) {
        rc = project_id_pair(dev, f->gate_exps, f->up_exps, x, m * hidden, s.ids, routes, used, s.g, s.u);
        // The down projection also combines (the last of a token's route blocks to finish a row tile adds them up),
        // which takes the shared expert's output: the side stream joins before it instead of before the combine.
        CombineTail tail{s.weights, s.shared, s.gate, out, dev->combine_counters, (uint32_t)used};
        const bool fuse = !dev->exact && f->down_exps->expert_rows() == hidden;
        if (fuse) {
            if (int rc2 = side_join(side)) rc = rc ? rc : rc2;
            if (!rc) rc = fq_check_binding(dev, out, m * hidden * 4, "out");
        }
        if (!rc) rc = project_gated(dev, f->down_exps, s.g, s.u, s.act, routes, s.ids, s.down, fuse ? &tail : nullptr, &combined);
    } else if (!rc) {
        // Expert-sorted rows through the tensor-core GEMM: activations rounded to bf16 once (at the gather and
        // at the gated unit), fp32 accumulation and fp32 results.
        rc = fq_moe_map(dev, s.ids, (uint32_t)experts, (uint32_t)routes, s.offsets, s.sorted, s.position);
        int nt = FQ_ERR_UNSUPPORTED;
        if (!rc) nt = moe_experts_f32(dev, f, x, s, s.offsets, (uint32_t)experts, routes, s.down);
        if (nt != FQ_ERR_UNSUPPORTED) rc = rc ? rc : nt;
        else {
        if (!rc) rc = fq_launch_moe_gather_bf16(dev, x, s.sorted, (uint32_t)hidden, (uint32_t)used, (uint32_t)routes, nullptr, 0, s.xg);
        if (!rc) rc = fq_project_mm_id(dev, f->gate_exps, s.xg, FQ_BF16, routes * hidden, s.offsets, nullptr, experts, m, s.g, FQ_F32, routes * ef);
        if (!rc) rc = fq_project_mm_id(dev, f->up_exps, s.xg, FQ_BF16, routes * hidden, s.offsets, nullptr, experts, m, s.u, FQ_F32, routes * ef);
        if (!rc) rc = fq_launch_glu_bf16(dev, s.g, s.u, routes * ef, nullptr, 0, (uint32_t)ef, s.act);
        if (!rc) rc = fq_project_mm_id(dev, f->down_exps, s.act, FQ_BF16, routes * ef, s.offsets, nullptr, experts, m, s.down, FQ_F32, routes * hidden);
        }
    }
    if (int rc2 = side_join(side)) rc = rc ? rc : rc2; // also after an error: a capture must not end with the branch open
    if (rc || combined) return rc;
    return fq_moe_combine(dev, s.down, s.weights, identity ? s.ids : s.position, s.shared, s.gate, (uint32_t)hidden,
                          (uint32_t)used, (uint32_t)m, identity, out);
}


// Expert-parallel MoE block: this rank stores experts [expert_first, expert_first + local) of `f->experts`
// (the expert matrices of `f` hold only those), x and the router are replicated, every rank routes all tokens
// and maps them expert-major; it then computes the rows of its own experts (always in expert-sorted order, so
// that a rank's rows are one contiguous run), the runs are exchanged through the communicator's symmetric
// buffer, and every rank combines.  Per-row arithmetic is that of `fq_moe_ffn`, so the result has the same bits.
extern "C" int fq_moe_ffn_ep(fq_device *dev, fq_comm *comm, size_t region_offset, const fq_moe_ffn_desc *f, uint32_t expert_first,
                             const float *x, size_t m, float *scratch, size_t scratch_elems, float *out) {
    if (!dev || !comm || !f || !f->router || !f->gate_exps || !f->up_exps || !f->down_exps || !f->shared_gate || !f->shared_up ||
        !f->shared_down)
        return fq_fail(dev, FQ_ERR_PARAM, "incomplete MoE description");
    const size_t experts = f->experts, used = f->used, hidden = f->hidden, ef = f->expert_ffn, local = f->gate_exps->experts;
    const int world = fq_comm_world(comm), rank = fq_comm_rank(comm);
    if (f->router->rows != experts || f->router->cols != hidden || f->gate_exps->expert_rows() != ef || f->gate_exps->cols != hidden ||
        f->up_exps->experts != local || f->up_exps->expert_rows() != ef || f->down_exps->experts != local ||
        f->down_exps->expert_rows() != hidden || f->down_exps->cols != ef || f->shared_gate->rows != f->shared_ffn ||
        f->shared_down->rows != hidden || local * (size_t)world != experts || expert_first != (size_t)rank * local)
        return fq_fail(dev, FQ_ERR_SHAPE, "MoE matrices do not match the description or the expert split");
    MoeScratch s = moe_layout(f, m, scratch);
    if (scratch_elems < s.total) return fq_fail(dev, FQ_ERR_SHAPE, "MoE scratch holds %zu of %zu floats", scratch_elems, s.total);
    const size_t routes = m * used;
    const bool narrow = (routes <= MV_ID_MAX_ROUTES && !dev->exact);
    // Wide inputs combine every token on ONE rank (tokens are split evenly, `per_rank` to a rank, a multiple of 4),
    // so the symmetric buffer holds the expert rows and, after them, the combined outputs of all tokens.
    const bool owner_combine = world > 1 && !narrow && !dev->exact;
    const size_t per_rank = ((m + world - 1) / world + 3) / 4 * 4;
    const size_t rows_bytes = (routes * hidden * 4 + 255) / 256 * 256, out_bytes = owner_combine ? per_rank * world * hidden * 4 : 0;
    if (region_offset % 16 || region_offset + rows_bytes + out_bytes > fq_comm_bytes(comm))
        return fq_fail(dev, FQ_ERR_RANGE, "%zu expert rows of %zu floats (and %zu bytes of outputs) at offset %zu do not fit the symmetric buffer", routes,
                       hidden, out_bytes, region_offset);
    float *down = (float *)(fq_comm_local(comm) + region_offset);
    // As in fq_moe_ffn: the (replicated) shared expert runs on the side stream, from the start at decode widths
    // and after the router at wide inputs.
    SideBranch side{dev, dev->stream, dev->xprep, dev->xprep_bytes, false};
    int rc = FQ_OK;
    auto shared_expert = [&]() {
        if (!dev->exact) side = side_begin(dev);
        const int r = fq_dense_ffn(dev, f->shared_gate, f->shared_up, f->shared_down, x, m, s.shared_tmp, 3 * m * f->shared_ffn, s.shared);
        const int r2 = side_detach(side);
        return r ? r : r2;
    };
    if (narrow) rc = shared_expert();
    const float *shared_w = f->shared_gate_inp ? f->shared_gate_inp : x;
    if (!rc) rc = fq_project(dev, f->router, x, FQ_F32, m * hidden, m, s.logits, FQ_F32, m * experts);
    if (!narrow) {
        const int r = shared_expert();
        rc = rc ? rc : r;
    }
    if (!rc)
        rc = fq_moe_route_map(dev, s.logits, x, shared_w, (uint32_t)experts, (uint32_t)used, (uint32_t)hidden, (uint32_t)m, f->sigmoid,
                              f->norm_weights, f->shared_gate_inp != nullptr, s.ids, s.weights, s.gate, s.offsets, s.sorted, s.position);
    const uint32_t *mine = s.offsets + expert_first; // mine[0] .. mine[local]: this rank's run of rows
    if (!rc && (routes <= MV_ID_MAX_ROUTES || dev->exact)) {
        // The decode kernel reads the map itself: sorted row r is route sorted[r] (token sorted[r] / used, expert
        // ids[sorted[r]] - expert_first), and rows of other ranks' experts are skipped.  Where it does not serve the
        // shapes: gather the rows and translate the ids first.
        int fast = project_id_pair(dev, f->gate_exps, f->up_exps, x, m * hidden, s.ids, routes, used, s.g, s.u, s.sorted, expert_first);
        if (fast == FQ_OK) {
            fast = project_gated(dev, f->down_exps, s.g, s.u, s.act, routes, s.ids, down, nullptr, nullptr, s.sorted, expert_first);
            if (fast != FQ_ERR_UNSUPPORTED) rc = fast;
        } else if (fast != FQ_ERR_UNSUPPORTED) {
            rc = fast;
        }
        if (fast == FQ_ERR_UNSUPPORTED) {
            uint32_t *local_ids = (uint32_t *)s.logits; // the logits are consumed by now, and routes <= m * experts
            rc = fq_moe_gather(dev, x, s.sorted, (uint32_t)hidden, (uint32_t)used, (uint32_t)routes, s.xg);
            if (!rc) rc = fq_launch_moe_local_ids(dev, s.ids, s.sorted, (uint32_t)routes, expert_first, (uint32_t)local, local_ids);
            if (!rc) rc = project_id_pair(dev, f->gate_exps, f->up_exps, s.xg, routes * hidden, local_ids, routes, 1, s.g, s.u);
            if (!rc) rc = project_gated(dev, f->down_exps, s.g, s.u, s.act, routes, local_ids, down);
        }
    } else if (!rc && (rc = moe_experts_f32(dev, f, x, s, mine, (uint32_t)local, routes, down)) != FQ_ERR_UNSUPPORTED) {
        // done (or failed) on the integer or the fp16 kernel
    } else if (!rc || rc == FQ_ERR_UNSUPPORTED) {
        rc = fq_launch_moe_gather_bf16(dev, x, s.sorted, (uint32_t)hidden, (uint32_t)used, (uint32_t)routes, mine, (uint32_t)local, s.xg);
        if (!rc) rc = fq_project_mm_id(dev, f->gate_exps, s.xg, FQ_BF16, routes * hidden, mine, nullptr, local, m, s.g, FQ_F32, routes * ef);
        if (!rc) rc = fq_project_mm_id(dev, f->up_exps, s.xg, FQ_BF16, routes * hidden, mine, nullptr, local, m, s.u, FQ_F32, routes * ef);
        if (!rc) rc = fq_launch_glu_bf16(dev, s.g, s.u, routes * ef, mine, (uint32_t)local, (uint32_t)ef, s.act);
        if (!rc) rc = fq_project_mm_id(dev, f->down_exps, s.act, FQ_BF16, routes * ef, mine, nullptr, local, m, down, FQ_F32, routes * hidden);
    }
    if (int rc2 = side_join(side)) rc = rc ? rc : rc2; // also after an error: a capture must not end with the branch open
    if (rc) return rc;
    if (owner_combine) {
        // All-to-all, dispatch half: a row goes only to the rank that combines its token.  That rank then has all
        // `used` rows of each of its tokens and combines them in the usual order; the outputs are gathered.
        if (int rc = fq_comm_dispatch_rows(dev, comm, region_offset, hidden * 4, s.offsets, (uint32_t)local, s.sorted, (uint32_t)used,
                                           (uint32_t)per_rank, routes))
            return rc;
        float *outs = (float *)(fq_comm_local(comm) + region_offset + rows_bytes);
        const size_t token0 = (size_t)rank * per_rank, mine_count = token0 < m ? std::min(per_rank, m - token0) : 0;
        if (int rc = fq_launch_moe_combine_range(dev, down, s.weights, s.position, s.shared, s.gate, (uint32_t)hidden, (uint32_t)used, (uint32_t)token0,
                                                 (uint32_t)mine_count, outs))
            return rc;
        if (int rc = fq_comm_all_gather(dev, comm, region_offset + rows_bytes, per_rank * hidden * 4)) return rc;
        if (int rc = fq_begin_enqueue(dev)) return rc;
        return fq_check_cuda(dev, cudaMemcpyAsync(out, outs, m * hidden * 4, cudaMemcpyDeviceToDevice, dev->stream), "output copy");
    }
    if (int rc = fq_comm_all_gather_rows(dev, comm, region_offset, hidden * 4, s.offsets, (uint32_t)local, routes)) return rc;
    return fq_moe_combine(dev, down, s.weights, s.position, s.shared, s.gate, (uint32_t)hidden, (uint32_t)used, (uint32_t)m, 0, out);
}

// ------------------------------------------------------------------ host-buffer entry points

extern "C" int fq_project_many_host(fq_device *dev, const fq_matrix *const *w, size_t count, const float *x_host,
                                    size_t m, float *const *y_host) {
    if (!dev || !w || !x_host || !y_host || count == 0 || m == 0) return fq_fail(dev, FQ_ERR_PARAM, "host projection arguments");
    const size_t cols = w[0]->cols;
    size_t need = align4(m * cols) * 4;
    for (size_t i = 0; i < count; i++) {
        if (!w[i] || w[i]->cols != cols) return fq_fail(dev, FQ_ERR_SHAPE, "matrices sharing an input differ in width");
        need += align4(m * w[i]->rows) * 4;
    }
    if (need > FQ_HOST_STAGING_BYTES) return fq_fail(dev, FQ_ERR_SHAPE, "%zu bytes exceed the %u-byte staging area", need, FQ_HOST_STAGING_BYTES);
    if (int rc = fq_begin_enqueue(dev)) return rc;
    float *xd = (float *)dev->staging_dev;
    // Pageable caller memory is staged through the pinned area so the copies are asynchronous.
    memcpy(dev->staging_host, x_host, m * cols * 4);
    if (int rc = fq_check_cuda(dev, cudaMemcpyAsync(xd, dev->staging_host, m * cols * 4, cudaMemcpyHostToDevice, dev->stream), "x upload")) return rc;
    dev->counters.bytes_uploaded += m * cols * 4;
    size_t at = align4(m * cols);
    std::vector<size_t> where(count);
    std::vector<void *> outs(count);
    for (size_t i = 0; i < count; i++) {
        outs[i] = (float *)dev->staging_dev + at;
        where[i] = at;
        at += align4(m * w[i]->rows);
    }
    if (count <= 8) {
        if (int rc = fq_project_many(dev, w, count, xd, FQ_F32, m * cols, m, outs.data(), FQ_F32)) return rc;
    } else {
        for (size_t i = 0; i < count; i++)
            if (int rc = fq_project(dev, w[i], xd, FQ_F32, m * cols, m, outs[i], FQ_F32, m * w[i]->rows)) return rc;
    }
    const size_t first = align4(m * cols);
    if (int rc = fq_check_cuda(dev, cudaMemcpyAsync((float *)dev->staging_host + first, (float *)dev->staging_dev + first,
                                                    (at - first) * 4, cudaMemcpyDeviceToHost, dev->stream), "y download")) return rc;
    dev->counters.bytes_downloaded += (at - first) * 4;
    if (int rc = fq_synchronize(dev)) return rc;
    for (size_t i = 0; i < count; i++) memcpy(y_host[i], (float *)dev->staging_host + where[i], m * w[i]->rows * 4);
    return FQ_OK;
}

extern "C" int fq_project_host(fq_device *dev, const fq_matrix *w, const float *x_host, size_t m, float *y_host) {
    const fq_matrix *ws[1] = {w};
    float *ys[1] = {y_host};
    return fq_project_many_host(dev, ws, 1, x_host, m, ys);
}
