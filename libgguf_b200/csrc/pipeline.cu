// Multi-GPU streaming conversion pipeline: the tensor loop of the converter.
//
// upstream's converter (csrc/quantize_gguf.cpp:1990-2223 with cuda_converter_context, :1732-1931)
// walks the tensor plan on one GPU with two pinned host slots and one stream: read rows into a
// pinned slot, h2d, quantize, d2h, write.  Here the same loop is a pool of per-GPU workers:
//   * every tensor of a batch is cut into shards of whole rows (at most `chunk_bytes` of source bytes; a 16-bit
//     source is uploaded as it is and widened on the GPU; F32 / F16 / BF16 targets are converted there too),
//   * shards go into one queue, largest first; each GPU's worker thread pulls the next shard when
//     one of its slots frees up, so load balances itself and no GPU waits for another,
//   * a worker owns `slots` independent streams, each with its own device input/output buffers
//     and pinned staging; a slot runs h2d -> quantize -> d2h in stream order, and consecutive
//     shards go to different slots so copies in both directions overlap the kernels,
//   * host memory that is already pinned (cudaHostAlloc / cudaHostRegister) is copied from and
//     to directly; pageable memory goes through the slot's pinned staging,
//   * a type that needs importance weights and got none gets them from a first pass over the tensor (column sums
//     of squares in row order) on the first GPU,
//   * there is no device-to-device traffic and no collective: a shard's bytes only ever cross
//     its own GPU's PCIe link.  Results land at their row offset in the caller's output.
// Host waits are cudaEventQuery polls with a deadline; a worker that sees an error (or an
// injected one, for tests) puts its shard back, retires, and the remaining GPUs finish the batch.
#include <algorithm>
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "../../include/libgguf.h"
#include "../../include/libgguf_cuda_native.h"
#include "device_state.h"
#include "gguf_common.cuh"
#include "kernels.h"

using namespace gguf;

namespace {

struct Shard {
    int tensor = 0;
    int64_t row0 = 0;
    int64_t rows = 0;
    size_t in_bytes = 0;
    size_t out_bytes = 0;
};

struct Slot {
    cudaStream_t stream = nullptr;
    cudaEvent_t done = nullptr;
    void *d_in = nullptr, *d_out = nullptr, *d_imatrix = nullptr, *d_wide = nullptr;  // d_wide: fp32 copy of a 16-bit source shard
    void *h_in = nullptr, *h_out = nullptr;
    size_t d_in_cap = 0, d_out_cap = 0, d_im_cap = 0, d_wide_cap = 0, h_in_cap = 0, h_out_cap = 0;
    bool busy = false;
    Shard shard;
    void *copy_out_to = nullptr;  // pageable destination waiting for the staged result
};

bool is_pinned(const void *p) {
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) { cudaGetLastError(); return false; }
    return attr.type == cudaMemoryTypeHost;
}

}  // namespace

struct libgguf_cuda_pipeline {
    std::vector<int> devices;
    int slots = 3;
    size_t chunk_bytes = size_t(128) << 20;
    int wait_timeout_ms = 60000;
    std::string last_error;
    // failure injection (host side only): device index -> fail when it has completed this many shards
    std::vector<int64_t> fail_after;
    // statistics of the last batch
    std::vector<int64_t> shards_done;
    std::vector<double> busy_seconds;
    int64_t requeued = 0;
    // per worker: its slots (streams, events, device and pinned buffers), created on first use and kept
    // until the pipeline is destroyed so that consecutive batches pay no allocation or stream set-up
    std::vector<std::vector<Slot>> worker_slots;
};

namespace {

// F32 / F16 / BF16 as the target: plain storage conversion of the rows (upstream libgguf_storage.cpp:105-125)
bool is_storage_type(int64_t qtype) { return qtype == GGML_TYPE_F32 || qtype == GGML_TYPE_F16 || qtype == GGML_TYPE_BF16; }

size_t source_elem_size(const int32_t *dtypes, int i) { return dtypes && dtypes[i] != LIBGGUF_CUDA_DEQUANTIZE_DTYPE_F32 ? 2 : 4; }

std::vector<Shard> plan_shards(const libgguf_cuda_tensor_desc *t, const int32_t *dtypes, int n, size_t chunk_bytes) {
    std::vector<Shard> shards;
    for (int i = 0; i < n; ++i) {
        const size_t in_row = (size_t)t[i].n_per_row * source_elem_size(dtypes, i);
        const size_t out_row = libgguf_row_size((enum ggml_type)t[i].qtype, t[i].n_per_row);
        int64_t rows_per = (int64_t)(chunk_bytes / in_row);
        if (rows_per < 1) rows_per = 1;
        for (int64_t r = 0; r < t[i].rows; r += rows_per) {
            Shard s;
            s.tensor = i;
            s.row0 = r;
            s.rows = std::min<int64_t>(rows_per, t[i].rows - r);
            s.in_bytes = (size_t)s.rows * in_row;
            s.out_bytes = (size_t)s.rows * out_row;
            shards.push_back(s);
        }
    }
    // largest first: the classic longest-processing-time order for a greedy pull queue
    std::stable_sort(shards.begin(), shards.end(), [](const Shard &a, const Shard &b) { return a.in_bytes > b.in_bytes; });
    return shards;
}

struct Batch {
    const libgguf_cuda_tensor_desc *tensors;
    const int32_t *dtypes = nullptr;
    std::vector<char> src_pinned, dst_pinned;
    std::mutex lock;
    std::deque<Shard> queue;
    std::atomic<int> live_workers{0};
    std::atomic<int64_t> remaining{0};
    std::string error;
    bool failed = false;
    std::vector<char> worker_failed;
    bool any_bulk_staged = false;  // some tensor's quantizer stages its input with bulk copies (see kernels.h)
};

bool grow_dev(void **p, size_t *cap, size_t need) {
    if (need <= *cap) return true;
    if (*p) cudaFree(*p);
    *p = nullptr; *cap = 0;
    if (cudaMalloc(p, need ? need : 16) != cudaSuccess) { cudaGetLastError(); return false; }
    *cap = need;
    return true;
}
bool grow_host(void **p, size_t *cap, size_t need) {
    if (need <= *cap) return true;
    if (*p) cudaFreeHost(*p);
    *p = nullptr; *cap = 0;
    if (cudaMallocHost(p, need ? need : 16) != cudaSuccess) { cudaGetLastError(); return false; }
    *cap = need;
    return true;
}

// Waits for the slot's event with a deadline; false on timeout or CUDA error.
bool wait_slot(Slot &s, int timeout_ms, std::string &err) {
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
    for (;;) {
        const cudaError_t q = cudaEventQuery(s.done);
        if (q == cudaSuccess) return true;
        if (q != cudaErrorNotReady) { err = cudaGetErrorString(q); cudaGetLastError(); return false; }
        if (std::chrono::steady_clock::now() > deadline) { err = "timed out waiting for a pipeline slot"; return false; }
        std::this_thread::yield();
    }
}

// Streams one tensor through GPU `dev` in row pieces and accumulates its column sums of squares in order.
bool auto_imatrix_pass(int dev, size_t chunk_bytes, const libgguf_cuda_tensor_desc &t, int dtype, float *out, std::string &err) {
    if (cudaSetDevice(dev) != cudaSuccess) { cudaGetLastError(); err = "cannot select device " + std::to_string(dev); return false; }
    const size_t esz = dtype != LIBGGUF_CUDA_DEQUANTIZE_DTYPE_F32 ? 2 : 4;
    const size_t row_bytes = (size_t)t.n_per_row * esz;
    int64_t piece = (int64_t)(chunk_bytes / row_bytes);
    if (piece < 1) piece = 1;
    cudaStream_t stream = nullptr;
    void *d_src[2] = {nullptr, nullptr}, *d_wide = nullptr, *h_stage[2] = {nullptr, nullptr};
    float *d_acc = nullptr;
    cudaEvent_t done[2] = {nullptr, nullptr};
    const bool pinned = is_pinned(t.src);
    bool ok = cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking) == cudaSuccess &&
              cudaMalloc((void **)&d_acc, (size_t)t.n_per_row * 4) == cudaSuccess &&
              cudaMemsetAsync(d_acc, 0, (size_t)t.n_per_row * 4, stream) == cudaSuccess;
    for (int k = 0; k < 2 && ok; ++k) {
        ok = cudaMalloc(&d_src[k], (size_t)piece * row_bytes) == cudaSuccess &&
             cudaEventCreateWithFlags(&done[k], cudaEventDisableTiming) == cudaSuccess &&
             (pinned || cudaMallocHost(&h_stage[k], (size_t)piece * row_bytes) == cudaSuccess);
    }
    if (ok && esz == 2) ok = cudaMalloc(&d_wide, (size_t)piece * t.n_per_row * 4) == cudaSuccess;
    int k = 0;
    bool used[2] = {false, false};
    for (int64_t r = 0; r < t.rows && ok; r += piece, k ^= 1) {
        const int64_t nr = std::min<int64_t>(piece, t.rows - r);
        if (used[k]) ok = cudaEventSynchronize(done[k]) == cudaSuccess;  // the piece that used this buffer has been consumed
        if (!ok) break;
        const char *src = (const char *)t.src + (size_t)r * row_bytes;
        if (!pinned) { std::memcpy(h_stage[k], src, (size_t)nr * row_bytes); src = (const char *)h_stage[k]; }
        ok = cudaMemcpyAsync(d_src[k], src, (size_t)nr * row_bytes, cudaMemcpyHostToDevice, stream) == cudaSuccess;
        const float *rows32 = (const float *)d_src[k];
        if (ok && esz == 2) {
            ok = launch_widen(dtype, d_src[k], (float *)d_wide, nr * t.n_per_row, stream) == cudaSuccess;
            rows32 = (const float *)d_wide;
        }
        if (ok) ok = launch_sumsq_columns(rows32, nr, t.n_per_row, d_acc, stream) == cudaSuccess;
        if (ok) ok = cudaEventRecord(done[k], stream) == cudaSuccess;
        used[k] = true;
    }
    if (ok) ok = cudaMemcpyAsync(out, d_acc, (size_t)t.n_per_row * 4, cudaMemcpyDeviceToHost, stream) == cudaSuccess;
    if (ok) ok = cudaStreamSynchronize(stream) == cudaSuccess;
    if (!ok) { err = std::string("imatrix pass failed: ") + cudaGetErrorString(cudaGetLastError()); }
    else cudaGetLastError();
    if (stream) cudaStreamSynchronize(stream);
    for (int j = 0; j < 2; ++j) {
        if (done[j]) cudaEventDestroy(done[j]);
        cudaFree(d_src[j]);
        if (h_stage[j]) cudaFreeHost(h_stage[j]);
    }
    cudaFree(d_wide);
    cudaFree(d_acc);
    if (stream) cudaStreamDestroy(stream);
    return ok;
}

void worker(libgguf_cuda_pipeline *pipe, Batch *batch, int widx) {
    const int dev = pipe->devices[widx];
    std::vector<Slot> &slots = pipe->worker_slots[widx];
    std::string err;
    bool ok = cudaSetDevice(dev) == cudaSuccess;
    if (ok && slots.empty()) {
        slots.resize(pipe->slots);
        for (Slot &s : slots) {
            if (!ok) break;
            ok = cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking) == cudaSuccess &&
                 cudaEventCreateWithFlags(&s.done, cudaEventDisableTiming) == cudaSuccess;
        }
    }
    if (!ok) err = "failed to set up streams on device " + std::to_string(dev);
    const auto t_begin = std::chrono::steady_clock::now();
    // the device's count of staged copies that never arrived, as it stood before this worker's first shard
    unsigned long long timeouts_before = 0;
    if (ok && batch->any_bulk_staged && read_staging_timeouts(&timeouts_before) != cudaSuccess) {
        cudaGetLastError();
        ok = false;
        err = "cannot read the staging counter of device " + std::to_string(dev);
    }

    auto finish = [&](Slot &s) -> bool {
        if (!s.busy) return true;
        if (!wait_slot(s, pipe->wait_timeout_ms, err)) return false;
        if (uses_bulk_staging((int)batch->tensors[s.shard.tensor].qtype)) {
            // a CTA that gave up on a staged copy returned without writing its rows: the shard has to be redone
            unsigned long long now = 0;
            if (read_staging_timeouts(&now) != cudaSuccess || now != timeouts_before) {
                cudaGetLastError();
                err = "a staged copy did not arrive within its wait limit on device " + std::to_string(dev) +
                      " (libgguf_cuda_staging_timeouts); the shard's output is incomplete";
                return false;
            }
        }
        if (s.copy_out_to) std::memcpy(s.copy_out_to, s.h_out, s.shard.out_bytes);
        s.busy = false;
        s.copy_out_to = nullptr;
        pipe->shards_done[widx]++;
        batch->remaining.fetch_sub(1);
        return true;
    };

    int next = 0;
    Shard cur;
    bool have_cur = false;
    while (ok) {
        {
            std::lock_guard<std::mutex> g(batch->lock);
            if (batch->failed || batch->queue.empty()) break;
            cur = batch->queue.front();
            batch->queue.pop_front();
            have_cur = true;
        }
        if (pipe->fail_after[widx] >= 0 && pipe->shards_done[widx] >= pipe->fail_after[widx]) {
            err = "injected failure on device " + std::to_string(dev);
            ok = false;
            break;
        }
        Slot &s = slots[next];
        next = (next + 1) % pipe->slots;
        if (!finish(s)) { ok = false; break; }
        const libgguf_cuda_tensor_desc &t = batch->tensors[cur.tensor];
        const size_t out_row = libgguf_row_size((enum ggml_type)t.qtype, t.n_per_row);
        const size_t esz = source_elem_size(batch->dtypes, cur.tensor);
        const char *src = (const char *)t.src + (size_t)cur.row0 * t.n_per_row * esz;
        char *dst = (char *)t.dst + (size_t)cur.row0 * out_row;
        const bool storage = is_storage_type(t.qtype);
        const DeviceState *state = storage ? nullptr : device_state_for((int)t.qtype, dev);
        ok = (storage || state) && grow_dev(&s.d_in, &s.d_in_cap, cur.in_bytes) && grow_dev(&s.d_out, &s.d_out_cap, cur.out_bytes);
        if (!ok) { err = "device allocation failed on device " + std::to_string(dev); break; }
        const void *h2d_from = src;
        if (!batch->src_pinned[cur.tensor]) {
            if (!grow_host(&s.h_in, &s.h_in_cap, cur.in_bytes)) { ok = false; err = "pinned allocation failed"; break; }
            std::memcpy(s.h_in, src, cur.in_bytes);
            h2d_from = s.h_in;
        }
        void *d2h_to = dst;
        if (!batch->dst_pinned[cur.tensor]) {
            if (!grow_host(&s.h_out, &s.h_out_cap, cur.out_bytes)) { ok = false; err = "pinned allocation failed"; break; }
            d2h_to = s.h_out;
            s.copy_out_to = dst;
        }
        const float *d_im = nullptr;
        cudaError_t e = cudaSuccess;
        if (t.imatrix) {
            ok = grow_dev(&s.d_imatrix, &s.d_im_cap, (size_t)t.n_per_row * 4);
            if (!ok) { err = "device allocation failed"; break; }
            e = cudaMemcpyAsync(s.d_imatrix, t.imatrix, (size_t)t.n_per_row * 4, cudaMemcpyHostToDevice, s.stream);
            d_im = (const float *)s.d_imatrix;
        }
        if (e == cudaSuccess) e = cudaMemcpyAsync(s.d_in, h2d_from, cur.in_bytes, cudaMemcpyHostToDevice, s.stream);
        const float *d_f32 = (const float *)s.d_in;
        if (esz == 2) {
            if (!grow_dev(&s.d_wide, &s.d_wide_cap, cur.in_bytes * 2)) { ok = false; err = "device allocation failed"; break; }
            if (e == cudaSuccess) e = launch_widen(batch->dtypes[cur.tensor], s.d_in, (float *)s.d_wide, cur.rows * t.n_per_row, s.stream);
            d_f32 = (const float *)s.d_wide;
        }
        if (e == cudaSuccess)
            e = storage ? launch_store((int)t.qtype, d_f32, s.d_out, cur.rows * t.n_per_row, s.stream)
                        : launch_quantize((int)t.qtype, d_f32, d_im, s.d_out, cur.rows, t.n_per_row, state, s.stream);
        if (e == cudaSuccess) e = cudaMemcpyAsync(d2h_to, s.d_out, cur.out_bytes, cudaMemcpyDeviceToHost, s.stream);
        if (e == cudaSuccess) e = cudaEventRecord(s.done, s.stream);
        if (e != cudaSuccess) { err = cudaGetErrorString(e); cudaGetLastError(); ok = false; break; }
        s.busy = true;
        s.shard = cur;
        have_cur = false;
    }
    // drain what is in flight; on failure give unfinished shards back to the queue
    for (Slot &s : slots) {
        if (ok) { if (!finish(s)) ok = false; }
    }
    if (!ok) {
        std::lock_guard<std::mutex> g(batch->lock);
        if (have_cur) { batch->queue.push_front(cur); pipe->requeued++; }
        for (Slot &s : slots) {
            if (s.busy) {
                // the slot may or may not have completed: redo the shard elsewhere (results are deterministic)
                cudaStreamSynchronize(s.stream);
                cudaGetLastError();
                batch->queue.push_front(s.shard);
                pipe->requeued++;
                s.busy = false;
            }
        }
        if (batch->error.empty()) batch->error = err;
        batch->worker_failed[widx] = 1;
    }
    for (Slot &s : slots) {
        if (s.stream) cudaStreamSynchronize(s.stream);
        s.busy = false;
        s.copy_out_to = nullptr;
    }
    cudaGetLastError();
    pipe->busy_seconds[widx] = std::chrono::duration<double>(std::chrono::steady_clock::now() - t_begin).count();
    batch->live_workers.fetch_sub(1);
}

}  // namespace

extern "C" {

int libgguf_cuda_pipeline_create(const int *devices, int n_devices, int slots, size_t chunk_bytes, libgguf_cuda_pipeline **out) {
    if (!out || n_devices <= 0 || !devices) return LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT;
    *out = nullptr;
    libgguf_cuda_pipeline *p = new (std::nothrow) libgguf_cuda_pipeline();
    if (!p) return LIBGGUF_CUDA_STATUS_ALLOCATION_FAILED;
    p->devices.assign(devices, devices + n_devices);
    if (slots > 0) p->slots = slots;
    if (chunk_bytes > 0) p->chunk_bytes = chunk_bytes;
    p->fail_after.assign(n_devices, -1);
    p->shards_done.assign(n_devices, 0);
    p->busy_seconds.assign(n_devices, 0.0);
    p->worker_slots.resize(n_devices);
    *out = p;
    return LIBGGUF_CUDA_STATUS_SUCCESS;
}

void libgguf_cuda_pipeline_destroy(libgguf_cuda_pipeline *pipe) {
    if (!pipe) return;
    for (size_t w = 0; w < pipe->worker_slots.size(); ++w) {
        if (pipe->worker_slots[w].empty() || cudaSetDevice(pipe->devices[w]) != cudaSuccess) continue;
        for (Slot &s : pipe->worker_slots[w]) {
            if (s.stream) { cudaStreamSynchronize(s.stream); cudaStreamDestroy(s.stream); }
            if (s.done) cudaEventDestroy(s.done);
            cudaFree(s.d_in); cudaFree(s.d_out); cudaFree(s.d_imatrix); cudaFree(s.d_wide);
            cudaFreeHost(s.h_in); cudaFreeHost(s.h_out);
        }
    }
    cudaGetLastError();
    delete pipe;
}

const char *libgguf_cuda_pipeline_last_error(const libgguf_cuda_pipeline *pipe) {
    return pipe ? pipe->last_error.c_str() : "libgguf CUDA pipeline is null";
}

int libgguf_cuda_pipeline_inject_failure(libgguf_cuda_pipeline *pipe, int device_slot, int64_t after_shards) {
    if (!pipe || device_slot < 0 || device_slot >= (int)pipe->devices.size()) return LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT;
    pipe->fail_after[device_slot] = after_shards;
    return LIBGGUF_CUDA_STATUS_SUCCESS;
}

int64_t libgguf_cuda_pipeline_plan(const libgguf_cuda_tensor_desc *tensors, int n_tensors, size_t chunk_bytes,
                                   libgguf_cuda_shard *out, int64_t max_out) {
    return libgguf_cuda_pipeline_plan_typed(tensors, nullptr, n_tensors, chunk_bytes, out, max_out);
}

static bool source_dtypes_valid(const int32_t *dtypes, int n) {
    for (int i = 0; dtypes && i < n; ++i)
        if (dtypes[i] != LIBGGUF_CUDA_DEQUANTIZE_DTYPE_F32 && dtypes[i] != LIBGGUF_CUDA_DEQUANTIZE_DTYPE_F16 &&
            dtypes[i] != LIBGGUF_CUDA_DEQUANTIZE_DTYPE_BF16) return false;
    return true;
}

int64_t libgguf_cuda_pipeline_plan_typed(const libgguf_cuda_tensor_desc *tensors, const int32_t *source_dtypes, int n_tensors,
                                         size_t chunk_bytes, libgguf_cuda_shard *out, int64_t max_out) {
    if (!tensors || n_tensors < 0 || !source_dtypes_valid(source_dtypes, n_tensors)) return -1;
    for (int i = 0; i < n_tensors; ++i)
        if (tensors[i].rows < 0 || tensors[i].n_per_row <= 0 || libgguf_row_size((enum ggml_type)tensors[i].qtype, tensors[i].n_per_row) == 0) return -1;
    const std::vector<Shard> shards = plan_shards(tensors, source_dtypes, n_tensors, chunk_bytes ? chunk_bytes : (size_t(128) << 20));
    for (int64_t i = 0; i < (int64_t)shards.size() && out && i < max_out; ++i) {
        out[i].tensor = shards[i].tensor;
        out[i].row0 = shards[i].row0;
        out[i].rows = shards[i].rows;
    }
    return (int64_t)shards.size();
}

int libgguf_cuda_pipeline_quantize(libgguf_cuda_pipeline *pipe, const libgguf_cuda_tensor_desc *tensors, int n_tensors) {
    return libgguf_cuda_pipeline_quantize_typed(pipe, tensors, nullptr, n_tensors);
}

int libgguf_cuda_pipeline_quantize_typed(libgguf_cuda_pipeline *pipe, const libgguf_cuda_tensor_desc *tensors,
                                         const int32_t *source_dtypes, int n_tensors) {
    if (!pipe || !tensors || n_tensors < 0) return LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT;
    pipe->last_error.clear();
    if (!source_dtypes_valid(source_dtypes, n_tensors)) {
        pipe->last_error = "source dtype must be F32 (0), F16 (1) or BF16 (2)";
        return LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT;
    }
    for (int i = 0; i < n_tensors; ++i) {
        const libgguf_cuda_tensor_desc &t = tensors[i];
        if (!t.src || !t.dst || t.rows < 0 || t.n_per_row <= 0) {
            pipe->last_error = "invalid tensor descriptor";
            return LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT;
        }
        if (t.qtype < 0 || t.qtype >= GGML_TYPE_COUNT || !(quantize_supported((int)t.qtype) || is_storage_type(t.qtype)) ||
            libgguf_row_size((enum ggml_type)t.qtype, t.n_per_row) == 0) {
            pipe->last_error = "unsupported quantization type or row width";
            return LIBGGUF_CUDA_STATUS_UNSUPPORTED_TYPE;
        }
    }
    // Types that require importance weights and got none: derive them from the tensor itself (column sums of
    // squares in row order, upstream _libgguf_module.cpp:1221-1242) in a first pass over that tensor on the
    // first GPU, then quantize with them like with caller-supplied weights.
    std::vector<libgguf_cuda_tensor_desc> with_auto;
    std::vector<std::vector<float>> auto_weights;
    for (int i = 0; i < n_tensors; ++i) {
        if (!libgguf_quantize_requires_imatrix((enum ggml_type)tensors[i].qtype) || tensors[i].imatrix) continue;
        if (with_auto.empty()) {
            with_auto.assign(tensors, tensors + n_tensors);
            auto_weights.resize(n_tensors);
        }
        auto_weights[i].assign((size_t)tensors[i].n_per_row, 0.f);
        std::string err;
        if (!auto_imatrix_pass(pipe->devices[0], pipe->chunk_bytes, tensors[i], source_dtypes ? source_dtypes[i] : 0, auto_weights[i].data(), err)) {
            pipe->last_error = err;
            return LIBGGUF_CUDA_STATUS_CUDA_ERROR;
        }
        with_auto[i].imatrix = auto_weights[i].data();
    }
    if (!with_auto.empty()) tensors = with_auto.data();
    Batch batch;
    batch.tensors = tensors;
    batch.dtypes = source_dtypes;
    batch.src_pinned.resize(n_tensors);
    batch.dst_pinned.resize(n_tensors);
    for (int i = 0; i < n_tensors; ++i) {
        batch.any_bulk_staged = batch.any_bulk_staged || uses_bulk_staging((int)tensors[i].qtype);
        batch.src_pinned[i] = is_pinned(tensors[i].src);
        batch.dst_pinned[i] = is_pinned(tensors[i].dst);
    }
    const std::vector<Shard> shards = plan_shards(tensors, source_dtypes, n_tensors, pipe->chunk_bytes);
    batch.queue.assign(shards.begin(), shards.end());
    batch.remaining = (int64_t)shards.size();
    batch.worker_failed.assign(pipe->devices.size(), 0);
    std::fill(pipe->shards_done.begin(), pipe->shards_done.end(), 0);
    pipe->requeued = 0;
    const int n = (int)pipe->devices.size();
    // Workers that fail retire; the survivors keep pulling until the queue is empty.  A second
    // round picks up shards that a failing worker handed back after the survivors had finished.
    std::vector<char> retired(n, 0);
    for (int round = 0; round < n && batch.remaining.load() > 0; ++round) {
        std::vector<std::thread> threads;
        batch.error.clear();
        batch.live_workers = 0;
        for (int w = 0; w < n; ++w) {
            if (retired[w]) continue;
            batch.live_workers.fetch_add(1);
            threads.emplace_back(worker, pipe, &batch, w);
        }
        if (threads.empty()) break;
        for (std::thread &t : threads) t.join();
        if (batch.remaining.load() > 0) {
            // somebody failed and handed shards back: retire the failed workers, let the others retry
            bool any = false;
            for (int w = 0; w < n; ++w) {
                if (!retired[w] && batch.worker_failed[w]) { retired[w] = 1; any = true; }
            }
            if (!any) break;
        }
    }
    if (batch.remaining.load() > 0) {
        pipe->last_error = batch.error.empty() ? "pipeline did not finish" : batch.error;
        return LIBGGUF_CUDA_STATUS_CUDA_ERROR;
    }
    return LIBGGUF_CUDA_STATUS_SUCCESS;
}

int libgguf_cuda_auto_imatrix_typed(const void *host_rows, int source_dtype, int64_t rows, int64_t n_per_row, float *host_imatrix) {
    if (rows < 0 || n_per_row <= 0 || !host_imatrix || (rows > 0 && !host_rows) || !source_dtypes_valid(&source_dtype, 1))
        return LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT;
    int dev = 0;
    const char *env = getenv("LIBGGUF_CUDA_DEVICE");
    if (env && env[0]) dev = atoi(env);
    else if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return LIBGGUF_CUDA_STATUS_CUDA_ERROR; }
    libgguf_cuda_tensor_desc t = {};
    t.src = (const float *)host_rows;
    t.rows = rows;
    t.n_per_row = n_per_row;
    std::string err;
    return auto_imatrix_pass(dev, size_t(64) << 20, t, source_dtype, host_imatrix, err) ? LIBGGUF_CUDA_STATUS_SUCCESS
                                                                                       : LIBGGUF_CUDA_STATUS_CUDA_ERROR;
}

int libgguf_cuda_pipeline_stats(const libgguf_cuda_pipeline *pipe, int64_t *shards_per_device, double *seconds_per_device,
                                int64_t *requeued) {
    if (!pipe) return LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT;
    for (size_t i = 0; i < pipe->devices.size(); ++i) {
        if (shards_per_device) shards_per_device[i] = pipe->shards_done[i];
        if (seconds_per_device) seconds_per_device[i] = pipe->busy_seconds[i];
    }
    if (requeued) *requeued = pipe->requeued;
    return LIBGGUF_CUDA_STATUS_SUCCESS;
}

}  // extern "C"
