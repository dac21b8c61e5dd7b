// Staging of the host-pointer calls (libgguf_quantize_chunk / libgguf_dequantize_chunk): the caller's buffers are
// ordinary pageable memory, which the driver can only move through its own small bounce buffers, one copy at a time.
// Here the bytes go through two pinned slots per direction instead, filled and drained by a few host threads while
// the device works on the neighbouring piece, so the call runs at the rate of the host link.
#include "host_stage.h"

#include <stdlib.h>
#include <string.h>

#include <condition_variable>
#include <mutex>
#include <thread>
#include <vector>

namespace gguf {
namespace {

constexpr size_t kPartBytes = size_t(1) << 20;  // smallest share worth handing to another thread

class CopyPool {
  public:
    static CopyPool &get() {
        static CopyPool *pool = new CopyPool();  // never destroyed: its threads may outlive static destruction
        return *pool;
    }
    void copy(char *dst, const char *src, size_t bytes) {
        if (workers_.empty() || bytes < 2 * kPartBytes) {
            memcpy(dst, src, bytes);
            return;
        }
        std::lock_guard<std::mutex> one_job(submit_);
        {
            std::lock_guard<std::mutex> guard(lock_);
            dst_ = dst;
            src_ = src;
            bytes_ = bytes;
            parts_ = (bytes + kPartBytes - 1) / kPartBytes;
            next_ = 0;
            left_ = parts_;
            ++generation_;
        }
        wake_.notify_all();
        work();
        std::unique_lock<std::mutex> guard(lock_);
        finished_.wait(guard, [&] { return left_ == 0; });
    }

  private:
    CopyPool() {
        int n = 0;
        if (const char *env = getenv("LIBGGUF_CUDA_COPY_THREADS")) n = atoi(env);
        if (n <= 0) {
            const unsigned hw = std::thread::hardware_concurrency();
            n = hw >= 16 ? 8 : hw >= 4 ? (int)hw / 2 : 1;
        }
        for (int i = 1; i < n; ++i) {  // the caller is the n-th
            workers_.emplace_back([this] { run(); });
            workers_.back().detach();
        }
    }
    void run() {
        uint64_t seen = 0;
        for (;;) {
            {
                std::unique_lock<std::mutex> guard(lock_);
                wake_.wait(guard, [&] { return generation_ != seen; });
                seen = generation_;
            }
            work();
        }
    }
    // Takes parts of the current job until none is left.  The index is drawn together with the job's pointers, so a
    // worker that is still looping when the next job is posted simply starts on that one.
    void work() {
        for (;;) {
            size_t part, bytes;
            char *dst;
            const char *src;
            {
                std::lock_guard<std::mutex> guard(lock_);
                if (next_ >= parts_) return;
                part = next_++;
                bytes = bytes_; dst = dst_; src = src_;
            }
            const size_t begin = part * kPartBytes, n = bytes - begin < kPartBytes ? bytes - begin : kPartBytes;
            memcpy(dst + begin, src + begin, n);
            std::lock_guard<std::mutex> guard(lock_);
            if (--left_ == 0) finished_.notify_all();
        }
    }

    std::mutex submit_, lock_;
    std::condition_variable wake_, finished_;
    std::vector<std::thread> workers_;
    char *dst_ = nullptr;
    const char *src_ = nullptr;
    size_t bytes_ = 0, parts_ = 0, left_ = 0;
    size_t next_ = 0;
    uint64_t generation_ = 0;
};

}  // namespace

void parallel_copy(void *dst, const void *src, size_t bytes) {
    CopyPool::get().copy(static_cast<char *>(dst), static_cast<const char *>(src), bytes);
}

bool StageRing::reserve(size_t in_bytes, size_t out_bytes) {
    for (int s = 0; s < 2; ++s) {
        if (!stream[s] && cudaStreamCreateWithFlags(&stream[s], cudaStreamNonBlocking) != cudaSuccess) return false;
        if (!in_free[s] && cudaEventCreateWithFlags(&in_free[s], cudaEventDisableTiming) != cudaSuccess) return false;
        if (!done[s] && cudaEventCreateWithFlags(&done[s], cudaEventDisableTiming) != cudaSuccess) return false;
    }
    auto grow_pair = [](void **host, void **device, size_t need) {
        if (*host) cudaFreeHost(*host);
        if (*device) cudaFree(*device);
        *host = *device = nullptr;
        return cudaHostAlloc(host, need, cudaHostAllocDefault) == cudaSuccess && cudaMalloc(device, need) == cudaSuccess;
    };
    if (in_bytes > in_cap) {
        in_cap = 0;
        for (int s = 0; s < 2; ++s) if (!grow_pair(&h_in[s], &d_in[s], in_bytes)) return false;
        in_cap = in_bytes;
    }
    if (out_bytes > out_cap) {
        out_cap = 0;
        for (int s = 0; s < 2; ++s) if (!grow_pair(&h_out[s], &d_out[s], out_bytes)) return false;
        out_cap = out_bytes;
    }
    return true;
}

void StageRing::release() {
    for (int s = 0; s < 2; ++s) {
        if (stream[s]) cudaStreamSynchronize(stream[s]);
        if (h_in[s]) cudaFreeHost(h_in[s]);
        if (h_out[s]) cudaFreeHost(h_out[s]);
        if (d_in[s]) cudaFree(d_in[s]);
        if (d_out[s]) cudaFree(d_out[s]);
        if (in_free[s]) cudaEventDestroy(in_free[s]);
        if (done[s]) cudaEventDestroy(done[s]);
        if (stream[s]) cudaStreamDestroy(stream[s]);
        h_in[s] = h_out[s] = d_in[s] = d_out[s] = nullptr;
        in_free[s] = done[s] = nullptr;
        stream[s] = nullptr;
    }
    in_cap = out_cap = 0;
}

cudaError_t run_staged(StageRing &ring, const char *in, size_t in_row, char *out, size_t out_row, int64_t rows,
                       int64_t rows_per_piece, const StageLaunch &launch) {
    const int64_t pieces = (rows + rows_per_piece - 1) / rows_per_piece;
    auto first = [&](int64_t p) { return p * rows_per_piece; };
    auto count = [&](int64_t p) { return rows - first(p) < rows_per_piece ? rows - first(p) : rows_per_piece; };
    auto copy_in = [&](int64_t p) { parallel_copy(ring.h_in[p & 1], in + (size_t)first(p) * in_row, (size_t)count(p) * in_row); };
    auto enqueue = [&](int64_t p) -> cudaError_t {
        const int s = (int)(p & 1);
        cudaError_t e = cudaMemcpyAsync(ring.d_in[s], ring.h_in[s], (size_t)count(p) * in_row, cudaMemcpyHostToDevice, ring.stream[s]);
        if (e == cudaSuccess) e = cudaEventRecord(ring.in_free[s], ring.stream[s]);
        if (e == cudaSuccess) e = launch(ring.d_in[s], ring.d_out[s], first(p), count(p), ring.stream[s]);
        if (e == cudaSuccess) e = cudaMemcpyAsync(ring.h_out[s], ring.d_out[s], (size_t)count(p) * out_row, cudaMemcpyDeviceToHost, ring.stream[s]);
        if (e == cudaSuccess) e = cudaEventRecord(ring.done[s], ring.stream[s]);
        return e;
    };
    auto copy_out = [&](int64_t p) -> cudaError_t {
        const cudaError_t e = cudaEventSynchronize(ring.done[p & 1]);
        if (e == cudaSuccess) parallel_copy(out + (size_t)first(p) * out_row, ring.h_out[p & 1], (size_t)count(p) * out_row);
        return e;
    };
    cudaError_t e = cudaSuccess;
    copy_in(0);
    for (int64_t p = 0; p < pieces && e == cudaSuccess; ++p) {
        e = enqueue(p);
        if (e == cudaSuccess && p + 1 < pieces) {
            // slot (p + 1) & 1 last carried piece p - 1: its pinned input may be overwritten once that copy has run
            if (p >= 1) e = cudaEventSynchronize(ring.in_free[(p + 1) & 1]);
            if (e == cudaSuccess) copy_in(p + 1);
        }
        if (e == cudaSuccess && p >= 1) e = copy_out(p - 1);
    }
    if (e == cudaSuccess) e = copy_out(pieces - 1);
    if (e != cudaSuccess) {  // leave nothing in flight that still points at the caller's or the ring's memory
        cudaStreamSynchronize(ring.stream[0]);
        cudaStreamSynchronize(ring.stream[1]);
    }
    return e;
}

}  // namespace gguf
