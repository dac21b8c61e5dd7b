// Host-built tables and their per-device copies.
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <mutex>
#include <utility>
#include <vector>

#include "../../include/libgguf_cuda_native.h"
#include "device_state.h"
#include "gguf_common.cuh"
#include "gguf_tables.cuh"
#include "iq_tables_host.h"

namespace gguf {
namespace {

struct Slot {
    std::mutex lock;
    DeviceState state;
    std::vector<void *> allocations;
};
Slot g_slots[kMaxDevices];

// floorf(log2f(x)) as computed by this machine's libm, per binade.  For t = -149..127 the entry is
// the smallest float x in [2^t, 2^(t+1)) with floorf(log2f(x)) == t+1, or +inf when every x of the
// binade gives t.  upstream mxfp4.cpp:39 takes the exponent from that libm expression, and a
// correctly rounded log2f of a value just below a power of two can round up to the integer.
// log2f is assumed monotonic (glibc's is), so a bisection over the mantissa finds the step.
std::vector<float> build_mx_steps() {
    std::vector<float> steps(277);
    for (int t = -149; t <= 127; ++t) {
        const float lo = ldexpf(1.0f, t);
        // largest float of the binade
        const float hi = t >= -126 ? nextafterf(ldexpf(1.0f, t + 1), 0.0f) : nextafterf(ldexpf(1.0f, t + 1), 0.0f);
        float result = INFINITY;
        if (floorf(log2f(hi)) >= (float)(t + 1)) {
            uint32_t a = f32_to_bits(lo), b = f32_to_bits(hi);  // positive floats order like their bits
            if (floorf(log2f(lo)) >= (float)(t + 1)) {
                b = a;
            } else {
                while (b - a > 1) {
                    const uint32_t mid = a + (b - a) / 2;
                    if (floorf(log2f(bits_to_f32(mid))) >= (float)(t + 1)) b = mid; else a = mid;
                }
            }
            result = bits_to_f32(b);
        }
        steps[t + 149] = result;
    }
    return steps;
}

const std::vector<float> &mx_steps_host() {
    static const std::vector<float> steps = build_mx_steps();
    return steps;
}

template <class T>
const T *upload(Slot &slot, const std::vector<T> &host) {
    void *p = nullptr;
    const size_t bytes = host.size() * sizeof(T);
    // 64 zero bytes follow every table (a look-ahead read just past the last entry stays inside the allocation)
    if (cudaMalloc(&p, bytes + 64) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    if (cudaMemset(static_cast<char *>(p) + bytes, 0, 64) != cudaSuccess ||
        (bytes && cudaMemcpy(p, host.data(), bytes, cudaMemcpyHostToDevice) != cudaSuccess)) {
        cudaGetLastError();
        cudaFree(p);
        return nullptr;
    }
    slot.allocations.push_back(p);
    return static_cast<const T *>(p);
}

int table_for_type(int type) {
    switch (type) {
        case GGML_TYPE_IQ2_XXS: return IQT_2XXS;
        case GGML_TYPE_IQ2_XS: return IQT_2XS;
        case GGML_TYPE_IQ1_S: case GGML_TYPE_IQ1_M: return IQT_1S;
        case GGML_TYPE_IQ2_S: return IQT_2S;
        case GGML_TYPE_IQ3_XXS: return IQT_3XXS;
        case GGML_TYPE_IQ3_S: return IQT_3S;
        default: return -1;
    }
}

// The IQ2 / IQ3 neighbour lists in the layout the scans read (see IqSearchTable), built on the host once per process.
struct IqScanRecords {
    bool valid = false;
    int record_steps = 0;            // steps of kIqStepEntries entries per record
    int hot_bytes = 0;               // whole lists at the front of `entries` that fit kIqHotBudget
    std::vector<uint16_t> entries;   // records back to back
    std::vector<int32_t> map_s;
};

const IqScanRecords &iq_scan_records(int id) {
    static IqScanRecords built[IQT_COUNT];
    static std::mutex lock;
    std::lock_guard<std::mutex> guard(lock);
    IqScanRecords &r = built[id];
    if (r.record_steps) return r;
    const IqHostTable &h = iq_host_table(id);
    // the codebook with the longest lists (IQ2_XS, mean 58 entries) uses two-step records: half as many list loads
    const uint32_t rec_steps = id == IQT_2XS ? 2 : 1, rec_entries = rec_steps * kIqStepEntries;
    r.record_steps = (int)rec_steps;
    r.map_s.resize(h.map.size());
    bool ok = (size_t)h.grid_size * h.dims * 2 <= 65536;
    // lattice points off the codebook, most common first: by the sum of their levels, then by index
    const int bits = h.dims == 8 ? 2 : 3;
    std::vector<uint32_t> order;
    for (size_t i = 0; i < h.map.size(); ++i) {
        if (h.map[i] >= 0) r.map_s[i] = h.map[i];
        else order.push_back((uint32_t)i);
    }
    auto level_sum = [&](uint32_t u) {
        int sum = 0;
        for (int c = 0; c < h.dims; ++c) {
            const int level = (int)((u >> (bits * c)) & ((1u << bits) - 1));
            sum += (bits == 2 && level == 3) ? 1000 : level;  // a 2-bit field of 3 is no level: the quantizers never look such a point up
        }
        return sum;
    };
    if (kIqHotBudget[id] < (1 << 20))   // (a codebook whose records all fit keeps them in index order)
        std::stable_sort(order.begin(), order.end(), [&](uint32_t a, uint32_t b) { return level_sum(a) < level_sum(b); });
    bool hot_open = true;
    for (size_t k = 0; ok && k < order.size(); ++k) {
        const uint32_t i = order[k];
        const uint32_t off = (uint32_t)(-h.map[i] - 1), n = h.neighbours[off];
        const uint32_t first_rec = (uint32_t)(r.entries.size() / rec_entries), nrec = (n + rec_entries - 1) / rec_entries;
        if (first_rec >= (1u << 22) || nrec >= (1u << 8)) { ok = false; break; }
        for (uint32_t e = 0; e < nrec * rec_entries; ++e)
            r.entries.push_back((uint16_t)(h.neighbours[off + 1 + (e < n ? e : 0)] * h.dims * 2));
        r.map_s[i] = -(int32_t)(((first_rec << 8) | nrec) + 1);
        const size_t bytes = r.entries.size() * sizeof(uint16_t);
        if (hot_open && bytes <= (size_t)kIqHotBudget[id]) {
            if (bytes % 16 == 0) r.hot_bytes = (int)bytes;   // the prefix is copied in 16-byte pieces
        } else {
            hot_open = false;
        }
    }
    while (r.entries.size() % 8) r.entries.push_back(0);     // a whole number of 16-byte pieces
    if (r.entries.size() * sizeof(uint16_t) <= (size_t)kIqHotBudget[id]) r.hot_bytes = (int)(r.entries.size() * sizeof(uint16_t));
    r.valid = ok;
    return r;
}

}  // namespace

const DeviceState *device_state_for(int type, int dev) {
    if (dev < 0 || dev >= kMaxDevices) return nullptr;
    Slot &slot = g_slots[dev];
    std::lock_guard<std::mutex> guard(slot.lock);
    slot.state.device = dev;
    if (type == GGML_TYPE_MXFP4 && !slot.state.mx_steps) {
        slot.state.mx_steps = upload(slot, mx_steps_host());
        if (!slot.state.mx_steps) return nullptr;
    }
    const int id = table_for_type(type);
    if (id >= 0 && !slot.state.iq[id].grid) {
        const IqHostTable &h = iq_host_table(id);
        IqSearchTable t;
        t.grid = upload(slot, h.grid);
        t.map = upload(slot, h.map);
        t.neighbours = upload(slot, h.neighbours);
        {   // one load then tells a scan where its list is and how many records it has
            const IqScanRecords &r = iq_scan_records(id);
            if (!r.valid) return nullptr;
            t.map_s = upload(slot, r.map_s);
            t.records = upload(slot, r.entries);
            t.record_steps = r.record_steps;
            t.records_bytes = (int)(r.entries.size() * sizeof(uint16_t));
            t.hot_bytes = r.hot_bytes;
            if (!t.map_s || !t.records) return nullptr;
        }
        if (!t.grid || !t.map || !t.neighbours) return nullptr;
        t.grid_size = h.grid_size;
        t.dims = h.dims;
        t.map_size = (int)h.map.size();
        t.neighbours_len = (int)h.neighbours.size();
        slot.state.iq[id] = t;
    }
    return &slot.state;
}

void device_state_release_all() {
    for (int dev = 0; dev < kMaxDevices; ++dev) {
        Slot &slot = g_slots[dev];
        std::lock_guard<std::mutex> guard(slot.lock);
        if (slot.allocations.empty()) continue;
        if (cudaSetDevice(dev) == cudaSuccess) {
            for (void *p : slot.allocations) cudaFree(p);
        }
        cudaGetLastError();
        slot.allocations.clear();
        slot.state = DeviceState();
    }
}

}  // namespace gguf

// Host view of one quantizer's search tables (no device involved).
extern "C" int libgguf_cuda_iq_search_table(int64_t qtype, int32_t *grid_size, int32_t *dims, const uint8_t **grid,
                                            const int32_t **map, int64_t *map_size, const uint16_t **neighbours,
                                            int64_t *neighbours_len) {
    const int id = gguf::table_for_type((int)qtype);
    if (id < 0) return LIBGGUF_CUDA_STATUS_UNSUPPORTED_TYPE;
    const gguf::IqHostTable &t = gguf::iq_host_table(id);
    if (grid_size) *grid_size = t.grid_size;
    if (dims) *dims = t.dims;
    if (grid) *grid = t.grid.data();
    if (map) *map = t.map.data();
    if (map_size) *map_size = (int64_t)t.map.size();
    if (neighbours) *neighbours = t.neighbours.data();
    if (neighbours_len) *neighbours_len = (int64_t)t.neighbours.size();
    return LIBGGUF_CUDA_STATUS_SUCCESS;
}

// Host view of the scan layout of one IQ2 / IQ3 quantizer's neighbour lists (no device involved).
extern "C" int libgguf_cuda_iq_scan_records(int64_t qtype, int32_t *record_entries, const uint16_t **entries, int64_t *entries_len,
                                            const int32_t **map_s, int64_t *map_size) {
    const int id = gguf::table_for_type((int)qtype);
    if (id < 0) return LIBGGUF_CUDA_STATUS_UNSUPPORTED_TYPE;
    const gguf::IqScanRecords &r = gguf::iq_scan_records(id);
    if (!r.valid) return LIBGGUF_CUDA_STATUS_INVALID_ARGUMENT;  // a codebook outside the layout's field widths
    if (record_entries) *record_entries = r.record_steps * gguf::kIqStepEntries;
    if (entries) *entries = r.entries.data();
    if (entries_len) *entries_len = (int64_t)r.entries.size();
    if (map_s) *map_s = r.map_s.data();
    if (map_size) *map_size = (int64_t)r.map_s.size();
    return LIBGGUF_CUDA_STATUS_SUCCESS;
}
