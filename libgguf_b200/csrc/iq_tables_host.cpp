// Search tables of the IQ quantizers, built on the host from the packed codebooks.
//
// For a lattice with `dims` coordinates of `bits` bits each, every lattice point is either a
// codebook entry (map >= 0 gives its index) or gets the list of codebook entries at the `nwant`
// smallest distinct squared distances from it, ordered by (distance, index).  The quantizers
// scan such a list and keep the first strict minimum, so the order is part of the result.
// This is the same construction as upstream libgguf_iq_tables.cpp:36-417 (iq2xs_init_impl) and
// :487-666 (iq3xs_init_impl); upstream orders with qsort on (d2, index), which is a total order,
// so any correct ordering -- here a bucket pass over the small integer distances -- gives the
// same lists.
#include "iq_tables_host.h"

#include <mutex>

#include "device_state.h"
#include "gguf_tables.cuh"

namespace gguf {
namespace {

IqHostTable build(const uint16_t *codebook, int grid_size, int dims, int bits, int nwant, int map_size) {
    IqHostTable t;
    t.grid_size = grid_size;
    t.dims = dims;
    t.grid.resize((size_t)grid_size * dims);
    t.map.assign(map_size, -1);
    const int mask = (1 << bits) - 1;
    for (int g = 0; g < grid_size; ++g) {
        for (int k = 0; k < dims; ++k) t.grid[(size_t)g * dims + k] = (uint8_t)(2 * ((codebook[g] >> (bits * k)) & mask) + 1);
        t.map[codebook[g]] = g;
    }
    const int max_d2 = dims * (2 * mask) * (2 * mask);
    std::vector<std::vector<uint16_t>> buckets(max_d2 + 1);
    std::vector<int> used;
    for (int i = 0; i < map_size; ++i) {
        if (t.map[i] >= 0) continue;
        int pos[8];
        for (int k = 0; k < dims; ++k) pos[k] = 2 * ((i >> (bits * k)) & mask) + 1;
        for (int d : used) buckets[d].clear();
        used.clear();
        for (int g = 0; g < grid_size; ++g) {
            const uint8_t *pg = &t.grid[(size_t)g * dims];
            int d2 = 0;
            for (int k = 0; k < dims; ++k) d2 += ((int)pg[k] - pos[k]) * ((int)pg[k] - pos[k]);
            if (buckets[d2].empty()) used.push_back(d2);
            buckets[d2].push_back((uint16_t)g);  // g ascending inside a bucket
        }
        t.map[i] = -((int32_t)t.neighbours.size() + 1);
        const size_t count_at = t.neighbours.size();
        t.neighbours.push_back(0);
        int have = 0, n = 0;
        for (int d2 = 0; d2 <= max_d2 && have < nwant; ++d2) {
            if (buckets[d2].empty()) continue;
            ++have;
            for (uint16_t g : buckets[d2]) { t.neighbours.push_back(g); ++n; }
        }
        t.neighbours[count_at] = (uint16_t)n;
    }
    return t;
}

}  // namespace

const IqHostTable &iq_host_table(int id) {
    static IqHostTable tables[IQT_COUNT];
    static std::once_flag once[IQT_COUNT];
    std::call_once(once[id], [id]() {
        switch (id) {
            case IQT_2XXS: tables[id] = build(k_codebook_IQ2XXS, 256, 8, 2, 2, 43692); break;
            case IQT_2XS: tables[id] = build(k_codebook_IQ2XS, 512, 8, 2, 2, 43692); break;
            case IQT_1S: tables[id] = build(k_codebook_IQ1S, 2048, 8, 2, 3, 43692); break;
            case IQT_2S: tables[id] = build(k_codebook_IQ2S, 1024, 8, 2, 1, 43692); break;
            case IQT_3XXS: tables[id] = build(k_codebook_IQ3XXS, 256, 4, 3, 2, 4096); break;
            case IQT_3S: tables[id] = build(k_codebook_IQ3S, 512, 4, 3, 3, 4096); break;
        }
    });
    return tables[id];
}

}  // namespace gguf
