// Host-side construction of the IQ quantizers' search tables.
#pragma once

#include <stdint.h>

#include <vector>

namespace gguf {

struct IqHostTable {
    int grid_size = 0;
    int dims = 0;                      // 8 (2-bit lattices) or 4 (3-bit lattices)
    std::vector<uint8_t> grid;         // grid_size * dims coordinates, value 2*code+1
    std::vector<int32_t> map;          // lattice index -> grid index, or -(offset+1) into neighbours
    std::vector<uint16_t> neighbours;  // runs: count, then `count` grid indices ordered by (distance, index)
};

// id is an IqTableId.  Built on first request, cached for the life of the process.
const IqHostTable &iq_host_table(int id);

}  // namespace gguf
