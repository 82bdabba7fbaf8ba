// Harness around the reference's own page-address rule (imparo-cuda/native/kv_paging.cuh:25-30,
// physical_row: a page-table entry is a 64-row block id, row = (table[pos >> 6] << 6) | (pos & 63)).
// It is compiled against that header, read-only, by make_kv_paging_golden.py; the header is not
// copied.  The table is a shuffled list of block ids from a small LCG, so the JSON is self-contained.
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "kv_paging.cuh"

static uint32_t lcg_state = 1;
static uint32_t lcg() {
    lcg_state = lcg_state * 1664525u + 1013904223u;
    return lcg_state >> 8;
}

int main(int argc, char** argv) {
    if (argc != 4) return 2;
    const uint32_t n_blocks = std::atoi(argv[1]), n_rows = std::atoi(argv[2]);
    lcg_state = std::atoi(argv[3]);
    std::vector<uint32_t> table(n_blocks);
    for (uint32_t i = 0; i < n_blocks; ++i) table[i] = i;
    for (uint32_t i = n_blocks; i > 1; --i) std::swap(table[i - 1], table[lcg() % i]);     // a permutation of the pool's blocks
    std::vector<uint32_t> logical(n_rows), physical(n_rows);
    for (uint32_t i = 0; i < n_rows; ++i) {
        // page edges first (0, 63, 64, 127, ...), then scattered positions
        logical[i] = i < 2 * n_blocks ? (i / 2) * imparo_cuda_kv::kPageCells + (i % 2 ? imparo_cuda_kv::kPageCells - 1 : 0)
                                      : lcg() % (n_blocks * imparo_cuda_kv::kPageCells);
        physical[i] = imparo_cuda_kv::physical_row(logical[i], 0, table.data());
    }
    std::printf("{\"page\": %u, \"table\": [", imparo_cuda_kv::kPageCells);
    for (uint32_t i = 0; i < n_blocks; ++i) std::printf("%s%u", i ? ", " : "", table[i]);
    std::printf("], \"logical\": [");
    for (uint32_t i = 0; i < n_rows; ++i) std::printf("%s%u", i ? ", " : "", logical[i]);
    std::printf("], \"physical\": [");
    for (uint32_t i = 0; i < n_rows; ++i) std::printf("%s%u", i ? ", " : "", physical[i]);
    std::printf("]}\n");
    return 0;
}
