// Harness around the reference's own host C++ for the gated short convolution
// (imparo-cuda/native/lfm2_ops.cuh: shortconv_reference, shortconv_state_reference).
// It is compiled against that header, read-only, by make_conv_golden.py; the header is
// not copied.  Inputs come from a small LCG so the JSON it prints is self-contained.
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "lfm2_ops.cuh"

static uint32_t lcg_state = 1;
static float lcg() {
    lcg_state = lcg_state * 1664525u + 1013904223u;
    return ((lcg_state >> 8) & 0xFFFF) / 32768.0f - 1.0f;   // [-1, 1)
}

static void dump(const char* name, const std::vector<float>& v, bool last = false) {
    std::printf("\"%s\": [", name);
    for (size_t i = 0; i < v.size(); ++i) std::printf("%s%.9g", i ? ", " : "", v[i]);
    std::printf("]%s\n", last ? "" : ",");
}

int main(int argc, char** argv) {
    if (argc != 5) return 2;
    const uint32_t width = std::atoi(argv[1]), kernel = std::atoi(argv[2]), n_tok = std::atoi(argv[3]);
    lcg_state = std::atoi(argv[4]);
    std::vector<float> bcx(size_t(n_tok) * 3 * width), w(size_t(width) * kernel), state(size_t(kernel - 1) * width);
    for (auto& v : bcx) v = lcg();
    for (auto& v : w) v = lcg();
    for (auto& v : state) v = lcg();
    std::vector<float> out(size_t(n_tok) * width), next(state.size());
    imparo_cuda_lfm2::shortconv_reference(bcx.data(), w.data(), state.data(), out.data(), width, kernel, n_tok);
    imparo_cuda_lfm2::shortconv_state_reference(bcx.data(), state.data(), next.data(), width, kernel, n_tok);
    std::printf("{\"width\": %u, \"kernel\": %u, \"n_tok\": %u,\n", width, kernel, n_tok);
    dump("bcx", bcx); dump("weights", w); dump("state", state); dump("output", out); dump("next_state", next, true);
    std::printf("}\n");
    return 0;
}
