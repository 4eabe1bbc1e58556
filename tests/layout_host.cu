// Test helper (host code only): applies the file -> tiled permutation and decodes every element back on the CPU,
// with the same index functions the device kernels use (exactinfer_b200/csrc/layout.cuh). Built by
// tests/test_layout_host.py with nvcc; never part of libelb.so.
#include <vector>

#include "../exactinfer_b200/csrc/layout.cuh"

namespace elb {
void set_error(const std::string&) {}
int fail(int code, const std::string&) { return code; }
}  // namespace elb

extern "C" int layout_roundtrip(int type, long long rows, long long n, const unsigned char* bytes, int pair,
                                float* out /* [ceil(rows/16)*16][n] */, int* qout) {
    using namespace elb;
    const int64_t tiles = (rows + 15) / 16;
    int64_t upt, unit;
    if (type == ELB_Q4_K) { upt = n / 256; unit = Q4K_UNIT; }
    else if (type == ELB_Q6_K) { upt = n / 256; unit = Q6K_UNIT; }
    else if (type == ELB_Q8_0) { upt = n / 128; unit = Q8_UNIT; }
    else return 1;
    std::vector<uint8_t> tiled(size_t(tiles * upt * unit));
    for (int64_t o = 0; o < int64_t(tiled.size()); ++o) {
        if (type == ELB_Q4_K) tiled[size_t(o)] = tile_byte_q4k(bytes, o, rows, n / 256, pair != 0);
        else if (type == ELB_Q6_K) tiled[size_t(o)] = tile_byte_q6k(bytes, o, rows, n / 256, pair != 0);
        else tiled[size_t(o)] = tile_byte_q8(bytes, o, rows, n / 32, pair != 0);
    }
    for (int64_t R = 0; R < tiles * 16; ++R)
        for (int64_t k = 0; k < n; ++k) {
            const QElem e = tiled_elem(type, tiled.data(), n, R, k);
            out[R * n + k] = elem_value(type, e);
            if (qout) qout[R * n + k] = e.sc * e.q;
        }
    return 0;
}
