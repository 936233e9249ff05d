// Host-side packers of the compressed sparse-ternary format, the counterpart of the
// reference's header-only SparseTernaryTensor (include/spbitnet/sparse_ternary_tensor.h).
// Plain host memory in, plain host memory out; no CUDA.
#include <cmath>
#include <cstdint>
#include <cstring>

#include "../../include/spbitnet_b200.h"

namespace spb {
int fail(int code, const char* fmt, ...);
}

namespace {

struct GroupBits {
    uint32_t bitmap = 0, signs = 0;
    int kept = 0;
    void keep(int pos, bool negative) {
        bitmap |= 1u << pos;
        signs |= static_cast<uint32_t>(negative) << kept;
        ++kept;
    }
};

inline void put_group(uint32_t* meta_row, uint32_t* values_row, int g, const GroupBits& b) {
    meta_row[g >> 3] |= b.bitmap << ((g & 7) * 4);
    values_row[g >> 4] |= b.signs << ((g & 15) * 2);
}

}  // namespace

extern "C" int spb_meta_words_per_row(int cols) { return (cols / 4 + 7) / 8; }
extern "C" int spb_values_words_per_row(int cols) { return (cols / 4 + 15) / 16; }

extern "C" int spb_pack_from_dense(const int8_t* weights, const uint8_t* mask, int rows, int cols,
                                   uint32_t* meta, uint32_t* values) {
    if (rows < 0 || cols < 0 || cols % 4 != 0)
        return spb::fail(SPB_E_INVALID, "spb_pack_from_dense: bad shape %dx%d", rows, cols);
    if (rows == 0 || cols == 0) return SPB_OK;
    if (!weights || !mask || !meta || !values)
        return spb::fail(SPB_E_INVALID, "spb_pack_from_dense: null pointer");
    const size_t ms = spb_meta_words_per_row(cols), vs = spb_values_words_per_row(cols);
    std::memset(meta, 0, sizeof(uint32_t) * ms * rows);
    std::memset(values, 0, sizeof(uint32_t) * vs * rows);
    for (int r = 0; r < rows; ++r) {
        const int8_t* wrow = weights + static_cast<size_t>(r) * cols;
        const uint8_t* mrow = mask + static_cast<size_t>(r) * cols;
        for (int g = 0; g < cols / 4; ++g) {
            GroupBits b;
            for (int i = 0; i < 4; ++i)
                if (mrow[4 * g + i]) b.keep(i, wrow[4 * g + i] < 0);  // a kept zero becomes +1
            if (b.kept != 2)
                return spb::fail(SPB_E_FORMAT, "spb_pack_from_dense: row %d group %d keeps %d of 4", r, g,
                                 b.kept);
            put_group(meta + r * ms, values + r * vs, g, b);
        }
    }
    return SPB_OK;
}

extern "C" int spb_pack_with_pruning(const float* latent, int rows, int cols, uint32_t* meta,
                                     uint32_t* values) {
    if (rows < 0 || cols < 0 || cols % 4 != 0)
        return spb::fail(SPB_E_INVALID, "spb_pack_with_pruning: bad shape %dx%d", rows, cols);
    if (rows == 0 || cols == 0) return SPB_OK;
    if (!latent || !meta || !values) return spb::fail(SPB_E_INVALID, "spb_pack_with_pruning: null pointer");
    const size_t ms = spb_meta_words_per_row(cols), vs = spb_values_words_per_row(cols);
    std::memset(meta, 0, sizeof(uint32_t) * ms * rows);
    std::memset(values, 0, sizeof(uint32_t) * vs * rows);
    for (int r = 0; r < rows; ++r) {
        const float* lrow = latent + static_cast<size_t>(r) * cols;
        for (int g = 0; g < cols / 4; ++g) {
            // Top two magnitudes; on ties the lower index wins (what a stable descending
            // sort of the four indices gives).
            int first = 0;
            for (int i = 1; i < 4; ++i)
                if (std::fabs(lrow[4 * g + i]) > std::fabs(lrow[4 * g + first])) first = i;
            int second = -1;
            for (int i = 0; i < 4; ++i) {
                if (i == first) continue;
                if (second < 0 || std::fabs(lrow[4 * g + i]) > std::fabs(lrow[4 * g + second])) second = i;
            }
            GroupBits b;
            for (int i = 0; i < 4; ++i)
                if (i == first || i == second) b.keep(i, lrow[4 * g + i] < -0.5f);
            put_group(meta + r * ms, values + r * vs, g, b);
        }
    }
    return SPB_OK;
}

extern "C" int spb_unpack_to_int8_host(const uint32_t* meta, const uint32_t* values, int rows, int cols,
                                       int meta_row_stride, int values_row_stride, int8_t* out) {
    if (rows < 0 || cols < 0 || cols % 4 != 0)
        return spb::fail(SPB_E_INVALID, "spb_unpack_to_int8_host: bad shape %dx%d", rows, cols);
    if (rows == 0 || cols == 0) return SPB_OK;
    if (!meta || !values || !out) return spb::fail(SPB_E_INVALID, "spb_unpack_to_int8_host: null pointer");
    std::memset(out, 0, static_cast<size_t>(rows) * cols);
    for (int r = 0; r < rows; ++r) {
        const uint32_t* mrow = meta + static_cast<size_t>(r) * meta_row_stride;
        const uint32_t* vrow = values + static_cast<size_t>(r) * values_row_stride;
        int8_t* orow = out + static_cast<size_t>(r) * cols;
        for (int g = 0; g < cols / 4; ++g) {
            const uint32_t bitmap = (mrow[g >> 3] >> ((g & 7) * 4)) & 0xFu;
            uint32_t signs = (vrow[g >> 4] >> ((g & 15) * 2)) & 0x3u;
            for (int i = 0; i < 4; ++i)
                if (bitmap & (1u << i)) {
                    orow[4 * g + i] = (signs & 1u) ? -1 : 1;
                    signs >>= 1;
                }
        }
    }
    return SPB_OK;
}

extern "C" int spb_validate_packed(const uint32_t* meta, int rows, int cols, int meta_row_stride) {
    if (rows < 0 || cols < 0 || cols % 4 != 0)
        return spb::fail(SPB_E_INVALID, "spb_validate_packed: bad shape %dx%d", rows, cols);
    if (rows == 0 || cols == 0) return SPB_OK;
    if (!meta) return spb::fail(SPB_E_INVALID, "spb_validate_packed: null pointer");
    for (int r = 0; r < rows; ++r)
        for (int g = 0; g < cols / 4; ++g) {
            const uint32_t b = (meta[static_cast<size_t>(r) * meta_row_stride + (g >> 3)] >> ((g & 7) * 4)) & 0xFu;
            if (__builtin_popcount(b) != 2)
                return spb::fail(SPB_E_FORMAT, "spb_validate_packed: row %d group %d has bitmap 0x%x", r, g, b);
        }
    return SPB_OK;
}
