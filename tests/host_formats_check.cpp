// Host build of the planar repack and the exact decoders of dwarfstar_red_lite_b200/csrc/redcuda_formats.cuh, so that
// the layout arithmetic and the decoders can be checked against the CPU oracle without a GPU (test helper only).
#include "../dwarfstar_red_lite_b200/csrc/redcuda_formats.cuh"
#include <vector>

extern "C" int host_repack_dequant(uint32_t type, const uint8_t *rows, uint32_t nrows, uint32_t ncols,
                                   const uint8_t *iq2, const uint32_t *iq3s, int use_dst_map, float *out) {
    const uint64_t bytes = rc_matrix_bytes(type, nrows, ncols);
    if (!bytes || !rc_is_quant(type)) return 0;
    const uint64_t nb = (uint64_t)nrows * (ncols / 256u);
    std::vector<uint8_t> planar(bytes, 0xEE);
    if (use_dst_map) {   // the per-byte destination map the device repack kernel uses
        const uint32_t bb = rc_block_bytes(type);
        for (uint64_t b = 0; b < nb; ++b) for (uint32_t off = 0; off < bb; ++off) planar[rc_planar_dst(type, nb, b, off)] = rows[b * bb + off];
    } else rc_repack_host(type, rows, planar.data(), nb);
    const RcBooks bk{iq2, iq3s};
    for (uint64_t b = 0; b < nb; ++b) for (uint32_t g = 0; g < 32u; ++g) rc_decode8(type, planar.data(), nb, b, g, bk, out + (b * 32u + g) * 8u);
    return 1;
}
