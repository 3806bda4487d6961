// Test helper (compiled by tests/test_kq_iq_host.py with nvcc for the HOST only): runs the library's own decoder of the
// IQ3_XXS / IQ2_S / IQ4_XS / IQ2_XS / IQ1_M blocks - the same inline function the CUDA kernels call - on the CPU and compares
// every value, bit for bit, with the CPU checker's dequantiser on random blocks and on special block scales.
// usage: kq_iq_host_check <libredcuda_oracle.so> <codebooks_iq3family.bin> <codebooks_iq2xs_iq1m.bin>
#include "redcuda_kquants_iq.cuh"
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <dlfcn.h>
#include <vector>
int main(int argc, char **argv) {
    void *h = dlopen(argv[1], RTLD_NOW);
    if (!h) { printf("dlopen: %s\n", dlerror()); return 2; }
    auto set_ext = (int (*)(const uint32_t *, const uint64_t *, const int8_t *))dlsym(h, "ro_set_codebooks_ext");
    auto deq = (int (*)(uint32_t, const uint8_t *, uint32_t, float *))dlsym(h, "ro_dequant_row");
    FILE *f = fopen(argv[2], "rb");
    std::vector<uint8_t> tab(9232);
    if (fread(tab.data(), 1, 9232, f) != 9232) return 3;
    fclose(f);
    FILE *f2 = fopen(argv[3], "rb");
    std::vector<uint8_t> tab2(20480);
    if (fread(tab2.data(), 1, 20480, f2) != 20480) return 3;
    fclose(f2);
    auto set_xs = (int (*)(const int8_t *, const int8_t *))dlsym(h, "ro_set_codebooks_xs");
    rc::KqIqTabs T{(const uint32_t *)tab.data(), (const uint64_t *)(tab.data() + 1024), (const int8_t *)(tab.data() + 9216), (const int8_t *)tab2.data(), (const int8_t *)(tab2.data() + 4096)};
    set_ext(T.iq3xxs, T.iq2s, T.iq4nl);
    set_xs(T.iq2xs, T.iq1m);
    srand(7);
    const uint32_t types[5] = {18u, 22u, 23u, 17u, 29u};
    for (uint32_t t : types) {
        const uint32_t bb = rc::kq_iq_block_bytes(t), nb = 4096;
        std::vector<uint8_t> row((size_t)nb * bb);
        for (auto &b : row) b = (uint8_t)(rand() >> 7);
        // a few special scales: zero, subnormal, negative, large
        const uint16_t special[6] = {0x0000, 0x0001, 0x8400, 0x7bff, 0x03ff, 0xbc00};
        auto put_d = [&](uint32_t i, uint16_t d) {
            uint8_t *bp = &row[(size_t)i * bb];
            if (t != 29u) { memcpy(bp, &d, 2); return; }
            for (uint32_t k = 0; k < 4; ++k) bp[49 + 2 * k] = (uint8_t)((bp[49 + 2 * k] & 0x0f) | (((d >> (4 * k)) & 0xf) << 4));    // top nibble of sc[k]
        };
        for (uint32_t i = 0; i < 6; ++i) put_d(i, special[i]);
        for (uint32_t i = 6; i < nb; ++i) put_d(i, (uint16_t)((0x1000 + (rand() % 0x2000)) | ((rand() & 1) << 15)));
        std::vector<float> want((size_t)nb * 256), got((size_t)nb * 256);
        if (deq(t, row.data(), nb * 256, want.data()) != 1) { printf("oracle refused type %u\n", t); return 4; }
        size_t bad = 0;
        for (uint32_t b = 0; b < nb; ++b)
            for (uint32_t j = 0; j < 256; ++j) {
                got[(size_t)b * 256 + j] = rc::kq_iq_value(t, &row[(size_t)b * bb], j, T);
                if (memcmp(&got[(size_t)b * 256 + j], &want[(size_t)b * 256 + j], 4) != 0) { if (bad < 5) printf("type %u block %u value %u: %a vs %a\n", t, b, j, got[(size_t)b * 256 + j], want[(size_t)b * 256 + j]); ++bad; }
            }
        printf("type %u: %zu of %zu values differ\n", t, bad, (size_t)nb * 256);
        if (bad) return 1;
    }
    return 0;
}
