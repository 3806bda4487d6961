/*
 * Test infrastructure. Compiled INTO the reference checker library only (oracle/Makefile target "ref").
 *
 * The reference keeps its IQ3 codebooks as `static const` arrays in native/redlite_native_iq3_tables.h, which a
 * shared library does not export. This shim includes that header from the reference tree at build time and hands
 * the arrays out through functions, so that the tests and the fixture generator can pass the very same tables to
 * the CUDA library and to the restated oracle. No table is retyped here.
 */
#include <stdint.h>
#include <stddef.h>
#include "redlite_native_iq3_tables.h"

const uint32_t *redcuda_ref_iq3s_grid(size_t *count) { if (count) *count = sizeof(rl_iq3s_grid) / sizeof(rl_iq3s_grid[0]); return rl_iq3s_grid; }
const uint32_t *redcuda_ref_iq3xxs_grid(size_t *count) { if (count) *count = sizeof(rl_iq3xxs_grid) / sizeof(rl_iq3xxs_grid[0]); return rl_iq3xxs_grid; }
const uint64_t *redcuda_ref_iq2s_grid(size_t *count) { if (count) *count = sizeof(rl_iq2s_grid) / sizeof(rl_iq2s_grid[0]); return rl_iq2s_grid; }
const int8_t *redcuda_ref_iq4nl_values(size_t *count) { if (count) *count = sizeof(rl_kvalues_iq4nl) / sizeof(rl_kvalues_iq4nl[0]); return rl_kvalues_iq4nl; }
