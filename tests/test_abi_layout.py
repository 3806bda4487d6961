"""Struct layouts and prototypes of include/rl_engine.h against the reference's own header
(native/redlite_native_engine.h:22-129): a C program compiled against each header prints sizeof / offsetof of the three
structs the ABI passes by pointer; the printouts must be identical. A second program, compiled against the REFERENCE
headers only, calls the engine and pool entry points and must link against libredcuda.so without an unresolved symbol.
Needs the reference tree (REF_ROOT, or its usual mount point); skipped where it is absent."""
import os
import subprocess

import pytest

import dwarfstar_red_lite_b200 as rc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("REF_ROOT") or os.path.join(os.sep, "root", "reference")
REF_NATIVE = os.path.join(REF, "native")
needs_ref = pytest.mark.skipif(not os.path.isfile(os.path.join(REF_NATIVE, "redlite_native_engine.h")), reason="reference tree not mounted")

PROBE = r'''
#include <stddef.h>
#include <stdio.h>
#include HEADER
#define F(T, m) printf(#T "." #m " %zu\n", offsetof(T, m))
int main(void) {
    printf("rl_engine_config %zu\n", sizeof(rl_engine_config));
    F(rl_engine_config, context); F(rl_engine_config, cache_mib); F(rl_engine_config, top_k); F(rl_engine_config, enable_cpu); F(rl_engine_config, enable_gpu);
    F(rl_engine_config, cpu_threads); F(rl_engine_config, prefill_batch); F(rl_engine_config, mtp_path);
    printf("rl_engine_info %zu\n", sizeof(rl_engine_info));
    F(rl_engine_info, n_layer); F(rl_engine_info, vocab); F(rl_engine_info, context); F(rl_engine_info, d_conv); F(rl_engine_info, head_v); F(rl_engine_info, n_head);
    F(rl_engine_info, rope_dims); F(rl_engine_info, rope_freq_base); F(rl_engine_info, rms_eps); F(rl_engine_info, dense_bytes); F(rl_engine_info, state_bytes);
    printf("rl_engine_step_stats %zu\n", sizeof(rl_engine_step_stats));
    F(rl_engine_step_stats, embed_ms); F(rl_engine_step_stats, total_ms); F(rl_engine_step_stats, gpu_ms); F(rl_engine_step_stats, expert_loads);
    F(rl_engine_step_stats, cache_misses); F(rl_engine_step_stats, ssd_reads); F(rl_engine_step_stats, resident_slots); F(rl_engine_step_stats, slot_capacity);
    F(rl_engine_step_stats, expert_plans); F(rl_engine_step_stats, prep_lru_ms); F(rl_engine_step_stats, prefetch_ms); F(rl_engine_step_stats, speculative);
    F(rl_engine_step_stats, speculative_fallback);
    printf("RL_BACKEND_GPU %d\n", (int)RL_BACKEND_GPU);
    return 0;
}
'''

LINK = r'''
#include <stdio.h>
#include "redlite_native_engine.h"
#include "redmetal_topk.h"
/* every call below is type-checked against the REFERENCE prototypes and resolved by libredcuda.so */
int main(int argc, char **argv) {
    char err[256];
    rl_engine_config cfg;
    rl_engine_config_default(&cfg);
    cfg.enable_cpu = 0; cfg.enable_gpu = 1; cfg.context = 64;
    if (redmetal_topk_abi_version() != 1u) return 2;
    if (argc < 2) { printf("linked\n"); return 0; }
    rl_engine *e = rl_engine_open(argv[1], &cfg, err, sizeof(err));
    if (!e) { printf("open failed: %s\n", err); return 3; }
    const rl_engine_info *in = rl_engine_info_get(e);
    rl_engine_step_stats st;
    uint32_t tok = 3;
    for (int i = 0; i < 8; ++i) {
        if (!rl_engine_step(e, RL_BACKEND_GPU, tok, NULL, &st, err, sizeof(err))) { printf("step failed: %s\n", err); return 4; }
        if (st.cache_misses || st.ssd_reads || st.ssd_bytes || st.expert_loads) { printf("a resident engine reported expert traffic\n"); return 5; }
        if (st.resident_slots != in->n_layer * in->n_expert || st.slot_capacity != st.resident_slots) { printf("slot counters\n"); return 6; }
        tok = (tok * 7u + 1u) % in->vocab;
    }
    double ms = 0.0;
    if (rl_engine_experts_preloaded(e, &ms) != 1) return 7;
    printf("ok position %u layers %u preload %.1f ms\n", rl_engine_position(e, RL_BACKEND_GPU), in->n_layer, ms);
    redmetal_topk_pool_t pool = redmetal_topk_pool_create(argv[1], 1u << 20, 1u << 16, 4, NULL, 0, NULL, 0);
    if (!pool || redmetal_topk_pool_capacity(pool) != 16u || redmetal_topk_pool_bytes_read(pool) != 0u) return 8;
    redmetal_topk_pool_destroy(pool);
    rl_engine_close(e);
    return 0;
}
'''


def _run_probe(tmp_path, header_dir, header, tag):
    src = tmp_path / f"probe_{tag}.c"
    src.write_text(PROBE.replace("HEADER", f'"{header}"'))
    exe = tmp_path / f"probe_{tag}"
    subprocess.check_call(["gcc", "-std=c11", "-I", header_dir, "-o", str(exe), str(src)])
    return subprocess.check_output([str(exe)], text=True)


@needs_ref
def test_struct_layouts_equal_the_reference_headers(tmp_path):
    ours = _run_probe(tmp_path, os.path.join(ROOT, "include"), "rl_engine.h", "ours")
    theirs = _run_probe(tmp_path, REF_NATIVE, "redlite_native_engine.h", "ref")
    assert ours == theirs, (ours, theirs)
    assert "rl_engine_step_stats" in ours


def _link(tmp_path):
    src = tmp_path / "link.c"
    src.write_text(LINK)
    exe = tmp_path / "link"
    libdir = os.path.dirname(rc.redcuda.LIB_PATH)
    subprocess.check_call(["gcc", "-std=c11", "-I", REF_NATIVE, "-o", str(exe), str(src), "-L", libdir, "-lredcuda", f"-Wl,-rpath,{libdir}", "-Wl,--no-undefined"])
    return exe


@needs_ref
def test_program_written_against_the_reference_headers_links(tmp_path):
    rc.lib()
    exe = _link(tmp_path)
    assert subprocess.check_output([str(exe)], text=True).strip() == "linked"
