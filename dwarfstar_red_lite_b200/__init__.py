"""redcuda: B200 (sm_100a) backend for the Qwen3-Next decode hot path of Red Lite.

The compute lives in libredcuda.so (hand-written CUDA behind the C ABI of include/redcuda.h); this package is the
thin Python host mirror of that ABI plus seeded synthetic inputs. There is no CPU path: every operation raises when
the library or a CUDA device is missing.
"""
from . import synth  # noqa: F401
from .redcuda import (MoeLayer, RedcudaError, deltanet_step, lib, nib_dequant_rows, quant_dequant_rows, quant_matmul_tc, quant_matvec,  # noqa: F401
                      router_select_softmax_topk, set_codebooks)
