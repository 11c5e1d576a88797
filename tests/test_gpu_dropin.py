"""The drop-in against the reference's own structures: oracle/_ref/libtie_ref_dropin.so holds the
reference's compiled sources, a TIEContext / Model / LayerWeights set up as the engine does, and
the glue a maintainer adds (tie_b200/dropin/tie_cuda_qwen3.c), linked with libtie_cuda.so.  The
MoE branch through the glue (one tie_cuda_moe_ffn call on ctx->mem buffers, host pointers, the
engine's own silu_table) must match the reference's CPU branch run on the same context."""
import os

import numpy as np
import pytest

from tie_b200 import synth, workloads

pytestmark = pytest.mark.gpu


def test_reference_context_through_the_glue(layer0):
    from oracle import ref
    if not os.path.exists(ref.LIB_DROPIN_PATH):
        pytest.skip("oracle/_ref/libtie_ref_dropin.so not built (make -C oracle dropin REF=<reference sources>)")
    R = ref.RefMoe(path=ref.LIB_DROPIN_PATH)
    R.set_layer(layer0)
    R.dropin_load(device=0, max_tokens=64)
    try:
        for n_tokens in (1, 3, 64):
            x = synth.make_x(workloads.BASE_SEED + 5, n_tokens)
            want, _, _ = R.moe_ffn(x)          # the reference's CPU branch
            got = R.dropin_moe_ffn(x)          # the same context through the glue and the GPU
            assert workloads.rel_rms_err(got, want).max() < 1e-3
    finally:
        R.dropin_unload()
