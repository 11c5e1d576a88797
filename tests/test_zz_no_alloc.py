"""GPU test of tie_cuda_route_noalloc, the routing entry point for callers that must not
allocate (a serving loop that bans allocator calls after start-up, an application with a fixed
memory budget).  Its logits scratch is a fixed array inside the library, so the test checks the
things a user of it relies on: it gives the same answer as the context-based tie_cuda_moe_route
and as the CPU restatement of the reference's router, it keeps doing so on a second call that
finds the first call's data still in the scratch, and a misaligned pointer is refused on the
host instead of faulting on the device.

Collected last on purpose (file name), and self-contained: it passes alone in a fresh process
and after every other test."""
import ctypes

import numpy as np
import pytest

from tie_b200 import synth, workloads

pytestmark = pytest.mark.gpu


def _route_noalloc(L, x, router, bias, n_tokens, hidden, n_expert, top_k, torch):
    idx = torch.full((n_tokens, top_k), -7, dtype=torch.int32, device="cuda")
    w = torch.full((n_tokens, top_k), float("nan"), dtype=torch.float32, device="cuda")
    rc = L.tie_cuda_route_noalloc(x.data_ptr(), router.data_ptr(), None if bias is None else bias.data_ptr(), n_tokens,
                                  hidden, n_expert, top_k, idx.data_ptr(), w.data_ptr(),
                                  torch.cuda.current_stream().cuda_stream)
    assert rc == 0, L.tie_cuda_strerror(rc)
    torch.cuda.synchronize()
    return idx.cpu().numpy(), w.cpu().numpy()


def test_route_noalloc_matches_context_route_on_two_calls_in_a_row(layer0, ref_silu_table, port_lib):
    import torch
    from tie_b200 import moe
    L = moe.load_library()
    s = layer0.shape
    be = moe.MoeBackend(max_tokens=64, silu_table=ref_silu_table)
    oracle = port_lib.PortMoe(layer0, silu=ref_silu_table)
    try:
        be.upload_layer(0, layer0)
        router = torch.from_numpy(layer0.router_w).cuda()
        # first call: 64 tokens fill the whole scratch; second call: 5 tokens of other data (and a
        # bias) must not be disturbed by what the first call left behind; third: 1 token.
        cases = [(64, 0, None), (5, 900, synth.zipf_logp(s.n_expert, 3)[0]), (1, 77, None)]
        for n_tokens, first, bias in cases:
            x = synth.make_x(workloads.BASE_SEED, n_tokens, first_token=first)
            want_idx, want_w, _ = be.route(0, x, router_bias=bias)
            bd = None if bias is None else torch.from_numpy(bias).cuda()
            got_idx, got_w = _route_noalloc(L, torch.from_numpy(x).cuda(), router, bd, n_tokens, s.hidden, s.n_expert,
                                            s.top_k, torch)
            assert np.array_equal(got_idx, want_idx)
            assert np.abs(got_w - want_w).max() <= 2e-7  # the tolerance the router tests use for gate weights
            # and directly against the CPU restatement of the reference's router (find_top_k + softmax)
            ref_idx, ref_w, _ = oracle.route(x, bias)
            assert np.array_equal(got_idx, ref_idx)
            assert np.abs(got_w - ref_w).max() <= 2e-7
    finally:
        be.close()


def test_route_noalloc_rejects_sizes_beyond_its_scratch(layer0):
    import torch
    from tie_b200 import moe
    L = moe.load_library()
    x = torch.zeros(65, 2048, device="cuda")
    router = torch.zeros(128, 2048, device="cuda")
    idx = torch.zeros(65, 8, dtype=torch.int32, device="cuda")
    w = torch.zeros(65, 8, device="cuda")
    rc = L.tie_cuda_route_noalloc(x.data_ptr(), router.data_ptr(), None, 65, 2048, 128, 8, idx.data_ptr(), w.data_ptr(), None)
    assert rc == moe.ETOOBIG and b"64" in L.tie_cuda_strerror(rc)
    rc = L.tie_cuda_route_noalloc(x.data_ptr(), router.data_ptr(), None, 4, 2048, 512, 8, idx.data_ptr(), w.data_ptr(), None)
    assert rc == moe.ETOOBIG
    rc = L.tie_cuda_route_noalloc(None, router.data_ptr(), None, 4, 2048, 128, 8, idx.data_ptr(), w.data_ptr(), None)
    assert rc == moe.EINVAL
    # x / router one float off a 16-byte boundary: refused on the host (the kernels load 128 bits at a time)
    rc = L.tie_cuda_route_noalloc(x.data_ptr() + 4, router.data_ptr(), None, 4, 2048, 128, 8, idx.data_ptr(), w.data_ptr(), None)
    assert rc == moe.EINVAL
    rc = L.tie_cuda_route_noalloc(x.data_ptr(), router.data_ptr() + 8, None, 4, 2048, 128, 8, idx.data_ptr(), w.data_ptr(), None)
    assert rc == moe.EINVAL
    torch.cuda.synchronize()
