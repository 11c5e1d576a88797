"""Expert parallelism over peer memory (tie_cuda_ep_*): G ranks emulated on ONE GPU as G contexts
of this process that share a stream.  Their kernels wait on one another's flags, so the phases
are enqueued rank by rank (all publishes, all computes, all gathers): every wait is already
satisfied when its kernel runs, nothing ever spins on work that is queued behind it.

The result must equal the single-context block on the concatenated tokens (same kernels, same
arithmetic per row) and stay within the parity bound of the CPU restatement.
"""
import numpy as np
import pytest

from tie_b200 import synth, workloads

pytestmark = pytest.mark.gpu

TOL = 1e-3


_streams = []


def _ranks(shape, layer_seed, G, t_max, silu):
    import torch
    from tie_b200 import moe
    n_local = shape.n_expert // G
    bes = []
    stream = torch.cuda.Stream()  # ONE stream for all emulated ranks: their kernels run in enqueue order
    _streams.append(stream)
    for r in range(G):
        b = moe.MoeBackend(hidden=shape.hidden, n_expert=shape.n_expert, top_k=shape.top_k, ffn_dim=shape.ffn_dim,
                           max_tokens=t_max * G, silu_table=silu, ep_rank=r, ep_size=G)
        b.upload_layer(0, synth.make_layer(layer_seed, shape, first_expert=r * n_local, n_local_expert=n_local))
        b.set_stream(stream.cuda_stream)
        bes.append(b)
    bases = [b.ep_region()[0] for b in bes]
    for b in bes:
        b.ep_attach(bases, moe.EP_PEER_POINTERS)
        b.ep_set_timeout_ms(200)
    return bes


def _step(bes, xs, outs, residuals=None):
    from tie_b200 import moe
    fl = moe.DEVICE | moe.NO_SYNC
    for b, x in zip(bes, xs):
        b.ep_publish_ptr(0, x if x.shape[0] else None, x.shape[0], None, fl)
    for b in bes:
        b.ep_compute(0, fl)
    for i, (b, o) in enumerate(zip(bes, outs)):
        b.ep_gather_ptr(o if o.shape[0] else None, None if residuals is None else residuals[i], fl)
    for b in bes:
        b.synchronize()


@pytest.mark.parametrize("G,tokens", [(1, [48]), (2, [40, 23]), (4, [17, 0, 64, 5]), (8, [9, 31, 1, 0, 12, 64, 7, 20])])
def test_emulated_ranks_small_shape(small_shape, small_layer, ref_silu_table, port_lib, G, tokens):
    import torch
    from tie_b200 import moe
    shape = small_shape
    seed = workloads.BASE_SEED + 1
    bes = _ranks(shape, seed, G, 64, ref_silu_table)
    one = moe.MoeBackend(hidden=shape.hidden, n_expert=shape.n_expert, top_k=shape.top_k, ffn_dim=shape.ffn_dim, max_tokens=256,
                         silu_table=ref_silu_table)
    try:
        one.upload_layer(0, small_layer)
        P = port_lib.PortMoe(small_layer, silu=ref_silu_table)
        for step in range(3):  # the regions and flags are re-used step after step
            first = 1000 * step
            xh = [synth.make_x(7, n, shape.hidden, first_token=first + 100 * r) for r, n in enumerate(tokens)]
            xs = [torch.from_numpy(x).cuda() for x in xh]
            outs = [torch.full_like(x, float("nan")) for x in xs]
            _step(bes, xs, outs)
            x_all = np.concatenate(xh)
            xa = torch.from_numpy(x_all).cuda()
            oa = torch.empty_like(xa)
            one.moe_ffn_ptr(0, xa, oa, x_all.shape[0], moe.DEVICE | moe.PATH_TENSOR)
            got = np.concatenate([o.cpu().numpy() for o in outs])
            assert np.isfinite(got).all()
            # the same kernels computed every row: identical up to the grouping of rows into tiles
            assert workloads.rel_rms_err(got, oa.cpu().numpy()).max() < 2e-5
            ref, _, _ = P.moe_ffn(x_all)
            assert workloads.rel_rms_err(got, ref).max() < TOL
        assert sum(b.last_active_experts() for b in bes) <= shape.n_expert
    finally:
        for b in bes:
            b.close()
        one.close()


def test_emulated_ranks_block_shape_with_residual(layer0, port0_ep, ref_silu_table):
    import torch
    shape = layer0.shape
    G, tokens = 2, [96, 64]
    bes = _ranks(shape, workloads.BASE_SEED, G, 128, ref_silu_table)
    try:
        xh = [synth.make_x(workloads.BASE_SEED, n, shape.hidden, first_token=200 * r) for r, n in enumerate(tokens)]
        xs = [torch.from_numpy(x).cuda() for x in xh]
        res = [torch.from_numpy(np.full_like(x, 0.5)).cuda() for x in xh]
        outs = [torch.empty_like(x) for x in xs]
        _step(bes, xs, outs, res)
        x_all = np.concatenate(xh)
        ref, _, _ = port0_ep.moe_ffn(x_all)
        got = np.concatenate([o.cpu().numpy() for o in outs])
        assert workloads.rel_rms_err(got - 0.5, ref).max() < TOL
    finally:
        for b in bes:
            b.close()


@pytest.fixture(scope="module")
def port0_ep(port_lib, layer0, ref_silu_table):
    return port_lib.PortMoe(layer0, silu=ref_silu_table)


def test_absent_rank_times_out_and_reports(small_shape, ref_silu_table):
    """A rank that never publishes: the others' waits run out (a flag nothing sets), the status
    word carries the time-out, the call returns an error code and the context stays usable."""
    import torch
    from tie_b200 import moe
    shape = small_shape
    bes = _ranks(shape, workloads.BASE_SEED + 1, 2, 64, ref_silu_table)
    try:
        b = bes[0]
        b.ep_set_timeout_ms(50)
        x = torch.from_numpy(synth.make_x(3, 8, shape.hidden)).cuda()
        out = torch.zeros_like(x)
        b.ep_publish_ptr(0, x, 8, None, moe.DEVICE | moe.NO_SYNC)
        with pytest.raises(moe.TieCudaError) as ei:
            b.ep_compute(0, moe.DEVICE)  # rank 1 has not published
        assert ei.value.code == moe.EKERNEL
        with pytest.raises(moe.TieCudaError):
            b.ep_gather_ptr(out, None, moe.DEVICE)  # rank 1 has not computed either
        # the context still serves other calls
        idx = torch.empty(8, shape.top_k, dtype=torch.int32, device="cuda")
        w = torch.empty(8, shape.top_k, dtype=torch.float32, device="cuda")
        b.route_ptr(0, x, 8, idx, w, None, None, moe.DEVICE)
        assert int(idx.min()) >= 0
    finally:
        for b in bes:
            b.close()


def test_group_recovers_after_a_time_out_by_detach_and_attach(small_shape, small_layer, ref_silu_table, port_lib):
    """After an absent-rank time-out the ranks' step numbers differ (rank 0 published, rank 1 did
    not) and rank 0's flags are stale.  Detach + attach on every rank starts a new epoch: the next
    step is correct, on both ranks, and so is the one after it."""
    import torch
    from tie_b200 import moe
    shape = small_shape
    bes = _ranks(shape, workloads.BASE_SEED + 1, 2, 64, ref_silu_table)
    try:
        # one good step, so that flags and counters are non-zero before the failure
        xh = [synth.make_x(5, n, shape.hidden, first_token=10 * r) for r, n in enumerate([12, 7])]
        xs = [torch.from_numpy(x).cuda() for x in xh]
        outs = [torch.empty_like(x) for x in xs]
        _step(bes, xs, outs)
        bes[0].ep_set_timeout_ms(50)
        bes[0].ep_publish_ptr(0, xs[0], 12, None, moe.DEVICE | moe.NO_SYNC)
        with pytest.raises(moe.TieCudaError) as ei:
            bes[0].ep_compute(0, moe.DEVICE)  # rank 1 never published this step
        assert ei.value.code == moe.EKERNEL
        # recovery as the header prescribes: all detach, (host barrier), all attach, (host barrier)
        for b in bes:
            b.ep_detach()
        bases = [b.ep_region()[0] for b in bes]
        for b in bes:
            b.ep_attach(bases, moe.EP_PEER_POINTERS)
            b.ep_set_timeout_ms(200)
        P = port_lib.PortMoe(small_layer, silu=ref_silu_table)
        for step in range(2):
            xh = [synth.make_x(6 + step, n, shape.hidden, first_token=10 * r) for r, n in enumerate([9, 20])]
            xs = [torch.from_numpy(x).cuda() for x in xh]
            outs = [torch.full_like(x, float("nan")) for x in xs]
            _step(bes, xs, outs)
            ref, _, _ = P.moe_ffn(np.concatenate(xh))
            got = np.concatenate([o.cpu().numpy() for o in outs])
            assert np.isfinite(got).all()
            assert workloads.rel_rms_err(got, ref).max() < TOL
    finally:
        for b in bes:
            b.close()


def _decode_step(bes, x, outs, residual=None):
    """One decode step on replicated tokens, phases enqueued rank by rank (the ranks share a GPU)."""
    from tie_b200 import moe
    fl = moe.DEVICE | moe.NO_SYNC
    n = x.shape[0]
    for b in bes:
        b.ep_publish_ptr(0, x, n, None, fl | moe.EP_REPLICATED)
    for b in bes:
        b.ep_compute(0, fl)
    for b, o in zip(bes, outs):
        b.ep_gather_ptr(o, residual, fl)
    for b in bes:
        b.synchronize()


@pytest.mark.parametrize("G", [1, 2, 4, 8])
@pytest.mark.parametrize("n_tokens", [1, 3])
def test_replicated_decode_emulated_ranks(layer0, port0_ep, ref_silu_table, G, n_tokens):
    """Expert-parallel decode (TIE_CUDA_EP_REPLICATED) of the Qwen3-30B-A3B-shaped block: every rank
    gets the same rows and must end with the same complete outputs — bit-identical to the one-GPU
    decode kernels (same per-slot products, combined in the same slot order) and within the parity
    bound of the CPU restatement.  Three steps over the same regions; prefill steps in between use
    the same flags."""
    import torch
    from tie_b200 import moe
    shape = layer0.shape
    bes = _ranks(shape, workloads.BASE_SEED, G, 8, ref_silu_table)
    one = moe.MoeBackend(max_tokens=8, silu_table=ref_silu_table)
    try:
        one.upload_layer(0, layer0)
        for step in range(3):
            xh = synth.make_x(workloads.BASE_SEED, n_tokens, shape.hidden, first_token=17 * step)
            x = torch.from_numpy(xh).cuda()
            outs = [torch.full_like(x, float("nan")) for _ in bes]
            res = torch.full_like(x, 0.25) if step == 1 else None
            _decode_step(bes, x, outs, res)
            want = torch.empty_like(x)
            one.moe_ffn_ptr(0, x, want, n_tokens, moe.DEVICE | moe.PATH_DECODE_CHAIN)
            w = want.cpu().numpy() + (0.25 if step == 1 else 0.0)
            ref, _, _ = port0_ep.moe_ffn(xh)
            for o in outs:
                got = o.cpu().numpy()
                if step != 1:
                    assert np.array_equal(got.view(np.uint32), w.astype(np.float32).view(np.uint32))
                assert workloads.rel_rms_err(got - (0.25 if step == 1 else 0.0), ref).max() < TOL
            if step == 0 and G > 1:  # a prefill-form step between decode steps
                xs = [torch.from_numpy(synth.make_x(9, 5, shape.hidden, first_token=10 * r)).cuda() for r in range(G)]
                po = [torch.empty_like(t) for t in xs]
                _step(bes, xs, po)
    finally:
        for b in bes:
            b.close()
        one.close()


def test_phase_order_is_checked(small_shape, ref_silu_table):
    from tie_b200 import moe
    bes = _ranks(small_shape, workloads.BASE_SEED + 1, 1, 64, ref_silu_table)
    try:
        with pytest.raises(moe.TieCudaError) as ei:
            bes[0].ep_compute(0, moe.DEVICE)
        assert ei.value.code == moe.EINVAL
        with pytest.raises(moe.TieCudaError):
            bes[0].ep_gather_ptr(None, None, moe.DEVICE)
    finally:
        bes[0].close()


def test_whole_step_replayed_from_a_graph(small_shape, small_layer, ref_silu_table):
    """tie_cuda_moe_ffn_ep with TIE_CUDA_GRAPH on a group of one rank: the step number advances on
    the device, so the replayed launches keep working step after step, with x in the region."""
    import torch
    from tie_b200 import moe
    shape = small_shape
    bes = _ranks(shape, workloads.BASE_SEED + 1, 1, 64, ref_silu_table)
    one = moe.MoeBackend(hidden=shape.hidden, n_expert=shape.n_expert, top_k=shape.top_k, ffn_dim=shape.ffn_dim, max_tokens=64,
                         silu_table=ref_silu_table)
    try:
        one.upload_layer(0, small_layer)
        b = bes[0]
        x = torch.empty(40, shape.hidden, device="cuda")
        out = torch.empty_like(x)
        ref = torch.empty_like(x)
        launches = []
        for step in range(4):
            x.copy_(torch.from_numpy(synth.make_x(11, 40, shape.hidden, first_token=50 * step)))
            torch.cuda.synchronize()
            l0 = b.launch_count
            b.moe_ffn_ep_ptr(0, x, out, 40, moe.DEVICE | moe.GRAPH)
            launches.append(b.launch_count - l0)
            one.moe_ffn_ptr(0, x, ref, 40, moe.DEVICE | moe.PATH_TENSOR)
            assert workloads.rel_rms_err(out.cpu().numpy(), ref.cpu().numpy()).max() < 2e-5
        assert len(set(launches)) == 1 and launches[0] >= 10
    finally:
        bes[0].close()
        one.close()


def test_block_inplace_ep_one_rank_group(small_shape, small_layer, ref_silu_table):
    """hidden += MoE(RMSNorm(hidden)) through tie_cuda_moe_block_inplace_ep (one call, one graph per
    step; the normed tokens are written straight into the region) on a group of one rank equals
    tie_cuda_moe_block_inplace.  (Ranks that share one GPU must interleave their phases, so larger
    groups of this one-call entry point are tested on separate GPUs.)"""
    import torch
    from tie_b200 import moe
    shape = small_shape
    norm_w = (1.0 + 0.1 * np.cos(np.arange(shape.hidden))).astype(np.float32)
    solo = _ranks(shape, workloads.BASE_SEED + 1, 1, 64, ref_silu_table)
    one = moe.MoeBackend(hidden=shape.hidden, n_expert=shape.n_expert, top_k=shape.top_k, ffn_dim=shape.ffn_dim, max_tokens=64,
                         silu_table=ref_silu_table)
    try:
        solo[0].upload_layer(0, small_layer, ffn_norm_w=norm_w)
        one.upload_layer(0, small_layer, ffn_norm_w=norm_w)
        got = torch.empty(64, shape.hidden, device="cuda")
        for step in range(3):  # the later passes replay the graph
            h0 = torch.from_numpy(synth.make_x(31 + step, 64, shape.hidden)).cuda()
            want = h0.clone()
            one.moe_block_inplace_ptr(0, want, 64, moe.DEVICE | moe.PATH_TENSOR)
            got.copy_(h0)
            torch.cuda.synchronize()
            solo[0].moe_block_inplace_ep_ptr(0, got, 64, moe.DEVICE | moe.GRAPH)
            assert workloads.rel_rms_err(got.cpu().numpy(), want.cpu().numpy()).max() < 2e-5
    finally:
        solo[0].close()
        one.close()
