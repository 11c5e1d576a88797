"""GPU parity tests: every call goes through the C ABI (tie_b200.moe -> libtie_cuda.so) and is
checked against the CPU restatement (oracle/) and against the golden vectors produced by the
reference's own compiled code.

Parity bound of this path: top-k expert ids identical, in order; outputs within 1e-3 per token,
measured as max_k |gpu - ref| / rms_k(ref) (fp32 accumulation on both sides).
"""
import numpy as np
import pytest

from tie_b200 import synth, workloads

pytestmark = pytest.mark.gpu

TOL = 1e-3


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


@pytest.fixture(scope="module")
def be(layer0, ref_silu_table):
    from tie_b200 import moe
    b = moe.MoeBackend(max_tokens=512, silu_table=ref_silu_table, n_layers=2)
    b.upload_layer(0, layer0, keep_host=True)
    yield b
    b.close()


@pytest.fixture(scope="module")
def port0(port_lib, layer0, ref_silu_table):
    return port_lib.PortMoe(layer0, silu=ref_silu_table)


@pytest.fixture(scope="module")
def be_small(small_layer, small_shape, ref_silu_table):
    from tie_b200 import moe
    s = small_shape
    b = moe.MoeBackend(hidden=s.hidden, n_expert=s.n_expert, top_k=s.top_k, ffn_dim=s.ffn_dim, max_tokens=256,
                       silu_table=ref_silu_table)
    b.upload_layer(0, small_layer, keep_host=True)
    yield b
    b.close()


# ---------------- router: bit-exact ----------------

def test_route_bit_exact_thousands_of_tokens(layer0, port0, ref_silu_table):
    """From 2048 tokens on the batched router uses its 8 x 8 register-tile variant; ragged count."""
    from tie_b200 import moe
    n = 2048 + 37
    x = synth.make_x(3, n)
    ref_idx, ref_w, ref_logits = port0.route(x)
    b = moe.MoeBackend(max_tokens=n, silu_table=ref_silu_table)
    try:
        b.upload_layer(0, layer0)
        idx, w, logits = b.route(0, x)
    finally:
        b.close()
    assert np.array_equal(logits.view(np.uint32), ref_logits.view(np.uint32))
    assert np.array_equal(idx, ref_idx)
    assert np.max(np.abs(w - ref_w)) < 2e-7


@pytest.mark.parametrize("n_tokens", [1, 3, 8, 9, 64, 512])
def test_route_bit_exact(be, port0, n_tokens):
    x = synth.make_x(0, n_tokens)
    idx, w, logits = be.route(0, x)
    i_r, w_r, l_r = port0.route(x)
    assert np.array_equal(bits(logits), bits(l_r)), "router logits must replay the AVX2 summation order bit for bit"
    assert np.array_equal(idx, i_r)
    assert np.abs(w - w_r).max() <= 2e-7  # expf: CUDA vs glibc, <= 2 ulp of values <= 1


def test_route_golden_and_bias(be, golden):
    g = golden("decode1.npz")
    idx, w, logits = be.route(0, synth.make_x(0, 1))
    assert np.array_equal(bits(logits), bits(g["logits"])) and np.array_equal(idx, g["idx"])
    gs = golden("batch64_skew.npz")
    idx, w, _ = be.route(0, synth.make_x(0, 64), router_bias=gs["bias"])
    assert np.array_equal(idx, gs["idx"])
    assert np.abs(w - gs["w"]).max() <= 2e-7


def test_route_tie_rule(be_small, small_shape):
    """Exact ties resolve to the lower expert id (find_top_k uses strict '>')."""
    s = small_shape
    x = np.zeros((2, s.hidden), dtype=np.float32)  # all logits 0 -> all tied
    bias = np.zeros(s.n_expert, dtype=np.float32)
    bias[[5, 17]] = 1.0
    idx, w, logits = be_small.route(0, x, router_bias=bias)
    assert idx[0].tolist() == [5, 17, 0, 1] and idx[1].tolist() == [5, 17, 0, 1]
    assert abs(w[0].sum() - 1.0) < 1e-6


# ---------------- the MoE feed-forward call ----------------

def _check_ffn(out, ref_out, tol=TOL):
    err = workloads.rel_rms_err(out, ref_out)
    assert np.isfinite(out).all()
    assert err.max() <= tol, f"max rel-rms error {err.max():.3e} at token {int(err.argmax())}"
    return float(err.max())


def test_decode1_matches_reference_golden(be, golden):
    from tie_b200 import moe
    g = golden("decode1.npz")
    out = be.moe_ffn(0, synth.make_x(0, 1))
    e = _check_ffn(out, g["out"])
    assert e < 1e-5  # fp32 CUDA-core path: summation-order noise only
    assert be.last_active_experts() == 8


@pytest.mark.parametrize("n_tokens", [2, 3, 4, 5])
def test_few_tokens_decode_kernels_and_general_streaming_kernels(be, port0, n_tokens):
    """1-4 tokens take the bulk-staged decode kernels; the same inputs through the general
    streaming kernels and through 5 tokens (first size past the decode path) must agree too."""
    from tie_b200 import moe
    x = synth.make_x(0, n_tokens, first_token=40)
    ref_out, _, _ = port0.moe_ffn(x)
    e = _check_ffn(be.moe_ffn(0, x), ref_out)
    assert e < 1e-5
    _check_ffn(be.moe_ffn(0, x, path=moe.PATH_STREAM | moe.PATH_LEGACY_STREAM), ref_out, tol=1e-5)


def _path_flags(path):
    """stream: CUDA-core streaming kernels; tensor: the grouped GEMM as CTA pairs (the default where
    the 128-row tiles pair up); tensor_single: one CTA per 128-row tile."""
    from tie_b200 import moe
    return {"stream": moe.PATH_STREAM, "tensor": moe.PATH_TENSOR, "tensor_single": moe.PATH_TENSOR | moe.PATH_NO_PAIR}[path]


@pytest.mark.parametrize("path", ["stream", "tensor", "tensor_single"])
def test_batch64_uniform_and_skewed(be, golden, port0, path):
    p = _path_flags(path)
    x = synth.make_x(0, 64)
    ref_out, _, _ = port0.moe_ffn(x)
    g = golden("batch64.npz")
    assert np.array_equal(bits(ref_out[g["rows"]]), bits(g["out_rows"]))  # restatement == reference
    out = be.moe_ffn(0, x, path=p)
    _check_ffn(out, ref_out)
    gs = golden("batch64_skew.npz")
    ref_s, _, _ = port0.moe_ffn(x, router_bias=gs["bias"])
    out_s = be.moe_ffn(0, x, router_bias=gs["bias"], path=p)
    _check_ffn(out_s, ref_s)
    _check_ffn(out_s[gs["rows"]], gs["out_rows"])


@pytest.mark.parametrize("path", ["tensor", "tensor_single", "stream"])
def test_prefill512(be, golden, port0, path):
    p = _path_flags(path)
    x = synth.make_x(0, 512)
    g = golden("prefill512.npz")
    out = be.moe_ffn(0, x, path=p)
    _check_ffn(out[g["rows"]], g["out_rows"])
    rms = np.sqrt((out.astype(np.float64) ** 2).mean(1))
    assert np.abs(rms / g["rms"] - 1).max() < 1e-4  # every token, via the golden per-token rms
    ref_out, _, _ = port0.moe_ffn(x)
    _check_ffn(out, ref_out)


def test_one_kernel_decode_equals_the_three_kernel_chain(be, be_small, small_shape, port0):
    """One token: the cooperative single-kernel step (default) and the chain of three decode
    kernels run the same per-lane arithmetic in the same order: identical bits, launch counts 1 / 3,
    also when replayed from a graph many times (the grid barriers' epoch advances on the device)."""
    import torch
    from tie_b200 import moe
    for b, hidden, seed in ((be, 2048, 21), (be_small, small_shape.hidden, 22)):
        for rep in range(3):
            x = torch.from_numpy(synth.make_x(seed + rep, 1, hidden)).cuda()
            o1, o3 = torch.empty_like(x), torch.empty_like(x)
            l0 = b.launch_count
            b.moe_ffn_ptr(0, x, o1, 1, moe.DEVICE)
            l1 = b.launch_count
            b.moe_ffn_ptr(0, x, o3, 1, moe.DEVICE | moe.PATH_DECODE_CHAIN)
            l3 = b.launch_count
            assert (l1 - l0, l3 - l1) == (1, 3)
            assert np.array_equal(bits(o1.cpu().numpy()), bits(o3.cpu().numpy()))
            for _ in range(5):
                og = torch.zeros_like(x)
                b.moe_ffn_ptr(0, x, og, 1, moe.DEVICE | moe.GRAPH)
                assert np.array_equal(bits(og.cpu().numpy()), bits(o1.cpu().numpy()))
    x = synth.make_x(23, 1)
    ref, _, _ = port0.moe_ffn(x)
    assert workloads.rel_rms_err(be.moe_ffn(0, x), ref).max() < TOL  # host pointers, default (one-kernel) path


def test_auto_path_and_determinism(be):
    x = synth.make_x(0, 512)
    a = be.moe_ffn(0, x)
    b = be.moe_ffn(0, x)
    assert np.array_equal(bits(a), bits(b)), "two runs must be bit-identical (no atomics on the data path)"


@pytest.mark.parametrize("n_tokens", [2, 5, 17, 33, 130])
def test_ragged_token_counts_small_shape(be_small, small_layer, small_shape, port_lib, ref_silu_table, n_tokens):
    from tie_b200 import moe
    P = port_lib.PortMoe(small_layer, silu=ref_silu_table)
    x = synth.make_x(workloads.BASE_SEED + 1, n_tokens, small_shape.hidden)
    ref_out, _, _ = P.moe_ffn(x)
    for p in (moe.PATH_STREAM, moe.PATH_TENSOR, moe.PATH_AUTO):
        _check_ffn(be_small.moe_ffn(0, x, path=p), ref_out)


def test_small_shape_golden(be_small, small_shape, golden):
    g = golden("small.npz")
    x = synth.make_x(workloads.BASE_SEED + 1, 24, small_shape.hidden)
    idx, w, logits = be_small.route(0, x)
    assert np.array_equal(bits(logits), bits(g["logits"])) and np.array_equal(idx, g["idx"])
    _check_ffn(be_small.moe_ffn(0, x), g["out"])


def test_all_tokens_to_the_same_experts(be_small, small_layer, small_shape, port_lib, ref_silu_table):
    """Maximum imbalance: a large bias sends every token to the same top-k experts (most experts
    receive nothing, a few receive every row — more than one token tile)."""
    from tie_b200 import moe
    s = small_shape
    bias = np.zeros(s.n_expert, dtype=np.float32)
    bias[[2, 3, 11, 30]] = 100.0
    x = synth.make_x(workloads.BASE_SEED + 1, 200, s.hidden)
    P = port_lib.PortMoe(small_layer, silu=ref_silu_table)
    ref_out, idx, _ = P.moe_ffn(x, router_bias=bias)
    assert set(np.unique(idx).tolist()) == {2, 3, 11, 30}
    for p in (moe.PATH_STREAM, moe.PATH_TENSOR):
        _check_ffn(be_small.moe_ffn(0, x, router_bias=bias, path=p), ref_out)
        assert be_small.last_active_experts() == 4


def test_down_tensor_as_q4k_and_gate_up_as_q6k(small_shape, ref_silu_table, port_lib):
    """Real Q4_K_M files mix types per tensor; any of the three may be Q4_K or Q6_K."""
    from tie_b200 import moe
    s = small_shape
    seed = 99
    gu_blocks = s.ffn_dim * (s.hidden // 256)
    dn_blocks = s.hidden * (s.ffn_dim // 256)
    router = synth.normal_f32(seed, synth.STREAM_ROUTER, s.n_expert * s.hidden, 0.02).reshape(s.n_expert, s.hidden)
    layer = synth.MoeLayer(s, router,
                           synth.q6k_blocks(seed, synth.STREAM_GATE, s.n_expert * gu_blocks),
                           synth.q6k_blocks(seed, synth.STREAM_UP, s.n_expert * gu_blocks),
                           synth.q4k_blocks(seed, synth.STREAM_DOWN, s.n_expert * dn_blocks),
                           gate_type=synth.GGML_Q6_K, up_type=synth.GGML_Q6_K, down_type=synth.GGML_Q4_K)
    P = port_lib.PortMoe(layer, silu=ref_silu_table)
    x = synth.make_x(seed, 40, s.hidden)
    ref_out, _, _ = P.moe_ffn(x)
    b = moe.MoeBackend(hidden=s.hidden, n_expert=s.n_expert, top_k=s.top_k, ffn_dim=s.ffn_dim, max_tokens=64,
                       silu_table=ref_silu_table)
    try:
        b.upload_layer(0, layer)
        for p in (moe.PATH_STREAM, moe.PATH_TENSOR):
            _check_ffn(b.moe_ffn(0, x, path=p), ref_out)
        # the decode kernels with these kinds: one token (the one-kernel step, then the chain), three tokens
        l0 = b.launch_count
        one = b.moe_ffn(0, x[:1])
        assert b.launch_count - l0 == 1
        _check_ffn(one, ref_out[:1])
        _check_ffn(b.moe_ffn(0, x[:1], path=moe.PATH_DECODE_CHAIN), ref_out[:1])
        _check_ffn(b.moe_ffn(0, x[:3]), ref_out[:3])
    finally:
        b.close()


def test_tensor_path_odd_block_counts_and_all_tile_sizes(ref_silu_table, port_lib):
    """Q4_K tensors with an odd number of super-blocks per row (3 and 1: the min phase pads its last
    16-deep k step with zeros and one producer group has no block), token tiles of all three box
    sizes (<= 16, <= 32, <= 64 rows) and an expert with more than one tile."""
    from tie_b200 import moe
    s = synth.MoeShape(hidden=768, n_expert=32, top_k=4, ffn_dim=256)
    seed = 321
    gu_blocks = s.ffn_dim * (s.hidden // 256)
    dn_blocks = s.hidden * (s.ffn_dim // 256)
    router = synth.normal_f32(seed, synth.STREAM_ROUTER, s.n_expert * s.hidden, 0.02).reshape(s.n_expert, s.hidden)
    layer = synth.MoeLayer(s, router,
                           synth.q4k_blocks(seed, synth.STREAM_GATE, s.n_expert * gu_blocks),
                           synth.q4k_blocks(seed, synth.STREAM_UP, s.n_expert * gu_blocks),
                           synth.q4k_blocks(seed, synth.STREAM_DOWN, s.n_expert * dn_blocks),
                           gate_type=synth.GGML_Q4_K, up_type=synth.GGML_Q4_K, down_type=synth.GGML_Q4_K)
    P = port_lib.PortMoe(layer, silu=ref_silu_table)
    T = 200
    x = synth.make_x(seed, T, s.hidden)
    bias = np.zeros(s.n_expert, np.float32)
    bias[5] = 3.0   # most tokens pick expert 5: more than 64 rows -> several tiles
    bias[9] = 0.4
    ref_out, idx, _ = P.moe_ffn(x, router_bias=bias)
    counts = np.bincount(idx.ravel(), minlength=s.n_expert)
    assert counts.max() > 64 and (counts <= 16).any() and ((counts > 16) & (counts <= 32)).any()
    b = moe.MoeBackend(hidden=s.hidden, n_expert=s.n_expert, top_k=s.top_k, ffn_dim=s.ffn_dim, max_tokens=256,
                       silu_table=ref_silu_table)
    try:
        b.upload_layer(0, layer)
        for p in (moe.PATH_STREAM, moe.PATH_TENSOR, moe.PATH_TENSOR | moe.PATH_NO_PAIR):
            _check_ffn(b.moe_ffn(0, x, router_bias=bias, path=p), ref_out)
    finally:
        b.close()


def test_upload_from_gguf_file(tmp_path, small_shape, ref_silu_table, port_lib):
    """Weights read from a GGUF file (mixed Q6_K / Q4_K down tensors per block) and uploaded from
    the mapping give the same outputs as the oracle on the generated arrays."""
    from tie_b200 import gguf, moe
    from test_gguf import moe_model, write_gguf
    kvs, tensors, layers = moe_model(small_shape, 2, seed=55, down_types=[synth.GGML_Q6_K, synth.GGML_Q4_K])
    path = str(tmp_path / "model.gguf")
    write_gguf(path, kvs, tensors)
    x = synth.make_x(55, 48, small_shape.hidden)
    with gguf.GgufFile(path) as g:
        cfg = g.moe_config()
        b = moe.MoeBackend(hidden=cfg["hidden"], n_expert=cfg["n_expert"], top_k=cfg["top_k"], ffn_dim=cfg["ffn_dim"],
                           n_layers=cfg["n_layers"], max_tokens=64, silu_table=ref_silu_table)
        try:
            assert gguf.upload_model(b, g) == 2
        finally:
            pass
    # the mapping is gone: the device copies are what the calls use
    try:
        for i, layer in enumerate(layers):
            ref_out, _, _ = port_lib.PortMoe(layer, silu=ref_silu_table).moe_ffn(x)
            for p in (moe.PATH_STREAM, moe.PATH_TENSOR):
                _check_ffn(b.moe_ffn(i, x, path=p), ref_out)
    finally:
        b.close()


def test_lfm2_routing_and_block(be, layer0, ref_silu_table, port_lib, golden):
    """The second caller of the expert kernels (model_lfm2.c:414-498): sigmoid routing with a
    selection bias and L1-normalised gates.  Selected experts identical to the compiled
    reference's (fixture), gates to 1e-6 (CUDA expf vs glibc, -ffast-math reciprocals in the
    reference), block outputs within the 1e-3 bound against the restatement."""
    from tie_b200 import moe
    g = golden("lfm2_route.npz")
    x = synth.make_x(0, 64)
    for bias, gi, gw in ((None, g["idx"], g["w"]), (g["bias"], g["idx_b"], g["w_b"])):
        idx, w, scores = be.route(0, x, router_bias=bias, lfm2=True)
        assert np.array_equal(idx, gi)
        assert np.max(np.abs(w - gw) / gw) < 2e-6
        assert np.max(np.abs(scores - g["scores"])) < 1e-6
    P = port_lib.PortMoe(layer0, silu=ref_silu_table)
    for T in (3, 64):
        ref_out, ref_idx, _ = P.moe_ffn_lfm2(x[:T], g["bias"])
        assert np.array_equal(ref_idx, g["idx_b"][:T])
        for p in ((moe.PATH_AUTO, moe.PATH_STREAM) if T == 3 else (moe.PATH_STREAM, moe.PATH_TENSOR)):
            _check_ffn(be.moe_ffn(0, x[:T], router_bias=g["bias"], path=p, lfm2=True), ref_out)


def test_prefill_4096_tokens_sampled_rows(layer0, port0, ref_silu_table):
    """The largest single-GPU configuration: every expert has several token tiles and a CTA of the
    grouped GEMM walks more work items than it stages in shared memory.  The reference path is per
    token, so a sample of rows is checked against the restatement run on those tokens alone."""
    from tie_b200 import moe
    T = 4096
    x = synth.make_x(11, T)
    rows = np.array([0, 1, 63, 64, 65, 511, 512, 1000, 2047, 2048, 3000, 4094, 4095])
    ref_out, _, _ = port0.moe_ffn(x[rows])
    b = moe.MoeBackend(max_tokens=T, silu_table=ref_silu_table)
    try:
        b.upload_layer(0, layer0)
        out = b.moe_ffn(0, x, path=moe.PATH_TENSOR)
    finally:
        b.close()
    assert np.isfinite(out).all()
    _check_ffn(out[rows], ref_out)


# ---------------- the FFN half of a layer, residual stream on the device ----------------

def test_block_inplace(be, layer0, golden):
    import torch
    from tie_b200 import moe
    g = golden("block_inplace.npz")
    be.upload_layer(1, layer0, ffn_norm_w=g["norm_w"])
    h = torch.from_numpy(g["hidden_in"].copy()).cuda()
    be.moe_block_inplace_ptr(1, h, h.shape[0], moe.DEVICE)
    out = h.cpu().numpy()
    _check_ffn(out, g["hidden_out"], tol=TOL)


def test_block_inplace_one_token_norm_inside_the_one_kernel_step(be, layer0, golden):
    """One token: the RMSNorm runs inside the cooperative decode kernel (one launch for
    h += MoE(RMSNorm(h))); identical bits to the RMSNorm kernel + three-kernel chain."""
    import torch
    from tie_b200 import moe
    g = golden("block_inplace.npz")
    be.upload_layer(1, layer0, ffn_norm_w=g["norm_w"])
    h0 = torch.from_numpy(g["hidden_in"][:1].copy()).cuda()
    a, b = h0.clone(), h0.clone()
    l0 = be.launch_count
    be.moe_block_inplace_ptr(1, a, 1, moe.DEVICE)
    l1 = be.launch_count
    be.moe_block_inplace_ptr(1, b, 1, moe.DEVICE | moe.PATH_DECODE_CHAIN)
    assert (l1 - l0, be.launch_count - l1) == (1, 4)
    assert np.array_equal(bits(a.cpu().numpy()), bits(b.cpu().numpy()))
    _check_ffn(a.cpu().numpy(), g["hidden_out"][:1], tol=TOL)
    for _ in range(3):  # graph replay, in place: each pass feeds the next
        be.moe_block_inplace_ptr(1, a, 1, moe.DEVICE | moe.GRAPH)
        be.moe_block_inplace_ptr(1, b, 1, moe.DEVICE | moe.GRAPH | moe.PATH_DECODE_CHAIN)
    assert np.array_equal(bits(a.cpu().numpy()), bits(b.cpu().numpy()))


def test_two_blocks_chained_teacher_forced(be, layer0, port_lib, ref_silu_table):
    """Two blocks back to back on the device (prefill- and decode-sized), each block checked
    against the oracle fed with the GPU's own input to that block (teacher forcing: a 1e-7
    difference can flip a near-tie in a later block, which is drift, not error)."""
    import torch
    from tie_b200 import moe
    layer1 = synth.make_layer(workloads.STACK_BASE_SEED + 1)
    ones = np.ones(2048, dtype=np.float32)
    b = moe.MoeBackend(max_tokens=64, silu_table=ref_silu_table, n_layers=2)
    try:
        b.upload_layer(0, layer0, ffn_norm_w=ones)
        b.upload_layer(1, layer1, ffn_norm_w=ones)
        ports = [port_lib.PortMoe(layer0, silu=ref_silu_table), port_lib.PortMoe(layer1, silu=ref_silu_table)]
        for T in (1, 40):
            h = torch.from_numpy(synth.make_x(workloads.STACK_BASE_SEED, T)).cuda()
            for l in range(2):
                h_in = h.cpu().numpy()
                b.moe_block_inplace_ptr(l, h, T, moe.DEVICE)
                want, _, _, _, _ = ports[l].moe_block_inplace(h_in, norm_w=ones, eps=1e-6)
                _check_ffn(h.cpu().numpy(), want)
    finally:
        b.close()


def test_stack_call_equals_the_per_layer_calls(layer0, ref_silu_table):
    """tie_cuda_moe_stack_inplace over three layers must leave the same bits as three
    tie_cuda_moe_block_inplace calls, for one token (one cooperative kernel per layer) and for a
    5-token batch; so must replays of the whole stack from its one CUDA graph."""
    import torch
    from tie_b200 import moe
    b = moe.MoeBackend(max_tokens=8, silu_table=ref_silu_table, n_layers=3)
    try:
        norm = (1.0 + 0.05 * np.sin(np.arange(2048))).astype(np.float32)
        b.upload_layer(0, layer0, ffn_norm_w=norm)
        b.upload_layer(1, synth.make_layer(workloads.STACK_BASE_SEED + 1), ffn_norm_w=np.ones(2048, np.float32))
        b.upload_layer(2, synth.make_layer(workloads.STACK_BASE_SEED + 2), ffn_norm_w=norm)
        for T in (1, 5):
            h0 = torch.from_numpy(synth.make_x(workloads.STACK_BASE_SEED, T)).cuda()
            want = h0.clone()
            for l in range(3):
                b.moe_block_inplace_ptr(l, want, T, moe.DEVICE)
            got = h0.clone()
            b.moe_stack_inplace_ptr(0, 3, got, T, moe.DEVICE)
            assert np.array_equal(bits(got.cpu().numpy()), bits(want.cpu().numpy()))
            g = h0.clone()
            for rep in range(3):  # capture, then replays; the epoch of the grid barriers advances on the device
                g.copy_(h0)
                b.moe_stack_inplace_ptr(0, 3, g, T, moe.DEVICE | moe.GRAPH)
                assert np.array_equal(bits(g.cpu().numpy()), bits(want.cpu().numpy())), rep
        # a sub-range, and arguments out of range
        h = torch.from_numpy(synth.make_x(5, 1)).cuda()
        w = h.clone()
        b.moe_block_inplace_ptr(1, w, 1, moe.DEVICE)
        b.moe_block_inplace_ptr(2, w, 1, moe.DEVICE)
        b.moe_stack_inplace_ptr(1, 2, h, 1, moe.DEVICE)
        assert np.array_equal(bits(h.cpu().numpy()), bits(w.cpu().numpy()))
        with pytest.raises(moe.TieCudaError) as ei:
            b.moe_stack_inplace_ptr(2, 2, h, 1, moe.DEVICE)
        assert ei.value.code == moe.EINVAL
    finally:
        b.close()


def test_all_48_blocks_of_the_stack_teacher_forced(port_lib, ref_silu_table):
    """The whole 48-block stack (independent seeded weights per block, h += MoE(RMSNorm(h)), norm
    weight 1, eps 1e-6) on 1 token (the one-kernel decode step with the RMSNorm inside) and on 4
    tokens (the decode kernels), the residual stream staying on the device from block to block.
    Every block is checked against the CPU restatement fed with the GPU's own input to that block.
    One layer slot is re-uploaded per block, so cached graphs of the previous block's weights must
    have been dropped by the upload."""
    import torch
    from tie_b200 import moe
    ones = np.ones(2048, dtype=np.float32)
    b = moe.MoeBackend(max_tokens=8, silu_table=ref_silu_table, n_layers=1)
    try:
        hs = {T: torch.from_numpy(synth.make_x(workloads.STACK_BASE_SEED, T)).cuda() for T in (1, 4)}
        worst = 0.0
        for l in range(48):
            layer = synth.make_layer(workloads.STACK_BASE_SEED + l)
            b.upload_layer(0, layer, ffn_norm_w=ones)
            P = port_lib.PortMoe(layer, silu=ref_silu_table)
            for T, h in hs.items():
                h_in = h.cpu().numpy()
                b.moe_block_inplace_ptr(0, h, T, moe.DEVICE | moe.GRAPH)
                want = P.moe_block_inplace(h_in, norm_w=ones, eps=1e-6)[0]
                got = h.cpu().numpy()
                assert np.isfinite(got).all(), (l, T)
                err = float(workloads.rel_rms_err(got, want).max())
                assert err <= TOL, (l, T, err)
                worst = max(worst, err)
        assert worst > 0.0  # (the two sides are different arithmetic: an exact zero would mean the check compared a value with itself)
    finally:
        b.close()


# ---------------- expert-parallel building blocks ----------------

def test_expert_rows_and_combine(be, port0, golden):
    import torch
    from tie_b200 import moe
    g = golden("batch64.npz")
    x = synth.make_x(0, 64)
    K = 8
    rows = np.repeat(x, K, axis=0)
    row_expert = g["idx"].reshape(-1).astype(np.int32)
    y_ref = port0.expert_rows(rows, row_expert)
    xr = torch.from_numpy(rows).cuda()
    re = torch.from_numpy(row_expert).cuda()
    for p in (moe.PATH_STREAM, moe.PATH_TENSOR):
        y = torch.empty_like(xr)
        be.expert_rows_ptr(0, xr, re, rows.shape[0], y, moe.DEVICE | p)
        _check_ffn(y.cpu().numpy(), y_ref)
    w = torch.from_numpy(g["w"]).cuda()
    out = torch.empty(64, 2048, device="cuda")
    be.combine_ptr(y, w, 64, out, moe.DEVICE)
    ref_out, _, _ = port0.moe_ffn(x)
    _check_ffn(out.cpu().numpy(), ref_out)


def test_expert_parallel_shard_rejects_foreign_experts(layer0, ref_silu_table):
    import torch
    from tie_b200 import moe
    part = synth.make_layer(0, layer0.shape, first_expert=16, n_local_expert=16)
    b = moe.MoeBackend(max_tokens=16, silu_table=ref_silu_table, ep_rank=1, ep_size=8)
    try:
        b.upload_layer(0, part)
        x = torch.zeros(4, 2048, device="cuda")
        y = torch.empty_like(x)
        ok = torch.tensor([16, 20, 31, 17], dtype=torch.int32, device="cuda")
        b.expert_rows_ptr(0, x, ok, 4, y, moe.DEVICE)
        bad = torch.tensor([16, 3, 31, 17], dtype=torch.int32, device="cuda")
        with pytest.raises(moe.TieCudaError) as ei:
            b.expert_rows_ptr(0, x, bad, 4, y, moe.DEVICE | moe.PATH_TENSOR)
        assert ei.value.code == moe.EKERNEL
        b.expert_rows_ptr(0, x, ok, 4, y, moe.DEVICE)  # the context stays usable
    finally:
        b.close()


# ---------------- math_dispatch rows ----------------

def test_dispatch_rows(be, layer0, port_lib, ref_silu_table):
    be.make_current()
    s = layer0.shape
    x = synth.make_x(0, 1)[0]
    e = 5
    gsz, dsz = s.gate_bytes_per_expert, s.down_bytes_per_expert
    g_ref = port_lib.mat_vec(x, layer0.gate[e * gsz:(e + 1) * gsz], 12, 2048, 768)
    u_ref = port_lib.mat_vec(x, layer0.up[e * gsz:(e + 1) * gsz], 12, 2048, 768)
    g = be.dispatch_mat_vec(x, layer0.gate.ctypes.data + e * gsz, 12, 2048, 0, 768)
    u = be.dispatch_mat_vec(x, layer0.up.ctypes.data + e * gsz, 12, 2048, 0, 768)
    assert np.abs(g - g_ref).max() <= 1e-5 * np.sqrt((g_ref ** 2).mean())
    assert np.abs(u - u_ref).max() <= 1e-5 * np.sqrt((u_ref ** 2).mean())
    # a row range, as the threaded dispatcher would call it (math_dispatch.c:262-283)
    part = be.dispatch_mat_vec(x, layer0.gate.ctypes.data + e * gsz, 12, 2048, 96, 192)
    assert np.array_equal(part[:96], np.zeros(96, dtype=np.float32)) and np.array_equal(bits(part[96:192]), bits(g[96:192]))
    h_ref = port_lib.swiglu(ref_silu_table, g_ref, u_ref)
    h = be.dispatch_swiglu(g_ref, u_ref)
    assert np.array_equal(bits(h), bits(h_ref)), "table SwiGLU is bit-exact given equal inputs"
    d_ref = port_lib.mat_vec(h_ref, layer0.down[e * dsz:(e + 1) * dsz], 14, 768, 2048)
    d = be.dispatch_mat_vec(h_ref, layer0.down.ctypes.data + e * dsz, 14, 768, 0, 2048)
    assert np.abs(d - d_ref).max() <= 1e-5 * np.sqrt((d_ref ** 2).mean())
    lg_ref = port_lib.mat_vec(x, layer0.router_w, 0, 2048, 128)
    lg = be.dispatch_mat_vec(x, layer0.router_w.ctypes.data, 0, 2048, 0, 128)
    assert np.array_equal(bits(lg), bits(lg_ref))


def test_dispatch_rows_from_several_host_threads(be, layer0):
    """The reference's threaded dispatcher (math_dispatch.c:262-283) hands disjoint row slices of one
    mat-vec to its pool workers, which call the row function at the same time.  Eight host threads
    do that here (ctypes releases the GIL during the call); every slice must equal the rows of a
    single whole-range call, bit for bit, for Q4_K, Q6_K (slices that start inside a group of 8
    rows of the re-ordered layout) and F32."""
    import threading
    be.make_current()
    s = layer0.shape
    x = synth.make_x(0, 1)[0]
    h = synth.make_x(1, 1, s.ffn_dim)[0]
    e = 3
    gsz, dsz = s.gate_bytes_per_expert, s.down_bytes_per_expert
    cases = [(x, layer0.gate.ctypes.data + e * gsz, 12, 2048, 768), (h, layer0.down.ctypes.data + e * dsz, 14, 768, 2048),
             (x, layer0.router_w.ctypes.data, 0, 2048, 128)]
    for vec, wptr, typ, in_dim, rows in cases:
        whole = be.dispatch_mat_vec(vec, wptr, typ, in_dim, 0, rows)
        n_thr = 8
        cuts = [rows * i // n_thr for i in range(n_thr + 1)]
        if typ == 14:
            cuts = [c + (3 if 0 < c < rows else 0) for c in cuts]  # slice starts off the 8-row groups
        out = np.full(rows, np.nan, dtype=np.float32)
        errs = []

        def work(a, b):
            try:
                for _ in range(3):
                    be.dispatch_mat_vec(vec, wptr, typ, in_dim, a, b, out=out)
            except Exception as ex:  # noqa: BLE001
                errs.append(ex)

        th = [threading.Thread(target=work, args=(cuts[i], cuts[i + 1])) for i in range(n_thr)]
        for t in th:
            t.start()
        for t in th:
            t.join()
        assert not errs, errs
        assert np.array_equal(bits(out), bits(whole))


@pytest.mark.parametrize("ggml_type,in_dim,out_dim,batch", [(12, 2048, 4096, 100), (14, 2048, 512, 37), (12, 768, 2048, 64),
                                                             (14, 768, 256, 1),
                                                             # the attention output projection of this model (model_qwen3.c:384): 4096 -> 2048;
                                                             # Q4_K rows of 16 super-blocks run as two launches of 8
                                                             (12, 4096, 2048, 70), (14, 4096, 2048, 33),
                                                             # other widths: 5 and 24 super-blocks per row, an odd number of 128-row tiles
                                                             (12, 1280, 384, 50), (14, 1024, 640, 17), (12, 6144, 256, 40)])
def test_dense_mat_mat_on_the_grouped_product(be, port_lib, ggml_type, in_dim, out_dim, batch):
    """dispatch_mat_mat (math_dispatch.c:304) for stand-alone Q4_K / Q6_K tensors — attention
    q/k/v-shaped [4096|512 x 2048], the attention output projection [2048 x 4096], FFN-shaped and
    odd-sized ones — against the restatement's mat-vec per row."""
    import torch
    from tie_b200 import moe
    nb = out_dim * (in_dim // 256)
    w = synth.q4k_blocks(77, 9, nb) if ggml_type == 12 else synth.q6k_blocks(77, 9, nb)
    w = np.ascontiguousarray(w)
    be.register_tensor(w, ggml_type, in_dim)
    x = synth.make_x(3, batch, in_dim)
    ref = np.stack([port_lib.mat_vec(x[i], w, ggml_type, in_dim, out_dim) for i in range(batch)])
    got = be.mat_mat(w, x, np.empty((batch, out_dim), dtype=np.float32), batch, in_dim, out_dim)  # host pointers
    scale = np.sqrt((ref.astype(np.float64) ** 2).mean(axis=1, keepdims=True))
    assert (np.abs(got - ref) / scale).max() < TOL
    xd = torch.from_numpy(x).cuda()
    od = torch.empty(batch, out_dim, device="cuda")
    be.mat_mat(w, xd, od, batch, in_dim, out_dim, moe.DEVICE)
    assert np.array_equal(bits(od.cpu().numpy()), bits(got))
    with pytest.raises(moe.TieCudaError) as ei:  # not the registered tensor's shape
        be.mat_mat(w, x, got, batch, in_dim + 256, out_dim)
    assert ei.value.code == moe.EINVAL
    # the MoE path of the context is undisturbed by the dense call's use of its operand scratch
    xs = synth.make_x(0, 40)
    a = be.moe_ffn(0, xs, path=moe.PATH_TENSOR)
    be.mat_mat(w, x, got, batch, in_dim, out_dim)
    assert np.array_equal(bits(be.moe_ffn(0, xs, path=moe.PATH_TENSOR)), bits(a))


def test_two_host_buffer_calls_in_flight(be, port0):
    """tie_cuda_moe_ffn_submit / _wait: the same result as the synchronous host-buffer call, with two
    calls in flight on alternating slots (different inputs, different token counts), over several
    rounds (the later rounds replay the slots' CUDA graphs); a busy slot, pageable memory and a bad
    slot number are refused."""
    import torch
    from tie_b200 import moe
    xs = [torch.from_numpy(synth.make_x(0, n, first_token=f)).pin_memory() for n, f in ((96, 0), (40, 300))]
    outs = [torch.empty_like(x).pin_memory() for x in xs]
    want = [be.moe_ffn(0, x.numpy()) for x in xs]
    for rnd in range(3):
        for o in outs:
            o.fill_(float("nan"))
        be.moe_ffn_submit(0, xs[0], outs[0], xs[0].shape[0], 0, moe.GRAPH)
        be.moe_ffn_submit(0, xs[1], outs[1], xs[1].shape[0], 1, moe.GRAPH)
        with pytest.raises(moe.TieCudaError) as ei:  # slot 0 is still in flight
            be.moe_ffn_submit(0, xs[0], outs[0], xs[0].shape[0], 0, moe.GRAPH)
        assert ei.value.code == moe.EINVAL
        be.moe_ffn_wait(0)
        be.moe_ffn_wait(1)
        for o, w in zip(outs, want):
            assert np.array_equal(bits(o.numpy()), bits(w)), rnd
    ref, _, _ = port0.moe_ffn(xs[1].numpy())
    _check_ffn(outs[1].numpy(), ref)
    with pytest.raises(moe.TieCudaError) as ei:
        be.moe_ffn_wait(0)  # nothing in flight
    assert ei.value.code == moe.EINVAL
    pageable = torch.zeros(4, 2048)
    with pytest.raises(moe.TieCudaError) as ei:
        be.moe_ffn_submit(0, pageable, outs[0], 4, 0)
    assert ei.value.code == moe.ENOTSUP
    with pytest.raises(moe.TieCudaError) as ei:
        be.moe_ffn_submit(0, xs[0], outs[0], 96, moe.N_SLOTS)
    assert ei.value.code == moe.EINVAL
    # three calls in flight on slots used in turn
    for o in outs:
        o.fill_(float("nan"))
    third = torch.empty_like(outs[0]).pin_memory()
    be.moe_ffn_submit(0, xs[0], outs[0], 96, 0, moe.GRAPH)
    be.moe_ffn_submit(0, xs[1], outs[1], 40, 1, moe.GRAPH)
    be.moe_ffn_submit(0, xs[0], third, 96, 2, moe.GRAPH)
    for slot in range(3):
        be.moe_ffn_wait(slot)
    assert np.array_equal(bits(outs[0].numpy()), bits(want[0])) and np.array_equal(bits(outs[1].numpy()), bits(want[1]))
    assert np.array_equal(bits(third.numpy()), bits(want[0]))


def test_errors_are_codes_not_exits(be):
    from tie_b200 import moe
    x = np.zeros((1, 2048), dtype=np.float32)
    with pytest.raises(moe.TieCudaError) as ei:
        be.moe_ffn(7, x)  # layer never uploaded / out of range
    assert ei.value.code == moe.EINVAL
    with pytest.raises(moe.TieCudaError) as ei:
        be.moe_ffn(0, np.zeros((513, 2048), dtype=np.float32))  # more tokens than max_tokens
    assert ei.value.code == moe.EINVAL
    be.make_current()
    with pytest.raises(moe.TieCudaError):
        be.dispatch_mat_vec(x[0], x.ctypes.data, 12, 2048, 0, 8)  # W is not an uploaded tensor
    assert be.launch_count > 0


# ---------------- expert-parallel dispatch / combine on one GPU ----------------

def test_ep_dispatch_and_combine_roundtrip(be, port0):
    """dispatch -> expert rows -> combine through the dispatch permutation == the plain call."""
    import torch
    from tie_b200 import moe
    T, K, H, E = 48, 8, 2048, 128
    x = synth.make_x(0, T, first_token=300)
    ref_out, ref_idx, _ = port0.moe_ffn(x)
    xd = torch.from_numpy(x).cuda()
    idx = torch.empty(T, K, dtype=torch.int32, device="cuda")
    w = torch.empty(T, K, dtype=torch.float32, device="cuda")
    be.route_ptr(0, xd, T, idx, w, None, None, moe.DEVICE)
    assert np.array_equal(idx.cpu().numpy(), ref_idx)
    rows = torch.empty(T * K, H, device="cuda")
    rexp = torch.empty(T * K, dtype=torch.int32, device="cuda")
    counts = torch.empty(E, dtype=torch.int32, device="cuda")
    be.ep_dispatch_ptr(xd, idx, T, rows, rexp, counts, moe.DEVICE)
    e = rexp.cpu().numpy()
    assert (np.diff(e) >= 0).all(), "rows must be grouped by expert id (hence by destination rank)"
    assert np.array_equal(counts.cpu().numpy(), np.bincount(ref_idx.reshape(-1), minlength=E))
    # stable: within an expert, rows keep (token, slot) order, and every row carries its token's x
    flat = ref_idx.reshape(-1)
    perm = np.argsort(flat, kind="stable")
    assert np.array_equal(e, flat[perm])
    assert np.array_equal(rows.cpu().numpy(), x[perm // K])
    y = torch.empty_like(rows)
    be.expert_rows_ptr(0, rows, rexp, T * K, y, moe.DEVICE)
    out = torch.empty(T, H, device="cuda")
    be.ep_combine_ptr(y, w, T, out, moe.DEVICE)
    _check_ffn(out.cpu().numpy(), ref_out)


# ---------------- graph replay ----------------

def test_graph_replay_matches_direct_launches(be):
    import torch
    from tie_b200 import moe
    s = torch.cuda.Stream()
    be.set_stream(s.cuda_stream)
    try:
        for T in (1, 64):
            xs = [torch.from_numpy(synth.make_x(0, T, first_token=o)).cuda() for o in (0, 700)]
            buf = torch.empty_like(xs[0])
            out = torch.empty_like(buf)
            for x in xs:  # same buffers, new contents: the cached graph must see the new data
                want = torch.empty_like(x)
                be.moe_ffn_ptr(0, x, want, T, moe.DEVICE)
                buf.copy_(x)
                torch.cuda.synchronize()
                be.moe_ffn_ptr(0, buf, out, T, moe.DEVICE | moe.GRAPH)
                assert np.array_equal(bits(out.cpu().numpy()), bits(want.cpu().numpy()))
        # host buffers through the graph path (pinned and pageable)
        x = synth.make_x(0, 8)
        want = be.moe_ffn(0, x)
        xp = torch.from_numpy(x).pin_memory()
        op = torch.empty_like(xp).pin_memory()
        for _ in range(2):
            be.moe_ffn_ptr(0, xp, op, 8, moe.HOST | moe.GRAPH)
            assert np.array_equal(bits(op.numpy()), bits(want))
        got = np.empty_like(x)
        be.moe_ffn_ptr(0, x, got, 8, moe.HOST | moe.GRAPH)
        assert np.array_equal(bits(got), bits(want))
    finally:
        be.set_stream(None)
