"""CPU tests: the synthetic generator, the plain-C restatement (oracle/moe_oracle.c) against the
golden vectors produced by the reference's own compiled code, and — where oracle/_ref has been
built — against that code live, bit for bit."""
import hashlib
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from tie_b200 import synth, workloads

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
GOLDEN = os.path.join(ROOT, "tests", "golden")


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


# ---------------- generator ----------------

def test_synth_known_answers(layer0):
    kat = json.load(open(os.path.join(GOLDEN, "synth_kat.json")))
    assert sha(layer0.router_w.reshape(-1)[:1024]) == kat["router_first_1024"]
    assert sha(layer0.gate[: 64 * 144]) == kat["gate_first_64_blocks"]
    assert sha(layer0.up[1000 * 144: 1064 * 144]) == kat["up_blocks_1000_1064"]
    assert sha(layer0.down[: 64 * 210]) == kat["down_first_64_blocks"]
    assert sha(layer0.gate) == kat["gate_total"]
    assert sha(layer0.down) == kat["down_total"]
    assert sha(synth.make_x(workloads.BASE_SEED, 2)) == kat["x_first_4096"]
    logp, ranks = synth.zipf_logp(128, workloads.BASE_SEED, 1.1)
    assert sha(logp) == kat["zipf_logp"] and sha(ranks) == kat["zipf_ranks"]
    assert sorted(ranks.tolist()) == list(range(1, 129))


def test_synth_slices_match_whole(layer0):
    """Expert-parallel ranks generate only their experts: same bytes as the slice of the whole."""
    s = layer0.shape
    part = synth.make_layer(workloads.BASE_SEED, s, first_expert=48, n_local_expert=16)
    g, d = s.gate_bytes_per_expert, s.down_bytes_per_expert
    assert np.array_equal(part.gate, layer0.gate[48 * g: 64 * g])
    assert np.array_equal(part.up, layer0.up[48 * g: 64 * g])
    assert np.array_equal(part.down, layer0.down[48 * d: 64 * d])
    x = synth.make_x(0, 16)
    assert np.array_equal(synth.make_x(0, 4, first_token=8), x[8:12])


def test_synth_distributions(layer0):
    s = layer0.shape
    L = synth.lib()
    blk = layer0.gate[: 4096 * 144].reshape(4096, 144)
    d = np.array([L.tie_synth_f16_to_f32(int(b[0]) | (int(b[1]) << 8)) for b in blk])
    dmin = np.array([L.tie_synth_f16_to_f32(int(b[2]) | (int(b[3]) << 8)) for b in blk])
    assert 1e-3 * 0.999 <= d.min() and d.max() <= 4e-3 * 1.001
    assert 0 <= dmin.min() and dmin.max() <= 2e-3 * 1.001
    assert (dmin < 6.2e-5).any(), "fp16-subnormal dmin must occur (it does ~3% of the time)"
    q6 = layer0.down[: 4096 * 210].reshape(4096, 210)
    sc = q6[:, 192:208].view(np.int8)
    assert sc.min() == -32 and sc.max() == 31
    assert abs(float(layer0.router_w.std()) - 0.02) < 5e-4
    x = synth.make_x(0, 64)
    assert abs(float(x.mean())) < 0.01 and abs(float(x.std()) - 1.0) < 0.01


def test_f16_conversion_exhaustive():
    """Every half value survives f16 -> f32 -> f16 (round trip of the generator's converters)."""
    L = synth.lib()
    for h in range(0, 0x7C00, 7):
        f = L.tie_synth_f16_to_f32(h)
        assert L.tie_synth_f32_to_f16(f) == h
    assert np.float32(L.tie_synth_f16_to_f32(0x3C00)) == 1.0
    assert L.tie_synth_f32_to_f16(65520.0) == 0x7C00
    assert L.tie_synth_f32_to_f16(2.0 ** -25) == 0  # tie to even
    assert L.tie_synth_f32_to_f16(np.float32(2.0 ** -25 * 1.0001)) == 1
    # against numpy's conversion on random values
    rng = np.random.default_rng(0)
    v = (rng.standard_normal(4000) * np.exp(rng.uniform(-18, 10, 4000))).astype(np.float32)
    got = np.array([L.tie_synth_f32_to_f16(float(t)) for t in v], dtype=np.uint16)
    with np.errstate(over="ignore"):
        assert np.array_equal(got, v.astype(np.float16).view(np.uint16))


# ---------------- restatement vs golden vectors (outputs of the reference's compiled code) ----------------

def _port(port_lib, layer, ref_silu_table):
    return port_lib.PortMoe(layer, silu=ref_silu_table)


def test_port_decode1_bit_exact(port_lib, layer0, ref_silu_table, golden):
    g = golden("decode1.npz")
    out, idx, w, logits = _port(port_lib, layer0, ref_silu_table).moe_ffn(synth.make_x(0, 1), want_logits=True)
    assert np.array_equal(bits(logits), bits(g["logits"]))
    assert np.array_equal(idx, g["idx"])
    assert np.array_equal(bits(w), bits(g["w"]))
    assert np.array_equal(bits(out), bits(g["out"]))


def test_port_batch64_bit_exact(port_lib, layer0, ref_silu_table, golden):
    P = _port(port_lib, layer0, ref_silu_table)
    x = synth.make_x(0, 64)
    g = golden("batch64.npz")
    out, idx, w, logits = P.moe_ffn(x, want_logits=True)
    assert np.array_equal(idx, g["idx"]) and np.array_equal(bits(w), bits(g["w"]))
    assert np.array_equal(bits(out[g["rows"]]), bits(g["out_rows"]))
    rms = np.sqrt((out.astype(np.float64) ** 2).mean(1)).astype(np.float32)
    assert np.array_equal(bits(rms), bits(g["rms"]))
    # skewed variant: the bias recipe reproduces the stored bias, then outputs match
    gs = golden("batch64_skew.npz")
    bias, alpha, share = workloads.skew_bias(logits, 8)
    assert np.array_equal(bits(bias), bits(gs["bias"])) and abs(share - 0.30) <= 0.01
    out_s, idx_s, w_s = P.moe_ffn(x, router_bias=bias)
    assert np.array_equal(idx_s, gs["idx"]) and np.array_equal(bits(w_s), bits(gs["w"]))
    assert np.array_equal(bits(out_s[gs["rows"]]), bits(gs["out_rows"]))
    hot = np.argsort(synth.zipf_logp(128, 0, 1.1)[1])[:4]
    assert abs(np.isin(idx_s, hot).mean() - 0.30) <= 0.01


def test_port_prefill512_bit_exact(port_lib, layer0, ref_silu_table, golden):
    g = golden("prefill512.npz")
    out, idx, w = _port(port_lib, layer0, ref_silu_table).moe_ffn(synth.make_x(0, 512))
    assert np.array_equal(idx, g["idx"]) and np.array_equal(bits(w), bits(g["w"]))
    assert np.array_equal(bits(out[g["rows"]]), bits(g["out_rows"]))
    rms = np.sqrt((out.astype(np.float64) ** 2).mean(1)).astype(np.float32)
    assert np.array_equal(bits(rms), bits(g["rms"]))


def test_port_small_shape_and_parallel_modes(port_lib, small_layer, small_shape, ref_silu_table, golden):
    g = golden("small.npz")
    P = _port(port_lib, small_layer, ref_silu_table)
    x = synth.make_x(workloads.BASE_SEED + 1, 24, small_shape.hidden)
    for mode in (0, 1, 2):
        out, idx, w, logits = P.moe_ffn(x, want_logits=True, parallel=mode)
        assert np.array_equal(bits(logits), bits(g["logits"]))
        assert np.array_equal(idx, g["idx"]) and np.array_equal(bits(w), bits(g["w"]))
        assert np.array_equal(bits(out), bits(g["out"]))
    # expert_rows is the same arithmetic applied row-wise
    rows = np.repeat(x, small_shape.top_k, axis=0)
    y = P.expert_rows(rows, g["idx"].reshape(-1))
    acc = np.zeros_like(x)
    for j in range(small_shape.top_k):  # fma from zero, j ascending
        acc = (np.float64(1) * acc + g["w"][:, j:j + 1].astype(np.float64) * y[j::small_shape.top_k].astype(np.float64)).astype(np.float32)
    assert workloads.rel_rms_err(acc, g["out"]).max() < 1e-6


def test_port_block_inplace(port_lib, layer0, ref_silu_table, golden):
    g = golden("block_inplace.npz")
    P = _port(port_lib, layer0, ref_silu_table)
    h, normed, ffn, idx, w = P.moe_block_inplace(g["hidden_in"], norm_w=g["norm_w"], eps=1e-6)
    # RMSNorm: the reference as built with -ffast-math evaluates 1/sqrt with the hardware estimate +
    # one Newton step (CPU-model dependent, up to 3 ulp from the exact value seen); allow 4 ulp
    ulp = np.abs(bits(normed).astype(np.int64) - bits(g["normed"]).astype(np.int64))
    assert ulp.max() <= 4
    assert np.array_equal(idx, g["idx"])
    assert workloads.rel_rms_err(h, g["hidden_out"]).max() < 1e-5


def test_port_lfm2_routing_against_reference_fixture(port_lib, layer0, ref_silu_table, golden):
    """LFM2-MoE routing (model_lfm2.c:438-473): same experts in the same order as the compiled
    reference; gates to a few ulp (the reference's two divisions are -ffast-math reciprocal
    estimates, glibc expf on both sides)."""
    g = golden("lfm2_route.npz")
    P = _port(port_lib, layer0, ref_silu_table)
    x = synth.make_x(0, 64)
    idx, w, scores = P.route_lfm2(x)
    assert np.array_equal(idx, g["idx"])
    assert np.max(np.abs(w - g["w"]) / g["w"]) < 1e-6
    assert np.max(np.abs(scores - g["scores"])) < 5e-7
    idx_b, w_b, _ = P.route_lfm2(x, g["bias"])
    assert np.array_equal(idx_b, g["idx_b"]) and (idx_b != idx).any()
    assert np.max(np.abs(w_b - g["w_b"]) / g["w_b"]) < 1e-6
    # gates are the unbiased sigmoids, L1-normalised with 1/(sum + 1e-6)
    sel = np.take_along_axis(scores, idx_b, axis=1)
    assert np.allclose(w_b, sel / (sel.sum(1, keepdims=True) + 1e-6), rtol=1e-6)


def test_port_silu_table_close_to_reference(port_lib, ref_silu_table):
    """The restated table (IEEE division) vs the compiled reference's (reciprocal estimate)."""
    t = port_lib.silu_table()
    assert np.abs(t - ref_silu_table).max() <= 2e-6
    # and it is nothing like a true SiLU: that is the reference's behaviour being reproduced
    xs = np.linspace(-10, 10, 8192)
    true = xs / (1 + np.exp(-xs))
    assert np.abs(ref_silu_table - true).max() > 0.04


def test_topk_tie_rule(port_lib, small_layer, ref_silu_table):
    """find_top_k keeps the lower index on exact ties (strict '>')."""
    import ctypes
    L = port_lib.lib()
    L.oracle_find_top_k.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    lg = np.zeros(32, dtype=np.float32)
    lg[[3, 9, 20]] = 5.0
    lg[[1, 30]] = 7.0
    idx = np.empty(4, dtype=np.int32)
    sc = np.empty(4, dtype=np.float32)
    L.oracle_find_top_k(lg.ctypes.data, 32, 4, idx.ctypes.data, sc.ctypes.data)
    assert idx.tolist() == [1, 30, 3, 9]


# ---------------- restatement vs the reference's compiled code, live ----------------

_REF_SCRIPT = r"""
import sys, json, numpy as np
sys.path.insert(0, %(root)r)
from oracle import ref, port
from tie_b200 import synth, workloads
R = ref.RefMoe(path=%(path)r)
layer = synth.make_layer(workloads.BASE_SEED)
R.set_layer(layer)
tab = R.silu_table()
P = port.PortMoe(layer, silu=tab)
x = synth.make_x(workloads.BASE_SEED, 24, first_token=1000)
o_r, i_r, w_r, l_r = R.moe_ffn(x, want_logits=True)
o_p, i_p, w_p, l_p = P.moe_ffn(x, want_logits=True)
b = lambda a: np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
res = dict(logits=bool(np.array_equal(b(l_r), b(l_p))), idx=bool(np.array_equal(i_r, i_p)),
           w=bool(np.array_equal(b(w_r), b(w_p))), out=bool(np.array_equal(b(o_r), b(o_p))),
           table=bool(np.array_equal(b(tab), b(np.fromfile(%(gold)r, dtype=np.float32)))))
e = 77
gsz = layer.shape.gate_bytes_per_expert; dsz = layer.shape.down_bytes_per_expert
g_r = R.mat_vec(x[0], layer.gate[e*gsz:(e+1)*gsz], 12, 2048, 768)
g_p = port.mat_vec(x[0], layer.gate[e*gsz:(e+1)*gsz], 12, 2048, 768)
u_r = R.mat_vec(x[0], layer.up[e*gsz:(e+1)*gsz], 12, 2048, 768)
h_r = R.swiglu(g_r, u_r); h_p = port.swiglu(tab, g_r, u_r)
d_r = R.mat_vec(h_r, layer.down[e*dsz:(e+1)*dsz], 14, 768, 2048)
d_p = port.mat_vec(h_r, layer.down[e*dsz:(e+1)*dsz], 14, 768, 2048)
res.update(q4k=bool(np.array_equal(b(g_r), b(g_p))), swiglu=bool(np.array_equal(b(h_r), b(h_p))),
           q6k=bool(np.array_equal(b(d_r), b(d_p))))
print("RESULT " + json.dumps(res))
"""


@pytest.mark.parametrize("which", ["portable", "native"])
def test_port_matches_compiled_reference_live(which):
    """Runs only where oracle/_ref has been built (it needs the reference's sources)."""
    from oracle import ref
    path = ref.LIB_PATH if which == "portable" else ref.LIB_NATIVE_PATH
    if not os.path.exists(path):
        pytest.skip(f"{os.path.basename(path)} not built")
    code = _REF_SCRIPT % dict(root=ROOT, path=path, gold=os.path.join(GOLDEN, "silu_table_ref.f32"))
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    line = [l for l in out.stdout.splitlines() if l.startswith("RESULT ")][-1]
    res = json.loads(line[len("RESULT "):])
    assert all(res.values()), res
