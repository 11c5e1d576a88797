"""GGUF reader (tie_b200/gguf): files written here with the public GGUF layout are read back, the
MoE tensors of a block come out as the bytes that went in, and damaged files are refused."""
import os
import struct

import numpy as np
import pytest

from tie_b200 import gguf, synth

VT = {"u8": 0, "i8": 1, "u16": 2, "i16": 3, "u32": 4, "i32": 5, "f32": 6, "bool": 7, "str": 8, "arr": 9, "u64": 10, "i64": 11, "f64": 12}
FMT = {"u8": "<B", "i8": "<b", "u16": "<H", "i16": "<h", "u32": "<I", "i32": "<i", "f32": "<f", "bool": "<B", "u64": "<Q", "i64": "<q", "f64": "<d"}


def _s(b: bytes) -> bytes:
    return struct.pack("<Q", len(b)) + b


def _value(kind, v) -> bytes:
    if kind == "str":
        return _s(v.encode())
    if kind == "arr":
        ek, items = v
        return struct.pack("<IQ", VT[ek], len(items)) + b"".join(_value(ek, x) for x in items)
    return struct.pack(FMT[kind], v)


def write_gguf(path, kvs, tensors, version=3, align=32, put_alignment_key=False):
    """kvs: [(key, kind, value)]; tensors: [(name, ggml_type, dims (contiguous first), bytes)]."""
    kvs = list(kvs)
    if put_alignment_key:
        kvs.append(("general.alignment", "u32", align))
    head = struct.pack("<IIQQ", 0x46554747, version, len(tensors), len(kvs))
    for k, kind, v in kvs:
        head += _s(k.encode()) + struct.pack("<I", VT[kind]) + _value(kind, v)
    off, infos, blobs = 0, b"", []
    for name, t, dims, data in tensors:
        infos += _s(name.encode()) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        infos += struct.pack("<IQ", t, off)
        blobs.append((off, bytes(data)))
        off = (off + len(data) + align - 1) // align * align
    body = head + infos
    body += b"\0" * ((len(body) + align - 1) // align * align - len(body))
    data = bytearray(off)
    for o, b in blobs:
        data[o:o + len(b)] = b
    with open(path, "wb") as f:
        f.write(body + data)


def moe_model(shape, n_layers, seed=7, down_types=None):
    """KVs and tensors of a qwen3moe-shaped file with only what the MoE path reads plus some noise."""
    s = shape
    kvs = [("general.architecture", "str", "qwen3moe"), ("general.name", "str", "synthetic"),
           ("qwen3moe.block_count", "u32", n_layers), ("qwen3moe.embedding_length", "u32", s.hidden),
           ("qwen3moe.expert_count", "u32", s.n_expert), ("qwen3moe.expert_used_count", "u32", s.top_k),
           ("qwen3moe.expert_feed_forward_length", "u32", s.ffn_dim),
           ("qwen3moe.attention.layer_norm_rms_epsilon", "f32", 1e-6),
           ("tokenizer.ggml.tokens", "arr", ("str", ["<a>", "b", "longer token"])),
           ("tokenizer.ggml.scores", "arr", ("f32", [0.5, -1.0, 2.0])),
           ("some.i64", "i64", 12345678901), ("some.bool", "bool", 1), ("some.f64", "f64", 2.5)]
    layers, tensors = [], [("token_embd.weight", 0, [s.hidden, 3], np.zeros(3 * s.hidden, np.float32).tobytes())]
    gu = s.n_expert * s.ffn_dim * (s.hidden // 256)
    dn = s.n_expert * s.hidden * (s.ffn_dim // 256)
    for i in range(n_layers):
        dt = (down_types or [synth.GGML_Q6_K] * n_layers)[i]
        router = synth.normal_f32(seed + i, synth.STREAM_ROUTER, s.n_expert * s.hidden, 0.02).reshape(s.n_expert, s.hidden)
        gate = synth.q4k_blocks(seed + i, synth.STREAM_GATE, gu)
        up = synth.q4k_blocks(seed + i, synth.STREAM_UP, gu)
        down = synth.q6k_blocks(seed + i, synth.STREAM_DOWN, dn) if dt == synth.GGML_Q6_K else synth.q4k_blocks(seed + i, synth.STREAM_DOWN, dn)
        norm = (1.0 + 0.01 * np.arange(s.hidden)).astype(np.float32)
        layers.append(synth.MoeLayer(s, router, gate, up, down, down_type=dt))
        tensors += [(f"blk.{i}.attn_q.weight", 0, [8, 2], np.ones(16, np.float32).tobytes()),
                    (f"blk.{i}.ffn_norm.weight", 0, [s.hidden], norm.tobytes()),
                    (f"blk.{i}.ffn_gate_inp.weight", 0, [s.hidden, s.n_expert], router.tobytes()),
                    (f"blk.{i}.ffn_gate_exps.weight", synth.GGML_Q4_K, [s.hidden, s.ffn_dim, s.n_expert], gate.tobytes()),
                    (f"blk.{i}.ffn_down_exps.weight", dt, [s.ffn_dim, s.hidden, s.n_expert], down.tobytes()),
                    (f"blk.{i}.ffn_up_exps.weight", synth.GGML_Q4_K, [s.hidden, s.ffn_dim, s.n_expert], up.tobytes())]
    return kvs, tensors, layers


SHAPE = synth.MoeShape(hidden=512, n_expert=8, top_k=2, ffn_dim=256)


@pytest.mark.parametrize("version,align,key", [(3, 32, False), (2, 64, True), (3, 4096, True)])
def test_roundtrip_moe_tensors(tmp_path, version, align, key):
    kvs, tensors, layers = moe_model(SHAPE, 2, down_types=[synth.GGML_Q6_K, synth.GGML_Q4_K])
    p = str(tmp_path / "m.gguf")
    write_gguf(p, kvs, tensors, version=version, align=align, put_alignment_key=key)
    with gguf.GgufFile(p) as g:
        assert g.version == version and g.n_tensors == len(tensors) and g.n_kv == len(kvs) + (1 if key else 0)
        cfg = g.moe_config()
        assert cfg == {"arch": "qwen3moe", "n_layers": 2, "hidden": 512, "n_expert": 8, "top_k": 2, "ffn_dim": 256,
                       "norm_eps": pytest.approx(1e-6)}
        assert g.get_str("general.name") == "synthetic" and g.get_int("some.i64") == 12345678901
        assert g.get_int("some.bool") == 1 and g.get_float("some.f64") == 2.5
        for i, want in enumerate(layers):
            got, norm = g.moe_layer(i)
            assert np.array_equal(got.router_w, want.router_w)
            assert np.array_equal(got.gate, want.gate) and np.array_equal(got.up, want.up) and np.array_equal(got.down, want.down)
            assert (got.gate_type, got.up_type, got.down_type) == (synth.GGML_Q4_K, synth.GGML_Q4_K, want.down_type)
            assert norm is not None and norm[3] == np.float32(1.03)
        data, t, dims = g.tensor("blk.1.attn_q.weight")
        assert t == 0 and dims == [8, 2] and data.nbytes == 64


def test_missing_and_mistyped_entries(tmp_path):
    kvs, tensors, _ = moe_model(SHAPE, 1)
    p = str(tmp_path / "m.gguf")
    write_gguf(p, kvs, [t for t in tensors if "ffn_up_exps" not in t[0] and "ffn_norm" not in t[0]])
    with gguf.GgufFile(p) as g:
        with pytest.raises(gguf.GgufError) as e:
            g.moe_layer(0)
        assert e.value.code == gguf.ENOTFOUND
        with pytest.raises(gguf.GgufError) as e:
            g.get_int("general.name")
        assert e.value.code == gguf.ETYPE
        with pytest.raises(gguf.GgufError) as e:
            g.get_int("no.such.key")
        assert e.value.code == gguf.ENOTFOUND
    # wrong shape: the router of another model
    bad = [(n, t, ([SHAPE.hidden, SHAPE.n_expert + 1] if "ffn_gate_inp" in n else d), (b + b"\0" * SHAPE.hidden * 4 if "ffn_gate_inp" in n else b))
           for n, t, d, b in tensors]
    write_gguf(p, kvs, bad)
    with gguf.GgufFile(p) as g:
        with pytest.raises(gguf.GgufError) as e:
            g.moe_layer(0)
        assert e.value.code == gguf.ETYPE
    # a file without the norm is accepted (the caller may keep the norm on the CPU side)
    write_gguf(p, kvs, [t for t in tensors if "ffn_norm" not in t[0]])
    with gguf.GgufFile(p) as g:
        _, norm = g.moe_layer(0)
        assert norm is None


def test_damaged_files_are_refused(tmp_path):
    kvs, tensors, _ = moe_model(SHAPE, 1)
    p = str(tmp_path / "m.gguf")
    write_gguf(p, kvs, tensors)
    raw = open(p, "rb").read()
    q = str(tmp_path / "bad.gguf")
    cases = {"magic": b"GGUX" + raw[4:], "version": raw[:4] + struct.pack("<I", 9) + raw[8:], "header only": raw[:24],
             "directory cut": raw[:300], "huge counts": raw[:8] + struct.pack("<QQ", 1 << 60, 1 << 60) + raw[24:]}
    for name, blob in cases.items():
        open(q, "wb").write(blob)
        with pytest.raises(gguf.GgufError) as e:
            gguf.GgufFile(q)
        assert e.value.code == gguf.EFORMAT, name
    # data section cut short: the directory parses, the tensor does not fit
    open(q, "wb").write(raw[:len(raw) - 4096])
    with gguf.GgufFile(q) as g:
        with pytest.raises(gguf.GgufError) as e:
            g.moe_layer(0)
        assert e.value.code == gguf.EFORMAT
    with pytest.raises(gguf.GgufError) as e:
        gguf.GgufFile(str(tmp_path / "absent.gguf"))
    assert e.value.code == gguf.EIO


def test_library_exports_what_the_header_declares():
    import re
    import subprocess
    hdr = open(os.path.join(os.path.dirname(__file__), "..", "include", "tie_gguf.h")).read()
    declared = set(re.findall(r"\b(tie_gguf_[a-z0-9_]+)\s*\(", hdr))
    out = subprocess.check_output(["nm", "-D", "--defined-only", gguf.build()], text=True)
    exported = {l.split()[-1] for l in out.splitlines() if " T " in l and "tie_gguf_" in l}
    assert declared == exported == set(gguf.EXPORTS)


# ---- the same file through the reference's own parser ----

def _ref_gguf_lib():
    """The compiled reference (oracle/_ref/libtie_ref.so holds its gguf.c unmodified), or None."""
    import ctypes
    from oracle import ref
    if not ref.available():
        return None
    L = ctypes.CDLL(ref.LIB_PATH)
    L.gguf_model_parse.restype = ctypes.c_void_p
    L.gguf_model_parse.argtypes = [ctypes.c_char_p]
    L.gguf_get_tensor.restype = ctypes.c_void_p
    L.gguf_get_tensor.argtypes = [ctypes.c_void_p, ctypes.c_char_p]
    L.gguf_metadata_get_value.restype = ctypes.c_int
    L.gguf_metadata_get_value.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p]
    L.gguf_metadata_get_string.restype = ctypes.c_char_p
    L.gguf_metadata_get_string.argtypes = [ctypes.c_void_p, ctypes.c_char_p]
    L.gguf_model_close.argtypes = [ctypes.c_void_p]
    return L


def test_reader_agrees_with_the_reference_parser_on_the_same_file(tmp_path):
    """One file, two readers: the reference's gguf_model_parse / gguf_get_tensor (gguf.c:892-1047,
    compiled unmodified into oracle/_ref) and tie_gguf_open.  Tensor types, dims, byte sizes, the
    position of every MoE tensor in the file and its bytes must agree, and so must the metadata
    keys the Qwen3-MoE loader reads (model_qwen3.c:54-63).  The reference places the data section
    on a 32-byte boundary whatever general.alignment says (gguf.c:941), so the file uses 32."""
    import ctypes
    L = _ref_gguf_lib()
    if L is None:
        pytest.skip("oracle/_ref/libtie_ref.so not built (needs the reference sources)")

    class RefTensor(ctypes.Structure):  # GGUFTensor, gguf.h:82-90
        _fields_ = [("name", ctypes.c_char_p), ("dimensions", ctypes.c_uint64 * 4), ("n_dims", ctypes.c_uint32),
                    ("type", ctypes.c_uint32), ("data", ctypes.c_void_p), ("offset", ctypes.c_int64), ("size", ctypes.c_size_t)]

    class RefModel(ctypes.Structure):  # struct GGUFModel, main.h:79-94 (leading fields)
        _fields_ = [("fd", ctypes.c_int), ("file_size", ctypes.c_size_t), ("mapped_data", ctypes.c_void_p), ("fptr", ctypes.c_void_p),
                    ("metadata_num", ctypes.c_uint64), ("tensor_count", ctypes.c_uint64), ("tensor_loaded", ctypes.c_uint64),
                    ("tensor_data_offset", ctypes.c_uint64)]

    kvs, tensors, _ = moe_model(SHAPE, 2, down_types=[synth.GGML_Q6_K, synth.GGML_Q4_K])
    # real model files carry general.basename, and the reference's detect_architecture (model.c:65-96)
    # reads it without a NULL check for the "qwen3" family
    kvs = kvs + [("general.basename", "str", "Qwen3")]
    p = str(tmp_path / "m.gguf")
    write_gguf(p, kvs, tensors, version=3, align=32)
    raw = open(p, "rb").read()
    rg = L.gguf_model_parse(p.encode())
    assert rg, "the reference's parser refused the file"
    try:
        rm = RefModel.from_address(rg)
        with gguf.GgufFile(p) as g:
            assert rm.tensor_count == g.n_tensors and rm.metadata_num == g.n_kv and rm.file_size == len(raw)
            # metadata of model_qwen3.c:54-63, read the way the reference's loader does (memcpy of the stored value)
            cfg = g.moe_config()
            for key, want in (("qwen3moe.block_count", cfg["n_layers"]), ("qwen3moe.embedding_length", cfg["hidden"]),
                              ("qwen3moe.expert_count", cfg["n_expert"]), ("qwen3moe.expert_used_count", cfg["top_k"]),
                              ("qwen3moe.expert_feed_forward_length", cfg["ffn_dim"])):
                v = ctypes.c_uint32(0)
                assert L.gguf_metadata_get_value(rg, key.encode(), ctypes.byref(v)) == 0
                assert v.value == want == g.get_int(key)
            eps = ctypes.c_float(0)
            assert L.gguf_metadata_get_value(rg, b"qwen3moe.attention.layer_norm_rms_epsilon", ctypes.byref(eps)) == 0
            assert eps.value == np.float32(cfg["norm_eps"])
            assert L.gguf_metadata_get_string(rg, b"general.architecture").decode() == cfg["arch"]
            names = [f"blk.{i}.{t}.weight" for i in range(2)
                     for t in ("ffn_gate_inp", "ffn_gate_exps", "ffn_up_exps", "ffn_down_exps", "ffn_norm", "attn_q")]
            for name in names + ["token_embd.weight"]:
                rt_p = L.gguf_get_tensor(rg, name.encode())
                assert rt_p, name
                rt = RefTensor.from_address(rt_p)
                data, typ, dims = g.tensor(name)
                assert typ == rt.type and rt.n_dims == len(dims) and list(rt.dimensions[:rt.n_dims]) == dims, name
                assert data.nbytes == rt.size, name
                off = rt.data - rm.mapped_data  # where the reference reads the tensor from
                assert off == rm.tensor_data_offset + rt.offset
                mine = np.frombuffer(data, dtype=np.uint8) if not isinstance(data, np.ndarray) else data.view(np.uint8).reshape(-1)
                assert bytes(mine[:64]) == raw[off:off + 64] and bytes(mine[-64:]) == raw[off + rt.size - 64:off + rt.size], name
                assert bytes(mine) == raw[off:off + rt.size], name
    finally:
        L.gguf_model_close(rg)
