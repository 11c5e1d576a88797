"""GGUF reader for the MoE feed-forward tensors (ctypes front-end of tie_gguf.c, include/tie_gguf.h).

Replaces, for this path only, the reference's gguf_model_parse / gguf_model_map_weights
(gguf.c:892-1047) and the per-layer tensor lookup (model.c:237-293; names model_qwen3.c:39-52):
the file is mapped, indexed, and the tensors of a block are handed to tie_cuda_upload_moe_layer as
pointers into the mapping — the "upload once at load" half of the drop-in.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
import threading

import numpy as np

from .. import synth

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtie_gguf.so")
EXPORTS = [
    "tie_gguf_open", "tie_gguf_close", "tie_gguf_strerror", "tie_gguf_version", "tie_gguf_tensor_count",
    "tie_gguf_kv_count", "tie_gguf_get_u64", "tie_gguf_get_f32", "tie_gguf_get_str", "tie_gguf_find_tensor",
    "tie_gguf_moe_config_read", "tie_gguf_moe_layer_read",
]
OK, EIO, EFORMAT, ENOTFOUND, ETYPE, EINVAL = 0, -1, -2, -3, -4, -5

_lib = None
_lock = threading.Lock()


class GgufError(RuntimeError):
    def __init__(self, code: int, what: str):
        super().__init__(what)
        self.code = code


class _Tensor(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p), ("nbytes", ctypes.c_uint64), ("type", ctypes.c_uint32),
                ("n_dims", ctypes.c_uint32), ("dims", ctypes.c_uint64 * 4)]


class _Config(ctypes.Structure):
    _fields_ = [("n_layers", ctypes.c_uint32), ("hidden", ctypes.c_uint32), ("n_expert", ctypes.c_uint32),
                ("top_k", ctypes.c_uint32), ("ffn_dim", ctypes.c_uint32), ("norm_eps", ctypes.c_float),
                ("arch", ctypes.c_char * 32)]


class _Layer(ctypes.Structure):
    _fields_ = [("router_w", ctypes.c_void_p), ("gate_exps", ctypes.c_void_p), ("up_exps", ctypes.c_void_p),
                ("down_exps", ctypes.c_void_p), ("ffn_norm_w", ctypes.c_void_p), ("gate_type", ctypes.c_int),
                ("up_type", ctypes.c_int), ("down_type", ctypes.c_int)]


def build(force: bool = False) -> str:
    """Compile tie_gguf.c into libtie_gguf.so next to it (gcc, no dependencies)."""
    src = os.path.join(_HERE, "tie_gguf.c")
    hdr = os.path.join(_HERE, "..", "..", "include", "tie_gguf.h")
    if force or not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < max(os.path.getmtime(src), os.path.getmtime(hdr)):
        subprocess.check_call(["gcc", "-O2", "-Wall", "-Wextra", "-fPIC", "-shared", "-o", LIB_PATH, src])
    return LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    with _lock:
        if _lib is None:
            build()
            L = ctypes.CDLL(LIB_PATH)
            vp, cp, u64p = ctypes.c_void_p, ctypes.c_char_p, ctypes.POINTER(ctypes.c_uint64)
            L.tie_gguf_open.argtypes = [cp, ctypes.POINTER(vp), cp, ctypes.c_size_t]
            L.tie_gguf_close.argtypes = [vp]
            L.tie_gguf_close.restype = None
            L.tie_gguf_strerror.argtypes = [ctypes.c_int]
            L.tie_gguf_strerror.restype = cp
            L.tie_gguf_version.argtypes = [vp]
            L.tie_gguf_version.restype = ctypes.c_uint32
            for n in ("tie_gguf_tensor_count", "tie_gguf_kv_count"):
                getattr(L, n).argtypes = [vp]
                getattr(L, n).restype = ctypes.c_uint64
            L.tie_gguf_get_u64.argtypes = [vp, cp, u64p]
            L.tie_gguf_get_f32.argtypes = [vp, cp, ctypes.POINTER(ctypes.c_float)]
            L.tie_gguf_get_str.argtypes = [vp, cp, cp, ctypes.c_size_t]
            L.tie_gguf_find_tensor.argtypes = [vp, cp, ctypes.POINTER(_Tensor)]
            L.tie_gguf_moe_config_read.argtypes = [vp, ctypes.POINTER(_Config)]
            L.tie_gguf_moe_layer_read.argtypes = [vp, ctypes.POINTER(_Config), ctypes.c_int, ctypes.POINTER(_Layer)]
            _lib = L
        return _lib


def _view(ptr: int, nbytes: int, dtype) -> np.ndarray:
    """numpy view (no copy) of nbytes at ptr inside the mapping."""
    buf = (ctypes.c_uint8 * nbytes).from_address(ptr)
    return np.frombuffer(buf, dtype=dtype)


class GgufFile:
    """A mapped GGUF file.  Arrays returned by tensor() / moe_layer() alias the mapping and must not
    be used after close()."""

    def __init__(self, path: str):
        self.L = lib()
        h = ctypes.c_void_p()
        err = ctypes.create_string_buffer(256)
        rc = self.L.tie_gguf_open(os.fsencode(path), ctypes.byref(h), err, len(err))
        if rc != OK:
            raise GgufError(rc, err.value.decode() or self.L.tie_gguf_strerror(rc).decode())
        self.h = h
        self._cfg = None

    def close(self):
        if self.h:
            self.L.tie_gguf_close(self.h)
            self.h = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def _check(self, rc: int, what: str):
        if rc != OK:
            raise GgufError(rc, f"{what}: {self.L.tie_gguf_strerror(rc).decode()}")

    @property
    def version(self) -> int:
        return int(self.L.tie_gguf_version(self.h))

    @property
    def n_tensors(self) -> int:
        return int(self.L.tie_gguf_tensor_count(self.h))

    @property
    def n_kv(self) -> int:
        return int(self.L.tie_gguf_kv_count(self.h))

    def get_int(self, key: str) -> int:
        v = ctypes.c_uint64()
        self._check(self.L.tie_gguf_get_u64(self.h, key.encode(), ctypes.byref(v)), key)
        return int(v.value)

    def get_float(self, key: str) -> float:
        v = ctypes.c_float()
        self._check(self.L.tie_gguf_get_f32(self.h, key.encode(), ctypes.byref(v)), key)
        return float(v.value)

    def get_str(self, key: str) -> str:
        buf = ctypes.create_string_buffer(256)
        self._check(self.L.tie_gguf_get_str(self.h, key.encode(), buf, len(buf)), key)
        return buf.value.decode()

    def tensor(self, name: str):
        """(bytes as uint8 view, GGMLType, dims with the contiguous dimension first)."""
        t = _Tensor()
        self._check(self.L.tie_gguf_find_tensor(self.h, name.encode(), ctypes.byref(t)), name)
        return _view(t.data, int(t.nbytes), np.uint8), int(t.type), [int(t.dims[i]) for i in range(t.n_dims)]

    def moe_config(self) -> dict:
        c = _Config()
        self._check(self.L.tie_gguf_moe_config_read(self.h, ctypes.byref(c)), "MoE metadata")
        self._cfg = c
        return {"arch": c.arch.decode(), "n_layers": c.n_layers, "hidden": c.hidden, "n_expert": c.n_expert,
                "top_k": c.top_k, "ffn_dim": c.ffn_dim, "norm_eps": c.norm_eps}

    def moe_layer(self, layer: int):
        """(tie_b200.synth.MoeLayer whose arrays alias the mapping, ffn_norm weights or None)."""
        if self._cfg is None:
            self.moe_config()
        c = self._cfg
        out = _Layer()
        self._check(self.L.tie_gguf_moe_layer_read(self.h, ctypes.byref(c), layer, ctypes.byref(out)), f"blk.{layer}")
        shape = synth.MoeShape(hidden=c.hidden, n_expert=c.n_expert, top_k=c.top_k, ffn_dim=c.ffn_dim)
        bb = {synth.GGML_Q4_K: synth.Q4K_BYTES, synth.GGML_Q6_K: synth.Q6K_BYTES}
        gu = c.n_expert * c.ffn_dim * (c.hidden // synth.QK_K)
        dn = c.n_expert * c.hidden * (c.ffn_dim // synth.QK_K)
        ml = synth.MoeLayer(
            shape, _view(out.router_w, c.n_expert * c.hidden * 4, np.float32).reshape(c.n_expert, c.hidden),
            _view(out.gate_exps, gu * bb[out.gate_type], np.uint8), _view(out.up_exps, gu * bb[out.up_type], np.uint8),
            _view(out.down_exps, dn * bb[out.down_type], np.uint8),
            gate_type=out.gate_type, up_type=out.up_type, down_type=out.down_type)
        norm = _view(out.ffn_norm_w, c.hidden * 4, np.float32) if out.ffn_norm_w else None
        return ml, norm


def upload_model(be, g: GgufFile, layers=None) -> int:
    """Uploads the MoE tensors of the given blocks (default: all the backend has room for) to the
    backend's HBM — what model_load_weights + the residency hook do at load.  Returns the count."""
    cfg = g.moe_config()
    layers = range(min(cfg["n_layers"], be.n_layers)) if layers is None else layers
    n = 0
    for i in layers:
        ml, norm = g.moe_layer(i)
        be.upload_layer(i, ml, ffn_norm_w=norm)
        n += 1
    return n
