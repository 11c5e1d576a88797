"""TEST INFRASTRUCTURE — ctypes front-end of oracle/libmoe_oracle.so (moe_oracle.c).

The plain-C restatement of the reference's AVX2 MoE feed-forward path.  Only tests, the smoke
check and the CPU-baseline leg of the benchmark may import this module; the product never does.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmoe_oracle.so")


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "moe_oracle.c")
    if force or not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(
            ["gcc", "-O2", "-mavx2", "-mfma", "-ffp-contract=off", "-fno-fast-math", "-fPIC", "-shared",
             "-fopenmp", "-o", LIB_PATH, src, "-lm"]
        )
    return LIB_PATH


class _Layer(ctypes.Structure):
    _fields_ = [
        ("hidden", ctypes.c_int), ("n_expert", ctypes.c_int), ("top_k", ctypes.c_int), ("ffn_dim", ctypes.c_int),
        ("router_w", ctypes.c_void_p),
        ("gate", ctypes.c_void_p), ("up", ctypes.c_void_p), ("down", ctypes.c_void_p),
        ("gate_type", ctypes.c_int), ("up_type", ctypes.c_int), ("down_type", ctypes.c_int),
        ("silu_table", ctypes.c_void_p),
    ]


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build()
        L = ctypes.CDLL(LIB_PATH)
        vp, i32, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
        L.oracle_silu_table_init.argtypes = [vp]
        L.oracle_swiglu.argtypes = [vp, vp, vp, i32]
        L.oracle_mat_vec.restype = i32
        L.oracle_mat_vec.argtypes = [vp, vp, i32, vp, i32, i32]
        L.oracle_rms_norm.argtypes = [vp, vp, vp, i32, f32]
        L.oracle_moe_ffn.restype = i32
        L.oracle_moe_ffn.argtypes = [vp, vp, i32, vp, vp, vp, vp, vp, i32]
        L.oracle_route.argtypes = [vp, vp, i32, vp, vp, vp, vp]
        L.oracle_route_lfm2.argtypes = [vp, vp, i32, vp, vp, vp, vp]
        L.oracle_route_lfm2.restype = None
        L.oracle_moe_block_inplace.restype = i32
        L.oracle_moe_block_inplace.argtypes = [vp, vp, i32, vp, f32, vp, vp, vp, vp, i32]
        L.oracle_expert_rows.restype = i32
        L.oracle_expert_rows.argtypes = [vp, vp, vp, i32, vp]
        L.oracle_time_moe_ffn.restype = ctypes.c_double
        L.oracle_time_moe_ffn.argtypes = [vp, vp, i32, vp, vp]
        _lib = L
    return _lib


def silu_table() -> np.ndarray:
    t = np.empty(8192, dtype=np.float32)
    lib().oracle_silu_table_init(t.ctypes.data)
    return t


def _p(a):
    return None if a is None else a.ctypes.data


class PortMoe:
    def __init__(self, layer, silu: np.ndarray | None = None):
        """layer: tie_b200.synth.MoeLayer with all experts.  silu: the 8192-entry table
        (defaults to the restated silu_table_init)."""
        assert layer.first_expert == 0
        self.L = lib()
        self.layer = layer
        self.silu = np.ascontiguousarray(silu if silu is not None else silu_table(), dtype=np.float32)
        s = layer.shape
        self.shape = s
        self.c = _Layer(s.hidden, s.n_expert, s.top_k, s.ffn_dim, layer.router_w.ctypes.data,
                        layer.gate.ctypes.data, layer.up.ctypes.data, layer.down.ctypes.data,
                        layer.gate_type, layer.up_type, layer.down_type, self.silu.ctypes.data)

    def moe_ffn(self, x, router_bias=None, want_logits=False, parallel=2):
        s = self.shape
        x = np.ascontiguousarray(x, dtype=np.float32)
        T = x.shape[0]
        out = np.empty((T, s.hidden), dtype=np.float32)
        idx = np.empty((T, s.top_k), dtype=np.int32)
        w = np.empty((T, s.top_k), dtype=np.float32)
        logits = np.empty((T, s.n_expert), dtype=np.float32) if want_logits else None
        if router_bias is not None:
            router_bias = np.ascontiguousarray(router_bias, dtype=np.float32)
        rc = self.L.oracle_moe_ffn(ctypes.byref(self.c), x.ctypes.data, T, _p(router_bias), out.ctypes.data,
                                   idx.ctypes.data, w.ctypes.data, _p(logits), parallel)
        if rc:
            raise RuntimeError(f"oracle_moe_ffn failed: {rc}")
        return (out, idx, w, logits) if want_logits else (out, idx, w)

    def route(self, x, router_bias=None):
        s = self.shape
        x = np.ascontiguousarray(x, dtype=np.float32)
        T = x.shape[0]
        idx = np.empty((T, s.top_k), dtype=np.int32)
        w = np.empty((T, s.top_k), dtype=np.float32)
        logits = np.empty((T, s.n_expert), dtype=np.float32)
        if router_bias is not None:
            router_bias = np.ascontiguousarray(router_bias, dtype=np.float32)
        self.L.oracle_route(ctypes.byref(self.c), x.ctypes.data, T, _p(router_bias), idx.ctypes.data,
                            w.ctypes.data, logits.ctypes.data)
        return idx, w, logits

    def route_lfm2(self, x, sel_bias=None):
        """LFM2-MoE routing (model_lfm2.c:438-473): ids, L1-normalised sigmoid gates, sigmoid scores."""
        s = self.shape
        x = np.ascontiguousarray(x, dtype=np.float32)
        T = x.shape[0]
        idx = np.empty((T, s.top_k), dtype=np.int32)
        w = np.empty((T, s.top_k), dtype=np.float32)
        scores = np.empty((T, s.n_expert), dtype=np.float32)
        if sel_bias is not None:
            sel_bias = np.ascontiguousarray(sel_bias, dtype=np.float32)
        self.L.oracle_route_lfm2(ctypes.byref(self.c), x.ctypes.data, T, _p(sel_bias), idx.ctypes.data,
                                 w.ctypes.data, scores.ctypes.data)
        return idx, w, scores

    def moe_ffn_lfm2(self, x, sel_bias=None):
        """The LFM2-MoE branch (model_lfm2.c:414-498): LFM2 routing, the same expert FFNs, the
        weighted accumulation in slot order."""
        s = self.shape
        x = np.ascontiguousarray(x, dtype=np.float32)
        idx, w, _ = self.route_lfm2(x, sel_bias)
        y = self.expert_rows(np.repeat(x, s.top_k, axis=0), idx.reshape(-1)).reshape(x.shape[0], s.top_k, s.hidden)
        out = np.zeros_like(x)
        for j in range(s.top_k):
            out += w[:, j:j + 1] * y[:, j, :]
        return out, idx, w

    def moe_block_inplace(self, hidden, norm_w=None, eps=1e-6, parallel=2):
        s = self.shape
        h = np.array(hidden, dtype=np.float32, order="C", copy=True)
        T = h.shape[0]
        if norm_w is None:
            norm_w = np.ones(s.hidden, dtype=np.float32)
        norm_w = np.ascontiguousarray(norm_w, dtype=np.float32)
        normed = np.empty_like(h)
        ffn = np.empty_like(h)
        idx = np.empty((T, s.top_k), dtype=np.int32)
        w = np.empty((T, s.top_k), dtype=np.float32)
        rc = self.L.oracle_moe_block_inplace(ctypes.byref(self.c), h.ctypes.data, T, norm_w.ctypes.data, eps,
                                             normed.ctypes.data, ffn.ctypes.data, idx.ctypes.data, w.ctypes.data,
                                             parallel)
        if rc:
            raise RuntimeError(f"oracle_moe_block_inplace failed: {rc}")
        return h, normed, ffn, idx, w

    def expert_rows(self, x_rows, row_expert):
        x_rows = np.ascontiguousarray(x_rows, dtype=np.float32)
        row_expert = np.ascontiguousarray(row_expert, dtype=np.int32)
        y = np.empty_like(x_rows)
        self.L.oracle_expert_rows(ctypes.byref(self.c), x_rows.ctypes.data, row_expert.ctypes.data,
                                  x_rows.shape[0], y.ctypes.data)
        return y

    def time_moe_ffn(self, x, router_bias=None) -> float:
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = np.empty_like(x)
        if router_bias is not None:
            router_bias = np.ascontiguousarray(router_bias, dtype=np.float32)
        return float(self.L.oracle_time_moe_ffn(ctypes.byref(self.c), x.ctypes.data, x.shape[0],
                                                _p(router_bias), out.ctypes.data))


def mat_vec(x, w, w_type, in_dim, out_dim):
    x = np.ascontiguousarray(x, dtype=np.float32)
    o = np.empty(out_dim, dtype=np.float32)
    rc = lib().oracle_mat_vec(x.ctypes.data, w.ctypes.data, w_type, o.ctypes.data, in_dim, out_dim)
    if rc:
        raise RuntimeError("unsupported weight type")
    return o


def swiglu(table, gate, up):
    g = np.array(gate, dtype=np.float32, order="C", copy=True)
    u = np.ascontiguousarray(up, dtype=np.float32)
    table = np.ascontiguousarray(table, dtype=np.float32)
    lib().oracle_swiglu(table.ctypes.data, g.ctypes.data, u.ctypes.data, g.size)
    return g


def rms_norm(x, w, eps):
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    o = np.empty_like(x)
    lib().oracle_rms_norm(x.ctypes.data, w.ctypes.data, o.ctypes.data, x.size, eps)
    return o
