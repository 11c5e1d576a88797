"""TEST INFRASTRUCTURE — ctypes front-end of oracle/_ref/libtie_ref.so.

That library is the reference's own C sources compiled unmodified (oracle/Makefile, target
`ref`) plus ref_harness.c, which re-drives the per-token MoE loop of model_qwen3.c:415-470
by calling the reference's compiled functions.  Nothing here is on the product path: only
tests, the smoke check and the CPU-baseline leg of the benchmark may import this module.
"""
from __future__ import annotations

import ctypes
import os
import sys

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libtie_ref.so")
LIB_NATIVE_PATH = os.path.join(_HERE, "_ref", "libtie_ref_native.so")
# the same sources + the reference-side glue of tie_b200/dropin, linked with tie_b200/libtie_cuda.so
LIB_DROPIN_PATH = os.path.join(_HERE, "_ref", "libtie_ref_dropin.so")


def available(path: str = LIB_PATH) -> bool:
    return os.path.exists(path)


class RefMoe:
    """One process-wide instance per loaded library (the reference keeps its thread pool and
    SiLU table in globals, threadpool.c:6 and engine.c:12)."""

    def __init__(self, hidden=2048, n_expert=128, top_k=8, ffn_dim=768, n_threads=None, path: str = LIB_PATH):
        if not os.path.exists(path):
            raise FileNotFoundError(f"{path} not built (make -C oracle ref REF=<reference sources>)")
        L = ctypes.CDLL(path)
        vp, i32, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
        L.tieref_init.restype = i32
        L.tieref_init.argtypes = [i32] * 5
        L.tieref_num_threads.restype = i32
        L.tieref_get_silu_table.argtypes = [vp]
        L.tieref_set_layer.argtypes = [vp, vp, i32, vp, i32, vp, i32, vp]
        L.tieref_moe_ffn.restype = i32
        L.tieref_moe_ffn.argtypes = [vp, i32, vp, vp, vp, vp, vp]
        L.tieref_route_lfm2.restype = i32
        L.tieref_route_lfm2.argtypes = [vp, i32, vp, vp, vp, vp]
        L.tieref_moe_block_inplace.restype = i32
        L.tieref_moe_block_inplace.argtypes = [vp, i32, f32, vp, vp, vp, vp]
        L.tieref_mat_vec.argtypes = [vp, vp, i32, vp, i32, i32]
        L.tieref_swiglu.argtypes = [vp, vp, i32]
        L.tieref_rms_norm.argtypes = [vp, vp, vp, i32, f32]
        L.tieref_time_moe_ffn.restype = ctypes.c_double
        L.tieref_time_moe_ffn.argtypes = [vp, i32, vp, vp]
        if hasattr(L, "tieref_dropin_load"):
            L.tieref_dropin_load.restype = i32
            L.tieref_dropin_load.argtypes = [i32, i32]
            L.tieref_dropin_moe_ffn.restype = i32
            L.tieref_dropin_moe_ffn.argtypes = [vp, i32, vp]
            L.tieref_dropin_unload.restype = None
        self.L = L
        self.hidden, self.n_expert, self.top_k, self.ffn_dim = hidden, n_expert, top_k, ffn_dim
        if n_threads is None:
            n_threads = min(os.cpu_count() or 8, 32)
        # math_dispatch_init() prints a banner to stdout; keep it out of callers' output
        sys.stdout.flush()
        saved = os.dup(1)
        devnull = os.open(os.devnull, os.O_WRONLY)
        try:
            os.dup2(devnull, 1)
            L.tieref_init(hidden, n_expert, top_k, ffn_dim, n_threads)
        finally:
            os.dup2(saved, 1)
            os.close(saved)
            os.close(devnull)
        self.n_threads = L.tieref_num_threads()
        self._keep = None

    def silu_table(self) -> np.ndarray:
        t = np.empty(8192, dtype=np.float32)
        self.L.tieref_get_silu_table(t.ctypes.data)
        return t

    def set_layer(self, layer, ffn_norm_w: np.ndarray | None = None):
        """layer: tie_b200.synth.MoeLayer holding ALL experts (first_expert == 0)."""
        assert layer.first_expert == 0
        if ffn_norm_w is None:
            ffn_norm_w = np.ones(self.hidden, dtype=np.float32)
        self._keep = (layer, ffn_norm_w)
        self.L.tieref_set_layer(
            layer.router_w.ctypes.data,
            layer.gate.ctypes.data, layer.gate_type,
            layer.up.ctypes.data, layer.up_type,
            layer.down.ctypes.data, layer.down_type,
            ffn_norm_w.ctypes.data,
        )

    def moe_ffn(self, x: np.ndarray, router_bias: np.ndarray | None = None, want_logits: bool = False):
        x = np.ascontiguousarray(x, dtype=np.float32)
        T = x.shape[0]
        out = np.empty((T, self.hidden), dtype=np.float32)
        idx = np.empty((T, self.top_k), dtype=np.int32)
        w = np.empty((T, self.top_k), dtype=np.float32)
        logits = np.empty((T, self.n_expert), dtype=np.float32) if want_logits else None
        bias_p = None
        if router_bias is not None:
            router_bias = np.ascontiguousarray(router_bias, dtype=np.float32)
            bias_p = router_bias.ctypes.data
        rc = self.L.tieref_moe_ffn(
            x.ctypes.data, T, bias_p, out.ctypes.data, idx.ctypes.data, w.ctypes.data,
            logits.ctypes.data if want_logits else None,
        )
        if rc:
            raise RuntimeError(f"tieref_moe_ffn failed: {rc}")
        return (out, idx, w, logits) if want_logits else (out, idx, w)

    def route_lfm2(self, x: np.ndarray, sel_bias: np.ndarray | None = None):
        """Routing step of the LFM2-MoE branch (model_lfm2.c:438-473): ids, gates, sigmoid scores."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        T = x.shape[0]
        idx = np.empty((T, self.top_k), dtype=np.int32)
        w = np.empty((T, self.top_k), dtype=np.float32)
        scores = np.empty((T, self.n_expert), dtype=np.float32)
        bias_p = None
        if sel_bias is not None:
            sel_bias = np.ascontiguousarray(sel_bias, dtype=np.float32)
            bias_p = sel_bias.ctypes.data
        rc = self.L.tieref_route_lfm2(x.ctypes.data, T, bias_p, idx.ctypes.data, w.ctypes.data, scores.ctypes.data)
        if rc:
            raise RuntimeError(f"tieref_route_lfm2 failed: {rc}")
        return idx, w, scores

    # -- the drop-in library only (LIB_DROPIN_PATH): the reference's structures driving the GPU backend --
    def dropin_load(self, device: int = 0, max_tokens: int = 512):
        """The glue's model_load hook on the layer given to set_layer (tie_cuda_qwen3_load)."""
        rc = self.L.tieref_dropin_load(device, max_tokens)
        if rc:
            raise RuntimeError(f"tieref_dropin_load failed: {rc}")

    def dropin_moe_ffn(self, x: np.ndarray) -> np.ndarray:
        """The is_moe branch through the glue (tie_cuda_qwen3_moe_ffn): ctx->mem.normed_ffn_input -> ffn_down_output."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = np.empty_like(x)
        rc = self.L.tieref_dropin_moe_ffn(x.ctypes.data, x.shape[0], out.ctypes.data)
        if rc:
            raise RuntimeError(f"tieref_dropin_moe_ffn failed: {rc}")
        return out

    def dropin_unload(self):
        self.L.tieref_dropin_unload()

    def moe_block_inplace(self, hidden: np.ndarray, eps: float = 1e-6):
        """hidden += MoE(RMSNorm(hidden)); returns (new_hidden, normed, ffn_out, idx, w)."""
        h = np.array(hidden, dtype=np.float32, order="C", copy=True)
        T = h.shape[0]
        normed = np.empty_like(h)
        ffn = np.empty_like(h)
        idx = np.empty((T, self.top_k), dtype=np.int32)
        w = np.empty((T, self.top_k), dtype=np.float32)
        rc = self.L.tieref_moe_block_inplace(h.ctypes.data, T, eps, normed.ctypes.data, ffn.ctypes.data, idx.ctypes.data, w.ctypes.data)
        if rc:
            raise RuntimeError(f"tieref_moe_block_inplace failed: {rc}")
        return h, normed, ffn, idx, w

    def mat_vec(self, x: np.ndarray, w: np.ndarray, w_type: int, in_dim: int, out_dim: int) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        o = np.empty(out_dim, dtype=np.float32)
        self.L.tieref_mat_vec(x.ctypes.data, w.ctypes.data, w_type, o.ctypes.data, in_dim, out_dim)
        return o

    def swiglu(self, gate: np.ndarray, up: np.ndarray) -> np.ndarray:
        g = np.array(gate, dtype=np.float32, order="C", copy=True)
        u = np.ascontiguousarray(up, dtype=np.float32)
        self.L.tieref_swiglu(g.ctypes.data, u.ctypes.data, g.size)
        return g

    def rms_norm(self, x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        w = np.ascontiguousarray(w, dtype=np.float32)
        o = np.empty_like(x)
        self.L.tieref_rms_norm(x.ctypes.data, w.ctypes.data, o.ctypes.data, x.size, eps)
        return o

    def time_moe_ffn(self, x: np.ndarray, router_bias: np.ndarray | None = None) -> float:
        """Seconds for x.shape[0] tokens through the reference path (after one warm token)."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = np.empty_like(x)
        bias_p = None
        if router_bias is not None:
            router_bias = np.ascontiguousarray(router_bias, dtype=np.float32)
            bias_p = router_bias.ctypes.data
        return float(self.L.tieref_time_moe_ffn(x.ctypes.data, x.shape[0], bias_p, out.ctypes.data))
