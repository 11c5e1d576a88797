"""Host-side front-end of libtie_cuda.so: the same calls, argument meaning and error codes as
include/tie_cuda.h, for Python drivers (tests, benchmark, expert-parallel runner).

The compute is entirely in the CUDA library.  If the library is missing or a call fails this
module raises — there is no CPU path behind it.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtie_cuda.so")

HOST, DEVICE, NO_SYNC, GRAPH = 0, 1, 2, 4
PATH_AUTO, PATH_STREAM, PATH_TENSOR = 0, 1 << 8, 2 << 8
PATH_LEGACY_STREAM = 1 << 10
PATH_DECODE_CHAIN = 1 << 11  # one token: three chained decode kernels instead of the single cooperative one
ROUTE_LFM2 = 1 << 12  # LFM2-MoE routing: sigmoid, selection bias, L1-normalised gates (model_lfm2.c:438-473)
PATH_NO_PAIR = 1 << 14  # tensor path: single-CTA grouped GEMM instead of CTA pairs
EP_REPLICATED = 1 << 13  # expert-parallel decode: the same 1-4 tokens on every rank
N_SLOTS = 4  # TIE_CUDA_N_SLOTS: host-buffer calls that can be in flight (moe_ffn_submit / moe_ffn_wait)
OK, EINVAL, ENOTSUP, ENOMEM, ECUDA, ENODEV, EKERNEL, ETOOBIG = 0, -1, -2, -3, -4, -5, -6, -7

# every symbol include/tie_cuda.h declares
EXPORTS = [
    "tie_cuda_init", "tie_cuda_destroy", "tie_cuda_strerror", "tie_cuda_last_cuda_error", "tie_cuda_set_stream",
    "tie_cuda_synchronize", "tie_cuda_silu_table_default", "tie_cuda_upload_moe_layer", "tie_cuda_weight_bytes",
    "tie_cuda_moe_ffn", "tie_cuda_moe_ffn_submit", "tie_cuda_moe_ffn_wait", "tie_cuda_moe_block_inplace", "tie_cuda_moe_stack_inplace", "tie_cuda_moe_route", "tie_cuda_moe_ffn_biased",
    "tie_cuda_moe_expert_rows", "tie_cuda_moe_combine", "tie_cuda_make_current", "tie_cuda_register_tensor",
    "tie_cuda_mat_vec_row_f32_q4k_f32", "tie_cuda_mat_vec_row_f32_q6k_f32", "tie_cuda_mat_vec_row_f32_f32_f32",
    "tie_cuda_swiglu_f32_f32", "tie_cuda_dispatch_status", "tie_cuda_launch_count", "tie_cuda_last_active_experts",
    "tie_cuda_version", "tie_cuda_set_profiling", "tie_cuda_get_profile", "tie_cuda_moe_ep_dispatch",
    "tie_cuda_moe_ep_combine", "tie_cuda_route_noalloc", "tie_cuda_ep_region", "tie_cuda_ep_ipc_handle",
    "tie_cuda_ep_attach", "tie_cuda_ep_detach", "tie_cuda_ep_set_timeout_ms", "tie_cuda_ep_publish", "tie_cuda_ep_compute",
    "tie_cuda_ep_gather", "tie_cuda_moe_ffn_ep", "tie_cuda_mat_mat",
    "tie_cuda_moe_block_inplace_ep",
]
EP_HANDLE_BYTES = 64
EP_PEER_POINTERS, EP_PEER_IPC_HANDLES = 0, 1
PHASES = ["router", "sort", "split", "gate_up", "swiglu", "down", "combine"]


class TieCudaError(RuntimeError):
    def __init__(self, code: int, what: str, detail: str = ""):
        self.code = code
        super().__init__(f"{what}: {code} ({detail})" if detail else f"{what}: {code}")


class Config(ctypes.Structure):
    _fields_ = [
        ("device", ctypes.c_int), ("hidden", ctypes.c_int), ("n_expert", ctypes.c_int), ("top_k", ctypes.c_int),
        ("ffn_dim", ctypes.c_int), ("n_layers", ctypes.c_int), ("max_tokens", ctypes.c_int),
        ("norm_eps", ctypes.c_float), ("silu_table", ctypes.c_void_p), ("ep_rank", ctypes.c_int),
        ("ep_size", ctypes.c_int),
    ]


_lib = None


def load_library() -> ctypes.CDLL:
    """dlopen the CUDA library and bind argument types.  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise FileNotFoundError(
            f"{LIB_PATH} is missing: build it with `python -m tie_b200.build` (nvcc, sm_100a). "
            "This package has no CPU implementation of the MoE path.")
    L = ctypes.CDLL(LIB_PATH)
    vp, i32, u32, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint, ctypes.c_float
    L.tie_cuda_init.restype = i32
    L.tie_cuda_init.argtypes = [ctypes.POINTER(vp), ctypes.POINTER(Config)]
    L.tie_cuda_destroy.restype = None
    L.tie_cuda_destroy.argtypes = [vp]
    L.tie_cuda_strerror.restype = ctypes.c_char_p
    L.tie_cuda_strerror.argtypes = [i32]
    L.tie_cuda_last_cuda_error.restype = ctypes.c_char_p
    L.tie_cuda_last_cuda_error.argtypes = [vp]
    L.tie_cuda_set_stream.restype = i32
    L.tie_cuda_set_stream.argtypes = [vp, vp]
    L.tie_cuda_synchronize.restype = i32
    L.tie_cuda_synchronize.argtypes = [vp]
    L.tie_cuda_silu_table_default.restype = None
    L.tie_cuda_silu_table_default.argtypes = [vp]
    L.tie_cuda_upload_moe_layer.restype = i32
    L.tie_cuda_upload_moe_layer.argtypes = [vp, i32, vp, vp, i32, vp, i32, vp, i32, vp]
    L.tie_cuda_weight_bytes.restype = ctypes.c_size_t
    L.tie_cuda_weight_bytes.argtypes = [vp]
    L.tie_cuda_moe_ffn.restype = i32
    L.tie_cuda_moe_ffn.argtypes = [vp, i32, vp, vp, i32, u32]
    L.tie_cuda_moe_ffn_biased.restype = i32
    L.tie_cuda_moe_ffn_biased.argtypes = [vp, i32, vp, vp, i32, vp, u32]
    L.tie_cuda_moe_block_inplace.restype = i32
    L.tie_cuda_moe_block_inplace.argtypes = [vp, i32, vp, i32, u32]
    L.tie_cuda_moe_ffn_submit.restype = i32
    L.tie_cuda_moe_ffn_submit.argtypes = [vp, i32, vp, vp, i32, i32, u32]
    L.tie_cuda_moe_ffn_wait.restype = i32
    L.tie_cuda_moe_ffn_wait.argtypes = [vp, i32]
    L.tie_cuda_moe_stack_inplace.restype = i32
    L.tie_cuda_moe_stack_inplace.argtypes = [vp, i32, i32, vp, i32, u32]
    L.tie_cuda_moe_route.restype = i32
    L.tie_cuda_moe_route.argtypes = [vp, i32, vp, i32, vp, vp, vp, vp, u32]
    L.tie_cuda_moe_expert_rows.restype = i32
    L.tie_cuda_moe_expert_rows.argtypes = [vp, i32, vp, vp, i32, vp, u32]
    L.tie_cuda_moe_combine.restype = i32
    L.tie_cuda_moe_combine.argtypes = [vp, vp, vp, i32, vp, u32]
    L.tie_cuda_moe_ep_dispatch.restype = i32
    L.tie_cuda_moe_ep_dispatch.argtypes = [vp, vp, vp, i32, vp, vp, vp, u32]
    L.tie_cuda_moe_ep_combine.restype = i32
    L.tie_cuda_moe_ep_combine.argtypes = [vp, vp, vp, i32, vp, u32]
    L.tie_cuda_route_noalloc.restype = i32
    L.tie_cuda_route_noalloc.argtypes = [vp, vp, vp, i32, i32, i32, i32, vp, vp, vp]
    L.tie_cuda_make_current.restype = i32
    L.tie_cuda_make_current.argtypes = [vp]
    L.tie_cuda_register_tensor.restype = i32
    L.tie_cuda_register_tensor.argtypes = [vp, vp, ctypes.c_size_t, i32, i32]
    for n in ("tie_cuda_mat_vec_row_f32_q4k_f32", "tie_cuda_mat_vec_row_f32_q6k_f32", "tie_cuda_mat_vec_row_f32_f32_f32"):
        f = getattr(L, n)
        f.restype = None
        f.argtypes = [vp, vp, vp, i32, i32, i32]
    L.tie_cuda_swiglu_f32_f32.restype = None
    L.tie_cuda_swiglu_f32_f32.argtypes = [vp, vp, i32]
    L.tie_cuda_dispatch_status.restype = i32
    L.tie_cuda_launch_count.restype = ctypes.c_uint64
    L.tie_cuda_launch_count.argtypes = [vp]
    L.tie_cuda_last_active_experts.restype = i32
    L.tie_cuda_last_active_experts.argtypes = [vp]
    L.tie_cuda_version.restype = ctypes.c_char_p
    L.tie_cuda_set_profiling.restype = i32
    L.tie_cuda_set_profiling.argtypes = [vp, i32]
    L.tie_cuda_get_profile.restype = i32
    L.tie_cuda_get_profile.argtypes = [vp, vp]
    L.tie_cuda_ep_region.restype = i32
    L.tie_cuda_ep_region.argtypes = [vp, ctypes.POINTER(vp), ctypes.POINTER(ctypes.c_size_t)]
    L.tie_cuda_ep_ipc_handle.restype = i32
    L.tie_cuda_ep_ipc_handle.argtypes = [vp, vp]
    L.tie_cuda_ep_attach.restype = i32
    L.tie_cuda_ep_attach.argtypes = [vp, ctypes.POINTER(vp), i32, i32]
    L.tie_cuda_ep_detach.restype = i32
    L.tie_cuda_ep_detach.argtypes = [vp]
    L.tie_cuda_ep_set_timeout_ms.restype = i32
    L.tie_cuda_ep_set_timeout_ms.argtypes = [vp, i32]
    L.tie_cuda_ep_publish.restype = i32
    L.tie_cuda_ep_publish.argtypes = [vp, i32, vp, i32, vp, u32]
    L.tie_cuda_ep_compute.restype = i32
    L.tie_cuda_ep_compute.argtypes = [vp, i32, u32]
    L.tie_cuda_ep_gather.restype = i32
    L.tie_cuda_ep_gather.argtypes = [vp, vp, vp, u32]
    L.tie_cuda_moe_ffn_ep.restype = i32
    L.tie_cuda_moe_ffn_ep.argtypes = [vp, i32, vp, vp, i32, u32]
    L.tie_cuda_moe_block_inplace_ep.restype = i32
    L.tie_cuda_moe_block_inplace_ep.argtypes = [vp, i32, vp, i32, u32]
    L.tie_cuda_mat_mat.restype = i32
    L.tie_cuda_mat_mat.argtypes = [vp, vp, vp, vp, i32, i32, i32, u32]
    _lib = L
    return L


def silu_table_default() -> np.ndarray:
    t = np.empty(8192, dtype=np.float32)
    load_library().tie_cuda_silu_table_default(t.ctypes.data)
    return t


def _ptr(a):
    """Address of a numpy array / torch tensor / int / None."""
    if a is None:
        return None
    if isinstance(a, int):
        return a
    if isinstance(a, np.ndarray):
        assert a.flags["C_CONTIGUOUS"]
        return a.ctypes.data
    if hasattr(a, "data_ptr"):
        assert a.is_contiguous()
        return a.data_ptr()
    raise TypeError(type(a))


class MoeBackend:
    """One tie_cuda context (one GPU).  Mirrors the C entry points one to one."""

    def __init__(self, hidden=2048, n_expert=128, top_k=8, ffn_dim=768, n_layers=1, max_tokens=4096, device=0,
                 norm_eps=1e-6, silu_table: np.ndarray | None = None, ep_rank=0, ep_size=1):
        self.L = load_library()
        self._silu = None if silu_table is None else np.ascontiguousarray(silu_table, dtype=np.float32)
        cfg = Config(device, hidden, n_expert, top_k, ffn_dim, n_layers, max_tokens, norm_eps,
                     None if self._silu is None else self._silu.ctypes.data, ep_rank, ep_size)
        self.cfg = cfg
        h = ctypes.c_void_p()
        rc = self.L.tie_cuda_init(ctypes.byref(h), ctypes.byref(cfg))
        if rc:
            raise TieCudaError(rc, "tie_cuda_init", self.L.tie_cuda_strerror(rc).decode())
        self.h = h
        self.hidden, self.n_expert, self.top_k, self.ffn_dim = hidden, n_expert, top_k, ffn_dim
        self.n_layers, self.max_tokens = n_layers, max_tokens
        self.ep_rank, self.ep_size = ep_rank, ep_size
        self._host_keep = {}

    # -- lifetime --
    def close(self):
        if getattr(self, "h", None):
            self.L.tie_cuda_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc: int, what: str):
        if rc:
            detail = self.L.tie_cuda_strerror(rc).decode()
            extra = self.L.tie_cuda_last_cuda_error(self.h).decode()
            raise TieCudaError(rc, what, f"{detail}; {extra}" if extra else detail)

    def set_stream(self, cuda_stream: int | None):
        self._check(self.L.tie_cuda_set_stream(self.h, cuda_stream), "tie_cuda_set_stream")

    def synchronize(self):
        self._check(self.L.tie_cuda_synchronize(self.h), "tie_cuda_synchronize")

    def set_profiling(self, on: bool):
        self._check(self.L.tie_cuda_set_profiling(self.h, 1 if on else 0), "tie_cuda_set_profiling")

    def get_profile(self):
        """(dict phase -> ms, used_tensor_path) for the most recent feed-forward call."""
        ms = (ctypes.c_float * len(PHASES))()
        rc = self.L.tie_cuda_get_profile(self.h, ms)
        if rc < 0:
            self._check(rc, "tie_cuda_get_profile")
        return {n: float(ms[i]) for i, n in enumerate(PHASES)}, bool(rc)

    @property
    def launch_count(self) -> int:
        return int(self.L.tie_cuda_launch_count(self.h))

    @property
    def weight_bytes(self) -> int:
        return int(self.L.tie_cuda_weight_bytes(self.h))

    def last_active_experts(self) -> int:
        n = self.L.tie_cuda_last_active_experts(self.h)
        if n < 0:
            self._check(n, "tie_cuda_last_active_experts")
        return n

    # -- weights --
    def upload_layer(self, layer_idx: int, layer, ffn_norm_w: np.ndarray | None = None, keep_host: bool = False):
        """layer: tie_b200.synth.MoeLayer (for ep_size > 1 its expert tensors hold this rank's experts)."""
        if ffn_norm_w is not None:
            ffn_norm_w = np.ascontiguousarray(ffn_norm_w, dtype=np.float32)
        rc = self.L.tie_cuda_upload_moe_layer(
            self.h, layer_idx, layer.router_w.ctypes.data, layer.gate.ctypes.data, layer.gate_type,
            layer.up.ctypes.data, layer.up_type, layer.down.ctypes.data, layer.down_type, _ptr(ffn_norm_w))
        self._check(rc, "tie_cuda_upload_moe_layer")
        if keep_host:
            self._host_keep[layer_idx] = layer

    # -- compute: numpy in / numpy out (host pointers) --
    def moe_ffn(self, layer_idx: int, x: np.ndarray, router_bias: np.ndarray | None = None, path: int = PATH_AUTO,
                out: np.ndarray | None = None, lfm2: bool = False) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        if out is None:
            out = np.empty_like(x)
        if router_bias is not None:
            router_bias = np.ascontiguousarray(router_bias, dtype=np.float32)
        rc = self.L.tie_cuda_moe_ffn_biased(self.h, layer_idx, x.ctypes.data, out.ctypes.data, x.shape[0],
                                            _ptr(router_bias), HOST | path | (ROUTE_LFM2 if lfm2 else 0))
        self._check(rc, "tie_cuda_moe_ffn")
        return out

    def route(self, layer_idx: int, x: np.ndarray, router_bias: np.ndarray | None = None, want_logits: bool = True,
              lfm2: bool = False):
        x = np.ascontiguousarray(x, dtype=np.float32)
        T = x.shape[0]
        idx = np.empty((T, self.top_k), dtype=np.int32)
        w = np.empty((T, self.top_k), dtype=np.float32)
        logits = np.empty((T, self.n_expert), dtype=np.float32) if want_logits else None
        if router_bias is not None:
            router_bias = np.ascontiguousarray(router_bias, dtype=np.float32)
        rc = self.L.tie_cuda_moe_route(self.h, layer_idx, x.ctypes.data, T, _ptr(router_bias), idx.ctypes.data,
                                       w.ctypes.data, _ptr(logits), HOST | (ROUTE_LFM2 if lfm2 else 0))
        self._check(rc, "tie_cuda_moe_route")
        return idx, w, logits

    # -- compute: raw pointers (device tensors owned by the caller, e.g. torch) --
    def moe_ffn_ptr(self, layer_idx: int, x, out, n_tokens: int, flags: int = DEVICE, router_bias=None):
        rc = self.L.tie_cuda_moe_ffn_biased(self.h, layer_idx, _ptr(x), _ptr(out), n_tokens, _ptr(router_bias), flags)
        self._check(rc, "tie_cuda_moe_ffn")

    def moe_block_inplace_ptr(self, layer_idx: int, hidden, n_tokens: int, flags: int = DEVICE):
        rc = self.L.tie_cuda_moe_block_inplace(self.h, layer_idx, _ptr(hidden), n_tokens, flags)
        self._check(rc, "tie_cuda_moe_block_inplace")

    def moe_ffn_submit(self, layer_idx: int, x_host, out_host, n_tokens: int, slot: int, flags: int = 0):
        """x_host / out_host: pinned host tensors or arrays; returns at once (see tie_cuda_moe_ffn_submit)."""
        rc = self.L.tie_cuda_moe_ffn_submit(self.h, layer_idx, _ptr(x_host), _ptr(out_host), n_tokens, slot, flags)
        self._check(rc, "tie_cuda_moe_ffn_submit")

    def moe_ffn_wait(self, slot: int):
        rc = self.L.tie_cuda_moe_ffn_wait(self.h, slot)
        self._check(rc, "tie_cuda_moe_ffn_wait")

    def moe_stack_inplace_ptr(self, first_layer: int, n_layers: int, hidden, n_tokens: int, flags: int = DEVICE):
        rc = self.L.tie_cuda_moe_stack_inplace(self.h, first_layer, n_layers, _ptr(hidden), n_tokens, flags)
        self._check(rc, "tie_cuda_moe_stack_inplace")

    def route_ptr(self, layer_idx: int, x, n_tokens: int, topk_idx, topk_w, logits=None, router_bias=None, flags: int = DEVICE):
        rc = self.L.tie_cuda_moe_route(self.h, layer_idx, _ptr(x), n_tokens, _ptr(router_bias), _ptr(topk_idx),
                                       _ptr(topk_w), _ptr(logits), flags)
        self._check(rc, "tie_cuda_moe_route")

    def expert_rows_ptr(self, layer_idx: int, x_rows, row_expert, n_rows: int, y_rows, flags: int = DEVICE):
        rc = self.L.tie_cuda_moe_expert_rows(self.h, layer_idx, _ptr(x_rows), _ptr(row_expert), n_rows, _ptr(y_rows), flags)
        self._check(rc, "tie_cuda_moe_expert_rows")

    def combine_ptr(self, y_rows, topk_w, n_tokens: int, out, flags: int = DEVICE):
        rc = self.L.tie_cuda_moe_combine(self.h, _ptr(y_rows), _ptr(topk_w), n_tokens, _ptr(out), flags)
        self._check(rc, "tie_cuda_moe_combine")

    def ep_dispatch_ptr(self, x, topk_idx, n_tokens: int, send_rows, send_expert, expert_counts, flags: int = DEVICE):
        rc = self.L.tie_cuda_moe_ep_dispatch(self.h, _ptr(x), _ptr(topk_idx), n_tokens, _ptr(send_rows), _ptr(send_expert),
                                             _ptr(expert_counts), flags)
        self._check(rc, "tie_cuda_moe_ep_dispatch")

    def ep_combine_ptr(self, y_sorted, topk_w, n_tokens: int, out, flags: int = DEVICE):
        rc = self.L.tie_cuda_moe_ep_combine(self.h, _ptr(y_sorted), _ptr(topk_w), n_tokens, _ptr(out), flags)
        self._check(rc, "tie_cuda_moe_ep_combine")

    # -- expert parallelism over peer memory --
    def ep_region(self):
        """(device address, bytes) of the region this rank exposes to its peers."""
        base, nbytes = ctypes.c_void_p(), ctypes.c_size_t()
        self._check(self.L.tie_cuda_ep_region(self.h, ctypes.byref(base), ctypes.byref(nbytes)), "tie_cuda_ep_region")
        return int(base.value), int(nbytes.value)

    def ep_ipc_handle(self) -> bytes:
        buf = ctypes.create_string_buffer(EP_HANDLE_BYTES)
        self._check(self.L.tie_cuda_ep_ipc_handle(self.h, buf), "tie_cuda_ep_ipc_handle")
        return buf.raw

    def ep_attach(self, peers, kind: int):
        """peers: per rank, a device address (EP_PEER_POINTERS) or a 64-byte handle (EP_PEER_IPC_HANDLES)."""
        n = len(peers)
        arr = (ctypes.c_void_p * n)()
        keep = []
        for i, p in enumerate(peers):
            if kind == EP_PEER_IPC_HANDLES:
                b = ctypes.create_string_buffer(bytes(p), EP_HANDLE_BYTES)
                keep.append(b)
                arr[i] = ctypes.cast(b, ctypes.c_void_p).value
            else:
                arr[i] = p
        self._check(self.L.tie_cuda_ep_attach(self.h, arr, n, kind), "tie_cuda_ep_attach")

    def ep_detach(self):
        self._check(self.L.tie_cuda_ep_detach(self.h), "tie_cuda_ep_detach")

    def ep_set_timeout_ms(self, ms: int):
        self._check(self.L.tie_cuda_ep_set_timeout_ms(self.h, ms), "tie_cuda_ep_set_timeout_ms")

    def ep_publish_ptr(self, layer_idx: int, x, n_tokens: int, router_bias=None, flags: int = DEVICE):
        self._check(self.L.tie_cuda_ep_publish(self.h, layer_idx, _ptr(x), n_tokens, _ptr(router_bias), flags), "tie_cuda_ep_publish")

    def ep_compute(self, layer_idx: int, flags: int = DEVICE):
        self._check(self.L.tie_cuda_ep_compute(self.h, layer_idx, flags), "tie_cuda_ep_compute")

    def ep_gather_ptr(self, out, residual=None, flags: int = DEVICE):
        self._check(self.L.tie_cuda_ep_gather(self.h, _ptr(out), _ptr(residual), flags), "tie_cuda_ep_gather")

    def moe_ffn_ep_ptr(self, layer_idx: int, x, out, n_tokens: int, flags: int = DEVICE):
        self._check(self.L.tie_cuda_moe_ffn_ep(self.h, layer_idx, _ptr(x), _ptr(out), n_tokens, flags), "tie_cuda_moe_ffn_ep")

    def moe_block_inplace_ep_ptr(self, layer_idx: int, hidden, n_tokens: int, flags: int = DEVICE):
        rc = self.L.tie_cuda_moe_block_inplace_ep(self.h, layer_idx, _ptr(hidden), n_tokens, flags)
        self._check(rc, "tie_cuda_moe_block_inplace_ep")

    # -- math_dispatch rows --
    def make_current(self):
        self._check(self.L.tie_cuda_make_current(self.h), "tie_cuda_make_current")

    def register_tensor(self, host: np.ndarray, ggml_type: int, in_dim: int):
        rc = self.L.tie_cuda_register_tensor(self.h, host.ctypes.data, host.nbytes, ggml_type, in_dim)
        self._check(rc, "tie_cuda_register_tensor")

    def mat_mat(self, w_host: np.ndarray, x, out, batch_len: int, in_dim: int, out_dim: int, flags: int = 0):
        """dispatch_mat_mat on a registered Q4_K / Q6_K tensor (w_host: the array given to register_tensor)."""
        rc = self.L.tie_cuda_mat_mat(self.h, w_host.ctypes.data, _ptr(x), _ptr(out), batch_len, in_dim, out_dim, flags)
        self._check(rc, "tie_cuda_mat_mat")
        return out

    def dispatch_mat_vec(self, x: np.ndarray, w_host_ptr: int, ggml_type: int, in_dim: int, start_row: int, end_row: int,
                         out: np.ndarray | None = None) -> np.ndarray:
        """Calls the dispatch-row function for ggml_type exactly as the reference's tables would."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        if out is None:
            out = np.zeros(end_row, dtype=np.float32)
        fn = {0: self.L.tie_cuda_mat_vec_row_f32_f32_f32, 12: self.L.tie_cuda_mat_vec_row_f32_q4k_f32,
              14: self.L.tie_cuda_mat_vec_row_f32_q6k_f32}[ggml_type]
        fn(x.ctypes.data, w_host_ptr, out.ctypes.data, in_dim, start_row, end_row)
        st = self.L.tie_cuda_dispatch_status()
        if st:
            self.L.tie_cuda_make_current(self.h)  # clears the sticky status
            raise TieCudaError(st, "tie_cuda_mat_vec_row", self.L.tie_cuda_strerror(st).decode())
        return out

    def dispatch_swiglu(self, gate: np.ndarray, up: np.ndarray) -> np.ndarray:
        g = np.array(gate, dtype=np.float32, order="C", copy=True)
        u = np.ascontiguousarray(up, dtype=np.float32)
        self.L.tie_cuda_swiglu_f32_f32(g.ctypes.data, u.ctypes.data, g.size)
        st = self.L.tie_cuda_dispatch_status()
        if st:
            self.L.tie_cuda_make_current(self.h)
            raise TieCudaError(st, "tie_cuda_swiglu_f32_f32", self.L.tie_cuda_strerror(st).decode())
        return g
