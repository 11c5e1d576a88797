"""Deterministic synthetic Qwen3-MoE block inputs (ctypes front-end of tie_synth.c).

A Qwen3-30B-A3B GGUF is not available where this code is measured, so weights and
activations with the shapes and value distributions of that model's MoE block are
generated from (seed, stream, index).  The block formats are the reference's
block_q4_k / block_q6_k (gguf.h:100-113); tensor layouts are the reference's stacked
expert tensors (expert-major, then output row, then blocks along the input dim —
engine.c:929-950).
"""
from __future__ import annotations

import ctypes
import os
import subprocess
import threading
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libtie_synth.so")

STREAM_ROUTER, STREAM_GATE, STREAM_UP, STREAM_DOWN, STREAM_X, STREAM_BIAS = 1, 2, 3, 4, 5, 6
Q4K_BYTES, Q6K_BYTES, QK_K = 144, 210, 256
GGML_F32, GGML_Q4_K, GGML_Q6_K = 0, 12, 14  # GGMLType values, gguf.h:7-40

_lib = None
_lock = threading.Lock()


def build(force: bool = False) -> str:
    """Compile tie_synth.c into libtie_synth.so next to it (gcc, no dependencies)."""
    src = os.path.join(_HERE, "tie_synth.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(
            ["gcc", "-O2", "-ffp-contract=off", "-fno-fast-math", "-fPIC", "-shared", "-o", _LIB_PATH, src]
        )
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(_LIB_PATH):
                build()
            L = ctypes.CDLL(_LIB_PATH)
            u64, vp, i32 = ctypes.c_uint64, ctypes.c_void_p, ctypes.c_int
            L.tie_synth_u64.restype = u64
            L.tie_synth_u64.argtypes = [u64, i32, u64]
            for name in ("tie_synth_q4k", "tie_synth_q6k"):
                f = getattr(L, name)
                f.restype = None
                f.argtypes = [vp, u64, i32, u64, u64]
            L.tie_synth_normal_f32.restype = None
            L.tie_synth_normal_f32.argtypes = [vp, u64, i32, u64, u64, ctypes.c_float]
            L.tie_synth_zipf_logp.restype = None
            L.tie_synth_zipf_logp.argtypes = [vp, vp, i32, u64, ctypes.c_double]
            L.tie_synth_f32_to_f16.restype = ctypes.c_uint16
            L.tie_synth_f32_to_f16.argtypes = [ctypes.c_float]
            L.tie_synth_f16_to_f32.restype = ctypes.c_float
            L.tie_synth_f16_to_f32.argtypes = [ctypes.c_uint16]
            _lib = L
    return _lib


def _parallel(fn, total: int, n_threads: int, min_chunk: int):
    """Run fn(first, count) over [0,total) on a few threads (ctypes releases the GIL)."""
    n_threads = max(1, min(n_threads, (total + min_chunk - 1) // min_chunk))
    if n_threads == 1:
        fn(0, total)
        return
    step = (total + n_threads - 1) // n_threads
    ts = []
    for i in range(n_threads):
        a = i * step
        c = min(step, total - a)
        if c <= 0:
            break
        t = threading.Thread(target=fn, args=(a, c))
        t.start()
        ts.append(t)
    for t in ts:
        t.join()


def _threads() -> int:
    return min(16, os.cpu_count() or 1)


def q4k_blocks(seed: int, stream: int, n_blocks: int, first_block: int = 0, out: np.ndarray | None = None) -> np.ndarray:
    L = lib()
    if out is None:
        out = np.empty(n_blocks * Q4K_BYTES, dtype=np.uint8)
    base = out.ctypes.data

    def fn(a, c):
        L.tie_synth_q4k(base + a * Q4K_BYTES, seed, stream, first_block + a, c)

    _parallel(fn, n_blocks, _threads(), 1 << 14)
    return out


def q6k_blocks(seed: int, stream: int, n_blocks: int, first_block: int = 0, out: np.ndarray | None = None) -> np.ndarray:
    L = lib()
    if out is None:
        out = np.empty(n_blocks * Q6K_BYTES, dtype=np.uint8)
    base = out.ctypes.data

    def fn(a, c):
        L.tie_synth_q6k(base + a * Q6K_BYTES, seed, stream, first_block + a, c)

    _parallel(fn, n_blocks, _threads(), 1 << 14)
    return out


def normal_f32(seed: int, stream: int, n: int, std: float = 1.0, first: int = 0) -> np.ndarray:
    L = lib()
    out = np.empty(n, dtype=np.float32)
    base = out.ctypes.data

    def fn(a, c):
        L.tie_synth_normal_f32(base + 4 * a, seed, stream, first + a, c, std)

    _parallel(fn, n, _threads(), 1 << 16)
    return out


def zipf_logp(n_expert: int, seed: int, s: float = 1.1):
    """ln(p_e * E) for p_e ~ rank_e^-s, and the 1-based ranks (seeded permutation)."""
    L = lib()
    out = np.empty(n_expert, dtype=np.float32)
    ranks = np.empty(n_expert, dtype=np.int32)
    L.tie_synth_zipf_logp(out.ctypes.data, ranks.ctypes.data, n_expert, seed, s)
    return out, ranks


@dataclass
class MoeShape:
    """Qwen3-30B-A3B MoE block: hidden 2048, 128 experts, top-8, expert FFN dim 768."""

    hidden: int = 2048
    n_expert: int = 128
    top_k: int = 8
    ffn_dim: int = 768

    @property
    def gate_bytes_per_expert(self) -> int:
        return self.ffn_dim * (self.hidden // QK_K) * Q4K_BYTES

    @property
    def down_bytes_per_expert(self) -> int:
        return self.hidden * (self.ffn_dim // QK_K) * Q6K_BYTES

    @property
    def expert_bytes(self) -> int:
        return 2 * self.gate_bytes_per_expert + self.down_bytes_per_expert

    @property
    def router_bytes(self) -> int:
        return self.n_expert * self.hidden * 4

    @property
    def flops_per_token(self) -> int:
        return 2 * self.n_expert * self.hidden + self.top_k * 3 * 2 * self.ffn_dim * self.hidden


@dataclass
class MoeLayer:
    """Host copies of one block's four tensors in the reference's GGUF layout."""

    shape: MoeShape
    router_w: np.ndarray  # f32 [n_expert, hidden]
    gate: np.ndarray  # u8, Q4_K [n_expert][ffn_dim][hidden/256] blocks
    up: np.ndarray  # u8, Q4_K same
    down: np.ndarray  # u8, Q6_K [n_expert][hidden][ffn_dim/256] blocks
    gate_type: int = GGML_Q4_K
    up_type: int = GGML_Q4_K
    down_type: int = GGML_Q6_K
    first_expert: int = 0
    n_local_expert: int | None = None


def make_layer(seed: int, shape: MoeShape | None = None, first_expert: int = 0, n_local_expert: int | None = None) -> MoeLayer:
    """One block's weights (seed = base_seed + layer index).  With first_expert/n_local_expert
    only that expert range of the three expert tensors is generated (expert parallelism);
    the bytes equal the corresponding slice of the full tensors."""
    shape = shape or MoeShape()
    nloc = shape.n_expert - first_expert if n_local_expert is None else n_local_expert
    router = normal_f32(seed, STREAM_ROUTER, shape.n_expert * shape.hidden, 0.02).reshape(shape.n_expert, shape.hidden)
    gu_blocks = shape.ffn_dim * (shape.hidden // QK_K)
    dn_blocks = shape.hidden * (shape.ffn_dim // QK_K)
    gate = q4k_blocks(seed, STREAM_GATE, nloc * gu_blocks, first_expert * gu_blocks)
    up = q4k_blocks(seed, STREAM_UP, nloc * gu_blocks, first_expert * gu_blocks)
    down = q6k_blocks(seed, STREAM_DOWN, nloc * dn_blocks, first_expert * dn_blocks)
    return MoeLayer(shape, router, gate, up, down, first_expert=first_expert, n_local_expert=nloc)


def make_x(seed: int, n_tokens: int, hidden: int = 2048, first_token: int = 0) -> np.ndarray:
    """Activations x ~ N(0,1), fp32 [n_tokens, hidden]; rows first_token.. of the seeded stream."""
    return normal_f32(seed, STREAM_X, n_tokens * hidden, 1.0, first_token * hidden).reshape(n_tokens, hidden)
