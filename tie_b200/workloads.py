"""The benchmark's workloads: seeded synthetic stand-ins for a Qwen3-30B-A3B MoE block.

decode1   1 token                       (HBM-bound: 25.5 MB of packed weights per token-block)
prefill   512 tokens                    (the configuration the headline metric is quoted on)
batch64   64 tokens, uniform or skewed  (skew: Zipf(1.1) router-logit bias, ~30 % of the
                                         assignments on the 4 most popular experts)
ep8192    8192 tokens, expert parallel
stack     48 blocks, h += MoE(RMSNorm(h))

All inputs come from tie_b200.synth with base seed 0 (1000 for the stack).
"""
from __future__ import annotations

import numpy as np

from . import synth

BASE_SEED = 0
STACK_BASE_SEED = 1000


def skew_bias(logits: np.ndarray, top_k: int, seed: int = BASE_SEED, s: float = 1.1, target: float = 0.30,
              n_hot: int = 4):
    """Router-logit bias alpha * ln(p_e * E), p_e ~ rank_e^-s, with alpha found by bisection so that
    the n_hot most popular experts receive `target` of the assignments for the given unbiased
    logits [T, E].  Returns (bias [E] float32, alpha, achieved share)."""
    T, E = logits.shape
    logp, ranks = synth.zipf_logp(E, seed, s)
    hot = np.argsort(ranks)[:n_hot]

    def share(alpha: float) -> float:
        b = (np.float32(alpha) * logp).astype(np.float32)
        lg = logits + b[None, :]
        top = np.argsort(-lg, axis=1, kind="stable")[:, :top_k]
        return float(np.isin(top, hot).sum()) / float(T * top_k)

    lo, hi = 0.0, 1.0
    while share(hi) < target and hi < 64:
        hi *= 2
    for _ in range(40):
        mid = 0.5 * (lo + hi)
        if share(mid) < target:
            lo = mid
        else:
            hi = mid
    alpha = hi
    bias = (np.float32(alpha) * logp).astype(np.float32)
    return bias, float(alpha), share(alpha)


def rel_rms_err(got: np.ndarray, ref: np.ndarray) -> np.ndarray:
    """Per token: max_k |got - ref| / rms_k(ref).  The parity bound on this path is 1e-3."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    rms = np.sqrt((ref * ref).mean(axis=-1))
    return np.abs(got - ref).max(axis=-1) / np.maximum(rms, 1e-30)


def algorithmic_bytes(shape: synth.MoeShape, n_tokens: int, active_experts: int) -> int:
    """Bytes a block must move: router weights + packed weights of every expert that received a
    token (once) + the activations in and out."""
    return shape.router_bytes + active_experts * shape.expert_bytes + 2 * n_tokens * shape.hidden * 4


def algorithmic_flops(shape: synth.MoeShape, n_tokens: int) -> int:
    """One multiply-add per weight element per token (never the split passes)."""
    return n_tokens * shape.flops_per_token
