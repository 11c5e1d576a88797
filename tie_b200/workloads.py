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


# dram__bytes_read.sum + dram__bytes_write.sum per launch of the two grouped GEMM kernels on the
# 512-token prefill workload, from the ncu capture summarised in
# profiles/grouped_gemm_sb_prefill512.md (bench.py reports them as roofline.traffic).
NCU_DRAM_BYTES_PER_LAUNCH = {"gate_up_tc": 282442752, "down_tc": 197401600}


def _main() -> None:
    """`python -m tie_b200.workloads decode1|batch64|prefill512 [--steps N]`: a few passes of one
    workload through the C ABI on cuda:0 with nothing else around them — the command the
    profiler captures (the kernels of the pass are then the only launches of the process after
    the one-off upload)."""
    import argparse

    import torch

    from . import moe

    ap = argparse.ArgumentParser()
    ap.add_argument("workload", choices=["decode1", "batch64", "prefill512"])
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--chain", action="store_true", help="decode1: the three chained decode kernels instead of the one-kernel step")
    args = ap.parse_args()
    n_tokens = {"decode1": 1, "batch64": 64, "prefill512": 512}[args.workload]
    be = moe.MoeBackend(max_tokens=n_tokens, silu_table=moe.silu_table_default())
    be.upload_layer(0, synth.make_layer(BASE_SEED))
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    be.set_stream(stream.cuda_stream)
    x = torch.from_numpy(synth.make_x(BASE_SEED, n_tokens)).cuda()
    out = torch.empty_like(x)
    flush = torch.empty(64 * 1024 * 1024, dtype=torch.float32, device="cuda")  # 256 MB > L2
    for _ in range(args.steps):
        flush.zero_()
        be.moe_ffn_ptr(0, x, out, n_tokens, moe.DEVICE | (moe.PATH_DECODE_CHAIN if args.chain else 0))
    be.synchronize()
    be.close()
    print(f"{args.workload}: {args.steps} passes ok")


if __name__ == "__main__":
    _main()
