// Device functions of the router shared by its kernels (router.cu) and the one-kernel decode
// step (decode_fused.cu): the AVX2 horizontal sum and the per-token selection.
#pragma once

#include "common.cuh"

namespace tie {

// hsum over the 8 lanes of one expert held in 8 consecutive threads of a warp.
__device__ __forceinline__ float hsum8_lanes(float acc)
{
	float v = __fadd_rn(acc, __shfl_down_sync(0xffffffffu, acc, 4, 8));  // lanes 0..3: l+l4
	float t = __fadd_rn(v, __shfl_down_sync(0xffffffffu, v, 1, 8));	     // lane 0: s0+s1, lane 2: s2+s3
	float r = __fadd_rn(t, __shfl_down_sync(0xffffffffu, t, 2, 8));	     // lane 0: (s0+s1)+(s2+s3)
	return r;
}

// One warp per token: k rounds of warp arg-max with key (score desc, index asc), then the
// softmax of the selected scores: max-subtract, expf, sequential sum, multiply by 1/sum.
__device__ __forceinline__ void topk_softmax_warp(const float *__restrict__ logits, int token, int lane, int n_expert, int top_k,
						  int *__restrict__ topk_idx, float *__restrict__ topk_w)
{
	const float *lg = logits + (size_t)token * n_expert;
	// lane holds experts lane, lane+32, ... (up to 8 per lane: n_expert <= 256)
	float v[8];
	const int per = (n_expert + 31) / 32;
#pragma unroll
	for (int i = 0; i < 8; i++) {
		int e = lane + 32 * i;
		v[i] = (i < per && e < n_expert) ? __ldcg(lg + e) : -INFINITY;
	}
	unsigned taken = 0;
	float my_score = 0.0f;
	int my_idx = -1;
	for (int r = 0; r < top_k; r++) {
		float best = -INFINITY;
		int bi = 0x7fffffff;
#pragma unroll
		for (int i = 0; i < 8; i++) {
			int e = lane + 32 * i;
			bool ok = !(taken & (1u << i)) && i < per && e < n_expert;
			// strictly greater wins; within a lane indices ascend, so ties keep the lower index
			if (ok && (v[i] > best || bi == 0x7fffffff)) {
				best = v[i];
				bi = e;
			}
		}
#pragma unroll
		for (int o = 16; o > 0; o >>= 1) {
			float ob = __shfl_xor_sync(0xffffffffu, best, o);
			int oi = __shfl_xor_sync(0xffffffffu, bi, o);
			bool take = (oi != 0x7fffffff) && (bi == 0x7fffffff || ob > best || (ob == best && oi < bi));
			if (take) {
				best = ob;
				bi = oi;
			}
		}
		if (bi != 0x7fffffff && (bi & 31) == lane)
			taken |= 1u << (bi >> 5);
		if (lane == r) {
			my_score = best;
			my_idx = (bi == 0x7fffffff) ? -1 : bi;
		}
	}
	// softmax over lanes 0..top_k-1 (scores are already sorted descending: lane 0 is the max)
	float mx = __shfl_sync(0xffffffffu, my_score, 0);
	float ex = (lane < top_k) ? expf(__fsub_rn(my_score, mx)) : 0.0f;
	float sum = 0.0f;
	for (int j = 0; j < top_k; j++)
		sum = __fadd_rn(sum, __shfl_sync(0xffffffffu, ex, j));
	float inv = __fdiv_rn(1.0f, sum);
	if (lane < top_k) {
		topk_idx[(size_t)token * top_k + lane] = my_idx;
		topk_w[(size_t)token * top_k + lane] = __fmul_rn(ex, inv);
	}
}

}  // namespace tie
