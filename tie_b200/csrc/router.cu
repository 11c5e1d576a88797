// Router: logits = x . W_router^T (bit-exact replay of the reference's AVX2 F32 mat-vec),
// optional bias, top-k with the reference's tie rule, softmax over the selected logits.
//
// Reference: dispatch_mat_vec on ffn_gate_inp (model_qwen3.c:431) -> mat_vec_row_f32_f32_f32_avx2
// (math_avx2.c:228-256): 8 independent lanes, lane l accumulates fma(x[8i+l], w[8i+l], acc_l)
// for i = 0..in_dim/8-1 in order, then hsum (math_avx2.c:14-21):
// ((l0+l4)+(l1+l5)) + ((l2+l6)+(l3+l7)).  Replaying that order gives bit-identical logits, which
// is what makes the top-k selection identical (the 8th/9th logit gap can be a few ulp).
// find_top_k: engine.c:891-914 (strict '>': ties keep the lower expert index, output sorted by
// score descending).  softmax: engine.c:864-888 over the k selected raw logits.
#include <mutex>

#include "common.cuh"
#include "ep_dev.cuh"
#include "kernels.cuh"

#include "router_topk.cuh"

namespace tie {

// Large token counts: CTA = TT tokens x EPC experts; thread = (expert, lane); router weights come
// straight from L2 (each loaded value feeds TT fused multiply-adds), x is staged in k-chunks.
template <int TT, int EPC, int KC>
__global__ void __launch_bounds__(EPC * 8) router_logits_tile(const float *__restrict__ x, const float *__restrict__ w,
							      const float *__restrict__ bias, float *__restrict__ logits,
							      int n_tokens, int hidden, int n_expert)
{
	__shared__ float xs[TT][KC];
	const int t0 = blockIdx.x * TT;
	const int e = blockIdx.y * EPC + (threadIdx.x >> 3);
	const int l = threadIdx.x & 7;
	const float *wr = w + (size_t)e * hidden;
	float acc[TT];
#pragma unroll
	for (int i = 0; i < TT; i++)
		acc[i] = 0.0f;
	for (int k0 = 0; k0 < hidden; k0 += KC) {
		__syncthreads();
		for (int i = threadIdx.x; i < TT * (KC / 4); i += EPC * 8) {
			int tt = i / (KC / 4), c = i % (KC / 4);
			float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
			if (t0 + tt < n_tokens)
				v = *reinterpret_cast<const float4 *>(x + (size_t)(t0 + tt) * hidden + k0 + 4 * c);
			*reinterpret_cast<float4 *>(&xs[tt][4 * c]) = v;
		}
		__syncthreads();
#pragma unroll 8
		for (int i = 0; i < KC / 8; i++) {
			float wv = __ldg(wr + k0 + 8 * i + l);
#pragma unroll
			for (int tt = 0; tt < TT; tt++)
				acc[tt] = __fmaf_rn(xs[tt][8 * i + l], wv, acc[tt]);
		}
	}
#pragma unroll
	for (int tt = 0; tt < TT; tt++) {
		float r = hsum8_lanes(acc[tt]);
		if (l == 0 && t0 + tt < n_tokens) {
			if (bias)
				r = __fadd_rn(r, bias[e]);
			logits[(size_t)(t0 + tt) * n_expert + e] = r;
		}
	}
}

// Batched token counts: thread = one AVX2 lane l of a TPT-token x EPT-expert register tile (each
// of its chains a strict i-ascending sequence of fused multiply-adds, so the result stays
// bit-identical).  The limit of this kernel is shared-memory-to-register bandwidth (one float per
// lane per cycle), so every loaded float must feed several multiply-adds from registers.
// Operands are staged by cp.async in k chunks (a 4-deep ring); a row pitch of KC+8 floats puts
// the 4 token groups of a warp on disjoint banks, and the 4 groups share their expert rows
// (broadcast loads).
constexpr int RMT_STAGES = 4;
// The hand-over of the tokens in an expert-parallel step rides along as one more row of CTAs, of
// which as many work as there are SMs the logits' CTAs leave free (at least 16): CTAs that share an
// SM with the logits take load/store slots from them (32 working CTAs lengthened the kernel by 10 us
// at 4 GPUs, 128 by 18 us).
constexpr int RMT_PUSH_ROWS = 1;
static int rmt_push_ctas(const tie_cuda_ctx *c, int logits_ctas, int most)
{
	int n = c->sm_count - logits_ctas;
	n = n < 16 ? 16 : n;
	return n < most ? n : most;
}

// TPT x EPT = tokens x experts per thread, TE = experts per CTA, KC = k chunk.  CTA = 4 TPT
// tokens x TE experts, 8 x 4 x TE/EPT threads.
//   <4, 4, 32, 128>: 16 x 32 tiles, 256 threads, 104 KB — a few hundred tokens (parallelism first);
//   <8, 8, 64, 64>:  32 x 64 tiles, 256 threads, 108 KB, two CTAs per SM — thousands of tokens
//                    (16 loads per 64 multiply-adds instead of 8 per 16).
template <int TPT, int EPT, int TE, int KC>
struct RmtCfg {
	static constexpr int TT = 4 * TPT, PITCH = KC + 8, THREADS = 8 * 4 * (TE / EPT);
	static constexpr int STAGE_FLOATS = (TT + TE) * PITCH;
	static constexpr int SMEM = RMT_STAGES * STAGE_FLOATS * (int)sizeof(float);
};

template <int TPT, int EPT, int TE, int KC>
__global__ void __launch_bounds__((RmtCfg<TPT, EPT, TE, KC>::THREADS), 2)
router_logits_mt(const float *__restrict__ x, const float *__restrict__ w, const float *__restrict__ bias, float *__restrict__ logits,
		 int n_tokens, int hidden, int n_expert, const EpPush push)
{
	using Cfg = RmtCfg<TPT, EPT, TE, KC>;
	constexpr int TT = Cfg::TT, PITCH = Cfg::PITCH, THREADS = Cfg::THREADS;
	extern __shared__ __align__(16) float rsm[];
	// Expert-parallel steps: RMT_PUSH_ROWS more rows of CTAs (blockIdx.y past the expert tiles) store this
	// rank's tokens into every rank's memory while the others compute the logits; they share nothing
	// with them.
	if (push.x && (int)blockIdx.y * TE >= n_expert) {
		const int row = (int)blockIdx.y - n_expert / TE, cta = row * (int)gridDim.x + (int)blockIdx.x;
		if (cta < push.n_ctas)
			ep_push_tokens_cta(push, cta, push.n_ctas);
		return;
	}
	const int t0 = blockIdx.x * TT, e0 = blockIdx.y * TE;
	const int l = threadIdx.x & 7;		// AVX2 lane
	const int tg = (threadIdx.x >> 3) & 3;	// tokens tg, tg+4, tg+8, ...
	const int eg = threadIdx.x >> 5;	// experts EPT*eg .. EPT*eg+EPT-1 (one warp per expert group)
	auto stage = [&](int buf, int k0) {
		float *xs = rsm + buf * Cfg::STAGE_FLOATS;
		float *ws = xs + TT * PITCH;
		for (int i = threadIdx.x; i < (TT + TE) * (KC / 4); i += THREADS) {
			const int r = i / (KC / 4), c4 = i % (KC / 4);
			const float *src;
			float *dst;
			if (r < TT) {
				const int t = min(t0 + r, n_tokens - 1);  // rows past the end are computed and dropped
				src = x + (size_t)t * hidden + k0 + 4 * c4;
				dst = xs + r * PITCH + 4 * c4;
			} else {
				src = w + (size_t)(e0 + r - TT) * hidden + k0 + 4 * c4;
				dst = ws + (r - TT) * PITCH + 4 * c4;
			}
			asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src)
				     : "memory");
		}
		asm volatile("cp.async.commit_group;" ::: "memory");
	};
	float acc[TPT][EPT];  // [token j][expert b]
#pragma unroll
	for (int j = 0; j < TPT; j++)
#pragma unroll
		for (int b = 0; b < EPT; b++)
			acc[j][b] = 0.0f;
	const int n_chunks = hidden / KC;
#pragma unroll
	for (int c = 0; c < RMT_STAGES - 1; c++) {
		if (c < n_chunks)
			stage(c, c * KC);
		else
			asm volatile("cp.async.commit_group;" ::: "memory");
	}
	for (int c = 0; c < n_chunks; c++) {
		if (c + RMT_STAGES - 1 < n_chunks)
			stage((c + RMT_STAGES - 1) % RMT_STAGES, (c + RMT_STAGES - 1) * KC);
		else
			asm volatile("cp.async.commit_group;" ::: "memory");
		asm volatile("cp.async.wait_group %0;" ::"n"(RMT_STAGES - 1) : "memory");
		__syncthreads();
		const float *xs = rsm + (c % RMT_STAGES) * Cfg::STAGE_FLOATS;
		const float *ws = xs + TT * PITCH;
		const float *xp = xs + tg * PITCH + l;
		const float *wp = ws + (EPT * eg) * PITCH + l;
#pragma unroll 2
		for (int i = 0; i < KC / 8; i++) {
			float xv[TPT], wv[EPT];
#pragma unroll
			for (int j = 0; j < TPT; j++)
				xv[j] = xp[(4 * j) * PITCH + 8 * i];
#pragma unroll
			for (int b = 0; b < EPT; b++)
				wv[b] = wp[b * PITCH + 8 * i];
#pragma unroll
			for (int j = 0; j < TPT; j++)
#pragma unroll
				for (int b = 0; b < EPT; b++)
					acc[j][b] = __fmaf_rn(xv[j], wv[b], acc[j][b]);
		}
		__syncthreads();
	}
#pragma unroll
	for (int j = 0; j < TPT; j++) {
		const int t = t0 + tg + 4 * j;
#pragma unroll
		for (int b = 0; b < EPT; b++) {
			const int e = e0 + EPT * eg + b;
			float r = hsum8_lanes(acc[j][b]);  // lanes l = 0..7 are 8 consecutive threads
			if (l == 0 && t < n_tokens) {
				if (bias)
					r = __fadd_rn(r, bias[e]);
				logits[(size_t)t * n_expert + e] = r;
			}
		}
	}
}

// Decode-sized token counts (<= 8 tokens): one expert per CTA so the 1 MB of router weights is
// pulled by many SMs at once; the row and the tokens are staged in shared memory with wide
// loads, then thread (token, lane) runs the sequential chain.
template <int MAXT>
__global__ void __launch_bounds__(64) router_logits_decode(const float *__restrict__ x, const float *__restrict__ w,
							   const float *__restrict__ bias, float *__restrict__ logits,
							   int n_tokens, int hidden, int n_expert)
{
	extern __shared__ float sm[];
	float *ws = sm;			  // [hidden]
	float *xs = sm + hidden;	  // [n_tokens][hidden + 8]  (row pad spreads tokens over banks)
	const int xstride = hidden + 8;
	const int e = blockIdx.x;
	const float4 *wr4 = reinterpret_cast<const float4 *>(w + (size_t)e * hidden);
	for (int i = threadIdx.x; i < hidden / 4; i += 64)
		reinterpret_cast<float4 *>(ws)[i] = __ldg(wr4 + i);
	for (int i = threadIdx.x; i < n_tokens * (hidden / 4); i += 64) {
		int tt = i / (hidden / 4), c4 = i % (hidden / 4);
		*reinterpret_cast<float4 *>(xs + (size_t)tt * xstride + 4 * c4) =
			*reinterpret_cast<const float4 *>(x + (size_t)tt * hidden + 4 * c4);
	}
	__syncthreads();
	const int tt = threadIdx.x >> 3, l = threadIdx.x & 7;
	float acc = 0.0f;
	if (tt < n_tokens) {
		const float *xr = xs + (size_t)tt * xstride;
#pragma unroll 16
		for (int i = 0; i < hidden / 8; i++)
			acc = __fmaf_rn(xr[8 * i + l], ws[8 * i + l], acc);
	}
	float r = hsum8_lanes(acc);
	if (l == 0 && tt < n_tokens) {
		if (bias)
			r = __fadd_rn(r, bias[e]);
		logits[(size_t)tt * n_expert + e] = r;
	}
}

__global__ void __launch_bounds__(128) router_topk(const float *__restrict__ logits, int n_tokens, int n_expert, int top_k,
						   int *__restrict__ topk_idx, float *__restrict__ topk_w)
{
	const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
	const int lane = threadIdx.x & 31;
	if (warp >= n_tokens)
		return;
	topk_softmax_warp(logits, warp, lane, n_expert, top_k, topk_idx, topk_w);
}

// LFM2-MoE routing (model_lfm2.c:438-473), one warp per token: s = sigmoid(logit) for every
// expert, selection by the same arg-max rounds on s + sel_bias (exp_probs_b, may be null), gates =
// the UNBIASED s of the selected experts, summed in slot order and scaled by 1/(sum + 1e-6).
// logits is overwritten with the sigmoid scores (the reference does the same to expert_scores).
__global__ void __launch_bounds__(128) router_topk_lfm2(float *__restrict__ logits, const float *__restrict__ sel_bias,
							int n_tokens, int n_expert, int top_k, int *__restrict__ topk_idx,
							float *__restrict__ topk_w)
{
	const int token = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
	const int lane = threadIdx.x & 31;
	if (token >= n_tokens)
		return;
	float *lg = logits + (size_t)token * n_expert;
	float sg[8], v[8];
	const int per = (n_expert + 31) / 32;
#pragma unroll
	for (int i = 0; i < 8; i++) {
		const int e = lane + 32 * i;
		const bool in = i < per && e < n_expert;
		sg[i] = in ? __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-__ldcg(lg + e)))) : 0.0f;
		v[i] = in ? (sel_bias ? __fadd_rn(sg[i], sel_bias[e]) : sg[i]) : -INFINITY;
		if (in)
			lg[e] = sg[i];
	}
	unsigned taken = 0;
	float my_gate = 0.0f;
	int my_idx = -1;
	for (int r = 0; r < top_k; r++) {
		float best = -INFINITY, best_sg = 0.0f;
		int bi = 0x7fffffff;
#pragma unroll
		for (int i = 0; i < 8; i++) {
			const int e = lane + 32 * i;
			const bool ok = !(taken & (1u << i)) && i < per && e < n_expert;
			// strictly greater wins; within a lane indices ascend, so ties keep the lower index
			if (ok && (v[i] > best || bi == 0x7fffffff)) {
				best = v[i];
				best_sg = sg[i];
				bi = e;
			}
		}
#pragma unroll
		for (int o = 16; o > 0; o >>= 1) {
			const float ob = __shfl_xor_sync(0xffffffffu, best, o), os = __shfl_xor_sync(0xffffffffu, best_sg, o);
			const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
			const bool take = (oi != 0x7fffffff) && (bi == 0x7fffffff || ob > best || (ob == best && oi < bi));
			if (take) {
				best = ob;
				best_sg = os;
				bi = oi;
			}
		}
		if (bi != 0x7fffffff && (bi & 31) == lane)
			taken |= 1u << (bi >> 5);
		if (lane == r) {
			my_gate = best_sg;
			my_idx = (bi == 0x7fffffff) ? -1 : bi;
		}
	}
	float sum = 0.0f;
	for (int j = 0; j < top_k; j++)
		sum = __fadd_rn(sum, __shfl_sync(0xffffffffu, my_gate, j));
	const float inv = __fdiv_rn(1.0f, __fadd_rn(sum, 1e-6f));
	if (lane < top_k) {
		topk_idx[(size_t)token * top_k + lane] = my_idx;
		topk_w[(size_t)token * top_k + lane] = __fmul_rn(my_gate, inv);
	}
}

// Decode: logits as in router_logits_decode, and the CTA that finishes last (a counter, no
// waiting) runs the selection for all tokens, saving a launch on the latency-bound path.
__global__ void __launch_bounds__(256) router_decode_fused(const float *__restrict__ x, const float *__restrict__ w,
							   const float *__restrict__ bias, float *__restrict__ logits, int n_tokens,
							   int hidden, int n_expert, int top_k, int *__restrict__ topk_idx,
							   float *__restrict__ topk_w, int *__restrict__ counter)
{
	extern __shared__ float sm[];
	__shared__ int s_last;
	float *ws = sm;
	float *xs = sm + hidden;
	const int xstride = hidden + 8;
	const int e = blockIdx.x;
	// let a dependent-launched successor (the decode gate/up kernel) become resident now; it waits
	// for this grid's results itself.  The wait below covers a predecessor that was itself
	// launched the same way.
	asm volatile("griddepcontrol.wait;" ::: "memory");
	asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
	// all loads of the staging are issued before the first store (at most 8 wide loads per thread)
	{
		const float4 *wr4 = reinterpret_cast<const float4 *>(w + (size_t)e * hidden);
		const int nw = hidden / 4, nx = n_tokens * (hidden / 4);
		float4 v[8];
#pragma unroll
		for (int j = 0; j < 8; j++) {
			const int i = threadIdx.x + 256 * j;
			if (i < nw)
				v[j] = __ldg(wr4 + i);
			else if (i - nw < nx && i >= nw)
				v[j] = __ldg(reinterpret_cast<const float4 *>(x) + (i - nw));
		}
#pragma unroll
		for (int j = 0; j < 8; j++) {
			const int i = threadIdx.x + 256 * j;
			if (i < nw) {
				reinterpret_cast<float4 *>(ws)[i] = v[j];
			} else if (i - nw < nx) {
				const int k = i - nw, tt = k / (hidden / 4), c4 = k % (hidden / 4);
				*reinterpret_cast<float4 *>(xs + (size_t)tt * xstride + 4 * c4) = v[j];
			}
		}
		for (int i = threadIdx.x + 2048; i < nw + nx; i += 256) {  // sizes beyond 8 loads per thread
			if (i < nw) {
				reinterpret_cast<float4 *>(ws)[i] = __ldg(wr4 + i);
			} else {
				const int k = i - nw, tt = k / (hidden / 4), c4 = k % (hidden / 4);
				*reinterpret_cast<float4 *>(xs + (size_t)tt * xstride + 4 * c4) = __ldg(reinterpret_cast<const float4 *>(x) + k);
			}
		}
	}
	__syncthreads();
	const int tt = threadIdx.x >> 3, l = threadIdx.x & 7;
	float acc = 0.0f;
	if (tt < n_tokens) {
		const float *xr = xs + (size_t)tt * xstride;
#pragma unroll 16
		for (int i = 0; i < hidden / 8; i++)
			acc = __fmaf_rn(xr[8 * i + l], ws[8 * i + l], acc);
	}
	float r = hsum8_lanes(acc);
	if (l == 0 && tt < n_tokens) {
		if (bias)
			r = __fadd_rn(r, bias[e]);
		__stcg(&logits[(size_t)tt * n_expert + e], r);
	}
	__threadfence();
	__syncthreads();
	if (threadIdx.x == 0)
		s_last = (atomicAdd(counter, 1) == (int)gridDim.x - 1);
	__syncthreads();
	if (!s_last)
		return;
	__threadfence();
	const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
	for (int t = warp; t < n_tokens; t += 8)
		topk_softmax_warp(logits, t, lane, n_expert, top_k, topk_idx, topk_w);
	if (threadIdx.x == 0)
		*counter = 0;
}

// lfm2 = 0: bias (optional) is added to the logits, top-k + softmax over the selected logits
// (Qwen3-MoE).  lfm2 = 1: LFM2-MoE routing, bias (optional) is the selection bias exp_probs_b.
// push (expert-parallel steps): the kernel of the logits takes the hand-over of this rank's tokens to
// its peers along as extra CTAs where it can; *push_taken tells whether it did.
int launch_router(tie_cuda_ctx *c, const float *x, const float *w, const float *bias, int n_tokens, float *logits,
		  int *topk_idx, float *topk_w, int lfm2, const EpPush *push, bool *push_taken)
{
	const int H = c->cfg.hidden, E = c->cfg.n_expert, K = c->cfg.top_k;
	EpPush f = {};
	if (push)
		f = *push;
	if (push_taken)
		*push_taken = false;
	const float *sel_bias = lfm2 ? bias : nullptr;
	if (lfm2)
		bias = nullptr;
	if (n_tokens <= 8) {
		size_t smem = ((size_t)H + (size_t)n_tokens * (H + 8)) * sizeof(float);
		if (smem > 200 * 1024)	// the limit router_setup opts this kernel into
			return TIE_CUDA_ENOTSUP;
		router_logits_decode<8><<<E, 64, smem, c->stream>>>(x, w, bias, logits, n_tokens, H, E);
		TIE_CUDA_LAUNCHED(c);
	} else if (E % 64 == 0 && H % 128 == 0 && n_tokens >= 2048) {
		using Cfg = RmtCfg<8, 8, 64, 64>;
		dim3 grid((n_tokens + Cfg::TT - 1) / Cfg::TT, E / 64 + (push ? RMT_PUSH_ROWS : 0));
		f.n_ctas = rmt_push_ctas(c, grid.x * (E / 64), grid.x * RMT_PUSH_ROWS);
		router_logits_mt<8, 8, 64, 64><<<grid, Cfg::THREADS, Cfg::SMEM, c->stream>>>(x, w, bias, logits, n_tokens, H, E, f);
		if (push_taken)
			*push_taken = push != nullptr;
		TIE_CUDA_LAUNCHED(c);
	} else if (E % 32 == 0 && H % 128 == 0) {
		using Cfg = RmtCfg<4, 4, 32, 128>;
		dim3 grid((n_tokens + Cfg::TT - 1) / Cfg::TT, E / 32 + (push ? RMT_PUSH_ROWS : 0));
		f.n_ctas = rmt_push_ctas(c, grid.x * (E / 32), grid.x * RMT_PUSH_ROWS);
		router_logits_mt<4, 4, 32, 128><<<grid, Cfg::THREADS, Cfg::SMEM, c->stream>>>(x, w, bias, logits, n_tokens, H, E, f);
		if (push_taken)
			*push_taken = push != nullptr;
		TIE_CUDA_LAUNCHED(c);
	} else if (n_tokens <= 512) {
		constexpr int TT = 8, EPC = 16;
		dim3 grid((n_tokens + TT - 1) / TT, E / EPC);
		router_logits_tile<TT, EPC, 256><<<grid, EPC * 8, 0, c->stream>>>(x, w, bias, logits, n_tokens, H, E);
		TIE_CUDA_LAUNCHED(c);
	} else {
		constexpr int TT = 32, EPC = 16;
		dim3 grid((n_tokens + TT - 1) / TT, E / EPC);
		router_logits_tile<TT, EPC, 256><<<grid, EPC * 8, 0, c->stream>>>(x, w, bias, logits, n_tokens, H, E);
		TIE_CUDA_LAUNCHED(c);
	}
	const int warps_per_block = 4;
	const int topk_blocks = (n_tokens + warps_per_block - 1) / warps_per_block;
	if (lfm2)
		router_topk_lfm2<<<topk_blocks, warps_per_block * 32, 0, c->stream>>>(logits, sel_bias, n_tokens, E, K, topk_idx, topk_w);
	else
		router_topk<<<topk_blocks, warps_per_block * 32, 0, c->stream>>>(logits, n_tokens, E, K, topk_idx, topk_w);
	TIE_CUDA_LAUNCHED(c);
	return TIE_CUDA_OK;
}

int launch_router_decode_fused(tie_cuda_ctx *c, const float *x, const float *w, const float *bias, int n_tokens, float *logits,
			       int *topk_idx, float *topk_w)
{
	const int H = c->cfg.hidden, E = c->cfg.n_expert;
	size_t smem = ((size_t)H + (size_t)n_tokens * (H + 8)) * sizeof(float);
	router_decode_fused<<<E, 256, smem, c->stream>>>(x, w, bias, logits, n_tokens, H, E, c->cfg.top_k, topk_idx, topk_w, c->s.counter);
	TIE_CUDA_LAUNCHED(c);
	return TIE_CUDA_OK;
}

// Opt-in shared-memory sizes are set once per context (never inside a stream capture).
int router_setup(tie_cuda_ctx *c)
{
	TIE_CUDA_TRY(c, cudaFuncSetAttribute(router_logits_decode<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
	TIE_CUDA_TRY(c, cudaFuncSetAttribute(router_decode_fused, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
	TIE_CUDA_TRY(c, cudaFuncSetAttribute(router_logits_mt<4, 4, 32, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
					     RmtCfg<4, 4, 32, 128>::SMEM));
	TIE_CUDA_TRY(c, cudaFuncSetAttribute(router_logits_mt<8, 8, 64, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
					     RmtCfg<8, 8, 64, 64>::SMEM));
	return TIE_CUDA_OK;
}

// Plain F32 mat-vec over the first n_rows rows of w (the math_dispatch F32 row), one vector.
int launch_router_rows(tie_cuda_ctx *c, const float *x, const float *w, int n_rows, int in_dim, float *out)
{
	size_t smem = ((size_t)in_dim + (size_t)(in_dim + 8)) * sizeof(float);
	if (smem > 200 * 1024)
		return TIE_CUDA_ENOTSUP;
	router_logits_decode<8><<<n_rows, 64, smem, c->stream>>>(x, w, nullptr, out, 1, in_dim, n_rows);
	TIE_CUDA_LAUNCHED(c);
	return TIE_CUDA_OK;
}

}  // namespace tie

// ---------------------------------------------------------------------------------------------
// Routing without any allocation.
//
// Some hosts of this library may not allocate device memory when they call it: a serving loop
// that forbids allocator calls once start-up is over, or an embedding application that gives the
// library a fixed memory budget and no allocator.  For them the logits scratch of the router lives in the
// library image itself: a file-scope __device__ array, present once on every GPU that loads the
// library, for as long as the process lives.
//
// TIE_ROUTE_NOALLOC_MAX_TOKENS x TIE_ROUTE_NOALLOC_MAX_EXPERTS floats = 64 KiB per GPU.
constexpr int TIE_ROUTE_NOALLOC_MAX_TOKENS = 64;
constexpr int TIE_ROUTE_NOALLOC_MAX_EXPERTS = 256;
static __device__ __align__(256) float g_route_scratch[TIE_ROUTE_NOALLOC_MAX_TOKENS * TIE_ROUTE_NOALLOC_MAX_EXPERTS];

namespace {
constexpr int NOALLOC_MAX_DEVICES = 64;
float *g_route_scratch_addr[NOALLOC_MAX_DEVICES] = {nullptr};  // device address of the array, per device
std::mutex g_route_scratch_mutex;			       // first calls of several host threads set up one at a time
}

extern "C" int tie_cuda_route_noalloc(const float *x_dev, const float *router_w_dev, const float *router_bias_dev, int n_tokens,
				      int hidden, int n_expert, int top_k, int *topk_idx_dev, float *topk_w_dev, void *cuda_stream)
{
	using namespace tie;
	if (!x_dev || !router_w_dev || !topk_idx_dev || !topk_w_dev || n_tokens <= 0 || hidden <= 0 || hidden % 8 || n_expert <= 0 ||
	    n_expert % 16 || top_k <= 0 || top_k > MAX_TOP_K || top_k > n_expert)
		return TIE_CUDA_EINVAL;
	// the kernels read x and the router matrix with 128-bit loads: an address that is not a
	// multiple of 16 bytes would be a misaligned-address fault on the device, so it is refused here
	if ((reinterpret_cast<uintptr_t>(x_dev) | reinterpret_cast<uintptr_t>(router_w_dev)) & 15u)
		return TIE_CUDA_EINVAL;
	if ((reinterpret_cast<uintptr_t>(topk_idx_dev) | reinterpret_cast<uintptr_t>(topk_w_dev) |
	     reinterpret_cast<uintptr_t>(router_bias_dev)) & 3u)
		return TIE_CUDA_EINVAL;
	if (n_tokens > TIE_ROUTE_NOALLOC_MAX_TOKENS || n_expert > TIE_ROUTE_NOALLOC_MAX_EXPERTS)
		return TIE_CUDA_ETOOBIG;
	const size_t smem = ((size_t)hidden + (size_t)n_tokens * (hidden + 8)) * sizeof(float);
	if (n_tokens <= 8 && smem > 200 * 1024)
		return TIE_CUDA_ETOOBIG;
	int dev = -1;
	if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES)
		return TIE_CUDA_ENODEV;
	std::unique_lock<std::mutex> setup_lock(g_route_scratch_mutex);
	if (!g_route_scratch_addr[dev]) {
		// First call on this device: resolve the array's DEVICE address.  In host code the name
		// g_route_scratch is only a handle for the runtime, not an address a kernel can use.
		// (Host threads that make their first call at the same time take turns here; the lock
		// orders the set-up only, not the kernels: overlapping calls still race on the array.)
		float *p = nullptr;
		if (cudaGetSymbolAddress(reinterpret_cast<void **>(&p), g_route_scratch) != cudaSuccess || !p) {
			cudaGetLastError();
			return TIE_CUDA_ECUDA;
		}
		if (cudaFuncSetAttribute(router_logits_decode<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) !=
		    cudaSuccess) {
			cudaGetLastError();
			return TIE_CUDA_ECUDA;
		}
		g_route_scratch_addr[dev] = p;
	}
	float *logits = g_route_scratch_addr[dev];
	setup_lock.unlock();
	cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
	if (n_tokens <= 8) {
		router_logits_decode<8><<<n_expert, 64, smem, st>>>(x_dev, router_w_dev, router_bias_dev, logits, n_tokens, hidden, n_expert);
	} else {
		constexpr int TT = 8, EPC = 16;
		if (hidden % 256)
			return TIE_CUDA_EINVAL;
		dim3 grid((n_tokens + TT - 1) / TT, n_expert / EPC);
		router_logits_tile<TT, EPC, 256><<<grid, EPC * 8, 0, st>>>(x_dev, router_w_dev, router_bias_dev, logits, n_tokens, hidden,
									      n_expert);
	}
	if (cudaGetLastError() != cudaSuccess)
		return TIE_CUDA_ECUDA;
	router_topk<<<(n_tokens + 3) / 4, 128, 0, st>>>(logits, n_tokens, n_expert, top_k, topk_idx_dev, topk_w_dev);
	if (cudaGetLastError() != cudaSuccess)
		return TIE_CUDA_ECUDA;
	return TIE_CUDA_OK;
}
