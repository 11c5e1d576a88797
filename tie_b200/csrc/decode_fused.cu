// Decode of ONE token as ONE kernel: router, selection, gate/up + SwiGLU, down + combine.
//
// Reference: the is_moe branch of transformer_layer_qwen3 for batch_len == 1
// (model_qwen3.c:403-471).  The three-kernel decode path (decode.cu) pays three launches and
// cannot keep the down tiles in flight under the gate/up kernel (the two kernels do not fit one
// SM together).  Here one cooperative grid (one CTA per SM, all co-resident) walks the phases
// with two grid-wide barriers:
//
//   R  CTA e < n_expert: logit e, the AVX2 lane order replayed (8 chains of sequential fused
//      multiply-adds, hsum tree: bit-exact, as router_decode_fused); every CTA meanwhile stages
//      x for its gate/up tile
//   -- barrier --
//      every CTA selects the experts itself from the 128 logits (one thread per expert counts
//      the experts ahead of it: cheaper than a broadcast), then requests, all at once, its gate
//      and up tiles AND the down tiles of all selected experts for its 16 output rows (bulk
//      copies, ~190 KB in flight per SM, one issuing thread per copy group)
//   G  CTA (slot, row tile): gate . x, up . x, table SwiGLU -> h (global, 24 KB)
//   -- barrier --
//   D  CTA (row tile): the down tiles are long there; slots are spread over the warp groups, the
//      per-slot dot products meet in shared memory and are combined in slot order from zero,
//      acc = fma(w_j, v_j, acc) (model_qwen3.c:458-467), + residual
//
// The barriers count arrivals in a device word that only grows (targets are relative to an epoch
// the last CTA of every launch advances), so the launch arguments never change and the kernel
// replays from a CUDA graph.  Every spin is bounded; a CTA that gives up flags the status word,
// waits (bounded) for its own copies in flight and returns.
#include "common.cuh"
#include "kernels.cuh"
#include "partdot.cuh"
#include "tc_ptx.cuh"
#include "decode_common.cuh"
#include "router_topk.cuh"
#define TIE_TIMING_DF_OWNER
#include "timing.cuh"

namespace tie {

constexpr int DF_THREADS = 512;
constexpr int DF_MAX_CHUNKS = 8;
constexpr int DF_MAX_PASSES = 4;
constexpr long long DF_WAIT_CYCLES = 1ll << 30;

struct DfShared {
	uint64_t bar_gu[DF_MAX_CHUNKS];
	uint64_t bar_dn[MAX_TOP_K];
	int idx[MAX_TOP_K];
	float w[MAX_TOP_K], score[MAX_TOP_K];
	float lg[256];	// the logits (n_expert <= 256)
	unsigned base;
	int ok;
	int dn_req[MAX_TOP_K];	// the down tile of slot j has been requested
	float inv;  // 1 / rms of the row (RMSNorm in the kernel)
};

struct DfArgs {
	const uint8_t *wg, *wu, *wd;
	size_t stride_gu, stride_dn;  // bytes per expert
	const float *x, *router_w, *bias, *residual, *silu;
	const float *norm_w;  // norm_eps >= 0: x is the un-normed hidden row, RMSNorm (weights norm_w or 1) happens in the kernel
	float norm_eps;
	float *logits, *h, *out, *topk_w;
	int *topk_idx;
	// bytes the NEXT launch reads first (the following block's router matrix), or nullptr: requested into
	// L2 while this block's down products run; whole 16-byte units
	const uint8_t *next;
	uint32_t next_bytes;
	unsigned *status, *sync;  // sync[0]: arrivals, sync[1]: epoch
	int n_expert, top_k, first_expert, n_local;
	int rpt_gu, tiles_gu, rpt_dn, tiles_dn;
	uint32_t off_b, off_c, off_v, off_n;  // shared-memory offsets: down tiles, staged x, slot products, normed x
};

__device__ __forceinline__ unsigned df_ld_acquire(const unsigned *p)
{
	unsigned v;
	asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
	return v;
}

// All CTAs of the (cooperative, co-resident) grid arrive; returns false after DF_WAIT_CYCLES.
__device__ __forceinline__ bool df_grid_barrier(unsigned *counter, unsigned target, DfShared *sh, unsigned *status)
{
	__syncthreads();
	if (threadIdx.x == 0) {
		__threadfence();
		atomicAdd(counter, 1u);
		const long long t0 = clock64();
		int ok = 1;
		while ((int)(df_ld_acquire(counter) - target) < 0) {
			if (clock64() - t0 > DF_WAIT_CYCLES) {
				atomicOr(status, ST_WAIT_TIMEOUT);
				ok = 0;
				break;
			}
		}
		sh->ok = ok;
	}
	__syncthreads();
	return sh->ok != 0;
}

template <WKind KIND, int LPR>
__device__ __forceinline__ void df_stage_lane_major_cg(const float *xrow, float *xs_t, int parts, int tid)
{
	// as stage_x_lane_major, with loads that bypass L1: the row was written by other CTAs of this grid
	for (int d = tid; d < 16 * parts; d += DF_THREADS) {
		const int r4 = d / parts, p = d % parts;
		const int k = PartDot<KIND>::src_index(p, 4 * r4);
		*reinterpret_cast<float4 *>(xs_t + (size_t)(r4 * LPR + p) * 4) = __ldcg(reinterpret_cast<const float4 *>(xrow + k));
	}
}

template <int KDIM>
struct DfDims {
	static constexpr int PARTS = KDIM / 64;
	static constexpr int LPR = PARTS > 16 ? 32 : (PARTS > 8 ? 16 : (PARTS > 4 ? 8 : 4));
	static constexpr int RPW = 32 / LPR;
	static constexpr int NB = KDIM / QK_K;
	static constexpr int RPP = (DF_THREADS / 32) * RPW;  // rows per pass of the whole CTA
};

template <WKind KG, int K, WKind KD, int F>
__global__ void __launch_bounds__(DF_THREADS, 1) decode1_fused(const DfArgs a)
{
	using DK = DfDims<K>;
	using DF = DfDims<F>;
	constexpr int CH = DK::RPP > 16 ? DK::RPP : 16;	 // rows per gate/up copy chunk (own barrier)
	extern __shared__ __align__(128) uint8_t dsm[];
	__shared__ DfShared sh;
	const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
	const int cta = blockIdx.x, G = gridDim.x;
	const int top_k = a.top_k;
	float *xs = reinterpret_cast<float *>(dsm + a.off_c);  // x, lane-major, for the gate/up reduction

	const bool gu_role = cta < top_k * a.tiles_gu, dn_role = cta < a.tiles_dn;
	const int slot = cta / a.tiles_gu;
	const int g0 = (cta % a.tiles_gu) * a.rpt_gu, g1 = min(g0 + a.rpt_gu, F);
	const int d0 = cta * a.rpt_dn, d1 = min(d0 + a.rpt_dn, K);
	const int n_chunks = gu_role ? (g1 - g0 + CH - 1) / CH : 0;
	const uint32_t tile_gu = (uint32_t)(tile_offset<KG>(DK::NB, g1) - tile_offset<KG>(DK::NB, g0));
	const uint32_t tile_dn = dn_role ? (uint32_t)(tile_offset<KD>(DF::NB, d1) - tile_offset<KD>(DF::NB, d0)) : 0;

	DF_STAMP(0);
	if (tid == 0) {
		for (int c = 0; c < DF_MAX_CHUNKS; c++)
			ptx::mbar_init(ptx::smem_u32(&sh.bar_gu[c]), 1);
		for (int j = 0; j < MAX_TOP_K; j++) {
			ptx::mbar_init(ptx::smem_u32(&sh.bar_dn[j]), 1);
			sh.dn_req[j] = 0;
		}
		ptx::fence_barrier_init();
		sh.base = df_ld_acquire(a.sync + 1);
	}

	// ---------------- (RMSNorm of the row, every CTA for itself: rms_norm_f32_f32_f32_avx2, math_avx2.c:56-97) ----------------
	const float *xin = a.x;
	if (a.norm_eps >= 0.0f) {
		float *xn = reinterpret_cast<float *>(dsm + a.off_n);
		for (int i = tid; i < K / 4; i += DF_THREADS)
			reinterpret_cast<float4 *>(xn)[i] = __ldcg(reinterpret_cast<const float4 *>(a.x) + i);  // (the row is overwritten in place at the end)
		__syncthreads();
		if (warp == 0) {
			float acc = 0.0f;
			if (lane < 8) {
#pragma unroll 16
				for (int i = 0; i < K / 8; i++) {
					const float v = xn[8 * i + lane];
					acc = __fmaf_rn(v, v, acc);
				}
			}
			const float ss = hsum8_lanes(acc);  // (l + l4), then + 1, then + 2: the reference's tree
			if (lane == 0)
				sh.inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)K), a.norm_eps)));
		}
		__syncthreads();
		const float inv = sh.inv;
		for (int i = tid; i < K; i += DF_THREADS)
			xn[i] = __fmul_rn(__fmul_rn(xn[i], a.norm_w ? a.norm_w[i] : 1.0f), inv);
		__syncthreads();
		xin = xn;
	}

	// ---------------- R: one router logit per CTA ----------------
	if (cta < a.n_expert) {
		float *ws = reinterpret_cast<float *>(dsm), *xr = ws + K;
		const float4 *w4 = reinterpret_cast<const float4 *>(a.router_w + (size_t)cta * K);
		const float4 *x4 = reinterpret_cast<const float4 *>(xin);
		for (int i = tid; i < K / 4; i += DF_THREADS) {
			const float4 wv = __ldg(w4 + i), xv = x4[i];
			reinterpret_cast<float4 *>(ws)[i] = wv;
			reinterpret_cast<float4 *>(xr)[i] = xv;
		}
		__syncthreads();
		if (warp == 0) {
			float acc = 0.0f;
			if (lane < 8) {
#pragma unroll 16
				for (int i = 0; i < K / 8; i++)
					acc = __fmaf_rn(xr[8 * i + lane], ws[8 * i + lane], acc);
			}
			float r = hsum8_lanes(acc);
			if (lane == 0) {
				if (a.bias)
					r = __fadd_rn(r, a.bias[cta]);
				__stcg(a.logits + cta, r);
			}
		}
	}
	if (gu_role)
		stage_x_lane_major<KG, DK::LPR>(xin, xs, DK::PARTS, tid, DF_THREADS);
	const unsigned base = (__syncthreads(), sh.base);
	DF_STAMP(1);
	if (!df_grid_barrier(a.sync, base + (unsigned)G, &sh, a.status))
		return;	 // nothing of this CTA is in flight yet
	DF_STAMP(2);

	// ---------------- selection (every CTA for itself) and all weight requests ----------------
	// find_top_k (engine.c:891-914) orders by (score descending, index ascending) — a total order, so
	// the slot of an expert is the number of experts ahead of it: one thread per expert counts them.
	if (tid < a.n_expert)
		sh.lg[tid] = __ldcg(a.logits + tid);
	__syncthreads();
	if (tid < a.n_expert) {
		const float v = sh.lg[tid];
		int rank = 0;
		for (int e = 0; e < a.n_expert; e++) {
			const float o = sh.lg[e];
			rank += (o > v || (o == v && e < tid)) ? 1 : 0;
		}
		if (rank < top_k) {
			sh.idx[rank] = tid;
			sh.score[rank] = v;
		}
	}
	__syncthreads();
	if (warp == 0) {  // softmax (engine.c:864-888) with the arithmetic of topk_softmax_warp
		const float my_score = lane < top_k ? sh.score[lane] : 0.0f;
		const float mx = __shfl_sync(0xffffffffu, my_score, 0);
		const float ex = (lane < top_k) ? expf(__fsub_rn(my_score, mx)) : 0.0f;
		float sum = 0.0f;
		for (int j = 0; j < top_k; j++)
			sum = __fadd_rn(sum, __shfl_sync(0xffffffffu, ex, j));
		const float inv = __fdiv_rn(1.0f, sum);
		if (lane < top_k)
			sh.w[lane] = __fmul_rn(ex, inv);
	}
	__syncthreads();
	bool bad = false;
	for (int j = 0; j < top_k; j++) {
		const int le = sh.idx[j] - a.first_expert;
		bad |= (le < 0 || le >= a.n_local);
	}
	if (cta == 0 && tid < top_k) {
		a.topk_idx[tid] = sh.idx[tid];
		a.topk_w[tid] = sh.w[tid];
	}
	if (bad && cta == 0 && tid == 0)
		atomicOr(a.status, ST_BAD_EXPERT);
	uint8_t *sg = dsm, *su = dsm + tile_gu, *sd = dsm + a.off_b;
	// one issuing thread per copy group (issuing a bulk copy costs ~100 cycles): warp c < 8 the
	// gate/up chunk c, warp 8 + j the down tile of slot j.  The down tiles are requested once the
	// first gate/up chunk has landed: asked for together with the gate/up tiles they shared the HBM
	// bandwidth with them and the first chunk arrived a microsecond later; they still have the whole
	// gate/up phase to arrive in.
	auto request_down = [&]() {  // lane 0 of warp 8 + j
		const int j = warp - DF_MAX_CHUNKS;
		if (dn_role && j >= 0 && j < top_k) {
			const uint32_t ba = ptx::smem_u32(&sh.bar_dn[j]);
			sh.dn_req[j] = 1;
			ptx::fence_proxy_async_smem();
			ptx::mbar_arrive_expect_tx(ba, tile_dn);
			bulk_g2s(ptx::smem_u32(sd + (size_t)j * tile_dn),
				 a.wd + (size_t)(sh.idx[j] - a.first_expert) * a.stride_dn + tile_offset<KD>(DF::NB, d0), tile_dn, ba);
		}
	};
	if (lane == 0 && !bad) {
		ptx::fence_proxy_async_smem();	// the tile area held the router's staging
		if (warp < DF_MAX_CHUNKS) {
			const int c = warp;
			if (gu_role && c < n_chunks) {
				const size_t eb = (size_t)(sh.idx[slot] - a.first_expert) * a.stride_gu;
				const int c0 = g0 + c * CH, c1 = min(c0 + CH, g1);
				const size_t o0 = tile_offset<KG>(DK::NB, c0), o1 = tile_offset<KG>(DK::NB, c1);
				const uint32_t bytes = (uint32_t)(o1 - o0), rel = (uint32_t)(o0 - tile_offset<KG>(DK::NB, g0));
				const uint32_t ba = ptx::smem_u32(&sh.bar_gu[c]);
				ptx::mbar_arrive_expect_tx(ba, 2 * bytes);
				bulk_g2s(ptx::smem_u32(sg + rel), a.wg + eb + o0, bytes, ba);
				bulk_g2s(ptx::smem_u32(su + rel), a.wu + eb + o0, bytes, ba);
			}
		} else if (!gu_role) {
			request_down();	 // (a CTA without gate/up rows: nothing to wait for)
		}
	}
	// waits (bounded) for every copy this CTA requested: before it gives up, and harmless otherwise
	auto drain = [&]() {
		if (bad)
			return;
		for (int c = 0; c < n_chunks; c++)
			dec_wait(ptx::smem_u32(&sh.bar_gu[c]), a.status);
		if (dn_role)
			for (int j = 0; j < top_k; j++)
				if (sh.dn_req[j])
					dec_wait(ptx::smem_u32(&sh.bar_dn[j]), a.status);
	};

	// ---------------- G: gate, up, SwiGLU ----------------
	DF_STAMP(3);
	bool alive = true;
	if (gu_role && !bad) {
		const int sub = lane / DK::LPR, part = lane % DK::LPR;
		const bool lane_on = part < DK::PARTS;
		float xr[64], sx[4];
		if (lane_on)
			load_x_lane_major<KG, DK::LPR>(xs, part, xr, sx);
		const uint8_t *vg = sg - tile_offset<KG>(DK::NB, g0), *vu = su - tile_offset<KG>(DK::NB, g0);
		float *hrow = a.h + (size_t)slot * F;
		int waited = -1;
		// The table look-ups of a row's SwiGLU are two dependent loads: done at the end of every pass they
		// stall the warp before its next pass.  After the reduction every lane of a row holds the sums, so
		// lane p of the row keeps those of pass p and all passes' look-ups are issued together at the end
		// (as long as a row has at least as many lanes as the tile has passes).
		const bool defer = (g1 - g0 + DK::RPP - 1) / DK::RPP <= DK::LPR;
		float keep_g = 0.f, keep_u = 0.f;
		int keep_row = -1, pass = 0;
		for (int rp = g0; rp < g1 && alive; rp += DK::RPP, pass++) {
			const int chunk = (rp - g0) / CH;
			if (chunk != waited) {
				alive = dec_wait(ptx::smem_u32(&sh.bar_gu[chunk]), a.status);
				waited = chunk;
				if (!alive)
					break;
				if (chunk == 0) {
					DF_STAMP(7);
					if (lane == 0 && warp >= DF_MAX_CHUNKS)
						request_down();
				}
			}
			const int row = rp + warp * DK::RPW + sub;
			float vgv = 0.f, vuv = 0.f;
			if (lane_on && row < g1) {
				vgv = PartDot<KG>::dot(PartDot<KG>::template load<true>(vg, DK::NB, row, part), part, xr, sx);
				vuv = PartDot<KG>::dot(PartDot<KG>::template load<true>(vu, DK::NB, row, part), part, xr, sx);
			}
#pragma unroll
			for (int o = DK::LPR / 2; o > 0; o >>= 1) {
				vgv += __shfl_xor_sync(0xffffffffu, vgv, o);
				vuv += __shfl_xor_sync(0xffffffffu, vuv, o);
			}
			if (defer) {
				if (part == pass && row < g1) {
					keep_g = vgv;
					keep_u = vuv;
					keep_row = row;
				}
			} else if (part == 0 && row < g1) {
				__stcg(hrow + row, swiglu_lut(a.silu, vgv, vuv));
			}
		}
		if (keep_row >= 0 && alive)
			__stcg(hrow + keep_row, swiglu_lut(a.silu, keep_g, keep_u));
		DF_STAMP(8);
	}
	alive = __syncthreads_and(alive);
	DF_STAMP(4);
	if (!alive) {  // a copy never landed: leave, but not with copies in flight
		if (tid == 0)
			drain();
		return;
	}
	if (!df_grid_barrier(a.sync, base + 2u * (unsigned)G, &sh, a.status)) {
		if (tid == 0)
			drain();
		return;
	}

	// ---------------- D: down + combine ----------------
	DF_STAMP(5);
	if (a.next && tid == 0) {  // this CTA's share of the next block's first bytes -> L2
		const uint32_t per = ((a.next_bytes + G - 1) / G + 15u) & ~15u, o = per * (uint32_t)cta;
		if (o < a.next_bytes) {
			const uint32_t n = min(per, a.next_bytes - o);
			asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(a.next + o), "r"(n) : "memory");
		}
	}
	if (dn_role && !bad) {
		float *hs = reinterpret_cast<float *>(dsm);  // top_k lane-major rows of h (the gate/up tiles are done with)
		float *vbuf = reinterpret_cast<float *>(dsm + a.off_v);
		constexpr int XS_T = DF::LPR * 64;
		for (int j = 0; j < top_k; j++)
			df_stage_lane_major_cg<KD, DF::LPR>(a.h + (size_t)j * F, hs + (size_t)j * XS_T, DF::PARTS, tid);
		__syncthreads();
		DF_STAMP(9);
		const int sub = lane / DF::LPR, part = lane % DF::LPR;
		const bool lane_on = part < DF::PARTS;
		const int rows = d1 - d0;
		// A (warp, sub-row) unit keeps ONE slot for the whole phase — its slice of that slot's h stays in
		// registers — and walks the rows of the tile: the units of slot j are j, j + top_k, ..., the
		// k-th of them takes rows k, k + n_j, ... (loading the activations once per unit instead of once
		// per slot and unit leaves only the packed rows to fetch inside the loop).
		const int unit = warp * DF::RPW + sub;	// (a pass has at least 16 units, a token at most 8 slots)
		{
			const int j = unit % top_k, r0 = unit / top_k;
			const int n_j = (DF::RPP - 1 - j) / top_k + 1;		    // units that share slot j
			const int trips = (rows + DF::RPP / top_k - 1) / (DF::RPP / top_k);  // the same for every lane of a warp
			float xr[64], sx[4];
			if (lane_on)
				load_x_lane_major<KD, DF::LPR>(hs + (size_t)j * XS_T, part, xr, sx);
			alive = __all_sync(0xffffffffu, dec_wait(ptx::smem_u32(&sh.bar_dn[j]), a.status));
			const uint8_t *vd = sd + (size_t)j * tile_dn - tile_offset<KD>(DF::NB, d0);
			for (int i = 0; i < trips && alive; i++) {
				const int lr = r0 + i * n_j;
				float v = 0.f;
				if (lane_on && lr < rows)
					v = PartDot<KD>::dot(PartDot<KD>::template load<true>(vd, DF::NB, d0 + lr, part), part, xr, sx);
#pragma unroll
				for (int o = DF::LPR / 2; o > 0; o >>= 1)
					v += __shfl_xor_sync(0xffffffffu, v, o);
				if (part == 0 && lr < rows)
					vbuf[j * a.rpt_dn + lr] = v;
			}
		}
		DF_STAMP(10);
		alive = __syncthreads_and(alive);
		if (alive) {
			for (int lr = tid; lr < rows; lr += DF_THREADS) {
				float acc = 0.f;
				for (int j = 0; j < top_k; j++)
					acc = __fmaf_rn(sh.w[j], vbuf[j * a.rpt_dn + lr], acc);	 // slot order, from zero
				if (a.residual)
					acc = __fadd_rn(a.residual[d0 + lr], acc);
				a.out[d0 + lr] = acc;
			}
		}
	}
	__syncthreads();
	DF_STAMP(6);
	if (tid == 0) {
		drain();
		// the last CTA out advances the epoch for the next launch
		if (alive && atomicAdd(a.sync, 1u) == base + 3u * (unsigned)G - 1u)
			atomicExch(a.sync + 1, base + 3u * (unsigned)G);
	}
}

// ---- host side ----

template <WKind KIND>
static size_t df_row_bytes(int k)
{
	return (size_t)(k / QK_K) * (KIND == W_Q4K ? Q4K_BYTES : Q6K_BYTES);
}

struct DfPlan {
	int rpt_gu, tiles_gu, rpt_dn, tiles_dn, grid;
	size_t smem, off_b, off_c, off_v, off_n;
	bool ok;
};

template <WKind KG, int K, WKind KD, int F>
static DfPlan df_plan(const tie_cuda_ctx *c)
{
	DfPlan p = {};
	const int top_k = c->cfg.top_k, sms = c->sm_count;
	const int want_gu = sms / top_k;
	if (want_gu < 1)
		return p;
	p.rpt_gu = ((F + want_gu - 1) / want_gu + 7) / 8 * 8;
	p.tiles_gu = (F + p.rpt_gu - 1) / p.rpt_gu;
	p.rpt_dn = ((K + sms - 1) / sms + 7) / 8 * 8;
	p.tiles_dn = (K + p.rpt_dn - 1) / p.rpt_dn;
	constexpr int RPP_K = DfDims<K>::RPP, RPP_F = DfDims<F>::RPP;
	constexpr int CH = RPP_K > 16 ? RPP_K : 16;
	if ((p.rpt_gu + CH - 1) / CH > DF_MAX_CHUNKS)
		return p;
	if (p.rpt_dn >= RPP_F ? (p.rpt_dn + RPP_F - 1) / RPP_F > DF_MAX_PASSES : RPP_F % p.rpt_dn != 0)
		return p;
	p.grid = max(c->cfg.n_expert, max(top_k * p.tiles_gu, p.tiles_dn));
	if (p.grid > sms)
		return p;
	const size_t tile_gu = (size_t)p.rpt_gu * df_row_bytes<KG>(K), tile_dn = (size_t)p.rpt_dn * df_row_bytes<KD>(F);
	size_t area_a = 2 * tile_gu;
	area_a = max(area_a, (size_t)2 * K * sizeof(float));				 // router staging
	area_a = max(area_a, (size_t)top_k * DfDims<F>::LPR * 64 * sizeof(float));	 // staged h rows
	p.off_b = (area_a + 127) / 128 * 128;
	p.off_c = (p.off_b + (size_t)top_k * tile_dn + 127) / 128 * 128;
	p.off_v = p.off_c + (size_t)DfDims<K>::LPR * 64 * sizeof(float);
	p.off_n = (p.off_v + (size_t)top_k * p.rpt_dn * sizeof(float) + 15) / 16 * 16;
	p.smem = p.off_n + (size_t)K * sizeof(float);
	p.ok = p.smem <= 220 * 1024;
	return p;
}

template <WKind KG, int K, WKind KD, int F>
static int df_launch(tie_cuda_ctx *c, const Layer &L, const float *x, const float *bias, const float *residual, float *out,
		     bool query_only, const float *norm_w, float norm_eps, const Layer *next)
{
	const DfPlan p = df_plan<KG, K, KD, F>(c);
	if (!p.ok)
		return TIE_CUDA_ENOTSUP;
	if (query_only)
		return TIE_CUDA_OK;
	Scratch &s = c->s;
	DfArgs a = {};
	a.wg = L.gate.ptr;
	a.wu = L.up.ptr;
	a.wd = L.down.ptr;
	a.stride_gu = L.gate.expert_stride;
	a.stride_dn = L.down.expert_stride;
	a.x = x;
	a.router_w = L.router_w;
	a.bias = bias;
	a.residual = residual;
	a.silu = c->silu;
	a.logits = s.logits;
	a.h = s.h;
	a.out = out;
	a.topk_w = s.topk_w;
	a.topk_idx = s.topk_idx;
	a.status = s.status;
	a.sync = s.dec_sync;
	a.n_expert = c->cfg.n_expert;
	a.top_k = c->cfg.top_k;
	a.first_expert = c->first_expert;
	a.n_local = c->n_local;
	a.rpt_gu = p.rpt_gu;
	a.tiles_gu = p.tiles_gu;
	a.rpt_dn = p.rpt_dn;
	a.tiles_dn = p.tiles_dn;
	a.off_b = (uint32_t)p.off_b;
	a.off_c = (uint32_t)p.off_c;
	a.off_v = (uint32_t)p.off_v;
	a.off_n = (uint32_t)p.off_n;
	a.norm_w = norm_w;
	a.norm_eps = norm_eps;
	if (next && next->router_w) {
		a.next = reinterpret_cast<const uint8_t *>(next->router_w);
		a.next_bytes = (uint32_t)((size_t)c->cfg.n_expert * K * sizeof(float));
	}
	auto kern = decode1_fused<KG, K, KD, F>;
	TIE_CUDA_TRY(c, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
	cudaLaunchConfig_t cfg = {};
	cfg.gridDim = dim3(p.grid);
	cfg.blockDim = dim3(DF_THREADS);
	cfg.dynamicSmemBytes = p.smem;
	cfg.stream = c->stream;
	cudaLaunchAttribute attr[1];
	attr[0].id = cudaLaunchAttributeCooperative;  // all CTAs co-resident: they wait on one another
	attr[0].val.cooperative = 1;
	cfg.attrs = attr;
	cfg.numAttrs = 1;
	const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, a);
	if (e == cudaErrorCooperativeLaunchTooLarge || e == cudaErrorNotSupported) {
		// the grid cannot be co-resident here (a shared or partitioned GPU): the caller takes the chain
		cudaGetLastError();
		c->coop_ok = false;
		return TIE_CUDA_ENOTSUP;
	}
	TIE_CUDA_TRY(c, e);
	c->launches++;
	return TIE_CUDA_OK;
}

// The (hidden, ffn_dim) pairs the one-kernel step is built for.
#define TIE_DF_SHAPES(X) X(2048, 768) X(512, 256)

static int df_dispatch(tie_cuda_ctx *c, const Layer &L, const float *x, const float *bias, const float *residual, float *out,
		       bool query_only, const float *norm_w = nullptr, float norm_eps = -1.0f, const Layer *next = nullptr)
{
	if (L.gate.kind != L.up.kind)
		return TIE_CUDA_ENOTSUP;
	const int K = c->cfg.hidden, F = c->cfg.ffn_dim;
#define X(KK, FF)                                                                                                              \
	if (K == KK && F == FF) {                                                                                              \
		if (L.gate.kind == W_Q4K && L.down.kind == W_Q6K_R8)                                                           \
			return df_launch<W_Q4K, KK, W_Q6K_R8, FF>(c, L, x, bias, residual, out, query_only, norm_w, norm_eps, next);                    \
		if (L.gate.kind == W_Q4K && L.down.kind == W_Q4K)                                                              \
			return df_launch<W_Q4K, KK, W_Q4K, FF>(c, L, x, bias, residual, out, query_only, norm_w, norm_eps, next);                      \
		if (L.gate.kind == W_Q6K_R8 && L.down.kind == W_Q6K_R8)                                                        \
			return df_launch<W_Q6K_R8, KK, W_Q6K_R8, FF>(c, L, x, bias, residual, out, query_only, norm_w, norm_eps, next);                \
		return df_launch<W_Q6K_R8, KK, W_Q4K, FF>(c, L, x, bias, residual, out, query_only, norm_w, norm_eps, next);                           \
	}
	TIE_DF_SHAPES(X)
#undef X
	return TIE_CUDA_ENOTSUP;
}

bool decode_fused_supported(tie_cuda_ctx *c, const Layer &L, int n_tokens)
{
	if (n_tokens != 1 || !c->coop_ok || c->cfg.top_k > MAX_TOP_K || c->cfg.n_expert > 256)
		return false;
	return df_dispatch(c, L, nullptr, nullptr, nullptr, nullptr, true) == TIE_CUDA_OK;
}

// norm_eps >= 0: x is the un-normed hidden row; the kernel applies RMSNorm (norm_w, or weight 1) first.
// next: the block that runs after this one (its router matrix is requested into L2 meanwhile), or nullptr.
int launch_decode_fused(tie_cuda_ctx *c, const Layer &L, const float *x, const float *bias, const float *residual, float *out,
			const float *norm_w, float norm_eps, const Layer *next)
{
	return df_dispatch(c, L, x, bias, residual, out, false, norm_w, norm_eps, next);
}

// One token through consecutive layers as ONE launch: not built (the layer loop inside the kernel
// pushed the reductions' activation registers into local memory and doubled the step's time); the
// caller runs the per-layer kernels from one CUDA graph instead.
int launch_decode_fused_stack(tie_cuda_ctx *, int, int, float *)
{
	return TIE_CUDA_ENOTSUP;
}

}  // namespace tie
