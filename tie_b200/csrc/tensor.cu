// Grouped expert GEMMs for prefill on the 5th-generation tensor cores (tcgen05.mma, accumulators
// and the weight operand in tensor memory), fed from packed Q4_K / Q6_K super-blocks.
//
// Reference: the same arithmetic as process_expert_task (engine.c:916-964) — gate/up products
// (math_avx2.c:535-604, 753-769), table SwiGLU (math_avx2.c:908-950), down product
// (math_avx2.c:411-495, 771-787) — but for all tokens routed to an expert at once instead of one
// token at a time (model_qwen3.c:415).
//
// Formulation: out^T = W . x^T.  The weight rows fill the 128-row M dimension of the MMA (expert
// row counts are multiples of 128), the ragged token count of an expert is the N dimension.
// A CTA owns one (expert, 128-row tile, token tile).  Per 64-wide k stage:
//   * 8 producer warps read packed blocks (128-bit loads, prefetched one 128-k group ahead into
//     registers), expand them in packed fp16 arithmetic to exact-hi + lo operand pairs
//     (tc_dequant.cuh) and write them to TENSOR MEMORY with tcgen05.st — the A operand of the MMA
//     is taken from TMEM, so shared memory carries only the token operand;
//   * one thread issues TMA tile loads of the token operand (already split into hi/lo fp16, in
//     expert-sorted row order, 16-row boxes: only rows the expert really has) into a ring that
//     runs several k stages ahead of the weight stages;
//   * one thread per weight matrix issues tcgen05.mma (kind::f16, fp32 accumulate in TMEM):
//     D += A_hi.B_hi + A_hi.B_lo + A_lo.B_hi.  hi+lo carries ~22 significand bits per operand; a
//     single fp16 or bf16 product per element is NOT accurate enough for the 1e-3 parity bound.
//     When the accumulators fit, B_hi and B_lo are stacked along N so that A_hi needs one MMA of
//     twice the width instead of two (fewer, larger instructions when an expert has few tokens);
//     the two column ranges are added in the epilogue.
// Stages are recycled through mbarriers (producers -> full -> MMA -> tcgen05.commit -> empty).
// Epilogue: tcgen05.ld from TMEM; gate/up: SwiGLU via the table, scaled by 2^-8, split to fp16
// hi/lo for the down GEMM; down: scaled back and scattered to the (token, slot) row.
// Every barrier wait is bounded; on timeout the CTA raises ST_WAIT_TIMEOUT in the status word,
// drains, frees its tensor memory and exits.
#include "common.cuh"
#include "kernels.cuh"
#include "tc_dequant.cuh"
#include "tc_ptx.cuh"

namespace tie {

constexpr int TC_BM = 128;
constexpr int TC_BK = 64;
constexpr int TC_PRODUCERS = 256;
constexpr int TC_PWARPS = TC_PRODUCERS / 32;
constexpr int TC_THREADS = TC_PRODUCERS + 96;  // + two MMA-issuer warps + TMA warp
constexpr long long TC_WAIT_CYCLES = 1ll << 30;	 // about half a second of SM clocks
constexpr float TC_H_SCALE = 1.0f / 256.0f;  // keeps SwiGLU outputs inside fp16 range; exact (power of two)

template <int NMAT, int NT>
struct TcCfg {
	static constexpr int B_TILE = NT * TC_BK * 2;  // bytes of one (hi or lo) token tile
	static constexpr int B_STAGE = 2 * B_TILE;
	static constexpr int A_COLS = 32;  // TMEM columns of one 128 x 64 fp16 weight tile
	// stack B_hi / B_lo along N when the doubled accumulators still leave room for weight stages
	static constexpr bool CONCAT = NMAT * 2 * NT <= 256;
	static constexpr int ACC_PER_MAT = CONCAT ? 2 * NT : NT;
	static constexpr int ACC_COLS = NMAT * ACC_PER_MAT;
	// With one matrix and a 64-token tile the CTA needs only half of an SM's tensor memory and
	// shared memory: two CTAs then share an SM and hide each other's latencies.
	static constexpr bool HALF_SM = ACC_COLS + 2 * NMAT * 2 * A_COLS <= 256;
	static constexpr int TMEM_COLS = HALF_SM ? 256 : 512;
	static constexpr int STAGES_RAW = (TMEM_COLS - ACC_COLS) / (NMAT * 2 * A_COLS);
	static constexpr int STAGES = STAGES_RAW > 4 ? 4 : STAGES_RAW;	// weight stages (tensor memory)
	static constexpr int SB_RAW = ((HALF_SM ? 100 : 200) * 1024) / B_STAGE;
	static constexpr int SB = SB_RAW > 8 ? 8 : SB_RAW;  // token-operand stages (shared memory)
	static constexpr int SMEM = SB * B_STAGE + 1024 /* alignment slack */ + 512 /* barriers */;
	static constexpr int CTAS_PER_SM = HALF_SM ? 2 : 1;
	static_assert(STAGES >= 2 && SB >= 2, "need at least two stages");
	static_assert(ACC_COLS + STAGES * NMAT * 2 * A_COLS <= TMEM_COLS, "tensor memory budget");
};

struct TcShared {
	uint64_t full[4];    // weight stage written by the producers
	uint64_t empty[4];   // weight stage consumed by the MMAs
	uint64_t bfull[8];   // token tiles landed (TMA transaction bytes)
	uint64_t bempty[8];  // token tiles consumed
	uint64_t done;
	uint32_t tmem_base;
	uint32_t abort;
};

// Bounded wait: false (and the abort flag raised) when the barrier does not flip in time or
// another CTA has already reported a timeout.  The cycle counter is read only after many failed
// polls.
__device__ __forceinline__ bool tc_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag, unsigned *status)
{
	long long t0 = 0;
	uint32_t spins = 0;
	while (!ptx::mbar_try_wait(bar, parity)) {
		if ((++spins & 1023u) == 0) {
			if (*abort_flag)
				return false;
			const long long now = clock64();
			if (t0 == 0)
				t0 = now;
			if (now - t0 > TC_WAIT_CYCLES || (*(volatile unsigned *)status & ST_WAIT_TIMEOUT)) {
				atomicOr(status, ST_WAIT_TIMEOUT);
				*abort_flag = 1;
				return false;
			}
		}
	}
	return true;
}

// One 8-wide k chunk (4 half2 words of hi, 4 of lo) of this thread's row -> 4 TMEM columns of the
// thread's lane in the hi and in the lo tile (2 halves per 32-bit column; c = chunk index 0..7).
__device__ __forceinline__ void put_chunk(uint32_t tile_hi, uint32_t tile_lo, uint32_t c, const uint32_t h0[2], const uint32_t h1[2],
					  const uint32_t l0[2], const uint32_t l1[2])
{
	ptx::tmem_st4(tile_hi + 4 * c, h0[0], h0[1], h1[0], h1[1]);
	ptx::tmem_st4(tile_lo + 4 * c, l0[0], l0[1], l1[0], l1[1]);
}

// Packed weights one producer thread needs for two consecutive k stages (128 k, "group" g) of
// its matrix row.  With two matrices (gate/up) a thread owns all 64 k of a stage for one
// (row, matrix); with one matrix (down) it owns the 32-k half-slice hs of a stage.
template <WKind KIND, int NMAT>
struct RawGroup;

template <int NMAT>
struct RawGroup<W_Q4K, NMAT> {
	static constexpr int NQ = (NMAT == 2) ? 2 : 1;
	uint4 hdr;
	uint4 q[2][NQ];
	__device__ __forceinline__ void load(const uint8_t *wexp, int nb, int row, int g, int hs)
	{
		const uint8_t *blk = wexp + ((size_t)row * nb + (g >> 1)) * Q4K_BYTES;
		hdr = __ldg(reinterpret_cast<const uint4 *>(blk));
#pragma unroll
		for (int st = 0; st < 2; st++) {
			const uint4 *base = reinterpret_cast<const uint4 *>(blk + 16 + 32 * ((g & 1) * 2 + st));
			if (NMAT == 2) {
				q[st][0] = __ldg(base);
				q[st][NQ - 1] = __ldg(base + 1);
			} else {
				q[st][0] = __ldg(base + hs);
			}
		}
	}
	// writes this thread's chunks of stage (2g + st) into the hi/lo tiles
	__device__ __forceinline__ void emit(int g, int st, int hs, uint32_t tile_hi, uint32_t tile_lo) const
	{
		const int p = (g & 1) * 2 + st;
		const float d = half_bits_to_float(hdr.x & 0xffffu), dmin = half_bits_to_float(hdr.x >> 16);
		const uint32_t sc[3] = {hdr.y, hdr.z, hdr.w};
		int s_lo, m_lo, s_hi, m_hi;
		q4k_scale_min(sc, 2 * p, s_lo, m_lo);
		q4k_scale_min(sc, 2 * p + 1, s_hi, m_hi);
		const H2x4 cl = q4k_consts(__fmul_rn(d, (float)s_lo), __fmul_rn(dmin, (float)m_lo));
		const H2x4 ch = q4k_consts(__fmul_rn(d, (float)s_hi), __fmul_rn(dmin, (float)m_hi));
		constexpr int NWORD = 4 * NQ;
		uint32_t w[NWORD];
#pragma unroll
		for (int i = 0; i < NQ; i++) {
			w[4 * i] = q[st][i].x;
			w[4 * i + 1] = q[st][i].y;
			w[4 * i + 2] = q[st][i].z;
			w[4 * i + 3] = q[st][i].w;
		}
		const uint32_t c0 = (NMAT == 2) ? 0u : 2u * hs;	 // first chunk of the low-nibble half
#pragma unroll
		for (int cc = 0; cc < NWORD / 2; cc++) {
			uint32_t h0[2], l0[2], h1[2], l1[2];
			q4k_word(w[2 * cc], 0, cl, h0, l0);
			q4k_word(w[2 * cc + 1], 0, cl, h1, l1);
			put_chunk(tile_hi, tile_lo, c0 + cc, h0, h1, l0, l1);
			q4k_word(w[2 * cc], 4, ch, h0, l0);
			q4k_word(w[2 * cc + 1], 4, ch, h1, l1);
			put_chunk(tile_hi, tile_lo, 4u + c0 + cc, h0, h1, l0, l1);
		}
	}
};

template <int NMAT>
struct RawGroup<W_Q6K_R8, NMAT> {
	static constexpr int NL = (NMAT == 2) ? 2 : 1;	// 16-wide l slices this thread owns
	uint4 a[NL], b[NL], h[NL];
	uint32_t scw[NL];
	float d;
	__device__ __forceinline__ void load(const uint8_t *wexp, int nb, int row, int g, int hs)
	{
		const uint8_t *grp = wexp + (size_t)(row >> 3) * q6k_r8_group_bytes(nb);
		const int r8 = row & 7, kb = g >> 1, n = g & 1;
#pragma unroll
		for (int i = 0; i < NL; i++) {
			const int l16 = (NMAT == 2) ? i : hs;
			const int pp = n * 2 + l16;
			const uint4 *ch = reinterpret_cast<const uint4 *>(grp + q6k_r8_chunk_off(nb, r8, kb, pp));
			a[i] = __ldg(ch);
			b[i] = __ldg(ch + 1);
			h[i] = __ldg(ch + 2);
			scw[i] = __ldg(reinterpret_cast<const uint32_t *>(grp + q6k_r8_scale_off(nb, r8, kb, pp)));
		}
		d = half_bits_to_float(__ldg(reinterpret_cast<const unsigned short *>(grp + q6k_r8_d_off(nb, r8, kb))));
	}
	__device__ __forceinline__ void emit(int g, int st, int hs, uint32_t tile_hi, uint32_t tile_lo) const
	{
#pragma unroll
		for (int i = 0; i < NL; i++) {
			const uint32_t l16 = (NMAT == 2) ? (uint32_t)i : (uint32_t)hs;
			const float sA = __fmul_rn(d, (float)(int)(signed char)((scw[i] >> (16 * st)) & 0xff));
			const float sB = __fmul_rn(d, (float)(int)(signed char)((scw[i] >> (16 * st + 8)) & 0xff));
			__half2 sAh, sAr, sBh, sBr;
			q6k_consts(sA, sAh, sAr);
			q6k_consts(sB, sBh, sBr);
			const uint32_t A[4] = {a[i].x, a[i].y, a[i].z, a[i].w}, B[4] = {b[i].x, b[i].y, b[i].z, b[i].w};
			const uint32_t Hh[4] = {h[i].x, h[i].y, h[i].z, h[i].w};
			uint32_t qa[4], qb[4];
#pragma unroll
			for (int k = 0; k < 4; k++) {
				if (st == 0) {
					qa[k] = (A[k] & 0x0F0F0F0Fu) | ((Hh[k] << 4) & 0x30303030u);
					qb[k] = (B[k] & 0x0F0F0F0Fu) | ((Hh[k] << 2) & 0x30303030u);
				} else {
					qa[k] = ((A[k] >> 4) & 0x0F0F0F0Fu) | (Hh[k] & 0x30303030u);
					qb[k] = ((B[k] >> 4) & 0x0F0F0F0Fu) | ((Hh[k] >> 2) & 0x30303030u);
				}
			}
#pragma unroll
			for (int cc = 0; cc < 2; cc++) {
				uint32_t h0[2], l0[2], h1[2], l1[2];
				q6k_word(qa[2 * cc], sAh, sAr, h0, l0);
				q6k_word(qa[2 * cc + 1], sAh, sAr, h1, l1);
				put_chunk(tile_hi, tile_lo, 2u * l16 + cc, h0, h1, l0, l1);
				q6k_word(qb[2 * cc], sBh, sBr, h0, l0);
				q6k_word(qb[2 * cc + 1], sBh, sBr, h1, l1);
				put_chunk(tile_hi, tile_lo, 4u + 2u * l16 + cc, h0, h1, l0, l1);
			}
		}
	}
};

// RAW (one matrix only): the products are stored as fp32 in expert-sorted row order,
// out[row0 + n][matrix * rows + mrow], for a separate SwiGLU pass; blockIdx.x then runs over the
// row tiles of w0 followed by those of w1 (gate, up).
template <WKind KIND, int NMAT, int NT, bool RAW>
__global__ void __launch_bounds__(TC_THREADS, (TcCfg<NMAT, NT>::CTAS_PER_SM))
grouped_gemm_tc(const __grid_constant__ CUtensorMap tm_hi, const __grid_constant__ CUtensorMap tm_lo,
		const uint8_t *__restrict__ w0, const uint8_t *__restrict__ w1, size_t expert_stride, int k_dim,
		const int *__restrict__ offsets, const int *__restrict__ tile_start, int n_local,
		__half *__restrict__ h_hi, __half *__restrict__ h_lo, float *__restrict__ y, const int *__restrict__ perm,
		int out_stride, const float *__restrict__ silu, unsigned *__restrict__ status, int rows_per_matrix)
{
	static_assert(!RAW || NMAT == 1, "raw output is for the one-matrix kernel");
	using Cfg = TcCfg<NMAT, NT>;
	constexpr int S = Cfg::STAGES, SB = Cfg::SB;
	constexpr bool CONCAT = Cfg::CONCAT;
	extern __shared__ uint8_t smem_raw[];

	// ---- which (expert, token tile) is this CTA? ----
	const int slot = blockIdx.y;
	__shared__ int s_skip;
	if (threadIdx.x == 0)
		s_skip = (slot >= tile_start[n_local]) || (*(volatile unsigned *)status & ST_WAIT_TIMEOUT);
	__syncthreads();
	if (s_skip)
		return;
	int lo_e = 0, hi_e = n_local - 1;  // largest le with tile_start[le] <= slot
	while (lo_e < hi_e) {
		int mid = (lo_e + hi_e + 1) >> 1;
		if (tile_start[mid] <= slot)
			lo_e = mid;
		else
			hi_e = mid - 1;
	}
	const int le = lo_e;
	const int row0 = offsets[le] + (slot - tile_start[le]) * NT;
	const int n_valid = min(NT, offsets[le + 1] - row0);
	if (n_valid <= 0) {
		if (threadIdx.x == 0)
			atomicOr(status, ST_BAD_TILE);
		return;
	}
	const int n_mma = (n_valid + 15) & ~15;	 // N of the MMAs: the tile's tokens rounded up to 16
	const int mat_sel = RAW ? (int)(blockIdx.x * TC_BM) / rows_per_matrix : 0;  // RAW: 0 = w0 (gate), 1 = w1 (up)
	const int m0 = blockIdx.x * TC_BM - mat_sel * rows_per_matrix;
	const int nb = k_dim / QK_K;
	const int k_iters = k_dim / TC_BK;

	const uint32_t raw = ptx::smem_u32(smem_raw);
	const uint32_t tiles = (raw + 1023u) & ~1023u;
	TcShared *sh = reinterpret_cast<TcShared *>(smem_raw + (tiles - raw) + (size_t)SB * Cfg::B_STAGE);
	const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

	// token tiles of ring stage sb: hi at the start; lo right behind the rows in use when the two
	// are stacked along N, else in the second half of the stage
	auto b_hi = [&](int sb) -> uint32_t { return tiles + sb * Cfg::B_STAGE; };
	auto b_lo = [&](int sb) -> uint32_t { return tiles + sb * Cfg::B_STAGE + (CONCAT ? n_mma * 128 : Cfg::B_TILE); };
	// TMEM column of weight tile (stage, matrix, hi/lo)
	auto a_col = [&](int s, int m, int hl) -> uint32_t { return Cfg::ACC_COLS + (s * NMAT * 2 + m * 2 + hl) * Cfg::A_COLS; };

	if (threadIdx.x == 0) {
		for (int s = 0; s < S; s++) {
			ptx::mbar_init(ptx::smem_u32(&sh->full[s]), TC_PWARPS);
			ptx::mbar_init(ptx::smem_u32(&sh->empty[s]), NMAT);
		}
		for (int s = 0; s < SB; s++) {
			ptx::mbar_init(ptx::smem_u32(&sh->bfull[s]), 1);
			ptx::mbar_init(ptx::smem_u32(&sh->bempty[s]), NMAT);
		}
		ptx::mbar_init(ptx::smem_u32(&sh->done), NMAT);
		sh->abort = 0;
		ptx::fence_barrier_init();
		ptx::fence_proxy_async_smem();
	}
	if (warp == TC_PWARPS) {  // first MMA warp owns the tensor-memory allocation
		ptx::tmem_alloc(ptx::smem_u32(&sh->tmem_base), Cfg::TMEM_COLS);
		ptx::tmem_relinquish();
	}
	if (warp == TC_PWARPS + 2 && lane == 0) {
		ptx::prefetch_tmap(&tm_hi);
		ptx::prefetch_tmap(&tm_lo);
	}
	ptx::tc_fence_before();
	__syncthreads();
	ptx::tc_fence_after();
	const uint32_t tmem = sh->tmem_base;
	volatile uint32_t *abort_flag = &sh->abort;

	if (warp < TC_PWARPS) {
		// ================= producers: packed blocks -> hi/lo weight tiles in tensor memory =================
		// thread = (row, matrix) for gate/up, (row, half-slice) for down
		const int row = threadIdx.x & 127, sel = threadIdx.x >> 7;
		const int m = (NMAT == 2) ? sel : 0, hs = (NMAT == 2) ? 0 : sel;
		const uint8_t *wexp = (((NMAT == 2 && sel) || (RAW && mat_sel)) ? w1 : w0) + (size_t)le * expert_stride;
		const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
		const int n_groups = k_iters >> 1;
		RawGroup<KIND, NMAT> cur, nxt;
		cur.load(wexp, nb, m0 + row, 0, hs);
		bool alive = true;
		for (int g = 0; g < n_groups && alive; g++) {
			if (g + 1 < n_groups)
				nxt.load(wexp, nb, m0 + row, g + 1, hs);
#pragma unroll
			for (int st = 0; st < 2; st++) {
				const int it = 2 * g + st;
				const int s = it % S;
				if (it >= S) {	// one lane polls the barrier for its warp
					int ok = 1;
					if (lane == 0)
						ok = tc_wait(ptx::smem_u32(&sh->empty[s]), ((it / S) & 1) ^ 1, abort_flag, status) ? 1 : 0;
					ok = __shfl_sync(0xffffffffu, ok, 0);
					if (!ok) {
						alive = false;
						break;
					}
					ptx::tc_fence_after();
				}
				cur.emit(g, st, hs, lane_base + a_col(s, m, 0), lane_base + a_col(s, m, 1));
				ptx::tmem_st_wait();
				ptx::tc_fence_before();
				__syncwarp();
				if (lane == 0)	// one arrival per producer warp
					ptx::mbar_arrive(ptx::smem_u32(&sh->full[s]));
			}
			cur = nxt;
		}
	} else if (warp < TC_PWARPS + NMAT) {
		// ================= MMA issuers: one thread per weight matrix =================
		if (lane == 0) {
			const int m = warp - TC_PWARPS;
			const uint32_t d = tmem + m * Cfg::ACC_PER_MAT;
			const uint32_t idesc_n = ptx::umma_idesc_f16(TC_BM, n_mma);
			const uint32_t idesc_2n = ptx::umma_idesc_f16(TC_BM, 2 * n_mma);
			for (int it = 0; it < k_iters; it++) {
				const int s = it % S, sb = it % SB;
				if (!tc_wait(ptx::smem_u32(&sh->bfull[sb]), (it / SB) & 1, abort_flag, status))
					break;
				if (!tc_wait(ptx::smem_u32(&sh->full[s]), (it / S) & 1, abort_flag, status))
					break;
				ptx::tc_fence_after();
#pragma unroll
				for (int kk = 0; kk < TC_BK / 16; kk++) {
					const uint64_t bh = ptx::umma_desc_sw128(b_hi(sb)) + 2 * kk;
					const uint32_t ah = tmem + a_col(s, m, 0) + 8 * kk, al = tmem + a_col(s, m, 1) + 8 * kk;
					const uint32_t acc = (it > 0 || kk > 0) ? 1u : 0u;
					if (CONCAT) {
						// columns [0, n): A_hi.B_hi + A_lo.B_hi; columns [n, 2n): A_hi.B_lo
						ptx::mma_f16_ts(d, ah, bh, idesc_2n, acc);
						ptx::mma_f16_ts(d, al, bh, idesc_n, 1u);
					} else {
						const uint64_t bl = ptx::umma_desc_sw128(b_lo(sb)) + 2 * kk;
						ptx::mma_f16_ts(d, ah, bh, idesc_n, acc);
						ptx::mma_f16_ts(d, al, bh, idesc_n, 1u);
						ptx::mma_f16_ts(d, ah, bl, idesc_n, 1u);
					}
				}
				ptx::mma_commit(ptx::smem_u32(&sh->empty[s]));
				ptx::mma_commit(ptx::smem_u32(&sh->bempty[sb]));
			}
			ptx::mma_commit(ptx::smem_u32(&sh->done));
		}
	} else if (warp == TC_PWARPS + 2) {
		// ================= TMA loader for the token operand =================
		if (lane == 0) {
			const int n16 = n_mma >> 4;
			for (int it = 0; it < k_iters; it++) {
				const int sb = it % SB;
				if (it >= SB && !tc_wait(ptx::smem_u32(&sh->bempty[sb]), ((it / SB) & 1) ^ 1, abort_flag, status))
					break;
				const uint32_t fb = ptx::smem_u32(&sh->bfull[sb]);
				// only the rows the MMA will read: 16-row boxes (2 KB each, whole swizzle groups)
				ptx::mbar_arrive_expect_tx(fb, (uint32_t)n16 * 2u * 16u * TC_BK * 2u);
				for (int r = 0; r < n16; r++) {
					ptx::tma_load_2d(b_hi(sb) + r * 2048, &tm_hi, fb, it * TC_BK, row0 + 16 * r);
					ptx::tma_load_2d(b_lo(sb) + r * 2048, &tm_lo, fb, it * TC_BK, row0 + 16 * r);
				}
			}
		}
	}

	// ================= epilogue: 8 warps, TMEM lane quadrant = warp % 4, columns split in two =================
	if (warp < TC_PWARPS) {
		const bool ok = tc_wait(ptx::smem_u32(&sh->done), 0, abort_flag, status);
		ptx::tc_fence_after();
		if (ok) {
			const int quad = warp & 3, chalf = warp >> 2;
			const int mrow = m0 + quad * 32 + lane;
			const uint32_t tlane = tmem + ((uint32_t)(quad * 32) << 16);
			for (int c0 = chalf * (NT / 2); c0 < (chalf + 1) * (NT / 2); c0 += 16) {
				if (c0 >= n_valid)
					break;
				uint32_t g[16], u[16];
				ptx::tmem_ld16(tlane + c0, g);
				if (NMAT == 2)
					ptx::tmem_ld16(tlane + Cfg::ACC_PER_MAT + c0, u);
				if (CONCAT) {
					uint32_t g2[16], u2[16];
					ptx::tmem_ld16(tlane + n_mma + c0, g2);
					if (NMAT == 2)
						ptx::tmem_ld16(tlane + Cfg::ACC_PER_MAT + n_mma + c0, u2);
					ptx::tmem_ld_wait();
#pragma unroll
					for (int j = 0; j < 16; j++) {
						g[j] = __float_as_uint(__uint_as_float(g[j]) + __uint_as_float(g2[j]));
						if (NMAT == 2)
							u[j] = __float_as_uint(__uint_as_float(u[j]) + __uint_as_float(u2[j]));
					}
				} else {
					ptx::tmem_ld_wait();
				}
#pragma unroll
				for (int j = 0; j < 16; j++) {
					const int n = c0 + j;
					if (n < n_valid) {
						if (NMAT == 2) {
							float hv = swiglu_lut(silu, __uint_as_float(g[j]), __uint_as_float(u[j])) * TC_H_SCALE;
							__half hh = __float2half_rn(hv);
							__half hl = __float2half_rn(hv - __half2float(hh));
							const size_t o = (size_t)(row0 + n) * out_stride + tc_kperm(mrow);
							h_hi[o] = hh;
							h_lo[o] = hl;
						} else if (RAW) {
							y[(size_t)(row0 + n) * out_stride + (size_t)mat_sel * rows_per_matrix + mrow] = __uint_as_float(g[j]);
						} else {
							const int rid = perm[row0 + n];
							y[(size_t)rid * out_stride + mrow] = __uint_as_float(g[j]) * (1.0f / TC_H_SCALE);
						}
					}
				}
			}
		}
	}
	if (*abort_flag) {
		// give copies that may still be in flight time to land before the CTA's memory is released
		for (int i = 0; i < 200; i++)
			__nanosleep(1000);
	}
	ptx::tc_fence_before();
	__syncthreads();
	if (warp == TC_PWARPS)
		ptx::tmem_dealloc(tmem, Cfg::TMEM_COLS);
}

// ---- host side ----

typedef CUresult (*PFN_encodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
				    const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
				    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static PFN_encodeTiled get_encode_fn()
{
	static PFN_encodeTiled fn = nullptr;
	if (!fn) {
		void *p = nullptr;
		cudaDriverEntryPointQueryResult qres;
		if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
		    qres == cudaDriverEntryPointSuccess)
			fn = reinterpret_cast<PFN_encodeTiled>(p);
	}
	return fn;
}

// fp16 [rows][cols] row-major, box = 64 columns x 16 rows, 128-byte swizzle.
static int make_tmap(tie_cuda_ctx *c, CUtensorMap *tm, void *base, size_t rows, size_t cols)
{
	PFN_encodeTiled enc = get_encode_fn();
	if (!enc) {
		snprintf(c->cuda_err, sizeof(c->cuda_err), "cuTensorMapEncodeTiled entry point not found");
		return TIE_CUDA_ECUDA;
	}
	cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
	cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
	cuuint32_t box[2] = {(cuuint32_t)TC_BK, 16u};
	cuuint32_t estr[2] = {1, 1};
	CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
			 CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
	if (r != CUDA_SUCCESS) {
		snprintf(c->cuda_err, sizeof(c->cuda_err), "cuTensorMapEncodeTiled failed: %d", (int)r);
		return TIE_CUDA_ECUDA;
	}
	return TIE_CUDA_OK;
}

int tc_setup(tie_cuda_ctx *c)
{
	Scratch &s = c->s;
	void *bases[4] = {s.xs_hi, s.xs_lo, s.hs_hi, s.hs_lo};
	size_t cols[4] = {(size_t)c->cfg.hidden, (size_t)c->cfg.hidden, (size_t)c->cfg.ffn_dim, (size_t)c->cfg.ffn_dim};
	for (int a = 0; a < 4; a++) {
		int rc = make_tmap(c, &c->tmap[a], bases[a], s.rows_pad, cols[a]);
		if (rc)
			return rc;
	}
#define TC_ATTR(KIND, NMAT, NT, RAW)                                                                                            \
	TIE_CUDA_TRY(c, cudaFuncSetAttribute(grouped_gemm_tc<KIND, NMAT, NT, RAW>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
					     TcCfg<NMAT, NT>::SMEM))
	TC_ATTR(W_Q4K, 1, 64, false);
	TC_ATTR(W_Q4K, 1, 128, false);
	TC_ATTR(W_Q4K, 1, 64, true);
	TC_ATTR(W_Q4K, 1, 128, true);
	TC_ATTR(W_Q4K, 2, 64, false);
	TC_ATTR(W_Q4K, 2, 128, false);
	TC_ATTR(W_Q6K_R8, 1, 64, false);
	TC_ATTR(W_Q6K_R8, 1, 128, false);
	TC_ATTR(W_Q6K_R8, 1, 64, true);
	TC_ATTR(W_Q6K_R8, 1, 128, true);
	TC_ATTR(W_Q6K_R8, 2, 64, false);
	TC_ATTR(W_Q6K_R8, 2, 128, false);
#undef TC_ATTR
	c->tmaps_ok = true;
	return TIE_CUDA_OK;
}

template <WKind KIND, int NMAT, int NT, bool RAW>
static int launch_tc_t(tie_cuda_ctx *c, const DevTensor &t0, const DevTensor *t1, const CUtensorMap &tmh, const CUtensorMap &tml,
		       int n_rows, float *y)
{
	Scratch &s = c->s;
	const int max_tiles = min(c->n_local, n_rows) + n_rows / NT;
	dim3 grid((RAW ? 2 : 1) * t0.rows / TC_BM, max_tiles);
	grouped_gemm_tc<KIND, NMAT, NT, RAW><<<grid, TC_THREADS, TcCfg<NMAT, NT>::SMEM, c->stream>>>(
		tmh, tml, t0.ptr, t1 ? t1->ptr : nullptr, t0.expert_stride, t0.k, s.offsets, s.tile_start, c->n_local, s.hs_hi, s.hs_lo,
		y, s.perm, RAW ? 2 * t0.rows : t0.rows, c->silu, s.status, t0.rows);
	TIE_CUDA_LAUNCHED(c);
	return TIE_CUDA_OK;
}

template <int NMAT, bool RAW>
static int launch_tc_n(tie_cuda_ctx *c, const DevTensor &t0, const DevTensor *t1, int arr, int n_tile, int n_rows, float *y)
{
	const CUtensorMap &tmh = c->tmap[arr], &tml = c->tmap[arr + 1];
	if (t0.kind == W_Q4K) {
		if (n_tile == 64)
			return launch_tc_t<W_Q4K, NMAT, 64, RAW>(c, t0, t1, tmh, tml, n_rows, y);
		return launch_tc_t<W_Q4K, NMAT, 128, RAW>(c, t0, t1, tmh, tml, n_rows, y);
	}
	if (n_tile == 64)
		return launch_tc_t<W_Q6K_R8, NMAT, 64, RAW>(c, t0, t1, tmh, tml, n_rows, y);
	return launch_tc_t<W_Q6K_R8, NMAT, 128, RAW>(c, t0, t1, tmh, tml, n_rows, y);
}

bool tc_supported(const tie_cuda_ctx *c, const Layer &L)
{
	return c->tmaps_ok && L.gate.kind == L.up.kind && L.gate.rows % TC_BM == 0 && L.down.rows % TC_BM == 0 &&
	       L.gate.k % QK_K == 0 && L.down.k % QK_K == 0;
}

// xs_hi/xs_lo must hold the split inputs in sorted order; writes hs_hi/hs_lo.
int launch_tc_gate_up(tie_cuda_ctx *c, const Layer &L, int n_rows, int n_tile)
{
	if (n_tile == 64) {
		// few tokens per expert: gate and up as independent one-matrix tiles (two CTAs per SM),
		// raw fp32 products to a scratch [row][gate | up], then one element-wise SwiGLU + split pass
		int rc = launch_tc_n<1, true>(c, L.gate, &L.up, 0, n_tile, n_rows, c->s.y);
		if (rc)
			return rc;
		return launch_swiglu_split(c, c->s.y, n_rows, L.gate.rows, TC_H_SCALE, c->s.hs_hi, c->s.hs_lo);
	}
	return launch_tc_n<2, false>(c, L.gate, &L.up, 0, n_tile, n_rows, nullptr);
}

// reads hs_hi/hs_lo; writes y[perm[p]].
int launch_tc_down(tie_cuda_ctx *c, const Layer &L, int n_rows, int n_tile, float *y)
{
	return launch_tc_n<1, false>(c, L.down, nullptr, 2, n_tile, n_rows, y);
}

}  // namespace tie
