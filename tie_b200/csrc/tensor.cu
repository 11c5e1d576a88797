// Grouped expert GEMMs for prefill on the 5th-generation tensor cores (tcgen05.mma with the
// weight operand and the accumulators in tensor memory), fed from packed Q4_K / Q6_K super-blocks.
//
// Reference: the same arithmetic as process_expert_task (engine.c:916-964) — gate/up products
// (math_avx2.c:535-604, 753-769), down product (math_avx2.c:411-495, 771-787) — but for all tokens
// routed to an expert at once instead of one token at a time (model_qwen3.c:415).
//
// Formulation: out^T = W . x^T.  Weight rows fill the 128-row M dimension of the MMA (expert row
// counts are multiples of 128), the ragged token count of an expert is the N dimension (tiles of
// up to 64 tokens).  A weight of a 256-wide super-block is d * (integer) - dmin * (integer)
// (tc_dequant.cuh), so the tensor cores multiply EXACT small-integer fp16 weights with the
// activations (split into fp16 hi + lo: 22 significand bits; one fp16 is not accurate enough
// for the 1e-3 parity bound) and the fp32 block factors are applied once per super-block:
//   out[r][n] = sum_B  d[r][B]    * sum_{k in B}  (sc*q)[r][k] * x[n][k]          ("P" partial sums)
//                    - dmin[r][B] * sum_{b in B}  m[r][b] * xsum[n][b]            ("M" partial sums)
// where xsum[n][b] is the sum of x[n] over the 32-wide sub-block b (Q4_K only; one extra 16-deep
// MMA step per super-block).
//
// The kernel is persistent: one CTA per SM walks (token tile, 128-row tile) work items.  Roles:
//   * 8 producer warps read packed blocks (128-bit loads, prefetched one 128-k group ahead, across
//     work items too), expand them with one HFMA2 per two weights and write the A tiles to TENSOR
//     MEMORY (tcgen05.st) into a ring of 64-k stages;
//   * one thread issues TMA tile loads of the token operand (hi/lo fp16, expert-sorted rows,
//     16-row boxes: only rows the expert really has) and of the sub-block sums into shared memory;
//   * one thread issues tcgen05.mma (kind::f16, fp32 accumulate): per 16-wide k step
//     P += A.B_hi, P += A.B_lo, into one of two accumulator buffers that alternate per super-block;
//   * 8 drain warps take a finished super-block out of tensor memory (tcgen05.ld), fold it into
//     fp32 registers with d / dmin, and after the last super-block of a work item store the rows —
//     while the MMAs of the next super-block / work item already run.
// All hand-offs go through mbarriers (tcgen05.commit on the MMA side).  Every wait is bounded: on
// a timeout the CTA raises ST_WAIT_TIMEOUT in the status word, all roles leave their loops, tensor
// memory is released and the kernel returns.
#include "common.cuh"
#include "kernels.cuh"
#include "tc_dequant.cuh"
#include "tc_ptx.cuh"

namespace tie {

constexpr int TC_BM = 128;
constexpr int TC_BK = 64;
constexpr int TC_NT = TC_TOKEN_TILE;  // tokens per tile (N of the MMAs, at most)
constexpr int TC_PWARPS = 8;		  // producer warps
constexpr int TC_DWARPS = 8;		  // drain warps
constexpr int TC_MWARPS = 2;		  // MMA issuer warps: one per accumulator buffer
constexpr int TC_THREADS = (TC_PWARPS + TC_DWARPS + TC_MWARPS + 1) * 32;
constexpr int TC_S = 7;	  // ring stages: weight tiles in tensor memory, token tiles in shared memory
constexpr int TC_XT = 2;  // 64-wide tiles of sub-block sums per work item, at most (k <= 4096)
constexpr long long TC_WAIT_CYCLES = 1ll << 30;	 // about half a second of SM clocks
constexpr float TC_H_SCALE = 1.0f / 256.0f;	 // keeps SwiGLU outputs inside fp16 range; exact (power of two)

// tensor-memory columns
constexpr uint32_t TC_COL_P = 0;      // 2 x 64: P partial sums
constexpr uint32_t TC_COL_M = 128;    // 2 x 64: M partial sums
constexpr uint32_t TC_COL_AM = 256;   // 2 x 8:  A tile of the M step (8 mins + 8 zeros per row)
constexpr uint32_t TC_COL_A = 288;    // TC_S x 32: A ring
constexpr uint32_t TC_TMEM_COLS = 512;
static_assert(TC_COL_A + TC_S * 32 <= TC_TMEM_COLS, "tensor memory budget");

constexpr int TC_B_TILE = TC_NT * TC_BK * 2;  // bytes of one (hi or lo) token tile
constexpr int TC_B_STAGE = 2 * TC_B_TILE;
constexpr int TC_SMEM = TC_S * TC_B_STAGE + 2 * TC_XT * TC_B_STAGE + 1024 /* alignment slack */ + 512 /* barriers */;

struct TcShared {
	uint64_t full[TC_S];	 // weight stage written by the producers
	uint64_t bfull[TC_S];	 // token tiles of the stage landed (TMA transaction bytes)
	uint64_t empty[TC_S];	 // stage consumed by the MMAs (both operands)
	uint64_t pfull[2];	 // accumulator buffer complete (one super-block)
	uint64_t pempty[2];	 // accumulator buffer read out by the drain warps
	uint64_t xfull[2];	 // sub-block sums of a work item landed
	uint64_t xempty[2];	 // ... and consumed
	uint32_t tmem_base;
	uint32_t abort;
};

// Optional cycle accounting per role (compile with -DTC_TIMING): lane 0 of one warp per role adds
// its clock64() deltas to g_tc_cycles; tie_debug_tc_cycles() reads and clears them.
#ifdef TC_TIMING
__device__ unsigned long long g_tc_cycles[32];
__device__ long long g_tc_trace[8][128];
#define TCT_TRACE(r, i)                                             \
	do {                                                        \
		if (blockIdx.x == 0 && (i) < 128u && (lane) == 0)   \
			g_tc_trace[r][i] = clock64();               \
	} while (0)
#define TCT_DECL(n) long long tct_[n] = {0}
#define TCT_NOW() clock64()
#define TCT_ADD(i, t0) tct_[i] += clock64() - (t0)
#define TCT_FLUSH(base, n)                                                        \
	do {                                                                      \
		for (int i_ = 0; i_ < (n); i_++)                                  \
			atomicAdd(&g_tc_cycles[(base) + i_], (unsigned long long)tct_[i_]); \
	} while (0)
#else
#define TCT_DECL(n)
#define TCT_NOW() 0ll
#define TCT_ADD(i, t0) (void)(t0)
#define TCT_FLUSH(base, n)
#define TCT_TRACE(r, i)
#endif

// Bounded wait: false (and the abort flag raised) when the barrier does not flip in time or
// another role / CTA has already reported a timeout.  After a first miss the thread lets the
// hardware suspend it between polls, so that waiting roles do not take issue slots from the
// producers.
__device__ __forceinline__ bool tc_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag, unsigned *status)
{
	if (ptx::mbar_try_wait(bar, parity))
		return true;
	const long long t0 = clock64();
	uint32_t spins = 0;
	while (!ptx::mbar_try_wait_suspend(bar, parity, 20000u)) {
		if (*abort_flag)
			return false;
		if (clock64() - t0 > TC_WAIT_CYCLES || ((++spins & 255u) == 0 && (*(volatile unsigned *)status & ST_WAIT_TIMEOUT))) {
			atomicOr(status, ST_WAIT_TIMEOUT);
			*abort_flag = 1;
			return false;
		}
	}
	return true;
}

// One lane polls for its warp; the verdict is shared.
__device__ __forceinline__ bool tc_wait_warp(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag, unsigned *status, int lane)
{
	int ok = 1;
	if (lane == 0)
		ok = tc_wait(bar, parity, abort_flag, status) ? 1 : 0;
	return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// A work item: token tile `slot` (expert le, sorted rows [row0, row0 + n_valid)) x 128-row tile.
struct TcItem {
	int le, row0, n_valid, n_mma;
	int mat_sel, m0;  // which matrix (RAW: 0 gate, 1 up) and first row inside it
};

__device__ __forceinline__ TcItem tc_item(int t, int m_tiles, const int4 *__restrict__ tile_info, int rows_per_matrix)
{
	TcItem it;
	const int slot = t / m_tiles, mt = t - slot * m_tiles;
	const int4 ti = __ldg(tile_info + slot);
	it.le = ti.x;
	it.row0 = ti.y;
	it.n_valid = ti.z;
	it.n_mma = (ti.z + 15) & ~15;
	it.mat_sel = (mt * TC_BM) / rows_per_matrix;
	it.m0 = mt * TC_BM - it.mat_sel * rows_per_matrix;
	return it;
}

// Packed weights one producer thread needs for two consecutive k stages (128 k, "group" g) of its
// row: the thread owns the 32-k half-slice hs of each 64-k stage.
template <WKind KIND>
struct RawGroup;

template <>
struct RawGroup<W_Q4K> {
	uint4 hdr;   // d | dmin, 12 bytes of 6-bit scales and mins
	uint4 q[2];  // 16 bytes of quants per stage
	__device__ __forceinline__ void load(const uint8_t *wexp, int nb, int row, int g, int hs)
	{
		const uint8_t *blk = wexp + ((size_t)row * nb + (g >> 1)) * Q4K_BYTES;
		hdr = __ldg(reinterpret_cast<const uint4 *>(blk));
#pragma unroll
		for (int st = 0; st < 2; st++)
			q[st] = __ldg(reinterpret_cast<const uint4 *>(blk + 16 + 32 * ((g & 1) * 2 + st)) + hs);
	}
	// this thread's 32 weights of stage (2g + st) -> 16 columns of its lane in the A tile
	__device__ __forceinline__ void emit(int g, int st, int hs, uint32_t tile) const
	{
		const int p = (g & 1) * 2 + st;
		const uint32_t sc[3] = {hdr.y, hdr.z, hdr.w};
		int s_lo, m_lo, s_hi, m_hi;
		q4k_scale_min(sc, 2 * p, s_lo, m_lo);
		q4k_scale_min(sc, 2 * p + 1, s_hi, m_hi);
		const Q4kConsts c = q4k_int_consts(s_lo, s_hi);
		const uint32_t w[4] = {q[st].x, q[st].y, q[st].z, q[st].w};
#pragma unroll
		for (int cc = 0; cc < 2; cc++) {
			uint32_t l0[2], h0[2], l1[2], h1[2];
			q4k_int_word(w[2 * cc], c, l0, h0);
			q4k_int_word(w[2 * cc + 1], c, l1, h1);
			ptx::tmem_st4(tile + 4u * (2u * hs + cc), l0[0], l0[1], l1[0], l1[1]);	     // k = 16 hs + 8 cc ..
			ptx::tmem_st4(tile + 4u * (4u + 2u * hs + cc), h0[0], h0[1], h1[0], h1[1]);  // k = 32 + 16 hs + 8 cc ..
		}
	}
	// A tile of the M step of super-block sbi: the 8 mins of the row in the half of the 16-deep
	// step that belongs to this super-block (sub-block sums of two super-blocks share a step).
	__device__ __forceinline__ void emit_mins(int sbi, uint32_t tile) const
	{
		const uint32_t sc[3] = {hdr.y, hdr.z, hdr.w};
		uint32_t mm[4];
#pragma unroll
		for (int j = 0; j < 4; j++) {
			int s0, m0, s1, m1;
			q4k_scale_min(sc, 2 * j, s0, m0);
			q4k_scale_min(sc, 2 * j + 1, s1, m1);
			mm[j] = h2_bits(__floats2half2_rn((float)m0, (float)m1));
		}
		const uint32_t odd = (uint32_t)(sbi & 1);
		ptx::tmem_st4(tile + 4u * odd, mm[0], mm[1], mm[2], mm[3]);
		ptx::tmem_st4(tile + 4u * (odd ^ 1u), 0u, 0u, 0u, 0u);
	}
};

template <>
struct RawGroup<W_Q6K_R8> {
	uint4 a, b, h;
	uint32_t scw;
	__device__ __forceinline__ void load(const uint8_t *wexp, int nb, int row, int g, int hs)
	{
		const uint8_t *grp = wexp + (size_t)(row >> 3) * q6k_r8_group_bytes(nb);
		const int r8 = row & 7, kb = g >> 1, pp = (g & 1) * 2 + hs;
		const uint4 *ch = reinterpret_cast<const uint4 *>(grp + q6k_r8_chunk_off(nb, r8, kb, pp));
		a = __ldg(ch);
		b = __ldg(ch + 1);
		h = __ldg(ch + 2);
		scw = __ldg(reinterpret_cast<const uint32_t *>(grp + q6k_r8_scale_off(nb, r8, kb, pp)));
	}
	__device__ __forceinline__ void emit(int g, int st, int hs, uint32_t tile) const
	{
		const float fA = (float)(int)(signed char)((scw >> (16 * st)) & 0xff);
		const float fB = (float)(int)(signed char)((scw >> (16 * st + 8)) & 0xff);
		const __half2 sA = __float2half2_rn(fA), cA = __float2half2_rn(-96.0f * fA);
		const __half2 sB = __float2half2_rn(fB), cB = __float2half2_rn(-96.0f * fB);
		const uint32_t A[4] = {a.x, a.y, a.z, a.w}, B[4] = {b.x, b.y, b.z, b.w}, Hh[4] = {h.x, h.y, h.z, h.w};
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
			uint32_t v0[2], v1[2];
			q6k_int_word(qa[2 * cc], sA, cA, v0);
			q6k_int_word(qa[2 * cc + 1], sA, cA, v1);
			ptx::tmem_st4(tile + 4u * (2u * hs + cc), v0[0], v0[1], v1[0], v1[1]);
			q6k_int_word(qb[2 * cc], sB, cB, v0);
			q6k_int_word(qb[2 * cc + 1], sB, cB, v1);
			ptx::tmem_st4(tile + 4u * (4u + 2u * hs + cc), v0[0], v0[1], v1[0], v1[1]);
		}
	}
	__device__ __forceinline__ void emit_mins(int, uint32_t) const {}
};

// fp32 block factors (d, dmin) of (row, super-block) for the drain warps.
template <WKind KIND>
__device__ __forceinline__ float2 tc_block_factors(const uint8_t *wexp, int nb, int row, int sbi)
{
	if (KIND == W_Q4K) {
		const uint32_t v = __ldg(reinterpret_cast<const uint32_t *>(wexp + ((size_t)row * nb + sbi) * Q4K_BYTES));
		return make_float2(half_bits_to_float(v & 0xffffu), half_bits_to_float(v >> 16));
	}
	const uint8_t *grp = wexp + (size_t)(row >> 3) * q6k_r8_group_bytes(nb);
	const unsigned short v = __ldg(reinterpret_cast<const unsigned short *>(grp + q6k_r8_d_off(nb, row & 7, sbi)));
	return make_float2(half_bits_to_float(v), 0.0f);
}

// RAW: products are stored as fp32 in expert-sorted row order, y[row0 + n][matrix * rows + mrow]
// (gate | up of one row side by side) for the SwiGLU pass; the 128-row tiles then run over w0
// followed by w1.  Otherwise (down) rows are scattered to y[perm[row0 + n]][mrow] * out_scale.
template <WKind KIND, bool RAW>
__global__ void __launch_bounds__(TC_THREADS, 1)
grouped_gemm_sb(const __grid_constant__ CUtensorMap tm_hi, const __grid_constant__ CUtensorMap tm_lo,
		const __grid_constant__ CUtensorMap tq_hi, const __grid_constant__ CUtensorMap tq_lo, const uint8_t *__restrict__ w0,
		const uint8_t *__restrict__ w1, size_t expert_stride, int k_dim, const int4 *__restrict__ tile_info,
		const int *__restrict__ tile_start, int n_local, int m_tiles, float *__restrict__ y, const int *__restrict__ perm,
		int out_stride, float out_scale, unsigned *__restrict__ status, int rows_per_matrix)
{
	extern __shared__ uint8_t smem_raw[];
	__shared__ int s_total;
	if (threadIdx.x == 0)
		s_total = (*(volatile unsigned *)status & ST_WAIT_TIMEOUT) ? 0 : tile_start[n_local] * m_tiles;
	__syncthreads();
	const int total = s_total;
	if ((int)blockIdx.x >= total)
		return;
	const int nb = k_dim / QK_K;
	const int k_iters = k_dim / TC_BK;
	const int xt_n = (nb + 7) >> 3;

	const uint32_t raw = ptx::smem_u32(smem_raw);
	const uint32_t tiles = (raw + 1023u) & ~1023u;
	const uint32_t xq_base = tiles + TC_S * TC_B_STAGE;
	TcShared *sh = reinterpret_cast<TcShared *>(smem_raw + (tiles - raw) + (size_t)(TC_S + 2 * TC_XT) * TC_B_STAGE);
	const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

	auto b_hi = [&](int sb) -> uint32_t { return tiles + sb * TC_B_STAGE; };
	auto b_lo = [&](int sb) -> uint32_t { return tiles + sb * TC_B_STAGE + TC_B_TILE; };
	auto xq_tile = [&](int tp, int xt, int hl) -> uint32_t { return xq_base + ((tp * TC_XT + xt) * 2 + hl) * TC_B_TILE; };

	if (threadIdx.x == 0) {
		for (int s = 0; s < TC_S; s++) {
			ptx::mbar_init(ptx::smem_u32(&sh->full[s]), TC_PWARPS);
			ptx::mbar_init(ptx::smem_u32(&sh->empty[s]), 1);
			ptx::mbar_init(ptx::smem_u32(&sh->bfull[s]), 1);
		}
		for (int s = 0; s < 2; s++) {
			ptx::mbar_init(ptx::smem_u32(&sh->pfull[s]), 1);
			ptx::mbar_init(ptx::smem_u32(&sh->pempty[s]), TC_DWARPS);
			ptx::mbar_init(ptx::smem_u32(&sh->xfull[s]), 1);
			ptx::mbar_init(ptx::smem_u32(&sh->xempty[s]), TC_MWARPS);
		}
		sh->abort = 0;
		ptx::fence_barrier_init();
		ptx::fence_proxy_async_smem();
	}
	if (warp == TC_PWARPS + TC_DWARPS) {  // the MMA warp owns the tensor-memory allocation
		ptx::tmem_alloc(ptx::smem_u32(&sh->tmem_base), TC_TMEM_COLS);
		ptx::tmem_relinquish();
	}
	if (warp == TC_PWARPS + TC_DWARPS + TC_MWARPS && lane == 0) {
		ptx::prefetch_tmap(&tm_hi);
		ptx::prefetch_tmap(&tm_lo);
		if (KIND == W_Q4K) {
			ptx::prefetch_tmap(&tq_hi);
			ptx::prefetch_tmap(&tq_lo);
		}
	}
	ptx::tc_fence_before();
	__syncthreads();
	ptx::tc_fence_after();
	const uint32_t tmem = sh->tmem_base;
	volatile uint32_t *abort_flag = &sh->abort;
	const int stride_t = gridDim.x;

	if (warp < TC_PWARPS) {
		// ================= producers: packed blocks -> integer A tiles in tensor memory =================
		const int row = threadIdx.x & 127, hs = threadIdx.x >> 7;
		const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
		const int n_groups = k_iters >> 1;
		int s = 0;
		uint32_t ph = 0, it = 0, g = 0;
		// Load cursor: runs three 128-k groups (about 5000 cycles of work, several HBM latencies)
		// ahead of the group being expanded, across work items.
		int lt = blockIdx.x, lgi = 0;
		TcItem litem = tc_item(lt, m_tiles, tile_info, rows_per_matrix);
		const uint8_t *lwexp = (litem.mat_sel ? w1 : w0) + (size_t)litem.le * expert_stride;
		bool lvalid = true;
		auto fetch = [&](RawGroup<KIND> &dst) {
			if (!lvalid)
				return;
			dst.load(lwexp, nb, litem.m0 + row, lgi, hs);
			if (++lgi == n_groups) {
				lgi = 0;
				lt += stride_t;
				lvalid = lt < total;
				if (lvalid) {
					litem = tc_item(lt, m_tiles, tile_info, rows_per_matrix);
					lwexp = (litem.mat_sel ? w1 : w0) + (size_t)litem.le * expert_stride;
				}
			}
		};
		RawGroup<KIND> q0, q1, q2, fresh;
		fetch(q0);
		fetch(q1);
		fetch(q2);
		bool alive = true;
		TCT_DECL(5);
		const long long tct_start = TCT_NOW();
		int t = blockIdx.x, gi = 0;
		while (alive) {
			fetch(fresh);
#pragma unroll
			for (int st = 0; st < 2; st++) {
				const long long tw = TCT_NOW();
				if (it >= (uint32_t)TC_S) {
					if (!tc_wait_warp(ptx::smem_u32(&sh->empty[s]), ph ^ 1u, abort_flag, status, lane)) {
						alive = false;
						break;
					}
					ptx::tc_fence_after();
				}
				TCT_ADD(0, tw);
				if (warp == 0)
					TCT_TRACE(0, it);
				const long long te = TCT_NOW();
				// first stage of a super-block: the A tile of its M step (rows are owned by the hs = 0 warps)
				if (KIND == W_Q4K && st == 0 && (gi & 1) == 0 && hs == 0)
					q0.emit_mins(gi >> 1, lane_base + TC_COL_AM + 8u * (g & 1u));
				q0.emit(gi, st, hs, lane_base + TC_COL_A + 32u * s);
				TCT_ADD(1, te);
				const long long ts = TCT_NOW();
				ptx::tmem_st_wait();
				TCT_ADD(2, ts);
				ptx::tc_fence_before();
				__syncwarp();
				if (lane == 0)
					ptx::mbar_arrive(ptx::smem_u32(&sh->full[s]));
				if (warp == 0)
					TCT_TRACE(1, it);
				if (warp == 7)
					TCT_TRACE(2, it);
				it++;
				if (++s == TC_S) {
					s = 0;
					ph ^= 1u;
				}
			}
			if (gi & 1)
				g++;
			q0 = q1;
			q1 = q2;
			q2 = fresh;
			if (++gi == n_groups) {
				gi = 0;
				t += stride_t;
				if (t >= total)
					break;
			}
		}
		TCT_ADD(3, tct_start);
#ifdef TC_TIMING
		tct_[4] = it;
#endif
		if (threadIdx.x == 0)
			TCT_FLUSH(0, 5);
	} else if (warp < TC_PWARPS + TC_DWARPS) {
		// ================= drain warps: super-block partial sums -> fp32 rows =================
		const int dw = warp - TC_PWARPS, quad = warp & 3, chalf = dw >> 2;
		const int c0 = chalf * (TC_NT / 2);
		const uint32_t tlane = tmem + ((uint32_t)(quad * 32) << 16);
		uint32_t g = 0;
		bool alive = true;
		TCT_DECL(4);
		const long long tct_start = TCT_NOW();
		for (int t = blockIdx.x; t < total && alive; t += stride_t) {
			const TcItem item = tc_item(t, m_tiles, tile_info, rows_per_matrix);
			const uint8_t *wexp = (item.mat_sel ? w1 : w0) + (size_t)item.le * expert_stride;
			const int mrow = item.m0 + quad * 32 + lane;
			float acc[TC_NT / 2];
#pragma unroll
			for (int j = 0; j < TC_NT / 2; j++)
				acc[j] = 0.0f;
			float2 fnext = tc_block_factors<KIND>(wexp, nb, mrow, 0);
			for (int sbi = 0; sbi < nb; sbi++) {
				const float2 f = fnext;
				if (sbi + 1 < nb)
					fnext = tc_block_factors<KIND>(wexp, nb, mrow, sbi + 1);
				const uint32_t buf = g & 1u;
				const long long tw = TCT_NOW();
				if (!tc_wait_warp(ptx::smem_u32(&sh->pfull[buf]), (g >> 1) & 1u, abort_flag, status, lane)) {
					alive = false;
					break;
				}
				TCT_ADD(0, tw);
				if (warp == TC_PWARPS)
					TCT_TRACE(5, g);
				const long long tl = TCT_NOW();
				ptx::tc_fence_after();
#pragma unroll
				for (int hf = 0; hf < 2; hf++) {
					if (c0 + 16 * hf < item.n_mma) {  // warp-uniform
						uint32_t p[16], m[16];
						ptx::tmem_ld16(tlane + TC_COL_P + 64u * buf + c0 + 16 * hf, p);
						if (KIND == W_Q4K)
							ptx::tmem_ld16(tlane + TC_COL_M + 64u * buf + c0 + 16 * hf, m);
						ptx::tmem_ld_wait();
#pragma unroll
						for (int j = 0; j < 16; j++) {
							float a = __fmaf_rn(f.x, __uint_as_float(p[j]), acc[16 * hf + j]);
							if (KIND == W_Q4K)
								a = __fmaf_rn(-f.y, __uint_as_float(m[j]), a);
							acc[16 * hf + j] = a;
						}
					}
				}
				ptx::tc_fence_before();
				__syncwarp();
				if (lane == 0)
					ptx::mbar_arrive(ptx::smem_u32(&sh->pempty[buf]));
				TCT_ADD(1, tl);
				if (warp == TC_PWARPS)
					TCT_TRACE(6, g);
				g++;
			}
			if (!alive)
				break;
			const long long tst = TCT_NOW();
			// rows of this work item: lanes hold consecutive output columns (coalesced 128-byte stores)
			int rid = 0;
			if (!RAW && c0 + lane < item.n_valid)
				rid = perm[item.row0 + c0 + lane];
#pragma unroll
			for (int j = 0; j < TC_NT / 2; j++) {
				const int n = c0 + j;
				const int rj = RAW ? 0 : __shfl_sync(0xffffffffu, rid, j);
				if (n < item.n_valid) {
					if (RAW)
						y[(size_t)(item.row0 + n) * out_stride + (size_t)item.mat_sel * rows_per_matrix + mrow] = acc[j];
					else
						y[(size_t)rj * out_stride + mrow] = acc[j] * out_scale;
				}
			}
			TCT_ADD(2, tst);
		}
		TCT_ADD(3, tct_start);
		if (warp == TC_PWARPS && lane == 0)
			TCT_FLUSH(8, 4);
	} else if (warp < TC_PWARPS + TC_DWARPS + TC_MWARPS) {
		// ================= MMA issuers =================
		// One thread can issue a tcgen05.mma only every ~110-130 cycles whatever its N, so the
		// super-blocks are dealt to TC_MWARPS issuer warps: warp w owns accumulator buffer w and the
		// super-blocks that use it; MMAs of different issuers run concurrently on different buffers.
		// The whole warp walks the loop (warp-uniform addresses and descriptors); lane 0 issues.
		{
			const uint32_t mw = warp - (TC_PWARPS + TC_DWARPS);
			const uint32_t leader = (lane == 0) ? 1u : 0u;
			int s = 0;
			uint32_t ph = 0, g = 0, tl = 0;
			bool alive = true;
			TCT_DECL(5);
			const long long tct_start = TCT_NOW();
			for (int t = blockIdx.x; t < total && alive; t += stride_t, tl++) {
				const TcItem item = tc_item(t, m_tiles, tile_info, rows_per_matrix);
#ifdef TC_EXP_N
				const uint32_t idesc = ptx::umma_idesc_f16(TC_BM, TC_EXP_N);
#else
				const uint32_t idesc = ptx::umma_idesc_f16(TC_BM, item.n_mma);
#endif
				const uint32_t tp = tl & 1u;
				bool need_x = KIND == W_Q4K;  // this issuer has not yet seen the work item's sub-block sums
				for (int sbi = 0; sbi < nb && alive; sbi++) {
					const uint32_t buf = g & 1u;
					if (buf != mw) {  // the other issuer's super-block: skip its stages
						s += QK_K / TC_BK;
						if (s >= TC_S) {
							s -= TC_S;
							ph ^= 1u;
						}
						g++;
						continue;
					}
					const long long tpe = TCT_NOW();
					if (g >= 2u) {
						const bool ok = tc_wait(ptx::smem_u32(&sh->pempty[buf]), ((g >> 1) & 1u) ^ 1u, abort_flag, status);
						if (!__all_sync(0xffffffffu, ok)) {
							alive = false;
							break;
						}
					}
					TCT_ADD(0, tpe);
					const uint32_t dP = tmem + TC_COL_P + 64u * buf;
					for (int q4 = 0; q4 < QK_K / TC_BK; q4++) {
						const long long tb = TCT_NOW();
						bool ok = tc_wait(ptx::smem_u32(&sh->bfull[s]), ph, abort_flag, status);
						TCT_ADD(1, tb);
						const long long tf = TCT_NOW();
						ok = ok && tc_wait(ptx::smem_u32(&sh->full[s]), ph, abort_flag, status);
						if (need_x) {
							ok = ok && tc_wait(ptx::smem_u32(&sh->xfull[tp]), (tl >> 1) & 1u, abort_flag, status);
							need_x = false;
						}
						if (!__all_sync(0xffffffffu, ok)) {
							alive = false;
							break;
						}
						TCT_ADD(2, tf);
						TCT_TRACE(3, g * 4u + q4);
						const long long ti = TCT_NOW();
						ptx::tc_fence_after();
						if (KIND == W_Q4K && q4 == 0) {
							// M step: mins (16-deep A tile) x sub-block sums of this super-block pair
							const int xt = sbi >> 3, j = (sbi & 7) >> 1;
							const uint32_t dM = tmem + TC_COL_M + 64u * buf, am = tmem + TC_COL_AM + 8u * buf;
							ptx::mma_f16_ts_if(dM, am, ptx::umma_desc_sw128(xq_tile(tp, xt, 0)) + 2 * j, idesc, 0u, leader);
							ptx::mma_f16_ts_if(dM, am, ptx::umma_desc_sw128(xq_tile(tp, xt, 1)) + 2 * j, idesc, 1u, leader);
						}
						const uint64_t bh = ptx::umma_desc_sw128(b_hi(s)), bl = ptx::umma_desc_sw128(b_lo(s));
						const uint32_t a = tmem + TC_COL_A + 32u * s;
#pragma unroll
						for (int kk = 0; kk < TC_BK / 16; kk++) {
							ptx::mma_f16_ts_if(dP, a + 8 * kk, bh + 2 * kk, idesc, (q4 > 0 || kk > 0) ? 1u : 0u, leader);
#ifndef TC_EXP_NOLO
							ptx::mma_f16_ts_if(dP, a + 8 * kk, bl + 2 * kk, idesc, 1u, leader);
#endif
						}
						ptx::mma_commit_if(ptx::smem_u32(&sh->empty[s]), leader);
						TCT_ADD(3, ti);
						TCT_TRACE(4, g * 4u + q4);
						if (++s == TC_S) {
							s = 0;
							ph ^= 1u;
						}
					}
					if (!alive)
						break;
					ptx::mma_commit_if(ptx::smem_u32(&sh->pfull[buf]), leader);
					g++;
				}
				if (KIND == W_Q4K && alive)
					ptx::mma_commit_if(ptx::smem_u32(&sh->xempty[tp]), leader);
			}
			TCT_ADD(4, tct_start);
			if (lane == 0 && mw == 0)
				TCT_FLUSH(16, 5);
		}
	} else {
		// ================= TMA loader: token operand and sub-block sums =================
		if (lane == 0) {
			int sb = 0;
			uint32_t bph = 0, bit = 0, tl = 0;
			bool alive = true;
			TCT_DECL(2);
			const long long tct_start = TCT_NOW();
			for (int t = blockIdx.x; t < total && alive; t += stride_t, tl++) {
				const TcItem item = tc_item(t, m_tiles, tile_info, rows_per_matrix);
				const int n16 = item.n_mma >> 4;
				if (KIND == W_Q4K) {
					const uint32_t tp = tl & 1u;
					if (tl >= 2u && !tc_wait(ptx::smem_u32(&sh->xempty[tp]), ((tl >> 1) & 1u) ^ 1u, abort_flag, status))
						break;
					const uint32_t xb = ptx::smem_u32(&sh->xfull[tp]);
					ptx::mbar_arrive_expect_tx(xb, (uint32_t)(xt_n * n16) * 2u * 2048u);
					for (int xt = 0; xt < xt_n; xt++)
						for (int r = 0; r < n16; r++) {
							ptx::tma_load_2d(xq_tile(tp, xt, 0) + r * 2048, &tq_hi, xb, xt * 64, item.row0 + 16 * r);
							ptx::tma_load_2d(xq_tile(tp, xt, 1) + r * 2048, &tq_lo, xb, xt * 64, item.row0 + 16 * r);
						}
				}
				for (int ki = 0; ki < k_iters; ki++) {
					const long long tw = TCT_NOW();
					if (bit >= (uint32_t)TC_S && !tc_wait(ptx::smem_u32(&sh->empty[sb]), bph ^ 1u, abort_flag, status)) {
						alive = false;
						break;
					}
					TCT_ADD(0, tw);
					const uint32_t fb = ptx::smem_u32(&sh->bfull[sb]);
					// only the rows the MMA will read: 16-row boxes (2 KB each, whole swizzle groups)
					ptx::mbar_arrive_expect_tx(fb, (uint32_t)n16 * 2u * 2048u);
					for (int r = 0; r < n16; r++) {
						ptx::tma_load_2d(b_hi(sb) + r * 2048, &tm_hi, fb, ki * TC_BK, item.row0 + 16 * r);
						ptx::tma_load_2d(b_lo(sb) + r * 2048, &tm_lo, fb, ki * TC_BK, item.row0 + 16 * r);
					}
					bit++;
					if (++sb == TC_S) {
						sb = 0;
						bph ^= 1u;
					}
				}
			}
			TCT_ADD(1, tct_start);
			TCT_FLUSH(24, 2);
		}
	}

	if (*abort_flag) {
		// give copies that may still be in flight time to land before the CTA's memory is released
		for (int i = 0; i < 200; i++)
			__nanosleep(1000);
	}
	ptx::tc_fence_before();
	__syncthreads();
	if (warp == TC_PWARPS + TC_DWARPS)
		ptx::tmem_dealloc(tmem, TC_TMEM_COLS);
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
	const size_t H = c->cfg.hidden, F = c->cfg.ffn_dim;
	void *bases[8] = {s.xs_hi, s.xs_lo, s.hs_hi, s.hs_lo, s.xq_hi, s.xq_lo, s.hq_hi, s.hq_lo};
	size_t cols[8] = {H, H, F, F, (size_t)xq_cols((int)H), (size_t)xq_cols((int)H), (size_t)xq_cols((int)F), (size_t)xq_cols((int)F)};
	for (int a = 0; a < 8; a++) {
		int rc = make_tmap(c, &c->tmap[a], bases[a], s.rows_pad, cols[a]);
		if (rc)
			return rc;
	}
#define TC_ATTR(KIND, RAW) \
	TIE_CUDA_TRY(c, cudaFuncSetAttribute(grouped_gemm_sb<KIND, RAW>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM))
	TC_ATTR(W_Q4K, false);
	TC_ATTR(W_Q4K, true);
	TC_ATTR(W_Q6K_R8, false);
	TC_ATTR(W_Q6K_R8, true);
#undef TC_ATTR
	c->tmaps_ok = true;
	return TIE_CUDA_OK;
}

// arr: 0 = the split inputs x (gate/up), 2 = the split activations h (down).
template <WKind KIND, bool RAW>
static int launch_tc_t(tie_cuda_ctx *c, const DevTensor &t0, const DevTensor *t1, int arr, float *y, float out_scale)
{
	Scratch &s = c->s;
	const int m_tiles = (RAW ? 2 : 1) * t0.rows / TC_BM;
	grouped_gemm_sb<KIND, RAW><<<c->sm_count, TC_THREADS, TC_SMEM, c->stream>>>(
		c->tmap[arr], c->tmap[arr + 1], c->tmap[4 + arr], c->tmap[5 + arr], t0.ptr, t1 ? t1->ptr : nullptr, t0.expert_stride, t0.k,
		s.tile_info, s.tile_start, c->n_local, m_tiles, y, s.perm, RAW ? 2 * t0.rows : t0.rows, out_scale, s.status, t0.rows);
	TIE_CUDA_LAUNCHED(c);
	return TIE_CUDA_OK;
}

bool tc_supported(const tie_cuda_ctx *c, const Layer &L)
{
	return c->tmaps_ok && L.gate.kind == L.up.kind && L.gate.rows % TC_BM == 0 && L.down.rows % TC_BM == 0 &&
	       L.gate.k % QK_K == 0 && L.down.k % QK_K == 0 && L.gate.k <= TC_XT * 2048 && L.down.k <= TC_XT * 2048;
}

// xs_hi/xs_lo (and xq_hi/xq_lo for Q4_K) must hold the split inputs in sorted order; the sort must
// have been run with TC_TOKEN_TILE.  Writes hs_hi/hs_lo (and hq_hi/hq_lo when the down matrix is Q4_K).
int launch_tc_gate_up(tie_cuda_ctx *c, const Layer &L, int n_rows)
{
	// gate and up as independent 128-row tiles; raw fp32 products to a scratch [row][gate | up],
	// then one element-wise SwiGLU + split pass
	int rc = (L.gate.kind == W_Q4K) ? launch_tc_t<W_Q4K, true>(c, L.gate, &L.up, 0, c->s.y, 1.0f)
					: launch_tc_t<W_Q6K_R8, true>(c, L.gate, &L.up, 0, c->s.y, 1.0f);
	if (rc)
		return rc;
	const bool sums = L.down.kind == W_Q4K;
	return launch_swiglu_split(c, c->s.y, n_rows, L.gate.rows, TC_H_SCALE, c->s.hs_hi, c->s.hs_lo, sums ? c->s.hq_hi : nullptr,
				   sums ? c->s.hq_lo : nullptr);
}

// reads hs_hi/hs_lo; writes y[perm[p]].
int launch_tc_down(tie_cuda_ctx *c, const Layer &L, int n_rows, float *y)
{
	(void)n_rows;
	if (L.down.kind == W_Q4K)
		return launch_tc_t<W_Q4K, false>(c, L.down, nullptr, 2, y, 1.0f / TC_H_SCALE);
	return launch_tc_t<W_Q6K_R8, false>(c, L.down, nullptr, 2, y, 1.0f / TC_H_SCALE);
}

}  // namespace tie

#ifdef TC_TIMING
// Debug builds only: copies out and clears the role cycle counters (32 values).
extern "C" int tie_debug_tc_cycles(unsigned long long *out)
{
	unsigned long long zero[32] = {0};
	if (cudaDeviceSynchronize() != cudaSuccess)
		return -1;
	if (cudaMemcpyFromSymbol(out, tie::g_tc_cycles, sizeof(zero)) != cudaSuccess)
		return -1;
	return cudaMemcpyToSymbol(tie::g_tc_cycles, zero, sizeof(zero)) == cudaSuccess ? 0 : -1;
}
extern "C" int tie_debug_tc_trace(long long *out)
{
	if (cudaDeviceSynchronize() != cudaSuccess)
		return -1;
	return cudaMemcpyFromSymbol(out, tie::g_tc_trace, sizeof(long long) * 8 * 128) == cudaSuccess ? 0 : -1;
}
#endif
