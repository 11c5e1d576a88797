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
//   out[r][n] = sum_B d[r][B] * sum_{k in B} (sc*q)[r][k] * x[n][k]  -  sum_b (dmin*m)[r][b] * xsum[n][b]
// where xsum[n][b] is the sum of x[n] over the 32-wide sub-block b (Q4_K only).  The second term
// is one small extra GEMM per work item (k = number of sub-blocks, at most 64): its weights
// dmin*m (17 significant bits) are split into fp16 hi + lo and it runs ahead of the super-blocks
// as a "min phase" through the same ring and accumulator buffers.
//
// The kernel is persistent: one CTA per SM walks (token tile, 128-row tile) work items.  Roles:
//   * a weight loader thread brings the packed blocks of one super-block x 128 rows into shared
//     memory with TMA (three super-blocks in flight: the HBM latency is hidden by the hardware,
//     not by registers, and no thread issues scattered 16-byte loads);
//   * 8 producer warps expand them (one HFMA2 per two weights) and write the A tiles to TENSOR
//     MEMORY (tcgen05.st) into a ring of 64-k stages;
//   * a token loader thread issues TMA tile loads of the token operand (hi/lo fp16, expert-sorted
//     rows, 16-row boxes: only rows the expert really has) and of the sub-block sums;
//   * two MMA issuer warps issue tcgen05.mma (kind::f16, fp32 accumulate), per 16-wide k step
//     P += A.B_hi, P += A.B_lo (one MMA over the stacked hi and lo rows when the tile has at most
//     32 tokens).  A thread can issue only one MMA per ~110-130 cycles whatever its N, so
//     consecutive super-blocks go to different issuers, each with two of the four accumulator
//     buffers;
//   * 8 drain warps take a finished super-block out of tensor memory (tcgen05.ld), fold it into
//     fp32 registers with d (-1 for the min phase), and after the last super-block of a work item
//     store the rows — while the MMAs of the next super-blocks / work item already run.
// All hand-offs go through mbarriers (tcgen05.commit on the MMA side).  Every wait is bounded: on
// a timeout the CTA raises ST_WAIT_TIMEOUT in the status word, all roles leave their loops, tensor
// memory is released and the kernel returns.
//
// PAIR: the kernel runs as clusters of two CTAs (two SMs) that share a token tile and take two
// neighbouring 128-row weight tiles.  Each CTA loads, expands and drains its own weight tile as
// above, but the MMAs are issued once for both by the even-ranked CTA (tcgen05.mma.cta_group::2,
// M = 256): the instruction issue rate of one thread, which bounds the single-CTA form (an MMA
// costs its issuer ~130 cycles whatever its size), is spent on twice the rows, and the token
// operand is split between the two CTAs' shared memories — the leader holds the hi rows of the
// tile, its peer the lo rows, so one MMA per k step covers both (N = 2 x rows) and each CTA
// fetches half the operand bytes.  Barriers that collect arrivals from both CTAs live in the
// leader (remote mbarrier arrivals; TMA loads of the peer count their bytes there); the MMA
// completions are committed to both CTAs at once.  No copy is delivered to more than one CTA.
#include "common.cuh"
#include "kernels.cuh"
#include "tc_dequant.cuh"
#include "tc_ptx.cuh"
#define TIE_TIMING_TC_OWNER
#include "timing.cuh"

namespace tie {

#ifndef TC_EMIT_UNROLL
#define TC_EMIT_UNROLL 2
#endif
constexpr int TC_EMIT_UNROLL_N = TC_EMIT_UNROLL;  // unrolling of the producers' expansion loop
constexpr int TC_BM = 128;
constexpr int TC_BK = 64;
constexpr int TC_SPB = QK_K / TC_BK;	  // stages per super-block
constexpr int TC_NT = TC_TOKEN_TILE;	  // tokens per tile (N of the MMAs, at most)
constexpr int TC_PWARPS = 8;		  // producer warps
constexpr int TC_DWARPS = 8;		  // drain warps
constexpr int TC_MWARPS = 2;		  // MMA issuer warps: one per accumulator buffer
constexpr int TC_THREADS = (TC_PWARPS + TC_DWARPS + TC_MWARPS + 2) * 32;  // + token loader + weight loader
constexpr int TC_S = 8;	    // ring stages: weight tiles in tensor memory, token tiles in shared memory
constexpr int TC_NBUF = 4;  // accumulator buffers of 64 columns (two per MMA issuer); pairs: two of 128 columns
constexpr int TC_NDS = 8;   // block-factor hand-off buffers (producers -> drain warps)
constexpr long long TC_WAIT_CYCLES = 1ll << 30;	 // about half a second of SM clocks
constexpr float TC_H_SCALE = 1.0f / 256.0f;	 // keeps SwiGLU outputs inside fp16 range; exact (power of two)

// tensor-memory columns
constexpr uint32_t TC_COL_P = 0;    // TC_NBUF x 64: partial sums of one super-block (or of the min phase)
constexpr uint32_t TC_COL_A = 256;  // TC_S x 32: A ring
constexpr uint32_t TC_TMEM_COLS = 512;
static_assert(TC_COL_A + TC_S * 32 <= TC_TMEM_COLS && TC_NBUF * 64 <= TC_COL_A, "tensor memory budget");

// shared memory
constexpr int TC_B_TILE = TC_NT * TC_BK * 2;  // bytes of one (hi or lo) token tile
constexpr int TC_B_STAGE = 2 * TC_B_TILE;
// packed super-block of 128 rows: the 144-byte Q4_K blocks resp. the 208-byte Q6_K records
// (192 bytes of quants + 16 bytes of scales) of the rows back to back, one TMA box.  Row strides
// of 9 and 13 x 16 bytes: 16-byte reads by 32 consecutive rows are bank-conflict free.
constexpr int TC_Q6_ROW = Q6K_RECORD;
constexpr int TC_NWB_MAX = 4;
template <WKind KIND>
struct TcSmem {
	static constexpr bool Q4 = KIND == W_Q4K;
	static constexpr int NWB = Q4 ? 4 : 3;	// packed super-blocks in flight
	static constexpr int WBUF = TC_BM * (Q4 ? Q4K_BYTES : TC_Q6_ROW);
	static constexpr int OFF_W = TC_S * TC_B_STAGE;
	static constexpr int OFF_XQ = OFF_W + NWB * WBUF;		  // sub-block sums of the work item (Q4_K)
	static constexpr int OFF_DS = OFF_XQ + (Q4 ? TC_B_STAGE : 0);	  // block factors (Q4_K)
	static constexpr int OFF_BAR = OFF_DS + (Q4 ? TC_NDS * TC_BM * 8 : 0);
	static constexpr int SMEM = OFF_BAR + 512 + 1024 /* alignment slack */;
	static_assert(WBUF % 1024 == 0 && NWB <= TC_NWB_MAX, "packed super-block buffers");
	static_assert(SMEM <= 227 * 1024, "shared memory budget");
};

struct TcShared {
	uint64_t full[TC_S];	      // weight stage written by its producer group
	uint64_t bfull[2 * TC_S];     // token tiles of the stage landed (TMA transaction bytes); pairs: a ring of its own, 16 deep
	uint64_t bempty[4];	      // pairs: the four token stages of a super-block consumed
	uint64_t empty[TC_S];	      // stage consumed by the MMAs (both operands)
	uint64_t wfull[TC_NWB_MAX];   // packed super-block landed
	uint64_t wempty[TC_NWB_MAX];  // ... and expanded
	uint64_t pfull[TC_NBUF];      // accumulator buffer complete (one super-block)
	uint64_t pempty[TC_NBUF];     // accumulator buffer read out by the drain warps
	uint64_t xfull;		      // sub-block sums of a work item landed
	uint64_t xempty;	      // ... and consumed by the min phase
	uint64_t msync;		      // producer warps have all written their part of the min-phase tiles
	uint32_t tmem_base;
	uint32_t abort;
};
static_assert(sizeof(TcShared) <= 512, "barrier block");

// Bounded wait: false (and the abort flag raised) when the barrier does not flip in time or
// another role / CTA has already reported a timeout.  After a first miss the thread lets the
// hardware suspend it between polls, so that waiting roles do not take issue slots from the
// producers.
// BACKOFF_NS > 0: roles that can afford a few hundred cycles of extra latency also sleep between polls.
// CL: the barrier collects arrivals of the peer CTA of a pair (acquire at cluster scope).
template <int BACKOFF_NS = 0, bool CL = false>
__device__ __forceinline__ bool tc_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag, unsigned *status)
{
	if (CL ? ptx::mbar_try_wait_cluster(bar, parity) : ptx::mbar_try_wait(bar, parity))
		return true;
	const long long t0 = clock64();
	uint32_t spins = 0;
	while (!(CL ? ptx::mbar_try_wait_suspend_cluster(bar, parity, 20000u) : ptx::mbar_try_wait_suspend(bar, parity, 20000u))) {
		if (BACKOFF_NS > 0)
			__nanosleep(BACKOFF_NS);
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

// A whole warp waits: every lane tests the barrier (no divergence around the wait — a single
// polling lane with a broadcast was measured 5 % slower over the whole kernel) and the warp votes.
template <int BACKOFF_NS = 0>
__device__ __forceinline__ bool tc_wait_warp(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag, unsigned *status, int lane)
{
	(void)lane;
	return __all_sync(0xffffffffu, tc_wait<BACKOFF_NS>(bar, parity, abort_flag, status));
}

// A work item: token tile `slot` (expert le, sorted rows [row0, row0 + n_valid)) x 128-row tile.
struct TcItem {
	int le, row0, n_valid, n_mma;
	int n_box;	  // token rows fetched per stage: 16, 32 or 64 (one TMA box holds the hi and the lo rows)
	int mat_sel, m0;  // which matrix (RAW: 0 gate, 1 up) and first row inside it
};

// tl: how many work items of this CTA precede t; the first TC_ITEMS token-tile records of a CTA
// are staged in shared memory (s_items) when the kernel starts.
constexpr int TC_ITEMS = 48;
// m_items: work items per token tile (128-row tiles, or pairs of them); a CTA of a pair takes the
// tile 2 * item + its rank.
template <bool PAIR>
__device__ __forceinline__ TcItem tc_item(int t, int tl, const int4 *s_items, int m_items, const int4 *__restrict__ tile_info,
					  int rows_per_matrix, uint32_t rank)
{
	TcItem it;
	const int slot = t / m_items, mi = t - slot * m_items;
	const int mt = PAIR ? 2 * mi + (int)rank : mi;
	const int4 ti = tl < TC_ITEMS ? s_items[tl] : __ldg(tile_info + slot);
	it.le = ti.x;
	it.row0 = ti.y;
	it.n_valid = ti.z;
	it.n_mma = (ti.z + 15) & ~15;
	it.n_box = ti.z <= 16 ? 16 : (ti.z <= 32 ? 32 : 64);
	it.mat_sel = (mt * TC_BM) / rows_per_matrix;
	it.m0 = mt * TC_BM - it.mat_sel * rows_per_matrix;
	return it;
}

__device__ __forceinline__ uint4 lds128(uint32_t addr)
{
	uint4 v;
	asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
	return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr)
{
	uint32_t v;
	asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
	return v;
}

// half2 (1024 + b_i, 1024 + b_j) from two bytes of a word: each byte becomes the low mantissa
// bits of 0x6400 | byte.  selector 0x7i5j picks bytes j (low half) and i (high half).
__device__ __forceinline__ __half2 byte_pair_1024(uint32_t w, uint32_t selector)
{
	return bits_h2(__byte_perm(w, 0x64006400u, selector));
}

// Expansion of one packed super-block (already in shared memory) by the producer thread of
// (row, half-slice hs): prepare() once per super-block, emit(p) for each of its four 64-k stages.
template <WKind KIND>
struct Expander;

template <>
struct Expander<W_Q4K> {
	uint32_t rowaddr;	  // this row's 144-byte block
	uint4 hdr;		  // its first 16 bytes: d | dmin, packed 6-bit scales and mins
	uint32_t sc8[2];	  // the 8 scales of the block as bytes (get_scale_min_k4, math_scalar.c:91-100)
	float2 factors;		  // d, dmin
	__device__ __forceinline__ void prepare(uint32_t wbuf, int row)
	{
		rowaddr = wbuf + (uint32_t)row * Q4K_BYTES;
		hdr = lds128(rowaddr);
		factors = make_float2(half_bits_to_float(hdr.x & 0xffffu), half_bits_to_float(hdr.x >> 16));
		sc8[0] = hdr.y & 0x3F3F3F3Fu;
		sc8[1] = (hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u);
	}
	__device__ __forceinline__ uint4 header() const { return hdr; }
	// this thread's 32 weights of stage p -> 16 columns of its lane in the A tile
	__device__ __forceinline__ void emit(int p, int hs, uint32_t tile) const
	{
		const __half2 k1024 = __float2half2_rn(1024.0f);
		const uint32_t sw = sc8[p >> 1];
		const __half2 s_lo = __hsub2(byte_pair_1024(sw, (p & 1) ? 0x7252u : 0x7050u), k1024);
		const __half2 s_hi = __hsub2(byte_pair_1024(sw, (p & 1) ? 0x7353u : 0x7151u), k1024);
		Q4kConsts c;
		c.sl = s_lo;
		c.cl = __hmul2(s_lo, __float2half2_rn(-1024.0f));
		c.sh = __hmul2(s_hi, __float2half2_rn(0.0625f));
		c.ch = __hmul2(s_hi, __float2half2_rn(-64.0f));
		const uint4 q = lds128(rowaddr + 16u + 32u * p + 16u * hs);
		const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
		for (int cc = 0; cc < 2; cc++) {
			uint32_t l0[2], h0[2], l1[2], h1[2];
			q4k_int_word(w[2 * cc], c, l0, h0);
			q4k_int_word(w[2 * cc + 1], c, l1, h1);
			ptx::tmem_st4(tile + 4u * (2u * hs + cc), l0[0], l0[1], l1[0], l1[1]);	     // k = 16 hs + 8 cc ..
			ptx::tmem_st4(tile + 4u * (4u + 2u * hs + cc), h0[0], h0[1], h1[0], h1[1]);  // k = 32 + 16 hs + 8 cc ..
		}
	}
	// Min phase: the products dmin * m of block B of this row (header hdr), exact in fp32 (11 x 6
	// bits), split into fp16 hi + lo: columns 4B .. 4B+3 of the thread's lane in the two A tiles.
	static __device__ __forceinline__ void emit_min_block(const uint4 &hdr, int B, uint32_t tile_hi, uint32_t tile_lo)
	{
		const float dmin = half_bits_to_float(hdr.x >> 16);
		const uint32_t mn[2] = {hdr.z & 0x3F3F3F3Fu, ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u)};
		uint32_t hi[4], lo[4];
#pragma unroll
		for (int j = 0; j < 4; j++) {
			const uint32_t w = mn[j >> 1] >> (16 * (j & 1));
			const float p0 = dmin * (float)(w & 0xffu), p1 = dmin * (float)((w >> 8) & 0xffu);
			const __half2 h = __floats2half2_rn(p0, p1);
			const float2 f = __half22float2(h);
			hi[j] = h2_bits(h);
			lo[j] = h2_bits(__floats2half2_rn(p0 - f.x, p1 - f.y));
		}
		ptx::tmem_st4(tile_hi + 4u * B, hi[0], hi[1], hi[2], hi[3]);
		ptx::tmem_st4(tile_lo + 4u * B, lo[0], lo[1], lo[2], lo[3]);
	}
};

template <>
struct Expander<W_Q6K_R8> {
	uint32_t rowaddr;  // this row's 4 x 48 bytes of quants
	uint32_t scaddr;   // this row's 16 scale bytes
	float2 factors;
	__device__ __forceinline__ uint4 header() const { return make_uint4(0, 0, 0, 0); }
	__device__ __forceinline__ void prepare(uint32_t wbuf, int row)
	{
		rowaddr = wbuf + (uint32_t)row * TC_Q6_ROW;
		scaddr = rowaddr + 192u;
		factors = make_float2(0.0f, 0.0f);
	}
	__device__ __forceinline__ void emit(int p, int hs, uint32_t tile) const
	{
		const int pp = (p >> 1) * 2 + hs, st = p & 1;
		const uint32_t chunk = rowaddr + 48u * pp;
		const uint4 a = lds128(chunk), b = lds128(chunk + 16u), h = lds128(chunk + 32u);
		// scales of the part: bytes {0,1} for st = 0, {2,3} for st = 1; int8 -> half as 1024 + (s ^ 0x80) - 1152
		const uint32_t scx = lds32(scaddr + 4u * pp) ^ 0x80808080u;
		const __half2 k1152 = __float2half2_rn(1152.0f), km96 = __float2half2_rn(-96.0f);
		const __half2 sA = __hsub2(byte_pair_1024(scx, st ? 0x7252u : 0x7050u), k1152);
		const __half2 sB = __hsub2(byte_pair_1024(scx, st ? 0x7353u : 0x7151u), k1152);
		const __half2 cA = __hmul2(sA, km96), cB = __hmul2(sB, km96);
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
};

// RAW: products are stored as fp32 in expert-sorted row order, y[row0 + n][matrix * rows + mrow]
// (gate | up of one row side by side) for the SwiGLU pass; the 128-row tiles then run over w0
// followed by w1.  Otherwise (down) rows are scattered to y[perm[row0 + n]][mrow] * out_scale.
// tm16/32/64: maps of the split token operand ([hi | lo][rows][k], box 64 k x 16/32/64 rows x 2);
// tq16/32/64: the same of its sub-block sums; tw0 / tw1: byte maps of the two weight tensors,
// box = packed super-block x 128 rows.
//
// Every role walks the same sequence of "phases": per work item the min phase (Q4_K; two ring
// stages: hi and lo tiles of dmin*m) and then the super-blocks (four ring stages each).  Phase
// number g selects the accumulator buffer (g % 4) and the MMA issuer (g % 2).
//
// A launch covers the super-blocks [sb0, sb0 + k_dim / 256) of rows that hold nb_total of them
// (k_dim is the launch's share of the input dimension); accumulate != 0 adds to what y already
// holds.  The expert products pass (0, k / 256, 0); a dense Q4_K tensor with more than 2048 inputs
// runs as several launches of at most 8 super-blocks (the min phase takes the sub-block sums of
// one 64-wide tile).
//
// PEER (expert parallelism over peer memory, down product only): sorted row p belongs to row
// dst.row[p] & 0xFFFFFF of rank dst.row[p] >> 24 and is stored there, into that rank's memory
// (dst.y[rank], plain stores over NVLink, 128 contiguous bytes per warp and row).
template <WKind KIND, bool RAW, bool PEER = false, bool PAIR = false>
__global__ void __launch_bounds__(TC_THREADS, 1)
grouped_gemm_sb(const __grid_constant__ CUtensorMap tm16, const __grid_constant__ CUtensorMap tm32,
		const __grid_constant__ CUtensorMap tm64, const __grid_constant__ CUtensorMap tq16,
		const __grid_constant__ CUtensorMap tq32, const __grid_constant__ CUtensorMap tq64,
		const __grid_constant__ CUtensorMap tw0, const __grid_constant__ CUtensorMap tw1, const uint8_t *__restrict__ w0,
		const uint8_t *__restrict__ w1, size_t expert_stride, int k_dim, const int4 *__restrict__ tile_info,
		const int *__restrict__ tile_start, int n_local, int m_tiles, float *__restrict__ y, const int *__restrict__ perm,
		int out_stride, float out_scale, unsigned *__restrict__ status, int rows_per_matrix, const EpDst dst,
		const int sb0, const int nb_total, const int accumulate)
{
	static_assert(!(RAW && PEER), "peer destinations exist for the down product only");
	using Sm = TcSmem<KIND>;
	constexpr bool Q4 = KIND == W_Q4K;
	extern __shared__ uint8_t smem_raw[];
	__shared__ int s_total;
	__shared__ int4 s_items[TC_ITEMS];
#ifdef TC_TIMING
	const long long tct_kernel_start = clock64();
#endif
	// a pair walks the work items together: its index among the pairs, and this CTA's rank in it
	const uint32_t rank = PAIR ? ptx::cluster_ctarank() : 0u;
	const int walker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
	const int stride_t = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
	const int m_items = PAIR ? m_tiles / 2 : m_tiles;
	constexpr int NBUF = PAIR ? 2 : TC_NBUF;	 // accumulator buffers ...
	constexpr uint32_t PW = PAIR ? 128u : 64u;	 // ... and their width in tensor-memory columns
	if (threadIdx.x == 0)
		s_total = (*(volatile unsigned *)status & ST_WAIT_TIMEOUT) ? 0 : tile_start[n_local] * m_items;
	__syncthreads();
	// (a CTA of a pair never returns early: its peer would wait for it at the cluster barrier below)
	const int total = s_total;
	if (!PAIR && walker >= total)
		return;
	if (threadIdx.x < TC_ITEMS) {
		const int t = walker + threadIdx.x * stride_t;
		if (t < total)
			s_items[threadIdx.x] = tile_info[t / m_items];
	}
	const int nb = k_dim / QK_K;
	const int k_iters = k_dim / TC_BK;
	const int min_k16 = (8 * nb + 15) >> 4;	 // 16-deep k steps of the min phase (8 sub-blocks per block)

	const uint32_t raw = ptx::smem_u32(smem_raw);
	const uint32_t tiles = (raw + 1023u) & ~1023u;
	uint8_t *smem = smem_raw + (tiles - raw);
	TcShared *sh = reinterpret_cast<TcShared *>(smem + Sm::OFF_BAR);
	float2 *ds = reinterpret_cast<float2 *>(smem + Sm::OFF_DS);  // [TC_NDS][128] (d, dmin) of the rows (Q4_K)
	const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

	// token tiles of ring stage s: n_box hi rows, directly followed by n_box lo rows.  Pairs: a CTA
	// holds one half of a tile (8 KB at most), in a ring of its own of 2 x TC_S stages — the
	// operand of four super-blocks in flight: the fetch of a stage needs the other CTA's consent
	// (barrier round trips between two SMs), which a ring in step with the weight stages exposes.
	auto b_hi = [&](int s) -> uint32_t { return tiles + s * (PAIR ? TC_B_STAGE / 2 : TC_B_STAGE); };
	const uint32_t xq_hi = tiles + Sm::OFF_XQ;
	auto w_buf = [&](int wb) -> uint32_t { return tiles + Sm::OFF_W + wb * Sm::WBUF; };

	if (threadIdx.x == 0) {
		for (int s = 0; s < TC_S; s++) {
			ptx::mbar_init(ptx::smem_u32(&sh->full[s]), (PAIR ? 2 : 1) * TC_PWARPS / 2);
			ptx::mbar_init(ptx::smem_u32(&sh->empty[s]), 1);
			ptx::mbar_init(ptx::smem_u32(&sh->bfull[s]), 1);
			ptx::mbar_init(ptx::smem_u32(&sh->bfull[TC_S + s]), 1);
		}
		for (int s = 0; s < 4; s++)
			ptx::mbar_init(ptx::smem_u32(&sh->bempty[s]), 1);
		for (int s = 0; s < Sm::NWB; s++) {
			ptx::mbar_init(ptx::smem_u32(&sh->wfull[s]), 1);
			ptx::mbar_init(ptx::smem_u32(&sh->wempty[s]), TC_PWARPS);
		}
		for (int s = 0; s < TC_NBUF; s++) {
			ptx::mbar_init(ptx::smem_u32(&sh->pfull[s]), 1);
			ptx::mbar_init(ptx::smem_u32(&sh->pempty[s]), (PAIR ? 2 : 1) * TC_DWARPS);
		}
		ptx::mbar_init(ptx::smem_u32(&sh->xfull), 1);
		ptx::mbar_init(ptx::smem_u32(&sh->xempty), 1);
		ptx::mbar_init(ptx::smem_u32(&sh->msync), TC_PWARPS);
		sh->abort = 0;
		ptx::fence_barrier_init();
		ptx::fence_proxy_async_smem();
	}
	constexpr int W_MMA0 = TC_PWARPS + TC_DWARPS, W_TOK = W_MMA0 + TC_MWARPS, W_WGT = W_TOK + 1;
	if (warp == W_MMA0) {  // the first MMA warp owns the tensor-memory allocation (pairs: one warp of each CTA, together)
		if (PAIR) {
			ptx::tmem_alloc_pair(ptx::smem_u32(&sh->tmem_base), TC_TMEM_COLS);
			ptx::tmem_relinquish_pair();
		} else {
			ptx::tmem_alloc(ptx::smem_u32(&sh->tmem_base), TC_TMEM_COLS);
			ptx::tmem_relinquish();
		}
	}
	if (warp == W_TOK && lane == 0) {
		ptx::prefetch_tmap(&tm16);
		ptx::prefetch_tmap(&tm32);
		ptx::prefetch_tmap(&tm64);
		if (Q4) {
			ptx::prefetch_tmap(&tq16);
			ptx::prefetch_tmap(&tq32);
			ptx::prefetch_tmap(&tq64);
		}
	}
	if (warp == W_WGT && lane == 0) {
		ptx::prefetch_tmap(&tw0);
		if (RAW)
			ptx::prefetch_tmap(&tw1);
	}
	ptx::tc_fence_before();
	__syncthreads();
	if (PAIR)
		ptx::cluster_sync_all();  // both CTAs' barriers are initialised before either signals the other's
	ptx::tc_fence_after();
	const uint32_t tmem = sh->tmem_base;
	volatile uint32_t *abort_flag = &sh->abort;
	// arrival on a barrier that the MMA issuers (in the leader CTA of a pair) wait on
	auto arrive_issuer = [&](uint64_t *bar) {
		if (PAIR)
			ptx::mbar_arrive_leader(ptx::smem_u32(bar));
		else
			ptx::mbar_arrive(ptx::smem_u32(bar));
	};

	if (warp < TC_PWARPS) {
		// ================= producers: packed blocks (shared memory) -> integer A tiles (tensor memory) =================
		// Two groups of four warps (one warp per 32-row quadrant of tensor memory): group j expands
		// stages 2j and 2j+1 of every super-block, each thread all 64 k of its row per stage, so that
		// a warp synchronises (ring barriers, tcgen05.wait::st) once per super-block instead of once
		// per stage and the two groups work on different stages at the same time.
		const int row = threadIdx.x & 127, grp = threadIdx.x >> 7;
		const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
		int s = 0, wb = 0;  // s: ring slot of the first stage of the next phase
		uint32_t ph = 0, wph = 0, mph = 0, it = 0, g = 0;
		bool alive = true;
		TCT_DECL(5);
		const long long tct_start = TCT_NOW();
		// ring slot and barrier phase of the stage `off` stages after (s, ph)
		auto slot_of = [&](int off, int &so, uint32_t &pho) {
			so = s + off;
			pho = ph;
			if (so >= TC_S) {
				so -= TC_S;
				pho ^= 1u;
			}
		};
		// min phase (after the super-blocks of a work item): this thread owns the blocks
		// [grp * hb, grp * hb + hb) of its row and keeps their headers as the super-blocks pass by
		const int hb = (nb + 1) >> 1;
		uint4 mh[4];
		for (int t = walker; t < total && alive; t += stride_t) {
			for (int sbi = 0; sbi < nb && alive; sbi++) {
				const long long tw = TCT_NOW();
				if (!tc_wait_warp(ptx::smem_u32(&sh->wfull[wb]), wph, abort_flag, status, lane)) {
					alive = false;
					break;
				}
				TCT_ADD(0, tw);
				if (warp == 0)
					TCT_TRACE(6, g);
				Expander<KIND> ex;
				ex.prepare(w_buf(wb), row);
				if (Q4 && grp == 0)
					ds[(g & (TC_NDS - 1)) * TC_BM + row] = ex.factors;
				if (Q4) {
#pragma unroll
					for (int i = 0; i < 4; i++)
						if (sbi == grp * hb + i)
							mh[i] = ex.header();
				}
				// this group's two stages of the super-block
				int sa, sb2;
				uint32_t pha, phb;
				slot_of(2 * grp, sa, pha);
				slot_of(2 * grp + 1, sb2, phb);
				const long long te = TCT_NOW();
				bool ok = true;
				// (ring stages are handed back in pairs — one commit per two stages — on the odd stage's barrier)
				if (it + 2 * grp >= (uint32_t)TC_S)
					ok = tc_wait_warp(ptx::smem_u32(&sh->empty[sb2]), phb ^ 1u, abort_flag, status, lane);
				if (!ok) {
					alive = false;
					break;
				}
				ptx::tc_fence_after();
				TCT_ADD(1, te);
				if ((warp & 3) == 0) {
					TCT_TRACE(0, it + 2 * grp);
					TCT_TRACE(0, it + 2 * grp + 1);
				}
				const long long tm = TCT_NOW();
				// (a loop unrolled twice: two expansions in flight hide their latencies; fully unrolled it is no faster)
#pragma unroll TC_EMIT_UNROLL_N
				for (int q = 0; q < 4; q++)
					ex.emit(2 * grp + (q >> 1), q & 1, lane_base + TC_COL_A + 32u * ((q >> 1) ? sb2 : sa));
				ptx::tmem_st_wait();
				TCT_ADD(2, tm);
				ptx::tc_fence_before();
				__syncwarp();
				if (lane == 0) {
					arrive_issuer(&sh->full[sa]);
					arrive_issuer(&sh->full[sb2]);
					// the packed super-block is expanded by this warp: hand the buffer back to the weight loader
					ptx::mbar_arrive(ptx::smem_u32(&sh->wempty[wb]));
				}
				if ((warp & 3) == 0) {
					TCT_TRACE(1, it + 2 * grp);
					TCT_TRACE(1, it + 2 * grp + 1);
				}
				it += TC_SPB;
				slot_of(TC_SPB, s, ph);
				if (++wb == Sm::NWB) {
					wb = 0;
					wph ^= 1u;
				}
				g++;
			}
			if (Q4 && alive) {
				// ---- min phase: two ring stages, the hi and the lo tile of dmin * m ----
				int s0, s1;
				uint32_t ph0, ph1;
				slot_of(0, s0, ph0);
				slot_of(1, s1, ph1);
				bool ok = true;
				if (it >= (uint32_t)TC_S)
					ok = tc_wait_warp(ptx::smem_u32(&sh->empty[s1]), ph1 ^ 1u, abort_flag, status, lane);
				if (!ok) {
					alive = false;
					break;
				}
				ptx::tc_fence_after();
				const uint32_t tile_hi = lane_base + TC_COL_A + 32u * s0, tile_lo = lane_base + TC_COL_A + 32u * s1;
#pragma unroll
				for (int i = 0; i < 4; i++) {
					const int B = grp * hb + i;
					if (i < hb && B < nb)
						Expander<W_Q4K>::emit_min_block(mh[i], B, tile_hi, tile_lo);
				}
				if ((nb & 1) && grp == 1) {  // pad the last 16-deep k step with zeros
					ptx::tmem_st4(tile_hi + 4u * nb, 0u, 0u, 0u, 0u);
					ptx::tmem_st4(tile_lo + 4u * nb, 0u, 0u, 0u, 0u);
				}
				ptx::tmem_st_wait();
				ptx::tc_fence_before();
				// both tiles are written by all eight warps: meet (bounded wait), then group j reports tile j
				__syncwarp();
				if (lane == 0)
					ptx::mbar_arrive(ptx::smem_u32(&sh->msync));
				if (!tc_wait_warp(ptx::smem_u32(&sh->msync), mph, abort_flag, status, lane)) {
					alive = false;
					break;
				}
				mph ^= 1u;
				if (lane == 0)
					arrive_issuer(&sh->full[grp ? s1 : s0]);
				it += 2;
				slot_of(2, s, ph);
				g++;
			}
		}
		TCT_ADD(3, tct_start);
#ifdef TC_TIMING
		tct_[4] = it;
		if (threadIdx.x == 0) {
			atomicMax(&g_tc_cycles[28], (unsigned long long)tct_[3]);
			atomicMax(&g_tc_cycles[29], (unsigned long long)it);
			atomicMax(&g_tc_cycles[30], (unsigned long long)(clock64() - tct_kernel_start));
		}
#endif
		if (threadIdx.x == 0)
			TCT_FLUSH(0, 5);
	} else if (warp < W_MMA0) {
		// ================= drain warps: partial sums of a phase -> fp32 rows =================
		const int dw = warp - TC_PWARPS, quad = warp & 3, chalf = dw >> 2;
		const int lrow = quad * 32 + lane;
		const uint32_t tlane = tmem + ((uint32_t)(quad * 32) << 16);
		uint32_t g = 0;
		bool alive = true;
		TCT_DECL(4);
		const long long tct_start = TCT_NOW();
		int dtl = 0;
		for (int t = walker; t < total && alive; t += stride_t, dtl++) {
			const TcItem item = tc_item<PAIR>(t, dtl, s_items, m_items, tile_info, rows_per_matrix, rank);
			const int mrow = item.m0 + lrow;
			// Tokens of this warp: half of the tile's token range, in chunks of 16 accumulator columns.
			// A tile of up to 32 tokens (any tile of a pair) has its hi and lo products side by side in
			// one accumulator (columns j and n_box + j, one MMA per k step); a larger tile of the
			// single-CTA form has them summed by two MMAs.
			const bool concat = PAIR || item.n_box <= 32;
			const int ntok = item.n_box == 64 ? 32 : 16;
			const int tok0 = chalf * ntok;
			float acc[TC_NT / 2];
#pragma unroll
			for (int j = 0; j < TC_NT / 2; j++)
				acc[j] = 0.0f;
			// Q6_K: d of (row, super-block) straight from global memory, one super-block ahead
			const uint8_t *grp = nullptr;
			float dnext = 0.0f;
			if (!Q4) {
				grp = (item.mat_sel ? w1 : w0) + (size_t)item.le * expert_stride + (size_t)(mrow >> 3) * q6k_r8_group_bytes(nb_total);
				dnext = half_bits_to_float(__ldg(reinterpret_cast<const unsigned short *>(grp + q6k_r8_d_off(nb_total, mrow & 7, sb0))));
			}
			// the phase after the last super-block is the min phase (Q4_K): its sums enter with factor -1
			for (int sbi = 0; sbi < (Q4 ? nb + 1 : nb); sbi++) {
				float scale = Q4 ? -1.0f : dnext;
				if (!Q4 && sbi + 1 < nb)
					dnext = half_bits_to_float(
						__ldg(reinterpret_cast<const unsigned short *>(grp + q6k_r8_d_off(nb_total, mrow & 7, sb0 + sbi + 1))));
				const uint32_t buf = g & (NBUF - 1);
				const long long tw = TCT_NOW();
				if (!tc_wait_warp<100>(ptx::smem_u32(&sh->pfull[buf]), (g / NBUF) & 1u, abort_flag, status, lane)) {
					alive = false;
					break;
				}
				TCT_ADD(0, tw);
				if (warp == TC_PWARPS)
					TCT_TRACE(4, g);
				const long long tl = TCT_NOW();
				ptx::tc_fence_after();
				if (Q4 && sbi < nb)
					scale = ds[(g & (TC_NDS - 1)) * TC_BM + lrow].x;
				const uint32_t pcol = tlane + TC_COL_P + PW * buf;
#pragma unroll
				for (int ch = 0; ch < 2; ch++) {  // chunks of 16 accumulator columns
					const int c0 = tok0 + 16 * ch;
					if (ch * 16 < ntok && c0 < item.n_mma) {  // warp-uniform
						uint32_t p[16], p2[16];
						ptx::tmem_ld16(pcol + c0, p);
						if (concat)
							ptx::tmem_ld16(pcol + item.n_box + c0, p2);
						ptx::tmem_ld_wait();
#pragma unroll
						for (int j = 0; j < 16; j++) {
							const float v = concat ? __uint_as_float(p[j]) + __uint_as_float(p2[j]) : __uint_as_float(p[j]);
							acc[16 * ch + j] = __fmaf_rn(scale, v, acc[16 * ch + j]);
						}
					}
				}
				ptx::tc_fence_before();
				__syncwarp();
				if (lane == 0)
					arrive_issuer(&sh->pempty[buf]);
				TCT_ADD(1, tl);
				if (warp == TC_PWARPS)
					TCT_TRACE(5, g);
				g++;
			}
			if (!alive)
				break;
			const long long tst = TCT_NOW();
			// rows of this work item: lanes hold consecutive output columns (coalesced 128-byte stores)
			int rid = 0;
			if (!RAW && lane < ntok && tok0 + lane < item.n_valid) {
				if (PEER)
					rid = (int)dst.row[item.row0 + tok0 + lane];
				else
					rid = perm ? perm[item.row0 + tok0 + lane] : item.row0 + tok0 + lane;
			}
#pragma unroll
			for (int j = 0; j < TC_NT / 2; j++) {
				const int n = tok0 + j;
				const int rj = RAW ? 0 : __shfl_sync(0xffffffffu, rid, j);
				if (j < ntok && n < item.n_valid) {
					if (RAW) {
						y[(size_t)(item.row0 + n) * out_stride + (size_t)item.mat_sel * rows_per_matrix + mrow] = acc[j];
					} else if (PEER) {
						dst.y[(unsigned)rj >> 24][(size_t)(rj & 0xFFFFFF) * out_stride + mrow] = acc[j] * out_scale;
					} else {
						float *yp = y + (size_t)rj * out_stride + mrow;
						*yp = accumulate ? __fadd_rn(*yp, acc[j] * out_scale) : acc[j] * out_scale;
					}
				}
			}
			TCT_ADD(2, tst);
		}
		TCT_ADD(3, tct_start);
		if (warp == TC_PWARPS && lane == 0)
			TCT_FLUSH(8, 4);
	} else if (warp < W_TOK) {
		// ================= MMA issuers =================
		// Issuer w owns the phases with g % 2 == w (accumulator buffers w and w + 2); MMAs of the two
		// issuers run concurrently on different buffers.  The whole warp walks the loop (warp-uniform
		// addresses and descriptors); lane 0 issues.
		const uint32_t mw = warp - W_MMA0;
		// (pairs: the MMAs of both CTAs are issued by the even-ranked one; its peer's issuer warps idle)
		// (one issuer alternating between two accumulator buffers was measured slower than two issuers with
		// one buffer each: the ring round trips of a single consumer are exposed)
		const uint32_t leader = (lane == 0 && rank == 0) ? 1u : 0u;
		const bool issuing = rank == 0;
		auto mma = [&](uint32_t d, uint32_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
			if (PAIR)
				ptx::mma_f16_ts_pair_if(d, a, b, idesc, accumulate, leader);
			else
				ptx::mma_f16_ts_if(d, a, b, idesc, accumulate, leader);
		};
		auto commit = [&](uint64_t *bar) {
			if (PAIR)
				ptx::mma_commit_pair_if(ptx::smem_u32(bar), leader);
			else
				ptx::mma_commit_if(ptx::smem_u32(bar), leader);
		};
		int s = 0;
		uint32_t ph = 0, g = 0, tl = 0, gst = 0;
		uint32_t bg = 0;  // pairs: super-blocks so far (the token ring holds four of them)
		bool alive = true;
		TCT_DECL(8);
		const long long tct_start = TCT_NOW();
		auto advance = [&](int n) {
			gst += n;
			s += n;
			if (s >= TC_S) {
				s -= TC_S;
				ph ^= 1u;
			}
		};
		for (int t = walker; t < total && alive && issuing; t += stride_t, tl++) {
			const long long tth = TCT_NOW();
			const TcItem item = tc_item<PAIR>(t, (int)tl, s_items, m_items, tile_info, rows_per_matrix, rank);
			// up to 32 tokens: hi and lo rows are one N = 2 n_box operand (one MMA per k step);
			// more: two MMAs of N = n_mma on the hi rows and on the lo rows behind them.
			// Pairs: always one MMA, the hi rows from the leader's shared memory and the lo rows from its peer's.
			const bool concat = PAIR || item.n_box <= 32;
			const uint32_t idesc = ptx::umma_idesc_f16(PAIR ? 2 * TC_BM : TC_BM, concat ? 2 * item.n_box : item.n_mma);
			// min phase, second product: the hi sums only (a pair cannot address one CTA's half: it takes
			// both, which adds the negligible lo x lo term)
			const uint32_t idesc_hi = PAIR ? idesc : ptx::umma_idesc_f16(TC_BM, concat ? item.n_box : item.n_mma);
			const uint32_t lo_off = (uint32_t)item.n_box * 128u;
			TCT_ADD(6, tth + (long long)(lo_off & 0u));
			for (int sbi = 0; sbi < (Q4 ? nb + 1 : nb) && alive; sbi++) {
				const uint32_t buf = g & (NBUF - 1);
				const bool min_phase = Q4 && sbi == nb;
				const int n_st = min_phase ? 2 : TC_SPB;
				if ((g & 1u) != mw) {  // the other issuer's phase: skip its stages
					advance(n_st);
					g++;
					if (!min_phase)
						bg++;
					continue;
				}
				const long long tpe = TCT_NOW();
				if (g >= (uint32_t)NBUF) {
					const bool ok = tc_wait(ptx::smem_u32(&sh->pempty[buf]), ((g / NBUF) & 1u) ^ 1u, abort_flag, status);
					if (!__all_sync(0xffffffffu, ok)) {
						alive = false;
						break;
					}
				}
				TCT_ADD(0, tpe);
				const uint32_t dP = tmem + TC_COL_P + PW * buf;
				if (min_phase) {
					// ---- min phase: D = A_hi.[X_hi | X_lo] + A_lo.X_hi over the sub-block sums ----
					const long long tmp0 = TCT_NOW();
					const int s0 = s;
					const uint32_t ph0 = ph;
					advance(1);
					const int s1 = s;
					const uint32_t ph1 = ph;
					advance(1);
					bool ok = tc_wait(ptx::smem_u32(&sh->full[s0]), ph0, abort_flag, status);
					ok = ok && tc_wait(ptx::smem_u32(&sh->full[s1]), ph1, abort_flag, status);
					ok = ok && tc_wait(ptx::smem_u32(&sh->xfull), tl & 1u, abort_flag, status);
					if (!__all_sync(0xffffffffu, ok)) {
						alive = false;
						break;
					}
					ptx::tc_fence_after();
					TCT_ADD(5, tmp0);
					TCT_TRACE(2, gst - 2);
					TCT_TRACE(2, gst - 1);
					const uint64_t xh = ptx::umma_desc_sw128(xq_hi), xl = ptx::umma_desc_sw128(xq_hi + lo_off);
					const uint32_t ah = tmem + TC_COL_A + 32u * s0, al = tmem + TC_COL_A + 32u * s1;
					for (int kk = 0; kk < min_k16; kk++) {
						mma(dP, ah + 8 * kk, xh + 2 * kk, idesc, kk > 0 ? 1u : 0u);
						if (!concat)
							mma(dP, ah + 8 * kk, xl + 2 * kk, idesc, 1u);
						mma(dP, al + 8 * kk, xh + 2 * kk, idesc_hi, 1u);
					}
					commit(&sh->empty[s1]);	 // both stages (a commit costs an MMA's issue time)
					commit(&sh->xempty);
					commit(&sh->pfull[buf]);
					TCT_TRACE(3, gst - 2);
					TCT_TRACE(3, gst - 1);
					TCT_ADD(7, tmp0);
					g++;
					continue;
				}
				for (int q4 = 0; q4 < TC_SPB; q4++) {
					const long long tb = TCT_NOW();
					// the token stage: the ring slot itself, or (pairs) slot q4 of the super-block's group in the token ring
					const int bs = PAIR ? (int)(bg & 3u) * TC_SPB + q4 : s;
					const uint32_t bph = PAIR ? (bg >> 2) & 1u : ph;
					// both tests issued back to back; the bounded waits only when one of them fails
					const bool okb = ptx::mbar_try_wait(ptx::smem_u32(&sh->bfull[bs]), bph);
					const bool okf = ptx::mbar_try_wait(ptx::smem_u32(&sh->full[s]), ph);
					bool ok = true;
					if (!okb)
						ok = tc_wait(ptx::smem_u32(&sh->bfull[bs]), bph, abort_flag, status);
					TCT_ADD(1, tb);
					const long long tf = TCT_NOW();
					if (ok && !okf)
						ok = tc_wait(ptx::smem_u32(&sh->full[s]), ph, abort_flag, status);
					if (!__all_sync(0xffffffffu, ok)) {
						alive = false;
						break;
					}
					TCT_ADD(2, tf);
					TCT_TRACE(2, gst);
					const long long ti = TCT_NOW();
					ptx::tc_fence_after();
					const uint64_t bh = ptx::umma_desc_sw128(b_hi(bs)), bl = ptx::umma_desc_sw128(b_hi(bs) + lo_off);
					const uint32_t a = tmem + TC_COL_A + 32u * s;
#pragma unroll
					for (int kk = 0; kk < TC_BK / 16; kk++) {
						mma(dP, a + 8 * kk, bh + 2 * kk, idesc, (q4 > 0 || kk > 0) ? 1u : 0u);
						if (!concat)
							mma(dP, a + 8 * kk, bl + 2 * kk, idesc, 1u);
					}
					if (q4 & 1)  // stages go back to the producers and the token loader in pairs
						commit(&sh->empty[s]);
					TCT_ADD(3, ti);
					TCT_TRACE(3, gst);
					advance(1);
				}
				if (!alive)
					break;
				if (PAIR)  // the super-block's token stages go back to both CTAs' token loaders
					commit(&sh->bempty[bg & 3u]);
				commit(&sh->pfull[buf]);
				g++;
				bg++;
			}
		}
		TCT_ADD(4, tct_start);
		if (lane == 0 && mw == 0)
			TCT_FLUSH(16, 8);
	} else if (warp == W_TOK) {
		// ================= token loader: token operand and sub-block sums (TMA) =================
		if (lane == 0) {
			int s = 0;
			uint32_t ph = 0, it = 0, tl = 0;
			uint32_t bgl = 0;  // pairs: super-blocks fetched so far
			bool alive = true;
			TCT_DECL(3);
			const long long tct_start = TCT_NOW();
			for (int t = walker; t < total && alive; t += stride_t, tl++) {
				const TcItem item = tc_item<PAIR>(t, (int)tl, s_items, m_items, tile_info, rows_per_matrix, rank);
				// hi + lo rows of one 64-k box.  A pair splits them: the leader fetches the hi rows, its peer the
				// lo rows (the same box of the operand's other half), each into its own shared memory; all the
				// bytes are counted on the leader's barrier, whose token loader announces them.
				const uint32_t box_bytes = 2u * (uint32_t)item.n_box * 128u;
				const CUtensorMap *tmp = item.n_box == 16 ? &tm16 : (item.n_box == 32 ? &tm32 : &tm64);
				// the sub-block sums of the work item (Q4_K) are fetched once the first super-block's tiles are on
				// their way (the previous work item's min phase is long over then)
				auto fetch_sums = [&]() -> bool {
					if (tl >= 1u && !tc_wait(ptx::smem_u32(&sh->xempty), (tl & 1u) ^ 1u, abort_flag, status))
						return false;
					const uint32_t xb = ptx::smem_u32(&sh->xfull);
					const CUtensorMap *tqp = item.n_box == 16 ? &tq16 : (item.n_box == 32 ? &tq32 : &tq64);
					if (PAIR) {
						if (rank == 0)
							ptx::mbar_arrive_expect_tx(xb, box_bytes);
						ptx::tma_load_3d_pair(xq_hi, tqp, xb, sb0 * 8, item.row0, (int)rank);
					} else {
						ptx::mbar_arrive_expect_tx(xb, box_bytes);
						ptx::tma_load_3d(xq_hi, tqp, xb, sb0 * 8, item.row0, 0);
					}
					return true;
				};
				if (PAIR) {
					// the token ring of a pair: groups of four stages (one super-block), handed back per group
					for (int sbi = 0; sbi < nb && alive; sbi++) {
						if (Q4 && sbi == (nb > 1 ? 1 : 0) && !fetch_sums()) {
							alive = false;
							break;
						}
						const uint32_t q = bgl & 3u;
						const long long tw = TCT_NOW();
						if (bgl >= 4u && !tc_wait<100>(ptx::smem_u32(&sh->bempty[q]), ((bgl >> 2) & 1u) ^ 1u, abort_flag, status)) {
							alive = false;
							break;
						}
						TCT_ADD(0, tw);
						const long long ti = TCT_NOW();
						for (int q4 = 0; q4 < TC_SPB; q4++) {
							const int bs = (int)q * TC_SPB + q4;
							const uint32_t fb = ptx::smem_u32(&sh->bfull[bs]);
							if (rank == 0)
								ptx::mbar_arrive_expect_tx(fb, box_bytes);
							ptx::tma_load_3d_pair(b_hi(bs), tmp, fb, ((sb0 + sbi) * TC_SPB + q4) * TC_BK, item.row0, (int)rank);
						}
						TCT_ADD(1, ti);
						bgl++;
					}
				} else {
				// the two stages of the min phase (after the super-blocks) carry no token tiles: they only
				// keep the barrier phases in step
				for (int ki = 0; ki < k_iters + (Q4 ? 2 : 0); ki++) {
					if (Q4 && ki == (k_iters > TC_SPB ? TC_SPB : 0) && !fetch_sums()) {
						alive = false;
						break;
					}
					const long long tw = TCT_NOW();
					if (it >= (uint32_t)TC_S && !tc_wait<100>(ptx::smem_u32(&sh->empty[s | 1]), ph ^ 1u, abort_flag, status)) {
						alive = false;
						break;
					}
					TCT_ADD(0, tw);
					const long long ti = TCT_NOW();
					const uint32_t fb = ptx::smem_u32(&sh->bfull[s]);
					if (ki >= k_iters) {
						ptx::mbar_arrive(fb);
					} else {
						// one box: 64 k x n_box rows x (hi, lo); a thread can issue a TMA only every ~100 cycles
						ptx::mbar_arrive_expect_tx(fb, box_bytes);
						ptx::tma_load_3d(b_hi(s), tmp, fb, (sb0 * TC_SPB + ki) * TC_BK, item.row0, 0);
					}
					TCT_ADD(1, ti);
					it++;
					if (++s == TC_S) {
						s = 0;
						ph ^= 1u;
					}
				}
				}
			}
			TCT_ADD(2, tct_start);
			TCT_FLUSH(24, 3);
		}
	} else {
		// ================= weight loader: packed super-blocks -> shared memory =================
		int wb = 0;
		uint32_t wph = 0, wc = 0;
		bool alive = true;
		int wtl = 0;
		for (int t = walker; t < total && alive; t += stride_t, wtl++) {
			const TcItem item = tc_item<PAIR>(t, wtl, s_items, m_items, tile_info, rows_per_matrix, rank);
			for (int sbi = 0; sbi < nb; sbi++) {
				if (wc >= (uint32_t)Sm::NWB && !tc_wait_warp<100>(ptx::smem_u32(&sh->wempty[wb]), wph ^ 1u, abort_flag, status, lane)) {
					alive = false;
					break;
				}
				const uint32_t bar = ptx::smem_u32(&sh->wfull[wb]);
				if (lane == 0) {
					ptx::mbar_arrive_expect_tx(bar, Sm::WBUF);
					if (Q4)	 // box = (one block, 128 rows)
						ptx::tma_load_2d(w_buf(wb), item.mat_sel ? &tw1 : &tw0, bar, (sb0 + sbi) * Q4K_BYTES,
								 item.le * rows_per_matrix + item.m0);
					else  // box = (one record, 8 rows of a group, 16 groups)
						ptx::tma_load_3d(w_buf(wb), item.mat_sel ? &tw1 : &tw0, bar, (sb0 + sbi) * TC_Q6_ROW, 0,
								 (item.le * rows_per_matrix + item.m0) >> 3);
				}
				wc++;
				if (++wb == Sm::NWB) {
					wb = 0;
					wph ^= 1u;
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
	if (PAIR)
		ptx::cluster_sync_all();  // neither CTA leaves while its peer may still signal its barriers or read its memories
	if (warp == W_MMA0) {
		if (PAIR)
			ptx::tmem_dealloc_pair(tmem, TC_TMEM_COLS);
		else
			ptx::tmem_dealloc(tmem, TC_TMEM_COLS);
	}
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

static int encode_2d(tie_cuda_ctx *c, CUtensorMap *tm, CUtensorMapDataType type, size_t elem, void *base, size_t rows, size_t cols,
		     unsigned box_cols, unsigned box_rows, CUtensorMapSwizzle swz)
{
	PFN_encodeTiled enc = get_encode_fn();
	if (!enc) {
		snprintf(c->cuda_err, sizeof(c->cuda_err), "cuTensorMapEncodeTiled entry point not found");
		return TIE_CUDA_ECUDA;
	}
	cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
	cuuint64_t strides[1] = {(cuuint64_t)cols * elem};
	cuuint32_t box[2] = {box_cols, box_rows};
	cuuint32_t estr[2] = {1, 1};
	CUresult r = enc(tm, type, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
			 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
	if (r != CUDA_SUCCESS) {
		snprintf(c->cuda_err, sizeof(c->cuda_err), "cuTensorMapEncodeTiled failed: %d", (int)r);
		return TIE_CUDA_ECUDA;
	}
	return TIE_CUDA_OK;
}

// Split fp16 operand [hi | lo][rows][cols] (lo array right behind hi), box = 64 columns x box_rows
// rows x 2, 128-byte swizzle: hi rows land first in shared memory, the lo rows directly behind.
// depth 2: one box brings the hi rows and the lo rows; depth 1: the box is one half (a CTA of a
// pair fetches the half its rank names with the third coordinate).
static int make_tmap(tie_cuda_ctx *c, CUtensorMap *tm, void *base, size_t rows, size_t cols, unsigned box_rows, unsigned depth = 2)
{
	PFN_encodeTiled enc = get_encode_fn();
	if (!enc) {
		snprintf(c->cuda_err, sizeof(c->cuda_err), "cuTensorMapEncodeTiled entry point not found");
		return TIE_CUDA_ECUDA;
	}
	cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, 2};
	cuuint64_t strides[2] = {(cuuint64_t)cols * 2, (cuuint64_t)rows * cols * 2};
	cuuint32_t box[3] = {(cuuint32_t)TC_BK, box_rows, depth};
	cuuint32_t estr[3] = {1, 1, 1};
	CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
			 CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
	if (r != CUDA_SUCCESS) {
		snprintf(c->cuda_err, sizeof(c->cuda_err), "cuTensorMapEncodeTiled (token operand) failed: %d", (int)r);
		return TIE_CUDA_ECUDA;
	}
	return TIE_CUDA_OK;
}

// Byte map of an expert tensor for the weight loader.  Q4_K: [experts x rows][row bytes], box = one
// 144-byte block x 128 rows.  Q6_K: [groups][8 rows][row records], box = one 208-byte record x 8 x 16.
int tc_make_weight_map(tie_cuda_ctx *c, DevTensor &t, int n_experts)
{
	if (n_experts <= 0)
		n_experts = c->n_local;
	t.has_map = false;
	if (t.rows % TC_BM || t.k % QK_K)
		return TIE_CUDA_OK;
	const int nb = t.k / QK_K;
	if (t.kind == W_Q4K) {
		int rc = encode_2d(c, &t.map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, t.ptr, (size_t)t.rows * n_experts, (size_t)nb * Q4K_BYTES,
				   Q4K_BYTES, TC_BM, CU_TENSOR_MAP_SWIZZLE_NONE);
		if (rc)
			return rc;
	} else {
		PFN_encodeTiled enc = get_encode_fn();
		if (!enc) {
			snprintf(c->cuda_err, sizeof(c->cuda_err), "cuTensorMapEncodeTiled entry point not found");
			return TIE_CUDA_ECUDA;
		}
		cuuint64_t dims[3] = {(cuuint64_t)nb * Q6K_RECORD, 8, (cuuint64_t)t.rows * n_experts / 8};
		cuuint64_t strides[2] = {(cuuint64_t)nb * Q6K_RECORD, (cuuint64_t)q6k_r8_group_bytes(nb)};
		cuuint32_t box[3] = {Q6K_RECORD, 8, TC_BM / 8};
		cuuint32_t estr[3] = {1, 1, 1};
		CUresult r = enc(&t.map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, t.ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
				 CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
		if (r != CUDA_SUCCESS) {
			snprintf(c->cuda_err, sizeof(c->cuda_err), "cuTensorMapEncodeTiled (Q6_K weights) failed: %d", (int)r);
			return TIE_CUDA_ECUDA;
		}
	}
	t.has_map = true;
	return TIE_CUDA_OK;
}

int tc_setup(tie_cuda_ctx *c)
{
	Scratch &s = c->s;
	const size_t H = c->cfg.hidden, F = c->cfg.ffn_dim;
	// tmap[array * 3 + box]: array 0 = x, 1 = h, 2 = sums of x, 3 = sums of h; box rows 16, 32, 64
	void *bases[4] = {s.xs_hi, s.hs_hi, s.xq_hi, s.hq_hi};
	size_t cols[4] = {H, F, (size_t)xq_cols((int)H), (size_t)xq_cols((int)F)};
	for (int a = 0; a < 4; a++)
		for (int b = 0; b < 3; b++) {
			int rc = make_tmap(c, &c->tmap[a * 3 + b], bases[a], s.rows_pad, cols[a], 16u << b);
			if (!rc)
				rc = make_tmap(c, &c->tmap_half[a * 3 + b], bases[a], s.rows_pad, cols[a], 16u << b, 1);
			if (rc)
				return rc;
		}
#define TC_ATTR(KIND, RAW) \
	TIE_CUDA_TRY(c, cudaFuncSetAttribute(grouped_gemm_sb<KIND, RAW>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcSmem<KIND>::SMEM))
	TC_ATTR(W_Q4K, false);
	TC_ATTR(W_Q4K, true);
	TC_ATTR(W_Q6K_R8, false);
	TC_ATTR(W_Q6K_R8, true);
#undef TC_ATTR
	TIE_CUDA_TRY(c, cudaFuncSetAttribute(grouped_gemm_sb<W_Q4K, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
					     TcSmem<W_Q4K>::SMEM));
	TIE_CUDA_TRY(c, cudaFuncSetAttribute(grouped_gemm_sb<W_Q6K_R8, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
					     TcSmem<W_Q6K_R8>::SMEM));
	// the CTA-pair forms; how many pairs the device holds at once sizes their (persistent) grids
#define TC_ATTR_PAIR(KIND, RAW, PEER)                                                                                          \
	TIE_CUDA_TRY(c, cudaFuncSetAttribute(grouped_gemm_sb<KIND, RAW, PEER, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
					     TcSmem<KIND>::SMEM));                                                             \
	TIE_CUDA_TRY(c, cudaFuncSetAttribute(grouped_gemm_sb<KIND, RAW, PEER, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 0))
	TC_ATTR_PAIR(W_Q4K, false, false);
	TC_ATTR_PAIR(W_Q4K, true, false);
	TC_ATTR_PAIR(W_Q4K, false, true);
	TC_ATTR_PAIR(W_Q6K_R8, false, false);
	TC_ATTR_PAIR(W_Q6K_R8, true, false);
	TC_ATTR_PAIR(W_Q6K_R8, false, true);
#undef TC_ATTR_PAIR
	{
		cudaLaunchConfig_t cfg = {};
		cfg.gridDim = dim3(c->sm_count & ~1);
		cfg.blockDim = dim3(TC_THREADS);
		cfg.dynamicSmemBytes = TcSmem<W_Q4K>::SMEM;
		cudaLaunchAttribute attr[1];
		attr[0].id = cudaLaunchAttributeClusterDimension;
		attr[0].val.clusterDim.x = 2;
		attr[0].val.clusterDim.y = 1;
		attr[0].val.clusterDim.z = 1;
		cfg.attrs = attr;
		cfg.numAttrs = 1;
		int n_clusters = 0;
		if (cudaOccupancyMaxActiveClusters(&n_clusters, grouped_gemm_sb<W_Q4K, true, false, true>, &cfg) != cudaSuccess) {
			cudaGetLastError();
			n_clusters = 0;
		}
		c->tc_pairs = n_clusters < c->sm_count / 2 ? n_clusters : c->sm_count / 2;
	}
	c->tmaps_ok = true;
	return TIE_CUDA_OK;
}

// arr: 0 = the split inputs x (gate/up), 1 = the split activations h (down).
template <WKind KIND, bool RAW, bool PEER = false>
static int launch_tc_t(tie_cuda_ctx *c, const DevTensor &t0, const DevTensor *t1, int arr, float *y, float out_scale,
		       bool sorted_out = false, const EpDst *dst = nullptr, int n_experts = -1, const DenseView *view = nullptr,
		       int sb0 = 0, int n_sb = 0, int accumulate = 0)
{
	Scratch &s = c->s;
	if (n_experts <= 0)
		n_experts = c->n_local;
	const int m_tiles = (RAW ? 2 : 1) * t0.rows / TC_BM;
	const CUtensorMap &w0m = t0.map;
	const CUtensorMap &w1m = t1 ? t1->map : t0.map;
	const uint8_t *w1p = t1 ? t1->ptr : nullptr;
	const int *perm = sorted_out ? nullptr : s.perm;
	const int out_stride = RAW ? 2 * t0.rows : t0.rows;
	const EpDst d = dst ? *dst : EpDst();
	const int nb_total = t0.k / QK_K;
	const int k_dim = (n_sb > 0 ? n_sb : nb_total) * QK_K;
	// a dense tensor brings the maps of its own view of the operand scratch (entries 0-2 operand, 3-5 sums)
	const CUtensorMap *mh = view ? view->half : c->tmap_half + arr * 3, *mhq = view ? view->half + 3 : c->tmap_half + (2 + arr) * 3;
	const CUtensorMap *mf = view ? view->full : c->tmap + arr * 3, *mfq = view ? view->full + 3 : c->tmap + (2 + arr) * 3;
	// pairs of CTAs (one MMA issue for two 128-row tiles) where the 128-row tiles pair up
	// (measured at 64, 512 and 4096 tokens: pairs win on rows of 8 super-blocks — gate/up, 15 % faster —
	// and lose on rows of 3 — down, 7 % slower: with few super-blocks per work item the pair's
	// hand-offs between two SMs are not amortised)
	if (c->tc_pairs > 0 && !c->tc_no_pair && m_tiles % 2 == 0 && k_dim >= 4 * QK_K) {
		cudaLaunchConfig_t cfg = {};
		cfg.gridDim = dim3(2 * c->tc_pairs);
		cfg.blockDim = dim3(TC_THREADS);
		cfg.dynamicSmemBytes = TcSmem<KIND>::SMEM;
		cfg.stream = c->stream;
		cudaLaunchAttribute attr[1];
		attr[0].id = cudaLaunchAttributeClusterDimension;
		attr[0].val.clusterDim.x = 2;
		attr[0].val.clusterDim.y = 1;
		attr[0].val.clusterDim.z = 1;
		cfg.attrs = attr;
		cfg.numAttrs = 1;
		TIE_CUDA_TRY(c, cudaLaunchKernelEx(&cfg, grouped_gemm_sb<KIND, RAW, PEER, true>, mh[0], mh[1], mh[2], mhq[0], mhq[1], mhq[2], w0m, w1m,
						   (const uint8_t *)t0.ptr, w1p, t0.expert_stride, k_dim, (const int4 *)s.tile_info,
						   (const int *)s.tile_start, n_experts, m_tiles, y, perm, out_stride, out_scale, s.status, t0.rows, d,
						   sb0, nb_total, accumulate));
		c->launches++;
		return TIE_CUDA_OK;
	}
	grouped_gemm_sb<KIND, RAW, PEER><<<c->sm_count, TC_THREADS, TcSmem<KIND>::SMEM, c->stream>>>(
		mf[0], mf[1], mf[2], mfq[0], mfq[1], mfq[2], w0m, w1m, t0.ptr, w1p, t0.expert_stride, k_dim, s.tile_info, s.tile_start, n_experts,
		m_tiles, y, perm, out_stride, out_scale, s.status, t0.rows, d, sb0, nb_total, accumulate);
	TIE_CUDA_LAUNCHED(c);
	return TIE_CUDA_OK;
}

static bool tc_tensor_ok(const DevTensor &t)
{
	// Q4_K needs all sub-block sums of a row in one 64-wide tile (k <= 2048)
	return t.has_map && t.rows % TC_BM == 0 && t.k % QK_K == 0 && (t.kind != W_Q4K || t.k <= 2048);
}

bool tc_supported(const tie_cuda_ctx *c, const Layer &L)
{
	return c->tmaps_ok && L.gate.kind == L.up.kind && tc_tensor_ok(L.gate) && tc_tensor_ok(L.up) && tc_tensor_ok(L.down);
}

// xs_hi/xs_lo (and xq_hi/xq_lo for Q4_K) must hold the split inputs in sorted order; the sort must
// have been run with TC_TOKEN_TILE.  Gate and up run as independent 128-row tiles; the raw fp32
// products go to the scratch s.y as [row][gate | up].
int launch_tc_gate_up(tie_cuda_ctx *c, const Layer &L, int n_rows)
{
	(void)n_rows;
	return (L.gate.kind == W_Q4K) ? launch_tc_t<W_Q4K, true>(c, L.gate, &L.up, 0, c->s.y, 1.0f)
				      : launch_tc_t<W_Q6K_R8, true>(c, L.gate, &L.up, 0, c->s.y, 1.0f);
}

// Element-wise SwiGLU of the raw gate | up products, scaled and split into hs_hi/hs_lo (and
// hq_hi/hq_lo when the down matrix is Q4_K).
int launch_tc_swiglu(tie_cuda_ctx *c, const Layer &L, int n_rows, const int *n_rows_dev)
{
	const bool sums = L.down.kind == W_Q4K;
	return launch_swiglu_split(c, c->s.y, n_rows, L.gate.rows, TC_H_SCALE, c->s.hs_hi, c->s.hs_lo, sums ? c->s.hq_hi : nullptr,
				   sums ? c->s.hq_lo : nullptr, n_rows_dev);
}

// reads hs_hi/hs_lo; writes y[perm[p]] (sorted_out: y[p]).
int launch_tc_down(tie_cuda_ctx *c, const Layer &L, int n_rows, float *y, bool sorted_out)
{
	(void)n_rows;
	if (L.down.kind == W_Q4K)
		return launch_tc_t<W_Q4K, false>(c, L.down, nullptr, 1, y, 1.0f / TC_H_SCALE, sorted_out);
	return launch_tc_t<W_Q6K_R8, false>(c, L.down, nullptr, 1, y, 1.0f / TC_H_SCALE, sorted_out);
}

// A dense tensor (one "expert") on the grouped product: y[p][row] = sum_k w[row][k] x[p][k].  The
// split operand of the batch lives in the context's x arrays, VIEWED with the tensor's own row
// length k (any multiple of 256): hi rows at the array's start, lo rows rows_view * k behind, the
// sub-block sums likewise in the sums array; the tensor carries the tensor maps of that view.
bool tc_dense_supported(const tie_cuda_ctx *c, const DevTensor &t)
{
	return c->tmaps_ok && t.has_map && t.view && t.rows % TC_BM == 0 && t.k % QK_K == 0;
}

int tc_make_dense_view(tie_cuda_ctx *c, DevTensor &t)
{
	Scratch &s = c->s;
	const size_t H = c->cfg.hidden, K = t.k, XH = xq_cols((int)H), XK = xq_cols((int)K);
	DenseView *v = new (std::nothrow) DenseView();
	if (!v)
		return TIE_CUDA_ENOMEM;
	const size_t rows_x = s.rows_pad * H / K, rows_q = s.rows_pad * XH / XK;
	v->rows = rows_x < rows_q ? rows_x : rows_q;
	v->lo_off = v->rows * K;
	v->q_lo_off = v->rows * XK;
	for (int b = 0; b < 3 && v->rows >= 64; b++) {
		int rc = make_tmap(c, &v->full[b], s.xs_hi, v->rows, K, 16u << b);
		if (!rc)
			rc = make_tmap(c, &v->half[b], s.xs_hi, v->rows, K, 16u << b, 1);
		if (!rc)
			rc = make_tmap(c, &v->full[3 + b], s.xq_hi, v->rows, XK, 16u << b);
		if (!rc)
			rc = make_tmap(c, &v->half[3 + b], s.xq_hi, v->rows, XK, 16u << b, 1);
		if (rc) {
			delete v;
			return rc;
		}
	}
	if (v->rows < 64) {  // the scratch of this context cannot hold a single tile of such rows
		delete v;
		return TIE_CUDA_OK;
	}
	t.view = v;
	return TIE_CUDA_OK;
}

int launch_tc_dense(tie_cuda_ctx *c, const DevTensor &t, float *y)
{
	const int nb = t.k / QK_K;
	// Q4_K: at most 8 super-blocks (64 sub-block sums) per launch; later launches add to y
	const int step = t.kind == W_Q4K ? 8 : nb;
	for (int sb0 = 0; sb0 < nb; sb0 += step) {
		const int n_sb = nb - sb0 < step ? nb - sb0 : step;
		int rc = t.kind == W_Q4K ? launch_tc_t<W_Q4K, false>(c, t, nullptr, 0, y, 1.0f, true, nullptr, 1, t.view, sb0, n_sb, sb0 > 0)
					 : launch_tc_t<W_Q6K_R8, false>(c, t, nullptr, 0, y, 1.0f, true, nullptr, 1, t.view, sb0, n_sb, sb0 > 0);
		if (rc)
			return rc;
	}
	return TIE_CUDA_OK;
}

// The down product of an expert-parallel step: row p goes to the rank and row dst->row[p] names.
int launch_tc_down_peer(tie_cuda_ctx *c, const Layer &L, const EpDst &dst)
{
	if (L.down.kind == W_Q4K)
		return launch_tc_t<W_Q4K, false, true>(c, L.down, nullptr, 1, nullptr, 1.0f / TC_H_SCALE, true, &dst);
	return launch_tc_t<W_Q6K_R8, false, true>(c, L.down, nullptr, 1, nullptr, 1.0f / TC_H_SCALE, true, &dst);
}

}  // namespace tie
