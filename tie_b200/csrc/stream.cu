// Streaming expert kernels for decode and small batches: grouped mat-vecs over packed
// Q4_K / Q6_K super-blocks, dequantised in registers, reduced with warp shuffles.
//
// Reference: process_expert_task (engine.c:916-964): gate and up mat-vecs
// (mat_vec_row_f32_q4k_f32_avx2 / dot_product_f32_q4k_avx2, math_avx2.c:753-769, 535-604),
// SwiGLU through the SiLU table (math_avx2.c:908-950), down mat-vec
// (mat_vec_row_f32_q6k_f32_avx2 / dot_product_f32_q6k_avx2, math_avx2.c:771-787, 411-495).
//
// Work split: a CTA owns (expert slot, tile of output rows); a lane owns a fixed 64-wide slice
// of the input dimension ("part"), keeps that slice of the activation in registers, and walks
// the CTA's rows streaming 48 bytes of packed weights per row with 128-bit loads.  The block
// algebra is factored so that integer quants meet the activation first and the block scales
// are applied once per part:
//   Q4_K:  sum_j x_j (d*sc*q_j - dmin*m) = (d*sc) * sum_j q_j x_j - (dmin*m) * sum_j x_j
//   Q6_K:  sum_j (d*sc) (q_j-32) x_j     = (d*sc) * sum_j (q_j-32) x_j
// (same value as the reference's per-element form up to fp32 rounding; accumulation is fp32).
#include "common.cuh"
#include "kernels.cuh"

namespace tie {

constexpr int STREAM_THREADS = 256;

// Exact small-integer -> float without the conversion pipe: place the byte in the low mantissa
// bits of 2^23 and subtract 2^23 (+ offset).
__device__ __forceinline__ float byte_to_float(uint32_t word, int k, float bias)
{
	uint32_t bits = __byte_perm(word, 0x4B000000u, 0x7650 | k);
	return __fsub_rn(__uint_as_float(bits), bias);
}

template <WKind KIND>
struct PartDot;

// ---- Q4_K: part = (block b, quarter p): qs[32p .. 32p+32), low nibbles = sub-block 2p
//      (elements 64p+i), high nibbles = sub-block 2p+1 (elements 64p+32+i) — math_scalar.c:216-255.
template <>
struct PartDot<W_Q4K> {
	// xr[0..63] = x[64*part .. 64*part+63]; sx[0] = sum xr[0..31], sx[1] = sum xr[32..63]
	__device__ static __forceinline__ void load_x(const float *xrow, int part, float xr[64], float sx[4])
	{
		const float4 *p = reinterpret_cast<const float4 *>(xrow + 64 * part);
		float s0 = 0.f, s1 = 0.f;
#pragma unroll
		for (int i = 0; i < 16; i++) {
			float4 v = p[i];
			xr[4 * i] = v.x;
			xr[4 * i + 1] = v.y;
			xr[4 * i + 2] = v.z;
			xr[4 * i + 3] = v.w;
			float t = (v.x + v.y) + (v.z + v.w);
			if (i < 8)
				s0 += t;
			else
				s1 += t;
		}
		sx[0] = s0;
		sx[1] = s1;
		sx[2] = sx[3] = 0.f;
	}
	struct Raw {
		uint4 hdr, q0, q1;
	};
	__device__ static __forceinline__ Raw load(const uint8_t *wexp, int nb, int row, int part)
	{
		const uint8_t *blk = wexp + ((size_t)row * nb + (part >> 2)) * Q4K_BYTES;
		Raw r;
		r.hdr = __ldg(reinterpret_cast<const uint4 *>(blk));
		const uint4 *q = reinterpret_cast<const uint4 *>(blk + 16 + 32 * (part & 3));
		r.q0 = __ldg(q);
		r.q1 = __ldg(q + 1);
		return r;
	}
	__device__ static __forceinline__ float dot(const Raw &r, int part, const float xr[64], const float sx[4])
	{
		const int p = part & 3;
		const float d = half_bits_to_float(r.hdr.x & 0xffffu);
		const float dmin = half_bits_to_float(r.hdr.x >> 16);
		const uint32_t sc[3] = {r.hdr.y, r.hdr.z, r.hdr.w};
		int s_lo, m_lo, s_hi, m_hi;
		q4k_scale_min(sc, 2 * p, s_lo, m_lo);
		q4k_scale_min(sc, 2 * p + 1, s_hi, m_hi);
		const uint32_t w[8] = {r.q0.x, r.q0.y, r.q0.z, r.q0.w, r.q1.x, r.q1.y, r.q1.z, r.q1.w};
		float al = 0.f, ah = 0.f;
#pragma unroll
		for (int k = 0; k < 8; k++) {
			uint32_t lo = w[k] & 0x0F0F0F0Fu, hi = (w[k] >> 4) & 0x0F0F0F0Fu;
#pragma unroll
			for (int j = 0; j < 4; j++) {
				al = __fmaf_rn(byte_to_float(lo, j, 8388608.0f), xr[4 * k + j], al);
				ah = __fmaf_rn(byte_to_float(hi, j, 8388608.0f), xr[32 + 4 * k + j], ah);
			}
		}
		float res = __fmul_rn(d, (float)s_lo) * al - __fmul_rn(dmin, (float)m_lo) * sx[0];
		res += __fmul_rn(d, (float)s_hi) * ah - __fmul_rn(dmin, (float)m_hi) * sx[1];
		return res;
	}
};

// ---- Q6_K in the R8 layout: part = (block b, half n, slice l16); 16 l's x 4 positions
//      (l, l+32, l+64, l+96 within the half) — math_scalar.c:257-287.
template <>
struct PartDot<W_Q6K_R8> {
	// xr[16*j + i] = x[256b + 128n + 16*l16 + 32*j + i]
	__device__ static __forceinline__ void load_x(const float *xrow, int part, float xr[64], float sx[4])
	{
		const int b = part >> 2, n = (part >> 1) & 1, l16 = part & 1;
		const float *base = xrow + 256 * b + 128 * n + 16 * l16;
#pragma unroll
		for (int j = 0; j < 4; j++) {
			const float4 *p = reinterpret_cast<const float4 *>(base + 32 * j);
#pragma unroll
			for (int i = 0; i < 4; i++) {
				float4 v = p[i];
				xr[16 * j + 4 * i] = v.x;
				xr[16 * j + 4 * i + 1] = v.y;
				xr[16 * j + 4 * i + 2] = v.z;
				xr[16 * j + 4 * i + 3] = v.w;
			}
		}
		sx[0] = sx[1] = sx[2] = sx[3] = 0.f;
	}
	struct Raw {
		uint4 a, b, h;
		uint32_t sc;
		float d;
	};
	__device__ static __forceinline__ Raw load(const uint8_t *wexp, int nb, int row, int part)
	{
		const uint8_t *grp = wexp + (size_t)(row >> 3) * q6k_r8_group_bytes(nb);
		const int r8 = row & 7, b = part >> 2, pp = part & 3;
		const uint4 *ch = reinterpret_cast<const uint4 *>(grp + q6k_r8_chunk_off(nb, r8, b, pp));
		Raw r;
		r.a = __ldg(ch);
		r.b = __ldg(ch + 1);
		r.h = __ldg(ch + 2);
		r.sc = __ldg(reinterpret_cast<const uint32_t *>(grp + q6k_r8_scale_off(nb, r8, b, pp)));
		r.d = half_bits_to_float(__ldg(reinterpret_cast<const unsigned short *>(grp + q6k_r8_d_off(nb, r8, b))));
		return r;
	}
	__device__ static __forceinline__ float dot(const Raw &r, int part, const float xr[64], const float sx[4])
	{
		const uint32_t A[4] = {r.a.x, r.a.y, r.a.z, r.a.w};
		const uint32_t B[4] = {r.b.x, r.b.y, r.b.z, r.b.w};
		const uint32_t Hh[4] = {r.h.x, r.h.y, r.h.z, r.h.w};
		float a1 = 0.f, a2 = 0.f, a3 = 0.f, a4 = 0.f;
		const float off = 8388608.0f + 32.0f;
#pragma unroll
		for (int k = 0; k < 4; k++) {
			uint32_t q1 = (A[k] & 0x0F0F0F0Fu) | ((Hh[k] << 4) & 0x30303030u);
			uint32_t q2 = (B[k] & 0x0F0F0F0Fu) | ((Hh[k] << 2) & 0x30303030u);
			uint32_t q3 = ((A[k] >> 4) & 0x0F0F0F0Fu) | (Hh[k] & 0x30303030u);
			uint32_t q4 = ((B[k] >> 4) & 0x0F0F0F0Fu) | ((Hh[k] >> 2) & 0x30303030u);
#pragma unroll
			for (int j = 0; j < 4; j++) {
				a1 = __fmaf_rn(byte_to_float(q1, j, off), xr[4 * k + j], a1);
				a2 = __fmaf_rn(byte_to_float(q2, j, off), xr[16 + 4 * k + j], a2);
				a3 = __fmaf_rn(byte_to_float(q3, j, off), xr[32 + 4 * k + j], a3);
				a4 = __fmaf_rn(byte_to_float(q4, j, off), xr[48 + 4 * k + j], a4);
			}
		}
		const float s1 = (float)(int)(signed char)(r.sc & 0xff), s2 = (float)(int)(signed char)((r.sc >> 8) & 0xff);
		const float s3 = (float)(int)(signed char)((r.sc >> 16) & 0xff), s4 = (float)(int)(signed char)(r.sc >> 24);
		return r.d * ((s1 * a1 + s2 * a2) + (s3 * a3 + s4 * a4));
	}
};

// K = input dim; NMAT = 2: gate+up with SwiGLU epilogue, NMAT = 1: plain mat-vec (down).
// LPR = lanes per row (power of two >= K/64); RPW = rows per warp pass.
template <WKind KIND, int K, int NMAT>
__global__ void __launch_bounds__(STREAM_THREADS, 1)
stream_rows(const uint8_t *__restrict__ w0, const uint8_t *__restrict__ w1, size_t expert_stride, int rows_per_expert,
	    int rows_per_tile, const float *__restrict__ xin, int in_by_perm, int src_div, float *__restrict__ yout,
	    int out_by_perm, int out_stride, const int *__restrict__ row_expert, const int *__restrict__ offsets,
	    const int *__restrict__ active, const int *__restrict__ n_active, const int *__restrict__ perm, int direct,
	    int first_expert, int n_local, const float *__restrict__ silu, unsigned *__restrict__ status)
{
	constexpr int PARTS = K / 64;
	constexpr int LPR = PARTS > 16 ? 32 : (PARTS > 8 ? 16 : (PARTS > 4 ? 8 : 4));
	constexpr int RPW = 32 / LPR;
	constexpr int NB = K / QK_K;
	__shared__ __align__(16) float xs[K];

	int le, p0, p1;
	if (direct) {
		le = row_expert[blockIdx.y] - first_expert;
		p0 = blockIdx.y;
		p1 = p0 + 1;
		if (le < 0 || le >= n_local) {
			if (threadIdx.x == 0 && blockIdx.x == 0)
				atomicOr(status, ST_BAD_EXPERT);
			return;
		}
	} else {
		if ((int)blockIdx.y >= *n_active)
			return;
		le = active[blockIdx.y];
		p0 = offsets[le];
		p1 = offsets[le + 1];
	}
	const uint8_t *we0 = w0 + (size_t)le * expert_stride;
	const uint8_t *we1 = (NMAT == 2) ? w1 + (size_t)le * expert_stride : nullptr;

	const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
	const int sub = lane / LPR, part = lane % LPR;
	const bool lane_on = part < PARTS;
	const int tile_r0 = blockIdx.x * rows_per_tile;
	const int tile_r1 = min(tile_r0 + rows_per_tile, rows_per_expert);
	constexpr int NWARP = STREAM_THREADS / 32;

	for (int p = p0; p < p1; p++) {
		const int rid = direct ? p : perm[p];
		const float *xrow = xin + (size_t)(in_by_perm ? (rid / src_div) : p) * K;
		__syncthreads();
		for (int i = threadIdx.x; i < K / 4; i += STREAM_THREADS)
			reinterpret_cast<float4 *>(xs)[i] = reinterpret_cast<const float4 *>(xrow)[i];
		__syncthreads();
		float xr[64], sx[4];
		if (lane_on)
			PartDot<KIND>::load_x(xs, part, xr, sx);
		float *orow = yout + (size_t)(out_by_perm ? rid : p) * out_stride;

		// rows of the tile are dealt to warps in passes of RPW rows; two passes are kept in flight
		for (int r = tile_r0 + warp * RPW; r < tile_r1; r += 2 * NWARP * RPW) {
			const int ra = r + sub, rb = r + NWARP * RPW + sub;
			const bool on_a = lane_on && ra < tile_r1, on_b = lane_on && rb < tile_r1;
			typename PartDot<KIND>::Raw a0, a1, b0, b1;
			if (on_a) {
				a0 = PartDot<KIND>::load(we0, NB, ra, part);
				if (NMAT == 2)
					a1 = PartDot<KIND>::load(we1, NB, ra, part);
			}
			if (on_b) {
				b0 = PartDot<KIND>::load(we0, NB, rb, part);
				if (NMAT == 2)
					b1 = PartDot<KIND>::load(we1, NB, rb, part);
			}
			float va0 = 0.f, va1 = 0.f, vb0 = 0.f, vb1 = 0.f;
			if (on_a) {
				va0 = PartDot<KIND>::dot(a0, part, xr, sx);
				if (NMAT == 2)
					va1 = PartDot<KIND>::dot(a1, part, xr, sx);
			}
			if (on_b) {
				vb0 = PartDot<KIND>::dot(b0, part, xr, sx);
				if (NMAT == 2)
					vb1 = PartDot<KIND>::dot(b1, part, xr, sx);
			}
#pragma unroll
			for (int o = LPR / 2; o > 0; o >>= 1) {
				va0 += __shfl_xor_sync(0xffffffffu, va0, o);
				vb0 += __shfl_xor_sync(0xffffffffu, vb0, o);
				if (NMAT == 2) {
					va1 += __shfl_xor_sync(0xffffffffu, va1, o);
					vb1 += __shfl_xor_sync(0xffffffffu, vb1, o);
				}
			}
			if (part == 0) {
				if (ra < tile_r1)
					orow[ra] = (NMAT == 2) ? swiglu_lut(silu, va0, va1) : va0;
				if (rb < tile_r1)
					orow[rb] = (NMAT == 2) ? swiglu_lut(silu, vb0, vb1) : vb0;
			}
		}
	}
}

template <WKind KIND, int K, int NMAT>
static int launch_stream_t(tie_cuda_ctx *c, const DevTensor &t0, const DevTensor *t1, const float *xin, int in_by_perm,
			   int src_div, float *yout, int out_by_perm, const int *row_expert, int n_rows, int direct)
{
	Scratch &s = c->s;
	const int rows = t0.rows;
	// one wave: about sm_count CTAs when few slots are active (decode), finer tiles otherwise
	int slots = direct ? n_rows : c->n_local;
	int want_tiles = direct ? max(1, c->sm_count / max(1, n_rows)) : 8;
	int rpt = (rows + want_tiles - 1) / want_tiles;
	rpt = ((rpt + 15) / 16) * 16;
	int tiles = (rows + rpt - 1) / rpt;
	dim3 grid(tiles, slots);
	stream_rows<KIND, K, NMAT><<<grid, STREAM_THREADS, 0, c->stream>>>(
		t0.ptr, t1 ? t1->ptr : nullptr, t0.expert_stride, rows, rpt, xin, in_by_perm, src_div, yout, out_by_perm, rows,
		row_expert, s.offsets, s.active, s.n_active, s.perm, direct, c->first_expert, c->n_local, c->silu, s.status);
	TIE_CUDA_LAUNCHED(c);
	return TIE_CUDA_OK;
}

template <int K, int NMAT>
static int launch_stream_k(tie_cuda_ctx *c, const DevTensor &t0, const DevTensor *t1, const float *xin, int in_by_perm,
			   int src_div, float *yout, int out_by_perm, const int *row_expert, int n_rows, int direct)
{
	if (t0.kind == W_Q4K)
		return launch_stream_t<W_Q4K, K, NMAT>(c, t0, t1, xin, in_by_perm, src_div, yout, out_by_perm, row_expert,
						       n_rows, direct);
	return launch_stream_t<W_Q6K_R8, K, NMAT>(c, t0, t1, xin, in_by_perm, src_div, yout, out_by_perm, row_expert, n_rows,
						  direct);
}

// Supported input dims are compiled in; anything else is TIE_CUDA_ENOTSUP.
#define TIE_STREAM_DIMS(X) X(256) X(512) X(768) X(1024) X(1536) X(2048) X(4096)

int launch_stream_gate_up(tie_cuda_ctx *c, const Layer &L, const float *xin, int src_div, const int *row_expert,
			  int n_rows, int direct)
{
	if (L.gate.kind != L.up.kind)
		return TIE_CUDA_ENOTSUP;
	switch (L.gate.k) {
#define X(KK)                                                                                                \
	case KK:                                                                                             \
		return launch_stream_k<KK, 2>(c, L.gate, &L.up, xin, 1, src_div, c->s.h, 0, row_expert, n_rows, \
					      direct);
		TIE_STREAM_DIMS(X)
#undef X
	default:
		return TIE_CUDA_ENOTSUP;
	}
}

int launch_stream_down(tie_cuda_ctx *c, const Layer &L, float *y, const int *row_expert, int n_rows, int direct)
{
	switch (L.down.k) {
#define X(KK)                                                                                                   \
	case KK:                                                                                                \
		return launch_stream_k<KK, 1>(c, L.down, nullptr, c->s.h, 0, 1, y, 1, row_expert, n_rows, direct);
		TIE_STREAM_DIMS(X)
#undef X
	default:
		return TIE_CUDA_ENOTSUP;
	}
}

// Single mat-vec over one uploaded tensor slice (the math_dispatch rows): rows [start,end) of
// the matrix at wexp, one input vector.
int launch_stream_matvec(tie_cuda_ctx *c, const uint8_t *wexp, WKind kind, int k, int rows_total, const float *x, float *o)
{
	DevTensor t;
	t.ptr = const_cast<uint8_t *>(wexp);
	t.kind = kind;
	t.rows = rows_total;
	t.k = k;
	t.expert_stride = 0;
	// direct mode with one slot whose "expert" is first_expert (offset 0 of wexp)
	Scratch &s = c->s;
	TIE_CUDA_TRY(c, cudaMemcpyAsync(s.row_expert, &c->first_expert, sizeof(int), cudaMemcpyHostToDevice, c->stream));
	switch (k) {
#define X(KK)                                                                                              \
	case KK:                                                                                           \
		return launch_stream_k<KK, 1>(c, t, nullptr, x, 0, 1, o, 0, s.row_expert, 1, 1);
		TIE_STREAM_DIMS(X)
#undef X
	default:
		return TIE_CUDA_ENOTSUP;
	}
}

}  // namespace tie
