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
#include "partdot.cuh"

namespace tie {

constexpr int STREAM_THREADS = 256;

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
