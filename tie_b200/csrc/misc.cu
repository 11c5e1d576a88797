// Small element-wise kernels around the expert products: RMSNorm, weighted combine (+ residual),
// the fp16 hi/lo split of activations for the tensor-core path, and the table SwiGLU on its own.
#include "common.cuh"
#include "kernels.cuh"

namespace tie {

// rms_norm_f32_f32_f32_avx2 (math_avx2.c:56-97): 8 lanes of sequential fma(x,x,acc), hsum tree,
// inv = 1/sqrtf(ss/n + eps), o = (x*w)*inv.  One warp per token: lane l < 8 runs lane l's chain
// over a shared-memory copy of the row (bit-identical sum of squares); all 32 lanes then scale.
__global__ void __launch_bounds__(128) rms_norm_rows(const float *__restrict__ x, const float *__restrict__ w,
						     float *__restrict__ o, int n_tokens, int n, float eps)
{
	extern __shared__ float sm[];
	const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
	const int t = blockIdx.x * (blockDim.x >> 5) + wib;
	if (t >= n_tokens)
		return;
	float *xs = sm + (size_t)wib * n;
	const float *xr = x + (size_t)t * n;
	for (int i = lane; i < n / 4; i += 32)
		reinterpret_cast<float4 *>(xs)[i] = reinterpret_cast<const float4 *>(xr)[i];
	__syncwarp();
	float acc = 0.f;
	if (lane < 8) {
#pragma unroll 8
		for (int i = 0; i < n / 8; i++) {
			float v = xs[8 * i + lane];
			acc = __fmaf_rn(v, v, acc);
		}
	}
	float v4 = __fadd_rn(acc, __shfl_down_sync(0xffffffffu, acc, 4));
	float t2 = __fadd_rn(v4, __shfl_down_sync(0xffffffffu, v4, 1));
	float ss = __fadd_rn(t2, __shfl_down_sync(0xffffffffu, t2, 2));
	ss = __shfl_sync(0xffffffffu, ss, 0);
	float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)n), eps)));
	float *orow = o + (size_t)t * n;
	for (int i = lane; i < n; i += 32)
		orow[i] = __fmul_rn(__fmul_rn(xs[i], w ? w[i] : 1.0f), inv);
}

// model_qwen3.c:458-467: acc = 0; acc += w_j * y_j, j ascending (fused multiply-add, as the
// reference compiles it).  residual != null: out = residual + acc (math_avx2.c:731-751).
// pos != null: the row of (t, j) is y[pos[t*top_k + j]] instead of y[t*top_k + j].
__global__ void __launch_bounds__(256) combine_rows(const float *__restrict__ y, const float *__restrict__ topk_w, int top_k,
						    int hidden, const float *__restrict__ residual, float *__restrict__ out,
						    const int *__restrict__ pos)
{
	const int t = blockIdx.x;
	float wj[MAX_TOP_K];
	size_t yrow[MAX_TOP_K];
#pragma unroll
	for (int j = 0; j < MAX_TOP_K; j++) {
		wj[j] = (j < top_k) ? topk_w[(size_t)t * top_k + j] : 0.f;
		yrow[j] = (j < top_k) ? (size_t)(pos ? pos[(size_t)t * top_k + j] : t * top_k + j) * hidden : 0;
	}
	for (int k = threadIdx.x * 4; k < hidden; k += blockDim.x * 4) {
		float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
		for (int j = 0; j < MAX_TOP_K; j++) {
			if (j < top_k) {
				float4 v = *reinterpret_cast<const float4 *>(y + yrow[j] + k);
				acc.x = __fmaf_rn(wj[j], v.x, acc.x);
				acc.y = __fmaf_rn(wj[j], v.y, acc.y);
				acc.z = __fmaf_rn(wj[j], v.z, acc.z);
				acc.w = __fmaf_rn(wj[j], v.w, acc.w);
			}
		}
		if (residual) {
			float4 r = *reinterpret_cast<const float4 *>(residual + (size_t)t * hidden + k);
			acc.x = __fadd_rn(r.x, acc.x);
			acc.y = __fadd_rn(r.y, acc.y);
			acc.z = __fadd_rn(r.z, acc.z);
			acc.w = __fadd_rn(r.w, acc.w);
		}
		*reinterpret_cast<float4 *>(out + (size_t)t * hidden + k) = acc;
	}
}

// Eight consecutive values v[0..7] (k = k0 .. k0+7, k0 a multiple of 8) -> their fp16 hi and lo
// halves (hi = rn16(v), lo = rn16(v - hi)) in the operand order [k0, k2, k1, k3] per group of 4, as
// one 16-byte store each; optionally the sum over the 32-wide sub-block the values belong to (four
// neighbouring lanes hold one sub-block), split the same way.
__device__ __forceinline__ void split8_store(const float v[8], int k0, __half *__restrict__ hi_row, __half *__restrict__ lo_row,
					     __half *__restrict__ q_hi_row, __half *__restrict__ q_lo_row, int lane)
{
	uint32_t h[4], l[4];
#pragma unroll
	for (int g = 0; g < 2; g++) {
		const float a = v[4 * g], b = v[4 * g + 1], c = v[4 * g + 2], d = v[4 * g + 3];
		const __half2 h0 = __floats2half2_rn(a, c), h1 = __floats2half2_rn(b, d);
		const float2 f0 = __half22float2(h0), f1 = __half22float2(h1);
		const __half2 l0 = __floats2half2_rn(a - f0.x, c - f0.y), l1 = __floats2half2_rn(b - f1.x, d - f1.y);
		h[2 * g] = *reinterpret_cast<const uint32_t *>(&h0);
		h[2 * g + 1] = *reinterpret_cast<const uint32_t *>(&h1);
		l[2 * g] = *reinterpret_cast<const uint32_t *>(&l0);
		l[2 * g + 1] = *reinterpret_cast<const uint32_t *>(&l1);
	}
	*reinterpret_cast<uint4 *>(hi_row + k0) = make_uint4(h[0], h[1], h[2], h[3]);
	*reinterpret_cast<uint4 *>(lo_row + k0) = make_uint4(l[0], l[1], l[2], l[3]);
	if (q_hi_row) {
		float sum = ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
		sum += __shfl_xor_sync(0xffffffffu, sum, 1);
		sum += __shfl_xor_sync(0xffffffffu, sum, 2);
		if ((lane & 3) == 0) {
			const __half hs = __float2half_rn(sum);
			q_hi_row[k0 >> 5] = hs;
			q_lo_row[k0 >> 5] = __float2half_rn(sum - __half2float(hs));
		}
	}
}

constexpr int ROWS_WARPS = 8;  // warps per CTA of the row passes: one row per warp at a time

// Gather rows into expert-sorted order and split each fp32 value v into fp16 hi + lo
// (hi = rn16(v), lo = rn16(v - hi)): hi+lo carries 22 significand bits, which the tensor-core
// scheme needs to stay within the 1e-3 parity bound.  q_hi/q_lo (optional, q_cols per row): the
// sums of the row over its 32-wide sub-blocks, split the same way (the Q4_K "min" term).
// A warp takes 1024 columns of a row at a time: eight values per lane and step (16-byte loads and
// stores), four steps' loads in flight; n_cols must be a multiple of 256.
__global__ void __launch_bounds__(ROWS_WARPS * 32) split_rows(const float *__restrict__ x, const int *__restrict__ perm, int src_div,
							      int n_rows, int n_cols, __half *__restrict__ hi, __half *__restrict__ lo,
							      __half *__restrict__ q_hi, __half *__restrict__ q_lo, int q_cols)
{
	const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
	const int upr = (n_cols + 1023) >> 10;	// units of 1024 columns per row
	for (int un = blockIdx.x * ROWS_WARPS + warp; un < n_rows * upr; un += gridDim.x * ROWS_WARPS) {
		const int p = un / upr;
		// (after a call with row experts out of range the sort has placed fewer rows than it was given and
		// the tail of perm is stale: an entry that is no row id of this call reads row 0)
		unsigned rid = perm ? (unsigned)perm[p] : (unsigned)p;
		if (perm && rid >= (unsigned)n_rows)
			rid = 0;
		const int src = perm ? (int)rid / src_div : p;
		const float *xr = x + (size_t)src * n_cols;
		__half *hr = hi + (size_t)p * n_cols, *lr = lo + (size_t)p * n_cols;
		__half *qh = q_hi ? q_hi + (size_t)p * q_cols : nullptr, *ql = q_hi ? q_lo + (size_t)p * q_cols : nullptr;
		{
			const int k0 = (un - p * upr) * 1024 + lane * 8;
			float4 v[4][2];
#pragma unroll
			for (int i = 0; i < 4; i++) {
				const int k = k0 + i * 256;
				if (k < n_cols) {
					v[i][0] = *reinterpret_cast<const float4 *>(xr + k);
					v[i][1] = *reinterpret_cast<const float4 *>(xr + k + 4);
				}
			}
#pragma unroll
			for (int i = 0; i < 4; i++) {
				const int k = k0 + i * 256;
				if (k < n_cols) {  // (uniform over the warp: n_cols is a multiple of 256)
					const float f[8] = {v[i][0].x, v[i][0].y, v[i][0].z, v[i][0].w, v[i][1].x, v[i][1].y, v[i][1].z, v[i][1].w};
					split8_store(f, k, hr, lr, qh, ql, lane);
				}
			}
		}
	}
}

// Expert-parallel dispatch payload: rows in expert-sorted order, their expert ids, and the
// inverse permutation (row id -> sorted position) for the combine on the way back.
__global__ void __launch_bounds__(256) gather_rows(const float *__restrict__ x, const int *__restrict__ row_expert,
						   const int *__restrict__ perm, int src_div, int n_cols,
						   float *__restrict__ rows_out, int *__restrict__ expert_out, int *__restrict__ inv)
{
	const int p = blockIdx.x;
	int rid = perm[p];
	if ((unsigned)rid >= gridDim.x)  // stale entry behind the rows the sort placed (an expert id was out of range)
		rid = 0;
	const float4 *xr = reinterpret_cast<const float4 *>(x + (size_t)(rid / src_div) * n_cols);
	float4 *orow = reinterpret_cast<float4 *>(rows_out + (size_t)p * n_cols);
	for (int k = threadIdx.x; k < n_cols / 4; k += blockDim.x)
		orow[k] = xr[k];
	if (threadIdx.x == 0) {
		expert_out[p] = row_expert[rid];
		inv[rid] = p;
	}
}

// gu [row][gate(ffn) | up(ffn)] fp32 -> h = SwiGLU(gate, up) * scale, split into fp16 hi + lo and
// stored in the k order of the tensor-core operand tiles ([k0, k2, k1, k3] per group of 4).
// The warps stride over units of 256 columns of a row, with the 32 KB table in shared memory (two
// look-ups per element: from global memory they were what bound the pass).  ffn must be a multiple
// of 256.
__global__ void __launch_bounds__(ROWS_WARPS * 32) swiglu_split_rows(const float *__restrict__ gu, int ffn, float scale,
								     const float *__restrict__ silu, __half *__restrict__ hi,
								     __half *__restrict__ lo, __half *__restrict__ q_hi,
								     __half *__restrict__ q_lo, int q_cols,
								     const int *__restrict__ n_rows_dev, int n_rows_host)
{
	__shared__ float tab[SILU_N];
	for (int i = threadIdx.x; i < SILU_N / 4; i += blockDim.x)
		reinterpret_cast<float4 *>(tab)[i] = __ldg(reinterpret_cast<const float4 *>(silu) + i);
	__syncthreads();
	const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
	const size_t n_rows = n_rows_dev ? (size_t)*n_rows_dev : (size_t)n_rows_host;
	const size_t upr = (size_t)(ffn >> 8);
	for (size_t un = (size_t)blockIdx.x * ROWS_WARPS + warp; un < n_rows * upr; un += (size_t)gridDim.x * ROWS_WARPS) {
		const size_t r = un / upr;
		const float *g = gu + r * 2 * ffn, *u = g + ffn;
		__half *hr = hi + r * ffn, *lr = lo + r * ffn;
		__half *qh = q_hi ? q_hi + r * q_cols : nullptr, *ql = q_hi ? q_lo + r * q_cols : nullptr;
		{
			const int k = (int)(un - r * upr) * 256 + lane * 8;
			const float4 g0 = *reinterpret_cast<const float4 *>(g + k), g1 = *reinterpret_cast<const float4 *>(g + k + 4);
			const float4 u0 = *reinterpret_cast<const float4 *>(u + k), u1 = *reinterpret_cast<const float4 *>(u + k + 4);
			const float f[8] = {swiglu_lut(tab, g0.x, u0.x) * scale, swiglu_lut(tab, g0.y, u0.y) * scale,
					    swiglu_lut(tab, g0.z, u0.z) * scale, swiglu_lut(tab, g0.w, u0.w) * scale,
					    swiglu_lut(tab, g1.x, u1.x) * scale, swiglu_lut(tab, g1.y, u1.y) * scale,
					    swiglu_lut(tab, g1.z, u1.z) * scale, swiglu_lut(tab, g1.w, u1.w) * scale};
			split8_store(f, k, hr, lr, qh, ql, lane);
		}
	}
}

__global__ void __launch_bounds__(256) swiglu_kernel(float *__restrict__ gate, const float *__restrict__ up, int n,
						     const float *__restrict__ silu)
{
	int i = blockIdx.x * blockDim.x + threadIdx.x;
	if (i < n)
		gate[i] = swiglu_lut(silu, gate[i], up[i]);
}

// Distinct experts with at least one row (for the traffic accounting of benchmarks).
__global__ void copy_int(const int *src, int *dst)
{
	*dst = *src;
}

int launch_rms_norm(tie_cuda_ctx *c, const float *x, const float *w, float *o, int n_tokens)
{
	const int H = c->cfg.hidden;
	const int wpb = 4;
	size_t smem = (size_t)wpb * H * sizeof(float);
	if (smem > 48 * 1024)  // the kernel runs within the default dynamic shared-memory limit
		return TIE_CUDA_ENOTSUP;
	rms_norm_rows<<<(n_tokens + wpb - 1) / wpb, wpb * 32, smem, c->stream>>>(x, w, o, n_tokens, H, c->cfg.norm_eps);
	TIE_CUDA_LAUNCHED(c);
	return TIE_CUDA_OK;
}

int launch_combine(tie_cuda_ctx *c, const float *y, const float *topk_w, int n_tokens, const float *residual, float *out,
		   const int *pos)
{
	combine_rows<<<n_tokens, 256, 0, c->stream>>>(y, topk_w, c->cfg.top_k, c->cfg.hidden, residual, out, pos);
	TIE_CUDA_LAUNCHED(c);
	return TIE_CUDA_OK;
}

int launch_split_rows(tie_cuda_ctx *c, const float *x, const int *perm, int src_div, int n_rows, int n_cols, __half *hi,
		      __half *lo, __half *q_hi, __half *q_lo)
{
	if (n_cols % 256)
		return TIE_CUDA_ENOTSUP;
	const int want = (n_rows * ((n_cols + 1023) / 1024) + ROWS_WARPS - 1) / ROWS_WARPS, cap = c->sm_count * 8;
	if (n_rows <= 0)
		return TIE_CUDA_OK;
	split_rows<<<want < cap ? want : cap, ROWS_WARPS * 32, 0, c->stream>>>(x, perm, src_div, n_rows, n_cols, hi, lo, q_hi, q_lo,
										xq_cols(n_cols));
	TIE_CUDA_LAUNCHED(c);
	return TIE_CUDA_OK;
}

int launch_gather_rows(tie_cuda_ctx *c, const float *x, const int *row_expert, const int *perm, int src_div, int n_rows,
		       float *rows_out, int *expert_out, int *inv)
{
	gather_rows<<<n_rows, 256, 0, c->stream>>>(x, row_expert, perm, src_div, c->cfg.hidden, rows_out, expert_out, inv);
	TIE_CUDA_LAUNCHED(c);
	return TIE_CUDA_OK;
}

int launch_swiglu_split(tie_cuda_ctx *c, const float *gu, int n_rows, int ffn, float scale, __half *hi, __half *lo, __half *q_hi,
			__half *q_lo, const int *n_rows_dev)
{
	if (ffn % 256)
		return TIE_CUDA_ENOTSUP;
	// (n_rows_dev: the row count is read on the device and n_rows is the grid the caller wants)
	const int want = (n_rows * (ffn / 256) + ROWS_WARPS - 1) / ROWS_WARPS, cap = c->sm_count * 4;
	const int grid = n_rows_dev ? n_rows : (want < cap ? want : cap);
	swiglu_split_rows<<<grid > 0 ? grid : 1, ROWS_WARPS * 32, 0, c->stream>>>(gu, ffn, scale, c->silu, hi, lo, q_hi, q_lo, xq_cols(ffn),
										   n_rows_dev, n_rows);
	TIE_CUDA_LAUNCHED(c);
	return TIE_CUDA_OK;
}

int launch_swiglu(tie_cuda_ctx *c, float *gate, const float *up, int n)
{
	swiglu_kernel<<<(n + 255) / 256, 256, 0, c->stream>>>(gate, up, n, c->silu);
	TIE_CUDA_LAUNCHED(c);
	return TIE_CUDA_OK;
}

}  // namespace tie
