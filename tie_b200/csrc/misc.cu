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

// Sum of v over the 8 lanes that hold one 32-wide sub-block (4 consecutive k per lane); the first
// lane of the group stores it split into fp16 hi + lo.
__device__ __forceinline__ void store_subblock_sum(float v, int k, __half *__restrict__ q_hi, __half *__restrict__ q_lo)
{
	v += __shfl_xor_sync(0xffffffffu, v, 1);
	v += __shfl_xor_sync(0xffffffffu, v, 2);
	v += __shfl_xor_sync(0xffffffffu, v, 4);
	if ((threadIdx.x & 7) == 0) {
		const __half h = __float2half_rn(v);
		q_hi[k >> 5] = h;
		q_lo[k >> 5] = __float2half_rn(v - __half2float(h));
	}
}

// Gather rows into expert-sorted order and split each fp32 value v into fp16 hi + lo
// (hi = rn16(v), lo = rn16(v - hi)): hi+lo carries 22 significand bits, which the tensor-core
// scheme needs to stay within the 1e-3 parity bound.  q_hi/q_lo (optional, q_cols per row): the
// sums of the row over its 32-wide sub-blocks, split the same way (the Q4_K "min" term).
// n_cols must be a multiple of 128 (whole warps per loop trip).
__global__ void __launch_bounds__(256) split_rows(const float *__restrict__ x, const int *__restrict__ perm, int src_div,
						  int n_cols, __half *__restrict__ hi, __half *__restrict__ lo,
						  __half *__restrict__ q_hi, __half *__restrict__ q_lo, int q_cols)
{
	const int p = blockIdx.x;
	// (after a call with row experts out of range the sort has placed fewer rows than the grid has
	// CTAs and the tail of perm is stale: an entry that is no row id of this call reads row 0)
	unsigned rid = perm ? (unsigned)perm[p] : (unsigned)p;
	if (perm && rid >= gridDim.x)
		rid = 0;
	const int src = perm ? (int)rid / src_div : p;
	const float *xr = x + (size_t)src * n_cols;
	__half2 *hr = reinterpret_cast<__half2 *>(hi + (size_t)p * n_cols);
	__half2 *lr = reinterpret_cast<__half2 *>(lo + (size_t)p * n_cols);
	for (int k = threadIdx.x * 4; k < n_cols; k += blockDim.x * 4) {
		float4 v = *reinterpret_cast<const float4 *>(xr + k);
		// stored order within a group of 4 is [k0, k2, k1, k3], the order the weight tiles use
		__half2 h0 = __floats2half2_rn(v.x, v.z), h1 = __floats2half2_rn(v.y, v.w);
		float2 f0 = __half22float2(h0), f1 = __half22float2(h1);
		__half2 l0 = __floats2half2_rn(v.x - f0.x, v.z - f0.y), l1 = __floats2half2_rn(v.y - f1.x, v.w - f1.y);
		hr[k / 2] = h0;
		hr[k / 2 + 1] = h1;
		lr[k / 2] = l0;
		lr[k / 2 + 1] = l1;
		if (q_hi)
			store_subblock_sum((v.x + v.y) + (v.z + v.w), k, q_hi + (size_t)p * q_cols, q_lo + (size_t)p * q_cols);
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
__global__ void __launch_bounds__(256) swiglu_split_rows(const float *__restrict__ gu, int ffn, float scale,
							 const float *__restrict__ silu, __half *__restrict__ hi,
							 __half *__restrict__ lo, __half *__restrict__ q_hi,
							 __half *__restrict__ q_lo, int q_cols, const int *__restrict__ n_rows_dev)
{
	// one row per CTA, or (row count on the device) the CTAs stride over the rows
	const size_t n_rows = n_rows_dev ? (size_t)*n_rows_dev : gridDim.x;
	for (size_t r = blockIdx.x; r < n_rows; r += gridDim.x) {
	const float *g = gu + r * 2 * ffn, *u = g + ffn;
	__half2 *hr = reinterpret_cast<__half2 *>(hi + r * ffn);
	__half2 *lr = reinterpret_cast<__half2 *>(lo + r * ffn);
	for (int k = threadIdx.x * 4; k < ffn; k += blockDim.x * 4) {
		const float4 gv = *reinterpret_cast<const float4 *>(g + k), uv = *reinterpret_cast<const float4 *>(u + k);
		const float h0 = swiglu_lut(silu, gv.x, uv.x) * scale, h1 = swiglu_lut(silu, gv.y, uv.y) * scale;
		const float h2 = swiglu_lut(silu, gv.z, uv.z) * scale, h3 = swiglu_lut(silu, gv.w, uv.w) * scale;
		const __half2 a = __floats2half2_rn(h0, h2), b = __floats2half2_rn(h1, h3);
		const float2 fa = __half22float2(a), fb = __half22float2(b);
		hr[k / 2] = a;
		hr[k / 2 + 1] = b;
		lr[k / 2] = __floats2half2_rn(h0 - fa.x, h2 - fa.y);
		lr[k / 2 + 1] = __floats2half2_rn(h1 - fb.x, h3 - fb.y);
		if (q_hi)
			store_subblock_sum((h0 + h1) + (h2 + h3), k, q_hi + r * q_cols, q_lo + r * q_cols);
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
	split_rows<<<n_rows, 256, 0, c->stream>>>(x, perm, src_div, n_cols, hi, lo, q_hi, q_lo, xq_cols(n_cols));
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
	swiglu_split_rows<<<n_rows, 256, 0, c->stream>>>(gu, ffn, scale, c->silu, hi, lo, q_hi, q_lo, xq_cols(ffn), n_rows_dev);
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
