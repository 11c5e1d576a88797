// Expert parallelism over peer memory: dispatch and combine fused into the kernels that consume
// the rows, no collective library call and no host synchronisation per block.
//
// The reference is one process and has no counterpart.  One process per GPU; rank r owns experts
// [r*E/G, (r+1)*E/G).  Every rank exposes one "region" of its HBM to its peers (CUDA IPC):
//
//   xs     fp32 [t_max][H]      this rank's tokens of the current step
//   ids    int  [t_max*K]       its (token, slot) row ids grouped by GLOBAL expert (stable sort)
//   counts int  [E]             rows per expert from this rank
//   pub    u32  [G]             pub[s]  = step number, written BY rank s once xs/ids/counts are final
//   done   u32  [G]             done[d] = step number, written BY rank d once its y rows are final
//   y      fp32 [rows_cap][H]   outputs of the rows this rank's experts processed
//
// A step (all ranks call the three phases in the same order with the same step number):
//   publish  route + sort locally into the region, then store the step number into pub[r] of
//            every peer (release, system scope)
//   compute  ep_index waits (bounded) for all G pub flags, reads every peer's counts (G x E ints)
//            and derives the whole row layout from them alone: the rows of local expert le from
//            source s sit at offsets[le] + sum_{s'<s} cnt[s'][le] + j — the receiver needs no
//            sort and no id exchange, and the source can compute where its rows' outputs will
//            be.  ep_split_rows then gathers the token rows straight out of the peers' xs
//            (plain loads over NVLink) into the fp16 hi/lo operand of the grouped product; the
//            down product writes y into the region; done[r] is stored to every peer
//   gather   ep_combine_rows waits (bounded) for the done flags and sums each token's top_k rows
//            out of the owners' y with the gate weights, in slot order (model_qwen3.c:458-467)
//
// Re-use of the region is safe without further flags: a rank's publish of step n+1 follows its
// own gather of step n in stream order, and a peer's compute of step n+1 (which overwrites y)
// starts after it has seen every pub flag of step n+1.
//
// Peer data is read with ld.global.cg (never through the non-coherent path); flags with
// ld.acquire.sys / st.release.sys.  Every wait is bounded by a cycle budget; on a time-out the
// kernel sets ST_WAIT_TIMEOUT, publishes an empty layout and returns.
#include "common.cuh"
#include "kernels.cuh"

namespace tie {

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned *p)
{
	unsigned v;
	asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
	return v;
}

__device__ __forceinline__ void st_release_sys(unsigned *p, unsigned v)
{
	asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// true once *flag has reached step (wrap-safe), false after `budget` cycles.
__device__ __forceinline__ bool ep_wait_flag(const unsigned *flag, unsigned step, long long budget)
{
	const long long t0 = clock64();
	for (;;) {
		if ((int)(ld_acquire_sys(flag) - step) >= 0)
			return true;
		if (clock64() - t0 > budget)
			return false;
		__nanosleep(200);
	}
}

template <typename T>
__device__ __forceinline__ T *ep_ptr(const EpView &v, int rank, size_t off)
{
	return reinterpret_cast<T *>(v.peer[rank] + off);
}

// One CTA: tells every peer that this rank's part of `step` is final.  which = 0: pub, 1: done.
__global__ void ep_signal(EpView v, int which, unsigned step)
{
	const int d = threadIdx.x;
	if (d < v.n_ranks) {
		__threadfence_system();
		st_release_sys(ep_ptr<unsigned>(v, d, which ? v.off_done : v.off_pub) + v.rank, step);
	}
}

constexpr int EP_INDEX_THREADS = 256;

// One CTA.  Outputs (this rank's scratch): counts/offsets/tile_start/tile_info/active/n_active
// exactly as sort_place leaves them for the grouped product, n_rows, the segment table
// seg_base[E+1] / seg_src[E] (segment i = le*G + s: first sorted row, first entry in s's ids)
// and ybase[E]: where, in the owner's y, the first row of (this rank, expert e) will be.
__global__ void __launch_bounds__(EP_INDEX_THREADS)
ep_index(EpView v, unsigned step, long long budget, int n_tile, int *__restrict__ counts, int *__restrict__ offsets,
	 int *__restrict__ tile_start, int4 *__restrict__ tile_info, int *__restrict__ active, int *__restrict__ n_active,
	 int *__restrict__ n_rows_out, int *__restrict__ seg_base, int *__restrict__ seg_src, int *__restrict__ ybase,
	 unsigned *__restrict__ status)
{
	extern __shared__ int sm[];
	const int G = v.n_ranks, E = v.n_expert, NL = v.n_local, fe = v.rank * NL;
	int *cnt = sm;		   // [G][E]
	int *tot = cnt + G * E;	   // [E]   rows of expert e over all sources
	int *loff = tot + E;	   // [NL + 1] exclusive prefix of tot over the local experts
	int *ltile = loff + NL + 1;  // [NL + 1] same for token tiles
	const int tid = threadIdx.x;

	bool ok = true;
	if (tid < G)
		ok = ep_wait_flag(ep_ptr<unsigned>(v, v.rank, v.off_pub) + tid, step, budget);
	ok = __syncthreads_and(ok);
	if (ok) {
		const int row_max = v.t_max * v.top_k;
		bool sane = true;
		for (int i = tid; i < G * E; i += EP_INDEX_THREADS) {
			const int c = __ldcg(ep_ptr<int>(v, i / E, v.off_counts) + i % E);
			sane = sane && c >= 0 && c <= row_max;
			cnt[i] = c;
		}
		ok = __syncthreads_and(sane);
		if (ok) {
			for (int e = tid; e < E; e += EP_INDEX_THREADS) {
				int t = 0;
				for (int s = 0; s < G; s++)
					t += cnt[s * E + e];
				tot[e] = t;
			}
			__syncthreads();
			if (tid == 0) {
				int o = 0, tl = 0;
				for (int le = 0; le < NL; le++) {
					loff[le] = o;
					ltile[le] = tl;
					o += tot[fe + le];
					tl += (tot[fe + le] + n_tile - 1) / n_tile;
				}
				loff[NL] = o;
				ltile[NL] = tl;
			}
			__syncthreads();
			ok = (long long)loff[NL] <= v.rows_cap;
		}
		if (!ok && tid == 0)
			atomicOr(status, ST_BAD_TILE);
	} else if (tid == 0) {
		atomicOr(status, ST_WAIT_TIMEOUT);
	}
	if (!ok) {  // an empty layout: the kernels that follow find no work
		for (int le = tid; le <= NL; le += EP_INDEX_THREADS) {
			offsets[le] = 0;
			tile_start[le] = 0;
			if (le < NL)
				counts[le] = 0;
		}
		for (int i = tid; i <= E; i += EP_INDEX_THREADS) {
			seg_base[i] = 0;
			if (i < E) {
				seg_src[i] = 0;
				ybase[i] = -1;
			}
		}
		if (tid == 0) {
			*n_active = 0;
			*n_rows_out = 0;
		}
		return;
	}
	// layout of the local experts
	for (int le = tid; le <= NL; le += EP_INDEX_THREADS) {
		offsets[le] = loff[le];
		tile_start[le] = ltile[le];
		if (le < NL) {
			const int c = tot[fe + le];
			counts[le] = c;
			for (int j = 0; j * n_tile < c; j++)
				tile_info[ltile[le] + j] = make_int4(le, loff[le] + j * n_tile, min(n_tile, c - j * n_tile), 0);
		}
	}
	if (tid == 0) {
		int a = 0;
		for (int le = 0; le < NL; le++)
			if (tot[fe + le] > 0)
				active[a++] = le;
		*n_active = a;
		*n_rows_out = loff[NL];
		seg_base[NL * G] = loff[NL];
	}
	// segments (le, s): where they start here, and where they start in the source's id list
	for (int i = tid; i < NL * G; i += EP_INDEX_THREADS) {
		const int le = i / G, s = i % G, e = fe + le;
		int b = loff[le];
		for (int s2 = 0; s2 < s; s2++)
			b += cnt[s2 * E + e];
		int so = 0;
		for (int e2 = 0; e2 < e; e2++)
			so += cnt[s * E + e2];
		seg_base[i] = b;
		seg_src[i] = so;
	}
	// where the owner of expert e puts this rank's rows of e
	for (int e = tid; e < E; e += EP_INDEX_THREADS) {
		const int d = e / NL;
		int b = 0;
		for (int e2 = d * NL; e2 < e; e2++)
			b += tot[e2];
		for (int s2 = 0; s2 < v.rank; s2++)
			b += cnt[s2 * E + e];
		ybase[e] = b;
	}
}

constexpr int EP_SPLIT_THREADS = 256;

// Sorted row p of this rank = row j of segment (le, s): token ids[seg_src + j] / top_k of rank s.
// Reads that token's fp32 row from rank s and writes the fp16 hi/lo operand row p (same
// arithmetic and element order as split_rows).  Grid-stride over the rows; n_rows is on the device.
__global__ void __launch_bounds__(EP_SPLIT_THREADS)
ep_split_rows(EpView v, const int *__restrict__ n_rows_dev, const int *__restrict__ seg_base, const int *__restrict__ seg_src,
	      __half *__restrict__ hi, __half *__restrict__ lo, __half *__restrict__ q_hi, __half *__restrict__ q_lo,
	      int q_cols, unsigned *__restrict__ status)
{
	__shared__ int s_base[257], s_src[256];
	const int n_seg = v.n_local * v.n_ranks;  // = n_expert
	for (int i = threadIdx.x; i <= n_seg; i += EP_SPLIT_THREADS) {
		s_base[i] = seg_base[i];
		if (i < n_seg)
			s_src[i] = seg_src[i];
	}
	__syncthreads();
	const int n_rows = *n_rows_dev, H = v.hidden;
	for (int p = blockIdx.x; p < n_rows; p += gridDim.x) {
		// last segment whose first row is <= p (empty segments share their successor's start)
		int lo_i = 0, hi_i = n_seg;
		while (hi_i - lo_i > 1) {
			const int mid = (lo_i + hi_i) >> 1;
			if (s_base[mid] <= p)
				lo_i = mid;
			else
				hi_i = mid;
		}
		const int s = lo_i % v.n_ranks;
		const int id = __ldcg(ep_ptr<int>(v, s, v.off_ids) + s_src[lo_i] + (p - s_base[lo_i]));
		const int token = id / v.top_k;
		if (token < 0 || token >= v.t_max) {
			if (threadIdx.x == 0)
				atomicOr(status, ST_BAD_TILE);
			continue;
		}
		const float *xr = ep_ptr<float>(v, s, v.off_xs) + (size_t)token * H;
		__half2 *hr = reinterpret_cast<__half2 *>(hi + (size_t)p * H);
		__half2 *lr = reinterpret_cast<__half2 *>(lo + (size_t)p * H);
		for (int k = threadIdx.x * 4; k < H; k += EP_SPLIT_THREADS * 4) {
			const float4 x4 = __ldcg(reinterpret_cast<const float4 *>(xr + k));
			const __half2 h0 = __floats2half2_rn(x4.x, x4.z), h1 = __floats2half2_rn(x4.y, x4.w);
			const float2 f0 = __half22float2(h0), f1 = __half22float2(h1);
			hr[k / 2] = h0;
			hr[k / 2 + 1] = h1;
			lr[k / 2] = __floats2half2_rn(x4.x - f0.x, x4.z - f0.y);
			lr[k / 2 + 1] = __floats2half2_rn(x4.y - f1.x, x4.w - f1.y);
			if (q_hi) {
				float sum = (x4.x + x4.y) + (x4.z + x4.w);
				sum += __shfl_xor_sync(0xffffffffu, sum, 1);
				sum += __shfl_xor_sync(0xffffffffu, sum, 2);
				sum += __shfl_xor_sync(0xffffffffu, sum, 4);
				if ((threadIdx.x & 7) == 0) {
					const __half h = __float2half_rn(sum);
					q_hi[(size_t)p * q_cols + (k >> 5)] = h;
					q_lo[(size_t)p * q_cols + (k >> 5)] = __float2half_rn(sum - __half2float(h));
				}
			}
		}
	}
}

// out[t] = (residual[t] +) sum_j w[t][j] * y_owner[row of (t, j)], j ascending, fused multiply-add
// from zero — the arithmetic of combine_rows, with each row read from its expert's owner.
__global__ void __launch_bounds__(256)
ep_combine_rows(EpView v, unsigned step, long long budget, int n_tokens, const int *__restrict__ topk_idx,
		const float *__restrict__ topk_w, const int *__restrict__ inv, const int *__restrict__ src_off,
		const int *__restrict__ ybase, const float *__restrict__ residual, float *__restrict__ out,
		unsigned *__restrict__ status)
{
	const int t = blockIdx.x, K = v.top_k, H = v.hidden;
	bool ok = true;
	if ((int)threadIdx.x < v.n_ranks)
		ok = ep_wait_flag(ep_ptr<unsigned>(v, v.rank, v.off_done) + threadIdx.x, step, budget);
	ok = __syncthreads_and(ok);
	if (!ok) {
		if (threadIdx.x == 0)
			atomicOr(status, ST_WAIT_TIMEOUT);
		return;
	}
	if (t >= n_tokens)  // a rank without tokens only waits
		return;
	float wj[MAX_TOP_K];
	const float *yrow[MAX_TOP_K];
	bool bad = false;
#pragma unroll
	for (int j = 0; j < MAX_TOP_K; j++) {
		wj[j] = 0.f;
		yrow[j] = nullptr;
		if (j < K) {
			const int e = topk_idx[(size_t)t * K + j];
			const int d = e / v.n_local;
			const long long pos = (long long)ybase[e] + inv[(size_t)t * K + j] - src_off[e];
			if (ybase[e] < 0 || pos < 0 || pos >= v.rows_cap) {
				bad = true;
			} else {
				wj[j] = topk_w[(size_t)t * K + j];
				yrow[j] = ep_ptr<float>(v, d, v.off_y) + (size_t)pos * H;
			}
		}
	}
	if (bad) {
		if (threadIdx.x == 0)
			atomicOr(status, ST_BAD_TILE);
		return;
	}
	for (int k = threadIdx.x * 4; k < H; k += blockDim.x * 4) {
		float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
		for (int j = 0; j < MAX_TOP_K; j++) {
			if (j < K) {
				const float4 y4 = __ldcg(reinterpret_cast<const float4 *>(yrow[j] + k));
				acc.x = __fmaf_rn(wj[j], y4.x, acc.x);
				acc.y = __fmaf_rn(wj[j], y4.y, acc.y);
				acc.z = __fmaf_rn(wj[j], y4.z, acc.z);
				acc.w = __fmaf_rn(wj[j], y4.w, acc.w);
			}
		}
		if (residual) {
			const float4 r = *reinterpret_cast<const float4 *>(residual + (size_t)t * H + k);
			acc.x = __fadd_rn(r.x, acc.x);
			acc.y = __fadd_rn(r.y, acc.y);
			acc.z = __fadd_rn(r.z, acc.z);
			acc.w = __fadd_rn(r.w, acc.w);
		}
		*reinterpret_cast<float4 *>(out + (size_t)t * H + k) = acc;
	}
}

int launch_ep_signal(tie_cuda_ctx *c, int which, unsigned step)
{
	ep_signal<<<1, 32, 0, c->stream>>>(c->ep.view, which, step);
	TIE_CUDA_LAUNCHED(c);
	return TIE_CUDA_OK;
}

int launch_ep_index(tie_cuda_ctx *c, unsigned step)
{
	Scratch &s = c->s;
	const EpView &v = c->ep.view;
	const size_t smem = ((size_t)v.n_ranks * v.n_expert + v.n_expert + 2 * (v.n_local + 1)) * sizeof(int);
	ep_index<<<1, EP_INDEX_THREADS, smem, c->stream>>>(v, step, c->ep.wait_cycles, TC_TOKEN_TILE, s.counts, s.offsets, s.tile_start,
							   s.tile_info, s.active, s.n_active, c->ep.n_rows, c->ep.seg_base,
							   c->ep.seg_src, c->ep.ybase, s.status);
	TIE_CUDA_LAUNCHED(c);
	return TIE_CUDA_OK;
}

int launch_ep_split_rows(tie_cuda_ctx *c, bool sums)
{
	Scratch &s = c->s;
	ep_split_rows<<<c->sm_count * 8, EP_SPLIT_THREADS, 0, c->stream>>>(c->ep.view, c->ep.n_rows, c->ep.seg_base, c->ep.seg_src,
									    s.xs_hi, s.xs_lo, sums ? s.xq_hi : nullptr,
									    sums ? s.xq_lo : nullptr, xq_cols(c->cfg.hidden), s.status);
	TIE_CUDA_LAUNCHED(c);
	return TIE_CUDA_OK;
}

int launch_ep_combine(tie_cuda_ctx *c, unsigned step, int n_tokens, const float *residual, float *out)
{
	Scratch &s = c->s;
	ep_combine_rows<<<n_tokens > 0 ? n_tokens : 1, 256, 0, c->stream>>>(c->ep.view, step, c->ep.wait_cycles, n_tokens, s.topk_idx,
									     s.topk_w, s.ep_inv, s.ep_offsets, c->ep.ybase, residual,
									     out, s.status);
	TIE_CUDA_LAUNCHED(c);
	return TIE_CUDA_OK;
}

}  // namespace tie
