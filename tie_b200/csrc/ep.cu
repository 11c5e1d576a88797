// Expert parallelism over peer memory: dispatch and combine fused into the kernels that consume
// the rows, no collective library call and no host synchronisation per block.
//
// The reference is one process and has no counterpart.  One process per GPU; rank r owns experts
// [r*E/G, (r+1)*E/G).  Every rank exposes one "region" of its HBM to its peers (CUDA IPC):
//
//   xs     fp32 [t_max][H]      this rank's tokens of the current step
//   ids    int  [t_max*K]       its (token, slot) row ids grouped by GLOBAL expert (stable sort);
//                               EP_FIRST_OF_TOKEN marks a token's first row for the owner's GPU
//   topk   int  [t_max*K]       the selected experts of its tokens, in slot order
//   inv    int  [t_max*K]       where each (token, slot) row stands in ids
//   counts int  [E]             rows per expert from this rank
//   cnt_all int [G][E]          row s: the counts of rank s, stored BY rank s with its pub flag
//   x_all  fp32 [G][t_max][H]   slot s: the tokens of rank s of the current step, stored BY rank s
//   pub    u32  [G]             pub[s]  = step number, written BY rank s once its slot of every x_all and
//                               its ids/counts are final
//   done   u32  [G]             done[d] = step number, written BY rank d once it has delivered its outputs
//   y      fp32 [t_max*K][H]    expert outputs of THIS rank's rows, in (token, slot) order, written
//                               by the owners of the experts
//
// A step (all ranks call the three phases in the same order):
//   publish  route + sort locally into the region while extra CTAs of the router's kernel store this
//            rank's tokens into its slot of every rank's x_all (plain stores over NVLink), then
//            store the step number into pub[r] of every peer (release, system scope)
//   compute  ep_index waits (bounded) for all G pub flags, reads the G x E count matrix (local)
//            and derives the whole row layout from it alone: the rows of local expert le from
//            source s sit at offsets[le] + sum_{s'<s} cnt[s'][le] + j — the receiver needs no
//            sort.  ep_split_rows then lays the token rows out (from x_all, local memory; the row
//            lists come straight out of the peers' regions, plain loads over NVLink) as the fp16
//            hi/lo operand of the grouped product and notes where each row came from; the down product's epilogue stores every output
//            row into ITS SOURCE's y (plain stores over NVLink, overlapped with the product);
//            done[r] is then stored to every peer
//   gather   ep_combine_rows waits (bounded) for the done flags of all owners and sums each
//            token's top_k rows of the local y with the gate weights, in slot order
//            (model_qwen3.c:458-467)
//
// Re-use of the region is safe without further flags: a rank's publish of step n+1 follows its
// own gather of step n in stream order, and a peer's compute of step n+1 (which overwrites that
// rank's y) starts after it has seen every pub flag of step n+1.
//
// Peer data is read with ld.global.cg (never through the non-coherent path); flags with
// ld.acquire.sys / st.release.sys.  Every wait is bounded by a cycle budget; on a time-out the
// kernel sets ST_WAIT_TIMEOUT, publishes an empty layout and returns.
#include "common.cuh"
#include "ep_dev.cuh"
#include "kernels.cuh"

namespace tie {

// One CTA: tells every peer that this rank's part of the current step is final.  which = 0 (pub)
// first advances the step counter, which = 1 (done) reads it.  The counter lives on the device so
// that a step's launches take the same arguments every time (they can be replayed from a graph).
__global__ void ep_signal(EpView v, int which, unsigned *__restrict__ step_dev)
{
	unsigned step = 0;
	if (threadIdx.x == 0) {
		step = *step_dev + (which ? 0u : 1u);
		if (!which)
			*step_dev = step;
	}
	step = __shfl_sync(0xffffffffu, step, 0);
	if (!which) {
		// this rank's rows per expert go to every rank's count matrix (row `rank`): the owners derive
		// their layout from local memory
		const int *cnt = ep_ptr<int>(v, v.rank, v.off_counts);
		for (int e = threadIdx.x; e < v.n_expert; e += 32) {
			const int c = __ldcg(cnt + e);
			for (int j = 0; j < v.n_ranks; j++)
				ep_ptr<int>(v, (v.rank + j) % v.n_ranks, v.off_cntall)[(size_t)v.rank * v.n_expert + e] = c;
		}
		__syncwarp();
	}
	const int d = threadIdx.x;
	if (d < v.n_ranks) {
		__threadfence_system();
		st_release_sys(ep_ptr<unsigned>(v, d, which ? v.off_done : v.off_pub) + v.rank, step);
	}
}

constexpr int EP_PUSH_THREADS = 256;

// The hand-over of this rank's tokens as a launch of its own (where it does not ride along with
// the router's kernel): ep_push_tokens_cta on every CTA.
__global__ void __launch_bounds__(EP_PUSH_THREADS) ep_push_tokens(EpPush f)
{
	ep_push_tokens_cta(f, blockIdx.x, gridDim.x);
}

constexpr int EP_INDEX_THREADS = 256;

// Exclusive prefix sum of one value per thread over the CTA (EP_INDEX_THREADS threads); total
// (optional) receives the sum.  wsum: EP_INDEX_THREADS / 32 ints of shared memory.
__device__ __forceinline__ int ep_block_scan(int val, int *wsum, int *total = nullptr)
{
	const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
	int incl = val;
#pragma unroll
	for (int o = 1; o < 32; o <<= 1) {
		const int t = __shfl_up_sync(0xffffffffu, incl, o);
		if (lane >= o)
			incl += t;
	}
	__syncthreads();  // wsum may still be read by the previous scan
	if (lane == 31)
		wsum[warp] = incl;
	__syncthreads();
	int before = 0, all = 0;
#pragma unroll
	for (int i = 0; i < EP_INDEX_THREADS / 32; i++) {
		const int w = wsum[i];
		before += i < warp ? w : 0;
		all += w;
	}
	if (total)
		*total = all;
	return before + incl - val;
}

// One CTA; thread i stands for expert i (n_expert <= EP_INDEX_THREADS).  Outputs (this rank's
// scratch): counts/offsets/tile_start/tile_info/active/n_active exactly as sort_scatter leaves
// them for the grouped product, n_rows, the segment table seg_base[E+1] / seg_src[E] (segment
// i = le*G + s: first sorted row, first entry in s's ids).
__global__ void __launch_bounds__(EP_INDEX_THREADS)
ep_index(EpView v, const unsigned *__restrict__ step_dev, long long budget, int n_tile, int *__restrict__ counts, int *__restrict__ offsets,
	 int *__restrict__ tile_start, int4 *__restrict__ tile_info, int *__restrict__ active, int *__restrict__ n_active,
	 int *__restrict__ n_rows_out, int *__restrict__ seg_base, int *__restrict__ seg_src, unsigned *__restrict__ status)
{
	extern __shared__ int sm[];
	__shared__ int wsum[EP_INDEX_THREADS / 32];
	const int G = v.n_ranks, E = v.n_expert, NL = v.n_local, fe = v.rank * NL;
	int *cnt = sm;		 // [G][E]  rows of source s for expert e
	int *soff = cnt + G * E; // [G][E]  exclusive prefix of cnt over e: where e starts in s's id list
	int *tpre = soff + G * E;  // [E + 1] exclusive prefix over e of the rows of e from all sources
	const int tid = threadIdx.x;
	const unsigned step = *step_dev;

	bool ok = true;
	if (tid < G)
		ok = ep_wait_flag(ep_ptr<unsigned>(v, v.rank, v.off_pub) + tid, step, budget);
	ok = __syncthreads_and(ok);
	if (!ok && tid == 0)
		atomicOr(status, ST_WAIT_TIMEOUT);
	int n_rows = 0;
	if (ok) {
		const int row_max = v.t_max * v.top_k;
		bool sane = true;
		const int *cnt_all = ep_ptr<int>(v, v.rank, v.off_cntall);  // row s: stored here by rank s with its pub flag
		for (int i = tid; i < G * E; i += EP_INDEX_THREADS) {
			const int c = __ldcg(cnt_all + i);
			sane = sane && c >= 0 && c <= row_max;
			cnt[i] = c;
		}
		ok = __syncthreads_and(sane);
		if (ok) {
			// where expert e starts in source s's id list: one warp per source, a lane takes a run of experts
			const int lane = tid & 31, per = (E + 31) / 32;  // per <= 8 (E <= 256)
			for (int s = tid >> 5; s < G; s += EP_INDEX_THREADS / 32) {
				int run = 0;
				for (int k = 0; k < per; k++) {
					const int e = lane * per + k;
					run += e < E ? cnt[s * E + e] : 0;
				}
				int incl = run;
#pragma unroll
				for (int o = 1; o < 32; o <<= 1) {
					const int t = __shfl_up_sync(0xffffffffu, incl, o);
					if (lane >= o)
						incl += t;
				}
				int pre = incl - run;
				for (int k = 0; k < per; k++) {
					const int e = lane * per + k;
					if (e < E) {
						soff[s * E + e] = pre;
						pre += cnt[s * E + e];
					}
				}
			}
			int tot = 0;
			if (tid < E)
				for (int s = 0; s < G; s++)
					tot += cnt[s * E + tid];
			int all = 0;
			const int pre = ep_block_scan(tot, wsum, &all);
			if (tid < E)
				tpre[tid] = pre;
			if (tid == 0)
				tpre[E] = all;
			__syncthreads();
			n_rows = tpre[fe + NL] - tpre[fe];
			ok = (long long)n_rows <= v.rows_cap;
		}
		if (!ok && tid == 0)
			atomicOr(status, ST_BAD_TILE);
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
			if (i < E)
				seg_src[i] = 0;
		}
		if (tid == 0) {
			*n_active = 0;
			*n_rows_out = 0;
		}
		return;
	}
	// layout of the local experts: thread le
	const bool local = tid < NL;
	const int e_loc = fe + tid;
	const int c_loc = local ? tpre[e_loc + 1] - tpre[e_loc] : 0;
	const int off_loc = local ? tpre[e_loc] - tpre[fe] : 0;
	int all_tiles = 0, all_active = 0;
	const int tile0 = ep_block_scan((c_loc + n_tile - 1) / n_tile, wsum, &all_tiles);
	const int act0 = ep_block_scan(c_loc > 0 ? 1 : 0, wsum, &all_active);
	if (local) {
		counts[tid] = c_loc;
		offsets[tid] = off_loc;
		tile_start[tid] = tile0;
		if (c_loc > 0)
			active[act0] = tid;
		for (int j = 0; j * n_tile < c_loc; j++)
			tile_info[tile0 + j] = make_int4(tid, off_loc + j * n_tile, min(n_tile, c_loc - j * n_tile), 0);
		// segments (le, s): where they start here, and where they start in the source's id list
		int b = off_loc;
		for (int s = 0; s < G; s++) {
			seg_base[tid * G + s] = b;
			seg_src[tid * G + s] = soff[s * E + e_loc];
			b += cnt[s * E + e_loc];
		}
	}
	if (tid == 0) {
		offsets[NL] = n_rows;
		tile_start[NL] = all_tiles;
		*n_active = all_active;
		*n_rows_out = n_rows;
		seg_base[NL * G] = n_rows;
	}
}

constexpr int EP_SPLIT_THREADS = 256;
constexpr int EP_SPLIT_F4 = 8;	// float4 loads a lane keeps in flight

// Sorted row p of this rank = row j of segment (le, s): entry ids[seg_src + j] of rank s, token
// id / top_k.  row_dst[p] = (s << 24) | row id tells the down product where the row's output goes.
// The token itself is in this rank's x_all (slot s), where rank s has stored it.  A token whose
// selected experts include several of this rank's is read ONCE: the warp of the token's first
// row here (EP_FIRST_OF_TOKEN in the entry, set by the source's sort) reads the fp32 row,
// together with the token's expert ids and the places of its rows in s's list (from rank s, over
// NVLink: a few bytes), and writes the fp16 hi/lo operand rows (same arithmetic and element order
// as split_rows) of all of the token's rows here; the warps of the other rows only note row_dst.
// One warp per row, EP_SPLIT_F4 16-byte loads in flight per lane; the warps stride over the rows,
// n_rows is on the device.
__global__ void __launch_bounds__(EP_SPLIT_THREADS)
ep_split_rows(EpView v, const int *__restrict__ n_rows_dev, const int *__restrict__ seg_base, const int *__restrict__ seg_src,
	      __half *__restrict__ hi, __half *__restrict__ lo, __half *__restrict__ q_hi, __half *__restrict__ q_lo,
	      int q_cols, unsigned *__restrict__ row_dst, unsigned *__restrict__ status)
{
	__shared__ int s_base[257], s_src[256];
	const int n_seg = v.n_local * v.n_ranks;  // = n_expert
	for (int i = threadIdx.x; i <= n_seg; i += EP_SPLIT_THREADS) {
		s_base[i] = seg_base[i];
		if (i < n_seg)
			s_src[i] = seg_src[i];
	}
	__syncthreads();
	const int n_rows = *n_rows_dev, H = v.hidden, K = v.top_k, fe = v.rank * v.n_local;
	const int lane = threadIdx.x & 31;
	const int warps = gridDim.x * (EP_SPLIT_THREADS / 32);
	for (int p = blockIdx.x * (EP_SPLIT_THREADS / 32) + (threadIdx.x >> 5); p < n_rows; p += warps) {
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
		const int entry = __ldcg(ep_ptr<int>(v, s, v.off_ids) + s_src[lo_i] + (p - s_base[lo_i]));
		const int id = entry & ~EP_FIRST_OF_TOKEN;
		const int token = id / K;
		if (entry < 0 || token >= v.t_max) {
			if (lane == 0) {
				atomicOr(status, ST_BAD_TILE);
				row_dst[p] = (unsigned)v.rank << 24;  // somewhere harmless: row 0 of this rank's own y
			}
			continue;
		}
		if (lane == 0)
			row_dst[p] = ((unsigned)s << 24) | (unsigned)id;
		if (!(entry & EP_FIRST_OF_TOKEN))
			continue;  // filled by the warp of the token's first row here
		// the token's rows here: lane j < K looks at slot j
		int pj = -1;
		if (lane < K) {
			const int ej = __ldcg(ep_ptr<int>(v, s, v.off_topk) + token * K + lane) - fe;
			if (ej >= 0 && ej < v.n_local) {
				const int seg = ej * v.n_ranks + s;
				const int q = s_base[seg] + (__ldcg(ep_ptr<int>(v, s, v.off_inv) + token * K + lane) - s_src[seg]);
				if (q >= s_base[seg] && q < s_base[seg + 1])
					pj = q;
				else
					atomicOr(status, ST_BAD_TILE);
			}
		}
		const unsigned mine = __ballot_sync(0xffffffffu, pj >= 0);
		// the token: slot s of this rank's x_all, where rank s has stored its tokens
		const float4 *xr = reinterpret_cast<const float4 *>(ep_ptr<float>(v, v.rank, v.off_xall) + ((size_t)s * v.t_max + token) * H);
		for (int c0 = 0; c0 < H / 4; c0 += 32 * EP_SPLIT_F4) {
			float4 x4[EP_SPLIT_F4];
#pragma unroll
			for (int i = 0; i < EP_SPLIT_F4; i++) {
				const int c = c0 + i * 32 + lane;
				x4[i] = c < H / 4 ? __ldcg(xr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
			}
#pragma unroll
			for (int i = 0; i < EP_SPLIT_F4; i++) {
				const int c = c0 + i * 32 + lane;  // float4 index; k = 4 c
				const __half2 h0 = __floats2half2_rn(x4[i].x, x4[i].z), h1 = __floats2half2_rn(x4[i].y, x4[i].w);
				const float2 f0 = __half22float2(h0), f1 = __half22float2(h1);
				const __half2 l0 = __floats2half2_rn(x4[i].x - f0.x, x4[i].z - f0.y);
				const __half2 l1 = __floats2half2_rn(x4[i].y - f1.x, x4[i].w - f1.y);
				const uint2 hv = make_uint2(*reinterpret_cast<const uint32_t *>(&h0), *reinterpret_cast<const uint32_t *>(&h1));
				const uint2 lv = make_uint2(*reinterpret_cast<const uint32_t *>(&l0), *reinterpret_cast<const uint32_t *>(&l1));
				float sum = (x4[i].x + x4[i].y) + (x4[i].z + x4[i].w);
				sum += __shfl_xor_sync(0xffffffffu, sum, 1);
				sum += __shfl_xor_sync(0xffffffffu, sum, 2);
				sum += __shfl_xor_sync(0xffffffffu, sum, 4);
				const __half sh = __float2half_rn(sum);
				const __half sl = __float2half_rn(sum - __half2float(sh));
				for (unsigned m = mine; m; m &= m - 1u) {
					const size_t q = (size_t)__shfl_sync(0xffffffffu, pj, __ffs(m) - 1);
					if (c < H / 4) {
						reinterpret_cast<uint2 *>(hi + q * H)[c] = hv;
						reinterpret_cast<uint2 *>(lo + q * H)[c] = lv;
						if (q_hi && (lane & 7) == 0) {
							q_hi[q * q_cols + (c >> 3)] = sh;
							q_lo[q * q_cols + (c >> 3)] = sl;
						}
					}
				}
			}
		}
	}
}

// out[t] = (residual[t] +) sum_j w[t][j] * y[t*top_k + j], j ascending, fused multiply-add from
// zero — the arithmetic of combine_rows — once every owner has delivered (done flags).
__global__ void __launch_bounds__(256)
ep_combine_rows(EpView v, const unsigned *__restrict__ step_dev, long long budget, int n_tokens,
		const float *__restrict__ topk_w, const float *__restrict__ residual, float *__restrict__ out,
		unsigned *__restrict__ status)
{
	const int t = blockIdx.x, K = v.top_k, H = v.hidden;
	const unsigned step = *step_dev;
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
	const float *y = ep_ptr<float>(v, v.rank, v.off_y) + (size_t)t * K * H;
	float wj[MAX_TOP_K];
#pragma unroll
	for (int j = 0; j < MAX_TOP_K; j++)
		wj[j] = j < K ? topk_w[(size_t)t * K + j] : 0.f;
	for (int k = threadIdx.x * 4; k < H; k += blockDim.x * 4) {
		float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
		for (int j = 0; j < MAX_TOP_K; j++) {
			if (j < K) {
				const float4 y4 = __ldcg(reinterpret_cast<const float4 *>(y + (size_t)j * H + k));
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

int launch_ep_signal(tie_cuda_ctx *c, int which)
{
	ep_signal<<<1, 32, 0, c->stream>>>(c->ep.view, which, c->ep.step_dev);
	TIE_CUDA_LAUNCHED(c);
	return TIE_CUDA_OK;
}

EpPush ep_push_args(tie_cuda_ctx *c, const float *x, int n_tokens)
{
	EpPush f;
	f.v = c->ep.view;
	f.x = x;
	f.n_tokens = n_tokens;
	f.n_ctas = 0;
	return f;
}

int launch_ep_push_tokens(tie_cuda_ctx *c, const float *x, int n_tokens)
{
	if (n_tokens <= 0)
		return TIE_CUDA_OK;
	ep_push_tokens<<<c->sm_count, EP_PUSH_THREADS, 0, c->stream>>>(ep_push_args(c, x, n_tokens));
	TIE_CUDA_LAUNCHED(c);
	return TIE_CUDA_OK;
}

int launch_ep_index(tie_cuda_ctx *c)
{
	Scratch &s = c->s;
	const EpView &v = c->ep.view;
	const size_t smem = ((size_t)2 * v.n_ranks * v.n_expert + v.n_expert + 1) * sizeof(int);
	ep_index<<<1, EP_INDEX_THREADS, smem, c->stream>>>(v, c->ep.step_dev, c->ep.wait_cycles, TC_TOKEN_TILE, s.counts, s.offsets, s.tile_start,
							   s.tile_info, s.active, s.n_active, c->ep.n_rows, c->ep.seg_base,
							   c->ep.seg_src, s.status);
	TIE_CUDA_LAUNCHED(c);
	return TIE_CUDA_OK;
}

int launch_ep_split_rows(tie_cuda_ctx *c, bool sums)
{
	Scratch &s = c->s;
	ep_split_rows<<<c->sm_count * 8, EP_SPLIT_THREADS, 0, c->stream>>>(c->ep.view, c->ep.n_rows, c->ep.seg_base, c->ep.seg_src,
									    s.xs_hi, s.xs_lo, sums ? s.xq_hi : nullptr,
									    sums ? s.xq_lo : nullptr, xq_cols(c->cfg.hidden), c->ep.row_dst,
									    s.status);
	TIE_CUDA_LAUNCHED(c);
	return TIE_CUDA_OK;
}

int launch_ep_combine(tie_cuda_ctx *c, int n_tokens, const float *residual, float *out)
{
	Scratch &s = c->s;
	ep_combine_rows<<<n_tokens > 0 ? n_tokens : 1, 256, 0, c->stream>>>(c->ep.view, c->ep.step_dev, c->ep.wait_cycles, n_tokens,
									     s.topk_w, residual, out, s.status);
	TIE_CUDA_LAUNCHED(c);
	return TIE_CUDA_OK;
}

}  // namespace tie
