// Token-to-expert dispatch: a counting sort of rows by expert id, deterministic and without
// atomics on the output positions.
//
// The reference has no such step — it walks tokens one by one and fans the 8 selected experts
// out to 8 pool threads (model_qwen3.c:415-456).  Here all (token, slot) rows are grouped by
// expert so that each expert's weights are streamed once per call.
//
// Pass 1 (grid = experts): each CTA counts the rows of its expert (ballot + popc, plain sums).
// Pass 2 (grid = experts): each CTA turns the counts into its exclusive offset (a warp scan over
// all experts — every CTA repeats it, it is 128 values), then walks the rows in order and writes
// its rows' ids at offset + rank, rank from a block-wide ballot prefix.  Rows of one expert keep
// their original order (stable), so the result does not depend on scheduling.
#include "common.cuh"
#include "kernels.cuh"

namespace tie {

constexpr int SORT_THREADS = 256;
constexpr int SORT_RPT = 8;  // rows per thread and chunk in sort_place

__global__ void __launch_bounds__(SORT_THREADS) sort_count(const int *__restrict__ row_expert, int n_rows, int first_expert,
							   int n_local, int *__restrict__ counts, unsigned *__restrict__ status)
{
	__shared__ int wsum[SORT_THREADS / 32];
	const int e = first_expert + blockIdx.x;
	int cnt = 0;
	bool bad = false;
	for (int r = threadIdx.x; r < n_rows; r += SORT_THREADS) {
		int re = row_expert[r];
		cnt += (re == e);
		if (blockIdx.x == 0 && (re < first_expert || re >= first_expert + n_local))
			bad = true;
	}
	if (bad)
		atomicOr(status, ST_BAD_EXPERT);
#pragma unroll
	for (int o = 16; o > 0; o >>= 1)
		cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
	if ((threadIdx.x & 31) == 0)
		wsum[threadIdx.x >> 5] = cnt;
	__syncthreads();
	if (threadIdx.x == 0) {
		int t = 0;
		for (int i = 0; i < SORT_THREADS / 32; i++)
			t += wsum[i];
		counts[blockIdx.x] = t;
	}
}

__global__ void __launch_bounds__(SORT_THREADS) sort_place(const int *__restrict__ row_expert, int n_rows, int first_expert,
							   int n_local, const int *__restrict__ counts, int n_tile,
							   int *__restrict__ offsets, int *__restrict__ tile_start,
							   int *__restrict__ active, int *__restrict__ n_active,
							   int *__restrict__ perm, int4 *__restrict__ tile_info)
{
	__shared__ int s_off, s_tiles;
	__shared__ int wcnt[SORT_THREADS / 32];
	const int le = blockIdx.x;
	const int e = first_expert + le;
	// exclusive prefix over experts < le, by warp 0 (n_local <= 256: 8 per lane)
	if (threadIdx.x < 32) {
		int off = 0, tiles = 0, act = 0, tot = 0, ttiles = 0, tact = 0;
		for (int i = threadIdx.x; i < n_local; i += 32) {
			int cnt = counts[i];
			int tl = (cnt + n_tile - 1) / n_tile;
			if (i < le) {
				off += cnt;
				tiles += tl;
				act += (cnt > 0);
			}
			tot += cnt;
			ttiles += tl;
			tact += (cnt > 0);
		}
#pragma unroll
		for (int o = 16; o > 0; o >>= 1) {
			off += __shfl_xor_sync(0xffffffffu, off, o);
			tiles += __shfl_xor_sync(0xffffffffu, tiles, o);
			act += __shfl_xor_sync(0xffffffffu, act, o);
			tot += __shfl_xor_sync(0xffffffffu, tot, o);
			ttiles += __shfl_xor_sync(0xffffffffu, ttiles, o);
			tact += __shfl_xor_sync(0xffffffffu, tact, o);
		}
		if (threadIdx.x == 0) {
			s_off = off;
			s_tiles = tiles;
			offsets[le] = off;
			tile_start[le] = tiles;
			if (counts[le] > 0)
				active[act] = le;
			if (le == n_local - 1) {
				offsets[n_local] = tot;
				tile_start[n_local] = ttiles;
				*n_active = tact;
			}
		}
	}
	__syncthreads();
	int base = s_off;
	if (tile_info) {  // the token tiles of this expert
		const int cnt = counts[le];
		for (int j = threadIdx.x; j * n_tile < cnt; j += SORT_THREADS)
			tile_info[s_tiles + j] = make_int4(le, base + j * n_tile, min(n_tile, cnt - j * n_tile), 0);
	}
	// each thread takes SORT_RPT consecutive rows of a chunk, so ranks follow the row order:
	// rank = rows of this expert in earlier chunks + in earlier threads (warp scan + warp totals)
	// + earlier ones among the thread's own
	const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
	constexpr int CHUNK = SORT_THREADS * SORT_RPT;
	for (int r0 = 0; r0 < n_rows; r0 += CHUNK) {
		const int rt = r0 + threadIdx.x * SORT_RPT;
		unsigned m = 0;
#pragma unroll
		for (int i = 0; i < SORT_RPT; i++)
			if (rt + i < n_rows && row_expert[rt + i] == e)
				m |= 1u << i;
		const int cnt = __popc(m);
		int incl = cnt;
#pragma unroll
		for (int o = 1; o < 32; o <<= 1) {
			const int v = __shfl_up_sync(0xffffffffu, incl, o);
			if (lane >= o)
				incl += v;
		}
		if (lane == 31)
			wcnt[warp] = incl;
		__syncthreads();
		int before = incl - cnt, total = 0;
#pragma unroll
		for (int i = 0; i < SORT_THREADS / 32; i++) {
			const int cw = wcnt[i];
			before += (i < warp) ? cw : 0;
			total += cw;
		}
		int pos = base + before;
#pragma unroll
		for (int i = 0; i < SORT_RPT; i++)
			if (m & (1u << i))
				perm[pos++] = rt + i;
		base += total;
		__syncthreads();
	}
}

int launch_sort(tie_cuda_ctx *c, const int *row_expert, int n_rows, int n_tile, int first_expert, int n_expert,
		const SortBufs &b)
{
	sort_count<<<n_expert, SORT_THREADS, 0, c->stream>>>(row_expert, n_rows, first_expert, n_expert, b.counts, c->s.status);
	TIE_CUDA_LAUNCHED(c);
	sort_place<<<n_expert, SORT_THREADS, 0, c->stream>>>(row_expert, n_rows, first_expert, n_expert, b.counts, n_tile,
							      b.offsets, b.tile_start, b.active, b.n_active, b.perm, b.tile_info);
	TIE_CUDA_LAUNCHED(c);
	return TIE_CUDA_OK;
}

int launch_sort(tie_cuda_ctx *c, const int *row_expert, int n_rows, int n_tile)
{
	Scratch &s = c->s;
	SortBufs b = {s.counts, s.offsets, s.tile_start, s.active, s.n_active, s.perm, s.tile_info};
	return launch_sort(c, row_expert, n_rows, n_tile, c->first_expert, c->n_local, b);
}

}  // namespace tie
