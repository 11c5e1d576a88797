// Token-to-expert dispatch: a counting sort of rows by expert id, deterministic and without
// atomics on the output positions.
//
// The reference has no such step — it walks tokens one by one and fans the 8 selected experts
// out to 8 pool threads (model_qwen3.c:415-456).  Here all (token, slot) rows are grouped by
// expert so that each expert's weights are streamed once per call.
//
// The rows are cut into slices of SORT_SLICE rows, one CTA per slice, one row per thread; a warp
// finds the rows of equal expert among its 32 (match_any) and every row is read twice:
// Pass 1 (sort_hist): each CTA counts its slice's rows per expert (per-warp counters written by
//   one lane per expert, then plain sums) into hist[slice][expert].
// Pass 2 (sort_scatter): each CTA adds up the histograms — the rows of an expert in all slices
//   (its count), in the slices before its own (where its rows start inside the expert's range) —
//   scans the counts over the experts into offsets, and writes each row's id at offset + rows of
//   that expert in earlier slices, earlier warps and earlier lanes.  Rows of one expert keep their
//   original order (stable), so the result does not depend on scheduling.  The first CTA also
//   writes the tables the grouped products read (counts, offsets, token tiles).
// The depth of both passes does not grow with the row count (the previous form, one CTA per
// expert scanning all rows, grew with rows x experts per CTA).
#include "common.cuh"
#include "kernels.cuh"

namespace tie {

constexpr int SORT_THREADS = 256;
constexpr int SORT_WARPS = SORT_THREADS / 32;
static_assert(SORT_SLICE == SORT_THREADS, "one row per thread: a warp owns 32 consecutive rows of the slice");
constexpr int SORT_MAX_E = 256;

// The thread's row of the slice: its expert in local numbering, or -1 (no row / id out of range),
// the lanes of its warp that hold a row of the same expert (in row order: lane order), and, into
// cnt[warp][expert], how many rows of each expert the warp holds (written by one lane per expert:
// the counters of a warp are its own, nothing is added atomically).
__device__ __forceinline__ int sort_my_row(const int *__restrict__ row_expert, int n_rows, int first_expert, int n_local,
					   int (*cnt)[SORT_MAX_E], unsigned &same, unsigned *status)
{
	const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
	for (int i = threadIdx.x; i < SORT_WARPS * SORT_MAX_E; i += SORT_THREADS)
		(&cnt[0][0])[i] = 0;
	const int r = blockIdx.x * SORT_SLICE + threadIdx.x;
	int le = -1;
	if (r < n_rows) {
		le = row_expert[r] - first_expert;
		if (le < 0 || le >= n_local) {
			le = -1;
			if (status)
				atomicOr(status, ST_BAD_EXPERT);
		}
	}
	__syncthreads();
	same = __match_any_sync(0xffffffffu, le);
	if (le >= 0 && (same & ((1u << lane) - 1u)) == 0)  // the first lane of its group
		cnt[warp][le] = __popc(same);
	__syncthreads();
	return le;
}

__global__ void __launch_bounds__(SORT_THREADS) sort_hist(const int *__restrict__ row_expert, int n_rows, int first_expert,
							  int n_local, int *__restrict__ hist, unsigned *__restrict__ status)
{
	__shared__ int cnt[SORT_WARPS][SORT_MAX_E];
	unsigned same;
	sort_my_row(row_expert, n_rows, first_expert, n_local, cnt, same, status);
	const int e = threadIdx.x;
	if (e < n_local) {
		int t = 0;
#pragma unroll
		for (int w = 0; w < SORT_WARPS; w++)
			t += cnt[w][e];
		hist[(size_t)blockIdx.x * n_local + e] = t;
	}
}

__global__ void __launch_bounds__(SORT_THREADS) sort_scatter(const int *__restrict__ row_expert, int n_rows, int first_expert,
							     int n_local, const int *__restrict__ hist, int n_tile,
							     int *__restrict__ counts, int *__restrict__ offsets, int *__restrict__ tile_start,
							     int *__restrict__ active, int *__restrict__ n_active, int *__restrict__ perm,
							     int4 *__restrict__ tile_info, int *__restrict__ inv, int owner_div, int top_k)
{
	__shared__ int cnt[SORT_WARPS][SORT_MAX_E];  // rows of expert e in warp w's 32 rows; then: where they start
	__shared__ int wsum[3][SORT_WARPS];
	unsigned same;
	const int le = sort_my_row(row_expert, n_rows, first_expert, n_local, cnt, same, nullptr);
	const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
	const int e = threadIdx.x;  // thread e stands for expert e
	int total = 0, before = 0;
	if (e < n_local) {
		for (int b = 0; b < (int)gridDim.x; b++) {
			const int h = hist[(size_t)b * n_local + e];
			total += h;
			before += b < (int)blockIdx.x ? h : 0;
		}
	}
	// exclusive scans over the experts: rows, token tiles, experts with rows
	const int tl = (total + n_tile - 1) / n_tile, act = total > 0 ? 1 : 0;
	int v[3] = {total, tl, act}, incl[3];
#pragma unroll
	for (int k = 0; k < 3; k++) {
		incl[k] = v[k];
#pragma unroll
		for (int o = 1; o < 32; o <<= 1) {
			const int t = __shfl_up_sync(0xffffffffu, incl[k], o);
			if (lane >= o)
				incl[k] += t;
		}
		if (lane == 31)
			wsum[k][warp] = incl[k];
	}
	__syncthreads();
	int excl[3], all[3];
#pragma unroll
	for (int k = 0; k < 3; k++) {
		int bw = 0, a = 0;
#pragma unroll
		for (int i = 0; i < SORT_WARPS; i++) {
			const int w = wsum[k][i];
			bw += i < warp ? w : 0;
			a += w;
		}
		excl[k] = bw + incl[k] - v[k];
		all[k] = a;
	}
	if (e < n_local) {
		// first sorted position of warp w's rows of expert e: the expert's range, the slices before this
		// one, the warps before w
		int pos = excl[0] + before;
#pragma unroll
		for (int w = 0; w < SORT_WARPS; w++) {
			const int c = cnt[w][e];
			cnt[w][e] = pos;
			pos += c;
		}
	}
	if (blockIdx.x == 0) {
		if (e < n_local) {
			counts[e] = total;
			offsets[e] = excl[0];
			tile_start[e] = excl[1];
			if (total > 0)
				active[excl[2]] = e;
			if (tile_info)
				for (int j = 0; j * n_tile < total; j++)
					tile_info[excl[1] + j] = make_int4(e, excl[0] + j * n_tile, min(n_tile, total - j * n_tile), 0);
		}
		if (e == 0) {
			offsets[n_local] = all[0];
			tile_start[n_local] = all[1];
			*n_active = all[2];
		}
	}
	__syncthreads();
	if (le >= 0) {	// rows of one expert keep their order: slices, warps and lanes are all in row order
		const int r = blockIdx.x * SORT_SLICE + threadIdx.x;
		const int pos = cnt[warp][le] + __popc(same & ((1u << lane) - 1u));
		int entry = r;
		if (owner_div > 0) {
			// no earlier slot of the token has an expert of the same owner
			const int slot = r % top_k, owner = le / owner_div;
			bool first = true;
			for (int j = 0; j < slot; j++) {
				const int ej = row_expert[r - slot + j] - first_expert;
				first = first && !(ej >= 0 && ej < n_local && ej / owner_div == owner);
			}
			entry |= first ? EP_FIRST_OF_TOKEN : 0;
		}
		perm[pos] = entry;
		if (inv)
			inv[r] = pos;
	}
}

int launch_sort(tie_cuda_ctx *c, const int *row_expert, int n_rows, int n_tile, int first_expert, int n_expert,
		const SortBufs &b)
{
	if (n_expert > 256)
		return TIE_CUDA_ENOTSUP;
	const int n_slices = n_rows > 0 ? (n_rows + SORT_SLICE - 1) / SORT_SLICE : 1;  // (no rows: one CTA writes the empty tables)
	if ((size_t)n_slices * n_expert > c->s.sort_hist_cap)
		return TIE_CUDA_EINVAL;
	sort_hist<<<n_slices, SORT_THREADS, 0, c->stream>>>(row_expert, n_rows, first_expert, n_expert, c->s.sort_hist, c->s.status);
	TIE_CUDA_LAUNCHED(c);
	sort_scatter<<<n_slices, SORT_THREADS, 0, c->stream>>>(row_expert, n_rows, first_expert, n_expert, c->s.sort_hist, n_tile, b.counts,
								b.offsets, b.tile_start, b.active, b.n_active, b.perm, b.tile_info, b.inv,
								b.top_k > 0 ? b.owner_div : 0, b.top_k);
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
