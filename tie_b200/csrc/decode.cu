// Decode path (1-4 tokens): the expert mat-vecs with each CTA's whole weight tile staged in
// shared memory by bulk asynchronous copies.
//
// Reference: process_expert_task (engine.c:916-964) for the 8 selected experts of a token and the
// weighted combine (model_qwen3.c:458-467).  At batch 1 the block is a pure stream of 25.5 MB of
// packed weights, so the only thing that matters is how many bytes are in flight: a CTA issues
// ONE bulk copy per weight matrix for its complete row tile (the rows of a tile are contiguous
// in the GGUF layout; up to ~110 KB per CTA, all outstanding at once), stages the activation
// while the copy flies, waits on the mbarrier and then reduces from shared memory with the same
// per-lane block algebra as the streaming kernels (partdot.cuh).
//
//   decode_gate_up       CTA = ((token, slot), row tile): gate and up tiles -> SwiGLU -> h
//   decode_down_combine  CTA = (token, 16-row tile): the tiles of ALL the token's experts are
//                        fetched at once; rows are reduced slot by slot and accumulated as
//                        acc = fma(w_j, row_j, acc), j ascending from zero — the reference's
//                        combine — so no per-slot output and no separate combine pass exist.
#include "common.cuh"
#include "kernels.cuh"
#include "partdot.cuh"
#include "tc_ptx.cuh"
#include "decode_common.cuh"

namespace tie {

constexpr int DEC_MAX_CHUNKS = 8;

template <WKind KIND, int K>
__global__ void __launch_bounds__(DEC_GU_THREADS, 1)
decode_gate_up(const uint8_t *__restrict__ wg, const uint8_t *__restrict__ wu, size_t expert_stride, int rows_per_expert,
	       int rows_per_tile, const float *__restrict__ x, int top_k, const int *__restrict__ topk_idx, float *__restrict__ h,
	       int first_expert, int n_local, const float *__restrict__ silu, unsigned *__restrict__ status, int n_expert_all)
{
	constexpr int PARTS = K / 64;
	constexpr int LPR = PARTS > 16 ? 32 : (PARTS > 8 ? 16 : (PARTS > 4 ? 8 : 4));
	constexpr int RPW = 32 / LPR;
	constexpr int NB = K / QK_K;
	constexpr int ROWS_PER_PASS = (DEC_GU_THREADS / 32) * RPW;
	constexpr int CH = ROWS_PER_PASS > 16 ? ROWS_PER_PASS : 16;  // rows per copy chunk (own barrier): a pass never spans two
	extern __shared__ __align__(128) uint8_t dsm[];
	__shared__ uint64_t bar[DEC_MAX_CHUNKS];
	const int slot = blockIdx.y;  // (token, j)
	const int r0 = blockIdx.x * rows_per_tile;
	const int r1 = min(r0 + rows_per_tile, rows_per_expert);
	const int n_chunks = (r1 - r0 + CH - 1) / CH;
	if (threadIdx.x == 0) {
		for (int c = 0; c < n_chunks; c++)
			ptx::mbar_init(ptx::smem_u32(&bar[c]), 1);
		ptx::fence_barrier_init();
		ptx::fence_proxy_async_smem();
	}
	pdl_wait();	// the router's top-k (and x) are visible from here on
	pdl_trigger();	// the down kernel may start fetching its weights
	const int ge = topk_idx[slot];
	const int le = ge - first_expert;
	if (le < 0 || le >= n_local) {
		// n_expert_all > 0 (expert-parallel decode on replicated tokens): the slot belongs to another rank
		if (!(n_expert_all > 0 && ge >= 0 && ge < n_expert_all) && threadIdx.x == 0 && blockIdx.x == 0)
			atomicOr(status, ST_BAD_EXPERT);
		return;
	}
	const uint32_t tile_bytes = (uint32_t)(tile_offset<KIND>(NB, r1) - tile_offset<KIND>(NB, r0));
	uint8_t *sg = dsm, *su = dsm + tile_bytes;
	float *xs = reinterpret_cast<float *>(dsm + 2 * (size_t)tile_bytes);
	if (threadIdx.x == 0) {
		const size_t base = (size_t)le * expert_stride;
		for (int c = 0; c < n_chunks; c++) {
			const int c0 = r0 + c * CH, c1 = min(c0 + CH, r1);
			const size_t o0 = tile_offset<KIND>(NB, c0), o1 = tile_offset<KIND>(NB, c1);
			const uint32_t bytes = (uint32_t)(o1 - o0), rel = (uint32_t)(o0 - tile_offset<KIND>(NB, r0));
			const uint32_t ba = ptx::smem_u32(&bar[c]);
			ptx::mbar_arrive_expect_tx(ba, 2 * bytes);
			bulk_g2s(ptx::smem_u32(sg + rel), wg + base + o0, bytes, ba);
			bulk_g2s(ptx::smem_u32(su + rel), wu + base + o0, bytes, ba);
		}
	}
	const float *xrow = x + (size_t)(slot / top_k) * K;
	stage_x_lane_major<KIND, LPR>(xrow, xs, PARTS, threadIdx.x, DEC_GU_THREADS);
	__syncthreads();  // also publishes the barrier initialisation
	const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
	const int sub = lane / LPR, part = lane % LPR;
	const bool lane_on = part < PARTS;
	float xr[64], sx[4];
	if (lane_on)
		load_x_lane_major<KIND, LPR>(xs, part, xr, sx);
	// PartDot addresses rows from the start of an expert: shift the tile bases accordingly
	const uint8_t *vg = sg - tile_offset<KIND>(NB, r0), *vu = su - tile_offset<KIND>(NB, r0);
	float *hrow = h + (size_t)slot * rows_per_expert;
	int waited = -1;
	// (the SwiGLU table look-ups of all passes go out together at the end: lane p of a row keeps the
	// sums of pass p, which every lane of the row holds after the reduction)
	const bool defer = (r1 - r0 + ROWS_PER_PASS - 1) / ROWS_PER_PASS <= LPR;
	float keep_g = 0.f, keep_u = 0.f;
	int keep_row = -1, pass = 0;
	for (int rp = r0; rp < r1; rp += ROWS_PER_PASS, pass++) {
		const int chunk = (rp - r0) / CH;
		if (chunk != waited) {	// rows of a pass share a chunk; chunks arrive in order
			if (!dec_wait(ptx::smem_u32(&bar[chunk]), status))
				return;
			waited = chunk;
		}
		const int row = rp + warp * RPW + sub;
		float vgv = 0.f, vuv = 0.f;
		if (lane_on && row < r1) {
			vgv = PartDot<KIND>::dot(PartDot<KIND>::template load<true>(vg, NB, row, part), part, xr, sx);
			vuv = PartDot<KIND>::dot(PartDot<KIND>::template load<true>(vu, NB, row, part), part, xr, sx);
		}
#pragma unroll
		for (int o = LPR / 2; o > 0; o >>= 1) {
			vgv += __shfl_xor_sync(0xffffffffu, vgv, o);
			vuv += __shfl_xor_sync(0xffffffffu, vuv, o);
		}
		if (defer) {
			if (part == pass && row < r1) {
				keep_g = vgv;
				keep_u = vuv;
				keep_row = row;
			}
		} else if (part == 0 && row < r1) {
			hrow[row] = swiglu_lut(silu, vgv, vuv);
		}
	}
	if (keep_row >= 0)
		hrow[keep_row] = swiglu_lut(silu, keep_g, keep_u);
}

template <WKind KIND, int K>
__global__ void __launch_bounds__(DEC_THREADS, 1)
decode_down_combine(const uint8_t *__restrict__ wd, size_t expert_stride, int rows_per_expert, int rows_per_tile,
		    const float *__restrict__ h, int top_k, const int *__restrict__ topk_idx, const float *__restrict__ topk_w,
		    const float *__restrict__ residual, float *__restrict__ out, int first_expert, int n_local,
		    unsigned *__restrict__ status)
{
	constexpr int PARTS = K / 64;
	constexpr int LPR = PARTS > 16 ? 32 : (PARTS > 8 ? 16 : (PARTS > 4 ? 8 : 4));
	constexpr int RPW = 32 / LPR;
	constexpr int NB = K / QK_K;
	constexpr int ROWS_PER_PASS = (DEC_THREADS / 32) * RPW;
	constexpr int MAX_PASSES = 4;
	constexpr int XS_T = LPR * 64;	// floats of one lane-major activation row
	extern __shared__ __align__(128) uint8_t dsm[];
	__shared__ uint64_t bar[MAX_TOP_K];  // one per slot: a slot's rows are reduced as soon as its tile lands
	__shared__ int s_le[MAX_TOP_K];
	__shared__ float s_w[MAX_TOP_K];
	const int t = blockIdx.y;
	const int r0 = blockIdx.x * rows_per_tile;
	const int r1 = min(r0 + rows_per_tile, rows_per_expert);
	const uint32_t tile_bytes = (uint32_t)(tile_offset<KIND>(NB, r1) - tile_offset<KIND>(NB, r0));
	float *hs = reinterpret_cast<float *>(dsm + (size_t)top_k * tile_bytes);  // two lane-major rows (double buffer)
	// The selection was written two kernels ago and the weights never change: the tiles of all the
	// token's experts are requested BEFORE waiting for the gate/up kernel, so this fetch overlaps it.
	if (threadIdx.x == 0) {
		for (int j = 0; j < top_k; j++)
			ptx::mbar_init(ptx::smem_u32(&bar[j]), 1);
		ptx::fence_barrier_init();
		ptx::fence_proxy_async_smem();
		bool bad = false;
		for (int j = 0; j < top_k; j++) {
			const int le = topk_idx[t * top_k + j] - first_expert;
			s_le[j] = le;
			s_w[j] = topk_w[t * top_k + j];
			bad |= (le < 0 || le >= n_local);
		}
		if (bad) {
			s_le[0] = -1;
			if (blockIdx.x == 0)
				atomicOr(status, ST_BAD_EXPERT);
		} else {
			for (int j = 0; j < top_k; j++) {
				const uint32_t ba = ptx::smem_u32(&bar[j]);
				ptx::mbar_arrive_expect_tx(ba, tile_bytes);
				bulk_g2s(ptx::smem_u32(dsm + (size_t)j * tile_bytes),
					 wd + (size_t)s_le[j] * expert_stride + tile_offset<KIND>(NB, r0), tile_bytes, ba);
			}
		}
	}
	pdl_wait();  // h of the gate/up kernel is visible from here on
	const float *hrow = h + (size_t)t * top_k * K;
	stage_x_lane_major<KIND, LPR>(hrow, hs, PARTS, threadIdx.x, DEC_THREADS);
	__syncthreads();
	if (s_le[0] < 0)
		return;
	const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
	const int sub = lane / LPR, part = lane % LPR;
	const bool lane_on = part < PARTS;
	float acc[MAX_PASSES];
#pragma unroll
	for (int p = 0; p < MAX_PASSES; p++)
		acc[p] = 0.f;
	for (int j = 0; j < top_k; j++) {
		float xr[64], sx[4];
		if (lane_on)
			load_x_lane_major<KIND, LPR>(hs + (size_t)(j & 1) * XS_T, part, xr, sx);
		if (j + 1 < top_k)  // next slot's activation into the other buffer (last read two slots ago)
			stage_x_lane_major<KIND, LPR>(hrow + (size_t)(j + 1) * K, hs + (size_t)((j + 1) & 1) * XS_T, PARTS, threadIdx.x, DEC_THREADS);
		if (!dec_wait(ptx::smem_u32(&bar[j]), status))
			return;
		const uint8_t *vd = dsm + (size_t)j * tile_bytes - tile_offset<KIND>(NB, r0);
		const float wj = s_w[j];
#pragma unroll
		for (int p = 0; p < MAX_PASSES; p++) {
			const int row = r0 + p * ROWS_PER_PASS + warp * RPW + sub;
			if (r0 + p * ROWS_PER_PASS >= r1)
				break;
			float v = 0.f;
			if (lane_on && row < r1)
				v = PartDot<KIND>::dot(PartDot<KIND>::template load<true>(vd, NB, row, part), part, xr, sx);
#pragma unroll
			for (int o = LPR / 2; o > 0; o >>= 1)
				v += __shfl_xor_sync(0xffffffffu, v, o);
			acc[p] = __fmaf_rn(wj, v, acc[p]);  // model_qwen3.c:458-467, slot order, from zero
		}
		__syncthreads();  // the staged row of slot j+1 is complete; buffer j&1 is free again
	}
#pragma unroll
	for (int p = 0; p < MAX_PASSES; p++) {
		const int row = r0 + p * ROWS_PER_PASS + warp * RPW + sub;
		if (part == 0 && row < r1 && r0 + p * ROWS_PER_PASS < r1) {
			float v = acc[p];
			if (residual)
				v = __fadd_rn(residual[(size_t)t * rows_per_expert + row], v);
			out[(size_t)t * rows_per_expert + row] = v;
		}
	}
}

// Expert-parallel decode on replicated tokens: every rank has routed the same tokens to the same
// experts; this rank reduces the down rows of the slots whose expert it owns and stores each
// unweighted row value into the y rows (token, slot) of EVERY rank's region (plain stores over
// NVLink, 64 bytes per tile, slot and rank).  The combine (ep_combine_rows) then runs on every rank
// over all slots in slot order — the reference's order (model_qwen3.c:458-467), so the result is
// bit-identical to the one-GPU decode kernels.  A peer's y rows of the previous step may only be
// overwritten once that peer has started this step (its pub flag): the CTA waits for all pub
// flags first (bounded; they are words of this rank's own region).
template <WKind KIND, int K>
__global__ void __launch_bounds__(DEC_THREADS, 1)
decode_down_peer(const uint8_t *__restrict__ wd, size_t expert_stride, int rows_per_expert, int rows_per_tile,
		 const float *__restrict__ h, int top_k, const int *__restrict__ topk_idx, const EpView v,
		 const unsigned *__restrict__ step_dev, long long budget, int first_expert, int n_local, unsigned *__restrict__ status)
{
	constexpr int PARTS = K / 64;
	constexpr int LPR = PARTS > 16 ? 32 : (PARTS > 8 ? 16 : (PARTS > 4 ? 8 : 4));
	constexpr int RPW = 32 / LPR;
	constexpr int NB = K / QK_K;
	constexpr int ROWS_PER_PASS = (DEC_THREADS / 32) * RPW;
	constexpr int MAX_PASSES = 4;
	extern __shared__ __align__(128) uint8_t dsm[];
	__shared__ uint64_t bar[MAX_TOP_K];
	__shared__ int s_le[MAX_TOP_K];
	const int t = blockIdx.y;
	const int r0 = blockIdx.x * rows_per_tile;
	const int r1 = min(r0 + rows_per_tile, rows_per_expert);
	const uint32_t tile_bytes = (uint32_t)(tile_offset<KIND>(NB, r1) - tile_offset<KIND>(NB, r0));
	float *hs = reinterpret_cast<float *>(dsm + (size_t)top_k * tile_bytes);
	if (threadIdx.x == 0) {
		for (int j = 0; j < top_k; j++)
			ptx::mbar_init(ptx::smem_u32(&bar[j]), 1);
		ptx::fence_barrier_init();
		ptx::fence_proxy_async_smem();
		bool bad = false;
		for (int j = 0; j < top_k; j++) {
			const int ge = topk_idx[t * top_k + j];
			const int le = ge - first_expert;
			bad |= (ge < 0 || ge >= v.n_expert);
			s_le[j] = (le >= 0 && le < n_local) ? le : -1;
		}
		if (bad) {
			for (int j = 0; j < top_k; j++)
				s_le[j] = -1;
			if (blockIdx.x == 0)
				atomicOr(status, ST_BAD_EXPERT);
		}
		for (int j = 0; j < top_k; j++) {
			if (s_le[j] < 0)
				continue;
			const uint32_t ba = ptx::smem_u32(&bar[j]);
			ptx::mbar_arrive_expect_tx(ba, tile_bytes);
			bulk_g2s(ptx::smem_u32(dsm + (size_t)j * tile_bytes), wd + (size_t)s_le[j] * expert_stride + tile_offset<KIND>(NB, r0),
				 tile_bytes, ba);
		}
	}
	pdl_wait();  // h of the gate/up kernel is visible from here on
	// every rank has started this step: its y rows of the previous step are combined and may be overwritten
	const unsigned step = *step_dev;
	bool ok = true;
	if ((int)threadIdx.x < v.n_ranks) {
		const unsigned *flag = reinterpret_cast<const unsigned *>(v.peer[v.rank] + v.off_pub) + threadIdx.x;
		const long long t0 = clock64();
		for (;;) {
			unsigned f;
			asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(f) : "l"(flag) : "memory");
			if ((int)(f - step) >= 0)
				break;
			if (clock64() - t0 > budget) {
				ok = false;
				break;
			}
			__nanosleep(100);
		}
	}
	ok = __syncthreads_and(ok);  // (also publishes the barrier initialisation and s_le)
	const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
	const int sub = lane / LPR, part = lane % LPR;
	const bool lane_on = part < PARTS;
	if (!ok && threadIdx.x == 0)
		atomicOr(status, ST_WAIT_TIMEOUT);
	for (int j = 0; j < top_k; j++) {
		if (s_le[j] < 0)
			continue;  // (uniform over the CTA)
		if (!ok) {  // leave, but not with copies in flight
			if (threadIdx.x == 0)
				dec_wait(ptx::smem_u32(&bar[j]), status);
			continue;
		}
		stage_x_lane_major<KIND, LPR>(h + (size_t)(t * top_k + j) * K, hs, PARTS, threadIdx.x, DEC_THREADS);
		__syncthreads();
		float xr[64], sx[4];
		if (lane_on)
			load_x_lane_major<KIND, LPR>(hs, part, xr, sx);
		if (!dec_wait(ptx::smem_u32(&bar[j]), status))
			ok = false;
		ok = __syncthreads_and(ok);  // hs is free again; a failed wait is seen by all
		if (!ok)
			continue;
		const uint8_t *vd = dsm + (size_t)j * tile_bytes - tile_offset<KIND>(NB, r0);
#pragma unroll
		for (int p = 0; p < MAX_PASSES; p++) {
			const int row = r0 + p * ROWS_PER_PASS + warp * RPW + sub;
			if (r0 + p * ROWS_PER_PASS >= r1)
				break;
			float val = 0.f;
			if (lane_on && row < r1)
				val = PartDot<KIND>::dot(PartDot<KIND>::template load<true>(vd, NB, row, part), part, xr, sx);
#pragma unroll
			for (int o = LPR / 2; o > 0; o >>= 1)
				val += __shfl_xor_sync(0xffffffffu, val, o);
			if (part == 0 && row < r1) {
				const size_t at = (size_t)(t * top_k + j) * rows_per_expert + row;
				for (int r = 0; r < v.n_ranks; r++)
					reinterpret_cast<float *>(v.peer[r] + v.off_y)[at] = val;
			}
		}
	}
}

// ---- host side ----

constexpr int DEC_MAX_SMEM = 200 * 1024;

template <WKind KIND>
static size_t row_bytes_of(int k)
{
	return (size_t)(k / QK_K) * (KIND == W_Q4K ? Q4K_BYTES : Q6K_BYTES);
}

template <WKind KIND, int K>
static int launch_dec_gu_t(tie_cuda_ctx *c, const Layer &L, const float *x, int n_rows, int n_expert_all)
{
	const int rows = L.gate.rows;
	const size_t rb = row_bytes_of<KIND>(K);
	int want_tiles = max(1, c->sm_count / max(1, n_rows));
	int rpt = (rows + want_tiles - 1) / want_tiles;
	rpt = ((rpt + 7) / 8) * 8;
	const int max_rpt = (int)(((DEC_MAX_SMEM - 2 * K * 4) / 2 / rb) / 8 * 8);
	rpt = max(8, min(rpt, max_rpt));
	const int tiles = (rows + rpt - 1) / rpt;
	rpt = min(rpt, 8 * 16);	 // at most DEC_MAX_CHUNKS copy chunks of 16 rows
	const size_t smem = 2 * (size_t)rpt * rb + (size_t)2 * K * 4;  // lane-major x needs LPR*64 <= 2K floats
	TIE_CUDA_TRY(c, cudaFuncSetAttribute(decode_gate_up<KIND, K>, cudaFuncAttributeMaxDynamicSharedMemorySize, DEC_MAX_SMEM));
	cudaLaunchConfig_t cfg = {};
	cfg.gridDim = dim3(tiles, n_rows);
	cfg.blockDim = dim3(DEC_GU_THREADS);
	cfg.dynamicSmemBytes = smem;
	cfg.stream = c->stream;
	cudaLaunchAttribute attr[1];
	attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
	attr[0].val.programmaticStreamSerializationAllowed = 1;
	cfg.attrs = attr;
	cfg.numAttrs = 1;
	TIE_CUDA_TRY(c, cudaLaunchKernelEx(&cfg, decode_gate_up<KIND, K>, (const uint8_t *)L.gate.ptr, (const uint8_t *)L.up.ptr,
					   L.gate.expert_stride, rows, rpt, x, c->cfg.top_k, (const int *)c->s.topk_idx, c->s.h,
					   c->first_expert, c->n_local, (const float *)c->silu, c->s.status, n_expert_all));
	c->launches++;
	return TIE_CUDA_OK;
}

template <WKind KIND, int K>
static int launch_dec_dn_t(tie_cuda_ctx *c, const Layer &L, int n_tokens, const float *residual, float *out)
{
	const int rows = L.down.rows, top_k = c->cfg.top_k;
	const size_t rb = row_bytes_of<KIND>(K);
	const int rpt = 16;
	const size_t smem = (size_t)top_k * rpt * rb + (size_t)2 * 2 * K * 4;  // weight tiles + two lane-major h rows
	if (smem > (size_t)DEC_MAX_SMEM)
		return TIE_CUDA_ENOTSUP;
	const int tiles = (rows + rpt - 1) / rpt;
	TIE_CUDA_TRY(c, cudaFuncSetAttribute(decode_down_combine<KIND, K>, cudaFuncAttributeMaxDynamicSharedMemorySize, DEC_MAX_SMEM));
	cudaLaunchConfig_t cfg = {};
	cfg.gridDim = dim3(tiles, n_tokens);
	cfg.blockDim = dim3(DEC_THREADS);
	cfg.dynamicSmemBytes = smem;
	cfg.stream = c->stream;
	cudaLaunchAttribute attr[1];
	attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
	attr[0].val.programmaticStreamSerializationAllowed = 1;
	cfg.attrs = attr;
	cfg.numAttrs = 1;
	TIE_CUDA_TRY(c, cudaLaunchKernelEx(&cfg, decode_down_combine<KIND, K>, (const uint8_t *)L.down.ptr, L.down.expert_stride, rows,
					   rpt, (const float *)c->s.h, top_k, (const int *)c->s.topk_idx, (const float *)c->s.topk_w,
					   residual, out, c->first_expert, c->n_local, c->s.status));
	c->launches++;
	return TIE_CUDA_OK;
}

template <WKind KIND, int K>
static int launch_dec_dn_peer_t(tie_cuda_ctx *c, const Layer &L, int n_tokens)
{
	const int rows = L.down.rows, top_k = c->cfg.top_k;
	const size_t rb = row_bytes_of<KIND>(K);
	const int rpt = 16;
	const size_t smem = (size_t)top_k * rpt * rb + (size_t)2 * 2 * K * 4;
	if (smem > (size_t)DEC_MAX_SMEM)
		return TIE_CUDA_ENOTSUP;
	const int tiles = (rows + rpt - 1) / rpt;
	TIE_CUDA_TRY(c, cudaFuncSetAttribute(decode_down_peer<KIND, K>, cudaFuncAttributeMaxDynamicSharedMemorySize, DEC_MAX_SMEM));
	cudaLaunchConfig_t cfg = {};
	cfg.gridDim = dim3(tiles, n_tokens);
	cfg.blockDim = dim3(DEC_THREADS);
	cfg.dynamicSmemBytes = smem;
	cfg.stream = c->stream;
	cudaLaunchAttribute attr[1];
	attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
	attr[0].val.programmaticStreamSerializationAllowed = 1;
	cfg.attrs = attr;
	cfg.numAttrs = 1;
	TIE_CUDA_TRY(c, cudaLaunchKernelEx(&cfg, decode_down_peer<KIND, K>, (const uint8_t *)L.down.ptr, L.down.expert_stride, rows, rpt,
					   (const float *)c->s.h, top_k, (const int *)c->s.topk_idx, c->ep.view,
					   (const unsigned *)c->ep.step_dev, c->ep.wait_cycles, c->first_expert, c->n_local, c->s.status));
	c->launches++;
	return TIE_CUDA_OK;
}

#define TIE_DEC_DIMS(X) X(256) X(512) X(768) X(1024) X(2048)

bool decode_supported(const tie_cuda_ctx *c, const Layer &L, int n_tokens)
{
	auto ok_dim = [](int k) { return k == 256 || k == 512 || k == 768 || k == 1024 || k == 2048; };
	return n_tokens <= 4 && L.gate.kind == L.up.kind && ok_dim(L.gate.k) && ok_dim(L.down.k) && L.down.rows % 16 == 0 &&
	       L.gate.rows % 8 == 0;
}

// x [n_tokens][hidden] -> h [(token, slot)][ffn] (sorted nowhere: rows are the top-k entries themselves)
int launch_decode_gate_up(tie_cuda_ctx *c, const Layer &L, const float *x, int n_tokens, bool foreign_slots_ok)
{
	const int n_rows = n_tokens * c->cfg.top_k;
	const int nea = foreign_slots_ok ? c->cfg.n_expert : 0;
	switch (L.gate.k) {
#define X(KK)                                                                                                   \
	case KK:                                                                                                \
		return L.gate.kind == W_Q4K ? launch_dec_gu_t<W_Q4K, KK>(c, L, x, n_rows, nea) : launch_dec_gu_t<W_Q6K_R8, KK>(c, L, x, n_rows, nea);
		TIE_DEC_DIMS(X)
#undef X
	default:
		return TIE_CUDA_ENOTSUP;
	}
}

// h -> out [n_tokens][hidden] (= residual + sum_j w_j * down_j(h_j))
int launch_decode_down_combine(tie_cuda_ctx *c, const Layer &L, int n_tokens, const float *residual, float *out)
{
	switch (L.down.k) {
#define X(KK)                                                                                                          \
	case KK:                                                                                                       \
		return L.down.kind == W_Q4K ? launch_dec_dn_t<W_Q4K, KK>(c, L, n_tokens, residual, out)                \
					    : launch_dec_dn_t<W_Q6K_R8, KK>(c, L, n_tokens, residual, out);
		TIE_DEC_DIMS(X)
#undef X
	default:
		return TIE_CUDA_ENOTSUP;
	}
}

// h (local slots) -> the y rows of every rank's region (expert-parallel decode on replicated tokens)
int launch_decode_down_peer(tie_cuda_ctx *c, const Layer &L, int n_tokens)
{
	switch (L.down.k) {
#define X(KK)                                                                                              \
	case KK:                                                                                           \
		return L.down.kind == W_Q4K ? launch_dec_dn_peer_t<W_Q4K, KK>(c, L, n_tokens) : launch_dec_dn_peer_t<W_Q6K_R8, KK>(c, L, n_tokens);
		TIE_DEC_DIMS(X)
#undef X
	default:
		return TIE_CUDA_ENOTSUP;
	}
}

}  // namespace tie
