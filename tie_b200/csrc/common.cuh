// Shared internals of the tie_cuda library (sm_100a only).
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <mutex>

#include "../../include/tie_cuda.h"

namespace tie {

constexpr int QK_K = 256;	  // gguf.h:100
constexpr int Q4K_BYTES = 144;	  // sizeof(block_q4_k), gguf.h:108-113
constexpr int Q6K_BYTES = 210;	  // sizeof(block_q6_k), gguf.h:101-106
constexpr int MAX_TOP_K = 8;
constexpr int TC_TOKEN_TILE = 64;  // rows of one expert per token tile of the tensor-core path
constexpr int SILU_N = TIE_CUDA_SILU_TABLE_SIZE;
constexpr int SORT_SLICE = 256;   // rows per CTA of the dispatch sort

// Device status word bits (set by kernels instead of trapping).
constexpr unsigned ST_BAD_EXPERT = 1u;	  // expert id outside this context's range
constexpr unsigned ST_WAIT_TIMEOUT = 2u;  // a bounded mbarrier wait gave up
constexpr unsigned ST_BAD_TILE = 4u;	  // tile bookkeeping out of range

// Weight storage kinds on the device.
//  Q4_K is kept byte-for-byte as in the GGUF (144-byte blocks are 16-byte aligned).
//  Q6_K is re-ordered at upload into groups of 8 rows ("R8", see repack.cu): same byte
//  count, 208-byte (row, block) records with every 48-byte quant chunk 16-byte aligned.
enum WKind : int { W_Q4K = 0, W_Q6K_R8 = 1 };

// A stand-alone (dense) tensor's view of the context's split-operand scratch, with row length k.
struct DenseView {
	CUtensorMap full[6], half[6];  // [0-2] operand boxes of 16/32/64 rows, [3-5] sub-block sums; (hi, lo) in one box / one half per box
	size_t rows = 0;	       // rows the view holds
	size_t lo_off = 0, q_lo_off = 0;  // element offsets of the lo halves behind the hi halves
};

struct DevTensor {
	uint8_t *ptr = nullptr;	 // device
	int ggml_type = -1;
	WKind kind = W_Q4K;
	int rows = 0;		 // output rows per expert
	int k = 0;		 // input dim
	size_t expert_stride = 0;  // bytes per expert
	size_t bytes = 0;
	const void *host_ptr = nullptr;	 // for the dispatch-row registry
	CUtensorMap map;	 // Q4_K: byte map for the tensor-core path's weight loader
	bool has_map = false;
	DenseView *view = nullptr;  // stand-alone tensors only (owned)
};

struct Layer {
	bool uploaded = false;
	float *router_w = nullptr;  // [E][H] f32
	float *norm_w = nullptr;    // [H] or null
	DevTensor gate, up, down;
	const void *router_host = nullptr;
};

// Weights of one layer as the one-token decode kernel reads them when it walks a stack of layers
// (device pointers; one entry per layer in the context's device table).
struct DfLayer {
	const uint8_t *wg, *wu, *wd;
	const float *router_w;
	const float *norm_w;  // or null: weight 1
};

// Scratch arena of one context, sized for max_tokens.
struct Scratch {
	float *x = nullptr;	    // [T][H]   staged input (host mode) / normed input (block mode)
	float *out = nullptr;	    // [T][H]   staged output
	float *logits = nullptr;    // [T][E]
	float *bias = nullptr;	    // [E]
	int *topk_idx = nullptr;    // [T][K]
	float *topk_w = nullptr;    // [T][K]
	int *counts = nullptr;	    // [E]
	int *offsets = nullptr;	    // [E+1]
	int *tile_start = nullptr;  // [E+1]
	int4 *tile_info = nullptr;  // [E + R/TC_TOKEN_TILE + 1]  token tiles: (expert, first sorted row, rows, 0)
	int *active = nullptr;	    // [E]  compact list of experts with rows
	int *n_active = nullptr;    // [1]
	int *perm = nullptr;	    // [R]  sorted position -> row id
	int *sort_hist = nullptr;   // [slices][experts] rows per (slice of SORT_SLICE rows, expert)
	size_t sort_hist_cap = 0;
	float *h = nullptr;	    // [R][F]  fp32 activations (stream path), sorted order
	float *y = nullptr;	    // [R][H]  per-row expert outputs, row-id order
	__half *xs_hi = nullptr, *xs_lo = nullptr;  // [Rpad][H]  split inputs, sorted order
	__half *hs_hi = nullptr, *hs_lo = nullptr;  // [Rpad][F]
	// sums of the rows above over 32-wide sub-blocks, split the same way; 64 columns per 2048 k
	__half *xq_hi = nullptr, *xq_lo = nullptr;  // [Rpad][xq_cols(H)]
	__half *hq_hi = nullptr, *hq_lo = nullptr;  // [Rpad][xq_cols(F)]
	unsigned *status = nullptr;		    // [1]
	int *counter = nullptr;			    // [1] last-CTA counter of the fused decode router (zero at rest)
	unsigned *dec_sync = nullptr;		    // [2] arrivals and epoch of the one-kernel decode step's grid barriers
	int *row_expert = nullptr;		    // [R] staging for expert_rows
	// expert-parallel dispatch state (sort of this rank's rows over ALL experts)
	int *ep_counts = nullptr, *ep_offsets = nullptr, *ep_tile_start = nullptr, *ep_active = nullptr, *ep_n_active = nullptr;
	int *ep_perm = nullptr, *ep_inv = nullptr;
	size_t rows_cap = 0;			    // R capacity
	size_t rows_pad = 0;			    // Rpad
};

// Expert parallelism over peer memory (ep.cu).  EpView is what the kernels get by value.
constexpr int EP_MAX_RANKS = 16;
// Bit of an entry of a rank's published row-id list: the row is the first of its token's rows (in
// slot order) that goes to the GPU that owns its expert — that GPU fetches the token once, for
// this row, and fills the token's other rows there from the same fetch.
constexpr int EP_FIRST_OF_TOKEN = 1 << 30;
struct EpView {
	uint8_t *peer[EP_MAX_RANKS];  // region base of every rank, as mapped into this process
	size_t off_xs, off_xall, off_ids, off_topk, off_inv, off_counts, off_cntall, off_pub, off_done, off_y;
	long long rows_cap;  // rows of this context's scratch (the worst case of one step)
	int n_ranks, rank, n_local, n_expert, top_k, hidden, t_max;
};
// Destinations of the down product's rows in an expert-parallel step (tensor.cu, PEER).
struct EpDst {
	float *y[EP_MAX_RANKS] = {nullptr};  // per rank: its [t_max * top_k][hidden] output rows
	const unsigned *row = nullptr;	     // per sorted row: (rank << 24) | row id at that rank
};
struct EpState {
	EpView view = {};
	uint8_t *region = nullptr;
	size_t region_bytes = 0;
	bool opened[EP_MAX_RANKS] = {false};  // mappings this context opened (CUDA IPC) and must close
	bool attached = false;
	unsigned *step_dev = nullptr;  // [1] number of the last published step (advanced on the device)
	int step_tokens = -1;	    // tokens of the step between publish and gather, else -1
	int phase = 0;		    // 0 idle, 1 published, 2 computed
	bool replicated = false;    // the step between publish and gather runs on tokens every rank holds (decode)
	const float *rep_x = nullptr;  // ... and these are they
	long long wait_cycles = 0;  // budget of every flag wait
	int *n_rows = nullptr, *seg_base = nullptr, *seg_src = nullptr;
	unsigned *row_dst = nullptr;  // [rows_cap] per sorted row: (source rank << 24) | its row id there
};

}  // namespace tie

struct tie_cuda_ctx {
	tie_cuda_config cfg;
	int device = 0;
	int sm_count = 0;
	bool coop_ok = false;  // cooperative launches available
	cudaStream_t own_stream = nullptr;
	cudaStream_t stream = nullptr;
	float *silu = nullptr;	// device [8192]
	tie::Layer *layers = nullptr;
	tie::DfLayer *df_table = nullptr;  // device [n_layers]: the layers' weight pointers (stack decode)
	tie::Scratch s;
	int first_expert = 0, n_local = 0;
	// pinned staging for host-pointer calls
	float *pin_x = nullptr, *pin_out = nullptr;
	int *pin_idx = nullptr;
	float *pin_w = nullptr, *pin_logits = nullptr;
	unsigned *pin_status = nullptr;
	// host-buffer calls in flight (tie_cuda_moe_ffn_submit / _wait): per slot a device copy of x and of
	// the result, a pinned status word and the events that order the copy streams with the compute stream
	struct Slot {
		float *x = nullptr, *out = nullptr;
		unsigned *pin_status = nullptr;
		cudaEvent_t in = nullptr, done = nullptr, outd = nullptr;
		bool busy = false;
	} slots[TIE_CUDA_N_SLOTS];
	cudaStream_t h2d_stream = nullptr, d2h_stream = nullptr;
	size_t weight_bytes = 0;
	uint64_t launches = 0;
	int last_direct_rows = -1;
	// optional per-phase timing (tie_cuda_set_profiling): events around the kernel groups of a call
	bool last_used_tc = false;
	bool prof_on = false;
	cudaEvent_t prof_ev[8] = {nullptr};
	bool prof_set[8] = {false};
	char cuda_err[1024] = {0};
	// tensor maps for the tcgen05 path: (x, h, sums of x, sums of h) x (16-, 32-, 64-row boxes)
	CUtensorMap tmap[12];
	CUtensorMap tmap_half[12];  // the same with boxes of one half (hi or lo): what a CTA of a pair fetches
	bool tmaps_ok = false;
	int tc_pairs = 0;	    // CTA pairs the device holds at once (0: the pair kernels are not used)
	bool tc_no_pair = false;    // this call asked for the single-CTA grouped GEMM (TIE_CUDA_PATH_NO_PAIR)
	// host registry for dispatch rows
	struct Reg {
		const void *host;
		size_t bytes;
		const uint8_t *dev;
		int type;
		tie::WKind kind;
		int rows, k;
		tie::DevTensor *dense;	// stand-alone quantised tensors: the view the tensor-core path takes (or null)
	} *regs = nullptr;
	int n_regs = 0, cap_regs = 0;
	// standalone tensors uploaded through tie_cuda_register_tensor
	uint8_t **extra = nullptr;
	int n_extra = 0, cap_extra = 0;
	// cache of instantiated CUDA graphs for calls made with TIE_CUDA_GRAPH
	struct GraphEntry {
		int kind, layer, n;
		const void *p0, *p1, *p2, *p3;
		unsigned flags;
		cudaGraphExec_t exec;
		uint64_t kernels;  // kernel launches recorded in the graph
		uint64_t stamp;
	} graphs[256];
	int n_graphs = 0;
	uint64_t graph_clock = 0;
	// small per-call device buffers for the dispatch rows
	float *row_x = nullptr, *row_o = nullptr;
	size_t row_cap = 0;
	std::mutex row_mutex;  // the dispatch rows may be called from several host threads at once
	tie::EpState ep;
};

namespace tie {

// ---- launch bookkeeping ----
#define TIE_CUDA_TRY(c, expr)                                                                    \
	do {                                                                                     \
		cudaError_t _e = (expr);                                                         \
		if (_e != cudaSuccess) {                                                         \
			snprintf((c)->cuda_err, sizeof((c)->cuda_err), "%s:%d %s: %s", __FILE__, \
				 __LINE__, #expr, cudaGetErrorString(_e));                       \
			return (_e == cudaErrorMemoryAllocation) ? TIE_CUDA_ENOMEM : TIE_CUDA_ECUDA; \
		}                                                                                \
	} while (0)

#define TIE_CUDA_LAUNCHED(c)                             \
	do {                                             \
		(c)->launches++;                         \
		TIE_CUDA_TRY(c, cudaGetLastError());     \
	} while (0)

// ---- device helpers ----
__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
	for (int o = 16; o > 0; o >>= 1)
		v += __shfl_xor_sync(0xffffffffu, v, o);
	return v;
}

// get_scale_min_k4 (math_scalar.c:91-100) on the 12 packed bytes held as three 32-bit words.
__device__ __forceinline__ void q4k_scale_min(const uint32_t sc[3], int j, int &s, int &m)
{
	// byte i of the 12-byte array = (sc[i/4] >> 8*(i%4)) & 0xff
	auto byte = [&](int i) -> uint32_t { return (sc[i >> 2] >> (8 * (i & 3))) & 0xffu; };
	if (j < 4) {
		s = byte(j) & 63;
		m = byte(j + 4) & 63;
	} else {
		s = (byte(j + 4) & 0xF) | ((byte(j - 4) >> 6) << 4);
		m = (byte(j + 4) >> 4) | ((byte(j) >> 6) << 4);
	}
}

// The reference's table-driven SwiGLU exactly as its AVX2 kernel evaluates it
// (math_avx2.c:908-950, built with -ffast-math: the division by 20 is a multiply by 0.05f):
// no range check — outside [-10,10] the first/last table segment is extrapolated.
__device__ __forceinline__ float swiglu_lut(const float *__restrict__ tab, float g, float u)
{
	float pos = __fmul_rn(__fmul_rn(__fadd_rn(g, 10.0f), 8191.0f), 0.05f);
	float r = rintf(pos);
	int idx;
	if (!(r >= -2147483648.0f && r < 2147483648.0f))
		idx = 0;  // cvtps2dq yields INT_MIN for NaN/out-of-range, which the clamp maps to 0
	else
		idx = (int)r;
	idx = max(0, min(idx, SILU_N - 2));
	float frac = __fsub_rn(pos, (float)idx);
	float y1 = tab[idx], y2 = tab[idx + 1];
	return __fmul_rn(__fmaf_rn(__fsub_rn(y2, y1), frac, y1), u);
}

// Columns of the sub-block-sum arrays for an input dim k: k/32 sums, padded to whole 64-wide tiles.
__host__ __device__ __forceinline__ int xq_cols(int k)
{
	return ((k / 32 + 63) / 64) * 64;
}

__device__ __forceinline__ float half_bits_to_float(uint32_t h16)
{
	return __half2float(__ushort_as_half((unsigned short)h16));
}

// Byte offset of (expert-local row, part) pieces in the Q6_K "R8" layout.
//   group g = row/8 holds 8 rows; nb = blocks per row.
//   [records: (r8, b) x 208 B][d: (r8, b) x 2 B]
//   record = [quant chunks: part x 48 B][scales: part x 4 B]
//   part = n*2 + l16  (n = 128-element half of the block, l16 = 16-wide slice of l)
//   chunk = ql[64n+16*l16 .. +16] | ql[64n+32+16*l16 .. +16] | qh[32n+16*l16 .. +16]
//   scales = scales[8n + l16 + {0,2,4,6}]
// Every 48-byte chunk is 16-byte aligned; the 208-byte records of one row are contiguous, so a
// (block, 8 rows, 16 groups) box of a 3-D tensor map fetches the packed weights of 128 rows with
// one TMA instruction, and 208 = 13 x 16 keeps 16-byte reads by consecutive rows conflict-free.
constexpr int Q6K_RECORD = 208;
__host__ __device__ __forceinline__ size_t q6k_r8_group_bytes(int nb)
{
	return (size_t)8 * nb * Q6K_BYTES;
}
__host__ __device__ __forceinline__ size_t q6k_r8_chunk_off(int nb, int r8, int b, int part)
{
	return (size_t)(r8 * nb + b) * Q6K_RECORD + (size_t)part * 48;
}
__host__ __device__ __forceinline__ size_t q6k_r8_scale_off(int nb, int r8, int b, int part)
{
	return (size_t)(r8 * nb + b) * Q6K_RECORD + 192 + (size_t)part * 4;
}
__host__ __device__ __forceinline__ size_t q6k_r8_d_off(int nb, int r8, int b)
{
	return (size_t)8 * nb * Q6K_RECORD + (size_t)(r8 * nb + b) * 2;
}

}  // namespace tie
