// Launch entry points of the kernel translation units (all enqueue on c->stream).
#pragma once
#include "common.cuh"

namespace tie {

// router.cu
struct EpPush;
int launch_router(tie_cuda_ctx *c, const float *x, const float *w, const float *bias, int n_tokens, float *logits,
		  int *topk_idx, float *topk_w, int lfm2 = 0, const EpPush *push = nullptr, bool *push_taken = nullptr);
int router_setup(tie_cuda_ctx *c);
int launch_router_decode_fused(tie_cuda_ctx *c, const float *x, const float *w, const float *bias, int n_tokens, float *logits,
			       int *topk_idx, float *topk_w);
// decode.cu
bool decode_supported(const tie_cuda_ctx *c, const Layer &L, int n_tokens);
// foreign_slots_ok: slots whose expert another rank owns are skipped instead of reported
int launch_decode_gate_up(tie_cuda_ctx *c, const Layer &L, const float *x, int n_tokens, bool foreign_slots_ok = false);
int launch_decode_down_peer(tie_cuda_ctx *c, const Layer &L, int n_tokens);
int launch_decode_down_combine(tie_cuda_ctx *c, const Layer &L, int n_tokens, const float *residual, float *out);
int launch_router_rows(tie_cuda_ctx *c, const float *x, const float *w, int n_rows, int in_dim, float *out);
// decode_fused.cu
bool decode_fused_supported(tie_cuda_ctx *c, const Layer &L, int n_tokens);
int launch_decode_fused(tie_cuda_ctx *c, const Layer &L, const float *x, const float *bias, const float *residual, float *out,
			const float *norm_w = nullptr, float norm_eps = -1.0f, const Layer *next = nullptr);
int launch_decode_fused_stack(tie_cuda_ctx *c, int layer, int n_layers, float *hidden);
// sort.cu
struct SortBufs {
	int *counts, *offsets, *tile_start, *active, *n_active, *perm;
	int4 *tile_info;  // optional: one entry per token tile (expert, first sorted row, rows, 0)
	// optional (expert-parallel publish): inv[row id] = where the row stands in perm, and, with
	// owner_div = experts per GPU and top_k > 0, EP_FIRST_OF_TOKEN set in the entries of perm
	int *inv = nullptr;
	int owner_div = 0, top_k = 0;
};
int launch_sort(tie_cuda_ctx *c, const int *row_expert, int n_rows, int n_tile);
int launch_sort(tie_cuda_ctx *c, const int *row_expert, int n_rows, int n_tile, int first_expert, int n_expert,
		const SortBufs &b);
// stream.cu
int launch_stream_gate_up(tie_cuda_ctx *c, const Layer &L, const float *xin, int src_div, const int *row_expert,
			  int n_rows, int direct);
int launch_stream_down(tie_cuda_ctx *c, const Layer &L, float *y, const int *row_expert, int n_rows, int direct);
int launch_stream_matvec(tie_cuda_ctx *c, const uint8_t *wexp, WKind kind, int k, int rows_total, const float *x, float *o);
// misc.cu
int launch_rms_norm(tie_cuda_ctx *c, const float *x, const float *w, float *o, int n_tokens);
int launch_combine(tie_cuda_ctx *c, const float *y, const float *topk_w, int n_tokens, const float *residual, float *out,
		   const int *pos = nullptr);
int launch_gather_rows(tie_cuda_ctx *c, const float *x, const int *row_expert, const int *perm, int src_div, int n_rows,
		       float *rows_out, int *expert_out, int *inv);
int launch_split_rows(tie_cuda_ctx *c, const float *x, const int *perm, int src_div, int n_rows, int n_cols, __half *hi,
		      __half *lo, __half *q_hi, __half *q_lo);
int launch_swiglu(tie_cuda_ctx *c, float *gate, const float *up, int n);
// n_rows_dev != null: the row count is read on the device and n_rows CTAs stride over the rows
int launch_swiglu_split(tie_cuda_ctx *c, const float *gu, int n_rows, int ffn, float scale, __half *hi, __half *lo, __half *q_hi,
			__half *q_lo, const int *n_rows_dev = nullptr);
// tensor.cu
int tc_setup(tie_cuda_ctx *c);
int tc_make_weight_map(tie_cuda_ctx *c, DevTensor &t, int n_experts = -1);  // default: the context's local experts
bool tc_dense_supported(const tie_cuda_ctx *c, const DevTensor &t);
int tc_make_dense_view(tie_cuda_ctx *c, DevTensor &t);
int launch_tc_dense(tie_cuda_ctx *c, const DevTensor &t, float *y);
bool tc_supported(const tie_cuda_ctx *c, const Layer &L);
int launch_tc_gate_up(tie_cuda_ctx *c, const Layer &L, int n_rows);
int launch_tc_swiglu(tie_cuda_ctx *c, const Layer &L, int n_rows, const int *n_rows_dev = nullptr);
// sorted_out: y[p] instead of y[perm[p]]
int launch_tc_down(tie_cuda_ctx *c, const Layer &L, int n_rows, float *y, bool sorted_out = false);
int launch_tc_down_peer(tie_cuda_ctx *c, const Layer &L, const EpDst &dst);
// ep.cu
int launch_ep_signal(tie_cuda_ctx *c, int which);
int launch_ep_push_tokens(tie_cuda_ctx *c, const float *x, int n_tokens);
EpPush ep_push_args(tie_cuda_ctx *c, const float *x, int n_tokens);  // (ep_dev.cuh defines EpPush)
int launch_ep_index(tie_cuda_ctx *c);
int launch_ep_split_rows(tie_cuda_ctx *c, bool sums);
int launch_ep_combine(tie_cuda_ctx *c, int n_tokens, const float *residual, float *out);
// repack.cu
int launch_repack_q6k_r8(tie_cuda_ctx *c, const uint8_t *raw, uint8_t *dst, size_t n_rows_total, int nb);

}  // namespace tie
