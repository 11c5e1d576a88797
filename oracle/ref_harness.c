/*
 * TEST INFRASTRUCTURE — not part of the product.
 *
 * Drives the reference's own compiled code through its Qwen3-MoE feed-forward
 * path.  The reference has no callable "MoE FFN" function: the path is inline
 * in transformer_layer_qwen3 (model_qwen3.c:403-471), which also needs
 * attention weights, a KV cache and RoPE tables.  This file restates ONLY the
 * per-token orchestration of that branch (the loop, the slot numbering, the
 * combine order) and calls the reference's functions for every arithmetic
 * step: dispatch_mat_vec, find_top_k, softmax, process_expert_task on the
 * reference's thread_pool, dispatch_convert, dispatch_rms_norm,
 * dispatch_apply_residual.  It is linked with the reference's objects (all
 * sources except main.c) into oracle/_ref/libtie_ref.so by oracle/Makefile.
 *
 * Only tests, the smoke check and the CPU-baseline leg of the benchmark load
 * that library.
 */
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>
#include <unistd.h>

#include "main.h"
#include "engine.h"
#include "math_dispatch.h"
#include "threadpool.h"

typedef struct {
	struct TIEContext ctx;
	Model model;
	LayerWeights layer;
	int hidden, n_expert, top_k, ffn_dim;
	int n_threads;
	int ready;
} ref_state_t;

static ref_state_t g;

/* The reference keeps these as process-wide singletons (threadpool.c:6, engine.c:12). */
static int g_global_init = 0;

int tieref_num_threads(void)
{
	return g.n_threads;
}

/* Mirrors engine_alloc (engine.c:14-44) for the parts this path needs, then the
 * MoE scratch allocation of model_init_mem_language (model.c:416-433). */
int tieref_init(int hidden, int n_expert, int top_k, int ffn_dim, int n_threads)
{
	if (n_threads < top_k)
		n_threads = top_k; /* tasks[num_threads] is indexed by slot j < top_k (model_qwen3.c:413,446) */
	if (n_threads > MAX_THREADS)
		n_threads = MAX_THREADS;
	if (!g_global_init) {
		thread_pool = thread_pool_create(n_threads);
		silu_table_init();
		math_dispatch_init();
		g_global_init = 1;
	}
	if (g.ready)
		return 0;
	memset(&g, 0, sizeof(g));
	g.n_threads = thread_pool->num_threads;
	g.hidden = hidden;
	g.n_expert = n_expert;
	g.top_k = top_k;
	g.ffn_dim = ffn_dim;
	g.model.embed_dim = hidden;
	g.model.expert_count = n_expert;
	g.model.expert_used_count = top_k;
	g.model.expert_ffn_dim = ffn_dim;
	g.model.is_moe = 1;
	g.model.num_layers = 1;
	g.model.norm_eps = 1e-6f;
	g.model.layers = &g.layer;
	g.ctx.model = &g.model;

	MemLayout *m = &g.ctx.mem;
	alloc_memtype(&m->expert_scores, GGML_TYPE_F32, n_expert);
	alloc_memtype(&m->expert_out_fp32, GGML_TYPE_F32, hidden);
	m->ffn_hidden1_scratch = calloc(n_expert, sizeof(MemType));
	m->ffn_hidden2_scratch = calloc(n_expert, sizeof(MemType));
	m->expert_outputs = calloc(n_expert, sizeof(MemType));
	for (int j = 0; j < top_k; j++) {
		alloc_memtype(&m->ffn_hidden1_scratch[j], GGML_TYPE_F32, ffn_dim);
		alloc_memtype(&m->ffn_hidden2_scratch[j], GGML_TYPE_F32, ffn_dim);
		alloc_memtype(&m->expert_outputs[j], GGML_TYPE_F32, hidden);
	}
	g.ready = 1;
	return 0;
}

void tieref_get_silu_table(float *out)
{
	memcpy(out, silu_table, sizeof(float) * SILU_TABLE_SIZE);
}

static void set_tensor(Tensor *t, const void *data, int type)
{
	memset(t, 0, sizeof(*t));
	t->mem.type = (GGMLType)type;
	t->mem.data = (void *)data;
}

void tieref_set_layer(const void *router_w, const void *gate, int gate_type, const void *up, int up_type,
		      const void *down, int down_type, const float *ffn_norm_w)
{
	set_tensor(&g.layer.ffn_gate_inp, router_w, GGML_TYPE_F32);
	set_tensor(&g.layer.ffn_gate_exps, gate, gate_type);
	set_tensor(&g.layer.ffn_up_exps, up, up_type);
	set_tensor(&g.layer.ffn_down_exps, down, down_type);
	set_tensor(&g.layer.ffn_norm, ffn_norm_w, GGML_TYPE_F32);
}

/*
 * The MoE branch, token by token (model_qwen3.c:415-470).  router_bias (may be
 * NULL) is added to the raw logits before find_top_k and feeds the softmax; the
 * Qwen3 path has no such bias — it exists for the skewed-load workload only.
 * Optional outputs: topk_idx / topk_w [T x top_k] in the reference's slot order
 * (descending score), logits [T x n_expert] (biased).
 */
int tieref_moe_ffn(const float *x, int n_tokens, const float *router_bias, float *out, int *topk_idx,
		   float *topk_w, float *logits)
{
	struct TIEContext *ctx = &g.ctx;
	LayerWeights *l = &g.layer;
	const int H = g.hidden, E = g.n_expert, K = g.top_k;

	size_t block_size_bytes = ggml_block_size(l->ffn_up_exps.mem.type);
	if (block_size_bytes == 0)
		return -1;

	expert_task_t tasks[MAX_THREADS];

	for (int i = 0; i < n_tokens; i++) {
		MemType xin = {.type = GGML_TYPE_F32, .data = (void *)(x + (size_t)i * H)};
		MemType oslice = {.type = GGML_TYPE_F32, .data = (void *)(out + (size_t)i * H)};
		float *acc = ctx->mem.expert_out_fp32.data;
		float *scores = ctx->mem.expert_scores.data;

		dispatch_mat_vec(ctx, &xin, &l->ffn_gate_inp, &ctx->mem.expert_scores, H, E, false);
		if (router_bias)
			for (int e = 0; e < E; e++)
				scores[e] += router_bias[e];
		if (logits)
			memcpy(logits + (size_t)i * E, scores, sizeof(float) * E);

		ExpertChoice top[K];
		find_top_k(scores, E, K, top);
		float gate[K];
		for (int j = 0; j < K; j++)
			gate[j] = top[j].score;
		softmax(gate, K);

		for (int j = 0; j < K; j++) {
			tasks[j] = (expert_task_t){
				.ctx = ctx, .thread_id = j, .layer_idx = 0, .expert_idx = top[j].index, .normed_input = xin};
			thread_pool_submit(thread_pool, process_expert_task, &tasks[j]);
		}
		thread_pool_wait(thread_pool);

		memset(acc, 0, sizeof(float) * H);
		for (int j = 0; j < K; j++) {
			float gv = gate[j];
			float *r = ctx->mem.expert_outputs[j].data;
			for (int k = 0; k < H; k++)
				acc[k] += gv * r[k];
		}
		dispatch_convert(&ctx->mem.expert_out_fp32, &oslice, H);

		if (topk_idx)
			for (int j = 0; j < K; j++)
				topk_idx[(size_t)i * K + j] = top[j].index;
		if (topk_w)
			for (int j = 0; j < K; j++)
				topk_w[(size_t)i * K + j] = gate[j];
	}
	return 0;
}

/* hidden += MoE(RMSNorm(hidden)) — model_qwen3.c:392-401, 403-471, 491.  normed (scratch,
 * [T x H]) and ffn_out ([T x H]) are caller buffers so the intermediate can be inspected. */
int tieref_moe_block_inplace(float *hidden, int n_tokens, float eps, float *normed, float *ffn_out, int *topk_idx,
			     float *topk_w)
{
	const int H = g.hidden;
	for (int i = 0; i < n_tokens; i++) {
		MemType hs = {.type = GGML_TYPE_F32, .data = hidden + (size_t)i * H};
		MemType ns = {.type = GGML_TYPE_F32, .data = normed + (size_t)i * H};
		dispatch_rms_norm(&hs, &g.layer.ffn_norm, &ns, H, eps);
	}
	int rc = tieref_moe_ffn(normed, n_tokens, NULL, ffn_out, topk_idx, topk_w, NULL);
	if (rc)
		return rc;
	MemType hall = {.type = GGML_TYPE_F32, .data = hidden};
	MemType fall = {.type = GGML_TYPE_F32, .data = ffn_out};
	dispatch_apply_residual(&hall, &fall, n_tokens * H);
	return 0;
}

/* Leaf operators exactly as the dispatch tables call them (math_dispatch.c:227-283, 510-528). */
void tieref_mat_vec(const float *x, const void *w, int w_type, float *o, int in_dim, int out_dim)
{
	MemType xin = {.type = GGML_TYPE_F32, .data = (void *)x};
	MemType oo = {.type = GGML_TYPE_F32, .data = o};
	Tensor t;
	set_tensor(&t, w, w_type);
	dispatch_mat_vec(&g.ctx, &xin, &t, &oo, in_dim, out_dim, false);
}

void tieref_swiglu(float *gate, const float *up, int size)
{
	MemType gm = {.type = GGML_TYPE_F32, .data = gate};
	MemType um = {.type = GGML_TYPE_F32, .data = (void *)up};
	dispatch_swiglu_activation(&gm, &um, size);
}

void tieref_rms_norm(const float *x, const float *w, float *o, int size, float eps)
{
	MemType xs = {.type = GGML_TYPE_F32, .data = (void *)x};
	MemType os = {.type = GGML_TYPE_F32, .data = o};
	Tensor t;
	set_tensor(&t, w, GGML_TYPE_F32);
	dispatch_rms_norm(&xs, &t, &os, size, eps);
}

/*
 * The routing step of the LFM2-MoE branch (model_lfm2.c:438-473), whose statements sit inline in
 * transformer_layer_lfm2: the reference's router mat-vec and find_top_k are called, the loops in
 * between are restated here and compiled with the reference's flags.  sel_bias = exp_probs_b
 * (may be NULL).  Outputs: topk_idx / topk_w [T x top_k], scores [T x n_expert] (sigmoid; optional).
 */
int tieref_route_lfm2(const float *x, int n_tokens, const float *sel_bias, int *topk_idx, float *topk_w, float *scores_out)
{
	struct TIEContext *ctx = &g.ctx;
	LayerWeights *l = &g.layer;
	const int H = g.hidden, E = g.n_expert, K = g.top_k;
	for (int i = 0; i < n_tokens; i++) {
		MemType xin = {.type = GGML_TYPE_F32, .data = (void *)(x + (size_t)i * H)};
		float *scores = ctx->mem.expert_scores.data;
		float selection_scores[E];
		dispatch_mat_vec(ctx, &xin, &l->ffn_gate_inp, &ctx->mem.expert_scores, H, E, false);
		for (int e = 0; e < E; e++)
			scores[e] = 1.0f / (1.0f + expf(-scores[e]));
		if (sel_bias) {
			for (int e = 0; e < E; e++)
				selection_scores[e] = scores[e] + sel_bias[e];
		} else {
			memcpy(selection_scores, scores, sizeof(float) * E);
		}
		ExpertChoice top[K];
		find_top_k(selection_scores, E, K, top);
		float gate_values[K];
		float sum_weights = 0.0f;
		for (int j = 0; j < K; j++) {
			gate_values[j] = scores[top[j].index];
			sum_weights += gate_values[j];
		}
		float inv_sum = 1.0f / (sum_weights + 1e-6f);
		for (int j = 0; j < K; j++) {
			topk_idx[(size_t)i * K + j] = top[j].index;
			topk_w[(size_t)i * K + j] = gate_values[j] * inv_sum;
		}
		if (scores_out)
			memcpy(scores_out + (size_t)i * E, scores, sizeof(float) * E);
	}
	return 0;
}

/* Wall-clock seconds for n_tokens tokens through tieref_moe_ffn (weights resident, pre-touched
 * by one untimed token).  Used as the CPU baseline next to the GPU number. */
double tieref_time_moe_ffn(const float *x, int n_tokens, const float *router_bias, float *out)
{
	struct timespec t0, t1;
	tieref_moe_ffn(x, 1, router_bias, out, NULL, NULL, NULL);
	clock_gettime(CLOCK_MONOTONIC, &t0);
	tieref_moe_ffn(x, n_tokens, router_bias, out, NULL, NULL, NULL);
	clock_gettime(CLOCK_MONOTONIC, &t1);
	return (double)(t1.tv_sec - t0.tv_sec) + 1e-9 * (double)(t1.tv_nsec - t0.tv_nsec);
}

#ifdef TIE_DROPIN
/*
 * The drop-in proved against the reference's own structures: the same TIEContext / Model /
 * LayerWeights the functions above drive, handed to the glue a maintainer would add to the
 * reference tree (tie_b200/dropin/tie_cuda_qwen3.c).  Built only into
 * oracle/_ref/libtie_ref_dropin.so, which links libtie_cuda.so.
 */
#include "tie_cuda_qwen3.h"

static tie_cuda_ctx *g_cuda;
static int g_cuda_cap;

/* model_load's hook: device context + one-time upload of the layer set by tieref_set_layer. */
int tieref_dropin_load(int device, int max_tokens)
{
	if (!g.ready || !g.layer.ffn_gate_exps.mem.data)
		return -100;
	if (g_cuda) {
		tie_cuda_destroy(g_cuda);
		g_cuda = NULL;
	}
	g_cuda_cap = max_tokens;
	return tie_cuda_qwen3_load(&g.ctx, &g_cuda, device, max_tokens);
}

void tieref_dropin_unload(void)
{
	if (g_cuda)
		tie_cuda_destroy(g_cuda);
	g_cuda = NULL;
}

/* The is_moe branch through the glue: x is placed in ctx->mem.normed_ffn_input, the result is
 * taken from ctx->mem.ffn_down_output (the buffers transformer_layer_qwen3 uses). */
int tieref_dropin_moe_ffn(const float *x, int n_tokens, float *out)
{
	struct TIEContext *ctx = &g.ctx;
	if (!g_cuda || n_tokens > g_cuda_cap)
		return -100;
	ctx->mem.normed_ffn_input = (MemType){.type = GGML_TYPE_F32, .data = (void *)x};
	ctx->mem.ffn_down_output = (MemType){.type = GGML_TYPE_F32, .data = (void *)out};
	return tie_cuda_qwen3_moe_ffn(ctx, g_cuda, 0, n_tokens);
}
#endif /* TIE_DROPIN */
