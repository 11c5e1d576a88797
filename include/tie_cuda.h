/*
 * tie_cuda.h — C ABI of the B200 (sm_100a) backend for TIE's Qwen3-MoE feed-forward path.
 *
 * The library replaces the `if (ctx->model->is_moe)` branch of transformer_layer_qwen3
 * (model_qwen3.c:403-471) and supplies CUDA rows for the math_dispatch.c operator tables.
 * Plain C: opaque handle, pointers and sizes only; every entry point returns 0 or a negative
 * TIE_CUDA_E* code and never calls exit().  There is no CPU fallback: an unsupported type or
 * shape is an error.  One context per GPU; a context is used from one thread at a time (the
 * reference calls transformer_layer from its single model thread, main.c:660).
 *
 * Citations are file:line into the reference (szemzoa/tie).
 */
#ifndef TIE_CUDA_H
#define TIE_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* GGMLType values used on this path (gguf.h:7-40). */
#define TIE_GGML_TYPE_F32 0
#define TIE_GGML_TYPE_Q4_K 12
#define TIE_GGML_TYPE_Q6_K 14

#define TIE_CUDA_SILU_TABLE_SIZE 8192 /* SILU_TABLE_SIZE, engine.h:10 */

/* error codes */
#define TIE_CUDA_OK 0
#define TIE_CUDA_EINVAL (-1)   /* bad argument (null pointer, size out of range, layer not uploaded) */
#define TIE_CUDA_ENOTSUP (-2)  /* tensor type / shape this backend has no kernel for */
#define TIE_CUDA_ENOMEM (-3)   /* device or pinned-host allocation failed */
#define TIE_CUDA_ECUDA (-4)    /* a CUDA runtime call or kernel failed; see tie_cuda_last_cuda_error */
#define TIE_CUDA_ENODEV (-5)   /* no usable sm_100 device */
#define TIE_CUDA_EKERNEL (-6)  /* a kernel reported an internal check failure (device status word) */
#define TIE_CUDA_ETOOBIG (-7)  /* size exceeds the fixed scratch of tie_cuda_route_noalloc */

/* flags for the x / out pointers of the compute entry points */
#define TIE_CUDA_HOST 0u         /* pointers are host memory (the drop-in case: ctx->mem.* buffers) */
#define TIE_CUDA_DEVICE 1u       /* pointers are device memory on the context's GPU */
#define TIE_CUDA_NO_SYNC 2u      /* device pointers only: enqueue on the context's stream and return */
/* Record the call's copies and kernels into a CUDA graph the first time it is seen with these
 * pointers, sizes and flags, and replay the graph afterwards (the reference calls the layer with
 * the same ctx->mem buffers every step, so decode steps become one graph launch).  Ignored while
 * the context runs on the legacy default stream or profiling is on. */
#define TIE_CUDA_GRAPH 4u
/* expert-kernel selection (default: chosen from n_tokens) */
#define TIE_CUDA_PATH_AUTO 0u
#define TIE_CUDA_PATH_STREAM (1u << 8) /* CUDA-core streaming kernels (decode / small batches) */
#define TIE_CUDA_PATH_TENSOR (2u << 8) /* tcgen05 grouped GEMM (prefill) */
#define TIE_CUDA_PATH_MASK (3u << 8)
#define TIE_CUDA_PATH_LEGACY_STREAM (1u << 10) /* with PATH_STREAM: use the general streaming kernels even for 1-4 tokens */
#define TIE_CUDA_PATH_DECODE_CHAIN (1u << 11) /* one token: the chain of three decode kernels instead of the single cooperative one */
#define TIE_CUDA_PATH_NO_PAIR (1u << 14) /* tensor path: one CTA per 128-row tile instead of CTA pairs sharing one MMA issue (M = 256) */
/* Routing of the LFM2-MoE branch (model_lfm2.c:438-473) instead of the Qwen3-MoE one
 * (model_qwen3.c:421-436): sigmoid of the logits, top-k on sigmoid + router_bias (router_bias is
 * then the layer's exp_probs_b selection bias, or NULL), gates = the unbiased sigmoids of the
 * selected experts divided by (their sum + 1e-6).  The logits output of tie_cuda_moe_route then
 * holds the sigmoid scores.  Accepted by tie_cuda_moe_route and tie_cuda_moe_ffn_biased; the
 * expert kernels and the combine are the same. */
#define TIE_CUDA_ROUTE_LFM2 (1u << 12)
/* Expert-parallel decode (tie_cuda_ep_publish, tie_cuda_moe_ffn_ep, tie_cuda_moe_block_inplace_ep):
 * the 1 to 4 tokens of the call are REPLICATED — every rank passes the same rows — instead of
 * each rank bringing tokens of its own.  Every rank routes them itself (the router is replicated
 * and bit-exact, so all ranks select the same experts), computes the slots whose experts it owns
 * and stores their down rows into every rank's region; every rank then combines all slots in the
 * reference's slot order and ends up with the same complete output rows.  n_tokens must be the
 * same on all ranks. */
#define TIE_CUDA_EP_REPLICATED (1u << 13)

typedef struct tie_cuda_ctx tie_cuda_ctx;

typedef struct {
	int device;	/* CUDA device ordinal */
	int hidden;	/* embed_dim          (qwen3moe: 2048) — multiple of 256 */
	int n_expert;	/* expert_count       (128) */
	int top_k;	/* expert_used_count  (8), <= 8 */
	int ffn_dim;	/* expert_ffn_dim     (768) — multiple of 256 */
	int n_layers;	/* number of layer slots */
	int max_tokens; /* largest n_tokens of any call (MAX_PROMPT_BATCH_SIZE 4096, config.h:16) */
	float norm_eps; /* RMSNorm epsilon for tie_cuda_moe_block_inplace */
	/* The reference's silu_table[] (engine.c:12, filled by silu_table_init, engine.c:297-303):
	 * TIE_CUDA_SILU_TABLE_SIZE floats, copied at init.  NULL = tie_cuda_silu_table_default(). */
	const float *silu_table;
	/* Expert parallelism: this context holds experts [ep_rank*n_expert/ep_size, +n_expert/ep_size).
	 * ep_size 1 = all experts.  The exchange between ranks is the caller's (see
	 * tie_cuda_moe_expert_rows / tie_cuda_moe_combine). */
	int ep_rank, ep_size;
} tie_cuda_config;

/* ---- lifetime ---- */
int tie_cuda_init(tie_cuda_ctx **out, const tie_cuda_config *cfg);
void tie_cuda_destroy(tie_cuda_ctx *c);
const char *tie_cuda_strerror(int code);
/* Text of the last CUDA runtime error seen by this context ("" if none). */
const char *tie_cuda_last_cuda_error(const tie_cuda_ctx *c);
/* Run all work of this context on the given cudaStream_t (NULL is the legacy default stream).
 * Until this is called the context uses a non-blocking stream of its own. */
int tie_cuda_set_stream(tie_cuda_ctx *c, void *cuda_stream);
int tie_cuda_synchronize(tie_cuda_ctx *c);

/* The table silu_table_init (engine.c:297-303, expf_fast engine.c:204-225) defines, evaluated
 * with IEEE division.  (The reference as built with -ffast-math uses a reciprocal estimate for
 * that division, so its own table differs from this one, and between CPU models, by a few ulp;
 * a drop-in caller passes its own table in tie_cuda_config.) */
void tie_cuda_silu_table_default(float *out /* [TIE_CUDA_SILU_TABLE_SIZE] */);

/* ---- weights: replaces the residency step of model_load_tensor (model.c:198-235) ----
 * Called once per layer after the loader has the four MoE tensors of LayerWeights
 * (engine.h:77-81) in host memory (mmapped or read).  Copies them to HBM; the host memory may be
 * unmapped afterwards.  Layouts are the GGUF ones the reference slices in process_expert_task
 * (engine.c:929-950): router F32 [n_expert][hidden]; gate/up [n_expert][ffn_dim][hidden/256]
 * blocks; down [n_expert][hidden][ffn_dim/256] blocks.  Types: gate/up/down each Q4_K or Q6_K.
 * With ep_size > 1 the three expert pointers address ONLY this rank's experts (the slice
 * starting at expert ep_rank*n_expert/ep_size); the router is always whole.
 * ffn_norm_w ([hidden] F32, LayerWeights.ffn_norm) may be NULL when
 * tie_cuda_moe_block_inplace is not used for the layer. */
int tie_cuda_upload_moe_layer(tie_cuda_ctx *c, int layer, const void *router_w_f32, const void *gate_exps,
			      int gate_type, const void *up_exps, int up_type, const void *down_exps, int down_type,
			      const float *ffn_norm_w);
/* Bytes of HBM holding weights of this context. */
size_t tie_cuda_weight_bytes(const tie_cuda_ctx *c);

/* ---- the MoE feed-forward call: replaces model_qwen3.c:403-471 ----
 * x   = ctx->mem.normed_ffn_input  fp32 [n_tokens][hidden]
 * out = ctx->mem.ffn_down_output   fp32 [n_tokens][hidden]
 * flags: TIE_CUDA_HOST or TIE_CUDA_DEVICE (| TIE_CUDA_NO_SYNC) (| TIE_CUDA_PATH_*).
 * Requires ep_size == 1. */
int tie_cuda_moe_ffn(tie_cuda_ctx *c, int layer, const float *x, float *out, int n_tokens, unsigned flags);

/* Several host-buffer calls in flight (the reference has no counterpart: its layer call is synchronous).
 * tie_cuda_moe_ffn_submit enqueues what tie_cuda_moe_ffn(.., TIE_CUDA_HOST) does — copy x in, the
 * block, copy the result out — and returns; tie_cuda_moe_ffn_wait(slot) returns when out_host of
 * that slot's call is complete (and reports the call's kernel status).  The copies run on
 * streams of their own, so with two or three slots used in turn the input copy of the next call
 * and the result copy of the previous one overlap the current call's kernels: a host that
 * streams independent batches through a layer pays max(kernels, copy in, copy out) per batch
 * instead of their sum.  slot is 0 .. TIE_CUDA_N_SLOTS - 1 (a slot's staging buffers are allocated
 * at its first use); a slot takes its next call after its wait; x_host and
 * out_host must be page-locked (TIE_CUDA_ENOTSUP otherwise) and must stay untouched until the
 * wait; the context must run on a stream of its own (not the legacy default stream).  flags:
 * TIE_CUDA_GRAPH, TIE_CUDA_PATH_*.  Kernels of different calls never overlap (they share the
 * context's scratch). */
#define TIE_CUDA_N_SLOTS 4
int tie_cuda_moe_ffn_submit(tie_cuda_ctx *c, int layer, const float *x_host, float *out_host, int n_tokens, int slot, unsigned flags);
int tie_cuda_moe_ffn_wait(tie_cuda_ctx *c, int slot);

/* hidden += MoE(RMSNorm(hidden) * ffn_norm_w): the FFN half of a layer, model_qwen3.c:392-401
 * (rms_norm, math_avx2.c:56-97), 403-471, 491 (residual, math_avx2.c:731-751), with the
 * residual stream resident on the device.  hidden_dev: device fp32 [n_tokens][hidden]. */
int tie_cuda_moe_block_inplace(tie_cuda_ctx *c, int layer, float *hidden_dev, int n_tokens, unsigned flags);

/* The same for n_layers consecutive layers, first_layer first: hidden += MoE_l(RMSNorm_l(hidden)) layer
 * after layer, the residual stream staying on the device — the FFN halves of a stack of MoE blocks
 * with nothing between them (a model's attention halves, model_qwen3.c:303-389, are not part of
 * this library; a caller that has them calls tie_cuda_moe_block_inplace per layer).  The layers'
 * kernels are enqueued back to back; with TIE_CUDA_GRAPH the whole stack replays from ONE CUDA
 * graph (one launch call per token instead of one per layer). */
int tie_cuda_moe_stack_inplace(tie_cuda_ctx *c, int first_layer, int n_layers, float *hidden_dev, int n_tokens, unsigned flags);

/* Router only: dispatch_mat_vec on ffn_gate_inp (model_qwen3.c:431, math_avx2.c:228-256),
 * find_top_k (engine.c:891-914), softmax over the selected logits (engine.c:864-888).
 * router_bias ([n_expert], may be NULL; not used by the Qwen3 path) is added to the logits
 * before selection.  topk_idx/topk_w: [n_tokens][top_k] in descending-score order; logits
 * ([n_tokens][n_expert], may be NULL).  All pointers host or all device per flags. */
int tie_cuda_moe_route(tie_cuda_ctx *c, int layer, const float *x, int n_tokens, const float *router_bias,
		       int *topk_idx, float *topk_w, float *logits, unsigned flags);
/* Same as tie_cuda_moe_ffn with a router bias (skewed-load workloads). */
int tie_cuda_moe_ffn_biased(tie_cuda_ctx *c, int layer, const float *x, float *out, int n_tokens,
			    const float *router_bias, unsigned flags);

/* ---- expert-parallel building blocks (the reference has no counterpart: it is one process) ----
 * y_rows[r] = FFN_{row_expert[r]}(x_rows[r]) = process_expert_task (engine.c:916-964) applied
 * to independent rows, unweighted.  row_expert holds GLOBAL expert ids, all owned by this
 * context.  fp32 [n_rows][hidden]; device pointers. */
int tie_cuda_moe_expert_rows(tie_cuda_ctx *c, int layer, const float *x_rows, const int *row_expert, int n_rows,
			     float *y_rows, unsigned flags);
/* out[t] = sum_j w[t][j] * y_rows[t*top_k + j], j ascending, fused multiply-add from zero
 * (model_qwen3.c:458-467).  Device pointers. */
int tie_cuda_moe_combine(tie_cuda_ctx *c, const float *y_rows, const float *topk_w, int n_tokens, float *out,
			 unsigned flags);

/* Dispatch for expert parallelism: group this rank's n_tokens*top_k (token, slot) rows by expert
 * id (a stable counting sort; experts of one rank are contiguous, so the result is also grouped
 * by destination rank).  send_rows[p] = x[token of row perm[p]] (fp32 [n_tokens*top_k][hidden]),
 * send_expert[p] = its expert id, expert_counts[e] = rows for expert e (int [n_expert]).  The
 * permutation stays in the context for tie_cuda_moe_ep_combine.  Device pointers. */
int tie_cuda_moe_ep_dispatch(tie_cuda_ctx *c, const float *x, const int *topk_idx, int n_tokens, float *send_rows,
			     int *send_expert, int *expert_counts, unsigned flags);
/* out[t] = sum_j w[t][j] * y_sorted[position of row (t, j) in the last dispatch], j ascending
 * (the combine of model_qwen3.c:458-467 on rows that came back in dispatch order). */
int tie_cuda_moe_ep_combine(tie_cuda_ctx *c, const float *y_sorted, const float *topk_w, int n_tokens, float *out,
			    unsigned flags);

/* ---- expert parallelism over peer memory (the reference has no counterpart) ----
 * One context per GPU (ep_rank / ep_size in the config; max_tokens = ep_size x the tokens one rank
 * brings per step, so that the scratch holds the worst case of every row landing on one rank).
 * Dispatch and combine are not collectives here: every rank exposes one region of its HBM, a
 * rank stores its tokens into every rank's region while it routes them, the owners read the
 * (small) row lists out of the sources' regions and the down product stores every output row
 * straight into its source's region (plain stores and loads over NVLink); ranks synchronise
 * through step-numbered flags they store into each other's regions.  No host synchronisation
 * per step.
 *
 * Set-up, once, collectively: tie_cuda_ep_ipc_handle() on every rank, exchange the 64-byte
 * handles by any host channel, tie_cuda_ep_attach(handles, ep_size, TIE_CUDA_EP_PEER_IPC_HANDLES).
 * Contexts of ONE process (several ranks emulated on one GPU, or one process driving several
 * GPUs with peer access enabled) pass tie_cuda_ep_region() base pointers instead
 * (TIE_CUDA_EP_PEER_POINTERS).  The entry of the calling rank itself is ignored.
 *
 * A step, on every rank, in this order (device pointers, TIE_CUDA_DEVICE; tensor-core path only):
 *   tie_cuda_ep_publish  routes x [n_tokens][hidden] (0 <= n_tokens <= max_tokens / ep_size, may
 *                        differ between ranks) and hands it to every rank meanwhile, sorts its
 *                        rows by expert and announces the step
 *   tie_cuda_ep_compute  waits for every rank's announcement, lays out the rows of this rank's
 *                        experts (tokens from its own memory, row lists from their sources), runs
 *                        gate/up, SwiGLU, down (outputs land at their sources)
 *   tie_cuda_ep_gather   waits for every owner, out[t] = (residual[t] +) sum_j w[t][j] * y(t, j)
 * With TIE_CUDA_EP_REPLICATED in the flags of tie_cuda_ep_publish the step is the decode form:
 * the same 1 to 4 tokens on every rank (no dispatch: publish only routes and announces the step;
 * compute runs gate/up and down for the locally owned slots and stores the down rows to all
 * ranks; gather combines).  Prefill and decode steps may alternate freely.
 * tie_cuda_moe_ffn_ep is the three in a row; with TIE_CUDA_GRAPH the whole step is replayed from a
 * CUDA graph (the step number advances on the device).
 * Kernels of different ranks wait on one another, so
 * ranks that share ONE GPU must enqueue phase by phase on one stream (all publishes, then all
 * computes, then all gathers) — a wait is then always already satisfied; on separate GPUs the
 * ranks run freely.  Every wait is bounded (tie_cuda_ep_set_timeout_ms, default 5 s): a rank that
 * never arrives makes the others return TIE_CUDA_EKERNEL with their contexts usable; the group
 * must then detach and attach again before its next step.  tie_cuda_ep_attach starts a new
 * epoch (step counter and flags of the calling rank's region back to zero), so attach is
 * collective: all ranks detach, host barrier, all ranks attach, host barrier, first publish —
 * the barriers keep a peer's flag store from crossing a rank's reset. */
#define TIE_CUDA_EP_HANDLE_BYTES 64
#define TIE_CUDA_EP_PEER_POINTERS 0
#define TIE_CUDA_EP_PEER_IPC_HANDLES 1
int tie_cuda_ep_region(tie_cuda_ctx *c, void **base, size_t *bytes);
int tie_cuda_ep_ipc_handle(tie_cuda_ctx *c, void *handle /* TIE_CUDA_EP_HANDLE_BYTES */);
int tie_cuda_ep_attach(tie_cuda_ctx *c, const void *const *peers, int n_peers, int kind);
int tie_cuda_ep_detach(tie_cuda_ctx *c);
int tie_cuda_ep_set_timeout_ms(tie_cuda_ctx *c, int ms);
int tie_cuda_ep_publish(tie_cuda_ctx *c, int layer, const float *x, int n_tokens, const float *router_bias, unsigned flags);
int tie_cuda_ep_compute(tie_cuda_ctx *c, int layer, unsigned flags);
int tie_cuda_ep_gather(tie_cuda_ctx *c, float *out, const float *residual, unsigned flags);
int tie_cuda_moe_ffn_ep(tie_cuda_ctx *c, int layer, const float *x, float *out, int n_tokens, unsigned flags);
/* hidden += MoE(RMSNorm(hidden)) for this rank's tokens, as tie_cuda_moe_block_inplace, with the
 * experts spread over the ranks (the layer's ffn_norm_w must have been uploaded). */
int tie_cuda_moe_block_inplace_ep(tie_cuda_ctx *c, int layer, float *hidden_dev, int n_tokens, unsigned flags);

/* ---- math_dispatch.c rows (accel = 2) ----
 * Same argument meaning as the reference's kernels are CALLED with (math_dispatch.c:224,254):
 * (X, W_data, O, in_dim, start_row, end_row); X, O host fp32.  W must point into (or at) a
 * host tensor registered by tie_cuda_upload_moe_layer / tie_cuda_register_tensor; the device
 * copy is found by host address.  They use the context made current by tie_cuda_make_current
 * (the reference's dispatch signatures carry no context) and return nothing, like the
 * reference's; failures are reported through tie_cuda_dispatch_status().
 * Threading: unlike the context entry points above, these rows may be called from several host
 * threads at once — the reference's threaded dispatcher (math_dispatch.c:262-283) gives each pool
 * worker a disjoint [start_row, end_row) slice of one mat-vec.  A call holds the current
 * context's row lock from its first use of the staging buffers to the read-back of the status
 * word, and computes the rows of its slice only.  tie_cuda_make_current itself is not meant to
 * race with calls in flight. */
int tie_cuda_make_current(tie_cuda_ctx *c);
/* Upload a stand-alone weight tensor (rows of in_dim inputs; F32, Q4_K or Q6_K) so that the rows
 * below can find it by host address (model_load_tensor, model.c:198-235, for non-MoE tensors). */
int tie_cuda_register_tensor(tie_cuda_ctx *c, const void *host_ptr, size_t n_bytes, int ggml_type, int in_dim);
/* dispatch_mat_mat (math_dispatch.c:304-370: O[i] = W . X[i] for the batch_len rows of X, the
 * reference runs its mat-vec row kernels per row) for a Q4_K / Q6_K tensor registered with
 * tie_cuda_register_tensor, on the tensor-core kernel of the expert products (the tensor is one
 * "expert" owning every row) — the dense FFN and attention projections of a prompt batch.
 * W: the registered host address; X [batch_len][in_dim], O [batch_len][out_dim] fp32, host or
 * device per flags.  Supported: any in_dim that is a multiple of 256 (a Q4_K tensor with more than
 * 2048 inputs runs as one launch per 2048 of them, each adding to O), out_dim a multiple of 128;
 * batch_len is bounded by the context's operand scratch viewed with rows of in_dim values
 * (about max_tokens * top_k * hidden / in_dim rows); otherwise TIE_CUDA_ENOTSUP / _ETOOBIG. */
int tie_cuda_mat_mat(tie_cuda_ctx *c, const void *W, const float *X, float *O, int batch_len, int in_dim, int out_dim,
		     unsigned flags);
void tie_cuda_mat_vec_row_f32_q4k_f32(const void *X, const void *W, void *O, int in_dim, int start_row, int end_row);
void tie_cuda_mat_vec_row_f32_q6k_f32(const void *X, const void *W, void *O, int in_dim, int start_row, int end_row);
void tie_cuda_mat_vec_row_f32_f32_f32(const void *X, const void *W, void *O, int in_dim, int start_row, int end_row);
/* swiglu_fn (math_dispatch.h:20; math_avx2.c:908-950): gate[i] = silu_table_lookup(gate[i]) * up[i]. */
void tie_cuda_swiglu_f32_f32(void *gate, const void *up, int size);
int tie_cuda_dispatch_status(void); /* 0, or the TIE_CUDA_E* of the last failing dispatch-row call */

/* ---- routing for callers that must not allocate ----
 * No counterpart in the reference (it is a CPU program with malloc'd buffers).
 *
 * Same result as tie_cuda_moe_route on device pointers, but without a context and without a
 * single allocation: no cudaMalloc / cudaFree / cudaMallocHost and no allocating library call,
 * on any call.  It is meant for hosts that cannot allocate when they call in: a serving loop
 * whose rules ban allocator calls once start-up is over (an allocation can block or fail at a
 * bad moment), or an application that runs under a fixed memory budget and hands the library no
 * allocator.  The logits scratch the router needs sits in a
 * fixed array inside the library image (64 KiB on every GPU that loads the library, held until
 * the process exits), so sizes are capped: n_tokens <= 64 and n_expert <= 256, and for
 * n_tokens <= 8 also (1 + n_tokens) * hidden floats <= 200 KB of shared memory; anything larger
 * returns TIE_CUDA_ETOOBIG.  hidden % 8 == 0 (% 256 when n_tokens > 8), n_expert % 16 == 0,
 * top_k <= 8.
 *
 * The caller passes every input and output (device memory on the current device): x
 * [n_tokens][hidden], router_w [n_expert][hidden], router_bias [n_expert] or NULL, topk_idx /
 * topk_w [n_tokens][top_k].  x and router_w are read with 128-bit loads and must be 16-byte
 * aligned (rows then are, hidden being a multiple of 8); the other pointers 4-byte aligned.  A
 * pointer that is not gets TIE_CUDA_EINVAL, not a fault on the device.  Work is enqueued on
 * cuda_stream (NULL = legacy default stream) and the call returns without synchronising.
 *
 * The first call on each device looks up the device address of the scratch array and sets a
 * kernel attribute (the device must be current); that first call should come before any stream
 * capture.  Host threads may make their first calls concurrently (the set-up is done under a
 * lock, once per device).  All calls on a device share the one scratch array: it keeps the
 * previous call's contents (every element a call reads it has written first, so nothing needs
 * clearing), and two calls whose kernels overlap on the GPU (for instance on different streams,
 * or from two host threads) race on it.  Serialise them. */
int tie_cuda_route_noalloc(const float *x_dev, const float *router_w_dev, const float *router_bias_dev, int n_tokens,
			   int hidden, int n_expert, int top_k, int *topk_idx_dev, float *topk_w_dev, void *cuda_stream);

/* ---- introspection for tests and benchmarks ---- */
/* Number of kernels this context has launched since init (all entry points). */
uint64_t tie_cuda_launch_count(const tie_cuda_ctx *c);
/* Distinct experts that received at least one row in the last tie_cuda_moe_ffn* / _expert_rows
 * call (read back from the device; synchronises). */
int tie_cuda_last_active_experts(tie_cuda_ctx *c);
/* Per-phase device times of a call, from CUDA events on the context's stream (off by default).
 * phase_ms[TIE_CUDA_N_PHASES]: router, dispatch sort, input split, gate/up product, SwiGLU pass
 * (zero where the gate/up kernel applies it itself), down product, combine — of the most recent
 * tie_cuda_moe_ffn* / _block_inplace call.
 * tie_cuda_get_profile synchronises; returns 1 if that call used the tensor-core kernels, 0 if
 * the streaming kernels, negative on error. */
#define TIE_CUDA_N_PHASES 7
int tie_cuda_set_profiling(tie_cuda_ctx *c, int on);
int tie_cuda_get_profile(tie_cuda_ctx *c, float *phase_ms);
const char *tie_cuda_version(void);

#ifdef __cplusplus
}
#endif
#endif /* TIE_CUDA_H */
