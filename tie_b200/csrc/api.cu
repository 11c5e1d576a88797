// C ABI of the library (include/tie_cuda.h): context, weight residency, the MoE feed-forward
// call and the math_dispatch rows.  Host logic only; kernels live in the other translation units.
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <mutex>

#include "common.cuh"
#include "ep_dev.cuh"
#include "kernels.cuh"

using namespace tie;

namespace {

tie_cuda_ctx *g_current = nullptr;
std::atomic<int> g_dispatch_status{0};
std::mutex g_mutex;

size_t block_bytes(int ggml_type)
{
	return ggml_type == TIE_GGML_TYPE_Q4_K ? Q4K_BYTES : (ggml_type == TIE_GGML_TYPE_Q6_K ? Q6K_BYTES : 0);
}

template <typename T>
int dev_alloc(tie_cuda_ctx *c, T **p, size_t n)
{
	TIE_CUDA_TRY(c, cudaMalloc(reinterpret_cast<void **>(p), n * sizeof(T)));
	return TIE_CUDA_OK;
}

#define TRY(expr)                 \
	do {                      \
		int _rc = (expr); \
		if (_rc)          \
			return _rc; \
	} while (0)

int alloc_scratch(tie_cuda_ctx *c)
{
	Scratch &s = c->s;
	const size_t T = c->cfg.max_tokens, H = c->cfg.hidden, E = c->cfg.n_expert, K = c->cfg.top_k, F = c->cfg.ffn_dim;
	const size_t R = T * K;
	s.rows_cap = R;
	s.rows_pad = R + 256;
	TRY(dev_alloc(c, &s.x, T * H));
	TRY(dev_alloc(c, &s.out, T * H));
	TRY(dev_alloc(c, &s.logits, T * E));
	TRY(dev_alloc(c, &s.bias, E));
	TRY(dev_alloc(c, &s.topk_idx, R));
	TRY(dev_alloc(c, &s.topk_w, R));
	TRY(dev_alloc(c, &s.counts, E));
	TRY(dev_alloc(c, &s.offsets, E + 1));
	TRY(dev_alloc(c, &s.tile_start, E + 1));
	TRY(dev_alloc(c, &s.tile_info, E + R / TC_TOKEN_TILE + 1));
	TRY(dev_alloc(c, &s.active, E));
	TRY(dev_alloc(c, &s.n_active, 1));
	TRY(dev_alloc(c, &s.perm, R));
	s.sort_hist_cap = ((R + SORT_SLICE - 1) / SORT_SLICE + 1) * E;
	TRY(dev_alloc(c, &s.sort_hist, s.sort_hist_cap));
	TRY(dev_alloc(c, &s.h, R * F));
	TRY(dev_alloc(c, &s.y, R * (H > 2 * F ? H : 2 * F)));  // also holds the raw gate|up products of the tensor path
	// hi and lo halves of each split array share one allocation (lo right behind hi): one 3-D TMA box fetches both
	TRY(dev_alloc(c, &s.xs_hi, 2 * s.rows_pad * H));
	s.xs_lo = s.xs_hi + s.rows_pad * H;
	TRY(dev_alloc(c, &s.hs_hi, 2 * s.rows_pad * F));
	s.hs_lo = s.hs_hi + s.rows_pad * F;
	const size_t XH = xq_cols((int)H), XF = xq_cols((int)F);
	TRY(dev_alloc(c, &s.xq_hi, 2 * s.rows_pad * XH));
	s.xq_lo = s.xq_hi + s.rows_pad * XH;
	TRY(dev_alloc(c, &s.hq_hi, 2 * s.rows_pad * XF));
	s.hq_lo = s.hq_hi + s.rows_pad * XF;
	TRY(dev_alloc(c, &s.status, 1));
	TRY(dev_alloc(c, &s.counter, 1));
	TIE_CUDA_TRY(c, cudaMemset(s.counter, 0, sizeof(int)));
	TRY(dev_alloc(c, &s.dec_sync, 2));
	TIE_CUDA_TRY(c, cudaMemset(s.dec_sync, 0, 2 * sizeof(unsigned)));
	TRY(dev_alloc(c, &s.row_expert, R));
	TRY(dev_alloc(c, &s.ep_counts, E));
	TRY(dev_alloc(c, &s.ep_offsets, E + 1));
	TRY(dev_alloc(c, &s.ep_tile_start, E + 1));
	TRY(dev_alloc(c, &s.ep_active, E));
	TRY(dev_alloc(c, &s.ep_n_active, 1));
	TRY(dev_alloc(c, &s.ep_perm, R));
	TRY(dev_alloc(c, &s.ep_inv, R));
	TIE_CUDA_TRY(c, cudaMemset(s.status, 0, sizeof(unsigned)));
	TIE_CUDA_TRY(c, cudaMemset(s.n_active, 0, sizeof(int)));
	// rows past the last real one are read (never used) by the tensor path: keep them finite
	TIE_CUDA_TRY(c, cudaMemset(s.xs_hi, 0, s.rows_pad * H * sizeof(__half)));
	TIE_CUDA_TRY(c, cudaMemset(s.xs_lo, 0, s.rows_pad * H * sizeof(__half)));
	TIE_CUDA_TRY(c, cudaMemset(s.hs_hi, 0, s.rows_pad * F * sizeof(__half)));
	TIE_CUDA_TRY(c, cudaMemset(s.hs_lo, 0, s.rows_pad * F * sizeof(__half)));
	// the padding columns of the sub-block sums are read by the tensor path and must stay zero
	TIE_CUDA_TRY(c, cudaMemset(s.xq_hi, 0, s.rows_pad * XH * sizeof(__half)));
	TIE_CUDA_TRY(c, cudaMemset(s.xq_lo, 0, s.rows_pad * XH * sizeof(__half)));
	TIE_CUDA_TRY(c, cudaMemset(s.hq_hi, 0, s.rows_pad * XF * sizeof(__half)));
	TIE_CUDA_TRY(c, cudaMemset(s.hq_lo, 0, s.rows_pad * XF * sizeof(__half)));
	TIE_CUDA_TRY(c, cudaMallocHost(reinterpret_cast<void **>(&c->pin_x), T * H * sizeof(float)));
	TIE_CUDA_TRY(c, cudaMallocHost(reinterpret_cast<void **>(&c->pin_out), T * H * sizeof(float)));
	TIE_CUDA_TRY(c, cudaMallocHost(reinterpret_cast<void **>(&c->pin_idx), R * sizeof(int)));
	TIE_CUDA_TRY(c, cudaMallocHost(reinterpret_cast<void **>(&c->pin_w), R * sizeof(float)));
	TIE_CUDA_TRY(c, cudaMallocHost(reinterpret_cast<void **>(&c->pin_logits), T * E * sizeof(float)));
	TIE_CUDA_TRY(c, cudaMallocHost(reinterpret_cast<void **>(&c->pin_status), sizeof(unsigned)));
	*c->pin_status = 0;
	return TIE_CUDA_OK;
}

void free_tensor(DevTensor &t)
{
	if (t.ptr)
		cudaFree(t.ptr);
	t = DevTensor();
}

// Copy one stacked expert tensor to the device (re-ordering Q6_K into R8).
int upload_tensor(tie_cuda_ctx *c, DevTensor &t, const void *host, int type, int rows, int k)
{
	const size_t bb = block_bytes(type);
	if (!bb)
		return TIE_CUDA_ENOTSUP;
	if (k % QK_K || rows % 8)
		return TIE_CUDA_ENOTSUP;
	const int nb = k / QK_K;
	free_tensor(t);
	t.ggml_type = type;
	t.kind = (type == TIE_GGML_TYPE_Q4_K) ? W_Q4K : W_Q6K_R8;
	t.rows = rows;
	t.k = k;
	t.expert_stride = (size_t)rows * nb * bb;
	t.bytes = t.expert_stride * c->n_local;
	t.host_ptr = host;
	TIE_CUDA_TRY(c, cudaMalloc(reinterpret_cast<void **>(&t.ptr), t.bytes));
	if (t.kind == W_Q4K) {
		TIE_CUDA_TRY(c, cudaMemcpyAsync(t.ptr, host, t.bytes, cudaMemcpyHostToDevice, c->stream));
	} else {
		uint8_t *raw = nullptr;
		TIE_CUDA_TRY(c, cudaMalloc(reinterpret_cast<void **>(&raw), t.bytes));
		cudaError_t e = cudaMemcpyAsync(raw, host, t.bytes, cudaMemcpyHostToDevice, c->stream);
		int rc = TIE_CUDA_OK;
		if (e == cudaSuccess)
			rc = launch_repack_q6k_r8(c, raw, t.ptr, (size_t)rows * c->n_local, nb);
		cudaStreamSynchronize(c->stream);
		cudaFree(raw);
		if (e != cudaSuccess) {
			snprintf(c->cuda_err, sizeof(c->cuda_err), "upload: %s", cudaGetErrorString(e));
			return TIE_CUDA_ECUDA;
		}
		if (rc)
			return rc;
	}
	TIE_CUDA_TRY(c, cudaStreamSynchronize(c->stream));
	c->weight_bytes += t.bytes;
	return tc_make_weight_map(c, t);
}

int add_reg(tie_cuda_ctx *c, const void *host, size_t bytes, const uint8_t *dev, int type, WKind kind, int rows, int k,
	    DevTensor *dense = nullptr)
{
	if (c->n_regs == c->cap_regs) {
		int nc = c->cap_regs ? c->cap_regs * 2 : 64;
		void *p = realloc(c->regs, nc * sizeof(*c->regs));
		if (!p)
			return TIE_CUDA_ENOMEM;
		c->regs = static_cast<decltype(c->regs)>(p);
		c->cap_regs = nc;
	}
	c->regs[c->n_regs++] = {host, bytes, dev, type, kind, rows, k, dense};
	return TIE_CUDA_OK;
}

// Before a layer's tensors are replaced: cached CUDA graphs of calls on that layer hold the old
// device pointers and tensor maps, and the dispatch-row registry the old device copies.
void forget_layer(tie_cuda_ctx *c, int layer, const Layer &L)
{
	if (c->stream)
		cudaStreamSynchronize(c->stream);
	for (int i = 0; i < c->n_graphs;) {
		if (c->graphs[i].layer == layer || c->graphs[i].kind == 8) {  // (a stack graph spans several layers)
			cudaGraphExecDestroy(c->graphs[i].exec);
			c->graphs[i] = c->graphs[--c->n_graphs];
		} else {
			i++;
		}
	}
	const uint8_t *old[4] = {reinterpret_cast<const uint8_t *>(L.router_w), L.gate.ptr, L.up.ptr, L.down.ptr};
	for (int i = 0; i < c->n_regs;) {
		bool hit = false;
		for (const uint8_t *p : old)
			hit = hit || (p && c->regs[i].dev == p);
		if (hit && !c->regs[i].dense)
			c->regs[i] = c->regs[--c->n_regs];
		else
			i++;
	}
}

bool is_pinned_host(const void *p)
{
	cudaPointerAttributes a;
	if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
		cudaGetLastError();
		return false;
	}
	return a.type == cudaMemoryTypeHost;
}

int report_status(tie_cuda_ctx *c, unsigned st);

int check_status(tie_cuda_ctx *c)
{
	unsigned st = 0;
	TIE_CUDA_TRY(c, cudaMemcpyAsync(&st, c->s.status, sizeof(st), cudaMemcpyDeviceToHost, c->stream));
	TIE_CUDA_TRY(c, cudaStreamSynchronize(c->stream));
	return report_status(c, st);
}

// The status word was copied to pinned memory by the stream's last operation (host-pointer calls:
// one synchronisation for the results and the status together).
int check_status_pinned(tie_cuda_ctx *c)
{
	TIE_CUDA_TRY(c, cudaStreamSynchronize(c->stream));
	return report_status(c, *static_cast<volatile unsigned *>(c->pin_status));
}

int report_status(tie_cuda_ctx *c, unsigned st)
{
	if (st) {
		snprintf(c->cuda_err, sizeof(c->cuda_err), "device status word 0x%x (%s%s%s)", st,
			 (st & ST_BAD_EXPERT) ? "expert id out of range " : "", (st & ST_WAIT_TIMEOUT) ? "barrier wait timed out " : "",
			 (st & ST_BAD_TILE) ? "tile bookkeeping " : "");
		cudaMemsetAsync(c->s.status, 0, sizeof(unsigned), c->stream);
		if (st & ST_WAIT_TIMEOUT)  // a grid barrier of the one-kernel decode step may have been left half-counted
			cudaMemsetAsync(c->s.dec_sync, 0, 2 * sizeof(unsigned), c->stream);
		return TIE_CUDA_EKERNEL;
	}
	return TIE_CUDA_OK;
}

// Phase marks: 0 start, 1 router done, 2 dispatch sort done, 3 input split done, 4 gate/up done,
// 5 SwiGLU pass done (only where it is a pass of its own), 6 down done, 7 combine done.
void prof_mark(tie_cuda_ctx *c, int id)
{
	if (!c->prof_on)
		return;
	if (id == 0)
		for (int i = 0; i < 8; i++)
			c->prof_set[i] = false;
	if (cudaEventRecord(c->prof_ev[id], c->stream) == cudaSuccess)
		c->prof_set[id] = true;
}

// The expert part on device rows.  x_src: fp32 rows; row r reads x_src[r / src_div].
// row_expert [n_rows] (device) gives the global expert of every row; y [n_rows][H] receives
// the unweighted expert outputs in row order.
int run_experts(tie_cuda_ctx *c, const Layer &L, const float *x_src, int src_div, const int *row_expert, int n_rows, float *y,
		unsigned flags)
{
	const unsigned path = flags & TIE_CUDA_PATH_MASK;
	bool use_tc;
	if (path == TIE_CUDA_PATH_TENSOR) {
		if (!tc_supported(c, L))
			return TIE_CUDA_ENOTSUP;
		use_tc = true;
	} else if (path == TIE_CUDA_PATH_STREAM) {
		use_tc = false;
	} else {
		use_tc = tc_supported(c, L) && n_rows >= 2 * c->n_local;
	}
	c->tc_no_pair = (flags & TIE_CUDA_PATH_NO_PAIR) != 0;
	const int direct = (!use_tc && n_rows <= c->cfg.top_k && src_div == c->cfg.top_k) ? 1 : 0;
	const int n_tile = TC_TOKEN_TILE;
	c->last_direct_rows = direct ? n_rows : -1;
	c->last_used_tc = use_tc;
	if (!direct)
		TRY(launch_sort(c, row_expert, n_rows, n_tile));
	prof_mark(c, 2);
	if (use_tc) {
		const bool sums = L.gate.kind == W_Q4K;	 // the Q4_K "min" term needs the sub-block sums of the inputs
		TRY(launch_split_rows(c, x_src, c->s.perm, src_div, n_rows, c->cfg.hidden, c->s.xs_hi, c->s.xs_lo,
				      sums ? c->s.xq_hi : nullptr, sums ? c->s.xq_lo : nullptr));
		prof_mark(c, 3);
		TRY(launch_tc_gate_up(c, L, n_rows));
		prof_mark(c, 4);
		TRY(launch_tc_swiglu(c, L, n_rows));
		prof_mark(c, 5);
		TRY(launch_tc_down(c, L, n_rows, y));
		prof_mark(c, 6);
	} else {
		prof_mark(c, 3);
		TRY(launch_stream_gate_up(c, L, x_src, src_div, row_expert, n_rows, direct));
		prof_mark(c, 4);
		TRY(launch_stream_down(c, L, y, row_expert, n_rows, direct));
		prof_mark(c, 6);
	}
	return TIE_CUDA_OK;
}

int get_layer(tie_cuda_ctx *c, int layer, Layer **L)
{
	if (!c || layer < 0 || layer >= c->cfg.n_layers || !c->layers[layer].uploaded)
		return TIE_CUDA_EINVAL;
	*L = &c->layers[layer];
	return TIE_CUDA_OK;
}

int moe_ffn_device(tie_cuda_ctx *c, Layer &L, const float *x, float *out, int n_tokens, const float *bias_dev,
		   const float *residual, unsigned flags)
{
	Scratch &s = c->s;
	const int lfm2 = (flags & TIE_CUDA_ROUTE_LFM2) ? 1 : 0;
	prof_mark(c, 0);
	const bool decode_paths = (flags & TIE_CUDA_PATH_MASK) != TIE_CUDA_PATH_TENSOR && !(flags & TIE_CUDA_PATH_LEGACY_STREAM);
	// one token: the whole block as one cooperative kernel
	if (decode_paths && !lfm2 && !(flags & TIE_CUDA_PATH_DECODE_CHAIN) && decode_fused_supported(c, L, n_tokens)) {
		const int rc = launch_decode_fused(c, L, x, bias_dev, residual, out);
		if (rc != TIE_CUDA_ENOTSUP) {  // (not supported after all: the chain below)
			if (rc)
				return rc;
			c->last_used_tc = false;
			c->last_direct_rows = c->cfg.top_k;
			for (int i = 1; i <= 7; i++)
				prof_mark(c, i);
			return TIE_CUDA_OK;
		}
	}
	// decode (1-4 tokens): three launches — router with fused selection, gate/up, down + combine
	if ((flags & TIE_CUDA_PATH_MASK) != TIE_CUDA_PATH_TENSOR && !(flags & TIE_CUDA_PATH_LEGACY_STREAM) &&
	    decode_supported(c, L, n_tokens)) {
		if (lfm2)  // the LFM2 selection is a kernel of its own
			TRY(launch_router(c, x, L.router_w, bias_dev, n_tokens, s.logits, s.topk_idx, s.topk_w, 1));
		else
			TRY(launch_router_decode_fused(c, x, L.router_w, bias_dev, n_tokens, s.logits, s.topk_idx, s.topk_w));
		prof_mark(c, 1);
		c->last_used_tc = false;
		c->last_direct_rows = n_tokens * c->cfg.top_k;
		prof_mark(c, 2);
		prof_mark(c, 3);
		TRY(launch_decode_gate_up(c, L, x, n_tokens));
		prof_mark(c, 4);
		TRY(launch_decode_down_combine(c, L, n_tokens, residual, out));
		prof_mark(c, 6);
		prof_mark(c, 7);
		return TIE_CUDA_OK;
	}
	TRY(launch_router(c, x, L.router_w, bias_dev, n_tokens, s.logits, s.topk_idx, s.topk_w, lfm2));
	prof_mark(c, 1);
	TRY(run_experts(c, L, x, c->cfg.top_k, s.topk_idx, n_tokens * c->cfg.top_k, s.y, flags));
	TRY(launch_combine(c, s.y, s.topk_w, n_tokens, residual, out));
	prof_mark(c, 7);
	return TIE_CUDA_OK;
}

struct GraphKey {
	int kind, layer, n;
	const void *p0, *p1, *p2, *p3;
	unsigned flags;
};

// Runs enqueue() either directly or, with TIE_CUDA_GRAPH, through a cached CUDA graph.
template <class F>
int run_maybe_graphed(tie_cuda_ctx *c, bool want_graph, const GraphKey &k, F enqueue)
{
	if (!want_graph || c->stream == nullptr || c->prof_on)
		return enqueue();
	for (int i = 0; i < c->n_graphs; i++) {
		auto &g = c->graphs[i];
		if (g.kind == k.kind && g.layer == k.layer && g.n == k.n && g.p0 == k.p0 && g.p1 == k.p1 && g.p2 == k.p2 &&
		    g.p3 == k.p3 && g.flags == k.flags) {
			g.stamp = ++c->graph_clock;
			TIE_CUDA_TRY(c, cudaGraphLaunch(g.exec, c->stream));
			c->launches += g.kernels;
			return TIE_CUDA_OK;
		}
	}
	const uint64_t before = c->launches;
	TIE_CUDA_TRY(c, cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
	int rc = enqueue();
	cudaGraph_t graph = nullptr;
	cudaError_t e = cudaStreamEndCapture(c->stream, &graph);
	const uint64_t kernels = c->launches - before;
	c->launches = before;
	if (rc || e != cudaSuccess || !graph) {
		if (graph)
			cudaGraphDestroy(graph);
		cudaGetLastError();
		if (rc)
			return rc;
		snprintf(c->cuda_err, sizeof(c->cuda_err), "stream capture failed: %s", cudaGetErrorString(e));
		return TIE_CUDA_ECUDA;
	}
	cudaGraphExec_t exec = nullptr;
	e = cudaGraphInstantiate(&exec, graph, 0);
	cudaGraphDestroy(graph);
	if (e != cudaSuccess) {
		snprintf(c->cuda_err, sizeof(c->cuda_err), "cudaGraphInstantiate: %s", cudaGetErrorString(e));
		return TIE_CUDA_ECUDA;
	}
	int slot = c->n_graphs;
	const int cap = (int)(sizeof(c->graphs) / sizeof(c->graphs[0]));
	if (slot == cap) {  // evict the least recently used
		slot = 0;
		for (int i = 1; i < cap; i++)
			if (c->graphs[i].stamp < c->graphs[slot].stamp)
				slot = i;
		cudaGraphExecDestroy(c->graphs[slot].exec);
	} else {
		c->n_graphs++;
	}
	c->graphs[slot] = {k.kind, k.layer, k.n, k.p0, k.p1, k.p2, k.p3, k.flags, exec, kernels, ++c->graph_clock};
	TIE_CUDA_TRY(c, cudaGraphLaunch(exec, c->stream));
	c->launches += kernels;
	return TIE_CUDA_OK;
}

int h2d(tie_cuda_ctx *c, void *dst, const void *src, size_t bytes, void *pin)
{
	if (is_pinned_host(src)) {
		TIE_CUDA_TRY(c, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, c->stream));
	} else {
		// the staging buffer is reused by the next call: make sure the previous copy out of it is done
		TIE_CUDA_TRY(c, cudaStreamSynchronize(c->stream));
		memcpy(pin, src, bytes);
		TIE_CUDA_TRY(c, cudaMemcpyAsync(dst, pin, bytes, cudaMemcpyHostToDevice, c->stream));
	}
	return TIE_CUDA_OK;
}

size_t align_up(size_t v, size_t a)
{
	return (v + a - 1) / a * a;
}

void ep_close_peers(tie_cuda_ctx *c)
{
	EpState &ep = c->ep;
	for (int i = 0; i < EP_MAX_RANKS; i++) {
		if (ep.opened[i] && ep.view.peer[i])
			cudaIpcCloseMemHandle(ep.view.peer[i]);
		ep.opened[i] = false;
		ep.view.peer[i] = nullptr;
	}
	ep.attached = false;
	ep.phase = 0;
	ep.step_tokens = -1;
	// graphs of whole steps hold the peers' addresses
	for (int i = 0; i < c->n_graphs;) {
		if (c->graphs[i].kind == 5 || c->graphs[i].kind == 6) {
			cudaGraphExecDestroy(c->graphs[i].exec);
			c->graphs[i] = c->graphs[--c->n_graphs];
		} else {
			i++;
		}
	}
}

void ep_release(tie_cuda_ctx *c)
{
	EpState &ep = c->ep;
	ep_close_peers(c);
	void *ptrs[] = {ep.region, ep.n_rows, ep.seg_base, ep.seg_src, ep.row_dst, ep.step_dev};
	for (void *p : ptrs)
		if (p)
			cudaFree(p);
	ep = EpState();
}

// Allocates the region peers map, on first use.
int ep_region(tie_cuda_ctx *c)
{
	EpState &ep = c->ep;
	if (ep.region)
		return TIE_CUDA_OK;
	const int G = c->cfg.ep_size;
	if (G > EP_MAX_RANKS || c->cfg.n_expert > 256 || c->cfg.max_tokens % G ||
	    (long long)(c->cfg.max_tokens / G) * c->cfg.top_k >= (1 << 24))
		return TIE_CUDA_ENOTSUP;
	EpView &v = ep.view;
	v = EpView();
	v.n_ranks = G;
	v.rank = c->cfg.ep_rank;
	v.n_local = c->n_local;
	v.n_expert = c->cfg.n_expert;
	v.top_k = c->cfg.top_k;
	v.hidden = c->cfg.hidden;
	v.t_max = c->cfg.max_tokens / G;
	v.rows_cap = (long long)c->s.rows_cap;
	size_t off = 0;
	v.off_xs = off;
	off = align_up(off + (size_t)v.t_max * v.hidden * sizeof(float), 256);
	v.off_xall = off;
	off = align_up(off + (size_t)G * v.t_max * v.hidden * sizeof(float), 256);
	v.off_ids = off;
	off = align_up(off + (size_t)v.t_max * v.top_k * sizeof(int), 256);
	v.off_topk = off;
	off = align_up(off + (size_t)v.t_max * v.top_k * sizeof(int), 256);
	v.off_inv = off;
	off = align_up(off + (size_t)v.t_max * v.top_k * sizeof(int), 256);
	v.off_counts = off;
	off = align_up(off + (size_t)v.n_expert * sizeof(int), 256);
	v.off_cntall = off;
	off = align_up(off + (size_t)G * v.n_expert * sizeof(int), 256);
	v.off_pub = off;
	off = align_up(off + EP_MAX_RANKS * sizeof(unsigned), 256);
	v.off_done = off;
	off = align_up(off + EP_MAX_RANKS * sizeof(unsigned), 256);
	v.off_y = off;
	off = align_up(off + (size_t)v.t_max * v.top_k * v.hidden * sizeof(float), 256);
	TIE_CUDA_TRY(c, cudaMalloc(reinterpret_cast<void **>(&ep.region), off));
	ep.region_bytes = off;
	// flags (and the small tables) start at zero; the token and output rows are written before they are read
	TIE_CUDA_TRY(c, cudaMemset(ep.region + v.off_ids, 0, v.off_y - v.off_ids));
	TRY(dev_alloc(c, &ep.n_rows, 1));
	TRY(dev_alloc(c, &ep.seg_base, v.n_expert + 1));
	TRY(dev_alloc(c, &ep.seg_src, v.n_expert));
	TRY(dev_alloc(c, &ep.row_dst, (size_t)v.rows_cap));
	TRY(dev_alloc(c, &ep.step_dev, 1));
	TIE_CUDA_TRY(c, cudaMemset(ep.step_dev, 0, sizeof(unsigned)));
	TIE_CUDA_TRY(c, cudaMemset(ep.n_rows, 0, sizeof(int)));
	TIE_CUDA_TRY(c, cudaDeviceSynchronize());
	int khz = 0;
	TIE_CUDA_TRY(c, cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, c->device));
	ep.wait_cycles = 5000ll * khz;	// 5 s
	return TIE_CUDA_OK;
}

}  // namespace

extern "C" {

const char *tie_cuda_version(void)
{
	return "tie_cuda 0.1 (sm_100a)";
}

const char *tie_cuda_strerror(int code)
{
	switch (code) {
	case TIE_CUDA_OK:
		return "ok";
	case TIE_CUDA_EINVAL:
		return "invalid argument";
	case TIE_CUDA_ENOTSUP:
		return "unsupported tensor type or shape";
	case TIE_CUDA_ENOMEM:
		return "out of memory";
	case TIE_CUDA_ECUDA:
		return "CUDA error";
	case TIE_CUDA_ENODEV:
		return "no usable sm_100 device";
	case TIE_CUDA_EKERNEL:
		return "kernel reported an internal check failure";
	case TIE_CUDA_ETOOBIG:
		return "size exceeds the fixed scratch of the no-allocation entry point (n_tokens <= 64, n_expert <= 256)";
	default:
		return "unknown error";
	}
}

const char *tie_cuda_last_cuda_error(const tie_cuda_ctx *c)
{
	return c ? c->cuda_err : "";
}

// engine.c:204-225 (expf_fast) and engine.c:297-303 (silu_table_init), with IEEE division.
void tie_cuda_silu_table_default(float *out)
{
	for (int i = 0; i < SILU_N; i++) {
		float x = fmaf(20.0f * (float)i, 1.0f / 8191.0f, -10.0f);
		float a = fmaxf(-88.37626266479492f, fminf(88.37626266479492f, -x));
		union {
			float f;
			int32_t i;
		} u;
		u.i = (int32_t)fmaf(12102203.0f, a, 1065353216.0f);
		float p = u.f;
		p = p * fmaf(1.9875691500E-4f, p, 1.3981999507E-3f);
		p = fmaf(p, p, p * fmaf(8.3334519073E-3f, p, 4.1665795894E-2f));
		p = fmaf(p, p, p * fmaf(1.6666665459E-1f, p, 5.0000001201E-1f));
		float e = fmaf(u.f, p, u.f);
		out[i] = x / (1.0f + e);
	}
}

int tie_cuda_init(tie_cuda_ctx **out, const tie_cuda_config *cfg)
{
	if (!out || !cfg)
		return TIE_CUDA_EINVAL;
	*out = nullptr;
	if (cfg->hidden <= 0 || cfg->hidden % QK_K || cfg->ffn_dim <= 0 || cfg->ffn_dim % QK_K || cfg->n_expert <= 0 ||
	    cfg->n_expert % 16 || cfg->n_expert > 256 || cfg->top_k <= 0 || cfg->top_k > MAX_TOP_K || cfg->top_k > cfg->n_expert ||
	    cfg->n_layers <= 0 || cfg->max_tokens <= 0 || cfg->ep_size <= 0 || cfg->ep_rank < 0 || cfg->ep_rank >= cfg->ep_size ||
	    cfg->n_expert % cfg->ep_size)
		return TIE_CUDA_EINVAL;
	int ndev = 0;
	if (cudaGetDeviceCount(&ndev) != cudaSuccess || cfg->device < 0 || cfg->device >= ndev) {
		cudaGetLastError();
		return TIE_CUDA_ENODEV;
	}
	cudaDeviceProp prop;
	if (cudaGetDeviceProperties(&prop, cfg->device) != cudaSuccess || prop.major != 10)
		return TIE_CUDA_ENODEV;
	tie_cuda_ctx *c = new (std::nothrow) tie_cuda_ctx();
	if (!c)
		return TIE_CUDA_ENOMEM;
	c->cfg = *cfg;
	c->cfg.silu_table = nullptr;
	c->device = cfg->device;
	c->sm_count = prop.multiProcessorCount;
	c->coop_ok = prop.cooperativeLaunch != 0;
	c->n_local = cfg->n_expert / cfg->ep_size;
	c->first_expert = cfg->ep_rank * c->n_local;
	int rc = TIE_CUDA_OK;
	auto fail = [&](int code) {
		tie_cuda_destroy(c);
		return code;
	};
	if (cudaSetDevice(c->device) != cudaSuccess)
		return fail(TIE_CUDA_ECUDA);
	if (cudaStreamCreateWithFlags(&c->own_stream, cudaStreamNonBlocking) != cudaSuccess)
		return fail(TIE_CUDA_ECUDA);
	c->stream = c->own_stream;
	c->layers = new (std::nothrow) Layer[cfg->n_layers];
	if (!c->layers)
		return fail(TIE_CUDA_ENOMEM);
	if (cudaMalloc(reinterpret_cast<void **>(&c->df_table), sizeof(DfLayer) * cfg->n_layers) != cudaSuccess ||
	    cudaMemset(c->df_table, 0, sizeof(DfLayer) * cfg->n_layers) != cudaSuccess)
		return fail(TIE_CUDA_ENOMEM);
	float *tab = static_cast<float *>(malloc(SILU_N * sizeof(float)));
	if (!tab)
		return fail(TIE_CUDA_ENOMEM);
	if (cfg->silu_table)
		memcpy(tab, cfg->silu_table, SILU_N * sizeof(float));
	else
		tie_cuda_silu_table_default(tab);
	cudaError_t e = cudaMalloc(reinterpret_cast<void **>(&c->silu), SILU_N * sizeof(float));
	if (e == cudaSuccess)
		e = cudaMemcpy(c->silu, tab, SILU_N * sizeof(float), cudaMemcpyHostToDevice);
	free(tab);
	if (e != cudaSuccess)
		return fail(e == cudaErrorMemoryAllocation ? TIE_CUDA_ENOMEM : TIE_CUDA_ECUDA);
	if ((rc = alloc_scratch(c)) != TIE_CUDA_OK)
		return fail(rc);
	if ((rc = tc_setup(c)) != TIE_CUDA_OK)
		return fail(rc);
	if ((rc = router_setup(c)) != TIE_CUDA_OK)
		return fail(rc);
	*out = c;
	return TIE_CUDA_OK;
}

void tie_cuda_destroy(tie_cuda_ctx *c)
{
	if (!c)
		return;
	cudaSetDevice(c->device);
	if (c->stream)
		cudaStreamSynchronize(c->stream);
	{
		std::lock_guard<std::mutex> lk(g_mutex);
		if (g_current == c)
			g_current = nullptr;
	}
	if (c->layers) {
		for (int i = 0; i < c->cfg.n_layers; i++) {
			Layer &L = c->layers[i];
			if (L.router_w)
				cudaFree(L.router_w);
			if (L.norm_w)
				cudaFree(L.norm_w);
			free_tensor(L.gate);
			free_tensor(L.up);
			free_tensor(L.down);
		}
		delete[] c->layers;
	}
	Scratch &s = c->s;
	void *dev_ptrs[] = {s.x,     s.out,   s.logits, s.bias,  s.topk_idx, s.topk_w, s.counts, s.offsets, s.tile_start, s.active, s.n_active,
			    s.perm,  s.h,     s.y,	s.xs_hi, s.hs_hi,  s.status,  s.counter, s.row_expert, c->silu,  c->row_x,
			    c->row_o, s.ep_counts, s.ep_offsets, s.ep_tile_start, s.ep_active, s.ep_n_active, s.ep_perm, s.ep_inv,
			    s.tile_info, s.xq_hi, s.hq_hi, s.dec_sync, c->df_table, s.sort_hist};
	for (void *p : dev_ptrs)
		if (p)
			cudaFree(p);
	void *pin_ptrs[] = {c->pin_x, c->pin_out, c->pin_idx, c->pin_w, c->pin_logits, c->pin_status};
	for (void *p : pin_ptrs)
		if (p)
			cudaFreeHost(p);
	for (auto &sl : c->slots) {
		if (sl.x)
			cudaFree(sl.x);
		if (sl.out)
			cudaFree(sl.out);
		if (sl.pin_status)
			cudaFreeHost(sl.pin_status);
		for (cudaEvent_t ev : {sl.in, sl.done, sl.outd})
			if (ev)
				cudaEventDestroy(ev);
	}
	if (c->h2d_stream)
		cudaStreamDestroy(c->h2d_stream);
	if (c->d2h_stream)
		cudaStreamDestroy(c->d2h_stream);
	for (int i = 0; i < c->n_graphs; i++)
		cudaGraphExecDestroy(c->graphs[i].exec);
	c->n_graphs = 0;
	for (int i = 0; i < 8; i++)
		if (c->prof_ev[i])
			cudaEventDestroy(c->prof_ev[i]);
	if (c->own_stream)
		cudaStreamDestroy(c->own_stream);
	for (int i = 0; i < c->n_extra; i++)
		cudaFree(c->extra[i]);
	free(c->extra);
	for (int i = 0; i < c->n_regs; i++) {
		if (c->regs[i].dense)
			delete c->regs[i].dense->view;
		delete c->regs[i].dense;
	}
	free(c->regs);
	ep_release(c);
	delete c;
}

int tie_cuda_set_profiling(tie_cuda_ctx *c, int on)
{
	if (!c)
		return TIE_CUDA_EINVAL;
	TIE_CUDA_TRY(c, cudaSetDevice(c->device));
	if (on && !c->prof_ev[0])
		for (int i = 0; i < 8; i++)
			TIE_CUDA_TRY(c, cudaEventCreate(&c->prof_ev[i]));
	c->prof_on = on != 0;
	return TIE_CUDA_OK;
}

int tie_cuda_get_profile(tie_cuda_ctx *c, float *phase_ms)
{
	if (!c || !phase_ms || !c->prof_ev[0])
		return TIE_CUDA_EINVAL;
	TIE_CUDA_TRY(c, cudaStreamSynchronize(c->stream));
	int prev = -1;
	for (int i = 0; i < TIE_CUDA_N_PHASES; i++)
		phase_ms[i] = 0.f;
	for (int i = 0; i <= TIE_CUDA_N_PHASES; i++) {
		if (!c->prof_set[i])
			continue;
		if (prev >= 0 && i >= 1) {
			float ms = 0.f;
			TIE_CUDA_TRY(c, cudaEventElapsedTime(&ms, c->prof_ev[prev], c->prof_ev[i]));
			phase_ms[i - 1] = ms;
		}
		prev = i;
	}
	return c->last_used_tc ? 1 : 0;
}

int tie_cuda_set_stream(tie_cuda_ctx *c, void *cuda_stream)
{
	if (!c)
		return TIE_CUDA_EINVAL;
	c->stream = static_cast<cudaStream_t>(cuda_stream);
	return TIE_CUDA_OK;
}

int tie_cuda_synchronize(tie_cuda_ctx *c)
{
	if (!c)
		return TIE_CUDA_EINVAL;
	TIE_CUDA_TRY(c, cudaStreamSynchronize(c->stream));
	return check_status(c);
}

size_t tie_cuda_weight_bytes(const tie_cuda_ctx *c)
{
	return c ? c->weight_bytes : 0;
}

uint64_t tie_cuda_launch_count(const tie_cuda_ctx *c)
{
	return c ? c->launches : 0;
}

int tie_cuda_last_active_experts(tie_cuda_ctx *c)
{
	if (!c)
		return TIE_CUDA_EINVAL;
	if (c->last_direct_rows >= 0)
		return c->last_direct_rows;
	int n = 0;
	TIE_CUDA_TRY(c, cudaMemcpyAsync(&n, c->s.n_active, sizeof(int), cudaMemcpyDeviceToHost, c->stream));
	TIE_CUDA_TRY(c, cudaStreamSynchronize(c->stream));
	return n;
}

int tie_cuda_upload_moe_layer(tie_cuda_ctx *c, int layer, const void *router_w_f32, const void *gate_exps, int gate_type,
			      const void *up_exps, int up_type, const void *down_exps, int down_type, const float *ffn_norm_w)
{
	if (!c || layer < 0 || layer >= c->cfg.n_layers || !router_w_f32 || !gate_exps || !up_exps || !down_exps)
		return TIE_CUDA_EINVAL;
	TIE_CUDA_TRY(c, cudaSetDevice(c->device));
	Layer &L = c->layers[layer];
	const int H = c->cfg.hidden, E = c->cfg.n_expert, F = c->cfg.ffn_dim;
	if (!block_bytes(gate_type) || !block_bytes(up_type) || !block_bytes(down_type))
		return TIE_CUDA_ENOTSUP;
	if (L.uploaded || L.router_w)
		forget_layer(c, layer, L);  // a re-upload: nothing may keep pointing at the tensors about to be freed
	L.uploaded = false;
	if (!L.router_w) {
		TRY(dev_alloc(c, &L.router_w, (size_t)E * H));
		c->weight_bytes += (size_t)E * H * sizeof(float);
	}
	TIE_CUDA_TRY(c, cudaMemcpyAsync(L.router_w, router_w_f32, (size_t)E * H * sizeof(float), cudaMemcpyHostToDevice, c->stream));
	L.router_host = router_w_f32;
	if (ffn_norm_w) {
		if (!L.norm_w)
			TRY(dev_alloc(c, &L.norm_w, (size_t)H));
		TIE_CUDA_TRY(c, cudaMemcpyAsync(L.norm_w, ffn_norm_w, (size_t)H * sizeof(float), cudaMemcpyHostToDevice, c->stream));
	}
	c->weight_bytes -= L.gate.bytes + L.up.bytes + L.down.bytes;
	TRY(upload_tensor(c, L.gate, gate_exps, gate_type, F, H));
	TRY(upload_tensor(c, L.up, up_exps, up_type, F, H));
	TRY(upload_tensor(c, L.down, down_exps, down_type, H, F));
	TIE_CUDA_TRY(c, cudaStreamSynchronize(c->stream));
	TRY(add_reg(c, router_w_f32, (size_t)E * H * sizeof(float), reinterpret_cast<const uint8_t *>(L.router_w), TIE_GGML_TYPE_F32,
		    W_Q4K, E, H));
	TRY(add_reg(c, gate_exps, L.gate.bytes, L.gate.ptr, gate_type, L.gate.kind, F, H));
	TRY(add_reg(c, up_exps, L.up.bytes, L.up.ptr, up_type, L.up.kind, F, H));
	TRY(add_reg(c, down_exps, L.down.bytes, L.down.ptr, down_type, L.down.kind, H, F));
	const DfLayer entry = {L.gate.ptr, L.up.ptr, L.down.ptr, L.router_w, ffn_norm_w ? L.norm_w : nullptr};
	TIE_CUDA_TRY(c, cudaMemcpy(c->df_table + layer, &entry, sizeof(entry), cudaMemcpyHostToDevice));
	L.uploaded = true;
	return TIE_CUDA_OK;
}

int tie_cuda_moe_ffn_biased(tie_cuda_ctx *c, int layer, const float *x, float *out, int n_tokens, const float *router_bias,
			    unsigned flags)
{
	Layer *L;
	TRY(get_layer(c, layer, &L));
	if (!x || !out || n_tokens <= 0 || n_tokens > c->cfg.max_tokens || c->cfg.ep_size != 1)
		return TIE_CUDA_EINVAL;
	TIE_CUDA_TRY(c, cudaSetDevice(c->device));
	const size_t bytes = (size_t)n_tokens * c->cfg.hidden * sizeof(float);
	const bool dev = flags & TIE_CUDA_DEVICE;
	const bool graph = flags & TIE_CUDA_GRAPH;
	const unsigned kflags = flags & (TIE_CUDA_DEVICE | TIE_CUDA_PATH_MASK | TIE_CUDA_PATH_LEGACY_STREAM | TIE_CUDA_ROUTE_LFM2 |
					 TIE_CUDA_PATH_DECODE_CHAIN | TIE_CUDA_PATH_NO_PAIR);
	const float *bias_dev = nullptr;
	if (router_bias) {
		if (dev) {
			bias_dev = router_bias;
		} else {
			TIE_CUDA_TRY(c, cudaMemcpyAsync(c->s.bias, router_bias, c->cfg.n_expert * sizeof(float), cudaMemcpyHostToDevice,
							c->stream));
			bias_dev = c->s.bias;
		}
	}
	if (dev) {
		GraphKey k = {1, layer, n_tokens, x, out, bias_dev, nullptr, kflags};
		TRY(run_maybe_graphed(c, graph, k, [&]() { return moe_ffn_device(c, *L, x, out, n_tokens, bias_dev, nullptr, flags); }));
		if (flags & TIE_CUDA_NO_SYNC)
			return TIE_CUDA_OK;
		return check_status(c);
	}
	// host pointers: pinned user memory is copied directly, pageable memory goes through the
	// context's pinned staging buffers
	const bool x_pinned = is_pinned_host(x), out_pinned = is_pinned_host(out);
	const void *src = x;
	void *dst = out;
	if (!x_pinned) {
		TIE_CUDA_TRY(c, cudaStreamSynchronize(c->stream));
		memcpy(c->pin_x, x, bytes);
		src = c->pin_x;
	}
	if (!out_pinned)
		dst = c->pin_out;
	GraphKey k = {2, layer, n_tokens, src, dst, bias_dev, nullptr, kflags};
	TRY(run_maybe_graphed(c, graph, k, [&]() -> int {
		TIE_CUDA_TRY(c, cudaMemcpyAsync(c->s.x, src, bytes, cudaMemcpyHostToDevice, c->stream));
		TRY(moe_ffn_device(c, *L, c->s.x, c->s.out, n_tokens, bias_dev, nullptr, flags));
		TIE_CUDA_TRY(c, cudaMemcpyAsync(dst, c->s.out, bytes, cudaMemcpyDeviceToHost, c->stream));
		TIE_CUDA_TRY(c, cudaMemcpyAsync(c->pin_status, c->s.status, sizeof(unsigned), cudaMemcpyDeviceToHost, c->stream));
		return TIE_CUDA_OK;
	}));
	TRY(check_status_pinned(c));
	if (!out_pinned)
		memcpy(out, c->pin_out, bytes);
	return TIE_CUDA_OK;
}

int tie_cuda_moe_ffn(tie_cuda_ctx *c, int layer, const float *x, float *out, int n_tokens, unsigned flags)
{
	return tie_cuda_moe_ffn_biased(c, layer, x, out, n_tokens, nullptr, flags);
}

// ---- several host-buffer calls in flight ----
// The copies of a call run on streams of their own: the input copy of call k+1 and the result copy
// of call k-1 overlap the kernels of call k (which stay on the context's stream, one call after
// the other: they share the scratch).  Slot staging and events are created on first use.
static int slot_setup(tie_cuda_ctx *c, tie_cuda_ctx::Slot &sl)
{
	if (sl.x)
		return TIE_CUDA_OK;
	const size_t n = (size_t)c->cfg.max_tokens * c->cfg.hidden;
	if (!c->h2d_stream) {
		TIE_CUDA_TRY(c, cudaStreamCreateWithFlags(&c->h2d_stream, cudaStreamNonBlocking));
		TIE_CUDA_TRY(c, cudaStreamCreateWithFlags(&c->d2h_stream, cudaStreamNonBlocking));
	}
	TRY(dev_alloc(c, &sl.x, n));
	TRY(dev_alloc(c, &sl.out, n));
	TIE_CUDA_TRY(c, cudaMallocHost(reinterpret_cast<void **>(&sl.pin_status), sizeof(unsigned)));
	TIE_CUDA_TRY(c, cudaEventCreateWithFlags(&sl.in, cudaEventDisableTiming));
	TIE_CUDA_TRY(c, cudaEventCreateWithFlags(&sl.done, cudaEventDisableTiming));
	TIE_CUDA_TRY(c, cudaEventCreateWithFlags(&sl.outd, cudaEventDisableTiming));
	return TIE_CUDA_OK;
}

int tie_cuda_moe_ffn_submit(tie_cuda_ctx *c, int layer, const float *x_host, float *out_host, int n_tokens, int slot, unsigned flags)
{
	Layer *L;
	TRY(get_layer(c, layer, &L));
	if (!x_host || !out_host || n_tokens <= 0 || n_tokens > c->cfg.max_tokens || c->cfg.ep_size != 1 || slot < 0 || slot >= TIE_CUDA_N_SLOTS ||
	    (flags & TIE_CUDA_DEVICE) || c->stream == nullptr)
		return TIE_CUDA_EINVAL;
	tie_cuda_ctx::Slot &sl = c->slots[slot];
	if (sl.busy)  // the previous call on this slot has not been waited for
		return TIE_CUDA_EINVAL;
	// (pageable memory would make the copies synchronous: the point of the call is lost, so it is refused)
	if (!is_pinned_host(x_host) || !is_pinned_host(out_host))
		return TIE_CUDA_ENOTSUP;
	TIE_CUDA_TRY(c, cudaSetDevice(c->device));
	TRY(slot_setup(c, sl));
	const size_t bytes = (size_t)n_tokens * c->cfg.hidden * sizeof(float);
	// input: after the kernels of this slot's previous call have read its x (they precede `done`)
	if (sl.done)
		TIE_CUDA_TRY(c, cudaStreamWaitEvent(c->h2d_stream, sl.done, 0));
	TIE_CUDA_TRY(c, cudaMemcpyAsync(sl.x, x_host, bytes, cudaMemcpyHostToDevice, c->h2d_stream));
	TIE_CUDA_TRY(c, cudaEventRecord(sl.in, c->h2d_stream));
	// kernels: after the input has landed and this slot's previous result has left the device
	TIE_CUDA_TRY(c, cudaStreamWaitEvent(c->stream, sl.in, 0));
	TIE_CUDA_TRY(c, cudaStreamWaitEvent(c->stream, sl.outd, 0));
	const unsigned dflags = (flags & ~(TIE_CUDA_HOST | TIE_CUDA_NO_SYNC)) | TIE_CUDA_DEVICE;
	const unsigned kflags = dflags & (TIE_CUDA_DEVICE | TIE_CUDA_PATH_MASK | TIE_CUDA_PATH_LEGACY_STREAM | TIE_CUDA_ROUTE_LFM2 |
					  TIE_CUDA_PATH_DECODE_CHAIN | TIE_CUDA_PATH_NO_PAIR);
	GraphKey k = {1, layer, n_tokens, sl.x, sl.out, nullptr, nullptr, kflags};
	TRY(run_maybe_graphed(c, flags & TIE_CUDA_GRAPH, k,
			      [&]() { return moe_ffn_device(c, *L, sl.x, sl.out, n_tokens, nullptr, nullptr, dflags); }));
	TIE_CUDA_TRY(c, cudaEventRecord(sl.done, c->stream));
	// result and status word
	TIE_CUDA_TRY(c, cudaStreamWaitEvent(c->d2h_stream, sl.done, 0));
	TIE_CUDA_TRY(c, cudaMemcpyAsync(out_host, sl.out, bytes, cudaMemcpyDeviceToHost, c->d2h_stream));
	TIE_CUDA_TRY(c, cudaMemcpyAsync(sl.pin_status, c->s.status, sizeof(unsigned), cudaMemcpyDeviceToHost, c->d2h_stream));
	TIE_CUDA_TRY(c, cudaEventRecord(sl.outd, c->d2h_stream));
	sl.busy = true;
	return TIE_CUDA_OK;
}

int tie_cuda_moe_ffn_wait(tie_cuda_ctx *c, int slot)
{
	if (!c || slot < 0 || slot >= TIE_CUDA_N_SLOTS || !c->slots[slot].busy)
		return TIE_CUDA_EINVAL;
	tie_cuda_ctx::Slot &sl = c->slots[slot];
	TIE_CUDA_TRY(c, cudaSetDevice(c->device));
	TIE_CUDA_TRY(c, cudaEventSynchronize(sl.outd));
	sl.busy = false;
	return report_status(c, *static_cast<volatile unsigned *>(sl.pin_status));
}

int tie_cuda_moe_block_inplace(tie_cuda_ctx *c, int layer, float *hidden_dev, int n_tokens, unsigned flags)
{
	Layer *L;
	TRY(get_layer(c, layer, &L));
	if (!hidden_dev || n_tokens <= 0 || n_tokens > c->cfg.max_tokens || c->cfg.ep_size != 1)
		return TIE_CUDA_EINVAL;
	TIE_CUDA_TRY(c, cudaSetDevice(c->device));
	GraphKey k = {3, layer, n_tokens, hidden_dev, nullptr, nullptr, nullptr,
		      flags & (TIE_CUDA_PATH_MASK | TIE_CUDA_PATH_LEGACY_STREAM | TIE_CUDA_PATH_DECODE_CHAIN | TIE_CUDA_ROUTE_LFM2 |
			       TIE_CUDA_PATH_NO_PAIR)};
	TRY(run_maybe_graphed(c, flags & TIE_CUDA_GRAPH, k, [&]() -> int {
		// one token: the RMSNorm is part of the one-kernel step
		if ((flags & TIE_CUDA_PATH_MASK) != TIE_CUDA_PATH_TENSOR &&
		    !(flags & (TIE_CUDA_PATH_LEGACY_STREAM | TIE_CUDA_PATH_DECODE_CHAIN | TIE_CUDA_ROUTE_LFM2)) &&
		    decode_fused_supported(c, *L, n_tokens)) {
			const int rc = launch_decode_fused(c, *L, hidden_dev, nullptr, hidden_dev, hidden_dev, L->norm_w, c->cfg.norm_eps);
			if (rc != TIE_CUDA_ENOTSUP) {
				if (!rc) {
					c->last_used_tc = false;
					c->last_direct_rows = c->cfg.top_k;
				}
				return rc;
			}
		}
		TRY(launch_rms_norm(c, hidden_dev, L->norm_w, c->s.x, n_tokens));
		return moe_ffn_device(c, *L, c->s.x, hidden_dev, n_tokens, nullptr, hidden_dev, flags);
	}));
	if (flags & TIE_CUDA_NO_SYNC)
		return TIE_CUDA_OK;
	return check_status(c);
}

int tie_cuda_moe_stack_inplace(tie_cuda_ctx *c, int first_layer, int n_layers, float *hidden_dev, int n_tokens, unsigned flags)
{
	if (!c || n_layers <= 0 || first_layer < 0 || first_layer + n_layers > c->cfg.n_layers || !hidden_dev || n_tokens <= 0 ||
	    n_tokens > c->cfg.max_tokens || c->cfg.ep_size != 1)
		return TIE_CUDA_EINVAL;
	for (int l = first_layer; l < first_layer + n_layers; l++)
		if (!c->layers[l].uploaded)
			return TIE_CUDA_EINVAL;
	TIE_CUDA_TRY(c, cudaSetDevice(c->device));
	const unsigned pflags = flags & (TIE_CUDA_PATH_MASK | TIE_CUDA_PATH_LEGACY_STREAM | TIE_CUDA_PATH_DECODE_CHAIN | TIE_CUDA_ROUTE_LFM2 |
					 TIE_CUDA_PATH_NO_PAIR);
	const bool decode_paths = (pflags & TIE_CUDA_PATH_MASK) != TIE_CUDA_PATH_TENSOR &&
				  !(pflags & (TIE_CUDA_PATH_LEGACY_STREAM | TIE_CUDA_PATH_DECODE_CHAIN | TIE_CUDA_ROUTE_LFM2));
	// (one token through all layers in ONE launch is tried first where the layers share tensor types;
	// launch_decode_fused_stack reports "not supported" while that kernel is not built)
	const Layer &L0 = c->layers[first_layer];
	bool one_launch = n_tokens == 1 && n_layers > 1 && decode_paths && decode_fused_supported(c, L0, 1);
	for (int l = first_layer + 1; l < first_layer + n_layers && one_launch; l++) {
		const Layer &L = c->layers[l];
		one_launch = L.gate.kind == L0.gate.kind && L.up.kind == L0.up.kind && L.down.kind == L0.down.kind &&
			     L.gate.expert_stride == L0.gate.expert_stride && L.down.expert_stride == L0.down.expert_stride;
	}
	GraphKey k = {8, first_layer, n_tokens, hidden_dev, nullptr, nullptr, reinterpret_cast<const void *>((size_t)n_layers), pflags};
	TRY(run_maybe_graphed(c, flags & TIE_CUDA_GRAPH, k, [&]() -> int {
		if (one_launch) {
			const int rc = launch_decode_fused_stack(c, first_layer, n_layers, hidden_dev);
			if (rc != TIE_CUDA_ENOTSUP) {
				if (!rc) {
					c->last_used_tc = false;
					c->last_direct_rows = c->cfg.top_k;
				}
				return rc;
			}
		}
		for (int l = first_layer; l < first_layer + n_layers; l++) {
			Layer &L = c->layers[l];
			if (decode_paths && decode_fused_supported(c, L, n_tokens)) {
				const Layer *next = l + 1 < first_layer + n_layers ? &c->layers[l + 1] : nullptr;
				const int rc = launch_decode_fused(c, L, hidden_dev, nullptr, hidden_dev, hidden_dev, L.norm_w, c->cfg.norm_eps, next);
				if (rc != TIE_CUDA_ENOTSUP) {
					if (rc)
						return rc;
					continue;
				}
			}
			TRY(launch_rms_norm(c, hidden_dev, L.norm_w, c->s.x, n_tokens));
			TRY(moe_ffn_device(c, L, c->s.x, hidden_dev, n_tokens, nullptr, hidden_dev, pflags));
		}
		return TIE_CUDA_OK;
	}));
	if (flags & TIE_CUDA_NO_SYNC)
		return TIE_CUDA_OK;
	return check_status(c);
}

int tie_cuda_moe_route(tie_cuda_ctx *c, int layer, const float *x, int n_tokens, const float *router_bias, int *topk_idx,
		       float *topk_w, float *logits, unsigned flags)
{
	Layer *L;
	TRY(get_layer(c, layer, &L));
	if (!x || !topk_idx || !topk_w || n_tokens <= 0 || n_tokens > c->cfg.max_tokens)
		return TIE_CUDA_EINVAL;
	TIE_CUDA_TRY(c, cudaSetDevice(c->device));
	const int H = c->cfg.hidden, E = c->cfg.n_expert, K = c->cfg.top_k;
	Scratch &s = c->s;
	if (flags & TIE_CUDA_DEVICE) {
		TRY(launch_router(c, x, L->router_w, router_bias, n_tokens, logits ? logits : s.logits, topk_idx, topk_w,
				  (flags & TIE_CUDA_ROUTE_LFM2) ? 1 : 0));
		if (flags & TIE_CUDA_NO_SYNC)
			return TIE_CUDA_OK;
		return check_status(c);
	}
	const float *bias_dev = nullptr;
	if (router_bias) {
		TIE_CUDA_TRY(c, cudaMemcpyAsync(s.bias, router_bias, E * sizeof(float), cudaMemcpyHostToDevice, c->stream));
		bias_dev = s.bias;
	}
	TRY(h2d(c, s.x, x, (size_t)n_tokens * H * sizeof(float), c->pin_x));
	TRY(launch_router(c, s.x, L->router_w, bias_dev, n_tokens, s.logits, s.topk_idx, s.topk_w, (flags & TIE_CUDA_ROUTE_LFM2) ? 1 : 0));
	TIE_CUDA_TRY(c, cudaMemcpyAsync(c->pin_idx, s.topk_idx, (size_t)n_tokens * K * sizeof(int), cudaMemcpyDeviceToHost, c->stream));
	TIE_CUDA_TRY(c, cudaMemcpyAsync(c->pin_w, s.topk_w, (size_t)n_tokens * K * sizeof(float), cudaMemcpyDeviceToHost, c->stream));
	if (logits)
		TIE_CUDA_TRY(c, cudaMemcpyAsync(c->pin_logits, s.logits, (size_t)n_tokens * E * sizeof(float), cudaMemcpyDeviceToHost,
						c->stream));
	TRY(check_status(c));
	memcpy(topk_idx, c->pin_idx, (size_t)n_tokens * K * sizeof(int));
	memcpy(topk_w, c->pin_w, (size_t)n_tokens * K * sizeof(float));
	if (logits)
		memcpy(logits, c->pin_logits, (size_t)n_tokens * E * sizeof(float));
	return TIE_CUDA_OK;
}

int tie_cuda_moe_expert_rows(tie_cuda_ctx *c, int layer, const float *x_rows, const int *row_expert, int n_rows, float *y_rows,
			     unsigned flags)
{
	Layer *L;
	TRY(get_layer(c, layer, &L));
	if (!(flags & TIE_CUDA_DEVICE) || !x_rows || !row_expert || !y_rows || n_rows < 0 || (size_t)n_rows > c->s.rows_cap)
		return TIE_CUDA_EINVAL;
	if (n_rows == 0)
		return TIE_CUDA_OK;
	TIE_CUDA_TRY(c, cudaSetDevice(c->device));
	TRY(run_experts(c, *L, x_rows, 1, row_expert, n_rows, y_rows, flags));
	if (flags & TIE_CUDA_NO_SYNC)
		return TIE_CUDA_OK;
	return check_status(c);
}

int tie_cuda_moe_combine(tie_cuda_ctx *c, const float *y_rows, const float *topk_w, int n_tokens, float *out, unsigned flags)
{
	if (!c || !(flags & TIE_CUDA_DEVICE) || !y_rows || !topk_w || !out || n_tokens <= 0)
		return TIE_CUDA_EINVAL;
	TIE_CUDA_TRY(c, cudaSetDevice(c->device));
	TRY(launch_combine(c, y_rows, topk_w, n_tokens, nullptr, out));
	if (flags & TIE_CUDA_NO_SYNC)
		return TIE_CUDA_OK;
	return check_status(c);
}

int tie_cuda_moe_ep_dispatch(tie_cuda_ctx *c, const float *x, const int *topk_idx, int n_tokens, float *send_rows,
			     int *send_expert, int *expert_counts, unsigned flags)
{
	if (!c || !(flags & TIE_CUDA_DEVICE) || !x || !topk_idx || !send_rows || !send_expert || !expert_counts || n_tokens <= 0 ||
	    (size_t)n_tokens * c->cfg.top_k > c->s.rows_cap)
		return TIE_CUDA_EINVAL;
	TIE_CUDA_TRY(c, cudaSetDevice(c->device));
	Scratch &s = c->s;
	const int R = n_tokens * c->cfg.top_k;
	SortBufs b = {expert_counts, s.ep_offsets, s.ep_tile_start, s.ep_active, s.ep_n_active, s.ep_perm, nullptr};
	TRY(launch_sort(c, topk_idx, R, 128, 0, c->cfg.n_expert, b));
	TRY(launch_gather_rows(c, x, topk_idx, s.ep_perm, c->cfg.top_k, R, send_rows, send_expert, s.ep_inv));
	if (flags & TIE_CUDA_NO_SYNC)
		return TIE_CUDA_OK;
	return check_status(c);
}

int tie_cuda_moe_ep_combine(tie_cuda_ctx *c, const float *y_sorted, const float *topk_w, int n_tokens, float *out, unsigned flags)
{
	if (!c || !(flags & TIE_CUDA_DEVICE) || !y_sorted || !topk_w || !out || n_tokens <= 0 ||
	    (size_t)n_tokens * c->cfg.top_k > c->s.rows_cap)
		return TIE_CUDA_EINVAL;
	TIE_CUDA_TRY(c, cudaSetDevice(c->device));
	TRY(launch_combine(c, y_sorted, topk_w, n_tokens, nullptr, out, c->s.ep_inv));
	if (flags & TIE_CUDA_NO_SYNC)
		return TIE_CUDA_OK;
	return check_status(c);
}

// ---- expert parallelism over peer memory (ep.cu) ----

int tie_cuda_ep_region(tie_cuda_ctx *c, void **base, size_t *bytes)
{
	if (!c)
		return TIE_CUDA_EINVAL;
	TIE_CUDA_TRY(c, cudaSetDevice(c->device));
	TRY(ep_region(c));
	if (base)
		*base = c->ep.region;
	if (bytes)
		*bytes = c->ep.region_bytes;
	return TIE_CUDA_OK;
}

int tie_cuda_ep_ipc_handle(tie_cuda_ctx *c, void *handle)
{
	static_assert(sizeof(cudaIpcMemHandle_t) == TIE_CUDA_EP_HANDLE_BYTES, "handle size");
	if (!c || !handle)
		return TIE_CUDA_EINVAL;
	TIE_CUDA_TRY(c, cudaSetDevice(c->device));
	TRY(ep_region(c));
	cudaIpcMemHandle_t h;
	TIE_CUDA_TRY(c, cudaIpcGetMemHandle(&h, c->ep.region));
	memcpy(handle, &h, sizeof(h));
	return TIE_CUDA_OK;
}

int tie_cuda_ep_attach(tie_cuda_ctx *c, const void *const *peers, int n_peers, int kind)
{
	if (!c || !peers || n_peers != c->cfg.ep_size || (kind != TIE_CUDA_EP_PEER_POINTERS && kind != TIE_CUDA_EP_PEER_IPC_HANDLES))
		return TIE_CUDA_EINVAL;
	TIE_CUDA_TRY(c, cudaSetDevice(c->device));
	TRY(ep_region(c));
	EpState &ep = c->ep;
	if (ep.attached)
		return TIE_CUDA_EINVAL;
	for (int i = 0; i < n_peers; i++) {
		if (i == c->cfg.ep_rank) {
			ep.view.peer[i] = ep.region;
			continue;
		}
		if (!peers[i]) {
			ep_close_peers(c);
			return TIE_CUDA_EINVAL;
		}
		if (kind == TIE_CUDA_EP_PEER_POINTERS) {
			ep.view.peer[i] = static_cast<uint8_t *>(const_cast<void *>(peers[i]));
		} else {
			cudaIpcMemHandle_t h;
			memcpy(&h, peers[i], sizeof(h));
			void *p = nullptr;
			cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
			if (e != cudaSuccess) {
				snprintf(c->cuda_err, sizeof(c->cuda_err), "cudaIpcOpenMemHandle(rank %d): %s", i, cudaGetErrorString(e));
				cudaGetLastError();
				ep_close_peers(c);
				return TIE_CUDA_ECUDA;
			}
			ep.view.peer[i] = static_cast<uint8_t *>(p);
			ep.opened[i] = true;
		}
	}
	// An attach starts a new epoch: the step counter and the flags the peers store into this rank's
	// region go back to zero, so that a group that re-forms after a time-out (where the ranks' step
	// numbers differ and stale flags are left behind) agrees again.  The caller separates the
	// attaches of all ranks from the first publish by a host barrier (a peer's first flag must not
	// arrive before this reset), and the detaches of all ranks from the attaches by another.
	cudaError_t e = cudaMemsetAsync(ep.step_dev, 0, sizeof(unsigned), c->stream);
	if (e == cudaSuccess)
		e = cudaMemsetAsync(ep.region + ep.view.off_pub, 0, EP_MAX_RANKS * sizeof(unsigned), c->stream);
	if (e == cudaSuccess)
		e = cudaMemsetAsync(ep.region + ep.view.off_done, 0, EP_MAX_RANKS * sizeof(unsigned), c->stream);
	if (e == cudaSuccess)
		e = cudaStreamSynchronize(c->stream);
	if (e != cudaSuccess) {
		snprintf(c->cuda_err, sizeof(c->cuda_err), "ep_attach: %s", cudaGetErrorString(e));
		ep_close_peers(c);
		return TIE_CUDA_ECUDA;
	}
	ep.attached = true;
	ep.phase = 0;
	return TIE_CUDA_OK;
}

int tie_cuda_ep_detach(tie_cuda_ctx *c)
{
	if (!c)
		return TIE_CUDA_EINVAL;
	cudaSetDevice(c->device);
	if (c->stream)
		cudaStreamSynchronize(c->stream);
	ep_close_peers(c);
	return TIE_CUDA_OK;
}

int tie_cuda_ep_set_timeout_ms(tie_cuda_ctx *c, int ms)
{
	if (!c || ms <= 0)
		return TIE_CUDA_EINVAL;
	int khz = 0;
	TIE_CUDA_TRY(c, cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, c->device));
	c->ep.wait_cycles = (long long)ms * khz;
	return TIE_CUDA_OK;
}

int tie_cuda_ep_publish(tie_cuda_ctx *c, int layer, const float *x, int n_tokens, const float *router_bias, unsigned flags)
{
	Layer *L;
	TRY(get_layer(c, layer, &L));
	EpState &ep = c->ep;
	if (!(flags & TIE_CUDA_DEVICE) || !ep.attached || ep.phase != 0 || n_tokens < 0 || n_tokens > ep.view.t_max || (n_tokens && !x))
		return TIE_CUDA_EINVAL;
	if (flags & TIE_CUDA_EP_REPLICATED) {
		// decode on replicated tokens: announce the step, route; nothing is dispatched
		if (n_tokens < 1 || n_tokens > 4 || (flags & TIE_CUDA_ROUTE_LFM2))
			return TIE_CUDA_EINVAL;
		if (!decode_supported(c, *L, n_tokens))
			return TIE_CUDA_ENOTSUP;
		TIE_CUDA_TRY(c, cudaSetDevice(c->device));
		prof_mark(c, 0);
		TRY(launch_ep_signal(c, 0));
		TRY(launch_router_decode_fused(c, x, L->router_w, router_bias, n_tokens, c->s.logits, c->s.topk_idx, c->s.topk_w));
		prof_mark(c, 1);
		prof_mark(c, 2);
		ep.phase = 1;
		ep.step_tokens = n_tokens;
		ep.replicated = true;
		ep.rep_x = x;
		if (flags & TIE_CUDA_NO_SYNC)
			return TIE_CUDA_OK;
		return check_status(c);
	}
	if (!tc_supported(c, *L))
		return TIE_CUDA_ENOTSUP;
	TIE_CUDA_TRY(c, cudaSetDevice(c->device));
	Scratch &s = c->s;
	const EpView &v = ep.view;
	const int R = n_tokens * c->cfg.top_k;
	ep.replicated = false;
	prof_mark(c, 0);
	// the selected experts go where the peers can read them: the owner of a token's first row on a GPU
	// looks up the token's other rows there
	int *topk_pub = reinterpret_cast<int *>(ep.region + v.off_topk);
	// The tokens do not depend on the routing: they go to every rank's memory beside the router, as
	// extra CTAs of its kernel (or, for shapes whose router kernel cannot take them along, as a launch
	// of its own); the pub flag below announces them together with the row lists.
	if (n_tokens) {
		const EpPush push = ep_push_args(c, x, n_tokens);
		bool taken = false;
		TRY(launch_router(c, x, L->router_w, router_bias, n_tokens, s.logits, topk_pub, s.topk_w, (flags & TIE_CUDA_ROUTE_LFM2) ? 1 : 0,
				  &push, &taken));
		if (!taken)
			TRY(launch_ep_push_tokens(c, x, n_tokens));
	}
	prof_mark(c, 1);
	SortBufs b = {reinterpret_cast<int *>(ep.region + v.off_counts),
		      s.ep_offsets,
		      s.ep_tile_start,
		      s.ep_active,
		      s.ep_n_active,
		      reinterpret_cast<int *>(ep.region + v.off_ids),
		      nullptr};
	b.inv = reinterpret_cast<int *>(ep.region + v.off_inv);
	b.owner_div = c->n_local;
	b.top_k = c->cfg.top_k;
	TRY(launch_sort(c, topk_pub, R, 128, 0, c->cfg.n_expert, b));
	TRY(launch_ep_signal(c, 0));
	prof_mark(c, 2);
	ep.phase = 1;
	ep.step_tokens = n_tokens;
	if (flags & TIE_CUDA_NO_SYNC)
		return TIE_CUDA_OK;
	return check_status(c);
}

int tie_cuda_ep_compute(tie_cuda_ctx *c, int layer, unsigned flags)
{
	Layer *L;
	TRY(get_layer(c, layer, &L));
	EpState &ep = c->ep;
	if (!ep.attached || ep.phase != 1)
		return TIE_CUDA_EINVAL;
	if (ep.replicated) {
		TIE_CUDA_TRY(c, cudaSetDevice(c->device));
		prof_mark(c, 3);
		TRY(launch_decode_gate_up(c, *L, ep.rep_x, ep.step_tokens, true));
		prof_mark(c, 4);
		TRY(launch_decode_down_peer(c, *L, ep.step_tokens));
		TRY(launch_ep_signal(c, 1));
		prof_mark(c, 6);
		c->last_used_tc = false;
		c->last_direct_rows = ep.step_tokens * c->cfg.top_k;
		ep.phase = 2;
		if (flags & TIE_CUDA_NO_SYNC)
			return TIE_CUDA_OK;
		return check_status(c);
	}
	if (!tc_supported(c, *L))
		return TIE_CUDA_ENOTSUP;
	TIE_CUDA_TRY(c, cudaSetDevice(c->device));
	c->tc_no_pair = (flags & TIE_CUDA_PATH_NO_PAIR) != 0;
	TRY(launch_ep_index(c));
	TRY(launch_ep_split_rows(c, L->gate.kind == W_Q4K));
	prof_mark(c, 3);
	TRY(launch_tc_gate_up(c, *L, 0));
	prof_mark(c, 4);
	TRY(launch_tc_swiglu(c, *L, c->sm_count * 8, ep.n_rows));
	prof_mark(c, 5);
	EpDst dst;
	for (int i = 0; i < ep.view.n_ranks; i++)
		dst.y[i] = reinterpret_cast<float *>(ep.view.peer[i] + ep.view.off_y);
	dst.row = ep.row_dst;
	TRY(launch_tc_down_peer(c, *L, dst));
	TRY(launch_ep_signal(c, 1));
	prof_mark(c, 6);
	c->last_used_tc = true;
	c->last_direct_rows = -1;
	ep.phase = 2;
	if (flags & TIE_CUDA_NO_SYNC)
		return TIE_CUDA_OK;
	return check_status(c);
}

int tie_cuda_ep_gather(tie_cuda_ctx *c, float *out, const float *residual, unsigned flags)
{
	if (!c)
		return TIE_CUDA_EINVAL;
	EpState &ep = c->ep;
	if (!ep.attached || ep.phase != 2 || (ep.step_tokens > 0 && !out))
		return TIE_CUDA_EINVAL;
	TIE_CUDA_TRY(c, cudaSetDevice(c->device));
	// (a rank without tokens still waits for its peers: they read its counts during compute)
	TRY(launch_ep_combine(c, ep.step_tokens, residual, out));
	prof_mark(c, 7);
	ep.phase = 0;
	ep.step_tokens = -1;
	ep.replicated = false;
	if (flags & TIE_CUDA_NO_SYNC)
		return TIE_CUDA_OK;
	return check_status(c);
}

int tie_cuda_moe_ffn_ep(tie_cuda_ctx *c, int layer, const float *x, float *out, int n_tokens, unsigned flags)
{
	if (!c || c->ep.phase != 0)
		return TIE_CUDA_EINVAL;
	const unsigned inner = (flags | TIE_CUDA_NO_SYNC) & ~TIE_CUDA_GRAPH;
	// the step number lives on the device: a step's launches never change and replay from a graph
	GraphKey k = {5, layer, n_tokens, x, out, nullptr, nullptr, inner};
	TRY(run_maybe_graphed(c, flags & TIE_CUDA_GRAPH, k, [&]() -> int {
		int rc = tie_cuda_ep_publish(c, layer, x, n_tokens, nullptr, inner);
		if (!rc)
			rc = tie_cuda_ep_compute(c, layer, inner);
		if (!rc)
			rc = tie_cuda_ep_gather(c, out, nullptr, inner);
		if (rc) {  // nothing of a failed capture runs
			c->ep.phase = 0;
			c->ep.step_tokens = -1;
		}
		return rc;
	}));
	if (flags & TIE_CUDA_NO_SYNC)
		return TIE_CUDA_OK;
	return check_status(c);
}

int tie_cuda_moe_block_inplace_ep(tie_cuda_ctx *c, int layer, float *hidden_dev, int n_tokens, unsigned flags)
{
	Layer *L;
	TRY(get_layer(c, layer, &L));
	EpState &ep = c->ep;
	if (!ep.attached || ep.phase != 0 || n_tokens < 0 || n_tokens > ep.view.t_max || (n_tokens && !hidden_dev))
		return TIE_CUDA_EINVAL;
	TIE_CUDA_TRY(c, cudaSetDevice(c->device));
	const unsigned inner = (flags | TIE_CUDA_NO_SYNC | TIE_CUDA_DEVICE) & ~TIE_CUDA_GRAPH;
	// (decode on replicated tokens: the normed rows stay in this rank's scratch, nobody else reads them)
	float *xs = (flags & TIE_CUDA_EP_REPLICATED) ? c->s.x : reinterpret_cast<float *>(ep.region + ep.view.off_xs);
	GraphKey k = {6, layer, n_tokens, hidden_dev, nullptr, nullptr, nullptr, inner};
	TRY(run_maybe_graphed(c, flags & TIE_CUDA_GRAPH, k, [&]() -> int {
		// the normed tokens go straight to where the peers read them
		int rc = n_tokens ? launch_rms_norm(c, hidden_dev, L->norm_w, xs, n_tokens) : TIE_CUDA_OK;
		if (!rc)
			rc = tie_cuda_ep_publish(c, layer, xs, n_tokens, nullptr, inner);
		if (!rc)
			rc = tie_cuda_ep_compute(c, layer, inner);
		if (!rc)
			rc = tie_cuda_ep_gather(c, hidden_dev, hidden_dev, inner);
		if (rc) {
			c->ep.phase = 0;
			c->ep.step_tokens = -1;
		}
		return rc;
	}));
	if (flags & TIE_CUDA_NO_SYNC)
		return TIE_CUDA_OK;
	return check_status(c);
}

// ---- math_dispatch rows ----

int tie_cuda_make_current(tie_cuda_ctx *c)
{
	std::lock_guard<std::mutex> lk(g_mutex);
	g_current = c;
	g_dispatch_status = 0;
	return TIE_CUDA_OK;
}

int tie_cuda_dispatch_status(void)
{
	return g_dispatch_status;
}

int tie_cuda_register_tensor(tie_cuda_ctx *c, const void *host_ptr, size_t n_bytes, int ggml_type, int in_dim)
{
	if (!c || !host_ptr || !n_bytes || in_dim <= 0)
		return TIE_CUDA_EINVAL;
	TIE_CUDA_TRY(c, cudaSetDevice(c->device));
	size_t row_bytes;
	if (ggml_type == TIE_GGML_TYPE_F32) {
		row_bytes = (size_t)in_dim * 4;
	} else {
		if (!block_bytes(ggml_type) || in_dim % QK_K)
			return TIE_CUDA_ENOTSUP;
		row_bytes = (size_t)(in_dim / QK_K) * block_bytes(ggml_type);
	}
	if (n_bytes % row_bytes)
		return TIE_CUDA_EINVAL;
	const size_t rows = n_bytes / row_bytes;
	const WKind kind = (ggml_type == TIE_GGML_TYPE_Q6_K) ? W_Q6K_R8 : W_Q4K;
	if (kind == W_Q6K_R8 && rows % 8)
		return TIE_CUDA_ENOTSUP;
	if (c->n_extra == c->cap_extra) {
		int nc = c->cap_extra ? c->cap_extra * 2 : 16;
		void *p = realloc(c->extra, nc * sizeof(uint8_t *));
		if (!p)
			return TIE_CUDA_ENOMEM;
		c->extra = static_cast<uint8_t **>(p);
		c->cap_extra = nc;
	}
	uint8_t *dev = nullptr;
	TIE_CUDA_TRY(c, cudaMalloc(reinterpret_cast<void **>(&dev), n_bytes));
	c->extra[c->n_extra++] = dev;
	if (kind == W_Q6K_R8) {
		uint8_t *raw = nullptr;
		TIE_CUDA_TRY(c, cudaMalloc(reinterpret_cast<void **>(&raw), n_bytes));
		cudaError_t e = cudaMemcpyAsync(raw, host_ptr, n_bytes, cudaMemcpyHostToDevice, c->stream);
		int rc = (e == cudaSuccess) ? launch_repack_q6k_r8(c, raw, dev, rows, in_dim / QK_K) : TIE_CUDA_ECUDA;
		cudaStreamSynchronize(c->stream);
		cudaFree(raw);
		if (rc)
			return rc;
	} else {
		TIE_CUDA_TRY(c, cudaMemcpyAsync(dev, host_ptr, n_bytes, cudaMemcpyHostToDevice, c->stream));
		TIE_CUDA_TRY(c, cudaStreamSynchronize(c->stream));
	}
	c->weight_bytes += n_bytes;
	DevTensor *dense = nullptr;
	if (ggml_type != TIE_GGML_TYPE_F32) {  // the view tie_cuda_mat_mat takes: one "expert" holding every row
		dense = new DevTensor();
		dense->ptr = dev;
		dense->ggml_type = ggml_type;
		dense->kind = kind;
		dense->rows = (int)rows;
		dense->k = in_dim;
		dense->expert_stride = n_bytes;
		dense->bytes = n_bytes;
		dense->host_ptr = host_ptr;
		int rc = tc_make_weight_map(c, *dense, 1);
		if (!rc && dense->has_map)
			rc = tc_make_dense_view(c, *dense);
		if (rc) {
			delete dense->view;
			delete dense;
			return rc;
		}
	}
	return add_reg(c, host_ptr, n_bytes, dev, ggml_type, kind, (int)rows, in_dim, dense);
}

int tie_cuda_mat_mat(tie_cuda_ctx *c, const void *w_host, const float *x, float *o, int batch_len, int in_dim, int out_dim,
		     unsigned flags)
{
	if (!c || !w_host || !x || !o || batch_len <= 0 || in_dim <= 0 || out_dim <= 0)
		return TIE_CUDA_EINVAL;
	const tie_cuda_ctx::Reg *reg = nullptr;
	for (int i = 0; i < c->n_regs; i++)
		if (c->regs[i].host == w_host)
			reg = &c->regs[i];
	if (!reg || reg->k != in_dim || reg->rows != out_dim)
		return TIE_CUDA_EINVAL;
	if (!reg->dense || !tc_dense_supported(c, *reg->dense))
		return TIE_CUDA_ENOTSUP;
	Scratch &s = c->s;
	const DenseView &v = *reg->dense->view;
	const size_t T = c->cfg.max_tokens, H = c->cfg.hidden, F = c->cfg.ffn_dim;
	const size_t y_cap = s.rows_cap * (H > 2 * F ? H : 2 * F);
	// (a token box of up to 64 rows may start at the last row: keep that much of the view beyond the batch)
	if ((size_t)batch_len > s.rows_cap || (size_t)batch_len + 64 > v.rows || (size_t)batch_len * out_dim > y_cap)
		return TIE_CUDA_ETOOBIG;
	TIE_CUDA_TRY(c, cudaSetDevice(c->device));
	c->tc_no_pair = (flags & TIE_CUDA_PATH_NO_PAIR) != 0;
	const bool dev = flags & TIE_CUDA_DEVICE;
	const float *x_dev = x;
	float *o_dev = o;
	if (!dev) {
		if ((size_t)batch_len * in_dim > T * H)
			return TIE_CUDA_ETOOBIG;
		TRY(h2d(c, s.x, x, (size_t)batch_len * in_dim * sizeof(float), c->pin_x));
		x_dev = s.x;
		o_dev = s.y;
	}
	// one "expert" owning every row: the tile table of the grouped product, rows in input order
	TIE_CUDA_TRY(c, cudaMemsetAsync(s.row_expert, 0, (size_t)batch_len * sizeof(int), c->stream));
	SortBufs b = {s.counts, s.offsets, s.tile_start, s.active, s.n_active, s.perm, s.tile_info};
	TRY(launch_sort(c, s.row_expert, batch_len, TC_TOKEN_TILE, 0, 1, b));
	// the batch, split into fp16 hi + lo (and its sub-block sums for Q4_K), in the tensor's view of the x arrays.
	// Columns of the sums that the row length leaves unused are read as padding of a 16-deep k step
	// and must be zero, in this view and, afterwards, in the context's own.
	const bool sums = reg->dense->kind == W_Q4K;
	const size_t q_bytes = (size_t)batch_len * xq_cols(in_dim) * sizeof(__half);
	if (sums) {
		TIE_CUDA_TRY(c, cudaMemsetAsync(s.xq_hi, 0, q_bytes, c->stream));
		TIE_CUDA_TRY(c, cudaMemsetAsync(s.xq_hi + v.q_lo_off, 0, q_bytes, c->stream));
	}
	TRY(launch_split_rows(c, x_dev, nullptr, 1, batch_len, in_dim, s.xs_hi, s.xs_hi + v.lo_off, sums ? s.xq_hi : nullptr,
			      sums ? s.xq_hi + v.q_lo_off : nullptr));
	TRY(launch_tc_dense(c, *reg->dense, o_dev));
	if (sums) {
		TIE_CUDA_TRY(c, cudaMemsetAsync(s.xq_hi, 0, q_bytes, c->stream));
		TIE_CUDA_TRY(c, cudaMemsetAsync(s.xq_hi + v.q_lo_off, 0, q_bytes, c->stream));
	}
	if (!dev) {
		TIE_CUDA_TRY(c, cudaMemcpyAsync(o, o_dev, (size_t)batch_len * out_dim * sizeof(float), cudaMemcpyDeviceToHost, c->stream));
		return check_status(c);
	}
	if (flags & TIE_CUDA_NO_SYNC)
		return TIE_CUDA_OK;
	return check_status(c);
}

static int ensure_row_buffers(tie_cuda_ctx *c, size_t n)
{
	if (c->row_cap >= n)
		return TIE_CUDA_OK;
	if (c->row_x)
		cudaFree(c->row_x);
	if (c->row_o)
		cudaFree(c->row_o);
	c->row_x = c->row_o = nullptr;
	c->row_cap = 0;
	TRY(dev_alloc(c, &c->row_x, n));
	TRY(dev_alloc(c, &c->row_o, n));
	c->row_cap = n;
	return TIE_CUDA_OK;
}

// One slice [start_row, end_row) of a mat-vec, as the reference's dispatcher calls its row kernels
// (math_dispatch.c:224, 254; the threaded dispatcher, :262-283, calls them concurrently from its
// pool workers with disjoint slices).  The slices of one context share its staging buffers,
// stream and status word, so a call holds the context's row lock from the first buffer use to
// the read-back of the status; only the rows of the slice are launched.
static int dispatch_mat_vec_row(const void *X, const void *W, void *O, int in_dim, int start_row, int end_row, int type)
{
	tie_cuda_ctx *c;
	{
		std::lock_guard<std::mutex> lk(g_mutex);
		c = g_current;
	}
	if (!c)
		return TIE_CUDA_EINVAL;
	if (!X || !W || !O || in_dim <= 0 || start_row < 0 || end_row <= start_row)
		return TIE_CUDA_EINVAL;
	std::lock_guard<std::mutex> row_lock(c->row_mutex);
	TIE_CUDA_TRY(c, cudaSetDevice(c->device));
	const uint8_t *w = static_cast<const uint8_t *>(W);
	const tie_cuda_ctx::Reg *reg = nullptr;
	for (int i = c->n_regs - 1; i >= 0; i--) {
		const uint8_t *h = static_cast<const uint8_t *>(c->regs[i].host);
		if (w >= h && w < h + c->regs[i].bytes) {
			reg = &c->regs[i];
			break;
		}
	}
	if (!reg || reg->type != type || reg->k != in_dim)
		return TIE_CUDA_EINVAL;
	const size_t off = w - static_cast<const uint8_t *>(reg->host);
	size_t row_bytes = (type == TIE_GGML_TYPE_F32) ? (size_t)in_dim * 4 : (size_t)(in_dim / QK_K) * block_bytes(type);
	if (off % row_bytes)
		return TIE_CUDA_EINVAL;
	const bool r8 = reg->kind == W_Q6K_R8 && type != TIE_GGML_TYPE_F32;
	if (r8 && (off / row_bytes) % 8)
		return TIE_CUDA_ENOTSUP;
	if (off + (size_t)end_row * row_bytes > reg->bytes)
		return TIE_CUDA_EINVAL;
	// the re-ordered Q6_K layout is addressed by groups of 8 rows: start at the slice's group
	const int first = r8 ? (start_row & ~7) : start_row;
	const int n_rows = end_row - first;
	size_t need = (size_t)((in_dim > n_rows) ? in_dim : n_rows);
	TRY(ensure_row_buffers(c, need));
	TIE_CUDA_TRY(c, cudaMemcpyAsync(c->row_x, X, (size_t)in_dim * sizeof(float), cudaMemcpyHostToDevice, c->stream));
	const uint8_t *w_dev = reg->dev + off + (size_t)first * row_bytes;
	if (type == TIE_GGML_TYPE_F32)
		TRY(launch_router_rows(c, c->row_x, reinterpret_cast<const float *>(w_dev), n_rows, in_dim, c->row_o));
	else
		TRY(launch_stream_matvec(c, w_dev, reg->kind, in_dim, n_rows, c->row_x, c->row_o));
	TIE_CUDA_TRY(c, cudaMemcpyAsync(static_cast<float *>(O) + start_row, c->row_o + (start_row - first),
					(size_t)(end_row - start_row) * sizeof(float), cudaMemcpyDeviceToHost, c->stream));
	return check_status(c);
}

void tie_cuda_mat_vec_row_f32_q4k_f32(const void *X, const void *W, void *O, int in_dim, int start_row, int end_row)
{
	int rc = dispatch_mat_vec_row(X, W, O, in_dim, start_row, end_row, TIE_GGML_TYPE_Q4_K);
	if (rc)
		g_dispatch_status = rc;
}

void tie_cuda_mat_vec_row_f32_q6k_f32(const void *X, const void *W, void *O, int in_dim, int start_row, int end_row)
{
	int rc = dispatch_mat_vec_row(X, W, O, in_dim, start_row, end_row, TIE_GGML_TYPE_Q6_K);
	if (rc)
		g_dispatch_status = rc;
}

void tie_cuda_mat_vec_row_f32_f32_f32(const void *X, const void *W, void *O, int in_dim, int start_row, int end_row)
{
	int rc = dispatch_mat_vec_row(X, W, O, in_dim, start_row, end_row, TIE_GGML_TYPE_F32);
	if (rc)
		g_dispatch_status = rc;
}

void tie_cuda_swiglu_f32_f32(void *gate, const void *up, int size)
{
	tie_cuda_ctx *c;
	{
		std::lock_guard<std::mutex> lk(g_mutex);
		c = g_current;
	}
	auto run = [&]() -> int {
		if (!c || !gate || !up || size <= 0)
			return TIE_CUDA_EINVAL;
		std::lock_guard<std::mutex> row_lock(c->row_mutex);
		TIE_CUDA_TRY(c, cudaSetDevice(c->device));
		TRY(ensure_row_buffers(c, (size_t)size));
		TIE_CUDA_TRY(c, cudaMemcpyAsync(c->row_x, gate, (size_t)size * sizeof(float), cudaMemcpyHostToDevice, c->stream));
		TIE_CUDA_TRY(c, cudaMemcpyAsync(c->row_o, up, (size_t)size * sizeof(float), cudaMemcpyHostToDevice, c->stream));
		TRY(launch_swiglu(c, c->row_x, c->row_o, size));
		TIE_CUDA_TRY(c, cudaMemcpyAsync(gate, c->row_x, (size_t)size * sizeof(float), cudaMemcpyDeviceToHost, c->stream));
		return check_status(c);
	};
	int rc = run();
	if (rc)
		g_dispatch_status = rc;
}

}  // extern "C"
