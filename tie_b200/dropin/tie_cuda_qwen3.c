/* See tie_cuda_qwen3.h.  Written against the reference's headers (main.h, engine.h, model.h):
 * struct TIEContext, Model, LayerWeights, Tensor, MemType, silu_table. */
#include <stddef.h>

#include "main.h"
#include "engine.h"

#include "tie_cuda_qwen3.h"

int tie_cuda_qwen3_load(struct TIEContext *ctx, tie_cuda_ctx **out, int device, int max_tokens)
{
	if (!ctx || !ctx->model || !out || !ctx->model->is_moe)
		return TIE_CUDA_EINVAL;
	const Model *m = ctx->model;
	tie_cuda_config cfg = {
		.device = device,
		.hidden = m->embed_dim,
		.n_expert = m->expert_count,
		.top_k = m->expert_used_count,
		.ffn_dim = m->expert_ffn_dim,
		.n_layers = m->num_layers,
		.max_tokens = max_tokens,
		.norm_eps = m->norm_eps,
		.silu_table = silu_table, /* the engine's own table (engine.c:204-225): results follow it bit for bit */
		.ep_rank = 0,
		.ep_size = 1,
	};
	tie_cuda_ctx *c = NULL;
	int rc = tie_cuda_init(&c, &cfg);
	if (rc)
		return rc;
	for (int i = 0; i < m->num_layers; i++) {
		const LayerWeights *l = &m->layers[i];
		if (!l->ffn_gate_exps.mem.data) /* a dense layer of a mixed model: stays on the CPU path */
			continue;
		/* the upload copies the router as F32 [n_expert][hidden]: a file that stores it in another
		 * type (F16, BF16) would be read past its end */
		if (l->ffn_gate_inp.mem.type != GGML_TYPE_F32) {
			tie_cuda_destroy(c);
			return TIE_CUDA_ENOTSUP;
		}
		rc = tie_cuda_upload_moe_layer(c, i, l->ffn_gate_inp.mem.data, l->ffn_gate_exps.mem.data,
					       (int)l->ffn_gate_exps.mem.type, l->ffn_up_exps.mem.data, (int)l->ffn_up_exps.mem.type,
					       l->ffn_down_exps.mem.data, (int)l->ffn_down_exps.mem.type,
					       l->ffn_norm.mem.type == GGML_TYPE_F32 ? l->ffn_norm.mem.data : NULL);
		if (rc) {
			tie_cuda_destroy(c);
			return rc;
		}
	}
	*out = c;
	return TIE_CUDA_OK;
}

int tie_cuda_qwen3_moe_ffn(struct TIEContext *ctx, tie_cuda_ctx *cuda, int layer_idx, int batch_len)
{
	if (!ctx || !cuda)
		return TIE_CUDA_EINVAL;
	const MemType *in = &ctx->mem.normed_ffn_input;
	MemType *outb = &ctx->mem.ffn_down_output;
	if (in->type != GGML_TYPE_F32 || outb->type != GGML_TYPE_F32)
		return TIE_CUDA_ENOTSUP;
	/* host-pointer mode: the library stages x to the device and the result back */
	return tie_cuda_moe_ffn(cuda, layer_idx, (const float *)in->data, (float *)outb->data, batch_len, 0);
}
