/* Glue between TIE's own structures and the tie_cuda library: what a maintainer adds to the
 * reference tree to put the Qwen3-MoE feed-forward branch on the GPU.  Compiles only inside the
 * reference tree (it includes the reference's headers); the library itself knows nothing about
 * the reference's structures. */
#ifndef TIE_CUDA_QWEN3_H
#define TIE_CUDA_QWEN3_H

#include "tie_cuda.h"

struct TIEContext;

/* After model_load (model.c:565) has mapped the GGUF and filled ctx->model->layers: create the
 * device context from the model's dimensions and the engine's silu_table, and upload the MoE
 * tensors of every layer once (host pointers into the mmap; engine.c:14-44, model.c:198-235).
 * max_tokens: the largest batch_len the engine will pass.  Returns a TIE_CUDA_E* code. */
int tie_cuda_qwen3_load(struct TIEContext *ctx, tie_cuda_ctx **out, int device, int max_tokens);

/* The body of `if (ctx->model->is_moe)` in transformer_layer_qwen3 (model_qwen3.c:403-471):
 * ctx->mem.normed_ffn_input [batch_len][embed_dim] -> ctx->mem.ffn_down_output, one call.
 * Returns 0, a TIE_CUDA_E* code, or TIE_CUDA_ENOTSUP when the buffers are not F32 (the caller
 * then keeps the CPU branch). */
int tie_cuda_qwen3_moe_ffn(struct TIEContext *ctx, tie_cuda_ctx *cuda, int layer_idx, int batch_len);

#endif
