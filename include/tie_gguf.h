/* GGUF reader for the MoE feed-forward tensors of a qwen3moe model file.
 *
 * Replaces, for this path only, the reference's gguf_model_parse / gguf_model_map_weights
 * (gguf.c:892-1047) and the per-layer tensor lookup of model_load_weights (model.c:237-293; tensor
 * names model_qwen3.c:39-52, metadata keys model_qwen3.c:54-63): the file is mapped read-only, the
 * key/value metadata and the tensor directory are indexed, and the four MoE tensors (+ the FFN
 * norm) of a block are returned as pointers into the mapping, ready for
 * tie_cuda_upload_moe_layer().  Nothing is converted or copied; tokenizer arrays and all other
 * tensors are skipped.  Host only (no CUDA), plain C ABI. */
#ifndef TIE_GGUF_H
#define TIE_GGUF_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct tie_gguf tie_gguf;

enum {
	TIE_GGUF_OK = 0,
	TIE_GGUF_EIO = -1,	/* open / stat / mmap failed */
	TIE_GGUF_EFORMAT = -2,	/* not a GGUF file, unsupported version, truncated or inconsistent directory */
	TIE_GGUF_ENOTFOUND = -3, /* key or tensor missing */
	TIE_GGUF_ETYPE = -4,	/* key or tensor has another type / shape than the path needs */
	TIE_GGUF_EINVAL = -5,
};

typedef struct {
	const void *data;  /* into the mapping */
	uint64_t nbytes;   /* from type and dims (block_q4_k 144 B, block_q6_k 210 B per 256 elements) */
	uint32_t type;	   /* GGMLType (gguf.h:7-40) */
	uint32_t n_dims;
	uint64_t dims[4];  /* dims[0] is the contiguous (input) dimension, as stored in the file */
} tie_gguf_tensor;

/* What tie_cuda_init / tie_cuda_upload_moe_layer need. */
typedef struct {
	uint32_t n_layers, hidden, n_expert, top_k, ffn_dim;
	float norm_eps;
	char arch[32];
} tie_gguf_moe_config;

typedef struct {
	const float *router_w;	/* blk.N.ffn_gate_inp.weight  F32 [n_expert][hidden] */
	const void *gate_exps;	/* blk.N.ffn_gate_exps.weight [n_expert][ffn_dim][hidden/256 blocks] */
	const void *up_exps;	/* blk.N.ffn_up_exps.weight   same */
	const void *down_exps;	/* blk.N.ffn_down_exps.weight [n_expert][hidden][ffn_dim/256 blocks] */
	const float *ffn_norm_w; /* blk.N.ffn_norm.weight F32 [hidden], or NULL when absent */
	int gate_type, up_type, down_type; /* GGMLType: 12 (Q4_K) or 14 (Q6_K) */
} tie_gguf_moe_layer;

/* Maps the file and indexes it.  err (optional) receives a one-line reason on failure. */
int tie_gguf_open(const char *path, tie_gguf **out, char *err, size_t err_len);
void tie_gguf_close(tie_gguf *g);
const char *tie_gguf_strerror(int code);

uint32_t tie_gguf_version(const tie_gguf *g);
uint64_t tie_gguf_tensor_count(const tie_gguf *g);
uint64_t tie_gguf_kv_count(const tie_gguf *g);

/* Scalar metadata.  Integer getters accept any integer value type that fits. */
int tie_gguf_get_u64(const tie_gguf *g, const char *key, uint64_t *value);
int tie_gguf_get_f32(const tie_gguf *g, const char *key, float *value);
/* Copies at most buf_len-1 bytes and terminates. */
int tie_gguf_get_str(const tie_gguf *g, const char *key, char *buf, size_t buf_len);

int tie_gguf_find_tensor(const tie_gguf *g, const char *name, tie_gguf_tensor *out);

/* "<arch>.block_count", ".embedding_length", ".expert_count", ".expert_used_count",
 * ".expert_feed_forward_length", ".attention.layer_norm_rms_epsilon" with arch = general.architecture. */
int tie_gguf_moe_config_read(const tie_gguf *g, tie_gguf_moe_config *cfg);
/* The MoE tensors of block `layer`, with types and shapes checked against cfg. */
int tie_gguf_moe_layer_read(const tie_gguf *g, const tie_gguf_moe_config *cfg, int layer, tie_gguf_moe_layer *out);

#ifdef __cplusplus
}
#endif
#endif
