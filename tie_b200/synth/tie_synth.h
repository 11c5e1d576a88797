/*
 * tie_synth — deterministic synthetic Qwen3-MoE block inputs.
 *
 * A real Qwen3-30B-A3B GGUF cannot be fetched where this code is measured, so
 * the benchmark and the parity tests draw router weights, activations and
 * packed Q4_K / Q6_K super-blocks from a counter-based generator.  Everything
 * is a pure function of (seed, stream, index): any slice of any tensor can be
 * regenerated anywhere (host threads, another process, another machine) and
 * comes out byte-identical.  Only integer arithmetic and IEEE +,-,*,/,sqrt in
 * a fixed order are used (no libm), so results do not depend on the C library.
 *
 * Block formats follow the reference's structs: block_q4_k (144 bytes:
 * d, dmin fp16, scales[12], qs[128]) and block_q6_k (210 bytes: ql[128],
 * qh[64], scales[16] int8, d fp16) — gguf.h:100-113.
 */
#ifndef TIE_SYNTH_H
#define TIE_SYNTH_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
	TIE_SYNTH_STREAM_ROUTER = 1,
	TIE_SYNTH_STREAM_GATE = 2,
	TIE_SYNTH_STREAM_UP = 3,
	TIE_SYNTH_STREAM_DOWN = 4,
	TIE_SYNTH_STREAM_X = 5,
	TIE_SYNTH_STREAM_BIAS = 6,
};

#define TIE_Q4K_BLOCK_BYTES 144
#define TIE_Q6K_BLOCK_BYTES 210
#define TIE_QK_K 256

/* 64-bit hash of (seed, stream, index): splitmix64 finaliser over a linear key. */
uint64_t tie_synth_u64(uint64_t seed, int stream, uint64_t index);

/* n_blocks Q4_K super-blocks starting at block index first_block of the tensor.
 * d = fp16(1e-3 + 3e-3 u), dmin = fp16(2e-3 u'), scales/qs uniform bytes. */
void tie_synth_q4k(void *dst, uint64_t seed, int stream, uint64_t first_block, uint64_t n_blocks);

/* n_blocks Q6_K super-blocks. d as above, scales uniform in [-32,31], ql/qh uniform bytes. */
void tie_synth_q6k(void *dst, uint64_t seed, int stream, uint64_t first_block, uint64_t n_blocks);

/* n floats ~ N(0, std^2) starting at element index first (Box-Muller, one draw per index). */
void tie_synth_normal_f32(float *dst, uint64_t seed, int stream, uint64_t first, uint64_t n, float std);

/* out[e] = ln(p_e * n_expert), p_e proportional to rank_e^-s with rank a seeded
 * permutation of the experts (rank 1 = most popular).  ranks_out (may be NULL)
 * receives rank_e in 1..n_expert.  A router-logit bias is alpha * out[e]. */
void tie_synth_zipf_logp(float *out, int *ranks_out, int n_expert, uint64_t seed, double s);

/* IEEE fp32 -> fp16 (round to nearest even) and back; bit-exact with hardware conversions. */
uint16_t tie_synth_f32_to_f16(float f);
float tie_synth_f16_to_f32(uint16_t h);

#ifdef __cplusplus
}
#endif
#endif
