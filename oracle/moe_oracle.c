/*
 * TEST INFRASTRUCTURE — CPU restatement ("port") of the reference's Qwen3-MoE
 * feed-forward path, in plain C.  Not part of the product: only tests, the smoke
 * check and the CPU-baseline leg of the benchmark load this library.
 *
 * The reference computes this path with AVX2 intrinsics (the scalar variants are
 * not equivalent: scalar silu_lookup yields NaN for gate inputs above ~88,
 * engine.c:204-225,305-328).  Each routine below replays the AVX2 routine's
 * arithmetic lane by lane — 8 independent lanes, the same fused multiply-adds,
 * the same horizontal-sum tree — so that it can be compared bit for bit with the
 * reference's compiled code (oracle/_ref) wherever the reference's result does
 * not depend on compiler freedom.  File:line citations are into the reference.
 *
 * Parity status: PINNED against the reference itself — tests/test_oracle.py runs
 * the reference's compiled code (oracle/_ref/libtie_ref.so) on the same seeded
 * inputs and compares, and tests/golden/ holds outputs of that code.  The
 * reference ships no tests or golden vectors of its own for this path.
 *
 * Build: gcc -O2 -mavx2 -mfma -ffp-contract=off (fmaf() must be a hardware FMA and
 * nothing else may be fused).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#define QK_K 256
#define Q4K_BYTES 144
#define Q6K_BYTES 210
#define SILU_N 8192
#define GGML_F32 0
#define GGML_Q4_K 12
#define GGML_Q6_K 14

/* math_scalar.c:46-67 — IEEE half to float, subnormals included. */
static inline float f16_to_f32(uint16_t h)
{
	uint32_t sign = ((uint32_t)(h >> 15) & 1u) << 31;
	int e = (h >> 10) & 0x1F;
	uint32_t m = (uint32_t)(h & 0x3FF) << 13;
	if (e == 0x1F) {
		e = 0xFF;
	} else if (e != 0) {
		e += 112;
	} else if (m != 0) {
		e = 113;
		while ((m & 0x7F800000u) == 0) {
			m <<= 1;
			e--;
		}
		m &= 0x007FFFFFu;
	}
	uint32_t b = sign | ((uint32_t)e << 23) | m;
	float f;
	memcpy(&f, &b, 4);
	return f;
}

/* math_avx2.c:14-21 — (lo+hi), hadd, hadd: ((l0+l4)+(l1+l5)) + ((l2+l6)+(l3+l7)). */
static inline float hsum8(const float *l)
{
	float s0 = l[0] + l[4], s1 = l[1] + l[5], s2 = l[2] + l[6], s3 = l[3] + l[7];
	return (s0 + s1) + (s2 + s3);
}

/* engine.c:204-225 — Schraudolph-style exp with a polynomial correction.  The clamp makes
 * 12102203*x + 1065353216 leave the int range for x > ~88.03 only when called unclamped;
 * with the clamp the conversion is always in range. */
static float expf_fast_ref(float x)
{
	x = fmaxf(-88.37626266479492f, fminf(88.37626266479492f, x));
	union {
		float f;
		int32_t i;
	} u;
	u.i = (int32_t)fmaf(12102203.0f, x, 1065353216.0f);
	float p = u.f;
	p = p * fmaf(1.9875691500E-4f, p, 1.3981999507E-3f);
	p = fmaf(p, p, p * fmaf(8.3334519073E-3f, p, 4.1665795894E-2f));
	p = fmaf(p, p, p * fmaf(1.6666665459E-1f, p, 5.0000001201E-1f));
	return fmaf(u.f, p, u.f);
}

/* engine.c:297-303.  The reference's table is NOT SiLU (its exp approximation is far off
 * for these arguments); what matters is reproducing the same 8192 numbers.  As compiled
 * with the reference's -ffast-math flags the final division x/(1+e) is a hardware
 * reciprocal ESTIMATE plus one Newton step (verified: that variant reproduces the compiled
 * table bit for bit on the machine it was built on), so the reference's own table depends
 * on the CPU model in its last bits.  This restatement divides exactly: it differs from a
 * compiled reference table by a few ulp (<= 2e-6 absolute).  Parity tests therefore feed
 * the reference's own table (tests/golden/silu_table_ref.f32) to both sides. */
void oracle_silu_table_init(float *t)
{
	for (int i = 0; i < SILU_N; i++) {
		float x = fmaf(20.0f * (float)i, 1.0f / 8191.0f, -10.0f);
		t[i] = x / (1.0f + expf_fast_ref(-x));
	}
}

/* math_avx2.c:908-950 as compiled with the reference's flags: pos = ((g+10)*8191)*0.05
 * (-ffast-math turns /20 into *0.05f), index by round-to-nearest-even clamped to
 * [0, 8190] with NO range check on g (outside [-10,10] the last segment is extrapolated),
 * silu = fma(t[i+1]-t[i], frac, t[i]), h = silu*up. */
static inline float swiglu_one(const float *tab, float g, float u)
{
	float pos = ((g - (-10.0f)) * 8191.0f) * 0.05f;
	float r = nearbyintf(pos); /* default rounding mode = nearest even, like cvtps2dq */
	int idx;
	if (!(r >= -2147483648.0f && r < 2147483648.0f))
		idx = INT32_MIN; /* cvtps2dq's "integer indefinite" */
	else
		idx = (int)r;
	if (idx < 0)
		idx = 0;
	if (idx > SILU_N - 2)
		idx = SILU_N - 2;
	float frac = pos - (float)idx;
	float y1 = tab[idx], y2 = tab[idx + 1];
	return fmaf(y2 - y1, frac, y1) * u;
}

void oracle_swiglu(const float *tab, float *gate, const float *up, int n)
{
	for (int i = 0; i < n; i++)
		gate[i] = swiglu_one(tab, gate[i], up[i]);
}

/* math_avx2.c:228-256 — F32 row dot: 8 lanes of sequential FMAs, then hsum. */
void oracle_mat_vec_f32(const float *x, const float *w, float *o, int in_dim, int start_row, int end_row)
{
	for (int r = start_row; r < end_row; r++) {
		const float *wr = w + (size_t)r * in_dim;
		float l[8] = {0, 0, 0, 0, 0, 0, 0, 0};
		int j = 0;
		for (; j <= in_dim - 8; j += 8)
			for (int k = 0; k < 8; k++)
				l[k] = fmaf(x[j + k], wr[j + k], l[k]);
		float s = hsum8(l);
		for (; j < in_dim; j++)
			s = fmaf(x[j], wr[j], s);
		o[r] = s;
	}
}

/* math_scalar.c:91-100 */
static inline void scale_min_k4(int j, const uint8_t *q, uint8_t *d, uint8_t *m)
{
	if (j < 4) {
		*d = q[j] & 63;
		*m = q[j + 4] & 63;
	} else {
		*d = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
		*m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
	}
}

/* math_avx2.c:535-604 — one Q4_K super-block against 256 floats.  Two 8-lane accumulators:
 * acc0 takes bytes [o, o+8) of each 16-byte chunk, acc1 bytes [o+8, o+16); for each byte
 * the low nibble (sub-block 2p, element 64p+i) is accumulated before the high nibble
 * (sub-block 2p+1, element 64p+32+i).  The weight (q*d - m) is a fused multiply-subtract
 * in the reference as compiled (-ffp-contract=fast). */
static float dot_q4k(const float *x, const uint8_t *blk)
{
	uint16_t hd, hm;
	memcpy(&hd, blk, 2);
	memcpy(&hm, blk + 2, 2);
	const float d = f16_to_f32(hd), dmin = f16_to_f32(hm);
	const uint8_t *sc = blk + 4;
	const uint8_t *q = blk + 16;
	float scales[8], mins[8];
	for (int i = 0; i < 8; i++) {
		uint8_t s, m;
		scale_min_k4(i, sc, &s, &m);
		scales[i] = d * (float)s;
		mins[i] = dmin * (float)m;
	}
	float a0[8] = {0}, a1[8] = {0};
	int is = 0;
	for (int j = 0; j < 256; j += 64) {
		const float d1 = scales[is], m1 = mins[is], d2 = scales[is + 1], m2 = mins[is + 1];
		for (int o = 0; o < 32; o += 16) {
			for (int k = 0; k < 8; k++) {
				float ql = (float)(q[o + k] & 0xF), qh = (float)(q[o + k] >> 4);
				a0[k] = fmaf(x[j + o + k], fmaf(ql, d1, -m1), a0[k]);
				a0[k] = fmaf(x[j + 32 + o + k], fmaf(qh, d2, -m2), a0[k]);
			}
			for (int k = 0; k < 8; k++) {
				float ql = (float)(q[o + 8 + k] & 0xF), qh = (float)(q[o + 8 + k] >> 4);
				a1[k] = fmaf(x[j + o + 8 + k], fmaf(ql, d1, -m1), a1[k]);
				a1[k] = fmaf(x[j + 32 + o + 8 + k], fmaf(qh, d2, -m2), a1[k]);
			}
		}
		q += 32;
		is += 2;
	}
	for (int k = 0; k < 8; k++)
		a0[k] = a0[k] + a1[k];
	return hsum8(a0);
}

/* math_avx2.c:411-495 — one Q6_K super-block.  For each half n and each group of 8 l's:
 * acc0 += (d*sc[is])*(q1*x[l]), acc1 += (d*sc[is+2])*(q2*x[l+32]),
 * acc0 += (d*sc[is+4])*(q3*x[l+64]), acc1 += (d*sc[is+6])*(q4*x[l+96]); is = l/16. */
static float dot_q6k(const float *x, const uint8_t *blk)
{
	const uint8_t *ql = blk, *qh = blk + 128;
	const int8_t *sc = (const int8_t *)(blk + 192);
	uint16_t hd;
	memcpy(&hd, blk + 208, 2);
	const float d = f16_to_f32(hd);
	float a0[8] = {0}, a1[8] = {0};
	for (int n = 0; n < 2; n++) {
		const float *xp = x + n * 128;
		const uint8_t *qlp = ql + n * 64, *qhp = qh + n * 32;
		const int8_t *scp = sc + n * 8;
		for (int l = 0; l < 32; l += 8) {
			int is = (l >= 16) ? 1 : 0;
			float w0 = d * (float)scp[is + 0], w1 = d * (float)scp[is + 2];
			float w2 = d * (float)scp[is + 4], w3 = d * (float)scp[is + 6];
			for (int k = 0; k < 8; k++) {
				uint8_t a = qlp[l + k], b = qlp[l + k + 32], h = qhp[l + k];
				float q1 = (float)(int8_t)(((a & 0xF) | ((h & 3) << 4)) - 32);
				float q2 = (float)(int8_t)(((b & 0xF) | (((h >> 2) & 3) << 4)) - 32);
				float q3 = (float)(int8_t)(((a >> 4) | (((h >> 4) & 3) << 4)) - 32);
				float q4 = (float)(int8_t)(((b >> 4) | (((h >> 6) & 3) << 4)) - 32);
				a0[k] = fmaf(w0, q1 * xp[l + k], a0[k]);
				a1[k] = fmaf(w1, q2 * xp[l + k + 32], a1[k]);
				a0[k] = fmaf(w2, q3 * xp[l + k + 64], a0[k]);
				a1[k] = fmaf(w3, q4 * xp[l + k + 96], a1[k]);
			}
		}
	}
	for (int k = 0; k < 8; k++)
		a0[k] = a0[k] + a1[k];
	return hsum8(a0);
}

/* math_avx2.c:753-787 — per output row: plain fp32 adds of the block dots, in block order. */
void oracle_mat_vec_quant(const float *x, const void *w, int w_type, float *o, int in_dim, int start_row,
			  int end_row)
{
	const int nb = in_dim / QK_K;
	const size_t bs = (w_type == GGML_Q4_K) ? Q4K_BYTES : Q6K_BYTES;
	for (int r = start_row; r < end_row; r++) {
		const uint8_t *row = (const uint8_t *)w + (size_t)r * nb * bs;
		float sum = 0.0f;
		for (int j = 0; j < nb; j++)
			sum += (w_type == GGML_Q4_K) ? dot_q4k(x + j * QK_K, row + j * bs)
						     : dot_q6k(x + j * QK_K, row + j * bs);
		o[r] = sum;
	}
}

int oracle_mat_vec(const float *x, const void *w, int w_type, float *o, int in_dim, int out_dim)
{
	if (w_type == GGML_F32)
		oracle_mat_vec_f32(x, (const float *)w, o, in_dim, 0, out_dim);
	else if (w_type == GGML_Q4_K || w_type == GGML_Q6_K)
		oracle_mat_vec_quant(x, w, w_type, o, in_dim, 0, out_dim);
	else
		return -1;
	return 0;
}

/* math_avx2.c:56-97.  inv_rms = 1/sqrtf(ss/n + eps) is evaluated exactly here; the
 * reference as compiled with -ffast-math may use a reciprocal-sqrt estimate plus one
 * Newton step, which differs in the last bits (up to 3 ulp seen; tests allow 4 ulp on this op). */
void oracle_rms_norm(const float *x, const float *w, float *o, int n, float eps)
{
	float l[8] = {0};
	int i = 0;
	for (; i <= n - 8; i += 8)
		for (int k = 0; k < 8; k++)
			l[k] = fmaf(x[i + k], x[i + k], l[k]);
	float ss = hsum8(l);
	for (; i < n; i++)
		ss = fmaf(x[i], x[i], ss);
	float inv = 1.0f / sqrtf(ss / (float)n + eps);
	for (i = 0; i < n; i++)
		o[i] = (x[i] * w[i]) * inv;
}

/* engine.c:891-914 — streaming insertion; strict '>' keeps the earlier (lower) index on ties. */
void oracle_find_top_k(const float *logits, int n, int k, int *idx, float *score)
{
	for (int i = 0; i < k; i++) {
		idx[i] = -1;
		score[i] = -INFINITY;
	}
	for (int i = 0; i < n; i++) {
		float s = logits[i];
		if (s > score[k - 1]) {
			idx[k - 1] = i;
			score[k - 1] = s;
			for (int j = k - 2; j >= 0; j--) {
				if (score[j + 1] > score[j]) {
					float ts = score[j];
					int ti = idx[j];
					score[j] = score[j + 1];
					idx[j] = idx[j + 1];
					score[j + 1] = ts;
					idx[j + 1] = ti;
				} else
					break;
			}
		}
	}
}

/* engine.c:864-888 — over the k selected raw logits. */
void oracle_softmax(float *x, int n)
{
	if (n == 0)
		return;
	float mx = x[0];
	for (int i = 1; i < n; i++)
		if (x[i] > mx)
			mx = x[i];
	float sum = 0.0f;
	for (int i = 0; i < n; i++) {
		x[i] = expf(x[i] - mx);
		sum = fmaf(x[i], 1.0f, sum);
	}
	/* -ffast-math (reciprocal-math) hoists 1/sum out of the loop in the reference as compiled */
	const float inv = 1.0f / sum;
	for (int i = 0; i < n; i++)
		x[i] *= inv;
}

typedef struct {
	int hidden, n_expert, top_k, ffn_dim;
	const float *router_w;
	const void *gate, *up, *down;
	int gate_type, up_type, down_type;
	const float *silu_table;
} oracle_layer_t;

static size_t block_bytes(int t)
{
	return t == GGML_Q4_K ? Q4K_BYTES : (t == GGML_Q6_K ? Q6K_BYTES : 0);
}

/* engine.c:916-964 — one expert for one token: slices by byte offset, gate, up, SwiGLU, down. */
static void expert_ffn(const oracle_layer_t *L, int e, const float *x, float *h1, float *h2, float *out)
{
	const int H = L->hidden, F = L->ffn_dim;
	size_t gu_bytes = (size_t)F * (H / QK_K) * block_bytes(L->gate_type);
	size_t up_bytes = (size_t)F * (H / QK_K) * block_bytes(L->up_type);
	size_t dn_bytes = (size_t)H * (F / QK_K) * block_bytes(L->down_type);
	oracle_mat_vec_quant(x, (const uint8_t *)L->gate + (size_t)e * gu_bytes, L->gate_type, h1, H, 0, F);
	oracle_mat_vec_quant(x, (const uint8_t *)L->up + (size_t)e * up_bytes, L->up_type, h2, H, 0, F);
	oracle_swiglu(L->silu_table, h1, h2, F);
	oracle_mat_vec_quant(h1, (const uint8_t *)L->down + (size_t)e * dn_bytes, L->down_type, out, F, 0, H);
}

/* model_qwen3.c:415-470 for one token.  scratch: top_k*(2F+H) floats. */
static void moe_token(const oracle_layer_t *L, const float *x, const float *bias, float *out, int *idx, float *w,
		      float *logits, float *scratch, int par_experts)
{
	const int H = L->hidden, E = L->n_expert, K = L->top_k, F = L->ffn_dim;
	float lg[E];
	oracle_mat_vec_f32(x, L->router_w, lg, H, 0, E);
	if (bias)
		for (int e = 0; e < E; e++)
			lg[e] += bias[e];
	if (logits)
		memcpy(logits, lg, sizeof(float) * E);
	oracle_find_top_k(lg, E, K, idx, w);
	oracle_softmax(w, K);
	const size_t per = (size_t)2 * F + H;
	if (par_experts) {
#pragma omp parallel for schedule(static)
		for (int j = 0; j < K; j++) {
			float *s = scratch + per * j;
			expert_ffn(L, idx[j], x, s, s + F, s + 2 * F);
		}
	} else {
		for (int j = 0; j < K; j++) {
			float *s = scratch + per * j;
			expert_ffn(L, idx[j], x, s, s + F, s + 2 * F);
		}
	}
	/* model_qwen3.c:458-467: acc = 0; acc += gate_j * out_j for j = 0..K-1 (slot order =
	 * descending score); a fused multiply-add in the reference as compiled. */
	for (int k = 0; k < H; k++) {
		float acc = 0.0f;
		for (int j = 0; j < K; j++)
			acc = fmaf(w[j], scratch[per * j + 2 * F + k], acc);
		out[k] = acc;
	}
}

/* Whole path for n_tokens tokens.  parallel: 0 = serial, 1 = the reference's own shape of
 * parallelism (the top_k experts of one token at a time), 2 = across tokens (fastest; for
 * tests).  All three give identical bits.  Optional outputs may be NULL. */
int oracle_moe_ffn(const oracle_layer_t *L, const float *x, int n_tokens, const float *bias, float *out,
		   int *topk_idx, float *topk_w, float *logits, int parallel)
{
	const int H = L->hidden, E = L->n_expert, K = L->top_k, F = L->ffn_dim;
	if (H % QK_K || F % QK_K || !block_bytes(L->gate_type) || !block_bytes(L->up_type) ||
	    !block_bytes(L->down_type))
		return -1;
	const size_t per = ((size_t)2 * F + H) * K;
	if (parallel == 2 && n_tokens > 1) {
		int fail = 0;
#pragma omp parallel
		{
			float *scratch = malloc(per * sizeof(float));
			int idx[K];
			float w[K];
			if (!scratch) {
#pragma omp atomic write
				fail = 1;
			} else {
#pragma omp for schedule(dynamic, 1)
				for (int t = 0; t < n_tokens; t++) {
					moe_token(L, x + (size_t)t * H, bias, out + (size_t)t * H, idx, w,
						  logits ? logits + (size_t)t * E : NULL, scratch, 0);
					if (topk_idx)
						memcpy(topk_idx + (size_t)t * K, idx, sizeof(int) * K);
					if (topk_w)
						memcpy(topk_w + (size_t)t * K, w, sizeof(float) * K);
				}
			}
			free(scratch);
		}
		return fail ? -2 : 0;
	}
	float *scratch = malloc(per * sizeof(float));
	if (!scratch)
		return -2;
	for (int t = 0; t < n_tokens; t++) {
		int idx[K];
		float w[K];
		moe_token(L, x + (size_t)t * H, bias, out + (size_t)t * H, idx, w,
			  logits ? logits + (size_t)t * E : NULL, scratch, parallel == 1);
		if (topk_idx)
			memcpy(topk_idx + (size_t)t * K, idx, sizeof(int) * K);
		if (topk_w)
			memcpy(topk_w + (size_t)t * K, w, sizeof(float) * K);
	}
	free(scratch);
	return 0;
}

/* Router only: logits (+bias), top-k, softmax weights. */
void oracle_route(const oracle_layer_t *L, const float *x, int n_tokens, const float *bias, int *topk_idx,
		  float *topk_w, float *logits)
{
	const int H = L->hidden, E = L->n_expert, K = L->top_k;
#pragma omp parallel for schedule(static)
	for (int t = 0; t < n_tokens; t++) {
		float lg[E];
		oracle_mat_vec_f32(x + (size_t)t * H, L->router_w, lg, H, 0, E);
		if (bias)
			for (int e = 0; e < E; e++)
				lg[e] += bias[e];
		if (logits)
			memcpy(logits + (size_t)t * E, lg, sizeof(float) * E);
		oracle_find_top_k(lg, E, K, topk_idx + (size_t)t * K, topk_w + (size_t)t * K);
		oracle_softmax(topk_w + (size_t)t * K, K);
	}
}

/* LFM2-MoE routing (model_lfm2.c:438-473): sigmoid of the raw logits, selection on
 * sigmoid + sel_bias (exp_probs_b, may be NULL) with the same find_top_k, gates = the UNBIASED
 * sigmoid of the selected experts, L1-normalised with 1/(sum + 1e-6).  scores (optional)
 * receives the sigmoid of every logit.  The reference is built with -ffast-math, so its two
 * divisions are reciprocal estimates refined once: gates agree to a few ulp, not bit for bit. */
void oracle_route_lfm2(const oracle_layer_t *L, const float *x, int n_tokens, const float *sel_bias, int *topk_idx,
		       float *topk_w, float *scores)
{
	const int H = L->hidden, E = L->n_expert, K = L->top_k;
#pragma omp parallel for schedule(static)
	for (int t = 0; t < n_tokens; t++) {
		float sg[E], sel[E], sc[K];
		int *idx = topk_idx + (size_t)t * K;
		float *w = topk_w + (size_t)t * K;
		oracle_mat_vec_f32(x + (size_t)t * H, L->router_w, sg, H, 0, E);
		for (int e = 0; e < E; e++) {
			sg[e] = 1.0f / (1.0f + expf(-sg[e]));
			sel[e] = sel_bias ? sg[e] + sel_bias[e] : sg[e];
		}
		if (scores)
			memcpy(scores + (size_t)t * E, sg, sizeof(float) * E);
		oracle_find_top_k(sel, E, K, idx, sc);
		float sum = 0.0f;
		for (int j = 0; j < K; j++) {
			w[j] = sg[idx[j]];
			sum += w[j];
		}
		const float inv = 1.0f / (sum + 1e-6f);
		for (int j = 0; j < K; j++)
			w[j] *= inv;
	}
}

/* hidden += MoE(RMSNorm(hidden)) — model_qwen3.c:392-401, 403-471, 491 (math_avx2.c:731-751). */
int oracle_moe_block_inplace(const oracle_layer_t *L, float *hidden, int n_tokens, const float *norm_w, float eps,
			     float *normed, float *ffn_out, int *topk_idx, float *topk_w, int parallel)
{
	const int H = L->hidden;
	for (int t = 0; t < n_tokens; t++)
		oracle_rms_norm(hidden + (size_t)t * H, norm_w, normed + (size_t)t * H, H, eps);
	int rc = oracle_moe_ffn(L, normed, n_tokens, NULL, ffn_out, topk_idx, topk_w, NULL, parallel);
	if (rc)
		return rc;
	for (size_t i = 0; i < (size_t)n_tokens * H; i++)
		hidden[i] += ffn_out[i];
	return 0;
}

/* One expert applied to independent rows: y[r] = FFN_{expert[r]}(x[r]), unweighted (the
 * checker for the expert-parallel entry point). */
int oracle_expert_rows(const oracle_layer_t *L, const float *x_rows, const int *row_expert, int n_rows,
		       float *y_rows)
{
	const int H = L->hidden, F = L->ffn_dim;
#pragma omp parallel
	{
		float *s = malloc(sizeof(float) * 2 * F);
#pragma omp for schedule(dynamic, 4)
		for (int r = 0; r < n_rows; r++)
			expert_ffn(L, row_expert[r], x_rows + (size_t)r * H, s, s + F, y_rows + (size_t)r * H);
		free(s);
	}
	return 0;
}

/* Seconds for n_tokens tokens with the reference's shape of parallelism (CPU baseline when the
 * reference library itself is not available). */
double oracle_time_moe_ffn(const oracle_layer_t *L, const float *x, int n_tokens, const float *bias, float *out)
{
	struct timespec t0, t1;
	oracle_moe_ffn(L, x, 1, bias, out, NULL, NULL, NULL, 1);
	clock_gettime(CLOCK_MONOTONIC, &t0);
	oracle_moe_ffn(L, x, n_tokens, bias, out, NULL, NULL, NULL, 1);
	clock_gettime(CLOCK_MONOTONIC, &t1);
	return (double)(t1.tv_sec - t0.tv_sec) + 1e-9 * (double)(t1.tv_nsec - t0.tv_nsec);
}
