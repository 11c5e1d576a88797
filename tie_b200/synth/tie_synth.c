/*
 * tie_synth — deterministic synthetic Qwen3-MoE block inputs (see tie_synth.h).
 *
 * Build with -ffp-contract=off and without -ffast-math: every floating-point
 * step below must be a single IEEE operation for the bytes to be reproducible.
 */
#include "tie_synth.h"

#include <string.h>

static inline uint64_t mix64(uint64_t z)
{
	z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
	z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
	return z ^ (z >> 31);
}

static inline uint64_t stream_key(uint64_t seed, int stream)
{
	return seed * 0x9E3779B97F4A7C15ULL + ((uint64_t)stream << 40);
}

uint64_t tie_synth_u64(uint64_t seed, int stream, uint64_t index)
{
	return mix64(stream_key(seed, stream) + index);
}

uint16_t tie_synth_f32_to_f16(float f)
{
	uint32_t x;
	memcpy(&x, &f, 4);
	uint32_t sign = (x >> 16) & 0x8000u;
	uint32_t a = x & 0x7FFFFFFFu;
	if (a >= 0x7F800000u) /* inf / nan */
		return (uint16_t)(sign | 0x7C00u | ((a > 0x7F800000u) ? 0x200u : 0));
	if (a >= 0x477FF000u) /* rounds to >= 65520 -> inf */
		return (uint16_t)(sign | 0x7C00u);
	if (a < 0x33000001u) /* <= 2^-25: rounds to zero (ties-to-even at exactly 2^-25) */
		return (uint16_t)sign;
	int e = (int)(a >> 23) - 127;
	uint32_t m = (a & 0x7FFFFFu) | 0x800000u; /* 24-bit significand */
	int shift;			  /* bits to drop */
	uint32_t base;
	if (e >= -14) { /* normal half */
		shift = 13;
		base = (uint32_t)(e + 15) << 10;
		m &= 0x7FFFFFu;
	} else { /* subnormal half: value = m * 2^(e-23), unit 2^-24 */
		shift = 13 + (-14 - e);
		base = 0;
	}
	uint32_t q = m >> shift;
	uint32_t rem = m & ((1u << shift) - 1u);
	uint32_t half = 1u << (shift - 1);
	if (rem > half || (rem == half && (q & 1u)))
		q++;
	return (uint16_t)(sign | (base + q)); /* carry into the exponent is correct by construction */
}

float tie_synth_f16_to_f32(uint16_t h)
{
	uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
	uint32_t e = (h >> 10) & 0x1Fu;
	uint32_t m = h & 0x3FFu;
	uint32_t bits;
	if (e == 0x1F) {
		bits = sign | 0x7F800000u | (m << 13);
	} else if (e != 0) {
		bits = sign | ((e + 112u) << 23) | (m << 13);
	} else if (m == 0) {
		bits = sign;
	} else {
		int ee = 113;
		while ((m & 0x400u) == 0) {
			m <<= 1;
			ee--;
		}
		bits = sign | ((uint32_t)ee << 23) | ((m & 0x3FFu) << 13);
	}
	float f;
	memcpy(&f, &bits, 4);
	return f;
}

/* d and dmin of a super-block from one extra hash of its first word. */
static inline void block_d(uint64_t w0, uint16_t *d, uint16_t *dmin)
{
	uint64_t h = mix64(w0 ^ 0xD1B54A32D192ED03ULL);
	float u = (float)(uint32_t)(h & 0xFFFFFFu) * (1.0f / 16777216.0f);
	float v = (float)(uint32_t)((h >> 24) & 0xFFFFFFu) * (1.0f / 16777216.0f);
	float fd = 3e-3f * u;
	fd = 1e-3f + fd;
	float fm = 2e-3f * v;
	*d = tie_synth_f32_to_f16(fd);
	if (dmin)
		*dmin = tie_synth_f32_to_f16(fm);
}

void tie_synth_q4k(void *dst, uint64_t seed, int stream, uint64_t first_block, uint64_t n_blocks)
{
	uint8_t *out = (uint8_t *)dst;
	const uint64_t key = stream_key(seed, stream);
	for (uint64_t b = 0; b < n_blocks; b++) {
		uint64_t base = key + (first_block + b) * 32u;
		uint64_t w[18];
		for (int k = 0; k < 18; k++)
			w[k] = mix64(base + (uint64_t)k);
		uint8_t *blk = out + b * TIE_Q4K_BLOCK_BYTES;
		memcpy(blk, w, TIE_Q4K_BLOCK_BYTES); /* little-endian byte order of the words */
		uint16_t d, dmin;
		block_d(w[0], &d, &dmin);
		blk[0] = (uint8_t)(d & 0xFF);
		blk[1] = (uint8_t)(d >> 8);
		blk[2] = (uint8_t)(dmin & 0xFF);
		blk[3] = (uint8_t)(dmin >> 8);
	}
}

void tie_synth_q6k(void *dst, uint64_t seed, int stream, uint64_t first_block, uint64_t n_blocks)
{
	uint8_t *out = (uint8_t *)dst;
	const uint64_t key = stream_key(seed, stream);
	for (uint64_t b = 0; b < n_blocks; b++) {
		uint64_t base = key + (first_block + b) * 32u;
		uint64_t w[27];
		for (int k = 0; k < 27; k++)
			w[k] = mix64(base + (uint64_t)k);
		uint8_t *blk = out + b * TIE_Q6K_BLOCK_BYTES;
		memcpy(blk, w, TIE_Q6K_BLOCK_BYTES);
		for (int i = 0; i < 16; i++) /* scales[16] at byte 192: uniform in [-32,31] */
			blk[192 + i] = (uint8_t)(int8_t)((int)(blk[192 + i] & 63u) - 32);
		uint16_t d;
		block_d(w[0], &d, NULL);
		blk[208] = (uint8_t)(d & 0xFF);
		blk[209] = (uint8_t)(d >> 8);
	}
}

/* ---- libm-free double-precision ln / exp / cos(2 pi u): fixed operation order ---- */

static double det_ln(double x) /* x > 0, finite, normal */
{
	uint64_t bits;
	memcpy(&bits, &x, 8);
	int e = (int)((bits >> 52) & 0x7FF) - 1023;
	bits = (bits & 0x000FFFFFFFFFFFFFULL) | 0x3FF0000000000000ULL;
	double m;
	memcpy(&m, &bits, 8); /* m in [1,2) */
	if (m > 1.4142135623730951) {
		m = m * 0.5;
		e++;
	}
	double t = (m - 1.0) / (m + 1.0);
	double t2 = t * t;
	double s = 0.0;
	for (int k = 25; k >= 1; k -= 2) /* Horner over odd powers: sum t^k / k */
		s = s * t2 + 1.0 / (double)k;
	return (double)e * 0.6931471805599453 + 2.0 * t * s;
}

static double det_exp(double y) /* |y| < 700 */
{
	double kf = y * 1.4426950408889634;
	long k = (long)(kf + (kf >= 0 ? 0.5 : -0.5));
	double r = y - (double)k * 0.6931471805599453;
	double s = 1.0;
	for (int n = 18; n >= 1; n--)
		s = 1.0 + s * r / (double)n;
	uint64_t bits = (uint64_t)(k + 1023) << 52;
	double p;
	memcpy(&p, &bits, 8);
	return s * p;
}

static double det_sqrt(double x)
{
	return __builtin_sqrt(x); /* IEEE-exact; compiles to sqrtsd */
}

static double det_cos2pi(double u) /* u in [0,1) */
{
	double a = u * 4.0;
	int q = (int)a;
	double th = (a - (double)q) * 1.5707963267948966;
	double t2 = th * th;
	double c = 1.0, s = 1.0;
	for (int n = 11; n >= 1; n--) {
		c = 1.0 - c * t2 / (double)((2 * n - 1) * (2 * n));
		s = 1.0 - s * t2 / (double)((2 * n) * (2 * n + 1));
	}
	s = s * th;
	switch (q & 3) {
	case 0:
		return c;
	case 1:
		return -s;
	case 2:
		return -c;
	default:
		return s;
	}
}

void tie_synth_normal_f32(float *dst, uint64_t seed, int stream, uint64_t first, uint64_t n, float std)
{
	const uint64_t key = stream_key(seed, stream);
	for (uint64_t i = 0; i < n; i++) {
		uint64_t h = mix64(key + first + i);
		double u1 = ((double)(uint32_t)(h >> 32) + 0.5) * (1.0 / 4294967296.0);
		double u2 = (double)(uint32_t)(h & 0xFFFFFFFFu) * (1.0 / 4294967296.0);
		double r = det_sqrt(-2.0 * det_ln(u1));
		dst[i] = (float)(r * det_cos2pi(u2) * (double)std);
	}
}

void tie_synth_zipf_logp(float *out, int *ranks_out, int n_expert, uint64_t seed, double s)
{
	/* rank_e = 1 + number of experts whose hash sorts before e's (ties by index). */
	double z = 0.0;
	for (int r = 1; r <= n_expert; r++)
		z += det_exp(-s * det_ln((double)r));
	double lnz = det_ln(z);
	double lne = det_ln((double)n_expert);
	for (int e = 0; e < n_expert; e++) {
		uint64_t he = tie_synth_u64(seed, TIE_SYNTH_STREAM_BIAS, (uint64_t)e);
		int rank = 1;
		for (int o = 0; o < n_expert; o++) {
			if (o == e)
				continue;
			uint64_t ho = tie_synth_u64(seed, TIE_SYNTH_STREAM_BIAS, (uint64_t)o);
			if (ho < he || (ho == he && o < e))
				rank++;
		}
		if (ranks_out)
			ranks_out[e] = rank;
		out[e] = (float)(-s * det_ln((double)rank) - lnz + lne);
	}
}
