// Dequantisation of packed Q4_K / Q6_K weights straight into fp16 hi + lo MMA operand pairs,
// in packed half2 arithmetic.
//
// A weight of a 32-wide (Q4_K) or 16-wide (Q6_K) sub-block is affine in its small integer quant:
//   Q4_K: w = s*q - m   (s = d*sc, m = dmin*mn, q in 0..15)      math_scalar.c:216-255
//   Q6_K: w = s*(q-32)  (s = d*sc, q in 0..63)                    math_scalar.c:257-287
// Per sub-block a power-of-two quantum u is chosen so that s_h = a*u and m_h = b*u with small
// integers a, b make  hi = s_h*q - m_h  an integer multiple of u below 2049*u: EXACT in fp16, one
// HFMA2 per two weights.  The remainders s_r = s - s_h, m_r = m - m_h (|.| <= u/2) give
// lo = rn16(s_r*q - m_r), again one HFMA2.  hi + lo equals the reference's fp32 weight to about
// 0.01*u, i.e. ~1e-5 of the sub-block's largest weight — the same order as the rounding of the
// tensor-core accumulation and far inside the 1e-3 parity bound.
//
// Quants become halves without a conversion instruction: (bits & 0x000F000F) | 0x64006400 is the
// half2 (1024+q_a, 1024+q_b); subtracting 1024 is exact.  The two lanes of such a half2 come from
// bytes 0 and 2 (or 1 and 3) of a 32-bit word, so within every group of 4 consecutive k the
// operand tiles hold the order [k0, k2, k1, k3]; the token operand is written in the same order
// (split_rows and the gate/up epilogue), so the contraction is unchanged.
#pragma once

#include "common.cuh"

namespace tie {

struct H2x4 {
	__half2 sh, mh, sr, mr;
};

__device__ __forceinline__ uint32_t h2_bits(__half2 v)
{
	return *reinterpret_cast<uint32_t *>(&v);
}
__device__ __forceinline__ __half2 bits_h2(uint32_t v)
{
	return *reinterpret_cast<__half2 *>(&v);
}

// s, m: fp32 scale and min of a Q4_K sub-block.
__device__ __forceinline__ H2x4 q4k_consts(float s, float m)
{
	const float M = fmaxf(15.0f * fabsf(s), fabsf(m));
	int eb = (__float_as_int(M) >> 23) & 0xff;
	eb = max(eb - 9, 103);	// u = 2^(eb-127) >= 2^-24; M/u in [512, 1024)
	const float u = __int_as_float(eb << 23), ui = __int_as_float((254 - eb) << 23);
	const float s_h = rintf(s * ui) * u, m_h = rintf(m * ui) * u;
	H2x4 c;
	c.sh = __float2half2_rn(s_h);
	c.mh = __float2half2_rn(-m_h);
	c.sr = __float2half2_rn(s - s_h);
	c.mr = __float2half2_rn(-(m - m_h));
	return c;
}

// s: fp32 scale of a Q6_K 16-wide sub-block (signed).
__device__ __forceinline__ void q6k_consts(float s, __half2 &sh, __half2 &sr)
{
	int eb = (__float_as_int(fabsf(s)) >> 23) & 0xff;
	eb = max(eb - 5, 103);	// |s|/u in [32, 64): |a*(q-32)| <= 2048
	const float u = __int_as_float(eb << 23), ui = __int_as_float((254 - eb) << 23);
	const float s_h = rintf(s * ui) * u;
	sh = __float2half2_rn(s_h);
	sr = __float2half2_rn(s - s_h);
}

// Four low-nibble (shift 0) or high-nibble (shift 4) quants of a word -> hi/lo half2 pairs:
// hi[0], lo[0] = bytes (0, 2); hi[1], lo[1] = bytes (1, 3).
__device__ __forceinline__ void q4k_word(uint32_t w, int shift, const H2x4 &c, uint32_t hi[2], uint32_t lo[2])
{
	const __half2 k1024 = __float2half2_rn(1024.0f);
	const uint32_t a = ((w >> shift) & 0x000F000Fu) | 0x64006400u;
	const uint32_t b = ((w >> (shift + 8)) & 0x000F000Fu) | 0x64006400u;
	const __half2 qa = __hsub2(bits_h2(a), k1024), qb = __hsub2(bits_h2(b), k1024);
	hi[0] = h2_bits(__hfma2(qa, c.sh, c.mh));
	hi[1] = h2_bits(__hfma2(qb, c.sh, c.mh));
	lo[0] = h2_bits(__hfma2(qa, c.sr, c.mr));
	lo[1] = h2_bits(__hfma2(qb, c.sr, c.mr));
}

// Four 6-bit quants held as the bytes of q (0..63 each) -> hi/lo pairs of s*(q-32).
__device__ __forceinline__ void q6k_word(uint32_t q, __half2 sh, __half2 sr, uint32_t hi[2], uint32_t lo[2])
{
	const __half2 k1056 = __float2half2_rn(1056.0f);
	const uint32_t a = (q & 0x00FF00FFu) | 0x64006400u;
	const uint32_t b = ((q >> 8) & 0x00FF00FFu) | 0x64006400u;
	const __half2 qa = __hsub2(bits_h2(a), k1056), qb = __hsub2(bits_h2(b), k1056);
	hi[0] = h2_bits(__hmul2(qa, sh));
	hi[1] = h2_bits(__hmul2(qb, sh));
	lo[0] = h2_bits(__hmul2(qa, sr));
	lo[1] = h2_bits(__hmul2(qb, sr));
}

__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d)
{
	asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// Position of element k inside its group of 4 in the operand tiles: [k0, k2, k1, k3].
__host__ __device__ __forceinline__ int tc_kperm(int k)
{
	return (k & ~3) | ((k & 1) << 1) | ((k >> 1) & 1);
}

}  // namespace tie
