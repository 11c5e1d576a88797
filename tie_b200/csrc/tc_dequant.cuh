// Packed Q4_K / Q6_K quants -> exact small-integer fp16 MMA operands, in packed half2 arithmetic.
//
// A weight of a super-block (256 k) factors as
//   Q4_K: w = d * (sc_b * q) - dmin * m_b      (sc_b, m_b 6-bit, q 4-bit)   math_scalar.c:216-255
//   Q6_K: w = d * (sc_b * (q - 32))            (sc_b int8, q 6-bit)         math_scalar.c:257-287
// with d, dmin constant over the super-block.  The integer products sc_b*q (<= 945) and
// sc_b*(q-32) are what the tensor cores multiply: they are EXACT in fp16 up to 2048 (the Q6_K
// product can reach 4096; above 2048 an odd product is rounded to even, a relative 2^-12 on that
// one weight).  The fp32 factors d and dmin are applied when a super-block's partial sums are
// taken out of tensor memory, so no low-order operand is needed for the weights.
//
// Quants become halves without conversion instructions: a 16-bit field 0x6400 | q is the half
// 1024 + q, 0x6400 | (q << 4) is 1024 + 16 q, 0x5400 | (q << 4) is 64 + q (q < 64); one HFMA2 with
// a per-sub-block scale and offset then yields sc*q resp. sc*(q-32) for two weights (the product
// inside the fused multiply-add is exact, so the result is the exact integer).  The two halves of
// such a pair come from bytes 0 and 2 (or 1 and 3) of a 32-bit word, so within every group of 4
// consecutive k the operand tiles hold the order [k0, k2, k1, k3]; the token operand is written in
// the same order (split_rows, swiglu_split_rows), so the contraction is unchanged.
#pragma once

#include "common.cuh"

namespace tie {

__device__ __forceinline__ uint32_t h2_bits(__half2 v)
{
	return *reinterpret_cast<uint32_t *>(&v);
}
__device__ __forceinline__ __half2 bits_h2(uint32_t v)
{
	return *reinterpret_cast<__half2 *>(&v);
}

// Scale constants of one Q4_K sub-block pair (low nibbles: sub-block 2p, high nibbles: 2p+1).
struct Q4kConsts {
	__half2 sl, cl;	 // low nibbles:  (1024 + q)    * s      - 1024 s
	__half2 sh, ch;	 // high nibbles: (1024 + 16 q) * (s/16) -   64 s
};

__device__ __forceinline__ Q4kConsts q4k_int_consts(int s_lo, int s_hi)
{
	Q4kConsts c;
	const float fl = (float)s_lo, fh = (float)s_hi;
	c.sl = __float2half2_rn(fl);
	c.cl = __float2half2_rn(-1024.0f * fl);
	c.sh = __float2half2_rn(fh * 0.0625f);
	c.ch = __float2half2_rn(-64.0f * fh);
	return c;
}

// One 32-bit word of Q4_K quants (4 bytes = 4 low + 4 high nibbles) -> sc*q as half2 pairs:
// lo[0] = bytes (0, 2), lo[1] = bytes (1, 3) of the low nibbles; hi[] the same of the high ones.
__device__ __forceinline__ void q4k_int_word(uint32_t w, const Q4kConsts &c, uint32_t lo[2], uint32_t hi[2])
{
	const uint32_t w8 = w >> 8;
	lo[0] = h2_bits(__hfma2(bits_h2((w & 0x000F000Fu) | 0x64006400u), c.sl, c.cl));
	lo[1] = h2_bits(__hfma2(bits_h2((w8 & 0x000F000Fu) | 0x64006400u), c.sl, c.cl));
	hi[0] = h2_bits(__hfma2(bits_h2((w & 0x00F000F0u) | 0x64006400u), c.sh, c.ch));
	hi[1] = h2_bits(__hfma2(bits_h2((w8 & 0x00F000F0u) | 0x64006400u), c.sh, c.ch));
}

// Four 6-bit quants held as the bytes of q (0..63 each) -> sc*(q-32) pairs: out[0] = bytes (0, 2),
// out[1] = bytes (1, 3).  s = half2(sc), c = half2(-96 sc).
__device__ __forceinline__ void q6k_int_word(uint32_t q, __half2 s, __half2 c, uint32_t out[2])
{
	out[0] = h2_bits(__hfma2(bits_h2(((q << 4) & 0x03F003F0u) | 0x54005400u), s, c));
	out[1] = h2_bits(__hfma2(bits_h2(((q >> 4) & 0x03F003F0u) | 0x54005400u), s, c));
}

// Position of element k inside its group of 4 in the operand tiles: [k0, k2, k1, k3].
__host__ __device__ __forceinline__ int tc_kperm(int k)
{
	return (k & ~3) | ((k & 1) << 1) | ((k >> 1) & 1);
}

}  // namespace tie
