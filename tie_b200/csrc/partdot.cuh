// Per-lane pieces of the streaming mat-vec kernels: a lane owns a 64-wide slice ("part") of the
// input dimension; PartDot<kind> loads the packed weights of that slice for one output row and
// reduces them against the lane's register copy of the activation slice.
#pragma once

#include "common.cuh"

namespace tie {

// Weights are read either from global memory through the read-only path or, when a kernel has
// staged its weight tile in shared memory, with plain loads.
template <bool SMEM, typename T>
__device__ __forceinline__ T ldw(const T *p)
{
	if (SMEM)
		return *p;
	return __ldg(p);
}

// Exact small-integer -> float without the conversion pipe: place the byte in the low mantissa
// bits of 2^23 and subtract 2^23 (+ offset).
__device__ __forceinline__ float byte_to_float(uint32_t word, int k, float bias)
{
	uint32_t bits = __byte_perm(word, 0x4B000000u, 0x7650 | k);
	return __fsub_rn(__uint_as_float(bits), bias);
}

template <WKind KIND>
struct PartDot;

// Lane-major staging of an activation row in shared memory: the r-th value (r = 0..63) of part p
// is stored at ((r/4) * LPR + p) * 4 + r%4, so that the 128-bit reads of a warp (same r, all
// parts) touch consecutive 16-byte words — no bank conflicts, unlike reading 64 contiguous floats
// per lane.  src_index(p, r) gives the element of the row that value is.
template <WKind KIND, int LPR>
__device__ __forceinline__ void stage_x_lane_major(const float *__restrict__ xrow, float *__restrict__ xs_t, int parts, int tid,
						   int nthreads)
{
	for (int d = tid; d < 16 * parts; d += nthreads) {  // one float4 per (r4, part)
		const int r4 = d / parts, p = d % parts;
		const int k = PartDot<KIND>::src_index(p, 4 * r4);
		*reinterpret_cast<float4 *>(xs_t + (size_t)(r4 * LPR + p) * 4) = *reinterpret_cast<const float4 *>(xrow + k);
	}
}
template <WKind KIND, int LPR>
__device__ __forceinline__ void load_x_lane_major(const float *__restrict__ xs_t, int part, float xr[64], float sx[4])
{
#pragma unroll
	for (int r4 = 0; r4 < 16; r4++) {
		const float4 v = *reinterpret_cast<const float4 *>(xs_t + (size_t)(r4 * LPR + part) * 4);
		xr[4 * r4] = v.x;
		xr[4 * r4 + 1] = v.y;
		xr[4 * r4 + 2] = v.z;
		xr[4 * r4 + 3] = v.w;
	}
	PartDot<KIND>::sums(xr, sx);
}

// ---- Q4_K: part = (block b, quarter p): qs[32p .. 32p+32), low nibbles = sub-block 2p
//      (elements 64p+i), high nibbles = sub-block 2p+1 (elements 64p+32+i) — math_scalar.c:216-255.
template <>
struct PartDot<W_Q4K> {
	__device__ static __forceinline__ int src_index(int part, int r) { return 64 * part + r; }
	__device__ static __forceinline__ void sums(const float xr[64], float sx[4])
	{
		float s0 = 0.f, s1 = 0.f;
#pragma unroll
		for (int i = 0; i < 8; i++) {
			s0 += (xr[4 * i] + xr[4 * i + 1]) + (xr[4 * i + 2] + xr[4 * i + 3]);
			s1 += (xr[32 + 4 * i] + xr[32 + 4 * i + 1]) + (xr[32 + 4 * i + 2] + xr[32 + 4 * i + 3]);
		}
		sx[0] = s0;
		sx[1] = s1;
		sx[2] = sx[3] = 0.f;
	}
	// xr[0..63] = x[64*part .. 64*part+63]; sx[0] = sum xr[0..31], sx[1] = sum xr[32..63]
	__device__ static __forceinline__ void load_x(const float *xrow, int part, float xr[64], float sx[4])
	{
		const float4 *p = reinterpret_cast<const float4 *>(xrow + 64 * part);
		float s0 = 0.f, s1 = 0.f;
#pragma unroll
		for (int i = 0; i < 16; i++) {
			float4 v = p[i];
			xr[4 * i] = v.x;
			xr[4 * i + 1] = v.y;
			xr[4 * i + 2] = v.z;
			xr[4 * i + 3] = v.w;
			float t = (v.x + v.y) + (v.z + v.w);
			if (i < 8)
				s0 += t;
			else
				s1 += t;
		}
		sx[0] = s0;
		sx[1] = s1;
		sx[2] = sx[3] = 0.f;
	}
	struct Raw {
		uint4 hdr, q0, q1;
	};
	template <bool SMEM = false>
	__device__ static __forceinline__ Raw load(const uint8_t *wexp, int nb, int row, int part)
	{
		const uint8_t *blk = wexp + ((size_t)row * nb + (part >> 2)) * Q4K_BYTES;
		Raw r;
		r.hdr = ldw<SMEM>(reinterpret_cast<const uint4 *>(blk));
		const uint4 *q = reinterpret_cast<const uint4 *>(blk + 16 + 32 * (part & 3));
		r.q0 = ldw<SMEM>(q);
		r.q1 = ldw<SMEM>(q + 1);
		return r;
	}
	__device__ static __forceinline__ float dot(const Raw &r, int part, const float xr[64], const float sx[4])
	{
		const int p = part & 3;
		const float d = half_bits_to_float(r.hdr.x & 0xffffu);
		const float dmin = half_bits_to_float(r.hdr.x >> 16);
		const uint32_t sc[3] = {r.hdr.y, r.hdr.z, r.hdr.w};
		int s_lo, m_lo, s_hi, m_hi;
		q4k_scale_min(sc, 2 * p, s_lo, m_lo);
		q4k_scale_min(sc, 2 * p + 1, s_hi, m_hi);
		const uint32_t w[8] = {r.q0.x, r.q0.y, r.q0.z, r.q0.w, r.q1.x, r.q1.y, r.q1.z, r.q1.w};
		float al = 0.f, ah = 0.f;
#pragma unroll
		for (int k = 0; k < 8; k++) {
			uint32_t lo = w[k] & 0x0F0F0F0Fu, hi = (w[k] >> 4) & 0x0F0F0F0Fu;
#pragma unroll
			for (int j = 0; j < 4; j++) {
				al = __fmaf_rn(byte_to_float(lo, j, 8388608.0f), xr[4 * k + j], al);
				ah = __fmaf_rn(byte_to_float(hi, j, 8388608.0f), xr[32 + 4 * k + j], ah);
			}
		}
		float res = __fmul_rn(d, (float)s_lo) * al - __fmul_rn(dmin, (float)m_lo) * sx[0];
		res += __fmul_rn(d, (float)s_hi) * ah - __fmul_rn(dmin, (float)m_hi) * sx[1];
		return res;
	}
};

// ---- Q6_K in the R8 layout: part = (block b, half n, slice l16); 16 l's x 4 positions
//      (l, l+32, l+64, l+96 within the half) — math_scalar.c:257-287.
template <>
struct PartDot<W_Q6K_R8> {
	__device__ static __forceinline__ int src_index(int part, int r)
	{
		return 256 * (part >> 2) + 128 * ((part >> 1) & 1) + 16 * (part & 1) + 32 * (r >> 4) + (r & 15);
	}
	__device__ static __forceinline__ void sums(const float[64], float sx[4]) { sx[0] = sx[1] = sx[2] = sx[3] = 0.f; }
	// xr[16*j + i] = x[256b + 128n + 16*l16 + 32*j + i]
	__device__ static __forceinline__ void load_x(const float *xrow, int part, float xr[64], float sx[4])
	{
		const int b = part >> 2, n = (part >> 1) & 1, l16 = part & 1;
		const float *base = xrow + 256 * b + 128 * n + 16 * l16;
#pragma unroll
		for (int j = 0; j < 4; j++) {
			const float4 *p = reinterpret_cast<const float4 *>(base + 32 * j);
#pragma unroll
			for (int i = 0; i < 4; i++) {
				float4 v = p[i];
				xr[16 * j + 4 * i] = v.x;
				xr[16 * j + 4 * i + 1] = v.y;
				xr[16 * j + 4 * i + 2] = v.z;
				xr[16 * j + 4 * i + 3] = v.w;
			}
		}
		sx[0] = sx[1] = sx[2] = sx[3] = 0.f;
	}
	struct Raw {
		uint4 a, b, h;
		uint32_t sc;
		float d;
	};
	template <bool SMEM = false>
	__device__ static __forceinline__ Raw load(const uint8_t *wexp, int nb, int row, int part)
	{
		const uint8_t *grp = wexp + (size_t)(row >> 3) * q6k_r8_group_bytes(nb);
		const int r8 = row & 7, b = part >> 2, pp = part & 3;
		const uint4 *ch = reinterpret_cast<const uint4 *>(grp + q6k_r8_chunk_off(nb, r8, b, pp));
		Raw r;
		r.a = ldw<SMEM>(ch);
		r.b = ldw<SMEM>(ch + 1);
		r.h = ldw<SMEM>(ch + 2);
		r.sc = ldw<SMEM>(reinterpret_cast<const uint32_t *>(grp + q6k_r8_scale_off(nb, r8, b, pp)));
		r.d = half_bits_to_float(ldw<SMEM>(reinterpret_cast<const unsigned short *>(grp + q6k_r8_d_off(nb, r8, b))));
		return r;
	}
	__device__ static __forceinline__ float dot(const Raw &r, int part, const float xr[64], const float sx[4])
	{
		const uint32_t A[4] = {r.a.x, r.a.y, r.a.z, r.a.w};
		const uint32_t B[4] = {r.b.x, r.b.y, r.b.z, r.b.w};
		const uint32_t Hh[4] = {r.h.x, r.h.y, r.h.z, r.h.w};
		float a1 = 0.f, a2 = 0.f, a3 = 0.f, a4 = 0.f;
		const float off = 8388608.0f + 32.0f;
#pragma unroll
		for (int k = 0; k < 4; k++) {
			uint32_t q1 = (A[k] & 0x0F0F0F0Fu) | ((Hh[k] << 4) & 0x30303030u);
			uint32_t q2 = (B[k] & 0x0F0F0F0Fu) | ((Hh[k] << 2) & 0x30303030u);
			uint32_t q3 = ((A[k] >> 4) & 0x0F0F0F0Fu) | (Hh[k] & 0x30303030u);
			uint32_t q4 = ((B[k] >> 4) & 0x0F0F0F0Fu) | ((Hh[k] >> 2) & 0x30303030u);
#pragma unroll
			for (int j = 0; j < 4; j++) {
				a1 = __fmaf_rn(byte_to_float(q1, j, off), xr[4 * k + j], a1);
				a2 = __fmaf_rn(byte_to_float(q2, j, off), xr[16 + 4 * k + j], a2);
				a3 = __fmaf_rn(byte_to_float(q3, j, off), xr[32 + 4 * k + j], a3);
				a4 = __fmaf_rn(byte_to_float(q4, j, off), xr[48 + 4 * k + j], a4);
			}
		}
		const float s1 = (float)(int)(signed char)(r.sc & 0xff), s2 = (float)(int)(signed char)((r.sc >> 8) & 0xff);
		const float s3 = (float)(int)(signed char)((r.sc >> 16) & 0xff), s4 = (float)(int)(signed char)(r.sc >> 24);
		return r.d * ((s1 * a1 + s2 * a2) + (s3 * a3 + s4 * a4));
	}
};

}  // namespace tie
