// Device pieces of the expert-parallel exchange that more than one kernel uses (ep.cu, router.cu).
#pragma once

#include "common.cuh"

namespace tie {

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned *p)
{
	unsigned v;
	asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
	return v;
}

__device__ __forceinline__ void st_release_sys(unsigned *p, unsigned v)
{
	asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// true once *flag has reached step (wrap-safe), false after `budget` cycles.
__device__ __forceinline__ bool ep_wait_flag(const unsigned *flag, unsigned step, long long budget)
{
	const long long t0 = clock64();
	for (;;) {
		if ((int)(ld_acquire_sys(flag) - step) >= 0)
			return true;
		if (clock64() - t0 > budget)
			return false;
		__nanosleep(200);
	}
}

template <typename T>
__device__ __forceinline__ T *ep_ptr(const EpView &v, int rank, size_t off)
{
	return reinterpret_cast<T *>(v.peer[rank] + off);
}

constexpr int EP_PUSH_F4 = 16;  // 16-byte loads a thread keeps in flight (each is stored to every rank)

// What the CTAs that hand this rank's tokens to its peers need (by value in the kernel
// parameters); x == nullptr: nothing to push.
struct EpPush {
	EpView v;
	const float *x;	 // this rank's tokens of the step [n_tokens][hidden]
	int n_tokens;
	int n_ctas;  // CTAs that take part (set by the launcher)
};

// CTA `cta` of `n_ctas` (all threads of the CTA call): stores this rank's tokens into slot `rank`
// of EVERY rank's x_all (its own included) — plain 16-byte stores over NVLink, which need no round
// trip, each value loaded once from local memory.  The tokens do not depend on the routing, so
// this runs beside the router; the flag that announces the step (pub) is stored by a later launch
// of the same stream, so the rows are complete in every peer's memory when it sees the flag.  Each
// rank starts with another peer, so that no rank's links take all writers at once.
__device__ __forceinline__ void ep_push_tokens_cta(const EpPush &f, int cta, int n_ctas)
{
	const EpView &v = f.v;
	const int G = v.n_ranks, tid = threadIdx.x, nthr = blockDim.x;
	const size_t n4 = (size_t)f.n_tokens * (v.hidden / 4), stride = (size_t)n_ctas * nthr;
	const size_t slot4 = (size_t)v.rank * v.t_max * (v.hidden / 4);
	const float4 *src = reinterpret_cast<const float4 *>(f.x);
	for (size_t i0 = (size_t)cta * nthr + tid; i0 < n4; i0 += stride * EP_PUSH_F4) {
		float4 t[EP_PUSH_F4];
#pragma unroll
		for (int u = 0; u < EP_PUSH_F4; u++)
			if (i0 + u * stride < n4)
				t[u] = __ldg(src + i0 + u * stride);
		for (int j = 0; j < G; j++) {
			float4 *dst = ep_ptr<float4>(v, (v.rank + j) % G, v.off_xall) + slot4;
#pragma unroll
			for (int u = 0; u < EP_PUSH_F4; u++)
				if (i0 + u * stride < n4)
					dst[i0 + u * stride] = t[u];
		}
	}
}

}  // namespace tie
