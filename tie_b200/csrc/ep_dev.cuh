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

constexpr int EP_FETCH_F4 = 16;	// 16-byte loads a thread keeps in flight

// What the CTAs that fetch the peers' tokens need (by value in the kernel parameters); x_all ==
// nullptr: nothing to fetch.
struct EpFetch {
	EpView v;
	const unsigned *step_dev;
	long long budget;
	float *x_all;
	unsigned *status;
};

// CTA `cta` of `n_ctas` (all threads of the CTA call; uses 64 bytes of static shared memory):
// copies every peer's tokens of the step into this rank's x_all, as soon as the peer has
// announced them (xpub; bounded wait).  The tokens do not depend on the routing, so this runs
// beside the router and the rows are laid out from local memory afterwards.  Each rank starts with
// another peer, so that no rank's links serve all readers at once.
__device__ __forceinline__ void ep_fetch_tokens_cta(const EpFetch &f, int cta, int n_ctas)
{
	__shared__ int s_ntok[EP_MAX_RANKS];
	const EpView &v = f.v;
	const int G = v.n_ranks, tid = threadIdx.x, nthr = blockDim.x;
	const unsigned step = *f.step_dev;
	bool ok = true;
	if (tid < G) {
		ok = ep_wait_flag(ep_ptr<unsigned>(v, v.rank, v.off_xpub) + tid, step, f.budget);
		const int n = ok ? __ldcg(ep_ptr<int>(v, tid, v.off_ntok)) : 0;
		s_ntok[tid] = min(max(n, 0), v.t_max);
	}
	ok = __syncthreads_and(ok);
	if (!ok) {
		if (tid == 0 && cta == 0)
			atomicOr(f.status, ST_WAIT_TIMEOUT);
		return;
	}
	const size_t stride = (size_t)n_ctas * nthr;
	for (int j = 1; j < G; j++) {
		const int s = (v.rank + j) % G;
		const size_t n4 = (size_t)s_ntok[s] * (v.hidden / 4);
		const float4 *src = reinterpret_cast<const float4 *>(ep_ptr<float>(v, s, v.off_xs));
		float4 *dst = reinterpret_cast<float4 *>(f.x_all + (size_t)s * v.t_max * v.hidden);
		for (size_t i0 = (size_t)cta * nthr + tid; i0 < n4; i0 += stride * EP_FETCH_F4) {
			float4 t[EP_FETCH_F4];
#pragma unroll
			for (int u = 0; u < EP_FETCH_F4; u++)
				if (i0 + u * stride < n4)
					t[u] = __ldcg(src + i0 + u * stride);
#pragma unroll
			for (int u = 0; u < EP_FETCH_F4; u++)
				if (i0 + u * stride < n4)
					dst[i0 + u * stride] = t[u];
		}
	}
}

}  // namespace tie
