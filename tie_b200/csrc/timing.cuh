// Optional instrumentation of the two hot kernels, off unless the library is built with
// -DTC_TIMING (grouped GEMM: per-role cycle counters and a per-stage event trace) or -DDF_TIMING
// (one-kernel decode step: globaltimer stamps at the phase boundaries of CTA 0).  Without those
// macros everything here expands to nothing.  The counters are private to the including
// translation unit; the read-out functions (extern "C" tie_debug_*) are emitted where
// TIE_TIMING_TC_OWNER (tensor.cu) resp. TIE_TIMING_DF_OWNER (decode_fused.cu) is defined.
#pragma once

#include <cuda_runtime.h>

namespace tie {

// Grouped GEMM: lane 0 of one warp per role adds its clock64() deltas to g_tc_cycles;
// tie_debug_tc_cycles() reads and clears them.
#ifdef TC_TIMING
static __device__ unsigned long long g_tc_cycles[32];
static __device__ long long g_tc_trace[8][256];
#define TCT_TRACE(r, i)                                            \
	do {                                                       \
		if (RAW && blockIdx.x == 0 && (i) < 256u && lane == 0)    \
			g_tc_trace[r][i] = clock64();              \
	} while (0)
#define TCT_DECL(n) long long tct_[n] = {0}
#define TCT_NOW() clock64()
#define TCT_ADD(i, t0) tct_[i] += clock64() - (t0)
#define TCT_FLUSH(base, n)                                                          \
	do {                                                                        \
		for (int i_ = 0; i_ < (n); i_++)                                    \
			atomicAdd(&g_tc_cycles[(base) + i_], (unsigned long long)tct_[i_]); \
	} while (0)
#else
#define TCT_DECL(n)
#define TCT_NOW() 0ll
#define TCT_ADD(i, t0) (void)(t0)
#define TCT_FLUSH(base, n)
#define TCT_TRACE(r, i)
#endif


#ifdef DF_TIMING
static __device__ unsigned long long g_df_stamps[16];
#define DF_STAMP(i)                                                                   \
	do {                                                                          \
		if (blockIdx.x == 0 && threadIdx.x == 0) {                            \
			unsigned long long t_;                                        \
			asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));        \
			g_df_stamps[i] = t_;                                          \
		}                                                                     \
	} while (0)
#else
#define DF_STAMP(i)
#endif

}  // namespace tie

#if defined(TC_TIMING) && defined(TIE_TIMING_TC_OWNER)
// Debug builds only: copies out and clears the role cycle counters (32 values).
extern "C" int tie_debug_tc_cycles(unsigned long long *out)
{
	unsigned long long zero[32] = {0};
	if (cudaDeviceSynchronize() != cudaSuccess)
		return -1;
	if (cudaMemcpyFromSymbol(out, tie::g_tc_cycles, sizeof(zero)) != cudaSuccess)
		return -1;
	return cudaMemcpyToSymbol(tie::g_tc_cycles, zero, sizeof(zero)) == cudaSuccess ? 0 : -1;
}
extern "C" int tie_debug_tc_trace(long long *out)
{
	if (cudaDeviceSynchronize() != cudaSuccess)
		return -1;
	return cudaMemcpyFromSymbol(out, tie::g_tc_trace, sizeof(long long) * 8 * 256) == cudaSuccess ? 0 : -1;
}
#endif

#if defined(DF_TIMING) && defined(TIE_TIMING_DF_OWNER)
// Debug builds only: globaltimer stamps (ns) of CTA 0 at the phase boundaries of the last launch.
extern "C" int tie_debug_df_stamps(unsigned long long *out)
{
	if (cudaDeviceSynchronize() != cudaSuccess)
		return -1;
	return cudaMemcpyFromSymbol(out, tie::g_df_stamps, sizeof(unsigned long long) * 16) == cudaSuccess ? 0 : -1;
}
#endif
