// Helpers shared by the decode kernels (decode.cu, decode_fused.cu): bulk copies into shared
// memory, the bounded wait on their barrier, offsets of row tiles, dependent-launch controls.
#pragma once

#include "common.cuh"
#include "tc_ptx.cuh"

namespace tie {

constexpr int DEC_THREADS = 256;
// gate/up: 16 warps per SM — the reduction out of shared memory is latency-bound (dependent
// unpack -> fma chains), so twice the warps per scheduler halve its time
constexpr int DEC_GU_THREADS = 512;
constexpr long long DEC_WAIT_CYCLES = 1ll << 30;

__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar)
{
	asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
		     "r"(bytes), "r"(bar)
		     : "memory");
}

// Bounded wait for the staged tiles; on timeout the status word is flagged and false returned.
__device__ __forceinline__ bool dec_wait(uint32_t bar, unsigned *status)
{
	long long t0 = 0;
	uint32_t spins = 0;
	while (!ptx::mbar_try_wait(bar, 0)) {
		if ((++spins & 1023u) == 0) {
			const long long now = clock64();
			if (t0 == 0)
				t0 = now;
			if (now - t0 > DEC_WAIT_CYCLES) {
				atomicOr(status, ST_WAIT_TIMEOUT);
				return false;
			}
		}
	}
	return true;
}

template <WKind KIND>
__host__ __device__ __forceinline__ size_t tile_offset(int nb, int r0)
{
	return KIND == W_Q4K ? (size_t)r0 * nb * Q4K_BYTES : (size_t)(r0 >> 3) * q6k_r8_group_bytes(nb);
}

// Programmatic dependent launch: a kernel launched with the attribute may start while its
// predecessor still runs; pdl_wait() blocks until the predecessor's memory is visible,
// pdl_trigger() lets the successor start.  Both are no-ops in an ordinary launch.
__device__ __forceinline__ void pdl_wait()
{
	asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void pdl_trigger()
{
	asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

}  // namespace tie
