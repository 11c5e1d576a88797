// Thin inline-PTX wrappers for the Blackwell (sm_100a) asynchronous machinery used by the
// grouped GEMM: mbarriers, TMA tile loads, tensor memory and tcgen05.mma.
#pragma once

#include <cuda.h>
#include <stdint.h>

namespace tie {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
	return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ uint64_t globaltimer_ns()
{
	uint64_t t;
	asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
	return t;
}

// ---- mbarrier ----
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
	asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init()
{
	asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// Make generic-proxy shared-memory writes of this thread visible to the async proxy
// (tcgen05.mma and TMA read shared memory through it).
__device__ __forceinline__ void fence_proxy_async_smem()
{
	asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
	asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
	asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
	uint32_t ok;
	asm volatile(
		"{\n\t"
		".reg .pred p;\n\t"
		"mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
		"selp.u32 %0, 1, 0, p;\n\t"
		"}"
		: "=r"(ok)
		: "r"(bar), "r"(parity)
		: "memory");
	return ok != 0;
}
// The same, allowing the hardware to suspend the thread for up to `ns` nanoseconds while the
// phase is incomplete (a suspended thread issues nothing; it resumes when the phase completes).
__device__ __forceinline__ bool mbar_try_wait_suspend(uint32_t bar, uint32_t parity, uint32_t ns)
{
	uint32_t ok;
	asm volatile(
		"{\n\t"
		".reg .pred p;\n\t"
		"mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
		"selp.u32 %0, 1, 0, p;\n\t"
		"}"
		: "=r"(ok)
		: "r"(bar), "r"(parity), "r"(ns)
		: "memory");
	return ok != 0;
}

// ---- cp.async: per-thread asynchronous copies global -> shared ----
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src)
{
	asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void *src)
{
	asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit()
{
	asm volatile("cp.async.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait()
{
	asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// ---- TMA: 2-D tile load global -> shared, completion counted on an mbarrier ----
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *tmap, uint32_t bar, int x, int y)
{
	asm volatile(
		"cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
		"l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(x), "r"(y)
		: "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *tmap, uint32_t bar, int x, int y, int z)
{
	asm volatile(
		"cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
		"l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(x), "r"(y), "r"(z)
		: "memory");
}
// 1-D bulk copy global -> shared (16-byte aligned addresses, size a multiple of 16 bytes).
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar)
{
	asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
		     "r"(bytes), "r"(bar)
		     : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap *tmap)
{
	asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

// ---- tensor memory ----
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t ncols)
{
	asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish()
{
	asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols)
{
	asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before()
{
	asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after()
{
	asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[smem] * B[smem]; one thread issues for the CTA.
__device__ __forceinline__ void mma_f16_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
	asm volatile(
		"{\n\t"
		".reg .pred p;\n\t"
		"setp.ne.b32 p, %4, 0;\n\t"
		"tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
		"}" ::"r"(d_tmem),
		"l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
		: "memory");
}
// Same with the A operand in tensor memory (lane = row, two 16-bit k elements per column).
__device__ __forceinline__ void mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
	asm volatile(
		"{\n\t"
		".reg .pred p;\n\t"
		"setp.ne.b32 p, %4, 0;\n\t"
		"tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
		"}" ::"r"(d_tmem),
		"r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
		: "memory");
}
// The same, executed by a whole warp in uniform control flow: only lanes with issue != 0 issue.
__device__ __forceinline__ void mma_f16_ts_if(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate,
					      uint32_t issue)
{
	asm volatile(
		"{\n\t"
		".reg .pred p, q;\n\t"
		"setp.ne.b32 p, %4, 0;\n\t"
		"setp.ne.b32 q, %5, 0;\n\t"
		"@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
		"}" ::"r"(d_tmem),
		"r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(issue)
		: "memory");
}
// 4 consecutive 32-bit columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_st4(uint32_t taddr, uint32_t a, uint32_t b, uint32_t c, uint32_t d)
{
	asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(a), "r"(b), "r"(c), "r"(d)
		     : "memory");
}
__device__ __forceinline__ void tmem_st_wait()
{
	asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// The mbarrier gets one arrival when all tcgen05 operations issued so far by this thread retire.
__device__ __forceinline__ void mma_commit(uint32_t bar)
{
	asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mma_commit_if(uint32_t bar, uint32_t issue)
{
	asm volatile(
		"{\n\t"
		".reg .pred q;\n\t"
		"setp.ne.b32 q, %1, 0;\n\t"
		"@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t"
		"}" ::"r"(bar),
		"r"(issue)
		: "memory");
}

// 16 consecutive fp32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t v[16])
{
	asm volatile(
		"tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
		: "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
		  "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
		: "r"(taddr)
		: "memory");
}
__device__ __forceinline__ void tmem_ld_wait()
{
	asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---- CTA pairs (clusters of two CTAs, tcgen05 cta_group::2) ----
// One tcgen05.mma.cta_group::2, issued by a thread of the even-ranked ("leader") CTA, multiplies
// 256 rows: rows 0..127 are the A tile in the leader's tensor memory and accumulate into the
// leader's, rows 128..255 the peer's; the N columns of B come half from each CTA's shared memory
// (the same offset in both).  Barriers that count arrivals from both CTAs live in the leader.
__device__ __forceinline__ uint32_t cluster_ctarank()
{
	uint32_t r;
	asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
	return r;
}
__device__ __forceinline__ void cluster_sync_all()
{
	asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The shared::cluster address of the same variable in the leader CTA of the pair (for the leader: its own).
__device__ __forceinline__ uint32_t leader_addr(uint32_t local_smem_addr)
{
	return local_smem_addr & 0xFEFFFFFFu;
}
// Arrival on a barrier of the leader CTA, from either CTA of the pair.  Relaxed: what the arrival
// announces (tensor-memory stores or loads of the arriving thread) is complete before it
// (tcgen05.wait), and no generic-proxy memory is handed over — a cluster-scope release here was
// measured to cost the arriving warp about a thousand cycles.
__device__ __forceinline__ void mbar_arrive_leader(uint32_t local_bar)
{
	asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(leader_addr(local_bar)) : "memory");
}
// try_wait that also orders the peer CTA's writes (its tensor-memory stores, its arrivals).
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity)
{
	uint32_t ok;
	asm volatile(
		"{\n\t"
		".reg .pred p;\n\t"
		"mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
		"selp.u32 %0, 1, 0, p;\n\t"
		"}"
		: "=r"(ok)
		: "r"(bar), "r"(parity)
		: "memory");
	return ok != 0;
}
__device__ __forceinline__ bool mbar_try_wait_suspend_cluster(uint32_t bar, uint32_t parity, uint32_t ns)
{
	uint32_t ok;
	asm volatile(
		"{\n\t"
		".reg .pred p;\n\t"
		"mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n\t"
		"selp.u32 %0, 1, 0, p;\n\t"
		"}"
		: "=r"(ok)
		: "r"(bar), "r"(parity), "r"(ns)
		: "memory");
	return ok != 0;
}
// TMA tile load into THIS CTA's shared memory whose completion bytes are counted on the barrier at
// the same address in the LEADER CTA (no multicast: one destination, one barrier).
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap *tmap, uint32_t local_bar, int x, int y, int z)
{
	asm volatile(
		"cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
		"l"(reinterpret_cast<uint64_t>(tmap)), "r"(leader_addr(local_bar)), "r"(x), "r"(y), "r"(z)
		: "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_result, uint32_t ncols)
{
	asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair()
{
	asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols)
{
	asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem of both CTAs] (+)= A[tmem of both CTAs] * B[shared memory of both CTAs]; lanes with issue != 0 issue.
__device__ __forceinline__ void mma_f16_ts_pair_if(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate,
						   uint32_t issue)
{
	asm volatile(
		"{\n\t"
		".reg .pred p, q;\n\t"
		"setp.ne.b32 p, %4, 0;\n\t"
		"setp.ne.b32 q, %5, 0;\n\t"
		"@q tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t"
		"}" ::"r"(d_tmem),
		"r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(issue)
		: "memory");
}
// One arrival on the barrier at this address in BOTH CTAs of the pair once the MMAs issued so far retire.
__device__ __forceinline__ void mma_commit_pair_if(uint32_t bar, uint32_t issue)
{
	asm volatile(
		"{\n\t"
		".reg .pred q;\n\t"
		"setp.ne.b32 q, %1, 0;\n\t"
		"@q tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %2;\n\t"
		"}" ::"r"(bar),
		"r"(issue), "h"((uint16_t)3)
		: "memory");
}

// Shared-memory matrix descriptor, K-major operand, 128-byte swizzle: rows of 64 fp16 (128 B),
// 8-row groups 1024 B apart (stride byte offset), tile base 1024-byte aligned.  Advancing the
// start address by 32 B selects the next 16-wide k slice inside the swizzled row.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr)
{
	uint64_t d = 0;
	d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);	// start address
	d |= (uint64_t)0 << 16;				// leading byte offset: unused for swizzled K-major
	d |= (uint64_t)(1024u >> 4) << 32;		// stride byte offset
	d |= (uint64_t)1 << 46;				// descriptor version (sm_100)
	d |= (uint64_t)2 << 61;				// layout: SWIZZLE_128B
	return d;
}

// Instruction descriptor for kind::f16: fp16 A and B (both K-major), fp32 accumulate, M x N tile.
__host__ __device__ constexpr uint32_t umma_idesc_f16(int m, int n)
{
	return (1u << 4)		      // D format: f32
	       | (0u << 7) | (0u << 10)	      // A, B format: f16
	       | (0u << 15) | (0u << 16)      // A, B K-major
	       | ((uint32_t)(n >> 3) << 17)   // N / 8
	       | ((uint32_t)(m >> 4) << 24);  // M / 16
}

}  // namespace ptx
}  // namespace tie
