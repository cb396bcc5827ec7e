// Thin inline-PTX wrappers for sm_100a: mbarrier, TMA (cp.async.bulk.tensor),
// tcgen05 (alloc / mma / commit / ld) and the fences that order them.
//
// Written from the PTX ISA description of each instruction.  Every wait in this
// file is bounded: a wait that runs out of time returns false instead of
// spinning forever, so a protocol bug surfaces as an error status on the host
// and never as a hung SM.  (The reference's mbarrier wait is an unbounded spin,
// swiglu/_matmul_silu_mul.cu:152-161.)
#pragma once

#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

namespace sgl {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// Address of the same shared-memory offset in CTA `rank` of this cluster.
__device__ __forceinline__ uint32_t mapa(uint32_t cta_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(cta_addr), "r"(rank));
  return r;
}

__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// ---------------------------------------------------------------- mbarrier

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

// Makes mbarrier initialisation visible to the async proxy and to peer CTAs.
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
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

// Bounded wait.  Polls the barrier until the phase with the given parity has
// completed, the CTA-wide abort flag is raised, or `limit_ns` elapses.  The
// clock is only consulted every 256 failed polls (reading %globaltimer costs
// far more than a poll, and each try_wait already suspends for a while), so a
// wait that completes promptly never touches it.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint64_t limit_ns,
                                          const volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  uint64_t t0 = 0;
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 255u) == 0u) {
      if (*abort_flag != 0) return false;
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > limit_ns) {
        return false;
      }
    }
  }
}

// Arrive on a barrier of this CTA.
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Arrive on a barrier anywhere in the cluster (address from mapa, or a local
// address, which is also a valid cluster address of the executing CTA).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}

// Arrive on a barrier of another CTA of the cluster so that this thread's earlier writes to
// its own shared memory (and those of threads it has synchronised with) are visible to whoever
// then waits on that barrier with cluster-scope acquire.
__device__ __forceinline__ void mbar_arrive_release_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait_acquire_cluster(uint32_t bar, uint32_t parity) {
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

// mbar_wait for a barrier that CTAs of the whole cluster arrive on (same bound, same abort flag).
__device__ __forceinline__ bool mbar_wait_acquire_cluster(uint32_t bar, uint32_t parity,
                                                          uint64_t limit_ns,
                                                          const volatile int* abort_flag) {
  if (mbar_try_wait_acquire_cluster(bar, parity)) return true;
  uint64_t t0 = 0;
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait_acquire_cluster(bar, parity)) return true;
    if ((it & 255u) == 0u) {
      if (*abort_flag != 0) return false;
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > limit_ns) {
        return false;
      }
    }
  }
}

// 16 bytes from the shared memory of a CTA of this cluster (address from mapa).
__device__ __forceinline__ float4 ld_shared_cluster_v4(uint32_t cluster_addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(cluster_addr)
               : "memory");
  return v;
}

__device__ __forceinline__ void mbar_arrive_expect_tx_cluster(uint32_t cluster_bar,
                                                              uint32_t bytes) {
  // Default semantics (release at CTA scope): a cluster-scope release here costs a
  // full memory fence per ring slot, which serialises the producer.
  asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_bar),
               "r"(bytes)
               : "memory");
}

// ---------------------------------------------------------------- TMA

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}

// L2 eviction-priority policy for the .L2::cache_hint forms below.
// kind: 0 = evict_normal, 1 = evict_first, 2 = evict_last.
__device__ __forceinline__ uint64_t make_l2_policy(int kind) {
  uint64_t p;
  if (kind == 1) {
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  } else if (kind == 2) {
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  } else {
    asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(p));
  }
  return p;
}

// 2-D tiled load, global -> this CTA's shared memory, completion reported on
// `bar` as transaction bytes.  x is the innermost (contiguous) coordinate and
// x * sizeof(element) must be a multiple of 16 bytes.
// kPeerBarrier = true adds .cta_group::2, which lets the barrier live in the
// peer CTA of a CTA pair (no multicast: each CTA loads only its own tile).
template <bool kPeerBarrier>
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* map, int x,
                                            int y, uint32_t bar, uint64_t policy) {
  if constexpr (kPeerBarrier) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.cta_group::2"
        ".L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;" ::"r"(smem_dst),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar), "l"(policy)
        : "memory");
  } else {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        ".L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;" ::"r"(smem_dst),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar), "l"(policy)
        : "memory");
  }
}

// 2-D tiled store, shared memory -> global; rows/columns outside the tensor
// are clipped by the hardware.  Part of the executing thread's bulk group.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int x, int y,
                                             uint32_t smem_src, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.global.shared::cta.bulk_group.L2::cache_hint"
      " [%0, {%1, %2}], [%3], %4;" ::"l"(reinterpret_cast<uint64_t>(map)),
      "r"(x), "r"(y), "r"(smem_src), "l"(policy)
      : "memory");
}

// 2-D tiled reduction, shared memory -> global: every element of the box is ADDED to the
// tensor in global memory (element type from the tensor map: bf16 or f32), atomically per
// element at the L2 / memory that owns the address, which may be a peer GPU's.
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, int x, int y,
                                                  uint32_t smem_src) {
  asm volatile(
      "cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group"
      " [%0, {%1, %2}], [%3];" ::"l"(reinterpret_cast<uint64_t>(map)),
      "r"(x), "r"(y), "r"(smem_src)
      : "memory");
}

// 16-byte store to global memory that may belong to a peer GPU (mapped into this process).
__device__ __forceinline__ void st_global_v4(void* addr, uint32_t a, uint32_t b, uint32_t c,
                                             uint32_t d) {
  asm volatile("st.global.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "r"(a), "r"(b), "r"(c),
               "r"(d)
               : "memory");
}

// 16-byte store to a MULTICAST address (an NVSwitch multicast object that maps the same
// offset of every member GPU's buffer): the switch replicates the data to all members, so the
// sender's link carries it once.  The address must come from a multicast mapping.
__device__ __forceinline__ void multimem_st_v4(void* mc_addr, uint32_t a, uint32_t b, uint32_t c,
                                               uint32_t d) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr),
               "f"(__uint_as_float(a)), "f"(__uint_as_float(b)), "f"(__uint_as_float(c)),
               "f"(__uint_as_float(d))
               : "memory");
}

__device__ __forceinline__ void bulk_commit_group() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// Wait until at most N of this thread's bulk groups still READ shared memory.
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

// Wait until at most N of this thread's bulk groups are incomplete.
template <int N>
__device__ __forceinline__ void bulk_wait_group() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// Orders generic-proxy shared-memory writes before later async-proxy reads.
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---------------------------------------------------------------- tcgen05

template <int kCtaGroup>
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result_slot, uint32_t ncols) {
  if constexpr (kCtaGroup == 2) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_result_slot),
                 "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  } else {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_result_slot),
                 "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
}

template <int kCtaGroup>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  if constexpr (kCtaGroup == 2) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
  } else {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
  }
}

__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[smem] * B[smem], bf16 inputs, fp32 accumulate.
template <int kCtaGroup>
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                          uint32_t idesc, uint32_t accumulate) {
  if constexpr (kCtaGroup == 2) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}

// Arrive on `bar` once every tcgen05 operation issued so far by this thread
// has completed.  For a CTA pair the arrive is delivered to the barrier at the
// same offset in every CTA named in cta_mask (an mbarrier signal fanned out to
// the pair, not a data copy).
template <int kCtaGroup>
__device__ __forceinline__ void umma_commit(uint32_t bar, uint16_t cta_mask) {
  if constexpr (kCtaGroup == 2) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64"
        " [%0], %1;" ::"r"(bar),
        "h"(cta_mask)
        : "memory");
  } else {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     bar)
                 : "memory");
  }
}

// 32 lanes x 32 consecutive fp32 columns: thread i of the warp receives lane
// (base lane + i); the warp may only address lanes 32*(warp_id % 4) .. +31.
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, float (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]),
        "=f"(v[7]), "=f"(v[8]), "=f"(v[9]), "=f"(v[10]), "=f"(v[11]), "=f"(v[12]), "=f"(v[13]),
        "=f"(v[14]), "=f"(v[15]), "=f"(v[16]), "=f"(v[17]), "=f"(v[18]), "=f"(v[19]),
        "=f"(v[20]), "=f"(v[21]), "=f"(v[22]), "=f"(v[23]), "=f"(v[24]), "=f"(v[25]),
        "=f"(v[26]), "=f"(v[27]), "=f"(v[28]), "=f"(v[29]), "=f"(v[30]), "=f"(v[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---------------------------------------------------------------- descriptors

// Shared-memory matrix descriptor, 128-byte swizzle.  Fields (PTX ISA,
// "tcgen05 shared memory descriptor"): [0,14) start address >> 4,
// [16,30) leading-dimension byte offset >> 4, [32,46) stride-dimension byte
// offset >> 4, [46,49) fixed 0b001, [61,64) swizzle mode (2 = 128B).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes,
                                                    uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
  return d;
}

// Instruction descriptor for kind::f16 with bf16 A/B and fp32 D:
// [4,6) D format (1 = f32), [7,10) A format (1 = bf16), [10,13) B format
// (1 = bf16), [15] A major (0 = K, 1 = MN), [16] B major (0 = K, 1 = MN), [17,23) N >> 3,
// [24,29) M >> 4.
__host__ __device__ constexpr uint32_t make_idesc_bf16(int m, int n, bool a_mn_major,
                                                       bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn_major ? 1u : 0u) << 15) |
         ((b_mn_major ? 1u : 0u) << 16) |
         ((static_cast<uint32_t>(n >> 3) & 0x3Fu) << 17) |
         ((static_cast<uint32_t>(m >> 4) & 0x1Fu) << 24);
}

}  // namespace ptx
}  // namespace sgl
