// Thin wrappers over the sm_100a instructions the GEMM kernels are built from:
// mbarrier, TMA (cp.async.bulk[.tensor]) and tcgen05 (TMEM allocation, MMA,
// commit, smem->TMEM copy, TMEM loads). One wrapper per instruction, no policy.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace sfq::ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ long long clock_now() {
  long long c;
  asm volatile("mov.u64 %0, %%clock64;" : "=l"(c));
  return c;
}

// True in exactly one lane of a converged warp (the same lane every time for the same mask).
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}

// Register rebalancing between warpgroups (every thread of a warpgroup executes the same one).
template <int N> __device__ __forceinline__ void reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N> __device__ __forceinline__ void reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(bar),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Non-blocking probe of a phase (try_wait may suspend the thread; this one never does).
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// ---------------------------------------------------------------- TMA
// 2D tiled load, no multicast: box lands at `dst`, bytes are counted on `bar`.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}
// Untiled bulk copy global -> shared; both addresses 16-byte aligned, size % 16 == 0.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ---------------------------------------------------------------- tcgen05
__device__ __forceinline__ void tmem_alloc(uint32_t smem_slot, uint32_t columns) {  // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot), "r"(columns)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {  // whole warp
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns) {  // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrives once on `bar` when every tcgen05 operation this thread issued so far has completed.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// smem (32 rows x 16 bytes) -> TMEM, replicated into the four 32-lane quadrants.
__device__ __forceinline__ void tc_copy_32x128b_x4(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]; `accumulate` == 0 overwrites D.
__device__ __forceinline__ void mma_i8(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d),
      "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_f16(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d),
      "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The same with the A operand in tensor memory: lanes are the rows of A, every 32-bit column holds two consecutive
// 16-bit elements of K (the lower index in the low half); `a_tmem` is a TMEM address (lane 0 of the tile).
__device__ __forceinline__ void mma_f16_ts(uint32_t d, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d),
      "r"(a_tmem), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Eight kind::f16 MMAs over one 128-byte-swizzled [rows x 128 columns of 16-bit] operand pair -- two 64-column slabs of
// `slab16` 16-byte units each, four K = 16 steps of 32 bytes per slab -- and the commits that follow them, as ONE
// instruction sequence from one thread: the descriptors advance by immediate adds inside the sequence, so the issuing
// thread spends tens of cycles per MMA instead of rebuilding two 64-bit descriptors for each. `accumulate_first` == 0
// makes the first MMA overwrite D. `bar2` gets a second commit when `commit2` != 0. The `_ts` form reads A from tensor
// memory (eight 32-bit columns of 16-bit pairs per K step, 64 columns in all).
__device__ __forceinline__ void mma_f16_x8_commit(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate_first,
                                                  uint32_t slab16, uint32_t bar1, uint32_t bar2, uint32_t commit2) {
  asm volatile(
      "{\n\t.reg .pred p, pt, pc;\n\t.reg .b64 s, a1, a2, a3, a4, a5, a6, a7, b1, b2, b3, b4, b5, b6, b7;\n\t"
      "setp.ne.b32 p, %4, 0;\n\tsetp.eq.b32 pt, 0, 0;\n\tsetp.ne.b32 pc, %8, 0;\n\tcvt.u64.u32 s, %5;\n\t"
      "add.s64 a1, %1, 2;\n\tadd.s64 a2, %1, 4;\n\tadd.s64 a3, %1, 6;\n\tadd.s64 a4, %1, s;\n\t"
      "add.s64 a5, a4, 2;\n\tadd.s64 a6, a4, 4;\n\tadd.s64 a7, a4, 6;\n\t"
      "add.s64 b1, %2, 2;\n\tadd.s64 b2, %2, 4;\n\tadd.s64 b3, %2, 6;\n\tadd.s64 b4, %2, s;\n\t"
      "add.s64 b5, b4, 2;\n\tadd.s64 b6, b4, 4;\n\tadd.s64 b7, b4, 6;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a1, b1, %3, pt;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a2, b2, %3, pt;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a3, b3, %3, pt;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a4, b4, %3, pt;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a5, b5, %3, pt;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a6, b6, %3, pt;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a7, b7, %3, pt;\n\t"
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%6];\n\t"
      "@pc tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%7];\n\t}" ::"r"(d),
      "l"(a), "l"(b), "r"(idesc), "r"(accumulate_first), "r"(slab16), "r"(bar1), "r"(bar2), "r"(commit2)
      : "memory");
}
__device__ __forceinline__ void mma_f16_ts_x8_commit(uint32_t d, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t accumulate_first,
                                                     uint32_t slab16, uint32_t bar1, uint32_t bar2, uint32_t commit2) {
  asm volatile(
      "{\n\t.reg .pred p, pt, pc;\n\t.reg .b64 s, b1, b2, b3, b4, b5, b6, b7;\n\t.reg .b32 a1, a2, a3, a4, a5, a6, a7;\n\t"
      "setp.ne.b32 p, %4, 0;\n\tsetp.eq.b32 pt, 0, 0;\n\tsetp.ne.b32 pc, %8, 0;\n\tcvt.u64.u32 s, %5;\n\t"
      "add.u32 a1, %1, 8;\n\tadd.u32 a2, %1, 16;\n\tadd.u32 a3, %1, 24;\n\tadd.u32 a4, %1, 32;\n\t"
      "add.u32 a5, %1, 40;\n\tadd.u32 a6, %1, 48;\n\tadd.u32 a7, %1, 56;\n\t"
      "add.s64 b1, %2, 2;\n\tadd.s64 b2, %2, 4;\n\tadd.s64 b3, %2, 6;\n\tadd.s64 b4, %2, s;\n\t"
      "add.s64 b5, b4, 2;\n\tadd.s64 b6, b4, 4;\n\tadd.s64 b7, b4, 6;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a1], b1, %3, pt;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a2], b2, %3, pt;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a3], b3, %3, pt;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a4], b4, %3, pt;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a5], b5, %3, pt;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a6], b6, %3, pt;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a7], b7, %3, pt;\n\t"
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%6];\n\t"
      "@pc tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%7];\n\t}" ::"r"(d),
      "r"(a_tmem), "l"(b), "r"(idesc), "r"(accumulate_first), "r"(slab16), "r"(bar1), "r"(bar2), "r"(commit2)
      : "memory");
}
// Block-scaled e2m1 x e2m1, one ue4m3 scale per 16 elements (four per K=64 instruction).
__device__ __forceinline__ void mma_nvfp4(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate,
                                          uint32_t sfa, uint32_t sfb) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}" ::"r"(d),
      "l"(a), "l"(b), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
      : "memory");
}

// ---------------------------------------------------------------- CTA pairs (cluster of two, cta_group::2)
// In a pair, one thread of the leader CTA (cluster rank 0) issues tcgen05.mma / cp / commit for both CTAs; every
// shared-memory descriptor and TMEM address is applied in each CTA to its own memory at the same offset.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {  // every thread of every CTA of the cluster; warps need not be converged
  asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}
// shared::cta address -> shared::cluster address of the same variable in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
// Arrive on a barrier that may live in the peer CTA. CTA-scope release (the default): what the waiter must see is
// ordered by the tcgen05 fences on either side, and a cluster-scope release measured ~1700 cycles per arrival here.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// 2D tiled load (no multicast) into this CTA's shared memory; the bytes are counted on the barrier at `bar`'s
// offset in the LEADER CTA of the pair (address bit 24 selects the CTA inside the pair's shared window).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(bar & 0xFEFFFFFFu)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_slot, uint32_t columns) {  // same warp of both CTAs
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot), "r"(columns)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}
// Arrives once on the barrier at `bar`'s offset in every CTA of `cta_mask` when the pair's MMAs issued so far are done.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar, uint16_t cta_mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
               "h"(cta_mask)
               : "memory");
}
// The same completion signal, delivered only to the barrier in the issuing (leader) CTA.
__device__ __forceinline__ void tc_commit_pair_local(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_copy_32x128b_x4_pair(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
// 256 x N tile over the pair: each CTA supplies 128 rows of A and N/2 rows of B and receives 128 x N of D.
__device__ __forceinline__ void mma_i8_pair(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d),
      "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_f16_pair(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d),
      "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_nvfp4_pair(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate,
                                               uint32_t sfa, uint32_t sfb) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}" ::"r"(d),
      "l"(a), "l"(b), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
      : "memory");
}

// One whole nvfp4 stage of the pair kernel from a single thread, scale copies included: probe the NEXT stage's barrier,
// then per 64-element k-block the three scale-atom copies shared memory -> TMEM (activation rows; weight rows 0-127 and
// 128-255 of the tile) followed by the MMA that reads them, then the commit. tcgen05.cp followed by tcgen05.mma from one
// thread execute in issue order, so no barrier stands between a copy and its MMA; and the tcgen05 instructions of an SM
// go through one issue path: these 17 from one thread take about 480 cycles of it and fit under the 512 the tensor pipe
// needs for the four MMAs, where copies from other warps with their own commits (21 instructions) take about 600.
// `sf_desc` is the shared-memory descriptor of the stage's first activation scale atom; the weights' atoms follow 2 KB on.
__device__ __forceinline__ uint32_t stage4_pair_nvfp4_cp(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate_first,
                                                        uint32_t sf_cols, uint64_t sf_desc, uint32_t commit_bar, uint32_t next_bar,
                                                        uint32_t next_parity) {
  uint32_t ready;
#define SFQ_CP "tcgen05.cp.cta_group::2.32x128b.warpx4 "
#define SFQ_MMA "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X "
  asm volatile(
      "{\n\t.reg .pred p, pt, pn;\n\t.reg .b64 a1, a2, a3, b1, b2, b3, sa1, sa2, sa3, sb0, sb1, sb2, sb3, sc0, sc1, sc2, sc3;\n\t"
      ".reg .b32 fa1, fa2, fa3, fb0, fb1, fb2, fb3, fc0, fc1, fc2, fc3;\n\t.reg .b16 m;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 pn, [%8], %9;\n\t"
      "setp.ne.b32 p, %5, 0;\n\tsetp.eq.b32 pt, 0, 0;\n\tmov.b16 m, 3;\n\t"
      "add.s64 a1, %2, 2;\n\tadd.s64 a2, %2, 4;\n\tadd.s64 a3, %2, 6;\n\t"
      "add.s64 b1, %3, 2;\n\tadd.s64 b2, %3, 4;\n\tadd.s64 b3, %3, 6;\n\t"
      "add.s64 sa1, %7, 32;\n\tadd.s64 sa2, %7, 64;\n\tadd.s64 sa3, %7, 96;\n\t"
      "add.s64 sb0, %7, 128;\n\tadd.s64 sb1, %7, 160;\n\tadd.s64 sb2, %7, 192;\n\tadd.s64 sb3, %7, 224;\n\t"
      "add.s64 sc0, %7, 256;\n\tadd.s64 sc1, %7, 288;\n\tadd.s64 sc2, %7, 320;\n\tadd.s64 sc3, %7, 352;\n\t"
      "add.u32 fa1, %6, 4;\n\tadd.u32 fa2, %6, 8;\n\tadd.u32 fa3, %6, 12;\n\t"
      "add.u32 fb0, %6, 16;\n\tadd.u32 fb1, %6, 24;\n\tadd.u32 fb2, %6, 32;\n\tadd.u32 fb3, %6, 40;\n\t"
      "add.u32 fc0, %6, 20;\n\tadd.u32 fc1, %6, 28;\n\tadd.u32 fc2, %6, 36;\n\tadd.u32 fc3, %6, 44;\n\t"
      SFQ_CP "[%6], %7;\n\t" SFQ_CP "[fb0], sb0;\n\t" SFQ_CP "[fc0], sc0;\n\t"
      SFQ_MMA "[%1], %2, %3, %4, [%6], [fb0], p;\n\t"
      SFQ_CP "[fa1], sa1;\n\t" SFQ_CP "[fb1], sb1;\n\t" SFQ_CP "[fc1], sc1;\n\t"
      SFQ_MMA "[%1], a1, b1, %4, [fa1], [fb1], pt;\n\t"
      SFQ_CP "[fa2], sa2;\n\t" SFQ_CP "[fb2], sb2;\n\t" SFQ_CP "[fc2], sc2;\n\t"
      SFQ_MMA "[%1], a2, b2, %4, [fa2], [fb2], pt;\n\t"
      SFQ_CP "[fa3], sa3;\n\t" SFQ_CP "[fb3], sb3;\n\t" SFQ_CP "[fc3], sc3;\n\t"
      SFQ_MMA "[%1], a3, b3, %4, [fa3], [fb3], pt;\n\t"
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%10], m;\n\t"
      "selp.u32 %0, 1, 0, pn;\n\t}"
      : "=r"(ready)
      : "r"(d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate_first), "r"(sf_cols), "l"(sf_desc), "r"(next_bar), "r"(next_parity),
        "r"(commit_bar)
      : "memory");
#undef SFQ_CP
#undef SFQ_MMA
  return ready;
}

// One whole pipeline stage of the pair kernel from a single thread: probe the NEXT stage's barrier without blocking,
// issue this stage's four MMAs (each advances the K offset of both descriptors by two 16-byte units; nvfp4 also
// advances the scale columns: four per MMA for the activations, `sfb_step` for the weights), then commit to
// `commit_bar` in both CTAs. The probe's verdict is read only after the MMAs and the commit are on their way, so the
// barrier's round trip hides behind their issue. `kind`: 0 int8, 1 nvfp4, 2 bf16.
template <int kind>
__device__ __forceinline__ uint32_t stage4_pair(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate_first,
                                                uint32_t sfa, uint32_t sfb, uint32_t sfb_step, uint32_t commit_bar,
                                                uint32_t next_bar, uint32_t next_parity) {
  uint32_t ready;
  if constexpr (kind == 1) {
    asm volatile(
        "{\n\t.reg .pred p, pt, pn;\n\t.reg .b64 a1, a2, a3, b1, b2, b3;\n\t.reg .b32 fa1, fa2, fa3, fb1, fb2, fb3;\n\t.reg .b16 m;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 pn, [%10], %11;\n\t"
        "setp.ne.b32 p, %5, 0;\n\tsetp.eq.b32 pt, 0, 0;\n\tmov.b16 m, 3;\n\t"
        "add.s64 a1, %2, 2;\n\tadd.s64 a2, %2, 4;\n\tadd.s64 a3, %2, 6;\n\t"
        "add.s64 b1, %3, 2;\n\tadd.s64 b2, %3, 4;\n\tadd.s64 b3, %3, 6;\n\t"
        "add.u32 fa1, %6, 4;\n\tadd.u32 fa2, %6, 8;\n\tadd.u32 fa3, %6, 12;\n\t"
        "add.u32 fb1, %7, %8;\n\tadd.u32 fb2, fb1, %8;\n\tadd.u32 fb3, fb2, %8;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%1], %2, %3, %4, [%6], [%7], p;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%1], a1, b1, %4, [fa1], [fb1], pt;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%1], a2, b2, %4, [fa2], [fb2], pt;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%1], a3, b3, %4, [fa3], [fb3], pt;\n\t"
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%9], m;\n\t"
        "selp.u32 %0, 1, 0, pn;\n\t}"
        : "=r"(ready)
        : "r"(d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate_first), "r"(sfa), "r"(sfb), "r"(sfb_step), "r"(commit_bar),
          "r"(next_bar), "r"(next_parity)
        : "memory");
  } else {
#define SFQ_STAGE4_PLAIN(KIND_STR)                                                                                      \
  asm volatile(                                                                                                         \
      "{\n\t.reg .pred p, pt, pn;\n\t.reg .b64 a1, a2, a3, b1, b2, b3;\n\t.reg .b16 m;\n\t"                              \
      "mbarrier.test_wait.parity.shared::cta.b64 pn, [%7], %8;\n\t"                                                     \
      "setp.ne.b32 p, %5, 0;\n\tsetp.eq.b32 pt, 0, 0;\n\tmov.b16 m, 3;\n\t"                                             \
      "add.s64 a1, %2, 2;\n\tadd.s64 a2, %2, 4;\n\tadd.s64 a3, %2, 6;\n\t"                                              \
      "add.s64 b1, %3, 2;\n\tadd.s64 b2, %3, 4;\n\tadd.s64 b3, %3, 6;\n\t"                                              \
      "tcgen05.mma.cta_group::2.kind::" KIND_STR " [%1], %2, %3, %4, p;\n\t"                                            \
      "tcgen05.mma.cta_group::2.kind::" KIND_STR " [%1], a1, b1, %4, pt;\n\t"                                           \
      "tcgen05.mma.cta_group::2.kind::" KIND_STR " [%1], a2, b2, %4, pt;\n\t"                                           \
      "tcgen05.mma.cta_group::2.kind::" KIND_STR " [%1], a3, b3, %4, pt;\n\t"                                           \
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%6], m;\n\t"          \
      "selp.u32 %0, 1, 0, pn;\n\t}"                                                                                     \
      : "=r"(ready)                                                                                                     \
      : "r"(d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate_first), "r"(commit_bar), "r"(next_bar), "r"(next_parity)      \
      : "memory")
    if constexpr (kind == 0)
      SFQ_STAGE4_PLAIN("i8");
    else
      SFQ_STAGE4_PLAIN("f16");
#undef SFQ_STAGE4_PLAIN
  }
  return ready;
}

// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp receives lane (base lane + t).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// The reverse direction: thread t of the warp writes 32 consecutive 32-bit columns of lane (base lane + t).
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
      "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
      "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
      "r"(r[31])
      : "memory");
}
// Sixteen consecutive 32-bit columns per lane.
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
      "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// ---------------------------------------------------------------- packed fp32 pairs
// Two fp32 in one 64-bit register; add / sub / mul / fma on both halves in one instruction (round to nearest even).
using f32x2 = unsigned long long;
__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
  f32x2 d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
  return d;
}
__device__ __forceinline__ void unpack2(f32x2 v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ f32x2 sub2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}

// ---------------------------------------------------------------- descriptors
// K-major operand tile stored as rows of 128 bytes with the 128-byte swizzle
// (what a TMA box {128 bytes, rows} with CU_TENSOR_MAP_SWIZZLE_128B writes):
// 8-row groups are 1024 bytes apart, the tile base is 1024-byte aligned.
// Fields: [0,14) address>>4, [16,30) leading offset>>4 (unused here),
// [32,46) stride offset>>4, [46,48) version = 1, [61,64) layout (2 = 128B swizzle).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
  return uint64_t((saddr >> 4) & 0x3FFFu) | (uint64_t(1024 >> 4) << 32) | (uint64_t(1) << 46) | (uint64_t(2) << 61);
}
// 32 rows x 16 bytes, unswizzled, rows contiguous (8-row groups 128 bytes apart): a scale-factor atom.
__device__ __forceinline__ uint64_t smem_desc_sf(uint32_t saddr) {
  return uint64_t((saddr >> 4) & 0x3FFFu) | (uint64_t(128 >> 4) << 32) | (uint64_t(1) << 46);
}

// Instruction descriptors. Common fields: [4,6) D format, [7,10) A format,
// [10,13) B format, bit 15/16 A/B major (0 = K), [17,23) N>>3, [24,29) M>>4.
__host__ __device__ constexpr uint32_t idesc_i8(int m, int n) {  // s8 x s8 -> s32
  return (2u << 4) | (1u << 7) | (1u << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}
__host__ __device__ constexpr uint32_t idesc_bf16(int m, int n) {  // bf16 x bf16 -> f32
  return (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}
// e2m1 x e2m1 with ue4m3 scales (bit 23 = 0), scale ids 0, K = 64 (bit 31 = 0).
__host__ __device__ constexpr uint32_t idesc_nvfp4(int m, int n) {
  return (1u << 7) | (1u << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}

}  // namespace sfq::ptx
