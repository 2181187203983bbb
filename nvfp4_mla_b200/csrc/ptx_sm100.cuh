// Thin inline-PTX wrappers for sm_100a: mbarrier, TMA (cp.async.bulk.tensor), tensor memory (tcgen05.alloc / ld / st),
// 5th-generation tensor-core MMA (tcgen05.mma) and its shared-memory / instruction descriptors, and the narrow
// float conversions the NVFP4 cache needs. Everything here is a single instruction or a fixed bit layout; policy
// (who waits on what) lives in the kernels.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ uint32_t lane_id() { return threadIdx.x & 31; }
// true in exactly one lane of a fully converged warp
__device__ __forceinline__ bool elect_one() {
  uint32_t p;
  asm volatile("{\n.reg .pred q;\nelect.sync _|q, 0xffffffff;\nselp.u32 %0, 1, 0, q;\n}" : "=r"(p));
  return p != 0;
}

// Register budget of the calling warp group (all four warps of the group must execute it). The kernel must be
// compiled with a fixed register count at entry (__launch_bounds__ with one CTA per SM) for these to take effect.
template <int REGS> __device__ __forceinline__ void reg_alloc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGS)); }
template <int REGS> __device__ __forceinline__ void reg_dealloc() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS)); }

// Programmatic dependent launch: a kernel launched with programmatic stream serialization may begin while its
// predecessor still runs. grid_dependency_wait() blocks until the predecessor has completed and its writes are visible;
// grid_launch_dependents() lets the successor begin (it still waits at its own grid_dependency_wait()).
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// arrive by the threads whose `pred` is set, without a branch (one elected lane of a warp, usually)
__device__ __forceinline__ void mbar_arrive_if(uint64_t* bar, bool pred) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.u32 p, %1, 0;\n"
      "@p mbarrier.arrive.shared::cta.b64 _, [%0];\n}" ::"r"(smem_u32(bar)), "r"(uint32_t(pred))
      : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait. Every wait in the kernels goes through this: after about a second of polling the waiter gives up,
// raises the CTA-wide abort flag and returns false; every other waiter sees the flag on its next poll and gives up
// too, so a protocol bug ends in an error status instead of a hung GPU.
constexpr long long kWaitLimitCycles = 1ll << 31;  // about a second of SM clock
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (uint32_t i = 1;; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 63) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > kWaitLimitCycles) break;
    }
  }
  *abort_flag = 1;
  return false;
}

// shared-memory accesses by 32-bit shared address (a generic pointer would cost an address translation per access)
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 d;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(d.x), "=r"(d.y), "=r"(d.z), "=r"(d.w) : "r"(addr));
  return d;
}
__device__ __forceinline__ void sts32(uint32_t addr, uint32_t v) { asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory"); }

// Split form of the bounded wait, for a barrier that has usually completed by the time it is needed: mbar_probe()
// issues the test early (its answer takes as long as any shared-memory round trip, during which the thread carries on
// with independent work), mbar_wait_probed() consumes the answer and only polls if the test failed.
__device__ __forceinline__ uint32_t mbar_probe(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok;
}
__device__ __forceinline__ bool mbar_wait_probed(uint32_t probed, uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  return probed != 0 || mbar_wait(bar, parity, abort_flag);
}

// ---------------------------------------------------------------------------------------------------------------
// fences between proxies / tcgen05 ordering
// ---------------------------------------------------------------------------------------------------------------
// generic-proxy writes to shared memory (st.shared) -> visible to the async proxy (TMA, tcgen05.mma operand reads)
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// named barrier among `count` threads (count a multiple of 32)
__device__ __forceinline__ void bar_sync(uint32_t id, uint32_t count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
// named barrier that also OR-reduces a predicate over the participants
__device__ __forceinline__ bool bar_red_or(uint32_t id, uint32_t count, bool pred) {
  uint32_t r;
  asm volatile(
      "{\n.reg .pred p, q;\n"
      "setp.ne.u32 p, %3, 0;\n"
      "bar.red.or.pred q, %1, %2, p;\n"
      "selp.u32 %0, 1, 0, q;\n}"
      : "=r"(r)
      : "r"(id), "r"(count), "r"(uint32_t(pred))
      : "memory");
  return r != 0;
}

// ---------------------------------------------------------------------------------------------------------------
// TMA: tiled 2-D loads global -> shared, completion on an mbarrier; L2 prefetch of the same boxes
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
// untiled bulk copy: both addresses 16-byte aligned, size a multiple of 16 bytes
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_prefetch_l2(const void* src, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap* map, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(map), "r"(x), "r"(y) : "memory");
}
// one 128-byte line into L2 (a hint: never faults, returns at once)
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---------------------------------------------------------------------------------------------------------------
// thread-block clusters: distributed shared memory between the CTAs of one cluster (same GPU)
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the peer CTA's copy of a shared-memory location of this CTA
__device__ __forceinline__ uint32_t map_to_cta(const void* local, uint32_t cta_rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(local)), "r"(cta_rank));
  return r;
}
// all threads of all CTAs of the cluster; orders shared-memory accesses (incl. mbarrier initialisation) before / after
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Bulk copy from this CTA's shared memory into a peer CTA's (asynchronous proxy on both ends): `bytes` (multiple of 16,
// both addresses 16-byte aligned) are counted on the PEER's mbarrier as completed transaction bytes.
__device__ __forceinline__ void bulk_copy_to_cta(uint32_t dst_cluster_addr, const void* src_local, uint32_t bytes, uint32_t mbar_cluster_addr) {
  asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst_cluster_addr), "r"(smem_u32(src_local)), "r"(bytes), "r"(mbar_cluster_addr)
               : "memory");
}
// arrive on a peer CTA's mbarrier (address from map_to_cta); this thread's earlier writes are released to the cluster
__device__ __forceinline__ void mbar_arrive_cta(uint32_t mbar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(mbar_cluster_addr) : "memory");
}

// ---------------------------------------------------------------------------------------------------------------
// tensor memory
// ---------------------------------------------------------------------------------------------------------------
// A TMEM address is (lane << 16) | column. A warp may touch only lanes [32 * (warp_id % 4), +32).
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {  // whole warp
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 32x32b: thread i of the warp <-> lane (base + i); register j <-> column (col + j)
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]),
        "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]),
        "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]),
               "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
      "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
      "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

// 16x128b.x8: 16 lanes (taddr's lane, a multiple of 16 inside the warp's quadrant) x 32 columns. Thread (g = lane / 4,
// q = lane % 4) writes register 2i to (lane g, column 4i + q) and register 2i + 1 to (lane g + 8, column 4i + q).
__device__ __forceinline__ void tmem_st_16x128b_x8(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.16x128b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

// ---------------------------------------------------------------------------------------------------------------
// ldmatrix, 8-bit, transposing: two 16 x 16 byte matrices; lanes 0-15 give the row addresses (16 bytes each) of the
// first, lanes 16-31 of the second. Thread (g = lane / 4, q = lane % 4) receives, per matrix, byte column g of rows
// 4q .. 4q + 3 (first register) and byte column g + 8 of the same rows (second register).
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void ldmatrix_x2_trans_b8(uint32_t saddr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m16n16.x2.trans.shared.b8 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(saddr)
               : "memory");
}

// by array length
__device__ __forceinline__ void tmem_ldn(uint32_t taddr, uint32_t (&r)[16]) { tmem_ld16(taddr, r); }
__device__ __forceinline__ void tmem_ldn(uint32_t taddr, uint32_t (&r)[32]) { tmem_ld32(taddr, r); }
__device__ __forceinline__ void tmem_stn(uint32_t taddr, const uint32_t (&r)[16]) { tmem_st16(taddr, r); }
__device__ __forceinline__ void tmem_stn(uint32_t taddr, const uint32_t (&r)[32]) { tmem_st32(taddr, r); }

// ---------------------------------------------------------------------------------------------------------------
// tcgen05.mma descriptors
// ---------------------------------------------------------------------------------------------------------------
// Shared-memory operand descriptor, 128-byte swizzle. The swizzle is a function of the absolute shared address
// (16-byte chunk index XOR (address bits 7..9)), so atoms must start on 1024-byte boundaries and a K step inside
// the 128-byte row is taken by advancing the start address.
//   K-major : rows of 128 B (64 x 16-bit or 128 x 8-bit along K); 8-row groups are `sbo` bytes apart
//   MN-major: rows of 128 B (64 x 16-bit or 128 x 8-bit along M/N), one row per K index; 8-row (8 x K) groups are
//             `sbo` bytes apart; the next 128-byte run along M/N is `lbo` bytes away
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= uint64_t((saddr >> 4) & 0x3FFF);
  d |= uint64_t((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= uint64_t((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= uint64_t(1) << 46;  // descriptor version of sm_100
  d |= uint64_t(2) << 61;  // SWIZZLE_128B
  return d;
}

enum : uint32_t { FMT_F16 = 0, FMT_BF16 = 1, FMT_E4M3 = 0 };
// Instruction descriptor for kind::f16 / kind::f8f6f4 with an fp32 accumulator.
__host__ __device__ constexpr uint32_t instr_desc(uint32_t m, uint32_t n, uint32_t a_fmt, uint32_t b_fmt, bool a_mn_major,
                                                   bool b_mn_major) {
  return (1u << 4) | (a_fmt << 7) | (b_fmt << 10) | (uint32_t(a_mn_major) << 15) | (uint32_t(b_mn_major) << 16) |
         ((n >> 3) << 17) | ((m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread
__device__ __forceinline__ void mma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accum)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accum)
      : "memory");
}
__device__ __forceinline__ void mma_f8_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accum)
      : "memory");
}
__device__ __forceinline__ void mma_f8_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, p;\n}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accum)
      : "memory");
}
// Instruction descriptor of kind::mxf4nvf4 (packed E2M1 operands, both K-major, one UE4M3 scale per 16 elements along K,
// fp32 accumulator): formats at bits 7 and 10 (E2M1 = 1), N / 8 at bit 17, scale format at bit 23 (UE4M3 = 0), M / 16 at
// bit 24; the scale-factor ids (bits 4-5 and 29-30) stay 0 because a K = 64 step uses all four bytes of a scale word.
__host__ __device__ constexpr uint32_t instr_desc_mxf4nvf4(uint32_t m, uint32_t n) {
  return (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
// D[tmem] (+)= (A[smem] x SFA[tmem]) * (B[smem] x SFB[tmem]), K = 64 packed E2M1 per operand row. Scale factors: the
// word (4 UE4M3 bytes = the 4 blocks of this K step) of operand row r lives in lane r % 32 of EVERY lane quadrant,
// column sf + r / 32; `sfa` / `sfb` must be multiples of four columns (an unaligned address faults).
__device__ __forceinline__ void mma_mxf4nvf4_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa_tmem,
                                                uint32_t sfb_tmem, uint32_t accum) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accum), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}
// mbarrier arrives once every tcgen05 operation this thread issued so far has completed
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// ---------------------------------------------------------------------------------------------------------------
// narrow float conversions
// ---------------------------------------------------------------------------------------------------------------
// four bytes of packed E2M1 pairs (low nibble = even channel) -> four f16x2 (exact)
__device__ __forceinline__ void e2m1x8_to_f16x8(uint32_t w, uint32_t (&h)[4]) {
  asm("{\n.reg .b8 b0, b1, b2, b3;\n"
      "mov.b32 {b0, b1, b2, b3}, %4;\n"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\ncvt.rn.f16x2.e2m1x2 %1, b1;\n"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\ncvt.rn.f16x2.e2m1x2 %3, b3;\n}"
      : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
      : "r"(w));
}
// eight floats -> eight E2M1 codes (round to nearest even, saturating at 6), element 0 in the lowest nibble, and what
// the codes decode to as four f16x2 (element pairs in order): one block, so the bytes never leave their registers
__device__ __forceinline__ uint32_t f32x8_to_e2m1x8(const float (&v)[8], uint32_t (&h)[4]) {
  uint32_t d;
  asm("{\n.reg .b8 b0, b1, b2, b3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %6, %5;\ncvt.rn.satfinite.e2m1x2.f32 b1, %8, %7;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %10, %9;\ncvt.rn.satfinite.e2m1x2.f32 b3, %12, %11;\n"
      "mov.b32 %0, {b0, b1, b2, b3};\n"
      "cvt.rn.f16x2.e2m1x2 %1, b0;\ncvt.rn.f16x2.e2m1x2 %2, b1;\n"
      "cvt.rn.f16x2.e2m1x2 %3, b2;\ncvt.rn.f16x2.e2m1x2 %4, b3;\n}"
      : "=&r"(d), "=&r"(h[0]), "=&r"(h[1]), "=&r"(h[2]), "=&r"(h[3])
      : "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]));
  return d;
}
// two E4M3 bytes -> f16x2 (exact)
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint16_t x) {
  uint32_t d;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(d) : "h"(x));
  return d;
}
// f16x2 -> two E4M3 bytes, round to nearest even, saturating
__device__ __forceinline__ uint32_t f16x2_to_e4m3x2(uint32_t h) {  // element i of the pair -> byte i
  uint16_t d;
  asm("cvt.rn.satfinite.e4m3x2.f16x2 %0, %1;" : "=h"(d) : "r"(h));
  return d;
}
// (hi, lo) floats -> two E4M3 bytes, lo in the low byte
__device__ __forceinline__ uint32_t f32x2_to_e4m3x2(float lo, float hi) {
  uint16_t d;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(d) : "f"(hi), "f"(lo));
  return d;
}
// four floats -> four E4M3 bytes (round to nearest even, saturating), p0 in the lowest byte
__device__ __forceinline__ uint32_t pack_e4m3x4(float p0, float p1, float p2, float p3) {
  uint32_t d;
  asm("{\n.reg .b16 lo, hi;\n"
      "cvt.rn.satfinite.e4m3x2.f32 lo, %2, %1;\n"
      "cvt.rn.satfinite.e4m3x2.f32 hi, %4, %3;\n"
      "mov.b32 %0, {lo, hi};\n}"
      : "=r"(d)
      : "f"(p0), "f"(p1), "f"(p2), "f"(p3));
  return d;
}
// two f16x2 (four halves) -> four E4M3 bytes, element 0 of `a` in the lowest byte
__device__ __forceinline__ uint32_t f16x4_to_e4m3x4(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("{\n.reg .b16 lo, hi;\n"
      "cvt.rn.satfinite.e4m3x2.f16x2 lo, %1;\n"
      "cvt.rn.satfinite.e4m3x2.f16x2 hi, %2;\n"
      "mov.b32 %0, {lo, hi};\n}"
      : "=r"(d)
      : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t hmul2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t f32x2_to_f16x2(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {  // one instruction on sm_100
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

}  // namespace ptx
