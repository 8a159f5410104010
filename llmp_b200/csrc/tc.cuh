// tcgen05 / TMA / mbarrier primitives shared by the tensor-core kernels
// (MXFP8 block-scaled GEMM, Q4_K x Q8_1 int8 GEMM, grouped expert GEMM).
// Inline PTX for sm_100a; every wait is bounded.
#ifndef LLMP_B200_CSRC_TC_CUH_
#define LLMP_B200_CSRC_TC_CUH_

#include <cuda.h>

#include "common.cuh"

namespace llmp_b200 {
namespace tc {

constexpr std::uint32_t kSpinLimit = 1u << 24;  // polls before a wait gives up

// ---------------------------------------------------------------- host side
// cuTensorMapEncodeTiled through the runtime's driver entry point, so the
// library carries no link-time dependency on libcuda.
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn EncodeTiled();

// A [rows, cols] row-major byte matrix (cols contiguous), boxes of
// box_cols x box_rows bytes, 128-byte swizzle, zero fill out of bounds.
bool MakeMapBytes2D(CUtensorMap* map, const void* base, std::uint64_t rows, std::uint64_t cols,
                    std::uint64_t row_pitch_bytes, std::uint32_t box_rows, std::uint32_t box_cols);

#ifdef __CUDACC__
// ---------------------------------------------------------------- device side
__device__ __forceinline__ std::uint32_t Smem(const void* p) {
  return static_cast<std::uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ bool ElectOne() {
  std::uint32_t pred = 0;
  asm volatile(
      "{\n"
      ".reg .b32 rx;\n"
      ".reg .pred px;\n"
      "elect.sync rx|px, 0xffffffff;\n"
      "selp.u32 %0, 1, 0, px;\n"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

__device__ __forceinline__ void MbarInit(std::uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(Smem(bar)), "r"(count));
}
__device__ __forceinline__ void MbarInitFence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void MbarExpectTx(std::uint64_t* bar, std::uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(Smem(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void MbarArrive(std::uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(Smem(bar)) : "memory");
}
// Bounded wait for the phase of parity `parity`; false when it ran out (`polls`
// polls: a pending try_wait suspends the thread for up to about a microsecond).
__device__ __forceinline__ bool MbarWait(std::uint64_t* bar, std::uint32_t parity,
                                         std::uint32_t polls = kSpinLimit) {
  const std::uint32_t addr = Smem(bar);
  for (std::uint32_t i = 0; i < polls; ++i) {
    std::uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}
// One non-blocking look at the phase (no suspension): for a look ahead whose answer is
// only needed after other work has been issued.
__device__ __forceinline__ bool MbarTest(std::uint64_t* bar, std::uint32_t parity) {
  std::uint32_t done;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(done)
      : "r"(Smem(bar)), "r"(parity)
      : "memory");
  return done != 0;
}
// The same with a sleep between polls: for a role that runs far ahead and whose
// polling would take issue slots from the warps doing the work.
__device__ __forceinline__ bool MbarWaitSleep(std::uint64_t* bar, std::uint32_t parity,
                                              unsigned ns) {
  const std::uint32_t addr = Smem(bar);
  for (std::uint32_t i = 0; i < kSpinLimit; ++i) {
    std::uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
    __nanosleep(ns);
  }
  return false;
}

// TMA: 2-D tile of a tensor map into shared memory (no multicast).
__device__ __forceinline__ void TmaLoad2D(void* smem, const CUtensorMap* map, int c0, int c1,
                                          std::uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(Smem(smem)), "l"(map), "r"(Smem(bar)), "r"(c0), "r"(c1)
      : "memory");
}
// Untiled bulk copy (16-byte aligned both ends, size a multiple of 16).
__device__ __forceinline__ void BulkLoad(void* smem, const void* gmem, std::uint32_t bytes,
                                         std::uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(Smem(smem)), "l"(gmem), "r"(bytes), "r"(Smem(bar))
      : "memory");
}
__device__ __forceinline__ void PrefetchMap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
__device__ __forceinline__ void FenceProxyAsync() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- tensor memory
__device__ __forceinline__ void TmemAlloc(std::uint32_t* smem_result, std::uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
               ::"r"(Smem(smem_result)), "r"(columns)
               : "memory");
}
__device__ __forceinline__ void TmemRelinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void TmemDealloc(std::uint32_t taddr, std::uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns)
               : "memory");
}
__device__ __forceinline__ void TcFenceBefore() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void TcFenceAfter() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// All MMAs (and copies) this thread issued so far arrive on `bar` when done.
__device__ __forceinline__ void TcCommit(std::uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(Smem(bar))
               : "memory");
}

// Shared-memory matrix descriptor (K-major operand).  swizzle128: rows of 128
// bytes in 8-row, 1024-byte swizzle atoms; else no swizzle (8 x 16-byte core
// matrices `sbo` bytes apart).
__device__ __forceinline__ std::uint64_t SmemDesc(const void* p, bool swizzle128,
                                                  std::uint32_t sbo_bytes) {
  std::uint64_t d = 0;
  d |= static_cast<std::uint64_t>((Smem(p) >> 4) & 0x3fffu);
  d |= static_cast<std::uint64_t>(swizzle128 ? 1u : 0u) << 16;      // leading offset (unused when swizzled)
  d |= static_cast<std::uint64_t>((sbo_bytes >> 4) & 0x3fffu) << 32;  // stride between 8-row groups
  d |= static_cast<std::uint64_t>(1u) << 46;                          // descriptor version
  d |= static_cast<std::uint64_t>(swizzle128 ? 2u : 0u) << 61;
  return d;
}

// Instruction descriptors.  kind::i8: A, B 8-bit integers, int32 accumulate.
__host__ __device__ constexpr std::uint32_t IdescI8(int m, int n, bool a_signed, bool b_signed) {
  return (2u << 4) | ((a_signed ? 1u : 0u) << 7) | ((b_signed ? 1u : 0u) << 10) |
         (static_cast<std::uint32_t>(n >> 3) << 17) | (static_cast<std::uint32_t>(m >> 4) << 24);
}
// kind::f16: A, B FP16 (or both BF16) K-major, F32 accumulate.
__host__ __device__ constexpr std::uint32_t IdescF16(int m, int n, bool bf16 = false) {
  return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) |
         (static_cast<std::uint32_t>(n >> 3) << 17) | (static_cast<std::uint32_t>(m >> 4) << 24);
}
// kind::mxf8f6f4.block_scale: E4M3 x E4M3, E8M0 scales per 32, F32 accumulate.
__host__ __device__ constexpr std::uint32_t IdescMxf8(int m, int n, int a_sf_id, int b_sf_id) {
  return (static_cast<std::uint32_t>(b_sf_id) << 4) | (static_cast<std::uint32_t>(n >> 3) << 17) |
         (1u << 23) | (static_cast<std::uint32_t>(m >> 4) << 24) |
         (static_cast<std::uint32_t>(a_sf_id) << 29);
}

__device__ __forceinline__ void MmaI8(std::uint32_t tmem_d, std::uint64_t a, std::uint64_t b,
                                      std::uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate ? 1u : 0u)
      : "memory");
}
__device__ __forceinline__ void MmaF16(std::uint32_t tmem_d, std::uint64_t a, std::uint64_t b,
                                       std::uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate ? 1u : 0u)
      : "memory");
}
__device__ __forceinline__ void MmaMxf8(std::uint32_t tmem_d, std::uint64_t a, std::uint64_t b,
                                        std::uint32_t idesc, bool accumulate,
                                        std::uint32_t tmem_sfa, std::uint32_t tmem_sfb) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n"
      "}\n"
      ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate ? 1u : 0u), "r"(tmem_sfa),
        "r"(tmem_sfb)
      : "memory");
}
// 32 lanes x 128 bits of shared memory (a 512-byte scale atom) into 4 TMEM
// columns, replicated to the four 32-lane quadrants.
__device__ __forceinline__ void TmemCopyScales(std::uint32_t taddr, std::uint64_t smem_desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(smem_desc)
               : "memory");
}

// ---- CTA pairs (cta_group::2): two CTAs of a cluster, ranks 2i and 2i+1, run one MMA over
// both SMs' shared and tensor memory.  The even CTA's thread issues; barriers of the other
// CTA are reached through its shared::cluster address.
__device__ __forceinline__ std::uint32_t ClusterCtaRank() {
  std::uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void ClusterBarrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n"
               "barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The shared::cluster address of `p` (an object of this CTA's shared memory) in CTA `rank`.
__device__ __forceinline__ std::uint32_t PeerSmem(const void* p, std::uint32_t rank) {
  std::uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(Smem(p)), "r"(rank));
  return out;
}
__device__ __forceinline__ void MbarArrivePeer(std::uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}
__device__ __forceinline__ void StorePeerU32(std::uint32_t cluster_addr, std::uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
// Tensor memory of both CTAs: the same warp of each CTA calls these, with the same arguments.
__device__ __forceinline__ void TmemAllocPair(std::uint32_t* smem_result, std::uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
               ::"r"(Smem(smem_result)), "r"(columns)
               : "memory");
}
__device__ __forceinline__ void TmemRelinquishPair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void TmemDeallocPair(std::uint32_t taddr, std::uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns)
               : "memory");
}
// The pair's MMAs and copies issued so far arrive, when done, on the barrier at this
// offset in every CTA of `cta_mask` (bit i = cluster rank i).
__device__ __forceinline__ void TcCommitPair(std::uint64_t* bar, std::uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
      "[%0], %1;"
      ::"r"(Smem(bar)), "h"(cta_mask)
      : "memory");
}
// M 256 (128 rows from each CTA's A tile), N columns (half of B's rows in each CTA).
__device__ __forceinline__ void MmaMxf8Pair(std::uint32_t tmem_d, std::uint64_t a, std::uint64_t b,
                                            std::uint32_t idesc, bool accumulate,
                                            std::uint32_t tmem_sfa, std::uint32_t tmem_sfb) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n"
      "}\n"
      ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate ? 1u : 0u), "r"(tmem_sfa),
        "r"(tmem_sfb)
      : "memory");
}
// A scale atom of each CTA's shared memory (same offset) into each CTA's tensor memory.
__device__ __forceinline__ void TmemCopyScalesPair(std::uint32_t taddr, std::uint64_t smem_desc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(smem_desc)
               : "memory");
}

// This warp's 32 TMEM lanes x 32 consecutive 32-bit columns into registers.
__device__ __forceinline__ void TmemLoad32(std::uint32_t taddr, std::uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
// 16 columns; the load is asynchronous until TmemLoadWait16 names its registers.
__device__ __forceinline__ void TmemLoad16(std::uint32_t taddr, std::uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
// Waits for this thread's tensor-memory loads; taking the registers as operands
// keeps the compiler from using them before the wait when other loads are in flight.
__device__ __forceinline__ void TmemLoadWait16(std::uint32_t (&r)[16]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]),
                 "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]),
                 "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
               :
               : "memory");
}
__device__ __forceinline__ void TmemLoadWait32(std::uint32_t (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]),
                 "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]),
                 "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]),
                 "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]),
                 "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]),
                 "+r"(r[31])
               :
               : "memory");
}
// The same 32 lanes x 32 columns written from registers.
__device__ __forceinline__ void TmemStore32(std::uint32_t taddr, const std::uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
        "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]),
        "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]),
        "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
// One value to this warp's 32 lanes x 32 columns.
__device__ __forceinline__ void TmemFill32(std::uint32_t taddr, std::uint32_t v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, "
      "%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1};"
      ::"r"(taddr), "r"(v)
      : "memory");
}
__device__ __forceinline__ void TmemStoreWait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void TmemLoadWait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
#endif  // __CUDACC__

}  // namespace tc
}  // namespace llmp_b200

#endif  // LLMP_B200_CSRC_TC_CUH_
