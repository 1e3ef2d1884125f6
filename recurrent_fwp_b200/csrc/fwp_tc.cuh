// Blackwell (sm_100a) building blocks: TMA tile loads, mbarriers with bounded waits, tensor memory (TMEM)
// allocation / load / store, tcgen05.mma issue and commit, and the shared-memory operand descriptors.
//
// Operand tiles in shared memory are 64 rows of 128 bytes (64 bf16) in the 128-byte-swizzle canonical
// layout: the 16-byte chunk j of row r sits at r * 128 + ((j ^ (r & 7)) << 4) from a 1024-byte aligned base.
// That is what a TMA tile load with CU_TENSOR_MAP_SWIZZLE_128B writes and what tcgen05.mma reads, both for
//   "K-major"  operands (rows = the M or N index, the 64 contiguous elements run along the contraction) and
//   "MN-major" operands (rows = the contraction index, the 64 contiguous elements run along M or N).
// One tcgen05.mma contracts 16 elements: the next 16 are 32 bytes further for a K-major operand and
// 16 rows (2048 bytes) further for an MN-major one.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace fwp {
namespace tc {

constexpr int kTileBytes = 64 * 128;          // one 64 x 64 bf16 operand tile

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// byte offset of element (row, col) of a swizzled 64 x 64 bf16 tile (col even: a bf16 pair never straddles a chunk)
__device__ __forceinline__ uint32_t swz(int row, int col) {
    return (uint32_t)(row * 128 + ((((col >> 3) ^ row) & 7) << 4) + ((col & 7) << 1));
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: gives up after `limit` polls (each poll itself waits up to the hardware's time limit), records
// that in *failed (a shared-memory word every later wait of the CTA checks first) and returns.  A CTA that gave
// up keeps walking its barriers without waiting, so it still reaches its clean-up (TMEM release) and exits.
// The poll loop must not be unrolled: the kernels call this from dozens of places and their code has to stay
// small enough for the instruction caches (an unrolled version made the tcgen05 forward 30 % slower).
__device__ __forceinline__ void mbar_wait(uint64_t* bar, uint32_t parity, volatile int* failed, uint32_t limit = 1u << 18) {
    if (*failed) return;
#pragma unroll 1
    for (uint32_t i = 0; i < limit; i++)
        if (mbar_try(bar, parity)) return;
    *failed = 1;
}
// true in exactly one lane of a converged warp
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred P;\n\t"
        "elect.sync _|P, 0xffffffff;\n\t"
        "selp.b32 %0, 1, 0, P;\n\t}"
        : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
// barrier among `count` threads of the CTA (a warp group), ids 1..15
__device__ __forceinline__ void group_sync(int id, int count) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
// generic-proxy writes to shared memory -> visible to the async proxy (tcgen05.mma operand reads, TMA stores)
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---------------------------------------------------------------- TMA (tile mode, this GPU's memory only, no multicast)
__device__ __forceinline__ void tma_load_4d(void* dst, const void* tmap, uint64_t* bar, int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_addr(dst)), "l"(tmap), "r"(smem_addr(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// ---------------------------------------------------------------- tensor memory
// One warp allocates / frees; the base address (lane 0, first column) lands in *slot.
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(slot)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_free(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 16 lanes x 64 columns of fp32 -> 32 registers per thread, in the accumulator-fragment arrangement of the warp-level
// mma: with g = lane / 4 and t = lane % 4, r[4j], r[4j+1] are (row g, columns 8j + 2t, 8j + 2t + 1) and
// r[4j+2], r[4j+3] the same columns of row g + 8.  `taddr` = (first lane << 16) | first column; the first lane is
// 32 * (warp % 4), the warp's own quarter of the 128 lanes.
__device__ __forceinline__ void tmem_ld_16x64(float (&r)[32], uint32_t taddr) {
    uint32_t* u = reinterpret_cast<uint32_t*>(r);
    asm volatile(
        "tcgen05.ld.sync.aligned.16x256b.x8.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]),
          "=r"(u[8]), "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15]),
          "=r"(u[16]), "=r"(u[17]), "=r"(u[18]), "=r"(u[19]), "=r"(u[20]), "=r"(u[21]), "=r"(u[22]), "=r"(u[23]),
          "=r"(u[24]), "=r"(u[25]), "=r"(u[26]), "=r"(u[27]), "=r"(u[28]), "=r"(u[29]), "=r"(u[30]), "=r"(u[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st_16x64(uint32_t taddr, const float (&r)[32]) {
    const uint32_t* u = reinterpret_cast<const uint32_t*>(r);
    asm volatile(
        "tcgen05.st.sync.aligned.16x256b.x8.b32 [%32], "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};"
        ::"r"(u[0]), "r"(u[1]), "r"(u[2]), "r"(u[3]), "r"(u[4]), "r"(u[5]), "r"(u[6]), "r"(u[7]),
          "r"(u[8]), "r"(u[9]), "r"(u[10]), "r"(u[11]), "r"(u[12]), "r"(u[13]), "r"(u[14]), "r"(u[15]),
          "r"(u[16]), "r"(u[17]), "r"(u[18]), "r"(u[19]), "r"(u[20]), "r"(u[21]), "r"(u[22]), "r"(u[23]),
          "r"(u[24]), "r"(u[25]), "r"(u[26]), "r"(u[27]), "r"(u[28]), "r"(u[29]), "r"(u[30]), "r"(u[31]),
          "r"(taddr) : "memory");
}

// ---------------------------------------------------------------- fragment <-> tile moves
// A warp's 16 x 64 tile in accumulator-fragment form, already packed to bf16 pairs: pk[2 * j + h] holds
// (row g + 8h, columns 8j + 2t, 8j + 2t + 1).  stmatrix writes four 8 x 8 blocks per instruction, every lane
// supplying the address of one 16-byte row piece, so a swizzled row needs no per-element address arithmetic.
// `tile` is the 64-row swizzled tile, `row0` the warp's first row.
__device__ __forceinline__ void st_frag_swz(unsigned char* tile, int row0, const uint32_t (&pk)[16], int lane) {
    const int mi = lane >> 3, rr = row0 + 8 * (mi & 1) + (lane & 7);       // block mi: row half mi & 1, column block 2jj + (mi >> 1)
#pragma unroll
    for (int jj = 0; jj < 4; jj++) {
        const int j = 2 * jj + (mi >> 1);
        const uint32_t a = smem_addr(tile) + rr * 128 + (((j ^ rr) & 7) << 4);
        asm volatile("stmatrix.sync.aligned.m8n8.x4.shared.b16 [%0], {%1, %2, %3, %4};"
                     ::"r"(a), "r"(pk[4 * jj]), "r"(pk[4 * jj + 1]), "r"(pk[4 * jj + 2]), "r"(pk[4 * jj + 3]) : "memory");
    }
}
// the same into a row-major tile with `ld` bf16 elements per row (ld a multiple of 8)
__device__ __forceinline__ void st_frag_rowmajor(__nv_bfloat16* tile, int ld, int row0, const uint32_t (&pk)[16], int lane) {
    const int mi = lane >> 3, rr = row0 + 8 * (mi & 1) + (lane & 7);
#pragma unroll
    for (int jj = 0; jj < 4; jj++) {
        const int j = 2 * jj + (mi >> 1);
        const uint32_t a = smem_addr(tile + rr * ld + 8 * j);
        asm volatile("stmatrix.sync.aligned.m8n8.x4.shared.b16 [%0], {%1, %2, %3, %4};"
                     ::"r"(a), "r"(pk[4 * jj]), "r"(pk[4 * jj + 1]), "r"(pk[4 * jj + 2]), "r"(pk[4 * jj + 3]) : "memory");
    }
}
// the inverse move: a warp's 16 x 64 part of a swizzled bf16 tile into pk[] (same indexing)
__device__ __forceinline__ void ld_frag_swz(uint32_t (&pk)[16], const unsigned char* tile, int row0, int lane) {
    const int mi = lane >> 3, rr = row0 + 8 * (mi & 1) + (lane & 7);
#pragma unroll
    for (int jj = 0; jj < 4; jj++) {
        const int j = 2 * jj + (mi >> 1);
        const uint32_t a = smem_addr(tile) + rr * 128 + (((j ^ rr) & 7) << 4);
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                     : "=r"(pk[4 * jj]), "=r"(pk[4 * jj + 1]), "=r"(pk[4 * jj + 2]), "=r"(pk[4 * jj + 3]) : "r"(a) : "memory");
    }
}

// ---------------------------------------------------------------- tcgen05.mma
// Shared-memory operand descriptor of a swizzled tile (both majors): start address, 1024 bytes between groups of
// eight rows, descriptor version 1 (sm_100), 128-byte swizzle.  The leading-dimension field is not used by a
// 64-element-wide swizzled operand; it holds the canonical value 1.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3FFF) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// MN-major operand 128 elements wide: two 64-element tiles `block_bytes` apart (the leading-dimension byte offset)
__device__ __forceinline__ uint64_t smem_desc_mn128(uint32_t saddr, uint32_t block_bytes) {
    return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)((block_bytes >> 4) & 0x3FFF) << 16) | (64ull << 32) | (1ull << 46) |
           (2ull << 61);
}
// Instruction descriptor: bf16 x bf16 -> fp32, M = 64, N = 64, dense; per-operand major and negation of A.
__host__ __device__ constexpr uint32_t idesc(bool a_mn_major, bool b_mn_major, bool negate_a, uint32_t n = 64) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((negate_a ? 1u : 0u) << 13) | ((a_mn_major ? 1u : 0u) << 15) |
           ((b_mn_major ? 1u : 0u) << 16) | ((n >> 3) << 17) | ((64u >> 4) << 24);
}
__device__ __forceinline__ void mma_issue(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t id, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(id), "r"(accumulate) : "memory");
}
// D (64 x 64 fp32 at d_tmem) = or += A B over the whole 64-deep contraction: four instructions.
// a_step / b_step: descriptor advance per instruction in 16-byte units (2 for a K-major operand, 128 for MN-major).
template <bool A_MN, bool B_MN, bool NEG_A>
__device__ __forceinline__ void mma_64x64x64(uint32_t d_tmem, uint32_t a_saddr, uint32_t b_saddr, bool accumulate) {
    constexpr uint32_t id = idesc(A_MN, B_MN, NEG_A);
    const uint64_t a0 = smem_desc(a_saddr), b0 = smem_desc(b_saddr);
#pragma unroll
    for (int k = 0; k < 4; k++)
        mma_issue(d_tmem, a0 + (uint64_t)(k * (A_MN ? 128 : 2)), b0 + (uint64_t)(k * (B_MN ? 128 : 2)), id,
                  (accumulate || k > 0) ? 1u : 0u);
}
// The barrier receives one arrival when every tcgen05.mma this thread issued before has completed.
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}

}  // namespace tc
}  // namespace fwp
