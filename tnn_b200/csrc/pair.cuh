// Building blocks of the kernels that run on CTA pairs (tcgen05 cta_group::2): the shared-memory plan of a pair tile
// and the pair forms of the TMA load, the UMMA, its commit and the TMEM allocation.
#pragma once
#include "linear_common.cuh"

namespace b200 {
namespace lin {

// Epilogue warps per CTA of the pair GEMM for a tile width: every warp drains 32 TMEM lanes (its quarter) x 64 or 128
// columns.  192-wide tiles get 12 warps (64 columns each): their GEMMs are short-K and the epilogue (GELU, residual)
// is what bounds them; more warps hide its latencies, and the register budget (128 per thread at 448 threads) holds.
template <int BN> constexpr int pair_epi_warps() { return BN == 192 ? 12 : 8; }

template <int BN, bool RES, bool FOLD, int EW = kEpiWarps>
struct PairCfg {
    static constexpr int A_BYTES = 128 * BK * 2;          // this CTA's 128 rows of x
    static constexpr int B_BYTES = (BN / 2) * BK * 2;     // this CTA's BN/2 rows of w
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    // output staging strips (TMA store); with RES two per warp, which also receive the residual tile (TMA load)
    static constexpr int EPI_WARPS = EW;
    static constexpr int THREADS = 64 + 32 * EW;
    static constexpr int COLS = BN / (EW / 4);            // accumulator columns drained by one epilogue warp
    static constexpr int OUT_BYTES = EW * kStageBytesPerWarp * strips_per_warp<RES>();
    static constexpr int TAIL_BYTES = OUT_BYTES + 512 + EW * vec_strips<FOLD>() * COLS * 4;   // + barriers + bias strips
    static constexpr int STAGES = (227 * 1024 - 1024 - TAIL_BYTES) / STAGE_BYTES > 8
                                      ? 8 : (227 * 1024 - 1024 - TAIL_BYTES) / STAGE_BYTES;
    static constexpr int OUT_OFFSET = STAGES * STAGE_BYTES;
    static constexpr int BAR_OFFSET = OUT_OFFSET + OUT_BYTES;
    static constexpr int BIAS_OFFSET = BAR_OFFSET + 512;
    static constexpr int SMEM_BYTES = OUT_OFFSET + TAIL_BYTES + 1024;
    static constexpr int TMEM_COLS = BN <= 64 ? 128 : (BN <= 128 ? 256 : 512);   // two accumulators of BN columns
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory object in the pair's leader CTA (cluster rank 0): the shared::cta address of a
// CTA in a cluster carries its rank in bit 24.
__device__ __forceinline__ uint32_t leader_addr(const void* p) { return smem_u32(p) & 0xFEFFFFFFu; }

__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t leader_bar, int32_t c0,
                                                 int32_t c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(leader_bar), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void umma_f16_ss_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                 uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// One arrival on the barrier at this shared-memory offset in both CTAs of the pair once all UMMAs issued so far are done.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    const uint16_t mask = 3;
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(smem_u32(bar)), "h"(mask)
        : "memory");
}
__device__ __forceinline__ void mbar_arrive_leader(uint64_t* bar) {
    asm volatile(
        "{\n\t.reg .b32 remote;\n\t"
        "mapa.shared::cluster.u32 remote, %0, 0;\n\t"
        "mbarrier.arrive.shared::cluster.b64 _, [remote];\n\t}\n"
        ::"r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

}  // namespace lin
}  // namespace b200
