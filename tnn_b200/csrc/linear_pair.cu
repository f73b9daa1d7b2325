// Projection / FFN GEMM on CTA pairs (tcgen05 cta_group::2): a cluster of two CTAs on neighbouring SMs computes one
// 256 x BN output tile.  Each CTA loads its own 128 rows of x and its own BN/2 rows of w per k-block (plain TMA, no
// multicast: the two CTAs load different data) and the UMMA of the pair reads both CTAs' shared memory, so per SM the
// w traffic from L2 and the shared-memory bandwidth spent on w are half of what a single-CTA 128 x BN tile needs, and
// the same 192 KB of pipeline stages covers 1.5x more tensor-core time.
//
// Roles per CTA (320 threads, 1 CTA per SM):
//   warp 0      : TMA producer for this CTA's halves; completion bytes of BOTH CTAs land on the leader's `full`
//                 barrier (cp.async.bulk.tensor ... .cta_group::2 with the barrier address of CTA rank 0).
//   warp 1      : TMEM allocation (cta_group::2, both CTAs); in the leader CTA one lane issues
//                 tcgen05.mma.cta_group::2 (256 x BN x 16) and commits, multicast to both CTAs' `empty` / `acc_full`.
//   warps 2..9  : epilogue of this CTA's 128 rows (its own TMEM), then arrive on the leader's `acc_empty`.
// Every wait is bounded; the two CTAs meet at a cluster barrier before either releases TMEM or exits.
#include "pair.cuh"

namespace b200 {
namespace lin {

namespace {

template <int BN, bool RES, bool FOLD>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(64 + 32 * pair_epi_warps<BN>(), 1)
linear_pair_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
                   const __grid_constant__ CUtensorMap tm_y, const __grid_constant__ CUtensorMap tm_r,
                   const LinearParams p) {
    constexpr int EW = pair_epi_warps<BN>();
    using C = PairCfg<BN, RES, FOLD, EW>;
    constexpr int STAGES = C::STAGES;
    extern __shared__ uint8_t smem_raw[];
    // Both CTAs of a pair must lay their buffers out at identical offsets: the dynamic shared-memory window starts at
    // the same offset in every CTA of a kernel, so rounding it up gives the same result in both.
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::BAR_OFFSET);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;
    uint64_t* acc_empty = acc_full + 2;
    uint64_t* res_bars = acc_empty + 2;                       // 3 per epilogue warp (RES only)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(res_bars + 3 * EW);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int pair_id = blockIdx.x >> 1;
    const int num_pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);    // leader's copy is the one in use: its own expect_tx arrival
            mbar_init(&empty[s], 1);   // one multicast commit per use
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 2 * EW);   // leader's copy: epilogue warps of both CTAs
        }
        for (int b = 0; b < 3 * EW; ++b) mbar_init(&res_bars[b], 1);
        *abort_flag = 0;
        mbar_fence_init();
        prefetch_tmap(&tm_x);
        prefetch_tmap(&tm_w);
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, C::TMEM_COLS);
        tmem_relinquish_pair();
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();   // the peer's barriers are initialised and its TMEM allocated before anything is signalled
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        // The weights are constants: while the previous kernel of the stream drains, the grid brings them from HBM
        // into L2 (every CTA a share of the (k-block, BN/2-row) boxes), so that the first wave of tiles does not pay
        // the HBM latency on its critical path.
        const int row_boxes = (p.N + BN / 2 - 1) / (BN / 2);
        const int boxes = p.num_k_blocks * row_boxes;
        for (int b = blockIdx.x; b < boxes; b += gridDim.x)
            tma_prefetch_l2_2d(&tm_w, (b % p.num_k_blocks) * BK, (b / p.num_k_blocks) * (BN / 2));
    }
    pdl_wait();   // x, the residual and the statistics come from earlier kernels; y may still be read by one

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (both CTAs)
        if (elect_one()) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = pair_id; ok && tile < p.num_tiles; tile += num_pairs) {
                const int m_blk = tile / p.num_n_tiles;
                const int n_blk = tile % p.num_n_tiles;
                for (int kb = 0; kb < p.num_k_blocks; ++kb, ++it) {
                    const uint32_t s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1u;
                    if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag)) { ok = false; break; }
                    uint8_t* a = smem + s * C::STAGE_BYTES;
                    uint8_t* b = a + C::A_BYTES;
                    if (leader) mbar_expect_tx(&full[s], 2 * C::STAGE_BYTES);
                    const uint32_t bar = leader_addr(&full[s]);
                    tma_load_2d_pair(a, &tm_x, bar, kb * BK, m_blk * 256 + static_cast<int>(rank) * 128);
                    tma_load_2d_pair(b, &tm_w, bar, kb * BK, n_blk * BN + static_cast<int>(rank) * (BN / 2));
                }
            }
            if (!ok) {
                for (int i = 0; i < 64; ++i) nanosleep(10000);   // let copies in flight land
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ UMMA issuer (leader CTA only)
        if (leader && elect_one()) {
            uint32_t it = 0, tcount = 0;
            bool ok = true;
            for (int tile = pair_id; ok && tile < p.num_tiles; tile += num_pairs, ++tcount) {
                const uint32_t buf = tcount & 1u;
                const uint32_t aph = (tcount >> 1) & 1u;
                if (!mbar_wait(&acc_empty[buf], aph ^ 1u, abort_flag)) { ok = false; break; }
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int kb = 0; kb < p.num_k_blocks; ++kb, ++it) {
                    const uint32_t s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1u;
                    if (!mbar_wait(&full[s], ph, abort_flag)) { ok = false; break; }
                    tcgen05_fence_after();
                    const uint32_t a_addr = smem_u32(smem + s * C::STAGE_BYTES);
                    const uint64_t a_desc = make_smem_desc_sw128(a_addr);
                    const uint64_t b_desc = make_smem_desc_sw128(a_addr + C::A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)
                        umma_f16_ss_pair(d_tmem, a_desc + 2u * k, b_desc + 2u * k, p.idesc, (kb | k) != 0 ? 1u : 0u);
                    umma_commit_pair(&empty[s]);
                }
                if (ok) umma_commit_pair(&acc_full[buf]);
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
        const int ew = warp - 2;
        const int quarter = warp & 3;
        const int half = ew >> 2;           // which COLS-wide part of the tile's columns this warp drains
        constexpr int COLS = C::COLS;
        constexpr int CHUNKS = COLS / 32;
        float* vec_w = reinterpret_cast<float*>(smem + C::BIAS_OFFSET) + ew * vec_strips<FOLD>() * COLS;
        WarpEpilogue<CHUNKS, RES, FOLD> epi{p, &tm_y, &tm_r,
                                            smem + C::OUT_OFFSET + ew * kStageBytesPerWarp * strips_per_warp<RES>(),
                                            res_bars + 3 * ew, abort_flag, lane, 0u};
        uint32_t tcount = 0;
        bool ok = true;
        const long long row_in_tile = static_cast<long long>(rank) * 128 + quarter * 32 + lane;
        if (pair_id < p.num_tiles)
            epi.prefetch_stats(static_cast<long long>(pair_id / p.num_n_tiles) * 256 + row_in_tile);
        for (int tile = pair_id; ok && tile < p.num_tiles; tile += num_pairs, ++tcount) {
            const int m_blk = tile / p.num_n_tiles;
            const int n_blk = tile % p.num_n_tiles;
            const uint32_t buf = tcount & 1u;
            const uint32_t aph = (tcount >> 1) & 1u;
            const long long row = static_cast<long long>(m_blk) * 256 + row_in_tile;
            epi.begin_tile(n_blk * BN + half * COLS, static_cast<int>(row) - lane);
            {   // the next tile's row statistics fly while this tile is drained
                const int next = tile + num_pairs;
                epi.prefetch_stats(next < p.num_tiles
                                       ? static_cast<long long>(next / p.num_n_tiles) * 256 + row_in_tile : -1);
            }
            stage_vectors<FOLD>(p, vec_w, n_blk * BN + half * COLS, COLS, lane);
            if (!mbar_wait(&acc_full[buf], aph, abort_flag)) { ok = false; break; }
            __syncwarp();
            tcgen05_fence_after();
            const uint32_t tacc = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN;
            if (!epi.template run<COLS>(vec_w, tacc, row, n_blk * BN, half * COLS)) { ok = false; break; }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (leader) mbar_arrive(&acc_empty[buf]);
                else mbar_arrive_leader(&acc_empty[buf]);
            }
        }
        // this warp's tile stores have read their strips; the writes themselves are complete when the grid is
        if (lane == 0) tma_store_wait_read<0>();
        __syncwarp();
    }

    // ---------------------------------------------------------------- teardown
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();   // neither CTA frees TMEM or leaves while the other may still signal or read it
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc_pair(tmem_base, C::TMEM_COLS);
    }
    if (threadIdx.x == 0 && *abort_flag != 0 && p.status != nullptr) atomicOr(p.status, 1u);
}

}  // namespace

template <int BN, bool RES, bool FOLD>
int launch_pair(const B200LinearDesc& d, cudaStream_t stream, int sm_count) {
    constexpr int EW = pair_epi_warps<BN>();
    using C = PairCfg<BN, RES, FOLD, EW>;
    static_assert(C::STAGES >= 3, "pipeline too shallow");
    static_assert(C::COLS % 32 == 0 && EW % 4 == 0, "every epilogue warp drains whole 32-column chunks");
    const uint64_t xd[2] = {static_cast<uint64_t>(d.K), static_cast<uint64_t>(d.M)};
    const uint64_t xs[1] = {static_cast<uint64_t>(d.ldx) * 2};
    const uint32_t xb[2] = {BK, 128};
    const uint64_t wd[2] = {static_cast<uint64_t>(d.K), static_cast<uint64_t>(d.N)};
    const uint64_t ws[1] = {static_cast<uint64_t>(d.ldw) * 2};
    const uint32_t wb[2] = {BK, BN / 2};
    CUtensorMap tx, tw, ty, tr;
    if (!get_tensor_map(&tx, d.x, 2, xd, xs, xb) || !get_tensor_map(&tw, d.w_nk, 2, wd, ws, wb)) return B200_ERR_DRIVER;
    ty = tx;   // placeholder when the output is fp32 (stored directly, map unused)
    if (d.out_dtype != B200_F32) {
        const uint64_t yd[2] = {static_cast<uint64_t>(d.N), static_cast<uint64_t>(d.M)};
        const uint64_t ys[1] = {static_cast<uint64_t>(d.ldy) * 2};
        const uint32_t yb[2] = {32, 32};
        if (!get_tensor_map(&ty, d.y, 2, yd, ys, yb, 64)) return B200_ERR_DRIVER;
    }
    tr = tx;   // placeholder without a residual
    if (RES) {
        const uint64_t rd[2] = {static_cast<uint64_t>(d.N), static_cast<uint64_t>(d.M)};
        const uint64_t rs[1] = {static_cast<uint64_t>(d.ldr) * 2};
        const uint32_t rb[2] = {32, 32};
        if (!get_tensor_map(&tr, d.residual, 2, rd, rs, rb, 64)) return B200_ERR_DRIVER;
    }

    LinearParams p;
    p.bias = d.bias;
    p.residual = d.residual;
    p.y = d.y;
    p.M = static_cast<int>(d.M);
    p.N = static_cast<int>(d.N);
    p.K = static_cast<int>(d.K);
    p.ldr = d.ldr;
    p.ldy = d.ldy;
    p.dtype = d.dtype;
    p.out_dtype = d.out_dtype;
    p.epilogue = d.epilogue;
    p.num_n_tiles = (p.N + BN - 1) / BN;
    p.num_tiles = ((p.M + 255) / 256) * p.num_n_tiles;
    p.num_k_blocks = (p.K + BK - 1) / BK;
    p.idesc = make_idesc_f16(256, BN, d.dtype == B200_BF16 ? 1 : 0, 0, 0);
    p.status = device_status_ptr();
    p.out_stats = d.out_stats;
    p.ln_in_stats = d.ln_in_stats;
    p.ln_c1 = d.ln_c1;
    p.ln_c2 = d.ln_c2;
    p.res_ln_stats = d.res_ln_stats;
    p.res_ln_gamma = d.res_ln_gamma;
    p.res_ln_beta = d.res_ln_beta;
    p.ln_eps = d.ln_eps;
    p.k_slots = (p.K + 31) / 32;
    p.n_slots = (p.N + 31) / 32;

    static PerDeviceOnce attr_once;
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_once.ensure(dev, []() {
            return cudaFuncSetAttribute(linear_pair_kernel<BN, RES, FOLD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        C::SMEM_BYTES) == cudaSuccess;
        }))
        return B200_ERR_LAUNCH;
    int pairs = max_active_pairs(BN);   // (the RES variant uses no more shared memory per CTA than its stage count allows)
    if (pairs <= 0) pairs = sm_count / 2;
    if (p.num_tiles < pairs) pairs = p.num_tiles;
    launch_kernel(linear_pair_kernel<BN, RES, FOLD>, dim3(2 * pairs), dim3(C::THREADS), C::SMEM_BYTES, stream, tx, tw,
                  ty, tr, p);
    count_launch();
    return check_launch();
}

namespace {
template <int BN>
int query_pairs(int sm_count) {
    // A persistent grid must not exceed what is co-resident: a pair that cannot be placed (GPCs with an odd number
    // of free SMs) would otherwise run as a second wave after the first has finished all the work.
    using C = PairCfg<BN, false, false, pair_epi_warps<BN>()>;
    if (cudaFuncSetAttribute(linear_pair_kernel<BN, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             C::SMEM_BYTES) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(sm_count & ~1), 1, 1);
    cfg.blockDim = dim3(C::THREADS, 1, 1);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, linear_pair_kernel<BN, false, false>, &cfg) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}
}  // namespace

int max_active_pairs(int bn) {
    static int cache[kMaxDevices][4] = {};
    static PerDeviceOnce once[4];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= kMaxDevices) return 0;
    const int idx = bn == 256 ? 0 : (bn == 192 ? 1 : (bn == 128 ? 2 : 3));
    once[idx].ensure(dev, [&]() {
        int sms = 0;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        int n = bn == 256 ? query_pairs<256>(sms) : (bn == 192 ? query_pairs<192>(sms)
                                                  : (bn == 128 ? query_pairs<128>(sms) : query_pairs<64>(sms)));
        if (n > sms / 2) n = sms / 2;
        cache[dev][idx] = n > 0 ? n : -1;
        return true;
    });
    return cache[dev][idx] > 0 ? cache[dev][idx] : 0;
}

template <int BN>
int launch_linear_pair(const B200LinearDesc& d, cudaStream_t stream, int sm_count) {
    // The TMA residual path needs 16-byte aligned residual rows (checked by the caller) and a half-precision residual.
    const bool fold = wants_fold(d);
    if (d.epilogue == B200_EPI_BIAS_RESIDUAL)
        return fold ? launch_pair<BN, true, true>(d, stream, sm_count) : launch_pair<BN, true, false>(d, stream, sm_count);
    return fold ? launch_pair<BN, false, true>(d, stream, sm_count) : launch_pair<BN, false, false>(d, stream, sm_count);
}

template int launch_linear_pair<256>(const B200LinearDesc&, cudaStream_t, int);
template int launch_linear_pair<192>(const B200LinearDesc&, cudaStream_t, int);
template int launch_linear_pair<128>(const B200LinearDesc&, cudaStream_t, int);
template int launch_linear_pair<64>(const B200LinearDesc&, cudaStream_t, int);

}  // namespace lin
}  // namespace b200
