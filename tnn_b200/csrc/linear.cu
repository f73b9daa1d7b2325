// Projection / FFN GEMM with fused epilogue for sm_100a:  y = epilogue(x . w^T + bias (+ residual)).
//
// Persistent, warp-specialised CTA (one per SM):
//   warp 0      : TMA producer   — x tile [128 x 64] and w tile [BN x 64] per k-block into a STAGES-deep ring of
//                                   128-byte-swizzled shared memory; completion on the stage's `full` mbarrier.
//   warp 1      : UMMA issuer    — owns the TMEM allocation (2 accumulators of BN fp32 columns); one elected lane
//                                   issues 4 x tcgen05.mma (128 x BN x 16) per k-block, commits the stage's `empty`
//                                   barrier, and commits `acc_full` after the last k-block of a tile.
//   warps 2..9  : epilogue       — tcgen05.ld of the accumulator (a thread owns one row: lane = row), bias / GELU /
//                                   residual in registers, 16-byte stores.  Two warps share a 32-row quarter and
//                                   split the columns.  While they drain accumulator b, the issuer fills b^1.
// Algorithmic work per launch: 2*M*N*K flop; HBM traffic at least (M*K + N*K + M*N (+ M*N residual)) elements.
#include "linear_common.cuh"

namespace b200 {
namespace lin {

template <int BN, int STAGES, bool FOLD>
struct Cfg {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int OUT_OFFSET = STAGES * STAGE_BYTES;               // output staging strips (TMA store)
    static constexpr int BAR_OFFSET = OUT_OFFSET + kEpiWarps * kStageBytesPerWarp;
    static constexpr int BIAS_OFFSET = BAR_OFFSET + 256;         // per-epilogue-warp bias slice: 8 x (BN/2) floats
    static constexpr int SMEM_BYTES = BIAS_OFFSET + kEpiWarps * vec_strips<FOLD>() * (BN / 2) * 4 + 1024;  // + slack for 1024-byte alignment
    static constexpr int TMEM_COLS = 2 * BN;                    // 128, 256 or 512: powers of two
};

template <int BN, int STAGES, bool FOLD>
__global__ void __launch_bounds__(kThreads, 1)
linear_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
              const __grid_constant__ CUtensorMap tm_y, const LinearParams p) {
    using C = Cfg<BN, STAGES, FOLD>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::BAR_OFFSET);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], kEpiWarps);
        }
        *abort_flag = 0;
        mbar_fence_init();
        prefetch_tmap(&tm_x);
        prefetch_tmap(&tm_w);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, C::TMEM_COLS);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();
    pdl_wait();   // inputs come from earlier kernels; the output may still be read by one

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (elect_one()) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x) {
                const int m_blk = tile / p.num_n_tiles;
                const int n_blk = tile % p.num_n_tiles;
                for (int kb = 0; kb < p.num_k_blocks; ++kb, ++it) {
                    const uint32_t s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1u;
                    if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag)) { ok = false; break; }
                    uint8_t* a = smem + s * C::STAGE_BYTES;
                    uint8_t* b = a + C::A_BYTES;
                    mbar_expect_tx(&full[s], C::STAGE_BYTES);
                    tma_load_2d(a, &tm_x, &full[s], kb * BK, m_blk * BM);
                    tma_load_2d(b, &tm_w, &full[s], kb * BK, n_blk * BN);
                }
            }
            if (!ok) {
                // Give copies already in flight time to land before the CTA's shared memory is released.
                for (int i = 0; i < 64; ++i) nanosleep(10000);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ UMMA issuer
        if (elect_one()) {
            uint32_t it = 0, tcount = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++tcount) {
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
                    for (int k = 0; k < BK / 16; ++k) {
                        // 16 elements along K = 32 bytes inside the 128-byte swizzled row: +2 in (address >> 4) units
                        umma_f16_ss(d_tmem, a_desc + 2u * k, b_desc + 2u * k, p.idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    umma_commit(&empty[s]);
                }
                if (ok) umma_commit(&acc_full[buf]);
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ epilogue
        const int ew = warp - 2;
        const int quarter = warp & 3;  // TMEM lanes 32*quarter .. 32*quarter+31 are the ones this warp may read
        const int half = ew >> 2;      // which half of the BN columns
        constexpr int COLS = BN / 2;
        constexpr int CHUNKS = COLS / 32;
        float* vec_w = reinterpret_cast<float*>(smem + C::BIAS_OFFSET) + ew * vec_strips<FOLD>() * COLS;  // private to this warp
        WarpEpilogue<CHUNKS, false, FOLD> epi{p, &tm_y, nullptr, smem + C::OUT_OFFSET + ew * kStageBytesPerWarp, nullptr,
                                        abort_flag, lane, 0u};
        uint32_t tcount = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++tcount) {
            const int m_blk = tile / p.num_n_tiles;
            const int n_blk = tile % p.num_n_tiles;
            const uint32_t buf = tcount & 1u;
            const uint32_t aph = (tcount >> 1) & 1u;
            // Stage this tile's bias slice while the accumulator is still being produced.
            const long long row = static_cast<long long>(m_blk) * BM + quarter * 32 + lane;
            epi.begin_tile(n_blk * BN + half * COLS, static_cast<int>(row) - lane);
            stage_vectors<FOLD>(p, vec_w, n_blk * BN + half * COLS, COLS, lane);
            if (!mbar_wait(&acc_full[buf], aph, abort_flag)) { ok = false; break; }
            __syncwarp();  // tcgen05.ld is warp-collective
            tcgen05_fence_after();
            const uint32_t tacc = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN;
            epi.template run<COLS>(vec_w, tacc, row, n_blk * BN, half * COLS);
            // This warp has read everything it needs from accumulator `buf`.
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
        if (lane == 0) tma_store_wait_all<0>();   // this warp's tile stores have left shared memory and landed
        __syncwarp();
    }

    // ---------------------------------------------------------------- teardown (also the exit of an aborted CTA)
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
    if (threadIdx.x == 0 && *abort_flag != 0 && p.status != nullptr) atomicOr(p.status, 1u);
}

int device_sm_count() {
    static std::atomic<int> sms[kMaxDevices];   // 0 = not looked up yet; every thread would store the same value
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= kMaxDevices) return 148;
    int v = sms[dev].load(std::memory_order_relaxed);
    if (v == 0) {
        int n = 0, major = 0;
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
        v = (major == 10) ? n : -1;
        sms[dev].store(v, std::memory_order_relaxed);
    }
    return v;
}

template <int BN, int STAGES, bool FOLD>
int launch_linear_t(const B200LinearDesc& d, cudaStream_t stream, int sm_count) {
    using C = Cfg<BN, STAGES, FOLD>;
    const uint64_t xd[2] = {static_cast<uint64_t>(d.K), static_cast<uint64_t>(d.M)};
    const uint64_t xs[1] = {static_cast<uint64_t>(d.ldx) * 2};
    const uint32_t xb[2] = {BK, BM};
    const uint64_t wd[2] = {static_cast<uint64_t>(d.K), static_cast<uint64_t>(d.N)};
    const uint64_t ws[1] = {static_cast<uint64_t>(d.ldw) * 2};
    const uint32_t wb[2] = {BK, BN};
    CUtensorMap tx, tw, ty;
    if (!get_tensor_map(&tx, d.x, 2, xd, xs, xb) || !get_tensor_map(&tw, d.w_nk, 2, wd, ws, wb)) return B200_ERR_DRIVER;
    ty = tx;   // placeholder when the output is fp32 (stored directly, map unused)
    if (d.out_dtype != B200_F32) {
        const uint64_t yd[2] = {static_cast<uint64_t>(d.N), static_cast<uint64_t>(d.M)};
        const uint64_t ys[1] = {static_cast<uint64_t>(d.ldy) * 2};
        const uint32_t yb[2] = {32, 32};
        if (!get_tensor_map(&ty, d.y, 2, yd, ys, yb, 64)) return B200_ERR_DRIVER;
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
    p.num_tiles = ((p.M + BM - 1) / BM) * p.num_n_tiles;
    p.num_k_blocks = (p.K + BK - 1) / BK;
    p.idesc = make_idesc_f16(BM, BN, d.dtype == B200_BF16 ? 1 : 0, 0, 0);
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
            return cudaFuncSetAttribute(linear_kernel<BN, STAGES, FOLD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        C::SMEM_BYTES) == cudaSuccess;
        }))
        return B200_ERR_LAUNCH;
    const int grid = p.num_tiles < sm_count ? p.num_tiles : sm_count;
    launch_kernel(linear_kernel<BN, STAGES, FOLD>, dim3(grid), dim3(kThreads), C::SMEM_BYTES, stream, tx, tw, ty, p);
    count_launch();
    return check_launch();
}

template <int BN, int STAGES>
int launch_linear(const B200LinearDesc& d, cudaStream_t stream, int sm_count) {
    if (wants_fold(d)) return launch_linear_t<BN, STAGES - 1, true>(d, stream, sm_count);
    return launch_linear_t<BN, STAGES, false>(d, stream, sm_count);
}

// Tile choice.  Estimated time ~ waves * (columns per tile * cost per column + fixed per-tile cost), in units of
// "accumulator columns per SM".  What bounds a k-block is the slower of the tensor pipe (2 clocks per accumulator
// column for a 256-row pair tile) and the SM's read port from L2 (64 bytes per clock: every SM of a pair fetches 128
// rows of x and BN/2 rows of w per k-block, (128 + BN/2) * 128 bytes): 512 | 512 clocks for BN = 256, 384 | 448 for 192,
// 256 | 384 for 128, 128 | 320 for 64 — the profile of the 256-wide tile shows 11.3 TB/s from L2 to the SMs, 80 % of
// 148 ports, at 89 % tensor-pipe activity.  Hence the cost per column rises as tiles narrow.  Single-CTA tiles
// (128 x BN) fetch BN rows of w per SM and k-block.
struct TileChoice {
    bool pair;
    int bn;
};
TileChoice choose_tile(int64_t M, int64_t N, int sm_count) {
    TileChoice best = {false, 128};
    double best_t = 1e300;
    if (M > 128) {
        const int bns[4] = {256, 192, 128, 64};
        const double cost[4] = {1.0, 1.17, 1.50, 2.50};
        for (int i = 0; i < 4; ++i) {
            int pairs = max_active_pairs(bns[i]);
            if (pairs <= 0) continue;
            const int64_t tiles = ((M + 255) / 256) * ((N + bns[i] - 1) / bns[i]);
            const int64_t waves = (tiles + pairs - 1) / pairs;
            const double t = static_cast<double>(waves) * (bns[i] * cost[i] + 16.0);
            if (t < best_t) {
                best_t = t;
                best = {true, bns[i]};
            }
        }
    }
    const int bns1[3] = {256, 128, 64};
    const double cost1[3] = {1.35, 1.50, 1.90};
    for (int i = 0; i < 3; ++i) {
        const int64_t tiles = ((M + BM - 1) / BM) * ((N + bns1[i] - 1) / bns1[i]);
        const int64_t waves = (tiles + sm_count - 1) / sm_count;
        const double t = static_cast<double>(waves) * (bns1[i] * cost1[i] + 16.0);
        if (t < best_t) {
            best_t = t;
            best = {false, bns1[i]};
        }
    }
    return best;
}

int validate_linear_desc(const B200LinearDesc* d) {
    if (!d || !d->x || !d->w_nk || !d->y) return B200_ERR_PARAM;
    if (d->M <= 0 || d->N <= 0 || d->K <= 0) return B200_ERR_PARAM;
    if (d->M > (1ll << 30) || d->N > (1ll << 30) || d->K > (1ll << 30)) return B200_ERR_UNSUPPORTED;
    if (!is_half_dtype(d->dtype)) return B200_ERR_PARAM;
    if (d->out_dtype != B200_F16 && d->out_dtype != B200_BF16 && d->out_dtype != B200_F32) return B200_ERR_PARAM;
    if (d->epilogue < B200_EPI_BIAS || d->epilogue > B200_EPI_BIAS_TANH) return B200_ERR_PARAM;
    if (d->epilogue == B200_EPI_BIAS_RESIDUAL && !d->residual) return B200_ERR_PARAM;
    if ((d->K % 8) || (d->N % 8) || (d->ldx % 8) || (d->ldw % 8) || (d->ldy % 8)) return B200_ERR_PARAM;
    if (d->ldx < d->K || d->ldw < d->K || d->ldy < d->N) return B200_ERR_PARAM;
    if (!aligned16(d->x) || !aligned16(d->w_nk) || !aligned16(d->y)) return B200_ERR_PARAM;
    if (d->bias && !aligned16(d->bias)) return B200_ERR_PARAM;
    if (d->epilogue == B200_EPI_BIAS_RESIDUAL && ((d->ldr % 8) || d->ldr < d->N || !aligned16(d->residual)))
        return B200_ERR_PARAM;
    if (d->ln_in_stats && (!d->ln_c1 || !d->ln_c2)) return B200_ERR_PARAM;
    if (d->res_ln_stats && (!d->res_ln_gamma || !d->res_ln_beta || d->epilogue != B200_EPI_BIAS_RESIDUAL))
        return B200_ERR_PARAM;
    return B200_OK;
}

}  // namespace lin
}  // namespace b200

extern "C" int b200_linear_fwd(const B200LinearDesc* d, b200_stream_t stream_) {
    using namespace b200;
    using namespace b200::lin;
    const int valid = validate_linear_desc(d);
    if (valid != B200_OK) return valid;
    const int sms = device_sm_count();
    if (sms <= 0) return B200_ERR_NOT_SM100;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    TileChoice tc;
    if (d->block_n == 0) {
        tc = choose_tile(d->M, d->N, sms);
    } else if (d->block_n > 0) {
        tc = {d->M > 128, d->block_n};
    } else {
        tc = {false, -d->block_n};
    }
    if (tc.pair) {
        switch (tc.bn) {
            case 256: return launch_linear_pair<256>(*d, stream, sms);
            case 192: return launch_linear_pair<192>(*d, stream, sms);
            case 128: return launch_linear_pair<128>(*d, stream, sms);
            case 64: return launch_linear_pair<64>(*d, stream, sms);
            default: return B200_ERR_PARAM;
        }
    }
    switch (tc.bn) {
        case 256: return launch_linear<256, 4>(*d, stream, sms);
        case 128: return launch_linear<128, 6>(*d, stream, sms);
        case 64: return launch_linear<64, 8>(*d, stream, sms);
        default: return B200_ERR_PARAM;
    }
}
