// Several dependent operators of an encoder layer in one persistent launch on CTA pairs.
//
// A chain is a list of phases: GEMMs with fused epilogues (256 x 192 tiles, tcgen05 cta_group::2, the machinery of
// linear_pair.cu) and LayerNorms (64-row items).  Work is dealt statically: GEMM tile number g of the chain (phases
// concatenated, row-block-major inside a phase) belongs to CTA pair g mod #pairs, LayerNorm item number j to CTA
// j mod #CTAs.  Every role walks the phases in order:
//   warp 0      producer: before the first load of a tile it waits until the 256-row block of x has been completed by
//               the phase that writes it, then streams the k-blocks (TMA, pair form);
//   warp 1      UMMA issuer of the leader CTA: tiles back to back into the double-buffered accumulators;
//   warps 2..9  consumers: epilogue of every GEMM tile of the CTA, and the CTA's LayerNorm items in between.
// Completion of a row block by a phase is a counter in global memory: every consumer warp adds 1 (release) after its
// part of a tile / item is in memory, readers poll it (acquire, bounded) against the number of warps that contribute.
// The grid never exceeds what is co-resident, every CTA finishes its items of a phase before it touches a later phase,
// and an item only depends on earlier phases, so the CTA that owns a missing dependency is never blocked behind its
// waiter; all polls are bounded anyway and report through the status word.
//
// A warp must not hold back a completion it owes while it blocks on something that may depend on it.  Completions of
// TMA-stored tiles are therefore published lazily (after the next tile, when the stores have long landed) only along
// paths that cannot block; every potentially blocking wait first publishes what is pending.
#include <cstring>
#include <mutex>

#include "pair.cuh"

namespace b200 {
namespace lin {

namespace {

constexpr int CBN = 192;
constexpr int kMaxPhases = B200_CHAIN_MAX_PHASES;
constexpr int kMaxGemms = B200_CHAIN_MAX_LINEAR;
constexpr int kLnRows = 64;                      // rows per LayerNorm item: 8 warps x 8 rows
constexpr int kLnItemsPerBlock = 256 / kLnRows;

struct ChainPhaseDev {
    int kind;
    int slot;              // GEMM: index into the tensor-map table
    int first;             // chain-wide number of the phase's first item (GEMM tiles and LayerNorm items count apart)
    int count;             // items of the phase
    int wait_a, wait_b;    // phase that writes x / the residual of this phase, or -1
    // GEMM
    const float* bias;
    int N, K, num_n_tiles, num_k_blocks, epilogue;
    // LayerNorm
    const void* x;
    void* y;
    const float* gamma;
    const float* beta;
    long long ldx, ldy;
    int H;
    float eps;
};

struct alignas(64) ChainParams {
    CUtensorMap maps[kMaxGemms][4];   // x, w, y, residual
    LinearParams lp[kMaxGemms];       // what the shared epilogue code reads (shape, bias, dtypes, epilogue)
    ChainPhaseDev ph[kMaxPhases];
    int num_phases;
    int M;
    int m_blocks;
    int dtype;
    uint32_t idesc;
    int* sync;                        // [num_phases][m_blocks]
    unsigned int* status;
};

// Number of warp arrivals that complete row block `mb` of a phase.
__device__ __forceinline__ int phase_target(const ChainPhaseDev& q, int mb, int M) {
    if (q.kind == B200_PHASE_LINEAR) return q.num_n_tiles * 2 * kEpiWarps;
    const int rows = min(256, M - mb * 256);
    return ((rows + kLnRows - 1) / kLnRows) * kEpiWarps;
}
// Local number of the first item of a phase owned by `me` when item `first + t` belongs to (first + t) mod n.
__device__ __forceinline__ int first_owned(int first, int me, int n) { return ((me - first) % n + n) % n; }

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
linear_chain_kernel(const __grid_constant__ ChainParams cp) {
    using C = PairCfg<CBN, true, false>;
    constexpr int STAGES = C::STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::BAR_OFFSET);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;
    uint64_t* acc_empty = acc_full + 2;
    uint64_t* res_bars = acc_empty + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(res_bars + 2 * kEpiWarps);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int pair_id = blockIdx.x >> 1;
    const int num_pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 2 * kEpiWarps);
        }
        for (int b = 0; b < 2 * kEpiWarps; ++b) mbar_init(&res_bars[b], 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, C::TMEM_COLS);
        tmem_relinquish_pair();
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();
    pdl_wait();   // inputs of the first phases come from earlier kernels; the counters were cleared before the launch

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (both CTAs)
        if (elect_one()) {
            uint32_t it = 0;
            bool ok = true;
            for (int ph = 0; ok && ph < cp.num_phases; ++ph) {
                const ChainPhaseDev& P = cp.ph[ph];
                if (P.kind != B200_PHASE_LINEAR) continue;
                const CUtensorMap* tm_x = &cp.maps[P.slot][0];
                const CUtensorMap* tm_w = &cp.maps[P.slot][1];
                for (int t = first_owned(P.first, pair_id, num_pairs); ok && t < P.count; t += num_pairs) {
                    const int m_blk = t / P.num_n_tiles;
                    const int n_blk = t % P.num_n_tiles;
                    if (P.wait_a >= 0) {
                        if (!wait_rows(cp.sync + P.wait_a * cp.m_blocks + m_blk,
                                       phase_target(cp.ph[P.wait_a], m_blk, cp.M), abort_flag)) { ok = false; break; }
                        fence_async_proxy_all();   // the loads below (async proxy) come after the acquire
                    }
                    for (int kb = 0; kb < P.num_k_blocks; ++kb, ++it) {
                        const uint32_t s = it % STAGES;
                        const uint32_t phs = (it / STAGES) & 1u;
                        if (!mbar_wait(&empty[s], phs ^ 1u, abort_flag)) { ok = false; break; }
                        uint8_t* a = smem + s * C::STAGE_BYTES;
                        uint8_t* b = a + C::A_BYTES;
                        if (leader) mbar_expect_tx(&full[s], 2 * C::STAGE_BYTES);
                        const uint32_t bar = leader_addr(&full[s]);
                        tma_load_2d_pair(a, tm_x, bar, kb * BK, m_blk * 256 + static_cast<int>(rank) * 128);
                        tma_load_2d_pair(b, tm_w, bar, kb * BK, n_blk * CBN + static_cast<int>(rank) * (CBN / 2));
                    }
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
            for (int ph = 0; ok && ph < cp.num_phases; ++ph) {
                const ChainPhaseDev& P = cp.ph[ph];
                if (P.kind != B200_PHASE_LINEAR) continue;
                for (int t = first_owned(P.first, pair_id, num_pairs); ok && t < P.count; t += num_pairs, ++tcount) {
                    const uint32_t buf = tcount & 1u;
                    const uint32_t aph = (tcount >> 1) & 1u;
                    if (!mbar_wait(&acc_empty[buf], aph ^ 1u, abort_flag)) { ok = false; break; }
                    tcgen05_fence_after();
                    const uint32_t d_tmem = tmem_base + buf * CBN;
                    for (int kb = 0; kb < P.num_k_blocks; ++kb, ++it) {
                        const uint32_t s = it % STAGES;
                        const uint32_t phs = (it / STAGES) & 1u;
                        if (!mbar_wait(&full[s], phs, abort_flag)) { ok = false; break; }
                        tcgen05_fence_after();
                        const uint32_t a_addr = smem_u32(smem + s * C::STAGE_BYTES);
                        const uint64_t a_desc = make_smem_desc_sw128(a_addr);
                        const uint64_t b_desc = make_smem_desc_sw128(a_addr + C::A_BYTES);
#pragma unroll
                        for (int k = 0; k < BK / 16; ++k)
                            umma_f16_ss_pair(d_tmem, a_desc + 2u * k, b_desc + 2u * k, cp.idesc, (kb | k) != 0 ? 1u : 0u);
                        umma_commit_pair(&empty[s]);
                    }
                    if (ok) umma_commit_pair(&acc_full[buf]);
                }
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ consumers (both CTAs): epilogues and LayerNorms
        const int ew = warp - 2;
        const int quarter = warp & 3;
        const int half = ew >> 2;
        constexpr int COLS = CBN / 2;
        constexpr int CHUNKS = COLS / 32;
        float* vec_w = reinterpret_cast<float*>(smem + C::BIAS_OFFSET) + ew * COLS;
        uint8_t* strips = smem + C::OUT_OFFSET + ew * kStageBytesPerWarp * 2;
        uint32_t tcount = 0, cc = 0, rpar = 0;
        bool ok = true;
        int* pending = nullptr;       // completion owed for the last tile drained (its stores may still be in flight)
        uint32_t pending_cc = 0;
        // Publish the pending completion.  `all`: wait for every store of this warp; otherwise at least CHUNKS stores
        // were committed after the pending tile's, and waiting for all but those is enough (and free by now).
        auto publish = [&](bool all) {
            if (pending != nullptr) {
                if (lane == 0) {
                    if (!all && cc - pending_cc >= static_cast<uint32_t>(CHUNKS)) tma_store_wait_all<CHUNKS>();
                    else tma_store_wait_all<0>();
                    fence_async_proxy_all();
                    add_release(pending);
                }
                pending = nullptr;
            }
        };
        // Dependency of this warp on row block `mb` of phase `dep`: publishes first if it has to block.
        auto acquire_rows = [&](int dep, int mb) -> bool {
            const int* ctr = cp.sync + dep * cp.m_blocks + mb;
            const int target = phase_target(cp.ph[dep], mb, cp.M);
            int ready = 0;
            if (lane == 0) ready = load_acquire(ctr) >= target ? 1 : 0;
            ready = __shfl_sync(0xffffffffu, ready, 0);
            if (!ready) {
                publish(true);
                if (lane == 0) ready = wait_rows(ctr, target, abort_flag) ? 1 : 0;
                ready = __shfl_sync(0xffffffffu, ready, 0);
            }
            return ready != 0;
        };

        for (int ph = 0; ok && ph < cp.num_phases; ++ph) {
            const ChainPhaseDev& P = cp.ph[ph];
            if (P.kind == B200_PHASE_LINEAR) {
                const LinearParams& lp = cp.lp[P.slot];
                WarpEpilogue<CHUNKS, true, false> epi{lp, &cp.maps[P.slot][2], &cp.maps[P.slot][3], strips,
                                                      res_bars + 2 * ew, abort_flag, lane, cc};
                epi.rpar = rpar;
                epi.res_on = P.epilogue == B200_EPI_BIAS_RESIDUAL;
                const long long row_in_tile = static_cast<long long>(rank) * 128 + quarter * 32 + lane;
                for (int t = first_owned(P.first, pair_id, num_pairs); t < P.count; t += num_pairs, ++tcount) {
                    const int m_blk = t / P.num_n_tiles;
                    const int n_blk = t % P.num_n_tiles;
                    const uint32_t buf = tcount & 1u;
                    const uint32_t aph = (tcount >> 1) & 1u;
                    const long long row = static_cast<long long>(m_blk) * 256 + row_in_tile;
                    if (epi.res_on && P.wait_b >= 0) {
                        if (!acquire_rows(P.wait_b, m_blk)) { ok = false; break; }
                        if (lane == 0) fence_async_proxy_all();
                    }
                    epi.begin_tile(n_blk * CBN + half * COLS, static_cast<int>(row) - lane);
                    stage_vectors<false>(lp, vec_w, n_blk * CBN + half * COLS, COLS, lane);
                    {
                        int ready = 0;
                        if (lane == 0) ready = mbar_try_wait(&acc_full[buf], aph) ? 1 : 0;
                        ready = __shfl_sync(0xffffffffu, ready, 0);
                        if (!ready) {
                            publish(true);
                            if (!mbar_wait(&acc_full[buf], aph, abort_flag)) { ok = false; break; }
                        }
                    }
                    __syncwarp();
                    tcgen05_fence_after();
                    const uint32_t tacc = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * CBN;
                    if (!epi.template run<COLS>(vec_w, tacc, row, n_blk * CBN, half * COLS)) { ok = false; break; }
                    tcgen05_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        if (leader) mbar_arrive(&acc_empty[buf]);
                        else mbar_arrive_leader(&acc_empty[buf]);
                    }
                    cc = epi.cc;
                    publish(false);
                    pending = cp.sync + ph * cp.m_blocks + m_blk;
                    pending_cc = cc;
                }
                cc = epi.cc;
                rpar = epi.rpar;
            } else {
                // ---- LayerNorm items of this CTA: 64 rows each, 8 rows per warp in two batches of 4
                const int cta = static_cast<int>(blockIdx.x);
                const int num_ctas = static_cast<int>(gridDim.x);
                for (int j = first_owned(P.first, cta, num_ctas); j < P.count; j += num_ctas) {
                    const int m_blk = j / kLnItemsPerBlock;
                    publish(true);
                    if (P.wait_a >= 0 && !acquire_rows(P.wait_a, m_blk)) { ok = false; break; }
                    const long long row0 = static_cast<long long>(j) * kLnRows + ew * 8;
                    layernorm_rows_warp<4>(P.x, P.ldx, P.y, P.ldy, P.gamma, P.beta, P.H, P.eps, cp.dtype, row0, 8, cp.M,
                                           lane);
                    fence_async_proxy_all();   // the rows are read through TMA by the next GEMM
                    __syncwarp();
                    if (lane == 0) {
                        __threadfence();
                        add_release(cp.sync + ph * cp.m_blocks + m_blk);
                    }
                }
            }
        }
        publish(true);
        if (lane == 0) tma_store_wait_all<0>();
        __syncwarp();
    }

    // ---------------------------------------------------------------- teardown
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc_pair(tmem_base, C::TMEM_COLS);
    }
    if (threadIdx.x == 0 && *abort_flag != 0 && cp.status != nullptr) atomicOr(cp.status, 1u);
}

bool chain_layernorm_ok(const B200LayerNormDesc& d, int64_t M, int dtype) {
    if (!d.x || !d.y || !d.gamma || !d.beta || d.residual) return false;
    if (d.rows != M || d.H <= 0 || (d.H % 8) || d.H > 1024) return false;
    if ((d.ldx % 8) || (d.ldy % 8) || d.ldx < d.H || d.ldy < d.H) return false;
    if (d.in_dtype != dtype || d.out_dtype != dtype) return false;
    return aligned16(d.x) && aligned16(d.y) && aligned16(d.gamma) && aligned16(d.beta);
}

}  // namespace
}  // namespace lin
}  // namespace b200

extern "C" {

size_t b200_chain_sync_bytes(int64_t rows, int32_t phase_count) {
    if (rows <= 0 || phase_count <= 0) return 0;
    return static_cast<size_t>((rows + 255) / 256) * static_cast<size_t>(phase_count) * sizeof(int32_t);
}

int b200_chain_fwd(const B200ChainPhase* phases, int32_t count, void* sync_words, b200_stream_t stream_) {
    using namespace b200;
    using namespace b200::lin;
    if (!phases || !sync_words || count <= 0 || count > kMaxPhases) return B200_ERR_PARAM;
    if (reinterpret_cast<uintptr_t>(sync_words) & 3u) return B200_ERR_PARAM;
    const int sms = device_sm_count();
    if (sms <= 0) return B200_ERR_NOT_SM100;

    static ChainParams cp;   // too large for the stack frames of some hosts; calls are serialised by the mutex below
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    std::memset(&cp, 0, sizeof(cp));

    int64_t M = -1;
    int dtype = -1;
    int gemms = 0, gemm_items = 0, ln_items = 0;
    const void* outs[kMaxPhases] = {nullptr};
    for (int i = 0; i < count; ++i) {
        const B200ChainPhase& ph = phases[i];
        ChainPhaseDev& P = cp.ph[i];
        P.wait_a = P.wait_b = -1;
        if (ph.kind == B200_PHASE_LINEAR) {
            const B200LinearDesc& d = ph.linear;
            const int valid = validate_linear_desc(&d);
            if (valid != B200_OK) return valid;
            if (wants_fold(d) || d.out_dtype != d.dtype) return B200_ERR_UNSUPPORTED;
            if (gemms >= kMaxGemms) return B200_ERR_UNSUPPORTED;
            if (M < 0) { M = d.M; dtype = d.dtype; }
            if (d.M != M || d.dtype != dtype) return B200_ERR_PARAM;
            const uint64_t xd[2] = {static_cast<uint64_t>(d.K), static_cast<uint64_t>(d.M)};
            const uint64_t xs[1] = {static_cast<uint64_t>(d.ldx) * 2};
            const uint32_t xb[2] = {BK, 128};
            const uint64_t wd[2] = {static_cast<uint64_t>(d.K), static_cast<uint64_t>(d.N)};
            const uint64_t ws[1] = {static_cast<uint64_t>(d.ldw) * 2};
            const uint32_t wb[2] = {BK, CBN / 2};
            const uint64_t yd[2] = {static_cast<uint64_t>(d.N), static_cast<uint64_t>(d.M)};
            const uint64_t ys[1] = {static_cast<uint64_t>(d.ldy) * 2};
            const uint32_t yb[2] = {32, 32};
            if (!encode_tensor_map(&cp.maps[gemms][0], d.x, 2, xd, xs, xb) ||
                !encode_tensor_map(&cp.maps[gemms][1], d.w_nk, 2, wd, ws, wb) ||
                !encode_tensor_map(&cp.maps[gemms][2], d.y, 2, yd, ys, yb, 64))
                return B200_ERR_DRIVER;
            if (d.epilogue == B200_EPI_BIAS_RESIDUAL) {
                const uint64_t rs[1] = {static_cast<uint64_t>(d.ldr) * 2};
                if (!encode_tensor_map(&cp.maps[gemms][3], d.residual, 2, yd, rs, yb, 64)) return B200_ERR_DRIVER;
            } else {
                cp.maps[gemms][3] = cp.maps[gemms][2];
            }
            LinearParams& lp = cp.lp[gemms];
            lp.bias = d.bias;
            lp.M = static_cast<int>(d.M);
            lp.N = static_cast<int>(d.N);
            lp.K = static_cast<int>(d.K);
            lp.dtype = d.dtype;
            lp.out_dtype = d.dtype;
            lp.epilogue = d.epilogue;
            P.kind = B200_PHASE_LINEAR;
            P.slot = gemms++;
            P.bias = d.bias;
            P.N = static_cast<int>(d.N);
            P.K = static_cast<int>(d.K);
            P.num_n_tiles = static_cast<int>((d.N + CBN - 1) / CBN);
            P.num_k_blocks = static_cast<int>((d.K + BK - 1) / BK);
            P.epilogue = d.epilogue;
            P.first = gemm_items;
            P.count = static_cast<int>((d.M + 255) / 256) * P.num_n_tiles;
            gemm_items += P.count;
            for (int j = 0; j < i; ++j) {
                if (outs[j] == d.x) P.wait_a = j;
                if (d.epilogue == B200_EPI_BIAS_RESIDUAL && outs[j] == d.residual) P.wait_b = j;
            }
            outs[i] = d.y;
        } else if (ph.kind == B200_PHASE_ADD_LAYERNORM) {
            const B200LayerNormDesc& d = ph.layernorm;
            if (M < 0) { M = d.rows; dtype = d.in_dtype; }
            if (!is_half_dtype(dtype) || !chain_layernorm_ok(d, M, dtype)) return B200_ERR_PARAM;
            P.kind = B200_PHASE_ADD_LAYERNORM;
            P.x = d.x;
            P.y = d.y;
            P.gamma = d.gamma;
            P.beta = d.beta;
            P.ldx = d.ldx;
            P.ldy = d.ldy;
            P.H = static_cast<int>(d.H);
            P.eps = d.eps;
            P.first = ln_items;
            P.count = static_cast<int>((d.rows + kLnRows - 1) / kLnRows);
            ln_items += P.count;
            for (int j = 0; j < i; ++j)
                if (outs[j] == d.x) P.wait_a = j;
            outs[i] = d.y;
        } else {
            return B200_ERR_PARAM;
        }
    }
    if (M <= 0 || M > (1ll << 30)) return B200_ERR_PARAM;
    if (gemms == 0) return B200_ERR_UNSUPPORTED;   // a chain without a GEMM is a plain LayerNorm launch
    cp.num_phases = count;
    cp.M = static_cast<int>(M);
    cp.m_blocks = static_cast<int>((M + 255) / 256);
    cp.dtype = dtype;
    cp.idesc = make_idesc_f16(256, CBN, dtype == B200_BF16 ? 1 : 0, 0, 0);
    cp.sync = static_cast<int*>(sync_words);
    cp.status = device_status_ptr();

    using C = PairCfg<CBN, true, false>;
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        if (cudaFuncSetAttribute(linear_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) !=
            cudaSuccess)
            return B200_ERR_LAUNCH;
        attr_set[dev] = true;
    }
    int pairs = max_active_pairs(CBN);
    if (pairs <= 0) pairs = sms / 2;
    const int want = gemm_items > (ln_items + 1) / 2 ? gemm_items : (ln_items + 1) / 2;
    if (want < pairs) pairs = want;
    launch_kernel(linear_chain_kernel, dim3(2 * pairs), dim3(kThreads), C::SMEM_BYTES,
                  static_cast<cudaStream_t>(stream_), cp);
    count_launch();
    return check_launch();
}

}  // extern "C"
