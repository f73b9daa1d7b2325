// Fused multi-head attention for sm_100a, head_dim 64:  out = softmax(scale * Q K^T + mask) V, flash-style: no score
// matrix ever leaves the SM.  Two kernels share the building blocks below:
//   attention_single_kernel   S <= 128: persistent CTAs (four per SM), one (sequence, head) item at a time;
//   attention_pingpong_kernel S  > 128: two 128-query tiles per CTA in ping-pong over a ring of 128-key tiles, one item
//                             (256 queries of one head of one sequence) per CTA: used for S > 1024;
//   attention_pingpong_persistent_kernel: the same with one CTA per SM walking a list of items without draining
//                             anything in between: used for 128 < S <= 1024.
//
//   TMA   : Q, K, V tiles [128 x 64] straight out of the token-major QKV activation (the head split of the unfused
//           graph's Reshape+Permute is just the TMA column coordinate h*64) into 128-byte-swizzled shared memory.
//   UMMA  : S = Q K^T (128 x 128 x 64, both operands K-major) and O = P V (128 x 64 x 128, P K-major from shared
//           memory, V MN-major exactly as TMA delivered it), fp32 accumulation in TMEM.
//   softmax: thread t owns query row t (TMEM lane t), so row max / row sum are in-thread; scores are scaled, the
//           additive key mask is applied in registers, excluded keys get weight exactly 0 (exp2(-inf)); P goes to the
//           second UMMA as half precision — through swizzled shared memory in the single-tile kernel, through tensor
//           memory in the long-sequence kernel.
// Algorithmic work per launch: 4 * S^2 * 64 * heads * B flop (QK^T and PV); HBM bytes: Q, K, V read once per CTA, O written.
#include <type_traits>

#include "common.cuh"
#include "ptx.cuh"

// 1: the next item's Q and K are loaded as soon as the scores are complete; 0: after PV (kept for A/B measurements)
#ifndef B200_ATTN_EARLY_QK
#define B200_ATTN_EARLY_QK 1
#endif

namespace b200 {
namespace {

// 2^x, one MUFU instruction: results below the normal range flush to zero, which is what a softmax weight wants.
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

constexpr int TQ = 128;   // queries per CTA
constexpr int TK = 128;   // keys per tile
constexpr int HD = 64;    // head dim
constexpr int kAttnThreads = 128;
constexpr int TILE_BYTES = 128 * HD * 2;  // 16 KB
// offsets of the Q, K and V tiles inside one shared-memory set of the single-tile kernel
constexpr int OFF_Q = 0;
constexpr int OFF_K = OFF_Q + TILE_BYTES;
constexpr int OFF_V = OFF_K + TILE_BYTES;

struct AttnParams {
    const float* mask_add;
    const int* kv_len;
    void* out;
    int S, heads;
    long long ldo;
    int dtype;
    float scale_log2;   // scale * log2(e)
    float mask_below;
    uint32_t idesc_qk, idesc_pv;
    unsigned int* status;
    int n_qb;            // long-sequence kernel: query blocks (NWG x 128 queries) per sequence
    long long n_items;   // long-sequence kernel: n_qb * heads * B
};

// ---------------------------------------------------------------------------------------------------------------
// Long sequences: two 128-query tiles per CTA, one softmax warpgroup each, so that the tensor pipe works on one tile's
// QK^T / PV while the other tile is in its softmax, and every K/V tile is loaded once for 256 queries.
// Roles (384 threads = 3 warpgroups, one CTA per SM; the control warpgroup hands most of its registers to the softmax
// warpgroups with setmaxnreg, 72 against 216 per thread):
//   warp 0      : producer — lane 0 issues the TMA loads (Q tiles once, then K/V tiles through a 4-stage ring); all 32
//                 lanes write the tile's key mask (log2 units, -inf = dropped) next to it and flag "plain" tiles;
//   warps 1, 2  : UMMA issuers, one per softmax warpgroup w.  As soon as the warpgroup has taken S_w(j) into registers
//                 the warp issues S_w(j+1) = Q_w K^T (both operands from shared memory) into TMEM columns
//                 [128w, 128w+128); when the warpgroup has written P_w(j) it issues O_w += P_w V with P_w read from TMEM
//                 columns [384+64w, +64) and V from shared memory, accumulated over all key tiles in TMEM columns
//                 [256+64w, +64).  A K/V stage is released by the commits of both warps;
//   warp 3      : idle;
//   warps 4..7  : softmax warpgroup 0 (query rows q0 .. q0+127), warps 8..11: warpgroup 1 (q0+128 .. q0+255);
//                 thread = row: the row's 128 scores come to registers in one TMEM load (the score columns are free for
//                 the next tile at once), maximum, then an exp pass (packed fp32 FMA / add, one MUFU per score) that
//                 writes P_w back to TMEM as packed half precision.  The running maximum is lazy: it only moves when a
//                 tile exceeds it by more than 2^8, and only then is O_w rescaled in place (tcgen05.ld / st); the row
//                 sum follows along.
// TMEM: 512 columns = 2 x (S 128 + O 64 + P 64).  All hand-offs are mbarriers with bounded waits (no named barriers:
// a role that gives up cannot strand another).
// What bounds it (d = 64): 128 x 128 scores cost 2 048 cycles of a scheduler's exp unit against 1 024 of the tensor pipe
// and ~1 100 of UMMA issue (a tcgen05.mma of these sizes occupies the pipe 44-57 cycles back to back).  The exp unit
// is saturated only while two warps of a scheduler are in their exp pass (see the phase offset below).
// NWG = softmax warpgroups (128-query tiles) per CTA; NWG = 1 gives two independent CTAs per SM (2-stage ring, half
// the TMEM each) and measures the same within a few percent.
#ifndef PP_NWG
#define PP_NWG 2
#endif
template <int NWG, int QSETS>
struct PPCfg {
    static constexpr int THREADS = 128 + 128 * NWG;               // control warpgroup + softmax warpgroups
    // registers per thread after the control warpgroup has handed most of its share to the softmax warpgroups
    static constexpr int REGS_CONTROL = 72;
    static constexpr int REGS_SOFTMAX = NWG == 1 ? 184 : 216;
    static constexpr int CTAS_PER_SM = NWG == 1 ? 2 : 1;
    // setmaxnreg moves registers inside the pool the CTA was launched with (threads x the launch-time count, which
    // the compiler caps at 65536 / threads-per-SM rounded down to 8): the raised count of the softmax warpgroups must
    // fit into what the control warpgroup gives up, or setmaxnreg.inc waits forever.
    static constexpr int REGS_LAUNCH = (65536 / (THREADS * (NWG == 1 ? 2 : 1))) / 8 * 8;
    static constexpr int NST = NWG == 1 ? 2 : 4;                  // K/V/mask ring depth (key tiles in flight)
    static constexpr int OFF_Q = 0;                               // two query sets of NWG x 16 KB (this item, the next)
    static constexpr int OFF_K = QSETS * NWG * TILE_BYTES;
    static constexpr int OFF_V = OFF_K + NST * TILE_BYTES;
    static constexpr int OFF_MASK = OFF_V + NST * TILE_BYTES;     // NST x 128 floats
    static constexpr int OFF_BAR = OFF_MASK + NST * TK * 4;
    static constexpr int SMEM = OFF_BAR + 512;
    static constexpr int TMEM_COLS = 256 * NWG;                   // per warpgroup: S 128 + O 64 + P 64
    static constexpr int COL_O = 128 * NWG;                       // + 64 * wg
    static constexpr int COL_P = 192 * NWG;                       // + 64 * wg
};
static_assert(128 * PPCfg<1, 1>::REGS_CONTROL + 128 * PPCfg<1, 1>::REGS_SOFTMAX <= PPCfg<1, 1>::THREADS * PPCfg<1, 1>::REGS_LAUNCH,
              "setmaxnreg: the softmax warpgroup's registers must come out of the CTA's own pool");
static_assert(128 * PPCfg<2, 1>::REGS_CONTROL + 256 * PPCfg<2, 1>::REGS_SOFTMAX <= PPCfg<2, 1>::THREADS * PPCfg<2, 1>::REGS_LAUNCH,
              "setmaxnreg: the softmax warpgroups' registers must come out of the CTA's own pool");
constexpr float kLazyLog2 = 8.0f;   // the running maximum moves only when a tile exceeds it by more than 2^8

template <int DT, int NWG>
__global__ void __launch_bounds__(PPCfg<NWG, 1>::THREADS, PPCfg<NWG, 1>::CTAS_PER_SM)
attention_pingpong_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                          const __grid_constant__ CUtensorMap tm_v, const AttnParams p) {
    using C = PPCfg<NWG, 1>;
    constexpr int PP_NST = C::NST;
    constexpr int PP_OFF_Q = C::OFF_Q, PP_OFF_K = C::OFF_K, PP_OFF_V = C::OFF_V, PP_OFF_MASK = C::OFF_MASK;
    constexpr int PP_OFF_BAR = C::OFF_BAR, PP_TMEM_COLS = C::TMEM_COLS;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + PP_OFF_BAR);
    uint64_t* q_full = bars + 0;
    uint64_t* k_full = bars + 1;                  // [PP_NST]
    uint64_t* v_full = k_full + PP_NST;           // [PP_NST]
    uint64_t* k_empty = v_full + PP_NST;          // [PP_NST]
    uint64_t* v_empty = k_empty + PP_NST;         // [PP_NST]
    uint64_t* m_full = v_empty + PP_NST;          // [PP_NST] mask of the stage written (32 arrivals)
    uint64_t* s_full = m_full + PP_NST;           // [2] per warpgroup
    uint64_t* p_full = s_full + 2;                // [2] (128 arrivals)
    uint64_t* o_full = p_full + 2;                // [2]
    uint64_t* s_free = o_full + 2;                // [2] the warpgroup holds its scores in registers (128 arrivals)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_free + 2);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    float* mask_s = reinterpret_cast<float*>(smem + PP_OFF_MASK);
    volatile uint32_t* plain_s = tmem_slot + 2;   // [PP_NST] per stage: every key valid, mask 0

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int q0 = blockIdx.x * NWG * TQ;
    const int head = blockIdx.y;
    const int b = blockIdx.z;

    if ((smem_u32(smem) & 1023u) != 0) {
        if (tid == 0 && p.status) atomicOr(p.status, 4u);
        return;
    }
    const bool two = NWG == 2 && (p.S - q0) > TQ;   // the second query tile exists

    if (tid == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < PP_NST; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&v_full[i], 1);
            mbar_init(&k_empty[i], two ? 2 : 1);   // one commit per UMMA-issuing warp
            mbar_init(&v_empty[i], two ? 2 : 1);
            mbar_init(&m_full[i], 32);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&s_full[i], 1);
            mbar_init(&p_full[i], 128);
            mbar_init(&o_full[i], 1);
            mbar_init(&s_free[i], 128);
        }
        *abort_flag = 0;
        mbar_fence_init();
        prefetch_tmap(&tm_q);
        prefetch_tmap(&tm_k);
        prefetch_tmap(&tm_v);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, PP_TMEM_COLS);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();
    pdl_wait();   // qkv and kv_len come from earlier kernels; the output may still be read by one

    // kv_len is written by a kernel earlier in the stream: it is read only here, behind the dependency wait.
    int kv_eff = p.S;
    bool additive_only = (p.mask_add == nullptr);
    if (p.kv_len != nullptr) {
        const int kl = p.kv_len[b];
        if (kl <= 0) additive_only = true;
        else kv_eff = kl < p.S ? kl : p.S;
    }
    const int n_tiles = (kv_eff + TK - 1) / TK;

    if (warp < 4) {
        setmaxnreg_dec<C::REGS_CONTROL>();   // the control warpgroup: producer, two UMMA issuers, an idle warp
        if (warp == 0) {
            // ------------------------------------------------------------ producer
            if (lane == 0) {
                mbar_expect_tx(q_full, (two ? 2 : 1) * TILE_BYTES);
                tma_load_3d(smem + PP_OFF_Q, &tm_q, q_full, head * HD, q0, b);
                if (two) tma_load_3d(smem + PP_OFF_Q + TILE_BYTES, &tm_q, q_full, head * HD, q0 + TQ, b);
            }
            bool ok = true;
            for (int j = 0; ok && j < n_tiles; ++j) {
                const int st = j % PP_NST;
                const uint32_t ph = (static_cast<uint32_t>(j) / PP_NST) & 1u;
                if (!mbar_wait(&k_empty[st], ph ^ 1u, abort_flag)) { ok = false; break; }
                if (lane == 0) {
                    mbar_expect_tx(&k_full[st], TILE_BYTES);
                    tma_load_3d(smem + PP_OFF_K + st * TILE_BYTES, &tm_k, &k_full[st], head * HD, j * TK, b);
                }
                // v_empty also says that both warpgroups are done with this stage's mask
                if (!mbar_wait(&v_empty[st], ph ^ 1u, abort_flag)) { ok = false; break; }
                if (lane == 0) {
                    mbar_expect_tx(&v_full[st], TILE_BYTES);
                    tma_load_3d(smem + PP_OFF_V + st * TILE_BYTES, &tm_v, &v_full[st], head * HD, j * TK, b);
                }
                bool zero = true;
    #pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int key = j * TK + lane * 4 + i;
                    float m = -INFINITY;
                    if (key < p.S) {
                        const float a = p.mask_add ? p.mask_add[static_cast<long long>(b) * p.S + key] : 0.f;
                        if (additive_only || a > p.mask_below) m = a * 1.4426950408889634f;
                    }
                    mask_s[st * TK + lane * 4 + i] = m;
                    zero = zero && m == 0.f;
                }
                // a "plain" tile (all 128 keys valid, additive mask 0) lets the softmax skip the mask altogether
                const bool plain_tile = __all_sync(0xffffffffu, zero) && p.scale_log2 > 0.f;
                if (lane == 0) plain_s[st] = plain_tile ? 1u : 0u;
                mbar_arrive(&m_full[st]);
            }
            if (!ok && lane == 0) {
                for (int i = 0; i < 64; ++i) nanosleep(10000);
            }
            __syncwarp();
        } else if (warp == 1 || (NWG == 2 && warp == 2 && two)) {
            // ------------------------------------------------------------ UMMA issuers (one warp per warpgroup)
            // The whole warp runs this role's control flow (all waits, all address arithmetic: warp-uniform, every
            // descriptor an immediate offset from one built once); lane 0 alone executes the tcgen05.mma and
            // tcgen05.commit instructions, so that each commit covers the UMMAs before it.
            bool ok = mbar_wait(q_full, 0, abort_flag);
            const uint32_t idesc_qk = p.idesc_qk, idesc_pv = p.idesc_pv;
            const uint64_t dq0 = make_smem_desc_sw128(smem_u32(smem + PP_OFF_Q));   // descriptor addresses: 16-byte units
            const uint64_t dk0 = make_smem_desc_sw128(smem_u32(smem + PP_OFF_K));   // + stage * (TILE_BYTES >> 4)
            const uint64_t dv0 = make_smem_desc_sw128(smem_u32(smem + PP_OFF_V));
            auto issue_s = [&](auto wg_c, const int st) {
                constexpr int wg = decltype(wg_c)::value;
                if (lane == 0) {
                    const uint64_t a_desc = dq0 + static_cast<uint64_t>(wg * (TILE_BYTES >> 4));
                    const uint64_t b_desc = dk0 + static_cast<uint64_t>(st * (TILE_BYTES >> 4));
                    const uint32_t d_tmem = tmem_base + wg * 128;
    #pragma unroll
                    for (int k = 0; k < HD / 16; ++k)
                        umma_f16_ss(d_tmem, a_desc + 2u * k, b_desc + 2u * k, idesc_qk, k != 0 ? 1u : 0u);
                    umma_commit(&s_full[wg]);
                }
                __syncwarp();
            };
            // Per key tile j and warpgroup w: as soon as the warpgroup holds S_w(j) in registers, S_w(j+1) is issued;
            // when it has written P_w(j), P_w V(j) follows.  `last` = this is the CTA's last warpgroup: its commits
            // release the K / V stages.
            auto step_s = [&](auto wg_c, const int j, const bool last) -> bool {
                constexpr int wg = decltype(wg_c)::value;
                if (j + 1 >= n_tiles) return true;
                const int st_next = (j + 1) % PP_NST;
                if (!mbar_wait(&s_free[wg], static_cast<uint32_t>(j) & 1u, abort_flag)) return false;
                if (!mbar_wait(&k_full[st_next], (static_cast<uint32_t>(j + 1) / PP_NST) & 1u, abort_flag)) return false;
                tcgen05_fence_after();
                issue_s(wg_c, st_next);
                if (last && lane == 0) umma_commit(&k_empty[st_next]);
                return true;
            };
            auto step_pv = [&](auto wg_c, const int j, const bool last) -> bool {
                constexpr int wg = decltype(wg_c)::value;
                const int st = j % PP_NST;
                if (!mbar_wait(&p_full[wg], static_cast<uint32_t>(j) & 1u, abort_flag)) return false;
                if (!mbar_wait(&v_full[st], (static_cast<uint32_t>(j) / PP_NST) & 1u, abort_flag)) return false;
                tcgen05_fence_after();
                if (lane == 0) {
                    const uint64_t b_desc = dv0 + static_cast<uint64_t>(st * (TILE_BYTES >> 4));
                    const uint32_t d_tmem = tmem_base + C::COL_O + wg * 64;
                    const uint32_t a_tmem = tmem_base + C::COL_P + wg * 64;
                    const uint32_t acc0 = j != 0 ? 1u : 0u;
                    // O_w accumulates in TMEM over all key tiles (the softmax rescales it in place when it must);
                    // P_w is read from TMEM (8 columns per 16 keys), V from shared memory (2 KB per 16 keys)
    #pragma unroll
                    for (int k = 0; k < TK / 16; ++k)
                        umma_f16_ts(d_tmem, a_tmem + k * 8, b_desc + static_cast<uint64_t>(k * (2048 >> 4)), idesc_pv,
                                    k != 0 ? 1u : acc0);
                    umma_commit(&o_full[wg]);
                    if (last) umma_commit(&v_empty[st]);
                }
                __syncwarp();
                return true;
            };
            if (ok) ok = mbar_wait(&k_full[0], 0, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            auto run = [&](auto wg_c) {
                if (ok) {
                    tcgen05_fence_after();
                    issue_s(wg_c, 0);
                    if (lane == 0) umma_commit(&k_empty[0]);
                }
                for (int j = 0; ok && j < n_tiles; ++j) {
                    ok = step_s(wg_c, j, true);
                    if (ok) ok = step_pv(wg_c, j, true);
                    ok = __all_sync(0xffffffffu, ok);
                }
            };
            if (warp == 1) run(std::integral_constant<int, 0>{});
            else run(std::integral_constant<int, NWG - 1>{});
            __syncwarp();
        }
    } else {
        setmaxnreg_inc<C::REGS_SOFTMAX>();
        // ------------------------------------------------------------ softmax warpgroups
        const int wg = (warp - 4) >> 2;   // warps 4..7 -> 0, 8..11 -> 1
        const int r_in_tile = ((warp & 3) << 5) + lane;          // TMEM lane = query row of the tile
        const uint32_t lane_field = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t t_s = tmem_base + lane_field + wg * 128;
        const uint32_t t_o = tmem_base + lane_field + C::COL_O + wg * 64;
        const uint32_t t_p = tmem_base + lane_field + C::COL_P + wg * 64;
        if (wg == 0 || two) {
            float m_run = -INFINITY, l_run = 0.f;
            bool ok = true;
            for (int j = 0; j < n_tiles; ++j) {
                const int st = j % PP_NST;
                const uint32_t ph = static_cast<uint32_t>(j) & 1u;
                if (!mbar_wait(&m_full[st], (static_cast<uint32_t>(j) / PP_NST) & 1u, abort_flag)) { ok = false; break; }
                if (!mbar_wait(&s_full[wg], ph, abort_flag)) { ok = false; break; }
                __syncwarp();
                tcgen05_fence_after();
                // The row's 128 scores move to registers in one go and the score columns are handed back at once:
                // the next tile's QK^T runs while this tile's softmax is still at work.
                uint32_t s[TK];
#pragma unroll
                for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x32(t_s + c * 32, reinterpret_cast<uint32_t(&)[32]>(s[c * 32]));
#pragma unroll
                for (int c = 0; c < 4; ++c) tmem_ld_wait(reinterpret_cast<uint32_t(&)[32]>(s[c * 32]));
                tcgen05_fence_before();
                mbar_arrive(&s_free[wg]);
                const float* mrow = mask_s + st * TK;
                const bool plain_tile = plain_s[st] != 0u;   // warp-uniform (CTA-uniform)
                float tmx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // independent chains (latency)
                if (plain_tile) {
#pragma unroll
                    for (int g = 0; g < TK / 8; ++g) {
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                            tmx[c] = fmax3(tmx[c], __uint_as_float(s[g * 8 + c * 2]), __uint_as_float(s[g * 8 + c * 2 + 1]));
                    }
                } else {
                    // s <- score * scale + mask (log2 units; -inf drops the key): the exp pass only subtracts the maximum
                    const uint64_t sc2 = pack_f32x2(p.scale_log2, p.scale_log2);
#pragma unroll
                    for (int g = 0; g < TK / 4; ++g) {
                        const float4 mk = *reinterpret_cast<const float4*>(mrow + g * 4);
                        float v0, v1, v2, v3;
                        unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(s[g * 4 + 0]), __uint_as_float(s[g * 4 + 1])), sc2,
                                               pack_f32x2(mk.x, mk.y)), v0, v1);
                        unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(s[g * 4 + 2]), __uint_as_float(s[g * 4 + 3])), sc2,
                                               pack_f32x2(mk.z, mk.w)), v2, v3);
                        s[g * 4 + 0] = __float_as_uint(v0);
                        s[g * 4 + 1] = __float_as_uint(v1);
                        s[g * 4 + 2] = __float_as_uint(v2);
                        s[g * 4 + 3] = __float_as_uint(v3);
                        tmx[g & 1] = fmax3(tmx[g & 1], v0, v1);
                        tmx[2 + (g & 1)] = fmax3(tmx[2 + (g & 1)], v2, v3);
                    }
                }
                float tmax = fmaxf(fmaxf(tmx[0], tmx[1]), fmaxf(tmx[2], tmx[3]));
                if (plain_tile) tmax *= p.scale_log2;   // = max of the scaled scores: the scale is positive
                // Lazy reference maximum: it only moves when the tile's maximum exceeds it by more than 2^kLazyLog2
                // (weights stay <= 2^kLazyLog2, exact in half precision and harmless in the fp32 sums), so most tiles
                // leave the output accumulator in TMEM untouched.
                const bool move = tmax > m_run + kLazyLog2;
                const float m_new = move ? tmax : m_run;
                const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
                const float alpha = move ? fast_exp2(m_run - m_use) : 1.f;
                // PV of the previous tile must be complete: it reads the P buffer written below, and it writes the
                // accumulator a rescale would touch.
                if (j > 0 && !mbar_wait(&o_full[wg], static_cast<uint32_t>(j - 1) & 1u, abort_flag)) { ok = false; break; }
                __syncwarp();
                if (j > 0 && __any_sync(0xffffffffu, move)) {
                    tcgen05_fence_after();
#pragma unroll
                    for (int cc = 0; cc < HD / 32; ++cc) {
                        uint32_t ro[32];
                        tmem_ld_32x32b_x32(t_o + cc * 32, ro);
                        tmem_ld_wait(ro);
#pragma unroll
                        for (int e = 0; e < 32; ++e) ro[e] = __float_as_uint(__uint_as_float(ro[e]) * alpha);
                        tmem_st_32x32b_x32(t_o + cc * 32, ro);
                    }
                }
                // Phase offset.  A scheduler's exp unit is saturated only while both of its softmax warps are in their exp
                // pass (8.9 cycles per score per scheduler), runs at ~70 % with one (11.6) and idles with none; started
                // together the two warpgroups stay in lockstep: both in the exp pass, then both out of it.  So warpgroup
                // 1 begins its first exp pass only when warpgroup 0 has finished its own; for the next tiles one's exp pass
                // covers the other's loads, maximum and hand-offs.  (The offset decays over ~6 tiles; renewing it every
                // tile, every second or every fourth tile, or holding it with a mutual rule, all measured slower than
                // letting it decay.)
                if (NWG == 2 && two && wg == 1 && j == 0 && !mbar_wait(&p_full[0], 0, abort_flag)) { ok = false; break; }
                // exp pass: P goes to tensor memory as the A operand of the PV UMMA, two consecutive keys per 32-bit
                // column, 32 keys at a time into columns [16c, 16c + 16) of the warpgroup's P region
                const uint64_t mul2 = plain_tile ? pack_f32x2(p.scale_log2, p.scale_log2) : pack_f32x2(1.f, 1.f);
                const uint64_t neg2 = pack_f32x2(-m_use, -m_use);
                uint64_t ps2[2] = {0ull, 0ull};   // 2 x 2 partial sums
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t pk[16];
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        const int i = c * 32 + e * 2;
                        float x0, x1;
                        unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(s[i]), __uint_as_float(s[i + 1])), mul2, neg2), x0, x1);
                        x0 = fast_exp2(x0);
                        x1 = fast_exp2(x1);
                        ps2[e & 1] = add_f32x2(ps2[e & 1], pack_f32x2(x0, x1));
                        pk[e] = pack2t<DT>(x0, x1);
                    }
                    tmem_st_32x32b_x16(t_p + c * 16, pk);
                }
                float a0, a1, a2, a3;
                unpack_f32x2(ps2[0], a0, a1);
                unpack_f32x2(ps2[1], a2, a3);
                l_run = l_run * alpha + ((a0 + a1) + (a2 + a3));
                m_run = m_new;
                tmem_st_wait();               // P (and a rescaled O) have reached tensor memory
                tcgen05_fence_before();
                mbar_arrive(&p_full[wg]);
            }
            // the last PV
            if (ok && n_tiles > 0 && !mbar_wait(&o_full[wg], static_cast<uint32_t>(n_tiles - 1) & 1u, abort_flag)) ok = false;
            __syncwarp();
            tcgen05_fence_after();
            const int q = q0 + wg * TQ + r_in_tile;
            if (ok) {   // warp-uniform: the TMEM loads are collective
                const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
                uint16_t* dst =
                    reinterpret_cast<uint16_t*>(p.out) + (static_cast<long long>(b) * p.S + q) * p.ldo + head * HD;
#pragma unroll
                for (int c = 0; c < HD / 32; ++c) {
                    uint32_t r[32];
                    tmem_ld_32x32b_x32(t_o + c * 32, r);
                    tmem_ld_wait(r);
                    if (q < p.S) {
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            uint4 qv;
                            qv.x = pack2t<DT>(__uint_as_float(r[g * 8 + 0]) * inv, __uint_as_float(r[g * 8 + 1]) * inv);
                            qv.y = pack2t<DT>(__uint_as_float(r[g * 8 + 2]) * inv, __uint_as_float(r[g * 8 + 3]) * inv);
                            qv.z = pack2t<DT>(__uint_as_float(r[g * 8 + 4]) * inv, __uint_as_float(r[g * 8 + 5]) * inv);
                            qv.w = pack2t<DT>(__uint_as_float(r[g * 8 + 6]) * inv, __uint_as_float(r[g * 8 + 7]) * inv);
                            *reinterpret_cast<uint4*>(dst + c * 32 + g * 8) = qv;
                        }
                    }
                }
            }
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, PP_TMEM_COLS);
    }
    if (tid == 0 && *abort_flag != 0 && p.status != nullptr) atomicOr(p.status, 2u);
}

// The same kernel as a persistent one, for items of up to 8 key tiles (S <= 1024), where what happens between two items
// weighs most: one CTA per resident slot, items dealt round-robin.  The tile loop is written out a second time instead
// of being shared with the kernel above: the throughput of both depends on the phase relation the two softmax
// warpgroups fall into, and that relation reacted to every restructuring that was measured (this form run with one
// item per CTA is 5-8 % slower than the kernel above on items of 16 and 32 tiles; with the UMMA-issuing warps
// specialised at compile time it is 8-16 % slower than as written here), so each form keeps the code it was tuned with.
template <int DT, int NWG>
__global__ void __launch_bounds__(PPCfg<NWG, 2>::THREADS, PPCfg<NWG, 2>::CTAS_PER_SM)
attention_pingpong_persistent_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                          const __grid_constant__ CUtensorMap tm_v, const AttnParams p) {
    using C = PPCfg<NWG, 2>;
    constexpr int PP_NST = C::NST;
    constexpr int PP_OFF_Q = C::OFF_Q, PP_OFF_K = C::OFF_K, PP_OFF_V = C::OFF_V, PP_OFF_MASK = C::OFF_MASK;
    constexpr int PP_OFF_BAR = C::OFF_BAR, PP_TMEM_COLS = C::TMEM_COLS;
    constexpr int Q_SET_BYTES = NWG * TILE_BYTES;   // the query tiles of one item
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + PP_OFF_BAR);
    uint64_t* q_full = bars + 0;                  // [2] the two query sets
    uint64_t* q_empty = bars + 2;                 // [2] every QK^T that reads the set has completed
    uint64_t* k_full = bars + 4;                  // [PP_NST]
    uint64_t* v_full = k_full + PP_NST;           // [PP_NST]
    uint64_t* k_empty = v_full + PP_NST;          // [PP_NST]
    uint64_t* v_empty = k_empty + PP_NST;         // [PP_NST]
    uint64_t* m_full = v_empty + PP_NST;          // [PP_NST] mask of the stage written (32 arrivals)
    uint64_t* s_full = m_full + PP_NST;           // [2] per warpgroup
    uint64_t* p_full = s_full + 2;                // [2] (128 arrivals)
    uint64_t* o_full = p_full + 2;                // [2]
    uint64_t* s_free = o_full + 2;                // [2] the warpgroup holds its scores in registers (128 arrivals)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_free + 2);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    float* mask_s = reinterpret_cast<float*>(smem + PP_OFF_MASK);
    volatile uint32_t* plain_s = tmem_slot + 2;   // [PP_NST] per stage: every key valid, mask 0
    volatile uint32_t* wg0_tiles = tmem_slot + 2 + PP_NST;   // key tiles warpgroup 0 has written its weights for

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;

    if ((smem_u32(smem) & 1023u) != 0) {
        if (tid == 0 && p.status) atomicOr(p.status, 4u);
        return;
    }

    if (tid == 0) {
        *wg0_tiles = 0;
        for (int i = 0; i < 2; ++i) {
            mbar_init(&q_full[i], 1);
            mbar_init(&q_empty[i], NWG);           // one commit per UMMA-issuing warp
        }
        for (int i = 0; i < PP_NST; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&v_full[i], 1);
            mbar_init(&k_empty[i], NWG);           // one commit per UMMA-issuing warp
            mbar_init(&v_empty[i], NWG);
            mbar_init(&m_full[i], 32);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&s_full[i], 1);
            mbar_init(&p_full[i], 128);
            mbar_init(&o_full[i], 1);
            mbar_init(&s_free[i], 128);
        }
        *abort_flag = 0;
        mbar_fence_init();
        prefetch_tmap(&tm_q);
        prefetch_tmap(&tm_k);
        prefetch_tmap(&tm_v);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, PP_TMEM_COLS);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();
    pdl_wait();   // qkv and kv_len come from earlier kernels; the output may still be read by one

    // Persistent CTAs: items (a block of NWG x 128 queries of one head of one sequence) are dealt round-robin, and every
    // role walks the same list.  Nothing is drained between items: the K/V ring, the score / weight / output columns
    // and all barriers carry on (phases follow running counters), the next item's queries land in the other of two
    // query sets while this item is still at work, and its first QK^T is issued during this item's last softmax.
    // `t0` = number of key tiles of all earlier items of this CTA (ring stage and phase of the item's first tile).
    struct Item {
        int b, head, q0, n_tiles;
        bool two;         // the second query tile exists
        bool additive_only;
    };
    auto load_item = [&](int id) -> Item {
        Item it;
        const int qb = id % p.n_qb;
        const int rest = id / p.n_qb;
        it.head = rest % p.heads;
        it.b = rest / p.heads;
        it.q0 = qb * NWG * TQ;
        it.two = NWG == 2 && (p.S - it.q0) > TQ;
        // kv_len is written by a kernel earlier in the stream: it is read only here, behind the dependency wait.
        int kv_eff = p.S;
        it.additive_only = (p.mask_add == nullptr);
        if (p.kv_len != nullptr) {
            const int kl = p.kv_len[it.b];
            if (kl <= 0) it.additive_only = true;
            else kv_eff = kl < p.S ? kl : p.S;
        }
        it.n_tiles = (kv_eff + TK - 1) / TK;
        return it;
    };
    const int n_items = static_cast<int>(p.n_items);
    const int id0 = static_cast<int>(blockIdx.x), id_step = static_cast<int>(gridDim.x);

    if (warp < 4) {
        setmaxnreg_dec<C::REGS_CONTROL>();   // the control warpgroup: producer, two UMMA issuers, an idle warp
        if (warp == 0) {
            // ------------------------------------------------------------ producer
            bool ok = true;
            uint32_t t0 = 0;   // key tiles of the CTA's earlier items
            int k = 0;         // items of the CTA so far
            for (int id = id0; ok && id < n_items; id += id_step, ++k) {
                const Item it = load_item(id);
                const int set = k & 1;
                // the set's previous item (two items back) must have finished its last QK^T
                if (!mbar_wait(&q_empty[set], ((static_cast<uint32_t>(k) >> 1) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
                if (lane == 0) {
                    uint8_t* qs = smem + PP_OFF_Q + set * Q_SET_BYTES;
                    mbar_expect_tx(&q_full[set], (it.two ? 2 : 1) * TILE_BYTES);
                    tma_load_3d(qs, &tm_q, &q_full[set], it.head * HD, it.q0, it.b);
                    if (it.two) tma_load_3d(qs + TILE_BYTES, &tm_q, &q_full[set], it.head * HD, it.q0 + TQ, it.b);
                }
                for (int j = 0; ok && j < it.n_tiles; ++j) {
                    const uint32_t t = t0 + static_cast<uint32_t>(j);
                    const int st = static_cast<int>(t % PP_NST);
                    const uint32_t ph = (t / PP_NST) & 1u;
                    if (!mbar_wait(&k_empty[st], ph ^ 1u, abort_flag)) { ok = false; break; }
                    if (lane == 0) {
                        mbar_expect_tx(&k_full[st], TILE_BYTES);
                        tma_load_3d(smem + PP_OFF_K + st * TILE_BYTES, &tm_k, &k_full[st], it.head * HD, j * TK, it.b);
                    }
                    // v_empty also says that both warpgroups are done with this stage's mask
                    if (!mbar_wait(&v_empty[st], ph ^ 1u, abort_flag)) { ok = false; break; }
                    if (lane == 0) {
                        mbar_expect_tx(&v_full[st], TILE_BYTES);
                        tma_load_3d(smem + PP_OFF_V + st * TILE_BYTES, &tm_v, &v_full[st], it.head * HD, j * TK, it.b);
                    }
                    bool zero = true;
    #pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int key = j * TK + lane * 4 + i;
                        float m = -INFINITY;
                        if (key < p.S) {
                            const float a = p.mask_add ? p.mask_add[static_cast<long long>(it.b) * p.S + key] : 0.f;
                            if (it.additive_only || a > p.mask_below) m = a * 1.4426950408889634f;
                        }
                        mask_s[st * TK + lane * 4 + i] = m;
                        zero = zero && m == 0.f;
                    }
                    // a "plain" tile (all 128 keys valid, additive mask 0) lets the softmax skip the mask altogether
                    const bool plain_tile = __all_sync(0xffffffffu, zero) && p.scale_log2 > 0.f;
                    if (lane == 0) plain_s[st] = plain_tile ? 1u : 0u;
                    mbar_arrive(&m_full[st]);
                }
                t0 += static_cast<uint32_t>(it.n_tiles);
            }
            if (!ok && lane == 0) {
                for (int i = 0; i < 64; ++i) nanosleep(10000);
            }
            __syncwarp();
        } else if (warp == 1 || (NWG == 2 && warp == 2)) {
            // ------------------------------------------------------------ UMMA issuers (one warp per warpgroup)
            // The whole warp runs this role's control flow (all waits, all address arithmetic: warp-uniform, every
            // descriptor an immediate offset from one built once); lane 0 alone executes the tcgen05.mma and
            // tcgen05.commit instructions, so that each commit covers the UMMAs before it.  Both warps walk every
            // item: where an item has no second query tile, warp 2 issues nothing but still waits for the stage's
            // loads and commits, so that every "empty" barrier gets its NWG arrivals once per use and in step.
            const int wg = warp - 1;
            const uint32_t idesc_qk = p.idesc_qk, idesc_pv = p.idesc_pv;
            const uint64_t dq0 = make_smem_desc_sw128(smem_u32(smem + PP_OFF_Q));   // descriptor addresses: 16-byte units
            const uint64_t dk0 = make_smem_desc_sw128(smem_u32(smem + PP_OFF_K));   // + stage * (TILE_BYTES >> 4)
            const uint64_t dv0 = make_smem_desc_sw128(smem_u32(smem + PP_OFF_V));
            uint32_t u_s = 0, u_pv = 0;   // score tiles / PV products this warp has issued
            // S_w = Q_w K^T of tile j of `it`: as soon as the warpgroup holds its previous scores in registers.
            // `k` = items of the CTA before this one (query set and its phase), `t0` = key tiles before it, `n` = its key
            // tiles, `two` = it has a second query tile.
            auto issue_s = [&](const int k, const uint32_t t0, const int n, const bool two_, const int j) -> bool {
                const uint32_t t = t0 + static_cast<uint32_t>(j);
                const int st = static_cast<int>(t % PP_NST);
                const int set = k & 1;
                const bool active = wg == 0 || two_;
                if (j == 0 && !mbar_wait(&q_full[set], (static_cast<uint32_t>(k) >> 1) & 1u, abort_flag)) return false;
                if (active && u_s > 0 && !mbar_wait(&s_free[wg], (u_s - 1u) & 1u, abort_flag)) return false;
                if (!mbar_wait(&k_full[st], (t / PP_NST) & 1u, abort_flag)) return false;
                tcgen05_fence_after();
                if (lane == 0) {
                    if (active) {
                        const uint64_t a_desc = dq0 + static_cast<uint64_t>((set * NWG + wg) * (TILE_BYTES >> 4));
                        const uint64_t b_desc = dk0 + static_cast<uint64_t>(st * (TILE_BYTES >> 4));
                        const uint32_t d_tmem = tmem_base + wg * 128;
    #pragma unroll
                        for (int kk = 0; kk < HD / 16; ++kk)
                            umma_f16_ss(d_tmem, a_desc + 2u * kk, b_desc + 2u * kk, idesc_qk, kk != 0 ? 1u : 0u);
                        umma_commit(&s_full[wg]);
                    }
                    umma_commit(&k_empty[st]);
                    if (j == n - 1) umma_commit(&q_empty[set]);
                }
                __syncwarp();
                if (active) ++u_s;
                return true;
            };
            // O_w (+)= P_w V of tile j: when the warpgroup has written P_w.
            auto issue_pv = [&](const uint32_t t0, const bool two_, const int j) -> bool {
                const uint32_t t = t0 + static_cast<uint32_t>(j);
                const int st = static_cast<int>(t % PP_NST);
                const bool active = wg == 0 || two_;
                if (active && !mbar_wait(&p_full[wg], u_pv & 1u, abort_flag)) return false;
                if (!mbar_wait(&v_full[st], (t / PP_NST) & 1u, abort_flag)) return false;
                tcgen05_fence_after();
                if (lane == 0) {
                    if (active) {
                        const uint64_t b_desc = dv0 + static_cast<uint64_t>(st * (TILE_BYTES >> 4));
                        const uint32_t d_tmem = tmem_base + C::COL_O + wg * 64;
                        const uint32_t a_tmem = tmem_base + C::COL_P + wg * 64;
                        const uint32_t acc0 = j != 0 ? 1u : 0u;
                        // O_w accumulates in TMEM over the item's key tiles (the softmax rescales it in place when it
                        // must); P_w is read from TMEM (8 columns per 16 keys), V from shared memory (2 KB per 16 keys)
    #pragma unroll
                        for (int kk = 0; kk < TK / 16; ++kk)
                            umma_f16_ts(d_tmem, a_tmem + kk * 8, b_desc + static_cast<uint64_t>(kk * (2048 >> 4)), idesc_pv,
                                        kk != 0 ? 1u : acc0);
                        umma_commit(&o_full[wg]);
                    }
                    umma_commit(&v_empty[st]);
                }
                __syncwarp();
                if (active) ++u_pv;
                return true;
            };
            bool ok = true;
            int id = id0, k = 0;
            uint32_t t0 = 0;
            int n = 0;
            bool two_ = false;
            if (id < n_items) {
                const Item it = load_item(id);
                n = it.n_tiles;
                two_ = it.two;
                ok = __all_sync(0xffffffffu, issue_s(k, t0, n, two_, 0));
            }
            while (ok && id < n_items) {
                const int id_n = id + id_step;
                int n_n = 0;
                bool two_n = false;
                if (id_n < n_items) {
                    const Item it = load_item(id_n);
                    n_n = it.n_tiles;
                    two_n = it.two;
                }
                for (int j = 0; ok && j < n; ++j) {
                    // the scores of the following tile (of this item, or the first of the next) before this tile's PV
                    if (j + 1 < n) ok = issue_s(k, t0, n, two_, j + 1);
                    else if (id_n < n_items) ok = issue_s(k + 1, t0 + static_cast<uint32_t>(n), n_n, two_n, 0);
                    if (ok) ok = issue_pv(t0, two_, j);
                    ok = __all_sync(0xffffffffu, ok);
                }
                t0 += static_cast<uint32_t>(n);
                id = id_n;
                ++k;
                n = n_n;
                two_ = two_n;
            }
            __syncwarp();
        }
    } else {
        setmaxnreg_inc<C::REGS_SOFTMAX>();
        // ------------------------------------------------------------ softmax warpgroups
        const int wg = (warp - 4) >> 2;   // warps 4..7 -> 0, 8..11 -> 1
        const int r_in_tile = ((warp & 3) << 5) + lane;          // TMEM lane = query row of the tile
        const uint32_t lane_field = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t t_s = tmem_base + lane_field + wg * 128;
        const uint32_t t_o = tmem_base + lane_field + C::COL_O + wg * 64;
        const uint32_t t_p = tmem_base + lane_field + C::COL_P + wg * 64;
        uint32_t u = 0;   // key tiles this warpgroup has been through (phase of its score / weight / output barriers)
        uint32_t t = 0;   // key tiles of the CTA so far (ring stage and phase)
        bool ok = true;
        // (only the id is carried through an item: the row of scores needs the registers; the output's coordinates are
        // decoded again when the item is done)
        for (int id = id0; ok && id < n_items; id += id_step) {
            int n_tiles;
            {
                const Item it = load_item(id);
                n_tiles = it.n_tiles;
                if (!(wg == 0 || it.two)) {
                    t += static_cast<uint32_t>(n_tiles);
                    continue;
                }
            }
            float m_run = -INFINITY, l_run = 0.f;
            for (int j = 0; j < n_tiles; ++j, ++u, ++t) {
                const int st = static_cast<int>(t % PP_NST);
                const uint32_t ph = u & 1u;
                if (!mbar_wait(&m_full[st], (t / PP_NST) & 1u, abort_flag)) { ok = false; break; }
                if (!mbar_wait(&s_full[wg], ph, abort_flag)) { ok = false; break; }
                __syncwarp();
                tcgen05_fence_after();
                // The row's 128 scores move to registers in one go and the score columns are handed back at once:
                // the next tile's QK^T runs while this tile's softmax is still at work.
                uint32_t s[TK];
#pragma unroll
                for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x32(t_s + c * 32, reinterpret_cast<uint32_t(&)[32]>(s[c * 32]));
#pragma unroll
                for (int c = 0; c < 4; ++c) tmem_ld_wait(reinterpret_cast<uint32_t(&)[32]>(s[c * 32]));
                tcgen05_fence_before();
                mbar_arrive(&s_free[wg]);
                const float* mrow = mask_s + st * TK;
                const bool plain_tile = plain_s[st] != 0u;   // warp-uniform (CTA-uniform)
                float tmx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // independent chains (latency)
                if (plain_tile) {
#pragma unroll
                    for (int g = 0; g < TK / 8; ++g) {
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                            tmx[c] = fmax3(tmx[c], __uint_as_float(s[g * 8 + c * 2]), __uint_as_float(s[g * 8 + c * 2 + 1]));
                    }
                } else {
                    // s <- score * scale + mask (log2 units; -inf drops the key): the exp pass only subtracts the maximum
                    const uint64_t sc2 = pack_f32x2(p.scale_log2, p.scale_log2);
#pragma unroll
                    for (int g = 0; g < TK / 4; ++g) {
                        const float4 mk = *reinterpret_cast<const float4*>(mrow + g * 4);
                        float v0, v1, v2, v3;
                        unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(s[g * 4 + 0]), __uint_as_float(s[g * 4 + 1])), sc2,
                                               pack_f32x2(mk.x, mk.y)), v0, v1);
                        unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(s[g * 4 + 2]), __uint_as_float(s[g * 4 + 3])), sc2,
                                               pack_f32x2(mk.z, mk.w)), v2, v3);
                        s[g * 4 + 0] = __float_as_uint(v0);
                        s[g * 4 + 1] = __float_as_uint(v1);
                        s[g * 4 + 2] = __float_as_uint(v2);
                        s[g * 4 + 3] = __float_as_uint(v3);
                        tmx[g & 1] = fmax3(tmx[g & 1], v0, v1);
                        tmx[2 + (g & 1)] = fmax3(tmx[2 + (g & 1)], v2, v3);
                    }
                }
                float tmax = fmaxf(fmaxf(tmx[0], tmx[1]), fmaxf(tmx[2], tmx[3]));
                if (plain_tile) tmax *= p.scale_log2;   // = max of the scaled scores: the scale is positive
                // Lazy reference maximum: it only moves when the tile's maximum exceeds it by more than 2^kLazyLog2
                // (weights stay <= 2^kLazyLog2, exact in half precision and harmless in the fp32 sums), so most tiles
                // leave the output accumulator in TMEM untouched.
                const bool move = tmax > m_run + kLazyLog2;
                const float m_new = move ? tmax : m_run;
                const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
                const float alpha = move ? fast_exp2(m_run - m_use) : 1.f;
                // PV of the item's previous tile must be complete: it reads the P buffer written below, and it writes
                // the accumulator a rescale would touch.  (For an item's first tile the previous item's last PV was
                // awaited before its output was read.)
                if (j > 0 && !mbar_wait(&o_full[wg], (u - 1u) & 1u, abort_flag)) { ok = false; break; }
                __syncwarp();
                if (j > 0 && __any_sync(0xffffffffu, move)) {
                    tcgen05_fence_after();
#pragma unroll
                    for (int cc = 0; cc < HD / 32; ++cc) {
                        uint32_t ro[32];
                        tmem_ld_32x32b_x32(t_o + cc * 32, ro);
                        tmem_ld_wait(ro);
#pragma unroll
                        for (int e = 0; e < 32; ++e) ro[e] = __float_as_uint(__uint_as_float(ro[e]) * alpha);
                        tmem_st_32x32b_x32(t_o + cc * 32, ro);
                    }
                }
                // Phase offset.  A scheduler's exp unit is saturated only while both of its softmax warps are in their exp
                // pass (8.9 cycles per score per scheduler), runs at ~70 % with one (11.6) and idles with none; started
                // together the two warpgroups stay in lockstep: both in the exp pass, then both out of it.  So warpgroup
                // 1 begins an item's first exp pass only when warpgroup 0 has finished its own (warpgroup 0 takes part in
                // every item, so its tile count is the CTA's, `t`); for the next tiles one's exp pass covers the other's
                // loads, maximum and hand-offs.  (The offset decays over ~6 tiles; renewing it every tile, every second or
                // every fourth tile, or holding it with a mutual rule, all measured slower than letting it decay within
                // an item; set only once per CTA the persistent kernel ran 10-13 % slower on long sequences.)
                // (A parity wait can only name the phase in progress or the one before it, and warpgroup 0 may be further
                // ahead than that: its own count of finished tiles is looked at first, the wait is tried a bounded number
                // of times, and nothing depends on its outcome but the timing.)
                if (NWG == 2 && wg == 1 && j == 0) {
                    for (int spin = 0; spin < 64 && *wg0_tiles <= t; ++spin)
                        if (mbar_try_wait(&p_full[0], t & 1u)) break;
                }
                // exp pass: P goes to tensor memory as the A operand of the PV UMMA, two consecutive keys per 32-bit
                // column, 32 keys at a time into columns [16c, 16c + 16) of the warpgroup's P region
                const uint64_t mul2 = plain_tile ? pack_f32x2(p.scale_log2, p.scale_log2) : pack_f32x2(1.f, 1.f);
                const uint64_t neg2 = pack_f32x2(-m_use, -m_use);
                uint64_t ps2[2] = {0ull, 0ull};   // 2 x 2 partial sums
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t pk[16];
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        const int i = c * 32 + e * 2;
                        float x0, x1;
                        unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(s[i]), __uint_as_float(s[i + 1])), mul2, neg2), x0, x1);
                        x0 = fast_exp2(x0);
                        x1 = fast_exp2(x1);
                        ps2[e & 1] = add_f32x2(ps2[e & 1], pack_f32x2(x0, x1));
                        pk[e] = pack2t<DT>(x0, x1);
                    }
                    tmem_st_32x32b_x16(t_p + c * 16, pk);
                }
                float a0, a1, a2, a3;
                unpack_f32x2(ps2[0], a0, a1);
                unpack_f32x2(ps2[1], a2, a3);
                l_run = l_run * alpha + ((a0 + a1) + (a2 + a3));
                m_run = m_new;
                tmem_st_wait();               // P (and a rescaled O) have reached tensor memory
                tcgen05_fence_before();
                if (NWG == 2 && wg == 0 && r_in_tile == 0) *wg0_tiles = t + 1u;   // before this thread's arrival: see above
                mbar_arrive(&p_full[wg]);
            }
            if (!ok) break;
            // the item's last PV, then its output: normalised and stored from registers.  The accumulator columns are
            // free for the next item as soon as they are in registers; its first PV is issued only after this
            // warpgroup's next p_full arrivals, which follow these loads in program order.
            if (n_tiles > 0 && !mbar_wait(&o_full[wg], (u - 1u) & 1u, abort_flag)) { ok = false; break; }
            __syncwarp();
            tcgen05_fence_after();
            const Item it = load_item(id);
            const int q = it.q0 + wg * TQ + r_in_tile;
            const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
            uint16_t* dst =
                reinterpret_cast<uint16_t*>(p.out) + (static_cast<long long>(it.b) * p.S + q) * p.ldo + it.head * HD;
#pragma unroll
            for (int c = 0; c < HD / 32; ++c) {
                uint32_t r[32];
                tmem_ld_32x32b_x32(t_o + c * 32, r);
                tmem_ld_wait(r);
                if (q < p.S) {
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        uint4 qv;
                        qv.x = pack2t<DT>(__uint_as_float(r[g * 8 + 0]) * inv, __uint_as_float(r[g * 8 + 1]) * inv);
                        qv.y = pack2t<DT>(__uint_as_float(r[g * 8 + 2]) * inv, __uint_as_float(r[g * 8 + 3]) * inv);
                        qv.z = pack2t<DT>(__uint_as_float(r[g * 8 + 4]) * inv, __uint_as_float(r[g * 8 + 5]) * inv);
                        qv.w = pack2t<DT>(__uint_as_float(r[g * 8 + 6]) * inv, __uint_as_float(r[g * 8 + 7]) * inv);
                        *reinterpret_cast<uint4*>(dst + c * 32 + g * 8) = qv;
                    }
                }
            }
            tcgen05_fence_before();
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, PP_TMEM_COLS);
    }
    if (tid == 0 && *abort_flag != 0 && p.status != nullptr) atomicOr(p.status, 2u);
}

// ---------------------------------------------------------------------------------------------------------------
// Sequences of at most 128 tokens (the benchmark's S = 128): one key tile per (sequence, head), so no running
// rescale.  An item is tiny (4.2 MFLOP on 48 KB of operands) and its steps depend on each other (loads -> QK^T ->
// max sweep -> exp sweep -> PV -> output), so throughput comes from overlapping items: persistent CTAs of 128 threads,
// four per SM (50 KB of shared memory and 128 TMEM columns each), walk the (sequence, head) items with a grid stride.
//   * TMEM columns: S in [0, 32*chunks); P (half precision, the A operand of the PV UMMA) is written over S columns
//     [0, 64) chunk by chunk — a thread has read the scores a P chunk replaces before it writes it; O in [64, 128),
//     scores that are dead by then;
//   * only ceil(kv_len / 32) 32-key chunks are computed: QK^T runs with N = 32*chunks, the softmax reads that many
//     chunks, PV runs 2*chunks k-steps — padded tails of short sequences cost nothing;
//   * operand tiles are handed to the next item as they die: Q and K when the scores are complete (the next item's Q
//     and K then travel during this item's softmax, PV and output: 1.2 % of a BERT-base step at 1024 sequences against
//     issuing them after PV), V when the output tile, which is staged (swizzled) in the V tile and leaves through one
//     TMA store clipped at row S, has been read by that store.  (Storing the output straight from registers — a thread
//     owns a query row, 128 contiguous bytes per head — frees V earlier but measured 35 % slower: 32 rows per store
//     instruction are 32 half-written sectors.)
constexpr int S1_OFF_MASK = 3 * TILE_BYTES;
constexpr int S1_OFF_BAR = S1_OFF_MASK + TK * 4;
constexpr int S1_SMEM = S1_OFF_BAR + 64;
constexpr int S1_TMEM_COLS = 128;
constexpr int S1_CTAS_PER_SM = 4;

template <int DT>
__global__ void __launch_bounds__(kAttnThreads, S1_CTAS_PER_SM)
attention_single_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                        const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                        const AttnParams p, const int num_items) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S1_OFF_BAR);
    uint64_t* bar_qk = bars + 0;
    uint64_t* bar_v = bars + 1;
    uint64_t* bar_s = bars + 2;
    uint64_t* bar_o = bars + 3;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    float* mask_s = reinterpret_cast<float*>(smem + S1_OFF_MASK);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;

    if ((smem_u32(smem) & 1023u) != 0) {
        if (tid == 0 && p.status) atomicOr(p.status, 4u);
        return;
    }
    if (tid == 0) {
        mbar_init(bar_qk, 1);
        mbar_init(bar_v, 1);
        mbar_init(bar_s, 1);
        mbar_init(bar_o, 1);
        *abort_flag = 0;
        mbar_fence_init();
        prefetch_tmap(&tm_q);
        prefetch_tmap(&tm_k);
        prefetch_tmap(&tm_v);
        prefetch_tmap(&tm_o);
    }
    if (warp == 0) {
        tmem_alloc(tmem_slot, S1_TMEM_COLS);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t lane_field = static_cast<uint32_t>(warp * 32) << 16;
    const uint32_t t_row = tmem_base + lane_field;   // this thread's TMEM lane (= query row), column 0
    pdl_launch_dependents();
    pdl_wait();   // qkv and kv_len come from earlier kernels; the output may still be read by one

    auto load_qk = [&](int item) {   // tid 0 only
        const int bb = item / p.heads, hh = item % p.heads;
        mbar_expect_tx(bar_qk, 2 * TILE_BYTES);
        tma_load_3d(smem + OFF_Q, &tm_q, bar_qk, hh * HD, 0, bb);
        tma_load_3d(smem + OFF_K, &tm_k, bar_qk, hh * HD, 0, bb);
    };
    auto load_v = [&](int item) {    // tid 0 only
        const int bb = item / p.heads, hh = item % p.heads;
        mbar_expect_tx(bar_v, TILE_BYTES);
        tma_load_3d(smem + OFF_V, &tm_v, bar_v, hh * HD, 0, bb);
    };
    // UMMA descriptors of the three tiles (tid 0 issues): built once
    const uint64_t desc_q = make_smem_desc_sw128(smem_u32(smem + OFF_Q));
    const uint64_t desc_k = make_smem_desc_sw128(smem_u32(smem + OFF_K));
    const uint64_t desc_v = make_smem_desc_sw128(smem_u32(smem + OFF_V));
    const uint32_t idesc_qk_base = p.idesc_qk & ~(0x3Fu << 17);
    const uint32_t idesc_pv = p.idesc_pv;
    if (tid == 0 && static_cast<int>(blockIdx.x) < num_items) {
        load_qk(blockIdx.x);
        load_v(blockIdx.x);
    }

    bool ok = true;
    uint32_t it = 0;
    for (int item = blockIdx.x; item < num_items; item += gridDim.x, ++it) {
        const uint32_t ph = it & 1u;
        const int b = item / p.heads;
        const int head = item % p.heads;

        int kv_eff = p.S;
        bool additive_only = (p.mask_add == nullptr);
        if (p.kv_len != nullptr) {
            const int kl = p.kv_len[b];
            if (kl <= 0) additive_only = true;
            else kv_eff = kl < p.S ? kl : p.S;
        }
        const int n_chunks = (kv_eff + 31) >> 5;   // 1..4
        {
            float m = -INFINITY;
            if (tid < p.S) {
                const float a = p.mask_add ? p.mask_add[static_cast<long long>(b) * p.S + tid] : 0.f;
                if (additive_only || a > p.mask_below) m = a * 1.4426950408889634f;
            }
            mask_s[tid] = m;   // the previous item's softmax finished before its closing __syncthreads
        }
        // "Plain" item: every key of the chunks that are computed is valid with additive mask 0 (the common case: a
        // full-length sequence, or all tiles below a ragged sequence's end).  The softmax then needs no mask reads and
        // can take the row maximum of the raw scores (the scale is positive).
        const bool plain = __syncthreads_and(tid >= n_chunks * 32 || mask_s[tid] == 0.f) != 0 && p.scale_log2 > 0.f;

        if (tid == 0) {
            if (mbar_wait(bar_qk, ph, abort_flag)) {
                tcgen05_fence_after();
                const uint32_t idesc = idesc_qk_base | (static_cast<uint32_t>(n_chunks * 4) << 17);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k)
                    umma_f16_ss(tmem_base, desc_q + 2u * k, desc_k + 2u * k, idesc, k != 0 ? 1u : 0u);
                umma_commit(bar_s);
            }
        }
        if (!mbar_wait(bar_s, ph, abort_flag)) { ok = false; break; }
        const int next = item + gridDim.x;
#if B200_ATTN_EARLY_QK
        // The scores are complete, so Q and K are dead: the next item's Q and K start travelling now and have the
        // whole softmax, PV and output of this item to arrive.
        if (tid == 0 && next < num_items) load_qk(next);
#endif
        __syncwarp();
        tcgen05_fence_after();
        float l_sum = 0.f;
        {
            float tmx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // independent chains (latency)
#pragma unroll 1
            for (int c = 0; c < n_chunks; ++c) {
                uint32_t r[32];
                tmem_ld_32x32b_x32(t_row + c * 32, r);
                tmem_ld_wait(r);
                if (plain) {
#pragma unroll
                    for (int g = 0; g < 8; ++g) {
                        tmx[0] = fmaxf(tmx[0], __uint_as_float(r[g * 4 + 0]));
                        tmx[1] = fmaxf(tmx[1], __uint_as_float(r[g * 4 + 1]));
                        tmx[2] = fmaxf(tmx[2], __uint_as_float(r[g * 4 + 2]));
                        tmx[3] = fmaxf(tmx[3], __uint_as_float(r[g * 4 + 3]));
                    }
                } else {
#pragma unroll
                    for (int g = 0; g < 8; ++g) {
                        const float4 mk = *reinterpret_cast<const float4*>(mask_s + c * 32 + g * 4);
                        tmx[0] = fmaxf(tmx[0], fmaf(__uint_as_float(r[g * 4 + 0]), p.scale_log2, mk.x));
                        tmx[1] = fmaxf(tmx[1], fmaf(__uint_as_float(r[g * 4 + 1]), p.scale_log2, mk.y));
                        tmx[2] = fmaxf(tmx[2], fmaf(__uint_as_float(r[g * 4 + 2]), p.scale_log2, mk.z));
                        tmx[3] = fmaxf(tmx[3], fmaf(__uint_as_float(r[g * 4 + 3]), p.scale_log2, mk.w));
                    }
                }
            }
            float tmax = fmaxf(fmaxf(tmx[0], tmx[1]), fmaxf(tmx[2], tmx[3]));
            if (plain) tmax *= p.scale_log2;   // fma(s, scale, 0) = s * scale exactly, and the scale is positive
            const float m_use = (tmax == -INFINITY) ? 0.f : tmax;
            const float neg_m = -m_use;
#pragma unroll 1
            for (int c = 0; c < n_chunks; ++c) {
                uint32_t r[32];
                tmem_ld_32x32b_x32(t_row + c * 32, r);
                tmem_ld_wait(r);
                float pv[32];
                if (plain) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) pv[i] = fast_exp2(fmaf(__uint_as_float(r[i]), p.scale_log2, neg_m));
                } else {
#pragma unroll
                    for (int g = 0; g < 8; ++g) {
                        const float4 mk = *reinterpret_cast<const float4*>(mask_s + c * 32 + g * 4);
                        pv[g * 4 + 0] = fast_exp2(fmaf(__uint_as_float(r[g * 4 + 0]), p.scale_log2, mk.x - m_use));
                        pv[g * 4 + 1] = fast_exp2(fmaf(__uint_as_float(r[g * 4 + 1]), p.scale_log2, mk.y - m_use));
                        pv[g * 4 + 2] = fast_exp2(fmaf(__uint_as_float(r[g * 4 + 2]), p.scale_log2, mk.z - m_use));
                        pv[g * 4 + 3] = fast_exp2(fmaf(__uint_as_float(r[g * 4 + 3]), p.scale_log2, mk.w - m_use));
                    }
                }
                {
                    float ps[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        ps[0] += pv[i];
                        ps[1] += pv[i + 1];
                        ps[2] += pv[i + 2];
                        ps[3] += pv[i + 3];
                    }
                    l_sum += (ps[0] + ps[1]) + (ps[2] + ps[3]);
                }
                // P chunk c -> TMEM columns [16c, 16c + 16): two keys per 32-bit column.  Those columns held the
                // scores of keys 32*(c/2) .. which this thread consumed above or in an earlier turn of this loop.
                uint32_t pk[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) pk[e] = pack2t<DT>(pv[2 * e], pv[2 * e + 1]);
                tmem_st_32x32b_x16(t_row + c * 16, pk);
            }
        }
        tmem_st_wait();
        tcgen05_fence_before();
        __syncthreads();

        if (tid == 0) {
            tcgen05_fence_after();
            if (mbar_wait(bar_v, ph, abort_flag)) {
                tcgen05_fence_after();
                const int ksteps = n_chunks * 2;
                for (int k = 0; k < ksteps; ++k)
                    umma_f16_ts(tmem_base + 64, tmem_base + k * 8, desc_v + static_cast<uint64_t>(k * (2048 >> 4)),
                                idesc_pv, k != 0 ? 1u : 0u);
                umma_commit(bar_o);
            }
        }
        if (!mbar_wait(bar_o, ph, abort_flag)) { ok = false; break; }
#if !B200_ATTN_EARLY_QK
        // Q, K, V are dead now: the next item's Q and K start travelling while this item's output is written
        if (tid == 0 && next < num_items) load_qk(next);
#endif
        __syncwarp();
        tcgen05_fence_after();
        {
            const float inv = l_sum > 0.f ? 1.0f / l_sum : 0.f;
            uint8_t* orow = smem + OFF_V + tid * 128;   // output tile staged in the V tile
#pragma unroll
            for (int c = 0; c < HD / 32; ++c) {
                uint32_t r[32];
                tmem_ld_32x32b_x32(t_row + 64 + c * 32, r);
                tmem_ld_wait(r);
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    uint4 qv;
                    qv.x = pack2t<DT>(__uint_as_float(r[g * 8 + 0]) * inv, __uint_as_float(r[g * 8 + 1]) * inv);
                    qv.y = pack2t<DT>(__uint_as_float(r[g * 8 + 2]) * inv, __uint_as_float(r[g * 8 + 3]) * inv);
                    qv.z = pack2t<DT>(__uint_as_float(r[g * 8 + 4]) * inv, __uint_as_float(r[g * 8 + 5]) * inv);
                    qv.w = pack2t<DT>(__uint_as_float(r[g * 8 + 6]) * inv, __uint_as_float(r[g * 8 + 7]) * inv);
                    const int chunk = (c * 4 + g) ^ (tid & 7);
                    *reinterpret_cast<uint4*>(orow + chunk * 16) = qv;
                }
            }
            fence_async_proxy_shared();
        }
        tcgen05_fence_before();
        __syncthreads();   // also orders this item's TMEM reads before the next item's UMMAs
        if (tid == 0) {
            asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                         ::"l"(reinterpret_cast<uint64_t>(&tm_o)), "r"(smem_u32(smem + OFF_V)), "r"(head * HD), "r"(0),
                           "r"(b)
                         : "memory");
            tma_store_commit();
            if (next < num_items) {
                tma_store_wait_read<0>();   // the store has read the staged tile: V may be overwritten
                load_v(next);
            }
        }
    }
    if (tid == 0) {
        if (ok) tma_store_wait_read<0>();
        else for (int i = 0; i < 64; ++i) nanosleep(10000);   // let copies in flight land
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 0) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, S1_TMEM_COLS);
    }
    if (tid == 0 && *abort_flag != 0 && p.status != nullptr) atomicOr(p.status, 2u);
}

// Dynamic shared-memory limits of the kernel instances, once per device (first launch on it).
bool set_attention_attributes(int dev) {
    static PerDeviceOnce once;
    return once.ensure(dev, []() {
        const bool ok =
            cudaFuncSetAttribute(attention_single_kernel<B200_F16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 S1_SMEM) == cudaSuccess &&
            cudaFuncSetAttribute(attention_single_kernel<B200_BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 S1_SMEM) == cudaSuccess &&
            cudaFuncSetAttribute(attention_pingpong_kernel<B200_F16, PP_NWG>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 PPCfg<PP_NWG, 1>::SMEM) == cudaSuccess &&
            cudaFuncSetAttribute(attention_pingpong_kernel<B200_BF16, PP_NWG>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 PPCfg<PP_NWG, 1>::SMEM) == cudaSuccess &&
            cudaFuncSetAttribute(attention_pingpong_persistent_kernel<B200_F16, PP_NWG>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, PPCfg<PP_NWG, 2>::SMEM) == cudaSuccess &&
            cudaFuncSetAttribute(attention_pingpong_persistent_kernel<B200_BF16, PP_NWG>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, PPCfg<PP_NWG, 2>::SMEM) == cudaSuccess;
        if (!ok) cudaGetLastError();
        return ok;
    });
}

// Launch of the long-sequence attention (S > 128).  Items of up to 8 key tiles (S <= 1024) go to the persistent kernel:
// one CTA per resident slot, nothing drained between items (6-14 % faster at S = 256 ... 1024).  Longer items run one
// per CTA: there the persistent form measured 5-8 % slower (S = 2048, 4096), with a fixed deal of items to CTAs as
// well as with one item per CTA.  `with_attributes` = launch with the programmatic-dependent-launch attribute.
int launch_pingpong(AttnParams& p, int dtype, long long S, int heads, long long B, int dev, cudaStream_t stream,
                    const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, bool with_attributes) {
    const int n_qb = static_cast<int>((S + PP_NWG * TQ - 1) / (PP_NWG * TQ));
    p.n_qb = n_qb;
    p.n_items = static_cast<long long>(n_qb) * heads * B;
    if (S <= 8 * TK) {
        if (p.n_items > 0x7fff0000ll) return B200_ERR_UNSUPPORTED;   // item ids are 32-bit in the kernel
        int sms = 0;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        const long long slots = static_cast<long long>(sms > 0 ? sms : 1) * PPCfg<PP_NWG, 2>::CTAS_PER_SM;
        const dim3 grid(static_cast<unsigned>(p.n_items < slots ? p.n_items : slots));
        const dim3 block(PPCfg<PP_NWG, 2>::THREADS);
        constexpr size_t smem = PPCfg<PP_NWG, 2>::SMEM;
        if (with_attributes) {
            if (dtype == B200_F16)
                launch_kernel(attention_pingpong_persistent_kernel<B200_F16, PP_NWG>, grid, block, smem, stream, tq, tk, tv, p);
            else
                launch_kernel(attention_pingpong_persistent_kernel<B200_BF16, PP_NWG>, grid, block, smem, stream, tq, tk, tv, p);
        } else if (dtype == B200_F16) {
            attention_pingpong_persistent_kernel<B200_F16, PP_NWG><<<grid, block, smem, stream>>>(tq, tk, tv, p);
        } else {
            attention_pingpong_persistent_kernel<B200_BF16, PP_NWG><<<grid, block, smem, stream>>>(tq, tk, tv, p);
        }
        return B200_OK;
    }
    const dim3 grid(static_cast<unsigned>(n_qb), static_cast<unsigned>(heads), static_cast<unsigned>(B));
    const dim3 block(PPCfg<PP_NWG, 1>::THREADS);
    constexpr size_t smem = PPCfg<PP_NWG, 1>::SMEM;
    if (with_attributes) {
        if (dtype == B200_F16)
            launch_kernel(attention_pingpong_kernel<B200_F16, PP_NWG>, grid, block, smem, stream, tq, tk, tv, p);
        else
            launch_kernel(attention_pingpong_kernel<B200_BF16, PP_NWG>, grid, block, smem, stream, tq, tk, tv, p);
    } else if (dtype == B200_F16) {
        attention_pingpong_kernel<B200_F16, PP_NWG><<<grid, block, smem, stream>>>(tq, tk, tv, p);
    } else {
        attention_pingpong_kernel<B200_BF16, PP_NWG><<<grid, block, smem, stream>>>(tq, tk, tv, p);
    }
    return B200_OK;
}

}  // namespace
}  // namespace b200

extern "C" int b200_attention_fwd(const B200AttentionDesc* d, b200_stream_t stream_) {
    using namespace b200;
    if (!d || !d->q || !d->k || !d->v || !d->out) return B200_ERR_PARAM;
    if (d->B <= 0 || d->S <= 0 || d->heads <= 0) return B200_ERR_PARAM;
    if (d->head_dim != HD) return B200_ERR_UNSUPPORTED;
    if (!is_half_dtype(d->dtype)) return B200_ERR_PARAM;
    const int64_t width = static_cast<int64_t>(d->heads) * HD;
    if ((d->ldq % 8) || (d->ldk % 8) || (d->ldv % 8) || (d->ldo % 8)) return B200_ERR_PARAM;
    if (d->ldq < width || d->ldk < width || d->ldv < width || d->ldo < width) return B200_ERR_PARAM;
    if (!aligned16(d->q) || !aligned16(d->k) || !aligned16(d->v) || !aligned16(d->out)) return B200_ERR_PARAM;
    if (d->B > 65535 || d->heads > 65535 || d->S > (1 << 24)) return B200_ERR_UNSUPPORTED;
    int dev = 0, major = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return B200_ERR_LAUNCH;
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (major != 10) return B200_ERR_NOT_SM100;

    const uint64_t dims[3] = {static_cast<uint64_t>(width), static_cast<uint64_t>(d->S), static_cast<uint64_t>(d->B)};
    const uint32_t box[3] = {HD, 128, 1};
    const uint64_t sq[2] = {static_cast<uint64_t>(d->ldq) * 2, static_cast<uint64_t>(d->ldq) * 2 * d->S};
    const uint64_t sk[2] = {static_cast<uint64_t>(d->ldk) * 2, static_cast<uint64_t>(d->ldk) * 2 * d->S};
    const uint64_t sv[2] = {static_cast<uint64_t>(d->ldv) * 2, static_cast<uint64_t>(d->ldv) * 2 * d->S};
    CUtensorMap tq, tk, tv;
    if (!get_tensor_map(&tq, d->q, 3, dims, sq, box) || !get_tensor_map(&tk, d->k, 3, dims, sk, box) ||
        !get_tensor_map(&tv, d->v, 3, dims, sv, box))
        return B200_ERR_DRIVER;

    AttnParams p;
    p.mask_add = d->mask_add;
    p.kv_len = d->kv_len;
    p.out = d->out;
    p.S = static_cast<int>(d->S);
    p.heads = d->heads;
    p.ldo = d->ldo;
    p.dtype = d->dtype;
    p.scale_log2 = d->scale * 1.4426950408889634f;
    p.mask_below = d->mask_exclude_below;
    const int fmt = d->dtype == B200_BF16 ? 1 : 0;
    p.idesc_qk = make_idesc_f16(128, TK, fmt, 0, 0);
    p.idesc_pv = make_idesc_f16(128, HD, fmt, 0, 1);  // B (= V) is MN-major
    p.status = device_status_ptr();

    if (d->S <= 128) {
        const uint64_t so[2] = {static_cast<uint64_t>(d->ldo) * 2, static_cast<uint64_t>(d->ldo) * 2 * d->S};
        CUtensorMap to;
        if (!get_tensor_map(&to, d->out, 3, dims, so, box)) return B200_ERR_DRIVER;
        if (!set_attention_attributes(dev)) return B200_ERR_LAUNCH;
        const long long items = static_cast<long long>(d->heads) * d->B;
        if (items > 0x7fffffff) return B200_ERR_UNSUPPORTED;
        int sms = 0;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        const long long grid1 = items < 1ll * S1_CTAS_PER_SM * sms ? items : 1ll * S1_CTAS_PER_SM * sms;
        const cudaStream_t st = static_cast<cudaStream_t>(stream_);
        if (d->dtype == B200_F16)
            launch_kernel(attention_single_kernel<B200_F16>, dim3(static_cast<unsigned>(grid1)), dim3(kAttnThreads),
                          S1_SMEM, st, tq, tk, tv, to, p, static_cast<int>(items));
        else
            launch_kernel(attention_single_kernel<B200_BF16>, dim3(static_cast<unsigned>(grid1)), dim3(kAttnThreads),
                          S1_SMEM, st, tq, tk, tv, to, p, static_cast<int>(items));
        count_launch();
        return check_launch();
    }

    if (!set_attention_attributes(dev)) return B200_ERR_LAUNCH;
    const int rc = launch_pingpong(p, d->dtype, d->S, d->heads, d->B, dev, static_cast<cudaStream_t>(stream_), tq, tk, tv, true);
    if (rc != B200_OK) return rc;
    count_launch();
    return check_launch();
}

// ---------------------------------------------------------------------------------------------------------------
// The allocation-free variant of masked attention (see include/tnn_b200.h).  Its only scratch, the kv_len array,
// is this file-scope device array.  In host code the name below is merely a handle for the symbol — not a device
// address — so the address is looked up once per device with cudaGetSymbolAddress and that pointer is what the
// kernels receive.
static __device__ __align__(256) int g_static_kv_len[B200_STATIC_MAX_BATCH];

namespace {
int* g_static_kv_len_ptr[b200::kMaxDevices] = {nullptr};   // per device, filled by the first call on that device
b200::PerDeviceOnce g_static_once;                          // guards that first call against a second host thread
}

extern "C" int b200_attention_masked_fwd_static(const B200AttentionDesc* d, b200_stream_t stream_) {
    using namespace b200;
    if (!d || !d->q || !d->k || !d->v || !d->out || !d->mask_add) return B200_ERR_PARAM;
    if (d->B <= 0 || d->S <= 0 || d->heads <= 0) return B200_ERR_PARAM;
    if (d->B > B200_STATIC_MAX_BATCH) return B200_ERR_STATIC_LIMIT;
    if (d->head_dim != HD) return B200_ERR_UNSUPPORTED;
    if (!is_half_dtype(d->dtype)) return B200_ERR_PARAM;
    const int64_t width = static_cast<int64_t>(d->heads) * HD;
    if ((d->ldq % 8) || (d->ldk % 8) || (d->ldv % 8) || (d->ldo % 8)) return B200_ERR_PARAM;
    if (d->ldq < width || d->ldk < width || d->ldv < width || d->ldo < width) return B200_ERR_PARAM;
    if (!aligned16(d->q) || !aligned16(d->k) || !aligned16(d->v) || !aligned16(d->out)) return B200_ERR_PARAM;
    if (d->heads > 65535 || d->S > (1 << 24)) return B200_ERR_UNSUPPORTED;
    int dev = 0, major = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return B200_ERR_LAUNCH;
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (major != 10) return B200_ERR_NOT_SM100;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);

    // One-time set-up on this device (current device = the one the launches below go to): the scratch array's device
    // address and the kernels' shared-memory attribute.  Two host threads making their first call at once are
    // serialised here; this takes a host mutex, no memory is allocated.
    if (!g_static_once.ensure(dev, [dev]() {
            int* ptr = nullptr;
            if (cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_kv_len) != cudaSuccess || ptr == nullptr) {
                cudaGetLastError();
                return false;
            }
            g_static_kv_len_ptr[dev] = ptr;
            return set_attention_attributes(dev);
        }))
        return B200_ERR_LAUNCH;
    int* kv_len = g_static_kv_len_ptr[dev];

    // kv_len of this call's mask into the static scratch (every entry that is read below is written here first)
    int rc = b200_mask_to_kv_len(d->mask_add, d->B, d->S, d->mask_exclude_below, kv_len, stream_);
    if (rc != B200_OK) return rc;

    // Tensor maps on the stack: nothing is cached, nothing allocated.
    const uint64_t dims[3] = {static_cast<uint64_t>(width), static_cast<uint64_t>(d->S), static_cast<uint64_t>(d->B)};
    const uint32_t box[3] = {HD, 128, 1};
    const uint64_t sq[2] = {static_cast<uint64_t>(d->ldq) * 2, static_cast<uint64_t>(d->ldq) * 2 * d->S};
    const uint64_t sk[2] = {static_cast<uint64_t>(d->ldk) * 2, static_cast<uint64_t>(d->ldk) * 2 * d->S};
    const uint64_t sv[2] = {static_cast<uint64_t>(d->ldv) * 2, static_cast<uint64_t>(d->ldv) * 2 * d->S};
    const uint64_t so[2] = {static_cast<uint64_t>(d->ldo) * 2, static_cast<uint64_t>(d->ldo) * 2 * d->S};
    CUtensorMap tq, tk, tv, to;
    if (!encode_tensor_map(&tq, d->q, 3, dims, sq, box) || !encode_tensor_map(&tk, d->k, 3, dims, sk, box) ||
        !encode_tensor_map(&tv, d->v, 3, dims, sv, box) || !encode_tensor_map(&to, d->out, 3, dims, so, box))
        return B200_ERR_DRIVER;

    AttnParams p;
    p.mask_add = d->mask_add;
    p.kv_len = kv_len;
    p.out = d->out;
    p.S = static_cast<int>(d->S);
    p.heads = d->heads;
    p.ldo = d->ldo;
    p.dtype = d->dtype;
    p.scale_log2 = d->scale * 1.4426950408889634f;
    p.mask_below = d->mask_exclude_below;
    const int fmt = d->dtype == B200_BF16 ? 1 : 0;
    p.idesc_qk = make_idesc_f16(128, TK, fmt, 0, 0);
    p.idesc_pv = make_idesc_f16(128, HD, fmt, 0, 1);
    p.status = device_status_ptr();

    if (d->S <= 128) {
        const long long items = static_cast<long long>(d->heads) * d->B;
        int sms = 0;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        const long long grid1 = items < 1ll * S1_CTAS_PER_SM * sms ? items : 1ll * S1_CTAS_PER_SM * sms;
        if (d->dtype == B200_F16)
            attention_single_kernel<B200_F16><<<static_cast<unsigned>(grid1), kAttnThreads, S1_SMEM, stream>>>(
                tq, tk, tv, to, p, static_cast<int>(items));
        else
            attention_single_kernel<B200_BF16><<<static_cast<unsigned>(grid1), kAttnThreads, S1_SMEM, stream>>>(
                tq, tk, tv, to, p, static_cast<int>(items));
    } else {
        const int rc = launch_pingpong(p, d->dtype, d->S, d->heads, d->B, dev, stream, tq, tk, tv, false);
        if (rc != B200_OK) return rc;
    }
    count_launch();
    return check_launch();
}
