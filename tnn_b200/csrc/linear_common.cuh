// Pieces shared by the two GEMM kernels (single-CTA tiles in linear.cu, CTA-pair tiles in linear_pair.cu): launch
// parameters, the erf-GELU evaluation and the per-tile epilogue (TMEM -> registers -> bias / GELU / residual -> global).
#pragma once
#include "common.cuh"
#include "ptx.cuh"

namespace b200 {
namespace lin {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kEpiWarps = 8;
constexpr int kThreads = 64 + kEpiWarps * 32;

struct LinearParams {
    const float* bias;
    const void* residual;
    void* y;
    int M, N, K;
    long long ldr, ldy;
    int dtype, out_dtype, epilogue;
    int num_n_tiles, num_tiles, num_k_blocks;
    uint32_t idesc;
    unsigned int* status;
    // LayerNorm folding (see B200LinearDesc): all null when off
    float* out_stats;
    const float* ln_in_stats;
    const float* ln_c1;
    const float* ln_c2;
    const float* res_ln_stats;
    const float* res_ln_gamma;
    const float* res_ln_beta;
    float ln_eps;
    int k_slots, n_slots;   // ceil(K/32), ceil(N/32)
};


// erf-form GELU, 0.5 x (1 + erf(x / sqrt 2)) = x * Phi(x), as the reference's CPU accs compute it, evaluated as
// 0.5 x (1 + tanh(x (a + b x^2 + c x^4))) with a, b, c fitted to the erf form (max abs deviation of the formula
// 2.5e-5 over all x; the reference's own vector path deviates from erf by ~1e-7) and the hardware tanh.approx.f32
// (relative error <= 2^-11, i.e. at most one half-precision ulp of the result, which is rounded to half precision
// anyway).  x^2 is clamped at 36, where tanh has saturated, so the negative x^4 term cannot turn the argument around.
// Cost: 1 MUFU + 7 FMA-pipe instructions instead of erff's ~30; with erff the epilogue of the 768 -> 3072 GEMM was
// MUFU/issue bound and exposed.
__device__ __forceinline__ float gelu_erf(float x) {
    const float x2 = fminf(x * x, 36.0f);
    const float poly = fmaf(x2, fmaf(x2, -3.51516788e-4f, 3.70056460e-2f), 7.97507884e-1f);
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(x * poly));
    const float h = 0.5f * x;
    return fmaf(h, t, h);
}

// Two values at once on the packed fp32 pipe (one issue slot per pair for every multiply / add / fma): the same
// operations with the same roundings as gelu_erf, so the results are identical bit for bit.  The epilogue of the
// 768-deep GEMMs is issue-bound (it has to finish within the next tile's mainloop), which is what this halves.
__device__ __forceinline__ void gelu_erf_x2(float& a, float& b) {
    const uint64_t x = pack_f32x2(a, b);
    float qa, qb;
    unpack_f32x2(mul_f32x2(x, x), qa, qb);
    const uint64_t x2 = pack_f32x2(fminf(qa, 36.0f), fminf(qb, 36.0f));
    const uint64_t poly = fma_f32x2(x2, fma_f32x2(x2, pack_f32x2(-3.51516788e-4f, -3.51516788e-4f),
                                                  pack_f32x2(3.70056460e-2f, 3.70056460e-2f)),
                                    pack_f32x2(7.97507884e-1f, 7.97507884e-1f));
    float ta, tb;
    unpack_f32x2(mul_f32x2(x, poly), ta, tb);
    asm("tanh.approx.f32 %0, %1;" : "=f"(ta) : "f"(ta));
    asm("tanh.approx.f32 %0, %1;" : "=f"(tb) : "f"(tb));
    const uint64_t h = mul_f32x2(x, pack_f32x2(0.5f, 0.5f));
    unpack_f32x2(fma_f32x2(h, pack_f32x2(ta, tb), h), a, b);
}

// Stage one warp's per-column vectors (COLS floats each, starting at column n_first) in its private shared-memory
// strips: strip 0 = bias (or c2 when the input LayerNorm is folded), 1 = c1, 2 = gamma, 3 = beta of a folded residual
// LayerNorm.  Columns at or beyond N read as 0, so that they contribute nothing anywhere.
template <bool FOLD>
__device__ __forceinline__ void stage_vectors(const LinearParams& p, float* vec_w, int n_first, int cols, int lane) {
    __syncwarp();
    const float* s0 = (FOLD && p.ln_in_stats) ? p.ln_c2 : p.bias;
    for (int i = lane; i < cols; i += 32) {
        const int n = n_first + i;
        const bool in = n < p.N;
        vec_w[i] = (s0 != nullptr && in) ? __ldg(s0 + n) : 0.f;
        if (FOLD && p.ln_in_stats) vec_w[cols + i] = in ? __ldg(p.ln_c1 + n) : 0.f;
        if (FOLD && p.res_ln_stats) {
            vec_w[2 * cols + i] = in ? __ldg(p.res_ln_gamma + n) : 0.f;
            vec_w[3 * cols + i] = in ? __ldg(p.res_ln_beta + n) : 0.f;
        }
    }
    __syncwarp();
}

// mean and 1/sqrt(var + eps) of one row from its per-chunk partial sums, layout [slots][M][2].
__device__ __forceinline__ void row_stats(const float* stats, int slots, long long row, int M, int width, float eps,
                                          float* mean, float* rstd) {
    float s = 0.f, q = 0.f;
    const float2* base = reinterpret_cast<const float2*>(stats) + row;
    // Batches of 8 independent loads: the whole batch is in flight at once (one L2 round trip per batch instead of
    // one per slot).
    for (int i0 = 0; i0 < slots; i0 += 8) {
        float2 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
            v[j] = (i0 + j < slots) ? __ldg(base + static_cast<long long>(i0 + j) * M) : make_float2(0.f, 0.f);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            s += v[j].x;
            q += v[j].y;
        }
    }
    const float inv = 1.0f / static_cast<float>(width);
    const float m = s * inv;
    const float var = fmaxf(q * inv - m * m, 0.f);
    *mean = m;
    *rstd = 1.0f / sqrtf(var + eps);
}

// Half-precision outputs leave through shared memory: the warp writes its 32 x 32 chunk (64 bytes per row, 64-byte
// swizzle so that the 16-byte stores of a quarter warp hit distinct banks) into one of its private 2 KB strips, and
// one lane issues a TMA tile store, which writes whole 32-byte sectors and clips rows / columns outside the tensor.
// (A thread storing its own row directly issues 16-byte pieces to 32 different rows per instruction; measured, that
// store pattern alone held the 768-deep GEMMs at 60 % of what the mainloop delivers.)  fp32 outputs (graph edge only)
// are stored directly.  (Rotating more strips per warp was tried: the wait for the TMA engine to have read a strip is
// not on the critical path, while the extra shared memory costs a pipeline stage.)
//
// With RES the residual tile comes in the same way: a TMA load of the 32 x 32 chunk into a strip one chunk ahead,
// read back swizzled, added, and the strip is then reused for the output of that chunk.  Three strips rotate: the strip
// that receives the residual of chunk c + 1 last held the output of chunk c - 2, whose store was issued a whole chunk
// ago and has read its source by now (with two strips it was the store issued an instant earlier, and every chunk of
// the short-K residual GEMMs, whose epilogue is co-critical, waited for the store engine).
//
// FOLD compiles the LayerNorm-folding paths in (row statistics in/out, folded input / residual LayerNorm); without
// it the kernel carries neither their registers nor their shared-memory strips.
constexpr int kStageBytesPerWarp = 32 * 64;
template <bool RES> constexpr int strips_per_warp() { return RES ? 3 : 1; }
template <bool FOLD> constexpr int vec_strips() { return FOLD ? 4 : 1; }   // bias|c2, c1, gamma, beta

template <int CHUNKS, bool RES, bool FOLD>
struct WarpEpilogue {
    static constexpr int NSTRIPS = RES ? 3 : 1;
    const LinearParams& p;
    const CUtensorMap* tm_y;
    const CUtensorMap* tm_r;
    uint8_t* strips;              // NSTRIPS strips of this warp
    uint64_t* rbars;              // RES: NSTRIPS mbarriers of this warp
    volatile uint32_t* abort_flag;
    int lane;
    uint32_t cc;                  // chunks processed so far by this warp (selects strip / barrier / phase)
    float mean_x = 0.f, rstd_x = 0.f;   // folded input LayerNorm: statistics of this thread's row of x
    float mean_r = 0.f, rstd_r = 0.f;   // folded residual LayerNorm: statistics of this thread's row of the residual
    // Row statistics of the NEXT tile, in flight while the current tile is drained (one L2 round trip per tile would
    // otherwise sit on the epilogue's critical path).  Serves the folded input LayerNorm if there is one, else the
    // folded residual LayerNorm; up to kPrefetchSlots slots (768 columns), wider rows take the slow path.
    static constexpr int kPrefetchSlots = FOLD ? 24 : 1;
    float2 pf[kPrefetchSlots];
    long long pf_row = -1;
    // RES kernels only: a kernel that runs several GEMMs in one launch switches the residual path per GEMM (`res_on`);
    // bit s of `rpar` is the phase parity of strip s's residual barrier (it flips with every residual tile received).
    uint32_t rpar = 0;
    bool res_on = true;

    __device__ __forceinline__ bool ln_in() const { return FOLD && p.ln_in_stats != nullptr; }
    __device__ __forceinline__ bool res_ln() const { return FOLD && p.res_ln_stats != nullptr; }
    __device__ __forceinline__ void prefetch_stats(long long row) {
        if (!FOLD) return;
        pf_row = -1;
        const float* st = p.ln_in_stats ? p.ln_in_stats : p.res_ln_stats;
        const int slots = p.ln_in_stats ? p.k_slots : p.n_slots;
        if (st == nullptr || slots > kPrefetchSlots || row >= p.M || row < 0) return;
        const float2* base = reinterpret_cast<const float2*>(st) + row;
#pragma unroll
        for (int j = 0; j < kPrefetchSlots; ++j)
            pf[j] = (j < slots) ? __ldg(base + static_cast<long long>(j) * p.M) : make_float2(0.f, 0.f);
        pf_row = row;
    }
    __device__ __forceinline__ void finish_stats(int width, float* mean, float* rstd) const {
        float s = 0.f, q = 0.f;
#pragma unroll
        for (int j = 0; j < kPrefetchSlots; ++j) {
            s += pf[j].x;
            q += pf[j].y;
        }
        const float inv = 1.0f / static_cast<float>(width);
        const float m = s * inv;
        *mean = m;
        *rstd = 1.0f / sqrtf(fmaxf(q * inv - m * m, 0.f) + p.ln_eps);
    }

    __device__ __forceinline__ bool chunk_valid(int c, int n_first, int row0) const {
        return c < CHUNKS && n_first + c * 32 < p.N && row0 < p.M;
    }
    // lane 0: start the residual load of the chunk that will be processed as number `seq`.  Its strip last held the
    // output of chunk seq - 3; at most the latest store (chunk seq - 2 or later) may still be reading its strip.
    __device__ __forceinline__ void issue_residual(uint32_t seq, int n0, int row0) {
        if (lane == 0) {
            tma_store_wait_read<1>();
            const uint32_t si = seq % NSTRIPS;
            mbar_expect_tx(rbars + si, kStageBytesPerWarp);
            tma_load_2d(strips + si * kStageBytesPerWarp, tm_r, rbars + si, n0, row0);
        }
    }
    // Call before waiting for the accumulator: overlaps the first residual load with the tile's mainloop.
    __device__ __forceinline__ void begin_tile(int n_first, int row0) {
        if (RES && res_on && chunk_valid(0, n_first, row0)) issue_residual(cc, n_first, row0);
        if (!FOLD) return;
        const long long row = static_cast<long long>(row0) + lane;
        const bool have_pf = pf_row == row && row < p.M;
        if (p.ln_in_stats) {
            mean_x = rstd_x = 0.f;
            if (have_pf) finish_stats(p.K, &mean_x, &rstd_x);
            else if (row < p.M) row_stats(p.ln_in_stats, p.k_slots, row, p.M, p.K, p.ln_eps, &mean_x, &rstd_x);
        }
        if (p.res_ln_stats) {
            mean_r = rstd_r = 0.f;
            if (have_pf && !p.ln_in_stats) finish_stats(p.N, &mean_r, &rstd_r);
            else if (row < p.M) row_stats(p.res_ln_stats, p.n_slots, row, p.M, p.N, p.ln_eps, &mean_r, &rstd_r);
        }
    }

    // v[0..7] += residual (8 half-precision values in q), through the folded residual LayerNorm if there is one.
    template <int COLS>
    __device__ __forceinline__ void add_residual8(const uint4& q, const float* vec_w, int col, float* v) const {
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
        float r[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = unpack2(w[e], p.dtype);
            r[2 * e] = f.x;
            r[2 * e + 1] = f.y;
        }
        if (res_ln()) {
#pragma unroll
            for (int e = 0; e < 8; ++e)
                r[e] = fmaf((r[e] - mean_r) * rstd_r, vec_w[2 * COLS + col + e], vec_w[3 * COLS + col + e]);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] += r[e];
    }

    // 32 fp32 values of this thread's row -> half precision -> the row's 64 bytes of the strip (64-byte swizzle)
    template <int DT>
    __device__ __forceinline__ void stage_chunk(const float (&v)[32], uint8_t* srow) const {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            uint4 q;
            q.x = pack2t<DT>(v[g * 8 + 0], v[g * 8 + 1]);
            q.y = pack2t<DT>(v[g * 8 + 2], v[g * 8 + 3]);
            q.z = pack2t<DT>(v[g * 8 + 4], v[g * 8 + 5]);
            q.w = pack2t<DT>(v[g * 8 + 6], v[g * 8 + 7]);
            *reinterpret_cast<uint4*>(srow + ((g ^ ((lane >> 1) & 3)) << 4)) = q;
        }
    }

    // Drain this warp's part of one accumulator: rows = the warp's 32 TMEM lanes (thread = row `row`), columns
    // [col_first, col_first + 32*CHUNKS) of the tile whose first global column is n_tile0.  `tacc` is the TMEM address
    // of the accumulator's column 0 with this warp's lane offset already applied.  Returns false if a wait ran out.
    template <int COLS>
    __device__ __forceinline__ bool run(const float* vec_w, uint32_t tacc, long long row, int n_tile0, int col_first) {
        const bool row_ok = row < p.M;
        const int row0 = static_cast<int>(row) - lane;
        const int n_first = n_tile0 + col_first;
        uint32_t r[32];
        if (chunk_valid(0, n_first, row0)) tmem_ld_32x32b_x32(tacc + col_first, r);
#pragma unroll 1
        for (int c = 0; c < CHUNKS; ++c) {
            if (!chunk_valid(c, n_first, row0)) break;   // uniform across the warp; validity is monotone in c
            const int col0 = col_first + c * 32;
            const int n0 = n_tile0 + col0;
            const bool next_valid = chunk_valid(c + 1, n_first, row0);
            if (RES && res_on && next_valid) issue_residual(cc + 1, n0 + 32, row0);
            tmem_ld_wait(r);
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
            // the next chunk's accumulator columns travel while this chunk is processed
            if (next_valid) tmem_ld_32x32b_x32(tacc + col0 + 32, r);
            if (ln_in()) {
                // LN(x).W + b = rstd * (x.W' - mean * c1) + c2
                const float nm = -mean_x;
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    const float4 c2 = *reinterpret_cast<const float4*>(vec_w + c * 32 + g * 4);
                    const float4 c1 = *reinterpret_cast<const float4*>(vec_w + COLS + c * 32 + g * 4);
                    v[g * 4 + 0] = fmaf(rstd_x, fmaf(nm, c1.x, v[g * 4 + 0]), c2.x);
                    v[g * 4 + 1] = fmaf(rstd_x, fmaf(nm, c1.y, v[g * 4 + 1]), c2.y);
                    v[g * 4 + 2] = fmaf(rstd_x, fmaf(nm, c1.z, v[g * 4 + 2]), c2.z);
                    v[g * 4 + 3] = fmaf(rstd_x, fmaf(nm, c1.w, v[g * 4 + 3]), c2.w);
                }
            } else {
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    const float4 b = *reinterpret_cast<const float4*>(vec_w + c * 32 + g * 4);
                    unpack_f32x2(add_f32x2(pack_f32x2(v[g * 4 + 0], v[g * 4 + 1]), pack_f32x2(b.x, b.y)), v[g * 4 + 0],
                                 v[g * 4 + 1]);
                    unpack_f32x2(add_f32x2(pack_f32x2(v[g * 4 + 2], v[g * 4 + 3]), pack_f32x2(b.z, b.w)), v[g * 4 + 2],
                                 v[g * 4 + 3]);
                }
            }
            if (p.epilogue == B200_EPI_BIAS_GELU) {
#pragma unroll
                for (int j = 0; j < 32; j += 2) gelu_erf_x2(v[j], v[j + 1]);
            } else if (p.epilogue == B200_EPI_BIAS_TANH) {
                // hardware tanh: relative error <= 2^-11, below the half-precision rounding of the result
#pragma unroll
                for (int j = 0; j < 32; ++j) asm("tanh.approx.f32 %0, %1;" : "=f"(v[j]) : "f"(v[j]));
            }
            const uint32_t si = cc % NSTRIPS;
            uint8_t* strip = strips + si * kStageBytesPerWarp;
            uint8_t* srow = strip + lane * 64;
            if (RES && res_on) {
                if (!mbar_wait(rbars + si, (rpar >> si) & 1u, abort_flag)) return false;
                rpar ^= 1u << si;
                __syncwarp();
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const uint4 q = *reinterpret_cast<const uint4*>(srow + ((g ^ ((lane >> 1) & 3)) << 4));
                    add_residual8<COLS>(q, vec_w, c * 32 + g * 8, &v[g * 8]);
                }
            } else if (p.epilogue == B200_EPI_BIAS_RESIDUAL && row_ok) {
                const uint16_t* rp = reinterpret_cast<const uint16_t*>(p.residual) + row * p.ldr + n0;
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    if (n0 + g * 8 < p.N) {
                        const uint4 q = __ldg(reinterpret_cast<const uint4*>(rp + g * 8));
                        add_residual8<COLS>(q, vec_w, c * 32 + g * 8, &v[g * 8]);
                    }
                }
            }
            if (FOLD && p.out_stats != nullptr && row_ok) {
                float s1 = 0.f, s2 = 0.f;
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    s1 += v[j];
                    s2 = fmaf(v[j], v[j], s2);
                }
                // slot-major layout: the 32 rows of the warp write 256 contiguous bytes
                reinterpret_cast<float2*>(p.out_stats)[static_cast<long long>(n0 >> 5) * p.M + row] = make_float2(s1, s2);
            }
            if (p.out_dtype == B200_F32) {
                if (row_ok) {
                    float* yp = reinterpret_cast<float*>(p.y) + row * p.ldy + n0;
#pragma unroll
                    for (int g = 0; g < 8; ++g) {
                        if (n0 + g * 4 < p.N) {
                            *reinterpret_cast<float4*>(yp + g * 4) =
                                make_float4(v[g * 4], v[g * 4 + 1], v[g * 4 + 2], v[g * 4 + 3]);
                        }
                    }
                }
            } else {
                if (!(RES && res_on)) {
                    // the previous store of this warp from this strip must have finished reading it (with a residual
                    // the wait sits in issue_residual)
                    if (lane == 0) tma_store_wait_read<NSTRIPS - 1>();
                    __syncwarp();
                }
                if (p.out_dtype == B200_F16) stage_chunk<B200_F16>(v, srow);   // warp-uniform branch, specialised bodies
                else stage_chunk<B200_BF16>(v, srow);
                fence_async_proxy_shared();
                __syncwarp();
                if (lane == 0) {
                    tma_store_2d(tm_y, strip, n0, row0);
                    tma_store_commit();
                }
            }
            ++cc;
        }
        return true;
    }
};

// CTA-pair kernel (linear_pair.cu).  BN in {64, 128, 192, 256}.
template <int BN>
int launch_linear_pair(const B200LinearDesc& d, cudaStream_t stream, int sm_count);
int device_sm_count();   // SMs of the current device, <= 0 if it is not an sm_100 GPU
// Argument checks of b200_linear_fwd (pointers, alignment, leading dimensions, epilogue consistency).
int validate_linear_desc(const B200LinearDesc* d);
inline bool wants_fold(const B200LinearDesc& d) { return d.out_stats || d.ln_in_stats || d.res_ln_stats; }
// Number of CTA pairs of the pair kernel that can be co-resident on the current device (cached; 0 if unknown).
int max_active_pairs(int bn);

}  // namespace lin
}  // namespace b200
