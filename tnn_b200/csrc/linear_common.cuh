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

// Stage one warp's bias slice (COLS floats starting at column n_first) in its private shared-memory strip.
__device__ __forceinline__ void stage_bias(const LinearParams& p, float* bias_w, int n_first, int cols, int lane) {
    __syncwarp();
    for (int i = lane; i < cols; i += 32) {
        const int n = n_first + i;
        bias_w[i] = (p.bias != nullptr && n < p.N) ? __ldg(p.bias + n) : 0.f;
    }
    __syncwarp();
}

// Drain this warp's part of one accumulator: rows = the warp's 32 TMEM lanes (thread = row `row`), columns
// [col_first, col_first + 32*CHUNKS) of the tile whose first global column is n_tile0.  `tacc` is the TMEM address of
// the accumulator's column 0 with this warp's lane offset already applied.
// Half-precision outputs leave through shared memory: the warp writes its 32 x 32 chunk (64 bytes per row, 64-byte
// swizzle so that the 16-byte stores of a quarter warp hit distinct banks) into a private 2 KB strip, and one lane
// issues a TMA tile store, which writes whole 32-byte sectors and clips rows / columns outside the tensor.
// (A thread storing its own row directly issues 16-byte pieces to 32 different rows per instruction; measured, that
// store pattern alone held the 768-deep GEMMs at 60 % of what the mainloop delivers.)  fp32 outputs (graph edge only)
// are stored directly.
//
// With RES the residual tile comes in the same way: a TMA load of the 32 x 32 chunk into the strip (one chunk ahead,
// two strips), read back swizzled, added, and the strip is then reused for the output of that chunk.
constexpr int kStageBytesPerWarp = 32 * 64;

template <int CHUNKS, bool RES>
struct WarpEpilogue {
    const LinearParams& p;
    const CUtensorMap* tm_y;
    const CUtensorMap* tm_r;
    uint8_t* strips;              // RES: 2 strips, else 1
    uint64_t* rbars;              // RES: 2 mbarriers of this warp
    volatile uint32_t* abort_flag;
    int lane;
    uint32_t cc;                  // chunks processed so far by this warp (selects strip / barrier / phase when RES)

    __device__ __forceinline__ bool chunk_valid(int c, int n_first, int row0) const {
        return c < CHUNKS && n_first + c * 32 < p.N && row0 < p.M;
    }
    // lane 0: start the residual load of the chunk that will be processed as number `seq`
    __device__ __forceinline__ void issue_residual(uint32_t seq, int n0, int row0) {
        if (lane == 0) {
            tma_store_wait_read<0>();   // the strip's previous output store has been read out
            uint64_t* bar = rbars + (seq & 1u);
            mbar_expect_tx(bar, kStageBytesPerWarp);
            tma_load_2d(strips + (seq & 1u) * kStageBytesPerWarp, tm_r, bar, n0, row0);
        }
    }
    // Call before waiting for the accumulator: overlaps the first residual load with the tile's mainloop.
    __device__ __forceinline__ void begin_tile(int n_first, int row0) {
        if (RES && chunk_valid(0, n_first, row0)) issue_residual(cc, n_first, row0);
    }

    // Drain this warp's part of one accumulator: rows = the warp's 32 TMEM lanes (thread = row `row`), columns
    // [col_first, col_first + 32*CHUNKS) of the tile whose first global column is n_tile0.  `tacc` is the TMEM address
    // of the accumulator's column 0 with this warp's lane offset already applied.  Returns false if a wait ran out.
    __device__ __forceinline__ bool run(const float* bias_w, uint32_t tacc, long long row, int n_tile0, int col_first) {
        const bool row_ok = row < p.M;
        const int row0 = static_cast<int>(row) - lane;
        const int n_first = n_tile0 + col_first;
#pragma unroll 1
        for (int c = 0; c < CHUNKS; ++c) {
            if (!chunk_valid(c, n_first, row0)) continue;   // uniform across the warp
            const int col0 = col_first + c * 32;
            const int n0 = n_tile0 + col0;
            if (RES && chunk_valid(c + 1, n_first, row0)) issue_residual(cc + 1, n0 + 32, row0);
            uint32_t r[32];
            tmem_ld_32x32b_x32(tacc + col0, r);
            tmem_ld_wait(r);
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
#pragma unroll
            for (int g = 0; g < 8; ++g) {
                const float4 b = *reinterpret_cast<const float4*>(bias_w + c * 32 + g * 4);
                v[g * 4 + 0] += b.x;
                v[g * 4 + 1] += b.y;
                v[g * 4 + 2] += b.z;
                v[g * 4 + 3] += b.w;
            }
            if (p.epilogue == B200_EPI_BIAS_GELU) {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = gelu_erf(v[j]);
            }
            uint8_t* strip = strips + (RES ? (cc & 1u) * kStageBytesPerWarp : 0u);
            uint8_t* srow = strip + lane * 64;
            if (RES) {
                if (!mbar_wait(rbars + (cc & 1u), (cc >> 1) & 1u, abort_flag)) return false;
                __syncwarp();
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const uint4 q = *reinterpret_cast<const uint4*>(srow + ((g ^ ((lane >> 1) & 3)) << 4));
                    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 f = unpack2(w[e], p.dtype);
                        v[g * 8 + e * 2 + 0] += f.x;
                        v[g * 8 + e * 2 + 1] += f.y;
                    }
                }
            } else if (p.epilogue == B200_EPI_BIAS_RESIDUAL && row_ok) {
                const uint16_t* rp = reinterpret_cast<const uint16_t*>(p.residual) + row * p.ldr + n0;
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    if (n0 + g * 8 < p.N) {
                        const uint4 q = __ldg(reinterpret_cast<const uint4*>(rp + g * 8));
                        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float2 f = unpack2(w[e], p.dtype);
                            v[g * 8 + e * 2 + 0] += f.x;
                            v[g * 8 + e * 2 + 1] += f.y;
                        }
                    }
                }
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
                if (!RES) {
                    // the previous TMA store of this warp must have finished reading the strip
                    if (lane == 0) tma_store_wait_read<0>();
                    __syncwarp();
                }
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    uint4 q;
                    q.x = pack2(v[g * 8 + 0], v[g * 8 + 1], p.out_dtype);
                    q.y = pack2(v[g * 8 + 2], v[g * 8 + 3], p.out_dtype);
                    q.z = pack2(v[g * 8 + 4], v[g * 8 + 5], p.out_dtype);
                    q.w = pack2(v[g * 8 + 6], v[g * 8 + 7], p.out_dtype);
                    *reinterpret_cast<uint4*>(srow + ((g ^ ((lane >> 1) & 3)) << 4)) = q;
                }
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
// Number of CTA pairs of the pair kernel that can be co-resident on the current device (cached; 0 if unknown).
int max_active_pairs(int bn);

}  // namespace lin
}  // namespace b200
