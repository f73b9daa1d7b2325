// HBM-bound kernels of the path: (residual +) LayerNorm, dtype conversion at the fp32 boundary of the fused region,
// the one-time weight pre-pack (fp32 [K,N] -> half [N,K]) and the mask -> kv_len reduction.
// All are plain coalesced 16-byte-vector kernels; their roofline is HBM bandwidth.
#include "common.cuh"
#include "ptx.cuh"

namespace b200 {
namespace {

// ---------------------------------------------------------------- vector load/store of 8 elements as fp32
__device__ __forceinline__ void load8(const void* base, long long elem_off, int dtype, float (&v)[8]) {
    if (dtype == B200_F32) {
        const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + elem_off);
        const float4 a = __ldg(p), b = __ldg(p + 1);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
        v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
        const uint4 q = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(base) + elem_off));
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = unpack2(w[e], dtype);
            v[2 * e] = f.x;
            v[2 * e + 1] = f.y;
        }
    }
}
__device__ __forceinline__ void store8(void* base, long long elem_off, int dtype, const float (&v)[8]) {
    if (dtype == B200_F32) {
        float4* p = reinterpret_cast<float4*>(reinterpret_cast<float*>(base) + elem_off);
        p[0] = make_float4(v[0], v[1], v[2], v[3]);
        p[1] = make_float4(v[4], v[5], v[6], v[7]);
    } else {
        uint4 q;
        q.x = pack2(v[0], v[1], dtype);
        q.y = pack2(v[2], v[3], dtype);
        q.z = pack2(v[4], v[5], dtype);
        q.w = pack2(v[6], v[7], dtype);
        *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(base) + elem_off) = q;
    }
}


// ---------------------------------------------------------------- (residual +) LayerNorm
// One warp per row; a lane holds NV groups of 8 consecutive elements (group g of the lane = elements
// (g*32 + lane)*8 ..), so every load/store instruction of the warp covers 512 (or 1024 for fp32) contiguous bytes.
// Algorithmic HBM bytes per row: H * (in + residual + out) element sizes (+ gamma/beta, L2-resident).
template <int NV>
__global__ void __launch_bounds__(256) add_layernorm_kernel(B200LayerNormDesc d) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    pdl_launch_dependents();
    pdl_wait();
    if (warp >= d.rows) return;
    const long long row = warp;
    const int groups = static_cast<int>(d.H >> 3);
    float v[NV][8];
    float sum = 0.f;
#pragma unroll
    for (int g = 0; g < NV; ++g) {
        const int gi = g * 32 + lane;
        if (gi < groups) {
            load8(d.x, row * d.ldx + gi * 8, d.in_dtype, v[g]);
            if (d.residual != nullptr) {
                float r[8];
                load8(d.residual, row * d.ldr + gi * 8, d.in_dtype, r);
#pragma unroll
                for (int e = 0; e < 8; ++e) v[g][e] += r[e];
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) sum += v[g][e];
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) v[g][e] = 0.f;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv_h = 1.0f / static_cast<float>(d.H);
    const float mean = sum * inv_h;
    float sq = 0.f;
#pragma unroll
    for (int g = 0; g < NV; ++g) {
        const int gi = g * 32 + lane;
        if (gi < groups) {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float c = v[g][e] - mean;
                sq += c * c;
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    const float rstd = 1.0f / sqrtf(sq * inv_h + d.eps);
#pragma unroll
    for (int g = 0; g < NV; ++g) {
        const int gi = g * 32 + lane;
        if (gi < groups) {
            float gm[8], bt[8], o[8];
            load8(d.gamma, gi * 8, B200_F32, gm);
            load8(d.beta, gi * 8, B200_F32, bt);
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] = (v[g][e] - mean) * rstd * gm[e] + bt[e];
            store8(d.y, row * d.ldy + gi * 8, d.out_dtype, o);
        }
    }
}

// Persistent variant for H <= 1024 (NV <= 4): 8 warps per block walk rows with a grid stride; gamma/beta sit in
// shared memory (the generic kernel re-reads 4x more gamma/beta bytes than activation bytes per row), and every warp
// has the next row's loads in flight while it reduces the current one, so that with 4 blocks per SM about 64 rows
// (100 KB) per SM are in flight — enough to cover HBM latency at full bandwidth.
// RESID compiles the residual operand in; without it (the encoder path: the residual is added in the GEMM epilogue)
// the kernel fits 64 registers and four blocks per SM — LayerNorm at these sizes is latency-bound per warp, so its
// speed is the number of resident warps.
template <int NV, bool F32IN, bool RESID>
__global__ void __launch_bounds__(256, (NV >= 4 || F32IN) ? 2 : (RESID ? 3 : 4)) add_layernorm_rows_kernel(B200LayerNormDesc d) {
    extern __shared__ float gb[];   // gamma | beta, NV * 256 floats each, in the lane-major layout described below
    const int lane = threadIdx.x & 31;
    const int H = static_cast<int>(d.H);
    const long long warp0 = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    const long long nwarps = static_cast<long long>(gridDim.x) * 8;
    const int groups = H >> 3;
    constexpr bool f32_in = F32IN;
    constexpr int Q = F32IN ? 2 : 1;   // 16-byte pieces per group of 8 elements
    uint4 raw[NV][Q], rres[RESID ? NV : 1][Q];
    auto fetch = [&](long long row) {
#pragma unroll
        for (int g = 0; g < NV; ++g) {
            const int gi = g * 32 + lane;
            if (gi < groups) {
                if (f32_in) {
                    const uint4* px = reinterpret_cast<const uint4*>(reinterpret_cast<const float*>(d.x) + row * d.ldx + gi * 8);
                    raw[g][0] = __ldg(px);
                    raw[g][Q - 1] = __ldg(px + 1);
                    if (RESID && d.residual) {
                        const uint4* pr = reinterpret_cast<const uint4*>(reinterpret_cast<const float*>(d.residual) + row * d.ldr + gi * 8);
                        rres[g][0] = __ldg(pr);
                        rres[g][Q - 1] = __ldg(pr + 1);
                    }
                } else {
                    raw[g][0] = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(d.x) + row * d.ldx + gi * 8));
                    if (RESID && d.residual)
                        rres[g][0] = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(d.residual) + row * d.ldr + gi * 8));
                }
            }
        }
    };
    auto decode = [&](const uint4 (&q)[Q], float (&v)[8]) {
        if (f32_in) {
            v[0] = __uint_as_float(q[0].x); v[1] = __uint_as_float(q[0].y);
            v[2] = __uint_as_float(q[0].z); v[3] = __uint_as_float(q[0].w);
            v[4] = __uint_as_float(q[Q - 1].x); v[5] = __uint_as_float(q[Q - 1].y);
            v[6] = __uint_as_float(q[Q - 1].z); v[7] = __uint_as_float(q[Q - 1].w);
        } else {
            const uint32_t w[4] = {q[0].x, q[0].y, q[0].z, q[0].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = unpack2(w[e], d.in_dtype);
                v[2 * e] = f.x;
                v[2 * e + 1] = f.y;
            }
        }
    };
    const float inv_h = 1.0f / static_cast<float>(d.H);
    long long row = warp0;
    // gamma/beta are constants: they are staged while the producer of x may still be running
    pdl_launch_dependents();
    // Layout: the two float4 halves of a lane's group of 8 live in separate planes, [g][half][lane], so that the 32 lanes
    // of a warp read 32 consecutive float4 (4 wavefronts per load, the minimum; in feature order the lanes would sit
    // 32 bytes apart, every load would take 8 wavefronts, and the kernel was bound by exactly that: 94 % of the
    // L1 / shared-memory pipe at 44 % of HBM in the profile).
    for (int j = threadIdx.x; j < H / 4; j += blockDim.x) {
        const int gi = j >> 1, half = j & 1;
        const int dst = (((gi >> 5) * 2 + half) * 32 + (gi & 31)) * 4;
        *reinterpret_cast<float4*>(gb + dst) = __ldg(reinterpret_cast<const float4*>(d.gamma) + j);
        *reinterpret_cast<float4*>(gb + NV * 256 + dst) = __ldg(reinterpret_cast<const float4*>(d.beta) + j);
    }
    pdl_wait();
    if (row < d.rows) fetch(row);
    __syncthreads();
    // The arithmetic runs on pairs (packed fp32: one issue slot per two adds / multiplies / fmas).  Under the power cap
    // of a long run the SM clock drops by 40 % while HBM keeps its rate, and this kernel, which is bound by HBM at full
    // clock, becomes bound by its instruction stream: halving the stream is what keeps it on the memory roof.
    for (; row < d.rows; row += nwarps) {
        uint64_t v[NV][4];   // the lane's elements as pairs (2e, 2e+1)
        uint64_t sum2 = 0ull;
#pragma unroll
        for (int g = 0; g < NV; ++g) {
            const int gi = g * 32 + lane;
            if (gi < groups) {
                float f[8];
                decode(raw[g], f);
                if (RESID && d.residual) {
                    float r[8];
                    decode(rres[g], r);
#pragma unroll
                    for (int e = 0; e < 8; ++e) f[e] += r[e];
                }
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    v[g][e] = pack_f32x2(f[2 * e], f[2 * e + 1]);
                    sum2 = add_f32x2(sum2, v[g][e]);
                }
            }
        }
        if (row + nwarps < d.rows) fetch(row + nwarps);   // next row's loads fly during the reductions below
        float s_lo, s_hi;
        unpack_f32x2(sum2, s_lo, s_hi);
        float sum = s_lo + s_hi;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        const float mean = sum * inv_h;
        const uint64_t nmean2 = pack_f32x2(-mean, -mean);
        uint64_t sq2 = 0ull;
#pragma unroll
        for (int g = 0; g < NV; ++g) {
            const int gi = g * 32 + lane;
            if (gi < groups) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    v[g][e] = add_f32x2(v[g][e], nmean2);        // deviations from the mean, kept for the output
                    sq2 = fma_f32x2(v[g][e], v[g][e], sq2);
                }
            }
        }
        float q_lo, q_hi;
        unpack_f32x2(sq2, q_lo, q_hi);
        float sq = q_lo + q_hi;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        const float rstd = 1.0f / sqrtf(sq * inv_h + d.eps);
        const uint64_t rstd2 = pack_f32x2(rstd, rstd);
#pragma unroll
        for (int g = 0; g < NV; ++g) {
            const int gi = g * 32 + lane;
            if (gi < groups) {
                const float4* gp = reinterpret_cast<const float4*>(gb) + g * 64 + lane;
                const float4* bp = reinterpret_cast<const float4*>(gb + NV * 256) + g * 64 + lane;
                const float4 g0 = gp[0], g1 = gp[32], b0 = bp[0], b1 = bp[32];
                const uint64_t gm[4] = {pack_f32x2(g0.x, g0.y), pack_f32x2(g0.z, g0.w), pack_f32x2(g1.x, g1.y),
                                        pack_f32x2(g1.z, g1.w)};
                const uint64_t bt[4] = {pack_f32x2(b0.x, b0.y), pack_f32x2(b0.z, b0.w), pack_f32x2(b1.x, b1.y),
                                        pack_f32x2(b1.z, b1.w)};
                float o[8];
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    unpack_f32x2(fma_f32x2(mul_f32x2(v[g][e], rstd2), gm[e], bt[e]), o[2 * e], o[2 * e + 1]);
                store8(d.y, row * d.ldy + gi * 8, d.out_dtype, o);
            }
        }
    }
}

// ---------------------------------------------------------------- conversion
__global__ void __launch_bounds__(256) convert_kernel(const void* src, int sdt, void* dst, int ddt, long long n8,
                                                      long long n) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    pdl_launch_dependents();
    pdl_wait();
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8; i += stride) {
        float v[8];
        load8(src, i * 8, sdt, v);
        store8(dst, i * 8, ddt, v);
    }
    // tail (n % 8 elements) by the first threads of the grid
    const long long tail0 = n8 * 8;
    const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (tail0 + t < n) {
        float x;
        const long long i = tail0 + t;
        if (sdt == B200_F32) x = reinterpret_cast<const float*>(src)[i];
        else if (sdt == B200_F16) x = __half2float(reinterpret_cast<const __half*>(src)[i]);
        else x = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(src)[i]);
        if (ddt == B200_F32) reinterpret_cast<float*>(dst)[i] = x;
        else if (ddt == B200_F16) reinterpret_cast<__half*>(dst)[i] = __float2half_rn(x);
        else reinterpret_cast<__nv_bfloat16*>(dst)[i] = __float2bfloat16_rn(x);
    }
}

// ---------------------------------------------------------------- weight pre-pack: fp32 [K,N] -> half [N,K]
__global__ void __launch_bounds__(256) pack_weight_kernel(const float* src, long long K, long long N, long long ld_src,
                                                          uint16_t* dst, long long ld_dst, int dtype,
                                                          const float* row_scale) {
    __shared__ float tile[32][33];
    const long long k0 = static_cast<long long>(blockIdx.y) * 32;
    const long long n0 = static_cast<long long>(blockIdx.x) * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
    for (int r = ty; r < 32; r += 8) {
        const long long k = k0 + r, n = n0 + tx;
        tile[r][tx] = (k < K && n < N) ? src[k * ld_src + n] * (row_scale ? row_scale[k] : 1.0f) : 0.f;
    }
    __syncthreads();
    for (int r = ty; r < 32; r += 8) {
        const long long n = n0 + r, k = k0 + tx;
        if (n < N && k < K) {
            const float x = tile[tx][r];
            uint16_t bits;
            if (dtype == B200_F16) {
                const __half h = __float2half_rn(x);
                bits = *reinterpret_cast<const uint16_t*>(&h);
            } else {
                const __nv_bfloat16 h = __float2bfloat16_rn(x);
                bits = *reinterpret_cast<const uint16_t*>(&h);
            }
            dst[n * ld_dst + k] = bits;
        }
    }
}

// c1[n] = sum_k packed[n,k] (the rounded, gamma-scaled weights), c2[n] = sum_k beta[k] * w[k,n] + bias[n].
// One warp per output column; runs once per weight at Init.
__global__ void __launch_bounds__(256) fold_vectors_kernel(const float* w_kn, long long K, long long N, long long ld_src,
                                                           const uint16_t* packed, long long ld_dst, int dtype,
                                                           const float* beta, const float* bias, float* c1, float* c2) {
    const long long n = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (n >= N) return;
    float s1 = 0.f, s2 = 0.f;
    for (long long k = lane; k < K; k += 32) {
        const uint16_t bits = packed[n * ld_dst + k];
        float w;
        if (dtype == B200_F16) w = __half2float(*reinterpret_cast<const __half*>(&bits));
        else w = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(&bits));
        s1 += w;
        s2 = fmaf(beta[k], w_kn[k * ld_src + n], s2);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        s1 += __shfl_xor_sync(0xffffffffu, s1, o);
        s2 += __shfl_xor_sync(0xffffffffu, s2, o);
    }
    if (lane == 0) {
        c1[n] = s1;
        c2[n] = s2 + (bias ? bias[n] : 0.f);
    }
}

// ---------------------------------------------------------------- mask -> kv_len
__global__ void __launch_bounds__(128) mask_to_kv_len_kernel(const float* mask, long long S, float below, int* out) {
    const long long b = blockIdx.x;
    int last = 0;
    for (long long k = threadIdx.x; k < S; k += blockDim.x)
        if (mask[b * S + k] > below) last = static_cast<int>(k) + 1;
    __shared__ int red[4];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) last = max(last, __shfl_xor_sync(0xffffffffu, last, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = last;
    __syncthreads();
    if (threadIdx.x == 0) out[b] = max(max(red[0], red[1]), max(red[2], red[3]));
}

bool valid_dtype(int dt) { return dt == B200_F16 || dt == B200_BF16 || dt == B200_F32; }

template <int NV, bool F32IN>
void launch_rows(bool resid, unsigned grid, size_t smem, cudaStream_t stream, const B200LayerNormDesc& d) {
    if (resid) launch_kernel(add_layernorm_rows_kernel<NV, F32IN, true>, dim3(grid), dim3(256), smem, stream, d);
    else launch_kernel(add_layernorm_rows_kernel<NV, F32IN, false>, dim3(grid), dim3(256), smem, stream, d);
}

}  // namespace
}  // namespace b200

extern "C" {

int b200_add_layernorm_fwd(const B200LayerNormDesc* d, b200_stream_t stream_) {
    using namespace b200;
    if (!d || !d->x || !d->y || !d->gamma || !d->beta) return B200_ERR_PARAM;
    if (d->rows < 0 || d->H <= 0) return B200_ERR_PARAM;
    if (!valid_dtype(d->in_dtype) || !valid_dtype(d->out_dtype)) return B200_ERR_PARAM;
    if ((d->H % 8) || (d->ldx % 8) || (d->ldy % 8) || d->ldx < d->H || d->ldy < d->H) return B200_ERR_PARAM;
    if (d->residual && ((d->ldr % 8) || d->ldr < d->H || !aligned16(d->residual))) return B200_ERR_PARAM;
    if (!aligned16(d->x) || !aligned16(d->y) || !aligned16(d->gamma) || !aligned16(d->beta)) return B200_ERR_PARAM;
    if (d->H > 4096) return B200_ERR_UNSUPPORTED;
    if (d->rows == 0) return B200_OK;
    if (d->rows > (1ll << 31) - 1) return B200_ERR_UNSUPPORTED;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const int warps_per_block = 8;
    const unsigned grid = static_cast<unsigned>((d->rows + warps_per_block - 1) / warps_per_block);
    const int nv = static_cast<int>((d->H / 8 + 31) / 32);
    if (nv <= 4) {
        // One resident wave of 3 (2 for the wider variants) blocks x 8 warps per SM; every warp then walks rows with a
        // grid stride.
        const bool f32 = d->in_dtype == B200_F32;
        const long long per_sm = (nv >= 4 || f32) ? 2 : (d->residual ? 3 : 4);
        long long blocks = (d->rows + 7) / 8;
        if (blocks > 148ll * per_sm) blocks = 148ll * per_sm;
        const unsigned g2 = static_cast<unsigned>(blocks);
        const int nv_t = nv <= 1 ? 1 : (nv <= 3 ? 3 : 4);                      // the template instance's groups per lane
        const size_t sm = static_cast<size_t>(nv_t) * 256 * 2 * sizeof(float);   // gamma and beta planes
        if (nv <= 1) {
            if (f32) launch_rows<1, true>(d->residual != nullptr, g2, sm, stream, *d);
            else launch_rows<1, false>(d->residual != nullptr, g2, sm, stream, *d);
        } else if (nv <= 3) {
            if (f32) launch_rows<3, true>(d->residual != nullptr, g2, sm, stream, *d);
            else launch_rows<3, false>(d->residual != nullptr, g2, sm, stream, *d);
        } else {
            if (f32) launch_rows<4, true>(d->residual != nullptr, g2, sm, stream, *d);
            else launch_rows<4, false>(d->residual != nullptr, g2, sm, stream, *d);
        }
    } else if (nv <= 8) launch_kernel(add_layernorm_kernel<8>, dim3(grid), dim3(256), 0, stream, *d);
    else launch_kernel(add_layernorm_kernel<16>, dim3(grid), dim3(256), 0, stream, *d);
    count_launch();
    return check_launch();
}

int b200_convert(const void* src, int sdt, void* dst, int ddt, int64_t n, b200_stream_t stream_) {
    using namespace b200;
    if (!src || !dst || n < 0 || !valid_dtype(sdt) || !valid_dtype(ddt)) return B200_ERR_PARAM;
    if (!aligned16(src) || !aligned16(dst)) return B200_ERR_PARAM;
    if (n == 0) return B200_OK;
    const long long n8 = n / 8;
    long long blocks = (n8 + 255) / 256;
    if (blocks < 1) blocks = 1;
    if (blocks > 148 * 16) blocks = 148 * 16;
    launch_kernel(convert_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, static_cast<cudaStream_t>(stream_),
                  src, sdt, dst, ddt, n8, n);
    count_launch();
    return check_launch();
}

int b200_pack_weight(const float* w_kn, int64_t K, int64_t N, int64_t ld_src, void* w_nk, int64_t ld_dst, int dtype,
                     b200_stream_t stream_) {
    using namespace b200;
    if (!w_kn || !w_nk || K <= 0 || N <= 0 || ld_src < N || ld_dst < K || !is_half_dtype(dtype)) return B200_ERR_PARAM;
    dim3 grid(static_cast<unsigned>((N + 31) / 32), static_cast<unsigned>((K + 31) / 32));
    if (grid.y > 65535) return B200_ERR_UNSUPPORTED;
    pack_weight_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream_)>>>(
        w_kn, K, N, ld_src, static_cast<uint16_t*>(w_nk), ld_dst, dtype, nullptr);
    count_launch();
    return check_launch();
}

int b200_fold_layernorm_weight(const float* w_kn, int64_t K, int64_t N, int64_t ld_src, const float* gamma,
                               const float* beta, const float* bias, void* w_nk, int64_t ld_dst, int dtype, float* c1,
                               float* c2, b200_stream_t stream_) {
    using namespace b200;
    if (!w_kn || !w_nk || !gamma || !beta || !c1 || !c2) return B200_ERR_PARAM;
    if (K <= 0 || N <= 0 || ld_src < N || ld_dst < K || !is_half_dtype(dtype)) return B200_ERR_PARAM;
    dim3 grid(static_cast<unsigned>((N + 31) / 32), static_cast<unsigned>((K + 31) / 32));
    if (grid.y > 65535) return B200_ERR_UNSUPPORTED;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    pack_weight_kernel<<<grid, 256, 0, stream>>>(w_kn, K, N, ld_src, static_cast<uint16_t*>(w_nk), ld_dst, dtype, gamma);
    const unsigned blocks = static_cast<unsigned>((N * 32 + 255) / 256);
    fold_vectors_kernel<<<blocks, 256, 0, stream>>>(w_kn, K, N, ld_src, static_cast<const uint16_t*>(w_nk), ld_dst, dtype,
                                                    beta, bias, c1, c2);
    count_launch(2);
    return check_launch();
}

int b200_mask_to_kv_len(const float* mask_add, int64_t B, int64_t S, float exclude_below, int32_t* kv_len,
                        b200_stream_t stream_) {
    using namespace b200;
    if (!mask_add || !kv_len || B < 0 || S <= 0) return B200_ERR_PARAM;
    if (B == 0) return B200_OK;
    mask_to_kv_len_kernel<<<static_cast<unsigned>(B), 128, 0, static_cast<cudaStream_t>(stream_)>>>(mask_add, S,
                                                                                                  exclude_below, kv_len);
    count_launch();
    return check_launch();
}

}  // extern "C"
