// Task heads after the encoder.  The span-extraction (question answering) head is a projection to very few outputs per
// token — start and end logits — followed by an "unstack" into one [B, S] array per output.  With N = 2 outputs this is
// a read of the activation matrix and nothing else: HBM-bound, algorithmic bytes per token H * element size + 4 N.
#include "common.cuh"
#include "ptx.cuh"

namespace b200 {
namespace {

constexpr int kHeadMaxN = 4;

// One warp per token row, two rows in flight per warp; a lane takes every 32nd group of 8 consecutive features (NV
// groups per lane, all loads of both rows issued before the first is used: an HBM-bound kernel lives on bytes in
// flight).  The weight lives in shared memory as float4 [N][2][H / 8]: the first and the second four of a group's 8
// features in separate planes, so that the 32 lanes of a warp read consecutive float4 (no bank conflicts; the plain
// transposed layout read with a 32-byte lane stride, two-way conflicts, and ncu showed the shared-memory pipe 85 %
// busy at 38 % of DRAM throughput); one read serves both rows.  fp32 accumulation in feature order within a lane,
// lanes combined by a butterfly.  Output n of token t goes to out[n * ld_out + t], or to out_n[n][t].
template <int N, int NV>
__global__ void __launch_bounds__(256) qa_head_kernel(B200QAHeadDesc d) {
    extern __shared__ __align__(16) float w_s[];
    const int lane = threadIdx.x & 31;
    const int H = static_cast<int>(d.H);
    const int groups = H >> 3;
    for (int i = threadIdx.x; i < H * N; i += blockDim.x) {
        const int k = i / N, n = i % N;   // the MatMul weight is [H, N] row-major
        w_s[(((n * 2 + ((k >> 2) & 1)) * groups) + (k >> 3)) * 4 + (k & 3)] = d.weight[i];
    }
    __syncthreads();
    float bias[N];
    float* dst[N];   // output n of token t goes to dst[n][t]
#pragma unroll
    for (int n = 0; n < N; ++n) {
        bias[n] = d.bias ? d.bias[n] : 0.f;
        dst[n] = d.out_n[0] != nullptr ? d.out_n[n] : d.out + n * d.ld_out;
    }
    const long long warp0 = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    const long long nwarps = static_cast<long long>(gridDim.x) * 8;
    pdl_launch_dependents();
    pdl_wait();
    for (long long t0 = warp0; t0 < d.M; t0 += 2 * nwarps) {
        const long long t1 = t0 + nwarps;
        const bool two = t1 < d.M;
        uint4 q[2][NV];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const uint16_t* row = reinterpret_cast<const uint16_t*>(d.x) + (r == 0 ? t0 : t1) * d.ldx;
#pragma unroll
            for (int g = 0; g < NV; ++g) {
                const int gi = g * 32 + lane;
                q[r][g] = (gi < groups && (r == 0 || two)) ? __ldg(reinterpret_cast<const uint4*>(row + gi * 8))
                                                            : make_uint4(0u, 0u, 0u, 0u);
            }
        }
        float acc[2][N];
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
            for (int n = 0; n < N; ++n) acc[r][n] = 0.f;
#pragma unroll
        for (int g = 0; g < NV; ++g) {
            const int gi = g * 32 + lane;
            if (gi < groups) {
                float v[2][8];
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    const uint32_t w[4] = {q[r][g].x, q[r][g].y, q[r][g].z, q[r][g].w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 f = unpack2(w[e], d.x_dtype);
                        v[r][2 * e] = f.x;
                        v[r][2 * e + 1] = f.y;
                    }
                }
#pragma unroll
                for (int n = 0; n < N; ++n) {
                    const float4 a = reinterpret_cast<const float4*>(w_s)[(n * 2 + 0) * groups + gi];
                    const float4 b = reinterpret_cast<const float4*>(w_s)[(n * 2 + 1) * groups + gi];
                    const float wv[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
                    for (int r = 0; r < 2; ++r)
#pragma unroll
                        for (int e = 0; e < 8; ++e) acc[r][n] = fmaf(v[r][e], wv[e], acc[r][n]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
            for (int n = 0; n < N; ++n) {
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) acc[r][n] += __shfl_xor_sync(0xffffffffu, acc[r][n], o);
            }
        if (lane == 0) {
#pragma unroll
            for (int n = 0; n < N; ++n) {
                dst[n][t0] = acc[0][n] + bias[n];
                if (two) dst[n][t1] = acc[1][n] + bias[n];
            }
        }
    }
}

template <int N>
void launch_qa(const B200QAHeadDesc& d, cudaStream_t stream) {
    long long blocks = (d.M + 7) / 8;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long long cap = 6ll * sms;
    if (blocks > cap) blocks = cap;
    const int nv = static_cast<int>((d.H / 8 + 31) / 32);
    const size_t smem = static_cast<size_t>(d.H) * N * sizeof(float);
    const dim3 grid(static_cast<unsigned>(blocks)), block(256);
    if (nv <= 3) launch_kernel(qa_head_kernel<N, 3>, grid, block, smem, stream, d);
    else if (nv <= 4) launch_kernel(qa_head_kernel<N, 4>, grid, block, smem, stream, d);
    else launch_kernel(qa_head_kernel<N, 16>, grid, block, smem, stream, d);
}

}  // namespace
}  // namespace b200

extern "C" int b200_qa_head_fwd(const B200QAHeadDesc* d, b200_stream_t stream_) {
    using namespace b200;
    if (!d || d->M < 0 || d->H <= 0 || d->N <= 0) return B200_ERR_PARAM;
    if (d->M == 0 && d->N <= kHeadMaxN && (d->H % 8) == 0) return B200_OK;   // nothing to do: pointers may be null
    if (!d->x || !d->weight) return B200_ERR_PARAM;
    if (d->out_n[0] != nullptr) {
        for (int n = 0; n < d->N && n < kHeadMaxN; ++n)
            if (d->out_n[n] == nullptr) return B200_ERR_PARAM;
    } else if (!d->out || d->ld_out < d->M) {
        return B200_ERR_PARAM;
    }
    if (!is_half_dtype(d->x_dtype)) return B200_ERR_PARAM;
    if ((d->H % 8) || (d->ldx % 8) || d->ldx < d->H) return B200_ERR_PARAM;
    if (!aligned16(d->x)) return B200_ERR_PARAM;
    if (d->N > kHeadMaxN || d->H * d->N * 4 > 48 * 1024 || d->H > 4096) return B200_ERR_UNSUPPORTED;
    int dev = 0, major = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return B200_ERR_LAUNCH;
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (major != 10) return B200_ERR_NOT_SM100;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    switch (d->N) {
        case 1: launch_qa<1>(*d, stream); break;
        case 2: launch_qa<2>(*d, stream); break;
        case 3: launch_qa<3>(*d, stream); break;
        default: launch_qa<4>(*d, stream); break;
    }
    count_launch();
    return check_launch();
}
