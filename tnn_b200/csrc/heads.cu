// Task heads after the encoder.  The span-extraction (question answering) head is a projection to very few outputs per
// token — start and end logits — followed by an "unstack" into one [B, S] array per output.  With N = 2 outputs this is
// a read of the activation matrix and nothing else: HBM-bound, algorithmic bytes per token H * element size + 4 N.
#include "common.cuh"
#include "ptx.cuh"

namespace b200 {
namespace {

constexpr int kHeadMaxN = 4;

// One warp per token row; a lane takes every 32nd group of 8 consecutive features.  The weight lives in shared memory
// transposed ([N][H], fp32) so that a lane reads 8 consecutive floats per output; fp32 accumulation in feature order
// within a lane, lanes combined by a butterfly.  Output n of token t goes to out[n * ld_out + t].
template <int N>
__global__ void __launch_bounds__(256) qa_head_kernel(B200QAHeadDesc d) {
    extern __shared__ __align__(16) float w_s[];   // [N][H]
    const int lane = threadIdx.x & 31;
    const int H = static_cast<int>(d.H);
    for (int i = threadIdx.x; i < H * N; i += blockDim.x) {
        const int k = i / N, n = i % N;
        w_s[n * H + k] = d.weight[i];   // the MatMul weight is [H, N] row-major
    }
    __syncthreads();
    float bias[N];
#pragma unroll
    for (int n = 0; n < N; ++n) bias[n] = d.bias ? d.bias[n] : 0.f;
    const long long warp0 = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    const long long nwarps = static_cast<long long>(gridDim.x) * 8;
    const int groups = H >> 3;
    pdl_launch_dependents();
    pdl_wait();
    for (long long t = warp0; t < d.M; t += nwarps) {
        float acc[N];
#pragma unroll
        for (int n = 0; n < N; ++n) acc[n] = 0.f;
        const uint16_t* row = reinterpret_cast<const uint16_t*>(d.x) + t * d.ldx;
        for (int g = lane; g < groups; g += 32) {
            const uint4 q = __ldg(reinterpret_cast<const uint4*>(row + g * 8));
            const uint32_t w[4] = {q.x, q.y, q.z, q.w};
            float v[8];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = unpack2(w[e], d.x_dtype);
                v[2 * e] = f.x;
                v[2 * e + 1] = f.y;
            }
#pragma unroll
            for (int n = 0; n < N; ++n) {
                const float4 a = *reinterpret_cast<const float4*>(w_s + n * H + g * 8);
                const float4 b = *reinterpret_cast<const float4*>(w_s + n * H + g * 8 + 4);
                acc[n] = fmaf(v[0], a.x, acc[n]);
                acc[n] = fmaf(v[1], a.y, acc[n]);
                acc[n] = fmaf(v[2], a.z, acc[n]);
                acc[n] = fmaf(v[3], a.w, acc[n]);
                acc[n] = fmaf(v[4], b.x, acc[n]);
                acc[n] = fmaf(v[5], b.y, acc[n]);
                acc[n] = fmaf(v[6], b.z, acc[n]);
                acc[n] = fmaf(v[7], b.w, acc[n]);
            }
        }
#pragma unroll
        for (int n = 0; n < N; ++n) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc[n] += __shfl_xor_sync(0xffffffffu, acc[n], o);
        }
        if (lane == 0) {
#pragma unroll
            for (int n = 0; n < N; ++n) d.out[n * d.ld_out + t] = acc[n] + bias[n];
        }
    }
}

template <int N>
void launch_qa(const B200QAHeadDesc& d, cudaStream_t stream) {
    long long blocks = (d.M + 7) / 8;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long long cap = 4ll * sms;
    if (blocks > cap) blocks = cap;
    const size_t smem = static_cast<size_t>(d.H) * N * sizeof(float);
    launch_kernel(qa_head_kernel<N>, dim3(static_cast<unsigned>(blocks)), dim3(256), smem, stream, d);
}

}  // namespace
}  // namespace b200

extern "C" int b200_qa_head_fwd(const B200QAHeadDesc* d, b200_stream_t stream_) {
    using namespace b200;
    if (!d || d->M < 0 || d->H <= 0 || d->N <= 0) return B200_ERR_PARAM;
    if (d->M == 0 && d->N <= kHeadMaxN && (d->H % 8) == 0) return B200_OK;   // nothing to do: pointers may be null
    if (!d->x || !d->weight || !d->out) return B200_ERR_PARAM;
    if (!is_half_dtype(d->x_dtype)) return B200_ERR_PARAM;
    if ((d->H % 8) || (d->ldx % 8) || d->ldx < d->H || d->ld_out < d->M) return B200_ERR_PARAM;
    if (!aligned16(d->x)) return B200_ERR_PARAM;
    if (d->N > kHeadMaxN || d->H * d->N * 4 > 48 * 1024) return B200_ERR_UNSUPPORTED;
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
