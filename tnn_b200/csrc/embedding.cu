// The step in front of the encoder path: embedding lookups + LayerNorm, and the additive key mask / kv_len from the
// 0/1 input mask.  HBM-bound gather kernels: per token 3 table rows in, one row out; algorithmic bytes per token
// H * (3 * table element size + output element size).
#include "common.cuh"
#include "ptx.cuh"

namespace b200 {
namespace {

// 8 consecutive elements of a table row as fp32
__device__ __forceinline__ void load_row8(const void* base, long long elem_off, int dtype, float (&v)[8]) {
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

// One warp per token; a lane holds NV groups of 8 consecutive elements (group g of the lane = elements
// (g*32 + lane)*8 ..).  Sum order as in the unfused graph: (word + segment) + position; LayerNorm arithmetic as in
// add_layernorm_rows_kernel (fp32 mean, fp32 mean of squared deviations).
template <int NV>
__global__ void __launch_bounds__(256) embedding_layernorm_kernel(B200EmbeddingDesc d, unsigned int* status) {
    const int lane = threadIdx.x & 31;
    const long long tokens = d.B * d.S;
    const long long warp0 = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    const long long nwarps = static_cast<long long>(gridDim.x) * 8;
    const int groups = static_cast<int>(d.H >> 3);
    const float inv_h = 1.0f / static_cast<float>(d.H);
    pdl_launch_dependents();
    pdl_wait();
    for (long long t = warp0; t < tokens; t += nwarps) {
        const int id = d.input_ids[t];
        const int seg = d.segment_ids ? d.segment_ids[t] : 0;
        const bool id_ok = id >= 0 && id < d.vocab;
        const bool seg_ok = d.type_emb == nullptr || (seg >= 0 && seg < d.type_vocab);
        if ((!id_ok || !seg_ok) && lane == 0 && status != nullptr) atomicOr(status, 8u);
        const long long pos = t % d.S;
        float v[NV][8];
        float sum = 0.f;
#pragma unroll
        for (int g = 0; g < NV; ++g) {
            const int gi = g * 32 + lane;
            if (gi < groups) {
                float w[8], s[8], p[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) w[e] = s[e] = 0.f;
                if (id_ok) load_row8(d.word_emb, id * d.ld_table + gi * 8, d.table_dtype, w);
                if (d.type_emb != nullptr && seg_ok) load_row8(d.type_emb, seg * d.ld_table + gi * 8, d.table_dtype, s);
                load_row8(d.pos_emb, pos * d.ld_table + gi * 8, d.table_dtype, p);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    v[g][e] = (w[e] + s[e]) + p[e];
                    sum += v[g][e];
                }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
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
                load_row8(d.gamma, gi * 8, B200_F32, gm);
                load_row8(d.beta, gi * 8, B200_F32, bt);
#pragma unroll
                for (int e = 0; e < 8; ++e) o[e] = (v[g][e] - mean) * rstd * gm[e] + bt[e];
                if (d.out_dtype == B200_F32) {
                    float4* q = reinterpret_cast<float4*>(reinterpret_cast<float*>(d.out) + t * d.ld_out + gi * 8);
                    q[0] = make_float4(o[0], o[1], o[2], o[3]);
                    q[1] = make_float4(o[4], o[5], o[6], o[7]);
                } else {
                    uint4 q;
                    q.x = pack2(o[0], o[1], d.out_dtype);
                    q.y = pack2(o[2], o[3], d.out_dtype);
                    q.z = pack2(o[4], o[5], d.out_dtype);
                    q.w = pack2(o[6], o[7], d.out_dtype);
                    *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(d.out) + t * d.ld_out + gi * 8) = q;
                }
            }
        }
    }
}

// One block per sequence: mask_add = (1 - m) * masked_value, kv_len = 1 + last key above the threshold.
__global__ void __launch_bounds__(128) mask_from_input_mask_kernel(const int32_t* input_mask, long long S,
                                                                   float masked_value, float below, float* mask_add,
                                                                   int* kv_len) {
    const long long b = blockIdx.x;
    int last = 0;
    pdl_launch_dependents();
    pdl_wait();
    for (long long k = threadIdx.x; k < S; k += blockDim.x) {
        const float a = (1.0f - static_cast<float>(input_mask[b * S + k])) * masked_value;
        mask_add[b * S + k] = a;
        if (a > below) last = static_cast<int>(k) + 1;
    }
    if (kv_len == nullptr) return;
    __shared__ int red[4];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) last = max(last, __shfl_xor_sync(0xffffffffu, last, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = last;
    __syncthreads();
    if (threadIdx.x == 0) kv_len[b] = max(max(red[0], red[1]), max(red[2], red[3]));
}

bool any_dtype(int dt) { return dt == B200_F16 || dt == B200_BF16 || dt == B200_F32; }

}  // namespace
}  // namespace b200

extern "C" {

int b200_embedding_layernorm_fwd(const B200EmbeddingDesc* d, b200_stream_t stream_) {
    using namespace b200;
    if (!d || !d->input_ids || !d->word_emb || !d->pos_emb || !d->gamma || !d->beta || !d->out) return B200_ERR_PARAM;
    if ((d->type_emb == nullptr) != (d->segment_ids == nullptr)) return B200_ERR_PARAM;
    if (d->B < 0 || d->S <= 0 || d->H <= 0 || d->vocab <= 0) return B200_ERR_PARAM;
    if (d->type_emb && d->type_vocab <= 0) return B200_ERR_PARAM;
    if (!any_dtype(d->table_dtype) || !any_dtype(d->out_dtype)) return B200_ERR_PARAM;
    if ((d->H % 8) || (d->ld_table % 8) || (d->ld_out % 8) || d->ld_table < d->H || d->ld_out < d->H) return B200_ERR_PARAM;
    if (!aligned16(d->word_emb) || !aligned16(d->pos_emb) || !aligned16(d->out) || !aligned16(d->gamma) ||
        !aligned16(d->beta) || (d->type_emb && !aligned16(d->type_emb)))
        return B200_ERR_PARAM;
    if (d->H > 1024) return B200_ERR_UNSUPPORTED;
    const long long tokens = d->B * d->S;
    if (tokens == 0) return B200_OK;
    if (tokens > (1ll << 31) - 1) return B200_ERR_UNSUPPORTED;
    long long blocks = (tokens + 7) / 8;
    if (blocks > 148ll * 8) blocks = 148ll * 8;
    const dim3 grid(static_cast<unsigned>(blocks)), block(256);
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    unsigned int* status = device_status_ptr();
    const int nv = static_cast<int>((d->H / 8 + 31) / 32);
    if (nv <= 1) launch_kernel(embedding_layernorm_kernel<1>, grid, block, 0, stream, *d, status);
    else if (nv <= 3) launch_kernel(embedding_layernorm_kernel<3>, grid, block, 0, stream, *d, status);
    else launch_kernel(embedding_layernorm_kernel<4>, grid, block, 0, stream, *d, status);
    count_launch();
    return check_launch();
}

int b200_mask_from_input_mask(const int32_t* input_mask, int64_t B, int64_t S, float masked_value, float exclude_below,
                              float* mask_add, int32_t* kv_len, b200_stream_t stream_) {
    using namespace b200;
    if (!input_mask || !mask_add || B < 0 || S <= 0) return B200_ERR_PARAM;
    if (B == 0) return B200_OK;
    if (B > (1ll << 31) - 1) return B200_ERR_UNSUPPORTED;
    launch_kernel(mask_from_input_mask_kernel, dim3(static_cast<unsigned>(B)), dim3(128), 0,
                  static_cast<cudaStream_t>(stream_), input_mask, static_cast<long long>(S), masked_value,
                  exclude_below, mask_add, kv_len);
    count_launch();
    return check_launch();
}

}  // extern "C"
