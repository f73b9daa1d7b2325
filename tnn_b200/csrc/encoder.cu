// One post-LN transformer-encoder layer as seven launches, and a stack of them.  This is the launch sequence the
// fused TNN graph executes (FusedLinear(QKV) -> FusedAttention -> FusedLinear(+residual) -> LayerNorm ->
// FusedLinear(+GELU) -> FusedLinear(+residual) -> LayerNorm), offered as one call for hosts that hold the weights
// themselves.  Everything is enqueued on the caller's stream; nothing is allocated or synchronised.
#include "common.cuh"

namespace {

inline size_t align256(size_t x) { return (x + 255) & ~static_cast<size_t>(255); }

struct Workspace {
    char *qkv, *ctx, *tmp, *h1, *ffn;
    float *stats1, *stats2;   // row statistics of the two pre-LayerNorm activations (fold_layernorm == 1)
    size_t total;
};

Workspace carve(char* base, int64_t tokens, int64_t H, int64_t F, int dtype) {
    const size_t es = b200::dtype_size(dtype);
    Workspace w;
    size_t off = 0;
    w.qkv = base + off; off += align256(static_cast<size_t>(tokens) * 3 * H * es);
    w.ctx = base + off; off += align256(static_cast<size_t>(tokens) * H * es);
    w.tmp = base + off; off += align256(static_cast<size_t>(tokens) * H * es);
    w.h1 = base + off;  off += align256(static_cast<size_t>(tokens) * H * es);
    w.ffn = base + off; off += align256(static_cast<size_t>(tokens) * F * es);
    const size_t stats_bytes = align256(static_cast<size_t>((H + 31) / 32) * tokens * 2 * sizeof(float));
    w.stats1 = reinterpret_cast<float*>(base + off); off += stats_bytes;
    w.stats2 = reinterpret_cast<float*>(base + off); off += stats_bytes;
    w.total = off;
    return w;
}

}  // namespace

extern "C" {

size_t b200_encoder_workspace_bytes(int64_t tokens, int64_t H, int64_t F, int dtype) {
    if (tokens <= 0 || H <= 0 || F <= 0) return 0;
    return carve(nullptr, tokens, H, F, dtype).total;
}

int b200_encoder_fwd(const B200EncoderDesc* d, b200_stream_t stream) {
    if (!d || !d->hidden || !d->layers || !d->workspace) return B200_ERR_PARAM;
    if (d->B <= 0 || d->S <= 0 || d->H <= 0 || d->F <= 0 || d->heads <= 0 || d->num_layers < 0) return B200_ERR_PARAM;
    if (d->H != static_cast<int64_t>(d->heads) * 64) return B200_ERR_UNSUPPORTED;
    if (!b200::is_half_dtype(d->dtype)) return B200_ERR_PARAM;
    if (reinterpret_cast<uintptr_t>(d->workspace) & 255u) return B200_ERR_PARAM;
    const int64_t tokens = d->B * d->S;
    const int64_t H = d->H, F = d->F;
    const Workspace w = carve(static_cast<char*>(d->workspace), tokens, H, F, d->dtype);

    if (d->fold_layernorm == 1) {
        // Five launches per layer.  t1 (= w.tmp) and t2 (= w.h1) hold the PRE-LayerNorm activations; stats1 / stats2
        // their row statistics.  The stack input is a plain activation, so the first layer's QKV projection and
        // out-projection residual are unfolded.
        const size_t es = b200::dtype_size(d->dtype);
        for (int l = 0; l < d->num_layers; ++l) {
            const B200EncoderLayerWeights& lw = d->layers[l];
            const bool first = l == 0;
            const B200EncoderLayerWeights* prev = first ? nullptr : &d->layers[l - 1];
            int rc;
            B200LinearDesc lin = {};
            lin.dtype = d->dtype;
            lin.out_dtype = d->dtype;
            lin.M = tokens;
            lin.ln_eps = d->ln_eps;

            // QKV projection of LN2(t2) (of the stack input for the first layer)
            lin.x = first ? d->hidden : static_cast<const void*>(w.h1); lin.ldx = H; lin.K = H;
            lin.w_nk = lw.w_qkv; lin.ldw = H; lin.bias = lw.b_qkv;
            lin.y = w.qkv; lin.N = 3 * H; lin.ldy = 3 * H;
            lin.epilogue = B200_EPI_BIAS;
            if (!first) {
                if (!lw.qkv_c1 || !lw.qkv_c2) return B200_ERR_PARAM;
                lin.ln_in_stats = w.stats2; lin.ln_c1 = lw.qkv_c1; lin.ln_c2 = lw.qkv_c2;
            }
            if ((rc = b200_linear_fwd(&lin, stream)) != B200_OK) return rc;

            B200AttentionDesc at = {};
            at.q = w.qkv; at.k = w.qkv + H * es; at.v = w.qkv + 2 * H * es;
            at.ldq = at.ldk = at.ldv = 3 * H;
            at.mask_add = d->mask_add; at.kv_len = d->kv_len;
            at.out = w.ctx; at.ldo = H;
            at.B = d->B; at.S = d->S; at.heads = d->heads; at.head_dim = 64; at.dtype = d->dtype;
            at.scale = 0.125f; at.mask_exclude_below = d->mask_exclude_below;
            if ((rc = b200_attention_fwd(&at, stream)) != B200_OK) return rc;

            // t1 = ctx.Wo + bo + LN2_prev(t2)   (+ statistics of t1)
            lin = B200LinearDesc{};
            lin.dtype = d->dtype; lin.out_dtype = d->dtype; lin.M = tokens; lin.ln_eps = d->ln_eps;
            lin.x = w.ctx; lin.ldx = H; lin.K = H;
            lin.w_nk = lw.w_o; lin.ldw = H; lin.bias = lw.b_o;
            lin.y = w.tmp; lin.N = H; lin.ldy = H;
            lin.epilogue = B200_EPI_BIAS_RESIDUAL; lin.ldr = H;
            if (first) {
                lin.residual = d->hidden;
            } else {
                lin.residual = w.h1;
                lin.res_ln_stats = w.stats2; lin.res_ln_gamma = prev->ln2_gamma; lin.res_ln_beta = prev->ln2_beta;
            }
            lin.out_stats = w.stats1;
            if ((rc = b200_linear_fwd(&lin, stream)) != B200_OK) return rc;

            // ffn = gelu(LN1(t1).W1 + b1)
            if (!lw.ffn1_c1 || !lw.ffn1_c2) return B200_ERR_PARAM;
            lin = B200LinearDesc{};
            lin.dtype = d->dtype; lin.out_dtype = d->dtype; lin.M = tokens; lin.ln_eps = d->ln_eps;
            lin.x = w.tmp; lin.ldx = H; lin.K = H;
            lin.w_nk = lw.w_ffn1; lin.ldw = H;
            lin.y = w.ffn; lin.N = F; lin.ldy = F;
            lin.epilogue = B200_EPI_BIAS_GELU;
            lin.ln_in_stats = w.stats1; lin.ln_c1 = lw.ffn1_c1; lin.ln_c2 = lw.ffn1_c2;
            if ((rc = b200_linear_fwd(&lin, stream)) != B200_OK) return rc;

            // t2 = ffn.W2 + b2 + LN1(t1)   (+ statistics of t2)
            lin = B200LinearDesc{};
            lin.dtype = d->dtype; lin.out_dtype = d->dtype; lin.M = tokens; lin.ln_eps = d->ln_eps;
            lin.x = w.ffn; lin.ldx = F; lin.K = F;
            lin.w_nk = lw.w_ffn2; lin.ldw = F; lin.bias = lw.b_ffn2;
            lin.y = w.h1; lin.N = H; lin.ldy = H;
            lin.epilogue = B200_EPI_BIAS_RESIDUAL; lin.residual = w.tmp; lin.ldr = H;
            lin.res_ln_stats = w.stats1; lin.res_ln_gamma = lw.ln1_gamma; lin.res_ln_beta = lw.ln1_beta;
            lin.out_stats = w.stats2;
            if ((rc = b200_linear_fwd(&lin, stream)) != B200_OK) return rc;
        }
        if (d->num_layers > 0) {
            const B200EncoderLayerWeights& last = d->layers[d->num_layers - 1];
            B200LayerNormDesc ln = {};
            ln.x = w.h1; ln.gamma = last.ln2_gamma; ln.beta = last.ln2_beta; ln.y = d->hidden;
            ln.rows = tokens; ln.H = H; ln.ldx = H; ln.ldy = H;
            ln.in_dtype = d->dtype; ln.out_dtype = d->dtype; ln.eps = d->ln_eps;
            const int rc = b200_add_layernorm_fwd(&ln, stream);
            if (rc != B200_OK) return rc;
        }
        return B200_OK;
    }

    // fold_layernorm == 0: the two LayerNorms as separate launches (seven launches per layer).
    for (int l = 0; l < d->num_layers; ++l) {
        const B200EncoderLayerWeights& lw = d->layers[l];
        int rc;

        B200LinearDesc lin = {};
        lin.dtype = d->dtype;
        lin.out_dtype = d->dtype;
        lin.M = tokens;
        lin.ln_eps = d->ln_eps;

        // 1. packed QKV projection
        lin.x = d->hidden; lin.ldx = H; lin.K = H;
        lin.w_nk = lw.w_qkv; lin.ldw = H; lin.bias = lw.b_qkv;
        lin.y = w.qkv; lin.N = 3 * H; lin.ldy = 3 * H;
        lin.epilogue = B200_EPI_BIAS; lin.residual = nullptr; lin.ldr = 0;
        if ((rc = b200_linear_fwd(&lin, stream)) != B200_OK) return rc;

        // 2. attention
        B200AttentionDesc at = {};
        const size_t es = b200::dtype_size(d->dtype);
        at.q = w.qkv; at.k = w.qkv + H * es; at.v = w.qkv + 2 * H * es;
        at.ldq = at.ldk = at.ldv = 3 * H;
        at.mask_add = d->mask_add; at.kv_len = d->kv_len;
        at.out = w.ctx; at.ldo = H;
        at.B = d->B; at.S = d->S; at.heads = d->heads; at.head_dim = 64; at.dtype = d->dtype;
        at.scale = 0.125f; at.mask_exclude_below = d->mask_exclude_below;
        if ((rc = b200_attention_fwd(&at, stream)) != B200_OK) return rc;

        // 3. output projection + residual
        lin.x = w.ctx; lin.ldx = H; lin.K = H;
        lin.w_nk = lw.w_o; lin.ldw = H; lin.bias = lw.b_o;
        lin.y = w.tmp; lin.N = H; lin.ldy = H;
        lin.epilogue = B200_EPI_BIAS_RESIDUAL; lin.residual = d->hidden; lin.ldr = H;
        if ((rc = b200_linear_fwd(&lin, stream)) != B200_OK) return rc;

        B200LayerNormDesc ln = {};
        ln.x = w.tmp; ln.residual = nullptr; ln.gamma = lw.ln1_gamma; ln.beta = lw.ln1_beta; ln.y = w.h1;
        ln.rows = tokens; ln.H = H; ln.ldx = H; ln.ldr = 0; ln.ldy = H;
        ln.in_dtype = d->dtype; ln.out_dtype = d->dtype; ln.eps = d->ln_eps;
        if ((rc = b200_add_layernorm_fwd(&ln, stream)) != B200_OK) return rc;   // 4. LayerNorm 1

        // 5. FFN up-projection + GELU
        lin.x = w.h1; lin.ldx = H; lin.K = H;
        lin.w_nk = lw.w_ffn1; lin.ldw = H; lin.bias = lw.b_ffn1;
        lin.y = w.ffn; lin.N = F; lin.ldy = F;
        lin.epilogue = B200_EPI_BIAS_GELU; lin.residual = nullptr; lin.ldr = 0;
        if ((rc = b200_linear_fwd(&lin, stream)) != B200_OK) return rc;

        // 6. FFN down-projection + residual
        lin.x = w.ffn; lin.ldx = F; lin.K = F;
        lin.w_nk = lw.w_ffn2; lin.ldw = F; lin.bias = lw.b_ffn2;
        lin.y = w.tmp; lin.N = H; lin.ldy = H;
        lin.epilogue = B200_EPI_BIAS_RESIDUAL; lin.residual = w.h1; lin.ldr = H;
        if ((rc = b200_linear_fwd(&lin, stream)) != B200_OK) return rc;

        // 7. LayerNorm 2 -> layer output
        ln.x = w.tmp; ln.gamma = lw.ln2_gamma; ln.beta = lw.ln2_beta; ln.y = d->hidden;
        if ((rc = b200_add_layernorm_fwd(&ln, stream)) != B200_OK) return rc;
    }
    return B200_OK;
}

}  // extern "C"
