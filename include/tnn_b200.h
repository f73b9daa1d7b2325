/*
 * tnn_b200 — C ABI of the B200 (sm_100a) kernels behind TNN's transformer-encoder attention path.
 *
 * Who calls this: the DEVICE_CUDA layer accs of the TNN plug-in (tnn_b200/tnn_plugin), one launcher per fused layer,
 * from `Init/Reshape/Forward`; and the Python/ctypes host mirror used by the tests and the benchmark.  Nothing here
 * takes a framework type: plain pointers, sizes and POD descriptor structs only.
 *
 * Conventions
 *   - every launcher enqueues on the given stream and returns immediately: no allocation, no synchronisation, no exit();
 *   - return value 0 = B200_OK, negative = error (b200_status_string() names it); the accs map it to a TNN `Status`
 *     (TNNERR_PARAM_ERR / TNNERR_CUDA_KERNEL_LAUNCH_ERROR, include/tnn/core/status.h:29-144) instead of the
 *     reference's abort-on-error CUDA_CHECK (source/tnn/device/cuda/cuda_macro.h:24-40);
 *   - device pointers are `(char*)BlobHandle.base + BlobHandle.bytes_offset` (include/tnn/core/blob.h:32-50);
 *   - activations are row-major `[tokens, features]` (a TNN blob `[B,S,H]` flattened over B and S);
 *   - kernels never spin unboundedly: a wait that runs out sets a bit in a per-device status word, the CTA tears
 *     down cleanly and b200_device_status() reports it after the stream is synchronised.
 */
#ifndef TNN_B200_H_
#define TNN_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define B200_API
#else
#define B200_API __attribute__((visibility("default")))
#endif

/* A CUDA stream handle (cudaStream_t) passed as an opaque pointer so that this header needs no CUDA header. */
typedef void* b200_stream_t;

enum {
    B200_OK                   = 0,
    B200_ERR_PARAM            = -1, /* null pointer, bad dtype, misaligned pointer or leading dimension            */
    B200_ERR_UNSUPPORTED      = -2, /* shape outside what the kernel handles (stated per entry point)              */
    B200_ERR_LAUNCH           = -3, /* cudaLaunch / cudaGetLastError reported an error                            */
    B200_ERR_DRIVER           = -4, /* tensor-map encode entry point missing or it refused the descriptor          */
    B200_ERR_DEVICE_TIMEOUT   = -5, /* reported by b200_device_status(): a bounded device-side wait ran out        */
    B200_ERR_NOT_SM100        = -6, /* the current device is not compute capability 10.x                           */
    B200_ERR_STATIC_LIMIT     = -7, /* b200_attention_masked_fwd_static: batch larger than its built-in scratch      */
    B200_ERR_INDEX            = -8  /* reported by b200_device_status(): an embedding index was outside its table      */
};

enum { B200_F16 = 0, B200_BF16 = 1, B200_F32 = 2 };

/* Epilogue of the projection GEMM; replaces the Add / GELU / Add layers that follow MatMul in the unfused graph. */
enum {
    B200_EPI_BIAS          = 0, /* y = x.W + b                       MatMul -> Add(bias)                              */
    B200_EPI_BIAS_GELU     = 1, /* y = gelu_erf(x.W + b)             MatMul -> Add(bias) -> GELU                      */
    B200_EPI_BIAS_RESIDUAL = 2, /* y = x.W + b + r                   MatMul -> Add(bias) -> Add(residual)             */
    B200_EPI_BIAS_TANH     = 3  /* y = tanh(x.W + b)                 MatMul -> Add(bias) -> Tanh  (the BERT pooler;    */
                                /*   source/tnn/device/x86/acc/x86_tanh_layer_acc.cc:19-31)                           */
};

/* -------------------------------------------------------------------------------------------------------------------
 * Weight pre-pack.  Replaces nothing in the reference's hot loop: TNN keeps MatMul weights as an fp32 `[K,N]`
 * RawBuffer (source/tnn/interpreter/layer_resource.h:165-169, y = x.W) and the x86 acc re-packs them on every call
 * (source/tnn/device/x86/acc/compute/jit/conv_sgemm_driver.cc:128-133); here it is done once at Init.
 * Reads fp32 `w_kn[K, N]` (row stride ld_src elements) and writes `dtype` `w_nk[N, K]` (row stride ld_dst elements),
 * i.e. transposed so that K is contiguous, rounding to nearest even.  Both pointers are device pointers.
 * To concatenate Q/K/V weights into one `[3H, K]` operand, call three times with dst offset by rows.
 */
B200_API int b200_pack_weight(const float* w_kn, int64_t K, int64_t N, int64_t ld_src, void* w_nk, int64_t ld_dst,
                              int dtype, b200_stream_t stream);

/* Weight pre-pack with a LayerNorm folded in (see B200LinearDesc: ln_in_stats).  For y = LN(x; gamma, beta).W + bias:
 *   w_nk[n, k] = round(gamma[k] * w_kn[k, n])           (dtype, [N, K] at row stride ld_dst)
 *   c1[n]      = sum_k float(w_nk[n, k])                 (the rounded values, so that the mean term cancels exactly)
 *   c2[n]      = sum_k beta[k] * w_kn[k, n] + bias[n]    (bias may be NULL)
 * One launch; c1, c2 are fp32 [N] device arrays. */
B200_API int b200_fold_layernorm_weight(const float* w_kn, int64_t K, int64_t N, int64_t ld_src, const float* gamma,
                                        const float* beta, const float* bias, void* w_nk, int64_t ld_dst, int dtype,
                                        float* c1, float* c2, b200_stream_t stream);

/* Element-wise dtype conversion of `n` contiguous elements (the fp32 <-> fp16/bf16 boundary of the fused region:
 * DefaultNetwork keeps every CUDA blob fp32, source/tnn/core/blob_manager.cc:101-117).  n*sizeof must keep both
 * pointers 16-byte aligned at their start. */
B200_API int b200_convert(const void* src, int src_dtype, void* dst, int dst_dtype, int64_t n, b200_stream_t stream);

/* -------------------------------------------------------------------------------------------------------------------
 * Projection / FFN GEMM with fused epilogue:  y[M,N] = epilogue(x[M,K] . w_nk[N,K]^T + bias[N] (+ residual[M,N])).
 * Replaces MatMulLayer (+ X86MatMulLayerAcc::DoForward, source/tnn/device/x86/acc/x86_mat_mul_layer_acc.cc:49-114;
 * the reference's CUDA MatMul acc is a batched GEMV only, source/tnn/device/cuda/acc/cuda_mat_mul_layer_acc.cu:181-249)
 * followed by the bias Add (source/tnn/device/x86/acc/x86_add_layer_acc.cc:66-92), and optionally GELU
 * (source/tnn/device/x86/acc/x86_gelu_layer_acc.cc:22-62, erf form) or the residual Add.
 * tcgen05 UMMA (fp32 accumulation in TMEM), operands by TMA into 128-byte-swizzled shared memory; tiles of 256 x BN
 * on pairs of SMs (cta_group::2) or 128 x BN on one SM.
 *   x, w_nk, residual : `dtype` (B200_F16 or B200_BF16); y : `out_dtype` (F16, BF16 or F32); bias : fp32 or NULL.
 *   Requirements: K % 8 == 0, ldx % 8 == 0, ldw % 8 == 0, x and w_nk 16-byte aligned; y/residual rows 16-byte aligned
 *   (N % 8 == 0, ldy % 8 == 0, ldr % 8 == 0).  M, N, K > 0 otherwise arbitrary (edge tiles are zero-filled/guarded).
 *   block_n: 0 = choose the tile; > 0 = tile width 64, 128, 192 (CTA-pair tiles only) or 256, on CTA-pair tiles
 *            (256 x block_n, two SMs per tile) when M > 128; < 0 = single-CTA tiles (128 x -block_n), for testing.
 */
typedef struct B200LinearDesc {
    const void*  x;
    const void*  w_nk;
    const float* bias;
    const void*  residual;
    void*        y;
    int64_t      M, N, K;
    int64_t      ldx, ldw, ldr, ldy;
    int32_t      dtype;
    int32_t      out_dtype;
    int32_t      epilogue;
    int32_t      block_n;
    /* ---- LayerNorm folding (all optional; zero-initialise the struct to leave it off) -------------------------------
     * The two LayerNorm layers of an encoder layer can be folded into the GEMMs around them, so that only the
     * PRE-LayerNorm activations t are ever written to HBM, together with per-row partial sums:
     *   row statistics: fp32 pairs (sum, sum of squares) per 32-column chunk, laid out [ceil(N/32)][M][2] ("slots").
     *   out_stats     : this GEMM writes the statistics of its output rows y (after residual), one slot per chunk.
     *   ln_in_stats   : x is a pre-LayerNorm activation with these statistics (K/32 slots of M rows).  w_nk must have
     *                   been packed with gamma folded in and ln_c1 / ln_c2 computed (b200_fold_layernorm_weight);
     *                   the kernel then evaluates LN(x).W + b as rstd*(x.W' - mean*c1) + c2.  `bias` is ignored.
     *   res_ln_stats  : the residual operand is a pre-LayerNorm activation with these statistics (N/32 slots); the
     *                   kernel adds LN(residual) = (r - mean)*rstd*res_ln_gamma + res_ln_beta instead of r.
     *   ln_eps        : epsilon of both normalisations.
     */
    float*       out_stats;
    const float* ln_in_stats;
    const float* ln_c1;
    const float* ln_c2;
    const float* res_ln_stats;
    const float* res_ln_gamma;
    const float* res_ln_beta;
    float        ln_eps;
    int32_t      reserved_;
} B200LinearDesc;
B200_API int b200_linear_fwd(const B200LinearDesc* desc, b200_stream_t stream);

/* -------------------------------------------------------------------------------------------------------------------
 * Fused multi-head attention:  out[b, q, h*D:(h+1)*D] = softmax_k(scale * Q_bh[q].K_bh[k] + mask_add[b,k]) . V_bh.
 * Replaces the unfused chain Reshape -> Permute -> MatMul(QK^T) -> Mul(scale) -> Add(mask) -> Softmax(axis 3) ->
 * MatMul(PV) -> Permute -> Reshape (source/tnn/layer/reshape_layer.cc:40-91, source/tnn/layer/permute_layer.cc:28-63,
 * source/tnn/device/x86/acc/x86_softmax_layer_acc.cc:28-83, source/tnn/device/x86/acc/x86_binary_op_layer_acc.cc:536-805).
 * The head split/merge is done by TMA coordinates; no [B,h,S,S] tensor ever reaches HBM.
 *   q, k, v : `dtype` (F16/BF16), token-major `[B, S, ld*]` with head h at columns h*64 .. h*64+63 (so a packed QKV
 *             activation `[B,S,3H]` is passed as q = base, k = base + H, v = base + 2H, ldq = ldk = ldv = 3H);
 *   mask_add: fp32 `[B, S]` additive key mask (0 valid, -10000 padded — TNN feeds it as a `[B,1,1,S]` blob) or NULL.
 *             A key whose mask value is <= mask_exclude_below gets weight exactly 0 (it is dropped, not merely
 *             down-weighted); other values are added to the scaled score.  A sequence with no key above the
 *             threshold is computed with purely additive semantics (what the reference's softmax yields then).
 *   kv_len  : int32 `[B]` = 1 + index of the last non-excluded key (from b200_mask_to_kv_len) or NULL (= S): whole
 *             key tiles at or beyond it are skipped.  Keys below kv_len are still tested one by one, so a mask with
 *             holes is exact.  When mask_add is given without kv_len, a sequence whose keys are all excluded yields
 *             zero rows (the additive fallback above needs kv_len to know about it).
 *   out     : `dtype` `[B, S, ldo]`.  Rows of padded queries are computed like any other row (as the reference does).
 *   Requirements: head_dim == 64; ld* % 8 == 0; pointers 16-byte aligned; S >= 1.
 */
typedef struct B200AttentionDesc {
    const void*    q;
    const void*    k;
    const void*    v;
    const float*   mask_add;
    const int32_t* kv_len;
    void*          out;
    int64_t        B, S;
    int64_t        ldq, ldk, ldv, ldo;
    int32_t        heads;
    int32_t        head_dim;
    int32_t        dtype;
    float          scale;
    float          mask_exclude_below;
} B200AttentionDesc;
B200_API int b200_attention_fwd(const B200AttentionDesc* desc, b200_stream_t stream);

/* Masked attention for callers that must not allocate.  (No counterpart in the reference: TNN's accs allocate their
 * temporaries freely, even inside Forward — source/tnn/device/cuda/cuda_context.cc:137-145.)
 *
 * b200_attention_fwd with a mask wants a kv_len array, and somebody has to own those B ints of device memory.  Some
 * hosts cannot provide them: an acc whose Forward is forbidden to allocate and was not given a workspace at Init, a
 * process running inside a fixed memory budget handed out once at start-up, a plug-in loaded into a server whose
 * allocator it may not touch.  This entry point takes the same descriptor (mask_add required, kv_len ignored),
 * derives kv_len on the device into a scratch array that is part of the library image — a static __device__ array
 * of B200_STATIC_MAX_BATCH int32 (16 KB, resident on every GPU that has loaded the library until the process
 * exits) — and then runs the same attention kernels.  It calls no cudaMalloc / cudaFree and no allocating routine,
 * on the device or on the host (its tensor maps live on the stack).
 *   - B > B200_STATIC_MAX_BATCH is refused with B200_ERR_STATIC_LIMIT; nothing is launched.
 *   - The first call on a device is the warm-up: it looks up the scratch array's device address
 *     (cudaGetSymbolAddress, with that device current) and sets the kernels' shared-memory attribute, under a host
 *     mutex so that two threads may make it at once; the CUDA runtime may also load the kernels' module on that first
 *     launch, which is the driver's business and outside this promise.  Make that call at start-up, before starting
 *     any stream capture on that device.  Later calls only launch (the status-word address and the driver's
 *     tensor-map encoder are looked up once per process behind a mutex / a function-local static; no memory is taken).
 *   - All calls on one GPU share the one scratch array.  Nothing in it needs clearing: each call overwrites the B
 *     entries it then reads, and entries beyond B are never read.  Two calls whose kernels can overlap on the GPU
 *     (different streams without an ordering between them) race on it: keep such calls on one stream, or order them.
 */
#define B200_STATIC_MAX_BATCH 4096
B200_API int b200_attention_masked_fwd_static(const B200AttentionDesc* desc, b200_stream_t stream);

/* kv_len[b] = 1 + max{k : mask_add[b,k] > exclude_below}, 0 if there is none.  The mask is a run-time input of the
 * graph, so this runs on the device once per Forward. */
B200_API int b200_mask_to_kv_len(const float* mask_add, int64_t B, int64_t S, float exclude_below, int32_t* kv_len,
                                 b200_stream_t stream);

/* -------------------------------------------------------------------------------------------------------------------
 * The step in front of the encoder path: embedding lookups + LayerNorm, and the additive key mask from the 0/1 input
 * mask.  Replaces, in a converted BERT graph, Gather(word) + Gather(segment) -> Add -> Add(position slice) ->
 * LayerNorm (source/tnn/device/x86/acc/x86_gather_layer_acc.cc:23-76, x86_add_layer_acc.cc:66-92,
 * x86_layer_norm_layer_acc.cc:26-86) and Unsqueeze -> Cast -> Sub -> Mul on the mask
 * (source/tnn/device/x86/acc/x86_binary_op_layer_acc.cc:536-805); int32 graph inputs as the reference's tokenizer
 * produces them (examples/base/bert_tokenizer.cc:351-355).
 *   out[t, :] = LayerNorm(word_emb[input_ids[t]] + type_emb[segment_ids[t]] + pos_emb[t mod S]) * gamma + beta
 *   tables    : `table_dtype` (F32, F16 or BF16) `[rows, H]` with row stride ld_table (elements); type_emb and
 *               segment_ids may both be NULL; pos_emb needs at least S rows.
 *   out       : `out_dtype` (F16/BF16/F32) `[B*S, ld_out]`.   Requirements: H % 8 == 0, H <= 1024, 16-byte aligned.
 *   An index outside its table makes the reference's Gather fail (TNNERR_MODEL_ERR); here the row is written as
 *   LayerNorm of the remaining terms with that term 0, and b200_device_status() reports B200_ERR_INDEX.
 */
typedef struct B200EmbeddingDesc {
    const int32_t* input_ids;
    const int32_t* segment_ids;
    const void*    word_emb;
    const void*    type_emb;
    const void*    pos_emb;
    const float*   gamma;
    const float*   beta;
    void*          out;
    int64_t        B, S, H;
    int64_t        vocab, type_vocab;
    int64_t        ld_table, ld_out;
    int32_t        table_dtype;
    int32_t        out_dtype;
    float          eps;
} B200EmbeddingDesc;
B200_API int b200_embedding_layernorm_fwd(const B200EmbeddingDesc* desc, b200_stream_t stream);

/* mask_add[b, s] = (1 - input_mask[b, s]) * masked_value (fp32, the reference's Sub and Mul; masked_value = -10000 in
 * BERT exports) and, if kv_len is not NULL, kv_len[b] = 1 + the last s with mask_add[b, s] > exclude_below — the two
 * arrays b200_attention_fwd takes.  input_mask: int32 `[B, S]`. */
B200_API int b200_mask_from_input_mask(const int32_t* input_mask, int64_t B, int64_t S, float masked_value,
                                       float exclude_below, float* mask_add, int32_t* kv_len, b200_stream_t stream);

/* -------------------------------------------------------------------------------------------------------------------
 * Span-extraction (question answering) head: logits = x . W + b with very few outputs per token (start, end), then
 * "unstack": output n of every token as its own contiguous array.  Replaces MatMul (constant weight [H, N],
 * source/tnn/device/x86/acc/x86_mat_mul_layer_acc.cc:49) + Add(bias) + SplitV (x86_splitv_layer_acc.cc:23) +
 * Squeeze (x86_squeeze_layer_acc.cc:23) at the end of the reading-comprehension graph, whose outputs the demo reads as
 * "unstack:0" / "unstack:1" (examples/linux/src/BertReadingComprehension/BertReadingComprehension.cc:109).
 *   x      : [M, H] half precision (x_dtype F16/BF16), row stride ldx (multiple of 8), 16-byte aligned
 *   weight : fp32 [H, N] row-major (the MatMul layer's constant), bias : fp32 [N] or NULL,  1 <= N <= 4
 *   out    : fp32, output n of token t at out[n * ld_out + t]  (ld_out >= M)
 * fp32 accumulation; HBM-bound (one read of x). */
typedef struct B200QAHeadDesc {
    const void* x;
    const float* weight;
    const float* bias;
    float* out;
    int64_t M, H;
    int64_t ldx, ld_out;
    int32_t N;
    int32_t x_dtype;
    /* Optional: one destination per output.  If out_n[0] is not NULL, output n of token t goes to out_n[n][t] for every
     * n < N (all N pointers must be set; `out` and `ld_out` are then ignored), so that a caller whose outputs are
     * separate buffers — the two output blobs of the TNN graph — needs no copy behind the kernel. */
    float* out_n[4];
} B200QAHeadDesc;
B200_API int b200_qa_head_fwd(const B200QAHeadDesc* desc, b200_stream_t stream);

/* -------------------------------------------------------------------------------------------------------------------
 * (residual +) LayerNorm over the last dimension:  y = (x (+ r) - mean) * rsqrt(var + eps) * gamma + beta.
 * Replaces Add(residual) + LayerNorm (source/tnn/device/x86/acc/x86_layer_norm_layer_acc.cc:26-86; gamma and beta are
 * the layer's input blobs 1 and 2, source/tnn/layer/layer_norm_layer.cc:28-30).  One warp per row, fp32 statistics,
 * variance as the mean of squared deviations (the reference's one-pass E[x^2]-mean^2 agrees to fp32 rounding).
 *   x, residual : in_dtype (F16/BF16/F32), residual may be NULL;  y : out_dtype;  gamma, beta : fp32 [H].
 *   Requirements: H % 8 == 0, H <= 4096, leading dimensions % 8 == 0, 16-byte aligned pointers.
 */
typedef struct B200LayerNormDesc {
    const void*  x;
    const void*  residual;
    const float* gamma;
    const float* beta;
    void*        y;
    int64_t      rows, H;
    int64_t      ldx, ldr, ldy;
    int32_t      in_dtype;
    int32_t      out_dtype;
    float        eps;
} B200LayerNormDesc;
B200_API int b200_add_layernorm_fwd(const B200LayerNormDesc* desc, b200_stream_t stream);

/* -------------------------------------------------------------------------------------------------------------------
 * One post-LN transformer-encoder layer (the fused form of the ~30 TNN layers of one BERT layer) and a whole encoder
 * stack, as a fixed sequence of the launchers above.  All buffers are the caller's.
 *   hidden  : `dtype` [tokens, H]   in/out (stack input, overwritten with the stack output)
 *   w_qkv   : [3H, H] packed, b_qkv fp32 [3H];  w_o : [H, H];  w_ffn1 : [F, H];  w_ffn2 : [H, F]  (all `[N,K]` packed)
 *   workspace: b200_encoder_workspace_bytes(tokens, H, F, dtype) bytes, 256-byte aligned.
 * fold_layernorm = 0: seven launches per layer (QKV, attention, out-proj+residual, LayerNorm, FFN1+GELU,
 *   FFN2+residual, LayerNorm).  The fastest form measured at 64 x 128 tokens.
 * fold_layernorm = 1: five launches per layer; both LayerNorms are folded into the neighbouring GEMMs (see
 *   B200LinearDesc) and only pre-LayerNorm activations are written.  The weights must then have been prepared with
 *   b200_fold_layernorm_weight: w_ffn1/ffn1_c1/ffn1_c2 from (W1, ln1 gamma/beta, b1) of the same layer, and for every
 *   layer but the first w_qkv/qkv_c1/qkv_c2 from (Wqkv, ln2 gamma/beta of the PREVIOUS layer, b_qkv).  One LayerNorm
 *   launch after the last layer produces the stack output.
 */
typedef struct B200EncoderLayerWeights {
    const void*  w_qkv;  const float* b_qkv;
    const void*  w_o;    const float* b_o;
    const float* ln1_gamma; const float* ln1_beta;
    const void*  w_ffn1; const float* b_ffn1;
    const void*  w_ffn2; const float* b_ffn2;
    const float* ln2_gamma; const float* ln2_beta;
    const float* qkv_c1;  const float* qkv_c2;     /* fold_layernorm == 1 only, layers > 0 */
    const float* ffn1_c1; const float* ffn1_c2;    /* fold_layernorm == 1 only */
} B200EncoderLayerWeights;

typedef struct B200EncoderDesc {
    void*                          hidden;
    const float*                   mask_add;   /* [B,S] or NULL */
    const int32_t*                 kv_len;     /* [B] or NULL   */
    const B200EncoderLayerWeights* layers;     /* host array of num_layers entries */
    void*                          workspace;
    int64_t                        B, S, H, F;
    int32_t                        heads;
    int32_t                        num_layers;
    int32_t                        dtype;
    float                          ln_eps;
    float                          mask_exclude_below;
    int32_t                        fold_layernorm;
} B200EncoderDesc;
B200_API size_t b200_encoder_workspace_bytes(int64_t tokens, int64_t H, int64_t F, int dtype);
B200_API int    b200_encoder_fwd(const B200EncoderDesc* desc, b200_stream_t stream);

/* -------------------------------------------------------------------------------------------------------------------
 * Housekeeping. */
B200_API const char* b200_status_string(int status);
/* Reads and clears the current device's status word (synchronous, small).  0, B200_ERR_DEVICE_TIMEOUT or
 * B200_ERR_INDEX (a timeout takes precedence). */
B200_API int         b200_device_status(void);
/* The same without blocking the host: enqueues a copy of the current device's raw status word into *host_word (page-
 * locked host memory, so that the copy is asynchronous) behind the work already in `stream`.  Once the stream has been
 * synchronised, b200_decode_status_word(*host_word) gives the status; the device word is NOT cleared (a non-zero word
 * is cleared by calling b200_device_status()). */
B200_API int         b200_device_status_async(unsigned int* host_word, b200_stream_t stream);
B200_API int         b200_decode_status_word(unsigned int word);
/* Number of kernel launches issued by this library in this process (all devices, all threads). */
B200_API uint64_t    b200_launch_count(void);
B200_API const char* b200_version(void);
/* Self-test of the tensor-map (TMA descriptor) cache the launchers share: `threads` host threads look maps up while
 * the cache, limited to `capacity` entries for the test, keeps evicting; a stand-in replaces the driver's encoder, so
 * no GPU or driver is needed.  Returns the number of maps that came back wrong (0 = pass) or B200_ERR_PARAM. */
/* Self-test of the bounded-wait convention: launches one warp that waits on a barrier nobody arrives at, with a limit
 * of 1024 polls (milliseconds at most); it gives up, sets the time-out bit of the status word and returns, so that
 * after a synchronise b200_device_status() reports B200_ERR_DEVICE_TIMEOUT (and clears it) and the device carries on
 * as before.  This is how every wait in the kernels ends when its partner never shows up; nothing traps or hangs. */
B200_API int         b200_selftest_bounded_wait(b200_stream_t stream);
B200_API int         b200_selftest_tensor_map_cache(int threads, int maps_per_thread, int capacity);

#ifdef __cplusplus
}
#endif
#endif /* TNN_B200_H_ */
