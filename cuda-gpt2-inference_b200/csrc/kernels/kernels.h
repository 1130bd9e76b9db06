// Internal launchers: each validates nothing (the C-ABI layer does) and enqueues kernels on
// ctx->stream, bumping ctx->launches once per kernel launch.
#pragma once
#include <utility>
#include "../api/ctx.h"

namespace b200 {

// flags for the row-wise producers
// OUT_BF16: the main output pointer addresses bf16 (16-bit) elements instead of fp32
// OUT_BF16X2: two bf16 planes instead, hi = bf16(y) at the pointer and lo = bf16(y - hi) one whole
// output (rows x C elements) further on
enum : int { ROUND_OUT_TF32 = 1, OUT_BF16 = 2, OUT_BF16X2 = 4 };

int launch_layernorm(b200_ctx* ctx, float* out, float* mean, float* rstd, const float* inp,
                     const float* weight, const float* bias, int M, int C, int flags);
int launch_fused_residual_layernorm(b200_ctx* ctx, float* res_out, float* ln_out, float* mean,
                                    float* rstd, const float* inp1, const float* inp2,
                                    const float* weight, const float* bias, int M, int C, int flags, const float* inp3 = nullptr);  // inp3: x = inp1 + (inp2 + inp3)
// hand-over words between two GPUs (peer-mapped memory): see rowwise.cu
int launch_peer_signal(b200_ctx* ctx, unsigned int* peer_word, unsigned int value);
int launch_peer_wait(b200_ctx* ctx, const unsigned int* my_word, unsigned int value, unsigned long long limit_ns = 0);  // 0: the 2 s of every device-side wait
int launch_peer_signal_many(b200_ctx* ctx, unsigned int* const* peer_words, int n, unsigned int value);  // null entries are skipped
int launch_peer_wait_many(b200_ctx* ctx, const unsigned int* my_words, int n, int skip, unsigned int value);  // words 0..n-1 but `skip`
// layernorm of this rank's rows over the sum of n partial sums, written to every rank's output (rowwise.cu: LnSpArgs)
int launch_layernorm_sp(b200_ctx* ctx, float* residual, const float* parts, float* const* dst, int n, int rows, int row0,
                        const float* weight, const float* bias, int M, int C, int flags);
int launch_residual(b200_ctx* ctx, float* out, const float* a, const float* b, size_t N);
int launch_gelu(b200_ctx* ctx, float* out, const float* inp, size_t N);
int launch_encoder(b200_ctx* ctx, float* out, const int* tok, const float* wte, const float* wpe,
                   int B, int T, int C, int vocab_rows /* <=0: unchecked */);
int launch_round_tf32_inplace(b200_ctx* ctx, float* data, size_t N);
// dst[0..n) = src_view[0..n): src_view is the device view of a pinned host buffer (16-byte aligned)
int launch_fetch_ints(b200_ctx* ctx, int* dst, const int* src_view, int n);
// out[i] = bf16(in[i]), round to nearest even; N a multiple of 4.  lo (may be null): lo[i] = bf16(in[i] - out[i])
int launch_convert_bf16(b200_ctx* ctx, uint16_t* out, const float* in, size_t N, uint16_t* lo = nullptr);
// hi[i] = fp16(clamp(in[i])), lo[i] = fp16(in[i] - hi[i]); N a multiple of 4
int launch_split_fp16(b200_ctx* ctx, uint16_t* hi, uint16_t* lo, const float* in, size_t N);
// out[i] = e4m3(in[i] * scale), round to nearest even, saturating at +-448 (N a multiple of 4)
int launch_quantize_e4m3(b200_ctx* ctx, uint8_t* out, const float* in, size_t N, float scale);
int launch_argmax_rows(b200_ctx* ctx, int* out, const float* logits, int M, int V, int ld);
// one draw per row from softmax(logits / temperature) (Gumbel-max; temperature <= 0: arg-max);
// row r uses the noise stream stream0 + r of the seed; 0 < top_k < V: only among the top_k largest logits;
// 0 < top_p < 1: then only the most likely columns that add up to top_p of the probability
int launch_sample_rows(b200_ctx* ctx, int* out, const float* logits, int M, int V, int ld, float temperature,
                       unsigned int seed, unsigned int stream0, int top_k = 0, float top_p = 0.f);
int launch_wait_timeout_probe(b200_ctx* ctx, unsigned long long limit_ns);
// Load the kernels of the single-pass TF32 forward now (CUDA loads a kernel lazily at its first use,
// which may allocate device memory): for callers that must not allocate later.
int preload_rowwise_kernels(b200_ctx* ctx);
int preload_gemm_kernels(b200_ctx* ctx);
int preload_attention_kernel(b200_ctx* ctx);

// epilogue flags of the GEMM
// GEMM_ACCUM_OUT: out += result instead of out = result (fp32 output without a residual operand: the
// tiles leave as TMA reductions).  With out = the residual stream this is the residual add.
// GEMM_PLANES_FP16: a split output (launch_gemm_bf16x3 with out_planes) is written as two fp16 planes instead of bf16
enum : int { GEMM_GELU = 1, GEMM_ROUND_OUT_TF32 = 2, GEMM_ACCUM_OUT = 4, GEMM_PLANES_FP16 = 8 };
struct GemmRowStats;
int launch_gemm_tf32(b200_ctx* ctx, float* out, const float* inp, const float* weight,
                     const float* bias, const float* residual, int M, int K, int N, int flags,
                     int mode, unsigned long long* argmax_keys = nullptr, int argmax_cols = 0, int store_period = 0,
                     const GemmRowStats* stats = nullptr);
// The same product with bf16 operands (tcgen05 kind::f16, fp32 accumulation): inp [M,K] and weight
// [N,K] hold bf16; the result goes to out (fp32) or, if out_h is not null, to out_h as bf16.
// flags: GEMM_GELU only.  K and N multiples of 8.
int launch_gemm_bf16(b200_ctx* ctx, float* out, uint16_t* out_h, const uint16_t* inp, const uint16_t* weight,
                     const float* bias, int M, int K, int N, int flags,
                     unsigned long long* argmax_keys = nullptr, int argmax_cols = 0, int store_period = 0);
// The same product from split bf16 operands (three kind::f16 products per K step, hi.hi + hi.lo +
// lo.hi: 16 significant bits per operand).  inp holds two bf16 planes of [M,K]: hi = bf16(x) and,
// M*K elements further on, lo = bf16(x - hi); weight_hi / weight_lo [N,K] likewise.  The result goes
// to out (fp32; GEMM_ACCUM_OUT adds onto it) or, if out_planes is not null, there as two bf16 planes
// of [M,N] in the same split form.  flags: GEMM_GELU, GEMM_ACCUM_OUT.  K and N multiples of 8.
// e4m3 operands (tcgen05 kind::f8f6f4, fp32 accumulation): out = act(alpha * inp_q . weight_q^T + bias), alpha
// undoing the scales the operands were quantised with; flags: GEMM_GELU, GEMM_ACCUM_OUT.  K a multiple of 16.
int launch_gemm_fp8(b200_ctx* ctx, float* out, const uint8_t* inp, const uint8_t* weight, const float* bias,
                    int M, int K, int N, int flags, float alpha);
int launch_gemm_bf16x3(b200_ctx* ctx, float* out, uint16_t* out_planes, const uint16_t* inp, const uint16_t* weight_hi,
                       const uint16_t* weight_lo, const float* bias, int M, int K, int N, int flags,
                       unsigned long long* argmax_keys = nullptr, int argmax_cols = 0, int store_period = 0,
                       const GemmRowStats* stats = nullptr, int lo_col0 = 0);  // lo_col0: with out_planes, columns below it get no plane of dropped parts
// Extras of the fused row reduction of a GEMM with arg-max keys (CTA-pair kernel only):
//   inv_temp > 0: the keys hold, instead of the arg-max, the column that maximises
//     sample_score(value, inv_temp, seed, stream0 + row, column) - a draw from softmax(row / temperature);
//   lse_part != null: per row and per (256-column tile, half of it) the maximum m and the sum of
//     exp(value - m) over the columns below argmax_cols, as float2 pairs [M][lse_slots]
//     (lse_slots = 2 * ceil(N / 256)); launch_lse_reduce folds them into log-sum-exp per row.
struct GemmRowStats {
    float inv_temp;
    unsigned int seed, stream0;
    float2* lse_part;
    int lse_slots;
};
// lse[r] = log sum_j exp(x[r][j]) from the partial pairs of a GEMM with GemmRowStats::lse_part
int launch_lse_reduce(b200_ctx* ctx, float* lse, const float2* part, int M, int slots);
// (store_period > 0, with the fused arg-max: rows come in sequences of store_period and only the
// 32-row blocks holding a sequence's last row are written to out)
// After the lm-head: turns the keys left by a GEMM with fused arg-max into column indices and
// zeroes them (keys may be null), and gathers the last position's logits of every sequence into
// last_dst[B,Vp] (may be null), and copies the context's status word to status_dst (may be null).
// out, last_dst and status_dst may be device views of pinned host memory.  Vp % 4 == 0.
int launch_host_results(b200_ctx* ctx, int* out, unsigned long long* keys, int M, float* last_dst,
                        const float* logits, int B, int T, int Vp, int* status_dst = nullptr);

int launch_attention(b200_ctx* ctx, float* out, float* lse, const float* qkv, int B, int T, int C,
                     int NH, int flags);

// The same on fp16 operands (attention_split.cu): qkv_split holds the packed buffer [B*T, 3C] as two
// fp16 planes, hi then lo (what launch_gemm_bf16x3 writes with out_planes and GEMM_PLANES_FP16);
// kind::f16 products q_hi.k_hi and p.v_hi + p.v_lo.  flags as launch_attention.
int launch_attention_split(b200_ctx* ctx, float* out, float* lse, const uint16_t* qkv_split, int B, int T, int C,
                           int NH, int flags);

// incremental decoding (decode.cu): B <= 16 rows, fp32 FMA, no TF32 rounding
// out[B,N] = act(x[B,K] * W[N,K]^T + bias[N])
// with ln_w: x = layernorm(x + branch) * ln_w + ln_b first (branch nullable), and x + branch is
// stored to resid_out (a buffer other than x)
// k_splits > 1 (plain product only): K is cut into that many slices computed by different CTAs, and
// out receives the partial results [k_splits][B][N] (the bias in slice 0) for a consumer that adds them
// up in order - the layernorm prologue does, given branch_parts = the producer's k_splits
int launch_skinny_gemm(b200_ctx* ctx, float* out, const float* x, const float* W, const float* bias, int B,
                       int K, int N, int gelu, const float* branch = nullptr, const float* ln_w = nullptr,
                       const float* ln_b = nullptr, float* resid_out = nullptr, int k_splits = 1, int branch_parts = 1);
int skinny_gemm_k_splits(const b200_ctx* ctx, int K, int N);  // the slices worth using for a [*,K] x [N,K]^T product
// k and v columns of qkv rows [B*T, 3C] -> caches [B][cache_T][C] at positions pos0 .. pos0+T-1
int launch_kv_append(b200_ctx* ctx, float* kcache, float* vcache, const float* qkv, int B, int T, int C, int pos0,
                     int cache_T);
// out[B,C]: stores k and v of the rows qkv[B,3C] at position *pos_ptr, then attention of their
// query parts over cached positions 0 .. *pos_ptr
// partial: scratch of B * NH * 4 * 66 floats; counters: B * NH zeroed words (left zeroed)
int launch_decode_attention(b200_ctx* ctx, float* out, const float* qkv, float* kcache, float* vcache, int B, int C,
                            int NH, const int* pos_ptr, int cache_T, float* partial, unsigned int* counters);
// out[B,C] = wte[tok[b]] + wpe[*pos_ptr]
int launch_decode_encoder(b200_ctx* ctx, float* out, const int* tok, const float* wte, const float* wpe,
                          const int* pos_ptr, int B, int C, int vocab_rows);
int launch_set_int(b200_ctx* ctx, int* dst, int value);

// 3xTF32 attention: qkv_small is a scratch buffer shaped like qkv ([B,T,3C]) that receives the
// dropped low parts of qkv; two kernel launches (split + attention)
int launch_attention_x3(b200_ctx* ctx, float* out, float* qkv_small, float* lse, const float* qkv, int B,
                        int T, int C, int NH);

// Launch with programmatic stream serialization: the kernel may begin its set-up while its
// predecessor in the stream drains.  ONLY for kernels that call griddep_wait() before their
// first global-memory access.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(b200_ctx* ctx, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// Counter-based random bits: two rounds of a 32-bit integer mixer over (seed, stream, column).
__device__ __forceinline__ uint32_t mix32(uint32_t x) {
    x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
    return x;
}
__device__ __forceinline__ float gumbel_noise(uint32_t seed, uint32_t stream, uint32_t col) {
    const uint32_t h = mix32(mix32(seed ^ (stream * 0x9E3779B1u)) ^ (col * 0x85EBCA77u));
    const float u = ((float)(h >> 8) + 0.5f) * (1.0f / 16777216.0f);  // (0,1), 24 bits
    return -__logf(-__logf(u));
}
// The score whose arg-max over the columns is a draw from softmax(logits / temperature) (Gumbel-max);
// one fused multiply-add, so that every kernel that draws gets the same bits for the same input.
__device__ __forceinline__ float sample_score(float logit, float inv_temp, uint32_t seed, uint32_t stream, uint32_t col) {
    return fmaf(logit, inv_temp, gumbel_noise(seed, stream, col));
}

// fast, accurate tanh-GELU: x * sigmoid(2u), u = sqrt(2/pi) * (x + 0.044715 x^3)
__device__ __forceinline__ float gelu_tanh(float x) {
    const float k2 = 1.5957691216057308f;  // 2*sqrt(2/pi)
    float u = k2 * (x + 0.044715f * x * x * x);
    return __fdividef(x, 1.0f + __expf(-u));
}

}  // namespace b200
