/*
 * b200gpt2.h - C ABI of the B200-native GPT-2 forward engine (libb200gpt2.so).
 *
 * The entry points keep the shape of the reference project's host wrappers
 * (GJ0407790/CUDA-GPT2-Inference, kernels/.../*.cuh): free functions that take DEVICE
 * float pointers and int dimensions, allocate nothing, and launch asynchronously.  Every
 * activation and parameter is fp32, row-major, laid out exactly as in the reference:
 *   activations [B,T,C]; linear weights [OC,C] (K contiguous); packed QKV [B,T,3,NH,HS].
 *
 * Two forms of every operator are exported:
 *   - b200_<op>(ctx, ...) returns an int status (B200_OK == 0) and launches on the
 *     context's stream;
 *   - <op>(...) is the reference-shaped void shim: it runs on a process-wide default
 *     context (current device, legacy default stream) and, like the reference's asserts,
 *     aborts the process with a message on a precondition failure.
 *
 * Threading: a context is owned by one host thread at a time.  Nothing here synchronises
 * the stream unless stated.  All pointers must be 16-byte aligned.  The b200_gpt2_* calls make the
 * context's device current while they run and put the caller's device back; the operator calls
 * expect it to be current already (as the reference's do).
 *
 * Device-side waits: every wait inside a kernel gives up after 2 s; the kernel then returns and
 * leaves a code in the context's status word.  b200_ctx_sync_check (or b200_gpt2_forward_host_wait)
 * reports it as B200_ERR_TIMEOUT and clears the status area, which also holds the attention
 * kernel's work counters and the GEMM's hand-over flags: after such an error call one of the two
 * before the context is used again.
 */
#ifndef B200GPT2_H
#define B200GPT2_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---------------------------------------------------------------- status codes */
enum {
    B200_OK = 0,
    B200_ERR_NULL = 1,       /* a required pointer is NULL                          */
    B200_ERR_SHAPE = 2,      /* a dimension violates a stated precondition          */
    B200_ERR_ALIGN = 3,      /* a pointer is not 16-byte aligned                    */
    B200_ERR_CUDA = 4,       /* a CUDA runtime/driver call failed (see last_error)  */
    B200_ERR_DEVICE = 5,     /* not an sm_100 device                                */
    B200_ERR_TIMEOUT = 6,    /* a device-side wait ran out; the kernel returned     */
    B200_ERR_STATE = 7,      /* object used before it was set up                    */
    B200_ERR_LIMIT = 8       /* size beyond a stated maximum                        */
};

/* GEMM arithmetic modes */
enum {
    B200_TF32 = 0,           /* one tcgen05 kind::tf32 pass (default)               */
    B200_TF32X3 = 1,         /* three-term split (big*big + small*big + big*small)  */
    B200_BF16 = 2,           /* bf16 operands (tcgen05 kind::f16), fp32 accumulation: model option only */
    B200_BF16X3 = 3          /* every fp32 operand as two bf16 terms (16 significant bits), three
                                kind::f16 products per K step, fp32 accumulation: model option and
                                b200_matmul_forward_bf16x3 */
};

/* GEMM epilogue activation */
enum { B200_ACT_NONE = 0, B200_ACT_GELU = 1 };

typedef struct b200_ctx b200_ctx;

/* Creates a context on `device` (made current).  `stream` is a cudaStream_t passed as
 * void* (NULL = legacy default stream, the reference's behaviour). */
int b200_ctx_create(b200_ctx** out, int device, void* stream);
int b200_ctx_destroy(b200_ctx* ctx);
int b200_ctx_set_stream(b200_ctx* ctx, void* stream);
/* Synchronises the stream, then returns B200_ERR_TIMEOUT / B200_ERR_CUDA if a kernel
 * recorded a device-side wait that ran out or CUDA reports an error; clears the word. */
int b200_ctx_sync_check(b200_ctx* ctx);
/* Self-test of the failure path: launches one thread that waits on an mbarrier nothing arrives
 * on and gives up after limit_ms (1..2000), exactly as the GEMM and attention roles do when a
 * wait runs out.  The kernel returns normally; the next b200_ctx_sync_check reports
 * B200_ERR_TIMEOUT once and the context stays usable. */
int b200_ctx_wait_timeout_probe(b200_ctx* ctx, int limit_ms);
/* The same for the wait on a hand-over word that another GPU writes (b200_gpt2_tp_peer_*): the kernel
 * waits limit_ms for a word that nothing sets, gives up and reports device status 105. */
int b200_ctx_peer_wait_probe(b200_ctx* ctx, int limit_ms);
/* Number of kernels this context has launched since creation (or the last reset). */
uint64_t b200_ctx_launch_count(const b200_ctx* ctx);
void b200_ctx_reset_launch_count(b200_ctx* ctx);
const char* b200_status_string(int status);
/* Text of the last failing CUDA call on this context ("" if none). */
const char* b200_ctx_last_error(const b200_ctx* ctx);

/* ------------------------------------------------------------------ operators */

/* out[B,T,OC] = act(inp[B,T,C] . weight[OC,C]^T + bias[OC]) (+ residual[B,T,OC]).
 * Replaces matmul_forward_tiling (kernels/matmul/1_matmul_tiling.cuh:57-65),
 * matmul_forward_cublas + add_bias (2_matmul_cublas.cuh:7-61), matmul_forward_ptx_2d
 * (5_matmul_ptx_2d.cuh:165-173) and matmul_forward_async_cg_tf32_gelu
 * (9_matmul_async_cg_tf32_gelu.cuh:237-246, whose `bool is_gelu` is `act`).
 * bias and residual may be NULL.  residual == out (the same pointer) adds the product onto out in
 * place: the tiles leave as element-wise fp32 reductions, one add per element, which is how the
 * driver puts the two projections of a block onto the residual stream.
 * Preconditions: C % 4 == 0, OC % 4 == 0. */
int b200_matmul_forward(b200_ctx* ctx, float* out, const float* inp, const float* weight,
                        const float* bias, int B, int T, int C, int OC, int act,
                        const float* residual, int mode);

/* The same product with bf16 operands (the reference's bf16 experiment, README.md:124-128 and
 * kernels/matmul/5_matmul_ptx_2d.cuh, is the counterpart): inp[B,T,C] and weight[OC,C] hold bf16
 * values (16 bits each, as uint16_t), accumulation is fp32; the result is written to out (fp32) or,
 * when out_bf16 is not NULL, to out_bf16 as bf16 (out is then ignored and may be NULL).  bias
 * (fp32) may be NULL.  Preconditions: C % 8 == 0, OC % 8 == 0. */
int b200_matmul_forward_bf16(b200_ctx* ctx, float* out, uint16_t* out_bf16, const uint16_t* inp,
                             const uint16_t* weight, const float* bias, int B, int T, int C, int OC, int act);
/* out[i] = bf16(inp[i]), round to nearest even; n % 4 == 0. */
int b200_convert_bf16(b200_ctx* ctx, uint16_t* out, const float* inp, size_t n);

/* The same product at close to fp32 precision on the bf16 tensor path (B200_BF16X3; like the
 * reference's bf16 experiment, README.md:124-128, but with every fp32 operand carried as TWO bf16
 * terms): x = hi + lo, hi = bf16(x), lo = bf16(x - hi), 16 significant bits; the kernel adds
 * hi.hi + hi.lo + lo.hi per K step in fp32.  inp_split holds the two planes of inp one after the
 * other ([2][B,T,C] bf16, as written by b200_split_bf16 with lo = hi + B*T*C); weight_hi /
 * weight_lo are the planes of weight[OC,C].  The result goes to out (fp32; accumulate != 0 adds
 * it onto out, as residual == out does in b200_matmul_forward) or, when out_split is not NULL, to
 * out_split in the same two-plane form ([2][B,T,OC]; needs B*T % 32 == 0, no accumulation) so that
 * it can feed the next product.  bias (fp32) may be NULL.  Preconditions: C % 8 == 0, OC % 8 == 0. */
int b200_matmul_forward_bf16x3(b200_ctx* ctx, float* out, uint16_t* out_split, const uint16_t* inp_split,
                               const uint16_t* weight_hi, const uint16_t* weight_lo, const float* bias, int B, int T,
                               int C, int OC, int act, int accumulate);
/* hi[i] = bf16(inp[i]) (round to nearest even), lo[i] = bf16(inp[i] - hi[i]); n % 4 == 0. */
int b200_split_bf16(b200_ctx* ctx, uint16_t* hi, uint16_t* lo, const float* inp, size_t n);

/* The same product with 8-bit floating-point operands (e4m3: 4 exponent, 3 mantissa bits; tcgen05
 * kind::f8f6f4, fp32 accumulation) - the second half of the reference's reduced-precision
 * experiment (README.md:124-128; kernels/matmul/5_matmul_ptx_2d.cuh:165-202 is its bf16 kernel):
 *     out = act(alpha * inp_q . weight_q^T + bias)          (accumulate != 0: out += ..., no act)
 * inp_q[B,T,C] and weight_q[OC,C] hold e4m3 values (one byte each) as b200_quantize_e4m3 writes
 * them, x_q = e4m3(x * scale); alpha = 1 / (scale_inp * scale_weight) undoes the two scales in the
 * epilogue (exactly, when they are powers of two).  Products of e4m3 values are exact in fp32, so
 * the result is the fp32-accumulated product of the quantised operands.
 * Preconditions: C % 16 == 0, OC % 8 == 0. */
int b200_matmul_forward_fp8(b200_ctx* ctx, float* out, const uint8_t* inp_q, const uint8_t* weight_q, const float* bias,
                            int B, int T, int C, int OC, int act, float alpha, int accumulate);
/* out[i] = e4m3(inp[i] * scale): round to nearest even, saturating at +-448; scale > 0, n % 4 == 0. */
int b200_quantize_e4m3(b200_ctx* ctx, uint8_t* out, const float* inp, size_t n, float scale);

/* Causal multi-head attention on the packed buffer inp[B,T,3C] -> out[B,T,C].
 * Replaces attention_forward_cublas (kernels/attention/1_attention_cublas.cuh:31-36),
 * flash_attention_forward (2_flash_attention.cuh:336-341) and
 * flash_attention_permute_forward (3_flash_attention_permute.cuh:346-351).
 * qkvr is unused and may be NULL.  If att is non-NULL it receives the softmax statistics
 * lse[B,NH,T] = log(sum_j exp(q.k_j/sqrt(HS))).  inp is not modified.
 * Preconditions: C/NH == 64, T % 64 == 0 (the reference's, 3_...cuh:336-337). */
int b200_attention_forward(b200_ctx* ctx, float* out, float* qkvr, float* att, const float* inp,
                           int B, int T, int C, int NH);

/* The same operator with split-operand (3xTF32) products, for the B200_TF32X3 mode: q.k and p.v
 * keep the low mantissa bits that a single TF32 pass drops.  qkvr is REQUIRED here: a scratch
 * buffer of the shape of inp ([B,T,3C], the buffer the reference's signature already carries,
 * kernels/attention/2_flash_attention.cuh:336-341) that receives the dropped parts of inp. */
int b200_attention_forward_x3(b200_ctx* ctx, float* out, float* qkvr, float* att, const float* inp,
                              int B, int T, int C, int NH);

/* The same operator on fp16 operands, the attention of the B200_BF16X3 mode: inp_split holds the
 * packed buffer as two fp16 planes, [2][B,T,3C] with value = hi + lo (b200_split_fp16 of the fp32
 * buffer; inside the driver the QKV GEMM writes it).  q.k is one kind::f16 product on the hi
 * planes (11 significant bits, rounded to nearest), p.v the sum of two (v with both terms, p
 * rounded to fp16 inside the kernel).  out fp32 [B,T,C]; att as above.  Values beyond the fp16
 * range (65504) are clamped by the split. */
int b200_attention_forward_fp16(b200_ctx* ctx, float* out, float* att, const uint16_t* inp_split,
                                int B, int T, int C, int NH);
/* hi[i] = fp16(inp[i]) (round to nearest even, clamped to +-65504), lo[i] = fp16(inp[i] - hi[i]); n % 4 == 0. */
int b200_split_fp16(b200_ctx* ctx, uint16_t* hi, uint16_t* lo, const float* inp, size_t n);

/* Replaces layernorm_forward_block / _block_vectorized / _warp
 * (kernels/layernorm/1_layernorm_block.cuh:63-65, 2_...:74-76, 3_layernorm_warp.cuh:78-80).
 * mean and rstd ([B,T]) may be NULL.  Precondition: C % 4 == 0, C <= 4096. */
int b200_layernorm_forward(b200_ctx* ctx, float* out, float* mean, float* rstd, const float* inp,
                           const float* weight, const float* bias, int B, int T, int C);

/* res_out = inp1 + inp2; layernorm_out = LN(res_out).  Replaces
 * fused_residual_layernorm_forward
 * (kernels/fused_residual_layernorm/fused_residual_layernorm.cuh:88-90).
 * res_out may alias inp1 or inp2. */
int b200_fused_residual_layernorm_forward(b200_ctx* ctx, float* res_out, float* layernorm_out,
                                          float* mean, float* rstd, const float* inp1,
                                          const float* inp2, const float* weight,
                                          const float* bias, int B, int T, int C);

/* out = inp1 + inp2.  Replaces residual_forward_naive / _cache_hint
 * (kernels/residual/1_residual_naive.cuh:15, 2_residual_cache_hint.cuh:15). */
int b200_residual_forward(b200_ctx* ctx, float* out, const float* inp1, const float* inp2,
                          size_t N);

/* tanh-GELU, the device function of kernels/matmul/9_matmul_async_cg_tf32_gelu.cuh:5-11 as a
 * stand-alone operator (the reference names the step in README.md:15 but ships no kernel). */
int b200_gelu_forward(b200_ctx* ctx, float* out, const float* inp, size_t N);

/* out[b,t,:] = wte[inp[b,t],:] + wpe[t,:].  The reference names the step (README.md:10) but
 * ships no kernel.  Token ids must lie in [0, vocabulary rows of wte). */
int b200_encoder_forward(b200_ctx* ctx, float* out, const int* inp, const float* wte,
                         const float* wpe, int B, int T, int C);

/* --------------------------------------------- reference-shaped void shims */
void matmul_forward(float* out, const float* inp, const float* weight, const float* bias, int B,
                    int T, int C, int OC);
void matmul_forward_gelu(float* out, const float* inp, const float* weight, const float* bias,
                         int B, int T, int C, int OC, int is_gelu);
void attention_forward(float* out, float* qkvr, float* att, const float* inp, int B, int T, int C,
                       int NH);
void layernorm_forward(float* out, float* mean, float* rstd, const float* inp, const float* weight,
                       const float* bias, int B, int T, int C);
void fused_residual_layernorm_forward(float* res_out, float* layernorm_out, float* mean,
                                      float* rstd, const float* inp1, const float* inp2,
                                      const float* weight, const float* bias, int B, int T, int C);
void fused_residual_layernorm(float* res_out, float* layernorm_out, float* mean, float* rstd,
                              const float* inp1, const float* inp2, const float* weight,
                              const float* bias, int B, int T, int C);
void residual_forward(float* out, const float* inp1, const float* inp2, int N);
void gelu_forward(float* out, const float* inp, int N);
void encoder_forward(float* out, const int* inp, const float* wte, const float* wpe, int B, int T,
                     int C);

/* ------------------------------------------------------------ gpt2_forward driver */
/* The driver the reference's kernels plug into (llm.c's gpt2_forward; README.md:19 and
 * images/gpt2/gpt2_flow.png give the operator order).  Forward only. */
typedef struct {
    int max_seq_len;        /* maxT, rows of wpe                       */
    int vocab_size;         /* V                                       */
    int padded_vocab_size;  /* Vp, rows of wte and width of the logits */
    int num_layers;         /* L                                       */
    int num_heads;          /* NH                                      */
    int channels;           /* C                                       */
} b200_gpt2_config;

typedef struct b200_gpt2 b200_gpt2;

/* Number of fp32 parameters, and the offsets (in floats) of the 16 parameter tensors in the
 * flat parameter array, in this order, each stacked over layers:
 *   wte[Vp,C] wpe[maxT,C] ln1w[L,C] ln1b[L,C] qkvw[L,3C,C] qkvb[L,3C] attprojw[L,C,C]
 *   attprojb[L,C] ln2w[L,C] ln2b[L,C] fcw[L,4C,C] fcb[L,4C] fcprojw[L,C,4C] fcprojb[L,C]
 *   lnfw[C] lnfb[C].   offsets has 17 entries; offsets[16] is the total. */
size_t b200_gpt2_param_offsets(const b200_gpt2_config* cfg, size_t* offsets);

/* Allocates device memory for the parameters and for the activations of a forward pass of up
 * to max_B x max_T tokens.  Forward-only, so one layer's activations are reused by every
 * layer.  This is the only allocating call. */
int b200_gpt2_create(b200_gpt2** out, b200_ctx* ctx, const b200_gpt2_config* cfg, int max_B,
                     int max_T);
int b200_gpt2_destroy(b200_gpt2* model);
/* Device pointer of the flat parameter array (fill it in place), or copy from the host. */
float* b200_gpt2_params(b200_gpt2* model);
int b200_gpt2_load_params_host(b200_gpt2* model, const float* host_params, size_t count);
/* Reads the parameters from a file: header_bytes are skipped, then the fp32 parameters follow in
 * the order of b200_gpt2_param_offsets (wte, wpe, ln1w, ln1b, qkvw, qkvb, attprojw, attprojb, ln2w,
 * ln2b, fcw, fcb, fcprojw, fcprojb, lnfw, lnfb), little endian, nothing after them.  Parsing a
 * checkpoint format's header (and choosing the configuration from it) is the caller's job; the
 * file size must be exactly header_bytes + 4 * parameter count (else B200_ERR_SHAPE; a file that
 * cannot be opened or read is B200_ERR_STATE).  The copy goes through pinned staging buffers in
 * 32 MB pieces.  Not for tensor-parallel models, whose parameters are stored sharded. */
int b200_gpt2_load_params_file(b200_gpt2* model, const char* path, size_t header_bytes);
/* Options (defaults: round_operands 1, both modes B200_BF16X3, use_graph 0; a tensor-parallel model
 * takes B200_BF16X3, B200_TF32 and B200_TF32X3, not B200_BF16).
 * round_operands != 0 makes every producer whose output feeds only a single-pass TF32 GEMM store
 * TF32-round-to-nearest values and makes those GEMMs read a rounded copy of the weight
 * matrices (made on the next forward; the parameters themselves are never modified, so the
 * encoder stays bit-exact and the decode step sees the weights as loaded).  The tensor core
 * truncates raw fp32 operands, which shrinks every product; rounding to nearest first removes
 * that bias (logit error 4.6e-4 rms instead of 7.9e-4 on GPT-2 124M).  gemm_mode applies to all
 * GEMMs; lmhead_mode to the lm-head alone.  B200_TF32X3 ignores operand rounding; with gemm_mode ==
 * B200_TF32X3 attention also runs with split operands (b200_attention_forward_x3; its scratch
 * buffer is allocated by this call).  B200_BF16 / B200_BF16X3 keep bf16 copies of the weight
 * matrices (made on the next forward) and have the layernorms, the attention and the GELU GEMM
 * write their outputs as bf16 / as two bf16 planes; with B200_BF16 attention stays single-pass
 * TF32 on rounded q, k, v, with B200_BF16X3 it runs on fp16 planes of q, k, v
 * (b200_gpt2_set_attention_mode overrides).  use_graph != 0 replays the
 * forward from a CUDA graph after the first call of a given (B,T). */
int b200_gpt2_set_options(b200_gpt2* model, int round_operands, int gemm_mode, int lmhead_mode,
                          int use_graph);
/* Attention arithmetic: -1 (default) follows gemm_mode (B200_BF16X3: fp16 attention,
 * b200_attention_forward_fp16; B200_TF32X3: b200_attention_forward_x3; otherwise single-pass
 * TF32), B200_TF32 forces the single-pass kernel, B200_TF32X3 the 3xTF32 one (with gemm_mode
 * B200_TF32, B200_TF32X3 or B200_BF16X3; allocates the scratch buffer on first use), B200_BF16X3
 * the fp16 one (gemm_mode B200_BF16X3 only). */
int b200_gpt2_set_attention_mode(b200_gpt2* model, int mode);
/* tokens: device int32 [B,T].  Asynchronous.  Logits: device [B,T,Vp], owned by the model. */
int b200_gpt2_forward(b200_gpt2* model, const int* tokens, int B, int T);
float* b200_gpt2_logits(b200_gpt2* model);
/* The forward with sampling (and the softmax normaliser) taken in the lm-head GEMM's epilogue, while
 * the logits are still accumulators: nothing has to read the 1.65 GB (124M, B=8, T=1024) of logits
 * again, and with store_logits == 0 they are not even written (only the 32-row blocks that hold
 * a sequence's last position are; the rest of the model's logits buffer is then stale).  No
 * counterpart in the reference, which stops at the logits.
 *   ids_out [B,T] (device int32): per position one token drawn from softmax(logits / temperature)
 *     over the real vocabulary [0,V) - the arg-max of logit / temperature + Gumbel noise, the
 *     noise a fixed function of (seed, row b*T + t, token id): exactly what
 *     b200_sample_rows(ctx, out, logits, B*T, V, Vp, temperature, 0, 0, seed, 0) draws from the
 *     stored logits.  temperature <= 0: the arg-max.
 *   lse_out [B,T] (device fp32, nullable): log sum_{j<V} exp(logit_j), so that
 *     exp(logit - lse) is the softmax probability of any logit the caller still has.  The first
 *     call with lse_out allocates the partial-sum buffer (25.8 MB for 124M at 8192 rows).
 * Asynchronous on the context's stream; never replayed from a graph.  lmhead_mode B200_BF16X3 or
 * B200_TF32; not on a tensor-parallel model. */
int b200_gpt2_forward_sample(b200_gpt2* model, const int* tokens, int B, int T, float temperature,
                             unsigned int seed, int* ids_out, float* lse_out, int store_logits);
/* Host-buffer form: copies tokens (host, ideally pinned) to the device, runs the forward,
 * and copies back what is asked for, synchronising before it returns:
 *   logits_host      [B,T,Vp]  all logits                     (nullable)
 *   last_logits_host [B,Vp]    logits of the last position    (nullable)
 *   argmax_host      [B,T]     arg-max token over [0,V) per position (nullable) 
 * When argmax_host is given and logits_host is NULL nobody needs the full logits: the lm-head then
 * writes only the last-position rows, and the model's device logits buffer holds nothing else. */
int b200_gpt2_forward_host(b200_gpt2* model, const int* tokens_host, int B, int T,
                           float* logits_host, float* last_logits_host, int* argmax_host);
/* The same call split in two, so that the host can prepare and enqueue the next batch while the
 * GPU works on the current one (two batches in flight, slot = 0 or 1): _enqueue queues the token
 * copy, the forward and the copies back and returns at once; _wait blocks until the results of
 * that slot are in the caller's buffers and reports a device-side error recorded up to then.  The
 * host buffers of a slot (pinned, for the copies to overlap) must stay untouched between the two
 * calls.  Work is stream-ordered: the batches run one after the other on the GPU. */
int b200_gpt2_forward_host_enqueue(b200_gpt2* model, const int* tokens_host, int B, int T,
                                   float* logits_host, float* last_logits_host, int* argmax_host, int slot);
int b200_gpt2_forward_host_wait(b200_gpt2* model, int slot);
/* ---- incremental decoding with a key/value cache (no counterpart in the reference, which has
 * full-sequence kernels only; the operators and their order are those of the forward above) ----
 * b200_gpt2_enable_kv_cache allocates the cache: keys and values of every layer for max_B
 * sequences of max_T positions, fp32, [L][max_B][max_T][C] each (2 x 302 MB for GPT-2 124M at
 * max_B = 8, max_T = 1024).  Not available on a tensor-parallel model.
 * b200_gpt2_prefill is b200_gpt2_forward that also stores the keys and values of positions
 * [0,T) (T % 64 == 0 as for the forward); logits as for b200_gpt2_forward.
 * b200_gpt2_decode_step takes one token per sequence (device int32 [B], B <= 16) standing at
 * position pos (0 <= pos < max_T; positions [0,pos) must be in the cache, from a prefill or
 * from earlier steps), appends its keys and values and leaves the logits of that position in
 * the first B rows of the model's logits buffer ([B,Vp]).  A step reads every weight and the
 * used part of the cache once, so it is bound by HBM bandwidth; it runs on the fp32 FMA pipe
 * (no TF32 rounding anywhere).  Starting at pos = 0 with an empty cache is allowed.
 * The decode step always reads the parameters as loaded, whatever gemm_mode says.
 * b200_gpt2_decode_step_host: tokens from the host, logits [B,Vp] and / or arg-max ids [B] back;
 * synchronises.  All calls are asynchronous on the context's stream unless stated. */
int b200_gpt2_enable_kv_cache(b200_gpt2* model);
int b200_gpt2_prefill(b200_gpt2* model, const int* tokens, int B, int T);
int b200_gpt2_decode_step(b200_gpt2* model, const int* tokens, int B, int pos);
int b200_gpt2_decode_step_host(b200_gpt2* model, const int* tokens_host, int B, int pos,
                               float* logits_host, int* argmax_host);
/* Greedy generation on top of the calls above.  prompt_host: int32 [B,T0] (T0 >= 1); out_host:
 * int32 [B,n_new] receives, per sequence, the arg-max continuation of n_new tokens
 * (T0 + n_new <= max_T).  If T0 is a multiple of 64 the prompt goes through the tensor-core
 * prefill, otherwise it is fed token by token.  The token ids stay on the device between steps
 * (the arg-max of a step is the input of the next); synchronises once at the end. */
int b200_gpt2_generate_greedy(b200_gpt2* model, const int* prompt_host, int B, int T0, int n_new,
                              int* out_host);
/* The same loop drawing every new token from softmax(logits / temperature) instead of taking the
 * arg-max (temperature <= 0: greedy).  The draw is the arg-max of logit / temperature + Gumbel
 * noise, the noise being a fixed function of (seed, position, sequence, token id): the same call
 * returns the same continuation.  top_k > 0 restricts every draw to the top_k most likely tokens
 * (tokens tied with the k-th included); 0 < top_p < 1 then keeps the most likely of those whose
 * probabilities add up to top_p (nucleus sampling); 0 for either switches it off. */
int b200_gpt2_generate(b200_gpt2* model, const int* prompt_host, int B, int T0, int n_new,
                       float temperature, int top_k, float top_p, unsigned int seed, int* out_host);
/* One draw per row of logits[M, ld] over columns [0,V) (device pointers; out int32 [M]), as used by
 * b200_gpt2_generate: row r takes the noise stream stream0 + r of the seed. */
int b200_sample_rows(b200_ctx* ctx, int* out, const float* logits, int M, int V, int ld,
                     float temperature, int top_k, float top_p, unsigned int seed, unsigned int stream0);

/* ---- tensor parallelism (optional; Megatron style, for models like GPT-2 XL) --------------
 * Rank r of tp_size holds the q/k/v rows and attn-proj input columns of its share of the heads
 * (NH/tp_size each, the first NH % tp_size ranks one more), 1/tp_size of the MLP hidden width,
 * and - when Vp divides evenly - 1/tp_size of the lm-head (logits stay sharded, [B,T,Vp/tp_size]).
 * Layernorms, the encoder and the residual stream are replicated.  The partial [B,T,C] sums
 * after attn-proj and after fc-proj are combined by ONE all-reduce each per block, issued
 * through a callback so that the communication library stays the caller's choice (NCCL's
 * ncclAllReduce, or torch.distributed): the callback must enqueue an in-place fp32 sum
 * all-reduce of buf[0..count) over the tensor-parallel group on `stream` and return 0.  `stream` is
 * the context's stream or, when b200_gpt2_set_tp_overlap asks for row chunks, the model's own
 * communication stream: the all-reduce of a chunk is then issued as soon as its GEMM is queued, so
 * that it runs under the next chunk's GEMM, and the callback is called once per chunk (same ranks,
 * same order on every rank).
 * Rank-local parameters use the same 16-tensor order with the local shapes;
 * b200_gpt2_shard_params_host cuts them out of a full host parameter array. */
typedef int (*b200_allreduce_fn)(void* user, float* buf, size_t count, void* stream);
int b200_gpt2_create_tp(b200_gpt2** out, b200_ctx* ctx, const b200_gpt2_config* cfg, int max_B,
                        int max_T, int tp_size, int tp_rank);
int b200_gpt2_set_allreduce(b200_gpt2* model, b200_allreduce_fn fn, void* user);
/* How a tensor-parallel projection overlaps its all-reduce: chunks = row chunks (1-8; 1 = the
 * whole GEMM, then one all-reduce on the compute stream), reserve_sms = SMs the GEMMs of the later
 * chunks leave free for the communication kernels that run beside them (0-64).  Default 1, 0: on
 * two B200s the chunked forms measured slower (GPT-2 XL, 8192 rows: 40.7 ms unchunked, 44.0 with
 * 2 chunks, 48.5 with 4), so the overlap is an option, not the default. */
int b200_gpt2_set_tp_overlap(b200_gpt2* model, int chunks, int reserve_sms);

/* Two-way tensor parallelism without all-reduces (tp_size == 2, B200_BF16X3 or B200_TF32 GEMMs, the two GPUs
 * connected by NVLink, one process each).  Each projection GEMM stores the tiles of its partial sum
 * a second time, straight into the other GPU's memory, while it computes; a word written behind
 * the GEMM tells the peer that the sum is complete, and the fused residual + layernorm that follows
 * adds the two partial sums itself - the same bits an all-reduce would have produced, on both
 * ranks.  What is left of the exchange on the critical path is a bounded wait on that word.
 *   b200_gpt2_tp_peer_export   allocates the receive buffers and writes three CUDA IPC memory
 *                              handles (3 x 64 bytes) for the peer process
 *   b200_gpt2_tp_peer_connect  takes the PEER's three handles and switches the hand-over on; the
 *                              all-reduce callback is then no longer called
 * Both ranks must run the same sequence of forwards: every projection waits (at most 2 s, then
 * B200_ERR_TIMEOUT at the next sync_check) for its counterpart on the peer.  The two ranks count their
 * projections; after a time-out the counts may disagree, and the pair of models has to be created
 * and connected anew.  connect is called once per model. */
int b200_gpt2_tp_peer_export(b200_gpt2* model, unsigned char* handles /* [192] */);
int b200_gpt2_tp_peer_connect(b200_gpt2* model, const unsigned char* peer_handles /* [192] */);
/* Switches the hand-over off (the all-reduce callback is used again) or back on; like every change of
 * the exchange, on both ranks between the same two forwards. */
int b200_gpt2_tp_peer_enable(b200_gpt2* model, int on);

/* The same idea for a tensor-parallel group of 2 to 8 ranks (one process per GPU, all GPUs peers over
 * NVLink): a sequence-parallel hand-over.  Rank r owns the rows [r, r+1) * B*T / tp_size of the residual
 * stream.  A projection GEMM stores every tile of its partial sum only into the memory of the rank
 * that owns the tile's rows; that rank's layernorm adds the tp_size partial sums for its rows (in rank
 * order: the same sum everywhere) and writes the normalised rows into the layernorm output of every
 * rank; epoch words order the steps (waits of at most 2 s).  Per projection a rank sends
 * (tp_size-1)/tp_size of the activation twice - what an all-reduce moves - but the first half
 * travels under the GEMM and no reduction kernel runs.  B*T must be a multiple of 256 * tp_size
 * (otherwise the forward falls back on the all-reduce callback, if one is set).
 *   b200_gpt2_tp_sp_export   writes this rank's three CUDA IPC handles (3 x 64 bytes)
 *   b200_gpt2_tp_sp_connect  takes the handles of ALL ranks, [tp_size][192] bytes in rank order (the own
 *                            entry is ignored), and switches the hand-over on
 *   b200_gpt2_tp_sp_enable   off / on again, on all ranks between the same two forwards */
int b200_gpt2_tp_sp_export(b200_gpt2* model, unsigned char* handles /* [192] */);
int b200_gpt2_tp_sp_connect(b200_gpt2* model, const unsigned char* all_handles /* [tp_size][192] */);
int b200_gpt2_tp_sp_enable(b200_gpt2* model, int on);
size_t b200_gpt2_param_offsets_tp(const b200_gpt2_config* cfg, int tp_size, int tp_rank, size_t* offsets);
int b200_gpt2_shard_params_host(const b200_gpt2_config* cfg, int tp_size, int tp_rank,
                                const float* full_params, float* local_params);

/* Per-operator device timing of the forward.  While enabled, every kernel launch of
 * b200_gpt2_forward is bracketed by a CUDA event pair on the context's stream (graph replay is
 * bypassed).  b200_gpt2_read_profile synchronises the stream, adds up the elapsed milliseconds
 * and launch counts per category since the previous read-out into ms[B200_PROF_NUM] and
 * launches[B200_PROF_NUM], and clears them. */
enum {
    B200_PROF_ENCODER = 0, B200_PROF_LAYERNORM, B200_PROF_GEMM_QKV, B200_PROF_ATTENTION,
    B200_PROF_GEMM_ATTPROJ, B200_PROF_FUSED_RES_LN, B200_PROF_GEMM_FC, B200_PROF_GEMM_FCPROJ,
    B200_PROF_GEMM_LMHEAD, B200_PROF_ALLREDUCE, B200_PROF_NUM
};
int b200_gpt2_set_profile(b200_gpt2* model, int enabled);
int b200_gpt2_read_profile(b200_gpt2* model, double* ms, long* launches);
/* Device pointer of an intermediate activation of the last forward, for tests:
 * name in {"encoded","ln_out","qkv","atty","branch","fch","residual","argmax"}; NULL if unknown. */
void* b200_gpt2_activation(b200_gpt2* model, const char* name);

/* ---------------------------------------------------------------- no-allocation forward */
/* No counterpart in the reference (which has no driver at all).
 *
 * b200_gpt2_forward for callers that must not allocate device memory - an application that has
 * given all of the GPU to its own pool, a plugin host that forbids driver allocations after
 * start-up, a serving loop that cannot take the device-wide synchronisation that cudaMalloc and
 * cudaFree imply.  The caller passes the inputs (flat fp32 parameters in the layout above, int32
 * token ids [B,T]) and the output (logits [B,T,Vp]), all in device memory; the activations
 * between them use a scratch array built into the library (8.65 MB of every GPU that loads it,
 * held until the process exits).  The call makes no cudaMalloc / cudaFree and uses no allocating
 * library; `ctx` must have been created earlier, when allocation was still allowed.
 *
 * Limit: B*T*C <= B200_STATIC_MAX_TOKEN_CHANNELS (e.g. GPT-2 124M with B=4, T=64); larger
 * problems return B200_ERR_LIMIT (text in b200_ctx_last_error) and must use b200_gpt2_create.
 * The arithmetic is that of b200_gpt2_forward with round_operands = 0 and both modes B200_TF32
 * (single-pass TF32 GEMMs straight from the caller's weights: the other modes need copies of
 * the weights, i.e. allocations), bit for bit.
 *
 * Set-up: b200_gpt2_static_prepare(ctx), called once per device while allocation is still allowed,
 * looks up the scratch array's device address (cudaGetSymbolAddress) and loads the code of every
 * kernel this forward can launch.  Both steps can make the CUDA runtime allocate device memory
 * (it loads a kernel's module lazily, at first use), which is exactly what these callers cannot
 * have later; after the set-up b200_gpt2_forward_static allocates nothing, implicitly or
 * explicitly.  Without it the first b200_gpt2_forward_static on a device does the same set-up
 * itself - make that first call (or the set-up) before any stream capture begins.  The set-up is
 * serialised by a lock, so contexts of several host threads may race to it.
 * All calls on a device share the one scratch array: it keeps the previous call's contents
 * (nothing needs clearing - every part is rewritten before it is read), and two calls that
 * overlap on the GPU (different streams or contexts of the same device) race on it.
 * Asynchronous on the context's stream, like b200_gpt2_forward; the caller's current device is
 * left as it was.  Devices 0-63. */
#define B200_STATIC_MAX_TOKEN_CHANNELS 196608 /* 256 tokens x 768 channels */
int b200_gpt2_static_prepare(b200_ctx* ctx);
int b200_gpt2_forward_static(b200_ctx* ctx, const b200_gpt2_config* cfg, const float* params,
                             const int* tokens, int B, int T, float* logits);

#ifdef __cplusplus
}
#endif
#endif /* B200GPT2_H */
