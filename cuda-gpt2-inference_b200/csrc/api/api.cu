// The C ABI of include/b200gpt2.h: context management, argument validation, and the
// reference-shaped void shims.  Validation plays the role of the reference's host asserts
// (kernels/matmul/9_matmul_async_cg_tf32_gelu.cuh:255-268,
// kernels/attention/3_flash_attention_permute.cuh:336-337, kernels/layernorm/3_layernorm_warp.cuh:82)
// but returns a status instead of aborting; the shims abort like the reference does.
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include "ctx.h"
#include "../kernels/kernels.h"

int b200_fail_cuda(b200_ctx* ctx, cudaError_t e, const char* what) {
    if (ctx) ctx->last_error = std::string(what) + ": " + cudaGetErrorString(e);
    return B200_ERR_CUDA;
}

int b200_get_tensor_map(b200_ctx* ctx, CUtensorMap* out, const float* ptr, uint64_t rows,
                        uint64_t cols, uint64_t ld, uint32_t box_rows, uint32_t box_cols,
                        int swizzle_atom32) {
    TensorMapKey key{ptr, rows, cols, ld, box_rows, box_cols, swizzle_atom32};
    auto it = ctx->tmap_cache.find(key);
    if (it != ctx->tmap_cache.end()) { *out = it->second; return B200_OK; }
    if (!ctx->encode_tiled) return B200_ERR_STATE;
    if (!b200_aligned16(ptr) || (ld * 4) % 16 != 0) return B200_ERR_ALIGN;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {ld * sizeof(float)};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUtensorMap m;
    CUresult r = ctx->encode_tiled(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(ptr), dims,
                                   strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                   swizzle_atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        ctx->last_error = "cuTensorMapEncodeTiled failed with CUresult " + std::to_string((int)r);
        return B200_ERR_CUDA;
    }
    if (ctx->tmap_cache.size() > 4096) ctx->tmap_cache.clear();
    ctx->tmap_cache.emplace(key, m);
    *out = m;
    return B200_OK;
}

int b200_get_tensor_map_bf16(b200_ctx* ctx, CUtensorMap* out, const void* ptr, uint64_t rows,
                             uint64_t cols, uint64_t ld, uint32_t box_rows, uint32_t box_cols) {
    TensorMapKey key{ptr, rows, cols, ld, box_rows, box_cols, 2};  // 2: 16-bit elements
    auto it = ctx->tmap_cache.find(key);
    if (it != ctx->tmap_cache.end()) { *out = it->second; return B200_OK; }
    if (!ctx->encode_tiled) return B200_ERR_STATE;
    if (!b200_aligned16(ptr) || (ld * 2) % 16 != 0) return B200_ERR_ALIGN;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {ld * 2};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUtensorMap m;
    CUresult r = ctx->encode_tiled(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims,
                                   strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        ctx->last_error = "cuTensorMapEncodeTiled (bf16) failed with CUresult " + std::to_string((int)r);
        return B200_ERR_CUDA;
    }
    if (ctx->tmap_cache.size() > 4096) ctx->tmap_cache.clear();
    ctx->tmap_cache.emplace(key, m);
    *out = m;
    return B200_OK;
}

int b200_get_tensor_map_u8(b200_ctx* ctx, CUtensorMap* out, const void* ptr, uint64_t rows,
                           uint64_t cols, uint64_t ld, uint32_t box_rows, uint32_t box_cols) {
    TensorMapKey key{ptr, rows, cols, ld, box_rows, box_cols, 3};  // 3: 8-bit elements
    auto it = ctx->tmap_cache.find(key);
    if (it != ctx->tmap_cache.end()) { *out = it->second; return B200_OK; }
    if (!ctx->encode_tiled) return B200_ERR_STATE;
    if (!b200_aligned16(ptr) || ld % 16 != 0) return B200_ERR_ALIGN;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {ld};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUtensorMap m;
    CUresult r = ctx->encode_tiled(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims,
                                   strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        ctx->last_error = "cuTensorMapEncodeTiled (8-bit) failed with CUresult " + std::to_string((int)r);
        return B200_ERR_CUDA;
    }
    if (ctx->tmap_cache.size() > 4096) ctx->tmap_cache.clear();
    ctx->tmap_cache.emplace(key, m);
    *out = m;
    return B200_OK;
}

extern "C" {

const char* b200_status_string(int s) {
    switch (s) {
        case B200_OK: return "ok";
        case B200_ERR_NULL: return "required pointer is NULL";
        case B200_ERR_SHAPE: return "dimension violates a precondition";
        case B200_ERR_ALIGN: return "pointer is not 16-byte aligned";
        case B200_ERR_CUDA: return "CUDA call failed";
        case B200_ERR_DEVICE: return "device is not sm_100";
        case B200_ERR_TIMEOUT: return "device-side wait ran out";
        case B200_ERR_STATE: return "object not set up";
        case B200_ERR_LIMIT: return "size beyond the stated maximum";
        default: return "unknown status";
    }
}

int b200_ctx_create(b200_ctx** out, int device, void* stream) {
    if (!out) return B200_ERR_NULL;
    *out = nullptr;
    b200_ctx* ctx = new b200_ctx();
    ctx->device = device;
    ctx->stream = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaSetDevice(device);
    cudaDeviceProp prop;
    if (e == cudaSuccess) e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) { delete ctx; return B200_ERR_CUDA; }
    if (prop.major != 10) { delete ctx; return B200_ERR_DEVICE; }
    ctx->num_sms = prop.multiProcessorCount;
    e = cudaMalloc(&ctx->d_status, 256);
    if (e == cudaSuccess) e = cudaMemset(ctx->d_status, 0, 256);
    if (e == cudaSuccess) e = cudaHostAlloc(&ctx->h_status, sizeof(int), cudaHostAllocDefault);
    ctx->split_flag_words = (size_t)1 << 18;  // 1 MB: up to 16384 K-slice tiles per launch
    if (e == cudaSuccess) e = cudaMalloc(&ctx->d_split_flags, ctx->split_flag_words * sizeof(unsigned int));
    if (e == cudaSuccess) e = cudaMemset(ctx->d_split_flags, 0, ctx->split_flag_words * sizeof(unsigned int));
    if (e != cudaSuccess) { cudaFree(ctx->d_status); cudaFree(ctx->d_split_flags); delete ctx; return B200_ERR_CUDA; }
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) {
        cudaFree(ctx->d_status);
        cudaFree(ctx->d_split_flags);
        cudaFreeHost(ctx->h_status);
        delete ctx;
        return B200_ERR_CUDA;
    }
    ctx->encode_tiled = reinterpret_cast<b200_encode_tiled_fn>(fn);
    if (const char* e = getenv("B200_PDL")) ctx->pdl = !(e[0] == '0');
    *out = ctx;
    return B200_OK;
}

int b200_ctx_destroy(b200_ctx* ctx) {
    if (!ctx) return B200_ERR_NULL;
    cudaSetDevice(ctx->device);
    cudaFree(ctx->d_status);
    cudaFree(ctx->d_split_flags);
    cudaFreeHost(ctx->h_status);
    delete ctx;
    return B200_OK;
}

int b200_ctx_set_stream(b200_ctx* ctx, void* stream) {
    if (!ctx) return B200_ERR_NULL;
    ctx->stream = static_cast<cudaStream_t>(stream);
    return B200_OK;
}

int b200_ctx_sync_check(b200_ctx* ctx) {
    if (!ctx) return B200_ERR_NULL;
    // the status word rides behind the queued work: one wait for both
    B200_CUDA(ctx, cudaMemcpyAsync(ctx->h_status, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    B200_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    const int word = *ctx->h_status;
    if (word != 0) {
        // the whole area: a kernel that gave up may have left its work counters behind (and a GEMM
        // with K slices its hand-over flags)
        B200_CUDA(ctx, cudaMemset(ctx->d_status, 0, 256));
        B200_CUDA(ctx, cudaMemset(ctx->d_split_flags, 0, ctx->split_flag_words * sizeof(unsigned int)));
        ctx->last_error = "device status word = " + std::to_string(word);
        return word == 201 ? B200_ERR_SHAPE : B200_ERR_TIMEOUT;
    }
    B200_CUDA(ctx, cudaGetLastError());
    return B200_OK;
}

int b200_ctx_wait_timeout_probe(b200_ctx* ctx, int limit_ms) {
    if (!ctx) return B200_ERR_NULL;
    if (limit_ms < 1 || limit_ms > 2000) return B200_ERR_SHAPE;
    return b200::launch_wait_timeout_probe(ctx, (unsigned long long)limit_ms * 1000000ull);
}

int b200_ctx_peer_wait_probe(b200_ctx* ctx, int limit_ms) {
    if (!ctx) return B200_ERR_NULL;
    if (limit_ms < 1 || limit_ms > 2000) return B200_ERR_SHAPE;
    // word 40 of the status area is never written: the wait for it to reach 1 runs out
    return b200::launch_peer_wait(ctx, reinterpret_cast<const unsigned int*>(ctx->d_status + 40), 1u, (unsigned long long)limit_ms * 1000000ull);
}

// debugging aid for kernel experiments: device address of the status words
void* b200_ctx_debug_status(b200_ctx* ctx) { return ctx ? ctx->d_status : nullptr; }

uint64_t b200_ctx_launch_count(const b200_ctx* ctx) { return ctx ? ctx->launches : 0; }
void b200_ctx_reset_launch_count(b200_ctx* ctx) { if (ctx) ctx->launches = 0; }
const char* b200_ctx_last_error(const b200_ctx* ctx) { return ctx ? ctx->last_error.c_str() : ""; }

#define REQUIRE_PTR(p) do { if (!(p)) return B200_ERR_NULL; if (!b200_aligned16(p)) return B200_ERR_ALIGN; } while (0)
#define OPTIONAL_PTR(p) do { if ((p) && !b200_aligned16(p)) return B200_ERR_ALIGN; } while (0)

int b200_matmul_forward(b200_ctx* ctx, float* out, const float* inp, const float* weight,
                        const float* bias, int B, int T, int C, int OC, int act,
                        const float* residual, int mode) {
    if (!ctx) return B200_ERR_NULL;
    REQUIRE_PTR(out); REQUIRE_PTR(inp); REQUIRE_PTR(weight);
    OPTIONAL_PTR(bias); OPTIONAL_PTR(residual);
    if (B <= 0 || T <= 0 || C <= 0 || OC <= 0 || C % 4 || OC % 4) return B200_ERR_SHAPE;
    if ((long long)B * T > 0x7fffffffLL) return B200_ERR_SHAPE;
    if (act != B200_ACT_NONE && act != B200_ACT_GELU) return B200_ERR_SHAPE;
    if (mode != B200_TF32 && mode != B200_TF32X3) return B200_ERR_SHAPE;
    int flags = act == B200_ACT_GELU ? b200::GEMM_GELU : 0;
    if (residual == out) {  // in place: the tiles are added onto out as they retire
        flags |= b200::GEMM_ACCUM_OUT;
        residual = nullptr;
    }
    return b200::launch_gemm_tf32(ctx, out, inp, weight, bias, residual, B * T, C, OC, flags, mode);
}

int b200_matmul_forward_bf16x3(b200_ctx* ctx, float* out, uint16_t* out_split, const uint16_t* inp_split,
                               const uint16_t* weight_hi, const uint16_t* weight_lo, const float* bias, int B, int T,
                               int C, int OC, int act, int accumulate) {
    if (!ctx) return B200_ERR_NULL;
    if (out_split) { REQUIRE_PTR(out_split); } else { REQUIRE_PTR(out); }
    REQUIRE_PTR(inp_split); REQUIRE_PTR(weight_hi); REQUIRE_PTR(weight_lo);
    OPTIONAL_PTR(bias);
    if (B <= 0 || T <= 0 || C <= 0 || OC <= 0 || C % 8 || OC % 8) return B200_ERR_SHAPE;
    if ((long long)B * T > 0x7fffffffLL) return B200_ERR_SHAPE;
    if (act != B200_ACT_NONE && act != B200_ACT_GELU) return B200_ERR_SHAPE;
    if (out_split && (accumulate || ((long long)B * T) % 32)) return B200_ERR_SHAPE;
    return b200::launch_gemm_bf16x3(ctx, out, out_split, inp_split, weight_hi, weight_lo, bias, B * T, C, OC,
                                    (act == B200_ACT_GELU ? b200::GEMM_GELU : 0) | (accumulate ? b200::GEMM_ACCUM_OUT : 0));
}

int b200_split_bf16(b200_ctx* ctx, uint16_t* hi, uint16_t* lo, const float* inp, size_t n) {
    if (!ctx) return B200_ERR_NULL;
    REQUIRE_PTR(hi); REQUIRE_PTR(lo); REQUIRE_PTR(inp);
    if (n == 0 || n % 4) return B200_ERR_SHAPE;
    return b200::launch_convert_bf16(ctx, hi, inp, n, lo);
}

int b200_quantize_e4m3(b200_ctx* ctx, uint8_t* out, const float* inp, size_t n, float scale) {
    if (!ctx) return B200_ERR_NULL;
    REQUIRE_PTR(out); REQUIRE_PTR(inp);
    if (n == 0 || n % 4 || !(scale > 0.f)) return B200_ERR_SHAPE;
    return b200::launch_quantize_e4m3(ctx, out, inp, n, scale);
}

int b200_matmul_forward_fp8(b200_ctx* ctx, float* out, const uint8_t* inp, const uint8_t* weight, const float* bias,
                            int B, int T, int C, int OC, int act, float alpha, int accumulate) {
    if (!ctx) return B200_ERR_NULL;
    REQUIRE_PTR(out); REQUIRE_PTR(inp); REQUIRE_PTR(weight);
    OPTIONAL_PTR(bias);
    if (B <= 0 || T <= 0 || C <= 0 || OC <= 0 || C % 16 || OC % 8) return B200_ERR_SHAPE;
    if ((long long)B * T > 0x7fffffffLL) return B200_ERR_SHAPE;
    if (act != B200_ACT_NONE && act != B200_ACT_GELU) return B200_ERR_SHAPE;
    if (accumulate && act != B200_ACT_NONE) return B200_ERR_SHAPE;
    return b200::launch_gemm_fp8(ctx, out, inp, weight, bias, B * T, C, OC,
                                 (act == B200_ACT_GELU ? b200::GEMM_GELU : 0) | (accumulate ? b200::GEMM_ACCUM_OUT : 0), alpha);
}

int b200_matmul_forward_bf16(b200_ctx* ctx, float* out, uint16_t* out_bf16, const uint16_t* inp,
                             const uint16_t* weight, const float* bias, int B, int T, int C, int OC, int act) {
    if (!ctx) return B200_ERR_NULL;
    if (out_bf16) { REQUIRE_PTR(out_bf16); } else { REQUIRE_PTR(out); }
    REQUIRE_PTR(inp); REQUIRE_PTR(weight);
    OPTIONAL_PTR(bias);
    if (B <= 0 || T <= 0 || C <= 0 || OC <= 0 || C % 8 || OC % 8) return B200_ERR_SHAPE;
    if ((long long)B * T > 0x7fffffffLL) return B200_ERR_SHAPE;
    if (act != B200_ACT_NONE && act != B200_ACT_GELU) return B200_ERR_SHAPE;
    return b200::launch_gemm_bf16(ctx, out, out_bf16, inp, weight, bias, B * T, C, OC,
                                  act == B200_ACT_GELU ? b200::GEMM_GELU : 0);
}

int b200_sample_rows(b200_ctx* ctx, int* out, const float* logits, int M, int V, int ld, float temperature,
                     int top_k, float top_p, unsigned int seed, unsigned int stream0) {
    if (!ctx || !out || !logits) return B200_ERR_NULL;
    if (M <= 0 || V <= 0 || ld < V || top_k < 0) return B200_ERR_SHAPE;
    if (temperature <= 0.f && (ld % 4 || !b200_aligned16(logits))) return B200_ERR_ALIGN;  // the arg-max reads float4
    return b200::launch_sample_rows(ctx, out, logits, M, V, ld, temperature, seed, stream0, top_k, top_p);
}

int b200_convert_bf16(b200_ctx* ctx, uint16_t* out, const float* inp, size_t n) {
    if (!ctx) return B200_ERR_NULL;
    REQUIRE_PTR(out); REQUIRE_PTR(inp);
    if (n == 0 || n % 4) return B200_ERR_SHAPE;
    return b200::launch_convert_bf16(ctx, out, inp, n);
}

int b200_attention_forward(b200_ctx* ctx, float* out, float* qkvr, float* att, const float* inp,
                           int B, int T, int C, int NH) {
    (void)qkvr;
    if (!ctx) return B200_ERR_NULL;
    REQUIRE_PTR(out); REQUIRE_PTR(inp); OPTIONAL_PTR(att);
    if (B <= 0 || T <= 0 || C <= 0 || NH <= 0 || C % NH || C / NH != 64 || T % 64) return B200_ERR_SHAPE;
    return b200::launch_attention(ctx, out, att, inp, B, T, C, NH, 0);
}

int b200_attention_forward_x3(b200_ctx* ctx, float* out, float* qkvr, float* att, const float* inp,
                              int B, int T, int C, int NH) {
    if (!ctx) return B200_ERR_NULL;
    REQUIRE_PTR(out); REQUIRE_PTR(inp); REQUIRE_PTR(qkvr); OPTIONAL_PTR(att);
    if (B <= 0 || T <= 0 || C <= 0 || NH <= 0 || C % NH || C / NH != 64 || T % 64) return B200_ERR_SHAPE;
    return b200::launch_attention_x3(ctx, out, qkvr, att, inp, B, T, C, NH);
}

int b200_split_fp16(b200_ctx* ctx, uint16_t* hi, uint16_t* lo, const float* inp, size_t n) {
    if (!ctx) return B200_ERR_NULL;
    REQUIRE_PTR(hi); REQUIRE_PTR(lo); REQUIRE_PTR(inp);
    if (n == 0 || n % 4) return B200_ERR_SHAPE;
    return b200::launch_split_fp16(ctx, hi, lo, inp, n);
}

int b200_attention_forward_fp16(b200_ctx* ctx, float* out, float* att, const uint16_t* inp_split,
                                int B, int T, int C, int NH) {
    if (!ctx) return B200_ERR_NULL;
    REQUIRE_PTR(out); REQUIRE_PTR(inp_split); OPTIONAL_PTR(att);
    if (B <= 0 || T <= 0 || C <= 0 || NH <= 0 || C % NH || C / NH != 64 || T % 64) return B200_ERR_SHAPE;
    return b200::launch_attention_split(ctx, out, att, inp_split, B, T, C, NH, 0);
}

int b200_layernorm_forward(b200_ctx* ctx, float* out, float* mean, float* rstd, const float* inp,
                           const float* weight, const float* bias, int B, int T, int C) {
    if (!ctx) return B200_ERR_NULL;
    REQUIRE_PTR(out); REQUIRE_PTR(inp); REQUIRE_PTR(weight); REQUIRE_PTR(bias);
    if (B <= 0 || T <= 0 || C <= 0 || C % 4 || C > 4096) return B200_ERR_SHAPE;
    return b200::launch_layernorm(ctx, out, mean, rstd, inp, weight, bias, B * T, C, 0);
}

int b200_fused_residual_layernorm_forward(b200_ctx* ctx, float* res_out, float* layernorm_out,
                                          float* mean, float* rstd, const float* inp1,
                                          const float* inp2, const float* weight,
                                          const float* bias, int B, int T, int C) {
    if (!ctx) return B200_ERR_NULL;
    REQUIRE_PTR(res_out); REQUIRE_PTR(layernorm_out); REQUIRE_PTR(inp1); REQUIRE_PTR(inp2);
    REQUIRE_PTR(weight); REQUIRE_PTR(bias);
    if (B <= 0 || T <= 0 || C <= 0 || C % 4 || C > 4096) return B200_ERR_SHAPE;
    return b200::launch_fused_residual_layernorm(ctx, res_out, layernorm_out, mean, rstd, inp1, inp2,
                                                 weight, bias, B * T, C, 0);
}

int b200_residual_forward(b200_ctx* ctx, float* out, const float* inp1, const float* inp2, size_t N) {
    if (!ctx) return B200_ERR_NULL;
    REQUIRE_PTR(out); REQUIRE_PTR(inp1); REQUIRE_PTR(inp2);
    if (N == 0) return B200_OK;
    return b200::launch_residual(ctx, out, inp1, inp2, N);
}

int b200_gelu_forward(b200_ctx* ctx, float* out, const float* inp, size_t N) {
    if (!ctx) return B200_ERR_NULL;
    REQUIRE_PTR(out); REQUIRE_PTR(inp);
    if (N == 0) return B200_OK;
    return b200::launch_gelu(ctx, out, inp, N);
}

int b200_encoder_forward(b200_ctx* ctx, float* out, const int* inp, const float* wte,
                         const float* wpe, int B, int T, int C) {
    if (!ctx) return B200_ERR_NULL;
    REQUIRE_PTR(out); REQUIRE_PTR(wte); REQUIRE_PTR(wpe);
    if (!inp) return B200_ERR_NULL;
    if (B <= 0 || T <= 0 || C <= 0 || C % 4) return B200_ERR_SHAPE;
    return b200::launch_encoder(ctx, out, inp, wte, wpe, B, T, C, 0);
}

// ----------------------------------------------------------------- void shims
static b200_ctx* default_ctx() {
    // one context per device, created on first use, bound to the legacy default stream
    static std::mutex mu;
    static b200_ctx* ctxs[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        fprintf(stderr, "b200gpt2: no current CUDA device\n");
        abort();
    }
    std::lock_guard<std::mutex> lock(mu);
    if (!ctxs[dev]) {
        int st = b200_ctx_create(&ctxs[dev], dev, nullptr);
        if (st != B200_OK) {
            fprintf(stderr, "b200gpt2: cannot create a context on device %d: %s\n", dev, b200_status_string(st));
            abort();
        }
    }
    return ctxs[dev];
}

static void shim_check(int st, const char* what) {
    if (st != B200_OK) {
        fprintf(stderr, "b200gpt2: %s failed: %s\n", what, b200_status_string(st));
        abort();
    }
}

void matmul_forward(float* out, const float* inp, const float* weight, const float* bias, int B,
                    int T, int C, int OC) {
    shim_check(b200_matmul_forward(default_ctx(), out, inp, weight, bias, B, T, C, OC, B200_ACT_NONE, nullptr, B200_TF32),
               "matmul_forward");
}
void matmul_forward_gelu(float* out, const float* inp, const float* weight, const float* bias,
                         int B, int T, int C, int OC, int is_gelu) {
    shim_check(b200_matmul_forward(default_ctx(), out, inp, weight, bias, B, T, C, OC,
                                   is_gelu ? B200_ACT_GELU : B200_ACT_NONE, nullptr, B200_TF32),
               "matmul_forward_gelu");
}
void attention_forward(float* out, float* qkvr, float* att, const float* inp, int B, int T, int C, int NH) {
    shim_check(b200_attention_forward(default_ctx(), out, qkvr, att, inp, B, T, C, NH), "attention_forward");
}
void layernorm_forward(float* out, float* mean, float* rstd, const float* inp, const float* weight,
                       const float* bias, int B, int T, int C) {
    shim_check(b200_layernorm_forward(default_ctx(), out, mean, rstd, inp, weight, bias, B, T, C), "layernorm_forward");
}
void fused_residual_layernorm_forward(float* res_out, float* layernorm_out, float* mean, float* rstd,
                                      const float* inp1, const float* inp2, const float* weight,
                                      const float* bias, int B, int T, int C) {
    shim_check(b200_fused_residual_layernorm_forward(default_ctx(), res_out, layernorm_out, mean, rstd, inp1,
                                                     inp2, weight, bias, B, T, C),
               "fused_residual_layernorm_forward");
}
void fused_residual_layernorm(float* res_out, float* layernorm_out, float* mean, float* rstd,
                              const float* inp1, const float* inp2, const float* weight,
                              const float* bias, int B, int T, int C) {
    fused_residual_layernorm_forward(res_out, layernorm_out, mean, rstd, inp1, inp2, weight, bias, B, T, C);
}
void residual_forward(float* out, const float* inp1, const float* inp2, int N) {
    shim_check(N < 0 ? B200_ERR_SHAPE : b200_residual_forward(default_ctx(), out, inp1, inp2, (size_t)N), "residual_forward");
}
void gelu_forward(float* out, const float* inp, int N) {
    shim_check(N < 0 ? B200_ERR_SHAPE : b200_gelu_forward(default_ctx(), out, inp, (size_t)N), "gelu_forward");
}
void encoder_forward(float* out, const int* inp, const float* wte, const float* wpe, int B, int T, int C) {
    shim_check(b200_encoder_forward(default_ctx(), out, inp, wte, wpe, B, T, C), "encoder_forward");
}

}  // extern "C"
