// Harness that exposes the reference project's own CUDA kernels through a C ABI.
// TEST INFRASTRUCTURE ONLY: it is built (oracle/Makefile, target `ref`) straight from the
// reference's headers where they lie (REF_ROOT, never copied into this repository) into
// oracle/_ref/libref_kernels.so, and is used (a) to record the golden fixtures under
// tests/golden/ and (b) to cross-check the CPU oracle on a GPU.  The product library
// never loads it.
//
// Only kernels that compile and are correct by reading are exposed:
//   kernels/matmul/1_matmul_tiling.cuh:57        matmul_forward_tiling (fp32 FMA, the math spec)
//   kernels/matmul/9_matmul_async_cg_tf32_gelu.cuh:237  TF32 wmma GEMM with bias (+GELU)
//   kernels/attention/3_flash_attention_permute.cuh:346 causal flash attention on packed QKV
//   kernels/layernorm/1_layernorm_block.cuh:63   layernorm (needs C == 4*blockDim, C <= 4096)
//   kernels/layernorm/2_layernorm_block_vectorized.cuh:74
//   kernels/residual/1_residual_naive.cuh:15     residual add
// Every pointer is a device pointer.  Each wrapper synchronises and returns the CUDA
// error code (0 = success).
#include <cassert>
#include <cfloat>
#include <cmath>
#include <cstdint>
#include <cuda_runtime.h>
#include "kernels/matmul/1_matmul_tiling.cuh"
#include "kernels/matmul/9_matmul_async_cg_tf32_gelu.cuh"
#include "kernels/attention/3_flash_attention_permute.cuh"
#include "kernels/layernorm/1_layernorm_block.cuh"
#include "kernels/layernorm/2_layernorm_block_vectorized.cuh"
#include "kernels/residual/1_residual_naive.cuh"

static int finish() {
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaGetLastError();
    return (int)e;
}

extern "C" {
int ref_matmul_forward_tiling(float* out, const float* inp, const float* weight, const float* bias,
                              int B, int T, int C, int OC) {
    matmul_forward_tiling(out, inp, weight, bias, B, T, C, OC);
    return finish();
}
int ref_matmul_forward_tf32_gelu(float* out, const float* inp, const float* weight,
                                 const float* bias, int B, int T, int C, int OC, int is_gelu) {
    if (C % 16 || OC % 128 || (B * T) % 128 || bias == nullptr) return -1;
    matmul_forward_async_cg_tf32_gelu(out, inp, weight, bias, B, T, C, OC, is_gelu != 0);
    return finish();
}
int ref_flash_attention_permute_forward(float* out, const float* inp, int B, int T, int C, int NH) {
    if (C / NH != 64 || T % 64) return -1;
    flash_attention_permute_forward(out, nullptr, nullptr, inp, B, T, C, NH);
    return finish();
}
int ref_layernorm_forward_block(float* out, float* mean, float* rstd, const float* inp,
                                const float* weight, const float* bias, int B, int T, int C) {
    if (C % 4 || C / 4 > 1024) return -1;
    layernorm_forward_block(out, mean, rstd, inp, weight, bias, B, T, C);
    return finish();
}
int ref_layernorm_forward_block_vectorized(float* out, float* mean, float* rstd, const float* inp,
                                           const float* weight, const float* bias, int B, int T,
                                           int C) {
    if (C % 4 || C / 4 > 1024) return -1;
    layernorm_forward_block_vectorized(out, mean, rstd, inp, weight, bias, B, T, C);
    return finish();
}
int ref_residual_forward_naive(float* out, const float* inp1, const float* inp2, int N) {
    residual_forward_naive(out, inp1, inp2, N);
    return finish();
}
}
