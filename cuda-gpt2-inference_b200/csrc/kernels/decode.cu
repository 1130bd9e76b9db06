// Incremental decoding: one new token per sequence against a key/value cache.
// Not part of the reference (it has full-sequence kernels only); the operators are the same as
// in the full forward - matmul + bias (+ tanh-GELU) as in kernels/matmul/1_matmul_tiling.cuh:25-54
// and 9_matmul_async_cg_tf32_gelu.cuh:5-11, causal attention with scale 1/sqrt(HS) as in
// kernels/attention/1_attention_cublas.cuh:50-61 - evaluated for M = B rows (B <= 16).
// With so few rows every weight is used B times only: the step is bound by reading the weights
// and the cache out of HBM once, not by arithmetic, so these kernels run on the fp32 FMA pipe
// (exact fp32 products, no TF32 rounding) and are organised around coalesced streaming:
//   skinny_gemm_kernel      out[b,n] = act(sum_k x[b,k] W[n,k] + bias[n]); a warp streams ROWS rows
//                           of W, 128 floats per step, against x staged in shared memory
//   kv_append_kernel        K and V columns of freshly computed qkv rows -> cache
//   decode_attention_kernel one CTA per (sequence, head): half-warps walk the cached positions
//                           with an online softmax, states are merged through shared memory
#include "kernels.h"
#include "../prim/sm100.cuh"

namespace b200 {

namespace {

constexpr int kSkinnyThreads = 256;
constexpr int kSkinnyKC = 1024;  // floats of K staged per pass (x chunk: NB * 4 KB of shared memory)

template <int NB, int ROWS>
__global__ void __launch_bounds__(kSkinnyThreads)
skinny_gemm_kernel(float* __restrict__ out, const float* __restrict__ x, const float* __restrict__ W,
                   const float* __restrict__ bias, int B, int N, int K, int gelu) {
    extern __shared__ float4 xs4[];  // [NB][kSkinnyKC / 4]
    griddep_wait();
    griddep_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int kWarps = kSkinnyThreads / 32;
    const int groups = (N + ROWS - 1) / ROWS;                  // row groups, one per warp at a time
    const int batches = (groups + kWarps - 1) / kWarps;        // a CTA takes kWarps groups at a time
    for (int batch = blockIdx.x; batch < batches; batch += gridDim.x) {
        const int n0 = (batch * kWarps + warp) * ROWS;
        float acc[ROWS][NB];
#pragma unroll
        for (int r = 0; r < ROWS; ++r)
#pragma unroll
            for (int b = 0; b < NB; ++b) acc[r][b] = 0.f;
        const float* wrow[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) wrow[r] = W + (size_t)min(n0 + r, N - 1) * K;  // clamped: masked at the store

        for (int kc0 = 0; kc0 < K; kc0 += kSkinnyKC) {
            const int kc = min(kSkinnyKC, K - kc0);  // multiple of 4
            __syncthreads();                         // the previous chunk is no longer read
            for (int i = threadIdx.x; i < NB * (kSkinnyKC / 4); i += kSkinnyThreads) {
                const int b = i / (kSkinnyKC / 4), k4 = i % (kSkinnyKC / 4);
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (b < B && k4 * 4 < kc) v = *reinterpret_cast<const float4*>(x + (size_t)b * K + kc0 + k4 * 4);
                xs4[i] = v;
            }
            __syncthreads();
            if (n0 < N) {
                const int steps = (kc + 127) / 128;
#pragma unroll 2
                for (int s = 0; s < steps; ++s) {
                    const int k4 = s * 32 + lane;  // float4 index inside the chunk
                    float4 w[ROWS];
#pragma unroll
                    for (int r = 0; r < ROWS; ++r)
                        w[r] = (k4 * 4 < kc) ? __ldg(reinterpret_cast<const float4*>(wrow[r] + kc0) + k4)
                                             : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int b = 0; b < NB; ++b) {
                        const float4 xv = xs4[b * (kSkinnyKC / 4) + k4];
#pragma unroll
                        for (int r = 0; r < ROWS; ++r)
                            acc[r][b] += (w[r].x * xv.x + w[r].y * xv.y) + (w[r].z * xv.z + w[r].w * xv.w);
                    }
                }
            }
        }
        // sum over the 32 lanes; afterwards every lane holds every total
#pragma unroll
        for (int r = 0; r < ROWS; ++r)
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                float v = acc[r][b];
#pragma unroll
                for (int s = 16; s >= 1; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
                acc[r][b] = v;
            }
        // lane i stores the totals i, i + 32, ... of the ROWS x NB block (row-major)
#pragma unroll
        for (int r = 0; r < ROWS; ++r)
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                if (((r * NB + b) & 31) == lane && n0 + r < N && b < B) {
                    float v = acc[r][b] + (bias ? __ldg(bias + n0 + r) : 0.f);
                    if (gelu) v = gelu_tanh(v);
                    out[(size_t)b * N + n0 + r] = v;
                }
            }
    }
}

// qkv rows [rows = B*T, 3C] (q | k | v): the k and v parts go to cache[b][pos0 + t][C]
__global__ void kv_append_kernel(float4* __restrict__ kcache, float4* __restrict__ vcache,
                                 const float4* __restrict__ qkv, int B, int T, int C4, int pos0, int cache_T) {
    griddep_wait();
    griddep_launch_dependents();
    const size_t total = (size_t)B * T * C4;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % C4);
        const size_t row = i / C4;
        const int t = (int)(row % T), b = (int)(row / T);
        const size_t dst = ((size_t)b * cache_T + pos0 + t) * C4 + c;
        kcache[dst] = qkv[row * 3 * C4 + C4 + c];
        vcache[dst] = qkv[row * 3 * C4 + 2 * C4 + c];
    }
}

constexpr int kDecAttThreads = 256;

// q: row b of qkv [B, 3C] (first C columns); caches [B][cache_T][C]; positions 0..pos take part
__global__ void __launch_bounds__(kDecAttThreads)
decode_attention_kernel(float* __restrict__ out, const float* __restrict__ qkv, const float* __restrict__ kcache,
                        const float* __restrict__ vcache, int C, int pos, int cache_T) {
    __shared__ float st_m[16], st_l[16];
    __shared__ float st_o[16][64];
    griddep_wait();
    griddep_launch_dependents();
    const int h = blockIdx.x, b = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int half = lane >> 4, hl = lane & 15;  // a half-warp covers the 64 floats of one cached row
    const int slot = warp * 2 + half;            // 16 half-warps walk positions slot, slot + 16, ...
    const float scale = 0.125f;                  // 1 / sqrt(64)
    float4 q = *reinterpret_cast<const float4*>(qkv + (size_t)b * 3 * C + h * 64 + hl * 4);
    q.x *= scale; q.y *= scale; q.z *= scale; q.w *= scale;
    const float* kbase = kcache + (size_t)b * cache_T * C + h * 64 + hl * 4;
    const float* vbase = vcache + (size_t)b * cache_T * C + h * 64 + hl * 4;
    float m = -INFINITY, l = 0.f;
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    // every half-warp makes the same number of trips so that the shuffles stay warp-wide
    const int trips = (pos + 16) / 16;
    for (int i = 0; i < trips; ++i) {
        const int t = i * 16 + slot;
        const bool live = t <= pos;
        float4 k4 = make_float4(0.f, 0.f, 0.f, 0.f), v4 = k4;
        if (live) {
            k4 = __ldg(reinterpret_cast<const float4*>(kbase + (size_t)t * C));
            v4 = __ldg(reinterpret_cast<const float4*>(vbase + (size_t)t * C));
        }
        float s = (q.x * k4.x + q.y * k4.y) + (q.z * k4.z + q.w * k4.w);
#pragma unroll
        for (int d = 8; d >= 1; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);  // within the half-warp
        if (live) {
            const float mn = fmaxf(m, s);
            const float corr = expf(m - mn), p = expf(s - mn);  // corr = 0 on the first position
            l = l * corr + p;
            o.x = o.x * corr + p * v4.x; o.y = o.y * corr + p * v4.y;
            o.z = o.z * corr + p * v4.z; o.w = o.w * corr + p * v4.w;
            m = mn;
        }
    }
    if (hl == 0) { st_m[slot] = m; st_l[slot] = l; }
    *reinterpret_cast<float4*>(&st_o[slot][hl * 4]) = o;
    __syncthreads();
    if (threadIdx.x < 64) {
        const int d = threadIdx.x;
        float mm = -INFINITY;
#pragma unroll
        for (int i = 0; i < 16; ++i) mm = fmaxf(mm, st_m[i]);
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float w = (st_m[i] == -INFINITY) ? 0.f : expf(st_m[i] - mm);  // a half-warp may have seen nothing
            L += st_l[i] * w;
            O += st_o[i][d] * w;
        }
        out[(size_t)b * C + h * 64 + d] = O / L;
    }
}

}  // namespace

int launch_skinny_gemm(b200_ctx* ctx, float* out, const float* x, const float* W, const float* bias, int B,
                       int K, int N, int gelu) {
    if (B < 1 || B > 16 || K % 4 || N < 1) return B200_ERR_SHAPE;
    const int nb = B <= 8 ? 8 : 16;
    // many rows: four per warp (each x value read from shared memory serves four rows); few rows:
    // two per warp, so that more SMs take part
    const int rows = (N >= 64 * ctx->num_sms) ? 4 : 2;
    const int groups = (N + rows - 1) / rows, batches = (groups + 7) / 8;
    const int grid = batches < 4 * ctx->num_sms ? batches : 4 * ctx->num_sms;
    const size_t smem = (size_t)nb * kSkinnyKC * sizeof(float);
    cudaError_t le = cudaSuccess;
#define B200_SKINNY(NB, ROWS)                                                                                       \
    do {                                                                                                            \
        static bool attr_set[64] = {};                                                                              \
        if (!attr_set[ctx->device & 63]) {                                                                          \
            B200_CUDA(ctx, cudaFuncSetAttribute(skinny_gemm_kernel<NB, ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
            attr_set[ctx->device & 63] = true;                                                                      \
        }                                                                                                           \
        le = launch_pdl(ctx, skinny_gemm_kernel<NB, ROWS>, dim3(grid), dim3(kSkinnyThreads), smem, out, x, W, bias, B, N, K, gelu); \
    } while (0)
    if (nb == 8 && rows == 4) B200_SKINNY(8, 4);
    else if (nb == 8) B200_SKINNY(8, 2);
    else if (rows == 4) B200_SKINNY(16, 4);
    else B200_SKINNY(16, 2);
#undef B200_SKINNY
    ctx->launches++;
    B200_CUDA(ctx, le);
    return B200_OK;
}

int launch_kv_append(b200_ctx* ctx, float* kcache, float* vcache, const float* qkv, int B, int T, int C, int pos0,
                     int cache_T) {
    const size_t total = (size_t)B * T * (C / 4);
    const int grid = (int)((total + 255) / 256 < (size_t)8 * ctx->num_sms ? (total + 255) / 256 : (size_t)8 * ctx->num_sms);
    cudaError_t le = launch_pdl(ctx, kv_append_kernel, dim3(grid), dim3(256), 0, reinterpret_cast<float4*>(kcache),
                                reinterpret_cast<float4*>(vcache), reinterpret_cast<const float4*>(qkv), B, T, C / 4,
                                pos0, cache_T);
    ctx->launches++;
    B200_CUDA(ctx, le);
    return B200_OK;
}

int launch_decode_attention(b200_ctx* ctx, float* out, const float* qkv, const float* kcache, const float* vcache,
                            int B, int C, int NH, int pos, int cache_T) {
    cudaError_t le = launch_pdl(ctx, decode_attention_kernel, dim3(NH, B), dim3(kDecAttThreads), 0, out, qkv, kcache,
                                vcache, C, pos, cache_T);
    ctx->launches++;
    B200_CUDA(ctx, le);
    return B200_OK;
}

}  // namespace b200
