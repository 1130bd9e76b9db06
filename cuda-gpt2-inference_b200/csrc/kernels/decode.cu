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
//                           (a variant that streamed W through a shared-memory ring with bulk
//                           copies was measured for the lm-head and was no faster)
//   kv_append_kernel        K and V columns of freshly computed qkv rows -> cache (prefill)
//   decode_attention_kernel one CTA per (sequence, head): stores the new position's K and V,
//                           then half-warps walk the cached positions with an online softmax
//                           and the states are merged through shared memory
//   decode_encoder_kernel   wte[token] + wpe[pos]
// The position is read from device memory, so one captured CUDA graph serves every step.
#include <cstdlib>
#include "kernels.h"
#include "../prim/sm100.cuh"

namespace b200 {

namespace {

constexpr int kSkinnyThreads = 256;
// STEPS (template): a warp covers 128 floats of a row per step and requests STEPS steps = STEPS * 128
// floats of K of its ROWS rows at once (8 steps = 8 float4 per lane and row; 6 for three rows per warp)

// Optional prologue (ln_w != nullptr): the input rows are first formed as
//   r = resid_in + branch (branch may be null),  x = layernorm(r) * ln_w + ln_b
// by every CTA for itself (B rows of C = K floats: a few KB), and CTA 0 also stores r to
// resid_out - a different buffer than resid_in, which other CTAs are still reading.  That is the
// forward's fused residual + layernorm (two-pass variance, eps 1e-5) without a kernel of its own.
struct SkinnyArgs {
    float* out;
    const float* x;         // [B,K] input rows, or resid_in when the prologue is on
    const float* W;
    const float* bias;
    const float* branch;    // prologue: added to x before the layernorm (nullable)
    const float* ln_w;      // prologue switch
    const float* ln_b;
    float* resid_out;       // prologue: r is stored here by CTA 0
    int B, N, K, gelu;
    int k_splits;       // > 1: K is cut into slices computed by different CTAs; slice s writes its partial sums to out + s*B*N
    int kslice;         // floats of K per slice (a multiple of 128; K when k_splits == 1)
    int branch_parts;   // prologue: branch holds this many partial results [parts][B][K], summed in order
};

// NV = float4 per lane that hold a row in the layernorm prologue (0: no prologue compiled in).
// (Splitting K between the warps of a row group, to put narrow outputs on more SMs, was measured
// and is slower: more batches per CTA means more weight round trips one after the other.)
template <int NB, int ROWS, int NV, int STEPS>
__global__ void __launch_bounds__(kSkinnyThreads)
skinny_gemm_kernel(const SkinnyArgs a) {
    constexpr int kSkinnySteps = STEPS, kSkinnyKC = STEPS * 128;
    extern __shared__ float4 xs4[];  // [NB][K / 4]: the input rows, staged once
    const int B = a.B, N = a.N, K = a.K, K4 = a.K >> 2;
    const float* __restrict__ W = a.W;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int kWarps = kSkinnyThreads / 32, kRowWarps = kWarps;
    const int rw = warp;
    const int groups = (N + ROWS - 1) / ROWS;                  // row groups, one per warp at a time
    const int batches = (groups + kRowWarps - 1) / kRowWarps;  // a CTA takes kRowWarps groups at a time
    // K slices (narrow outputs: more CTAs, each with a shorter chain of weight round trips; the
    // consumer's prologue adds the partial results up in slice order).  The grid is a multiple of
    // k_splits, so a CTA keeps its slice over all of its units.
    const int ks = blockIdx.x % a.k_splits;
    const int units = batches * a.k_splits;
    const int kbeg = ks * a.kslice, kend = min(K, kbeg + a.kslice);
    const int KS4 = (kend - kbeg) >> 2;  // staged floats per input row, in float4
    // The kernel is a chain of memory round trips (each several hundred to two thousand cycles),
    // so everything that does not depend on the previous kernel is requested before waiting for
    // it: the first chunk of this warp's weight rows, the bias, the layernorm parameters.
    float4 w[kSkinnySteps][ROWS];
    auto request_w = [&](int n0, int kc0) {
        const int kc = min(kSkinnyKC, kend - kc0);
#pragma unroll
        for (int s = 0; s < kSkinnySteps; ++s) {
            const int k4 = s * 32 + lane;  // float4 index inside the chunk
#pragma unroll
            for (int r = 0; r < ROWS; ++r)
                w[s][r] = (n0 < N && k4 * 4 < kc)
                              ? __ldg(reinterpret_cast<const float4*>(W + (size_t)min(n0 + r, N - 1) * K + kc0) + k4)
                              : make_float4(0.f, 0.f, 0.f, 0.f);  // rows clamped: masked at the store
        }
    };
    request_w(((blockIdx.x / a.k_splits) * kRowWarps + rw) * ROWS, kbeg);
    float4* lnw4 = xs4 + NB * K4;  // layernorm weight and bias, behind the input rows
    float4* lnb4 = lnw4 + K4;
    if (NV > 0) {
        for (int c = threadIdx.x; c < K4; c += kSkinnyThreads) {
            lnw4[c] = __ldg(reinterpret_cast<const float4*>(a.ln_w) + c);
            lnb4[c] = __ldg(reinterpret_cast<const float4*>(a.ln_b) + c);
        }
    }
    griddep_wait();
    griddep_launch_dependents();
    if (NV > 0) {
        __syncthreads();
        // one warp per row; a lane holds float4 number lane, lane + 32, ... of the row
        constexpr int NVV = NV > 0 ? NV : 1;
        for (int b = warp; b < NB; b += kWarps) {
            float4 v[NVV], t[NVV];
#pragma unroll
            for (int i = 0; i < NVV; ++i) {
                const int c = lane + i * 32;
                v[i] = t[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (b < B && c < K4) v[i] = *reinterpret_cast<const float4*>(a.x + (size_t)b * K + c * 4);
            }
            if (a.branch) {
#pragma unroll
                for (int i = 0; i < NVV; ++i) {
                    const int c = lane + i * 32;
                    if (b < B && c < K4) t[i] = *reinterpret_cast<const float4*>(a.branch + (size_t)b * K + c * 4);
                }
                for (int part = 1; part < a.branch_parts; ++part) {  // the producer's K slices, in order
#pragma unroll
                    for (int i = 0; i < NVV; ++i) {
                        const int c = lane + i * 32;
                        if (b < B && c < K4) {
                            const float4 u = *reinterpret_cast<const float4*>(a.branch + ((size_t)part * B + b) * K + c * 4);
                            t[i].x += u.x; t[i].y += u.y; t[i].z += u.z; t[i].w += u.w;
                        }
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < NVV; ++i) {
                const int c = lane + i * 32;
                v[i].x += t[i].x; v[i].y += t[i].y; v[i].z += t[i].z; v[i].w += t[i].w;
                if (blockIdx.x == 0 && b < B && c < K4) *reinterpret_cast<float4*>(a.resid_out + (size_t)b * K + c * 4) = v[i];
            }
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < NVV; ++i) s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
#pragma unroll
            for (int d = 16; d >= 1; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
            const float mean = s / (float)K;
            float q = 0.f;
#pragma unroll
            for (int i = 0; i < NVV; ++i) {
                if (lane + i * 32 < K4) {
                    const float dx = v[i].x - mean, dy = v[i].y - mean, dz = v[i].z - mean, dw = v[i].w - mean;
                    q += (dx * dx + dy * dy) + (dz * dz + dw * dw);
                }
            }
#pragma unroll
            for (int d = 16; d >= 1; d >>= 1) q += __shfl_xor_sync(0xffffffffu, q, d);
            const float rstd = rsqrtf(q / (float)K + 1e-5f);
#pragma unroll
            for (int i = 0; i < NVV; ++i) {
                const int c = lane + i * 32;
                if (c < K4) {
                    float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (b < B) {
                        const float4 lw = lnw4[c], lb = lnb4[c];
                        y.x = (v[i].x - mean) * rstd * lw.x + lb.x;
                        y.y = (v[i].y - mean) * rstd * lw.y + lb.y;
                        y.z = (v[i].z - mean) * rstd * lw.z + lb.z;
                        y.w = (v[i].w - mean) * rstd * lw.w + lb.w;
                    }
                    xs4[b * K4 + c] = y;
                }
            }
        }
    } else {
        // eight independent loads per thread in flight at a time
        const int total = NB * KS4;
        for (int i0 = threadIdx.x; i0 < total; i0 += 8 * kSkinnyThreads) {
            float4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int i = i0 + u * kSkinnyThreads;
                v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                const int b = i / KS4, c = i - b * KS4;  // this CTA's K slice of row b
                if (i < B * KS4) v[u] = *reinterpret_cast<const float4*>(a.x + (size_t)b * K + kbeg + c * 4);
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int i = i0 + u * kSkinnyThreads;
                if (i < total) xs4[i] = v[u];
            }
        }
    }
    __syncthreads();
    const int xs_stride = (NV > 0) ? K4 : KS4;  // the prologue stages whole rows
    float* __restrict__ out = a.out + (size_t)ks * B * N;
    for (int unit = blockIdx.x; unit < units; unit += gridDim.x) {
        const int batch = unit / a.k_splits;
        const int n0 = (batch * kRowWarps + rw) * ROWS;
        float bias_r[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) bias_r[r] = (a.bias && ks == 0 && n0 + r < N) ? __ldg(a.bias + n0 + r) : 0.f;
        float acc[ROWS][NB];
#pragma unroll
        for (int r = 0; r < ROWS; ++r)
#pragma unroll
            for (int b = 0; b < NB; ++b) acc[r][b] = 0.f;
        for (int kc0 = kbeg; kc0 < kend; kc0 += kSkinnyKC) {
            const int kc = min(kSkinnyKC, kend - kc0);  // multiple of 4
            // the chunk was requested earlier (before the kernel's wait, or at the end of the
            // previous chunk); take it over and request the next one before using it
            float4 wc[kSkinnySteps][ROWS];
#pragma unroll
            for (int s = 0; s < kSkinnySteps; ++s)
#pragma unroll
                for (int r = 0; r < ROWS; ++r) wc[s][r] = w[s][r];
            if (kc0 + kSkinnyKC < kend) request_w(n0, kc0 + kSkinnyKC);
            else if (unit + (int)gridDim.x < units) request_w((((unit + gridDim.x) / a.k_splits) * kRowWarps + rw) * ROWS, kbeg);
            if (n0 < N) {
#pragma unroll
                for (int s = 0; s < kSkinnySteps; ++s) {
                    const int k4 = s * 32 + lane;
                    if (k4 * 4 < kc) {
#pragma unroll
                        for (int b = 0; b < NB; ++b) {
                            const float4 xv = xs4[b * xs_stride + ((kc0 - kbeg) >> 2) + k4];
#pragma unroll
                            for (int r = 0; r < ROWS; ++r) {
                                float t = acc[r][b];
                                t = fmaf(wc[s][r].x, xv.x, t);
                                t = fmaf(wc[s][r].y, xv.y, t);
                                t = fmaf(wc[s][r].z, xv.z, t);
                                t = fmaf(wc[s][r].w, xv.w, t);
                                acc[r][b] = t;
                            }
                        }
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
        {
#pragma unroll
            for (int r = 0; r < ROWS; ++r)
#pragma unroll
                for (int b = 0; b < NB; ++b) {
                    if (((r * NB + b) & 31) == lane && n0 + r < N && b < B) {
                        float v = acc[r][b] + bias_r[r];
                        if (a.gelu) v = gelu_tanh(v);
                        out[(size_t)b * N + n0 + r] = v;
                    }
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
#ifndef B200_DEC_SPLITS
#define B200_DEC_SPLITS 4
#endif
constexpr int kDecAttSplits = B200_DEC_SPLITS;  // CTAs per (sequence, head): each walks its share of the positions (at most 8: the state buffer's size; 8 measured slower, 593 vs 560 us per step)

// q: row b of qkv [B, 3C] (first C columns); caches [B][cache_T][C]; positions 0..pos take part.
// grid (NH, B, kDecAttSplits).  Every CTA leaves its softmax state {m, l, o[64]} in `partial`;
// the last one of a (sequence, head) to finish - found with a counter - merges the states in
// split order (so the result does not depend on which CTA that was) and resets the counter.
__global__ void __launch_bounds__(kDecAttThreads)
decode_attention_kernel(float* __restrict__ out, const float* __restrict__ qkv, float* kcache, float* vcache, int C,
                        const int* __restrict__ pos_ptr, int cache_T, float* partial, unsigned int* counters) {
    __shared__ float st_m[16], st_l[16];
    __shared__ float st_o[16][64];
    __shared__ int is_last;
    griddep_wait();
    griddep_launch_dependents();
    const int h = blockIdx.x, b = blockIdx.y, z = blockIdx.z;
    // the query is requested together with the position (two independent round trips, not one after the other)
    const int hl0 = threadIdx.x & 15;
    float4 q = *reinterpret_cast<const float4*>(qkv + (size_t)b * 3 * C + h * 64 + hl0 * 4);
    const int pos = *pos_ptr;
    const int per = (((pos + kDecAttSplits) / kDecAttSplits + 15) / 16) * 16;  // positions per split
    const int t_begin = z * per, t_end = min(pos + 1, t_begin + per);
    // this head's slice of the new position goes into the cache first, by the split that will
    // read it (ordinary loads below: the read-only path need not see stores of the same kernel)
    if (threadIdx.x < 32 && pos >= t_begin && pos < t_end) {
        const int which = threadIdx.x >> 4, c = (threadIdx.x & 15) * 4;
        float* cache = which ? vcache : kcache;
        *reinterpret_cast<float4*>(cache + ((size_t)b * cache_T + pos) * C + h * 64 + c) =
            *reinterpret_cast<const float4*>(qkv + (size_t)b * 3 * C + (1 + which) * C + h * 64 + c);
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int half = lane >> 4, hl = lane & 15;  // a half-warp covers the 64 floats of one cached row
    const int slot = warp * 2 + half;            // 16 half-warps walk positions slot, slot + 16, ...
    const float scale = 0.125f;                  // 1 / sqrt(64)
    q.x *= scale; q.y *= scale; q.z *= scale; q.w *= scale;
    const float* kbase = kcache + (size_t)b * cache_T * C + h * 64 + hl * 4;
    const float* vbase = vcache + (size_t)b * cache_T * C + h * 64 + hl * 4;
    float m = -INFINITY, l = 0.f;
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    // every half-warp makes the same number of trips so that the shuffles stay warp-wide
    const int trips = (max(t_end - t_begin, 0) + 15) / 16;
    constexpr int U = 8;  // positions requested per half-warp before anything waits (bytes in flight)
    for (int i0 = 0; i0 < trips; i0 += U) {
        float4 k4[U], v4[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int t = t_begin + (i0 + u) * 16 + slot;
            k4[u] = v4[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (t < t_end) {
                k4[u] = *reinterpret_cast<const float4*>(kbase + (size_t)t * C);
                v4[u] = *reinterpret_cast<const float4*>(vbase + (size_t)t * C);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int t = t_begin + (i0 + u) * 16 + slot;
            float s = (q.x * k4[u].x + q.y * k4[u].y) + (q.z * k4[u].z + q.w * k4[u].w);
#pragma unroll
            for (int d = 8; d >= 1; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);  // within the half-warp
            if (t < t_end) {
                const float mn = fmaxf(m, s);
                const float corr = expf(m - mn), p = expf(s - mn);  // corr = 0 on the first position
                l = l * corr + p;
                o.x = o.x * corr + p * v4[u].x; o.y = o.y * corr + p * v4[u].y;
                o.z = o.z * corr + p * v4[u].z; o.w = o.w * corr + p * v4[u].w;
                m = mn;
            }
        }
    }
    if (hl == 0) { st_m[slot] = m; st_l[slot] = l; }
    *reinterpret_cast<float4*>(&st_o[slot][hl * 4]) = o;
    __syncthreads();
    // this CTA's state: thread d < 64 owns output column d; threads 64 and 65 own l and m
    const size_t bh = (size_t)b * gridDim.x + h;
    float* mine = partial + (bh * kDecAttSplits + z) * 66;
    float cm = -INFINITY;
#pragma unroll
    for (int i = 0; i < 16; ++i) cm = fmaxf(cm, st_m[i]);
    if (threadIdx.x < 66) {
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float w = (st_m[i] == -INFINITY) ? 0.f : expf(st_m[i] - cm);  // a half-warp may have seen nothing
            acc += (threadIdx.x < 64 ? st_o[i][threadIdx.x] : st_l[i]) * w;
        }
        mine[threadIdx.x] = (threadIdx.x == 65) ? cm : acc;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) is_last = (atomicAdd(counters + bh, 1u) == kDecAttSplits - 1);
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if (threadIdx.x < 64) {
        const float* all = partial + bh * kDecAttSplits * 66;
        float mm = -INFINITY;
#pragma unroll
        for (int s = 0; s < kDecAttSplits; ++s) mm = fmaxf(mm, __ldcg(all + s * 66 + 65));
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int s = 0; s < kDecAttSplits; ++s) {
            const float ms = __ldcg(all + s * 66 + 65);
            const float w = (ms == -INFINITY) ? 0.f : expf(ms - mm);  // an empty split
            L += __ldcg(all + s * 66 + 64) * w;
            O += __ldcg(all + s * 66 + threadIdx.x) * w;
        }
        out[(size_t)b * C + h * 64 + threadIdx.x] = O / L;
    }
    if (threadIdx.x == 0) counters[bh] = 0u;  // for the next launch
}

// out[b,:] = wte[tok[b],:] + wpe[pos,:]  (one fp32 add, as the full-sequence encoder)
__global__ void decode_encoder_kernel(float4* __restrict__ out, const int* __restrict__ tok, const float4* __restrict__ wte,
                                      const float4* __restrict__ wpe, const int* __restrict__ pos_ptr, int B, int C4,
                                      int vocab_rows, int* status) {
    griddep_wait();
    griddep_launch_dependents();
    const int pos = *pos_ptr;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < B * C4; i += gridDim.x * blockDim.x) {
        const int b = i / C4, c = i % C4;
        int id = tok[b];
        if (id < 0 || id >= vocab_rows) {  // reported like the full-sequence encoder does
            atomicCAS(status, 0, 201);
            id = 0;
        }
        const float4 e = __ldg(wte + (size_t)id * C4 + c), p = __ldg(wpe + (size_t)pos * C4 + c);
        out[i] = make_float4(e.x + p.x, e.y + p.y, e.z + p.z, e.w + p.w);
    }
}

__global__ void set_int_kernel(int* dst, int value) { *dst = value; }

}  // namespace

int launch_set_int(b200_ctx* ctx, int* dst, int value) {
    set_int_kernel<<<1, 1, 0, ctx->stream>>>(dst, value);
    ctx->launches++;
    B200_CUDA(ctx, cudaGetLastError());
    return B200_OK;
}

int launch_decode_encoder(b200_ctx* ctx, float* out, const int* tok, const float* wte, const float* wpe,
                          const int* pos_ptr, int B, int C, int vocab_rows) {
    const int n = B * (C / 4);
    cudaError_t le = launch_pdl(ctx, decode_encoder_kernel, dim3((n + 255) / 256), dim3(256), 0, reinterpret_cast<float4*>(out), tok,
                                reinterpret_cast<const float4*>(wte), reinterpret_cast<const float4*>(wpe), pos_ptr, B, C / 4,
                                vocab_rows, ctx->d_status);
    ctx->launches++;
    B200_CUDA(ctx, le);
    return B200_OK;
}

// K slices of a plain product (no prologue, no activation) whose output is so narrow that its row
// batches leave most SMs idle: as many as fit in one wave, at most 4, each at least 256 floats of K
// in whole steps of 128.  The caller hands the same number to the consumer as branch_parts.
int skinny_gemm_k_splits(const b200_ctx* ctx, int K, int N) {
    // tuning hook: B200_DECODE_KSPLIT=1 switches the slices off, 2-4 caps their number
    static const int forced = [] { const char* e = getenv("B200_DECODE_KSPLIT"); return e ? atoi(e) : 0; }();
    if (forced == 1) return 1;
    const int cap = (forced >= 2 && forced <= 4) ? forced : 4;
    const int batches = ((N + 1) / 2 + 7) / 8;
    int ks = ctx->num_sms / (batches > 0 ? batches : 1);
    if (ks > cap) ks = cap;
    while (ks > 1 && (K % (128 * ks) || K / ks < 256)) --ks;
    return ks < 1 ? 1 : ks;
}

int launch_skinny_gemm(b200_ctx* ctx, float* out, const float* x, const float* W, const float* bias, int B,
                       int K, int N, int gelu, const float* branch, const float* ln_w, const float* ln_b,
                       float* resid_out, int k_splits, int branch_parts) {
    if (B < 1 || B > 16 || K % 4 || N < 1) return B200_ERR_SHAPE;
    if (ln_w && (K > 1664 || !ln_b || !resid_out || resid_out == x)) return B200_ERR_SHAPE;
    if (k_splits < 1 || branch_parts < 1) return B200_ERR_SHAPE;
    if (k_splits > 1 && (ln_w || gelu || K % (128 * k_splits))) return B200_ERR_SHAPE;
    const int nb = B <= 8 ? 8 : 16;
    const int kslice = K / k_splits;
    const size_t x_bytes = ((size_t)nb * kslice * 4 + 127) & ~(size_t)127;
    if (x_bytes > (size_t)200 * 1024) return B200_ERR_LIMIT;
    SkinnyArgs a;
    a.out = out; a.x = x; a.W = W; a.bias = bias; a.branch = branch; a.ln_w = ln_w; a.ln_b = ln_b; a.resid_out = resid_out;
    a.B = B; a.N = N; a.K = K; a.gelu = gelu;
    a.k_splits = k_splits; a.kslice = kslice; a.branch_parts = branch_parts;
    // rows per warp: two, i.e. 16 output rows per CTA and batch; three (with a shorter K chunk, for the
    // registers) where that turns one and a bit rounds of batches into a single wave - the GELU GEMM
    // of the 124M model: 192 batches of 16 rows on 148 SMs, 128 batches of 24
    int rows = 2;
    static const int rows3_off = [] { const char* e = getenv("B200_DECODE_ROWS3"); return e && e[0] == '0'; }();  // tuning hook
    if (!rows3_off && k_splits == 1 && K <= 768 && ((N + 1) / 2 + 7) / 8 > ctx->num_sms && ((N + 2) / 3 + 7) / 8 <= ctx->num_sms) rows = 3;
    const int groups = (N + rows - 1) / rows;
    const int batches = (groups + 7) / 8;
    if (k_splits > 1 && batches * k_splits > ctx->num_sms) return B200_ERR_SHAPE;  // the slices of a unit run side by side
    // one wave: a CTA stages the input rows (and normalises them) once and then loops over its batches
    const int grid = batches * k_splits < ctx->num_sms ? batches * k_splits : ctx->num_sms;
    const int nv = !ln_w ? 0 : (K <= 768 ? 6 : 13);
    const size_t smem = x_bytes + (ln_w ? (size_t)2 * K * 4 : 0);
    cudaError_t le = cudaSuccess;
#define B200_SKINNY(NB, ROWS_, NV, STEPS_)                                                                          \
    do {                                                                                                            \
        static bool attr_set[64] = {};                                                                              \
        if (!attr_set[ctx->device & 63]) {                                                                          \
            B200_CUDA(ctx, cudaFuncSetAttribute(skinny_gemm_kernel<NB, ROWS_, NV, STEPS_>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)); \
            attr_set[ctx->device & 63] = true;                                                                      \
        }                                                                                                           \
        le = launch_pdl(ctx, skinny_gemm_kernel<NB, ROWS_, NV, STEPS_>, dim3(grid), dim3(kSkinnyThreads), smem, a); \
    } while (0)
    if (rows == 3) {
        if (nb == 8) { if (nv == 0) B200_SKINNY(8, 3, 0, 6); else B200_SKINNY(8, 3, 6, 6); }
        else { if (nv == 0) B200_SKINNY(16, 3, 0, 6); else B200_SKINNY(16, 3, 6, 6); }
    } else if (nb == 8) { if (nv == 0) B200_SKINNY(8, 2, 0, 8); else if (nv == 6) B200_SKINNY(8, 2, 6, 8); else B200_SKINNY(8, 2, 13, 8); }
    else { if (nv == 0) B200_SKINNY(16, 2, 0, 8); else if (nv == 6) B200_SKINNY(16, 2, 6, 8); else B200_SKINNY(16, 2, 13, 8); }
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

int launch_decode_attention(b200_ctx* ctx, float* out, const float* qkv, float* kcache, float* vcache, int B, int C,
                            int NH, const int* pos_ptr, int cache_T, float* partial, unsigned int* counters) {
    cudaError_t le = launch_pdl(ctx, decode_attention_kernel, dim3(NH, B, kDecAttSplits), dim3(kDecAttThreads), 0, out, qkv,
                                kcache, vcache, C, pos_ptr, cache_T, partial, counters);
    ctx->launches++;
    B200_CUDA(ctx, le);
    return B200_OK;
}

}  // namespace b200
