// HBM-bound row-wise kernels of the GPT-2 forward: layernorm, fused residual+layernorm,
// residual add, GELU, the token+position encoder gather, and two small helpers of the driver
// (TF32 rounding of weights, per-row arg-max).  float4-coalesced access, one warp per row for
// the normalisations with the row held in registers and warp-shuffle reductions; no tensor
// cores.  Grids are sized from the SM count.
//
// Math follows kernels/layernorm/1_layernorm_block.cuh:32-60 (biased variance, eps 1e-5,
// mean/rstd outputs), kernels/fused_residual_layernorm/fused_residual_layernorm.cuh:28-36,59-81
// (intent; that kernel's float4 pointer stride at :19,48-50 is not followed),
// kernels/residual/1_residual_naive.cuh:9-12 and kernels/matmul/9_matmul_async_cg_tf32_gelu.cuh:5-11.
#include <cstdlib>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "kernels.h"
#include "../prim/sm100.cuh"

namespace b200 {

namespace {

constexpr int kRowWarps = 8;  // rows per CTA in the normalisation kernels

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
    return v;
}

// One warp per row.  NV = float4 per lane held in registers (covers C <= 128*NV).
// FUSED: x = inp1 + inp2 is stored to res_out first (which may alias an input: every
// element is read before it is written, by the same lane).  With inp3: x = inp1 + (inp2 + inp3),
// the two partial sums of a two-way tensor-parallel projection (inp2 + inp3 is what an all-reduce
// would have left in inp2, bit for bit, on either rank).
template <int NV, bool FUSED>
__global__ void __launch_bounds__(kRowWarps * 32)
layernorm_rows_kernel(float* __restrict__ out, float* res_out, float* __restrict__ mean,
                      float* __restrict__ rstd, const float* inp1, const float* inp2,
                      const float* __restrict__ weight, const float* __restrict__ bias, int M, int C,
                      int flags, const float* inp3) {
    griddep_wait();
    griddep_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * kRowWarps + (threadIdx.x >> 5);
    if (row >= M) return;
    const int C4 = C >> 2;
    const float4* x1 = reinterpret_cast<const float4*>(inp1 + (size_t)row * C);
    const float4* x2 = FUSED ? reinterpret_cast<const float4*>(inp2 + (size_t)row * C) : nullptr;
    const float4* x3 = (FUSED && inp3) ? reinterpret_cast<const float4*>(inp3 + (size_t)row * C) : nullptr;

    float4 v[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = lane + i * 32;
        if (c < C4) {
            v[i] = x1[c];
            if (FUSED) {
                float4 b = x2[c];
                if (x3) {
                    const float4 b3 = x3[c];
                    b.x += b3.x; b.y += b3.y; b.z += b3.z; b.w += b3.w;
                }
                v[i].x += b.x; v[i].y += b.y; v[i].z += b.z; v[i].w += b.w;
            }
        } else {
            v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    if (FUSED) {
        float4* ro = reinterpret_cast<float4*>(res_out + (size_t)row * C);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int c = lane + i * 32;
            if (c < C4) ro[c] = v[i];
        }
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    const float m = warp_sum(s) / (float)C;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = lane + i * 32;
        if (c < C4) {
            const float dx = v[i].x - m, dy = v[i].y - m, dz = v[i].z - m, dw = v[i].w - m;
            q += (dx * dx + dy * dy) + (dz * dz + dw * dw);
        }
    }
    const float r = rsqrtf(warp_sum(q) / (float)C + 1e-5f);
    if (lane == 0) {
        if (mean) mean[row] = m;
        if (rstd) rstd[row] = r;
    }
    const float4* w4 = reinterpret_cast<const float4*>(weight);
    const float4* b4 = reinterpret_cast<const float4*>(bias);
    float4* o = reinterpret_cast<float4*>(out + (size_t)row * C);
    uint2* oh = reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(out) + (size_t)row * C);  // OUT_BF16
    const bool rnd = (flags & ROUND_OUT_TF32) != 0;
    const bool as_bf16 = (flags & (OUT_BF16 | OUT_BF16X2)) != 0;
    const bool planes = (flags & OUT_BF16X2) != 0;
    uint2* ol = oh + (size_t)M * C4;  // OUT_BF16X2: the plane of the dropped parts
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = lane + i * 32;
        if (c < C4) {
            const float4 w = __ldg(w4 + c), b = __ldg(b4 + c);
            float4 y;
            y.x = (v[i].x - m) * r * w.x + b.x;
            y.y = (v[i].y - m) * r * w.y + b.y;
            y.z = (v[i].z - m) * r * w.z + b.z;
            y.w = (v[i].w - m) * r * w.w + b.w;
            if (as_bf16) {
                const __nv_bfloat162 p0 = __floats2bfloat162_rn(y.x, y.y), p1 = __floats2bfloat162_rn(y.z, y.w);
                oh[c] = make_uint2(*reinterpret_cast<const uint32_t*>(&p0), *reinterpret_cast<const uint32_t*>(&p1));
                if (planes) {
                    const __nv_bfloat162 q0 = __floats2bfloat162_rn(y.x - __low2float(p0), y.y - __high2float(p0));
                    const __nv_bfloat162 q1 = __floats2bfloat162_rn(y.z - __low2float(p1), y.w - __high2float(p1));
                    ol[c] = make_uint2(*reinterpret_cast<const uint32_t*>(&q0), *reinterpret_cast<const uint32_t*>(&q1));
                }
                continue;
            }
            if (rnd) { y.x = round_tf32(y.x); y.y = round_tf32(y.y); y.z = round_tf32(y.z); y.w = round_tf32(y.w); }
            o[c] = y;
        }
    }
}

// Layernorm of a tensor-parallel rank's OWN rows (sequence-parallel hand-over, see driver/gpt2.cu):
//   x = residual + (part[0] + part[1] + ... + part[n-1])      the n ranks' partial sums of a projection
// for the `rows` rows from row0 on; x goes back to residual (this rank's rows only), and the
// normalised row is written to the same place of EVERY rank's layernorm output (dst[0..n), peers'
// memory included): as fp32 (TF32-rounded on request) or as two bf16 planes (OUT_BF16X2, the second
// plane plane_stride elements further down).  One warp per row; NV float4 per lane.
struct LnSpArgs {
    float* residual;         // [M, C], local
    const float* parts;      // [n][rows][C], local: what the ranks' GEMMs stored for these rows
    float* dst[8];           // every rank's layernorm output buffer
    const float* weight;
    const float* bias;
    int n, rows, row0, C, flags;
    size_t plane_stride;     // elements between the two bf16 planes (M * C)
};
template <int NV>
__global__ void __launch_bounds__(kRowWarps * 32)
layernorm_sp_kernel(const LnSpArgs a) {
    griddep_wait();
    griddep_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int rl = blockIdx.x * kRowWarps + (threadIdx.x >> 5);
    if (rl >= a.rows) return;
    const int C = a.C, C4 = C >> 2;
    const size_t grow = (size_t)(a.row0 + rl) * C;
    float4* res = reinterpret_cast<float4*>(a.residual + grow);
    float4 v[NV], t[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = lane + i * 32;
        v[i] = t[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < C4) {
            v[i] = res[c];
            t[i] = reinterpret_cast<const float4*>(a.parts + (size_t)rl * C)[c];
        }
    }
    for (int s = 1; s < a.n; ++s) {  // the partial sums in rank order: the same sum on every rank
        const float4* ps = reinterpret_cast<const float4*>(a.parts + ((size_t)s * a.rows + rl) * C);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int c = lane + i * 32;
            if (c < C4) {
                const float4 u = ps[c];
                t[i].x += u.x; t[i].y += u.y; t[i].z += u.z; t[i].w += u.w;
            }
        }
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = lane + i * 32;
        v[i].x += t[i].x; v[i].y += t[i].y; v[i].z += t[i].z; v[i].w += t[i].w;
        if (c < C4) res[c] = v[i];
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    const float m = warp_sum(s) / (float)C;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        if (lane + i * 32 < C4) {
            const float dx = v[i].x - m, dy = v[i].y - m, dz = v[i].z - m, dw = v[i].w - m;
            q += (dx * dx + dy * dy) + (dz * dz + dw * dw);
        }
    }
    const float r = rsqrtf(warp_sum(q) / (float)C + 1e-5f);
    const float4* w4 = reinterpret_cast<const float4*>(a.weight);
    const float4* b4 = reinterpret_cast<const float4*>(a.bias);
    const bool rnd = (a.flags & ROUND_OUT_TF32) != 0;
    const bool planes = (a.flags & OUT_BF16X2) != 0;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = lane + i * 32;
        if (c >= C4) continue;
        const float4 w = __ldg(w4 + c), b = __ldg(b4 + c);
        float4 y;
        y.x = (v[i].x - m) * r * w.x + b.x;
        y.y = (v[i].y - m) * r * w.y + b.y;
        y.z = (v[i].z - m) * r * w.z + b.z;
        y.w = (v[i].w - m) * r * w.w + b.w;
        if (planes) {
            const __nv_bfloat162 p0 = __floats2bfloat162_rn(y.x, y.y), p1 = __floats2bfloat162_rn(y.z, y.w);
            const __nv_bfloat162 q0 = __floats2bfloat162_rn(y.x - __low2float(p0), y.y - __high2float(p0));
            const __nv_bfloat162 q1 = __floats2bfloat162_rn(y.z - __low2float(p1), y.w - __high2float(p1));
            const uint2 hi = make_uint2(*reinterpret_cast<const uint32_t*>(&p0), *reinterpret_cast<const uint32_t*>(&p1));
            const uint2 lo = make_uint2(*reinterpret_cast<const uint32_t*>(&q0), *reinterpret_cast<const uint32_t*>(&q1));
            for (int d = 0; d < a.n; ++d) {
                uint2* oh = reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(a.dst[d]) + grow);
                oh[c] = hi;
                (oh + a.plane_stride / 4)[c] = lo;
            }
        } else {
            if (rnd) { y.x = round_tf32(y.x); y.y = round_tf32(y.y); y.z = round_tf32(y.z); y.w = round_tf32(y.w); }
            for (int d = 0; d < a.n; ++d) reinterpret_cast<float4*>(a.dst[d] + grow)[c] = y;
        }
    }
}

template <bool FUSED>
int launch_ln_any(b200_ctx* ctx, float* out, float* res_out, float* mean, float* rstd,
                  const float* inp1, const float* inp2, const float* weight, const float* bias,
                  int M, int C, int flags, const float* inp3 = nullptr) {
    const int nv = (C / 4 + 31) / 32;
    const dim3 grid((M + kRowWarps - 1) / kRowWarps), block(kRowWarps * 32);
    cudaError_t le = cudaSuccess;
#define B200_LN_CASE(NV)                                                                                    \
    le = launch_pdl(ctx, layernorm_rows_kernel<NV, FUSED>, grid, block, 0, out, res_out, mean, rstd, inp1, \
                    inp2, weight, bias, M, C, flags, inp3)
    if (nv <= 2) B200_LN_CASE(2);
    else if (nv <= 4) B200_LN_CASE(4);
    else if (nv <= 6) B200_LN_CASE(6);       // C = 768
    else if (nv <= 8) B200_LN_CASE(8);       // C = 1024
    else if (nv <= 10) B200_LN_CASE(10);     // C = 1280
    else if (nv <= 13) B200_LN_CASE(13);     // C = 1600
    else if (nv <= 16) B200_LN_CASE(16);
    else B200_LN_CASE(32);                   // C <= 4096
#undef B200_LN_CASE
    ctx->launches++;
    B200_CUDA(ctx, le);
    return B200_OK;
}

__global__ void residual_kernel(float4* __restrict__ out, const float4* __restrict__ a,
                                const float4* __restrict__ b, size_t n4, float* out_s,
                                const float* a_s, const float* b_s, size_t n) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i < n4; i += stride) {
        const float4 x = a[i], y = b[i];
        out[i] = make_float4(x.x + y.x, x.y + y.y, x.z + y.z, x.w + y.w);
    }
    // scalar tail (N % 4)
    i = n4 * 4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out_s[i] = a_s[i] + b_s[i];
}

__global__ void gelu_kernel(float4* __restrict__ out, const float4* __restrict__ inp, size_t n4,
                            float* out_s, const float* inp_s, size_t n) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i < n4; i += stride) {
        const float4 x = inp[i];
        out[i] = make_float4(gelu_tanh(x.x), gelu_tanh(x.y), gelu_tanh(x.z), gelu_tanh(x.w));
    }
    i = n4 * 4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out_s[i] = gelu_tanh(inp_s[i]);
}

__global__ void convert_bf16_kernel(uint2* __restrict__ out, const float4* __restrict__ in, size_t n4, uint2* __restrict__ dropped) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        const float4 x = in[i];
        const __nv_bfloat162 p0 = __floats2bfloat162_rn(x.x, x.y), p1 = __floats2bfloat162_rn(x.z, x.w);
        out[i] = make_uint2(*reinterpret_cast<const uint32_t*>(&p0), *reinterpret_cast<const uint32_t*>(&p1));
        if (dropped) {  // what the rounding dropped, again as bf16 (x - bf16(x) is exact in fp32)
            const __nv_bfloat162 q0 = __floats2bfloat162_rn(x.x - __low2float(p0), x.y - __high2float(p0));
            const __nv_bfloat162 q1 = __floats2bfloat162_rn(x.z - __low2float(p1), x.w - __high2float(p1));
            dropped[i] = make_uint2(*reinterpret_cast<const uint32_t*>(&q0), *reinterpret_cast<const uint32_t*>(&q1));
        }
    }
}

// out[i] = e4m3(in[i] * scale): round to nearest even, saturating at the largest finite value (448)
__global__ void quantize_e4m3_kernel(uint32_t* __restrict__ out, const float4* __restrict__ in, size_t n4, float scale) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        const float4 v = __ldg(in + i);
        uint16_t lo, hi;  // two e4m3 values each: the second source operand lands in the low byte
        asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(v.y * scale), "f"(v.x * scale));
        asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(v.w * scale), "f"(v.z * scale));
        out[i] = (uint32_t)lo | ((uint32_t)hi << 16);
    }
}

__global__ void split_fp16_kernel(uint2* __restrict__ hi, uint2* __restrict__ lo, const float4* __restrict__ in, size_t n4) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        float4 x = in[i];
        x.x = fminf(fmaxf(x.x, -65504.f), 65504.f); x.y = fminf(fmaxf(x.y, -65504.f), 65504.f);
        x.z = fminf(fmaxf(x.z, -65504.f), 65504.f); x.w = fminf(fmaxf(x.w, -65504.f), 65504.f);
        const __half2 p0 = __floats2half2_rn(x.x, x.y), p1 = __floats2half2_rn(x.z, x.w);
        const __half2 q0 = __floats2half2_rn(x.x - __low2float(p0), x.y - __high2float(p0));
        const __half2 q1 = __floats2half2_rn(x.z - __low2float(p1), x.w - __high2float(p1));
        hi[i] = make_uint2(*reinterpret_cast<const uint32_t*>(&p0), *reinterpret_cast<const uint32_t*>(&p1));
        lo[i] = make_uint2(*reinterpret_cast<const uint32_t*>(&q0), *reinterpret_cast<const uint32_t*>(&q1));
    }
}

__global__ void round_tf32_kernel(float4* data, size_t n4, float* data_s, size_t n) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i < n4; i += stride) {
        float4 x = data[i];
        data[i] = make_float4(round_tf32(x.x), round_tf32(x.y), round_tf32(x.z), round_tf32(x.w));
    }
    i = n4 * 4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) data_s[i] = round_tf32(data_s[i]);
}

// out[bt, :] = wte[tok[bt], :] + wpe[bt % T, :]; one fp32 add per element (bit-exact).
// An id outside [0, vocab_rows) (when checked) is recorded in *status and treated as 0.
// One warp per row: the token id is read once per row (it may sit in pinned host memory and
// come over PCIe) and handed to the other lanes by shuffle.
__global__ void __launch_bounds__(kRowWarps * 32)
encoder_kernel(float4* __restrict__ out, const int* __restrict__ tok,
               const float4* __restrict__ wte, const float4* __restrict__ wpe,
               int M, int T, int C4, int vocab_rows, int* status) {
    griddep_wait();
    griddep_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int warps = gridDim.x * kRowWarps;
    for (int bt = blockIdx.x * kRowWarps + (threadIdx.x >> 5); bt < M; bt += warps) {
        int id = 0;
        if (lane == 0) {
            id = tok[bt];
            if (vocab_rows > 0 && (id < 0 || id >= vocab_rows)) {
                atomicCAS(status, 0, 201);
                id = 0;
            }
        }
        id = __shfl_sync(0xffffffffu, id, 0);
        const float4* e4 = wte + (size_t)id * C4;
        const float4* p4 = wpe + (size_t)(bt % T) * C4;
        float4* o4 = out + (size_t)bt * C4;
        for (int c = lane; c < C4; c += 32) {
            const float4 e = __ldg(e4 + c);
            const float4 p = __ldg(p4 + c);
            o4[c] = make_float4(e.x + p.x, e.y + p.y, e.z + p.z, e.w + p.w);
        }
    }
}

// dst[i] = src[i] for n ints, src being the device view of a pinned host buffer: the token ids
// come over PCIe in 16-byte pieces (a few hundred read requests for a whole batch; reading them
// one id at a time from the consumer would be thousands of PCIe round trips).
__global__ void fetch_ints_kernel(int* __restrict__ dst, const int* __restrict__ src, int n) {
    griddep_wait();
    griddep_launch_dependents();
    const int n4 = n >> 2;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n4) reinterpret_cast<int4*>(dst)[i] = reinterpret_cast<const int4*>(src)[i];
    if (i < (n & 3)) dst[n4 * 4 + i] = src[n4 * 4 + i];
}

// arg-max over columns [0,V) of each row (ties -> lowest index); one CTA per row.
__global__ void __launch_bounds__(256)
argmax_rows_kernel(int* __restrict__ out, const float* __restrict__ logits, int V, int ld) {
    const float* row = logits + (size_t)blockIdx.x * ld;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    const int V4 = V >> 2;
    const float4* r4 = reinterpret_cast<const float4*>(row);
    for (int i = threadIdx.x; i < V4; i += blockDim.x) {
        const float4 x = r4[i];
        const float xs[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
        for (int k = 0; k < 4; ++k)
            if (xs[k] > best) { best = xs[k]; bi = i * 4 + k; }
    }
    for (int i = V4 * 4 + threadIdx.x; i < V; i += blockDim.x)
        if (row[i] > best) { best = row[i]; bi = i; }
    __shared__ float sb[8];
    __shared__ int si[8];
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, s);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, s);
        if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sb[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w)
            if (sb[w] > best || (sb[w] == best && si[w] < bi)) { best = sb[w]; bi = si[w]; }
        out[blockIdx.x] = bi;
    }
}

// fp32 -> uint32 with the same order (larger value, larger key)
__device__ __forceinline__ uint32_t order_key(float f) {
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// One step of a radix select over the keys of a row: histogram of `bits` key bits at `shift` among
// the keys whose higher bits equal `prefix` (all keys if prefix_bits == 0), then the bin that
// holds the k-th largest of them.  Returns that bin; k is reduced by the keys in higher bins.
// 256 threads; hist has 2048 entries, part 256.
__device__ __forceinline__ uint32_t radix_select_step(const float* __restrict__ row, int V, uint32_t prefix, int prefix_bits,
                                                      int shift, int bits, int& k, int* hist, int* part, int* found) {
    const int nbins = 1 << bits;
    for (int i = threadIdx.x; i < nbins; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const uint32_t key = order_key(row[i]);
        if (prefix_bits == 0 || (key >> (32 - prefix_bits)) == prefix) atomicAdd(&hist[(key >> shift) & (nbins - 1)], 1);
    }
    __syncthreads();
    const int per = nbins / 256;  // bins per thread (8 or 4)
    int sum = 0;
    for (int j = 0; j < per; ++j) sum += hist[threadIdx.x * per + j];
    part[threadIdx.x] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        int above = 0, g = 255;
        for (; g > 0 && above + part[g] < k; --g) above += part[g];  // group g holds the k-th largest
        int b = g * per + per - 1;
        for (; b > g * per && above + hist[b] < k; --b) above += hist[b];
        found[0] = b;
        found[1] = k - above;
    }
    __syncthreads();
    k = found[1];
    const uint32_t bin = (uint32_t)found[0];
    __syncthreads();
    return bin;
}

// The same step over probability mass instead of counts, for nucleus (top-p) sampling: a key
// weighs exp((x - m) * inv_temp); columns with a key below min_key do not take part.  Finds the
// bin in which the mass of the larger keys reaches `target`, and reduces target by the mass of
// the higher bins.  (Shared-memory float atomics: the sums depend on the order of arrival in
// the last bits, which can move a column that sits exactly on the boundary in or out.)
__device__ __forceinline__ uint32_t radix_select_mass_step(const float* __restrict__ row, int V, uint32_t min_key, uint32_t prefix,
                                                           int prefix_bits, int shift, int bits, float& target, float m,
                                                           float inv_temp, float* hist, float* part, int* found_i,
                                                           float* found_f) {
    const int nbins = 1 << bits;
    for (int i = threadIdx.x; i < nbins; i += blockDim.x) hist[i] = 0.f;
    __syncthreads();
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float x = row[i];
        const uint32_t key = order_key(x);
        if (key < min_key) continue;
        if (prefix_bits == 0 || (key >> (32 - prefix_bits)) == prefix)
            atomicAdd(&hist[(key >> shift) & (nbins - 1)], __expf((x - m) * inv_temp));
    }
    __syncthreads();
    const int per = nbins / 256;
    float sum = 0.f;
    for (int j = 0; j < per; ++j) sum += hist[threadIdx.x * per + j];
    part[threadIdx.x] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        float above = 0.f;
        int g = 255;
        for (; g > 0 && above + part[g] < target; --g) above += part[g];
        int b = g * per + per - 1;
        for (; b > g * per && above + hist[b] < target; --b) above += hist[b];
        found_i[0] = b;
        found_f[0] = target - above;
    }
    __syncthreads();
    target = found_f[0];
    const uint32_t bin = (uint32_t)found_i[0];
    __syncthreads();
    return bin;
}

// Draws one column per row from softmax(logits / temperature) over columns [0,V): the arg-max of
// logit * inv_temp + Gumbel noise has exactly that distribution, so sampling is the greedy
// reduction with a perturbed score.  The noise is a pure function of (seed, stream0 + row,
// column): the same call gives the same tokens.  0 < top_k < V restricts the draw to the top_k
// largest logits of the row (all columns tied with the k-th one included): their threshold is
// found first, by a three-step radix select (11 + 11 + 10 key bits).  0 < top_p < 1 then keeps,
// of what is left, the most likely columns whose probabilities (at this temperature) add up to
// top_p - the smallest such set, columns tied with its last member included - by the same
// select over probability mass.  One CTA per row.
__global__ void __launch_bounds__(256)
sample_rows_kernel(int* __restrict__ out, const float* __restrict__ logits, int V, int ld, float inv_temp,
                   uint32_t seed, uint32_t stream0, int top_k, float top_p) {
    const float* row = logits + (size_t)blockIdx.x * ld;
    const uint32_t stream = stream0 + blockIdx.x;
    uint32_t min_key = 0u;  // columns with a smaller key are left out
    __shared__ int hist[2048];
    __shared__ int part[256];
    __shared__ int found[2];
    __shared__ float red[8];
    if (top_k > 0 && top_k < V) {
        int k = top_k;
        const uint32_t b0 = radix_select_step(row, V, 0u, 0, 21, 11, k, hist, part, found);
        const uint32_t b1 = radix_select_step(row, V, b0, 11, 10, 11, k, hist, part, found);
        const uint32_t b2 = radix_select_step(row, V, (b0 << 11) | b1, 22, 0, 10, k, hist, part, found);
        min_key = (b0 << 21) | (b1 << 10) | b2;
    }
    if (top_p > 0.f && top_p < 1.f) {
        // the row maximum and the total mass of the columns still in play
        float m = -INFINITY;
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const float x = row[i];
            if (order_key(x) >= min_key) m = fmaxf(m, x);
        }
#pragma unroll
        for (int s = 16; s >= 1; s >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, s));
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
        __syncthreads();
        m = red[0];
        for (int w = 1; w < 8; ++w) m = fmaxf(m, red[w]);
        __syncthreads();
        float z = 0.f;
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const float x = row[i];
            if (order_key(x) >= min_key) z += __expf((x - m) * inv_temp);
        }
#pragma unroll
        for (int s = 16; s >= 1; s >>= 1) z += __shfl_xor_sync(0xffffffffu, z, s);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = z;
        __syncthreads();
        z = 0.f;
        for (int w = 0; w < 8; ++w) z += red[w];
        __syncthreads();
        float target = top_p * z;
        float* histf = reinterpret_cast<float*>(hist);
        float* partf = reinterpret_cast<float*>(part);
        const uint32_t b0 = radix_select_mass_step(row, V, min_key, 0u, 0, 21, 11, target, m, inv_temp, histf, partf, found, red);
        const uint32_t b1 = radix_select_mass_step(row, V, min_key, b0, 11, 10, 11, target, m, inv_temp, histf, partf, found, red);
        const uint32_t b2 = radix_select_mass_step(row, V, min_key, (b0 << 11) | b1, 22, 0, 10, target, m, inv_temp, histf, partf, found, red);
        const uint32_t key_p = (b0 << 21) | (b1 << 10) | b2;
        if (key_p > min_key) min_key = key_p;
    }
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float x = row[i];
        if (order_key(x) < min_key) continue;
        const float sc = sample_score(x, inv_temp, seed, stream, (uint32_t)i);
        if (sc > best) { best = sc; bi = i; }
    }
    __shared__ float sb[8];
    __shared__ int si[8];
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, s);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, s);
        if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sb[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w)
            if (sb[w] > best || (sb[w] == best && si[w] < bi)) { best = sb[w]; bi = si[w]; }
        out[blockIdx.x] = bi;
    }
}

// Exercises the bounded-wait path on purpose-built inputs: one thread waits on an mbarrier that
// nothing ever arrives on, gives up after limit_ns, and records the time-out exactly as the
// GEMM / attention roles do.  The kernel returns normally and the context stays usable.
__global__ void wait_timeout_probe_kernel(int* status, unsigned long long limit_ns) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_flag = 0;
        fence_barrier_init();
        if (!mbar_wait(&bar, 0, &abort_flag, limit_ns)) atomicCAS(status, 0, DEV_TIMEOUT_PRODUCER);
    }
}

inline int stream_grid(const b200_ctx* ctx, size_t n4, int block, int ctas_per_sm) {
    size_t want = (n4 + block - 1) / block;
    size_t cap = (size_t)ctx->num_sms * ctas_per_sm;
    if (want < 1) want = 1;
    return (int)(want < cap ? want : cap);
}

}  // namespace

int launch_layernorm(b200_ctx* ctx, float* out, float* mean, float* rstd, const float* inp,
                     const float* weight, const float* bias, int M, int C, int flags) {
    return launch_ln_any<false>(ctx, out, nullptr, mean, rstd, inp, nullptr, weight, bias, M, C, flags);
}

int launch_fused_residual_layernorm(b200_ctx* ctx, float* res_out, float* ln_out, float* mean,
                                    float* rstd, const float* inp1, const float* inp2,
                                    const float* weight, const float* bias, int M, int C, int flags, const float* inp3) {
    return launch_ln_any<true>(ctx, ln_out, res_out, mean, rstd, inp1, inp2, weight, bias, M, C, flags, inp3);
}

// ---- hand-over between two GPUs whose kernels write into each other's memory ------------------
// signal: one release store (system scope) of `value` into a word of the peer's memory, after
// everything queued before it on this stream - including a GEMM whose epilogue stored tiles into
// the peer's memory - has completed.  wait: spins, for a bounded time, until this GPU's own word
// has reached `value`.  Both are plain launches (no programmatic early start): the kernels
// around them in the stream are ordered by them.
__global__ void peer_signal_kernel(unsigned int* peer_word, unsigned int value) {
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peer_word), "r"(value) : "memory");
}
__global__ void peer_wait_kernel(const unsigned int* my_word, unsigned int value, int* status, unsigned long long limit_ns) {
    const uint64_t t0 = globaltimer_ns();
    while (true) {
        unsigned int v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(my_word) : "memory");
        if ((int)(v - value) >= 0) return;  // epochs only grow (compared modulo 2^32)
        if (globaltimer_ns() - t0 > limit_ns) {
            atomicCAS(status, 0, DEV_TIMEOUT_PEER);
            return;
        }
        __nanosleep(200);
    }
}

int launch_peer_signal(b200_ctx* ctx, unsigned int* peer_word, unsigned int value) {
    peer_signal_kernel<<<1, 1, 0, ctx->stream>>>(peer_word, value);
    ctx->launches++;
    B200_CUDA(ctx, cudaGetLastError());
    return B200_OK;
}
int launch_peer_wait(b200_ctx* ctx, const unsigned int* my_word, unsigned int value, unsigned long long limit_ns) {
    peer_wait_kernel<<<1, 1, 0, ctx->stream>>>(my_word, value, ctx->d_status, limit_ns ? limit_ns : kWaitLimitNs);
    ctx->launches++;
    B200_CUDA(ctx, cudaGetLastError());
    return B200_OK;
}

// the same hand-over words towards / from several peers at once (thread i serves peer i)
struct PeerWords { unsigned int* w[8]; int n; };
__global__ void peer_signal_many_kernel(const PeerWords p, unsigned int value) {
    if ((int)threadIdx.x >= p.n || !p.w[threadIdx.x]) return;
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.w[threadIdx.x]), "r"(value) : "memory");
}
__global__ void peer_wait_many_kernel(const unsigned int* words, int n, int skip, unsigned int value, int* status, unsigned long long limit_ns) {
    if ((int)threadIdx.x >= n || (int)threadIdx.x == skip) return;
    const uint64_t t0 = globaltimer_ns();
    while (true) {
        unsigned int v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(words + threadIdx.x) : "memory");
        if ((int)(v - value) >= 0) return;
        if (globaltimer_ns() - t0 > limit_ns) {
            atomicCAS(status, 0, DEV_TIMEOUT_PEER);
            return;
        }
        __nanosleep(200);
    }
}
int launch_peer_signal_many(b200_ctx* ctx, unsigned int* const* peer_words, int n, unsigned int value) {
    PeerWords p;
    p.n = n;
    for (int i = 0; i < 8; ++i) p.w[i] = i < n ? peer_words[i] : nullptr;
    peer_signal_many_kernel<<<1, 32, 0, ctx->stream>>>(p, value);
    ctx->launches++;
    B200_CUDA(ctx, cudaGetLastError());
    return B200_OK;
}
int launch_peer_wait_many(b200_ctx* ctx, const unsigned int* my_words, int n, int skip, unsigned int value) {
    peer_wait_many_kernel<<<1, 32, 0, ctx->stream>>>(my_words, n, skip, value, ctx->d_status, kWaitLimitNs);
    ctx->launches++;
    B200_CUDA(ctx, cudaGetLastError());
    return B200_OK;
}

int launch_layernorm_sp(b200_ctx* ctx, float* residual, const float* parts, float* const* dst, int n, int rows, int row0,
                        const float* weight, const float* bias, int M, int C, int flags) {
    if (n < 2 || n > 8 || C % 4 || rows < 1) return B200_ERR_SHAPE;
    LnSpArgs a;
    a.residual = residual; a.parts = parts; a.weight = weight; a.bias = bias;
    a.n = n; a.rows = rows; a.row0 = row0; a.C = C; a.flags = flags;
    a.plane_stride = (size_t)M * C;
    for (int i = 0; i < 8; ++i) a.dst[i] = i < n ? dst[i] : nullptr;
    const int nv = (C / 4 + 31) / 32;
    const dim3 grid((rows + kRowWarps - 1) / kRowWarps), block(kRowWarps * 32);
    cudaError_t le = cudaSuccess;
    if (nv <= 6) le = launch_pdl(ctx, layernorm_sp_kernel<6>, grid, block, 0, a);
    else if (nv <= 13) le = launch_pdl(ctx, layernorm_sp_kernel<13>, grid, block, 0, a);
    else if (nv <= 32) le = launch_pdl(ctx, layernorm_sp_kernel<32>, grid, block, 0, a);
    else return B200_ERR_LIMIT;
    ctx->launches++;
    B200_CUDA(ctx, le);
    return B200_OK;
}

int launch_residual(b200_ctx* ctx, float* out, const float* a, const float* b, size_t N) {
    const size_t n4 = N / 4;
    const int grid = stream_grid(ctx, n4 > 0 ? n4 : 1, 256, 16);
    residual_kernel<<<grid, 256, 0, ctx->stream>>>(reinterpret_cast<float4*>(out),
                                                   reinterpret_cast<const float4*>(a),
                                                   reinterpret_cast<const float4*>(b), n4, out, a, b, N);
    ctx->launches++;
    B200_CUDA(ctx, cudaGetLastError());
    return B200_OK;
}

int launch_gelu(b200_ctx* ctx, float* out, const float* inp, size_t N) {
    const size_t n4 = N / 4;
    const int grid = stream_grid(ctx, n4 > 0 ? n4 : 1, 256, 16);
    gelu_kernel<<<grid, 256, 0, ctx->stream>>>(reinterpret_cast<float4*>(out),
                                               reinterpret_cast<const float4*>(inp), n4, out, inp, N);
    ctx->launches++;
    B200_CUDA(ctx, cudaGetLastError());
    return B200_OK;
}

// Loads the code of the forward's row-wise kernels now (CUDA loads a kernel's module lazily, at its
// first use, and that may allocate device memory).
int preload_rowwise_kernels(b200_ctx* ctx) {
    cudaFuncAttributes fa;
    B200_CUDA(ctx, cudaFuncGetAttributes(&fa, encoder_kernel));
    B200_CUDA(ctx, cudaFuncGetAttributes(&fa, layernorm_rows_kernel<2, false>));
    B200_CUDA(ctx, cudaFuncGetAttributes(&fa, layernorm_rows_kernel<4, false>));
    B200_CUDA(ctx, cudaFuncGetAttributes(&fa, layernorm_rows_kernel<6, false>));
    B200_CUDA(ctx, cudaFuncGetAttributes(&fa, layernorm_rows_kernel<8, false>));
    B200_CUDA(ctx, cudaFuncGetAttributes(&fa, layernorm_rows_kernel<10, false>));
    B200_CUDA(ctx, cudaFuncGetAttributes(&fa, layernorm_rows_kernel<13, false>));
    B200_CUDA(ctx, cudaFuncGetAttributes(&fa, layernorm_rows_kernel<16, false>));
    B200_CUDA(ctx, cudaFuncGetAttributes(&fa, layernorm_rows_kernel<32, false>));
    return B200_OK;
}

int launch_round_tf32_inplace(b200_ctx* ctx, float* data, size_t N) {
    const size_t n4 = N / 4;
    const int grid = stream_grid(ctx, n4 > 0 ? n4 : 1, 256, 16);
    round_tf32_kernel<<<grid, 256, 0, ctx->stream>>>(reinterpret_cast<float4*>(data), n4, data, N);
    ctx->launches++;
    B200_CUDA(ctx, cudaGetLastError());
    return B200_OK;
}

int launch_convert_bf16(b200_ctx* ctx, uint16_t* out, const float* in, size_t N, uint16_t* lo) {
    if (N % 4) { ctx->last_error = "bf16 conversion: element count must be a multiple of 4"; return B200_ERR_SHAPE; }
    const size_t n4 = N / 4;
    const int grid = stream_grid(ctx, n4 > 0 ? n4 : 1, 256, 16);
    convert_bf16_kernel<<<grid, 256, 0, ctx->stream>>>(reinterpret_cast<uint2*>(out), reinterpret_cast<const float4*>(in), n4,
                                                       reinterpret_cast<uint2*>(lo));
    ctx->launches++;
    B200_CUDA(ctx, cudaGetLastError());
    return B200_OK;
}

int launch_quantize_e4m3(b200_ctx* ctx, uint8_t* out, const float* in, size_t N, float scale) {
    if (N % 4) { ctx->last_error = "e4m3 quantisation: element count must be a multiple of 4"; return B200_ERR_SHAPE; }
    const size_t n4 = N / 4;
    const int grid = stream_grid(ctx, n4 > 0 ? n4 : 1, 256, 16);
    quantize_e4m3_kernel<<<grid, 256, 0, ctx->stream>>>(reinterpret_cast<uint32_t*>(out), reinterpret_cast<const float4*>(in), n4, scale);
    ctx->launches++;
    B200_CUDA(ctx, cudaGetLastError());
    return B200_OK;
}

int launch_split_fp16(b200_ctx* ctx, uint16_t* hi, uint16_t* lo, const float* in, size_t N) {
    if (N % 4) { ctx->last_error = "fp16 split: element count must be a multiple of 4"; return B200_ERR_SHAPE; }
    const size_t n4 = N / 4;
    const int grid = stream_grid(ctx, n4 > 0 ? n4 : 1, 256, 16);
    split_fp16_kernel<<<grid, 256, 0, ctx->stream>>>(reinterpret_cast<uint2*>(hi), reinterpret_cast<uint2*>(lo), reinterpret_cast<const float4*>(in), n4);
    ctx->launches++;
    B200_CUDA(ctx, cudaGetLastError());
    return B200_OK;
}

int launch_encoder(b200_ctx* ctx, float* out, const int* tok, const float* wte, const float* wpe,
                   int B, int T, int C, int vocab_rows) {
    int grid = (B * T + kRowWarps - 1) / kRowWarps;
    if (grid > 16 * ctx->num_sms) grid = 16 * ctx->num_sms;
    cudaError_t le = launch_pdl(ctx, encoder_kernel, dim3(grid), dim3(kRowWarps * 32), 0, reinterpret_cast<float4*>(out), tok,
                                reinterpret_cast<const float4*>(wte), reinterpret_cast<const float4*>(wpe), B * T, T,
                                C / 4, vocab_rows, ctx->d_status);
    ctx->launches++;
    B200_CUDA(ctx, le);
    return B200_OK;
}

int launch_fetch_ints(b200_ctx* ctx, int* dst, const int* src_view, int n) {
    const int threads = 256, grid = (n / 4 + threads) / threads;
    cudaError_t le = launch_pdl(ctx, fetch_ints_kernel, dim3(grid), dim3(threads), 0, dst, src_view, n);
    ctx->launches++;
    B200_CUDA(ctx, le);
    return B200_OK;
}

int launch_wait_timeout_probe(b200_ctx* ctx, unsigned long long limit_ns) {
    wait_timeout_probe_kernel<<<1, 32, 0, ctx->stream>>>(ctx->d_status, limit_ns);
    ctx->launches++;
    B200_CUDA(ctx, cudaGetLastError());
    return B200_OK;
}

// What the host-buffer forward sends back, prepared in one pass behind the lm-head:
//  * keys != null: the arg-max keys become column indices (0 for an untouched key) and are put
//    back to zero, which is the state the next lm-head with fused arg-max starts from;
//  * last_dst != null: the logits of the last position of every sequence, rows (b, T-1) of
//    logits[B*T, Vp], are gathered into the contiguous last_dst[B, Vp] (one plain copy to the
//    host instead of a strided one);
//  * status_dst != null: the context's status word as it stands behind all earlier kernels.
// out, last_dst and status_dst may address pinned host memory mapped into the device's address
// space: the results then cross PCIe from here and no copy is queued behind the forward.
__global__ void host_results_kernel(int* __restrict__ out, unsigned long long* __restrict__ keys, int M,
                                    float4* __restrict__ last_dst, const float4* __restrict__ logits, int B, int T,
                                    int Vp4, int* status_dst, const int* status_src) {
    griddep_wait();
    if (status_dst && blockIdx.x == 0 && threadIdx.x == 0) *status_dst = *status_src;
    const int stride = gridDim.x * blockDim.x;
    const int t0 = blockIdx.x * blockDim.x + threadIdx.x;
    if (keys) {
        for (int i = t0; i < M; i += stride) {
            const unsigned long long k = keys[i];
            out[i] = k ? (int)(0xFFFFFFFFu - (uint32_t)(k & 0xFFFFFFFFull)) : 0;
            keys[i] = 0ull;
        }
    }
    if (last_dst) {
        const int total = B * Vp4;
        for (int i = t0; i < total; i += stride) {
            const int b = i / Vp4, c = i - b * Vp4;
            last_dst[i] = logits[((size_t)b * T + (T - 1)) * Vp4 + c];
        }
    }
}

int launch_host_results(b200_ctx* ctx, int* out, unsigned long long* keys, int M, float* last_dst,
                        const float* logits, int B, int T, int Vp, int* status_dst) {
    const int work = (keys ? M : 0) > (last_dst ? B * (Vp / 4) : 0) ? M : (last_dst ? B * (Vp / 4) : M);
    int grid = (work + 255) / 256;
    if (grid > 4 * ctx->num_sms) grid = 4 * ctx->num_sms;
    if (grid < 1) grid = 1;
    cudaError_t le = launch_pdl(ctx, host_results_kernel, dim3(grid), dim3(256), 0, out, keys, M,
                                reinterpret_cast<float4*>(last_dst), reinterpret_cast<const float4*>(logits), B, T, Vp / 4,
                                status_dst, static_cast<const int*>(ctx->d_status));
    ctx->launches++;
    B200_CUDA(ctx, le);
    return B200_OK;
}

namespace {
// lse[r] = m + log(sum_i s_i * exp(m_i - m)), m = max_i m_i over the row's partial pairs (m_i, s_i);
// one warp per row
__global__ void __launch_bounds__(256)
lse_reduce_kernel(float* __restrict__ lse, const float2* __restrict__ part, int M, int slots) {
    griddep_wait();
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= M) return;
    const float2* p = part + (size_t)row * slots;
    float m = -INFINITY;
    for (int i = lane; i < slots; i += 32) m = fmaxf(m, p[i].x);
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, s));
    float sum = 0.f;
    for (int i = lane; i < slots; i += 32) {
        const float2 v = p[i];
        if (v.y > 0.f) sum += v.y * __expf(v.x - m);
    }
    sum = warp_sum(sum);
    if (lane == 0) lse[row] = m + logf(sum);
}
}  // namespace

int launch_lse_reduce(b200_ctx* ctx, float* lse, const float2* part, int M, int slots) {
    cudaError_t le = launch_pdl(ctx, lse_reduce_kernel, dim3((M + 7) / 8), dim3(256), 0, lse, part, M, slots);
    ctx->launches++;
    B200_CUDA(ctx, le);
    return B200_OK;
}

int launch_argmax_rows(b200_ctx* ctx, int* out, const float* logits, int M, int V, int ld) {
    argmax_rows_kernel<<<M, 256, 0, ctx->stream>>>(out, logits, V, ld);
    ctx->launches++;
    B200_CUDA(ctx, cudaGetLastError());
    return B200_OK;
}

int launch_sample_rows(b200_ctx* ctx, int* out, const float* logits, int M, int V, int ld, float temperature,
                       unsigned int seed, unsigned int stream0, int top_k, float top_p) {
    if (!(temperature > 0.f)) return launch_argmax_rows(ctx, out, logits, M, V, ld);
    sample_rows_kernel<<<M, 256, 0, ctx->stream>>>(out, logits, V, ld, 1.0f / temperature, seed, stream0, top_k, top_p);
    ctx->launches++;
    B200_CUDA(ctx, cudaGetLastError());
    return B200_OK;
}

}  // namespace b200
