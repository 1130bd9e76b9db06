// Causal attention with split-operand (3xTF32) products: the same math and layouts as
// attention.cu (reference: kernels/attention/3_flash_attention_permute.cuh:46-58,149-153,216-221,
// 306,342), for the B200_TF32X3 mode, where q.k and p.v must not lose the low 13 mantissa bits of
// their fp32 operands.
//
// The tensor core truncates an fp32 operand x to TF32, i.e. it multiplies with x_big = trunc(x).
// A small pre-pass writes the dropped parts  x_small = x - trunc(x)  of the whole packed QKV
// buffer into a scratch buffer of the same shape (the `qkvr` argument of the reference's
// attention signature), and every product is then accumulated from three UMMAs:
//     S = Q K^T  ~  Q.K + Q_small.K + Q.K_small          O = P V  ~  P.V + P_small.V + P.V_small
// (the operands named without suffix are the raw fp32 values, which the hardware truncates).
// P is split by the softmax threads themselves; the row sum uses the full fp32 P.
//
// One CTA = 128 query rows of one (batch, head), keys in blocks of 64 (both big and small tiles
// of K and V have to fit a 2-stage ring): warp 0 TMA producer, warp 1 tensor-memory owner and
// UMMA issuer (S_{j+1} is issued before P_j is needed), warps 2-5 softmax with one row per
// thread.  P and P_small live in tensor memory and are read as the A operand from there.
// Every wait is time-bounded (prim/sm100.cuh).
#include "kernels.h"
#include "../prim/sm100.cuh"

namespace b200 {

namespace {

constexpr int HS = 64;
constexpr int BQ = 128;
constexpr int BKV = 64;
constexpr int kThreads = 192;
constexpr int kQBlk = 16384;  // {32 fp32 x 128 rows}
constexpr int kKBlk = 8192;   // {32 fp32 x 64 rows}

struct Smem {
    static constexpr int Q_OFF = 0;                      // Q: 2 blocks
    static constexpr int QS_OFF = Q_OFF + 2 * kQBlk;     // Q_small: 2 blocks
    static constexpr int ST_OFF = QS_OFF + 2 * kQBlk;    // 2 stages x {K, K_small, V, V_small} x 2 blocks
    static constexpr int STAGE = 8 * kKBlk;
    static constexpr int BAR_OFF = ST_OFF + 2 * STAGE;
    static constexpr int TOTAL = 1024 + BAR_OFF + 256;
};
static_assert(Smem::TOTAL <= 232448 && Smem::TOTAL > 117 * 1024, "one CTA per SM, within 227 KB");
// tensor-memory columns: S0 [0,64) S1 [64,128) P [128,192) P_small [192,256) O0 [256,320) O1 [320,384)
constexpr int kTmemCols = 512, kPCol = 128, kPsCol = 192, kOCol = 256;

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

struct Args {
    float* out;
    float* lse;
    int B, T, C, NH;
    int num_qt;
    float scale_log2;
    int* status;
};

__global__ void __launch_bounds__(kThreads, 1)
attention_x3_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_qs,
                    const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_ks,
                    const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_vs,
                    const Args args) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* q_s = smem + Smem::Q_OFF;
    uint8_t* qs_s = smem + Smem::QS_OFF;
    uint8_t* st_s = smem + Smem::ST_OFF;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Smem::BAR_OFF);
    uint64_t* q_full = bars;          // [1]
    uint64_t* kv_full = bars + 1;     // [2]
    uint64_t* kv_empty = bars + 3;    // [2]
    uint64_t* s_full = bars + 5;      // [2]
    uint64_t* p_full = bars + 7;      // [1]
    uint64_t* o_full = bars + 8;      // [2]
    uint64_t* drain_bar = bars + 10;  // [1]
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 11);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int qt = args.num_qt - 1 - blockIdx.x;  // heaviest query tiles first
    const int h = blockIdx.y;
    const int b = blockIdx.z;
    const int q0 = qt * BQ;
    const int n_kv = 2 * qt + 2;  // key blocks 0 .. 2*qt+1; the last two straddle the diagonal
    const int row_base = b * args.T;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&kv_full[s], 1);
            mbar_init(&kv_empty[s], 1);
            mbar_init(&s_full[s], 1);
            mbar_init(&o_full[s], 1);
        }
        mbar_init(p_full, 128);
        mbar_init(drain_bar, 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_holder, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            bool ok = true;
            const int xq = h * HS, xk = args.C + h * HS, xv = 2 * args.C + h * HS;
            mbar_arrive_expect_tx(q_full, 4 * kQBlk);
            tma_load_2d(q_s, &map_q, xq, row_base + q0, q_full);
            tma_load_2d(q_s + kQBlk, &map_q, xq + 32, row_base + q0, q_full);
            tma_load_2d(qs_s, &map_qs, xq, row_base + q0, q_full);
            tma_load_2d(qs_s + kQBlk, &map_qs, xq + 32, row_base + q0, q_full);
            for (int j = 0; j < n_kv; ++j) {
                const int s = j & 1;
                if (!mbar_wait(&kv_empty[s], ((j >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
                mbar_arrive_expect_tx(&kv_full[s], Smem::STAGE);
                uint8_t* st = st_s + s * Smem::STAGE;
                const int y = row_base + j * BKV;
                tma_load_2d(st + 0 * kKBlk, &map_k, xk, y, &kv_full[s]);
                tma_load_2d(st + 1 * kKBlk, &map_k, xk + 32, y, &kv_full[s]);
                tma_load_2d(st + 2 * kKBlk, &map_ks, xk, y, &kv_full[s]);
                tma_load_2d(st + 3 * kKBlk, &map_ks, xk + 32, y, &kv_full[s]);
                tma_load_2d(st + 4 * kKBlk, &map_v, xv, y, &kv_full[s]);
                tma_load_2d(st + 5 * kKBlk, &map_v, xv + 32, y, &kv_full[s]);
                tma_load_2d(st + 6 * kKBlk, &map_vs, xv, y, &kv_full[s]);
                tma_load_2d(st + 7 * kKBlk, &map_vs, xv + 32, y, &kv_full[s]);
            }
            if (!ok) atomicCAS(args.status, 0, DEV_TIMEOUT_PRODUCER);
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------- UMMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_s = make_idesc_tf32(BQ, BKV, 0);  // S: N = 64 keys
            constexpr uint32_t idesc_o = make_idesc_tf32(BQ, HS, 1);   // O: N = 64, V MN-major
            bool ok = true;
            auto issue_s = [&](int j) {
                const int s = j & 1;
                const uint8_t* st = st_s + s * Smem::STAGE;
                const uint32_t d = tmem_base + s * BKV;
                // three passes: Q.K, Q_small.K, Q.K_small
#pragma unroll
                for (int pass = 0; pass < 3; ++pass) {
                    const uint32_t a_base = smem_u32(pass == 1 ? qs_s : q_s);
                    const uint32_t b_base = smem_u32(st + (pass == 2 ? 2 : 0) * kKBlk);
#pragma unroll
                    for (int kk = 0; kk < 8; ++kk) {
                        const uint64_t a = make_smem_desc_sw128(a_base + (kk >> 2) * kQBlk + (kk & 3) * 32, 16, 1024);
                        const uint64_t bd = make_smem_desc_sw128(b_base + (kk >> 2) * kKBlk + (kk & 3) * 32, 16, 1024);
                        umma_tf32_ss(d, a, bd, idesc_s, (pass | kk) != 0);
                    }
                }
                umma_commit(&s_full[s]);
            };
            ok = mbar_wait(q_full, 0, abort_flag);
            if (ok) ok = mbar_wait(&kv_full[0], 0, abort_flag);
            if (ok) {
                tc_fence_after_sync();
                issue_s(0);
            }
            for (int j = 0; j < n_kv && ok; ++j) {
                if (j + 1 < n_kv) {
                    if (!mbar_wait(&kv_full[(j + 1) & 1], ((j + 1) >> 1) & 1, abort_flag)) { ok = false; break; }
                    tc_fence_after_sync();
                    issue_s(j + 1);
                }
                if (!mbar_wait(p_full, j & 1, abort_flag)) { ok = false; break; }
                tc_fence_after_sync();
                const int s = j & 1;
                const uint8_t* st = st_s + s * Smem::STAGE;
                const uint32_t d = tmem_base + kOCol + s * HS;
                // three passes: P.V, P_small.V, P.V_small  (P from tensor memory; V MN-major:
                // 8 keys = 8 rows of 128 bytes = two 4-row swizzle groups 512 bytes apart, the
                // two 32-wide halves of the head dimension kKBlk apart)
#pragma unroll
                for (int pass = 0; pass < 3; ++pass) {
                    const uint32_t a_col = tmem_base + (pass == 1 ? kPsCol : kPCol);
                    const uint32_t b_base = smem_u32(st + (pass == 2 ? 6 : 4) * kKBlk);
#pragma unroll
                    for (int ks = 0; ks < BKV / 8; ++ks) {
                        const uint64_t bd = make_smem_desc_sw128<1>(b_base + ks * 1024, kKBlk, 512);
                        umma_tf32_ts(d, a_col + ks * 8, bd, idesc_o, (pass | ks) != 0);
                    }
                }
                umma_commit(&o_full[s]);
                umma_commit(&kv_empty[s]);
            }
            umma_commit(drain_bar);
            if (!mbar_wait(drain_bar, 0, abort_flag)) ok = false;
            if (!ok) atomicCAS(args.status, 0, DEV_TIMEOUT_MMA);
        }
    } else {
        // ----------------------------------------------------------------- softmax
        const int qd = warp & 3;
        const int r = qd * 32 + lane;  // query row inside the tile = tensor-memory lane
        const uint32_t lane_addr = uint32_t(qd * 32) << 16;
        float m = -INFINITY, l = 0.f, alpha_prev = 0.f;
        float o_acc[HS];
#pragma unroll
        for (int i = 0; i < HS; ++i) o_acc[i] = 0.f;
        bool ok = true;

        auto accumulate_o = [&](float alpha, int buf) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t t[32];
                tmem_ld_32x32b_x32(tmem_base + lane_addr + kOCol + buf * HS + c * 32, t);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) o_acc[c * 32 + i] = o_acc[c * 32 + i] * alpha + __uint_as_float(t[i]);
            }
        };

        for (int j = 0; j < n_kv; ++j) {
            const int s = j & 1;
            if (!mbar_wait(&s_full[s], (j >> 1) & 1, abort_flag)) { ok = false; break; }
            tc_fence_after_sync();
            // keys of this block visible to row r: columns c <= lim (lim >= 63: all; lim < 0: none)
            const int lim = q0 + r - j * BKV;
            uint32_t t0[32], t1[32];
            const uint32_t s_addr = tmem_base + lane_addr + s * BKV;
            tmem_ld_32x32b_x32(s_addr, t0);
            tmem_ld_32x32b_x32(s_addr + 32, t1);
            tmem_ld_wait();
            float mx_raw = -INFINITY;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                if (i <= lim) mx_raw = fmaxf(mx_raw, __uint_as_float(t0[i]));
                if (32 + i <= lim) mx_raw = fmaxf(mx_raw, __uint_as_float(t1[i]));
            }
            // a row with no visible key in this block keeps its running maximum (finite from block 0 on)
            const float mx = fmaxf(m, mx_raw * args.scale_log2);
            const float alpha = ex2_approx(m - mx);
            m = mx;
            if (j > 0) {
                // O_{j-1} has retired: fold it in, and the P columns may be overwritten
                if (!mbar_wait(&o_full[(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag)) { ok = false; break; }
                tc_fence_after_sync();
                accumulate_o(alpha_prev, (j - 1) & 1);
            }
            float sum = 0.f;
            const float neg_mx = -mx;
            uint32_t ps[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                float p = ex2_approx(fmaf(__uint_as_float(t0[i]), args.scale_log2, neg_mx));
                if (i > lim) p = 0.f;
                sum += p;
                const uint32_t big = __float_as_uint(p) & 0xFFFFE000u;
                t0[i] = big;
                ps[i] = __float_as_uint(p - __uint_as_float(big));
            }
            tmem_st_32x32b_x32(tmem_base + lane_addr + kPCol, t0);
            tmem_st_32x32b_x32(tmem_base + lane_addr + kPsCol, ps);
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                float p = ex2_approx(fmaf(__uint_as_float(t1[i]), args.scale_log2, neg_mx));
                if (32 + i > lim) p = 0.f;
                sum += p;
                const uint32_t big = __float_as_uint(p) & 0xFFFFE000u;
                t1[i] = big;
                ps[i] = __float_as_uint(p - __uint_as_float(big));
            }
            tmem_st_32x32b_x32(tmem_base + lane_addr + kPCol + 32, t1);
            tmem_st_32x32b_x32(tmem_base + lane_addr + kPsCol + 32, ps);
            tmem_st_wait();
            l = l * alpha + sum;
            alpha_prev = alpha;
            tc_fence_before_sync();
            mbar_arrive(p_full);
        }
        if (ok) {
            if (mbar_wait(&o_full[(n_kv - 1) & 1], ((n_kv - 1) >> 1) & 1, abort_flag)) {
                tc_fence_after_sync();
                accumulate_o(alpha_prev, (n_kv - 1) & 1);
                const int t_idx = q0 + r;
                if (t_idx < args.T) {
                    const float inv_l = 1.0f / l;
                    float* o = args.out + ((size_t)(row_base + t_idx) * args.C) + h * HS;
#pragma unroll
                    for (int i = 0; i < HS / 4; ++i)
                        *reinterpret_cast<float4*>(o + 4 * i) =
                            make_float4(o_acc[4 * i] * inv_l, o_acc[4 * i + 1] * inv_l, o_acc[4 * i + 2] * inv_l,
                                        o_acc[4 * i + 3] * inv_l);
                    if (args.lse)
                        args.lse[((size_t)b * args.NH + h) * args.T + t_idx] = m * 0.6931471805599453f + logf(l);
                }
            } else {
                ok = false;
            }
        }
        if (!ok && lane == 0) atomicCAS(args.status, 0, DEV_TIMEOUT_SOFTMAX);
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// small = x - trunc_tf32(x): the part of every fp32 value that the tensor core drops
__global__ void split_tf32_kernel(float4* __restrict__ small, const float4* __restrict__ x, size_t n4) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        const float4 v = x[i];
        float4 s;
        s.x = v.x - __uint_as_float(__float_as_uint(v.x) & 0xFFFFE000u);
        s.y = v.y - __uint_as_float(__float_as_uint(v.y) & 0xFFFFE000u);
        s.z = v.z - __uint_as_float(__float_as_uint(v.z) & 0xFFFFE000u);
        s.w = v.w - __uint_as_float(__float_as_uint(v.w) & 0xFFFFE000u);
        small[i] = s;
    }
}

}  // namespace

int launch_attention_x3(b200_ctx* ctx, float* out, float* qkv_small, float* lse, const float* qkv, int B, int T,
                        int C, int NH) {
    static bool attr_set[64] = {};
    if (!attr_set[ctx->device & 63]) {
        B200_CUDA(ctx, cudaFuncSetAttribute(attention_x3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::TOTAL));
        attr_set[ctx->device & 63] = true;
    }
    const size_t n4 = (size_t)B * T * 3 * C / 4;
    size_t blocks = (n4 + 255) / 256;
    const size_t cap = (size_t)ctx->num_sms * 16;
    if (blocks > cap) blocks = cap;
    split_tf32_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(reinterpret_cast<float4*>(qkv_small),
                                                                reinterpret_cast<const float4*>(qkv), n4);
    ctx->launches++;
    B200_CUDA(ctx, cudaGetLastError());

    const uint64_t rows = (uint64_t)B * T, cols = (uint64_t)3 * C;
    CUtensorMap mq, mqs, mk, mks, mv, mvs;
    int st;
    if ((st = b200_get_tensor_map(ctx, &mq, qkv, rows, cols, cols, BQ, 32, 0)) != B200_OK) return st;
    if ((st = b200_get_tensor_map(ctx, &mqs, qkv_small, rows, cols, cols, BQ, 32, 0)) != B200_OK) return st;
    if ((st = b200_get_tensor_map(ctx, &mk, qkv, rows, cols, cols, BKV, 32, 0)) != B200_OK) return st;
    if ((st = b200_get_tensor_map(ctx, &mks, qkv_small, rows, cols, cols, BKV, 32, 0)) != B200_OK) return st;
    if ((st = b200_get_tensor_map(ctx, &mv, qkv, rows, cols, cols, BKV, 32, 1)) != B200_OK) return st;
    if ((st = b200_get_tensor_map(ctx, &mvs, qkv_small, rows, cols, cols, BKV, 32, 1)) != B200_OK) return st;
    Args a;
    a.out = out; a.lse = lse; a.B = B; a.T = T; a.C = C; a.NH = NH;
    a.num_qt = (T + BQ - 1) / BQ;
    a.scale_log2 = 1.4426950408889634f / sqrtf((float)HS);
    a.status = ctx->d_status;
    dim3 grid(a.num_qt, NH, B);
    attention_x3_kernel<<<grid, kThreads, Smem::TOTAL, ctx->stream>>>(mq, mqs, mk, mks, mv, mvs, a);
    ctx->launches++;
    B200_CUDA(ctx, cudaGetLastError());
    return B200_OK;
}

}  // namespace b200
