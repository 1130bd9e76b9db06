// Causal multi-head attention, flash style, on the 5th-generation tensor cores.
//   out[b,t,h,:] = softmax_{j<=t}(q_t . k_j / sqrt(HS)) V        (HS = 64)
// Q, K and V are read by TMA straight out of the packed buffer inp[B,T,3,NH,HS] (row stride
// 3C), and the result is written in [B,T,NH,HS] order, so there are no permute / unpermute
// passes - the idea of kernels/attention/3_flash_attention_permute.cuh:46-58,306.  The math
// (scale 1/sqrt(HS), causal mask col <= row, online softmax) follows that file's
// :149-153,216-221,342 and kernels/attention/1_attention_cublas.cuh:50-61; the scores are
// never written to memory.  Unlike the reference's flash kernels (3_...cuh:349) the softmax
// statistics lse[B,NH,T] are written when asked for.
//
// One CTA = 128 query rows of one (batch, head), 6 warps:
//   warp 0     TMA producer: Q once, then K/V blocks of 128 keys into a 2-stage ring
//   warp 1     tensor-memory owner and UMMA issuer:  S_j = Q K_j^T  (kind::tf32, both operands
//              K-major from shared memory, accumulator in tensor memory, double buffered) and
//              O_j = P_j V_j (P from shared memory, V as an MN-major operand, loaded with the
//              32-byte-chunk swizzle that MN-major TF32 operands require)
//   warps 2-5  softmax: one query row per thread (no shuffles in the 32x32b tensor-memory
//              layout); two passes over S in tensor memory (row max, then exp2), P written to
//              shared memory in the swizzled K-major operand layout, O_j accumulated in fp32
//              registers with the usual rescale.  S_{j+1} is issued before P_j is needed, so the
//              tensor pipe works under the softmax.
// P is rounded to TF32 before it is both summed and multiplied, so the denominator matches
// the numerator.  Every wait is time-bounded (see prim/sm100.cuh).
#include "kernels.h"
#include "../prim/sm100.cuh"

namespace b200 {

namespace {

constexpr int HS = 64;
constexpr int BQ = 128;
constexpr int BKV = 128;
constexpr int kAttThreads = 192;
constexpr int kBlk = 16384;  // bytes of one {32 fp32 x 128 rows} swizzled block

struct AttSmem {
    static constexpr int Q_OFF = 0;                     // 2 blocks (hs 0-31, 32-63)
    static constexpr int K_OFF = Q_OFF + 2 * kBlk;      // 2 stages x 2 blocks
    static constexpr int V_OFF = K_OFF + 4 * kBlk;      // 2 stages x 2 blocks
    static constexpr int P_OFF = V_OFF + 4 * kBlk;      // 4 blocks (keys 0-31, ...)
    static constexpr int BAR_OFF = P_OFF + 4 * kBlk;
    static constexpr int TOTAL = 1024 + BAR_OFF + 256;
};
static_assert(AttSmem::TOTAL <= 232448, "shared memory over the 227 KB limit");
constexpr int kTmemCols = 512;  // S0 [0,128)  S1 [128,256)  O [256,320)

struct AttArgs {
    float* out;
    float* lse;
    int B, T, C, NH;
    int num_qt;
    float scale_log2;
    int round_out;  // store TF32-rounded outputs (they feed only the next GEMM)
    int* status;
};

__global__ void __launch_bounds__(kAttThreads, 1)
attention_kernel(const __grid_constant__ CUtensorMap tmap_qkv, const __grid_constant__ CUtensorMap tmap_v,
                 const AttArgs args) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* q_s = smem + AttSmem::Q_OFF;
    uint8_t* k_s = smem + AttSmem::K_OFF;
    uint8_t* v_s = smem + AttSmem::V_OFF;
    uint8_t* p_s = smem + AttSmem::P_OFF;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + AttSmem::BAR_OFF);
    uint64_t* q_full = bars;          // [1]
    uint64_t* kv_full = bars + 1;     // [2]
    uint64_t* kv_empty = bars + 3;    // [2]
    uint64_t* s_full = bars + 5;      // [2]
    uint64_t* p_full = bars + 7;      // [1]
    uint64_t* o_full = bars + 8;      // [1]
    uint64_t* drain_bar = bars + 9;   // [1]
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 10);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // heaviest (last) query tiles first
    const int qt = args.num_qt - 1 - blockIdx.x;
    const int h = blockIdx.y;
    const int b = blockIdx.z;
    const int q0 = qt * BQ;
    const int n_kv = qt + 1;
    const int row_base = b * args.T;  // first row of this sequence in the [B*T, 3C] matrix

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < 2; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); mbar_init(&s_full[s], 1); }
        mbar_init(p_full, 128);
        mbar_init(o_full, 1);
        mbar_init(drain_bar, 1);
        *abort_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tmap_qkv);
        tma_prefetch_desc(&tmap_v);
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
            mbar_arrive_expect_tx(q_full, 2 * kBlk);
            tma_load_2d(q_s, &tmap_qkv, xq, row_base + q0, q_full);
            tma_load_2d(q_s + kBlk, &tmap_qkv, xq + 32, row_base + q0, q_full);
            for (int j = 0; j < n_kv; ++j) {
                const int s = j & 1;
                const uint32_t ph = (j >> 1) & 1;
                if (!mbar_wait(&kv_empty[s], ph ^ 1, abort_flag)) { ok = false; break; }
                mbar_arrive_expect_tx(&kv_full[s], 4 * kBlk);
                const int y = row_base + j * BKV;
                tma_load_2d(k_s + (2 * s) * kBlk, &tmap_qkv, xk, y, &kv_full[s]);
                tma_load_2d(k_s + (2 * s + 1) * kBlk, &tmap_qkv, xk + 32, y, &kv_full[s]);
                tma_load_2d(v_s + (2 * s) * kBlk, &tmap_v, xv, y, &kv_full[s]);
                tma_load_2d(v_s + (2 * s + 1) * kBlk, &tmap_v, xv + 32, y, &kv_full[s]);
            }
            if (!ok) atomicCAS(args.status, 0, DEV_TIMEOUT_PRODUCER);
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_s = make_idesc_tf32(BQ, BKV, 0);  // S = Q K^T, N = 128 keys
            constexpr uint32_t idesc_o = make_idesc_tf32(BQ, HS, 1);   // O = P V,   N = 64, V MN-major
            bool ok = true;
            auto issue_s = [&](int j) {
                const int s = j & 1;
                const uint32_t d = tmem_base + s * BKV;
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    const uint32_t off = (kk >> 2) * kBlk + (kk & 3) * 32;
                    const uint64_t a = make_smem_desc_sw128(smem_u32(q_s) + off, 16, 1024);
                    const uint64_t bd = make_smem_desc_sw128(smem_u32(k_s + 2 * s * kBlk) + off, 16, 1024);
                    umma_tf32_ss(d, a, bd, idesc_s, kk != 0);
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
                const uint32_t d = tmem_base + 2 * BKV;
#pragma unroll
                for (int ks = 0; ks < BKV / 8; ++ks) {
                    // A: P, K-major, 8 keys = 32 bytes inside the 32-key block
                    const uint64_t a = make_smem_desc_sw128(smem_u32(p_s) + (ks >> 2) * kBlk + (ks & 3) * 32, 16, 1024);
                    // B: V, MN-major (32-byte-chunk swizzle): 8 keys = 8 rows of 128 bytes = two
                    // 4-row swizzle groups 512 bytes apart; the two 32-wide halves of the head
                    // dimension lie kBlk apart
                    const uint64_t bd = make_smem_desc_sw128<1>(smem_u32(v_s + 2 * s * kBlk) + ks * 1024, kBlk, 512);
                    umma_tf32_ss(d, a, bd, idesc_o, ks != 0);
                }
                umma_commit(o_full);
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

        auto accumulate_o = [&](float alpha) {
#pragma unroll
            for (int c = 0; c < HS / 32; ++c) {
                uint32_t t[32];
                tmem_ld_32x32b_x32(tmem_base + lane_addr + 2 * BKV + c * 32, t);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) o_acc[c * 32 + i] = o_acc[c * 32 + i] * alpha + __uint_as_float(t[i]);
            }
        };

        for (int j = 0; j < n_kv; ++j) {
            const int s = j & 1;
            if (!mbar_wait(&s_full[s], (j >> 1) & 1, abort_flag)) { ok = false; break; }
            tc_fence_after_sync();
            const bool diag = (j == n_kv - 1);
            const uint32_t s_addr = tmem_base + lane_addr + s * BKV;
            // pass 1: row maximum (log2 domain)
            float mx = m;
#pragma unroll 1
            for (int c = 0; c < BKV / 32; ++c) {
                uint32_t t[32];
                tmem_ld_32x32b_x32(s_addr + c * 32, t);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const float sv = __uint_as_float(t[i]) * args.scale_log2;
                    if (!diag || (c * 32 + i) <= r) mx = fmaxf(mx, sv);
                }
            }
            const float alpha = exp2f(m - mx);  // 0 on the first block (m = -inf, mx finite)
            m = mx;
            // O_{j-1} must have left P (and landed in tensor memory) before P is overwritten
            if (j > 0) {
                if (!mbar_wait(o_full, (j - 1) & 1, abort_flag)) { ok = false; break; }
                tc_fence_after_sync();
                accumulate_o(alpha_prev);
            }
            // pass 2: P = exp2(s - m), rounded to TF32, summed and stored as the A operand
            float sum = 0.f;
#pragma unroll 1
            for (int c = 0; c < BKV / 32; ++c) {
                uint32_t t[32];
                tmem_ld_32x32b_x32(s_addr + c * 32, t);
                tmem_ld_wait();
                float p[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const float sv = __uint_as_float(t[i]) * args.scale_log2;
                    float pv = round_tf32(exp2f(sv - mx));
                    if (diag && (c * 32 + i) > r) pv = 0.f;
                    p[i] = pv;
                    sum += pv;
                }
                uint8_t* prow = p_s + c * kBlk + r * 128;
#pragma unroll
                for (int j4 = 0; j4 < 8; ++j4) {
                    *reinterpret_cast<float4*>(prow + ((j4 ^ (r & 7)) << 4)) =
                        make_float4(p[4 * j4], p[4 * j4 + 1], p[4 * j4 + 2], p[4 * j4 + 3]);
                }
            }
            l = l * alpha + sum;
            alpha_prev = alpha;
            fence_proxy_async_smem();   // P (generic-proxy stores) -> visible to the UMMA reads
            tc_fence_before_sync();     // the tcgen05.ld of S are ordered before the arrive
            mbar_arrive(p_full);
        }
        if (ok) {
            if (mbar_wait(o_full, (n_kv - 1) & 1, abort_flag)) {
                tc_fence_after_sync();
                accumulate_o(alpha_prev);
                const int t_idx = q0 + r;
                if (t_idx < args.T) {
                    const float inv_l = 1.0f / l;
                    float* o = args.out + ((size_t)(row_base + t_idx) * args.C) + h * HS;
#pragma unroll
                    for (int i = 0; i < HS / 4; ++i) {
                        float4 v = make_float4(o_acc[4 * i] * inv_l, o_acc[4 * i + 1] * inv_l,
                                               o_acc[4 * i + 2] * inv_l, o_acc[4 * i + 3] * inv_l);
                        if (args.round_out) { v.x = round_tf32(v.x); v.y = round_tf32(v.y); v.z = round_tf32(v.z); v.w = round_tf32(v.w); }
                        *reinterpret_cast<float4*>(o + 4 * i) = v;
                    }
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

}  // namespace

int launch_attention(b200_ctx* ctx, float* out, float* lse, const float* qkv, int B, int T, int C,
                     int NH, int flags) {
    static bool attr_set[64] = {};
    if (!attr_set[ctx->device & 63]) {
        B200_CUDA(ctx, cudaFuncSetAttribute(attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AttSmem::TOTAL));
        attr_set[ctx->device & 63] = true;
    }
    CUtensorMap tm;
    int st = b200_get_tensor_map(ctx, &tm, qkv, (uint64_t)B * T, (uint64_t)3 * C, (uint64_t)3 * C, BKV, 32);
    if (st != B200_OK) return st;
    CUtensorMap tmv;  // V is consumed as an MN-major operand: 32-byte-chunk swizzle
    st = b200_get_tensor_map(ctx, &tmv, qkv, (uint64_t)B * T, (uint64_t)3 * C, (uint64_t)3 * C, BKV, 32, 1);
    if (st != B200_OK) return st;
    AttArgs a;
    a.out = out; a.lse = lse; a.B = B; a.T = T; a.C = C; a.NH = NH;
    a.num_qt = (T + BQ - 1) / BQ;
    a.scale_log2 = 1.4426950408889634f / sqrtf((float)HS);
    a.round_out = (flags & ROUND_OUT_TF32) ? 1 : 0;
    a.status = ctx->d_status;
    dim3 grid(a.num_qt, NH, B);
    attention_kernel<<<grid, kAttThreads, AttSmem::TOTAL, ctx->stream>>>(tm, tmv, a);
    ctx->launches++;
    B200_CUDA(ctx, cudaGetLastError());
    return B200_OK;
}

}  // namespace b200
