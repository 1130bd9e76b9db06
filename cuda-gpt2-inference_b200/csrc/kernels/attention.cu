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
// One CTA = 128 query rows of one (batch, head), 11 warps:
//   warp 0      TMA producer: Q once, then K/V blocks of 128 keys into a 3-stage ring
//   warp 1      tensor-memory owner; one lane issues  S_j = Q K_j^T  (kind::tf32, both operands
//               K-major from shared memory, accumulator double buffered in tensor memory)
//   warp 10     one lane issues  O_j = P_j V_j  (P read from tensor memory, where the softmax
//               wrote it; V as an MN-major operand from shared memory, loaded with the
//               32-byte-chunk swizzle that MN-major TF32 operands require).  P never touches
//               shared memory: fp32 operands make shared-memory bandwidth the scarce resource.
//               Two issuing threads, because a UMMA covers only 8 of the 128 keys and the
//               issue rate of one thread (about 65 cycles per instruction) would otherwise
//               bound the loop.
//   warps 2-9   softmax: a query row is a tensor-memory lane, shared by two threads (warps w and
//               w+4) that each take 64 of the 128 keys and 32 of the 64 output columns.  Each
//               reads its scores once into registers (freeing the S buffer early), the two
//               exchange their row maxima through shared memory, then P = exp2(s*scale - m) is
//               cut to TF32, summed, and stored into the P columns of tensor memory; O_j
//               (double buffered in tensor memory) is accumulated in fp32 registers with the
//               usual rescale, one block behind.  All tensor-memory reads of an iteration
//               (O_{j-1}, S_{j+1}) happen before P_j is handed to the tensor core; the
//               arithmetic runs under its UMMAs.
// P is cut to TF32 before it is both summed and multiplied, so the denominator matches the
// numerator.  Every wait is time-bounded (see prim/sm100.cuh).
#include "kernels.h"
#include "../prim/sm100.cuh"

namespace b200 {

namespace {

constexpr int HS = 64;
constexpr int BQ = 128;
constexpr int BKV = 128;
constexpr int kAttThreads = 352;
constexpr int kBlk = 16384;  // bytes of one {32 fp32 x 128 rows} swizzled block
constexpr int kStages = 3;   // K/V ring

struct AttSmem {
    static constexpr int Q_OFF = 0;                     // 2 blocks (hs 0-31, 32-63)
    static constexpr int K_OFF = Q_OFF + 2 * kBlk;            // kStages x 2 blocks
    static constexpr int V_OFF = K_OFF + 2 * kStages * kBlk;  // kStages x 2 blocks
    static constexpr int X_OFF = V_OFF + 2 * kStages * kBlk;  // exchange buffer: 2 halves x 128 floats
    static constexpr int BAR_OFF = X_OFF + 2 * 128 * 4;
    static constexpr int TOTAL = 1024 + BAR_OFF + 128;
};
static_assert(AttSmem::TOTAL <= 232448, "shared memory over the 227 KB limit");
constexpr int kTmemCols = 512;  // S0 [0,128)  S1 [128,256)  P [256,384)  O0 [384,448)  O1 [448,512)
constexpr int kPCol = 256, kOCol = 384;

// 2^x on the special-function unit (one instruction; 2^-inf = 0)
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// barrier among the two warps that share a group of 32 query rows
__device__ __forceinline__ void pair_bar_sync(int id) {
    asm volatile("bar.sync %0, 64;" ::"r"(id) : "memory");
}

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
    float* xchg = reinterpret_cast<float*>(smem + AttSmem::X_OFF);  // [2][128]
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + AttSmem::BAR_OFF);
    uint64_t* q_full = bars;          // [1]  TMA: Q landed
    uint64_t* kv_full = bars + 1;     // [3]  TMA: K/V block landed
    uint64_t* kv_empty = bars + 4;    // [3]  PV of the block retired
    uint64_t* s_full = bars + 7;      // [2]  S computed
    uint64_t* s_free = bars + 9;      // [2]  S read into registers by all 256 softmax threads
    uint64_t* p_full = bars + 11;     // [1]  P written by all 256 softmax threads
    uint64_t* o_full = bars + 12;     // [2]  O_j in tensor memory
    uint64_t* drain_bar = bars + 14;  // [1]
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 15);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

#ifdef B200_ATT_TIMING
    const unsigned long long dbg_t_start = globaltimer_ns();
#endif
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
        for (int s = 0; s < kStages; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
        for (int s = 0; s < 2; ++s) { mbar_init(&s_full[s], 1); mbar_init(&s_free[s], 256); mbar_init(&o_full[s], 1); }
        mbar_init(p_full, 256);
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
    griddep_wait();  // set-up done; from here on global memory is touched

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            bool ok = true;
            const int xq = h * HS, xk = args.C + h * HS, xv = 2 * args.C + h * HS;
            mbar_arrive_expect_tx(q_full, 2 * kBlk);
            tma_load_2d(q_s, &tmap_qkv, xq, row_base + q0, q_full);
            tma_load_2d(q_s + kBlk, &tmap_qkv, xq + 32, row_base + q0, q_full);
            for (int j = 0; j < n_kv; ++j) {
                const int s = j % kStages;
                const uint32_t ph = (j / kStages) & 1;
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
        // ------------------------------------------------------- S = Q K^T issuer
        if (lane == 0) {
            constexpr uint32_t idesc_s = make_idesc_tf32(BQ, BKV, 0);  // N = 128 keys
            bool ok = mbar_wait(q_full, 0, abort_flag);
            for (int j = 0; j < n_kv && ok; ++j) {
                const int s = j & 1, ks3 = j % kStages;
                if (!mbar_wait(&kv_full[ks3], (j / kStages) & 1, abort_flag)) { ok = false; break; }
                // the softmax has read S_{j-2} out of these columns
                if (!mbar_wait(&s_free[s], ((j >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t d = tmem_base + s * BKV;
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    const uint32_t off = (kk >> 2) * kBlk + (kk & 3) * 32;
                    const uint64_t a = make_smem_desc_sw128(smem_u32(q_s) + off, 16, 1024);
                    const uint64_t bd = make_smem_desc_sw128(smem_u32(k_s + 2 * ks3 * kBlk) + off, 16, 1024);
                    umma_tf32_ss(d, a, bd, idesc_s, kk != 0);
                }
                umma_commit(&s_full[s]);
            }
            if (!ok) atomicCAS(args.status, 0, DEV_TIMEOUT_MMA);
        }
    } else if (warp == 10) {
        // --------------------------------------------------------- O = P V issuer
        if (lane == 0) {
            constexpr uint32_t idesc_o = make_idesc_tf32(BQ, HS, 1);  // N = 64, V MN-major
            bool ok = true;
            for (int j = 0; j < n_kv && ok; ++j) {
                const int s = j & 1, ks3 = j % kStages;
                if (!mbar_wait(p_full, j & 1, abort_flag)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t d = tmem_base + kOCol + s * HS;
#pragma unroll
                for (int ks = 0; ks < BKV / 8; ++ks) {
                    // A: P_j in tensor memory, 8 keys = 8 columns per instruction
                    const uint32_t a = tmem_base + kPCol + ks * 8;
                    // B: V, MN-major (32-byte-chunk swizzle): 8 keys = 8 rows of 128 bytes = two
                    // 4-row swizzle groups 512 bytes apart; the two 32-wide halves of the head
                    // dimension lie kBlk apart
                    const uint64_t bd = make_smem_desc_sw128<1>(smem_u32(v_s + 2 * ks3 * kBlk) + ks * 1024, kBlk, 512);
                    umma_tf32_ts(d, a, bd, idesc_o, ks != 0);
                }
                umma_commit(&o_full[s]);
                umma_commit(&kv_empty[ks3]);
            }
            // both issuers' work has retired once this commit arrives (the last PV depends on
            // the last S through the softmax)
            umma_commit(drain_bar);
            if (!mbar_wait(drain_bar, 0, abort_flag)) ok = false;
            if (!ok) atomicCAS(args.status, 0, DEV_TIMEOUT_MMA);
        }
    } else {
        // ----------------------------------------------------------------- softmax
        const int qd = warp & 3;                 // tensor-memory lane quarter of this warp
        const int hf = (warp - 2) >> 2;          // which 64 keys / 32 output columns
        const int r = qd * 32 + lane;            // query row inside the tile = tensor-memory lane
        const uint32_t lane_addr = uint32_t(qd * 32) << 16;
        const int bar_id = 1 + qd;               // named barrier of the two warps sharing the rows
        float m = -INFINITY, l = 0.f, alpha_prev = 0.f;
        float o_acc[HS / 2];
#pragma unroll
        for (int i = 0; i < HS / 2; ++i) o_acc[i] = 0.f;
        bool ok = true;

        auto accumulate_o = [&](float alpha, int buf) {
            uint32_t t[32];
            tmem_ld_32x32b_x32(tmem_base + lane_addr + kOCol + buf * HS + hf * 32, t);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o_acc[i] = o_acc[i] * alpha + __uint_as_float(t[i]);
        };

        // No early exit from this loop: after a wait has run out the remaining waits are skipped
        // but every pair barrier is still executed, so the partner warp can never be left alone
        // in one (the results are discarded and the status word says why).
        // Every tensor-memory read of an iteration is done before p_full is signalled, i.e.
        // while the tensor core is not running O = P V (whose P operand also comes out of tensor
        // memory and would stall the loads); the arithmetic on the values runs under the UMMAs.
        uint32_t t0[32], t1[32];  // this thread's 64 scores of the current block, then its P
        if (ok && !mbar_wait(&s_full[0], 0, abort_flag)) ok = false;
        tc_fence_after_sync();
        {
            const uint32_t s_addr = tmem_base + lane_addr + hf * 64;
            tmem_ld_32x32b_x32(s_addr, t0);
            tmem_ld_32x32b_x32(s_addr + 32, t1);
            tmem_ld_wait();
            tc_fence_before_sync();
            mbar_arrive(&s_free[0]);
        }
        const uint32_t p_addr = tmem_base + lane_addr + kPCol + hf * 64;
        // No early exit from this loop: after a wait has run out the remaining waits are skipped
        // but every pair barrier is still executed, so the partner warp can never be left alone
        // in one (the results are discarded and the status word says why).
        for (int j = 0; j < n_kv; ++j) {
            const bool diag = (j == n_kv - 1);
            // row maximum of the raw scores (the scale is positive, so it commutes with max)
            const int c0 = hf * 64;  // first key column of this thread within the block
            float pm = -INFINITY;
            if (!diag) {
#pragma unroll
                for (int i = 0; i < 32; ++i) pm = fmaxf(pm, fmaxf(__uint_as_float(t0[i]), __uint_as_float(t1[i])));
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    if (c0 + i <= r) pm = fmaxf(pm, __uint_as_float(t0[i]));
                    if (c0 + 32 + i <= r) pm = fmaxf(pm, __uint_as_float(t1[i]));
                }
            }
            xchg[hf * 128 + r] = pm;
            pair_bar_sync(bar_id);
            pm = fmaxf(pm, xchg[(hf ^ 1) * 128 + r]);
            pair_bar_sync(bar_id);  // both have read before either writes again
            const float mx = fmaxf(m, pm * args.scale_log2);  // log2 domain; finite (column 0 <= row)
            const float alpha = ex2_approx(m - mx);           // 0 on the first block (m = -inf)
            m = mx;
            // P = exp2(s*scale - m): one FMA + one special-function op per score.  P is cut to TF32
            // (the low 13 bits dropped, one logic op - exactly what the tensor core would do to it
            // as an operand) BEFORE it is summed, so numerator and denominator use the same
            // weights and the cut only adds noise that the normalisation centres.
            float sum = 0.f;
            const float neg_mx = -mx;
            if (!diag) {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const uint32_t u0 = __float_as_uint(ex2_approx(fmaf(__uint_as_float(t0[i]), args.scale_log2, neg_mx))) & 0xFFFFE000u;
                    const uint32_t u1 = __float_as_uint(ex2_approx(fmaf(__uint_as_float(t1[i]), args.scale_log2, neg_mx))) & 0xFFFFE000u;
                    sum += __uint_as_float(u0) + __uint_as_float(u1);
                    t0[i] = u0;
                    t1[i] = u1;
                }
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    uint32_t u0 = __float_as_uint(ex2_approx(fmaf(__uint_as_float(t0[i]), args.scale_log2, neg_mx))) & 0xFFFFE000u;
                    uint32_t u1 = __float_as_uint(ex2_approx(fmaf(__uint_as_float(t1[i]), args.scale_log2, neg_mx))) & 0xFFFFE000u;
                    if (c0 + i > r) u0 = 0u;
                    if (c0 + 32 + i > r) u1 = 0u;
                    sum += __uint_as_float(u0) + __uint_as_float(u1);
                    t0[i] = u0;
                    t1[i] = u1;
                }
            }
            l = l * alpha + sum;  // this thread's half of the row sum
            // O_{j-1} has retired: its result can be read and the P columns overwritten
            uint32_t o_prev[32];
            if (j > 0) {
                if (ok && !mbar_wait(&o_full[(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag)) ok = false;
                tc_fence_after_sync();
                tmem_ld_32x32b_x32(tmem_base + lane_addr + kOCol + ((j - 1) & 1) * HS + hf * 32, o_prev);
            }
            tmem_st_32x32b_x32(p_addr, t0);
            tmem_st_32x32b_x32(p_addr + 32, t1);
            tmem_st_wait();
            // the next block's scores, while nothing else is using tensor memory
            if (j + 1 < n_kv) {
                const int sn = (j + 1) & 1;
                if (ok && !mbar_wait(&s_full[sn], ((j + 1) >> 1) & 1, abort_flag)) ok = false;
                tc_fence_after_sync();
                const uint32_t s_addr = tmem_base + lane_addr + sn * BKV + hf * 64;
                tmem_ld_32x32b_x32(s_addr, t0);
                tmem_ld_32x32b_x32(s_addr + 32, t1);
            }
            tmem_ld_wait();
            tc_fence_before_sync();
            if (j + 1 < n_kv) mbar_arrive(&s_free[(j + 1) & 1]);
            mbar_arrive(p_full);
            // under the UMMAs of O_j: fold O_{j-1} in
            if (j > 0) {
#pragma unroll
                for (int i = 0; i < 32; ++i) o_acc[i] = o_acc[i] * alpha_prev + __uint_as_float(o_prev[i]);
            }
            alpha_prev = alpha;
        }
        if (ok && !mbar_wait(&o_full[(n_kv - 1) & 1], ((n_kv - 1) >> 1) & 1, abort_flag)) ok = false;
        tc_fence_after_sync();
        accumulate_o(alpha_prev, (n_kv - 1) & 1);
        // combine the two halves of the row sum
        xchg[hf * 128 + r] = l;
        pair_bar_sync(bar_id);
        l += xchg[(hf ^ 1) * 128 + r];
        const int t_idx = q0 + r;
        if (ok && t_idx < args.T) {
            const float inv_l = 1.0f / l;
            float* o = args.out + ((size_t)(row_base + t_idx) * args.C) + h * HS + hf * 32;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float4 v = make_float4(o_acc[4 * i] * inv_l, o_acc[4 * i + 1] * inv_l,
                                       o_acc[4 * i + 2] * inv_l, o_acc[4 * i + 3] * inv_l);
                if (args.round_out) { v.x = round_tf32(v.x); v.y = round_tf32(v.y); v.z = round_tf32(v.z); v.w = round_tf32(v.w); }
                *reinterpret_cast<float4*>(o + 4 * i) = v;
            }
#ifndef B200_ATT_TIMING
            if (args.lse && hf == 0)
                args.lse[((size_t)b * args.NH + h) * args.T + t_idx] = m * 0.6931471805599453f + logf(l);
#endif
        }
        if (!ok && lane == 0) atomicCAS(args.status, 0, DEV_TIMEOUT_SOFTMAX);
    }

    griddep_launch_dependents();
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
#ifdef B200_ATT_TIMING
    if (threadIdx.x == 0 && args.lse) {
        unsigned long long* dbg = reinterpret_cast<unsigned long long*>(args.lse);
        const int idx = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
        unsigned smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        dbg[idx * 4 + 0] = dbg_t_start;
        dbg[idx * 4 + 1] = globaltimer_ns();
        dbg[idx * 4 + 2] = smid;
        dbg[idx * 4 + 3] = n_kv;
    }
#endif
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
    cudaError_t le = launch_pdl(ctx, attention_kernel, grid, dim3(kAttThreads), AttSmem::TOTAL, tm, tmv, a);
    ctx->launches++;
    B200_CUDA(ctx, le);
    return B200_OK;
}

}  // namespace b200
