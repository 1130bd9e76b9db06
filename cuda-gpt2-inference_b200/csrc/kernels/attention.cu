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
// Persistent kernel: one CTA per SM pulls work items - 128 query rows of one (batch, head),
// heaviest first - from a global counter, so tensor memory, barriers and the pipeline are set up
// once and the loads and first UMMAs of the next item run under the tail of the current one.
// 11 warps:
//   warp 0      work fetch + TMA producer: Q (double buffered), then K/V blocks of 128 keys into
//               2-stage rings (separate for K and V: K is free once its S has retired)
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
// numerator.  Every wait is time-bounded (see prim/sm100.cuh).  The work counter lives in the
// context's status area and is put back to zero by the last CTA to finish.
#include <cuda_bf16.h>
#include "kernels.h"
#include "../prim/sm100.cuh"

namespace b200 {

namespace {

constexpr int HS = 64;
constexpr int BQ = 128;
constexpr int BKV = 128;
constexpr int kAttThreads = 352;
constexpr int kBlk = 16384;  // bytes of one {32 fp32 x 128 rows} swizzled block
constexpr int kStages = 2;   // K/V ring
constexpr int kSoftmaxThreads = 256;

struct AttSmem {
    static constexpr int Q_OFF = 0;                           // 2 buffers x 2 blocks (hs 0-31, 32-63)
    static constexpr int K_OFF = Q_OFF + 4 * kBlk;            // kStages x 2 blocks
    static constexpr int V_OFF = K_OFF + 2 * kStages * kBlk;  // kStages x 2 blocks
    static constexpr int OUT_OFF = V_OFF + 2 * kStages * kBlk;  // output staging: 2 blocks (hs 0-31, 32-63)
    static constexpr int X_OFF = OUT_OFF + 2 * kBlk;            // exchange buffer: 2 halves x 128 floats
    static constexpr int BAR_OFF = X_OFF + 2 * 128 * 4;
    static constexpr int TOTAL = 1024 + BAR_OFF + 256;
};
static_assert(AttSmem::TOTAL <= 232448 && AttSmem::TOTAL > 117 * 1024, "one CTA per SM, within 227 KB");
constexpr int kTmemCols = 512;  // S0 [0,128)  S1 [128,256)  P [256,384)  O0 [384,448)  O1 [448,512)
constexpr int kPCol = 256, kOCol = 384;
constexpr int kWorkWord = 60;  // index of the work counter in the context's 64-word status area

// 2^x on the special-function unit (one instruction; 2^-inf = 0)
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// three-input maximum (one instruction on sm_100)
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float y;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
    return y;
}
// barrier among the two warps that share a group of 32 query rows
__device__ __forceinline__ void pair_bar_sync(int id) {
    asm volatile("bar.sync %0, 64;" ::"r"(id) : "memory");
}
// barrier among all 256 softmax threads
__device__ __forceinline__ void softmax_bar_sync() {
    asm volatile("bar.sync 5, 256;" ::: "memory");
}
// the same barrier, returning whether `ok` holds in all 256 threads
__device__ __forceinline__ bool softmax_bar_all(bool ok) {
    uint32_t r;
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        "setp.ne.u32 q, %1, 0;\n\t"
        "bar.red.and.pred p, 5, 256, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(r)
        : "r"((uint32_t)ok)
        : "memory");
    return r != 0;
}

struct AttArgs {
    float* out;
    float* lse;
    int B, T, C, NH;
    int num_qt;
    int num_items;  // num_qt * NH * B
    float scale_log2;
    int round_out;  // store TF32-rounded outputs (they feed only the next GEMM)
    int tma_out;    // T is a multiple of 128: whole tiles leave through shared memory and a TMA store
    int out_bf16;   // 1: out addresses bf16 elements (the next GEMM runs with bf16 operands); 2: two bf16 planes,
                    // bf16(o) and, B*T rows further down, bf16(o - bf16(o)) (split operands of a bf16x3 GEMM)
    int* status;    // [0] error word; [kWorkWord], [kWorkWord+1]: work and finished-CTA counters (zero between launches)
};

// item index -> (query tile, head, batch); heavy (late) query tiles come first
__device__ __forceinline__ void decode_item(const AttArgs& a, int item, int& qt, int& h, int& b) {
    const int hb = a.NH * a.B;
    qt = a.num_qt - 1 - item / hb;
    const int r = item % hb;
    h = r % a.NH;
    b = r / a.NH;
}

__global__ void __launch_bounds__(kAttThreads, 1)
attention_kernel(const __grid_constant__ CUtensorMap tmap_qkv, const __grid_constant__ CUtensorMap tmap_v,
                 const __grid_constant__ CUtensorMap tmap_out, const AttArgs args) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* q_s = smem + AttSmem::Q_OFF;
    uint8_t* k_s = smem + AttSmem::K_OFF;
    uint8_t* v_s = smem + AttSmem::V_OFF;
    uint8_t* out_s = smem + AttSmem::OUT_OFF;
    float* xchg = reinterpret_cast<float*>(smem + AttSmem::X_OFF);  // [2][128]
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + AttSmem::BAR_OFF);
    uint64_t* item_full = bars;        // [2]  work item published
    uint64_t* item_empty = bars + 2;   // [2]  all consumers are done with the item slot
    uint64_t* q_full = bars + 4;       // [2]  TMA: Q landed
    uint64_t* q_empty = bars + 6;      // [2]  every S of the item retired
    uint64_t* k_full = bars + 8;       // [2]  TMA: K block landed
    uint64_t* k_empty = bars + 10;     // [2]  S of the block retired
    uint64_t* v_full = bars + 12;      // [2]  TMA: V block landed
    uint64_t* v_empty = bars + 14;     // [2]  PV of the block retired
    uint64_t* s_full = bars + 16;      // [2]  S computed
    uint64_t* s_free = bars + 18;      // [2]  S read into registers by all softmax threads
    uint64_t* p_full = bars + 20;      // [1]  P written by all softmax threads
    uint64_t* o_full = bars + 21;      // [2]  O_j in tensor memory
    uint64_t* drain_bar = bars + 23;   // [1]
    int* item_slot = reinterpret_cast<int*>(bars + 24);              // [2]
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(item_slot + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < 2; ++s) {
            mbar_init(&item_full[s], 1);
            mbar_init(&item_empty[s], kSoftmaxThreads + 2);  // softmax threads + the two issuers
            mbar_init(&q_full[s], 1);
            mbar_init(&q_empty[s], 1);
            mbar_init(&k_full[s], 1);
            mbar_init(&k_empty[s], 1);
            mbar_init(&v_full[s], 1);
            mbar_init(&v_empty[s], 1);
            mbar_init(&s_full[s], 1);
            mbar_init(&s_free[s], kSoftmaxThreads);
            mbar_init(&o_full[s], 1);
        }
        mbar_init(p_full, kSoftmaxThreads);
        mbar_init(drain_bar, 1);
        *abort_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tmap_qkv);
        tma_prefetch_desc(&tmap_v);
        tma_prefetch_desc(&tmap_out);
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

    // Every role walks the same sequence of items n = 0, 1, ... (slot n & 1) and keeps a running
    // count g of K/V blocks, from which all ring indices and barrier phases follow.
    if (warp == 0) {
        // ------------------------------------------- work fetch + TMA producer
        if (lane == 0) {
            bool ok = true;
            uint32_t g = 0;
            for (uint32_t n = 0; ok; ++n) {
                const int slot = n & 1;
                int item = atomicAdd(args.status + kWorkWord, 1);
                if (item >= args.num_items) item = -1;
                if (!mbar_wait(&item_empty[slot], ((n >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
                item_slot[slot] = item;
                mbar_arrive(&item_full[slot]);  // release: the slot write is visible to the waiters
                if (item < 0) break;
                int qt, h, b;
                decode_item(args, item, qt, h, b);
                const int row_base = b * args.T, q0 = qt * BQ, n_kv = qt + 1;
                const int xq = h * HS, xk = args.C + h * HS, xv = 2 * args.C + h * HS;
                if (!mbar_wait(&q_empty[slot], ((n >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
                mbar_arrive_expect_tx(&q_full[slot], 2 * kBlk);
                tma_load_2d(q_s + (2 * slot) * kBlk, &tmap_qkv, xq, row_base + q0, &q_full[slot]);
                tma_load_2d(q_s + (2 * slot + 1) * kBlk, &tmap_qkv, xq + 32, row_base + q0, &q_full[slot]);
                for (int j = 0; j < n_kv; ++j, ++g) {
                    const int s = g % kStages;
                    const uint32_t ph = ((g / kStages) & 1) ^ 1;
                    const int y = row_base + j * BKV;
                    // K is free again as soon as its S has retired, V only after its PV: separate
                    // rings let the S issuer run two blocks ahead with two stages each
                    if (!mbar_wait(&k_empty[s], ph, abort_flag)) { ok = false; break; }
                    mbar_arrive_expect_tx(&k_full[s], 2 * kBlk);
                    tma_load_2d(k_s + (2 * s) * kBlk, &tmap_qkv, xk, y, &k_full[s]);
                    tma_load_2d(k_s + (2 * s + 1) * kBlk, &tmap_qkv, xk + 32, y, &k_full[s]);
                    if (!mbar_wait(&v_empty[s], ph, abort_flag)) { ok = false; break; }
                    mbar_arrive_expect_tx(&v_full[s], 2 * kBlk);
                    tma_load_2d(v_s + (2 * s) * kBlk, &tmap_v, xv, y, &v_full[s]);
                    tma_load_2d(v_s + (2 * s + 1) * kBlk, &tmap_v, xv + 32, y, &v_full[s]);
                }
            }
            if (!ok) atomicCAS(args.status, 0, DEV_TIMEOUT_PRODUCER);
        }
    } else if (warp == 1) {
        // ------------------------------------------------------- S = Q K^T issuer
        if (lane == 0) {
            constexpr uint32_t idesc_s = make_idesc_tf32(BQ, BKV, 0);  // N = 128 keys
            bool ok = true;
            uint32_t g = 0;
            for (uint32_t n = 0; ok; ++n) {
                const int slot = n & 1;
                if (!mbar_wait(&item_full[slot], (n >> 1) & 1, abort_flag)) { ok = false; break; }
                const int item = item_slot[slot];
                if (item < 0) break;
                int qt, h, b;
                decode_item(args, item, qt, h, b);
                const int n_kv = qt + 1;
                if (!mbar_wait(&q_full[slot], (n >> 1) & 1, abort_flag)) { ok = false; break; }
                for (int j = 0; j < n_kv; ++j, ++g) {
                    const int s = g & 1, ks = g % kStages;
                    if (!mbar_wait(&k_full[ks], (g / kStages) & 1, abort_flag)) { ok = false; break; }
                    // the softmax has read the scores of two blocks ago out of these columns
                    if (!mbar_wait(&s_free[s], ((g >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t d = tmem_base + s * BKV;
#pragma unroll
                    for (int kk = 0; kk < 8; ++kk) {
                        const uint32_t off = (kk >> 2) * kBlk + (kk & 3) * 32;
                        const uint64_t a = make_smem_desc_sw128(smem_u32(q_s + 2 * slot * kBlk) + off, 16, 1024);
                        const uint64_t bd = make_smem_desc_sw128(smem_u32(k_s + 2 * ks * kBlk) + off, 16, 1024);
                        umma_tf32_ss(d, a, bd, idesc_s, kk != 0);
                    }
                    umma_commit(&s_full[s]);
                    umma_commit(&k_empty[ks]);
                }
                umma_commit(&q_empty[slot]);  // Q may be overwritten once these UMMAs have retired
                mbar_arrive(&item_empty[slot]);
            }
            if (!ok) atomicCAS(args.status, 0, DEV_TIMEOUT_MMA);
        }
    } else if (warp == 10) {
        // --------------------------------------------------------- O = P V issuer
        if (lane == 0) {
            constexpr uint32_t idesc_o = make_idesc_tf32(BQ, HS, 1);  // N = 64, V MN-major
            bool ok = true;
            uint32_t g = 0;
            for (uint32_t n = 0; ok; ++n) {
                const int slot = n & 1;
                if (!mbar_wait(&item_full[slot], (n >> 1) & 1, abort_flag)) { ok = false; break; }
                const int item = item_slot[slot];
                if (item < 0) break;
                int qt, h, b;
                decode_item(args, item, qt, h, b);
                const int n_kv = qt + 1;
                for (int j = 0; j < n_kv; ++j, ++g) {
                    const int s = g & 1, ks3 = g % kStages;
                    if (!mbar_wait(&v_full[ks3], (g / kStages) & 1, abort_flag)) { ok = false; break; }
                    if (!mbar_wait(p_full, g & 1, abort_flag)) { ok = false; break; }
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
                    umma_commit(&v_empty[ks3]);
                }
                mbar_arrive(&item_empty[slot]);
            }
            // everything issued by both issuers has retired once this commit arrives (the last PV
            // depends on the last S through the softmax)
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
        const uint32_t p_addr = tmem_base + lane_addr + kPCol + hf * 64;
        const int c0 = hf * 64;                  // first key column of this thread within a block
        bool ok = true;
        uint32_t g = 0;
        // All softmax warps leave together: the decision is taken once per item, on a barrier
        // that also tells whether any of the 256 threads has had a wait run out.  Inside an item
        // there is no early exit: after a failed wait the remaining waits are skipped but every
        // barrier is still executed, so no warp can be left alone in one (the results are
        // discarded and the status word says why).
        for (uint32_t n = 0;; ++n) {
            const int slot = n & 1;
            if (ok && !mbar_wait(&item_full[slot], (n >> 1) & 1, abort_flag)) ok = false;
            const bool all_ok = softmax_bar_all(ok);
            const int item = all_ok ? item_slot[slot] : -1;
            if (item < 0) break;
            int qt, h, b;
            decode_item(args, item, qt, h, b);
            const int n_kv = qt + 1, q0 = qt * BQ, row_base = b * args.T;
            float m = -INFINITY, l = 0.f, alpha_prev = 0.f;
            float o_acc[HS / 2];
#pragma unroll
            for (int i = 0; i < HS / 2; ++i) o_acc[i] = 0.f;

            // Every tensor-memory read of an iteration is done before p_full is signalled, i.e.
            // while the tensor core is not running O = P V (whose P operand also comes out of
            // tensor memory); the arithmetic on the values runs under the UMMAs.
            uint32_t t0[32], t1[32];  // this thread's 64 scores of the current block, then its P
            if (ok && !mbar_wait(&s_full[g & 1], (g >> 1) & 1, abort_flag)) ok = false;
            tc_fence_after_sync();
            {
                const uint32_t s_addr = tmem_base + lane_addr + (g & 1) * BKV + hf * 64;
                tmem_ld_32x32b_x32(s_addr, t0);
                tmem_ld_32x32b_x32(s_addr + 32, t1);
                tmem_ld_wait();
                tc_fence_before_sync();
                mbar_arrive(&s_free[g & 1]);
            }
            for (int j = 0; j < n_kv; ++j, ++g) {
                const bool diag = (j == n_kv - 1);
                // row maximum of the raw scores (the scale is positive, so it commutes with max)
                // (four independent chains of three-input maxima: the loop is latency-bound)
                float pm0 = -INFINITY, pm1 = -INFINITY, pm2 = -INFINITY, pm3 = -INFINITY;
                if (!diag) {
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        pm0 = fmax3(pm0, __uint_as_float(t0[i]), __uint_as_float(t0[i + 1]));
                        pm1 = fmax3(pm1, __uint_as_float(t0[i + 2]), __uint_as_float(t0[i + 3]));
                        pm2 = fmax3(pm2, __uint_as_float(t1[i]), __uint_as_float(t1[i + 1]));
                        pm3 = fmax3(pm3, __uint_as_float(t1[i + 2]), __uint_as_float(t1[i + 3]));
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        pm0 = fmax3(pm0, c0 + i <= r ? __uint_as_float(t0[i]) : -INFINITY, c0 + i + 1 <= r ? __uint_as_float(t0[i + 1]) : -INFINITY);
                        pm1 = fmax3(pm1, c0 + i + 2 <= r ? __uint_as_float(t0[i + 2]) : -INFINITY, c0 + i + 3 <= r ? __uint_as_float(t0[i + 3]) : -INFINITY);
                        pm2 = fmax3(pm2, c0 + 32 + i <= r ? __uint_as_float(t1[i]) : -INFINITY, c0 + 32 + i + 1 <= r ? __uint_as_float(t1[i + 1]) : -INFINITY);
                        pm3 = fmax3(pm3, c0 + 32 + i + 2 <= r ? __uint_as_float(t1[i + 2]) : -INFINITY, c0 + 32 + i + 3 <= r ? __uint_as_float(t1[i + 3]) : -INFINITY);
                    }
                }
                float pm = fmaxf(fmaxf(pm0, pm1), fmaxf(pm2, pm3));
                xchg[hf * 128 + r] = pm;
                pair_bar_sync(bar_id);
                pm = fmaxf(pm, xchg[(hf ^ 1) * 128 + r]);
                pair_bar_sync(bar_id);  // both have read before either writes again
                const float mx = fmaxf(m, pm * args.scale_log2);  // log2 domain; finite (column 0 <= row)
                const float alpha = ex2_approx(m - mx);           // 0 on the first block (m = -inf)
                m = mx;
                // P = exp2(s*scale - m): one FMA + one special-function op per score.  P is cut to
                // TF32 (the low 13 bits dropped, one logic op - exactly what the tensor core would
                // do to it as an operand) BEFORE it is summed, so numerator and denominator use the
                // same weights and the cut only adds noise that the normalisation centres.
                float sum0 = 0.f, sum1 = 0.f, sum2 = 0.f, sum3 = 0.f;
                const float neg_mx = -mx;
                if (!diag) {
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const uint32_t u0 = __float_as_uint(ex2_approx(fmaf(__uint_as_float(t0[i]), args.scale_log2, neg_mx))) & 0xFFFFE000u;
                        const uint32_t u1 = __float_as_uint(ex2_approx(fmaf(__uint_as_float(t1[i]), args.scale_log2, neg_mx))) & 0xFFFFE000u;
                        const uint32_t u2 = __float_as_uint(ex2_approx(fmaf(__uint_as_float(t0[i + 1]), args.scale_log2, neg_mx))) & 0xFFFFE000u;
                        const uint32_t u3 = __float_as_uint(ex2_approx(fmaf(__uint_as_float(t1[i + 1]), args.scale_log2, neg_mx))) & 0xFFFFE000u;
                        sum0 += __uint_as_float(u0);
                        sum1 += __uint_as_float(u1);
                        sum2 += __uint_as_float(u2);
                        sum3 += __uint_as_float(u3);
                        t0[i] = u0;
                        t1[i] = u1;
                        t0[i + 1] = u2;
                        t1[i + 1] = u3;
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        uint32_t u0 = __float_as_uint(ex2_approx(fmaf(__uint_as_float(t0[i]), args.scale_log2, neg_mx))) & 0xFFFFE000u;
                        uint32_t u1 = __float_as_uint(ex2_approx(fmaf(__uint_as_float(t1[i]), args.scale_log2, neg_mx))) & 0xFFFFE000u;
                        uint32_t u2 = __float_as_uint(ex2_approx(fmaf(__uint_as_float(t0[i + 1]), args.scale_log2, neg_mx))) & 0xFFFFE000u;
                        uint32_t u3 = __float_as_uint(ex2_approx(fmaf(__uint_as_float(t1[i + 1]), args.scale_log2, neg_mx))) & 0xFFFFE000u;
                        if (c0 + i > r) u0 = 0u;
                        if (c0 + 32 + i > r) u1 = 0u;
                        if (c0 + i + 1 > r) u2 = 0u;
                        if (c0 + 32 + i + 1 > r) u3 = 0u;
                        sum0 += __uint_as_float(u0);
                        sum1 += __uint_as_float(u1);
                        sum2 += __uint_as_float(u2);
                        sum3 += __uint_as_float(u3);
                        t0[i] = u0;
                        t1[i] = u1;
                        t0[i + 1] = u2;
                        t1[i + 1] = u3;
                    }
                }
                l = l * alpha + ((sum0 + sum1) + (sum2 + sum3));  // this thread's half of the row sum
                // O_{j-1} has retired: its result can be read and the P columns overwritten
                uint32_t o_prev[32];
                if (j > 0) {
                    if (ok && !mbar_wait(&o_full[(g - 1) & 1], ((g - 1) >> 1) & 1, abort_flag)) ok = false;
                    tc_fence_after_sync();
                    tmem_ld_32x32b_x32(tmem_base + lane_addr + kOCol + ((g - 1) & 1) * HS + hf * 32, o_prev);
                }
                tmem_st_32x32b_x32(p_addr, t0);
                tmem_st_32x32b_x32(p_addr + 32, t1);
                tmem_st_wait();
                // the next block's scores, while nothing else is using tensor memory
                if (j + 1 < n_kv) {
                    const int sn = (g + 1) & 1;
                    if (ok && !mbar_wait(&s_full[sn], ((g + 1) >> 1) & 1, abort_flag)) ok = false;
                    tc_fence_after_sync();
                    const uint32_t s_addr = tmem_base + lane_addr + sn * BKV + hf * 64;
                    tmem_ld_32x32b_x32(s_addr, t0);
                    tmem_ld_32x32b_x32(s_addr + 32, t1);
                }
                tmem_ld_wait();
                tc_fence_before_sync();
                if (j + 1 < n_kv) mbar_arrive(&s_free[(g + 1) & 1]);
                mbar_arrive(p_full);
                // under the UMMAs of O_j: fold O_{j-1} in
                if (j > 0) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) o_acc[i] = o_acc[i] * alpha_prev + __uint_as_float(o_prev[i]);
                }
                alpha_prev = alpha;
            }
            // the last block of the item (g has moved past it)
            if (ok && !mbar_wait(&o_full[(g - 1) & 1], ((g - 1) >> 1) & 1, abort_flag)) ok = false;
            tc_fence_after_sync();
            {
                uint32_t t[32];
                tmem_ld_32x32b_x32(tmem_base + lane_addr + kOCol + ((g - 1) & 1) * HS + hf * 32, t);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) o_acc[i] = o_acc[i] * alpha_prev + __uint_as_float(t[i]);
            }
            // combine the two halves of the row sum
            xchg[hf * 128 + r] = l;
            pair_bar_sync(bar_id);
            l += xchg[(hf ^ 1) * 128 + r];
            pair_bar_sync(bar_id);
            const int t_idx = q0 + r;
            const float inv_l = 1.0f / l;
            if (args.tma_out) {
                // Whole tile: each thread puts its 32 columns (one 128-byte row of block hf) into
                // the staging buffer in the 128-byte-swizzled layout, and one thread sends the two
                // blocks off with TMA stores - full-line writes instead of 16-byte pieces of 32
                // different rows per instruction.
                if (threadIdx.x == 64) tma_store_wait_read();  // the previous tile has left the buffer
                softmax_bar_sync();
                if (args.out_bf16) {
                    // 64 bf16 columns are one 128-byte row: this thread's 32 columns are chunks
                    // 4*hf .. 4*hf+3 of row r, and the tile leaves as one {128 x 64} store (two with
                    // split outputs: the dropped parts are staged in the second block)
                    uint4* rowh = reinterpret_cast<uint4*>(out_s + r * 128);
                    uint4* rowl = reinterpret_cast<uint4*>(out_s + kBlk + r * 128);
                    const bool planes = args.out_bf16 == 2;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint32_t ph[4], pl[4];
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const float a = o_acc[8 * i + 2 * k] * inv_l, b2 = o_acc[8 * i + 2 * k + 1] * inv_l;
                            const __nv_bfloat162 hh = __floats2bfloat162_rn(a, b2);
                            const __nv_bfloat162 ll = __floats2bfloat162_rn(a - __low2float(hh), b2 - __high2float(hh));
                            ph[k] = *reinterpret_cast<const uint32_t*>(&hh);
                            pl[k] = *reinterpret_cast<const uint32_t*>(&ll);
                        }
                        rowh[(hf * 4 + i) ^ (r & 7)] = make_uint4(ph[0], ph[1], ph[2], ph[3]);
                        if (planes) rowl[(hf * 4 + i) ^ (r & 7)] = make_uint4(pl[0], pl[1], pl[2], pl[3]);
                    }
                    fence_proxy_async_smem();
                    softmax_bar_sync();
                    if (threadIdx.x == 64 && ok) {
                        tma_store_2d(&tmap_out, h * HS, row_base + q0, out_s);
                        if (planes) tma_store_2d(&tmap_out, h * HS, args.B * args.T + row_base + q0, out_s + kBlk);
                        tma_store_commit();
                    }
                } else {
                float4* row = reinterpret_cast<float4*>(out_s + hf * kBlk + r * 128);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    float4 v = make_float4(o_acc[4 * i] * inv_l, o_acc[4 * i + 1] * inv_l,
                                           o_acc[4 * i + 2] * inv_l, o_acc[4 * i + 3] * inv_l);
                    if (args.round_out) { v.x = round_tf32(v.x); v.y = round_tf32(v.y); v.z = round_tf32(v.z); v.w = round_tf32(v.w); }
                    row[i ^ (r & 7)] = v;
                }
                fence_proxy_async_smem();
                softmax_bar_sync();
                if (threadIdx.x == 64 && ok) {
                    tma_store_2d(&tmap_out, h * HS, row_base + q0, out_s);
                    tma_store_2d(&tmap_out, h * HS + 32, row_base + q0, out_s + kBlk);
                    tma_store_commit();
                }
                }
            } else if (ok && t_idx < args.T && args.out_bf16) {
                uint16_t* oh = reinterpret_cast<uint16_t*>(args.out) + ((size_t)(row_base + t_idx) * args.C) + h * HS + hf * 32;
                uint4* o = reinterpret_cast<uint4*>(oh);
                uint4* o2 = reinterpret_cast<uint4*>(oh + (size_t)args.B * args.T * args.C);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint32_t ph[4], pl[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const float a = o_acc[8 * i + 2 * k] * inv_l, b2 = o_acc[8 * i + 2 * k + 1] * inv_l;
                        const __nv_bfloat162 hh = __floats2bfloat162_rn(a, b2);
                        const __nv_bfloat162 ll = __floats2bfloat162_rn(a - __low2float(hh), b2 - __high2float(hh));
                        ph[k] = *reinterpret_cast<const uint32_t*>(&hh);
                        pl[k] = *reinterpret_cast<const uint32_t*>(&ll);
                    }
                    o[i] = make_uint4(ph[0], ph[1], ph[2], ph[3]);
                    if (args.out_bf16 == 2) o2[i] = make_uint4(pl[0], pl[1], pl[2], pl[3]);
                }
            } else if (ok && t_idx < args.T) {
                float* o = args.out + ((size_t)(row_base + t_idx) * args.C) + h * HS + hf * 32;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    float4 v = make_float4(o_acc[4 * i] * inv_l, o_acc[4 * i + 1] * inv_l,
                                           o_acc[4 * i + 2] * inv_l, o_acc[4 * i + 3] * inv_l);
                    if (args.round_out) { v.x = round_tf32(v.x); v.y = round_tf32(v.y); v.z = round_tf32(v.z); v.w = round_tf32(v.w); }
                    *reinterpret_cast<float4*>(o + 4 * i) = v;
                }
            }
            if (ok && t_idx < args.T && args.lse && hf == 0)
                args.lse[((size_t)b * args.NH + h) * args.T + t_idx] = m * 0.6931471805599453f + logf(l);
            tc_fence_before_sync();
            mbar_arrive(&item_empty[slot]);
        }
        if (threadIdx.x == 64) tma_store_wait_all();
        if (!ok && lane == 0) atomicCAS(args.status, 0, DEV_TIMEOUT_SOFTMAX);
    }

    griddep_launch_dependents();
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
    // the last CTA to finish puts the work counters back to zero for the next launch
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(args.status + kWorkWord + 1, 1) == (int)gridDim.x - 1) {
            args.status[kWorkWord] = 0;
            args.status[kWorkWord + 1] = 0;
            __threadfence();
        }
    }
}

}  // namespace

int preload_attention_kernel(b200_ctx* ctx) {
    B200_CUDA(ctx, cudaFuncSetAttribute(attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AttSmem::TOTAL));
    return B200_OK;
}

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
    a.tma_out = (T % BQ == 0) ? 1 : 0;
    CUtensorMap tmo = tm;  // not used unless whole tiles are stored
    a.out_bf16 = (flags & OUT_BF16X2) ? 2 : ((flags & OUT_BF16) ? 1 : 0);
    if (a.tma_out) {
        if (a.out_bf16) st = b200_get_tensor_map_bf16(ctx, &tmo, out, (uint64_t)B * T * a.out_bf16, (uint64_t)C, (uint64_t)C, BQ, 64);
        else st = b200_get_tensor_map(ctx, &tmo, out, (uint64_t)B * T, (uint64_t)C, (uint64_t)C, BQ, 32);
        if (st != B200_OK) return st;
    }
    a.out = out; a.lse = lse; a.B = B; a.T = T; a.C = C; a.NH = NH;
    a.num_qt = (T + BQ - 1) / BQ;
    a.num_items = a.num_qt * NH * B;
    a.scale_log2 = 1.4426950408889634f / sqrtf((float)HS);
    a.round_out = (flags & ROUND_OUT_TF32) ? 1 : 0;
    a.status = ctx->d_status;
    const int grid = a.num_items < ctx->num_sms ? a.num_items : ctx->num_sms;
    cudaError_t le = launch_pdl(ctx, attention_kernel, dim3(grid), dim3(kAttThreads), AttSmem::TOTAL, tm, tmv, tmo, a);
    ctx->launches++;
    B200_CUDA(ctx, le);
    return B200_OK;
}

}  // namespace b200
