// Causal multi-head attention on fp16 operands (the attention of the B200_BF16X3 mode):
//   out[b,t,h,:] = softmax_{j<=t}(q_t . k_j / sqrt(HS)) V        (HS = 64)
// the same math as attention.cu (reference: kernels/attention/3_flash_attention_permute.cuh:
// 46-58,149-153,216-221,306,342).  Q, K and V arrive the way the QKV GEMM of that mode writes
// them: two fp16 planes of the packed buffer [B,T,3,NH,HS], value = hi + lo (22 significant bits).
// The products are kind::f16 UMMAs:
//     S = Q K^T ~ Qhi.Khi                    O = P V ~ P.Vhi + P.Vlo
// fp16 keeps 11 significant bits, round to nearest - what the single-pass TF32 kernel has on its
// rounded q and k, so the scores need one product (measured on the GPT-2 forward: that part of
// the error is 2e-5 of the 1.1e-4 rms the TF32 kernel leaves in the logits).  What dominated
// there was P.V with V cut to 11 bits and P truncated; here V enters with both terms and P is
// rounded to nearest fp16 by the softmax threads and written as packed pairs into tensor memory
// (two keys per 32-bit column), from where the second product reads it as its A operand.
// V is an MN-major operand; for 16-bit elements that is the ordinary 128-byte swizzle (rows of 64
// values, 8-row atoms), so one tensor map serves every tile.
// The two operands of a kind::f16 UMMA must have the same format: fp16 P with bf16 V is an illegal
// instruction, which is why the QKV GEMM writes fp16 planes for this kernel.
//
// Work distribution.  A work item is a PAIR of neighbouring query tiles (2 x 128 rows) of one
// (batch, head); the CTA runs one pipeline per tile of the pair, and the two pipelines share
// every K and V block that the producer loads (tile 2p needs blocks 0..2p, tile 2p+1 one more).
// Measured on the one-tile-per-CTA version of this kernel: its time was neither the tensor pipe
// (18 %) nor the special-function pipe (38 %) but the fact that all softmax warps are in the
// same phase at the same time - row maximum, exponentials, tensor-memory traffic, waits -
// so each unit idles while the others work.  Two independent tiles per CTA fall out of step by
// themselves, and one's exponentials run under the other's waits and UMMAs.
//
// A query row is one thread (no exchange between threads inside the loop): 128 scores are read
// from tensor memory into registers, reduced to the block maximum, turned into P and written
// back as fp16 pairs.  O stays in tensor memory and accumulates over the blocks (the UMMAs add
// to it); the reference maximum of a row is only moved - and O and the row sum rescaled - when
// a block raises it by more than 2^8, so P never exceeds 256 (far inside fp16's range) and the
// rescale, which needs a round trip of O through registers, is rare after the first blocks.
//
// Persistent kernel, 11 warps: warp 0 work fetch + TMA producer (Q pair double buffered, K and
// V blocks of 128 keys in separate 2-stage rings), warps 1 and 2 the UMMA issuers of pipeline 0
// and 1 (warp 1 also owns the tensor memory), warps 3-6 and 7-10 the softmax threads of
// pipeline 0 and 1.  Every wait is time-bounded (prim/sm100.cuh); the work counter lives in the
// context's status area and is put back to zero by the last CTA to finish.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "kernels.h"
#include "../prim/sm100.cuh"

namespace b200 {

namespace {

constexpr int HS = 64;
constexpr int BQ = 128;
constexpr int BKV = 128;
constexpr int kAttThreads = 352;
constexpr int kBlk = 16384;  // bytes of one {64 fp16 x 128 rows} swizzled tile (one plane of Q, K or V)
constexpr int kStages = 2;   // K/V ring
constexpr int kPipeThreads = 128;  // softmax threads of one pipeline (one per query row)

struct AttSmem {
    static constexpr int Q_OFF = 0;                              // 2 slots x 2 tiles (hi plane of each tile of the pair)
    static constexpr int K_OFF = Q_OFF + 4 * kBlk;               // kStages x 1 tile (hi plane)
    static constexpr int V_OFF = K_OFF + kStages * kBlk;         // kStages x 2 tiles (hi plane, lo plane)
    static constexpr int OUT_OFF = V_OFF + 2 * kStages * kBlk;   // output staging: 2 pipelines x 2 blocks
    static constexpr int BAR_OFF = OUT_OFF + 4 * kBlk;
    static constexpr int TOTAL = 1024 + BAR_OFF + 512;
};
static_assert(AttSmem::TOTAL <= 232448 && AttSmem::TOTAL > 117 * 1024, "one CTA per SM, within 227 KB");
// tensor memory, per pipeline x (256 columns): S [0,128)  P [128,192) (fp16 pairs)  O [192,256)
constexpr int kTmemCols = 512;
constexpr int kPipeCols = 256, kPCol = 128, kOCol = 192;
constexpr int kWorkWord = 58;  // index of the work counter in the context's 64-word status area
constexpr float kRescaleStep = 8.0f;  // log2 of the largest P before the reference maximum moves

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
// barrier among the 128 softmax threads of one pipeline (id 1 or 2)
__device__ __forceinline__ void pipe_bar_sync(int id) {
    asm volatile("bar.sync %0, 128;" ::"r"(id) : "memory");
}
// the same barrier, returning whether `ok` holds in all 128 threads
__device__ __forceinline__ bool pipe_bar_all(int id, bool ok) {
    uint32_t r;
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        "setp.ne.u32 q, %2, 0;\n\t"
        "bar.red.and.pred p, %1, 128, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(r)
        : "r"(id), "r"((uint32_t)ok)
        : "memory");
    return r != 0;
}

struct AttArgs {
    float* out;
    float* lse;
    int B, T, C, NH;
    int plane_rows;  // B*T: the lo plane of the packed buffer starts this many rows below the hi plane
    int num_qt;      // query tiles of 128 rows
    int num_pairs;   // ceil(num_qt / 2)
    int num_items;   // num_pairs * NH * B
    float scale_log2;
    int round_out;  // store TF32-rounded outputs (they feed only the next GEMM)
    int tma_out;    // T is a multiple of 128: whole tiles leave through shared memory and a TMA store
    int out_bf16;   // 1: out addresses bf16 elements (the next GEMM runs with bf16 operands); 2: two bf16 planes,
                    // bf16(o) and, B*T rows further down, bf16(o - bf16(o)) (split operands of a bf16x3 GEMM)
    int* status;    // [0] error word; [kWorkWord], [kWorkWord+1]: work and finished-CTA counters (zero between launches)
};

// item index -> (tile pair, head, batch); heavy (late) pairs come first
__device__ __forceinline__ void decode_item(const AttArgs& a, int item, int& pair, int& h, int& b) {
    const int hb = a.NH * a.B;
    pair = a.num_pairs - 1 - item / hb;
    const int r = item % hb;
    h = r % a.NH;
    b = r / a.NH;
}
// number of key blocks pipeline x works through for a pair (0: the pair has no second tile)
__device__ __forceinline__ int pipe_blocks(const AttArgs& a, int pair, int x) {
    const int qt = 2 * pair + x;
    return qt < a.num_qt ? qt + 1 : 0;
}

__global__ void __launch_bounds__(kAttThreads, 1)
attention_split_kernel(const __grid_constant__ CUtensorMap tmap_qkv, const __grid_constant__ CUtensorMap tmap_out, const AttArgs args) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* q_s = smem + AttSmem::Q_OFF;
    uint8_t* k_s = smem + AttSmem::K_OFF;
    uint8_t* v_s = smem + AttSmem::V_OFF;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + AttSmem::BAR_OFF);
    uint64_t* item_full = bars;        // [2]  work item published
    uint64_t* item_empty = bars + 2;   // [2]  all consumers are done with the item slot
    uint64_t* q_full = bars + 4;       // [2]  TMA: the Q tiles of the pair landed
    uint64_t* q_empty = bars + 6;      // [2]  every S of the item retired (both pipelines)
    uint64_t* k_full = bars + 8;       // [2]  TMA: K block landed
    uint64_t* k_empty = bars + 10;     // [2]  S of the block retired in both pipelines
    uint64_t* v_full = bars + 12;      // [2]  TMA: V block landed
    uint64_t* v_empty = bars + 14;     // [2]  PV of the block retired in both pipelines
    uint64_t* s_full = bars + 16;      // [pipeline]  S computed
    uint64_t* s_free = bars + 18;      // [pipeline]  S read into registers by all threads of the pipeline
    uint64_t* p_full = bars + 20;      // [pipeline]  P written (and O rescaled if needed)
    uint64_t* o_full = bars + 22;      // [pipeline]  P V of a block retired: O updated, P free
    uint64_t* drain_bar = bars + 24;   // [pipeline]
    int* item_slot = reinterpret_cast<int*>(bars + 26);              // [2]
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(item_slot + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < 2; ++s) {
            mbar_init(&item_full[s], 1);
            mbar_init(&item_empty[s], 2 * kPipeThreads + 2);  // softmax threads + the two issuers
            mbar_init(&q_full[s], 1);
            mbar_init(&q_empty[s], 2);
            mbar_init(&k_full[s], 1);
            mbar_init(&k_empty[s], 2);
            mbar_init(&v_full[s], 1);
            mbar_init(&v_empty[s], 2);
            mbar_init(&s_full[s], 1);
            mbar_init(&s_free[s], kPipeThreads);
            mbar_init(&p_full[s], kPipeThreads);
            mbar_init(&o_full[s], 1);
            mbar_init(&drain_bar[s], 1);
        }
        *abort_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tmap_qkv);
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

    // Every role walks the same sequence of items n = 0, 1, ... (slot n & 1).  The K/V ring is
    // indexed by a running count of the blocks the producer loads (per item: as many as the
    // longer pipeline needs); each pipeline keeps its own running count of the blocks it works
    // through, from which the phases of its own barriers follow.
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
                int pair, h, b;
                decode_item(args, item, pair, h, b);
                const int n1 = pipe_blocks(args, pair, 1);
                const int n_item = n1 > 0 ? n1 : pipe_blocks(args, pair, 0);
                const int row_base = b * args.T, q0 = 2 * pair * BQ;
                const int xq = h * HS, xk = args.C + h * HS, xv = 2 * args.C + h * HS;
                if (!mbar_wait(&q_empty[slot], ((n >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
                mbar_arrive_expect_tx(&q_full[slot], n1 > 0 ? 2 * kBlk : kBlk);
                tma_load_2d(q_s + (2 * slot) * kBlk, &tmap_qkv, xq, row_base + q0, &q_full[slot]);
                if (n1 > 0) tma_load_2d(q_s + (2 * slot + 1) * kBlk, &tmap_qkv, xq, row_base + q0 + BQ, &q_full[slot]);
                // K runs one block ahead of V: K_{j+1} is wanted a whole block earlier than V_j (the
                // scores of block j+1 are computed while the softmax threads work on block j), and
                // its stage is free as soon as S_{j-1} has retired, V_j's only after P V of block j-2
                for (int j = -1; j < n_item && ok; ++j) {
                    if (j + 1 < n_item) {
                        const uint32_t gk = g + j + 1;
                        const int s = gk % kStages;
                        if (!mbar_wait(&k_empty[s], ((gk / kStages) & 1) ^ 1, abort_flag)) { ok = false; break; }
                        mbar_arrive_expect_tx(&k_full[s], kBlk);
                        tma_load_2d(k_s + s * kBlk, &tmap_qkv, xk, row_base + (j + 1) * BKV, &k_full[s]);
                    }
                    if (j >= 0) {
                        const uint32_t gv = g + j;
                        const int s = gv % kStages;
                        const int y = row_base + j * BKV;
                        if (!mbar_wait(&v_empty[s], ((gv / kStages) & 1) ^ 1, abort_flag)) { ok = false; break; }
                        mbar_arrive_expect_tx(&v_full[s], 2 * kBlk);
                        tma_load_2d(v_s + (2 * s) * kBlk, &tmap_qkv, xv, y, &v_full[s]);
                        tma_load_2d(v_s + (2 * s + 1) * kBlk, &tmap_qkv, xv, args.plane_rows + y, &v_full[s]);
                    }
                }
                g += n_item;
            }
            if (!ok) atomicCAS(args.status, 0, DEV_TIMEOUT_PRODUCER);
        }
    } else if (warp <= 2) {
        // ------------------------------------- UMMA issuer of pipeline x: S = Q K^T and O += P V
        // Order of issue per block j: S_{j+1} (as soon as the softmax threads have taken S_j into
        // registers), then P_j V_j (when P_j is written) - so the next scores are ready long
        // before the softmax threads come back for them.
        // A barrier that counts one arrival per pipeline (q_empty, k_empty, v_empty) is only
        // arrived on after the matching "full" barrier of the same use has been seen: that orders
        // the arrival behind the completion of the barrier's previous phase also for a pipeline
        // that has no use for the block (the shorter tile of the pair, or a pair without a
        // second tile).
        if (lane == 0) {
            const int x = warp - 1;
            constexpr uint32_t idesc_s = make_idesc_f16(BQ, BKV, 0);  // N = 128 keys
            constexpr uint32_t idesc_o = make_idesc_f16(BQ, HS, 1);   // N = 64, V MN-major
            const uint32_t tm = tmem_base + x * kPipeCols;
            bool ok = true;
            uint32_t g0 = 0;  // blocks loaded before this item (ring position)
            uint32_t gx = 0;  // blocks of this pipeline before this item
            for (uint32_t n = 0; ok; ++n) {
                const int slot = n & 1;
                if (!mbar_wait(&item_full[slot], (n >> 1) & 1, abort_flag)) { ok = false; break; }
                const int item = item_slot[slot];
                if (item < 0) break;
                int pair, h, b;
                decode_item(args, item, pair, h, b);
                const int n1 = pipe_blocks(args, pair, 1);
                const int n_item = n1 > 0 ? n1 : pipe_blocks(args, pair, 0);
                const int n_kv = pipe_blocks(args, pair, x);
                if (!mbar_wait(&q_full[slot], (n >> 1) & 1, abort_flag)) { ok = false; break; }
                if (n_kv == 0) mbar_arrive(&q_empty[slot]);
                const uint32_t q_addr = smem_u32(q_s + (2 * slot + x) * kBlk);
                // j walks the blocks of the item; S of block j and P V of block j-1 per step
                for (int j = 0; j <= n_item && ok; ++j) {
                    if (j < n_item) {
                        const uint32_t g = g0 + j;
                        const int ks = g % kStages;
                        if (!mbar_wait(&k_full[ks], (g / kStages) & 1, abort_flag)) { ok = false; break; }
                        if (j < n_kv) {
                            // the softmax threads have read the previous scores out of these columns
                            if (!mbar_wait(&s_free[x], ((gx + j) & 1) ^ 1, abort_flag)) { ok = false; break; }
                            tc_fence_after_sync();
#pragma unroll
                            for (int kk = 0; kk < 4; ++kk) {  // 16 of the 64 head dimensions (32 bytes of the swizzled row) per instruction
                                const uint64_t qh = make_smem_desc_sw128(q_addr + kk * 32, 16, 1024);
                                const uint64_t kh = make_smem_desc_sw128(smem_u32(k_s + ks * kBlk) + kk * 32, 16, 1024);
                                umma_f16_ss(tm, qh, kh, idesc_s, kk != 0);
                            }
                            umma_commit(&s_full[x]);
                            umma_commit(&k_empty[ks]);
                            if (j == n_kv - 1) umma_commit(&q_empty[slot]);  // Q may be overwritten once these UMMAs have retired
                        } else {
                            mbar_arrive(&k_empty[ks]);
                        }
                    }
                    if (j > 0) {
                        const int i = j - 1;
                        const uint32_t g = g0 + i;
                        const int vs = g % kStages;
                        if (!mbar_wait(&v_full[vs], (g / kStages) & 1, abort_flag)) { ok = false; break; }
                        if (i < n_kv) {
                            if (!mbar_wait(&p_full[x], (gx + i) & 1, abort_flag)) { ok = false; break; }
                            tc_fence_after_sync();
#pragma unroll
                            for (int ks = 0; ks < BKV / 16; ++ks) {
                                // A: P in tensor memory, 16 keys = 8 columns of packed pairs per instruction
                                const uint32_t pa = tm + kPCol + ks * 8;
                                // B: V, MN-major: 16 keys = 16 rows of 128 bytes = two 8-row swizzle atoms 1024 bytes apart
                                const uint64_t vh = make_smem_desc_sw128(smem_u32(v_s + 2 * vs * kBlk) + ks * 2048, 16, 1024);
                                const uint64_t vl = make_smem_desc_sw128(smem_u32(v_s + (2 * vs + 1) * kBlk) + ks * 2048, 16, 1024);
                                umma_f16_ts(tm + kOCol, pa, vh, idesc_o, (i | ks) != 0);  // the first block of an item starts O afresh
                                umma_f16_ts(tm + kOCol, pa, vl, idesc_o, 1);
                            }
                            umma_commit(&o_full[x]);
                            umma_commit(&v_empty[vs]);
                        } else {
                            mbar_arrive(&v_empty[vs]);
                        }
                    }
                }
                g0 += n_item;
                gx += n_kv;
                mbar_arrive(&item_empty[slot]);
            }
            // everything this issuer has issued has retired once this commit arrives
            umma_commit(&drain_bar[x]);
            if (!mbar_wait(&drain_bar[x], 0, abort_flag)) ok = false;
            if (!ok) atomicCAS(args.status, 0, DEV_TIMEOUT_MMA);
        }
    } else {
        // ----------------------------------------------------------------- softmax
        const int x = (warp - 3) >> 2;           // pipeline = tile of the pair
        const int qd = warp & 3;                 // tensor-memory lane quarter of this warp
        const int r = qd * 32 + lane;            // query row inside the tile = tensor-memory lane
        const uint32_t tm = tmem_base + (uint32_t(qd * 32) << 16) + x * kPipeCols;
        const int bar_id = 1 + x;
        const bool leader = (threadIdx.x == 96 + x * kPipeThreads);  // issues the pipeline's TMA stores
        uint8_t* out_s = smem + AttSmem::OUT_OFF + x * 2 * kBlk;
        bool ok = true;
        uint32_t gx = 0;  // blocks of this pipeline before this item
        // The threads of a pipeline leave together: the decision is taken once per item, on a
        // barrier that also tells whether any of them has had a wait run out.  Inside an item there
        // is no early exit: after a failed wait the remaining waits are skipped but every barrier
        // is still executed, so no warp can be left alone in one (the results are discarded and
        // the status word says why).
        for (uint32_t n = 0;; ++n) {
            const int slot = n & 1;
            if (ok && !mbar_wait(&item_full[slot], (n >> 1) & 1, abort_flag)) ok = false;
            const bool all_ok = pipe_bar_all(bar_id, ok);
            const int item = all_ok ? item_slot[slot] : -1;
            if (item < 0) break;
            int pair, h, b;
            decode_item(args, item, pair, h, b);
            const int n_kv = pipe_blocks(args, pair, x);
            if (n_kv == 0) {  // the pair has no second tile
                mbar_arrive(&item_empty[slot]);
                continue;
            }
            const int q0 = (2 * pair + x) * BQ, row_base = b * args.T;
            float m_ref = -INFINITY, l = 0.f;
            for (int j = 0; j < n_kv; ++j) {
                const uint32_t gi = gx + j;
                const bool diag = (j == n_kv - 1);
                uint32_t t[4][32];  // this row's 128 scores of the block
                if (ok && !mbar_wait(&s_full[x], gi & 1, abort_flag)) ok = false;
                tc_fence_after_sync();
#pragma unroll
                for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x32(tm + c * 32, t[c]);
                tmem_ld_wait();
                tc_fence_before_sync();
                mbar_arrive(&s_free[x]);  // the next block's scores may overwrite the columns
                // Diagonal block: keys behind the query (key > row r) do not count.  They are set to
                // -inf here, once, so that the maximum and the exponentials below (2^-inf = 0) need no
                // compare-and-select per score in the other blocks.
                if (diag) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (c * 32 + i > r) t[c][i] = 0xff800000u;
                    }
                }
                // row maximum of the raw scores (the scale is positive, so it commutes with max)
                float pm0 = -INFINITY, pm1 = -INFINITY, pm2 = -INFINITY, pm3 = -INFINITY;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        pm0 = fmax3(pm0, __uint_as_float(t[c][i]), __uint_as_float(t[c][i + 1]));
                        pm1 = fmax3(pm1, __uint_as_float(t[c][i + 2]), __uint_as_float(t[c][i + 3]));
                        pm2 = fmax3(pm2, __uint_as_float(t[c][i + 4]), __uint_as_float(t[c][i + 5]));
                        pm3 = fmax3(pm3, __uint_as_float(t[c][i + 6]), __uint_as_float(t[c][i + 7]));
                    }
                }
                // log2 domain; finite (key 0 of every block counts for every row)
                const float cand = fmaxf(m_ref, fmaxf(fmaxf(pm0, pm1), fmaxf(pm2, pm3)) * args.scale_log2);
                // The reference maximum moves for the whole warp at once (the tensor-memory round
                // trip of O is a warp-wide operation), and only when some row needs it.
                const bool moved = __any_sync(0xffffffffu, cand > m_ref + kRescaleStep);
                float alpha = 1.f;
                if (moved) {
                    alpha = ex2_approx(m_ref - cand);  // 0 on the first block (m_ref = -inf)
                    m_ref = cand;
                }
                // P = exp2(s*scale - m_ref): one FMA + one special-function op per score; neighbouring
                // keys are packed two to a register as fp16, the A operand of O += P V.  The row sum is
                // taken from the fp32 values.
                float sum0 = 0.f, sum1 = 0.f, sum2 = 0.f, sum3 = 0.f;
                const float neg_m = -m_ref;
                uint32_t pk[2][32];  // keys (2k, 2k+1) of the block in register k
#pragma unroll
                for (int c = 0; c < 4; ++c) {
#pragma unroll
                    for (int k = 0; k < 16; k += 2) {
                        float a0 = ex2_approx(fmaf(__uint_as_float(t[c][2 * k]), args.scale_log2, neg_m));
                        float a1 = ex2_approx(fmaf(__uint_as_float(t[c][2 * k + 1]), args.scale_log2, neg_m));
                        float b0 = ex2_approx(fmaf(__uint_as_float(t[c][2 * k + 2]), args.scale_log2, neg_m));
                        float b1 = ex2_approx(fmaf(__uint_as_float(t[c][2 * k + 3]), args.scale_log2, neg_m));
                        sum0 += a0;
                        sum1 += a1;
                        sum2 += b0;
                        sum3 += b1;
                        const __half2 ah = __floats2half2_rn(a0, a1), bh = __floats2half2_rn(b0, b1);
                        pk[c >> 1][(c & 1) * 16 + k] = *reinterpret_cast<const uint32_t*>(&ah);
                        pk[c >> 1][(c & 1) * 16 + k + 1] = *reinterpret_cast<const uint32_t*>(&bh);
                    }
                }
                // P V of the previous block has retired: the P columns are free and O is complete
                if (j > 0) {
                    if (ok && !mbar_wait(&o_full[x], (gi - 1) & 1, abort_flag)) ok = false;
                    tc_fence_after_sync();
                    if (moved) {  // O *= alpha, through registers
#pragma unroll
                        for (int hh = 0; hh < 2; ++hh) {
                            uint32_t o[32];
                            tmem_ld_32x32b_x32(tm + kOCol + hh * 32, o);
                            tmem_ld_wait();
#pragma unroll
                            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                            tmem_st_32x32b_x32(tm + kOCol + hh * 32, o);
                        }
                    }
                }
                tmem_st_32x32b_x32(tm + kPCol, pk[0]);
                tmem_st_32x32b_x32(tm + kPCol + 32, pk[1]);
                tmem_st_wait();
                tc_fence_before_sync();
                mbar_arrive(&p_full[x]);
                l = l * alpha + ((sum0 + sum1) + (sum2 + sum3));
            }
            gx += n_kv;
            // the last P V of the item
            if (ok && !mbar_wait(&o_full[x], (gx - 1) & 1, abort_flag)) ok = false;
            tc_fence_after_sync();
            const int t_idx = q0 + r;
            const float inv_l = 1.0f / l;
            const bool planes = args.out_bf16 == 2;
            if (args.tma_out) {
                // Whole tile: each thread puts its row into the pipeline's staging buffer in the
                // 128-byte-swizzled layout, and one thread sends the blocks off with TMA stores.
                if (leader) tma_store_wait_read();  // the previous tile has left the buffer
                pipe_bar_sync(bar_id);
            }
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {  // 32 output columns at a time
                uint32_t o[32];
                tmem_ld_32x32b_x32(tm + kOCol + hh * 32, o);
                tmem_ld_wait();
                if (args.out_bf16) {
                    // 64 bf16 columns are one 128-byte row: chunks 4*hh .. 4*hh+3 of row r; with split
                    // outputs the dropped parts go to the second block
                    uint4 vh[4], vl[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint32_t ph[4], pl[4];
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const float a = __uint_as_float(o[8 * i + 2 * k]) * inv_l, b2 = __uint_as_float(o[8 * i + 2 * k + 1]) * inv_l;
                            const __nv_bfloat162 hv = __floats2bfloat162_rn(a, b2);
                            const __nv_bfloat162 lv = __floats2bfloat162_rn(a - __low2float(hv), b2 - __high2float(hv));
                            ph[k] = *reinterpret_cast<const uint32_t*>(&hv);
                            pl[k] = *reinterpret_cast<const uint32_t*>(&lv);
                        }
                        vh[i] = make_uint4(ph[0], ph[1], ph[2], ph[3]);
                        vl[i] = make_uint4(pl[0], pl[1], pl[2], pl[3]);
                    }
                    if (args.tma_out) {
                        uint4* rowh = reinterpret_cast<uint4*>(out_s + r * 128);
                        uint4* rowl = reinterpret_cast<uint4*>(out_s + kBlk + r * 128);
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            rowh[(hh * 4 + i) ^ (r & 7)] = vh[i];
                            if (planes) rowl[(hh * 4 + i) ^ (r & 7)] = vl[i];
                        }
                    } else if (ok && t_idx < args.T) {
                        uint16_t* oh = reinterpret_cast<uint16_t*>(args.out) + ((size_t)(row_base + t_idx) * args.C) + h * HS + hh * 32;
                        uint4* o1 = reinterpret_cast<uint4*>(oh);
                        uint4* o2 = reinterpret_cast<uint4*>(oh + (size_t)args.B * args.T * args.C);
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            o1[i] = vh[i];
                            if (planes) o2[i] = vl[i];
                        }
                    }
                } else {
                    // fp32: block hh holds columns 32*hh .. +31 as 128-byte rows
                    float4* row = reinterpret_cast<float4*>(out_s + hh * kBlk + r * 128);
                    float* og = args.out + ((size_t)(row_base + t_idx) * args.C) + h * HS + hh * 32;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        float4 v = make_float4(__uint_as_float(o[4 * i]) * inv_l, __uint_as_float(o[4 * i + 1]) * inv_l,
                                               __uint_as_float(o[4 * i + 2]) * inv_l, __uint_as_float(o[4 * i + 3]) * inv_l);
                        if (args.round_out) { v.x = round_tf32(v.x); v.y = round_tf32(v.y); v.z = round_tf32(v.z); v.w = round_tf32(v.w); }
                        if (args.tma_out) row[i ^ (r & 7)] = v;
                        else if (ok && t_idx < args.T) *reinterpret_cast<float4*>(og + 4 * i) = v;
                    }
                }
            }
            if (args.tma_out) {
                fence_proxy_async_smem();
                pipe_bar_sync(bar_id);
                if (leader && ok) {
                    if (args.out_bf16) {
                        tma_store_2d(&tmap_out, h * HS, row_base + q0, out_s);
                        if (planes) tma_store_2d(&tmap_out, h * HS, args.B * args.T + row_base + q0, out_s + kBlk);
                    } else {
                        tma_store_2d(&tmap_out, h * HS, row_base + q0, out_s);
                        tma_store_2d(&tmap_out, h * HS + 32, row_base + q0, out_s + kBlk);
                    }
                    tma_store_commit();
                }
            }
            if (ok && t_idx < args.T && args.lse)
                args.lse[((size_t)b * args.NH + h) * args.T + t_idx] = m_ref * 0.6931471805599453f + logf(l);
            tc_fence_before_sync();
            mbar_arrive(&item_empty[slot]);
        }
        if (leader) tma_store_wait_all();
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

// qkv_split: the packed buffer [B*T, 3C] as two fp16 planes (hi, then lo B*T rows further down)
int launch_attention_split(b200_ctx* ctx, float* out, float* lse, const uint16_t* qkv_split, int B, int T, int C,
                           int NH, int flags) {
    static bool attr_set[64] = {};
    if (!attr_set[ctx->device & 63]) {
        B200_CUDA(ctx, cudaFuncSetAttribute(attention_split_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AttSmem::TOTAL));
        attr_set[ctx->device & 63] = true;
    }
    CUtensorMap tm;  // one map for Q, K and V tiles of both planes: 128 rows x 64 16-bit values, 128-byte swizzle
    int st = b200_get_tensor_map_bf16(ctx, &tm, qkv_split, (uint64_t)2 * B * T, (uint64_t)3 * C, (uint64_t)3 * C, BKV, 64);
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
    a.plane_rows = B * T;
    a.num_qt = (T + BQ - 1) / BQ;
    a.num_pairs = (a.num_qt + 1) / 2;
    a.num_items = a.num_pairs * NH * B;
    a.scale_log2 = 1.4426950408889634f / sqrtf((float)HS);
    a.round_out = (flags & ROUND_OUT_TF32) ? 1 : 0;
    a.status = ctx->d_status;
    const int grid = a.num_items < ctx->num_sms ? a.num_items : ctx->num_sms;
    cudaError_t le = launch_pdl(ctx, attention_split_kernel, dim3(grid), dim3(kAttThreads), AttSmem::TOTAL, tm, tmo, a);
    ctx->launches++;
    B200_CUDA(ctx, le);
    return B200_OK;
}

}  // namespace b200
