// GEMM on CTA pairs (tcgen05 cta_group::2): the same math and epilogue as gemm_tf32.cu
// (out = act(inp . weight^T + bias) (+ residual); reference semantics
// kernels/matmul/1_matmul_tiling.cuh:25-54, fused bias/GELU of 9_matmul_async_cg_tf32_gelu.cuh
// :57-84,196-212), but two CTAs of a cluster compute one 256 x W tile together.
//
// Why pairs: a 128 x 256 tile computed by one CTA has to pull 96 bytes of operands per tensor-pipe
// cycle out of L2, and an SM gets about 52.  In a pair, CTA r loads rows [128r,128r+128) of
// the inp tile and only half of the weight tile (rows [W/2*r, W/2*r+W/2)); one
// tcgen05.mma.cta_group::2 (M = 256) issued by the even CTA reads both halves of the weight tile
// from the two CTAs' shared memories, and each CTA's tensor memory receives its 128 x W part
// of the accumulator.  No load is broadcast across the cluster: every CTA issues its own TMA loads.
//
// Work distribution: tiles of 256 rows x W columns (W fixed per launch, chosen on the host from a
// cost model: a multiple of 32 up to 256; the UMMA's N, the weight box and the epilogue's chunk
// count follow it) are dealt to the resident CTA pairs round robin - columns fastest when the
// weight matrix stays in L2, so that the pairs working side by side share an activation tile,
// rows fastest for the lm-head, so that they share a few weight tiles while the weights stream
// once.  (Handing every pair an equal contiguous share of finer column units was measured and
// dropped: it removes the partly empty last wave but makes the tiles narrower, and a narrow tile
// re-reads its 256 activation rows for fewer columns - the L2 feed, not the tensor pipe, sets the
// pace - QKV 54 -> 86 us, fc-proj 85 -> 139 us.)
// Split K (only for results that are ADDED onto the output, GEMM_ACCUM_OUT): with N = 768 a
// launch has 96 or 128 tiles for 74 pairs, i.e. a second wave that is mostly empty.  K is then cut
// into 2-4 slices that are separate tiles, each adding its partial sum onto the output with the
// same TMA reductions; so that the sum of an element is always formed in the same order (residual
// + slice 0 + slice 1 ...), the epilogue warp of slice s waits - bounded - for a flag that the warp
// which owns the same rows and columns in slice s-1 sets once its reductions have completed.
// Slice s-1 of a tile always precedes slice s in the dealing order and all pairs are resident,
// so the wait cannot deadlock.  A flag has one writer and one reader, who puts it back to zero:
// the words are all zero again when the kernel ends (also under graph replay).
//
// Arithmetic (template MODE):
//   PAIR_TF32    fp32 operands, tcgen05.mma kind::tf32 (the tensor core reads the upper 19 bits)
//   PAIR_BF16    bf16 operands, kind::f16
//   PAIR_FP8     e4m3 operands, kind::f8f6f4 (128 elements of K per 128-byte block, 32 per instruction)
//   PAIR_BF16X3  both operands given as two bf16 planes, x = hi + lo with hi = bf16(x) and
//                lo = bf16(x - hi) (16 significant bits); three kind::f16 products per K step,
//                hi.hi + hi.lo + lo.hi, accumulated in fp32: the dropped lo.lo term and the
//                third-order parts are below 2^-16 of the product.  Same operand bytes as fp32,
//                1.5 x the tensor time of one TF32 pass, about 30 x smaller error.
//
// Per CTA (10 warps): warp 0 TMA producer, warp 1 tensor-memory allocation (+ UMMA issue in the
// even CTA), warps 2-9 epilogue (warp w reads lane quarter w % 4; warps 2-5 drain the first half
// of the tile's columns, warps 6-9 the second, one 4 KB staging buffer each).  Barriers:
//   full[s]        in the even CTA: its producer's one arrival announces both CTAs' TMA bytes
//   empty[s]       in each CTA, signalled by tcgen05.commit from the even CTA (one per CTA)
//   tmem_full[a]   in each CTA, likewise
//   tmem_empty[a]  in the even CTA, 16 arrivals (one per epilogue warp of both CTAs)
// Every wait is time-bounded; the two CTAs synchronise on the cluster barrier after set-up and
// before tensor memory is freed, so neither leaves while the other can still touch its shared
// memory.
#include <cstdlib>
#include "gemm_common.cuh"

namespace b200 {

namespace {

constexpr int BM = kGemmBM;  // rows per CTA; 2*BM per pair
constexpr int kEpiWarps = 8;  // two per tensor-memory lane quarter, each draining half of the columns
constexpr int kThreads = 64 + 32 * kEpiWarps;
constexpr int kMaxW = 256;    // widest tile: two accumulators of 256 columns fill tensor memory

template <int MODE>
struct PairCfg {
    static constexpr int PARTS = (MODE == PAIR_BF16X3) ? 2 : 1;  // operand planes per matrix
    static constexpr int A_BYTES = BM * 128;                     // one plane: 128 rows x one 128-byte K block
    static constexpr int B_BYTES = (kMaxW / 2) * 128;            // one plane of this CTA's half of a full-width weight tile
    static constexpr int STAGE_BYTES = PARTS * (A_BYTES + B_BYTES);
    static constexpr int BAR_BYTES = 512;
    static constexpr int STAGES_RAW = (kGemmMaxSmem - 1024 - BAR_BYTES - kGemmEpiBytes) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
    static constexpr int SMEM = 1024 + STAGES * STAGE_BYTES + kGemmEpiBytes + BAR_BYTES;
    static constexpr int TMEM_COLS = 512;
    // elements of K per 128-byte block
    static constexpr int BKE = (MODE == PAIR_TF32) ? kGemmBK : (MODE == PAIR_FP8 ? kGemmBKQ : kGemmBKH);
    static_assert(SMEM > 117 * 1024, "a second resident CTA could block in tcgen05.alloc");
    static_assert(SMEM <= kGemmMaxSmem, "shared memory over the 227 KB limit");
    static_assert(STAGES >= 2, "need at least a double buffer");
    static_assert(STAGES * STAGE_BYTES >= kEpiWarps * 4 * 4096, "the last tile's epilogue stages four buffers per warp in the operand ring");
};

// The tiles of one CTA pair, in order.  Every role of both CTAs walks the same sequence.
struct TileWalk {
    int cur, step, total, tiles;
    __device__ TileWalk(const GemmArgs& a, int pair, int num_pairs)
        : cur(pair), step(num_pairs), tiles(a.num_m_blocks * a.num_n_blocks) {
        total = a.tail_sub > 1 ? a.n_main + (tiles - a.n_main) * a.tail_sub : a.k_splits * tiles;
    }
    // next tile: 256 rows from m_blk * 256, `width` columns from col0, K blocks [kb0, kb1) (slice ks
    // of K); `tile` numbers the output tile (the same for all its K slices); narrow: one of the
    // tail_sub parts of a left-over tile (its weight rows come in boxes of their own size)
    __device__ bool next(const GemmArgs& a, int num_kb, int& m_blk, int& col0, int& width, int& kb0, int& kb1, int& ks, int& tile, bool& narrow) {
        if (cur >= total) return false;
        int part = -1;
        if (a.tail_sub > 1) {  // (only without K slices)
            ks = 0;
            tile = cur;
            if (cur >= a.n_main) {
                const int v = cur - a.n_main;
                tile = a.n_main + v / a.tail_sub;
                part = v - (v / a.tail_sub) * a.tail_sub;
            }
        } else {
            ks = cur / tiles;
            tile = cur - ks * tiles;
        }
        int n_blk;
        if (a.n_fastest) { m_blk = tile / a.num_n_blocks; n_blk = tile - m_blk * a.num_n_blocks; }
        else { n_blk = tile / a.num_m_blocks; m_blk = tile - n_blk * a.num_m_blocks; }
        col0 = n_blk * a.tile_w;
        const int rest = (a.N - col0 + a.unit_cols - 1) / a.unit_cols * a.unit_cols;
        width = rest < a.tile_w ? rest : a.tile_w;
        narrow = part >= 0;
        if (narrow) {  // N is a multiple of tile_w here: every part is whole
            width = a.tile_w / a.tail_sub;
            col0 += part * width;
        }
        kb0 = (int)((long)num_kb * ks / a.k_splits);
        kb1 = (int)((long)num_kb * (ks + 1) / a.k_splits);
        cur += step;
        return true;
    }
};

// flag word of (K slice, output tile, CTA of the pair, epilogue warp)
__device__ __forceinline__ unsigned int* split_flag(const GemmArgs& a, int ks, int tile, int tiles, int rank, int ew) {
    return a.split_flags + ((size_t)(ks * tiles + tile) * 2 + rank) * kEpiWarps + ew;
}

template <int MODE>
__global__ void __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_a_lo,
                 const __grid_constant__ CUtensorMap tmap_b, const __grid_constant__ CUtensorMap tmap_b_lo,
                 const __grid_constant__ CUtensorMap tmap_out,
                 const __grid_constant__ CUtensorMap tmap_bn, const __grid_constant__ CUtensorMap tmap_bn_lo,  // weight boxes of the narrow tail tiles
                 const GemmArgs args) {
    using Cfg = PairCfg<MODE>;
    constexpr int STAGES = Cfg::STAGES;
    constexpr int PARTS = Cfg::PARTS;
    constexpr int BKE = Cfg::BKE;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* smem_a = smem;                                   // [STAGES][PARTS][A_BYTES]
    uint8_t* smem_b = smem_a + STAGES * PARTS * Cfg::A_BYTES;  // [STAGES][PARTS][B_BYTES]
    uint8_t* smem_epi = smem + STAGES * Cfg::STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_epi + kGemmEpiBytes);
    uint64_t* full_bar = bars;                     // [STAGES] used in the even CTA
    uint64_t* empty_bar = bars + STAGES;           // [STAGES] each CTA
    uint64_t* tmem_full_bar = bars + 2 * STAGES;   // [2] each CTA
    uint64_t* tmem_empty_bar = tmem_full_bar + 2;  // [2] used in the even CTA
    uint64_t* drain_bar = tmem_empty_bar + 2;      // [1] even CTA
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(drain_bar + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();  // 0 = even CTA (issues the UMMAs), 1 = its peer
    const int pair = blockIdx.x >> 1;
    const int num_pairs = gridDim.x >> 1;
    const int num_kb = (args.K + BKE - 1) / BKE;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(&tmem_full_bar[a], 1); mbar_init(&tmem_empty_bar[a], 2 * kEpiWarps); }
        mbar_init(drain_bar, 1);
        *abort_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_b);
        tma_prefetch_desc(&tmap_out);
        if (PARTS == 2) {
            tma_prefetch_desc(&tmap_a_lo);
            tma_prefetch_desc(&tmap_b_lo);
        }
        if (args.tail_sub > 1) {
            tma_prefetch_desc(&tmap_bn);
            if (PARTS == 2) tma_prefetch_desc(&tmap_bn_lo);
        }
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_holder, Cfg::TMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();  // the peer's barriers are initialised before anything arrives on them
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;
    griddep_wait();  // set-up done; from here on global memory is touched

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            TileWalk walk(args, pair, num_pairs);
            int m_blk, col0, width, kb0, kb1, ks, tile;
            bool narrow;
            while (ok && walk.next(args, num_kb, m_blk, col0, width, kb0, kb1, ks, tile, narrow)) {
                // weight rows per load: this CTA's half of a full-width tile (of a narrow tail tile)
                const int box_b = narrow ? (width >> 1) : (args.tile_w >> 1);
                const uint32_t tx = (uint32_t)PARTS * (Cfg::A_BYTES + box_b * 128);  // per CTA; the same in both
                const CUtensorMap* map_b = narrow ? &tmap_bn : &tmap_b;
                const CUtensorMap* map_b_lo = narrow ? &tmap_bn_lo : &tmap_b_lo;
                // a ragged last tile is narrower: its halves start closer together, the box keeps its
                // size (the rows behind the half are loaded but not multiplied)
                const int row_a = m_blk * 2 * BM + (int)rank * BM;
                const int row_b = col0 + (int)rank * (width >> 1);
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag)) { ok = false; break; }
                    const uint32_t full_leader = map_to_cta(smem_u32(&full_bar[s]), 0);
                    // The even CTA announces the bytes of both CTAs with its one arrival.  The
                    // peer's bytes may land before that arrival; the phase cannot complete
                    // without it, and the peer cannot be a whole phase ahead because its stage is
                    // only freed by the even CTA's commit.
                    if (rank == 0) mbar_arrive_expect_tx(&full_bar[s], 2 * tx);
#pragma unroll
                    for (int p = 0; p < PARTS; ++p) {
                        tma_load_2d_pair(smem_a + (s * PARTS + p) * Cfg::A_BYTES, p ? &tmap_a_lo : &tmap_a, kb * BKE, row_a, full_leader);
                        tma_load_2d_pair(smem_b + (s * PARTS + p) * Cfg::B_BYTES, p ? map_b_lo : map_b, kb * BKE, row_b, full_leader);
                    }
                }
            }
            if (!ok) atomicCAS(args.status, 0, DEV_TIMEOUT_PRODUCER);
        }
    } else if (warp == 1) {
        // ------------------------------------------- UMMA issuer (even CTA only)
        if (rank == 0 && lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            int tile_iter = 0;
            TileWalk walk(args, pair, num_pairs);
            int m_blk, col0, width, kb0, kb1, ks, tile;
            bool narrow;
            while (ok && walk.next(args, num_kb, m_blk, col0, width, kb0, kb1, ks, tile, narrow)) {
                const int acc = tile_iter & 1;
                const uint32_t acc_ph = (tile_iter >> 1) & 1;
                ++tile_iter;
                if (!mbar_wait_cluster(&tmem_empty_bar[acc], acc_ph ^ 1, abort_flag)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t idesc = (MODE == PAIR_TF32) ? make_idesc_tf32(2 * BM, width, 0)
                                     : (MODE == PAIR_FP8 ? make_idesc_e4m3(2 * BM, width, 0) : make_idesc_bf16(2 * BM, width, 0));
                const uint32_t d_tmem = tmem_base + acc * kMaxW;
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(&full_bar[s], ph, abort_flag)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint64_t a_desc = make_smem_desc_sw128(smem_u32(smem_a + s * PARTS * Cfg::A_BYTES), 16, 1024);
                    const uint64_t b_desc = make_smem_desc_sw128(smem_u32(smem_b + s * PARTS * Cfg::B_BYTES), 16, 1024);
                    if (MODE == PAIR_BF16X3) {
                        const uint64_t al_desc = make_smem_desc_sw128(smem_u32(smem_a + (s * PARTS + 1) * Cfg::A_BYTES), 16, 1024);
                        const uint64_t bl_desc = make_smem_desc_sw128(smem_u32(smem_b + (s * PARTS + 1) * Cfg::B_BYTES), 16, 1024);
#pragma unroll
                        for (int k = 0; k < 4; ++k) {  // 16 bf16 = 32 bytes of K per instruction
                            umma_f16_ss_pair(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, ((kb - kb0) | k) != 0);
                            umma_f16_ss_pair(d_tmem, a_desc + 2 * k, bl_desc + 2 * k, idesc, 1);
                            umma_f16_ss_pair(d_tmem, al_desc + 2 * k, b_desc + 2 * k, idesc, 1);
                        }
                    } else {
#pragma unroll
                        for (int k = 0; k < 4; ++k) {  // 32 bytes of K per instruction: 8 tf32, 16 bf16 or 32 e4m3
                            if (MODE == PAIR_BF16) umma_f16_ss_pair(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, ((kb - kb0) | k) != 0);
                            else if (MODE == PAIR_FP8) umma_f8_ss_pair(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, ((kb - kb0) | k) != 0);
                            else umma_tf32_ss_pair(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, ((kb - kb0) | k) != 0);
                        }
                    }
                    // free the stage in both CTAs
                    const uint32_t e = smem_u32(&empty_bar[s]);
                    umma_commit_pair(map_to_cta(e, 0));
                    umma_commit_pair(map_to_cta(e, 1));
                }
                if (ok) {
                    const uint32_t f = smem_u32(&tmem_full_bar[acc]);
                    umma_commit_pair(map_to_cta(f, 0));
                    umma_commit_pair(map_to_cta(f, 1));
                }
            }
            // wait (bounded) until everything issued has retired before tensor memory is freed
            umma_commit_pair(map_to_cta(smem_u32(drain_bar), 0));
            if (!mbar_wait(drain_bar, 0, abort_flag)) ok = false;
            if (!ok) atomicCAS(args.status, 0, DEV_TIMEOUT_MMA);
        }
    } else {
        // ---------------------------------------------------------------- epilogue
        const int q = warp & 3;
        const int ew = warp - 2;  // 0..7
        // column split in units of one chunk (two for a bf16 output, whose stores take 64 columns)
        const int unit = args.out_h ? 2 : 1;
        bool ok = true;
        int tile_iter = 0;
        TileWalk walk(args, pair, num_pairs);
        int m_blk, col0, width, kb0, kb1, ks, tile;
        bool narrow;
        while (ok && walk.next(args, num_kb, m_blk, col0, width, kb0, kb1, ks, tile, narrow)) {
            const int n_units = (width >> 5) / unit;
            const int c_mid = ((n_units + 1) / 2) * unit;
            const int c_begin = (ew < 4) ? 0 : c_mid;
            const int c_end = (ew < 4) ? c_mid : (width >> 5);
            const int acc = tile_iter & 1;
            const uint32_t acc_ph = (tile_iter >> 1) & 1;
            ++tile_iter;
            const float* bias = ks == 0 ? args.bias : nullptr;  // added once, by the first K slice
            const float bias_first = gemm_bias_chunk(bias, args.N, col0, c_begin, lane);  // on its way while the tile is computed
            if (!mbar_wait(&tmem_full_bar[acc], acc_ph, abort_flag)) { ok = false; break; }
            tc_fence_after_sync();
            if (ks > 0) {
                // the partial sum of the previous K slice must be in the output before this one is added
                if (lane == 0) {
                    const unsigned int* f = split_flag(args, ks - 1, tile, walk.tiles, (int)rank, ew);
                    const uint64_t t0 = globaltimer_ns();
                    unsigned int v;
                    while (true) {
                        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
                        if (v != 0u || *abort_flag != 0) break;
                        if (globaltimer_ns() - t0 > kWaitLimitNs) { *abort_flag = 1; break; }
                        __nanosleep(100);
                    }
                    if (v == 0u) ok = false;
                    else *const_cast<volatile unsigned int*>(f) = 0u;  // consumed: zero again for the next launch
                }
                ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
                if (!ok) break;
            }
            // The pair's last tile: every UMMA has retired and nothing is loaded any more, so the operand
            // ring is free, and each warp takes four staging buffers out of it instead of its one -
            // no chunk waits for the store before it, which shortens the tail every launch ends with
            // (measured per launch: 12-14 thousand cycles with one buffer for the accumulating and the
            // two-plane epilogues).
            const bool last_tile = walk.cur >= walk.total;
            uint8_t* staging = last_tile ? smem + ew * 4 * 4096 : smem_epi + ew * 4096;
            if (c_begin < c_end || args.lse_part != nullptr)  // (an empty share still owes its log-sum-exp slot)
                gemm_drain_accumulator(args, bias, &tmap_out, tmem_base + acc * kMaxW, q, lane,
                                       m_blk * 2 * BM + (int)rank * BM + q * 32, col0,
                                       staging, bias_first, c_begin, c_end, last_tile ? 4 : 1, 2 * (col0 / kMaxW) + (ew < 4 ? 0 : 1));
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty_bar[acc]), 0));
                if (args.k_splits > 1 && ks + 1 < args.k_splits) {
                    // this warp's reductions have been performed: the next slice may add its own
                    tma_store_wait_all();
                    __threadfence();
                    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(split_flag(args, ks, tile, walk.tiles, (int)rank, ew)), "r"(1u) : "memory");
                }
            }
        }
        if (lane == 0) tma_store_wait_all();  // the staging buffers must outlive the stores reading them
        if (!ok && lane == 0) atomicCAS(args.status, 0, DEV_TIMEOUT_EPILOGUE);
    }

    griddep_launch_dependents();
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();  // the peer is done with this CTA's shared and tensor memory
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
    }
}

template <int MODE>
int launch_pair(b200_ctx* ctx, const CUtensorMap* maps, GemmArgs& a, int num_pairs_max) {
    using Cfg = PairCfg<MODE>;
    static int resident_pairs[64] = {};  // CTA pairs the device can keep resident at once
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = Cfg::SMEM;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->pdl ? 2 : 1;
    if (!resident_pairs[ctx->device & 63]) {
        B200_CUDA(ctx, cudaFuncSetAttribute(gemm_pair_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM));
        cfg.gridDim = dim3(2 * num_pairs_max);
        int n = 0;
        B200_CUDA(ctx, cudaOccupancyMaxActiveClusters(&n, gemm_pair_kernel<MODE>, &cfg));
        if (n < 1) n = 1;
        resident_pairs[ctx->device & 63] = n < num_pairs_max ? n : num_pairs_max;
    }
    // persistent: never more pairs than can be resident together (the K slices of a tile wait for
    // one another, and the rest would run as a tail anyway), never more than there are tiles
    const int total = a.k_splits * a.num_m_blocks * a.num_n_blocks;
    int pairs = total < resident_pairs[ctx->device & 63] ? total : resident_pairs[ctx->device & 63];
    if (pairs > num_pairs_max) pairs = num_pairs_max;  // the caller may have set SMs aside
    cfg.gridDim = dim3(2 * pairs);
    // a.tail_sub arrives as the candidate (the narrow weight maps exist): split the left-over tiles of the last,
    // partly empty round if their parts still fit into one round
    if (a.tail_sub > 1) {
        const int tiles = a.num_m_blocks * a.num_n_blocks, left = tiles % pairs;
        static const bool tail_off = [] { const char* e = getenv("B200_GEMM_TAIL"); return e && e[0] == '0'; }();  // tuning hook
        if (!tail_off && tiles > pairs && left > 0 && left * a.tail_sub <= pairs) a.n_main = tiles - left;
        else a.tail_sub = 1;
    }
    B200_CUDA(ctx, cudaLaunchKernelEx(&cfg, gemm_pair_kernel<MODE>, maps[0], maps[1], maps[2], maps[3], maps[4], maps[5], maps[6], a));
    ctx->launches++;
    return B200_OK;
}

}  // namespace

int preload_gemm_pair_kernels(b200_ctx* ctx) {
    B200_CUDA(ctx, cudaFuncSetAttribute(gemm_pair_kernel<PAIR_TF32>, cudaFuncAttributeMaxDynamicSharedMemorySize, PairCfg<PAIR_TF32>::SMEM));
    return B200_OK;
}

int launch_gemm_pair(b200_ctx* ctx, float* out, const void* inp, const void* inp_lo, const void* weight, const void* weight_lo,
                     const float* bias, const float* residual, int M, int K, int N, int flags,
                     unsigned long long* argmax_keys, int argmax_cols, int kind, uint16_t* out_h, int out_planes,
                     int store_period, const GemmRowStats* stats, float alpha, int lo_col0) {
    const int num_pairs_max = ctx->num_sms / 2;
    const bool half = kind == PAIR_BF16 || kind == PAIR_BF16X3;
    GemmArgs a;
    a.out = out; a.out_h = out_h; a.bias = bias; a.residual = residual;
    a.M = M; a.N = N; a.K = K;
    a.alpha = alpha;
    a.lo_col0 = lo_col0;
    a.tmap_out2 = static_cast<const CUtensorMap*>(ctx->next_gemm_out2);
    ctx->next_gemm_out2 = nullptr;
    a.out2_rows = a.tmap_out2 ? ctx->next_gemm_out2_rows : 0;
    ctx->next_gemm_out2_rows = 0;
    if (a.tmap_out2 && (out_h || residual || (flags & GEMM_ACCUM_OUT) || store_period)) {
        ctx->last_error = "a second output needs a plain fp32 store epilogue";
        return B200_ERR_STATE;
    }
    a.num_m_blocks = (M + 2 * BM - 1) / (2 * BM);
    // weight small enough to stay in L2: columns fastest, so the pairs working side by side share an
    // inp tile; otherwise rows fastest, so that they share a few weight tiles while the weights stream once
    a.n_fastest = ((size_t)N * K * 4 <= (size_t)32 << 20) ? 1 : 0;
    a.flags = flags;
    a.status = ctx->d_status;
    a.argmax_keys = argmax_keys;
    a.argmax_cols = argmax_cols;
    a.store_period = store_period;
    a.out_planes = out_planes;
    a.sample_inv_temp = stats ? stats->inv_temp : 0.f;
    a.sample_seed = stats ? stats->seed : 0u;
    a.sample_stream0 = stats ? stats->stream0 : 0u;
    a.lse_part = stats ? stats->lse_part : nullptr;
    a.lse_slots = stats ? stats->lse_slots : 0;
    if (stats && (!argmax_keys || (stats->lse_part && stats->lse_slots < 2 * ((N + kMaxW - 1) / kMaxW)))) {
        ctx->last_error = "row statistics need the fused arg-max keys and 2 * ceil(N / 256) partial slots per row";
        return B200_ERR_STATE;
    }
    a.unit_cols = out_h ? 64 : 32;
    // Tile width and K slices: fewest estimated cycles.  Per 128-byte K block a tile needs 2*W cycles
    // of the tensor pipe per product (three products with split operands) and (128 + W/2) * 128 bytes
    // per operand plane out of L2, of which an SM gets about 52 per cycle; plus a fixed cost per tile
    // (pipeline fill, the part of the epilogue that is not hidden).
    const int bke = half ? kGemmBKH : (kind == PAIR_FP8 ? kGemmBKQ : kGemmBK);
    const int num_kb = (K + bke - 1) / bke;
    const int parts = kind == PAIR_BF16X3 ? 2 : 1, products = kind == PAIR_BF16X3 ? 3 : 1;
    const bool may_split = (flags & GEMM_ACCUM_OUT) && !(flags & (GEMM_GELU | GEMM_ROUND_OUT_TF32)) && ctx->d_split_flags != nullptr;
    int best_w = kMaxW, best_ks = 1;
    double best_cost = -1.0;
    for (int w = kMaxW; w >= ((stats && stats->lse_part) ? kMaxW : 64); w -= 64) {  // the partial slots are numbered by 256-column tiles
        const long tiles = (long)a.num_m_blocks * ((N + w - 1) / w);
        for (int ks = 1; ks <= (may_split ? 4 : 1); ++ks) {
            if (ks > 1 && (num_kb / ks < 6 || tiles * ks * 2 * kEpiWarps > (long)ctx->split_flag_words)) break;
            double waves = (double)((tiles * ks + num_pairs_max - 1) / num_pairs_max);
            // full-width tiles without K slices: what is left over after the last full round is computed in
            // quarter-width tiles (GemmArgs::tail_sub).  Measured on the GELU GEMM of the 124M model
            // (8192 x 3072 x 768, split operands): 91 us against 95 without the tail and 97 with 192-wide
            // tiles, which this model would otherwise prefer by a percent - hence the 0.4 of a round.
            const long left = tiles % num_pairs_max;
            if (ks == 1 && w == kMaxW && N % kMaxW == 0 && !stats && !argmax_keys && tiles > num_pairs_max && left > 0 && left * 4 <= num_pairs_max)
                waves = (double)(tiles / num_pairs_max) + 0.4;
            const double tensor = 2.0 * w * products, feed = parts * (128.0 + w / 2) * 128.0 / 52.0;
            // a slice also waits for its predecessor's sums to land and for its own before it signals
            const double cost = waves * (((num_kb + ks - 1) / ks) * (tensor > feed ? tensor : feed) + (ks > 1 ? 3500.0 : 2000.0));
            if (best_cost < 0 || cost < best_cost * 0.999) { best_cost = cost; best_w = w; best_ks = ks; }
        }
    }
    // tuning hooks: B200_GEMM_BN = tile width (64, 128, 192, 256), B200_GEMM_KSPLIT = K slices (1-4)
    static const int forced_w = [] { const char* e = getenv("B200_GEMM_BN"); return e ? atoi(e) : 0; }();
    static const int forced_ks = [] { const char* e = getenv("B200_GEMM_KSPLIT"); return e ? atoi(e) : 0; }();
    if ((forced_w == 64 || forced_w == 128 || forced_w == 192 || forced_w == 256) && !(stats && stats->lse_part)) best_w = forced_w;
    if (forced_ks >= 1 && forced_ks <= 4 && (forced_ks == 1 || may_split)) {
        best_ks = forced_ks;
        const long tiles = (long)a.num_m_blocks * ((N + best_w - 1) / best_w);
        if (num_kb < best_ks || tiles * best_ks * 2 * kEpiWarps > (long)ctx->split_flag_words) best_ks = 1;
    }
    a.tile_w = best_w;
    a.num_n_blocks = (N + best_w - 1) / best_w;
    a.k_splits = best_ks;
    a.split_flags = ctx->d_split_flags;

    CUtensorMap maps[7];  // inp, inp (lo plane), weight, weight (lo plane), out, weight in narrow boxes (and its lo plane)
    int st;
    const uint32_t box_b = (uint32_t)(best_w / 2);
    if (half) {
        st = b200_get_tensor_map_bf16(ctx, &maps[0], inp, (uint64_t)M, (uint64_t)K, (uint64_t)K, BM, bke);
        if (st == B200_OK) st = b200_get_tensor_map_bf16(ctx, &maps[2], weight, (uint64_t)N, (uint64_t)K, (uint64_t)K, box_b, bke);
        if (st != B200_OK) return st;
        if (kind == PAIR_BF16X3) {
            st = b200_get_tensor_map_bf16(ctx, &maps[1], inp_lo, (uint64_t)M, (uint64_t)K, (uint64_t)K, BM, bke);
            if (st == B200_OK) st = b200_get_tensor_map_bf16(ctx, &maps[3], weight_lo, (uint64_t)N, (uint64_t)K, (uint64_t)K, box_b, bke);
            if (st != B200_OK) return st;
        } else {
            maps[1] = maps[0]; maps[3] = maps[2];
        }
    } else if (kind == PAIR_FP8) {
        st = b200_get_tensor_map_u8(ctx, &maps[0], inp, (uint64_t)M, (uint64_t)K, (uint64_t)K, BM, bke);
        if (st == B200_OK) st = b200_get_tensor_map_u8(ctx, &maps[2], weight, (uint64_t)N, (uint64_t)K, (uint64_t)K, box_b, bke);
        if (st != B200_OK) return st;
        maps[1] = maps[0]; maps[3] = maps[2];
    } else {
        st = b200_get_tensor_map(ctx, &maps[0], static_cast<const float*>(inp), (uint64_t)M, (uint64_t)K, (uint64_t)K, BM, bke);
        if (st == B200_OK) st = b200_get_tensor_map(ctx, &maps[2], static_cast<const float*>(weight), (uint64_t)N, (uint64_t)K, (uint64_t)K, box_b, bke);
        if (st != B200_OK) return st;
        maps[1] = maps[0]; maps[3] = maps[2];
    }
    // the output in 32 x 32 boxes of fp32 (32 x 64 of bf16, both planes in one map), for the epilogue's TMA stores
    if (out_h) st = b200_get_tensor_map_bf16(ctx, &maps[4], out_h, (uint64_t)M * (out_planes ? 2 : 1), (uint64_t)N, (uint64_t)N, 32, 64);
    else st = b200_get_tensor_map(ctx, &maps[4], out, (uint64_t)M, (uint64_t)N, (uint64_t)N, 32, 32);
    if (st != B200_OK) return st;
    // Tail of the tile sequence in narrow tiles (see GemmArgs::tail_sub): full-width tiles, whole in N, no K
    // slices, no per-tile row statistics; the weight comes in boxes of a quarter of the rows
    maps[5] = maps[2]; maps[6] = maps[3];
    a.tail_sub = 1; a.n_main = 0;
    if (best_ks == 1 && best_w == kMaxW && N % kMaxW == 0 && !stats && !argmax_keys) {
        const uint32_t box_n = (uint32_t)(best_w / 4 / 2);
        if (kind == PAIR_FP8) st = b200_get_tensor_map_u8(ctx, &maps[5], weight, (uint64_t)N, (uint64_t)K, (uint64_t)K, box_n, bke);
        else if (half) st = b200_get_tensor_map_bf16(ctx, &maps[5], weight, (uint64_t)N, (uint64_t)K, (uint64_t)K, box_n, bke);
        else st = b200_get_tensor_map(ctx, &maps[5], static_cast<const float*>(weight), (uint64_t)N, (uint64_t)K, (uint64_t)K, box_n, bke);
        if (st == B200_OK && kind == PAIR_BF16X3) st = b200_get_tensor_map_bf16(ctx, &maps[6], weight_lo, (uint64_t)N, (uint64_t)K, (uint64_t)K, box_n, bke);
        if (st != B200_OK) return st;
        a.tail_sub = 4;  // candidate: launch_pair decides once it knows how many pairs run
    }
    switch (kind) {
        case PAIR_BF16X3: return launch_pair<PAIR_BF16X3>(ctx, maps, a, num_pairs_max);
        case PAIR_BF16: return launch_pair<PAIR_BF16>(ctx, maps, a, num_pairs_max);
        case PAIR_FP8: return launch_pair<PAIR_FP8>(ctx, maps, a, num_pairs_max);
        default: return launch_pair<PAIR_TF32>(ctx, maps, a, num_pairs_max);
    }
}

}  // namespace b200
