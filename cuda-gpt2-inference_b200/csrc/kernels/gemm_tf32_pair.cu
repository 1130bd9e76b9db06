// TF32 GEMM on CTA pairs (tcgen05 cta_group::2): the same math and epilogue as gemm_tf32.cu
// (out = act(inp . weight^T + bias) (+ residual); reference semantics
// kernels/matmul/1_matmul_tiling.cuh:25-54, fused bias/GELU of 9_matmul_async_cg_tf32_gelu.cuh
// :57-84,196-212), but two CTAs of a cluster compute one 256 x BN tile together.
//
// Why: a 128 x 256 tile computed by one CTA has to pull 96 bytes of operands per tensor-pipe
// cycle out of L2, and an SM gets about 52.  In a pair, CTA r loads rows [128r,128r+128) of
// the inp tile and only half of the weight tile (rows [BN/2*r, BN/2*r+BN/2)); one
// tcgen05.mma.cta_group::2 (M = 256) issued by the even CTA reads both halves of the weight tile
// from the two CTAs' shared memories, and each CTA's tensor memory receives its 128 x BN part
// of the accumulator.  Per CTA that is (128 + BN/2) x 128 bytes per K block: 64 bytes per
// tensor-pipe cycle at BN = 256, with six stages in flight instead of four.
// No load is broadcast across the cluster: every CTA issues its own TMA loads.
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
#include <cstdio>
#include <cstdlib>
#include "gemm_common.cuh"

namespace b200 {

namespace {

constexpr int BM = kGemmBM;  // rows per CTA; 2*BM per pair
constexpr int BK = kGemmBK;
constexpr int kEpiWarps = 8;  // two per tensor-memory lane quarter, each draining half of the columns
constexpr int kThreads = 64 + 32 * kEpiWarps;

template <int BN>
struct PairCfg {
    static constexpr int A_BYTES = BM * BK * 4;
    static constexpr int B_BYTES = (BN / 2) * BK * 4;  // this CTA's half of the weight tile
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int BAR_BYTES = 512;
    static constexpr int STAGES_RAW = (kGemmMaxSmem - 1024 - BAR_BYTES - kGemmEpiBytes) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
    static constexpr int SMEM = 1024 + STAGES * STAGE_BYTES + kGemmEpiBytes + BAR_BYTES;
    static constexpr int TMEM_COLS = (2 * BN <= 128) ? 128 : (2 * BN <= 256 ? 256 : 512);
    static_assert(SMEM > 117 * 1024, "a second resident CTA could block in tcgen05.alloc");
    static_assert(SMEM <= kGemmMaxSmem, "shared memory over the 227 KB limit");
    static_assert(BN % 32 == 0 && BN >= 64 && BN <= 256, "BN: multiple of 32, 64..256");
};

template <int BN, bool BF16>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tf32_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                      const __grid_constant__ CUtensorMap tmap_out,
                      const GemmArgs args) {
    using Cfg = PairCfg<BN>;
    constexpr int STAGES = Cfg::STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem_a + STAGES * Cfg::A_BYTES;
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
    const int num_tiles = args.num_m_blocks * args.num_n_blocks;
    constexpr int BKE = BF16 ? kGemmBKH : BK;  // elements per 128-byte K block
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

    auto tile_coords = [&](int tile, int& m_blk, int& n_blk) {
        if (args.n_fastest) { n_blk = tile % args.num_n_blocks; m_blk = tile / args.num_n_blocks; }
        else { m_blk = tile % args.num_m_blocks; n_blk = tile / args.num_m_blocks; }
    };

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
                int m_blk, n_blk;
                tile_coords(tile, m_blk, n_blk);
                const int row_a = m_blk * 2 * BM + (int)rank * BM;
                const int row_b = n_blk * BN + (int)rank * (BN / 2);
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag)) { ok = false; break; }
                    const uint32_t full_leader = map_to_cta(smem_u32(&full_bar[s]), 0);
                    // The even CTA announces the bytes of both CTAs with its one arrival.  The
                    // peer's bytes may land before that arrival; the phase cannot complete
                    // without it, and the peer cannot be a whole phase ahead because its stage is
                    // only freed by the even CTA's commit.
                    if (rank == 0) mbar_arrive_expect_tx(&full_bar[s], 2 * Cfg::STAGE_BYTES);
                    tma_load_2d_pair(smem_a + s * Cfg::A_BYTES, &tmap_a, kb * BKE, row_a, full_leader);
                    tma_load_2d_pair(smem_b + s * Cfg::B_BYTES, &tmap_b, kb * BKE, row_b, full_leader);
                }
            }
            if (!ok) atomicCAS(args.status, 0, DEV_TIMEOUT_PRODUCER);
        }
    } else if (warp == 1) {
        // ------------------------------------------- UMMA issuer (even CTA only)
        if (rank == 0 && lane == 0) {
            constexpr uint32_t idesc = BF16 ? make_idesc_bf16(2 * BM, BN, 0) : make_idesc_tf32(2 * BM, BN, 0);
            uint32_t it = 0;
            bool ok = true;
            int tile_iter = 0;
#ifdef B200_GEMM_TIMING
            long long t_wait = 0, t_mma = 0, t_commit = 0, t_acc = 0, t0 = clock64(), t_first = 0;
            const long long t_begin = t0;
#endif
            for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++tile_iter) {
                const int acc = tile_iter & 1;
                const uint32_t acc_ph = (tile_iter >> 1) & 1;
                if (!mbar_wait_cluster(&tmem_empty_bar[acc], acc_ph ^ 1, abort_flag)) { ok = false; break; }
                tc_fence_after_sync();
#ifdef B200_GEMM_TIMING
                { long long t1 = clock64(); t_acc += t1 - t0; t0 = t1; }
#endif
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(&full_bar[s], ph, abort_flag)) { ok = false; break; }
                    tc_fence_after_sync();
#ifdef B200_GEMM_TIMING
                    { long long t1 = clock64(); t_wait += t1 - t0; t0 = t1; if (it == 0) t_first = t1 - t_begin; }
#endif
                    const uint64_t a_desc = make_smem_desc_sw128(smem_u32(smem_a + s * Cfg::A_BYTES), 16, 1024);
                    const uint64_t b_desc = make_smem_desc_sw128(smem_u32(smem_b + s * Cfg::B_BYTES), 16, 1024);
#pragma unroll
                    for (int k = 0; k < BK / 8; ++k) {  // 32 bytes of K per instruction: 8 tf32 or 16 bf16
                        if (BF16) umma_f16_ss_pair(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0);
                        else umma_tf32_ss_pair(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0);
                    }
#ifdef B200_GEMM_TIMING
                    { long long t1 = clock64(); t_mma += t1 - t0; t0 = t1; }
#endif
                    // free the stage in both CTAs
                    const uint32_t e = smem_u32(&empty_bar[s]);
                    umma_commit_pair(map_to_cta(e, 0));
                    umma_commit_pair(map_to_cta(e, 1));
#ifdef B200_GEMM_TIMING
                    { long long t1 = clock64(); t_commit += t1 - t0; t0 = t1; }
#endif
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
#ifdef B200_GEMM_TIMING
            if (blockIdx.x == 0) {
                long long* dbg = reinterpret_cast<long long*>(args.status + 2);
                dbg[0] = t_wait; dbg[1] = t_mma; dbg[2] = t_commit; dbg[3] = t_acc; dbg[4] = it;
                dbg[5] = t_first; dbg[6] = clock64() - t_begin;
            }
#endif
        }
    } else {
        // ---------------------------------------------------------------- epilogue
        const int q = warp & 3;
        const int ew = warp - 2;  // 0..7
        // column split in units of one chunk (two for a bf16 output, whose stores take 64 columns)
        const int unit = args.out_h ? 2 : 1;
        const int n_units = BN / 32 / unit;
        const int c_begin = (ew < 4) ? 0 : ((n_units + 1) / 2) * unit;
        const int c_end = (ew < 4) ? ((n_units + 1) / 2) * unit : BN / 32;
        bool ok = true;
        int tile_iter = 0;
        for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++tile_iter) {
            int m_blk, n_blk;
            tile_coords(tile, m_blk, n_blk);
            const int acc = tile_iter & 1;
            const uint32_t acc_ph = (tile_iter >> 1) & 1;
            const float bias_first = gemm_bias_chunk(args, n_blk * BN, c_begin, lane);  // on its way while the tile is computed
            if (!mbar_wait(&tmem_full_bar[acc], acc_ph, abort_flag)) { ok = false; break; }
            tc_fence_after_sync();
            gemm_drain_accumulator<BN>(args, &tmap_out, tmem_base + acc * BN, q, lane,
                                       m_blk * 2 * BM + (int)rank * BM + q * 32, n_blk * BN,
                                       smem_epi + ew * 4096, bias_first, c_begin, c_end, 1);
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty_bar[acc]), 0));
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

// Estimated cycles of one 256 x BN pair tile (per CTA): per 32-deep K block the tensor pipe
// needs 2*BN cycles and the SM pulls about 52 bytes per cycle from L2.
inline long pair_tile_cost(int bn, int num_kb) {
    const long tensor = 2L * bn, feed = (128L + bn / 2) * 128 / 52;
    return num_kb * (tensor > feed ? tensor : feed) + 1500;
}

template <int BN, bool BF16>
int launch_pair(b200_ctx* ctx, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& to, GemmArgs& a,
                int num_pairs_max) {
    using Cfg = PairCfg<BN>;
    static_assert(!BF16 || BN % 64 == 0, "the bf16 epilogue stores 64 columns at a time");
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
        B200_CUDA(ctx, cudaFuncSetAttribute(gemm_tf32_pair_kernel<BN, BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM));
        cfg.gridDim = dim3(2 * num_pairs_max);
        int n = 0;
        B200_CUDA(ctx, cudaOccupancyMaxActiveClusters(&n, gemm_tf32_pair_kernel<BN, BF16>, &cfg));
        if (n < 1) n = 1;
        resident_pairs[ctx->device & 63] = n < num_pairs_max ? n : num_pairs_max;
        if (getenv("B200_GEMM_DEBUG")) fprintf(stderr, "gemm_tf32_pair_kernel<%d>: %d resident CTA pairs (occupancy query %d), %d stages\n", BN, resident_pairs[ctx->device & 63], n, Cfg::STAGES);
    }
    // persistent: never more pairs than can be resident together, or the rest would run as a tail
    const int tiles = a.num_m_blocks * a.num_n_blocks;
    const int pairs = tiles < resident_pairs[ctx->device & 63] ? tiles : resident_pairs[ctx->device & 63];
    cfg.gridDim = dim3(2 * pairs);
    B200_CUDA(ctx, cudaLaunchKernelEx(&cfg, gemm_tf32_pair_kernel<BN, BF16>, ta, tb, to, a));
    ctx->launches++;
    return B200_OK;
}

}  // namespace

int launch_gemm_tf32_pair(b200_ctx* ctx, float* out, const float* inp, const float* weight,
                          const float* bias, const float* residual, int M, int K, int N, int flags,
                          unsigned long long* argmax_keys, int argmax_cols, int bf16, uint16_t* out_h, int store_period) {
    const int num_pairs_max = ctx->num_sms / 2;
    const int num_m = (M + 2 * BM - 1) / (2 * BM);
    const int bke = bf16 ? kGemmBKH : BK;
    const int num_kb = (K + bke - 1) / bke;
    const int cands[4] = {256, 192, 128, 64};
    int best_bn = 256;
    long best_cost = -1;
    for (int i = 0; i < 4; ++i) {
        const int bn = cands[i];
        const long tiles = (long)num_m * ((N + bn - 1) / bn);
        const long waves = (tiles + num_pairs_max - 1) / num_pairs_max;
        const long cost = waves * pair_tile_cost(bn, num_kb);
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best_bn = bn; }
    }
    // tuning hook: B200_GEMM_BN=<64|128|192|256> forces the N tile
    static const int forced_bn = [] { const char* e = getenv("B200_GEMM_BN"); return e ? atoi(e) : 0; }();
    if (forced_bn == 64 || forced_bn == 128 || forced_bn == 192 || forced_bn == 256) best_bn = forced_bn;

    GemmArgs a;
    a.out = out; a.out_h = out_h; a.bias = bias; a.residual = residual;
    a.M = M; a.N = N; a.K = K;
    a.num_m_blocks = num_m;
    a.num_n_blocks = (N + best_bn - 1) / best_bn;
    // weight small enough to stay in L2: sweep N fastest so each inp tile is fetched once;
    // otherwise sweep M fastest so the (smaller) inp stays resident while weight streams
    a.n_fastest = ((size_t)N * K * (bf16 ? 2 : 4) <= (size_t)32 << 20) ? 1 : 0;
    a.flags = flags;
    a.status = ctx->d_status;
    a.argmax_keys = argmax_keys;
    a.argmax_cols = argmax_cols;
    a.store_period = store_period;

    CUtensorMap ta, tb, to;
    int st;
    if (bf16) {
        st = b200_get_tensor_map_bf16(ctx, &ta, inp, (uint64_t)M, (uint64_t)K, (uint64_t)K, BM, kGemmBKH);
        if (st != B200_OK) return st;
        st = b200_get_tensor_map_bf16(ctx, &tb, weight, (uint64_t)N, (uint64_t)K, (uint64_t)K, (uint32_t)(best_bn / 2), kGemmBKH);
        if (st != B200_OK) return st;
    } else {
        st = b200_get_tensor_map(ctx, &ta, inp, (uint64_t)M, (uint64_t)K, (uint64_t)K, BM, BK);
        if (st != B200_OK) return st;
        st = b200_get_tensor_map(ctx, &tb, weight, (uint64_t)N, (uint64_t)K, (uint64_t)K, (uint32_t)(best_bn / 2), BK);
        if (st != B200_OK) return st;
    }
    // the output in 32 x 32 boxes of fp32 (32 x 64 of bf16), for the epilogue's TMA stores
    if (out_h) st = b200_get_tensor_map_bf16(ctx, &to, out_h, (uint64_t)M, (uint64_t)N, (uint64_t)N, 32, 64);
    else st = b200_get_tensor_map(ctx, &to, out, (uint64_t)M, (uint64_t)N, (uint64_t)N, 32, 32);
    if (st != B200_OK) return st;
    if (bf16) {
        switch (best_bn) {
            case 256: return launch_pair<256, true>(ctx, ta, tb, to, a, num_pairs_max);
            case 192: return launch_pair<192, true>(ctx, ta, tb, to, a, num_pairs_max);
            case 128: return launch_pair<128, true>(ctx, ta, tb, to, a, num_pairs_max);
            default:  return launch_pair<64, true>(ctx, ta, tb, to, a, num_pairs_max);
        }
    }
    switch (best_bn) {
        case 256: return launch_pair<256, false>(ctx, ta, tb, to, a, num_pairs_max);
        case 192: return launch_pair<192, false>(ctx, ta, tb, to, a, num_pairs_max);
        case 128: return launch_pair<128, false>(ctx, ta, tb, to, a, num_pairs_max);
        default:  return launch_pair<64, false>(ctx, ta, tb, to, a, num_pairs_max);
    }
}

}  // namespace b200
