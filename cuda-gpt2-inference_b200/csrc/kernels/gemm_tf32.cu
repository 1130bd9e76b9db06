// out[M,N] = act(inp[M,K] . weight[N,K]^T + bias[N]) (+ residual[M,N]) on the 5th-generation
// tensor cores: tcgen05.mma kind::tf32, fp32 operand bits staged by TMA into 128-byte-swizzled
// shared memory, fp32 accumulators in tensor memory, bias / tanh-GELU / residual applied in the
// epilogue straight out of tensor memory.  One kernel replaces the reference's whole matmul
// family (kernels/matmul/1_matmul_tiling.cuh:5-73 is the math; 9_matmul_async_cg_tf32_gelu.cuh
// :13-275 the best variant, whose bias pre-load :57-84 and GELU epilogue :196-212 are the fused
// steps kept here) and its separate add_bias pass (2_matmul_cublas.cuh:7-32).
//
// Both operands are K-major as stored (inp rows and weight rows are K-contiguous), so no
// transposes are needed.
//
// CTA = 6 warps (10 in the 3xTF32 mode), persistent over output tiles of 128 x BN:
//   warp 0      TMA producer: per 32-wide K block one {32 x 128} box of inp and one {32 x BN}
//               box of weight into a ring of STAGES shared-memory stages (full/empty mbarriers)
//   warp 1      allocates tensor memory; one elected lane issues the UMMAs (K = 8 each) of a
//               stage and commits the stage's empty barrier; commits tmem_full after the last
//               K block
//   warps 2-5   epilogue: tcgen05.ld 32 lanes x 32 columns at a time, transposed through a
//               swizzled shared-memory buffer, bias/GELU/residual, row-contiguous float4
//               stores.  Two accumulators (2 x BN columns) let the epilogue of tile i overlap
//               the main loop of tile i+1.
//   warps 6-9   (3xTF32 only) split warps: the tensor core reads only the upper 19 bits of an
//               fp32 operand (it truncates), so for every staged tile they write the dropped
//               part  x_small = x - trunc_tf32(x)  into a second buffer, and the issuer
//               accumulates  A.B + A_small.B + A.B_small : fp32-level products on the TF32 pipe.
// Every wait is time-bounded; a wait that runs out makes all roles leave, the CTA frees its
// tensor memory and records a code in the context's status word.
#include <cstdlib>
#include "gemm_common.cuh"

namespace b200 {

namespace {

constexpr int BM = kGemmBM;
constexpr int BK = kGemmBK;
constexpr int kMaxSmem = kGemmMaxSmem;

template <int BN, bool X3>
struct GemmCfg {
    static constexpr int THREADS = X3 ? 320 : 192;
    static constexpr int A_BYTES = BM * BK * 4;
    static constexpr int B_BYTES = BN * BK * 4;
    static constexpr int STAGE_BYTES = (A_BYTES + B_BYTES) * (X3 ? 2 : 1);
    static constexpr int TX_BYTES = A_BYTES + B_BYTES;  // what TMA delivers per stage
    static constexpr int BAR_BYTES = 512;
    // epilogue staging (transposes the row-per-thread tensor-memory layout into row-contiguous,
    // coalesced global stores)
    static constexpr int EPI_BYTES = kGemmEpiBytes;
    static constexpr int STAGES_RAW = (kMaxSmem - 1024 - BAR_BYTES - EPI_BYTES) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
    static constexpr int SMEM = 1024 + STAGES * STAGE_BYTES + EPI_BYTES + BAR_BYTES;
    static constexpr int TMEM_COLS = (2 * BN <= 128) ? 128 : (2 * BN <= 256 ? 256 : 512);
    // one CTA per SM is guaranteed by shared memory (> half of the SM's), so a 512-column
    // allocation can never wait on a co-resident CTA
    static_assert(SMEM > 117 * 1024, "a second resident CTA could block in tcgen05.alloc");
    static_assert(SMEM <= kMaxSmem, "shared memory over the 227 KB limit");
    static_assert(BN % 32 == 0 && BN >= 32 && BN <= 256, "BN: multiple of 32 up to 256");
    static_assert(STAGES >= 2, "need at least a double buffer");
};

__device__ __forceinline__ float tf32_dropped_part(float x) {
    return x - __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
}

template <int BN, bool X3, bool BF16>
__global__ void __launch_bounds__(GemmCfg<BN, X3>::THREADS, 1)
gemm_tf32_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_out,
                 const GemmArgs args) {
    using Cfg = GemmCfg<BN, X3>;
    constexpr int STAGES = Cfg::STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* smem_a = smem;                                        // [STAGES][A_BYTES]
    uint8_t* smem_b = smem_a + STAGES * Cfg::A_BYTES;              // [STAGES][B_BYTES]
    uint8_t* smem_as = smem_b + STAGES * Cfg::B_BYTES;             // X3: dropped parts of A
    uint8_t* smem_bs = smem_as + (X3 ? STAGES * Cfg::A_BYTES : 0); // X3: dropped parts of B
    uint8_t* smem_epi = smem + STAGES * Cfg::STAGE_BYTES;          // [4 warps][2][32 x 128 B]
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_epi + Cfg::EPI_BYTES);
    uint64_t* full_bar = bars;                     // [STAGES] TMA landed
    uint64_t* empty_bar = bars + STAGES;           // [STAGES] UMMAs of the stage retired
    uint64_t* split_bar = bars + 2 * STAGES;       // [STAGES] X3: dropped parts written
    uint64_t* tmem_full_bar = bars + 3 * STAGES;   // [2]
    uint64_t* tmem_empty_bar = tmem_full_bar + 2;  // [2]
    uint64_t* drain_bar = tmem_empty_bar + 2;      // [1]
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(drain_bar + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int num_tiles = args.num_m_blocks * args.num_n_blocks;
    constexpr int BKE = BF16 ? kGemmBKH : BK;  // elements per 128-byte K block
    const int num_kb = (args.K + BKE - 1) / BKE;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
            mbar_init(&split_bar[s], 128);
        }
        for (int a = 0; a < 2; ++a) { mbar_init(&tmem_full_bar[a], 1); mbar_init(&tmem_empty_bar[a], 128); }
        mbar_init(drain_bar, 1);
        *abort_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_b);
        tma_prefetch_desc(&tmap_out);
    }
    if (warp == 1) {
        tmem_alloc(tmem_holder, Cfg::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
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
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                int m_blk, n_blk;
                tile_coords(tile, m_blk, n_blk);
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag)) { ok = false; break; }
                    mbar_arrive_expect_tx(&full_bar[s], Cfg::TX_BYTES);
                    tma_load_2d(smem_a + s * Cfg::A_BYTES, &tmap_a, kb * BKE, m_blk * BM, &full_bar[s]);
                    tma_load_2d(smem_b + s * Cfg::B_BYTES, &tmap_b, kb * BKE, n_blk * BN, &full_bar[s]);
                }
            }
            if (!ok) atomicCAS(args.status, 0, DEV_TIMEOUT_PRODUCER);
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = BF16 ? make_idesc_bf16(BM, BN, 0) : make_idesc_tf32(BM, BN, 0);
            uint32_t it = 0;
            bool ok = true;
            int tile_iter = 0;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tile_iter) {
                const int acc = tile_iter & 1;
                const uint32_t acc_ph = (tile_iter >> 1) & 1;
                if (!mbar_wait(&tmem_empty_bar[acc], acc_ph ^ 1, abort_flag)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    // in the 3xTF32 mode the split warps signal after the TMA data has landed
                    if (!mbar_wait(X3 ? &split_bar[s] : &full_bar[s], ph, abort_flag)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint64_t a_desc = make_smem_desc_sw128(smem_u32(smem_a + s * Cfg::A_BYTES), 16, 1024);
                    const uint64_t b_desc = make_smem_desc_sw128(smem_u32(smem_b + s * Cfg::B_BYTES), 16, 1024);
#pragma unroll
                    for (int k = 0; k < BK / 8; ++k) {
                        // advance 8 fp32 (16 bf16) = 32 bytes along K inside the swizzled row: +2 in
                        // the (address >> 4) field
                        if (BF16) umma_f16_ss(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0);
                        else umma_tf32_ss(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0);
                    }
                    if (X3) {
                        const uint64_t as_desc = make_smem_desc_sw128(smem_u32(smem_as + s * Cfg::A_BYTES), 16, 1024);
                        const uint64_t bs_desc = make_smem_desc_sw128(smem_u32(smem_bs + s * Cfg::B_BYTES), 16, 1024);
#pragma unroll
                        for (int k = 0; k < BK / 8; ++k) {
                            umma_tf32_ss(d_tmem, as_desc + 2 * k, b_desc + 2 * k, idesc, 1);
                            umma_tf32_ss(d_tmem, a_desc + 2 * k, bs_desc + 2 * k, idesc, 1);
                        }
                    }
                    umma_commit(&empty_bar[s]);
                }
                if (ok) umma_commit(&tmem_full_bar[acc]);
            }
            // wait (bounded) until everything issued has retired before tensor memory is freed
            umma_commit(drain_bar);
            if (!mbar_wait(drain_bar, 0, abort_flag)) ok = false;
            if (!ok) atomicCAS(args.status, 0, DEV_TIMEOUT_MMA);
        }
    } else if (warp < 6) {
        // ---------------------------------------------------------------- epilogue
        const int q = warp & 3;  // the lane quarter this warp may read
        bool ok = true;
        int tile_iter = 0;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tile_iter) {
            int m_blk, n_blk;
            tile_coords(tile, m_blk, n_blk);
            const int acc = tile_iter & 1;
            const uint32_t acc_ph = (tile_iter >> 1) & 1;
            const float bias_first = gemm_bias_chunk(args.bias, args.N, n_blk * BN, 0, lane);  // on its way while the tile is computed
            if (!mbar_wait(&tmem_full_bar[acc], acc_ph, abort_flag)) { ok = false; break; }
            tc_fence_after_sync();
            gemm_drain_accumulator(args, args.bias, &tmap_out, tmem_base + acc * BN, q, lane, m_blk * BM + q * 32, n_blk * BN,
                                   smem_epi + q * 2 * 4096, bias_first, 0, BN / 32, 2);
            tc_fence_before_sync();
            mbar_arrive(&tmem_empty_bar[acc]);
        }
        if (lane == 0) tma_store_wait_all();  // the staging buffers must outlive the stores reading them
        if (!ok && lane == 0) atomicCAS(args.status, 0, DEV_TIMEOUT_EPILOGUE);
    } else if (X3) {
        // ------------------------------------------------------- split warps (3xTF32)
        const int t = threadIdx.x - 192;  // 0..127
        uint32_t it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
            for (int kb = 0; kb < num_kb; ++kb, ++it) {
                const int s = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1;
                if (!mbar_wait(&full_bar[s], ph, abort_flag)) { ok = false; break; }
                // element-wise, so the swizzled placement carries over unchanged
                const float4* a_src = reinterpret_cast<const float4*>(smem_a + s * Cfg::A_BYTES);
                float4* a_dst = reinterpret_cast<float4*>(smem_as + s * Cfg::A_BYTES);
#pragma unroll
                for (int i = 0; i < Cfg::A_BYTES / 16 / 128; ++i) {
                    const float4 v = a_src[i * 128 + t];
                    a_dst[i * 128 + t] = make_float4(tf32_dropped_part(v.x), tf32_dropped_part(v.y),
                                                     tf32_dropped_part(v.z), tf32_dropped_part(v.w));
                }
                const float4* b_src = reinterpret_cast<const float4*>(smem_b + s * Cfg::B_BYTES);
                float4* b_dst = reinterpret_cast<float4*>(smem_bs + s * Cfg::B_BYTES);
#pragma unroll
                for (int i = 0; i < Cfg::B_BYTES / 16 / 128; ++i) {
                    const float4 v = b_src[i * 128 + t];
                    b_dst[i * 128 + t] = make_float4(tf32_dropped_part(v.x), tf32_dropped_part(v.y),
                                                     tf32_dropped_part(v.z), tf32_dropped_part(v.w));
                }
                fence_proxy_async_smem();
                mbar_arrive(&split_bar[s]);
            }
        }
        if (!ok && lane == 0) atomicCAS(args.status, 0, DEV_TIMEOUT_MMA);
    }

    griddep_launch_dependents();
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

// Estimated cycles of one 128 x BN output tile.  Per 32-deep K block the tensor pipe needs
// 2*BN cycles, but the SM can only pull about 52 bytes per cycle from L2 (measured: the five
// tile widths all saturate near 15 TB/s of L2->SM traffic), so a block costs
// max(2*BN, (128+BN)*128/52); plus the part of the epilogue that is not hidden.
inline long tile_cost(int bn, int num_kb) {
    const long tensor = 2L * bn, feed = (128L + bn) * 128 / 52;
    return num_kb * (tensor > feed ? tensor : feed) + 1500;
}

template <int BN, bool X3, bool BF16>
int launch_one(b200_ctx* ctx, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& to, GemmArgs& a) {
    using Cfg = GemmCfg<BN, X3>;
    static_assert(!BF16 || (BN % 64 == 0 && !X3), "the bf16 epilogue stores 64 columns at a time");
    static bool attr_set[64] = {};
    if (!attr_set[ctx->device & 63]) {
        B200_CUDA(ctx, cudaFuncSetAttribute(gemm_tf32_kernel<BN, X3, BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM));
        attr_set[ctx->device & 63] = true;
    }
    const int tiles = a.num_m_blocks * a.num_n_blocks;
    const int grid = tiles < ctx->num_sms ? tiles : ctx->num_sms;
    cudaError_t le = launch_pdl(ctx, gemm_tf32_kernel<BN, X3, BF16>, dim3(grid), dim3(Cfg::THREADS), Cfg::SMEM, ta, tb, to, a);
    ctx->launches++;
    B200_CUDA(ctx, le);
    return B200_OK;
}

}  // namespace

namespace {

// bf16 != 0: inp / weight hold bf16 elements and out_h (if not null) receives the output as bf16.
int launch_gemm_any(b200_ctx* ctx, float* out, uint16_t* out_h, const void* inp, const void* weight,
                    const float* bias, const float* residual, int M, int K, int N, int flags,
                    int mode, unsigned long long* argmax_keys, int argmax_cols, bool bf16, int store_period, const GemmRowStats* stats) {
    if ((flags & GEMM_ACCUM_OUT) && (residual || out_h)) { ctx->last_error = "GEMM_ACCUM_OUT: fp32 output without a residual operand"; return B200_ERR_STATE; }
    if (store_period && (store_period % 32 || residual || !argmax_keys)) { ctx->last_error = "store_period: multiple of 32, with the fused arg-max only"; return B200_ERR_STATE; }
    const bool x3 = (mode == B200_TF32X3);
    // the fused arg-max looks at the raw accumulator: only with a plain epilogue
    if (argmax_keys && (bias || residual || flags != 0 || out_h)) { ctx->last_error = "fused arg-max needs a plain GEMM epilogue"; return B200_ERR_STATE; }
    const int bke = bf16 ? kGemmBKH : BK;
    const int num_kb = (K + bke - 1) / bke;
    const int num_m = (M + BM - 1) / BM;
    // pick the N tile that minimises waves x per-tile cost on this GPU's SM count
    int best_bn = 128;
    long best_cost = -1;
    if (!x3) {
        const int cands[5] = {256, 192, 128, 96, 64};
        for (int i = 0; i < 5; ++i) {
            const int bn = cands[i];
            if (bf16 && bn % 64) continue;
            const long tiles = (long)num_m * ((N + bn - 1) / bn);
            const long waves = (tiles + ctx->num_sms - 1) / ctx->num_sms;
            const long cost = waves * tile_cost(bn, num_kb);
            if (best_cost < 0 || cost < best_cost) { best_cost = cost; best_bn = bn; }
        }
        // tuning hook: B200_GEMM_BN=<64|96|128|192|256> forces the N tile
        static const int forced_bn = [] { const char* e = getenv("B200_GEMM_BN"); return e ? atoi(e) : 0; }();
        if ((forced_bn == 64 || forced_bn == 96 || forced_bn == 128 || forced_bn == 192 || forced_bn == 256) && !(bf16 && forced_bn % 64)) best_bn = forced_bn;
    }
    // CTA pairs pull a third less operand traffic out of L2 per flop and drain the accumulator
    // with eight warps; measured inside the forward (124M and XL shapes, 8192 rows) they win
    // everywhere except the square attention projection (N = K = C: few, short tiles, where the
    // single-CTA kernel's finer N tiles quantise better).  With bf16 operands the tensor pipe
    // needs the same bytes in half the time, so the operand feed decides nearly everywhere and
    // pairs are used whenever there are whole pair tiles for every SM pair.
    // B200_GEMM_PAIR=0/1 forces the choice.
    static const int pair_env = [] { const char* e = getenv("B200_GEMM_PAIR"); return (e && (e[0] == '0' || e[0] == '1')) ? e[0] - '0' : -1; }();
    bool use_pair = M >= 2048 && (N >= 2048 || K >= 2048);
    if (bf16) use_pair = M >= 2048 && (long)((M + 255) / 256) * ((N + 255) / 256) >= ctx->num_sms / 2;
    if (pair_env >= 0) use_pair = pair_env == 1;
    if (stats) {  // the sampling / log-sum-exp epilogue lives in the CTA-pair kernel
        if (x3) { ctx->last_error = "row statistics are not available with 3xTF32 GEMMs"; return B200_ERR_STATE; }
        use_pair = true;
    }
    if (!x3 && use_pair)
        return launch_gemm_pair(ctx, out, inp, nullptr, weight, nullptr, bias, residual, M, K, N, flags, argmax_keys, argmax_cols,
                                bf16 ? PAIR_BF16 : PAIR_TF32, out_h, 0, store_period, stats);
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
    a.out_planes = 0;
    a.sample_inv_temp = 0.f;
    a.sample_seed = a.sample_stream0 = 0u;
    a.lse_part = nullptr;
    a.lse_slots = 0;
    a.tile_w = a.unit_cols = 0;
    a.k_splits = 1;
    a.split_flags = nullptr;
    a.tmap_out2 = static_cast<const CUtensorMap*>(ctx->next_gemm_out2);
    ctx->next_gemm_out2 = nullptr;
    a.out2_rows = a.tmap_out2 ? ctx->next_gemm_out2_rows : 0;
    ctx->next_gemm_out2_rows = 0;
    if (a.tmap_out2 && (out_h || residual || (flags & GEMM_ACCUM_OUT) || store_period || x3)) {
        ctx->last_error = "a second output needs a plain fp32 store epilogue";
        return B200_ERR_STATE;
    }

    CUtensorMap ta, tb, to;
    int st;
    if (bf16) {
        st = b200_get_tensor_map_bf16(ctx, &ta, inp, (uint64_t)M, (uint64_t)K, (uint64_t)K, BM, kGemmBKH);
        if (st != B200_OK) return st;
        st = b200_get_tensor_map_bf16(ctx, &tb, weight, (uint64_t)N, (uint64_t)K, (uint64_t)K, (uint32_t)best_bn, kGemmBKH);
        if (st != B200_OK) return st;
    } else {
        st = b200_get_tensor_map(ctx, &ta, static_cast<const float*>(inp), (uint64_t)M, (uint64_t)K, (uint64_t)K, BM, BK);
        if (st != B200_OK) return st;
        st = b200_get_tensor_map(ctx, &tb, static_cast<const float*>(weight), (uint64_t)N, (uint64_t)K, (uint64_t)K, (uint32_t)best_bn, BK);
        if (st != B200_OK) return st;
    }
    // the output in 32 x 32 boxes of fp32 (32 x 64 of bf16), for the epilogue's TMA stores
    if (out_h) st = b200_get_tensor_map_bf16(ctx, &to, out_h, (uint64_t)M, (uint64_t)N, (uint64_t)N, 32, 64);
    else st = b200_get_tensor_map(ctx, &to, out, (uint64_t)M, (uint64_t)N, (uint64_t)N, 32, 32);
    if (st != B200_OK) return st;
    if (bf16) {
        switch (best_bn) {
            case 256: return launch_one<256, false, true>(ctx, ta, tb, to, a);
            case 192: return launch_one<192, false, true>(ctx, ta, tb, to, a);
            case 128: return launch_one<128, false, true>(ctx, ta, tb, to, a);
            default:  return launch_one<64, false, true>(ctx, ta, tb, to, a);
        }
    }
    if (x3) return launch_one<128, true, false>(ctx, ta, tb, to, a);
    switch (best_bn) {
        case 256: return launch_one<256, false, false>(ctx, ta, tb, to, a);
        case 192: return launch_one<192, false, false>(ctx, ta, tb, to, a);
        case 128: return launch_one<128, false, false>(ctx, ta, tb, to, a);
        case 96:  return launch_one<96, false, false>(ctx, ta, tb, to, a);
        default:  return launch_one<64, false, false>(ctx, ta, tb, to, a);
    }
}

}  // namespace

namespace {
template <int BN>
int preload_one(b200_ctx* ctx) {
    B200_CUDA(ctx, cudaFuncSetAttribute(gemm_tf32_kernel<BN, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmCfg<BN, false>::SMEM));
    return B200_OK;
}
}  // namespace

// Loads the single-pass TF32 GEMM kernels (every tile width) now rather than at their first launch.
int preload_gemm_kernels(b200_ctx* ctx) {
    int st = preload_one<256>(ctx);
    if (st == B200_OK) st = preload_one<192>(ctx);
    if (st == B200_OK) st = preload_one<128>(ctx);
    if (st == B200_OK) st = preload_one<96>(ctx);
    if (st == B200_OK) st = preload_one<64>(ctx);
    if (st == B200_OK) st = preload_gemm_pair_kernels(ctx);
    return st;
}

int launch_gemm_tf32(b200_ctx* ctx, float* out, const float* inp, const float* weight,
                     const float* bias, const float* residual, int M, int K, int N, int flags,
                     int mode, unsigned long long* argmax_keys, int argmax_cols, int store_period, const GemmRowStats* stats) {
    return launch_gemm_any(ctx, out, nullptr, inp, weight, bias, residual, M, K, N, flags, mode, argmax_keys, argmax_cols, false, store_period, stats);
}

int launch_gemm_bf16x3(b200_ctx* ctx, float* out, uint16_t* out_planes, const uint16_t* inp, const uint16_t* weight_hi,
                       const uint16_t* weight_lo, const float* bias, int M, int K, int N, int flags,
                       unsigned long long* argmax_keys, int argmax_cols, int store_period, const GemmRowStats* stats, int lo_col0) {
    if (K % 8 || N % 8) { ctx->last_error = "bf16x3 GEMM: K and N must be multiples of 8"; return B200_ERR_SHAPE; }
    if (out_planes && (M % 32 || (flags & GEMM_ACCUM_OUT))) { ctx->last_error = "bf16x3 GEMM: a split output needs M % 32 == 0 and no accumulation"; return B200_ERR_SHAPE; }
    if (store_period && (store_period % 32 || !argmax_keys)) { ctx->last_error = "store_period: multiple of 32, with the fused arg-max only"; return B200_ERR_STATE; }
    if (argmax_keys && (bias || flags != 0 || out_planes)) { ctx->last_error = "fused arg-max needs a plain GEMM epilogue"; return B200_ERR_STATE; }
    if (!out_planes && !out) return B200_ERR_NULL;
    return launch_gemm_pair(ctx, out, inp, inp + (size_t)M * K, weight_hi, weight_lo, bias, nullptr, M, K, N,
                            flags & (GEMM_GELU | GEMM_ROUND_OUT_TF32 | GEMM_ACCUM_OUT), argmax_keys, argmax_cols, PAIR_BF16X3, out_planes,
                            out_planes ? ((flags & GEMM_PLANES_FP16) ? 2 : 1) : 0, store_period, stats, 1.0f, lo_col0);
}

int launch_gemm_bf16(b200_ctx* ctx, float* out, uint16_t* out_h, const uint16_t* inp, const uint16_t* weight,
                     const float* bias, int M, int K, int N, int flags,
                     unsigned long long* argmax_keys, int argmax_cols, int store_period) {
    if (K % 8 || N % 8) { ctx->last_error = "bf16 GEMM: K and N must be multiples of 8"; return B200_ERR_SHAPE; }
    return launch_gemm_any(ctx, out, out_h, inp, weight, bias, nullptr, M, K, N, flags & (GEMM_GELU | GEMM_ROUND_OUT_TF32 | GEMM_ACCUM_OUT), B200_TF32, argmax_keys, argmax_cols, true, store_period, nullptr);
}

// e4m3 operands: always on CTA pairs (the kernel clips ragged edges itself)
int launch_gemm_fp8(b200_ctx* ctx, float* out, const uint8_t* inp, const uint8_t* weight, const float* bias,
                    int M, int K, int N, int flags, float alpha) {
    if (K % 16 || N % 8) { ctx->last_error = "fp8 GEMM: K must be a multiple of 16 and N of 8"; return B200_ERR_SHAPE; }
    return launch_gemm_pair(ctx, out, inp, nullptr, weight, nullptr, bias, nullptr, M, K, N, flags & (GEMM_GELU | GEMM_ACCUM_OUT),
                            nullptr, 0, PAIR_FP8, nullptr, 0, 0, nullptr, alpha);
}

}  // namespace b200
