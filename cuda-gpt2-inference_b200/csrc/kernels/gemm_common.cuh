// Pieces shared by the single-CTA and the CTA-pair TF32 GEMM kernels: the argument block and
// the epilogue that drains one 128 x BN accumulator out of tensor memory.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "kernels.h"
#include "../prim/sm100.cuh"

namespace b200 {

constexpr int kGemmBM = 128;       // accumulator rows per CTA (tensor-memory lanes)
constexpr int kGemmBK = 32;        // fp32 elements per K block = 128 bytes = one swizzle row
constexpr int kGemmBKH = 64;       // bf16 elements per K block: the same 128 bytes
constexpr int kGemmBKQ = 128;      // 8-bit elements per K block
constexpr int kGemmMaxSmem = 232448;  // 227 KB
constexpr int kGemmEpiBytes = 4 * 2 * 4096;  // per epilogue warp two {32 rows x 128 B} buffers

struct GemmArgs {
    float* out;
    uint16_t* out_h;  // not null: the output is written as bf16 here instead (plain / bias / GELU epilogue only)
    const float* bias;
    const float* residual;
    int M, N, K;
    int num_m_blocks, num_n_blocks;  // tiles along M (of 128, or 256 for CTA pairs) and N
    int n_fastest;
    int flags;
    int* status;
    // optional fused arg-max over columns [0, argmax_cols) of every output row (null: off);
    // only for a plain epilogue (no bias, activation, residual or rounding)
    unsigned long long* argmax_keys;
    int argmax_cols;
    // > 0: rows come in sequences of store_period (a multiple of 32) and only the 32-row blocks that
    // hold a sequence's last row are written; the rest of the output is wanted as arg-max only
    int store_period;
    // with argmax_keys (CTA-pair kernel): sample_inv_temp > 0 turns the arg-max into a draw (see
    // GemmRowStats); lse_part receives the log-sum-exp partials of every row
    float sample_inv_temp;
    unsigned int sample_seed, sample_stream0;
    float2* lse_part;
    int lse_slots;
    // out_h only: it holds two 16-bit planes of [M,N], the value rounded to bf16 (1) or to fp16 (2:
    // clamped to the fp16 range first) and, M rows further down, what that rounding dropped in the
    // same format: the split operands of a bf16x3 product / of the fp16 attention
    int out_planes;
    // CTA-pair kernel: tiles of 256 rows x tile_w columns (a ragged last one narrower, in whole units
    // of unit_cols), K cut into k_splits slices that are tiles of their own; see gemm_tf32_pair.cu
    int tile_w, unit_cols, k_splits;
    unsigned int* split_flags;   // per (K slice, tile, CTA, epilogue warp): set once its sums are in the output, cleared by its reader
    float alpha = 1.0f;          // the accumulator is multiplied by this before the epilogue (fp8 operands: undoes their scales)
    // not null: a tensor map in global memory (same shape and 32 x 32 box as the output's) through which every
    // tile of a plain-store fp32 epilogue is stored a second time - into a peer GPU's memory (tensor parallel)
    const CUtensorMap* tmap_out2 = nullptr;
    // > 0: tmap_out2 is an array of maps, one per owner of out2_rows consecutive output rows (each over that owner's
    // buffer of out2_rows rows); a tile is stored ONLY through the map of the owner of its rows, not through tmap_out
    int out2_rows = 0;
    // two-plane output: the plane of the dropped parts is only written for columns >= lo_col0 (the fp16 attention
    // reads q and k from their hi planes alone: their lo planes need neither be formed nor stored)
    int lo_col0 = 0;
    // CTA-pair kernel, tail of the tile sequence: the tiles from number n_main on - what is left over after
    // the last full round of the resident pairs - are each computed as tail_sub tiles of tile_w / tail_sub
    // columns, so that the partly empty last round costs a fraction of a tile's time (1: off)
    int tail_sub = 1, n_main = 0;
};

// Arg-max keys: the value as an order-preserving 32-bit integer in the high half, the inverted
// column in the low half, so that an unsigned 64-bit maximum picks the largest value and, among
// equal values, the lowest column.  Keys start at zero (below every real value).
__device__ __forceinline__ uint32_t argmax_enc(float f) {
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float argmax_dec(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k ^ 0x80000000u) : ~k);
}

// One epilogue warp drains its 32 lanes x BN columns.  Thread `lane` holds row (q*32 + lane) of
// the accumulator, 32 columns at a time.  Writing that straight to global memory would scatter
// 16-byte pieces over 32 rows per instruction, so each chunk goes through a swizzled
// shared-memory buffer and comes back with 8 lanes covering 128 contiguous bytes of one row;
// bias, tanh-GELU, residual add and TF32 rounding are applied on the way out.
// Without a residual the chunk does not come back at all: bias / GELU / rounding are applied in
// registers, the buffer is filled in the 128-byte-swizzled layout and one lane sends it off as
// a 32 x 32 TMA store (which also clips at the edges of the matrix).
//   tmem_acc : tensor-memory address of the accumulator (column offset included, lane 0)
//   row0     : global row of accumulator lane q*32
//   col0     : global column of accumulator column 0
//   stage2   : this warp's nbuf (1, 2 or 4) staging buffers of 4 KB
//   c_begin, c_end : the 32-column chunks of the accumulator this warp drains (two warps can share
//                    a lane quarter and split the columns; with a bf16 output c_begin is even)
// The bias of a 32-column chunk: lane l fetches column l's (one coalesced 128-byte load per warp)
// and the others get it by shuffle.  Fetched one chunk ahead - the first one by the caller, before
// it waits for the accumulator - so that no chunk waits for an L2 round trip.
__device__ __forceinline__ float gemm_bias_chunk(const float* bias, int N, int col0, int c, int lane) {
    const int col = col0 + c * 32 + lane;
    return (bias && col < N) ? __ldg(bias + col) : 0.f;
}

// The same for a bf16 output (no arg-max, no residual): 64 columns x 2 bytes fill one 128-byte row,
// so the accumulator is drained two 32-column chunks at a time and every such unit leaves as one
// {32 rows x 64 columns} TMA store.  With out_planes the unit is stored twice: the values rounded to
// bf16 into the first plane and, through the same staging buffer once that store has read it, what
// the rounding dropped (as bf16) into the second plane M rows further down.  c_begin, c_end even.
__device__ __forceinline__ void gemm_drain_accumulator_bf16(const GemmArgs& args, const float* bias, const CUtensorMap* tmap_out, uint32_t tmem_acc,
                                                            int q, int lane, int row0, int col0, uint8_t* stage2, float bias_first,
                                                            int c_begin, int c_end, int nbuf) {
    const bool do_gelu = (args.flags & GEMM_GELU) != 0;
    const bool planes = args.out_planes != 0;
    if (lane == 0) tma_store_wait_read();  // the stores of the previous tile have left the staging buffers
    __syncwarp();
    float bias0 = bias_first;
#pragma unroll 1
    for (int c = c_begin; c < c_end; c += 2) {
        const int ui = (c - c_begin) >> 1;
        const int cbase = col0 + c * 32;
        const float bias1 = gemm_bias_chunk(bias, args.N, col0, c + 1, lane);
        uint32_t r0[32], r1[32];
        tmem_ld_32x32b_x32(tmem_acc + (uint32_t(q * 32) << 16) + c * 32, r0);
        tmem_ld_32x32b_x32(tmem_acc + (uint32_t(q * 32) << 16) + c * 32 + 32, r1);
        tmem_ld_wait();
        if (args.alpha != 1.0f) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                r0[i] = __float_as_uint(__uint_as_float(r0[i]) * args.alpha);
                r1[i] = __float_as_uint(__uint_as_float(r1[i]) * args.alpha);
            }
        }
        // buffers: without planes unit ui uses buffer ui mod nbuf; with planes its two stores use buffers
        // 2ui and 2ui + 1 mod nbuf (one and the same buffer when there is only one)
        const int bi = planes ? 2 * ui : ui;
        uint8_t* sth = stage2 + (bi & (nbuf - 1)) * 4096;
        uint8_t* stl = stage2 + ((bi + 1) & (nbuf - 1)) * 4096;
        if (bi >= nbuf) {  // the store that last used this buffer has read it
            if (lane == 0) { if (!planes && nbuf == 2) tma_store_wait_read_but_one(); else tma_store_wait_read(); }
            __syncwarp();
        }
        uint32_t lo[32];  // the dropped parts, packed two to a register (planes only)
        const bool want_lo = planes && cbase >= args.lo_col0;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float v[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(h ? r1[8 * j + i] : r0[8 * j + i]);
                if (bias) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) v[i] += __shfl_sync(0xffffffffu, h ? bias1 : bias0, 8 * j + i);
                }
                if (do_gelu) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) v[i] = gelu_tanh(v[i]);
                }
                uint32_t pk[4];
                if (args.out_planes == 2) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float x0 = fminf(fmaxf(v[2 * i], -65504.f), 65504.f), x1 = fminf(fmaxf(v[2 * i + 1], -65504.f), 65504.f);
                        const __half2 hh = __floats2half2_rn(x0, x1);
                        pk[i] = *reinterpret_cast<const uint32_t*>(&hh);
                        if (want_lo) {
                            const __half2 ll = __floats2half2_rn(x0 - __low2float(hh), x1 - __high2float(hh));
                            lo[h * 16 + j * 4 + i] = *reinterpret_cast<const uint32_t*>(&ll);
                        }
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const __nv_bfloat162 hh = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                        pk[i] = *reinterpret_cast<const uint32_t*>(&hh);
                        if (want_lo) {
                            const __nv_bfloat162 ll = __floats2bfloat162_rn(v[2 * i] - __low2float(hh), v[2 * i + 1] - __high2float(hh));
                            lo[h * 16 + j * 4 + i] = *reinterpret_cast<const uint32_t*>(&ll);
                        }
                    }
                }
                const int chunk = h * 4 + j;
                *reinterpret_cast<uint4*>(sth + lane * 128 + ((chunk ^ (lane & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            }
        }
        fence_proxy_async_smem();
        __syncwarp();
        const bool in_range = cbase < args.N && row0 < args.M;
        if (lane == 0 && in_range) {
            tma_store_2d(tmap_out, cbase, row0, sth);
            tma_store_commit();
        }
        if (want_lo) {
            if (bi + 1 >= nbuf) {  // with one buffer: the store just issued has to have read it
                if (lane == 0) tma_store_wait_read();
                __syncwarp();
            }
#pragma unroll
            for (int chunk = 0; chunk < 8; ++chunk)
                *reinterpret_cast<uint4*>(stl + lane * 128 + ((chunk ^ (lane & 7)) << 4)) =
                    make_uint4(lo[4 * chunk], lo[4 * chunk + 1], lo[4 * chunk + 2], lo[4 * chunk + 3]);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0 && in_range) {
                tma_store_2d(tmap_out, cbase, args.M + row0, stl);
                tma_store_commit();
            }
        }
        bias0 = (c + 2 < c_end) ? gemm_bias_chunk(bias, args.N, col0, c + 2, lane) : 0.f;
    }
}

//   bias_first : gemm_bias_chunk(bias, args.N, col0, c_begin, lane)
__device__ __forceinline__ void gemm_drain_accumulator(const GemmArgs& args, const float* bias, const CUtensorMap* tmap_out, uint32_t tmem_acc,
                                                       int q, int lane, int row0, int col0, uint8_t* stage2, float bias_first,
                                                       int c_begin, int c_end, int nbuf, int lse_slot = 0) {
    const bool do_gelu = (args.flags & GEMM_GELU) != 0;
    const bool do_round = (args.flags & GEMM_ROUND_OUT_TF32) != 0;
    const int sub_row = lane >> 3;  // 0..3: row within a group of four
    const int sub_chk = lane & 7;   // 16-byte chunk within the 128-byte row piece
    // Fused arg-max: this thread owns one row of the tile.  It starts from the row's best key so
    // far (other tiles of the row may have been finished by other CTAs; a stale value only costs
    // a needless update), filters each 32-column chunk by its maximum, and looks for the column
    // only in the rare chunk that beats the best - a handful of times per row over a whole GEMM.
    const bool do_argmax = args.argmax_keys != nullptr;
    const int my_row = row0 + lane;
    unsigned long long best_key = 0ull;
    float best_v = -INFINITY;
    bool improved = false;
    if (do_argmax && my_row < args.M) {
        best_key = args.argmax_keys[my_row];
        if (best_key != 0ull) best_v = argmax_dec((uint32_t)(best_key >> 32));
    }
    const bool do_sample = do_argmax && args.sample_inv_temp > 0.f;
    const bool do_lse = do_argmax && args.lse_part != nullptr;
    float lse_m = -INFINITY, lse_s = 0.f;  // running maximum and sum of exp(value - maximum) of this thread's columns
    const bool via_tma = args.residual == nullptr;
    if (args.tmap_out2 && lane == 0 && row0 < args.M) tma_acquire_global_desc(args.tmap_out2 + (args.out2_rows > 0 ? row0 / args.out2_rows : 0));  // once per tile and warp: cheap next to the tile
    const bool skip_store = args.store_period > 0 && (row0 % args.store_period) < args.store_period - 32;
    if (via_tma) {  // the stores of the previous tile have left the staging buffers
        if (lane == 0) tma_store_wait_read();
        __syncwarp();
    }
    if (args.out_h) {
        gemm_drain_accumulator_bf16(args, bias, tmap_out, tmem_acc, q, lane, row0, col0, stage2, bias_first, c_begin, c_end, nbuf);
        return;
    }
    float bias_next = bias_first;
#pragma unroll 1
    for (int c = c_begin; c < c_end; ++c) {
        const int ci = c - c_begin;
        const float bias_cur = bias_next;
        if (c + 1 < c_end) bias_next = gemm_bias_chunk(bias, args.N, col0, c + 1, lane);
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_acc + (uint32_t(q * 32) << 16) + c * 32, r);
        tmem_ld_wait();
        if (args.alpha != 1.0f) {
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * args.alpha);
        }
        if (do_lse) {
            const int cbase = col0 + c * 32;
            float cm = -INFINITY;
#pragma unroll
            for (int i = 0; i < 32; ++i) cm = fmaxf(cm, cbase + i < args.argmax_cols ? __uint_as_float(r[i]) : -INFINITY);
            if (cm > -INFINITY) {
                const float mn = fmaxf(lse_m, cm);
                float sum = 0.f;
#pragma unroll
                for (int i = 0; i < 32; ++i) sum += cbase + i < args.argmax_cols ? __expf(__uint_as_float(r[i]) - mn) : 0.f;
                lse_s = lse_s * __expf(lse_m - mn) + sum;  // exp(-inf) = 0 on the first chunk
                lse_m = mn;
            }
        }
        if (do_sample) {
            const int cbase = col0 + c * 32;
            if (cbase < args.argmax_cols && my_row < args.M) {
#pragma unroll 8
                for (int i = 0; i < 32; ++i) {
                    const float sc = sample_score(__uint_as_float(r[i]), args.sample_inv_temp, args.sample_seed,
                                                  args.sample_stream0 + (uint32_t)my_row, (uint32_t)(cbase + i));
                    const unsigned long long key = ((unsigned long long)argmax_enc(sc) << 32) | (0xFFFFFFFFu - (uint32_t)(cbase + i));
                    if (cbase + i < args.argmax_cols && key > best_key) { best_key = key; improved = true; }
                }
            }
        } else if (do_argmax) {
            const int cbase = col0 + c * 32;
            float cm = -INFINITY;  // chunk maximum (columns beyond the limit count too: only a filter)
#pragma unroll
            for (int i = 0; i < 32; i += 4)
                cm = fmaxf(cm, fmaxf(fmaxf(__uint_as_float(r[i]), __uint_as_float(r[i + 1])),
                                     fmaxf(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]))));
            if (cm >= best_v && cbase < args.argmax_cols) {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const unsigned long long key =
                        ((unsigned long long)argmax_enc(__uint_as_float(r[i])) << 32) | (0xFFFFFFFFu - (uint32_t)(cbase + i));
                    if (cbase + i < args.argmax_cols && key > best_key) { best_key = key; improved = true; }
                }
                best_v = argmax_dec((uint32_t)(best_key >> 32));
            }
        }
        if (skip_store) continue;
        uint8_t* stage = stage2 + (ci & (nbuf - 1)) * 4096;
        if (via_tma) {
            const int cbase = col0 + c * 32;
            if (ci >= nbuf) {  // the store that last used this buffer has read it
                if (lane == 0) { if (nbuf == 4) tma_store_wait_read_but_three(); else if (nbuf == 2) tma_store_wait_read_but_one(); else tma_store_wait_read(); }
                __syncwarp();
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                float4 v = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                       __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                if (bias) {
                    v.x += __shfl_sync(0xffffffffu, bias_cur, 4 * j);
                    v.y += __shfl_sync(0xffffffffu, bias_cur, 4 * j + 1);
                    v.z += __shfl_sync(0xffffffffu, bias_cur, 4 * j + 2);
                    v.w += __shfl_sync(0xffffffffu, bias_cur, 4 * j + 3);
                }
                if (do_gelu) { v.x = gelu_tanh(v.x); v.y = gelu_tanh(v.y); v.z = gelu_tanh(v.z); v.w = gelu_tanh(v.w); }
                if (do_round) { v.x = round_tf32(v.x); v.y = round_tf32(v.y); v.z = round_tf32(v.z); v.w = round_tf32(v.w); }
                *reinterpret_cast<float4*>(stage + lane * 128 + ((j ^ (lane & 7)) << 4)) = v;
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0 && cbase < args.N && row0 < args.M) {
                if (args.out2_rows > 0) {
                    tma_store_2d(args.tmap_out2 + row0 / args.out2_rows, cbase, row0 % args.out2_rows, stage);
                } else {
                    if (args.flags & GEMM_ACCUM_OUT) tma_reduce_add_2d(tmap_out, cbase, row0, stage);
                    else tma_store_2d(tmap_out, cbase, row0, stage);
                    if (args.tmap_out2) tma_store_2d(args.tmap_out2, cbase, row0, stage);
                }
                tma_store_commit();
            }
            continue;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            *reinterpret_cast<uint4*>(stage + lane * 128 + ((j ^ (lane & 7)) << 4)) =
                make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
        }
        __syncwarp();
        const int col = col0 + c * 32 + sub_chk * 4;
        if (col < args.N) {
            float4 b4 = make_float4(0.f, 0.f, 0.f, 0.f);
            if (bias) b4 = __ldg(reinterpret_cast<const float4*>(bias + col));
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int rl = i * 4 + sub_row;
                const int row = row0 + rl;
                float4 v = *reinterpret_cast<const float4*>(stage + rl * 128 + ((sub_chk ^ (rl & 7)) << 4));
                if (row < args.M) {
                    v.x += b4.x; v.y += b4.y; v.z += b4.z; v.w += b4.w;
                    if (do_gelu) { v.x = gelu_tanh(v.x); v.y = gelu_tanh(v.y); v.z = gelu_tanh(v.z); v.w = gelu_tanh(v.w); }
                    if (args.residual) {
                        const float4 rr = *reinterpret_cast<const float4*>(args.residual + (size_t)row * args.N + col);
                        v.x += rr.x; v.y += rr.y; v.z += rr.z; v.w += rr.w;
                    }
                    if (do_round) { v.x = round_tf32(v.x); v.y = round_tf32(v.y); v.z = round_tf32(v.z); v.w = round_tf32(v.w); }
                    *reinterpret_cast<float4*>(args.out + (size_t)row * args.N + col) = v;
                }
            }
        }
        // the buffer used two chunks ago is free again once every lane is past this point
        __syncwarp();
    }
    if (do_argmax && improved && my_row < args.M) atomicMax(args.argmax_keys + my_row, best_key);
    if (do_lse && my_row < args.M) args.lse_part[(size_t)my_row * args.lse_slots + lse_slot] = make_float2(lse_m, lse_s);
}

// CTA-pair GEMM (gemm_tf32_pair.cu): 256-row tiles computed by two CTAs sharing one UMMA.
// kind: PAIR_TF32 = fp32 operands (TF32 product); PAIR_BF16 = bf16 operands; PAIR_BF16X3 = split bf16
// operands: inp / weight address the first (hi) plane, inp_lo / weight_lo the second.  out_h as in
// GemmArgs (out_planes: M must be a multiple of 32).
enum : int { PAIR_TF32 = 0, PAIR_BF16 = 1, PAIR_BF16X3 = 2, PAIR_FP8 = 3 };  // PAIR_FP8: e4m3 operands (kind::f8f6f4)
int preload_gemm_pair_kernels(b200_ctx* ctx);  // the PAIR_TF32 kernel: loaded now, not at its first launch
int launch_gemm_pair(b200_ctx* ctx, float* out, const void* inp, const void* inp_lo, const void* weight, const void* weight_lo,
                     const float* bias, const float* residual, int M, int K, int N, int flags,
                     unsigned long long* argmax_keys, int argmax_cols, int kind, uint16_t* out_h = nullptr,
                     int out_planes = 0, int store_period = 0, const GemmRowStats* stats = nullptr, float alpha = 1.0f, int lo_col0 = 0);

}  // namespace b200
