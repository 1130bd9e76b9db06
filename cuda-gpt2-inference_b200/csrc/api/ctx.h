// Internal definition of the context behind the C ABI (include/b200gpt2.h).
#pragma once
#include <cstdint>
#include <string>
#include <unordered_map>
#include <cuda.h>
#include <cuda_runtime.h>
#include "../../../include/b200gpt2.h"

typedef CUresult (*b200_encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                         const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                         const cuuint32_t*, CUtensorMapInterleave,
                                         CUtensorMapSwizzle, CUtensorMapL2promotion,
                                         CUtensorMapFloatOOBfill);

struct TensorMapKey {
    const void* ptr;
    uint64_t rows, cols, ld;
    uint32_t box_rows, box_cols;
    int swizzle;
    bool operator==(const TensorMapKey& o) const {
        return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld &&
               box_rows == o.box_rows && box_cols == o.box_cols && swizzle == o.swizzle;
    }
};
struct TensorMapKeyHash {
    size_t operator()(const TensorMapKey& k) const {
        uint64_t h = reinterpret_cast<uint64_t>(k.ptr) * 0x9E3779B97F4A7C15ull;
        h ^= (k.rows + 0x7F4A7C15ull) * 0xBF58476D1CE4E5B9ull;
        h ^= (k.cols << 20) ^ (k.ld << 40) ^ (uint64_t(k.box_rows) << 8) ^ k.box_cols ^ (uint64_t(k.swizzle) << 60);
        return static_cast<size_t>(h ^ (h >> 29));
    }
};

struct b200_ctx {
    int device = 0;
    int num_sms = 148;
    cudaStream_t stream = nullptr;
    int* d_status = nullptr;  // device word: first device-side error code of any kernel
    int* h_status = nullptr;  // pinned host copy of that word, filled by b200_ctx_sync_check
    // CTA-pair GEMM with K slices: one flag word per (slice, tile, CTA, epilogue warp); all zero between launches
    unsigned int* d_split_flags = nullptr;
    // one-shot: device address of a CUtensorMap; the next fp32 plain-store GEMM launch on this context also stores
    // its output tiles through it (into a peer GPU's memory) and clears the field
    const void* next_gemm_out2 = nullptr;
    int next_gemm_out2_rows = 0;  // > 0 with it: an array of maps by owner of that many rows, and the only store (GemmArgs::out2_rows)
    size_t split_flag_words = 0;
    uint64_t launches = 0;
    bool pdl = true;  // launch with programmatic stream serialization (B200_PDL=0 turns it off)
    std::string last_error;
    b200_encode_tiled_fn encode_tiled = nullptr;
    std::unordered_map<TensorMapKey, CUtensorMap, TensorMapKeyHash> tmap_cache;
};

// Records a failing CUDA call on the context and returns B200_ERR_CUDA.
int b200_fail_cuda(b200_ctx* ctx, cudaError_t e, const char* what);
#define B200_CUDA(ctx, call)                                              \
    do {                                                                  \
        cudaError_t e__ = (call);                                         \
        if (e__ != cudaSuccess) return b200_fail_cuda((ctx), e__, #call); \
    } while (0)

// Tiled fp32 2-D tensor map over a row-major [rows, cols] matrix with leading dimension ld
// (elements), box = box_rows x box_cols, zero fill outside the matrix.  swizzle_atom32 == 0:
// 128-byte swizzle of 16-byte chunks (K-major UMMA operands); != 0: 128-byte swizzle of 32-byte
// chunks (the only layout the tensor core accepts for an MN-major TF32 operand).
// Cached per context.  Returns B200_OK or an error status.
int b200_get_tensor_map(b200_ctx* ctx, CUtensorMap* out, const float* ptr, uint64_t rows,
                        uint64_t cols, uint64_t ld, uint32_t box_rows, uint32_t box_cols,
                        int swizzle_atom32 = 0);

// The same over a matrix of bf16 (16-bit) elements: 128-byte swizzle of 16-byte chunks.
int b200_get_tensor_map_bf16(b200_ctx* ctx, CUtensorMap* out, const void* ptr, uint64_t rows,
                             uint64_t cols, uint64_t ld, uint32_t box_rows, uint32_t box_cols);

// The same over a matrix of 8-bit elements (e4m3 operands of the fp8 GEMM).
int b200_get_tensor_map_u8(b200_ctx* ctx, CUtensorMap* out, const void* ptr, uint64_t rows,
                           uint64_t cols, uint64_t ld, uint32_t box_rows, uint32_t box_cols);

// Makes the context's device current for the lifetime of the guard (streams, events and launches
// belong to a device) and puts the caller's device back afterwards.
struct b200_device_guard {
    int prev = -1;
    bool switched = false;
    explicit b200_device_guard(const b200_ctx* ctx) {
        if (cudaGetDevice(&prev) == cudaSuccess && prev != ctx->device) switched = cudaSetDevice(ctx->device) == cudaSuccess;
    }
    ~b200_device_guard() { if (switched) cudaSetDevice(prev); }
    b200_device_guard(const b200_device_guard&) = delete;
    b200_device_guard& operator=(const b200_device_guard&) = delete;
};

inline bool b200_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
