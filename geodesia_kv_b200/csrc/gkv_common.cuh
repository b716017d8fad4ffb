// Shared device/host helpers of the packed-KV kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "../../include/geodesia_kv_b200.h"

namespace gkv {

constexpr int kP = 64;        // tokens per block (the only block size the format defines)
constexpr int kMaxD = 256;    // largest head dim accepted (the reference's MAX_D)
constexpr int kNumSM = 148;   // B200

extern int g_last_cuda_error;

inline int cuda_fail(cudaError_t e) {
    g_last_cuda_error = (int)e;
    return GKV_E_CUDA;
}

#define GKV_CUDA_TRY(expr)                                    \
    do {                                                      \
        cudaError_t _e = (expr);                              \
        if (_e != cudaSuccess) return ::gkv::cuda_fail(_e);   \
    } while (0)

#define GKV_LAUNCH_CHECK()                                    \
    do {                                                      \
        cudaError_t _e = cudaGetLastError();                  \
        if (_e != cudaSuccess) return ::gkv::cuda_fail(_e);   \
    } while (0)

// Bytes of the K (or V) half of one block at a rung.
__host__ __device__ __forceinline__ int half_bytes(int level, int D) {
    return level == 1 ? D * 2 : level == 16 ? kP * D * 2 : (kP * D * level) / 8;
}

__host__ __device__ __forceinline__ bool level_ok(int level) {
    return level == 16 || level == 8 || level == 4 || level == 2 || level == 1;
}

// Ladder index 0..4 for rungs 16, 8, 4, 2, 1.
__host__ __device__ __forceinline__ int ladder_index(int level) {
    return level == 16 ? 0 : level == 8 ? 1 : level == 4 ? 2 : level == 2 ? 3 : 4;
}
__host__ __device__ __forceinline__ int ladder_level(int idx) {
    return idx == 0 ? 16 : idx == 1 ? 8 : idx == 2 ? 4 : idx == 3 ? 2 : 1;
}

__device__ __forceinline__ float bf16_bits_to_float(uint32_t b) { return __uint_as_float(b << 16); }

__device__ __forceinline__ float half_bits_to_float(uint16_t h) {
    return __half2float(__ushort_as_half(h));
}

// One code of a packed plane: element idx of a `bits`-bit little-endian-in-byte stream.
__device__ __forceinline__ int unpack_code(const uint8_t* __restrict__ p, int idx, int bits) {
    if (bits == 8) return p[idx];
    const int per = 8 / bits;
    return (p[idx / per] >> ((idx % per) * bits)) & ((1 << bits) - 1);
}

}  // namespace gkv
