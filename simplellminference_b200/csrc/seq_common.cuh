// csrc/seq_common.cuh — helpers shared by the ragged-token-batch kernels (seq_*.cu): loads of fp32 / bf16 storage, activations.
#pragma once
#include <algorithm>

#include "common.cuh"

namespace sllm {

#ifdef __CUDACC__

// element i of a weight / cache array stored as fp32 or bf16
__device__ __forceinline__ float seq_ldw(const void* p, int dtype, size_t i) {
    if (dtype == SLLM_F32) return reinterpret_cast<const float*>(p)[i];
    return __uint_as_float((uint32_t) reinterpret_cast<const uint16_t*>(p)[i] << 16);
}
__device__ __forceinline__ float seq_ld(const float* p, size_t i) { return p[i]; }
__device__ __forceinline__ float seq_ld(const uint16_t* p, size_t i) { return __uint_as_float((uint32_t)p[i] << 16); }
__device__ __forceinline__ void seq_st(float* p, size_t i, float v) { p[i] = v; }
__device__ __forceinline__ void seq_st(uint16_t* p, size_t i, float v) { p[i] = f32_to_bf16_bits(v); }
__device__ __forceinline__ float seq_round_bf16(float v) { return __uint_as_float((uint32_t)f32_to_bf16_bits(v) << 16); }

__device__ __forceinline__ float seq_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
// log(1 + e^z) without overflow
__device__ __forceinline__ float seq_softplus(float z) { return fmaxf(z, 0.0f) + log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float seq_gelu_tanh(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// element index of (page, kv head, row in page, 0) in a pool [pages][kv_heads][page_len][width]
__device__ __forceinline__ size_t seq_pool_row(int page, int kv_heads, int g, int page_len, int in_page, int width) {
    return (((size_t)page * kv_heads + g) * page_len + in_page) * width;
}

#endif

}  // namespace sllm
