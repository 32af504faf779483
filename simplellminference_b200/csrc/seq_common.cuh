// csrc/seq_common.cuh — helpers shared by the ragged-token-batch kernels (seq_*.cu): loads of fp32 / bf16 storage, activations.
#pragma once
#include <algorithm>

#include <cuda_bf16.h>

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
// 16 bytes of a pool as floats (4 fp32 or 8 bf16 values); `take` false = zeros without touching memory
__device__ __forceinline__ void seq_ld16(const float* p, bool take, float (&out)[4]) {
    const float4 v = take ? *reinterpret_cast<const float4*>(p) : make_float4(0.f, 0.f, 0.f, 0.f);
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
}
__device__ __forceinline__ void seq_ld16(const uint16_t* p, bool take, float (&out)[8]) {
    const uint4 v = take ? *reinterpret_cast<const uint4*>(p) : make_uint4(0u, 0u, 0u, 0u);
    out[0] = bf16_lo(v.x); out[1] = bf16_hi(v.x); out[2] = bf16_lo(v.y); out[3] = bf16_hi(v.y);
    out[4] = bf16_lo(v.z); out[5] = bf16_hi(v.z); out[6] = bf16_lo(v.w); out[7] = bf16_hi(v.w);
}
__device__ __forceinline__ void seq_st(float* p, size_t i, float v) { p[i] = v; }
__device__ __forceinline__ void seq_st(uint16_t* p, size_t i, float v) { p[i] = f32_to_bf16_bits(v); }
// nearest-even rounding to bf16 and back: one cvt instruction + one shift (the same values as f32_to_bf16_bits for finite inputs)
__device__ __forceinline__ float seq_round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__device__ __forceinline__ float seq_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
// log(1 + e^z) without overflow
__device__ __forceinline__ float seq_softplus(float z) { return fmaxf(z, 0.0f) + log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float seq_gelu_tanh(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// cos and sin of pos * freq. The product is formed and reduced in double: at position 1000 an fp32 product is already off by up to
// 3e-5 rad, five hundred times the rounding of everything else in the layer, and the error would grow with the position.
__device__ __forceinline__ void seq_angle(int pos, double freq, float* sn, float* cs) {
    double s, c;
    sincos((double)pos * freq, &s, &c);
    *sn = (float)s;
    *cs = (float)c;
}

// element index of (page, kv head, row in page, 0) in a pool [pages][kv_heads][page_len][width]
__device__ __forceinline__ size_t seq_pool_row(int page, int kv_heads, int g, int page_len, int in_page, int width) {
    return (((size_t)page * kv_heads + g) * page_len + in_page) * width;
}

#endif

}  // namespace sllm
