// Shared device/host helpers of libcbl (codebook-linear kernels for sm_100a).
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include "../../include/cbl.h"

extern int g_cbl_last_cuda_error;

static inline int cbl_check_launch() {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        g_cbl_last_cuda_error = (int)e;
        return CBL_ECUDA;
    }
    return CBL_OK;
}

#define CBL_CUDA(call)                           \
    do {                                         \
        cudaError_t e_ = (call);                 \
        if (e_ != cudaSuccess) {                 \
            g_cbl_last_cuda_error = (int)e_;     \
            return CBL_ECUDA;                    \
        }                                        \
    } while (0)

static inline int cbl_ceil_div(int a, int b) { return (a + b - 1) / b; }

// Number of SMs of the current device (cached per device id).
int cbl_sm_count();

__device__ __forceinline__ uint32_t cbl_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Tag j of a row's little-endian bit stream (file layout, shapequant/packed.py:8-11).
__device__ __forceinline__ uint32_t cbl_read_tag(const int32_t* __restrict__ row_words, int W, int j, int bits) {
    uint32_t pos = (uint32_t)j * (uint32_t)bits;
    uint32_t wi = pos >> 5, sh = pos & 31u;
    uint32_t lo = (uint32_t)__ldg(row_words + wi);
    uint32_t hi = (sh + bits > 32u && (int)(wi + 1) < W) ? (uint32_t)__ldg(row_words + wi + 1) : 0u;
    return __funnelshift_r(lo, hi, sh) & ((1u << bits) - 1u);
}

__device__ __forceinline__ uint4 cbl_ldg_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ uint4 cbl_lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

__device__ __forceinline__ float cbl_lds_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}

// D += A(16x16, row) * B(16x8, col), fp16 inputs, fp32 accumulate.
__device__ __forceinline__ void cbl_mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// D = A(16x8, row) * B(8x8, col), fp16 inputs, fp32 result (zero accumulator).
__device__ __forceinline__ void cbl_mma1688(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
                 : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
                 : "r"(a0), "r"(a1), "r"(b0), "f"(0.0f));
}

template <typename T> __device__ __forceinline__ T cbl_cvt_out(float v);
template <> __device__ __forceinline__ float cbl_cvt_out<float>(float v) { return v; }
template <> __device__ __forceinline__ __half cbl_cvt_out<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 cbl_cvt_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ void cbl_store_out(void* y, int dtype, int64_t i, float v) {
    if (dtype == CBL_BF16) ((__nv_bfloat16*)y)[i] = __float2bfloat16_rn(v);
    else if (dtype == CBL_F16) ((__half*)y)[i] = __float2half_rn(v);
    else ((float*)y)[i] = v;
}

__device__ __forceinline__ float cbl_load_in(const void* x, int dtype, int64_t i) {
    if (dtype == CBL_BF16) return __bfloat162float(((const __nv_bfloat16*)x)[i]);
    if (dtype == CBL_F16) return __half2float(((const __half*)x)[i]);
    return ((const float*)x)[i];
}
