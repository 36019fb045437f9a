// Small device helpers shared by the kernels.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace kb {

__device__ __forceinline__ float warp_reduce_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ int warp_reduce_sum(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// result broadcast to every thread; `scratch` holds one value per warp (<= 32 warps)
__device__ __forceinline__ float block_reduce_max(float v, float *scratch) {
    v = warp_reduce_max(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = lane < nwarps ? scratch[lane] : 0.0f;
    return warp_reduce_max(r);
}
__device__ __forceinline__ int block_reduce_sum(int v, int *scratch) {
    v = warp_reduce_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    int r = lane < nwarps ? scratch[lane] : 0;
    return warp_reduce_sum(r);
}

// q = clamp(rne(x / s), -127, 127); NaN -> 0
__device__ __forceinline__ int quantise_one(float x, float s) {
    int q = __float2int_rn(__fdiv_rn(x, s));
    return max(-127, min(127, q));
}

// Same result as quantise_one without a division per element.  r = 1/s (correctly
// rounded).  t = x*r is within ~1.5e-5 of the true quotient for |x/s| <= 127, so
// rint(t) equals rint(fl(x/s)) unless t sits within 1e-3 of a rounding tie; only then
// is the exact IEEE division evaluated.
__device__ __forceinline__ int quantise_one_fast(float x, float s, float r) {
    const float t = x * r;
    const float frac = fabsf(t - rintf(t));
    int q = __float2int_rn(t);
    if (frac > 0.499f) q = __float2int_rn(__fdiv_rn(x, s));
    return max(-127, min(127, q));
}

// sum over four (unsigned byte of a) * (signed byte of b) + c
__device__ __forceinline__ int dp4a_u8s8(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// 16-byte read-only streaming load that does not allocate in L1
__device__ __forceinline__ uint4 ld_stream_v4(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// y = (float(acc) * sw) * sx (+ bias), every operation separately rounded
__device__ __forceinline__ float dequant_out(int acc, float sw, float sx, float bias, bool has_bias) {
    float v = __fmul_rn(__fmul_rn(__int2float_rn(acc), sw), sx);
    return has_bias ? __fadd_rn(v, bias) : v;
}

// one pair, one 8-byte store: value and epoch become visible together
__device__ __forceinline__ void st_pair(float *base, size_t o, float value, uint32_t epoch) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};" ::"l"(reinterpret_cast<uint2 *>(base) + o), "r"(__float_as_uint(value)),
                 "r"(epoch)
                 : "memory");
}


}  // namespace kb
