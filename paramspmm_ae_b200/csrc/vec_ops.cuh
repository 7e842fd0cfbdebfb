// Width-generic helpers for 32/64/128-bit global accesses of fp32 data (sm_100a).
#pragma once

#include <cuda_runtime.h>

template <int VW>
struct FVec {
    float v[VW];
};

// Read-only load of VW consecutive floats; p must be VW*4-byte aligned.
template <int VW>
__device__ __forceinline__ FVec<VW> ldg_vec(const float *p)
{
    FVec<VW> r;
    if constexpr (VW == 4) {
        float4 t = __ldg(reinterpret_cast<const float4 *>(p));
        r.v[0] = t.x; r.v[1] = t.y; r.v[2] = t.z; r.v[3] = t.w;
    } else if constexpr (VW == 2) {
        float2 t = __ldg(reinterpret_cast<const float2 *>(p));
        r.v[0] = t.x; r.v[1] = t.y;
    } else {
        r.v[0] = __ldg(p);
    }
    return r;
}

// Predicated read-only load: returns zeros and touches no memory when `on` is false.  Written
// as one predicated PTX instruction so that a batch of these stays straight-line code and the
// loads of the whole batch can be in flight together (a C++ conditional around a load may
// become a branch per load, which serialises the gathers).
template <int VW>
__device__ __forceinline__ FVec<VW> ldg_vec_if(const float *p, bool on)
{
    FVec<VW> r;
    const int flag = on ? 1 : 0;
    if constexpr (VW == 4) {
        asm("{\n\t.reg .pred q;\n\tsetp.ne.s32 q, %5, 0;\n\t"
            "mov.f32 %0, 0f00000000;\n\tmov.f32 %1, 0f00000000;\n\t"
            "mov.f32 %2, 0f00000000;\n\tmov.f32 %3, 0f00000000;\n\t"
            "@q ld.global.nc.v4.f32 {%0, %1, %2, %3}, [%4];\n\t}"
            : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3])
            : "l"(p), "r"(flag));
    } else if constexpr (VW == 2) {
        asm("{\n\t.reg .pred q;\n\tsetp.ne.s32 q, %3, 0;\n\t"
            "mov.f32 %0, 0f00000000;\n\tmov.f32 %1, 0f00000000;\n\t"
            "@q ld.global.nc.v2.f32 {%0, %1}, [%2];\n\t}"
            : "=f"(r.v[0]), "=f"(r.v[1])
            : "l"(p), "r"(flag));
    } else {
        asm("{\n\t.reg .pred q;\n\tsetp.ne.s32 q, %2, 0;\n\t"
            "mov.f32 %0, 0f00000000;\n\t"
            "@q ld.global.nc.f32 %0, [%1];\n\t}"
            : "=f"(r.v[0])
            : "l"(p), "r"(flag));
    }
    return r;
}

template <int VW>
__device__ __forceinline__ FVec<VW> zero_vec()
{
    FVec<VW> r;
#pragma unroll
    for (int i = 0; i < VW; ++i)
        r.v[i] = 0.f;
    return r;
}

// Streaming (evict-first) store: the output is written once and not re-read by the kernel.
template <int VW>
__device__ __forceinline__ void st_stream_vec(float *p, const float *v)
{
    if constexpr (VW == 4) {
        __stcs(reinterpret_cast<float4 *>(p), make_float4(v[0], v[1], v[2], v[3]));
    } else if constexpr (VW == 2) {
        __stcs(reinterpret_cast<float2 *>(p), make_float2(v[0], v[1]));
    } else {
        __stcs(p, v[0]);
    }
}

// Plain store (keeps the line resident), used for rows that other pieces will add to.
template <int VW>
__device__ __forceinline__ void st_vec(float *p, const float *v)
{
    if constexpr (VW == 4) {
        *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
    } else if constexpr (VW == 2) {
        *reinterpret_cast<float2 *>(p) = make_float2(v[0], v[1]);
    } else {
        *p = v[0];
    }
}

// Vector reduction into global memory (one RED per 16 / 8 / 4 bytes, no return value).
template <int VW>
__device__ __forceinline__ void red_add_vec(float *p, const float *v)
{
    if constexpr (VW == 4) {
        atomicAdd(reinterpret_cast<float4 *>(p), make_float4(v[0], v[1], v[2], v[3]));
    } else if constexpr (VW == 2) {
        atomicAdd(reinterpret_cast<float2 *>(p), make_float2(v[0], v[1]));
    } else {
        atomicAdd(p, v[0]);
    }
}
