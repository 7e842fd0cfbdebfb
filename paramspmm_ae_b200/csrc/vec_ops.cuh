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
    if constexpr (VW == 8) {
        // 256-bit read-only load (sm_100): p must be 32-byte aligned
        asm("ld.global.nc.v8.f32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
            : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3]), "=f"(r.v[4]), "=f"(r.v[5]), "=f"(r.v[6]),
              "=f"(r.v[7])
            : "l"(p));
    } else if constexpr (VW == 4) {
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

// L2 eviction policies (createpolicy).  `keep` marks a fraction of the touched lines
// evict_last so that a stable subset of a randomly gathered operand stays resident when the
// whole operand does not fit; `stream` marks lines evict_first (data read or written once).
__device__ __forceinline__ unsigned long long l2_policy_keep(float fraction)
{
    unsigned long long pol;
    asm volatile("createpolicy.fractional.L2::evict_last.L2::evict_unchanged.b64 %0, %1;" : "=l"(pol) : "f"(fraction));
    return pol;
}
__device__ __forceinline__ unsigned long long l2_policy_stream()
{
    unsigned long long pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}

// Read-only load of VW floats with an L2 cache-policy hint.
template <int VW>
__device__ __forceinline__ FVec<VW> ldg_vec_hint(const float *p, unsigned long long pol)
{
    FVec<VW> r;
    if constexpr (VW == 4) {
        asm("ld.global.nc.L2::cache_hint.v4.f32 {%0, %1, %2, %3}, [%4], %5;"
            : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3]) : "l"(p), "l"(pol));
    } else if constexpr (VW == 2) {
        asm("ld.global.nc.L2::cache_hint.v2.f32 {%0, %1}, [%2], %3;"
            : "=f"(r.v[0]), "=f"(r.v[1]) : "l"(p), "l"(pol));
    } else {
        asm("ld.global.nc.L2::cache_hint.f32 %0, [%1], %2;" : "=f"(r.v[0]) : "l"(p), "l"(pol));
    }
    return r;
}

// Streaming 32-bit read (index / value arrays): no L1 allocation, evict-first in L2.
__device__ __forceinline__ int ldg_stream_b32(const void *p, unsigned long long pol)
{
    int r;
    asm("ld.global.nc.L1::no_allocate.L2::cache_hint.b32 %0, [%1], %2;" : "=r"(r) : "l"(p), "l"(pol));
    return r;
}

// Store of VW floats with an L2 cache-policy hint.
template <int VW>
__device__ __forceinline__ void st_vec_hint(float *p, const float *v, unsigned long long pol)
{
    if constexpr (VW == 4) {
        asm volatile("st.global.L2::cache_hint.v4.f32 [%0], {%1, %2, %3, %4}, %5;"
                     :: "l"(p), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "l"(pol) : "memory");
    } else if constexpr (VW == 2) {
        asm volatile("st.global.L2::cache_hint.v2.f32 [%0], {%1, %2}, %3;"
                     :: "l"(p), "f"(v[0]), "f"(v[1]), "l"(pol) : "memory");
    } else {
        asm volatile("st.global.L2::cache_hint.f32 [%0], %1, %2;" :: "l"(p), "f"(v[0]), "l"(pol) : "memory");
    }
}

// Address of a lane's slice of dense row c: base + c * ld_bytes as one 32x32+64 multiply-add.
__device__ __forceinline__ const float *row_slice(const char *base, int c, unsigned ld_bytes)
{
    unsigned long long r;
    asm("mad.wide.u32 %0, %1, %2, %3;" : "=l"(r) : "r"((unsigned)c), "r"(ld_bytes), "l"(base));
    return reinterpret_cast<const float *>(r);
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
    if constexpr (VW == 8) {
        asm("{\n\t.reg .pred q;\n\tsetp.ne.s32 q, %9, 0;\n\t"
            "mov.f32 %0, 0f00000000;\n\tmov.f32 %1, 0f00000000;\n\t"
            "mov.f32 %2, 0f00000000;\n\tmov.f32 %3, 0f00000000;\n\t"
            "mov.f32 %4, 0f00000000;\n\tmov.f32 %5, 0f00000000;\n\t"
            "mov.f32 %6, 0f00000000;\n\tmov.f32 %7, 0f00000000;\n\t"
            "@q ld.global.nc.v8.f32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];\n\t}"
            : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3]), "=f"(r.v[4]), "=f"(r.v[5]), "=f"(r.v[6]),
              "=f"(r.v[7])
            : "l"(p), "r"(flag));
    } else if constexpr (VW == 4) {
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
    if constexpr (VW == 8) {
        __stcs(reinterpret_cast<float4 *>(p), make_float4(v[0], v[1], v[2], v[3]));
        __stcs(reinterpret_cast<float4 *>(p) + 1, make_float4(v[4], v[5], v[6], v[7]));
    } else if constexpr (VW == 4) {
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
    if constexpr (VW == 8) {
        *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
        *(reinterpret_cast<float4 *>(p) + 1) = make_float4(v[4], v[5], v[6], v[7]);
    } else if constexpr (VW == 4) {
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
