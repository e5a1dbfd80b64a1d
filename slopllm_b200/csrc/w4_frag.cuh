// Register-level pieces shared by the NVFP4 weight-streaming kernels: warp MMA wrappers, the
// E2M1 -> f16 row expansion and cache-hinted 16-byte loads.
#pragma once

#include "common.cuh"

__device__ __forceinline__ void mma_f16_m16n8k16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mma_bf16_m16n8k16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ __half2 e4m3x2_to_half2(uint16_t v) {
    __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)v, __NV_E4M3);
    return *reinterpret_cast<__half2*>(&h);
}

// Expand one lane's 16 bytes (32 codes) of a row into 16 half2, scaled by the two block scales.
__device__ __forceinline__ void expand_row(const uint4& w, uint16_t sc, __half2 (&out)[16]) {
    const __half2 s = e4m3x2_to_half2(sc);
    const __half2 s0 = __half2half2(__low2half(s)), s1 = __half2half2(__high2half(s));
    const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        __half2 h[4];
        e2m1x8_to_half2x4(words[q], h);
        const __half2 sq = q < 2 ? s0 : s1;
#pragma unroll
        for (int i = 0; i < 4; ++i) out[q * 4 + i] = __hmul2(h[i], sq);
    }
}

// One 128-index group of a 16-row weight tile times eight activation rows: `lo` / `hi` are the lane's 32 expanded codes of
// rows g and g + 8, `xv[j]` the lane's activation unit j of the group (see the permuted layout in common.cuh).
__device__ __forceinline__ void mma_group_w4(float (&acc)[4], const __half2 (&lo)[16], const __half2 (&hi)[16], const uint4 (&xv)[4]) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint32_t a[4];
        a[0] = *reinterpret_cast<const uint32_t*>(&lo[4 * j + 0]);
        a[1] = *reinterpret_cast<const uint32_t*>(&hi[4 * j + 0]);
        a[2] = *reinterpret_cast<const uint32_t*>(&lo[4 * j + 1]);
        a[3] = *reinterpret_cast<const uint32_t*>(&hi[4 * j + 1]);
        mma_f16_m16n8k16(acc, a, xv[j].x, xv[j].y);
        a[0] = *reinterpret_cast<const uint32_t*>(&lo[4 * j + 2]);
        a[1] = *reinterpret_cast<const uint32_t*>(&hi[4 * j + 2]);
        a[2] = *reinterpret_cast<const uint32_t*>(&lo[4 * j + 3]);
        a[3] = *reinterpret_cast<const uint32_t*>(&hi[4 * j + 3]);
        mma_f16_m16n8k16(acc, a, xv[j].z, xv[j].w);
    }
}

__device__ __forceinline__ uint4 ldg_ca_16(const void* p) {
    uint4 v;
    asm volatile("ld.global.ca.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
// L2-only loads: data written earlier in the same kernel by other thread blocks.
__device__ __forceinline__ uint4 ldg_cg_16(const void* p) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ int ldg_cg_i32(const void* p) {
    int v;
    asm volatile("ld.global.cg.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float ldg_cg_f32(const void* p) {
    float v;
    asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t ld_acquire_gpu_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
