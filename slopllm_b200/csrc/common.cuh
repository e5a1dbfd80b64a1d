// Shared device helpers for the sm_100a kernels: vector loads, warp/block reductions,
// E2M1 / E4M3 decode, bounded flag waits.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <cfloat>
#include <cstdint>

#define SL_API extern "C" __attribute__((visibility("default")))

typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;

#define SL_LAUNCH_CHECK() (int)cudaGetLastError()

// ---- programmatic dependent launch ------------------------------------------------------------
// Every kernel starts with pdl_grid_sync(): it first lets the next kernel in the stream be
// scheduled (its blocks become resident and park in their own pdl_grid_sync), then waits until
// the kernels it depends on have finished and their writes are visible.  Nothing that reads or
// writes activation memory may precede it.  On a launch without the programmatic attribute both
// instructions do nothing.
// SL_PDL_MODE selects where a kernel lets its successor start:
//   0  at kernel exit (implicit trigger): only the launch latency overlaps
//   1  after the main loop of the heavy kernels (pdl_trigger_late): the successor's blocks become resident and run
//      their prologue under this kernel's epilogue
//   2  at kernel entry, and the weight-streaming kernels prefetch their first weight rows into L2 before they wait
//      for the predecessor (weights do not depend on it), so consecutive kernels' memory streams overlap
//   3  at kernel entry, nothing else: the successor's blocks become resident as soon as there is room and park in their
//      dependency wait
#ifndef SL_PDL_MODE
#define SL_PDL_MODE 0
#endif
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_grid_sync() {
#if SL_PDL_MODE >= 2
    pdl_trigger();
#endif
    pdl_wait();
}
__device__ __forceinline__ void pdl_trigger_late() {
#if SL_PDL_MODE == 1
    pdl_trigger();
#endif
}
__device__ __forceinline__ void prefetch_l2_line(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
// All threads of the block: prefetch `rows` rows of `row_bytes` bytes starting at `base` (row stride = row_bytes).
__device__ __forceinline__ void prefetch_l2_rows(const void* base, int rows, size_t row_bytes, size_t max_bytes_per_row = 1 << 20) {
    const size_t rb = row_bytes < max_bytes_per_row ? row_bytes : max_bytes_per_row;
    const int lines = (int)((rb + 127) / 128);
    for (int i = threadIdx.x; i < rows * lines; i += blockDim.x)
        prefetch_l2_line(reinterpret_cast<const uint8_t*>(base) + (size_t)(i / lines) * row_bytes + (size_t)(i % lines) * 128);
}
// Kernel entry of a weight-streaming kernel: `PREFETCH` may only touch memory that no kernel of the step writes.
#if SL_PDL_MODE == 2
#define PDL_ENTRY_WITH_PREFETCH(PREFETCH) \
    do {                                  \
        pdl_trigger();                    \
        PREFETCH;                         \
        pdl_wait();                       \
    } while (0)
#else
#define PDL_ENTRY_WITH_PREFETCH(PREFETCH) pdl_grid_sync()
#endif

// Process-wide switch (sl_set_pdl); on by default.
extern int g_sl_pdl_enabled;
// Kernels launched through sl_launch since the library was loaded (sl_kernel_launches): what a captured step really costs.
extern unsigned long long g_sl_kernel_launches;

template <typename... KArgs, typename... Args>
inline cudaError_t sl_launch(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_sl_pdl_enabled ? 1 : 0;
    ++g_sl_kernel_launches;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum; `scratch` holds >= 33 floats.  All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nw ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nw ? scratch[lane] : -FLT_MAX;
        t = warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

__device__ __forceinline__ uint4 ldg_nc_16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ldg_nc_8(const void* p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}

__device__ __forceinline__ float2 bf162_to_f2(uint32_t u) {
    return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
}
__device__ __forceinline__ uint32_t f2_to_bf162(float a, float b) {
    bf162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

// Four packed bytes (8 E2M1 codes, low nibble = even element) -> 8 halves as 4 half2.
__device__ __forceinline__ void e2m1x8_to_half2x4(uint32_t packed, __half2 out[4]) {
    uint32_t r0, r1, r2, r3;
    asm volatile(
        "{\n"
        ".reg .b8 b0, b1, b2, b3;\n"
        "mov.b32 {b0, b1, b2, b3}, %4;\n"
        "cvt.rn.f16x2.e2m1x2 %0, b0;\n"
        "cvt.rn.f16x2.e2m1x2 %1, b1;\n"
        "cvt.rn.f16x2.e2m1x2 %2, b2;\n"
        "cvt.rn.f16x2.e2m1x2 %3, b3;\n"
        "}\n"
        : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(packed));
    out[0] = *reinterpret_cast<__half2*>(&r0);
    out[1] = *reinterpret_cast<__half2*>(&r1);
    out[2] = *reinterpret_cast<__half2*>(&r2);
    out[3] = *reinterpret_cast<__half2*>(&r3);
}

__device__ __forceinline__ float e4m3_to_float(uint8_t b) {
    __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
    return __half2float(*reinterpret_cast<__half*>(&h));
}
__device__ __forceinline__ float2 e4m3x2_to_float2(uint16_t b) {
    __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)b, __NV_E4M3);
    return __half22float2(*reinterpret_cast<__half2*>(&h));
}
__device__ __forceinline__ uint8_t float_to_e4m3(float v) {
    return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}

// Power-of-two scale >= max(amax, 1e-4) / 448 (indexer K / Q rows).
__device__ __forceinline__ float pow2_scale_ceil(float amax) {
    float raw = fmaxf(amax, 1e-4f) / 448.f;
    uint32_t bits = __float_as_uint(raw);
    if (bits & 0x007fffffu) bits = (bits + 0x00800000u) & 0x7f800000u;
    return __uint_as_float(bits);
}

// ---- permuted f16 activation copy for the NVFP4 tensor-core kernels --------------------------------
// 16-byte unit (token, group, j, c) of the copy holds x[token][group*128 + c*32 + j*8 .. +7] at unit index
// (token*G + group)*16 + j*4 + c, G = K/128 (see permute_x_kernel, csrc/gemv_mma.cu).  A producer that already
// has four consecutive bf16-rounded values of a row (columns 4i .. 4i+3, packed as two bf16x2 words) stores its
// half unit here, which saves the separate permute launch in front of the consumer.
__device__ __forceinline__ void store_perm4(uint4* xp, int tok, int K, int i, uint32_t lo_bf162, uint32_t hi_bf162) {
    const int u = i >> 1, group = u >> 4, within = u & 15, c = within >> 2, j = within & 3;
    const float2 a = bf162_to_f2(lo_bf162), b = bf162_to_f2(hi_bf162);
    const __half2 h0 = __floats2half2_rn(a.x, a.y), h1 = __floats2half2_rn(b.x, b.y);
    uint2 v;
    v.x = *reinterpret_cast<const uint32_t*>(&h0);
    v.y = *reinterpret_cast<const uint32_t*>(&h1);
    reinterpret_cast<uint2*>(xp + ((size_t)tok * (K / 128) + group) * 16 + j * 4 + c)[i & 1] = v;
}

// ---- index self-checks ----------------------------------------------------------------------------
// Every index that a kernel reads from device metadata (cache slots, page-table entries) is checked
// against its bound before it is used as an address.  A bad index is recorded once in `guard`
// ({site, value, limit, block}) and the access is skipped, so a corrupt table shows up as a host-side
// error after the step instead of a memory fault.  `guard` may be null (no record, access still skipped).
__device__ __forceinline__ bool guard_ok(int* guard, int site, long long value, long long limit) {
    if (value >= 0 && value < limit) return true;
    if (guard != nullptr && atomicCAS(guard, 0, site) == 0) {
        guard[1] = (int)value;
        guard[2] = (int)limit;
        guard[3] = (int)blockIdx.x;
    }
    return false;
}

// ---- bounded waits on flags written by other GPUs ---------------------------------------------
// Every wait gives up after `max_spins` polls, records where it stopped in `status`
// (status[0] = code, [1] = site, [2] = expected, [3] = observed) and lets the kernel
// finish normally; the host reads the status word after the step.
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Flag publication after one `__threadfence_system()`: the fence orders the data stores, so the flag stores
// themselves need no release semantics and can all be in flight at once (a release store would wait for the
// acknowledgement of everything before it, one NVLink round trip per peer).
__device__ __forceinline__ void st_relaxed_sys_u32(uint32_t* p, uint32_t v) {
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Arrival counter in (possibly another GPU's) memory: add with release semantics at system scope, no return value.
__device__ __forceinline__ void red_release_sys_add_u32(uint32_t* p, uint32_t v) {
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_relaxed_sys_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ bool wait_flag_geq(const uint32_t* flag, uint32_t target, uint32_t max_spins,
                                              int* status, int site) {
    uint32_t seen = 0;
    for (uint32_t i = 0; i < max_spins; ++i) {
        seen = ld_acquire_sys_u32(flag);
        if ((int32_t)(seen - target) >= 0) return true;
        if (i > 64) __nanosleep(i > 4096 ? 256 : 32);
    }
    if (status != nullptr && atomicCAS(status, 0, 1) == 0) {
        status[1] = site;
        status[2] = (int)target;
        status[3] = (int)seen;
    }
    return false;
}
