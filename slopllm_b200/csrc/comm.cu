// In-kernel NVLink collectives fused with their consumers.
//
//  * ar_add_rmsnorm_kernel: the consumer half of the fused all-reduce.  Producers (GEMV / MoE /
//    tcgen05 epilogues, see push.cuh) have stored every rank's partial rows into this rank's
//    receive slots; this kernel waits (bounded) for the epoch flags of all ranks, sums the slots
//    in rank order (deterministic), adds the residual, applies RMSNorm and writes the normed
//    activations + new residual.  One kernel replaces all-reduce + fused add + RMSNorm
//    (reference: `csrc/glm_p2p.cu:238-460` rmsnorm_pointers_smem_kernel, `csrc/glm_ops.cu:358`).
//  * flag_barrier_kernel: arrive + bounded wait on peer flags (reference `p2p_barrier_kernel`,
//    `csrc/glm_p2p.cu:180`, whose wait is unbounded).
//  * cp_merge_push_kernel / cp_merge_local: context-parallel attention merge - every rank pushes
//    its partial (o, lse) head slices to the rank that owns those heads, the owner combines by
//    log-sum-exp (reference `csrc/glm_context_parallel.cu:277-540`).
//  * topk_merge_push: per-rank top-k candidate lists pushed to every rank for the global re-select
//    (reference `src/parallel_ops.ts:4233-4330`).
//
// Every wait is bounded: on expiry the kernel records {code, site, expected, observed} in a
// status word block and finishes normally.
#include "push.cuh"
#include <cstring>

struct RecvCtx {
    uint32_t* buf;             // this rank's receive buffer [world][slot_rows][row_len] of {bf16 value, 16-bit tag} words
    const uint32_t* flags;     // unused by the tagged protocol
    uint32_t* epoch;           // completed collectives on this buffer (incremented here)
    uint32_t* done_counter;    // consumer blocks that have finished
    int* status;               // [4] error record
    int world, slot_rows, row_len;
    uint32_t max_spins;
};

__device__ __forceinline__ uint4 ld_volatile_16(const void* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

// Four consecutive tagged words of every rank's slot (element columns 4i .. 4i+3 of row t, one 16-byte load per
// rank): all loads of a poll round are issued before any tag is tested, so a round costs one memory latency, not one
// per rank.  Rounds repeat until every tag equals `tag`; after max_spins rounds the timeout is recorded in `status` and
// the last values seen are used (the host reads the status word after the step).  The sum runs in rank order
// (deterministic).  The words are zeroed once used (see csrc/push.cuh).
__device__ __forceinline__ float4 ll_gather_sum(const RecvCtx& c, int t, int i, uint32_t tag) {
    uint4 w[SL_MAX_RANKS];
    for (uint32_t spin = 0;; ++spin) {
#pragma unroll
        for (int r = 0; r < SL_MAX_RANKS; ++r)
            if (r < c.world) w[r] = ld_volatile_16(c.buf + ((size_t)r * c.slot_rows + t) * c.row_len + 4 * i);
        bool ok = true;
        uint32_t seen = tag;
#pragma unroll
        for (int r = 0; r < SL_MAX_RANKS; ++r) {
            if (r < c.world) {
                if ((w[r].x & 0xffffu) != tag) { ok = false; seen = w[r].x & 0xffffu; }
                if ((w[r].y & 0xffffu) != tag) { ok = false; seen = w[r].y & 0xffffu; }
                if ((w[r].z & 0xffffu) != tag) { ok = false; seen = w[r].z & 0xffffu; }
                if ((w[r].w & 0xffffu) != tag) { ok = false; seen = w[r].w & 0xffffu; }
            }
        }
        if (ok) break;
        if (spin >= c.max_spins) {
            if (c.status != nullptr && atomicCAS(c.status, 0, 1) == 0) {
                c.status[1] = 1;
                c.status[2] = (int)tag;
                c.status[3] = (int)seen;
            }
            break;
        }
        if (spin > 64) __nanosleep(64);
    }
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int r = 0; r < SL_MAX_RANKS; ++r) {
        if (r < c.world) {
            a.x += __uint_as_float(w[r].x & 0xffff0000u); a.y += __uint_as_float(w[r].y & 0xffff0000u);
            a.z += __uint_as_float(w[r].z & 0xffff0000u); a.w += __uint_as_float(w[r].w & 0xffff0000u);
            *reinterpret_cast<uint4*>(c.buf + ((size_t)r * c.slot_rows + t) * c.row_len + 4 * i) = make_uint4(0u, 0u, 0u, 0u);
        }
    }
    return a;
}

// One block per token row.  H % 4 == 0, H <= 16384.  Sums the ranks' slots in rank order (deterministic).
__global__ void __launch_bounds__(512) ar_add_rmsnorm_kernel(RecvCtx c, bf16* __restrict__ out, float* __restrict__ res_out,
                                                              const float* __restrict__ res_in, const bf16* __restrict__ w,
                                                              int H, float eps, uint4* __restrict__ xp) {
    pdl_grid_sync();
    __shared__ float scratch[33];
    const int t = blockIdx.x, nt = blockDim.x, n4 = H / 4;
    const uint32_t target = *c.epoch + 1u, tag = push_tag_of(*c.epoch);
    float4 v[8];
    float ss = 0.f;
#pragma unroll
    for (int q = 0; q < 8; ++q) {
        const int i = threadIdx.x + q * nt;
        if (i < n4) {
            float4 a = ll_gather_sum(c, t, i, tag);
            if (res_in != nullptr) {
                const float4 r = reinterpret_cast<const float4*>(res_in + (size_t)t * H)[i];
                a.x += r.x; a.y += r.y; a.z += r.z; a.w += r.w;
            }
            v[q] = a;
            ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)H + eps);
#pragma unroll
    for (int q = 0; q < 8; ++q) {
        const int i = threadIdx.x + q * nt;
        if (i < n4) {
            if (res_out != nullptr) reinterpret_cast<float4*>(res_out + (size_t)t * H)[i] = v[q];
            const uint2 wu = reinterpret_cast<const uint2*>(w)[i];
            const float2 w0 = bf162_to_f2(wu.x), w1 = bf162_to_f2(wu.y);
            uint2 o;
            o.x = f2_to_bf162(v[q].x * inv * w0.x, v[q].y * inv * w0.y);
            o.y = f2_to_bf162(v[q].z * inv * w1.x, v[q].w * inv * w1.y);
            reinterpret_cast<uint2*>(out + (size_t)t * H)[i] = o;
            if (xp != nullptr) store_perm4(xp, t, H, i, o.x, o.y);
        }
    }
    // the last block to finish closes the epoch (producers of the next use read it)
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned prev = atomicAdd(c.done_counter, 1u);
        if (prev == gridDim.x - 1) {
            *c.done_counter = 0;
            *c.epoch = target;
            __threadfence();
        }
    }
}

SL_API int sl_ar_add_rmsnorm(const RecvCtx* c, void* out, void* res_out, const void* res_in, const void* w, int T, int H,
                             float eps, void* xp, cudaStream_t s) {
    if (T == 0) return 0;
    if (H % 4 != 0 || H > 16384 || c->world > SL_MAX_RANKS || (xp != nullptr && H % 128 != 0)) return -1;
    int threads = ((H / 4 + 3) / 4 + 31) / 32 * 32;           // four float4 per thread up to H = 8192, eight beyond
    if (threads < 128) threads = 128;
    if (threads > 512) threads = 512;
    sl_launch(ar_add_rmsnorm_kernel, T, threads, 0, s, *c, (bf16*)out, (float*)res_out, (const float*)res_in, (const bf16*)w, H, eps,
              (uint4*)xp);
    return SL_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// Plain push of an existing fp32 [T, row_len] tensor (producers that are not fused yet, and tests).
__global__ void push_rows_kernel(PushCtx c, const float* __restrict__ x, int T, int N) {
    pdl_grid_sync();
    const size_t total = (size_t)T * N;
    const uint32_t tag = push_tag(c);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int row = (int)(i / N), col = (int)(i % N);
        const float v = x[i];
        push_store_all(c, row, col, v, tag);
    }
}

SL_API int sl_push_rows(const PushCtx* c, const void* x, int T, int N, cudaStream_t s) {
    if (T == 0) return 0;
    if (T > c->slot_rows || N > c->row_len) return -1;
    int blocks = (int)(((size_t)T * N + 255) / 256);
    if (blocks > 148) blocks = 148;
    sl_launch(push_rows_kernel, blocks, 256, 0, s, *c, (const float*)x, T, N);
    return SL_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// Flag barrier: publish `value` into slot `rank` of every peer's flag array, then wait (bounded)
// until every slot of the local array has reached `value`.
struct PtrTable { uint32_t* p[SL_MAX_RANKS]; };
__global__ void flag_barrier_kernel_v(PtrTable peers, uint32_t* local_flags, int rank, int world, uint32_t value,
                                      uint32_t max_spins, int* status) {
    pdl_grid_sync();
    const int p = threadIdx.x;
    if (p < world) {
        __threadfence_system();
        st_release_sys_u32(peers.p[p] + rank, value);
        wait_flag_geq(local_flags + p, value, max_spins, status, 2);
    }
}

SL_API int sl_flag_barrier(void* const* peer_flags, void* local_flags, int rank, int world, unsigned value, unsigned max_spins,
                           void* status, cudaStream_t s) {
    if (world > SL_MAX_RANKS) return -1;
    PtrTable t;
    for (int i = 0; i < SL_MAX_RANKS; ++i) t.p[i] = i < world ? (uint32_t*)peer_flags[i] : nullptr;
    flag_barrier_kernel_v<<<1, 32, 0, s>>>(t, (uint32_t*)local_flags, rank, world, value, max_spins, (int*)status);
    return SL_LAUNCH_CHECK();
}

// A wait that nothing satisfies, used by the tests of the timeout path: returns after max_spins
// polls with the status record filled in.
__global__ void wait_only_kernel(const uint32_t* flag, uint32_t target, uint32_t max_spins, int* status) {
    pdl_grid_sync();
    if (threadIdx.x == 0) wait_flag_geq(flag, target, max_spins, status, 3);
}
SL_API int sl_wait_flag(const void* flag, unsigned target, unsigned max_spins, void* status, cudaStream_t s) {
    wait_only_kernel<<<1, 32, 0, s>>>((const uint32_t*)flag, target, max_spins, (int*)status);
    return SL_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// Context-parallel attention merge, push form.  Rank r holds partial o[T, h, R] (fp32) and
// lse[T, h] over its KV shard for ALL heads.  Head slice [owner*hl, (owner+1)*hl) is pushed into
// the owner's staging [world][T, hl, R] / [world][T, hl]; after the flags arrive the owner merges.
struct CpPushCtx {
    float* o_stage[SL_MAX_RANKS];     // owner's staging: [world][Tmax][hl][R]
    float* lse_stage[SL_MAX_RANKS];   // [world][Tmax][hl]
    uint32_t* flags[SL_MAX_RANKS];
    const uint32_t* epoch;
    uint32_t* block_counter;
    int rank, world, Tmax, h, hl, R;
};

__global__ void cp_merge_push_kernel(CpPushCtx c, const float* __restrict__ o, const float* __restrict__ lse, int T) {
    pdl_grid_sync();
    // grid (h, T): one block per (head, token)
    const int head = blockIdx.x, t = blockIdx.y;
    const int owner = head / c.hl, hh = head % c.hl;
    // staging is double-buffered by epoch parity (see gather_push_kernel)
    const size_t par = *c.epoch & 1u;
    const float4* src = reinterpret_cast<const float4*>(o + ((size_t)t * c.h + head) * c.R);
    float4* dst = reinterpret_cast<float4*>(c.o_stage[owner] + (((par * c.world + c.rank) * c.Tmax + t) * c.hl + hh) * c.R);
    for (int i = threadIdx.x; i < c.R / 4; i += blockDim.x) dst[i] = src[i];
    if (threadIdx.x == 0) c.lse_stage[owner][((par * c.world + c.rank) * c.Tmax + t) * c.hl + hh] = lse[(size_t)t * c.h + head];
    __syncthreads();
    if (threadIdx.x == 0) {
        // device-scope fence here, system-scope fence once in the last block: the counter chains the blocks' stores
        // before the flag stores (a system fence per block costs microseconds each)
        __threadfence();
        const unsigned prev = atomicAdd(c.block_counter, 1u);
        if (prev == gridDim.x * gridDim.y - 1) {
            *c.block_counter = 0;
            __threadfence_system();
            const uint32_t e = *c.epoch + 1u;
            for (int p = 0; p < c.world; ++p) st_relaxed_sys_u32(c.flags[p] + c.rank, e);
        }
    }
}

SL_API int sl_cp_merge_push(const CpPushCtx* c, const void* o, const void* lse, int T, cudaStream_t s) {
    if (T == 0) return 0;
    if (T > c->Tmax || c->R % 4 != 0) return -1;
    sl_launch(cp_merge_push_kernel, dim3(c->h, T), 128, 0, s, *c, (const float*)o, (const float*)lse, T);
    return SL_LAUNCH_CHECK();
}

// Owner side: wait for all ranks, then the combine kernel (csrc/sparse_mla.cu) merges the world
// staged partials per local head.  This kernel only waits and closes the epoch.
__global__ void epoch_wait_kernel(const uint32_t* flags, uint32_t* epoch, int world, uint32_t max_spins, int* status, int site) {
    pdl_grid_sync();
    const uint32_t target = *epoch + 1u;
    if (threadIdx.x < world) wait_flag_geq(flags + threadIdx.x, target, max_spins, status, site);
    __syncthreads();
    if (threadIdx.x == 0) { *epoch = target; __threadfence(); }
}

SL_API int sl_epoch_wait(const void* flags, void* epoch, int world, unsigned max_spins, void* status, int site, cudaStream_t s) {
    epoch_wait_kernel<<<1, 32, 0, s>>>((const uint32_t*)flags, (uint32_t*)epoch, world, max_spins, (int*)status, site);
    return SL_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// Generic all-gather by push: every rank stores `bytes` of local data into slot `rank` of every
// peer's buffer (16-byte granularity), then publishes the epoch flag.
struct GatherPushCtx {
    uint8_t* bufs[SL_MAX_RANKS];      // [world][slot_bytes]
    uint32_t* flags[SL_MAX_RANKS];
    const uint32_t* epoch;
    uint32_t* block_counter;
    int rank, world;
    size_t slot_bytes;
};

__global__ void gather_push_kernel(GatherPushCtx c, const uint4* __restrict__ src, size_t n16) {
    pdl_grid_sync();
    // two buffer halves, chosen by the parity of the epoch: a rank can be at most one collective ahead of the slowest
    // one (it waits for every rank's flag each time), so it never overwrites a half that a peer is still reading
    const size_t half = (size_t)(*c.epoch & 1u) * c.world * c.slot_bytes;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x) {
        const uint4 v = src[i];
        for (int p = 0; p < c.world; ++p) reinterpret_cast<uint4*>(c.bufs[p] + half + (size_t)c.rank * c.slot_bytes)[i] = v;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        // device-scope fence here, system-scope fence once in the last block: the counter chains the blocks' stores
        // before the flag stores (a system fence per block costs microseconds each)
        __threadfence();
        const unsigned prev = atomicAdd(c.block_counter, 1u);
        if (prev == gridDim.x - 1) {
            *c.block_counter = 0;
            __threadfence_system();
            const uint32_t e = *c.epoch + 1u;
            for (int p = 0; p < c.world; ++p) st_relaxed_sys_u32(c.flags[p] + c.rank, e);
        }
    }
}

// Copy the `world` slots of the half that the just-completed gather used (the epoch was advanced by the wait kernel,
// so that half is (epoch - 1) & 1) into a private tensor [world, bytes].  Reading the parity on the device keeps the
// sequence valid inside a replayed CUDA graph.
__global__ void gather_fetch_kernel(uint4* __restrict__ out, const uint8_t* __restrict__ local_buf, const uint32_t* __restrict__ epoch,
                                    int world, size_t slot_bytes, size_t n16) {
    pdl_grid_sync();
    const size_t half = (size_t)((*epoch - 1u) & 1u) * world * slot_bytes;
    const size_t total = (size_t)world * n16;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / n16, j = i % n16;
        out[i] = reinterpret_cast<const uint4*>(local_buf + half + r * slot_bytes)[j];
    }
}

SL_API int sl_gather_fetch(void* out, const void* local_buf, const void* epoch, int world, size_t slot_bytes, size_t bytes,
                           cudaStream_t s) {
    if (bytes == 0) return 0;
    if (bytes % 16 != 0 || bytes > slot_bytes) return -1;
    const size_t n16 = bytes / 16;
    int blocks = (int)((world * n16 + 255) / 256);
    if (blocks > 148) blocks = 148;
    sl_launch(gather_fetch_kernel, blocks, 256, 0, s, (uint4*)out, (const uint8_t*)local_buf, (const uint32_t*)epoch, world, slot_bytes, n16);
    return SL_LAUNCH_CHECK();
}

SL_API int sl_gather_push(const GatherPushCtx* c, const void* src, size_t bytes, cudaStream_t s) {
    if (bytes == 0) return 0;
    if (bytes % 16 != 0 || bytes > c->slot_bytes) return -1;
    const size_t n16 = bytes / 16;
    int blocks = (int)((n16 + 255) / 256);
    if (blocks > 148) blocks = 148;
    sl_launch(gather_push_kernel, blocks, 256, 0, s, *c, (const uint4*)src, n16);
    return SL_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// Peer mapping of the symmetric region through CUDA IPC (one process per GPU on one node).
// Every rank exports the allocation that holds its region, the 64-byte handles travel over the
// process group, every rank opens the others' handles (peer access is enabled lazily by the
// open).  Reference: `glm_cuda_ipc_get/open/close_mem_handle` (`csrc/glm_device.cpp`),
// `glm_p2p_enable_peer_access` (`csrc/glm_p2p.cu:723-744`).
#include <cuda.h>

typedef CUresult (*PFN_getAddressRange)(CUdeviceptr*, size_t*, CUdeviceptr);

SL_API int sl_ipc_export(const void* ptr, void* handle_out, unsigned long long* offset_out) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &q) != cudaSuccess || fn == nullptr) return -100;
    CUdeviceptr base = 0;
    size_t size = 0;
    if (((PFN_getAddressRange)fn)(&base, &size, (CUdeviceptr)ptr) != CUDA_SUCCESS) return -101;
    cudaIpcMemHandle_t h;
    const cudaError_t e = cudaIpcGetMemHandle(&h, (void*)base);
    if (e != cudaSuccess) return (int)e;
    memcpy(handle_out, &h, sizeof(h));
    *offset_out = (unsigned long long)((CUdeviceptr)ptr - base);
    return 0;
}

SL_API int sl_ipc_open(const void* handle, unsigned long long offset, void** ptr_out) {
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void* base = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return (int)e;
    *ptr_out = (char*)base + offset;
    return 0;
}

SL_API int sl_ipc_close(void* ptr, unsigned long long offset) {
    return (int)cudaIpcCloseMemHandle((char*)ptr - offset);
}
