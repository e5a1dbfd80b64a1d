// Producer-side half of the fused compute + all-reduce: a kernel's epilogue stores its partial
// result straight into every rank's receive slot over NVLink peer mappings (plain st.global, no
// multicast).  Every fp32 value travels as an 8-byte word {value bits, tag} written by one
// 8-byte store; tag = (number of collectives completed on this buffer) + 1.  The consumer
// (`ar_add_rmsnorm_kernel`, csrc/comm.cu) polls each word until its tag matches, so neither side
// needs a memory fence, a block counter or a separate flag store: the latency of the exchange
// is one NVLink store plus the poll.  (A system-scope fence per producer block cost more than
// the GEMM itself at decode sizes.)  Buffers alternate between uses, so a producer can only
// overwrite a slot after every rank has consumed its previous content.
//
// The reference does the same exchange with separate kernels: `p2p_reduce_scatter_write_kernel`
// + `p2p_barrier_kernel` + `p2p_reduce_gather_write_kernel` (`csrc/glm_p2p.cu:560-700`).
#pragma once

#include "common.cuh"

#define SL_MAX_RANKS 8

struct PushCtx {
    uint2* bufs[SL_MAX_RANKS];        // receive buffer of each rank: [world][slot_rows][row_len] {value, tag}
    uint32_t* flags[SL_MAX_RANKS];    // unused by the tagged protocol (kept for the flag-based collectives)
    const uint32_t* epoch;            // local: number of completed collectives on this buffer
    uint32_t* block_counter;          // unused by the tagged protocol
    int rank, world;
    int slot_rows, row_len;           // receive slot geometry
};

// Tag of the collective in flight on this buffer (read once per thread).
__device__ __forceinline__ uint32_t push_tag(const PushCtx& c) { return *c.epoch + 1u; }

// Store element (row, col) of this rank's partial into peer p's receive slot.
__device__ __forceinline__ void push_store(const PushCtx& c, int p, int row, int col, float v, uint32_t tag) {
    uint2* dst = c.bufs[p] + ((size_t)c.rank * c.slot_rows + row) * c.row_len + col;
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(dst), "r"(__float_as_uint(v)), "r"(tag) : "memory");
}

// ... and into every rank's slot (including this rank's own).
__device__ __forceinline__ void push_store_all(const PushCtx& c, int row, int col, float v, uint32_t tag) {
    for (int p = 0; p < c.world; ++p) push_store(c, p, row, col, v, tag);
}
