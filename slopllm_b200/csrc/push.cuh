// Producer-side half of the fused compute + all-reduce: a kernel's epilogue stores its partial
// result straight into every rank's receive slot over NVLink peer mappings (plain st.global, no
// multicast).  Every value travels as a 4-byte word {bf16 value in the high half, 16-bit tag in the
// low half} written by one store; tag = (number of collectives completed on this buffer) mod
// 65535 + 1, never 0.  The consumer (`ar_add_rmsnorm_kernel`, csrc/comm.cu) polls each word until
// its tag matches, so neither side needs a memory fence, a block counter or a separate flag store:
// the latency of the exchange is one NVLink store plus the poll.  (A system-scope fence per
// producer block cost more than the GEMM itself at decode sizes.)  Buffers alternate between uses,
// so a producer can only overwrite a slot after every rank has consumed its previous content; the
// consumer zeroes every word it has used, so a slot that later collectives do not write (a row
// beyond their row count) never holds a tag that a wrapped counter could match.
// The partial sums cross the link rounded to bf16 (the reference all-reduces bf16 too) and are
// summed in fp32; 4-byte words halve the NVLink bytes of the 8-byte {fp32, tag} form, which bound
// the exchange from 8 rows x 8 ranks up.
//
// The reference does the same exchange with separate kernels: `p2p_reduce_scatter_write_kernel`
// + `p2p_barrier_kernel` + `p2p_reduce_gather_write_kernel` (`csrc/glm_p2p.cu:560-700`).
#pragma once

#include "common.cuh"

#define SL_MAX_RANKS 8

struct PushCtx {
    uint32_t* bufs[SL_MAX_RANKS];     // receive buffer of each rank: [world][slot_rows][row_len] words {bf16 value, tag}
    uint32_t* flags[SL_MAX_RANKS];    // unused by the tagged protocol (kept for the flag-based collectives)
    const uint32_t* epoch;            // local: number of completed collectives on this buffer
    uint32_t* block_counter;          // unused by the tagged protocol
    int rank, world;
    int slot_rows, row_len;           // receive slot geometry
};

// Tag of the collective in flight on this buffer (read once per thread).
__device__ __forceinline__ uint32_t push_tag_of(uint32_t epoch) { return epoch % 65535u + 1u; }
__device__ __forceinline__ uint32_t push_tag(const PushCtx& c) { return push_tag_of(*c.epoch); }

// Store element (row, col) of this rank's partial into peer p's receive slot.
__device__ __forceinline__ void push_store(const PushCtx& c, int p, int row, int col, float v, uint32_t tag) {
    uint32_t* dst = c.bufs[p] + ((size_t)c.rank * c.slot_rows + row) * c.row_len + col;
    const uint32_t word = ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(v)) << 16) | tag;
    asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(dst), "r"(word) : "memory");
}

// ... and into every rank's slot (including this rank's own).
__device__ __forceinline__ void push_store_all(const PushCtx& c, int row, int col, float v, uint32_t tag) {
    for (int p = 0; p < c.world; ++p) push_store(c, p, row, col, v, tag);
}
