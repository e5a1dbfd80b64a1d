// Producer-side half of the fused compute + all-reduce: a kernel's epilogue stores its partial
// result straight into every rank's receive slot over NVLink peer mappings (plain st.global, no
// multicast) and the last block of the grid publishes an epoch flag to each peer with
// st.release.sys.  The consumer (`ar_add_rmsnorm_kernel`, csrc/comm.cu) waits for the flags of
// all ranks with a bounded spin, then reduces its local slots in rank order.
//
// The reference does the same exchange with separate kernels: `p2p_reduce_scatter_write_kernel`
// + `p2p_barrier_kernel` + `p2p_reduce_gather_write_kernel` (`csrc/glm_p2p.cu:560-700`).
#pragma once

#include "common.cuh"

#define SL_MAX_RANKS 8

struct PushCtx {
    float* bufs[SL_MAX_RANKS];        // receive buffer of each rank: [world][slot_rows][row_len] fp32
    uint32_t* flags[SL_MAX_RANKS];    // flag array of each rank: [world] (one word per source rank)
    const uint32_t* epoch;            // local: number of completed collectives on this buffer
    uint32_t* block_counter;          // local: blocks of the current producer grid that have finished
    int rank, world;
    int slot_rows, row_len;           // receive slot geometry
};

// Address of element (row, col) of this rank's slot in peer p's receive buffer.
__device__ __forceinline__ float* push_dst(const PushCtx& c, int p, int row, int col) {
    return c.bufs[p] + ((size_t)c.rank * c.slot_rows + row) * c.row_len + col;
}

// Call once per block after its last store (all threads).  The last block to arrive publishes
// flag = epoch + 1 to every rank (including itself).
__device__ __forceinline__ void push_finish(const PushCtx& c, unsigned total_blocks) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        const unsigned prev = atomicAdd(c.block_counter, 1u);
        if (prev == total_blocks - 1) {
            *c.block_counter = 0;
            __threadfence_system();
            const uint32_t e = *c.epoch + 1u;
            for (int p = 0; p < c.world; ++p) st_relaxed_sys_u32(c.flags[p] + c.rank, e);
        }
    }
}
