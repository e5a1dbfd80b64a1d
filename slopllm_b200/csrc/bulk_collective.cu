// All-reduce of prefill-sized partial sums ([T, H] with thousands of rows) as reduce-scatter + all-gather over
// NVLink peer memory, fused with its neighbours:
//
//   producer   the tcgen05 GEMM's epilogue (sl_gemm_bf16_tcgen05_rs, csrc/gemm_tcgen05.cu) stores each bf16 tile
//              row into the staging area of the rank that owns the row while later tiles are still being computed,
//              and counts the delivered columns in the owner's per-32-row arrival counter.  rs_push_rows_kernel
//              does the same for a tensor that already exists (producers without a fused epilogue).
//   owner      rs_reduce_ag_kernel: per owned row, a block waits (bounded) until world * H columns of its 32-row
//              group have arrived, sums the `world` staged rows in rank order (deterministic), and stores the bf16
//              sum into every rank's gathered buffer, then counts one arrival per row on every rank.
//   consumer   bulk_add_rmsnorm_kernel: per row, a block waits (bounded) until the owner of the row has delivered
//              all of its rows, then residual add + RMSNorm in the same pass.
//
// Rank o owns rows [o * R, (o + 1) * R), R = T / world (R % 32 == 0).  Counters count "arrivals of this use" and are
// set back to zero by the last block that has passed its wait; a counter cannot receive an arrival of the next use
// before that, because a rank starts its next producer only after its consumer kernel, which needs every owner's rows,
// each of which is sent after the owner's block has passed (and possibly reset) its counter.  For the same reason one
// staging area and one gathered buffer suffice - as long as the three kernels of consecutive uses run in one stream.
// Plain peer loads / stores and `red` only (no multimem, no multicast).  On a timeout the kernels record
// {1, site, expected, observed} in `status` and finish with whatever has arrived; the host raises after the step.
//
// Reference: `p2p_reduce_scatter_write_kernel` + barrier + `p2p_reduce_gather_write_kernel` + barrier +
// `fused_add_rmsnorm_kernel` (`csrc/glm_p2p.cu:560-700`, `csrc/glm_ops.cu:358`), five launches after the GEMM.
#include "push.cuh"

struct BulkCtx {
    bf16* stage[SL_MAX_RANKS];           // rank r's staging area [world][R][H]
    uint32_t* rs_count[SL_MAX_RANKS];    // rank r's arrival counters, one per 32-row group of its slice
    bf16* full[SL_MAX_RANKS];            // rank r's gathered sums [world * R][H]
    uint32_t* ag_count[SL_MAX_RANKS];    // rank r's arrival counters, one per source rank
    uint32_t* rs_done;                   // local: blocks past their wait, per 32-row group
    uint32_t* ag_done;                   // local: blocks past their wait, per source rank
    int* status;                         // local: [4] error record
    int rank, world, slot_rows, row_len; // R, H of this use
    uint32_t max_spins;
};

namespace {

__device__ __forceinline__ void acc8(float (&a)[8], const uint4& v) {
    const float2 p0 = bf162_to_f2(v.x), p1 = bf162_to_f2(v.y), p2 = bf162_to_f2(v.z), p3 = bf162_to_f2(v.w);
    a[0] += p0.x; a[1] += p0.y; a[2] += p1.x; a[3] += p1.y;
    a[4] += p2.x; a[5] += p2.y; a[6] += p3.x; a[7] += p3.y;
}

__device__ __forceinline__ uint4 pack8(const float (&a)[8]) {
    return make_uint4(f2_to_bf162(a[0], a[1]), f2_to_bf162(a[2], a[3]), f2_to_bf162(a[4], a[5]), f2_to_bf162(a[6], a[7]));
}

// One block per 32-row group of x [T, H] (fp32 or bf16, row stride ldx elements).
template <bool F32>
__global__ void __launch_bounds__(256) rs_push_rows_kernel(BulkCtx c, const void* __restrict__ x, int ldx) {
    pdl_grid_sync();
    const int row0 = blockIdx.x * 32, R = c.slot_rows, H = c.row_len;
    const int owner = row0 / R;
    const int units = H / 8;
    bf16* dst0 = c.stage[owner] + ((size_t)c.rank * R + (row0 - owner * R)) * H;
    for (int i = threadIdx.x; i < 32 * units; i += blockDim.x) {
        const int r = i / units, u = i % units;
        uint4 v;
        if (F32) {
            const float4* src = reinterpret_cast<const float4*>((const float*)x + (size_t)(row0 + r) * ldx + u * 8);
            const float4 a = src[0], b = src[1];
            v = make_uint4(f2_to_bf162(a.x, a.y), f2_to_bf162(a.z, a.w), f2_to_bf162(b.x, b.y), f2_to_bf162(b.z, b.w));
        } else {
            v = *reinterpret_cast<const uint4*>((const bf16*)x + (size_t)(row0 + r) * ldx + u * 8);
        }
        *reinterpret_cast<uint4*>(dst0 + (size_t)r * H + u * 8) = v;
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) red_release_sys_add_u32(c.rs_count[owner] + (row0 - owner * R) / 32, (uint32_t)H);
}

// Blocks walk the owned rows (row i, i + gridDim.x, ...).  The grid is at most two blocks per SM: a block that is
// waiting for other GPUs must not keep kernels of another stream (the other half-chunk of a phased prefill, whose
// progress the other GPUs may in turn be waiting for) off the SMs.
__global__ void __launch_bounds__(256) rs_reduce_ag_kernel(BulkCtx c) {
    pdl_grid_sync();
    const int R = c.slot_rows, H = c.row_len, W = c.world;
    for (int i = blockIdx.x; i < R; i += gridDim.x) {
        const int g = i / 32;
        if (threadIdx.x == 0) {
            uint32_t* cnt = c.rs_count[c.rank] + g;
            wait_flag_geq(cnt, (uint32_t)W * (uint32_t)H, c.max_spins, c.status, 20);
            // the last of the group's 32 blocks to get here sets the counter back for the next use
            if (atomicAdd(c.rs_done + g, 1u) == 31u) {
                atomicExch(cnt, 0u);
                atomicExch(c.rs_done + g, 0u);
            }
        }
        __syncthreads();
        const bf16* mine = c.stage[c.rank];
        const size_t out_off = ((size_t)c.rank * R + i) * H;
        for (int u = threadIdx.x; u < H / 8; u += blockDim.x) {
            float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int r = 0; r < W; ++r)                       // rank order: every rank would get the same bits
                acc8(a, __ldcg(reinterpret_cast<const uint4*>(mine + ((size_t)r * R + i) * H + u * 8)));
            const uint4 v = pack8(a);
            for (int k = 0; k < W; ++k) {                     // start at the own copy, then one peer after the other
                const int p = (c.rank + k) % W;
                *reinterpret_cast<uint4*>(c.full[p] + out_off + u * 8) = v;
            }
        }
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x < W) red_release_sys_add_u32(c.ag_count[threadIdx.x] + c.rank, 1u);
    }
}

// Blocks walk the rows of the full [T, H] result (same bound on the grid as above); a thread owns up to NORM_MAX_U
// 16-byte units of a row.
constexpr int NORM_THREADS = 256, NORM_MAX_U = 8;       // H <= 256 * 8 * 8 = 16384

__global__ void __launch_bounds__(NORM_THREADS) bulk_add_rmsnorm_kernel(BulkCtx c, bf16* __restrict__ out, float* __restrict__ res_out,
                                                                        const float* __restrict__ res_in, const bf16* __restrict__ w,
                                                                        float eps) {
    pdl_grid_sync();
    __shared__ float scratch[33];
    const int R = c.slot_rows, H = c.row_len, T = c.world * c.slot_rows;
    for (int t = blockIdx.x; t < T; t += gridDim.x) {
        const int src = t / R;
        if (threadIdx.x == 0) {
            uint32_t* cnt = c.ag_count[c.rank] + src;
            wait_flag_geq(cnt, (uint32_t)R, c.max_spins, c.status, 21);
            if (atomicAdd(c.ag_done + src, 1u) == (uint32_t)R - 1u) {
                atomicExch(cnt, 0u);
                atomicExch(c.ag_done + src, 0u);
            }
        }
        __syncthreads();
        const bf16* x = c.full[c.rank] + (size_t)t * H;
        const int units = H / 8;
        float v[NORM_MAX_U][8];
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < NORM_MAX_U; ++k) {
            const int u = threadIdx.x + k * NORM_THREADS;
            if (u < units) {
#pragma unroll
                for (int j = 0; j < 8; ++j) v[k][j] = 0.f;
                acc8(v[k], __ldcg(reinterpret_cast<const uint4*>(x + u * 8)));
                if (res_in != nullptr) {
                    const float4* rp = reinterpret_cast<const float4*>(res_in + (size_t)t * H + u * 8);
                    const float4 a = rp[0], b = rp[1];
                    v[k][0] += a.x; v[k][1] += a.y; v[k][2] += a.z; v[k][3] += a.w;
                    v[k][4] += b.x; v[k][5] += b.y; v[k][6] += b.z; v[k][7] += b.w;
                }
                float4* ro = reinterpret_cast<float4*>(res_out + (size_t)t * H + u * 8);
                ro[0] = make_float4(v[k][0], v[k][1], v[k][2], v[k][3]);
                ro[1] = make_float4(v[k][4], v[k][5], v[k][6], v[k][7]);
#pragma unroll
                for (int j = 0; j < 8; ++j) ss += v[k][j] * v[k][j];
            }
        }
        ss = block_sum(ss, scratch);
        const float inv = rsqrtf(ss / (float)H + eps);
#pragma unroll
        for (int k = 0; k < NORM_MAX_U; ++k) {
            const int u = threadIdx.x + k * NORM_THREADS;
            if (u < units) {
                const uint4 wv = *reinterpret_cast<const uint4*>(w + u * 8);
                float g[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                acc8(g, wv);
                float o[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = v[k][j] * inv * g[j];
                *reinterpret_cast<uint4*>(out + (size_t)t * H + u * 8) = pack8(o);
            }
        }
    }
}

// Two blocks per SM at most, see rs_reduce_ag_kernel.
int waiting_grid(int rows) {
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    return rows < 2 * sms ? rows : 2 * sms;
}

int check_ctx(const BulkCtx* c) {
    if (c == nullptr || c->world < 1 || c->world > SL_MAX_RANKS || c->rank < 0 || c->rank >= c->world) return -1;
    if (c->slot_rows <= 0 || c->slot_rows % 32 != 0 || c->row_len <= 0 || c->row_len % 8 != 0) return -1;
    return 0;
}

}  // namespace

// Producer for a tensor that already exists: x [world * R, H], fp32 (x_f32) or bf16, row stride ldx elements
// (ldx % 8 == 0).  Rows are stored as bf16 into their owners' staging areas.
SL_API int sl_rs_push_rows(const BulkCtx* c, const void* x, int ldx, int x_f32, cudaStream_t s) {
    if (check_ctx(c) || x == nullptr || ldx % 8 != 0 || ldx < c->row_len) return -1;
    const int groups = c->world * c->slot_rows / 32;
    if (x_f32) sl_launch(rs_push_rows_kernel<true>, groups, 256, 0, s, *c, x, ldx);
    else sl_launch(rs_push_rows_kernel<false>, groups, 256, 0, s, *c, x, ldx);
    return SL_LAUNCH_CHECK();
}

// Owner step: reduce this rank's R rows over the `world` staged partials and store the sums on every rank.
SL_API int sl_rs_reduce_ag(const BulkCtx* c, cudaStream_t s) {
    if (check_ctx(c)) return -1;
    sl_launch(rs_reduce_ag_kernel, waiting_grid(c->slot_rows), 256, 0, s, *c);
    return SL_LAUNCH_CHECK();
}

// Consumer: out[t] = RMSNorm(res_in[t] + sum[t]) * w (bf16), res_out[t] = res_in[t] + sum[t] (fp32) for all world * R rows.
// res_in may be null.
SL_API int sl_bulk_add_rmsnorm(const BulkCtx* c, void* out, void* res_out, const void* res_in, const void* w, float eps,
                               cudaStream_t s) {
    if (check_ctx(c) || out == nullptr || res_out == nullptr || w == nullptr) return -1;
    if (c->row_len > NORM_THREADS * NORM_MAX_U * 8) return -1;
    sl_launch(bulk_add_rmsnorm_kernel, waiting_grid(c->world * c->slot_rows), NORM_THREADS, 0, s, *c, (bf16*)out, (float*)res_out,
              (const float*)res_in, (const bf16*)w, eps);
    return SL_LAUNCH_CHECK();
}
