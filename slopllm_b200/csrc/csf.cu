// GPU decoder of the NVFP4 compressed-scale planes (`byte-window4-fixed-stream-u24-exceptions/1`):
// out[r, c] = base[row0 + r] + nibble(row0 + r, col0 + c), then replacement words are applied, then the
// decoded window is validated.  A TP rank decodes only its window (row0/col0/out_rows/out_cols) of the
// logical [rows, cols] scale matrix.  Contract violations set bits in a status word instead of
// trapping:  1 = scale code above 0x7e,  2 = exception words unsorted / out of range,  4 = row base
// above 240.  Reference: `csf_expand_kernel` / `csf_exceptions_kernel` / `csf_validate_kernel`
// (`csrc/glm_ops.cu:1346-1405`).
#include "common.cuh"

__global__ void csf_expand_kernel(uint8_t* __restrict__ out, const uint8_t* __restrict__ fixed, int cols, int row0, int col0,
                                  int out_rows, int out_cols, int* __restrict__ status) {
    const int sel = cols / 2, stride = 16 * (1 + sel);
    const size_t total = (size_t)out_rows * out_cols;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int r = (int)(i / out_cols), c = (int)(i % out_cols);
        const int row = row0 + r, col = col0 + c;
        const uint8_t* slab = fixed + (size_t)(row / 16) * stride;
        const int base = slab[row % 16];
        if (base > 240) atomicOr(status, 4);
        const uint8_t b = slab[16 + (row % 16) * sel + (col >> 1)];
        out[i] = (uint8_t)(base + ((col & 1) ? (b >> 4) : (b & 0x0f)));
    }
}

__global__ void csf_exceptions_kernel(uint8_t* __restrict__ out, const uint32_t* __restrict__ words, int n, int rows, int cols,
                                      int row0, int col0, int out_rows, int out_cols, int* __restrict__ status) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint32_t w = words[i];
    const uint32_t pos = w & 0xffffffu;
    if (pos >= (uint32_t)rows * (uint32_t)cols || (i > 0 && (words[i - 1] & 0xffffffu) >= pos)) {
        atomicOr(status, 2);
        return;
    }
    const int row = (int)(pos / cols) - row0, col = (int)(pos % cols) - col0;
    if (row >= 0 && row < out_rows && col >= 0 && col < out_cols) out[(size_t)row * out_cols + col] = (uint8_t)(w >> 24);
}

__global__ void csf_validate_kernel(const uint8_t* __restrict__ out, size_t total, int* __restrict__ status) {
    bool bad = false;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        bad |= out[i] > 0x7e;
    if (bad) atomicOr(status, 1);
}

SL_API int sl_csf_decode(void* out, const void* fixed, const void* exceptions, int n_exceptions, int rows, int cols, int row0,
                         int out_rows, int col0, int out_cols, void* status, cudaStream_t s) {
    if (rows <= 0 || cols <= 0 || rows % 16 || cols % 2 || row0 < 0 || col0 < 0 || row0 + out_rows > rows ||
        col0 + out_cols > cols)
        return -1;
    const size_t total = (size_t)out_rows * out_cols;
    if (total == 0) return 0;
    int blocks = (int)((total + 255) / 256);
    if (blocks > 148 * 8) blocks = 148 * 8;
    csf_expand_kernel<<<blocks, 256, 0, s>>>((uint8_t*)out, (const uint8_t*)fixed, cols, row0, col0, out_rows, out_cols, (int*)status);
    if (n_exceptions > 0)
        csf_exceptions_kernel<<<(n_exceptions + 255) / 256, 256, 0, s>>>((uint8_t*)out, (const uint32_t*)exceptions, n_exceptions, rows,
                                                                        cols, row0, col0, out_rows, out_cols, (int*)status);
    csf_validate_kernel<<<blocks, 256, 0, s>>>((const uint8_t*)out, total, (int*)status);
    return SL_LAUNCH_CHECK();
}
