// Checkpoint reader of the host runtime: read-only file mappings and multi-threaded copies of strided windows.
//
// A tensor-parallel rank needs a window of most weight matrices: rows [r0, r1) of a column-parallel weight, columns
// [c0, c1) of a row-parallel one.  rt_mmap_copy_rows copies such a window - `rows` pieces of `row_bytes` bytes that lie
// `row_stride` bytes apart in the file - into one contiguous destination, normally a pinned host buffer from which a
// single asynchronous copy takes it to the GPU.  The pieces are split over a few threads, so the page faults of a cold
// mapping (the actual disk reads) overlap each other and the copy.
//
// Reference: `glm_mmap_open`, `glm_mmap_load`, `glm_mmap_close` (`csrc/glm_device.cpp:19-395`) and the strided TP upload of
// `loadTensorStrided` (`src/chat_model.ts:536-591`).
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#define RT_API extern "C" __attribute__((visibility("default")))

namespace {

struct Mapping {
    const uint8_t* data = nullptr;
    uint64_t size = 0;
};

void copy_piece(const uint8_t* src, uint64_t row_stride, uint64_t row_bytes, uint8_t* dst, uint64_t first, uint64_t last) {
    if (row_stride == row_bytes) {                       // the window is contiguous in the file
        std::memcpy(dst + first * row_bytes, src + first * row_stride, (last - first) * row_bytes);
        return;
    }
    for (uint64_t r = first; r < last; ++r) std::memcpy(dst + r * row_bytes, src + r * row_stride, row_bytes);
}

}  // namespace

// Maps `path` read-only.  Returns a handle (null on failure) and the file size.
RT_API void* rt_mmap_open(const char* path, uint64_t* size_out) {
    const int fd = ::open(path, O_RDONLY | O_CLOEXEC);
    if (fd < 0) return nullptr;
    struct stat st;
    if (::fstat(fd, &st) != 0 || st.st_size <= 0) {
        ::close(fd);
        return nullptr;
    }
    void* p = ::mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_SHARED, fd, 0);
    ::close(fd);                                          // the mapping keeps the file open
    if (p == MAP_FAILED) return nullptr;
    auto* m = new Mapping{static_cast<const uint8_t*>(p), (uint64_t)st.st_size};
    if (size_out != nullptr) *size_out = m->size;
    return m;
}

RT_API void rt_mmap_close(void* h) {
    auto* m = static_cast<Mapping*>(h);
    if (m == nullptr) return;
    ::munmap(const_cast<uint8_t*>(m->data), (size_t)m->size);
    delete m;
}

// Asks the kernel to start reading [offset, offset + length) (page-aligned outwards).  0 on success.
RT_API int rt_mmap_advise(void* h, uint64_t offset, uint64_t length) {
    auto* m = static_cast<Mapping*>(h);
    if (m == nullptr || offset > m->size || length > m->size - offset) return -1;
    const uint64_t page = (uint64_t)::sysconf(_SC_PAGESIZE);
    const uint64_t lo = offset / page * page;
    return ::madvise(const_cast<uint8_t*>(m->data) + lo, (size_t)(offset + length - lo), MADV_WILLNEED) == 0 ? 0 : -2;
}

// dst[r * row_bytes .. +row_bytes) = file[offset + r * row_stride .. +row_bytes) for r < rows, on up to `threads` threads.
// -1: the window does not lie inside the file (or a null argument); 0: copied.
RT_API int rt_mmap_copy_rows(void* h, uint64_t offset, uint64_t row_stride, uint64_t row_bytes, uint64_t rows, void* dst,
                             int threads) {
    auto* m = static_cast<Mapping*>(h);
    if (m == nullptr || (dst == nullptr && rows * row_bytes > 0)) return -1;
    if (rows == 0 || row_bytes == 0) return 0;
    if (row_stride < row_bytes && rows > 1) return -1;
    // last byte read: offset + (rows - 1) * row_stride + row_bytes, checked without overflow
    if (offset > m->size || row_bytes > m->size - offset) return -1;
    if (rows > 1 && (m->size - offset - row_bytes) / row_stride < rows - 1) return -1;
    const uint8_t* src = m->data + offset;
    uint8_t* out = static_cast<uint8_t*>(dst);
    const uint64_t total = rows * row_bytes;
    uint64_t n = threads < 1 ? 1 : (uint64_t)threads;
    n = std::min<uint64_t>(n, std::max<uint64_t>(1, total >> 20));       // at least 1 MiB of payload per thread
    n = std::min<uint64_t>(n, rows);
    if (n <= 1) {
        copy_piece(src, row_stride, row_bytes, out, 0, rows);
        return 0;
    }
    std::vector<std::thread> pool;
    const uint64_t per = (rows + n - 1) / n;
    for (uint64_t t = 0; t < n; ++t) {
        const uint64_t first = t * per, last = std::min(rows, first + per);
        if (first >= last) break;
        pool.emplace_back(copy_piece, src, row_stride, row_bytes, out, first, last);
    }
    for (auto& th : pool) th.join();
    return 0;
}
