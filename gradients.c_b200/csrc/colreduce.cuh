// Column sums over the rows of a [rows, cols] 16-bit matrix (optionally of an elementwise product
// with a second matrix and a per-row FP32 factor): y[c] = sum_r a[r, c] (* b[r, c] * f[r]).
// Used for bias gradients (gd_backend_reduce_rows) and the RMSNorm weight gradient. HBM-bound:
// every lane reads 16 bytes per row, a warp covers 256 adjacent columns of a row, the 8 warps of a
// block take rows round-robin with 4 rows in flight, partial sums per row chunk go to an FP32
// workspace [chunks, cols]; the block that arrives last at a column tile (ticket counter) sums the
// chunks in a fixed order and rounds once, so no second launch is needed and the result does not
// depend on which block was last.
#pragma once
#include "common.cuh"

namespace gdb_colreduce {

constexpr int TILE_COLS = 256, WARPS = 8;
constexpr int UNROLL = 8;   // rows in flight per warp (16 bytes per lane each)

// MUL: multiply by b[r, c] * f[r]. lda/ldb in elements. cols % 8 == 0, bases 16-byte aligned.
template <typename T, bool MUL>
__global__ void __launch_bounds__(256)
stage_kernel(const T *__restrict__ a, size_t lda, const T *__restrict__ b, size_t ldb, const float *__restrict__ f,
             float *__restrict__ partial, size_t rows, size_t cols, size_t chunk, T *__restrict__ y, unsigned *__restrict__ tickets)
{
    gdb_pdl_sync();
    __shared__ float sh[WARPS][TILE_COLS + 8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const size_t col = (size_t)blockIdx.x * TILE_COLS + (size_t)lane * 8;
    const size_t r0 = (size_t)blockIdx.y * chunk;
    const size_t r1 = r0 + chunk < rows ? r0 + chunk : rows;
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.0f;
    if (col < cols) {
        size_t r = r0 + warp;
        for (; r + (UNROLL - 1) * WARPS < r1; r += UNROLL * WARPS) {
            gdb_vec8<T> va[UNROLL], vb[MUL ? UNROLL : 1];
            float fr[MUL ? UNROLL : 1];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                va[u].raw = *reinterpret_cast<const uint4 *>(a + (r + u * WARPS) * lda + col);
                if (MUL) {
                    vb[MUL ? u : 0].raw = *reinterpret_cast<const uint4 *>(b + (r + u * WARPS) * ldb + col);
                    fr[MUL ? u : 0] = __ldg(&f[r + u * WARPS]);
                }
            }
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    acc[e] += MUL ? va[u].get(e) * vb[MUL ? u : 0].get(e) * fr[MUL ? u : 0] : va[u].get(e);
                }
            }
        }
        for (; r < r1; r += WARPS) {
            gdb_vec8<T> va, vb;
            va.raw = *reinterpret_cast<const uint4 *>(a + r * lda + col);
            float fr = 1.0f;
            if (MUL) {
                vb.raw = *reinterpret_cast<const uint4 *>(b + r * ldb + col);
                fr = __ldg(&f[r]);
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                acc[e] += MUL ? va.get(e) * vb.get(e) * fr : va.get(e);
            }
        }
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) sh[warp][lane * 8 + e] = acc[e];
    __syncthreads();
    const size_t c = (size_t)blockIdx.x * TILE_COLS + threadIdx.x;
    if (c < cols) {
        float s = 0.0f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) s += sh[w][threadIdx.x];
        partial[(size_t)blockIdx.y * cols + c] = s;
    }
    if (tickets == nullptr) {
        return;   // a separate final_kernel sums the chunks
    }
    __shared__ bool last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        last = atomicAdd(&tickets[blockIdx.x], 1U) == gridDim.y - 1U;
    }
    __syncthreads();
    if (last) {
        __threadfence();
        // warp w adds the chunks w, w + 8, ... for the lane's 8 columns; the warps' sums meet in shared memory
        float t8[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) t8[e] = 0.0f;
        if (col < cols) {
            for (unsigned k = warp; k < gridDim.y; k += WARPS) {
                const float4 p0 = __ldcg(reinterpret_cast<const float4 *>(partial + (size_t)k * cols + col));
                const float4 p1 = __ldcg(reinterpret_cast<const float4 *>(partial + (size_t)k * cols + col + 4));
                t8[0] += p0.x; t8[1] += p0.y; t8[2] += p0.z; t8[3] += p0.w;
                t8[4] += p1.x; t8[5] += p1.y; t8[6] += p1.z; t8[7] += p1.w;
            }
        }
        __syncthreads();   // sh is reused
#pragma unroll
        for (int e = 0; e < 8; ++e) sh[warp][lane * 8 + e] = t8[e];
        __syncthreads();
        if (c < cols) {
            float t = 0.0f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) t += sh[w][threadIdx.x];
            gdb_io<T>::st(y, c, t);
        }
        if (threadIdx.x == 0) tickets[blockIdx.x] = 0U;   // leave the counter ready for the next reduction
    }
}

// y[c] = round(sum_chunk partial[chunk, c]); block = 32 columns x 8 chunk groups.
template <typename T>
__global__ void __launch_bounds__(256)
final_kernel(const float *__restrict__ partial, T *__restrict__ y, size_t chunks, size_t cols)
{
    gdb_pdl_sync();
    __shared__ float sh[8][33];
    const int cx = threadIdx.x & 31, gy = threadIdx.x >> 5;
    const size_t c = (size_t)blockIdx.x * 32 + cx;
    float s = 0.0f;
    if (c < cols) {
        for (size_t k = gy; k < chunks; k += 8) s += partial[k * cols + c];
    }
    sh[gy][cx] = s;
    __syncthreads();
    if (gy == 0 && c < cols) {
        float t = 0.0f;
#pragma unroll
        for (int w = 0; w < 8; ++w) t += sh[w][cx];
        gdb_io<T>::st(y, c, t);
    }
}

static inline bool usable(const void *a, size_t lda, const void *b, size_t ldb, size_t cols)
{
    return (cols % 8U) == 0U && (lda % 8U) == 0U && ((uintptr_t)a % 16U) == 0U &&
           (b == NULL || ((ldb % 8U) == 0U && ((uintptr_t)b % 16U) == 0U));
}

// Number of row chunks: about four waves of blocks, at least 128 rows per chunk, capped by capacity.
static inline size_t pick_chunks(const gd_backend *be, size_t rows, size_t cols, size_t capacity_chunks)
{
    const size_t col_tiles = (cols + TILE_COLS - 1U) / TILE_COLS;
    size_t chunks = ((size_t)be->sm_count * 4U + col_tiles - 1U) / col_tiles;
    const size_t by_rows = (rows + 2U * UNROLL * WARPS - 1U) / (2U * UNROLL * WARPS);   // at least two unrolled sweeps per warp
    if (chunks > by_rows) chunks = by_rows;
    if (chunks > capacity_chunks) chunks = capacity_chunks;
    if (chunks > 65535U) chunks = 65535U;
    return chunks == 0U ? 1U : chunks;
}

template <typename T, bool MUL>
gd_status run(gd_backend *be, const void *a, size_t lda, const void *b, size_t ldb, const float *f, float *partial,
              size_t capacity_chunks, void *y, size_t rows, size_t cols)
{
    size_t chunks = pick_chunks(be, rows, cols, capacity_chunks);
    const size_t chunk = (rows + chunks - 1U) / chunks;
    chunks = (rows + chunk - 1U) / chunk;
    dim3 grid((unsigned)((cols + TILE_COLS - 1U) / TILE_COLS), (unsigned)chunks);
    const bool fused = grid.x <= (unsigned)GDB_TICKET_WORDS;
    gdb_launch(stage_kernel<T, MUL>, grid, 256, 0, be->stream, (const T *)a, lda, (const T *)b, ldb, f, partial, rows, cols, chunk, (T *)y,
                                                       fused ? gdb_tickets(be) : nullptr);
    gd_status st = gdb_launched(be, "column reduce stage");
    if (st != GD_OK || fused) {
        return st;
    }
    gdb_launch(final_kernel<T>, (unsigned)((cols + 31U) / 32U), 256, 0, be->stream, partial, (T *)y, chunks, cols);
    return gdb_launched(be, "column reduce final");
}

}  // namespace gdb_colreduce
