// Tensor-core flash attention for packed variable-length causal sequences (forward and backward).
//
// Fast path of gd_backend_sdpa_varlen / _backward for 16-bit storage, head_dim 64 or 128, causal,
// optional sliding window, no prefix, grouped-query heads. Other configurations return
// GD_ERR_UNSUPPORTED and run on the general kernels of attention.cu.
//
// Work is cut in 64-row chunks of the PACKED token stream, not per sequence: a chunk may span
// several sequences. Every query row carries the start of its own sequence and every key row the end
// of its own sequence (binary search in cu_seqlens), and the mask is evaluated in packed coordinates:
//   allowed(i, j)  <=>  seg_start(i) <= j <= i  and  (window == 0 or i - j < window)
// which is the reference's rule (src/ops/sdpa_varlen/metal_sdpa_varlen.metal:30-55) for prefix 0.
// No work list and no per-sequence launch geometry are needed, and short sequences waste nothing
// (the reference's per-sequence launch wastes 2.66x on its data, docs/optim_quickwins.md:450-457).
//
// Math (FP32 softmax, exp2 with log2(e) folded into the scale):
//   forward : online softmax over key tiles, O = P V, stats = (row max, sum of exp, 0)
//   backward 1 (query-stationary): P from the saved stats, dP = dO V^T, D = rowsum(P o dP),
//             dQ = scale * (sum_j P dP k_j - D * sum_j P k_j); D goes to stats[.., 2]
//   backward 2 (key-stationary)  : S^T = K Q^T, dP^T = V dO^T, dS^T = P^T o (dP^T - D) * scale,
//             dV += P^T dO, dK += dS^T Q, summed over the query heads of the group
// The output tensor of the forward pass is not an input of the reference's backward entry
// (src/core/backend.h:699-709), hence D is computed from P and dP instead of rowsum(dO o O).
//
// Tensor cores are driven with mma.sync.m16n8k16 (legacy path): tiles are at most 64 x 64 x 128 and
// the kernels are latency- and softmax-bound at the model's sequence lengths (<= 512).
#include "attention.cuh"

#include <math.h>

namespace {

constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

struct flash_params {
    int n_tokens, batch, hq, hkv, dh, window;
    float scale;
};

__device__ __forceinline__ int seg_of(const int *cu, int batch, int row)
{
    int lo = 0, hi = batch;
    while (lo + 1 < hi) {
        const int mid = (lo + hi) >> 1;
        if (cu[mid] <= row) lo = mid; else hi = mid;
    }
    return lo;
}

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void *dst, const void *src, bool valid)
{
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void *p)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void *p)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}

template <typename T> struct mma16816;
template <> struct mma16816<__half> {
    static __device__ __forceinline__ void run(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
    {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    static __device__ __forceinline__ uint32_t pack(float x, float y)
    {
        const __half2 h = __floats2half2_rn(x, y);
        return *reinterpret_cast<const uint32_t *>(&h);
    }
};
template <> struct mma16816<__nv_bfloat16> {
    static __device__ __forceinline__ void run(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
    {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    static __device__ __forceinline__ uint32_t pack(float x, float y)
    {
        const __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
        return *reinterpret_cast<const uint32_t *>(&h);
    }
};

// Copy `rows` x DH 16-bit elements (row r of the tile = packed row row0 + r, head `head` of `heads`)
// into a padded shared tile; rows at or beyond n_rows are zero-filled. 128 threads.
template <typename T, int DH, int ROWS>
__device__ __forceinline__ void load_tile(T *dst, const T *src, int row0, int n_rows, int heads, int head)
{
    constexpr int LD = DH + 8, CHUNKS = DH / 8;
    for (int c = threadIdx.x; c < ROWS * CHUNKS; c += 128) {
        const int r = c / CHUNKS, ch = c - r * CHUNKS;
        const int row = row0 + r;
        const bool ok = row >= 0 && row < n_rows;
        const T *s = src + ((size_t)(ok ? row : 0) * heads + head) * DH + ch * 8;
        cp_async16(dst + r * LD + ch * 8, s, ok);
    }
}

// A fragment (16 x 16) at (row0, col0) of a padded tile.
template <int LD, typename T>
__device__ __forceinline__ void load_a(uint32_t (&a)[4], const T *tile, int row0, int col0, int lane)
{
    ldmatrix_x4(a, tile + (row0 + (lane & 15)) * LD + col0 + (lane >> 4) * 8);
}
// B fragments of two adjacent n-tiles (n0..n0+15) for k0..k0+15 from a tile stored [n][k].
template <int LD, typename T>
__device__ __forceinline__ void load_b_nk(uint32_t (&b)[4], const T *tile, int n0, int k0, int lane)
{
    ldmatrix_x4(b, tile + (n0 + (lane & 7) + (lane >> 4) * 8) * LD + k0 + ((lane >> 3) & 1) * 8);
}
// B fragments of two adjacent n-tiles for k0..k0+15 from a tile stored [k][n].
template <int LD, typename T>
__device__ __forceinline__ void load_b_kn(uint32_t (&b)[4], const T *tile, int k0, int n0, int lane)
{
    ldmatrix_x4_trans(b, tile + (k0 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + n0 + (lane >> 4) * 8);
}

__device__ __forceinline__ float quad_max(float v)
{
    v = fmaxf(v, __shfl_xor_sync(0xffffffffU, v, 1));
    return fmaxf(v, __shfl_xor_sync(0xffffffffU, v, 2));
}
__device__ __forceinline__ float quad_sum(float v)
{
    v += __shfl_xor_sync(0xffffffffU, v, 1);
    return v + __shfl_xor_sync(0xffffffffU, v, 2);
}

// ------------------------------------------------------------------------------------------------
// Query-stationary kernel. MODE 0: forward (out + optional stats). MODE 1: statistics only.
// MODE 2: backward part 1 (dQ and D from saved statistics).
// grid = (ceil(N / 64), Hq), 128 threads; warp w owns query rows 16w..16w+15 of the chunk.
// ------------------------------------------------------------------------------------------------
template <typename T, int DH, int BKV, int MODE>
__global__ void __launch_bounds__(128, 3)
flash_q_kernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v, const T *__restrict__ go,
               const int *__restrict__ cu, T *__restrict__ out, float *__restrict__ stats, flash_params p)
{
    gdb_pdl_sync();
    constexpr int LD = DH + 8, BQ = 64, NT = BKV / 8, KT = DH / 16;
    extern __shared__ __align__(16) unsigned char fsm[];
    T *Qs = reinterpret_cast<T *>(fsm);
    T *Gs = Qs + BQ * LD;                                   // dO tile (MODE 2 only)
    T *Ks = Gs + (MODE == 2 ? BQ * LD : 0);                 // [2][BKV][LD]
    T *Vs = Ks + 2 * BKV * LD;                              // [2][BKV][LD]

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int q0 = blockIdx.x * BQ, h = blockIdx.y, hk = h / (p.hq / p.hkv);
    const int n_valid = min(cu[p.batch], p.n_tokens);
    const int rowA = q0 + warp * 16 + g, rowB = rowA + 8;
    const size_t oA = ((size_t)rowA * p.hq + h) * DH, oB = ((size_t)rowB * p.hq + h) * DH;

    if (q0 >= n_valid) {
        // rows behind the last sequence: zero output / gradient
        if constexpr (MODE != 1) {
#pragma unroll
            for (int n = 0; n < DH / 8; ++n) {
                if (rowA < p.n_tokens) *reinterpret_cast<uint32_t *>(out + oA + n * 8 + 2 * t) = 0U;
                if (rowB < p.n_tokens) *reinterpret_cast<uint32_t *>(out + oB + n * 8 + 2 * t) = 0U;
            }
        }
        return;
    }
    const int startA = rowA < n_valid ? cu[seg_of(cu, p.batch, rowA)] : 0x7fffffff;
    const int startB = rowB < n_valid ? cu[seg_of(cu, p.batch, rowB)] : 0x7fffffff;
    int kv_lo = cu[seg_of(cu, p.batch, q0)];
    if (p.window > 0) kv_lo = max(kv_lo, q0 - p.window + 1);
    const int kv_hi = min(q0 + BQ, n_valid);                // exclusive
    const int tile0 = kv_lo / BKV, n_tiles = (kv_hi - 1) / BKV - tile0 + 1;

    load_tile<T, DH, BQ>(Qs, q, q0, n_valid, p.hq, h);
    if constexpr (MODE == 2) load_tile<T, DH, BQ>(Gs, go, q0, n_valid, p.hq, h);
    load_tile<T, DH, BKV>(Ks, k, tile0 * BKV, n_valid, p.hkv, hk);
    load_tile<T, DH, BKV>(Vs, v, tile0 * BKV, n_valid, p.hkv, hk);
    cp_async_commit();

    const float sl2 = p.scale * LOG2E;
    float mA = -INFINITY, mB = -INFINITY, lA = 0.0f, lB = 0.0f;   // MODE 0/1: running max (log2 domain) and partial sums
    float invA = 0.0f, invB = 0.0f, dA = 0.0f, dB = 0.0f;          // MODE 2: 1/l and partial D
    if constexpr (MODE == 2) {
        if (rowA < n_valid) {
            const float *s = stats + ((size_t)rowA * p.hq + h) * 3;
            mA = s[0] * LOG2E;
            invA = s[1] > 0.0f ? 1.0f / s[1] : 0.0f;
        }
        if (rowB < n_valid) {
            const float *s = stats + ((size_t)rowB * p.hq + h) * 3;
            mB = s[0] * LOG2E;
            invB = s[1] > 0.0f ? 1.0f / s[1] : 0.0f;
        }
        if (mA == -INFINITY) mA = 0.0f;
        if (mB == -INFINITY) mB = 0.0f;
    }
    float acc[DH / 8][4];        // MODE 0: O;  MODE 2: sum P dP k
    float acc2[MODE == 2 ? DH / 8 : 1][4];  // MODE 2: sum P k
#pragma unroll
    for (int n = 0; n < DH / 8; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            acc[n][e] = 0.0f;
            if constexpr (MODE == 2) acc2[n][e] = 0.0f;
        }
    }

    for (int it = 0; it < n_tiles; ++it) {
        const int st = it & 1;
        if (it + 1 < n_tiles) {
            load_tile<T, DH, BKV>(Ks + (st ^ 1) * BKV * LD, k, (tile0 + it + 1) * BKV, n_valid, p.hkv, hk);
            load_tile<T, DH, BKV>(Vs + (st ^ 1) * BKV * LD, v, (tile0 + it + 1) * BKV, n_valid, p.hkv, hk);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const T *Kt = Ks + st * BKV * LD, *Vt = Vs + st * BKV * LD;
        const int kv0 = (tile0 + it) * BKV;

        float s[NT][4], dp[MODE == 2 ? NT : 1][4];
#pragma unroll
        for (int n = 0; n < NT; ++n) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                s[n][e] = 0.0f;
                if constexpr (MODE == 2) dp[n][e] = 0.0f;
            }
        }
#pragma unroll
        for (int kk = 0; kk < KT; ++kk) {
            uint32_t a[4], ag[4];
            load_a<LD>(a, Qs, warp * 16, kk * 16, lane);
            if constexpr (MODE == 2) load_a<LD>(ag, Gs, warp * 16, kk * 16, lane);
#pragma unroll
            for (int np = 0; np < NT / 2; ++np) {
                uint32_t b[4];
                load_b_nk<LD>(b, Kt, np * 16, kk * 16, lane);
                mma16816<T>::run(s[2 * np], a, b[0], b[1]);
                mma16816<T>::run(s[2 * np + 1], a, b[2], b[3]);
                if constexpr (MODE == 2) {
                    load_b_nk<LD>(b, Vt, np * 16, kk * 16, lane);
                    mma16816<T>::run(dp[2 * np], ag, b[0], b[1]);
                    mma16816<T>::run(dp[2 * np + 1], ag, b[2], b[3]);
                }
            }
        }
        // scale, mask
        float tmaxA = -INFINITY, tmaxB = -INFINITY;
#pragma unroll
        for (int n = 0; n < NT; ++n) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = kv0 + n * 8 + 2 * t + (e & 1);
                const int i = (e < 2) ? rowA : rowB;
                const int start = (e < 2) ? startA : startB;
                const bool ok = j >= start && j <= i && (p.window == 0 || i - j < p.window);
                const float x = ok ? s[n][e] * sl2 : -INFINITY;
                s[n][e] = x;
                if (e < 2) tmaxA = fmaxf(tmaxA, x); else tmaxB = fmaxf(tmaxB, x);
            }
        }
        uint32_t pa[NT / 2][4], pb[MODE == 2 ? NT / 2 : 1][4];   // A fragments: P (or P o dP) and P
        if constexpr (MODE != 2) {
            tmaxA = quad_max(tmaxA);
            tmaxB = quad_max(tmaxB);
            const float nA = fmaxf(mA, tmaxA), nB = fmaxf(mB, tmaxB);
            const float uA = nA == -INFINITY ? 0.0f : nA, uB = nB == -INFINITY ? 0.0f : nB;
            const float cA = exp2f(mA - uA), cB = exp2f(mB - uB);
            mA = nA;
            mB = nB;
            lA *= cA;
            lB *= cB;
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                s[n][0] = exp2f(s[n][0] - uA);
                s[n][1] = exp2f(s[n][1] - uA);
                s[n][2] = exp2f(s[n][2] - uB);
                s[n][3] = exp2f(s[n][3] - uB);
                lA += s[n][0] + s[n][1];
                lB += s[n][2] + s[n][3];
            }
            if constexpr (MODE == 0) {
#pragma unroll
                for (int n = 0; n < DH / 8; ++n) {
                    acc[n][0] *= cA;
                    acc[n][1] *= cA;
                    acc[n][2] *= cB;
                    acc[n][3] *= cB;
                }
            }
        } else {
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                s[n][0] = exp2f(s[n][0] - mA) * invA;
                s[n][1] = exp2f(s[n][1] - mA) * invA;
                s[n][2] = exp2f(s[n][2] - mB) * invB;
                s[n][3] = exp2f(s[n][3] - mB) * invB;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    dp[n][e] *= s[n][e];                       // P o dP
                }
                dA += dp[n][0] + dp[n][1];
                dB += dp[n][2] + dp[n][3];
            }
        }
        if constexpr (MODE != 1) {
#pragma unroll
            for (int kk = 0; kk < NT / 2; ++kk) {
                if constexpr (MODE == 2) {
                    pa[kk][0] = mma16816<T>::pack(dp[2 * kk][0], dp[2 * kk][1]);
                    pa[kk][1] = mma16816<T>::pack(dp[2 * kk][2], dp[2 * kk][3]);
                    pa[kk][2] = mma16816<T>::pack(dp[2 * kk + 1][0], dp[2 * kk + 1][1]);
                    pa[kk][3] = mma16816<T>::pack(dp[2 * kk + 1][2], dp[2 * kk + 1][3]);
                    pb[kk][0] = mma16816<T>::pack(s[2 * kk][0], s[2 * kk][1]);
                    pb[kk][1] = mma16816<T>::pack(s[2 * kk][2], s[2 * kk][3]);
                    pb[kk][2] = mma16816<T>::pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                    pb[kk][3] = mma16816<T>::pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
                } else {
                    pa[kk][0] = mma16816<T>::pack(s[2 * kk][0], s[2 * kk][1]);
                    pa[kk][1] = mma16816<T>::pack(s[2 * kk][2], s[2 * kk][3]);
                    pa[kk][2] = mma16816<T>::pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                    pa[kk][3] = mma16816<T>::pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
                }
            }
            const T *Bt = MODE == 2 ? Kt : Vt;                 // [key][DH]: k = key, n = head dim
#pragma unroll
            for (int kk = 0; kk < NT / 2; ++kk) {
#pragma unroll
                for (int np = 0; np < DH / 16; ++np) {
                    uint32_t b[4];
                    load_b_kn<LD>(b, Bt, kk * 16, np * 16, lane);
                    mma16816<T>::run(acc[2 * np], pa[kk], b[0], b[1]);
                    mma16816<T>::run(acc[2 * np + 1], pa[kk], b[2], b[3]);
                    if constexpr (MODE == 2) {
                        mma16816<T>::run(acc2[2 * np], pb[kk], b[0], b[1]);
                        mma16816<T>::run(acc2[2 * np + 1], pb[kk], b[2], b[3]);
                    }
                }
            }
        }
        __syncthreads();
    }

    if constexpr (MODE == 2) {
        dA = quad_sum(dA);
        dB = quad_sum(dB);
#pragma unroll
        for (int n = 0; n < DH / 8; ++n) {
            if (rowA < p.n_tokens) {
                const float x = rowA < n_valid ? p.scale * (acc[n][0] - dA * acc2[n][0]) : 0.0f;
                const float y = rowA < n_valid ? p.scale * (acc[n][1] - dA * acc2[n][1]) : 0.0f;
                *reinterpret_cast<uint32_t *>(out + oA + n * 8 + 2 * t) = mma16816<T>::pack(x, y);
            }
            if (rowB < p.n_tokens) {
                const float x = rowB < n_valid ? p.scale * (acc[n][2] - dB * acc2[n][2]) : 0.0f;
                const float y = rowB < n_valid ? p.scale * (acc[n][3] - dB * acc2[n][3]) : 0.0f;
                *reinterpret_cast<uint32_t *>(out + oB + n * 8 + 2 * t) = mma16816<T>::pack(x, y);
            }
        }
        if (t == 0) {
            if (rowA < n_valid) stats[((size_t)rowA * p.hq + h) * 3 + 2] = dA;
            if (rowB < n_valid) stats[((size_t)rowB * p.hq + h) * 3 + 2] = dB;
        }
        return;
    }
    lA = quad_sum(lA);
    lB = quad_sum(lB);
    if constexpr (MODE == 0) {
        const float iA = lA > 0.0f ? 1.0f / lA : 0.0f, iB = lB > 0.0f ? 1.0f / lB : 0.0f;
#pragma unroll
        for (int n = 0; n < DH / 8; ++n) {
            if (rowA < p.n_tokens) *reinterpret_cast<uint32_t *>(out + oA + n * 8 + 2 * t) = mma16816<T>::pack(acc[n][0] * iA, acc[n][1] * iA);
            if (rowB < p.n_tokens) *reinterpret_cast<uint32_t *>(out + oB + n * 8 + 2 * t) = mma16816<T>::pack(acc[n][2] * iB, acc[n][3] * iB);
        }
    }
    if (stats != nullptr && t == 0) {
        if (rowA < n_valid) {
            float *s = stats + ((size_t)rowA * p.hq + h) * 3;
            s[0] = mA == -INFINITY ? mA : mA * LN2;
            s[1] = lA;
            s[2] = 0.0f;
        }
        if (rowB < n_valid) {
            float *s = stats + ((size_t)rowB * p.hq + h) * 3;
            s[0] = mB == -INFINITY ? mB : mB * LN2;
            s[1] = lB;
            s[2] = 0.0f;
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Key-stationary backward: dK, dV for a 64-key chunk of one KV head.
// grid = (ceil(N / 64), Hkv), 128 threads; warp w owns keys 16w..16w+15 of the chunk.
// ------------------------------------------------------------------------------------------------
// FUSE_DQ: the kernel also forms dQ. Each warp multiplies its dS slice (16 keys, transposed in registers with movmatrix)
// by its 16 rows of K and adds the 64 x DH partial product to an FP32 accumulator in global memory (red.add), so the
// query-stationary pass is not needed when D is known beforehand; dq32 [N, Hq, DH] must be zero on entry.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a)
{
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}
__device__ __forceinline__ void red_add_v2(float *addr, float a, float b)
{
    asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(addr), "f"(a), "f"(b) : "memory");
}

template <typename T, int DH, int BQT, bool FUSE_DQ = false>
__global__ void __launch_bounds__(128, 3)
flash_kv_kernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v, const T *__restrict__ go,
                const int *__restrict__ cu, const float *__restrict__ stats, T *__restrict__ dk, T *__restrict__ dv,
                flash_params p, float *__restrict__ dq32)
{
    gdb_pdl_sync();
    constexpr int LD = DH + 8, BK = 64, NT = BQT / 8, KT = DH / 16;
    extern __shared__ __align__(16) unsigned char fsm[];
    T *Ks = reinterpret_cast<T *>(fsm);
    T *Vs = Ks + BK * LD;
    T *Qs = Vs + BK * LD;                  // [2][BQT][LD]
    T *Gs = Qs + 2 * BQT * LD;             // [2][BQT][LD]
    float *St = reinterpret_cast<float *>(Gs + 2 * BQT * LD);  // [2][BQT][3]: m (log2), 1/l, D
    constexpr int LDS = BK + 8;
    T *Ds = reinterpret_cast<T *>(St + 2 * BQT * 3);          // FUSE_DQ: dS tile [BQT][LDS]

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int k0 = blockIdx.x * BK, hk = blockIdx.y, group = p.hq / p.hkv;
    const int n_valid = min(cu[p.batch], p.n_tokens);
    const int keyA = k0 + warp * 16 + g, keyB = keyA + 8;
    const size_t oA = ((size_t)keyA * p.hkv + hk) * DH, oB = ((size_t)keyB * p.hkv + hk) * DH;

    float acck[DH / 8][4], accv[DH / 8][4];
#pragma unroll
    for (int n = 0; n < DH / 8; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) acck[n][e] = accv[n][e] = 0.0f;
    }
    if (k0 < n_valid) {
        const int endA = keyA < n_valid ? cu[seg_of(cu, p.batch, keyA) + 1] : 0;
        const int endB = keyB < n_valid ? cu[seg_of(cu, p.batch, keyB) + 1] : 0;
        const int last_key = min(k0 + BK, n_valid) - 1;
        int q_hi = cu[seg_of(cu, p.batch, last_key) + 1];       // exclusive
        if (p.window > 0) q_hi = min(q_hi, last_key + p.window);
        q_hi = min(q_hi, n_valid);
        const int tile0 = k0 / BQT, n_tiles = (q_hi - 1) / BQT - tile0 + 1;
        const float sl2 = p.scale * LOG2E;

        load_tile<T, DH, BK>(Ks, k, k0, n_valid, p.hkv, hk);
        load_tile<T, DH, BK>(Vs, v, k0, n_valid, p.hkv, hk);
        const int total = n_tiles * group;
        auto issue = [&](int w, int stg) {
            const int h = hk * group + w / n_tiles, qt0 = (tile0 + w % n_tiles) * BQT;
            load_tile<T, DH, BQT>(Qs + stg * BQT * LD, q, qt0, n_valid, p.hq, h);
            load_tile<T, DH, BQT>(Gs + stg * BQT * LD, go, qt0, n_valid, p.hq, h);
            for (int r = threadIdx.x; r < BQT; r += 128) {
                const int row = qt0 + r;
                float m = 0.0f, inv = 0.0f, d = 0.0f;
                if (row < n_valid) {
                    const float *s = stats + ((size_t)row * p.hq + h) * 3;
                    m = s[0] == -INFINITY ? 0.0f : s[0] * LOG2E;
                    inv = s[1] > 0.0f ? 1.0f / s[1] : 0.0f;
                    d = s[2];
                }
                float *dst = St + (stg * BQT + r) * 3;
                dst[0] = m;
                dst[1] = inv;
                dst[2] = d;
            }
        };
        issue(0, 0);
        cp_async_commit();
        for (int w = 0; w < total; ++w) {
            const int stg = w & 1;
            if (w + 1 < total) {
                issue(w + 1, stg ^ 1);
                cp_async_commit();
                cp_async_wait<1>();
            } else {
                cp_async_wait<0>();
            }
            __syncthreads();
            const T *Qt = Qs + stg * BQT * LD, *Gt = Gs + stg * BQT * LD;
            const float *Sq = St + stg * BQT * 3;
            const int qt0 = (tile0 + w % n_tiles) * BQT;

            float sT[NT][4], dpT[NT][4];
#pragma unroll
            for (int n = 0; n < NT; ++n) {
#pragma unroll
                for (int e = 0; e < 4; ++e) sT[n][e] = dpT[n][e] = 0.0f;
            }
#pragma unroll
            for (int kk = 0; kk < KT; ++kk) {
                uint32_t ak[4], av[4];
                load_a<LD>(ak, Ks, warp * 16, kk * 16, lane);
                load_a<LD>(av, Vs, warp * 16, kk * 16, lane);
#pragma unroll
                for (int np = 0; np < NT / 2; ++np) {
                    uint32_t b[4];
                    load_b_nk<LD>(b, Qt, np * 16, kk * 16, lane);
                    mma16816<T>::run(sT[2 * np], ak, b[0], b[1]);
                    mma16816<T>::run(sT[2 * np + 1], ak, b[2], b[3]);
                    load_b_nk<LD>(b, Gt, np * 16, kk * 16, lane);
                    mma16816<T>::run(dpT[2 * np], av, b[0], b[1]);
                    mma16816<T>::run(dpT[2 * np + 1], av, b[2], b[3]);
                }
            }
#pragma unroll
            for (int n = 0; n < NT; ++n) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int qi = n * 8 + 2 * t + (e & 1);
                    const int i = qt0 + qi;
                    const int j = (e < 2) ? keyA : keyB;
                    const int end = (e < 2) ? endA : endB;
                    const bool ok = i >= j && i < end && (p.window == 0 || i - j < p.window);
                    const float pr = ok ? exp2f(sT[n][e] * sl2 - Sq[qi * 3]) * Sq[qi * 3 + 1] : 0.0f;
                    sT[n][e] = pr;                                           // P^T
                    dpT[n][e] = pr * (dpT[n][e] - Sq[qi * 3 + 2]) * p.scale;  // dS^T
                }
            }
#pragma unroll
            for (int kk = 0; kk < NT / 2; ++kk) {
                uint32_t ap[4], ad[4];
                ap[0] = mma16816<T>::pack(sT[2 * kk][0], sT[2 * kk][1]);
                ap[1] = mma16816<T>::pack(sT[2 * kk][2], sT[2 * kk][3]);
                ap[2] = mma16816<T>::pack(sT[2 * kk + 1][0], sT[2 * kk + 1][1]);
                ap[3] = mma16816<T>::pack(sT[2 * kk + 1][2], sT[2 * kk + 1][3]);
                ad[0] = mma16816<T>::pack(dpT[2 * kk][0], dpT[2 * kk][1]);
                ad[1] = mma16816<T>::pack(dpT[2 * kk][2], dpT[2 * kk][3]);
                ad[2] = mma16816<T>::pack(dpT[2 * kk + 1][0], dpT[2 * kk + 1][1]);
                ad[3] = mma16816<T>::pack(dpT[2 * kk + 1][2], dpT[2 * kk + 1][3]);
#pragma unroll
                for (int np = 0; np < DH / 16; ++np) {
                    uint32_t b[4];
                    load_b_kn<LD>(b, Gt, kk * 16, np * 16, lane);
                    mma16816<T>::run(accv[2 * np], ap, b[0], b[1]);
                    mma16816<T>::run(accv[2 * np + 1], ap, b[2], b[3]);
                    load_b_kn<LD>(b, Qt, kk * 16, np * 16, lane);
                    mma16816<T>::run(acck[2 * np], ad, b[0], b[1]);
                    mma16816<T>::run(acck[2 * np + 1], ad, b[2], b[3]);
                }
                if (FUSE_DQ) {
                    // dS[q rows 16 kk .. +15, this warp's 16 keys] goes to shared memory as [q][key] (transposed in registers)
                    const uint32_t t0 = movmatrix_trans(ad[0]), t1 = movmatrix_trans(ad[2]), t2 = movmatrix_trans(ad[1]), t3 = movmatrix_trans(ad[3]);
                    T *rowp = Ds + (kk * 16 + g) * LDS + warp * 16 + 2 * t;
                    *reinterpret_cast<uint32_t *>(rowp) = t0;
                    *reinterpret_cast<uint32_t *>(rowp + 8 * LDS) = t1;
                    *reinterpret_cast<uint32_t *>(rowp + 8) = t2;
                    *reinterpret_cast<uint32_t *>(rowp + 8 * LDS + 8) = t3;
                }
            }
            if (FUSE_DQ) {
                // dQ[q rows 16 warp .. +15, :] += dS[q, all 64 keys of the chunk] K: one red per element and chunk
                __syncthreads();
                float dqa[DH / 8][4];
#pragma unroll
                for (int n = 0; n < DH / 8; ++n) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) dqa[n][e] = 0.0f;
                }
#pragma unroll
                for (int k2 = 0; k2 < BK / 16; ++k2) {
                    uint32_t a4[4];
                    load_a<LDS>(a4, Ds, warp * 16, k2 * 16, lane);
#pragma unroll
                    for (int np = 0; np < DH / 16; ++np) {
                        uint32_t b[4];
                        load_b_kn<LD>(b, Ks, k2 * 16, np * 16, lane);
                        mma16816<T>::run(dqa[2 * np], a4, b[0], b[1]);
                        mma16816<T>::run(dqa[2 * np + 1], a4, b[2], b[3]);
                    }
                }
                const int rowA = qt0 + warp * 16 + g, rowB = rowA + 8;
                const int hcur = hk * group + w / n_tiles;
                float *dA = dq32 + ((size_t)rowA * p.hq + hcur) * DH + 2 * t, *dB = dq32 + ((size_t)rowB * p.hq + hcur) * DH + 2 * t;
#pragma unroll
                for (int n = 0; n < DH / 8; ++n) {
                    if (rowA < n_valid) red_add_v2(dA + n * 8, dqa[n][0], dqa[n][1]);
                    if (rowB < n_valid) red_add_v2(dB + n * 8, dqa[n][2], dqa[n][3]);
                }
            }
            // The Q / dO stage of this iteration is last read before the barrier that precedes the dQ product, and the dS
            // tile is next written after the barrier at the top of the next iteration: the fused form needs no third barrier.
            if (!FUSE_DQ) __syncthreads();
        }
    }
#pragma unroll
    for (int n = 0; n < DH / 8; ++n) {
        if (keyA < p.n_tokens) {
            *reinterpret_cast<uint32_t *>(dk + oA + n * 8 + 2 * t) = mma16816<T>::pack(acck[n][0], acck[n][1]);
            *reinterpret_cast<uint32_t *>(dv + oA + n * 8 + 2 * t) = mma16816<T>::pack(accv[n][0], accv[n][1]);
        }
        if (keyB < p.n_tokens) {
            *reinterpret_cast<uint32_t *>(dk + oB + n * 8 + 2 * t) = mma16816<T>::pack(acck[n][2], acck[n][3]);
            *reinterpret_cast<uint32_t *>(dv + oB + n * 8 + 2 * t) = mma16816<T>::pack(accv[n][2], accv[n][3]);
        }
    }
}

template <typename T, int DH, int BKV, int MODE>
gd_status launch_q(gd_backend *be, const gdb_flash_args *a, const flash_params &p, void *out)
{
    constexpr int LD = DH + 8;
    constexpr size_t smem = (size_t)((MODE == 2 ? 2 : 1) * 64 * LD + 4 * BKV * LD) * 2U;
    auto kern = flash_q_kernel<T, DH, BKV, MODE>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return gdb_fail(be, e, "flash attention smem attribute");
        configured = true;
    }
    dim3 grid((unsigned)((a->n_tokens + 63) / 64), (unsigned)a->hq);
    gdb_launch(kern, grid, 128, smem, be->stream, (const T *)a->q, (const T *)a->k, (const T *)a->v, (const T *)a->grad_out, a->cu, (T *)out, a->stats, p);
    return gdb_launched(be, MODE == 0 ? "flash_forward" : (MODE == 1 ? "flash_stats" : "flash_backward_dq"));
}

template <typename T, int DH, int BQT, bool FUSE_DQ = false>
gd_status launch_kv(gd_backend *be, const gdb_flash_args *a, const flash_params &p, float *dq32 = nullptr)
{
    constexpr int LD = DH + 8;
    constexpr size_t smem = (size_t)(2 * 64 * LD + 4 * BQT * LD) * 2U + (size_t)2 * BQT * 3 * sizeof(float) + (FUSE_DQ ? (size_t)BQT * (64 + 8) * 2U : 0U);
    auto kern = flash_kv_kernel<T, DH, BQT, FUSE_DQ>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return gdb_fail(be, e, "flash attention smem attribute");
        configured = true;
    }
    dim3 grid((unsigned)((a->n_tokens + 63) / 64), (unsigned)a->hkv);
    gdb_launch(kern, grid, 128, smem, be->stream, (const T *)a->q, (const T *)a->k, (const T *)a->v, (const T *)a->grad_out, a->cu, a->stats, (T *)a->dk, (T *)a->dv, p, dq32);
    return gdb_launched(be, "flash_backward_dkv");
}

bool fast_path(const gdb_flash_args *a)
{
    const uintptr_t al = (uintptr_t)a->q | (uintptr_t)a->k | (uintptr_t)a->v;
    return (a->dtype == GDB_DTYPE_F16 || a->dtype == GDB_DTYPE_BF16) && (a->dh == 64 || a->dh == 128) && a->causal != 0 &&
           a->prefix == 0 && a->window >= 0 && (al % 16U) == 0U && a->hkv > 0 && (a->hq % a->hkv) == 0 && a->hq <= 65535;
}

flash_params make_params(const gdb_flash_args *a)
{
    flash_params p;
    p.n_tokens = a->n_tokens;
    p.batch = a->batch;
    p.hq = a->hq;
    p.hkv = a->hkv;
    p.dh = a->dh;
    p.window = a->window;
    p.scale = a->scale;
    return p;
}

template <typename T>
gd_status forward_typed(gd_backend *be, const gdb_flash_args *a, const flash_params &p)
{
    return a->dh == 64 ? launch_q<T, 64, 64, 0>(be, a, p, a->out_or_dq) : launch_q<T, 128, 64, 0>(be, a, p, a->out_or_dq);
}

// dq[i] = round(dq32[i]), eight values per thread.
template <typename T>
__global__ void dq_convert_kernel(const float4 *__restrict__ src, uint4 *__restrict__ dst, size_t n8)
{
    gdb_pdl_sync();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += stride) {
        const float4 a = src[2 * i], b = src[2 * i + 1];
        uint4 o;
        o.x = mma16816<T>::pack(a.x, a.y);
        o.y = mma16816<T>::pack(a.z, a.w);
        o.z = mma16816<T>::pack(b.x, b.y);
        o.w = mma16816<T>::pack(b.z, b.w);
        dst[i] = o;
    }
}

// Preparation of the single-pass backward: D[row, head] = sum_c dO * O (stats[.., 2]) and dq32 = 0.
// Eight threads per (row, head) of 64 elements, 16 bytes of dO and of O each. With `meta` != NULL it also leaves the mask
// bounds the tensor-memory kernel reads instead of searching cu_seqlens per step: meta[row] = first key row `row` may
// attend to (start of its sequence, moved up by the window; INT_MAX behind the last sequence), and, for every tile of 128
// keys, meta[n_tokens + tile] = number of 128-row query tiles, starting with the tile's own, that hold a query allowed to
// see one of its keys (0 behind the last sequence).
template <typename T>
__global__ void bwd_prep_kernel(const uint4 *__restrict__ go, const uint4 *__restrict__ out, float *__restrict__ stats, float4 *__restrict__ dq32,
                                size_t n_vec, const int *__restrict__ cu, int batch, int n_tokens, int hq, int window, int *__restrict__ meta)
{
    gdb_pdl_sync();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;   // one 8-element piece; n_vec is a multiple of 8
    float s = 0.0f;
    if (i < n_vec) {
        gdb_vec8<T> a, b;
        a.raw = go[i];
        b.raw = out[i];
#pragma unroll
        for (int e = 0; e < 8; ++e) s += a.get(e) * b.get(e);
        dq32[2 * i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        dq32[2 * i + 1] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) s += __shfl_xor_sync(0xffffffffU, s, o);
    if (i < n_vec && (threadIdx.x & 7) == 0) stats[(i >> 3) * 3U + 2U] = s;
    if (meta != nullptr && i < n_vec && (i % ((size_t)hq * 8U)) == 0U) {
        const int row = (int)(i / ((size_t)hq * 8U));
        const int n_valid = min(cu[batch], n_tokens);
        int lo = 0x7fffffff;
        if (row < n_valid) {
            lo = cu[seg_of(cu, batch, row)];
            if (window > 0) lo = max(lo, row - window + 1);
        }
        meta[row] = lo;
        if ((row & 127) == 0) {
            int n_qt = 0;
            if (row < n_valid) {
                const int last_key = min(row + 128, n_valid) - 1;
                int q_hi = cu[seg_of(cu, batch, last_key) + 1];       // exclusive
                if (window > 0) q_hi = min(q_hi, last_key + window);
                q_hi = min(q_hi, n_valid);
                n_qt = (q_hi - 1) / 128 - row / 128 + 1;
            }
            meta[n_tokens + (row >> 7)] = n_qt;
        }
    }
}

// Backward in one attention pass (head_dim 64, statistics (max, sum) saved by the forward): D from dO and the forward
// output, then the key-stationary kernel forms dK, dV and accumulates dQ in FP32, then dQ is rounded.
template <typename T>
gd_status backward_single_pass(gd_backend *be, const gdb_flash_args *a, const flash_params &p, const void *out, float *dq32)
{
    const size_t n = (size_t)a->n_tokens * a->hq * 64U, n_vec = n / 8U;
    // mask bounds for the tensor-memory kernel live at the start of the backend workspace between the two launches
    const size_t meta_bytes = ((size_t)a->n_tokens + (size_t)(a->n_tokens + 127) / 128U) * sizeof(int);
    int *meta = (be->attn_mode == 0 && meta_bytes <= be->ws_bytes) ? (int *)be->ws : nullptr;
    gdb_launch(bwd_prep_kernel<T>, (unsigned)((n_vec + 255U) / 256U), 256, 0, be->stream, (const uint4 *)a->grad_out, (const uint4 *)out, a->stats,
               (float4 *)dq32, n_vec, a->cu, a->batch, a->n_tokens, a->hq, a->window, meta);
    gd_status st = gdb_launched(be, "flash_backward_prep");
    if (st != GD_OK) return st;
    st = meta != nullptr ? gdb_attn5_backward(be, a, dq32, meta) : GD_ERR_UNSUPPORTED;   // tensor-memory kernel where the shape allows
    if (st == GD_ERR_UNSUPPORTED) st = launch_kv<T, 64, 64, true>(be, a, p, dq32);
    if (st != GD_OK) return st;
    if (a->keep_dq32 != 0) {
        return GD_OK;   // the caller's next kernel reads the accumulator and rounds on load
    }
    gdb_launch(dq_convert_kernel<T>, gdb_grid_for(n_vec, 256, be, 8), 256, 0, be->stream, (const float4 *)dq32, (uint4 *)a->out_or_dq, n_vec);
    return gdb_launched(be, "flash_backward_dq_convert");
}

template <typename T>
gd_status backward_typed(gd_backend *be, const gdb_flash_args *a, const flash_params &p, bool have_stats)
{
    gd_status st;
    if (!have_stats) {
        st = a->dh == 64 ? launch_q<T, 64, 64, 1>(be, a, p, NULL) : launch_q<T, 128, 64, 1>(be, a, p, NULL);
        if (st != GD_OK) return st;
    }
    st = a->dh == 64 ? launch_q<T, 64, 64, 2>(be, a, p, a->out_or_dq) : launch_q<T, 128, 32, 2>(be, a, p, a->out_or_dq);
    if (st != GD_OK) return st;
    return a->dh == 64 ? launch_kv<T, 64, 64>(be, a, p) : launch_kv<T, 128, 32>(be, a, p);
}

}  // namespace

gd_status gdb_flash_varlen_forward(gd_backend *be, const gdb_flash_args *a)
{
    if (!fast_path(a) || ((uintptr_t)a->out_or_dq % 16U) != 0U) {
        return GD_ERR_UNSUPPORTED;
    }
    if (be->attn_mode == 0) {
        const gd_status st = gdb_attn5_forward(be, a);
        if (st != GD_ERR_UNSUPPORTED) {
            return st;
        }
    }
    const flash_params p = make_params(a);
    return a->dtype == GDB_DTYPE_F16 ? forward_typed<__half>(be, a, p) : forward_typed<__nv_bfloat16>(be, a, p);
}

gd_status gdb_flash_varlen_backward(gd_backend *be, const gdb_flash_args *a, bool have_forward_stats)
{
    const uintptr_t al = (uintptr_t)a->grad_out | (uintptr_t)a->out_or_dq | (uintptr_t)a->dk | (uintptr_t)a->dv;
    if (!fast_path(a) || (al % 16U) != 0U || a->stats == NULL) {
        return GD_ERR_UNSUPPORTED;
    }
    const flash_params p = make_params(a);
    return a->dtype == GDB_DTYPE_F16 ? backward_typed<__half>(be, a, p, have_forward_stats)
                                     : backward_typed<__nv_bfloat16>(be, a, p, have_forward_stats);
}

// Backward with the forward output at hand (not part of the reference's entry, src/core/backend.h:699-709): D = rowsum(dO o O)
// replaces the query-stationary pass. `dq32`: FP32 scratch [N, Hq, 64]. GD_ERR_UNSUPPORTED outside head_dim 64 / the fast path.
gd_status gdb_flash_varlen_backward_with_out(gd_backend *be, const gdb_flash_args *a, const void *out, float *dq32)
{
    const uintptr_t al = (uintptr_t)a->grad_out | (uintptr_t)a->out_or_dq | (uintptr_t)a->dk | (uintptr_t)a->dv | (uintptr_t)out | (uintptr_t)dq32;
    if (!fast_path(a) || a->dh != 64 || (al % 16U) != 0U || a->stats == NULL || out == NULL || dq32 == NULL) {
        return GD_ERR_UNSUPPORTED;
    }
    const flash_params p = make_params(a);
    return a->dtype == GDB_DTYPE_F16 ? backward_single_pass<__half>(be, a, p, out, dq32) : backward_single_pass<__nv_bfloat16>(be, a, p, out, dq32);
}
