// Blackwell (sm_100a) dense contraction: TMA-fed shared-memory ring, tcgen05.mma with the FP32
// accumulator in tensor memory, warp-specialised roles.
//
//   C[M, N] = A * B (+ bias), 16-bit operands (F16 / BF16), FP32 accumulation, one rounding.
//   A is either K-major (stored [M, K], "x" of matmul / matmul_nt) or MN-major (stored [K, M],
//   "x" of matmul_tn); B is either K-major (stored [N, K], "w" of matmul_nt) or MN-major
//   (stored [K, N], "w" of matmul / matmul_tn / linear). Both major-ness bits of the UMMA
//   instruction descriptor are used, so no operand is ever transposed in memory.
//
// CTA = 192 threads: warp 0 issues TMA loads, warp 1 allocates tensor memory and issues the MMAs,
// warps 2-5 drain the accumulator (tcgen05.ld), add the bias in FP32, round and store. One CTA
// computes one 128 x BN tile (optionally one K-slice of it: split-K writes FP32 partials that a
// second kernel sums, used for the weight-gradient shapes whose contraction runs over all tokens).
//
// Shared-memory operand layout is the canonical 128-byte-swizzled UMMA layout that TMA writes
// directly: K-major tiles are rows of 64 elements (128 B), 8-row groups 1024 B apart (SBO);
// MN-major tiles are blocks of 64 MN-elements x BK k-rows, each k-row 128 B, 8-k-row groups
// 1024 B apart (SBO) and the 64-element MN blocks BK*128 B apart (LBO).
//
// Every mbarrier wait is bounded: when a wait gives up the kernel records an error code in
// gd_backend::err_flag, falls through to the common exit (tensor memory is released there) and
// gd_backend_flush reports GD_ERR_INTERNAL.
#include "common.cuh"

#include "tcgen05.cuh"

namespace {
using namespace gdb_t5;



template <int BN, int STAGES>
struct smem_plan {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int BAR_BYTES = 256;
    static constexpr int TOTAL = STAGES * STAGE_BYTES + BAR_BYTES + 1024;  // + slack for 1024-byte alignment
};


// grid = (n tiles, m tiles, k splits), or, BATCHED, (n tiles, m tiles, batch): the tensor maps then have the batch as third
// dimension (a broadcast operand has extent 1 there and is always read at index 0: za / zb say which), the output of
// batch element z starts c_batch elements after that of z - 1, and there is no split over k.
template <typename T, int BN, int STAGES, bool A_MN, bool B_MN, bool SPLITK, bool BATCHED = false>
__global__ void __launch_bounds__(192, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, T *__restrict__ c,
                    size_t ldc, const T *__restrict__ bias, float *__restrict__ partial, uint32_t M, uint32_t N, uint32_t K,
                    uint32_t k_iters_per_split, int bias_mode, int *err_flag, size_t c_batch, int a_bcast, int b_bcast)
{
    static_assert(!(SPLITK && BATCHED), "a batched launch uses the third grid dimension for the batch");
    using plan = smem_plan<BN, STAGES>;
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = (unsigned char *)(((uintptr_t)smem_raw + 1023U) & ~(uintptr_t)1023U);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + STAGES * plan::STAGE_BYTES);
    // bars[0..STAGES) full, bars[STAGES..2*STAGES) empty, bars[2*STAGES] accumulator ready
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const uint32_t total_k_iters = (K + BK - 1) / BK;
    const uint32_t k_begin = BATCHED ? 0U : blockIdx.z * k_iters_per_split;
    const int za = (BATCHED && !a_bcast) ? (int)blockIdx.z : 0, zb = (BATCHED && !b_bcast) ? (int)blockIdx.z : 0;
    if (BATCHED) c += (size_t)blockIdx.z * c_batch;
    const uint32_t k_end = min(total_k_iters, k_begin + k_iters_per_split);
    const uint32_t n_iters = k_end > k_begin ? k_end - k_begin : 0U;

    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]), accum_bar = smem_u32(&bars[2 * STAGES]);
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(accum_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // everything above touches only shared / tensor memory: it may run while the preceding kernel finishes
    gdb_pdl_sync();

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            for (uint32_t it = 0; it < n_iters; ++it) {
                const uint32_t s = it % STAGES, ph = (it / STAGES) & 1U;
                if (!mbar_wait(empty0 + 8 * s, ph ^ 1U)) {
                    atomicExch(err_flag, 101);
                    break;
                }
                const uint32_t a_dst = smem_u32(smem + s * plan::STAGE_BYTES);
                const uint32_t b_dst = a_dst + plan::A_BYTES;
                const int k0 = (int)((k_begin + it) * BK);
                mbar_expect_tx(full0 + 8 * s, plan::STAGE_BYTES);
                auto load_a = [&](uint32_t dst, int x, int y) {
                    if (BATCHED) tma_load_3d(dst, &tma_a, x, y, za, full0 + 8 * s); else tma_load_2d(dst, &tma_a, x, y, full0 + 8 * s);
                };
                auto load_b = [&](uint32_t dst, int x, int y) {
                    if (BATCHED) tma_load_3d(dst, &tma_b, x, y, zb, full0 + 8 * s); else tma_load_2d(dst, &tma_b, x, y, full0 + 8 * s);
                };
                if (A_MN) {
                    // global [K, M]: box {64 m, BK k}; two boxes cover the 128 rows of the tile
                    load_a(a_dst, (int)m0, k0);
                    load_a(a_dst + BK * 128, (int)m0 + 64, k0);
                } else {
                    load_a(a_dst, k0, (int)m0);  // global [M, K]: box {64 k, 128 m}
                }
                if (B_MN) {
#pragma unroll
                    for (int j = 0; j < BN / 64; ++j) {
                        load_b(b_dst + j * BK * 128, (int)n0 + 64 * j, k0);
                    }
                } else {
                    load_b(b_dst, k0, (int)n0);  // global [N, K]: box {64 k, BN n}
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t FMT = std::is_same<T, __nv_bfloat16>::value ? 1U : 0U;
            constexpr uint32_t IDESC = (1U << 4) | (FMT << 7) | (FMT << 10) | ((A_MN ? 1U : 0U) << 15) | ((B_MN ? 1U : 0U) << 16) |
                                       ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            bool ok = true;
            for (uint32_t it = 0; it < n_iters && ok; ++it) {
                const uint32_t s = it % STAGES, ph = (it / STAGES) & 1U;
                if (!mbar_wait(full0 + 8 * s, ph)) {
                    atomicExch(err_flag, 102);
                    ok = false;
                    break;
                }
                tcgen05_fence_after();
                const uint32_t a_base = smem_u32(smem + s * plan::STAGE_BYTES);
                const uint32_t b_base = a_base + plan::A_BYTES;
#pragma unroll
                for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                    // K-major: step 16 elements = 32 bytes inside the swizzle row.
                    // MN-major: step 16 k-rows = 2048 bytes.
                    const uint64_t adesc = A_MN ? make_smem_desc(a_base + kk * 2048, BK * 128, 1024)
                                                : make_smem_desc(a_base + kk * 32, 16, 1024);
                    const uint64_t bdesc = B_MN ? make_smem_desc(b_base + kk * 2048, BK * 128, 1024)
                                                : make_smem_desc(b_base + kk * 32, 16, 1024);
                    tcgen05_mma_f16(tmem_base, adesc, bdesc, IDESC, (it != 0 || kk != 0) ? 1U : 0U);
                }
                tcgen05_commit(empty0 + 8 * s);  // frees the stage once these MMAs have read it
            }
            tcgen05_commit(accum_bar);           // accumulator complete (or nothing was issued)
        }
    } else {
        // ---------------- epilogue: warps 2..5 own TMEM lane quadrants 2,3,0,1 ----------------
        const int quad = warp & 3;
        const uint32_t row = m0 + quad * 32 + lane;
        const bool ok = mbar_wait(accum_bar, 0);
        if (!ok && lane == 0) {
            atomicExch(err_flag, 103);
        }
        tcgen05_fence_after();
        if (ok) {
#pragma unroll 1
            for (int cb = 0; cb < BN / 32; ++cb) {
                uint32_t v[32];
                if (n_iters != 0) {
                    tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(cb * 32), v);
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = 0U;
                }
                const uint32_t col0 = n0 + cb * 32;
                if (row < M && col0 < N) {
                    if (SPLITK) {
                        float *dst = partial + ((size_t)blockIdx.z * M + row) * N + col0;
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            if (col0 + j < N) {
                                *reinterpret_cast<float4 *>(dst + j) = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]),
                                                                                   __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
                            }
                        }
                    } else {
                        T *dst = c + (size_t)row * ldc + col0;
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            if (col0 + j < N) {
                                float f[8];
#pragma unroll
                                for (int e = 0; e < 8; ++e) {
                                    f[e] = __uint_as_float(v[j + e]);
                                    if (bias != nullptr) {
                                        // mode 2 reproduces "round the product, then a rounded bias add"
                                        if (bias_mode == 2) f[e] = gdb_io<T>::rnd(f[e]);
                                        f[e] += gdb_io<T>::ld(bias, col0 + j + e);
                                    }
                                }
                                uint4 o;
                                o.x = half_pack<T>::pack(f[0], f[1]);
                                o.y = half_pack<T>::pack(f[2], f[3]);
                                o.z = half_pack<T>::pack(f[4], f[5]);
                                o.w = half_pack<T>::pack(f[6], f[7]);
                                *reinterpret_cast<uint4 *>(dst + j) = o;
                            }
                        }
                    }
                }
            }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)BN) : "memory");
    }
}

// out[m, n] = round(sum_z partial[z, m, n] + bias[n])
template <typename T>
__global__ void splitk_reduce_kernel(const float *__restrict__ partial, T *__restrict__ c, size_t ldc, const T *__restrict__ bias,
                                     uint32_t M, uint32_t N, uint32_t splits, int bias_mode, const float *__restrict__ colsum_partial,
                                     T *__restrict__ colsum)
{
    gdb_pdl_sync();
    if (colsum_partial != nullptr) {
        // colsum[m] = round(sum_z colsum_partial[z, m])
        for (size_t m = (size_t)blockIdx.x * blockDim.x + threadIdx.x; m < M; m += (size_t)gridDim.x * blockDim.x) {
            float acc = 0.0f;
            for (uint32_t z = 0; z < splits; ++z) acc += colsum_partial[(size_t)z * M + m];
            gdb_io<T>::st(colsum, m, acc);
        }
    }
    const size_t quads = (size_t)M * (N / 4), stride = (size_t)gridDim.x * blockDim.x;
    for (size_t q = (size_t)blockIdx.x * blockDim.x + threadIdx.x; q < quads; q += stride) {
        const uint32_t row = (uint32_t)(q / (N / 4)), col = (uint32_t)(q % (N / 4)) * 4;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (uint32_t z = 0; z < splits; ++z) {
            const float4 p = *reinterpret_cast<const float4 *>(partial + ((size_t)z * M + row) * N + col);
            acc.x += p.x;
            acc.y += p.y;
            acc.z += p.z;
            acc.w += p.w;
        }
        if (bias != nullptr) {
            if (bias_mode == 2) {
                acc.x = gdb_io<T>::rnd(acc.x);
                acc.y = gdb_io<T>::rnd(acc.y);
                acc.z = gdb_io<T>::rnd(acc.z);
                acc.w = gdb_io<T>::rnd(acc.w);
            }
            acc.x += gdb_io<T>::ld(bias, col);
            acc.y += gdb_io<T>::ld(bias, col + 1);
            acc.z += gdb_io<T>::ld(bias, col + 2);
            acc.w += gdb_io<T>::ld(bias, col + 3);
        }
        uint2 o;
        o.x = half_pack<T>::pack(acc.x, acc.y);
        o.y = half_pack<T>::pack(acc.z, acc.w);
        *reinterpret_cast<uint2 *>(c + (size_t)row * ldc + col) = o;
    }
}

template <typename T, int BN, int STAGES, bool A_MN, bool B_MN, bool SPLITK>
gd_status launch(gd_backend *be, const CUtensorMap &ta, const CUtensorMap &tb, void *c, size_t ldc, const void *bias,
                 float *partial, uint32_t M, uint32_t N, uint32_t K, uint32_t splits, uint32_t k_per_split, int bias_mode)
{
    using plan = smem_plan<BN, STAGES>;
    auto kern = gemm_tcgen05_kernel<T, BN, STAGES, A_MN, B_MN, SPLITK>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, plan::TOTAL);
        if (e != cudaSuccess) {
            return gdb_fail(be, e, "tcgen05 gemm smem attribute");
        }
        configured = true;
    }
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM, splits);
    gdb_launch(kern, grid, 192, plan::TOTAL, be->stream, ta, tb, (T *)c, ldc, (const T *)bias, partial, M, N, K, k_per_split, bias_mode, be->err_flag, (size_t)0, 0, 0);
    return gdb_launched(be, "gemm_tcgen05");
}

template <typename T, int BN, int STAGES>
gd_status dispatch_major(gd_backend *be, int ta, int tb, const CUtensorMap &ma, const CUtensorMap &mb, void *c, size_t ldc,
                         const void *bias, float *partial, uint32_t M, uint32_t N, uint32_t K, uint32_t splits, uint32_t kps, int bias_mode)
{
    const bool sk = splits > 1;
#define GDB_GO(AM, BMJ)                                                                                              \
    (sk ? launch<T, BN, STAGES, AM, BMJ, true>(be, ma, mb, c, ldc, bias, partial, M, N, K, splits, kps, bias_mode) \
        : launch<T, BN, STAGES, AM, BMJ, false>(be, ma, mb, c, ldc, bias, partial, M, N, K, splits, kps, bias_mode))
    if (ta) {
        return tb ? GDB_GO(true, false) : GDB_GO(true, true);
    }
    return tb ? GDB_GO(false, false) : GDB_GO(false, true);
#undef GDB_GO
}

gd_status reduce_partials(gd_backend *be, uint32_t dtype, const float *partial, void *c, size_t ldc, const void *bias, uint32_t M,
                          uint32_t N, uint32_t splits, int bias_mode, const float *colsum_partial = nullptr, void *colsum = nullptr)
{
    const size_t quads = (size_t)M * (N / 4U);
    if (dtype == GDB_DTYPE_F16) {
        gdb_launch(splitk_reduce_kernel<__half>, gdb_grid_for(quads, 256, be, 8), 256, 0, be->stream, partial, (__half *)c, ldc, (const __half *)bias, M, N, splits, bias_mode, colsum_partial, (__half *)colsum);
    } else {
        gdb_launch(splitk_reduce_kernel<__nv_bfloat16>, gdb_grid_for(quads, 256, be, 8), 256, 0, be->stream, partial, (__nv_bfloat16 *)c, ldc, (const __nv_bfloat16 *)bias, M, N, splits, bias_mode, colsum_partial, (__nv_bfloat16 *)colsum);
    }
    return gdb_launched(be, "gemm_splitk_reduce");
}

template <typename T, bool A_MN, bool B_MN>
gd_status launch_batched(gd_backend *be, const CUtensorMap &ta, const CUtensorMap &tb, void *c, size_t ldc, size_t c_batch, uint32_t M, uint32_t N,
                         uint32_t K, uint32_t batch, int a_bcast, int b_bcast)
{
    using plan = smem_plan<128, 4>;
    auto kern = gemm_tcgen05_kernel<T, 128, 4, A_MN, B_MN, false, true>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, plan::TOTAL);
    if (e != cudaSuccess) {
        return gdb_fail(be, e, "tcgen05 batched gemm smem attribute");
    }
    dim3 grid((N + 127) / 128, (M + BM - 1) / BM, batch);
    gdb_launch(kern, grid, 192, plan::TOTAL, be->stream, ta, tb, (T *)c, ldc, (const T *)nullptr, (float *)nullptr, M, N, K, (K + BK - 1) / BK, 0,
               be->err_flag, c_batch, a_bcast, b_bcast);
    return gdb_launched(be, "gemm_tcgen05_batched");
}

}  // namespace

// `batch` contractions of one shape in ONE launch (the batch index is the third grid dimension and the third tensor-map
// coordinate): C_z[M, N] = A_z B_z, z < batch, with byte pitches between consecutive batch elements; a pitch of 0
// broadcasts that operand. GD_ERR_UNSUPPORTED when the shape or the alignment cannot use the TMA path.
gd_status gdb_gemm_tcgen05_batched(gd_backend *be, int ta, int tb, uint32_t dtype, const void *a, size_t lda_bytes, size_t a_batch_bytes,
                                   const void *b, size_t ldb_bytes, size_t b_batch_bytes, void *c, size_t ldc_bytes, size_t c_batch_bytes,
                                   uint32_t M, uint32_t N, uint32_t K, uint32_t batch)
{
    if ((dtype != GDB_DTYPE_F16 && dtype != GDB_DTYPE_BF16) || be->gemm_mode == 1 || batch == 0U || batch > 65535U) {
        return GD_ERR_UNSUPPORTED;
    }
    if ((((uintptr_t)a | (uintptr_t)b | (uintptr_t)c) % 16U) != 0U || (lda_bytes % 16U) != 0U || (ldb_bytes % 16U) != 0U || (ldc_bytes % 16U) != 0U ||
        (a_batch_bytes % 16U) != 0U || (b_batch_bytes % 16U) != 0U || (c_batch_bytes % 2U) != 0U || (N % 8U) != 0U || (K % 8U) != 0U ||
        M < 64U || N < 64U || K < 64U) {
        return GD_ERR_UNSUPPORTED;
    }
    const int a_bcast = a_batch_bytes == 0U, b_bcast = b_batch_bytes == 0U;
    const uint64_t a_n = a_bcast ? 1U : batch, b_n = b_bcast ? 1U : batch;
    // a broadcast operand still needs a valid (non-zero) batch pitch in its map: one whole matrix
    const uint64_t a_bp = a_bcast ? (uint64_t)lda_bytes * (ta ? K : M) : a_batch_bytes, b_bp = b_bcast ? (uint64_t)ldb_bytes * (tb ? N : K) : b_batch_bytes;
    CUtensorMap ma, mb;
    const bool oka = ta ? make_tmap_batched(&ma, dtype, a, a_n, K, M, lda_bytes, a_bp, 64, BK) : make_tmap_batched(&ma, dtype, a, a_n, M, K, lda_bytes, a_bp, BK, BM);
    const bool okb = tb ? make_tmap_batched(&mb, dtype, b, b_n, N, K, ldb_bytes, b_bp, BK, 128) : make_tmap_batched(&mb, dtype, b, b_n, K, N, ldb_bytes, b_bp, 64, BK);
    if (!oka || !okb) {
        return GD_ERR_UNSUPPORTED;
    }
    const size_t ldc = ldc_bytes / 2U, cb = c_batch_bytes / 2U;
#define GDB_GO_B(TT) (ta ? (tb ? launch_batched<TT, true, false>(be, ma, mb, c, ldc, cb, M, N, K, batch, a_bcast, b_bcast)  \
                               : launch_batched<TT, true, true>(be, ma, mb, c, ldc, cb, M, N, K, batch, a_bcast, b_bcast))  \
                         : (tb ? launch_batched<TT, false, false>(be, ma, mb, c, ldc, cb, M, N, K, batch, a_bcast, b_bcast) \
                               : launch_batched<TT, false, true>(be, ma, mb, c, ldc, cb, M, N, K, batch, a_bcast, b_bcast)))
    return dtype == GDB_DTYPE_F16 ? GDB_GO_B(__half) : GDB_GO_B(__nv_bfloat16);
#undef GDB_GO_B
}

// ta: A stored [K, M] (MN-major); tb: B stored [N, K] (K-major). Leading dimensions in bytes.
gd_status gdb_gemm_tcgen05(gd_backend *be, int ta, int tb, uint32_t dtype, const void *a, size_t lda_bytes, const void *b,
                           size_t ldb_bytes, void *c, size_t ldc_bytes, const void *bias, int bias_mode, uint32_t M, uint32_t N, uint32_t K)
{
    if (dtype != GDB_DTYPE_F16 && dtype != GDB_DTYPE_BF16) {
        return GD_ERR_UNSUPPORTED;
    }
    // TMA needs 16-byte aligned bases and pitches; vector stores need N % 8 == 0; tiny problems are
    // cheaper on the portable kernel than a 128-row tile with bounded-wait pipeline set-up.
    if ((((uintptr_t)a | (uintptr_t)b | (uintptr_t)c) % 16U) != 0U || (lda_bytes % 16U) != 0U || (ldb_bytes % 16U) != 0U ||
        (ldc_bytes % 16U) != 0U || (N % 8U) != 0U || (K % 8U) != 0U || M < 64U || N < 64U || K < 64U) {
        return GD_ERR_UNSUPPORTED;
    }
    if (bias != NULL && ((uintptr_t)bias % 2U) != 0U) {
        return GD_ERR_UNSUPPORTED;
    }
    const size_t ldc = ldc_bytes / 2U;
    float *partial = (float *)be->ws;
    uint32_t splits = 1;
    if (be->gemm_mode != 3) {
        gd_status pst = gdb_gemm_tcgen05_pair(be, ta, tb, dtype, a, lda_bytes, b, ldb_bytes, c, ldc_bytes, bias, bias_mode, M, N, K, &splits);
        if (pst == GD_OK) {
            return splits == 1U ? GD_OK : reduce_partials(be, dtype, partial, c, ldc, bias, M, N, splits, bias_mode);
        }
        if (pst != GD_ERR_UNSUPPORTED) {
            return pst;
        }
        splits = 1;
    }
    const int bn = (N % 256U == 0U && (size_t)((M + BM - 1) / BM) * (N / 256U) >= (size_t)be->sm_count) ? 256 : 128;
    CUtensorMap ma, mb;
    const bool oka = ta ? make_tmap(&ma, dtype, a, K, M, lda_bytes, 64, BK) : make_tmap(&ma, dtype, a, M, K, lda_bytes, BK, BM);
    const bool okb = tb ? make_tmap(&mb, dtype, b, N, K, ldb_bytes, BK, (uint32_t)bn) : make_tmap(&mb, dtype, b, K, N, ldb_bytes, 64, BK);
    if (!oka || !okb) {
        return GD_ERR_UNSUPPORTED;
    }
    // split-K when the tile grid cannot fill the machine and the contraction is long
    const uint32_t tiles = ((M + BM - 1) / BM) * ((N + bn - 1) / bn);
    const uint32_t total_k = (K + BK - 1) / BK;
    if (tiles < (uint32_t)be->sm_count && total_k >= 16U) {
        splits = ((uint32_t)be->sm_count * 2U + tiles - 1U) / tiles;
        if (splits > total_k / 4U) splits = total_k / 4U;
        if (splits > 32U) splits = 32U;
        while (splits > 1U && (size_t)splits * M * N * sizeof(float) > be->ws_bytes / 2U) --splits;
        if (splits < 1U) splits = 1U;
    }
    uint32_t kps = (total_k + splits - 1U) / splits;
    splits = (total_k + kps - 1U) / kps;
    gd_status st;
    if (dtype == GDB_DTYPE_F16) {
        st = bn == 256 ? dispatch_major<__half, 256, 4>(be, ta, tb, ma, mb, c, ldc, bias, partial, M, N, K, splits, kps, bias_mode)
                       : dispatch_major<__half, 128, 3>(be, ta, tb, ma, mb, c, ldc, bias, partial, M, N, K, splits, kps, bias_mode);
    } else {
        st = bn == 256 ? dispatch_major<__nv_bfloat16, 256, 4>(be, ta, tb, ma, mb, c, ldc, bias, partial, M, N, K, splits, kps, bias_mode)
                       : dispatch_major<__nv_bfloat16, 128, 3>(be, ta, tb, ma, mb, c, ldc, bias, partial, M, N, K, splits, kps, bias_mode);
    }
    if (st != GD_OK || splits == 1U) {
        return st;
    }
    return reduce_partials(be, dtype, partial, c, ldc, bias, M, N, splits, bias_mode);
}

void gdb_tmap_cache_destroy(gd_backend *be) { (void)be; }

gd_status gdb_gemm_tcgen05_tn_colsum(gd_backend *be, uint32_t dtype, const void *a, size_t lda_bytes, const void *b, size_t ldb_bytes,
                                     void *c, size_t ldc_bytes, void *colsum, uint32_t M, uint32_t N, uint32_t K)
{
    if ((dtype != GDB_DTYPE_F16 && dtype != GDB_DTYPE_BF16) || be->gemm_mode == 1 || be->gemm_mode == 3 || colsum == NULL ||
        (((uintptr_t)a | (uintptr_t)b | (uintptr_t)c) % 16U) != 0U || (lda_bytes % 16U) != 0U || (ldb_bytes % 16U) != 0U ||
        (ldc_bytes % 16U) != 0U || (N % 8U) != 0U || (K % 8U) != 0U) {
        return GD_ERR_UNSUPPORTED;
    }
    uint32_t splits = 1;
    float *cs = nullptr;
    gd_status st = gdb_gemm_tcgen05_pair(be, 1, 0, dtype, a, lda_bytes, b, ldb_bytes, c, ldc_bytes, NULL, 1, M, N, K, &splits, &cs);
    if (st != GD_OK) {
        return st;
    }
    return reduce_partials(be, dtype, (const float *)be->ws, c, ldc_bytes / 2U, NULL, M, N, splits, 1, cs, colsum);
}

