// Persistent CTA-pair contraction for sm_100a: two CTAs on neighbouring SMs share one
// 256 x 256 output tile (tcgen05.mma.cta_group::2), so each CTA fetches only its own 128 rows of
// A and its own 128 columns of B per k-step, which cuts the shared-memory fill traffic per flop
// by a third against a single-CTA 128 x 256 tile.
//
//   C[M, N] = A * B (+ bias), 16-bit operands, FP32 accumulation in tensor memory, one rounding;
//   with SPLITK the kernel writes FP32 partial tiles [splits, M, N] that splitk_reduce sums.
//
// One cluster of two CTAs per SM pair, resident for the whole launch; work units (output tile x
// k-slice) are dealt round-robin to the clusters. Tensor memory holds two accumulators of 256
// columns, so the MMA issuer starts the next unit while the epilogue warps drain the previous one.
//
// Roles per CTA (320 threads): warp 0 = TMA producer for this CTA's operand halves (completion
// bytes of both CTAs are signalled on the leader CTA's "full" barrier); warp 1 = tensor-memory
// allocation, and in the leader CTA the MMA issuer for the pair (tcgen05.commit multicasts the
// "stage free" and "accumulator ready" arrivals to both CTAs); warps 2-9 = epilogue (two warps per
// tensor-memory lane quadrant, each draining half of the tile's columns): tcgen05.ld,
// bias add and rounding in registers, 128-byte-swizzled staging in shared memory, TMA tile
// stores (clipped at the matrix edges by the tensor map).
//
// No load uses cluster multicast. Every mbarrier wait is bounded; a wait that gives up records a
// code in gd_backend::err_flag and the role leaves its loop, so the kernel always reaches the
// common exit where tensor memory is released.
#include "tcgen05.cuh"

namespace {
using namespace gdb_t5;

constexpr int PBN = 256;         // tile columns of the pair
constexpr int P_STAGES_DEFAULT = 5;
constexpr int P_EPI_WARPS = 8;   // two warps per tensor-memory lane quadrant, each drains half of the tile columns
constexpr int P_THREADS = 32 * (2 + P_EPI_WARPS);
constexpr int P_A_BYTES = BM * BK * 2;
constexpr int P_B_BYTES = (PBN / 2) * BK * 2;
constexpr int P_STAGE_BYTES = P_A_BYTES + P_B_BYTES;
// default: two 32-row x 128-byte staging buffers per epilogue warp
constexpr int P_SMEM_TOTAL = P_STAGES_DEFAULT * P_STAGE_BYTES + P_EPI_WARPS * 2 * 4096 + 256 + 1024;
constexpr int P_SMEM_TOTAL_COLSUM = P_STAGES_DEFAULT * P_STAGE_BYTES + P_EPI_WARPS * 2 * 4096 + 1024 + 1024 + 1024;   // barriers padded to 1 KB, ones tile, alignment slack
constexpr int P_SMEM_TOTAL_SWIGLU = (P_STAGES_DEFAULT - 1) * P_STAGE_BYTES + P_EPI_WARPS * 3 * 4096 + 256 + 1024;

// COLSUM (split-K output only): the units of the first tile column also accumulate the sums of A over the
// contraction, colsum[m] = sum_k A[m, k], by one more MMA per k-step against a tile of ones (N = 16; every output
// column holds the sum), and write them per k-slice to colsum_partial[splits, M]. This is the bias gradient of a
// linear layer for free while its weight gradient dW = dY^T X is computed (A = dY^T). Tensor memory then holds ONE
// accumulator (256 columns) plus the 16 column-sum columns, so units are not overlapped (split-K launches run about one
// unit per CTA pair anyway).
//
// SWIGLU (up / gate projection of a SwiGLU block, w stored [2F, K] with the x1 rows first: reference
// src/ops/swiglu_split_linear/core_swiglu_split_linear.c:226-301 composes matmul_nt + add + swiglu_split): a unit covers 128
// columns j of the activation. CTA 0 of the pair fetches weight rows j (x1), CTA 1 weight rows F + j (x2), so the pair's
// accumulator holds the x1 tile in columns 0..127 and the matching x2 tile in columns 128..255, and the epilogue forms
// x12 = round(round(acc) + bias) and act = round(x1 * x2 * sigmoid(x2)) from one pass over tensor memory, with the rounding
// points of the three separate calls. N is then F, tma_c maps the [M, 2F] x12 matrix (kept for the backward pass) and
// tma_act the [M, F] activation; a warp stages its x1, x2 and act tile (32 rows x 64 columns each) and issues three TMA stores.
//
// SWIGLU_BWD (input gradient of the down projection of a SwiGLU block, y = act w, w stored [F, N_out]: dact = g w^T is an
// x w^T contraction with N = F): the epilogue does not write dact but the gradient of the up / gate projection's output,
// d_x1 = dact x2 sigmoid(x2) and d_x2 = dact x1 sigmoid(x2) (1 + x2 (1 - sigmoid(x2))) with dact rounded to storage first
// (the rounding point of the separate swiglu_split_backward call, src/ops/swiglu_split_linear/core_swiglu_split_linear.c:303-420).
// x1 / x2 come from `aux` = the saved [M, 2F] x12 matrix (16-byte loads, a row per thread); tma_c maps d_x12 [M, 2F].
template <typename T, bool A_MN, bool B_MN, bool SPLITK, bool COLSUM, bool SWIGLU = false, bool SWIGLU_BWD = false>
__global__ void __launch_bounds__(P_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const __grid_constant__ CUtensorMap tma_c, const T *__restrict__ bias, uint32_t M, uint32_t N, uint32_t K,
                 uint32_t tiles_m, uint32_t tiles_n, uint32_t splits, uint32_t k_iters_per_split, int bias_mode, int *err_flag,
                 float *__restrict__ colsum_partial, const __grid_constant__ CUtensorMap tma_act, const T *__restrict__ aux, size_t ld_aux)
{
    static_assert(!COLSUM || SPLITK, "column sums ride on the split-K (FP32 partial) output path");
    static_assert(!SWIGLU || (!SPLITK && !A_MN && !B_MN), "the SwiGLU epilogue belongs to y = x w^T with direct output");
    static_assert(!SWIGLU_BWD || (!SPLITK && !A_MN && !B_MN && !SWIGLU), "the SwiGLU backward epilogue belongs to dact = g w^T with direct output");
    // The SwiGLU epilogue stages three output tiles per warp (x1, x2, act) instead of two alternating ones: it runs with
    // one operand stage less to make room for them.
    constexpr int PSTAGES = SWIGLU ? P_STAGES_DEFAULT - 1 : P_STAGES_DEFAULT;
    constexpr int P_STAGING_PER_WARP = SWIGLU ? 3 * 4096 : 2 * 4096;
    constexpr int P_STAGING_BYTES = P_EPI_WARPS * P_STAGING_PER_WARP;
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = (unsigned char *)(((uintptr_t)smem_raw + 1023U) & ~(uintptr_t)1023U);
    unsigned char *staging = smem + PSTAGES * P_STAGE_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(staging + P_STAGING_BYTES);
    // bars: [0, S) full, [S, 2S) empty, [2S, 2S+2) accumulator full, [2S+2, 2S+4) accumulator empty
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * PSTAGES + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const uint32_t cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
    const uint32_t total_k_iters = (K + BK - 1) / BK;
    const uint32_t units = tiles_m * tiles_n * splits;

    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[PSTAGES]);
    const uint32_t tfull0 = smem_u32(&bars[2 * PSTAGES]), tempty0 = smem_u32(&bars[2 * PSTAGES + 2]);
    unsigned char *ones_tile = staging + P_STAGING_BYTES + 1024;   // 1 KB, 1024-byte aligned: 8 rows x 64 k of 1.0
    if (COLSUM) {
        const uint32_t one2 = std::is_same<T, __nv_bfloat16>::value ? 0x3F803F80U : 0x3C003C00U;
        for (int i = threadIdx.x; i < 256; i += blockDim.x) reinterpret_cast<uint32_t *>(ones_tile)[i] = one2;
        fence_proxy_async_smem();   // the MMA reads this tile through the async proxy
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < PSTAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(tfull0 + 8 * b, 1);
            mbar_init(tempty0 + 8 * b, 2 * P_EPI_WARPS);   // the epilogue warps of the two CTAs
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)(2 * PBN)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    cluster_sync_all();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // everything above touches only shared / tensor memory: it may run while the preceding kernel finishes
    gdb_pdl_sync();

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs, own operand halves) ----------------
        if (lane == 0) {
            const uint32_t full_leader = mapa_shared(full0, 0);
            uint32_t it = 0;
            bool ok = true;
            for (uint32_t u = cluster_id; u < units && ok; u += n_clusters) {
                const uint32_t tn = u % tiles_n, tm = (u / tiles_n) % tiles_m, z = u / (tiles_n * tiles_m);
                const int am = (int)(tm * 2 * BM + rank * BM), bn = SWIGLU ? (int)(tn * (PBN / 2) + rank * N) : (int)(tn * PBN + rank * (PBN / 2));
                const uint32_t k_begin = z * k_iters_per_split;
                const uint32_t k_end = min(total_k_iters, k_begin + k_iters_per_split);
                for (uint32_t kb = k_begin; kb < k_end; ++kb, ++it) {
                    const uint32_t s = it % PSTAGES, ph = (it / PSTAGES) & 1U;
                    if (!mbar_wait(empty0 + 8 * s, ph ^ 1U)) {
                        atomicExch(err_flag, 201);
                        ok = false;
                        break;
                    }
                    if (rank == 0) {
                        mbar_expect_tx(full0 + 8 * s, 2 * P_STAGE_BYTES);
                    }
                    const uint32_t a_dst = smem_u32(smem + s * P_STAGE_BYTES), b_dst = a_dst + P_A_BYTES;
                    const uint32_t bar = full_leader + 8 * s;
                    const int k0 = (int)(kb * BK);
                    if (A_MN) {
                        tma_load_2d_pair(a_dst, &tma_a, am, k0, bar);
                        tma_load_2d_pair(a_dst + BK * 128, &tma_a, am + 64, k0, bar);
                    } else {
                        tma_load_2d_pair(a_dst, &tma_a, k0, am, bar);
                    }
                    if (B_MN) {
                        tma_load_2d_pair(b_dst, &tma_b, bn, k0, bar);
                        tma_load_2d_pair(b_dst + BK * 128, &tma_b, bn + 64, k0, bar);
                    } else {
                        tma_load_2d_pair(b_dst, &tma_b, k0, bn, bar);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader CTA only) ----------------
        if (lane == 0 && rank == 0) {
            constexpr uint32_t FMT = std::is_same<T, __nv_bfloat16>::value ? 1U : 0U;
            constexpr uint32_t IDESC = (1U << 4) | (FMT << 7) | (FMT << 10) | ((A_MN ? 1U : 0U) << 15) | ((B_MN ? 1U : 0U) << 16) |
                                       ((uint32_t)(PBN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
            uint32_t it = 0, unit_idx = 0;
            bool ok = true;
            for (uint32_t u = cluster_id; u < units && ok; u += n_clusters, ++unit_idx) {
                const uint32_t z = u / (tiles_n * tiles_m);
                const uint32_t k_begin = z * k_iters_per_split;
                const uint32_t k_end = min(total_k_iters, k_begin + k_iters_per_split);
                const uint32_t buf = COLSUM ? 0U : (unit_idx & 1U), acc_ph = COLSUM ? (unit_idx & 1U) : ((unit_idx >> 1) & 1U);
                const bool do_colsum = COLSUM && (u % tiles_n) == 0U;
                if (!mbar_wait(tempty0 + 8 * buf, acc_ph ^ 1U)) {
                    atomicExch(err_flag, 202);
                    break;
                }
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + buf * PBN;
                for (uint32_t kb = k_begin; kb < k_end; ++kb, ++it) {
                    const uint32_t s = it % PSTAGES, ph = (it / PSTAGES) & 1U;
                    if (!mbar_wait(full0 + 8 * s, ph)) {
                        atomicExch(err_flag, 203);
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after();
                    const uint32_t a_base = smem_u32(smem + s * P_STAGE_BYTES), b_base = a_base + P_A_BYTES;
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                        const uint64_t adesc = A_MN ? make_smem_desc(a_base + kk * 2048, BK * 128, 1024)
                                                    : make_smem_desc(a_base + kk * 32, 16, 1024);
                        const uint64_t bdesc = B_MN ? make_smem_desc(b_base + kk * 2048, BK * 128, 1024)
                                                    : make_smem_desc(b_base + kk * 32, 16, 1024);
                        tcgen05_mma_f16_pair(d_tmem, adesc, bdesc, IDESC, (kb != k_begin || kk != 0) ? 1U : 0U);
                        if (do_colsum) {
                            // sum over k of the same A tile: B = ones (K-major, 8 rows per CTA), N = 16, columns 256..271
                            constexpr uint32_t IDESC_ONES = (1U << 4) | (FMT << 7) | (FMT << 10) | ((A_MN ? 1U : 0U) << 15) |
                                                            ((uint32_t)(16 >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
                            tcgen05_mma_f16_pair(tmem_base + PBN, adesc, make_smem_desc(smem_u32(ones_tile) + kk * 32, 16, 1024), IDESC_ONES,
                                                 (kb != k_begin || kk != 0) ? 1U : 0U);
                        }
                    }
                    tcgen05_commit_pair(empty0 + 8 * s, 3);
                }
                if (ok) {
                    tcgen05_commit_pair(tfull0 + 8 * buf, 3);
                }
            }
        }
    } else {
        // ---------------- epilogue: warps 2..9; warps w and w + 4 share lane quadrant w & 3 and split the columns ----------------
        const int quad = warp & 3, chalf = (warp - 2) >> 2;
        unsigned char *my_stage = staging + (warp - 2) * P_STAGING_PER_WARP;
        const uint32_t tempty_leader = mapa_shared(tempty0, 0);
        uint32_t unit_idx = 0, store_cnt = 0;
        constexpr int CHUNK_COLS = SPLITK ? 32 : 64;   // 128 bytes of output per row
        for (uint32_t u = cluster_id; u < units; u += n_clusters, ++unit_idx) {
            const uint32_t tn = u % tiles_n, tm = (u / tiles_n) % tiles_m, z = u / (tiles_n * tiles_m);
            const uint32_t buf = COLSUM ? 0U : (unit_idx & 1U), acc_ph = COLSUM ? (unit_idx & 1U) : ((unit_idx >> 1) & 1U);
            const bool got = mbar_wait(tfull0 + 8 * buf, acc_ph);
            if (!got) {
                if (lane == 0) atomicExch(err_flag, 204);
                break;
            }
            tcgen05_fence_after();
            const uint32_t row0 = tm * 2 * BM + rank * BM + quad * 32;
            const uint32_t tbase = tmem_base + ((uint32_t)(quad * 32) << 16) + buf * PBN;
            if (COLSUM && tn == 0U && chalf == 0) {
                uint32_t cs[32];
                tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(quad * 32) << 16) + PBN, cs);   // every column holds the row's sum
                const uint32_t row = row0 + lane;
                if (row < M) colsum_partial[(size_t)z * M + row] = __uint_as_float(cs[0]);
            }
            if (SWIGLU) {
                // this warp: 32 rows x 64 activation columns, 32 at a time (x1 and x2 values of the same columns); the three
                // staged tiles of the previous unit have been read by their stores long ago (a whole unit lies between)
                if (lane == 0) bulk_wait_group_read<0>();
                __syncwarp();
                unsigned char *r1 = my_stage + lane * 128, *r2 = r1 + 4096, *ra = r2 + 4096;
                const uint32_t acol = tn * (PBN / 2) + (uint32_t)(chalf * 64);    // first activation column of this warp
#pragma unroll 1
                for (int c = 0; c < 2; ++c) {
                    const uint32_t lc = (uint32_t)(chalf * 64 + c * 32);   // column inside the unit's 128
                    uint32_t v1[32], v2[32];
                    tmem_ld_32x32b_x32_nowait(tbase + lc, v1);
                    tmem_ld_32x32b_x32_nowait(tbase + PBN / 2 + lc, v2);
                    tmem_ld_wait();
                    if (c == 1) {
                        tcgen05_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_cluster(tempty_leader + 8 * buf);
                    }
                    const uint32_t col0 = acol + c * 32;       // activation column = x1 column; x2 column = N + col0
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        uint32_t o1[4], o2[4], oa[4];
#pragma unroll
                        for (int e = 0; e < 8; e += 2) {
                            float a0 = __uint_as_float(v1[j + e]), a1 = __uint_as_float(v1[j + e + 1]);
                            float z0 = __uint_as_float(v2[j + e]), z1 = __uint_as_float(v2[j + e + 1]);
                            if (bias != nullptr) {
                                if (bias_mode == 2) {
                                    a0 = gdb_io<T>::rnd(a0);
                                    a1 = gdb_io<T>::rnd(a1);
                                    z0 = gdb_io<T>::rnd(z0);
                                    z1 = gdb_io<T>::rnd(z1);
                                }
                                const uint32_t cc = col0 + j + e;
                                a0 += cc < N ? gdb_io<T>::ld(bias, cc) : 0.0f;
                                a1 += cc + 1 < N ? gdb_io<T>::ld(bias, cc + 1) : 0.0f;
                                z0 += cc < N ? gdb_io<T>::ld(bias, N + cc) : 0.0f;
                                z1 += cc + 1 < N ? gdb_io<T>::ld(bias, N + cc + 1) : 0.0f;
                            }
                            a0 = gdb_io<T>::rnd(a0);
                            a1 = gdb_io<T>::rnd(a1);
                            z0 = gdb_io<T>::rnd(z0);
                            z1 = gdb_io<T>::rnd(z1);
                            o1[e >> 1] = half_pack<T>::pack(a0, a1);
                            o2[e >> 1] = half_pack<T>::pack(z0, z1);
                            oa[e >> 1] = half_pack<T>::pack(a0 * (z0 * gdb_swiglu_sigmoid(z0)), a1 * (z1 * gdb_swiglu_sigmoid(z1)));
                        }
                        const int chunk = ((c * 4 + (j >> 3)) ^ (lane & 7)) << 4;   // 16-byte chunk of the 128-byte swizzled row
                        *reinterpret_cast<uint4 *>(r1 + chunk) = make_uint4(o1[0], o1[1], o1[2], o1[3]);
                        *reinterpret_cast<uint4 *>(r2 + chunk) = make_uint4(o2[0], o2[1], o2[2], o2[3]);
                        *reinterpret_cast<uint4 *>(ra + chunk) = make_uint4(oa[0], oa[1], oa[2], oa[3]);
                    }
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    if (row0 < M && acol < N) {
                        tma_store_2d(&tma_c, (int)acol, (int)row0, smem_u32(my_stage));
                        tma_store_2d(&tma_c, (int)(N + acol), (int)row0, smem_u32(my_stage + 4096));
                        tma_store_2d(&tma_act, (int)acol, (int)row0, smem_u32(my_stage + 8192));
                    }
                    bulk_commit_group();
                }
                continue;
            }
            if (SWIGLU_BWD) {
                const uint32_t row = row0 + lane;
#pragma unroll 1
                for (int c = chalf * 2; c < chalf * 2 + 2; ++c) {          // two chunks of 64 columns per warp
                    const uint32_t col0 = tn * PBN + c * 64;
                    if (lane == 0) bulk_wait_group_read<0>();               // the two staged tiles of the previous chunk have been read
                    __syncwarp();
                    unsigned char *r1 = my_stage + lane * 128, *r2 = r1 + 4096;
#pragma unroll 1
                    for (int pc = 0; pc < 2; ++pc) {                        // 32 columns at a time
                        const uint32_t cc0 = col0 + pc * 32;
                        uint4 xa[4], xb[4];
                        const bool in = row < M && cc0 < N;
                        const uint4 *p1 = reinterpret_cast<const uint4 *>(aux + (size_t)row * ld_aux + cc0);
                        const uint4 *p2 = reinterpret_cast<const uint4 *>(aux + (size_t)row * ld_aux + N + cc0);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            xa[j] = in ? p1[j] : make_uint4(0U, 0U, 0U, 0U);
                            xb[j] = in ? p2[j] : make_uint4(0U, 0U, 0U, 0U);
                        }
                        uint32_t v[32];
                        tmem_ld_32x32b_x32(tbase + c * 64 + pc * 32, v);
                        if (c == chalf * 2 + 1 && pc == 1) {
                            tcgen05_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive_cluster(tempty_leader + 8 * buf);
                        }
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            gdb_vec8<T> a, b, d1, d2;
                            a.raw = xa[j];
                            b.raw = xb[j];
#pragma unroll
                            for (int e = 0; e < 8; ++e) {
                                const float gv = gdb_io<T>::rnd(__uint_as_float(v[j * 8 + e]));
                                const float z = b.get(e), sg = gdb_swiglu_sigmoid(z);
                                d1.set(e, gv * (z * sg));
                                d2.set(e, gv * a.get(e) * (sg * (1.0f + z * (1.0f - sg))));
                            }
                            const int chunk = ((pc * 4 + j) ^ (lane & 7)) << 4;
                            *reinterpret_cast<uint4 *>(r1 + chunk) = d1.raw;
                            *reinterpret_cast<uint4 *>(r2 + chunk) = d2.raw;
                        }
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        if (row0 < M && col0 < N) {
                            tma_store_2d(&tma_c, (int)col0, (int)row0, smem_u32(my_stage));
                            tma_store_2d(&tma_c, (int)(N + col0), (int)row0, smem_u32(my_stage + 4096));
                        }
                        bulk_commit_group();
                    }
                }
                continue;
            }
            constexpr int NCH = PBN / CHUNK_COLS / 2;   // chunks per warp
#pragma unroll 1
            for (int c = chalf * NCH; c < (chalf + 1) * NCH; ++c) {
                uint32_t v0[32], v1[32];
                tmem_ld_32x32b_x32_nowait(tbase + c * CHUNK_COLS, v0);
                if (!SPLITK) {
                    tmem_ld_32x32b_x32_nowait(tbase + c * CHUNK_COLS + 32, v1);
                }
                tmem_ld_wait();
                if (c == (chalf + 1) * NCH - 1) {
                    // the accumulator has been copied out: hand the buffer back to the MMA issuer
                    tcgen05_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(tempty_leader + 8 * buf);
                }
                unsigned char *sb = my_stage + (store_cnt & 1U) * 4096;
                if (lane == 0) bulk_wait_group_read<1>();   // the store that last used this buffer has read it
                __syncwarp();
                const uint32_t col0 = tn * PBN + c * CHUNK_COLS;
                unsigned char *rowp = sb + lane * 128;
                if (SPLITK) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        *reinterpret_cast<uint4 *>(rowp + ((j ^ (lane & 7)) << 4)) = make_uint4(v0[4 * j], v0[4 * j + 1], v0[4 * j + 2], v0[4 * j + 3]);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        float f[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const int idx = j * 8 + e;
                            f[e] = __uint_as_float(idx < 32 ? v0[idx & 31] : v1[idx & 31]);
                            if (bias != nullptr) {
                                // mode 2 reproduces "round the product, then a rounded bias add"
                                if (bias_mode == 2) f[e] = gdb_io<T>::rnd(f[e]);
                                const uint32_t col = col0 + idx;
                                f[e] += col < N ? gdb_io<T>::ld(bias, col) : 0.0f;
                            }
                        }
                        uint4 o;
                        o.x = half_pack<T>::pack(f[0], f[1]);
                        o.y = half_pack<T>::pack(f[2], f[3]);
                        o.z = half_pack<T>::pack(f[4], f[5]);
                        o.w = half_pack<T>::pack(f[6], f[7]);
                        *reinterpret_cast<uint4 *>(rowp + ((j ^ (lane & 7)) << 4)) = o;
                    }
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    if (row0 < M && col0 < N) {
                        if (SPLITK) {
                            tma_store_3d(&tma_c, (int)col0, (int)row0, (int)z, smem_u32(sb));
                        } else {
                            tma_store_2d(&tma_c, (int)col0, (int)row0, smem_u32(sb));
                        }
                    }
                    bulk_commit_group();
                }
                ++store_cnt;
            }
        }
        if (lane == 0) bulk_wait_all();
    }
    __syncwarp();
    tcgen05_fence_before();
    cluster_sync_all();   // neither CTA releases tensor memory while its peer may still use it
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)(2 * PBN)) : "memory");
    }
}

int max_clusters(gd_backend *be, const void *kern, int smem_bytes)
{
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.gridDim = dim3((unsigned)be->sm_count & ~1U);
    cfg.blockDim = dim3(P_THREADS);
    cfg.dynamicSmemBytes = (size_t)smem_bytes;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
        (void)cudaGetLastError();
        return 0;
    }
    return n < be->sm_count / 2 ? n : be->sm_count / 2;
}

template <typename T, bool A_MN, bool B_MN, bool SPLITK, bool COLSUM = false, bool SWIGLU = false, bool SWIGLU_BWD = false>
gd_status launch_pair(gd_backend *be, const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &tc, const void *bias, uint32_t M,
                      uint32_t N, uint32_t K, uint32_t tiles_m, uint32_t tiles_n, uint32_t splits, uint32_t kps, int bias_mode, int *clusters_out,
                      float *colsum_partial = nullptr, const CUtensorMap *tact = nullptr, const void *aux = nullptr, size_t ld_aux = 0)
{
    constexpr int SMEM = SWIGLU ? P_SMEM_TOTAL_SWIGLU : (COLSUM ? P_SMEM_TOTAL_COLSUM : P_SMEM_TOTAL);
    auto kern = gemm_pair_kernel<T, A_MN, B_MN, SPLITK, COLSUM, SWIGLU, SWIGLU_BWD>;
    static int clusters = -1;
    if (clusters < 0) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) {
            return gdb_fail(be, e, "tcgen05 pair gemm smem attribute");
        }
        clusters = max_clusters(be, (const void *)kern, SMEM);
    }
    if (clusters_out != nullptr) {
        *clusters_out = clusters;
        return GD_OK;
    }
    if (clusters <= 0) {
        return GD_ERR_UNSUPPORTED;
    }
    const uint32_t units = tiles_m * tiles_n * splits;
    const int usable = clusters - (be->sm_reserve + 1) / 2 > 0 ? clusters - (be->sm_reserve + 1) / 2 : 1;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // see gdb_pdl_sync()
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.gridDim = dim3(2U * (units < (uint32_t)usable ? units : (uint32_t)usable));
    cfg.blockDim = dim3(P_THREADS);
    cfg.dynamicSmemBytes = SMEM;
    cfg.stream = be->stream;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, ta, tb, tc, (const T *)bias, M, N, K, tiles_m, tiles_n, splits, kps, bias_mode, be->err_flag, colsum_partial,
                                       tact != nullptr ? *tact : tc, (const T *)aux, ld_aux);
    if (e != cudaSuccess) {
        be->launches += 1U;
        return gdb_fail(be, e, "gemm_tcgen05_pair");
    }
    return gdb_launched(be, "gemm_tcgen05_pair");
}

template <typename T>
gd_status dispatch_pair(gd_backend *be, int ta, int tb, bool sk, const CUtensorMap &ma, const CUtensorMap &mb, const CUtensorMap &mc,
                        const void *bias, uint32_t M, uint32_t N, uint32_t K, uint32_t tiles_m, uint32_t tiles_n, uint32_t splits,
                        uint32_t kps, int bias_mode, int *clusters_out)
{
#define GDB_GO(AM, BMJ)                                                                                                         \
    (sk ? launch_pair<T, AM, BMJ, true>(be, ma, mb, mc, bias, M, N, K, tiles_m, tiles_n, splits, kps, bias_mode, clusters_out) \
        : launch_pair<T, AM, BMJ, false>(be, ma, mb, mc, bias, M, N, K, tiles_m, tiles_n, splits, kps, bias_mode, clusters_out))
    if (ta) {
        return tb ? GDB_GO(true, false) : GDB_GO(true, true);
    }
    return tb ? GDB_GO(false, false) : GDB_GO(false, true);
#undef GDB_GO
}

}  // namespace

// Same contract as gdb_gemm_tcgen05 (which calls this first). Returns GD_ERR_UNSUPPORTED when the
// problem is too small for 256-row tiles or clusters of two cannot be scheduled; `*splits_out`
// receives the number of FP32 partial slices written to the workspace (1 = C was written directly).
// `colsum_partial_out` != NULL (only for ta = 1, tb = 0, the weight-gradient layout): the FP32 partial path is taken even
// for a single k-slice, and *colsum_partial_out receives the workspace address of colsum partials [*splits_out, M].
gd_status gdb_gemm_tcgen05_pair(gd_backend *be, int ta, int tb, uint32_t dtype, const void *a, size_t lda_bytes, const void *b,
                                size_t ldb_bytes, void *c, size_t ldc_bytes, const void *bias, int bias_mode, uint32_t M, uint32_t N,
                                uint32_t K, uint32_t *splits_out, float **colsum_partial_out)
{
    *splits_out = 1;
    const bool want_colsum = colsum_partial_out != nullptr;
    if (M < 256U || N < 128U || K < 64U || (want_colsum && !(ta && !tb))) {
        return GD_ERR_UNSUPPORTED;
    }
    CUtensorMap ma, mb, mc;
    const bool oka = ta ? make_tmap(&ma, dtype, a, K, M, lda_bytes, 64, BK) : make_tmap(&ma, dtype, a, M, K, lda_bytes, BK, BM);
    const bool okb = tb ? make_tmap(&mb, dtype, b, N, K, ldb_bytes, BK, PBN / 2) : make_tmap(&mb, dtype, b, K, N, ldb_bytes, 64, BK);
    if (!oka || !okb) {
        return GD_ERR_UNSUPPORTED;
    }
    int clusters = 0;
    gd_status st = dtype == GDB_DTYPE_F16
                       ? dispatch_pair<__half>(be, ta, tb, false, ma, mb, ma, bias, M, N, K, 0, 0, 1, 0, bias_mode, &clusters)
                       : dispatch_pair<__nv_bfloat16>(be, ta, tb, false, ma, mb, ma, bias, M, N, K, 0, 0, 1, 0, bias_mode, &clusters);
    if (st != GD_OK || clusters <= 0) {
        return GD_ERR_UNSUPPORTED;
    }
    const uint32_t tiles_m = (M + 2 * BM - 1) / (2 * BM), tiles_n = (N + PBN - 1) / PBN, tiles = tiles_m * tiles_n;
    const uint32_t total_k = (K + BK - 1) / BK;
    uint32_t splits = 1;
    if (tiles * 2U <= (uint32_t)clusters && total_k >= 16U) {
        splits = (uint32_t)clusters / tiles;
        if (splits > total_k / 4U) splits = total_k / 4U;
        while (splits > 1U && (size_t)splits * M * N * sizeof(float) > be->ws_bytes / 2U) --splits;
        if (splits < 1U) splits = 1U;
    }
    if (splits == 1U && tiles * 4U < (uint32_t)clusters) {
        return GD_ERR_UNSUPPORTED;   // a handful of tiles: the single-CTA kernel spreads them over more SMs
    }
    uint32_t kps = (total_k + splits - 1U) / splits;
    splits = (total_k + kps - 1U) / kps;
    if (want_colsum) {
        const size_t dw_bytes = ((size_t)splits * M * N * sizeof(float) + 255U) & ~(size_t)255U;
        if (dw_bytes + (size_t)splits * M * sizeof(float) > be->ws_bytes / 2U) {
            return GD_ERR_UNSUPPORTED;
        }
        float *cs = reinterpret_cast<float *>(be->ws + dw_bytes);
        if (!make_tmap_f32_3d(&mc, be->ws, splits, M, N, 32)) {
            return GD_ERR_UNSUPPORTED;
        }
        st = dtype == GDB_DTYPE_F16
                 ? launch_pair<__half, true, true, true, true>(be, ma, mb, mc, bias, M, N, K, tiles_m, tiles_n, splits, kps, bias_mode, nullptr, cs)
                 : launch_pair<__nv_bfloat16, true, true, true, true>(be, ma, mb, mc, bias, M, N, K, tiles_m, tiles_n, splits, kps, bias_mode, nullptr, cs);
        if (st == GD_OK) {
            *splits_out = splits;
            *colsum_partial_out = cs;
        }
        return st;
    }
    const bool sk = splits > 1U;
    const bool okc = sk ? make_tmap_f32_3d(&mc, be->ws, splits, M, N, 32) : make_tmap(&mc, dtype, c, M, N, ldc_bytes, 64, 32);
    if (!okc) {
        return GD_ERR_UNSUPPORTED;
    }
    st = dtype == GDB_DTYPE_F16
             ? dispatch_pair<__half>(be, ta, tb, sk, ma, mb, mc, bias, M, N, K, tiles_m, tiles_n, splits, kps, bias_mode, nullptr)
             : dispatch_pair<__nv_bfloat16>(be, ta, tb, sk, ma, mb, mc, bias, M, N, K, tiles_m, tiles_n, splits, kps, bias_mode, nullptr);
    if (st == GD_OK) {
        *splits_out = splits;
    }
    return st;
}

// x12[M, 2F] = round(round(x w^T) + bias) and act[M, F] = x1 * x2 * sigmoid(x2) from ONE contraction (w stored [2F, K], x1
// rows first): the SwiGLU epilogue of the CTA-pair kernel. GD_ERR_UNSUPPORTED when the shape does not fit it (the caller
// then issues the three separate calls, which give the same bits).
gd_status gdb_gemm_tcgen05_pair_swiglu(gd_backend *be, uint32_t dtype, const void *x, size_t ldx_bytes, const void *w, size_t ldw_bytes,
                                       const void *bias, void *x12, size_t ld12_bytes, void *act, size_t ldact_bytes, uint32_t M, uint32_t F,
                                       uint32_t K)
{
    const uintptr_t al = (uintptr_t)x | (uintptr_t)w | (uintptr_t)x12 | (uintptr_t)act;
    if ((dtype != GDB_DTYPE_F16 && dtype != GDB_DTYPE_BF16) || M < 256U || F < 128U || (F % 128U) != 0U || K < 64U || (K % 8U) != 0U || (al % 16U) != 0U ||
        (ldx_bytes % 16U) != 0U || (ldw_bytes % 16U) != 0U || (ld12_bytes % 16U) != 0U || (ldact_bytes % 16U) != 0U || bias == nullptr) {
        return GD_ERR_UNSUPPORTED;
    }
    CUtensorMap ma, mb, m12, mact;
    if (!make_tmap(&ma, dtype, x, M, K, ldx_bytes, BK, BM) || !make_tmap(&mb, dtype, w, 2ULL * F, K, ldw_bytes, BK, PBN / 2) ||
        !make_tmap(&m12, dtype, x12, M, 2ULL * F, ld12_bytes, 64, 32) || !make_tmap(&mact, dtype, act, M, F, ldact_bytes, 64, 32)) {
        return GD_ERR_UNSUPPORTED;
    }
    const uint32_t tiles_m = (M + 2 * BM - 1) / (2 * BM), tiles_n = F / (PBN / 2), kps = (K + BK - 1) / BK;
    return dtype == GDB_DTYPE_F16
               ? launch_pair<__half, false, false, false, false, true>(be, ma, mb, m12, bias, M, F, K, tiles_m, tiles_n, 1, kps, 2, nullptr, nullptr, &mact)
               : launch_pair<__nv_bfloat16, false, false, false, false, true>(be, ma, mb, m12, bias, M, F, K, tiles_m, tiles_n, 1, kps, 2, nullptr, nullptr, &mact);
}

// d_x12[M, 2F] = swiglu_split_backward(x12, round(g w^T)) for w stored [F, K] (the down projection's weight, K = its output
// width): the input gradient of the down projection with the SwiGLU backward in the epilogue, so dact never reaches memory.
// GD_ERR_UNSUPPORTED when the shape does not fit (the caller then issues matmul_nt + swiglu_split_backward: same bits).
gd_status gdb_gemm_tcgen05_pair_swiglu_bwd(gd_backend *be, uint32_t dtype, const void *g, size_t ldg_bytes, const void *w, size_t ldw_bytes,
                                           const void *x12, size_t ld12_bytes, void *d_x12, size_t ldd_bytes, uint32_t M, uint32_t F, uint32_t K)
{
    const uintptr_t al = (uintptr_t)g | (uintptr_t)w | (uintptr_t)x12 | (uintptr_t)d_x12;
    if ((dtype != GDB_DTYPE_F16 && dtype != GDB_DTYPE_BF16) || M < 256U || F < 256U || (F % 64U) != 0U || K < 64U || (K % 8U) != 0U || (al % 16U) != 0U ||
        (ldg_bytes % 16U) != 0U || (ldw_bytes % 16U) != 0U || (ld12_bytes % 16U) != 0U || (ldd_bytes % 16U) != 0U) {
        return GD_ERR_UNSUPPORTED;
    }
    CUtensorMap ma, mb, md;
    if (!make_tmap(&ma, dtype, g, M, K, ldg_bytes, BK, BM) || !make_tmap(&mb, dtype, w, F, K, ldw_bytes, BK, PBN / 2) ||
        !make_tmap(&md, dtype, d_x12, M, 2ULL * F, ldd_bytes, 64, 32)) {
        return GD_ERR_UNSUPPORTED;
    }
    const uint32_t tiles_m = (M + 2 * BM - 1) / (2 * BM), tiles_n = (F + PBN - 1) / PBN, kps = (K + BK - 1) / BK;
    return dtype == GDB_DTYPE_F16
               ? launch_pair<__half, false, false, false, false, false, true>(be, ma, mb, md, nullptr, M, F, K, tiles_m, tiles_n, 1, kps, 0, nullptr, nullptr,
                                                                              nullptr, x12, ld12_bytes / 2U)
               : launch_pair<__nv_bfloat16, false, false, false, false, false, true>(be, ma, mb, md, nullptr, M, F, K, tiles_m, tiles_n, 1, kps, 0, nullptr,
                                                                                     nullptr, nullptr, x12, ld12_bytes / 2U);
}
