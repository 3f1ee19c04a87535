// Contraction with at most 64 output rows (one KV-decode step: M = batch): C[M, N] = A[M, K] * B (+ bias).
//
// At this size a 128-row tcgen05 tile pipeline is all fixed latency (tensor-map fetch, tensor-memory
// allocation, mbarrier round trips) and fills a dozen SMs; the operands are a few hundred KB and sit
// in L2. Here one CTA owns 16 output columns, so N / 16 CTAs spread the weight read over the chip;
// its 8 warps split K, each issues all of its fragment loads straight from global memory (one round
// trip), runs mma.sync m16n8k16 with FP32 accumulators, and the partial tiles are summed through
// shared memory before the bias add and the single rounding.
#include "common.cuh"
#include "decode_parts.cuh"

#include <stdlib.h>

namespace {

using namespace gdb_dec;

// B_KMAJOR: B stored [N, K] (matmul_nt); otherwise B stored [K, N] (matmul / linear).
template <typename T, bool B_KMAJOR>
__global__ void __launch_bounds__(SK_WARPS * 32)
gemm_skinny_kernel(const T *__restrict__ A, size_t lda, const T *__restrict__ B, size_t ldb, T *__restrict__ C, size_t ldc,
                   const T *__restrict__ bias, int bias_mode, uint32_t M, uint32_t N, uint32_t K)
{
    gdb_pdl_sync();
    __shared__ float red[SK_WARPS][SK_ROWS][SK_COLS + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const uint32_t n0 = blockIdx.x * SK_COLS;
    const uint32_t k_steps = K / 16U, per_warp = (k_steps + SK_WARPS - 1) / SK_WARPS;
    const uint32_t ks0 = min(k_steps, warp * per_warp), ks1 = min(k_steps, ks0 + per_warp);
    float acc[4][2][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.0f;
    const unsigned short *Bu = reinterpret_cast<const unsigned short *>(B);
#pragma unroll 4
    for (uint32_t ks = ks0; ks < ks1; ++ks) {
        const uint32_t k0 = ks * 16U;
        uint32_t a[4][4], b[2][2];
#pragma unroll
        for (int mt = 0; mt < 4; ++mt) {
            const uint32_t r0 = mt * 16 + g, r1 = r0 + 8;
            const T *p0 = A + (size_t)r0 * lda + k0 + 2 * t, *p1 = A + (size_t)r1 * lda + k0 + 2 * t;
            a[mt][0] = r0 < M ? __ldg(reinterpret_cast<const uint32_t *>(p0)) : 0U;
            a[mt][1] = r1 < M ? __ldg(reinterpret_cast<const uint32_t *>(p1)) : 0U;
            a[mt][2] = r0 < M ? __ldg(reinterpret_cast<const uint32_t *>(p0 + 8)) : 0U;
            a[mt][3] = r1 < M ? __ldg(reinterpret_cast<const uint32_t *>(p1 + 8)) : 0U;
        }
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            const uint32_t n = n0 + nt * 8 + g;
            if (B_KMAJOR) {
                const T *p = B + (size_t)n * ldb + k0 + 2 * t;
                b[nt][0] = __ldg(reinterpret_cast<const uint32_t *>(p));
                b[nt][1] = __ldg(reinterpret_cast<const uint32_t *>(p + 8));
            } else {
                const unsigned short *p = Bu + (size_t)(k0 + 2 * t) * ldb + n;
                b[nt][0] = (uint32_t)__ldg(p) | ((uint32_t)__ldg(p + ldb) << 16);
                b[nt][1] = (uint32_t)__ldg(p + 8 * ldb) | ((uint32_t)__ldg(p + 9 * ldb) << 16);
            }
        }
#pragma unroll
        for (int mt = 0; mt < 4; ++mt)
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) mma16816<T>::run(acc[mt][nt], a[mt], b[nt]);
    }
#pragma unroll
    for (int mt = 0; mt < 4; ++mt)
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            const int r = mt * 16 + g, c = nt * 8 + 2 * t;
            red[warp][r][c] = acc[mt][nt][0];
            red[warp][r][c + 1] = acc[mt][nt][1];
            red[warp][r + 8][c] = acc[mt][nt][2];
            red[warp][r + 8][c + 1] = acc[mt][nt][3];
        }
    __syncthreads();
    for (int o = threadIdx.x; o < SK_ROWS * SK_COLS; o += SK_WARPS * 32) {
        const int r = o / SK_COLS, c = o % SK_COLS;
        if ((uint32_t)r >= M) continue;
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < SK_WARPS; ++w) v += red[w][r][c];
        if (bias != nullptr) {
            if (bias_mode == 2) v = gdb_io<T>::rnd(v);   // "round the product, then a rounded bias add"
            v += gdb_io<T>::ld(bias, n0 + c);
        }
        gdb_io<T>::st(C, (size_t)r * ldc + n0 + c, v);
    }
}

// ---- staged variant: operands reach shared memory with coalesced 16-byte cp.async, fragments come from ldmatrix
// (helpers and the per-chunk multiply in decode_parts.cuh) ----
// K is walked in chunks of CH (a multiple of 128): per chunk the CTA stages A[64, CH] and its 16 columns of B, each
// warp multiplies its CH / 8 slice, and with more than one chunk the next one is in flight (two stages).
// SWIGLU (B K-major, i.e. a transposed weight [2N, K] = [up | gate] rows): the CTA takes 8 "up" rows and the 8 "gate"
// rows N further down, and its epilogue applies out = up * silu(gate) to the two rounded linear outputs, so C is the
// [M, N] activation and the [M, 2N] intermediate is never written. Rounding points are those of the two separate
// calls: round(product), round(+ bias), round(up * silu(gate)).
template <typename T, bool B_KMAJOR, bool SWIGLU = false>
__global__ void __launch_bounds__(SK_WARPS * 32)
gemm_skinny_staged_kernel(const T *__restrict__ A, size_t lda, const T *__restrict__ B, size_t ldb, T *__restrict__ C, size_t ldc,
                          const T *__restrict__ bias, int bias_mode, uint32_t M, uint32_t N, uint32_t K, uint32_t CH, int stages)
{
    gdb_pdl_sync();
    extern __shared__ __align__(16) unsigned char sk_sm[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    static_assert(!SWIGLU || B_KMAJOR, "the fused SwiGLU epilogue reads a transposed weight");
    const uint32_t n0 = blockIdx.x * (SWIGLU ? SK_COLS / 2 : SK_COLS);
    const uint32_t LDA = CH + 8U, LDW = B_KMAJOR ? CH + 8U : 24U;
    const uint32_t a_bytes = SK_ROWS * LDA * 2U, w_bytes = (B_KMAJOR ? (uint32_t)SK_COLS : CH) * LDW * 2U, stage_bytes = a_bytes + w_bytes;
    const uint32_t n_chunks = K / CH, segs = CH / 8U;
    auto load_chunk = [&](uint32_t ci, uint32_t st) {
        T *As = reinterpret_cast<T *>(sk_sm + st * stage_bytes), *Ws = reinterpret_cast<T *>(sk_sm + st * stage_bytes + a_bytes);
        const size_t k0 = (size_t)ci * CH;
        for (uint32_t i = tid; i < SK_ROWS * segs; i += SK_WARPS * 32) {
            const uint32_t r = i / segs, sgm = i % segs;
            sk_cp16(As + r * LDA + sgm * 8U, A + (size_t)(r < M ? r : 0U) * lda + k0 + sgm * 8U, r < M);
        }
        if (B_KMAJOR) {
            for (uint32_t i = tid; i < SK_COLS * segs; i += SK_WARPS * 32) {
                const uint32_t r = i / segs, sgm = i % segs;
                const uint32_t wrow = SWIGLU ? (r < 8U ? n0 + r : N + n0 + (r - 8U)) : n0 + r;
                sk_cp16(Ws + r * LDW + sgm * 8U, B + (size_t)wrow * ldb + k0 + sgm * 8U, true);
            }
        } else {
            for (uint32_t i = tid; i < CH * 2U; i += SK_WARPS * 32) {
                const uint32_t k = i >> 1, sgm = i & 1U;
                sk_cp16(Ws + k * LDW + sgm * 8U, B + (k0 + k) * ldb + n0 + sgm * 8U, true);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    load_chunk(0, 0);
    if (stages == 2 && n_chunks > 1U) load_chunk(1, 1);
    float acc[4][2][4];
    sk_zero(acc);
    const uint32_t kw = CH / SK_WARPS;   // k elements per warp and chunk (a multiple of 16)
    for (uint32_t ci = 0; ci < n_chunks; ++ci) {
        const uint32_t st = stages == 2 ? (ci & 1U) : 0U;
        if (stages == 2 && ci + 1U < n_chunks) {
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const T *As = reinterpret_cast<const T *>(sk_sm + st * stage_bytes), *Ws = reinterpret_cast<const T *>(sk_sm + st * stage_bytes + a_bytes);
        sk_mma_chunk<T, B_KMAJOR>(acc, As, Ws, LDA, LDW, warp * kw, (warp + 1U) * kw, lane);
        __syncthreads();   // every warp is done with this stage before it is refilled (or reused for the reduction)
        if (stages == 2) {
            if (ci + 2U < n_chunks) load_chunk(ci + 2U, st);
        } else if (ci + 1U < n_chunks) {
            load_chunk(ci + 1U, 0);
        }
    }
    sk_red_t red = reinterpret_cast<sk_red_t>(sk_sm);
    sk_store_partials(red, acc, warp, lane);
    __syncthreads();
    if (SWIGLU) {
        for (int o = tid; o < SK_ROWS * (SK_COLS / 2); o += SK_WARPS * 32) {
            const int r = o / (SK_COLS / 2), c = o % (SK_COLS / 2);
            if ((uint32_t)r >= M) continue;
            const float up = sk_sum(red, r, c), gate = sk_sum(red, r, c + 8);
            gdb_io<T>::st(C, (size_t)r * ldc + n0 + c, sk_swiglu<T>(up, gate, bias, bias_mode, n0 + c, N + n0 + c));
        }
        return;
    }
    for (int o = tid; o < SK_ROWS * SK_COLS; o += SK_WARPS * 32) {
        const int r = o / SK_COLS, c = o % SK_COLS;
        if ((uint32_t)r >= M) continue;
        gdb_io<T>::st(C, (size_t)r * ldc + n0 + c, sk_bias<T>(sk_sum(red, r, c), bias, bias_mode, n0 + c));
    }
}

template <typename T, bool B_KMAJOR, bool SWIGLU = false>
gd_status launch_staged(gd_backend *be, const void *a, size_t lda, const void *b, size_t ldb, void *c, size_t ldc, const void *bias, int bias_mode,
                        uint32_t M, uint32_t N, uint32_t K, uint32_t ch)
{
    auto kern = gemm_skinny_staged_kernel<T, B_KMAJOR, SWIGLU>;
    const int stages = K / ch > 1U ? 2 : 1;
    const uint32_t a_bytes = SK_ROWS * (ch + 8U) * 2U, w_bytes = B_KMAJOR ? SK_COLS * (ch + 8U) * 2U : ch * 24U * 2U;
    size_t smem = (size_t)stages * (a_bytes + w_bytes);
    const size_t red_bytes = SK_RED_BYTES;
    if (smem < red_bytes) smem = red_bytes;
    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return gdb_fail(be, e, "skinny gemm smem attribute");
        configured = smem;
    }
    gdb_launch(kern, N / (SWIGLU ? SK_COLS / 2 : SK_COLS), SK_WARPS * 32, smem, be->stream, (const T *)a, lda, (const T *)b, ldb, (T *)c, ldc, (const T *)bias, bias_mode, M, N, K, ch, stages);
    return gdb_launched(be, "gemm_skinny_staged");
}

}  // namespace

// Returns GD_ERR_UNSUPPORTED unless M <= 64, N % 16 == 0, K % 16 == 0 and the operands are 4-byte aligned.
gd_status gdb_gemm_skinny(gd_backend *be, int tb, uint32_t dtype, const void *a, size_t lda_bytes, const void *b, size_t ldb_bytes,
                          void *c, size_t ldc_bytes, const void *bias, int bias_mode, uint32_t M, uint32_t N, uint32_t K)
{
    if ((dtype != GDB_DTYPE_F16 && dtype != GDB_DTYPE_BF16) || M == 0U || M > (uint32_t)SK_ROWS || (N % SK_COLS) != 0U || (K % 16U) != 0U ||
        K == 0U || (((uintptr_t)a | (uintptr_t)b | lda_bytes | ldb_bytes) % 4U) != 0U || (ldc_bytes % 2U) != 0U) {
        return GD_ERR_UNSUPPORTED;
    }
    const size_t lda = lda_bytes / 2U, ldb = ldb_bytes / 2U, ldc = ldc_bytes / 2U;
    // staged variant: K in chunks of 512 / 256 / 128 and 16-byte aligned rows
    const uint32_t ch = sk_chunk_for(K);
    if (ch != 0U && (((uintptr_t)a | (uintptr_t)b | lda_bytes | ldb_bytes) % 16U) == 0U && getenv("GDB200_SKINNY_DIRECT") == NULL) {
        if (dtype == GDB_DTYPE_F16) {
            return tb ? launch_staged<__half, true>(be, a, lda, b, ldb, c, ldc, bias, bias_mode, M, N, K, ch)
                      : launch_staged<__half, false>(be, a, lda, b, ldb, c, ldc, bias, bias_mode, M, N, K, ch);
        }
        return tb ? launch_staged<__nv_bfloat16, true>(be, a, lda, b, ldb, c, ldc, bias, bias_mode, M, N, K, ch)
                  : launch_staged<__nv_bfloat16, false>(be, a, lda, b, ldb, c, ldc, bias, bias_mode, M, N, K, ch);
    }
    const unsigned grid = N / SK_COLS;
#define GDB_SK(TT, KM) gdb_launch(gemm_skinny_kernel<TT, KM>, grid, SK_WARPS * 32, 0, be->stream, (const TT *)a, lda, (const TT *)b, ldb, (TT *)c, ldc, (const TT *)bias, bias_mode, M, N, K)
    if (dtype == GDB_DTYPE_F16) {
        if (tb) GDB_SK(__half, true); else GDB_SK(__half, false);
    } else {
        if (tb) GDB_SK(__nv_bfloat16, true); else GDB_SK(__nv_bfloat16, false);
    }
#undef GDB_SK
    return gdb_launched(be, "gemm_skinny");
}

// out[M, N] = swiglu(x W^T + bias) for a transposed weight W [2N, K] = [up rows | gate rows] and bias [2N]: the linear layer
// and the gate of examples/gpt_lm/gpt_lm_shared.c:1032-1046 (gd_linear_transposed_weight + gd_swiglu_split) in one launch,
// with the rounding points of the two calls. Returns GD_ERR_UNSUPPORTED unless M <= 64, N % 8 == 0, K a multiple of 128
// and everything 16-byte aligned (the caller then issues the two calls).
gd_status gdb_gemm_skinny_swiglu(gd_backend *be, uint32_t dtype, const void *a, size_t lda_bytes, const void *w, size_t ldw_bytes,
                                 const void *bias, void *c, size_t ldc_bytes, uint32_t M, uint32_t N, uint32_t K)
{
    const uint32_t ch = sk_chunk_for(K);
    if ((dtype != GDB_DTYPE_F16 && dtype != GDB_DTYPE_BF16) || M == 0U || M > (uint32_t)SK_ROWS || N == 0U || (N % 8U) != 0U || ch == 0U ||
        (((uintptr_t)a | (uintptr_t)w | lda_bytes | ldw_bytes) % 16U) != 0U || (ldc_bytes % 2U) != 0U || getenv("GDB200_SKINNY_DIRECT") != NULL) {
        return GD_ERR_UNSUPPORTED;
    }
    const size_t lda = lda_bytes / 2U, ldw = ldw_bytes / 2U, ldc = ldc_bytes / 2U;
    return dtype == GDB_DTYPE_F16 ? launch_staged<__half, true, true>(be, a, lda, w, ldw, c, ldc, bias, 2, M, N, K, ch)
                                  : launch_staged<__nv_bfloat16, true, true>(be, a, lda, w, ldw, c, ldc, bias, 2, M, N, K, ch);
}
