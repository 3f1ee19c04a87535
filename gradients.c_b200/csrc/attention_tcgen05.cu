// Packed causal attention forward on the sm_100a tensor path: S = Q K^T and O = P V are
// tcgen05.mma instructions with FP32 accumulators in tensor memory, operands arrive by TMA.
//
// Fast path of gd_backend_sdpa_varlen for 16-bit storage, head_dim 64, causal (+ optional sliding
// window), no prefix. One CTA owns 128 consecutive rows of the PACKED token stream for one head; the
// mask is evaluated in packed coordinates exactly as in the mma.sync kernels (attention_flash.cu):
//   allowed(i, j)  <=>  seg_start(i) <= j <= i  and  (window == 0 or i - j < window)
// (src/ops/sdpa_varlen/metal_sdpa_varlen.metal:30-55, prefix 0), so a tile may span sequences.
//
// Roles (192 threads): warp 0 = TMA producer (Q once, K double-buffered, V single-buffered);
// warp 1 = MMA issuer; warps 2-5 = softmax, ONE THREAD PER QUERY ROW: a thread reads its row of S
// from tensor memory (tcgen05.ld 32x32b), so row max / row sum need no shuffles. Per key tile:
//   pass 1: row max of S over the allowed columns
//   (deferred) o += alpha * O_part of the previous tile, read back from tensor memory
//   pass 2: p = exp2(s * scale * log2e - m), written as 16-bit into the 128-byte-swizzled K-major
//           shared tile that the P V MMA reads as its A operand; running sum l
// Tensor memory: 2 buffers of BKV columns; S[t] lives in buffer t & 1 and, once consumed, the same
// buffer receives O_part[t] (64 columns), so 256 columns suffice and two CTAs share an SM.
// The MMA issuer keeps one S tile ahead: S[t+1] is issued while the softmax warps work on S[t].
//
// Statistics written for the backward pass: (row max in natural-log units, sum of exp, 0).
// Every mbarrier wait is bounded and reports through gd_backend::err_flag.
#include "attention.cuh"
#include "tcgen05.cuh"

namespace {
using namespace gdb_t5;

constexpr float LOG2E_F = 1.4426950408889634f;
constexpr float LN2_F = 0.6931471805599453f;
constexpr int A_BQ = 128, A_DH = 64;
constexpr int A_MAX_CU = 1024;

struct attn5_params {
    int n_tokens, batch, hq, hkv, window;
    float scale;
};

template <int BKV>
struct attn5_plan {
    static constexpr int Q_BYTES = A_BQ * 128;          // 128 rows x 64 x 2 B
    static constexpr int KV_BYTES = BKV * 128;
    static constexpr int P_BYTES = A_BQ * BKV * 2;      // BKV / 64 blocks of [128 rows x 128 B]
    static constexpr int OFF_K = Q_BYTES, OFF_V = OFF_K + 2 * KV_BYTES, OFF_P = OFF_V + KV_BYTES, OFF_BAR = OFF_P + P_BYTES;
    static constexpr int TOTAL = OFF_BAR + 256 + 1024;
    static constexpr int TMEM_COLS = 2 * BKV;
};

__device__ __forceinline__ float ex2_approx(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ int seg_start_of(const int *cu_s, int batch, int row)
{
    int lo = 0, hi = batch;
    while (lo + 1 < hi) {
        const int mid = (lo + hi) >> 1;
        if (cu_s[mid] <= row) lo = mid; else hi = mid;
    }
    return cu_s[lo];
}

template <typename T, int BKV>
__global__ void __launch_bounds__(192, 2)
attn5_fwd_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                 const __grid_constant__ CUtensorMap tma_v, const __grid_constant__ CUtensorMap tma_o,
                 const int *__restrict__ cu, float *__restrict__ stats, attn5_params p, int *err_flag)
{
    using plan = attn5_plan<BKV>;
    extern __shared__ unsigned char smem_raw[];
    __shared__ int cu_s[A_MAX_CU + 1];
    unsigned char *smem = (unsigned char *)(((uintptr_t)smem_raw + 1023U) & ~(uintptr_t)1023U);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + plan::OFF_BAR);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 16);
    enum { Q_FULL = 0, K_FULL = 1, K_EMPTY = 3, V_FULL = 5, V_EMPTY = 6, S_FULL = 7, P_FULL = 9, P_EMPTY = 10, O_FULL = 11, BUF_FREE = 13 };
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [&](int i) { return bar0 + 8U * (uint32_t)i; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q0 = blockIdx.x * A_BQ, h = blockIdx.y, hk = h / (p.hq / p.hkv);

    for (int i = threadIdx.x; i <= p.batch; i += blockDim.x) cu_s[i] = cu[i];
    if (threadIdx.x == 0) {
        for (int i = 0; i < 15; ++i) {
            const bool four = i == P_FULL || i == BUF_FREE || i == BUF_FREE + 1;
            mbar_init(bar(i), four ? 4U : 1U);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)plan::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int n_valid = min(cu_s[p.batch], p.n_tokens);
    int kv_begin = 0, n_tiles = 0;
    if (q0 < n_valid) {
        kv_begin = seg_start_of(cu_s, p.batch, q0);
        if (p.window > 0) kv_begin = max(kv_begin, q0 - p.window + 1);
        const int kv_end = min(q0 + A_BQ, n_valid);   // exclusive
        n_tiles = (kv_end - kv_begin + BKV - 1) / BKV;
    }

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0 && n_tiles > 0) {
            mbar_expect_tx(bar(Q_FULL), plan::Q_BYTES);
            tma_load_2d(smem_u32(smem), &tma_q, h * A_DH, q0, bar(Q_FULL));
            for (int t = 0; t < n_tiles; ++t) {
                const int key0 = kv_begin + t * BKV, ks = t & 1;
                if (!mbar_wait(bar(K_EMPTY + ks), ((t >> 1) & 1) ^ 1)) {
                    atomicExch(err_flag, 301);
                    break;
                }
                mbar_expect_tx(bar(K_FULL + ks), plan::KV_BYTES);
                tma_load_2d(smem_u32(smem + plan::OFF_K + ks * plan::KV_BYTES), &tma_k, hk * A_DH, key0, bar(K_FULL + ks));
                if (!mbar_wait(bar(V_EMPTY), (t & 1) ^ 1)) {
                    atomicExch(err_flag, 302);
                    break;
                }
                mbar_expect_tx(bar(V_FULL), plan::KV_BYTES);
                tma_load_2d(smem_u32(smem + plan::OFF_V), &tma_v, hk * A_DH, key0, bar(V_FULL));
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0 && n_tiles > 0) {
            constexpr uint32_t FMT = std::is_same<T, __nv_bfloat16>::value ? 1U : 0U;
            constexpr uint32_t IDESC_S = (1U << 4) | (FMT << 7) | (FMT << 10) | ((uint32_t)(BKV >> 3) << 17) | ((uint32_t)(A_BQ >> 4) << 24);
            constexpr uint32_t IDESC_PV = (1U << 4) | (FMT << 7) | (FMT << 10) | (1U << 16) | ((uint32_t)(A_DH >> 3) << 17) | ((uint32_t)(A_BQ >> 4) << 24);
            const uint32_t q_base = smem_u32(smem), p_base = smem_u32(smem + plan::OFF_P), v_base = smem_u32(smem + plan::OFF_V);
            auto issue_s = [&](int t) -> bool {
                const int ks = t & 1, b = t & 1;
                if (!mbar_wait(bar(K_FULL + ks), (t >> 1) & 1)) {
                    atomicExch(err_flag, 303);
                    return false;
                }
                if (t >= 2 && !mbar_wait(bar(BUF_FREE + b), ((t - 2) >> 1) & 1)) {   // O_part[t-2] has been read back
                    atomicExch(err_flag, 304);
                    return false;
                }
                tcgen05_fence_after();
                const uint32_t k_base = smem_u32(smem + plan::OFF_K + ks * plan::KV_BYTES);
#pragma unroll
                for (int kk = 0; kk < A_DH / UMMA_K; ++kk) {
                    tcgen05_mma_f16(tmem_base + b * BKV, make_smem_desc(q_base + kk * 32, 16, 1024), make_smem_desc(k_base + kk * 32, 16, 1024),
                                    IDESC_S, kk != 0 ? 1U : 0U);
                }
                tcgen05_commit(bar(S_FULL + b));
                tcgen05_commit(bar(K_EMPTY + ks));
                return true;
            };
            bool ok = mbar_wait(bar(Q_FULL), 0);
            if (!ok) atomicExch(err_flag, 305);
            ok = ok && issue_s(0);
            for (int t = 0; t < n_tiles && ok; ++t) {
                const int b = t & 1;
                if (t + 1 < n_tiles) {
                    ok = issue_s(t + 1);
                    if (!ok) break;
                }
                if (!mbar_wait(bar(P_FULL), t & 1) || !mbar_wait(bar(V_FULL), t & 1)) {
                    atomicExch(err_flag, 306);
                    break;
                }
                tcgen05_fence_after();
#pragma unroll
                for (int kk = 0; kk < BKV / UMMA_K; ++kk) {
                    // A = P, K-major, blocks of 64 keys 16 KB apart; B = V stored [key][dh]: MN-major, 16 keys = 2048 B
                    tcgen05_mma_f16(tmem_base + b * BKV, make_smem_desc(p_base + (kk >> 2) * (A_BQ * 128) + (kk & 3) * 32, 16, 1024),
                                    make_smem_desc(v_base + kk * 2048, BKV * 128, 1024), IDESC_PV, kk != 0 ? 1U : 0U);
                }
                tcgen05_commit(bar(O_FULL + b));
                tcgen05_commit(bar(V_EMPTY));
                tcgen05_commit(bar(P_EMPTY));
            }
        }
    } else {
        // ---------------- softmax: one thread per query row ----------------
        const int quad = warp & 3, r = quad * 32 + lane, qi = q0 + r;
        const bool valid = qi < n_valid;
        int lo_key = 0x7fffffff;
        if (valid) {
            lo_key = seg_start_of(cu_s, p.batch, qi);
            if (p.window > 0) lo_key = max(lo_key, qi - p.window + 1);
        }
        const float sl2 = p.scale * LOG2E_F;
        float m = -INFINITY, l = 0.0f, alpha_pending = 1.0f;
        float o[A_DH];
#pragma unroll
        for (int i = 0; i < A_DH; ++i) o[i] = 0.0f;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
        unsigned char *p_row = smem + plan::OFF_P + r * 128;
        bool ok = true;
        auto accumulate_o = [&](int t_prev) -> bool {
            const int b = t_prev & 1;
            if (!mbar_wait(bar(O_FULL + b), (t_prev >> 1) & 1)) {
                if (lane == 0) atomicExch(err_flag, 307);
                return false;
            }
            tcgen05_fence_after();
            uint32_t v0[32], v1[32];
            tmem_ld_32x32b_x32_nowait(lane_base + b * BKV, v0);
            tmem_ld_32x32b_x32_nowait(lane_base + b * BKV + 32, v1);
            tmem_ld_wait();
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar(BUF_FREE + b)) : "memory");
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                o[i] = o[i] * alpha_pending + __uint_as_float(v0[i]);
                o[32 + i] = o[32 + i] * alpha_pending + __uint_as_float(v1[i]);
            }
            return true;
        };
        for (int t = 0; t < n_tiles && ok; ++t) {
            const int b = t & 1, key0 = kv_begin + t * BKV;
            if (!mbar_wait(bar(S_FULL + b), (t >> 1) & 1)) {
                if (lane == 0) atomicExch(err_flag, 308);
                ok = false;
                break;
            }
            tcgen05_fence_after();
            // allowed local columns [c_lo, c_hi]
            const int c_lo = valid ? max(0, lo_key - key0) : BKV, c_hi = valid ? min(BKV - 1, qi - key0) : -1;
            float tmax = -INFINITY;
#pragma unroll 1
            for (int c = 0; c < BKV / 32; ++c) {
                const bool mine = c_lo <= c * 32 + 31 && c_hi >= c * 32;
                if (!__any_sync(0xffffffffU, mine)) continue;
                uint32_t v[32];
                tmem_ld_32x32b_x32(lane_base + b * BKV + c * 32, v);
                if (__all_sync(0xffffffffU, c_lo <= c * 32 && c_hi >= c * 32 + 31)) {
                    // every row of the warp allows the whole chunk: no per-element mask
#pragma unroll
                    for (int i = 0; i < 32; i += 2) tmax = fmaxf(tmax, fmaxf(__uint_as_float(v[i]), __uint_as_float(v[i + 1])));
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int col = c * 32 + i;
                        const float s = __uint_as_float(v[i]);
                        tmax = (col >= c_lo && col <= c_hi) ? fmaxf(tmax, s) : tmax;
                    }
                }
            }
            if (t >= 1) {
                ok = accumulate_o(t - 1);
                if (!ok) break;
            }
            const float m_new = fmaxf(m, tmax * sl2);
            const float alpha = m == -INFINITY ? (m_new == -INFINITY ? 1.0f : 0.0f) : ex2_approx(m - m_new);
            const float m_use = m_new == -INFINITY ? 0.0f : m_new;
            if (!mbar_wait(bar(P_EMPTY), (t & 1) ^ 1)) {       // P V of the previous tile has read the P tile
                if (lane == 0) atomicExch(err_flag, 309);
                ok = false;
                break;
            }
            float rsum = 0.0f;
#pragma unroll 1
            for (int c = 0; c < BKV / 32; ++c) {
                const bool mine = c_lo <= c * 32 + 31 && c_hi >= c * 32;
                uint32_t packed[16];
                if (__any_sync(0xffffffffU, mine)) {
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(lane_base + b * BKV + c * 32, v);
                    if (__all_sync(0xffffffffU, c_lo <= c * 32 && c_hi >= c * 32 + 31)) {
#pragma unroll
                        for (int i = 0; i < 32; i += 2) {
                            const float p0 = ex2_approx(fmaf(__uint_as_float(v[i]), sl2, -m_use));
                            const float p1 = ex2_approx(fmaf(__uint_as_float(v[i + 1]), sl2, -m_use));
                            rsum += p0 + p1;
                            packed[i >> 1] = half_pack<T>::pack(p0, p1);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; i += 2) {
                            const int col = c * 32 + i;
                            const float p0 = (col >= c_lo && col <= c_hi) ? ex2_approx(fmaf(__uint_as_float(v[i]), sl2, -m_use)) : 0.0f;
                            const float p1 = (col + 1 >= c_lo && col + 1 <= c_hi) ? ex2_approx(fmaf(__uint_as_float(v[i + 1]), sl2, -m_use)) : 0.0f;
                            rsum += p0 + p1;
                            packed[i >> 1] = half_pack<T>::pack(p0, p1);
                        }
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) packed[i] = 0U;
                }
                // columns c*32 .. c*32+31 = 64 bytes = chunks (c & 1) * 4 .. +3 of 64-key block c >> 1
                unsigned char *blk = p_row + (c >> 1) * (A_BQ * 128);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int chunk = (c & 1) * 4 + j;
                    *reinterpret_cast<uint4 *>(blk + ((chunk ^ (r & 7)) << 4)) = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
                }
            }
            l = l * alpha + rsum;
            m = m_new;
            alpha_pending = alpha;
            tcgen05_fence_before();
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar(P_FULL)) : "memory");
        }
        if (ok && n_tiles > 0) {
            ok = accumulate_o(n_tiles - 1);
        }
        // ---- normalise, stage through shared memory (the Q tile is no longer read), TMA store ----
        const float inv = (ok && l > 0.0f) ? 1.0f / l : 0.0f;
        unsigned char *o_row = smem + r * 128;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            uint4 w;
            w.x = half_pack<T>::pack(o[8 * j] * inv, o[8 * j + 1] * inv);
            w.y = half_pack<T>::pack(o[8 * j + 2] * inv, o[8 * j + 3] * inv);
            w.z = half_pack<T>::pack(o[8 * j + 4] * inv, o[8 * j + 5] * inv);
            w.w = half_pack<T>::pack(o[8 * j + 6] * inv, o[8 * j + 7] * inv);
            *reinterpret_cast<uint4 *>(o_row + ((j ^ (r & 7)) << 4)) = w;
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
            if (q0 + quad * 32 < p.n_tokens) {
                tma_store_2d(&tma_o, h * A_DH, q0 + quad * 32, smem_u32(smem + quad * 32 * 128));
            }
            bulk_commit_group();
            bulk_wait_all();
        }
        if (stats != nullptr && valid) {
            float *s = stats + ((size_t)qi * p.hq + h) * 3;
            s[0] = m == -INFINITY ? m : m * LN2_F;
            s[1] = l;
            s[2] = 0.0f;
        }
    }
    __syncwarp();
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)plan::TMEM_COLS) : "memory");
    }
}

template <typename T, int BKV>
gd_status launch_fwd(gd_backend *be, const gdb_flash_args *a)
{
    using plan = attn5_plan<BKV>;
    auto kern = attn5_fwd_kernel<T, BKV>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, plan::TOTAL);
        if (e != cudaSuccess) return gdb_fail(be, e, "tcgen05 attention smem attribute");
        configured = true;
    }
    CUtensorMap mq, mk, mv, mo;
    const uint64_t n = (uint64_t)a->n_tokens;
    const bool ok = make_tmap(&mq, a->dtype, a->q, n, (uint64_t)a->hq * A_DH, (uint64_t)a->hq * A_DH * 2U, 64, A_BQ) &&
                    make_tmap(&mk, a->dtype, a->k, n, (uint64_t)a->hkv * A_DH, (uint64_t)a->hkv * A_DH * 2U, 64, BKV) &&
                    make_tmap(&mv, a->dtype, a->v, n, (uint64_t)a->hkv * A_DH, (uint64_t)a->hkv * A_DH * 2U, 64, BKV) &&
                    make_tmap(&mo, a->dtype, a->out_or_dq, n, (uint64_t)a->hq * A_DH, (uint64_t)a->hq * A_DH * 2U, 64, 32);
    if (!ok) {
        return GD_ERR_UNSUPPORTED;
    }
    attn5_params p = {a->n_tokens, a->batch, a->hq, a->hkv, a->window, a->scale};
    dim3 grid((unsigned)((a->n_tokens + A_BQ - 1) / A_BQ), (unsigned)a->hq);
    kern<<<grid, 192, plan::TOTAL, be->stream>>>(mq, mk, mv, mo, a->cu, a->stats, p, be->err_flag);
    return gdb_launched(be, "attn5_forward");
}

}  // namespace

// Returns GD_ERR_UNSUPPORTED outside the fast path (the caller then runs the mma.sync kernels).
gd_status gdb_attn5_forward(gd_backend *be, const gdb_flash_args *a)
{
    const uintptr_t al = (uintptr_t)a->q | (uintptr_t)a->k | (uintptr_t)a->v | (uintptr_t)a->out_or_dq;
    if ((a->dtype != GDB_DTYPE_F16 && a->dtype != GDB_DTYPE_BF16) || a->dh != A_DH || a->causal == 0 || a->prefix != 0 || a->window < 0 ||
        (al % 16U) != 0U || a->hkv <= 0 || (a->hq % a->hkv) != 0 || a->hq > 65535 || a->batch > A_MAX_CU || a->n_tokens < A_BQ) {
        return GD_ERR_UNSUPPORTED;
    }
    return a->dtype == GDB_DTYPE_F16 ? launch_fwd<__half, 128>(be, a) : launch_fwd<__nv_bfloat16, 128>(be, a);
}
