// Packed causal attention backward on the sm_100a tensor path (key-stationary): for a tile of 128 keys of one
// KV head the kernel walks the query tiles that may attend to it and forms, with tcgen05.mma and FP32 accumulators
// in tensor memory,
//     S  = Q K^T          dP = dO V^T                         (128 queries x 128 keys each)
//     P  = exp(S scale - m) / l,   dS = P o (dP - D) scale    (softmax warps, from tcgen05.ld; m, l, D = saved statistics)
//     dV += P^T dO        dK += dS^T Q                        (128 keys x 64, accumulated over the query tiles)
//     dQ_tile = dS K                                          (128 queries x 64, added to an FP32 accumulator in global memory)
// (reference semantics: src/ops/sdpa_varlen/metal_sdpa_varlen.metal:30-55 for the mask, :1138-1909 for the backward;
// CPU restatement tests/test_sdpa_varlen.c:232-371). Fast path: 16-bit storage, head_dim 64, causal (+ window), prefix 0,
// statistics (max, sum, D) complete on entry, dq32 zeroed. The mask is evaluated in packed coordinates:
//     allowed(i, j)  <=>  seg_start(i) <= j <= i  and  (window == 0 or i - j < window).
//
// One persistent CTA per SM, 448 threads:
//   warp 0      TMA producer: K / V of an item (two stages), Q / dO of a query tile (two stages)
//   warp 1      MMA issuer; S / dP run one query tile ahead of the dV / dK / dQ products of the previous tile
//   warps 2-9   softmax: one thread per query row and 64-key half; P and dS go to shared memory as 16-bit tiles in the
//               128-byte-swizzled layout that serves both as K-major A operand (dQ = dS K) and as MN-major A operand
//               (dV = P^T dO, dK = dS^T Q) without a transpose
//   warps 10-13 drain: dQ tiles out of tensor memory into the global FP32 accumulator (red.add), and at the end of an
//               item dK / dV out of tensor memory, rounded, to global memory
// Tensor memory (512 columns): S 128, dP 128, dK 64, dV 64, dQ 2 x 64.
// Shared memory: K, V 2 x 32 KB; Q, dO 2 x 32 KB; P, dS 64 KB.
// Every mbarrier wait is bounded and reports through gd_backend::err_flag; a role that gives up stops issuing work and
// the others run into their own limits, so the kernel always returns.
#include "attention.cuh"
#include "tcgen05.cuh"

namespace {
using namespace gdb_t5;

constexpr float B_LOG2E = 1.4426950408889634f;
constexpr int B_T = 128, B_DH = 64;       // tile edge (queries and keys), head dim
constexpr int B_MAX_CU = 1024;
constexpr int B_THREADS = 448;

struct attn5b_params {
    int n_tokens, batch, hq, hkv, window, n_items;
    float scale;
};

struct attn5b_plan {
    static constexpr int TILE = B_T * 128;                 // 128 rows x 64 x 2 B = 16 KB
    static constexpr int OFF_KV = 0;                       // [2 stages][K, V]
    static constexpr int OFF_QG = OFF_KV + 4 * TILE;       // [2 stages][Q, dO]
    static constexpr int OFF_P = OFF_QG + 4 * TILE;        // two blocks (64 keys each) of [128 rows x 128 B]
    static constexpr int OFF_DS = OFF_P + 2 * TILE;
    static constexpr int OFF_BAR = OFF_DS + 2 * TILE;
    static constexpr int TOTAL = OFF_BAR + 256 + 1024;
    static constexpr int TMEM_COLS = 512;
    static constexpr uint32_t COL_S = 0, COL_DP = 128, COL_DK = 256, COL_DV = 320, COL_DQ = 384;
};

__device__ __forceinline__ float b_ex2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ void b_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void b_red_add_v4(float *addr, float a, float b, float c, float d)
{
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// index of the sequence that holds packed row `row` (row < cu_s[batch])
__device__ __forceinline__ int b_seg_of(const int *cu_s, int batch, int row)
{
    int lo = 0, hi = batch;
    while (lo + 1 < hi) {
        const int mid = (lo + hi) >> 1;
        if (cu_s[mid] <= row) lo = mid; else hi = mid;
    }
    return lo;
}

// number of query tiles (starting with the key tile's own) that hold a query allowed to see a key of tile k0
__device__ __forceinline__ int b_item_qtiles(const int *cu_s, const attn5b_params &p, int n_valid, int k0)
{
    if (k0 >= n_valid) return 0;
    const int last_key = min(k0 + B_T, n_valid) - 1;
    int q_hi = cu_s[b_seg_of(cu_s, p.batch, last_key) + 1];   // exclusive
    if (p.window > 0) q_hi = min(q_hi, last_key + p.window);
    q_hi = min(q_hi, n_valid);
    return (q_hi - 1) / B_T - k0 / B_T + 1;
}

// The steps of a CTA in order: items blockIdx.x, + gridDim.x, ...; per item the query heads of the KV head's group, per
// head the query tiles. Every role walks its own copy.
struct b_cursor {
    int item, step, n_steps, n_qt, k0, hk;
    __device__ __forceinline__ void seek(const int *cu_s, const attn5b_params &p, int n_valid, int stride)
    {
        // advance `item` (already pointing at a candidate) to the next item that has steps
        for (; item < p.n_items; item += stride) {
            k0 = (item / p.hkv) * B_T;
            hk = item % p.hkv;
            n_qt = b_item_qtiles(cu_s, p, n_valid, k0);
            if (n_qt > 0) {
                n_steps = n_qt * (p.hq / p.hkv);
                step = 0;
                return;
            }
        }
        n_steps = 0;
    }
    __device__ __forceinline__ bool done(const attn5b_params &p) const { return item >= p.n_items; }
    __device__ __forceinline__ int q0() const { return k0 + (step % n_qt) * B_T; }
    __device__ __forceinline__ int head(const attn5b_params &p) const { return hk * (p.hq / p.hkv) + step / n_qt; }
    __device__ __forceinline__ bool first() const { return step == 0; }
    __device__ __forceinline__ bool last() const { return step == n_steps - 1; }
    __device__ __forceinline__ void next(const int *cu_s, const attn5b_params &p, int n_valid, int stride)
    {
        if (++step == n_steps) {
            item += stride;
            seek(cu_s, p, n_valid, stride);
        }
    }
};

template <typename T>
__global__ void __launch_bounds__(B_THREADS, 1)
attn5_bwd_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                 const __grid_constant__ CUtensorMap tma_v, const __grid_constant__ CUtensorMap tma_go,
                 const int *__restrict__ cu, const float *__restrict__ stats, T *__restrict__ dk, T *__restrict__ dv,
                 float *__restrict__ dq32, attn5b_params p, int *err_flag)
{
    using plan = attn5b_plan;
    extern __shared__ unsigned char smem_raw[];
    __shared__ int cu_s[B_MAX_CU + 1];
    unsigned char *smem = (unsigned char *)(((uintptr_t)smem_raw + 1023U) & ~(uintptr_t)1023U);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + plan::OFF_BAR);
    enum { KV_FULL = 0, KV_EMPTY = 2, QG_FULL = 4, QG_EMPTY = 6, S_FULL = 8, S_FREE = 9, P_FULL = 10, P_EMPTY = 11,
           DQ_FULL = 12, DQ_FREE = 14, ACC_FULL = 16, ACC_FREE = 17, N_BARS = 18 };
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + N_BARS);
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [&](int i) { return bar0 + 8U * (uint32_t)i; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int stride = (int)gridDim.x;

    if (threadIdx.x == 0) {
        for (int i = 0; i < N_BARS; ++i) {
            uint32_t count = 1U;
            if (i == S_FREE || i == P_FULL) count = 8U;                               // the softmax warps
            if (i == DQ_FREE || i == DQ_FREE + 1 || i == ACC_FREE) count = 4U;        // the drain warps
            mbar_init(bar(i), count);
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
    gdb_pdl_sync();
    for (int i = threadIdx.x; i <= p.batch; i += blockDim.x) cu_s[i] = cu[i];
    __syncthreads();
    const int n_valid = min(cu_s[p.batch], p.n_tokens);

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            b_cursor c;
            c.item = blockIdx.x;
            c.seek(cu_s, p, n_valid, stride);
            uint32_t g = 0, n_item = 0;
            while (!c.done(p)) {
                if (c.first()) {
                    const uint32_t s = n_item & 1U;
                    if (!mbar_wait(bar(KV_EMPTY + s), ((n_item >> 1) & 1U) ^ 1U)) {
                        atomicExch(err_flag, 320);
                        break;
                    }
                    mbar_expect_tx(bar(KV_FULL + s), 2 * plan::TILE);
                    tma_load_2d(smem_u32(smem + plan::OFF_KV + (2 * s) * plan::TILE), &tma_k, c.hk * B_DH, c.k0, bar(KV_FULL + s));
                    tma_load_2d(smem_u32(smem + plan::OFF_KV + (2 * s + 1) * plan::TILE), &tma_v, c.hk * B_DH, c.k0, bar(KV_FULL + s));
                    ++n_item;
                }
                const uint32_t s = g & 1U;
                if (!mbar_wait(bar(QG_EMPTY + s), ((g >> 1) & 1U) ^ 1U)) {
                    atomicExch(err_flag, 321);
                    break;
                }
                const int h = c.head(p), q0 = c.q0();
                mbar_expect_tx(bar(QG_FULL + s), 2 * plan::TILE);
                tma_load_2d(smem_u32(smem + plan::OFF_QG + (2 * s) * plan::TILE), &tma_q, h * B_DH, q0, bar(QG_FULL + s));
                tma_load_2d(smem_u32(smem + plan::OFF_QG + (2 * s + 1) * plan::TILE), &tma_go, h * B_DH, q0, bar(QG_FULL + s));
                ++g;
                c.next(cu_s, p, n_valid, stride);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t FMT = std::is_same<T, __nv_bfloat16>::value ? 1U : 0U;
            constexpr uint32_t ID_BASE = (1U << 4) | (FMT << 7) | (FMT << 10) | ((uint32_t)(B_T >> 4) << 24);
            constexpr uint32_t IDESC_S = ID_BASE | ((uint32_t)(B_T >> 3) << 17);                              // A, B K-major, N = 128
            constexpr uint32_t IDESC_ACC = ID_BASE | (1U << 15) | (1U << 16) | ((uint32_t)(B_DH >> 3) << 17);   // A, B MN-major, N = 64
            constexpr uint32_t IDESC_DQ = ID_BASE | (1U << 16) | ((uint32_t)(B_DH >> 3) << 17);                // A K-major, B MN-major, N = 64
            const uint32_t p_base = smem_u32(smem + plan::OFF_P), ds_base = smem_u32(smem + plan::OFF_DS);
            b_cursor cs, ca;   // cs: cursor of the S / dP issue (one step ahead), ca: cursor of dV / dK / dQ
            cs.item = ca.item = blockIdx.x;
            cs.seek(cu_s, p, n_valid, stride);
            ca.seek(cu_s, p, n_valid, stride);
            uint32_t gs = 0, ga = 0, is = 0, ia = 0;   // step and item counters of the two cursors
            bool ok = true;
            auto issue_s = [&]() -> bool {
                const uint32_t kvs = is & 1U, qs = gs & 1U;
                if (cs.first() && !mbar_wait(bar(KV_FULL + kvs), (is >> 1) & 1U)) {
                    atomicExch(err_flag, 322);
                    return false;
                }
                if (!mbar_wait(bar(QG_FULL + qs), (gs >> 1) & 1U)) {
                    atomicExch(err_flag, 323);
                    return false;
                }
                if (!mbar_wait(bar(S_FREE), (gs & 1U) ^ 1U)) {       // the softmax warps have read S / dP of the previous step
                    atomicExch(err_flag, 324);
                    return false;
                }
                tcgen05_fence_after();
                const uint32_t k_base = smem_u32(smem + plan::OFF_KV + (2 * kvs) * plan::TILE), v_base = k_base + plan::TILE;
                const uint32_t q_base = smem_u32(smem + plan::OFF_QG + (2 * qs) * plan::TILE), g_base = q_base + plan::TILE;
#pragma unroll
                for (int kk = 0; kk < B_DH / UMMA_K; ++kk) {
                    tcgen05_mma_f16(tmem_base + plan::COL_S, make_smem_desc(q_base + kk * 32, 16, 1024), make_smem_desc(k_base + kk * 32, 16, 1024),
                                    IDESC_S, kk != 0 ? 1U : 0U);
                }
#pragma unroll
                for (int kk = 0; kk < B_DH / UMMA_K; ++kk) {
                    tcgen05_mma_f16(tmem_base + plan::COL_DP, make_smem_desc(g_base + kk * 32, 16, 1024), make_smem_desc(v_base + kk * 32, 16, 1024),
                                    IDESC_S, kk != 0 ? 1U : 0U);
                }
                tcgen05_commit(bar(S_FULL));
                ++gs;
                if (cs.last()) ++is;
                cs.next(cu_s, p, n_valid, stride);
                return true;
            };
            if (!cs.done(p)) ok = issue_s();
            while (ok && !ca.done(p)) {
                if (!cs.done(p)) {
                    ok = issue_s();
                    if (!ok) break;
                }
                const uint32_t kvs = ia & 1U, qs = ga & 1U, dqb = ga & 1U;
                if (!mbar_wait(bar(P_FULL), ga & 1U)) {
                    atomicExch(err_flag, 325);
                    break;
                }
                if (!mbar_wait(bar(DQ_FREE + dqb), ((ga >> 1) & 1U) ^ 1U)) {
                    atomicExch(err_flag, 326);
                    break;
                }
                if (ca.first() && !mbar_wait(bar(ACC_FREE), (ia & 1U) ^ 1U)) {   // dK / dV of the previous item have been read back
                    atomicExch(err_flag, 327);
                    break;
                }
                tcgen05_fence_after();
                const uint32_t k_base = smem_u32(smem + plan::OFF_KV + (2 * kvs) * plan::TILE);
                const uint32_t q_base = smem_u32(smem + plan::OFF_QG + (2 * qs) * plan::TILE), g_base = q_base + plan::TILE;
                const uint32_t acc = ca.first() ? 0U : 1U;
                // dV += P^T dO and dK += dS^T Q: A = the [query][key] tile read MN-major (M = keys: two 64-key blocks 16 KB apart,
                // 16 queries = 2048 B per step), B = dO / Q stored [query][dh] read MN-major
#pragma unroll
                for (int kk = 0; kk < B_T / UMMA_K; ++kk) {
                    tcgen05_mma_f16(tmem_base + plan::COL_DV, make_smem_desc(p_base + kk * 2048, plan::TILE, 1024),
                                    make_smem_desc(g_base + kk * 2048, plan::TILE, 1024), IDESC_ACC, (acc | (kk != 0 ? 1U : 0U)));
                }
#pragma unroll
                for (int kk = 0; kk < B_T / UMMA_K; ++kk) {
                    tcgen05_mma_f16(tmem_base + plan::COL_DK, make_smem_desc(ds_base + kk * 2048, plan::TILE, 1024),
                                    make_smem_desc(q_base + kk * 2048, plan::TILE, 1024), IDESC_ACC, (acc | (kk != 0 ? 1U : 0U)));
                }
                tcgen05_commit(bar(QG_EMPTY + qs));
                // dQ tile = dS K: A = dS K-major (blocks of 64 keys 16 KB apart), B = K stored [key][dh] read MN-major
#pragma unroll
                for (int kk = 0; kk < B_T / UMMA_K; ++kk) {
                    tcgen05_mma_f16(tmem_base + plan::COL_DQ + dqb * B_DH, make_smem_desc(ds_base + (kk >> 2) * plan::TILE + (kk & 3) * 32, 16, 1024),
                                    make_smem_desc(k_base + kk * 2048, plan::TILE, 1024), IDESC_DQ, kk != 0 ? 1U : 0U);
                }
                tcgen05_commit(bar(DQ_FULL + dqb));
                tcgen05_commit(bar(P_EMPTY));
                if (ca.last()) {
                    tcgen05_commit(bar(ACC_FULL));
                    tcgen05_commit(bar(KV_EMPTY + kvs));
                    ++ia;
                }
                ++ga;
                ca.next(cu_s, p, n_valid, stride);
            }
        }
    } else if (warp < 10) {
        // ---------------- softmax: one thread per query row and 64-key half ----------------
        const int quad = warp & 3, half = (warp - 2) >> 2;
        const int r = quad * 32 + lane;
        const float sl2 = p.scale * B_LOG2E;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
        unsigned char *p_row = smem + plan::OFF_P + half * plan::TILE + r * 128;
        unsigned char *ds_row = smem + plan::OFF_DS + half * plan::TILE + r * 128;
        bool dead = false;
        auto wait_or_die = [&](int which, uint32_t parity, int code) {
            if (!dead && !mbar_wait(bar(which), parity)) {
                dead = true;
                if (lane == 0) atomicExch(err_flag, code);
            }
        };
        b_cursor c;
        c.item = blockIdx.x;
        c.seek(cu_s, p, n_valid, stride);
        for (uint32_t g = 0; !c.done(p) && !dead; ++g, c.next(cu_s, p, n_valid, stride)) {
            const int q0 = c.q0(), h = c.head(p), qi = q0 + r;
            const int key0 = c.k0 + half * 64;
            const bool valid = qi < n_valid;
            float m2 = 0.0f, inv_l = 0.0f, dsum = 0.0f;
            int lo_key = 0x7fffffff;
            if (valid) {
                const float *st = stats + ((size_t)qi * p.hq + h) * 3;
                const float m = st[0], l = st[1];
                dsum = st[2];
                m2 = m == -INFINITY ? 0.0f : m * B_LOG2E;
                inv_l = l > 0.0f ? 1.0f / l : 0.0f;
                lo_key = cu_s[b_seg_of(cu_s, p.batch, qi)];
                if (p.window > 0) lo_key = max(lo_key, qi - p.window + 1);
            }
            // allowed local columns [c_lo, c_hi] of this thread's 64 keys
            const int c_lo = valid ? max(0, lo_key - key0) : 64, c_hi = valid ? min(63, qi - key0) : -1;
            wait_or_die(S_FULL, g & 1U, 328);
            tcgen05_fence_after();
            const bool any0 = !dead && __any_sync(0xffffffffU, c_lo <= 31 && c_hi >= 0), any1 = !dead && __any_sync(0xffffffffU, c_lo <= 63 && c_hi >= 32);
            const bool all0 = __all_sync(0xffffffffU, c_lo <= 0 && c_hi >= 31), all1 = __all_sync(0xffffffffU, c_lo <= 32 && c_hi >= 63);
            const float ps = inv_l, gs = inv_l * p.scale;
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
                const bool anyc = cc == 0 ? any0 : any1, allc = cc == 0 ? all0 : all1;
                uint32_t pk[16], dk_[16];
                if (anyc) {
                    uint32_t vs[32], vp[32];
                    tmem_ld_32x32b_x32_nowait(lane_base + plan::COL_S + half * 64 + cc * 32, vs);
                    tmem_ld_32x32b_x32_nowait(lane_base + plan::COL_DP + half * 64 + cc * 32, vp);
                    tmem_ld_wait();
                    if (cc == 1) {
                        tcgen05_fence_before();
                        __syncwarp();
                        if (lane == 0) b_arrive(bar(S_FREE));
                    }
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        float e0 = b_ex2(fmaf(__uint_as_float(vs[i]), sl2, -m2));
                        float e1 = b_ex2(fmaf(__uint_as_float(vs[i + 1]), sl2, -m2));
                        float d0 = e0 * gs * (__uint_as_float(vp[i]) - dsum), d1 = e1 * gs * (__uint_as_float(vp[i + 1]) - dsum);
                        if (!allc) {
                            const int col = cc * 32 + i;
                            const bool a0 = col >= c_lo && col <= c_hi, a1 = col + 1 >= c_lo && col + 1 <= c_hi;
                            e0 = a0 ? e0 : 0.0f;
                            e1 = a1 ? e1 : 0.0f;
                            d0 = a0 ? d0 : 0.0f;
                            d1 = a1 ? d1 : 0.0f;
                        }
                        pk[i >> 1] = half_pack<T>::pack(e0 * ps, e1 * ps);
                        dk_[i >> 1] = half_pack<T>::pack(d0, d1);
                    }
                } else {
                    if (cc == 1) {
                        tcgen05_fence_before();
                        __syncwarp();
                        if (lane == 0) b_arrive(bar(S_FREE));
                    }
#pragma unroll
                    for (int i = 0; i < 16; ++i) pk[i] = dk_[i] = 0U;
                }
                if (cc == 0) wait_or_die(P_EMPTY, (g & 1U) ^ 1U, 329);   // the products of the previous step have read P / dS
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int chunk = cc * 4 + j;
                    *reinterpret_cast<uint4 *>(p_row + ((chunk ^ (r & 7)) << 4)) = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
                    *reinterpret_cast<uint4 *>(ds_row + ((chunk ^ (r & 7)) << 4)) = make_uint4(dk_[4 * j], dk_[4 * j + 1], dk_[4 * j + 2], dk_[4 * j + 3]);
                }
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) b_arrive(bar(P_FULL));
        }
    } else {
        // ---------------- drain: dQ tiles per step, dK / dV per item ----------------
        const int quad = warp & 3;
        const int r = quad * 32 + lane;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
        bool dead = false;
        auto wait_or_die = [&](int which, uint32_t parity, int code) {
            if (!dead && !mbar_wait(bar(which), parity)) {
                dead = true;
                if (lane == 0) atomicExch(err_flag, code);
            }
        };
        // key tiles that no query can see (rows behind the last sequence): their dK / dV rows are zero
        for (int it = blockIdx.x; it < p.n_items; it += stride) {
            const int k0 = (it / p.hkv) * B_T, hk = it % p.hkv, row = k0 + r;
            if (k0 >= n_valid && row < p.n_tokens) {
                uint4 *a = reinterpret_cast<uint4 *>(dk + ((size_t)row * p.hkv + hk) * B_DH), *b = reinterpret_cast<uint4 *>(dv + ((size_t)row * p.hkv + hk) * B_DH);
#pragma unroll
                for (int j = 0; j < 8; ++j) a[j] = b[j] = make_uint4(0U, 0U, 0U, 0U);
            }
        }
        b_cursor c;
        c.item = blockIdx.x;
        c.seek(cu_s, p, n_valid, stride);
        uint32_t n_item = 0;
        for (uint32_t g = 0; !c.done(p) && !dead; ++g) {
            const uint32_t dqb = g & 1U;
            const int qi = c.q0() + r, h = c.head(p);
            wait_or_die(DQ_FULL + dqb, (g >> 1) & 1U, 330);
            if (dead) break;
            tcgen05_fence_after();
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
                uint32_t v[32];
                tmem_ld_32x32b_x32(lane_base + plan::COL_DQ + dqb * B_DH + cc * 32, v);
                if (cc == 1) {
                    tcgen05_fence_before();
                    __syncwarp();
                    if (lane == 0) b_arrive(bar(DQ_FREE + dqb));
                }
                if (qi < n_valid) {
                    float *dst = dq32 + ((size_t)qi * p.hq + h) * B_DH + cc * 32;
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        b_red_add_v4(dst + i, __uint_as_float(v[i]), __uint_as_float(v[i + 1]), __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
                    }
                }
            }
            if (c.last()) {
                wait_or_die(ACC_FULL, n_item & 1U, 331);
                if (dead) break;
                tcgen05_fence_after();
                const int row = c.k0 + r;
#pragma unroll
                for (int which = 0; which < 2; ++which) {
                    T *dst = (which == 0 ? dk : dv) + ((size_t)row * p.hkv + c.hk) * B_DH;
#pragma unroll
                    for (int cc = 0; cc < 2; ++cc) {
                        uint32_t v[32];
                        tmem_ld_32x32b_x32(lane_base + (which == 0 ? plan::COL_DK : plan::COL_DV) + cc * 32, v);
                        if (which == 1 && cc == 1) {
                            tcgen05_fence_before();
                            __syncwarp();
                            if (lane == 0) b_arrive(bar(ACC_FREE));
                        }
                        if (row < p.n_tokens) {
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                uint4 w;
                                w.x = half_pack<T>::pack(__uint_as_float(v[8 * j]), __uint_as_float(v[8 * j + 1]));
                                w.y = half_pack<T>::pack(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]));
                                w.z = half_pack<T>::pack(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]));
                                w.w = half_pack<T>::pack(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7]));
                                *reinterpret_cast<uint4 *>(dst + cc * 32 + 8 * j) = w;
                            }
                        }
                    }
                }
                ++n_item;
            }
            c.next(cu_s, p, n_valid, stride);
        }
    }
    __syncwarp();
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)plan::TMEM_COLS) : "memory");
    }
}

template <typename T>
gd_status launch_bwd(gd_backend *be, const gdb_flash_args *a, float *dq32)
{
    using plan = attn5b_plan;
    auto kern = attn5_bwd_kernel<T>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, plan::TOTAL);   // per device; cheap
    if (e != cudaSuccess) return gdb_fail(be, e, "tcgen05 attention backward smem attribute");
    CUtensorMap mq, mk, mv, mg;
    const uint64_t n = (uint64_t)a->n_tokens;
    const bool ok = make_tmap(&mq, a->dtype, a->q, n, (uint64_t)a->hq * B_DH, (uint64_t)a->hq * B_DH * 2U, 64, B_T) &&
                    make_tmap(&mk, a->dtype, a->k, n, (uint64_t)a->hkv * B_DH, (uint64_t)a->hkv * B_DH * 2U, 64, B_T) &&
                    make_tmap(&mv, a->dtype, a->v, n, (uint64_t)a->hkv * B_DH, (uint64_t)a->hkv * B_DH * 2U, 64, B_T) &&
                    make_tmap(&mg, a->dtype, a->grad_out, n, (uint64_t)a->hq * B_DH, (uint64_t)a->hq * B_DH * 2U, 64, B_T);
    if (!ok) {
        return GD_ERR_UNSUPPORTED;
    }
    attn5b_params p = {a->n_tokens, a->batch, a->hq, a->hkv, a->window, ((a->n_tokens + B_T - 1) / B_T) * a->hkv, a->scale};
    const int resident = be->sm_count - be->sm_reserve;
    const unsigned grid = (unsigned)(p.n_items < resident ? p.n_items : resident);
    gdb_launch(kern, grid, B_THREADS, plan::TOTAL, be->stream, mq, mk, mv, mg, a->cu, (const float *)a->stats, (T *)a->dk, (T *)a->dv, dq32, p, be->err_flag);
    return gdb_launched(be, "attn5_backward");
}

}  // namespace

// dK, dV and the FP32 dQ accumulator (zero on entry) from statistics (max, sum, D) that are complete on entry.
// Returns GD_ERR_UNSUPPORTED outside the fast path (the caller then runs the mma.sync kernel).
gd_status gdb_attn5_backward(gd_backend *be, const gdb_flash_args *a, float *dq32)
{
    const uintptr_t al = (uintptr_t)a->q | (uintptr_t)a->k | (uintptr_t)a->v | (uintptr_t)a->grad_out | (uintptr_t)a->dk | (uintptr_t)a->dv | (uintptr_t)dq32;
    if ((a->dtype != GDB_DTYPE_F16 && a->dtype != GDB_DTYPE_BF16) || a->dh != B_DH || a->causal == 0 || a->prefix != 0 || a->window < 0 ||
        (al % 16U) != 0U || a->hkv <= 0 || (a->hq % a->hkv) != 0 || a->hq > 65535 || a->batch > B_MAX_CU || a->n_tokens < B_T ||
        a->stats == NULL || dq32 == NULL) {
        return GD_ERR_UNSUPPORTED;
    }
    return a->dtype == GDB_DTYPE_F16 ? launch_bwd<__half>(be, a, dq32) : launch_bwd<__nv_bfloat16>(be, a, dq32);
}
