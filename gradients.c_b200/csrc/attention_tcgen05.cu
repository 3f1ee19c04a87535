// Packed causal attention forward on the sm_100a tensor path: S = Q K^T and O = P V are
// tcgen05.mma instructions with FP32 accumulators in tensor memory, operands arrive by TMA.
//
// Fast path of gd_backend_sdpa_varlen for 16-bit storage, head_dim 64, causal (+ optional sliding
// window), no prefix. A work item is 128 consecutive rows of the PACKED token stream for one head;
// the mask is evaluated in packed coordinates exactly as in the mma.sync kernels (attention_flash.cu):
//   allowed(i, j)  <=>  seg_start(i) <= j <= i  and  (window == 0 or i - j < window)
// (src/ops/sdpa_varlen/metal_sdpa_varlen.metal:30-55, prefix 0), so a tile may span sequences.
//
// The kernel is persistent: two CTAs per SM stay resident and draw items from a launch-wide ticket counter
// (an item costs 1-5 key tiles, so a fixed deal leaves CTAs up to 1.6x out of balance), so tensor-memory
// allocation, barrier set-up and the cu_seqlens copy are paid once per CTA, and the TMA producer and
// the MMA issuer run ahead into the next item while the softmax warps finish the current one (at the
// model's sequence lengths an item has only 1-5 key tiles).
//
// Roles (320 threads): warp 0 = TMA producer (Q per item, K double-buffered, V single-buffered);
// warp 1 = MMA issuer; warps 2-9 = softmax. A query row is shared by TWO threads of the same
// tensor-memory lane quadrant (warps w and w + 4): each owns 64 of the 128 key columns of S and 32 of
// the 64 output columns, reads them with tcgen05.ld 32x32b (no shuffles) and the two exchange only
// the row maximum through shared memory. Per key tile:
//   pass 1: row max of S over the allowed columns (+ exchange)
//   (deferred) o += alpha * O_part of the previous tile, read back from tensor memory
//   pass 2: p = exp2(s * scale * log2e - m), written as 16-bit into the 128-byte-swizzled K-major
//           shared tile that the P V MMA reads as its A operand; running partial sum l
// Tensor memory: 2 buffers of 128 columns; S[g] lives in buffer g & 1 and, once consumed, the same
// buffer receives O_part[g] (64 columns), so 256 columns suffice for a CTA. The MMA issuer keeps one
// S tile ahead: S[g+1] is issued while the softmax warps work on S[g].
//
// Statistics written for the backward pass: (row max in natural-log units, sum of exp, 0).
// Every mbarrier wait is bounded and reports through gd_backend::err_flag.
#include "attention.cuh"
#include "tcgen05.cuh"

namespace {
using namespace gdb_t5;

constexpr float LOG2E_F = 1.4426950408889634f;
constexpr float LN2_F = 0.6931471805599453f;
constexpr int A_BQ = 128, A_DH = 64, A_BKV = 128;
constexpr int A_MAX_CU = 1024;
constexpr int A_THREADS = 320;

struct attn5_params {
    int n_tokens, batch, hq, hkv, window, n_items;
    float scale;
};

struct attn5_plan {
    static constexpr int Q_BYTES = A_BQ * 128;          // 128 rows x 64 x 2 B
    static constexpr int KV_BYTES = A_BKV * 128;
    static constexpr int P_BYTES = A_BQ * A_BKV * 2;    // two blocks (64 keys each) of [128 rows x 128 B]
    static constexpr int OFF_K = Q_BYTES, OFF_V = OFF_K + 2 * KV_BYTES, OFF_P = OFF_V + KV_BYTES, OFF_BAR = OFF_P + P_BYTES;
    static constexpr int TOTAL = OFF_BAR + 256 + 1024;
    static constexpr int TMEM_COLS = 2 * A_BKV;
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

// Key range of a work item: first key and number of 128-key tiles (0 when the rows lie behind the last sequence).
__device__ __forceinline__ void item_range(const int *cu_s, const attn5_params &p, int n_valid, int q0, int *kv_begin, int *n_tiles)
{
    *kv_begin = 0;
    *n_tiles = 0;
    if (q0 < n_valid) {
        int kb = seg_start_of(cu_s, p.batch, q0);
        if (p.window > 0) kb = max(kb, q0 - p.window + 1);
        const int kv_end = min(q0 + A_BQ, n_valid);   // exclusive
        *kv_begin = kb;
        *n_tiles = (kv_end - kb + A_BKV - 1) / A_BKV;
    }
}

__device__ __forceinline__ void mbar_arrive_local(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

template <typename T>
__global__ void __launch_bounds__(A_THREADS, 2)
attn5_fwd_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                 const __grid_constant__ CUtensorMap tma_v, T *__restrict__ out,
                 const int *__restrict__ cu, float *__restrict__ stats, attn5_params p, int *err_flag, unsigned *work_counter,
                 unsigned *done_counter)
{
    using plan = attn5_plan;
    extern __shared__ unsigned char smem_raw[];
    __shared__ int cu_s[A_MAX_CU + 1];
    __shared__ float xch[2][2][A_BQ];   // [tile parity][column half][row]: row maxima of the two column halves
    __shared__ float xsum[2][2][A_BQ];  // [item parity][column half][row]: partial sums of exp, exchanged once per item
    __shared__ int sched_item[4];       // work items handed out by the producer thread (-1: no more work)
    unsigned char *smem = (unsigned char *)(((uintptr_t)smem_raw + 1023U) & ~(uintptr_t)1023U);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + plan::OFF_BAR);
    enum { Q_FULL = 0, Q_EMPTY = 1, K_FULL = 2, K_EMPTY = 4, V_FULL = 6, V_EMPTY = 7, S_FULL = 8, P_FULL = 10, P_EMPTY = 11, O_FULL = 12, BUF_FREE = 14,
           SCHED_FULL = 16, SCHED_EMPTY = 20, PAIR = 24, N_BARS = 28 };
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + N_BARS);
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [&](int i) { return bar0 + 8U * (uint32_t)i; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int group = p.hq / p.hkv;

    if (threadIdx.x == 0) {
        for (int i = 0; i < N_BARS; ++i) {
            const bool eight = i == P_FULL || i == BUF_FREE || i == BUF_FREE + 1;
            // schedule slots are released by the MMA thread and the 8 softmax warps; pair barriers by 2 warps
            const uint32_t count = eight ? 8U : (i >= SCHED_EMPTY && i < SCHED_EMPTY + 4 ? 9U : (i >= PAIR ? 2U : 1U));
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
    // barrier set-up and tensor-memory allocation may overlap the preceding kernel; global memory is read from here on
    gdb_pdl_sync();
    for (int i = threadIdx.x; i <= p.batch; i += blockDim.x) cu_s[i] = cu[i];
    __syncthreads();
    const int n_valid = min(cu_s[p.batch], p.n_tokens);

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t g = 0, iq = 0, si = 0;   // running key-tile, item-with-tiles and schedule counters
            bool ok = true;
            // Draws a ticket from the launch-wide counter and publishes the item to the other roles of this CTA.
            // Tickets count down the item list: the query tiles past the last token (no key tiles) come first, and
            // within a sequence the later query tiles (more key tiles) go before the earlier ones.
            auto draw = [&]() -> int {
                const uint32_t slot = si & 3U;
                if (!mbar_wait(bar(SCHED_EMPTY + slot), ((si >> 2) & 1U) ^ 1U)) {
                    atomicExch(err_flag, 310);
                    ok = false;
                    return -1;
                }
                const int ticket = (int)atomicAdd(work_counter, 1U);
                const int it = ticket < p.n_items ? p.n_items - 1 - ticket : -1;
                sched_item[slot] = it;
                mbar_arrive_local(bar(SCHED_FULL + slot));
                ++si;
                return it;
            };
            // The schedule runs one item ahead of the loads: the MMA thread looks up the next item right after the
            // last S of the current one, while this thread may still wait for a V slot that only a later P V frees.
            int item = draw(), next = -1;
            for (; ok && item >= 0; item = next) {
                next = draw();
                const int q0 = (item / p.hq) * A_BQ, h = item % p.hq, hk = h / group;
                int kv_begin, n_tiles;
                item_range(cu_s, p, n_valid, q0, &kv_begin, &n_tiles);
                if (n_tiles == 0) continue;
                if (!mbar_wait(bar(Q_EMPTY), (iq & 1U) ^ 1U)) {
                    atomicExch(err_flag, 300);
                    break;
                }
                mbar_expect_tx(bar(Q_FULL), plan::Q_BYTES);
                tma_load_2d(smem_u32(smem), &tma_q, h * A_DH, q0, bar(Q_FULL));
                ++iq;
                for (int t = 0; t < n_tiles; ++t, ++g) {
                    const int key0 = kv_begin + t * A_BKV, ks = g & 1U;
                    if (!mbar_wait(bar(K_EMPTY + ks), ((g >> 1) & 1U) ^ 1U)) {
                        atomicExch(err_flag, 301);
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(bar(K_FULL + ks), plan::KV_BYTES);
                    tma_load_2d(smem_u32(smem + plan::OFF_K + ks * plan::KV_BYTES), &tma_k, hk * A_DH, key0, bar(K_FULL + ks));
                    if (!mbar_wait(bar(V_EMPTY), (g & 1U) ^ 1U)) {
                        atomicExch(err_flag, 302);
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(bar(V_FULL), plan::KV_BYTES);
                    tma_load_2d(smem_u32(smem + plan::OFF_V), &tma_v, hk * A_DH, key0, bar(V_FULL));
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t FMT = std::is_same<T, __nv_bfloat16>::value ? 1U : 0U;
            constexpr uint32_t IDESC_S = (1U << 4) | (FMT << 7) | (FMT << 10) | ((uint32_t)(A_BKV >> 3) << 17) | ((uint32_t)(A_BQ >> 4) << 24);
            constexpr uint32_t IDESC_PV = (1U << 4) | (FMT << 7) | (FMT << 10) | (1U << 16) | ((uint32_t)(A_DH >> 3) << 17) | ((uint32_t)(A_BQ >> 4) << 24);
            const uint32_t q_base = smem_u32(smem), p_base = smem_u32(smem + plan::OFF_P), v_base = smem_u32(smem + plan::OFF_V);
            // Walks the same (item, tile) sequence twice: `s_*` is the cursor of the S issue (one tile ahead),
            // `pv_g` the cursor of the P V issue.
            int s_item = -1, s_t = 0, s_tiles = 0;
            uint32_t s_g = 0, s_iq = 0, s_si = 0;
            bool ok = true;
            auto s_seek = [&]() {   // position the S cursor on the next scheduled item that has tiles
                for (;;) {
                    const uint32_t slot = s_si & 3U;
                    if (!mbar_wait(bar(SCHED_FULL + slot), (s_si >> 2) & 1U)) {
                        atomicExch(err_flag, 311);
                        s_item = -1;
                    } else {
                        s_item = *reinterpret_cast<volatile int *>(&sched_item[slot]);
                        mbar_arrive_local(bar(SCHED_EMPTY + slot));
                        ++s_si;
                    }
                    s_tiles = 0;
                    if (s_item < 0) return;
                    int kb;
                    item_range(cu_s, p, n_valid, (s_item / p.hq) * A_BQ, &kb, &s_tiles);
                    if (s_tiles > 0) return;
                }
            };
            auto issue_s = [&]() -> bool {   // S[s_g] = Q K^T for tile s_t of item s_item
                const uint32_t ks = s_g & 1U, b = s_g & 1U;
                if (s_t == 0 && !mbar_wait(bar(Q_FULL), s_iq & 1U)) {
                    atomicExch(err_flag, 305);
                    return false;
                }
                if (!mbar_wait(bar(K_FULL + ks), (s_g >> 1) & 1U)) {
                    atomicExch(err_flag, 303);
                    return false;
                }
                if (s_g >= 2U && !mbar_wait(bar(BUF_FREE + b), ((s_g - 2U) >> 1) & 1U)) {   // O_part[s_g - 2] has been read back
                    atomicExch(err_flag, 304);
                    return false;
                }
                tcgen05_fence_after();
                const uint32_t k_base = smem_u32(smem + plan::OFF_K + ks * plan::KV_BYTES);
#pragma unroll
                for (int kk = 0; kk < A_DH / UMMA_K; ++kk) {
                    tcgen05_mma_f16(tmem_base + b * A_BKV, make_smem_desc(q_base + kk * 32, 16, 1024), make_smem_desc(k_base + kk * 32, 16, 1024),
                                    IDESC_S, kk != 0 ? 1U : 0U);
                }
                tcgen05_commit(bar(S_FULL + b));
                tcgen05_commit(bar(K_EMPTY + ks));
                ++s_g;
                if (++s_t == s_tiles) {   // last S of the item: the Q tile may be replaced
                    tcgen05_commit(bar(Q_EMPTY));
                    ++s_iq;
                    s_t = 0;
                    s_seek();
                }
                return true;
            };
            s_seek();
            uint32_t pv_g = 0;
            if (s_tiles > 0) ok = issue_s();
            while (ok && pv_g < s_g) {
                // The next S is issued ahead of the pending P V only inside an item. The first S of the NEXT
                // item waits for that item's Q tile, and must not hold back the last P V of this one.
                const bool s_first = s_tiles > 0 && s_t != 0;
                if (s_first) {
                    ok = issue_s();
                    if (!ok) break;
                }
                const uint32_t b = pv_g & 1U;
                if (!mbar_wait(bar(P_FULL), pv_g & 1U) || !mbar_wait(bar(V_FULL), pv_g & 1U)) {
                    atomicExch(err_flag, 306);
                    break;
                }
                tcgen05_fence_after();
#pragma unroll
                for (int kk = 0; kk < A_BKV / UMMA_K; ++kk) {
                    // A = P, K-major, blocks of 64 keys 16 KB apart; B = V stored [key][dh]: MN-major, 16 keys = 2048 B
                    tcgen05_mma_f16(tmem_base + b * A_BKV, make_smem_desc(p_base + (kk >> 2) * (A_BQ * 128) + (kk & 3) * 32, 16, 1024),
                                    make_smem_desc(v_base + kk * 2048, A_BKV * 128, 1024), IDESC_PV, kk != 0 ? 1U : 0U);
                }
                tcgen05_commit(bar(O_FULL + b));
                tcgen05_commit(bar(V_EMPTY));
                tcgen05_commit(bar(P_EMPTY));
                ++pv_g;
                if (!s_first && s_tiles > 0) {
                    ok = issue_s();
                }
            }
        }
    } else {
        // ---------------- softmax: two threads per query row ----------------
        const int quad = warp & 3, half = (warp - 2) >> 2;          // half 0: key columns 0..63, output columns 0..31
        const int r = quad * 32 + lane;
        const float sl2 = p.scale * LOG2E_F;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
        unsigned char *p_row = smem + plan::OFF_P + half * (A_BQ * 128) + r * 128;   // this thread's 64 keys = one 128-byte row of block `half`
        uint32_t g = 0, n_item = 0;
        // A wait that gives up makes the warp "dead": it records the error, stops waiting and reading
        // tensor memory, but keeps walking the loops so that its partner warp never blocks on a named barrier.
        bool dead = false;
        auto wait_or_die = [&](int which, uint32_t parity, int code) {
            if (!dead && !mbar_wait(bar(which), parity)) {
                dead = true;
                if (lane == 0) atomicExch(err_flag, code);
            }
        };
        // bounded rendezvous of the two warps of a lane quadrant (mbarrier with two arrivals per phase)
        uint32_t pair_phase = 0;
        auto pair_sync = [&]() {
            __syncwarp();
            if (lane == 0) mbar_arrive_local(bar(PAIR + quad));
            wait_or_die(PAIR + quad, pair_phase & 1U, 312);
            ++pair_phase;
        };
        for (uint32_t si = 0;; ++si) {
            // next scheduled item; a dead warp stops consuming (its partner then gives up at the next rendezvous)
            const uint32_t slot = si & 3U;
            wait_or_die(SCHED_FULL + slot, (si >> 2) & 1U, 313);
            if (dead) break;
            const int item = *reinterpret_cast<volatile int *>(&sched_item[slot]);
            __syncwarp();
            if (lane == 0) mbar_arrive_local(bar(SCHED_EMPTY + slot));
            if (item < 0) break;
            const int q0 = (item / p.hq) * A_BQ, h = item % p.hq, qi = q0 + r;
            int kv_begin, n_tiles;
            item_range(cu_s, p, n_valid, q0, &kv_begin, &n_tiles);
            const bool valid = qi < n_valid;
            int lo_key = 0x7fffffff;
            if (valid) {
                lo_key = seg_start_of(cu_s, p.batch, qi);
                if (p.window > 0) lo_key = max(lo_key, qi - p.window + 1);
            }
            float m = -INFINITY, l = 0.0f, alpha_pending = 1.0f;
            float o[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = 0.0f;
            auto accumulate_o = [&](uint32_t g_prev) {
                const uint32_t b = g_prev & 1U;
                wait_or_die(O_FULL + b, (g_prev >> 1) & 1U, 307);
                if (dead) return;
                tcgen05_fence_after();
                uint32_t v[32];
                tmem_ld_32x32b_x32(lane_base + b * A_BKV + half * 32, v);
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_local(bar(BUF_FREE + b));
#pragma unroll
                for (int i = 0; i < 32; ++i) o[i] = o[i] * alpha_pending + __uint_as_float(v[i]);
            };
            for (int t = 0; t < n_tiles; ++t, ++g) {
                const uint32_t b = g & 1U;
                const int key0 = kv_begin + t * A_BKV + half * 64;   // first key of this thread's 64 columns
                wait_or_die(S_FULL + b, (g >> 1) & 1U, 308);
                tcgen05_fence_after();
                // allowed local columns [c_lo, c_hi] of this thread's half
                const int c_lo = valid ? max(0, lo_key - key0) : 64, c_hi = valid ? min(63, qi - key0) : -1;
                const uint32_t s_addr = lane_base + b * A_BKV + half * 64;
                const bool any0 = !dead && __any_sync(0xffffffffU, c_lo <= 31 && c_hi >= 0), any1 = !dead && __any_sync(0xffffffffU, c_lo <= 63 && c_hi >= 32);
                const bool all0 = __all_sync(0xffffffffU, c_lo <= 0 && c_hi >= 31), all1 = __all_sync(0xffffffffU, c_lo <= 32 && c_hi >= 63);
                float tmax = -INFINITY;
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    if (!(c == 0 ? any0 : any1)) continue;
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(s_addr + c * 32, v);
                    if (c == 0 ? all0 : all1) {
#pragma unroll
                        for (int i = 0; i < 32; i += 2) tmax = fmaxf(tmax, fmaxf(__uint_as_float(v[i]), __uint_as_float(v[i + 1])));
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) tmax = (c * 32 + i >= c_lo && c * 32 + i <= c_hi) ? fmaxf(tmax, __uint_as_float(v[i])) : tmax;
                    }
                }
                // exchange the row maximum with the thread that owns the other 64 columns
                xch[g & 1U][half][r] = tmax;
                pair_sync();
                tmax = fmaxf(tmax, xch[g & 1U][half ^ 1][r]);
                if (t >= 1) accumulate_o(g - 1U);
                const float m_new = fmaxf(m, tmax * sl2);
                const float alpha = m == -INFINITY ? (m_new == -INFINITY ? 1.0f : 0.0f) : ex2_approx(m - m_new);
                const float m_use = m_new == -INFINITY ? 0.0f : m_new;
                wait_or_die(P_EMPTY, (g & 1U) ^ 1U, 309);       // P V of the previous tile has read the P tile
                float rsum = 0.0f;
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const bool anyc = c == 0 ? any0 : any1, allc = c == 0 ? all0 : all1;
                    uint32_t packed[16];
                    if (anyc) {
                        uint32_t v[32];
                        tmem_ld_32x32b_x32(s_addr + c * 32, v);
                        if (allc) {
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
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int chunk = c * 4 + j;
                        *reinterpret_cast<uint4 *>(p_row + ((chunk ^ (r & 7)) << 4)) = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
                    }
                }
                l = l * alpha + rsum;
                m = m_new;
                alpha_pending = alpha;
                tcgen05_fence_before();
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive_local(bar(P_FULL));
            }
            if (n_tiles > 0) accumulate_o(g - 1U);   // also implies that every MMA of this item has completed
            // ---- total row sum, normalise, store this thread's 32 output columns (two full 32-byte sectors) ----
            xsum[n_item & 1U][half][r] = l;
            pair_sync();
            const float l_tot = l + xsum[n_item & 1U][half ^ 1][r];
            ++n_item;
            const float inv = (!dead && l_tot > 0.0f) ? 1.0f / l_tot : 0.0f;
            if (qi < p.n_tokens) {
                T *dst = out + ((size_t)qi * p.hq + h) * A_DH + half * 32;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint4 w;
                    w.x = half_pack<T>::pack(o[8 * j] * inv, o[8 * j + 1] * inv);
                    w.y = half_pack<T>::pack(o[8 * j + 2] * inv, o[8 * j + 3] * inv);
                    w.z = half_pack<T>::pack(o[8 * j + 4] * inv, o[8 * j + 5] * inv);
                    w.w = half_pack<T>::pack(o[8 * j + 6] * inv, o[8 * j + 7] * inv);
                    *reinterpret_cast<uint4 *>(dst + 8 * j) = w;
                }
            }
            if (stats != nullptr && valid && half == 0) {
                float *s = stats + ((size_t)qi * p.hq + h) * 3;
                s[0] = m == -INFINITY ? m : m * LN2_F;
                s[1] = l_tot;
                s[2] = 0.0f;
            }
        }
    }
    __syncwarp();
    tcgen05_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) {
        // the CTA that leaves last puts the launch-wide counters back to zero for the next launch
        __threadfence();
        if (atomicAdd(done_counter, 1U) == gridDim.x - 1U) {
            *work_counter = 0U;
            *done_counter = 0U;
        }
    }
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)plan::TMEM_COLS) : "memory");
    }
}

template <typename T>
gd_status launch_fwd(gd_backend *be, const gdb_flash_args *a)
{
    using plan = attn5_plan;
    auto kern = attn5_fwd_kernel<T>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, plan::TOTAL);
        if (e != cudaSuccess) return gdb_fail(be, e, "tcgen05 attention smem attribute");
        configured = true;
    }
    // Two CTAs fit an SM by construction (2 x 256 tensor-memory columns, 2 x 106 KB shared memory, 2 x 30720
    // registers). Nothing waits across CTAs, so if fewer were co-resident the rest would simply run later.
    const int resident = 2 * (be->sm_count - be->sm_reserve);
    CUtensorMap mq, mk, mv;
    const uint64_t n = (uint64_t)a->n_tokens;
    const bool ok = make_tmap(&mq, a->dtype, a->q, n, (uint64_t)a->hq * A_DH, (uint64_t)a->hq * A_DH * 2U, 64, A_BQ) &&
                    make_tmap(&mk, a->dtype, a->k, n, (uint64_t)a->hkv * A_DH, (uint64_t)a->hkv * A_DH * 2U, 64, A_BKV) &&
                    make_tmap(&mv, a->dtype, a->v, n, (uint64_t)a->hkv * A_DH, (uint64_t)a->hkv * A_DH * 2U, 64, A_BKV);
    if (!ok) {
        return GD_ERR_UNSUPPORTED;
    }
    attn5_params p = {a->n_tokens, a->batch, a->hq, a->hkv, a->window, ((a->n_tokens + A_BQ - 1) / A_BQ) * a->hq, a->scale};
    const unsigned grid = (unsigned)(p.n_items < resident ? p.n_items : resident);
    gdb_launch(kern, grid, A_THREADS, plan::TOTAL, be->stream, mq, mk, mv, (T *)a->out_or_dq, a->cu, a->stats, p, be->err_flag,
               gdb_tickets(be) + (GDB_TICKET_WORDS - 2), gdb_tickets(be) + (GDB_TICKET_WORDS - 3));
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
    return a->dtype == GDB_DTYPE_F16 ? launch_fwd<__half>(be, a) : launch_fwd<__nv_bfloat16>(be, a);
}
