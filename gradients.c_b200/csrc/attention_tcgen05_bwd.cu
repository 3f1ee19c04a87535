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
// One persistent CTA per SM, 800 threads:
//   warp 0       TMA producer: K / V of an item (two stages), Q / dO of a query tile (three stages)
//   warps 1-4    MMA issuers, one thread each: S and dP (which run one query tile ahead), dV, dK, dQ. The tensor pipe needs
//                at least ~61 cycles per MMA instruction of one thread whatever its width, but takes MMAs of several threads
//                at the rate the operand reads allow (~48 cycles for a 128 x 64 x 16 product), and MMAs of one thread
//                execute in order, which the accumulation of dV and of dK relies on
//   warps 5-20   softmax: one thread per query row and 32-key quarter; P and dS go to shared memory as 16-bit tiles in
//                the 128-byte-swizzled layout that serves both as K-major A operand (dQ = dS K) and as MN-major A operand
//                (dV = P^T dO, dK = dS^T Q) without a transpose. Sixteen warps: the exponentials of a tile keep the
//                special-function unit busy for ~1000 cycles and one thread's chain (exp2 -> scale -> round) has no
//                parallelism of its own. A step's values are formed in registers before the wait for the shared tiles, so
//                that this work overlaps the products of the previous step
//   warps 21-24  drain: dQ tiles out of tensor memory into the global FP32 accumulator (red.add), and at the end of an
//                item dK / dV out of tensor memory, rounded, to global memory
// Tensor memory (512 columns): S 128, dP 128, dK 64, dV 64, dQ 2 x 64.
// Shared memory: K, V 2 x 32 KB; Q, dO 3 x 32 KB; P, dS 64 KB.
// Every mbarrier wait is bounded and reports through gd_backend::err_flag; a role that gives up stops issuing work and
// the others run into their own limits, so the kernel always returns.
#include "attention.cuh"
#include "tcgen05.cuh"

namespace {
using namespace gdb_t5;

constexpr float B_LOG2E = 1.4426950408889634f;
constexpr int B_T = 128, B_DH = 64;       // tile edge (queries and keys), head dim
constexpr int B_THREADS = 800;

struct attn5b_params {
    int n_tokens, batch, hq, hkv, window, n_items;
    float scale;
};

struct attn5b_plan {
    static constexpr int TILE = B_T * 128;                 // 128 rows x 64 x 2 B = 16 KB
    static constexpr int OFF_KV = 0;                       // [2 stages][K, V]
    static constexpr int QG_STAGES = 3;
    static constexpr int OFF_QG = OFF_KV + 4 * TILE;       // [3 stages][Q, dO]
    static constexpr int OFF_P = OFF_QG + 2 * QG_STAGES * TILE;   // two blocks (64 keys each) of [128 rows x 128 B]
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

// The steps of a CTA in order: items blockIdx.x, + gridDim.x, ...; per item the query heads of the KV head's group, per
// head the query tiles (tile_nqt[key tile] of them, from the preparation kernel). Every role walks its own copy; no
// division and no search per step, because single threads walk it too.
struct b_cursor {
    int item, n_qt, k0, hk, t, hg, group;
    __device__ __forceinline__ void seek(const int *__restrict__ tile_nqt, const attn5b_params &p, int stride)
    {
        // advance `item` (already pointing at a candidate) to the next item that has steps
        for (; item < p.n_items; item += stride) {
            const int tile = item / p.hkv;
            k0 = tile * B_T;
            hk = item - tile * p.hkv;
            n_qt = __ldg(tile_nqt + tile);
            if (n_qt > 0) break;
        }
        t = 0;
        hg = 0;
    }
    __device__ __forceinline__ bool done(const attn5b_params &p) const { return item >= p.n_items; }
    __device__ __forceinline__ int q0() const { return k0 + t * B_T; }
    __device__ __forceinline__ int head() const { return hk * group + hg; }
    __device__ __forceinline__ bool first() const { return t == 0 && hg == 0; }
    __device__ __forceinline__ bool last() const { return t == n_qt - 1 && hg == group - 1; }
    __device__ __forceinline__ void next(const int *__restrict__ tile_nqt, const attn5b_params &p, int stride)
    {
        if (++t == n_qt) {
            t = 0;
            if (++hg == group) {
                item += stride;
                seek(tile_nqt, p, stride);
            }
        }
    }
};

__device__ __forceinline__ void tmem_ld_32x32b_x16_nowait(uint32_t taddr, uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

template <typename T>
__global__ void __launch_bounds__(B_THREADS, 1)
attn5_bwd_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                 const __grid_constant__ CUtensorMap tma_v, const __grid_constant__ CUtensorMap tma_go,
                 const int *__restrict__ cu, const float *__restrict__ stats, T *__restrict__ dk, T *__restrict__ dv,
                 float *__restrict__ dq32, const int *__restrict__ meta, attn5b_params p, int *err_flag)
{
    using plan = attn5b_plan;
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = (unsigned char *)(((uintptr_t)smem_raw + 1023U) & ~(uintptr_t)1023U);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + plan::OFF_BAR);
    enum { KV_FULL = 0, KV_EMPTY = 2, QG_FULL = 4, QG_EMPTY = 7, S_FULL = 10, S_FREE = 11, P_FULL = 12, P_EMPTY = 13,
           DQ_FULL = 14, DQ_FREE = 16, ACC_FULL = 18, ACC_FREE = 19, N_BARS = 20 };
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + N_BARS);
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [&](int i) { return bar0 + 8U * (uint32_t)i; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int stride = (int)gridDim.x;

    if (threadIdx.x == 0) {
        for (int i = 0; i < N_BARS; ++i) {
            uint32_t count = 1U;
            if (i == S_FREE || i == P_FULL) count = 16U;                              // the softmax warps
            if (i == DQ_FREE || i == DQ_FREE + 1 || i == ACC_FREE) count = 4U;        // the drain warps
            if (i == KV_EMPTY || i == KV_EMPTY + 1 || i == ACC_FULL) count = 2U;      // S/dP + dQ issuers; dV + dK issuers
            if ((i >= QG_EMPTY && i < QG_EMPTY + 3) || i == P_EMPTY) count = 3U;      // S/dP, dV, dK issuers; dV, dK, dQ issuers
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
    const int *__restrict__ row_lo = meta, *__restrict__ tile_nqt = meta + p.n_tokens;
    const int n_valid = min(__ldg(cu + p.batch), p.n_tokens);

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            b_cursor c;
            c.item = blockIdx.x;
            c.group = p.hq / p.hkv;
            c.seek(tile_nqt, p, stride);
            uint32_t g = 0, n_item = 0, qs = 0, qphase = 0;   // Q / dO stage of the step and how often the ring has wrapped
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
                if (!mbar_wait(bar(QG_EMPTY + qs), (qphase & 1U) ^ 1U)) {
                    atomicExch(err_flag, 321);
                    break;
                }
                const int h = c.head(), q0 = c.q0();
                mbar_expect_tx(bar(QG_FULL + qs), 2 * plan::TILE);
                tma_load_2d(smem_u32(smem + plan::OFF_QG + (2 * qs) * plan::TILE), &tma_q, h * B_DH, q0, bar(QG_FULL + qs));
                tma_load_2d(smem_u32(smem + plan::OFF_QG + (2 * qs + 1) * plan::TILE), &tma_go, h * B_DH, q0, bar(QG_FULL + qs));
                if (++qs == plan::QG_STAGES) {
                    qs = 0;
                    ++qphase;
                }
                ++g;
                c.next(tile_nqt, p, stride);
            }
        }
    } else if (warp <= 4) {
        // ---------------- MMA issuers: warp 1 S and dP, warp 2 dV, warp 3 dK, warp 4 dQ ----------------
        if (lane == 0) {
            constexpr uint32_t FMT = std::is_same<T, __nv_bfloat16>::value ? 1U : 0U;
            constexpr uint32_t ID_BASE = (1U << 4) | (FMT << 7) | (FMT << 10) | ((uint32_t)(B_T >> 4) << 24);
            constexpr uint32_t IDESC_S = ID_BASE | ((uint32_t)(B_T >> 3) << 17);                              // A, B K-major, N = 128
            constexpr uint32_t IDESC_ACC = ID_BASE | (1U << 15) | (1U << 16) | ((uint32_t)(B_DH >> 3) << 17);   // A, B MN-major, N = 64
            constexpr uint32_t IDESC_DQ = ID_BASE | (1U << 16) | ((uint32_t)(B_DH >> 3) << 17);                // A K-major, B MN-major, N = 64
            // Shared-memory matrix descriptors: the start address sits in the low 14 bits (16-byte units), so moving to
            // another stage or stepping through a tile is a 64-bit add.
            const uint32_t kv0 = smem_u32(smem + plan::OFF_KV), qg0 = smem_u32(smem + plan::OFF_QG);
            constexpr uint64_t STEP_K = 32 >> 4, STEP_MN = 2048 >> 4, BLOCK = plan::TILE >> 4;
            b_cursor c;
            c.item = blockIdx.x;
            c.group = p.hq / p.hkv;
            c.seek(tile_nqt, p, stride);
            uint32_t g = 0, n_item = 0, qs = 0, qphase = 0;
            auto advance = [&]() {
                if (c.last()) ++n_item;
                if (++qs == plan::QG_STAGES) {
                    qs = 0;
                    ++qphase;
                }
                ++g;
                c.next(tile_nqt, p, stride);
            };
            if (warp == 1) {
                // S = Q K^T and dP = dO V^T of step g, as soon as the softmax warps have read S / dP of step g - 1
                const uint64_t k_k = make_smem_desc(kv0, 16, 1024), v_k = make_smem_desc(kv0 + plan::TILE, 16, 1024);
                const uint64_t q_k = make_smem_desc(qg0, 16, 1024), g_k = make_smem_desc(qg0 + plan::TILE, 16, 1024);
                for (; !c.done(p); advance()) {
                    const uint32_t kvs = n_item & 1U;
                    if (c.first() && !mbar_wait(bar(KV_FULL + kvs), (n_item >> 1) & 1U)) {
                        atomicExch(err_flag, 322);
                        break;
                    }
                    if (!mbar_wait(bar(QG_FULL + qs), qphase & 1U)) {
                        atomicExch(err_flag, 323);
                        break;
                    }
                    if (!mbar_wait(bar(S_FREE), (g & 1U) ^ 1U)) {
                        atomicExch(err_flag, 324);
                        break;
                    }
                    tcgen05_fence_after();
                    const uint64_t kd = k_k + kvs * (2 * BLOCK), vd = v_k + kvs * (2 * BLOCK), qd = q_k + qs * (2 * BLOCK), gd = g_k + qs * (2 * BLOCK);
#pragma unroll
                    for (int kk = 0; kk < B_DH / UMMA_K; ++kk) {
                        tcgen05_mma_f16(tmem_base + plan::COL_S, qd + kk * STEP_K, kd + kk * STEP_K, IDESC_S, kk != 0 ? 1U : 0U);
                    }
#pragma unroll
                    for (int kk = 0; kk < B_DH / UMMA_K; ++kk) {
                        tcgen05_mma_f16(tmem_base + plan::COL_DP, gd + kk * STEP_K, vd + kk * STEP_K, IDESC_S, kk != 0 ? 1U : 0U);
                    }
                    tcgen05_commit(bar(S_FULL));
                    tcgen05_commit(bar(QG_EMPTY + qs));
                    if (c.last()) tcgen05_commit(bar(KV_EMPTY + kvs));
                }
            } else if (warp == 2 || warp == 3) {
                // warp 2: dV += P^T dO; warp 3: dK += dS^T Q. A = the [query][key] tile read MN-major (M = keys: two 64-key
                // blocks 16 KB apart, 16 queries = 2048 B per MMA), B = dO / Q stored [query][dh] read MN-major
                const uint64_t a_m = make_smem_desc(smem_u32(smem + (warp == 2 ? plan::OFF_P : plan::OFF_DS)), plan::TILE, 1024);
                const uint64_t b_m = make_smem_desc(qg0 + (warp == 2 ? plan::TILE : 0), plan::TILE, 1024);
                const uint32_t d_col = tmem_base + (warp == 2 ? plan::COL_DV : plan::COL_DK);
                for (; !c.done(p); advance()) {
                    if (!mbar_wait(bar(P_FULL), g & 1U)) {
                        atomicExch(err_flag, 325);
                        break;
                    }
                    if (c.first() && !mbar_wait(bar(ACC_FREE), (n_item & 1U) ^ 1U)) {   // dK / dV of the previous item have been read back
                        atomicExch(err_flag, 327);
                        break;
                    }
                    tcgen05_fence_after();
                    const uint64_t bd = b_m + qs * (2 * BLOCK);
                    const uint32_t acc = c.first() ? 0U : 1U;
#pragma unroll
                    for (int kk = 0; kk < B_T / UMMA_K; ++kk) {
                        tcgen05_mma_f16(d_col, a_m + kk * STEP_MN, bd + kk * STEP_MN, IDESC_ACC, kk != 0 ? 1U : acc);
                    }
                    tcgen05_commit(bar(QG_EMPTY + qs));
                    tcgen05_commit(bar(P_EMPTY));
                    if (c.last()) tcgen05_commit(bar(ACC_FULL));
                }
            } else {
                // dQ tile = dS K: A = dS K-major (blocks of 64 keys 16 KB apart), B = K stored [key][dh] read MN-major
                const uint64_t ds_k = make_smem_desc(smem_u32(smem + plan::OFF_DS), 16, 1024);
                const uint64_t k_m = make_smem_desc(kv0, plan::TILE, 1024);
                for (; !c.done(p); advance()) {
                    const uint32_t kvs = n_item & 1U, dqb = g & 1U;
                    if (!mbar_wait(bar(P_FULL), g & 1U)) {
                        atomicExch(err_flag, 325);
                        break;
                    }
                    if (!mbar_wait(bar(DQ_FREE + dqb), ((g >> 1) & 1U) ^ 1U)) {
                        atomicExch(err_flag, 326);
                        break;
                    }
                    tcgen05_fence_after();
                    const uint64_t km = k_m + kvs * (2 * BLOCK);
#pragma unroll
                    for (int kk = 0; kk < B_T / UMMA_K; ++kk) {
                        tcgen05_mma_f16(tmem_base + plan::COL_DQ + dqb * B_DH, ds_k + (kk >> 2) * BLOCK + (kk & 3) * STEP_K, km + kk * STEP_MN, IDESC_DQ,
                                        kk != 0 ? 1U : 0U);
                    }
                    tcgen05_commit(bar(DQ_FULL + dqb));
                    tcgen05_commit(bar(P_EMPTY));
                    if (c.last()) tcgen05_commit(bar(KV_EMPTY + kvs));
                }
            }
        }
    } else if (warp < 21) {
        // ---------------- softmax: one thread per query row and 32-key quarter ----------------
        const int quad = warp & 3, colq = (warp - 5) >> 2;          // lane quadrant of tensor memory, 32-column quarter
        const int r = quad * 32 + lane;
        const float sl2 = p.scale * B_LOG2E;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
        // this thread's 32 keys = four 16-byte chunks of one 128-byte row of block colq / 2
        unsigned char *p_row = smem + plan::OFF_P + (colq >> 1) * plan::TILE + r * 128;
        unsigned char *ds_row = smem + plan::OFF_DS + (colq >> 1) * plan::TILE + r * 128;
        const int chunk0 = (colq & 1) * 4;
        bool dead = false;
        // one lane polls the barrier (32 lanes polling the same word keep the shared-memory pipe busy for nothing), the
        // result reaches the others through the shuffle, which also orders their later reads behind the observed phase
        auto wait_or_die = [&](int which, uint32_t parity, int code) {
            if (dead) return;
            int ok = 1;
            if (lane == 0) ok = mbar_wait(bar(which), parity) ? 1 : 0;
            ok = __shfl_sync(0xffffffffU, ok, 0);
            if (!ok) {
                dead = true;
                if (lane == 0) atomicExch(err_flag, code);
            }
        };
        b_cursor c;
        c.item = blockIdx.x;
        c.group = p.hq / p.hkv;
        c.seek(tile_nqt, p, stride);
        // Row metadata (first allowed key, statistics) of a step is fetched one step ahead: the loads' latency would
        // otherwise sit on the path every step has to wait for. The loads are unconditional (row clamped), so that
        // nothing waits for one of them before the others are issued.
        // (nothing may consume a loaded value before the next step either: a select on it here would wait for the load)
        int n_lo = 0x7fffffff;
        bool n_in = false;
        float n_m = 0.0f, n_l = 0.0f, n_d = 0.0f;
        auto fetch_meta = [&](const b_cursor &cc) {
            n_in = !cc.done(p) && cc.q0() + r < p.n_tokens;
            const int row = n_in ? cc.q0() + r : 0, hh = n_in ? cc.head() : 0;
            const float *st = stats + ((size_t)row * p.hq + hh) * 3;
            n_lo = __ldg(row_lo + row);
            n_m = st[0];
            n_l = st[1];
            n_d = st[2];
        };
        fetch_meta(c);
        for (uint32_t g = 0; !c.done(p) && !dead; ++g) {
            const int q0 = c.q0(), qi = q0 + r;
            const int key0 = c.k0 + colq * 32;
            const int lo_key = n_in ? n_lo : 0x7fffffff;
            const bool valid = lo_key != 0x7fffffff;
            // P = exp(s scale - m) / l = exp2(s sl2 - (m log2e + log2 l))
            const float m2 = (valid && n_l > 0.0f && n_m != -INFINITY) ? fmaf(n_m, B_LOG2E, __log2f(n_l)) : INFINITY;
            const float dsc = valid ? n_d * p.scale : 0.0f;
            c.next(tile_nqt, p, stride);
            fetch_meta(c);                                   // for the next step; consumed after this step's work
            // allowed local columns [c_lo, c_hi] of this thread's 32 keys
            const int c_lo = valid ? max(0, lo_key - key0) : 32, c_hi = valid ? min(31, qi - key0) : -1;
            wait_or_die(S_FULL, g & 1U, 328);
            tcgen05_fence_after();
            const bool anyc = !dead && __any_sync(0xffffffffU, c_lo <= 31 && c_hi >= 0);
            const bool allc = __all_sync(0xffffffffU, c_lo <= 0 && c_hi >= 31);
            uint32_t pk[16], dk_[16];
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {                         // two sub-chunks of 16 columns
                if (anyc) {
                    uint32_t vs[16], vp[16];
                    tmem_ld_32x32b_x16_nowait(lane_base + plan::COL_S + colq * 32 + cc * 16, vs);
                    tmem_ld_32x32b_x16_nowait(lane_base + plan::COL_DP + colq * 32 + cc * 16, vp);
                    tmem_ld_wait();
                    if (cc == 1) {
                        tcgen05_fence_before();
                        __syncwarp();
                        if (lane == 0) b_arrive(bar(S_FREE));
                    }
#pragma unroll
                    for (int i = 0; i < 16; i += 2) {
                        // P = exp2(s sl2 - m2);  dS = P (dP scale - D scale)
                        float p0 = b_ex2(fmaf(__uint_as_float(vs[i]), sl2, -m2));
                        float p1 = b_ex2(fmaf(__uint_as_float(vs[i + 1]), sl2, -m2));
                        float d0 = p0 * fmaf(__uint_as_float(vp[i]), p.scale, -dsc), d1 = p1 * fmaf(__uint_as_float(vp[i + 1]), p.scale, -dsc);
                        if (!allc) {
                            const int col = cc * 16 + i;
                            const bool a0 = col >= c_lo && col <= c_hi, a1 = col + 1 >= c_lo && col + 1 <= c_hi;
                            p0 = a0 ? p0 : 0.0f;
                            p1 = a1 ? p1 : 0.0f;
                            d0 = a0 ? d0 : 0.0f;
                            d1 = a1 ? d1 : 0.0f;
                        }
                        pk[cc * 8 + (i >> 1)] = half_pack<T>::pack(p0, p1);
                        dk_[cc * 8 + (i >> 1)] = half_pack<T>::pack(d0, d1);
                    }
                } else {
                    if (cc == 1) {
                        tcgen05_fence_before();
                        __syncwarp();
                        if (lane == 0) b_arrive(bar(S_FREE));
                    }
#pragma unroll
                    for (int i = 0; i < 8; ++i) pk[cc * 8 + i] = dk_[cc * 8 + i] = 0U;
                }
            }
            wait_or_die(P_EMPTY, (g & 1U) ^ 1U, 329);       // the products of the previous step have read P / dS
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int chunk = chunk0 + j;
                *reinterpret_cast<uint4 *>(p_row + ((chunk ^ (r & 7)) << 4)) = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
                *reinterpret_cast<uint4 *>(ds_row + ((chunk ^ (r & 7)) << 4)) = make_uint4(dk_[4 * j], dk_[4 * j + 1], dk_[4 * j + 2], dk_[4 * j + 3]);
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
        // one lane polls the barrier (32 lanes polling the same word keep the shared-memory pipe busy for nothing), the
        // result reaches the others through the shuffle, which also orders their later reads behind the observed phase
        auto wait_or_die = [&](int which, uint32_t parity, int code) {
            if (dead) return;
            int ok = 1;
            if (lane == 0) ok = mbar_wait(bar(which), parity) ? 1 : 0;
            ok = __shfl_sync(0xffffffffU, ok, 0);
            if (!ok) {
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
        c.group = p.hq / p.hkv;
        c.seek(tile_nqt, p, stride);
        uint32_t n_item = 0;
        for (uint32_t g = 0; !c.done(p) && !dead; ++g) {
            const uint32_t dqb = g & 1U;
            const int qi = c.q0() + r, h = c.head();
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
            c.next(tile_nqt, p, stride);
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
gd_status launch_bwd(gd_backend *be, const gdb_flash_args *a, float *dq32, const int *meta)
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
    gdb_launch(kern, grid, B_THREADS, plan::TOTAL, be->stream, mq, mk, mv, mg, a->cu, (const float *)a->stats, (T *)a->dk, (T *)a->dv, dq32, meta, p, be->err_flag);
    return gdb_launched(be, "attn5_backward");
}

}  // namespace

// dK, dV and the FP32 dQ accumulator (zero on entry) from statistics (max, sum, D) that are complete on entry and the
// mask bounds `meta` (first allowed key per query row, then query tiles per key tile) of the preparation kernel.
// Returns GD_ERR_UNSUPPORTED outside the fast path (the caller then runs the mma.sync kernel).
gd_status gdb_attn5_backward(gd_backend *be, const gdb_flash_args *a, float *dq32, const int *meta)
{
    const uintptr_t al = (uintptr_t)a->q | (uintptr_t)a->k | (uintptr_t)a->v | (uintptr_t)a->grad_out | (uintptr_t)a->dk | (uintptr_t)a->dv | (uintptr_t)dq32;
    if ((a->dtype != GDB_DTYPE_F16 && a->dtype != GDB_DTYPE_BF16) || a->dh != B_DH || a->causal == 0 || a->prefix != 0 || a->window < 0 ||
        (al % 16U) != 0U || a->hkv <= 0 || (a->hq % a->hkv) != 0 || a->hq > 65535 || a->n_tokens < B_T ||
        a->stats == NULL || dq32 == NULL || meta == NULL) {
        return GD_ERR_UNSUPPORTED;
    }
    return a->dtype == GDB_DTYPE_F16 ? launch_bwd<__half>(be, a, dq32, meta) : launch_bwd<__nv_bfloat16>(be, a, dq32, meta);
}
