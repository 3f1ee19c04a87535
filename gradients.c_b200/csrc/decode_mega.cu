// One KV-cache decode step (gpt_block_decode_cached, examples/gpt_lm/gpt_lm_shared.c:961-1115, the logits head
// :1204-1246 and greedy sampling :1388-1398) as ONE persistent kernel: one CTA per SM, launched cooperatively, walks
// through the phases of a step and of the following steps, separated by grid-wide barriers instead of kernel launches.
//
// A decode step of the benchmark model moves 22.5 MB of weights and the live K / V (174 MB on average): 27 us at the
// measured copy bandwidth. As 28 dependent launches it takes 183 us, nearly all of it launch and drain latency. Here a
// step is 5 phases per layer + 2:
//   A  [embedding +] RMSNorm as the prologue of the QKV projection, RoPE and the K / V append as its epilogue (a CTA's
//      16 output columns are 8 rotation pairs of one head, or 16 value columns)
//   B  attention over the cache: the 16 warps of a CTA are heads x key ranges of one sequence, each streaming its keys
//      through a private shared-memory ring (cp.async, three tiles of 16 keys in flight), merged in shared memory
//   C  attention output projection, residual add in its epilogue
//   D  RMSNorm as the prologue of the up / gate projection, SwiGLU as its epilogue
//   E  down projection, residual add in its epilogue
//   F  final RMSNorm as the prologue of the logits projection
//   G  greedy sampling (soft cap, first maximum), token / position feedback for the next step
// Every phase runs the device functions of decode_parts.cuh that the stand-alone kernels run, on the same partition
// of the work (16-column units with K split over eight warps, the same key splits), so a step gives the same bits as
// the 28 launches and the generated ids are identical.
//
// Grid barrier: a monotonically increasing counter in global memory; thread 0 of each CTA adds 1 (release) and polls
// (acquire) until the counter reaches the phase's target. The poll is bounded: when it runs out, the CTA stores code 398
// in the backend's error word, raises the abort bit of the counter word that every other CTA's poll also sees, and the
// kernel returns.
// Buffers written inside the kernel are read with plain or L2 loads after a barrier, never through the read-only path.
#include "common.cuh"
#include "decode_parts.cuh"
#include "tcgen05.cuh"   // cluster rank, mapa, cluster barrier

#include <stdlib.h>

namespace {

using namespace gdb_dec;

constexpr int MG_THREADS = 512, MG_WARPS = MG_THREADS / 32;
constexpr unsigned MG_SPIN_LIMIT = 1U << 22;   // polls of the barrier word (about a microsecond each) before giving up
constexpr int MG_ERR_BARRIER = 398;
constexpr int MG_OT_LD = SK_COLS + 1;
constexpr uint32_t MG_EPI_BYTES = 64U + SK_ROWS * SK_COLS * 2U;   // a unit's bias (two 16-byte pieces) and its residual tile [64][16]
constexpr uint32_t MG_RING_BYTES = 3U * 2U * 4U * 512U;   // per warp: three tiles of two key groups, K and V halves, 16 bytes per lane

struct mg_layout {
    uint32_t stage_bytes, red_off, ot_off, epi_off, total;
};
__host__ __device__ inline mg_layout mg_layout_for(uint32_t ch_max)
{
    mg_layout l;
    l.stage_bytes = SK_ROWS * (ch_max + 8U) * 2U + ch_max * 48U;   // A tile [64][ch + 8] + the larger of the two weight tiles ([ch][24])
    l.red_off = 2U * l.stage_bytes;
    l.ot_off = l.red_off + (uint32_t)SK_RED_BYTES;
    l.epi_off = l.ot_off + (uint32_t)(SK_ROWS * MG_OT_LD * sizeof(float));
    l.total = l.epi_off + 2U * MG_EPI_BYTES;
    const uint32_t attn = MG_WARPS * MG_RING_BYTES + MG_WARPS * (2U + 64U) * (uint32_t)sizeof(float);   // the attention phase's rings and partials alias the stages
    if (l.total < attn) l.total = attn;
    return l;
}

struct mg_ctx {
    unsigned char *sm;
    mg_layout lay;
    int tid, warp, lane;
    unsigned target;   // barrier count this CTA waits for next
    int *ok_flag;      // shared word: outcome of the last barrier
    unsigned long long *timeline;
};

// sync[0]: bits 0..30 count arrivals (monotonically, never reset inside a launch), bit 31 is the abort flag; one
// acquire load per poll sees both.
__device__ __forceinline__ bool mg_barrier(mg_ctx &c, unsigned *sync, int *err_flag)
{
    __syncthreads();
    c.target += gridDim.x;
    if (c.tid == 0) {
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(&sync[0]) : "memory");
        int ok = 1;
        unsigned spins = 0;
        for (;;) {
            unsigned v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(&sync[0]) : "memory");
            if ((v & 0x80000000U) != 0U || ++spins > MG_SPIN_LIMIT) {
                ok = 0;
                break;
            }
            if (v >= c.target) break;
        }
        if (!ok) {
            atomicOr(&sync[0], 0x80000000U);
            atomicCAS(err_flag, 0, MG_ERR_BARRIER);
        }
        *c.ok_flag = ok;
    }
    __syncthreads();
    if (c.timeline != nullptr && blockIdx.x == 0 && c.tid == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        *c.timeline++ = t;
    }
    return *c.ok_flag != 0;
}

// ---- operand staging ----
template <typename T>
__device__ __forceinline__ void mg_load_a(T *As, uint32_t LDA, const T *A, size_t lda, uint32_t CH, size_t k0, uint32_t M, int tid)
{
    const uint32_t segs = CH / 8U;
    for (uint32_t i = tid; i < SK_ROWS * segs; i += MG_THREADS) {
        const uint32_t r = i / segs, sgm = i % segs;
        sk_cp16(As + r * LDA + sgm * 8U, A + (size_t)(r < M ? r : 0U) * lda + k0 + sgm * 8U, r < M);
    }
}
// B_KMAJOR: the unit's 16 weight rows are rows row_lo .. row_lo + 7 and row_hi .. row_hi + 7 of B [N, K]; otherwise the
// unit's 16 columns start at row_lo of B [K, N].
template <typename T, bool B_KMAJOR>
__device__ __forceinline__ void mg_load_w(T *Ws, const T *B, size_t ldb, uint32_t CH, size_t k0, uint32_t row_lo, uint32_t row_hi, int tid)
{
    if (B_KMAJOR) {
        const uint32_t segs = CH / 8U, LDW = CH + 8U;
        for (uint32_t i = tid; i < SK_COLS * segs; i += MG_THREADS) {
            const uint32_t r = i / segs, sgm = i % segs;
            const uint32_t wrow = r < 8U ? row_lo + r : row_hi + (r - 8U);
            sk_cp16(Ws + r * LDW + sgm * 8U, B + (size_t)wrow * ldb + k0 + sgm * 8U, true);
        }
    } else {
        for (uint32_t i = tid; i < CH * 2U; i += MG_THREADS) {
            const uint32_t k = i >> 1, sgm = i & 1U;
            sk_cp16(Ws + k * 24U + sgm * 8U, B + (k0 + k) * ldb + row_lo + sgm * 8U, true);
        }
    }
}
__device__ __forceinline__ void mg_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void mg_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void mg_wait_one() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }

template <typename T> struct mg_nan_pair;
template <> struct mg_nan_pair<__half> { static constexpr unsigned word = 0x7e007e00U; };
template <> struct mg_nan_pair<__nv_bfloat16> { static constexpr unsigned word = 0x7fc07fc0U; };

// ---- [embedding] + RMSNorm into the resident A tile ----
// GATHER: row r = table[ids[r]] (an id outside the table gives a NaN row, as the embedding kernel does); otherwise row r of
// x [B, D]. mg_stage_rows puts every row in flight at once with cp.async; after the wait, mg_norm_rows replaces row r by
// round(x * w * rsqrt(mean(x^2) + eps)) in the per-lane order of rms_fwd_kernel (lane takes the 8-element vectors lane,
// lane + 32), one warp per row, the warp's four rows interleaved.
template <typename T, bool GATHER>
__device__ __forceinline__ void mg_stage_rows(T *As, uint32_t LDA, const T *x, const int32_t *ids, uint32_t vocab, int B, int D, int tid,
                                              uint32_t row0, uint32_t nrows)
{
    const uint32_t vecs = (uint32_t)D / 8U;
    for (uint32_t i = tid; i < nrows * vecs; i += MG_THREADS) {
        const uint32_t r = row0 + i / vecs, v = i % vecs;
        T *dst = As + (size_t)r * LDA + v * 8U;
        if (GATHER) {
            const int id = (int)r < B ? ids[r] : 0;
            if ((int)r < B && (id < 0 || (uint32_t)id >= vocab)) {
                const unsigned nw = mg_nan_pair<T>::word;
                *reinterpret_cast<uint4 *>(dst) = make_uint4(nw, nw, nw, nw);
            } else {
                sk_cp16(dst, x + (size_t)((int)r < B ? id : 0) * D + v * 8U, (int)r < B);
            }
        } else {
            sk_cp16(dst, x + (size_t)((int)r < B ? r : 0U) * D + v * 8U, (int)r < B);
        }
    }
}

// `wraw`: the lane's two vectors of the norm weight, loaded by the caller before it waited for the rows.
// The two CTAs of a cluster share the work: this CTA normalises rows row0 .. row0 + 31 (staged in its own tile) and writes
// the result into its own tile and, through distributed shared memory, into the same place of its peer's tile
// (`peer_delta` = the peer's shared-memory window minus this CTA's, as a shared::cluster address difference); rows at
// or beyond B are written as zeros. The caller's cluster barrier makes both halves visible to both CTAs.
template <typename T>
__device__ __forceinline__ void mg_norm_rows(T *As, uint32_t LDA, const uint4 (&wraw)[2], int B, int D, float eps, int warp, int lane,
                                             uint32_t row0, uint32_t peer_rank)
{
    constexpr int RPW = (SK_ROWS / 2) / MG_WARPS;   // rows per warp: 32 rows per CTA of the pair
    const uint32_t vecs = (uint32_t)D / 8U;         // at most 64 (D <= 512): two vectors per lane
    float ss[RPW];
#pragma unroll
    for (int q = 0; q < RPW; ++q) {
        const int r = (int)row0 + warp + q * MG_WARPS;
        ss[q] = 0.0f;
        if (r < B) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const uint32_t v = (uint32_t)lane + 32U * (uint32_t)i;
                if (v < vecs) {
                    const uint4 a = *reinterpret_cast<const uint4 *>(As + (size_t)r * LDA + v * 8U);
                    const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const float2 f = pack2<T>::up(aw[k]);
                        ss[q] += f.x * f.x;
                        ss[q] += f.y * f.y;
                    }
                }
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
        for (int q = 0; q < RPW; ++q) ss[q] += __shfl_xor_sync(0xffffffffU, ss[q], o);
    }
    float wf[2][8];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const uint32_t ww[4] = {wraw[i].x, wraw[i].y, wraw[i].z, wraw[i].w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 f = pack2<T>::up(ww[k]);
            wf[i][2 * k] = f.x;
            wf[i][2 * k + 1] = f.y;
        }
    }
#pragma unroll
    for (int q = 0; q < RPW; ++q) {
        const int r = (int)row0 + warp + q * MG_WARPS;
        const float inv = r < B ? rsqrtf(ss[q] / (float)(size_t)D + eps) : 0.0f;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const uint32_t v = (uint32_t)lane + 32U * (uint32_t)i;
            if (v < vecs) {
                T *p = As + (size_t)r * LDA + v * 8U;
                uint4 o = make_uint4(0U, 0U, 0U, 0U);
                if (r < B) {
                    const uint4 a = *reinterpret_cast<const uint4 *>(p);
                    const float2 x0 = pack2<T>::up(a.x), x1 = pack2<T>::up(a.y), x2 = pack2<T>::up(a.z), x3 = pack2<T>::up(a.w);
                    o.x = pack2<T>::down(x0.x * wf[i][0] * inv, x0.y * wf[i][1] * inv);
                    o.y = pack2<T>::down(x1.x * wf[i][2] * inv, x1.y * wf[i][3] * inv);
                    o.z = pack2<T>::down(x2.x * wf[i][4] * inv, x2.y * wf[i][5] * inv);
                    o.w = pack2<T>::down(x3.x * wf[i][6] * inv, x3.y * wf[i][7] * inv);
                }
                *reinterpret_cast<uint4 *>(p) = o;
                const uint32_t remote = gdb_t5::mapa_shared(sk_smem(p), peer_rank);
                asm volatile("st.shared::cluster.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(remote), "r"(o.x), "r"(o.y), "r"(o.z), "r"(o.w) : "memory");
            }
        }
    }
}

enum { EPI_PLAIN = 0, EPI_ROPE = 1, EPI_SWIGLU = 2, EPI_RESID = 3 };
enum { PRO_GLOBAL = 0, PRO_EMB = 1, PRO_ROWS = 2 };

template <typename T> struct mg_gemm {
    // operands
    const T *A;            // PRO_GLOBAL: activations [B, K]
    const T *W;            // weight: K-major [N, K] or [K, N]
    const T *bias;
    T *C;                  // PLAIN / SWIGLU / RESID destination [B, N]
    uint32_t K, N, CH;
    int bias_mode;
    // prologue (PRO_EMB: x = table rows of ids; PRO_ROWS: x [B, K])
    const T *x, *norm_w;
    const int32_t *ids;
    uint32_t vocab;
    // RESID epilogue: C = round(res + round(linear)); res [B, N], or rows res_ids of the table `res` when res_ids != NULL
    const T *res;
    const int32_t *res_ids;
    // rope epilogue
    T *q, *kc, *vc;
    const int32_t *positions;
};

// One phase = one contraction [B <= 64, K] x [K, N] spread over the CTAs in units of 16 output columns. Warps w and
// w + 8 share the k range w of a chunk and take 32 of the 64 rows each, so the sum of an output over k is formed exactly
// as in the eight-warp stand-alone kernel.
template <typename T, bool B_KMAJOR, int EPI, int PRO>
__device__ __forceinline__ void mg_gemm_phase(mg_ctx &c, const gdb_mega_args &a, const mg_gemm<T> &g)
{
    uint32_t nunits;
    if (EPI == EPI_ROPE) {
        nunits = 2U * (uint32_t)a.H * 4U + (uint32_t)a.D / 16U;   // q and k: 8 rotation pairs of one head each; v: 16 columns
    } else if (EPI == EPI_SWIGLU) {
        nunits = g.N / 8U;                                         // 8 up + 8 gate columns
    } else {
        nunits = g.N / 16U;
    }
    // Resident-A phases run on CTA pairs (clusters of two): a pair takes part when either of its CTAs has a unit, because
    // each CTA normalises half of the rows for both.
    if (PRO == PRO_GLOBAL ? blockIdx.x >= nunits : (blockIdx.x & ~1U) >= nunits) return;
    const uint32_t CH = g.CH, LDA = CH + 8U, LDW = B_KMAJOR ? CH + 8U : 24U, a_bytes = SK_ROWS * LDA * 2U;
    const uint32_t n_chunks = g.K / CH, kw = CH / SK_WARPS;
    const uint32_t M = (uint32_t)a.B;
    const uint32_t kslot = (uint32_t)c.warp & 7U;
    const size_t ldw = B_KMAJOR ? (size_t)g.K : (size_t)g.N;
    sk_red_t red = reinterpret_cast<sk_red_t>(c.sm + c.lay.red_off);
    float(*ot)[MG_OT_LD] = reinterpret_cast<float(*)[MG_OT_LD]>(c.sm + c.lay.ot_off);
    auto stage_a = [&](uint32_t st) { return reinterpret_cast<T *>(c.sm + st * c.lay.stage_bytes); };
    auto stage_w = [&](uint32_t st) { return reinterpret_cast<T *>(c.sm + st * c.lay.stage_bytes + a_bytes); };
    auto unit_rows = [&](uint32_t unit, uint32_t *lo, uint32_t *hi) {
        if (EPI == EPI_ROPE) {
            const uint32_t nrope = 2U * (uint32_t)a.H * 4U;
            if (unit < nrope) {
                const uint32_t region = unit / ((uint32_t)a.H * 4U), hg = unit % ((uint32_t)a.H * 4U);
                *lo = region * (uint32_t)a.D + (hg / 4U) * 64U + (hg % 4U) * 8U;
                *hi = *lo + 32U;
            } else {
                *lo = 2U * (uint32_t)a.D + (unit - nrope) * 16U;
                *hi = *lo + 8U;
            }
        } else if (EPI == EPI_SWIGLU) {
            *lo = unit * 8U;
            *hi = g.N + unit * 8U;
        } else {
            *lo = unit * 16U;
            *hi = *lo + 8U;
        }
    };
    // the unit's epilogue operands ride along with its weights: bias pieces, and for RESID the residual tile
    auto load_epi = [&](uint32_t lo, uint32_t hi, uint32_t eb) {
        T *sm_bias = reinterpret_cast<T *>(c.sm + c.lay.epi_off + eb * MG_EPI_BYTES), *sm_res = sm_bias + 32;
        if (g.bias != nullptr && c.tid < 2) sk_cp16(sm_bias + c.tid * 8, g.bias + (c.tid == 0 ? lo : hi), true);
        if (EPI == EPI_RESID) {
            for (uint32_t i = c.tid; i < SK_ROWS * 2U; i += MG_THREADS) {
                const uint32_t r = i >> 1, pc = i & 1U;
                T *dst = sm_res + r * SK_COLS + pc * 8U;
                if (r >= M) continue;
                if (g.res_ids != nullptr) {
                    const int id = g.res_ids[r];
                    if (id < 0 || (uint32_t)id >= g.vocab) {
                        const unsigned nw = mg_nan_pair<T>::word;
                        *reinterpret_cast<uint4 *>(dst) = make_uint4(nw, nw, nw, nw);
                    } else {
                        sk_cp16(dst, g.res + (size_t)id * g.N + lo + pc * 8U, true);
                    }
                } else {
                    sk_cp16(dst, g.res + (size_t)r * g.N + lo + pc * 8U, true);
                }
            }
        }
    };
    uint32_t wst = 0U;   // weight stage / epilogue-operand buffer of the current unit (resident-A phases)
    if (PRO != PRO_GLOBAL) {
        // The first unit's weights stream in while the prologue runs. This CTA stages and normalises rows
        // rank * 32 .. + 31 and writes them into both tiles of the pair; the cluster barrier publishes both halves.
        const uint32_t rank = gdb_t5::cluster_ctarank() & 1U, row0 = rank * (SK_ROWS / 2);
        uint4 wraw[2] = {make_uint4(0U, 0U, 0U, 0U), make_uint4(0U, 0U, 0U, 0U)};
        if (blockIdx.x < nunits) {
            uint32_t lo, hi;
            unit_rows(blockIdx.x, &lo, &hi);
            mg_load_w<T, B_KMAJOR>(stage_w(0), g.W, ldw, CH, 0, lo, hi, c.tid);
            load_epi(lo, hi, 0U);
        }
        if (PRO == PRO_EMB) {
            mg_stage_rows<T, true>(stage_a(0), LDA, g.x, g.ids, g.vocab, a.B, a.D, c.tid, row0, SK_ROWS / 2);
        } else {
            mg_stage_rows<T, false>(stage_a(0), LDA, g.x, nullptr, 0U, a.B, a.D, c.tid, row0, SK_ROWS / 2);
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const uint32_t v = (uint32_t)c.lane + 32U * (uint32_t)i;
            if (v < (uint32_t)a.D / 8U) wraw[i] = __ldg(reinterpret_cast<const uint4 *>(g.norm_w) + v);
        }
        mg_commit();
        mg_wait_all();
        __syncthreads();
        mg_norm_rows<T>(stage_a(0), LDA, wraw, a.B, a.D, a.eps, c.warp, c.lane, row0, rank ^ 1U);
        gdb_t5::cluster_sync_all();   // every thread of both CTAs: the whole normalised tile is in both shared memories
        if (blockIdx.x >= nunits) return;
    }
    for (uint32_t unit = blockIdx.x; unit < nunits; unit += gridDim.x) {
        uint32_t lo, hi;
        unit_rows(unit, &lo, &hi);
        float acc[2][2][4];
        sk_zero(acc);
        auto mma = [&](const T *As, const T *Ws) {
            if (c.warp < SK_WARPS) {
                sk_mma_chunk<T, B_KMAJOR, 0, 2>(acc, As, Ws, LDA, LDW, kslot * kw, (kslot + 1U) * kw, c.lane);
            } else {
                sk_mma_chunk<T, B_KMAJOR, 2, 2>(acc, As, Ws, LDA, LDW, kslot * kw, (kslot + 1U) * kw, c.lane);
            }
        };
        if (PRO != PRO_GLOBAL) {
            // resident A (single chunk): this unit's weights and epilogue operands are in stage / buffer `wst` (loaded by the
            // prologue or prefetched during the previous unit); those of the CTA's next unit go to the other one now
            if (unit + gridDim.x < nunits) {
                uint32_t nlo, nhi;
                unit_rows(unit + gridDim.x, &nlo, &nhi);
                mg_load_w<T, B_KMAJOR>(stage_w(wst ^ 1U), g.W, ldw, CH, 0, nlo, nhi, c.tid);
                load_epi(nlo, nhi, wst ^ 1U);
            }
            mg_commit();
            mg_wait_one();   // everything but the next unit's operands
            __syncthreads();
            mma(stage_a(0), stage_w(wst));
        } else {
            auto load_chunk = [&](uint32_t ci, uint32_t st) {
                mg_load_a<T>(stage_a(st), LDA, g.A, (size_t)g.K, CH, (size_t)ci * CH, M, c.tid);
                mg_load_w<T, B_KMAJOR>(stage_w(st), g.W, ldw, CH, (size_t)ci * CH, lo, hi, c.tid);
                if (ci == 0U) load_epi(lo, hi, 0U);
                mg_commit();
            };
            load_chunk(0, 0);
            if (n_chunks > 1U) load_chunk(1, 1);
            for (uint32_t ci = 0; ci < n_chunks; ++ci) {
                const uint32_t st = ci & 1U;
                if (ci + 1U < n_chunks) {
                    mg_wait_one();
                } else {
                    mg_wait_all();
                }
                __syncthreads();
                mma(stage_a(st), stage_w(st));
                __syncthreads();
                if (ci + 2U < n_chunks) load_chunk(ci + 2U, st);
            }
        }
        if (c.warp < SK_WARPS) {
            sk_store_partials<0, 2>(red, acc, (int)kslot, c.lane);
        } else {
            sk_store_partials<2, 2>(red, acc, (int)kslot, c.lane);
        }
        __syncthreads();
        const uint32_t eb = PRO != PRO_GLOBAL ? wst : 0U;
        const T *sm_bias_u = reinterpret_cast<const T *>(c.sm + c.lay.epi_off + eb * MG_EPI_BYTES), *sm_res_u = sm_bias_u + 32;
        const T *bias = g.bias != nullptr ? sm_bias_u : nullptr;   // local columns: 0..7 = lo.., 8..15 = hi..
        if (EPI == EPI_SWIGLU) {
            for (int o = c.tid; o < SK_ROWS * (SK_COLS / 2); o += MG_THREADS) {
                const int r = o / (SK_COLS / 2), cc = o % (SK_COLS / 2);
                if ((uint32_t)r >= M) continue;
                const float up = sk_sum(red, r, cc), gate = sk_sum(red, r, cc + 8);
                gdb_io<T>::st(g.C, (size_t)r * g.N + lo + cc, sk_swiglu<T>(up, gate, bias, g.bias_mode, (uint32_t)cc, (uint32_t)cc + 8U));
            }
        } else if (EPI == EPI_PLAIN) {
            for (int o = c.tid; o < SK_ROWS * SK_COLS; o += MG_THREADS) {
                const int r = o / SK_COLS, cc = o % SK_COLS;
                if ((uint32_t)r >= M) continue;
                gdb_io<T>::st(g.C, (size_t)r * g.N + lo + cc, sk_bias<T>(sk_sum(red, r, cc), bias, g.bias_mode, (uint32_t)cc));
            }
        } else if (EPI == EPI_RESID) {
            // the rounded linear output, then the residual add with its own rounding (gd_backend_add after the linear layer)
            for (int o = c.tid; o < SK_ROWS * SK_COLS; o += MG_THREADS) {
                const int r = o / SK_COLS, cc = o % SK_COLS;
                if ((uint32_t)r >= M) continue;
                const float y = gdb_io<T>::rnd(sk_bias<T>(sk_sum(red, r, cc), bias, g.bias_mode, (uint32_t)cc));
                gdb_io<T>::st(g.C, (size_t)r * g.N + lo + cc, gdb_io<T>::ld(sm_res_u, (size_t)r * SK_COLS + cc) + y);
            }
        } else {
            // the rounded linear output of the unit, then the rotation of qkv_split_rope and the append of kv_cache_append
            for (int o = c.tid; o < SK_ROWS * SK_COLS; o += MG_THREADS) {
                const int r = o / SK_COLS, cc = o % SK_COLS;
                ot[r][cc] = (uint32_t)r < M ? gdb_io<T>::rnd(sk_bias<T>(sk_sum(red, r, cc), bias, g.bias_mode, (uint32_t)cc)) : 0.0f;
            }
            __syncthreads();
            const uint32_t nrope = 2U * (uint32_t)a.H * 4U, area = (uint32_t)a.D;
            if (unit < nrope) {
                const uint32_t region = unit / ((uint32_t)a.H * 4U), hg = unit % ((uint32_t)a.H * 4U);
                const uint32_t hcol = (hg / 4U) * 64U + (hg % 4U) * 8U, grp = hg % 4U;
                for (int o = c.tid; o < SK_ROWS * 8; o += MG_THREADS) {
                    const int r = o / 8, e = o % 8;
                    if ((uint32_t)r >= M) continue;
                    const int pos = g.positions[r];
                    float cs, sn;
                    rope_cos_sin(a.rope, a.rope_table, grp * 8U + (unsigned)e, pos, &cs, &sn);
                    const float x0 = ot[r][e], x1 = ot[r][8 + e];
                    const float y0 = rope_lo(x0, x1, cs, sn), y1 = rope_hi(x0, x1, cs, sn);
                    if (region == 0U) {
                        gdb_io<T>::st(g.q, (size_t)r * area + hcol + e, y0);
                        gdb_io<T>::st(g.q, (size_t)r * area + hcol + 32U + e, y1);
                    } else if (pos >= 0 && pos < a.CAP) {
                        const size_t kv = ((size_t)r * a.CAP + (size_t)pos) * area + hcol + e;
                        gdb_io<T>::st(g.kc, kv, y0);
                        gdb_io<T>::st(g.kc, kv + 32U, y1);
                    }
                }
            } else {
                for (int o = c.tid; o < SK_ROWS * SK_COLS; o += MG_THREADS) {
                    const int r = o / SK_COLS, cc = o % SK_COLS;
                    if ((uint32_t)r >= M) continue;
                    const int pos = g.positions[r];
                    if (pos < 0 || pos >= a.CAP) continue;
                    gdb_io<T>::st(g.vc, ((size_t)r * a.CAP + (size_t)pos) * area + (lo - 2U * area) + cc, ot[r][cc]);
                }
            }
        }
        __syncthreads();   // the weight stage, the reduction buffer and the epilogue operands are reused by the CTA's next unit
        wst ^= 1U;
    }
}

template <typename T>
__global__ void __launch_bounds__(MG_THREADS, 1) decode_mega_kernel(const __grid_constant__ gdb_mega_args a, const mg_layout lay)
{
    extern __shared__ __align__(16) unsigned char mg_sm[];
    __shared__ int ok_flag;
    __shared__ float am_sv[32];
    __shared__ uint32_t am_si[32];
    mg_ctx c;
    c.sm = mg_sm;
    c.lay = lay;
    c.tid = threadIdx.x;
    c.warp = threadIdx.x >> 5;
    c.lane = threadIdx.x & 31;
    c.target = 0U;
    c.ok_flag = &ok_flag;
    c.timeline = a.timeline;
    const uint32_t D = (uint32_t)a.D, F = (uint32_t)a.F, V = (uint32_t)a.V;
    const uint32_t ch_f = (F % 512U) == 0U ? 512U : ((F % 256U) == 0U ? 256U : 128U);
    const int t0 = *a.step_counter;   // advanced once, after the last step
    decode_params dp;
    dp.batch = a.B;
    dp.tq = 1;
    dp.tmax = a.CAP;
    dp.hq = a.H;
    dp.hkv = a.H;
    dp.dh = 64;
    dp.window = a.window;
    dp.prefix = 0;
    dp.pos_mode = 2;
    dp.cache_pos = 0;
    dp.scale = a.scale;
    for (int step = 0; step < a.n_steps; ++step) {
        for (int layer = 0; layer < a.L; ++layer) {
            const void *const *lw = a.lw[layer];
            T *kc = (T *)a.kc[layer], *vc = (T *)a.vc[layer];
            {   // A: norm + QKV + RoPE + append
                mg_gemm<T> g = {};
                g.W = (const T *)lw[1];
                g.bias = (const T *)lw[2];
                g.K = D;
                g.N = 3U * D;
                g.CH = D;
                g.bias_mode = 2;
                g.norm_w = (const T *)lw[0];
                g.q = (T *)a.q;
                g.kc = kc;
                g.vc = vc;
                g.positions = a.positions;
                if (layer == 0) {
                    g.x = (const T *)a.emb;
                    g.ids = a.tokens;
                    g.vocab = V;
                    mg_gemm_phase<T, true, EPI_ROPE, PRO_EMB>(c, a, g);
                } else {
                    g.x = (const T *)a.xbuf;
                    mg_gemm_phase<T, true, EPI_ROPE, PRO_ROWS>(c, a, g);
                }
            }
            if (!mg_barrier(c, a.sync, a.err_flag)) return;
            {   // B: attention; a CTA takes `hpc` heads x `splits` key ranges of one sequence and merges the ranges in shared memory
                const int hpc = 16 / a.splits, groups = a.H / hpc, units = a.B * groups;
                float *sm_ml = reinterpret_cast<float *>(c.sm + MG_WARPS * MG_RING_BYTES), *sm_acc = sm_ml + MG_WARPS * 2;
                for (int unit = blockIdx.x; unit < units; unit += gridDim.x) {
                    const int b = unit / groups, hl = c.warp % hpc, split = c.warp / hpc;
                    const long long w = (long long)b * a.H + (unit % groups) * hpc + hl;
                    const int item = hl * a.splits + split;   // the query's splits side by side
                    if (split < a.splits) {
                        decode_split_item<T, 64, true>((const T *)a.q, kc, vc, a.positions, sm_ml + item * 2, sm_acc + item * 64, dp, a.splits, w, split,
                                                      c.lane, c.sm + (size_t)c.warp * MG_RING_BYTES);
                    }
                    __syncthreads();
                    if (c.warp < hpc) {
                        decode_combine_query<T, false>(sm_ml + c.warp * a.splits * 2, sm_acc + c.warp * a.splits * 64,
                                                       (T *)a.attn + (size_t)((long long)b * a.H + (unit % groups) * hpc + c.warp) * 64, 64, a.splits, c.lane);
                    }
                    __syncthreads();
                }
            }
            if (!mg_barrier(c, a.sync, a.err_flag)) return;
            {   // C: attention output projection + residual: resid = x + proj (layer 0: x = the embedding rows)
                mg_gemm<T> g = {};
                g.A = (const T *)a.attn;
                g.W = (const T *)lw[3];
                g.bias = (const T *)lw[4];
                g.C = (T *)a.resid;
                g.K = D;
                g.N = D;
                g.CH = D;
                g.bias_mode = 2;
                if (layer == 0) {
                    g.res = (const T *)a.emb;
                    g.res_ids = a.tokens;
                    g.vocab = V;
                } else {
                    g.res = (const T *)a.xbuf;
                }
                mg_gemm_phase<T, true, EPI_RESID, PRO_GLOBAL>(c, a, g);
            }
            if (!mg_barrier(c, a.sync, a.err_flag)) return;
            {   // D: norm + up / gate + SwiGLU
                mg_gemm<T> g = {};
                g.W = (const T *)lw[6];
                g.bias = (const T *)lw[7];
                g.C = (T *)a.act;
                g.K = D;
                g.N = F;
                g.CH = D;
                g.bias_mode = 2;
                g.x = (const T *)a.resid;
                g.norm_w = (const T *)lw[5];
                mg_gemm_phase<T, true, EPI_SWIGLU, PRO_ROWS>(c, a, g);
            }
            if (!mg_barrier(c, a.sync, a.err_flag)) return;
            {   // E: down projection (weight stored [F, D]) + residual: x = resid + mlp
                mg_gemm<T> g = {};
                g.A = (const T *)a.act;
                g.W = (const T *)lw[8];
                g.bias = (const T *)lw[9];
                g.C = (T *)a.xbuf;
                g.K = F;
                g.N = D;
                g.CH = ch_f;
                g.bias_mode = 1;
                g.res = (const T *)a.resid;
                mg_gemm_phase<T, false, EPI_RESID, PRO_GLOBAL>(c, a, g);
            }
            if (!mg_barrier(c, a.sync, a.err_flag)) return;
        }
        {   // F: final norm + logits
            mg_gemm<T> g = {};
            g.W = (const T *)a.w_lm;
            g.bias = (const T *)a.b_lm;
            g.C = (T *)a.logits;
            g.K = D;
            g.N = V;
            g.CH = D;
            g.bias_mode = 2;
            g.x = (const T *)a.xbuf;
            g.norm_w = (const T *)a.w_final;
            mg_gemm_phase<T, true, EPI_PLAIN, PRO_ROWS>(c, a, g);
        }
        if (!mg_barrier(c, a.sync, a.err_flag)) return;
        // G: greedy sampling and the feedback of ids and positions
        for (int row = blockIdx.x; row < a.B; row += gridDim.x) {
            const int32_t id = argmax_row<T>((const T *)a.logits + (size_t)row * V, V, a.softcap, am_sv, am_si);
            if (c.tid == 0) {
                a.tokens[row] = id;
                const int t = t0 + step;
                if (t >= 0 && t < a.max_steps) a.out_tokens[(size_t)t * a.B + row] = id;
                a.positions[row] += 1;
            }
            __syncthreads();
        }
        if (!mg_barrier(c, a.sync, a.err_flag)) return;
    }
    if (blockIdx.x == 0 && c.tid == 0) *a.step_counter = t0 + a.n_steps;
}

}  // namespace

bool gdb_decode_mega_supported(const gd_backend *be, uint32_t dtype, int B, int D, int F, int V, int H, int Dh, int L)
{
    if (be == NULL || (dtype != GDB_DTYPE_F16 && dtype != GDB_DTYPE_BF16) || be->gemm_mode != 0) return false;
    if (getenv("GDB200_DECODE_MEGA") != NULL && getenv("GDB200_DECODE_MEGA")[0] == '0') return false;
    if (getenv("GDB200_SKINNY_DIRECT") != NULL) return false;
    if (B < 1 || B > SK_ROWS || L < 1 || L > GDB_MEGA_MAX_LAYERS || Dh != 64 || H * Dh != D) return false;
    if (D != 128 && D != 256 && D != 512) return false;              // the normalised activations stay resident: one K chunk
    if (sk_chunk_for((uint32_t)F) == 0U || (V % 16) != 0) return false;   // F % 128 == 0 covers the 8-column SwiGLU units
    return true;
}

gd_status gdb_decode_mega_launch(gd_backend *be, uint32_t dtype, const gdb_mega_args *a)
{
    const uint32_t ch_f = sk_chunk_for((uint32_t)a->F);
    const mg_layout lay = mg_layout_for((uint32_t)a->D > ch_f ? (uint32_t)a->D : ch_f);
    void (*kern)(const gdb_mega_args, const mg_layout) = dtype == GDB_DTYPE_F16 ? decode_mega_kernel<__half> : decode_mega_kernel<__nv_bfloat16>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)lay.total);
    if (e != cudaSuccess) return gdb_fail(be, e, "decode step kernel: shared memory attribute");
    int per_sm = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, MG_THREADS, lay.total);
    if (e != cudaSuccess || per_sm < 1) {
        return e != cudaSuccess ? gdb_fail(be, e, "decode step kernel: occupancy") : GD_ERR_UNSUPPORTED;
    }
    // Cooperative (every CTA resident: the grid barriers need it) and in clusters of two (the CTAs of a pair share the
    // normalised activation tile through distributed shared memory).
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 2;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.gridDim = dim3((unsigned)be->sm_count & ~1U);
    cfg.blockDim = dim3(MG_THREADS);
    cfg.dynamicSmemBytes = lay.total;
    cfg.stream = be->stream;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    int clusters = 0;
    e = cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg);
    if (e != cudaSuccess || clusters * 2 < (int)cfg.gridDim.x) {
        (void)cudaGetLastError();
        return GD_ERR_UNSUPPORTED;   // the pairs cannot all be resident: the caller enqueues one launch per operation
    }
    e = cudaLaunchKernelEx(&cfg, kern, *a, lay);
    if (e == cudaErrorCooperativeLaunchTooLarge || e == cudaErrorNotSupported || e == cudaErrorInvalidValue || e == cudaErrorInvalidConfiguration) {
        (void)cudaGetLastError();   // this device / driver does not take the launch: the caller enqueues one launch per operation
        return GD_ERR_UNSUPPORTED;
    }
    if (e != cudaSuccess) return gdb_fail(be, e, "decode step kernel: launch");
    return gdb_launched(be, "decode step kernel");
}
