// Device-side building blocks of one KV-cache decode step, shared by the stand-alone kernels (one
// launch per operation: gemm_skinny.cu, embedding_rope.cu, attention.cu, the argmax of gpt_lm_native.cu)
// and by the persistent whole-step kernel of decode_mega.cu. Both sides call the same functions, so a
// step computed by one launch per operation and a step computed by the persistent kernel perform the
// same floating-point operations in the same order and produce the same bits.
#ifndef GDB200_DECODE_PARTS_CUH
#define GDB200_DECODE_PARTS_CUH

#include "common.cuh"

#include <math.h>

namespace gdb_dec {

// ------------------------------------------------------------------ 64-row contraction (mma.sync, K split over 8 warps)
template <typename T> struct mma16816;
template <> struct mma16816<__half> {
    static __device__ __forceinline__ void run(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2])
    {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
    }
};
template <> struct mma16816<__nv_bfloat16> {
    static __device__ __forceinline__ void run(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2])
    {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
    }
};

constexpr int SK_ROWS = 64, SK_COLS = 16, SK_WARPS = 8;
typedef float (*sk_red_t)[SK_ROWS][SK_COLS + 1];
constexpr size_t SK_RED_BYTES = sizeof(float) * SK_WARPS * SK_ROWS * (SK_COLS + 1);

__device__ __forceinline__ uint32_t sk_smem(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void sk_cp16(void *dst, const void *src, bool valid)
{
    const int bytes = valid ? 16 : 0;   // zero-fill rows beyond M
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(sk_smem(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void sk_ldm4(uint32_t (&r)[4], const void *p)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(sk_smem(p)));
}
__device__ __forceinline__ void sk_ldm4t(uint32_t (&r)[4], const void *p)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(sk_smem(p)));
}

template <int MTN>
__device__ __forceinline__ void sk_zero(float (&acc)[MTN][2][4])
{
#pragma unroll
    for (int i = 0; i < MTN; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.0f;
}

// One warp's share [k_begin, k_end) of a staged chunk: As [64][LDA] row-major activations, Ws either [16][LDW]
// (B_KMAJOR: one row per output column) or [chunk][LDW = 24] (one row per k). The warp multiplies the 16-row tiles
// MT0 .. MT0 + MTN - 1 (all four, or two when two warps share a k range); acc is indexed by tile - MT0.
template <typename T, bool B_KMAJOR, int MT0 = 0, int MTN = 4>
__device__ __forceinline__ void sk_mma_chunk(float (&acc)[MTN][2][4], const T *As, const T *Ws, uint32_t LDA, uint32_t LDW,
                                             uint32_t k_begin, uint32_t k_end, int lane)
{
    for (uint32_t k = k_begin; k < k_end; k += 16U) {
        uint32_t a[MTN][4], b4[4];
#pragma unroll
        for (int mt = 0; mt < MTN; ++mt) sk_ldm4(a[mt], As + ((MT0 + mt) * 16 + (lane & 15)) * LDA + k + (lane >> 4) * 8);
        if (B_KMAJOR) {
            sk_ldm4(b4, Ws + ((lane & 7) + ((lane >> 4) << 3)) * LDW + k + ((lane >> 3) & 1) * 8);
        } else {
            sk_ldm4t(b4, Ws + (k + (lane & 7) + ((lane >> 3) & 1) * 8) * LDW + (lane >> 4) * 8);
        }
        const uint32_t b0[2] = {b4[0], b4[1]}, b1[2] = {b4[2], b4[3]};
#pragma unroll
        for (int mt = 0; mt < MTN; ++mt) {
            mma16816<T>::run(acc[mt][0], a[mt], b0);
            mma16816<T>::run(acc[mt][1], a[mt], b1);
        }
    }
}

// A warp's partial tile (row tiles MT0 .. MT0 + MTN - 1 of the 64 x 16 unit) into slot `kslot` of the reduction buffer.
template <int MT0 = 0, int MTN = 4>
__device__ __forceinline__ void sk_store_partials(sk_red_t red, const float (&acc)[MTN][2][4], int kslot, int lane)
{
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int mt = 0; mt < MTN; ++mt)
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            const int r = (MT0 + mt) * 16 + g, c = nt * 8 + 2 * t;
            red[kslot][r][c] = acc[mt][nt][0];
            red[kslot][r][c + 1] = acc[mt][nt][1];
            red[kslot][r + 8][c] = acc[mt][nt][2];
            red[kslot][r + 8][c + 1] = acc[mt][nt][3];
        }
}

// Sum of the eight warps' partials of one output, in warp order.
__device__ __forceinline__ float sk_sum(sk_red_t red, int r, int c)
{
    float v = 0.0f;
#pragma unroll
    for (int w = 0; w < SK_WARPS; ++w) v += red[w][r][c];
    return v;
}

// Bias of a linear layer: bias_mode 2 = "round the product, then a rounded bias add" (matmul_nt followed by add),
// bias_mode 1 = bias added in FP32 before the single rounding (linear). The caller rounds at its store.
template <typename T>
__device__ __forceinline__ float sk_bias(float v, const T *bias, int bias_mode, uint32_t col)
{
    if (bias != nullptr) {
        if (bias_mode == 2) v = gdb_io<T>::rnd(v);
        v += gdb_io<T>::ld(bias, col);
    }
    return v;
}

// out = up * silu(gate) of the two rounded linear outputs (gd_swiglu_split after gd_linear_transposed_weight).
template <typename T>
__device__ __forceinline__ float sk_swiglu(float up, float gate, const T *bias, int bias_mode, uint32_t up_col, uint32_t gate_col)
{
    if (bias != nullptr) {
        if (bias_mode == 2) {
            up = gdb_io<T>::rnd(up);
            gate = gdb_io<T>::rnd(gate);
        }
        up += gdb_io<T>::ld(bias, up_col);
        gate += gdb_io<T>::ld(bias, gate_col);
    }
    up = gdb_io<T>::rnd(up);       // the values the separate linear call would have stored
    gate = gdb_io<T>::rnd(gate);
    return up * (gate * gdb_swiglu_sigmoid(gate));
}

// K chunk of the staged kernel for a contraction length K (0: the staged kernel does not take it).
static inline uint32_t sk_chunk_for(uint32_t K)
{
    return (K % 512U) == 0U ? 512U : ((K % 256U) == 0U ? 256U : ((K % 128U) == 0U ? 128U : 0U));
}

// ------------------------------------------------------------------ rotary embedding
constexpr unsigned TABLE_POSITIONS = 512, TABLE_HEAD_DIM = 64, TABLE_PAIRS = 32;
constexpr float TABLE_THETA = 10000.0f;

struct rope_params {
    size_t tokens;
    unsigned heads, head_dim, n_dims, interleaved;
    float freq_scale, sin_sign;
    int use_table;
};

__device__ __forceinline__ void rope_cos_sin(const rope_params &p, const float *table, unsigned pair, int pos, float *c, float *s)
{
    if (p.use_table && pos >= 0 && (unsigned)pos < TABLE_POSITIONS && pair < TABLE_PAIRS) {
        const float2 cs = __ldg(reinterpret_cast<const float2 *>(table) + (size_t)pos * TABLE_PAIRS + pair);
        *c = cs.x;
        *s = cs.y * p.sin_sign;
        return;
    }
    const float angle = (float)pos * exp2f((float)pair * p.freq_scale);
    float sv, cv;
    sincosf(angle, &sv, &cv);
    *c = cv;
    *s = sv * p.sin_sign;
}
// The rotated pair (x0, x1) -> (x0 c - x1 s, x0 s + x1 c).
__device__ __forceinline__ float rope_lo(float x0, float x1, float c, float s) { return x0 * c - x1 * s; }
__device__ __forceinline__ float rope_hi(float x0, float x1, float c, float s) { return x0 * s + x1 * c; }

// ------------------------------------------------------------------ packed storage pairs
// Two storage elements in one 32-bit word. add() is the packed storage-precision add: for operands of the storage type it
// returns round(a + b) exactly as an FP32 add followed by the rounding store does (the FP32 sum of two 11-bit or 8-bit
// significands is rounded once more to the same result: 24 >= 2 p + 2).
template <typename T> struct pack2;
template <> struct pack2<__half> {
    static __device__ __forceinline__ float2 up(uint32_t w) { return __half22float2(*reinterpret_cast<const __half2 *>(&w)); }
    static __device__ __forceinline__ uint32_t down(float a, float b)
    {
        const __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<const uint32_t *>(&h);
    }
    static __device__ __forceinline__ uint32_t add(uint32_t a, uint32_t b)
    {
        const __half2 r = __hadd2(*reinterpret_cast<const __half2 *>(&a), *reinterpret_cast<const __half2 *>(&b));
        return *reinterpret_cast<const uint32_t *>(&r);
    }
};
template <> struct pack2<__nv_bfloat16> {
    static __device__ __forceinline__ float2 up(uint32_t w) { return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000U)); }
    static __device__ __forceinline__ uint32_t down(float a, float b)
    {
        const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<const uint32_t *>(&h);
    }
    static __device__ __forceinline__ uint32_t add(uint32_t a, uint32_t b)
    {
        const float2 x = up(a), y = up(b);
        return down(x.x + y.x, x.y + y.y);
    }
};
// The 8 elements of a 16-byte vector as floats.
template <typename T>
__device__ __forceinline__ void unpack8(const uint4 &raw, float (&f)[8])
{
    const float2 a = pack2<T>::up(raw.x), b = pack2<T>::up(raw.y), c = pack2<T>::up(raw.z), d = pack2<T>::up(raw.w);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}

// ------------------------------------------------------------------ split-K decode attention
struct decode_params {
    int batch, tq, tmax, hq, hkv, dh;
    int window, prefix;
    int pos_mode;  // 0 scalar argument, 1 one-element tensor, 2 per-batch tensor
    int cache_pos;
    float scale;
};

__device__ __forceinline__ bool mask_allowed(int i, int j, int causal, int window, int prefix)
{
    if (causal != 0) {
        if (prefix > 0) {
            if (i < prefix) {
                if (j >= prefix) return false;
            } else if (j > i) {
                return false;
            }
        } else if (j > i) {
            return false;
        }
    }
    if (window > 0) {
        if (prefix > 0) {
            if (i >= prefix && j >= prefix && (i - j) >= window) return false;
        } else if ((i - j) >= window) {
            return false;
        }
    }
    return true;
}
__device__ __forceinline__ bool decode_allowed(int qpos, int j, int window, int prefix)
{
    return mask_allowed(qpos, j, 1, window, prefix);
}

// Number of key splits per query. One new token per sequence, head_dim 64 and at most 64 sequences (the shapes the
// persistent decode kernel takes): the 16 warps of a CTA are `heads_per_cta` heads x `splits` key ranges of ONE sequence,
// merged through shared memory; heads_per_cta is the smallest power of two (dividing hq, at most 16) that still gives every
// CTA a unit, batch * hq / heads_per_cta <= sm_count, else the largest. Other shapes: as many splits as keep
// `warps_per_sm` warps per SM busy, at least 32 keys of the cache per split, at most 16.
static inline int decode_heads_per_cta(int sm_count, int batch, int hq)
{
    int largest = 0, chosen = 0;
    for (int hg = 16; hg >= 1; hg >>= 1) {
        if (hg > hq || (hq % hg) != 0) continue;
        if (largest == 0) largest = hg;
        if ((long long)batch * (hq / hg) > sm_count) break;
        chosen = hg;
    }
    return chosen != 0 ? chosen : largest;
}
static inline int decode_choose_splits(int sm_count, int batch, int tq, int hq, int dh, int tmax, int warps_per_sm)
{
    if (tq == 1 && dh == 64 && batch <= 64) {
        return 16 / decode_heads_per_cta(sm_count, batch, hq);
    }
    const long long total_queries = (long long)batch * tq * hq;
    int splits = (int)(((long long)sm_count * warps_per_sm) / total_queries);
    const int max_splits = (tmax + 31) / 32;
    if (splits > max_splits) splits = max_splits;
    if (splits < 1) splits = 1;
    if (splits > 16) splits = 16;
    return splits;
}

// Merge of the per-split partials of one query: out = sum_s acc_s e^(m_s - m) / sum_s l_s e^(m_s - m). `ml` [splits, 2] and
// `acc` [splits, dh] are the query's partials, `out` its dh outputs. GLOBAL: the partials were written by other CTAs
// (L2 loads); otherwise they lie in shared memory.
template <typename T, bool GLOBAL>
__device__ __forceinline__ void decode_combine_query(const float *ml, const float *acc, T *out, int dh, int splits, int lane)
{
    auto ld = [](const float *p) { return GLOBAL ? __ldcg(p) : *p; };
    float m = -INFINITY;
    for (int s = 0; s < splits; ++s) m = fmaxf(m, ld(&ml[s * 2]));
    float l = 0.0f;
    for (int s = 0; s < splits; ++s) {
        const float pm = ld(&ml[s * 2]);
        l += pm == -INFINITY ? 0.0f : ld(&ml[s * 2 + 1]) * __expf(pm - m);
    }
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
    for (int c = lane; c < dh; c += 32) {
        float a = 0.0f;
        for (int s = 0; s < splits; ++s) {
            const float pm = ld(&ml[s * 2]);
            if (pm != -INFINITY) a += ld(&acc[(size_t)s * dh + c]) * __expf(pm - m);
        }
        gdb_io<T>::st(out, (size_t)c, a * inv);
    }
}

// One warp: query w = (b, t, hq) against the keys of split `split` of its live range. A key is handled by DH / 16
// adjacent lanes (16 head dims = two 16-byte pieces each of K and V), so a warp takes 32 / (DH / 16) keys per group and
// two groups per tile, folded into the running (max, sum, acc) with one rescale per tile; the partial goes to
// ml_item [2] = (max, sum) and acc_item [DH] (global or shared memory).
// RING = false: a tile's loads go to registers and are consumed at once. RING = true (DH = 64): `ring` is 12 KB of
// shared memory owned by this warp, three tiles of 16 keys deep; the warp copies a tile with cp.async, 4 keys x 128
// contiguous bytes per instruction (full sectors), the 16-byte pieces of key k stored at piece ^ (k & 7) so that the
// lanes' reads hit distinct banks, and up to three tiles (48 keys) are in flight per warp with no register cost. Both
// variants fold the keys into (m, l, acc) with the same operations in the same order.
template <typename T, int DH, bool RING>
__device__ __forceinline__ void decode_split_item(const T *q, const T *kc, const T *vc, const int *pos_buf, float *ml_item, float *acc_item,
                                                  const decode_params &p, int splits, long long w, int split, int lane,
                                                  unsigned char *ring = nullptr)
{
    static_assert(!RING || DH == 64, "the shared-memory ring is laid out for head_dim 64");
    constexpr int LPK = DH / 16, KPW = 32 / LPK, TILE = 2 * KPW;
    const int sub = lane % LPK, kg = lane / LPK;
    const int h = (int)(w % p.hq);
    const int t = (int)((w / p.hq) % p.tq);
    const int b = (int)(w / ((long long)p.hq * p.tq));
    const int hk = h / (p.hq / p.hkv);
    const int pos = p.pos_mode == 0 ? p.cache_pos : pos_buf[p.pos_mode == 2 ? b : 0];
    float m = -INFINITY, l = 0.0f;
    float acc[16], qr[16];
#pragma unroll
    for (int c = 0; c < 16; ++c) acc[c] = 0.0f;
    // one tile = two groups of keys: both scores, ONE running-max update, both keys folded into (l, acc)
    auto fold2 = [&](const bool (&valid)[2], const uint4 (&k0)[2], const uint4 (&k1)[2], const uint4 (&v0)[2], const uint4 (&v1)[2]) {
        float s[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            s[u] = 0.0f;
            if (valid[u]) {
                float ka[8], kb[8];
                unpack8<T>(k0[u], ka);
                unpack8<T>(k1[u], kb);
#pragma unroll
                for (int e = 0; e < 8; ++e) s[u] = fmaf(qr[e], ka[e], s[u]);
#pragma unroll
                for (int e = 0; e < 8; ++e) s[u] = fmaf(qr[8 + e], kb[e], s[u]);
            }
        }
#pragma unroll
        for (int o = 1; o < LPK; o <<= 1) {
            s[0] += __shfl_xor_sync(0xffffffffU, s[0], o);
            s[1] += __shfl_xor_sync(0xffffffffU, s[1], o);
        }
        const float s0 = valid[0] ? s[0] : -INFINITY, s1 = valid[1] ? s[1] : -INFINITY;
        const float mnew = fmaxf(m, fmaxf(s0, s1));
        if (mnew != -INFINITY) {
            const float corr = __expf(m - mnew), e0 = __expf(s0 - mnew), e1 = __expf(s1 - mnew);   // exp(-inf) = 0
            l = l * corr + e0 + e1;
            float va[8], vb[8];
            if (valid[0]) {
                unpack8<T>(v0[0], va);
                unpack8<T>(v1[0], vb);
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    acc[c] = fmaf(e0, va[c], acc[c] * corr);
                    acc[8 + c] = fmaf(e0, vb[c], acc[8 + c] * corr);
                }
            } else {
#pragma unroll
                for (int c = 0; c < 16; ++c) acc[c] *= corr;
            }
            if (valid[1]) {
                unpack8<T>(v0[1], va);
                unpack8<T>(v1[1], vb);
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    acc[c] = fmaf(e1, va[c], acc[c]);
                    acc[8 + c] = fmaf(e1, vb[c], acc[8 + c]);
                }
            }
            m = mnew;
        }
    };
    if (pos >= 0) {
        int live = pos + p.tq;
        if (live > p.tmax) live = p.tmax;
        const int qpos = pos + t;
        int j_hi = qpos + 1;
        if (p.prefix > 0 && qpos < p.prefix) j_hi = p.prefix;
        if (j_hi > live) j_hi = live;
        int j_lo = 0;
        if (p.window > 0 && p.prefix <= 0 && qpos - p.window + 1 > 0) j_lo = qpos - p.window + 1;
        const int span = j_hi > j_lo ? j_hi - j_lo : 0;
        const int chunk = (span + splits - 1) / splits;
        const int s_lo = j_lo + split * chunk;
        int s_hi = s_lo + chunk;
        if (s_hi > j_hi) s_hi = j_hi;
        const size_t qb = (((size_t)b * p.tq + t) * p.hq + h) * DH + sub * 16;
        auto key_valid = [&](int j) { return j < s_hi && decode_allowed(qpos, j, p.window, p.prefix); };
        if (RING) {
            const int n_tiles = s_hi > s_lo ? (s_hi - s_lo + TILE - 1) / TILE : 0;
            const size_t head_base = ((size_t)b * p.tmax * p.hkv + hk) * DH;    // + j * hkv * DH per key
            const int piece = lane & 7, krow = lane >> 3;                       // copy: lane -> (key within a group of 4, 16-byte piece)
            auto issue = [&](int tile, int slot) {
                if (tile < n_tiles) {
                    unsigned char *base = ring + (size_t)slot * 4096U;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int kl = i * 4 + krow, j = s_lo + tile * TILE + kl;
                        if (j < s_hi) {
                            const size_t src = head_base + (size_t)j * p.hkv * DH + (size_t)piece * 8U;
                            unsigned char *dst = base + kl * 128 + ((piece ^ (kl & 7)) << 4);
                            sk_cp16(dst, kc + src, true);
                            sk_cp16(dst + 2048, vc + src, true);
                        }
                    }
                }
                asm volatile("cp.async.commit_group;" ::: "memory");
            };
            issue(0, 0);
            issue(1, 1);
            issue(2, 2);
#pragma unroll
            for (int c = 0; c < 16; ++c) qr[c] = gdb_io<T>::ld(q, qb + c) * p.scale;
            int slot = 0;
            for (int tile = 0; tile < n_tiles; ++tile) {
                asm volatile("cp.async.wait_group 2;" ::: "memory");
                __syncwarp();   // every lane's copies of this tile have landed
                const int jb = s_lo + tile * TILE;
                const unsigned char *base = ring + (size_t)slot * 4096U;
                bool valid[2];
                uint4 k0[2], k1[2], v0[2], v1[2];
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const int kl = u * KPW + kg;
                    valid[u] = key_valid(jb + kl);
                    if (valid[u]) {
                        const unsigned char *row = base + kl * 128;
                        const int p0 = ((sub * 2) ^ (kl & 7)) << 4, p1 = ((sub * 2 + 1) ^ (kl & 7)) << 4;
                        k0[u] = *reinterpret_cast<const uint4 *>(row + p0);
                        k1[u] = *reinterpret_cast<const uint4 *>(row + p1);
                        v0[u] = *reinterpret_cast<const uint4 *>(row + 2048 + p0);
                        v1[u] = *reinterpret_cast<const uint4 *>(row + 2048 + p1);
                    }
                }
                fold2(valid, k0, k1, v0, v1);
                __syncwarp();   // every lane is done with the slot before it is refilled
                issue(tile + 3, slot);
                slot = slot == 2 ? 0 : slot + 1;
            }
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        } else {
            auto key_base = [&](int j) { return (((size_t)b * p.tmax + (size_t)j) * p.hkv + hk) * DH + sub * 16; };
#pragma unroll
            for (int c = 0; c < 16; ++c) qr[c] = gdb_io<T>::ld(q, qb + c) * p.scale;
            for (int jb = s_lo; jb < s_hi; jb += TILE) {
                uint4 k0[2], k1[2], v0[2], v1[2];
                bool valid[2];
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const int j = jb + u * KPW + kg;
                    valid[u] = key_valid(j);
                    if (valid[u]) {
                        const size_t kb = key_base(j);
                        k0[u] = *reinterpret_cast<const uint4 *>(kc + kb);
                        k1[u] = *reinterpret_cast<const uint4 *>(kc + kb + 8);
                        v0[u] = *reinterpret_cast<const uint4 *>(vc + kb);
                        v1[u] = *reinterpret_cast<const uint4 *>(vc + kb + 8);
                    }
                }
                fold2(valid, k0, k1, v0, v1);
            }
        }
    }
    // merge the key groups of the warp (lanes with equal `sub`)
    float wm = m;
#pragma unroll
    for (int o = LPK; o < 32; o <<= 1) wm = fmaxf(wm, __shfl_xor_sync(0xffffffffU, wm, o));
    const float f = (m == -INFINITY) ? 0.0f : __expf(m - wm);
    l *= f;
#pragma unroll
    for (int o = LPK; o < 32; o <<= 1) l += __shfl_xor_sync(0xffffffffU, l, o);
    float *pa = acc_item + sub * 16;
#pragma unroll
    for (int c = 0; c < 16; ++c) {
        float a = acc[c] * f;
#pragma unroll
        for (int o = LPK; o < 32; o <<= 1) a += __shfl_xor_sync(0xffffffffU, a, o);
        if (kg == 0) pa[c] = a;
    }
    if (lane == 0) {
        ml_item[0] = wm;
        ml_item[1] = l;
    }
}

// ------------------------------------------------------------------ greedy sampling
// One block per row: soft cap, non-finite -> -inf, first maximum wins (gpt_sample_next_token,
// examples/gpt_lm/gpt_lm_shared.c:1388-1398). Returns the winner to thread 0 (index 0 when nothing is finite);
// `sv` / `si` are 32-entry shared arrays. Every thread of the block must call it.
template <typename T>
__device__ __forceinline__ int32_t argmax_row(const T *x, uint32_t classes, float softcap, float *sv, uint32_t *si)
{
    float best = -INFINITY;
    uint32_t best_i = 0xFFFFFFFFU;
    for (uint32_t i = threadIdx.x; i < classes; i += blockDim.x) {
        float v = gdb_io<T>::ld(x, i);
        if (softcap > 0.0f) v = softcap * tanhf(v / softcap);
        if (!isfinite(v)) v = -INFINITY;
        if (v > best || best_i == 0xFFFFFFFFU) {   // strided scan visits indices in increasing order
            best = v;
            best_i = i;
        }
    }
    auto merge = [](float &a, uint32_t &ai, float b, uint32_t bi) {
        if (bi != 0xFFFFFFFFU && (ai == 0xFFFFFFFFU || b > a || (b == a && bi < ai))) {
            a = b;
            ai = bi;
        }
    };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffU, best, o);
        const uint32_t oi = __shfl_xor_sync(0xffffffffU, best_i, o);
        merge(best, best_i, ob, oi);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    if (lane == 0) {
        sv[warp] = best;
        si[warp] = best_i;
    }
    __syncthreads();
    if (warp == 0) {
        best = lane < nw ? sv[lane] : -INFINITY;
        best_i = lane < nw ? si[lane] : 0xFFFFFFFFU;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffU, best, o);
            const uint32_t oi = __shfl_xor_sync(0xffffffffU, best_i, o);
            merge(best, best_i, ob, oi);
        }
    }
    return best_i == 0xFFFFFFFFU ? 0 : (int32_t)best_i;
}

}  // namespace gdb_dec

// ------------------------------------------------------------------ persistent whole-step decode kernel (decode_mega.cu)
constexpr int GDB_MEGA_MAX_LAYERS = 16;
// Per-layer weights in the order of the model's parameter list: norm1 w, Wqkv [3D, D], bqkv, Wo [D, D], bo, norm2 w,
// Wupgate [2F, D], bupgate, Wdown [F, D], bdown.
struct gdb_mega_args {
    const void *emb, *w_final, *w_lm, *b_lm;
    const void *lw[GDB_MEGA_MAX_LAYERS][10];
    void *kc[GDB_MEGA_MAX_LAYERS], *vc[GDB_MEGA_MAX_LAYERS];
    int B, D, F, V, H, L, CAP, window, splits, max_steps, n_steps;
    float eps, scale, softcap;
    gdb_dec::rope_params rope;
    const float *rope_table;
    void *xbuf, *resid, *q, *attn, *act, *logits;                // activations of one step, [B, D | F | V]
    unsigned *sync;                                               // [0] barrier counter (bit 31: abort)
    int32_t *tokens, *positions, *out_tokens, *step_counter;
    int *err_flag;
    unsigned long long *timeline;   // diagnostic (NULL = off): global timer of CTA 0 after every barrier, [n_steps, 5 L + 2]
};
// Shapes the persistent kernel takes (everything else runs as one launch per operation).
bool gdb_decode_mega_supported(const gd_backend *be, uint32_t dtype, int B, int D, int F, int V, int H, int Dh, int L);
// n_steps decode steps in ONE cooperative launch. a->sync must be zeroed by the caller (stream-ordered) before the launch.
gd_status gdb_decode_mega_launch(gd_backend *be, uint32_t dtype, const gdb_mega_args *a);
gd_status gdb_rope_params_for_decode(gd_backend *be, uint32_t n_heads, uint32_t head_dim, const gd_backend_rope_args *args, size_t tokens,
                                     gdb_dec::rope_params *out);

#endif  // GDB200_DECODE_PARTS_CUH
