// RMSNorm forward / backward / weight-gradient kernels (HBM-bound, one warp per row).
//
// Reference arithmetic: src/ops/rms_norm/metal_rms_norm.metal:29-608
//   inv  = rsqrt(mean(x^2) + eps)                         (:59)
//   out  = x * w * inv                                    (:64)
//   dx   = inv * g * w - x * inv^3 / cols * sum(g * w * x) (:249-262)
//   dw   = sum_rows g * x * inv, via FP32 partials [row_blocks, cols] (:414-447, :554-580)
// The simdgroup counts in gd_backend_rms_norm_args describe the Metal launch and are ignored.
#include "common.cuh"
#include "colreduce.cuh"

namespace {

constexpr int ROWS_PER_BLOCK = 4;  // 4 warps per block, one row each


// MODE 0: out only; MODE 1: out + inv; MODE 2: inv only.
template <typename T, int MODE>
__global__ void rms_fwd_kernel(const T *x, const T *w, T *out, float *inv_out, size_t rows, size_t cols, float eps)
{
    gdb_pdl_sync();
    const int lane = threadIdx.x & 31;
    const size_t row = (size_t)blockIdx.x * ROWS_PER_BLOCK + (threadIdx.x >> 5);
    if (row >= rows) {
        return;
    }
    const T *xr = x + row * cols;
    float ss = 0.0f;
    bool vec = false;
    if constexpr (sizeof(T) == 2) {
        vec = (cols % 8U) == 0U && ((uintptr_t)xr % 16U) == 0U &&
              (MODE == 2 || (((uintptr_t)(out + row * cols) | (uintptr_t)w) % 16U) == 0U);
        if (vec) {
            const uint4 *xv = reinterpret_cast<const uint4 *>(xr);
            for (size_t v = lane; v < cols / 8U; v += 32) {
                gdb_vec8<T> a;
                a.raw = xv[v];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float f = a.get(e);
                    ss += f * f;
                }
            }
        }
    }
    if (!vec) {
        for (size_t c = lane; c < cols; c += 32) {
            const float f = gdb_io<T>::ld(xr, c);
            ss += f * f;
        }
    }
    ss = gdb_warp_sum(ss);
    const float inv = rsqrtf(ss / (float)cols + eps);
    if (MODE != 0 && lane == 0) {
        inv_out[row] = inv;
    }
    if (MODE == 2) {
        return;
    }
    T *orow = out + row * cols;
    if constexpr (sizeof(T) == 2) {
        if (vec) {
            const uint4 *xv = reinterpret_cast<const uint4 *>(xr);
            const uint4 *wv = reinterpret_cast<const uint4 *>(w);
            uint4 *ov = reinterpret_cast<uint4 *>(orow);
            for (size_t v = lane; v < cols / 8U; v += 32) {
                gdb_vec8<T> a, b;
                a.raw = xv[v];
                b.raw = __ldg(&wv[v]);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    a.set(e, a.get(e) * b.get(e) * inv);
                }
                ov[v] = a.raw;
            }
            return;
        }
    }
    for (size_t c = lane; c < cols; c += 32) {
        gdb_io<T>::st(orow, c, gdb_io<T>::ld(xr, c) * gdb_io<T>::ld(w, c) * inv);
    }
}

// sum = round(x + y); out = round(sum * w * inv_rms(sum)): gd_backend_add followed by rms_norm_forward in one launch
// (same rounding points). Warp per row, cols % 8 == 0, 16-byte aligned 16-bit tensors.
// DROP: y goes through inverted dropout first (round(y * scale) or 0, decision per element index, mask bytes written),
// i.e. gd_backend_dropout_add_forward; inv_out != NULL saves 1 / rms per row (rms_norm_forward_stats).
// GATHER (with DROP): there is no residual; y is an embedding table [vocab, cols] and row r of the input is table row ids[r] (NaN
// for an id outside the table), so sum = dropout(embedding(ids)): gd_backend_embedding_forward, gd_backend_dropout_forward and
// gd_backend_rms_norm_forward_stats in one launch.
template <typename T, bool DROP, bool GATHER = false>
__global__ void add_rms_fwd_kernel(const uint4 *x, const uint4 *y, const uint4 *w, uint4 *sum, uint4 *out, size_t rows, size_t cols, float eps,
                                   uint2 *mask_out, float *inv_out, float scale, uint64_t seed, unsigned threshold, const int *ids = nullptr,
                                   size_t vocab = 0, unsigned nan_word = 0)
{
    gdb_pdl_sync();
    const int lane = threadIdx.x & 31;
    const size_t row = (size_t)blockIdx.x * ROWS_PER_BLOCK + (threadIdx.x >> 5);
    if (row >= rows) {
        return;
    }
    const size_t vecs = cols / 8U, base = row * vecs;
    int id = 0;
    if (GATHER) id = __ldg(&ids[row]);
    const bool in_table = !GATHER || (id >= 0 && (size_t)id < vocab);
    float ss = 0.0f;
    if (vecs <= 64U) {
        // rows of up to 512 elements: the lane's two vectors of the sum stay in registers between the two passes and all four
        // loads are in flight together (same arithmetic, element for element, as the general loop below)
        gdb_vec8<T> a[2], b[2], wv[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const size_t v = (size_t)lane + 32U * (size_t)i;
            if (v < vecs) {
                if (GATHER) {
                    b[i].raw = in_table ? __ldg(&y[(size_t)id * vecs + v]) : make_uint4(nan_word, nan_word, nan_word, nan_word);
                } else {
                    a[i].raw = x[base + v];
                    b[i].raw = y[base + v];
                }
                wv[i].raw = __ldg(&w[v]);
            }
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const size_t v = (size_t)lane + 32U * (size_t)i;
            if (v < vecs) {
                uint2 m = make_uint2(0U, 0U);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    float add = b[i].get(e);
                    if (DROP) {
                        const bool keep = gdb_dropout_keep(seed, (uint64_t)(base + v) * 8U + (uint64_t)e, threshold);
                        unsigned *mw = e < 4 ? &m.x : &m.y;
                        *mw |= (keep ? 1U : 0U) << (8U * (unsigned)(e & 3));
                        add = keep ? gdb_io<T>::rnd(add * scale) : 0.0f;
                    }
                    a[i].set(e, GATHER ? add : a[i].get(e) + add);
                    const float f = a[i].get(e);
                    ss += f * f;
                }
                sum[base + v] = a[i].raw;
                if (DROP) mask_out[base + v] = m;
            }
        }
        ss = gdb_warp_sum(ss);
        const float inv = rsqrtf(ss / (float)cols + eps);
        if (inv_out != nullptr && lane == 0) inv_out[row] = inv;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const size_t v = (size_t)lane + 32U * (size_t)i;
            if (v < vecs) {
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    a[i].set(e, a[i].get(e) * wv[i].get(e) * inv);
                }
                out[base + v] = a[i].raw;
            }
        }
        return;
    }
    for (size_t v = lane; v < vecs; v += 32) {
        gdb_vec8<T> a, b;
        if (GATHER) {
            b.raw = in_table ? __ldg(&y[(size_t)id * vecs + v]) : make_uint4(nan_word, nan_word, nan_word, nan_word);
        } else {
            a.raw = x[base + v];
            b.raw = y[base + v];
        }
        uint2 m = make_uint2(0U, 0U);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            float add = b.get(e);
            if (DROP) {
                const bool keep = gdb_dropout_keep(seed, (uint64_t)(base + v) * 8U + (uint64_t)e, threshold);
                unsigned *mw = e < 4 ? &m.x : &m.y;
                *mw |= (keep ? 1U : 0U) << (8U * (unsigned)(e & 3));
                add = keep ? gdb_io<T>::rnd(add * scale) : 0.0f;
            }
            a.set(e, GATHER ? add : a.get(e) + add);
            const float f = a.get(e);
            ss += f * f;
        }
        sum[base + v] = a.raw;
        if (DROP) mask_out[base + v] = m;
    }
    ss = gdb_warp_sum(ss);
    const float inv = rsqrtf(ss / (float)cols + eps);
    if (inv_out != nullptr && lane == 0) inv_out[row] = inv;
    for (size_t v = lane; v < vecs; v += 32) {
        gdb_vec8<T> a, b;
        a.raw = sum[base + v];   // written by this lane above
        b.raw = __ldg(&w[v]);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            a.set(e, a.get(e) * b.get(e) * inv);
        }
        out[base + v] = a.raw;
    }
}

// STATS true: inv read from inv_in; false: recomputed from x.
template <typename T, bool STATS>
__global__ void rms_bwd_kernel(const T *x, const T *w, const float *inv_in, const T *g, T *dx, size_t rows, size_t cols, float eps, bool add_to_dx)
{
    gdb_pdl_sync();
    const int lane = threadIdx.x & 31;
    const size_t row = (size_t)blockIdx.x * ROWS_PER_BLOCK + (threadIdx.x >> 5);
    if (row >= rows) {
        return;
    }
    const T *xr = x + row * cols, *gr = g + row * cols;
    T *dr = dx + row * cols;
    float a = 0.0f, ss = 0.0f;
    bool vec = false;
    if constexpr (sizeof(T) == 2) {
        vec = (cols % 8U) == 0U && (((uintptr_t)xr | (uintptr_t)gr | (uintptr_t)dr | (uintptr_t)w) % 16U) == 0U;
        if (vec) {
            const uint4 *xv = reinterpret_cast<const uint4 *>(xr), *gv = reinterpret_cast<const uint4 *>(gr);
            const uint4 *wv = reinterpret_cast<const uint4 *>(w);
            for (size_t v = lane; v < cols / 8U; v += 32) {
                gdb_vec8<T> xa, ga, wa;
                xa.raw = xv[v];
                ga.raw = gv[v];
                wa.raw = __ldg(&wv[v]);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float xf = xa.get(e);
                    a += ga.get(e) * wa.get(e) * xf;
                    ss += xf * xf;
                }
            }
        }
    }
    if (!vec) {
        for (size_t c = lane; c < cols; c += 32) {
            const float xf = gdb_io<T>::ld(xr, c);
            a += gdb_io<T>::ld(gr, c) * gdb_io<T>::ld(w, c) * xf;
            ss += xf * xf;
        }
    }
    a = gdb_warp_sum(a);
    float inv;
    if (STATS) {
        inv = inv_in[row];
    } else {
        ss = gdb_warp_sum(ss);
        inv = rsqrtf(ss / (float)cols + eps);
    }
    const float k = inv * inv * inv / (float)cols;
    if constexpr (sizeof(T) == 2) {
        if (vec) {
            const uint4 *xv = reinterpret_cast<const uint4 *>(xr), *gv = reinterpret_cast<const uint4 *>(gr);
            const uint4 *wv = reinterpret_cast<const uint4 *>(w);
            uint4 *dv = reinterpret_cast<uint4 *>(dr);
            for (size_t v = lane; v < cols / 8U; v += 32) {
                gdb_vec8<T> xa, ga, wa;
                xa.raw = xv[v];
                ga.raw = gv[v];
                wa.raw = __ldg(&wv[v]);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    ga.set(e, inv * ga.get(e) * wa.get(e) - xa.get(e) * k * a);
                }
                if (add_to_dx) {
                    // dx += rounded gradient, rounded again: rms_norm_backward followed by gd_backend_accumulate, in place
                    gdb_vec8<T> da;
                    da.raw = dv[v];
#pragma unroll
                    for (int e = 0; e < 8; ++e) ga.set(e, da.get(e) + ga.get(e));
                }
                dv[v] = ga.raw;
            }
            return;
        }
    }
    for (size_t c = lane; c < cols; c += 32) {
        const float val = inv * gdb_io<T>::ld(gr, c) * gdb_io<T>::ld(w, c) - gdb_io<T>::ld(xr, c) * k * a;
        gdb_io<T>::st(dr, c, add_to_dx ? gdb_io<T>::ld(dr, c) + gdb_io<T>::rnd(val) : val);
    }
}

// Input gradient AND weight gradient of RMSNorm from one pass over x and g (rms_norm_backward_stats [+ accumulate] and
// rms_norm_weight_backward_stats in one launch): 16-bit storage, cols <= 512 and a multiple of 8, 16-byte aligned rows.
// One block of 16 warps per SM. A warp takes rows blockIdx.x * 16 + warp, + gridDim.x * 16, ... and streams them through
// a private shared-memory ring three rows deep: every lane copies its own 16-byte pieces of x, g (and of dx when the
// gradient is accumulated) with cp.async and reads them back itself, so two rows per warp (96 KB per SM) are in flight
// while one is consumed, with no register cost and no synchronisation between lanes. The lane accumulates g * x * inv of
// its 16 columns over its rows; the warps of a block are summed through shared memory into partial[blockIdx.x, cols]
// (FP32), and the block that arrives last (ticket) sums the blocks' partials in block order and rounds dw once, so the
// result does not depend on which block was last. dx is computed exactly as rms_bwd_kernel does.
constexpr int RBW_WARPS = 16, RBW_MAX_COLS = 512, RBW_DEPTH = 3;
constexpr int RBW_ROW_BYTES = RBW_MAX_COLS * 2;                          // one 16-bit row
constexpr int RBW_MASK_BYTES = RBW_MAX_COLS;                             // one byte per element of a dropout mask row
constexpr int RBW_SLOT_BYTES = 3 * RBW_ROW_BYTES + RBW_MASK_BYTES;       // x, g, dx, mask
constexpr int RBW_SMEM = RBW_WARPS * RBW_DEPTH * RBW_SLOT_BYTES;         // 168 KB; the block reduction reuses it
static_assert(RBW_SMEM >= (int)sizeof(float) * RBW_WARPS * RBW_MAX_COLS, "the reduction buffer aliases the rings");
template <typename T>
__global__ void __launch_bounds__(RBW_WARPS * 32, 1)
rms_bwd_wgrad_kernel(const T *__restrict__ x, const T *__restrict__ w, const float *__restrict__ inv_in, const T *__restrict__ g, T *dx,
                     T *__restrict__ dw, float *__restrict__ partial, unsigned *__restrict__ ticket, size_t rows, size_t cols, bool add_to_dx,
                     const unsigned char *__restrict__ mask, T *__restrict__ masked, float mask_scale, T *__restrict__ masked_colsum)
{
    // masked_colsum != nullptr (with mask): masked_colsum[c] = sum over rows of masked[:, c] as well, the bias gradient of the
    // projection whose output the dropped branch is (reduce_rows of the same tensor); its partial sums use the second half of `partial`.
    // mask != nullptr: masked = dropout_backward_mask(mask, dx, mask_scale) as well, i.e. the gradient that flows into the
    // dropped branch next to the residual one, formed from the stored (rounded) dx as the separate entry would read it.
    gdb_pdl_sync();
    extern __shared__ __align__(16) unsigned char rbw_sm[];
    __shared__ bool last;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const size_t vecs = cols / 8U;
    unsigned char *ring = rbw_sm + (size_t)warp * RBW_DEPTH * RBW_SLOT_BYTES;
    float dwacc[2][8], wf[2][8], csacc[2][8];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
#pragma unroll
        for (int e = 0; e < 8; ++e) dwacc[i][e] = csacc[i][e] = 0.0f;
        const size_t v = (size_t)lane + 32U * (size_t)i;
        gdb_vec8<T> wa;
        wa.raw = v < vecs ? __ldg(reinterpret_cast<const uint4 *>(w) + v) : make_uint4(0U, 0U, 0U, 0U);
#pragma unroll
        for (int e = 0; e < 8; ++e) wf[i][e] = wa.get(e);
    }
    const size_t row0 = (size_t)blockIdx.x * RBW_WARPS + warp, stride = (size_t)gridDim.x * RBW_WARPS;
    auto cp16 = [](void *dst, const void *src) {
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
    };
    auto cp8 = [](void *dst, const void *src) {
        asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
    };
    auto issue = [&](size_t row, int slot) {
        if (row < rows) {
            unsigned char *base = ring + (size_t)slot * RBW_SLOT_BYTES;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const size_t v = (size_t)lane + 32U * (size_t)i;
                if (v < vecs) {
                    cp16(base + v * 16U, reinterpret_cast<const uint4 *>(x + row * cols) + v);
                    cp16(base + RBW_ROW_BYTES + v * 16U, reinterpret_cast<const uint4 *>(g + row * cols) + v);
                    if (add_to_dx) cp16(base + 2 * RBW_ROW_BYTES + v * 16U, reinterpret_cast<const uint4 *>(dx + row * cols) + v);
                    if (mask != nullptr) cp8(base + 3 * RBW_ROW_BYTES + v * 8U, reinterpret_cast<const uint2 *>(mask + row * cols) + v);
                }
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    issue(row0, 0);
    issue(row0 + stride, 1);
    int slot = 0;
    float inv_next = row0 < rows ? inv_in[row0] : 0.0f;   // 1 / rms of the row after this one, loaded a row ahead
    for (size_t row = row0; row < rows; row += stride) {
        issue(row + 2U * stride, slot == 0 ? 2 : slot - 1);   // the slot consumed one iteration ago
        const float inv = inv_next;
        if (row + stride < rows) inv_next = inv_in[row + stride];
        asm volatile("cp.async.wait_group 2;" ::: "memory");
        const unsigned char *base = ring + (size_t)slot * RBW_SLOT_BYTES;
        float xf[2][8], gf[2][8];   // x and g of the lane's 16 columns
        float a = 0.0f;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const size_t v = (size_t)lane + 32U * (size_t)i;
            if (v < vecs) {
                gdb_vec8<T> xa, ga;
                xa.raw = *reinterpret_cast<const uint4 *>(base + v * 16U);
                ga.raw = *reinterpret_cast<const uint4 *>(base + RBW_ROW_BYTES + v * 16U);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    xf[i][e] = xa.get(e);
                    gf[i][e] = ga.get(e);
                    a += gf[i][e] * wf[i][e] * xf[i][e];
                    dwacc[i][e] += gf[i][e] * xf[i][e] * inv;
                }
            }
        }
        a = gdb_warp_sum(a);
        const float k = inv * inv * inv / (float)cols;
        uint4 *dv = reinterpret_cast<uint4 *>(dx + row * cols);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const size_t v = (size_t)lane + 32U * (size_t)i;
            if (v < vecs) {
                gdb_vec8<T> o;
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    o.set(e, inv * gf[i][e] * wf[i][e] - xf[i][e] * k * a);
                }
                if (add_to_dx) {
                    // dx += rounded gradient, rounded again: rms_norm_backward followed by gd_backend_accumulate, in place
                    gdb_vec8<T> da;
                    da.raw = *reinterpret_cast<const uint4 *>(base + 2 * RBW_ROW_BYTES + v * 16U);
#pragma unroll
                    for (int e = 0; e < 8; ++e) o.set(e, da.get(e) + o.get(e));
                }
                dv[v] = o.raw;
                if (mask != nullptr) {
                    const uint2 m = *reinterpret_cast<const uint2 *>(base + 3 * RBW_ROW_BYTES + v * 8U);
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const bool keep = (((e < 4 ? m.x : m.y) >> (8U * (unsigned)(e & 3))) & 255U) != 0U;
                        o.set(e, keep ? o.get(e) * mask_scale : 0.0f);
                        csacc[i][e] += o.get(e);
                    }
                    reinterpret_cast<uint4 *>(masked + row * cols)[v] = o.raw;
                }
            }
        }
        slot = slot == RBW_DEPTH - 1 ? 0 : slot + 1;
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();   // every warp is done with its ring: the reduction buffer reuses the memory
    float(*sh)[RBW_MAX_COLS] = reinterpret_cast<float(*)[RBW_MAX_COLS]>(rbw_sm);
    // this block's column sums of the lanes' accumulators, warps added in warp order, into row `slab_row` of partial
    auto publish = [&](const float (&acc)[2][8], size_t slab_row) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const size_t v = (size_t)lane + 32U * (size_t)i;
            if (v < vecs) {
#pragma unroll
                for (int e = 0; e < 8; ++e) sh[warp][v * 8U + e] = acc[i][e];
            }
        }
        __syncthreads();
        for (size_t c = threadIdx.x; c < cols; c += blockDim.x) {
            float s = 0.0f;
#pragma unroll
            for (int wi = 0; wi < RBW_WARPS; ++wi) s += sh[wi][c];
            partial[slab_row * cols + c] = s;
        }
    };
    publish(dwacc, blockIdx.x);
    if (masked_colsum != nullptr) {
        __syncthreads();
        publish(csacc, (size_t)gridDim.x + blockIdx.x);
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) last = atomicAdd(ticket, 1U) == gridDim.x - 1U;
    __syncthreads();
    if (last) {
        __threadfence();
        auto merge = [&](const float *slab, T *out) {
            for (size_t c = threadIdx.x; c < cols; c += blockDim.x) {
                float s = 0.0f;
                unsigned b = 0;
                for (; b + 8U <= gridDim.x; b += 8U) {   // eight loads in flight, summed in block order
                    float t[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) t[u] = __ldcg(&slab[(size_t)(b + u) * cols + c]);
#pragma unroll
                    for (int u = 0; u < 8; ++u) s += t[u];
                }
                for (; b < gridDim.x; ++b) s += __ldcg(&slab[(size_t)b * cols + c]);
                gdb_io<T>::st(out, c, s);
            }
        };
        merge(partial, dw);
        if (masked_colsum != nullptr) merge(partial + (size_t)gridDim.x * cols, masked_colsum);
        if (threadIdx.x == 0) *ticket = 0U;
    }
}

// Stage 1 of dw: block (cb, rb) sums rows [rb*chunk, rb*chunk+chunk) of columns
// [cb*256, cb*256+256) into partial[rb, c]; thread t owns column cb*256+t, 4 rows in flight.
template <typename T>
__global__ void rms_wgrad_stage_kernel(const T *x, const float *inv, const T *g, float *partial,
                                       size_t rows, size_t cols, size_t chunk)
{
    gdb_pdl_sync();
    const size_t c = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t r0 = (size_t)blockIdx.y * chunk;
    size_t r1 = r0 + chunk;
    if (r1 > rows) {
        r1 = rows;
    }
    if (c >= cols) {
        return;
    }
    float acc0 = 0.0f, acc1 = 0.0f, acc2 = 0.0f, acc3 = 0.0f;
    size_t r = r0;
    for (; r + 4 <= r1; r += 4) {
        acc0 += gdb_io<T>::ld(g, (r + 0) * cols + c) * gdb_io<T>::ld(x, (r + 0) * cols + c) * __ldg(&inv[r + 0]);
        acc1 += gdb_io<T>::ld(g, (r + 1) * cols + c) * gdb_io<T>::ld(x, (r + 1) * cols + c) * __ldg(&inv[r + 1]);
        acc2 += gdb_io<T>::ld(g, (r + 2) * cols + c) * gdb_io<T>::ld(x, (r + 2) * cols + c) * __ldg(&inv[r + 2]);
        acc3 += gdb_io<T>::ld(g, (r + 3) * cols + c) * gdb_io<T>::ld(x, (r + 3) * cols + c) * __ldg(&inv[r + 3]);
    }
    for (; r < r1; ++r) {
        acc0 += gdb_io<T>::ld(g, r * cols + c) * gdb_io<T>::ld(x, r * cols + c) * __ldg(&inv[r]);
    }
    partial[(size_t)blockIdx.y * cols + c] = (acc0 + acc1) + (acc2 + acc3);
}

template <typename T>
__global__ void rms_wgrad_reduce_kernel(const float *partial, T *dw, size_t blocks, size_t cols)
{
    gdb_pdl_sync();
    const size_t c = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) {
        return;
    }
    float s = 0.0f;
    for (size_t b = 0; b < blocks; ++b) {
        s += partial[b * cols + c];
    }
    gdb_io<T>::st(dw, c, s);
}

bool args_ok(const gd_backend_rms_norm_args *a)
{
    return a != NULL && a->rows > 0U && a->cols > 0U && a->rows <= SIZE_MAX / a->cols && a->eps >= 0.0f;
}

template <typename T, int MODE>
gd_status fwd_launch(gd_backend *be, const void *x, const void *w, void *out, float *inv, const gd_backend_rms_norm_args *a)
{
    const unsigned grid = (unsigned)((a->rows + ROWS_PER_BLOCK - 1) / ROWS_PER_BLOCK);
    gdb_launch(rms_fwd_kernel<T, MODE>, grid, 32 * ROWS_PER_BLOCK, 0, be->stream, (const T *)x, (const T *)w, (T *)out, inv, a->rows, a->cols, a->eps);
    return gdb_launched(be, "rms_norm_forward");
}

template <int MODE>
gd_status fwd_dispatch(gd_backend *be, const gd_backend_tensor_view *x, const gd_backend_tensor_view *weight,
                       const gd_backend_tensor_view *out, const gd_backend_tensor_view *inv_rms,
                       const gd_backend_rms_norm_args *a)
{
    if (be == NULL || x == NULL || !args_ok(a) || x->count != a->rows * a->cols) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (!gdb_is_float_dtype(x->dtype)) {
        return GD_ERR_UNSUPPORTED;
    }
    const void *xp = gdb_tv_ptr(x, x->dtype), *wp = NULL;
    void *op = NULL;
    float *ip = NULL;
    if (MODE != 2) {
        if (weight == NULL || out == NULL || weight->count != a->cols || out->count != x->count) {
            return GD_ERR_INVALID_ARGUMENT;
        }
        wp = gdb_tv_ptr(weight, x->dtype);
        op = gdb_tv_ptr(out, x->dtype);
        if (wp == NULL || op == NULL) {
            return GD_ERR_INVALID_ARGUMENT;
        }
    }
    if (MODE != 0) {
        if (inv_rms == NULL || inv_rms->count != a->rows) {
            return GD_ERR_INVALID_ARGUMENT;
        }
        ip = (float *)gdb_tv_ptr(inv_rms, GDB_DTYPE_F32);
        if (ip == NULL) {
            return GD_ERR_INVALID_ARGUMENT;
        }
    }
    if (xp == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (x->dtype == GDB_DTYPE_F16) {
        return fwd_launch<__half, MODE>(be, xp, wp, op, ip, a);
    }
    if (x->dtype == GDB_DTYPE_BF16) {
        return fwd_launch<__nv_bfloat16, MODE>(be, xp, wp, op, ip, a);
    }
    return fwd_launch<float, MODE>(be, xp, wp, op, ip, a);
}

template <bool STATS>
gd_status bwd_dispatch(gd_backend *be, const gd_backend_tensor_view *x, const gd_backend_tensor_view *weight,
                       const gd_backend_tensor_view *inv_rms, const gd_backend_tensor_view *grad_out,
                       const gd_backend_tensor_view *grad_x, const gd_backend_rms_norm_args *a, bool add_to_dx = false)
{
    if (be == NULL || x == NULL || weight == NULL || grad_out == NULL || grad_x == NULL || !args_ok(a) ||
        x->count != a->rows * a->cols || weight->count != a->cols || grad_out->count != x->count ||
        grad_x->count != x->count || (STATS && (inv_rms == NULL || inv_rms->count != a->rows))) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (!gdb_is_float_dtype(x->dtype)) {
        return GD_ERR_UNSUPPORTED;
    }
    const void *xp = gdb_tv_ptr(x, x->dtype), *wp = gdb_tv_ptr(weight, x->dtype), *gp = gdb_tv_ptr(grad_out, x->dtype);
    void *dp = gdb_tv_ptr(grad_x, x->dtype);
    const float *ip = STATS ? (const float *)gdb_tv_ptr(inv_rms, GDB_DTYPE_F32) : NULL;
    if (xp == NULL || wp == NULL || gp == NULL || dp == NULL || (STATS && ip == NULL)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const unsigned grid = (unsigned)((a->rows + ROWS_PER_BLOCK - 1) / ROWS_PER_BLOCK);
    const unsigned threads = 32 * ROWS_PER_BLOCK;
    if (x->dtype == GDB_DTYPE_F16) {
        gdb_launch(rms_bwd_kernel<__half, STATS>, grid, threads, 0, be->stream, (const __half *)xp, (const __half *)wp, ip, (const __half *)gp, (__half *)dp, a->rows, a->cols, a->eps, add_to_dx);
    } else if (x->dtype == GDB_DTYPE_BF16) {
        gdb_launch(rms_bwd_kernel<__nv_bfloat16, STATS>, grid, threads, 0, be->stream, (const __nv_bfloat16 *)xp, (const __nv_bfloat16 *)wp, ip, (const __nv_bfloat16 *)gp, (__nv_bfloat16 *)dp, a->rows, a->cols, a->eps, add_to_dx);
    } else {
        gdb_launch(rms_bwd_kernel<float, STATS>, grid, threads, 0, be->stream, (const float *)xp, (const float *)wp, ip, (const float *)gp, (float *)dp, a->rows, a->cols, a->eps, add_to_dx);
    }
    return gdb_launched(be, "rms_norm_backward");
}

}  // namespace

extern "C" {

gd_status gd_backend_rms_norm_forward(gd_backend *be, const gd_backend_tensor_view *x, const gd_backend_tensor_view *weight, const gd_backend_tensor_view *out, const gd_backend_rms_norm_args *args)
{
    return fwd_dispatch<0>(be, x, weight, out, NULL, args);
}

gd_status gd_backend_rms_norm_forward_stats(gd_backend *be, const gd_backend_tensor_view *x, const gd_backend_tensor_view *weight, const gd_backend_tensor_view *out, const gd_backend_tensor_view *inv_rms, const gd_backend_rms_norm_args *args)
{
    return fwd_dispatch<1>(be, x, weight, out, inv_rms, args);
}

gd_status gd_backend_rms_norm_inv(gd_backend *be, const gd_backend_tensor_view *x, const gd_backend_tensor_view *inv_rms, const gd_backend_rms_norm_args *args)
{
    return fwd_dispatch<2>(be, x, NULL, NULL, inv_rms, args);
}

gd_status gd_backend_rms_norm_backward(gd_backend *be, const gd_backend_tensor_view *x, const gd_backend_tensor_view *weight, const gd_backend_tensor_view *grad_out, const gd_backend_tensor_view *grad_x, const gd_backend_rms_norm_args *args)
{
    return bwd_dispatch<false>(be, x, weight, NULL, grad_out, grad_x, args);
}

gd_status gd_backend_rms_norm_backward_stats(gd_backend *be, const gd_backend_tensor_view *x, const gd_backend_tensor_view *weight, const gd_backend_tensor_view *inv_rms, const gd_backend_tensor_view *grad_out, const gd_backend_tensor_view *grad_x, const gd_backend_rms_norm_args *args)
{
    return bwd_dispatch<true>(be, x, weight, inv_rms, grad_out, grad_x, args);
}

// The caller provides partial [row_blocks, cols] F32; its content is private to the backend.
// This implementation uses min(row_blocks, enough blocks for ~4 waves) row chunks.
gd_status gd_backend_rms_norm_weight_backward_stats(gd_backend *be, const gd_backend_tensor_view *x, const gd_backend_tensor_view *inv_rms, const gd_backend_tensor_view *grad_out, const gd_backend_tensor_view *grad_weight, const gd_backend_tensor_view *partial, const gd_backend_rms_norm_args *a)
{
    if (be == NULL || x == NULL || inv_rms == NULL || grad_out == NULL || grad_weight == NULL || partial == NULL ||
        !args_ok(a) || a->row_blocks == 0U || x->count != a->rows * a->cols || grad_out->count != x->count ||
        inv_rms->count != a->rows || grad_weight->count != a->cols || partial->count < a->row_blocks * a->cols) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (!gdb_is_float_dtype(x->dtype)) {
        return GD_ERR_UNSUPPORTED;
    }
    const void *xp = gdb_tv_ptr(x, x->dtype), *gp = gdb_tv_ptr(grad_out, x->dtype);
    const float *ip = (const float *)gdb_tv_ptr(inv_rms, GDB_DTYPE_F32);
    float *pp = (float *)gdb_tv_ptr(partial, GDB_DTYPE_F32);
    void *dw = gdb_tv_ptr(grad_weight, x->dtype);
    if (xp == NULL || gp == NULL || ip == NULL || pp == NULL || dw == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (x->dtype != GDB_DTYPE_F32 && gdb_colreduce::usable(gp, a->cols, xp, a->cols, a->cols)) {
        return x->dtype == GDB_DTYPE_F16
                   ? gdb_colreduce::run<__half, true>(be, gp, a->cols, xp, a->cols, ip, pp, a->row_blocks, dw, a->rows, a->cols)
                   : gdb_colreduce::run<__nv_bfloat16, true>(be, gp, a->cols, xp, a->cols, ip, pp, a->row_blocks, dw, a->rows, a->cols);
    }
    const unsigned col_blocks = (unsigned)((a->cols + 255U) / 256U);
    size_t blocks = a->row_blocks;
    const size_t want = ((size_t)be->sm_count * 8U + col_blocks - 1U) / col_blocks;
    if (blocks > want) {
        blocks = want;
    }
    if (blocks > 65535U) {
        blocks = 65535U;
    }
    const size_t chunk = (a->rows + blocks - 1U) / blocks;
    blocks = (a->rows + chunk - 1U) / chunk;
    dim3 grid(col_blocks, (unsigned)blocks);
    if (x->dtype == GDB_DTYPE_F16) {
        gdb_launch(rms_wgrad_stage_kernel<__half>, grid, 256, 0, be->stream, (const __half *)xp, ip, (const __half *)gp, pp, a->rows, a->cols, chunk);
    } else if (x->dtype == GDB_DTYPE_BF16) {
        gdb_launch(rms_wgrad_stage_kernel<__nv_bfloat16>, grid, 256, 0, be->stream, (const __nv_bfloat16 *)xp, ip, (const __nv_bfloat16 *)gp, pp, a->rows, a->cols, chunk);
    } else {
        gdb_launch(rms_wgrad_stage_kernel<float>, grid, 256, 0, be->stream, (const float *)xp, ip, (const float *)gp, pp, a->rows, a->cols, chunk);
    }
    gd_status st = gdb_launched(be, "rms_norm_wgrad_stage");
    if (st != GD_OK) {
        return st;
    }
    if (x->dtype == GDB_DTYPE_F16) {
        gdb_launch(rms_wgrad_reduce_kernel<__half>, col_blocks, 256, 0, be->stream, pp, (__half *)dw, blocks, a->cols);
    } else if (x->dtype == GDB_DTYPE_BF16) {
        gdb_launch(rms_wgrad_reduce_kernel<__nv_bfloat16>, col_blocks, 256, 0, be->stream, pp, (__nv_bfloat16 *)dw, blocks, a->cols);
    } else {
        gdb_launch(rms_wgrad_reduce_kernel<float>, col_blocks, 256, 0, be->stream, pp, (float *)dw, blocks, a->cols);
    }
    return gdb_launched(be, "rms_norm_wgrad_reduce");
}

}  // extern "C"

// Internal fusion used by the decode driver; GD_ERR_UNSUPPORTED when the vector path does not apply.
gd_status gdb_add_rms_norm(gd_backend *be, const gd_backend_tensor_view *x, const gd_backend_tensor_view *y, const gd_backend_tensor_view *weight,
                           const gd_backend_tensor_view *sum, const gd_backend_tensor_view *out, size_t rows, size_t cols, float eps)
{
    if (be == NULL || x == NULL || y == NULL || weight == NULL || sum == NULL || out == NULL || rows == 0U || cols == 0U) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const uint32_t dt = x->dtype;
    if ((dt != GDB_DTYPE_F16 && dt != GDB_DTYPE_BF16) || (cols % 8U) != 0U) {
        return GD_ERR_UNSUPPORTED;
    }
    if (x->count != rows * cols || y->count != x->count || sum->count != x->count || out->count != x->count || weight->count != cols) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const void *xp = gdb_tv_ptr(x, dt), *yp = gdb_tv_ptr(y, dt), *wp = gdb_tv_ptr(weight, dt);
    void *sp = gdb_tv_ptr(sum, dt), *op = gdb_tv_ptr(out, dt);
    if (xp == NULL || yp == NULL || wp == NULL || sp == NULL || op == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if ((((uintptr_t)xp | (uintptr_t)yp | (uintptr_t)wp | (uintptr_t)sp | (uintptr_t)op) % 16U) != 0U) {
        return GD_ERR_UNSUPPORTED;
    }
    const unsigned grid = (unsigned)((rows + ROWS_PER_BLOCK - 1) / ROWS_PER_BLOCK);
    if (dt == GDB_DTYPE_F16) {
        gdb_launch(add_rms_fwd_kernel<__half, false>, grid, 32 * ROWS_PER_BLOCK, 0, be->stream, (const uint4 *)xp, (const uint4 *)yp, (const uint4 *)wp, (uint4 *)sp, (uint4 *)op, rows, cols, eps,
                   (uint2 *)nullptr, (float *)nullptr, 1.0f, (uint64_t)0, 0U, (const int *)nullptr, (size_t)0, 0U);
    } else {
        gdb_launch(add_rms_fwd_kernel<__nv_bfloat16, false>, grid, 32 * ROWS_PER_BLOCK, 0, be->stream, (const uint4 *)xp, (const uint4 *)yp, (const uint4 *)wp, (uint4 *)sp, (uint4 *)op, rows, cols, eps,
                   (uint2 *)nullptr, (float *)nullptr, 1.0f, (uint64_t)0, 0U, (const int *)nullptr, (size_t)0, 0U);
    }
    return gdb_launched(be, "add_rms_norm");
}

// grad_accum += rms_norm_backward(x, weight, inv_rms, grad_out): gd_backend_rms_norm_backward_stats followed by
// gd_backend_accumulate of its result (src/autograd/autograd.c:517-685: 16-bit storage rounds after every add) in one launch.
gd_status gdb_rms_norm_backward_accumulate(gd_backend *be, const gd_backend_tensor_view *x, const gd_backend_tensor_view *weight,
                                           const gd_backend_tensor_view *inv_rms, const gd_backend_tensor_view *grad_out,
                                           const gd_backend_tensor_view *grad_accum, const gd_backend_rms_norm_args *args)
{
    return bwd_dispatch<true>(be, x, weight, inv_rms, grad_out, grad_accum, args, true);
}

// rms_norm_backward_stats (+ accumulate into grad_x when add_to_dx) and rms_norm_weight_backward_stats in one launch.
// `partial`: F32 scratch of at least row_blocks * cols elements. GD_ERR_UNSUPPORTED when the fused kernel does not take
// the shape (the caller then issues the two entries).
gd_status gdb_rms_norm_backward_with_weight(gd_backend *be, const gd_backend_tensor_view *x, const gd_backend_tensor_view *weight,
                                            const gd_backend_tensor_view *inv_rms, const gd_backend_tensor_view *grad_out,
                                            const gd_backend_tensor_view *grad_x, bool add_to_dx, const gd_backend_tensor_view *grad_weight,
                                            const gd_backend_tensor_view *partial, const gd_backend_rms_norm_args *a,
                                            const gd_backend_tensor_view *mask, const gd_backend_tensor_view *masked, float mask_scale,
                                            const gd_backend_tensor_view *masked_colsum)
{
    // mask / masked (both or neither): masked = gd_backend_dropout_backward_mask(mask, grad_x, mask_scale) from the same launch;
    // masked_colsum (optional, with mask): [cols] = sum over rows of masked, then `partial` needs 2 * row_blocks * cols elements
    const unsigned char *mp = NULL;
    void *mop = NULL, *mcp = NULL;
    if (masked_colsum != NULL) {
        if (mask == NULL || x == NULL || a == NULL || masked_colsum->count != a->cols || masked_colsum->dtype != x->dtype ||
            (mcp = gdb_tv_ptr(masked_colsum, x->dtype)) == NULL) {
            return GD_ERR_INVALID_ARGUMENT;
        }
    }
    if ((mask == NULL) != (masked == NULL)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (mask != NULL) {
        if (x == NULL || mask->count != x->count || masked->count != x->count || masked->dtype != x->dtype || !(mask_scale > 0.0f)) {
            return GD_ERR_INVALID_ARGUMENT;
        }
        mp = (const unsigned char *)gdb_tv_ptr(mask, GDB_DTYPE_U8);
        mop = gdb_tv_ptr(masked, masked->dtype);
        if (mp == NULL || mop == NULL) {
            return GD_ERR_INVALID_ARGUMENT;
        }
        if (((uintptr_t)mp % 8U) != 0U || ((uintptr_t)mop % 16U) != 0U) {
            return GD_ERR_UNSUPPORTED;
        }
    }
    if (be == NULL || x == NULL || weight == NULL || inv_rms == NULL || grad_out == NULL || grad_x == NULL || grad_weight == NULL ||
        partial == NULL || !args_ok(a) || a->row_blocks == 0U || x->count != a->rows * a->cols || grad_out->count != x->count ||
        grad_x->count != x->count || weight->count != a->cols || grad_weight->count != a->cols || inv_rms->count != a->rows ||
        partial->count < a->row_blocks * a->cols) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const uint32_t dt = x->dtype;
    if ((dt != GDB_DTYPE_F16 && dt != GDB_DTYPE_BF16) || a->cols > (size_t)RBW_MAX_COLS || (a->cols % 8U) != 0U) {
        return GD_ERR_UNSUPPORTED;
    }
    const void *xp = gdb_tv_ptr(x, dt), *wp = gdb_tv_ptr(weight, dt), *gp = gdb_tv_ptr(grad_out, dt);
    void *dp = gdb_tv_ptr(grad_x, dt), *dwp = gdb_tv_ptr(grad_weight, dt);
    const float *ip = (const float *)gdb_tv_ptr(inv_rms, GDB_DTYPE_F32);
    float *pp = (float *)gdb_tv_ptr(partial, GDB_DTYPE_F32);
    if (xp == NULL || wp == NULL || gp == NULL || dp == NULL || dwp == NULL || ip == NULL || pp == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if ((((uintptr_t)xp | (uintptr_t)wp | (uintptr_t)gp | (uintptr_t)dp) % 16U) != 0U) {
        return GD_ERR_UNSUPPORTED;
    }
    size_t blocks = (size_t)be->sm_count;   // one block (144 KB of rings) per SM
    const size_t need = (a->rows + RBW_WARPS - 1U) / RBW_WARPS, room = partial->count / a->cols / (mcp != NULL ? 2U : 1U);
    if (room == 0U) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (blocks > need) blocks = need;
    if (blocks > room) blocks = room;   // one FP32 row of partial sums per block
    unsigned *ticket = gdb_tickets(be);
    {
        static bool configured = false;   // one device per process
        if (!configured) {
            cudaError_t e = cudaFuncSetAttribute(rms_bwd_wgrad_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, RBW_SMEM);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(rms_bwd_wgrad_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, RBW_SMEM);
            if (e != cudaSuccess) return gdb_fail(be, e, "rms_norm backward + weight gradient: shared memory attribute");
            configured = true;
        }
    }
    if (dt == GDB_DTYPE_F16) {
        gdb_launch(rms_bwd_wgrad_kernel<__half>, (unsigned)blocks, RBW_WARPS * 32, RBW_SMEM, be->stream, (const __half *)xp, (const __half *)wp, ip, (const __half *)gp,
                   (__half *)dp, (__half *)dwp, pp, ticket, a->rows, a->cols, add_to_dx, mp, (__half *)mop, mask_scale, (__half *)mcp);
    } else {
        gdb_launch(rms_bwd_wgrad_kernel<__nv_bfloat16>, (unsigned)blocks, RBW_WARPS * 32, RBW_SMEM, be->stream, (const __nv_bfloat16 *)xp, (const __nv_bfloat16 *)wp, ip,
                   (const __nv_bfloat16 *)gp, (__nv_bfloat16 *)dp, (__nv_bfloat16 *)dwp, pp, ticket, a->rows, a->cols, add_to_dx, mp, (__nv_bfloat16 *)mop, mask_scale, (__nv_bfloat16 *)mcp);
    }
    return gdb_launched(be, "rms_norm_backward + weight gradient");
}

extern "C" gd_status gdb200_rms_norm_backward_with_weight(gd_backend *be, const gd_backend_tensor_view *x, const gd_backend_tensor_view *weight,
                                                          const gd_backend_tensor_view *inv_rms, const gd_backend_tensor_view *grad_out,
                                                          const gd_backend_tensor_view *grad_x, int32_t accumulate,
                                                          const gd_backend_tensor_view *grad_weight, const gd_backend_tensor_view *partial,
                                                          const gd_backend_rms_norm_args *args)
{
    return gdb_rms_norm_backward_with_weight(be, x, weight, inv_rms, grad_out, grad_x, accumulate != 0, grad_weight, partial, args, NULL, NULL, 1.0f, NULL);
}

extern "C" gd_status gdb200_rms_norm_backward_with_weight_dropout(gd_backend *be, const gd_backend_tensor_view *x, const gd_backend_tensor_view *weight,
                                                                  const gd_backend_tensor_view *inv_rms, const gd_backend_tensor_view *grad_out,
                                                                  const gd_backend_tensor_view *grad_x, int32_t accumulate,
                                                                  const gd_backend_tensor_view *grad_weight, const gd_backend_tensor_view *partial,
                                                                  const gd_backend_rms_norm_args *args, const gd_backend_tensor_view *mask,
                                                                  const gd_backend_tensor_view *grad_dropped, float scale,
                                                                  const gd_backend_tensor_view *grad_dropped_colsum)
{
    if (mask == NULL || grad_dropped == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    return gdb_rms_norm_backward_with_weight(be, x, weight, inv_rms, grad_out, grad_x, accumulate != 0, grad_weight, partial, args, mask, grad_dropped, scale,
                                             grad_dropped_colsum);
}

gd_status gdb_dropout_add_rms_norm(gd_backend *be, const gd_backend_tensor_view *residual, const gd_backend_tensor_view *x,
                                   const gd_backend_tensor_view *weight, const gd_backend_tensor_view *sum, const gd_backend_tensor_view *mask,
                                   const gd_backend_tensor_view *out, const gd_backend_tensor_view *inv, size_t rows, size_t cols, float eps,
                                   float p, uint64_t seed)
{
    if (be == NULL || residual == NULL || x == NULL || weight == NULL || sum == NULL || mask == NULL || out == NULL || inv == NULL || rows == 0U ||
        cols == 0U || !(p >= 0.0f && p < 1.0f)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const uint32_t dt = x->dtype;
    if ((dt != GDB_DTYPE_F16 && dt != GDB_DTYPE_BF16) || (cols % 8U) != 0U) {
        return GD_ERR_UNSUPPORTED;
    }
    if (x->count != rows * cols || residual->count != x->count || sum->count != x->count || out->count != x->count || mask->count != x->count ||
        weight->count != cols || inv->count != rows || residual->dtype != dt || sum->dtype != dt || out->dtype != dt || weight->dtype != dt) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const void *rp = gdb_tv_ptr(residual, dt), *xp = gdb_tv_ptr(x, dt), *wp = gdb_tv_ptr(weight, dt);
    void *sp = gdb_tv_ptr(sum, dt), *op = gdb_tv_ptr(out, dt), *mp = gdb_tv_ptr(mask, GDB_DTYPE_U8);
    float *ip = (float *)gdb_tv_ptr(inv, GDB_DTYPE_F32);
    if (rp == NULL || xp == NULL || wp == NULL || sp == NULL || op == NULL || mp == NULL || ip == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if ((((uintptr_t)rp | (uintptr_t)xp | (uintptr_t)wp | (uintptr_t)sp | (uintptr_t)op) % 16U) != 0U || ((uintptr_t)mp % 8U) != 0U) {
        return GD_ERR_UNSUPPORTED;
    }
    cudaSetDevice(be->device);
    const unsigned grid = (unsigned)((rows + ROWS_PER_BLOCK - 1) / ROWS_PER_BLOCK);
    const float scale = 1.0f / (1.0f - p);
    const unsigned threshold = gdb_dropout_threshold(p);
    if (dt == GDB_DTYPE_F16) {
        gdb_launch(add_rms_fwd_kernel<__half, true>, grid, 32 * ROWS_PER_BLOCK, 0, be->stream, (const uint4 *)rp, (const uint4 *)xp, (const uint4 *)wp, (uint4 *)sp, (uint4 *)op, rows, cols, eps,
                   (uint2 *)mp, ip, scale, seed, threshold, (const int *)nullptr, (size_t)0, 0U);
    } else {
        gdb_launch(add_rms_fwd_kernel<__nv_bfloat16, true>, grid, 32 * ROWS_PER_BLOCK, 0, be->stream, (const uint4 *)rp, (const uint4 *)xp, (const uint4 *)wp, (uint4 *)sp, (uint4 *)op, rows, cols, eps,
                   (uint2 *)mp, ip, scale, seed, threshold, (const int *)nullptr, (size_t)0, 0U);
    }
    return gdb_launched(be, "dropout_add_rms_norm");
}

// sum = dropout(embedding(table, ids)) (mask written), out = rms_norm(sum, weight), inv_rms saved: gd_backend_embedding_forward,
// gd_backend_dropout_forward and gd_backend_rms_norm_forward_stats in one launch, same rounding points and the same keep decision
// per element index. GD_ERR_UNSUPPORTED when the vector path does not apply.
gd_status gdb_embedding_dropout_rms_norm(gd_backend *be, const gd_backend_tensor_view *table, const gd_backend_tensor_view *ids,
                                         const gd_backend_tensor_view *weight, const gd_backend_tensor_view *sum, const gd_backend_tensor_view *mask,
                                         const gd_backend_tensor_view *out, const gd_backend_tensor_view *inv, size_t rows, size_t cols, size_t vocab,
                                         float eps, float p, uint64_t seed)
{
    if (be == NULL || table == NULL || ids == NULL || weight == NULL || sum == NULL || mask == NULL || out == NULL || inv == NULL || rows == 0U ||
        cols == 0U || vocab == 0U || !(p >= 0.0f && p < 1.0f)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const uint32_t dt = table->dtype;
    if ((dt != GDB_DTYPE_F16 && dt != GDB_DTYPE_BF16) || (cols % 8U) != 0U) {
        return GD_ERR_UNSUPPORTED;
    }
    if (table->count != vocab * cols || ids->count != rows || sum->count != rows * cols || out->count != sum->count || mask->count != sum->count ||
        weight->count != cols || inv->count != rows || sum->dtype != dt || out->dtype != dt || weight->dtype != dt) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const void *tp = gdb_tv_ptr(table, dt), *wp = gdb_tv_ptr(weight, dt);
    const int *ip = (const int *)gdb_tv_ptr(ids, GDB_DTYPE_I32);
    void *sp = gdb_tv_ptr(sum, dt), *op = gdb_tv_ptr(out, dt), *mp = gdb_tv_ptr(mask, GDB_DTYPE_U8);
    float *vp = (float *)gdb_tv_ptr(inv, GDB_DTYPE_F32);
    if (tp == NULL || wp == NULL || ip == NULL || sp == NULL || op == NULL || mp == NULL || vp == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if ((((uintptr_t)tp | (uintptr_t)wp | (uintptr_t)sp | (uintptr_t)op) % 16U) != 0U || ((uintptr_t)mp % 8U) != 0U) {
        return GD_ERR_UNSUPPORTED;
    }
    cudaSetDevice(be->device);
    const unsigned grid = (unsigned)((rows + ROWS_PER_BLOCK - 1) / ROWS_PER_BLOCK);
    const float scale = 1.0f / (1.0f - p);
    const unsigned threshold = gdb_dropout_threshold(p);
    if (dt == GDB_DTYPE_F16) {
        gdb_launch(add_rms_fwd_kernel<__half, true, true>, grid, 32 * ROWS_PER_BLOCK, 0, be->stream, (const uint4 *)nullptr, (const uint4 *)tp, (const uint4 *)wp, (uint4 *)sp,
                   (uint4 *)op, rows, cols, eps, (uint2 *)mp, vp, scale, seed, threshold, ip, vocab, 0x7e007e00U);
    } else {
        gdb_launch(add_rms_fwd_kernel<__nv_bfloat16, true, true>, grid, 32 * ROWS_PER_BLOCK, 0, be->stream, (const uint4 *)nullptr, (const uint4 *)tp, (const uint4 *)wp, (uint4 *)sp,
                   (uint4 *)op, rows, cols, eps, (uint2 *)mp, vp, scale, seed, threshold, ip, vocab, 0x7fc07fc0U);
    }
    return gdb_launched(be, "embedding + dropout + rms_norm");
}

extern "C" gd_status gdb200_embedding_dropout_rms_norm(gd_backend *be, const gd_backend_tensor_view *table, const gd_backend_tensor_view *ids,
                                                       const gd_backend_tensor_view *weight, const gd_backend_tensor_view *x, const gd_backend_tensor_view *mask,
                                                       const gd_backend_tensor_view *normed, const gd_backend_tensor_view *inv_rms, float eps, float p,
                                                       uint64_t seed)
{
    if (table == NULL || ids == NULL || table->rank != 2U || table->shape[0] <= 0 || table->shape[1] <= 0) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    return gdb_embedding_dropout_rms_norm(be, table, ids, weight, x, mask, normed, inv_rms, (size_t)ids->count, (size_t)table->shape[1],
                                          (size_t)table->shape[0], eps, p, seed);
}
