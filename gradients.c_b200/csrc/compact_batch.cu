// Expansion of compact GPT-LM records into the packed batch the training step consumes, on the device.
//
// The reference stores a training sample as context_length + 1 little-endian u16 tokens plus the I32 lengths of
// the documents ("segments") packed into it, expands each sample on a loader thread into I32 input ids, next-token
// targets (targets that would cross into another document are replaced by the pad id) and positions that restart
// per segment (examples/gpt_lm/main.c:873-970), and lets the packed-sequence collate generate cu_seqlens as the
// running sum of all segment lengths of the batch (src/dataset/gdds_dataset.c:2191-2224). Doing the expansion here
// means a step copies 2 bytes per token (+ 4 per segment) to the device instead of 12.
//
// Integer work, HBM-bound in principle (14 bytes per token: 2 read, 12 written) but launch-bound at the sizes of
// a step (64 records of 512 tokens = 0.46 MB). Two launches: one block scans the segment lengths (and validates
// them), then one thread per token expands.
#include "common.cuh"

namespace {

constexpr int SCAN_THREADS = 1024;

// cu[0] = 0, cu[s + 1] = cu[s] + len[s]; *status = flags of what the reference's transform would have rejected:
// a length <= 0, or a record whose own lengths do not add up to context_length (main.c:945-959; with all lengths
// positive that holds for every record iff record r's first segment starts at token r * context_length and the
// total is n_records * context_length).
__global__ void __launch_bounds__(SCAN_THREADS)
compact_scan_kernel(const int32_t *__restrict__ len, const int32_t *__restrict__ rec_off, int32_t *cu, int32_t *__restrict__ status,
                    long long n_segments, long long n_records, long long total_tokens, int context_length)
{
    gdb_pdl_sync();
    __shared__ long long warp_sum[SCAN_THREADS / 32];
    __shared__ long long carry_s;
    __shared__ int flags_s;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        carry_s = 0;
        flags_s = 0;
        cu[0] = 0;
    }
    __syncthreads();
    int flags = 0;
    for (long long base = 0; base < n_segments; base += SCAN_THREADS) {
        const long long s = base + threadIdx.x;
        const long long l = s < n_segments ? (long long)len[s] : 0;
        if (s < n_segments && l <= 0) flags |= GDB200_COMPACT_BAD_LENGTH;
        long long x = l;   // inclusive scan inside the warp
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const long long y = __shfl_up_sync(0xffffffffU, x, d);
            if (lane >= d) x += y;
        }
        if (lane == 31) warp_sum[warp] = x;
        __syncthreads();
        if (warp == 0) {
            long long w = warp_sum[lane];
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const long long y = __shfl_up_sync(0xffffffffU, w, d);
                if (lane >= d) w += y;
            }
            warp_sum[lane] = w;   // inclusive sums of the warps
        }
        __syncthreads();
        const long long end = carry_s + (warp > 0 ? warp_sum[warp - 1] : 0) + x;   // exclusive end of segment s
        if (s < n_segments) {
            const long long begin = end - l;
            if (l > 0 && (end > total_tokens || begin / context_length != (end - 1) / context_length)) flags |= GDB200_COMPACT_BAD_COVER;   // main.c:946
            cu[s + 1] = (int32_t)(end < 0 ? 0 : (end > 0x7fffffffLL ? 0x7fffffffLL : end));
        }
        __syncthreads();
        if (threadIdx.x == SCAN_THREADS - 1) carry_s = end;
        __syncthreads();
    }
    // record r owns segments rec_off[r] .. rec_off[r + 1] - 1, and they must start at token r * context_length
    for (long long r = threadIdx.x; r <= n_records; r += SCAN_THREADS) {
        const long long o = rec_off[r];
        const bool ordered = r == n_records ? o == n_segments : (o >= 0 && o < n_segments && o < (long long)rec_off[r + 1]);
        if (!ordered || (r == 0 && o != 0) || (long long)cu[o] != r * context_length) flags |= GDB200_COMPACT_BAD_COVER;
    }
    if (flags != 0) atomicOr(&flags_s, flags);
    __syncthreads();
    if (threadIdx.x == 0) {
        *status = flags_s | (carry_s != total_tokens ? GDB200_COMPACT_BAD_COVER : 0);
    }
}

// One thread per packed token i = r * context_length + j.
__global__ void __launch_bounds__(256)
compact_expand_kernel(const uint16_t *__restrict__ tokens, const int32_t *__restrict__ cu, int32_t *__restrict__ ids,
                      int32_t *__restrict__ targets, int32_t *__restrict__ positions, int32_t *__restrict__ status, long long n_segments,
                      long long total_tokens, int context_length, int vocab_size, int pad_id, int im_start_id, int im_end_id)
{
    gdb_pdl_sync();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total_tokens) return;
    const long long r = i / context_length;
    const int j = (int)(i - r * context_length);
    const uint16_t *rec = tokens + r * ((long long)context_length + 1);
    const int tok = rec[j], next = rec[j + 1];
    if (tok >= vocab_size || next >= vocab_size) atomicOr(status, GDB200_COMPACT_BAD_TOKEN);   // main.c:934-939
    // segment of token i: the largest s with cu[s] <= i
    long long lo = 0, hi = n_segments;
    while (lo + 1 < hi) {
        const long long mid = (lo + hi) >> 1;
        if ((long long)__ldg(&cu[mid]) <= i) lo = mid; else hi = mid;
    }
    const long long seg_begin = __ldg(&cu[lo]), seg_end = __ldg(&cu[lo + 1]);
    int target = next;
    if (j == context_length - 1) {
        if (tok == im_end_id && next == im_start_id) target = pad_id;        // main.c:960-963
    } else if (i == seg_end - 1) {
        target = pad_id;                                                     // main.c:953-955
    }
    ids[i] = tok;
    targets[i] = target;
    positions[i] = (int32_t)(i - seg_begin);
}

}  // namespace

extern "C" gd_status gdb200_gpt_compact_expand(gd_backend *be, const gdb200_gpt_compact_batch *b)
{
    if (be == NULL || b == NULL || b->buffer == NULL || b->n_records <= 0 || b->context_length <= 0 || b->vocab_size <= 0 ||
        b->vocab_size > 65536 || b->pad_id < 0 || b->pad_id >= b->vocab_size || b->im_start_id < 0 || b->im_end_id < 0) {
        return GD_ERR_INVALID_ARGUMENT;   // the configuration checks of main.c:891-896
    }
    if (b->n_records > (int64_t)0x7fffffff / b->context_length) {
        return GD_ERR_INVALID_ARGUMENT;   // cu_seqlens is I32 (gdds_dataset.c:2217)
    }
    const long long total = (long long)b->n_records * b->context_length;
    if (b->n_segments < b->n_records || b->n_segments > total) {
        return GD_ERR_INVALID_ARGUMENT;   // every record holds between 1 and context_length segments (main.c:910-911)
    }
    const size_t tok_bytes = (size_t)b->n_records * ((size_t)b->context_length + 1U) * 2U;
    const size_t out_bytes = (size_t)total * 4U;
    if ((b->tokens_offset % 2U) != 0U || ((b->segment_lengths_offset | b->record_offsets_offset | b->input_ids_offset | b->targets_offset | b->positions_offset |
                                            b->cu_seqlens_offset | b->status_offset) % 4U) != 0U ||
        !gdb_range_ok(b->buffer, b->tokens_offset, tok_bytes) || !gdb_range_ok(b->buffer, b->segment_lengths_offset, (size_t)b->n_segments * 4U) ||
        !gdb_range_ok(b->buffer, b->record_offsets_offset, ((size_t)b->n_records + 1U) * 4U) ||
        !gdb_range_ok(b->buffer, b->input_ids_offset, out_bytes) || !gdb_range_ok(b->buffer, b->targets_offset, out_bytes) ||
        !gdb_range_ok(b->buffer, b->positions_offset, out_bytes) || !gdb_range_ok(b->buffer, b->cu_seqlens_offset, ((size_t)b->n_segments + 1U) * 4U) ||
        !gdb_range_ok(b->buffer, b->status_offset, 4U)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    cudaSetDevice(be->device);
    unsigned char *base = b->buffer->dptr;
    int32_t *cu = (int32_t *)(base + b->cu_seqlens_offset), *status = (int32_t *)(base + b->status_offset);
    gdb_launch(compact_scan_kernel, 1, SCAN_THREADS, 0, be->stream, (const int32_t *)(base + b->segment_lengths_offset),
               (const int32_t *)(base + b->record_offsets_offset), cu, status, (long long)b->n_segments, (long long)b->n_records, total,
               (int)b->context_length);
    gd_status st = gdb_launched(be, "compact scan");
    if (st != GD_OK) {
        return st;
    }
    gdb_launch(compact_expand_kernel, (unsigned)((total + 255) / 256), 256, 0, be->stream, (const uint16_t *)(base + b->tokens_offset),
               (const int32_t *)cu, (int32_t *)(base + b->input_ids_offset), (int32_t *)(base + b->targets_offset),
               (int32_t *)(base + b->positions_offset), status, (long long)b->n_segments, total, (int)b->context_length, (int)b->vocab_size,
               (int)b->pad_id, (int)b->im_start_id, (int)b->im_end_id);
    return gdb_launched(be, "compact expand");
}
