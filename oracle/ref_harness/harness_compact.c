/* Exports the compact-record transform of examples/gpt_lm/main.c:873-970 (u16 tokens[context + 1] and the
 * record's segment lengths -> input ids, next-token targets with cross-document targets masked, positions that
 * restart per segment). Test infrastructure only. */
#define main gdref_gpt_lm_unused_main
#include GDREF_GPT_LM_MAIN
#undef main
#include "dataset/dataset_internal.h"

/* Runs the reference transform on one record. Returns its gd_status; on GD_OK the three outputs hold
 * `context_length` values each. */
int gdref_compact_transform(const uint16_t *tokens, int32_t context_length, const int32_t *segment_lengths, int32_t n_segments,
                            int32_t vocab_size, int32_t pad_id, int32_t im_start_id, int32_t im_end_id, int32_t *input_ids,
                            int32_t *positions, int32_t *target_ids)
{
    gpt_lm_compact_transform cfg;
    gd_sample_field src_fields[GPT_COMPACT_SRC_FIELD_COUNT];
    gd_sample_field dst_fields[GPT_FIELD_COUNT];
    gd_sample src, dst;
    gd_status st;
    int i;
    memset(&cfg, 0, sizeof(cfg));
    memset(src_fields, 0, sizeof(src_fields));
    memset(dst_fields, 0, sizeof(dst_fields));
    cfg.context_length = context_length;
    cfg.record_length = context_length + 1;
    cfg.vocab_size = vocab_size;
    cfg.pad_id = pad_id;
    cfg.im_start_id = im_start_id;
    cfg.im_end_id = im_end_id;
    src_fields[GPT_COMPACT_SRC_TOKENS].dtype = GD_DTYPE_U16;
    src_fields[GPT_COMPACT_SRC_TOKENS].rank = 1;
    src_fields[GPT_COMPACT_SRC_TOKENS].shape[0] = (int64_t)context_length + 1;
    src_fields[GPT_COMPACT_SRC_TOKENS].data = tokens;
    src_fields[GPT_COMPACT_SRC_TOKENS].nbytes = ((size_t)context_length + 1U) * sizeof(uint16_t);
    src_fields[GPT_COMPACT_SRC_SEGMENT_LENGTHS].dtype = GD_DTYPE_I32;
    src_fields[GPT_COMPACT_SRC_SEGMENT_LENGTHS].rank = 1;
    src_fields[GPT_COMPACT_SRC_SEGMENT_LENGTHS].shape[0] = n_segments;
    src_fields[GPT_COMPACT_SRC_SEGMENT_LENGTHS].data = segment_lengths;
    src_fields[GPT_COMPACT_SRC_SEGMENT_LENGTHS].nbytes = (size_t)(n_segments > 0 ? n_segments : 0) * sizeof(int32_t);
    src.n_fields = GPT_COMPACT_SRC_FIELD_COUNT;
    src.fields = src_fields;
    for (i = 0; i < GPT_FIELD_COUNT; ++i) {
        dst_fields[i].writable = 1;
    }
    dst.n_fields = GPT_FIELD_COUNT;
    dst.fields = dst_fields;
    st = gpt_lm_compact_transform_fn(&src, &dst, &cfg);
    if (st == GD_OK) {
        memcpy(input_ids, dst_fields[GPT_FIELD_INPUT_IDS].data, (size_t)context_length * sizeof(int32_t));
        memcpy(positions, dst_fields[GPT_FIELD_POSITIONS].data, (size_t)context_length * sizeof(int32_t));
        memcpy(target_ids, dst_fields[GPT_FIELD_TARGET_IDS].data, (size_t)context_length * sizeof(int32_t));
    }
    for (i = 0; i < GPT_FIELD_COUNT; ++i) {
        free(dst_fields[i].owned_data);
    }
    return (int)st;
}
