/* The reference's own C host running its gpt_lm model on the B200 backend, fed with synthetic batches.
 *
 * Everything that computes here is the reference's code, compiled from the reference tree where it lies:
 * examples/gpt_lm/gpt_lm_shared.c (gpt_lm_init, gpt_lm_forward :751-823, gpt_block_forward :602-749), the op capsules
 * under src/ops, the tape (src/autograd/autograd.c), gd_backward_amp and gd_optimizer_step_amp_clip_lr
 * (src/optim/adamw.c:2163-2270), inside the gd_begin_step / gd_end_step scopes of src/core/memory.c. The training
 * step below is the body of gd_train_batch (src/train/trainer.c:75-223) with one difference: the batch does not
 * come from a gd_dataloader (the reference's loaders read GDDS files from disk); the step is begun on
 * gd_batch_empty() and the four I32 fields are placed in the data slot the way the loader threads do it
 * (memcpy through the span's host pointer, src/dataset/dataloader.c:487-492) or through gd_tensor_write.
 * The model dimensions are the reference's compile-time defaults (gpt_lm_shared.h:10-28: vocab 2048, context 512,
 * d_model 512, 8 x 64 heads, SwiGLU hidden 1024, tied LM head, window 256).
 *
 * Usage: gpt_lm_synth --batches FILE [--steps K] [--warmup W] [--layers L] [--feed hostptr|upload]
 *                     [--scratch-slots N] [--data-slots N] [--dump-params FILE] [--read-loss] [--dropout P] [--seed S]
 * --scratch-slots / --data-slots override the ring sizes of gpt_memory_config (the example runs with one scratch slot,
 * gpt_lm_shared.c:175, and workers x prefetch + 1 data slots); with one of either the host waits for the previous step.
 * FILE: int32 magic 0x47445342, int32 n_batches, then per batch int32 n_tokens, int32 n_cu, ids[n_tokens],
 * targets[n_tokens], positions[n_tokens], cu_seqlens[n_cu] (all int32), int32 real_tokens.
 * Batches are used round-robin. Prints one JSON line with the per-step losses and the timing.
 */
#include "gpt_lm_shared.h"

#include "core/memory_internal.h"

#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

/* additive entries of the B200 backend library used for timing only */
void *gdb200_event_record(gd_backend *backend);
float gdb200_event_elapsed_ms(void *start, void *stop);
void gdb200_event_destroy(void *event);
uint64_t gdb200_launch_count(const gd_backend *backend);

typedef struct synth_batch {
    int32_t n_tokens, n_cu, real_tokens;
    int32_t *ids, *targets, *positions, *cu;
} synth_batch;

static double now_s(void)
{
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (double)ts.tv_sec + 1.0e-9 * (double)ts.tv_nsec;
}

static void die(const char *what)
{
    fprintf(stderr, "gpt_lm_synth: %s\n", what);
    exit(2);
}

static int32_t *read_i32(FILE *f, size_t n)
{
    int32_t *p = (int32_t *)malloc((n == 0U ? 1U : n) * sizeof(int32_t));
    if (p == NULL || fread(p, sizeof(int32_t), n, f) != n) die("short batch file");
    return p;
}

static synth_batch *load_batches(const char *path, int32_t *count_out)
{
    FILE *f = fopen(path, "rb");
    int32_t head[2];
    synth_batch *b;
    int32_t i;
    if (f == NULL) die("cannot open the batch file");
    if (fread(head, sizeof(int32_t), 2U, f) != 2U || head[0] != 0x47445342 || head[1] <= 0) die("bad batch file header");
    b = (synth_batch *)calloc((size_t)head[1], sizeof(*b));
    if (b == NULL) die("out of memory");
    for (i = 0; i < head[1]; ++i) {
        int32_t dims[2];
        if (fread(dims, sizeof(int32_t), 2U, f) != 2U || dims[0] <= 0 || dims[1] < 2) die("bad batch header");
        b[i].n_tokens = dims[0];
        b[i].n_cu = dims[1];
        b[i].ids = read_i32(f, (size_t)dims[0]);
        b[i].targets = read_i32(f, (size_t)dims[0]);
        b[i].positions = read_i32(f, (size_t)dims[0]);
        b[i].cu = read_i32(f, (size_t)dims[1]);
        if (fread(&b[i].real_tokens, sizeof(int32_t), 1U, f) != 1U) die("short batch file");
    }
    fclose(f);
    *count_out = head[1];
    return b;
}

static void place(gd_context *ctx, gd_tensor *t, const int32_t *src, int32_t n, int use_host_ptr)
{
    int64_t shape[1];
    shape[0] = n;
    TRY(ctx, gd_tensor_empty(ctx, GD_ARENA_DATA, GD_DTYPE_I32, gd_shape_make(1U, shape), GPT_ALIGNMENT, t));
    if (use_host_ptr) {
        /* what a loader thread does with a collated field */
        if (t->storage.host_ptr == NULL) die("data span has no host pointer");
        memcpy((unsigned char *)t->storage.host_ptr + t->view_offset, src, (size_t)n * sizeof(int32_t));
    } else {
        TRY(ctx, gd_tensor_write(ctx, t, src, (size_t)n * sizeof(int32_t)));
    }
}

static void dump_tensor(gd_context *ctx, FILE *f, const char *name, const gd_tensor *t)
{
    int64_t n = 0;
    float *v;
    int32_t len = (int32_t)strlen(name);
    TRY(ctx, gd_tensor_numel(t, &n));
    v = (float *)malloc((size_t)n * sizeof(float));
    if (v == NULL) die("out of memory");
    TRY(ctx, gd_tensor_read_f32(ctx, t, v, (size_t)n));
    fwrite(&len, sizeof(len), 1U, f);
    fwrite(name, 1U, (size_t)len, f);
    fwrite(&n, sizeof(n), 1U, f);
    fwrite(v, sizeof(float), (size_t)n, f);
    free(v);
}

/* parameters in the order and under the names of the Python mirror (host/gpt_lm.py param_specs) */
static void dump_params(gd_context *ctx, const gpt_lm *m, const char *path)
{
    FILE *f = fopen(path, "wb");
    char name[96];
    int i;
    if (f == NULL) die("cannot open the parameter dump");
    dump_tensor(ctx, f, "token_embedding", &m->token_embedding);
    for (i = 0; i < m->n_layers; ++i) {
        const gpt_block *b = &m->block_items[i];
        const struct { const char *n; const gd_tensor *t; } items[] = {
            {"attn_norm_w", &b->attn_norm_w}, {"qkv_proj.weight", &b->qkv_proj.weight}, {"qkv_proj.bias", &b->qkv_proj.bias},
            {"attn_proj.weight", &b->attn_proj.weight}, {"attn_proj.bias", &b->attn_proj.bias}, {"mlp_norm_w", &b->mlp_norm_w},
            {"up_gate.weight", &b->up_gate.weight}, {"up_gate.bias", &b->up_gate.bias},
            {"down_proj.weight", &b->down_proj.weight}, {"down_proj.bias", &b->down_proj.bias}};
        size_t k;
        for (k = 0U; k < sizeof(items) / sizeof(items[0]); ++k) {
            snprintf(name, sizeof(name), "blocks.%d.%s", i, items[k].n);
            dump_tensor(ctx, f, name, items[k].t);
        }
    }
    dump_tensor(ctx, f, "final_norm_w", &m->final_norm_w);
    dump_tensor(ctx, f, "lm_head_bias", &m->lm_head_bias);
    fclose(f);
}

int main(int argc, char **argv)
{
    const char *batch_path = NULL, *dump_path = NULL;
    int steps = 20, warmup = 3, layers = GPT_DEFAULT_LAYERS, use_host_ptr = 1, read_loss = 0, scratch_slots = 1, data_slots = 1;
    float dropout_p = GPT_DEFAULT_DROPOUT_P;
    uint64_t seed = GPT_DEFAULT_SEED;
    gpt_config config;
    gd_memory_config mem;
    gd_context *ctx = NULL;
    gpt_lm model;
    gd_param_set params;
    gd_optimizer *optimizer = NULL;
    gd_amp_scaler *scaler = NULL;
    gd_adamw_config adam;
    gd_amp_config amp;
    synth_batch *batches;
    int32_t n_batches = 0;
    float *losses;
    int i, s;
    double t0 = 0.0, wall = 0.0, enqueue_s = 0.0, first_step_host_s = 0.0;
    long long tokens = 0;
    void *ev0 = NULL, *ev1 = NULL;
    uint64_t launches0 = 0U, launches1 = 0U;
    gd_backend *backend;
    gd_status st;

    for (i = 1; i < argc; ++i) {
        if (strcmp(argv[i], "--batches") == 0 && i + 1 < argc) batch_path = argv[++i];
        else if (strcmp(argv[i], "--steps") == 0 && i + 1 < argc) steps = atoi(argv[++i]);
        else if (strcmp(argv[i], "--warmup") == 0 && i + 1 < argc) warmup = atoi(argv[++i]);
        else if (strcmp(argv[i], "--layers") == 0 && i + 1 < argc) layers = atoi(argv[++i]);
        else if (strcmp(argv[i], "--scratch-slots") == 0 && i + 1 < argc) scratch_slots = atoi(argv[++i]);
        else if (strcmp(argv[i], "--data-slots") == 0 && i + 1 < argc) data_slots = atoi(argv[++i]);
        else if (strcmp(argv[i], "--dropout") == 0 && i + 1 < argc) dropout_p = (float)atof(argv[++i]);
        else if (strcmp(argv[i], "--seed") == 0 && i + 1 < argc) seed = strtoull(argv[++i], NULL, 0);
        else if (strcmp(argv[i], "--dump-params") == 0 && i + 1 < argc) dump_path = argv[++i];
        else if (strcmp(argv[i], "--read-loss") == 0) read_loss = 1;
        else if (strcmp(argv[i], "--feed") == 0 && i + 1 < argc) use_host_ptr = strcmp(argv[++i], "upload") != 0;
        else die("unknown argument");
    }
    if (batch_path == NULL || steps <= 0 || warmup < 0 || layers <= 0 || scratch_slots < 1) die("--batches FILE is required; --steps > 0");
    batches = load_batches(batch_path, &n_batches);

    memset(&config, 0, sizeof(config));
    config.epochs = 1;
    config.batch_size = GPT_DEFAULT_BATCH_SIZE;
    config.n_layers = layers;
    config.dataloader_workers = 0;           /* no loader threads: one reserved data slot */
    config.dataloader_prefetch_factor = 0;
    config.seed = seed;
    config.dropout_p = dropout_p;
    config.lr_max = GPT_DEFAULT_LR_MAX;
    config.lr_min = GPT_DEFAULT_LR_MIN;
    config.weight_decay = GPT_DEFAULT_WEIGHT_DECAY;
    config.grad_clip_norm = GPT_DEFAULT_GRAD_CLIP_NORM;
    config.logits_softcap = 30.0f;           /* examples/gpt_lm/config.yaml */
    config.pad_token_id = -1;
    config.architecture = GPT_ARCH_GPT;
    config.minimax_m3_init_blocks = -1;
    config.minimax_m3_local_blocks = -1;

    mem = gpt_memory_config(&config);
    mem.scratch_slots = (uint32_t)scratch_slots;
    mem.data_slots = (uint32_t)(data_slots < 1 ? 1 : data_slots);
    st = gd_context_create(&mem, &ctx);
    if (st != GD_OK) {
        fprintf(stderr, "gpt_lm_synth: gd_context_create failed with status %d\n", (int)st);
        return 3;
    }
    backend = gd_context_backend(ctx);
    memset(&model, 0, sizeof(model));
    memset(&params, 0, sizeof(params));
    gpt_lm_init(ctx, &model, &config);
    {
        const gd_param_group groups[] = {
            gd_param_group_build("no_decay_norm", "gpt_lm.*norm_w", 1.0f, 0.0f, true),
            gd_param_group_build("no_decay_bias", "gpt_lm.*bias", 1.0f, 0.0f, true),
            gd_param_group_build("decay", "gpt_lm.*", 1.0f, config.weight_decay, true),
        };
        TRY(ctx, gd_module_collect_params(ctx, &model.mod, groups, sizeof(groups) / sizeof(groups[0]), &params));
    }
    adam = gd_adamw_config_default();        /* examples/gpt_lm/main.c:1125-1146 */
    adam.lr = config.lr_max;
    adam.weight_decay = config.weight_decay;
    adam.beta1 = 0.9f;
    adam.beta2 = 0.95f;
    adam.eps = 1.0e-8f;
    adam.bias_correction = true;
    amp = gd_amp_config_default();
    amp.init_scale = 65536.0f;
    amp.growth_factor = 2.0f;
    amp.backoff_factor = 0.5f;
    amp.growth_interval = 2000U;
    TRY(ctx, gd_adamw_create(ctx, &params, &adam, &optimizer));
    TRY(ctx, gd_amp_scaler_create(ctx, &amp, &scaler));
    TRY(ctx, gd_context_seal_params(ctx));
    if (dump_path != NULL) dump_params(ctx, &model, dump_path);

    losses = (float *)calloc((size_t)(steps + warmup), sizeof(float));
    if (losses == NULL) die("out of memory");
    for (s = 0; s < warmup + steps; ++s) {
        const synth_batch *b = &batches[s % n_batches];
        gd_tensor ids, targets, positions, cu, loss;
        double e0;
        if (s == warmup) {
            TRY(ctx, gd_synchronize(ctx));
            ev0 = gdb200_event_record(backend);
            launches0 = gdb200_launch_count(backend);
            t0 = now_s();
        }
        e0 = now_s();
        memset(&loss, 0, sizeof(loss));
        TRY(ctx, gd_begin_step(ctx, GD_SCOPE_TRAIN, gd_batch_empty()));
        place(ctx, &ids, b->ids, b->n_tokens, use_host_ptr);
        place(ctx, &targets, b->targets, b->n_tokens, use_host_ptr);
        place(ctx, &positions, b->positions, b->n_tokens, use_host_ptr);
        place(ctx, &cu, b->cu, b->n_cu, use_host_ptr);
        TRY(ctx, gpt_lm_forward(ctx, &model, &ids, &targets, &positions, &cu, (uint64_t)s + 1U, &loss));
        TRY(ctx, gd_backward_amp(ctx, &loss, NULL, scaler));
        TRY(ctx, gd_optimizer_step_amp_clip_lr(ctx, optimizer, scaler, config.lr_max, config.grad_clip_norm));
        TRY(ctx, gd_end_step(ctx));
        if (s >= warmup) {
            enqueue_s += now_s() - e0;
            tokens += b->real_tokens;
        }
        /* the first timed step starts on an idle device with an empty launch queue: its host time is what the host
         * itself needs to issue one step (later steps also contain waits for the device) */
        if (s == warmup) first_step_host_s = now_s() - e0;
        if (read_loss || s == warmup + steps - 1) {
            TRY(ctx, gd_tensor_item(ctx, &loss, &losses[s]));
        }
    }
    ev1 = gdb200_event_record(backend);
    TRY(ctx, gd_synchronize(ctx));
    wall = now_s() - t0;
    launches1 = gdb200_launch_count(backend);
    {
        const float dev_ms = gdb200_event_elapsed_ms(ev0, ev1);
        gd_memory_stats stats;
        memset(&stats, 0, sizeof(stats));
        (void)gd_memory_stats_query(ctx, &stats);
        printf("{\"host\": \"reference C host (gpt_lm_shared.c + tape + adamw.c) on libgd_backend_b200\", \"steps\": %d, \"warmup\": %d, "
               "\"layers\": %d, \"feed\": \"%s\", \"scratch_slots\": %d, \"data_slots\": %d, \"tokens\": %lld, \"device_ms_per_step\": %.6f, "
               "\"wall_ms_per_step\": %.6f, \"host_call_ms_per_step\": %.6f, \"host_issue_ms_first_step\": %.6f, \"tokens_per_s\": %.3f, \"launches_per_step\": %.2f, "
               "\"scratch_ring_waits\": %llu, \"losses\": [",
               steps, warmup, layers, use_host_ptr ? "hostptr" : "upload", scratch_slots, data_slots, tokens, (double)dev_ms / steps,
               1000.0 * wall / steps, 1000.0 * enqueue_s / steps, 1000.0 * first_step_host_s, (double)tokens / wall, (double)(launches1 - launches0) / steps,
               (unsigned long long)stats.scratch.waits);
        for (s = 0; s < warmup + steps; ++s) printf("%s%.9g", s == 0 ? "" : ", ", (double)losses[s]);
        printf("]}\n");
    }
    gdb200_event_destroy(ev0);
    gdb200_event_destroy(ev1);
    gd_amp_scaler_destroy(scaler);
    gd_optimizer_destroy(optimizer);
    gd_param_set_free(&params);
    gpt_lm_deinit(&model);
    gd_context_destroy(ctx);
    return 0;
}
