/* TEST INFRASTRUCTURE: a small C program that drives a device backend through the
 * reference's own, unmodified host code. It is compiled together with the reference's
 * h3_dit.c, h3_dit_schedule.c, h3_host.c, h3_weights.c and h3_safetensors.c (read in place
 * from the reference tree by oracle/build_ref.py) and linked once against libh3b200.so and
 * once against the reference's CUDA backend; tests/test_gpu_ref_host.py runs both on the
 * same synthetic checkpoint and compares what they produce.
 *
 * What it calls is what the reference's pipeline calls (h3.c:1503-1646):
 *   h3_layout_build, h3_serving_schedule_build,
 *   h3_dit_load_t2va     -> weight store, refine_text, h3_dit_schedule_precompute,
 *                           prepare_rope / prepare_maps, load_core, allocate_activations
 *   h3_dit_forward       -> one velocity evaluation at step 0
 *   then one sampler pass per remaining argument, each from the same seeded noise after
 *   h3_dit_reset_run: "euler:N" = h3_dit_denoise_euler_preview with reuse interval N (the
 *   serving sampler, device-resident Euler loop), "res" = h3_dit_denoise (the RES multistep
 *   solver, host-side update around h3_dit_forward).
 * Inputs come from the reference's generator (h3_rng, h3_host.c:496-530) with fixed seeds.
 *
 * usage: dit_host <weight dir> <output file> text_len latent_t latent_h latent_w audio_t
 *                 steps core_reuse token_reduction ssd_streaming pass [pass ...]
 * output file: int32 video_count, audio_count, passes, then F32: video velocity, audio
 *              velocity, and per pass the final video latent and final audio latent.
 */
#include "h3_dit.h"

#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

static double now(void) {
    struct timespec t;
    clock_gettime(CLOCK_MONOTONIC, &t);
    return (double)t.tv_sec + (double)t.tv_nsec * 1e-9;
}

static void die(const char *what, const char *detail) {
    fprintf(stderr, "dit_host: %s: %s\n", what, detail ? detail : "");
    exit(1);
}

static uint16_t to_bf16(float value) {
    uint32_t bits;
    memcpy(&bits, &value, sizeof(bits));
    bits += 0x7fffu + ((bits >> 16) & 1u);
    return (uint16_t)(bits >> 16);
}

static void progress(const char *phase, int completed, int total, void *opaque) {
    (void)opaque;
    if (completed == total) fprintf(stderr, "dit_host: %s %d/%d\n", phase, completed, total);
}

int main(int argc, char **argv) {
    if (argc < 13) die("usage", "dit_host dir out text_len t h w audio_t steps core_reuse token_reduction ssd pass...");
    const char *directory = argv[1], *output_path = argv[2];
    int text_len = atoi(argv[3]), latent_t = atoi(argv[4]), latent_h = atoi(argv[5]);
    int latent_w = atoi(argv[6]), audio_t = atoi(argv[7]), steps = atoi(argv[8]);
    int core_reuse = atoi(argv[9]), token_reduction = atoi(argv[10]), ssd = atoi(argv[11]);
    int passes = argc - 12;
    char error[512] = {0};

    h3_rng rng;
    size_t text_count = (size_t)text_len * H3_TEXT_HIDDEN_SIZE;
    uint16_t *text_values = malloc(text_count * sizeof(*text_values));
    if (!text_values) die("out of memory", "text");
    h3_rng_seed(&rng, 2);
    for (size_t i = 0; i < text_count; i++) text_values[i] = to_bf16(h3_rng_normal(&rng));
    h3_text_embedding text;
    memset(&text, 0, sizeof(text));
    text.tokens = (size_t)text_len;
    text.width = H3_TEXT_HIDDEN_SIZE;
    text.values = text_values;

    h3_layout_spec spec = {text_len, latent_t, latent_h, latent_w, audio_t, 5, NULL, 0, NULL, 0};
    h3_layout layout;
    if (!h3_layout_build(&spec, &layout, error, sizeof(error))) die("layout", error);
    h3_sigma_schedule sigmas;
    if (!h3_serving_schedule_build(steps, &sigmas)) die("schedule", "cannot build the sigma schedule");

    double t0 = now();
    h3_dit *dit = h3_dit_load_t2va(directory, "unused", &text, &layout, &sigmas, 50,
                                   (unsigned)core_reuse, token_reduction, ssd, 1.0f,
                                   0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, progress, NULL, error, sizeof(error));
    if (!dit) die("load", error);
    double load_seconds = now() - t0;

    size_t video_count = h3_dit_video_elements(dit), audio_count = h3_dit_audio_elements(dit);
    float *video = malloc(video_count * sizeof(float)), *audio = malloc(audio_count * sizeof(float));
    float *video_velocity = malloc(video_count * sizeof(float));
    float *audio_velocity = malloc(audio_count * sizeof(float));
    if (!video || !audio || !video_velocity || !audio_velocity) die("out of memory", "latents");
    FILE *out = fopen(output_path, "wb");
    if (!out) die("cannot write", output_path);
    int32_t counts[3] = {(int32_t)video_count, (int32_t)audio_count, (int32_t)passes};
    fwrite(counts, sizeof(counts), 1, out);

    h3_rng_seed(&rng, 1);
    h3_rng_fill_normal(&rng, video, video_count);
    h3_rng_seed(&rng, 3);
    h3_rng_fill_normal(&rng, audio, audio_count);
    t0 = now();
    if (!h3_dit_forward(dit, 0, video, audio, video_velocity, audio_velocity, error, sizeof(error)))
        die("forward", error);
    double forward_seconds = now() - t0;
    fwrite(video_velocity, sizeof(float), video_count, out);
    fwrite(audio_velocity, sizeof(float), audio_count, out);

    for (int pass = 0; pass < passes; pass++) {
        const char *what = argv[12 + pass];
        h3_rng_seed(&rng, 1);
        h3_rng_fill_normal(&rng, video, video_count);
        h3_rng_seed(&rng, 3);
        h3_rng_fill_normal(&rng, audio, audio_count);
        if (!h3_dit_reset_run(dit, NULL, 0, NULL, 0, error, sizeof(error))) die("reset", error);
        t0 = now();
        int ok;
        if (!strcmp(what, "res"))
            ok = h3_dit_denoise(dit, video, audio, progress, NULL, error, sizeof(error));
        else if (!strncmp(what, "euler:", 6))
            ok = h3_dit_denoise_euler_preview(dit, video, audio, atoi(what + 6), progress, NULL, NULL,
                                              NULL, error, sizeof(error));
        else
            die("unknown pass", what);
        if (!ok) die(what, error);
        printf("dit_host: pass %s: %.3f s\n", what, now() - t0);
        fwrite(video, sizeof(float), video_count, out);
        fwrite(audio, sizeof(float), audio_count, out);
    }
    fclose(out);

    h3_gpu_stats stats;
    if (!h3_dit_get_gpu_stats(dit, &stats)) die("stats", "cannot read the device statistics");
    printf("dit_host: sequence %zu rows, load %.2f s (%.2f GiB into tensors, %.2f GiB/s), forward %.3f s; "
           "%llu projections, %llu attention calls, %llu other kernels, %llu submissions\n",
           layout.seq_len, load_seconds, (double)stats.allocated_bytes / 1073741824.0,
           (double)stats.allocated_bytes / 1073741824.0 / load_seconds, forward_seconds,
           (unsigned long long)stats.mps_linear_dispatches, (unsigned long long)stats.mps_sdpa_dispatches,
           (unsigned long long)stats.direct_dispatches, (unsigned long long)stats.submissions);

    h3_dit_free(dit);
    h3_layout_free(&layout);
    free(text_values); free(video); free(audio); free(video_velocity); free(audio_velocity);
    return 0;
}
