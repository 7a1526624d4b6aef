/* TEST INFRASTRUCTURE: drives a device backend through the reference's own, unmodified
 * video-VAE decoder host code. It is compiled together with the reference's h3_video_vae.c,
 * h3_weights.c and h3_safetensors.c (read in place from the reference tree by
 * oracle/build_ref.py) and linked once against libh3b200.so and once against the reference's
 * CUDA backend; tests/test_gpu_ref_vae.py runs both on the same synthetic checkpoint and
 * compares the decoded frames.
 *
 * What it calls is what the reference's pipeline calls after the denoiser (h3.c, video decode
 * phase): h3_video_vae_decode -> for one tile and seven latent frames: load_input_weights,
 * prepare_input, prepare_rope, run_decoder (36 x load_block / run_block / free_block),
 * unpack_frames; for anything larger decode_chunked: the resident decoder (all weights loaded
 * once), 256-pixel overlapping tiles, temporal chunks of seven latent frames, blending on the host.
 *
 * usage: vae_host <weights dir> <output file> latent_t latent_h latent_w seed
 * input: normalized latent [24 channels][t][h][w], uniform in [-1.7, 1.7] from a 64-bit LCG.
 * output file: int32 frames, height, width, then frames x height x width x 3 F32 RGB.
 */
#include "h3_video_vae.h"

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

static void progress(int completed, int total, void *opaque) {
    (void)opaque;
    if (completed == total) fprintf(stderr, "vae_host: %d/%d blocks\n", completed, total);
}

int main(int argc, char **argv) {
    if (argc != 7) {
        fprintf(stderr, "usage: vae_host dir out latent_t latent_h latent_w seed\n");
        return 2;
    }
    int latent_t = atoi(argv[3]), latent_h = atoi(argv[4]), latent_w = atoi(argv[5]);
    uint64_t state = strtoull(argv[6], NULL, 10) * 0x9e3779b97f4a7c15ull + 1;
    size_t count = (size_t)24 * latent_t * latent_h * latent_w;
    float *latent = malloc(count * sizeof(*latent));
    if (!latent) return 1;
    for (size_t i = 0; i < count; i++) {
        state = state * 6364136223846793005ull + 1442695040888963407ull;
        latent[i] = ((float)(state >> 40) / 16777216.0f * 2.0f - 1.0f) * 1.7f;
    }
    char error[512] = {0};
    h3_video_frames frames;
    double t0 = now();
    if (!h3_video_vae_decode(argv[1], "unused", latent, latent_t, latent_h, latent_w, progress, NULL,
                             &frames, error, sizeof(error))) {
        fprintf(stderr, "vae_host: decode: %s\n", error);
        return 1;
    }
    double seconds = now() - t0;
    FILE *out = fopen(argv[2], "wb");
    if (!out) return 1;
    int32_t header[3] = {frames.frames, frames.height, frames.width};
    fwrite(header, sizeof(header), 1, out);
    fwrite(frames.rgb, sizeof(float), (size_t)frames.frames * frames.height * frames.width * 3, out);
    fclose(out);
    printf("vae_host: %d frames of %d x %d in %.3f s (device %.3f s); %llu projections, %llu attention calls, "
           "%llu other kernels, %llu submissions\n",
           frames.frames, frames.width, frames.height, seconds, frames.gpu_stats.gpu_seconds,
           (unsigned long long)frames.gpu_stats.mps_linear_dispatches,
           (unsigned long long)frames.gpu_stats.mps_sdpa_dispatches,
           (unsigned long long)frames.gpu_stats.direct_dispatches,
           (unsigned long long)frames.gpu_stats.submissions);
    h3_video_frames_free(&frames);
    free(latent);
    return 0;
}
