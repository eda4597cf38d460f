/* A C99 client of the engine's C ABI: what a host written in plain C (or a cgo / JNI / FFI stub) sees.
 * Creates an engine, prints its description and a group advantage computed on the device; exits 3 with the
 * library's error text when there is no usable GPU (the library has no CPU fallback). */
#include <stdio.h>
#include <string.h>

#include "nn_b200.h"

int main(void)
{
    nnb_engine* e = NULL;
    if (nnb_engine_create(0, &e) != NNB_OK) {
        fprintf(stderr, "engine: %s\n", nnb_last_error());
        return 3;
    }
    char text[256];
    if (nnb_engine_describe(e, text, sizeof text) != NNB_OK) return 4;
    printf("%s\n", text);
    const float returns[6] = {1.f, 2.f, 3.f, 5.f, 5.f, 5.f};
    const int32_t first[2] = {0, 3}, count[2] = {3, 3};
    float *d_ret = NULL, *d_adv = NULL, adv[6];
    if (nnb_alloc(e, sizeof returns, (void**)&d_ret) != NNB_OK || nnb_alloc(e, sizeof adv, (void**)&d_adv) != NNB_OK) return 5;
    if (nnb_upload(e, d_ret, returns, sizeof returns) != NNB_OK) return 6;
    if (nnb_group_advantage(e, d_ret, 6, first, count, 2, 1e-8f, d_adv) != NNB_OK) {
        fprintf(stderr, "group_advantage: %s\n", nnb_last_error());
        return 7;
    }
    if (nnb_download(e, adv, d_adv, sizeof adv) != NNB_OK) return 8;
    /* {1,2,3} -> {-1/s, 0, 1/s} with s = sqrt(2/3); a constant group -> zeros */
    printf("%.6f %.6f %.6f %.6f %.6f %.6f\n", adv[0], adv[1], adv[2], adv[3], adv[4], adv[5]);
    nnb_free(e, d_ret);
    nnb_free(e, d_adv);
    nnb_engine_destroy(e);
    return 0;
}
