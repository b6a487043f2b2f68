/* A C program over the library's C interface (bn_api.h), as tests/test_capi_gpu.py builds and
 * runs it: load a model folder, prefill a prompt, step token by token, sample, run a batch step,
 * generate for a batch, and print everything as one JSON object.
 * usage: capi_smoke MODEL_DIR DTYPE */
#include <stdio.h>
#include <stdlib.h>
#include "bn_api.h"

#define CHECK(x) do { if (!(x)) { fprintf(stderr, "failed: %s: %s\n", #x, bn_last_error()); return 1; } } while (0)

static void print_row(const char *name, const float *v, int n, int last) {
    printf("\"%s\": [", name);
    for (int i = 0; i < n; i++) printf("%s%.9g", i ? ", " : "", v[i]);
    printf("]%s", last ? "" : ", ");
}

int main(int argc, char **argv) {
    if (argc != 3) return 2;
    BnCacheParams cp = {0, 4};
    BnModel *m = bn_model_load(argv[1], argv[2], 0, &cp);
    CHECK(m != NULL);
    int V = bn_model_vocab_size(m);
    int prompt[6] = {5, 17, 3, 200, 9, 41};
    printf("{\"vocab\": %d, \"seq_len\": %d, ", V, bn_model_seq_len(m));

    BnSession *s = bn_session_create(m);
    CHECK(s != NULL);
    const float *l = bn_prefill(m, s, prompt, 4, 0, 0);
    CHECK(l != NULL && bn_session_pos(s) == 4);
    print_row("prefill4", l, V, 0);
    l = bn_transformer_forward(m, s, prompt[4], 4);
    CHECK(l != NULL);
    print_row("forward5", l, V, 0);
    CHECK(bn_prefill(m, s, prompt, 2, 0, 0) == NULL);  /* wrong position: refused, message kept */
    printf("\"refusal\": \"%s\", ", bn_last_error());
    CHECK(bn_session_reset(s) == 0 && bn_session_pos(s) == 0);
    float *all = (float *)malloc((size_t)6 * V * sizeof(float));
    CHECK(bn_transformer_prefill_all(m, s, prompt, 6, 0, all) == 0);
    print_row("all6_last", all + 5 * V, V, 0);

    /* the sampler on the last row: greedy, and two draws with a temperature */
    BnSamplerParams greedy = {0.0f, 0.9f, 1.0f, 64, 42};
    BnSampler *sa = bn_sampler_create(V, &greedy);
    CHECK(sa != NULL);
    printf("\"greedy\": %d, ", bn_sampler_sample(sa, all + 5 * V));
    bn_sampler_free(sa);
    BnSamplerParams warm = {0.8f, 0.9f, 1.0f, 64, 1234};
    sa = bn_sampler_create(V, &warm);
    CHECK(sa != NULL);
    int d0 = bn_sampler_sample(sa, all + 5 * V), d1 = bn_sampler_sample(sa, all + 4 * V);
    printf("\"draws\": [%d, %d], ", d0, d1);
    bn_sampler_free(sa);

    /* a batch step of two sessions of unequal lengths */
    BnSession *t = bn_session_create(m);
    CHECK(t != NULL);
    CHECK(bn_session_reset(s) == 0);
    BnSession *both[2] = {s, t};
    int n_new[2] = {4, 2}, packed[6] = {5, 17, 3, 200, 9, 41};
    float *two = (float *)malloc((size_t)2 * V * sizeof(float));
    CHECK(bn_step(m, both, 2, n_new, packed, two) == 0);
    print_row("step_a", two, V, 0);
    print_row("step_b", two + V, V, 0);
    bn_session_free(s);
    bn_session_free(t);

    /* generation for three prompts of unequal lengths */
    const int *prompts[3] = {prompt, prompt + 4, prompt + 2};
    int lens[3] = {4, 1, 3}, counts[3];
    int out0[8], out1[8], out2[8];
    int *outs[3] = {out0, out1, out2};
    CHECK(bn_generate_batch(m, prompts, lens, 3, 8, &greedy, NULL, 0, outs, counts) == 0);
    printf("\"generated\": [");
    for (int i = 0; i < 3; i++) {
        printf("%s[", i ? ", " : "");
        for (int j = 0; j < counts[i]; j++) printf("%s%d", j ? ", " : "", outs[i][j]);
        printf("]");
    }
    printf("]}\n");
    bn_model_free(m);
    return 0;
}
