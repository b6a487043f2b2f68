/* Times artalis-io/bitnet.c's own engine on a random model of given layer sizes.
 *
 * Links against the objects of an unmodified checkout of the reference (built with its own
 * Makefile) and drives only its public calls: bn_session_create, bn_prefill,
 * bn_prompt_cache_store/restore, bn_transformer_forward, bn_sampler_sample.  The reference loads GGUF files only and has no
 * random-weights mode, so the model is built in memory the way its own session test does
 * (test/test_session.c:16-30): a BnConfig filled by hand and BnQWeight descriptors that point at
 * arrays made here.  Weights are BF16 (BN_GGUF_TENSOR_BF16), activations and caches are what the
 * engine makes them (float32).  The thread pool is the one src/main.c makes
 * (bn_tp_create + bn_tp_set_cpu_decode_policy, src/main.c:1129,1272-1273).
 *
 * The reference serves one sequence per BnSession (include/session.h:12-20); a batch of B
 * requests is B sessions, each stepped once per decode step.  The requests share all but the
 * last token of their prompt: the first session runs the prompt through bn_prefill, its keys
 * and values go into the reference's prompt cache (include/prompt_cache.h), and every other
 * session restores the shared prefix from there and runs its own last token.
 *
 * usage: ref_harness dim hidden layers heads kv_heads head_size vocab seq_len theta eps
 *                    batch prompt_len steps warmup prefill_tokens threads prefill_budget_ms
 * Prints one JSON object: per-step decode times at the batch and for one request alone, the
 * prompt's time, and the time of one prompt of prefill_tokens tokens (left out, -1, if the
 * prompt's time says that it would take longer than prefill_budget_ms).
 */
#include "model.h"
#include "model_internal.h"
#include "session.h"
#include "transformer.h"
#include "generate.h"
#include "sampler.h"
#include "threadpool.h"
#include "platform.h"
#include "gguf.h"
#include "prompt_cache.h"
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

static uint64_t rng_state = 0x9E3779B97F4A7C15ULL;

static inline uint32_t rng_u32(void) {
    rng_state ^= rng_state >> 12; rng_state ^= rng_state << 25; rng_state ^= rng_state >> 27;
    return (uint32_t)((rng_state * 0x2545F4914F6CDD1DULL) >> 32);
}

/* roughly N(0, std): sum of four uniforms, centred */
static inline float rng_normal(float std) {
    float s = 0.f;
    for (int i = 0; i < 4; i++) s += (float)(rng_u32() >> 8) * (1.0f / 16777216.0f);
    return (s - 2.0f) * 1.7320508f * std;
}

static inline uint16_t to_bf16(float v) {
    uint32_t b; memcpy(&b, &v, 4);
    b += 0x7FFFu + ((b >> 16) & 1u);
    return (uint16_t)(b >> 16);
}

/* A BF16 matrix of rows x cols.  The first `fresh` elements are drawn; the rest repeat them, so
 * that 16 GB need not be drawn one value at a time.  Every matrix has memory of its own. */
static uint16_t *bf16_matrix(size_t n, float std) {
    uint16_t *p = (uint16_t *)bn_platform_aligned_alloc(64, n * sizeof(uint16_t));
    if (!p) { fprintf(stderr, "out of memory (%zu bytes)\n", n * 2); exit(1); }
    size_t fresh = n < ((size_t)1 << 22) ? n : ((size_t)1 << 22);
    for (size_t i = 0; i < fresh; i++) p[i] = to_bf16(rng_normal(std));
    for (size_t done = fresh; done < n; ) {
        size_t chunk = n - done < fresh ? n - done : fresh;
        /* shifted by an odd count so that rows do not repeat each other exactly */
        size_t shift = (size_t)(rng_u32() % 4093u);
        if (shift + chunk > fresh) shift = 0;
        memcpy(p + done, p + shift, chunk * sizeof(uint16_t));
        done += chunk;
    }
    return p;
}

static float *ones(int n) {
    float *p = (float *)malloc((size_t)n * sizeof(float));
    for (int i = 0; i < n; i++) p[i] = 1.0f;
    return p;
}

static BnQWeight qw(uint16_t *data, int rows, int cols) {
    BnQWeight w;
    memset(&w, 0, sizeof(w));
    w.data = data; w.type = BN_GGUF_TENSOR_BF16; w.rows = rows; w.cols = cols; w.scale = 1.0f;
    return w;
}

int main(int argc, char **argv) {
    if (argc != 18) {
        fprintf(stderr, "usage: %s dim hidden layers heads kv_heads head_size vocab seq_len theta eps "
                        "batch prompt_len steps warmup prefill_tokens threads prefill_budget_ms\n", argv[0]);
        return 2;
    }
    int dim = atoi(argv[1]), hidden = atoi(argv[2]), L = atoi(argv[3]), H = atoi(argv[4]), KV = atoi(argv[5]),
        hs = atoi(argv[6]), V = atoi(argv[7]), S = atoi(argv[8]);
    float theta = (float)atof(argv[9]), eps = (float)atof(argv[10]);
    int B = atoi(argv[11]), P = atoi(argv[12]), steps = atoi(argv[13]), warmup = atoi(argv[14]),
        prefill_tokens = atoi(argv[15]), threads = atoi(argv[16]);
    double prefill_budget_ms = atof(argv[17]);
    if (P + warmup + steps + 1 > S || prefill_tokens > S) { fprintf(stderr, "context too short\n"); return 2; }

    double t_build = bn_platform_time_ms();
    BnModel m;
    memset(&m, 0, sizeof(m));
    BnConfig *c = &m.config;
    c->dim = dim; c->hidden_dim = hidden; c->n_layers = L; c->n_heads = H; c->n_kv_heads = KV;
    c->vocab_size = V; c->seq_len = S; c->rope_theta = theta; c->norm_eps = eps;
    c->head_size = hs; c->kv_dim = KV * hs; c->kv_mul = H / KV;
    c->has_ffn_gate = 1; c->act_type = BN_MODEL_ACTIVATION_SILU;

    m.weights.token_embedding = bf16_matrix((size_t)V * dim, 0.02f);
    m.weights.emb_type = BN_GGUF_TENSOR_BF16;
    m.weights.layers = (BnLayerWeights *)calloc((size_t)L, sizeof(BnLayerWeights));
    for (int l = 0; l < L; l++) {
        BnLayerWeights *lw = &m.weights.layers[l];
        lw->block_kind = BN_LAYER_BLOCK_ATTENTION;
        lw->ffn_kind = BN_LAYER_FFN_DENSE;
        lw->norm.attn_norm = ones(dim);
        lw->attn.wq = qw(bf16_matrix((size_t)H * hs * dim, 0.02f), H * hs, dim);
        lw->attn.wk = qw(bf16_matrix((size_t)KV * hs * dim, 0.02f), KV * hs, dim);
        lw->attn.wv = qw(bf16_matrix((size_t)KV * hs * dim, 0.02f), KV * hs, dim);
        lw->attn.wo = qw(bf16_matrix((size_t)dim * H * hs, 0.02f), dim, H * hs);
        lw->attn.head_size = hs; lw->attn.kv_dim = KV * hs; lw->attn.kv_mul = H / KV;
        lw->attn.n_kv_heads = KV; lw->attn.q_dim = H * hs; lw->attn.has_kv = 1;
        lw->attn.kv_reuse_layer = -1;
        lw->norm.ffn_norm = ones(dim);
        lw->ffn.ffn_gate = qw(bf16_matrix((size_t)hidden * dim, 0.02f), hidden, dim);
        lw->ffn.ffn_up = qw(bf16_matrix((size_t)hidden * dim, 0.02f), hidden, dim);
        lw->ffn.ffn_down = qw(bf16_matrix((size_t)dim * hidden, 0.02f), dim, hidden);
    }
    m.weights.output_norm = ones(dim);
    m.weights.output_weight = qw(bf16_matrix((size_t)V * dim, 0.02f), V, dim);
    t_build = bn_platform_time_ms() - t_build;

    bn_model_set_thread_pool(&m, bn_tp_create(threads > 1 ? threads - 1 : 0), 1);
    bn_tp_set_cpu_decode_policy(bn_model_pool(&m));

    BnSession **sessions = (BnSession **)calloc((size_t)B, sizeof(BnSession *));
    BnSampler *samplers = (BnSampler *)calloc((size_t)B, sizeof(BnSampler));
    int *next = (int *)calloc((size_t)B, sizeof(int));
    int *pos = (int *)calloc((size_t)B, sizeof(int));
    int *prompt = (int *)malloc((size_t)(P > prefill_tokens ? P : prefill_tokens) * sizeof(int));

    /* the prompts: bn_prefill for the first request, the prompt cache for the others */
    BnPromptCache *pc = bn_prompt_cache_create(0, NULL);
    if (!pc) { fprintf(stderr, "prompt cache create failed\n"); return 1; }
    for (int t = 0; t < P; t++) prompt[t] = (int)(rng_u32() % (uint32_t)V);
    double prompt_ms = 0.0, t_prompts = bn_platform_time_ms();
    for (int b = 0; b < B; b++) {
        sessions[b] = bn_session_create(&m, NULL);
        if (!sessions[b]) { fprintf(stderr, "session create failed\n"); return 1; }
        if (bn_sampler_init(&samplers[b], V, 0.0f, 0.0f, 42) != 0) { fprintf(stderr, "sampler init failed\n"); return 1; }
        int have = 0;
        if (b > 0) {
            prompt[P - 1] = (int)(rng_u32() % (uint32_t)V);
            have = bn_prompt_cache_restore(pc, &m, sessions[b], prompt, P);
            if (have >= P) have = P - 1;
            if (have != (P > 1 ? P - 1 : 0)) { fprintf(stderr, "prompt cache restored %d of %d tokens\n", have, P - 1); return 1; }
        }
        double t0 = bn_platform_time_ms();
        float *logits = bn_prefill(&m, sessions[b], prompt + have, P - have, have, 0);
        if (!logits) { fprintf(stderr, "prefill failed\n"); return 1; }
        sessions[b]->pos = P;  /* the caller keeps a session's position (include/session.h) */
        if (b == 0) {
            prompt_ms = bn_platform_time_ms() - t0;
            if (B > 1 && bn_prompt_cache_store(pc, &m, sessions[0], prompt, P) != 0) {
                fprintf(stderr, "prompt cache store failed\n"); return 1;
            }
        }
        pos[b] = P;
        next[b] = bn_sampler_sample(&samplers[b], logits);
    }
    t_prompts = bn_platform_time_ms() - t_prompts;

    /* decode: one forward and one greedy choice per request per step */
    double *step_ms = (double *)calloc((size_t)(warmup + steps), sizeof(double));
    for (int i = 0; i < warmup + steps; i++) {
        double t0 = bn_platform_time_ms();
        for (int b = 0; b < B; b++) {
            float *logits = bn_transformer_forward(&m, sessions[b], next[b], pos[b]);
            if (!logits) { fprintf(stderr, "forward failed\n"); return 1; }
            pos[b]++;
            next[b] = bn_sampler_sample(&samplers[b], logits);
        }
        step_ms[i] = bn_platform_time_ms() - t0;
    }

    /* the first request alone, going on from where it is */
    int b1_steps = steps < 8 ? steps : 8;
    double *b1_ms = (double *)calloc((size_t)b1_steps + 1, sizeof(double));
    for (int i = 0; i < b1_steps && pos[0] + 1 < S; i++) {
        double t0 = bn_platform_time_ms();
        float *logits = bn_transformer_forward(&m, sessions[0], next[0], pos[0]);
        if (!logits) { fprintf(stderr, "forward failed\n"); return 1; }
        pos[0]++;
        next[0] = bn_sampler_sample(&samplers[0], logits);
        b1_ms[i] = bn_platform_time_ms() - t0;
    }

    /* one prompt of prefill_tokens tokens through bn_prefill in a fresh session */
    double prefill_ms = -1.0;
    double estimate = prompt_ms * (double)prefill_tokens / (double)P * 1.15;
    if (prefill_tokens > 0 && estimate <= prefill_budget_ms) {
        bn_session_reset(sessions[0], &m);
        for (int t = 0; t < prefill_tokens; t++) prompt[t] = (int)(rng_u32() % (uint32_t)V);
        double t0 = bn_platform_time_ms();
        float *logits = bn_prefill(&m, sessions[0], prompt, prefill_tokens, 0, 0);
        prefill_ms = bn_platform_time_ms() - t0;
        if (!logits) { fprintf(stderr, "prefill failed\n"); return 1; }
    }

    printf("{\"threads\": %d, \"build_ms\": %.1f, \"prompts_ms\": %.1f, \"prompt_ms\": %.1f, \"prefill_tokens\": %d, "
           "\"prefill_ms\": %.1f, \"prefill_estimate_ms\": %.1f, \"last_token\": %d, \"step_ms\": [",
           bn_tp_num_threads(bn_model_pool(&m)), t_build, t_prompts, prompt_ms, prefill_tokens, prefill_ms, estimate, next[0]);
    for (int i = warmup; i < warmup + steps; i++) printf("%s%.3f", i > warmup ? ", " : "", step_ms[i]);
    printf("], \"b1_step_ms\": [");
    for (int i = 0; i < b1_steps; i++) printf("%s%.3f", i ? ", " : "", b1_ms[i]);
    printf("]}\n");
    return 0;
}
