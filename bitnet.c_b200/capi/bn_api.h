/* C interface of bitnet.c_b200, in the shape of artalis-io/bitnet.c's public headers
 * (include/model.h:22-38, include/session.h:25-31, include/transformer.h:9-30,
 * include/generate.h:51-71, include/sampler.h:33-38): an immutable model shared by all
 * requests, a session per request, prefill and single-token forward that return a pointer to
 * float32 logits, a sampler, and a generate call.  What this library adds to that shape is the
 * batch: a cache that many sessions live in, one step for a batch of sessions, and
 * bn_generate_batch.
 *
 * The engine behind it is this library's one engine: its model, cache, step function, generation
 * loop and CUDA kernels.  The interface holds no forward pass, cache or loader of its own; it
 * carries the calls into the library's Python host (an interpreter embedded in this shared
 * object, started by the first call) and the results back as plain C arrays.
 *
 * Errors: functions that return pointers return NULL, functions that return int return a
 * negative value; bn_last_error() then gives the message.  Not thread-safe: call from one
 * thread at a time.
 */
#ifndef BN_B200_API_H
#define BN_B200_API_H

#ifdef __cplusplus
extern "C" {
#endif

typedef struct BnModel BnModel;     /* immutable after load, shared by all sessions */
typedef struct BnSession BnSession; /* one request: a slot of the model's cache and its position */

typedef struct {
    int max_tokens;        /* tokens all live sessions may hold together, each rounded up to 64 (0: max_seqs x context) */
    int max_seqs;          /* sessions alive at the same time */
} BnCacheParams;

typedef struct {
    float temperature;     /* 0 = greedy */
    float topp;            /* nucleus, used when temperature > 0; <= 0 or >= 1: off */
    float repeat_penalty;  /* 1 = off */
    int repeat_window;     /* recent tokens the penalty looks at (the reference: 64) */
    unsigned long long seed;
} BnSamplerParams;

/* model_dir: a folder with config.json and model.safetensors.  dtype: "bfloat16" or "float32".
 * max_seq_len > 0 caps the context (the reference's --maxseq).  The cache is created with the
 * model (a session is a slot of it). */
BnModel *bn_model_load(const char *model_dir, const char *dtype, int max_seq_len, const BnCacheParams *cache);
void bn_model_free(BnModel *m);
int bn_model_vocab_size(const BnModel *m);
int bn_model_seq_len(const BnModel *m);

BnSession *bn_session_create(BnModel *m);
void bn_session_free(BnSession *s);
/* Forget the session's tokens; its slot stays. */
int bn_session_reset(BnSession *s);
int bn_session_pos(const BnSession *s);

/* n_tokens from position pos0 on (pos0 must be the session's position); logits of the last
 * token, [vocab] floats owned by the session and valid until its next call.  no_prefill != 0
 * feeds the tokens one per step. */
const float *bn_prefill(BnModel *m, BnSession *s, const int *tokens, int n_tokens, int pos0, int no_prefill);
int bn_prefill_no_logits(BnModel *m, BnSession *s, const int *tokens, int n_tokens, int pos0, int no_prefill);
/* One token at position pos (the session's position). */
const float *bn_transformer_forward(BnModel *m, BnSession *s, int token, int pos);
/* Logits at every position: all_logits is [n_tokens * vocab], caller-allocated. */
int bn_transformer_prefill_all(BnModel *m, BnSession *s, const int *tokens, int n_tokens, int pos0, float *all_logits);

/* One step of a batch: session i brings n_new[i] tokens (packed in tokens) and wants the logits
 * of its last token in logits_out[i * vocab ...] (logits_out may be NULL).  The sessions either
 * all start or all go on; see the library's step function. */
int bn_step(BnModel *m, BnSession *const *sessions, int n_sessions, const int *n_new, const int *tokens, float *logits_out);

/* Sample one token from logits with the reference's sampler (greedy with the lowest index on
 * ties, temperature, nucleus, repeat penalty over the tokens accepted so far; xorshift64*). */
typedef struct BnSampler BnSampler;
BnSampler *bn_sampler_create(int vocab_size, const BnSamplerParams *params);
void bn_sampler_free(BnSampler *s);
void bn_sampler_accept(BnSampler *s, int token);
int bn_sampler_sample(BnSampler *s, const float *logits);

/* Generate for n prompts as batches that start together (all prompts in one step, then one token
 * per running request per step; a request that ends leaves the batch).  out_tokens[i] must hold
 * max_new_tokens ints; out_counts[i] receives the number generated.  stop_ids may be NULL. */
int bn_generate_batch(BnModel *m, const int *const *prompts, const int *prompt_lens, int n_prompts, int max_new_tokens,
                      const BnSamplerParams *sampling, const int *stop_ids, int n_stop_ids, int *const *out_tokens,
                      int *out_counts);

const char *bn_last_error(void);

#ifdef __cplusplus
}
#endif
#endif
