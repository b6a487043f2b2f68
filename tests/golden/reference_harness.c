/* Drives the reference's own CPU engine (artalis-io/bitnet.c) on a tiny random model.
 *
 * The reference loads GGUF files only and its loader refuses widths that are not multiples
 * of 128 (src/model.c:303-310), so the model is built in memory the way the reference's own
 * session test does (test/test_session.c:16-30): a BnConfig filled by hand and BnQWeight
 * descriptors of type F32 that point at arrays read from a flat file.  Then it runs
 * bn_transformer_forward token by token and bn_transformer_prefill over the whole prompt and
 * writes the logits.  Built and run by make_golden.py; not part of the library.
 *
 * Input file: int32 header {dim, hidden_dim, n_layers, n_heads, n_kv_heads, vocab, seq_len,
 * head_size, tied, n_tokens}, float32 {rope_theta, norm_eps}, int32 tokens[n_tokens], then
 * float32 weights: token_embd, per layer attn_norm, wq, wk, wv, wo, ffn_norm, gate, up, down,
 * then output_norm and (if not tied) output.
 * Output file: float32 [n_tokens, vocab] from token-by-token forward, then float32 [vocab]
 * from the prefill of the whole prompt.
 *
 * With a third and fourth argument it also runs the reference's sampler (src/sampler.c) over
 * the token-by-token logits.  Settings file: int32 n, then n records of float32 {temperature,
 * top_p, repeat_penalty, logit_scale} and int32 {seed, window}.  For each setting a sampler is
 * made (bn_sampler_init, bn_sampler_set_repeat_penalty when the penalty is above 1), the prompt's
 * tokens are accepted as src/main.c:1648 does, and for every position t one id is drawn from
 * logits[t] * logit_scale and accepted.  Output: int32 [n, n_tokens].
 */
#include "model.h"
#include "session.h"
#include "transformer.h"
#include "gguf.h"
#include "sampler.h"
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

static float *take(float **cursor, size_t n) { float *p = *cursor; *cursor += n; return p; }

static BnQWeight qw(float *data, int rows, int cols) {
    BnQWeight w;
    memset(&w, 0, sizeof(w));
    w.data = data; w.type = BN_GGUF_TENSOR_F32; w.rows = rows; w.cols = cols; w.scale = 1.0f;
    return w;
}

int main(int argc, char **argv) {
    if (argc != 3 && argc != 5) { fprintf(stderr, "usage: %s in.bin out.bin [settings.bin ids.bin]\n", argv[0]); return 2; }
    FILE *f = fopen(argv[1], "rb");
    if (!f) { perror("open"); return 1; }
    fseek(f, 0, SEEK_END); long size = ftell(f); fseek(f, 0, SEEK_SET);
    char *buf = malloc(size);
    if (fread(buf, 1, size, f) != (size_t)size) { perror("read"); return 1; }
    fclose(f);
    int *hi = (int *)buf;
    int dim = hi[0], hidden = hi[1], L = hi[2], H = hi[3], KV = hi[4], V = hi[5], S = hi[6], hs = hi[7],
        tied = hi[8], T = hi[9];
    float *hf = (float *)(hi + 10);
    float theta = hf[0], eps = hf[1];
    int *tokens = (int *)(hf + 2);
    float *cur = (float *)(tokens + T);

    BnModel m;
    memset(&m, 0, sizeof(m));
    BnConfig *c = &m.config;
    c->dim = dim; c->hidden_dim = hidden; c->n_layers = L; c->n_heads = H; c->n_kv_heads = KV;
    c->vocab_size = V; c->seq_len = S; c->rope_theta = theta; c->norm_eps = eps;
    c->head_size = hs; c->kv_dim = KV * hs; c->kv_mul = H / KV;
    c->has_ffn_gate = 1; c->act_type = BN_MODEL_ACTIVATION_SILU;

    m.weights.token_embedding = take(&cur, (size_t)V * dim);
    m.weights.emb_type = BN_GGUF_TENSOR_F32;
    m.weights.layers = calloc(L, sizeof(BnLayerWeights));
    for (int l = 0; l < L; l++) {
        BnLayerWeights *lw = &m.weights.layers[l];
        lw->block_kind = BN_LAYER_BLOCK_ATTENTION;
        lw->ffn_kind = BN_LAYER_FFN_DENSE;
        lw->norm.attn_norm = take(&cur, dim);
        lw->attn.wq = qw(take(&cur, (size_t)H * hs * dim), H * hs, dim);
        lw->attn.wk = qw(take(&cur, (size_t)KV * hs * dim), KV * hs, dim);
        lw->attn.wv = qw(take(&cur, (size_t)KV * hs * dim), KV * hs, dim);
        lw->attn.wo = qw(take(&cur, (size_t)dim * H * hs), dim, H * hs);
        lw->attn.head_size = hs; lw->attn.kv_dim = KV * hs; lw->attn.kv_mul = H / KV;
        lw->attn.n_kv_heads = KV; lw->attn.q_dim = H * hs; lw->attn.has_kv = 1;
        lw->attn.kv_reuse_layer = -1;
        lw->norm.ffn_norm = take(&cur, dim);
        lw->ffn.ffn_gate = qw(take(&cur, (size_t)hidden * dim), hidden, dim);
        lw->ffn.ffn_up = qw(take(&cur, (size_t)hidden * dim), hidden, dim);
        lw->ffn.ffn_down = qw(take(&cur, (size_t)dim * hidden), dim, hidden);
    }
    m.weights.output_norm = take(&cur, dim);
    if (!tied) m.weights.output_weight = qw(take(&cur, (size_t)V * dim), V, dim);
    if ((char *)cur - buf != size) { fprintf(stderr, "input size mismatch\n"); return 1; }

    FILE *o = fopen(argv[2], "wb");
    BnSession *s = bn_session_create(&m, NULL);
    if (!s) { fprintf(stderr, "session create failed\n"); return 1; }
    float *all = malloc((size_t)T * V * sizeof(float));
    for (int t = 0; t < T; t++) {
        float *logits = bn_transformer_forward(&m, s, tokens[t], t);
        if (!logits) { fprintf(stderr, "forward failed at %d\n", t); return 1; }
        fwrite(logits, sizeof(float), V, o);
        memcpy(all + (size_t)t * V, logits, (size_t)V * sizeof(float));
    }
    bn_session_reset(s, &m);
    float *pl = bn_transformer_prefill(&m, s, tokens, T, 0);
    if (!pl) { fprintf(stderr, "prefill failed\n"); return 1; }
    fwrite(pl, sizeof(float), V, o);
    fclose(o);
    bn_session_free(s, NULL);
    if (argc == 5) {
        FILE *sf = fopen(argv[3], "rb");
        FILE *idf = fopen(argv[4], "wb");
        int n = 0;
        if (!sf || !idf || fread(&n, sizeof(int), 1, sf) != 1) { fprintf(stderr, "settings unreadable\n"); return 1; }
        float *buf = malloc((size_t)V * sizeof(float));
        for (int i = 0; i < n; i++) {
            float f[4]; int k[2];
            if (fread(f, sizeof(float), 4, sf) != 4 || fread(k, sizeof(int), 2, sf) != 2) { fprintf(stderr, "settings short\n"); return 1; }
            BnSampler sp;
            if (bn_sampler_init(&sp, V, f[0], f[1], (uint64_t)k[0]) != 0) return 1;
            if (f[2] > 1.0f) bn_sampler_set_repeat_penalty(&sp, f[2], k[1]);
            for (int t = 0; t < T; t++) bn_sampler_accept(&sp, tokens[t]);
            for (int t = 0; t < T; t++) {
                for (int v = 0; v < V; v++) buf[v] = all[(size_t)t * V + v] * f[3];
                int id = bn_sampler_sample(&sp, buf);
                bn_sampler_accept(&sp, id);
                fwrite(&id, sizeof(int), 1, idf);
            }
            bn_sampler_free(&sp);
        }
        fclose(sf); fclose(idf);
    }
    return 0;
}
