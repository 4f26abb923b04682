/*
 * lthn_oracle_decoder.c — CPU reference of one Gemma-style 4-bit decoder built
 * from the reference's own CPU primitives (see lthn_oracle.c).
 *
 * THIS FILE IS TEST INFRASTRUCTURE (checker + timed CPU baseline), never linked
 * into or called by the shipped library.
 *
 * Op order follows the reference's CPU layer oracle
 * engine/hip/hip_gemma4_q4_oracle_test.go:873-961 (hipOracleReferenceLayer) and
 * the device forward engine/hip/hip_gemma4_q4_layer.go:1441-2067, restricted to
 * the gemma3 block declared by model/arch/google/gemma3/gemma3.go:141-161:
 * four block norms, per-head Q/K RMSNorm, full NeoX rotary, AttnScale
 * 1/sqrt(head_dim), no value-norm, no soft-cap, no per-layer input, layer scalar 1,
 * tied embedding / lm_head, embedding scaled by bf16(sqrt(hidden))
 * (hip_gemma4_q4_layer.go:2757-2763). Activations are f32 (the HIP family);
 * projections are hipReferenceMLXAffineProjection (f32 serial); the KV cache
 * holds bf16-rounded K and V (the seq-major bf16 cache of
 * engine/metal/decode_step.go:20-26). Norm weights are the effective weights
 * (the gemma "(1+w)" fold of model/norm_bias.go is applied by the caller).
 * Parity status: each primitive is pinned by the KATs listed in lthn_oracle.c;
 * the composition itself has no golden vector in the reference (its layer oracle
 * needs a downloaded checkpoint and a HIP device), so whole-decoder parity is
 * "pinned by construction from pinned primitives".
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

int lthn_o_hip_affine_projection_rows(const float *x, long tokens, const uint32_t *weights,
                                      const uint16_t *scales, const uint16_t *biases, long rows, long cols,
                                      int gs, int bits, float *out);
int lthn_o_rmsnorm(const float *input, const float *weight, long n, float eps, float *out);
int lthn_o_rope_neox(const float *input, long n, long position, double base, long freq_dim, long rotary,
                     double freq_scale, float *out);
int lthn_o_attention_single_head(const float *query, const float *keys, const float *values, long count,
                                 long dim, long stride, float scale, float *out, float *weights_scratch);
long lthn_o_kv_head_for_query(long query_head, long query_heads, long kv_heads);
void lthn_o_gelu_tanh(const float *input, long n, float *out);
long lthn_o_greedy_f32(const float *logits, long n);
void lthn_o_round_bf16_inplace(float *v, long n);
int lthn_o_affine_embedding_row(const uint32_t *weights, const uint16_t *scales, const uint16_t *biases,
                                long vocab, long hidden, int gs, int bits, long id, float *out);

typedef struct {
    int32_t layers, hidden, q_heads, kv_heads, head_dim, ffn, vocab, gs, bits, max_len;
    float eps, rope_base, attn_scale, embed_scale;
    int32_t kv_bf16; /* 1: round K/V to bf16 when appended */
    /* 1: forwards of more than 32 tokens follow the prefill contract of the reference's Metal
     * engine, which routes M > 1 through affine_qmm_t with bf16 operands (engine/metal/
     * quant_seam_backend.go:37-68,84-110): the activations entering a projection and the
     * dequantised weights are rounded to bf16, products accumulate in f64, outputs stay f32;
     * the attention query is rounded to bf16 too. Shorter forwards (decode) stay f32. */
    int32_t prefill_bf16;
    /* gemma3 sliding/global pattern (model/arch/google/gemma3/gemma3.go:111-158): with sliding_window > 0,
     * block i is a sliding block unless (i+1) % sliding_pattern == 0; a sliding block attends the last
     * sliding_window keys (what the ring of engine/metal/decode_step.go:298-316 holds) and rotates with
     * rope_local_base. */
    int32_t sliding_window, sliding_pattern;
    float rope_local_base;
} lthn_o_decoder_config;

enum { L_Q = 0, L_K, L_V, L_O, L_GATE, L_UP, L_DOWN, L_COUNT };
enum { N_INPUT = 0, N_POST_ATTN, N_PRE_FF, N_POST_FF, N_QNORM, N_KNORM, N_COUNT };

typedef struct { const uint32_t *w; const uint16_t *s, *b; long rows, cols; int bits; /* 0: the model's width */ } lin_t;

typedef struct {
    lthn_o_decoder_config c;
    lin_t *lin;          /* [layers][L_COUNT] */
    const float **norm;  /* [layers][N_COUNT] */
    lin_t embed;         /* [vocab, hidden], tied lm_head */
    const float *final_norm;
    float *kc, *vc;      /* [layers][max_len][kv_heads*head_dim] */
    long pos;
    /* optional stage taps for one layer (set by lthn_o_decoder_set_tap) */
    int tap_layer;
    float *tap[8];
} dec_t;

void *lthn_o_decoder_create(const lthn_o_decoder_config *cfg) {
    dec_t *d = (dec_t *)calloc(1, sizeof(dec_t));
    d->c = *cfg;
    d->lin = (lin_t *)calloc((size_t)cfg->layers * L_COUNT, sizeof(lin_t));
    d->norm = (const float **)calloc((size_t)cfg->layers * N_COUNT, sizeof(float *));
    size_t kv = (size_t)cfg->layers * cfg->max_len * cfg->kv_heads * cfg->head_dim;
    d->kc = (float *)calloc(kv, sizeof(float));
    d->vc = (float *)calloc(kv, sizeof(float));
    d->tap_layer = -1;
    return d;
}
void lthn_o_decoder_destroy(void *h) {
    dec_t *d = (dec_t *)h;
    if (!d) return;
    free(d->lin); free((void *)d->norm); free(d->kc); free(d->vc); free(d);
}
/* Weight pointers are borrowed: the caller keeps the arrays alive. */
int lthn_o_decoder_set_linear(void *h, int layer, int role, const uint32_t *w, const uint16_t *s,
                              const uint16_t *b, long rows, long cols) {
    dec_t *d = (dec_t *)h;
    lin_t l = {w, s, b, rows, cols, 0};
    if (layer < 0) { d->embed = l; return 0; }
    if (layer >= d->c.layers || role < 0 || role >= L_COUNT) return 1;
    d->lin[layer * L_COUNT + role] = l;
    return 0;
}
/* A linear whose quantization override names its own code width (model/quant_config.go:39-88);
 * call after lthn_o_decoder_set_linear. */
int lthn_o_decoder_set_linear_bits(void *h, int layer, int role, int bits) {
    dec_t *d = (dec_t *)h;
    if (layer < 0 || layer >= d->c.layers || role < 0 || role >= L_COUNT) return 1;
    d->lin[layer * L_COUNT + role].bits = bits;
    return 0;
}
int lthn_o_decoder_set_norm(void *h, int layer, int role, const float *w) {
    dec_t *d = (dec_t *)h;
    if (layer < 0) { d->final_norm = w; return 0; }
    if (layer >= d->c.layers || role < 0 || role >= N_COUNT) return 1;
    d->norm[layer * N_COUNT + role] = w;
    return 0;
}
long lthn_o_decoder_pos(void *h) { return ((dec_t *)h)->pos; }
void lthn_o_decoder_reset(void *h) { ((dec_t *)h)->pos = 0; }
/* Stage taps (hipOracleLayerReference fields, oracle_test.go:860-871):
 * 0 inputNorm 1 attention 2 attentionProjection 3 attentionResidual
 * 4 preFeedForward 5 mlp 6 finalHidden 7 query (after norm+rope). Each buffer
 * must hold tokens*width floats for the next forward call. */
void lthn_o_decoder_set_tap(void *h, int layer, int which, float *buf) {
    dec_t *d = (dec_t *)h;
    d->tap_layer = layer;
    if (which >= 0 && which < 8) d->tap[which] = buf;
}

int lthn_o_proj_bf16_contract(const float *x, long tokens, const uint32_t *weights, const uint16_t *scales,
                              const uint16_t *biases, long rows, long cols, int gs, int bits, float *out);
static int g_bf16_contract = 0; /* set per forward call (the oracle is driven from one thread) */
static void proj(const lin_t *l, const float *x, long tokens, int gs, int bits, float *out) {
    if (l->bits) bits = l->bits;
    if (g_bf16_contract) lthn_o_proj_bf16_contract(x, tokens, l->w, l->s, l->b, l->rows, l->cols, gs, bits, out);
    else lthn_o_hip_affine_projection_rows(x, tokens, l->w, l->s, l->b, l->rows, l->cols, gs, bits, out);
}
static void norm_rows(const float *in, const float *w, long rows, long width, float eps, float *out) {
    /* oracle_test.go:981-990 hipOracleReferenceNormRows */
    for (long r = 0; r < rows; r++) lthn_o_rmsnorm(in + r * width, w, width, eps, out + r * width);
}
static void tapcpy(dec_t *d, int layer, int which, const float *src, long n) {
    if (d->tap_layer == layer && d->tap[which]) memcpy(d->tap[which], src, sizeof(float) * (size_t)n);
}

/* Appends n tokens at the current position (prefill when n>1, decode when n==1)
 * and returns the logits of the LAST token (vocab floats) if logits != NULL.
 * hidden_last (hidden floats, after the final norm) is optional. */
int lthn_o_decoder_forward(void *h, const int32_t *ids, long n, float *logits, float *hidden_last) {
    dec_t *d = (dec_t *)h;
    const lthn_o_decoder_config *c = &d->c;
    if (n <= 0 || d->pos + n > c->max_len) return 1;
    const int long_prefill = c->prefill_bf16 && n > 32;
    g_bf16_contract = long_prefill;
    long H = c->hidden, D = c->head_dim, QR = (long)c->q_heads * D, KR = (long)c->kv_heads * D, F = c->ffn;
    float *hid = (float *)malloc(sizeof(float) * n * H);
    float *xn = (float *)malloc(sizeof(float) * n * H);
    float *q = (float *)malloc(sizeof(float) * n * QR);
    float *k = (float *)malloc(sizeof(float) * n * KR);
    float *v = (float *)malloc(sizeof(float) * n * KR);
    float *att = (float *)malloc(sizeof(float) * n * QR);
    float *ao = (float *)malloc(sizeof(float) * n * H);
    float *h1 = (float *)malloc(sizeof(float) * n * H);
    float *gate = (float *)malloc(sizeof(float) * n * F);
    float *up = (float *)malloc(sizeof(float) * n * F);
    float *tmp = (float *)malloc(sizeof(float) * (D > H ? D : H));
    float *sc = (float *)malloc(sizeof(float) * (size_t)c->max_len);

    for (long t = 0; t < n; t++) {
        if (lthn_o_affine_embedding_row(d->embed.w, d->embed.s, d->embed.b, c->vocab, H, c->gs, c->bits, ids[t], hid + t * H))
            return 2;
        for (long i = 0; i < H; i++) hid[t * H + i] = hid[t * H + i] * c->embed_scale;
    }
    for (int L = 0; L < c->layers; L++) {
        const lin_t *lin = d->lin + L * L_COUNT;
        const float **nw = d->norm + L * N_COUNT;
        float *kc = d->kc + (size_t)L * c->max_len * KR, *vc = d->vc + (size_t)L * c->max_len * KR;
        const int pattern = c->sliding_pattern > 0 ? c->sliding_pattern : 6;
        const int sliding = c->sliding_window > 0 && (L + 1) % pattern != 0;
        const double rope_base = sliding ? (double)(c->rope_local_base > 0 ? c->rope_local_base : 10000.0f) : (double)c->rope_base;
        norm_rows(hid, nw[N_INPUT], n, H, c->eps, xn);
        tapcpy(d, L, 0, xn, n * H);
        proj(&lin[L_Q], xn, n, c->gs, c->bits, q);
        proj(&lin[L_K], xn, n, c->gs, c->bits, k);
        proj(&lin[L_V], xn, n, c->gs, c->bits, v);
        /* oracle_test.go:1103-1118 hipOracleNormRoPEHeads: per head RMSNorm then NeoX RoPE */
        for (long t = 0; t < n; t++) {
            long p = d->pos + t;
            for (long hh = 0; hh < c->q_heads; hh++) {
                float *qh = q + t * QR + hh * D;
                lthn_o_rmsnorm(qh, nw[N_QNORM], D, c->eps, tmp);
                lthn_o_rope_neox(tmp, D, p, rope_base, D, D, 1.0, qh);
            }
            for (long hh = 0; hh < c->kv_heads; hh++) {
                float *kh = k + t * KR + hh * D;
                lthn_o_rmsnorm(kh, nw[N_KNORM], D, c->eps, tmp);
                lthn_o_rope_neox(tmp, D, p, rope_base, D, D, 1.0, kh);
            }
            memcpy(kc + p * KR, k + t * KR, sizeof(float) * KR);
            memcpy(vc + p * KR, v + t * KR, sizeof(float) * KR);
            if (c->kv_bf16) { lthn_o_round_bf16_inplace(kc + p * KR, KR); lthn_o_round_bf16_inplace(vc + p * KR, KR); }
        }
        if (long_prefill) lthn_o_round_bf16_inplace(q, n * QR); /* the prefill attention multiplies bf16 queries */
        tapcpy(d, L, 7, q, n * QR);
        /* oracle_test.go:907-924: causal attention per token, GQA head map */
#pragma omp parallel
        {
            float *lsc = (float *)malloc(sizeof(float) * (size_t)c->max_len);
#pragma omp for collapse(2) schedule(dynamic)
            for (long t = 0; t < n; t++)
                for (long hh = 0; hh < c->q_heads; hh++) {
                    long kvh = lthn_o_kv_head_for_query(hh, c->q_heads, c->kv_heads);
                    const long count = d->pos + t + 1;
                    const long first = sliding && count > c->sliding_window ? count - c->sliding_window : 0;
                    lthn_o_attention_single_head(q + t * QR + hh * D, kc + first * KR + kvh * D, vc + first * KR + kvh * D, count - first, D, KR,
                                                 c->attn_scale, att + t * QR + hh * D, lsc);
                }
            free(lsc);
        }
        tapcpy(d, L, 1, att, n * QR);
        proj(&lin[L_O], att, n, c->gs, c->bits, ao);
        tapcpy(d, L, 2, ao, n * H);
        norm_rows(ao, nw[N_POST_ATTN], n, H, c->eps, xn);
        for (long i = 0; i < n * H; i++) h1[i] = hid[i] + xn[i] * 1.0f; /* hipOracleAddRows scale 1 */
        tapcpy(d, L, 3, h1, n * H);
        norm_rows(h1, nw[N_PRE_FF], n, H, c->eps, xn);
        tapcpy(d, L, 4, xn, n * H);
        proj(&lin[L_GATE], xn, n, c->gs, c->bits, gate);
        proj(&lin[L_UP], xn, n, c->gs, c->bits, up);
        lthn_o_gelu_tanh(gate, n * F, gate);
        for (long i = 0; i < n * F; i++) gate[i] = gate[i] * up[i]; /* hipGemma4Q4HostMultiply */
        proj(&lin[L_DOWN], gate, n, c->gs, c->bits, ao);
        tapcpy(d, L, 5, ao, n * H);
        norm_rows(ao, nw[N_POST_FF], n, H, c->eps, xn);
        for (long i = 0; i < n * H; i++) hid[i] = h1[i] + xn[i] * 1.0f;
        tapcpy(d, L, 6, hid, n * H);
    }
    d->pos += n;
    g_bf16_contract = 0; /* the lm_head of the last row is a single-row matvec: f32 like decode */
    if (logits || hidden_last) {
        lthn_o_rmsnorm(hid + (n - 1) * H, d->final_norm, H, c->eps, xn);
        if (hidden_last) memcpy(hidden_last, xn, sizeof(float) * H);
        if (logits) proj(&d->embed, xn, 1, c->gs, c->bits, logits);
    }
    g_bf16_contract = 0;
    free(hid); free(xn); free(q); free(k); free(v); free(att); free(ao); free(h1); free(gate); free(up); free(tmp); free(sc);
    return 0;
}

/* Greedy continuation (engine/session.go:49 GenerateFromCacheEach semantics with
 * eosID<0). The caller has prefilled and passes the last prompt token's logits;
 * their argmax is generated token 0, which is fed back to produce token 1, and so
 * on. The last generated token is not fed. Per step the top-1 minus top-2 logit
 * margin is recorded so a harness can tell a real divergence from a numerical
 * near-tie. first_logits: vocab floats from the prefill call. */
int lthn_o_decoder_generate(void *h, const float *first_logits, long max_new, int32_t *out_ids, float *out_margin) {
    dec_t *d = (dec_t *)h;
    long V = d->c.vocab;
    float *logits = (float *)malloc(sizeof(float) * V);
    memcpy(logits, first_logits, sizeof(float) * V);
    for (long i = 0; i < max_new; i++) {
        long best = lthn_o_greedy_f32(logits, V);
        float second = -INFINITY;
        for (long j = 0; j < V; j++) if (j != best && logits[j] > second) second = logits[j];
        out_ids[i] = (int32_t)best;
        if (out_margin) out_margin[i] = logits[best] - second;
        if (i + 1 == max_new) break;
        int32_t id = (int32_t)best;
        int rc = lthn_o_decoder_forward(h, &id, 1, logits, NULL);
        if (rc) { free(logits); return rc; }
    }
    free(logits);
    return 0;
}

/* KV cache read-out for parity checks: copies K (which=0) or V (which=1) of
 * `layer`, positions [0,pos), as f32 [pos, kv_heads*head_dim]. */
void lthn_o_decoder_read_kv(void *h, int layer, int which, float *out) {
    dec_t *d = (dec_t *)h;
    long KR = (long)d->c.kv_heads * d->c.head_dim;
    const float *src = (which ? d->vc : d->kc) + (size_t)layer * d->c.max_len * KR;
    memcpy(out, src, sizeof(float) * (size_t)d->pos * KR);
}
