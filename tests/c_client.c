/*
 * A caller of libllmtie_b200.so written in plain C, the way the reference's
 * Rust `Gpu` methods would call it: no Python, no torch, nothing but the
 * header. One layer's life on one sequence - prefill a prompt, then decode a
 * token - through the entry points that replace
 *   zeros_f16 / the cache policy   (crates/llmtie-chat/src/model.rs:714-747)
 *   rope_scaled, cache_append_f16  (src/model.rs:848-889)
 *   flash_attn_f16                 (crates/llmtie-cuda/src/device.rs:5754-5799)
 *   rope_cache_f16                 (device.rs:2915-3000)
 *   attn_decode_f16 and its twin   (device.rs:5949-6038)
 * and checks every result against the oracle library built from oracle/oracle.c
 * (test infrastructure: linked here as the checker only).
 *
 * Built and run by tests/test_gpu_c_client.py:
 *   gcc -O2 -I include -I oracle tests/c_client.c -o <tmp>/c_client \
 *       -L ttsxabe_b200 -lllmtie_b200 -L oracle -loracle -lm
 * Prints one line per check and exits non-zero at the first failure.
 */
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "llmtie_b200.h"
#include "oracle.h"

#define CHECK(call)                                                                   \
    do {                                                                              \
        const llmtie_status st_ = (call);                                             \
        if (st_ != LLMTIE_OK) {                                                       \
            fprintf(stderr, "%s:%d: %s -> %d: %s\n", __FILE__, __LINE__, #call, st_, \
                    llmtie_last_error());                                             \
            return 1;                                                                 \
        }                                                                             \
    } while (0)

static int close_to(const char *what, const float *want, const float *got, size_t n,
                    double max_abs, double rel_l2)
{
    /* max_abs is a fraction of the largest expected magnitude (the generator's
     * values reach 6, so the outputs are not of order one) */
    double worst = 0.0, num = 0.0, den = 0.0, full = 1.0;
    for (size_t i = 0; i < n; i++) {
        const double d = fabs((double)want[i] - (double)got[i]);
        if (!(d <= worst)) worst = d;   /* catches NaN as well */
        if (fabs((double)want[i]) > full) full = fabs((double)want[i]);
        num += d * d;
        den += (double)want[i] * (double)want[i];
    }
    const double rel = den > 0.0 ? sqrt(num / den) : sqrt(num);
    const int ok = worst <= max_abs * full && rel <= rel_l2;
    printf("%-34s max-abs %.3e  rel-L2 %.3e  %s\n", what, worst, rel, ok ? "ok" : "FAIL");
    return ok ? 0 : 1;
}

int main(void)
{
    const size_t heads = 8, kv = 2, hd = 128, prompt = 200, max_pos = 4096;
    const size_t nq = heads * hd, nkv = kv * hd;
    const float theta = 10000.0f, scale = 1.0f / sqrtf((float)hd);

    llmtie_gpu *g = NULL;
    CHECK(llmtie_open(0, &g));

    /* the cache policy: an empty cache that must take the prompt */
    const size_t cap = llmtie_kv_want_capacity(0, 0, prompt, max_pos);
    if (cap != 512) {   /* next_pow2(200 + 256) */
        fprintf(stderr, "capacity policy: wanted 512, got %zu\n", cap);
        return 1;
    }
    uint16_t *kc = NULL, *vc = NULL;
    CHECK(llmtie_kv_alloc_f16(g, kv, hd, cap, &kc, &vc));

    /* host activations: the reference's own test generator, rounded through f16 */
    float *q = malloc(prompt * nq * sizeof(float));
    float *k = malloc(prompt * nkv * sizeof(float));
    float *v = malloc(prompt * nkv * sizeof(float));
    uint16_t *tmp = malloc(prompt * nq * sizeof(uint16_t));
    orc_seq(q, prompt * nq, 11);
    orc_seq(k, prompt * nkv, 12);
    orc_seq(v, prompt * nkv, 13);
    orc_round_f16(q, tmp, prompt * nq), orc_widen_f16(tmp, q, prompt * nq);
    orc_round_f16(k, tmp, prompt * nkv), orc_widen_f16(tmp, k, prompt * nkv);
    orc_round_f16(v, tmp, prompt * nkv), orc_widen_f16(tmp, v, prompt * nkv);

    float *dq = NULL, *dk = NULL, *dv = NULL, *dout = NULL;
    CHECK(llmtie_alloc(g, prompt * nq * sizeof(float), (void **)&dq));
    CHECK(llmtie_alloc(g, prompt * nkv * sizeof(float), (void **)&dk));
    CHECK(llmtie_alloc(g, prompt * nkv * sizeof(float), (void **)&dv));
    CHECK(llmtie_alloc(g, prompt * nq * sizeof(float), (void **)&dout));
    CHECK(llmtie_upload(g, dq, q, prompt * nq * sizeof(float)));
    CHECK(llmtie_upload(g, dk, k, prompt * nkv * sizeof(float)));
    CHECK(llmtie_upload(g, dv, v, prompt * nkv * sizeof(float)));

    /* ---- prefill: rope q and k, append k and v, attend -------------------------- */
    CHECK(llmtie_rope_scaled(g, dq, prompt * nq, 0, NULL, prompt, heads, hd, theta, 0));
    CHECK(llmtie_rope_scaled(g, dk, prompt * nkv, 0, NULL, prompt, kv, hd, theta, 0));
    CHECK(llmtie_cache_append_f16(g, dk, prompt * nkv, 0, kc, kv * cap * hd, prompt, kv, hd, cap, 0,
                                  0));
    CHECK(llmtie_cache_append_f16(g, dv, prompt * nkv, 0, vc, kv * cap * hd, prompt, kv, hd, cap, 0,
                                  1));
    CHECK(llmtie_flash_attn_f16(g, dq, prompt * nq, kc, kv * cap * hd, vc, kv * cap * hd, dout,
                                prompt * nq, prompt, 0, heads, kv, hd, cap, scale, 1));
    float *got = malloc(prompt * nq * sizeof(float));
    uint16_t *hk = malloc(kv * cap * hd * sizeof(uint16_t));
    uint16_t *hv = malloc(kv * cap * hd * sizeof(uint16_t));
    CHECK(llmtie_download(g, got, dout, prompt * nq * sizeof(float)));
    CHECK(llmtie_download(g, hk, kc, kv * cap * hd * sizeof(uint16_t)));
    CHECK(llmtie_download(g, hv, vc, kv * cap * hd * sizeof(uint16_t)));

    /* the oracle's side of the same steps */
    float *oq = malloc(prompt * nq * sizeof(float));
    float *ok_ = malloc(prompt * nkv * sizeof(float));
    memcpy(oq, q, prompt * nq * sizeof(float));
    memcpy(ok_, k, prompt * nkv * sizeof(float));
    orc_rope(oq, prompt, heads, hd, theta, 0, NULL);
    orc_rope(ok_, prompt, kv, hd, theta, 0, NULL);
    uint16_t *wk = calloc(kv * cap * hd, sizeof(uint16_t));
    uint16_t *wv = calloc(kv * cap * hd, sizeof(uint16_t));
    orc_cache_append_f16(ok_, wk, prompt, kv, hd, cap, 0, 0);
    orc_cache_append_f16(v, wv, prompt, kv, hd, cap, 0, 1);
    int bad = 0;
    if (memcmp(hv, wv, kv * cap * hd * sizeof(uint16_t)) != 0) {
        printf("value cache differs from the oracle's FAIL\n");
        bad = 1;
    } else {
        printf("%-34s bit for bit  ok\n", "value cache (transposed f16)");
    }
    {
        /* rotated keys: device sincosf and the host's may differ in the last bit */
        float *a = malloc(kv * cap * hd * sizeof(float)), *b = malloc(kv * cap * hd * sizeof(float));
        orc_widen_f16(hk, a, kv * cap * hd);
        orc_widen_f16(wk, b, kv * cap * hd);
        bad |= close_to("key cache (rotated, f16)", b, a, kv * cap * hd, 4e-3, 1e-3);
        free(a), free(b);
    }
    float *want = malloc(prompt * nq * sizeof(float));
    /* attention over the caches the DEVICE wrote, so that only attention is compared */
    orc_prefill(oq, nq, hk, hv, 1, prompt, 0, 0, heads, kv, hd, cap, scale, 1, 0, want, nq);
    bad |= close_to("prefill, 200 tokens, causal", want, got, prompt * nq, 2e-3, 1e-3);

    /* ---- decode one token: fused rope + cache write, attention, int8 twin -------- */
    float tok[3 * 1024];
    orc_seq(tok, nq + 2 * nkv, 21);
    orc_round_f16(tok, tmp, nq + 2 * nkv), orc_widen_f16(tmp, tok, nq + 2 * nkv);
    float *dtok = NULL, *dctx = NULL, *dsc = NULL;
    int8_t *dcodes = NULL;
    CHECK(llmtie_alloc(g, (nq + 2 * nkv) * sizeof(float), (void **)&dtok));
    CHECK(llmtie_alloc(g, nq * sizeof(float), (void **)&dctx));
    CHECK(llmtie_zeros(g, nq, (void **)&dcodes));
    CHECK(llmtie_zeros(g, nq / 32 * sizeof(float), (void **)&dsc));
    CHECK(llmtie_upload(g, dtok, tok, (nq + 2 * nkv) * sizeof(float)));
    /* q, k and v are offsets into one allocation, as a stacked projection leaves them */
    CHECK(llmtie_rope_cache_f16(g, dtok, nq + 2 * nkv, 0, dtok, nq + 2 * nkv, nq, dtok,
                                nq + 2 * nkv, nq + nkv, NULL, heads, kv, hd, theta, prompt, kc,
                                kv * cap * hd, vc, kv * cap * hd, cap));
    llmtie_decode_scratch *scratch = NULL;
    CHECK(llmtie_decode_scratch_new(g, &scratch));
    CHECK(llmtie_attn_decode_f16_q(g, dtok, nq + 2 * nkv, 0, kc, kv * cap * hd, vc, kv * cap * hd,
                                   heads, kv, hd, prompt + 1, cap, scale, 0, scratch, dctx, nq, 0,
                                   dcodes, nq, dsc, nq / 32));
    float ctx[1024], sc[32], rq[1024];
    int8_t codes[1024];
    CHECK(llmtie_download(g, ctx, dctx, nq * sizeof(float)));
    CHECK(llmtie_download(g, codes, dcodes, nq));
    CHECK(llmtie_download(g, sc, dsc, nq / 32 * sizeof(float)));
    CHECK(llmtie_download(g, rq, dtok, nq * sizeof(float)));   /* the rotated query */
    CHECK(llmtie_download(g, hk, kc, kv * cap * hd * sizeof(uint16_t)));
    CHECK(llmtie_download(g, hv, vc, kv * cap * hd * sizeof(uint16_t)));
    float wctx[1024];
    orc_decode_f64(rq, hk, hv, heads, kv, hd, 0, prompt + 1, cap, scale, 0, wctx, NULL, NULL, NULL);
    bad |= close_to("decode, 201 keys", wctx, ctx, nq, 2e-5, 1e-4);
    int8_t wc[1024];
    float ws[32];
    orc_quantize_q8(ctx, nq, wc, ws);
    const int twin_ok = memcmp(wc, codes, nq) == 0 && memcmp(ws, sc, nq / 32 * sizeof(float)) == 0;
    printf("%-34s %s\n", "int8 twin of the context", twin_ok ? "bit for bit  ok" : "FAIL");
    bad |= !twin_ok;

    /* ---- a refusal names what is wrong and launches nothing ----------------------- */
    const llmtie_status refused = llmtie_flash_attn_f16(g, dq, prompt * nq, kc, kv * cap * hd, vc,
                                                        kv * cap * hd, dout, prompt * nq, prompt,
                                                        cap, heads, kv, hd, cap, scale, 1);
    printf("%-34s status %d (%s)  %s\n", "past + tq beyond the capacity", refused,
           llmtie_last_error(), refused == LLMTIE_ERR_CACHE_OVERRUN ? "ok" : "FAIL");
    bad |= refused != LLMTIE_ERR_CACHE_OVERRUN;

    CHECK(llmtie_synchronize(g));
    llmtie_decode_scratch_free(g, scratch);
    llmtie_free(g, dq), llmtie_free(g, dk), llmtie_free(g, dv), llmtie_free(g, dout);
    llmtie_free(g, dtok), llmtie_free(g, dctx), llmtie_free(g, dcodes), llmtie_free(g, dsc);
    llmtie_free(g, kc), llmtie_free(g, vc);
    llmtie_close(g);
    printf(bad ? "FAILED\n" : "all checks passed\n");
    return bad;
}
