/*
 * CPU oracle for the attention hot path of llmtie-rs (TEST INFRASTRUCTURE).
 * PARITY UNPINNED - see oracle.h for what that means and what anchors it.
 * Each function cites the reference routine it restates.
 */
#include "oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <pthread.h>
#include <stdatomic.h>
#include <unistd.h>

/* ---- binary16, round to nearest even ----------------------------------- */

uint16_t orc_f32_to_f16(float x)
{
    uint32_t u;
    memcpy(&u, &x, 4);
    const uint32_t sign = (u >> 16) & 0x8000u;
    const uint32_t mag = u & 0x7fffffffu;
    if (mag >= 0x7f800000u) { /* inf / nan */
        return (uint16_t)(sign | 0x7c00u | ((mag > 0x7f800000u) ? 0x0200u : 0u));
    }
    if (mag >= 0x477ff000u) { /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (mag < 0x33000001u) { /* below half the smallest subnormal -> 0 */
        return (uint16_t)sign;
    }
    int32_t e = (int32_t)(mag >> 23) - 127;
    uint32_t m = (mag & 0x7fffffu) | 0x800000u;
    uint32_t shift;
    uint32_t base;
    if (e < -14) { /* subnormal result */
        shift = (uint32_t)(13 + (-14 - e));
        base = 0;
    } else {
        shift = 13;
        base = (uint32_t)(e + 15) << 10;
        m &= 0x7fffffu;
    }
    uint32_t q = m >> shift;
    const uint32_t rem = m & ((1u << shift) - 1u);
    const uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) {
        q += 1; /* a carry out of the mantissa walks into the exponent, as it should */
    }
    return (uint16_t)(sign | (base + q));
}

float orc_f16_to_f32(uint16_t h)
{
    const uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    const uint32_t e = (h >> 10) & 0x1fu;
    uint32_t m = h & 0x3ffu;
    uint32_t u;
    if (e == 0) {
        if (m == 0) {
            u = sign;
        } else {
            int s = 0;
            while (!(m & 0x400u)) {
                m <<= 1;
                s++;
            }
            m &= 0x3ffu;
            u = sign | ((uint32_t)(127 - 15 - s + 1) << 23) | (m << 13);
        }
    } else if (e == 31) {
        u = sign | 0x7f800000u | (m << 13);
    } else {
        u = sign | ((e + 112u) << 23) | (m << 13);
    }
    float f;
    memcpy(&f, &u, 4);
    return f;
}

void orc_round_f16(const float *src, uint16_t *dst, size_t n)
{
    for (size_t i = 0; i < n; i++) dst[i] = orc_f32_to_f16(src[i]);
}

void orc_widen_f16(const uint16_t *src, float *dst, size_t n)
{
    for (size_t i = 0; i < n; i++) dst[i] = orc_f16_to_f32(src[i]);
}

/* ---- the reference's test generator ------------------------------------ */

/* crates/llmtie-cuda/tests/kernels.rs:35-45 */
void orc_seq(float *out, size_t n, uint64_t salt)
{
    uint64_t s = (salt * 0x9E3779B97F4A7C15ull) | 1ull;
    for (size_t i = 0; i < n; i++) {
        s ^= s << 13;
        s ^= s >> 7;
        s ^= s << 17;
        out[i] = ((float)(s >> 40) / 8388608.0f) * 4.0f - 2.0f;
    }
}

/* ---- RoPE ---------------------------------------------------------------- */

/* crates/llmtie-dsp/src/rope.rs:83-126 */
void orc_rope(float *x, size_t t, size_t heads, size_t hd, float theta,
              size_t first, const float *freq_div)
{
    const size_t half = hd / 2;
    for (size_t p = 0; p < t; p++) {
        for (size_t h = 0; h < heads; h++) {
            const size_t base = (p * heads + h) * hd;
            for (size_t i = 0; i < half; i++) {
                float inv = powf(theta, -2.0f * (float)i / (float)hd);
                if (freq_div) inv /= freq_div[i];
                const float angle = (float)(first + p) * inv;
                const float sn = sinf(angle), cs = cosf(angle);
                const float a = x[base + i], b = x[base + i + half];
                x[base + i] = a * cs - b * sn;
                x[base + i + half] = b * cs + a * sn;
            }
        }
    }
}

/* ---- KV cache ------------------------------------------------------------ */

/* crates/llmtie-cuda/src/kernels.rs:5287-5317 */
void orc_cache_append_f16(const float *src, uint16_t *dst, size_t n,
                          size_t kv_heads, size_t hd, size_t cap, size_t past,
                          int transposed)
{
    const size_t d = kv_heads * hd;
    for (size_t i = 0; i < n * d; i++) {
        const size_t ti = i / d, h = (i % d) / hd, j = i % hd;
        const size_t at = transposed ? (h * hd + j) * cap + past + ti
                                     : (h * cap + past + ti) * hd + j;
        dst[at] = orc_f32_to_f16(src[i]);
    }
}

/* crates/llmtie-cuda/src/kernels.rs:5244-5277 */
void orc_cache_append_f32(const float *src, float *dst, size_t n,
                          size_t kv_heads, size_t hd, size_t cap, size_t past,
                          int transposed)
{
    const size_t d = kv_heads * hd;
    for (size_t i = 0; i < n * d; i++) {
        const size_t ti = i / d, h = (i % d) / hd, j = i % hd;
        const size_t at = transposed ? (h * hd + j) * cap + past + ti
                                     : (h * cap + past + ti) * hd + j;
        dst[at] = src[i];
    }
}

/* crates/llmtie-cuda/src/kernels.rs:5397-5423, run geometry device.rs:3173-3181 */
void orc_cache_grow(const void *src, void *dst, size_t kv_heads, size_t hd,
                    size_t old_cap, size_t new_cap, size_t live,
                    int transposed, size_t esize)
{
    const size_t rows = transposed ? kv_heads * hd : kv_heads;
    const size_t len = transposed ? live : live * hd;
    const size_t ss = transposed ? old_cap : old_cap * hd;
    const size_t ds = transposed ? new_cap : new_cap * hd;
    for (size_t r = 0; r < rows; r++) {
        memcpy((char *)dst + r * ds * esize, (const char *)src + r * ss * esize,
               len * esize);
    }
}

/* crates/llmtie-cuda/src/kernels.rs:5334-5378 */
void orc_rope_cache_f16(float *q, const float *k, const float *v,
                        const float *freq_div, size_t heads, size_t kv_heads,
                        size_t hd, float theta, size_t pos, uint16_t *kc,
                        uint16_t *vc, size_t cap)
{
    const size_t half = hd / 2;
    for (size_t h = 0; h < heads + kv_heads; h++) {
        const int is_q = h < heads;
        const size_t hh = is_q ? h : h - heads;
        for (size_t j = 0; j < half; j++) {
            float inv = powf(theta, -2.0f * (float)j / (float)hd);
            if (freq_div) inv /= freq_div[j];
            const float angle = (float)pos * inv;
            const float sn = sinf(angle), cs = cosf(angle);
            if (is_q) {
                float *b = q + hh * hd + j;
                const float a0 = b[0], b0 = b[half];
                b[0] = a0 * cs - b0 * sn;
                b[half] = b0 * cs + a0 * sn;
            } else {
                const float a0 = k[hh * hd + j], b0 = k[hh * hd + j + half];
                uint16_t *d = kc + (hh * cap + pos) * hd;
                d[j] = orc_f32_to_f16(a0 * cs - b0 * sn);
                d[j + half] = orc_f32_to_f16(b0 * cs + a0 * sn);
            }
        }
    }
    for (size_t e = 0; e < kv_heads * hd; e++) {
        const size_t h = e / hd, j = e % hd;
        vc[(h * hd + j) * cap + pos] = orc_f32_to_f16(v[e]);
    }
}

/* ---- prefill ------------------------------------------------------------- */

/* Widens a cache to f64 through f16: an f32 cache is rounded to f16 first,
 * as the kernel's staging does; an f16 cache is taken as it is. */
static double *widen_cache(const void *p, int f16, size_t n)
{
    double *w = (double *)malloc((n ? n : 1) * sizeof(double));
    for (size_t i = 0; i < n; i++) {
        const uint16_t h = f16 ? ((const uint16_t *)p)[i]
                               : orc_f32_to_f16(((const float *)p)[i]);
        w[i] = (double)orc_f16_to_f32(h);
    }
    return w;
}

/* crates/llmtie-cuda/tests/kernels.rs:2300-2364 */
void orc_prefill(const float *q, size_t q_stride, const void *k, const void *v,
                 int kv_f16, size_t tq, size_t past, size_t tk_override,
                 size_t heads, size_t kv_heads, size_t hd, size_t cap,
                 float scale, int causal, int scale_q, float *out,
                 size_t out_stride)
{
    const size_t tk = tk_override ? tk_override : past + tq;
    const size_t group = heads / kv_heads;
    double *kd = widen_cache(k, kv_f16, kv_heads * cap * hd);
    double *vd = widen_cache(v, kv_f16, kv_heads * cap * hd);
    double *s = (double *)malloc(tk * sizeof(double));
    double *e = (double *)malloc(tk * sizeof(double));
    double *qh = (double *)malloc(hd * sizeof(double));
    for (size_t h = 0; h < heads; h++) {
        const size_t kh = h / group;
        for (size_t r = 0; r < tq; r++) {
            size_t last = causal ? past + r : tk - 1;
            if (last > tk - 1) last = tk - 1;
            for (size_t d = 0; d < hd; d++) {
                const float x = q[r * q_stride + h * hd + d];
                qh[d] = (double)orc_f16_to_f32(
                    orc_f32_to_f16(scale_q ? x * scale : x));
            }
            double m = -INFINITY;
            for (size_t p = 0; p <= last; p++) {
                const double *kr = kd + (kh * cap + p) * hd;
                double acc = 0.0;
                for (size_t d = 0; d < hd; d++) acc += qh[d] * kr[d];
                s[p] = scale_q ? acc : acc * (double)scale;
                if (s[p] > m) m = s[p];
            }
            double l = 0.0;
            for (size_t p = 0; p <= last; p++) {
                const double ep = exp(s[p] - m);
                l += ep; /* the normaliser takes the un-rounded probability */
                e[p] = (double)orc_f16_to_f32(orc_f32_to_f16((float)ep));
            }
            for (size_t d = 0; d < hd; d++) {
                const double *vr = vd + (kh * hd + d) * cap;
                double acc = 0.0;
                for (size_t p = 0; p <= last; p++) acc += e[p] * vr[p];
                out[r * out_stride + h * hd + d] = (float)(acc / l);
            }
        }
    }
    free(s);
    free(e);
    free(qh);
    free(kd);
    free(vd);
}

/* ---- decode -------------------------------------------------------------- */

/* crates/llmtie-cuda/tests/kernels.rs:2733-2774 */
void orc_decode_f32(const float *q, const float *k, const float *v,
                    size_t heads, size_t kv_heads, size_t hd, size_t tk,
                    size_t cap, float scale, int scale_q, float *out)
{
    const size_t group = heads / kv_heads;
    float *s = (float *)malloc(tk * sizeof(float));
    for (size_t qh = 0; qh < heads; qh++) {
        const size_t h = qh / group;
        const float *qr = q + qh * hd;
        for (size_t t = 0; t < tk; t++) {
            const float *kr = k + (h * cap + t) * hd;
            float dot = 0.0f;
            for (size_t d = 0; d < hd; d++) {
                dot += scale_q ? qr[d] * scale * kr[d] : qr[d] * kr[d];
            }
            s[t] = scale_q ? dot : dot * scale;
        }
        float m = -INFINITY;
        for (size_t t = 0; t < tk; t++) m = s[t] > m ? s[t] : m;
        float l = 0.0f;
        for (size_t t = 0; t < tk; t++) {
            s[t] = expf(s[t] - m);
            l += s[t];
        }
        for (size_t d = 0; d < hd; d++) {
            const float *vr = v + (h * hd + d) * cap;
            float acc = 0.0f;
            for (size_t t = 0; t < tk; t++) acc += s[t] * vr[t];
            out[qh * hd + d] = acc / l;
        }
    }
    free(s);
}

/* The same arithmetic at f64 over keys [t0, t1) of an f16 cache; the
 * un-normalised triple follows crates/llmtie-cuda/src/kernels.rs:5836-5879. */
void orc_decode_f64(const float *q, const uint16_t *k, const uint16_t *v,
                    size_t heads, size_t kv_heads, size_t hd, size_t t0,
                    size_t t1, size_t cap, float scale, int scale_q,
                    float *out, float *o_un, float *m_out, float *l_out)
{
    const size_t group = heads / kv_heads;
    const size_t n = t1 - t0;
    double *s = (double *)malloc((n ? n : 1) * sizeof(double));
    for (size_t qh = 0; qh < heads; qh++) {
        const size_t h = qh / group;
        const float *qr = q + qh * hd;
        double m = -INFINITY;
        for (size_t t = t0; t < t1; t++) {
            const uint16_t *kr = k + (h * cap + t) * hd;
            double dot = 0.0;
            for (size_t d = 0; d < hd; d++) {
                const double qd = scale_q ? (double)(qr[d] * scale) : (double)qr[d];
                dot += qd * (double)orc_f16_to_f32(kr[d]);
            }
            s[t - t0] = scale_q ? dot : dot * (double)scale;
            if (s[t - t0] > m) m = s[t - t0];
        }
        double l = 0.0;
        for (size_t t = 0; t < n; t++) {
            s[t] = exp(s[t] - m);
            l += s[t];
        }
        for (size_t d = 0; d < hd; d++) {
            const uint16_t *vr = v + (h * hd + d) * cap + t0;
            double acc = 0.0;
            for (size_t t = 0; t < n; t++) acc += s[t] * (double)orc_f16_to_f32(vr[t]);
            if (out) out[qh * hd + d] = (float)(acc / l);
            if (o_un) o_un[qh * hd + d] = (float)acc;
        }
        if (m_out) m_out[qh] = (float)m;
        if (l_out) l_out[qh] = (float)l;
    }
    free(s);
}

/* crates/llmtie-cuda/src/kernels.rs:5836-5879 */
void orc_quantize_q8(const float *x, size_t n, int8_t *codes, float *scales)
{
    for (size_t g = 0; g < n / 32; g++) {
        float mx = 0.0f;
        for (size_t i = 0; i < 32; i++) {
            const float a = fabsf(x[g * 32 + i]);
            if (a > mx) mx = a;
        }
        const float d = mx * (1.0f / 127.0f);
        const float inv = d > 0.0f ? 1.0f / d : 0.0f;
        for (size_t i = 0; i < 32; i++) {
            /* rintf under the default rounding mode is round-half-even, what
             * __float2int_rn does */
            codes[g * 32 + i] = (int8_t)(int)rintf(x[g * 32 + i] * inv);
        }
        scales[g] = d;
    }
}

void orc_lse_merge(const float *o, const float *m, const float *l,
                   size_t parts, size_t rows, size_t hd, float *out)
{
    for (size_t r = 0; r < rows; r++) {
        double M = -INFINITY;
        for (size_t i = 0; i < parts; i++) {
            if ((double)m[i * rows + r] > M) M = (double)m[i * rows + r];
        }
        double L = 0.0;
        for (size_t i = 0; i < parts; i++) {
            const double mi = (double)m[i * rows + r];
            if (mi == -INFINITY) continue;
            L += (double)l[i * rows + r] * exp(mi - M);
        }
        for (size_t d = 0; d < hd; d++) {
            double acc = 0.0;
            for (size_t i = 0; i < parts; i++) {
                const double mi = (double)m[i * rows + r];
                if (mi == -INFINITY) continue;
                acc += (double)o[(i * rows + r) * hd + d] * exp(mi - M);
            }
            out[r * hd + d] = L > 0.0 ? (float)(acc / L) : 0.0f;
        }
    }
}

/* ---- timed CPU baseline (same arithmetic, f32 accumulation, threads) ----- */

#if defined(__FLT16_MANT_DIG__)
typedef _Float16 h16;
static inline float h2f(const uint16_t *p, size_t i)
{
    return (float)((const h16 *)p)[i];
}
#else
static inline float h2f(const uint16_t *p, size_t i)
{
    return orc_f16_to_f32(p[i]);
}
#endif

int orc_max_threads(void)
{
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    return n > 0 ? (int)n : 1;
}

/* A parallel for over `jobs` with a shared counter: plain pthreads, so the
 * library needs no OpenMP runtime where it lands. */
typedef void (*job_fn)(long job, void *ctx, void *scratch);
struct pool {
    atomic_long next;
    long jobs;
    job_fn fn;
    void *ctx;
    size_t scratch_bytes;
};

static void *pool_worker(void *arg)
{
    struct pool *p = (struct pool *)arg;
    void *scratch = malloc(p->scratch_bytes ? p->scratch_bytes : 1);
    for (;;) {
        const long j = atomic_fetch_add(&p->next, 1);
        if (j >= p->jobs) break;
        p->fn(j, p->ctx, scratch);
    }
    free(scratch);
    return NULL;
}

static void parallel_for(long jobs, int threads, job_fn fn, void *ctx,
                         size_t scratch_bytes)
{
    struct pool p;
    atomic_init(&p.next, 0);
    p.jobs = jobs;
    p.fn = fn;
    p.ctx = ctx;
    p.scratch_bytes = scratch_bytes;
    if (threads <= 1) {
        pool_worker(&p);
        return;
    }
    pthread_t *th = (pthread_t *)malloc((size_t)threads * sizeof(pthread_t));
    int made = 0;
    for (int i = 0; i < threads - 1; i++) {
        if (pthread_create(&th[made], NULL, pool_worker, &p) == 0) made++;
    }
    pool_worker(&p);
    for (int i = 0; i < made; i++) pthread_join(th[i], NULL);
    free(th);
}

struct prefill_ctx {
    const float *q;
    size_t q_stride;
    const void *k, *v;
    int kv_f16;
    size_t tq, past, tk, heads, group, hd, cap;
    float scale;
    int causal, scale_q;
    float *out;
    size_t out_stride;
};

/* One job is eight query rows of one head. */
#define PREFILL_ROWS 8
static void prefill_job(long job, void *vctx, void *scratch)
{
    const struct prefill_ctx *c = (const struct prefill_ctx *)vctx;
    const size_t blocks = (c->tq + PREFILL_ROWS - 1) / PREFILL_ROWS;
    const size_t h = (size_t)job / blocks;
    const size_t r0 = ((size_t)job % blocks) * PREFILL_ROWS;
    const size_t kh = h / c->group, hd = c->hd, cap = c->cap, tk = c->tk;
    float *s = (float *)scratch;
    float *qh = s + tk;
    for (size_t r = r0; r < r0 + PREFILL_ROWS && r < c->tq; r++) {
        size_t last = c->causal ? c->past + r : tk - 1;
        if (last > tk - 1) last = tk - 1;
        for (size_t d = 0; d < hd; d++) {
            const float x = c->q[r * c->q_stride + h * hd + d];
            qh[d] = orc_f16_to_f32(orc_f32_to_f16(c->scale_q ? x * c->scale : x));
        }
        float m = -INFINITY;
        for (size_t p = 0; p <= last; p++) {
            float acc = 0.0f;
            if (c->kv_f16) {
                const uint16_t *kr = (const uint16_t *)c->k + (kh * cap + p) * hd;
                for (size_t d = 0; d < hd; d++) acc += qh[d] * h2f(kr, d);
            } else {
                const float *kr = (const float *)c->k + (kh * cap + p) * hd;
                for (size_t d = 0; d < hd; d++) acc += qh[d] * kr[d];
            }
            s[p] = c->scale_q ? acc : acc * c->scale;
            m = s[p] > m ? s[p] : m;
        }
        float l = 0.0f;
        for (size_t p = 0; p <= last; p++) {
            s[p] = expf(s[p] - m);
            l += s[p];
        }
        for (size_t d = 0; d < hd; d++) {
            float acc = 0.0f;
            if (c->kv_f16) {
                const uint16_t *vr = (const uint16_t *)c->v + (kh * hd + d) * cap;
                for (size_t p = 0; p <= last; p++) acc += s[p] * h2f(vr, p);
            } else {
                const float *vr = (const float *)c->v + (kh * hd + d) * cap;
                for (size_t p = 0; p <= last; p++) acc += s[p] * vr[p];
            }
            c->out[r * c->out_stride + h * hd + d] = acc / l;
        }
    }
}

int orc_prefill_fast(const float *q, size_t q_stride, const void *k,
                     const void *v, int kv_f16, size_t tq, size_t past,
                     size_t tk_override, size_t heads, size_t kv_heads,
                     size_t hd, size_t cap, float scale, int causal,
                     int scale_q, float *out, size_t out_stride, int threads)
{
    struct prefill_ctx c = {q, q_stride, k, v, kv_f16, tq, past,
                            tk_override ? tk_override : past + tq, heads,
                            heads / kv_heads, hd, cap, scale, causal, scale_q,
                            out, out_stride};
    if (threads <= 0) threads = orc_max_threads();
    const size_t blocks = (tq + PREFILL_ROWS - 1) / PREFILL_ROWS;
    parallel_for((long)(heads * blocks), threads, prefill_job, &c,
                 (c.tk + hd) * sizeof(float));
    return threads;
}

/* One job per (query head, key slab); slabs merge with the log-sum-exp
 * algebra so a single long sequence still spreads over every core. */
#define DECODE_SLAB 4096
struct decode_ctx {
    const float *q;
    const uint16_t *k, *v;
    size_t heads, group, hd, tk, cap, slabs;
    float scale;
    int scale_q;
    float *po, *pm, *pl;
};

static void decode_job(long job, void *vctx, void *scratch)
{
    const struct decode_ctx *c = (const struct decode_ctx *)vctx;
    const size_t qh = (size_t)job / c->slabs, sl = (size_t)job % c->slabs;
    const size_t h = qh / c->group, hd = c->hd, cap = c->cap;
    const size_t t0 = sl * DECODE_SLAB;
    const size_t t1 = (t0 + DECODE_SLAB < c->tk) ? t0 + DECODE_SLAB : c->tk;
    float *s = (float *)scratch;
    float *qs = s + DECODE_SLAB;
    for (size_t d = 0; d < hd; d++) {
        qs[d] = c->scale_q ? c->q[qh * hd + d] * c->scale : c->q[qh * hd + d];
    }
    float m = -INFINITY;
    for (size_t t = t0; t < t1; t++) {
        const uint16_t *kr = c->k + (h * cap + t) * hd;
        float dot = 0.0f;
        for (size_t d = 0; d < hd; d++) dot += qs[d] * h2f(kr, d);
        s[t - t0] = c->scale_q ? dot : dot * c->scale;
        m = s[t - t0] > m ? s[t - t0] : m;
    }
    float l = 0.0f;
    for (size_t t = 0; t < t1 - t0; t++) {
        s[t] = expf(s[t] - m);
        l += s[t];
    }
    for (size_t d = 0; d < hd; d++) {
        const uint16_t *vr = c->v + (h * hd + d) * cap + t0;
        float acc = 0.0f;
        for (size_t t = 0; t < t1 - t0; t++) acc += s[t] * h2f(vr, t);
        c->po[(qh * c->slabs + sl) * hd + d] = acc;
    }
    c->pm[qh * c->slabs + sl] = m;
    c->pl[qh * c->slabs + sl] = l;
}

int orc_decode_fast(const float *q, const uint16_t *k, const uint16_t *v,
                    size_t heads, size_t kv_heads, size_t hd, size_t tk,
                    size_t cap, float scale, int scale_q, float *out,
                    int threads)
{
    if (threads <= 0) threads = orc_max_threads();
    const size_t slabs = (tk + DECODE_SLAB - 1) / DECODE_SLAB;
    float *po = (float *)malloc(heads * slabs * hd * sizeof(float));
    float *pm = (float *)malloc(heads * slabs * sizeof(float));
    float *pl = (float *)malloc(heads * slabs * sizeof(float));
    struct decode_ctx c = {q, k, v, heads, heads / kv_heads, hd, tk, cap, slabs,
                           scale, scale_q, po, pm, pl};
    parallel_for((long)(heads * slabs), threads, decode_job, &c,
                 (DECODE_SLAB + hd) * sizeof(float));
    for (size_t qh = 0; qh < heads; qh++) {
        float M = -INFINITY;
        for (size_t i = 0; i < slabs; i++) M = pm[qh * slabs + i] > M ? pm[qh * slabs + i] : M;
        float L = 0.0f;
        for (size_t i = 0; i < slabs; i++) L += pl[qh * slabs + i] * expf(pm[qh * slabs + i] - M);
        for (size_t d = 0; d < hd; d++) {
            float acc = 0.0f;
            for (size_t i = 0; i < slabs; i++) {
                acc += po[(qh * slabs + i) * hd + d] * expf(pm[qh * slabs + i] - M);
            }
            out[qh * hd + d] = acc / L;
        }
    }
    free(po);
    free(pm);
    free(pl);
    return threads;
}

/* ---- Whisper cross-attention cache build -------------------------------------- */

/* crates/llmtie-cuda/src/kernels.rs:5089-5139 (split_heads_f16 and
 * split_heads_t_f16): x f32 [t][heads*hd] plus an optional bias row, rounded
 * to f16 into [heads][cap][hd] or, transposed, [heads][hd][cap]. The
 * reference's buffers have cap == t; positions past t are not written. */
void orc_split_heads_f16(const float *x, const float *bias, uint16_t *out,
                         size_t t, size_t heads, size_t hd, size_t cap,
                         int transposed)
{
    const size_t d = heads * hd;
    for (size_t i = 0; i < t * d; i++) {
        const size_t ti = i / d, h = (i % d) / hd, j = i % hd;
        const float v = x[i] + (bias ? bias[i % d] : 0.0f);
        const size_t at = transposed ? (h * hd + j) * cap + ti
                                     : (h * cap + ti) * hd + j;
        out[at] = orc_f32_to_f16(v);
    }
}

/* crates/llmtie-cuda/src/kernels.rs:5598-5613 (rope_gptj): partial,
 * interleaved rotary embedding in place; the reference's kernel takes the
 * fast sine and cosine, this takes libm's. */
void orc_rope_gptj(float *x, const float *inv_freq, size_t positions,
                   size_t dim, size_t rot_dim)
{
    const size_t pairs = rot_dim / 2;
    for (size_t pos = 0; pos < positions; pos++) {
        for (size_t j = 0; j < pairs; j++) {
            const float ang = (float)pos * inv_freq[j];
            const float c = cosf(ang), s = sinf(ang);
            float *at = x + pos * dim + 2 * j;
            const float a = at[0], b = at[1];
            at[0] = a * c - b * s;
            at[1] = b * c + a * s;
        }
    }
}

/* ---- the stacked attention projection ------------------------------------------ */

/* crates/llmtie-cuda/src/kernels.rs:6876-6913 (gemv_qkv_f16): column c of the
 * stacked [3d][k] f16 weight times the row a, plus its third's bias; q into a
 * row, k into [d/hd][cap][hd] at pos, v into [d][cap] at pos. The reference
 * sums per lane in f32; this sums in f64 and rounds once. */
void orc_gemv_qkv_f16(const float *a, const uint16_t *w, const float *qb,
                      const float *kb, const float *vb, size_t k, size_t d,
                      size_t hd, size_t cap, size_t pos, float *q, float *kc,
                      float *vc)
{
    for (size_t col = 0; col < 3 * d; col++) {
        double acc = 0.0;
        for (size_t i = 0; i < k; i++) {
            acc += (double)a[i] * (double)orc_f16_to_f32(w[col * k + i]);
        }
        const size_t part = col / d, c = col % d;
        if (part == 0) {
            q[c] = (float)acc + (qb ? qb[c] : 0.0f);
        } else if (part == 1) {
            kc[((c / hd) * cap + pos) * hd + c % hd] = (float)acc + (kb ? kb[c] : 0.0f);
        } else {
            vc[c * cap + pos] = (float)acc + (vb ? vb[c] : 0.0f);
        }
    }
}
