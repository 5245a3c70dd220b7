/*
 * CPU oracle for the attention hot path of llmtie-rs (TEST INFRASTRUCTURE).
 *
 * PARITY UNPINNED: the reference ships no golden vectors or known-answer
 * files for attention, RoPE or the KV cache, and it cannot be compiled where
 * this oracle was written (Rust, no toolchain). Every function below is a
 * restatement, in plain C, of a scalar routine of the reference, cited by the
 * reference's file:line. What anchors it is (1) the reference's own test
 * generator `seq`, restated bit for bit, so its test cases are reproduced on
 * identical inputs, (2) an independent numpy restatement that the tests diff
 * against this C code, and (3) analytic known answers.
 *
 * Nothing shipped may call into this library: only tests, the smoke check and
 * the benchmark's cpu_baseline / reference arm use it, as the checker or as
 * the timed CPU side, never as the product path.
 *
 * Layouts (crates/llmtie-cuda/src/kernels.rs:5244-5317):
 *   Q      f32  [tq][heads*hd]          (row stride q_stride elements)
 *   K      [kv_heads][cap][hd]          element ((kh*cap + pos)*hd + d)
 *   V      [kv_heads][hd][cap]          element ((kh*hd + d)*cap + pos)
 * f16 values travel as uint16_t bit patterns.
 */
#ifndef LLMTIE_ORACLE_H
#define LLMTIE_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* IEEE binary16 <-> binary32, round to nearest even: what half::f16::from_f32
 * and cvt.rn.f16.f32 do (crates/llmtie-cuda/src/kernels.rs:117-131). */
uint16_t orc_f32_to_f16(float x);
float orc_f16_to_f32(uint16_t h);
void orc_round_f16(const float *src, uint16_t *dst, size_t n);
void orc_widen_f16(const uint16_t *src, float *dst, size_t n);

/* The reference's deterministic test generator, values in [-2, 6)
 * (crates/llmtie-cuda/tests/kernels.rs:35-45). */
void orc_seq(float *out, size_t n, uint64_t salt);

/* NeoX/halves RoPE in place over [t][heads*hd], f32 powf/sinf/cosf
 * (crates/llmtie-dsp/src/rope.rs:83-126). freq_div may be NULL. */
void orc_rope(float *x, size_t t, size_t heads, size_t hd, float theta,
              size_t first, const float *freq_div);

/* cache_append{,_t}{,_f16}: src [n][kv_heads*hd] f32 -> cache at `past`
 * (crates/llmtie-cuda/src/kernels.rs:5244-5317). */
void orc_cache_append_f16(const float *src, uint16_t *dst, size_t n,
                          size_t kv_heads, size_t hd, size_t cap, size_t past,
                          int transposed);
void orc_cache_append_f32(const float *src, float *dst, size_t n,
                          size_t kv_heads, size_t hd, size_t cap, size_t past,
                          int transposed);

/* cache_grow{,_f16}: re-stride `rows` runs of `len`
 * (crates/llmtie-cuda/src/kernels.rs:5397-5423; run geometry from
 * crates/llmtie-cuda/src/device.rs:3173-3181). esize is 2 or 4. */
void orc_cache_grow(const void *src, void *dst, size_t kv_heads, size_t hd,
                    size_t old_cap, size_t new_cap, size_t live,
                    int transposed, size_t esize);

/* rope_cache_f16: one decoded position; q rotated in place, rotated k and v
 * stored at `pos` (crates/llmtie-cuda/src/kernels.rs:5334-5378). */
void orc_rope_cache_f16(float *q, const float *k, const float *v,
                        const float *freq_div, size_t heads, size_t kv_heads,
                        size_t hd, float theta, size_t pos, uint16_t *kc,
                        uint16_t *vc, size_t cap);

/*
 * Prefill / encoder / cross attention, the scalar reference inside
 * `fused_attention_sized` (crates/llmtie-cuda/tests/kernels.rs:2300-2364):
 * operands through f16, f64 accumulation, score*scale, exp(x-m), the
 * normaliser from un-rounded probabilities, probabilities through f16 on
 * their way into the value product.
 *
 *   scale_q != 0: the scale goes on q before q is rounded to f16 and the
 *   scores are not scaled (crates/llmtie-cuda/src/kernels.rs:3080-3098).
 *   causal: row r sees keys 0..=past+r; otherwise keys 0..tk-1, tk = past+tq
 *   unless tk_override > 0 (cross attention: tq queries over tk keys).
 *   kv_f16 != 0: k and v point at uint16_t bit patterns, else at f32 (which
 *   are rounded to f16 as the kernel's staging does).
 *   out: f32 [tq][heads*hd].
 */
void orc_prefill(const float *q, size_t q_stride, const void *k, const void *v,
                 int kv_f16, size_t tq, size_t past, size_t tk_override,
                 size_t heads, size_t kv_heads, size_t hd, size_t cap,
                 float scale, int causal, int scale_q, float *out,
                 size_t out_stride);

/* The same arithmetic with f32 accumulation and one thread per (head, row)
 * block: the timed CPU baseline. Returns the thread count it used. */
int orc_prefill_fast(const float *q, size_t q_stride, const void *k,
                     const void *v, int kv_f16, size_t tq, size_t past,
                     size_t tk_override, size_t heads, size_t kv_heads,
                     size_t hd, size_t cap, float scale, int causal,
                     int scale_q, float *out, size_t out_stride, int threads);

/*
 * Decode: `decode_attention_ref`, f32 and sequential
 * (crates/llmtie-cuda/tests/kernels.rs:2733-2774). k and v are f32 arrays in
 * the cache layouts, already rounded to the width the device copy holds.
 * q is [heads*hd]; out is [heads*hd].
 */
void orc_decode_f32(const float *q, const float *k, const float *v,
                    size_t heads, size_t kv_heads, size_t hd, size_t tk,
                    size_t cap, float scale, int scale_q, float *out);

/* The same with f64 accumulation off an f16 cache: the tighter variant the
 * GPU path is held to. Also writes the un-normalised triple when o_un, m_out
 * and l_out are non-NULL: o_un [heads][hd] = sum p*v, m = max score,
 * l = sum p, p = exp(score - m) (the algebra of
 * crates/llmtie-cuda/src/kernels.rs:5836-5879). Keys [t0, t1) only. */
void orc_decode_f64(const float *q, const uint16_t *k, const uint16_t *v,
                    size_t heads, size_t kv_heads, size_t hd, size_t t0,
                    size_t t1, size_t cap, float scale, int scale_q,
                    float *out, float *o_un, float *m_out, float *l_out);

/* The activation quantiser whose output the decode attention's int8 "twin" must
 * equal (crates/llmtie-cuda/src/kernels.rs:693-719, and ad_emit :5755-5773):
 * per group of 32 consecutive values d = max|x| * (1/127) in f32, code =
 * round-to-nearest-even(x * (1/d)) (0 when d is 0), scale = d. n a multiple
 * of 32; codes [n], scales [n/32]. */
void orc_quantize_q8(const float *x, size_t n, int8_t *codes, float *scales);

/* Log-sum-exp merge of `parts` un-normalised triples
 * (crates/llmtie-cuda/src/kernels.rs:5836-5879):
 * M = max m_i, f_i = exp(m_i - M), out = (sum o_i f_i) / (sum l_i f_i).
 * o [parts][rows][hd], m and l [parts][rows]; out [rows][hd]. */
void orc_lse_merge(const float *o, const float *m, const float *l,
                   size_t parts, size_t rows, size_t hd, float *out);

/* Decode off an f16 cache with f32 accumulation, threads over
 * (sequence, head): the timed CPU baseline. Returns the thread count. */
int orc_decode_fast(const float *q, const uint16_t *k, const uint16_t *v,
                    size_t heads, size_t kv_heads, size_t hd, size_t tk,
                    size_t cap, float scale, int scale_q, float *out,
                    int threads);

int orc_max_threads(void);

/* crates/llmtie-cuda/src/kernels.rs:6876-6913: the stacked q/k/v projection of
 * one row, placed into a row and the two f32 caches at pos (f64 sums). */
void orc_gemv_qkv_f16(const float *a, const uint16_t *w, const float *qb,
                      const float *kb, const float *vb, size_t k, size_t d,
                      size_t hd, size_t cap, size_t pos, float *q, float *kc,
                      float *vc);

/* crates/llmtie-cuda/src/kernels.rs:5598-5613: GPT-J style rotary embedding
 * over the interleaved pairs of the first rot_dim of each dim-wide row. */
void orc_rope_gptj(float *x, const float *inv_freq, size_t positions,
                   size_t dim, size_t rot_dim);

/* crates/llmtie-cuda/src/kernels.rs:5089-5139: x f32 [t][heads*hd] (+ bias
 * row or NULL) rounded to f16 into [heads][cap][hd] or, transposed,
 * [heads][hd][cap]; positions past t are not written. */
void orc_split_heads_f16(const float *x, const float *bias, uint16_t *out,
                         size_t t, size_t heads, size_t hd, size_t cap,
                         int transposed);

#ifdef __cplusplus
}
#endif
#endif
