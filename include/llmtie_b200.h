/*
 * llmtie_b200 - the attention hot path of llmtie-rs as precompiled sm_100a
 * kernels behind a C ABI.
 *
 * This library stands where `llmtie_cuda::Gpu` (crates/llmtie-cuda/src/device.rs)
 * stands for attention, RoPE and the KV cache: it replaces the NVRTC module
 * loader (`Gpu::open`, device.rs:737-842) with kernels compiled ahead of
 * time, and the cache allocator policy of the model crates with
 * `llmtie_kv_*`. Every entry point below names the reference method it
 * replaces. Conventions, all taken from the reference:
 *
 *   - device buffers are raw device pointers plus their length in ELEMENTS,
 *     so memory owned by the caller's allocator (cudarc in the reference) can
 *     be passed straight through and every range is checked on the host
 *     before anything is launched (error.rs:140-277);
 *   - f16 travels as uint16_t bit patterns;
 *   - offsets are element offsets into a buffer, never sub-slices, because
 *     projections may alias one allocation (device.rs:2909-2913);
 *   - all work is asynchronous on the handle's own non-blocking stream and
 *     stream-ordered; nothing here synchronises the host except
 *     llmtie_synchronize, llmtie_download and llmtie_kprof_report (and every
 *     launch while kprof is on);
 *   - a call that is refused returns a non-zero status, launches nothing and
 *     leaves a message for llmtie_last_error() (thread-local).
 *
 * There is no CPU fallback: without a usable device llmtie_open fails with
 * LLMTIE_ERR_NO_DEVICE and nothing else can be called.
 */
#ifndef LLMTIE_B200_H
#define LLMTIE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct llmtie_gpu llmtie_gpu;
typedef struct llmtie_decode_scratch llmtie_decode_scratch;
typedef int32_t llmtie_status;

/* Status codes: one per `CudaError` variant the path can raise
 * (crates/llmtie-cuda/src/error.rs). */
enum {
    LLMTIE_OK = 0,
    LLMTIE_ERR_NO_DEVICE = 1,             /* CudaError::NoDevice */
    LLMTIE_ERR_DRIVER = 2,                /* CudaError::Driver */
    LLMTIE_ERR_SLICE_OVERRUN = 3,         /* CudaError::SliceOverrun */
    LLMTIE_ERR_CACHE_OVERRUN = 4,         /* CudaError::CacheOverrun */
    LLMTIE_ERR_ODD_CACHE_CAPACITY = 5,    /* CudaError::OddCacheCapacity */
    LLMTIE_ERR_ODD_HEAD_DIM = 6,          /* CudaError::OddHeadDim */
    LLMTIE_ERR_UNSUPPORTED_ATTENTION = 7, /* CudaError::UnsupportedAttention */
    LLMTIE_ERR_RAGGED_BLOCK = 8,          /* CudaError::RaggedBlock */
    LLMTIE_ERR_MISALIGNED = 9,            /* CudaError::Misaligned */
    LLMTIE_ERR_MISSING_KERNEL = 10,       /* CudaError::MissingKernel */
    LLMTIE_ERR_TIMEOUT = 11,              /* a bounded device wait ran out */
    LLMTIE_ERR_INVALID = 12               /* null handle, negative size */
};

/* ---- device handle ------------------------------------------------------ */

/* Gpu::open (device.rs:737-842): binds the device, creates the handle's
 * non-blocking stream and checks that the device is an sm_100 part. */
llmtie_status llmtie_open(int32_t ordinal, llmtie_gpu **out);
/* The same, adopting a stream the caller owns (a cudaStream_t). */
llmtie_status llmtie_open_on_stream(int32_t ordinal, void *stream, llmtie_gpu **out);
void llmtie_close(llmtie_gpu *g);
/* Message of the last refused or failed call on this thread. */
const char *llmtie_last_error(void);
/* The handle's cudaStream_t. */
void *llmtie_stream(llmtie_gpu *g);
int32_t llmtie_ordinal(llmtie_gpu *g);
/* Gpu::synchronize (device.rs:1433-1440). Also surfaces LLMTIE_ERR_TIMEOUT if
 * a kernel's bounded wait gave up since the last report (llmtie_download
 * reports it as well). A timeout is reported once; reporting it clears the
 * arrival counters of every decode scratch of the handle, so the next call
 * starts clean. What the kernel that gave up should have written is
 * undefined. */
llmtie_status llmtie_synchronize(llmtie_gpu *g);
/* How long a device-side wait (an mbarrier of the tensor-memory prefill, a
 * flag another GPU raises) may spin before it gives up, in SM cycles. The
 * default, also restored by cycles <= 0, is 2^31: about a second. No
 * counterpart in the reference, whose kernels never wait on one another. */
llmtie_status llmtie_set_wait_limit_cycles(llmtie_gpu *g, int64_t cycles);

/* Gpu::uninit / zeros / zeros_f16 (device.rs:937-983): stream-ordered. */
llmtie_status llmtie_alloc(llmtie_gpu *g, size_t bytes, void **dptr);
llmtie_status llmtie_zeros(llmtie_gpu *g, size_t bytes, void **dptr);
llmtie_status llmtie_free(llmtie_gpu *g, void *dptr);
/* Gpu::upload / download (device.rs:898-935): host <-> device on the stream;
 * download waits for the stream, and returns LLMTIE_ERR_TIMEOUT (the bytes
 * are copied all the same) if a kernel's bounded wait gave up before it. */
llmtie_status llmtie_upload(llmtie_gpu *g, void *dst, const void *src, size_t bytes);
llmtie_status llmtie_download(llmtie_gpu *g, void *dst, const void *src, size_t bytes);
/* Gpu::upload_f16 (device.rs:1422-1431): f32 on the device -> f16 bits, RNE. */
llmtie_status llmtie_round_f16(llmtie_gpu *g, const float *src, uint16_t *dst, size_t n);

/* ---- KV-cache allocator -------------------------------------------------- */

/* The growth policy of crates/llmtie-chat/src/model.rs:714-747 and
 * crates/llmtie-translate/src/model.rs:662-694: the capacity to allocate when
 * a cache of `cap` must hold past + n positions (0 = it already does).
 * want = min(max(next_pow2(past + n + (n > 1 ? 256 : 0)), 256),
 *            max(max_positions, past + n)). */
size_t llmtie_kv_want_capacity(size_t cap, size_t past, size_t n, size_t max_positions);
/* Prefix::shared_with and the cut complete_in makes with it
 * (crates/llmtie-chat/src/generate.rs:264-272, :139-141): how many leading
 * tokens of `ids` a cache that holds the tokens `held` can keep, never all of
 * `ids` (the last token is always run, for its logits). The cache is then
 * truncated to that length - Cache::truncate, chat/model.rs:259-261, only
 * lowers the live length, nothing is zeroed - and the prompt prefilled from
 * there with past = the returned value. Host only. */
size_t llmtie_kv_shared_prefix(const uint32_t *held, size_t held_len, const uint32_t *ids,
                               size_t ids_len);
/* zeros_f16(want * kv_dim) twice (chat/model.rs:722-731): zeroed K
 * [kv_heads][cap][hd] and V [kv_heads][hd][cap]. cap must be even. */
llmtie_status llmtie_kv_alloc_f16(llmtie_gpu *g, size_t kv_heads, size_t head_dim,
                                  size_t cap, uint16_t **k, uint16_t **v);
/* Gpu::cache_grow_f16 / cache_grow (device.rs:3086-3212): re-stride `live`
 * positions from a cache of old_cap into one of new_cap. */
llmtie_status llmtie_cache_grow_f16(llmtie_gpu *g, const uint16_t *src, size_t src_len,
                                    uint16_t *dst, size_t dst_len, size_t kv_heads,
                                    size_t head_dim, size_t old_cap, size_t new_cap,
                                    size_t live, int32_t transposed);
llmtie_status llmtie_cache_grow(llmtie_gpu *g, const float *src, size_t src_len,
                                float *dst, size_t dst_len, size_t kv_heads,
                                size_t head_dim, size_t old_cap, size_t new_cap,
                                size_t live, int32_t transposed);
/* Gpu::cache_append_f16 / cache_append (device.rs:2849-2901, :3013-3078):
 * src [n][kv_heads*head_dim] f32 at src_off -> cache positions past..past+n. */
llmtie_status llmtie_cache_append_f16(llmtie_gpu *g, const float *src, size_t src_len,
                                      size_t src_off, uint16_t *dst, size_t dst_len,
                                      size_t n, size_t kv_heads, size_t head_dim,
                                      size_t cap, size_t past, int32_t transposed);
llmtie_status llmtie_cache_append(llmtie_gpu *g, const float *src, size_t src_len,
                                  size_t src_off, float *dst, size_t dst_len, size_t n,
                                  size_t kv_heads, size_t head_dim, size_t cap,
                                  size_t past, int32_t transposed);

/* ---- the projection in front of the Whisper decoder's self-attention ---------- */

/* Gpu::gemv_qkv_f16 (device.rs:4393-4479, kernels.rs:6876-6913): the three
 * attention projections of one row a f32 [k] in one launch, each placed where
 * the attention reads it: w is the three [d][k] f16 weights stacked into
 * [3d][k]; q = Wq a (+ q_bias) into q f32 [d]; the keys into kc f32 [d/
 * head_dim][cap][head_dim] at `pos`; the values into the transposed vc f32
 * [d][cap] at `pos` - the caches llmtie_attn_decode reads. Each bias is f32
 * [d] or NULL (the keys have none in any Whisper checkpoint). k must be even.
 * Products accumulate in f32 in a fixed order, so a call is reproducible. */
llmtie_status llmtie_gemv_qkv_f16(llmtie_gpu *g, const float *a, size_t a_len,
                                  const uint16_t *w, size_t w_len, const float *q_bias,
                                  const float *k_bias, const float *v_bias, size_t bias_len,
                                  size_t k, size_t d, size_t head_dim, size_t cap, size_t pos,
                                  float *q, size_t q_len, float *kc, size_t kc_len, float *vc,
                                  size_t vc_len);

/* ---- Whisper cross-attention cache build ------------------------------------- */

/* Gpu::split_heads_f16_at / split_heads_t_f16_at (device.rs:5636-5665, kernels
 * kernels.rs:5089-5139): the block x[x_off .. x_off + t*heads*head_dim] of f32
 * [t][heads*head_dim], plus the row bias[bias_off ..] when bias is not NULL
 * (the f32 add a projection's epilogue would have made), rounded to f16 into
 * keys [heads][cap][head_dim] or, transposed, values [heads][head_dim][cap].
 * The reference allocates the result at cap == t; here the caller passes a
 * zeroed buffer (llmtie_zeros) and may ask for cap > t: positions past t are
 * left as they are, so a cache of 1500 frames can be given a capacity of 1504
 * and its value rows 16-byte alignment, which is what lets the cross-attention
 * calls below stream it through the fast decode kernel. */
llmtie_status llmtie_split_heads_f16_at(llmtie_gpu *g, const float *x, size_t x_len,
                                        size_t x_off, const float *bias, size_t bias_len,
                                        size_t bias_off, uint16_t *out, size_t out_len, size_t t,
                                        size_t heads, size_t head_dim, size_t cap,
                                        int32_t transposed);
/* AsrModel::cache's loop over the decoder layers (crates/llmtie-asr/src/model.rs:
 * 917-939) in two launches: k_all and v_all f32 [layers][t][heads*head_dim] are
 * the batched projections of the encoder output, v_bias f32 [layers][heads*
 * head_dim] the value biases (NULL: none). k_out f16 [layers][heads][cap]
 * [head_dim] and v_out f16 [layers][heads][head_dim][cap], both zeroed by the
 * caller; layer l's caches start l*heads*cap*head_dim elements in. */
llmtie_status llmtie_cross_kv_build(llmtie_gpu *g, const float *k_all, size_t k_len,
                                    const float *v_all, size_t v_len, const float *v_bias,
                                    size_t v_bias_len, uint16_t *k_out, size_t k_out_len,
                                    uint16_t *v_out, size_t v_out_len, size_t layers, size_t t,
                                    size_t heads, size_t head_dim, size_t cap);

/* Gpu::split_heads / split_heads_t (device.rs:5573-5598, kernels.rs:5002-5075:
 * the f32 twins of the above), as crates/llmtie-cosy/src/flow.rs:
 * 560-566 lays out the keys and values of its non-causal attention for
 * llmtie_flash_attn: x f32 [t][heads*head_dim] at x_off -> f32 [heads][cap]
 * [head_dim] or, transposed, [heads][head_dim][cap]; out zeroed by the caller. */
llmtie_status llmtie_split_heads(llmtie_gpu *g, const float *x, size_t x_len, size_t x_off,
                                 float *out, size_t out_len, size_t t, size_t heads,
                                 size_t head_dim, size_t cap, int32_t transposed);

/* ---- RoPE ----------------------------------------------------------------- */

/* Gpu::rope_gptj (device.rs:4853-4873, kernels.rs:5583-5613; the kernel
 * itself :5598): GPT-J style
 * partial rotary embedding in place on x f32 [positions][dim]. Only the first
 * rot_dim of each row turns, element 2j pairs with 2j+1, angle = position *
 * inv_freq[j] with the frequencies from a buffer of rot_dim/2, fast sine and
 * cosine as the reference's kernel. The CosyVoice flow model's q and k rows
 * go through it before llmtie_flash_attn (crates/llmtie-cosy/src/flow.rs:545-553). */
llmtie_status llmtie_rope_gptj(llmtie_gpu *g, float *x, size_t x_len, const float *inv_freq,
                               size_t inv_len, size_t positions, size_t dim, size_t rot_dim);

/* Gpu::rope / rope_scaled (device.rs:5410-5471): NeoX/halves RoPE in place on
 * x[off .. off + t*heads*head_dim]; freq_div is NULL or head_dim/2 floats. */
llmtie_status llmtie_rope_scaled(llmtie_gpu *g, float *x, size_t x_len, size_t off,
                                 const float *freq_div, size_t t, size_t heads,
                                 size_t head_dim, float theta, size_t first);
/* Gpu::rope_cache_f16 (device.rs:2915-3000): one decoded position. q is
 * rotated in place; rotated k and v go to the f16 caches at `pos`; the
 * projection buffers for k and v are not written. q, k and v may be offsets
 * into one allocation. */
llmtie_status llmtie_rope_cache_f16(llmtie_gpu *g, float *q, size_t q_len, size_t q_off,
                                    const float *k, size_t k_len, size_t k_off,
                                    const float *v, size_t v_len, size_t v_off,
                                    const float *freq_div, size_t heads, size_t kv_heads,
                                    size_t head_dim, float theta, size_t pos,
                                    uint16_t *kc, size_t kc_len, uint16_t *vc,
                                    size_t vc_len, size_t cap);

/* Gpu::rope_cache_f16 for `batch` sequences decoding together, one launch:
 * what crates/llmtie-translate/src/model.rs:824-846 does as a loop. q f32
 * [batch][heads*hd] is rotated in place; k and v f32 [batch][kv_heads*hd]
 * go to each sequence's own caches at pos[b]. pos, cap, kc_ptrs and vc_ptrs
 * are HOST arrays of `batch`. Bit for bit the single-sequence entry. */
llmtie_status llmtie_rope_cache_batched(llmtie_gpu *g, float *q, size_t q_len, const float *k,
                                        size_t k_len, const float *v, size_t v_len,
                                        const float *freq_div, size_t batch, size_t heads,
                                        size_t kv_heads, size_t head_dim, float theta,
                                        const int32_t *pos, uint16_t *const *kc_ptrs,
                                        uint16_t *const *vc_ptrs, const int32_t *cap);

/* ---- prefill / encoder attention ------------------------------------------- */

/* Gpu::supports_flash (device.rs:5697-5699). */
int32_t llmtie_supports_flash(size_t head_dim, size_t heads, size_t kv_heads);
/* Gpu::flash_attn_f16 (device.rs:5754-5799): q f32 [tq][heads*hd] (already
 * rotated), K f16 [kv][cap][hd], V f16 [kv][hd][cap] holding past+tq
 * positions; out f32 [tq][heads*hd]. head_dim 128 only, cap even. (Caches
 * whose value rows are not 16-byte aligned - a capacity that is not a
 * multiple of 8 - cost one more launch: their live keys are copied into
 * aligned caches that the handle keeps for the purpose.) */
llmtie_status llmtie_flash_attn_f16(llmtie_gpu *g, const float *q, size_t q_len,
                                    const uint16_t *k, size_t k_len, const uint16_t *v,
                                    size_t v_len, float *out, size_t out_len, size_t tq,
                                    size_t past, size_t heads, size_t kv_heads,
                                    size_t head_dim, size_t cap, float scale,
                                    int32_t causal);
/* Gpu::flash_attn (device.rs:5702-5745): the same off f32 caches, head_dim 64
 * or 128; K and V are rounded to f16 on their way into the products: here
 * once, the live keys into f16 caches that the handle keeps for the purpose
 * (grown on the stream when a longer context comes), ahead of the attention
 * kernel. */
llmtie_status llmtie_flash_attn(llmtie_gpu *g, const float *q, size_t q_len,
                                const float *k, size_t k_len, const float *v,
                                size_t v_len, float *out, size_t out_len, size_t tq,
                                size_t past, size_t heads, size_t kv_heads,
                                size_t head_dim, size_t cap, float scale, int32_t causal);
/* Gpu::flash_attn_rows (device.rs:5812-5865): the Whisper encoder. qkv f32
 * [t][3*heads*hd] (q | k | v column blocks), non-causal, scale on q before it
 * is rounded, context returned f16 [t][heads*hd]. head_dim 64 only.
 * `work` is NULL (the call allocates and frees its own staging buffers on the
 * stream) or a buffer of llmtie_flash_rows_work_bytes(t, heads, head_dim). */
llmtie_status llmtie_flash_attn_rows(llmtie_gpu *g, const float *qkv, size_t qkv_len,
                                     uint16_t *out, size_t out_len, size_t t,
                                     size_t heads, size_t head_dim, float scale,
                                     void *work, size_t work_bytes);
/* llmtie_flash_attn_rows for `batch` utterances of the same length in two
 * launches (the reference has no batch here: the encoder calls once per
 * utterance, crates/llmtie-asr/src/model.rs:792-822). qkv f32 [batch][t][3*d],
 * out f16 [batch][t][d]; `work` NULL or batch times the single-utterance size. */
llmtie_status llmtie_flash_attn_rows_batched(llmtie_gpu *g, const float *qkv, size_t qkv_len,
                                             uint16_t *out, size_t out_len, size_t batch,
                                             size_t t, size_t heads, size_t head_dim,
                                             float scale, void *work, size_t work_bytes);
size_t llmtie_flash_rows_work_bytes(size_t t, size_t heads, size_t head_dim);

/* ---- decode attention ------------------------------------------------------- */

/* DecodeScratch (device.rs:166-233, :6332-6359): the split-KV workspace a
 * caller keeps per cache. It grows inside the attention call when a longer
 * context needs more partials; its counters rest at zero between calls. */
llmtie_status llmtie_decode_scratch_new(llmtie_gpu *g, llmtie_decode_scratch **out);
void llmtie_decode_scratch_free(llmtie_gpu *g, llmtie_decode_scratch *s);

/* Gpu::attn_decode_f16 / attn_decode_f16_q_row without the int8 twin
 * (device.rs:5949-6038, :6224-6413): one query position, q f32 [heads*hd] at
 * q_off with a group's rows adjacent, f16 caches holding tk <= cap positions,
 * out f32 [heads*hd] at out_off (out_off % 32 == 0). scale_q puts the scale
 * on q; otherwise on the scores. head_dim 64 or 128; heads/kv_heads at most 4
 * at 128 and 8 at 64, as the reference's instantiations. */
llmtie_status llmtie_attn_decode_f16(llmtie_gpu *g, const float *q, size_t q_len,
                                     size_t q_off, const uint16_t *k, size_t k_len,
                                     const uint16_t *v, size_t v_len, size_t heads,
                                     size_t kv_heads, size_t head_dim, size_t tk,
                                     size_t cap, float scale, int32_t scale_q,
                                     llmtie_decode_scratch *scratch, float *out,
                                     size_t out_len, size_t out_off);
/* Gpu::attn_decode_f16_q / attn_decode_f16_q_row (device.rs:5973-6038): the
 * same, and the context's int8 "twin" beside it, made by the kernel on the
 * row it just produced (ad_emit, kernels.rs:5755-5773 = quantize_q8's
 * arithmetic): per 32 consecutive elements scale = max|y| / 127 and code =
 * round-to-nearest-even(y / scale) (0 when the group is all zero). codes int8
 * [rows][heads*hd] and scales f32 [rows][heads*hd/32] are written from
 * element out_off and out_off/32, as out is from out_off. */
llmtie_status llmtie_attn_decode_f16_q(llmtie_gpu *g, const float *q, size_t q_len,
                                       size_t q_off, const uint16_t *k, size_t k_len,
                                       const uint16_t *v, size_t v_len, size_t heads,
                                       size_t kv_heads, size_t head_dim, size_t tk, size_t cap,
                                       float scale, int32_t scale_q,
                                       llmtie_decode_scratch *scratch, float *out,
                                       size_t out_len, size_t out_off, int8_t *codes,
                                       size_t codes_len, float *scales, size_t scales_len);
/* Gpu::attn_decode (device.rs:6132-6168): the same off f32 caches, head_dim 64
 * (the Whisper decoder's self-attention). With a scratch every head's keys are
 * cut over up to eight blocks whose partial results meet there; without one
 * (NULL) the launch is one block a head. The key cache 16-byte aligned. */
llmtie_status llmtie_attn_decode(llmtie_gpu *g, const float *q, size_t q_len, size_t q_off,
                                 const float *k, size_t k_len, const float *v,
                                 size_t v_len, size_t heads, size_t kv_heads,
                                 size_t head_dim, size_t tk, size_t cap, float scale,
                                 int32_t scale_q, llmtie_decode_scratch *scratch,
                                 float *out, size_t out_len, size_t out_off);

/* llmtie_attn_decode_f16 for callers that cannot allocate. This entry has no
 * counterpart in the reference: there, as in llmtie_attn_decode_f16, the
 * caller's DecodeScratch grows by a stream-ordered allocation inside the
 * call. A per-token thread of a voice pipeline that must never wait on the
 * driver, or a process that handed the whole device to its own pool, cannot
 * take that, so here the partials and counters live in a static device array
 * inside the library (about 1.3 MB on every GPU that loads it, until exit)
 * and the call allocates and frees nothing.
 * Limits, refused by name: at most 64 kv heads; capacity a multiple of 8 and
 * 16-byte aligned caches (LLMTIE_ERR_MISALIGNED otherwise); head_dim and
 * group as llmtie_attn_decode_f16.
 * The first call on a device resolves the array's address; make that call
 * before any stream capture. All calls share the array: it keeps the last
 * call's contents (the call clears what must start at zero), and two calls
 * that overlap on the GPU race - order them one after another. */
llmtie_status llmtie_attn_decode_f16_noalloc(llmtie_gpu *g, const float *q, size_t q_len,
                                             size_t q_off, const uint16_t *k, size_t k_len,
                                             const uint16_t *v, size_t v_len, size_t heads,
                                             size_t kv_heads, size_t head_dim, size_t tk,
                                             size_t cap, float scale, int32_t scale_q,
                                             float *out, size_t out_len, size_t out_off);

/* ---- batched and sharded entries (supersets; the reference loops) ------------ */

/* What crates/llmtie-translate/src/model.rs:824-859 does as a loop of
 * single-sequence launches, in one launch: `batch` sequences, each with its
 * own f16 caches, live length and capacity. q and out are f32
 * [batch][heads*hd]. k_ptrs, v_ptrs, tk and cap are HOST arrays of `batch`.
 * If `partial` is non-zero, out is instead [batch][heads][hd+2]: the
 * un-normalised context, the maximum score and the sum of exponentials
 * (kernels.rs:5791-5799), for llmtie_lse_merge. */
llmtie_status llmtie_decode_batched(llmtie_gpu *g, const float *q, size_t q_len,
                                    const uint16_t *const *k_ptrs,
                                    const uint16_t *const *v_ptrs, const int32_t *tk,
                                    const int32_t *cap, size_t batch, size_t heads,
                                    size_t kv_heads, size_t head_dim, float scale,
                                    int32_t scale_q, llmtie_decode_scratch *scratch,
                                    float *out, size_t out_len, int32_t partial);
/* The merge of ad_publish_merge (kernels.rs:5836-5879) over `parts` triples
 * laid out [parts][rows][hd+2], e.g. an all-gather of each GPU's
 * llmtie_decode_batched(partial=1) output; out f32 [rows][hd]. */
llmtie_status llmtie_lse_merge(llmtie_gpu *g, const float *parts_buf, size_t parts_len,
                               size_t parts, size_t rows, size_t head_dim, float *out,
                               size_t out_len);
/* The same two steps with the exchange between GPUs fused into the kernels
 * (no counterpart in the reference, which has no multi-GPU path). Every rank
 * holds a slice of each sequence's positions. `gather[r]` and `flags[r]` are
 * rank r's buffers as mapped into this process (symmetric / peer memory):
 * gather is f32 [2][world][batch*heads][head_dim+2], flags uint32 [world],
 * both zero before the first step; `step` is a uint32 of this rank's own,
 * zero before the first step.
 * llmtie_decode_batched_push decodes this rank's slice and stores the
 * un-normalised triples straight into slot [step&1][rank] of EVERY rank's
 * gather buffer with plain peer stores over NVLink; the block that finishes
 * the launch's last head then raises flag [rank] on every rank and advances
 * `step`. llmtie_lse_merge_wait, enqueued after it on the same stream, waits
 * (bounded: about a second, then LLMTIE_ERR_TIMEOUT at the next synchronize)
 * until all `world` flags have reached this rank's step and merges. All ranks
 * must make the same sequence of calls. At most 32 sequences a call; caches
 * 16-byte aligned with capacities that are multiples of 8. */
typedef struct llmtie_exchange {
    int32_t world;
    int32_t rank;
    float *const *gather;     /* HOST array of `world` device pointers */
    uint32_t *const *flags;   /* HOST array of `world` device pointers */
    uint32_t *step;           /* device pointer, this rank's */
} llmtie_exchange;
llmtie_status llmtie_decode_batched_push(llmtie_gpu *g, const float *q, size_t q_len,
                                         const uint16_t *const *k_ptrs,
                                         const uint16_t *const *v_ptrs, const int32_t *tk,
                                         const int32_t *cap, size_t batch, size_t heads,
                                         size_t kv_heads, size_t head_dim, float scale,
                                         int32_t scale_q, llmtie_decode_scratch *scratch,
                                         const llmtie_exchange *xch);
llmtie_status llmtie_lse_merge_wait(llmtie_gpu *g, const llmtie_exchange *xch, size_t rows,
                                    size_t head_dim, float *out, size_t out_len);
/* How a batched decode launch over contexts tk[0..batch) would be cut over
 * the grid (host only, no device needed; no counterpart in the reference):
 * grid_out = blocks launched on a device of sm_count SMs, ustart[c] = the
 * first 128-key unit of block c, ustart[grid] = all units. Units are laid end
 * to end, sequence after sequence, KV head after KV head. For tests and for
 * sizing scratch ahead of time (a launch uses 2*grid partial slots). This is
 * the cut by work; a launch whose pairs are few and short, or all of one
 * length and about half as many as the SMs, gives every pair a thread-block
 * cluster of 2, 4 or 8 blocks instead, which writes no partials at all. */
llmtie_status llmtie_decode_cut(const int32_t *tk, size_t batch, size_t kv_heads,
                                size_t head_dim, int32_t sm_count, int32_t *ustart,
                                size_t ustart_len, int32_t *grid_out);
/* The whole choice a launch makes (host only, no device needed; no counterpart
 * in the reference): for `batch` sequences of tk[b] keys, `rows` query rows a
 * KV head (the GQA group, or the rows of llmtie_cross_attn), on a device of
 * sm_count SMs that holds resident2 / resident4 / resident8 clusters of 2 / 4 /
 * 8 blocks of the decode kernel at once (the launch asks the driver; a B200
 * answers 74 / 33 / 15 at head_dim 128 and 148 / 71 / 33 at 64). blocks_a_pair_out = 0: cut by work as
 * llmtie_decode_cut describes; 1: every pair a block of its own; 2, 4, 8: every
 * pair a thread-block cluster of that many blocks. grid_out and ustart as for
 * llmtie_decode_cut. */
/* How many thread-block clusters of `blocks` (2, 4 or 8) blocks of the decode
 * kernel the handle's device holds at once, as the driver answers (0: none,
 * or a bad argument): what llmtie_decode_plan takes as resident2 / 4 / 8. */
int32_t llmtie_decode_resident_clusters(llmtie_gpu *g, size_t head_dim, int32_t blocks);
llmtie_status llmtie_decode_plan(const int32_t *tk, size_t batch, size_t kv_heads, size_t rows,
                                 size_t head_dim, int32_t sm_count, int32_t resident2,
                                 int32_t resident4, int32_t resident8, int32_t *ustart,
                                 size_t ustart_len, int32_t *grid_out,
                                 int32_t *blocks_a_pair_out);
/* The whole sharded step in ONE kernel (no counterpart in the reference):
 * llmtie_decode_batched_push with the merge fused in as well. The block that
 * finishes a (sequence, KV head) pair on this rank stores the pair's triple
 * into every rank's gather buffer and raises that pair's flag there;
 * before it exits it waits (bounded: about a second, then LLMTIE_ERR_TIMEOUT
 * at the next synchronize) for the other ranks' flags of the same pair and
 * merges the pair into out f32 [batch][heads*hd], normalised. So the cross-
 * rank merge of early pairs overlaps the streaming of later ones, and only
 * the last pairs' exchange is exposed. xch->flags is unused; pair_flags is a
 * HOST array of `world` device pointers, each rank's [batch*kv_heads][world]
 * words, zero before the first step. gather and step as for the push entry.
 * A world of one rank is allowed (the rank merges its own triples). All
 * ranks must make the same sequence of calls; at most 32 sequences a call. */
llmtie_status llmtie_decode_batched_fused(llmtie_gpu *g, const float *q, size_t q_len,
                                          const uint16_t *const *k_ptrs,
                                          const uint16_t *const *v_ptrs, const int32_t *tk,
                                          const int32_t *cap, size_t batch, size_t heads,
                                          size_t kv_heads, size_t head_dim, float scale,
                                          int32_t scale_q, llmtie_decode_scratch *scratch,
                                          const llmtie_exchange *xch,
                                          uint32_t *const *pair_flags, float *out,
                                          size_t out_len);
/* The sharded step in two kernels that overlap (no counterpart in the
 * reference): llmtie_decode_batched_signal is llmtie_decode_batched_push with a
 * flag per (sequence, KV head) pair instead of one per rank - the block that
 * finishes a pair stores its triple into every rank's gather buffer and raises
 * [pair][rank] of every rank's pair_flags (HOST array of `world` device
 * pointers, each [batch*kv_heads][world] words, zero before the first step).
 * llmtie_lse_merge_pairs, enqueued right after it on the same stream, is
 * launched as a programmatic dependent: its blocks are resident while the
 * decode kernel still streams, each waits (bounded, as above) for the `world`
 * flags of its row's pair and merges the row at once, so the merge's launch
 * and every pair's exchange but the last are off the step's critical path.
 * pair_flags there is THIS rank's array; merge_step is a device uint32[2] of
 * this rank's own, zero before the first step (the merge counts its own
 * steps); rows = batch*heads, rows_per_pair = heads/kv_heads. gather and step
 * as for the push entry; xch->flags is unused. */
llmtie_status llmtie_decode_batched_signal(llmtie_gpu *g, const float *q, size_t q_len,
                                           const uint16_t *const *k_ptrs,
                                           const uint16_t *const *v_ptrs, const int32_t *tk,
                                           const int32_t *cap, size_t batch, size_t heads,
                                           size_t kv_heads, size_t head_dim, float scale,
                                           int32_t scale_q, llmtie_decode_scratch *scratch,
                                           const llmtie_exchange *xch,
                                           uint32_t *const *pair_flags);
llmtie_status llmtie_lse_merge_pairs(llmtie_gpu *g, const llmtie_exchange *xch,
                                     const uint32_t *pair_flags, uint32_t *merge_step, size_t rows,
                                     size_t rows_per_pair, size_t head_dim, float *out,
                                     size_t out_len);
/* AsrModel::attend (crates/llmtie-asr/src/model.rs:573-641) fused: n query
 * rows (q f32 [n][heads*hd], scale applied to q) over f16 cross caches
 * K [heads][cap][hd], V [heads][hd][cap] with tk live keys, non-causal;
 * out f32 [n][heads*hd]. */
llmtie_status llmtie_cross_attn(llmtie_gpu *g, const float *q, size_t q_len,
                                const uint16_t *k, size_t k_len, const uint16_t *v,
                                size_t v_len, size_t n, size_t heads, size_t head_dim,
                                size_t tk, size_t cap, float scale,
                                llmtie_decode_scratch *scratch, float *out,
                                size_t out_len);
/* ChatModel::run's prefill of one layer (crates/llmtie-chat/src/model.rs:
 * 848-889, :967-980) for `batch` packed ragged sequences in one call: RoPE on
 * q and k, the new K/V written into each sequence's f16 cache at past[b], and
 * causal attention. q f32 [total][heads*hd], k and v f32 [total][kv_heads*hd],
 * all three unrotated and none of them written (the reference's chain rotates
 * q in place; here q is rotated on its way into the attention kernel, in two
 * launches where the caches are 16-byte aligned with capacities that are
 * multiples of 8, and a copy of it otherwise). cu_seqlens HOST int32 [batch+1], past/cap/k_ptrs/v_ptrs HOST
 * arrays; out f32 [total][heads*hd]. */
llmtie_status llmtie_prefill_varlen(llmtie_gpu *g, const float *q, size_t q_len, const float *k,
                                    size_t k_len, const float *v, size_t v_len,
                                    const int32_t *cu_seqlens, size_t batch,
                                    uint16_t *const *k_ptrs, uint16_t *const *v_ptrs,
                                    const int32_t *past, const int32_t *cap,
                                    const float *freq_div, size_t heads, size_t kv_heads,
                                    size_t head_dim, float theta, float scale, float *out,
                                    size_t out_len);

/* ---- profiling ---------------------------------------------------------------- */

/* kprof (device.rs:1490-1565): with it on, every launch is bracketed by
 * events and charged to its kernel's name. The report is "name count ms"
 * lines; returns the bytes needed. */
void llmtie_kprof_enable(llmtie_gpu *g, int32_t on);
void llmtie_kprof_reset(llmtie_gpu *g);
size_t llmtie_kprof_report(llmtie_gpu *g, char *buf, size_t cap);
/* Gpu::kernel_resources (device.rs:1458-1465): registers per thread, local
 * bytes per thread, static shared bytes. */
llmtie_status llmtie_kernel_resources(const char *name, int32_t *regs, int32_t *local_bytes,
                                      int32_t *shared_bytes);
/* Kernels launched through this handle since it was opened. */
uint64_t llmtie_launch_count(llmtie_gpu *g);

#ifdef __cplusplus
}
#endif
#endif
