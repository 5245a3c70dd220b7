// The C ABI of llmtie_b200: the handle, host-side refusals and the dispatch
// to the kernels. Every range is checked here, before anything is launched,
// and refused by name, as `llmtie_cuda::Gpu` does
// (crates/llmtie-cuda/src/device.rs, error.rs:140-277).
#include "common.cuh"

#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <new>

namespace {

thread_local char g_err[512] = "";

constexpr float kLog2e = 1.4426950408889634f;

llmtie_status driver_fail(const char *what, cudaError_t e)
{
    return llmtie_fail(LLMTIE_ERR_DRIVER, "%s: %s", what, cudaGetErrorString(e));
}

size_t next_pow2(size_t x)
{
    size_t p = 1;
    while (p < x) p <<= 1;
    return p;
}

bool fits_i32(size_t x) { return x <= 0x7fffffffu; }

}  // namespace

static std::map<std::string, const void *> &kernel_table()
{
    static std::map<std::string, const void *> t;
    return t;
}

KernelReg::KernelReg(const char *name, const void *fn) { kernel_table()[name] = fn; }

const void *llmtie_kernel_symbol(const char *name)
{
    const auto it = kernel_table().find(name);
    return it == kernel_table().end() ? nullptr : it->second;
}

llmtie_status llmtie_fail(llmtie_status code, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

extern "C" const char *llmtie_last_error(void) { return g_err; }

void *workspace_reserve(Workspace &w, size_t bytes, cudaStream_t st, cudaError_t *err)
{
    *err = cudaSuccess;
    if (bytes <= w.bytes) return w.ptr;
    if (w.ptr) cudaFreeAsync(w.ptr, st);
    w.ptr = nullptr;
    w.bytes = 0;
    size_t want = 1 << 20;
    while (want < bytes) want <<= 1;
    *err = cudaMallocAsync(&w.ptr, want, st);
    if (*err != cudaSuccess) {
        w.ptr = nullptr;
        return nullptr;
    }
    w.bytes = want;
    return w.ptr;
}

LaunchScope::LaunchScope(llmtie_gpu *g_, const char *name_) : g(g_), name(name_)
{
    if (g->kprof) cudaEventRecord(g->ev0, g->stream);
}

llmtie_status LaunchScope::done()
{
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return driver_fail(name, e);
    g->launches++;
    if (g->kprof) {
        cudaEventRecord(g->ev1, g->stream);
        cudaEventSynchronize(g->ev1);
        float ms = 0.0f;
        cudaEventElapsedTime(&ms, g->ev0, g->ev1);
        KprofEntry &en = g->prof[name];
        en.count++;
        en.ms += ms;
    }
    return LLMTIE_OK;
}

#define NEED_HANDLE(g)                                                          \
    do {                                                                        \
        if (!(g)) return llmtie_fail(LLMTIE_ERR_INVALID, "null device handle"); \
        cudaSetDevice((g)->ordinal);                                            \
    } while (0)

// ---- handle ---------------------------------------------------------------

static llmtie_status open_impl(int32_t ordinal, void *stream, bool adopt, llmtie_gpu **out)
{
    if (!out) return llmtie_fail(LLMTIE_ERR_INVALID, "null output handle");
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        cudaGetLastError();
        return llmtie_fail(LLMTIE_ERR_NO_DEVICE, "no usable CUDA device: %s",
                           e != cudaSuccess ? cudaGetErrorString(e) : "no device present");
    }
    if (ordinal < 0 || ordinal >= count) {
        return llmtie_fail(LLMTIE_ERR_NO_DEVICE, "no usable CUDA device: ordinal %d of %d",
                           ordinal, count);
    }
    e = cudaSetDevice(ordinal);
    if (e != cudaSuccess) {
        return llmtie_fail(LLMTIE_ERR_NO_DEVICE, "no usable CUDA device: %s",
                           cudaGetErrorString(e));
    }
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, ordinal);
    if (e != cudaSuccess) return driver_fail("reading device properties", e);
    if (prop.major != 10) {
        // The kernels are compiled for sm_100a only; there is nothing to fall
        // back to, so a different part is "kernel not in the module".
        return llmtie_fail(LLMTIE_ERR_MISSING_KERNEL,
                           "kernels are built for sm_100a, device %d is sm_%d%d", ordinal,
                           prop.major, prop.minor);
    }
    llmtie_gpu *g = new (std::nothrow) llmtie_gpu();
    if (!g) return llmtie_fail(LLMTIE_ERR_DRIVER, "allocating the handle");
    g->ordinal = ordinal;
    g->sm_count = prop.multiProcessorCount;
    if (adopt) {
        g->stream = (cudaStream_t)stream;
        g->owns_stream = false;
    } else {
        e = cudaStreamCreateWithFlags(&g->stream, cudaStreamNonBlocking);
        if (e != cudaSuccess) {
            delete g;
            return driver_fail("creating the stream", e);
        }
        g->owns_stream = true;
    }
    cudaEventCreate(&g->ev0);
    cudaEventCreate(&g->ev1);
    // Keep freed blocks in the pool rather than returning them to the
    // driver between calls (device.rs:769-781).
    cudaMemPool_t pool;
    if (cudaDeviceGetDefaultMemPool(&pool, ordinal) == cudaSuccess) {
        uint64_t keep = UINT64_MAX;
        cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
    }
    e = cudaHostAlloc((void **)&g->timeout_host, sizeof(int), cudaHostAllocMapped);
    if (e == cudaSuccess) {
        *g->timeout_host = 0;
        e = cudaHostGetDevicePointer((void **)&g->timeout_site, g->timeout_host, 0);
    }
    if (e == cudaSuccess) e = cudaMalloc(&g->abort_epoch, sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(g->abort_epoch, 0, sizeof(int));
    if (e != cudaSuccess) {
        llmtie_close(g);
        return driver_fail("allocating the status word", e);
    }
    *out = g;
    return LLMTIE_OK;
}

extern "C" llmtie_status llmtie_open(int32_t ordinal, llmtie_gpu **out)
{
    return open_impl(ordinal, nullptr, false, out);
}

extern "C" llmtie_status llmtie_open_on_stream(int32_t ordinal, void *stream, llmtie_gpu **out)
{
    return open_impl(ordinal, stream, true, out);
}

extern "C" void llmtie_close(llmtie_gpu *g)
{
    if (!g) return;
    cudaSetDevice(g->ordinal);
    if (g->stream) cudaStreamSynchronize(g->stream);
    if (g->ws_rope.ptr) cudaFreeAsync(g->ws_rope.ptr, g->stream);
    if (g->ws_part.ptr) cudaFreeAsync(g->ws_part.ptr, g->stream);
    if (g->ws_kv16.ptr) cudaFreeAsync(g->ws_kv16.ptr, g->stream);
    if (g->stream) cudaStreamSynchronize(g->stream);
    if (g->abort_epoch) cudaFree(g->abort_epoch);
    if (g->timeout_host) cudaFreeHost(g->timeout_host);
    if (g->ev0) cudaEventDestroy(g->ev0);
    if (g->ev1) cudaEventDestroy(g->ev1);
    if (g->owns_stream && g->stream) cudaStreamDestroy(g->stream);
    delete g;
}

extern "C" void *llmtie_stream(llmtie_gpu *g) { return g ? (void *)g->stream : nullptr; }
extern "C" int32_t llmtie_ordinal(llmtie_gpu *g) { return g ? g->ordinal : -1; }

// After the stream has been waited for: whether a bounded device wait gave up
// since the last report. The word is host memory the kernels write through a
// mapping, so looking at it costs nothing. A timeout is reported once; the
// words are cleared, and so are the arrival counters of every DecodeScratch
// of this handle, which a launch that gave up may have left mid-count.
static llmtie_status report_device_timeout(llmtie_gpu *g)
{
    const int site = *(volatile int *)g->timeout_host;
    if (site == 0) return LLMTIE_OK;
    *(volatile int *)g->timeout_host = 0;
    cudaMemsetAsync(g->abort_epoch, 0, sizeof(int), g->stream);
    for (llmtie_decode_scratch *s : g->scratches) {
        if (s->ctr) cudaMemsetAsync(s->ctr, 0, s->ctr_words * sizeof(unsigned), g->stream);
    }
    return llmtie_fail(LLMTIE_ERR_TIMEOUT, "a bounded device wait gave up (site %d)", site);
}

extern "C" llmtie_status llmtie_synchronize(llmtie_gpu *g)
{
    NEED_HANDLE(g);
    const cudaError_t e = cudaStreamSynchronize(g->stream);
    if (e != cudaSuccess) return driver_fail("synchronizing", e);
    return report_device_timeout(g);
}

extern "C" llmtie_status llmtie_set_wait_limit_cycles(llmtie_gpu *g, int64_t cycles)
{
    NEED_HANDLE(g);
    g->wait_cycles = cycles > 0 ? (long long)cycles : (1ll << 31);
    return LLMTIE_OK;
}

// What a tensor-memory prefill launch is given for its bounded waits; every
// launch gets a number of its own.
static WaitCtl next_wait_ctl(llmtie_gpu *g)
{
    g->epoch = g->epoch == 0x7fffffff ? 1 : g->epoch + 1;
    return WaitCtl{g->timeout_site, g->abort_epoch, g->epoch, g->wait_cycles, g->sm_count,
                   &g->ws_part};
}

extern "C" llmtie_status llmtie_alloc(llmtie_gpu *g, size_t bytes, void **dptr)
{
    NEED_HANDLE(g);
    if (!dptr) return llmtie_fail(LLMTIE_ERR_INVALID, "null output pointer");
    cudaSetDevice(g->ordinal);
    const cudaError_t e = cudaMallocAsync(dptr, bytes ? bytes : 1, g->stream);
    if (e != cudaSuccess) return driver_fail("allocating", e);
    return LLMTIE_OK;
}

extern "C" llmtie_status llmtie_zeros(llmtie_gpu *g, size_t bytes, void **dptr)
{
    const llmtie_status s = llmtie_alloc(g, bytes, dptr);
    if (s != LLMTIE_OK) return s;
    const cudaError_t e = cudaMemsetAsync(*dptr, 0, bytes ? bytes : 1, g->stream);
    if (e != cudaSuccess) return driver_fail("zeroing", e);
    return LLMTIE_OK;
}

extern "C" llmtie_status llmtie_free(llmtie_gpu *g, void *dptr)
{
    NEED_HANDLE(g);
    if (!dptr) return LLMTIE_OK;
    const cudaError_t e = cudaFreeAsync(dptr, g->stream);
    if (e != cudaSuccess) return driver_fail("freeing", e);
    return LLMTIE_OK;
}

extern "C" llmtie_status llmtie_upload(llmtie_gpu *g, void *dst, const void *src, size_t bytes)
{
    NEED_HANDLE(g);
    const cudaError_t e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, g->stream);
    if (e != cudaSuccess) return driver_fail("uploading", e);
    return LLMTIE_OK;
}

extern "C" llmtie_status llmtie_download(llmtie_gpu *g, void *dst, const void *src, size_t bytes)
{
    NEED_HANDLE(g);
    cudaError_t e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, g->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(g->stream);
    if (e != cudaSuccess) return driver_fail("downloading", e);
    // What was just copied may be what a kernel that gave up never wrote.
    return report_device_timeout(g);
}

extern "C" llmtie_status llmtie_round_f16(llmtie_gpu *g, const float *src, uint16_t *dst,
                                          size_t n)
{
    NEED_HANDLE(g);
    LaunchScope ls(g, "round_f16");
    launch_round_f16(g->stream, src, dst, n);
    return ls.done();
}

// ---- KV-cache allocator ------------------------------------------------------

extern "C" size_t llmtie_kv_want_capacity(size_t cap, size_t past, size_t n,
                                          size_t max_positions)
{
    if (cap >= past + n) return 0;
    const size_t reserve = n > 1 ? 256 : 0;
    size_t want = std::max<size_t>(next_pow2(past + n + reserve), 256);
    want = std::min(want, std::max(max_positions, past + n));
    return want;
}

extern "C" size_t llmtie_kv_shared_prefix(const uint32_t *held, size_t held_len,
                                          const uint32_t *ids, size_t ids_len)
{
    if (!held || !ids || ids_len == 0) return 0;
    size_t n = 0;
    while (n < held_len && n < ids_len && held[n] == ids[n]) n++;
    return std::min(n, ids_len - 1);
}

extern "C" llmtie_status llmtie_kv_alloc_f16(llmtie_gpu *g, size_t kv_heads, size_t head_dim,
                                             size_t cap, uint16_t **k, uint16_t **v)
{
    NEED_HANDLE(g);
    if (!k || !v) return llmtie_fail(LLMTIE_ERR_INVALID, "null output pointer");
    if (cap % 2 != 0) {
        return llmtie_fail(LLMTIE_ERR_ODD_CACHE_CAPACITY,
                           "an f16 cache with an odd capacity of %zu", cap);
    }
    const size_t bytes = kv_heads * head_dim * cap * sizeof(uint16_t);
    llmtie_status s = llmtie_zeros(g, bytes, (void **)k);
    if (s != LLMTIE_OK) return s;
    s = llmtie_zeros(g, bytes, (void **)v);
    if (s != LLMTIE_OK) {
        llmtie_free(g, *k);
        *k = nullptr;
    }
    return s;
}

static llmtie_status grow_impl(llmtie_gpu *g, const void *src, size_t src_len, void *dst,
                               size_t dst_len, size_t kv_heads, size_t hd, size_t old_cap,
                               size_t new_cap, size_t live, bool transposed, int esize,
                               const char *name)
{
    NEED_HANDLE(g);
    if (live > old_cap || new_cap < old_cap) {
        return llmtie_fail(LLMTIE_ERR_CACHE_OVERRUN,
                           "appending at %zu to a cache with room for %zu",
                           std::max(live, old_cap), std::min(new_cap, old_cap));
    }
    const size_t rows = transposed ? kv_heads * hd : kv_heads;
    const size_t len = transposed ? live : live * hd;
    const size_t ss = transposed ? old_cap : old_cap * hd;
    const size_t ds = transposed ? new_cap : new_cap * hd;
    if (rows * ss > src_len) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu",
                           rows * ss, src_len);
    }
    if (rows * ds > dst_len) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu",
                           rows * ds, dst_len);
    }
    if (rows * len == 0) return LLMTIE_OK;
    LaunchScope ls(g, name);
    launch_cache_grow(g->stream, src, dst, (long long)rows, (long long)len, (long long)ss,
                      (long long)ds, esize);
    return ls.done();
}

extern "C" llmtie_status llmtie_cache_grow_f16(llmtie_gpu *g, const uint16_t *src,
                                               size_t src_len, uint16_t *dst, size_t dst_len,
                                               size_t kv_heads, size_t head_dim, size_t old_cap,
                                               size_t new_cap, size_t live, int32_t transposed)
{
    return grow_impl(g, src, src_len, dst, dst_len, kv_heads, head_dim, old_cap, new_cap, live,
                     transposed != 0, 2, "cache_grow_f16");
}

extern "C" llmtie_status llmtie_cache_grow(llmtie_gpu *g, const float *src, size_t src_len,
                                           float *dst, size_t dst_len, size_t kv_heads,
                                           size_t head_dim, size_t old_cap, size_t new_cap,
                                           size_t live, int32_t transposed)
{
    return grow_impl(g, src, src_len, dst, dst_len, kv_heads, head_dim, old_cap, new_cap, live,
                     transposed != 0, 4, "cache_grow");
}

static llmtie_status append_impl(llmtie_gpu *g, const float *src, size_t src_len,
                                 size_t src_off, void *dst, size_t dst_len, size_t n,
                                 size_t kv_heads, size_t hd, size_t cap, size_t past,
                                 bool transposed, bool f16)
{
    NEED_HANDLE(g);
    if (past + n > cap) {
        return llmtie_fail(LLMTIE_ERR_CACHE_OVERRUN,
                           "appending at %zu to a cache with room for %zu", past + n, cap);
    }
    if (f16 && cap % 2 != 0) {
        return llmtie_fail(LLMTIE_ERR_ODD_CACHE_CAPACITY,
                           "an f16 cache with an odd capacity of %zu", cap);
    }
    const size_t total = n * kv_heads * hd;
    if (src_off + total > src_len) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu",
                           src_off + total, src_len);
    }
    if (kv_heads * hd * cap > dst_len) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu",
                           kv_heads * hd * cap, dst_len);
    }
    if (!fits_i32(cap) || !fits_i32(n) || !fits_i32(kv_heads * hd)) {
        return llmtie_fail(LLMTIE_ERR_INVALID, "cache geometry does not fit 32 bits");
    }
    if (total == 0) return LLMTIE_OK;
    const char *name = f16 ? (transposed ? "cache_append_t_f16" : "cache_append_f16")
                           : (transposed ? "cache_append_t" : "cache_append");
    LaunchScope ls(g, name);
    launch_cache_append(g->stream, src, (long long)src_off, dst, (int)n, (int)kv_heads, (int)hd,
                        (int)cap, (int)past, transposed, f16);
    return ls.done();
}

extern "C" llmtie_status llmtie_cache_append_f16(llmtie_gpu *g, const float *src,
                                                 size_t src_len, size_t src_off, uint16_t *dst,
                                                 size_t dst_len, size_t n, size_t kv_heads,
                                                 size_t head_dim, size_t cap, size_t past,
                                                 int32_t transposed)
{
    return append_impl(g, src, src_len, src_off, dst, dst_len, n, kv_heads, head_dim, cap, past,
                       transposed != 0, true);
}

extern "C" llmtie_status llmtie_cache_append(llmtie_gpu *g, const float *src, size_t src_len,
                                             size_t src_off, float *dst, size_t dst_len,
                                             size_t n, size_t kv_heads, size_t head_dim,
                                             size_t cap, size_t past, int32_t transposed)
{
    return append_impl(g, src, src_len, src_off, dst, dst_len, n, kv_heads, head_dim, cap, past,
                       transposed != 0, false);
}

static llmtie_status misaligned(const char *what, const void *p, size_t align)
{
    return llmtie_fail(LLMTIE_ERR_MISALIGNED, "%s starts at %zu, which is not a multiple of %zu",
                       what, (size_t)(uintptr_t)p, align);
}

// ---- the projection in front of the Whisper decoder's self-attention -------------

extern "C" llmtie_status llmtie_gemv_qkv_f16(llmtie_gpu *g, const float *a, size_t a_len,
                                             const uint16_t *w, size_t w_len, const float *q_bias,
                                             const float *k_bias, const float *v_bias,
                                             size_t bias_len, size_t k, size_t d, size_t head_dim,
                                             size_t cap, size_t pos, float *q, size_t q_len,
                                             float *kc, size_t kc_len, float *vc, size_t vc_len)
{
    NEED_HANDLE(g);
    if (k % 2 != 0) {
        return llmtie_fail(LLMTIE_ERR_RAGGED_BLOCK,
                           "a contraction of %zu does not divide into pairs", k);
    }
    if (head_dim == 0 || d % head_dim != 0) {
        return llmtie_fail(LLMTIE_ERR_RAGGED_BLOCK, "a row of %zu does not divide into blocks of %zu",
                           d, head_dim);
    }
    if (pos >= cap) {
        return llmtie_fail(LLMTIE_ERR_CACHE_OVERRUN,
                           "appending at %zu to a cache with room for %zu", pos + 1, cap);
    }
    if (a_len < k) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu", k, a_len);
    }
    if (w_len < 3 * d * k) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu",
                           3 * d * k, w_len);
    }
    if (q_len < d) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu", d, q_len);
    }
    if (kc_len < d * cap || vc_len < d * cap) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu", d * cap,
                           std::min(kc_len, vc_len));
    }
    if ((q_bias || k_bias || v_bias) && bias_len < d) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu", d,
                           bias_len);
    }
    if (((uintptr_t)w & 3u) != 0) return misaligned("the stacked weight", w, 4);
    if (!fits_i32(k) || !fits_i32(3 * d) || !fits_i32(cap) || k * sizeof(float) > 200 * 1024) {
        return llmtie_fail(LLMTIE_ERR_INVALID, "projection geometry out of range");
    }
    if (d == 0) return LLMTIE_OK;
    LaunchScope ls(g, "gemv_qkv_f16");
    const cudaError_t e = launch_gemv_qkv_f16(g->stream, a, w, q_bias, k_bias, v_bias, (int)k, (int)d,
                                              (int)head_dim, (int)cap, (int)pos, q, kc, vc);
    if (e != cudaSuccess) return driver_fail("gemv_qkv_f16", e);
    return ls.done();
}

// ---- Whisper cross-attention cache build ----------------------------------------

static llmtie_status split_impl(llmtie_gpu *g, const float *x, size_t x_len, size_t x_off,
                                size_t x_layer, const float *bias, size_t bias_len,
                                size_t bias_off, size_t bias_layer, uint16_t *out, size_t out_len,
                                size_t layers, size_t t, size_t heads, size_t hd, size_t cap,
                                bool transposed)
{
    NEED_HANDLE(g);
    const size_t d = heads * hd, n = t * d;
    if (layers == 0 || n == 0) return LLMTIE_OK;
    if (cap < t) {
        return llmtie_fail(LLMTIE_ERR_CACHE_OVERRUN,
                           "appending at %zu to a cache with room for %zu", t, cap);
    }
    if (x_off + (layers - 1) * x_layer + n > x_len) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu",
                           x_off + (layers - 1) * x_layer + n, x_len);
    }
    if (bias && bias_off + (layers - 1) * bias_layer + d > bias_len) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu",
                           bias_off + (layers - 1) * bias_layer + d, bias_len);
    }
    if (layers * heads * cap * hd > out_len) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu",
                           layers * heads * cap * hd, out_len);
    }
    if (!fits_i32(t) || !fits_i32(d) || !fits_i32(cap) || !fits_i32(layers)) {
        return llmtie_fail(LLMTIE_ERR_INVALID, "cache geometry does not fit 32 bits");
    }
    LaunchScope ls(g, transposed ? "split_heads_t_f16" : "split_heads_f16");
    launch_split_heads(g->stream, x + x_off, (long long)x_layer, bias ? bias + bias_off : nullptr,
                       (long long)bias_layer, out, (long long)(heads * cap * hd), (int)layers,
                       (int)t, (int)heads, (int)hd, (int)cap, transposed);
    return ls.done();
}

extern "C" llmtie_status llmtie_split_heads_f16_at(llmtie_gpu *g, const float *x, size_t x_len,
                                                   size_t x_off, const float *bias,
                                                   size_t bias_len, size_t bias_off,
                                                   uint16_t *out, size_t out_len, size_t t,
                                                   size_t heads, size_t head_dim, size_t cap,
                                                   int32_t transposed)
{
    return split_impl(g, x, x_len, x_off, 0, bias, bias_len, bias_off, 0, out, out_len, 1, t, heads,
                      head_dim, cap, transposed != 0);
}

extern "C" llmtie_status llmtie_cross_kv_build(llmtie_gpu *g, const float *k_all, size_t k_len,
                                               const float *v_all, size_t v_len,
                                               const float *v_bias, size_t v_bias_len,
                                               uint16_t *k_out, size_t k_out_len, uint16_t *v_out,
                                               size_t v_out_len, size_t layers, size_t t,
                                               size_t heads, size_t head_dim, size_t cap)
{
    if (cap % 2 != 0) {
        return llmtie_fail(LLMTIE_ERR_ODD_CACHE_CAPACITY,
                           "an f16 cache with an odd capacity of %zu", cap);
    }
    const size_t d = heads * head_dim;
    llmtie_status s = split_impl(g, k_all, k_len, 0, t * d, nullptr, 0, 0, 0, k_out, k_out_len,
                                 layers, t, heads, head_dim, cap, false);
    if (s != LLMTIE_OK) return s;
    return split_impl(g, v_all, v_len, 0, t * d, v_bias, v_bias_len, 0, d, v_out, v_out_len, layers,
                      t, heads, head_dim, cap, true);
}

extern "C" llmtie_status llmtie_split_heads(llmtie_gpu *g, const float *x, size_t x_len,
                                            size_t x_off, float *out, size_t out_len, size_t t,
                                            size_t heads, size_t head_dim, size_t cap,
                                            int32_t transposed)
{
    NEED_HANDLE(g);
    const size_t n = t * heads * head_dim;
    if (n == 0) return LLMTIE_OK;
    if (cap < t) {
        return llmtie_fail(LLMTIE_ERR_CACHE_OVERRUN,
                           "appending at %zu to a cache with room for %zu", t, cap);
    }
    if (x_off + n > x_len) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu",
                           x_off + n, x_len);
    }
    if (heads * cap * head_dim > out_len) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu",
                           heads * cap * head_dim, out_len);
    }
    if (!fits_i32(t) || !fits_i32(heads * head_dim) || !fits_i32(cap)) {
        return llmtie_fail(LLMTIE_ERR_INVALID, "cache geometry does not fit 32 bits");
    }
    LaunchScope ls(g, transposed ? "split_heads_t" : "split_heads");
    launch_split_heads_f32(g->stream, x + x_off, out, (int)t, (int)heads, (int)head_dim, (int)cap,
                           transposed != 0);
    return ls.done();
}

// ---- RoPE ---------------------------------------------------------------------

extern "C" llmtie_status llmtie_rope_gptj(llmtie_gpu *g, float *x, size_t x_len,
                                          const float *inv_freq, size_t inv_len,
                                          size_t positions, size_t dim, size_t rot_dim)
{
    NEED_HANDLE(g);
    if (rot_dim % 2 != 0) {
        return llmtie_fail(LLMTIE_ERR_ODD_HEAD_DIM, "a rotary head of odd width %zu", rot_dim);
    }
    if (rot_dim > dim || positions * dim > x_len) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu",
                           rot_dim > dim ? rot_dim : positions * dim, rot_dim > dim ? dim : x_len);
    }
    if (inv_len < rot_dim / 2) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu",
                           rot_dim / 2, inv_len);
    }
    if (!fits_i32(positions) || !fits_i32(dim)) {
        return llmtie_fail(LLMTIE_ERR_INVALID, "rope geometry does not fit 32 bits");
    }
    if (positions * rot_dim == 0) return LLMTIE_OK;
    LaunchScope ls(g, "rope_gptj");
    launch_rope_gptj(g->stream, x, inv_freq, (int)positions, (int)dim, (int)rot_dim);
    return ls.done();
}

extern "C" llmtie_status llmtie_rope_scaled(llmtie_gpu *g, float *x, size_t x_len, size_t off,
                                            const float *freq_div, size_t t, size_t heads,
                                            size_t head_dim, float theta, size_t first)
{
    NEED_HANDLE(g);
    if (head_dim % 2 != 0) {
        return llmtie_fail(LLMTIE_ERR_ODD_HEAD_DIM, "a rotary head of odd width %zu", head_dim);
    }
    if (off + t * heads * head_dim > x_len) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu",
                           off + t * heads * head_dim, x_len);
    }
    if (!fits_i32(t) || !fits_i32(heads * head_dim) || !fits_i32(first + t)) {
        return llmtie_fail(LLMTIE_ERR_INVALID, "rope geometry does not fit 32 bits");
    }
    if (t * heads * head_dim == 0) return LLMTIE_OK;
    LaunchScope ls(g, "rope");
    launch_rope(g->stream, x, (long long)off, freq_div, (int)t, (int)heads, (int)head_dim, theta,
                (int)first);
    return ls.done();
}

extern "C" llmtie_status llmtie_rope_cache_f16(llmtie_gpu *g, float *q, size_t q_len,
                                               size_t q_off, const float *k, size_t k_len,
                                               size_t k_off, const float *v, size_t v_len,
                                               size_t v_off, const float *freq_div, size_t heads,
                                               size_t kv_heads, size_t head_dim, float theta,
                                               size_t pos, uint16_t *kc, size_t kc_len,
                                               uint16_t *vc, size_t vc_len, size_t cap)
{
    NEED_HANDLE(g);
    if (pos >= cap) {
        return llmtie_fail(LLMTIE_ERR_CACHE_OVERRUN,
                           "appending at %zu to a cache with room for %zu", pos + 1, cap);
    }
    if (cap % 2 != 0) {
        return llmtie_fail(LLMTIE_ERR_ODD_CACHE_CAPACITY,
                           "an f16 cache with an odd capacity of %zu", cap);
    }
    if (head_dim % 2 != 0) {
        return llmtie_fail(LLMTIE_ERR_ODD_HEAD_DIM, "a rotary head of odd width %zu", head_dim);
    }
    const size_t spans[3][3] = {{q_off, heads * head_dim, q_len},
                                {k_off, kv_heads * head_dim, k_len},
                                {v_off, kv_heads * head_dim, v_len}};
    for (const auto &s : spans) {
        if (s[0] + s[1] > s[2]) {
            return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu",
                               s[0] + s[1], s[2]);
        }
    }
    const size_t want = cap * kv_heads * head_dim;
    if (kc_len < want || vc_len < want) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu", want,
                           std::min(kc_len, vc_len));
    }
    if (!fits_i32(cap) || !fits_i32(heads * head_dim)) {
        return llmtie_fail(LLMTIE_ERR_INVALID, "cache geometry does not fit 32 bits");
    }
    // a batch of one through the batched kernel
    RopeBatchParams p;
    memset(&p, 0, sizeof(p));
    p.nseq = 1;
    p.seq[0] = {kc, vc, (int)pos, (int)cap, (long long)q_off, (long long)k_off, (long long)v_off};
    p.q = q;
    p.k = k;
    p.v = v;
    p.freq_div = freq_div;
    p.heads = (int)heads;
    p.kv_heads = (int)kv_heads;
    p.hd = (int)head_dim;
    p.theta = theta;
    LaunchScope ls(g, "rope_cache_f16");
    launch_rope_cache_batched(g->stream, p);
    return ls.done();
}

extern "C" llmtie_status llmtie_rope_cache_batched(
    llmtie_gpu *g, float *q, size_t q_len, const float *k, size_t k_len, const float *v,
    size_t v_len, const float *freq_div, size_t batch, size_t heads, size_t kv_heads,
    size_t head_dim, float theta, const int32_t *pos, uint16_t *const *kc_ptrs,
    uint16_t *const *vc_ptrs, const int32_t *cap)
{
    NEED_HANDLE(g);
    if (!pos || !kc_ptrs || !vc_ptrs || !cap) {
        return llmtie_fail(LLMTIE_ERR_INVALID, "null sequence table");
    }
    if (head_dim % 2 != 0) {
        return llmtie_fail(LLMTIE_ERR_ODD_HEAD_DIM, "a rotary head of odd width %zu", head_dim);
    }
    if (q_len < batch * heads * head_dim) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu",
                           batch * heads * head_dim, q_len);
    }
    if (k_len < batch * kv_heads * head_dim || v_len < batch * kv_heads * head_dim) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu",
                           batch * kv_heads * head_dim, std::min(k_len, v_len));
    }
    for (size_t b = 0; b < batch; b++) {
        if (cap[b] <= 0 || cap[b] % 2 != 0) {
            return llmtie_fail(LLMTIE_ERR_ODD_CACHE_CAPACITY,
                               "an f16 cache with an odd capacity of %d", cap[b]);
        }
        if (pos[b] < 0 || pos[b] >= cap[b]) {
            return llmtie_fail(LLMTIE_ERR_CACHE_OVERRUN,
                               "appending at %d to a cache with room for %d", pos[b] + 1, cap[b]);
        }
    }
    for (size_t b0 = 0; b0 < batch; b0 += 32) {
        const size_t nb = std::min<size_t>(32, batch - b0);
        RopeBatchParams p;
        memset(&p, 0, sizeof(p));
        p.nseq = (int)nb;
        for (size_t b = 0; b < nb; b++) {
            p.seq[b] = {kc_ptrs[b0 + b], vc_ptrs[b0 + b], pos[b0 + b], cap[b0 + b],
                        (long long)(b * heads * head_dim), (long long)(b * kv_heads * head_dim),
                        (long long)(b * kv_heads * head_dim)};
        }
        p.q = q + b0 * heads * head_dim;
        p.k = k + b0 * kv_heads * head_dim;
        p.v = v + b0 * kv_heads * head_dim;
        p.freq_div = freq_div;
        p.heads = (int)heads;
        p.kv_heads = (int)kv_heads;
        p.hd = (int)head_dim;
        p.theta = theta;
        LaunchScope ls(g, "rope_cache_f16");
        launch_rope_cache_batched(g->stream, p);
        const llmtie_status s = ls.done();
        if (s != LLMTIE_OK) return s;
    }
    return LLMTIE_OK;
}

// ---- prefill / encoder attention -----------------------------------------------

extern "C" int32_t llmtie_supports_flash(size_t head_dim, size_t heads, size_t kv_heads)
{
    return (head_dim == 64 || head_dim == 128) && heads % std::max<size_t>(kv_heads, 1) == 0;
}

static llmtie_status unsupported(size_t hd, size_t heads, size_t kv)
{
    return llmtie_fail(LLMTIE_ERR_UNSUPPORTED_ATTENTION,
                       "fused attention wants head_dim 64 or 128 and heads a multiple of "
                       "kv_heads, got head_dim %zu, %zu heads over %zu",
                       hd, heads, kv);
}


// Whether a prefill takes the tensor-memory kernel (aligned f16 caches at
// head_dim 128) or the general one. LLMTIE_B200_NO_TC forces the general one.
static bool use_tc(const PrefillParams &p, int hd)
{
    static const bool off = getenv("LLMTIE_B200_NO_TC") != nullptr;
    return !off && prefill_tc_eligible(p, hd);
}

// One sequence through the fused prefill kernels.
static llmtie_status flash_impl(llmtie_gpu *g, const char *name, const float *q, size_t q_len,
                                const void *k, size_t k_len, const void *v, size_t v_len,
                                void *out, size_t out_len, size_t tq, size_t past, size_t heads,
                                size_t kv_heads, size_t hd, size_t cap, float scale, bool causal,
                                bool kv_f32)
{
    NEED_HANDLE(g);
    if (kv_heads == 0 || heads % kv_heads != 0) return unsupported(hd, heads, kv_heads);
    if (past + tq > cap) {
        return llmtie_fail(LLMTIE_ERR_CACHE_OVERRUN,
                           "appending at %zu to a cache with room for %zu", past + tq, cap);
    }
    if (tq * heads * hd > q_len) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu",
                           tq * heads * hd, q_len);
    }
    if (tq * heads * hd > out_len) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu",
                           tq * heads * hd, out_len);
    }
    const size_t need = kv_heads * cap * hd;
    if (k_len < need || v_len < need) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu", need,
                           std::min(k_len, v_len));
    }
    if (((uintptr_t)q & 15u) != 0) return misaligned("the query", q, 16);
    if (((uintptr_t)k & 15u) != 0) return misaligned("the key cache", k, 16);
    if (((uintptr_t)out & 7u) != 0) return misaligned("the output", out, 8);
    if (!fits_i32(cap) || !fits_i32(tq) || !fits_i32(heads * hd)) {
        return llmtie_fail(LLMTIE_ERR_INVALID, "attention geometry does not fit 32 bits");
    }
    if (tq == 0) return LLMTIE_OK;
    PrefillParams p;
    memset(&p, 0, sizeof(p));
    p.nseq = 1;
    p.seq[0].k = k;
    p.seq[0].v = v;
    p.seq[0].row0 = 0;
    p.seq[0].tq = (int)tq;
    p.seq[0].past = (int)past;
    p.seq[0].cap = (int)cap;
    p.seq[0].tk = (int)(past + tq);
    p.q = q;
    p.q_stride = (long long)(heads * hd);
    p.out = out;
    p.out_stride = (long long)(heads * hd);
    p.heads = (int)heads;
    p.kv_heads = (int)kv_heads;
    p.causal = causal ? 1 : 0;
    p.kv_f32 = kv_f32 ? 1 : 0;
    p.out_f16 = 0;
    p.q_scale = 1.0f;
    p.sl2 = scale * kLog2e;
    // Caches the tensor-memory kernel cannot lay its tiles over go through an
    // f16 copy of their live keys, in caches of the handle's own, first:
    // - f32 caches (Whisper's self-attention twins, the speech LM's prefill,
    //   the flow model's attention): the fused kernels round K and V to f16 as
    //   they read them (crates/llmtie-cuda/src/kernels.rs:3078-3269), so the
    //   live keys are rounded once and the same numbers go through tcgen05
    //   instead of mma.sync;
    // - f16 caches whose value rows are not 16-byte aligned (a capacity that
    //   is not a multiple of 8, an odd address): re-strided bit for bit.
    // (LLMTIE_B200_NO_STAGING keeps such calls on the general kernel: an A/B
    // switch.)
    static const bool no_staging = getenv("LLMTIE_B200_NO_STAGING") != nullptr;
    bool staged = false;
    if (!no_staging && (kv_f32 || !use_tc(p, (int)hd))) {
        const size_t live = past + tq;
        const size_t cap16 = (live + 7) / 8 * 8;
        const size_t half = kv_heads * cap16 * hd * sizeof(uint16_t);
        PrefillParams t = p;
        t.kv_f32 = 0;
        t.seq[0].cap = (int)cap16;
        cudaError_t werr;
        // (eligibility is a matter of shapes and alignments: asked with a
        // stand-in pointer before anything is allocated)
        t.seq[0].k = t.seq[0].v = (const void *)(uintptr_t)256;
        if (use_tc(t, (int)hd)) {
            void *work = workspace_reserve(g->ws_kv16, 2 * half + 256, g->stream, &werr);
            if (!work) return driver_fail("allocating", werr);
            uint16_t *k16 = (uint16_t *)work;
            uint16_t *v16 = (uint16_t *)((char *)work + (half + 255) / 256 * 256);
            {
                LaunchScope ls(g, "caches_to_f16");
                launch_caches_to_f16(g->stream, k, v, kv_f32, k16, v16, (int)kv_heads, (int)hd,
                                     (int)cap, (int)cap16, (int)live);
                const llmtie_status st = ls.done();
                if (st != LLMTIE_OK) return st;
            }
            p = t;
            p.seq[0].k = k16;
            p.seq[0].v = v16;
            static const bool no_pdl = getenv("LLMTIE_B200_NO_PDL") != nullptr;
            p.after_prepass = (!no_pdl && !g->kprof) ? 1 : 0;   // under the copy's tail
            staged = true;
        }
    }
    // kprof tells the two kernels apart: the tensor-memory one is charged to
    // "flash_attn_h_tc" (f16 caches as they lie) or "flash_attn_tc" (staged)
    const bool tc = staged || use_tc(p, (int)hd);
    LaunchScope ls(g, tc ? (staged ? "flash_attn_tc" : "flash_attn_h_tc") : name);
    const cudaError_t e = tc ? launch_prefill_tc(g->stream, p, (int)hd, next_wait_ctl(g))
                             : launch_prefill_mma(g->stream, p, (int)hd);
    if (e != cudaSuccess) return driver_fail(name, e);
    return ls.done();
}

extern "C" llmtie_status llmtie_flash_attn_f16(llmtie_gpu *g, const float *q, size_t q_len,
                                               const uint16_t *k, size_t k_len,
                                               const uint16_t *v, size_t v_len, float *out,
                                               size_t out_len, size_t tq, size_t past,
                                               size_t heads, size_t kv_heads, size_t head_dim,
                                               size_t cap, float scale, int32_t causal)
{
    if (head_dim != 128) return unsupported(head_dim, heads, kv_heads);
    if (cap % 2 != 0) {
        return llmtie_fail(LLMTIE_ERR_ODD_CACHE_CAPACITY,
                           "an f16 cache with an odd capacity of %zu", cap);
    }
    return flash_impl(g, "flash_attn_h", q, q_len, k, k_len, v, v_len, out, out_len, tq, past,
                      heads, kv_heads, head_dim, cap, scale, causal != 0, false);
}

extern "C" llmtie_status llmtie_flash_attn(llmtie_gpu *g, const float *q, size_t q_len,
                                           const float *k, size_t k_len, const float *v,
                                           size_t v_len, float *out, size_t out_len, size_t tq,
                                           size_t past, size_t heads, size_t kv_heads,
                                           size_t head_dim, size_t cap, float scale,
                                           int32_t causal)
{
    if (head_dim != 64 && head_dim != 128) return unsupported(head_dim, heads, kv_heads);
    return flash_impl(g, head_dim == 128 ? "flash_attn" : "flash_attn_64", q, q_len, k, k_len, v,
                      v_len, out, out_len, tq, past, heads, kv_heads, head_dim, cap, scale,
                      causal != 0, true);
}

static size_t rows_pad(size_t t) { return (t + 127) / 128 * 128; }

extern "C" size_t llmtie_flash_rows_work_bytes(size_t t, size_t heads, size_t head_dim)
{
    return 2 * heads * rows_pad(t) * head_dim * sizeof(uint16_t);
}

static llmtie_status flash_rows_impl(llmtie_gpu *g, const float *qkv, size_t qkv_len,
                                     uint16_t *out, size_t out_len, size_t batch, size_t t,
                                     size_t heads, size_t head_dim, float scale, void *work,
                                     size_t work_bytes)
{
    NEED_HANDLE(g);
    if (head_dim != 64) return unsupported(head_dim, heads, heads);
    const size_t d = heads * head_dim;
    if (qkv_len < batch * t * 3 * d) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu",
                           batch * t * 3 * d, qkv_len);
    }
    if (out_len < batch * t * d) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu",
                           batch * t * d, out_len);
    }
    if (((uintptr_t)qkv & 15u) != 0) return misaligned("the stacked product", qkv, 16);
    if (((uintptr_t)out & 3u) != 0) return misaligned("the output", out, 4);
    if (!fits_i32(batch * t) || !fits_i32(3 * d) || batch > 65535) {
        return llmtie_fail(LLMTIE_ERR_INVALID, "attention geometry does not fit 32 bits");
    }
    if (t == 0 || heads == 0 || batch == 0) return LLMTIE_OK;
    const size_t one = llmtie_flash_rows_work_bytes(t, heads, head_dim);
    const size_t need = batch * one;
    void *own = nullptr;
    if (work) {
        if (work_bytes < need) {
            return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu",
                               need, work_bytes);
        }
        if (((uintptr_t)work & 15u) != 0) return misaligned("the work buffer", work, 16);
    } else {
        const llmtie_status s = llmtie_alloc(g, need, &own);
        if (s != LLMTIE_OK) return s;
        work = own;
    }
    const size_t tp = rows_pad(t);
    uint16_t *ks = (uint16_t *)work;
    uint16_t *vs = ks + heads * tp * head_dim;
    llmtie_status st;
    {
        LaunchScope ls(g, "rows_stage");
        launch_rows_stage(g->stream, qkv, ks, vs, (int)t, (int)tp, (int)heads, (int)head_dim,
                          (int)batch);
        st = ls.done();
    }
    // the attention kernel carries LLMTIE_TC_MAX_SEQ utterances a launch
    for (size_t b0 = 0; b0 < batch && st == LLMTIE_OK; b0 += LLMTIE_TC_MAX_SEQ) {
        const size_t nb = std::min<size_t>(LLMTIE_TC_MAX_SEQ, batch - b0);
        PrefillParams p;
        memset(&p, 0, sizeof(p));
        p.nseq = (int)nb;
        for (size_t b = 0; b < nb; b++) {
            p.seq[b].k = ks + (b0 + b) * (one / sizeof(uint16_t));
            p.seq[b].v = vs + (b0 + b) * (one / sizeof(uint16_t));
            p.seq[b].row0 = (int)(b * t);
            p.seq[b].tq = (int)t;
            p.seq[b].cap = (int)tp;
            p.seq[b].tk = (int)t;
        }
        p.q = qkv + b0 * t * 3 * d;
        p.q_stride = (long long)(3 * d);
        p.out = out + b0 * t * d;
        p.out_stride = (long long)d;
        p.heads = (int)heads;
        p.kv_heads = (int)heads;
        p.causal = 0;
        p.kv_f32 = 0;
        p.out_f16 = 1;
        p.q_scale = scale;   // on q before it is rounded, as the encoder does
        p.sl2 = kLog2e;
        // (the first launch sets itself up under the staging kernel's tail)
        static const bool no_pdl = getenv("LLMTIE_B200_NO_PDL") != nullptr;
        p.after_prepass = (b0 == 0 && !no_pdl && !g->kprof) ? 1 : 0;
        const bool tc = use_tc(p, 64);
        LaunchScope ls(g, tc ? "flash_attn_64_rows_tc" : "flash_attn_64_rows");
        const cudaError_t e = tc ? launch_prefill_tc(g->stream, p, 64, next_wait_ctl(g))
                                 : launch_prefill_mma(g->stream, p, 64);
        st = (e != cudaSuccess) ? driver_fail("flash_attn_64_rows", e) : ls.done();
    }
    if (own) llmtie_free(g, own);
    return st;
}

extern "C" llmtie_status llmtie_flash_attn_rows(llmtie_gpu *g, const float *qkv, size_t qkv_len,
                                                uint16_t *out, size_t out_len, size_t t,
                                                size_t heads, size_t head_dim, float scale,
                                                void *work, size_t work_bytes)
{
    return flash_rows_impl(g, qkv, qkv_len, out, out_len, 1, t, heads, head_dim, scale, work,
                           work_bytes);
}

extern "C" llmtie_status llmtie_flash_attn_rows_batched(
    llmtie_gpu *g, const float *qkv, size_t qkv_len, uint16_t *out, size_t out_len, size_t batch,
    size_t t, size_t heads, size_t head_dim, float scale, void *work, size_t work_bytes)
{
    return flash_rows_impl(g, qkv, qkv_len, out, out_len, batch, t, heads, head_dim, scale, work,
                           work_bytes);
}

// ---- decode attention -----------------------------------------------------------

extern "C" llmtie_status llmtie_decode_scratch_new(llmtie_gpu *g, llmtie_decode_scratch **out)
{
    NEED_HANDLE(g);
    if (!out) return llmtie_fail(LLMTIE_ERR_INVALID, "null output pointer");
    *out = new (std::nothrow) llmtie_decode_scratch();
    if (!*out) return llmtie_fail(LLMTIE_ERR_DRIVER, "allocating the scratch");
    g->scratches.push_back(*out);
    return LLMTIE_OK;
}

extern "C" void llmtie_decode_scratch_free(llmtie_gpu *g, llmtie_decode_scratch *s)
{
    if (!s) return;
    if (g) {
        if (s->part) cudaFreeAsync(s->part, g->stream);
        if (s->ctr) cudaFreeAsync(s->ctr, g->stream);
        g->scratches.erase(std::remove(g->scratches.begin(), g->scratches.end(), s),
                           g->scratches.end());
    }
    delete s;
}

// Grows the scratch to hold `partials` partial triples and `pairs` counters. Stream-ordered,
// so a kernel still reading the old buffers is not disturbed; counters are
// zero when allocated and every launch leaves them at zero.
static llmtie_status scratch_reserve(llmtie_gpu *g, llmtie_decode_scratch *s, size_t pairs,
                                     size_t partials, size_t hd)
{
    const size_t floats = partials * 8 * (hd + 2);
    if (floats > s->part_floats) {
        if (s->part) cudaFreeAsync(s->part, g->stream);
        s->part = nullptr;
        s->part_floats = 0;
        const size_t want = next_pow2(floats);
        const cudaError_t e = cudaMallocAsync((void **)&s->part, want * sizeof(float), g->stream);
        if (e != cudaSuccess) return driver_fail("allocating", e);
        s->part_floats = want;
    }
    if (pairs > s->ctr_words) {
        if (s->ctr) cudaFreeAsync(s->ctr, g->stream);
        s->ctr = nullptr;
        s->ctr_words = 0;
        const size_t want = next_pow2(pairs);
        cudaError_t e = cudaMallocAsync((void **)&s->ctr, want * sizeof(unsigned), g->stream);
        if (e == cudaSuccess) e = cudaMemsetAsync(s->ctr, 0, want * sizeof(unsigned), g->stream);
        if (e != cudaSuccess) return driver_fail("allocating", e);
        s->ctr_words = want;
    }
    return LLMTIE_OK;
}

// Picks how the keys are cut into blocks of the grid. Every block should be
// resident at once and finish with the others, so the span is the smallest
// multiple of 128 keys for which the whole launch is at most one wave.
static void decode_plan(llmtie_gpu *g, DecodeParams &p, int hd)
{
    int max_tk = 0;
    long long keys = 0;
    for (int b = 0; b < p.nseq; b++) {
        max_tk = std::max(max_tk, p.seq[b].tk);
        keys += p.seq[b].tk;
    }
    // Long rows are worth reading in longer runs along the transposed value
    // cache; short contexts want the finest split instead.
    static const int forced = [] {
        const char *e = getenv("LLMTIE_B200_DECODE_NB");
        return e ? atoi(e) : 0;
    }();
    const long long per_pair = keys / std::max(1, p.nseq);
    int nb = per_pair >= 8192 ? 2 : 1;
    if (forced == 1 || forced == 2 || forced == 4 || forced == 8) nb = forced;
    p.nb = nb;
    const int slots = decode_resident_blocks(hd, g->sm_count, nb);
    const long long pairs = (long long)p.kv_heads * p.row_chunks;
    long long per = 1;   // span in units of 128 keys
    for (;;) {
        long long blocks = 0;
        for (int b = 0; b < p.nseq; b++) {
            blocks += ((p.seq[b].tk + per * 128 - 1) / (per * 128)) * pairs;
        }
        if (blocks <= slots || per * 128 >= max_tk) break;
        // jump straight to the span the block count suggests, then refine
        const long long guess = (per * blocks + slots - 1) / slots;
        per = std::max(per + 1, guess);
    }
    p.span = (int)(per * 128);
    p.max_splits = (max_tk + p.span - 1) / p.span;
}

// What the fused exchange adds to an exchange descriptor: every rank's pair
// flags and where this rank's merged rows go.
struct FusedMerge {
    uint32_t *const *pair_flags;
    float *out;
    int mode;   // 1: merge inside the decode kernel; 2: raise the pair flags only
};

static llmtie_status decode_launch(llmtie_gpu *g, const char *name, DecodeParams &p, int hd,
                                   llmtie_decode_scratch *scratch,
                                   const llmtie_exchange *xch = nullptr,
                                   const FusedMerge *fused = nullptr)
{
    // `aligned`: a tensor map can be laid over the value rows too; `ring`: the
    // ring kernel can take the launch (the keys by TMA; value rows that are
    // only 8-byte aligned by cp.async from the lanes)
    bool aligned = true, ring = true;
    for (int b = 0; b < p.nseq; b++) {
        if (p.seq[b].cap % 8 != 0 || ((uintptr_t)p.seq[b].v & 15u) != 0) aligned = false;
        if (p.seq[b].cap % 4 != 0 || ((uintptr_t)p.seq[b].v & 7u) != 0 ||
            ((uintptr_t)p.seq[b].k & 15u) != 0) {
            ring = false;
        }
    }
    static const bool no_stream = getenv("LLMTIE_B200_DECODE_NO_STREAM") != nullptr;
    static const bool no_plain = getenv("LLMTIE_B200_DECODE_NO_PLAIN_V") != nullptr;
    if (no_plain && !aligned) ring = false;
    if (xch && !aligned) {
        return llmtie_fail(LLMTIE_ERR_MISALIGNED,
                           "the exchanging decode wants 16-byte aligned caches and capacities "
                           "that are multiples of 8");
    }
    if (ring && (!no_stream || xch)) {
        // The ring kernel, cut by work: one block per SM, never more blocks
        // than 128-key units.
        DecodeStreamParams sp;
        memset(&sp, 0, sizeof(sp));
        const int inner = p.kv_heads * p.row_chunks;
        long long units = 0;
        for (int b = 0; b < p.nseq; b++) {
            sp.seq[b] = p.seq[b];
            sp.unit0[b] = units;
            sp.pair0[b] = b * inner;
            units += (long long)((p.seq[b].tk + 127) / 128) * inner;
        }
        sp.unit0[p.nseq] = units;
        sp.pair0[p.nseq] = p.nseq * inner;
        sp.total_units = units;
        sp.q = p.q;
        sp.q_seq = p.q_seq;
        sp.q_kv = p.q_kv;
        sp.q_row = p.q_row;
        sp.out = p.out;
        sp.out_seq = p.out_seq;
        sp.out_kv = p.out_kv;
        sp.out_row = p.out_row;
        sp.rows = p.rows;
        sp.row_chunks = p.row_chunks;
        sp.kv_heads = p.kv_heads;
        sp.nseq = p.nseq;
        sp.partial = p.partial;
        sp.q_scale = p.q_scale;
        sp.sl2 = p.sl2;
        sp.twin_q = p.twin_q;
        sp.twin_s = p.twin_s;
        sp.status = g->timeout_site;
        sp.wait_cycles = g->wait_cycles;
        sp.v_plain = aligned ? 0 : 1;
        // The tensor maps of the caches, kept with the scratch: they are made
        // again only when a cache has moved or changed shape.
        for (int b = 0; b < p.nseq; b++) {
            DecodeMapKey &key = scratch->map_key[b];
            if (key.k != p.seq[b].k || key.v != p.seq[b].v || key.cap != p.seq[b].cap ||
                key.kv_heads != p.kv_heads || key.hd != hd || (aligned && !key.has_v)) {
                if (!decode_tensor_maps(&scratch->kmap[b], aligned ? &scratch->vmap[b] : nullptr,
                                        p.seq[b].k, p.seq[b].v, p.kv_heads, p.seq[b].cap, hd)) {
                    key = DecodeMapKey();
                    return llmtie_fail(LLMTIE_ERR_DRIVER, "making the tensor maps of a cache");
                }
                key.k = p.seq[b].k;
                key.v = p.seq[b].v;
                key.cap = p.seq[b].cap;
                key.kv_heads = p.kv_heads;
                key.hd = hd;
                key.has_v = aligned;
            }
            sp.kmap[b] = scratch->kmap[b];
            sp.vmap[b] = scratch->vmap[b];
        }
        // One block per SM, but never fewer than four units (512 keys) a block:
        // a short context cut any finer spends longer merging partials than
        // it saved streaming them. (Whole pairs are another matter: as many
        // blocks as pairs cost no merge at all, and spare a block from walking
        // several short pairs one after the other.)
        // (LLMTIE_B200_DECODE_GRID caps the block count: a tuning switch)
        static const int grid_cap = [] {
            const char *e = getenv("LLMTIE_B200_DECODE_GRID");
            const int v = e ? atoi(e) : 0;
            return v > 0 ? v : LLMTIE_STREAM_MAX_BLOCKS;
        }();
        const int grid =
            decode_work_grid(units, (long long)p.nseq * inner, std::min(g->sm_count, grid_cap));
        const size_t pairs = (size_t)p.nseq * inner;
        const llmtie_status s =
            scratch_reserve(g, scratch, pairs + 1, (size_t)grid * 2, (size_t)hd);
        if (s != LLMTIE_OK) return s;
        sp.part = scratch->part;
        sp.ctr = scratch->ctr;
        if (xch) {
            sp.xch_world = xch->world;
            sp.xch_rank = xch->rank;
            for (int r = 0; r < xch->world; r++) {
                sp.xch_gather[r] = xch->gather[r];
                sp.xch_flags[r] = xch->flags[r];
            }
            sp.xch_step = xch->step;
            sp.xch_done = scratch->ctr + pairs;   // one more counter after the pairs'
            sp.xch_pairs = (int)pairs;
            sp.xch_rank_stride = (long long)p.nseq * p.out_seq;
            if (fused) {
                sp.xch_fused = fused->mode;
                for (int r = 0; r < xch->world; r++) sp.xch_pflags[r] = fused->pair_flags[r];
                sp.xch_out = fused->out;
                sp.xch_status = g->timeout_site;
                sp.xch_wait_cycles = g->wait_cycles;
            }
        }
        LaunchScope ls(g, name);
        const cudaError_t e = launch_decode_stream(g->stream, sp, hd, grid);
        if (e != cudaSuccess) return driver_fail(name, e);
        return ls.done();
    }
    decode_plan(g, p, hd);
    const size_t pairs = (size_t)p.nseq * p.row_chunks * p.kv_heads;
    const llmtie_status s =
        scratch_reserve(g, scratch, pairs, pairs * (size_t)p.max_splits, (size_t)hd);
    if (s != LLMTIE_OK) return s;
    p.part = scratch->part;
    p.ctr = scratch->ctr;
    LaunchScope ls(g, name);
    const cudaError_t e = launch_decode_f16(g->stream, p, hd);
    if (e != cudaSuccess) return driver_fail(name, e);
    return ls.done();
}

static llmtie_status attn_decode_f16_impl(llmtie_gpu *g, const float *q, size_t q_len,
                                          size_t q_off, const uint16_t *k, size_t k_len,
                                          const uint16_t *v, size_t v_len, size_t heads,
                                          size_t kv_heads, size_t head_dim, size_t tk, size_t cap,
                                          float scale, int32_t scale_q,
                                          llmtie_decode_scratch *scratch, float *out,
                                          size_t out_len, size_t out_off, int8_t *codes,
                                          size_t codes_len, float *scales, size_t scales_len,
                                          bool twin)
{
    NEED_HANDLE(g);
    if (!scratch) return llmtie_fail(LLMTIE_ERR_INVALID, "null decode scratch");
    if (cap % 2 != 0) {
        return llmtie_fail(LLMTIE_ERR_ODD_CACHE_CAPACITY,
                           "an f16 cache with an odd capacity of %zu", cap);
    }
    if (head_dim != 64 && head_dim != 128) return unsupported(head_dim, heads, kv_heads);
    // The widest query group the reference's instantiations carry: four at
    // 128, eight at 64 (device.rs:6043-6049, :6245-6252).
    const size_t gmax = head_dim == 128 ? 4 : 8;
    if (kv_heads == 0 || heads % kv_heads != 0 || heads / kv_heads > gmax) {
        return unsupported(head_dim, heads, kv_heads);
    }
    if (tk == 0 || tk > cap) {
        return llmtie_fail(LLMTIE_ERR_CACHE_OVERRUN,
                           "appending at %zu to a cache with room for %zu", tk, cap);
    }
    if ((cap * 2) % 8 != 0) {
        return llmtie_fail(LLMTIE_ERR_ODD_CACHE_CAPACITY,
                           "an f16 cache with an odd capacity of %zu", cap);
    }
    const size_t need = kv_heads * cap * head_dim;
    if (k_len < need || v_len < need) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu", need,
                           std::min(k_len, v_len));
    }
    const size_t n = heads * head_dim;
    if (q_len < q_off + n) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu",
                           q_off + n, q_len);
    }
    if (out_len < out_off + n) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu",
                           out_off + n, out_len);
    }
    if (out_off % 32 != 0) {
        return llmtie_fail(LLMTIE_ERR_RAGGED_BLOCK,
                           "a row of %zu does not divide into blocks of 32", out_off);
    }
    if (((uintptr_t)k & 15u) != 0) return misaligned("the key cache", k, 16);
    if (((uintptr_t)v & 7u) != 0) return misaligned("the value cache", v, 8);
    if (!fits_i32(cap)) return llmtie_fail(LLMTIE_ERR_INVALID, "capacity does not fit 32 bits");
    const size_t group = heads / kv_heads;
    DecodeParams p;
    memset(&p, 0, sizeof(p));
    p.nseq = 1;
    p.seq[0].k = k;
    p.seq[0].v = v;
    p.seq[0].tk = (int)tk;
    p.seq[0].cap = (int)cap;
    p.q = q + q_off;
    p.q_kv = (long long)(group * head_dim);
    p.q_row = (long long)head_dim;
    p.out = out + out_off;
    p.out_kv = (long long)(group * head_dim);
    p.out_row = (long long)head_dim;
    p.rows = (int)group;
    p.row_chunks = 1;
    p.kv_heads = (int)kv_heads;
    p.partial = 0;
    p.q_scale = scale_q ? scale : 1.0f;
    p.sl2 = (scale_q ? 1.0f : scale) * kLog2e;
    if (twin) {
        if (!codes || !scales) return llmtie_fail(LLMTIE_ERR_INVALID, "null twin buffers");
        if (codes_len < out_off + n) {
            return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu",
                               out_off + n, codes_len);
        }
        if (scales_len < (out_off + n) / 32) {
            return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu",
                               (out_off + n) / 32, scales_len);
        }
        // indexed as `out` is, from the same offset (out_off is a multiple of 32)
        p.twin_q = (signed char *)codes + out_off;
        p.twin_s = scales + out_off / 32;
    }
    return decode_launch(g, head_dim == 128 ? "attn_decode_h128" : "attn_decode_h64", p,
                         (int)head_dim, scratch);
}

extern "C" llmtie_status llmtie_attn_decode_f16(llmtie_gpu *g, const float *q, size_t q_len,
                                                size_t q_off, const uint16_t *k, size_t k_len,
                                                const uint16_t *v, size_t v_len, size_t heads,
                                                size_t kv_heads, size_t head_dim, size_t tk,
                                                size_t cap, float scale, int32_t scale_q,
                                                llmtie_decode_scratch *scratch, float *out,
                                                size_t out_len, size_t out_off)
{
    return attn_decode_f16_impl(g, q, q_len, q_off, k, k_len, v, v_len, heads, kv_heads, head_dim,
                                tk, cap, scale, scale_q, scratch, out, out_len, out_off, nullptr,
                                0, nullptr, 0, false);
}

extern "C" llmtie_status llmtie_attn_decode_f16_q(
    llmtie_gpu *g, const float *q, size_t q_len, size_t q_off, const uint16_t *k, size_t k_len,
    const uint16_t *v, size_t v_len, size_t heads, size_t kv_heads, size_t head_dim, size_t tk,
    size_t cap, float scale, int32_t scale_q, llmtie_decode_scratch *scratch, float *out,
    size_t out_len, size_t out_off, int8_t *codes, size_t codes_len, float *scales,
    size_t scales_len)
{
    return attn_decode_f16_impl(g, q, q_len, q_off, k, k_len, v, v_len, heads, kv_heads, head_dim,
                                tk, cap, scale, scale_q, scratch, out, out_len, out_off, codes,
                                codes_len, scales, scales_len, true);
}

extern "C" llmtie_status llmtie_attn_decode(llmtie_gpu *g, const float *q, size_t q_len,
                                            size_t q_off, const float *k, size_t k_len,
                                            const float *v, size_t v_len, size_t heads,
                                            size_t kv_heads, size_t head_dim, size_t tk,
                                            size_t cap, float scale, int32_t scale_q,
                                            llmtie_decode_scratch *scratch, float *out,
                                            size_t out_len, size_t out_off)
{
    NEED_HANDLE(g);
    if (head_dim != 64) return unsupported(head_dim, heads, kv_heads);
    if (kv_heads == 0 || heads % kv_heads != 0 || heads / kv_heads > 8) {
        return unsupported(head_dim, heads, kv_heads);
    }
    if (tk == 0 || tk > cap) {
        return llmtie_fail(LLMTIE_ERR_CACHE_OVERRUN,
                           "appending at %zu to a cache with room for %zu", tk, cap);
    }
    if ((cap * 4) % 8 != 0) {
        return llmtie_fail(LLMTIE_ERR_ODD_CACHE_CAPACITY,
                           "an f16 cache with an odd capacity of %zu", cap);
    }
    const size_t need = kv_heads * cap * head_dim;
    if (k_len < need || v_len < need) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu", need,
                           std::min(k_len, v_len));
    }
    const size_t n = heads * head_dim;
    if (q_len < q_off + n) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu",
                           q_off + n, q_len);
    }
    if (out_len < out_off + n) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu",
                           out_off + n, out_len);
    }
    if (out_off % 32 != 0) {
        return llmtie_fail(LLMTIE_ERR_RAGGED_BLOCK,
                           "a row of %zu does not divide into blocks of 32", out_off);
    }
    if (!fits_i32(cap)) return llmtie_fail(LLMTIE_ERR_INVALID, "capacity does not fit 32 bits");
    if (((uintptr_t)k & 15u) != 0) return misaligned("the key cache", k, 16);
    // A partial (o, m, l) per block and a counter per head live in the
    // caller's scratch (sized there in slots of 8 rows of hd + 2 floats);
    // without one the launch is one block a head.
    if (scratch) {
        const size_t splits = (size_t)decode_f32_splits((int)tk);
        const llmtie_status rs =
            scratch_reserve(g, scratch, heads, (heads * splits + 7) / 8, head_dim);
        if (rs != LLMTIE_OK) return rs;
    }
    LaunchScope ls(g, "attn_decode_f64");
    launch_decode_f32(g->stream, q, (long long)q_off, k, v, out, (long long)out_off, (int)heads,
                      (int)kv_heads, (int)head_dim, (int)tk, (int)cap, scale_q ? scale : 1.0f,
                      scale_q ? 1.0f : scale, scratch ? scratch->part : nullptr,
                      scratch ? scratch->ctr : nullptr);
    return ls.done();
}

static llmtie_status decode_batched_impl(llmtie_gpu *g, const float *q, size_t q_len,
                                         const uint16_t *const *k_ptrs,
                                         const uint16_t *const *v_ptrs, const int32_t *tk,
                                         const int32_t *cap, size_t batch, size_t heads,
                                         size_t kv_heads, size_t head_dim, float scale,
                                         int32_t scale_q, llmtie_decode_scratch *scratch,
                                         float *out, size_t out_len, int32_t partial,
                                         const llmtie_exchange *xch,
                                         const FusedMerge *fused = nullptr)
{
    NEED_HANDLE(g);
    if (!scratch) return llmtie_fail(LLMTIE_ERR_INVALID, "null decode scratch");
    if (!k_ptrs || !v_ptrs || !tk || !cap) {
        return llmtie_fail(LLMTIE_ERR_INVALID, "null sequence table");
    }
    if (head_dim != 64 && head_dim != 128) return unsupported(head_dim, heads, kv_heads);
    if (kv_heads == 0 || heads % kv_heads != 0 || heads / kv_heads > 8) {
        return unsupported(head_dim, heads, kv_heads);
    }
    const size_t n = heads * head_dim;
    const size_t on = partial ? heads * (head_dim + 2) : n;
    if (q_len < batch * n) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu",
                           batch * n, q_len);
    }
    if (!xch && out_len < batch * on) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu",
                           batch * on, out_len);
    }
    if (xch) {
        // (a world of one rank is a valid fused exchange: the rank merges its own triple)
        if (xch->world < (fused ? 1 : 2) || xch->world > LLMTIE_MAX_RANKS || xch->rank < 0 ||
            xch->rank >= xch->world || !xch->gather || !xch->step ||
            (fused ? !fused->pair_flags || (fused->mode == 1 && !fused->out) : !xch->flags)) {
            return llmtie_fail(LLMTIE_ERR_INVALID, "a malformed exchange descriptor");
        }
        if (batch > LLMTIE_DECODE_MAX_SEQ) {
            return llmtie_fail(LLMTIE_ERR_INVALID, "the exchanging decode takes at most %d "
                               "sequences a call", LLMTIE_DECODE_MAX_SEQ);
        }
    }
    for (size_t b = 0; b < batch; b++) {
        if (cap[b] <= 0 || cap[b] % 4 != 0) {
            return llmtie_fail(LLMTIE_ERR_ODD_CACHE_CAPACITY,
                               "an f16 cache with an odd capacity of %d", cap[b]);
        }
        if (tk[b] <= 0 || tk[b] > cap[b]) {
            return llmtie_fail(LLMTIE_ERR_CACHE_OVERRUN,
                               "appending at %d to a cache with room for %d", tk[b], cap[b]);
        }
        if (((uintptr_t)k_ptrs[b] & 15u) != 0) return misaligned("a key cache", k_ptrs[b], 16);
        if (((uintptr_t)v_ptrs[b] & 7u) != 0) return misaligned("a value cache", v_ptrs[b], 8);
    }
    const size_t group = heads / kv_heads;
    const size_t ostride = partial ? head_dim + 2 : head_dim;
    for (size_t b0 = 0; b0 < batch; b0 += LLMTIE_DECODE_MAX_SEQ) {
        const size_t nb = std::min<size_t>(LLMTIE_DECODE_MAX_SEQ, batch - b0);
        DecodeParams p;
        memset(&p, 0, sizeof(p));
        p.nseq = (int)nb;
        for (size_t b = 0; b < nb; b++) {
            p.seq[b].k = k_ptrs[b0 + b];
            p.seq[b].v = v_ptrs[b0 + b];
            p.seq[b].tk = tk[b0 + b];
            p.seq[b].cap = cap[b0 + b];
        }
        p.q = q + b0 * n;
        p.q_seq = (long long)n;
        p.q_kv = (long long)(group * head_dim);
        p.q_row = (long long)head_dim;
        p.out = out + b0 * on;
        p.out_seq = (long long)on;
        p.out_kv = (long long)(group * ostride);
        p.out_row = (long long)ostride;
        p.rows = (int)group;
        p.row_chunks = 1;
        p.kv_heads = (int)kv_heads;
        p.partial = partial ? 1 : 0;
        p.q_scale = scale_q ? scale : 1.0f;
        p.sl2 = (scale_q ? 1.0f : scale) * kLog2e;
        const llmtie_status s = decode_launch(
            g, head_dim == 128 ? "attn_decode_h128" : "attn_decode_h64", p, (int)head_dim,
            scratch, xch, fused);
        if (s != LLMTIE_OK) return s;
    }
    return LLMTIE_OK;
}

extern "C" llmtie_status llmtie_decode_batched(llmtie_gpu *g, const float *q, size_t q_len,
                                               const uint16_t *const *k_ptrs,
                                               const uint16_t *const *v_ptrs, const int32_t *tk,
                                               const int32_t *cap, size_t batch, size_t heads,
                                               size_t kv_heads, size_t head_dim, float scale,
                                               int32_t scale_q, llmtie_decode_scratch *scratch,
                                               float *out, size_t out_len, int32_t partial)
{
    return decode_batched_impl(g, q, q_len, k_ptrs, v_ptrs, tk, cap, batch, heads, kv_heads,
                               head_dim, scale, scale_q, scratch, out, out_len, partial, nullptr);
}

extern "C" llmtie_status llmtie_decode_batched_push(
    llmtie_gpu *g, const float *q, size_t q_len, const uint16_t *const *k_ptrs,
    const uint16_t *const *v_ptrs, const int32_t *tk, const int32_t *cap, size_t batch,
    size_t heads, size_t kv_heads, size_t head_dim, float scale, int32_t scale_q,
    llmtie_decode_scratch *scratch, const llmtie_exchange *xch)
{
    if (!xch) return llmtie_fail(LLMTIE_ERR_INVALID, "null exchange descriptor");
    return decode_batched_impl(g, q, q_len, k_ptrs, v_ptrs, tk, cap, batch, heads, kv_heads,
                               head_dim, scale, scale_q, scratch, nullptr, 0, 1, xch);
}

extern "C" llmtie_status llmtie_decode_batched_fused(
    llmtie_gpu *g, const float *q, size_t q_len, const uint16_t *const *k_ptrs,
    const uint16_t *const *v_ptrs, const int32_t *tk, const int32_t *cap, size_t batch,
    size_t heads, size_t kv_heads, size_t head_dim, float scale, int32_t scale_q,
    llmtie_decode_scratch *scratch, const llmtie_exchange *xch, uint32_t *const *pair_flags,
    float *out, size_t out_len)
{
    if (!xch) return llmtie_fail(LLMTIE_ERR_INVALID, "null exchange descriptor");
    if (out_len < batch * heads * head_dim) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu",
                           batch * heads * head_dim, out_len);
    }
    const FusedMerge fused = {pair_flags, out, 1};
    return decode_batched_impl(g, q, q_len, k_ptrs, v_ptrs, tk, cap, batch, heads, kv_heads,
                               head_dim, scale, scale_q, scratch, nullptr, 0, 1, xch, &fused);
}

extern "C" llmtie_status llmtie_decode_batched_signal(
    llmtie_gpu *g, const float *q, size_t q_len, const uint16_t *const *k_ptrs,
    const uint16_t *const *v_ptrs, const int32_t *tk, const int32_t *cap, size_t batch,
    size_t heads, size_t kv_heads, size_t head_dim, float scale, int32_t scale_q,
    llmtie_decode_scratch *scratch, const llmtie_exchange *xch, uint32_t *const *pair_flags)
{
    if (!xch) return llmtie_fail(LLMTIE_ERR_INVALID, "null exchange descriptor");
    if (xch->world < 2) return llmtie_fail(LLMTIE_ERR_INVALID, "a malformed exchange descriptor");
    const FusedMerge fused = {pair_flags, nullptr, 2};
    return decode_batched_impl(g, q, q_len, k_ptrs, v_ptrs, tk, cap, batch, heads, kv_heads,
                               head_dim, scale, scale_q, scratch, nullptr, 0, 1, xch, &fused);
}

extern "C" llmtie_status llmtie_lse_merge_pairs(llmtie_gpu *g, const llmtie_exchange *xch,
                                                const uint32_t *pair_flags, uint32_t *merge_step,
                                                size_t rows, size_t rows_per_pair,
                                                size_t head_dim, float *out, size_t out_len)
{
    NEED_HANDLE(g);
    if (!xch || xch->world < 2 || xch->world > LLMTIE_MAX_RANKS || xch->rank < 0 ||
        xch->rank >= xch->world || !xch->gather || !pair_flags || !merge_step) {
        return llmtie_fail(LLMTIE_ERR_INVALID, "a malformed exchange descriptor");
    }
    if (out_len < rows * head_dim) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu",
                           rows * head_dim, out_len);
    }
    if (head_dim == 0 || head_dim > 1024) return unsupported(head_dim, rows, rows);
    if (rows_per_pair == 0 || rows % rows_per_pair != 0) {
        return llmtie_fail(LLMTIE_ERR_RAGGED_BLOCK, "a row of %zu does not divide into blocks of %zu",
                           rows, rows_per_pair);
    }
    if (rows == 0) return LLMTIE_OK;
    // (LLMTIE_B200_NO_PDL launches it as an ordinary kernel: an A/B switch)
    static const bool plain = getenv("LLMTIE_B200_NO_PDL") != nullptr;
    LaunchScope ls(g, "lse_merge_pairs");
    const cudaError_t e = launch_lse_merge_pairs(
        g->stream, xch->gather[xch->rank], pair_flags, merge_step, xch->world, (int)rows,
        (int)rows_per_pair, (int)head_dim, out, g->timeout_site, g->wait_cycles, !plain && !g->kprof);
    if (e != cudaSuccess) return driver_fail("lse_merge_pairs", e);
    return ls.done();
}

extern "C" llmtie_status llmtie_lse_merge_wait(llmtie_gpu *g, const llmtie_exchange *xch,
                                               size_t rows, size_t head_dim, float *out,
                                               size_t out_len)
{
    NEED_HANDLE(g);
    if (!xch || xch->world < 2 || xch->world > LLMTIE_MAX_RANKS || xch->rank < 0 ||
        xch->rank >= xch->world || !xch->gather || !xch->flags || !xch->step) {
        return llmtie_fail(LLMTIE_ERR_INVALID, "a malformed exchange descriptor");
    }
    if (out_len < rows * head_dim) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu",
                           rows * head_dim, out_len);
    }
    if (head_dim == 0 || head_dim > 1024) return unsupported(head_dim, rows, rows);
    if (rows == 0) return LLMTIE_OK;
    LaunchScope ls(g, "lse_merge_wait");
    launch_lse_merge_wait(g->stream, xch->gather[xch->rank], xch->flags[xch->rank], xch->step,
                          xch->world, (int)rows, (int)head_dim, out, g->timeout_site,
                          g->wait_cycles);
    return ls.done();
}

extern "C" llmtie_status llmtie_lse_merge(llmtie_gpu *g, const float *parts_buf,
                                          size_t parts_len, size_t parts, size_t rows,
                                          size_t head_dim, float *out, size_t out_len)
{
    NEED_HANDLE(g);
    if (parts_len < parts * rows * (head_dim + 2)) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu",
                           parts * rows * (head_dim + 2), parts_len);
    }
    if (out_len < rows * head_dim) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu",
                           rows * head_dim, out_len);
    }
    if (head_dim == 0 || head_dim > 1024) return unsupported(head_dim, rows, rows);
    if (parts == 0 || rows == 0) return LLMTIE_OK;
    LaunchScope ls(g, "lse_merge");
    launch_lse_merge(g->stream, parts_buf, (int)parts, (int)rows, (int)head_dim, out);
    return ls.done();
}

extern "C" llmtie_status llmtie_cross_attn(llmtie_gpu *g, const float *q, size_t q_len,
                                           const uint16_t *k, size_t k_len, const uint16_t *v,
                                           size_t v_len, size_t n, size_t heads, size_t head_dim,
                                           size_t tk, size_t cap, float scale,
                                           llmtie_decode_scratch *scratch, float *out,
                                           size_t out_len)
{
    NEED_HANDLE(g);
    if (!scratch) return llmtie_fail(LLMTIE_ERR_INVALID, "null decode scratch");
    if (head_dim != 64 && head_dim != 128) return unsupported(head_dim, heads, heads);
    if (heads == 0) return unsupported(head_dim, heads, heads);
    if (tk == 0 || tk > cap) {
        return llmtie_fail(LLMTIE_ERR_CACHE_OVERRUN,
                           "appending at %zu to a cache with room for %zu", tk, cap);
    }
    if (cap % 4 != 0) {
        return llmtie_fail(LLMTIE_ERR_ODD_CACHE_CAPACITY,
                           "an f16 cache with an odd capacity of %zu", cap);
    }
    const size_t need = heads * cap * head_dim;
    if (k_len < need || v_len < need) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu", need,
                           std::min(k_len, v_len));
    }
    const size_t d = heads * head_dim;
    if (q_len < n * d || out_len < n * d) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu", n * d,
                           std::min(q_len, out_len));
    }
    if (((uintptr_t)k & 15u) != 0) return misaligned("the key cache", k, 16);
    if (((uintptr_t)v & 7u) != 0) return misaligned("the value cache", v, 8);
    if (!fits_i32(cap) || !fits_i32(n * d)) {
        return llmtie_fail(LLMTIE_ERR_INVALID, "attention geometry does not fit 32 bits");
    }
    if (n == 0) return LLMTIE_OK;
    // The query rows of one head share its keys exactly as a GQA group's
    // heads do, so they ride the decode kernel eight rows a block.
    DecodeParams p;
    memset(&p, 0, sizeof(p));
    p.nseq = 1;
    p.seq[0].k = k;
    p.seq[0].v = v;
    p.seq[0].tk = (int)tk;
    p.seq[0].cap = (int)cap;
    p.q = q;
    p.q_kv = (long long)head_dim;
    p.q_row = (long long)d;
    p.out = out;
    p.out_kv = (long long)head_dim;
    p.out_row = (long long)d;
    p.rows = (int)n;
    p.row_chunks = (int)((n + 7) / 8);
    p.kv_heads = (int)heads;
    p.partial = 0;
    p.q_scale = scale;
    p.sl2 = kLog2e;
    return decode_launch(g, head_dim == 128 ? "cross_attn_h128" : "cross_attn_h64", p,
                         (int)head_dim, scratch);
}

extern "C" llmtie_status llmtie_prefill_varlen(
    llmtie_gpu *g, const float *q, size_t q_len, const float *k, size_t k_len, const float *v,
    size_t v_len, const int32_t *cu_seqlens, size_t batch, uint16_t *const *k_ptrs,
    uint16_t *const *v_ptrs, const int32_t *past, const int32_t *cap, const float *freq_div,
    size_t heads, size_t kv_heads, size_t head_dim, float theta, float scale, float *out,
    size_t out_len)
{
    NEED_HANDLE(g);
    if (!cu_seqlens || !k_ptrs || !v_ptrs || !past || !cap) {
        return llmtie_fail(LLMTIE_ERR_INVALID, "null sequence table");
    }
    if (head_dim != 128) return unsupported(head_dim, heads, kv_heads);
    if (kv_heads == 0 || heads % kv_heads != 0) return unsupported(head_dim, heads, kv_heads);
    if (batch == 0) return LLMTIE_OK;
    const size_t total = (size_t)cu_seqlens[batch];
    if (q_len < total * heads * head_dim || out_len < total * heads * head_dim) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu",
                           total * heads * head_dim, std::min(q_len, out_len));
    }
    if (k_len < total * kv_heads * head_dim || v_len < total * kv_heads * head_dim) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu",
                           total * kv_heads * head_dim, std::min(k_len, v_len));
    }
    if (((uintptr_t)q & 15u) != 0) return misaligned("the query", q, 16);
    if (((uintptr_t)v & 15u) != 0) return misaligned("the value rows", v, 16);
    if (((uintptr_t)out & 7u) != 0) return misaligned("the output", out, 8);
    for (size_t b = 0; b < batch; b++) {
        const int n = cu_seqlens[b + 1] - cu_seqlens[b];
        if (n < 0) return llmtie_fail(LLMTIE_ERR_INVALID, "cu_seqlens is not ascending");
        if (cap[b] % 2 != 0) {
            return llmtie_fail(LLMTIE_ERR_ODD_CACHE_CAPACITY,
                               "an f16 cache with an odd capacity of %d", cap[b]);
        }
        if (past[b] < 0 || past[b] + n > cap[b]) {
            return llmtie_fail(LLMTIE_ERR_CACHE_OVERRUN,
                               "appending at %d to a cache with room for %d", past[b] + n,
                               cap[b]);
        }
        if (((uintptr_t)k_ptrs[b] & 15u) != 0) return misaligned("a key cache", k_ptrs[b], 16);
    }
    for (size_t b0 = 0; b0 < batch; b0 += LLMTIE_PREFILL_MAX_SEQ) {
        const size_t nb = std::min<size_t>(LLMTIE_PREFILL_MAX_SEQ, batch - b0);
        VarlenParams vp;
        PrefillParams pp;
        memset(&vp, 0, sizeof(vp));
        memset(&pp, 0, sizeof(pp));
        const int base = cu_seqlens[b0];
        // (a sequence that brings no new token takes no part: it has no rows,
        // its caches are not touched, and a tensor map of no keys cannot be made)
        int m = 0;
        for (size_t b = 0; b < nb; b++) {
            const int row0 = cu_seqlens[b0 + b] - base;
            const int n = cu_seqlens[b0 + b + 1] - cu_seqlens[b0 + b];
            if (n == 0) continue;
            vp.seq[m] = {k_ptrs[b0 + b], v_ptrs[b0 + b], row0, n, past[b0 + b], cap[b0 + b]};
            pp.seq[m].k = k_ptrs[b0 + b];
            pp.seq[m].v = v_ptrs[b0 + b];
            pp.seq[m].row0 = row0;
            pp.seq[m].tq = n;
            pp.seq[m].past = past[b0 + b];
            pp.seq[m].cap = cap[b0 + b];
            pp.seq[m].tk = past[b0 + b] + n;
            m++;
        }
        vp.nseq = pp.nseq = m;
        vp.total = cu_seqlens[b0 + nb] - base;
        if (vp.total == 0) continue;
        const float *q0 = q + (size_t)base * heads * head_dim;
        vp.k = k + (size_t)base * kv_heads * head_dim;
        vp.v = v + (size_t)base * kv_heads * head_dim;
        vp.freq_div = freq_div;
        vp.heads = (int)heads;
        vp.kv_heads = (int)kv_heads;
        vp.hd = (int)head_dim;
        vp.theta = theta;
        pp.q = q0;
        pp.q_stride = (long long)(heads * head_dim);
        pp.out = out + (size_t)base * heads * head_dim;
        pp.out_stride = (long long)(heads * head_dim);
        pp.heads = (int)heads;
        pp.kv_heads = (int)kv_heads;
        pp.causal = 1;
        pp.q_scale = 1.0f;
        pp.sl2 = scale * kLog2e;
        // The tensor-core kernel carries a tensor map per sequence and so at
        // most LLMTIE_TC_MAX_SEQ of them a launch: a longer batch goes in groups.
        bool all_tc = true;
        for (int s0 = 0; s0 < pp.nseq; s0 += LLMTIE_TC_MAX_SEQ) {
            PrefillParams part = pp;
            part.nseq = std::min(LLMTIE_TC_MAX_SEQ, pp.nseq - s0);
            for (int b = 0; b < part.nseq; b++) part.seq[b] = pp.seq[s0 + b];
            all_tc = all_tc && use_tc(part, (int)head_dim);
        }
        if (getenv("LLMTIE_B200_NO_ROPE_FUSE")) all_tc = false;   // (an A/B switch)
        // Where every group takes the tensor-memory kernel, q is rotated as
        // that kernel stages it, from a table of the rows' cosines and sines
        // that the one-launch pre-pass leaves (it rotates k into the caches
        // and transposes v into them): two launches a group in all. Otherwise
        // a copy of q is rotated by the stand-alone kernel, as the reference's
        // chain does (crates/llmtie-chat/src/model.rs:848-889).
        const size_t work_floats =
            (size_t)vp.total * (all_tc ? head_dim : heads * head_dim);
        cudaError_t werr;
        void *work = workspace_reserve(g->ws_rope, work_floats * sizeof(float), g->stream, &werr);
        if (!work) return driver_fail("allocating", werr);
        llmtie_status st = LLMTIE_OK;
        if (all_tc) {
            vp.rope_tab = (float *)work;
            pp.rope_tab = (const float *)work;
        } else {
            const cudaError_t e = cudaMemcpyAsync(work, q0, work_floats * sizeof(float),
                                                  cudaMemcpyDeviceToDevice, g->stream);
            if (e != cudaSuccess) return driver_fail("copying the query", e);
            vp.q = (float *)work;
            pp.q = (const float *)work;
        }
        {
            LaunchScope ls(g, all_tc ? "varlen_kv" : "varlen_rope_append");
            launch_varlen_rope_append(g->stream, vp);
            if (!all_tc) g->launches++;   // two kernels in that launcher then
            st = ls.done();
        }
        for (int s0 = 0; s0 < pp.nseq && st == LLMTIE_OK; s0 += LLMTIE_TC_MAX_SEQ) {
            PrefillParams part = pp;
            part.nseq = std::min(LLMTIE_TC_MAX_SEQ, pp.nseq - s0);
            for (int b = 0; b < part.nseq; b++) part.seq[b] = pp.seq[s0 + b];
            const bool tc = all_tc || use_tc(part, (int)head_dim);
            // the first attention launch behind the one-launch pre-pass sets itself
            // up under that kernel's tail (LLMTIE_B200_NO_PDL: an A/B switch)
            static const bool no_pdl = getenv("LLMTIE_B200_NO_PDL") != nullptr;
            part.after_prepass = (all_tc && s0 == 0 && !no_pdl && !g->kprof) ? 1 : 0;
            LaunchScope ls(g, tc ? "flash_attn_h_tc" : "flash_attn_h");
            const cudaError_t e =
                tc ? launch_prefill_tc(g->stream, part, (int)head_dim, next_wait_ctl(g))
                   : launch_prefill_mma(g->stream, part, (int)head_dim);
            st = e != cudaSuccess ? driver_fail("flash_attn_h", e) : ls.done();
        }
        if (st != LLMTIE_OK) return st;
    }
    return LLMTIE_OK;
}

// ---- profiling -------------------------------------------------------------------

extern "C" void llmtie_kprof_enable(llmtie_gpu *g, int32_t on)
{
    if (g) g->kprof = on != 0;
}

extern "C" void llmtie_kprof_reset(llmtie_gpu *g)
{
    if (g) g->prof.clear();
}

extern "C" size_t llmtie_kprof_report(llmtie_gpu *g, char *buf, size_t cap)
{
    if (!g) return 0;
    // most expensive first, as the reference's report is (device.rs:1556-1563)
    std::vector<std::pair<std::string, KprofEntry>> rows(g->prof.begin(), g->prof.end());
    std::stable_sort(rows.begin(), rows.end(),
                     [](const auto &x, const auto &y) { return x.second.ms > y.second.ms; });
    std::string s;
    for (const auto &kv : rows) {
        char line[256];
        snprintf(line, sizeof(line), "%s %llu %.6f\n", kv.first.c_str(),
                 (unsigned long long)kv.second.count, kv.second.ms);
        s += line;
    }
    if (buf && cap > 0) {
        const size_t n = std::min(cap - 1, s.size());
        memcpy(buf, s.data(), n);
        buf[n] = 0;
    }
    return s.size() + 1;
}

extern "C" llmtie_status llmtie_kernel_resources(const char *name, int32_t *regs,
                                                 int32_t *local_bytes, int32_t *shared_bytes)
{
    const void *fn = name ? llmtie_kernel_symbol(name) : nullptr;
    if (!fn) {
        return llmtie_fail(LLMTIE_ERR_MISSING_KERNEL, "kernel %s is not in the module",
                           name ? name : "(null)");
    }
    cudaFuncAttributes a;
    const cudaError_t e = cudaFuncGetAttributes(&a, fn);
    if (e != cudaSuccess) return driver_fail("reading kernel attributes", e);
    if (regs) *regs = a.numRegs;
    if (local_bytes) *local_bytes = (int32_t)a.localSizeBytes;
    if (shared_bytes) *shared_bytes = (int32_t)a.sharedSizeBytes;
    return LLMTIE_OK;
}

extern "C" uint64_t llmtie_launch_count(llmtie_gpu *g) { return g ? g->launches : 0; }
