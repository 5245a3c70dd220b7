// RoPE and the KV-cache movers: the element-wise kernels either side of
// attention. Arithmetic follows the reference's kernels exactly where a bit
// could differ: accurate powf / sincosf in f32 for the rotation
// (crates/llmtie-cuda/src/kernels.rs:4915-4959) and round-to-nearest-even
// into the f16 caches (kernels.rs:5287-5317).
#include "common.cuh"

namespace {

__device__ __forceinline__ uint16_t f16_bits(float x)
{
    return __half_as_ushort(__float2half_rn(x));
}

// The rotation of one pair, with the roundings spelled out so that every
// kernel that rotates produces the same bits whatever the compiler would have
// contracted: the fused decode-step and ragged-prefill kernels are held to
// bit equality with rope followed by an append.
__device__ __forceinline__ void rotate(float a, float b, float cs, float sn, float &lo, float &hi)
{
    lo = __fmaf_rn(a, cs, -__fmul_rn(b, sn));
    hi = __fmaf_rn(b, cs, __fmul_rn(a, sn));
}

// The angle of pair j at position pos: f32 throughout, accurate powf.
__device__ __forceinline__ void pair_sincos(float theta, int j, int hd, const float *freq_div,
                                            int pos, float &sn, float &cs)
{
    float inv = powf(theta, __fdiv_rn(__fmul_rn(-2.0f, (float)j), (float)hd));
    if (freq_div) inv = __fdiv_rn(inv, freq_div[j]);
    sincosf(__fmul_rn((float)pos, inv), &sn, &cs);
}

// One thread per rotating pair (j, j + hd/2).
__global__ void rope_kernel(float *__restrict__ x, long long off,
                            const float *__restrict__ freq_div, int t, int heads, int hd,
                            float theta, int first)
{
    const int half = hd >> 1;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)t * heads * half) return;
    const int j = (int)(i % half);
    const int h = (int)((i / half) % heads);
    const int p = (int)(i / ((long long)half * heads));
    float sn, cs;
    pair_sincos(theta, j, hd, freq_div, first + p, sn, cs);
    const size_t base = (size_t)off + ((size_t)p * heads + h) * hd + j;
    float lo, hi;
    rotate(x[base], x[base + half], cs, sn, lo, hi);
    x[base] = lo;
    x[base + half] = hi;
}

// One decoded position: q rotated in place, rotated k and plain v into the
// f16 caches at `pos`. q, k and v may alias one allocation, so no restrict.
__global__ void rope_cache_f16_kernel(float *q, long long q_off, const float *k,
                                      long long k_off, const float *v, long long v_off,
                                      const float *__restrict__ freq_div, int heads,
                                      int kv_heads, int hd, float theta, int pos,
                                      uint16_t *__restrict__ kc, uint16_t *__restrict__ vc,
                                      int cap)
{
    const int half = hd >> 1;
    const int nq = heads * half;
    const int nk = kv_heads * half;
    const int nv = kv_heads * hd;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < nq + nk) {
        const bool is_q = i < nq;
        const int e = is_q ? i : i - nq;
        const int j = e % half;
        const int h = e / half;
        float sn, cs, lo, hi;
        pair_sincos(theta, j, hd, freq_div, pos, sn, cs);
        if (is_q) {
            const size_t base = (size_t)q_off + (size_t)h * hd + j;
            rotate(q[base], q[base + half], cs, sn, lo, hi);
            q[base] = lo;
            q[base + half] = hi;
        } else {
            const size_t base = (size_t)k_off + (size_t)h * hd + j;
            rotate(k[base], k[base + half], cs, sn, lo, hi);
            uint16_t *d = kc + ((size_t)h * cap + pos) * hd;
            d[j] = f16_bits(lo);
            d[j + half] = f16_bits(hi);
        }
    } else if (i < nq + nk + nv) {
        const int e = i - nq - nk;
        const int h = e / hd;
        const int j = e % hd;
        vc[((size_t)h * hd + j) * cap + pos] = f16_bits(v[(size_t)v_off + e]);
    }
}

// rope_cache_f16_kernel for a batch of sequences decoding together: sequence
// blockIdx.y takes row blockIdx.y of q, k and v and its own caches, position
// and capacity. The arithmetic per element is the single-sequence kernel's.
__global__ void rope_cache_batched_kernel(const __grid_constant__ RopeBatchParams p)
{
    const RopeBatchSeq &sq = p.seq[blockIdx.y];
    const int half = p.hd >> 1;
    const int nq = p.heads * half;
    const int nk = p.kv_heads * half;
    const int nv = p.kv_heads * p.hd;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    float *q = p.q + (size_t)blockIdx.y * p.heads * p.hd;
    const float *k = p.k + (size_t)blockIdx.y * p.kv_heads * p.hd;
    const float *v = p.v + (size_t)blockIdx.y * p.kv_heads * p.hd;
    if (i < nq + nk) {
        const bool is_q = i < nq;
        const int e = is_q ? i : i - nq;
        const int j = e % half;
        const int h = e / half;
        float sn, cs, lo, hi;
        pair_sincos(p.theta, j, p.hd, p.freq_div, sq.pos, sn, cs);
        if (is_q) {
            const size_t base = (size_t)h * p.hd + j;
            rotate(q[base], q[base + half], cs, sn, lo, hi);
            q[base] = lo;
            q[base + half] = hi;
        } else {
            const size_t base = (size_t)h * p.hd + j;
            rotate(k[base], k[base + half], cs, sn, lo, hi);
            uint16_t *d = sq.kc + ((size_t)h * sq.cap + sq.pos) * p.hd;
            d[j] = f16_bits(lo);
            d[j + half] = f16_bits(hi);
        }
    } else if (i < nq + nk + nv) {
        const int e = i - nq - nk;
        const int h = e / p.hd;
        const int j = e % p.hd;
        sq.vc[((size_t)h * p.hd + j) * sq.cap + sq.pos] = f16_bits(v[e]);
    }
}

// src [n][kv_heads*hd] -> K layout [kv][cap][hd]. Consecutive threads take
// consecutive source elements, which are consecutive destination elements
// within a head row, so both sides coalesce.
template <typename T>
__global__ void cache_append_kernel(const float *__restrict__ src, long long src_off,
                                    T *__restrict__ dst, int n, int kv_heads, int hd, int cap,
                                    int past)
{
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int d = kv_heads * hd;
    if (i >= (size_t)n * d) return;
    const int ti = (int)(i / d);
    const int h = (int)((i % d) / hd);
    const int j = (int)(i % hd);
    const float x = src[(size_t)src_off + i];
    T *o = dst + ((size_t)h * cap + past + ti) * hd + j;
    if constexpr (sizeof(T) == 2) {
        *o = f16_bits(x);
    } else {
        *o = x;
    }
}

// src [n][kv_heads*hd] -> V layout [kv][hd][cap]: a transpose. A block stages
// 32 positions x 32 channels through shared memory so the reads run along the
// channels and the writes along the positions.
template <typename T>
__global__ void cache_append_t_kernel(const float *__restrict__ src, long long src_off,
                                      T *__restrict__ dst, int n, int kv_heads, int hd,
                                      int cap, int past)
{
    __shared__ float tile[32][33];
    const int d = kv_heads * hd;
    const int c0 = blockIdx.x * 32;   // channel (h*hd + j)
    const int t0 = blockIdx.y * 32;   // position within the step
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        const int ti = t0 + r, c = c0 + threadIdx.x;
        tile[r][threadIdx.x] =
            (ti < n && c < d) ? src[(size_t)src_off + (size_t)ti * d + c] : 0.0f;
    }
    __syncthreads();
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        const int c = c0 + r, ti = t0 + threadIdx.x;
        if (c < d && ti < n) {
            T *o = dst + (size_t)c * cap + past + ti;   // c = h*hd + j
            const float x = tile[threadIdx.x][r];
            if constexpr (sizeof(T) == 2) {
                *o = f16_bits(x);
            } else {
                *o = x;
            }
        }
    }
}

template <typename T>
__global__ void cache_grow_kernel(const T *__restrict__ src, T *__restrict__ dst,
                                  long long rows, long long len, long long src_stride,
                                  long long dst_stride)
{
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * len) return;
    const long long r = i / len;
    const long long j = i % len;
    dst[r * dst_stride + j] = src[r * src_stride + j];
}

__global__ void round_f16_kernel(const float *__restrict__ src, uint16_t *__restrict__ dst,
                                 size_t n)
{
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = f16_bits(src[i]);
}

// Whisper encoder staging (hd 64): the k and v column blocks of qkv f32
// [t][3*heads*64] go to K f16 [heads][tp][64] and V f16 [heads][64][tp], zero
// padded to tp. One block = one head x 64 frames: every global access is a
// whole 128-byte line or more (float4 loads of a frame's 64 channels, 8-byte
// stores of four halves), the value tile is transposed through shared memory.
// blockIdx.z is the utterance: its own [t][3d] product, its own staged K and V.
__global__ void __launch_bounds__(256)
rows_stage_kernel(const float *__restrict__ qkv, uint16_t *__restrict__ k,
                  uint16_t *__restrict__ v, int t, int tp, int heads, int hd)
{
    __shared__ float tile[64][65];
    const int d = heads * hd;
    qkv += (size_t)blockIdx.z * t * 3 * d;
    k += (size_t)blockIdx.z * 2 * heads * tp * hd;
    v += (size_t)blockIdx.z * 2 * heads * tp * hd;
    const int h = blockIdx.x;
    const int t0 = blockIdx.y * 64;
    const size_t row = (size_t)3 * d;
    const int tid = threadIdx.x;
    const int c4 = tid & 15;          // which float4 of the head's 64 channels
    const int f0 = tid >> 4;          // frame within a pass of 16
    // keys: cast and copy; values: into the tile
#pragma unroll
    for (int pass = 0; pass < 4; pass++) {
        const int f = pass * 16 + f0;
        const int ti = t0 + f;
        float4 kx = make_float4(0.f, 0.f, 0.f, 0.f), vx = kx;
        if (ti < t) {
            const float *src = qkv + (size_t)ti * row + (size_t)h * hd + 4 * c4;
            kx = __ldg((const float4 *)(src + d));
            vx = __ldg((const float4 *)(src + 2 * d));
        }
        if (ti < tp) {
            uint2 o;
            o.x = (uint32_t)f16_bits(kx.x) | ((uint32_t)f16_bits(kx.y) << 16);
            o.y = (uint32_t)f16_bits(kx.z) | ((uint32_t)f16_bits(kx.w) << 16);
            *(uint2 *)(k + ((size_t)h * tp + ti) * hd + 4 * c4) = o;
        }
        tile[f][4 * c4 + 0] = vx.x;
        tile[f][4 * c4 + 1] = vx.y;
        tile[f][4 * c4 + 2] = vx.z;
        tile[f][4 * c4 + 3] = vx.w;
    }
    __syncthreads();
    // values, transposed: thread = (channel, four consecutive frames)
    const int f4 = tid & 15;
    const int ch0 = tid >> 4;
#pragma unroll
    for (int pass = 0; pass < 4; pass++) {
        const int ch = pass * 16 + ch0;
        const int ti = t0 + 4 * f4;
        if (ti < tp) {   // tp is a multiple of 128: four frames are in or out together
            uint2 o;
            o.x = (uint32_t)f16_bits(tile[4 * f4 + 0][ch]) |
                  ((uint32_t)f16_bits(tile[4 * f4 + 1][ch]) << 16);
            o.y = (uint32_t)f16_bits(tile[4 * f4 + 2][ch]) |
                  ((uint32_t)f16_bits(tile[4 * f4 + 3][ch]) << 16);
            *(uint2 *)(v + ((size_t)h * hd + ch) * tp + ti) = o;
        }
    }
}


// Packed ragged sequences: which sequence a packed row belongs to.
__device__ __forceinline__ int varlen_seq_of(const VarlenParams &p, int row)
{
    int b = 0;
    while (b + 1 < p.nseq && row >= p.seq[b + 1].row0) b++;
    return b;
}

// RoPE on q (in place) and on k (into the f16 K cache at past + position). One
// thread per (row, rotating pair): the angle depends on the position and the
// pair only, so its accurate powf / sincosf is taken once and reused over every
// head. The arithmetic per element is `rope_kernel`'s followed by the append's
// rounding, so the result equals the two-launch chain bit for bit.
__global__ void varlen_rope_kernel(const __grid_constant__ VarlenParams p)
{
    const int half = p.hd >> 1;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)p.total * half) return;
    const int row = (int)(i / half);
    const int j = (int)(i % half);
    const int b = varlen_seq_of(p, row);
    const VarlenSeq &sq = p.seq[b];
    const int ti = row - sq.row0;
    float sn, cs, lo, hi;
    pair_sincos(p.theta, j, p.hd, p.freq_div, sq.past + ti, sn, cs);
    // Eight heads at a time, every load of a batch issued before its first
    // store: a plain load-rotate-store loop over the heads keeps one access
    // in flight a thread and runs at a third of the memory system's speed.
    constexpr int kBatch = 8;
    float *xq = p.q + (size_t)row * p.heads * p.hd + j;
    for (int h0 = 0; h0 < p.heads; h0 += kBatch) {
        float a[kBatch], b[kBatch];
#pragma unroll
        for (int e = 0; e < kBatch; e++) {
            if (h0 + e < p.heads) {
                a[e] = xq[(size_t)(h0 + e) * p.hd];
                b[e] = xq[(size_t)(h0 + e) * p.hd + half];
            }
        }
#pragma unroll
        for (int e = 0; e < kBatch; e++) {
            if (h0 + e < p.heads) {
                rotate(a[e], b[e], cs, sn, lo, hi);
                xq[(size_t)(h0 + e) * p.hd] = lo;
                xq[(size_t)(h0 + e) * p.hd + half] = hi;
            }
        }
    }
    const float *xk = p.k + (size_t)row * p.kv_heads * p.hd + j;
    for (int h0 = 0; h0 < p.kv_heads; h0 += kBatch) {
        float a[kBatch], b[kBatch];
#pragma unroll
        for (int e = 0; e < kBatch; e++) {
            if (h0 + e < p.kv_heads) {
                a[e] = xk[(size_t)(h0 + e) * p.hd];
                b[e] = xk[(size_t)(h0 + e) * p.hd + half];
            }
        }
#pragma unroll
        for (int e = 0; e < kBatch; e++) {
            if (h0 + e < p.kv_heads) {
                rotate(a[e], b[e], cs, sn, lo, hi);
                uint16_t *d = sq.k + ((size_t)(h0 + e) * sq.cap + sq.past + ti) * p.hd;
                d[j] = f16_bits(lo);
                d[j + half] = f16_bits(hi);
            }
        }
    }
}

// v [n][kv*hd] of each sequence -> its transposed f16 V cache, through a
// 32 x 32 shared tile. grid.z is the sequence.
__global__ void varlen_append_v_kernel(const __grid_constant__ VarlenParams p)
{
    __shared__ float tile[32][33];
    const VarlenSeq &sq = p.seq[blockIdx.z];
    const int d = p.kv_heads * p.hd;
    const int c0 = blockIdx.x * 32;
    const int t0 = blockIdx.y * 32;
    if (t0 >= sq.n) return;
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        const int ti = t0 + r, c = c0 + threadIdx.x;
        tile[r][threadIdx.x] =
            (ti < sq.n && c < d) ? p.v[(size_t)(sq.row0 + ti) * d + c] : 0.0f;
    }
    __syncthreads();
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        const int c = c0 + r, ti = t0 + threadIdx.x;
        if (c < d && ti < sq.n) {
            sq.v[(size_t)c * sq.cap + sq.past + ti] = f16_bits(tile[threadIdx.x][r]);
        }
    }
}

inline unsigned flat_blocks(size_t n, int threads)
{
    return (unsigned)((n + threads - 1) / threads);
}

}  // namespace

void launch_rope(cudaStream_t st, float *x, long long off, const float *freq_div, int t,
                 int heads, int hd, float theta, int first)
{
    const size_t n = (size_t)t * heads * (hd / 2);
    if (n == 0) return;
    rope_kernel<<<flat_blocks(n, 256), 256, 0, st>>>(x, off, freq_div, t, heads, hd, theta,
                                                    first);
}

void launch_rope_cache_f16(cudaStream_t st, float *q, long long q_off, const float *k,
                           long long k_off, const float *v, long long v_off,
                           const float *freq_div, int heads, int kv_heads, int hd,
                           float theta, int pos, uint16_t *kc, uint16_t *vc, int cap)
{
    const size_t n = (size_t)heads * hd / 2 + (size_t)kv_heads * hd / 2 + (size_t)kv_heads * hd;
    rope_cache_f16_kernel<<<flat_blocks(n, 256), 256, 0, st>>>(
        q, q_off, k, k_off, v, v_off, freq_div, heads, kv_heads, hd, theta, pos, kc, vc, cap);
}

void launch_cache_append(cudaStream_t st, const float *src, long long src_off, void *dst,
                         int n, int kv_heads, int hd, int cap, int past, bool transposed,
                         bool f16)
{
    const size_t total = (size_t)n * kv_heads * hd;
    if (total == 0) return;
    if (!transposed) {
        if (f16) {
            cache_append_kernel<uint16_t><<<flat_blocks(total, 256), 256, 0, st>>>(
                src, src_off, (uint16_t *)dst, n, kv_heads, hd, cap, past);
        } else {
            cache_append_kernel<float><<<flat_blocks(total, 256), 256, 0, st>>>(
                src, src_off, (float *)dst, n, kv_heads, hd, cap, past);
        }
    } else {
        const dim3 grid((kv_heads * hd + 31) / 32, (n + 31) / 32);
        const dim3 block(32, 8);
        if (f16) {
            cache_append_t_kernel<uint16_t><<<grid, block, 0, st>>>(
                src, src_off, (uint16_t *)dst, n, kv_heads, hd, cap, past);
        } else {
            cache_append_t_kernel<float><<<grid, block, 0, st>>>(
                src, src_off, (float *)dst, n, kv_heads, hd, cap, past);
        }
    }
}

void launch_cache_grow(cudaStream_t st, const void *src, void *dst, long long rows,
                       long long len, long long src_stride, long long dst_stride, int esize)
{
    const size_t total = (size_t)rows * len;
    if (total == 0) return;
    if (esize == 2) {
        cache_grow_kernel<uint16_t><<<flat_blocks(total, 256), 256, 0, st>>>(
            (const uint16_t *)src, (uint16_t *)dst, rows, len, src_stride, dst_stride);
    } else {
        cache_grow_kernel<float><<<flat_blocks(total, 256), 256, 0, st>>>(
            (const float *)src, (float *)dst, rows, len, src_stride, dst_stride);
    }
}

void launch_round_f16(cudaStream_t st, const float *src, uint16_t *dst, size_t n)
{
    if (n == 0) return;
    round_f16_kernel<<<flat_blocks(n, 256), 256, 0, st>>>(src, dst, n);
}

void launch_rows_stage(cudaStream_t st, const float *qkv, uint16_t *k, uint16_t *v, int t,
                       int tp, int heads, int hd, int batch)
{
    const dim3 grid(heads, (tp + 63) / 64, batch);   // hd is 64: a block is one head x 64 frames
    rows_stage_kernel<<<grid, 256, 0, st>>>(qkv, k, v, t, tp, heads, hd);
}

void launch_varlen_rope_append(cudaStream_t st, const VarlenParams &p)
{
    if (p.total == 0) return;
    const size_t n = (size_t)p.total * (p.hd / 2);
    varlen_rope_kernel<<<flat_blocks(n, 128), 128, 0, st>>>(p);
    int max_n = 0;
    for (int b = 0; b < p.nseq; b++) max_n = p.seq[b].n > max_n ? p.seq[b].n : max_n;
    const dim3 grid((p.kv_heads * p.hd + 31) / 32, (max_n + 31) / 32, p.nseq);
    varlen_append_v_kernel<<<grid, dim3(32, 8), 0, st>>>(p);
}

void launch_rope_cache_batched(cudaStream_t st, const RopeBatchParams &p)
{
    const size_t n = (size_t)p.heads * p.hd / 2 + (size_t)p.kv_heads * p.hd / 2 +
                     (size_t)p.kv_heads * p.hd;
    rope_cache_batched_kernel<<<dim3(flat_blocks(n, 256), p.nseq), 256, 0, st>>>(p);
}
