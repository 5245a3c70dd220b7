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

__device__ __forceinline__ void rotate(float a, float b, float cs, float sn, float &lo, float &hi)
{
    rope_rotate(a, b, cs, sn, lo, hi);
}

// The inverse frequency of pair j: f32 throughout, accurate powf.
__device__ __forceinline__ float inv_freq(float theta, int j, int hd, const float *freq_div)
{
    float inv = powf(theta, __fdiv_rn(__fmul_rn(-2.0f, (float)j), (float)hd));
    if (freq_div) inv = __fdiv_rn(inv, freq_div[j]);
    return inv;
}
// The angle of a pair at position pos, and its sine and cosine (accurate).
__device__ __forceinline__ void angle_sincos(float inv, int pos, float &sn, float &cs)
{
    sincosf(__fmul_rn((float)pos, inv), &sn, &cs);
}
// The accurate powf is some hundreds of instructions, far more than anything
// else these kernels do, and depends on the pair alone: a block works the
// inverse frequencies of its pairs out once, into shared memory (every thread
// of the block must call). Pairs past kInvMax are worked out where they are
// needed (no model is that wide).
constexpr int kInvMax = 256;
__device__ __forceinline__ void block_inv_freq(float *inv_s, float theta, int hd,
                                               const float *freq_div)
{
    const int n = min(hd >> 1, kInvMax);
    const int tid = threadIdx.y * blockDim.x + threadIdx.x;
    for (int j = tid; j < n; j += blockDim.x * blockDim.y) inv_s[j] = inv_freq(theta, j, hd, freq_div);
    __syncthreads();
}
__device__ __forceinline__ float inv_of(const float *inv_s, float theta, int j, int hd,
                                        const float *freq_div)
{
    return j < kInvMax ? inv_s[j] : inv_freq(theta, j, hd, freq_div);
}

// RoPE in place over x [t][heads][hd]. The angle of a pair depends on the
// position and on j only, so a thread takes VEC neighbouring pairs of one
// position, works their sines and cosines out once, and walks a chunk of the
// heads with them (blockIdx.y picks the chunk): with VEC = 4 every access is
// a 16-byte one, and the accurate powf / sincosf, which cost more than the
// memory traffic, are shared by the heads of the chunk.
constexpr int kRopeHeadChunk = 8;

template <int VEC>
__global__ void rope_kernel(float *__restrict__ x, long long off,
                            const float *__restrict__ freq_div, int t, int heads, int hd,
                            float theta, int first)
{
    __shared__ float inv_s[kInvMax];
    block_inv_freq(inv_s, theta, hd, freq_div);
    const int half = hd >> 1;
    const int per_pos = half / VEC;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)t * per_pos) return;
    const int pos = (int)(i / per_pos);
    const int j0 = (int)(i % per_pos) * VEC;
    float sn[VEC], cs[VEC];
#pragma unroll
    for (int e = 0; e < VEC; e++) {
        angle_sincos(inv_of(inv_s, theta, j0 + e, hd, freq_div), first + pos, sn[e], cs[e]);
    }
    const int h0 = blockIdx.y * kRopeHeadChunk;
    const int h1 = min(heads, h0 + kRopeHeadChunk);
    float *row = x + (size_t)off + ((size_t)pos * heads + h0) * hd + j0;
    // every load of the chunk is issued before its first store
    float a[kRopeHeadChunk][VEC], b[kRopeHeadChunk][VEC];
#pragma unroll
    for (int h = 0; h < kRopeHeadChunk; h++) {
        if (h0 + h < h1) {
            if constexpr (VEC == 4) {
                const float4 lo = *(const float4 *)(row + (size_t)h * hd);
                const float4 hi = *(const float4 *)(row + (size_t)h * hd + half);
                a[h][0] = lo.x; a[h][1] = lo.y; a[h][2] = lo.z; a[h][3] = lo.w;
                b[h][0] = hi.x; b[h][1] = hi.y; b[h][2] = hi.z; b[h][3] = hi.w;
            } else {
                a[h][0] = row[(size_t)h * hd];
                b[h][0] = row[(size_t)h * hd + half];
            }
        }
    }
#pragma unroll
    for (int h = 0; h < kRopeHeadChunk; h++) {
        if (h0 + h < h1) {
            float lo[VEC], hi[VEC];
#pragma unroll
            for (int e = 0; e < VEC; e++) rotate(a[h][e], b[h][e], cs[e], sn[e], lo[e], hi[e]);
            if constexpr (VEC == 4) {
                *(float4 *)(row + (size_t)h * hd) = make_float4(lo[0], lo[1], lo[2], lo[3]);
                *(float4 *)(row + (size_t)h * hd + half) = make_float4(hi[0], hi[1], hi[2], hi[3]);
            } else {
                row[(size_t)h * hd] = lo[0];
                row[(size_t)h * hd + half] = hi[0];
            }
        }
    }
}

// GPT-J style partial rotary embedding (crates/llmtie-cuda/src/kernels.rs:
// 5598-5613): only the first rot_dim of each dim-wide row turns, element 2j
// pairs with 2j + 1, the frequencies come from a buffer and the sine and
// cosine are the fast intrinsics, as the reference's are. A thread takes one
// pair as one 8-byte access (or two 4-byte ones where the row is not aligned).
__global__ void rope_gptj_kernel(float *__restrict__ x, const float *__restrict__ inv_freq,
                                 int positions, int dim, int rot_dim, int wide)
{
    const int pairs = rot_dim >> 1;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)positions * pairs) return;
    const int pos = (int)(i / pairs), j = (int)(i % pairs);
    const float ang = (float)pos * inv_freq[j];
    const float c = __cosf(ang), s = __sinf(ang);
    float *at = x + (size_t)pos * dim + 2 * j;
    float a, b;
    if (wide) {
        const float2 v = *(const float2 *)at;
        a = v.x;
        b = v.y;
    } else {
        a = at[0];
        b = at[1];
    }
    const float lo = a * c - b * s, hi = b * c + a * s;
    if (wide) {
        *(float2 *)at = make_float2(lo, hi);
    } else {
        at[0] = lo;
        at[1] = hi;
    }
}

// The decode step's RoPE and cache write for a batch of sequences (one is a
// batch of one): sequence blockIdx.y rotates its q row in place, writes its
// rotated k row into its f16 K cache and its v row into its transposed f16 V
// cache, all at its own position. A thread owns pair j of one row of the
// stacked [q heads | k heads]; the thread of a k row also moves the two
// values that sit where its pair does, so no thread range is set aside for
// v. q, k and v may be one allocation (offsets per sequence), so none of the
// three is restrict.
__global__ void rope_cache_batched_kernel(const __grid_constant__ RopeBatchParams p)
{
    __shared__ float inv_s[kInvMax];
    block_inv_freq(inv_s, p.theta, p.hd, p.freq_div);
    const RopeBatchSeq &sq = p.seq[blockIdx.y];
    const int half = p.hd >> 1;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const int row = i / half;           // 0..heads-1: q heads, then the kv heads
    const int j = i - row * half;
    if (row >= p.heads + p.kv_heads) return;
    float sn, cs, lo, hi;
    angle_sincos(inv_of(inv_s, p.theta, j, p.hd, p.freq_div), sq.pos, sn, cs);
    if (row < p.heads) {
        float *x = p.q + sq.q_off + (size_t)row * p.hd + j;
        rotate(x[0], x[half], cs, sn, lo, hi);
        x[0] = lo;
        x[half] = hi;
        return;
    }
    const int h = row - p.heads;
    const float *x = p.k + sq.k_off + (size_t)h * p.hd + j;
    rotate(x[0], x[half], cs, sn, lo, hi);
    uint16_t *kd = sq.kc + ((size_t)h * sq.cap + sq.pos) * p.hd + j;
    kd[0] = f16_bits(lo);
    kd[half] = f16_bits(hi);
    const float *y = p.v + sq.v_off + (size_t)h * p.hd + j;
    uint16_t *vd = sq.vc + ((size_t)h * p.hd + j) * sq.cap + sq.pos;
    vd[0] = f16_bits(y[0]);
    vd[(size_t)half * sq.cap] = f16_bits(y[half]);
}

// src [n][kv_heads*hd] -> K layout [kv][cap][hd]: position ti of head h is a
// run of hd elements on both sides, so a thread moves VEC neighbours of one
// run (16 bytes in, 8 or 16 out when VEC = 4).
template <typename T, int VEC>
__global__ void cache_append_kernel(const float *__restrict__ src, long long src_off,
                                    T *__restrict__ dst, int n, int kv_heads, int hd, int cap,
                                    int past)
{
    const int per_run = hd / VEC;
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)n * kv_heads * per_run) return;
    const int j = (int)(i % per_run) * VEC;
    const int h = (int)((i / per_run) % kv_heads);
    const int ti = (int)(i / ((size_t)per_run * kv_heads));
    const float *in = src + (size_t)src_off + ((size_t)ti * kv_heads + h) * hd + j;
    T *o = dst + ((size_t)h * cap + past + ti) * hd + j;
    if constexpr (VEC == 4) {
        const float4 x = *(const float4 *)in;
        if constexpr (sizeof(T) == 2) {
            uint2 w;
            w.x = (uint32_t)f16_bits(x.x) | ((uint32_t)f16_bits(x.y) << 16);
            w.y = (uint32_t)f16_bits(x.z) | ((uint32_t)f16_bits(x.w) << 16);
            *(uint2 *)o = w;
        } else {
            *(float4 *)o = x;
        }
    } else {
        if constexpr (sizeof(T) == 2) {
            *o = f16_bits(*in);
        } else {
            *o = *in;
        }
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

// Re-strides `rows` runs of `len` elements from a cache of one capacity into
// one of another. blockIdx.y is the run; the threads of a block walk it, 16
// bytes at a time when both runs allow (U = uint4), else element by element.
template <typename U>
__global__ void cache_grow_kernel(const U *__restrict__ src, U *__restrict__ dst, long long len,
                                  long long src_stride, long long dst_stride)
{
    const U *in = src + (long long)blockIdx.y * src_stride;
    U *out = dst + (long long)blockIdx.y * dst_stride;
    for (long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x; j < len;
         j += (long long)gridDim.x * blockDim.x) {
        out[j] = in[j];
    }
}

__global__ void round_f16_kernel(const float *__restrict__ src, uint16_t *__restrict__ dst,
                                 size_t n)
{
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = f16_bits(src[i]);
}

// The live part of a pair of caches as f16 caches of capacity `cap16` (live
// rounded up to eight keys): K [kv][cap][hd] -> [kv][cap16][hd], V
// [kv][hd][cap] -> [kv][hd][cap16], what lies past the live keys zero. f32
// caches are rounded to nearest, as the attention kernels round their
// operands; f16 caches (T = uint16_t: a capacity or an address the copy
// engine's tiles cannot be laid over) are re-strided bit for bit. A thread a
// pair of neighbouring elements of either output.
__device__ __forceinline__ uint32_t as_f16_bits(float x) { return f16_bits(x); }
__device__ __forceinline__ uint32_t as_f16_bits(uint16_t x) { return x; }

template <typename T>
__global__ void caches_to_f16_kernel(const T *__restrict__ k32, const T *__restrict__ v32,
                                     uint32_t *__restrict__ k16, uint32_t *__restrict__ v16,
                                     int kv_heads, int hd, int cap, int cap16, int live)
{
    // (the attention kernel behind this one may set itself up meanwhile)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const long long nk = (long long)kv_heads * cap16 * hd / 2;     // pairs of the key cache
    const long long nv = (long long)kv_heads * hd * cap16 / 2;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nk + nv;
         i += (long long)gridDim.x * blockDim.x) {
        if (i < nk) {
            const long long e = 2 * i;                  // element of [kv][cap16][hd]
            const int d = (int)(e % hd);
            const long long row = e / hd;
            const int r = (int)(row % cap16), h = (int)(row / cap16);
            uint32_t w = 0u;
            if (r < live) {
                const T *src = k32 + ((long long)h * cap + r) * hd + d;
                w = as_f16_bits(src[0]) | (as_f16_bits(src[1]) << 16);
            }
            k16[i] = w;
        } else {
            const long long e = 2 * (i - nk);           // element of [kv][hd][cap16]
            const int c = (int)(e % cap16);
            const long long row = e / cap16;            // h * hd + d
            const T *src = v32 + row * cap + c;
            const uint32_t lo = c < live ? as_f16_bits(src[0]) : 0u;
            const uint32_t hi = c + 1 < live ? as_f16_bits(src[1]) : 0u;
            v16[i - nk] = lo | (hi << 16);
        }
    }
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
    // (the attention kernel behind this one may set itself up meanwhile)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
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


// The Whisper cross-attention caches from the decoder layers' projections of
// the encoder output (crates/llmtie-asr/src/model.rs:891-939): x f32
// [layers][t][d] (+ a bias row [layers][d] or none) -> f16 caches of `cap`
// positions a head, zero past t: keys [layers][heads][cap][hd], or transposed
// values [layers][heads][hd][cap]. blockIdx = (64-channel chunk, 64-frame
// chunk, layer); float4 loads along the channels, 8-byte stores (of four
// channels for keys, of four frames - through a shared tile - for values).
// Needs d % 4 == 0, hd % 4 == 0 and, transposed, cap % 4 == 0.
template <bool T>
__global__ void __launch_bounds__(256)
split_heads_kernel(const float *__restrict__ x, long long x_layer, const float *__restrict__ bias,
                   long long bias_layer, uint16_t *__restrict__ out, long long out_layer, int t,
                   int d, int hd, int cap)
{
    __shared__ float tile[64][65];
    x += (size_t)blockIdx.z * x_layer;
    out += (size_t)blockIdx.z * out_layer;
    if (bias) bias += (size_t)blockIdx.z * bias_layer;
    const int c0 = blockIdx.x * 64, t0 = blockIdx.y * 64;
    const int tid = threadIdx.x;
    const int c4 = tid & 15, f0 = tid >> 4;
    const int c = c0 + 4 * c4;
    float4 bz = make_float4(0.f, 0.f, 0.f, 0.f);
    if (bias && c < d) bz = __ldg((const float4 *)(bias + c));
#pragma unroll
    for (int pass = 0; pass < 4; pass++) {
        const int f = pass * 16 + f0;
        const int ti = t0 + f;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (ti < t && c < d) {
            v = __ldg((const float4 *)(x + (size_t)ti * d + c));
            // the same f32 add the projection's epilogue would have made
            v.x = __fadd_rn(v.x, bz.x);
            v.y = __fadd_rn(v.y, bz.y);
            v.z = __fadd_rn(v.z, bz.z);
            v.w = __fadd_rn(v.w, bz.w);
        }
        if constexpr (!T) {
            if (ti < t && c < d) {
                const int h = c / hd, j = c % hd;
                uint2 o;
                o.x = (uint32_t)f16_bits(v.x) | ((uint32_t)f16_bits(v.y) << 16);
                o.y = (uint32_t)f16_bits(v.z) | ((uint32_t)f16_bits(v.w) << 16);
                *(uint2 *)(out + ((size_t)h * cap + ti) * hd + j) = o;
            }
        } else {
            tile[f][4 * c4 + 0] = v.x;
            tile[f][4 * c4 + 1] = v.y;
            tile[f][4 * c4 + 2] = v.z;
            tile[f][4 * c4 + 3] = v.w;
        }
    }
    if constexpr (T) {
        __syncthreads();
        const int f4 = tid & 15, ch0 = tid >> 4;
#pragma unroll
        for (int pass = 0; pass < 4; pass++) {
            const int ch = pass * 16 + ch0;
            const int cc = c0 + ch, ti = t0 + 4 * f4;
            if (cc >= d || ti >= t) continue;
            uint16_t *dst = out + (size_t)cc * cap + ti;     // cc = h*hd + j
            if (ti + 4 <= t) {
                uint2 o;
                o.x = (uint32_t)f16_bits(tile[4 * f4 + 0][ch]) |
                      ((uint32_t)f16_bits(tile[4 * f4 + 1][ch]) << 16);
                o.y = (uint32_t)f16_bits(tile[4 * f4 + 2][ch]) |
                      ((uint32_t)f16_bits(tile[4 * f4 + 3][ch]) << 16);
                *(uint2 *)dst = o;
            } else {
                for (int e = 0; e < 4 && ti + e < t; e++) dst[e] = f16_bits(tile[4 * f4 + e][ch]);
            }
        }
    }
}

// The same for shapes the wide kernel does not take: one element a thread.
template <bool T, typename O = uint16_t>
__global__ void split_heads_any_kernel(const float *__restrict__ x, long long x_layer,
                                       const float *__restrict__ bias, long long bias_layer,
                                       O *__restrict__ out, long long out_layer, int t, int d,
                                       int hd, int cap)
{
    x += (size_t)blockIdx.y * x_layer;
    out += (size_t)blockIdx.y * out_layer;
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)t * d) return;
    const int ti = (int)(i / d), c = (int)(i % d);
    float v = x[i];
    if (bias) v = __fadd_rn(v, bias[(size_t)blockIdx.y * bias_layer + c]);
    O w;
    if constexpr (sizeof(O) == 2) {
        w = f16_bits(v);
    } else {
        w = v;
    }
    if constexpr (T) {
        out[(size_t)c * cap + ti] = w;
    } else {
        out[((size_t)(c / hd) * cap + ti) * hd + c % hd] = w;
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
    __shared__ float inv_s[kInvMax];
    block_inv_freq(inv_s, p.theta, p.hd, p.freq_div);
    const int half = p.hd >> 1;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)p.total * half) return;
    const int row = (int)(i / half);
    const int j = (int)(i % half);
    const int b = varlen_seq_of(p, row);
    const VarlenSeq &sq = p.seq[b];
    const int ti = row - sq.row0;
    float sn, cs, lo, hi;
    angle_sincos(inv_of(inv_s, p.theta, j, p.hd, p.freq_div), sq.past + ti, sn, cs);
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

// The ragged prefill's pre-pass in one launch, for the attention kernel that
// rotates q itself: blocks [0, rope_blocks) take a (row, pair) each - the
// pair's cosine and sine go to the table, the rotated keys of every kv head
// into the f16 K cache; the blocks after them transpose v into the f16 V
// caches through 64 x 64 tiles (tile = blockIdx - rope_blocks over
// [sequence][position tile][channel tile]). Bits as varlen_rope_kernel's and
// varlen_append_v_kernel's.
__global__ void __launch_bounds__(256)
varlen_kv_kernel(const __grid_constant__ VarlenParams p, int rope_blocks, int ctiles, int ttiles)
{
    // The attention kernel that follows may be launched as this kernel's
    // programmatic dependent: its blocks set themselves up meanwhile and wait
    // for this kernel's end before they read what it writes.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int half = p.hd >> 1;
    if ((int)blockIdx.x < rope_blocks) {
        __shared__ float inv_s[kInvMax];
        block_inv_freq(inv_s, p.theta, p.hd, p.freq_div);
        const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
        if (i >= (long long)p.total * half) return;
        const int row = (int)(i / half);
        const int j = (int)(i % half);
        const VarlenSeq &sq = p.seq[varlen_seq_of(p, row)];
        const int ti = row - sq.row0;
        float sn, cs, lo, hi;
        angle_sincos(inv_of(inv_s, p.theta, j, p.hd, p.freq_div), sq.past + ti, sn, cs);
        p.rope_tab[(size_t)row * p.hd + j] = cs;
        p.rope_tab[(size_t)row * p.hd + half + j] = sn;
        const float *xk = p.k + (size_t)row * p.kv_heads * p.hd + j;
        constexpr int kBatch = 8;
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
        return;
    }
    // values: a tile of 64 positions x 64 channels, float4 loads along the
    // channels, then (where the cache rows allow 8-byte stores) four
    // consecutive positions of a channel a store
    __shared__ float tile[64][65];
    const int tile_i = (int)blockIdx.x - rope_blocks;
    const VarlenSeq &sq = p.seq[tile_i / (ctiles * ttiles)];
    const int t0 = ((tile_i / ctiles) % ttiles) * 64;
    const int c0 = (tile_i % ctiles) * 64;
    if (t0 >= sq.n) return;
    const int d = p.kv_heads * p.hd;            // a multiple of 4 (hd is even, checked: hd % 4)
    const int tid = threadIdx.x;
    const int c4 = tid & 15, f0 = tid >> 4;
#pragma unroll
    for (int pass = 0; pass < 4; pass++) {
        const int f = pass * 16 + f0;
        const int ti = t0 + f, c = c0 + 4 * c4;
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (ti < sq.n && c < d) x = __ldg((const float4 *)(p.v + (size_t)(sq.row0 + ti) * d + c));
        tile[f][4 * c4 + 0] = x.x;
        tile[f][4 * c4 + 1] = x.y;
        tile[f][4 * c4 + 2] = x.z;
        tile[f][4 * c4 + 3] = x.w;
    }
    __syncthreads();
    const bool wide = ((sq.cap | sq.past) & 3) == 0 && (((uintptr_t)sq.v) & 7u) == 0;
    const int f4 = tid & 15, ch0 = tid >> 4;
#pragma unroll
    for (int pass = 0; pass < 4; pass++) {
        const int ch = pass * 16 + ch0;
        const int c = c0 + ch, ti = t0 + 4 * f4;
        if (c >= d || ti >= sq.n) continue;
        uint16_t *dst = sq.v + (size_t)c * sq.cap + sq.past + ti;
        if (wide && ti + 4 <= sq.n) {
            uint2 o;
            o.x = (uint32_t)f16_bits(tile[4 * f4 + 0][ch]) | ((uint32_t)f16_bits(tile[4 * f4 + 1][ch]) << 16);
            o.y = (uint32_t)f16_bits(tile[4 * f4 + 2][ch]) | ((uint32_t)f16_bits(tile[4 * f4 + 3][ch]) << 16);
            *(uint2 *)dst = o;
        } else {
            for (int e = 0; e < 4 && ti + e < sq.n; e++) dst[e] = f16_bits(tile[4 * f4 + e][ch]);
        }
    }
}

inline unsigned flat_blocks(size_t n, int threads)
{
    return (unsigned)((n + threads - 1) / threads);
}

// names as the reference registers its kernels (device.rs:604-733)
const KernelReg reg_rope("rope", (const void *)rope_kernel<4>);
const KernelReg reg_rope_gptj("rope_gptj", (const void *)rope_gptj_kernel);
const KernelReg reg_rope_cache("rope_cache_f16", (const void *)rope_cache_batched_kernel);
const KernelReg reg_append("cache_append_f16", (const void *)cache_append_kernel<uint16_t, 4>);
const KernelReg reg_append_t("cache_append_t_f16", (const void *)cache_append_t_kernel<uint16_t>);
const KernelReg reg_grow("cache_grow_f16", (const void *)cache_grow_kernel<uint4>);
const KernelReg reg_rows_stage("rows_stage", (const void *)rows_stage_kernel);
const KernelReg reg_split("split_heads_f16", (const void *)split_heads_kernel<false>);
const KernelReg reg_split_t("split_heads_t_f16", (const void *)split_heads_kernel<true>);

}  // namespace

void launch_rope(cudaStream_t st, float *x, long long off, const float *freq_div, int t,
                 int heads, int hd, float theta, int first)
{
    const int half = hd / 2;
    if ((size_t)t * heads * half == 0) return;
    const unsigned chunks = (unsigned)((heads + kRopeHeadChunk - 1) / kRopeHeadChunk);
    const bool vec4 = half % 4 == 0 && off % 4 == 0 && ((uintptr_t)x & 15u) == 0;
    if (vec4) {
        const dim3 grid(flat_blocks((size_t)t * (half / 4), 128), chunks);
        rope_kernel<4><<<grid, 128, 0, st>>>(x, off, freq_div, t, heads, hd, theta, first);
    } else {
        const dim3 grid(flat_blocks((size_t)t * half, 128), chunks);
        rope_kernel<1><<<grid, 128, 0, st>>>(x, off, freq_div, t, heads, hd, theta, first);
    }
}

void launch_cache_append(cudaStream_t st, const float *src, long long src_off, void *dst,
                         int n, int kv_heads, int hd, int cap, int past, bool transposed,
                         bool f16)
{
    const size_t total = (size_t)n * kv_heads * hd;
    if (total == 0) return;
    if (!transposed) {
        const bool vec4 = hd % 4 == 0 && src_off % 4 == 0 && ((uintptr_t)src & 15u) == 0 &&
                          ((uintptr_t)dst & 15u) == 0;
        const unsigned blocks = flat_blocks(vec4 ? total / 4 : total, 256);
        if (f16 && vec4) {
            cache_append_kernel<uint16_t, 4><<<blocks, 256, 0, st>>>(
                src, src_off, (uint16_t *)dst, n, kv_heads, hd, cap, past);
        } else if (f16) {
            cache_append_kernel<uint16_t, 1><<<blocks, 256, 0, st>>>(
                src, src_off, (uint16_t *)dst, n, kv_heads, hd, cap, past);
        } else if (vec4) {
            cache_append_kernel<float, 4><<<blocks, 256, 0, st>>>(
                src, src_off, (float *)dst, n, kv_heads, hd, cap, past);
        } else {
            cache_append_kernel<float, 1><<<blocks, 256, 0, st>>>(
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
    if (rows * len == 0) return;
    // 16-byte moves when every run starts and ends on a 16-byte boundary
    const long long per16 = 16 / esize;
    const bool wide = len % per16 == 0 && src_stride % per16 == 0 && dst_stride % per16 == 0 &&
                      ((uintptr_t)src & 15u) == 0 && ((uintptr_t)dst & 15u) == 0;
    const long long n = wide ? len / per16 : len;
    // rows ride blockIdx.y (at most 65535 a launch)
    for (long long r0 = 0; r0 < rows; r0 += 65535) {
        const long long nr = rows - r0 < 65535 ? rows - r0 : 65535;
        const dim3 grid((unsigned)((n + 255) / 256 < 64 ? (n + 255) / 256 : 64), (unsigned)nr);
        const char *s8 = (const char *)src + r0 * src_stride * esize;
        char *d8 = (char *)dst + r0 * dst_stride * esize;
        if (wide) {
            cache_grow_kernel<uint4><<<grid, 256, 0, st>>>((const uint4 *)s8, (uint4 *)d8, n,
                                                          src_stride / per16, dst_stride / per16);
        } else if (esize == 2) {
            cache_grow_kernel<uint16_t><<<grid, 256, 0, st>>>((const uint16_t *)s8, (uint16_t *)d8,
                                                             n, src_stride, dst_stride);
        } else {
            cache_grow_kernel<float><<<grid, 256, 0, st>>>((const float *)s8, (float *)d8, n,
                                                          src_stride, dst_stride);
        }
    }
}

void launch_split_heads(cudaStream_t st, const float *x, long long x_layer, const float *bias,
                        long long bias_layer, uint16_t *out, long long out_layer, int layers, int t,
                        int heads, int hd, int cap, bool transposed)
{
    const int d = heads * hd;
    if ((size_t)layers * t * d == 0) return;
    const bool wide = d % 4 == 0 && hd % 4 == 0 && x_layer % 4 == 0 && out_layer % 4 == 0 &&
                      ((uintptr_t)x & 15u) == 0 && ((uintptr_t)out & 7u) == 0 &&
                      (!bias || (((uintptr_t)bias & 15u) == 0 && bias_layer % 4 == 0)) &&
                      (!transposed || cap % 4 == 0) && layers <= 65535;
    if (wide) {
        const dim3 grid((d + 63) / 64, (t + 63) / 64, layers);
        if (transposed) {
            split_heads_kernel<true><<<grid, 256, 0, st>>>(x, x_layer, bias, bias_layer, out,
                                                          out_layer, t, d, hd, cap);
        } else {
            split_heads_kernel<false><<<grid, 256, 0, st>>>(x, x_layer, bias, bias_layer, out,
                                                           out_layer, t, d, hd, cap);
        }
        return;
    }
    for (int l0 = 0; l0 < layers; l0 += 65535) {
        const int nl = layers - l0 < 65535 ? layers - l0 : 65535;
        const dim3 grid(flat_blocks((size_t)t * d, 256), nl);
        const float *xs = x + (size_t)l0 * x_layer;
        const float *bs = bias ? bias + (size_t)l0 * bias_layer : nullptr;
        uint16_t *os = out + (size_t)l0 * out_layer;
        if (transposed) {
            split_heads_any_kernel<true><<<grid, 256, 0, st>>>(xs, x_layer, bs, bias_layer, os,
                                                              out_layer, t, d, hd, cap);
        } else {
            split_heads_any_kernel<false><<<grid, 256, 0, st>>>(xs, x_layer, bs, bias_layer, os,
                                                               out_layer, t, d, hd, cap);
        }
    }
}

void launch_split_heads_f32(cudaStream_t st, const float *x, float *out, int t, int heads, int hd,
                            int cap, bool transposed)
{
    const int d = heads * hd;
    if ((size_t)t * d == 0) return;
    const dim3 grid(flat_blocks((size_t)t * d, 256), 1);
    if (transposed) {
        split_heads_any_kernel<true, float><<<grid, 256, 0, st>>>(x, 0, nullptr, 0, out, 0, t, d, hd,
                                                                 cap);
    } else {
        split_heads_any_kernel<false, float><<<grid, 256, 0, st>>>(x, 0, nullptr, 0, out, 0, t, d,
                                                                  hd, cap);
    }
}

void launch_rope_gptj(cudaStream_t st, float *x, const float *inv_freq, int positions, int dim,
                      int rot_dim)
{
    const size_t n = (size_t)positions * (rot_dim / 2);
    if (n == 0) return;
    const int wide = dim % 2 == 0 && ((uintptr_t)x & 7u) == 0;
    rope_gptj_kernel<<<flat_blocks(n, 256), 256, 0, st>>>(x, inv_freq, positions, dim, rot_dim,
                                                         wide);
}

void launch_caches_to_f16(cudaStream_t st, const void *k, const void *v, bool src_f32,
                          uint16_t *k16, uint16_t *v16, int kv_heads, int hd, int cap, int cap16,
                          int live)
{
    const size_t pairs = (size_t)kv_heads * cap16 * hd;      // half of each cache, twice
    if (src_f32) {
        caches_to_f16_kernel<float><<<flat_blocks(pairs, 256), 256, 0, st>>>(
            (const float *)k, (const float *)v, (uint32_t *)k16, (uint32_t *)v16, kv_heads, hd, cap,
            cap16, live);
    } else {
        caches_to_f16_kernel<uint16_t><<<flat_blocks(pairs, 256), 256, 0, st>>>(
            (const uint16_t *)k, (const uint16_t *)v, (uint32_t *)k16, (uint32_t *)v16, kv_heads,
            hd, cap, cap16, live);
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
    if (p.rope_tab) {
        int longest = 0;
        for (int b = 0; b < p.nseq; b++) longest = p.seq[b].n > longest ? p.seq[b].n : longest;
        const int rope_blocks = (int)flat_blocks(n, 256);
        const int ctiles = (p.kv_heads * p.hd + 63) / 64, ttiles = (longest + 63) / 64;
        varlen_kv_kernel<<<rope_blocks + ctiles * ttiles * p.nseq, 256, 0, st>>>(p, rope_blocks,
                                                                               ctiles, ttiles);
        return;
    }
    varlen_rope_kernel<<<flat_blocks(n, 128), 128, 0, st>>>(p);
    int max_n = 0;
    for (int b = 0; b < p.nseq; b++) max_n = p.seq[b].n > max_n ? p.seq[b].n : max_n;
    const dim3 grid((p.kv_heads * p.hd + 31) / 32, (max_n + 31) / 32, p.nseq);
    varlen_append_v_kernel<<<grid, dim3(32, 8), 0, st>>>(p);
}

void launch_rope_cache_batched(cudaStream_t st, const RopeBatchParams &p)
{
    const size_t n = (size_t)(p.heads + p.kv_heads) * (p.hd / 2);
    rope_cache_batched_kernel<<<dim3(flat_blocks(n, 128), p.nseq), 128, 0, st>>>(p);
}
