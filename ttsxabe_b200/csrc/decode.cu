// Single-query (decode) attention off the f16 KV cache, split over the keys.
//
// What the kernel computes is the reference's decode arithmetic
// (crates/llmtie-cuda/src/kernels.rs:5976-6164, :6334-6505): f32 query, f16
// keys and values, scores and probabilities kept at f32 precision, one
// partial (o, m, l) per block of keys and a log-sum-exp merge by the last
// block to arrive (kernels.rs:5779-5903).
//
// How it computes it is built for a bandwidth-bound B200: the kernel is a
// stream of 128-bit loads that land directly in tensor-core fragment
// registers, with no shared-memory staging and no block-wide barrier in the
// key loop. A warp owns 32 consecutive keys at a time and up to eight query
// rows that share them (the query heads of one GQA group). Both products run
// on mma.m16n8k16 with f32 accumulation; f32 precision of the query and of
// the probabilities is kept by splitting each into an f16 head and an f16
// remainder, which ride in the two halves of the 16-row A operand, so the
// split costs no extra instruction:
//
//   rows 0..7  of A : hi(x) = f16(x)          rows 8..15 : lo(x) = f16(x - hi(x))
//   C rows r and r+8 summed in the same thread = x . k to ~2^-22.
//
// The cache layouts make both B operands K-major as they lie in memory: a
// key row [hd] for q.K^T and a value row of the transposed cache [cap] for
// P.V. The contraction index of an MMA is a dummy, so it is permuted to let
// each thread fetch 16 contiguous bytes per fragment pair:
//
//   q.K^T: thread (g = lane/4, c = lane%4) loads 8 halves of key n(g) at
//          hd offset 32 i + 8 c and feeds them to two MMAs; the query
//          fragment is built once with the same permutation.
//   P.V  : the same thread loads 8 consecutive keys 8 c .. 8 c + 7 of value
//          row d = 8 j + g; score tile (mm, h) is given the keys
//          8 (n/2) + 4 mm + 2 h + n%2 so that its accumulator registers are
//          exactly the A fragment the value product wants.
#include "common.cuh"

#include <string.h>

#include <math_constants.h>

namespace {

__device__ __forceinline__ void ldg128(uint32_t (&r)[4], const void *p)
{
    asm("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
        : "l"(p));
}

__device__ __forceinline__ void ldg64(uint32_t &r0, uint32_t &r1, const void *p)
{
    asm("ld.global.nc.L1::no_allocate.v2.u32 {%0, %1}, [%2];" : "=r"(r0), "=r"(r1) : "l"(p));
}

// A load that bypasses L1 (the partials were written by other blocks). Not
// volatile on purpose: the merge issues many of these and they must be free
// to overlap; the fence and barrier before the merge keep them in place.
__device__ __forceinline__ float ldcg(const float *p) { return __ldcg(p); }

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
        "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float ex2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// f16 head and f16 remainder of a pair of floats, packed low half first.
__device__ __forceinline__ void split_pair(float x0, float x1, uint32_t &hi, uint32_t &lo)
{
    const __half h0 = __float2half_rn(x0), h1 = __float2half_rn(x1);
    const __half l0 = __float2half_rn(x0 - __half2float(h0));
    const __half l1 = __float2half_rn(x1 - __half2float(h1));
    hi = (uint32_t)__half_as_ushort(h0) | ((uint32_t)__half_as_ushort(h1) << 16);
    lo = (uint32_t)__half_as_ushort(l0) | ((uint32_t)__half_as_ushort(l1) << 16);
}

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kRows = 8;   // query rows a block carries

template <int HD, bool V16, int NB>
__global__ void __launch_bounds__(kThreads, NB == 1 ? 3 : 2)
decode_f16_kernel(const __grid_constant__ DecodeParams p)
{
    constexpr int KI = HD / 32;
    constexpr int NT = HD / 8;
    constexpr float kLn2 = 0.6931471805599453f;

    __shared__ float sm_o[kWarps][kRows][HD];
    __shared__ float sm_m[kWarps][kRows];
    __shared__ float sm_l[kWarps][kRows];
    __shared__ float sm_M[kRows];
    __shared__ int sm_last;

    const int split = blockIdx.x;
    const int kh = blockIdx.y;
    const int b = blockIdx.z / p.row_chunks;
    const int rc = blockIdx.z % p.row_chunks;
    const uint16_t *kbase = p.seq[b].k;
    const uint16_t *vbase = p.seq[b].v;
    const int tk = p.seq[b].tk;
    const int cap = p.seq[b].cap;
    const int nsplit = (tk + p.span - 1) / p.span;
    if (split >= nsplit) return;
    const int k_begin = split * p.span;
    const int k_end = min(tk, k_begin + p.span);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int g = lane >> 2;
    const int c = lane & 3;
    const int rows_here = min(kRows, p.rows - rc * kRows);

    // The query fragments, permuted as the key loads are, split hi / lo.
    uint32_t qa[KI][2][4];
    {
        const float *qrow = p.q + (long long)b * p.q_seq + (long long)kh * p.q_kv +
                            (long long)(rc * kRows + g) * p.q_row;
        const bool live = g < rows_here;
#pragma unroll
        for (int i = 0; i < KI; i++) {
#pragma unroll
            for (int u = 0; u < 2; u++) {
                const int at = 32 * i + 8 * c + 4 * u;
                float x[4];
#pragma unroll
                for (int e = 0; e < 4; e++) x[e] = live ? qrow[at + e] * p.q_scale : 0.0f;
                split_pair(x[0], x[1], qa[i][u][0], qa[i][u][1]);
                split_pair(x[2], x[3], qa[i][u][2], qa[i][u][3]);
            }
        }
    }

    float m = -CUDART_INF_F;   // running maximum, in log2 units
    float l = 0.0f;            // this thread's share of the running sum
    float o[NT][4];
#pragma unroll
    for (int j = 0; j < NT; j++) {
        o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;
    }

    // A warp takes 32 * NB consecutive keys a step. The scores of all of them
    // are taken first, so that the value rows - one DRAM page each in the
    // transposed cache - are then read 64 * NB contiguous bytes at a time.
    for (int blk = k_begin + warp * 32 * NB; blk < k_end; blk += kWarps * 32 * NB) {
        // ---- scores: NB sub-blocks of four 8-key tiles ----------------------
        float t[NB][2][2][2];
#pragma unroll
        for (int sb = 0; sb < NB; sb++) {
#pragma unroll
            for (int mm = 0; mm < 2; mm++) {
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const int key = blk + 32 * sb + 8 * (g >> 1) + 4 * mm + 2 * h + (g & 1);
                    const uint16_t *krow = kbase + ((size_t)kh * cap + key) * HD + 8 * c;
                    const bool live = key < k_end;
                    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                    for (int i = 0; i < KI; i++) {
                        uint32_t r[4] = {0u, 0u, 0u, 0u};
                        if (live) ldg128(r, krow + 32 * i);
                        mma16816(acc, qa[i][0][0], qa[i][0][1], qa[i][0][2], qa[i][0][3], r[0],
                                 r[1]);
                        mma16816(acc, qa[i][1][0], qa[i][1][1], qa[i][1][2], qa[i][1][3], r[2],
                                 r[3]);
                    }
                    // this thread's two columns: keys blk + 32sb + 8c + 4mm + 2h + {0, 1}
                    const int k0 = blk + 32 * sb + 8 * c + 4 * mm + 2 * h;
                    t[sb][mm][h][0] = (k0 < k_end) ? (acc[0] + acc[2]) * p.sl2 : -CUDART_INF_F;
                    t[sb][mm][h][1] =
                        (k0 + 1 < k_end) ? (acc[1] + acc[3]) * p.sl2 : -CUDART_INF_F;
                }
            }
        }

        // ---- online softmax over the step ------------------------------------
        float bm = -CUDART_INF_F;
#pragma unroll
        for (int sb = 0; sb < NB; sb++) {
#pragma unroll
            for (int mm = 0; mm < 2; mm++) {
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    bm = fmaxf(bm, fmaxf(t[sb][mm][h][0], t[sb][mm][h][1]));
                }
            }
        }
        bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 1));
        bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 2));
        const float m_new = fmaxf(m, bm);
        if (__any_sync(0xffffffffu, m_new > m)) {
            const float alpha = ex2(m - m_new);   // 0 on the first step
            l *= alpha;
#pragma unroll
            for (int j = 0; j < NT; j++) {
                o[j][0] *= alpha;
                o[j][1] *= alpha;
                o[j][2] *= alpha;
                o[j][3] *= alpha;
            }
        }
        m = m_new;
        uint32_t pa[NB][2][4];
#pragma unroll
        for (int sb = 0; sb < NB; sb++) {
#pragma unroll
            for (int mm = 0; mm < 2; mm++) {
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const float p0 = ex2(t[sb][mm][h][0] - m);
                    const float p1 = ex2(t[sb][mm][h][1] - m);
                    l += p0 + p1;
                    split_pair(p0, p1, pa[sb][mm][2 * h], pa[sb][mm][2 * h + 1]);
                }
            }
        }

        // ---- context: HD/8 tiles of 8 value rows, NB loads along each row ------
#pragma unroll
        for (int j = 0; j < NT; j++) {
            const uint16_t *vrow = vbase + ((size_t)kh * HD + 8 * j + g) * cap + blk + 8 * c;
            uint32_t r[NB][4];
#pragma unroll
            for (int sb = 0; sb < NB; sb++) {
                const int nlive = k_end - (blk + 32 * sb + 8 * c);   // keys of its eight that exist
                r[sb][0] = r[sb][1] = r[sb][2] = r[sb][3] = 0u;
                if (V16) {
                    if (nlive > 0) ldg128(r[sb], vrow + 32 * sb);
                } else {
                    if (nlive > 0) ldg64(r[sb][0], r[sb][1], vrow + 32 * sb);
                    if (nlive > 4) ldg64(r[sb][2], r[sb][3], vrow + 32 * sb + 4);
                }
                if (nlive < 8) {
                    // Capacity past the live keys may hold anything, and 0 * NaN
                    // is NaN: clear what lies beyond.
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        if (nlive <= 2 * i) {
                            r[sb][i] = 0u;
                        } else if (nlive == 2 * i + 1) {
                            r[sb][i] &= 0x0000ffffu;
                        }
                    }
                }
            }
#pragma unroll
            for (int sb = 0; sb < NB; sb++) {
                mma16816(o[j], pa[sb][0][0], pa[sb][0][1], pa[sb][0][2], pa[sb][0][3], r[sb][0],
                         r[sb][1]);
                mma16816(o[j], pa[sb][1][0], pa[sb][1][1], pa[sb][1][2], pa[sb][1][3], r[sb][2],
                         r[sb][3]);
            }
        }
    }

    // ---- the block's four warps merge through shared memory -----------------
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    if (c == 0) {
        sm_m[warp][g] = m;
        sm_l[warp][g] = l;
    }
#pragma unroll
    for (int j = 0; j < NT; j++) {
        sm_o[warp][g][8 * j + 2 * c] = o[j][0] + o[j][2];
        sm_o[warp][g][8 * j + 2 * c + 1] = o[j][1] + o[j][3];
    }
    __syncthreads();

    const int pair = (b * p.row_chunks + rc) * p.kv_heads + kh;
    float *part = p.part + ((size_t)pair * p.max_splits + split) * kRows * (HD + 2);
    float *orow0 = p.out + (long long)b * p.out_seq + (long long)kh * p.out_kv +
                   (long long)(rc * kRows) * p.out_row;
    for (int idx = tid; idx < rows_here * HD; idx += kThreads) {
        const int row = idx / HD, d = idx % HD;
        float M = sm_m[0][row];
#pragma unroll
        for (int w = 1; w < kWarps; w++) M = fmaxf(M, sm_m[w][row]);
        float O = 0.0f, L = 0.0f;
#pragma unroll
        for (int w = 0; w < kWarps; w++) {
            const float mw = sm_m[w][row];
            const float f = (mw == -CUDART_INF_F) ? 0.0f : ex2(mw - M);
            O += f * sm_o[w][row][d];
            L += f * sm_l[w][row];
        }
        if (nsplit == 1) {
            float *orow = orow0 + (long long)row * p.out_row;
            if (p.partial) {
                orow[d] = O;
                if (d == 0) {
                    orow[HD] = M * kLn2;
                    orow[HD + 1] = L;
                }
            } else {
                const float y = L > 0.0f ? O / L : 0.0f;
                orow[d] = y;
                if (p.twin_q) emit_twin(p.twin_q, p.twin_s, (orow - p.out) + d, y);
            }
        } else {
            float *pr = part + row * (HD + 2);
            pr[d] = O;
            if (d == 0) {
                pr[HD] = M;
                pr[HD + 1] = L;
            }
        }
    }
    if (nsplit == 1) return;

    // ---- the last block of this head to arrive merges every partial ---------
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned prev = atomicAdd(p.ctr + pair, 1u);
        sm_last = (prev == (unsigned)(nsplit - 1));
    }
    __syncthreads();
    if (!sm_last) return;
    __threadfence();
    const float *all = p.part + (size_t)pair * p.max_splits * kRows * (HD + 2);
    if (tid < rows_here) {
        float M = -CUDART_INF_F;
        for (int i = 0; i < nsplit; i++) {
            M = fmaxf(M, ldcg(all + ((size_t)i * kRows + tid) * (HD + 2) + HD));
        }
        sm_M[tid] = M;
    }
    __syncthreads();
    for (int idx = tid; idx < rows_here * HD; idx += kThreads) {
        const int row = idx / HD, d = idx % HD;
        const float M = sm_M[row];
        float O = 0.0f, L = 0.0f;
        for (int i = 0; i < nsplit; i++) {
            const float *pr = all + ((size_t)i * kRows + row) * (HD + 2);
            const float mi = ldcg(pr + HD);
            const float f = (mi == -CUDART_INF_F) ? 0.0f : ex2(mi - M);
            O += f * ldcg(pr + d);
            L += f * ldcg(pr + HD + 1);
        }
        float *orow = orow0 + (long long)row * p.out_row;
        if (p.partial) {
            orow[d] = O;
            if (d == 0) {
                orow[HD] = M * kLn2;
                orow[HD + 1] = L;
            }
        } else {
            const float y = L > 0.0f ? O / L : 0.0f;
            orow[d] = y;
            if (p.twin_q) emit_twin(p.twin_q, p.twin_s, (orow - p.out) + d, y);
        }
    }
    if (tid == 0) p.ctr[pair] = 0u;   // at rest again for the next call
}

// Decode off an f32 cache (the Whisper decoder's self-attention: 64-wide
// heads, at most a few hundred keys), plain f32 FMA as the reference's
// `attn_decode_f64` entry keeps it. Every head's keys are cut over
// `gridDim.y` blocks: one block a head would be twenty blocks on 148 SMs,
// each walking its few hundred keys alone. A block takes `span` keys in
// chunks of 64: four lanes a key for the scores (a warp reads eight whole key
// rows, 2 KB on end), a thread a channel and a quarter of the chunk's keys
// for the context. It leaves an un-normalised (o, m, l) in `part`; the last
// block of a head to arrive (`ctr`, which it leaves at zero) merges them.
template <int HD>
__global__ void __launch_bounds__(256)
decode_f32_split_kernel(const float *__restrict__ q, long long q_off, const float *__restrict__ k,
                        const float *__restrict__ v, float *__restrict__ out, long long out_off,
                        int group, int tk, int cap, float q_scale, float s_scale, int span,
                        float *__restrict__ part, unsigned *__restrict__ ctr)
{
    constexpr int CH = 64;               // keys of a chunk
    constexpr int QW = HD / 4;           // channels a lane of a key's four takes
    __shared__ float sq[HD];
    __shared__ float sp[CH];
    __shared__ float red[8];
    __shared__ float so[4][HD];
    __shared__ int s_last;
    const int head = blockIdx.x;
    const int kh = head / group;
    const int tid = threadIdx.x;
    const int k0 = blockIdx.y * span, k1 = min(tk, k0 + span);
    if (tid < HD) sq[tid] = q[q_off + (long long)head * HD + tid] * q_scale;
    __syncthreads();
    const int d = tid % HD, quarter = tid / HD;     // context: channel, and keys quarter, +4, ...
    const int ki = tid >> 2, kq = tid & 3;          // scores: key of the chunk, which 16 channels
    float m = -CUDART_INF_F, l = 0.0f, acc = 0.0f;
    for (int c0 = k0; c0 < k1; c0 += CH) {
        const int key = c0 + ki;
        float dot = 0.0f;
        if (key < k1) {
            const float4 *kr = (const float4 *)(k + ((size_t)kh * cap + key) * HD + kq * QW);
#pragma unroll
            for (int e = 0; e < QW / 4; e++) {
                const float4 x = __ldg(kr + e);
                const float *qs = sq + kq * QW + 4 * e;
                dot += qs[0] * x.x;
                dot += qs[1] * x.y;
                dot += qs[2] * x.z;
                dot += qs[3] * x.w;
            }
        }
        dot += __shfl_xor_sync(0xffffffffu, dot, 1);
        dot += __shfl_xor_sync(0xffffffffu, dot, 2);
        const float sc = key < k1 ? dot * s_scale : -CUDART_INF_F;
        float bm = sc;
        for (int w = 16; w > 0; w >>= 1) bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, w));
        if ((tid & 31) == 0) red[tid >> 5] = bm;
        __syncthreads();
        bm = red[0];
        for (int w = 1; w < 8; w++) bm = fmaxf(bm, red[w]);
        const float m_new = fmaxf(m, bm);
        const float alpha = (m == -CUDART_INF_F) ? 0.0f : __expf(m - m_new);
        const float pv = (key < k1) ? __expf(sc - m_new) : 0.0f;
        if (kq == 0) sp[ki] = pv;
        float bs = kq == 0 ? pv : 0.0f;
        __syncthreads();                 // red was read; sp is written
        for (int w = 16; w > 0; w >>= 1) bs += __shfl_xor_sync(0xffffffffu, bs, w);
        if ((tid & 31) == 0) red[tid >> 5] = bs;
        __syncthreads();
        bs = 0.0f;
        for (int w = 0; w < 8; w++) bs += red[w];
        l = l * alpha + bs;
        m = m_new;
        acc *= alpha;
        // (all of the chunk's loads of a thread in flight at once; past the
        // slice's last key the probability is zero and nothing is read)
        const int n = min(CH, k1 - c0);
        const float *vr = v + ((size_t)kh * HD + d) * cap + c0;
        float x[CH * HD / 256];
#pragma unroll
        for (int i = 0; i < CH * HD / 256; i++) {
            const int e = quarter + i * (256 / HD);
            x[i] = e < n ? __ldg(vr + e) : 0.0f;
        }
#pragma unroll
        for (int i = 0; i < CH * HD / 256; i++) acc += sp[quarter + i * (256 / HD)] * x[i];
        __syncthreads();
    }
    so[quarter][d] = acc;
    __syncthreads();
    const int S = gridDim.y;
    float a = 0.0f;
    if (tid < HD) {
#pragma unroll
        for (int w = 0; w < 256 / HD; w++) a += so[w][tid];
    }
    if (S == 1) {
        if (tid < HD) out[out_off + (long long)head * HD + tid] = l > 0.0f ? a / l : 0.0f;
        return;
    }
    float *mine = part + ((size_t)head * S + blockIdx.y) * (HD + 2);
    if (tid < HD) mine[tid] = a;
    if (tid == 0) {
        mine[HD] = m;
        mine[HD + 1] = l;
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = atomicAdd(ctr + head, 1u) == (unsigned)(S - 1);
    __syncthreads();
    if (!s_last) return;
    if (tid < HD) {
        const float *all = part + (size_t)head * S * (HD + 2);
        float M = -CUDART_INF_F;
        for (int i = 0; i < S; i++) M = fmaxf(M, __ldcg(all + (size_t)i * (HD + 2) + HD));
        float O = 0.0f, L = 0.0f;
        for (int i = 0; i < S; i++) {
            const float *pr = all + (size_t)i * (HD + 2);
            const float mi = __ldcg(pr + HD);
            const float f = (mi == -CUDART_INF_F) ? 0.0f : __expf(mi - M);
            O += f * __ldcg(pr + tid);
            L += f * __ldcg(pr + HD + 1);
        }
        out[out_off + (long long)head * HD + tid] = L > 0.0f ? O / L : 0.0f;
    }
    if (tid == 0) ctr[head] = 0u;        // at rest again for the next call
}

// out[row] = sum_i o_i exp(m_i - M) / sum_i l_i exp(m_i - M) over `parts`
// triples laid out [parts][rows][hd + 2].
__global__ void lse_merge_kernel(const float *__restrict__ buf, int parts, int rows, int hd,
                                 float *__restrict__ out)
{
    const int row = blockIdx.x;
    const int stride = hd + 2;
    float M = -CUDART_INF_F;
    for (int i = 0; i < parts; i++) {
        M = fmaxf(M, buf[((size_t)i * rows + row) * stride + hd]);
    }
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float O = 0.0f, L = 0.0f;
        for (int i = 0; i < parts; i++) {
            const float *pr = buf + ((size_t)i * rows + row) * stride;
            const float mi = pr[hd];
            const float f = (mi == -CUDART_INF_F) ? 0.0f : __expf(mi - M);
            O += f * pr[d];
            L += f * pr[hd + 1];
        }
        out[(size_t)row * hd + d] = L > 0.0f ? O / L : 0.0f;
    }
}

const KernelReg reg_d128("attn_decode_h128", (const void *)decode_f16_kernel<128, true, 1>);
const KernelReg reg_d128w("attn_decode_h128_wide", (const void *)decode_f16_kernel<128, true, 4>);
const KernelReg reg_d128u("attn_decode_h128_unaligned",
                          (const void *)decode_f16_kernel<128, false, 1>);
const KernelReg reg_d64("attn_decode_h64", (const void *)decode_f16_kernel<64, true, 1>);
const KernelReg reg_d64w("attn_decode_h64_wide", (const void *)decode_f16_kernel<64, true, 4>);
const KernelReg reg_d64u("attn_decode_h64_unaligned",
                         (const void *)decode_f16_kernel<64, false, 1>);
const KernelReg reg_df32("attn_decode_f64", (const void *)decode_f32_split_kernel<64>);
const KernelReg reg_merge("lse_merge", (const void *)lse_merge_kernel);

template <int HD, bool V16, int NB>
cudaError_t launch_one(cudaStream_t st, const DecodeParams &p)
{
    const dim3 grid(p.max_splits, p.kv_heads, p.nseq * p.row_chunks);
    decode_f16_kernel<HD, V16, NB><<<grid, kThreads, 0, st>>>(p);
    return cudaGetLastError();
}

template <int HD>
cudaError_t launch_hd(cudaStream_t st, const DecodeParams &p, bool v16)
{
    if (!v16) return launch_one<HD, false, 1>(st, p);
    switch (p.nb) {
    case 8: return launch_one<HD, true, 8>(st, p);
    case 4: return launch_one<HD, true, 4>(st, p);
    case 2: return launch_one<HD, true, 2>(st, p);
    default: return launch_one<HD, true, 1>(st, p);
    }
}

template <int HD>
int resident(int nb)
{
    int per_sm = 0;
    cudaError_t e;
    switch (nb) {
    case 8: e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(
                &per_sm, decode_f16_kernel<HD, true, 8>, kThreads, 0); break;
    case 4: e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(
                &per_sm, decode_f16_kernel<HD, true, 4>, kThreads, 0); break;
    case 2: e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(
                &per_sm, decode_f16_kernel<HD, true, 2>, kThreads, 0); break;
    default: e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(
                 &per_sm, decode_f16_kernel<HD, true, 1>, kThreads, 0); break;
    }
    if (e != cudaSuccess || per_sm < 1) per_sm = 1;
    return per_sm;
}

// The same merge over the gather buffer that the ranks' decode kernels
// filled directly (peer stores over NVLink). Thread 0 of each block first
// waits, bounded, until every rank's flag has reached this rank's step: a
// flag is raised only after all of that rank's triples are visible
// system-wide. Layout: gather [2][world][rows][hd + 2], flags [world].
__global__ void lse_merge_wait_kernel(const float *__restrict__ gather,
                                      const unsigned *flags, const unsigned *step, int world,
                                      int rows, int hd, float *__restrict__ out, int *status,
                                      long long wait_cycles)
{
    __shared__ unsigned s_expected;
    __shared__ int s_ok;
    if (threadIdx.x == 0) {
        const unsigned expected = *(volatile const unsigned *)step;
        const long long t0 = clock64();
        int ok = 1;
        // The flags are raised by other GPUs after a system-wide fence: the
        // consumer's half of that is an acquire at system scope.
        for (int r = 0; r < world && ok; r++) {
            while ((int)(ld_acquire_sys(flags + r) - expected) < 0) {
                if (clock64() - t0 > wait_cycles) {
                    ok = 0;
                    report_timeout(status, 60 + r);
                    break;
                }
            }
        }
        s_expected = expected;
        s_ok = ok;
    }
    __syncthreads();
    if (!s_ok) return;
    const int row = blockIdx.x;
    const int stride = hd + 2;
    const float *buf = gather + (size_t)((s_expected - 1u) & 1u) * world * rows * stride;
    // every rank's (m, l) and this thread's channel of o in flight at once:
    // the kernel is one trip to L2, not one per pass
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float mi[LLMTIE_MAX_RANKS], li[LLMTIE_MAX_RANKS], oi[LLMTIE_MAX_RANKS];
#pragma unroll
        for (int i = 0; i < LLMTIE_MAX_RANKS; i++) {
            const float *pr = buf + ((size_t)min(i, world - 1) * rows + row) * stride;
            mi[i] = __ldcg(pr + hd);
            li[i] = __ldcg(pr + hd + 1);
            oi[i] = __ldcg(pr + d);
        }
        float M = -CUDART_INF_F;
#pragma unroll
        for (int i = 0; i < LLMTIE_MAX_RANKS; i++) M = fmaxf(M, mi[i]);   // repeats are harmless
        float O = 0.0f, L = 0.0f;
#pragma unroll
        for (int i = 0; i < LLMTIE_MAX_RANKS; i++) {
            if (i < world) {
                const float f = (mi[i] == -CUDART_INF_F) ? 0.0f : __expf(mi[i] - M);
                O += f * oi[i];
                L += f * li[i];
            }
        }
        out[(size_t)row * hd + d] = L > 0.0f ? O / L : 0.0f;
    }
}

const KernelReg reg_merge_wait("lse_merge_wait", (const void *)lse_merge_wait_kernel);

// The merge of a step whose decode kernels raise a flag per (sequence, KV head)
// pair and source rank. Launched as a programmatic dependent of this rank's
// decode kernel, so its blocks are resident and polling while that kernel
// still streams: a row is merged as soon as every rank's triple of its pair
// has landed, and neither this kernel's launch nor the exchange of any pair
// but the last lies on the step's critical path. It never waits for the
// decode kernel as a whole, only for flags (bounded), and counts its own
// steps: mstep[0] is the step it is about to merge, advanced by the last
// block to finish (mstep[1] counts the blocks out). Layout: gather
// [2][world][rows][hd + 2], pflags [rows / rows_per_pair][world].
__global__ void lse_merge_pairs_kernel(const float *__restrict__ gather, const unsigned *pflags,
                                       unsigned *mstep, int world, int rows, int rows_per_pair,
                                       int hd, float *__restrict__ out, int *status,
                                       long long wait_cycles)
{
    __shared__ int s_ok;
    const unsigned step = *(volatile const unsigned *)mstep;
    const int row = blockIdx.x;
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if ((int)threadIdx.x < world) {
        const unsigned *f = pflags + (size_t)(row / rows_per_pair) * world + threadIdx.x;
        const long long t0 = clock64();
        // (polled at leisure: these blocks sit beside a kernel that is still
        // streaming, and a flag only matters once it is up)
        while ((int)(ld_acquire_sys(f) - (step + 1u)) < 0) {
            if (clock64() - t0 > wait_cycles) {
                s_ok = 0;
                report_timeout(status, 90 + (int)threadIdx.x);
                break;
            }
            __nanosleep(200);
        }
    }
    __syncthreads();
    if (s_ok) {
        const int stride = hd + 2;
        const float *buf = gather + (size_t)(step & 1u) * world * rows * stride;
        float M = -CUDART_INF_F;
        for (int i = 0; i < world; i++) {
            M = fmaxf(M, __ldcg(buf + ((size_t)i * rows + row) * stride + hd));
        }
        for (int d = threadIdx.x; d < hd; d += blockDim.x) {
            float O = 0.0f, L = 0.0f;
            for (int i = 0; i < world; i++) {
                const float *pr = buf + ((size_t)i * rows + row) * stride;
                const float mi = __ldcg(pr + hd);
                const float f = (mi == -CUDART_INF_F) ? 0.0f : __expf(mi - M);
                O += f * __ldcg(pr + d);
                L += f * __ldcg(pr + hd + 1);
            }
            out[(size_t)row * hd + d] = L > 0.0f ? O / L : 0.0f;
        }
    }
    // count the block out; the last one advances the step (every block has
    // read it by then)
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned prev = atomicAdd(mstep + 1, 1u);
        if (prev == gridDim.x - 1) {
            mstep[1] = 0u;
            __threadfence();
            *(volatile unsigned *)mstep = step + 1u;
        }
    }
}

const KernelReg reg_merge_pairs("lse_merge_pairs", (const void *)lse_merge_pairs_kernel);

}  // namespace

void launch_lse_merge_wait(cudaStream_t st, const float *gather, const unsigned *flags,
                           const unsigned *step, int world, int rows, int hd, float *out,
                           int *status, long long wait_cycles)
{
    lse_merge_wait_kernel<<<rows, hd, 0, st>>>(gather, flags, step, world, rows, hd, out, status,
                                               wait_cycles);
}

cudaError_t launch_lse_merge_pairs(cudaStream_t st, const float *gather, const unsigned *pflags,
                                   unsigned *mstep, int world, int rows, int rows_per_pair, int hd,
                                   float *out, int *status, long long wait_cycles, bool early)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(rows);
    cfg.blockDim = dim3(hd < 32 ? 32 : (hd > 256 ? 256 : hd));
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = early ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, lse_merge_pairs_kernel, gather, pflags, mstep, world, rows,
                              rows_per_pair, hd, out, status, wait_cycles);
}

cudaError_t launch_decode_f16(cudaStream_t st, const DecodeParams &p, int hd)
{
    bool v16 = true;
    for (int b = 0; b < p.nseq; b++) {
        if (p.seq[b].cap % 8 != 0 || ((uintptr_t)p.seq[b].v & 15u) != 0) v16 = false;
    }
    return hd == 128 ? launch_hd<128>(st, p, v16) : launch_hd<64>(st, p, v16);
}

int decode_resident_blocks(int hd, int sm_count, int nb)
{
    return (hd == 128 ? resident<128>(nb) : resident<64>(nb)) * sm_count;
}

int decode_f32_splits(int tk)
{
    return std::max(1, std::min(8, (tk + 63) / 64));
}

void launch_decode_f32(cudaStream_t st, const float *q, long long q_off, const float *k,
                       const float *v, float *out, long long out_off, int heads, int kv_heads,
                       int hd, int tk, int cap, float q_scale, float s_scale, float *part,
                       unsigned *ctr)
{
    (void)hd;   // 64: the only width the f32 cache is decoded at
    // up to eight blocks a head, each a whole number of 64-key chunks
    const int splits = part ? decode_f32_splits(tk) : 1;
    const int span = ((tk + splits - 1) / splits + 63) / 64 * 64;
    const dim3 grid(heads, (tk + span - 1) / span);
    decode_f32_split_kernel<64><<<grid, 256, 0, st>>>(q, q_off, k, v, out, out_off,
                                                     heads / kv_heads, tk, cap, q_scale, s_scale,
                                                     span, part, ctr);
}

void launch_lse_merge(cudaStream_t st, const float *parts_buf, int parts, int rows, int hd,
                      float *out)
{
    lse_merge_kernel<<<rows, hd, 0, st>>>(parts_buf, parts, rows, hd, out);
}
