// Fused attention over many query rows, straight from the caches' own
// layouts: the general kernel behind flash_attn / flash_attn_f16 /
// flash_attn_rows / cross attention. It takes every shape the reference's
// `flash_attn_impl` takes (crates/llmtie-cuda/src/kernels.rs:3026-3270): head
// widths 64 and 128, f16 or f32 caches, any even capacity, causal or not, a
// prefix already in the cache.
//
// Arithmetic (kernels.rs:3078-3269): q rounded to f16 (after the scale when
// the scale goes on q), scores in f32, logits in log2 units, online softmax
// with ex2, the normaliser from un-rounded probabilities, probabilities
// rounded to f16 into the value product, f32 accumulation, O / l at the end.
//
// A warp owns sixteen query rows of one head and walks the keys 32 at a
// time. Both B operands are read directly from global memory into MMA
// fragment registers with the permuted contraction index described in
// decode.cu, so there is no shared-memory staging; the query heads of one
// KV group sit in one block and run in step, which makes their K/V reads L1
// hits. This kernel is the path for layouts the tensor-memory kernel cannot
// take (unaligned capacities, f32 caches, short rows).
#include "common.cuh"

#include <math_constants.h>

namespace {

__device__ __forceinline__ void ld128(uint32_t (&r)[4], const void *p)
{
    asm("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
        : "l"(p));
}

__device__ __forceinline__ uint32_t ld32(const void *p)
{
    uint32_t r;
    asm("ld.global.nc.u32 %0, [%1];" : "=r"(r) : "l"(p));
    return r;
}

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

__device__ __forceinline__ uint32_t pack_f16(float x0, float x1)
{
    return (uint32_t)__half_as_ushort(__float2half_rn(x0)) |
           ((uint32_t)__half_as_ushort(__float2half_rn(x1)) << 16);
}

// Eight consecutive cache elements starting at `p`, as four packed half2.
// f16 caches: one 16-byte load when aligned, four 4-byte loads otherwise.
// f32 caches: eight scalar loads, rounded to f16 as the reference's staging
// rounds them.
template <bool KV32, bool A16>
__device__ __forceinline__ void load8(uint32_t (&r)[4], const void *p, int nlive)
{
    if constexpr (KV32) {
        const float *f = (const float *)p;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float x0 = (nlive > 2 * i) ? __ldg(f + 2 * i) : 0.0f;
            const float x1 = (nlive > 2 * i + 1) ? __ldg(f + 2 * i + 1) : 0.0f;
            r[i] = pack_f16(x0, x1);
        }
    } else {
        if constexpr (A16) {
            if (nlive > 0) ld128(r, p);
        } else {
            const uint32_t *w = (const uint32_t *)p;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                if (nlive > 2 * i) r[i] = ld32(w + i);
            }
        }
        if (nlive < 8) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                if (nlive <= 2 * i) {
                    r[i] = 0u;
                } else if (nlive == 2 * i + 1) {
                    r[i] &= 0x0000ffffu;
                }
            }
        }
    }
}

template <int HD, bool KV32, bool A16>
__global__ void __launch_bounds__(128)
prefill_mma_kernel(const __grid_constant__ PrefillParams p)
{
    constexpr int KI = HD / 32;
    constexpr int NT = HD / 8;
    using KV = typename std::conditional<KV32, float, uint16_t>::type;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2;
    const int c = lane & 3;

    // As much of a KV group as four warps hold shares a block; the rest of
    // the warps take further row tiles of the same heads.
    const int group = p.heads / p.kv_heads;
    const int gb = (group % 4 == 0) ? 4 : (group % 2 == 0) ? 2 : 1;
    const int head = blockIdx.y * gb + (warp % gb);
    const int tile = blockIdx.x * (4 / gb) + warp / gb;
    const int r0 = tile * 16;
    const PrefillSeq &sq = p.seq[blockIdx.z];
    const int tq = sq.tq, past = sq.past, cap = sq.cap;
    if (r0 >= tq) return;
    const int kh = head / group;

    const KV *kbase = (const KV *)sq.k + (size_t)kh * cap * HD;
    const KV *vbase = (const KV *)sq.v + (size_t)kh * HD * cap;
    const float *qbase = p.q + (long long)sq.row0 * p.q_stride;

    const int row_a = r0 + g, row_b = r0 + g + 8;
    // Keys each row sees: [0, lim). Rows past tq are computed on a clamped
    // copy of the last row and never stored.
    const int all = p.causal ? past + tq : sq.tk;
    const int lim_a = p.causal ? min(past + row_a + 1, all) : all;
    const int lim_b = p.causal ? min(past + row_b + 1, all) : all;
    const int kend = p.causal ? min(past + r0 + 16, all) : all;   // the warp's

    uint32_t qa[KI][2][4];
    {
        const float *qa_row = qbase + (long long)min(row_a, tq - 1) * p.q_stride + head * HD;
        const float *qb_row = qbase + (long long)min(row_b, tq - 1) * p.q_stride + head * HD;
#pragma unroll
        for (int i = 0; i < KI; i++) {
#pragma unroll
            for (int u = 0; u < 2; u++) {
                const int at = 32 * i + 8 * c + 4 * u;
                const float4 xa = *(const float4 *)(qa_row + at);
                const float4 xb = *(const float4 *)(qb_row + at);
                qa[i][u][0] = pack_f16(xa.x * p.q_scale, xa.y * p.q_scale);
                qa[i][u][1] = pack_f16(xb.x * p.q_scale, xb.y * p.q_scale);
                qa[i][u][2] = pack_f16(xa.z * p.q_scale, xa.w * p.q_scale);
                qa[i][u][3] = pack_f16(xb.z * p.q_scale, xb.w * p.q_scale);
            }
        }
    }

    float m_a = -CUDART_INF_F, m_b = -CUDART_INF_F;
    float l_a = 0.0f, l_b = 0.0f;
    float o[NT][4];
#pragma unroll
    for (int j = 0; j < NT; j++) {
        o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;
    }

    for (int blk = 0; blk < kend; blk += 32) {
        float ta[2][2][2], tb[2][2][2];
#pragma unroll
        for (int mm = 0; mm < 2; mm++) {
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const int key = blk + 8 * (g >> 1) + 4 * mm + 2 * h + (g & 1);
                const KV *krow = kbase + (size_t)key * HD + 8 * c;
                const int nlive = key < kend ? 8 : 0;
                float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int i = 0; i < KI; i++) {
                    uint32_t r[4] = {0u, 0u, 0u, 0u};
                    load8<KV32, true>(r, krow + 32 * i, nlive);
                    mma16816(acc, qa[i][0][0], qa[i][0][1], qa[i][0][2], qa[i][0][3], r[0], r[1]);
                    mma16816(acc, qa[i][1][0], qa[i][1][1], qa[i][1][2], qa[i][1][3], r[2], r[3]);
                }
                const int k0 = blk + 8 * c + 4 * mm + 2 * h;
                ta[mm][h][0] = (k0 < lim_a) ? acc[0] * p.sl2 : -CUDART_INF_F;
                ta[mm][h][1] = (k0 + 1 < lim_a) ? acc[1] * p.sl2 : -CUDART_INF_F;
                tb[mm][h][0] = (k0 < lim_b) ? acc[2] * p.sl2 : -CUDART_INF_F;
                tb[mm][h][1] = (k0 + 1 < lim_b) ? acc[3] * p.sl2 : -CUDART_INF_F;
            }
        }

        float bm_a = -CUDART_INF_F, bm_b = -CUDART_INF_F;
#pragma unroll
        for (int mm = 0; mm < 2; mm++) {
#pragma unroll
            for (int h = 0; h < 2; h++) {
                bm_a = fmaxf(bm_a, fmaxf(ta[mm][h][0], ta[mm][h][1]));
                bm_b = fmaxf(bm_b, fmaxf(tb[mm][h][0], tb[mm][h][1]));
            }
        }
        bm_a = fmaxf(bm_a, __shfl_xor_sync(0xffffffffu, bm_a, 1));
        bm_a = fmaxf(bm_a, __shfl_xor_sync(0xffffffffu, bm_a, 2));
        bm_b = fmaxf(bm_b, __shfl_xor_sync(0xffffffffu, bm_b, 1));
        bm_b = fmaxf(bm_b, __shfl_xor_sync(0xffffffffu, bm_b, 2));
        const float mn_a = fmaxf(m_a, bm_a), mn_b = fmaxf(m_b, bm_b);
        // A row whose keys in this block are all masked keeps -inf here only
        // if it has seen no key at all, which a causal row never is past its
        // first block; the guards keep exp2(-inf - -inf) out of the sums.
        if (__any_sync(0xffffffffu, mn_a > m_a || mn_b > m_b)) {
            const float al_a = (mn_a == -CUDART_INF_F) ? 1.0f : ex2(m_a - mn_a);
            const float al_b = (mn_b == -CUDART_INF_F) ? 1.0f : ex2(m_b - mn_b);
            l_a *= al_a;
            l_b *= al_b;
#pragma unroll
            for (int j = 0; j < NT; j++) {
                o[j][0] *= al_a;
                o[j][1] *= al_a;
                o[j][2] *= al_b;
                o[j][3] *= al_b;
            }
        }
        m_a = mn_a;
        m_b = mn_b;
        const float sub_a = (m_a == -CUDART_INF_F) ? 0.0f : m_a;
        const float sub_b = (m_b == -CUDART_INF_F) ? 0.0f : m_b;
        uint32_t pa[2][4];
#pragma unroll
        for (int mm = 0; mm < 2; mm++) {
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const float a0 = ex2(ta[mm][h][0] - sub_a), a1 = ex2(ta[mm][h][1] - sub_a);
                const float b0 = ex2(tb[mm][h][0] - sub_b), b1 = ex2(tb[mm][h][1] - sub_b);
                l_a += a0 + a1;
                l_b += b0 + b1;
                pa[mm][2 * h] = pack_f16(a0, a1);
                pa[mm][2 * h + 1] = pack_f16(b0, b1);
            }
        }

        const int g0 = blk + 8 * c;
        const int nlive = kend - g0;
#pragma unroll
        for (int j = 0; j < NT; j++) {
            const KV *vrow = vbase + (size_t)(8 * j + g) * cap + g0;
            uint32_t r[4] = {0u, 0u, 0u, 0u};
            load8<KV32, A16>(r, vrow, nlive);
            mma16816(o[j], pa[0][0], pa[0][1], pa[0][2], pa[0][3], r[0], r[1]);
            mma16816(o[j], pa[1][0], pa[1][1], pa[1][2], pa[1][3], r[2], r[3]);
        }
    }

    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
    const float inv_a = l_a > 0.0f ? 1.0f / l_a : 0.0f;
    const float inv_b = l_b > 0.0f ? 1.0f / l_b : 0.0f;
#pragma unroll
    for (int j = 0; j < NT; j++) {
        const int col = head * HD + 8 * j + 2 * c;
        if (p.out_f16) {
            uint16_t *out = (uint16_t *)p.out + (long long)sq.row0 * p.out_stride;
            if (row_a < tq) {
                *(uint32_t *)(out + (long long)row_a * p.out_stride + col) =
                    pack_f16(o[j][0] * inv_a, o[j][1] * inv_a);
            }
            if (row_b < tq) {
                *(uint32_t *)(out + (long long)row_b * p.out_stride + col) =
                    pack_f16(o[j][2] * inv_b, o[j][3] * inv_b);
            }
        } else {
            float *out = (float *)p.out + (long long)sq.row0 * p.out_stride;
            if (row_a < tq) {
                *(float2 *)(out + (long long)row_a * p.out_stride + col) =
                    make_float2(o[j][0] * inv_a, o[j][1] * inv_a);
            }
            if (row_b < tq) {
                *(float2 *)(out + (long long)row_b * p.out_stride + col) =
                    make_float2(o[j][2] * inv_b, o[j][3] * inv_b);
            }
        }
    }
}

template <int HD>
cudaError_t launch_hd(cudaStream_t st, const PrefillParams &p)
{
    const int group = p.heads / p.kv_heads;
    const int gb = (group % 4 == 0) ? 4 : (group % 2 == 0) ? 2 : 1;
    const int rows_per_block = 16 * (4 / gb);
    int max_tq = 0;
    bool a16 = !p.kv_f32;
    for (int b = 0; b < p.nseq; b++) {
        max_tq = p.seq[b].tq > max_tq ? p.seq[b].tq : max_tq;
        if (p.seq[b].cap % 8 != 0 || ((uintptr_t)p.seq[b].v & 15u) != 0) a16 = false;
    }
    if (max_tq == 0) return cudaSuccess;
    const dim3 grid((max_tq + rows_per_block - 1) / rows_per_block, p.heads / gb, p.nseq);
    if (p.kv_f32) {
        prefill_mma_kernel<HD, true, false><<<grid, 128, 0, st>>>(p);
    } else if (a16) {
        prefill_mma_kernel<HD, false, true><<<grid, 128, 0, st>>>(p);
    } else {
        prefill_mma_kernel<HD, false, false><<<grid, 128, 0, st>>>(p);
    }
    return cudaGetLastError();
}

const KernelReg reg_f128h("flash_attn_h", (const void *)prefill_mma_kernel<128, false, true>);
const KernelReg reg_f128hu("flash_attn_h_unaligned", (const void *)prefill_mma_kernel<128, false, false>);
const KernelReg reg_f128("flash_attn", (const void *)prefill_mma_kernel<128, true, false>);
const KernelReg reg_f64("flash_attn_64", (const void *)prefill_mma_kernel<64, true, false>);
const KernelReg reg_f64r("flash_attn_64_rows", (const void *)prefill_mma_kernel<64, false, true>);

}  // namespace

cudaError_t launch_prefill_mma(cudaStream_t st, const PrefillParams &p, int hd)
{
    return hd == 128 ? launch_hd<128>(st, p) : launch_hd<64>(st, p);
}
