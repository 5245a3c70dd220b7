// The stacked attention projection of one decoded row, each column placed
// where attention reads it (crates/llmtie-cuda/src/kernels.rs:6876-6913,
// `gemv_qkv_f16`): q = Wq a (+ bq) into a row, k = Wk a (+ bk) into the
// head-major f32 key cache at `pos`, v = Wv a (+ bv) into the transposed f32
// value cache at `pos`. W is the three [d][k] f16 weights stacked. This is the
// step in front of the Whisper decoder's self-attention (llmtie_attn_decode):
// one launch instead of three mat-vecs and two cache appends.
//
// Bound by the weight stream (3 d k halves, 9.8 MB at d = k = 1280): a warp
// takes a column and reads it 16 bytes a lane a step, the activation row
// waits in shared memory, and the products accumulate in f32 in a fixed
// order - lane partial sums over the lane's chunks in ascending order, then a
// shuffle tree - so a call is reproducible run to run.
#include "common.cuh"

namespace {

constexpr int kGemvWarps = 8;

__device__ __forceinline__ float2 unpack_f16x2(uint32_t w)
{
    const __half2 h = *reinterpret_cast<const __half2 *>(&w);
    return __half22float2(h);
}

template <bool WIDE>
__global__ void __launch_bounds__(kGemvWarps * 32)
gemv_qkv_kernel(const float *__restrict__ a, const uint16_t *__restrict__ w,
                const float *__restrict__ qb, const float *__restrict__ kb,
                const float *__restrict__ vb, int k, int d, int hd, int cap, int pos,
                float *__restrict__ q, float *__restrict__ kc, float *__restrict__ vc)
{
    extern __shared__ float a_s[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < k; i += blockDim.x) a_s[i] = a[i];
    __syncthreads();
    const int col = blockIdx.x * kGemvWarps + warp;
    if (col >= 3 * d) return;
    const uint16_t *row = w + (size_t)col * k;
    float acc = 0.0f;
    if constexpr (WIDE) {
        // eight halves a lane a step, two steps in flight
        const uint4 *r4 = reinterpret_cast<const uint4 *>(row);
        const int n8 = k >> 3;
        for (int i = lane; i < n8; i += 64) {
            const uint4 x0 = __ldg(r4 + i);
            const bool two = i + 32 < n8;
            const uint4 x1 = two ? __ldg(r4 + i + 32) : make_uint4(0u, 0u, 0u, 0u);
            const float *as0 = a_s + 8 * i;
            const uint32_t ws0[4] = {x0.x, x0.y, x0.z, x0.w};
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float2 f = unpack_f16x2(ws0[e]);
                acc = fmaf(as0[2 * e], f.x, acc);
                acc = fmaf(as0[2 * e + 1], f.y, acc);
            }
            if (two) {
                const float *as1 = a_s + 8 * (i + 32);
                const uint32_t ws1[4] = {x1.x, x1.y, x1.z, x1.w};
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float2 f = unpack_f16x2(ws1[e]);
                    acc = fmaf(as1[2 * e], f.x, acc);
                    acc = fmaf(as1[2 * e + 1], f.y, acc);
                }
            }
        }
    } else {
        const uint32_t *r2 = reinterpret_cast<const uint32_t *>(row);
        for (int i = lane; i < (k >> 1); i += 32) {
            const float2 f = unpack_f16x2(__ldg(r2 + i));
            acc = fmaf(a_s[2 * i], f.x, acc);
            acc = fmaf(a_s[2 * i + 1], f.y, acc);
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, off);
    if (lane != 0) return;
    const int part = col / d, c = col - part * d;
    if (part == 0) {
        q[c] = acc + (qb ? qb[c] : 0.0f);
    } else if (part == 1) {
        const int hh = c / hd, j = c - hh * hd;
        kc[((size_t)hh * cap + pos) * hd + j] = acc + (kb ? kb[c] : 0.0f);
    } else {
        vc[(size_t)c * cap + pos] = acc + (vb ? vb[c] : 0.0f);
    }
}

const KernelReg reg_gemv_qkv("gemv_qkv_f16", (const void *)gemv_qkv_kernel<true>);

}  // namespace

cudaError_t launch_gemv_qkv_f16(cudaStream_t st, const float *a, const uint16_t *w, const float *qb,
                                const float *kb, const float *vb, int k, int d, int hd, int cap,
                                int pos, float *q, float *kc, float *vc)
{
    const unsigned blocks = (unsigned)((3 * d + kGemvWarps - 1) / kGemvWarps);
    const size_t smem = (size_t)k * sizeof(float);
    const bool wide = k % 8 == 0 && ((uintptr_t)w & 15u) == 0;
    if (smem > 48 * 1024) {
        static bool raised[64] = {false};
        int dev = 0;
        cudaGetDevice(&dev);
        if (dev >= 0 && dev < 64 && !raised[dev]) {
            cudaFuncSetAttribute(gemv_qkv_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 200 * 1024);
            cudaFuncSetAttribute(gemv_qkv_kernel<false>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            raised[dev] = true;
        }
    }
    if (wide) {
        gemv_qkv_kernel<true><<<blocks, kGemvWarps * 32, smem, st>>>(a, w, qb, kb, vb, k, d, hd, cap,
                                                                    pos, q, kc, vc);
    } else {
        gemv_qkv_kernel<false><<<blocks, kGemvWarps * 32, smem, st>>>(a, w, qb, kb, vb, k, d, hd,
                                                                     cap, pos, q, kc, vc);
    }
    return cudaGetLastError();
}
