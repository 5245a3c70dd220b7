// The long-context decode kernel: the arithmetic of decode.cu (f32-exact
// query and probabilities on mma.m16n8k16 by hi/lo splitting, permuted
// contraction index, log-sum-exp merge by the last block to arrive), fed
// through a per-warp ring of asynchronous copies and cut over the grid by
// work rather than by head.
//
// Why a ring. The kernel is bound by HBM, and a B200 needs tens of kilobytes
// per SM in flight to cover DRAM latency. Loads that land in registers hold a
// register for every byte in flight; cp.async lands in shared memory instead,
// so each warp keeps two whole 32-key blocks (K 8 KB + V 8 KB each at
// head_dim 128) in flight while it computes on a third. A warp owns its ring
// outright: there is no block-wide barrier in the key loop, only
// cp.async.wait_group and __syncwarp.
//
// Why by work. One block per SM is resident (the ring is 192 KB), and a grid
// cut by (sequence, KV head) leaves SMs idle whenever their count does not
// divide 148. Instead all 128-key units of the launch are laid end to end,
// pair after pair, and block c takes units [c W / G, (c + 1) W / G). A block
// whose range covers a whole (sequence, KV head) pair writes its output
// directly; a range that cuts a pair writes a partial (o, m, l), and the last
// block of that pair to arrive merges (crates/llmtie-cuda/src/kernels.rs:
// 5779-5903 does the same with one counter a head).
//
// Needs 16-byte aligned value rows (capacity a multiple of 8); other caches
// take the register kernel in decode.cu.
#include "common.cuh"

#include <math_constants.h>
#include <string.h>

namespace {

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kRows = 8;
constexpr int kStages = 3;

__device__ __forceinline__ void cp_async16(void *smem, const void *gmem, int src_bytes)
{
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem),
                 "r"(src_bytes)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit()
{
    asm volatile("cp.async.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait()
{
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void lds128(uint32_t (&r)[4], const void *smem)
{
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(a));
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

__device__ __forceinline__ void split_pair(float x0, float x1, uint32_t &hi, uint32_t &lo)
{
    const __half h0 = __float2half_rn(x0), h1 = __float2half_rn(x1);
    const __half l0 = __float2half_rn(x0 - __half2float(h0));
    const __half l1 = __float2half_rn(x1 - __half2float(h1));
    hi = (uint32_t)__half_as_ushort(h0) | ((uint32_t)__half_as_ushort(h1) << 16);
    lo = (uint32_t)__half_as_ushort(l0) | ((uint32_t)__half_as_ushort(l1) << 16);
}

// The block that holds unit u when W units are cut over G blocks as
// [c W / G, (c + 1) W / G): the largest c with floor(c W / G) <= u.
__device__ __forceinline__ int covering(long long u, long long W, long long G)
{
    return (int)(((u + 1) * G + W - 1) / W - 1);
}

// One finished value of a pair: normalised into `out`, or the un-normalised
// triple - into `out`, or, when ranks exchange, straight into every rank's
// gather buffer over NVLink (this rank's included).
template <int HD>
__device__ __forceinline__ void emit_value(const DecodeStreamParams &p, long long ooff,
                                           unsigned xch_step, int row, int d, float O, float M,
                                           float L)
{
    constexpr float kLn2 = 0.6931471805599453f;
    const long long at = ooff + (long long)row * p.out_row;
    if (!p.partial) {
        p.out[at + d] = L > 0.0f ? O / L : 0.0f;
    } else if (p.xch_world == 0) {
        p.out[at + d] = O;
        if (d == 0) {
            p.out[at + HD] = M * kLn2;
            p.out[at + HD + 1] = L;
        }
    } else {
        const long long slot_at =
            ((long long)(xch_step & 1u) * p.xch_world + p.xch_rank) * p.xch_rank_stride + at;
        for (int r = 0; r < p.xch_world; r++) {
            float *dst = p.xch_gather[r] + slot_at;
            dst[d] = O;
            if (d == 0) {
                dst[HD] = M * kLn2;
                dst[HD + 1] = L;
            }
        }
    }
}

// The last block of a pair to arrive merges every partial of the pair. Kept
// out of line: its register needs must not shape the allocation of the key
// loop, which is what the kernel's bandwidth hangs on.
template <int HD>
__device__ __noinline__ void merge_pair(const DecodeStreamParams &p, long long pair_u0,
                                        int c_first, int c_last, int rows_here, long long W,
                                        long long G, long long ooff, unsigned xch_step)
{
    const int tid = threadIdx.x;
    const int count = c_last - c_first + 1;
    auto emit = [&](int row, int d, float O, float M, float L) {
        emit_value<HD>(p, ooff, xch_step, row, d, O, M, L);
    };
                // Each thread owns column tid % HD of every row. Rows are taken
    // four at a time and contributors four at a time, so that all of
    // a batch's loads are in flight together: with at most four
    // contributors (the usual case) the whole merge is one trip to
    // L2. m and l are read by every thread (a broadcast), so no
    // exchange through shared memory is needed.
    const int d = tid % HD;
    for (int r0 = 0; r0 < rows_here; r0 += 4) {
        float Mx[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
        if (count > 4) {
            for (int c0 = c_first; c0 <= c_last; c0 += 8) {
                float mi[4][8];
#pragma unroll
                for (int rr = 0; rr < 4; rr++) {
#pragma unroll
                    for (int e = 0; e < 8; e++) {
                        const int cc = min(c0 + e, c_last);
                        const int sl = ((long long)cc * W / G >= pair_u0) ? 0 : 1;
                        const int row = min(r0 + rr, rows_here - 1);
                        mi[rr][e] = ldcg(p.part + (((size_t)cc * 2 + sl) * kRows + row) *
                                                      (HD + 2) + HD);
                    }
                }
#pragma unroll
                for (int rr = 0; rr < 4; rr++) {
#pragma unroll
                    for (int e = 0; e < 8; e++) Mx[rr] = fmaxf(Mx[rr], mi[rr][e]);
                }
            }
        }
        float Ox[4] = {0.0f, 0.0f, 0.0f, 0.0f}, Lx[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int c0 = c_first; c0 <= c_last; c0 += 4) {
            float mi[4][4], li[4][4], oi[4][4];
#pragma unroll
            for (int rr = 0; rr < 4; rr++) {
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int cc = min(c0 + e, c_last);
                    const int sl = ((long long)cc * W / G >= pair_u0) ? 0 : 1;
                    const int row = min(r0 + rr, rows_here - 1);
                    const float *pr =
                        p.part + (((size_t)cc * 2 + sl) * kRows + row) * (HD + 2);
                    mi[rr][e] = ldcg(pr + HD);
                    li[rr][e] = ldcg(pr + HD + 1);
                    oi[rr][e] = ldcg(pr + d);
                }
            }
            if (count <= 4) {
#pragma unroll
                for (int rr = 0; rr < 4; rr++) {
#pragma unroll
                    for (int e = 0; e < 4; e++) Mx[rr] = fmaxf(Mx[rr], mi[rr][e]);
                }
            }
#pragma unroll
            for (int rr = 0; rr < 4; rr++) {
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    if (c0 + e <= c_last) {
                        const float f = (mi[rr][e] == -CUDART_INF_F)
                                            ? 0.0f
                                            : ex2(mi[rr][e] - Mx[rr]);
                        Ox[rr] += f * oi[rr][e];
                        Lx[rr] += f * li[rr][e];
                    }
                }
            }
        }
        if (tid < HD) {
#pragma unroll
            for (int rr = 0; rr < 4; rr++) {
                if (r0 + rr < rows_here) emit(r0 + rr, d, Ox[rr], Mx[rr], Lx[rr]);
            }
        }
    }
}

template <int HD>
__global__ void __launch_bounds__(kThreads, 1)
decode_stream_kernel(const __grid_constant__ DecodeStreamParams p)
{
    constexpr int KI = HD / 32;
    constexpr int NT = HD / 8;
    constexpr int KROW = HD * 2;            // bytes of one key row
    constexpr int KBYTES = 32 * KROW;       // one 32-key block of keys
    constexpr int VBYTES = HD * 64;         // the same block of the transposed values
    constexpr int STAGE = KBYTES + VBYTES;
    constexpr int KCH = KROW / 16;          // 16-byte chunks in a key row
    constexpr float kLn2 = 0.6931471805599453f;

    extern __shared__ __align__(128) unsigned char ring_all[];
    __shared__ float sm_o[kWarps][kRows][HD];
    __shared__ float sm_m[kWarps][kRows];
    __shared__ float sm_l[kWarps][kRows];
    __shared__ float sm_M[kRows];
    __shared__ int sm_last;

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int g = lane >> 2;
    const int c = lane & 3;
    unsigned char *ring = ring_all + (size_t)warp * kStages * STAGE;

    // When ranks exchange, the step number picks which of the two gather
    // buffers this launch fills; every block reads it before any block can
    // have finished the launch and advanced it.
    const unsigned xch_step = p.xch_world ? *(volatile const unsigned *)p.xch_step : 0u;

    const long long W = p.total_units;
    const long long G = gridDim.x;
    const long long u0 = (long long)blockIdx.x * W / G;
    const long long u1 = (long long)(blockIdx.x + 1) * W / G;
    const int inner_pairs = p.kv_heads * p.row_chunks;

    long long u = u0;
    while (u < u1) {
        // ---- which pair this unit lies in, and how much of it is ours ---------
        int b = 0;
        while (b + 1 < p.nseq && u >= p.unit0[b + 1]) b++;
        const int tk = p.seq[b].tk;
        const int cap = p.seq[b].cap;
        const int n_units = (tk + 127) >> 7;                 // units of one pair
        const long long rel = u - p.unit0[b];
        const int inner = (int)(rel / n_units);              // rc * kv_heads + kh
        const int off = (int)(rel % n_units);
        const int rc = inner / p.kv_heads;
        const int kh = inner % p.kv_heads;
        const int seg_end = (int)min((long long)n_units, off + (u1 - u));
        const int k_begin = off * 128;
        const int k_end = min(tk, seg_end * 128);
        const bool whole = (off == 0 && seg_end == n_units);
        const long long pair_u0 = p.unit0[b] + (long long)inner * n_units;
        const int pair = p.pair0[b] + inner;
        const uint16_t *kbase = p.seq[b].k + (size_t)kh * cap * HD;
        const uint16_t *vbase = p.seq[b].v + (size_t)kh * HD * cap;
        const int rows_here = min(kRows, p.rows - rc * kRows);

        // ---- query fragments, permuted as the key loads are, split hi / lo ------
        uint32_t qa[KI][2][4];
        {
            const float *qrow = p.q + (long long)b * p.q_seq + (long long)kh * p.q_kv +
                                (long long)(rc * kRows + g) * p.q_row;
            const bool live = g < rows_here;
#pragma unroll
            for (int i = 0; i < KI; i++) {
#pragma unroll
                for (int uu = 0; uu < 2; uu++) {
                    const int at = 32 * i + 8 * c + 4 * uu;
                    float x[4];
#pragma unroll
                    for (int e = 0; e < 4; e++) x[e] = live ? qrow[at + e] * p.q_scale : 0.0f;
                    split_pair(x[0], x[1], qa[i][uu][0], qa[i][uu][1]);
                    split_pair(x[2], x[3], qa[i][uu][2], qa[i][uu][3]);
                }
            }
        }

        float m = -CUDART_INF_F;
        float l = 0.0f;
        float o[NT][4];
#pragma unroll
        for (int j = 0; j < NT; j++) {
            o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;
        }

        // Copies block `blk` (32 keys) into ring stage `st`. Keys past k_end are
        // zero-filled (a copy of zero source bytes); a key row's two 64-byte
        // halves are swapped on odd rows so that the fragment reads of two
        // adjacent rows fall on different banks.
        auto issue = [&](int blk, int st) {
            unsigned char *ks = ring + st * STAGE;
            unsigned char *vs = ks + KBYTES;
#pragma unroll
            for (int it = 0; it < KBYTES / 16 / 32; it++) {
                const int chunk = lane + 32 * it;
                const int row = chunk / KCH, ch = chunk % KCH;
                const int key = blk + row;
                const bool live = key < k_end;
                const uint16_t *src = kbase + (size_t)(live ? key : k_begin) * HD + ch * 8;
                cp_async16(ks + row * KROW + ((ch ^ ((row & 1) << 2)) << 4), src, live ? 16 : 0);
            }
#pragma unroll
            for (int it = 0; it < VBYTES / 16 / 32; it++) {
                const int chunk = lane + 32 * it;
                const int row = chunk >> 2, ch = chunk & 3;
                const int k0 = blk + 8 * ch;
                const bool live = k0 < k_end;
                const uint16_t *src = vbase + (size_t)row * cap + (live ? k0 : k_begin);
                cp_async16(vs + row * 64 + ch * 16, src, live ? 16 : 0);
            }
        };

        // This warp's blocks: k_begin + (warp + kWarps * i) * 32.
        const int first = k_begin + warp * 32;
        const int nblk = first < k_end ? (k_end - first + kWarps * 32 - 1) / (kWarps * 32) : 0;
#pragma unroll
        for (int s = 0; s < kStages - 1; s++) {
            if (s < nblk) issue(first + s * kWarps * 32, s);
            cp_async_commit();
        }

        for (int i = 0; i < nblk; i++) {
            // Start the copy two blocks ahead, into the stage the last
            // iteration finished with, then wait for this block's.
            {
                const int nx = i + kStages - 1;
                if (nx < nblk) issue(first + nx * kWarps * 32, nx % kStages);
                cp_async_commit();
            }
            cp_async_wait<kStages - 1>();
            __syncwarp();

            const int blk = first + i * kWarps * 32;
            const unsigned char *ks = ring + (i % kStages) * STAGE;
            const unsigned char *vs = ks + KBYTES;

            // ---- scores: four 8-key tiles ----------------------------------------
            float t[2][2][2];
#pragma unroll
            for (int mm = 0; mm < 2; mm++) {
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const int row = 8 * (g >> 1) + 4 * mm + 2 * h + (g & 1);
                    const unsigned char *krow = ks + row * KROW;
                    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                    for (int ii = 0; ii < KI; ii++) {
                        uint32_t r[4];
                        lds128(r, krow + (((4 * ii + c) ^ ((g & 1) << 2)) << 4));
                        mma16816(acc, qa[ii][0][0], qa[ii][0][1], qa[ii][0][2], qa[ii][0][3],
                                 r[0], r[1]);
                        mma16816(acc, qa[ii][1][0], qa[ii][1][1], qa[ii][1][2], qa[ii][1][3],
                                 r[2], r[3]);
                    }
                    const int k0 = blk + 8 * c + 4 * mm + 2 * h;
                    t[mm][h][0] = (k0 < k_end) ? (acc[0] + acc[2]) * p.sl2 : -CUDART_INF_F;
                    t[mm][h][1] = (k0 + 1 < k_end) ? (acc[1] + acc[3]) * p.sl2 : -CUDART_INF_F;
                }
            }

            // ---- online softmax over the block -------------------------------------
            float bm = -CUDART_INF_F;
#pragma unroll
            for (int mm = 0; mm < 2; mm++) {
#pragma unroll
                for (int h = 0; h < 2; h++) bm = fmaxf(bm, fmaxf(t[mm][h][0], t[mm][h][1]));
            }
            bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 1));
            bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 2));
            const float m_new = fmaxf(m, bm);
            if (__any_sync(0xffffffffu, m_new > m)) {
                const float alpha = ex2(m - m_new);   // 0 on the first block
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
            uint32_t pa[2][4];
#pragma unroll
            for (int mm = 0; mm < 2; mm++) {
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const float p0 = ex2(t[mm][h][0] - m);
                    const float p1 = ex2(t[mm][h][1] - m);
                    l += p0 + p1;
                    split_pair(p0, p1, pa[mm][2 * h], pa[mm][2 * h + 1]);
                }
            }

            // ---- context ---------------------------------------------------------------
            const int nlive = k_end - (blk + 8 * c);   // keys of this thread's eight that exist
#pragma unroll
            for (int j = 0; j < NT; j++) {
                uint32_t r[4];
                lds128(r, vs + (8 * j + g) * 64 + c * 16);
                if (nlive < 8) {
                    // Capacity past the live keys may hold anything, and
                    // 0 * NaN is NaN: clear what lies beyond.
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        if (nlive <= 2 * e) {
                            r[e] = 0u;
                        } else if (nlive == 2 * e + 1) {
                            r[e] &= 0x0000ffffu;
                        }
                    }
                }
                mma16816(o[j], pa[0][0], pa[0][1], pa[0][2], pa[0][3], r[0], r[1]);
                mma16816(o[j], pa[1][0], pa[1][1], pa[1][2], pa[1][3], r[2], r[3]);
            }
            __syncwarp();   // every lane is done with this stage before it is refilled
        }
        cp_async_wait<0>();

        // ---- the block's four warps merge through shared memory ----------------------
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

        // A range that starts inside the pair is this block's first segment
        // (slot 0); one that started before it is its last (slot 1).
        const int slot = (u == u0) ? 0 : 1;
        float *part = p.part + ((size_t)blockIdx.x * 2 + slot) * kRows * (HD + 2);
        const long long ooff = (long long)b * p.out_seq + (long long)kh * p.out_kv +
                               (long long)(rc * kRows) * p.out_row;
        auto emit = [&](int row, int d, float O, float M, float L) {
            emit_value<HD>(p, ooff, xch_step, row, d, O, M, L);
        };
        // After a pair's values are out: count it, and the block that finishes
        // the launch's last pair raises this rank's flag on every rank.
        auto pair_done = [&]() {
            if (p.xch_world == 0) return;
            __threadfence_system();
            __syncthreads();
            if (tid == 0) {
                const unsigned prev = atomicAdd(p.xch_done, 1u);
                if (prev == (unsigned)(p.xch_pairs - 1)) {
                    *p.xch_done = 0u;
                    const unsigned next = xch_step + 1u;
                    __threadfence_system();
                    for (int r = 0; r < p.xch_world; r++) {
                        *(volatile unsigned *)(p.xch_flags[r] + p.xch_rank) = next;
                    }
                    *(volatile unsigned *)p.xch_step = next;
                }
            }
        };
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
            if (whole) {
                emit(row, d, O, M, L);
            } else {
                float *pr = part + row * (HD + 2);
                pr[d] = O;
                if (d == 0) {
                    pr[HD] = M;
                    pr[HD + 1] = L;
                }
            }
        }

        if (whole) pair_done();
        if (!whole) {
            // ---- the last block of this pair to arrive merges every partial -------------
            const int c_first = covering(pair_u0, W, G);
            const int c_last = covering(pair_u0 + n_units - 1, W, G);
            const int count = c_last - c_first + 1;
            __threadfence();
            __syncthreads();
            if (tid == 0) {
                const unsigned prev = atomicAdd(p.ctr + pair, 1u);
                sm_last = (prev == (unsigned)(count - 1));
            }
            __syncthreads();
            if (sm_last) {
                __threadfence();
                merge_pair<HD>(p, pair_u0, c_first, c_last, rows_here, W, G, ooff, xch_step);
                pair_done();
                if (tid == 0) p.ctr[pair] = 0u;   // at rest again for the next call
            }
        }
        __syncthreads();   // shared memory is reused by the next segment
        u += seg_end - off;
    }
}

template <int HD>
constexpr int ring_bytes()
{
    return kWarps * kStages * (32 * HD * 2 + HD * 64);
}

const KernelReg reg_s128("attn_decode_h128_run", (const void *)decode_stream_kernel<128>);
const KernelReg reg_s64("attn_decode_h64_run", (const void *)decode_stream_kernel<64>);

}  // namespace

cudaError_t launch_decode_stream(cudaStream_t st, const DecodeStreamParams &p, int hd, int grid)
{
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaFuncSetAttribute(decode_stream_kernel<128>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, ring_bytes<128>());
        cudaFuncSetAttribute(decode_stream_kernel<64>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, ring_bytes<64>());
        configured[dev] = true;
    }
    if (hd == 128) {
        decode_stream_kernel<128><<<grid, kThreads, ring_bytes<128>(), st>>>(p);
    } else {
        decode_stream_kernel<64><<<grid, kThreads, ring_bytes<64>(), st>>>(p);
    }
    return cudaGetLastError();
}

// ---- a decode entry point that allocates nothing -----------------------------------
//
// llmtie_attn_decode_f16 grows its caller's DecodeScratch with a stream-ordered
// allocation whenever a longer context needs more partials. Some callers
// cannot have that: a voice pipeline's per-token thread, where an allocation
// that has to go to the driver stalls every other stream on the card; or a
// process that gave the whole device to its own pool up front and has nothing
// left for anyone else to allocate from. For them the partials and the
// arrival counters live in the two arrays below, which every GPU that loads
// this library carries from load until exit (about 1.3 MB).
//
// The array names are host-side stand-ins, not device addresses. The address
// the kernel is given comes from cudaGetSymbolAddress, taken once per device
// with that device current, on the first call made on that device - so that
// first call should be made before any stream capture begins.
//
// Every call shares the arrays, and they keep what the last call left:
// the partials are always written before they are read, and the counters are
// cleared at the start of each call. Two calls that overlap on the GPU (two
// streams, two handles, two threads) would race on them; calls must be
// ordered one after another.
namespace {

constexpr int kStaticMaxBlocks = 160;   // blocks the launch may use (one per SM)
constexpr int kStaticMaxPairs = 64;     // kv heads it may carry
constexpr size_t kStaticPartFloats = (size_t)kStaticMaxBlocks * 2 * kRows * (128 + 2);

static __device__ __align__(256) float g_static_part[kStaticPartFloats];
static __device__ __align__(256) unsigned g_static_ctr[kStaticMaxPairs];

struct StaticScratch {
    bool ready = false;
    float *part = nullptr;
    unsigned *ctr = nullptr;
};
StaticScratch g_static_addr[64];

}  // namespace

extern "C" llmtie_status llmtie_attn_decode_f16_noalloc(
    llmtie_gpu *g, const float *q, size_t q_len, size_t q_off, const uint16_t *k, size_t k_len,
    const uint16_t *v, size_t v_len, size_t heads, size_t kv_heads, size_t head_dim, size_t tk,
    size_t cap, float scale, int32_t scale_q, float *out, size_t out_len, size_t out_off)
{
    if (!g) return llmtie_fail(LLMTIE_ERR_INVALID, "null device handle");
    if (g->ordinal < 0 || g->ordinal >= 64) {
        return llmtie_fail(LLMTIE_ERR_INVALID, "device ordinal %d is out of range", g->ordinal);
    }
    cudaSetDevice(g->ordinal);
    if (head_dim != 64 && head_dim != 128) {
        return llmtie_fail(LLMTIE_ERR_UNSUPPORTED_ATTENTION,
                           "fused attention wants head_dim 64 or 128, got %zu", head_dim);
    }
    const size_t gmax = head_dim == 128 ? 4 : 8;
    if (kv_heads == 0 || heads % kv_heads != 0 || heads / kv_heads > gmax) {
        return llmtie_fail(LLMTIE_ERR_UNSUPPORTED_ATTENTION,
                           "fused attention wants heads a multiple of kv_heads with a group of "
                           "at most %zu, got %zu heads over %zu", gmax, heads, kv_heads);
    }
    if (kv_heads > (size_t)kStaticMaxPairs) {
        return llmtie_fail(LLMTIE_ERR_UNSUPPORTED_ATTENTION,
                           "%zu kv heads is more than the %d the static scratch carries",
                           kv_heads, kStaticMaxPairs);
    }
    if (tk == 0 || tk > cap) {
        return llmtie_fail(LLMTIE_ERR_CACHE_OVERRUN,
                           "appending at %zu to a cache with room for %zu", tk, cap);
    }
    if (cap > 0x7fffffffu) {
        return llmtie_fail(LLMTIE_ERR_INVALID, "capacity does not fit 32 bits");
    }
    if (cap % 8 != 0 || ((uintptr_t)v & 15u) != 0 || ((uintptr_t)k & 15u) != 0) {
        return llmtie_fail(LLMTIE_ERR_MISALIGNED,
                           "the allocation-free decode wants 16-byte aligned caches and a "
                           "capacity that is a multiple of 8, got %zu", cap);
    }
    const size_t need = kv_heads * cap * head_dim;
    if (k_len < need || v_len < need) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %zu in a buffer of %zu", need,
                           k_len < v_len ? k_len : v_len);
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

    StaticScratch &ss = g_static_addr[g->ordinal];
    if (!ss.ready) {
        cudaError_t e = cudaGetSymbolAddress((void **)&ss.part, g_static_part);
        if (e == cudaSuccess) e = cudaGetSymbolAddress((void **)&ss.ctr, g_static_ctr);
        if (e != cudaSuccess) {
            return llmtie_fail(LLMTIE_ERR_DRIVER, "resolving the static scratch: %s",
                               cudaGetErrorString(e));
        }
        ss.ready = true;
    }

    const size_t group = heads / kv_heads;
    DecodeStreamParams sp;
    memset(&sp, 0, sizeof(sp));
    const long long units = (long long)((tk + 127) / 128) * (long long)kv_heads;
    sp.nseq = 1;
    sp.seq[0].k = k;
    sp.seq[0].v = v;
    sp.seq[0].tk = (int)tk;
    sp.seq[0].cap = (int)cap;
    sp.unit0[0] = 0;
    sp.unit0[1] = units;
    sp.pair0[0] = 0;
    sp.pair0[1] = (int)kv_heads;
    sp.total_units = units;
    sp.q = q + q_off;
    sp.q_kv = (long long)(group * head_dim);
    sp.q_row = (long long)head_dim;
    sp.out = out + out_off;
    sp.out_kv = (long long)(group * head_dim);
    sp.out_row = (long long)head_dim;
    sp.rows = (int)group;
    sp.row_chunks = 1;
    sp.kv_heads = (int)kv_heads;
    sp.partial = 0;
    sp.q_scale = scale_q ? scale : 1.0f;
    sp.sl2 = (scale_q ? 1.0f : scale) * 1.4426950408889634f;
    sp.part = ss.part;
    sp.ctr = ss.ctr;
    long long grid = g->sm_count < kStaticMaxBlocks ? g->sm_count : kStaticMaxBlocks;
    if (units < grid) grid = units;
    // The counters must start at zero whatever an earlier call left behind.
    cudaError_t e = cudaMemsetAsync(ss.ctr, 0, sizeof(unsigned) * kStaticMaxPairs, g->stream);
    if (e != cudaSuccess) {
        return llmtie_fail(LLMTIE_ERR_DRIVER, "clearing the static counters: %s",
                           cudaGetErrorString(e));
    }
    LaunchScope ls(g, head_dim == 128 ? "attn_decode_h128_run" : "attn_decode_h64_run");
    e = launch_decode_stream(g->stream, sp, (int)head_dim, (int)grid);
    if (e != cudaSuccess) {
        return llmtie_fail(LLMTIE_ERR_DRIVER, "attn_decode (static scratch): %s",
                           cudaGetErrorString(e));
    }
    return ls.done();
}
