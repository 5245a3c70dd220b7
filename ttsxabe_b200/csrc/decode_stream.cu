// The long-context decode kernel: the arithmetic of decode.cu (f32-exact
// query and probabilities on mma.m16n8k16 by hi/lo splitting, permuted
// contraction index, log-sum-exp merge by the last block to arrive), fed
// through a per-warp ring of TMA copies and cut over the grid by work rather
// than by head.
//
// Why a ring. The kernel is bound by HBM, and a B200 needs tens of kilobytes
// per SM in flight to cover DRAM latency. Loads that land in registers hold a
// register for every byte in flight; bulk tensor copies land in shared memory
// instead, so each warp keeps two whole 32-key blocks (K 8 KB + V 8 KB each
// at head_dim 128) in flight while it computes on a third. A warp owns its
// ring outright: there is no block-wide barrier in the key loop, only the
// ring's own mbarriers and __syncwarp.
//
// Why TMA. With one warp to a scheduler the loop runs at the speed of that
// warp's instruction stream, and half of that stream used to be the address
// arithmetic of thirty-two 16-byte asynchronous copies a lane per block. One
// lane now issues two tensor copies per block (the key rows as 64-byte
// column chunks, which also keeps the fragment reads free of bank conflicts;
// the value rows as they lie) and the warp spends its issue slots on the
// products. No multicast: every block fetches its own tiles.
//
// Why by work. One block per SM is resident (the ring is 192 KB), and a grid
// cut by (sequence, KV head) leaves SMs idle whenever their count does not
// divide 148. Instead all 128-key units of the launch are laid end to end,
// pair after pair, and block c takes a contiguous run of them (the host cuts
// the runs, see stream_partition). A block
// whose range covers a whole (sequence, KV head) pair writes its output
// directly; a range that cuts a pair writes a partial (o, m, l), and the last
// block of that pair to arrive merges (crates/llmtie-cuda/src/kernels.rs:
// 5779-5903 does the same with one counter a head).
//
// Needs 16-byte aligned value rows (capacity a multiple of 8); other caches
// take the register kernel in decode.cu.
#include "common.cuh"

#include <math_constants.h>

#include <algorithm>
#include <mutex>
#include <stdlib.h>
#include <string.h>

namespace {

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kRows = 8;
constexpr int kStages = 3;

__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Waits until a ring stage has landed. Bounded: after `limit` SM cycles it
// gives up and returns false (the copy engine never completed the stage).
__device__ __forceinline__ bool ring_wait(uint32_t bar, uint32_t parity, long long limit)
{
    if (mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t it = 1;; it++) {
        if (mbar_try(bar, parity)) return true;
        if ((it & 63u) == 0 && clock64() - t0 > limit) return false;
    }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar,
                                            int x, int y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
        "l"(map), "r"(bar), "r"(x), "r"(y)
        : "memory");
}
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

// Four 8 x 8 matrices of halves, one 16-byte row a lane; lane (g, c) receives
// row g, columns 2c and 2c + 1 of each.
__device__ __forceinline__ void ldmatrix4(uint32_t (&r)[4], uint32_t addr)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
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

__device__ __forceinline__ void split_pair(float x0, float x1, uint32_t &hi, uint32_t &lo)
{
    const __half h0 = __float2half_rn(x0), h1 = __float2half_rn(x1);
    const __half l0 = __float2half_rn(x0 - __half2float(h0));
    const __half l1 = __float2half_rn(x1 - __half2float(h1));
    hi = (uint32_t)__half_as_ushort(h0) | ((uint32_t)__half_as_ushort(h1) << 16);
    lo = (uint32_t)__half_as_ushort(l0) | ((uint32_t)__half_as_ushort(l1) << 16);
}

// The block whose run holds unit u: the largest c with ustart[c] <= u. The
// runs are strictly increasing, so it is unique.
__device__ __forceinline__ int block_of(const int *ustart, int u, int G)
{
    int lo = 0, hi = G - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (ustart[mid] <= u) {
            lo = mid;
        } else {
            hi = mid - 1;
        }
    }
    return lo;
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
        const float y = L > 0.0f ? O / L : 0.0f;
        p.out[at + d] = y;
        if (p.twin_q) emit_twin(p.twin_q, p.twin_s, at + d, y);   // whole warps get here
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
//
// The partials are brought into the (now idle) ring with asynchronous copies,
// every one of them in flight at once, so the merge costs one trip to L2
// however many blocks contributed; cp.async.cg reads L2, where the other
// blocks' stores are after their fences. Up to kMergeBatch contributors fit
// the ring at a time; more are folded in batch after batch under a running
// maximum.
template <int HD>
__device__ __noinline__ void merge_pair(const DecodeStreamParams &p, unsigned char *stage,
                                        const int *ustart, int pair_u0, int c_first, int c_last, int rows_here,
                                        long long ooff, unsigned xch_step)
{
    constexpr int SLOT = kRows * (HD + 2);            // floats of one partial slot
    constexpr int kMergeBatch = 32;
    constexpr int RSTEP = kThreads / HD;              // rows a pass of the block covers
    constexpr int RMAX = kRows / RSTEP;
    static_assert(kMergeBatch * SLOT * 4 <= kWarps * kStages * (32 * HD * 2 + HD * 64),
                  "a merge batch must fit the ring");
    const int tid = threadIdx.x;
    const int d = tid % HD;
    const int rg = tid / HD;
    const int chunks = (rows_here * (HD + 2) * 4 + 15) >> 4;   // 16-byte chunks a contributor
    const float *st = (const float *)stage;

    float Mx[RMAX], Ox[RMAX], Lx[RMAX];
#pragma unroll
    for (int i = 0; i < RMAX; i++) {
        Mx[i] = -CUDART_INF_F;
        Ox[i] = 0.0f;
        Lx[i] = 0.0f;
    }
    if (c_last - c_first < 4) {
        // Up to four contributors (the usual case): every load straight into
        // registers, all in flight together, and no pass through the ring.
        const int count = c_last - c_first + 1;
        const float *src[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int cc = min(c_first + e, c_last);
            const int sl = (ustart[cc] >= pair_u0) ? 0 : 1;
            src[e] = p.part + ((size_t)cc * 2 + sl) * SLOT;
        }
        float mi[RMAX][4], li[RMAX][4], oi[RMAX][4];
#pragma unroll
        for (int i = 0; i < RMAX; i++) {
            const int row = min(rg + i * RSTEP, rows_here - 1);
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float *pr = src[e] + row * (HD + 2);
                mi[i][e] = __ldcg(pr + HD);
                li[i][e] = __ldcg(pr + HD + 1);
                oi[i][e] = __ldcg(pr + d);
            }
        }
#pragma unroll
        for (int i = 0; i < RMAX; i++) {
            const int row = rg + i * RSTEP;
            if (row < rows_here) {
                float M = -CUDART_INF_F;
#pragma unroll
                for (int e = 0; e < 4; e++) M = fmaxf(M, mi[i][e]);   // repeats are harmless
                float O = 0.0f, L = 0.0f;
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    if (e < count) {
                        const float f = (mi[i][e] == -CUDART_INF_F) ? 0.0f : ex2(mi[i][e] - M);
                        O += f * oi[i][e];
                        L += f * li[i][e];
                    }
                }
                emit_value<HD>(p, ooff, xch_step, row, d, O, M, L);
            }
        }
        return;
    }
    for (int c0 = c_first; c0 <= c_last; c0 += kMergeBatch) {
        const int nb = min(kMergeBatch, c_last - c0 + 1);
        for (int idx = tid; idx < nb * chunks; idx += kThreads) {
            const int e = idx / chunks, ch = idx - e * chunks;
            const int cc = c0 + e;
            const int sl = (ustart[cc] >= pair_u0) ? 0 : 1;
            cp_async16(stage + ((size_t)e * SLOT * 4 + ch * 16),
                       p.part + ((size_t)cc * 2 + sl) * SLOT + ch * 4, 16);
        }
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();
#pragma unroll
        for (int i = 0; i < RMAX; i++) {
            const int row = rg + i * RSTEP;
            if (row < rows_here) {
                float bm = -CUDART_INF_F;
                for (int e = 0; e < nb; e++) bm = fmaxf(bm, st[e * SLOT + row * (HD + 2) + HD]);
                const float m_new = fmaxf(Mx[i], bm);
                const float keep = (Mx[i] == -CUDART_INF_F) ? 0.0f : ex2(Mx[i] - m_new);
                float O = Ox[i] * keep, L = Lx[i] * keep;
                for (int e = 0; e < nb; e++) {
                    const float *pr = st + e * SLOT + row * (HD + 2);
                    const float mi = pr[HD];
                    const float f = (mi == -CUDART_INF_F) ? 0.0f : ex2(mi - m_new);
                    O += f * pr[d];
                    L += f * pr[HD + 1];
                }
                Mx[i] = m_new;
                Ox[i] = O;
                Lx[i] = L;
            }
        }
        __syncthreads();   // the stage is free for the next batch
    }
#pragma unroll
    for (int i = 0; i < RMAX; i++) {
        const int row = rg + i * RSTEP;
        if (row < rows_here) emit_value<HD>(p, ooff, xch_step, row, d, Ox[i], Mx[i], Lx[i]);
    }
}

// The cross-rank half of a fused step: waits until every rank has delivered
// its triple of `pair` for this step into this rank's gather buffer (each
// rank raises the pair's flag after a system-wide fence), then merges the
// `world` triples of each of the pair's rows into xch_out, normalised. The
// wait is bounded (about a second); when it runs out the status word is set
// and the pair is left unmerged, so the launch still ends. `s_dead` is the
// block's own flag (shared memory, zero at the start of the block): once one
// wait of the block has run out, its later pairs are not waited for again.
template <int HD>
__device__ __noinline__ void cross_merge(const DecodeStreamParams &p, int pair, int row0,
                                         int rows_here, unsigned xch_step, int *s_dead)
{
    constexpr int RSTEP = kThreads / HD;
    const int tid = threadIdx.x;
    const int world = p.xch_world;
    const unsigned want = xch_step + 1u;
    __syncthreads();
    if (*(volatile int *)s_dead) return;
    if (tid < world) {
        const unsigned *f = p.xch_pflags[p.xch_rank] + (size_t)pair * world + tid;
        const long long t0 = clock64();
        while ((int)(ld_acquire_sys(f) - want) < 0) {
            if (clock64() - t0 > p.xch_wait_cycles) {
                *(volatile int *)s_dead = 1;
                report_timeout(p.xch_status, 70 + tid);
                break;
            }
        }
    }
    __syncthreads();
    if (*(volatile int *)s_dead) return;
    const float *buf =
        p.xch_gather[p.xch_rank] + (size_t)(xch_step & 1u) * world * p.xch_rank_stride;
    const int d = tid % HD;
    for (int row = tid / HD; row < rows_here; row += RSTEP) {
        float mi[LLMTIE_MAX_RANKS], li[LLMTIE_MAX_RANKS], oi[LLMTIE_MAX_RANKS];
#pragma unroll
        for (int r = 0; r < LLMTIE_MAX_RANKS; r++) {
            const int rr = min(r, world - 1);
            const float *pr = buf + (size_t)rr * p.xch_rank_stride +
                              (size_t)(row0 + row) * (HD + 2);
            mi[r] = __ldcg(pr + HD);
            li[r] = __ldcg(pr + HD + 1);
            oi[r] = __ldcg(pr + d);
        }
        float M = -CUDART_INF_F;
#pragma unroll
        for (int r = 0; r < LLMTIE_MAX_RANKS; r++) M = fmaxf(M, mi[r]);
        float O = 0.0f, L = 0.0f;
#pragma unroll
        for (int r = 0; r < LLMTIE_MAX_RANKS; r++) {
            if (r < world) {
                const float f = (mi[r] == -CUDART_INF_F) ? 0.0f : __expf(mi[r] - M);
                O += f * oi[r];
                L += f * li[r];
            }
        }
        p.xch_out[(size_t)(row0 + row) * HD + d] = L > 0.0f ? O / L : 0.0f;
    }
}

constexpr int kClusterMax = 8;   // blocks a pair at most (the portable cluster size)

template <int HD>
__global__ void __launch_bounds__(kThreads, 1)
decode_stream_kernel(const __grid_constant__ DecodeStreamParams p)
{
    constexpr int KI = HD / 32;
    constexpr int NT = HD / 8;
    constexpr int KBYTES = 32 * HD * 2;     // one 32-key block of keys
    constexpr int VBYTES = HD * 64;         // the same block of the transposed values
    constexpr int STAGE = KBYTES + VBYTES;
    constexpr int KSUB = 32 * 128;          // a sub-tile of the key block: 32 rows x 64 channels

    extern __shared__ unsigned char ring_raw[];
    // the 128-byte swizzle of the key tiles is a function of the address: the
    // ring starts on a 1024-byte boundary
    unsigned char *ring_all = ring_raw + ((1024u - (smem_u32(ring_raw) & 1023u)) & 1023u);
    __shared__ __align__(8) uint64_t sm_bar[kWarps][kStages];
    __shared__ __align__(16) float sm_o[kWarps][kRows][HD + 8];   // +8: rows 0-3 and 4-7 tile the banks
    __shared__ float sm_m[kWarps][kRows];
    __shared__ float sm_l[kWarps][kRows];
    __shared__ int sm_last;
    // Pairs by cluster. Two blocks a pair: both blocks' merged triples in the
    // leading block's slots, the peer's pushed there through distributed shared
    // memory. More blocks a pair: every block keeps its triple in its own
    // slot 0 and the leading block fetches them.
    __shared__ __align__(16) float sm_pair[2][kRows][HD + 2];
    __shared__ int sm_dead;                // a cross-rank wait of this block ran out
    constexpr int kMineMax = 16;
    __shared__ int sm_mine[kMineMax][3];   // pairs this block finished: pair, first row, rows
    int nmine = 0;                         // (the same in every thread)
    // The cut of the grid, out of the parameter bank (where every probe of a
    // search would be a cold miss) into shared memory once.
    __shared__ int sm_ustart[LLMTIE_STREAM_MAX_BLOCKS + 1];

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int g = lane >> 2;
    const int c = lane & 3;
    unsigned char *ring = ring_all + (size_t)warp * kStages * STAGE;
    const uint32_t ring_s = smem_u32(ring);
    // The warp's ring barriers: one a stage, completed by the bytes of the
    // stage's two copies. The stage and phase counters run on across the
    // segments of the block's run.
    const uint32_t bar0 = smem_u32(&sm_bar[warp][0]);
    if (lane == 0) {
        // one arrival a stage (the lane that announces the bytes), and where the
        // values come by cp.async one more of every lane, when its copies land
#pragma unroll
        for (int s = 0; s < kStages; s++) mbar_init(bar0 + 8u * s, p.v_plain ? 33u : 1u);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    uint32_t st_use = 0, ph_use = 0;   // the stage the next block is consumed from, its phase
    uint32_t st_put = 0;               // the stage the next copy goes to
    bool ring_ok = true;

    // When ranks exchange, the step number picks which of the two gather
    // buffers this launch fills; every block reads it before any block can
    // have finished the launch and advanced it.
    const unsigned xch_step = p.xch_world ? *(volatile const unsigned *)p.xch_step : 0u;
    // A kernel launched as this one's programmatic dependent (the merge of a
    // sharded step) may become resident from here on; it waits on flags, not
    // on this kernel's end.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (threadIdx.x == 0) sm_dead = 0;
    const int G = gridDim.x;
    const int u0 = p.ustart[blockIdx.x];
    const int u1 = p.ustart[blockIdx.x + 1];

    int u = u0;
    while (u < u1) {
        // ---- which pair this unit lies in, and how much of it is ours ---------
        int b = 0;
        while (b + 1 < p.nseq && u >= (int)p.unit0[b + 1]) b++;
        const int tk = p.seq[b].tk;
        const int cap = p.seq[b].cap;
        const int n_units = (tk + 127) >> 7;                 // units of one pair
        const int rel = u - (int)p.unit0[b];
        const int inner = rel / n_units;                     // rc * kv_heads + kh
        const int off = rel - inner * n_units;
        const int rc = inner / p.kv_heads;
        const int kh = inner % p.kv_heads;
        const int seg_end = min(n_units, off + (u1 - u));
        const int k_begin = off * 128;
        const int k_end = min(tk, seg_end * 128);
        const bool whole = (off == 0 && seg_end == n_units);
        const int pair_u0 = (int)p.unit0[b] + inner * n_units;
        const int pair = p.pair0[b] + inner;
        const int rows_here = min(kRows, p.rows - rc * kRows);

        float m = -CUDART_INF_F;
        float l = 0.0f;
        float o[NT][4];
#pragma unroll
        for (int j = 0; j < NT; j++) {
            o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;
        }

        // Copies block `blk` (32 keys) into the ring's next stage: the key rows
        // as HD/64 sub-tiles of [32 keys][128 bytes] (128-byte swizzle), the
        // value rows [HD][64 bytes] (64-byte swizzle): whole lines from memory,
        // and ldmatrix reads both without bank conflicts. Whatever lies past k_end comes along (the next keys of the
        // cache, its unused capacity, or zeros past its end) and is masked
        // where it is used.
        const CUtensorMap *kmap = &p.kmap[b];
        const CUtensorMap *vmap = &p.vmap[b];
        const int krow0 = kh * cap, vrow0 = kh * HD;
        const uint16_t *vsrc = (const uint16_t *)p.seq[b].v + (size_t)vrow0 * cap;
        auto issue = [&](int blk) {
            const uint32_t dst = ring_s + st_put * STAGE;
            const uint32_t bar = bar0 + 8u * st_put;
            if (lane == 0) {
                mbar_expect_tx(bar, p.v_plain ? KBYTES : STAGE);
#pragma unroll
                for (int kt = 0; kt < HD / 64; kt++) {
                    tma_load_2d(dst + kt * KSUB, kmap, bar, 64 * kt, krow0 + blk);
                }
                if (!p.v_plain) tma_load_2d(dst + KBYTES, vmap, bar, blk, vrow0);
            }
            if (p.v_plain) {
                // Eight lanes a channel row, 8 bytes (four keys) a lane, into the
                // layout the tensor map's 64-byte swizzle would have made: 16-byte
                // chunk c of row d at chunk c ^ ((d >> 1) & 3). Four keys are inside
                // the cache or outside it together (its capacity is a multiple of
                // four); outside, nothing is read and zeros are written.
                const int j = lane & 7;                          // which 8 bytes of the row
                const uint32_t bytes = (blk + 4 * j < cap) ? 8u : 0u;
#pragma unroll
                for (int i = 0; i < HD / 4; i++) {
                    const int d = 4 * i + (lane >> 3);
                    const uint32_t to = dst + KBYTES + (uint32_t)d * 64u +
                                        (uint32_t)(((j >> 1) ^ ((d >> 1) & 3)) << 4) +
                                        (uint32_t)(j & 1) * 8u;
                    const uint16_t *from = vsrc + (size_t)d * cap + blk + 4 * j;
                    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(to),
                                 "l"(bytes ? from : vsrc), "r"(bytes)
                                 : "memory");
                }
                asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar)
                             : "memory");
            }
            st_put = (st_put + 1 == kStages) ? 0u : st_put + 1;
        };

        // The query row goes out first, ahead of the ring's first copies in the
        // load pipe, and is consumed after them: the two latencies overlap.
        // (fragment layout of the m16n8k16 A operand: step s of sixteen channels,
        // this lane's columns 2c, 2c + 1 and 2c + 8, 2c + 9 of it)
        constexpr int KS = HD / 16;
        float qx[KS][4];
        {
            const float *qrow = p.q + (long long)b * p.q_seq + (long long)kh * p.q_kv +
                                (long long)(rc * kRows + g) * p.q_row;
            const bool live = g < rows_here;
#pragma unroll
            for (int ks_ = 0; ks_ < KS; ks_++) {
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int at = 16 * ks_ + 2 * c + 8 * (e >> 1) + (e & 1);
                    qx[ks_][e] = live ? __ldg(qrow + at) * p.q_scale : 0.0f;
                }
            }
        }

        // This warp's blocks: k_begin + (warp + kWarps * i) * 32.
        const int first = k_begin + warp * 32;
        const int nblk = first < k_end ? (k_end - first + kWarps * 32 - 1) / (kWarps * 32) : 0;
#pragma unroll
        for (int s = 0; s < kStages - 1; s++) {
            if (s < nblk) issue(first + s * kWarps * 32);
        }
        // The cut goes into shared memory now, under the first copies' flight:
        // a lane an entry out of the parameter bank is a replay a lane. (Only
        // the merge of runs that share a pair looks it up - clusters do not -
        // and this segment's barriers order the stores before that.)
        if (u == u0 && !p.by_cluster) {
            for (int i = threadIdx.x; i <= G; i += kThreads) sm_ustart[i] = p.ustart[i];
        }

        // ---- query fragments, split hi / lo: a0 a2 carry the heads (rows 0-7 of
        // the operand), a1 a3 the remainders (rows 8-15) ---------------------------
        uint32_t qa[KS][4];
#pragma unroll
        for (int ks_ = 0; ks_ < KS; ks_++) {
            split_pair(qx[ks_][0], qx[ks_][1], qa[ks_][0], qa[ks_][1]);
            split_pair(qx[ks_][2], qx[ks_][3], qa[ks_][2], qa[ks_][3]);
        }
        // ldmatrix row addresses of this lane: matrix lane >> 3, row lane & 7
        const int lm = lane >> 3, li = lane & 7;

        for (int i = 0; i < nblk; i++) {
            // Start the copy two blocks ahead, into the stage the last
            // iteration finished with, then wait for this block's.
            {
                const int nx = i + kStages - 1;
                if (nx < nblk) issue(first + nx * kWarps * 32);
            }
            if (ring_ok && !ring_wait(bar0 + 8u * st_use, ph_use, p.wait_cycles)) {
                // The stage never landed: say so, and finish the run on
                // whatever the ring holds rather than wait again.
                ring_ok = false;
                if (lane == 0) report_timeout(p.status, 80 + warp);
            }

            const int blk = first + i * kWarps * 32;
            const unsigned char *ks = ring + st_use * STAGE;
            const unsigned char *vs = ks + KBYTES;
            if (++st_use == kStages) {
                st_use = 0;
                ph_use ^= 1u;
            }

            // ---- scores: four 8-key tiles ----------------------------------------
            // Tile T is keys 8T..8T+7 of the block; one ldmatrix brings 32
            // channels of them (four 8 x 8 matrices) for two MMAs.
            const uint32_t ks_s = smem_u32(ks), vs_s = smem_u32(vs);
            float t[4][2];
#pragma unroll
            for (int T = 0; T < 4; T++) {
                float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                const uint32_t krow = ks_s + (uint32_t)(8 * T + li) * 128u;
#pragma unroll
                for (int ii = 0; ii < KI; ii++) {
                    uint32_t r[4];
                    ldmatrix4(r, krow + (uint32_t)(ii >> 1) * KSUB +
                                     (uint32_t)(((4 * (ii & 1) + lm) ^ li) << 4));
                    mma16816(acc, qa[2 * ii][0], qa[2 * ii][1], qa[2 * ii][2], qa[2 * ii][3], r[0],
                             r[1]);
                    mma16816(acc, qa[2 * ii + 1][0], qa[2 * ii + 1][1], qa[2 * ii + 1][2],
                             qa[2 * ii + 1][3], r[2], r[3]);
                }
                const int k0 = blk + 8 * T + 2 * c;
                t[T][0] = (k0 < k_end) ? (acc[0] + acc[2]) * p.sl2 : -CUDART_INF_F;
                t[T][1] = (k0 + 1 < k_end) ? (acc[1] + acc[3]) * p.sl2 : -CUDART_INF_F;
            }

            // ---- online softmax over the block -------------------------------------
            float bm = -CUDART_INF_F;
#pragma unroll
            for (int T = 0; T < 4; T++) bm = fmaxf(bm, fmaxf(t[T][0], t[T][1]));
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
            // the probabilities of tiles 2u and 2u + 1 are the A operand of the
            // value product over keys 16u..16u+15
            uint32_t pa[2][4];
#pragma unroll
            for (int T = 0; T < 4; T++) {
                const float p0 = ex2(t[T][0] - m);
                const float p1 = ex2(t[T][1] - m);
                l += p0 + p1;
                split_pair(p0, p1, pa[T >> 1][2 * (T & 1)], pa[T >> 1][2 * (T & 1) + 1]);
            }

            // ---- context ---------------------------------------------------------------
            // Channel tile j is channels 8j..8j+7; one ldmatrix brings the block's
            // 32 keys of them: register x holds keys 8x + 2c and 8x + 2c + 1.
            const bool ragged = blk + 32 > k_end;
#pragma unroll
            for (int j = 0; j < NT; j++) {
                uint32_t r[4];
                const int d = 8 * j + li;
                ldmatrix4(r, vs_s + (uint32_t)d * 64u + (uint32_t)((lm ^ ((d >> 1) & 3)) << 4));
                if (ragged) {
                    // Capacity past the live keys may hold anything, and
                    // 0 * NaN is NaN: clear what lies beyond.
#pragma unroll
                    for (int x = 0; x < 4; x++) {
                        const int k0 = blk + 8 * x + 2 * c;
                        if (k0 >= k_end) {
                            r[x] = 0u;
                        } else if (k0 + 1 >= k_end) {
                            r[x] &= 0x0000ffffu;
                        }
                    }
                }
                mma16816(o[j], pa[0][0], pa[0][1], pa[0][2], pa[0][3], r[0], r[1]);
                mma16816(o[j], pa[1][0], pa[1][1], pa[1][2], pa[1][3], r[2], r[3]);
            }
            __syncwarp();   // every lane is done with this stage before it is refilled
        }

        // ---- the block's four warps merge through shared memory ----------------------
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        if (c == 0) {
            sm_m[warp][g] = m;
            sm_l[warp][g] = l;
        }
#pragma unroll
        for (int j = 0; j < NT; j++) {
            *reinterpret_cast<float2 *>(&sm_o[warp][g][8 * j + 2 * c]) =
                make_float2(o[j][0] + o[j][2], o[j][1] + o[j][3]);
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
            if (p.xch_fused) {
                // This pair's triple is on its way to every rank: raise the
                // pair's flag there, and remember the pair for the merge
                // this block owes it before it exits. One fence, by the
                // threads that raise the flags, after the barrier: it orders
                // every store the barrier ordered before it (the pattern of a
                // grid-wide barrier's arrival).
                __syncthreads();
                if (tid < p.xch_world) {
                    __threadfence_system();
                    *(volatile unsigned *)(p.xch_pflags[tid] + (size_t)pair * p.xch_world +
                                           p.xch_rank) = xch_step + 1u;
                }
                if (p.xch_fused == 2) return;      // a dependent kernel merges
                const int row0 = (int)(ooff / (HD + 2));
                if (nmine < kMineMax) {
                    if (tid == 0) {
                        sm_mine[nmine][0] = pair;
                        sm_mine[nmine][1] = row0;
                        sm_mine[nmine][2] = rows_here;
                    }
                    nmine++;
                } else {
                    cross_merge<HD>(p, pair, row0, rows_here, xch_step, &sm_dead);
                }
                return;
            }
            // One fence, by the thread that counts the pair, after the barrier:
            // it orders every store the barrier ordered before it.
            __syncthreads();
            if (tid == 0) {
                __threadfence_system();
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
            } else if (p.by_cluster > 2) {
                sm_pair[0][row][d] = O;
                if (d == 0) {
                    sm_pair[0][row][HD] = M;
                    sm_pair[0][row][HD + 1] = L;
                }
            } else if (p.by_cluster) {
                // into the leading block's shared memory, slot = this block's rank
                uint32_t crank;
                asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(crank));
                const uint32_t mine = smem_u32(&sm_pair[crank][row][0]);
                uint32_t there;
                asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(there) : "r"(mine));
                asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(there + 4u * d), "f"(O)
                             : "memory");
                if (d == 0) {
                    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(there + 4u * HD), "f"(M)
                                 : "memory");
                    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(there + 4u * (HD + 1)),
                                 "f"(L)
                                 : "memory");
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

        if (whole) pair_done();
        if (!whole && p.by_cluster > 2) {
            // ---- the cluster's blocks meet; each fetches and merges its share of the rows
            // (row r goes to block r mod C: the fetches of a pair's rows are spread
            // over the cluster instead of queueing in the leading block)
            asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
            asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
            uint32_t crank;
            asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(crank));
            {
                const int C = p.by_cluster;
                const int mine_n = (rows_here - (int)crank + C - 1) / C;     // rows crank, crank + C, ...
                for (int idx = tid; idx < mine_n * HD; idx += kThreads) {
                    const int row = (int)crank + (idx / HD) * C, d = idx % HD;
                    const uint32_t mine = smem_u32(&sm_pair[0][row][0]);
                    // every block's three words of this value are asked for at once
                    float mi[kClusterMax], li[kClusterMax], oi[kClusterMax];
#pragma unroll
                    for (int r = 0; r < kClusterMax; r++) {
                        uint32_t there;
                        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
                                     : "=r"(there)
                                     : "r"(mine), "r"((uint32_t)min(r, C - 1)));
                        asm volatile("ld.shared::cluster.f32 %0, [%1];"
                                     : "=f"(mi[r])
                                     : "r"(there + 4u * HD)
                                     : "memory");
                        asm volatile("ld.shared::cluster.f32 %0, [%1];"
                                     : "=f"(li[r])
                                     : "r"(there + 4u * (HD + 1))
                                     : "memory");
                        asm volatile("ld.shared::cluster.f32 %0, [%1];"
                                     : "=f"(oi[r])
                                     : "r"(there + 4u * d)
                                     : "memory");
                    }
                    float M = -CUDART_INF_F;
#pragma unroll
                    for (int r = 0; r < kClusterMax; r++) M = fmaxf(M, mi[r]);   // repeats are harmless
                    float O = 0.0f, L = 0.0f;
#pragma unroll
                    for (int r = 0; r < kClusterMax; r++) {
                        if (r < C) {
                            const float f = (mi[r] == -CUDART_INF_F) ? 0.0f : ex2(mi[r] - M);
                            O += f * oi[r];
                            L += f * li[r];
                        }
                    }
                    emit(row, d, O, M, L);
                }
            }
            // nobody's slot is reused (or goes away with its block) before it was
            // read; and every row of the pair is out before the pair is counted
            asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
            asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
            if (crank == 0) pair_done();
        } else if (!whole && p.by_cluster) {
            // ---- the cluster's two blocks meet; the leading one merges -------------------
            asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
            asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
            uint32_t crank;
            asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(crank));
            if (crank == 0) {
                for (int idx = tid; idx < rows_here * HD; idx += kThreads) {
                    const int row = idx / HD, d = idx % HD;
                    const float m0 = sm_pair[0][row][HD], m1 = sm_pair[1][row][HD];
                    const float M = fmaxf(m0, m1);
                    const float f0 = (m0 == -CUDART_INF_F) ? 0.0f : ex2(m0 - M);
                    const float f1 = (m1 == -CUDART_INF_F) ? 0.0f : ex2(m1 - M);
                    emit(row, d, f0 * sm_pair[0][row][d] + f1 * sm_pair[1][row][d], M,
                         f0 * sm_pair[0][row][HD + 1] + f1 * sm_pair[1][row][HD + 1]);
                }
                pair_done();
            }
        } else if (!whole) {
            // ---- the last block of this pair to arrive merges every partial -------------
            const int c_first = block_of(sm_ustart, pair_u0, G);
            const int c_last = block_of(sm_ustart, pair_u0 + n_units - 1, G);
            const int count = c_last - c_first + 1;
            __threadfence();
            __syncthreads();
            if (tid == 0) {
                const unsigned prev = atomicAdd(p.ctr + pair, 1u);
                sm_last = (prev == (unsigned)(count - 1));
            }
            __syncthreads();
            if (sm_last) {
                // No second fence: the merge reads the partials from L2 (ld.cg /
                // cp.async.cg), after the barrier that followed the counter's
                // answer, so it cannot see anything older than their fences.
                merge_pair<HD>(p, ring_all, sm_ustart, pair_u0, c_first, c_last, rows_here, ooff, xch_step);
                pair_done();
                if (tid == 0) p.ctr[pair] = 0u;   // at rest again for the next call
            }
        }
        // shared memory is reused by the next segment; what the merge wrote into
        // the ring is ordered before the copy engine's next writes to it
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncthreads();
        u += seg_end - off;
    }

    if (p.xch_fused) {
        // Count the block out (every block has read the step by the time the
        // last one is counted, and nothing reads it again before the next
        // launch, so the last one may advance it now, off the critical path);
        // then merge across the ranks the pairs this block finished.
        if (tid == 0) {
            const unsigned prev = atomicAdd(p.xch_done, 1u);
            if (prev == (unsigned)(G - 1)) {
                *p.xch_done = 0u;
                __threadfence();
                *(volatile unsigned *)p.xch_step = xch_step + 1u;
            }
        }
        for (int i = 0; i < nmine; i++) {
            cross_merge<HD>(p, sm_mine[i][0], sm_mine[i][1], sm_mine[i][2], xch_step, &sm_dead);
        }
    }
}

template <int HD>
constexpr int ring_bytes()
{
    return kWarps * kStages * (32 * HD * 2 + HD * 64) + 1024;   // + room to align the ring
}

const KernelReg reg_s128("attn_decode_h128_run", (const void *)decode_stream_kernel<128>);
const KernelReg reg_s64("attn_decode_h64_run", (const void *)decode_stream_kernel<64>);

}  // namespace

bool decode_tensor_maps(CUtensorMap *kmap, CUtensorMap *vmap, const void *k, const void *v,
                        int kv_heads, int cap, int hd)
{
    // keys: the rows of every kv head one after another; a box is 32 rows by 64
    // channels (whole 128-byte lines), swizzled by the row
    const uint64_t kd[2] = {(uint64_t)hd, (uint64_t)kv_heads * (uint64_t)cap};
    const uint64_t ks[1] = {(uint64_t)hd * 2};
    const uint32_t kb[2] = {64, 32};
    if (!llmtie_encode_tiled_f16(kmap, 2, k, kd, ks, kb, 128)) return false;
    if (!vmap) return true;
    // values: a row of `cap` keys per (kv head, channel); a box is hd rows by 32 keys
    const uint64_t vd[2] = {(uint64_t)cap, (uint64_t)kv_heads * (uint64_t)hd};
    const uint64_t vs[1] = {(uint64_t)cap * 2};
    const uint32_t vb[2] = {32, (uint32_t)hd};
    return llmtie_encode_tiled_f16(vmap, 2, v, vd, vs, vb, 64);
}

// Cuts the launch's units into one contiguous run a block.
//
// A block pays a fixed price for every (sequence, KV head) pair it touches -
// a drained ring to refill, a partial to publish, an arrival to count - worth
// a few units of streaming. A block whose run crosses from one pair into the
// next pays it twice, and the launch ends when the slowest block does. So the
// cut is even not in units but in units plus `ov` virtual ones at the head of
// every pair: a run that crosses a pair boundary swallows that pair's virtual
// units and carries that many fewer real ones.
int decode_work_grid(long long units, long long pairs, int sm_count)
{
    return (int)std::min<long long>(std::min(sm_count, LLMTIE_STREAM_MAX_BLOCKS),
                                    std::max<long long>(std::max<long long>(1, units / 4), pairs));
}

static void stream_partition(DecodeStreamParams &p, int hd, int grid)
{
    // (LLMTIE_B200_DECODE_OV overrides the count: a tuning switch)
    static const int ov_env = [] {
        const char *e = getenv("LLMTIE_B200_DECODE_OV");
        return e ? atoi(e) : -1;
    }();
    // Five units' worth measured best on long pairs (128 units each: 4-6 all
    // within a percent, 3 and 8 some 3 % slower); short pairs, where a run is
    // only a few units, do better with three.
    const long long pairs_all = std::max<long long>(1, (long long)p.nseq * p.kv_heads * p.row_chunks);
    const int credit = p.total_units / pairs_all >= 64 ? 5 : 3;
    const long long ov = (ov_env >= 0 ? ov_env : credit) * (hd == 128 ? 1 : 2);   // the same time at either width
    const int inner = p.kv_heads * p.row_chunks;
    const long long W = p.total_units;
    const long long V = W + ov * (long long)p.nseq * inner;
    bool ok = true;
    {
        int b = 0;
        for (int c = 0; c < grid; c++) {
            const long long v = (long long)c * V / grid;
            while (b + 1 < p.nseq && v >= p.unit0[b + 1] + ov * p.pair0[b + 1]) b++;
            const long long n = (p.seq[b].tk + 127) / 128;
            const long long rel = v - (p.unit0[b] + ov * p.pair0[b]);
            const long long i = rel / (n + ov);
            const long long r = rel % (n + ov);
            p.ustart[c] = (int)(p.unit0[b] + i * n + (r > ov ? r - ov : 0));
        }
        p.ustart[grid] = (int)W;
        for (int c = 0; c < grid; c++) ok = ok && p.ustart[c] < p.ustart[c + 1];
        ok = ok && p.ustart[0] == 0;
    }
    if (!ok) {
        for (int c = 0; c <= grid; c++) p.ustart[c] = (int)((long long)c * W / grid);
    }
}

extern "C" llmtie_status llmtie_decode_cut(const int32_t *tk, size_t batch, size_t kv_heads,
                                           size_t head_dim, int32_t sm_count, int32_t *ustart,
                                           size_t ustart_len, int32_t *grid_out)
{
    if (!tk || !ustart || !grid_out || batch == 0 || batch > LLMTIE_DECODE_MAX_SEQ ||
        kv_heads == 0 || sm_count < 1 || (head_dim != 64 && head_dim != 128)) {
        return llmtie_fail(LLMTIE_ERR_INVALID, "a malformed decode description");
    }
    DecodeStreamParams p;
    memset(&p, 0, sizeof(p));
    p.nseq = (int)batch;
    p.kv_heads = (int)kv_heads;
    p.row_chunks = 1;
    long long units = 0;
    for (size_t b = 0; b < batch; b++) {
        if (tk[b] <= 0) return llmtie_fail(LLMTIE_ERR_INVALID, "an empty context");
        p.seq[b].tk = tk[b];
        p.unit0[b] = units;
        p.pair0[b] = (int)(b * kv_heads);
        units += (long long)((tk[b] + 127) / 128) * (long long)kv_heads;
    }
    p.unit0[batch] = units;
    p.pair0[batch] = (int)(batch * kv_heads);
    p.total_units = units;
    if (units > 0x7fffffffLL) return llmtie_fail(LLMTIE_ERR_INVALID, "too many keys for one launch");
    const int grid = decode_work_grid(units, (long long)(batch * kv_heads), sm_count);
    if (ustart_len < (size_t)grid + 1) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %d in a buffer of %zu", grid + 1,
                           ustart_len);
    }
    stream_partition(p, (int)head_dim, grid);
    for (int c = 0; c <= grid; c++) ustart[c] = p.ustart[c];
    *grid_out = grid;
    return LLMTIE_OK;
}

static bool cluster_cut(DecodeStreamParams &p, const int *resident, int sm_count, int *grid);
static bool pair_cut(DecodeStreamParams &p, int hd, int sm_count, int *grid);

// The whole choice a launch makes, on the host (no device): the cut by work,
// a block a pair, or a cluster of 2, 4 or 8 blocks a pair. What the device
// would be asked - how many clusters of each size it holds at once - is an
// argument here.
extern "C" llmtie_status llmtie_decode_plan(const int32_t *tk, size_t batch, size_t kv_heads,
                                            size_t rows, size_t head_dim, int32_t sm_count,
                                            int32_t resident2, int32_t resident4,
                                            int32_t resident8, int32_t *ustart, size_t ustart_len,
                                            int32_t *grid_out, int32_t *blocks_a_pair_out)
{
    if (!tk || !ustart || !grid_out || !blocks_a_pair_out || batch == 0 ||
        batch > LLMTIE_DECODE_MAX_SEQ || kv_heads == 0 || rows == 0 || sm_count < 1 ||
        (head_dim != 64 && head_dim != 128)) {
        return llmtie_fail(LLMTIE_ERR_INVALID, "a malformed decode description");
    }
    DecodeStreamParams p;
    memset(&p, 0, sizeof(p));
    p.nseq = (int)batch;
    p.kv_heads = (int)kv_heads;
    p.row_chunks = (int)((rows + kRows - 1) / kRows);
    const int inner = p.kv_heads * p.row_chunks;
    long long units = 0;
    for (size_t b = 0; b < batch; b++) {
        if (tk[b] <= 0) return llmtie_fail(LLMTIE_ERR_INVALID, "an empty context");
        p.seq[b].tk = tk[b];
        p.unit0[b] = units;
        p.pair0[b] = (int)b * inner;
        units += (long long)((tk[b] + 127) / 128) * inner;
    }
    p.unit0[batch] = units;
    p.pair0[batch] = (int)batch * inner;
    p.total_units = units;
    if (units > 0x7fffffffLL) return llmtie_fail(LLMTIE_ERR_INVALID, "too many keys for one launch");
    int grid = decode_work_grid(units, (long long)batch * inner, sm_count);
    int resident[kClusterMax + 1] = {0};
    resident[2] = resident2;
    resident[4] = resident4;
    resident[8] = resident8;
    int mode = 0;
    if (cluster_cut(p, resident, sm_count, &grid)) {
        mode = p.by_cluster;
    } else if (pair_cut(p, (int)head_dim, sm_count, &grid)) {
        mode = 1;
    } else {
        stream_partition(p, (int)head_dim, grid);
    }
    if (ustart_len < (size_t)grid + 1) {
        return llmtie_fail(LLMTIE_ERR_SLICE_OVERRUN, "reading to %d in a buffer of %zu", grid + 1,
                           ustart_len);
    }
    for (int c = 0; c <= grid; c++) ustart[c] = p.ustart[c];
    *grid_out = grid;
    *blocks_a_pair_out = mode;
    return LLMTIE_OK;
}

// The ring needs more shared memory than a kernel gets unasked: once a device.
static void configure_decode_stream(int dev)
{
    static bool configured[64] = {false};
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaFuncSetAttribute(decode_stream_kernel<128>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, ring_bytes<128>());
        cudaFuncSetAttribute(decode_stream_kernel<64>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, ring_bytes<64>());
        configured[dev] = true;
    }
}

// How many clusters of `c` blocks of this kernel the device holds at once
// (a cluster needs its SMs in one GPC, so this is less than SMs / c); asked of
// the driver once per device, width and size.
static int resident_clusters(int dev, int hd, int c)
{
    static int memo[64][2][kClusterMax + 1];   // 0: not asked yet
    static std::mutex lock;
    if (dev < 0 || dev >= 64 || c < 1 || c > kClusterMax) return 0;
    std::lock_guard<std::mutex> hold(lock);
    int &slot = memo[dev][hd == 128 ? 1 : 0][c];
    if (slot == 0) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(c * 64);
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = hd == 128 ? ring_bytes<128>() : ring_bytes<64>();
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = c;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int n = 0;
        const cudaError_t e =
            hd == 128 ? cudaOccupancyMaxActiveClusters(&n, decode_stream_kernel<128>, &cfg)
                      : cudaOccupancyMaxActiveClusters(&n, decode_stream_kernel<64>, &cfg);
        slot = (e == cudaSuccess && n > 0) ? n : -1;
        if (e != cudaSuccess) cudaGetLastError();
    }
    return slot > 0 ? slot : 0;
}

extern "C" int32_t llmtie_decode_resident_clusters(llmtie_gpu *g, size_t head_dim, int32_t blocks)
{
    if (!g || (head_dim != 64 && head_dim != 128)) return 0;
    int dev = 0;
    cudaGetDevice(&dev);
    configure_decode_stream(dev);
    return resident_clusters(dev, (int)head_dim, blocks);
}

// Whether the launch goes pair by cluster: every sequence the same length, and
// either two blocks a pair filling at least four fifths of the SMs, with runs
// short enough (at most 256 units a block) for the launch's fixed costs to
// matter - a long launch is bound by HBM either way and does better on every
// SM - or, for a few short pairs (a few sequences of a few thousand keys,
// where the step is nothing but latency), as many blocks a pair - eight, four
// or two - as leaves every block a unit and all clusters resident at once.
static bool cluster_cut(DecodeStreamParams &p, const int *resident, int sm_count, int *grid)
{
    static const bool never = getenv("LLMTIE_B200_DECODE_NO_CLUSTER") != nullptr;
    const long long pairs = (long long)p.nseq * p.kv_heads * p.row_chunks;
    if (never) return false;
    int n = (p.seq[0].tk + 127) / 128, n_max = n;     // fewest and most units of a pair
    for (int b = 1; b < p.nseq; b++) {
        n = std::min(n, (p.seq[b].tk + 127) / 128);
        n_max = std::max(n_max, (p.seq[b].tk + 127) / 128);
    }
    const bool even = n == n_max;
    int C = 0;
    if (even && pairs * 2 <= sm_count && pairs * 2 * 5 >= (long long)sm_count * 4 && n >= 16 &&
        n <= 512) {
        C = 2;
    } else if (n_max <= 64) {
        // As many blocks as the device holds at once: one an SM at head_dim
        // 128, two at 64, where the ring is half the size (which shows in how
        // many clusters of two are resident).
        const long long room =
            std::min<long long>(LLMTIE_STREAM_MAX_BLOCKS, std::max(sm_count, 2 * resident[2]));
        // (sequences of unequal length: only while the longest run stays
        // short - eight units - since the clusters then end at different times)
        for (int c = kClusterMax; c >= 2 && C == 0; c >>= 1) {
            if (n >= c && pairs * c >= 32 && pairs * c <= room &&
                pairs <= resident[c] && (even || (n_max + c - 1) / c <= 8)) {
                C = c;
            }
        }
    }
    if (C == 0 || pairs * C > LLMTIE_STREAM_MAX_BLOCKS) return false;
    const int inner = p.kv_heads * p.row_chunks;
    for (int b = 0; b < p.nseq; b++) {
        const long long nb = (p.seq[b].tk + 127) / 128;
        for (int q = 0; q < inner; q++) {
            const long long at = (long long)(p.pair0[b] + q) * C;
            for (int i = 0; i < C; i++) {
                p.ustart[at + i] = (int)(p.unit0[b] + q * nb + (i * nb + C - 1) / C);
            }
        }
    }
    p.ustart[C * pairs] = (int)p.total_units;
    p.by_cluster = C;
    *grid = (int)(C * pairs);
    return true;
}

// Whether every pair simply gets a block of its own: pairs of one length,
// more of them than half the SMs (two blocks a pair do not fit), and short
// enough that a block walking its pair alone ends before the work cut's
// blocks would - those share the bytes over every SM, but a run that crosses
// from one pair into the next drains and refills its ring, and every pair
// ends with a merge through global memory (fence, arrival count, reload):
// about 8 us against a block a pair, measured on 128 pairs of 8 and 16 units.
// A block streams about 52 GB/s.
static bool pair_cut(DecodeStreamParams &p, int hd, int sm_count, int *grid)
{
    static const bool never = getenv("LLMTIE_B200_DECODE_NO_CLUSTER") != nullptr;
    const long long pairs = (long long)p.nseq * p.kv_heads * p.row_chunks;
    if (never || pairs > sm_count || pairs * 2 <= sm_count || pairs > LLMTIE_STREAM_MAX_BLOCKS) {
        return false;
    }
    const int n = (p.seq[0].tk + 127) / 128;
    for (int b = 1; b < p.nseq; b++) {
        if ((p.seq[b].tk + 127) / 128 != n) return false;
    }
    const double unit_us = (hd == 128 ? 65536.0 : 32768.0) / 52.0e3;     // a unit of one block
    if (n * unit_us * (1.0 - (double)pairs / sm_count) >= 8.0) return false;
    for (long long q = 0; q <= pairs; q++) p.ustart[q] = (int)(q * n);
    *grid = (int)pairs;
    return true;
}

cudaError_t launch_decode_stream(cudaStream_t st, const DecodeStreamParams &p_in, int hd, int grid)
{
    if (grid < 1 || grid > LLMTIE_STREAM_MAX_BLOCKS || p_in.total_units > 0x7fffffffLL ||
        p_in.total_units < grid) {
        return cudaErrorInvalidValue;
    }
    DecodeStreamParams p = p_in;
    p.by_cluster = 0;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    configure_decode_stream(dev);
    int resident[kClusterMax + 1] = {0};
    for (int c = 2; c <= kClusterMax; c <<= 1) resident[c] = resident_clusters(dev, hd, c);
    if (!cluster_cut(p, resident, sms, &grid) && !pair_cut(p, hd, sms, &grid)) {
        stream_partition(p, hd, grid);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = hd == 128 ? ring_bytes<128>() : ring_bytes<64>();
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = p.by_cluster ? p.by_cluster : 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = p.by_cluster ? 1 : 0;
    return hd == 128 ? cudaLaunchKernelEx(&cfg, decode_stream_kernel<128>, p)
                     : cudaLaunchKernelEx(&cfg, decode_stream_kernel<64>, p);
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
    sp.status = g->timeout_site;
    sp.wait_cycles = g->wait_cycles;
    // (making the tensor maps is arithmetic on the host: nothing is allocated)
    if (!decode_tensor_maps(&sp.kmap[0], &sp.vmap[0], k, v, (int)kv_heads, (int)cap,
                            (int)head_dim)) {
        return llmtie_fail(LLMTIE_ERR_DRIVER, "making the tensor maps of the caches");
    }
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
