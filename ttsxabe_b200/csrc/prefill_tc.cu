// Fused prefill attention on the 5th-generation tensor cores: TMA-staged K/V
// tiles, tcgen05.mma for both products with the accumulators in tensor
// memory, softmax in registers one thread a query row.
//
// Arithmetic is the reference's `flash_attn_impl`
// (crates/llmtie-cuda/src/kernels.rs:3078-3269): q rounded to f16, scores in
// f32, logits in log2 units, ex2, the normaliser from un-rounded
// probabilities, probabilities rounded to f16 into the value product, f32
// accumulation, O / l at the end. The one liberty is the running maximum: it
// is only moved when a tile's maximum exceeds it by more than 8 (in log2
// units), so probabilities are bounded by 2^8 rather than 1 - well inside f16
// - and the accumulator in tensor memory is rescaled only on those tiles.
//
// A block carries two query tiles of 128 rows that share their K/V tiles: two
// query heads of one KV group at the same positions (grouped models), or two
// consecutive row blocks of one head (ungrouped). Roles by warp:
//
//   warps 0-3   softmax of tile A: thread r owns row r (tensor-memory lane r)
//   warps 4-7   softmax of tile B
//   warp  8     TMA producer: K tile [128 keys][128] and V tile [128][128 keys]
//               per step, two stages each, 128-byte swizzle, no multicast
//   warps 10-11 idle (they complete the third warpgroup for setmaxnreg)
//   warp  9     MMA issuer: S_t = Q_t K^T (SS), O_t += P_t V (P from tensor
//               memory), in the order S_A S_B | PV_A S_A' PV_B S_B' | ... so
//               that one tile's softmax runs under the other tile's MMAs
//
// Tensor memory (512 columns): S_A [0,128) S_B [128,256) O_A [256,384)
// O_B [384,512); P_t overwrites the first 64 columns of S_t as packed f16.
// Both caches are K-major as they lie in memory (key rows for Q K^T, rows of
// the transposed value cache for P V), so both B operands come straight from
// TMA tiles with no transposition.
//
// Every wait on an mbarrier is bounded; a wait that runs out records its site
// in the handle's status word, the block drains and frees its tensor memory,
// and the host reports LLMTIE_ERR_TIMEOUT.
#include <cuda.h>

#include "common.cuh"

#include <math_constants.h>

#include <algorithm>
#include <functional>
#include <mutex>
#include <vector>
#include <stdio.h>
#include <stdlib.h>

namespace {

constexpr int BM = 128;            // query rows of a tile
constexpr int BN = 128;            // keys of a step
constexpr int kThreads = 384;   // three warpgroups: softmax A, softmax B, {TMA, MMA, idle, idle}
constexpr int SUB = 128 * 64 * 2;  // a swizzled Q or K sub-tile: 128 rows x 64 halves

// Shared-memory geometry at head width HD. Q and K tiles are [128][HD] in
// HD/64 sub-tiles of 128 x 64 halves; a V tile is [HD][128 keys] in two
// sub-tiles of HD x 64 halves.
template <int HD>
struct Geo {
    static constexpr int KT = HD / 64;
    static constexpr int TILE_QK = KT * SUB;
    static constexpr int SUBV = HD * 64 * 2;
    static constexpr int TILE_V = 2 * SUBV;
    static constexpr int SMEM = 2 * TILE_QK + 2 * TILE_QK + 2 * TILE_V + 1024;
};

enum Bar {
    Q_FULL = 0,    // +t
    K_FULL = 2,    // +stage
    K_EMPTY = 4,
    V_FULL = 6,
    V_EMPTY = 8,
    S_FULL = 10,   // +t
    P_FULL = 12,   // +t
    O_DONE = 14,   // +t
    S_FREE = 16,   // +t (head_dim 64 only)
    NBARS = 18
};

// ---- PTX wrappers -----------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// The waiting form: the thread is suspended by the hardware until the phase
// completes or a time limit of the hardware's own runs out (then: false), so a
// waiting warp takes no issue slots from the warp that shares its scheduler.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
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

// Bounded wait: a plain poll of the barrier's phase with no sleep of its own
// (nanosleep's granularity is far coarser than the few hundred nanoseconds a
// pipeline step lasts). The bound is a deadline in
// SM cycles, checked every 256 polls together with the block's abort flag.
// Returns false once the deadline passed or another role gave up; the caller
// then leaves its loop.
struct Waiter {
    volatile int *abort_flag;   // the block's own (shared memory)
    int *status;                // the handle's site word
    int *abort_epoch;           // the handle's word naming the launch that gave up
    int epoch;
    long long cycles;
};
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const Waiter &w, int site)
{
    if (mbar_try(bar, parity)) return true;
    const long long start = clock64();
    for (uint32_t it = 1;; it++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 15u) == 0) {
            if (*w.abort_flag) return false;
            if (clock64() - start > w.cycles) break;
        }
    }
    *w.abort_flag = 1;
    atomicExch(w.abort_epoch, w.epoch);
    report_timeout(w.status, site);
    return false;
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar,
                                            int x, int y, int z)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
        "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z)
        : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void mma_ss(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc)
{
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d),
        "l"(a), "l"(b), "r"(idesc), "r"(acc)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void mma_ts(uint32_t d, uint32_t a, uint64_t b, uint32_t idesc, uint32_t acc)
{
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
        "}\n" ::"r"(d),
        "r"(a), "l"(b), "r"(idesc), "r"(acc)
        : "memory");
}

// 32 consecutive columns of this thread's tensor-memory lane.
__device__ __forceinline__ void tmem_ld32(uint32_t addr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(addr)
        : "memory");
}
// Sixteen lanes by 64 columns in the accumulator-fragment layout: lane i of
// the warp gets, for each group j of eight columns, columns 8j + 2(i % 4) and
// the next of tensor-memory lane i / 4 (r[4j], r[4j + 1]) and of lane
// i / 4 + 8 (r[4j + 2], r[4j + 3]). Four lanes hold 32 consecutive bytes of a
// row, which is what makes a store straight from these registers whole sectors.
__device__ __forceinline__ void tmem_ld_16x256b_x8(uint32_t addr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.16x256b.x8.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(addr)
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t addr, const uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(addr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
        "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]),
        "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]),
        "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t addr, const uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(addr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
        "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float ex2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Three-input maximum and the packed two-float FMA / add of this architecture:
// the softmax is bound by how many instructions one warp per scheduler can
// issue, so each of these halves a part of its stream.
__device__ __forceinline__ float max3(float a, float b, float c)
{
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ uint64_t pack2(float lo, float hi)
{
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
    return d;
}
__device__ __forceinline__ void unpack2(uint64_t v, float &lo, float &hi)
{
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c)
{
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b)
{
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// Two floats to packed f16, x0 in the low half: one cvt.rn.f16x2.f32. (Two
// scalar conversions would each take a slot of the transcendental pipe, which
// is the pipe this kernel is bound by.)
__device__ __forceinline__ uint32_t pack_f16(float x0, float x1)
{
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(x1), "f"(x0));
    return r;
}

// Shared-memory matrix descriptor of a K-major, 128-byte-swizzled operand
// whose rows are 128 bytes: 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3ffffu) >> 4);   // start address
    d |= (uint64_t)1 << 16;                    // leading byte offset (unused when swizzled)
    d |= (uint64_t)(1024 >> 4) << 32;          // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                    // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                    // 128-byte swizzle
    return d;
}

// kind::f16 instruction descriptor: f16 x f16 -> f32, both operands K-major,
// M = 128, N = n.
__host__ __device__ constexpr uint32_t idesc_n(uint32_t n) { return (1u << 4) | ((n >> 3) << 17) | ((128u >> 4) << 24); }

struct Tile {
    int head;
    int r0;
    int n;   // key tiles it attends to (0: idle)
};

template <int HD>
__global__ void __launch_bounds__(kThreads, 1)
prefill_tc_kernel(const __grid_constant__ PrefillTcParams p)
{
    using G = Geo<HD>;
    constexpr int TILE_QK = G::TILE_QK, TILE_V = G::TILE_V, SUBV = G::SUBV, KT = G::KT;
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bars[NBARS];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag_s;
    volatile int *abort_flag = &abort_flag_s;
    const Waiter wt = {abort_flag, p.status, p.abort_epoch, p.epoch, p.wait_cycles};

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;

    // ---- which two tiles this block carries ------------------------------------------
    // which sequence and which of its row-block slots (0 = the longest rows)
    const uint32_t item = p.n_order ? p.order[blockIdx.y] : 0u;
    const int seq_i = p.n_order ? (int)((item >> 8) & 63u) : (int)blockIdx.z;
    const int slot_y = p.n_order ? (int)(item & 255u) : (int)blockIdx.y;
    const int pieces = p.n_order ? (int)(item >> 20) : 1;      // 1: the row block is whole
    const int piece = (int)((item >> 14) & 63u);
    const PrefillTcSeq sq = p.seq[seq_i];
    const int group = p.heads / p.kv_heads;
    const int row_blocks = (sq.tq + BM - 1) / BM;
    int kh, head_a, head_b, r0_a, r0_b;
    // blockIdx.x runs over the heads (neighbours share a KV head's tiles in L2),
    // blockIdx.y over the row blocks, longest rows first.
    if (!p.pair_rows) {
        const int pairs = group >> 1;
        kh = blockIdx.x / pairs;
        const int rb = row_blocks - 1 - slot_y;
        head_a = kh * group + 2 * (blockIdx.x % pairs);
        head_b = head_a + 1;
        r0_a = r0_b = rb * BM;
    } else {
        kh = blockIdx.x / group;
        const int rp = (row_blocks + 1) / 2 - 1 - slot_y;
        head_a = head_b = blockIdx.x;
        r0_a = 2 * rp * BM;
        r0_b = (2 * rp + 1) * BM;
    }
    const int all_keys = p.causal ? sq.past + sq.tq : sq.tk;
    auto tiles_of = [&](int r0) {
        if (r0 < 0 || r0 >= sq.tq) return 0;
        const int last = p.causal ? min(sq.past + r0 + BM, all_keys) : all_keys;
        return (last + BN - 1) / BN;
    };
    // The key tiles this block takes: all of the row block's, or piece `piece`
    // of `pieces` equal shares (both tiles see the same keys then: pieces are
    // only cut where the two tiles are two heads at the same rows).
    const int all_a = tiles_of(r0_a), all_b = tiles_of(r0_b);
    const int jbeg = pieces > 1 ? (piece * all_a) / pieces : 0;
    const int n_a = pieces > 1 ? ((piece + 1) * all_a) / pieces - jbeg : all_a;
    const int n_b = pieces > 1 ? n_a : all_b;
    auto n_of = [n_a, n_b](int t) { return t == 0 ? n_a : n_b; };
    const int n_max = max(n_a, n_b);
    if (n_max == 0) return;

    // ---- shared memory carve-up (1024-byte aligned for the swizzle) -------------------
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    // Addresses by arithmetic, not tables: a table indexed by a stage or tile
    // number that is not a compile-time constant would live in local memory.
    const uint32_t bar0 = smem_u32(&bars[0]);
    auto BAR = [bar0](int i) { return bar0 + 8u * (uint32_t)i; };
    auto q_smem = [base](int t) { return base + (uint32_t)t * TILE_QK; };
    auto k_smem = [base](int s) { return base + (uint32_t)(2 + s) * TILE_QK; };
    auto v_smem = [base](int s) { return base + (uint32_t)(4 * TILE_QK) + (uint32_t)s * TILE_V; };
    // Tensor memory: S_A, S_B (128 columns each), then O_A, O_B (HD each). At
    // head_dim 128 that is all 512 columns and P overwrites its S; at head_dim 64
    // the last 128 columns are free and P gets them, so that S of the next step
    // can be issued as soon as the softmax has read this step's S into registers
    // instead of after this step's P.V: the softmax then never waits for an MMA.
    constexpr bool kSplit = (HD == 64);
    auto s_col = [](int t) { return (uint32_t)t * 128u; };
    auto o_col = [](int t) { return 256u + (uint32_t)t * (uint32_t)HD; };
    auto p_col = [](int t) { return kSplit ? 384u + (uint32_t)t * 64u : (uint32_t)t * 128u; };

    if (tid == 0) {
        // a block that starts after a block of this same launch gave up does
        // nothing but allocate and free
        abort_flag_s = (*(volatile int *)p.abort_epoch == p.epoch) ? 1 : 0;
        // the softmax warpgroups arrive once per warp (lane 0 after a __syncwarp)
        mbar_init(BAR(Q_FULL + 0), 4);
        mbar_init(BAR(Q_FULL + 1), 4);
        for (int s = 0; s < 2; s++) {
            mbar_init(BAR(K_FULL + s), 1);
            mbar_init(BAR(K_EMPTY + s), 1);
            mbar_init(BAR(V_FULL + s), 1);
            mbar_init(BAR(V_EMPTY + s), 1);
            mbar_init(BAR(S_FULL + s), 1);
            mbar_init(BAR(P_FULL + s), 4);
            mbar_init(BAR(O_DONE + s), 1);
            mbar_init(BAR(S_FREE + s), 4);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 8) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(
                         smem_u32(&tmem_slot))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    const bool dead = abort_flag_s != 0;
    // a dependent kernel (the merge of cut row blocks) may be set up from here on
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // and where this launch is itself the dependent of the pre-pass that rotates
    // the keys into the caches and leaves the cosines and sines, nothing of that
    // kernel's is read before it has ended (a no-op in an ordinary launch)
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // The register file is split by role: a warp scheduler holds one warp of
    // each warpgroup, and 208 + 208 + 88 registers are the 3 x 168 per lane the block was launched with (asking for more would wait forever).
    if (warp < 8) {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
    } else {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 88;");
    }

    if (dead) {
        // nothing: fall through to the drain
    } else if (warp < 8) {
        // =========================== softmax warpgroups ===================================
        const int t = warp >> 2;
        Tile me;
        me.head = t == 0 ? head_a : head_b;
        me.r0 = t == 0 ? r0_a : r0_b;
        me.n = n_of(t);
        const int row = tid & 127;                       // query row in the tile = lane
        const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        if (me.n > 0) {
            // -- stage Q: f32 rows -> f16, scaled, into the swizzled K-major layout ------
            {
                const float *qh = p.q + (long long)sq.row0 * p.q_stride + me.head * HD;
                const int w = warp & 3;
                constexpr int LPR = HD / 4;        // lanes (of four floats each) per row
                constexpr int RPI = 32 / LPR;      // rows a warp covers per load
                const int sub_row = lane / LPR;
                const int col4 = lane % LPR;
                if (p.rope_tab) {
                    // RoPE on the way in: a lane takes four pairs of a row - its
                    // floats j..j+3 and their partners hd/2 further on - with the
                    // row's cosines and sines from the pre-pass's table, rotates
                    // them with the arithmetic of the stand-alone kernel (the same
                    // bits), and stores both halves.
                    constexpr int LPRr = HD / 8;        // lanes per row, each with both halves
                    constexpr int RPIr = 32 / LPRr;
                    const int sub = lane / LPRr, c = lane % LPRr;
                    const float *tab = p.rope_tab + (long long)sq.row0 * HD;
#pragma unroll
                    for (int rr0 = 0; rr0 < 32; rr0 += 4 * RPIr) {
                        float4 a[4], b[4], cs[4], sn[4];
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            const int r = 32 * w + rr0 + u * RPIr + sub;
                            a[u] = b[u] = cs[u] = sn[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                            if (me.r0 + r < sq.tq) {
                                const float *src = qh + (long long)(me.r0 + r) * p.q_stride + 4 * c;
                                const float *tr = tab + (long long)(me.r0 + r) * HD + 4 * c;
                                a[u] = __ldg((const float4 *)src);
                                b[u] = __ldg((const float4 *)(src + HD / 2));
                                cs[u] = __ldg((const float4 *)tr);
                                sn[u] = __ldg((const float4 *)(tr + HD / 2));
                            }
                        }
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            const int r = 32 * w + rr0 + u * RPIr + sub;
                            float lo[4], hi[4];
                            rope_rotate(a[u].x, b[u].x, cs[u].x, sn[u].x, lo[0], hi[0]);
                            rope_rotate(a[u].y, b[u].y, cs[u].y, sn[u].y, lo[1], hi[1]);
                            rope_rotate(a[u].z, b[u].z, cs[u].z, sn[u].z, lo[2], hi[2]);
                            rope_rotate(a[u].w, b[u].w, cs[u].w, sn[u].w, lo[3], hi[3]);
#pragma unroll
                            for (int hh = 0; hh < 2; hh++) {
                                const float *y = hh ? hi : lo;
                                const int cc = c + hh * LPRr;          // this half's float4 index
                                const uint32_t w0 = pack_f16(y[0] * p.q_scale, y[1] * p.q_scale);
                                const uint32_t w1 = pack_f16(y[2] * p.q_scale, y[3] * p.q_scale);
                                const int chunk = (cc & 15) >> 1;
                                const uint32_t dst = q_smem(t) + (uint32_t)(cc >> 4) * SUB +
                                                     (uint32_t)r * 128 +
                                                     (uint32_t)((chunk ^ (r & 7)) << 4) +
                                                     (uint32_t)(cc & 1) * 8;
                                asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(dst), "r"(w0),
                                             "r"(w1)
                                             : "memory");
                            }
                        }
                    }
                } else {
                // eight loads in flight at a time: one load per iteration
                // would serialise that many global-memory latencies
#pragma unroll
                for (int rr0 = 0; rr0 < 32; rr0 += 8 * RPI) {
                    float4 x[8];
#pragma unroll
                    for (int u = 0; u < 8; u++) {
                        const int r = 32 * w + rr0 + u * RPI + sub_row;
                        x[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (me.r0 + r < sq.tq) {
                            x[u] = __ldg((const float4 *)(qh + (long long)(me.r0 + r) * p.q_stride +
                                                          4 * col4));
                        }
                    }
#pragma unroll
                    for (int u = 0; u < 8; u++) {
                        const int r = 32 * w + rr0 + u * RPI + sub_row;
                        const uint32_t lo = pack_f16(x[u].x * p.q_scale, x[u].y * p.q_scale);
                        const uint32_t hi = pack_f16(x[u].z * p.q_scale, x[u].w * p.q_scale);
                        const int chunk = (col4 & 15) >> 1;
                        const uint32_t dst = q_smem(t) + (uint32_t)(col4 >> 4) * SUB +
                                             (uint32_t)r * 128 + (uint32_t)((chunk ^ (r & 7)) << 4) +
                                             (uint32_t)(col4 & 1) * 8;
                        asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(dst), "r"(lo), "r"(hi)
                                     : "memory");
                    }
                }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(BAR(Q_FULL + t));
            }

            const float sl2 = p.sl2;
            const float thr = 8.0f / sl2;      // how far a tile maximum may exceed the reference
            float m_ref = -CUDART_INF_F;       // in score units
            float l = 0.0f;
            const int my_pos = sq.past + me.r0 + row;   // causal: last key this row sees
            bool ok = true;

            for (int j = 0; j < me.n && ok; j++) {
                ok = mbar_wait(BAR(S_FULL + t), (uint32_t)(j & 1), wt, 10 + t);
                if (!ok) break;
                tc_fence_after();
                uint32_t s[4][32];
#pragma unroll
                for (int c = 0; c < 4; c++) tmem_ld32(lane_addr + s_col(t) + 32 * c, s[c]);
                tmem_wait_ld();
                if (kSplit) {
                    // S is in registers: its columns may take the next step's scores
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(BAR(S_FREE + t));
                }
                // With P apart, P.V of the previous step must be done before this
                // step rescales O or overwrites P: one barrier phase a step,
                // looked at as late as possible (the step's maxima come first).
                bool pv_done = !kSplit || j == 0;

                // -- mask the tiles that reach past what this row may see -----------------
                const int key0 = (jbeg + j) * BN;
                const int lim = (p.causal ? min(my_pos, all_keys - 1) : all_keys - 1) - key0;
                if (key0 + BN - 1 > (p.causal ? sq.past + me.r0 : all_keys - 1)) {
#pragma unroll
                    for (int c = 0; c < 4; c++) {
#pragma unroll
                        for (int i = 0; i < 32; i++) {
                            if (32 * c + i > lim) s[c][i] = __float_as_uint(-CUDART_INF_F);
                        }
                    }
                }

                // -- tile maximum, lazy move of the reference maximum ----------------------
                // four independent chains: one 128-long chain of dependent
                // maxima would cost more than the exponentials
                float mc[4];
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    mc[c] = fmaxf(__uint_as_float(s[c][0]), __uint_as_float(s[c][1]));
#pragma unroll
                    for (int i = 2; i < 32; i += 2) {
                        mc[c] = max3(mc[c], __uint_as_float(s[c][i]), __uint_as_float(s[c][i + 1]));
                    }
                }
                const float mt = fmaxf(fmaxf(mc[0], mc[1]), fmaxf(mc[2], mc[3]));
                if (j == 0) {
                    m_ref = mt;
                } else {
                    const bool move = mt > m_ref + thr;
                    if (__any_sync(0xffffffffu, move)) {
                        const float m_new = move ? mt : m_ref;
                        const float f = ex2((m_ref - m_new) * sl2);
                        // O may be rescaled in place once P.V of the previous step is
                        // complete. With P over S that is implied (this step's S was
                        // committed after it).
                        if (!pv_done) {
                            ok = mbar_wait(BAR(O_DONE + t), (uint32_t)((j - 1) & 1), wt, 22 + t);
                            if (!ok) break;
                            tc_fence_after();
                            pv_done = true;
                        }
#pragma unroll
                        for (int c = 0; c < HD / 32; c++) {
                            uint32_t o[32];
                            tmem_ld32(lane_addr + o_col(t) + 32 * c, o);
                            tmem_wait_ld();
#pragma unroll
                            for (int i = 0; i < 32; i++) {
                                o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
                            }
                            tmem_st32(lane_addr + o_col(t) + 32 * c, o);
                        }
                        tmem_wait_st();
                        l *= f;
                        m_ref = m_new;
                    }
                }

                if (!pv_done) {
                    ok = mbar_wait(BAR(O_DONE + t), (uint32_t)((j - 1) & 1), wt, 22 + t);
                    if (!ok) break;
                    tc_fence_after();
                }

                // -- probabilities: l from the un-rounded values, P rounded to f16 -----------
                const uint64_t sl2_2 = pack2(sl2, sl2);
                // (a row that has seen no key yet - possible in a piece that starts
                // past the row's last key - keeps probabilities of zero)
                const float neg = (m_ref == -CUDART_INF_F) ? 0.0f : -m_ref * sl2;
                const uint64_t neg_2 = pack2(neg, neg);
                uint64_t lc[4] = {0ull, 0ull, 0ull, 0ull};   // four pairs of partial sums
                // All 64 pairs first, the four stores to tensor memory after them:
                // a store fences the compiler's scheduling, and the more independent
                // pairs it may interleave, the better the latency of ex2 and of the
                // conversions is hidden (one warp has the scheduler almost to itself).
                uint32_t pk[4][16];
#pragma unroll
                for (int c = 0; c < 4; c++) {
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        const uint64_t x = fma2(pack2(__uint_as_float(s[c][2 * i]),
                                                      __uint_as_float(s[c][2 * i + 1])),
                                                sl2_2, neg_2);
                        float p0, p1;
                        unpack2(x, p0, p1);
                        p0 = ex2(p0);
                        p1 = ex2(p1);
                        lc[i & 3] = add2(lc[i & 3], pack2(p0, p1));
                        pk[c][i] = pack_f16(p0, p1);
                    }
                }
#pragma unroll
                for (int c = 0; c < 4; c++) tmem_st16(lane_addr + p_col(t) + 16 * c, pk[c]);
                {
                    float a0, a1, b0, b1;
                    unpack2(add2(lc[0], lc[1]), a0, a1);
                    unpack2(add2(lc[2], lc[3]), b0, b1);
                    l += (a0 + a1) + (b0 + b1);
                }
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(BAR(P_FULL + t));
            }

            // -- epilogue: O / l to global ------------------------------------------------
            if (ok) {
                ok = mbar_wait(BAR(O_DONE + t), kSplit ? (uint32_t)((me.n - 1) & 1) : 0u, wt, 20 + t);
            }
            if (ok) {
                tc_fence_after();
                // A piece leaves its rows un-normalised, with the maximum they
                // are relative to and their sum, for the merge.
                const bool part = pieces > 1;
                const float inv = part ? 1.0f : (l > 0.0f ? 1.0f / l : 0.0f);
                const long long ptile =
                    ((long long)p.pslot[blockIdx.y] * gridDim.x + blockIdx.x) * 2 + t;
                if (part) p.part_ml[ptile * BM + row] = make_float2(m_ref * sl2, l);
                const bool out16 = p.out_f16 && !part;
                const long long ostride = part ? HD : p.out_stride;      // elements
                const int esize = out16 ? 2 : 4;
                unsigned char *obase =
                    part ? (unsigned char *)(p.part_o + (ptile * BM + 32 * (warp & 3)) * HD)
                         : (unsigned char *)p.out +
                               ((long long)(sq.row0 + me.r0 + 32 * (warp & 3)) * p.out_stride +
                                me.head * HD) * esize;
                if (!out16) {
                    // f32 rows go out straight from the registers, read from tensor
                    // memory in the fragment layout: four lanes write the 32 bytes
                    // of a sector, a warp instruction eight rows of them. (A row's
                    // 1 / l lives in the lane that owns the row in the softmax's
                    // layout.)
                    const int fr = lane >> 2, fc = 2 * (lane & 3);
#pragma unroll
                    for (int half = 0; half < 2; half++) {
                        const int ra = 16 * half + fr, rb = ra + 8;      // rows within the warp's 32
                        const float inv_a = __shfl_sync(0xffffffffu, inv, ra);
                        const float inv_b = __shfl_sync(0xffffffffu, inv, rb);
                        const bool live_a = part || me.r0 + 32 * (warp & 3) + ra < sq.tq;
                        const bool live_b = part || me.r0 + 32 * (warp & 3) + rb < sq.tq;
                        float *pa = (float *)(obase + (long long)ra * ostride * 4) + fc;
                        float *pb = (float *)(obase + (long long)rb * ostride * 4) + fc;
#pragma unroll
                        for (int cg = 0; cg < HD / 64; cg++) {
                            uint32_t o[32];
                            tmem_ld_16x256b_x8(lane_addr + ((uint32_t)(16 * half) << 16) + o_col(t) +
                                                   64u * cg,
                                               o);
                            tmem_wait_ld();
#pragma unroll
                            for (int j = 0; j < 8; j++) {
                                if (live_a) {
                                    *(float2 *)(pa + 64 * cg + 8 * j) =
                                        make_float2(__uint_as_float(o[4 * j]) * inv_a,
                                                    __uint_as_float(o[4 * j + 1]) * inv_a);
                                }
                                if (live_b) {
                                    *(float2 *)(pb + 64 * cg + 8 * j) =
                                        make_float2(__uint_as_float(o[4 * j + 2]) * inv_b,
                                                    __uint_as_float(o[4 * j + 3]) * inv_b);
                                }
                            }
                        }
                    }
                } else {
                    // f16 rows: in that layout four lanes would write 16 bytes, half
                    // a sector. Each warp turns its 32 rows through shared memory
                    // instead - its quarter of the tile's Q, which no MMA reads any
                    // more - a thread writing its own row, and stores whole rows
                    // of RB bytes, a row per LPR lanes. 16-byte chunks are swizzled
                    // by the row so that neither side has bank conflicts.
                    constexpr int RB = HD * 2;                 // bytes of a row
                    constexpr int LPR = RB / 16;               // lanes to a row on the way out
                    constexpr int RPI = 32 / LPR;              // rows an instruction stores
                    const uint32_t scratch = q_smem(t) + (uint32_t)(warp & 3) * (32u * RB);
#pragma unroll
                    for (int c = 0; c < HD / 32; c++) {
                        uint32_t o[32];
                        tmem_ld32(lane_addr + o_col(t) + 32 * c, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            uint32_t v0 = pack_f16(__uint_as_float(o[8 * i]) * inv, __uint_as_float(o[8 * i + 1]) * inv);
                            uint32_t v1 = pack_f16(__uint_as_float(o[8 * i + 2]) * inv, __uint_as_float(o[8 * i + 3]) * inv);
                            uint32_t v2 = pack_f16(__uint_as_float(o[8 * i + 4]) * inv, __uint_as_float(o[8 * i + 5]) * inv);
                            uint32_t v3 = pack_f16(__uint_as_float(o[8 * i + 6]) * inv, __uint_as_float(o[8 * i + 7]) * inv);
                            const int k = 4 * c + i;   // 16-byte chunk of the row
                            const uint32_t dst = scratch + (uint32_t)lane * RB +
                                                 (uint32_t)((k ^ (lane & (LPR - 1))) << 4);
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst),
                                         "r"(v0), "r"(v1), "r"(v2), "r"(v3)
                                         : "memory");
                        }
                    }
                    __syncwarp();
                    const int k = lane % LPR;
#pragma unroll
                    for (int it = 0; it < 32 / RPI; it++) {
                        const int r = it * RPI + lane / LPR;
                        uint4 v;
                        const uint32_t src = scratch + (uint32_t)r * RB +
                                             (uint32_t)((k ^ (r & (LPR - 1))) << 4);
                        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                                     : "r"(src));
                        if (me.r0 + 32 * (warp & 3) + r < sq.tq) {
                            *(uint4 *)(obase + (long long)r * ostride * 2 + k * 16) = v;
                        }
                    }
                    __syncwarp();
                }
            }
            tc_fence_before();
        }
    } else if (warp == 8) {
        // =============================== TMA producer =======================================
        if (lane == 0) {
            const CUtensorMap *kmap = &p.kmap[seq_i];
            const CUtensorMap *vmap = &p.vmap[seq_i];
            for (int j = 0; j < n_max; j++) {
                const int s = j & 1;
                const uint32_t ph = (uint32_t)((j >> 1) & 1);
                if (!mbar_wait(BAR(K_EMPTY + s), ph ^ 1u, wt, 30)) break;
                mbar_expect_tx(BAR(K_FULL + s), TILE_QK);
#pragma unroll
                for (int kt = 0; kt < KT; kt++) {
                    tma_load_3d(k_smem(s) + kt * SUB, kmap, BAR(K_FULL + s), 64 * kt,
                                (jbeg + j) * BN, kh);
                }
                if (!mbar_wait(BAR(V_EMPTY + s), ph ^ 1u, wt, 31)) break;
                mbar_expect_tx(BAR(V_FULL + s), TILE_V);
                tma_load_3d(v_smem(s), vmap, BAR(V_FULL + s), (jbeg + j) * BN, 0, kh);
                tma_load_3d(v_smem(s) + SUBV, vmap, BAR(V_FULL + s), (jbeg + j) * BN + 64, 0, kh);
            }
        }
    } else if (warp == 9) {
        // ================================ MMA issuer =========================================
        if (lane == 0) {
            bool ok = true;
            for (int t = 0; t < 2 && ok; t++) {
                if (n_of(t) > 0) ok = mbar_wait(BAR(Q_FULL + t), 0u, wt, 40 + t);
            }
            // Descriptors are built once; a k-step of 16 halves (32 bytes) adds 2
            // to the start-address field, the second 64-wide sub-tile SUB >> 4.
            const uint64_t dq0 = smem_desc(q_smem(0)), dk0 = smem_desc(k_smem(0)),
                           dv0 = smem_desc(v_smem(0));
            constexpr uint64_t kQkStep = TILE_QK >> 4, kVStep = TILE_V >> 4;
            constexpr uint64_t kSubStep = SUB >> 4, kSubVStep = SUBV >> 4;
            constexpr uint32_t kIdescS = idesc_n(BN), kIdescPV = idesc_n(HD);
            auto issue_s = [&](int t, int stage) {
                const uint64_t a = dq0 + (uint64_t)t * kQkStep;
                const uint64_t b = dk0 + (uint64_t)stage * kQkStep;
#pragma unroll
                for (int ks = 0; ks < HD / 16; ks++) {
                    const uint64_t off = (uint64_t)(ks >> 2) * kSubStep + (uint64_t)(ks & 3) * 2;
                    mma_ss(tmem + s_col(t), a + off, b + off, kIdescS, ks > 0 ? 1u : 0u);
                }
                tc_commit(BAR(S_FULL + t));
            };
            auto issue_pv = [&](int t, int stage, bool first, bool last) {
                const uint64_t b = dv0 + (uint64_t)stage * kVStep;
#pragma unroll
                for (int ks = 0; ks < BN / 16; ks++) {
                    const uint64_t off = (uint64_t)(ks >> 2) * kSubVStep + (uint64_t)(ks & 3) * 2;
                    mma_ts(tmem + o_col(t), tmem + p_col(t) + 8 * ks, b + off, kIdescPV,
                           (first && ks == 0) ? 0u : 1u);
                }
                if (last || kSplit) tc_commit(BAR(O_DONE + t));
            };
            if (ok) ok = mbar_wait(BAR(K_FULL + 0), 0u, wt, 42);
            if (ok) {
                tc_fence_after();
                for (int t = 0; t < 2; t++) {
                    if (n_of(t) > 0) issue_s(t, 0);
                }
                tc_commit(BAR(K_EMPTY + 0));
            }
            for (int j = 0; j < n_max && ok; j++) {
                const int s = j & 1;
                const uint32_t ph = (uint32_t)((j >> 1) & 1);
                bool k_ready = false;
                if (kSplit) {
                    // The next step's scores first, each as soon as its softmax
                    // has taken this step's out of tensor memory.
                    for (int t = 0; t < 2 && ok; t++) {
                        if (j + 1 < n_of(t)) {
                            ok = mbar_wait(BAR(S_FREE + t), (uint32_t)(j & 1), wt, 47 + t);
                            if (!ok) break;
                            if (!k_ready) {
                                ok = mbar_wait(BAR(K_FULL + (s ^ 1)),
                                               (uint32_t)(((j + 1) >> 1) & 1), wt, 44);
                                if (!ok) break;
                                k_ready = true;
                            }
                            tc_fence_after();
                            issue_s(t, s ^ 1);
                        }
                    }
                    if (!ok) break;
                    if (j + 1 < n_max) tc_commit(BAR(K_EMPTY + (s ^ 1)));
                }
                ok = mbar_wait(BAR(V_FULL + s), ph, wt, 43);
                if (!ok) break;
                for (int t = 0; t < 2 && ok; t++) {
                    if (j < n_of(t)) {
                        ok = mbar_wait(BAR(P_FULL + t), (uint32_t)(j & 1), wt, 45 + t);
                        if (!ok) break;
                        tc_fence_after();
                        issue_pv(t, s, j == 0, j == n_of(t) - 1);
                    }
                    if (!kSplit && j + 1 < n_of(t)) {
                        if (!k_ready) {
                            ok = mbar_wait(BAR(K_FULL + (s ^ 1)), (uint32_t)(((j + 1) >> 1) & 1),
                                           wt, 44);
                            if (!ok) break;
                            tc_fence_after();
                            k_ready = true;
                        }
                        issue_s(t, s ^ 1);
                    }
                }
                if (!ok) break;
                tc_commit(BAR(V_EMPTY + s));
                if (!kSplit && j + 1 < n_max) tc_commit(BAR(K_EMPTY + (s ^ 1)));
            }
        }
    }

    // ---- drain and free ----------------------------------------------------------------
    if (*abort_flag) {
        // Give copies and MMAs still in flight time to land before the shared
        // and tensor memory go back to the SM.
        for (int i = 0; i < 64; i++) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 8) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem) : "memory");
    }
}

typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                             const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                             const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn()
{
    static EncodeFn fn = [] {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &res) !=
                cudaSuccess ||
            res != cudaDriverEntryPointSuccess) {
            ptr = nullptr;
        }
        return (EncodeFn)ptr;
    }();
    return fn;
}

// A 3-d map over one cache: `inner` contiguous elements, `rows` rows `row_stride`
// elements apart, `planes` kv heads `plane_stride` elements apart; tiles of
// 64 x box_rows x 1 with the 128-byte swizzle. Reads past any extent return zero.
bool encode_map(CUtensorMap *map, const void *basep, uint64_t inner, uint64_t rows, uint64_t planes,
                uint64_t row_stride, uint64_t plane_stride, uint32_t box_rows)
{
    EncodeFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[3] = {inner, rows, planes};
    const cuuint64_t strides[2] = {row_stride * 2, plane_stride * 2};
    const cuuint32_t box[3] = {64, box_rows, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void *>(basep), dims, strides, box,
              estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// ---- merge of the pieces of cut row blocks -------------------------------------------
constexpr int kMergeGroups = 128;
struct PrefillMergeParams {
    PrefillMergeGroup group[kMergeGroups];
    int n_groups;
    const float *part_o;
    const float2 *part_ml;
    void *out;
    long long out_stride;
    int out_f16;
    int heads_per_x;          // a grid column of the attention kernel is two heads
    int grid_x;
    int row0[64], tq[64];     // per sequence
};

// Row r of head h of a cut row block: out = sum_p O_p 2^(m_p - M) / sum_p l_p 2^(m_p - M)
// over its pieces (crates/llmtie-cuda/src/kernels.rs:5836-5879 is the same
// algebra for decode). A warp takes one row, a lane four channels of it (HD
// 128) or two (HD 64); blockIdx = (row block, grid column x tile, 4-row slab).
// The loads of up to eight pieces are all issued before the first is used:
// the kernel is nothing but their latency.
template <int HD>
__global__ void __launch_bounds__(128) prefill_merge_kernel(const __grid_constant__ PrefillMergeParams p)
{
    constexpr int V = HD / 32;                 // channels a lane carries
    constexpr int kBatch = 8;
    // (launched as the attention kernel's programmatic dependent: nothing of
    // that kernel's may be read before it has ended)
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const PrefillMergeGroup g = p.group[blockIdx.x];
    const int x = blockIdx.y >> 1, t = blockIdx.y & 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = x * p.heads_per_x + t;
    const int rbs = (p.tq[g.seq] + BM - 1) / BM;
    const int r0 = (rbs - 1 - g.slot) * BM;
    const int row = 4 * blockIdx.z + warp;
    if (r0 + row >= p.tq[g.seq]) return;
    const long long tile0 = ((long long)g.pslot0 * p.grid_x + x) * 2 + t;
    const long long tile_step = (long long)p.grid_x * 2;    // from one piece to the next
    float M = -CUDART_INF_F, L = 0.0f, acc[V];
#pragma unroll
    for (int e = 0; e < V; e++) acc[e] = 0.0f;
    for (int k0 = 0; k0 < g.pieces; k0 += kBatch) {
        float2 ml[kBatch];
        float o[kBatch][V];
#pragma unroll
        for (int k = 0; k < kBatch; k++) {
            const long long tile = tile0 + (long long)min(k0 + k, g.pieces - 1) * tile_step;
            ml[k] = __ldg(&p.part_ml[tile * BM + row]);
            const float *src = p.part_o + (tile * BM + row) * HD + V * lane;
            if constexpr (V == 4) {
                const float4 v = __ldg((const float4 *)src);
                o[k][0] = v.x; o[k][1] = v.y; o[k][2] = v.z; o[k][3] = v.w;
            } else {
                const float2 v = __ldg((const float2 *)src);
                o[k][0] = v.x; o[k][1] = v.y;
            }
        }
        float bm = M;
#pragma unroll
        for (int k = 0; k < kBatch; k++) bm = fmaxf(bm, ml[k].x);   // repeats are harmless
        const float keep = (M == -CUDART_INF_F) ? 0.0f : ex2(M - bm);
        L *= keep;
#pragma unroll
        for (int e = 0; e < V; e++) acc[e] *= keep;
#pragma unroll
        for (int k = 0; k < kBatch; k++) {
            if (k0 + k < g.pieces) {
                const float f = (ml[k].x == -CUDART_INF_F) ? 0.0f : ex2(ml[k].x - bm);
                L += f * ml[k].y;
#pragma unroll
                for (int e = 0; e < V; e++) acc[e] += f * o[k][e];
            }
        }
        M = bm;
    }
    const float inv = L > 0.0f ? 1.0f / L : 0.0f;
    const long long at = (long long)(p.row0[g.seq] + r0 + row) * p.out_stride + head * HD + V * lane;
    if (p.out_f16) {
        uint32_t *dst = (uint32_t *)((uint16_t *)p.out + at);
        dst[0] = pack_f16(acc[0] * inv, acc[1] * inv);
        if constexpr (V == 4) dst[1] = pack_f16(acc[2] * inv, acc[3] * inv);
    } else {
        float *dst = (float *)p.out + at;
        if constexpr (V == 4) {
            *(float4 *)dst = make_float4(acc[0] * inv, acc[1] * inv, acc[2] * inv, acc[3] * inv);
        } else {
            *(float2 *)dst = make_float2(acc[0] * inv, acc[1] * inv);
        }
    }
}

const KernelReg reg_tc("flash_attn_h_tc", (const void *)prefill_tc_kernel<128>);
const KernelReg reg_tc64("flash_attn_64_tc", (const void *)prefill_tc_kernel<64>);
const KernelReg reg_tcm("flash_attn_h_merge", (const void *)prefill_merge_kernel<128>);

}  // namespace

bool llmtie_encode_tiled_f16(CUtensorMap *map, int rank, const void *base, const uint64_t *dims,
                             const uint64_t *strides_bytes, const uint32_t *box, int swizzle_bytes)
{
    EncodeFn fn = encode_fn();
    if (!fn || rank < 1 || rank > 5) return false;
    cuuint64_t d[5], s[4];
    cuuint32_t b[5], e[5];
    for (int i = 0; i < rank; i++) {
        d[i] = dims[i];
        b[i] = box[i];
        e[i] = 1;
        if (i + 1 < rank) s[i] = strides_bytes[i];
    }
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, (cuuint32_t)rank, const_cast<void *>(base), d, s,
              b, e, CU_TENSOR_MAP_INTERLEAVE_NONE,
              swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
              : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                    : CU_TENSOR_MAP_SWIZZLE_NONE,
              CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool prefill_tc_eligible(const PrefillParams &p, int hd)
{
    if ((hd != 128 && hd != 64) || p.kv_f32) return false;
    if (p.nseq > LLMTIE_TC_MAX_SEQ) return false;
    if (((uintptr_t)p.q & 15u) != 0 || (p.q_stride & 3) != 0) return false;
    if (((uintptr_t)p.out & 15u) != 0 || (p.out_stride & (p.out_f16 ? 7 : 3)) != 0) return false;
    for (int b = 0; b < p.nseq; b++) {
        if (p.seq[b].cap % 8 != 0) return false;
        // (a sequence shorter than a tile is fine: a box may be wider than its
        // tensor, and what it reads past the live keys is zeros)
        if (((uintptr_t)p.seq[b].k & 15u) != 0 || ((uintptr_t)p.seq[b].v & 15u) != 0) return false;
    }
    return encode_fn() != nullptr;
}

cudaError_t launch_prefill_tc(cudaStream_t st, const PrefillParams &p, int hd, const WaitCtl &w)
{
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaFuncSetAttribute(prefill_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Geo<128>::SMEM);
        cudaFuncSetAttribute(prefill_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Geo<64>::SMEM);
        configured[dev] = true;
    }
    const uint64_t HD = (uint64_t)hd;
    PrefillTcParams tp;
    memset(&tp, 0, sizeof(tp));
    int max_tq = 0;
    for (int b = 0; b < p.nseq; b++) {
        const PrefillSeq &s = p.seq[b];
        const int live = p.causal ? s.past + s.tq : s.tk;
        tp.seq[b].row0 = s.row0;
        tp.seq[b].tq = s.tq;
        tp.seq[b].past = s.past;
        tp.seq[b].tk = live;
        // keys: [kv][cap][hd] -> inner hd, rows = live keys, planes = kv heads
        if (!encode_map(&tp.kmap[b], s.k, HD, (uint64_t)live, (uint64_t)p.kv_heads, HD,
                        (uint64_t)s.cap * HD, 128)) {
            return cudaErrorInvalidValue;
        }
        // values: [kv][hd][cap] -> inner = live keys, rows = hd, planes = kv heads
        if (!encode_map(&tp.vmap[b], s.v, (uint64_t)live, HD, (uint64_t)p.kv_heads,
                        (uint64_t)s.cap, (uint64_t)s.cap * HD, (uint32_t)hd)) {
            return cudaErrorInvalidValue;
        }
        max_tq = s.tq > max_tq ? s.tq : max_tq;
    }
    if (max_tq == 0) return cudaSuccess;
    tp.nseq = p.nseq;
    tp.q = p.q;
    tp.q_stride = p.q_stride;
    tp.out = p.out;
    tp.out_f16 = p.out_f16;
    tp.out_stride = p.out_stride;
    tp.heads = p.heads;
    tp.kv_heads = p.kv_heads;
    tp.causal = p.causal;
    tp.q_scale = p.q_scale;
    tp.sl2 = p.sl2;
    tp.rope_tab = p.rope_tab;
    tp.status = w.status;
    tp.abort_epoch = w.abort_epoch;
    tp.epoch = w.epoch;
    tp.wait_cycles = w.cycles;
    const int group = p.heads / p.kv_heads;
    tp.pair_rows = (group % 2 != 0) ? 1 : 0;
    const int row_blocks = (max_tq + BM - 1) / BM;
    dim3 grid;
    if (!tp.pair_rows) {
        grid = dim3(p.kv_heads * (group / 2), row_blocks, p.nseq);
    } else {
        grid = dim3(p.heads, (row_blocks + 1) / 2, p.nseq);
    }
    // Key tiles row-block slot y of sequence b attends to (0: no rows).
    auto tiles_of_slot = [&](int b, int y) {
        const PrefillSeq &s = p.seq[b];
        const int rbs = (s.tq + BM - 1) / BM;
        const int slots = tp.pair_rows ? (rbs + 1) / 2 : rbs;
        if (y >= slots) return 0;
        const int top = tp.pair_rows ? std::min(rbs, 2 * (slots - 1 - y) + 2)
                                     : rbs - y;          // row blocks up to and with it
        const int keys = p.causal ? s.past + std::min(s.tq, top * BM) : s.tk;
        return (keys + BN - 1) / BN;
    };
    // Whether to cut long row blocks into pieces of their key range. A causal
    // launch is a set of blocks of very unequal length (1 to tq/128 key
    // tiles); when there are too few of them for the SMs - a short sequence,
    // or one KV head's share of a long one - the longest block is the launch.
    // Pieces of at most `cut` tiles write partial results that a second
    // kernel merges. A piece is a block with a block's fixed costs (its
    // query tiles staged, first scores, epilogue: some five tile steps), so
    // the cut is chosen by playing the launch through: blocks go to the SMs
    // in grid order, longest first, each to the SM that is free first.
    int cut = 0;
    {
        static const bool never = getenv("LLMTIE_B200_NO_SPLIT") != nullptr;
        std::vector<int> lens;
        long long work = 0;
        int longest = 0;
        for (int b = 0; b < p.nseq; b++) {
            for (int y = 0;; y++) {
                const int n = tiles_of_slot(b, y);
                if (n == 0) break;
                lens.push_back(n);
                work += n;
                longest = std::max(longest, n);
            }
        }
        const int sms = std::max(1, w.sm_count);
        const double share = (double)work * grid.x / sms;
        if (!never && !tp.pair_rows && p.nseq <= 64 && longest >= 8 && longest > 1.25 * share) {
            constexpr double kBlockCost = 5.5;   // a block's fixed costs, in tile steps
            constexpr double kMergeCost = 5.0;   // the merge kernel, in tile steps
            auto makespan = [&](int c) {
                std::vector<int> items;
                for (int n : lens) {
                    const int pieces = (c > 0 && n > c) ? (n + c - 1) / c : 1;
                    for (int k = 0; k < pieces; k++) {
                        items.push_back(((k + 1) * n) / pieces - (k * n) / pieces);
                    }
                }
                if (items.size() > LLMTIE_TC_MAX_ORDER) return 1e30;
                std::sort(items.begin(), items.end(), std::greater<int>());
                std::vector<double> free_at(sms, 0.0);   // a heap of the SMs' finishing times
                auto later = std::greater<double>();
                for (int len : items) {
                    for (unsigned x = 0; x < grid.x; x++) {
                        std::pop_heap(free_at.begin(), free_at.end(), later);
                        free_at.back() += len + kBlockCost;
                        std::push_heap(free_at.begin(), free_at.end(), later);
                    }
                }
                return *std::max_element(free_at.begin(), free_at.end()) + (c > 0 ? kMergeCost : 0.0);
            };
            // The search costs a fraction of a millisecond of host time, and a
            // caller repeats the same shapes: the last answers are kept.
            struct Memo { long long work; int longest, gx, n, sms, cut; };
            static std::mutex memo_lock;
            static std::vector<Memo> memo;
            bool known = false;
            {
                std::lock_guard<std::mutex> hold(memo_lock);
                for (const Memo &m : memo) {
                    if (m.work == work && m.longest == longest && m.gx == (int)grid.x &&
                        m.n == (int)lens.size() && m.sms == sms) {
                        cut = m.cut;
                        known = true;
                    }
                }
            }
            if (!known) {
                double best = makespan(0);
                for (int c = (longest + 1) / 2; c >= 6; c -= (c > 24 ? 2 : 1)) {
                    const double t = makespan(c);
                    if (t < 0.95 * best && (cut == 0 || t < best)) {
                        best = t;
                        cut = c;
                    }
                }
                std::lock_guard<std::mutex> hold(memo_lock);
                if (memo.size() >= 64) memo.erase(memo.begin());
                memo.push_back({work, longest, (int)grid.x, (int)lens.size(), sms, cut});
            }
        }
    }
    static const bool tell = getenv("LLMTIE_B200_TELL_CUT") != nullptr;
    if (tell) fprintf(stderr, "prefill: row blocks cut at %d tiles\n", cut);
    std::vector<PrefillMergeGroup> groups;
    int n_pslots = 0;
    if (p.nseq > 1 || cut > 0) {
        // One grid row per (sequence, row-block slot, piece) that has work,
        // those with the most key tiles first over the whole launch, so that
        // the SMs' last blocks are the short ones.
        struct Item { int tiles, seq, slot, piece, pieces, pslot; };
        std::vector<Item> items;
        for (int b = 0; b < p.nseq; b++) {
            for (int y = 0;; y++) {
                const int n = tiles_of_slot(b, y);
                if (n == 0) break;
                const int pieces = (cut > 0 && n > cut) ? (n + cut - 1) / cut : 1;
                if (pieces > 1) groups.push_back({b, y, n_pslots, pieces});
                for (int k = 0; k < pieces; k++) {
                    const int len = ((k + 1) * n) / pieces - (k * n) / pieces;
                    items.push_back({len, b, y, k, pieces, pieces > 1 ? n_pslots + k : 0});
                }
                if (pieces > 1) n_pslots += pieces;
            }
        }
        if (!items.empty() && items.size() <= LLMTIE_TC_MAX_ORDER && n_pslots <= 65535) {
            std::stable_sort(items.begin(), items.end(),
                             [](const Item &a, const Item &b) { return a.tiles > b.tiles; });
            tp.n_order = (int)items.size();
            for (size_t i = 0; i < items.size(); i++) {
                tp.order[i] = ((uint32_t)items[i].pieces << 20) | ((uint32_t)items[i].piece << 14) |
                              ((uint32_t)items[i].seq << 8) | (uint32_t)items[i].slot;
                tp.pslot[i] = (uint16_t)items[i].pslot;
            }
            grid = dim3(grid.x, (unsigned)items.size(), 1);
        } else {
            groups.clear();
            n_pslots = 0;
        }
    }
    void *part = nullptr;
    if (n_pslots > 0) {
        const size_t tiles = (size_t)n_pslots * grid.x * 2;
        const size_t o_bytes = tiles * BM * (size_t)hd * sizeof(float);
        const size_t ml_bytes = tiles * BM * sizeof(float2);
        cudaError_t e;
        part = workspace_reserve(*w.part, o_bytes + ml_bytes, st, &e);
        if (!part) return e;
        tp.part_o = (float *)part;
        tp.part_ml = (float2 *)((char *)part + o_bytes);
    }
    cudaError_t err;
    {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = hd == 128 ? Geo<128>::SMEM : Geo<64>::SMEM;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = p.after_prepass ? 1 : 0;
        err = hd == 128 ? cudaLaunchKernelEx(&cfg, prefill_tc_kernel<128>, tp)
                        : cudaLaunchKernelEx(&cfg, prefill_tc_kernel<64>, tp);
    }
    if (part) {
        if (err == cudaSuccess) {
            // the row blocks that were cut: merge their pieces into the output
            PrefillMergeParams mp;
            memset(&mp, 0, sizeof(mp));
            mp.part_o = tp.part_o;
            mp.part_ml = tp.part_ml;
            mp.out = p.out;
            mp.out_stride = p.out_stride;
            mp.out_f16 = p.out_f16;
            mp.heads_per_x = 2;
            mp.grid_x = (int)grid.x;
            for (int b = 0; b < p.nseq; b++) {
                mp.row0[b] = p.seq[b].row0;
                mp.tq[b] = p.seq[b].tq;
            }
            for (size_t g0 = 0; g0 < groups.size() && err == cudaSuccess; g0 += kMergeGroups) {
                mp.n_groups = (int)std::min<size_t>(kMergeGroups, groups.size() - g0);
                for (int i = 0; i < mp.n_groups; i++) mp.group[i] = groups[g0 + i];
                const dim3 mg((unsigned)mp.n_groups, grid.x * 2, BM / 4);
                // A programmatic dependent of the attention kernel: its blocks are
                // set up while that kernel's last blocks still run, and wait for
                // its end (griddepcontrol.wait) before they read anything.
                cudaLaunchConfig_t cfg = {};
                cfg.gridDim = mg;
                cfg.blockDim = dim3(128);
                cfg.stream = st;
                cudaLaunchAttribute attr[1];
                attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
                attr[0].val.programmaticStreamSerializationAllowed = 1;
                cfg.attrs = attr;
                cfg.numAttrs = (g0 == 0) ? 1 : 0;
                err = hd == 128 ? cudaLaunchKernelEx(&cfg, prefill_merge_kernel<128>, mp)
                                : cudaLaunchKernelEx(&cfg, prefill_merge_kernel<64>, mp);
            }
        }
    }
    return err;
}
