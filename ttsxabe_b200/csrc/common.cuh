// Shared declarations for the llmtie_b200 library: the device handle, the
// launch bookkeeping every entry point goes through, and the host-callable
// launchers each kernel file exports to the C ABI in abi.cu.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <map>
#include <string>
#include <vector>

#include "../../include/llmtie_b200.h"

struct KprofEntry {
    uint64_t count = 0;
    double ms = 0.0;
};

// A device buffer the handle keeps between calls and only ever grows, so that
// a call which needs scratch memory allocates nothing once it is warm. Work
// on a handle is stream-ordered, so one call's use ends before the next's begins.
struct Workspace {
    void *ptr = nullptr;
    size_t bytes = 0;
};
// Returns at least `bytes` of it (null and *err set if the allocation failed).
void *workspace_reserve(Workspace &w, size_t bytes, cudaStream_t st, cudaError_t *err);

struct llmtie_gpu {
    int ordinal = 0;
    cudaStream_t stream = nullptr;
    bool owns_stream = false;
    int sm_count = 0;
    uint64_t launches = 0;
    bool kprof = false;
    std::map<std::string, KprofEntry> prof;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    // Where a bounded device wait that gave up leaves its site code: one word
    // of pinned host memory mapped into the device, so that the host reads it
    // after any stream synchronisation without a copy. `timeout_site` is the
    // device's view of the same word.
    int *timeout_host = nullptr;
    int *timeout_site = nullptr;
    // A device word holding the number (`epoch`) of the tensor-memory prefill
    // launch that gave up, zero at rest: blocks of that same launch that start
    // later leave at once; other launches are not affected.
    int *abort_epoch = nullptr;
    int epoch = 0;
    // How long a device-side wait may spin, in SM cycles (about a second).
    long long wait_cycles = 1ll << 31;
    // Every DecodeScratch made through this handle: their arrival counters
    // are cleared when a timeout is reported, since a launch that gave up may
    // have left them mid-count.
    std::vector<llmtie_decode_scratch *> scratches;
    Workspace ws_rope;   // the ragged prefill's table of cosines and sines (or its copy of q)
    Workspace ws_part;   // partial results of a prefill whose long row blocks were cut
    Workspace ws_kv16;   // f16 copies of the live keys of caches the tensor-memory prefill cannot map
};

// The caches a tensor map was made for: a map is made again only when one of
// these changes (a cache is reallocated on growth, not on every token).
struct DecodeMapKey {
    const void *k = nullptr;
    const void *v = nullptr;
    int cap = 0, kv_heads = 0, hd = 0;
    bool has_v = false;   // the value map was made too (it is not where the values come by cp.async)
};

struct llmtie_decode_scratch {
    float *part = nullptr;     // [pairs][splits][8][hd + 2]
    unsigned *ctr = nullptr;   // [pairs], zero at rest
    size_t part_floats = 0;
    size_t ctr_words = 0;
    // tensor maps of the caches this scratch was last used with, per sequence slot
    DecodeMapKey map_key[32];
    alignas(64) CUtensorMap kmap[32];
    alignas(64) CUtensorMap vmap[32];
};

// Sets the thread's error message and returns `code`.
llmtie_status llmtie_fail(llmtie_status code, const char *fmt, ...);

// Brackets one launch: counts it, and under kprof times it with events and
// charges it to `name` (what `launched()` does in the reference's device.rs).
struct LaunchScope {
    llmtie_gpu *g;
    const char *name;
    LaunchScope(llmtie_gpu *g_, const char *name_);
    // Checks the launch; returns LLMTIE_OK or a driver error.
    llmtie_status done();
};

// ---- launchers (defined beside their kernels) --------------------------------

// rope_cache.cu
void launch_rope(cudaStream_t st, float *x, long long off, const float *freq_div, int t,
                 int heads, int hd, float theta, int first);
struct RopeBatchSeq {
    uint16_t *kc;
    uint16_t *vc;
    int pos, cap;
    long long q_off, k_off, v_off;   // where this sequence's rows start in q, k and v
};
struct RopeBatchParams {
    RopeBatchSeq seq[32];
    int nseq;
    float *q;              // heads*hd floats at seq[b].q_off, rotated in place
    const float *k;        // kv_heads*hd floats at seq[b].k_off
    const float *v;        //   (q, k and v may be one allocation)
    const float *freq_div;
    int heads, kv_heads, hd;
    float theta;
};
void launch_rope_cache_batched(cudaStream_t st, const RopeBatchParams &p);
void launch_cache_append(cudaStream_t st, const float *src, long long src_off, void *dst,
                         int n, int kv_heads, int hd, int cap, int past, bool transposed,
                         bool f16);
void launch_cache_grow(cudaStream_t st, const void *src, void *dst, long long rows,
                       long long len, long long src_stride, long long dst_stride, int esize);
void launch_round_f16(cudaStream_t st, const float *src, uint16_t *dst, size_t n);
// the live keys of f32 (rounded) or f16 (re-strided) caches as f16 caches of
// capacity cap16 (a multiple of 8)
void launch_caches_to_f16(cudaStream_t st, const void *k, const void *v, bool src_f32,
                          uint16_t *k16, uint16_t *v16, int kv_heads, int hd, int cap, int cap16,
                          int live);
void launch_rope_gptj(cudaStream_t st, float *x, const float *inv_freq, int positions, int dim,
                      int rot_dim);
void launch_split_heads_f32(cudaStream_t st, const float *x, float *out, int t, int heads, int hd,
                            int cap, bool transposed);
// `layers` blocks of x f32 [t][heads*hd], x_layer elements apart (+ bias rows
// bias_layer apart, or null), into f16 caches out_layer apart: keys
// [heads][cap][hd] or, transposed, values [heads][hd][cap]. Positions past t
// are not written.
void launch_split_heads(cudaStream_t st, const float *x, long long x_layer, const float *bias,
                        long long bias_layer, uint16_t *out, long long out_layer, int layers, int t,
                        int heads, int hd, int cap, bool transposed);
// Whisper encoder staging: qkv f32 [t][3*heads*64] -> K f16 [heads][tp][64],
// V f16 [heads][64][tp] (tp = padded t), zero padded; `batch` utterances one
// after another in qkv, each with its K then V in the staging buffer.
void launch_rows_stage(cudaStream_t st, const float *qkv, uint16_t *k, uint16_t *v, int t,
                       int tp, int heads, int hd, int batch);

// decode.cu
#define LLMTIE_DECODE_MAX_SEQ 32
struct DecodeSeq {
    const uint16_t *k;
    const uint16_t *v;
    int tk;
    int cap;
};
struct DecodeParams {
    DecodeSeq seq[LLMTIE_DECODE_MAX_SEQ];
    const float *q;        // row r of (sequence b, kv head kh, row chunk rc) at
    long long q_seq;       //   q + b*q_seq + kh*q_kv + (rc*8 + r)*q_row
    long long q_kv;
    long long q_row;
    float *out;            // same addressing with its own strides
    long long out_seq;
    long long out_kv;
    long long out_row;
    float *part;           // partials [pair][split][8][hd + 2]
    unsigned *ctr;         // arrival counters [pair]
    int rows;              // query rows per kv head (all chunks together)
    int row_chunks;        // ceil(rows / 8)
    int kv_heads;
    int nseq;
    int span;              // keys per block of the grid, a multiple of 128
    int max_splits;        // grid.x
    int nb;                // 32-key sub-blocks a warp takes per step: 1, 2, 4 or 8
    int partial;           // write (o, m, l) un-normalised, row stride hd + 2
    float q_scale;         // scale when it goes on q, else 1
    float sl2;             // (scale on the scores, else 1) * log2(e)
    signed char *twin_q;   // int8 twin of the output, same indexing as out (or null)
    float *twin_s;         //   its scales, one per 32 outputs
};
#ifdef __CUDACC__
// Records that a bounded wait gave up at `site` (host-mapped word: a plain
// store and a system-wide fence; whichever site wins a race is as good).
__device__ __forceinline__ void report_timeout(int *site_word, int site)
{
    *(volatile int *)site_word = site;
    __threadfence_system();
}
// The rotation of one RoPE pair, with the roundings spelled out so that every
// kernel that rotates produces the same bits whatever the compiler would have
// contracted: the fused decode-step and ragged-prefill paths are held to bit
// equality with rope followed by an append.
__device__ __forceinline__ void rope_rotate(float a, float b, float cs, float sn, float &lo,
                                            float &hi)
{
    lo = __fmaf_rn(a, cs, -__fmul_rn(b, sn));
    hi = __fmaf_rn(b, cs, __fmul_rn(a, sn));
}
// Acquire load at system scope: the consumer's half of a flag another GPU
// raised after its own system-wide fence.
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned *p)
{
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// The int8 "twin" of one context element, quantize_q8's arithmetic on the row
// the block just produced (crates/llmtie-cuda/src/kernels.rs:5755-5773): the
// 32 lanes of the calling warp hold 32 consecutive elements of one scale group
// (idx a multiple of 32 at lane 0), code = rn(y * 127 / max|y|), scale =
// max|y| / 127. Every lane of the warp must call.
__device__ __forceinline__ void emit_twin(signed char *__restrict__ qa, float *__restrict__ asc,
                                          long long idx, float y)
{
    float mx = fabsf(y);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    const float d = mx * (1.0f / 127.0f);
    const float inv = d > 0.0f ? 1.0f / d : 0.0f;
    qa[idx] = (signed char)__float2int_rn(y * inv);
    if ((threadIdx.x & 31) == 0) asc[idx >> 5] = d;
}
#endif
// hd is 64 or 128. Returns the cudaError of the launch.
cudaError_t launch_decode_f16(cudaStream_t st, const DecodeParams &p, int hd);
// How many blocks of the decode kernel fit the device at once.
int decode_resident_blocks(int hd, int sm_count, int nb);
#define LLMTIE_MAX_RANKS 8
// decode_stream.cu: the same operands cut over the grid by work (see there).
#define LLMTIE_STREAM_MAX_BLOCKS 160
struct DecodeStreamParams {
    // Tensor maps of each sequence's caches (see decode_tensor_maps): keys as
    // [kv*cap][hd], values as [kv*hd][cap].
    alignas(64) CUtensorMap kmap[LLMTIE_DECODE_MAX_SEQ];
    alignas(64) CUtensorMap vmap[LLMTIE_DECODE_MAX_SEQ];
    DecodeSeq seq[LLMTIE_DECODE_MAX_SEQ];
    int ustart[LLMTIE_STREAM_MAX_BLOCKS + 1];     // block c takes units [ustart[c], ustart[c+1])
    long long unit0[LLMTIE_DECODE_MAX_SEQ + 1];   // first 128-key unit of each sequence
    int pair0[LLMTIE_DECODE_MAX_SEQ + 1];         // first (row chunk, kv head) pair of each
    long long total_units;
    const float *q;
    long long q_seq, q_kv, q_row;
    float *out;
    long long out_seq, out_kv, out_row;
    float *part;           // partials [block][2][8][hd + 2]
    unsigned *ctr;         // arrival counters [pair]
    int rows, row_chunks, kv_heads, nseq;
    int partial;
    float q_scale, sl2;
    // Exchange between ranks (xch_world > 0, partial mode): finished triples go
    // to slot [step & 1][xch_rank] of every rank's gather buffer instead of `out`.
    int xch_world, xch_rank;
    float *xch_gather[LLMTIE_MAX_RANKS];     // every rank's gather buffer, as mapped here
    unsigned *xch_flags[LLMTIE_MAX_RANKS];   // every rank's flag array [world]
    unsigned *xch_step;                      // this rank's step counter
    unsigned *xch_done;                      // pairs finished in this launch, zero at rest
    int xch_pairs;                           // pairs in this launch
    long long xch_rank_stride;               // floats one rank's triples take
    // Fused merge (xch_fused = 1): the block that finishes a pair on this rank
    // raises that pair's flag on every rank, and before it exits waits for the
    // other ranks' flags of the pair and merges it into xch_out, normalised.
    // xch_fused = 2: the flags only; a dependent kernel merges.
    int xch_fused;
    unsigned *xch_pflags[LLMTIE_MAX_RANKS];  // every rank's pair flags [pairs][world]
    float *xch_out;                          // [rows][hd], this rank's merged result
    int *xch_status;                         // set when a bounded wait gave up
    long long xch_wait_cycles;               // how long such a wait may spin
    signed char *twin_q;                     // int8 twin of the output (or null), as in DecodeParams
    float *twin_s;
    int *status;                             // set when a wait on the ring's barriers gave up
    long long wait_cycles;                   // how long such a wait may spin
    // Pairs by cluster (set by the launcher; 0 or the cluster's size: 2, 4 or
    // 8): every (sequence, KV head) pair is cut over the blocks of one
    // thread-block cluster, which merge through distributed shared memory; no
    // run crosses a pair, no partial goes through global memory.
    int by_cluster;
    // Value rows that are only 8-byte aligned (a capacity that is a multiple of
    // 4 but not of 8: no tensor map can be laid over them): the value blocks
    // come by 8-byte cp.async from the lanes instead, into the same swizzled
    // layout; the keys still come by TMA. vmap is not used then.
    int v_plain;
};
cudaError_t launch_decode_stream(cudaStream_t st, const DecodeStreamParams &p, int hd, int grid);
// Blocks of the cut by work: one per SM, never fewer than four units a block
// unless that is fewer blocks than pairs.
int decode_work_grid(long long units, long long pairs, int sm_count);
// The two tensor maps the ring kernel reads one sequence's caches through:
// keys [kv][cap][hd] seen as kv*cap rows (boxes of 32 rows x 128 bytes, 128-byte
// swizzle), values [kv][hd][cap] seen as kv*hd rows of `cap` (boxes of hd rows
// x 64 bytes, 64-byte swizzle): what ldmatrix reads without bank conflicts.
// Reads past the end return zero.
// (vmap may be null: the key map alone)
bool decode_tensor_maps(CUtensorMap *kmap, CUtensorMap *vmap, const void *k, const void *v,
                        int kv_heads, int cap, int hd);
// cuTensorMapEncodeTiled for f16 data, through the runtime's driver entry point.
bool llmtie_encode_tiled_f16(CUtensorMap *map, int rank, const void *base, const uint64_t *dims,
                             const uint64_t *strides_bytes, const uint32_t *box, int swizzle_bytes);
void launch_decode_f32(cudaStream_t st, const float *q, long long q_off, const float *k,
                       const float *v, float *out, long long out_off, int heads, int kv_heads,
                       int hd, int tk, int cap, float q_scale, float s_scale, float *part,
                       unsigned *ctr);
int decode_f32_splits(int tk);   // blocks a head of that launch (partials a head it needs)
void launch_lse_merge(cudaStream_t st, const float *parts_buf, int parts, int rows, int hd,
                      float *out);
// Waits (bounded) until every rank's flag has reached this rank's step, then
// merges the gather buffer the step filled.
void launch_lse_merge_wait(cudaStream_t st, const float *gather, const unsigned *flags,
                           const unsigned *step, int world, int rows, int hd, float *out,
                           int *status, long long wait_cycles);

// gemv_qkv.cu: the stacked attention projection of one row into q and the f32 caches.
cudaError_t launch_gemv_qkv_f16(cudaStream_t st, const float *a, const uint16_t *w, const float *qb,
                                const float *kb, const float *vb, int k, int d, int hd, int cap,
                                int pos, float *q, float *kc, float *vc);

// The merge of a step signalled pair by pair (see lse_merge_pairs_kernel);
// `early` launches it as a programmatic dependent of the kernel before it.
cudaError_t launch_lse_merge_pairs(cudaStream_t st, const float *gather, const unsigned *pflags,
                                   unsigned *mstep, int world, int rows, int rows_per_pair, int hd,
                                   float *out, int *status, long long wait_cycles, bool early);

// prefill_mma.cu
#define LLMTIE_PREFILL_MAX_SEQ 32
struct PrefillSeq {
    const void *k;         // [kv][cap][hd], f16 bits or f32
    const void *v;         // [kv][hd][cap]
    int row0;              // first row of this sequence in q and out
    int tq;                // query rows
    int past;              // positions already in the cache before them
    int cap;
    int tk;                // keys visible when not causal
    int pad_;
};
struct PrefillParams {
    PrefillSeq seq[LLMTIE_PREFILL_MAX_SEQ];
    int nseq;
    const float *q;        // row r, head h at q + r*q_stride + h*hd
    long long q_stride;
    void *out;             // f32 or f16, row stride out_stride
    long long out_stride;
    int heads, kv_heads;
    int causal;
    int kv_f32;            // caches are f32 (rounded to f16 on load)
    int out_f16;
    float q_scale;         // scale when it goes on q before rounding, else 1
    float sl2;             // (scale on the scores, else 1) * log2(e)
    const float *rope_tab; // tensor-memory kernel only: rotate q while staging it (see PrefillTcParams)
    int after_prepass;     // tensor-memory kernel only: launch as the programmatic dependent of the
                           // kernel before it in the stream (the pre-pass that writes rope_tab and the caches)
};
cudaError_t launch_prefill_mma(cudaStream_t st, const PrefillParams &p, int hd);

// prefill_tc.cu: the tensor-memory kernel for aligned f16 caches at head_dim 64 or 128.
#define LLMTIE_TC_MAX_SEQ 8
struct PrefillTcSeq {
    int row0, tq, past, tk;   // tk: keys the sequence holds (past + tq when causal)
};
#define LLMTIE_TC_MAX_ORDER 1024
struct PrefillTcParams {
    alignas(64) CUtensorMap kmap[LLMTIE_TC_MAX_SEQ];
    alignas(64) CUtensorMap vmap[LLMTIE_TC_MAX_SEQ];
    PrefillTcSeq seq[LLMTIE_TC_MAX_SEQ];
    int nseq;
    const float *q;
    long long q_stride;
    void *out;                // f32, or f16 when out_f16
    long long out_stride;
    int out_f16;
    int heads, kv_heads, causal;
    int pair_rows;            // pair two row blocks of one head instead of two heads of a group
    float q_scale, sl2;
    int *status;              // set to a site code when a bounded wait gives up
    int *abort_epoch;         // set to `epoch` then: later blocks of this launch leave at once
    int epoch;
    long long wait_cycles;    // how long a wait on a barrier may spin
    // The work of grid row blockIdx.y, longest first over the whole launch and
    // without the empty ones: a (sequence, row-block slot) or, where long row
    // blocks are cut so that a small launch still fills the device, one piece
    // of its key tiles. n_order == 0 means blockIdx.z is the sequence and
    // blockIdx.y the row block, whole.
    int n_order;
    uint32_t order[LLMTIE_TC_MAX_ORDER];   // pieces << 20 | piece << 14 | sequence << 8 | slot
    uint16_t pslot[LLMTIE_TC_MAX_ORDER];   // where a piece's partial result goes
    // Partial results of the pieces, merged by prefill_merge_kernel:
    // part_o [pslot][gridDim.x][2 tiles][128 rows][hd] f32, un-normalised,
    // part_ml [..][128 rows] (reference maximum in log2 units, sum).
    float *part_o;
    float2 *part_ml;
    // RoPE fused into the staging of q (or null: q arrives rotated): per packed
    // row, hd/2 cosines then hd/2 sines of the row's position.
    const float *rope_tab;
};
// One row block whose key tiles were cut into pieces: where its rows go.
struct PrefillMergeGroup {
    int seq, slot, pslot0, pieces;
};
bool prefill_tc_eligible(const PrefillParams &p, int hd);
// What a launch needs of the handle for its bounded waits.
struct WaitCtl {
    int *status;
    int *abort_epoch;
    int epoch;
    long long cycles;
    int sm_count;             // SMs of the device (decides whether long row blocks are cut)
    Workspace *part;          // where the pieces of cut row blocks leave their partial results
};
cudaError_t launch_prefill_tc(cudaStream_t st, const PrefillParams &p, int hd, const WaitCtl &w);

// rope_cache.cu: packed ragged sequences, RoPE on q (in place) and k (into
// the f16 K caches), v transposed into the f16 V caches.
struct VarlenSeq {
    uint16_t *k;
    uint16_t *v;
    int row0, n, past, cap;
};
struct VarlenParams {
    VarlenSeq seq[LLMTIE_PREFILL_MAX_SEQ];
    int nseq;
    int total;             // rows over all sequences
    float *q;              // [total][heads*hd], rotated in place (unless rope_tab)
    const float *k;        // [total][kv_heads*hd]
    const float *v;
    const float *freq_div;
    int heads, kv_heads, hd;
    float theta;
    // When set, q is left alone and the rows' cosines and sines are written
    // here instead ([total][hd]: hd/2 cosines, hd/2 sines), for the attention
    // kernel to rotate q with as it stages it; one launch instead of two.
    float *rope_tab;
};
void launch_varlen_rope_append(cudaStream_t st, const VarlenParams &p);

// Name -> kernel table behind llmtie_kernel_resources: each kernel file
// registers its entries from a static initialiser.
const void *llmtie_kernel_symbol(const char *name);
struct KernelReg {
    KernelReg(const char *name, const void *fn);
};

