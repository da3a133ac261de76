// All transformer blocks of one int4 decode step as ONE persistent kernel.
//
// A decode step of GPT-2 XL launched per operation is 7 kernels per block x 48 blocks, each a few
// microseconds of work behind a few microseconds of launch hand-over.  Here one cooperative grid (one
// thread block per SM) walks the whole depth.  Per transformer block (gpt2.rs:172-204):
//
//   LN1 | QKV GEMM | attention | out-projection GEMM | LN2 | FC GEMM | bias+GELU | MLP-projection GEMM
//
// with a grid-wide arrive/wait on a global counter between phases.  What the design buys:
//   * the packed int4 weight tiles never depend on activations, so the producer warp streams them
//     through a shared-memory ring of bulk async copies straight across the phase boundaries: HBM
//     stays busy while the grid synchronises;
//   * every GEMM phase is cut "stream-K": its (feature tile x 64-wide K block) units are dealt out
//     evenly over the blocks in one contiguous range each, a block accumulates each run of K blocks of
//     one feature tile in tensor memory (tcgen05.mma, weights dequantised into TMEM as the A operand,
//     activations written by loader warps into the 128-byte-swizzled B operand) and adds its partial
//     tile to an f32 buffer with L2 reductions.  The consumer of that buffer adds the bias: attention
//     finalises q, k, v (and appends k, v to the fp16 cache), the bias+GELU phase finalises the MLP
//     hidden layer; the two projections add straight into the f32 residual stream;
//   * the cached K/V rows of a block's (sequence, head) items are asked into L2 a few phases ahead,
//     and each attention warp streams its rows through its own ring of bulk copies.
//
// Every wait (mbarrier or grid counter) is bounded: when one runs out the block records a code in the
// device error word and every role walks the rest of its phase list without working, so that all
// block-level barriers are still reached, tensor memory is freed and the kernel returns.
//
// Replaces the per-operation launch structure of TransformerBlock::forward / Int4TransformerBlock::forward
// (crates/core/gpu-host/src/nn/models/gpt2.rs:249-288, 1284-1339) for decode steps of 3..256 rows.
#include <cuda.h>

#include <algorithm>

#include "device_utils.cuh"
#include "model.h"
#include "tc_ptx.cuh"

namespace pd {

constexpr int NG = 2;                         // dequant groups of four warps
constexpr int W_PROD = 0, W_MMA = 1, W_LD0 = 2, LD_WARPS = 1, W_DQ0 = W_LD0 + LD_WARPS, DQ_WARPS = 4 * NG;
constexpr int N_WARPS = W_DQ0 + DQ_WARPS;     // 11
constexpr int THREADS = 32 * N_WARPS;         // 352
constexpr int DQ_THREADS = 32 * DQ_WARPS;     // 256: dequant / epilogue / LayerNorm / attention / activation
constexpr int AREA_A = 128 * 1024;            // B-operand stages during GEMM phases, K/V rings during attention
constexpr int W_STAGE = TILE_BYTES + 256;     // packed tile + the 128 fp16 group scales of its rows
constexpr int NP = 16;                        // weight stages in flight
constexpr int ATT_NST = 2, ATT_ROWS = 32, ATT_STAGE = 2 * ATT_ROWS * 128, ATT_RING = ATT_NST * ATT_STAGE;
constexpr int MAX_REC = 32, REC_FLOATS = 66;  // partial (max, sum, out[64]) records of a block's split items
constexpr int BAR_BYTES = 1024;
constexpr int TRACE_PHASES = 32;              // phases (from the start of the kernel) a trace covers
constexpr int TRACE_EXTRA = 256 * TRACE_PHASES * 2 - 64; // first of 64 free-form stamp slots behind the per-block ones
constexpr int SMEM_BYTES = 1024 + AREA_A + NP * W_STAGE + BAR_BYTES + MAX_REC * REC_FLOATS * 4;
constexpr int TMEM_COLS = 512, TMEM_A0 = 256; // accumulator at column 0, dequantised weight stages from column 256
constexpr int LN_V = 2;                       // float4 per thread of a row held in registers: d <= 2048
static_assert(ATT_RING * DQ_WARPS <= AREA_A, "attention rings must fit the operand area");
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget exceeded");

enum : uint32_t { E_P_EMPTY = 0x201, E_P_FULL, E_AX_DQ, E_AX_LD, E_A_FULL, E_ACC, E_GRID, E_ATT };
enum { PH_LN1 = 0, PH_QKV, PH_ATT, PH_PROJ, PH_LN2, PH_FC, PH_ACT, PH_FCPROJ, PH_COUNT };

struct Layer {
    const uint8_t *tiles[4]; // qkv, proj, fc, fcproj: re-tiled packed weights
    const __half *scales[4]; // fp16 group scales [n_groups][n_pad]
    const float *bias[4];    // may be null
    const float *ln_g[2], *ln_b[2];
    __half *kc, *vc;         // this layer's cache [seq][head][cap][64]
};

struct alignas(64) Params {
    CUtensorMap tmap[3];     // fp16 activations as [rows, K] with [MB x 64] boxes, 128-byte swizzle: ln, att, hbuf
    const Layer *layers;
    int n_layer, M, d, H, cap, act, MB, ns_shift, att_G, group;
    float eps;
    int K[4], N[4], kb[4], nt[4], npad[4];
    const int *pos_ptr;
    float *x;          // residual stream [M, d] f32
    __half *ln;        // LayerNorm output [M, d]
    float *qkv_acc;    // [M, 3d] f32, zero at rest
    __half *att;       // attention output [M, d]
    float *fc_acc;     // [M, 4d] f32, zero at rest
    __half *hbuf;      // GELU(fc) [M, 4d]
    unsigned *bar;     // grid barrier counter, zero at launch
    uint32_t *dev_err;
    unsigned long long *prof;  // optional: nanoseconds block 0 spent per phase kind [PH_COUNT]
    unsigned long long *trace; // optional: [block][TRACE_PHASES][2] globaltimer stamps (inputs ready, arrival)
    int pf_items;      // (sequence, head) items whose cached rows are asked into L2 ahead of their phase
    long long grid_wait_cycles;
    int fault_block, fault_phase; // test hook: that block skips that arrival (-1: none)
};

__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_add_f32(float *p, float v) {
    asm volatile("red.global.add.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory");
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// Orders what this thread has observed through the generic proxy (other blocks' stores, acquired through
// the grid counter) before its later async-proxy operations (TMA loads of those bytes).
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
// 16-byte asynchronous copy global -> shared through L2 only (the source was written by other blocks
// during this kernel: no L1 copy may be used); src_bytes 0 writes zeros.
__device__ __forceinline__ void cp_async_16(uint32_t smem_dst, const void *gsrc, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_dst), "l"(gsrc), "r"(src_bytes) : "memory");
}
// Arrives on the mbarrier once every asynchronous copy this thread has issued so far has landed
// (the arrival is counted in the barrier's expected count).
__device__ __forceinline__ void cp_async_arrive(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
template <int THREADS_>
__device__ __forceinline__ void named_sync(int id) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "n"(THREADS_) : "memory");
}
__device__ __forceinline__ float f16_round(float v) { return __half2float(__float2half_rn(v)); }

// Waits until the grid counter has reached `target` (every block has finished the phases counted in
// it).  One lane polls; bounded by `limit` clock cycles, by another role of this block giving up and
// by another block having recorded an error.  Warp-uniform result.
__device__ __forceinline__ bool grid_wait(const unsigned *bar, unsigned target, volatile int *abort_flag,
                                          uint32_t *dev_err, long long limit) {
    bool ok = true;
    if ((threadIdx.x & 31) == 0) {
        if (*abort_flag) ok = false;
        else if ((int)(ld_acquire_u32(bar) - target) < 0) {
            const long long t0 = clock64();
            unsigned it = 0;
            while ((int)(ld_acquire_u32(bar) - target) < 0) {
                if (*abort_flag) { ok = false; break; }
                if ((++it & 31u) == 0 &&
                    (clock64() - t0 > limit || *reinterpret_cast<volatile uint32_t *>(dev_err) != 0u)) {
                    *abort_flag = 1;
                    atomicCAS(dev_err, 0u, (uint32_t)E_GRID);
                    ok = false;
                    break;
                }
                __nanosleep(20);
            }
        }
    }
    return __all_sync(0xffffffffu, ok);
}

__device__ __forceinline__ void half8_to_float(const uint4 &u, float (&f)[8]) {
    const __half2 *h = reinterpret_cast<const __half2 *>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 t = __half22float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}

constexpr float ATT_SCALE_LOG2E = 0.125f * 1.4426950408889634f;
constexpr float NEG_BIG = -1.0e30f;

// Online-softmax update of one lane group's state with up to 16 rows of a stage (rows base..base+15 of
// the stage, 4 per lane group; lane c of a group owns dims 8c..8c+7).
__device__ __forceinline__ void att_rows16(const uint4 *ks, const uint4 *vs, int base, int rows, int g, int c,
                                           const float (&qf)[8], float &m, float &l, float (&acc)[8]) {
    constexpr int R = 4;
    uint4 kr[R], vr[R];
    bool valid[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int row = base + r * 4 + g;
        valid[r] = row < rows;
        kr[r] = make_uint4(0, 0, 0, 0);
        vr[r] = kr[r];
        if (valid[r]) {
            kr[r] = ks[row * 8 + c];
            vr[r] = vs[row * 8 + c];
        }
    }
    float sc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        float kf[8];
        half8_to_float(kr[r], kf);
        float t = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) t = fmaf(qf[i], kf[i], t);
        sc[r] = t;
    }
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) {
#pragma unroll
        for (int r = 0; r < R; ++r) sc[r] += __shfl_xor_sync(0xffffffffu, sc[r], o);
    }
    float m_new = m;
#pragma unroll
    for (int r = 0; r < R; ++r)
        if (valid[r]) m_new = fmaxf(m_new, sc[r]);
    const float corr = exp2f(m - m_new);
    l *= corr;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] *= corr;
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const float p = valid[r] ? exp2f(sc[r] - m_new) : 0.0f;
        l += p;
        float vf[8];
        half8_to_float(vr[r], vf);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = fmaf(p, vf[i], acc[i]);
    }
    m = m_new;
}

__global__ void __launch_bounds__(THREADS, 1) decode_layers_kernel(const __grid_constant__ Params P) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ int abort_flag;
    __shared__ float ln_red[2][DQ_WARPS];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nblk = gridDim.x, blk = blockIdx.x;
    const int NS = 1 << P.ns_shift, MB = P.MB, M = P.M, d = P.d, H = P.H;
    const uint32_t X_BYTES = (uint32_t)MB * 128u;

    const uint32_t base = (tc::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *gen_base = smem_raw + (base - tc::smem_u32(smem_raw));
    const uint32_t S_A = base, S_W = base + AREA_A;
    uint32_t b = S_W + NP * W_STAGE;
    const uint32_t p_full = b;   b += NP * 8;
    const uint32_t p_empty = b;  b += NP * 8;
    const uint32_t a_full = b;   b += 8 * 8;
    const uint32_t ax_empty = b; b += 8 * 8;
    const uint32_t acc_full = b; b += 8;
    const uint32_t att_full = b; b += DQ_WARPS * ATT_NST * 8;
    const uint32_t tmem_slot = b; b += 8;
    float *rec = reinterpret_cast<float *>(gen_base + (S_W + NP * W_STAGE + BAR_BYTES - base));

    if (tid == 0) {
        abort_flag = 0;
        for (int i = 0; i < NP; ++i) {
            tc::mbar_init(p_full + 8 * i, 1);
            tc::mbar_init(p_empty + 8 * i, 4);  // the four warps of the dequant group that took the tile
        }
        for (int i = 0; i < 8; ++i) {
            tc::mbar_init(a_full + 8 * i, 5);   // one dequant group + the activation tile's expect_tx
            tc::mbar_init(ax_empty + 8 * i, 1); // tcgen05.commit
        }
        tc::mbar_init(acc_full, 1);
        for (int i = 0; i < DQ_WARPS * ATT_NST; ++i) tc::mbar_init(att_full + 8 * i, 1);
        tc::fence_mbar_init();
    }
    if (warp == W_LD0 && lane < 3) tc::prefetch_tmap(&P.tmap[lane]);
    if (warp == W_MMA) tc::tmem_alloc(tmem_slot, TMEM_COLS);
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(gen_base + (tmem_slot - base));
    const uint32_t tmem_a = tmem_base + TMEM_A0;
    int pos = *P.pos_ptr; // index of the row this step appends; rows 0..pos-1 are cached
    pos = max(0, min(pos, P.cap - 1));

    // this block's contiguous share of a phase's (feature tile, K block) units
    auto unit_range = [&](int g, int &u0, int &u1) {
        const long long U = (long long)P.nt[g] * P.kb[g];
        u0 = (int)(U * blk / nblk);
        u1 = (int)(U * (blk + 1) / nblk);
    };

    if (warp == W_PROD) {
        // ---- packed weight tiles + their scales: HBM -> shared memory ring, through every phase ----
        uint32_t i = 0;
        bool ok = true;
        for (int l = 0; l < P.n_layer && ok; ++l) {
            const Layer *Lp = P.layers + l;
            // cached rows of this layer's attention items -> L2 (they do not change during the step)
            if (P.pf_items > 0 && pos > 0) {
                for (int it = blk + nblk * lane; it < P.pf_items; it += nblk * 32) {
                    tc::bulk_prefetch_l2(Lp->kc + (size_t)it * P.cap * 64, (uint32_t)pos * 128u);
                    tc::bulk_prefetch_l2(Lp->vc + (size_t)it * P.cap * 64, (uint32_t)pos * 128u);
                }
            }
            __syncwarp();
            for (int g = 0; g < 4 && ok; ++g) {
                const uint8_t *tiles = Lp->tiles[g];
                const __half *scales = Lp->scales[g];
                const int kbg = P.kb[g], npad = P.npad[g];
                int u0, u1;
                unit_range(g, u0, u1);
                int nt = u0 / kbg, kb = u0 - nt * kbg;
                for (int u = u0; u < u1; ++u, ++i) {
                    const uint32_t s = i % NP;
                    if (i >= NP) {
                        ok = tc::mbar_wait(p_empty + 8 * s, ((i / NP) & 1) ^ 1, &abort_flag, P.dev_err, E_P_EMPTY);
                        if (!ok) break;
                    }
                    if (tc::elect_one()) {
                        const uint32_t dst = S_W + s * W_STAGE;
                        tc::mbar_expect_tx(p_full + 8 * s, W_STAGE);
                        tc::tma_load_1d(dst, tiles + ((size_t)nt * kbg + kb) * TILE_BYTES, TILE_BYTES, p_full + 8 * s);
                        tc::tma_load_1d(dst + TILE_BYTES, scales + (size_t)((kb * TILE_K) / P.group) * npad + nt * TILE_N,
                                        256, p_full + 8 * s);
                    }
                    __syncwarp();
                    if (++kb == kbg) { kb = 0; ++nt; }
                }
            }
        }
    } else if (warp == W_LD0) {
        // ---- activation tiles [MB rows x 64 k] of every unit through the tensor maps (zero fill past M),
        //      as soon as the phase that produces them is complete on every block ----
        uint32_t ti = 0;
        bool ok = true;
        for (int l = 0; l < P.n_layer && ok; ++l) {
            for (int g = 0; g < 4 && ok; ++g) {
                const int kbg = P.kb[g];
                const CUtensorMap *tm = &P.tmap[g == 0 || g == 2 ? 0 : g == 1 ? 1 : 2];
                int u0, u1;
                unit_range(g, u0, u1);
                if (u0 == u1) continue;
                // inputs of phase 2g+1 of this layer: every block has finished the 8l + 2g + 1 phases before it
                ok = grid_wait(P.bar, (unsigned)nblk * (unsigned)(8 * l + 2 * g + 1), &abort_flag, P.dev_err, P.grid_wait_cycles);
                if (!ok) break;
                fence_proxy_async_all();
                const bool dbg = P.trace && blk == 0 && lane == 0 && l == 1 && g == 2;
                if (dbg) P.trace[TRACE_EXTRA - 64 + 0] = globaltimer_ns();
                int kb = u0 % kbg;
                for (int u = u0; u < u1; ++u, ++ti) {
                    const uint32_t sa = ti & (NS - 1);
                    if (ti >= (uint32_t)NS) {
                        ok = tc::mbar_wait(ax_empty + 8 * sa, ((ti >> P.ns_shift) & 1) ^ 1, &abort_flag, P.dev_err, E_AX_LD);
                        if (!ok) break;
                    }
                    if (tc::elect_one()) {
                        tc::mbar_expect_tx(a_full + 8 * sa, X_BYTES);
                        tc::tma_load_2d(S_A + sa * X_BYTES, tm, kb * TILE_K, 0, a_full + 8 * sa);
                    }
                    __syncwarp();
                    if (++kb == kbg) kb = 0;
                }
                if (dbg) P.trace[TRACE_EXTRA - 64 + 1] = globaltimer_ns();
            }
        }
    } else if (warp == W_MMA) {
        // ---- MMA issue: per unit four K=16 MMAs (A from tensor memory, B from shared memory) ----
        const uint32_t idesc = tc::umma_idesc_f16(128, MB);
        const uint64_t bd0 = tc::umma_desc_sw128(S_A);
        uint32_t ti = 0;
        bool ok = true;
        for (int l = 0; l < P.n_layer && ok; ++l) {
            for (int g = 0; g < 4 && ok; ++g) {
                const int kbg = P.kb[g];
                int u0, u1;
                unit_range(g, u0, u1);
                const bool dbg = P.trace && blk == 0 && lane == 0 && l == 1 && g == 2;
                int dbg_n = 0;
                for (int u = u0; u < u1 && ok;) {
                    const int nt = u / kbg, k0 = u - nt * kbg, k1 = min(kbg, k0 + (u1 - u));
                    for (int kb = k0; kb < k1; ++kb, ++ti) {
                        const uint32_t sa = ti & (NS - 1);
                        ok = tc::mbar_wait(a_full + 8 * sa, (ti >> P.ns_shift) & 1, &abort_flag, P.dev_err, E_A_FULL);
                        if (!ok) break;
                        if (dbg && dbg_n < 14) P.trace[TRACE_EXTRA - 64 + 4 + dbg_n++] = globaltimer_ns();
                        tc::tc_fence_after_sync();
                        const uint64_t bd = bd0 + (uint64_t)((sa * X_BYTES) >> 4);
                        const uint32_t ad = tmem_a + sa * 32;
                        if (tc::elect_one()) {
                            tc::umma_f16_ts(tmem_base, ad, bd, idesc, kb != k0);
                            tc::umma_f16_ts(tmem_base, ad + 8, bd + 2, idesc, 1u);
                            tc::umma_f16_ts(tmem_base, ad + 16, bd + 4, idesc, 1u);
                            tc::umma_f16_ts(tmem_base, ad + 24, bd + 6, idesc, 1u);
                            tc::umma_commit(ax_empty + 8 * sa);
                        }
                        __syncwarp();
                    }
                    if (ok && tc::elect_one()) tc::umma_commit(acc_full); // this run of K blocks is complete
                    __syncwarp();
                    if (dbg && dbg_n < 14) P.trace[TRACE_EXTRA - 64 + 4 + dbg_n++] = globaltimer_ns();
                    u += k1 - k0;
                }
            }
        }
    } else {
        // ---- the eight worker warps: dequant + GEMM epilogue, LayerNorm, attention, activation ----
        const int wt = tid - W_DQ0 * 32, aw = wt >> 5; // 0..255, 0..7
        const int grp = wt >> 7, quad = warp & 3, row = quad * 32 + lane;
        const int g4 = lane >> 3, c8 = lane & 7; // attention: lane group, 16-byte column of a 128-byte row
        uint32_t ti = 0, segn = 0, att_issued = 0, att_consumed = 0;
        int dbg_n = 0;
        unsigned phases_done = 0;
        bool ok = true;
        unsigned long long t_last = 0;
        const bool prof_thread = P.prof && blk == 0 && wt == 0;
        if (prof_thread) t_last = globaltimer_ns();

        auto phase_end = [&](int kind) {
            named_sync<DQ_THREADS>(1);
            if (wt == 0) {
                if (P.trace && blk == 0 && phases_done == 13) P.trace[TRACE_EXTRA - 64 + 44] = globaltimer_ns();
                __threadfence();
                if (P.trace && blk == 0 && phases_done == 13) P.trace[TRACE_EXTRA - 64 + 45] = globaltimer_ns();
                if (!(blk == P.fault_block && (int)phases_done == P.fault_phase)) atomicAdd(P.bar, 1u);
                if (P.trace && phases_done < (unsigned)TRACE_PHASES)
                    P.trace[((size_t)blk * TRACE_PHASES + phases_done) * 2 + 1] = globaltimer_ns();
                if (prof_thread) {
                    const unsigned long long t = globaltimer_ns();
                    P.prof[kind] += t - t_last;
                    t_last = t;
                }
            }
            ++phases_done;
        };
        // One warp polls the grid counter for the block (a poll per warp of every block would queue more
        // than a thousand loads on one L2 line in front of the arrivals); the others meet it at a named
        // barrier and read the block's abort flag.
        auto wait_inputs = [&]() {
            if (aw == 0 && ok) ok = grid_wait(P.bar, (unsigned)nblk * phases_done, &abort_flag, P.dev_err, P.grid_wait_cycles);
            named_sync<DQ_THREADS>(4);
            if (*reinterpret_cast<volatile int *>(&abort_flag)) ok = false;
            if (P.trace && wt == 0 && phases_done < (unsigned)TRACE_PHASES)
                P.trace[((size_t)blk * TRACE_PHASES + phases_done) * 2] = globaltimer_ns();
        };

        // LayerNorm of the residual rows r = blk, blk + nblk, ... into the fp16 buffer: the whole block
        // works on one row (its 256 threads hold up to two float4 each), two block reductions (mean, then
        // the variance around it).  Scale and shift are fetched before the wait for the inputs.
        auto ln_phase = [&](const float *gam, const float *bet) {
            const int n4 = d >> 2;
            float4 gg[LN_V], bb[LN_V];
#pragma unroll
            for (int i = 0; i < LN_V; ++i) {
                const int j = wt + DQ_THREADS * i;
                gg[i] = bb[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (j < n4) {
                    gg[i] = __ldg(reinterpret_cast<const float4 *>(gam) + j);
                    bb[i] = __ldg(reinterpret_cast<const float4 *>(bet) + j);
                }
            }
            wait_inputs();
            for (int r = blk; r < M; r += nblk) { // block-uniform trip count: the named barriers below are safe
                const float4 *xr = reinterpret_cast<const float4 *>(P.x + (size_t)r * d);
                float4 v[LN_V];
                float s = 0.0f;
#pragma unroll
                for (int i = 0; i < LN_V; ++i) {
                    const int j = wt + DQ_THREADS * i;
                    v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (ok && j < n4) v[i] = __ldcg(xr + j);
                    s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
                }
                s = warp_sum(s);
                if (lane == 0) ln_red[0][aw] = s;
                named_sync<DQ_THREADS>(5);
                float tot = 0.0f;
#pragma unroll
                for (int w = 0; w < DQ_WARPS; ++w) tot += ln_red[0][w];
                const float mean = tot / (float)d;
                float q = 0.0f;
#pragma unroll
                for (int i = 0; i < LN_V; ++i) {
                    const int j = wt + DQ_THREADS * i;
                    if (j < n4) {
                        const float a0 = v[i].x - mean, a1 = v[i].y - mean, a2 = v[i].z - mean, a3 = v[i].w - mean;
                        q += (a0 * a0 + a1 * a1) + (a2 * a2 + a3 * a3);
                    }
                }
                q = warp_sum(q);
                if (lane == 0) ln_red[1][aw] = q;
                named_sync<DQ_THREADS>(6);
                float qt = 0.0f;
#pragma unroll
                for (int w = 0; w < DQ_WARPS; ++w) qt += ln_red[1][w];
                const float inv_std = rsqrtf(qt / (float)d + P.eps);
                __half *orow = P.ln + (size_t)r * d;
#pragma unroll
                for (int i = 0; i < LN_V; ++i) {
                    const int j = wt + DQ_THREADS * i;
                    if (ok && j < n4) {
                        __half2 lo = __floats2half2_rn((v[i].x - mean) * inv_std * gg[i].x + bb[i].x,
                                                       (v[i].y - mean) * inv_std * gg[i].y + bb[i].y);
                        __half2 hi = __floats2half2_rn((v[i].z - mean) * inv_std * gg[i].z + bb[i].z,
                                                       (v[i].w - mean) * inv_std * gg[i].w + bb[i].w);
                        *reinterpret_cast<uint2 *>(orow + 4 * j) =
                            make_uint2(*reinterpret_cast<uint32_t *>(&lo), *reinterpret_cast<uint32_t *>(&hi));
                    }
                }
            }
        };

        // Dequant side of a GEMM phase, then the epilogue of each run of K blocks: the partial
        // [M x 128] tile is added to `target` (leading dimension ld) with reductions at L2; the run that
        // starts at K block 0 also adds the bias when one is given.
        auto gemm_dq = [&](int g, float *target, int ld, const float *bias) {
            const int kbg = P.kb[g], Ng = P.N[g];
            int u0, u1;
            unit_range(g, u0, u1);
            // The grid counter only counts arrivals: it tells "every block has finished phase p" only if no
            // block arrives for phase p+1 before phase p is complete everywhere.  A block with units gets
            // that from its data (its MMAs need activations the loaders fetch after that wait); a block
            // without units has to wait here before it may arrive.
            if (u0 == u1) wait_inputs();
            for (int u = u0; u < u1;) {
                const int nt = u / kbg, k0 = u - nt * kbg, k1 = min(kbg, k0 + (u1 - u));
                const int n = nt * TILE_N + row;
                const bool n_ok = n < Ng;
                const float bv = (bias && k0 == 0 && n_ok) ? __ldg(bias + n) : 0.0f;
                for (int kb = k0; kb < k1; ++kb, ++ti) {
                    if (!ok || (int)(ti % NG) != grp) continue;
                    const uint32_t sp = ti % NP, sa = ti & (NS - 1);
                    ok = tc::mbar_wait(p_full + 8 * sp, (ti / NP) & 1, &abort_flag, P.dev_err, E_P_FULL);
                    if (!ok) continue;
                    const uint8_t *pk = gen_base + (S_W - base) + sp * W_STAGE;
                    const uint4 w0 = *reinterpret_cast<const uint4 *>(pk + row * 16);        // k  0..31 of the block
                    const uint4 w1 = *reinterpret_cast<const uint4 *>(pk + 2048 + row * 16); // k 32..63
                    const __half2 s2 = __half2half2(*reinterpret_cast<const __half *>(pk + TILE_BYTES + row * 2));
                    __syncwarp();
                    if (lane == 0) tc::mbar_arrive(p_empty + 8 * sp);
                    if (ti >= (uint32_t)NS) {
                        ok = tc::mbar_wait(ax_empty + 8 * sa, ((ti >> P.ns_shift) & 1) ^ 1, &abort_flag, P.dev_err, E_AX_DQ);
                        if (!ok) continue;
                    }
                    tc::tc_fence_after_sync();
                    const uint32_t a_addr = tmem_a + ((uint32_t)(quad * 32) << 16) + sa * 32;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint4 w = h ? w1 : w0;
                        const uint32_t wv[4] = {w.x, w.y, w.z, w.w};
                        uint32_t o[16];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            __half2 q[4];
                            unpack8_int4(wv[j], q);
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                __half2 r = __hmul2(q[e], s2);
                                o[4 * j + e] = *reinterpret_cast<uint32_t *>(&r);
                            }
                        }
                        tc::tmem_st_x16(a_addr + 16 * h, o);
                    }
                    tc::tmem_st_wait();
                    tc::tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) tc::mbar_arrive(a_full + 8 * sa);
                }
                // epilogue of this run
                const bool dbg = P.trace && blk == 0 && wt == 0 && phases_done == 13;
                if (dbg && dbg_n < 20) P.trace[TRACE_EXTRA - 64 + 20 + dbg_n++] = globaltimer_ns();
                if (ok) ok = tc::mbar_wait(acc_full, segn & 1, &abort_flag, P.dev_err, E_ACC);
                ++segn;
                if (dbg && dbg_n < 20) P.trace[TRACE_EXTRA - 64 + 20 + dbg_n++] = globaltimer_ns();
                if (ok) {
                    tc::tc_fence_after_sync();
                    const int cpg = MB / NG; // accumulator columns (token rows) per dequant group
                    for (int c0 = grp * cpg; c0 < (grp + 1) * cpg && c0 < M; c0 += 16) {
                        uint32_t v[16];
                        tc::tmem_ld_x16(tmem_base + ((uint32_t)(quad * 32) << 16) + c0, v);
                        if (n_ok) {
                            float *dst = target + (size_t)c0 * ld + n;
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                if (c0 + j < M) red_add_f32(dst + (size_t)j * ld, __uint_as_float(v[j]) + bv);
                        }
                    }
                    tc::tc_fence_before_sync();
                }
                if (dbg && dbg_n < 20) P.trace[TRACE_EXTRA - 64 + 20 + dbg_n++] = globaltimer_ns();
                named_sync<DQ_THREADS>(2); // every read of the accumulator is done before the next run overwrites it
                if (dbg && dbg_n < 20) P.trace[TRACE_EXTRA - 64 + 20 + dbg_n++] = globaltimer_ns();
                u += k1 - k0;
            }
        };

        // Decode attention of this block's (sequence, head) items it = blk + nblk*j.  An item's cached
        // rows are split into att_G parts of whole 16-row groups; part p of item j is sub-item j*G+p and
        // sub-items go round-robin to the eight warps.  The part that owns the end also finalises k and v
        // of the new position (bias, fp16), appends them to the cache and attends to them from registers.
        // The cached rows do not depend on this step, so each warp asks for its first stages before the
        // wait for the q/k/v accumulator.
        auto attention = [&](const Layer *Lp) {
            const int items = M * H, G = P.att_G;
            const int nj = items > blk ? (items - blk + nblk - 1) / nblk : 0, nsub = nj * G;
            const int chunk = ((pos + G - 1) / G + 15) & ~15;
            const float *bq = Lp->bias[0];
            const uint32_t ring = S_A + aw * ATT_RING;
            const uint8_t *ring_gen = gen_base + (ring - base);
            const bool stamp = P.trace && blk == 0 && aw == 0 && lane == 0 && phases_done == 10;
            int n_stamp = 0;
            auto mark = [&]() {
                if (stamp && n_stamp < 60) P.trace[TRACE_EXTRA + n_stamp++] = globaltimer_ns();
            };
            // producer cursor over the same sub-item sequence, skipping parts without cached rows
            int pi_sub = aw, pi_row = 0, pi_end = 0;
            auto pi_open = [&]() {
                while (pi_sub < nsub) {
                    const int p = pi_sub % G;
                    pi_row = min(p * chunk, pos);
                    pi_end = min(pos, p * chunk + chunk);
                    if (pi_row < pi_end) return;
                    pi_sub += DQ_WARPS;
                }
            };
            auto top_up = [&]() {
                while (att_issued - att_consumed < (uint32_t)ATT_NST && pi_sub < nsub) {
                    const uint32_t s = att_issued % ATT_NST;
                    if (lane == 0) {
                        const int rows = min(ATT_ROWS, pi_end - pi_row);
                        const int it = blk + nblk * (pi_sub / G);
                        const uint32_t bar = att_full + 8 * (aw * ATT_NST + s), dst = ring + s * ATT_STAGE;
                        const size_t off = ((size_t)it * P.cap + pi_row) * 64;
                        tc::mbar_expect_tx(bar, rows * 256);
                        tc::tma_load_1d(dst, Lp->kc + off, rows * 128, bar);
                        tc::tma_load_1d(dst + ATT_ROWS * 128, Lp->vc + off, rows * 128, bar);
                    }
                    ++att_issued;
                    pi_row += ATT_ROWS;
                    if (pi_row >= pi_end) { pi_sub += DQ_WARPS; pi_open(); }
                }
            };
            mark();
            if (ok) {
                pi_open();
                top_up();
            }
            wait_inputs();
            mark();
            for (int sidx = aw; sidx < nsub && ok; sidx += DQ_WARPS) {
                const int j = sidx / G, p = sidx - j * G, it = blk + nblk * j, sq = it / H, hh = it - sq * H;
                const int r0 = min(p * chunk, pos), r1 = min(pos, p * chunk + chunk);
                const bool owns_new = (p == G - 1);
                const float *qa = P.qkv_acc + (size_t)sq * 3 * d + hh * 64 + c8 * 8;
                float qf[8], kn[8], vn[8];
                {
                    const float4 a0 = __ldcg(reinterpret_cast<const float4 *>(qa)), a1 = __ldcg(reinterpret_cast<const float4 *>(qa) + 1);
                    float4 b0 = make_float4(0.f, 0.f, 0.f, 0.f), b1 = b0;
                    if (bq) {
                        b0 = __ldg(reinterpret_cast<const float4 *>(bq + hh * 64 + c8 * 8));
                        b1 = __ldg(reinterpret_cast<const float4 *>(bq + hh * 64 + c8 * 8) + 1);
                    }
                    const float t[8] = {a0.x + b0.x, a0.y + b0.y, a0.z + b0.z, a0.w + b0.w,
                                        a1.x + b1.x, a1.y + b1.y, a1.z + b1.z, a1.w + b1.w};
#pragma unroll
                    for (int i = 0; i < 8; ++i) qf[i] = f16_round(t[i]) * ATT_SCALE_LOG2E;
                }
                if (owns_new) {
#pragma unroll
                    for (int kv = 0; kv < 2; ++kv) {
                        const float *src = qa + (size_t)(kv + 1) * d;
                        const float4 a0 = __ldcg(reinterpret_cast<const float4 *>(src)), a1 = __ldcg(reinterpret_cast<const float4 *>(src) + 1);
                        float4 b0 = make_float4(0.f, 0.f, 0.f, 0.f), b1 = b0;
                        if (bq) {
                            const float *bp = bq + (size_t)(kv + 1) * d + hh * 64 + c8 * 8;
                            b0 = __ldg(reinterpret_cast<const float4 *>(bp));
                            b1 = __ldg(reinterpret_cast<const float4 *>(bp) + 1);
                        }
                        __half2 h0 = __floats2half2_rn(a0.x + b0.x, a0.y + b0.y), h1 = __floats2half2_rn(a0.z + b0.z, a0.w + b0.w);
                        __half2 h2 = __floats2half2_rn(a1.x + b1.x, a1.y + b1.y), h3 = __floats2half2_rn(a1.z + b1.z, a1.w + b1.w);
                        uint4 pk;
                        pk.x = *reinterpret_cast<uint32_t *>(&h0);
                        pk.y = *reinterpret_cast<uint32_t *>(&h1);
                        pk.z = *reinterpret_cast<uint32_t *>(&h2);
                        pk.w = *reinterpret_cast<uint32_t *>(&h3);
                        if (g4 == 0)
                            *reinterpret_cast<uint4 *>((kv ? Lp->vc : Lp->kc) + ((size_t)it * P.cap + pos) * 64 + c8 * 8) = pk;
                        if (kv) half8_to_float(pk, vn); else half8_to_float(pk, kn);
                    }
                }
                float m = NEG_BIG, l = 0.0f, acc[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
                mark();
                for (int r = r0; r < r1; r += ATT_ROWS) {
                    top_up();
                    const uint32_t s = att_consumed % ATT_NST;
                    ok = tc::mbar_wait(att_full + 8 * (aw * ATT_NST + s), (att_consumed / ATT_NST) & 1, &abort_flag, P.dev_err, E_ATT);
                    if (!ok) break;
                    __syncwarp();
                    mark();
                    const uint4 *ks = reinterpret_cast<const uint4 *>(ring_gen + s * ATT_STAGE);
                    const uint4 *vs = reinterpret_cast<const uint4 *>(ring_gen + s * ATT_STAGE + ATT_ROWS * 128);
                    const int rows = min(ATT_ROWS, r1 - r);
                    att_rows16(ks, vs, 0, rows, g4, c8, qf, m, l, acc);
                    if (rows > 16) att_rows16(ks, vs, 16, rows, g4, c8, qf, m, l, acc);
                    __syncwarp(); // every lane has read the stage: it may be requested again
                    ++att_consumed;
                    mark();
                }
                if (!ok) break;
                top_up(); // the next sub-item's first rows travel while this one is finished
                if (owns_new) { // the new position, from registers, into lane group 0's state
                    float t = 0.0f;
#pragma unroll
                    for (int i = 0; i < 8; ++i) t = fmaf(qf[i], kn[i], t);
#pragma unroll
                    for (int o = 1; o < 8; o <<= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
                    if (g4 == 0) {
                        const float m_new = fmaxf(m, t), corr = exp2f(m - m_new), pw = exp2f(t - m_new);
                        l = l * corr + pw;
#pragma unroll
                        for (int i = 0; i < 8; ++i) acc[i] = fmaf(pw, vn[i], acc[i] * corr);
                        m = m_new;
                    }
                }
                // merge the four lane groups (lanes 8 and 16 apart hold the same 8 dims)
#pragma unroll
                for (int off = 8; off <= 16; off <<= 1) {
                    const float m_o = __shfl_xor_sync(0xffffffffu, m, off), l_o = __shfl_xor_sync(0xffffffffu, l, off);
                    const float m_n = fmaxf(m, m_o);
                    const float ws = exp2f(m - m_n), wo = exp2f(m_o - m_n);
                    l = l * ws + l_o * wo;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float a_o = __shfl_xor_sync(0xffffffffu, acc[i], off);
                        acc[i] = acc[i] * ws + a_o * wo;
                    }
                    m = m_n;
                }
                if (G == 1) {
                    if (g4 == 0) {
                        const float inv = 1.0f / l;
                        __half2 h0 = __floats2half2_rn(acc[0] * inv, acc[1] * inv), h1 = __floats2half2_rn(acc[2] * inv, acc[3] * inv);
                        __half2 h2 = __floats2half2_rn(acc[4] * inv, acc[5] * inv), h3 = __floats2half2_rn(acc[6] * inv, acc[7] * inv);
                        uint4 v;
                        v.x = *reinterpret_cast<uint32_t *>(&h0);
                        v.y = *reinterpret_cast<uint32_t *>(&h1);
                        v.z = *reinterpret_cast<uint32_t *>(&h2);
                        v.w = *reinterpret_cast<uint32_t *>(&h3);
                        *reinterpret_cast<uint4 *>(P.att + (size_t)sq * d + hh * 64 + c8 * 8) = v;
                    }
                } else if (g4 == 0) {
                    float *rc = rec + (size_t)sidx * REC_FLOATS;
                    if (c8 == 0) { rc[0] = m; rc[1] = l; }
#pragma unroll
                    for (int i = 0; i < 8; ++i) rc[2 + c8 * 8 + i] = acc[i];
                }
                mark();
            }
            if (G > 1) {
                named_sync<DQ_THREADS>(3); // all partial records of the block are written
                mark();
                if (ok) {
                    for (int j = aw; j < nj; j += DQ_WARPS) { // lane owns output dims 2*lane, 2*lane+1
                        const float *r0 = rec + (size_t)j * G * REC_FLOATS;
                        float Mx = NEG_BIG;
                        for (int p = 0; p < G; ++p) Mx = fmaxf(Mx, r0[p * REC_FLOATS]);
                        float L = 0.0f, o0 = 0.0f, o1 = 0.0f;
                        for (int p = 0; p < G; ++p) {
                            const float w = exp2f(r0[p * REC_FLOATS] - Mx);
                            L += r0[p * REC_FLOATS + 1] * w;
                            o0 += r0[p * REC_FLOATS + 2 + 2 * lane] * w;
                            o1 += r0[p * REC_FLOATS + 3 + 2 * lane] * w;
                        }
                        const int it = blk + nblk * j, sq = it / H, hh = it - sq * H;
                        const float inv = 1.0f / L;
                        *reinterpret_cast<__half2 *>(P.att + (size_t)sq * d + hh * 64 + 2 * lane) = __floats2half2_rn(o0 * inv, o1 * inv);
                    }
                }
            }
            mark();
        };

        for (int l = 0; l < P.n_layer; ++l) {
            const Layer *Lp = P.layers + l;
            // ---- LN1 ----
            ln_phase(Lp->ln_g[0], Lp->ln_b[0]);
            phase_end(PH_LN1);
            // ---- QKV GEMM -> qkv_acc ----
            gemm_dq(0, P.qkv_acc, 3 * d, nullptr);
            phase_end(PH_QKV);
            // ---- attention (finalises q, k, v; appends k, v) -> att ----
            attention(Lp);
            phase_end(PH_ATT);
            // ---- out-projection GEMM -> residual ----
            gemm_dq(1, P.x, d, Lp->bias[1]);
            phase_end(PH_PROJ);
            // ---- LN2; the q/k/v accumulator goes back to zero ----
            ln_phase(Lp->ln_g[1], Lp->ln_b[1]);
            if (ok) {
                float4 *z = reinterpret_cast<float4 *>(P.qkv_acc);
                const int nz = (M * 3 * d) >> 2;
                for (int i = blk * DQ_THREADS + wt; i < nz; i += nblk * DQ_THREADS) z[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
            phase_end(PH_LN2);
            // ---- FC GEMM -> fc_acc ----
            gemm_dq(2, P.fc_acc, 4 * d, nullptr);
            phase_end(PH_FC);
            // ---- bias + GELU -> hidden fp16; the accumulator goes back to zero ----
            wait_inputs();
            if (ok) {
                float4 *a4 = reinterpret_cast<float4 *>(P.fc_acc);
                const float *bfc = Lp->bias[2];
                const int n4 = d, tot = M * n4; // 4d/4 float4 per row
                for (int i = blk * DQ_THREADS + wt; i < tot; i += nblk * DQ_THREADS) {
                    const int col4 = i % n4;
                    float4 v = __ldcg(a4 + i);
                    if (bfc) {
                        const float4 bb = __ldg(reinterpret_cast<const float4 *>(bfc) + col4);
                        v.x += bb.x; v.y += bb.y; v.z += bb.z; v.w += bb.w;
                    }
                    __half2 lo = __floats2half2_rn(apply_act(v.x, P.act), apply_act(v.y, P.act));
                    __half2 hi = __floats2half2_rn(apply_act(v.z, P.act), apply_act(v.w, P.act));
                    *reinterpret_cast<uint2 *>(P.hbuf + (size_t)i * 4) =
                        make_uint2(*reinterpret_cast<uint32_t *>(&lo), *reinterpret_cast<uint32_t *>(&hi));
                    a4[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
            phase_end(PH_ACT);
            // ---- MLP-projection GEMM -> residual ----
            gemm_dq(3, P.x, d, Lp->bias[3]);
            phase_end(PH_FCPROJ);
        }
    }

    // ---- teardown (also the path taken after a wait gave up) ----
    if (abort_flag) { // let copies still in flight land before the block's memory is released
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    if (warp == W_MMA) tc::tmem_dealloc(tmem_base, TMEM_COLS);
}

}  // namespace pd

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
bool decode_persistent_supported(const b200nn_gpt2 *m, int rows) {
    const b200nn_ctx *ctx = m->ctx;
    if (!ctx->persist || !m->int4) return false;
    if (rows <= ctx->gemv_max_rows || rows < ctx->persist_min_rows || rows > std::min(256, ctx->persist_max_rows)) return false;
    const int d = m->cfg.n_embd;
    if (d % 64 != 0 || d > 4 * pd::DQ_THREADS * pd::LN_V || d / m->cfg.n_head != 64) return false;
    for (const BlockW &b : m->blocks)
        for (const LinearAny *l : {&b.qkv, &b.proj, &b.fc, &b.fcproj})
            if (!l->int4 || !l->q.fast || l->q.group != m->blocks[0].qkv.q.group) return false;
    return true;
}

int decode_persistent_prepare(b200nn_session *s) {
    b200nn_gpt2 *m = s->m;
    b200nn_ctx *ctx = m->ctx;
    const size_t B = s->batch, d = m->cfg.n_embd, L = m->cfg.n_layer;
    std::vector<pd::Layer> h(L);
    for (size_t l = 0; l < L; ++l) {
        const BlockW &b = m->blocks[l];
        const LinearAny *lin[4] = {&b.qkv, &b.proj, &b.fc, &b.fcproj};
        for (int g = 0; g < 4; ++g) {
            h[l].tiles[g] = (const uint8_t *)lin[g]->q.tiled->p;
            h[l].scales[g] = (const __half *)lin[g]->q.scales_h->p;
            h[l].bias[g] = lin[g]->bias();
        }
        h[l].ln_g[0] = (const float *)b.ln1_g->p;
        h[l].ln_b[0] = (const float *)b.ln1_b->p;
        h[l].ln_g[1] = (const float *)b.ln2_g->p;
        h[l].ln_b[1] = (const float *)b.ln2_b->p;
        h[l].kc = s->kv.kl((int)l);
        h[l].vc = s->kv.vl((int)l);
    }
    TRY(dev_alloc(ctx, L * sizeof(pd::Layer), &s->pd_layers));
    CK(ctx, cudaMemcpy(s->pd_layers->p, h.data(), L * sizeof(pd::Layer), cudaMemcpyHostToDevice));
    TRY(dev_alloc(ctx, B * 3 * d * 4, &s->pd_qkv_acc));
    TRY(dev_alloc(ctx, B * 4 * d * 4, &s->pd_fc_acc));
    TRY(dev_alloc(ctx, 256, &s->pd_sync)); // [0] grid counter; bytes 64.. : per-phase nanoseconds
    CK(ctx, cudaMemsetAsync(s->pd_qkv_acc->p, 0, B * 3 * d * 4, ctx->stream));
    CK(ctx, cudaMemsetAsync(s->pd_fc_acc->p, 0, B * 4 * d * 4, ctx->stream));
    CK(ctx, cudaMemsetAsync(s->pd_sync->p, 0, 256, ctx->stream));
    return B200NN_OK;
}

int launch_decode_layers(b200nn_session *s, bool profile) {
    b200nn_gpt2 *m = s->m;
    b200nn_ctx *ctx = m->ctx;
    const int B = (int)s->batch, d = m->cfg.n_embd, H = m->cfg.n_head;
    static bool attr_done[16] = {};
    static int max_blocks[16] = {};
    if (!attr_done[ctx->device & 15]) {
        CK(ctx, cudaFuncSetAttribute(pd::decode_layers_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, pd::SMEM_BYTES));
        prefer_max_smem(pd::decode_layers_kernel);
        int per_sm = 0;
        CK(ctx, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, pd::decode_layers_kernel, pd::THREADS, pd::SMEM_BYTES));
        max_blocks[ctx->device & 15] = per_sm * ctx->sm_count;
        attr_done[ctx->device & 15] = true;
    }
    const int grid = std::min(ctx->sm_count, max_blocks[ctx->device & 15]);
    if (grid < 1) return set_error(ctx, B200NN_ERR_UNSUPPORTED, "decode_layers_kernel does not fit on this device");
    pd::Params P = {};
    P.layers = (const pd::Layer *)s->pd_layers->p;
    P.n_layer = m->cfg.n_layer;
    P.M = B;
    P.d = d;
    P.H = H;
    P.cap = (int)s->kv.cap;
    P.act = m->act();
    P.MB = B <= 32 ? 32 : B <= 64 ? 64 : B <= 128 ? 128 : 256;
    P.ns_shift = P.MB == 256 ? 2 : 3;
    P.eps = m->cfg.layer_norm_epsilon;
    const BlockW &b0 = m->blocks[0];
    const LinearAny *lin[4] = {&b0.qkv, &b0.proj, &b0.fc, &b0.fcproj};
    for (int g = 0; g < 4; ++g) {
        P.K[g] = lin[g]->q.K;
        P.N[g] = lin[g]->q.N;
        P.kb[g] = lin[g]->q.k_blocks;
        P.nt[g] = lin[g]->q.n_tiles;
        P.npad[g] = lin[g]->q.n_pad;
    }
    P.group = b0.qkv.q.group;
    // parts per (sequence, head) item: as many as keep a block's partial records within their buffer,
    // so that the eight attention warps of a block all have rows to stream
    const int items = B * H, nj = (items + grid - 1) / grid;
    int G = 1;
    while (G < 8 && nj * G * 2 <= pd::MAX_REC && nj * G < 3 * pd::DQ_WARPS) G *= 2;
    P.att_G = G;
    P.pos_ptr = s->pos_ptr();
    P.x = (float *)s->ws_step.x->p;
    P.ln = (__half *)s->ws_step.ln->p;
    P.qkv_acc = (float *)s->pd_qkv_acc->p;
    P.att = (__half *)s->ws_step.att->p;
    P.fc_acc = (float *)s->pd_fc_acc->p;
    P.hbuf = (__half *)s->ws_step.fc->p;
    P.bar = (unsigned *)s->pd_sync->p;
    P.dev_err = ctx->dev_err;
    P.prof = profile ? (unsigned long long *)((char *)s->pd_sync->p + 64) : nullptr;
    P.trace = (unsigned long long *)ctx->persist_trace;
    // the three fp16 activation buffers as 2-D tensors [rows, K] with [MB x 64] boxes, 128-byte swizzle
    if (!ctx->encode_tiled) return set_error(ctx, B200NN_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled is unavailable");
    {
        typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                          const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                          CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
        void *bufs[3] = {P.ln, P.att, P.hbuf};
        const int ks[3] = {d, d, 4 * d};
        for (int i = 0; i < 3; ++i) {
            cuuint64_t gdim[2] = {(cuuint64_t)ks[i], (cuuint64_t)B};
            cuuint64_t gstride[1] = {(cuuint64_t)ks[i] * sizeof(__half)};
            cuuint32_t box[2] = {TILE_K, (cuuint32_t)P.MB};
            cuuint32_t estr[2] = {1, 1};
            CUresult r = ((EncodeTiledFn)ctx->encode_tiled)(&P.tmap[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, bufs[i], gdim, gstride,
                                                            box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                                            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return set_error(ctx, B200NN_ERR_CUDA, "cuTensorMapEncodeTiled failed: " + std::to_string((int)r));
        }
    }
    const size_t item_bytes = (size_t)2 * s->kv.cap * 128;
    P.pf_items = (int)std::min<size_t>((size_t)items, ((size_t)ctx->persist_prefetch_mb << 20) / item_bytes);
    P.grid_wait_cycles = ctx->persist_wait_cycles > 0 ? ctx->persist_wait_cycles : tc::WAIT_CYCLES;
    P.fault_block = ctx->persist_fault_phase >= 0 ? 0 : -1;
    P.fault_phase = ctx->persist_fault_phase;
    CK(ctx, cudaMemsetAsync(s->pd_sync->p, 0, 4, ctx->stream));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(pd::THREADS);
    cfg.dynamicSmemBytes = pd::SMEM_BYTES;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative; // every block resident at once: they wait on one another
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    CK(ctx, cudaLaunchKernelEx(&cfg, pd::decode_layers_kernel, P));
    CK_LAUNCH(ctx, "decode_layers_kernel");
    return B200NN_OK;
}
