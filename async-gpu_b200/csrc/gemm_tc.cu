// int4 weight-only Linear on the 5th-generation tensor cores (tcgen05, operands and accumulators in
// tensor memory).
//
//   y[m,n] = sum_k x[m,k] * (nibble(k,n)-8) * scale[k/group,n]  (+ bias, activation, residual, KV write)
//
// The weight is the MMA's A operand (128 output features = the 128 TMEM lanes), the activations are
// the B operand (MB token rows = the MMA's N, 32..256), so a decode batch of 32 costs a 128x32 MMA
// instead of a 128-row tile padded with 96 dead rows.
//
// Block = 96 + 128*NG threads, one 128-feature tile x one K split x one MB-row tile:
//   warp 0      streams packed 4 KB weight tiles HBM -> shared memory with 1-D bulk async copies
//               (the tiles are contiguous in the re-tiled layout), NP stages deep;
//   warp 1      loads the fp16 activation tile [MB x 64] through a 2-D tensor map with 128-byte
//               swizzle, which lands it in the canonical K-major UMMA layout (the B operand);
//   warp 2      owns TMEM (alloc / dealloc) and issues four tcgen05.mma (K=16 each, A from TMEM,
//               B from shared memory) per 64-wide K block, then tcgen05.commit to release the stage;
//   dequant     NG groups of four warps take K blocks round-robin.  A thread owns one weight row of
//   warps       the block: 32 packed bytes -> 64 fp16 values (lop3 magic-number unpack to the exact
//               integer, times the fp16 group scale held in shared memory) written with tcgen05.st
//               into its own TMEM lane: the dequantised tile never touches shared memory, so there
//               is no swizzled store and no generic->async proxy fence on the critical path.
//               Afterwards the same warps move the accumulator TMEM -> shared memory and run the
//               epilogue row-wise: one warp per token row, 4 features per lane, so that every
//               global access is a 512-byte contiguous row segment.
// K can be split across blocks.  The residual epilogue adds every split's partial tile into the f32
// residual stream with vector reductions at L2 (order of the additions not fixed).  The other
// epilogues need the complete sum: up to eight splits run as one thread-block cluster and add their
// staged partial tiles through distributed shared memory in split order (deterministic); beyond
// eight (only by override) partial tiles go to scratch and the last block to arrive sums them.
//
// Every wait on an mbarrier is bounded: when it runs out the block records a code in the device
// error word, all roles leave their loops, TMEM is freed and the kernel returns.
#include <cooperative_groups.h>
#include <cuda.h>

#include "device_utils.cuh"
#include "tc_ptx.cuh"

namespace cg = cooperative_groups;

namespace {

enum : uint32_t { ERR_P_EMPTY = 0x101, ERR_X_EMPTY, ERR_A_FULL, ERR_X_FULL, ERR_P_FULL, ERR_A_EMPTY, ERR_ACC };

constexpr int A_COLS = TILE_K / 2; // 32-bit TMEM columns of one dequantised 64-wide K block

struct Smem {
    uint32_t x, p;                                      // ring bases (shared-space addresses)
    uint32_t p_full, p_empty, x_full, a_full, ax_empty; // barrier array bases
    uint32_t acc_full, tmem_slot, sc;
};

template <int NTHREADS>
__device__ __forceinline__ void bar_sync_dequant() {
    asm volatile("bar.sync 1, %0;" ::"n"(NTHREADS) : "memory");
}

// MB: token-tile width; NS: operand stages (activation tiles in shared memory, dequantised weight
// tiles in TMEM); NP: packed-weight stages; NG: dequant groups; TC: TMEM columns to allocate.
template <int MB, int NS, int NP, int NG, int TC>
__global__ void __launch_bounds__(96 + 128 * NG, NG == 2 ? 2 : 1)
int4_gemm_tc_kernel(const uint8_t *__restrict__ tiles, const __half *__restrict__ scales,
                    const __grid_constant__ CUtensorMap tmap_x, int M, int N, int k_blocks, int n_pad, int group,
                    int kb_per_split, int cluster_mode, Epilogue epi, float *__restrict__ scratch,
                    unsigned *__restrict__ counters, uint32_t *__restrict__ dev_err, long long *__restrict__ trace) {
#ifdef B200NN_TRACE
#define TRACE(slot)                                                                                     \
    do {                                                                                                \
        if (trace && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) trace[slot] = clock64();    \
    } while (0)
#else
#define TRACE(slot) do { } while (0)
#endif
#define ROWSTAT(c) (epi.ln_stats ? rowstat[c] : make_float2(0.f, 0.f))
    constexpr int X_BYTES = MB * 128;
    constexpr int DQ = 128 * NG; // dequant / epilogue threads
    static_assert(MB + NS * A_COLS <= TC, "TMEM budget exceeded");
    // A dequant group waits for "the MMAs of K block i-NS have retired" by the phase parity of that
    // stage's barrier.  Parity only tells the last two phases apart, so the barrier must never be two
    // phases behind the waiter: the group's previous K block (i-NG) has already waited for the MMAs of
    // K block i-NG-NS, MMAs retire in order, hence K block i-2*NS has retired whenever NS >= NG.
    // (With 3 operand stages and 4 groups a group that ran ahead took the phase before last for its
    // own, overwrote a live TMEM stage and unbalanced the barrier's transaction count: the launch failed.)
    static_assert(NS >= NG && NP >= NG, "fewer stages than dequant groups: phase parity would alias");
    extern __shared__ uint8_t smem_raw[];
    __shared__ int abort_flag;
    __shared__ int is_last;
    __shared__ float2 rowstat[MB]; // (mean, rstd) of the tile's token rows when a LayerNorm is folded in

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nt = blockIdx.x, split = blockIdx.y, splits = gridDim.y, mt = blockIdx.z;
    const int kb0 = split * kb_per_split;
    const int nkb = min(kb_per_split, k_blocks - kb0);
    if (tid == 0) TRACE(0);
    pdl_trigger(); // the next kernel may start its own prologue / weight prefetch

    // carve shared memory: rings 1024-byte aligned, barriers and group scales behind them
    const uint32_t base = (tc::smem_u32(smem_raw) + 1023u) & ~1023u;
    Smem S;
    S.x = base;
    S.p = S.x + NS * X_BYTES;
    uint32_t b = S.p + NP * TILE_BYTES;
    S.p_full = b;            b += NP * 8;
    S.p_empty = b;           b += NP * 8;
    S.x_full = b;            b += NS * 8;
    S.a_full = b;            b += NS * 8;
    S.ax_empty = b;          b += NS * 8;
    S.acc_full = b;          b += 8;
    S.tmem_slot = b;         b += 8;
    S.sc = (b + 15u) & ~15u;
    uint8_t *gen_base = smem_raw + (base - tc::smem_u32(smem_raw)); // generic pointer to `base`

    if (tid == 0) {
        abort_flag = 0;
        for (int i = 0; i < NP; ++i) {
            tc::mbar_init(S.p_full + 8 * i, 1);
            tc::mbar_init(S.p_empty + 8 * i, 4); // one arrival per warp of the dequant group
        }
        for (int i = 0; i < NS; ++i) {
            tc::mbar_init(S.x_full + 8 * i, 1);
            tc::mbar_init(S.a_full + 8 * i, 5); // four dequant warps + the activation tile's expect_tx
            tc::mbar_init(S.ax_empty + 8 * i, 1); // tcgen05.commit
        }
        tc::mbar_init(S.acc_full, 1);
        tc::fence_mbar_init();
    }
    if (warp == 1 && lane == 0) tc::prefetch_tmap(&tmap_x);
    if (warp == 2) tc::tmem_alloc(S.tmem_slot, TC);
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    if (tid == 0) TRACE(1);
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(gen_base + (S.tmem_slot - base));
    const uint32_t tmem_a = tmem_base + MB; // dequantised weight stages follow the accumulator columns

    // the epilogue's per-thread constants (filled by the epilogue warps, used in both of its places):
    // lane l owns features 4l..4l+3 of a token row
    const int n4 = nt * TILE_N + lane * 4;
    float4 b4 = make_float4(0.f, 0.f, 0.f, 0.f), g4 = b4;
    Epilogue e2 = epi; // the device-side position is read once per thread, not once per element
    e2.pos_ptr = nullptr;

    if (warp == 0) {
        // ---- packed weight tiles: HBM -> shared, NP stages in flight (one elected lane) ----
        const uint8_t *src = tiles + ((size_t)nt * k_blocks + kb0) * TILE_BYTES;
        int s = 0;
        uint32_t ph = 1; // parity that is already complete on a fresh barrier
        for (int i = 0; i < nkb; ++i) {
            if (i >= NP && !tc::mbar_wait(S.p_empty + 8 * s, ph, &abort_flag, dev_err, ERR_P_EMPTY)) break;
            if (tc::elect_one()) {
                tc::mbar_expect_tx(S.p_full + 8 * s, TILE_BYTES);
                tc::tma_load_1d(S.p + s * TILE_BYTES, src, TILE_BYTES, S.p_full + 8 * s);
                if (i < 32) TRACE(32 + i);
            }
            src += TILE_BYTES;
            if (++s == NP) { s = 0; ph ^= 1; }
        }
    } else if (warp == 1) {
        // ---- activation tiles [MB rows x 64 k] through the tensor map (zero fill past M); their
        //      bytes are expected on the same barrier the dequant warps arrive on ----
        int s = 0, kx = kb0 * TILE_K;
        uint32_t ph = 1;
        pdl_wait(); // the activations are the previous kernel's output
        for (int i = 0; i < nkb; ++i) {
            if (i >= NS && !tc::mbar_wait(S.ax_empty + 8 * s, ph, &abort_flag, dev_err, ERR_X_EMPTY)) break;
            if (tc::elect_one()) {
                tc::mbar_expect_tx(S.a_full + 8 * s, X_BYTES);
                tc::tma_load_2d(S.x + s * X_BYTES, &tmap_x, kx, mt * MB, S.a_full + 8 * s);
            }
            kx += TILE_K;
            if (++s == NS) { s = 0; ph ^= 1; }
        }
    } else if (warp == 2) {
        // ---- MMA issue (one elected lane; the stream of instructions per K block is kept short
        //      because this warp shares its scheduler with dequant warps) ----
        // The whole warp runs the loop (uniform control flow, operands stay warp-uniform); one
        // elected lane issues.
        constexpr uint32_t idesc = tc::umma_idesc_f16(128, MB);
        const uint64_t bd0 = tc::umma_desc_sw128(S.x);
        bool ok = true;
        int s = 0;
        uint32_t ph = 0;
        for (int i = 0; i < nkb; ++i) {
            ok = tc::mbar_wait(S.a_full + 8 * s, ph, &abort_flag, dev_err, ERR_A_FULL);
            if (!ok) break;
            tc::tc_fence_after_sync();
            const uint64_t bd = bd0 + (uint64_t)((s * X_BYTES) >> 4);
            const uint32_t ad = tmem_a + s * A_COLS;
            if (tc::elect_one()) {
                if (i < 32) TRACE(64 + i);
                tc::umma_f16_ts(tmem_base, ad, bd, idesc, i != 0);
                tc::umma_f16_ts(tmem_base, ad + 8, bd + 2, idesc, 1u);  // per MMA: 8 TMEM columns of A,
                tc::umma_f16_ts(tmem_base, ad + 16, bd + 4, idesc, 1u); // +32 bytes of B along K
                tc::umma_f16_ts(tmem_base, ad + 24, bd + 6, idesc, 1u);
                tc::umma_commit(S.ax_empty + 8 * s); // operand stage reusable once these MMAs retire
            }
            __syncwarp();
            if (++s == NS) { s = 0; ph ^= 1; }
        }
        if (ok && tc::elect_one()) tc::umma_commit(S.acc_full);
        if (lane == 0) TRACE(2);
        __syncwarp();
    } else {
        // ---- dequantise, then epilogue ----
        const int t = tid - 96, grp = t >> 7;
        const int quad = warp & 3;          // the TMEM lanes this warp may touch: 32*quad .. +31
        const int row = quad * 32 + lane;   // weight row (output feature) of the tile owned by this thread
        const int dw_lane0 = (lane == 0);
        // group scales of this block's K range -> shared memory, all loads in flight at once
        const int g0 = (kb0 * TILE_K) / group;
        const int ng = ((kb0 + nkb) * TILE_K - 1) / group - g0 + 1;
        __half *sc_s = reinterpret_cast<__half *>(gen_base + (S.sc - base));
        for (int idx = t; idx < ng * TILE_N; idx += DQ)
            sc_s[idx] = scales[(size_t)(g0 + (idx >> 7)) * n_pad + nt * TILE_N + (idx & 127)];
        bar_sync_dequant<DQ>();
        for (int i = grp; i < nkb; i += NG) {
            const int sp = i % NP, php = (i / NP) & 1, sa = i % NS, pha = (i / NS) & 1;
            if (!tc::mbar_wait(S.p_full + 8 * sp, php, &abort_flag, dev_err, ERR_P_FULL)) break;
            if (t == 0 && i < 32) TRACE(96 + i);
            const uint8_t *pk = gen_base + (S.p - base) + sp * TILE_BYTES + row * 16;
            const uint4 w0 = *reinterpret_cast<const uint4 *>(pk);        // k  0..31 of the block
            const uint4 w1 = *reinterpret_cast<const uint4 *>(pk + 2048); // k 32..63
            const __half2 s2 = __half2half2(sc_s[(((kb0 + i) * TILE_K) / group - g0) * TILE_N + row]);
            __syncwarp();
            if (dw_lane0) tc::mbar_arrive(S.p_empty + 8 * sp); // this warp has its packed words in registers
            if (i >= NS && !tc::mbar_wait(S.ax_empty + 8 * sa, pha ^ 1, &abort_flag, dev_err, ERR_A_EMPTY)) break;
            tc::tc_fence_after_sync();
            const uint32_t a_addr = tmem_a + ((uint32_t)(quad * 32) << 16) + sa * A_COLS;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint4 w = h ? w1 : w0;
                const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
                uint32_t o[16];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    __half2 q[4];
                    unpack8_int4(ww[j], q);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        __half2 r = __hmul2(q[e], s2); // (k, k+1) -> low, high half of one 32-bit column
                        o[4 * j + e] = *reinterpret_cast<uint32_t *>(&r);
                    }
                }
                tc::tmem_st_x16(a_addr + 16 * h, o);
            }
            tc::tmem_st_wait();
            tc::tc_fence_before_sync();
            __syncwarp();
            if (dw_lane0) tc::mbar_arrive(S.a_full + 8 * sa);
            if (t == 0 && i < 32) TRACE(128 + i);
        }
        pdl_wait(); // the epilogue touches buffers the previous kernel may still be using
        // bias and the device-side position are fetched now, under the wait for the last MMAs
        b4 = epi_bias4(epi, n4, N);
        g4 = epi_fold4(epi, n4, N);
        // folded LayerNorm: one thread per token row adds up the row's partial sums (the barrier below publishes them)
        if (epi.ln_stats && t < MB && mt * MB + t < M) rowstat[t] = epi_row_mean_rstd(epi, mt * MB + t);
        if (epi.mode == EPI_QKV && epi.pos_ptr) e2.pos_off = epi.pos_off + *epi.pos_ptr;
        bar_sync_dequant<DQ>();
        if (!abort_flag) tc::mbar_wait(S.acc_full, 0, &abort_flag, dev_err, ERR_ACC);
        bar_sync_dequant<DQ>();
        if (!abort_flag) {
            tc::tc_fence_after_sync();
            if (t == 0) TRACE(3);
            // phase 1: accumulator TMEM -> shared memory stage[MB][128] f32 (the rings are idle by
            // now: every copy into them has been consumed and every MMA has retired)
            float *stage = reinterpret_cast<float *>(gen_base);
            {
                const int colh = (warp - 3) >> 2; // the NG warps of a quadrant split the columns
                constexpr int COLS = MB / NG;
                static_assert(COLS >= 8, "token tile too narrow for this many epilogue warps");
                constexpr int W = COLS >= 16 ? 16 : 8;
                const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + colh * COLS;
#pragma unroll 1
                for (int c0 = 0; c0 < COLS; c0 += W) {
                    uint32_t v[W];
                    if constexpr (W == 16) tc::tmem_ld_x16(taddr + c0, v); else tc::tmem_ld_x8(taddr + c0, v);
#pragma unroll
                    for (int j = 0; j < W; ++j) stage[(colh * COLS + c0 + j) * TILE_N + row] = __uint_as_float(v[j]);
                }
            }
            bar_sync_dequant<DQ>();
            if (t == 0) TRACE(4);
            // phase 2: one warp per token row, lane l owns features 4l..4l+3
            const int w8 = warp - 3;
            constexpr int NW = 4 * NG; // epilogue warps
            const int tile_lin = mt * gridDim.x + nt;
            const float4 *stage4 = reinterpret_cast<const float4 *>(stage);
            const int rows = min(MB, M - mt * MB);
            if (splits == 1) {
                for (int c = w8; c < rows; c += NW)
                    epi_emit4(e2, epi, mt * MB + c, n4, stage4[c * 32 + lane], g4, b4, ROWSTAT(c),
                              epi_resid_old4(epi, mt * MB + c, n4, N), N);
            } else if (epi.mode == EPI_RESID) {
                // residual epilogue with split K: every split adds its partial tile straight into the
                // f32 residual stream with vector reductions at L2 (no scratch, no second pass); the
                // bias goes in with split 0.  The order in which the splits' partials are added is not
                // fixed, so the last bits of the sum can differ between runs.
                const float4 add0 = (split == 0) ? b4 : make_float4(0.f, 0.f, 0.f, 0.f);
                for (int c = w8; c < rows; c += NW)
                    epi_resid_red4(epi, mt * MB + c, n4, f4_add(stage4[c * 32 + lane], add0), N);
            } else if (cluster_mode) {
                // the K splits of this tile are one thread-block cluster: their staged partial tiles are
                // summed through distributed shared memory below, where every thread of the block can
                // take part in the cluster barrier
            } else {
                float4 *part4 = reinterpret_cast<float4 *>(scratch + (((size_t)tile_lin * splits + split) * MB) * TILE_N);
                for (int c = w8; c < rows; c += NW) part4[c * 32 + lane] = stage4[c * 32 + lane];
                __threadfence();
                bar_sync_dequant<DQ>();
                if (t == 0) {
                    unsigned prev = atomicAdd(&counters[tile_lin], 1u);
                    is_last = (prev == (unsigned)(splits - 1));
                    if (is_last) counters[tile_lin] = 0u;
                }
                bar_sync_dequant<DQ>();
                if (is_last) {
                    __threadfence();
                    // the last block to arrive sums the partial tiles in split order
                    const float4 *p4 = reinterpret_cast<const float4 *>(scratch + ((size_t)tile_lin * splits * MB) * TILE_N);
                    for (int c = w8; c < rows; c += NW) {
                        const float4 r_old = epi_resid_old4(epi, mt * MB + c, n4, N);
                        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
                        int sp = 0;
                        for (; sp + 4 <= splits; sp += 4) { // four independent 512-byte row reads in flight
                            float4 t0 = __ldcg(p4 + ((size_t)(sp + 0) * MB + c) * 32 + lane);
                            float4 t1 = __ldcg(p4 + ((size_t)(sp + 1) * MB + c) * 32 + lane);
                            float4 t2 = __ldcg(p4 + ((size_t)(sp + 2) * MB + c) * 32 + lane);
                            float4 t3 = __ldcg(p4 + ((size_t)(sp + 3) * MB + c) * 32 + lane);
                            sum = f4_add(f4_add(f4_add(f4_add(sum, t0), t1), t2), t3);
                        }
                        for (; sp < splits; ++sp) sum = f4_add(sum, __ldcg(p4 + ((size_t)sp * MB + c) * 32 + lane));
                        epi_emit4(e2, epi, mt * MB + c, n4, sum, g4, b4, ROWSTAT(c), r_old, N);
                    }
                }
            }
            if (t == 0) TRACE(5);
        }
    }

    // ---- split K inside a cluster: block `split` finishes the token rows c = split, split+splits, ...
    //      of the tile, adding the partial rows of all blocks in split order (deterministic).  Both
    //      cluster barriers are reached by every thread on every path, aborted or not. ----
    if (cluster_mode) {
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync(); // every block of the cluster has staged its partial tile
        if (warp >= 3 && !abort_flag) {
            constexpr int NW = 4 * NG;
            const int w8 = warp - 3;
            const float4 *stage4 = reinterpret_cast<const float4 *>(gen_base);
            const int rows = min(MB, M - mt * MB);
            for (int c = split + splits * w8; c < rows; c += splits * NW) {
                const float4 r_old = epi_resid_old4(epi, mt * MB + c, n4, N); // in flight under the partial rows' reads
                float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int sp = 0; sp < splits; ++sp)
                    sum = f4_add(sum, cluster.map_shared_rank(stage4, sp)[c * 32 + lane]);
                epi_emit4(e2, epi, mt * MB + c, n4, sum, g4, b4, ROWSTAT(c), r_old, N);
            }
        }
        cluster.sync(); // no block leaves while its shared memory may still be read
    }

    // ---- teardown (also the path taken after a wait gave up) ----
    if (abort_flag && warp < 2) { // let copies still in flight land before the block's memory is released
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    if (warp == 2) tc::tmem_dealloc(tmem_base, TC);
#undef TRACE
#undef ROWSTAT
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

constexpr int kMaxScaleGroups = 64; // group scales of one block's K range held in shared memory

template <int MB, int NS, int NP, int NG, int TC>
int launch_cfg(b200nn_ctx *ctx, const Int4Weight &w, const __half *x, int M, const Epilogue &epi) {
    constexpr size_t ring = (size_t)NS * MB * 128 + (size_t)NP * TILE_BYTES;
    static_assert(ring >= (size_t)MB * TILE_N * sizeof(float), "epilogue stage must fit in the operand rings");
    // barriers behind the rings: NP*16 + NS*24 + 16 bytes, then 16-byte alignment of the scale buffer
    constexpr size_t bar_bytes = 512;
    static_assert(NP * 16 + NS * 24 + 16 + 16 <= bar_bytes, "barrier area too small");
    constexpr size_t smem_max = 1024 + ring + bar_bytes + (size_t)kMaxScaleGroups * TILE_N * sizeof(__half);
    static_assert(smem_max <= 227 * 1024, "shared memory budget exceeded");
    static bool attr_done[16] = {};
    auto kern = int4_gemm_tc_kernel<MB, NS, NP, NG, TC>;
    if (!attr_done[ctx->device & 15]) {
        CK(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_max));
        prefer_max_smem(kern);
        attr_done[ctx->device & 15] = true;
    }
    // activations as a 2-D tensor [M rows, K cols] fp16, box [MB x 64] with 128-byte swizzle
    CUtensorMap tmap;
    cuuint64_t gdim[2] = {(cuuint64_t)w.K, (cuuint64_t)M};
    cuuint64_t gstride[1] = {(cuuint64_t)w.K * sizeof(__half)};
    cuuint32_t box[2] = {TILE_K, (cuuint32_t)MB};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = ((EncodeTiledFn)ctx->encode_tiled)(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void *)x, gdim, gstride, box,
                                                    estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(ctx, B200NN_ERR_CUDA, "cuTensorMapEncodeTiled failed: " + std::to_string((int)r));

    const int m_tiles = (M + MB - 1) / MB;
    const int base_ctas = w.n_tiles * m_tiles;
    // shared memory without the scale buffer, which is sized per launch below
    constexpr size_t smem_fixed = 1024 + ring + bar_bytes;
    // Blocks an SM holds at once: two for the variants with two dequant groups (352 threads, built
    // for at most 93 registers) when their shared memory and TMEM columns fit twice, else one.
    const int ctas_per_sm = (NG == 2 && smem_fixed + 8192 <= 113 * 1024 && 2 * TC <= 512) ? 2 : 1;
    // K split: fills the GPU when there are few (feature tile x token tile) pairs.  The count is
    // rounded down, because one block more than the SMs can hold costs a whole second wave.  The
    // residual epilogue reduces its splits with L2 vector adds, which is cheap, so it splits down to
    // tc_min_kb K blocks per block.  The other epilogues need the complete sum: up to eight splits
    // run as one thread-block cluster and add their partial tiles through distributed shared memory
    // (a cluster barrier and a few shared-memory reads); more splits than a cluster holds (only by
    // override) go through scratch, where the last block to arrive makes a second pass.
    const int target = ctx->sm_count * ctas_per_sm;
    int splits = 1;
    const int min_kb = ctx->tc_min_kb > 0 ? ctx->tc_min_kb : (M <= 64 ? 2 : 3);
    if (epi.mode == EPI_RESID)
        splits = std::min(std::max(1, target / base_ctas), std::max(1, w.k_blocks / min_kb));
    else
        splits = std::min(std::min(8, std::max(1, target / base_ctas)), std::max(1, w.k_blocks / ctx->tc_min_kb_cluster));
    splits = std::max(1, std::min(splits, 32));
    if (ctx->tc_splits > 0) splits = std::min(ctx->tc_splits, w.k_blocks);
    int per = (w.k_blocks + splits - 1) / splits;
    const int per_max = std::max(1, (kMaxScaleGroups - 2) * w.group / TILE_K); // scales must fit their buffer
    per = std::min(per, per_max);
    splits = (w.k_blocks + per - 1) / per;
    const int cluster_mode = (splits > 1 && splits <= 8 && epi.mode != EPI_RESID) ? 1 : 0;
    if (splits > 1 && epi.mode != EPI_RESID && !cluster_mode)
        TRY(ensure_scratch(ctx, (size_t)base_ctas * splits * MB * TILE_N * sizeof(float), (size_t)base_ctas));
    // group scales of one block's K range (one extra group on either side for ranges that start or end inside a group)
    const int sc_groups = std::min(kMaxScaleGroups, per * TILE_K / w.group + 2);
    const size_t smem = smem_fixed + (size_t)sc_groups * TILE_N * sizeof(__half);
    dim3 grid(w.n_tiles, splits, m_tiles);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(96 + 128 * NG);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (cluster_mode) { // the K splits of one tile form a cluster
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = 1;
        attr[na].val.clusterDim.y = splits;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    if (ctx->pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    CK(ctx, cudaLaunchKernelEx(&cfg, kern, (const uint8_t *)w.tiled->p, (const __half *)w.scales_h->p, tmap, M, w.N,
                               w.k_blocks, w.n_pad, w.group, per, cluster_mode, epi, ctx->scratch, ctx->counters,
                               ctx->dev_err, ctx->trace));
    CK_LAUNCH(ctx, "int4_gemm_tc_kernel");
    return B200NN_OK;
}

}  // namespace

bool int4_gemm_tc_supported(const Int4Weight &w, int M) { return w.fast && M >= 1 && w.k_blocks >= 1; }

int launch_int4_gemm_tc(b200nn_ctx *ctx, const Int4Weight &w, const __half *x, int M, const Epilogue &epi) {
    if (!int4_gemm_tc_supported(w, M)) return set_error(ctx, B200NN_ERR_UNSUPPORTED, "shape not supported by the tensor-core GEMM");
    if (!ctx->encode_tiled) return set_error(ctx, B200NN_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled is unavailable");
    // token-tile width: the smallest power of two covering M, capped (ctx->tc_mb overrides the cap).
    // 256-token tiles halve the dequantisation work per flop and make the main loop MMA-bound
    // (measured +30..40 % at 16384 rows), but need enough rows to keep two waves of blocks on every
    // SM; below that 128-token tiles win by filling more SMs.
    int cap = 128;
    if ((long long)w.n_tiles * ((M + 255) / 256) >= 2LL * ctx->sm_count) cap = 256;
    if (ctx->tc_mb > 0) cap = ctx->tc_mb;
    int mb = 32;
    while (mb < M && mb < cap) mb <<= 1;
    switch (mb) { //            MB  NS  NP NG  TMEM columns
        case 32: return launch_cfg<32, 7, 16, 2, 256>(ctx, w, x, M, epi);
        case 64: return launch_cfg<64, 6, 12, 4, 256>(ctx, w, x, M, epi);
        case 128: return launch_cfg<128, 4, 12, 4, 256>(ctx, w, x, M, epi); // 8 stages measured no faster
        default: return launch_cfg<256, 4, 8, 4, 512>(ctx, w, x, M, epi);
    }
}
