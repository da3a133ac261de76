// f32 Linear on the 5th-generation tensor cores: y = x * W + b with fp16 operands and f32
// accumulation in tensor memory.
//
// Replaces the reference's f32 matmul dispatch + bias_add (ops/gemm.rs:20-346, reshape.rs:112-156;
// layers/linear.rs:283-313) for more than four rows.  The reference multiplies in f32 (its own FMA
// kernels or cuBLAS SGEMM); here the weight keeps its f32 copy for the few-row GEMV path and gets an
// fp16 representation stored [out, in] so that both MMA operands are K-major: `hi` = the weight
// rounded to fp16 and, with TW = 2, `lo` = the rounded remainder w - hi, so that hi + lo carries about
// 22 significant bits and the products x*hi + x*lo leave only the rounding of the activations, the
// same as on the int4 path.  The activations arrive as fp16 from the producing kernel (LayerNorm,
// attention, the previous Linear's epilogue) or are converted once by the caller.
//
// Block = 64 + 128*NE threads, one 128-feature tile x one MB-row token tile x one K split:
//   warp 0   TMA producer: per 64-wide K block TW [128 x 64] weight boxes and one [MB x 64] activation
//            box through 2-D tensor maps with 128-byte swizzle (the canonical K-major UMMA layout; rows
//            and columns past the tensor's extent are zero-filled), NS stages in flight;
//   warp 1   owns TMEM and issues 4*TW tcgen05.mma kind::f16 (K = 16 each, both operands from shared
//            memory, accumulator [128 lanes x MB columns] in TMEM) per K block, then tcgen05.commit
//            to hand the stage back to the producer;
//   4*NE     epilogue warps: accumulator TMEM -> shared memory [MB][128] f32 -> row-wise fused
//   warps    epilogue (bias, GELU, residual, q + fp16 K/V cache write), one warp per token row so that
//            every global access is a 512-byte row segment.
// K splits: the residual epilogue adds its partial tiles with L2 vector reductions; the other
// epilogues run their splits as one thread-block cluster and sum the staged partial tiles through
// distributed shared memory in split order (deterministic).
//
// Every mbarrier wait is bounded; when one runs out the block records a code in the device error
// word, all roles leave their loops, TMEM is freed and the kernel returns.
//
// Further down: f16_gemm_tc_persistent_kernel, the same GEMM for passes of many tiles (one block per
// SM, two accumulators), and int4_dequant_f16_kernel, through which an int4 Linear's prefill pass
// reaches it.
#include <cooperative_groups.h>
#include <cuda.h>

#include "device_utils.cuh"
#include "tc_ptx.cuh"

namespace cg = cooperative_groups;

namespace {

enum : uint32_t { ERR_EMPTY = 0x201, ERR_FULL, ERR_ACC };

constexpr int BK = 64;                 // fp16 elements per K block = one 128-byte swizzle row
constexpr int W_BYTES = 128 * BK * 2;  // weight box: 128 features x 64 k

template <int NTHREADS>
__device__ __forceinline__ void bar_sync_epi() {
    asm volatile("bar.sync 1, %0;" ::"n"(NTHREADS) : "memory");
}

// MB: token-tile width (the MMA's N); NS: operand stages; NE: epilogue groups of four warps;
// TW: fp16 terms of the weight (1: hi, 2: hi + lo; tmap_w2 is read only with TW = 2).
template <int MB, int NS, int NE, int TW>
__global__ void __launch_bounds__(64 + 128 * NE, 1)
f16_gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_w2,
                   const __grid_constant__ CUtensorMap tmap_x, int M, int N, int k_blocks, int kb_per_split,
                   int cluster_mode, Epilogue epi, uint32_t *__restrict__ dev_err) {
    constexpr int X_BYTES = MB * BK * 2;
    constexpr int WT_BYTES = TW * W_BYTES; // the weight boxes of one stage, hi then lo
    constexpr int STAGE = WT_BYTES + X_BYTES;
    constexpr int EPI = 128 * NE;
    constexpr int TC = MB < 32 ? 32 : MB; // TMEM columns: a power of two >= 32
    static_assert((size_t)NS * STAGE >= (size_t)MB * 128 * sizeof(float), "epilogue stage must fit in the operand ring");
    extern __shared__ uint8_t smem_raw[];
    __shared__ int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nt = blockIdx.x, split = blockIdx.y, splits = gridDim.y, mt = blockIdx.z;
    const int kb0 = split * kb_per_split;
    const int nkb = min(kb_per_split, k_blocks - kb0);
    pdl_trigger(); // the next kernel may start its prologue

    const uint32_t base = (tc::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *gen_base = smem_raw + (base - tc::smem_u32(smem_raw));
    const uint32_t bars = base + NS * STAGE;
    const uint32_t full = bars, empty = bars + 8 * NS, acc_full = bars + 16 * NS, tmem_slot = acc_full + 8;

    if (tid == 0) {
        abort_flag = 0;
        for (int i = 0; i < NS; ++i) {
            tc::mbar_init(full + 8 * i, 1);  // the producer's expect_tx arrival
            tc::mbar_init(empty + 8 * i, 1); // tcgen05.commit
        }
        tc::mbar_init(acc_full, 1);
        tc::fence_mbar_init();
    }
    if (warp == 0 && lane == 0) {
        tc::prefetch_tmap(&tmap_w);
        if (TW == 2) tc::prefetch_tmap(&tmap_w2);
        tc::prefetch_tmap(&tmap_x);
    }
    if (warp == 1) tc::tmem_alloc(tmem_slot, TC);
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(gen_base + (tmem_slot - base));
    // the epilogue's per-thread constants (filled by the epilogue warps, used in both of its places):
    // lane l owns features 4l..4l+3 of a token row
    const int n4 = nt * 128 + lane * 4;
    float4 b4 = make_float4(0.f, 0.f, 0.f, 0.f);
    Epilogue e2 = epi; // the device-side position is read once per thread
    e2.pos_ptr = nullptr;

    if (warp == 0) {
        // ---- producer.  The weight boxes of the first stages do not depend on the previous kernel
        //      and are requested before the grid dependency is awaited; the activations after it. ----
        const int npre = min(NS, nkb);
        if (tc::elect_one()) {
            for (int i = 0; i < npre; ++i) {
                tc::mbar_expect_tx(full + 8 * i, STAGE);
                tc::tma_load_2d(base + i * STAGE, &tmap_w, (kb0 + i) * BK, nt * 128, full + 8 * i);
                if (TW == 2) tc::tma_load_2d(base + i * STAGE + W_BYTES, &tmap_w2, (kb0 + i) * BK, nt * 128, full + 8 * i);
            }
        }
        __syncwarp();
        pdl_wait();
        if (tc::elect_one()) {
            for (int i = 0; i < npre; ++i)
                tc::tma_load_2d(base + i * STAGE + WT_BYTES, &tmap_x, (kb0 + i) * BK, mt * MB, full + 8 * i);
        }
        __syncwarp();
        int s = 0;
        uint32_t ph = 0; // first reuse of a stage waits for the first completion of its `empty` barrier
        for (int i = npre; i < nkb; ++i) {
            if (!tc::mbar_wait(empty + 8 * s, ph, &abort_flag, dev_err, ERR_EMPTY)) break;
            if (tc::elect_one()) {
                tc::mbar_expect_tx(full + 8 * s, STAGE);
                tc::tma_load_2d(base + s * STAGE, &tmap_w, (kb0 + i) * BK, nt * 128, full + 8 * s);
                if (TW == 2) tc::tma_load_2d(base + s * STAGE + W_BYTES, &tmap_w2, (kb0 + i) * BK, nt * 128, full + 8 * s);
                tc::tma_load_2d(base + s * STAGE + WT_BYTES, &tmap_x, (kb0 + i) * BK, mt * MB, full + 8 * s);
            }
            __syncwarp();
            if (++s == NS) { s = 0; ph ^= 1; }
        }
    } else if (warp == 1) {
        // ---- MMA issue: the whole warp runs the loop, one elected lane issues ----
        constexpr uint32_t idesc = tc::umma_idesc_f16(128, MB);
        const uint64_t d0 = tc::umma_desc_sw128(base);
        bool ok = true;
        int s = 0;
        uint32_t ph = 0;
        for (int i = 0; i < nkb; ++i) {
            ok = tc::mbar_wait(full + 8 * s, ph, &abort_flag, dev_err, ERR_FULL);
            if (!ok) break;
            tc::tc_fence_after_sync();
            const uint64_t ad = d0 + (uint64_t)((s * STAGE) >> 4);
            const uint64_t bd = ad + (uint64_t)(WT_BYTES >> 4);
            if (tc::elect_one()) {
                tc::umma_f16_ss(tmem_base, ad, bd, idesc, i != 0);
                tc::umma_f16_ss(tmem_base, ad + 2, bd + 2, idesc, 1u); // +32 bytes along K inside the swizzle row
                tc::umma_f16_ss(tmem_base, ad + 4, bd + 4, idesc, 1u);
                tc::umma_f16_ss(tmem_base, ad + 6, bd + 6, idesc, 1u);
                if (TW == 2) { // the remainder term of the weight against the same activation tile
                    const uint64_t ad2 = ad + (uint64_t)(W_BYTES >> 4);
                    tc::umma_f16_ss(tmem_base, ad2, bd, idesc, 1u);
                    tc::umma_f16_ss(tmem_base, ad2 + 2, bd + 2, idesc, 1u);
                    tc::umma_f16_ss(tmem_base, ad2 + 4, bd + 4, idesc, 1u);
                    tc::umma_f16_ss(tmem_base, ad2 + 6, bd + 6, idesc, 1u);
                }
                tc::umma_commit(empty + 8 * s); // stage reusable once these MMAs retire
            }
            __syncwarp();
            if (++s == NS) { s = 0; ph ^= 1; }
        }
        if (ok && tc::elect_one()) tc::umma_commit(acc_full);
        __syncwarp();
    } else {
        // ---- epilogue ----
        const int quad = warp & 3;        // the TMEM lanes this warp may touch: 32*quad .. +31
        const int row = quad * 32 + lane; // output feature of the tile owned by this thread
        const int w8 = warp - 2;          // epilogue warp index
        const int colh = w8 >> 2;         // the NE warps of a quadrant split the token columns
        pdl_wait(); // the epilogue touches buffers the previous kernel may still be using
        // bias and the device-side position are fetched under the wait for the accumulator
        b4 = epi_bias4(epi, n4, N);
        if (epi.mode == EPI_QKV && epi.pos_ptr) e2.pos_off = epi.pos_off + *epi.pos_ptr;
        // (the vote keeps the warp converged for the warp-collective wait)
        if (!__any_sync(0xffffffffu, abort_flag != 0)) tc::mbar_wait(acc_full, 0, &abort_flag, dev_err, ERR_ACC);
        bar_sync_epi<EPI>();
        if (!abort_flag) {
            tc::tc_fence_after_sync();
            // phase 1: accumulator TMEM -> shared memory stage[MB][128] f32 (the ring is idle: every
            // copy into it has been consumed and every MMA has retired)
            float *stage = reinterpret_cast<float *>(gen_base);
            {
                constexpr int COLS = MB / NE;
                static_assert(COLS >= 8, "token tile too narrow for this many epilogue warps");
                constexpr int W = COLS >= 16 ? 16 : 8;
                const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + colh * COLS;
#pragma unroll 1
                for (int c0 = 0; c0 < COLS; c0 += W) {
                    uint32_t v[W];
                    if constexpr (W == 16) tc::tmem_ld_x16(taddr + c0, v); else tc::tmem_ld_x8(taddr + c0, v);
#pragma unroll
                    for (int j = 0; j < W; ++j) stage[(colh * COLS + c0 + j) * 128 + row] = __uint_as_float(v[j]);
                }
            }
            bar_sync_epi<EPI>();
            // phase 2: one warp per token row, lane l owns features 4l..4l+3
            constexpr int NW = 4 * NE;
            const float4 *stage4 = reinterpret_cast<const float4 *>(stage);
            const int rows = min(MB, M - mt * MB);
            if (splits == 1) {
                for (int c = w8; c < rows; c += NW) {
                    const float4 v = f4_add(stage4[c * 32 + lane], b4);
                    epi_store4(e2, mt * MB + c, n4, v, N);
                    if (epi.amax_val) epi_argmax4(epi, mt * MB + c, n4, v, N);
                }
            } else if (epi.mode == EPI_RESID) {
                // every split adds its partial tile into the f32 residual stream with vector
                // reductions at L2; the bias goes in with split 0.  The order of the additions is not
                // fixed, so the last bits of the sum can differ between runs.
                const float4 add0 = (split == 0) ? b4 : make_float4(0.f, 0.f, 0.f, 0.f);
                for (int c = w8; c < rows; c += NW)
                    epi_resid_red4(epi, mt * MB + c, n4, f4_add(stage4[c * 32 + lane], add0), N);
            } // else: the splits are one cluster, summed below
        }
    }

    // ---- split K inside a cluster: block `split` finishes token rows split, split+splits, ... of the
    //      tile, adding the partial rows of all blocks in split order.  Both cluster barriers are
    //      reached by every thread on every path, aborted or not. ----
    if (cluster_mode) {
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync(); // every block of the cluster has staged its partial tile
        if (warp >= 2 && !abort_flag) {
            constexpr int NW = 4 * NE;
            const int w8 = warp - 2;
            const float4 *stage4 = reinterpret_cast<const float4 *>(gen_base);
            const int rows = min(MB, M - mt * MB);
            for (int c = split + splits * w8; c < rows; c += splits * NW) {
                float4 sum = b4;
                for (int sp = 0; sp < splits; ++sp)
                    sum = f4_add(sum, cluster.map_shared_rank(stage4, sp)[c * 32 + lane]);
                epi_store4(e2, mt * MB + c, n4, sum, N);
                if (epi.amax_val) epi_argmax4(epi, mt * MB + c, n4, sum, N);
            }
        }
        cluster.sync(); // no block leaves while its shared memory may still be read
    }

    // ---- teardown (also the path taken after a wait gave up) ----
    if (abort_flag && warp == 0) { // let copies still in flight land before the block's memory is released
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tc::tmem_dealloc(tmem_base, TC);
}

// Barrier over the epilogue threads that also ORs a predicate: every thread gets the same answer,
// so a decision to leave the tile loop is taken by all of them or by none.
template <int NTHREADS>
__device__ __forceinline__ bool bar_or_epi(bool pred) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 q, %1, 0;\n\t"
        "bar.red.or.pred p, 1, %2, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(r)
        : "r"((uint32_t)pred), "n"(NTHREADS)
        : "memory");
    return r != 0;
}

// The same GEMM for many tiles (a prefill pass): one block per SM walks the (token tile, feature
// tile) pairs blockIdx.x, blockIdx.x + gridDim.x, ... with the operand pipeline running straight
// through tile boundaries, and two accumulators in tensor memory: while the epilogue warps drain one
// (64 token rows at a time through a 32 KB shared-memory stage of its own), the MMA lane already
// fills the other with the next tile's K loop.  No K split.
//   full[s] / empty[s]      operand stage s loaded / its MMAs retired (as above);
//   acc_full[b] / acc_empty[b]  accumulator b complete (tcgen05.commit) / read out (one arrival per
//                               epilogue warp).
template <int MB, int NS, int NE, int TW>
__global__ void __launch_bounds__(64 + 128 * NE, 1)
f16_gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_w2,
                              const __grid_constant__ CUtensorMap tmap_x, int M, int N, int k_blocks, int n_tiles,
                              int total_tiles, Epilogue epi, uint32_t *__restrict__ dev_err) {
    constexpr int X_BYTES = MB * BK * 2;
    constexpr int WT_BYTES = TW * W_BYTES;
    constexpr int STAGE = WT_BYTES + X_BYTES;
    constexpr int EPI = 128 * NE;
    constexpr int CH = 64;                 // token rows per epilogue pass
    constexpr int OUT_BYTES = CH * 128 * 4; // the epilogue's own stage
    constexpr int TC = 2 * MB;             // two accumulators
    static_assert(TC <= 512 && (TC & (TC - 1)) == 0 && TC >= 32, "TMEM columns: a power of two in 32..512");
    static_assert(MB % CH == 0 && CH % NE == 0 && CH / NE >= 8, "epilogue pass must divide among the warps");
    extern __shared__ uint8_t smem_raw[];
    __shared__ int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    pdl_trigger();

    const uint32_t base = (tc::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *gen_base = smem_raw + (base - tc::smem_u32(smem_raw));
    const uint32_t out_stage = base + NS * STAGE;
    const uint32_t bars = out_stage + OUT_BYTES;
    const uint32_t full = bars, empty = bars + 8 * NS, acc_full = bars + 16 * NS, acc_empty = acc_full + 16,
                   tmem_slot = acc_empty + 16;

    if (tid == 0) {
        abort_flag = 0;
        for (int i = 0; i < NS; ++i) {
            tc::mbar_init(full + 8 * i, 1);
            tc::mbar_init(empty + 8 * i, 1);
        }
        for (int b = 0; b < 2; ++b) {
            tc::mbar_init(acc_full + 8 * b, 1);
            tc::mbar_init(acc_empty + 8 * b, 4 * NE);
        }
        tc::fence_mbar_init();
    }
    if (warp == 0 && lane == 0) {
        tc::prefetch_tmap(&tmap_w);
        if (TW == 2) tc::prefetch_tmap(&tmap_w2);
        tc::prefetch_tmap(&tmap_x);
    }
    if (warp == 1) tc::tmem_alloc(tmem_slot, TC);
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(gen_base + (tmem_slot - base));

    if (warp == 0) {
        // ---- producer: one stream of K blocks over all of this block's tiles ----
        pdl_wait();
        int s = 0;
        uint32_t ph = 1; // parity that is already complete on a fresh barrier: the first NS fills do not wait
        bool ok = true;
        for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
            const int mt = t / n_tiles, nt = t - mt * n_tiles;
            for (int kb = 0; kb < k_blocks; ++kb) {
                ok = tc::mbar_wait(empty + 8 * s, ph, &abort_flag, dev_err, ERR_EMPTY);
                if (!ok) break;
                if (tc::elect_one()) {
                    tc::mbar_expect_tx(full + 8 * s, STAGE);
                    tc::tma_load_2d(base + s * STAGE, &tmap_w, kb * BK, nt * 128, full + 8 * s);
                    if (TW == 2) tc::tma_load_2d(base + s * STAGE + W_BYTES, &tmap_w2, kb * BK, nt * 128, full + 8 * s);
                    tc::tma_load_2d(base + s * STAGE + WT_BYTES, &tmap_x, kb * BK, mt * MB, full + 8 * s);
                }
                __syncwarp();
                if (++s == NS) { s = 0; ph ^= 1; }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issue ----
        constexpr uint32_t idesc = tc::umma_idesc_f16(128, MB);
        const uint64_t d0 = tc::umma_desc_sw128(base);
        int s = 0;
        uint32_t ph = 0;
        bool ok = true;
        int j = 0;
        for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x, ++j) {
            const int b = j & 1;
            // accumulator b was last used by tile j-2: wait until the epilogue has read it out
            ok = tc::mbar_wait(acc_empty + 8 * b, ((j >> 1) & 1) ^ 1, &abort_flag, dev_err, ERR_ACC);
            if (!ok) break;
            tc::tc_fence_after_sync();
            const uint32_t acc = tmem_base + b * MB;
            for (int kb = 0; kb < k_blocks; ++kb) {
                ok = tc::mbar_wait(full + 8 * s, ph, &abort_flag, dev_err, ERR_FULL);
                if (!ok) break;
                tc::tc_fence_after_sync();
                const uint64_t ad = d0 + (uint64_t)((s * STAGE) >> 4);
                const uint64_t bd = ad + (uint64_t)(WT_BYTES >> 4);
                if (tc::elect_one()) {
                    tc::umma_f16_ss(acc, ad, bd, idesc, kb != 0);
                    tc::umma_f16_ss(acc, ad + 2, bd + 2, idesc, 1u);
                    tc::umma_f16_ss(acc, ad + 4, bd + 4, idesc, 1u);
                    tc::umma_f16_ss(acc, ad + 6, bd + 6, idesc, 1u);
                    if (TW == 2) {
                        const uint64_t ad2 = ad + (uint64_t)(W_BYTES >> 4);
                        tc::umma_f16_ss(acc, ad2, bd, idesc, 1u);
                        tc::umma_f16_ss(acc, ad2 + 2, bd + 2, idesc, 1u);
                        tc::umma_f16_ss(acc, ad2 + 4, bd + 4, idesc, 1u);
                        tc::umma_f16_ss(acc, ad2 + 6, bd + 6, idesc, 1u);
                    }
                    tc::umma_commit(empty + 8 * s);
                }
                __syncwarp();
                if (++s == NS) { s = 0; ph ^= 1; }
            }
            if (ok && tc::elect_one()) tc::umma_commit(acc_full + 8 * b);
            __syncwarp();
        }
    } else {
        // ---- epilogue: drains accumulator j & 1 while the MMA lane fills the other one ----
        const int quad = warp & 3, row = quad * 32 + lane, w8 = warp - 2, colh = w8 >> 2;
        constexpr int NW = 4 * NE;
        constexpr int COLS = CH / NE; // token columns per warp and pass
        constexpr int W = COLS >= 16 ? 16 : 8;
        float *stage = reinterpret_cast<float *>(gen_base + (out_stage - base));
        const float4 *stage4 = reinterpret_cast<const float4 *>(stage);
        Epilogue e2 = epi;
        pdl_wait(); // the epilogue writes buffers the previous kernel may still be using
        if (epi.mode == EPI_QKV && epi.pos_ptr) e2.pos_off = epi.pos_off + *epi.pos_ptr;
        e2.pos_ptr = nullptr;
        int j = 0;
        for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++j) {
            const int b = j & 1;
            const int mt = t / n_tiles, nt = t - mt * n_tiles;
            const int n4 = nt * 128 + lane * 4;
            const float4 b4 = epi_bias4(epi, n4, N); // fetched under the wait for the accumulator
            bool ok = true;
            if (!__any_sync(0xffffffffu, abort_flag != 0))
                ok = tc::mbar_wait(acc_full + 8 * b, (j >> 1) & 1, &abort_flag, dev_err, ERR_ACC);
            if (bar_or_epi<EPI>(!ok || abort_flag != 0)) break; // the same decision in every epilogue thread
            tc::tc_fence_after_sync();
            const int rows = min(MB, M - mt * MB);
#pragma unroll 1
            for (int c0 = 0; c0 < MB; c0 += CH) {
                if (c0 < rows) { // token columns past the last row hold products of zero-filled rows: skipped
                    const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + b * MB + c0 + colh * COLS;
#pragma unroll
                    for (int c = 0; c < COLS; c += W) {
                        uint32_t v[W];
                        if constexpr (W == 16) tc::tmem_ld_x16(taddr + c, v); else tc::tmem_ld_x8(taddr + c, v);
#pragma unroll
                        for (int q = 0; q < W; ++q) stage[(colh * COLS + c + q) * 128 + row] = __uint_as_float(v[q]);
                    }
                }
                bar_sync_epi<EPI>();
                const int lim = min(CH, rows - c0);
                if (epi.mode == EPI_RESID) {
                    // this block is the only one that adds to these elements: a reduction at L2 does
                    // the read-modify-write there, with no load for the warp to wait on
                    for (int c = w8; c < lim; c += NW)
                        epi_resid_red4(epi, mt * MB + c0 + c, n4, f4_add(stage4[c * 32 + lane], b4), N);
                } else {
                    for (int c = w8; c < lim; c += NW) {
                        const float4 v = f4_add(stage4[c * 32 + lane], b4);
                        epi_store4(e2, mt * MB + c0 + c, n4, v, N);
                        if (epi.amax_val) epi_argmax4(epi, mt * MB + c0 + c, n4, v, N);
                    }
                }
                bar_sync_epi<EPI>(); // the stage is free for the next pass
            }
            // accumulator b has been read out completely (every tcgen05.ld above has been waited for)
            tc::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(acc_empty + 8 * b);
        }
    }

    // ---- teardown (also the path taken after a wait gave up) ----
    if (abort_flag && warp == 0) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tc::tmem_dealloc(tmem_base, TC);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// fp16 matrix [rows, K] row-major as a 2-D tensor map with a [box_rows x 64] box and 128-byte swizzle
int make_map(b200nn_ctx *ctx, const void *p, int rows, int K, int box_rows, CUtensorMap *out) {
    cuuint64_t gdim[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t gstride[1] = {(cuuint64_t)K * sizeof(__half)};
    cuuint32_t box[2] = {BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = ((EncodeTiledFn)ctx->encode_tiled)(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void *)p, gdim, gstride, box, estr,
                                                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(ctx, B200NN_ERR_CUDA, "cuTensorMapEncodeTiled failed: " + std::to_string((int)r));
    return B200NN_OK;
}

// The weight operand of one launch: hi (and lo, for TW = 2) as [N,K] fp16 matrices.  `constant` says
// that no earlier kernel on the stream writes them, so the launch may overlap the previous kernel's
// tail (the producer of the one-tile kernel requests weight boxes before it waits for the grid
// dependency).
struct WOperand {
    const __half *hi, *lo;
    int N, K;
    bool constant;
};

template <int MB, int NS, int NE, int TW>
int launch_cfg(b200nn_ctx *ctx, const WOperand &w, const __half *x, int M, const Epilogue &epi) {
    constexpr size_t ring = (size_t)NS * (TW * W_BYTES + MB * BK * 2);
    constexpr size_t smem = 1024 + ring + 256;
    static_assert(16 * NS + 16 <= 256, "barrier area too small");
    static_assert(smem <= 227 * 1024, "shared memory budget exceeded");
    static bool attr_done[16] = {};
    auto kern = f16_gemm_tc_kernel<MB, NS, NE, TW>;
    if (!attr_done[ctx->device & 15]) {
        CK(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        prefer_max_smem(kern);
        attr_done[ctx->device & 15] = true;
    }
    CUtensorMap tmap_w, tmap_w2, tmap_x;
    TRY(make_map(ctx, w.hi, w.N, w.K, 128, &tmap_w));
    TRY(make_map(ctx, TW == 2 ? w.lo : w.hi, w.N, w.K, 128, &tmap_w2));
    TRY(make_map(ctx, x, M, w.K, MB, &tmap_x));

    const int k_blocks = (w.K + BK - 1) / BK;
    const int n_tiles = (w.N + 127) / 128, m_tiles = (M + MB - 1) / MB;
    const int base_ctas = n_tiles * m_tiles;
    // K split (rounded down: one block more than the SMs hold costs a second wave).  The residual
    // epilogue reduces with L2 adds and splits down to tc_min_kb K blocks per block; the others need
    // the complete sum and run up to eight splits as one cluster.
    const int target = ctx->sm_count;
    int splits;
    if (epi.mode == EPI_RESID)
        splits = std::min(std::max(1, target / base_ctas), std::max(1, k_blocks / (ctx->tc_min_kb > 0 ? ctx->tc_min_kb : 3)));
    else
        splits = std::min(std::min(8, std::max(1, target / base_ctas)), std::max(1, k_blocks / ctx->tc_min_kb_cluster));
    splits = std::max(1, std::min(splits, 32));
    if (ctx->tc_splits > 0) splits = std::min(ctx->tc_splits, epi.mode == EPI_RESID ? k_blocks : std::min(8, k_blocks));
    const int per = (k_blocks + splits - 1) / splits;
    splits = (k_blocks + per - 1) / per;
    const int cluster_mode = (splits > 1 && epi.mode != EPI_RESID) ? 1 : 0;

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_tiles, splits, m_tiles);
    cfg.blockDim = dim3(64 + 128 * NE);
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
    if (ctx->pdl && w.constant) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    CK(ctx, cudaLaunchKernelEx(&cfg, kern, tmap_w, tmap_w2, tmap_x, M, w.N, k_blocks, per, cluster_mode, epi, ctx->dev_err));
    CK_LAUNCH(ctx, "f16_gemm_tc_kernel");
    return B200NN_OK;
}

// Many tiles (at least two per SM): one persistent block per SM, 256-row token tiles.
template <int NS, int TW>
int launch_persistent(b200nn_ctx *ctx, const WOperand &w, const __half *x, int M, const Epilogue &epi) {
    constexpr int MB = 256, NE = 4;
    constexpr size_t smem = 1024 + (size_t)NS * (TW * W_BYTES + MB * BK * 2) + 64 * 128 * 4 + 256;
    static_assert(16 * NS + 48 <= 256, "barrier area too small");
    static_assert(smem <= 227 * 1024, "shared memory budget exceeded");
    static bool attr_done[16] = {};
    auto kern = f16_gemm_tc_persistent_kernel<MB, NS, NE, TW>;
    if (!attr_done[ctx->device & 15]) {
        CK(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        prefer_max_smem(kern);
        attr_done[ctx->device & 15] = true;
    }
    CUtensorMap tmap_w, tmap_w2, tmap_x;
    TRY(make_map(ctx, w.hi, w.N, w.K, 128, &tmap_w));
    TRY(make_map(ctx, TW == 2 ? w.lo : w.hi, w.N, w.K, 128, &tmap_w2));
    TRY(make_map(ctx, x, M, w.K, MB, &tmap_x));
    const int k_blocks = (w.K + BK - 1) / BK;
    const int n_tiles = (w.N + 127) / 128, m_tiles = (M + MB - 1) / MB;
    const int total = n_tiles * m_tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(std::min(total, ctx->sm_count));
    cfg.blockDim = dim3(64 + 128 * NE);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (ctx->pdl && w.constant) ? 1 : 0;
    CK(ctx, cudaLaunchKernelEx(&cfg, kern, tmap_w, tmap_w2, tmap_x, M, w.N, k_blocks, n_tiles, total, epi, ctx->dev_err));
    CK_LAUNCH(ctx, "f16_gemm_tc_persistent_kernel");
    return B200NN_OK;
}

// Token-tile width: the smallest power of two covering M, capped at 128 unless 256-row tiles still
// give every SM a block (ctx->tc_mb overrides the cap).
int pick_mb(const b200nn_ctx *ctx, int N, int M) {
    const int n_tiles = (N + 127) / 128;
    int cap = 128;
    if ((long long)n_tiles * ((M + 255) / 256) >= ctx->sm_count) cap = 256;
    if (ctx->tc_mb > 0) cap = ctx->tc_mb;
    int mb = 32;
    while (mb < M && mb < cap) mb <<= 1;
    return mb;
}

bool use_persistent(const b200nn_ctx *ctx, int N, int M, int mb) {
    return ctx->tc_persistent && mb == 256 && (long long)((N + 127) / 128) * ((M + 255) / 256) >= 2LL * ctx->sm_count;
}

int launch_terms(b200nn_ctx *ctx, const WOperand &w, int terms, const __half *x, int M, const Epilogue &epi) {
    const int mb = pick_mb(ctx, w.N, M);
    if (terms == 1) { // the weight as one fp16 matrix
        if (use_persistent(ctx, w.N, M, mb)) return launch_persistent<4, 1>(ctx, w, x, M, epi);
        switch (mb) { //            MB  NS NE TW
            case 32: return launch_cfg<32, 8, 2, 1>(ctx, w, x, M, epi);
            case 64: return launch_cfg<64, 8, 2, 1>(ctx, w, x, M, epi);
            case 128: return launch_cfg<128, 6, 4, 1>(ctx, w, x, M, epi);
            default: return launch_cfg<256, 4, 4, 1>(ctx, w, x, M, epi);
        }
    }
    // rounded weight + rounded remainder, two products per K block
    if (use_persistent(ctx, w.N, M, mb)) return launch_persistent<3, 2>(ctx, w, x, M, epi);
    switch (mb) {
        case 32: return launch_cfg<32, 5, 2, 2>(ctx, w, x, M, epi);
        case 64: return launch_cfg<64, 5, 2, 2>(ctx, w, x, M, epi);
        case 128: return launch_cfg<128, 4, 4, 2>(ctx, w, x, M, epi);
        default: return launch_cfg<256, 3, 4, 2>(ctx, w, x, M, epi);
    }
}

// One block per (128-feature tile, 64-wide K block) of the tiled int4 layout: thread r unpacks row r
// of the tile (32 packed bytes -> 64 fp16 values, exactly the values the int4 GEMM feeds its MMAs:
// the integer times the fp16 group scale, rounded to fp16) into shared memory; the block then writes
// the [128 x 64] piece of the [N,K] matrix with 128-byte row segments.
__global__ void __launch_bounds__(128)
int4_dequant_f16_kernel(const uint8_t *__restrict__ tiles, const __half *__restrict__ scales, int N, int K, int k_blocks,
                        int n_pad, int group, __half *__restrict__ out) {
    __shared__ __align__(16) uint8_t st[128 * 144]; // 128-byte rows, 16 bytes of padding each
    const int nt = blockIdx.x, kb = blockIdx.y, r = threadIdx.x;
    const uint8_t *pk = tiles + ((size_t)nt * k_blocks + kb) * TILE_BYTES + r * 16;
    const uint4 w0 = *reinterpret_cast<const uint4 *>(pk);        // k  0..31 of the block
    const uint4 w1 = *reinterpret_cast<const uint4 *>(pk + 2048); // k 32..63
    const __half2 s2 = __half2half2(scales[(size_t)((kb * TILE_K) / group) * n_pad + nt * TILE_N + r]);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint4 w = h ? w1 : w0;
        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            __half2 q[4];
            unpack8_int4(ww[j], q);
            uint4 o;
            __half2 r0 = __hmul2(q[0], s2), r1 = __hmul2(q[1], s2), r2 = __hmul2(q[2], s2), r3 = __hmul2(q[3], s2);
            o.x = *reinterpret_cast<uint32_t *>(&r0);
            o.y = *reinterpret_cast<uint32_t *>(&r1);
            o.z = *reinterpret_cast<uint32_t *>(&r2);
            o.w = *reinterpret_cast<uint32_t *>(&r3);
            *reinterpret_cast<uint4 *>(st + r * 144 + (h * 4 + j) * 16) = o; // k = 32h + 8j .. +7
        }
    }
    __syncthreads();
    // 8 threads per row: one 16-byte piece each; 16 rows per pass
    const int piece = r & 7;
    for (int row = r >> 3; row < 128; row += 16) {
        const int n = nt * TILE_N + row;
        if (n < N)
            *reinterpret_cast<uint4 *>(out + (size_t)n * K + kb * TILE_K + piece * 8) =
                *reinterpret_cast<const uint4 *>(st + row * 144 + piece * 16);
    }
}

}  // namespace

// The tensor maps need 16-byte aligned bases and row strides: K a multiple of 8.
bool f16_gemm_tc_supported(const b200nn_ctx *ctx, const F32Weight &w, int M) {
    return ctx->f32_tc && ctx->encode_tiled && w.w_nk_h && M > 4 && (w.K % 8) == 0;
}

int launch_f16_gemm_tc(b200nn_ctx *ctx, const F32Weight &w, const __half *x, int M, const Epilogue &epi) {
    if (!f16_gemm_tc_supported(ctx, w, M) || ((uintptr_t)x & 15))
        return set_error(ctx, B200NN_ERR_UNSUPPORTED, "shape not supported by the fp16 tensor-core GEMM");
    const __half *hi = (const __half *)w.w_nk_h->p;
    const WOperand op{hi, hi + (size_t)w.N * w.K, w.N, w.K, true};
    return launch_terms(ctx, op, ctx->f32_tc == 1 ? 1 : 2, x, M, epi);
}

// int4 Linear over the rows of a prefill pass: the weight is first written out as the [N,K] fp16
// matrix the int4 GEMM would have built tile by tile in tensor memory (into a buffer the context
// keeps), then multiplied by the persistent fp16 GEMM, whose K loop runs through tile boundaries with
// nothing to dequantise and whose epilogue overlaps the next tile.  The operand values are the same,
// so the results differ from the int4 GEMM's by accumulation order at most.  Taken only where the
// persistent kernel applies (at least two 256-row tiles per SM) and, while a graph is being captured,
// only if the buffer is already large enough.
bool int4_via_f16_supported(const b200nn_ctx *ctx, const Int4Weight &w, int M) {
    // (2048 rows: a prefill pass, not the LM head of a decode step, whose 393 feature tiles alone would qualify)
    return ctx->int4_via_f16 && M >= 2048 && ctx->encode_tiled && w.fast && (w.K % TILE_K) == 0 && (w.group % TILE_K) == 0 &&
           use_persistent(ctx, w.N, M, pick_mb(ctx, w.N, M)) &&
           !(ctx->capturing && (!ctx->wh || ctx->wh->bytes < (size_t)w.N * w.K * sizeof(__half)));
}

int launch_int4_via_f16(b200nn_ctx *ctx, const Int4Weight &w, const __half *x, int M, const Epilogue &epi) {
    if (!int4_via_f16_supported(ctx, w, M) || ((uintptr_t)x & 15))
        return set_error(ctx, B200NN_ERR_UNSUPPORTED, "shape not supported by the dequantise-then-multiply path");
    const size_t need = (size_t)w.N * w.K * sizeof(__half);
    if (!ctx->wh || ctx->wh->bytes < need) {
        ctx->wh.reset();
        TRY(dev_alloc(ctx, need, &ctx->wh));
    }
    int4_dequant_f16_kernel<<<dim3(w.n_tiles, w.k_blocks), 128, 0, ctx->stream>>>(
        (const uint8_t *)w.tiled->p, (const __half *)w.scales_h->p, w.N, w.K, w.k_blocks, w.n_pad, w.group, (__half *)ctx->wh->p);
    CK_LAUNCH(ctx, "int4_dequant_f16_kernel");
    const WOperand op{(const __half *)ctx->wh->p, nullptr, w.N, w.K, false};
    return launch_terms(ctx, op, 1, x, M, epi);
}
