// int4 weight-only Linear on the 5th-generation tensor cores (tcgen05, accumulators in TMEM).
//
//   y[m,n] = sum_k x[m,k] * (nibble(k,n)-8) * scale[k/group,n]  (+ bias, activation, residual, KV write)
//
// The weight is the MMA's A operand (128 output features = the 128 TMEM lanes), the activations are
// the B operand (MB token rows = the MMA's N, 16..256), so a decode batch of 32 costs a 128x32 MMA
// instead of a 128-row tile padded with 96 dead rows, and the accumulator row a thread reads back
// in the epilogue is one output feature: its group scale and bias are per-thread scalars.
//
// Block = 352 threads, one 128-feature tile x one K split x one MB-row tile:
//   warp 0      streams packed 4 KB weight tiles HBM -> shared memory with 1-D bulk async copies
//               (the tiles are contiguous in the re-tiled layout), NP stages deep;
//   warp 1      loads the fp16 activation tile [MB x 64] through a 2-D tensor map with 128-byte
//               swizzle, which lands it in the canonical K-major UMMA layout;
//   warp 2      owns TMEM (alloc / dealloc) and issues four tcgen05.mma (K=16 each) per 64-wide
//               K block, then tcgen05.commit to release the operand stage;
//   warps 3-10  dequantise: one thread per (row, half K block): 16 packed bytes -> 32 fp16 values
//               (lop3 magic-number unpack, exact integer, times the fp16 group scale) written into
//               the 128-byte-swizzled A tile; afterwards the same warps read the accumulator from
//               TMEM (each warp its own 32-lane quadrant) and run the epilogue.
// K can be split across blocks; partial tiles go to scratch and the last block to arrive sums them
// in split order (deterministic) before the epilogue.
//
// Every wait on an mbarrier is bounded: when it runs out the block records a code in the device
// error word, all roles leave their loops, TMEM is freed and the kernel returns.
#include <cuda.h>

#include "device_utils.cuh"
#include "tc_ptx.cuh"

namespace {

constexpr int kThreads = 352;
constexpr int kDequantThreads = 256;
constexpr int A_BYTES = TILE_N * TILE_K * 2; // 16384: dequantised fp16 tile

enum : uint32_t { ERR_P_EMPTY = 0x101, ERR_X_EMPTY, ERR_A_FULL, ERR_X_FULL, ERR_P_FULL, ERR_A_EMPTY, ERR_ACC };

struct Smem {
    uint32_t a, x, p;                                   // ring bases (shared-space addresses)
    uint32_t p_full, p_empty, x_full, a_full, ax_empty; // barrier array bases
    uint32_t acc_full, tmem_slot;
};

__device__ __forceinline__ void bar_sync_dequant() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

template <int MB, int NA, int NP>
__global__ void __launch_bounds__(kThreads, 1)
int4_gemm_tc_kernel(const uint8_t *__restrict__ tiles, const __half *__restrict__ scales,
                    const __grid_constant__ CUtensorMap tmap_x, int M, int N, int k_blocks, int n_pad, int group,
                    int kb_per_split, Epilogue epi, float *__restrict__ scratch, unsigned *__restrict__ counters,
                    uint32_t *__restrict__ dev_err) {
    constexpr int X_BYTES = MB * 128;
    constexpr int TMEM_COLS = MB < 32 ? 32 : MB;
    extern __shared__ uint8_t smem_raw[];
    __shared__ int abort_flag;
    __shared__ int is_last;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nt = blockIdx.x, split = blockIdx.y, splits = gridDim.y, mt = blockIdx.z;
    const int kb0 = split * kb_per_split;
    const int nkb = min(kb_per_split, k_blocks - kb0);

    // carve shared memory: operand rings 1024-byte aligned, barriers behind them
    const uint32_t base = (tc::smem_u32(smem_raw) + 1023u) & ~1023u;
    Smem S;
    S.a = base;
    S.x = S.a + NA * A_BYTES;
    S.p = S.x + NA * X_BYTES;
    uint32_t b = S.p + NP * TILE_BYTES;
    S.p_full = b;            b += NP * 8;
    S.p_empty = b;           b += NP * 8;
    S.x_full = b;            b += NA * 8;
    S.a_full = b;            b += NA * 8;
    S.ax_empty = b;          b += NA * 8;
    S.acc_full = b;          b += 8;
    S.tmem_slot = b;
    uint8_t *gen_base = smem_raw + (base - tc::smem_u32(smem_raw)); // generic pointer to `base`

    if (tid == 0) {
        abort_flag = 0;
        for (int i = 0; i < NP; ++i) {
            tc::mbar_init(S.p_full + 8 * i, 1);
            tc::mbar_init(S.p_empty + 8 * i, 8); // one arrival per dequant warp
        }
        for (int i = 0; i < NA; ++i) {
            tc::mbar_init(S.x_full + 8 * i, 1);
            tc::mbar_init(S.a_full + 8 * i, 8);
            tc::mbar_init(S.ax_empty + 8 * i, 1); // tcgen05.commit
        }
        tc::mbar_init(S.acc_full, 1);
        tc::fence_mbar_init();
    }
    if (warp == 1 && lane == 0) tc::prefetch_tmap(&tmap_x);
    if (warp == 2) tc::tmem_alloc(S.tmem_slot, TMEM_COLS);
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(gen_base + (S.tmem_slot - base));

    if (warp == 0) {
        // ---- packed weight tiles: HBM -> shared, NP stages in flight ----
        const uint8_t *src = tiles + ((size_t)nt * k_blocks + kb0) * TILE_BYTES;
        for (int i = 0; i < nkb; ++i) {
            const int s = i % NP, ph = (i / NP) & 1;
            if (!tc::mbar_wait(S.p_empty + 8 * s, ph ^ 1, &abort_flag, dev_err, ERR_P_EMPTY)) break;
            if (lane == 0) {
                tc::mbar_expect_tx(S.p_full + 8 * s, TILE_BYTES);
                tc::tma_load_1d(S.p + s * TILE_BYTES, src + (size_t)i * TILE_BYTES, TILE_BYTES, S.p_full + 8 * s);
            }
            __syncwarp();
        }
    } else if (warp == 1) {
        // ---- activation tiles [MB rows x 64 k] through the tensor map (zero fill past M) ----
        for (int i = 0; i < nkb; ++i) {
            const int s = i % NA, ph = (i / NA) & 1;
            if (!tc::mbar_wait(S.ax_empty + 8 * s, ph ^ 1, &abort_flag, dev_err, ERR_X_EMPTY)) break;
            if (lane == 0) {
                tc::mbar_expect_tx(S.x_full + 8 * s, X_BYTES);
                tc::tma_load_2d(S.x + s * X_BYTES, &tmap_x, (kb0 + i) * TILE_K, mt * MB, S.x_full + 8 * s);
            }
            __syncwarp();
        }
    } else if (warp == 2) {
        // ---- MMA issue ----
        constexpr uint32_t idesc = tc::umma_idesc_f16(128, MB);
        bool ok = true;
        for (int i = 0; i < nkb && ok; ++i) {
            const int s = i % NA, ph = (i / NA) & 1;
            ok = tc::mbar_wait(S.a_full + 8 * s, ph, &abort_flag, dev_err, ERR_A_FULL) &&
                 tc::mbar_wait(S.x_full + 8 * s, ph, &abort_flag, dev_err, ERR_X_FULL);
            if (!ok) break;
            tc::tc_fence_after_sync();
            if (lane == 0) {
                const uint64_t ad = tc::umma_desc_sw128(S.a + s * A_BYTES);
                const uint64_t bd = tc::umma_desc_sw128(S.x + s * X_BYTES);
#pragma unroll
                for (int j = 0; j < TILE_K / 16; ++j) // +32 bytes along K per MMA = +2 in the address field
                    tc::umma_f16_ss(tmem_base, ad + 2 * j, bd + 2 * j, idesc, (i | j) != 0);
                tc::umma_commit(S.ax_empty + 8 * s); // operand stage reusable once these MMAs retire
            }
            __syncwarp();
        }
        if (ok && lane == 0) tc::umma_commit(S.acc_full);
        __syncwarp();
    } else {
        // ---- dequantise, then epilogue ----
        const int t = tid - 96, row = t & 127, half = t >> 7;
        const int dw_lane0 = (lane == 0);
        const int n = nt * TILE_N + row;
        const __half *sc_ptr = scales + n;
        for (int i = 0; i < nkb; ++i) {
            const int sp = i % NP, php = (i / NP) & 1, sa = i % NA, pha = (i / NA) & 1;
            const __half sc = sc_ptr[(size_t)(((kb0 + i) * TILE_K) / group) * n_pad]; // issued before the wait
            if (!tc::mbar_wait(S.p_full + 8 * sp, php, &abort_flag, dev_err, ERR_P_FULL)) break;
            const uint4 w = *reinterpret_cast<const uint4 *>(gen_base + (S.p - base) + sp * TILE_BYTES +
                                                             (half * 128 + row) * 16);
            __syncwarp();
            if (dw_lane0) tc::mbar_arrive(S.p_empty + 8 * sp); // this warp has its packed words in registers
            if (!tc::mbar_wait(S.ax_empty + 8 * sa, pha ^ 1, &abort_flag, dev_err, ERR_A_EMPTY)) break;
            const __half2 s2 = __half2half2(sc);
            uint8_t *arow = gen_base + (S.a - base) + sa * A_BYTES + row * 128;
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
                const int chunk = half * 4 + j; // 16-byte chunk of the 128-byte row, XOR-swizzled by row
                *reinterpret_cast<uint4 *>(arow + ((chunk ^ (row & 7)) << 4)) = o;
            }
            tc::fence_proxy_async_smem(); // make the generic-proxy stores visible to the MMA's reads
            __syncwarp();
            if (dw_lane0) tc::mbar_arrive(S.a_full + 8 * sa);
        }
        bar_sync_dequant();
        if (!abort_flag) tc::mbar_wait(S.acc_full, 0, &abort_flag, dev_err, ERR_ACC);
        bar_sync_dequant();
        if (!abort_flag) {
            tc::tc_fence_after_sync();
            const int quad = warp & 3;             // TMEM lanes this warp may read: 32*quad .. +31
            const int colh = (warp - 3) >> 2;      // the two warps of a quadrant split the columns
            constexpr int COLS = MB / 2;
            const int r_loc = quad * 32 + lane;
            const int nn = nt * TILE_N + r_loc;
            const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + colh * COLS;
            const int tile_lin = mt * gridDim.x + nt;
            float *part = scratch + (((size_t)tile_lin * splits + split) * MB) * TILE_N;
#pragma unroll 1
            for (int c0 = 0; c0 < COLS; c0 += (COLS >= 16 ? 16 : 8)) {
                constexpr int W = COLS >= 16 ? 16 : 8;
                uint32_t v[W];
                if constexpr (W == 16) tc::tmem_ld_x16(taddr + c0, v); else tc::tmem_ld_x8(taddr + c0, v);
#pragma unroll
                for (int j = 0; j < W; ++j) {
                    const int c = colh * COLS + c0 + j, m = mt * MB + c;
                    const float acc = __uint_as_float(v[j]);
                    if (splits == 1) {
                        if (m < M && nn < N) epi_apply(epi, m, nn, acc);
                    } else {
                        part[(size_t)c * TILE_N + r_loc] = acc;
                    }
                }
            }
            if (splits > 1) {
                __threadfence();
                bar_sync_dequant();
                if (t == 0) {
                    unsigned prev = atomicAdd(&counters[tile_lin], 1u);
                    is_last = (prev == (unsigned)(splits - 1));
                    if (is_last) counters[tile_lin] = 0u;
                }
                bar_sync_dequant();
                if (is_last) {
                    __threadfence();
                    const float *p0 = scratch + ((size_t)tile_lin * splits * MB) * TILE_N;
                    if (nn < N) {
                        for (int c = colh * COLS; c < (colh + 1) * COLS; ++c) {
                            const int m = mt * MB + c;
                            if (m >= M) break;
                            float sum = 0.0f;
                            for (int sp = 0; sp < splits; ++sp)
                                sum += __ldcg(p0 + ((size_t)sp * MB + c) * TILE_N + r_loc);
                            epi_apply(epi, m, nn, sum);
                        }
                    }
                }
            }
        }
    }

    // ---- teardown (also the path taken after a wait gave up) ----
    if (abort_flag && warp < 2) { // let copies still in flight land before the block's memory is released
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    if (warp == 2) tc::tmem_dealloc(tmem_base, TMEM_COLS);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

template <int MB, int NA, int NP>
int launch_cfg(b200nn_ctx *ctx, const Int4Weight &w, const __half *x, int M, const Epilogue &epi) {
    constexpr size_t smem = 1024 + (size_t)NA * (A_BYTES + MB * 128) + (size_t)NP * TILE_BYTES + 256;
    static bool attr_done[16] = {};
    auto kern = int4_gemm_tc_kernel<MB, NA, NP>;
    if (!attr_done[ctx->device & 15]) {
        CK(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
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
    const int ctas_per_sm = smem <= 110 * 1024 ? 2 : 1;
    int splits = (ctx->sm_count * ctas_per_sm + base_ctas - 1) / base_ctas;
    splits = std::min(splits, std::max(1, w.k_blocks / 4)); // at least four K blocks per split
    splits = std::max(1, std::min(splits, 32));
    int per = (w.k_blocks + splits - 1) / splits;
    splits = (w.k_blocks + per - 1) / per;
    if (splits > 1)
        TRY(ensure_scratch(ctx, (size_t)base_ctas * splits * MB * TILE_N * sizeof(float), (size_t)base_ctas));
    dim3 grid(w.n_tiles, splits, m_tiles);
    kern<<<grid, kThreads, smem, ctx->stream>>>((const uint8_t *)w.tiled->p, (const __half *)w.scales_h->p, tmap, M, w.N,
                                                w.k_blocks, w.n_pad, w.group, per, epi, ctx->scratch, ctx->counters,
                                                ctx->dev_err);
    CK_LAUNCH(ctx, "int4_gemm_tc_kernel");
    return B200NN_OK;
}

}  // namespace

bool int4_gemm_tc_supported(const Int4Weight &w, int M) { return w.fast && M >= 1 && w.k_blocks >= 1; }

int launch_int4_gemm_tc(b200nn_ctx *ctx, const Int4Weight &w, const __half *x, int M, const Epilogue &epi) {
    if (!int4_gemm_tc_supported(w, M)) return set_error(ctx, B200NN_ERR_UNSUPPORTED, "shape not supported by the tensor-core GEMM");
    if (!ctx->encode_tiled) return set_error(ctx, B200NN_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled is unavailable");
    if (M <= 16) return launch_cfg<16, 3, 8>(ctx, w, x, M, epi);
    if (M <= 32) return launch_cfg<32, 3, 8>(ctx, w, x, M, epi);
    if (M <= 64) return launch_cfg<64, 3, 8>(ctx, w, x, M, epi);
    if (M <= 128) return launch_cfg<128, 3, 8>(ctx, w, x, M, epi);
    return launch_cfg<256, 3, 6>(ctx, w, x, M, epi);
}
