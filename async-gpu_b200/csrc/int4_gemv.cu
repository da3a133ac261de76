// Group-wise int4 weight-only Linear on CUDA cores.
//
//   int4_gemv_kernel   few input rows (decode of one or two sequences): HBM-bound streaming of the
//                      tiled nibbles with 128-bit coalesced loads (two K blocks per thread in
//                      flight, the first ones issued before the wait on the preceding kernel:
//                      weights do not depend on it), in-register dequantisation, f32 accumulation.
//                      K is split four ways inside a block and up to eight ways across the blocks of
//                      a thread-block cluster; the cluster's partial sums are reduced through
//                      distributed shared memory by the cluster's first block (fixed order, no
//                      global scratch, no atomics), which then runs the fused bias / activation /
//                      residual / KV-cache epilogue.
//   int4_naive_kernel  any K%8==0 and any group size, reference layout, one thread per output as
//                      crates/kernel/gpu-kernel-compute/src/compute_gemm.rs:2849-2910 does.
//
// Both compute y[m,n] = sum_k x[m,k] * (nibble(k,n)-8) * scale[k/group,n] (+ bias[n]).
#include <cooperative_groups.h>

#include "device_utils.cuh"

namespace cg = cooperative_groups;

static constexpr int GEMV_THREADS = 512; // 128 weight rows x 4 K slices
static constexpr int GEMV_SLICES = 4;

template <int MT>
__device__ __forceinline__ void gemv_block_fma(const uint4 &wa, const uint4 &wb, float s, const float *xb, int len,
                                               float (&acc)[MT]) {
    const uint32_t w[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
    float part[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) part[m] = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        __half2 q[4];
        unpack8_int4(w[j], q);
        const float2 f0 = __half22float2(q[0]), f1 = __half22float2(q[1]);
        const float2 f2 = __half22float2(q[2]), f3 = __half22float2(q[3]);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const float4 xa = *reinterpret_cast<const float4 *>(xb + m * len + 8 * j);
            const float4 xc = *reinterpret_cast<const float4 *>(xb + m * len + 8 * j + 4);
            float p = part[m];
            p = fmaf(xa.x, f0.x, p); p = fmaf(xa.y, f0.y, p);
            p = fmaf(xa.z, f1.x, p); p = fmaf(xa.w, f1.y, p);
            p = fmaf(xc.x, f2.x, p); p = fmaf(xc.y, f2.y, p);
            p = fmaf(xc.z, f3.x, p); p = fmaf(xc.w, f3.y, p);
            part[m] = p;
        }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = fmaf(s, part[m], acc[m]);
}

// grid (n_tiles, splits), cluster (1, splits, 1): the blocks of a cluster share one 128-row tile.
template <int MT, typename XT>
__global__ void __launch_bounds__(GEMV_THREADS)
int4_gemv_kernel(const uint4 *__restrict__ tiles, const __half *__restrict__ scales, const XT *__restrict__ x,
                 int m_valid, int m0, int K, int N, int k_blocks, int n_pad, int group, int kb_per_split,
                 Epilogue epi) {
    extern __shared__ float smem_f[];
    cg::cluster_group cluster = cg::this_cluster();
    const int nt = blockIdx.x, split = blockIdx.y, splits = gridDim.y;
    const int tid = threadIdx.x, r = tid & 127, slice = tid >> 7;
    const int kb0 = split * kb_per_split;
    const int kb1 = min(kb0 + kb_per_split, k_blocks);
    const int len = kb_per_split * 64;
    const int n = nt * TILE_N + r;
    float *xs = smem_f;                       // [MT][len] activations of this block's K range
    float *red = smem_f + MT * len;           // [GEMV_SLICES][MT][128] slice sums
    float *part = red + GEMV_SLICES * MT * 128; // [MT][128] this block's partial tile (read by the cluster)
    pdl_trigger();

    // weights and scales of the first two K blocks of this thread: issued before the wait on the
    // previous kernel (they are constants), so that their DRAM latency overlaps its tail
    const uint4 *tile0 = tiles + (size_t)nt * k_blocks * (TILE_BYTES / 16);
    auto load_block = [&](int kb, uint4 &a, uint4 &b, float &s) {
        const uint4 *tp = tile0 + (size_t)kb * (TILE_BYTES / 16);
        a = __ldg(tp + r);
        b = __ldg(tp + 128 + r);
        s = __half2float(scales[(size_t)((kb * 64) / group) * n_pad + n]);
    };
    int kb = kb0 + slice;
    uint4 a0 = make_uint4(0, 0, 0, 0), b0 = a0, a1 = a0, b1 = a0;
    float s0 = 0.0f, s1 = 0.0f;
    bool v0 = kb < kb1, v1 = kb + GEMV_SLICES < kb1;
    if (v0) load_block(kb, a0, b0, s0);
    if (v1) load_block(kb + GEMV_SLICES, a1, b1, s1);

    pdl_wait();
    for (int i = tid; i < MT * len; i += GEMV_THREADS) {
        const int m = i / len, kk = i - m * len;
        const int k = kb0 * 64 + kk;
        xs[i] = (m < m_valid && k < kb1 * 64) ? load_as_float<XT>(x, (size_t)m * K + k) : 0.0f;
    }
    __syncthreads();

    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.0f;
    while (v0) {
        const uint4 ca = a0, cb = b0;
        const float cs = s0;
        const int ckb = kb;
        a0 = a1; b0 = b1; s0 = s1; v0 = v1;
        kb += GEMV_SLICES;
        v1 = kb + GEMV_SLICES < kb1;
        if (v1) load_block(kb + GEMV_SLICES, a1, b1, s1); // stays two K blocks ahead
        gemv_block_fma<MT>(ca, cb, cs, xs + (ckb - kb0) * 64, len, acc);
    }

#pragma unroll
    for (int m = 0; m < MT; ++m) red[(slice * MT + m) * 128 + r] = acc[m];
    __syncthreads();
    if (slice == 0) {
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            float t = 0.0f;
#pragma unroll
            for (int sl = 0; sl < GEMV_SLICES; ++sl) t += red[(sl * MT + m) * 128 + r];
            part[m * 128 + r] = t;
        }
    }
    cluster.sync(); // every block's partial tile is in its shared memory
    if (cluster.block_rank() == 0 && slice == 0) { // warps 0..3: 32 consecutive features each
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m >= m_valid) break;
            float t = 0.0f;
            for (int sp = 0; sp < splits; ++sp) // fixed order: the result does not depend on timing
                t += cluster.map_shared_rank(part, sp)[m * 128 + r];
            if (n < N) epi_apply(epi, m0 + m, n, t);
            if (epi.amax_val) epi_argmax1(epi, m0 + m, n, t + (epi.bias && n < N ? epi.bias[n] : 0.0f), n < N);
        }
    }
    cluster.sync(); // no block leaves while its shared memory may still be read
}

template <typename XT>
__global__ void int4_naive_kernel(const uint32_t *__restrict__ packed, const float *__restrict__ scales,
                                  const XT *__restrict__ x, int M, int N, int K, int group, Epilogue epi) {
    size_t id = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (id >= (size_t)M * N) return;
    int row = id / N, col = id % N;
    float acc = 0.0f;
    for (int kp = 0; kp < K / 8; ++kp) {
        uint32_t w = packed[(size_t)kp * N + col];
#pragma unroll
        for (int bit = 0; bit < 8; ++bit) {
            int ki = kp * 8 + bit;
            int q = (int)((w >> (bit * 4)) & 0xFu) - 8;
            float wf = (float)q * scales[(size_t)(ki / group) * N + col];
            acc = fmaf(load_as_float<XT>(x, (size_t)row * K + ki), wf, acc);
        }
    }
    epi_apply(epi, row, col, acc);
}

int launch_int4_naive(b200nn_ctx *ctx, const Int4Weight &w, const void *x, bool x_half, int M, const Epilogue &epi) {
    if (M <= 0) return B200NN_OK;
    if (!w.ref_packed) return set_error(ctx, B200NN_ERR_UNSUPPORTED, "int4 weight has no reference-layout copy");
    size_t total = (size_t)M * w.N;
    int grid = (int)((total + 255) / 256);
    PREFER_SMEM_ONCE(int4_naive_kernel<__half>);
    PREFER_SMEM_ONCE(int4_naive_kernel<float>);
    if (x_half)
        int4_naive_kernel<__half><<<grid, 256, 0, ctx->stream>>>((const uint32_t *)w.ref_packed->p,
                                                                 (const float *)w.ref_scales->p, (const __half *)x, M,
                                                                 w.N, w.K, w.group, epi);
    else
        int4_naive_kernel<float><<<grid, 256, 0, ctx->stream>>>((const uint32_t *)w.ref_packed->p,
                                                                (const float *)w.ref_scales->p, (const float *)x, M,
                                                                w.N, w.K, w.group, epi);
    CK_LAUNCH(ctx, "int4_naive_kernel");
    return B200NN_OK;
}

template <int MT, typename XT>
static int gemv_chunk(b200nn_ctx *ctx, const Int4Weight &w, const XT *x, int m_valid, int m0, const Epilogue &epi) {
    // K split across a cluster of up to eight blocks so that about one block per SM is resident
    int splits = (ctx->sm_count + w.n_tiles - 1) / w.n_tiles;
    splits = std::max(1, std::min(splits, 8));
    splits = std::min(splits, std::max(1, w.k_blocks / GEMV_SLICES));
    const int per = (w.k_blocks + splits - 1) / splits;
    splits = (w.k_blocks + per - 1) / per;
    const size_t smem = ((size_t)MT * per * 64 + (size_t)(GEMV_SLICES + 1) * MT * 128) * sizeof(float);
    auto kern = int4_gemv_kernel<MT, XT>;
    static bool attr_done[16] = {}; // function attributes are per device
    if (!attr_done[ctx->device & 15]) {
        CK(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        prefer_max_smem(kern);
        attr_done[ctx->device & 15] = true;
    }
    if (smem > 200 * 1024) return set_error(ctx, B200NN_ERR_UNSUPPORTED, "int4 GEMV: K too large for one cluster");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(w.n_tiles, splits);
    cfg.blockDim = dim3(GEMV_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = splits;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->pdl ? 2 : 1;
    CK(ctx, cudaLaunchKernelEx(&cfg, kern, (const uint4 *)w.tiled->p, (const __half *)w.scales_h->p, x, m_valid, m0, w.K,
                               w.N, w.k_blocks, w.n_pad, w.group, per, epi));
    CK_LAUNCH(ctx, "int4_gemv_kernel");
    return B200NN_OK;
}

template <typename XT>
static int gemv_all(b200nn_ctx *ctx, const Int4Weight &w, const XT *x, int M, const Epilogue &epi) {
    int m0 = 0;
    while (m0 < M) {
        int left = M - m0;
        const XT *xp = x + (size_t)m0 * w.K;
        if (left >= 4) {
            TRY((gemv_chunk<4, XT>(ctx, w, xp, 4, m0, epi)));
            m0 += 4;
        } else if (left >= 2) {
            TRY((gemv_chunk<2, XT>(ctx, w, xp, 2, m0, epi)));
            m0 += 2;
        } else {
            TRY((gemv_chunk<1, XT>(ctx, w, xp, 1, m0, epi)));
            m0 += 1;
        }
    }
    return B200NN_OK;
}

int launch_int4_gemv(b200nn_ctx *ctx, const Int4Weight &w, const void *x, bool x_half, int M, const Epilogue &epi) {
    if (M <= 0) return B200NN_OK;
    if (epi.ln_stats || epi.mode == EPI_RESID_LN) { // folded LayerNorms exist in the tensor-core GEMM's epilogue only
        if (!(w.fast && M > ctx->gemv_max_rows && x_half && int4_gemm_tc_supported(w, M)) || int4_via_f16_supported(ctx, w, M))
            return set_error(ctx, B200NN_ERR_UNSUPPORTED, "folded LayerNorm: this Linear does not run on the tensor-core GEMM");
        return launch_int4_gemm_tc(ctx, w, (const __half *)x, M, epi);
    }
    if (!w.fast) return launch_int4_naive(ctx, w, x, x_half, M, epi);
    return x_half ? gemv_all<__half>(ctx, w, (const __half *)x, M, epi) : gemv_all<float>(ctx, w, (const float *)x, M, epi);
}

int launch_int4_linear(b200nn_ctx *ctx, const Int4Weight &w, const void *x, bool x_half, int M, const Epilogue &epi) {
    if (M <= 0) return B200NN_OK;
    if (epi.ln_stats || epi.mode == EPI_RESID_LN) { // folded LayerNorms exist in the tensor-core GEMM's epilogue only
        if (!(w.fast && M > ctx->gemv_max_rows && x_half && int4_gemm_tc_supported(w, M)) || int4_via_f16_supported(ctx, w, M))
            return set_error(ctx, B200NN_ERR_UNSUPPORTED, "folded LayerNorm: this Linear does not run on the tensor-core GEMM");
        return launch_int4_gemm_tc(ctx, w, (const __half *)x, M, epi);
    }
    if (!w.fast) return launch_int4_naive(ctx, w, x, x_half, M, epi);
    // a prefill pass with at least two 256-row tiles per SM: dequantise once, persistent fp16 GEMM
    if (x_half && !((uintptr_t)x & 15) && int4_via_f16_supported(ctx, w, M))
        return launch_int4_via_f16(ctx, w, (const __half *)x, M, epi);
    if (M > ctx->gemv_max_rows && x_half && int4_gemm_tc_supported(w, M))
        return launch_int4_gemm_tc(ctx, w, (const __half *)x, M, epi);
    return launch_int4_gemv(ctx, w, x, x_half, M, epi);
}
