// Group-wise int4 weight-only Linear on CUDA cores.
//
//   int4_gemv_kernel   few input rows (decode of one or two sequences): HBM-bound streaming of the
//                      tiled nibbles with 128-bit coalesced loads, in-register dequantisation,
//                      f32 accumulation, K split across the two thread slices of a block, across
//                      blocks (deterministic: the last block to arrive sums the partials in split
//                      order) and the fused bias / activation / residual / KV-cache epilogue.
//   int4_naive_kernel  any K%8==0 and any group size, reference layout, one thread per output as
//                      crates/kernel/gpu-kernel-compute/src/compute_gemm.rs:2849-2910 does.
//
// Both compute y[m,n] = sum_k x[m,k] * (nibble(k,n)-8) * scale[k/group,n] (+ bias[n]).
#include "device_utils.cuh"

template <int MT, typename XT>
__global__ void __launch_bounds__(256)
int4_gemv_kernel(const uint4 *__restrict__ tiles, const __half *__restrict__ scales, const XT *__restrict__ x,
                 int m_valid, int m0, int K, int N, int k_blocks, int n_pad, int group, int kb_per_split,
                 Epilogue epi, float *__restrict__ scratch, unsigned *__restrict__ counters) {
    extern __shared__ float xs[]; // [MT][kb_per_split*64], then the cross-slice buffer [MT][128]
    __shared__ int is_last;
    const int nt = blockIdx.x, split = blockIdx.y, splits = gridDim.y;
    const int tid = threadIdx.x, r = tid & 127, slice = tid >> 7;
    const int kb0 = split * kb_per_split;
    const int kb1 = min(kb0 + kb_per_split, k_blocks);
    const int len = kb_per_split * 64;
    const int n = nt * TILE_N + r;
    pdl_trigger();
    pdl_wait();

    for (int i = tid; i < MT * len; i += 256) {
        int m = i / len, kk = i - m * len;
        int k = kb0 * 64 + kk;
        xs[i] = (m < m_valid && k < kb1 * 64) ? load_as_float<XT>(x, (size_t)m * K + k) : 0.0f;
    }
    __syncthreads();

    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.0f;

    for (int kb = kb0 + slice; kb < kb1; kb += 2) {
        const uint4 *tp = tiles + ((size_t)nt * k_blocks + kb) * (TILE_BYTES / 16);
        uint4 wa = tp[r], wb = tp[128 + r];
        float s = __half2float(scales[(size_t)((kb * 64) / group) * n_pad + n]);
        uint32_t w[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
        float part[MT];
#pragma unroll
        for (int m = 0; m < MT; ++m) part[m] = 0.0f;
        const float *xb = xs + (kb - kb0) * 64;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            __half2 q[4];
            unpack8_int4(w[j], q);
            float2 f0 = __half22float2(q[0]), f1 = __half22float2(q[1]);
            float2 f2 = __half22float2(q[2]), f3 = __half22float2(q[3]);
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

    // slice 1 hands its sums to slice 0
    float *xred = xs + MT * len;
    if (slice == 1) {
#pragma unroll
        for (int m = 0; m < MT; ++m) xred[m * 128 + r] = acc[m];
    }
    __syncthreads();
    if (slice == 0) {
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[m] += xred[m * 128 + r];
    }

    if (splits == 1) {
        if (slice == 0 && n < N) {
#pragma unroll
            for (int m = 0; m < MT; ++m)
                if (m < m_valid) epi_apply(epi, m0 + m, n, acc[m]);
        }
        return;
    }
    // partial sums -> scratch [split][MT][n_pad]; the last block of this tile reduces them
    if (slice == 0) {
#pragma unroll
        for (int m = 0; m < MT; ++m) scratch[((size_t)split * MT + m) * n_pad + n] = acc[m];
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        unsigned prev = atomicAdd(&counters[nt], 1u);
        is_last = (prev == (unsigned)(splits - 1));
        if (is_last) counters[nt] = 0u;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if (slice == 0 && n < N) {
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m >= m_valid) break;
            float t = 0.0f;
            for (int sp = 0; sp < splits; ++sp) t += __ldcg(&scratch[((size_t)sp * MT + m) * n_pad + n]);
            epi_apply(epi, m0 + m, n, t);
        }
    }
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
    // choose the K split so that the grid is about two waves of blocks and a split is <= 16 blocks
    int target = 2 * ctx->sm_count;
    int splits = (target + w.n_tiles - 1) / w.n_tiles;
    if (splits > w.k_blocks) splits = w.k_blocks;
    if (splits < 1) splits = 1;
    int per = (w.k_blocks + splits - 1) / splits;
    if (per > 16) per = 16;
    if (per & 1) per += 1; // both slices get work
    splits = (w.k_blocks + per - 1) / per;
    size_t smem = (size_t)MT * per * 64 * 4 + (size_t)MT * 128 * 4;
    if (splits > 1) TRY(ensure_scratch(ctx, (size_t)splits * MT * w.n_pad * 4, (size_t)w.n_tiles));
    dim3 grid(w.n_tiles, splits);
    PREFER_SMEM_ONCE((int4_gemv_kernel<MT, XT>));
    launch_pdl(ctx, int4_gemv_kernel<MT, XT>, grid, dim3(256), smem, (const uint4 *)w.tiled->p,
               (const __half *)w.scales_h->p, x, m_valid, m0, w.K, w.N, w.k_blocks, w.n_pad, w.group, per, epi, ctx->scratch,
               ctx->counters);
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
    if (!w.fast) return launch_int4_naive(ctx, w, x, x_half, M, epi);
    return x_half ? gemv_all<__half>(ctx, w, (const __half *)x, M, epi) : gemv_all<float>(ctx, w, (const float *)x, M, epi);
}

int launch_int4_linear(b200nn_ctx *ctx, const Int4Weight &w, const void *x, bool x_half, int M, const Epilogue &epi) {
    if (M <= 0) return B200NN_OK;
    if (!w.fast) return launch_int4_naive(ctx, w, x, x_half, M, epi);
    if (M > ctx->gemv_max_rows && x_half && int4_gemm_tc_supported(w, M))
        return launch_int4_gemm_tc(ctx, w, (const __half *)x, M, epi);
    return launch_int4_gemv(ctx, w, x, x_half, M, epi);
}
