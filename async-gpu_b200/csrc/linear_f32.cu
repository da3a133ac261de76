// f32 Linear (y = x * W + b with W stored [K,N]) on CUDA cores with the shared fused epilogue.
// Replaces the reference's matmul dispatch + bias_add pair (ops/gemm.rs:20-299, reshape.rs:112-156)
// for the f32 model family.  Two kernels:
//   f32_gemv_kernel  M <= 4 rows: one thread per output column, weights read once, coalesced
//                    along N, K split across blocks with the deterministic last-block reduction.
//   f32_gemm_kernel  64x64x16 shared-memory tiles, 4x4 outputs per thread, any M.
#include "device_utils.cuh"

template <int MT, typename XT>
__global__ void __launch_bounds__(256)
f32_gemv_kernel(const float *__restrict__ w, const XT *__restrict__ x, int m_valid, int m0, int K, int N,
                int k_per_split, Epilogue epi, float *__restrict__ scratch, unsigned *__restrict__ counters) {
    extern __shared__ float xs[]; // [MT][k_per_split]
    __shared__ int is_last;
    const int n = blockIdx.x * 256 + threadIdx.x;
    const int split = blockIdx.y, splits = gridDim.y;
    const int k0 = split * k_per_split, k1 = min(k0 + k_per_split, K);
    for (int i = threadIdx.x; i < MT * k_per_split; i += 256) {
        int m = i / k_per_split, kk = i - m * k_per_split;
        xs[i] = (m < m_valid && k0 + kk < k1) ? load_as_float<XT>(x, (size_t)m * K + k0 + kk) : 0.0f;
    }
    __syncthreads();
    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.0f;
    if (n < N) {
        const float *wp = w + (size_t)k0 * N + n;
        int k = 0, len = k1 - k0;
        for (; k + 4 <= len; k += 4) {
            float w0 = wp[(size_t)k * N], w1 = wp[(size_t)(k + 1) * N], w2 = wp[(size_t)(k + 2) * N],
                  w3 = wp[(size_t)(k + 3) * N];
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                const float *xm = xs + m * k_per_split + k;
                acc[m] = fmaf(xm[0], w0, acc[m]);
                acc[m] = fmaf(xm[1], w1, acc[m]);
                acc[m] = fmaf(xm[2], w2, acc[m]);
                acc[m] = fmaf(xm[3], w3, acc[m]);
            }
        }
        for (; k < len; ++k) {
            float w0 = wp[(size_t)k * N];
#pragma unroll
            for (int m = 0; m < MT; ++m) acc[m] = fmaf(xs[m * k_per_split + k], w0, acc[m]);
        }
    }
    if (splits == 1) {
        if (n < N)
#pragma unroll
            for (int m = 0; m < MT; ++m)
                if (m < m_valid) epi_apply(epi, m0 + m, n, acc[m]);
        return;
    }
    if (n < N)
#pragma unroll
        for (int m = 0; m < MT; ++m) scratch[((size_t)split * MT + m) * N + n] = acc[m];
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned prev = atomicAdd(&counters[blockIdx.x], 1u);
        is_last = (prev == (unsigned)(splits - 1));
        if (is_last) counters[blockIdx.x] = 0u;
    }
    __syncthreads();
    if (!is_last || n >= N) return;
    __threadfence();
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        if (m >= m_valid) break;
        float t = 0.0f;
        for (int sp = 0; sp < splits; ++sp) t += __ldcg(&scratch[((size_t)sp * MT + m) * N + n]);
        epi_apply(epi, m0 + m, n, t);
    }
}

template <typename XT>
__global__ void __launch_bounds__(256)
f32_gemm_kernel(const float *__restrict__ w, const XT *__restrict__ x, int M, int K, int N, Epilogue epi) {
    __shared__ float xs[16][64 + 1]; // [k][m]
    __shared__ float ws[16][64];     // [k][n]
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m_base = blockIdx.y * 64, n_base = blockIdx.x * 64;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
    for (int k0 = 0; k0 < K; k0 += 16) {
        for (int i = threadIdx.x; i < 64 * 16; i += 256) {
            int mm = i >> 4, kk = i & 15; // consecutive threads walk k: contiguous in x
            int m = m_base + mm, k = k0 + kk;
            xs[kk][mm] = (m < M && k < K) ? load_as_float<XT>(x, (size_t)m * K + k) : 0.0f;
        }
        for (int i = threadIdx.x; i < 16 * 64; i += 256) {
            int kk = i >> 6, nn = i & 63;
            int k = k0 + kk, n = n_base + nn;
            ws[kk][nn] = (k < K && n < N) ? w[(size_t)k * N + n] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[kk][tx + 16 * j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int m = m_base + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int n = n_base + tx + 16 * j;
            if (n < N) epi_apply(epi, m, n, acc[i][j]);
        }
    }
}

template <int MT, typename XT>
static int f32_gemv_chunk(b200nn_ctx *ctx, const F32Weight &w, const XT *x, int m_valid, int m0, const Epilogue &epi) {
    int col_blocks = (w.N + 255) / 256;
    int target = 2 * ctx->sm_count;
    int splits = (target + col_blocks - 1) / col_blocks;
    int per = (w.K + splits - 1) / splits;
    if (per < 64) per = 64;
    if (per > 2048) per = 2048;
    per = (per + 3) & ~3;
    splits = (w.K + per - 1) / per;
    if (splits > 1) TRY(ensure_scratch(ctx, (size_t)splits * MT * w.N * 4, (size_t)col_blocks));
    dim3 grid(col_blocks, splits);
    PREFER_SMEM_ONCE((f32_gemv_kernel<MT, XT>));
    f32_gemv_kernel<MT, XT><<<grid, 256, (size_t)MT * per * 4, ctx->stream>>>(
        (const float *)w.w_kn->p, x, m_valid, m0, w.K, w.N, per, epi, ctx->scratch, ctx->counters);
    CK_LAUNCH(ctx, "f32_gemv_kernel");
    return B200NN_OK;
}

template <typename XT>
static int f32_linear_t(b200nn_ctx *ctx, const F32Weight &w, const XT *x, int M, const Epilogue &epi) {
    if (M <= 4) {
        if (M == 4) return f32_gemv_chunk<4, XT>(ctx, w, x, 4, 0, epi);
        if (M >= 2) {
            TRY((f32_gemv_chunk<2, XT>(ctx, w, x, 2, 0, epi)));
            if (M == 3) return f32_gemv_chunk<1, XT>(ctx, w, x + (size_t)2 * w.K, 1, 2, epi);
            return B200NN_OK;
        }
        return f32_gemv_chunk<1, XT>(ctx, w, x, 1, 0, epi);
    }
    dim3 grid((w.N + 63) / 64, (M + 63) / 64);
    PREFER_SMEM_ONCE(f32_gemm_kernel<XT>);
    f32_gemm_kernel<XT><<<grid, 256, 0, ctx->stream>>>((const float *)w.w_kn->p, x, M, w.K, w.N, epi);
    CK_LAUNCH(ctx, "f32_gemm_kernel");
    return B200NN_OK;
}

int launch_f32_linear(b200nn_ctx *ctx, const F32Weight &w, const void *x, bool x_half, int M, const Epilogue &epi) {
    if (M <= 0) return B200NN_OK;
    if (f16_gemm_tc_supported(ctx, w, M) && !((uintptr_t)x & 15)) {
        // more than four rows: fp16 operands on the tensor cores.  f32 activations are converted once
        // into a buffer the context keeps (grown outside stream capture only).
        if (x_half) return launch_f16_gemm_tc(ctx, w, (const __half *)x, M, epi);
        const size_t need = (size_t)M * w.K * sizeof(__half);
        if (!ctx->xh || ctx->xh->bytes < need) {
            if (ctx->capturing) return set_error(ctx, B200NN_ERR_UNSUPPORTED, "activation buffer cannot grow during graph capture");
            ctx->xh.reset();
            TRY(dev_alloc(ctx, need, &ctx->xh));
        }
        TRY(launch_f32_to_half(ctx, (const float *)x, (__half *)ctx->xh->p, (size_t)M * w.K));
        return launch_f16_gemm_tc(ctx, w, (const __half *)ctx->xh->p, M, epi);
    }
    return x_half ? f32_linear_t<__half>(ctx, w, (const __half *)x, M, epi)
                  : f32_linear_t<float>(ctx, w, (const float *)x, M, epi);
}
