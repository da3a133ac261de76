// Attention over the fp16 KV cache [sequence][head][capacity][64] (head_dim is 64 for every GPT-2
// size, as the reference's kernels assume: compute_transformer.rs:597-816, flash_attn_v3.cu:29-34).
//
//   decode_attn_kernel   one query row per (sequence, head) against ctx cached positions: streams K
//                        and V rows (128 B each) with 16-byte loads, 8 lanes per row, online softmax
//                        in f32, split over the context across blocks when (sequences x heads) is
//                        too small to fill the GPU; the last block to arrive merges the partial
//                        (max, sum, output) triples in split order.  Replaces flash_attention_kv
//                        (compute_transformer.rs:1076-1288) and the host loop around it
//                        (layers/attention.rs:133-178).
//   prefill_attn_kernel  causal attention of S new rows per sequence on CUDA cores (first version of
//                        the prefill path; 64 queries per block, K/V tiles staged in shared memory).
//
// Scores are q.k/sqrt(64); softmax is computed with exp2 on scores pre-multiplied by log2(e).
#include "device_utils.cuh"

static constexpr float ATT_SCALE_LOG2E = 0.125f * 1.4426950408889634f;
static constexpr float NEG_BIG = -1.0e30f;

__device__ __forceinline__ void half8_to_float(const uint4 &u, float (&f)[8]) {
    const __half2 *h = reinterpret_cast<const __half2 *>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 t = __half22float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}

template <typename QT, typename OT>
__global__ void __launch_bounds__(128, 6)
decode_attn_kernel(const QT *__restrict__ q, int ldq, const __half *__restrict__ kc, const __half *__restrict__ vc,
                   int H, int cap, const int *__restrict__ pos_ptr, int pos_off, OT *__restrict__ out, int ldo,
                   float *__restrict__ scratch, unsigned *__restrict__ counters) {
    __shared__ float sm_m[16], sm_l[16];
    __shared__ float sm_acc[16][64];
    __shared__ int is_last;
    const int h = blockIdx.x, b = blockIdx.y, split = blockIdx.z, n_splits = gridDim.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 3, c = lane & 7;
    pdl_trigger();
    pdl_wait();
    int ctx = (pos_ptr ? *pos_ptr : 0) + pos_off + 1;
    if (ctx > cap) ctx = cap;
    int chunk = (((ctx + n_splits - 1) / n_splits) + 15) & ~15;
    const int p0 = split * chunk, p1 = min(p0 + chunk, ctx);

    float qf[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
        qf[i] = load_as_float<QT>(q, (size_t)b * ldq + h * 64 + c * 8 + i) * ATT_SCALE_LOG2E;

    const size_t base = ((size_t)b * H + h) * cap;
    const uint4 *kp = reinterpret_cast<const uint4 *>(kc + base * 64);
    const uint4 *vp = reinterpret_cast<const uint4 *>(vc + base * 64);

    float m = NEG_BIG, l = 0.0f, acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.0f;

    constexpr int R = 4; // rows per lane group per trip: R x (K + V) 16-byte loads in flight per thread
    for (int jw = p0 + warp * 4; jw < p1; jw += 16 * R) { // warp-uniform trip count (full-mask shuffles)
        // rows jw+g, jw+g+16, ...: all loads are issued before any math
        uint4 kr[R], vr[R];
        bool valid[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int j = jw + g + 16 * r;
            valid[r] = j < p1;
            kr[r] = make_uint4(0, 0, 0, 0);
            vr[r] = kr[r];
            if (valid[r]) {
                kr[r] = __ldg(kp + (size_t)j * 8 + c);
                vr[r] = __ldg(vp + (size_t)j * 8 + c);
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

    const int grp = warp * 4 + g;
    if (c == 0) { sm_m[grp] = m; sm_l[grp] = l; }
#pragma unroll
    for (int i = 0; i < 8; ++i) sm_acc[grp][c * 8 + i] = acc[i];
    __syncthreads();

    float M = NEG_BIG, L = 0.0f, O = 0.0f;
    if (tid < 64) {
#pragma unroll
        for (int i = 0; i < 16; ++i) M = fmaxf(M, sm_m[i]);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            float w = exp2f(sm_m[i] - M);
            L += sm_l[i] * w;
            O += sm_acc[i][tid] * w;
        }
    }
    if (n_splits == 1) {
        if (tid < 64) {
            float r = O / L;
            size_t oi = (size_t)b * ldo + h * 64 + tid;
            if constexpr (sizeof(OT) == 2) out[oi] = __float2half_rn(r); else out[oi] = r;
        }
        return;
    }
    // partial record: [M, L, O[64]] per (b, h, split)
    float *rec = scratch + (((size_t)b * H + h) * n_splits + split) * 66;
    if (tid < 64) {
        rec[2 + tid] = O;
        if (tid == 0) { rec[0] = M; rec[1] = L; }
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        unsigned prev = atomicAdd(&counters[b * H + h], 1u);
        is_last = (prev == (unsigned)(n_splits - 1));
        if (is_last) counters[b * H + h] = 0u;
    }
    __syncthreads();
    if (!is_last || tid >= 64) return;
    __threadfence();
    const float *r0 = scratch + ((size_t)b * H + h) * n_splits * 66;
    float Mx = NEG_BIG;
    for (int s = 0; s < n_splits; ++s) Mx = fmaxf(Mx, __ldcg(r0 + s * 66));
    float Ls = 0.0f, Os = 0.0f;
    for (int s = 0; s < n_splits; ++s) {
        float w = exp2f(__ldcg(r0 + s * 66) - Mx);
        Ls += __ldcg(r0 + s * 66 + 1) * w;
        Os += __ldcg(r0 + s * 66 + 2 + tid) * w;
    }
    float r = Os / Ls;
    size_t oi = (size_t)b * ldo + h * 64 + tid;
    if constexpr (sizeof(OT) == 2) out[oi] = __float2half_rn(r); else out[oi] = r;
}

int launch_decode_attention(b200nn_ctx *ctx, const void *q, bool q_half, int ldq, const __half *kc,
                            const __half *vc, int B, int H, int cap, const int *pos_ptr, int pos_off, void *out,
                            bool out_half, int max_ctx_hint) {
    if (B <= 0) return B200NN_OK;
    int pairs = B * H;
    int n_splits = (4 * ctx->sm_count + pairs - 1) / pairs;
    int max_splits = (max_ctx_hint + 63) / 64;
    if (n_splits > max_splits) n_splits = max_splits;
    if (n_splits > 32) n_splits = 32;
    if (n_splits < 1) n_splits = 1;
    if (n_splits > 1) TRY(ensure_scratch(ctx, (size_t)pairs * n_splits * 66 * 4, (size_t)pairs));
    dim3 grid(H, B, n_splits);
    int ldo = H * 64;
#define DA(QT, OT)                                                                                                  \
    {                                                                                                               \
        PREFER_SMEM_ONCE((decode_attn_kernel<QT, OT>));                                                             \
        launch_pdl(ctx, decode_attn_kernel<QT, OT>, grid, dim3(128), 0, (const QT *)q, ldq, kc, vc, H, cap, pos_ptr, \
                   pos_off, (OT *)out, ldo, ctx->scratch, ctx->counters);                                           \
    }
    if (q_half && out_half) DA(__half, __half)
    else if (q_half) DA(__half, float)
    else if (out_half) DA(float, __half)
    else DA(float, float)
#undef DA
    CK_LAUNCH(ctx, "decode_attn_kernel");
    return B200NN_OK;
}

// ---------------------------------------------------------------------------------------------
// Prefill: S new query rows per sequence at absolute positions past..past+S-1; row i attends to
// cached positions 0..past+i (layers/attention.rs:69-102 forward_causal when past == 0,
// 112-184 forward_cached otherwise).  Four threads share a query row, 16 dims each.
// ---------------------------------------------------------------------------------------------
template <typename QT, typename OT>
__global__ void __launch_bounds__(256)
prefill_attn_kernel(const QT *__restrict__ q, int ldq, const __half *__restrict__ kc, const __half *__restrict__ vc,
                    int H, int cap, int S, int past, OT *__restrict__ out, int ldo) {
    __shared__ __align__(16) __half ks[64][64];
    __shared__ __align__(16) __half vs[64][64];
    const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, qi = tid >> 2, qd = tid & 3;
    const int s_row = qt * 64 + qi;
    const bool q_valid = s_row < S;
    const int a = past + s_row; // absolute position of this query
    float qf[16];
#pragma unroll
    for (int e = 0; e < 16; ++e)
        qf[e] = q_valid ? load_as_float<QT>(q, ((size_t)b * S + s_row) * ldq + h * 64 + qd * 16 + e) * ATT_SCALE_LOG2E
                        : 0.0f;
    const size_t base = ((size_t)b * H + h) * cap;
    const uint4 *kp = reinterpret_cast<const uint4 *>(kc + base * 64);
    const uint4 *vp = reinterpret_cast<const uint4 *>(vc + base * 64);
    const int kv_end = min(past + min(S, qt * 64 + 64), cap); // keys this block can see

    float m = NEG_BIG, l = 0.0f, acc[16];
#pragma unroll
    for (int e = 0; e < 16; ++e) acc[e] = 0.0f;

    for (int j0 = 0; j0 < kv_end; j0 += 64) {
        __syncthreads();
        for (int i = tid; i < 512; i += 256) {
            int r = i >> 3, cc = i & 7;
            uint4 kz = make_uint4(0, 0, 0, 0), vz = kz;
            if (j0 + r < kv_end) {
                kz = kp[(size_t)(j0 + r) * 8 + cc];
                vz = vp[(size_t)(j0 + r) * 8 + cc];
            }
            reinterpret_cast<uint4 *>(&ks[r][0])[cc] = kz;
            reinterpret_cast<uint4 *>(&vs[r][0])[cc] = vz;
        }
        __syncthreads();
        const int jn = min(64, kv_end - j0);
        for (int c0 = 0; c0 < jn; c0 += 8) {
            float sc[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const uint4 *kr = reinterpret_cast<const uint4 *>(&ks[c0 + u][qd * 16]);
                float kf[8], d = 0.0f;
                half8_to_float(kr[0], kf);
#pragma unroll
                for (int e = 0; e < 8; ++e) d = fmaf(qf[e], kf[e], d);
                half8_to_float(kr[1], kf);
#pragma unroll
                for (int e = 0; e < 8; ++e) d = fmaf(qf[8 + e], kf[e], d);
                d += __shfl_xor_sync(0xffffffffu, d, 1);
                d += __shfl_xor_sync(0xffffffffu, d, 2);
                sc[u] = d;
            }
            float m_new = m;
            bool ok[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                int j = j0 + c0 + u;
                ok[u] = q_valid && j <= a && j < kv_end;
                if (ok[u]) m_new = fmaxf(m_new, sc[u]);
            }
            float corr = exp2f(m - m_new);
            l *= corr;
#pragma unroll
            for (int e = 0; e < 16; ++e) acc[e] *= corr;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                float p = ok[u] ? exp2f(sc[u] - m_new) : 0.0f;
                l += p;
                const uint4 *vr = reinterpret_cast<const uint4 *>(&vs[c0 + u][qd * 16]);
                float vf[8];
                half8_to_float(vr[0], vf);
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[e] = fmaf(p, vf[e], acc[e]);
                half8_to_float(vr[1], vf);
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[8 + e] = fmaf(p, vf[e], acc[8 + e]);
            }
            m = m_new;
        }
    }
    if (q_valid) {
        float inv = 1.0f / l;
        size_t oi = ((size_t)b * S + s_row) * ldo + h * 64 + qd * 16;
#pragma unroll
        for (int e = 0; e < 16; ++e) {
            float r = acc[e] * inv;
            if constexpr (sizeof(OT) == 2) out[oi + e] = __float2half_rn(r); else out[oi + e] = r;
        }
    }
}

int launch_prefill_attention(b200nn_ctx *ctx, const void *q, bool q_half, int ldq, const __half *kc,
                             const __half *vc, int B, int H, int cap, int S, int past, void *out, bool out_half) {
    if (B <= 0 || S <= 0) return B200NN_OK;
    dim3 grid((S + 63) / 64, H, B);
    int ldo = H * 64;
#define PA(QT, OT)                                                                                                \
    {                                                                                                             \
        PREFER_SMEM_ONCE((prefill_attn_kernel<QT, OT>));                                                          \
        prefill_attn_kernel<QT, OT><<<grid, 256, 0, ctx->stream>>>((const QT *)q, ldq, kc, vc, H, cap, S, past,    \
                                                                   (OT *)out, ldo);                               \
    }
    if (q_half && out_half) PA(__half, __half)
    else if (q_half) PA(__half, float)
    else if (out_half) PA(float, __half)
    else PA(float, float)
#undef PA
    CK_LAUNCH(ctx, "prefill_attn_kernel");
    return B200NN_OK;
}
