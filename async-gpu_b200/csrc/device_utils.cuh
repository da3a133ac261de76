// Device-side helpers shared by the kernels: activations, the Linear epilogue, reductions.
#pragma once
#include "common.h"

// Programmatic dependent launch: wait until the preceding kernel on the stream has completed and
// its writes are visible (a no-op when the kernel was not launched as a programmatic dependent),
// and allow the following kernel to begin launching.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ float gelu_tanh_f(float x) {
    // x*0.5*(1+tanh(sqrt(2/pi)*(x+0.044715x^3))): the GPT-2 form used by the reference's CPU model
    // (crates/test/gpu-test-harness/src/tests_inference.rs:3680-3685).
    // 0.5*(1+tanh(u)) == 1/(1+exp(-2u)): one exponential and one division instead of tanhf's ~25
    // instructions (the GELU of a 256x128 tile was two thirds of the FC epilogue's time).  u is
    // clamped where the result is already zero to within 1e-30 so that the exponential stays finite.
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    float inner = fmaxf(k0 * (x + k1 * x * x * x), -40.0f);
    return __fdividef(x, 1.0f + __expf(-2.0f * inner));
}

__device__ __forceinline__ float gelu_sigmoid_f(float x) {
    // x*sigmoid(1.702x): crates/kernel/gpu-kernel-compute/src/compute_transformer.rs:1486-1504.
    return x / (1.0f + __expf(-1.702f * x));
}

__device__ __forceinline__ float apply_act(float v, int act) {
    switch (act) {
        case B200NN_ACT_GELU_TANH: return gelu_tanh_f(v);
        case B200NN_ACT_GELU_SIGMOID: return gelu_sigmoid_f(v);
        case B200NN_ACT_RELU: return fmaxf(v, 0.0f);
        case B200NN_ACT_SILU: return v / (1.0f + __expf(-v));
        case B200NN_ACT_SIGMOID: return 1.0f / (1.0f + __expf(-v));
        default: return v;
    }
}

// Consumes one finished output value v (bias already added) for row m (token), column n (feature).
__device__ __forceinline__ void epi_store(const Epilogue &e, int m, int n, float v) {
    if (e.no_store) return;
    if (e.mode == EPI_RESID) {
        size_t i = (size_t)m * e.ldo + n;
        e.resid[i] += v;
        return;
    }
    if (e.mode == EPI_QKV && n >= e.d_model) {
        int c = n - e.d_model;
        __half *cache = e.kc;
        if (c >= e.d_model) {
            c -= e.d_model;
            cache = e.vc;
        }
        int head = c >> 6, el = c & 63;
        int b = m / e.rows_per_seq, s = m - b * e.rows_per_seq;
        int pos = (e.pos_ptr ? *e.pos_ptr : 0) + e.pos_off + s;
        if (pos < e.cap) cache[(((size_t)b * e.n_head + head) * e.cap + pos) * 64 + el] = __float2half_rn(v);
        return;
    }
    v = apply_act(v, e.act);
    size_t i = (size_t)m * e.ldo + n;
    if (e.out_half)
        static_cast<__half *>(e.out)[i] = __float2half_rn(v);
    else
        static_cast<float *>(e.out)[i] = v;
}

// Four consecutive columns n..n+3 (n % 4 == 0) of row m in one go: 16-byte (f32) or 8-byte (fp16)
// stores when the destination allows it, element-wise otherwise.  pos_ptr must already be folded
// into e.pos_off by the caller (it is not dereferenced here for the vector path).
__device__ __forceinline__ void epi_store4(const Epilogue &e, int m, int n, float4 v, int N) {
    if (e.no_store) return;
    const bool vec = (n + 3 < N) && ((e.ldo & 3) == 0) && (e.pos_ptr == nullptr);
    if (!vec) {
        if (n < N) epi_store(e, m, n, v.x);
        if (n + 1 < N) epi_store(e, m, n + 1, v.y);
        if (n + 2 < N) epi_store(e, m, n + 2, v.z);
        if (n + 3 < N) epi_store(e, m, n + 3, v.w);
        return;
    }
    if (e.mode == EPI_RESID) {
        float4 *p = reinterpret_cast<float4 *>(e.resid + (size_t)m * e.ldo + n);
        float4 r = *p;
        r.x += v.x; r.y += v.y; r.z += v.z; r.w += v.w;
        *p = r;
        return;
    }
    if (e.mode == EPI_QKV && n >= e.d_model) {
        int c = n - e.d_model;
        __half *cache = e.kc;
        if (c >= e.d_model) {
            c -= e.d_model;
            cache = e.vc;
        }
        const int head = c >> 6, el = c & 63;
        const int b = m / e.rows_per_seq, s = m - b * e.rows_per_seq;
        const int pos = e.pos_off + s;
        if (pos < e.cap) {
            __half2 lo = __floats2half2_rn(v.x, v.y), hi = __floats2half2_rn(v.z, v.w);
            uint2 u = make_uint2(*reinterpret_cast<uint32_t *>(&lo), *reinterpret_cast<uint32_t *>(&hi));
            *reinterpret_cast<uint2 *>(cache + (((size_t)b * e.n_head + head) * e.cap + pos) * 64 + el) = u;
        }
        return;
    }
    v.x = apply_act(v.x, e.act); v.y = apply_act(v.y, e.act);
    v.z = apply_act(v.z, e.act); v.w = apply_act(v.w, e.act);
    const size_t i = (size_t)m * e.ldo + n;
    if (e.out_half) {
        __half2 lo = __floats2half2_rn(v.x, v.y), hi = __floats2half2_rn(v.z, v.w);
        *reinterpret_cast<uint2 *>(static_cast<__half *>(e.out) + i) =
            make_uint2(*reinterpret_cast<uint32_t *>(&lo), *reinterpret_cast<uint32_t *>(&hi));
    } else {
        *reinterpret_cast<float4 *>(static_cast<float *>(e.out) + i) = v;
    }
}

// ---- greedy pick fused into the epilogue ---------------------------------------------------------
// The better of two (value, index) candidates: larger value; on equal values the lower index, or the
// higher with keep_last (Rust's max_by, gpt2.rs:991-997).  NaN never wins, as in argmax_kernel.
__device__ __forceinline__ void amax_merge(float &bv, int &bi, float v, int i, int keep_last) {
    if (v > bv || (v == bv && (keep_last ? i > bi : i < bi))) {
        bv = v;
        bi = i;
    }
}
// Warp-collective (all 32 lanes, converged).  The lane holds the finished values of features n..n+3 of
// row m (n a multiple of 4, consecutive lanes consecutive groups of four): each group of eight lanes
// covers 32 features = one entry of the partial-argmax table.
__device__ __forceinline__ void epi_argmax4(const Epilogue &e, int m, int n, float4 v, int N) {
    float bv = -INFINITY;
    int bi = e.amax_keep_last ? -1 : 0x7fffffff;
    if (n < N) amax_merge(bv, bi, v.x, n, e.amax_keep_last);
    if (n + 1 < N) amax_merge(bv, bi, v.y, n + 1, e.amax_keep_last);
    if (n + 2 < N) amax_merge(bv, bi, v.z, n + 2, e.amax_keep_last);
    if (n + 3 < N) amax_merge(bv, bi, v.w, n + 3, e.amax_keep_last);
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        amax_merge(bv, bi, ov, oi, e.amax_keep_last);
    }
    if ((threadIdx.x & 7) == 0 && (n >> 5) < e.amax_entries) {
        const size_t at = (size_t)m * e.amax_entries + (n >> 5);
        e.amax_val[at] = bv;
        e.amax_idx[at] = bi;
    }
}
// Warp-collective.  The lane holds the finished value of feature n of row m, the warp 32 consecutive
// features starting at a multiple of 32 (valid = the lane's feature exists).
__device__ __forceinline__ void epi_argmax1(const Epilogue &e, int m, int n, float v, bool valid) {
    float bv = valid ? v : -INFINITY;
    int bi = valid && v == v ? n : (e.amax_keep_last ? -1 : 0x7fffffff);
    if (!(bv == bv)) bv = -INFINITY; // NaN never wins
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        amax_merge(bv, bi, ov, oi, e.amax_keep_last);
    }
    if ((threadIdx.x & 31) == 0 && (n >> 5) < e.amax_entries) {
        const size_t at = (size_t)m * e.amax_entries + (n >> 5);
        e.amax_val[at] = bv;
        e.amax_idx[at] = bi;
    }
}

// Bias of the four features n..n+3 (zero without a bias and past N).
__device__ __forceinline__ float4 epi_bias4(const Epilogue &e, int n, int N) {
    float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
    if (e.bias) {
        if (n < N) b.x = e.bias[n];
        if (n + 1 < N) b.y = e.bias[n + 1];
        if (n + 2 < N) b.z = e.bias[n + 2];
        if (n + 3 < N) b.w = e.bias[n + 3];
    }
    return b;
}

// Residual epilogue as a reduction at L2: resid[m, n..n+3] += v with one vector `red` (no load for
// the warp to wait on), element-wise atomics where the row is not 16-byte aligned or crosses N.
// Several K splits may add to the same element; the order of their additions is then not fixed.
__device__ __forceinline__ void epi_resid_red4(const Epilogue &e, int m, int n, float4 v, int N) {
    float *dst = e.resid + (size_t)m * e.ldo + n;
    if ((n + 3 < N) && ((e.ldo & 3) == 0)) {
        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
                     : "memory");
    } else {
        if (n < N) atomicAdd(dst, v.x);
        if (n + 1 < N) atomicAdd(dst + 1, v.y);
        if (n + 2 < N) atomicAdd(dst + 2, v.z);
        if (n + 3 < N) atomicAdd(dst + 3, v.w);
    }
}

__device__ __forceinline__ float4 f4_add(float4 a, float4 b) {
    return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
}

// ---- LayerNorm folded into the neighbouring GEMMs (see Epilogue) ---------------------------------
// A row's (mean, 1/sqrt(var + eps)) from the partial sums its producer left, added in tile order.
__device__ __forceinline__ float2 epi_row_mean_rstd(const Epilogue &e, int m) {
    const float2 *p = reinterpret_cast<const float2 *>(e.ln_stats) + (size_t)m * e.ln_nt;
    float s1 = 0.0f, s2 = 0.0f;
    for (int j = 0; j < e.ln_nt; ++j) {
        const float2 v = __ldcg(p + j);
        s1 += v.x;
        s2 += v.y;
    }
    const float mean = s1 * e.ln_inv_d;
    return make_float2(mean, rsqrtf(fmaxf(s2 * e.ln_inv_d - mean * mean, 0.0f) + e.ln_eps));
}
// The four sums of products acc (features n..n+3 of a row) -> finished values: plain bias add, or with
// ln_stats the normalisation applied after the product (mr = the row's mean and rstd, g4 =
// ln_gsum[n..n+3], b4 = bias[n..n+3]).
__device__ __forceinline__ float4 epi_finish4(const Epilogue &e, float4 acc, float4 g4, float4 b4, float2 mr) {
    if (!e.ln_stats) return f4_add(acc, b4);
    const float mean = mr.x, rstd = mr.y;
    return make_float4(fmaf(rstd, fmaf(-mean, g4.x, acc.x), b4.x), fmaf(rstd, fmaf(-mean, g4.y, acc.y), b4.y),
                       fmaf(rstd, fmaf(-mean, g4.z, acc.z), b4.z), fmaf(rstd, fmaf(-mean, g4.w, acc.w), b4.w));
}
// The per-lane constant of the LayerNorm fold: the consumer's ln_gsum[n..n+3], or the producer's
// next_g[n..n+3] (no Linear is both).
__device__ __forceinline__ float4 epi_fold4(const Epilogue &e, int n, int N) {
    const float *src = e.mode == EPI_RESID_LN ? e.next_g : e.ln_gsum;
    float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
    if (src) {
        if (n < N) g.x = src[n];
        if (n + 1 < N) g.y = src[n + 1];
        if (n + 2 < N) g.z = src[n + 2];
        if (n + 3 < N) g.w = src[n + 3];
    }
    return g;
}
// The residual values a producer row will be added to (fetched early, under the reduction of the sums).
__device__ __forceinline__ float4 epi_resid_old4(const Epilogue &e, int m, int n, int N) {
    if (e.mode != EPI_RESID_LN || n >= N) return make_float4(0.f, 0.f, 0.f, 0.f);
    return *reinterpret_cast<const float4 *>(e.resid + (size_t)m * e.ldo + n);
}
// Residual epilogue that also prepares the next LayerNorm.  Warp-collective: the 32 lanes are converged on
// one token row m, lane l holding features n..n+3 (n = 128 * tile + 4 l); v = the finished values (bias
// included), r = epi_resid_old4, ng = next_g[n..n+3].  N and ldo are multiples of 4 (the model width).
__device__ __forceinline__ void epi_resid_ln4(const Epilogue &e, int m, int n, float4 v, float4 r, float4 ng, int N) {
    float s1 = 0.0f, s2 = 0.0f;
    if (n < N) {
        const size_t i = (size_t)m * e.ldo + n;
        r.x += v.x; r.y += v.y; r.z += v.z; r.w += v.w;
        *reinterpret_cast<float4 *>(e.resid + i) = r;
        __half2 lo = __floats2half2_rn(r.x * ng.x, r.y * ng.y), hi = __floats2half2_rn(r.z * ng.z, r.w * ng.w);
        *reinterpret_cast<uint2 *>(e.xg_out + i) = make_uint2(*reinterpret_cast<uint32_t *>(&lo), *reinterpret_cast<uint32_t *>(&hi));
        s1 = (r.x + r.y) + (r.z + r.w);
        s2 = (r.x * r.x + r.y * r.y) + (r.z * r.z + r.w * r.w);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        s1 += __shfl_xor_sync(0xffffffffu, s1, o);
        s2 += __shfl_xor_sync(0xffffffffu, s2, o);
    }
    if ((threadIdx.x & 31) == 0)
        *reinterpret_cast<float2 *>(e.stats_out + ((size_t)m * e.stats_nt + (n >> 7)) * 2) = make_float2(s1, s2);
}
// One finished row of a 128-feature tile leaves the GEMM (warp-collective as above): acc = the complete
// sums of products, f4 = epi_fold4, mr = the row's (mean, rstd) when ln_stats is set, r = epi_resid_old4.
__device__ __forceinline__ void epi_emit4(const Epilogue &e2, const Epilogue &epi, int m, int n, float4 acc, float4 f4,
                                          float4 b4, float2 mr, float4 r, int N) {
    const float4 v = epi_finish4(epi, acc, f4, b4, mr);
    if (epi.mode == EPI_RESID_LN) {
        epi_resid_ln4(epi, m, n, v, r, f4, N);
    } else {
        epi_store4(e2, m, n, v, N);
        if (epi.amax_val) epi_argmax4(epi, m, n, v, N);
    }
}

// Same, from a raw accumulated dot product.
__device__ __forceinline__ void epi_apply(const Epilogue &e, int m, int n, float acc) {
    epi_store(e, m, n, acc + (e.bias ? e.bias[n] : 0.0f));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over the block; every thread gets the result.  red must hold 32 floats.
__device__ __forceinline__ float block_sum(float v, float *red) {
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    float t = (lane < nw) ? red[lane] : 0.0f;
    return warp_sum(t);
}

template <typename T>
__device__ __forceinline__ float load_as_float(const T *p, size_t i);
template <>
__device__ __forceinline__ float load_as_float<float>(const float *p, size_t i) { return p[i]; }
template <>
__device__ __forceinline__ float load_as_float<__half>(const __half *p, size_t i) { return __half2float(p[i]); }

// Unpacks one 32-bit word of the tiled int4 layout (nibble positions 0..7 = k offsets
// 0,2,4,6,1,3,5,7, each stored +8) into four half2 holding the exact integers (k0,k1) (k2,k3)
// (k4,k5) (k6,k7) in [-8,7].
__device__ __forceinline__ void unpack8_int4(uint32_t w, __half2 (&q)[4]) {
    const uint32_t MAGIC = 0x64006400u; // 1024.0 in both halves
    uint32_t h0, h1, h2, h3;
    asm("lop3.b32 %0, %1, 0x000f000f, %2, 0xea;" : "=r"(h0) : "r"(w), "r"(MAGIC));
    asm("lop3.b32 %0, %1, 0x00f000f0, %2, 0xea;" : "=r"(h1) : "r"(w), "r"(MAGIC));
    uint32_t w8 = w >> 8;
    asm("lop3.b32 %0, %1, 0x000f000f, %2, 0xea;" : "=r"(h2) : "r"(w8), "r"(MAGIC));
    asm("lop3.b32 %0, %1, 0x00f000f0, %2, 0xea;" : "=r"(h3) : "r"(w8), "r"(MAGIC));
    const __half2 c1032 = __floats2half2_rn(1032.0f, 1032.0f);
    const __half2 c16th = __floats2half2_rn(0.0625f, 0.0625f);
    const __half2 cm72 = __floats2half2_rn(-72.0f, -72.0f);
    q[0] = __hsub2(*reinterpret_cast<__half2 *>(&h0), c1032);       // (1024+n) - 1032
    q[1] = __hfma2(*reinterpret_cast<__half2 *>(&h1), c16th, cm72); // (1024+16n)/16 - 72
    q[2] = __hsub2(*reinterpret_cast<__half2 *>(&h2), c1032);
    q[3] = __hfma2(*reinterpret_cast<__half2 *>(&h3), c16th, cm72);
}
