// Causal prefill attention on the tensor cores (tcgen05, accumulators in tensor memory).
//
// One block per (128-query tile, head, sequence).  Per 128-key tile of the fp16 KV cache:
//   S = Q K^T        tcgen05.mma, both operands in shared memory (K-major, 128-byte swizzle), f32 in TMEM
//   softmax          thread r owns query row r (= TMEM lane r): two passes over its 128 scores (row
//                    maximum, then p = exp2(s*scale - max)), causal mask by column index, P written
//                    back to TMEM as packed fp16 pairs
//   O_tile = P V     tcgen05.mma with the A operand (P) read from tensor memory and V^T from shared
//                    memory (V is transposed on its way into shared memory so that it is K-major)
//   O = O*corr + O_tile in registers (64 f32 per thread), online-softmax rescaling across key tiles.
// Replaces flash_attention_v2 / flash_attn_v3.cu of the reference (compute_transformer.rs:597-816,
// cuda/flash_attn_v3.cu:29-283) for the model path, where q and the output are fp16.
//
// Every mbarrier wait is bounded: on expiry the block records a code in the device error word,
// skips its stores, frees its TMEM columns and returns.
#include "device_utils.cuh"
#include "tc_ptx.cuh"

namespace {

constexpr float SCALE_LOG2E = 0.125f * 1.4426950408889634f;
constexpr float NEG_BIG = -1.0e30f;
constexpr uint32_t ERR_ATT_S = 0x41, ERR_ATT_O = 0x42;
// TMEM columns: S occupies 0..127.  P (fp16 pairs, 64 columns) is written over S's columns 0..63 as
// the second softmax pass goes along: the 16 P columns of step c0 cover S columns c0/2 .. c0/2+15,
// all of which that pass has already loaded (a thread only ever touches its own lane).  O_tile
// takes S's columns 64..127 once every thread is past the softmax.  128 columns per block let the
// register-limited three blocks per SM be resident.
constexpr int TM_COLS = 128, P_COL = 0, O_COL = 64;
constexpr int SMEM_BYTES = 3 * 16384 + 1024; // Q, K, V^T tiles + alignment slack

__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
}

__global__ void __launch_bounds__(128)
prefill_attn_tc_kernel(const __half *__restrict__ q, int ldq, const __half *__restrict__ kc,
                       const __half *__restrict__ vc, int H, int cap, int S, int past, __half *__restrict__ out, int ldo,
                       uint32_t *__restrict__ dev_err) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5;
    const uint32_t base = (tc::smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sQ = base, sK = base + 16384, sV = base + 32768;
    uint8_t *gen = smem_raw + (base - tc::smem_u32(smem_raw));
    const uint32_t bar_s = tc::smem_u32(&bars[0]), bar_o = tc::smem_u32(&bars[1]);

    if (tid == 0) {
        abort_flag = 0;
        tc::mbar_init(bar_s, 1);
        tc::mbar_init(bar_o, 1);
        tc::fence_mbar_init();
    }
    if (warp == 0) tc::tmem_alloc(tc::smem_u32(&tmem_slot), TM_COLS);
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(&tmem_slot);
    const uint32_t lane_base = tmem_base + ((uint32_t)(warp * 32) << 16); // this warp's 32 TMEM lanes

    // Q tile -> shared, rows of 128 bytes, 16-byte chunk c of row r stored at chunk (c ^ (r & 7))
    for (int i = tid; i < 1024; i += 128) {
        const int r = i >> 3, c = i & 7, s_row = qt * 128 + r;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (s_row < S) v = __ldg(reinterpret_cast<const uint4 *>(q + ((size_t)b * S + s_row) * ldq + h * 64) + c);
        *reinterpret_cast<uint4 *>(gen + r * 128 + ((c ^ (r & 7)) << 4)) = v;
    }

    const size_t cache_base = ((size_t)b * H + h) * cap * 64;
    const uint4 *kp = reinterpret_cast<const uint4 *>(kc + cache_base);
    const uint4 *vp = reinterpret_cast<const uint4 *>(vc + cache_base);
    const int kv_end = min(past + min(S, qt * 128 + 128), cap); // keys this tile's queries can see
    const int n_tiles = (kv_end + 127) / 128;
    const int s_row = qt * 128 + tid;
    const bool row_valid = s_row < S;
    const int a_pos = past + s_row; // absolute position of this thread's query

    constexpr uint32_t idesc_s = tc::umma_idesc_f16(128, 128);
    constexpr uint32_t idesc_o = tc::umma_idesc_f16(128, 64);
    const uint64_t dq = tc::umma_desc_sw128(sQ), dk = tc::umma_desc_sw128(sK), dv = tc::umma_desc_sw128(sV);

    float m = NEG_BIG, l = 0.0f, acc[64];
#pragma unroll
    for (int e = 0; e < 64; ++e) acc[e] = 0.0f;
    bool ok = true;

    for (int kt = 0; kt < n_tiles; ++kt) {
        const int j0 = kt * 128;
        const uint32_t ph = kt & 1;
        // K tile, same layout as Q; rows past kv_end are zero
        for (int i = tid; i < 1024; i += 128) {
            const int r = i >> 3, c = i & 7, j = j0 + r;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (j < kv_end) v = __ldg(kp + (size_t)j * 8 + c);
            *reinterpret_cast<uint4 *>(gen + 16384 + r * 128 + ((c ^ (r & 7)) << 4)) = v;
        }
        // V tile transposed: V^T[dim][key], two 64-key blocks of [64 dims][128 bytes].  A warp takes 32
        // consecutive keys of one 8-dim chunk, so its 2-byte stores fall in one 128-byte row.
#pragma unroll 2
        for (int c = 0; c < 8; ++c) {
            const int r = tid, j = j0 + r;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (j < kv_end) v = __ldg(vp + (size_t)j * 8 + c);
            const __half *hv = reinterpret_cast<const __half *>(&v);
            uint8_t *blk = gen + 32768 + (r >> 6) * 8192;
            const int kk = r & 63;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const int dim = c * 8 + e;
                *reinterpret_cast<__half *>(blk + dim * 128 + (((kk >> 3) ^ (dim & 7)) << 4) + (kk & 7) * 2) = hv[e];
            }
        }
        tc::fence_proxy_async_smem();
        tc::tc_fence_before_sync();
        __syncthreads();
        if (warp == 0) {
            tc::tc_fence_after_sync();
            if (tc::elect_one()) {
#pragma unroll
                for (int k = 0; k < 4; ++k) tc::umma_f16_ss(tmem_base, dq + 2 * k, dk + 2 * k, idesc_s, k != 0);
                tc::umma_commit(bar_s);
            }
            __syncwarp();
        }
        ok = tc::mbar_wait(bar_s, ph, &abort_flag, dev_err, ERR_ATT_S);
        ok = __syncthreads_and(ok);
        if (!ok) break;
        tc::tc_fence_after_sync();

        // columns of this tile the row may attend to: keys j0 .. min(a_pos, kv_end-1)
        int nvalid = row_valid ? min(a_pos, kv_end - 1) - j0 + 1 : 0;
        nvalid = max(0, min(nvalid, 128));
        float mloc = NEG_BIG;
#pragma unroll
        for (int c0 = 0; c0 < 128; c0 += 16) {
            uint32_t v[16];
            tc::tmem_ld_x16(lane_base + c0, v);
#pragma unroll
            for (int e = 0; e < 16; ++e)
                if (c0 + e < nvalid) mloc = fmaxf(mloc, __uint_as_float(v[e]));
        }
        const float m_new = fmaxf(m, mloc * SCALE_LOG2E);
        const float corr = exp2f(m - m_new);
        float lsum = 0.0f;
#pragma unroll
        for (int c0 = 0; c0 < 128; c0 += 32) {
            uint32_t v0[16], v1[16], o[16];
            tc::tmem_ld_x16(lane_base + c0, v0);
            tc::tmem_ld_x16(lane_base + c0 + 16, v1);
#pragma unroll
            for (int e = 0; e < 16; e += 2) {
                float p0 = (c0 + e < nvalid) ? exp2f(__uint_as_float(v0[e]) * SCALE_LOG2E - m_new) : 0.0f;
                float p1 = (c0 + e + 1 < nvalid) ? exp2f(__uint_as_float(v0[e + 1]) * SCALE_LOG2E - m_new) : 0.0f;
                float p2 = (c0 + 16 + e < nvalid) ? exp2f(__uint_as_float(v1[e]) * SCALE_LOG2E - m_new) : 0.0f;
                float p3 = (c0 + 17 + e < nvalid) ? exp2f(__uint_as_float(v1[e + 1]) * SCALE_LOG2E - m_new) : 0.0f;
                const uint32_t w0 = pack_half2(p0, p1), w1 = pack_half2(p2, p3);
                // the row sum uses the rounded probabilities the MMA will multiply with
                const float2 f0 = __half22float2(*reinterpret_cast<const __half2 *>(&w0));
                const float2 f1 = __half22float2(*reinterpret_cast<const __half2 *>(&w1));
                lsum += (f0.x + f0.y) + (f1.x + f1.y);
                o[e >> 1] = w0;
                o[8 + (e >> 1)] = w1;
            }
            tc::tmem_st_x16(lane_base + P_COL + (c0 >> 1), o);
        }
        tc::tmem_st_wait();
        tc::tc_fence_before_sync();
        __syncthreads();
        if (warp == 0) {
            tc::tc_fence_after_sync();
            if (tc::elect_one()) {
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    tc::umma_f16_ts(tmem_base + O_COL, tmem_base + P_COL + 8 * k, dv + (uint64_t)((k >> 2) * (8192 >> 4) + 2 * (k & 3)),
                                    idesc_o, k != 0);
                tc::umma_commit(bar_o);
            }
            __syncwarp();
        }
        ok = tc::mbar_wait(bar_o, ph, &abort_flag, dev_err, ERR_ATT_O);
        ok = __syncthreads_and(ok);
        if (!ok) break;
        tc::tc_fence_after_sync();
        l = l * corr + lsum;
        m = m_new;
#pragma unroll
        for (int c0 = 0; c0 < 64; c0 += 16) {
            uint32_t v[16];
            tc::tmem_ld_x16(lane_base + O_COL + c0, v);
#pragma unroll
            for (int e = 0; e < 16; ++e) acc[c0 + e] = fmaf(acc[c0 + e], corr, __uint_as_float(v[e]));
        }
        tc::tc_fence_before_sync(); // the next tile's MMAs overwrite S and O_tile
    }

    if (ok && row_valid) {
        const float inv = 1.0f / l;
        uint4 *dst = reinterpret_cast<uint4 *>(out + ((size_t)b * S + s_row) * ldo + h * 64);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            uint4 v;
            v.x = pack_half2(acc[8 * c + 0] * inv, acc[8 * c + 1] * inv);
            v.y = pack_half2(acc[8 * c + 2] * inv, acc[8 * c + 3] * inv);
            v.z = pack_half2(acc[8 * c + 4] * inv, acc[8 * c + 5] * inv);
            v.w = pack_half2(acc[8 * c + 6] * inv, acc[8 * c + 7] * inv);
            dst[c] = v;
        }
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tc::tmem_dealloc(tmem_base, TM_COLS);
}

}  // namespace

// q, out fp16; rows of q / out are ldq / H*64 halves apart and must be 16-byte aligned.
int launch_prefill_attention_tc(b200nn_ctx *ctx, const __half *q, int ldq, const __half *kc, const __half *vc, int B, int H,
                                int cap, int S, int past, __half *out) {
    static bool attr_done[16] = {};
    if (!attr_done[ctx->device & 15]) {
        CK(ctx, cudaFuncSetAttribute(prefill_attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        prefer_max_smem(prefill_attn_tc_kernel);
        attr_done[ctx->device & 15] = true;
    }
    dim3 grid((S + 127) / 128, H, B);
    prefill_attn_tc_kernel<<<grid, 128, SMEM_BYTES, ctx->stream>>>(q, ldq, kc, vc, H, cap, S, past, out, H * 64, ctx->dev_err);
    CK_LAUNCH(ctx, "prefill_attn_tc_kernel");
    return B200NN_OK;
}
