// Causal prefill attention on the tensor cores (tcgen05, accumulators in tensor memory), pipelined.
//
// One block per (128-query tile, head, sequence), six warps with fixed roles:
//   warp 0      copies: the Q tile once, then the K and V tiles of every 128-key step through tensor maps
//               (cp.async.bulk.tensor, 128-byte swizzle, zero fill past the last cached row) into two-stage
//               rings; no hand-written shared-memory stores anywhere
//   warp 1      MMA issue: S_j = Q K_j^T into one of two score buffers in TMEM, then O_j = P_j V_j with
//               P read from tensor memory (A operand) and V straight from its row-major tile (B operand
//               MN-major: no transposition)
//   warps 2..5  softmax: thread r owns query row r (= TMEM lane r).  Pass 1 takes the row maximum of S_j;
//               then the previous step's O_{j-1} is fetched from TMEM and folded into the running output
//               (64 f32 per thread, rescaled by that step's correction); pass 2 writes
//               p = exp2(s*scale - max) back over S_j as packed fp16.
// Per step the tensor pipe therefore works on S_{j+1} and O_{j-1} while the softmax warps are busy
// with step j; two blocks per SM cover what is left of each other's gaps.
//
// TMEM (256 columns per block): score buffer b at columns 128 b .. 128 b + 127.  P_j (64 columns of fp16
// pairs) overwrites columns 0..63 of its own buffer as pass 2 goes along (the 16 P columns written at
// score column c0 cover score columns c0/2 .. c0/2+15, all loaded by then; a thread only touches its
// own lane); O_j lands in columns 64..127 of the same buffer, free once pass 2 is over.
//
// Replaces flash_attention_v2 / flash_attn_v3.cu of the reference (compute_transformer.rs:597-816,
// cuda/flash_attn_v3.cu:29-283) for the model path, where q and the output are fp16.
//
// Every mbarrier wait is bounded: on expiry the block records a code in the device error word, all
// roles leave their loops, nothing is stored, the TMEM columns are freed and the kernel returns.
#include <cuda.h>

#include "device_utils.cuh"
#include "tc_ptx.cuh"

namespace {

constexpr float SCALE_LOG2E = 0.125f * 1.4426950408889634f;
constexpr float NEG_BIG = -1.0e30f;
enum : uint32_t { ERR_ATT_Q = 0x41, ERR_ATT_K, ERR_ATT_V, ERR_ATT_S, ERR_ATT_P, ERR_ATT_O, ERR_ATT_FREE, ERR_ATT_KE, ERR_ATT_VE };
constexpr int TM_COLS = 256;                // two score buffers
constexpr int KV_STAGES = 2;
constexpr int TILE = 16384;                 // 128 rows x 64 fp16
constexpr int SMEM_BYTES = (1 + 2 * KV_STAGES) * TILE + 1024; // Q, K ring, V ring + alignment slack
constexpr int NTHREADS = 192;

__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
}

struct Bars {
    uint64_t q_full;
    uint64_t k_full[KV_STAGES], k_empty[KV_STAGES], v_full[KV_STAGES], v_empty[KV_STAGES];
    uint64_t s_full[2], p_full[2], o_full[2], s_free[2];
};

__global__ void __launch_bounds__(NTHREADS, 2)
prefill_attn_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                       const __grid_constant__ CUtensorMap tm_v, int H, int cap, int S, int past, __half *__restrict__ out,
                       int ldo, uint32_t *__restrict__ dev_err) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) Bars bars;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    // the query tiles with the most key tiles are scheduled first (blocks start in index order)
    const int qt = gridDim.z - 1 - blockIdx.z, h = blockIdx.y, b = blockIdx.x;
    const int tid = threadIdx.x, warp = tid >> 5;
    const uint32_t base = (tc::smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sQ = base, sK = base + TILE, sV = base + TILE * (1 + KV_STAGES);
    auto bar = [&](const uint64_t &x) { return tc::smem_u32(&x); };

    if (tid == 0) {
        abort_flag = 0;
        tc::mbar_init(bar(bars.q_full), 1);
        for (int i = 0; i < KV_STAGES; ++i) {
            tc::mbar_init(bar(bars.k_full[i]), 1);
            tc::mbar_init(bar(bars.k_empty[i]), 1);
            tc::mbar_init(bar(bars.v_full[i]), 1);
            tc::mbar_init(bar(bars.v_empty[i]), 1);
        }
        for (int i = 0; i < 2; ++i) {
            tc::mbar_init(bar(bars.s_full[i]), 1);
            tc::mbar_init(bar(bars.p_full[i]), 128); // every softmax thread
            tc::mbar_init(bar(bars.o_full[i]), 1);
            tc::mbar_init(bar(bars.s_free[i]), 128);
        }
        tc::fence_mbar_init();
    }
    if (warp == 0) {
        tc::prefetch_tmap(&tm_q);
        tc::prefetch_tmap(&tm_k);
        tc::prefetch_tmap(&tm_v);
    }
    if (warp == 1) tc::tmem_alloc(tc::smem_u32(&tmem_slot), TM_COLS);
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(&tmem_slot);

    const int kv_end = min(past + min(S, qt * 128 + 128), cap); // keys this tile's queries can see
    const int n_tiles = (kv_end + 127) / 128;
    const int bh = b * H + h;

    if (warp == 0) {
        // ---- copies (one elected lane issues; the warp stays converged on the waits) ----
        if (tc::elect_one()) {
            tc::mbar_expect_tx(bar(bars.q_full), TILE);
            tc::tma_load_2d(sQ, &tm_q, h * 64, b * S + qt * 128, bar(bars.q_full));
        }
        for (int j = 0; j < n_tiles; ++j) {
            const int st = j % KV_STAGES, u = j / KV_STAGES;
            if (j >= KV_STAGES && !tc::mbar_wait(bar(bars.k_empty[st]), (u - 1) & 1, &abort_flag, dev_err, ERR_ATT_KE)) break;
            if (tc::elect_one()) {
                tc::mbar_expect_tx(bar(bars.k_full[st]), TILE);
                tc::tma_load_3d(sK + st * TILE, &tm_k, 0, j * 128, bh, bar(bars.k_full[st]));
            }
            if (j >= KV_STAGES && !tc::mbar_wait(bar(bars.v_empty[st]), (u - 1) & 1, &abort_flag, dev_err, ERR_ATT_VE)) break;
            if (tc::elect_one()) {
                tc::mbar_expect_tx(bar(bars.v_full[st]), TILE);
                tc::tma_load_3d(sV + st * TILE, &tm_v, 0, j * 128, bh, bar(bars.v_full[st]));
            }
        }
    } else if (warp == 1) {
        // ---- MMA issue: S_j as early as its buffer and K tile allow, then O_{j-1} once P_{j-1} is written ----
        constexpr uint32_t idesc_s = tc::umma_idesc_f16(128, 128);
        constexpr uint32_t idesc_o = tc::umma_idesc_f16_bmn(128, 64);
        const uint64_t dq = tc::umma_desc_sw128(sQ);
        bool ok = tc::mbar_wait(bar(bars.q_full), 0, &abort_flag, dev_err, ERR_ATT_Q);
        for (int j = 0; ok && j <= n_tiles; ++j) {
            if (j < n_tiles) {
                const int bf = j & 1, st = j % KV_STAGES, u = j / KV_STAGES;
                if (j >= 2) ok = tc::mbar_wait(bar(bars.s_free[bf]), ((j >> 1) - 1) & 1, &abort_flag, dev_err, ERR_ATT_FREE);
                if (ok) ok = tc::mbar_wait(bar(bars.k_full[st]), u & 1, &abort_flag, dev_err, ERR_ATT_K);
                if (!ok) break;
                tc::tc_fence_after_sync();
                if (tc::elect_one()) {
                    const uint64_t dk = tc::umma_desc_sw128(sK + st * TILE);
#pragma unroll
                    for (int k = 0; k < 4; ++k) tc::umma_f16_ss(tmem_base + bf * 128, dq + 2 * k, dk + 2 * k, idesc_s, k != 0);
                    tc::umma_commit(bar(bars.s_full[bf]));
                    tc::umma_commit(bar(bars.k_empty[st]));
                }
                __syncwarp();
            }
            if (j >= 1) {
                const int jp = j - 1, bp = jp & 1, st = jp % KV_STAGES, u = jp / KV_STAGES;
                ok = tc::mbar_wait(bar(bars.p_full[bp]), (jp >> 1) & 1, &abort_flag, dev_err, ERR_ATT_P);
                if (ok) ok = tc::mbar_wait(bar(bars.v_full[st]), u & 1, &abort_flag, dev_err, ERR_ATT_V);
                if (!ok) break;
                tc::tc_fence_after_sync();
                if (tc::elect_one()) {
                    const uint64_t dv = tc::umma_desc_sw128_mn64(sV + st * TILE);
                    const uint32_t buf = tmem_base + bp * 128;
#pragma unroll
                    for (int k = 0; k < 8; ++k) // 16 keys per MMA: 8 TMEM columns of P, 2048 bytes of V
                        tc::umma_f16_ts(buf + 64, buf + 8 * k, dv + (uint64_t)(k * (2048 >> 4)), idesc_o, k != 0);
                    tc::umma_commit(bar(bars.o_full[bp]));
                    tc::umma_commit(bar(bars.v_empty[st]));
                }
                __syncwarp();
            }
        }
    } else {
        // ---- softmax and the running output: thread = query row = TMEM lane ----
        const int quad = warp & 3, row = quad * 32 + (tid & 31);
        const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
        const int s_row = qt * 128 + row;
        const bool row_valid = s_row < S;
        const int a_pos = past + s_row; // absolute position of this thread's query
        float m = NEG_BIG, l = 0.0f, corr_prev = 1.0f, acc[64];
#pragma unroll
        for (int e = 0; e < 64; ++e) acc[e] = 0.0f;
        bool ok = true;
        // acc = acc * c + O_tile of score buffer bp (one TMEM round trip)
        auto fold_output = [&](int bp, float c) {
            uint32_t v[64];
            tc::tmem_ld_x64(lane_base + bp * 128 + 64, v);
#pragma unroll
            for (int e = 0; e < 64; ++e) acc[e] = fmaf(acc[e], c, __uint_as_float(v[e]));
        };
        for (int j = 0; j < n_tiles; ++j) {
            const int bf = j & 1, j0 = j * 128;
            const uint32_t sbuf = lane_base + bf * 128;
            ok = tc::mbar_wait(bar(bars.s_full[bf]), (j >> 1) & 1, &abort_flag, dev_err, ERR_ATT_S);
            if (!ok) break;
            tc::tc_fence_after_sync();
            // columns of this tile the row may attend to: keys j0 .. min(a_pos, kv_end-1); only the tile on
            // the diagonal (and rows past the sequence) need the mask, the others take the short loops
            int nvalid = row_valid ? min(a_pos, kv_end - 1) - j0 + 1 : 0;
            nvalid = max(0, min(nvalid, 128));
            const bool full = __all_sync(0xffffffffu, nvalid == 128);
            float mx[4] = {NEG_BIG, NEG_BIG, NEG_BIG, NEG_BIG}; // four independent chains
#pragma unroll 1
            for (int hf = 0; hf < 2; ++hf) { // pass 1: row maximum, 64 scores per round trip
                uint32_t v[64];
                tc::tmem_ld_x64(sbuf + 64 * hf, v);
                if (full) {
#pragma unroll
                    for (int e = 0; e < 64; e += 8) {
                        mx[0] = tc::fmax3(mx[0], __uint_as_float(v[e]), __uint_as_float(v[e + 1]));
                        mx[1] = tc::fmax3(mx[1], __uint_as_float(v[e + 2]), __uint_as_float(v[e + 3]));
                        mx[2] = tc::fmax3(mx[2], __uint_as_float(v[e + 4]), __uint_as_float(v[e + 5]));
                        mx[3] = tc::fmax3(mx[3], __uint_as_float(v[e + 6]), __uint_as_float(v[e + 7]));
                    }
                } else {
#pragma unroll
                    for (int e = 0; e < 64; ++e)
                        if (64 * hf + e < nvalid) mx[e & 3] = fmaxf(mx[e & 3], __uint_as_float(v[e]));
                }
            }
            const float mloc = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
            const float m_new = fmaxf(m, mloc * SCALE_LOG2E);
            const float corr = tc::ex2_approx(m - m_new);
            if (j >= 1) { // the previous step's P V has had pass 1 to finish
                ok = tc::mbar_wait(bar(bars.o_full[bf ^ 1]), ((j - 1) >> 1) & 1, &abort_flag, dev_err, ERR_ATT_O);
                if (!ok) break;
                tc::tc_fence_after_sync();
                fold_output(bf ^ 1, corr_prev);
                tc::tc_fence_before_sync();
                tc::mbar_arrive(bar(bars.s_free[bf ^ 1])); // that buffer may take S_{j+1}
            }
            float ls[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 1
            for (int hf = 0; hf < 2; ++hf) { // pass 2: p = 2^(s*scale - max) as fp16 pairs over the scores
                uint32_t v[64], o[32];
                tc::tmem_ld_x64(sbuf + 64 * hf, v);
#pragma unroll
                for (int e = 0; e < 64; e += 2) {
                    float p0 = tc::ex2_approx(fmaf(__uint_as_float(v[e]), SCALE_LOG2E, -m_new));
                    float p1 = tc::ex2_approx(fmaf(__uint_as_float(v[e + 1]), SCALE_LOG2E, -m_new));
                    if (!full) {
                        if (64 * hf + e >= nvalid) p0 = 0.0f;
                        if (64 * hf + e + 1 >= nvalid) p1 = 0.0f;
                    }
                    ls[(e >> 1) & 3] += p0 + p1;
                    o[e >> 1] = pack_half2(p0, p1);
                }
                tc::tmem_st_x32(sbuf + 32 * hf, o);
            }
            tc::tmem_st_wait();
            tc::tc_fence_before_sync();
            tc::mbar_arrive(bar(bars.p_full[bf]));
            l = l * corr + ((ls[0] + ls[1]) + (ls[2] + ls[3]));
            m = m_new;
            corr_prev = corr;
        }
        if (ok) {
            const int bl = (n_tiles - 1) & 1;
            ok = tc::mbar_wait(bar(bars.o_full[bl]), ((n_tiles - 1) >> 1) & 1, &abort_flag, dev_err, ERR_ATT_O);
            if (ok) {
                tc::tc_fence_after_sync();
                fold_output(bl, corr_prev);
            }
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
    }

    // ---- teardown (also the path taken after a wait gave up) ----
    if (abort_flag && warp == 0) { // let copies still in flight land before the block's memory is released
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tc::tmem_dealloc(tmem_base, TM_COLS);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

}  // namespace

// q, out fp16; rows of q / out are ldq / H*64 halves apart and must be 16-byte aligned, as must q, kc and vc.
int launch_prefill_attention_tc(b200nn_ctx *ctx, const __half *q, int ldq, const __half *kc, const __half *vc, int B, int H,
                                int cap, int S, int past, __half *out) {
    if (!ctx->encode_tiled) return set_error(ctx, B200NN_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled is unavailable");
    if (((uintptr_t)q | (uintptr_t)kc | (uintptr_t)vc | (uintptr_t)out) & 15 || (ldq & 7))
        return set_error(ctx, B200NN_ERR_ARG, "prefill attention: q, K, V and out must be 16-byte aligned, rows of q a multiple of 8 halves");
    static bool attr_done[16] = {};
    if (!attr_done[ctx->device & 15]) {
        CK(ctx, cudaFuncSetAttribute(prefill_attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        prefer_max_smem(prefill_attn_tc_kernel);
        attr_done[ctx->device & 15] = true;
    }
    const EncodeTiledFn encode = (EncodeTiledFn)ctx->encode_tiled;
    CUtensorMap tq, tk, tv;
    const cuuint32_t ones[3] = {1, 1, 1};
    {   // queries: [B*S rows][H*64] fp16, rows ldq halves apart; one box = 128 rows of one head
        cuuint64_t dim[2] = {(cuuint64_t)H * 64, (cuuint64_t)B * S};
        cuuint64_t stride[1] = {(cuuint64_t)ldq * sizeof(__half)};
        cuuint32_t box[2] = {64, 128};
        CUresult r = encode(&tq, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void *)q, dim, stride, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return set_error(ctx, B200NN_ERR_CUDA, "cuTensorMapEncodeTiled (q) failed: " + std::to_string((int)r));
    }
    // K and V caches: [B*H][cap rows][64] fp16; the row extent is the number of rows written so far, so
    // that a box reaching past it is zero-filled instead of reading rows nothing has written
    const cuuint64_t rows = (cuuint64_t)std::min(past + S, cap);
    cuuint64_t dim[3] = {64, rows, (cuuint64_t)B * H};
    cuuint64_t stride[2] = {64 * sizeof(__half), (cuuint64_t)cap * 64 * sizeof(__half)};
    cuuint32_t box[3] = {64, 128, 1};
    for (int which = 0; which < 2; ++which) {
        CUresult r = encode(which ? &tv : &tk, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, (void *)(which ? vc : kc), dim, stride, box, ones,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return set_error(ctx, B200NN_ERR_CUDA, "cuTensorMapEncodeTiled (K/V) failed: " + std::to_string((int)r));
    }
    if (B > 65535 || (S + 127) / 128 > 65535) return set_error(ctx, B200NN_ERR_SHAPE, "prefill attention: more than 65535 sequences or query tiles");
    dim3 grid(B, H, (S + 127) / 128);
    prefill_attn_tc_kernel<<<grid, NTHREADS, SMEM_BYTES, ctx->stream>>>(tq, tk, tv, H, cap, S, past, out, H * 64, ctx->dev_err);
    CK_LAUNCH(ctx, "prefill_attn_tc_kernel");
    return B200NN_OK;
}
