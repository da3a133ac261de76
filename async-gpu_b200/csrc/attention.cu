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
#include "tc_ptx.cuh"

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

// ---------------------------------------------------------------------------------------------
// decode_attn_stream_kernel: the same computation for many (sequence, head) pairs, fed by TMA.
//
// One persistent block per SM, WARPS (8 or 16) warps, each warp an independent pipeline: it takes
// (sequence, head) items from a device-side work counter (whole items, then half-items for the
// units the grid finishes on, merged through a small scratch record) and streams the item's K and V rows
// through its own ring of shared-memory stages with bulk async copies (ROWS = 32 or 16 rows of K and of V
// per stage, 8 or 4 KB, plus the query row with the item's first stage), always two stages ahead of the
// rows it is working on.  The memory system therefore sees up to ~200 KB in flight per SM regardless of
// what the arithmetic is doing, where the plain-load kernel above stalls its loads behind its own
// shuffles and exponentials.  A warp keeps the online-softmax state of its item in registers
// (4 lane groups x 8 lanes, merged with shuffles at the end), so there is no block-level
// synchronisation at all after start-up.  Every mbarrier wait is bounded.
// ---------------------------------------------------------------------------------------------
// B200NN_ATTN_PROBE (compile-time, default 0): builds of decode_attn_stream_kernel without parts of its
// arithmetic, to time the TMA ring alone.  Any other value than 0 gives wrong results.
#ifndef B200NN_ATTN_PROBE
#define B200NN_ATTN_PROBE 0
#endif
namespace stream_attn {
// Two shapes of the block: 8 warps with 32-row stages (fewest pairs per warp needed), and 16 warps with
// 16-row stages (same bytes in flight; a warp's own instruction stream is what limits it, so twice the
// warps hide more of the arithmetic: 52.5 against 54.3 µs per launch at 6400 pairs, but slower below
// ~2.5 pairs per warp, where the last round of items is long).
constexpr int NST = 3;
__host__ __device__ constexpr int stage_bytes(int rows) { return 2 * rows * 128 + 256; } // K rows, V rows, query row (fp16 or f32)
__host__ __device__ constexpr int smem_bytes(int warps, int rows) { return warps * NST * stage_bytes(rows) + 128; }
constexpr uint32_t ERR_FULL = 0x51;
constexpr int REC_FLOATS = 80; // half-item record: [0] max, [1] sum, [8..71] output (16-byte aligned parts)
}  // namespace stream_attn

template <typename QT, typename OT, int WARPS, int ROWS>
__global__ void __launch_bounds__(WARPS * 32, 1)
decode_attn_stream_kernel(const QT *__restrict__ q, int ldq, const __half *__restrict__ kc,
                          const __half *__restrict__ vc, int H, int cap, const int *__restrict__ pos_ptr, int pos_off,
                          OT *__restrict__ out, int ldo, int n_items, int pf_items, int split_items,
                          unsigned *__restrict__ work, float *__restrict__ scratch, unsigned *__restrict__ counters, uint32_t *__restrict__ dev_err) {
    using namespace stream_attn;
    constexpr int STAGE_BYTES = stage_bytes(ROWS);
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[WARPS][NST];
    __shared__ int2 meta[WARPS][NST]; // (item, chunk) held by each stage
    __shared__ int abort_flag;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 3, c = lane & 7;
    if (tid == 0) abort_flag = 0;
    if (lane == 0) {
        for (int s = 0; s < NST; ++s) tc::mbar_init(tc::smem_u32(&full_bar[warp][s]), 1);
        tc::fence_mbar_init();
    }
    __syncthreads();
    pdl_trigger();
    // Cached rows older than this step never change, and the projection that runs before this
    // kernel leaves HBM idle: ask for the K and V rows of the items the grid will work on first to
    // be brought into L2 while that projection is still running.  The position read here may be one
    // step behind (the kernel that advances it may not have finished); fewer rows are harmless.
    if (lane == 0 && pf_items > 0) {
        int old_rows = (pos_ptr ? *reinterpret_cast<const volatile int *>(pos_ptr) : 0) + pos_off;
        old_rows = min(max(old_rows, 0), cap);
        if (old_rows > 0) {
            const int n_w = gridDim.x * WARPS;
            for (int it = blockIdx.x * WARPS + warp; it < pf_items; it += n_w) {
                tc::bulk_prefetch_l2(kc + (size_t)it * cap * 64, (uint32_t)old_rows * 128u);
                tc::bulk_prefetch_l2(vc + (size_t)it * cap * 64, (uint32_t)old_rows * 128u);
            }
        }
    }
    pdl_wait();
    int ctx = (pos_ptr ? *pos_ptr : 0) + pos_off + 1;
    if (ctx > cap) ctx = cap;
    const int nch = (ctx + ROWS - 1) / ROWS;
    const uint32_t ring = ((tc::smem_u32(smem_raw) + 127u) & ~127u) + warp * NST * STAGE_BYTES;
    uint8_t *ring_gen = smem_raw + (ring - tc::smem_u32(smem_raw));

    // Work units, handed out in this order: whole items 0 .. n_full-1, then the last n_warps items
    // as two half-items each (chunk ranges [0, mid) and [mid, nch)), so that the units the grid
    // finishes on are half as long and the warps end closer together.  A warp's first unit is its own
    // index in the grid (what the prefetch before the dependency wait assumed); the rest come from
    // the shared counter, requested one unit ahead so that the atomic's round trip is never waited for.
    const int n_warps = gridDim.x * WARPS, gw = blockIdx.x * WARPS + warp;
    const int n_split = max(0, min(split_items, n_items - n_warps)); // items handed out as halves
    const int n_full = n_items - n_split, n_units = n_items + n_split, mid = (nch + 1) / 2;
    unsigned next_raw = 0; // lane 0: the unit after the current one, already requested
    if (lane == 0) next_raw = atomicAdd(&work[0], 1u) + (unsigned)n_warps;
    // the unit being requested: item, chunk range, part (0 whole item, 1 head half, 2 tail half)
    int p_item = 0, p_ch = 0, p_end = 0, p_part = 0;
    bool p_valid = false;
    auto open_unit = [&](unsigned u) {
        p_valid = u < (unsigned)n_units;
        if (!p_valid) return;
        if ((int)u < n_full) {
            p_item = (int)u; p_ch = 0; p_end = nch; p_part = 0;
        } else {
            const int k = (int)u - n_full, half = k & 1;
            p_item = n_full + (k >> 1);
            if (nch < 2) { // nothing to halve: the head half is the whole item, the tail half is empty
                p_ch = 0; p_end = half ? 0 : nch; p_part = 0;
            } else {
                p_ch = half ? mid : 0; p_end = half ? nch : mid; p_part = 1 + half;
            }
        }
    };
    auto next_unit = [&]() {
        do {
            const unsigned u = __shfl_sync(0xffffffffu, next_raw, 0);
            if (lane == 0 && u < (unsigned)n_units) next_raw = atomicAdd(&work[0], 1u) + (unsigned)n_warps;
            open_unit(u);
        } while (p_valid && p_ch >= p_end); // skip empty units
    };
    open_unit((unsigned)gw);
    int issued = 0, consumed = 0;   // chunks requested / finished by this warp
    float m = NEG_BIG, l = 0.0f;
    float2 acc2[4], qf2[4]; // dims (2i, 2i+1) of this lane's eight: accumulator and scaled query
    bool ok = true;

    while (true) {
        // keep NST stages requested
        while (issued - consumed < NST && p_valid) {
            const int s = issued % NST;
            const bool first = (p_ch == 0) || (p_part == 2 && p_ch == mid), last = (p_ch == p_end - 1);
            if (lane == 0) {
                const int rows = min(ROWS, ctx - p_ch * ROWS);
                const uint32_t bar = tc::smem_u32(&full_bar[warp][s]), dst = ring + s * STAGE_BYTES;
                const size_t off = ((size_t)p_item * cap + (size_t)p_ch * ROWS) * 64;
                tc::mbar_expect_tx(bar, rows * 256 + (first ? 64 * (uint32_t)sizeof(QT) : 0u));
                tc::tma_load_1d(dst, kc + off, rows * 128, bar);
                tc::tma_load_1d(dst + ROWS * 128, vc + off, rows * 128, bar);
                if (first) {
                    const int pb = p_item / H, ph = p_item - pb * H;
                    tc::tma_load_1d(dst + 2 * ROWS * 128, q + (size_t)pb * ldq + ph * 64, 64 * (uint32_t)sizeof(QT), bar);
                }
                meta[warp][s] = make_int2(p_item, p_ch | (first ? 0x100 : 0) | (last ? 0x200 : 0) | (p_part << 10));
            }
            ++issued;
            if (++p_ch == p_end) next_unit();
        }
        if (consumed == issued) break;
        const int s = consumed % NST;
        ok = tc::mbar_wait(tc::smem_u32(&full_bar[warp][s]), (consumed / NST) & 1, &abort_flag, dev_err, ERR_FULL);
        if (!ok) break;
        __syncwarp();
        const int2 mraw = meta[warp][s];
        const int2 mt = make_int2(mraw.x, mraw.y & 0xff); // (item, chunk)
        const bool u_first = (mraw.y & 0x100) != 0, u_last = (mraw.y & 0x200) != 0;
        const int u_part = mraw.y >> 10;
        const uint8_t *st = ring_gen + s * STAGE_BYTES;
        if (u_first) {
            m = NEG_BIG;
            l = 0.0f;
#pragma unroll
            for (int i = 0; i < 4; ++i) acc2[i] = make_float2(0.0f, 0.0f);
            const QT *qs = reinterpret_cast<const QT *>(st + 2 * ROWS * 128);
#pragma unroll
            for (int i = 0; i < 4; ++i)
                qf2[i] = make_float2(load_as_float<QT>(qs, c * 8 + 2 * i) * ATT_SCALE_LOG2E,
                                     load_as_float<QT>(qs, c * 8 + 2 * i + 1) * ATT_SCALE_LOG2E);
        }
        const int rows = min(ROWS, ctx - mt.y * ROWS);
        const uint4 *ks = reinterpret_cast<const uint4 *>(st);
        const uint4 *vs = reinterpret_cast<const uint4 *>(st + ROWS * 128);
#if B200NN_ATTN_PROBE == 1
        if (rows < 0) // measurement build: no arithmetic, the warp only waits for its stages and releases them
#endif
#pragma unroll
        for (int half = 0; half < ROWS / 16; ++half) {
            constexpr int R = 4;
            uint4 kr[R], vr[R];
            bool valid[R];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int row = half * 16 + r * 4 + g;
                valid[r] = row < rows;
                kr[r] = make_uint4(0, 0, 0, 0);
                vr[r] = kr[r];
                if (valid[r]) {
                    kr[r] = ks[row * 8 + c];
#if B200NN_ATTN_PROBE != 3
                    vr[r] = vs[row * 8 + c];
#endif
                }
            }
            float sc[R];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                // packed f32x2 FMAs: even dims in .x, odd dims in .y, one add at the end
                const __half2 *kh = reinterpret_cast<const __half2 *>(&kr[r]);
                float2 t2 = make_float2(0.0f, 0.0f);
#pragma unroll
                for (int i = 0; i < 4; ++i) t2 = __ffma2_rn(qf2[i], __half22float2(kh[i]), t2);
                sc[r] = t2.x + t2.y;
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
            for (int i = 0; i < 4; ++i) acc2[i] = __fmul2_rn(acc2[i], make_float2(corr, corr));
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const float p = valid[r] ? exp2f(sc[r] - m_new) : 0.0f;
                l += p;
#if B200NN_ATTN_PROBE == 2   // measurement build: V rows read, no conversion and no p·V
                acc2[r].x += p * __uint_as_float(vr[r].x ^ vr[r].y ^ vr[r].z ^ vr[r].w);
#elif B200NN_ATTN_PROBE == 3 // measurement build: V rows not read from shared memory either
                acc2[r].x += p;
#else
                const __half2 *vh = reinterpret_cast<const __half2 *>(&vr[r]);
                const float2 p2 = make_float2(p, p);
#pragma unroll
                for (int i = 0; i < 4; ++i) acc2[i] = __ffma2_rn(p2, __half22float2(vh[i]), acc2[i]);
#endif
            }
            m = m_new;
        }
        __syncwarp(); // every lane has read the stage: it may be requested again
        ++consumed;
        if (u_last) {
            float acc[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) { acc[2 * i] = acc2[i].x; acc[2 * i + 1] = acc2[i].y; }
            // merge the four lane groups (lanes 8 and 16 apart hold the same 8 dims)
#pragma unroll
            for (int off = 8; off <= 16; off <<= 1) {
                const float m_o = __shfl_xor_sync(0xffffffffu, m, off), l_o = __shfl_xor_sync(0xffffffffu, l, off);
                const float m_n = fmaxf(m, m_o);
                const float ws = exp2f(m - m_n), wo = exp2f(m_o - m_n);
                l = l * ws + l_o * wo;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float a_o = __shfl_xor_sync(0xffffffffu, acc[i], off);
                    acc[i] = acc[i] * ws + a_o * wo;
                }
                m = m_n;
            }
            bool write_out = true;
            if (u_part != 0) {
                // half of an item: leave a (max, sum, output) record; the half that arrives second on
                // the item's counter merges both and writes the result
                const int slot = mt.x - n_full;
                float *rec = scratch + ((size_t)slot * 2 + (u_part - 1)) * REC_FLOATS;
                if (g == 0) {
                    if (c == 0) { rec[0] = m; rec[1] = l; }
                    *reinterpret_cast<float4 *>(rec + 8 + c * 8) = make_float4(acc[0], acc[1], acc[2], acc[3]);
                    *reinterpret_cast<float4 *>(rec + 12 + c * 8) = make_float4(acc[4], acc[5], acc[6], acc[7]);
                }
                __threadfence();
                __syncwarp();
                unsigned prev = 0;
                if (lane == 0) {
                    prev = atomicAdd(&counters[slot], 1u);
                    if (prev == 1u) counters[slot] = 0u; // both halves are in: zero at rest again
                }
                prev = __shfl_sync(0xffffffffu, prev, 0);
                write_out = (prev == 1u);
                if (write_out) {
                    __threadfence();
                    const float *oth = scratch + ((size_t)slot * 2 + (2 - u_part)) * REC_FLOATS;
                    const float m_o = __ldcg(oth), l_o = __ldcg(oth + 1);
                    const float4 a0 = __ldcg(reinterpret_cast<const float4 *>(oth + 8 + c * 8));
                    const float4 a1 = __ldcg(reinterpret_cast<const float4 *>(oth + 12 + c * 8));
                    const float ao[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
                    const float m_n = fmaxf(m, m_o);
                    const float ws = exp2f(m - m_n), wo = exp2f(m_o - m_n);
                    // separately rounded products and a plain add: the same bits whichever half merges
                    l = __fadd_rn(__fmul_rn(l, ws), __fmul_rn(l_o, wo));
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[i] = __fadd_rn(__fmul_rn(acc[i], ws), __fmul_rn(ao[i], wo));
                }
            }
            if (g == 0 && write_out) {
                const float inv = 1.0f / l;
                const int ob = mt.x / H, oh = mt.x - ob * H;
                OT *dst = out + (size_t)ob * ldo + oh * 64 + c * 8;
                if constexpr (sizeof(OT) == 2) {
                    uint4 v;
                    __half2 h0 = __floats2half2_rn(acc[0] * inv, acc[1] * inv), h1 = __floats2half2_rn(acc[2] * inv, acc[3] * inv);
                    __half2 h2 = __floats2half2_rn(acc[4] * inv, acc[5] * inv), h3 = __floats2half2_rn(acc[6] * inv, acc[7] * inv);
                    v.x = *reinterpret_cast<uint32_t *>(&h0);
                    v.y = *reinterpret_cast<uint32_t *>(&h1);
                    v.z = *reinterpret_cast<uint32_t *>(&h2);
                    v.w = *reinterpret_cast<uint32_t *>(&h3);
                    *reinterpret_cast<uint4 *>(dst) = v;
                } else {
                    *reinterpret_cast<float4 *>(dst) = make_float4(acc[0] * inv, acc[1] * inv, acc[2] * inv, acc[3] * inv);
                    *reinterpret_cast<float4 *>(dst + 4) = make_float4(acc[4] * inv, acc[5] * inv, acc[6] * inv, acc[7] * inv);
                }
            }
        }
    }
    // Copies still in flight into this block's shared memory must land before the block exits.
    if (!ok) {
        for (; consumed < issued; ++consumed) {
            const uint32_t bar = tc::smem_u32(&full_bar[warp][consumed % NST]);
            const long long t0 = clock64();
            while (!tc::mbar_test(bar, (consumed / NST) & 1) && clock64() - t0 < tc::WAIT_CYCLES) { }
        }
    }
    // the last warp of the grid to finish puts the work counters back to zero for the next launch
    if (lane == 0) {
        __threadfence();
        const unsigned done = atomicAdd(&work[1], 1u);
        if (done == gridDim.x * WARPS - 1) {
            work[0] = 0u;
            work[1] = 0u;
            __threadfence();
        }
    }
}

int launch_decode_attention(b200nn_ctx *ctx, const void *q, bool q_half, int ldq, const __half *kc,
                            const __half *vc, int B, int H, int cap, const int *pos_ptr, int pos_off, void *out,
                            bool out_half, int max_ctx_hint) {
    if (B <= 0) return B200NN_OK;
    int pairs = B * H;
    const size_t q_elem = q_half ? 2 : 4;
    // block shape of the TMA-fed kernel by pairs per warp of its grid: 16 warps, else 8 warps, else the split kernel
    const bool wide = ctx->attn_stream_wide_min10 > 0 && cap <= 255 * 16 && // a stage's chunk index has eight bits
                      10LL * pairs >= (long long)ctx->attn_stream_wide_min10 * ctx->sm_count * 16;
    const int s_warps = wide ? 16 : 8, s_rows = wide ? 16 : 32;
    if (ctx->attn_stream && 10LL * pairs >= (long long)ctx->attn_stream_min10 * ctx->sm_count * s_warps &&
        cap <= 255 * s_rows &&
        ((uintptr_t)q & 15) == 0 &&
        (ldq * q_elem) % 16 == 0 && ((uintptr_t)out & 15) == 0) {
        const int ldo_s = H * 64;
        unsigned *work = reinterpret_cast<unsigned *>(ctx->dev_err) + 2;
        // records and counters of the half-items the grid finishes on (two halves of n_warps items)
        const size_t n_w = (size_t)ctx->sm_count * s_warps;
        TRY(ensure_scratch(ctx, n_w * 2 * stream_attn::REC_FLOATS * sizeof(float), n_w));
        // items whose cached rows are requested into L2 ahead of the dependency wait
        const size_t item_bytes = (size_t)2 * cap * 128;
        const int pf_items = (int)std::min<size_t>((size_t)pairs, ((size_t)ctx->kv_prefetch_mb << 20) / item_bytes);
#define DS2(QT, OT, W, R)                                                                                            \
    {                                                                                                                \
        static bool attr_done[16] = {};                                                                              \
        if (!attr_done[ctx->device & 15]) {                                                                          \
            CK(ctx, cudaFuncSetAttribute(decode_attn_stream_kernel<QT, OT, W, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                         stream_attn::smem_bytes(W, R)));                                            \
            prefer_max_smem(decode_attn_stream_kernel<QT, OT, W, R>);                                                \
            attr_done[ctx->device & 15] = true;                                                                      \
        }                                                                                                            \
        launch_pdl(ctx, decode_attn_stream_kernel<QT, OT, W, R>, dim3(ctx->sm_count), dim3(W * 32),                  \
                   stream_attn::smem_bytes(W, R), (const QT *)q, ldq, kc, vc, H, cap, pos_ptr, pos_off, (OT *)out,   \
                   ldo_s, pairs, pf_items, std::min(ctx->attn_split_items, (int)n_w), work, ctx->scratch,           \
                   ctx->counters, ctx->dev_err);                                                                     \
    }
#define DS(QT, OT)                                                                                                   \
    {                                                                                                                \
        if (wide) DS2(QT, OT, 16, 16) else DS2(QT, OT, 8, 32)                                                        \
    }
        if (q_half && out_half) DS(__half, __half)
        else if (q_half) DS(__half, float)
        else if (out_half) DS(float, __half)
        else DS(float, float)
#undef DS
#undef DS2
        CK_LAUNCH(ctx, "decode_attn_stream_kernel");
        return B200NN_OK;
    }
    int n_splits = (ctx->attn_blocks_per_sm * ctx->sm_count + pairs - 1) / pairs;
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
    if (q_half && out_half && ctx->attn_tc && (ldq & 7) == 0 && ((uintptr_t)q & 15) == 0 && ((uintptr_t)out & 15) == 0)
        return launch_prefill_attention_tc(ctx, (const __half *)q, ldq, kc, vc, B, H, cap, S, past, (__half *)out);
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

// ---------------------------------------------------------------------------------------------
// Decode attention for callers that must not allocate device memory.
//
// The split-context form of decode_attn_kernel needs scratch: one (max, sum, output[64]) record per
// (sequence, head, split) and one arrival counter per (sequence, head).  The regular entry points
// take it from the context's scratch buffer, which grows with cudaMalloc on demand.  Some callers
// cannot have that: code running in a real-time loop, where cudaMalloc would synchronise the
// device and stall everything queued on it, or a host application whose memory budget is fixed up front and
// that hands this library only the buffers it owns.  For them the scratch below lives in the
// library's own image: two file-scope __device__ arrays of fixed size (about 4.2 MB, present on
// every GPU that loads the library until the process exits).
//
// In host code the array names are host-side stand-ins, not device addresses; the device address
// is obtained once per device with cudaGetSymbolAddress (with that device current) and passed to
// the kernel.  That first call on a device is the set-up and should come before any stream
// capture.  All calls share the arrays: the counters are cleared on the caller's stream before
// every launch, the records are fully rewritten by each call, and two calls that overlap on the
// GPU (different streams) race on them.
// ---------------------------------------------------------------------------------------------
static constexpr int NOALLOC_MAX_PAIRS = 4096;    // sequences x heads
static constexpr int NOALLOC_MAX_RECORDS = 16384; // sequences x heads x splits
static __device__ __align__(256) float g_noalloc_records[NOALLOC_MAX_RECORDS * 66];
static __device__ __align__(256) unsigned g_noalloc_counters[NOALLOC_MAX_PAIRS];

namespace {
constexpr int NOALLOC_MAX_DEVICES = 64;
struct NoAllocDevice {
    bool ready = false;
    float *records = nullptr;
    unsigned *counters = nullptr;
    int sm_count = 0;
};
NoAllocDevice g_noalloc_dev[NOALLOC_MAX_DEVICES];
std::mutex g_noalloc_mu;
thread_local char g_noalloc_error[256] = "";

int noalloc_fail(int code, const char *msg, cudaError_t e = cudaSuccess) {
    if (e != cudaSuccess)
        snprintf(g_noalloc_error, sizeof(g_noalloc_error), "%s: %s", msg, cudaGetErrorString(e));
    else
        snprintf(g_noalloc_error, sizeof(g_noalloc_error), "%s", msg);
    return code;
}
}  // namespace

extern "C" const char *b200nn_noalloc_last_error(void) { return g_noalloc_error; }

extern "C" int32_t b200nn_decode_attention_noalloc(int32_t device, void *stream, const float *q_dev,
                                                   const void *k_cache_dev, const void *v_cache_dev, int32_t batch,
                                                   int32_t n_heads, int32_t capacity, int32_t ctx_len, float *out_dev) {
    if (!q_dev || !k_cache_dev || !v_cache_dev || !out_dev) return noalloc_fail(B200NN_ERR_ARG, "null buffer");
    // the kernel reads cached rows with 16-byte loads: a misaligned cache would fault on the device
    if ((reinterpret_cast<uintptr_t>(k_cache_dev) | reinterpret_cast<uintptr_t>(v_cache_dev)) & 15)
        return noalloc_fail(B200NN_ERR_ARG, "k_cache_dev and v_cache_dev must be 16-byte aligned");
    if (device < 0 || device >= NOALLOC_MAX_DEVICES) return noalloc_fail(B200NN_ERR_ARG, "device ordinal out of range");
    if (batch <= 0 || n_heads <= 0 || capacity <= 0 || ctx_len <= 0 || ctx_len > capacity)
        return noalloc_fail(B200NN_ERR_SHAPE, "batch, n_heads, capacity must be positive and 1 <= ctx_len <= capacity");
    const long long pairs = (long long)batch * n_heads;
    if (pairs > NOALLOC_MAX_PAIRS)
        return noalloc_fail(B200NN_ERR_SHAPE, "batch * n_heads exceeds the fixed scratch (4096 pairs)");
    int prev = -1;
    cudaError_t e = cudaGetDevice(&prev);
    if (e != cudaSuccess) return noalloc_fail(B200NN_ERR_CUDA, "cudaGetDevice", e);
    if (prev != device && (e = cudaSetDevice(device)) != cudaSuccess) return noalloc_fail(B200NN_ERR_CUDA, "cudaSetDevice", e);
    int rc = B200NN_OK;
    NoAllocDevice &D = g_noalloc_dev[device];
    std::lock_guard<std::mutex> setup_guard(g_noalloc_mu); // host threads may share a device's set-up
    if (!D.ready) { // set-up, once per device, with that device current
        void *rp = nullptr, *cp = nullptr;
        if ((e = cudaGetSymbolAddress(&rp, g_noalloc_records)) != cudaSuccess)
            rc = noalloc_fail(B200NN_ERR_CUDA, "cudaGetSymbolAddress(records)", e);
        else if ((e = cudaGetSymbolAddress(&cp, g_noalloc_counters)) != cudaSuccess)
            rc = noalloc_fail(B200NN_ERR_CUDA, "cudaGetSymbolAddress(counters)", e);
        else if ((e = cudaDeviceGetAttribute(&D.sm_count, cudaDevAttrMultiProcessorCount, device)) != cudaSuccess)
            rc = noalloc_fail(B200NN_ERR_CUDA, "cudaDeviceGetAttribute", e);
        else {
            D.records = static_cast<float *>(rp);
            D.counters = static_cast<unsigned *>(cp);
            D.ready = true;
        }
    }
    if (rc == B200NN_OK) {
        // same split rule as the regular path, bounded by the fixed scratch
        int n_splits = (int)((4LL * D.sm_count + pairs - 1) / pairs);
        n_splits = std::min(n_splits, (ctx_len + 63) / 64);
        n_splits = std::min(n_splits, 32);
        n_splits = std::min(n_splits, (int)(NOALLOC_MAX_RECORDS / pairs));
        n_splits = std::max(n_splits, 1);
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        if ((e = cudaMemsetAsync(D.counters, 0, (size_t)pairs * sizeof(unsigned), st)) != cudaSuccess)
            rc = noalloc_fail(B200NN_ERR_CUDA, "cudaMemsetAsync(counters)", e);
        else {
            dim3 grid(n_heads, batch, n_splits);
            decode_attn_kernel<float, float><<<grid, 128, 0, st>>>(
                q_dev, n_heads * 64, static_cast<const __half *>(k_cache_dev), static_cast<const __half *>(v_cache_dev),
                n_heads, capacity, nullptr, ctx_len - 1, out_dev, n_heads * 64, D.records, D.counters);
            if ((e = cudaPeekAtLastError()) != cudaSuccess) rc = noalloc_fail(B200NN_ERR_CUDA, "kernel launch", e);
        }
    }
    if (prev != device && prev >= 0) cudaSetDevice(prev);
    return rc;
}
