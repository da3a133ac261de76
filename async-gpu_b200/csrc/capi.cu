// extern "C" surface: context, tensors, stateless ops and the single layers.
#include <algorithm>
#include <cmath>
#include <cstring>

#include "model.h"

extern "C" const char *b200nn_version(void) { return "b200nn 0.1 (sm_100a)"; }

// ---------------------------------------------------------------------------------------------
// context
// ---------------------------------------------------------------------------------------------
extern "C" int32_t b200nn_ctx_create(int32_t device, b200nn_ctx **out) {
    if (!out) return B200NN_ERR_ARG;
    *out = nullptr;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n <= 0 || device < 0 || device >= n) return B200NN_ERR_CUDA; // no CPU fallback
    auto *ctx = new b200nn_ctx();
    ctx->device = device;
    auto fail = [&](cudaError_t err) {
        (void)err;
        delete ctx;
        return (int32_t)B200NN_ERR_CUDA;
    };
    if ((e = cudaSetDevice(device)) != cudaSuccess) return fail(e);
    cudaDeviceProp prop;
    if ((e = cudaGetDeviceProperties(&prop, device)) != cudaSuccess) return fail(e);
    if (prop.major != 10) { // kernels are built for sm_100a only
        delete ctx;
        return B200NN_ERR_UNSUPPORTED;
    }
    ctx->sm_count = prop.multiProcessorCount;
    if ((e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking)) != cudaSuccess) return fail(e);
    // word 0: device error word; words 2,3: the streaming decode attention's work counters (zero at rest)
    if ((e = cudaMalloc(&ctx->dev_err, 4 * sizeof(uint32_t))) != cudaSuccess) return fail(e);
    if ((e = cudaMemset(ctx->dev_err, 0, 4 * sizeof(uint32_t))) != cudaSuccess) return fail(e);
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ctx->encode_tiled, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
        ctx->encode_tiled = nullptr;
    if (ensure_scratch(ctx, (size_t)32 << 20, 65536) != B200NN_OK) return fail(cudaErrorMemoryAllocation);
    *out = ctx;
    return B200NN_OK;
}

extern "C" void b200nn_ctx_destroy(b200nn_ctx *ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    if (ctx->stream) {
        cudaStreamSynchronize(ctx->stream);
        cudaStreamDestroy(ctx->stream);
    }
    if (ctx->dev_err) cudaFree(ctx->dev_err);
    if (ctx->host_err) cudaFreeHost(ctx->host_err);
    if (ctx->persist_trace) cudaFree(ctx->persist_trace);
    if (ctx->scratch) cudaFree(ctx->scratch);
    if (ctx->counters) cudaFree(ctx->counters);
    for (void *p : ctx->retired) cudaFree(p);
    ctx->xh.reset();
    ctx->wh.reset();
    pool_trim(ctx);
    {
        std::lock_guard<std::mutex> g(ctx->pool->mu);
        ctx->pool->alive = false; // buffers that outlive the context free directly
    }
    delete ctx;
}

extern "C" int32_t b200nn_ctx_trim(b200nn_ctx *ctx) {
    if (!ctx) return B200NN_ERR_ARG;
    CK(ctx, cudaSetDevice(ctx->device));
    CK(ctx, cudaStreamSynchronize(ctx->stream));
    pool_trim(ctx);
    return B200NN_OK;
}

extern "C" int32_t b200nn_ctx_synchronize(b200nn_ctx *ctx) {
    if (!ctx) return B200NN_ERR_ARG;
    CK(ctx, cudaSetDevice(ctx->device));
    return stream_sync_check(ctx);
}
extern "C" void *b200nn_ctx_stream(b200nn_ctx *ctx) { return ctx ? (void *)ctx->stream : nullptr; }
extern "C" const char *b200nn_last_error_message(b200nn_ctx *ctx) { return ctx ? ctx->last_error.c_str() : "null context"; }
extern "C" int32_t b200nn_last_cuda_error(b200nn_ctx *ctx) { return ctx ? ctx->last_cuda : 0; }
extern "C" uint64_t b200nn_ctx_launch_count(b200nn_ctx *ctx) { return ctx ? ctx->launches : 0; }
extern "C" int32_t b200nn_ctx_set_gemv_max_rows(b200nn_ctx *ctx, int32_t rows) {
    if (!ctx) return B200NN_ERR_ARG;
    ctx->gemv_max_rows = rows < 0 ? 2 : rows;
    return B200NN_OK;
}
extern "C" int32_t b200nn_ctx_set_tuning(b200nn_ctx *ctx, const char *key, int32_t value) {
    if (!ctx || !key) return B200NN_ERR_ARG;
    if (!strcmp(key, "tc_mb")) ctx->tc_mb = value;
    else if (!strcmp(key, "tc_splits")) ctx->tc_splits = value;
    else if (!strcmp(key, "tc_min_kb")) ctx->tc_min_kb = value < 0 ? 0 : value;
    else if (!strcmp(key, "tc_min_kb_cluster")) ctx->tc_min_kb_cluster = value < 1 ? 1 : value;
    else if (!strcmp(key, "pdl")) ctx->pdl = value ? 1 : 0;
    else if (!strcmp(key, "f32_tc")) ctx->f32_tc = value < 0 ? 2 : (value > 2 ? 2 : value);
    else if (!strcmp(key, "tc_persistent")) ctx->tc_persistent = value ? 1 : 0;
    else if (!strcmp(key, "int4_via_f16")) ctx->int4_via_f16 = value ? 1 : 0;
    else if (!strcmp(key, "attn_tc")) ctx->attn_tc = value ? 1 : 0;
    else if (!strcmp(key, "attn_stream")) ctx->attn_stream = value ? 1 : 0;
    else if (!strcmp(key, "attn_stream_min10")) ctx->attn_stream_min10 = value < 1 ? 1 : value;
    else if (!strcmp(key, "attn_stream_wide_min10")) ctx->attn_stream_wide_min10 = value < 0 ? 0 : value;
    else if (!strcmp(key, "kv_prefetch_mb")) ctx->kv_prefetch_mb = value < 0 ? 0 : value;
    else if (!strcmp(key, "attn_split_items")) ctx->attn_split_items = value < 0 ? 0 : value;
    else if (!strcmp(key, "attn_blocks_per_sm")) ctx->attn_blocks_per_sm = value < 1 ? 4 : value;
    else if (!strcmp(key, "trace")) { // value != 0: allocate (once) and clear a 256-slot stamp buffer
        if (value && !ctx->trace && cudaMalloc(&ctx->trace, 256 * sizeof(long long)) != cudaSuccess) return B200NN_ERR_CUDA;
        if (ctx->trace) cudaMemset(ctx->trace, 0, 256 * sizeof(long long));
        if (!value && ctx->trace) { cudaFree(ctx->trace); ctx->trace = nullptr; }
    }
    else if (!strcmp(key, "gemv_max_rows")) ctx->gemv_max_rows = value < 0 ? 2 : value;
    else if (!strcmp(key, "fused_argmax")) ctx->fused_argmax = value ? 1 : 0;
    else if (!strcmp(key, "ln_fold")) ctx->ln_fold = value ? 1 : 0;
    else if (!strcmp(key, "ln_rows_min")) ctx->ln_rows_min = value > 0 ? value : 1024;
    else if (!strcmp(key, "persist")) ctx->persist = value ? 1 : 0;
    else if (!strcmp(key, "persist_min_rows")) ctx->persist_min_rows = value < 1 ? 3 : value;
    else if (!strcmp(key, "persist_max_rows")) ctx->persist_max_rows = value < 1 ? 256 : value;
    else if (!strcmp(key, "persist_prefetch_mb")) ctx->persist_prefetch_mb = value < 0 ? 0 : value;
    else if (!strcmp(key, "persist_wait_kcycles")) ctx->persist_wait_cycles = value <= 0 ? 0 : 1000LL * value;
    else if (!strcmp(key, "persist_fault_phase")) ctx->persist_fault_phase = value;
    else if (!strcmp(key, "persist_trace")) { // value != 0: allocate (once) and clear the phase-stamp buffer
        const size_t bytes = (size_t)256 * 32 * 2 * sizeof(unsigned long long);
        if (value && !ctx->persist_trace && cudaMalloc(&ctx->persist_trace, bytes) != cudaSuccess) return B200NN_ERR_CUDA;
        if (ctx->persist_trace) cudaMemset(ctx->persist_trace, 0, bytes);
        if (!value && ctx->persist_trace) { cudaStreamSynchronize(ctx->stream); cudaFree(ctx->persist_trace); ctx->persist_trace = nullptr; }
    }
    else return set_error(ctx, B200NN_ERR_UNSUPPORTED, std::string("unknown tuning key ") + key);
    return B200NN_OK;
}
extern "C" int32_t b200nn_ctx_read_trace(b200nn_ctx *ctx, long long *out256) {
    if (!ctx || !out256 || !ctx->trace) return B200NN_ERR_ARG;
    CK(ctx, cudaStreamSynchronize(ctx->stream));
    CK(ctx, cudaMemcpy(out256, ctx->trace, 256 * sizeof(long long), cudaMemcpyDeviceToHost));
    return B200NN_OK;
}
extern "C" int32_t b200nn_ctx_read_persist_trace(b200nn_ctx *ctx, unsigned long long *out, size_t capacity) {
    if (!ctx || !out || !ctx->persist_trace) return B200NN_ERR_ARG;
    const size_t n = std::min(capacity, (size_t)256 * 32 * 2);
    CK(ctx, cudaStreamSynchronize(ctx->stream));
    CK(ctx, cudaMemcpy(out, ctx->persist_trace, n * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
    return B200NN_OK;
}
extern "C" int32_t b200nn_ctx_device_error(b200nn_ctx *ctx, uint32_t *word_out) {
    if (!ctx || !word_out) return B200NN_ERR_ARG;
    CK(ctx, cudaSetDevice(ctx->device));
    CK(ctx, cudaMemcpyAsync(word_out, ctx->dev_err, 4, cudaMemcpyDeviceToHost, ctx->stream));
    CK(ctx, cudaStreamSynchronize(ctx->stream));
    if (*word_out) CK(ctx, cudaMemsetAsync(ctx->dev_err, 0, 4, ctx->stream));
    return *word_out ? B200NN_ERR_DEVICE : B200NN_OK;
}

// ---------------------------------------------------------------------------------------------
// tensors
// ---------------------------------------------------------------------------------------------
static std::vector<size_t> shape_vec(const size_t *shape, int32_t ndim) { return std::vector<size_t>(shape, shape + ndim); }

extern "C" int32_t b200nn_tensor_from_host(b200nn_ctx *ctx, const float *host, const size_t *shape, int32_t ndim,
                                           b200nn_tensor **out) {
    if (!ctx || !shape || ndim <= 0 || !out) return B200NN_ERR_ARG;
    b200nn_tensor *t = nullptr;
    TRY(tensor_alloc(ctx, shape_vec(shape, ndim), false, &t));
    if (t->numel) {
        if (!host) { delete t; return B200NN_ERR_ARG; }
        cudaError_t e = cudaMemcpyAsync(t->buf->p, host, t->numel * 4, cudaMemcpyHostToDevice, ctx->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
        if (e != cudaSuccess) { delete t; return set_cuda_error(ctx, e, "tensor_from_host"); }
    }
    *out = t;
    return B200NN_OK;
}
extern "C" int32_t b200nn_tensor_from_device(b200nn_ctx *ctx, const float *dev, const size_t *shape, int32_t ndim,
                                             b200nn_tensor **out) {
    if (!ctx || !shape || ndim <= 0 || !out) return B200NN_ERR_ARG;
    b200nn_tensor *t = nullptr;
    TRY(tensor_alloc(ctx, shape_vec(shape, ndim), false, &t));
    if (t->numel) {
        if (!dev) { delete t; return B200NN_ERR_ARG; }
        cudaError_t e = cudaMemcpyAsync(t->buf->p, dev, t->numel * 4, cudaMemcpyDeviceToDevice, ctx->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
        if (e != cudaSuccess) { delete t; return set_cuda_error(ctx, e, "tensor_from_device"); }
    }
    *out = t;
    return B200NN_OK;
}
extern "C" int32_t b200nn_tensor_zeros(b200nn_ctx *ctx, const size_t *shape, int32_t ndim, b200nn_tensor **out) {
    if (!ctx || !shape || ndim <= 0 || !out) return B200NN_ERR_ARG;
    return tensor_alloc(ctx, shape_vec(shape, ndim), true, out);
}
extern "C" int32_t b200nn_tensor_to_host(const b200nn_tensor *t, float *host, size_t capacity_elems) {
    if (!t || !host) return B200NN_ERR_ARG;
    b200nn_ctx *ctx = t->ctx;
    if (capacity_elems < t->numel) return set_error(ctx, B200NN_ERR_SHAPE, "to_host: destination too small");
    CK(ctx, cudaSetDevice(ctx->device));
    CK(ctx, cudaMemcpyAsync(host, t->buf->p, t->numel * 4, cudaMemcpyDeviceToHost, ctx->stream));
    return stream_sync_check(ctx);
}
extern "C" int32_t b200nn_tensor_ndim(const b200nn_tensor *t) { return t ? (int32_t)t->shape.size() : 0; }
extern "C" size_t b200nn_tensor_numel(const b200nn_tensor *t) { return t ? t->numel : 0; }
extern "C" int32_t b200nn_tensor_shape(const b200nn_tensor *t, size_t *shape_out, int32_t capacity) {
    if (!t || !shape_out) return B200NN_ERR_ARG;
    if (capacity < (int32_t)t->shape.size()) return B200NN_ERR_DIM;
    for (size_t i = 0; i < t->shape.size(); ++i) shape_out[i] = t->shape[i];
    return B200NN_OK;
}
extern "C" int32_t b200nn_tensor_reshape(const b200nn_tensor *t, const size_t *shape, int32_t ndim, b200nn_tensor **out) {
    if (!t || !shape || ndim <= 0 || !out) return B200NN_ERR_ARG;
    size_t n = 1;
    for (int i = 0; i < ndim; ++i) n *= shape[i];
    if (n != t->numel) return set_error(t->ctx, B200NN_ERR_SHAPE, "reshape: element count differs"); // tensor.rs:201-221
    auto *r = new b200nn_tensor(*t); // shares the buffer, as the reference's Arc<CudaSlice> does
    r->shape = shape_vec(shape, ndim);
    *out = r;
    return B200NN_OK;
}
extern "C" int32_t b200nn_tensor_clone(const b200nn_tensor *t, b200nn_tensor **out) {
    if (!t || !out) return B200NN_ERR_ARG;
    b200nn_ctx *ctx = t->ctx;
    b200nn_tensor *c = nullptr;
    TRY(tensor_alloc(ctx, t->shape, false, &c));
    cudaError_t e = cudaMemcpyAsync(c->buf->p, t->buf->p, t->numel * 4, cudaMemcpyDeviceToDevice, ctx->stream);
    if (e != cudaSuccess) { delete c; return set_cuda_error(ctx, e, "tensor_clone"); }
    *out = c;
    return B200NN_OK;
}
// GpuTensor::transpose / concat / split (tensor.rs:227-393), on the device.
extern "C" int32_t b200nn_tensor_transpose(const b200nn_tensor *t, size_t dim0, size_t dim1, b200nn_tensor **out) {
    if (!t || !out) return B200NN_ERR_ARG;
    b200nn_ctx *ctx = t->ctx;
    const size_t nd = t->shape.size();
    if (dim0 >= nd || dim1 >= nd)
        return set_error(ctx, B200NN_ERR_DIM, "transpose: dim " + std::to_string(dim0 >= nd ? dim0 : dim1) + " out of range for " +
                                                  std::to_string(nd) + " dimensions");
    if (dim0 == dim1) return b200nn_tensor_clone(t, out);
    std::vector<size_t> oshape(t->shape);
    std::swap(oshape[dim0], oshape[dim1]);
    b200nn_tensor *r = nullptr;
    TRY(tensor_alloc(ctx, oshape, false, &r));
    int rc = launch_tensor_transpose(ctx, t->data(), r->data(), t->shape, (int)dim0, (int)dim1);
    if (rc != B200NN_OK) { delete r; return rc; }
    *out = r;
    return B200NN_OK;
}

// A contiguous tensor seen as [outer][shape[dim]][inner].
static void outer_inner(const std::vector<size_t> &shape, size_t dim, size_t *outer, size_t *inner) {
    *outer = *inner = 1;
    for (size_t d = 0; d < dim; ++d) *outer *= shape[d];
    for (size_t d = dim + 1; d < shape.size(); ++d) *inner *= shape[d];
}

extern "C" int32_t b200nn_tensor_concat(const b200nn_tensor *const *tensors, size_t count, size_t dim, b200nn_tensor **out) {
    if (!tensors || !out) return B200NN_ERR_ARG;
    if (count == 0) return B200NN_ERR_SHAPE; // "at least one tensor"
    for (size_t i = 0; i < count; ++i)
        if (!tensors[i]) return B200NN_ERR_ARG;
    b200nn_ctx *ctx = tensors[0]->ctx;
    const std::vector<size_t> &s0 = tensors[0]->shape;
    const size_t nd = s0.size();
    if (dim >= nd) return set_error(ctx, B200NN_ERR_DIM, "concat: dim out of range");
    size_t total = 0;
    for (size_t i = 0; i < count; ++i) {
        const std::vector<size_t> &si = tensors[i]->shape;
        if (si.size() != nd) return set_error(ctx, B200NN_ERR_SHAPE, "concat: tensor " + std::to_string(i) + " has another number of dimensions");
        for (size_t d = 0; d < nd; ++d)
            if (d != dim && si[d] != s0[d])
                return set_error(ctx, B200NN_ERR_SHAPE, "concat: tensor " + std::to_string(i) + " differs in dim " + std::to_string(d));
        total += si[dim];
    }
    std::vector<size_t> oshape(s0);
    oshape[dim] = total;
    size_t outer, inner;
    outer_inner(oshape, dim, &outer, &inner);
    b200nn_tensor *r = nullptr;
    TRY(tensor_alloc(ctx, oshape, false, &r));
    size_t off = 0;
    for (size_t i = 0; i < count; ++i) {
        const size_t w = tensors[i]->shape[dim] * inner * sizeof(float);
        if (w && outer) {
            cudaError_t e = cudaMemcpy2DAsync(r->data() + off * inner, total * inner * sizeof(float), tensors[i]->data(), w, w, outer,
                                              cudaMemcpyDeviceToDevice, ctx->stream);
            if (e != cudaSuccess) { delete r; return set_cuda_error(ctx, e, "tensor_concat"); }
        }
        off += tensors[i]->shape[dim];
    }
    *out = r;
    return B200NN_OK;
}

extern "C" int32_t b200nn_tensor_split(const b200nn_tensor *t, size_t dim, const size_t *sizes, size_t count, b200nn_tensor **outs) {
    if (!t || !sizes || !outs) return B200NN_ERR_ARG;
    b200nn_ctx *ctx = t->ctx;
    const size_t nd = t->shape.size();
    if (dim >= nd) return set_error(ctx, B200NN_ERR_DIM, "split: dim out of range");
    size_t total = 0;
    for (size_t i = 0; i < count; ++i) total += sizes[i];
    if (total != t->shape[dim])
        return set_error(ctx, B200NN_ERR_SHAPE, "split: sizes sum to " + std::to_string(total) + ", dimension holds " + std::to_string(t->shape[dim]));
    size_t outer, inner;
    outer_inner(t->shape, dim, &outer, &inner);
    size_t off = 0;
    for (size_t i = 0; i < count; ++i) outs[i] = nullptr;
    for (size_t i = 0; i < count; ++i) {
        std::vector<size_t> cshape(t->shape);
        cshape[dim] = sizes[i];
        b200nn_tensor *c = nullptr;
        int rc = tensor_alloc(ctx, cshape, false, &c);
        const size_t w = sizes[i] * inner * sizeof(float);
        if (rc == B200NN_OK && w && outer) {
            cudaError_t e = cudaMemcpy2DAsync(c->data(), w, t->data() + off * inner, t->shape[dim] * inner * sizeof(float), w, outer,
                                              cudaMemcpyDeviceToDevice, ctx->stream);
            if (e != cudaSuccess) rc = set_cuda_error(ctx, e, "tensor_split");
        }
        if (rc != B200NN_OK) {
            delete c;
            for (size_t j = 0; j < i; ++j) { delete outs[j]; outs[j] = nullptr; }
            return rc;
        }
        outs[i] = c;
        off += sizes[i];
    }
    return B200NN_OK;
}

extern "C" float *b200nn_tensor_data(b200nn_tensor *t) { return t ? t->data() : nullptr; }
extern "C" void b200nn_tensor_destroy(b200nn_tensor *t) { delete t; }

// ---------------------------------------------------------------------------------------------
// host quantiser wrappers
// ---------------------------------------------------------------------------------------------
extern "C" int32_t b200nn_quantize_weight_int4(const float *weight_t, size_t k, size_t n, size_t group,
                                               uint32_t *packed, float *scales) {
    if (!weight_t || !packed || !scales) return B200NN_ERR_ARG;
    return host_quantize_weight_int4(weight_t, k, n, group, packed, scales);
}
extern "C" int32_t b200nn_quantize_int4_per_group(const float *data, size_t len, size_t group, uint32_t *packed,
                                                  float *scales) {
    // quantize.rs:56-89
    if (!data || !packed || !scales || group == 0) return B200NN_ERR_ARG;
    if (len % 8 != 0) return B200NN_ERR_SHAPE;
    size_t n_groups = (len + group - 1) / group;
    memset(packed, 0, (len / 8) * 4);
    for (size_t g = 0; g < n_groups; ++g) {
        size_t s = g * group, e = std::min(len, s + group);
        float mx = 0.0f;
        for (size_t i = s; i < e; ++i) mx = std::max(mx, std::fabs(data[i]));
        float scale = mx < 1e-12f ? 1.0f : mx / 7.0f, inv = 1.0f / scale;
        scales[g] = scale;
        for (size_t i = s; i < e; ++i) {
            int q = (int)std::round(data[i] * inv);
            q = std::max(-8, std::min(7, q));
            packed[i / 8] |= ((uint32_t)(q + 8) & 0xFu) << ((i % 8) * 4);
        }
    }
    return B200NN_OK;
}
extern "C" int32_t b200nn_unpack_int4(uint32_t packed, int32_t index) { // quantize.rs:158-162
    return (int32_t)((packed >> ((index & 7) * 4)) & 0xFu) - 8;
}
extern "C" int32_t b200nn_pack_int8_to_u32(const int8_t *values, size_t n, uint32_t *packed) { // quantize.rs:23-32
    if (!values || !packed) return B200NN_ERR_ARG;
    memset(packed, 0, ((n + 3) / 4) * 4);
    for (size_t i = 0; i < n; ++i) packed[i / 4] |= ((uint32_t)(uint8_t)values[i]) << ((i % 4) * 8);
    return B200NN_OK;
}
extern "C" int32_t b200nn_quantize_int8_per_tensor(const float *data, size_t n, int8_t *q, float *scale) { // quantize.rs:5-18
    if (!data || !q || !scale) return B200NN_ERR_ARG;
    float mx = 0.0f;
    for (size_t i = 0; i < n; ++i) mx = std::max(mx, std::fabs(data[i]));
    float s = mx < 1e-12f ? 1.0f : mx / 127.0f, inv = 1.0f / s;
    for (size_t i = 0; i < n; ++i) q[i] = (int8_t)std::max(-128.0f, std::min(127.0f, std::round(data[i] * inv)));
    *scale = s;
    return B200NN_OK;
}
