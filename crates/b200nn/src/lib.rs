//! Safe layer over `b200nn_sys`: the reference's `gpu_host::nn` names for the GPT-2 inference path.
//! Every type owns one library handle and frees it on `Drop`; every method is one call into
//! `libb200nn` with the status mapped back to [`NnError`].  File:line citations are relative to the
//! reference repository (GH = crates/core/gpu-host/src).
//!
//! Not compiled on the machine this repository was developed on (no Rust toolchain there); it
//! follows `include/b200nn.hpp`, which is compiled and tested, method for method.

use std::ffi::CStr;
use std::ptr;
use std::sync::Arc;

use b200nn_sys as sys;

/// `NnError` (GH/nn/error.rs:7-29) plus the library's own kinds.
#[derive(Debug, Clone, PartialEq)]
pub enum NnError {
    ShapeMismatch(String),
    DimOutOfRange(String),
    KernelNotFound(String),
    Cuda(String),
    /// a kernel's bounded wait ran out; the context stays usable
    Device(String),
    Arg(String),
    /// `ModelError::Io` / `::SafeTensor` (GH/model.rs:30-62)
    Io(String),
    /// `ModelError::MissingTensor`
    MissingTensor(String),
}

impl std::fmt::Display for NnError {
    fn fmt(&self, f: &mut std::fmt::Formatter<'_>) -> std::fmt::Result {
        write!(f, "{:?}", self)
    }
}
impl std::error::Error for NnError {}

pub type Result<T> = std::result::Result<T, NnError>;

fn error_from(code: i32, message: String) -> NnError {
    match code {
        sys::B200NN_ERR_SHAPE => NnError::ShapeMismatch(message),
        sys::B200NN_ERR_DIM => NnError::DimOutOfRange(message),
        sys::B200NN_ERR_UNSUPPORTED => NnError::KernelNotFound(message),
        sys::B200NN_ERR_CUDA => NnError::Cuda(message),
        sys::B200NN_ERR_DEVICE => NnError::Device(message),
        sys::B200NN_ERR_IO => NnError::Io(message),
        sys::B200NN_ERR_MISSING => NnError::MissingTensor(message),
        _ => NnError::Arg(message),
    }
}

/// `KernelRegistry` (GH/nn/registry.rs:29-147): one per GPU, owns the library context.  The by-name
/// kernel lookups and launch-geometry helpers have no counterpart: kernels are linked into the library.
pub struct KernelRegistry {
    ctx: *mut sys::b200nn_ctx,
    device: i32,
}
// one context is used from one host thread at a time; moving it between threads is allowed
unsafe impl Send for KernelRegistry {}
unsafe impl Sync for KernelRegistry {}

impl KernelRegistry {
    /// `KernelRegistry::init_default` (registry.rs:131-135): device 0.
    pub fn init_default() -> Result<Arc<Self>> {
        Self::new(0)
    }
    pub fn new(device: i32) -> Result<Arc<Self>> {
        let mut ctx = ptr::null_mut();
        let rc = unsafe { sys::b200nn_ctx_create(device, &mut ctx) };
        if rc != sys::B200NN_OK {
            return Err(error_from(rc, format!("no context on CUDA device {device}")));
        }
        Ok(Arc::new(Self { ctx, device }))
    }
    pub fn device(&self) -> i32 {
        self.device
    }
    pub fn as_ptr(&self) -> *mut sys::b200nn_ctx {
        self.ctx
    }
    pub fn synchronize(&self) -> Result<()> {
        self.check(unsafe { sys::b200nn_ctx_synchronize(self.ctx) })
    }
    pub fn launch_count(&self) -> u64 {
        unsafe { sys::b200nn_ctx_launch_count(self.ctx) }
    }
    /// Reads and clears the device-side error word.
    pub fn device_error(&self) -> Result<u32> {
        let mut w = 0u32;
        self.check(unsafe { sys::b200nn_ctx_device_error(self.ctx, &mut w) })?;
        Ok(w)
    }
    /// Status -> `Result`, with the library's message for this context.
    pub fn check(&self, rc: i32) -> Result<()> {
        if rc == sys::B200NN_OK {
            return Ok(());
        }
        let p = unsafe { sys::b200nn_last_error_message(self.ctx) };
        let message = if p.is_null() { String::new() } else { unsafe { CStr::from_ptr(p) }.to_string_lossy().into_owned() };
        Err(error_from(rc, message))
    }
}

impl Drop for KernelRegistry {
    fn drop(&mut self) {
        unsafe { sys::b200nn_ctx_destroy(self.ctx) }
    }
}

/// `GpuTensor` (GH/nn/tensor.rs:45-393): f32, row-major, contiguous, on the registry's device.
pub struct GpuTensor {
    h: *mut sys::b200nn_tensor,
    registry: Arc<KernelRegistry>,
}

impl GpuTensor {
    fn wrap(registry: &Arc<KernelRegistry>, rc: i32, h: *mut sys::b200nn_tensor) -> Result<Self> {
        registry.check(rc)?;
        Ok(Self { h, registry: Arc::clone(registry) })
    }
    /// `from_host` (tensor.rs:83-110): `data.len()` must equal the product of `shape`.
    pub fn from_host(data: &[f32], shape: &[usize], registry: &Arc<KernelRegistry>) -> Result<Self> {
        let n: usize = shape.iter().product();
        if n != data.len() {
            return Err(NnError::ShapeMismatch(format!("expected {n} elements, got {}", data.len())));
        }
        let mut h = ptr::null_mut();
        let rc = unsafe { sys::b200nn_tensor_from_host(registry.ctx, data.as_ptr(), shape.as_ptr(), shape.len() as i32, &mut h) };
        Self::wrap(registry, rc, h)
    }
    /// `from_data` (tensor.rs:67-77): over f32 values already on the device; they are copied.
    ///
    /// # Safety
    /// `dev` must point to at least `shape.iter().product()` f32 values on the registry's device.
    pub unsafe fn from_data(dev: *const f32, shape: &[usize], registry: &Arc<KernelRegistry>) -> Result<Self> {
        let mut h = ptr::null_mut();
        let rc = sys::b200nn_tensor_from_device(registry.ctx, dev, shape.as_ptr(), shape.len() as i32, &mut h);
        Self::wrap(registry, rc, h)
    }
    pub fn zeros(shape: &[usize], registry: &Arc<KernelRegistry>) -> Result<Self> {
        let mut h = ptr::null_mut();
        let rc = unsafe { sys::b200nn_tensor_zeros(registry.ctx, shape.as_ptr(), shape.len() as i32, &mut h) };
        Self::wrap(registry, rc, h)
    }
    pub fn to_host(&self) -> Result<Vec<f32>> {
        let mut out = vec![0f32; self.numel()];
        self.registry.check(unsafe { sys::b200nn_tensor_to_host(self.h, out.as_mut_ptr(), out.len()) })?;
        Ok(out)
    }
    pub fn numel(&self) -> usize {
        unsafe { sys::b200nn_tensor_numel(self.h) }
    }
    pub fn ndim(&self) -> usize {
        unsafe { sys::b200nn_tensor_ndim(self.h) as usize }
    }
    pub fn shape(&self) -> Vec<usize> {
        let mut s = vec![0usize; self.ndim()];
        unsafe { sys::b200nn_tensor_shape(self.h, s.as_mut_ptr(), s.len() as i32) };
        s
    }
    pub fn strides(&self) -> Vec<usize> {
        let s = self.shape();
        let mut st = vec![0usize; s.len()];
        let mut acc = 1usize;
        for i in (0..s.len()).rev() {
            st[i] = acc;
            acc *= s[i];
        }
        st
    }
    pub fn is_contiguous(&self) -> bool {
        true
    }
    pub fn size_bytes(&self) -> usize {
        self.numel() * std::mem::size_of::<f32>()
    }
    /// Device pointer of the data.
    pub fn as_ptr(&self) -> *mut f32 {
        unsafe { sys::b200nn_tensor_data(self.h) }
    }
    pub fn handle(&self) -> *mut sys::b200nn_tensor {
        self.h
    }
    pub fn reshape(&self, shape: &[usize]) -> Result<Self> {
        let mut h = ptr::null_mut();
        let rc = unsafe { sys::b200nn_tensor_reshape(self.h, shape.as_ptr(), shape.len() as i32, &mut h) };
        Self::wrap(&self.registry, rc, h)
    }
    pub fn clone_tensor(&self) -> Result<Self> {
        let mut h = ptr::null_mut();
        let rc = unsafe { sys::b200nn_tensor_clone(self.h, &mut h) };
        Self::wrap(&self.registry, rc, h)
    }
    pub fn transpose(&self, dim0: usize, dim1: usize) -> Result<Self> {
        let mut h = ptr::null_mut();
        let rc = unsafe { sys::b200nn_tensor_transpose(self.h, dim0, dim1, &mut h) };
        Self::wrap(&self.registry, rc, h)
    }
    pub fn concat(tensors: &[&GpuTensor], dim: usize) -> Result<Self> {
        let first = tensors.first().ok_or_else(|| NnError::ShapeMismatch("concat of an empty list".into()))?;
        let hs: Vec<*const sys::b200nn_tensor> = tensors.iter().map(|t| t.h as *const _).collect();
        let mut h = ptr::null_mut();
        let rc = unsafe { sys::b200nn_tensor_concat(hs.as_ptr(), hs.len(), dim, &mut h) };
        Self::wrap(&first.registry, rc, h)
    }
    pub fn split(&self, dim: usize, sizes: &[usize]) -> Result<Vec<Self>> {
        let mut hs: Vec<*mut sys::b200nn_tensor> = vec![ptr::null_mut(); sizes.len()];
        self.registry.check(unsafe { sys::b200nn_tensor_split(self.h, dim, sizes.as_ptr(), sizes.len(), hs.as_mut_ptr()) })?;
        Ok(hs.into_iter().map(|h| Self { h, registry: Arc::clone(&self.registry) }).collect())
    }
}

impl Drop for GpuTensor {
    fn drop(&mut self) {
        unsafe { sys::b200nn_tensor_destroy(self.h) }
    }
}

/// `Activation` (GH/nn/layers/linear.rs:24-33).
#[derive(Clone, Copy, Debug, PartialEq, Eq)]
pub enum Activation {
    Gelu,
    Relu,
    Silu,
    Sigmoid,
}
impl Activation {
    fn code(self) -> i32 {
        match self {
            Activation::Gelu => sys::B200NN_ACT_GELU_TANH,
            Activation::Relu => sys::B200NN_ACT_RELU,
            Activation::Silu => sys::B200NN_ACT_SILU,
            Activation::Sigmoid => sys::B200NN_ACT_SIGMOID,
        }
    }
}

/// `FusedActivation` (GH/nn/ops/gemm.rs:803-808); its GELU is `x * sigmoid(1.702 x)`.
#[derive(Clone, Copy, Debug, PartialEq, Eq)]
pub enum FusedActivation {
    Gelu,
    Relu,
}
impl FusedActivation {
    fn code(self) -> i32 {
        match self {
            FusedActivation::Gelu => sys::B200NN_ACT_GELU_SIGMOID,
            FusedActivation::Relu => sys::B200NN_ACT_RELU,
        }
    }
}

/// Stateless ops (GH/nn/ops/mod.rs:19-37); each takes the registry last, as there.
pub mod ops {
    use super::*;

    fn activation(x: &GpuTensor, act: i32, registry: &Arc<KernelRegistry>) -> Result<GpuTensor> {
        let mut h = ptr::null_mut();
        let rc = unsafe { sys::b200nn_activation(registry.as_ptr(), x.handle(), act, &mut h) };
        GpuTensor::wrap(registry, rc, h)
    }
    /// `ops::layer_norm` (ops/norm.rs:14-81)
    pub fn layer_norm(x: &GpuTensor, gamma: &GpuTensor, beta: &GpuTensor, eps: f32, registry: &Arc<KernelRegistry>) -> Result<GpuTensor> {
        let mut h = ptr::null_mut();
        let rc = unsafe { sys::b200nn_layer_norm(registry.as_ptr(), x.handle(), gamma.handle(), beta.handle(), eps, &mut h) };
        GpuTensor::wrap(registry, rc, h)
    }
    /// `ops::layer_norm_residual_dual` (ops/norm.rs:248-400): `(a + b, LayerNorm(a + b))`
    pub fn layer_norm_residual_dual(
        a: &GpuTensor,
        b: &GpuTensor,
        gamma: &GpuTensor,
        beta: &GpuTensor,
        eps: f32,
        registry: &Arc<KernelRegistry>,
    ) -> Result<(GpuTensor, GpuTensor)> {
        let (mut s, mut n) = (ptr::null_mut(), ptr::null_mut());
        let rc = unsafe {
            sys::b200nn_layer_norm_residual_dual(registry.as_ptr(), a.handle(), b.handle(), gamma.handle(), beta.handle(), eps, &mut s, &mut n)
        };
        registry.check(rc)?;
        Ok((GpuTensor { h: s, registry: Arc::clone(registry) }, GpuTensor { h: n, registry: Arc::clone(registry) }))
    }
    /// `ops::layer_norm_residual` (ops/norm.rs:88-246): `LayerNorm(x + residual)`
    pub fn layer_norm_residual(
        x: &GpuTensor,
        residual: &GpuTensor,
        gamma: &GpuTensor,
        beta: &GpuTensor,
        eps: f32,
        registry: &Arc<KernelRegistry>,
    ) -> Result<GpuTensor> {
        Ok(layer_norm_residual_dual(x, residual, gamma, beta, eps, registry)?.1)
    }
    /// `ops::gelu` (ops/activation.rs:14-16): the sigmoid form `x * sigmoid(1.702 x)` of `gelu_forward_v2`
    /// when `sigmoid_form`, else the tanh form of the CPU reference.
    pub fn gelu(x: &GpuTensor, sigmoid_form: bool, registry: &Arc<KernelRegistry>) -> Result<GpuTensor> {
        activation(x, if sigmoid_form { sys::B200NN_ACT_GELU_SIGMOID } else { sys::B200NN_ACT_GELU_TANH }, registry)
    }
    pub fn silu(x: &GpuTensor, registry: &Arc<KernelRegistry>) -> Result<GpuTensor> {
        activation(x, sys::B200NN_ACT_SILU, registry)
    }
    pub fn sigmoid(x: &GpuTensor, registry: &Arc<KernelRegistry>) -> Result<GpuTensor> {
        activation(x, sys::B200NN_ACT_SIGMOID, registry)
    }
    pub fn relu(x: &GpuTensor, registry: &Arc<KernelRegistry>) -> Result<GpuTensor> {
        activation(x, sys::B200NN_ACT_RELU, registry)
    }
    /// `ops::bias_add` (ops/reshape.rs:112-156): in place
    pub fn bias_add(data: &mut GpuTensor, bias: &GpuTensor, registry: &Arc<KernelRegistry>) -> Result<()> {
        registry.check(unsafe { sys::b200nn_bias_add(registry.as_ptr(), data.handle(), bias.handle()) })
    }
    /// `ops::elementwise_add` (ops/reshape.rs:166-186): `a += b`
    pub fn elementwise_add(a: &mut GpuTensor, b: &GpuTensor, registry: &Arc<KernelRegistry>) -> Result<()> {
        registry.check(unsafe { sys::b200nn_elementwise_add(registry.as_ptr(), a.handle(), b.handle()) })
    }
    /// `ops::elementwise_add_out` (ops/reshape.rs:219-290)
    pub fn elementwise_add_out(a: &GpuTensor, b: &GpuTensor, registry: &Arc<KernelRegistry>) -> Result<GpuTensor> {
        if a.numel() != b.numel() {
            return Err(NnError::ShapeMismatch(format!("expected same numel, a has {}, b has {}", a.numel(), b.numel())));
        }
        let mut out = a.clone_tensor()?;
        elementwise_add(&mut out, b, registry)?;
        Ok(out)
    }
    /// `ops::matmul` (ops/gemm.rs:20-212): `[M,K] x [K,N]`; `matmul_v2` / `_v4` / `_v4_1` are the same contract.
    pub fn matmul(a: &GpuTensor, b: &GpuTensor, registry: &Arc<KernelRegistry>) -> Result<GpuTensor> {
        let mut h = ptr::null_mut();
        let rc = unsafe { sys::b200nn_matmul(registry.as_ptr(), a.handle(), b.handle(), &mut h) };
        GpuTensor::wrap(registry, rc, h)
    }
    pub use self::matmul as matmul_v2;
    pub use self::matmul as matmul_v4;
    pub use self::matmul as matmul_v4_1;
    /// `ops::matmul_fused` (ops/gemm.rs:814-977): `activation(a x b + bias)`
    pub fn matmul_fused(
        a: &GpuTensor,
        b: &GpuTensor,
        bias: &GpuTensor,
        act: FusedActivation,
        registry: &Arc<KernelRegistry>,
    ) -> Result<GpuTensor> {
        if a.ndim() != 2 || b.ndim() != 2 {
            return Err(NnError::ShapeMismatch(format!("expected 2D tensors, actual a.ndim={}, b.ndim={}", a.ndim(), b.ndim())));
        }
        let (ash, bsh) = (a.shape(), b.shape());
        if ash[1] != bsh[0] {
            return Err(NnError::ShapeMismatch(format!("expected a.shape[1]={} == b.shape[0], actual b.shape[0]={}", ash[1], bsh[0])));
        }
        if bias.ndim() != 1 || bias.shape()[0] != bsh[1] {
            return Err(NnError::ShapeMismatch(format!("expected bias.shape=[{}], actual bias.shape={:?}", bsh[1], bias.shape())));
        }
        let mut y = matmul(a, b, registry)?;
        bias_add(&mut y, bias, registry)?;
        activation(&y, act.code(), registry)
    }
    /// `ops::int4_matmul` (ops/gemm.rs:1186-1266): quantise `b` `[K,N]` (host) per group, then `a [M,K] x dequant(b)`
    pub fn int4_matmul(a: &GpuTensor, b_host: &[f32], k: usize, n: usize, group: usize, registry: &Arc<KernelRegistry>) -> Result<GpuTensor> {
        if b_host.len() != k * n {
            return Err(NnError::ShapeMismatch(format!("expected {} values in b, got {}", k * n, b_host.len())));
        }
        let mut h = ptr::null_mut();
        let rc = unsafe { sys::b200nn_int4_matmul(registry.as_ptr(), a.handle(), b_host.as_ptr(), k, n, group, &mut h) };
        GpuTensor::wrap(registry, rc, h)
    }
    /// `ops::scaled_dot_product_attention_kv` (ops/attention.rs:557-606): one head, `q [q_len,64]` against `k, v [kv_len,64]`
    pub fn scaled_dot_product_attention_kv(
        q: &GpuTensor,
        k: &GpuTensor,
        v: &GpuTensor,
        causal: bool,
        q_offset: usize,
        registry: &Arc<KernelRegistry>,
    ) -> Result<GpuTensor> {
        let mut h = ptr::null_mut();
        let rc = unsafe { sys::b200nn_attention_kv(registry.as_ptr(), q.handle(), k.handle(), v.handle(), causal as i32, q_offset, &mut h) };
        GpuTensor::wrap(registry, rc, h)
    }
    /// `ops::scaled_dot_product_attention` (ops/attention.rs:17-103)
    pub fn scaled_dot_product_attention(q: &GpuTensor, k: &GpuTensor, v: &GpuTensor, causal: bool, registry: &Arc<KernelRegistry>) -> Result<GpuTensor> {
        scaled_dot_product_attention_kv(q, k, v, causal, 0, registry)
    }
    /// `ops::quantize_weight_int4` (ops/quantize.rs:102-153): `weight_t [K,N]` -> `(packed [K/8,N], scales [ceil(K/group),N])`
    pub fn quantize_weight_int4(weight_t: &[f32], k: usize, n: usize, group: usize) -> Result<(Vec<u32>, Vec<f32>)> {
        if weight_t.len() != k * n || group == 0 {
            return Err(NnError::ShapeMismatch("weight_t must hold k*n values and group be non-zero".into()));
        }
        let mut packed = vec![0u32; k / 8 * n];
        let mut scales = vec![0f32; (k + group - 1) / group * n];
        let rc = unsafe { sys::b200nn_quantize_weight_int4(weight_t.as_ptr(), k, n, group, packed.as_mut_ptr(), scales.as_mut_ptr()) };
        if rc != sys::B200NN_OK {
            return Err(error_from(rc, "quantize_weight_int4: k must be a multiple of 8".into()));
        }
        Ok((packed, scales))
    }
    /// `ops::unpack_int4` (ops/quantize.rs:158-162): nibble `index` of a word as a value in [-8, 7]
    pub fn unpack_int4(packed: u32, index: usize) -> i32 {
        unsafe { sys::b200nn_unpack_int4(packed, index as i32) }
    }
}

fn opt_ptr(v: Option<&[f32]>) -> *const f32 {
    v.map_or(ptr::null(), |s| s.as_ptr())
}

/// `Linear` (GH/nn/layers/linear.rs:58-313): weight `[out,in]` row-major, optional bias `[out]`.
pub struct Linear {
    h: *mut sys::b200nn_linear,
    registry: Arc<KernelRegistry>,
}
impl Linear {
    pub fn new(weight: &[f32], bias: Option<&[f32]>, in_features: usize, out_features: usize, registry: &Arc<KernelRegistry>) -> Result<Self> {
        if weight.len() != in_features * out_features {
            return Err(NnError::ShapeMismatch(format!("weight: expected {out_features}x{in_features}, got {} elements", weight.len())));
        }
        if bias.map_or(false, |b| b.len() != out_features) {
            return Err(NnError::ShapeMismatch(format!("bias: expected {out_features}")));
        }
        let mut h = ptr::null_mut();
        registry.check(unsafe { sys::b200nn_linear_create(registry.as_ptr(), weight.as_ptr(), opt_ptr(bias), in_features, out_features, &mut h) })?;
        Ok(Self { h, registry: Arc::clone(registry) })
    }
    pub fn forward(&self, x: &GpuTensor) -> Result<GpuTensor> {
        let mut y = ptr::null_mut();
        let rc = unsafe { sys::b200nn_linear_forward(self.h, x.handle(), &mut y) };
        GpuTensor::wrap(&self.registry, rc, y)
    }
    /// `forward_fused` (linear.rs:131-166)
    pub fn forward_fused(&self, x: &GpuTensor, activation: FusedActivation) -> Result<GpuTensor> {
        let mut y = ptr::null_mut();
        let rc = unsafe { sys::b200nn_linear_forward_fused(self.h, x.handle(), activation.code(), &mut y) };
        GpuTensor::wrap(&self.registry, rc, y)
    }
    /// `forward_auto_fused` (linear.rs:184-278); no run-time code generator is needed, the epilogues are in the library
    pub fn forward_auto_fused(&self, x: &GpuTensor, activation: Activation) -> Result<GpuTensor> {
        let mut y = ptr::null_mut();
        let rc = unsafe { sys::b200nn_linear_forward_fused(self.h, x.handle(), activation.code(), &mut y) };
        GpuTensor::wrap(&self.registry, rc, y)
    }
}
impl Drop for Linear {
    fn drop(&mut self) {
        unsafe { sys::b200nn_linear_destroy(self.h) }
    }
}

/// `Int4Linear` (GH/nn/layers/int4_linear.rs:24-147): packed `[K/8,N]` u32, scales `[ceil(K/group),N]` f32.
pub struct Int4Linear {
    h: *mut sys::b200nn_int4_linear,
    registry: Arc<KernelRegistry>,
}
impl Int4Linear {
    pub fn new(
        packed: &[u32],
        scales: &[f32],
        bias: Option<&[f32]>,
        in_features: usize,
        out_features: usize,
        group_size: usize,
        registry: &Arc<KernelRegistry>,
    ) -> Result<Self> {
        let groups = if group_size == 0 { 0 } else { (in_features + group_size - 1) / group_size };
        if in_features % 8 != 0 || packed.len() != in_features / 8 * out_features || scales.len() != groups * out_features {
            return Err(NnError::ShapeMismatch("packed must be [K/8,N] and scales [ceil(K/group),N] with K%8==0".into()));
        }
        if bias.map_or(false, |b| b.len() != out_features) {
            return Err(NnError::ShapeMismatch(format!("bias: expected {out_features}")));
        }
        let mut h = ptr::null_mut();
        registry.check(unsafe {
            sys::b200nn_int4_linear_create(registry.as_ptr(), packed.as_ptr(), scales.as_ptr(), opt_ptr(bias), in_features, out_features, group_size, &mut h)
        })?;
        Ok(Self { h, registry: Arc::clone(registry) })
    }
    pub fn forward(&self, x: &GpuTensor) -> Result<GpuTensor> {
        let mut y = ptr::null_mut();
        let rc = unsafe { sys::b200nn_int4_linear_forward(self.h, x.handle(), &mut y) };
        GpuTensor::wrap(&self.registry, rc, y)
    }
    pub fn memory_bytes(&self) -> usize {
        unsafe { sys::b200nn_int4_linear_memory_bytes(self.h) }
    }
}
impl Drop for Int4Linear {
    fn drop(&mut self) {
        unsafe { sys::b200nn_int4_linear_destroy(self.h) }
    }
}

/// `LayerNorm` (GH/nn/layers/norm.rs:24-55)
pub struct LayerNorm {
    h: *mut sys::b200nn_layernorm,
    gamma: Vec<f32>,
    beta: Vec<f32>,
    registry: Arc<KernelRegistry>,
}
impl LayerNorm {
    pub fn new(gamma: &[f32], beta: &[f32], eps: f32, registry: &Arc<KernelRegistry>) -> Result<Self> {
        if gamma.len() != beta.len() || gamma.is_empty() {
            return Err(NnError::ShapeMismatch("gamma and beta must have the same non-zero length".into()));
        }
        let mut h = ptr::null_mut();
        registry.check(unsafe { sys::b200nn_layernorm_create(registry.as_ptr(), gamma.as_ptr(), beta.as_ptr(), gamma.len(), eps, &mut h) })?;
        Ok(Self { h, gamma: gamma.to_vec(), beta: beta.to_vec(), registry: Arc::clone(registry) })
    }
    pub fn forward(&self, x: &GpuTensor) -> Result<GpuTensor> {
        let mut y = ptr::null_mut();
        let rc = unsafe { sys::b200nn_layernorm_forward(self.h, x.handle(), &mut y) };
        GpuTensor::wrap(&self.registry, rc, y)
    }
    /// `gamma` / `beta` (norm.rs:41-48) as device tensors
    pub fn gamma(&self) -> Result<GpuTensor> {
        GpuTensor::from_host(&self.gamma, &[self.gamma.len()], &self.registry)
    }
    pub fn beta(&self) -> Result<GpuTensor> {
        GpuTensor::from_host(&self.beta, &[self.beta.len()], &self.registry)
    }
}
impl Drop for LayerNorm {
    fn drop(&mut self) {
        unsafe { sys::b200nn_layernorm_destroy(self.h) }
    }
}

/// `Embedding` (GH/nn/layers/embedding.rs:25-93)
pub struct Embedding {
    h: *mut sys::b200nn_embedding,
    registry: Arc<KernelRegistry>,
}
impl Embedding {
    pub fn new(wte: &[f32], wpe: &[f32], vocab_size: usize, max_seq_len: usize, d_model: usize, registry: &Arc<KernelRegistry>) -> Result<Self> {
        if wte.len() != vocab_size * d_model || wpe.len() != max_seq_len * d_model {
            return Err(NnError::ShapeMismatch("wte must be [vocab,d] and wpe [max_seq,d]".into()));
        }
        let mut h = ptr::null_mut();
        registry.check(unsafe { sys::b200nn_embedding_create(registry.as_ptr(), wte.as_ptr(), wpe.as_ptr(), vocab_size, max_seq_len, d_model, &mut h) })?;
        Ok(Self { h, registry: Arc::clone(registry) })
    }
    pub fn forward_tokens(&self, token_ids: &[u32]) -> Result<GpuTensor> {
        self.forward_tokens_with_offset(token_ids, 0)
    }
    pub fn forward_tokens_with_offset(&self, token_ids: &[u32], pos_offset: usize) -> Result<GpuTensor> {
        let mut y = ptr::null_mut();
        let rc = unsafe { sys::b200nn_embedding_forward_tokens(self.h, token_ids.as_ptr(), token_ids.len(), pos_offset, &mut y) };
        GpuTensor::wrap(&self.registry, rc, y)
    }
}
impl Drop for Embedding {
    fn drop(&mut self) {
        unsafe { sys::b200nn_embedding_destroy(self.h) }
    }
}

/// `MultiHeadAttention` (GH/nn/layers/attention.rs:30-184); `new_int4` is `Int4MultiHeadAttention::new`
/// (GH/nn/models/gpt2.rs:1141-1188).  `qkv_weight [3d,d]`, `out_weight [d,d]` in Linear layout.
pub struct MultiHeadAttention {
    h: *mut sys::b200nn_attention,
    n_heads: usize,
    d_head: usize,
    registry: Arc<KernelRegistry>,
}
impl MultiHeadAttention {
    fn check_sizes(qkv_weight: &[f32], qkv_bias: &[f32], out_weight: &[f32], out_bias: &[f32], n_embd: usize, n_heads: usize) -> Result<()> {
        if n_heads == 0 || qkv_weight.len() != 3 * n_embd * n_embd || qkv_bias.len() != 3 * n_embd || out_weight.len() != n_embd * n_embd || out_bias.len() != n_embd {
            return Err(NnError::ShapeMismatch("attention weights do not match n_embd".into()));
        }
        Ok(())
    }
    pub fn new(
        qkv_weight: &[f32],
        qkv_bias: &[f32],
        out_weight: &[f32],
        out_bias: &[f32],
        n_embd: usize,
        n_heads: usize,
        registry: &Arc<KernelRegistry>,
    ) -> Result<Self> {
        Self::check_sizes(qkv_weight, qkv_bias, out_weight, out_bias, n_embd, n_heads)?;
        let mut h = ptr::null_mut();
        registry.check(unsafe {
            sys::b200nn_attention_create(registry.as_ptr(), qkv_weight.as_ptr(), qkv_bias.as_ptr(), out_weight.as_ptr(), out_bias.as_ptr(), n_embd, n_heads, &mut h)
        })?;
        Ok(Self { h, n_heads, d_head: n_embd / n_heads, registry: Arc::clone(registry) })
    }
    #[allow(clippy::too_many_arguments)]
    pub fn new_int4(
        qkv_weight: &[f32],
        qkv_bias: &[f32],
        out_weight: &[f32],
        out_bias: &[f32],
        n_embd: usize,
        n_heads: usize,
        group_size: usize,
        registry: &Arc<KernelRegistry>,
    ) -> Result<Self> {
        Self::check_sizes(qkv_weight, qkv_bias, out_weight, out_bias, n_embd, n_heads)?;
        let mut h = ptr::null_mut();
        registry.check(unsafe {
            sys::b200nn_int4_attention_create(
                registry.as_ptr(), qkv_weight.as_ptr(), qkv_bias.as_ptr(), out_weight.as_ptr(), out_bias.as_ptr(), n_embd, n_heads, group_size, &mut h,
            )
        })?;
        Ok(Self { h, n_heads, d_head: n_embd / n_heads, registry: Arc::clone(registry) })
    }
    pub fn n_heads(&self) -> usize {
        self.n_heads
    }
    pub fn d_head(&self) -> usize {
        self.d_head
    }
    pub fn forward_causal(&self, x: &GpuTensor) -> Result<GpuTensor> {
        let mut y = ptr::null_mut();
        let rc = unsafe { sys::b200nn_attention_forward_causal(self.h, x.handle(), &mut y) };
        GpuTensor::wrap(&self.registry, rc, y)
    }
    /// `forward_cached` (attention.rs:133-178): `cached_k` / `cached_v` are `[n_heads][kv_len*d_head]`;
    /// returns the output and the new K and V rows `[n_heads][new_len*d_head]`.
    pub fn forward_cached(&self, x: &GpuTensor, cached_k: &[f32], cached_v: &[f32], kv_len: usize) -> Result<(GpuTensor, Vec<f32>, Vec<f32>)> {
        if cached_k.len() != self.n_heads * kv_len * self.d_head || cached_v.len() != cached_k.len() {
            return Err(NnError::ShapeMismatch("cached K/V must be [n_heads][kv_len*d_head]".into()));
        }
        let new_len = x.shape()[0];
        let mut nk = vec![0f32; self.n_heads * new_len * self.d_head];
        let mut nv = vec![0f32; nk.len()];
        let (pk, pv) = if kv_len == 0 { (ptr::null(), ptr::null()) } else { (cached_k.as_ptr(), cached_v.as_ptr()) };
        let mut y = ptr::null_mut();
        let rc = unsafe { sys::b200nn_attention_forward_cached(self.h, x.handle(), pk, pv, kv_len, &mut y, nk.as_mut_ptr(), nv.as_mut_ptr()) };
        Ok((GpuTensor::wrap(&self.registry, rc, y)?, nk, nv))
    }
}
impl Drop for MultiHeadAttention {
    fn drop(&mut self) {
        unsafe { sys::b200nn_attention_destroy(self.h) }
    }
}

/// `Gpt2Config` (GH/nn/models/gpt2.rs:20-93)
#[derive(Clone, Copy, Debug, PartialEq)]
pub struct Gpt2Config {
    pub n_layer: usize,
    pub n_embd: usize,
    pub n_head: usize,
    pub vocab_size: usize,
    pub n_positions: usize,
    pub layer_norm_epsilon: f32,
}
impl Gpt2Config {
    fn preset(name: &'static [u8]) -> Self {
        let mut c = sys::b200nn_gpt2_config { n_layer: 0, n_embd: 0, n_head: 0, vocab_size: 0, n_positions: 0, layer_norm_epsilon: 0.0 };
        // the four names below are the ones the library knows, so the call cannot fail
        unsafe { sys::b200nn_gpt2_config_preset(name.as_ptr() as *const std::ffi::c_char, &mut c) };
        Self::from_c(&c)
    }
    pub fn small() -> Self {
        Self::preset(b"small\0")
    }
    pub fn medium() -> Self {
        Self::preset(b"medium\0")
    }
    pub fn large() -> Self {
        Self::preset(b"large\0")
    }
    pub fn xl() -> Self {
        Self::preset(b"xl\0")
    }
    pub fn head_dim(&self) -> usize {
        self.n_embd / self.n_head
    }
    pub fn ffn_dim(&self) -> usize {
        4 * self.n_embd
    }
    fn to_c(self) -> sys::b200nn_gpt2_config {
        sys::b200nn_gpt2_config {
            n_layer: self.n_layer as i32,
            n_embd: self.n_embd as i32,
            n_head: self.n_head as i32,
            vocab_size: self.vocab_size as i32,
            n_positions: self.n_positions as i32,
            layer_norm_epsilon: self.layer_norm_epsilon,
        }
    }
    fn from_c(c: &sys::b200nn_gpt2_config) -> Self {
        Self {
            n_layer: c.n_layer as usize,
            n_embd: c.n_embd as usize,
            n_head: c.n_head as usize,
            vocab_size: c.vocab_size as usize,
            n_positions: c.n_positions as usize,
            layer_norm_epsilon: c.layer_norm_epsilon,
        }
    }
}

/// `TransformerLayerWeights` / `Gpt2Weights` (GH/model.rs:112-154): host f32, dense weights in the
/// checkpoint's Conv1D layout `[in,out]`.
#[derive(Clone, Debug, Default)]
pub struct TransformerLayerWeights {
    pub ln_1_weight: Vec<f32>,
    pub ln_1_bias: Vec<f32>,
    pub c_attn_weight: Vec<f32>,
    pub c_attn_bias: Vec<f32>,
    pub c_proj_weight: Vec<f32>,
    pub c_proj_bias: Vec<f32>,
    pub ln_2_weight: Vec<f32>,
    pub ln_2_bias: Vec<f32>,
    pub mlp_fc_weight: Vec<f32>,
    pub mlp_fc_bias: Vec<f32>,
    pub mlp_proj_weight: Vec<f32>,
    pub mlp_proj_bias: Vec<f32>,
}
#[derive(Clone, Debug, Default)]
pub struct Gpt2Weights {
    pub wte: Vec<f32>,
    pub wpe: Vec<f32>,
    pub ln_f_weight: Vec<f32>,
    pub ln_f_bias: Vec<f32>,
    pub layers: Vec<TransformerLayerWeights>,
}

/// `SimpleRng` (gpt2.rs:1000-1023): xorshift64
pub struct SimpleRng {
    state: u64,
}
impl SimpleRng {
    pub fn new(seed: u64) -> Self {
        Self { state: unsafe { sys::b200nn_simple_rng_new(seed) } }
    }
    pub fn next_f32(&mut self) -> f32 {
        unsafe { sys::b200nn_simple_rng_next_f32(&mut self.state) }
    }
}

/// `top_k_sample` (gpt2.rs:1029-1058)
pub fn top_k_sample(logits: &[f32], k: usize, temperature: f32, rng: &mut SimpleRng) -> u32 {
    let mut token = 0u32;
    // fails only for empty logits or k = 0, where the reference would index out of bounds
    unsafe { sys::b200nn_top_k_sample(logits.as_ptr(), logits.len(), k, temperature, &mut rng.state, &mut token) };
    token
}

/// `Gpt2Model` (gpt2.rs:293-977).  [`Int4Gpt2Model`] (gpt2.rs:1343-1576) is the same handle created
/// through `b200nn_int4_gpt2_create`.
pub struct Gpt2Model {
    h: *mut sys::b200nn_gpt2,
    config: Gpt2Config,
    group_size: usize,
    registry: Arc<KernelRegistry>,
}

fn create_model(w: &Gpt2Weights, config: &Gpt2Config, group_size: usize, flags: u32, registry: &Arc<KernelRegistry>) -> Result<Gpt2Model> {
    if w.layers.len() != config.n_layer {
        return Err(NnError::ShapeMismatch(format!("weights hold {} layers, config says {}", w.layers.len(), config.n_layer)));
    }
    let layers: Vec<sys::b200nn_gpt2_layer_weights> = w
        .layers
        .iter()
        .map(|l| sys::b200nn_gpt2_layer_weights {
            ln_1_weight: l.ln_1_weight.as_ptr(),
            ln_1_bias: l.ln_1_bias.as_ptr(),
            c_attn_weight: l.c_attn_weight.as_ptr(),
            c_attn_bias: l.c_attn_bias.as_ptr(),
            c_proj_weight: l.c_proj_weight.as_ptr(),
            c_proj_bias: l.c_proj_bias.as_ptr(),
            ln_2_weight: l.ln_2_weight.as_ptr(),
            ln_2_bias: l.ln_2_bias.as_ptr(),
            mlp_fc_weight: l.mlp_fc_weight.as_ptr(),
            mlp_fc_bias: l.mlp_fc_bias.as_ptr(),
            mlp_proj_weight: l.mlp_proj_weight.as_ptr(),
            mlp_proj_bias: l.mlp_proj_bias.as_ptr(),
        })
        .collect();
    let cw = sys::b200nn_gpt2_weights {
        wte: w.wte.as_ptr(),
        wpe: w.wpe.as_ptr(),
        ln_f_weight: w.ln_f_weight.as_ptr(),
        ln_f_bias: w.ln_f_bias.as_ptr(),
        layers: layers.as_ptr(),
    };
    let cc = config.to_c();
    let mut h = ptr::null_mut();
    let rc = unsafe {
        if group_size == 0 {
            sys::b200nn_gpt2_create(registry.as_ptr(), &cc, &cw, flags, &mut h)
        } else {
            sys::b200nn_int4_gpt2_create(registry.as_ptr(), &cc, &cw, group_size, flags, &mut h)
        }
    };
    registry.check(rc)?;
    Ok(Gpt2Model { h, config: *config, group_size, registry: Arc::clone(registry) })
}

impl Gpt2Model {
    /// `Gpt2Model::from_weights` (gpt2.rs:337-404)
    pub fn from_weights(weights: &Gpt2Weights, config: &Gpt2Config, registry: &Arc<KernelRegistry>) -> Result<Self> {
        create_model(weights, config, 0, 0, registry)
    }
    pub fn config(&self) -> &Gpt2Config {
        &self.config
    }
    /// `forward` (gpt2.rs:481-499): logits `[seq_len, vocab]` of one sequence
    pub fn forward(&self, token_ids: &[u32]) -> Result<GpuTensor> {
        let mut y = ptr::null_mut();
        let rc = unsafe { sys::b200nn_gpt2_forward(self.h, token_ids.as_ptr(), token_ids.len(), &mut y) };
        GpuTensor::wrap(&self.registry, rc, y)
    }
    /// `forward_auto_fused` (gpt2.rs:505-523): the fused epilogues are always on
    pub fn forward_auto_fused(&self, token_ids: &[u32]) -> Result<GpuTensor> {
        self.forward(token_ids)
    }
    /// `forward_features` (gpt2.rs:570-581)
    pub fn forward_features(&self, token_ids: &[u32]) -> Result<GpuTensor> {
        let mut y = ptr::null_mut();
        let rc = unsafe { sys::b200nn_gpt2_forward_features(self.h, token_ids.as_ptr(), token_ids.len(), &mut y) };
        GpuTensor::wrap(&self.registry, rc, y)
    }
    /// `forward_cached` (gpt2.rs:712-734): `token_ids` is `[batch,new_len]` for the cache's batch
    pub fn forward_cached(&self, token_ids: &[u32], new_len: usize, cache: &mut KvCache) -> Result<GpuTensor> {
        let mut y = ptr::null_mut();
        let rc = unsafe { sys::b200nn_gpt2_forward_cached(self.h, token_ids.as_ptr(), new_len, cache.h, &mut y) };
        GpuTensor::wrap(&self.registry, rc, y)
    }
    fn run_generate(
        &self,
        f: unsafe extern "C" fn(*mut sys::b200nn_gpt2, *const u32, usize, usize, u32, *mut u32, *mut usize) -> i32,
        prompt: &[u32],
        max_new_tokens: usize,
    ) -> Result<Vec<u32>> {
        let mut out = vec![0u32; prompt.len() + max_new_tokens];
        let mut n = 0usize;
        self.registry.check(unsafe { f(self.h, prompt.as_ptr(), prompt.len(), max_new_tokens, sys::B200NN_STOP_ON_EOS, out.as_mut_ptr(), &mut n) })?;
        out.truncate(n);
        Ok(out)
    }
    /// `generate` (gpt2.rs:672-706): greedy; prompt followed by the new tokens; stops before appending 50256
    pub fn generate(&self, prompt_tokens: &[u32], max_new_tokens: usize) -> Result<Vec<u32>> {
        self.run_generate(sys::b200nn_gpt2_generate, prompt_tokens, max_new_tokens)
    }
    /// `generate_cached` (gpt2.rs:740-783)
    pub fn generate_cached(&self, prompt_tokens: &[u32], max_new_tokens: usize) -> Result<Vec<u32>> {
        self.run_generate(sys::b200nn_gpt2_generate_cached, prompt_tokens, max_new_tokens)
    }
    /// Batched greedy decoding (an added axis): `prompts [batch,prompt_len]` -> `(tokens [batch,prompt_len+max_new], lengths)`
    pub fn generate_batch(&self, prompts: &[u32], batch: usize, prompt_len: usize, max_new_tokens: usize) -> Result<(Vec<u32>, Vec<usize>)> {
        if prompts.len() != batch * prompt_len {
            return Err(NnError::ShapeMismatch("prompts must be [batch,prompt_len]".into()));
        }
        let mut out = vec![0u32; batch * (prompt_len + max_new_tokens)];
        let mut lens = vec![0usize; batch];
        self.registry.check(unsafe {
            sys::b200nn_gpt2_generate_batch(self.h, prompts.as_ptr(), batch, prompt_len, max_new_tokens, 0, out.as_mut_ptr(), lens.as_mut_ptr())
        })?;
        Ok((out, lens))
    }
    /// `generate_cached_sampling` (gpt2.rs:933-977)
    pub fn generate_cached_sampling(
        &self,
        prompt_tokens: &[u32],
        max_new_tokens: usize,
        top_k: usize,
        temperature: f32,
        rng: &mut SimpleRng,
    ) -> Result<Vec<u32>> {
        let mut out = vec![0u32; prompt_tokens.len() + max_new_tokens];
        let mut n = 0usize;
        self.registry.check(unsafe {
            sys::b200nn_gpt2_generate_cached_sampling(
                self.h, prompt_tokens.as_ptr(), prompt_tokens.len(), max_new_tokens, top_k, temperature, &mut rng.state, out.as_mut_ptr(), &mut n,
            )
        })?;
        out.truncate(n);
        Ok(out)
    }
    /// `forward_early_exit` (gpt2.rs:797-830) -> `(logits, blocks run)`
    pub fn forward_early_exit(&self, token_ids: &[u32], threshold: f32) -> Result<(GpuTensor, usize)> {
        let mut y = ptr::null_mut();
        let mut used = 0i32;
        let rc = unsafe { sys::b200nn_gpt2_forward_early_exit(self.h, token_ids.as_ptr(), token_ids.len(), threshold, &mut y, &mut used) };
        Ok((GpuTensor::wrap(&self.registry, rc, y)?, used as usize))
    }
}
impl Drop for Gpt2Model {
    fn drop(&mut self) {
        unsafe { sys::b200nn_gpt2_destroy(self.h) }
    }
}

/// `Int4Gpt2Model` (gpt2.rs:1343-1576): every block Linear quantised per group at construction.
pub struct Int4Gpt2Model(Gpt2Model);
impl Int4Gpt2Model {
    /// `Int4Gpt2Model::from_weights` (gpt2.rs:1356-1436)
    pub fn from_weights(weights: &Gpt2Weights, config: &Gpt2Config, group_size: usize, registry: &Arc<KernelRegistry>) -> Result<Self> {
        if group_size == 0 {
            return Err(NnError::Arg("group_size must be non-zero".into()));
        }
        Ok(Self(create_model(weights, config, group_size, 0, registry)?))
    }
    pub fn config(&self) -> &Gpt2Config {
        self.0.config()
    }
    pub fn group_size(&self) -> usize {
        self.0.group_size
    }
    pub fn forward(&self, token_ids: &[u32]) -> Result<GpuTensor> {
        self.0.forward(token_ids)
    }
    pub fn generate(&self, prompt_tokens: &[u32], max_new_tokens: usize) -> Result<Vec<u32>> {
        self.0.generate(prompt_tokens, max_new_tokens)
    }
    /// `quantized_memory_bytes` (gpt2.rs:1563-1576)
    pub fn quantized_memory_bytes(&self) -> usize {
        unsafe { sys::b200nn_gpt2_quantized_memory_bytes(self.0.h) }
    }
    /// The batched, KV-cached and sampling calls of [`Gpt2Model`] work on an int4 model as well.
    pub fn as_model(&self) -> &Gpt2Model {
        &self.0
    }
}

/// `KvCache` (gpt2.rs:1064-1117): on the device, fp16, one slot per sequence of a batch.
pub struct KvCache {
    h: *mut sys::b200nn_kvcache,
    registry: Arc<KernelRegistry>,
}
impl KvCache {
    pub fn new(model: &Gpt2Model, batch: usize, capacity: usize) -> Result<Self> {
        let mut h = ptr::null_mut();
        model.registry.check(unsafe { sys::b200nn_kvcache_create(model.h, batch, capacity, &mut h) })?;
        Ok(Self { h, registry: Arc::clone(&model.registry) })
    }
    pub fn len(&self) -> usize {
        unsafe { sys::b200nn_kvcache_len(self.h) }
    }
    pub fn is_empty(&self) -> bool {
        self.len() == 0
    }
    pub fn reset(&mut self) -> Result<()> {
        self.registry.check(unsafe { sys::b200nn_kvcache_reset(self.h) })
    }
}
impl Drop for KvCache {
    fn drop(&mut self) {
        unsafe { sys::b200nn_kvcache_destroy(self.h) }
    }
}

/// The twelve slices `TransformerBlock::new` takes (gpt2.rs:120-135), dense weights in Linear layout `[out,in]`.
#[derive(Clone, Debug, Default)]
pub struct BlockWeights {
    pub ln_1_weight: Vec<f32>,
    pub ln_1_bias: Vec<f32>,
    pub attn_qkv_weight: Vec<f32>,
    pub attn_qkv_bias: Vec<f32>,
    pub attn_out_weight: Vec<f32>,
    pub attn_out_bias: Vec<f32>,
    pub ln_2_weight: Vec<f32>,
    pub ln_2_bias: Vec<f32>,
    pub ffn_up_weight: Vec<f32>,
    pub ffn_up_bias: Vec<f32>,
    pub ffn_down_weight: Vec<f32>,
    pub ffn_down_bias: Vec<f32>,
}

/// `TransformerBlock` (gpt2.rs:98-289); `new_int4` is `Int4TransformerBlock::new` (gpt2.rs:1232-1296).
pub struct TransformerBlock {
    h: *mut sys::b200nn_block,
    registry: Arc<KernelRegistry>,
}
impl TransformerBlock {
    fn create(w: &BlockWeights, config: &Gpt2Config, group_size: usize, registry: &Arc<KernelRegistry>) -> Result<Self> {
        let d = config.n_embd;
        if w.attn_qkv_weight.len() != 3 * d * d
            || w.attn_out_weight.len() != d * d
            || w.ffn_up_weight.len() != 4 * d * d
            || w.ffn_down_weight.len() != 4 * d * d
            || w.ln_1_weight.len() != d
            || w.ln_2_weight.len() != d
        {
            return Err(NnError::ShapeMismatch("block weights do not match n_embd".into()));
        }
        let cw = sys::b200nn_block_weights {
            ln_1_weight: w.ln_1_weight.as_ptr(),
            ln_1_bias: w.ln_1_bias.as_ptr(),
            attn_qkv_weight: w.attn_qkv_weight.as_ptr(),
            attn_qkv_bias: w.attn_qkv_bias.as_ptr(),
            attn_out_weight: w.attn_out_weight.as_ptr(),
            attn_out_bias: w.attn_out_bias.as_ptr(),
            ln_2_weight: w.ln_2_weight.as_ptr(),
            ln_2_bias: w.ln_2_bias.as_ptr(),
            ffn_up_weight: w.ffn_up_weight.as_ptr(),
            ffn_up_bias: w.ffn_up_bias.as_ptr(),
            ffn_down_weight: w.ffn_down_weight.as_ptr(),
            ffn_down_bias: w.ffn_down_bias.as_ptr(),
        };
        let cc = config.to_c();
        let mut h = ptr::null_mut();
        let rc = unsafe {
            if group_size == 0 {
                sys::b200nn_block_create(registry.as_ptr(), &cc, &cw, 0, &mut h)
            } else {
                sys::b200nn_int4_block_create(registry.as_ptr(), &cc, &cw, group_size, 0, &mut h)
            }
        };
        registry.check(rc)?;
        Ok(Self { h, registry: Arc::clone(registry) })
    }
    pub fn new(weights: &BlockWeights, config: &Gpt2Config, registry: &Arc<KernelRegistry>) -> Result<Self> {
        Self::create(weights, config, 0, registry)
    }
    pub fn new_int4(weights: &BlockWeights, config: &Gpt2Config, group_size: usize, registry: &Arc<KernelRegistry>) -> Result<Self> {
        if group_size == 0 {
            return Err(NnError::Arg("group_size must be non-zero".into()));
        }
        Self::create(weights, config, group_size, registry)
    }
    /// `forward` / `forward_auto_fused` (gpt2.rs:172-243, 1299-1339): `x [seq_len,d]` of one sequence, causal
    pub fn forward(&self, x: &GpuTensor) -> Result<GpuTensor> {
        let mut y = ptr::null_mut();
        let rc = unsafe { sys::b200nn_block_forward(self.h, x.handle(), &mut y) };
        GpuTensor::wrap(&self.registry, rc, y)
    }
    pub fn forward_auto_fused(&self, x: &GpuTensor) -> Result<GpuTensor> {
        self.forward(x)
    }
}
impl Drop for TransformerBlock {
    fn drop(&mut self) {
        unsafe { sys::b200nn_block_destroy(self.h) }
    }
}

/// The batched generate loop in pieces, state resident on the device (no counterpart in the reference, whose
/// `generate` handles one sequence): prefill the prompts, run greedy steps without host synchronisation, read tokens.
pub struct DecodeSession {
    h: *mut sys::b200nn_session,
    batch: usize,
    capacity: usize,
    registry: Arc<KernelRegistry>,
}
impl DecodeSession {
    pub fn new(model: &Gpt2Model, batch: usize, capacity: usize) -> Result<Self> {
        let mut h = ptr::null_mut();
        model.registry.check(unsafe { sys::b200nn_session_create(model.h, batch, capacity, 0, &mut h) })?;
        Ok(Self { h, batch, capacity, registry: Arc::clone(&model.registry) })
    }
    pub fn prefill(&mut self, prompts: &[u32], prompt_len: usize) -> Result<()> {
        if prompts.len() != self.batch * prompt_len {
            return Err(NnError::ShapeMismatch("prompts must be [batch,prompt_len]".into()));
        }
        self.registry.check(unsafe { sys::b200nn_session_prefill(self.h, prompts.as_ptr(), prompt_len) })
    }
    pub fn step(&mut self, n_steps: usize) -> Result<()> {
        self.registry.check(unsafe { sys::b200nn_session_step(self.h, n_steps) })
    }
    pub fn position(&self) -> usize {
        unsafe { sys::b200nn_session_position(self.h) }
    }
    /// Tokens generated so far, one vector per sequence.
    pub fn tokens(&self) -> Result<Vec<Vec<u32>>> {
        let mut flat = vec![0u32; self.batch * self.capacity];
        let mut generated = 0usize;
        self.registry.check(unsafe { sys::b200nn_session_tokens(self.h, flat.as_mut_ptr(), self.capacity, &mut generated) })?;
        Ok((0..self.batch).map(|b| flat[b * self.capacity..b * self.capacity + generated].to_vec()).collect())
    }
}
impl Drop for DecodeSession {
    fn drop(&mut self) {
        unsafe { sys::b200nn_session_destroy(self.h) }
    }
}
