//! B200-native replacement for the quantized GEMM / GEMV dispatch of `oxicuda-blas`: the same item names and
//! signatures (`BlasHandle`, `BlasError`, `MatrixDesc`, `gemm::<E4M3>`, `EpilogueOp`, `Int8GemmConfig`,
//! `Fp4GemmConfig`, `MicroScalingQuantizer`, `classify_workload`, `Fp8Config::tile_config`, `grouped_gemm`) over the
//! C ABI of libb2q.so.  Nothing here computes: every method validates as the reference does, then makes one call.
//!
//! Reference items: `crates/oxicuda-blas/src/{handle.rs,error.rs,types.rs}`, `level3/gemm_api.rs:82-231`,
//! `level3/gemm/epilogue.rs:29-120`, `precision/{fp8_ops.rs,fp4_fp6_ops.rs,int_ops.rs}`, `batched/grouped_gemm.rs:46-78`.
use std::ffi::CStr;
use std::marker::PhantomData;
use std::os::raw::c_void;

pub use b2q_sys as sys;

/// Device address, as the reference passes it (`CUdeviceptr`, `types.rs:540-552`).
pub type CUdeviceptr = u64;

// ---------------------------------------------------------------------------------------------------------------
// errors: BlasError, crates/oxicuda-blas/src/error.rs:17-60
// ---------------------------------------------------------------------------------------------------------------
#[derive(Debug, Clone, PartialEq)]
pub enum BlasError {
    Cuda(String),
    InvalidDimension(String),
    BufferTooSmall { expected: usize, actual: usize },
    DimensionMismatch(String),
    UnsupportedOperation(String),
    PtxGeneration(String),
    LaunchFailed(String),
    InvalidArgument(String),
    AutotuneError(String),
    /// A bounded device-side wait gave up (`B2Q_ERR_TIMEOUT`) or a collective failed (`B2Q_ERR_NCCL`).
    Device(i32, String),
}
pub type BlasResult<T> = Result<T, BlasError>;

impl std::fmt::Display for BlasError {
    fn fmt(&self, f: &mut std::fmt::Formatter<'_>) -> std::fmt::Result {
        match self {
            Self::Cuda(m) => write!(f, "CUDA driver error: {m}"),
            Self::InvalidDimension(m) => write!(f, "invalid matrix dimensions: {m}"),
            Self::BufferTooSmall { expected, actual } => write!(f, "buffer too small: expected at least {expected} elements, got {actual}"),
            Self::DimensionMismatch(m) => write!(f, "dimension mismatch: {m}"),
            Self::UnsupportedOperation(m) => write!(f, "unsupported operation: {m}"),
            Self::PtxGeneration(m) => write!(f, "PTX generation error: {m}"),
            Self::LaunchFailed(m) => write!(f, "kernel launch failed: {m}"),
            Self::InvalidArgument(m) => write!(f, "invalid argument: {m}"),
            Self::AutotuneError(m) => write!(f, "autotuner error: {m}"),
            Self::Device(code, m) => write!(f, "device status {code}: {m}"),
        }
    }
}
impl std::error::Error for BlasError {}

/// Maps a libb2q status (include/b2q.h) to the reference's variant.
pub fn status_to_error(status: i32, message: String) -> BlasError {
    match status {
        sys::B2Q_ERR_CUDA => BlasError::Cuda(message),
        sys::B2Q_ERR_INVALID_DIMENSION => BlasError::InvalidDimension(message),
        sys::B2Q_ERR_BUFFER_TOO_SMALL => BlasError::BufferTooSmall { expected: 0, actual: 0 },
        sys::B2Q_ERR_DIMENSION_MISMATCH => BlasError::DimensionMismatch(message),
        sys::B2Q_ERR_UNSUPPORTED => BlasError::UnsupportedOperation(message),
        sys::B2Q_ERR_LAUNCH_FAILED => BlasError::LaunchFailed(message),
        sys::B2Q_ERR_INVALID_ARGUMENT => BlasError::InvalidArgument(message),
        other => BlasError::Device(other, message),
    }
}

// ---------------------------------------------------------------------------------------------------------------
// BlasHandle, crates/oxicuda-blas/src/handle.rs:43-264 (Send, not Sync: one per host thread)
// ---------------------------------------------------------------------------------------------------------------
#[derive(Debug, Clone, Copy, PartialEq, Eq, PartialOrd, Ord)]
pub enum SmVersion { Sm100 }

pub struct BlasHandle {
    raw: sys::b2q_handle,
    device: i32,
    _not_sync: PhantomData<*const ()>,
}
unsafe impl Send for BlasHandle {}

impl BlasHandle {
    /// `BlasHandle::new` (`handle.rs:80-95`): binds to `device`; fails without an sm_100 GPU (there is no CPU fallback).
    pub fn new(device: i32) -> BlasResult<Self> {
        let mut raw: sys::b2q_handle = std::ptr::null_mut();
        let st = unsafe { sys::b2q_create(&mut raw, device) };
        if st != sys::B2Q_OK {
            return Err(status_to_error(st, "b2q_create failed (no CUDA device, or not an sm_100 GPU)".into()));
        }
        Ok(Self { raw, device, _not_sync: PhantomData })
    }
    /// `with_stream` / `set_stream` (`handle.rs:243-255`): `stream` is a `CUstream` / `cudaStream_t`.
    pub fn set_stream(&mut self, stream: *mut c_void) -> BlasResult<()> { self.check(unsafe { sys::b2q_set_stream(self.raw, stream) }) }
    pub fn sm_version(&self) -> SmVersion { SmVersion::Sm100 }
    pub fn device(&self) -> i32 { self.device }
    pub fn raw(&self) -> sys::b2q_handle { self.raw }
    /// Synchronises the stream and returns what kernels recorded on the device (non-finite FP8 input, timeouts).
    pub fn check_device_status(&self) -> BlasResult<()> { self.check(unsafe { sys::b2q_check(self.raw) }) }
    pub fn check(&self, status: i32) -> BlasResult<()> {
        if status == sys::B2Q_OK { return Ok(()); }
        let msg = unsafe { CStr::from_ptr(sys::b2q_last_error(self.raw)) }.to_string_lossy().into_owned();
        Err(status_to_error(status, msg))
    }
}
impl Drop for BlasHandle {
    fn drop(&mut self) { unsafe { sys::b2q_destroy(self.raw); } }
}

// ---------------------------------------------------------------------------------------------------------------
// types: crates/oxicuda-blas/src/types.rs:139-197, :354-483, :540-740
// ---------------------------------------------------------------------------------------------------------------
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
pub enum Transpose { NoTrans, Trans, ConjTrans }
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
pub enum Layout { RowMajor, ColMajor }

/// 8-bit float storage types of the reference (`types.rs:354-483`).
#[repr(transparent)] #[derive(Debug, Clone, Copy, PartialEq, Eq, Default)]
pub struct E4M3(pub u8);
#[repr(transparent)] #[derive(Debug, Clone, Copy, PartialEq, Eq, Default)]
pub struct E5M2(pub u8);
/// bf16 bit pattern (the output type of the FP8 GEMM).
#[repr(transparent)] #[derive(Debug, Clone, Copy, PartialEq, Eq, Default)]
pub struct Bf16(pub u16);

pub trait Fp8Element: Copy { const FMT: i32; }
impl Fp8Element for E4M3 { const FMT: i32 = sys::B2Q_FP8_E4M3; }
impl Fp8Element for E5M2 { const FMT: i32 = sys::B2Q_FP8_E5M2; }

#[derive(Debug, Clone, Copy)]
pub struct MatrixDesc<T> { pub ptr: CUdeviceptr, pub rows: u32, pub cols: u32, pub ld: u32, pub layout: Layout, _p: PhantomData<T> }
#[derive(Debug)]
pub struct MatrixDescMut<T> { pub ptr: CUdeviceptr, pub rows: u32, pub cols: u32, pub ld: u32, pub layout: Layout, _p: PhantomData<T> }
impl<T> MatrixDesc<T> {
    pub fn from_raw(ptr: CUdeviceptr, rows: u32, cols: u32, ld: u32, layout: Layout) -> Self { Self { ptr, rows, cols, ld, layout, _p: PhantomData } }
}
impl<T> MatrixDescMut<T> {
    pub fn from_raw(ptr: CUdeviceptr, rows: u32, cols: u32, ld: u32, layout: Layout) -> Self { Self { ptr, rows, cols, ld, layout, _p: PhantomData } }
}

/// EpilogueOp, `level3/gemm/epilogue.rs:29-45`.
#[derive(Debug, Clone, Copy, PartialEq, Eq, Hash)]
pub enum EpilogueOp { LinearCombination, LinearCombinationRelu, LinearCombinationGelu, LinearCombinationBias, LinearCombinationBiasRelu }
impl EpilogueOp {
    pub fn needs_bias(self) -> bool { matches!(self, Self::LinearCombinationBias | Self::LinearCombinationBiasRelu) }
    fn code(self) -> i32 { self as i32 }
}

/// Per-tensor or per-row dequantization scales of an FP8 operand (device f32).
#[derive(Debug, Clone, Copy)]
pub enum Fp8Scale { PerTensor(CUdeviceptr), PerRow(CUdeviceptr) }
impl Fp8Scale {
    fn parts(self) -> (*const f32, i32) {
        match self { Self::PerTensor(p) => (p as *const f32, sys::B2Q_SCALE_SCALAR), Self::PerRow(p) => (p as *const f32, sys::B2Q_SCALE_PER_ROW) }
    }
}

/// `gemm::<E4M3>` (`level3/gemm_api.rs:82-231`) in the form that works for FP8: C = op(alpha * A . B * sa * sb + beta * C
/// + bias), A `[M x K]` row-major, B either the reference's row-major `[K x N]` (`trans_b = NoTrans`) or the
/// "out x in" weight `[N x K]` (`trans_b = Trans`, no copy), C `[M x N]` bf16.  Validation order as `gemm_impl`:
/// zero dimensions, inner mismatch, layout / padding, overlap.
#[allow(clippy::too_many_arguments)]
pub fn gemm_fp8<T: Fp8Element>(handle: &BlasHandle, trans_a: Transpose, trans_b: Transpose, alpha: f32, a: &MatrixDesc<T>, scale_a: Fp8Scale,
                               b: &MatrixDesc<T>, scale_b: Fp8Scale, beta: f32, c: &mut MatrixDescMut<Bf16>, epilogue: EpilogueOp,
                               bias: Option<CUdeviceptr>) -> BlasResult<()> {
    if a.rows == 0 || a.cols == 0 || b.rows == 0 || b.cols == 0 {
        return Err(BlasError::InvalidDimension("GEMM dimensions must be non-zero".into()));
    }
    if trans_a != Transpose::NoTrans { return Err(BlasError::UnsupportedOperation("FP8 GEMM takes A untransposed (K-major)".into())); }
    let (m, k) = (a.rows as i64, a.cols as i64);
    let (kb, n, w_layout) = match trans_b {
        Transpose::NoTrans => (b.rows as i64, b.cols as i64, sys::B2Q_W_KN),
        _ => (b.cols as i64, b.rows as i64, sys::B2Q_W_NK),
    };
    if k != kb { return Err(BlasError::DimensionMismatch(format!("A is {m}x{k} but op(B) has {kb} rows"))); }
    if a.layout != Layout::RowMajor || b.layout != Layout::RowMajor || c.layout != Layout::RowMajor || a.ld != a.cols || b.ld != b.cols || c.ld != c.cols {
        return Err(BlasError::InvalidArgument("row-major, unpadded operands only".into()));
    }
    if c.rows as i64 != m || c.cols as i64 != n { return Err(BlasError::DimensionMismatch("C must be M x N".into())); }
    if epilogue.needs_bias() && bias.is_none() { return Err(BlasError::InvalidArgument("this epilogue needs a bias vector".into())); }
    let (sa, ka) = scale_a.parts();
    let (sb, kbk) = scale_b.parts();
    let d = sys::b2q_gemm_fp8_desc {
        a: a.ptr as *const u8, w: b.ptr as *const u8, m, n, k, fmt: T::FMT, scale_a: sa, scale_a_kind: ka, scale_w: sb, scale_w_kind: kbk,
        out: c.ptr as *mut c_void, out_type: sys::B2Q_OUT_BF16, alpha, beta, bias: bias.map_or(std::ptr::null(), |p| p as *const f32),
        epilogue: epilogue.code(), w_layout,
    };
    handle.check(unsafe { sys::b2q_gemm_fp8_ex(handle.raw(), &d) })
}

// ---------------------------------------------------------------------------------------------------------------
// tile heuristics: precision/fp8_ops.rs:42-397, fp4_fp6_ops.rs:996-1075, int_ops.rs:141-176, level3/gemm/dispatch.rs:57-107
// ---------------------------------------------------------------------------------------------------------------
pub type TileConfig = sys::b2q_tile_config;
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
pub enum Fp8WorkloadClass { SmallSquare, LargeSquare, SkinnyM, SkinnyN, SkinnyK, General }
pub fn classify_workload(m: u32, n: u32, k: u32) -> Fp8WorkloadClass {
    match unsafe { sys::b2q_classify_workload(m, n, k) } {
        0 => Fp8WorkloadClass::SmallSquare, 1 => Fp8WorkloadClass::LargeSquare, 2 => Fp8WorkloadClass::SkinnyM,
        3 => Fp8WorkloadClass::SkinnyN, 4 => Fp8WorkloadClass::SkinnyK, _ => Fp8WorkloadClass::General,
    }
}
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
pub enum QuantDtype { Fp8 = 0, Fp4 = 1, Int8 = 2 }
pub struct Fp8Config;
impl Fp8Config {
    /// `Fp8Config::tile_config(Sm100, m, n, k)` (`fp8_ops.rs:239-304`): the reference's Blackwell heuristic.
    pub fn tile_config(m: u32, n: u32, k: u32) -> BlasResult<TileConfig> { ref_tile(QuantDtype::Fp8, m, n, k) }
    pub fn compute_split_k(m: u32, n: u32, k: u32) -> u32 { unsafe { sys::b2q_fp8_compute_split_k(m, n, k) } }
}
pub fn select_fp4_tile(m: u32, n: u32, k: u32) -> BlasResult<TileConfig> { ref_tile(QuantDtype::Fp4, m, n, k) }
fn ref_tile(dtype: QuantDtype, m: u32, n: u32, k: u32) -> BlasResult<TileConfig> {
    let mut t = TileConfig::default();
    match unsafe { sys::b2q_ref_tile_config(dtype as i32, m, n, k, &mut t) } {
        sys::B2Q_OK => Ok(t),
        st => Err(status_to_error(st, "tile_config: dimensions must be non-zero".into())),
    }
}
/// The static per-shape table the library dispatches with (the autotuner's role): tile and kernel family.
pub fn select_tile(dtype: QuantDtype, m: u32, n: u32, k: u32) -> BlasResult<(TileConfig, i32)> {
    let mut t = TileConfig::default();
    let mut kernel = 0;
    match unsafe { sys::b2q_select_tile(dtype as i32, m, n, k, &mut t, &mut kernel) } {
        sys::B2Q_OK => Ok((t, kernel)),
        st => Err(status_to_error(st, "select_tile: dimensions must be non-zero".into())),
    }
}

// ---------------------------------------------------------------------------------------------------------------
// INT8 GEMM: Int8GemmConfig, precision/int_ops.rs:36-189
// ---------------------------------------------------------------------------------------------------------------
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
pub enum AccType { I32, F32 }
#[derive(Debug, Clone, Copy)]
pub struct Int8GemmConfig { pub m: u32, pub n: u32, pub k: u32, pub accumulator: AccType }
impl Int8GemmConfig {
    /// `validate` (`int_ops.rs:105-125`): non-zero dimensions, K a multiple of 4.
    pub fn validate(&self) -> BlasResult<()> {
        if self.m == 0 || self.n == 0 || self.k == 0 { return Err(BlasError::InvalidDimension("INT8 GEMM dimensions must be non-zero".into())); }
        if self.k % 4 != 0 { return Err(BlasError::InvalidDimension(format!("INT8 GEMM K must be a multiple of 4, got {}", self.k))); }
        Ok(())
    }
    pub fn tile_config(&self) -> BlasResult<TileConfig> { ref_tile(QuantDtype::Int8, self.m, self.n, self.k) }
    /// C = A . B^T with exact s32 accumulation; A `[M x K]`, B `[N x K]` int8 row-major (the values of the reference's
    /// K-packed `[K/4 x N]` operand); `c_s32` and / or `c_f32` (scaled by `scale_a[m] * scale_b[n]` when given).
    pub fn launch(&self, handle: &BlasHandle, a: CUdeviceptr, b: CUdeviceptr, c_s32: Option<CUdeviceptr>, c_f32: Option<CUdeviceptr>,
                  scale_a: Option<CUdeviceptr>, scale_b: Option<CUdeviceptr>) -> BlasResult<()> {
        self.validate()?;
        let p = |o: Option<CUdeviceptr>| o.unwrap_or(0);
        handle.check(unsafe {
            sys::b2q_gemm_i8(handle.raw(), a as *const i8, b as *const i8, self.m as i64, self.n as i64, self.k as i64, p(c_s32) as *mut i32,
                             p(c_f32) as *mut f32, p(scale_a) as *const f32, p(scale_b) as *const f32)
        })
    }
}

// ---------------------------------------------------------------------------------------------------------------
// FP4: Fp4Format, MicroScalingConfig, MicroScalingQuantizer, Fp4GemmConfig, precision/fp4_fp6_ops.rs:107-258, :746-898
// ---------------------------------------------------------------------------------------------------------------
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
pub enum Fp4Format { E2M1 = 0, Int4 = 1 }
/// `ScalingFormat` (`fp4_fp6_ops.rs:142-171`); every reference code path stores f32, E8M0 is this library's addition.
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
pub enum ScalingFormat { Fp32 = 0, E8M0 = 1 }
#[derive(Debug, Clone, Copy)]
pub struct MicroScalingConfig { pub block_size: usize, pub scaling_format: ScalingFormat }
impl MicroScalingConfig {
    pub fn validate(&self) -> BlasResult<()> {
        if ![32usize, 64, 128].contains(&self.block_size) {
            return Err(BlasError::InvalidArgument(format!("MicroScaling block_size must be one of [32, 64, 128], got {}", self.block_size)));
        }
        Ok(())
    }
    pub fn num_scales(&self, n: usize) -> usize { (n + self.block_size - 1) / self.block_size }
}
pub struct MicroScalingQuantizer { pub config: MicroScalingConfig }
impl MicroScalingQuantizer {
    pub fn new(config: MicroScalingConfig) -> Self { Self { config } }
    /// `quantize_fp4` (`fp4_fp6_ops.rs:849-876`) on device buffers: `values` f32 `[n]` -> packed `[n / 2]` bytes + scales.
    pub fn quantize_fp4(&self, handle: &BlasHandle, values: CUdeviceptr, n: usize, format: Fp4Format, packed: CUdeviceptr, scales: CUdeviceptr) -> BlasResult<()> {
        self.config.validate()?;
        handle.check(unsafe {
            sys::b2q_fp4_block_quantize_f32(handle.raw(), values as *const f32, n as i64, self.config.block_size as i32, format as i32,
                                            self.config.scaling_format as i32, packed as *mut u8, scales as *mut c_void)
        })
    }
    /// `dequantize_fp4` (`fp4_fp6_ops.rs:879-897`).
    pub fn dequantize_fp4(&self, handle: &BlasHandle, packed: CUdeviceptr, scales: CUdeviceptr, format: Fp4Format, original_len: usize, out: CUdeviceptr) -> BlasResult<()> {
        self.config.validate()?;
        handle.check(unsafe {
            sys::b2q_fp4_block_dequantize_f32(handle.raw(), packed as *const u8, original_len as i64, self.config.block_size as i32, format as i32,
                                              self.config.scaling_format as i32, scales as *const c_void, out as *mut f32)
        })
    }
}
/// `Fp4GemmConfig` (`fp4_fp6_ops.rs:231-258`, `:337-395`): weight-only C = dequant(W) . X.  The reference's `m` is the
/// number of quantized rows (out features), its `n` the columns of the dense operand (tokens).
#[derive(Debug, Clone, Copy)]
pub struct Fp4GemmConfig { pub m: u32, pub n: u32, pub k: u32, pub format: Fp4Format, pub micro_scaling: MicroScalingConfig }
impl Fp4GemmConfig {
    pub fn validate(&self) -> BlasResult<()> {
        if self.m == 0 || self.n == 0 || self.k == 0 {
            return Err(BlasError::InvalidDimension(format!("FP4 GEMM dimensions must be non-zero: m={}, n={}, k={}", self.m, self.n, self.k)));
        }
        if self.k % 2 != 0 { return Err(BlasError::InvalidDimension(format!("FP4 GEMM K dimension must be even for packing, got k={}", self.k))); }
        self.micro_scaling.validate()
    }
    /// Activations `[tokens x K]` bf16 (token-major; the reference's dense operand is `[K x tokens]` f32), output
    /// `[tokens x m]` bf16.  32 tokens or fewer take the decode GEMV, more the prefill GEMM.
    pub fn launch(&self, handle: &BlasHandle, codes: CUdeviceptr, scales: CUdeviceptr, x_bf16: CUdeviceptr, out_bf16: CUdeviceptr) -> BlasResult<()> {
        self.validate()?;
        handle.check(unsafe {
            sys::b2q_gemm_fp4_wo(handle.raw(), codes as *const u8, scales as *const c_void, self.micro_scaling.scaling_format as i32,
                                 self.micro_scaling.block_size as i32, self.format as i32, x_bf16 as *const c_void, self.n as i64, self.m as i64,
                                 self.k as i64, out_bf16 as *mut c_void, sys::B2Q_OUT_BF16)
        })
    }
}

// ---------------------------------------------------------------------------------------------------------------
// grouped GEMM: batched/grouped_gemm.rs:46-78
// ---------------------------------------------------------------------------------------------------------------
pub type GroupedGemmProblem = sys::b2q_gemm_fp8_problem;
pub fn grouped_gemm(handle: &BlasHandle, problems: &[GroupedGemmProblem]) -> BlasResult<()> {
    handle.check(unsafe { sys::b2q_grouped_gemm_fp8(handle.raw(), problems.as_ptr(), problems.len() as i32, sys::B2Q_FP8_E4M3, sys::B2Q_OUT_BF16) })
}

// ---------------------------------------------------------------------------------------------------------------
// INT4 helpers: pack_int4 / unpack_int4 / Int4GemmConfig, precision/int_ops.rs:215-428
// ---------------------------------------------------------------------------------------------------------------
pub fn pack_int4(handle: &BlasHandle, values_i8: CUdeviceptr, n: usize, packed: CUdeviceptr) -> BlasResult<()> {
    handle.check(unsafe { sys::b2q_pack_int4(handle.raw(), values_i8 as *const i8, n as i64, packed as *mut u32) })
}
pub fn unpack_int4(handle: &BlasHandle, packed: CUdeviceptr, words: usize, out_i8: CUdeviceptr) -> BlasResult<()> {
    handle.check(unsafe { sys::b2q_unpack_int4(handle.raw(), packed as *const u32, words as i64, out_i8 as *mut i8) })
}
