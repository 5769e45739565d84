//! B200-native replacement for the weight-only quantization module of `oxicuda-dnn`
//! (`crates/oxicuda-dnn/src/quantize/gptq_awq.rs`) and for its scalar quantize surface
//! (`crates/oxicuda-dnn/src/quantize/{fp8_quantize.rs,int8_quantize.rs}`): the same item names, fields, validation and
//! error kinds over the C ABI of libb2q.so.  Where the reference's `WeightQuantPlan` returns the PTX text of a kernel
//! (`generate_*_ptx`) for the caller to load and launch, the plan here has a `launch_*` method that runs the kernel of
//! that role on device buffers in the reference's layout (`QuantizedWeight`).
//!
//! Written without a Rust toolchain at hand: `tests/test_host_logic.py` checks every `sys::` item used here against the
//! generated bindings.
use std::os::raw::c_void;

use oxicuda_blas_b200::{sys, BlasError, BlasHandle, CUdeviceptr};

// ---- DnnError, crates/oxicuda-dnn/src/error.rs (the variants this module produces) -------------------------------
#[derive(Debug, Clone, PartialEq)]
pub enum DnnError {
    InvalidArgument(String),
    InvalidDimension(String),
    BufferTooSmall { expected: usize, actual: usize },
    /// Kept for signature parity: nothing here generates PTX.
    PtxGeneration(String),
    /// CUDA errors, launch failures and anything else the device layer reports.
    Device(BlasError),
}
impl std::fmt::Display for DnnError {
    fn fmt(&self, f: &mut std::fmt::Formatter<'_>) -> std::fmt::Result {
        match self {
            DnnError::InvalidArgument(m) => write!(f, "invalid argument: {m}"),
            DnnError::InvalidDimension(m) => write!(f, "invalid dimension: {m}"),
            DnnError::BufferTooSmall { expected, actual } => write!(f, "buffer too small: expected {expected}, actual {actual}"),
            DnnError::PtxGeneration(m) => write!(f, "PTX generation: {m}"),
            DnnError::Device(e) => write!(f, "{e}"),
        }
    }
}
impl std::error::Error for DnnError {}
pub type DnnResult<T> = Result<T, DnnError>;

fn map_status(h: &BlasHandle, st: i32) -> DnnResult<()> {
    match h.check(st) {
        Ok(()) => Ok(()),
        Err(BlasError::InvalidArgument(m)) => Err(DnnError::InvalidArgument(m)),
        Err(BlasError::InvalidDimension(m)) => Err(DnnError::InvalidDimension(m)),
        Err(BlasError::BufferTooSmall { expected, actual }) => Err(DnnError::BufferTooSmall { expected, actual }),
        Err(e) => Err(DnnError::Device(e)),
    }
}

/// Thread block of the reference's kernels (`gptq_awq.rs:26`); only `launch_params` reports it.
pub const QUANT_BLOCK_SIZE: u32 = 256;

// ---- configuration, gptq_awq.rs:37-199 ---------------------------------------------------------------------------
#[derive(Debug, Clone)]
pub enum WeightQuantMethod { Gptq(GptqConfig), Awq(AwqConfig) }
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
pub enum QuantMethodTag { Gptq, Awq }

#[derive(Debug, Clone)]
pub struct GptqConfig {
    pub bits: u32,
    pub group_size: usize,
    pub block_size: usize,
    pub damp_percent: f32,
    pub symmetric: bool,
    pub act_order: bool,
    pub true_sequential: bool,
}
impl Default for GptqConfig {
    fn default() -> Self {
        Self { bits: 4, group_size: 128, block_size: 128, damp_percent: 0.01, symmetric: true, act_order: false, true_sequential: true }
    }
}
impl GptqConfig {
    /// `validate` (`gptq_awq.rs:102-127`).
    pub fn validate(&self) -> DnnResult<()> {
        if !matches!(self.bits, 2 | 3 | 4 | 8) { return Err(DnnError::InvalidArgument(format!("GPTQ bits must be 2, 3, 4, or 8; got {}", self.bits))); }
        if self.group_size == 0 { return Err(DnnError::InvalidArgument("GPTQ group_size must be non-zero".into())); }
        if self.block_size == 0 { return Err(DnnError::InvalidArgument("GPTQ block_size must be non-zero".into())); }
        if self.damp_percent < 0.0 { return Err(DnnError::InvalidArgument(format!("GPTQ damp_percent must be non-negative; got {}", self.damp_percent))); }
        Ok(())
    }
}

#[derive(Debug, Clone)]
pub struct AwqConfig {
    pub bits: u32,
    pub group_size: usize,
    pub zero_point: bool,
    pub search_alpha_min: f32,
    pub search_alpha_max: f32,
    pub search_steps: usize,
}
impl Default for AwqConfig {
    fn default() -> Self { Self { bits: 4, group_size: 128, zero_point: true, search_alpha_min: 0.0, search_alpha_max: 1.0, search_steps: 20 } }
}
impl AwqConfig {
    /// `validate` (`gptq_awq.rs:174-199`).
    pub fn validate(&self) -> DnnResult<()> {
        if !matches!(self.bits, 4 | 8) { return Err(DnnError::InvalidArgument(format!("AWQ bits must be 4 or 8; got {}", self.bits))); }
        if self.group_size == 0 { return Err(DnnError::InvalidArgument("AWQ group_size must be non-zero".into())); }
        if self.search_alpha_min > self.search_alpha_max {
            return Err(DnnError::InvalidArgument(format!("AWQ search_alpha_min ({}) must be <= search_alpha_max ({})", self.search_alpha_min, self.search_alpha_max)));
        }
        if self.search_steps == 0 { return Err(DnnError::InvalidArgument("AWQ search_steps must be non-zero".into())); }
        Ok(())
    }
}

/// `QuantizedWeight` (`gptq_awq.rs:209-232`): element counts of the device buffers of one quantized matrix.
#[derive(Debug, Clone)]
pub struct QuantizedWeight {
    pub method: QuantMethodTag,
    pub bits: u32,
    pub group_size: usize,
    pub rows: usize,
    pub cols: usize,
    pub packed_weight_elements: usize,
    pub scale_elements: usize,
    pub zero_point_elements: usize,
    pub has_zero_point: bool,
}

// ---- WeightQuantPlan, gptq_awq.rs:240-1085 -----------------------------------------------------------------------
#[derive(Debug)]
pub struct WeightQuantPlan { method: WeightQuantMethod, weight_rows: usize, weight_cols: usize }

impl WeightQuantPlan {
    /// `new` (`gptq_awq.rs:254-283`).
    pub fn new(method: WeightQuantMethod, rows: usize, cols: usize) -> DnnResult<Self> {
        if rows == 0 || cols == 0 { return Err(DnnError::InvalidDimension("weight dimensions must be non-zero".into())); }
        let group_size = match &method {
            WeightQuantMethod::Gptq(cfg) => { cfg.validate()?; cfg.group_size }
            WeightQuantMethod::Awq(cfg) => { cfg.validate()?; cfg.group_size }
        };
        if cols % group_size != 0 { return Err(DnnError::InvalidArgument(format!("cols ({cols}) must be divisible by group_size ({group_size})"))); }
        Ok(Self { method, weight_rows: rows, weight_cols: cols })
    }
    fn bits(&self) -> u32 { match &self.method { WeightQuantMethod::Gptq(c) => c.bits, WeightQuantMethod::Awq(c) => c.bits } }
    fn group_size(&self) -> usize { match &self.method { WeightQuantMethod::Gptq(c) => c.group_size, WeightQuantMethod::Awq(c) => c.group_size } }
    pub fn elements_per_u32(&self) -> u32 { 32 / self.bits() }
    fn groups_per_row(&self) -> usize { self.weight_cols / self.group_size() }

    /// `quantized_weight_info` (`gptq_awq.rs:996-1027`).
    pub fn quantized_weight_info(&self) -> QuantizedWeight {
        let total = self.weight_rows * self.weight_cols;
        let epu = self.elements_per_u32() as usize;
        let scale_elements = self.weight_rows * self.groups_per_row();
        let (has_zero_point, method) = match &self.method {
            WeightQuantMethod::Gptq(c) => (!c.symmetric, QuantMethodTag::Gptq),
            WeightQuantMethod::Awq(c) => (c.zero_point, QuantMethodTag::Awq),
        };
        QuantizedWeight { method, bits: self.bits(), group_size: self.group_size(), rows: self.weight_rows, cols: self.weight_cols,
                          packed_weight_elements: (total + epu - 1) / epu, scale_elements,
                          zero_point_elements: if has_zero_point { scale_elements } else { 0 }, has_zero_point }
    }
    /// `workspace_bytes` (`gptq_awq.rs:1029-1052`): what the reference's full algorithm would need; the kernels here need none.
    pub fn workspace_bytes(&self) -> usize {
        match &self.method {
            WeightQuantMethod::Gptq(c) => self.weight_cols * 4 + if c.act_order { self.weight_cols * 4 } else { 0 } + self.weight_rows * c.block_size * 4,
            WeightQuantMethod::Awq(c) => self.weight_cols * 4 + self.weight_cols * 4 + c.search_steps * 4,
        }
    }
    /// `shared_memory_bytes` (`gptq_awq.rs:1057-1066`).
    pub fn shared_memory_bytes(&self) -> usize {
        match &self.method { WeightQuantMethod::Gptq(c) => c.block_size * 4, WeightQuantMethod::Awq(c) => c.group_size * 4 }
    }
    /// `launch_params` (`gptq_awq.rs:1071-1080`): the reference's (grid, block); informational here.
    pub fn launch_params(&self) -> (usize, usize) {
        let block = QUANT_BLOCK_SIZE as usize;
        let threads = match &self.method { WeightQuantMethod::Gptq(_) => self.weight_rows, WeightQuantMethod::Awq(_) => self.weight_rows * self.weight_cols };
        ((threads + block - 1) / block, block)
    }

    fn gptq(&self, what: &str) -> DnnResult<&GptqConfig> {
        match &self.method { WeightQuantMethod::Gptq(c) => Ok(c), WeightQuantMethod::Awq(_) => Err(DnnError::InvalidArgument(format!("{what} called on AWQ plan"))) }
    }
    fn awq(&self, what: &str) -> DnnResult<&AwqConfig> {
        match &self.method { WeightQuantMethod::Awq(c) => Ok(c), WeightQuantMethod::Gptq(_) => Err(DnnError::InvalidArgument(format!("{what} called on GPTQ plan"))) }
    }

    /// The kernel of `generate_gptq_quantize_ptx` (`gptq_awq.rs:329-499`): weight [rows x cols] f32, hessian_diag [cols] f32
    /// -> packed u32 words (no clearing needed) and scales [rows x groups].
    pub fn launch_gptq_quantize(&self, h: &BlasHandle, weight: CUdeviceptr, hessian_diag: CUdeviceptr, out_packed: CUdeviceptr, scales: CUdeviceptr) -> DnnResult<()> {
        let c = self.gptq("generate_gptq_quantize_ptx")?;
        map_status(h, unsafe {
            sys::b2q_gptq_quantize_f32(h.raw(), weight as *const f32, hessian_diag as *const f32, self.weight_rows as i64, self.weight_cols as i64,
                                       c.group_size as i64, c.bits as i32, c.symmetric as i32, out_packed as *mut u32, scales as *mut f32)
        })
    }
    /// The kernel of `generate_gptq_dequantize_ptx` (`gptq_awq.rs:509-616`): out [rows x cols] f32; `zeros` is read by an
    /// asymmetric plan only, as in the reference.
    pub fn launch_gptq_dequantize(&self, h: &BlasHandle, packed: CUdeviceptr, scales: CUdeviceptr, zeros: CUdeviceptr, out: CUdeviceptr) -> DnnResult<()> {
        let c = self.gptq("generate_gptq_dequantize_ptx")?;
        let z = if c.symmetric { std::ptr::null() } else { zeros as *const f32 };
        map_status(h, unsafe {
            sys::b2q_wq_dequantize(h.raw(), packed as *const u32, scales as *const f32, z, self.weight_rows as i64, self.weight_cols as i64,
                                   c.group_size as i64, c.bits as i32, out as *mut c_void, sys::B2Q_OUT_F32 as i32)
        })
    }
    /// The kernel of `generate_awq_scale_search_ptx` (`gptq_awq.rs:626-713`): scale_out[c] = a * rsqrt(a), a = max(|act|, 1e-7).
    pub fn launch_awq_scale_search(&self, h: &BlasHandle, act_stats: CUdeviceptr, scale_out: CUdeviceptr, num_channels: usize) -> DnnResult<()> {
        self.awq("generate_awq_scale_search_ptx")?;
        map_status(h, unsafe { sys::b2q_awq_scale_search_f32(h.raw(), act_stats as *const f32, num_channels as i64, scale_out as *mut f32) })
    }
    /// The kernel of `generate_awq_quantize_ptx` (`gptq_awq.rs:723-857`): group scales are an input, zero points receive 0.
    pub fn launch_awq_quantize(&self, h: &BlasHandle, weight: CUdeviceptr, channel_scales: CUdeviceptr, out_packed: CUdeviceptr, group_scales: CUdeviceptr,
                               zeros: CUdeviceptr) -> DnnResult<()> {
        let c = self.awq("generate_awq_quantize_ptx")?;
        let z = if c.zero_point { zeros as *mut f32 } else { std::ptr::null_mut() };
        map_status(h, unsafe {
            sys::b2q_awq_quantize_f32(h.raw(), weight as *const f32, channel_scales as *const f32, group_scales as *const f32, self.weight_rows as i64,
                                      self.weight_cols as i64, c.group_size as i64, c.bits as i32, out_packed as *mut u32, z)
        })
    }
    /// The kernel of `generate_fused_dequant_gemv_ptx` (`gptq_awq.rs:867-986`): y [rows] = dequant(W) x in the reference's
    /// summation order (bit-exact).  `launch_fused_dequant_gemv_split` lets the library cut the columns over more threads.
    pub fn launch_fused_dequant_gemv(&self, h: &BlasHandle, packed: CUdeviceptr, scales: CUdeviceptr, x: CUdeviceptr, y: CUdeviceptr) -> DnnResult<()> {
        self.gemv(h, packed, scales, 0, x, y, 1)
    }
    pub fn launch_fused_dequant_gemv_split(&self, h: &BlasHandle, packed: CUdeviceptr, scales: CUdeviceptr, zeros: CUdeviceptr, x: CUdeviceptr, y: CUdeviceptr) -> DnnResult<()> {
        self.gemv(h, packed, scales, zeros, x, y, 0)
    }
    fn gemv(&self, h: &BlasHandle, packed: CUdeviceptr, scales: CUdeviceptr, zeros: CUdeviceptr, x: CUdeviceptr, y: CUdeviceptr, split_k: i32) -> DnnResult<()> {
        map_status(h, unsafe {
            sys::b2q_fused_dequant_gemv_f32(h.raw(), packed as *const u32, scales as *const f32, zeros as *const f32, x as *const f32, self.weight_rows as i64,
                                            self.weight_cols as i64, self.group_size() as i64, self.bits() as i32, split_k, y as *mut f32)
        })
    }
}

// ---- GptqState / AwqChannelScales, gptq_awq.rs:1090-1197 (host bookkeeping) --------------------------------------
#[derive(Debug, Clone)]
pub struct GptqState { pub rows: usize, pub cols: usize, pub group_size: usize, pub bits: u32, pub columns_processed: usize, pub quantization_error: f64 }
impl GptqState {
    pub fn new(rows: usize, cols: usize, config: &GptqConfig) -> Self {
        Self { rows, cols, group_size: config.group_size, bits: config.bits, columns_processed: 0, quantization_error: 0.0 }
    }
    pub fn num_groups(&self) -> usize { (self.cols + self.group_size - 1) / self.group_size }
    pub fn num_column_blocks(&self) -> usize { (self.cols + self.group_size - 1) / self.group_size }
    pub fn elements_per_packed_word(&self) -> u32 { 32 / self.bits }
    pub fn is_complete(&self) -> bool { self.columns_processed >= self.cols }
}
#[derive(Debug, Clone)]
pub struct AwqChannelScales { pub num_channels: usize, pub scales: Vec<f32>, pub best_alpha: f32 }
impl AwqChannelScales {
    pub fn new(num_channels: usize) -> Self { Self { num_channels, scales: vec![1.0; num_channels], best_alpha: 0.5 } }
    pub fn set_scale(&mut self, channel: usize, scale: f32) -> DnnResult<()> {
        if channel >= self.num_channels {
            return Err(DnnError::InvalidArgument(format!("channel index {channel} out of range (num_channels = {})", self.num_channels)));
        }
        self.scales[channel] = scale;
        Ok(())
    }
    pub fn apply_alpha(&mut self, alpha: f32) {
        self.best_alpha = alpha;
        for s in &mut self.scales { *s = s.powf(alpha); }
    }
}

// ---- scalar quantize surface, fp8_quantize.rs:45-170 and int8_quantize.rs:31-160 ----------------------------------
/// `quantize_to_fp8`: E4M3 bytes [n] and scale[0] = max(absmax / 448, 1e-12), both on the device.
pub fn quantize_to_fp8(h: &BlasHandle, input: CUdeviceptr, n: usize, output: CUdeviceptr, scale: CUdeviceptr) -> DnnResult<()> {
    map_status(h, unsafe { sys::b2q_dnn_quantize_to_fp8_f32(h.raw(), input as *const f32, n as i64, output as *mut u8, scale as *mut f32) })
}
/// `dequantize_from_fp8`: out[i] = e4m3(input[i]) * scale[0].
pub fn dequantize_from_fp8(h: &BlasHandle, input: CUdeviceptr, scale: CUdeviceptr, n: usize, output: CUdeviceptr) -> DnnResult<()> {
    map_status(h, unsafe { sys::b2q_dnn_dequantize_from_fp8_f32(h.raw(), input as *const u8, scale as *const f32, n as i64, output as *mut f32) })
}
/// `quantize_to_int8`: scale[0] = max(absmax / 127, 1e-12), ties to even.
pub fn quantize_to_int8(h: &BlasHandle, input: CUdeviceptr, n: usize, output: CUdeviceptr, scale: CUdeviceptr) -> DnnResult<()> {
    map_status(h, unsafe { sys::b2q_dnn_quantize_to_int8_f32(h.raw(), input as *const f32, n as i64, output as *mut i8, scale as *mut f32) })
}
/// `dequantize_from_int8`: out[i] = input[i] * scale[0].
pub fn dequantize_from_int8(h: &BlasHandle, input: CUdeviceptr, scale: CUdeviceptr, n: usize, output: CUdeviceptr) -> DnnResult<()> {
    map_status(h, unsafe { sys::b2q_dnn_dequantize_from_int8_f32(h.raw(), input as *const i8, scale as *const f32, n as i64, output as *mut f32) })
}
/// `quantize_block_scaled` (`block_scale.rs:51-150`): bytes clamp(rne(x / scale) + 6) and one scale per block.
pub fn quantize_block_scaled(h: &BlasHandle, input: CUdeviceptr, n: usize, block_size: u32, output: CUdeviceptr, scales: CUdeviceptr) -> DnnResult<()> {
    map_status(h, unsafe { sys::b2q_dnn_quantize_block_scaled_f32(h.raw(), input as *const f32, n as i64, block_size, output as *mut u8, scales as *mut f32) })
}
