//! B200-native replacement for the quantize / dequantize entry points of `oxicuda-quant`: the same item names and
//! signatures (`MinMaxQuantizer`, `QuantParams`, `Fp8Codec`, `Fp8Format`, `Nf4Quantizer`, `LlmInt8Quantizer`,
//! `KvCacheQuantizer`) over the C ABI of libb2q.so.  The reference's methods take host slices and return `Vec`s; the
//! methods here keep those signatures (upload, one kernel call, download) and add `*_device` forms that work on
//! buffers already in HBM, which is what a serving loop calls.
//!
//! Reference items: `crates/oxicuda-quant/src/scheme/{minmax.rs,fp8.rs,nf4.rs,llm_int8.rs,kv_cache.rs}`,
//! `crates/oxicuda-quant/src/error.rs:10-58`.
use std::os::raw::c_void;

use oxicuda_blas_b200::{sys, BlasError, BlasHandle, CUdeviceptr};

// ---- QuantError, crates/oxicuda-quant/src/error.rs:10-58 ------------------------------------------------------
#[derive(Debug, Clone, PartialEq)]
pub enum QuantError {
    EmptyInput(String),
    DimensionMismatch { expected: usize, got: usize },
    GroupSizeMismatch { len: usize, group: usize },
    InvalidScale { scale: f32 },
    NonFiniteFp8(f32),
    InvalidConfig(String),
    InvalidBitWidth { bits: u32 },
    /// Anything the device layer reports that has no variant of its own (CUDA errors, launch failures).
    Device(BlasError),
}
pub type QuantResult<T> = Result<T, QuantError>;

fn map_status(h: &BlasHandle, st: i32) -> QuantResult<()> {
    match st {
        sys::B2Q_OK => Ok(()),
        sys::B2Q_ERR_EMPTY_INPUT => Err(QuantError::EmptyInput("empty input".into())),
        sys::B2Q_ERR_GROUP_SIZE_MISMATCH => Err(QuantError::GroupSizeMismatch { len: 0, group: 0 }),
        sys::B2Q_ERR_INVALID_SCALE => Err(QuantError::InvalidScale { scale: f32::NAN }),
        sys::B2Q_ERR_NON_FINITE_FP8 => Err(QuantError::NonFiniteFp8(f32::NAN)),
        sys::B2Q_ERR_INVALID_CONFIG => Err(QuantError::InvalidConfig("invalid configuration".into())),
        sys::B2Q_ERR_INVALID_BIT_WIDTH => Err(QuantError::InvalidBitWidth { bits: 0 }),
        other => Err(QuantError::Device(h.check(other).unwrap_err())),
    }
}

// ---- device memory for the host-slice forms (CUDA runtime, linked by b2q-sys) -----------------------------------
extern "C" {
    fn cudaMalloc(ptr: *mut *mut c_void, bytes: usize) -> i32;
    fn cudaFree(ptr: *mut c_void) -> i32;
    fn cudaMemcpy(dst: *mut c_void, src: *const c_void, bytes: usize, kind: i32) -> i32;
}
/// An owned device allocation of `len` elements of `T`.
pub struct DeviceBuffer<T> { ptr: *mut c_void, len: usize, _p: std::marker::PhantomData<T> }
impl<T: Copy> DeviceBuffer<T> {
    pub fn alloc(len: usize) -> QuantResult<Self> {
        let mut p: *mut c_void = std::ptr::null_mut();
        let st = unsafe { cudaMalloc(&mut p, len.max(1) * std::mem::size_of::<T>()) };
        if st != 0 { return Err(QuantError::Device(BlasError::Cuda(format!("cudaMalloc failed with {st}")))); }
        Ok(Self { ptr: p, len, _p: std::marker::PhantomData })
    }
    pub fn from_host(data: &[T]) -> QuantResult<Self> {
        let b = Self::alloc(data.len())?;
        let st = unsafe { cudaMemcpy(b.ptr, data.as_ptr() as *const c_void, std::mem::size_of_val(data), 1) };
        if st != 0 { return Err(QuantError::Device(BlasError::Cuda(format!("cudaMemcpy H2D failed with {st}")))); }
        Ok(b)
    }
    pub fn to_host(&self) -> QuantResult<Vec<T>> where T: Default {
        let mut v = vec![T::default(); self.len];
        let st = unsafe { cudaMemcpy(v.as_mut_ptr() as *mut c_void, self.ptr, self.len * std::mem::size_of::<T>(), 2) };
        if st != 0 { return Err(QuantError::Device(BlasError::Cuda(format!("cudaMemcpy D2H failed with {st}")))); }
        Ok(v)
    }
    pub fn as_device_ptr(&self) -> CUdeviceptr { self.ptr as CUdeviceptr }
    pub fn len(&self) -> usize { self.len }
    pub fn is_empty(&self) -> bool { self.len == 0 }
}
impl<T> Drop for DeviceBuffer<T> { fn drop(&mut self) { unsafe { cudaFree(self.ptr); } } }

// ---- MinMaxQuantizer, crates/oxicuda-quant/src/scheme/minmax.rs:26-324 -----------------------------------------
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
pub enum QuantScheme { Symmetric = 0, Asymmetric = 1 }
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
pub enum QuantGranularity { PerTensor, PerChannel { axis: usize }, PerGroup { group_size: usize } }
#[derive(Debug, Clone, PartialEq)]
pub struct QuantParams { pub scales: Vec<f32>, pub zero_points: Vec<i32>, pub bits: u32, pub scheme: QuantScheme }
impl QuantParams {
    /// `q_max` / `q_min` (`minmax.rs:62-80`).
    pub fn q_max(&self) -> f32 { if self.scheme == QuantScheme::Symmetric { ((1u32 << (self.bits - 1)) - 1) as f32 } else { ((1u32 << self.bits) - 1) as f32 } }
    pub fn q_min(&self) -> f32 { if self.scheme == QuantScheme::Symmetric { -((1u32 << (self.bits - 1)) as f32) } else { 0.0 } }
}
pub struct MinMaxQuantizer<'h> { pub bits: u32, pub scheme: QuantScheme, pub granularity: QuantGranularity, handle: &'h BlasHandle }
impl<'h> MinMaxQuantizer<'h> {
    pub fn new(handle: &'h BlasHandle, bits: u32, scheme: QuantScheme, granularity: QuantGranularity) -> Self { Self { bits, scheme, granularity, handle } }
    pub fn int8_symmetric(handle: &'h BlasHandle) -> Self { Self::new(handle, 8, QuantScheme::Symmetric, QuantGranularity::PerTensor) }
    pub fn int4_per_group(handle: &'h BlasHandle, group_size: usize) -> Self { Self::new(handle, 4, QuantScheme::Symmetric, QuantGranularity::PerGroup { group_size }) }

    fn slices(&self, len: usize) -> QuantResult<(i64, i64)> {
        match self.granularity {
            // `calibrate` treats PerChannel as per-tensor (minmax.rs:140-145); real per-row statistics are `calibrate_2d`
            QuantGranularity::PerTensor | QuantGranularity::PerChannel { .. } => Ok((1, len as i64)),
            QuantGranularity::PerGroup { group_size } => {
                if group_size == 0 || len % group_size != 0 { return Err(QuantError::GroupSizeMismatch { len, group: group_size }); }
                Ok(((len / group_size) as i64, group_size as i64))
            }
        }
    }
    fn calibrate_rows(&self, tensor: &[f32], rows: i64, cols: i64) -> QuantResult<QuantParams> {
        let x = DeviceBuffer::from_host(tensor)?;
        let scales = DeviceBuffer::<f32>::alloc(rows as usize)?;
        let zps = DeviceBuffer::<i32>::alloc(rows as usize)?;
        map_status(self.handle, unsafe {
            sys::b2q_minmax_calibrate_f32(self.handle.raw(), x.as_device_ptr() as *const f32, rows, cols, self.bits as i32, self.scheme as i32,
                                          scales.as_device_ptr() as *mut f32, zps.as_device_ptr() as *mut i32)
        })?;
        Ok(QuantParams { scales: scales.to_host()?, zero_points: zps.to_host()?, bits: self.bits, scheme: self.scheme })
    }
    /// `calibrate` (`minmax.rs:134-171`).
    pub fn calibrate(&self, tensor: &[f32]) -> QuantResult<QuantParams> {
        if tensor.is_empty() { return Err(QuantError::EmptyInput("calibrate: empty tensor".into())); }
        let (rows, cols) = self.slices(tensor.len())?;
        self.calibrate_rows(tensor, rows, cols)
    }
    /// `calibrate_2d` (`minmax.rs:179-207`): rows are channels.
    pub fn calibrate_2d(&self, tensor: &[f32], rows: usize, cols: usize) -> QuantResult<QuantParams> {
        if tensor.len() != rows * cols { return Err(QuantError::DimensionMismatch { expected: rows * cols, got: tensor.len() }); }
        if tensor.is_empty() { return Err(QuantError::EmptyInput("calibrate_2d: empty tensor".into())); }
        self.calibrate_rows(tensor, rows as i64, cols as i64)
    }
    /// `quantize` / `quantize_grouped` (`minmax.rs:252-299`): one i32 per code, as the reference returns them.
    pub fn quantize(&self, tensor: &[f32], params: &QuantParams) -> QuantResult<Vec<i32>> {
        if tensor.is_empty() { return Err(QuantError::EmptyInput("quantize: empty tensor".into())); }
        let rows = params.scales.len() as i64;
        let cols = tensor.len() as i64 / rows.max(1);
        let (x, s, z) = (DeviceBuffer::from_host(tensor)?, DeviceBuffer::from_host(&params.scales)?, DeviceBuffer::from_host(&params.zero_points)?);
        let codes = DeviceBuffer::<i32>::alloc(tensor.len())?;
        map_status(self.handle, unsafe {
            sys::b2q_minmax_quantize_f32(self.handle.raw(), x.as_device_ptr() as *const f32, rows, cols, s.as_device_ptr() as *const f32,
                                         z.as_device_ptr() as *const i32, params.bits as i32, params.scheme as i32, codes.as_device_ptr() as *mut i32)
        })?;
        codes.to_host()
    }
    /// `dequantize` / `dequantize_grouped` (`minmax.rs:302-324`).
    pub fn dequantize(&self, codes: &[i32], params: &QuantParams) -> QuantResult<Vec<f32>> {
        let rows = params.scales.len() as i64;
        let cols = codes.len() as i64 / rows.max(1);
        let (c, s, z) = (DeviceBuffer::from_host(codes)?, DeviceBuffer::from_host(&params.scales)?, DeviceBuffer::from_host(&params.zero_points)?);
        let out = DeviceBuffer::<f32>::alloc(codes.len())?;
        map_status(self.handle, unsafe {
            sys::b2q_minmax_dequantize_f32(self.handle.raw(), c.as_device_ptr() as *const i32, rows, cols, s.as_device_ptr() as *const f32,
                                           z.as_device_ptr() as *const i32, out.as_device_ptr() as *mut f32)
        })?;
        out.to_host()
    }
}

// ---- Fp8Codec, crates/oxicuda-quant/src/scheme/fp8.rs:32-261 ----------------------------------------------------
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
pub enum Fp8Format { E4M3 = 0, E5M2 = 1 }
impl Fp8Format { pub fn max_val(self) -> f32 { if self == Self::E4M3 { 448.0 } else { 57344.0 } } }
/// `Rounding::Reference` reproduces `Fp8Codec::fp32_to_fp8` bit for bit (truncating mantissa, `fp8.rs:163-208`);
/// `Rounding::NearestEven` is the hardware conversion (and the encoder of oxicuda-dnn).
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
pub enum Rounding { Reference = 0, NearestEven = 1 }
pub struct Fp8Codec<'h> { pub format: Fp8Format, pub saturate: bool, pub rounding: Rounding, handle: &'h BlasHandle }
impl<'h> Fp8Codec<'h> {
    pub fn e4m3(handle: &'h BlasHandle) -> Self { Self { format: Fp8Format::E4M3, saturate: true, rounding: Rounding::Reference, handle } }
    pub fn e5m2(handle: &'h BlasHandle) -> Self { Self { format: Fp8Format::E5M2, saturate: true, rounding: Rounding::Reference, handle } }
    /// `encode` (`fp8.rs:135-137`); a NaN / Inf input is `QuantError::NonFiniteFp8` (`:115-118`), detected on the device.
    pub fn encode(&self, data: &[f32]) -> QuantResult<Vec<u8>> {
        let x = DeviceBuffer::from_host(data)?;
        let codes = DeviceBuffer::<u8>::alloc(data.len())?;
        self.encode_device(x.as_device_ptr(), data.len(), codes.as_device_ptr())?;
        map_status(self.handle, unsafe { sys::b2q_check(self.handle.raw()) })?;
        codes.to_host()
    }
    pub fn encode_device(&self, x: CUdeviceptr, n: usize, codes: CUdeviceptr) -> QuantResult<()> {
        map_status(self.handle, unsafe { sys::b2q_fp8_encode_f32(self.handle.raw(), x as *const f32, n as i64, self.format as i32, self.rounding as i32, codes as *mut u8) })
    }
    /// `decode` (`fp8.rs:140-142`).
    pub fn decode(&self, data: &[u8]) -> QuantResult<Vec<f32>> {
        let c = DeviceBuffer::from_host(data)?;
        let out = DeviceBuffer::<f32>::alloc(data.len())?;
        map_status(self.handle, unsafe {
            sys::b2q_fp8_decode_f32(self.handle.raw(), c.as_device_ptr() as *const u8, data.len() as i64, self.format as i32, self.rounding as i32,
                                    out.as_device_ptr() as *mut f32)
        })?;
        out.to_host()
    }
    /// Absmax-scaled quantization of `rows` slices on the device (per-tensor: rows = 1; per-token / per-channel: rows > 1):
    /// the rule of `crates/oxicuda-dnn/src/quantize/fp8_quantize.rs:28-34` composed with this codec.
    pub fn quantize_rows_device(&self, x_f32: CUdeviceptr, rows: usize, cols: usize, scales: CUdeviceptr, codes: CUdeviceptr) -> QuantResult<()> {
        map_status(self.handle, unsafe {
            sys::b2q_fp8_quantize_rows_f32(self.handle.raw(), x_f32 as *const f32, rows as i64, cols as i64, self.format as i32, self.rounding as i32,
                                           scales as *mut f32, codes as *mut u8)
        })
    }
    pub fn quantize_rows_bf16_device(&self, x_bf16: CUdeviceptr, rows: usize, cols: usize, scales: CUdeviceptr, codes: CUdeviceptr) -> QuantResult<()> {
        map_status(self.handle, unsafe {
            sys::b2q_fp8_quantize_rows_bf16(self.handle.raw(), x_bf16 as *const c_void, rows as i64, cols as i64, self.format as i32, self.rounding as i32,
                                            scales as *mut f32, codes as *mut u8)
        })
    }
}

// ---- Nf4Quantizer, crates/oxicuda-quant/src/scheme/nf4.rs:59-203 ------------------------------------------------
pub struct Nf4Quantizer<'h> { pub block_size: usize, handle: &'h BlasHandle }
impl<'h> Nf4Quantizer<'h> {
    pub fn new(handle: &'h BlasHandle, block_size: usize) -> Self { Self { block_size, handle } }
    /// `encode` (`nf4.rs:93-125`) -> (packed bytes, per-block absmax).
    pub fn encode(&self, data: &[f32]) -> QuantResult<(Vec<u8>, Vec<f32>)> {
        if data.is_empty() { return Err(QuantError::EmptyInput("nf4 encode: empty input".into())); }
        let x = DeviceBuffer::from_host(data)?;
        let packed = DeviceBuffer::<u8>::alloc((data.len() + 1) / 2)?;
        let absmax = DeviceBuffer::<f32>::alloc((data.len() + self.block_size - 1) / self.block_size)?;
        map_status(self.handle, unsafe {
            sys::b2q_nf4_encode_f32(self.handle.raw(), x.as_device_ptr() as *const f32, data.len() as i64, self.block_size as i32,
                                    packed.as_device_ptr() as *mut u8, absmax.as_device_ptr() as *mut f32)
        })?;
        Ok((packed.to_host()?, absmax.to_host()?))
    }
    /// `decode` (`nf4.rs:127-150`).
    pub fn decode(&self, packed: &[u8], absmaxs: &[f32]) -> QuantResult<Vec<f32>> {
        let (p, a) = (DeviceBuffer::from_host(packed)?, DeviceBuffer::from_host(absmaxs)?);
        let out = DeviceBuffer::<f32>::alloc(packed.len() * 2)?;
        map_status(self.handle, unsafe {
            sys::b2q_nf4_decode_f32(self.handle.raw(), p.as_device_ptr() as *const u8, packed.len() as i64, self.block_size as i32,
                                    a.as_device_ptr() as *const f32, out.as_device_ptr() as *mut f32)
        })?;
        out.to_host()
    }
}

// ---- LlmInt8Quantizer, crates/oxicuda-quant/src/scheme/llm_int8.rs:45-311 ---------------------------------------
#[derive(Debug, Clone, Copy)]
pub struct LlmInt8Config { pub threshold: f32, pub row_wise_activations: bool }
impl LlmInt8Config {
    /// `new` (`llm_int8.rs:69-74`): the threshold must be positive and finite.
    pub fn new(threshold: f32, row_wise_activations: bool) -> QuantResult<Self> {
        if !(threshold.is_finite() && threshold > 0.0) { return Err(QuantError::InvalidConfig(format!("threshold must be positive and finite, got {threshold}"))); }
        Ok(Self { threshold, row_wise_activations })
    }
}
#[derive(Debug, Clone)]
pub struct LlmInt8Output { pub output: Vec<f32>, pub n_outlier_cols: usize, pub outlier_fraction: f32 }
pub struct LlmInt8Quantizer<'h> { pub config: LlmInt8Config, handle: &'h BlasHandle }
impl<'h> LlmInt8Quantizer<'h> {
    pub fn new(handle: &'h BlasHandle, config: LlmInt8Config) -> Self { Self { config, handle } }
    /// `matmul` (`llm_int8.rs:175-288`): x `[samples x cols]`, w `[rows x cols]` -> `[samples x rows]`, exact integer
    /// accumulation over the non-outlier columns plus the f32 product over the outlier columns.
    pub fn matmul(&self, x: &[f32], w: &[f32], samples: usize, rows: usize, cols: usize) -> QuantResult<LlmInt8Output> {
        if x.len() != samples * cols { return Err(QuantError::DimensionMismatch { expected: samples * cols, got: x.len() }); }
        if w.len() != rows * cols { return Err(QuantError::DimensionMismatch { expected: rows * cols, got: w.len() }); }
        let (xd, wd) = (DeviceBuffer::from_host(x)?, DeviceBuffer::from_host(w)?);
        let out = DeviceBuffer::<f32>::alloc(samples * rows)?;
        let n_out = DeviceBuffer::<i32>::alloc(1)?;
        let null = std::ptr::null_mut::<c_void>();
        map_status(self.handle, unsafe {
            sys::b2q_llm_int8_linear_f32(self.handle.raw(), xd.as_device_ptr() as *const f32, wd.as_device_ptr() as *const f32, samples as i64, rows as i64,
                                         cols as i64, self.config.threshold, self.config.row_wise_activations as i32, out.as_device_ptr() as *mut f32,
                                         null as *mut i8, null as *mut f32, null as *mut i8, null as *mut f32, null as *mut i32,
                                         n_out.as_device_ptr() as *mut i32)
        })?;
        let n = n_out.to_host()?[0] as usize;
        Ok(LlmInt8Output { output: out.to_host()?, n_outlier_cols: n, outlier_fraction: n as f32 / cols as f32 })
    }
}

// ---- KvCacheQuantizer, crates/oxicuda-quant/src/scheme/kv_cache.rs:33-282 ---------------------------------------
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
pub enum KvAxis { PerToken = 0, PerChannel = 1 }
pub struct KvCacheQuantizer<'h> { pub bits: u32, pub axis: KvAxis, handle: &'h BlasHandle }
impl<'h> KvCacheQuantizer<'h> {
    /// `KvCacheConfig::new` (`kv_cache.rs:59-64`): 2 to 8 bits.
    pub fn new(handle: &'h BlasHandle, bits: u32, axis: KvAxis) -> QuantResult<Self> {
        if !(2..=8).contains(&bits) { return Err(QuantError::InvalidBitWidth { bits }); }
        Ok(Self { bits, axis, handle })
    }
    /// `quantize` (`kv_cache.rs:146-221`) on device buffers; bf16 input as a serving cache holds it.
    pub fn quantize_bf16_device(&self, x_bf16: CUdeviceptr, n_tokens: usize, head_dim: usize, codes: CUdeviceptr, scales: CUdeviceptr, zero_points: CUdeviceptr) -> QuantResult<()> {
        map_status(self.handle, unsafe {
            sys::b2q_kv_cache_quantize_bf16(self.handle.raw(), x_bf16 as *const c_void, n_tokens as i64, head_dim as i64, self.bits as i32, self.axis as i32,
                                            codes as *mut u8, scales as *mut f32, zero_points as *mut f32)
        })
    }
    /// `dequantize` (`kv_cache.rs:224-238`).
    pub fn dequantize_bf16_device(&self, codes: CUdeviceptr, n_tokens: usize, head_dim: usize, scales: CUdeviceptr, zero_points: CUdeviceptr, out_bf16: CUdeviceptr) -> QuantResult<()> {
        map_status(self.handle, unsafe {
            sys::b2q_kv_cache_dequantize_bf16(self.handle.raw(), codes as *const u8, n_tokens as i64, head_dim as i64, self.axis as i32,
                                              scales as *const f32, zero_points as *const f32, out_bf16 as *mut c_void)
        })
    }
}

// ---- GGML block codecs, crates/oxicuda-quant/src/scheme/ggml.rs:147-518 -------------------------------------------
/// `GgmlType` (`ggml.rs:147-185`).
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
#[allow(non_camel_case_types)]
pub enum GgmlType { Q8_0 = 0, Q4_0 = 1, Q4_1 = 2, Q4_K = 3 }
impl GgmlType {
    pub fn block_size(self) -> usize { if self == GgmlType::Q4_K { 256 } else { 32 } }
    /// Bytes of one packed record: the reference struct's fields in order, little-endian.
    pub fn block_bytes(self) -> usize { match self { GgmlType::Q8_0 => 34, GgmlType::Q4_0 => 18, GgmlType::Q4_1 => 20, GgmlType::Q4_K => 148 } }
}
/// `BlockQ8_0` (`ggml.rs:189-195`); the other block structs unpack the same way from their records.
#[derive(Debug, Clone, PartialEq, Eq)]
pub struct BlockQ8_0 { pub d: u16, pub qs: [i8; 32] }

pub struct GgmlCodec<'h> { handle: &'h BlasHandle }
impl<'h> GgmlCodec<'h> {
    pub fn new(handle: &'h BlasHandle) -> Self { Self { handle } }
    /// Packed records of the weights: `quantize_q8_0 / q4_0 / q4_1 / q4_k` (`ggml.rs:243-472`).
    pub fn quantize_records(&self, weights: &[f32], ty: GgmlType) -> QuantResult<Vec<u8>> {
        let w = DeviceBuffer::from_host(weights)?;
        let out = DeviceBuffer::<u8>::alloc((weights.len() / ty.block_size()).max(1) * ty.block_bytes())?;
        map_status(self.handle, unsafe { sys::b2q_ggml_quantize_f32(self.handle.raw(), ty as i32, w.as_device_ptr() as *const f32, weights.len() as i64, out.as_device_ptr() as *mut u8) })?;
        out.to_host()
    }
    /// `quantize_q8_0` with the reference's return type.
    pub fn quantize_q8_0(&self, weights: &[f32]) -> QuantResult<Vec<BlockQ8_0>> {
        let rec = self.quantize_records(weights, GgmlType::Q8_0)?;
        Ok(rec.chunks_exact(34).map(|r| {
            let mut qs = [0i8; 32];
            for (q, &b) in qs.iter_mut().zip(&r[2..]) { *q = b as i8; }
            BlockQ8_0 { d: u16::from_le_bytes([r[0], r[1]]), qs }
        }).collect())
    }
    /// `dequantize_*` (`ggml.rs:265-506`) over packed records.
    pub fn dequantize_records(&self, records: &[u8], ty: GgmlType) -> QuantResult<Vec<f32>> {
        let n = records.len() / ty.block_bytes() * ty.block_size();
        let r = DeviceBuffer::from_host(records)?;
        let out = DeviceBuffer::<f32>::alloc(n)?;
        map_status(self.handle, unsafe { sys::b2q_ggml_dequantize(self.handle.raw(), ty as i32, r.as_device_ptr() as *const u8, n as i64, out.as_device_ptr() as *mut c_void, sys::B2Q_OUT_F32) })?;
        out.to_host()
    }
    /// Records already in HBM (a GGUF tensor-data region uploaded as it is) -> bf16 weights in HBM.
    pub fn dequantize_bf16_device(&self, records: CUdeviceptr, n_weights: usize, ty: GgmlType, out_bf16: CUdeviceptr) -> QuantResult<()> {
        map_status(self.handle, unsafe { sys::b2q_ggml_dequantize(self.handle.raw(), ty as i32, records as *const u8, n_weights as i64, out_bf16 as *mut c_void, sys::B2Q_OUT_BF16) })
    }
    /// `fake_quantize` (`ggml.rs:511-518`).
    pub fn fake_quantize(&self, weights: &[f32], ty: GgmlType) -> QuantResult<Vec<f32>> {
        let rec = self.quantize_records(weights, ty)?;
        self.dequantize_records(&rec, ty)
    }
}
