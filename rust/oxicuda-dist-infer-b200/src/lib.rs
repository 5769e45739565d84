//! B200-native replacement for the tensor-parallel linears of `oxicuda-dist-infer`: `DistInferHandle`,
//! `ParallelismConfig`, `ColumnLinear`, `RowLinear` and the SwiGLU MLP built from them, one rank per process and GPU,
//! over the `b2q_tp_*` entry points of libb2q.so.  The reference simulates the ranks in one thread and sums `Vec`s;
//! here the boundary collectives run on the GPU (a peer-memory all-reduce kernel for few tokens, NCCL overlapped with
//! the GEMMs for many).
//!
//! Reference items: `crates/oxicuda-dist-infer/src/handle.rs:17-239`,
//! `tensor_parallel/column_parallel.rs:25-205`, `tensor_parallel/row_parallel.rs:22-224`.
use std::os::raw::c_void;

use oxicuda_blas_b200::{sys, BlasError, BlasHandle, BlasResult, CUdeviceptr};

/// `ParallelismConfig` (`handle.rs:17-60`).
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
pub struct ParallelismConfig { pub tp: usize, pub sp: usize, pub ep: usize }
impl ParallelismConfig { pub fn world_size(&self) -> usize { self.tp * self.sp * self.ep } }

/// `RankCoordinates` / `DistInferHandle` (`handle.rs:62-239`): tp_rank = g % tp, sp_rank = (g / tp) % sp, ep_rank = g / (tp * sp).
#[derive(Debug, Clone)]
pub struct DistInferHandle { pub global_rank: usize, pub config: ParallelismConfig }
impl DistInferHandle {
    pub fn new(global_rank: usize, config: ParallelismConfig) -> BlasResult<Self> {
        if config.tp == 0 || config.sp == 0 || config.ep == 0 { return Err(BlasError::InvalidArgument("parallelism degrees must be >= 1".into())); }
        if global_rank >= config.world_size() { return Err(BlasError::InvalidArgument(format!("rank {global_rank} outside world {}", config.world_size()))); }
        Ok(Self { global_rank, config })
    }
    pub fn tp_rank(&self) -> usize { self.global_rank % self.config.tp }
    pub fn sp_rank(&self) -> usize { (self.global_rank / self.config.tp) % self.config.sp }
    pub fn ep_rank(&self) -> usize { self.global_rank / (self.config.tp * self.config.sp) }
}

/// The library's tensor-parallel group: a `BlasHandle` bound to an NCCL communicator (`ncclComm_t`) of the tp ranks.
pub struct TpGroup<'h> { raw: sys::b2q_tp, handle: &'h BlasHandle, pub tp: usize, pub rank: usize }
impl<'h> TpGroup<'h> {
    /// `nccl_comm` is the caller's `ncclComm_t` (or one made with [`TpGroup::comm_init`]); null for tp = 1.
    pub fn new(handle: &'h BlasHandle, nccl_comm: *mut c_void, dist: &DistInferHandle) -> BlasResult<Self> {
        let mut raw: sys::b2q_tp = std::ptr::null_mut();
        handle.check(unsafe { sys::b2q_tp_create(handle.raw(), nccl_comm, dist.config.tp as i32, dist.tp_rank() as i32, &mut raw) })?;
        Ok(Self { raw, handle, tp: dist.config.tp, rank: dist.tp_rank() })
    }
    /// ncclGetUniqueId on one rank; the 128 bytes travel to the others over any host channel.
    pub fn unique_id() -> BlasResult<[u8; 128]> {
        let mut id = [0u8; 128];
        match unsafe { sys::b2q_tp_unique_id(id.as_mut_ptr()) } { sys::B2Q_OK => Ok(id), st => Err(BlasError::Device(st, "ncclGetUniqueId failed".into())) }
    }
    /// ncclCommInitRank on the current device.
    pub fn comm_init(id: &[u8; 128], tp: usize, rank: usize) -> BlasResult<*mut c_void> {
        let mut comm: *mut c_void = std::ptr::null_mut();
        match unsafe { sys::b2q_tp_comm_init(id.as_ptr(), tp as i32, rank as i32, &mut comm) } {
            sys::B2Q_OK => Ok(comm),
            st => Err(BlasError::Device(st, "ncclCommInitRank failed".into())),
        }
    }
    /// This rank's CUDA IPC handle of its exchange buffer (64 bytes), to be gathered from every rank in rank order ...
    pub fn ipc_handle(&self) -> BlasResult<[u8; 64]> {
        let mut hd = [0u8; 64];
        self.handle.check(unsafe { sys::b2q_tp_exchange_buffer(self.raw, std::ptr::null_mut(), hd.as_mut_ptr()) })?;
        Ok(hd)
    }
    /// ... and handed back here (tp x 64 bytes): enables the peer-memory all-reduce of few-token results.
    pub fn attach_peers(&mut self, handles: &[u8]) -> BlasResult<()> {
        if handles.len() != 64 * self.tp { return Err(BlasError::InvalidArgument(format!("expected {} bytes of IPC handles", 64 * self.tp))); }
        self.handle.check(unsafe { sys::b2q_tp_attach_peers(self.raw, handles.as_ptr(), std::ptr::null()) })
    }
    pub fn raw(&self) -> sys::b2q_tp { self.raw }
    fn check(&self, st: i32) -> BlasResult<()> { self.handle.check(st) }
}
impl Drop for TpGroup<'_> { fn drop(&mut self) { unsafe { sys::b2q_tp_destroy(self.raw); } } }

/// An FP8 (E4M3) weight shard in HBM: codes `[rows x cols]` and one f32 scale per row.
#[derive(Debug, Clone, Copy)]
pub struct Fp8Shard { pub codes: CUdeviceptr, pub scales: CUdeviceptr, pub rows: usize, pub cols: usize }

/// `ColumnLinear` (`column_parallel.rs:103-205`): this rank owns `out / tp` consecutive rows of `W[out x in]`.
pub struct ColumnLinear { pub shard: Fp8Shard, pub bias: Option<CUdeviceptr>, pub total_out: usize }
impl ColumnLinear {
    /// Row range of rank `rank` (`column_parallel.rs:115-166`).
    pub fn shard_rows(out_features: usize, tp: usize, rank: usize) -> BlasResult<(usize, usize)> {
        if out_features % tp != 0 { return Err(BlasError::InvalidDimension(format!("out_features {out_features} not divisible by tp {tp}"))); }
        let lo = out_features / tp;
        Ok((rank * lo, (rank + 1) * lo))
    }
    /// `forward` (`:168-179`) and, with `y_gathered`, `all_gather` (`:181-204`).
    pub fn forward(&self, g: &TpGroup, x_codes: CUdeviceptr, x_scales: CUdeviceptr, tokens: usize, y_local: CUdeviceptr, y_gathered: Option<CUdeviceptr>) -> BlasResult<()> {
        g.check(unsafe {
            sys::b2q_column_linear_forward(g.raw(), x_codes as *const u8, x_scales as *const f32, self.shard.codes as *const u8, self.shard.scales as *const f32,
                                           self.bias.map_or(std::ptr::null(), |b| b as *const f32), tokens as i64, self.shard.cols as i64, self.shard.rows as i64,
                                           y_local as *mut c_void, y_gathered.map_or(std::ptr::null_mut(), |p| p as *mut c_void))
        })
    }
}

/// `RowLinear` (`row_parallel.rs:97-224`): this rank owns `in / tp` consecutive columns of every row; the bias is
/// added on rank 0 only (`:183-190`); `forward` returns the sum over ranks (`all_reduce`, `:202-223`).
pub struct RowLinear { pub shard: Fp8Shard, pub bias: Option<CUdeviceptr> }
impl RowLinear {
    pub fn shard_cols(in_features: usize, tp: usize, rank: usize) -> BlasResult<(usize, usize)> {
        if in_features % tp != 0 { return Err(BlasError::InvalidDimension(format!("in_features {in_features} not divisible by tp {tp}"))); }
        let li = in_features / tp;
        Ok((rank * li, (rank + 1) * li))
    }
    pub fn forward(&self, g: &TpGroup, x_codes: CUdeviceptr, x_scales: CUdeviceptr, tokens: usize, y: CUdeviceptr) -> BlasResult<()> {
        g.check(unsafe {
            sys::b2q_row_linear_forward_allreduce(g.raw(), x_codes as *const u8, x_scales as *const f32, self.shard.codes as *const u8,
                                                  self.shard.scales as *const f32, self.bias.map_or(std::ptr::null(), |b| b as *const f32), tokens as i64,
                                                  self.shard.cols as i64, self.shard.rows as i64, y as *mut c_void)
        })
    }
}

/// SwiGLU MLP over a column-parallel gate | up shard `[2 * ffn / tp x hidden]` and a row-parallel down shard
/// `[hidden x ffn / tp]` (`SwiGluExpert::forward`, `crates/oxicuda-moe/src/expert/ffn.rs:208-243`).
pub struct TpFp8Mlp { pub gate_up: Fp8Shard, pub down: Fp8Shard }
impl TpFp8Mlp {
    pub fn forward(&self, g: &TpGroup, x_bf16: CUdeviceptr, tokens: usize, y_bf16: CUdeviceptr) -> BlasResult<()> {
        let hidden = self.gate_up.cols;
        let ffn_local = self.gate_up.rows / 2;
        g.check(unsafe {
            sys::b2q_mlp_swiglu_fp8_forward(g.raw(), x_bf16 as *const c_void, self.gate_up.codes as *const u8, self.gate_up.scales as *const f32,
                                            self.down.codes as *const u8, self.down.scales as *const f32, tokens as i64, hidden as i64, ffn_local as i64,
                                            sys::B2Q_ROUND_RNE, y_bf16 as *mut c_void)
        })
    }
}
