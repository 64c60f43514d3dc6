//! Rust binding of the B200 GEMM library (`include/patina_gemm.h`, `libpatina_gemm.so`).
//!
//! Where it goes: `crates/patina/src/gemm.rs`, behind `feature = "cuda"` like `run.rs`; the
//! crate's `build.rs` gains `println!("cargo:rustc-link-lib=dylib=patina_gemm")` and a search
//! path. It replaces the launch half of `run::run_gemm` (crates/patina/src/run.rs:462-529): the
//! caller keeps its device buffers, this module enqueues the GEMM on them.
//!
//! Style follows the crate's existing FFI (crates/patina/src/ffi.rs:11-87): a raw `extern "C"`
//! block that mirrors the header declaration for declaration, an owning handle with `Drop`,
//! heap strings taken and freed in one place, `Result<_, String>` everywhere.
//!
//! The image this library is built in has no Rust toolchain: this file is source text, kept in
//! step with the header by `tests/test_bindings.py` (every exported function, its argument
//! count, and every struct's field list must match), but it has not been compiled.

use std::ffi::{c_char, c_void, CStr};

/// Opaque context (one per device).
#[repr(C)]
pub struct PatinaGemmContext {
    _private: [u8; 0],
}

pub const PATINA_GEMM_OK: i32 = 0;
pub const PATINA_GEMM_ERR_INVALID_ARG: i32 = 1;
pub const PATINA_GEMM_ERR_UNSUPPORTED_ARCH: i32 = 2;
pub const PATINA_GEMM_ERR_CUDA: i32 = 3;
pub const PATINA_GEMM_ERR_TIMEOUT: i32 = 4;

pub const PATINA_IN_F16: i32 = 0;
pub const PATINA_IN_BF16: i32 = 1;
pub const PATINA_IN_E4M3: i32 = 2;
pub const PATINA_IN_MXE4M3: i32 = 3;
pub const PATINA_OUT_BF16: i32 = 0;
pub const PATINA_OUT_F32: i32 = 1;
pub const PATINA_OUT_E4M3: i32 = 2;

pub const PATINA_GEMM_NOALLOC_PARTIAL_BYTES: usize = 16 * 1024 * 1024;

#[repr(C)]
#[derive(Clone, Copy)]
pub struct PatinaGemmConfig {
    pub cta_group: i32,
    pub block_n: i32,
    pub stages: i32,
    pub group_m: i32,
    pub max_ctas: i32,
    pub m_sub: i32,
    pub stream_k: i32,
    pub cluster_k: i32,
    pub k_order: i32,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct PatinaGemmPlan {
    pub cta_group: i32,
    pub block_n: i32,
    pub stages: i32,
    pub group_m: i32,
    pub m_sub: i32,
    pub tile_m: u32,
    pub tiles_m: u32,
    pub tiles_n: u32,
    pub num_tiles: u32,
    pub k_blocks: u32,
    pub grid: u32,
    pub block: u32,
    pub cluster: u32,
    pub smem_bytes: u32,
    pub tmem_cols: u32,
    pub stage_bytes: u32,
    pub expect_tx_bytes: u32,
    pub idesc: u32,
    pub half_tiles: u32,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct PatinaGemmEpilogue {
    pub bias: *const c_void,
    pub residual: *const c_void,
    pub ldr: i64,
    pub beta: f32,
    pub activation: i32,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct PatinaStreamKPlan {
    pub grid: u32,
    pub tiles: u32,
    pub k_blocks: u32,
    pub m_pad: u32,
    pub max_contrib: u32,
    pub stages: u32,
    pub smem_bytes: u32,
    pub units: u64,
    pub partial_bytes: u64,
    pub counter_bytes: u64,
}

#[link(name = "patina_gemm")]
extern "C" {
    pub fn patina_gemm_context_create(device: i32, out: *mut *mut PatinaGemmContext) -> i32;
    pub fn patina_gemm_context_destroy(ctx: *mut PatinaGemmContext);
    pub fn patina_gemm_last_error(ctx: *mut PatinaGemmContext) -> *mut c_char;
    pub fn patina_gemm_string_free(s: *mut c_char);
    pub fn patina_gemm_set_wait_limit_ns(ctx: *mut PatinaGemmContext, ns: u64) -> i32;
    pub fn patina_gemm_status(ctx: *mut PatinaGemmContext, stream: *mut c_void) -> i32;
    pub fn patina_gemm_launch_count(ctx: *mut PatinaGemmContext) -> u64;
    pub fn patina_gemm_bf16_tn(ctx: *mut PatinaGemmContext, a: *const c_void, lda: i64, b: *const c_void,
        ldb: i64, c: *mut c_void, ldc: i64, m: i64, n: i64, k: i64, alpha: f32, stream: *mut c_void) -> i32;
    pub fn patina_gemm_fp8e4m3_tn(ctx: *mut PatinaGemmContext, a: *const c_void, lda: i64, b: *const c_void,
        ldb: i64, c: *mut c_void, ldc: i64, m: i64, n: i64, k: i64, scale_a: f32, scale_b: f32, stream: *mut
        c_void) -> i32;
    pub fn patina_gemm_f16_tn_f32out(ctx: *mut PatinaGemmContext, a: *const c_void, lda: i64, b: *const
        c_void, ldb: i64, c: *mut c_void, ldc: i64, m: i64, n: i64, k: i64, alpha: f32, stream: *mut c_void)
        -> i32;
    pub fn patina_gemm_ex(ctx: *mut PatinaGemmContext, in_type: i32, out_type: i32, a: *const c_void, lda:
        i64, b: *const c_void, ldb: i64, c: *mut c_void, ldc: i64, m: i64, n: i64, k: i64, alpha: f32, cfg:
        *const PatinaGemmConfig, stream: *mut c_void) -> i32;
    pub fn patina_gemm_bf16_tn_fused(ctx: *mut PatinaGemmContext, a: *const c_void, lda: i64, b: *const
        c_void, ldb: i64, c: *mut c_void, ldc: i64, m: i64, n: i64, k: i64, alpha: f32, epi: *const
        PatinaGemmEpilogue, stream: *mut c_void) -> i32;
    pub fn patina_gemm_bf16_tn_fused_fp8out(ctx: *mut PatinaGemmContext, a: *const c_void, lda: i64, b:
        *const c_void, ldb: i64, c: *mut c_void, ldc: i64, m: i64, n: i64, k: i64, alpha: f32, epi: *const
        PatinaGemmEpilogue, out_scale: f32, amax: *mut f32, stream: *mut c_void) -> i32;
    pub fn patina_gemm_bf16_tn_scatter(ctx: *mut PatinaGemmContext, a: *const c_void, lda: i64, b: *const
        c_void, ldb: i64, c_dests: *const *mut c_void, n_dests: i32, ldc: i64, m: i64, n: i64, k: i64,
        alpha: f32, stream: *mut c_void) -> i32;
    pub fn patina_gemm_bf16_tn_grouped(ctx: *mut PatinaGemmContext, a: *const c_void, lda: i64, b: *const
        c_void, ldb: i64, c: *mut c_void, ldc: i64, group_rows: *const i32, n_groups: i32, total_rows: i64,
        n: i64, k: i64, alpha: f32, config: *const PatinaGemmConfig, stream: *mut c_void) -> i32;
    pub fn patina_gemm_fp8e4m3_tn_grouped(ctx: *mut PatinaGemmContext, a: *const c_void, lda: i64, b: *const
        c_void, ldb: i64, c: *mut c_void, ldc: i64, group_rows: *const i32, n_groups: i32, total_rows: i64,
        n: i64, k: i64, scale_a: f32, group_scale_b: *const f32, config: *const PatinaGemmConfig, stream:
        *mut c_void) -> i32;
    pub fn patina_gemm_mxfp8_tn(ctx: *mut PatinaGemmContext, a: *const c_void, lda: i64, scales_a: *const
        c_void, b: *const c_void, ldb: i64, scales_b: *const c_void, c: *mut c_void, ldc: i64, m: i64, n:
        i64, k: i64, alpha: f32, config: *const PatinaGemmConfig, stream: *mut c_void) -> i32;
    pub fn patina_gemm_mx_scale_bytes(rows: i64, k: i64) -> u64;
    pub fn patina_gemm_mx_scale_offset(row: i64, k_block32: i64, k: i64) -> u64;
    pub fn patina_gemm_column_shard(n: i64, world: i32, rank: i32, n0: *mut i64, n1: *mut i64);
    pub fn patina_gemm_sharded_bf16_tn(ctxs: *const *mut PatinaGemmContext, n_shards: i32,
        a: *const *const c_void, lda: i64, b_shards: *const *const c_void, ldb: i64,
        c_shards: *const *mut c_void, ldc: i64, m: i64, n: i64, k: i64, alpha: f32,
        streams: *const *mut c_void) -> i32;
    pub fn patina_gemm_peer_alloc(ctx: *mut PatinaGemmContext, bytes: usize, ptr: *mut *mut c_void,
        handle_out: *mut u8) -> i32;
    pub fn patina_gemm_peer_open(ctx: *mut PatinaGemmContext, handle: *const u8, ptr: *mut *mut c_void) ->
        i32;
    pub fn patina_gemm_peer_close(ctx: *mut PatinaGemmContext, ptr: *mut c_void) -> i32;
    pub fn patina_gemm_peer_free(ctx: *mut PatinaGemmContext, ptr: *mut c_void) -> i32;
    pub fn patina_gemm_host(ctx: *mut PatinaGemmContext, in_type: i32, out_type: i32, hosta: *const c_void,
        lda: i64, hostb: *const c_void, ldb: i64, hostc: *mut c_void, ldc: i64, m: i64, n: i64, k: i64,
        alpha: f32, cfg: *const PatinaGemmConfig, stream: *mut c_void) -> i32;
    pub fn patina_gemm_bf16_tn_skinny_noalloc(a: *const c_void, lda: i64, b: *const c_void, ldb: i64, c:
        *mut c_void, ldc: i64, m: i64, n: i64, k: i64, alpha: f32, stream: *mut c_void, err_buf: *mut
        c_char, err_buf_len: usize) -> i32;
    pub fn patina_gemm_validate(in_type: i32, out_type: i32, a: *const c_void, lda: i64, b: *const c_void,
        ldb: i64, c: *const c_void, ldc: i64, m: i64, n: i64, k: i64, err_out: *mut *mut c_char) -> i32;
    pub fn patina_gemm_plan(in_type: i32, out_type: i32, m: i64, n: i64, k: i64, cfg: *const
        PatinaGemmConfig, num_sms: i32, out: *mut PatinaGemmPlan) -> i32;
    pub fn patina_gemm_streamk_plan(in_type: i32, m: i64, n: i64, k: i64, num_sms: i32, out: *mut
        PatinaStreamKPlan) -> i32;
    pub fn patina_gemm_streamk_range(cta: u64, units: u64, parts: u64, begin: *mut u64, end: *mut u64);
    pub fn patina_gemm_streamk_chosen(in_type: i32, out_type: i32, m: i64, n: i64, k: i64, num_sms: i32) ->
        i32;
    pub fn patina_gemm_cluster_k_chosen(in_type: i32, out_type: i32, m: i64, n: i64, k: i64, num_sms: i32) -> i32;
    pub fn patina_gemm_streamk_owner(unit: u64, units: u64, parts: u64) -> u32;
    pub fn patina_gemm_smem_desc(smem_addr: u32, lbo_bytes: u32, sbo_bytes: u32, swizzle_code: i32) -> u64;
    pub fn patina_gemm_idesc(in_type: i32, umma_m: u32, umma_n: u32) -> u32;
    pub fn patina_gemm_idesc_mx(umma_m: u32, umma_n: u32, a_sf_id: u32, b_sf_id: u32) -> u32;
    pub fn patina_gemm_k_advance_units(k_elems: u32, in_type: i32) -> u32;
    pub fn patina_gemm_tmem_lane_offset(warp_quarter: u32) -> u32;
    pub fn patina_gemm_tile_coord(t: u32, tiles_m: u32, tiles_n: u32, group_m: u32, m_block: *mut u32,
        n_block: *mut u32);
    pub fn patina_gemm_version() -> *const c_char;
}

impl Default for PatinaGemmConfig {
    /// All zero: "choose for me" in every field.
    fn default() -> Self {
        PatinaGemmConfig { cta_group: 0, block_n: 0, stages: 0, group_m: 0, max_ctas: 0, m_sub: 0, stream_k: 0,
                           cluster_k: 0, k_order: 0 }
    }
}

/// Element types of the operands.
#[derive(Clone, Copy, PartialEq, Eq, Debug)]
pub enum InType {
    F16 = 0,
    Bf16 = 1,
    E4m3 = 2,
}

/// A device matrix the caller owns: pointer, rows, columns, leading dimension in elements.
#[derive(Clone, Copy)]
pub struct DeviceMatrix {
    pub ptr: *mut c_void,
    pub rows: i64,
    pub cols: i64,
    pub ld: i64,
}

/// Owning handle of a `PatinaGemmContext` (counterpart of `run::Cuda`, run.rs:246-394).
pub struct Gemm {
    raw: *mut PatinaGemmContext,
}

/// Copy a heap string returned by the library and free it (ffi.rs `take_string`).
unsafe fn take_string(s: *mut c_char) -> Option<String> {
    if s.is_null() {
        return None;
    }
    let owned = CStr::from_ptr(s).to_string_lossy().into_owned();
    patina_gemm_string_free(s);
    Some(owned)
}

impl Gemm {
    /// One context per device. `Err` names the reason; a device that is not sm_100 gives the
    /// same message `run_gemm` gives before it touches any PTX (run.rs:476-481).
    pub fn new(device: i32) -> Result<Gemm, String> {
        let mut raw = std::ptr::null_mut();
        match unsafe { patina_gemm_context_create(device, &mut raw) } {
            PATINA_GEMM_OK => Ok(Gemm { raw }),
            PATINA_GEMM_ERR_UNSUPPORTED_ARCH => Err("device is not sm_100a; tcgen05 needs Blackwell".into()),
            rc => Err(format!("patina_gemm_context_create failed ({rc})")),
        }
    }

    fn check(&self, rc: i32) -> Result<(), String> {
        if rc == PATINA_GEMM_OK {
            return Ok(());
        }
        let msg = unsafe { take_string(patina_gemm_last_error(self.raw)) };
        Err(msg.unwrap_or_else(|| format!("patina_gemm error {rc}")))
    }

    /// C[M,N] = alpha * A[M,K] * B[N,K]^T, bf16 in, bf16 out, enqueued on `stream`.
    pub fn bf16_tn(&self, a: DeviceMatrix, b: DeviceMatrix, c: DeviceMatrix, alpha: f32,
                   stream: *mut c_void) -> Result<(), String> {
        if a.cols != b.cols || c.rows != a.rows || c.cols != b.rows {
            return Err("shapes do not agree: A is [M,K], B is [N,K], C is [M,N]".into());
        }
        let rc = unsafe {
            patina_gemm_bf16_tn(self.raw, a.ptr, a.ld, b.ptr, b.ld, c.ptr, c.ld, a.rows, b.rows, a.cols, alpha, stream)
        };
        self.check(rc)
    }

    /// The reference kernel's own types: f16 in, f32 out (harness/gemm_check.cpp:9-10).
    pub fn f16_tn_f32out(&self, a: DeviceMatrix, b: DeviceMatrix, c: DeviceMatrix, alpha: f32,
                         stream: *mut c_void) -> Result<(), String> {
        let rc = unsafe {
            patina_gemm_f16_tn_f32out(self.raw, a.ptr, a.ld, b.ptr, b.ld, c.ptr, c.ld, a.rows, b.rows, a.cols, alpha,
                                      stream)
        };
        self.check(rc)
    }

    /// fp8 e4m3 in, bf16 out scaled by `scale_a * scale_b`.
    pub fn fp8e4m3_tn(&self, a: DeviceMatrix, b: DeviceMatrix, c: DeviceMatrix, scale_a: f32, scale_b: f32,
                      stream: *mut c_void) -> Result<(), String> {
        let rc = unsafe {
            patina_gemm_fp8e4m3_tn(self.raw, a.ptr, a.ld, b.ptr, b.ld, c.ptr, c.ld, a.rows, b.rows, a.cols, scale_a,
                                   scale_b, stream)
        };
        self.check(rc)
    }

    /// Block-scaled fp8: one E8M0 scale per 32 K elements of a row, scale buffers in the atom
    /// layout the header describes.
    pub fn mxfp8_tn(&self, a: DeviceMatrix, scales_a: *const c_void, b: DeviceMatrix, scales_b: *const c_void,
                    c: DeviceMatrix, alpha: f32, stream: *mut c_void) -> Result<(), String> {
        let rc = unsafe {
            patina_gemm_mxfp8_tn(self.raw, a.ptr, a.ld, scales_a, b.ptr, b.ld, scales_b, c.ptr, c.ld, a.rows, b.rows,
                                 a.cols, alpha, std::ptr::null(), stream)
        };
        self.check(rc)
    }

    /// Any type pair with an explicit tile configuration.
    pub fn gemm_ex(&self, in_type: InType, out_type: i32, a: DeviceMatrix, b: DeviceMatrix, c: DeviceMatrix,
                   alpha: f32, cfg: Option<&PatinaGemmConfig>, stream: *mut c_void) -> Result<(), String> {
        let cfg_ptr = cfg.map_or(std::ptr::null(), |c| c as *const PatinaGemmConfig);
        let rc = unsafe {
            patina_gemm_ex(self.raw, in_type as i32, out_type, a.ptr, a.ld, b.ptr, b.ld, c.ptr, c.ld, a.rows, b.rows,
                           a.cols, alpha, cfg_ptr, stream)
        };
        self.check(rc)
    }

    /// bias / residual / activation applied to the fp32 accumulator before the one rounding.
    pub fn bf16_tn_fused(&self, a: DeviceMatrix, b: DeviceMatrix, c: DeviceMatrix, alpha: f32,
                         epi: &PatinaGemmEpilogue, stream: *mut c_void) -> Result<(), String> {
        let rc = unsafe {
            patina_gemm_bf16_tn_fused(self.raw, a.ptr, a.ld, b.ptr, b.ld, c.ptr, c.ld, a.rows, b.rows, a.cols, alpha,
                                      epi as *const PatinaGemmEpilogue, stream)
        };
        self.check(rc)
    }

    /// Ragged groups that share N and K in one launch; `group_rows` is a DEVICE array.
    pub fn bf16_tn_grouped(&self, a: DeviceMatrix, b: DeviceMatrix, c: DeviceMatrix, group_rows: *const i32,
                           n_groups: i32, n: i64, alpha: f32, stream: *mut c_void) -> Result<(), String> {
        let rc = unsafe {
            patina_gemm_bf16_tn_grouped(self.raw, a.ptr, a.ld, b.ptr, b.ld, c.ptr, c.ld, group_rows, n_groups, a.rows,
                                        n, a.cols, alpha, std::ptr::null(), stream)
        };
        self.check(rc)
    }

    /// The same GEMM stored to several destinations (column-shard scatter over NVLink).
    pub fn bf16_tn_scatter(&self, a: DeviceMatrix, b: DeviceMatrix, dests: &[*mut c_void], ldc: i64, alpha: f32,
                           stream: *mut c_void) -> Result<(), String> {
        let rc = unsafe {
            patina_gemm_bf16_tn_scatter(self.raw, a.ptr, a.ld, b.ptr, b.ld, dests.as_ptr(), dests.len() as i32, ldc,
                                        a.rows, b.rows, a.cols, alpha, stream)
        };
        self.check(rc)
    }

    /// Host buffers in and out: the whole of `run::run_gemm` (run.rs:484-528) in one call.
    pub fn host(&self, in_type: InType, out_type: i32, a: *const c_void, lda: i64, b: *const c_void, ldb: i64,
                c: *mut c_void, ldc: i64, m: i64, n: i64, k: i64, alpha: f32, stream: *mut c_void)
                -> Result<(), String> {
        let rc = unsafe {
            patina_gemm_host(self.raw, in_type as i32, out_type, a, lda, b, ldb, c, ldc, m, n, k, alpha,
                             std::ptr::null(), stream)
        };
        self.check(rc)
    }

    /// Synchronise `stream`; `Err` if a device-side wait ran out (the reference's waits are
    /// unbounded spins, v2_gemm_pipelined.ptx:111-113).
    pub fn status(&self, stream: *mut c_void) -> Result<(), String> {
        let rc = unsafe { patina_gemm_status(self.raw, stream) };
        self.check(rc)
    }

    pub fn set_wait_limit_ns(&self, ns: u64) -> Result<(), String> {
        let rc = unsafe { patina_gemm_set_wait_limit_ns(self.raw, ns) };
        self.check(rc)
    }

    pub fn launch_count(&self) -> u64 {
        unsafe { patina_gemm_launch_count(self.raw) }
    }

    /// Device memory that other processes of the node can map (CUDA IPC), for the scatter.
    pub fn peer_alloc(&self, bytes: usize) -> Result<(*mut c_void, [u8; 64]), String> {
        let mut ptr = std::ptr::null_mut();
        let mut handle = [0u8; 64];
        let rc = unsafe { patina_gemm_peer_alloc(self.raw, bytes, &mut ptr, handle.as_mut_ptr()) };
        self.check(rc).map(|_| (ptr, handle))
    }

    pub fn peer_open(&self, handle: &[u8; 64]) -> Result<*mut c_void, String> {
        let mut ptr = std::ptr::null_mut();
        let rc = unsafe { patina_gemm_peer_open(self.raw, handle.as_ptr(), &mut ptr) };
        self.check(rc).map(|_| ptr)
    }

    pub fn peer_close(&self, ptr: *mut c_void) -> Result<(), String> {
        let rc = unsafe { patina_gemm_peer_close(self.raw, ptr) };
        self.check(rc)
    }

    pub fn peer_free(&self, ptr: *mut c_void) -> Result<(), String> {
        let rc = unsafe { patina_gemm_peer_free(self.raw, ptr) };
        self.check(rc)
    }
}

impl Drop for Gemm {
    fn drop(&mut self) {
        unsafe { patina_gemm_context_destroy(self.raw) }
    }
}

/// Shard `rank` of `world`: its columns [n0, n1) of an N-wide problem.
pub fn column_shard(n: i64, world: i32, rank: i32) -> (i64, i64) {
    let (mut n0, mut n1) = (0i64, 0i64);
    unsafe { patina_gemm_column_shard(n, world, rank, &mut n0, &mut n1) };
    (n0, n1)
}

/// The skinny GEMM (1 <= M <= 128) that allocates nothing: no context, fixed scratch inside the
/// library, on the current device. Make the first call per device a start-up warm-up.
pub fn bf16_tn_skinny_noalloc(a: DeviceMatrix, b: DeviceMatrix, c: DeviceMatrix, alpha: f32,
                              stream: *mut c_void) -> Result<(), String> {
    let mut err = [0u8; 256];
    let rc = unsafe {
        patina_gemm_bf16_tn_skinny_noalloc(a.ptr, a.ld, b.ptr, b.ld, c.ptr, c.ld, a.rows, b.rows, a.cols, alpha,
                                           stream, err.as_mut_ptr() as *mut c_char, err.len())
    };
    if rc == PATINA_GEMM_OK {
        return Ok(());
    }
    let end = err.iter().position(|&ch| ch == 0).unwrap_or(err.len());
    Err(String::from_utf8_lossy(&err[..end]).into_owned())
}

/// What a call would launch, computed on the host (no device needed).
pub fn plan(in_type: InType, out_type: i32, m: i64, n: i64, k: i64, cfg: Option<&PatinaGemmConfig>,
            num_sms: i32) -> Result<PatinaGemmPlan, String> {
    let mut out: PatinaGemmPlan = unsafe { std::mem::zeroed() };
    let cfg_ptr = cfg.map_or(std::ptr::null(), |c| c as *const PatinaGemmConfig);
    match unsafe { patina_gemm_plan(in_type as i32, out_type, m, n, k, cfg_ptr, num_sms, &mut out) } {
        PATINA_GEMM_OK => Ok(out),
        rc => Err(format!("patina_gemm_plan failed ({rc})")),
    }
}

/// The argument check every entry point runs; `Err` carries the library's diagnostic.
pub fn validate(in_type: InType, out_type: i32, a: DeviceMatrix, b: DeviceMatrix, c: DeviceMatrix)
                -> Result<(), String> {
    let mut err: *mut c_char = std::ptr::null_mut();
    let rc = unsafe {
        patina_gemm_validate(in_type as i32, out_type, a.ptr, a.ld, b.ptr, b.ld, c.ptr, c.ld, a.rows, b.rows, a.cols,
                             &mut err)
    };
    if rc == PATINA_GEMM_OK {
        Ok(())
    } else {
        Err(unsafe { take_string(err) }.unwrap_or_else(|| format!("error {rc}")))
    }
}

pub fn version() -> String {
    unsafe { CStr::from_ptr(patina_gemm_version()) }.to_string_lossy().into_owned()
}
