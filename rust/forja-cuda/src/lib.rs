//! `forja-cuda`: `forja_core::Backend` for NVIDIA B200 (sm_100a), a thin shim over the C ABI of
//! `libforja_cuda.so` (`include/forja_cuda.h`).
//!
//! NOT COMPILED IN THIS REPOSITORY'S BUILD IMAGE: there is no Rust toolchain there. The file is
//! written against the trait as it stands in `crates/forja-core/src/backend.rs:606-984` and the
//! CPU backend's implementation of it (`crates/forja-cpu/src/lib.rs:1334-1516`); the same call
//! sequence is exercised from Python by the repository's GPU tests. A maintainer adds the crate to
//! the workspace, a `Cuda` arm next to `NativeDevice::{Cpu, Metal}`
//! (`crates/forja-sdk/src/lib.rs:190-203`) and one in `crates/forja/src/verify.rs:242` /
//! `crates/forja/src/engine.rs:354`.
//!
//! Everything that is pure layout arithmetic stays in Rust (`view`, `tensor`): only descriptors
//! cross the boundary. Storage lives in the library's registry; this side keeps forja's own
//! `AllocationRegistry` so that handles are validated exactly as on the other backends.

#![allow(unsafe_code)]

use std::{
    ffi::c_void,
    ops::Range,
    sync::Mutex,
    time::Duration,
};

use forja_core::{
    AllocationRegistry, Backend, BackendError, BufferId, CommandList, CompletionResource, DType,
    DeviceInfo, Dispatch, KernelSignature, Layout, MappedRegion, MemoryUsage, Op,
    PagedCopyDirection, PreparedGraph, ReadonlyImport, Submission, SubmissionProfile, Tensor,
    ValidatedProgram, ViewOp,
};

// ---- the C ABI (include/forja_cuda.h) ------------------------------------------------------

#[repr(C)]
#[derive(Clone, Copy)]
struct FjTensor {
    buffer: u64,
    dtype: u32,
    rank: u32,
    offset: u64,
    shape: [u32; 8],
    strides: [u64; 8],
}

#[repr(C)]
struct FjDispatch {
    op: u32,
    n_inputs: u32,
    n_outputs: u32,
    u0: u32,
    u1: u32,
    u2: u32,
    u3: u32,
    f0: f32,
    program: u64,
    inputs: *const FjTensor,
    outputs: *const FjTensor,
}

#[repr(C)]
#[derive(Default)]
struct FjDeviceError {
    submission: u64,
    dispatch: u32,
    op: u32,
    flag: u32,
    value: u32,
    code: i64,
}

#[link(name = "forja_cuda")]
unsafe extern "C" {
    fn fj_backend_create(device: i32, memory_limit: u64, out: *mut *mut c_void) -> i32;
    fn fj_backend_destroy(be: *mut c_void);
    fn fj_set_memory_limit(be: *mut c_void, bytes: u64) -> i32;
    fn fj_memory_usage(be: *mut c_void, used: *mut u64, limit: *mut u64) -> i32;
    fn fj_alloc(be: *mut c_void, bytes: u64, buffer: *mut u64) -> i32;
    fn fj_import_readonly(be: *mut c_void, host: *const u8, bytes: u64, buffer: *mut u64) -> i32;
    fn fj_release(be: *mut c_void, buffer: u64) -> i32;
    fn fj_write(be: *mut c_void, buffer: u64, byte_offset: u64, src: *const u8, len: u64) -> i32;
    fn fj_read(be: *mut c_void, buffer: u64, byte_offset: u64, dst: *mut u8, len: u64) -> i32;
    fn fj_read_strided(be: *mut c_void, view: *const FjTensor, dst: *mut u8) -> i32;
    fn fj_program_prepare(
        be: *mut c_void,
        kind: u32,
        insts: *const u32,
        n_insts: u32,
        outputs: *const u32,
        n_outputs: u32,
        handle: *mut u64,
    ) -> i32;
    fn fj_submit(
        be: *mut c_void,
        dispatches: *const FjDispatch,
        count: u32,
        profiled: u32,
        out: *mut *mut c_void,
    ) -> i32;
    fn fj_sub_wait(sub: *mut c_void, timeout_ns: u64) -> i32;
    fn fj_sub_gpu_time_ns(sub: *mut c_void, ns: *mut u64) -> i32;
    fn fj_sub_completion_serial(sub: *mut c_void) -> u64;
    fn fj_sub_error(sub: *mut c_void, out: *mut FjDeviceError) -> i32;
    fn fj_sub_destroy(sub: *mut c_void);
}

const FJ_OK: i32 = 0;

/// `fj_status` -> `BackendError` (same variants, `crates/forja-core/src/backend.rs:362-426`).
fn check(status: i32) -> Result<(), BackendError> {
    match status {
        FJ_OK => Ok(()),
        1 => Err(BackendError::QuotaExceeded),
        2 => Err(BackendError::AllocationFailed),
        3 => Err(BackendError::ExecutionFailed),
        6 => Err(BackendError::Timeout),
        7 => Err(BackendError::InvalidInput),
        8 => Err(BackendError::UnsupportedOperation),
        _ => Err(BackendError::ExecutionFailed),
    }
}

fn dtype_code(dtype: DType) -> u32 {
    match dtype {
        DType::F32 => 0,
        DType::F16 => 1,
        DType::BF16 => 2,
        DType::I32 => 3,
        DType::U32 => 4,
    }
}

fn lower_tensor(tensor: &Tensor) -> Result<FjTensor, BackendError> {
    let layout = tensor.layout();
    let (shape, strides) = (layout.shape(), layout.strides());
    if shape.len() > 8 {
        return Err(BackendError::InvalidInput);
    }
    let mut out = FjTensor {
        buffer: tensor.buffer().allocation(),
        dtype: dtype_code(layout.dtype()),
        rank: shape.len() as u32,
        offset: layout.offset(),
        shape: [0; 8],
        strides: [0; 8],
    };
    out.shape[..shape.len()].copy_from_slice(shape);
    out.strides[..strides.len()].copy_from_slice(strides);
    Ok(out)
}

/// `Op` -> (`fj_op`, u0, u1, u2, u3, f0); operand orders are the reference's own.
fn lower_op(op: Op) -> Result<(u32, [u32; 4], f32), BackendError> {
    Ok(match op {
        Op::Program(_) => (1, [0; 4], 0.0),
        Op::Copy => (2, [0; 4], 0.0),
        Op::PagedCopy { direction, start, page_tokens } => {
            let out_of_pages = matches!(direction, PagedCopyDirection::OutOfPages) as u32;
            (3, [out_of_pages, start, page_tokens, 0], 0.0)
        }
        Op::RmsNorm { eps } => (4, [0; 4], eps),
        Op::Argmax { .. } => (5, [0; 4], 0.0),
        Op::TopK { k, normalize, .. } => (6, [k, normalize as u32, 0, 0], 0.0),
        Op::Rope { theta } => (7, [0; 4], theta),
        Op::Embed => (8, [0; 4], 0.0),
        Op::QuantEmbed { bits, group_size } => (9, [bits.into(), group_size, 0, 0], 0.0),
        Op::Matmul => (10, [0; 4], 0.0),
        Op::QuantMatmul { bits, group_size } => (11, [bits.into(), group_size, 0, 0], 0.0),
        Op::GatherQuantMatmul { bits, group_size } => (12, [bits.into(), group_size, 0, 0], 0.0),
        Op::PagedSdpa { scale, causal, q_start, key_length, page_tokens } => {
            (13, [causal as u32, q_start, key_length, page_tokens], scale)
        }
        Op::PagedSdpaAppend { scale, q_start, page_tokens } => (14, [0, q_start, 0, page_tokens], scale),
        Op::Sdpa { scale, causal, q_start } => (15, [causal as u32, q_start, 0, 0], scale),
        Op::Sample { position, .. } | Op::SampleMasked { position, .. } => (16, [position, 0, 0, 0], 0.0),
        Op::GatherMatmul => (17, [0; 4], 0.0),
        Op::State(_) => return Err(BackendError::UnsupportedOperation),
    })
}

/// The library handle; `Send + Sync` because the library serialises calls on its own mutex
/// (the reference CPU backend does the same, `crates/forja-cpu/src/lib.rs:22-24`).
struct Raw(*mut c_void);
unsafe impl Send for Raw {}
unsafe impl Sync for Raw {}

/// forja backend for one B200.
pub struct CudaBackend {
    raw: Raw,
    registry: Mutex<AllocationRegistry>,
}

impl CudaBackend {
    /// Opens CUDA device `device`. There is no fallback: without a usable device this fails.
    ///
    /// # Errors
    /// `AllocationFailed` when the device or the library cannot be opened.
    pub fn new(device: i32) -> Result<Self, BackendError> {
        let mut raw = std::ptr::null_mut();
        check(unsafe { fj_backend_create(device, 0, &mut raw) })?;
        Ok(Self { raw: Raw(raw), registry: Mutex::new(AllocationRegistry::new()) })
    }

    fn registry(&self) -> Result<std::sync::MutexGuard<'_, AllocationRegistry>, BackendError> {
        self.registry.lock().map_err(|_| BackendError::ExecutionFailed)
    }

    fn lower_and_submit(&self, commands: CommandList, profiled: bool) -> Result<CudaSubmission, BackendError> {
        let dispatches = commands.into_dispatches();
        // tensors first, so that the pointers in FjDispatch stay valid until fj_submit returns
        let mut tensors: Vec<(Vec<FjTensor>, Vec<FjTensor>)> = Vec::with_capacity(dispatches.len());
        for dispatch in &dispatches {
            let inputs = dispatch.inputs().iter().map(lower_tensor).collect::<Result<Vec<_>, _>>()?;
            let outputs = dispatch.outputs().iter().map(lower_tensor).collect::<Result<Vec<_>, _>>()?;
            tensors.push((inputs, outputs));
        }
        let lowered = dispatches
            .iter()
            .zip(&tensors)
            .map(|(dispatch, (inputs, outputs))| {
                let (op, u, f0) = lower_op(dispatch.op())?;
                Ok(FjDispatch {
                    op,
                    n_inputs: inputs.len() as u32,
                    n_outputs: outputs.len() as u32,
                    u0: u[0],
                    u1: u[1],
                    u2: u[2],
                    u3: u[3],
                    f0,
                    program: program_handle(dispatch),
                    inputs: inputs.as_ptr(),
                    outputs: outputs.as_ptr(),
                })
            })
            .collect::<Result<Vec<_>, BackendError>>()?;
        let mut sub = std::ptr::null_mut();
        check(unsafe { fj_submit(self.raw.0, lowered.as_ptr(), lowered.len() as u32, profiled as u32, &mut sub) })?;
        Ok(CudaSubmission { raw: Raw(sub), owners: Mutex::new(Vec::new()) })
    }
}

/// The handle `prepare_program` returned for the dispatch's bound program or epilogue, else 0.
fn program_handle(dispatch: &Dispatch) -> u64 {
    dispatch
        .bound_program()
        .and_then(|program| program.backend_handle::<u64>().copied())
        .or_else(|| dispatch.prepared_epilogue().and_then(|epilogue| epilogue.backend_handle::<u64>().copied()))
        .unwrap_or(0)
}

impl Drop for CudaBackend {
    fn drop(&mut self) {
        unsafe { fj_backend_destroy(self.raw.0) };
    }
}

/// A submission in flight on the backend's stream.
pub struct CudaSubmission {
    raw: Raw,
    /// `CompletionResource`s stay alive until physical completion, also across caller timeouts
    /// (`crates/forja-core/src/backend.rs:14-26, 785-796`): they are dropped by `wait` once the
    /// library reports completion, or with the submission (whose destroy call waits for the device).
    owners: Mutex<Vec<CompletionResource>>,
}

impl CudaSubmission {
    fn finish(&self, status: i32) -> Result<(), BackendError> {
        if status != 6 {
            if let Ok(mut owners) = self.owners.lock() {
                owners.clear();
            }
        }
        match status {
            4 | 5 | 9 => {
                let mut error = FjDeviceError::default();
                unsafe { fj_sub_error(self.raw.0, &mut error) };
                Err(match status {
                    4 => BackendError::DeviceExecutionFailed { submission: error.submission, code: error.code },
                    5 => BackendError::DeviceErrorFlag {
                        submission: error.submission,
                        dispatch: error.dispatch,
                        operation: error.op,
                        flag: error.flag,
                        value: error.value,
                    },
                    _ => BackendError::IndexOutOfRange { index: error.value },
                })
            }
            other => check(other),
        }
    }
}

impl Submission for CudaSubmission {
    fn completion_serial(&self) -> Option<u64> {
        Some(unsafe { fj_sub_completion_serial(self.raw.0) })
    }

    fn wait(&self) -> Result<(), BackendError> {
        self.finish(unsafe { fj_sub_wait(self.raw.0, 0) })
    }

    fn wait_timeout(&self, timeout: Duration) -> Result<(), BackendError> {
        let ns = u64::try_from(timeout.as_nanos()).unwrap_or(u64::MAX).max(1);
        self.finish(unsafe { fj_sub_wait(self.raw.0, ns) })
    }

    fn gpu_time(&self) -> Option<Duration> {
        let mut ns = 0_u64;
        (unsafe { fj_sub_gpu_time_ns(self.raw.0, &mut ns) } == FJ_OK).then(|| Duration::from_nanos(ns))
    }

    fn profile(&self) -> Option<SubmissionProfile> {
        None // fj_sub_profile carries {op, kernels, ns, read/write bytes, flops} per dispatch; mapping it onto SubmissionProfile is left to the maintainer
    }
}

impl Drop for CudaSubmission {
    fn drop(&mut self) {
        unsafe { fj_sub_destroy(self.raw.0) }; // waits for physical completion before the owners go
    }
}

impl Backend for CudaBackend {
    type Submission = CudaSubmission;
    type ProgramHandle = u64;

    fn memory_usage(&self) -> MemoryUsage {
        let (mut used, mut limit) = (0_u64, 0_u64);
        unsafe { fj_memory_usage(self.raw.0, &mut used, &mut limit) };
        MemoryUsage { used_bytes: used, limit_bytes: limit, ..MemoryUsage::default() }
    }

    fn device_info(&self) -> Result<DeviceInfo, BackendError> {
        Err(BackendError::UnsupportedOperation) // fj_device_info -> DeviceInfo: field mapping left to the maintainer
    }

    fn set_memory_limit(&self, bytes: u64) {
        unsafe { fj_set_memory_limit(self.raw.0, bytes) };
    }

    /// Structural recognition in the library; programs outside its set are refused, there is
    /// no interpreter fallback on the device.
    fn prepare_program(&self, program: &ValidatedProgram, _signature: &KernelSignature) -> Result<u64, BackendError> {
        let (kind, insts, outputs) = program.flat_ir(); // {tag, a, b, c} words as documented in forja_cuda.h
        let mut handle = 0_u64;
        check(unsafe {
            fj_program_prepare(
                self.raw.0,
                kind,
                insts.as_ptr(),
                (insts.len() / 4) as u32,
                outputs.as_ptr(),
                (outputs.len() / 2) as u32,
                &mut handle,
            )
        })?;
        Ok(handle)
    }

    fn alloc(&self, dtype: DType, shape: &[u32]) -> Result<Tensor, BackendError> {
        let elements = shape.iter().try_fold(1_u64, |n, &extent| n.checked_mul(u64::from(extent)));
        let bytes = elements.and_then(|n| n.checked_mul(dtype.byte_size())).ok_or(BackendError::InvalidInput)?;
        let mut id = 0_u64;
        check(unsafe { fj_alloc(self.raw.0, bytes, &mut id) })?;
        self.registry()?.insert_external(id, bytes, dtype, shape, true)
    }

    fn import_readonly(&self, bytes: MappedRegion) -> Result<ReadonlyImport, BackendError> {
        let len = u64::try_from(bytes.len()).map_err(|_| BackendError::AllocationFailed)?;
        let mut id = 0_u64;
        check(unsafe { fj_import_readonly(self.raw.0, bytes.bytes().as_ptr(), len, &mut id) })?;
        Ok(ReadonlyImport::Copied(self.registry()?.insert_external_buffer(id, len, false)?))
    }

    fn read_buffer_range(&self, buffer: BufferId, range: Range<u64>) -> Result<Vec<u8>, BackendError> {
        let len = range.end.checked_sub(range.start).ok_or(BackendError::InvalidInput)?;
        let mut out = vec![0_u8; usize::try_from(len).map_err(|_| BackendError::InvalidInput)?];
        check(unsafe { fj_read(self.raw.0, buffer.allocation(), range.start, out.as_mut_ptr(), len) })?;
        Ok(out)
    }

    fn tensor(&self, buffer: BufferId, layout: Layout) -> Result<Tensor, BackendError> {
        self.registry()?.tensor(buffer, layout)
    }

    fn view(&self, tensor: &Tensor, op: ViewOp) -> Result<Tensor, BackendError> {
        self.registry()?.view(tensor, op) // metadata only, exactly as CpuBackend::view
    }

    fn write(&self, tensor: &Tensor, bytes: &[u8]) -> Result<(), BackendError> {
        let layout = tensor.layout();
        if !tensor.is_writable() || !layout.is_contiguous() || bytes.len() as u64 != layout.byte_len() {
            return Err(BackendError::InvalidInput);
        }
        let offset = layout.offset() * layout.dtype().byte_size();
        check(unsafe { fj_write(self.raw.0, tensor.buffer().allocation(), offset, bytes.as_ptr(), bytes.len() as u64) })
    }

    fn read(&self, tensor: &Tensor) -> Result<Vec<u8>, BackendError> {
        let mut out = vec![0_u8; usize::try_from(tensor.layout().byte_len()).map_err(|_| BackendError::InvalidInput)?];
        check(unsafe { fj_read_strided(self.raw.0, &lower_tensor(tensor)?, out.as_mut_ptr()) })?;
        Ok(out)
    }

    fn release(&self, tensor: &Tensor) -> Result<(), BackendError> {
        self.registry()?.release(tensor)?; // invalidates every view
        check(unsafe { fj_release(self.raw.0, tensor.buffer().allocation()) })
    }

    fn submit(&self, commands: CommandList) -> Result<CudaSubmission, BackendError> {
        self.lower_and_submit(commands, false)
    }

    fn submit_retained(&self, commands: CommandList, owners: Vec<CompletionResource>) -> Result<CudaSubmission, BackendError> {
        let submission = self.lower_and_submit(commands, false)?;
        *submission.owners.lock().map_err(|_| BackendError::ExecutionFailed)? = owners;
        Ok(submission)
    }

    fn submit_profiled_retained(&self, commands: CommandList, owners: Vec<CompletionResource>) -> Result<CudaSubmission, BackendError> {
        let submission = self.lower_and_submit(commands, true)?;
        *submission.owners.lock().map_err(|_| BackendError::ExecutionFailed)? = owners;
        Ok(submission)
    }

    fn prepare_graph(&self, graph: forja_core::GraphTemplate) -> Result<PreparedGraph, BackendError> {
        // The default tier (instantiate + submit) already works through `submit`. A maintainer who wants the library to
        // keep the template lowers every TemplateOp / TemplateTensor::Symbolic field that is Affine{offset, scale, param}
        // to one fj_graph_binding and stores the fj_graph handle with PreparedGraph::with_backend_state.
        Ok(PreparedGraph::new(graph))
    }

    fn supports_replay_overlap(&self) -> bool {
        true // submissions run on the backend's stream; fj_submit returns once the work is enqueued
    }
}
