//! Eclat backend for NVIDIA B200 (sm_100a): the `BackendRegistry` / `Buffer` / `Kernel`
//! implementation that puts `libeb200` behind eclat's own plugin surface
//! (src/backend/device.rs:83-171, src/backend/traits.rs:455-587), registered like the
//! existing backends (crates/backend-c/src/lib.rs:128-137).
//!
//! Where the other backends render source text and run a compiler, `compile_ast` here
//! walks the one lowered `AstNode::Kernel` into an `eb200_kernel_desc` (see `lower.rs`)
//! and asks the library for the hand-written kernel that serves it.  A loop nest no
//! kernel class serves is an error, never a CPU fallback.
//!
//! Registration: `DeviceKind` is a closed enum (src/backend/global.rs:32-46).  Either add
//! `DeviceKind::B200` (plus `"b200"` in `parse_backend`, src/backend/device.rs:516-528) --
//! preferred, because `DeviceKind::Cuda` switches on the GPU-parallelising AST suggesters
//! that rewrite the loop nests before a backend sees them (src/backend/compile.rs:138-143)
//! -- or register as `Cuda` instead of `eclat-backend-cuda` and run with
//! `ECLAT_OPT_LEVEL=0`.  This file assumes the first.
//!
//! Written without a Rust toolchain at hand: this crate has not been compiled.

mod ffi;
mod lower;

use std::any::Any;
use std::collections::HashMap;
use std::sync::{Arc, Mutex};

use eclat::ast::{AstNode, DType};
use eclat::backend::global::DeviceKind;
use eclat::backend::{Buffer, DeviceError, Kernel, KernelConfig, KernelSignature};

pub use lower::{lower_kernel_to_desc, Lowered, Unsupported};

type DynError = Box<dyn std::error::Error + Send + Sync>;

fn dyn_err(msg: String) -> DynError {
    msg.into()
}

/// One B200: the library's device handle (one stream, one stream-ordered pool).
pub struct B200Device {
    handle: *mut ffi::eb200_device,
    pub index: usize,
    pub sm_count: i32,
}

// The library serialises access per device internally; handles may cross threads.
unsafe impl Send for B200Device {}
unsafe impl Sync for B200Device {}

impl Drop for B200Device {
    fn drop(&mut self) {
        unsafe { ffi::eb200_device_close(self.handle); }
    }
}

impl B200Device {
    pub fn synchronize(&self) -> Result<(), DynError> {
        ffi::check(unsafe { ffi::eb200_device_sync(self.handle) }).map_err(dyn_err)
    }
}

/// Device buffer: zero-filled on allocation like `CBuffer` (crates/backend-c/src/buffer.rs:84-93);
/// `clone_buffer` is a value copy implemented as shared storage with copy-on-write.
pub struct B200Buffer {
    handle: *mut ffi::eb200_buffer,
    shape: Vec<usize>,
    dtype: DType,
    bytes: usize,
}

unsafe impl Send for B200Buffer {}
unsafe impl Sync for B200Buffer {}

impl Drop for B200Buffer {
    fn drop(&mut self) {
        unsafe { ffi::eb200_buffer_release(self.handle); }
    }
}

fn dtype_bytes(dt: &DType) -> usize {
    match dt {
        DType::Bool | DType::I8 | DType::U8 => 1,
        DType::I64 | DType::U64 | DType::F64 => 8,
        DType::F16 | DType::BF16 | DType::I16 | DType::U16 => 2,
        _ => 4,
    }
}

impl Buffer for B200Buffer {
    fn shape(&self) -> &[usize] { &self.shape }
    fn dtype(&self) -> DType { self.dtype.clone() }
    fn byte_len(&self) -> usize { self.bytes }

    fn read_to_host(&self) -> Result<Vec<u8>, DynError> {
        // orders after every launch queued on the device so far (the reference's backends are
        // synchronous; callers read results right after `execute`)
        let mut out = vec![0u8; self.bytes];
        ffi::check(unsafe { ffi::eb200_buffer_read(self.handle, out.as_mut_ptr() as *mut _, self.bytes) }).map_err(dyn_err)?;
        Ok(out)
    }

    fn write_from_host(&mut self, data: &[u8]) -> Result<(), DynError> {
        // a size mismatch is the library's error, with CBuffer's message (crates/backend-c/src/buffer.rs:151-160)
        ffi::check(unsafe { ffi::eb200_buffer_write(self.handle, data.as_ptr() as *const _, data.len()) }).map_err(dyn_err)
    }

    fn clone_buffer(&self) -> Box<dyn Buffer> {
        let mut h: *mut ffi::eb200_buffer = std::ptr::null_mut();
        let st = unsafe { ffi::eb200_buffer_clone(self.handle, &mut h) };
        assert_eq!(st, ffi::OK, "eb200_buffer_clone: {}", ffi::last_error());
        Box::new(B200Buffer { handle: h, shape: self.shape.clone(), dtype: self.dtype.clone(), bytes: self.bytes })
    }

    fn as_any(&self) -> &dyn Any { self }
    fn as_any_mut(&mut self) -> &mut dyn Any { self }
}

/// A selected hand-written kernel.  `operand_buffer[i]` says which of `execute`'s input
/// buffers the descriptor's operand `i` reads (one buffer read through two views is two
/// operands).
pub struct B200Kernel {
    handle: *mut ffi::eb200_kernel,
    device: Arc<B200Device>,
    config: KernelConfig,
    operand_buffer: Vec<usize>,
    desc: Box<ffi::eb200_kernel_desc>,
}

unsafe impl Send for B200Kernel {}
unsafe impl Sync for B200Kernel {}

impl Drop for B200Kernel {
    fn drop(&mut self) {
        unsafe { ffi::eb200_kernel_release(self.handle); }
    }
}

impl B200Kernel {
    fn create(device: Arc<B200Device>, lowered: Lowered, entry: String) -> Result<Self, DeviceError> {
        let desc = Box::new(lowered.desc);
        let mut h: *mut ffi::eb200_kernel = std::ptr::null_mut();
        ffi::check(unsafe { ffi::eb200_kernel_create(device.handle, desc.as_ref(), &mut h) })
            .map_err(DeviceError::InitializationError)?;
        Ok(B200Kernel { handle: h, device, config: KernelConfig::new(entry), operand_buffer: lowered.operand_buffer, desc })
    }
}

impl Kernel for B200Kernel {
    fn clone_kernel(&self) -> Box<dyn Kernel> {
        let mut h: *mut ffi::eb200_kernel = std::ptr::null_mut();
        let st = unsafe { ffi::eb200_kernel_create(self.device.handle, self.desc.as_ref(), &mut h) };
        assert_eq!(st, ffi::OK, "eb200_kernel_create: {}", ffi::last_error());
        Box::new(B200Kernel { handle: h, device: self.device.clone(), config: self.config.clone(),
                              operand_buffer: self.operand_buffer.clone(), desc: self.desc.clone() })
    }

    fn config(&self) -> &KernelConfig { &self.config }
    fn device_kind(&self) -> DeviceKind { DeviceKind::B200 }

    /// Inputs first, then outputs, in `Kernel.params` order (src/backend/traits.rs:545-550).
    /// The launch is asynchronous on the device's stream; `read_to_host` orders after it.
    fn execute(&self, inputs: &[&dyn Buffer], outputs: &mut [&mut dyn Buffer]) -> Result<(), DynError> {
        let mut ins: Vec<*mut ffi::eb200_buffer> = Vec::with_capacity(self.operand_buffer.len());
        for &b in &self.operand_buffer {
            let buf = inputs.get(b).ok_or_else(|| dyn_err(format!("kernel reads input {b}, {} given", inputs.len())))?;
            // a foreign buffer type is a caller bug; the C backend panics here (crates/backend-c/src/kernel.rs:196-210)
            let buf = buf.as_any().downcast_ref::<B200Buffer>().ok_or_else(|| dyn_err("B200Kernel requires B200Buffer arguments".into()))?;
            ins.push(buf.handle);
        }
        if outputs.len() != 1 { return Err(dyn_err(format!("kernel writes 1 output, {} given", outputs.len()))); }
        let out = outputs[0].as_any().downcast_ref::<B200Buffer>().ok_or_else(|| dyn_err("B200Kernel requires B200Buffer arguments".into()))?;
        let outs = [out.handle];
        ffi::check(unsafe { ffi::eb200_kernel_launch(self.handle, ins.as_ptr(), ins.len() as i32, outs.as_ptr(), 1) }).map_err(dyn_err)
    }

    fn execute_with_sizes(&self, inputs: &[&dyn Buffer], outputs: &mut [&mut dyn Buffer], _grid: [usize; 3], _local: [usize; 3]) -> Result<(), DynError> {
        // grid and block belong to the hand-written kernel, not to the caller
        self.execute(inputs, outputs)
    }

    fn as_any(&self) -> &dyn Any { self }
}

pub struct B200BackendRegistry {
    /// numel of the buffers a kernel's parameters name, recorded at allocate_buffer time by shape
    /// (the executor allocates every output from the lowerer's shape map before it compiles the
    /// kernel, src/backend/executor.rs:286-339); filled through `note_buffer`.
    sizes: Mutex<HashMap<String, i64>>,
}

impl B200BackendRegistry {
    pub fn new() -> Self { B200BackendRegistry { sizes: Mutex::new(HashMap::new()) } }

    /// The executor knows each parameter's shape (`Lowerer::buffer_shape`, src/lowerer/lower.rs:1194-1234);
    /// it tells the backend before `compile_ast` so descriptors carry buffer sizes for validation.
    pub fn note_buffer(&self, name: &str, numel: i64) {
        self.sizes.lock().unwrap().insert(name.to_string(), numel);
    }

    fn device<'a>(&self, device: &'a dyn Any) -> Result<&'a Arc<B200Device>, DeviceError> {
        device.downcast_ref::<Arc<B200Device>>()
            .ok_or_else(|| DeviceError::InitializationError("not a B200 device".to_string()))
    }
}

impl eclat::backend::device::BackendRegistry for B200BackendRegistry {
    fn kind(&self) -> DeviceKind { DeviceKind::B200 }
    fn name(&self) -> &str { "B200 (sm_100a, hand-written kernels)" }

    fn is_available(&self) -> bool {
        let mut n = 0;
        ffi::check_abi().is_ok() && unsafe { ffi::eb200_device_count(&mut n) } == ffi::OK && n > 0
    }

    fn list_devices(&self) -> Vec<String> {
        let mut n = 0;
        if unsafe { ffi::eb200_device_count(&mut n) } != ffi::OK { return vec![]; }
        (0..n).map(|i| format!("b200:{i}")).collect()
    }

    fn supports_runtime(&self) -> bool { true }

    fn create_device(&self, index: usize) -> Result<Arc<dyn Any + Send + Sync>, DeviceError> {
        ffi::check_abi().map_err(DeviceError::InitializationError)?;
        let mut h: *mut ffi::eb200_device = std::ptr::null_mut();
        ffi::check(unsafe { ffi::eb200_device_open(index as i32, &mut h) }).map_err(DeviceError::InitializationError)?;
        let mut props: ffi::eb200_device_props = unsafe { std::mem::zeroed() };
        ffi::check(unsafe { ffi::eb200_device_get_props(h, &mut props) }).map_err(DeviceError::InitializationError)?;
        let dev: Arc<B200Device> = Arc::new(B200Device { handle: h, index, sm_count: props.sm_count });
        Ok(Arc::new(dev))
    }

    fn allocate_buffer(&self, device: &dyn Any, shape: Vec<usize>, dtype: DType) -> Result<Box<dyn Buffer>, DeviceError> {
        let dev = self.device(device)?;
        let bytes = shape.iter().product::<usize>().max(1) * dtype_bytes(&dtype);
        let mut h: *mut ffi::eb200_buffer = std::ptr::null_mut();
        ffi::check(unsafe { ffi::eb200_buffer_alloc(dev.handle, bytes, &mut h) }).map_err(DeviceError::InitializationError)?;
        Ok(Box::new(B200Buffer { handle: h, shape, dtype, bytes }))
    }

    /// `program` holds exactly one `Kernel` (src/backend/executor.rs:323-339).  Must NOT go through
    /// `Pipeline::compile_ast`: its second AST beam search rewrites the loop nest (src/backend/pipeline.rs:219-279).
    fn compile_ast(&self, device: &dyn Any, program: AstNode, signature: KernelSignature) -> Result<Box<dyn Kernel>, DeviceError> {
        let dev = self.device(device)?.clone();
        let kernel = match &program {
            AstNode::Program { functions, .. } if functions.len() == 1 => &functions[0],
            AstNode::Kernel { .. } => &program,
            _ => return Err(DeviceError::InitializationError("compile_ast expects a program with one kernel".to_string())),
        };
        let entry = match kernel { AstNode::Kernel { name: Some(n), .. } => n.clone(), _ => "kernel".to_string() };
        // buffer sizes: from the signature's shapes where it has them, else from note_buffer
        let sizes = self.sizes.lock().unwrap().clone();
        let sig_sizes: HashMap<String, i64> = signature.inputs.iter().chain(signature.outputs.iter())
            .map(|b| (b.name.clone(), b.shape.iter().map(|&s| s as i64).product::<i64>().max(1))).collect();
        let numel_of = |name: &str| sig_sizes.get(name).copied().or_else(|| sizes.get(name).copied());
        let lowered = lower_kernel_to_desc(kernel, &numel_of)
            .map_err(|e| DeviceError::InitializationError(format!("no B200 kernel class serves {entry}: {}", e.0)))?;
        Ok(Box::new(B200Kernel::create(dev, lowered, entry)?))
    }
}

/// Data-parallel helper over `eb200_comm_*`: one process per GPU; rank 0 makes the id, the host
/// program carries the 128 bytes to the other ranks.
pub struct B200Comm {
    handle: *mut ffi::eb200_comm,
}

unsafe impl Send for B200Comm {}

impl B200Comm {
    pub fn unique_id() -> Result<[i8; 128], String> {
        let mut id = ffi::eb200_comm_id { bytes: [0; 128] };
        ffi::check(unsafe { ffi::eb200_comm_unique_id(&mut id) })?;
        Ok(id.bytes)
    }

    pub fn new(device: &B200Device, rank: usize, nranks: usize, id: Option<[i8; 128]>) -> Result<Self, String> {
        let cid = id.map(|b| ffi::eb200_comm_id { bytes: b });
        let mut h: *mut ffi::eb200_comm = std::ptr::null_mut();
        let p = cid.as_ref().map(|c| c as *const _).unwrap_or(std::ptr::null());
        ffi::check(unsafe { ffi::eb200_comm_init(device.handle, rank as i32, nranks as i32, p, &mut h) })?;
        Ok(B200Comm { handle: h })
    }

    /// params -= lr * (sum over ranks of grads): the gradient all-reduce fused with SGD::step
    /// (crates/nn/src/optim/sgd.rs:91-95), one kernel.
    pub fn allreduce_sgd(&self, params: &B200Buffer, grads: &B200Buffer, count: usize, lr: f32) -> Result<(), String> {
        ffi::check(unsafe { ffi::eb200_comm_allreduce_sgd(self.handle, params.handle, grads.handle, 0, count as i64, lr) })
    }

    pub fn allreduce(&self, buf: &B200Buffer, count: usize, reduce_op: i32) -> Result<(), String> {
        ffi::check(unsafe { ffi::eb200_comm_allreduce(self.handle, buf.handle, 0, count as i64, reduce_op) })
    }
}

impl Drop for B200Comm {
    fn drop(&mut self) {
        unsafe { ffi::eb200_comm_destroy(self.handle); }
    }
}

/// Registers the backend (called automatically when the crate is linked).
pub fn init() {
    eclat::backend::register_backend(Box::new(B200BackendRegistry::new()));
}

#[ctor::ctor]
fn auto_init() {
    init();
}
