//! Raw bindings of `include/eb200.h` (ABI version 2).
//!
//! Layouts are `#[repr(C)]` copies of the header's structs; `check_abi()` compares
//! their sizes with what the loaded library reports (`eb200_abi_sizes`) before the
//! first real call, so a header / crate mismatch fails loudly instead of corrupting
//! a descriptor.
//!
//! Written without a Rust toolchain at hand: this file has not been compiled.
#![allow(non_camel_case_types, dead_code)]

use std::os::raw::{c_char, c_int, c_void};

pub const EB200_ABI_VERSION: c_int = 2;
pub const MAX_DIMS: usize = 8;
pub const MAX_INPUTS: usize = 8;
pub const MAX_BOUNDS: usize = 4;
pub const MAX_INSNS: usize = 96;

// eb200_status
pub const OK: c_int = 0;
pub const ERR_UNSUPPORTED: c_int = 2;

// eb200_dtype
pub const F32: i32 = 0;
pub const BOOL: i32 = 1;
pub const I32: i32 = 2;
pub const I64: i32 = 3;
pub const F16: i32 = 4;
pub const BF16: i32 = 5;

// eb200_kclass
pub const K_ELEMENTWISE: i32 = 0;
pub const K_REDUCE: i32 = 1;
pub const K_COPY: i32 = 2;
pub const K_SCATTER: i32 = 3;
pub const K_SGD: i32 = 4;
pub const K_CONV2D: i32 = 5;
pub const K_SCAN: i32 = 6;
pub const K_SGD_MOMENTUM: i32 = 7;
pub const K_ADAM: i32 = 8;
pub const K_SOFTMAX_XENT: i32 = 9;
pub const K_MAXPOOL2D: i32 = 10;

// eb200_reduce_op
pub const R_NONE: i32 = 0;
pub const R_SUM: i32 = 1;
pub const R_MAX: i32 = 2;
pub const R_MIN: i32 = 3;
pub const R_PROD: i32 = 4;

// eb200_opcode
pub const OP_LOAD: i32 = 0;
pub const OP_CONST: i32 = 1;
pub const OP_ADD: i32 = 2;
pub const OP_MUL: i32 = 3;
pub const OP_MAX: i32 = 4;
pub const OP_RECIP: i32 = 5;
pub const OP_SQRT: i32 = 6;
pub const OP_LOG2: i32 = 7;
pub const OP_EXP2: i32 = 8;
pub const OP_SIN: i32 = 9;
pub const OP_FLOOR: i32 = 10;
pub const OP_LT: i32 = 11;
pub const OP_AND: i32 = 12;
pub const OP_NOT: i32 = 13;
pub const OP_SELECT: i32 = 14;
pub const OP_REM: i32 = 15;
pub const OP_IDIV: i32 = 16;
pub const OP_CAST: i32 = 17;
pub const OP_FMA: i32 = 18;

#[repr(C)]
#[derive(Clone, Copy, Default)]
pub struct eb200_insn {
    pub op: i32,
    pub arg: i32,
    pub imm: f32,
    pub _pad: i32,
}

#[repr(C)]
#[derive(Clone, Copy, Default)]
pub struct eb200_bound {
    pub coef: [i64; MAX_DIMS],
    pub c: i64,
    pub lo: i64,
    pub hi: i64,
}

#[repr(C)]
#[derive(Clone, Copy, Default)]
pub struct eb200_operand {
    pub dtype: i32,
    pub n_bounds: i32,
    pub offset: i64,
    pub strides: [i64; MAX_DIMS],
    pub numel: i64,
    pub pad_value: f32,
    pub _pad: i32,
    pub bounds: [eb200_bound; MAX_BOUNDS],
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct eb200_kernel_desc {
    pub kclass: i32,
    pub ndim: i32,
    pub shape: [i64; MAX_DIMS],
    pub n_inputs: i32,
    pub reduce_op: i32,
    pub reduce_axis: i32,
    pub n_insns: i32,
    pub gemm_mode: i32,
    pub flags: i32,
    pub scalar: f32,
    pub hyper: [f32; 7],
    pub inputs: [eb200_operand; MAX_INPUTS],
    pub output: eb200_operand,
    pub prog: [eb200_insn; MAX_INSNS],
}

impl Default for eb200_kernel_desc {
    fn default() -> Self {
        // all-zero is a valid "empty" descriptor (plain-old-data, no pointers)
        unsafe { std::mem::zeroed() }
    }
}

#[repr(C)]
pub struct eb200_device_props {
    pub name: [c_char; 128],
    pub cc_major: i32,
    pub cc_minor: i32,
    pub sm_count: i32,
    pub _pad: i32,
    pub total_mem_bytes: i64,
    pub l2_bytes: i64,
    pub smem_per_block_optin: i64,
}

#[repr(C)]
pub struct eb200_kernel_info {
    pub impl_name: [c_char; 64],
    pub launches: i32,
    pub specialised: i32,
    pub scratch_bytes: i64,
    pub algo_bytes: i64,
    pub algo_flops: i64,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct eb200_comm_id {
    pub bytes: [c_char; 128],
}

// opaque handles
pub enum eb200_device {}
pub enum eb200_buffer {}
pub enum eb200_kernel {}
pub enum eb200_comm {}
pub enum eb200_graph {}

extern "C" {
    pub fn eb200_abi_version() -> c_int;
    pub fn eb200_last_error() -> *const c_char;
    pub fn eb200_abi_sizes(kernel_desc: *mut usize, operand: *mut usize, device_props: *mut usize, kernel_info: *mut usize) -> c_int;

    pub fn eb200_device_count(count: *mut c_int) -> c_int;
    pub fn eb200_device_open(index: c_int, dev: *mut *mut eb200_device) -> c_int;
    pub fn eb200_device_close(dev: *mut eb200_device) -> c_int;
    pub fn eb200_device_sync(dev: *mut eb200_device) -> c_int;
    pub fn eb200_device_get_props(dev: *mut eb200_device, props: *mut eb200_device_props) -> c_int;

    pub fn eb200_buffer_alloc(dev: *mut eb200_device, bytes: usize, buf: *mut *mut eb200_buffer) -> c_int;
    pub fn eb200_buffer_release(buf: *mut eb200_buffer) -> c_int;
    pub fn eb200_buffer_write(buf: *mut eb200_buffer, host: *const c_void, bytes: usize) -> c_int;
    pub fn eb200_buffer_read(buf: *mut eb200_buffer, host: *mut c_void, bytes: usize) -> c_int;
    pub fn eb200_buffer_clone(buf: *mut eb200_buffer, out: *mut *mut eb200_buffer) -> c_int;

    pub fn eb200_kernel_create(dev: *mut eb200_device, desc: *const eb200_kernel_desc, k: *mut *mut eb200_kernel) -> c_int;
    pub fn eb200_kernel_get_info(k: *mut eb200_kernel, info: *mut eb200_kernel_info) -> c_int;
    pub fn eb200_kernel_query(desc: *const eb200_kernel_desc, sm_count: c_int, info: *mut eb200_kernel_info) -> c_int;
    pub fn eb200_kernel_launch(k: *mut eb200_kernel, inputs: *const *mut eb200_buffer, n_inputs: c_int,
                               outputs: *const *mut eb200_buffer, n_outputs: c_int) -> c_int;
    pub fn eb200_kernel_release(k: *mut eb200_kernel) -> c_int;

    pub fn eb200_graph_begin(dev: *mut eb200_device) -> c_int;
    pub fn eb200_graph_end(dev: *mut eb200_device, graph: *mut *mut eb200_graph) -> c_int;
    pub fn eb200_graph_launch(graph: *mut eb200_graph) -> c_int;
    pub fn eb200_graph_release(graph: *mut eb200_graph) -> c_int;

    pub fn eb200_comm_unique_id(id: *mut eb200_comm_id) -> c_int;
    pub fn eb200_comm_init(dev: *mut eb200_device, rank: c_int, nranks: c_int, id: *const eb200_comm_id, comm: *mut *mut eb200_comm) -> c_int;
    pub fn eb200_comm_allreduce(comm: *mut eb200_comm, buf: *mut eb200_buffer, offset: i64, count: i64, reduce_op: c_int) -> c_int;
    pub fn eb200_comm_allreduce_async(comm: *mut eb200_comm, buf: *mut eb200_buffer, offset: i64, count: i64, reduce_op: c_int) -> c_int;
    pub fn eb200_comm_join(comm: *mut eb200_comm) -> c_int;
    pub fn eb200_comm_allreduce_sgd(comm: *mut eb200_comm, params: *mut eb200_buffer, grads: *mut eb200_buffer, offset: i64, count: i64, lr: f32) -> c_int;
    pub fn eb200_comm_allreduce_sgd_async(comm: *mut eb200_comm, params: *mut eb200_buffer, grads: *mut eb200_buffer, offset: i64, count: i64, lr: f32) -> c_int;
    pub fn eb200_kernel_set_allreduce(k: *mut eb200_kernel, comm: *mut eb200_comm) -> c_int;
    pub fn eb200_comm_destroy(comm: *mut eb200_comm) -> c_int;
}

/// Message of the last failed call on this thread.
pub fn last_error() -> String {
    unsafe {
        let p = eb200_last_error();
        if p.is_null() { String::new() } else { std::ffi::CStr::from_ptr(p).to_string_lossy().into_owned() }
    }
}

/// Turns a status code into a `Result`.
pub fn check(status: c_int) -> Result<(), String> {
    if status == OK { Ok(()) } else { Err(format!("eb200 status {status}: {}", last_error())) }
}

/// Verifies version and struct layouts against the loaded library (call once).
pub fn check_abi() -> Result<(), String> {
    unsafe {
        if eb200_abi_version() != EB200_ABI_VERSION {
            return Err(format!("libeb200 ABI {} != crate ABI {}", eb200_abi_version(), EB200_ABI_VERSION));
        }
        let (mut a, mut b, mut c, mut d) = (0usize, 0usize, 0usize, 0usize);
        check(eb200_abi_sizes(&mut a, &mut b, &mut c, &mut d))?;
        if a != std::mem::size_of::<eb200_kernel_desc>() || b != std::mem::size_of::<eb200_operand>()
            || c != std::mem::size_of::<eb200_device_props>() || d != std::mem::size_of::<eb200_kernel_info>() {
            return Err("struct layout differs from libeb200".to_string());
        }
    }
    Ok(())
}
