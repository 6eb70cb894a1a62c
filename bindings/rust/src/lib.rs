//! Volta's optimizer API (`Adam::new / SGD::new / Muon::new`, `step()`, `zero_grad()`;
//! src/nn/optim/adam.rs:18-95, sgd.rs:28-90, muon.rs:19-163) over the C ABI of
//! `include/volta_b200.h`.
//!
//! The optimizers are generic over [`OptimizerTensor`], the three things Volta's optimizers
//! touch on a `Tensor` (`Rc<RefCell<RawTensor>>`, src/tensor.rs:23,38-46): the f32 data, the
//! optional gradient and the shape.  Inside Volta the impl is a dozen lines over `borrow()` /
//! `borrow_mut()`; with it in place `volta::nn::Adam` can re-export [`Adam<Tensor>`] and every
//! call site (`Adam::new(params, lr, betas, eps, wd)`, `opt.step()`, `opt.zero_grad()`) compiles
//! unchanged.
//!
//! This crate is not compiled in the repository that carries it (no Rust toolchain there);
//! the same entry points are exercised from C++ and Python by its tests.

use std::ffi::CStr;
use std::os::raw::{c_char, c_int, c_void};

#[allow(non_camel_case_types)]
pub mod ffi {
    use super::*;

    #[repr(C)]
    pub struct vb_engine {
        _private: [u8; 0],
    }
    #[repr(C)]
    pub struct vb_optimizer {
        _private: [u8; 0],
    }

    /// Same layout as `volta::gpu::OptimizerStepParams` (src/gpu/kernels.rs:42-54).
    #[repr(C)]
    #[derive(Copy, Clone, Debug, Default)]
    pub struct vb_optimizer_step_params {
        pub op: u32,
        pub lr: f32,
        pub beta1: f32,
        pub beta2: f32,
        pub t: f32,
        pub eps: f32,
        pub weight_decay: f32,
        pub padding: f32,
    }

    pub const VB_OK: c_int = 0;
    pub const VB_NS_F32: c_int = 0;
    pub const VB_NS_BF16: c_int = 1;
    pub const VB_NS_F32_TC: c_int = 2;
    /// Flags of `vb_optimizer_step_ex`.
    pub const VB_STEP_DEFAULT: u32 = 0;
    pub const VB_STEP_NO_EXCHANGE: u32 = 1;
    pub const VB_STEP_EXCHANGE_BF16: u32 = 2;
    pub const VB_STEP_REDUCE_GRADS: u32 = 4;
    pub const VB_STEP_MEAN_GRADS: u32 = 8;
    pub const VB_IPC_HANDLE_BYTES: usize = 64;

    unsafe extern "C" {
        pub fn vb_abi_version() -> c_int;
        pub fn vb_last_error() -> *const c_char;
        pub fn vb_engine_create(device: c_int, out: *mut *mut vb_engine) -> c_int;
        pub fn vb_engine_destroy(engine: *mut vb_engine) -> c_int;
        pub fn vb_engine_synchronize(engine: *mut vb_engine) -> c_int;
        pub fn vb_engine_synchronize_deadline(engine: *mut vb_engine, timeout_ms: f64) -> c_int;
        pub fn vb_engine_set_wait_limit_ms(engine: *mut vb_engine, milliseconds: u32) -> c_int;
        pub fn vb_engine_set_replicated_fraction(engine: *mut vb_engine, fraction: f64) -> c_int;
        pub fn vb_adam_create(
            engine: *mut vb_engine, n_tensors: i64, sizes: *const i64, lr: f32, beta1: f32, beta2: f32,
            eps: f32, weight_decay: f32, out: *mut *mut vb_optimizer,
        ) -> c_int;
        pub fn vb_sgd_create(
            engine: *mut vb_engine, n_tensors: i64, sizes: *const i64, lr: f32, momentum: f32,
            weight_decay: f32, out: *mut *mut vb_optimizer,
        ) -> c_int;
        pub fn vb_muon_create(
            engine: *mut vb_engine, n_tensors: i64, rows: *const i64, cols: *const i64, lr: f32,
            momentum: f32, nesterov: c_int, ns_steps: c_int, ns_mode: c_int, out: *mut *mut vb_optimizer,
        ) -> c_int;
        pub fn vb_optimizer_destroy(opt: *mut vb_optimizer) -> c_int;
        pub fn vb_optimizer_upload_params(opt: *mut vb_optimizer, tensor: i64, host: *const f32, n: i64) -> c_int;
        pub fn vb_optimizer_download_params(opt: *mut vb_optimizer, tensor: i64, host: *mut f32, n: i64) -> c_int;
        pub fn vb_optimizer_upload_grad(opt: *mut vb_optimizer, tensor: i64, host: *const f32, n: i64) -> c_int;
        pub fn vb_optimizer_set_grad_present(opt: *mut vb_optimizer, tensor: i64, present: c_int) -> c_int;
        pub fn vb_optimizer_step(opt: *mut vb_optimizer) -> c_int;
        pub fn vb_optimizer_zero_grad(opt: *mut vb_optimizer) -> c_int;
        // one process per GPU: communicator, sharded step, fused exchanges (no counterpart in Volta)
        pub fn vb_comm_unique_id(id128: *mut c_void) -> c_int;
        pub fn vb_engine_comm_init(engine: *mut vb_engine, id128: *const c_void, rank: c_int, world: c_int) -> c_int;
        pub fn vb_optimizer_step_ex(opt: *mut vb_optimizer, flags: u32) -> c_int;
        pub fn vb_plan_muon_owners(
            n_tensors: i64, rows: *const i64, cols: *const i64, world_size: c_int, ns_mode: c_int, ns_steps: c_int,
            owner_out: *mut i32, rank_cost_out: *mut f64,
        ) -> c_int;
        // every rank gathers all fingerprints before the first sharded step; a mismatch is an error on all ranks
        pub fn vb_optimizer_plan_fingerprint(opt: *mut vb_optimizer, fingerprint: *mut u64) -> c_int;
        pub fn vb_plan_fingerprints_agree(fingerprints: *const u64, n_ranks: c_int, first_mismatch: *mut c_int) -> c_int;
        pub fn vb_optimizer_ipc_handle(opt: *mut vb_optimizer, handle64: *mut c_void) -> c_int;
        pub fn vb_optimizer_open_peers(opt: *mut vb_optimizer, handles: *const c_void, n_handles: c_int) -> c_int;
        pub fn vb_optimizer_ipc_handle_grads(opt: *mut vb_optimizer, handle64: *mut c_void) -> c_int;
        pub fn vb_optimizer_open_peers_grads(opt: *mut vb_optimizer, handles: *const c_void, n_handles: c_int) -> c_int;
        pub fn vb_optimizer_enable_bf16_params(opt: *mut vb_optimizer) -> c_int;
        pub fn vb_optimizer_param_bf16_ptr(opt: *mut vb_optimizer, tensor: i64, out: *mut *mut c_void) -> c_int;
        pub fn vb_optimizer_download_params_bf16(opt: *mut vb_optimizer, tensor: i64, host: *mut u16, n: i64) -> c_int;
        pub fn vb_optimizer_ipc_handle_bf16(opt: *mut vb_optimizer, handle64: *mut c_void) -> c_int;
        pub fn vb_optimizer_open_peers_bf16(opt: *mut vb_optimizer, handles: *const c_void, n_handles: c_int) -> c_int;
        pub fn vb_multi_tensor_step(
            engine: *mut vb_engine, hp: *const vb_optimizer_step_params, n_tensors: i64, sizes: *const i64,
            params: *const *mut c_void, grads: *const *const c_void, state1: *const *mut c_void,
            state2: *const *mut c_void,
        ) -> c_int;
    }
}

/// What an optimizer needs from a parameter tensor.
pub trait OptimizerTensor {
    /// Number of f32 elements.
    fn len(&self) -> usize;
    /// Shape, as `RawTensor::shape`.
    fn shape(&self) -> Vec<usize>;
    /// Calls `f` with the parameter values.
    fn with_data<R>(&self, f: impl FnOnce(&[f32]) -> R) -> R;
    /// Calls `f` with the parameter values, mutably (the updated values are written here).
    fn with_data_mut<R>(&self, f: impl FnOnce(&mut [f32]) -> R) -> R;
    /// Calls `f` with the gradient if there is one (`grad: Option<Storage>`).
    fn with_grad<R>(&self, f: impl FnOnce(Option<&[f32]>) -> R) -> R;
    /// `grad = None`.
    fn clear_grad(&self);
}

/// Volta's optimizers panic on invariant violations (adam.rs:164,169,195); so does the shim.
fn check(status: c_int) {
    if status != ffi::VB_OK {
        let msg = unsafe { CStr::from_ptr(ffi::vb_last_error()) }.to_string_lossy().into_owned();
        panic!("volta_b200: {msg}");
    }
}

/// One engine per thread on device 0 (Volta is single threaded; its GPU context is a global).
fn engine() -> *mut ffi::vb_engine {
    struct Holder(*mut ffi::vb_engine);
    impl Drop for Holder {
        fn drop(&mut self) {
            unsafe { ffi::vb_engine_destroy(self.0) };
        }
    }
    thread_local! {
        static ENGINE: Holder = {
            let mut e = std::ptr::null_mut();
            check(unsafe { ffi::vb_engine_create(0, &mut e) });
            Holder(e)
        };
    }
    ENGINE.with(|h| h.0)
}

struct Core<T: OptimizerTensor> {
    params: Vec<T>,
    handle: *mut ffi::vb_optimizer,
}

impl<T: OptimizerTensor> Core<T> {
    fn adopt(params: Vec<T>, handle: *mut ffi::vb_optimizer) -> Self {
        for (i, p) in params.iter().enumerate() {
            p.with_data(|d| check(unsafe { ffi::vb_optimizer_upload_params(handle, i as i64, d.as_ptr(), d.len() as i64) }));
        }
        Self { params, handle }
    }

    fn step(&mut self) {
        for (i, p) in self.params.iter().enumerate() {
            p.with_grad(|g| match g {
                Some(g) => check(unsafe { ffi::vb_optimizer_upload_grad(self.handle, i as i64, g.as_ptr(), g.len() as i64) }),
                None => check(unsafe { ffi::vb_optimizer_set_grad_present(self.handle, i as i64, 0) }),
            });
        }
        check(unsafe { ffi::vb_optimizer_step(self.handle) });
        for (i, p) in self.params.iter().enumerate() {
            p.with_data_mut(|d| check(unsafe { ffi::vb_optimizer_download_params(self.handle, i as i64, d.as_mut_ptr(), d.len() as i64) }));
        }
    }

    fn zero_grad(&self) {
        for p in &self.params {
            p.clear_grad();
        }
        check(unsafe { ffi::vb_optimizer_zero_grad(self.handle) });
    }
}

impl<T: OptimizerTensor> Drop for Core<T> {
    fn drop(&mut self) {
        unsafe { ffi::vb_optimizer_destroy(self.handle) };
    }
}

fn sizes<T: OptimizerTensor>(params: &[T]) -> Vec<i64> {
    params.iter().map(|p| p.len() as i64).collect()
}

/// `Adam::new(params, lr, betas, eps, weight_decay)` (src/nn/optim/adam.rs:18-60).
pub struct Adam<T: OptimizerTensor>(Core<T>);

impl<T: OptimizerTensor> Adam<T> {
    #[must_use]
    pub fn new(params: Vec<T>, lr: f32, betas: (f32, f32), eps: f32, weight_decay: f32) -> Self {
        let s = sizes(&params);
        let mut h = std::ptr::null_mut();
        check(unsafe { ffi::vb_adam_create(engine(), s.len() as i64, s.as_ptr(), lr, betas.0, betas.1, eps, weight_decay, &mut h) });
        Self(Core::adopt(params, h))
    }
    pub fn step(&mut self) {
        self.0.step();
    }
    pub fn zero_grad(&self) {
        self.0.zero_grad();
    }
}

/// `SGD::new(params, lr, momentum, weight_decay)` (src/nn/optim/sgd.rs:28-52).
pub struct SGD<T: OptimizerTensor>(Core<T>);

impl<T: OptimizerTensor> SGD<T> {
    #[must_use]
    pub fn new(params: Vec<T>, lr: f32, momentum: f32, weight_decay: f32) -> Self {
        let s = sizes(&params);
        let mut h = std::ptr::null_mut();
        check(unsafe { ffi::vb_sgd_create(engine(), s.len() as i64, s.as_ptr(), lr, momentum, weight_decay, &mut h) });
        Self(Core::adopt(params, h))
    }
    pub fn step(&mut self) {
        self.0.step();
    }
    pub fn zero_grad(&self) {
        self.0.zero_grad();
    }
}

/// `Muon::new(params, lr, momentum, nesterov, ns_steps)` (src/nn/optim/muon.rs:19-38).
pub struct Muon<T: OptimizerTensor>(Core<T>);

impl<T: OptimizerTensor> Muon<T> {
    #[must_use]
    pub fn new(params: Vec<T>, lr: f32, momentum: f32, nesterov: bool, ns_steps: usize) -> Self {
        Self::with_mode(params, lr, momentum, nesterov, ns_steps, ffi::VB_NS_F32)
    }

    /// `ns_mode`: `ffi::VB_NS_F32` (bit-faithful), `ffi::VB_NS_BF16` or `ffi::VB_NS_F32_TC`.
    #[must_use]
    pub fn with_mode(params: Vec<T>, lr: f32, momentum: f32, nesterov: bool, ns_steps: usize, ns_mode: c_int) -> Self {
        // (rows, cols) as Muon::step flattens a shape (muon.rs:117-130)
        let (rows, cols): (Vec<i64>, Vec<i64>) = params
            .iter()
            .map(|p| {
                let shape = p.shape();
                if shape.len() < 2 {
                    (shape.first().copied().unwrap_or(1) as i64, 1_i64)
                } else {
                    (shape[0] as i64, shape[1..].iter().product::<usize>() as i64)
                }
            })
            .unzip();
        let mut h = std::ptr::null_mut();
        check(unsafe {
            ffi::vb_muon_create(engine(), rows.len() as i64, rows.as_ptr(), cols.as_ptr(), lr, momentum,
                                c_int::from(nesterov), ns_steps as c_int, ns_mode, &mut h)
        });
        Self(Core::adopt(params, h))
    }
    pub fn step(&mut self) {
        self.0.step();
    }
    pub fn zero_grad(&self) {
        self.0.zero_grad();
    }
}

/// Host tensor for tests and for callers without Volta's types.
pub mod host {
    use super::OptimizerTensor;
    use std::cell::RefCell;
    use std::rc::Rc;

    pub struct RawTensor {
        pub data: Vec<f32>,
        pub shape: Vec<usize>,
        pub grad: Option<Vec<f32>>,
    }
    pub type Tensor = Rc<RefCell<RawTensor>>;

    pub fn tensor(data: Vec<f32>, shape: &[usize]) -> Tensor {
        assert_eq!(data.len(), shape.iter().product::<usize>());
        Rc::new(RefCell::new(RawTensor { data, shape: shape.to_vec(), grad: None }))
    }

    impl OptimizerTensor for Tensor {
        fn len(&self) -> usize {
            self.borrow().data.len()
        }
        fn shape(&self) -> Vec<usize> {
            self.borrow().shape.clone()
        }
        fn with_data<R>(&self, f: impl FnOnce(&[f32]) -> R) -> R {
            f(&self.borrow().data)
        }
        fn with_data_mut<R>(&self, f: impl FnOnce(&mut [f32]) -> R) -> R {
            f(&mut self.borrow_mut().data)
        }
        fn with_grad<R>(&self, f: impl FnOnce(Option<&[f32]>) -> R) -> R {
            f(self.borrow().grad.as_deref())
        }
        fn clear_grad(&self) {
            self.borrow_mut().grad = None;
        }
    }
}

#[cfg(test)]
mod tests {
    use super::host::tensor;
    use super::*;

    // tests/test_optimizers.rs:168-196 of the reference
    #[test]
    fn test_sgd_no_momentum_simple() {
        let t = tensor(vec![5.0], &[1]);
        t.borrow_mut().grad = Some(vec![2.0]);
        let mut opt = SGD::new(vec![t.clone()], 0.1, 0.0, 0.0);
        opt.step();
        assert!((t.borrow().data[0] - (5.0 - 0.1 * 2.0)).abs() < 1e-7);
    }

    // tests/test_optimizers.rs:13-48 of the reference
    #[test]
    fn test_adam_bias_correction() {
        let (lr, b1, b2, eps, g, p0) = (0.01_f32, 0.9_f32, 0.999_f32, 1e-8_f32, 0.5_f32, 1.0_f32);
        let t = tensor(vec![p0], &[1]);
        t.borrow_mut().grad = Some(vec![g]);
        let mut opt = Adam::new(vec![t.clone()], lr, (b1, b2), eps, 0.0);
        opt.step();
        let m_hat = ((1.0 - b1) * g) / (1.0 - b1);
        let v_hat = ((1.0 - b2) * g * g) / (1.0 - b2);
        let expected = p0 - lr * m_hat / (v_hat.sqrt() + eps);
        assert!((t.borrow().data[0] - expected).abs() < 1e-7);
    }
}
