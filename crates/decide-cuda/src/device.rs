//! The device layer: what `decide_metal::DecideDevice` is to the reference (device.rs:55-130), for one GPU.
use crate::ffi;
use anyhow::{bail, Result};
use std::os::raw::{c_char, c_void};

/// A CUDA stream handle (`cudaStream_t`); the ordering primitive, as the serial compute encoder is in the reference (forward.rs:31-38).
#[derive(Clone, Copy)]
pub struct Stream(pub *mut c_void);
impl Stream {
    pub fn raw(&self) -> *mut c_void { self.0 }
}

/// Device memory owned by the caller: a base address and a length in bytes.
pub struct DeviceBuffer {
    pub ptr: u64,
    pub len: usize,
}

/// A buffer and a byte offset into it (kernels/mod.rs:31-32).
pub type Arg<'a> = (&'a DeviceBuffer, u64);

pub(crate) fn ptr(a: Arg) -> *const c_void {
    debug_assert!(a.1 as usize <= a.0.len);
    (a.0.ptr + a.1) as *const c_void
}
pub(crate) fn ptr_mut(a: Arg) -> *mut c_void { ptr(a) as *mut c_void }

pub struct DecideDevice {
    pub(crate) ctx: *mut ffi::DcCtx,
}
// One context serves one stream at a time (see include/decide_cuda.h); callers serialise, as `Forward::logits(&mut self)` does.
unsafe impl Send for DecideDevice {}

impl DecideDevice {
    /// `DecideDevice::shared` + `Kernels::new`: opens GPU `device`; there is no CPU path.
    pub fn open(device: i32) -> Result<Self> {
        let mut err = [0 as c_char; 512];
        let ctx = unsafe { ffi::dc_open(device, err.as_mut_ptr(), err.len()) };
        if ctx.is_null() {
            bail!("{}", unsafe { std::ffi::CStr::from_ptr(err.as_ptr()) }.to_string_lossy());
        }
        Ok(Self { ctx })
    }

    /// The latched error message, cleared by reading it.
    pub fn last_error(&self) -> String {
        let mut buf = [0 as c_char; 1024];
        unsafe { ffi::dc_last_error(self.ctx, buf.as_mut_ptr(), buf.len()) };
        unsafe { std::ffi::CStr::from_ptr(buf.as_ptr()) }.to_string_lossy().into_owned()
    }

    pub(crate) fn check(&self, rc: i32, what: &str) {
        assert!(rc == ffi::DC_OK, "{what}: {}", self.last_error());   // the reference asserts on contract violations
    }

    /// `Gemm::warm_up` (gemm.rs:89-107): every kernel variant launchable, scratch reserved and frozen.
    pub fn warm_up(&self, scratch_bytes: usize) -> Result<()> {
        for rc in unsafe { [ffi::dc_warm_up(self.ctx), ffi::dc_reserve_workspace(self.ctx, scratch_bytes), ffi::dc_set_workspace_frozen(self.ctx, 1)] } {
            if rc != ffi::DC_OK { bail!("{}", self.last_error()); }
        }
        Ok(())
    }

    /// The command-buffer status check (forward.rs:1022-1042): waits for `st`; an error if a bounded device wait ran out.
    pub fn check_status(&self, st: &Stream) -> Result<()> {
        if unsafe { ffi::dc_check_status(self.ctx, st.raw()) } != ffi::DC_OK { bail!("{}", self.last_error()); }
        Ok(())
    }
}

impl Drop for DecideDevice {
    fn drop(&mut self) { unsafe { ffi::dc_close(self.ctx) } }
}
