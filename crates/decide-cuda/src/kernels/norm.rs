//! kernels/norm.rs on `dc_rmsnorm`.
use super::Dims;
use crate::device::{ptr, ptr_mut, Arg, DecideDevice, Stream};
use crate::ffi;
use std::rc::Rc;

pub struct Norm { pub(crate) dev: Rc<DecideDevice>, pub(crate) d: Dims }

impl Norm {
    /// norm.rs:26-33. `rowmap = None` is the identity (the reference binds an iota buffer).
    #[allow(clippy::too_many_arguments)]
    pub fn rmsnorm(&self, st: &Stream, x: Arg, w: Arg, y: Arg, rowmap: Option<Arg>, rows: usize, h: usize, ld_in: usize, ld_out: usize, add_one: bool) {
        let map = rowmap.map_or(std::ptr::null(), |a| ptr(a) as *const u32);
        let rc = unsafe { ffi::dc_rmsnorm(self.dev.ctx, st.raw(), ptr(x) as *const f32, ptr(w) as *const f32, ptr_mut(y), map,
                                          rows as u32, h as u32, ld_in as u32, ld_out as u32, self.d.eps, add_one as u32) };
        self.dev.check(rc, "rmsnorm");
    }
}
