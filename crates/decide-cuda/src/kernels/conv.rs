//! kernels/conv.rs on `dc_conv_silu_l2` and `dc_conv_state_update`.
use super::Dims;
use crate::device::{ptr, ptr_mut, Arg, DecideDevice, Stream};
use crate::ffi;
use std::rc::Rc;

pub struct Conv { pub(crate) dev: Rc<DecideDevice>, pub(crate) d: Dims }

impl Conv {
    /// `cpu_ref::conv_silu_l2` (conv.rs:27-36).
    #[allow(clippy::too_many_arguments)]
    pub fn conv_silu_l2(&self, st: &Stream, p: Arg, prev: Arg, w: Arg, q: Arg, k: Arg, v: Arg, t: usize, ldp: usize) {
        let d = &self.d;
        let rc = unsafe { ffi::dc_conv_silu_l2(self.dev.ctx, st.raw(), ptr(p) as *const f32, ptr(prev) as *const f32, ptr(w) as *const f32, ptr_mut(q) as *mut f32,
                                               ptr_mut(k) as *mut f32, ptr_mut(v) as *mut f32, t as u32, ldp as u32, d.gdn_nk as u32, d.gdn_nv as u32, d.dk as u32,
                                               d.dv as u32, std::ptr::null(), 1, t as u32) };
        self.dev.check(rc, "conv_silu_l2");
    }
    /// The 3 raw rows that end the chunk (conv.rs:40-46).
    pub fn conv_state_update(&self, st: &Stream, p: Arg, prev_in: Arg, prev_out: Arg, t: usize, ldp: usize) {
        let conv_dim = (2 * self.d.gdn_nk * self.d.dk + self.d.gdn_nv * self.d.dv) as u32;
        let rc = unsafe { ffi::dc_conv_state_update(self.dev.ctx, st.raw(), ptr(p) as *const f32, ptr(prev_in) as *const f32, ptr_mut(prev_out) as *mut f32, t as u32, ldp as u32, conv_dim) };
        self.dev.check(rc, "conv_state_update");
    }
}
