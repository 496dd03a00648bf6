//! kernels/delta.rs on `dc_gated_delta`.
use super::Dims;
use crate::device::{ptr, ptr_mut, Arg, DecideDevice, Stream};
use crate::ffi;
use std::rc::Rc;

pub struct Delta { pub(crate) dev: Rc<DecideDevice>, pub(crate) d: Dims }

impl Delta {
    /// `cpu_ref::gated_delta` over `t` rows (delta.rs:68-100); `state_in` may be `state_out`. The fast kernels are the
    /// chunk-64 form and take scratch from the context's workspace: reserve `scratch_bytes(t)` at start-up.
    #[allow(clippy::too_many_arguments)]
    pub fn gated_delta(&self, st: &Stream, q: Arg, k: Arg, v: Arg, a: Arg, b: Arg, a_log: Arg, dt_bias: Arg, state_in: Arg, state_out: Arg, o: Arg,
                       t: usize, ldab: usize, write_state: bool) {
        let d = &self.d;
        let rc = unsafe { ffi::dc_gated_delta(self.dev.ctx, st.raw(), ptr(q) as *const f32, ptr(k) as *const f32, ptr(v) as *const f32, ptr(a) as *const f32,
                                              ptr(b) as *const f32, ptr(a_log) as *const f32, ptr(dt_bias) as *const f32, ptr(state_in) as *const f32,
                                              ptr_mut(state_out) as *mut f32, ptr_mut(o) as *mut f32, t as u32, ldab as u32, write_state as u32,
                                              d.gdn_nk as u32, d.gdn_nv as u32, d.dk as u32, d.dv as u32, std::ptr::null(), 1, t as u32) };
        self.dev.check(rc, "gated_delta");
    }
    pub fn scratch_bytes(&self, t: usize) -> usize { unsafe { ffi::dc_gated_delta_scratch_bytes(t as u32, 1, self.d.gdn_nv as u32) } }
}
