//! kernels/gnorm.rs on `dc_gated_rmsnorm_silu`.
use super::Dims;
use crate::device::{ptr, ptr_mut, Arg, DecideDevice, Stream};
use crate::ffi;
use std::rc::Rc;

pub struct GNorm { pub(crate) dev: Rc<DecideDevice>, pub(crate) d: Dims }

impl GNorm {
    /// Per (row, value head): RMSNorm of `o` × SiLU(z) (gnorm.rs:24-31).
    pub fn gated_rmsnorm_silu(&self, st: &Stream, o: Arg, z: Arg, w: Arg, y: Arg, t: usize, ldz: usize) {
        let rc = unsafe { ffi::dc_gated_rmsnorm_silu(self.dev.ctx, st.raw(), ptr(o) as *const f32, ptr(z) as *const f32, ptr(w) as *const f32, ptr_mut(y),
                                                     t as u32, self.d.gdn_nv as u32, self.d.dv as u32, ldz as u32, self.d.eps) };
        self.dev.check(rc, "gated_rmsnorm_silu");
    }
}
