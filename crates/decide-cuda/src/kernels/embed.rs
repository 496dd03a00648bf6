//! kernels/embed.rs on `dc_embed`.
use super::Dims;
use crate::device::{ptr, ptr_mut, Arg, DecideDevice, Stream};
use crate::ffi;
use std::rc::Rc;

pub struct Embed { pub(crate) dev: Rc<DecideDevice>, pub(crate) d: Dims }

impl Embed {
    /// out[t] = embed[ids[t]] (bf16 → f32), rows [T, HIDDEN] (embed.rs:17-22).
    pub fn embed(&self, st: &Stream, ids: Arg, table: Arg, out: Arg, t: usize) {
        let rc = unsafe { ffi::dc_embed(self.dev.ctx, st.raw(), ptr(ids) as *const u32, ptr(table), ptr_mut(out) as *mut f32, t as u32, self.d.hidden as u32) };
        self.dev.check(rc, "embed");
    }
}
