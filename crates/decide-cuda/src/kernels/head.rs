//! kernels/head.rs on `dc_gather_rows_*` and `dc_final_head`.
use super::Dims;
use crate::device::{ptr, ptr_mut, Arg, DecideDevice, Stream};
use crate::ffi;
use std::rc::Rc;

pub struct Head { pub(crate) dev: Rc<DecideDevice>, pub(crate) d: Dims }

impl Head {
    /// out[i] = x[rowmap[i]] for `rows` f32 rows of `h` elements (head.rs:29).
    pub fn gather_rows_f32(&self, st: &Stream, x: Arg, rowmap: Arg, out: Arg, rows: usize, h: usize) {
        let rc = unsafe { ffi::dc_gather_rows_f32(self.dev.ctx, st.raw(), ptr(x) as *const f32, ptr(rowmap) as *const u32, ptr_mut(out) as *mut f32, rows as u32, h as u32) };
        self.dev.check(rc, "gather_rows_f32");
    }
    /// The same for 16-bit rows (head.rs:34).
    pub fn gather_rows_f16(&self, st: &Stream, x: Arg, rowmap: Arg, out: Arg, rows: usize, h: usize) {
        let rc = unsafe { ffi::dc_gather_rows_bf16(self.dev.ctx, st.raw(), ptr(x), ptr(rowmap) as *const u32, ptr_mut(out), rows as u32, h as u32) };
        self.dev.check(rc, "gather_rows_f16");
    }
    /// Final norm + candidate logits (head.rs:54-60). `table` is the whole device-resident bf16 embedding table and `cand`
    /// holds token ids: the rows are gathered on the device (the reference stages them on the CPU, forward.rs:40-45).
    #[allow(clippy::too_many_arguments)]
    pub fn final_head(&self, st: &Stream, x: Arg, w: Arg, table: Arg, cand: Arg, ncand: Arg, logits: Arg, rows: usize, max_cand: usize) {
        let rc = unsafe { ffi::dc_final_head(self.dev.ctx, st.raw(), ptr(x) as *const f32, ptr(w) as *const f32, ptr(table), ptr(cand) as *const u32,
                                             ptr(ncand) as *const u32, ptr_mut(logits) as *mut f32, rows as u32, self.d.hidden as u32, max_cand as u32, self.d.eps) };
        self.dev.check(rc, "final_head");
    }
}
