//! kernels/rope.rs on `dc_q_norm_rope` and `dc_kv_norm_rope`.
use super::Dims;
use crate::device::{ptr, ptr_mut, Arg, DecideDevice, Stream};
use crate::ffi;
use std::rc::Rc;

pub struct Rope { pub(crate) dev: Rc<DecideDevice>, pub(crate) d: Dims }

impl Rope {
    /// Head norm + RoPE of the q heads of `rows` rows of `pq` (rope.rs:30-37).
    #[allow(clippy::too_many_arguments)]
    pub fn q_norm_rope(&self, st: &Stream, pq: Arg, qw: Arg, inv_freq: Arg, qpos: Arg, qo: Arg, rows: usize, ldq: usize) {
        let d = &self.d;
        let rc = unsafe { ffi::dc_q_norm_rope(self.dev.ctx, st.raw(), ptr(pq) as *const f32, ptr(qw) as *const f32, ptr(inv_freq) as *const f32,
                                              ptr(qpos) as *const u32, ptr_mut(qo), rows as u32, ldq as u32, d.nq as u32, d.head_dim as u32, d.rot_dim as u32, d.eps) };
        self.dev.check(rc, "q_norm_rope");
    }
    /// Head norm + RoPE of the k heads into the K cache, v heads into the V cache, rows `pos0..pos0+rows` (rope.rs:43-51).
    #[allow(clippy::too_many_arguments)]
    pub fn kv_norm_rope(&self, st: &Stream, pkv: Arg, kw: Arg, inv_freq: Arg, kc: Arg, vc: Arg, rows: usize, ldkv: usize, kcol: usize, vcol: usize, pos0: usize) {
        let d = &self.d;
        let rc = unsafe { ffi::dc_kv_norm_rope(self.dev.ctx, st.raw(), ptr(pkv) as *const f32, ptr(kw) as *const f32, ptr(inv_freq) as *const f32, ptr_mut(kc), ptr_mut(vc),
                                               rows as u32, ldkv as u32, kcol as u32, vcol as u32, pos0 as u32, std::ptr::null(), d.max_tokens as u32,
                                               d.nkv as u32, d.head_dim as u32, d.rot_dim as u32, d.eps) };
        self.dev.check(rc, "kv_norm_rope");
    }
}
