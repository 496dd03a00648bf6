//! kernels/attn.rs on `dc_attention` / `dc_attention_rows`.
use super::Dims;
use crate::device::{ptr, ptr_mut, Arg, DecideDevice, Stream};
use crate::ffi;
use std::rc::Rc;

pub struct Attn { pub(crate) dev: Rc<DecideDevice>, pub(crate) d: Dims }

impl Attn {
    /// `cpu_ref::attention` (attn.rs:93-118): row r at position `qpos[r]` attends cache rows `0..=qpos[r]`; the gate is read
    /// from `pq` (the rows' fused projection, row stride `ldq`) at the gate's column, as the reference's kernel does.
    #[allow(clippy::too_many_arguments)]
    pub fn attention(&self, st: &Stream, q: Arg, kc: Arg, vc: Arg, pq: Arg, qpos: Arg, y: Arg, rows: usize, ldq: usize) {
        let d = &self.d;
        let gate = if d.attn_gate { (pq.0.ptr + pq.1 + (d.nq * d.head_dim * 4) as u64) as *const f32 } else { std::ptr::null() };
        // few rows over a long cache (the pruned last layer, forward.rs:1176-1178) take the answer-row kernel
        let rc = if rows <= 64 {
            unsafe { ffi::dc_attention_rows(self.dev.ctx, st.raw(), ptr(q), ptr(kc), ptr(vc), gate, ptr(qpos) as *const u32, std::ptr::null(), ptr_mut(y),
                                            rows as u32, ldq as u32, d.nq as u32, d.nkv as u32, d.head_dim as u32) }
        } else {
            unsafe { ffi::dc_attention(self.dev.ctx, st.raw(), ptr(q), ptr(kc), ptr(vc), gate, ptr(qpos) as *const u32, ptr_mut(y), rows as u32, ldq as u32,
                                       d.nq as u32, d.nkv as u32, d.head_dim as u32, std::ptr::null(), 1, 0) }   // 0: cache length not given (see attention_in_cache)
        };
        self.dev.check(rc, "attention");
    }

    /// The same for a chunk of one request whose cache holds `cache_rows` rows in use (positions below it): `Forward` knows
    /// `pos0 + rows` (forward.rs:1236-1246); with it a chunk of 64 rows or more runs on the tcgen05 kernel.
    #[allow(clippy::too_many_arguments)]
    pub fn attention_in_cache(&self, st: &Stream, q: Arg, kc: Arg, vc: Arg, pq: Arg, qpos: Arg, y: Arg, rows: usize, ldq: usize, cache_rows: usize) {
        let d = &self.d;
        let gate = if d.attn_gate { (pq.0.ptr + pq.1 + (d.nq * d.head_dim * 4) as u64) as *const f32 } else { std::ptr::null() };
        let rc = unsafe { ffi::dc_attention(self.dev.ctx, st.raw(), ptr(q), ptr(kc), ptr(vc), gate, ptr(qpos) as *const u32, ptr_mut(y), rows as u32, ldq as u32,
                                            d.nq as u32, d.nkv as u32, d.head_dim as u32, std::ptr::null(), 1, cache_rows as u32) };
        self.dev.check(rc, "attention");
    }
}
