//! kernels/gemm.rs of the reference on `dc_gemm`.
use crate::device::{ptr, ptr_mut, Arg, DecideDevice, Stream};
use crate::ffi;
use std::rc::Rc;

/// kernels/gemm.rs:16-26; the 16-bit outputs are in the context's 16-bit type (fp16 by default).
#[repr(u32)] #[derive(Clone, Copy, PartialEq, Eq, Debug)]
pub enum Epilogue { StoreF32 = 0, StoreF16 = 1, AddF32 = 2, SwigluF16 = 3 }

pub const SWIGLU_BLOCK: usize = 16;   // config.rs:31

pub struct Gemm { pub(crate) dev: Rc<DecideDevice> }

impl Gemm {
    /// `Y = X · Wᵀ`, then `epi` (gemm.rs:138-175). The contract (N, K multiples of 32, strides covering K, alignment of
    /// the fast path) is checked by the library, which returns DC_INVALID_ARG where the reference asserts.
    #[allow(clippy::too_many_arguments)]
    pub fn gemm(&self, st: &Stream, x: Arg, w: Arg, y: Arg, m: usize, n: usize, k: usize, ldx: usize, ldw: usize, ldy: usize, epi: Epilogue) {
        let rc = unsafe { ffi::dc_gemm(self.dev.ctx, st.raw(), ptr(x), ptr(w), ptr_mut(y), m as u32, n as u32, k as u32,
                                       ldx as u32, ldw as u32, ldy as u32, epi as u32, SWIGLU_BLOCK as u32) };
        self.dev.check(rc, "gemm");
    }

    /// What `gemm_configs::plan` is to the reference (gemm_configs.rs:312): (tile width, K split of the tail wave).
    pub fn plan(&self, m: usize, n: usize, k: usize, epi: Epilogue) -> (u32, u32) {
        let mut split = 0u32;
        let bn = unsafe { ffi::dc_gemm_plan_for(self.dev.ctx, m as u32, n as u32, k as u32, epi as u32, 0, &mut split) };
        (bn, split)
    }
}
