//! Dispatch wrappers with the reference's shape (crates/decide-engine/src/kernels/mod.rs): one struct per
//! kernel family, one method per kernel, reached as `k.<family>.<method>(…)`. Methods only enqueue on the
//! stream; the caller synchronises. The model dims the reference compiles in are fields of `Dims`.
use crate::device::DecideDevice;
use std::rc::Rc;

mod attn;
mod conv;
mod delta;
mod embed;
mod gemm;
mod gnorm;
mod head;
mod norm;
mod rope;

pub use attn::Attn;
pub use conv::Conv;
pub use delta::Delta;
pub use embed::Embed;
pub use gemm::{Epilogue, Gemm};
pub use gnorm::GNorm;
pub use head::Head;
pub use norm::Norm;
pub use rope::Rope;
pub use crate::device::Arg;

/// config.rs:4-37 as a value.
#[derive(Clone, Copy, Debug)]
pub struct Dims {
    pub hidden: usize, pub nq: usize, pub nkv: usize, pub head_dim: usize, pub rot_dim: usize,
    pub gdn_nk: usize, pub gdn_nv: usize, pub dk: usize, pub dv: usize, pub max_tokens: usize, pub attn_gate: bool, pub eps: f32,
}

pub struct Kernels {
    pub embed: Embed, pub norm: Norm, pub gemm: Gemm, pub conv: Conv, pub delta: Delta,
    pub gnorm: GNorm, pub rope: Rope, pub attn: Attn, pub head: Head,
}

impl Kernels {
    /// `Kernels::new(dev)` (mod.rs:54-66). The reference's `Ane` family is gone with the Neural Engine.
    pub fn new(dev: Rc<DecideDevice>, d: Dims) -> anyhow::Result<Self> {
        Ok(Self {
            embed: Embed { dev: dev.clone(), d }, norm: Norm { dev: dev.clone(), d }, gemm: Gemm { dev: dev.clone() },
            conv: Conv { dev: dev.clone(), d }, delta: Delta { dev: dev.clone(), d }, gnorm: GNorm { dev: dev.clone(), d },
            rope: Rope { dev: dev.clone(), d }, attn: Attn { dev: dev.clone(), d }, head: Head { dev, d },
        })
    }
}
