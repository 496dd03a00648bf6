//! decide-cuda: libdecide_cuda.so behind the `Kernels` interface of decide-engine
//! (crates/decide-engine/src/kernels/mod.rs:40-67), replacing decide-metal + kernels/*.metal.
//!
//! `DecideDevice` plays decide-metal's part (one context per GPU, error latch, status word);
//! `kernels::Kernels` has the reference's families and methods with a CUDA stream where the
//! reference passes a compute encoder. Not compiled where it was written (no Rust toolchain): unverified.
pub mod device;
pub mod ffi;
pub mod kernels;

pub use device::{DecideDevice, DeviceBuffer, Stream};
