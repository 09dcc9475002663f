//! strix-backend-cuda: `WeightAccel` for one NVIDIA B200 (sm_100a) over libstrix_cuda.so.
//! Uncompiled in this repository (no Rust toolchain in its build image).
pub mod accel;
pub mod ffi;
pub use accel::CudaWeightAccel;
