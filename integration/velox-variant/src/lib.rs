//! Hardware variant of this build: **B200** (branch `b200`).
//!
//! The contract every branch exposes (see the generic variant on `main`,
//! crates/velox-variant/src/lib.rs:15-33):
//!
//! - `INFO: VariantInfo`: id, branch, the profiles it tunes and the architectures its kernels run on;
//! - `plan_policy(&DeviceProfile) -> PlanPolicy`: VRAM reserve and workspace per card;
//! - with the `cuda` feature, `cuda_kernels(&DeviceInfo) -> Result<Arc<dyn CudaKernels>>`.
//!
//! This variant serves the quantized `linear` family (NVFP4, FP8-E4M3 rows, GGML Q4_K) with the
//! sm_100a kernels in `kernels/` and leaves every other op to the portable kernels.
//!
//! Status: written against the reference's public types without a Rust toolchain at hand; it has
//! not been compiled. The C side it binds (`kernels/velox_sm100.h`) is built and tested.

use velox_core::profile::GpuArch;
use velox_core::{DeviceProfile, PlanPolicy, VariantInfo};

#[cfg(feature = "cuda")]
mod sm100;

pub static INFO: VariantInfo = VariantInfo {
    id: "b200",
    branch: "b200",
    description: "tcgen05 / TMA kernels for the NVFP4, FP8-row and Q4_K linear family on B200 (sm_100a)",
    profiles: &["b200"],
    archs: &[GpuArch::Cuda { major: 10, minor: 0 }],
};

pub fn plan_policy(profile: &DeviceProfile) -> PlanPolicy {
    PlanPolicy::for_profile(profile)
}

#[cfg(feature = "cuda")]
pub fn cuda_kernels(
    device: &velox_cuda::DeviceInfo,
) -> velox_core::Result<std::sync::Arc<dyn velox_cuda::CudaKernels>> {
    velox_cuda::require_arch(device, &INFO)?;
    Ok(std::sync::Arc::new(sm100::Sm100Kernels))
}
