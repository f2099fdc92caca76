// One more entry for `CATALOG` in crates/velox-core/src/profile.rs (the list at :120): the card this
// branch tunes. Figures from NVIDIA's public B200 specification (HGX B200: 180 GB HBM3e per GPU,
// 148 SMs, 7.7 TB/s); `nvidia-smi` on the card reports 183,359 MiB = 179 GiB.
DeviceProfile {
    id: "b200",
    name: "NVIDIA B200",
    arch: GpuArch::Cuda {
        major: 10,
        minor: 0,
    },
    form_factor: FormFactor::Desktop,
    vram_gib: 179,
    sm_count: 148,
    mem_bandwidth_gbs: 7700,
    reserved_mib: 2048,
    tuned_branch: Some("b200"),
},
