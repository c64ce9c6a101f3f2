// Stand-ins for the whole-token kernel's instantiations in the core library (make core): a build that holds everything
// but those kernels, for models that never run on them (layered architectures, and any model with YALM_B200_MEGA=0).
// kernel_of() reports "not compiled" for every variant, plan() then refuses, and models fall back to the per-op kernels.
namespace yalm {
namespace mega {
const void *kernel_f32(int, int, bool) { return nullptr; }
const void *kernel_f16(int, int, bool) { return nullptr; }
const void *kernel_f8(int, int, bool) { return nullptr; }
const void *kernel_f32_pipe(int, int, bool) { return nullptr; }
const void *kernel_f16_pipe(int, int, bool) { return nullptr; }
const void *kernel_f8_pipe(int, int, bool) { return nullptr; }
const void *kernel_f16_mma(int, int, bool) { return nullptr; }
} // namespace mega
} // namespace yalm
