// softmax / log-softmax kernels: forward f16 -> float, backward (float grad, float output) -> f16.
#include "softmax_launch.cuh"

namespace b2n {
B2N_SOFTMAX_TYPED_DEFINE(f16_f32, f16, float, float, f16)
}  // namespace b2n
