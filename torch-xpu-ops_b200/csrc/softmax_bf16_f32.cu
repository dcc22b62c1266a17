// softmax / log-softmax kernels: forward bf16 -> float, backward (float grad, float output) -> bf16.
#include "softmax_launch.cuh"

namespace b2n {
B2N_SOFTMAX_TYPED_DEFINE(bf16_f32, bf16, float, float, bf16)
}  // namespace b2n
