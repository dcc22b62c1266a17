// softmax / log-softmax kernels: forward float -> float, backward (float grad, float output) -> float.
#include "softmax_launch.cuh"

namespace b2n {
B2N_SOFTMAX_TYPED_DEFINE(f32, float, float, float, float)
}  // namespace b2n
