// softmax / log-softmax kernels: forward f16 -> f16, backward (f16 grad, f16 output) -> f16.
#include "softmax_launch.cuh"

namespace b2n {
B2N_SOFTMAX_TYPED_DEFINE(f16, f16, f16, f16, f16)
}  // namespace b2n
