// Layer norm / RMS norm kernels for x of type f16 with weights of type float.
#include "norm_launch.cuh"

namespace b2n {
B2N_NORM_TYPED_DEFINE(f16_w32, f16, float)
}  // namespace b2n
