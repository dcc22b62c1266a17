// Layer norm / RMS norm kernels for x of type float with weights of type float.
#include "norm_launch.cuh"

namespace b2n {
B2N_NORM_TYPED_DEFINE(f32, float, float)
}  // namespace b2n
