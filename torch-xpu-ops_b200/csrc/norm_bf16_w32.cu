// Layer norm / RMS norm kernels for x of type bf16 with weights of type float.
#include "norm_launch.cuh"

namespace b2n {
B2N_NORM_TYPED_DEFINE(bf16_w32, bf16, float)
}  // namespace b2n
