// Layer norm / RMS norm kernels for x of type f16 with weights of type f16.
#include "norm_launch.cuh"

namespace b2n {
B2N_NORM_TYPED_DEFINE(f16, f16, f16)
}  // namespace b2n
