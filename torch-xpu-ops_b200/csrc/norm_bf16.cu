// Layer norm / RMS norm kernels for x of type bf16 with weights of type bf16.
#include "norm_launch.cuh"

namespace b2n {
B2N_NORM_TYPED_DEFINE(bf16, bf16, bf16)
}  // namespace b2n
