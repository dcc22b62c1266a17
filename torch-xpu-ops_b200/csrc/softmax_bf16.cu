// softmax / log-softmax kernels: forward bf16 -> bf16, backward (bf16 grad, bf16 output) -> bf16.
#include "softmax_launch.cuh"

namespace b2n {
B2N_SOFTMAX_TYPED_DEFINE(bf16, bf16, bf16, bf16, bf16)
}  // namespace b2n
