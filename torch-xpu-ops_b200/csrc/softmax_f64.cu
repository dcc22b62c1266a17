// softmax / log-softmax kernels: forward double -> double, backward (double grad, double output) -> double.
#include "softmax_launch.cuh"

namespace b2n {
B2N_SOFTMAX_TYPED_DEFINE(f64, double, double, double, double)
}  // namespace b2n
