// Layer norm / RMS norm kernels for x of type double with weights of type double.
#include "norm_launch.cuh"

namespace b2n {
B2N_NORM_TYPED_DEFINE(f64, double, double)
}  // namespace b2n
