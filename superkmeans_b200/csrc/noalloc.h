// Exact assignment without any device allocation; see noalloc.cu.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace skmb {
namespace noalloc {

void find_nearest(int device, const float* x_dev, const float* y_dev, size_t n, size_t k, size_t d, uint32_t* out_knn_dev, float* out_dist_dev, cudaStream_t stream);

} // namespace noalloc
} // namespace skmb
