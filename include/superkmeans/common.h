// Drop-in counterpart of include/superkmeans/common.h of the SuperKMeans repository: the enums that
// appear in the public class templates.  Only <Quantization::f32, DistanceFunction::l2> is functional,
// as in the reference (distance_computers/batch_computers.h:15-22).
#pragma once

#include <cstddef>
#include <cstdint>

namespace skmeans {

enum class DistanceFunction : uint8_t { l2, dp };
enum class Quantization : uint8_t { f32, u8, f16, bf16 };

template <Quantization q>
using skmeans_value_t = float;
template <Quantization q>
using skmeans_centroid_value_t = float;
template <Quantization q>
using skmeans_distance_t = float;

} // namespace skmeans
