// create_function(): the by-name dispatcher behind the C bindings (see create_function.hpp).
#include "create_function.hpp"

#include <nbla_b200/b200.hpp>

#include <nbla/exception.hpp>
#include <nbla/function.hpp>
#include <nbla/variable.hpp>

#include <nbla/function/add2.hpp>
#include <nbla/function/affine.hpp>
#include <nbla/function/batch_normalization.hpp>
#include <nbla/function/binary_connect_affine.hpp>
#include <nbla/function/binary_connect_convolution.hpp>
#include <nbla/function/binary_weight_affine.hpp>
#include <nbla/function/binary_weight_convolution.hpp>
#include <nbla/function/convolution.hpp>
#include <nbla/function/fixed_point_quantize.hpp>
#include <nbla/function/global_average_pooling.hpp>
#include <nbla/function/inq_affine.hpp>
#include <nbla/function/inq_convolution.hpp>
#include <nbla/function/max_pooling.hpp>
#include <nbla/function/binary_sigmoid.hpp>
#include <nbla/function/binary_tanh.hpp>
#include <nbla/function/dequantize_linear.hpp>
#include <nbla/function/min_max_quantize.hpp>
#include <nbla/function/prune.hpp>
#include <nbla/function/quantize_linear.hpp>
#include <nbla/function/pow2_quantize.hpp>
#include <nbla/function/relu.hpp>

#include <chrono>
#include <cstdint>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

using namespace nbla;

namespace nbla_b200_runner {

Context context_for(const std::string &backend, const std::string &device_id) {
  if (backend == "cpu:float")
    return Context({"cpu:float"}, "CpuCachedArray", device_id);
  NBLA_CHECK(backend == "b200:float" || backend == "b200:half", error_code::value, "unknown backend %s",
             backend.c_str());
  init_b200();
  return b200_context(device_id, backend == "b200:half" ? "half" : "float");
}

FunctionPtr create_function(const std::string &name, const Context &ctx, const double *s, int n_s,
                            const std::vector<std::vector<int>> &ivs) {
  auto S = [&](int i) -> double {
    NBLA_CHECK(i < n_s, error_code::value, "missing scalar argument %d", i);
    return s[i];
  };
  auto V = [&](size_t i) -> const std::vector<int> & {
    NBLA_CHECK(i < ivs.size(), error_code::value, "missing vector argument %d", (int)i);
    return ivs[i];
  };
  if (name == "FixedPointQuantize")
    return create_FixedPointQuantize(ctx, S(0) != 0, (int)S(1), (float)S(2), S(3) != 0);
  if (name == "Pow2Quantize")
    return create_Pow2Quantize(ctx, S(0) != 0, S(1) != 0, (int)S(2), (int)S(3), S(4) != 0);
  if (name == "MinMaxQuantize")
    return create_MinMaxQuantize(ctx, (float)S(0), S(1) != 0, S(2) != 0, S(3) != 0, (float)S(4));
  if (name == "BinaryWeightAffine")
    return create_BinaryWeightAffine(ctx, (int)S(0), (float)S(1));
  if (name == "BinaryConnectAffine")
    return create_BinaryConnectAffine(ctx, (int)S(0), (float)S(1));
  if (name == "BinaryWeightConvolution")
    return create_BinaryWeightConvolution(ctx, (int)S(0), V(0), V(1), V(2), (int)S(1), (float)S(2));
  if (name == "BinaryConnectConvolution")
    return create_BinaryConnectConvolution(ctx, (int)S(0), V(0), V(1), V(2), (int)S(1), (float)S(2));
  if (name == "Affine")
    return create_Affine(ctx, (int)S(0));
  if (name == "Convolution")
    return create_Convolution(ctx, (int)S(0), V(0), V(1), V(2), (int)S(1), S(2) != 0);
  if (name == "BatchNormalization")
    return create_BatchNormalization(ctx, V(0), (float)S(0), (float)S(1), S(2) != 0, S(3) != 0, S(4) != 0);
  if (name == "ReLU")
    return create_ReLU(ctx, S(0) != 0);
  if (name == "MaxPooling")
    return create_MaxPooling(ctx, V(0), V(1), S(0) != 0, V(2), S(1) != 0);
  if (name == "GlobalAveragePooling")
    return create_GlobalAveragePooling(ctx);
  if (name == "Add2")
    return create_Add2(ctx, S(0) != 0);
  if (name == "BinarySigmoid")
    return create_BinarySigmoid(ctx);
  if (name == "BinaryTanh")
    return create_BinaryTanh(ctx);
  if (name == "INQAffine") // scalars: base_axis, num_bits, selection (0 = largest_abs, 1 = random), seed; ivecs: inq_iterations
    return create_INQAffine(ctx, (int)S(0), (int)S(1), ivs.at(0), S(2) != 0 ? "random" : "largest_abs", (int)S(3));
  if (name == "INQConvolution") // scalars: base_axis, group, num_bits, selection, seed; ivecs: pad, stride, dilation, inq_iterations
    return create_INQConvolution(ctx, (int)S(0), V(0), V(1), V(2), (int)S(1), (int)S(2), ivs.at(3),
                                 S(3) != 0 ? "random" : "largest_abs", (int)S(4));
  if (name == "QuantizeLinear") // scalars: round mode (0 = HALF_AWAY_FROM_ZERO, 1 = HALF_TO_EVEN), narrow_range, dtype
    return create_QuantizeLinear(ctx, S(0) != 0 ? "HALF_TO_EVEN" : "HALF_AWAY_FROM_ZERO", S(1) != 0, (int)S(2));
  if (name == "DequantizeLinear")
    return create_DequantizeLinear(ctx);
  if (name == "Prune")
    return create_Prune(ctx, (float)S(0));
  NBLA_ERROR(error_code::value, "unknown function %s", name.c_str());
}
} // namespace nbla_b200_runner
