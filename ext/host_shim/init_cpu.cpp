// Hand-written init_cpu() for the oracle build of the reference runtime.
// The reference generates this file with Mako from src/nbla/init.cpp.tmpl:44-111;
// Mako is unavailable, so the registrations the hot path needs are written
// out here: the "cpu" backend, the CPU array classes with their
// synchronizers and group, and one NBLA_REGISTER_FUNCTION_IMPL per function
// for the "cpu:float" type configuration.
// TEST INFRASTRUCTURE ONLY.
#include <nbla/array/cpu_array.hpp>
#include <nbla/array_registry.hpp>
#include <nbla/backend_registry.hpp>
#include <nbla/cpu.hpp>
#include <nbla/function_registry.hpp>
#include <nbla/init.hpp>

#include <nbla/function/abs.hpp>
#include <nbla/function/add2.hpp>
#include <nbla/function/add_scalar.hpp>
#include <nbla/function/affine.hpp>
#include <nbla/function/average_pooling.hpp>
#include <nbla/function/batch_normalization.hpp>
#include <nbla/function/bc_add2.hpp>
#include <nbla/function/binary_connect_affine.hpp>
#include <nbla/function/binary_connect_convolution.hpp>
#include <nbla/function/binary_weight_affine.hpp>
#include <nbla/function/binary_weight_convolution.hpp>
#include <nbla/function/broadcast.hpp>
#include <nbla/function/convolution.hpp>
#include <nbla/function/div2.hpp>
#include <nbla/function/fixed_point_quantize.hpp>
#include <nbla/function/global_average_pooling.hpp>
#include <nbla/function/greater.hpp>
#include <nbla/function/greater_equal.hpp>
#include <nbla/function/identity.hpp>
#include <nbla/function/less.hpp>
#include <nbla/function/less_equal.hpp>
#include <nbla/function/max.hpp>
#include <nbla/function/max_pooling.hpp>
#include <nbla/function/maximum2.hpp>
#include <nbla/function/min.hpp>
#include <nbla/function/binary_sigmoid.hpp>
#include <nbla/function/binary_tanh.hpp>
#include <nbla/function/dequantize_linear.hpp>
#include <nbla/function/min_max_quantize.hpp>
#include <nbla/function/prune.hpp>
#include <nbla/function/quantize_linear.hpp>
#include <nbla/function/minimum2.hpp>
#include <nbla/function/mul2.hpp>
#include <nbla/function/mul_scalar.hpp>
#include <nbla/function/pow2_quantize.hpp>
#include <nbla/function/pow_scalar.hpp>
#include <nbla/function/relu.hpp>
#include <nbla/function/round.hpp>
#include <nbla/function/sign.hpp>
#include <nbla/function/sub2.hpp>
#include <nbla/function/inq_affine.hpp>
#include <nbla/function/inq_convolution.hpp>
#include <nbla/function/sum.hpp>
#include <nbla/function/transpose.hpp>

#include <mutex>

namespace nbla {

#define REG(NAME, ...)                                                         \
  {                                                                            \
    using NAME##_float = NAME<float>;                                          \
    NBLA_REGISTER_FUNCTION_IMPL(NAME, NAME##_float, "cpu:float",               \
                                ##__VA_ARGS__);                                \
  }

void init_cpu() {
  static std::mutex m;
  std::lock_guard<std::mutex> lock(m);
  static volatile bool is_initialized = false;
  if (is_initialized)
    return;
  is_initialized = true;

  NBLA_REGISTER_BACKEND("cpu", []() { return SingletonManager::get<Cpu>(); });

  NBLA_REGISTER_ARRAY_CREATOR(CpuArray);
  SingletonManager::get<Cpu>()->register_array_class("CpuArray");
  NBLA_REGISTER_ARRAY_CREATOR(CpuCachedArray);
  SingletonManager::get<Cpu>()->register_array_class("CpuCachedArray");
  NBLA_REGISTER_ARRAY_SYNCHRONIZER(CpuArray, CpuCachedArray,
                                   synchronizer_default);
  NBLA_REGISTER_ARRAY_SYNCHRONIZER(CpuCachedArray, CpuArray,
                                   synchronizer_default);
  NBLA_REGISTER_ARRAY_GROUP(CpuArray, cpu);
  NBLA_REGISTER_ARRAY_GROUP(CpuCachedArray, cpu);

  typedef const vector<int> &ivec;
  REG(FixedPointQuantize, bool, int, float, bool);
  REG(Pow2Quantize, bool, bool, int, int, bool);
  REG(MinMaxQuantize, float, bool, bool, bool, float);
  REG(BinaryWeightAffine, int, float);
  REG(BinaryWeightConvolution, int, ivec, ivec, ivec, int, float);
  REG(BinaryConnectAffine, int, float);
  REG(BinaryConnectConvolution, int, ivec, ivec, ivec, int, float);
  REG(Sign, float);
  REG(Abs);
  REG(Sum, ivec, bool);
  REG(MulScalar, double, bool);
  REG(AddScalar, double, bool);
  REG(PowScalar, double, bool);
  REG(Mul2, bool);
  REG(Add2, bool);
  REG(BcAdd2, bool);
  REG(Sub2, bool);
  REG(Div2, bool);
  REG(Round);
  REG(Minimum2);
  REG(Maximum2);
  REG(Min, ivec, bool, bool, bool);
  REG(Max, ivec, bool, bool, bool);
  REG(Broadcast, ivec);
  REG(Identity);
  REG(Transpose, ivec);
  REG(Greater);
  REG(GreaterEqual);
  REG(Less);
  REG(LessEqual);
  REG(Affine, int);
  REG(Convolution, int, ivec, ivec, ivec, int, bool);
  REG(BatchNormalization, ivec, float, float, bool, bool, bool);
  REG(ReLU, bool);
  REG(MaxPooling, ivec, ivec, bool, ivec, bool);
  REG(AveragePooling, ivec, ivec, bool, ivec, bool, bool);
  REG(GlobalAveragePooling);
  REG(BinarySigmoid);
  REG(BinaryTanh);
  REG(QuantizeLinear, const string &, bool, int);
  REG(DequantizeLinear);
  REG(Prune, float);
  {
    using INQAffine_float_int = INQAffine<float, int>;
    NBLA_REGISTER_FUNCTION_IMPL(INQAffine, INQAffine_float_int, "cpu:float", int, int, ivec, const string &, int);
    using INQConvolution_float_int = INQConvolution<float, int>;
    NBLA_REGISTER_FUNCTION_IMPL(INQConvolution, INQConvolution_float_int, "cpu:float", int, ivec, ivec, ivec, int, int,
                                ivec, const string &, int);
  }
}

void clear_cpu_memory_cache() {
  SingletonManager::get<Cpu>()->caching_allocator()->free_unused_caches();
}
void print_cpu_memory_cache_map() {
  SingletonManager::get<Cpu>()->caching_allocator()->print_memory_cache_map();
}
vector<string> cpu_array_classes() {
  return SingletonManager::get<Cpu>()->array_classes();
}
void _cpu_set_array_classes(const vector<string> &a) {
  return SingletonManager::get<Cpu>()->_set_array_classes(a);
}
void cpu_device_synchronize(const string &device) {}
int cpu_get_device_count() { return 1; }
vector<string> cpu_get_devices() { return {"0"}; }
} // namespace nbla
