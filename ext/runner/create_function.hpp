// Function creation by name for the C bindings of this directory: the
// constructor arguments arrive as a list of scalars and a list of integer
// vectors, in the order of the function's NBLA_REGISTER_FUNCTION_HEADER.
#ifndef NBLA_B200_RUNNER_CREATE_FUNCTION_HPP_
#define NBLA_B200_RUNNER_CREATE_FUNCTION_HPP_

#include <nbla/context.hpp>
#include <nbla/function.hpp>

#include <string>
#include <vector>

namespace nbla_b200_runner {
nbla::FunctionPtr create_function(const std::string &name, const nbla::Context &ctx, const double *scalars,
                                  int n_scalars, const std::vector<std::vector<int>> &int_vectors);
/// Context for a backend string: "cpu:float" or "b200:float" (loads the extension on first use).
nbla::Context context_for(const std::string &backend, const std::string &device_id = "0");
} // namespace nbla_b200_runner
#endif
