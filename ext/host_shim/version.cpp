// Replaces the generated src/nbla/version.cpp (version.cpp.tmpl) for the
// oracle build of the reference runtime. TEST INFRASTRUCTURE ONLY.
#include <nbla/common.hpp>
#include <string>
namespace nbla {
using std::string;
const string nbla_version(void) { return "1.40.0.dev1+oracle"; }
const string nbla_author(void) { return "reference runtime, oracle build"; }
const string nbla_author_email(void) { return ""; }
const string nbla_build_number(void) { return "0"; }
}
