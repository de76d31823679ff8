// One explicit-instantiation translation unit per template-bodied reference
// function, the hand-written equivalent of what the reference's code generator
// emits from src/nbla/function/function.cpp.tmpl:21-29. The Makefile compiles
// this file once per function with
//   -DNBHOST_SRC='<path of the reference .cpp>' -DNBHOST_CLASS=<ClassName>
// so the reference source is compiled where it lies and never copied.
// TEST INFRASTRUCTURE ONLY (part of the oracle build).
#include NBHOST_SRC
namespace nbla {
#ifdef NBHOST_TWO_TYPES // functions with a second type parameter for integer side data (INQAffine<float, int>)
template class NBHOST_CLASS<float, int>;
#else
template class NBHOST_CLASS<float>;
#endif
}
