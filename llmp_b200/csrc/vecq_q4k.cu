// Q4_K instantiations of the vecq kernels.
#include "vecq_impl.cuh"
namespace llmp_b200 {
namespace vecq {
template cudaError_t LaunchType<Q4KUnit>(const Desc&, int, const Variant&, cudaStream_t);
}  // namespace vecq
}  // namespace llmp_b200
