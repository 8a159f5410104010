// Q4_K instantiations of the vecq kernels.
#include "vecq_stream.cuh"
namespace llmp_b200 {
namespace vecq {
template cudaError_t LaunchType<Q4KUnit>(const Desc&, int, const Variant&, cudaStream_t);
template cudaError_t LaunchStream<Q4KUnit>(const Desc&, int, const StreamPlan&, cudaStream_t);
template cudaError_t LaunchStream<Q4KBlockUnit>(const Desc&, int, const StreamPlan&, cudaStream_t);
}  // namespace vecq
}  // namespace llmp_b200
