// Q8_0 instantiations of the vecq kernels (8-byte aligned units and the
// 2-byte aligned fallback).
#include "vecq_stream.cuh"
namespace llmp_b200 {
namespace vecq {
template cudaError_t LaunchType<Q8_0Unit<4>>(const Desc&, int, const Variant&, cudaStream_t);
template cudaError_t LaunchType<Q8_0Unit<1>>(const Desc&, int, const Variant&, cudaStream_t);
template cudaError_t LaunchStream<Q8_0Unit<4>>(const Desc&, int, const StreamPlan&, cudaStream_t);
}  // namespace vecq
}  // namespace llmp_b200
