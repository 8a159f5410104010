// Q4_K instantiations of the vecq kernels.
#include "vecq_rowlane.cuh"
#include "vecq_rowmma.cuh"
namespace llmp_b200 {
namespace vecq {
template cudaError_t LaunchType<Q4KUnit>(const Desc&, int, const Variant&, cudaStream_t);
template cudaError_t LaunchStream<Q4KUnit>(const Desc&, int, const StreamPlan&, cudaStream_t);
template cudaError_t LaunchStream<Q4KBlockUnit>(const Desc&, int, const StreamPlan&, cudaStream_t);

cudaError_t LaunchRowLane(const Desc& d, int p, const RowLanePlan& plan, cudaStream_t stream) {
  const bool glu = d.glu != LLMP_B200_GLU_NONE;
#define LLMP_P(PP)                                                   \
  if (p == PP)                                                       \
    return plan.half ? (glu ? LaunchRowLaneOne<PP, true, true>(d, plan, stream)    \
                            : LaunchRowLaneOne<PP, false, true>(d, plan, stream))  \
                     : (glu ? LaunchRowLaneOne<PP, true, false>(d, plan, stream)   \
                            : LaunchRowLaneOne<PP, false, false>(d, plan, stream));
  LLMP_P(1) LLMP_P(2) LLMP_P(4) LLMP_P(8)
#undef LLMP_P
  return cudaErrorInvalidValue;
}

cudaError_t LaunchRowMma(const Desc& d, int p, const RowMmaPlan& plan, cudaStream_t stream) {
  const bool glu = d.glu != LLMP_B200_GLU_NONE;
#define LLMP_P(PP)                                                       \
  if (p == PP)                                                           \
    return glu ? LaunchRowMmaOne<PP, true>(d, plan, stream)              \
               : LaunchRowMmaOne<PP, false>(d, plan, stream);
  LLMP_P(1) LLMP_P(2) LLMP_P(4) LLMP_P(8)
#undef LLMP_P
  return cudaErrorInvalidValue;
}
cudaError_t LaunchRowMmaTokens(const Desc& d, const RowMmaPlan& plan, cudaStream_t stream) {
  return d.glu != LLMP_B200_GLU_NONE ? LaunchRowMmaTokensOne<true>(d, plan, stream)
                                     : LaunchRowMmaTokensOne<false>(d, plan, stream);
}
}  // namespace vecq
}  // namespace llmp_b200
