// llmp.vecq over the other block types (vecq_more.cuh): instantiations and their launcher.
#include "vecq_more.cuh"

namespace llmp_b200 {
namespace vecq {
namespace {

template <typename Unit, int P>
cudaError_t LaunchP(const Desc& d, cudaStream_t stream) {
  // One configuration a type: 8 lanes a row, one row a team, one unit a lane in flight.
  return d.glu != LLMP_B200_GLU_NONE ? LaunchOne<Unit, P, 8, 1, 1, true>(d, 4, stream)
                                     : LaunchOne<Unit, P, 8, 1, 1, false>(d, 4, stream);
}

template <typename Unit>
cudaError_t LaunchUnit(const Desc& d, int p, cudaStream_t stream) {
  switch (p) {
    case 1: return LaunchP<Unit, 1>(d, stream);
    case 2: return LaunchP<Unit, 2>(d, stream);
    case 4: return LaunchP<Unit, 4>(d, stream);
    default: return LaunchP<Unit, 8>(d, stream);
  }
}

}  // namespace

cudaError_t LaunchMore(int type, const Desc& d, int p, cudaStream_t stream) {
  switch (type) {
    case LLMP_B200_TYPE_Q4_0: return LaunchUnit<Small32Unit<LLMP_B200_TYPE_Q4_0>>(d, p, stream);
    case LLMP_B200_TYPE_Q5_0: return LaunchUnit<Small32Unit<LLMP_B200_TYPE_Q5_0>>(d, p, stream);
    case LLMP_B200_TYPE_IQ4_NL: return LaunchUnit<Small32Unit<LLMP_B200_TYPE_IQ4_NL>>(d, p, stream);
    case LLMP_B200_TYPE_Q5_K: return LaunchUnit<Q5KUnit>(d, p, stream);
    case LLMP_B200_TYPE_Q6_K: return LaunchUnit<Q6KUnit>(d, p, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace vecq
}  // namespace llmp_b200
