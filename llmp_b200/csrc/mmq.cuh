// Internal launcher of the Q4_K x Q8_1-MMQ tensor-core GEMM, shared by the
// dense / per-expert entry point and the grouped (worklist) one.
#ifndef LLMP_B200_CSRC_MMQ_CUH_
#define LLMP_B200_CSRC_MMQ_CUH_

#include <cstdint>

#include "llmp_b200.h"

namespace llmp_b200 {

constexpr int kMmqTileCols = 128;  // token columns a tile

// The GLU write-back: where the Q8_1-MMQ blocks of the GLU go, which GLU.
struct MmqGlu {
  void* blocks;
  int glu;
  float limit;
};

// worklist (device, or null): int32 {count, (expert, first column) x count};
// grid row y takes entry y and exits when y >= count.  max_tiles: its capacity.
// sums (device, or null): verification output, the int32 group sums [col][row][k / 32].
// glu (or null): the slab interleaves gate and up rows; the GLU of every pair is requantized
// into glu->blocks instead of the F32 output.
int LaunchMmq(const llmp_b200_mmq_desc& d, const std::int32_t* worklist, int max_tiles,
              void* stream, std::int32_t* sums = nullptr, const MmqGlu* glu = nullptr);

}  // namespace llmp_b200

#endif  // LLMP_B200_CSRC_MMQ_CUH_
