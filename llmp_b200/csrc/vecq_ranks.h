// Measured ranks of the dense Q4_K llmp.vecq launch configurations on B200 (the role of the
// reference's src/kernels/ggml/measured_ranks.h and src/execution/rank_data.h: checked-in
// measurements that pick an implementation per shape; unmeasured shapes keep the ordinary
// rule).  Each row is the fastest configuration of one (k, n, fused GLU, tokens) product among
// the row-lane, row-MMA (sub-block columns and token columns), stream and generic kernels, each timed as a CUDA-graph replay over
// weight copies that together exceed the L2 (median of 6), on one B200 at 1,965 MHz; a
// configuration displaces the plain row-lane kernel only when it measured more than 3 %
// faster.  tests/test_vecq_gpu.py fails when a row names a configuration the library no
// longer has.
#ifndef LLMP_B200_CSRC_VECQ_RANKS_H_
#define LLMP_B200_CSRC_VECQ_RANKS_H_

namespace llmp_b200 {
namespace vecq {

struct MeasuredRank {
  int k, n, glu, tokens;  // tokens: the pass size 1, 2, 4 or 8 the row stands for
  const char* variant;
  float microseconds;
  int gbs;
};

constexpr MeasuredRank kMeasuredRanks[] = {
    // k, n, fused GLU, tokens, variant, microseconds a launch, GB/s of weight bytes
    {2560, 10240, 1, 1, "rowlane", 7.287f, 4047},
    {2560, 10240, 1, 2, "rowlane", 8.946f, 3297},
    {2560, 10240, 1, 4, "rowlane", 12.542f, 2351},
    {2560, 10240, 1, 8, "rowmma.t8", 16.011f, 1842},
    {10240, 2560, 0, 1, "rowmma.c2", 5.213f, 2829},
    {10240, 2560, 0, 2, "rowlane", 7.483f, 1971},
    {10240, 2560, 0, 4, "rowmma.t8", 10.561f, 1396},
    {10240, 2560, 0, 8, "rowmma.t8", 11.093f, 1329},
    {4096, 4096, 0, 1, "rowlane", 4.016f, 2350},
    {4096, 4096, 0, 2, "rowlane", 4.806f, 1964},
    {4096, 4096, 0, 4, "rowlane", 6.474f, 1458},
    {4096, 4096, 0, 8, "rowmma.t8c2", 7.079f, 1333},
    {4096, 14336, 1, 1, "rowlane", 16.293f, 4055},
    {4096, 14336, 1, 2, "rowlane", 20.101f, 3286},
    {4096, 14336, 1, 4, "l8r1u2w4", 28.192f, 2343},
    {4096, 14336, 1, 8, "rowmma.t8", 30.523f, 2164},
    {14336, 4096, 0, 1, "rowlane", 10.299f, 3207},
    {14336, 4096, 0, 2, "rowlane", 11.459f, 2882},
    {14336, 4096, 0, 4, "rowlane", 15.789f, 2092},
    {14336, 4096, 0, 8, "rowlane", 26.141f, 1264},
    {2048, 2048, 0, 1, "rowlane", 2.075f, 1137},
    {2048, 2048, 0, 2, "rowlane", 2.759f, 855},
    {2048, 2048, 0, 4, "rowlane", 4.255f, 554},
    {2048, 2048, 0, 8, "rowmma.t8", 5.214f, 452},
    {8192, 8192, 0, 1, "rowlane", 11.215f, 3366},
    {8192, 8192, 0, 2, "rowlane", 12.262f, 3079},
    {8192, 8192, 0, 4, "rowlane", 16.625f, 2271},
    {8192, 8192, 0, 8, "rowmma.t8", 24.492f, 1541},
    {2048, 1536, 0, 1, "rowlane", 2.056f, 861},
    {2048, 1536, 0, 2, "rowlane", 2.730f, 648},
    {2048, 1536, 0, 4, "rowlane", 4.215f, 420},
    {2048, 1536, 0, 8, "rowmma.t8", 5.112f, 346},
    {2048, 6144, 1, 1, "rowlane", 4.712f, 3004},
    {2048, 6144, 1, 2, "rowlane", 6.038f, 2344},
    {2048, 6144, 1, 4, "rowlane", 9.007f, 1572},
    {2048, 6144, 1, 8, "rowmma.t8c2", 10.270f, 1378},
    {6144, 2048, 0, 1, "rowlane", 3.928f, 1802},
    {6144, 2048, 0, 2, "rowlane", 4.724f, 1498},
    {6144, 2048, 0, 4, "rowmma", 5.646f, 1254},
    {6144, 2048, 0, 8, "rowmma.t8", 6.528f, 1084},
    {4096, 11008, 1, 1, "rowlane", 10.908f, 4650},
    {4096, 11008, 1, 2, "rowlane", 13.192f, 3845},
    {4096, 11008, 1, 4, "rowlane", 20.132f, 2520},
    {4096, 11008, 1, 8, "rowmma.t8", 23.428f, 2165},
    {11008, 4096, 0, 1, "rowmma", 8.008f, 3167},
    {11008, 4096, 0, 2, "rowlane", 9.796f, 2589},
    {11008, 4096, 0, 4, "rowlane", 13.428f, 1889},
    {11008, 4096, 0, 8, "rowmma.t8", 13.928f, 1821},
    {5120, 5120, 0, 1, "rowlane", 4.912f, 3002},
    {5120, 5120, 0, 2, "rowlane", 6.379f, 2312},
    {5120, 5120, 0, 4, "rowlane", 9.393f, 1570},
    {5120, 5120, 0, 8, "rowmma.t8", 10.183f, 1448},
    {5120, 27648, 1, 1, "l8r1u2w4", 33.920f, 4695},
    {5120, 27648, 1, 2, "l8r1u2w4", 40.944f, 3890},
    {5120, 27648, 1, 4, "l8r1u2w4", 60.360f, 2638},
    {5120, 27648, 1, 8, "rowmma.t8", 112.272f, 1418},
    {27648, 5120, 0, 1, "rowlane", 20.390f, 3905},
    {27648, 5120, 0, 2, "rowlane", 24.013f, 3316},
    {27648, 5120, 0, 4, "rowlane", 34.688f, 2295},
    {27648, 5120, 0, 8, "rowlane", 34.515f, 2307},
};
constexpr int kMeasuredRankCount = static_cast<int>(sizeof(kMeasuredRanks) / sizeof(kMeasuredRanks[0]));

}  // namespace vecq
}  // namespace llmp_b200

#endif  // LLMP_B200_CSRC_VECQ_RANKS_H_
