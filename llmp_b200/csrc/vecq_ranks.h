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
    {2560, 10240, 1, 1, "rowlane", 8.432f, 3498},
    {2560, 10240, 1, 2, "rowlane", 10.405f, 2834},
    {2560, 10240, 1, 4, "rowlane", 13.886f, 2124},
    {2560, 10240, 1, 8, "rowmma.t8", 15.849f, 1861},
    {10240, 2560, 0, 1, "rowmma.c2", 5.298f, 2783},
    {10240, 2560, 0, 2, "rowlane", 8.546f, 1725},
    {10240, 2560, 0, 4, "rowmma.t8", 10.827f, 1362},
    {10240, 2560, 0, 8, "rowmma.t8", 11.311f, 1304},
    {4096, 4096, 0, 1, "rowlane", 3.350f, 2817},
    {4096, 4096, 0, 2, "rowmma", 4.714f, 2002},
    {4096, 4096, 0, 4, "rowmma.t8c2", 6.498f, 1452},
    {4096, 4096, 0, 8, "rowmma.t8c2", 7.071f, 1335},
    {4096, 14336, 1, 1, "l8r1u2w4", 16.800f, 3932},
    {4096, 14336, 1, 2, "l8r1u2w4", 20.677f, 3195},
    {4096, 14336, 1, 4, "l8r1u2w4", 28.357f, 2330},
    {4096, 14336, 1, 8, "rowmma.t8", 30.517f, 2165},
    {14336, 4096, 0, 1, "rowmma", 11.085f, 2980},
    {14336, 4096, 0, 2, "rowmma", 13.259f, 2491},
    {14336, 4096, 0, 4, "rowmma", 17.568f, 1880},
    {14336, 4096, 0, 8, "rowlane", 28.381f, 1164},
    {2048, 2048, 0, 1, "rowlane", 2.231f, 1058},
    {2048, 2048, 0, 2, "rowlane", 3.021f, 781},
    {2048, 2048, 0, 4, "rowmma", 4.293f, 550},
    {2048, 2048, 0, 8, "rowmma.t8", 5.197f, 454},
    {8192, 8192, 0, 1, "rowmma.c2", 11.232f, 3361},
    {8192, 8192, 0, 2, "rowmma.c2", 13.391f, 2819},
    {8192, 8192, 0, 4, "rowmma", 18.703f, 2018},
    {8192, 8192, 0, 8, "rowmma.t8", 24.515f, 1540},
    {2048, 1536, 0, 1, "rowlane", 2.265f, 781},
    {2048, 1536, 0, 2, "rowlane", 2.956f, 599},
    {2048, 1536, 0, 4, "rowmma", 4.101f, 431},
    {2048, 1536, 0, 8, "rowmma.t8", 5.095f, 347},
    {2048, 6144, 1, 1, "l8r1u2w4", 5.114f, 2768},
    {2048, 6144, 1, 2, "l8r1u2w4", 6.406f, 2210},
    {2048, 6144, 1, 4, "rowlane", 9.587f, 1477},
    {2048, 6144, 1, 8, "rowmma.t8c2", 10.269f, 1378},
    {6144, 2048, 0, 1, "rowlane", 3.477f, 2036},
    {6144, 2048, 0, 2, "rowlane", 4.994f, 1417},
    {6144, 2048, 0, 4, "rowmma", 5.704f, 1241},
    {6144, 2048, 0, 8, "rowmma.t8", 6.554f, 1080},
    {4096, 11008, 1, 1, "rowlane", 12.748f, 3979},
    {4096, 11008, 1, 2, "rowlane", 15.992f, 3172},
    {4096, 11008, 1, 4, "rowlane", 22.240f, 2281},
    {4096, 11008, 1, 8, "rowmma.t8", 23.632f, 2146},
    {11008, 4096, 0, 1, "rowmma", 8.058f, 3147},
    {11008, 4096, 0, 2, "rowmma", 9.834f, 2579},
    {11008, 4096, 0, 4, "rowmma.t8", 13.492f, 1880},
    {11008, 4096, 0, 8, "rowmma.t8", 14.060f, 1804},
    {5120, 5120, 0, 1, "rowlane", 5.691f, 2591},
    {5120, 5120, 0, 2, "rowlane", 7.486f, 1970},
    {5120, 5120, 0, 4, "rowmma.t8", 9.502f, 1552},
    {5120, 5120, 0, 8, "rowmma.t8", 10.155f, 1452},
    {5120, 27648, 1, 1, "l8r1u2w4", 34.120f, 4667},
    {5120, 27648, 1, 2, "l8r1u2w4", 41.416f, 3845},
    {5120, 27648, 1, 4, "l8r1u2w4", 60.928f, 2614},
    {5120, 27648, 1, 8, "rowmma.t8", 112.464f, 1416},
    {27648, 5120, 0, 1, "rowlane", 23.635f, 3369},
    {27648, 5120, 0, 2, "rowlane", 28.685f, 2776},
    {27648, 5120, 0, 4, "rowlane", 40.064f, 1987},
    {27648, 5120, 0, 8, "rowlane", 39.642f, 2009},
};
constexpr int kMeasuredRankCount = static_cast<int>(sizeof(kMeasuredRanks) / sizeof(kMeasuredRanks[0]));

}  // namespace vecq
}  // namespace llmp_b200

#endif  // LLMP_B200_CSRC_VECQ_RANKS_H_
