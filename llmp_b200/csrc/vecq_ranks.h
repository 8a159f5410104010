// Measured ranks of the dense Q4_K llmp.vecq launch configurations on B200 (the role of the
// reference's src/kernels/ggml/measured_ranks.h and src/execution/rank_data.h: checked-in
// measurements that pick an implementation per shape; unmeasured shapes keep the ordinary
// rule).  Each row is the fastest configuration of one (k, n, fused GLU, tokens) product among
// the row-lane, row-MMA, stream and generic kernels, each timed as a CUDA-graph replay over
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
    {2560, 10240, 1, 1, "rowlane", 8.784f, 3357},
    {2560, 10240, 1, 2, "rowlane", 10.567f, 2791},
    {2560, 10240, 1, 4, "rowlane", 14.096f, 2092},
    {2560, 10240, 1, 8, "rowlane", 31.543f, 935},
    {10240, 2560, 0, 1, "rowmma.c2", 5.202f, 2835},
    {10240, 2560, 0, 2, "rowmma", 8.281f, 1781},
    {10240, 2560, 0, 4, "rowmma", 11.224f, 1314},
    {10240, 2560, 0, 8, "rowmma", 17.074f, 864},
    {4096, 4096, 0, 1, "rowlane", 3.631f, 2599},
    {4096, 4096, 0, 2, "rowmma", 4.657f, 2026},
    {4096, 4096, 0, 4, "rowlane", 7.164f, 1317},
    {4096, 4096, 0, 8, "rowmma.c2", 9.474f, 996},
    {4096, 14336, 1, 1, "l8r1u2w4", 18.464f, 3578},
    {4096, 14336, 1, 2, "rowlane", 25.883f, 2552},
    {4096, 14336, 1, 4, "rowmma", 32.251f, 2048},
    {4096, 14336, 1, 8, "rowlane", 63.216f, 1045},
    {14336, 4096, 0, 1, "rowmma", 11.069f, 2984},
    {14336, 4096, 0, 2, "rowmma", 13.099f, 2522},
    {14336, 4096, 0, 4, "rowmma", 17.533f, 1884},
    {14336, 4096, 0, 8, "rowlane", 29.213f, 1131},
    {2048, 2048, 0, 1, "rowlane", 2.398f, 984},
    {2048, 2048, 0, 2, "rowlane", 3.021f, 781},
    {2048, 2048, 0, 4, "rowmma", 4.269f, 553},
    {2048, 2048, 0, 8, "rowmma", 6.031f, 391},
    {8192, 8192, 0, 1, "rowmma.c2", 11.040f, 3419},
    {8192, 8192, 0, 2, "rowmma.c2", 13.344f, 2829},
    {8192, 8192, 0, 4, "rowmma", 18.263f, 2067},
    {8192, 8192, 0, 8, "rowlane", 31.200f, 1210},
    {2048, 1536, 0, 1, "rowlane", 2.232f, 793},
    {2048, 1536, 0, 2, "rowlane", 2.979f, 594},
    {2048, 1536, 0, 4, "rowmma", 4.114f, 430},
    {2048, 1536, 0, 8, "rowmma", 5.839f, 303},
    {2048, 6144, 1, 1, "rowlane", 5.259f, 2692},
    {2048, 6144, 1, 2, "rowlane", 6.814f, 2077},
    {2048, 6144, 1, 4, "rowlane", 9.784f, 1447},
    {2048, 6144, 1, 8, "rowlane", 17.121f, 827},
    {6144, 2048, 0, 1, "rowlane", 3.742f, 1891},
    {6144, 2048, 0, 2, "rowmma", 4.934f, 1435},
    {6144, 2048, 0, 4, "rowmma", 5.655f, 1252},
    {6144, 2048, 0, 8, "rowmma", 8.567f, 826},
    {4096, 11008, 1, 1, "rowlane", 13.408f, 3783},
    {4096, 11008, 1, 2, "rowlane", 16.432f, 3087},
    {4096, 11008, 1, 4, "rowlane", 22.896f, 2215},
    {4096, 11008, 1, 8, "rowmma", 55.968f, 906},
    {11008, 4096, 0, 1, "rowmma", 7.922f, 3202},
    {11008, 4096, 0, 2, "rowmma", 9.710f, 2612},
    {11008, 4096, 0, 4, "rowmma", 14.074f, 1802},
    {11008, 4096, 0, 8, "rowmma", 20.650f, 1228},
    {5120, 5120, 0, 1, "rowlane", 6.037f, 2443},
    {5120, 5120, 0, 2, "rowmma", 7.333f, 2011},
    {5120, 5120, 0, 4, "rowmma", 10.033f, 1470},
    {5120, 5120, 0, 8, "rowmma", 15.009f, 982},
    {5120, 27648, 1, 1, "l8r1u2w4", 36.536f, 4359},
    {5120, 27648, 1, 2, "l8r1u2w4", 56.240f, 2832},
    {5120, 27648, 1, 4, "rowmma", 75.648f, 2105},
    {5120, 27648, 1, 8, "rowlane", 150.488f, 1058},
    {27648, 5120, 0, 1, "rowlane", 25.574f, 3114},
    {27648, 5120, 0, 2, "rowlane", 30.720f, 2592},
    {27648, 5120, 0, 4, "rowlane", 41.792f, 1905},
    {27648, 5120, 0, 8, "rowlane", 41.818f, 1904},
};
constexpr int kMeasuredRankCount = static_cast<int>(sizeof(kMeasuredRanks) / sizeof(kMeasuredRanks[0]));

}  // namespace vecq
}  // namespace llmp_b200

#endif  // LLMP_B200_CSRC_VECQ_RANKS_H_
