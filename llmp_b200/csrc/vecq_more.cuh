// Units of the other block types llmp.vecq takes (the reference hands them to GGML's vec_dot
// functions, src/kernels/ggml/vecq.cu:54-96): Q4_0, Q5_0, IQ4_NL (32-value blocks) and Q5_K,
// Q6_K (256-value super-blocks), for the generic kernel of vecq_impl.cuh.  The layouts are
// GGML's published block formats; the decode arithmetic here is this build's own and is
// checked against the double product of the decoded operands.  A unit gives, for each of its
// 32-value sub-blocks, that sub-block's share of the dot product with a Q8_1 block
// (`Dot`: d8 the block's scale, d8sum = d8 * sum of its codes).  Blocks are only 2-byte
// aligned in general (18, 22, 210 bytes), so units are fetched in 32-bit words where the
// address allows and in 16-bit halves otherwise.  Functional, not tuned: one launch
// configuration a type.
#ifndef LLMP_B200_CSRC_VECQ_MORE_CUH_
#define LLMP_B200_CSRC_VECQ_MORE_CUH_

#include "vecq_impl.cuh"

namespace llmp_b200 {
namespace vecq {

// `words` 32-bit words starting at a 2-byte aligned address.
template <int kWords>
__device__ __forceinline__ void LoadWords(const std::uint8_t* p, std::uint32_t (&w)[kWords]) {
  if ((reinterpret_cast<std::uintptr_t>(p) & 3u) == 0) {
    const auto* q = reinterpret_cast<const std::uint32_t*>(p);
#pragma unroll
    for (int i = 0; i < kWords; ++i) w[i] = __ldg(q + i);
  } else {
    const auto* h = reinterpret_cast<const unsigned short*>(p);
#pragma unroll
    for (int i = 0; i < kWords; ++i) {
      w[i] = static_cast<std::uint32_t>(__ldg(h + (2 * i))) |
             (static_cast<std::uint32_t>(__ldg(h + (2 * i) + 1)) << 16);
    }
  }
}

// Bits 0..3 of b to bit 4 of bytes 0..3.
__device__ __forceinline__ std::uint32_t FifthBits(std::uint32_t b) {
  return ((b & 1u) | ((b & 2u) << 7) | ((b & 4u) << 14) | ((b & 8u) << 21)) << 4;
}

__device__ __forceinline__ int Dot8(const int (&w)[8], const int (&xs)[8]) {
  int s = 0;
#pragma unroll
  for (int q = 0; q < 8; ++q) s = Dp4a(w[q], xs[q], s);
  return s;
}

// Q4_0 / Q5_0 / IQ4_NL: four blocks a unit (128 values).
template <int kTypeId>
struct Small32Unit {
  static constexpr int kType = kTypeId;
  static constexpr int kBlockBytes = kTypeId == LLMP_B200_TYPE_Q5_0 ? 22 : 18;
  static constexpr int kBlockElems = 32;
  static constexpr int kUnitElems = 128;
  static constexpr int kWords = kBlockBytes;  // 4 blocks * bytes / 4
  std::uint32_t w[kWords];

  static __device__ __forceinline__ int UnitsPerRow(int k) { return k / kUnitElems; }
  __device__ __forceinline__ void Zero() {
#pragma unroll
    for (int i = 0; i < kWords; ++i) w[i] = 0;
  }
  __device__ __forceinline__ void Load(const std::uint8_t* row, int u) {
    LoadWords<kWords>(row + (static_cast<std::size_t>(u) * kBlockBytes * 4), w);
  }
  // Byte `at` .. at + 3 of the unit (at even).
  __device__ __forceinline__ std::uint32_t Word(int at) const {
    if ((at & 3) == 0) return w[at >> 2];
    return __byte_perm(w[at >> 2], w[(at >> 2) + 1], 0x5432);
  }
  __device__ __forceinline__ float Dot(int b, const int (&xs)[8], float d8, float d8sum) const {
    const int base = b * kBlockBytes;
    const std::uint32_t head = Word(base & ~3);
    const float d = HalfBitsToFloat((base & 2) ? (head >> 16) : (head & 0xffffu));
    int v[8];
    if constexpr (kTypeId == LLMP_B200_TYPE_Q5_0) {
      const std::uint32_t top = Word(base + 2);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const std::uint32_t q = Word(base + 6 + (4 * j));
        v[j] = static_cast<int>((q & 0x0f0f0f0fu) | FifthBits((top >> (4 * j)) & 15u));
        v[4 + j] = static_cast<int>(((q >> 4) & 0x0f0f0f0fu) | FifthBits((top >> (16 + (4 * j))) & 15u));
      }
      // codes 0..31 stand for -16..15: the offset leaves through the block's code sum
      return d * ((d8 * static_cast<float>(Dot8(v, xs))) - (16.0f * d8sum));
    } else if constexpr (kTypeId == LLMP_B200_TYPE_Q4_0) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const std::uint32_t q = Word(base + 2 + (4 * j));
        v[j] = static_cast<int>(q & 0x0f0f0f0fu);
        v[4 + j] = static_cast<int>((q >> 4) & 0x0f0f0f0fu);
      }
      return d * ((d8 * static_cast<float>(Dot8(v, xs))) - (8.0f * d8sum));
    } else {
      // IQ4_NL: a nibble names one of 16 fixed levels (GGML's published table), four to a word.
      constexpr std::uint32_t kLevels[4] = {0xbfad9881u, 0xf6eaddcfu, 0x26190d01u, 0x71594535u};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const std::uint32_t q = Word(base + 2 + (4 * j));
        std::uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const std::uint32_t a = (q >> (8 * c)) & 15u, h = (q >> ((8 * c) + 4)) & 15u;
          lo |= ((kLevels[a >> 2] >> (8 * (a & 3u))) & 0xffu) << (8 * c);
          hi |= ((kLevels[h >> 2] >> (8 * (h & 3u))) & 0xffu) << (8 * c);
        }
        v[j] = static_cast<int>(lo);
        v[4 + j] = static_cast<int>(hi);
      }
      return d * d8 * static_cast<float>(Dot8(v, xs));
    }
  }
};

// Q5_K: 64 values a unit (sub-blocks 2j and 2j + 1 of chunk j), as Q4KUnit plus the fifth bits.
struct Q5KUnit {
  static constexpr int kType = LLMP_B200_TYPE_Q5_K;
  static constexpr int kBlockBytes = 176;
  static constexpr int kBlockElems = 256;
  static constexpr int kUnitElems = 64;
  uint4 head;      // d, dmin, scales[12]
  uint4 top[2];    // fifth bits: byte l, bit g = value l of sub-block g
  uint4 q[2];      // the chunk's 32 nibble bytes
  int chunk;

  static __device__ __forceinline__ int UnitsPerRow(int k) { return k / kUnitElems; }
  __device__ __forceinline__ void Zero() {
    head = top[0] = top[1] = q[0] = q[1] = make_uint4(0, 0, 0, 0);
    chunk = 0;
  }
  __device__ __forceinline__ void Load(const std::uint8_t* row, int u) {
    const std::uint8_t* sb = row + (static_cast<std::size_t>(u >> 2) * kBlockBytes);  // 16-byte aligned
    chunk = u & 3;
    head = LoadStream16(sb);
    top[0] = LoadStream16(sb + 16);
    top[1] = LoadStream16(sb + 32);
    q[0] = LoadStream16(sb + 48 + (chunk * 32));
    q[1] = LoadStream16(sb + 64 + (chunk * 32));
  }
  __device__ __forceinline__ float Dot(int b, const int (&xs)[8], float d8, float d8sum) const {
    std::uint32_t sc, mn;
    Q4KScalePair(head.y, head.z, head.w, chunk, &sc, &mn);
    const float d = HalfBitsToFloat(head.x & 0xffffu), dmin = HalfBitsToFloat(head.x >> 16);
    const std::uint32_t nib[8] = {q[0].x, q[0].y, q[0].z, q[0].w, q[1].x, q[1].y, q[1].z, q[1].w};
    const std::uint32_t tops[8] = {top[0].x, top[0].y, top[0].z, top[0].w,
                                   top[1].x, top[1].y, top[1].z, top[1].w};
    const int g = (2 * chunk) + b;
    int v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      v[j] = static_cast<int>(((nib[j] >> (4 * b)) & 0x0f0f0f0fu) | (((tops[j] >> g) & 0x01010101u) << 4));
    }
    const float scale = static_cast<float>((sc >> (8 * b)) & 0xffu);
    const float minimum = static_cast<float>((mn >> (8 * b)) & 0xffu);
    return ((d * scale) * d8 * static_cast<float>(Dot8(v, xs))) - ((dmin * minimum) * d8sum);
  }
};

// Q6_K: half a super-block a unit (128 values: sub-blocks l, l + 32, l + 64, l + 96).
struct Q6KUnit {
  static constexpr int kType = LLMP_B200_TYPE_Q6_K;
  static constexpr int kBlockBytes = 210;
  static constexpr int kBlockElems = 256;
  static constexpr int kUnitElems = 128;
  std::uint32_t lows[16];  // 64 bytes
  std::uint32_t tops[8];   // 32 bytes
  std::uint32_t scales[2]; // 8 int8
  std::uint32_t d;         // FP16 bits

  static __device__ __forceinline__ int UnitsPerRow(int k) { return k / kUnitElems; }
  __device__ __forceinline__ void Zero() {
#pragma unroll
    for (int i = 0; i < 16; ++i) lows[i] = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) tops[i] = 0;
    scales[0] = scales[1] = d = 0;
  }
  __device__ __forceinline__ void Load(const std::uint8_t* row, int u) {
    const std::uint8_t* sb = row + (static_cast<std::size_t>(u >> 1) * kBlockBytes);
    const int half = u & 1;
    LoadWords<16>(sb + (64 * half), lows);
    LoadWords<8>(sb + 128 + (32 * half), tops);
    LoadWords<2>(sb + 192 + (8 * half), scales);
    d = __ldg(reinterpret_cast<const unsigned short*>(sb + 208));
  }
  __device__ __forceinline__ float Dot(int b, const int (&xs)[8], float d8, float d8sum) const {
    (void)d8sum;
    // sub-block b: nibbles of bytes 32 * (b & 1) .., low (b < 2) or high; tops' bits 2b, 2b + 1
    int v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const std::uint32_t nib = (lows[(8 * (b & 1)) + j] >> (4 * (b >> 1))) & 0x0f0f0f0fu;
      const std::uint32_t two = ((tops[j] >> (2 * b)) & 0x03030303u) << 4;
      v[j] = static_cast<int>(__vsub4(nib | two, 0x20202020u));  // 0..63 -> -32..31
    }
    int s0 = 0, s1 = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      s0 = Dp4a(v[j], xs[j], s0);
      s1 = Dp4a(v[4 + j], xs[4 + j], s1);
    }
    // one int8 scale per 16 values: scales[2b], scales[2b + 1] of the half
    const std::uint32_t word = scales[b >> 1];
    const int sc0 = static_cast<int>(static_cast<signed char>((word >> (16 * (b & 1))) & 0xffu));
    const int sc1 = static_cast<int>(static_cast<signed char>((word >> ((16 * (b & 1)) + 8)) & 0xffu));
    return HalfBitsToFloat(d) * d8 * static_cast<float>((sc0 * s0) + (sc1 * s1));
  }
};

}  // namespace vecq
}  // namespace llmp_b200

#endif  // LLMP_B200_CSRC_VECQ_MORE_CUH_
