// Routed-expert (MoE) products on B200: the expert counting sort, the grouped
// expert GEMM over expert-sorted rows, the GLU + requantization between the
// two expert GEMMs, and the ordered weighted combine.
//
// Interfaces follow the reference's routed path (src/kernels/ggml/moe_layout.h
// :47-83 RouteLayout, llmp_moe.cu:81-160 route, :308-435 quantize / GLU /
// combine, moe_cutlass.h:48-76 grouped GEMM).  The reference's grouped GEMM
// multiplies NVFP4 operands with CUTLASS; this build's experts are Q4_K, so
// the grouped GEMM is the Q4_K x Q8_1-MMQ tensor-core kernel of mmq.cu driven
// by a tile worklist built ON THE DEVICE from the route's offsets (the role
// of the reference's SetupGroups): nothing waits on the host.
#include "mmq.cuh"
#include "tc.cuh"

namespace llmp_b200 {
namespace {

constexpr int kRouteChunk = 64;   // tokens a counting block (moe_layout.h:42)
constexpr int kScaleRows = 128;   // rows a group's scales are padded to (:44)
constexpr int kMaxExperts = 1024;

struct Route {
  std::int32_t* offsets;
  std::int32_t* scale_rows;
  std::int32_t* position;
  std::int32_t* token;
  std::int32_t* expert;
  std::int32_t* counts;
  int experts, used, tokens, chunks;
};

__host__ Route RouteOf(std::int32_t* base, int experts, int used, int tokens) {
  const std::int64_t slots = static_cast<std::int64_t>(used) * tokens;
  Route r;
  r.experts = experts;
  r.used = used;
  r.tokens = tokens;
  r.chunks = (tokens + kRouteChunk - 1) / kRouteChunk;
  r.offsets = base;
  r.scale_rows = base + (experts + 1);
  r.position = base + (2 * (experts + 1));
  r.token = r.position + slots;
  r.expert = r.token + slots;
  r.counts = r.expert + slots;
  return r;
}

// The whole counting sort in ONE launch (the reference queues three kernels,
// llmp_moe.cu:81-160; the blob they leave, moe_layout.h:47-83, is reproduced
// word for word).  A thread-block cluster of 1 to 8 CTAs, sized by the chunk
// count, walks four phases separated by cluster barriers:
//   1. a warp owns whole 64-token chunks.  It clears its chunk's row of
//      `counts`, then takes the chunk's slots 32 at a time in slot order:
//      lanes naming the same expert find each other with match.any, the first
//      of them bumps the chunk's count for that expert (a plain read-modify-
//      write: the row is the warp's own) and every lane learns its ordinal
//      within (chunk, expert), parked in position[slot];
//   2. a thread an expert turns its column of `counts` into the exclusive
//      prefix over the chunks and leaves the expert's total in offsets[e + 1];
//   3. every CTA scans the totals into its own shared copy of the offsets
//      (CTA 0 also writes offsets and scale_rows out, after a barrier that
//      lets the others finish reading the totals);
//   4. a thread a slot: row = offsets[e] + counts[chunk][e] + ordinal.
// No atomics, and rows keep token order within an expert by construction.
constexpr int kRouteThreads = 1024;

__device__ __forceinline__ void ClusterSync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n"
               "barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ unsigned ClusterRank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ unsigned ClusterSize() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}

__global__ void __launch_bounds__(kRouteThreads, 1)
RouteKernel(const std::int32_t* __restrict__ ids, int ids_stride, Route r) {
  __shared__ int base[kMaxExperts + 1];   // this CTA's copy of the offsets
  __shared__ int warp_sums[2][32];
  const int tid = static_cast<int>(threadIdx.x);
  const int lane = tid & 31;
  const int ctas = static_cast<int>(ClusterSize());
  const int cta = static_cast<int>(ClusterRank());
  const int gthread = (cta * kRouteThreads) + tid;
  const int gthreads = ctas * kRouteThreads;
  const int gwarp = gthread >> 5;
  const int gwarps = gthreads >> 5;
  const std::int64_t slots = static_cast<std::int64_t>(r.used) * r.tokens;

  // Rows no slot reaches read as row 0 of expert 0.
  for (std::int64_t i = gthread; i < slots; i += gthreads) {
    r.token[i] = 0;
    r.expert[i] = 0;
  }
  // ---- 1: per-chunk counts and each slot's ordinal within (chunk, expert)
  for (int c = gwarp; c < r.chunks; c += gwarps) {
    std::int32_t* row = r.counts + (static_cast<std::int64_t>(c) * r.experts);
    for (int e = lane; e < r.experts; e += 32) row[e] = 0;
    __syncwarp();
    const int t0 = c * kRouteChunk;
    const int n = (min(t0 + kRouteChunk, r.tokens) - t0) * r.used;
    for (int i0 = 0; i0 < n; i0 += 32) {
      const int i = i0 + lane;
      int e = -1;
      if (i < n) {
        e = ids[(static_cast<std::int64_t>(t0 + (i / r.used)) * ids_stride) + (i % r.used)];
        if (e < 0 || e >= r.experts) e = -1;
      }
      // lanes without a valid id all fall in the -1 group and write nothing
      const unsigned same = __match_any_sync(0xffffffffu, e);
      const int first = __ffs(static_cast<int>(same)) - 1;
      int seen = 0;
      if (e >= 0 && lane == first) {
        seen = row[e];
        row[e] = seen + __popc(same);
      }
      seen = __shfl_sync(0xffffffffu, seen, first);
      if (i < n) {
        r.position[(static_cast<std::int64_t>(t0) * r.used) + i] =
            e < 0 ? -1 : seen + __popc(same & ((1u << lane) - 1u));
      }
      __syncwarp();  // the next batch's leaders read what this batch's wrote
    }
  }
  ClusterSync();
  // ---- 2: counts -> exclusive prefix over the chunks; totals into offsets[e + 1]
  for (int e = gthread; e < r.experts; e += gthreads) {
    int running = 0;
    for (int c = 0; c < r.chunks; ++c) {
      std::int32_t* at = r.counts + (static_cast<std::int64_t>(c) * r.experts) + e;
      const int v = *at;
      *at = running;
      running += v;
    }
    r.offsets[e + 1] = running;
  }
  ClusterSync();
  // ---- 3: the offsets (and the rows rounded up to 128 per expert): a block scan
  // of up to 1024 totals, one a thread, kept in shared memory by every CTA.
  {
    const int total = tid < r.experts ? r.offsets[tid + 1] : 0;
    int v[2] = {total, (total + kScaleRows - 1) / kScaleRows * kScaleRows};
#pragma unroll
    for (int w = 0; w < 2; ++w) {
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, v[w], d);
        if (lane >= d) v[w] += up;
      }
      if (lane == 31) warp_sums[w][tid >> 5] = v[w];
    }
    __syncthreads();
    if (tid < 32) {
#pragma unroll
      for (int w = 0; w < 2; ++w) {
        int x = warp_sums[w][tid];
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const int up = __shfl_up_sync(0xffffffffu, x, d);
          if (lane >= d) x += up;
        }
        warp_sums[w][tid] = x;  // inclusive over the warps
      }
    }
    __syncthreads();
    const int before0 = (tid >> 5) > 0 ? warp_sums[0][(tid >> 5) - 1] : 0;
    const int before1 = (tid >> 5) > 0 ? warp_sums[1][(tid >> 5) - 1] : 0;
    if (tid == 0) base[0] = 0;
    if (tid < r.experts) base[tid + 1] = before0 + v[0];
    ClusterSync();  // every CTA has read the totals: CTA 0 may overwrite them
    if (cta == 0) {
      if (tid == 0) {
        r.offsets[0] = 0;
        r.scale_rows[0] = 0;
      }
      if (tid < r.experts) {
        r.offsets[tid + 1] = before0 + v[0];
        r.scale_rows[tid + 1] = before1 + v[1];
      }
    }
  }
  __syncthreads();
  // ---- 4: each slot's sorted row; each row's token and expert
  for (std::int64_t slot = gthread; slot < slots; slot += gthreads) {
    const int ordinal = r.position[slot];
    if (ordinal < 0) continue;
    const int t = static_cast<int>(slot / r.used);
    const int e = ids[(static_cast<std::int64_t>(t) * ids_stride) + (slot % r.used)];
    const int row = base[e] + r.counts[(static_cast<std::int64_t>(t / kRouteChunk) * r.experts) + e] +
                    ordinal;
    r.position[slot] = row;
    r.token[row] = t;
    r.expert[row] = e;
  }
}

// The grouped GEMM's tile list from the experts' offsets: entry 0 the count,
// then (expert, first column) per 128-column tile, experts in order.
__global__ void BuildTiles(const std::int32_t* __restrict__ offsets, int groups, int capacity,
                           std::int32_t* __restrict__ worklist) {
  extern __shared__ int first[];  // groups + 1 tile prefix
  if (threadIdx.x == 0) {
    int running = 0;
    for (int e = 0; e < groups; ++e) {
      first[e] = running;
      running += (offsets[e + 1] - offsets[e] + kMmqTileCols - 1) / kMmqTileCols;
    }
    first[groups] = running;
    worklist[0] = min(running, capacity);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < groups; e += blockDim.x) {
    const int tiles = first[e + 1] - first[e];
    for (int i = 0; i < tiles; ++i) {
      const int at = first[e] + i;
      if (at < capacity) {
        worklist[1 + (2 * at)] = e;
        worklist[2 + (2 * at)] = offsets[e] + (i * kMmqTileCols);
      }
    }
  }
}

// GLU of the gate and up halves of a row, then the Q8_1-MMQ quantizer of
// mmq.cu on the result (llmp.moe.glu_quantize, llmp_moe.cu:348-392, with this
// build's activation format).  x: F32 [rows][2 f], gate first.
__global__ void __launch_bounds__(256)
GluQuantizeKernel(const float* __restrict__ x, std::int64_t row_stride, int f, std::int64_t rows,
                  int glu, float limit, std::uint8_t* __restrict__ out, std::int64_t lanes_total) {
  GridLaunchDependents();
  // (the index arithmetic runs beside the tail of the kernel before, not after it)
  const std::int64_t i = (static_cast<std::int64_t>(blockIdx.x) * 256) + threadIdx.x;
  const bool live = i < lanes_total;
  const std::int64_t group = (live ? i : 0) / 8;
  const int part = static_cast<int>(i % 8);
  const int groups = f / 32;
  const std::int64_t row = group / groups;
  const int g = static_cast<int>(group - (row * groups));
  GridDependencyWait();
  float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  if (live) {
    const float* p = x + (row * row_stride) + (g * 32) + (part * 4);
    const float4 gate = *reinterpret_cast<const float4*>(p);
    const float4 up = *reinterpret_cast<const float4*>(p + f);
    v[0] = Glu(glu, gate.x, up.x, limit);
    v[1] = Glu(glu, gate.y, up.y, limit);
    v[2] = Glu(glu, gate.z, up.z, limit);
    v[3] = Glu(glu, gate.w, up.w, limit);
  }
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
  float sum = ((v[0] + v[1]) + v[2]) + v[3];
#pragma unroll
  for (int offset = 4; offset > 0; offset >>= 1) {
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, offset));
    sum = sum + __shfl_xor_sync(0xffffffffu, sum, offset);
  }
  if (!live) return;
  std::uint32_t packed = 0;
  float d = 0.0f;
  if (amax > 0.0f) {
    const float d_inv = 127.0f / amax;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int q = static_cast<int>(roundf(v[c] * d_inv));
      packed |= (static_cast<std::uint32_t>(q) & 0xffu) << (8 * c);
    }
    d = 1.0f / d_inv;
  }
  std::uint8_t* block = out + ((static_cast<std::int64_t>(g / 4) * rows + row) * 144);
  *reinterpret_cast<std::uint32_t*>(block + 16 + ((g % 4) * 32) + (part * 4)) = packed;
  if (part == 0) {
    const std::uint32_t ds = static_cast<std::uint32_t>(__half_as_ushort(__float2half_rn(d))) |
                             (static_cast<std::uint32_t>(__half_as_ushort(__float2half_rn(sum)))
                              << 16);
    *reinterpret_cast<std::uint32_t*>(block + ((g % 4) * 4)) = ds;
  }
}

// dst[t][c] = sum over the token's slots, in slot order, of rows[position][c] *
// weight; a slot outside the experts contributes NaN (llmp_moe.cu:393-435
// without the NVFP4 global scales and the shared expert).
__global__ void CombineKernel(const float* __restrict__ rows, std::int64_t row_stride,
                              const std::int32_t* __restrict__ position,
                              const float* __restrict__ weights, int used, int width4,
                              std::int64_t total4, float4* __restrict__ dst) {
  const std::int64_t i = (static_cast<std::int64_t>(blockIdx.x) * blockDim.x) + threadIdx.x;
  if (i >= total4) return;
  const std::int64_t t = i / width4;
  const std::int64_t c4 = i % width4;
  const float nan = __uint_as_float(0x7fc00000u);
  float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  for (int j = 0; j < used; ++j) {
    const int p = position != nullptr ? position[(t * used) + j] : static_cast<int>((t * used) + j);
    const float w = weights[(t * used) + j];
    float4 v = make_float4(nan, nan, nan, nan);
    if (p >= 0) v = *reinterpret_cast<const float4*>(rows + (static_cast<std::int64_t>(p) * row_stride) + (c4 * 4));
    const float4 e = make_float4(__fmul_rn(v.x, w), __fmul_rn(v.y, w), __fmul_rn(v.z, w),
                                 __fmul_rn(v.w, w));
    acc = j == 0 ? e : make_float4(acc.x + e.x, acc.y + e.y, acc.z + e.z, acc.w + e.w);
  }
  dst[i] = acc;
}

// Expert-parallel dispatch with lanes of fixed capacity: a warp a (token, slot).
// `route` is this library's route blob over the slots' OWNER RANKS (the counting sort
// with the ranks as its experts), so position[slot] - offsets[rank] is the slot's
// ordinal among the rows this rank sends to that owner, in (token, slot) order.
__global__ void __launch_bounds__(256)
EpPackKernel(const float* __restrict__ x, std::int64_t x_stride, int hidden,
             const std::int32_t* __restrict__ ids, int ids_stride, int used, int tokens,
             int per_rank, int world, int capacity, const std::int32_t* __restrict__ offsets,
             const std::int32_t* __restrict__ position, float* __restrict__ send_rows,
             std::int32_t* __restrict__ send_ids, std::int32_t* __restrict__ home,
             std::int32_t* __restrict__ dropped) {
  GridLaunchDependents();
  GridDependencyWait();
  const int lane = static_cast<int>(threadIdx.x) & 31;
  const std::int64_t slot = (static_cast<std::int64_t>(blockIdx.x) * 8) + (threadIdx.x >> 5);
  if (slot >= static_cast<std::int64_t>(tokens) * used) return;
  const int t = static_cast<int>(slot / used);
  const int e = ids[(static_cast<std::int64_t>(t) * ids_stride) + (slot % used)];
  const int row = position[slot];
  if (row < 0 || e < 0 || e >= per_rank * world) {  // an id outside the experts
    if (lane == 0) home[slot] = -1;
    return;
  }
  const int rank = e / per_rank;
  const int i = row - offsets[rank];
  if (i >= capacity) {  // more rows for one owner than a lane block holds
    if (lane == 0) {
      home[slot] = -1;
      atomicAdd(dropped, 1);
    }
    return;
  }
  const std::int64_t at = (static_cast<std::int64_t>(rank) * capacity) + i;
  const float4* src = reinterpret_cast<const float4*>(x + (static_cast<std::int64_t>(t) * x_stride));
  float4* dst = reinterpret_cast<float4*>(send_rows + (at * hidden));
  for (int c = lane; c < hidden / 4; c += 32) dst[c] = src[c];
  if (lane == 0) {
    send_ids[at] = e - (rank * per_rank);
    home[slot] = static_cast<std::int32_t>(at);
  }
}

// Lanes nothing was packed into carry the id -1.
__global__ void FillKernel(std::int32_t* __restrict__ p, std::int64_t n, std::int32_t v) {
  const std::int64_t i = (static_cast<std::int64_t>(blockIdx.x) * blockDim.x) + threadIdx.x;
  if (i < n) p[i] = v;
}

int CheckGrouped(const llmp_b200_grouped_gemm_desc& g, bool no_f32_output = false) {
  if (g.groups < 1 || g.groups > kMaxExperts || g.n < 1 || g.k < 256 || g.k % 256 != 0 ||
      g.rows < 1) {
    return Reject("grouped_gemm: 1..1024 groups, n >= 1, k a positive multiple of 256, rows >= 1");
  }
  if (g.offsets == nullptr || g.a == nullptr || (g.weights == nullptr && g.weights_slab == nullptr) ||
      (g.d == nullptr && !no_f32_output)) {
    return Reject("grouped_gemm: offsets, activation blocks, weights (blocks or slab) and an output");
  }
  if (g.expert_stride % 144 != 0 || g.expert_stride < static_cast<std::uint64_t>(g.n) * (g.k / 256) * 144) {
    return Reject("grouped_gemm: expert stride a whole number of Q4_K blocks covering n rows");
  }
  return 0;
}

llmp_b200_mmq_desc MmqOf(const llmp_b200_grouped_gemm_desc& g) {
  llmp_b200_mmq_desc d{};
  d.type = LLMP_B200_TYPE_Q4_K;
  d.w = g.weights;
  d.y = g.a;
  d.ids_dst = nullptr;
  d.expert_bounds = g.offsets;
  d.dst = static_cast<float*>(g.d);
  d.k = g.k;
  d.nrows = g.n;
  d.ncols = g.rows;
  d.stride_row = g.k / 256;
  d.stride_expert = static_cast<int>(g.expert_stride / 144);
  d.dst_col_stride = g.n;
  d.experts = g.groups;
  d.max_cols_per_expert = g.rows;
  d.w_slab = g.weights_slab;
  d.scratch = nullptr;
  return d;
}

int TileCapacity(int groups, int rows) { return ((rows + kMmqTileCols - 1) / kMmqTileCols) + groups; }

// ---- the tile list of llmp_b200_grouped_gemm_static --------------------------
// Sized for the largest problem that entry point takes: 256 groups over 65,536
// sorted rows is at most 512 + 256 tiles.  Every GPU that loads the library
// holds these 6,400 bytes until the process exits.
constexpr int kStaticMaxGroups = 256;
constexpr int kStaticMaxRows = 65536;
constexpr int kStaticMaxTiles = (kStaticMaxRows / kMmqTileCols) + kStaticMaxGroups;
static __device__ __align__(256) std::int32_t g_static_tiles[1 + (2 * kStaticMaxTiles) + 63];

// The array's DEVICE address on the current device.  `g_static_tiles` named in
// host code is only the host-side handle of the symbol, never an address a
// kernel may dereference; the runtime translates it, once per device, with
// that device current.
std::int32_t* StaticTiles() {
  constexpr int kMaxDevices = 64;
  static std::int32_t* table[kMaxDevices] = {};
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) {
    cudaGetLastError();
    return nullptr;
  }
  if (table[device] == nullptr) {
    void* address = nullptr;
    if (cudaGetSymbolAddress(&address, g_static_tiles) != cudaSuccess || address == nullptr) {
      cudaGetLastError();
      return nullptr;
    }
    table[device] = static_cast<std::int32_t*>(address);  // the same value whoever stores it
  }
  return table[device];
}

}  // namespace
}  // namespace llmp_b200

extern "C" {

int64_t llmp_b200_moe_route_ints(int experts, int used, int tokens) {
  const int64_t slots = static_cast<int64_t>(used) * tokens;
  const int64_t chunks = (tokens + llmp_b200::kRouteChunk - 1) / llmp_b200::kRouteChunk;
  return (2 * (static_cast<int64_t>(experts) + 1)) + (3 * slots) + (chunks * experts);
}

int llmp_b200_moe_route(const int32_t* ids, int ids_stride, int experts, int used, int tokens,
                        int32_t* out, void* stream) {
  using namespace llmp_b200;
  if (ids == nullptr || out == nullptr || experts < 1 || experts > kMaxExperts || used < 1 ||
      tokens < 1 || ids_stride < used || used * kRouteChunk > 8192) {
    return Reject("moe.route: ids I32 [used, tokens], 1..1024 experts, used <= 128");
  }
  if (const int status = DeviceStatus(); status != 0) return status;
  auto* s = static_cast<cudaStream_t>(stream);
  const Route r = RouteOf(out, experts, used, tokens);
  // A cluster of 1 to 8 CTAs: 32 warps each, a warp a chunk at a time.
  int ctas = (r.chunks + 31) / 32;
  ctas = ctas < 1 ? 1 : ctas > 8 ? 8 : ctas;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(static_cast<unsigned>(ctas));
  config.blockDim = dim3(kRouteThreads);
  config.stream = s;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeClusterDimension;
  attribute[0].val.clusterDim.x = static_cast<unsigned>(ctas);
  attribute[0].val.clusterDim.y = 1;
  attribute[0].val.clusterDim.z = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&config, RouteKernel, ids, ids_stride, r);
  if (e != cudaSuccess) return Failed(e, "moe.route launch");
  return Launched("moe.route launch");
}

int llmp_b200_grouped_gemm_available(void) { return llmp_b200_available(); }

size_t llmp_b200_grouped_gemm_scratch(int groups, int rows, int sms) {
  (void)sms;
  if (groups < 1 || rows < 1) return 0;
  const size_t ints = 1 + (2 * static_cast<size_t>(llmp_b200::TileCapacity(groups, rows)));
  return (ints * sizeof(int32_t) + 255) / 256 * 256;
}

namespace llmp_b200 {
namespace {
int GroupedGemm(const llmp_b200_grouped_gemm_desc* gemm, const MmqGlu* glu, void* stream);
}  // namespace
}  // namespace llmp_b200

int llmp_b200_grouped_gemm(const llmp_b200_grouped_gemm_desc* gemm, int sms, void* stream) {
  (void)sms;
  return llmp_b200::GroupedGemm(gemm, nullptr, stream);
}

int llmp_b200_grouped_gemm_glu(const llmp_b200_grouped_gemm_desc* gemm, int glu, float limit,
                               void* blocks, int sms, void* stream) {
  (void)sms;
  const llmp_b200::MmqGlu g{blocks, glu, limit};
  return llmp_b200::GroupedGemm(gemm, &g, stream);
}

}  // extern "C"

namespace llmp_b200 {
namespace {
int GroupedGemm(const llmp_b200_grouped_gemm_desc* gemm, const MmqGlu* glu, void* stream) {
  if (gemm == nullptr) return Reject("grouped_gemm: null descriptor");
  const llmp_b200_grouped_gemm_desc& g = *gemm;
  if (const int status = CheckGrouped(g, glu != nullptr); status != 0) return status;
  if (g.scratch == nullptr || !Aligned(g.scratch, 256)) {
    return Reject("grouped_gemm: 256-byte aligned scratch of llmp_b200_grouped_gemm_scratch bytes");
  }
  if (const int status = DeviceStatus(); status != 0) return status;
  const int capacity = TileCapacity(g.groups, g.rows);
  auto* worklist = static_cast<std::int32_t*>(g.scratch);
  BuildTiles<<<1, 256, (g.groups + 1) * sizeof(int), static_cast<cudaStream_t>(stream)>>>(
      g.offsets, g.groups, capacity, worklist);
  if (const int status = Launched("grouped_gemm tile list"); status != 0) return status;
  const int status = LaunchMmq(MmqOf(g), worklist, capacity, stream, nullptr, glu);
  // The tile list is queued: a refusal now would leave work behind, so report
  // it as a failure after queueing.
  return status > 0 ? -status : status;
}
}  // namespace
}  // namespace llmp_b200

extern "C" {

int llmp_b200_grouped_gemm_static(const llmp_b200_grouped_gemm_desc* gemm, int sms, void* stream) {
  using namespace llmp_b200;
  (void)sms;
  if (gemm == nullptr) return Reject("grouped_gemm_static: null descriptor");
  const llmp_b200_grouped_gemm_desc& g = *gemm;
  if (const int status = CheckGrouped(g); status != 0) return status;
  if (g.groups > kStaticMaxGroups || g.rows > kStaticMaxRows) {
    return Reject("grouped_gemm_static: %d groups over %d rows is beyond the built-in tile list "
                  "(at most %d groups, %d rows); use llmp_b200_grouped_gemm with caller scratch",
                  g.groups, g.rows, kStaticMaxGroups, kStaticMaxRows);
  }
  if (const int status = DeviceStatus(); status != 0) return status;
  std::int32_t* worklist = StaticTiles();  // first call on a device resolves the address
  if (worklist == nullptr) {
    return Reject("grouped_gemm_static: the runtime gave no device address for the tile list");
  }
  const int capacity = TileCapacity(g.groups, g.rows);
  // BuildTiles rewrites the count and every entry it will hand out, so nothing
  // of an earlier call's list needs clearing.
  BuildTiles<<<1, 256, (g.groups + 1) * sizeof(int), static_cast<cudaStream_t>(stream)>>>(
      g.offsets, g.groups, capacity, worklist);
  if (const int status = Launched("grouped_gemm_static tile list"); status != 0) return status;
  const int status = LaunchMmq(MmqOf(g), worklist, capacity, stream);
  return status > 0 ? -status : status;
}

int llmp_b200_moe_glu_quantize(const float* gate_up, int64_t row_stride, int f, int64_t rows,
                               int glu, float limit, void* out, void* stream) {
  using namespace llmp_b200;
  if (gate_up == nullptr || out == nullptr || f < 128 || f % 128 != 0 || rows < 1 ||
      row_stride < 2 * static_cast<int64_t>(f) || glu < 1 || glu > 3) {
    return Reject("moe.glu_quantize: F32 [2 f, rows] with f a positive multiple of 128, a GLU");
  }
  if (!Aligned(gate_up, 16) || row_stride % 4 != 0 || !Aligned(out, 16)) {
    return Reject("moe.glu_quantize: rows and output 16-byte aligned");
  }
  if (const int status = DeviceStatus(); status != 0) return status;
  const std::int64_t lanes = rows * (f / 32) * 8;
  const std::int64_t grid = (lanes + 255) / 256;
  if (grid > 0x7fffffffLL) return Reject("moe.glu_quantize: more blocks than a grid holds");
  const cudaError_t e = LaunchPdl(GluQuantizeKernel, dim3(static_cast<unsigned>(grid)), dim3(256), 0,
                                  static_cast<cudaStream_t>(stream), gate_up, row_stride, f, rows,
                                  glu, limit, static_cast<std::uint8_t*>(out), lanes);
  if (e != cudaSuccess) return Failed(e, "moe.glu_quantize launch");
  return 0;
}

int llmp_b200_moe_ep_pack(const float* x, int64_t x_stride, int hidden, const int32_t* ids,
                          int ids_stride, int used, int tokens, int experts, int world, int capacity,
                          const int32_t* route, float* send_rows, int32_t* send_ids, int32_t* home,
                          int32_t* dropped, void* stream) {
  using namespace llmp_b200;
  if (x == nullptr || ids == nullptr || route == nullptr || send_rows == nullptr ||
      send_ids == nullptr || home == nullptr || dropped == nullptr) {
    return Reject("moe.ep_pack: rows, ids, the owners' route and the four outputs");
  }
  if (hidden < 4 || hidden % 4 != 0 || x_stride < hidden || x_stride % 4 != 0 || used < 1 ||
      tokens < 1 || ids_stride < used || world < 1 || world > kMaxExperts || experts < world ||
      experts % world != 0 || capacity < 1) {
    return Reject("moe.ep_pack: hidden a positive multiple of 4, experts a multiple of the ranks, "
                  "a positive capacity");
  }
  if (!Aligned(x, 16) || !Aligned(send_rows, 16)) return Reject("moe.ep_pack: 16-byte aligned rows");
  if (const int status = DeviceStatus(); status != 0) return status;
  auto* s = static_cast<cudaStream_t>(stream);
  const std::int64_t lanes = static_cast<std::int64_t>(world) * capacity;
  FillKernel<<<static_cast<unsigned>((lanes + 255) / 256), 256, 0, s>>>(send_ids, lanes, -1);
  if (const int status = Launched("moe.ep_pack fill"); status != 0) return status;
  const Route r = RouteOf(const_cast<std::int32_t*>(route), world, used, tokens);
  const std::int64_t slots = static_cast<std::int64_t>(tokens) * used;
  const cudaError_t e = LaunchPdl(EpPackKernel, dim3(static_cast<unsigned>((slots + 7) / 8)), dim3(256),
                                  0, s, x, x_stride, hidden, ids, ids_stride, used, tokens,
                                  experts / world, world, capacity,
                                  static_cast<const std::int32_t*>(r.offsets),
                                  static_cast<const std::int32_t*>(r.position), send_rows, send_ids,
                                  home, dropped);
  if (e != cudaSuccess) return Failed(e, "moe.ep_pack launch");
  return 0;
}

int llmp_b200_moe_combine(const float* rows, int64_t row_stride, const int32_t* position,
                          const float* weights, int used, int tokens, int width, float* dst,
                          void* stream) {
  using namespace llmp_b200;
  if (rows == nullptr || weights == nullptr || dst == nullptr || used < 1 ||
      tokens < 1 || width < 4 || width % 4 != 0 || row_stride < width || row_stride % 4 != 0) {
    return Reject("moe.combine: sorted rows F32 [width, slots], width a positive multiple of 4");
  }
  if (!Aligned(rows, 16) || !Aligned(dst, 16)) return Reject("moe.combine: 16-byte aligned rows");
  if (const int status = DeviceStatus(); status != 0) return status;
  const std::int64_t total4 = static_cast<std::int64_t>(tokens) * (width / 4);
  CombineKernel<<<static_cast<unsigned>((total4 + 255) / 256), 256, 0,
                  static_cast<cudaStream_t>(stream)>>>(rows, row_stride, position, weights, used,
                                                       width / 4, total4,
                                                       reinterpret_cast<float4*>(dst));
  return Launched("moe.combine launch");
}

}  // extern "C"
