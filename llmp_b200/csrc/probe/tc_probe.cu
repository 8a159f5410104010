// Microbenchmarks of the Blackwell tensor-core path on the device at hand: the
// figures the GEMM kernels' rooflines and design notes rest on.  Built by
// `make -C llmp_b200/csrc probe` into llmp_b200/_lib/tc_probe; run without
// arguments.  Every wait is bounded (tc::MbarWait) and reported as "timeouts".
//
//   peaks   back-to-back tcgen05.mma issue rate, kind::i8 and
//           kind::mxf8f6f4.block_scale, 128 x N x 32, one CTA per SM;
//   commit  cycles from one small MMA + tcgen05.commit to the mbarrier flip,
//           the cost of further MMAs before the commit, and the rate of a ring
//           of three accumulators each reissued after its own commit lands;
//   tmemld  tcgen05.ld (32x32b) bytes per clock per SM by width and warps;
//   sync    cycles of the small synchronisation pieces in a warp's loop.
#include <cstdio>
#include <cstring>

#include "../tc.cuh"

using namespace llmp_b200;

namespace {

unsigned int* g_bad = nullptr;

// ------------------------------------------------------------------ peaks
template <int kKind, int kN>
__global__ void __launch_bounds__(128, 1) PeakKernel(int iters, unsigned int* bad) {
  extern __shared__ unsigned char raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<std::uintptr_t>(raw) + 1023) & ~static_cast<std::uintptr_t>(1023));
  __shared__ std::uint64_t bar;
  __shared__ std::uint32_t tbase;
  for (int i = threadIdx.x; i < (128 + 256) * 128 / 4; i += 128) {
    reinterpret_cast<std::uint32_t*>(smem)[i] = 0x01010101u;
  }
  if (threadIdx.x == 0) {
    tc::MbarInit(&bar, 1);
    tc::MbarInitFence();
  }
  if (threadIdx.x < 32) {
    tc::TmemAlloc(&tbase, 512);
    tc::TmemRelinquish();
  }
  tc::FenceProxyAsync();
  tc::TcFenceBefore();
  __syncthreads();
  tc::TcFenceAfter();
  const std::uint32_t tmem = tbase;
  if (threadIdx.x == 0) {
    const std::uint64_t a = tc::SmemDesc(smem, true, 1024);
    const std::uint64_t b = tc::SmemDesc(smem + (128 * 128), true, 1024);
    for (int it = 0; it < iters; ++it) {
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        if (kKind == 0) {
          tc::MmaI8(tmem, a + (kk * 2), b + (kk * 2), tc::IdescI8(128, kN, false, true), true);
        } else {
          tc::MmaMxf8(tmem, a + (kk * 2), b + (kk * 2), tc::IdescMxf8(128, kN, kk, kk), true,
                      tmem + 300, tmem + 320);
        }
      }
    }
    tc::TcCommit(&bar);
    if (!tc::MbarWait(&bar, 0)) atomicAdd(bad, 1u);
  }
  tc::TcFenceBefore();
  __syncthreads();
  if (threadIdx.x < 32) {
    tc::TcFenceAfter();
    tc::TmemDealloc(tmem, 512);
  }
}

template <int kKind, int kN>
void RunPeak(const char* name, int sms) {
  const int smem = ((128 + 256) * 128) + 2048;
  cudaFuncSetAttribute(PeakKernel<kKind, kN>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  const int iters = 20000;
  float best = 1e9f;
  for (int r = 0; r < 4; ++r) {
    cudaEventRecord(e0);
    PeakKernel<kKind, kN><<<sms, 128, smem>>>(iters, g_bad);
    cudaEventRecord(e1);
    cudaEventSynchronize(e1);
    float ms;
    cudaEventElapsedTime(&ms, e0, e1);
    if (ms < best) best = ms;
  }
  const double ops = static_cast<double>(sms) * iters * 4 * 2.0 * 128 * kN * 32;
  std::printf("peaks  %-22s N=%3d: %.3f ms -> %.1f T(FL)OP/s\n", name, kN, best, ops / best / 1e9);
}

// ------------------------------------------------------------------ commit
__global__ void __launch_bounds__(128, 1)
CommitKernel(int iters, int nmma, unsigned long long* out, unsigned int* bad) {
  extern __shared__ unsigned char raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<std::uintptr_t>(raw) + 1023) & ~static_cast<std::uintptr_t>(1023));
  __shared__ std::uint64_t bar[4];
  __shared__ std::uint32_t tbase;
  for (int i = threadIdx.x; i < (128 + 128) * 128 / 4; i += 128) {
    reinterpret_cast<std::uint32_t*>(smem)[i] = 0x01010101u;
  }
  if (threadIdx.x == 0) {
    for (int i = 0; i < 4; ++i) tc::MbarInit(&bar[i], 1);
    tc::MbarInitFence();
  }
  if (threadIdx.x < 32) {
    tc::TmemAlloc(&tbase, 512);
    tc::TmemRelinquish();
  }
  tc::FenceProxyAsync();
  tc::TcFenceBefore();
  __syncthreads();
  tc::TcFenceAfter();
  const std::uint32_t tmem = tbase;
  if (threadIdx.x == 0) {
    const std::uint64_t a = tc::SmemDesc(smem, true, 1024);
    const std::uint64_t b = tc::SmemDesc(smem + (128 * 128), true, 1024);
    const std::uint32_t idesc = tc::IdescI8(128, 128, false, true);
    long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {  // MMA(s), commit, wait
      for (int m = 0; m < nmma; ++m) tc::MmaI8(tmem, a + ((m & 3) * 2), b + ((m & 3) * 2), idesc, false);
      tc::TcCommit(&bar[0]);
      if (!tc::MbarWait(&bar[0], it & 1)) {
        atomicAdd(bad, 1u);
        break;
      }
    }
    long long t1 = clock64();
    out[0] = static_cast<unsigned long long>(t1 - t0);
    t0 = clock64();
    for (int it = 0; it < iters; ++it) {  // three accumulators, each reissued after its commit
      const int bb = 1 + (it % 3);
      if (it >= 3 && !tc::MbarWait(&bar[bb], ((it / 3) - 1) & 1)) {
        atomicAdd(bad, 1u);
        break;
      }
      tc::MmaI8(tmem + ((bb - 1) * 128), a, b, idesc, false);
      tc::TcCommit(&bar[bb]);
    }
    t1 = clock64();
    out[1] = static_cast<unsigned long long>(t1 - t0);
  }
  tc::TcFenceBefore();
  __syncthreads();
  if (threadIdx.x < 32) {
    tc::TcFenceAfter();
    tc::TmemDealloc(tmem, 512);
  }
}

void RunCommit(int sms) {
  unsigned long long* out;
  cudaMalloc(&out, 16);
  const int smem = ((128 + 128) * 128) + 2048;
  cudaFuncSetAttribute(CommitKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  const int iters = 999;
  for (int nmma : {1, 4, 16}) {
    CommitKernel<<<sms, 128, smem>>>(iters, nmma, out, g_bad);
    CommitKernel<<<sms, 128, smem>>>(iters, nmma, out, g_bad);
    cudaDeviceSynchronize();
    unsigned long long h[2];
    cudaMemcpy(h, out, 16, cudaMemcpyDeviceToHost);
    std::printf("commit %2d x i8 128x128x32 + commit + wait: %7.1f cycles;  ring of 3 (1 MMA + commit "
                "each): %6.1f cycles an MMA\n", nmma, double(h[0]) / iters, double(h[1]) / iters);
  }
  cudaFree(out);
}

// ------------------------------------------------------------------ tmemld
template <int kX>
__device__ __forceinline__ void Load(std::uint32_t taddr, std::uint32_t* r);
template <>
__device__ __forceinline__ void Load<16>(std::uint32_t taddr, std::uint32_t* r) {
  tc::TmemLoad16(taddr, *reinterpret_cast<std::uint32_t(*)[16]>(r));
}
template <>
__device__ __forceinline__ void Load<32>(std::uint32_t taddr, std::uint32_t* r) {
  tc::TmemLoad32(taddr, *reinterpret_cast<std::uint32_t(*)[32]>(r));
}

template <int kX, int kInFlight>
__global__ void __launch_bounds__(512, 1)
TmemLoadKernel(int iters, unsigned long long* cycles, std::uint32_t* sink) {
  __shared__ std::uint32_t tbase;
  const int warp = threadIdx.x >> 5;
  if (warp == 0) {
    tc::TmemAlloc(&tbase, 512);
    tc::TmemRelinquish();
  }
  tc::TcFenceBefore();
  __syncthreads();
  tc::TcFenceAfter();
  const std::uint32_t tmem = tbase;
  const std::uint32_t lane_base = static_cast<std::uint32_t>((warp & 3) * 32) << 16;
  std::uint32_t r[kInFlight][kX];
  std::uint32_t x = 0;
  const long long t0 = clock64();
  for (int it = 0; it < iters; ++it) {
#pragma unroll
    for (int f = 0; f < kInFlight; ++f) {
      Load<kX>(tmem + lane_base + (((f * kX) + (it * 16)) & 255), r[f]);
    }
    tc::TmemLoadWait();
#pragma unroll
    for (int f = 0; f < kInFlight; ++f) {
#pragma unroll
      for (int j = 0; j < kX; ++j) x ^= r[f][j];
    }
  }
  const long long t1 = clock64();
  if (threadIdx.x == 0 && blockIdx.x == 0) *cycles = static_cast<unsigned long long>(t1 - t0);
  if (x == 0x12345678u) sink[0] = x;
  tc::TcFenceBefore();
  __syncthreads();
  if (warp == 0) {
    tc::TcFenceAfter();
    tc::TmemDealloc(tmem, 512);
  }
}

template <int kX, int kF>
void RunTmemLoad(int sms, int threads) {
  unsigned long long* cyc;
  std::uint32_t* sink;
  cudaMalloc(&cyc, 8);
  cudaMalloc(&sink, 4);
  const int iters = 2000;
  TmemLoadKernel<kX, kF><<<sms, threads>>>(iters, cyc, sink);
  TmemLoadKernel<kX, kF><<<sms, threads>>>(iters, cyc, sink);
  cudaDeviceSynchronize();
  unsigned long long c = 0;
  cudaMemcpy(&c, cyc, 8, cudaMemcpyDeviceToHost);
  const double bytes = double(iters) * kF * kX * 4.0 * threads;
  std::printf("tmemld 32x32b.x%-2d, %d in flight, %2d warps: %6.1f cycles a round, %6.1f B/clk/SM\n", kX,
              kF, threads / 32, double(c) / iters, bytes / double(c));
  cudaFree(cyc);
  cudaFree(sink);
}

// ------------------------------------------------------------------ sync
__global__ void __launch_bounds__(128, 1) SyncKernel(int iters, unsigned long long* out) {
  __shared__ std::uint64_t bar;
  __shared__ std::uint32_t tbase;
  __shared__ volatile std::uint32_t flag;
  if (threadIdx.x == 0) {
    tc::MbarInit(&bar, (1u << 20) - 1u);  // the largest count: the arrivals below never flip it
    tc::MbarInitFence();
    flag = 0;
  }
  if (threadIdx.x < 32) {
    tc::TmemAlloc(&tbase, 512);
    tc::TmemRelinquish();
  }
  tc::TcFenceBefore();
  __syncthreads();
  tc::TcFenceAfter();
  const std::uint32_t tmem = tbase;
  if (threadIdx.x < 32) {
    long long t0, t1;
    unsigned acc = 0;
    auto poll = [&](std::uint32_t parity) {
      std::uint32_t d;
      asm volatile(
          "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
          "selp.u32 %0, 1, 0, p;\n}\n"
          : "=r"(d)
          : "r"(tc::Smem(&bar)), "r"(parity)
          : "memory");
      return d;
    };
    t0 = clock64(); for (int i = 0; i < iters; ++i) tc::TcFenceAfter(); t1 = clock64();
    if (threadIdx.x == 0) out[0] = t1 - t0;
    t0 = clock64(); for (int i = 0; i < iters; ++i) tc::TcFenceBefore(); t1 = clock64();
    if (threadIdx.x == 0) out[1] = t1 - t0;
    t0 = clock64();
    for (int i = 0; i < iters; ++i) {
      __syncwarp();
      if (threadIdx.x == 0) tc::MbarArrive(&bar);
    }
    t1 = clock64();
    if (threadIdx.x == 0) out[2] = t1 - t0;
    t0 = clock64(); for (int i = 0; i < iters; ++i) acc += flag; t1 = clock64();
    if (threadIdx.x == 0) out[3] = t1 - t0;
    t0 = clock64(); for (int i = 0; i < iters; ++i) tc::FenceProxyAsync(); t1 = clock64();
    if (threadIdx.x == 0) out[4] = t1 - t0;
    t0 = clock64(); for (int i = 0; i < iters; ++i) acc += poll(1u); t1 = clock64();
    if (threadIdx.x == 0) out[5] = t1 - t0;
    t0 = clock64(); for (int i = 0; i < 64; ++i) acc += poll(0u); t1 = clock64();
    if (threadIdx.x == 0) out[6] = (t1 - t0) * (iters / 64);
    t0 = clock64(); for (int i = 0; i < iters; ++i) acc += __shfl_sync(0xffffffffu, acc, 0); t1 = clock64();
    if (threadIdx.x == 0) out[7] = t1 - t0;
    if (acc == 0x12345u) out[15] = acc;
  }
  tc::TcFenceBefore();
  __syncthreads();
  if (threadIdx.x < 32) {
    tc::TcFenceAfter();
    tc::TmemDealloc(tmem, 512);
  }
}

void RunSync() {
  unsigned long long* out;
  cudaMalloc(&out, 128);
  cudaMemset(out, 0, 128);
  const int iters = 1024;
  SyncKernel<<<1, 128>>>(iters, out);
  cudaDeviceSynchronize();
  unsigned long long h[16];
  cudaMemcpy(h, out, 128, cudaMemcpyDeviceToHost);
  const char* names[] = {"tcgen05.fence::after_thread_sync", "tcgen05.fence::before_thread_sync",
                         "syncwarp + lane-0 mbarrier.arrive", "volatile shared read",
                         "fence.proxy.async", "mbarrier.try_wait, phase complete",
                         "mbarrier.try_wait, phase pending", "shfl.sync"};
  for (int i = 0; i < 8; ++i) std::printf("sync   %-36s %8.1f cycles\n", names[i], double(h[i]) / iters);
  cudaFree(out);
}

}  // namespace

int main() {
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, 0) != cudaSuccess || prop.major != 10) {
    std::printf("tc_probe: needs a compute-capability 10.x device\n");
    return 2;
  }
  const int sms = prop.multiProcessorCount;
  cudaMalloc(&g_bad, 4);
  cudaMemset(g_bad, 0, 4);
  std::printf("%s, %d SMs, %d MHz\n", prop.name, sms, prop.clockRate / 1000);
  RunPeak<1, 256>("mxf8f6f4.block_scale", sms);
  RunPeak<1, 128>("mxf8f6f4.block_scale", sms);
  RunPeak<0, 256>("i8", sms);
  RunPeak<0, 128>("i8", sms);
  RunCommit(sms);
  RunTmemLoad<16, 1>(sms, 256);
  RunTmemLoad<16, 4>(sms, 256);
  RunTmemLoad<32, 2>(sms, 256);
  RunTmemLoad<32, 1>(sms, 512);
  RunTmemLoad<32, 2>(sms, 512);
  RunSync();
  unsigned int bad = 0;
  cudaMemcpy(&bad, g_bad, 4, cudaMemcpyDeviceToHost);
  std::printf("timeouts %u, %s\n", bad, cudaGetErrorString(cudaGetLastError()));
  return bad == 0 ? 0 : 1;
}
