// Stand-alone microbenchmarks of the tcgen05 behaviour the attention kernel's schedule is built around (not part of
// libhdit_b200.so). Build and run on a B200:
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o tcgen05_issue hetu_dit_b200/csrc/microbench/tcgen05_issue.cu
//   ./tcgen05_issue
// Part 1: cycles per tcgen05.mma for shapes / operand sources / accumulator patterns (issue time of the issuing
//         thread and completion time). Part 2: the attention kernel's MMA sequence gated by the S-full / P-ready
//         mbarrier hand-shake with softmax warpgroups that do nothing else. Part 3: latency of each hop of that
//         hand-shake (commit -> waiter, arrive -> issuer), try_wait against test_wait polling.
// Every wait is bounded.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../ptx_sm100.cuh"
using namespace hdit;

namespace part1 {
// Microbenchmark: cycles per tcgen05.mma for dependent / independent accumulator chains.


__device__ long long g_out[64];

template <int PATTERN>
__device__ void run_pattern(uint32_t tmem, uint32_t a_addr, uint32_t b_addr, uint64_t* bar, int reps, int slot, uint32_t& phase) {
  constexpr uint32_t id128 = make_idesc_f16(128, 128, 1, 0);
  constexpr uint32_t id256 = make_idesc_f16(128, 256, 1, 0);
  constexpr uint32_t id64 = make_idesc_f16(128, 64, 1, 0);
  constexpr uint32_t id128n = make_idesc_f16(128, 128, 1, 1);
  constexpr uint32_t id64n = make_idesc_f16(128, 64, 1, 1);
  const uint64_t a0 = make_smem_desc_sw128(a_addr, 16, 1024);
  const uint64_t b0 = make_smem_desc_sw128(b_addr, 16, 1024);
  const uint64_t v0 = make_smem_desc_sw128(b_addr, 16384, 1024);
  long long t0 = clock64();
  int count = 0;
  for (int r = 0; r < reps; ++r) {
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      const uint32_t off = ((kk & 3) * 32) >> 4;
      if (PATTERN == 1) { umma_ss(tmem, a0 + off, b0 + off, id128, 1); count++; }
      if (PATTERN == 2) { umma_ss(tmem + (kk & 1) * 128, a0 + off, b0 + off, id128, 1); count++; }
      if (PATTERN == 3) { umma_ss(tmem, a0 + off, b0 + off, id256, 1); count++; }
      if (PATTERN == 4) { umma_ss(tmem, a0 + off, b0 + off, id64, 1); count++; }
      if (PATTERN == 5) { umma_ts(tmem, tmem + 256 + kk * 8, v0 + ((kk * 2048) >> 4), id128n, 1); count++; }
      if (PATTERN == 6) { umma_ts(tmem, tmem + 256 + kk * 8, v0 + ((kk * 2048) >> 4), id64n, 1); count++; }
      if (PATTERN == 8) { umma_ts(tmem, tmem + 256 + kk * 8, v0 + ((kk * 2048) >> 4), id128n, 1);
                          umma_ss(tmem + 128, a0 + off, b0 + off, id128, 1); count += 2; }
      if (PATTERN == 9) { umma_ss(tmem + (kk & 3) * 128, a0 + off, b0 + off, id128, 1); count++; }
      if (PATTERN == 10) { umma_ss(tmem + (kk & 1) * 256, a0 + off, b0 + off, id256, 1); count++; }
      if (PATTERN == 11) { umma_ss(tmem + (kk & 3) * 64, a0 + off, b0 + off, id64, 1); count++; }
      if (PATTERN == 12) { umma_ts(tmem + (kk & 1) * 128, tmem + 256 + kk * 8, v0 + ((kk * 2048) >> 4), id128n, 1); count++; }
    }
    if (PATTERN == 7) {
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) { umma_ts(tmem, tmem + 256 + kk * 8, v0 + ((kk * 2048) >> 4), id128n, 1); }
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) { const uint32_t off = ((kk & 3) * 32) >> 4; umma_ss(tmem + 128, a0 + off, b0 + off, id128, 1); }
      count += 16;
    }
  }
  long long t1 = clock64();
  tc_commit(bar);
  while (!mbar_try_wait(bar, phase)) {}
  phase ^= 1;
  long long t2 = clock64();
  g_out[slot * 3 + 0] = t1 - t0;
  g_out[slot * 3 + 1] = t2 - t0;
  g_out[slot * 3 + 2] = count;
}

__global__ void __launch_bounds__(128, 1) bench_kernel(int reps) {
  extern __shared__ char smem_raw[];
  char* smem = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  char* sa = smem;            // 16 KB
  char* sb = smem + 16384;    // 32 KB
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + 16384 + 32768);
  uint32_t* slot = reinterpret_cast<uint32_t*>(bar + 1);
  for (int i = threadIdx.x; i < (16384 + 32768) / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0x3c003c00u;
  if (threadIdx.x == 0) { mbar_init(bar, 1); fence_mbar_init(); fence_proxy_async_smem(); }
  if (threadIdx.x < 32) { tmem_alloc(slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *slot;
  if (threadIdx.x == 0) {
    uint32_t phase = 0;
    const uint32_t a = smem_u32(sa), b = smem_u32(sb);
    run_pattern<1>(tmem, a, b, bar, reps, 0, phase);   // warm
    run_pattern<1>(tmem, a, b, bar, reps, 1, phase);
    run_pattern<2>(tmem, a, b, bar, reps, 2, phase);
    run_pattern<3>(tmem, a, b, bar, reps, 3, phase);
    run_pattern<4>(tmem, a, b, bar, reps, 4, phase);
    run_pattern<5>(tmem, a, b, bar, reps, 5, phase);
    run_pattern<6>(tmem, a, b, bar, reps, 6, phase);
    run_pattern<7>(tmem, a, b, bar, reps, 7, phase);
    run_pattern<8>(tmem, a, b, bar, reps, 8, phase);
    run_pattern<9>(tmem, a, b, bar, reps, 9, phase);
    run_pattern<10>(tmem, a, b, bar, reps, 10, phase);
    run_pattern<11>(tmem, a, b, bar, reps, 11, phase);
    run_pattern<12>(tmem, a, b, bar, reps, 12, phase);
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}


}  // namespace part1
namespace part2 {
// Microbenchmark 4: MMA groups gated by the S-full / P-ready handshake with two "softmax" warpgroups that do
// nothing but the handshake. Measures the round trip commit -> softmax wake -> arrive -> MMA wake.

__device__ long long g_out[256];

// mode 0: kernel-like (all 128 threads poll s_full, lane 0 of each warp arrives, count 4)
// mode 1: only lane 0 of each warp polls, then __syncwarp, lane 0 arrives
// mode 2: like 0 but softmax warps also read S (tcgen05.ld 128 cols + wait) and write P (st 64 cols + wait) before arriving
__global__ void __launch_bounds__(384, 1) bench_kernel(int nblk, int mode, int slot_out) {
  extern __shared__ char smem_raw[];
  char* smem = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  char* sq = smem;
  char* sk = smem + 65536;
  char* sv = smem + 98304;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 131072);
  uint64_t* s_full = bars;       // [2]
  uint64_t* p_ready = bars + 2;  // [2]
  uint64_t* done = bars + 4;
  uint32_t* slot = reinterpret_cast<uint32_t*>(bars + 8);
  for (int i = threadIdx.x; i < 131072 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0x3c003c00u;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) { mbar_init(&s_full[i], 1); mbar_init(&p_ready[i], 4); }
    mbar_init(done, 1);
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == 9) { tmem_alloc(slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *slot;
  const uint32_t kSpin = 50u * 1000u * 1000u;
  if (warp == 9) {
    if (lane == 0) {
      constexpr uint32_t id_qk = make_idesc_f16(128, 128, 1, 0);
      constexpr uint32_t id_pv = make_idesc_f16(128, 128, 1, 1);
      const uint64_t q0 = make_smem_desc_sw128(smem_u32(sq), 16, 1024);
      const uint64_t k0 = make_smem_desc_sw128(smem_u32(sk), 16, 1024);
      const uint64_t v0 = make_smem_desc_sw128(smem_u32(sv), 16384, 1024);
      auto pv = [&](int t) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) umma_ts(tmem + 256 + t * 128, tmem + t * 128 + kk * 8, v0 + ((kk * 2048) >> 4), id_pv, 1);
      };
      auto qk = [&](int t) {
        const uint64_t a0 = q0 + ((t * 32768) >> 4);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = ((kk >> 2) * 16384 + (kk & 3) * 32) >> 4;
          umma_ss(tmem + t * 128, a0 + off, k0 + off, id_qk, kk > 0);
        }
      };
      long long t0 = clock64();
      qk(0); tc_commit(&s_full[0]);
      qk(1); tc_commit(&s_full[1]);
      long long wait_cycles = 0;
      bool ok = true;
      for (int j = 0; j < nblk && ok; ++j) {
        for (int t = 0; t < 2; ++t) {
          long long w0 = clock64();
          uint32_t sp = 0;
          while (!mbar_try_wait(&p_ready[t], j & 1) && sp < kSpin) ++sp;
          if (sp >= kSpin) { ok = false; break; }
          wait_cycles += clock64() - w0;
          tc_fence_after();
          pv(t);
          if (j + 1 < nblk) { qk(t); tc_commit(&s_full[t]); }
        }
      }
      tc_commit(done);
      { uint32_t sp = 0; while (!mbar_try_wait(done, 0) && sp < kSpin) ++sp; }
      long long t2 = clock64();
      g_out[slot_out * 3 + 0] = t2 - t0;
      g_out[slot_out * 3 + 1] = wait_cycles;
      g_out[slot_out * 3 + 2] = ok ? nblk : -1;
    }
  } else if (warp < 8) {
    const int t = warp >> 2;
    const uint32_t tm_s = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16) + t * 128;
    for (int j = 0; j < nblk; ++j) {
      bool got = true;
      if (mode == 1) {
        if (lane == 0) { uint32_t sp = 0; while (!mbar_try_wait(&s_full[t], j & 1) && sp < kSpin) ++sp; got = sp < kSpin; }
        got = __shfl_sync(0xffffffffu, got, 0);
      } else {
        uint32_t sp = 0;
        while (!mbar_try_wait(&s_full[t], j & 1) && sp < kSpin) ++sp;
        got = __all_sync(0xffffffffu, sp < kSpin);
      }
      if (!got) break;
      tc_fence_after();
      if (mode == 2) {
        uint32_t s[4][32];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32(tm_s + c * 32, s[c]);
        tc_wait_ld();
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_st16(tm_s + c * 16, s[c]);
        tc_wait_st();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[t]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}


}  // namespace part2
namespace part3 {
// Microbenchmark 5: latency of each hop of the handshake, isolated: 8 MMAs + commit -> waiter sees the barrier;
// waiter arrives -> MMA thread sees it. try_wait vs test_wait polling.

__device__ long long g_out[256];

__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
template <bool TEST>
__device__ __forceinline__ bool wait_on(uint64_t* bar, uint32_t parity) {
  for (uint32_t i = 0; i < 50000000u; ++i) {
    if (TEST ? mbar_test_wait(bar, parity) : mbar_try_wait(bar, parity)) return true;
  }
  return false;
}

template <bool TEST>
__global__ void __launch_bounds__(384, 1) bench_kernel(int iters, int slot_out) {
  extern __shared__ char smem_raw[];
  char* smem = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  char* sq = smem;
  char* sk = smem + 65536;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 131072);
  uint64_t* s_full = bars;
  uint64_t* p_ready = bars + 1;
  volatile long long* stamps = reinterpret_cast<volatile long long*>(bars + 4);  // [0] seen, [1] arrive
  uint32_t* slot = reinterpret_cast<uint32_t*>(bars + 8);
  for (int i = threadIdx.x; i < 131072 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0x3c003c00u;
  if (threadIdx.x == 0) {
    mbar_init(s_full, 1);
    mbar_init(p_ready, 4);
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == 9) { tmem_alloc(slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *slot;
  if (warp == 9) {
    if (lane == 0) {
      constexpr uint32_t id_qk = make_idesc_f16(128, 128, 1, 0);
      const uint64_t q0 = make_smem_desc_sw128(smem_u32(sq), 16, 1024);
      const uint64_t k0 = make_smem_desc_sw128(smem_u32(sk), 16, 1024);
      long long sum_issue = 0, sum_seen = 0, sum_back = 0, sum_total = 0;
      for (int it = 0; it < iters; ++it) {
        const long long t0 = clock64();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = ((kk >> 2) * 16384 + (kk & 3) * 32) >> 4;
          umma_ss(tmem, q0 + off, k0 + off, id_qk, kk > 0);
        }
        tc_commit(s_full);
        const long long t1 = clock64();
        if (!wait_on<TEST>(p_ready, it & 1)) break;
        const long long t2 = clock64();
        tc_fence_after();
        sum_issue += t1 - t0;
        sum_seen += stamps[0] - t0;     // issue start -> waiter saw S full
        sum_back += t2 - stamps[1];     // waiter arrived -> MMA thread saw P ready
        sum_total += t2 - t0;
      }
      g_out[slot_out * 4 + 0] = sum_issue / iters;
      g_out[slot_out * 4 + 1] = sum_seen / iters;
      g_out[slot_out * 4 + 2] = sum_back / iters;
      g_out[slot_out * 4 + 3] = sum_total / iters;
    }
  } else if (warp < 4) {
    for (int it = 0; it < iters; ++it) {
      const bool got = __all_sync(0xffffffffu, wait_on<TEST>(s_full, it & 1));
      if (!got) break;
      if (threadIdx.x == 0) stamps[0] = clock64();
      tc_fence_after();
      tc_fence_before();
      __syncwarp();
      if (threadIdx.x == 96) stamps[1] = clock64();   // the last warp's arrival completes the barrier (roughly)
      if (lane == 0) mbar_arrive(p_ready);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}


}  // namespace part3
namespace part1 {
int run_part1() {
  const char* names[] = {"warm", "SS N128 same acc", "SS N128 2 accs", "SS N256 same acc", "SS N64 same acc", "TS N128 same acc",
                         "TS N64 same acc", "8xTS(O) then 8xSS(S) [attention order]", "TS/SS alternating instr", "SS N128 4 accs",
                         "SS N256 2 accs", "SS N64 4 accs", "TS N128 2 accs"};
  const int smem = 16384 + 32768 + 1024 + 64;
  cudaFuncSetAttribute(bench_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  for (int grid : {1, 148}) {
    bench_kernel<<<grid, 128, smem>>>(32);
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { printf("error %s\n", cudaGetErrorString(e)); return 1; }
    long long out[64];
    cudaMemcpyFromSymbol(out, g_out, sizeof(out));
    printf("grid %d\n", grid);
    for (int i = 1; i <= 12; ++i)
      printf("  %-42s issue %6.1f cyc/mma   complete %6.1f cyc/mma  (n=%lld)\n", names[i], (double)out[i * 3] / out[i * 3 + 2],
             (double)out[i * 3 + 1] / out[i * 3 + 2], out[i * 3 + 2]);
  }
  return 0;
}

}
namespace part2 {
int run_part2() {
  const int smem = 131072 + 1024 + 256;
  cudaFuncSetAttribute(bench_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  const char* names[] = {"all threads poll, 4 arrivals", "lane 0 polls, 4 arrivals", "all poll + S read / P write"};
  for (int mode = 0; mode < 3; ++mode) {
    bench_kernel<<<148, 384, smem>>>(64, mode, mode);
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { printf("error %s\n", cudaGetErrorString(e)); return 1; }
    long long out[256];
    cudaMemcpyFromSymbol(out, g_out, sizeof(out));
    printf("  %-32s %7.0f cycles per KV block (32 MMAs), MMA warp waited %6.0f of them  (n=%lld)\n", names[mode],
           (double)out[mode * 3] / 64, (double)out[mode * 3 + 1] / 64, out[mode * 3 + 2]);
  }
  return 0;
}

}
namespace part3 {
int run_part3() {
  const int smem = 131072 + 1024 + 256;
  cudaFuncSetAttribute(bench_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  cudaFuncSetAttribute(bench_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  for (int mode = 0; mode < 2; ++mode) {
    if (mode == 0) bench_kernel<false><<<148, 384, smem>>>(200, mode);
    else bench_kernel<true><<<148, 384, smem>>>(200, mode);
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { printf("error %s\n", cudaGetErrorString(e)); return 1; }
    long long out[256];
    cudaMemcpyFromSymbol(out, g_out, sizeof(out));
    printf("  %-10s issue of 8 MMAs + commit %5lld | issue start -> waiter saw S full %5lld (8 MMAs execute in ~520) | "
           "arrive -> MMA thread saw P ready %5lld | round trip %5lld\n", mode ? "test_wait" : "try_wait", out[mode * 4],
           out[mode * 4 + 1], out[mode * 4 + 2], out[mode * 4 + 3]);
  }
  return 0;
}

}

int main() {
  printf("== part 1: cycles per tcgen05.mma (M = 128, K = 16, bf16)\n");
  if (part1::run_part1()) return 1;
  printf("== part 2: 32 MMAs per KV block behind the S-full / P-ready hand-shake\n");
  if (part2::run_part2()) return 1;
  printf("== part 3: hand-shake hop latencies\n");
  return part3::run_part3();
}
