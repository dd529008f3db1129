// Linear layer with a fused epilogue for sm_100a:  out = epilogue(A W^T + bias).
//
// A is (M, K) and W is (N, K), both K-contiguous 16-bit, so both MMA operands are K-major and come straight
// from 128-byte-swizzled TMA tiles. Persistent CTAs (one per SM) walk the output tiles:
//
//   warp 0      TMA producer : A and W tiles of one 64-wide K block per ring stage
//   warp 1      MMA issuer   : four tcgen05.mma (K = 16 each) per stage and 128-row block of the tile
//   warps 2..   epilogue     : four warps per 128-row block. A thread reads its accumulator row from TMEM 64
//                              columns at a time, adds the bias in fp32 and rounds to the storage type (the value
//                              an unfused linear layer would have written); the warp transposes the 32 x 64 piece
//                              through a swizzled 4 KB staging buffer so that eight lanes cover one 128-byte row
//                              segment, applies the tail there -- nothing, tanh-GELU, or residual + gate * value --
//                              and every global load and store of the tail is a full 128-byte line
//
// Tile shapes (rows x columns of the output one CTA owns at a time):
//   128 x 256, 128 x 128  two accumulators in TMEM: the tensor pipe starts the next tile while the previous one is
//                         written out. At full tensor rate a 128 x 256 tile asks L2 for 96 bytes per clock per SM;
//                         measured, the MMA thread waits for operands a fifth of the time.
//   256 x 256             fills all 512 TMEM columns with one tile (its write-out is exposed) but asks for a third
//                         fewer operand bytes per flop.
//   pair                  two CTAs of a cluster (an SM pair) share a 256 x 256 tile with tcgen05.mma.cta_group::2:
//                         each CTA loads its 128 rows of A and HALF of the W tile (128 rows), the pair's tensor
//                         cores exchange the W halves, each CTA accumulates and writes out its own 128 x 256 half
//                         with two accumulators in TMEM. Operand bytes per flop of 256 x 256 and overlapped
//                         write-out. Only the even CTA issues MMAs: both CTAs' copies complete on the even CTA's
//                         "operands landed" barrier (cp.async.bulk.tensor with .cta_group::2 may signal the
//                         partner's barrier), the odd CTA's epilogue warps hand accumulators back by arriving on
//                         the even CTA's barrier, and tcgen05.commit multicasts "stage consumed" / "accumulator
//                         ready" to both CTAs. No TMA multicast is used.
//
// The fused tails remove one full read + write of the activation per layer (GELU) or a read of it plus a write
// (gated residual) that separate elementwise kernels would spend on HBM.
//
// Ragged edges: TMA zero-fills rows beyond M / N and columns beyond K, the epilogue masks its stores.
// All waits on mbarriers are bounded; on time-out the CTA records where it gave up in the device status block,
// waits (bounded) for its copies and MMAs in flight, frees its TMEM and returns (its pair partner runs into its
// own bounded waits and does the same).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <math.h>

#include <mutex>

#include "host_common.h"
#include "ptx_sm100.cuh"

namespace hdit {
namespace {

constexpr int kTileK = 64;  // one 128-byte swizzle row of 16-bit elements
constexpr uint32_t kSpinLimit = 8u * 1000u * 1000u;
constexpr int kMaxSmem = 232448;  // 227 KiB opt-in limit per CTA
// Relative time per 128 x 128 of output for each work-unit shape (1 = the tensor pipe never waits), from
// measurement; used only to choose a shape.
constexpr double kCost128x256 = 1.2, kCost128x128 = 1.75, kCost256x256 = 1.3, kCostPair = 1.05;

#ifdef HDIT_GEMM_TRACE
// per CTA: MMA thread {total, waiting for operands, waiting for a free accumulator, tiles}, epilogue warp 2
// {accumulator ready -> handed back, accumulator ready -> stores issued, tiles, 0}
__device__ long long g_gemm_trace[256][8];
#endif

enum GemmWait : int {
  G_PROD_EMPTY = 201,
  G_MMA_FULL = 202,
  G_MMA_ACC_EMPTY = 203,
  G_EPI_ACC_FULL = 204,
};

template <int BM, int BN, bool PAIR>
struct GemmCfg {
  static_assert(!PAIR || (BM == 128 && BN == 256), "a CTA of a pair owns 128 x 256 of the pair's 256 x 256 tile");
  static constexpr int kHalves = BM / 128;                 // 128-row MMA blocks per CTA tile
  static constexpr int kAccBufs = (kHalves == 1) ? 2 : 1;  // accumulator tiles resident in TMEM
  static constexpr int kEpiWarps = 4 * kHalves;
  static constexpr int kThreads = 64 + 32 * kEpiWarps;
  static constexpr int kTileRows = PAIR ? 2 * BM : BM;     // rows of the scheduling unit's tile
  static constexpr int kBRows = PAIR ? BN / 2 : BN;        // rows of W this CTA loads per stage
  static constexpr int kABytes = BM * kTileK * 2;
  static constexpr int kBBytes = kBRows * kTileK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStagingBytes = kEpiWarps * 4096;   // 32 rows x 128 bytes per epilogue warp
  static constexpr int kBarBytes = 256;
  static constexpr int kStagesFit = (kMaxSmem - 1024 - kBarBytes - kStagingBytes) / kStageBytes;
  static constexpr int kStages = kStagesFit > 8 ? 8 : kStagesFit;
  static constexpr int kTmemCols = kHalves * kAccBufs * BN;
  static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kStagingBytes + kBarBytes;
  static_assert(kTmemCols == 256 || kTmemCols == 512, "TMEM allocation must be a power of two");
  static_assert(kStages >= 3, "ring too short");
};

struct GemmParams {
  CUtensorMap a_map;
  CUtensorMap w_map;
  int M, N, K;
  int m_tiles, n_tiles, k_blocks;
  int group_m;  // tiles are walked in bands of group_m tile rows, so that a wave of CTAs covers a near-square region
  int epilogue;
  int rows_per_batch;
  const uint16_t* bias;
  uint16_t* out;
  long long ldo;
  const uint16_t* residual;
  long long ldr;
  const uint16_t* gate;
  long long gate_batch_stride;
  int32_t* status;
};

// Tile index -> (tile row, tile column): bands of group_m tile rows, column-major inside a band. CTAs that run
// at the same time then share both a few A row blocks and a few W row blocks in L2, instead of one W block and all of A.
__device__ __forceinline__ void tile_coords(const GemmParams& p, int tile, int& m_t, int& n_t) {
  const int per_band = p.group_m * p.n_tiles;
  const int band = tile / per_band, r = tile - band * per_band;
  const int m0 = band * p.group_m;
  const int rows = min(p.group_m, p.m_tiles - m0);
  n_t = r / rows;
  m_t = m0 + (r - n_t * rows);
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const void* tmap, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}

// ---- CTA-pair helpers ------------------------------------------------------------------------------------
// Tiled load into this CTA's shared memory that completes on a barrier of either CTA of the pair
// (`bar_cluster_addr` is a shared::cluster address).
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const void* tmap, uint32_t bar_cluster_addr, int c0,
                                                 int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], "
      "[%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `p` (an address in this CTA's shared memory) as seen in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(const void* p, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
  return r;
}
// What the arrival orders is tensor-memory traffic (tcgen05.fence on both sides), not generic-proxy data, so the
// default semantics suffice; a cluster-scope acquire on the waiting side cost ~500 cycles per wait when measured.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem of both CTAs] (+)= A[smem of each CTA] * B[smem halves of both CTAs]; issued by the even CTA only
__device__ __forceinline__ void umma_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the barrier at `bar`'s offset in both CTAs of the pair once every MMA issued so far is done.
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"(static_cast<uint16_t>(3))
      : "memory");
}

template <bool FP16>
__device__ __forceinline__ float to_f(uint16_t v) {
  if constexpr (FP16) return __half2float(__ushort_as_half(v));
  else return __bfloat162float(__ushort_as_bfloat16(v));
}
template <bool FP16>
__device__ __forceinline__ uint16_t from_f(float f) {
  if constexpr (FP16) return __half_as_ushort(__float2half_rn(f));
  else return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}
template <bool FP16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  return static_cast<uint32_t>(from_f<FP16>(lo)) | (static_cast<uint32_t>(from_f<FP16>(hi)) << 16);
}

__device__ __forceinline__ float gelu_tanh_f(float x) {
  const float u = 0.7978845608028654f * fmaf(0.044715f * x, x * x, x);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  return 0.5f * x * (1.0f + t);
}

template <int BM, int BN, bool PAIR, bool FP16>
__global__ void __launch_bounds__(GemmCfg<BM, BN, PAIR>::kThreads, 1)
    linear_fused_kernel(const __grid_constant__ GemmParams p) {
  using C = GemmCfg<BM, BN, PAIR>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_base = smem;
  uint8_t* staging_base = smem + C::kStages * C::kStageBytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(staging_base + C::kStagingBytes);
  uint64_t* empty = full + 8;
  uint64_t* acc_full = empty + 8;
  uint64_t* acc_empty = acc_full + 2;
  uint64_t* drain_bar = acc_empty + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drain_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;  // position in the CTA pair
  const bool leader = rank == 0;
  const int unit = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int n_units = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&p.a_map);
    tma_prefetch_desc(&p.w_map);
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&full[s], 1);  // pair: only the even CTA's is used; both CTAs' copies complete on it
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < C::kAccBufs; ++i) {
      mbar_init(&acc_full[i], 1);
      // one arrival per epilogue warp; the even CTA of a pair collects both CTAs' epilogue warps
      mbar_init(&acc_empty[i], PAIR ? 2 * C::kEpiWarps : C::kEpiWarps);
    }
    mbar_init(drain_bar, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    if constexpr (PAIR) {
      tmem_alloc_pair(tmem_slot, C::kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, C::kTmemCols);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();  // the partner's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int total_tiles = p.m_tiles * p.n_tiles;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = unit; tile < total_tiles && ok; tile += n_units) {
        int m_t, n_t;
        tile_coords(p, tile, m_t, n_t);
        const int a_row = m_t * C::kTileRows + static_cast<int>(rank) * BM;
        const int w_row = n_t * BN + static_cast<int>(rank) * C::kBRows;
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const uint32_t s = it % C::kStages, round = it / C::kStages;
          if (round > 0 && !mbar_wait_bounded(&empty[s], (round - 1) & 1, abort_flag, kSpinLimit)) {
            report_failure(p.status, abort_flag, HDIT_ERR_PEER_TIMEOUT, G_PROD_EMPTY, static_cast<int>(it));
            ok = false;
            break;
          }
          uint8_t* a_dst = stage_base + s * C::kStageBytes;
          if constexpr (PAIR) {
            // The even CTA announces both CTAs' bytes. The odd CTA's bytes of a round can only come after the
            // even CTA's MMAs of the previous round have released the stage, i.e. never into an earlier phase.
            if (leader) mbar_expect_tx(&full[s], 2 * C::kStageBytes);
            const uint32_t bar = map_to_cta(&full[s], 0);
            tma_load_2d_pair(a_dst, &p.a_map, bar, kb * kTileK, a_row);
            tma_load_2d_pair(a_dst + C::kABytes, &p.w_map, bar, kb * kTileK, w_row);
          } else {
            mbar_expect_tx(&full[s], C::kStageBytes);
            tma_load_2d(a_dst, &p.a_map, &full[s], kb * kTileK, a_row);
            tma_load_2d(a_dst + C::kABytes, &p.w_map, &full[s], kb * kTileK, w_row);
          }
        }
      }
      if (PAIR && !leader) {
        // this CTA's copies complete on the partner's barrier, which cannot be polled from here: after a
        // failure give the few copies in flight time to land before the shared memory is given back
        if (*abort_flag != 0)
          for (int i = 0; i < 64; ++i) __nanosleep(1000);
      } else if (*abort_flag != 0) {
        // copies still in flight must land before the CTA's shared memory is given back
        volatile int never = 0;
        for (uint32_t s = 0; s < static_cast<uint32_t>(C::kStages) && s < it; ++s) {
          const uint32_t last = ((it - 1 - s) / C::kStages) * C::kStages + s;  // last issue that used stage s
          if (last < it) mbar_wait_bounded(&full[s], (last / C::kStages) & 1, &never, kSpinLimit);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && (!PAIR || leader)) {
      // ------------------------------------------------------------------ MMA issuer
      constexpr uint32_t idesc = make_idesc_f16(PAIR ? 256 : 128, BN, FP16 ? 0u : 1u, 0u);
      uint32_t it = 0;
      uint32_t local = 0;
      bool ok = true;
#ifdef HDIT_GEMM_TRACE
      long long tr_wait_full = 0, tr_wait_acc = 0;
      const long long tr_start = clock64();
#endif
      for (int tile = unit; tile < total_tiles && ok; tile += n_units, ++local) {
        const uint32_t acc = local % C::kAccBufs, use = local / C::kAccBufs;
#ifdef HDIT_GEMM_TRACE
        const long long tr_a0 = clock64();
#endif
        if (use > 0 && !mbar_wait_bounded(&acc_empty[acc], (use - 1) & 1, abort_flag, kSpinLimit)) {
          report_failure(p.status, abort_flag, HDIT_ERR_PEER_TIMEOUT, G_MMA_ACC_EMPTY, static_cast<int>(local));
          ok = false;
          break;
        }
        tc_fence_after();
#ifdef HDIT_GEMM_TRACE
        tr_wait_acc += clock64() - tr_a0;
#endif
        const uint32_t d_tmem = tmem_base + acc * C::kHalves * BN;
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const uint32_t s = it % C::kStages, round = it / C::kStages;
#ifdef HDIT_GEMM_TRACE
          const long long tr_f0 = clock64();
#endif
          if (!mbar_wait_bounded(&full[s], round & 1, abort_flag, kSpinLimit)) {
            report_failure(p.status, abort_flag, HDIT_ERR_PEER_TIMEOUT, G_MMA_FULL, static_cast<int>(it));
            ok = false;
            break;
          }
          tc_fence_after();
#ifdef HDIT_GEMM_TRACE
          tr_wait_full += clock64() - tr_f0;
#endif
          const uint32_t a_addr = smem_u32(stage_base + s * C::kStageBytes);
          const uint64_t b_desc = make_smem_desc_sw128(a_addr + C::kABytes, 16, 1024);
#pragma unroll
          for (int h = 0; h < C::kHalves; ++h) {
            const uint64_t a_desc = make_smem_desc_sw128(a_addr + h * (128 * kTileK * 2), 16, 1024);
#pragma unroll
            for (int kk = 0; kk < kTileK / 16; ++kk) {
              const uint64_t off = static_cast<uint64_t>((kk * 32) >> 4);  // 16 elements = 32 bytes along K
              if constexpr (PAIR)
                umma_ss_pair(d_tmem, a_desc + off, b_desc + off, idesc, (kb | kk) != 0 ? 1u : 0u);
              else
                umma_ss(d_tmem + h * BN, a_desc + off, b_desc + off, idesc, (kb | kk) != 0 ? 1u : 0u);
            }
          }
          if constexpr (PAIR) tc_commit_pair(&empty[s]);
          else tc_commit(&empty[s]);
        }
        if (ok) {
          if constexpr (PAIR) tc_commit_pair(&acc_full[acc]);
          else tc_commit(&acc_full[acc]);
        }
      }
#ifdef HDIT_GEMM_TRACE
      g_gemm_trace[blockIdx.x & 255][0] = clock64() - tr_start;
      g_gemm_trace[blockIdx.x & 255][1] = tr_wait_full;
      g_gemm_trace[blockIdx.x & 255][2] = tr_wait_acc;
      g_gemm_trace[blockIdx.x & 255][3] = local;
#endif
      if (*abort_flag != 0) {
        // let the MMAs in flight finish before the TMEM they write is freed
        volatile int never = 0;
        if constexpr (PAIR) tc_commit_pair(drain_bar);
        else tc_commit(drain_bar);
        mbar_wait_bounded(drain_bar, 0, &never, kSpinLimit);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int quarter = warp & 3;  // the TMEM lanes this warp may read: [32 * quarter, 32 * quarter + 32)
    const int half = (warp - 2) >> 2;  // which 128-row block of the tile
    uint8_t* staging = staging_base + (warp - 2) * 4096;
    const int sub_row = lane >> 3, chunk = lane & 7;  // store phase: 4 rows per instruction, 8 lanes per row
    uint32_t local = 0;
    bool ok = true;
#ifdef HDIT_GEMM_TRACE
    long long tr_drain = 0, tr_done = 0, tr_e0 = 0;
#endif
    for (int tile = unit; tile < total_tiles && ok; tile += n_units, ++local) {
      int m_t, n_t;
        tile_coords(p, tile, m_t, n_t);
      const uint32_t acc = local % C::kAccBufs, use = local / C::kAccBufs;
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(&acc_full[acc], use & 1, abort_flag, kSpinLimit))) {
        if (lane == 0) report_failure(p.status, abort_flag, HDIT_ERR_PEER_TIMEOUT, G_EPI_ACC_FULL, static_cast<int>(local));
        ok = false;
        break;
      }
      tc_fence_after();
#ifdef HDIT_GEMM_TRACE
      tr_e0 = clock64();
#endif
      // first of the 32 rows this warp owns
      const long long row0 = static_cast<long long>(m_t) * C::kTileRows + static_cast<long long>(rank) * BM + half * 128 +
                             quarter * 32;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + (acc * C::kHalves + half) * BN;
      long long batch0 = 0, next_batch_row = p.M;
      if (p.epilogue == HDIT_GEMM_BIAS_GATE_RESIDUAL && row0 < p.M) {
        batch0 = static_cast<long long>(static_cast<unsigned>(row0) / static_cast<unsigned>(p.rows_per_batch));
        next_batch_row = (batch0 + 1) * p.rows_per_batch;
      }
#pragma unroll 1
      for (int c = 0; c < BN / 64; ++c) {
        uint32_t r[64];
        tmem_ld32(taddr + c * 64, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
        tmem_ld32(taddr + c * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
        tc_wait_ld();
        if (c == BN / 64 - 1) {
          // the accumulator is in registers: hand it back to the MMA warp before the rest of the last piece
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            if constexpr (PAIR) mbar_arrive_remote(map_to_cta(&acc_empty[acc], 0));
            else mbar_arrive(&acc_empty[acc]);
          }
#ifdef HDIT_GEMM_TRACE
          tr_drain += clock64() - tr_e0;
#endif
        }
        const int col0 = n_t * BN + c * 64;
        // phase 1: row `lane` -> + bias, round, stage (16-byte chunk j of row r sits at chunk j ^ (r & 7))
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          uint4 bv = make_uint4(0, 0, 0, 0);
          if (p.bias != nullptr && col0 + j * 8 < p.N) bv = __ldg(reinterpret_cast<const uint4*>(p.bias + col0 + j * 8));
          const uint16_t* be = reinterpret_cast<const uint16_t*>(&bv);
          uint4 v;
          v.x = pack2<FP16>(__uint_as_float(r[j * 8 + 0]) + to_f<FP16>(be[0]), __uint_as_float(r[j * 8 + 1]) + to_f<FP16>(be[1]));
          v.y = pack2<FP16>(__uint_as_float(r[j * 8 + 2]) + to_f<FP16>(be[2]), __uint_as_float(r[j * 8 + 3]) + to_f<FP16>(be[3]));
          v.z = pack2<FP16>(__uint_as_float(r[j * 8 + 4]) + to_f<FP16>(be[4]), __uint_as_float(r[j * 8 + 5]) + to_f<FP16>(be[5]));
          v.w = pack2<FP16>(__uint_as_float(r[j * 8 + 6]) + to_f<FP16>(be[6]), __uint_as_float(r[j * 8 + 7]) + to_f<FP16>(be[7]));
          *reinterpret_cast<uint4*>(staging + lane * 128 + ((j ^ (lane & 7)) << 4)) = v;
        }
        __syncwarp();
        // phase 2: eight lanes per row, 128 contiguous bytes; the tail runs here
        const int col = col0 + chunk * 8;
        if (col < p.N) {
          if (p.epilogue == HDIT_GEMM_BIAS_GATE_RESIDUAL) {
            uint4 xv[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const long long row = row0 + i * 4 + sub_row;
              xv[i] = (row < p.M) ? *reinterpret_cast<const uint4*>(p.residual + row * p.ldr + col) : make_uint4(0, 0, 0, 0);
            }
            // the 32 rows of this warp lie in at most two batch entries
            const uint4 g_lo = __ldg(reinterpret_cast<const uint4*>(p.gate + batch0 * p.gate_batch_stride + col));
            const uint4 g_hi = (row0 + 31 >= next_batch_row && next_batch_row < p.M)
                                   ? __ldg(reinterpret_cast<const uint4*>(p.gate + (batch0 + 1) * p.gate_batch_stride + col))
                                   : g_lo;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int rl = i * 4 + sub_row;
              const long long row = row0 + rl;
              if (row >= p.M) continue;
              uint4 v = *reinterpret_cast<const uint4*>(staging + rl * 128 + ((chunk ^ (rl & 7)) << 4));
              const uint4 gv = row >= next_batch_row ? g_hi : g_lo;
              const uint16_t* xe = reinterpret_cast<const uint16_t*>(&xv[i]);
              const uint16_t* ge = reinterpret_cast<const uint16_t*>(&gv);
              uint16_t* ve = reinterpret_cast<uint16_t*>(&v);
#pragma unroll
              for (int k = 0; k < 8; ++k)
                ve[k] = from_f<FP16>(fmaf(to_f<FP16>(ge[k]), to_f<FP16>(ve[k]), to_f<FP16>(xe[k])));
              *reinterpret_cast<uint4*>(p.out + row * p.ldo + col) = v;
            }
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int rl = i * 4 + sub_row;
              const long long row = row0 + rl;
              if (row >= p.M) continue;
              uint4 v = *reinterpret_cast<const uint4*>(staging + rl * 128 + ((chunk ^ (rl & 7)) << 4));
              if (p.epilogue == HDIT_GEMM_BIAS_GELU_TANH) {
                uint16_t* ve = reinterpret_cast<uint16_t*>(&v);
#pragma unroll
                for (int k = 0; k < 8; ++k) ve[k] = from_f<FP16>(gelu_tanh_f(to_f<FP16>(ve[k])));
              }
              *reinterpret_cast<uint4*>(p.out + row * p.ldo + col) = v;
            }
          }
        }
        __syncwarp();  // the staging buffer is overwritten by the next piece
      }
#ifdef HDIT_GEMM_TRACE
      tr_done += clock64() - tr_e0;
#endif
    }
#ifdef HDIT_GEMM_TRACE
    if (warp == 2 && lane == 0) {
      g_gemm_trace[blockIdx.x & 255][4] = tr_drain;
      g_gemm_trace[blockIdx.x & 255][5] = tr_done;
      g_gemm_trace[blockIdx.x & 255][6] = local;
    }
#endif
  }

  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();  // nothing of the partner's may still arrive here or read TMEM there
  if (warp == 1) {
    tc_fence_after();
    if constexpr (PAIR) tmem_dealloc_pair(tmem_base, C::kTmemCols);
    else tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// Descriptor over a (rows, K) matrix with K contiguous; box = 64 elements x box_rows rows.
int encode_matrix(CUtensorMap* map, const void* ptr, long long rows, long long k, long long ld, int box_rows,
                  int dtype) {
  EncodeTiledFn enc = encode_fn();
  if (enc == nullptr) return set_error(HDIT_ERR_CUDA, "cuTensorMapEncodeTiled entry point unavailable");
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(kTileK), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = (dtype == HDIT_FP16) ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const CUresult r = enc(map, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return set_error(HDIT_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (rows=%lld k=%lld ld=%lld)",
                     static_cast<int>(r), rows, k, ld);
  return HDIT_OK;
}

int sm_count() {
  static int counts[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (counts[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    counts[dev] = n;
  }
  return counts[dev];
}

template <int BM, int BN, bool PAIR, bool FP16>
int launch_gemm(GemmParams& kp, const hdit_gemm_args* a, cudaStream_t stream) {
  using C = GemmCfg<BM, BN, PAIR>;
  auto kernel = linear_fused_kernel<BM, BN, PAIR, FP16>;
  static int last_dev = -1;
  int dev = 0;
  HDIT_CUDA_OK(cudaGetDevice(&dev));
  if (dev != last_dev) {
    HDIT_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
    last_dev = dev;
  }
  int rc = encode_matrix(&kp.a_map, a->a, a->m, a->k, a->lda, BM, a->dtype);
  if (rc != HDIT_OK) return rc;
  rc = encode_matrix(&kp.w_map, a->w, a->n, a->k, a->ldw, C::kBRows, a->dtype);
  if (rc != HDIT_OK) return rc;
  kp.m_tiles = static_cast<int>((a->m + C::kTileRows - 1) / C::kTileRows);
  kp.n_tiles = static_cast<int>((a->n + BN - 1) / BN);
  const long long tiles = static_cast<long long>(kp.m_tiles) * kp.n_tiles;
  if (tiles > 0x7fffffffLL) return set_error(HDIT_ERR_TOO_LARGE, "more than 2^31 output tiles");
  long long ctas = a->max_ctas > 0 ? a->max_ctas : sm_count();
  {
    // band height: a wave of `units` tiles should read about as many A bytes as W bytes
    const double units = static_cast<double>(PAIR ? (ctas / 2 > 0 ? ctas / 2 : 1) : ctas);
    int g = static_cast<int>(sqrt(units * BN / C::kTileRows) + 0.5);
    if (g < 1) g = 1;
    if (g > kp.m_tiles) g = kp.m_tiles;
    kp.group_m = g;
  }
  if (PAIR) {
    long long pairs = ctas / 2 > 0 ? ctas / 2 : 1;
    if (pairs > tiles) pairs = tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs));
    cfg.blockDim = dim3(C::kThreads);
    cfg.dynamicSmemBytes = C::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    HDIT_CUDA_OK(cudaLaunchKernelEx(&cfg, kernel, kp));
    return HDIT_OK;
  }
  if (ctas > tiles) ctas = tiles;
  kernel<<<static_cast<unsigned>(ctas), C::kThreads, C::kSmemBytes, stream>>>(kp);
  HDIT_CUDA_OK(cudaGetLastError());
  return HDIT_OK;
}

}  // namespace
}  // namespace hdit

#ifdef HDIT_GEMM_TRACE
extern "C" HDIT_API int hdit_gemm_trace_read(long long* out) {
  if (cudaMemcpyFromSymbol(out, hdit::g_gemm_trace, sizeof(long long) * 256 * 8) != cudaSuccess) return 3;
  void* sym = nullptr;
  if (cudaGetSymbolAddress(&sym, hdit::g_gemm_trace) != cudaSuccess) return 3;
  return cudaMemset(sym, 0, sizeof(long long) * 256 * 8) == cudaSuccess ? 0 : 3;
}
#endif

extern "C" int hdit_linear_fused(const hdit_gemm_args* a) {
  using namespace hdit;
  if (a == nullptr) return set_error(HDIT_ERR_BAD_ARG, "null args");
  if (a->dtype != HDIT_BF16 && a->dtype != HDIT_FP16) return set_error(HDIT_ERR_BAD_ARG, "dtype must be bf16 or fp16");
  if (a->epilogue < HDIT_GEMM_BIAS || a->epilogue > HDIT_GEMM_BIAS_GATE_RESIDUAL)
    return set_error(HDIT_ERR_BAD_ARG, "unknown epilogue %d", a->epilogue);
  if (a->m < 0 || a->n <= 0 || a->k <= 0) return set_error(HDIT_ERR_BAD_ARG, "bad m / n / k");
  if (a->m == 0) return HDIT_OK;
  if (a->m > 0x7fffffffLL || a->n > 0x7fffffffLL || a->k > 0x7fffffffLL)
    return set_error(HDIT_ERR_TOO_LARGE, "m, n, k must fit 31 bits");
  if (a->a == nullptr || a->w == nullptr || a->out == nullptr) return set_error(HDIT_ERR_BAD_ARG, "null a / w / out");
  if (a->n % 8 != 0 || a->k % 8 != 0) return set_error(HDIT_ERR_SHAPE, "n and k must be multiples of 8");
  auto bad = [](const void* ptr, long long ld) { return (reinterpret_cast<uintptr_t>(ptr) & 15) != 0 || ld % 8 != 0; };
  if (bad(a->a, a->lda) || bad(a->w, a->ldw) || bad(a->out, a->ldo) || a->lda < a->k || a->ldw < a->k || a->ldo < a->n)
    return set_error(HDIT_ERR_SHAPE, "a / w / out need 16-byte aligned pointers and row strides that are multiples of 8 "
                                     "and cover a row");
  if (a->bias != nullptr && (reinterpret_cast<uintptr_t>(a->bias) & 15) != 0)
    return set_error(HDIT_ERR_SHAPE, "bias pointer not 16-byte aligned");
  if (a->epilogue == HDIT_GEMM_BIAS_GATE_RESIDUAL) {
    if (a->residual == nullptr || a->gate == nullptr || a->rows_per_batch <= 0)
      return set_error(HDIT_ERR_BAD_ARG, "the gated-residual epilogue needs residual, gate and rows_per_batch > 0");
    if (a->rows_per_batch < 32 && a->rows_per_batch < a->m)
      return set_error(HDIT_ERR_SHAPE, "the gated-residual epilogue needs at least 32 rows per batch entry "
                                       "(a warp's 32 rows may span two entries, not more)");
    if (bad(a->residual, a->ldr) || bad(a->gate, a->gate_batch_stride) || a->ldr < a->n)
      return set_error(HDIT_ERR_SHAPE, "residual / gate need 16-byte aligned pointers and strides that are multiples of 8");
  }
  if (a->tile_n != 0 && a->tile_n != 128 && a->tile_n != 256) return set_error(HDIT_ERR_BAD_ARG, "tile_n must be 0, 128 or 256");
  if (a->tile_m != 0 && a->tile_m != 128 && a->tile_m != 256) return set_error(HDIT_ERR_BAD_ARG, "tile_m must be 0, 128 or 256");
  if (a->tile_m == 256 && a->tile_n == 128) return set_error(HDIT_ERR_BAD_ARG, "256-row tiles are 256 columns wide");
  if (a->cta_pair < 0 || a->cta_pair > 2) return set_error(HDIT_ERR_BAD_ARG, "cta_pair must be 0 (choose), 1 (never) or 2 (always)");
  if (a->cta_pair == 2 && (a->tile_m == 128 || a->tile_n == 128))
    return set_error(HDIT_ERR_BAD_ARG, "a CTA pair works on 256 x 256 tiles");

  GemmParams kp;
  kp.M = static_cast<int>(a->m);
  kp.N = static_cast<int>(a->n);
  kp.K = static_cast<int>(a->k);
  kp.m_tiles = 0;
  kp.n_tiles = 0;
  kp.group_m = 1;
  kp.k_blocks = static_cast<int>((a->k + kTileK - 1) / kTileK);
  kp.epilogue = a->epilogue;
  kp.rows_per_batch = static_cast<int>(a->rows_per_batch > 0x7fffffffLL ? 0x7fffffffLL : (a->rows_per_batch > 0 ? a->rows_per_batch : 1));
  kp.bias = static_cast<const uint16_t*>(a->bias);
  kp.out = static_cast<uint16_t*>(a->out);
  kp.ldo = a->ldo;
  kp.residual = static_cast<const uint16_t*>(a->residual);
  kp.ldr = a->ldr;
  kp.gate = static_cast<const uint16_t*>(a->gate);
  kp.gate_batch_stride = a->gate_batch_stride;
  kp.status = device_status_ptr();
  if (kp.status == nullptr) return HDIT_ERR_CUDA;

  // Shape of the work unit: 0 = 128 x 256, 1 = 128 x 128, 2 = 256 x 256 in one CTA, 3 = 256 x 256 on a CTA pair.
  int shape;
  if (a->cta_pair == 2) {
    shape = 3;
  } else if (a->tile_m == 256) {
    shape = 2;
  } else if (a->tile_m == 128 && a->tile_n != 0) {
    shape = a->tile_n == 256 ? 0 : 1;
  } else {
    // Fewest waves, each wave weighted by the time one unit's tile takes: 128 x 128 columns of MMA work per SM,
    // with the measured penalty of the shapes that wait for operands (128-row tiles of one CTA) or expose their
    // write-out (256 x 256 in one CTA).
    const long long sms = a->max_ctas > 0 ? a->max_ctas : sm_count();
    struct Cand { int shape, rows, cols, units_div; double per_tile; };
    const Cand cand[4] = {{0, 128, 256, 1, 2.0 * kCost128x256}, {1, 128, 128, 1, 1.0 * kCost128x128},
                          {2, 256, 256, 1, 4.0 * kCost256x256}, {3, 256, 256, 2, 2.0 * kCostPair}};
    double best = -1.0;
    shape = 0;
    for (const Cand& c : cand) {
      if (a->tile_m != 0 && a->tile_m != c.rows) continue;
      if (a->tile_n != 0 && a->tile_n != c.cols) continue;
      if (c.shape == 3 && a->cta_pair == 1) continue;
      if (c.shape == 2 && a->tile_m != 256) continue;  // one CTA per 256 x 256 tile only on request
      const long long units = sms / c.units_div > 0 ? sms / c.units_div : 1;
      const long long tiles = ((a->m + c.rows - 1) / c.rows) * ((a->n + c.cols - 1) / c.cols);
      const double cost = static_cast<double>((tiles + units - 1) / units) * c.per_tile;
      if (best < 0 || cost < best) best = cost, shape = c.shape;
    }
  }
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(a->stream);
  const bool fp16 = a->dtype == HDIT_FP16;
  switch (shape) {
    case 3: return fp16 ? launch_gemm<128, 256, true, true>(kp, a, stream) : launch_gemm<128, 256, true, false>(kp, a, stream);
    case 2: return fp16 ? launch_gemm<256, 256, false, true>(kp, a, stream) : launch_gemm<256, 256, false, false>(kp, a, stream);
    case 1: return fp16 ? launch_gemm<128, 128, false, true>(kp, a, stream) : launch_gemm<128, 128, false, false>(kp, a, stream);
    default: return fp16 ? launch_gemm<128, 256, false, true>(kp, a, stream) : launch_gemm<128, 256, false, false>(kp, a, stream);
  }
}
