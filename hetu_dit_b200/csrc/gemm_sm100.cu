// Linear layer with a fused epilogue for sm_100a:  out = epilogue(A W^T + bias).
//
// A is (M, K) and W is (N, K), both K-contiguous 16-bit, so both MMA operands are K-major and come straight
// from 128-byte-swizzled TMA tiles. One persistent CTA per SM walks output tiles of BM x BN:
//
//   warp 0      TMA producer : A (BM x 64) and W (BN x 64) tiles of one 64-wide K block per ring stage
//   warp 1      MMA issuer   : four tcgen05.mma 128 x BN x 16 per stage and 128-row half of the tile
//   warps 2..   epilogue     : four warps per 128-row half, one thread per accumulator row; tcgen05.ld 32 columns
//                              at a time, add the bias in fp32, round to the storage type (the value an unfused
//                              linear layer would have written), apply the tail -- nothing, tanh-GELU, or
//                              residual + gate * value -- and store 16 bytes per 8 columns
//
// Tile shapes: 128 x 256 and 128 x 128 keep TWO accumulators in TMEM (2 x BN columns), so the tensor pipe starts
// the next tile while the previous one is still being written out. 256 x 256 fills all 512 TMEM columns with one
// tile (its write-out is exposed) but reads a third fewer operand bytes per flop from L2 -- the SM's ingest from
// L2, not HBM, is what a 128 x 256 tile presses against at full tensor rate (96 bytes per clock per SM).
//
// The fused tails remove one full read + write of the activation per layer (GELU) or a read of it plus a write
// (gated residual) that separate elementwise kernels would spend on HBM.
//
// Ragged edges: TMA zero-fills rows beyond M / N and columns beyond K, the epilogue masks its stores.
// All waits are bounded; on time-out the CTA records where it gave up in the device status block, waits
// (bounded) for its copies and MMAs in flight, frees its TMEM and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <mutex>

#include "host_common.h"
#include "ptx_sm100.cuh"

namespace hdit {
namespace {

constexpr int kTileK = 64;  // one 128-byte swizzle row of 16-bit elements
constexpr uint32_t kSpinLimit = 8u * 1000u * 1000u;
constexpr bool kAuto256 = false;  // whether the automatic choice considers 256 x 256 tiles

enum GemmWait : int {
  G_PROD_EMPTY = 201,
  G_MMA_FULL = 202,
  G_MMA_ACC_EMPTY = 203,
  G_EPI_ACC_FULL = 204,
};

template <int BM, int BN>
struct GemmCfg {
  static constexpr int kHalves = BM / 128;                 // 128-row MMA blocks per tile
  static constexpr int kAccBufs = (kHalves == 1) ? 2 : 1;  // accumulator tiles resident in TMEM
  static constexpr int kEpiWarps = 4 * kHalves;
  static constexpr int kThreads = 64 + 32 * kEpiWarps;
  static constexpr int kABytes = BM * kTileK * 2;
  static constexpr int kBBytes = BN * kTileK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (192 * 1024) / kStageBytes;
  static constexpr int kTmemCols = kHalves * kAccBufs * BN;
  static constexpr int kBarBytes = 256;
  static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kBarBytes;
  static_assert(kTmemCols == 256 || kTmemCols == 512, "TMEM allocation must be a power of two");
};

struct GemmParams {
  CUtensorMap a_map;
  CUtensorMap w_map;
  int M, N, K;
  int m_tiles, n_tiles, k_blocks;
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

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const void* tmap, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
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

__device__ __forceinline__ float gelu_tanh_f(float x) {
  const float u = 0.7978845608028654f * fmaf(0.044715f * x, x * x, x);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  return 0.5f * x * (1.0f + t);
}

template <int BM, int BN, bool FP16>
__global__ void __launch_bounds__(GemmCfg<BM, BN>::kThreads, 1) linear_fused_kernel(const __grid_constant__ GemmParams p) {
  using C = GemmCfg<BM, BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_base = smem;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::kStages * C::kStageBytes);
  uint64_t* empty = full + C::kStages;
  uint64_t* acc_full = empty + C::kStages;
  uint64_t* acc_empty = acc_full + 2;
  uint64_t* drain_bar = acc_empty + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drain_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&p.a_map);
    tma_prefetch_desc(&p.w_map);
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < C::kAccBufs; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], C::kEpiWarps);  // one arrival per epilogue warp
    }
    mbar_init(drain_bar, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int total_tiles = p.m_tiles * p.n_tiles;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int m_t = tile % p.m_tiles, n_t = tile / p.m_tiles;
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const uint32_t s = it % C::kStages, round = it / C::kStages;
          if (round > 0 && !mbar_wait_bounded(&empty[s], (round - 1) & 1, abort_flag, kSpinLimit)) {
            report_failure(p.status, abort_flag, HDIT_ERR_PEER_TIMEOUT, G_PROD_EMPTY, static_cast<int>(it));
            ok = false;
            break;
          }
          uint8_t* a_dst = stage_base + s * C::kStageBytes;
          mbar_expect_tx(&full[s], C::kStageBytes);
          tma_load_2d(a_dst, &p.a_map, &full[s], kb * kTileK, m_t * BM);
          tma_load_2d(a_dst + C::kABytes, &p.w_map, &full[s], kb * kTileK, n_t * BN);
        }
      }
      if (*abort_flag != 0) {
        // copies still in flight must land before the CTA's shared memory is given back
        volatile int never = 0;
        for (uint32_t s = 0; s < static_cast<uint32_t>(C::kStages) && s < it; ++s) {
          const uint32_t last = ((it - 1 - s) / C::kStages) * C::kStages + s;  // last issue that used stage s
          if (last < it) mbar_wait_bounded(&full[s], (last / C::kStages) & 1, &never, kSpinLimit);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(128, BN, FP16 ? 0u : 1u, 0u);
      uint32_t it = 0;
      uint32_t local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
        const uint32_t acc = local % C::kAccBufs, use = local / C::kAccBufs;
        if (use > 0 && !mbar_wait_bounded(&acc_empty[acc], (use - 1) & 1, abort_flag, kSpinLimit)) {
          report_failure(p.status, abort_flag, HDIT_ERR_PEER_TIMEOUT, G_MMA_ACC_EMPTY, static_cast<int>(local));
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * C::kHalves * BN;
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const uint32_t s = it % C::kStages, round = it / C::kStages;
          if (!mbar_wait_bounded(&full[s], round & 1, abort_flag, kSpinLimit)) {
            report_failure(p.status, abort_flag, HDIT_ERR_PEER_TIMEOUT, G_MMA_FULL, static_cast<int>(it));
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(stage_base + s * C::kStageBytes);
          const uint64_t b_desc = make_smem_desc_sw128(a_addr + C::kABytes, 16, 1024);
#pragma unroll
          for (int h = 0; h < C::kHalves; ++h) {
            const uint64_t a_desc = make_smem_desc_sw128(a_addr + h * (128 * kTileK * 2), 16, 1024);
#pragma unroll
            for (int kk = 0; kk < kTileK / 16; ++kk) {
              const uint64_t off = static_cast<uint64_t>((kk * 32) >> 4);  // 16 elements = 32 bytes along K
              umma_ss(d_tmem + h * BN, a_desc + off, b_desc + off, idesc, (kb | kk) != 0 ? 1u : 0u);
            }
          }
          tc_commit(&empty[s]);
        }
        if (ok) tc_commit(&acc_full[acc]);
      }
      if (*abort_flag != 0) {
        // let the MMAs in flight finish before the TMEM they write is freed
        volatile int never = 0;
        tc_commit(drain_bar);
        mbar_wait_bounded(drain_bar, 0, &never, kSpinLimit);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int quarter = warp & 3;  // the TMEM lanes this warp may read: [32 * quarter, 32 * quarter + 32)
    const int half = (warp - 2) >> 2;  // which 128-row block of the tile
    uint32_t local = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
      const int m_t = tile % p.m_tiles, n_t = tile / p.m_tiles;
      const uint32_t acc = local % C::kAccBufs, use = local / C::kAccBufs;
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(&acc_full[acc], use & 1, abort_flag, kSpinLimit))) {
        if (lane == 0) report_failure(p.status, abort_flag, HDIT_ERR_PEER_TIMEOUT, G_EPI_ACC_FULL, static_cast<int>(local));
        ok = false;
        break;
      }
      tc_fence_after();
      const long long row = static_cast<long long>(m_t) * BM + half * 128 + quarter * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + (acc * C::kHalves + half) * BN;
      uint16_t* out_row = p.out + row * p.ldo;
      const uint16_t* res_row = (p.epilogue == HDIT_GEMM_BIAS_GATE_RESIDUAL) ? p.residual + row * p.ldr : nullptr;
      const uint16_t* gate_row = nullptr;
      if (p.epilogue == HDIT_GEMM_BIAS_GATE_RESIDUAL && row_ok)
        gate_row = p.gate + (row / p.rows_per_batch) * p.gate_batch_stride;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(taddr + c * 32, r);
        tc_wait_ld();
        if (c == BN / 32 - 1) {
          // the accumulator is in registers: hand it back to the MMA warp before the arithmetic of the last chunk
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty[acc]);
        }
        const int col0 = n_t * BN + c * 32;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int col = col0 + g * 8;
          if (!row_ok || col >= p.N) continue;
          uint4 bv = make_uint4(0, 0, 0, 0);
          if (p.bias != nullptr) bv = __ldg(reinterpret_cast<const uint4*>(p.bias + col));
          const uint16_t* be = reinterpret_cast<const uint16_t*>(&bv);
          uint4 o;
          uint16_t* oe = reinterpret_cast<uint16_t*>(&o);
          if (p.epilogue == HDIT_GEMM_BIAS_GATE_RESIDUAL) {
            const uint4 xv = *reinterpret_cast<const uint4*>(res_row + col);
            const uint4 gv = __ldg(reinterpret_cast<const uint4*>(gate_row + col));
            const uint16_t* xe = reinterpret_cast<const uint16_t*>(&xv);
            const uint16_t* ge = reinterpret_cast<const uint16_t*>(&gv);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const float y = to_f<FP16>(from_f<FP16>(__uint_as_float(r[g * 8 + k]) + to_f<FP16>(be[k])));
              oe[k] = from_f<FP16>(fmaf(to_f<FP16>(ge[k]), y, to_f<FP16>(xe[k])));
            }
          } else if (p.epilogue == HDIT_GEMM_BIAS_GELU_TANH) {
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const float y = to_f<FP16>(from_f<FP16>(__uint_as_float(r[g * 8 + k]) + to_f<FP16>(be[k])));
              oe[k] = from_f<FP16>(gelu_tanh_f(y));
            }
          } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) oe[k] = from_f<FP16>(__uint_as_float(r[g * 8 + k]) + to_f<FP16>(be[k]));
          }
          *reinterpret_cast<uint4*>(out_row + col) = o;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
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

template <int BM, int BN, bool FP16>
int launch_gemm(GemmParams& kp, const hdit_gemm_args* a, cudaStream_t stream) {
  using C = GemmCfg<BM, BN>;
  auto kernel = linear_fused_kernel<BM, BN, FP16>;
  static int last_dev = -1;
  int dev = 0;
  HDIT_CUDA_OK(cudaGetDevice(&dev));
  if (dev != last_dev) {
    HDIT_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
    last_dev = dev;
  }
  int rc = encode_matrix(&kp.a_map, a->a, a->m, a->k, a->lda, BM, a->dtype);
  if (rc != HDIT_OK) return rc;
  rc = encode_matrix(&kp.w_map, a->w, a->n, a->k, a->ldw, BN, a->dtype);
  if (rc != HDIT_OK) return rc;
  kp.m_tiles = static_cast<int>((a->m + BM - 1) / BM);
  kp.n_tiles = static_cast<int>((a->n + BN - 1) / BN);
  const long long tiles = static_cast<long long>(kp.m_tiles) * kp.n_tiles;
  long long grid = a->max_ctas > 0 ? a->max_ctas : sm_count();
  if (grid > tiles) grid = tiles;
  kernel<<<static_cast<unsigned>(grid), C::kThreads, C::kSmemBytes, stream>>>(kp);
  HDIT_CUDA_OK(cudaGetLastError());
  return HDIT_OK;
}

}  // namespace
}  // namespace hdit

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
    if (bad(a->residual, a->ldr) || bad(a->gate, a->gate_batch_stride) || a->ldr < a->n)
      return set_error(HDIT_ERR_SHAPE, "residual / gate need 16-byte aligned pointers and strides that are multiples of 8");
  }
  if (a->tile_n != 0 && a->tile_n != 128 && a->tile_n != 256) return set_error(HDIT_ERR_BAD_ARG, "tile_n must be 0, 128 or 256");
  if (a->tile_m != 0 && a->tile_m != 128 && a->tile_m != 256) return set_error(HDIT_ERR_BAD_ARG, "tile_m must be 0, 128 or 256");
  if (a->tile_m == 256 && a->tile_n == 128) return set_error(HDIT_ERR_BAD_ARG, "256-row tiles are 256 columns wide");

  GemmParams kp;
  kp.M = static_cast<int>(a->m);
  kp.N = static_cast<int>(a->n);
  kp.K = static_cast<int>(a->k);
  kp.m_tiles = 0;
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

  int tile_m = a->tile_m, tile_n = a->tile_n;
  if (tile_m == 0 || tile_n == 0) {
    // Fewest waves of one-CTA-per-SM work, counted in 128 x 128 units; ties go to the larger tile (fewer operand
    // bytes per flop).
    const long long sms = a->max_ctas > 0 ? a->max_ctas : sm_count();
    auto cost = [&](int bm, int bn) {
      const long long tiles = ((a->m + bm - 1) / bm) * ((a->n + bn - 1) / bn);
      return ((tiles + sms - 1) / sms) * (bm / 128) * (bn / 128);
    };
    const int cand[3][2] = {{128, 256}, {128, 128}, {256, 256}};
    long long best = -1;
    int bm_best = 128, bn_best = 256;
    for (int i = 0; i < 3; ++i) {
      const int bm = cand[i][0], bn = cand[i][1];
      if ((tile_m != 0 && tile_m != bm) || (tile_n != 0 && tile_n != bn)) continue;
      if (bm == 256 && !kAuto256) continue;
      const long long c = cost(bm, bn);
      if (best < 0 || c < best) best = c, bm_best = bm, bn_best = bn;
    }
    if (best < 0) bm_best = tile_m != 0 ? tile_m : 128, bn_best = tile_n != 0 ? tile_n : 256;
    tile_m = bm_best;
    tile_n = bn_best;
    if (tile_m == 256) tile_n = 256;
  }
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(a->stream);
  const bool fp16 = a->dtype == HDIT_FP16;
  if (tile_m == 256) return fp16 ? launch_gemm<256, 256, true>(kp, a, stream) : launch_gemm<256, 256, false>(kp, a, stream);
  if (tile_n == 256) return fp16 ? launch_gemm<128, 256, true>(kp, a, stream) : launch_gemm<128, 256, false>(kp, a, stream);
  return fp16 ? launch_gemm<128, 128, true>(kp, a, stream) : launch_gemm<128, 128, false>(kp, a, stream);
}
