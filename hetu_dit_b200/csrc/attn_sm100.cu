// Joint flash-attention forward for sm_100a.
//
// One CTA owns two 128-row Q tiles of one (batch, head) and walks the KV
// sequence in 128-row blocks:
//
//   warp 8      TMA producer   : Q tiles once, then K/V blocks through two rings
//   warp 9      MMA issuer     : S = Q K^T (tcgen05.mma, smem x smem -> TMEM)
//                                O += P V  (tcgen05.mma, TMEM x smem -> TMEM)
//                                (issuing a tcgen05.mma holds the issuing thread for about as long as the
//                                MMA runs -- 64 cycles at 128x128x16 -- so whatever else this thread does
//                                between two MMAs idles the tensor pipe: operand barriers are polled before
//                                the softmax hand-over, never after it)
//   warps 10-11 idle           : complete the third warpgroup so registers can be handed over
//                                (setmaxnreg: 72 per thread there, 216 for the softmax threads;
//                                72 + 2 * 216 = 3 * 168, the pool the CTA was launched with --
//                                asking for more would block in setmaxnreg.inc for ever)
//   warps 0-3   softmax group 0: owns Q tile 0, one thread per row
//   warps 4-7   softmax group 1: owns Q tile 1
//
// The two softmax groups ping-pong against the tensor pipe: while group 0
// exponentiates S0 the tensor pipe runs P1 V and the next Q1 K^T, and vice versa.
//
// Small grids (fewer tile pairs than SMs, e.g. the head-sharded calls after a Ulysses exchange) run in
// "interleaved" mode instead: a CTA owns ONE Q tile, its two halves (softmax group + MMA issuer each)
// take the even and the odd KV blocks, and the two partial results are merged through shared memory in
// the epilogue -- twice as many CTAs, each half as long, no round trip through HBM.
// P overwrites S in TMEM as packed 16-bit pairs and is consumed from there.
// The running maximum is updated lazily (only when it grows by more than 2^8),
// so O is rescaled in TMEM rarely.
//
// TMEM columns: S0/P0 [0,128)  S1/P1 [128,256)  O0 [256,256+D)  O1 [256+D,256+2D).
//
// Q and K/V are lists of segments (image tokens, text tokens, ring blocks), each
// with its own TMA descriptor, so no concatenated copy exists; a tile or block
// never straddles two segments and ragged tails are masked per block.
//
// All waits are bounded; on time-out the CTA records where it gave up in the
// device status block, drains, frees its TMEM and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>

#include <mutex>
#include <type_traits>

#include "host_common.h"
#include "ptx_sm100.cuh"

namespace hdit {
namespace {

constexpr int kBlockM = 128;
constexpr int kBlockN = 128;
constexpr int kNumThreads = 384;  // 2 softmax warpgroups + 1 warpgroup holding the TMA and MMA warps
constexpr int kPanelBytes = 128 * 128;  // 128 rows x 64 16-bit elements, 128B-swizzled
constexpr uint32_t kSpinLimit = 8u * 1000u * 1000u;
constexpr float kRescaleThreshold = 8.0f;  // log2 units
constexpr float kLn2 = 0.69314718055994531f;
constexpr int kSmCount = 148;

// Development aid (off in the shipped library): -DHDIT_ATTN_TRACE records SM cycle stamps of one CTA's
// softmax and MMA phases for the first 64 KV blocks; hdit_attn_trace_read() copies them out.
#ifdef HDIT_ATTN_TRACE
__device__ long long g_attn_trace[2][64][8];      // [tile][block][event]
__device__ long long g_attn_trace_mma[2][64][4];  // [tile][block][event]
#if HDIT_ATTN_TRACE == 2  // only the loop-start / loop-end stamps of the MMA warp
#define HDIT_TRACE_SM(ev) do {} while (0)
#define HDIT_TRACE_MMA(tt, jj, ev) do {} while (0)
#else
#define HDIT_TRACE_SM(ev)                                                                  \
  do {                                                                                     \
    if (trace_on && row == 0 && j < 64) g_attn_trace[t][j][ev] = clock64();                \
  } while (0)
#define HDIT_TRACE_MMA(tt, jj, ev)                                                         \
  do {                                                                                     \
    if (trace_on && (jj) < 63) g_attn_trace_mma[tt][jj][ev] = clock64();                   \
  } while (0)
#endif
#else
#define HDIT_TRACE_SM(ev) do {} while (0)
#define HDIT_TRACE_MMA(tt, jj, ev) do {} while (0)
#endif

enum Where : int {
  W_PROD_KEMPTY = 1,
  W_PROD_VEMPTY = 2,
  W_MMA_QFULL = 3,
  W_MMA_KFULL = 4,
  W_MMA_VFULL = 5,
  W_MMA_PREADY = 6,
  W_SM_SFULL = 7,
  W_SM_ODONE = 8,
  W_PEER_FLAGS = 9,
};

struct alignas(64) AttnKernelParams {
  CUtensorMap q_map[HDIT_MAX_Q_SEG];
  CUtensorMap k_map[HDIT_MAX_KV_SEG];
  CUtensorMap v_map[HDIT_MAX_KV_SEG];
  int q_len[HDIT_MAX_Q_SEG];
  int kv_len[HDIT_MAX_KV_SEG];
  // 1 if the descriptor's dims are (D, S, H, B) instead of (D, H, S, B)
  unsigned char q_swap[HDIT_MAX_Q_SEG];
  unsigned char k_swap[HDIT_MAX_KV_SEG];
  unsigned char v_swap[HDIT_MAX_KV_SEG];
  int n_q_seg, n_kv_seg;
  int batch, heads;
  int n_tiles_seg0, n_tiles, n_pairs;
  int n_kv_blocks;
  int mode;
  float scale_log2;
  void* out;
  long long out_sb, out_ss, out_sh;
  float* lse;
  float* acc_out;
  float* acc_lse;
  long long sq_total;
  int32_t* status;
  // split-KV: blockIdx.y owns KV blocks [y * kv_split_blocks, ...) and writes its partial result to
  // acc_out + y * split_acc_stride / acc_lse + y * split_lse_stride (0 = no split)
  int kv_split_blocks;
  long long split_acc_stride, split_lse_stride;
  // interleaved mode: one Q tile per CTA, even KV blocks on half 0, odd ones on half 1
  int interleave;
  // result scatter (reverse all-to-all from the epilogue): n_dst == 0 writes `out` only
  int n_dst;
  void* dst[8];
  long long seg_rows_per_dst[HDIT_MAX_Q_SEG];  // 0 = rows of the segment go to every destination
  long long seg_dst_row0[HDIT_MAX_Q_SEG];
  // peers' arrival flags to wait for before the first load (n_wait == 0: none)
  int n_wait;
  const int32_t* wait_slot[8];
  const int32_t* wait_epoch;
  unsigned wait_spins;
};

// Tuning switches (compile-time so that variants can be measured against each other). The defaults are what
// measured fastest on B200: the stale maximum, the polynomial exp2 and a third V stage each measured neutral or
// slower (the S -> P -> MMA chain, not the special-function unit or the loads, bounds a KV block).
//   HDIT_ATTN_STALE_MAX  1: from the second KV block on, exponentiate against the running maximum known
//                           *before* the block (its own maximum is computed alongside and takes effect one
//                           block later), which takes the row-maximum pass off the S -> P critical path.
//   HDIT_ATTN_POLY8      of every 8 scores, how many (0, 2, 4) take a degree-3 polynomial exp2 on the FMA
//                           pipe instead of ex2 on the special-function unit.
//   HDIT_ATTN_VSTAGES128 V ring depth at head_dim 128 (K stays at 2: 227 KB of shared memory).
#ifndef HDIT_ATTN_STALE_MAX
#define HDIT_ATTN_STALE_MAX 0
#endif
#ifndef HDIT_ATTN_POLY8
#define HDIT_ATTN_POLY8 0
#endif
#ifndef HDIT_ATTN_SPLIT_P
#define HDIT_ATTN_SPLIT_P 0  // 1: head_dim 64 keeps P in TMEM columns of its own (see Cfg::kSplitP); measured slower
#endif
#ifndef HDIT_ATTN_LATE_KWAIT
#define HDIT_ATTN_LATE_KWAIT 1  // 1: poll the next K block between P V and Q K^T instead of before the hand-over
#endif
#ifndef HDIT_ATTN_VSTAGES128
#define HDIT_ATTN_VSTAGES128 2
#endif
constexpr float kOverflowGuard = 64.0f;  // log2 units a block may exceed the stale maximum before it is redone

template <int D>
struct Cfg {
  static constexpr int kPanels = D / 64;
  static constexpr int kTileBytes = kPanels * kPanelBytes;
  static constexpr int kStagesK = (D == 128) ? 2 : 4;
  static constexpr int kStagesV = (D == 128) ? HDIT_ATTN_VSTAGES128 : 4;
  static constexpr int kSmemQ = 2 * kTileBytes;
  static constexpr int kSmemK = kStagesK * kTileBytes;
  static constexpr int kSmemV = kStagesV * kTileBytes;
  static constexpr int kSmemBytes = kSmemQ + kSmemK + kSmemV + 1024 /*align*/ + 512 /*barriers etc.*/;
  static_assert(kSmemBytes <= 232448, "exceeds the 227 KB a CTA may use");
  static constexpr uint32_t kTmemCols = 512;
  static constexpr uint32_t kColS = 0;      // + t * 128
  static constexpr uint32_t kColO = 256;    // + t * D
  // head_dim 64 leaves 128 TMEM columns free. With HDIT_ATTN_SPLIT_P, P gets columns of its own there instead of
  // overwriting S, so the next Q K^T of a tile may run as soon as the softmax threads have *read* S, which cuts
  // the S -> P -> P V -> Q K^T chain. Measured on B200 it is slower than the aliased layout (499 vs 596 TFLOP/s at
  // 24 heads x 4429 tokens): both softmax groups then run in phase and contend for the special-function unit,
  // where the aliased schedule keeps them half a block apart. Off by default.
  static constexpr bool kSplitP = (D == 64) && (HDIT_ATTN_SPLIT_P != 0);
  static constexpr uint32_t kColP = kSplitP ? 384 : kColS;  // + t * 64 when split, + t * 128 when aliased on S
  static constexpr uint32_t kStrideP = kSplitP ? 64 : 128;
};

struct KvCursor {
  int seg;
  int row0;
  __device__ __forceinline__ void advance(const AttnKernelParams& p) {
    row0 += kBlockN;
    if (row0 >= p.kv_len[seg]) {
      ++seg;
      row0 = 0;
    }
  }
};

__device__ __forceinline__ void tile_coords(const AttnKernelParams& p, int tile, int& seg, int& row0, int& out_row0) {
  if (tile < p.n_tiles_seg0) {
    seg = 0;
    row0 = tile * kBlockM;
    out_row0 = row0;
  } else {
    seg = 1;
    row0 = (tile - p.n_tiles_seg0) * kBlockM;
    out_row0 = p.q_len[0] + row0;
  }
}

__device__ __forceinline__ void load_tile(const CUtensorMap* map, bool swapped, char* smem, uint64_t* bar, int panels,
                                          int h, int row0, int b) {
  for (int pn = 0; pn < panels; ++pn) {
    if (swapped)
      tma_load_4d(smem + pn * kPanelBytes, map, bar, pn * 64, row0, h, b);
    else
      tma_load_4d(smem + pn * kPanelBytes, map, bar, pn * 64, h, row0, b);
  }
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

template <bool FP16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (FP16) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}

// 2^x for a pair of scores on the FMA pipe: x = n + f with n = round(x), f in [-0.5, 0.5]; 2^f by a degree-3
// polynomial (relative error 7.5e-5, well below the 16-bit rounding of P), 2^n by adding n to the exponent
// field. Inputs below -126 (masked scores are -inf) clamp to 2^-126.
__device__ __forceinline__ float2 ex2_poly2(float2 x) {
  x.x = fmaxf(x.x, -126.0f);
  x.y = fmaxf(x.y, -126.0f);
  const float2 magic = make_float2(12582912.0f, 12582912.0f);  // 1.5 * 2^23: the sum's low mantissa bits hold n
  const float2 t = __fadd2_rn(x, magic);
  const float2 r = __fadd2_rn(t, make_float2(-12582912.0f, -12582912.0f));
  const float2 f = __ffma2_rn(r, make_float2(-1.0f, -1.0f), x);
  float2 q = __ffma2_rn(f, make_float2(0.05517167f, 0.05517167f), make_float2(0.24261113f, 0.24261113f));
  q = __ffma2_rn(q, f, make_float2(0.69326097f, 0.69326097f));
  q = __ffma2_rn(q, f, make_float2(0.99992806f, 0.99992806f));
  float2 out;
  out.x = __int_as_float(__float_as_int(q.x) + (__float_as_int(t.x) << 23));
  out.y = __int_as_float(__float_as_int(q.y) + (__float_as_int(t.y) << 23));
  return out;
}

template <int D, bool FP16, bool IL>
__global__ void __launch_bounds__(kNumThreads, 1) attn_fwd_kernel(const __grid_constant__ AttnKernelParams p) {
  using C = Cfg<D>;
  extern __shared__ char smem_raw[];
  char* smem = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  char* smem_q = smem;
  char* smem_k = smem_q + C::kSmemQ;
  char* smem_v = smem_k + C::kSmemK;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_v + C::kSmemV);
  uint64_t* q_full = bars;                       // [2]
  uint64_t* k_full = q_full + 2;                 // [K stages]
  uint64_t* k_empty = k_full + C::kStagesK;      // [K stages]
  uint64_t* v_full = k_empty + C::kStagesK;      // [V stages]
  uint64_t* v_empty = v_full + C::kStagesV;      // [V stages]
  uint64_t* s_full = v_empty + C::kStagesV;      // [2]
  uint64_t* p_ready = s_full + 2;                // [2]
  uint64_t* o_done = p_ready + 2;                // [2]
  uint64_t* merge_bar = o_done + 2;              // [1] interleaved mode: half 1's partial result is in smem
  uint64_t* s_free = merge_bar + 1;              // [2] split-P: the softmax threads have read S into registers
  uint64_t* pv_done = s_free + 2;                // [2] split-P: P V is done (P may be overwritten, O is stable)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // ---- work item -------------------------------------------------------
  int idx = blockIdx.x;
  const int pair = idx % p.n_pairs;
  idx /= p.n_pairs;
  const int h = idx % p.heads;
  const int b = idx / p.heads;
  constexpr bool il = IL;  // interleaved mode is its own instantiation: the paired loop carries none of its branches
  const int tile0 = il ? pair : pair * 2;
  int j_begin = 0;
  int nblk = p.n_kv_blocks;
  if (p.kv_split_blocks > 0) {
    j_begin = static_cast<int>(blockIdx.y) * p.kv_split_blocks;
    nblk = min(p.n_kv_blocks - j_begin, p.kv_split_blocks);
  }
  // half t (softmax group t + MMA issuer t): its Q tile, and which KV blocks it walks
  const bool half1_active = il ? (nblk >= 2) : ((tile0 + 1) < p.n_tiles);
  const int blk_step = il ? 2 : 1;
  float* const acc_out = p.acc_out + static_cast<long long>(blockIdx.y) * p.split_acc_stride;
  float* const acc_lse = p.acc_lse + static_cast<long long>(blockIdx.y) * p.split_lse_stride;
#ifdef HDIT_ATTN_TRACE
  const bool trace_on = blockIdx.x == gridDim.x / 2 && blockIdx.y == 0;
#endif

  // ---- set-up ----------------------------------------------------------
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_ready[i], 4);  // one arrival per softmax warp
      mbar_init(&o_done[i], 1);
      mbar_init(&s_free[i], 4);
      mbar_init(&pv_done[i], 1);
    }
    mbar_init(merge_bar, 4);
    for (int i = 0; i < C::kStagesK; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
    }
    for (int i = 0; i < C::kStagesV; ++i) {
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Register hand-over between warpgroups: a softmax thread keeps a whole 128-column row of S.
  // Each warpgroup changes its budget at the top of its own branch so the allocation of the code
  // below it is known.
  if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
    if (warp == 8) {
      // =========================== TMA producer ===========================
      bool inputs_ready = true;
      if (p.n_wait > 0) {
        // Q, K and V were stored into this rank's buffers by its Ulysses peers: wait (bounded) until each of them
        // has published the epoch this rank's own exchange kernel advanced to, one lane per peer. The loads below
        // go through the async proxy, hence the proxy fence after the acquire.
        const int32_t epoch = *p.wait_epoch;
        bool seen = true;
        if (lane < p.n_wait && p.wait_slot[lane] != nullptr) {
          seen = false;
          for (unsigned i = 0; i < p.wait_spins; ++i) {
            int32_t v;
            asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p.wait_slot[lane]) : "memory");
            if (v - epoch >= 0) {
              seen = true;
              break;
            }
            __nanosleep(32);
          }
          if (!seen) report_failure(p.status, abort_flag, HDIT_ERR_PEER_TIMEOUT, W_PEER_FLAGS, lane);
        }
        inputs_ready = __all_sync(0xffffffffu, seen);
        asm volatile("fence.proxy.async;" ::: "memory");
      }
      if (lane == 0 && inputs_ready) {
        for (int s = 0; s < p.n_q_seg; ++s) tma_prefetch_desc(&p.q_map[s]);
        for (int s = 0; s < p.n_kv_seg; ++s) {
          tma_prefetch_desc(&p.k_map[s]);
          tma_prefetch_desc(&p.v_map[s]);
        }
        for (int t = 0; t < 2; ++t) {
          if (t == 1 && (il || !half1_active)) break;  // interleaved: both halves share the tile in slot 0
          int seg, row0, orow;
          tile_coords(p, tile0 + t, seg, row0, orow);
          mbar_expect_tx(&q_full[t], C::kTileBytes);
          load_tile(&p.q_map[seg], p.q_swap[seg], smem_q + t * C::kTileBytes, &q_full[t], C::kPanels, h, row0, b);
        }
        KvCursor cur{0, 0};
        for (int i = 0; i < j_begin; ++i) cur.advance(p);
        bool ok = true;
        for (int j = 0; j < nblk && ok; ++j) {
          const int sk = j % C::kStagesK, sv = j % C::kStagesV;
          const uint32_t nk = static_cast<uint32_t>(j / C::kStagesK), nv = static_cast<uint32_t>(j / C::kStagesV);
          if (j >= C::kStagesK) {
            if (!mbar_wait_bounded(&k_empty[sk], (nk - 1) & 1, abort_flag, kSpinLimit)) {
              report_failure(p.status, abort_flag, HDIT_ERR_PEER_TIMEOUT, W_PROD_KEMPTY, j);
              ok = false;
              break;
            }
          }
#if defined(HDIT_ATTN_PROBE) && HDIT_ATTN_PROBE == 3
          // timing probe (wrong results): after the first ring fill nothing is loaded any more
          if (j >= C::kStagesK) {
            mbar_arrive(&k_full[sk]);
          } else
#endif
          {
            mbar_expect_tx(&k_full[sk], C::kTileBytes);
            load_tile(&p.k_map[cur.seg], p.k_swap[cur.seg], smem_k + sk * C::kTileBytes, &k_full[sk], C::kPanels, h,
                      cur.row0, b);
          }
          if (j >= C::kStagesV) {
            if (!mbar_wait_bounded(&v_empty[sv], (nv - 1) & 1, abort_flag, kSpinLimit)) {
              report_failure(p.status, abort_flag, HDIT_ERR_PEER_TIMEOUT, W_PROD_VEMPTY, j);
              ok = false;
              break;
            }
          }
#if defined(HDIT_ATTN_PROBE) && HDIT_ATTN_PROBE == 3
          if (j >= C::kStagesV) {
            mbar_arrive(&v_full[sv]);
          } else
#endif
          {
            mbar_expect_tx(&v_full[sv], C::kTileBytes);
            load_tile(&p.v_map[cur.seg], p.v_swap[cur.seg], smem_v + sv * C::kTileBytes, &v_full[sv], C::kPanels, h,
                      cur.row0, b);
          }
          cur.advance(p);
        }
      }
    } else if (warp == 9) {
      // ============================ MMA issuer ============================
      // One thread issues for both halves. (A second issuing thread, one per half, measured slower: 852 vs
      // 1023 TFLOP/s at the Flux shape -- concurrent issuers slow each other down more than the barrier polls
      // of a single one idle the pipe.)
      if (lane == 0) {
        constexpr uint32_t kFmt = FP16 ? 0u : 1u;
        constexpr uint32_t idesc_qk = make_idesc_f16(kBlockM, kBlockN, kFmt, 0);
        constexpr uint32_t idesc_pv = make_idesc_f16(kBlockM, D, kFmt, 1);
        bool ok = true;
        const int last_t = half1_active ? 1 : 0;
        const int n_iter = il ? (nblk + 1) / 2 : nblk;

        // Descriptors differ from a per-tile base only in the start-address field (low word, units of
        // 16 bytes), so a k-step costs one 32-bit add instead of a rebuilt 64-bit descriptor.
        const uint64_t q_desc0 = make_smem_desc_sw128(smem_u32(smem_q), 16, 1024);
        const uint64_t k_desc0 = make_smem_desc_sw128(smem_u32(smem_k), 16, 1024);
        const uint64_t v_desc0 = make_smem_desc_sw128(smem_u32(smem_v), kPanelBytes, 1024);
        auto issue_qk = [&](int t, int stage) {
          const uint32_t d_tmem = tmem_base + C::kColS + t * 128;
          const uint64_t a0 = q_desc0 + static_cast<uint32_t>(((il ? 0 : t) * C::kTileBytes) >> 4);
          const uint64_t b0 = k_desc0 + static_cast<uint32_t>((stage * C::kTileBytes) >> 4);
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t off = ((kk >> 2) * kPanelBytes + (kk & 3) * 32) >> 4;
            umma_ss(d_tmem, a0 + off, b0 + off, idesc_qk, kk > 0 ? 1u : 0u);
          }
        };
        auto issue_pv = [&](int t, int stage, bool accumulate) {
          const uint32_t d_tmem = tmem_base + C::kColO + t * D;
          const uint32_t a_tmem = tmem_base + C::kColP + t * C::kStrideP;
          const uint64_t b0 = v_desc0 + static_cast<uint32_t>((stage * C::kTileBytes) >> 4);
#pragma unroll
          for (int kk = 0; kk < kBlockN / 16; ++kk) {
            umma_ts(d_tmem, a_tmem + kk * 8, b0 + static_cast<uint32_t>((kk * 2048) >> 4), idesc_pv,
                    (accumulate || kk > 0) ? 1u : 0u);
          }
        };
        auto wait = [&](uint64_t* bar, uint32_t parity, int where, int iter) {
          if (!ok) return;
          if (!mbar_wait_bounded(bar, parity, abort_flag, kSpinLimit)) {
            report_failure(p.status, abort_flag, HDIT_ERR_PEER_TIMEOUT, where, iter);
            ok = false;
          }
        };
        auto k_stage = [](int j) { return j % C::kStagesK; };
        auto k_phase = [](int j) { return static_cast<uint32_t>(j / C::kStagesK) & 1; };
        auto v_stage = [](int j) { return j % C::kStagesV; };
        auto v_phase = [](int j) { return static_cast<uint32_t>(j / C::kStagesV) & 1; };

        // prologue: S of each half's first block (block 0 for both when paired; blocks 0 and 1 when interleaved)
        wait(&q_full[0], 0, W_MMA_QFULL, 0);
        wait(&k_full[0], 0, W_MMA_KFULL, 0);
        if (ok) {
          tc_fence_after();
          issue_qk(0, 0);
          tc_commit(&s_full[0]);
          if (il) tc_commit(&k_empty[0]);
        }
        if (half1_active) {
          const int j1 = il ? 1 : 0;
          if (!il) wait(&q_full[1], 0, W_MMA_QFULL, 1);
          if (il) wait(&k_full[k_stage(1)], k_phase(1), W_MMA_KFULL, 1);
          if (ok) {
            tc_fence_after();
            issue_qk(1, k_stage(j1));
            tc_commit(&s_full[1]);
            if (il) tc_commit(&k_empty[k_stage(1)]);
          }
        }
        if (ok && !il) tc_commit(&k_empty[0]);

#ifdef HDIT_ATTN_TRACE
        if (trace_on) {
          unsigned long long ns;
          asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ns));
          g_attn_trace_mma[0][63][0] = clock64();
          g_attn_trace_mma[0][63][1] = static_cast<long long>(ns);
        }
#endif
        if constexpr (C::kSplitP) {
          // P has its own columns: per round, first the next Q K^T of every half (needs only that the softmax
          // threads have read the current S), then the P V of every half as its P arrives.
          for (int i = 0; i < n_iter && ok; ++i) {
            for (int t = 0; t <= last_t && ok; ++t) {
              const int j = il ? 2 * i + t : i;
              const int jn = j + blk_step;
              if (j >= nblk || jn >= nblk) continue;
              if (il || t == 0) wait(&k_full[k_stage(jn)], k_phase(jn), W_MMA_KFULL, jn);
              wait(&s_free[t], i & 1, W_MMA_PREADY, 1000 + i * 2 + t);
              if (!ok) break;
              tc_fence_after();
              issue_qk(t, k_stage(jn));
              tc_commit(&s_full[t]);
              if (il || t == last_t) tc_commit(&k_empty[k_stage(jn)]);
            }
            for (int t = 0; t <= last_t && ok; ++t) {
              const int j = il ? 2 * i + t : i;
              if (j >= nblk) break;
              if (il || t == 0) wait(&v_full[v_stage(j)], v_phase(j), W_MMA_VFULL, j);
              wait(&p_ready[t], i & 1, W_MMA_PREADY, i * 2 + t);
              if (!ok) break;
              tc_fence_after();
              issue_pv(t, v_stage(j), i > 0);
              tc_commit(&pv_done[t]);
              if (j + blk_step >= nblk) tc_commit(&o_done[t]);
              if (il || t == last_t) tc_commit(&v_empty[v_stage(j)]);
            }
          }
        } else
        for (int i = 0; i < n_iter && ok; ++i) {
          for (int t = 0; t <= last_t && ok; ++t) {
            // half t's i-th KV block and the one after it
            const int j = il ? 2 * i + t : i;
            if (j >= nblk) break;  // interleaved, odd block count: half 1 has one block fewer
            const int jn = j + blk_step;
            const bool has_next = jn < nblk;
            const bool releases = il || t == last_t;  // the last reader of a stage hands it back
            if (il || t == 0) {
              wait(&v_full[v_stage(j)], v_phase(j), W_MMA_VFULL, j);
#if !HDIT_ATTN_LATE_KWAIT
              if (has_next) wait(&k_full[k_stage(jn)], k_phase(jn), W_MMA_KFULL, jn);
#endif
            }
            HDIT_TRACE_MMA(t, i, 0);
            wait(&p_ready[t], i & 1, W_MMA_PREADY, i * 2 + t);
            HDIT_TRACE_MMA(t, i, 1);
            if (!ok) break;
            tc_fence_after();
            issue_pv(t, v_stage(j), i > 0);
            if (releases) tc_commit(&v_empty[v_stage(j)]);  // at once: the V ring is only two deep at head_dim 128
            if (has_next) {
#if HDIT_ATTN_LATE_KWAIT
              if (il || t == 0) wait(&k_full[k_stage(jn)], k_phase(jn), W_MMA_KFULL, jn);
              if (!ok) break;
#endif
              issue_qk(t, k_stage(jn));
              tc_commit(&s_full[t]);
              if (releases) tc_commit(&k_empty[k_stage(jn)]);
            } else {
              tc_commit(&o_done[t]);
            }
            HDIT_TRACE_MMA(t, i, 2);
          }
        }
#ifdef HDIT_ATTN_TRACE
        if (trace_on) {
          unsigned long long ns;
          asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ns));
          g_attn_trace_mma[0][63][2] = clock64();
          g_attn_trace_mma[0][63][3] = static_cast<long long>(ns);
        }
#endif
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
    // ========================= softmax / epilogue =========================
    const int t = warp >> 2;           // which half (Q tile, or KV parity when interleaved) this warpgroup owns
    const int quarter = warp & 3;      // TMEM lane quarter this warp may touch
    const int row = quarter * 32 + lane;
    const bool active = (t == 0) || half1_active;
    if (active) {
      const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
      const uint32_t tm_s = tmem_base + lane_base + C::kColS + t * 128;
      const uint32_t tm_p = tmem_base + lane_base + C::kColP + t * C::kStrideP;
      const uint32_t tm_o = tmem_base + lane_base + C::kColO + t * D;
      const float scale_log2 = p.scale_log2;
      float m_run = -INFINITY;   // maximum the stored P and O are scaled against (log2 units)
      float m_pend = -INFINITY;  // largest score seen so far; m_run catches up with it lazily
      float l_run = 0.f;
      bool ok = true;
      const int first = il ? t : 0;
      const int n_mine = il ? (nblk - t + 1) / 2 : nblk;
      KvCursor cur{0, 0};
      for (int i = 0; i < j_begin + first; ++i) cur.advance(p);

      for (int j = 0; j < n_mine; ++j) {  // j counts this half's blocks
        HDIT_TRACE_SM(0);
        // warp-uniform outcome: the tcgen05.ld/st below need the whole warp converged
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(&s_full[t], j & 1, abort_flag, kSpinLimit))) {
          report_failure(p.status, abort_flag, HDIT_ERR_PEER_TIMEOUT, W_SM_SFULL, j * 2 + t);
          ok = false;
          break;
        }
        tc_fence_after();
        HDIT_TRACE_SM(1);
        const int valid = min(kBlockN, p.kv_len[cur.seg] - cur.row0);
        for (int i = 0; i < blk_step; ++i) cur.advance(p);
#if defined(HDIT_ATTN_PROBE) && (HDIT_ATTN_PROBE == 1 || HDIT_ATTN_PROBE == 3)
        // timing probe (wrong results): no softmax work at all, only the barrier hand-shake
        m_run = 0.f;
        l_run = 1.f;
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_ready[t]);
        continue;
#endif
        uint32_t s[4][32];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32(tm_s + c * 32, s[c]);
        tc_wait_ld();
        HDIT_TRACE_SM(2);
        if constexpr (C::kSplitP) {
          // S is in registers: the issuer may overwrite it with the next block's scores
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&s_free[t]);
        }

#if defined(HDIT_ATTN_PROBE) && HDIT_ATTN_PROBE == 2
        // timing probe (wrong results): S is read and P written, but nothing is computed
        m_run = 0.f;
        l_run = 1.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_st16(tm_s + c * 16, s[c]);
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_ready[t]);
        continue;
#endif
        if (valid < kBlockN) {
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (c * 32 + i >= valid) s[c][i] = 0xff800000u;  // -inf
        }

        // split-P: the previous P V of this half must be done before its P is overwritten or O is rescaled. The
        // wait sits as late as possible (before the first P store / inside the rare rescale), so that the P V
        // runs under this block's load and maximum passes.
        bool pv_waited = !C::kSplitP || j == 0;
        auto wait_pv_done = [&]() {
          if (pv_waited) return;
          pv_waited = true;
          if (!__all_sync(0xffffffffu, mbar_wait_bounded(&pv_done[t], (j - 1) & 1, abort_flag, kSpinLimit))) {
            report_failure(p.status, abort_flag, HDIT_ERR_PEER_TIMEOUT, W_SM_ODONE, 100 + j * 2 + t);
            ok = false;
          }
          tc_fence_after();
        };
        // Rescale the running state to a larger maximum (rare: only when it grows by more than 2^8).
        auto rescale_to = [&](bool grow, float m_new) {
          const float alpha = grow ? ex2_approx(m_run - m_new) : 1.0f;
          if (grow) m_run = m_new;
          l_run *= alpha;
          if (j > 0) {
            // O(t) is stable here: the commit that raised s_full covered the previous P V (split-P: wait for it)
            wait_pv_done();
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
              uint32_t o[32];
              tmem_ld32(tm_o + c * 32, o);
              tc_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              tmem_st32(tm_o + c * 32, o);
            }
          }
        };
        // P = 2^(s * scale - m_run) for the whole row, stored over S as packed 16-bit pairs; returns the row sum.
        // With track_max the row maximum of the raw scores is computed in the same pass. Packed fp32x2 FMA and
        // add halve the issue slots; of every 8 scores the last HDIT_ATTN_POLY8 take the polynomial exp2.
        auto exp_pass = [&](auto track_max, float& raw_max) -> float {
          const float2 scale2 = make_float2(scale_log2, scale_log2);
          const float2 neg_m2 = make_float2(-m_run, -m_run);
          float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
          float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t pk[16];
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              const float2 r0 = make_float2(__uint_as_float(s[c][i]), __uint_as_float(s[c][i + 1]));
              const float2 r1 = make_float2(__uint_as_float(s[c][i + 2]), __uint_as_float(s[c][i + 3]));
              if constexpr (decltype(track_max)::value) {
                mx0 = max3(mx0, r0.x, r0.y);
                mx1 = max3(mx1, r1.x, r1.y);
              }
              const float2 x0 = __ffma2_rn(r0, scale2, neg_m2);
              const float2 x1 = __ffma2_rn(r1, scale2, neg_m2);
              // position of this group of four within its group of eight decides the pipe
              constexpr int kPolyPairs = HDIT_ATTN_POLY8 / 2;
              const bool second_half = (i & 4) != 0;
              const bool poly0 = second_half ? (kPolyPairs >= 2) : (kPolyPairs >= 4);
              const bool poly1 = second_half ? (kPolyPairs >= 1) : (kPolyPairs >= 3);
              const float2 p0 = poly0 ? ex2_poly2(x0) : make_float2(ex2_approx(x0.x), ex2_approx(x0.y));
              const float2 p1 = poly1 ? ex2_poly2(x1) : make_float2(ex2_approx(x1.x), ex2_approx(x1.y));
              acc0 = __fadd2_rn(acc0, p0);
              acc1 = __fadd2_rn(acc1, p1);
              pk[i >> 1] = pack2<FP16>(p0.x, p0.y);
              pk[(i >> 1) + 1] = pack2<FP16>(p1.x, p1.y);
            }
            if (c == 0) wait_pv_done();
            tmem_st16(tm_p + c * 16, pk);
          }
          raw_max = fmaxf(mx0, mx1);
          return (acc0.x + acc0.y) + (acc1.x + acc1.y);
        };

        bool classic = (j == 0) || (HDIT_ATTN_STALE_MAX == 0);
        if (!classic) {
          // The maximum used for this block is the one known before it; what the previous block added to it
          // takes effect now.
          const bool grow = (m_pend - m_run) > kRescaleThreshold;
          if (__any_sync(0xffffffffu, grow)) rescale_to(grow, m_pend);
          HDIT_TRACE_SM(3);
          float raw_max;
          const float sum = exp_pass(std::true_type{}, raw_max);
          const float m_blk = raw_max * scale_log2;
          if (__any_sync(0xffffffffu, (m_blk - m_run) > kOverflowGuard)) {
            classic = true;  // a score far above everything seen so far: redo the block against its own maximum
          } else {
            l_run += sum;
            m_pend = fmaxf(m_run, m_blk);
          }
        }
        if (classic) {
          float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              mx0 = max3(mx0, __uint_as_float(s[c][i]), __uint_as_float(s[c][i + 1]));
              mx1 = max3(mx1, __uint_as_float(s[c][i + 2]), __uint_as_float(s[c][i + 3]));
              mx2 = max3(mx2, __uint_as_float(s[c][i + 4]), __uint_as_float(s[c][i + 5]));
              mx3 = max3(mx3, __uint_as_float(s[c][i + 6]), __uint_as_float(s[c][i + 7]));
            }
          const float m_blk = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * scale_log2;
          const float m_new = fmaxf(m_run, m_blk);
          const bool grow = (m_new - m_run) > kRescaleThreshold;  // true on the first block (m_run = -inf)
          if (__any_sync(0xffffffffu, grow)) rescale_to(grow, m_new);
          if (j == 0) HDIT_TRACE_SM(3);
          float unused;
          l_run += exp_pass(std::false_type{}, unused);
          m_pend = fmaxf(m_run, m_blk);
        }
        HDIT_TRACE_SM(4);
        if (!ok) break;
        tc_wait_st();
        tc_fence_before();
        // one arrival per warp: 128 arrivals on one barrier word would serialise on the S -> P -> MMA path
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_ready[t]);
        HDIT_TRACE_SM(5);
      }

      // ------------------------------ epilogue ------------------------------
      if (ok && !__all_sync(0xffffffffu, mbar_wait_bounded(&o_done[t], 0, abort_flag, kSpinLimit))) {
        report_failure(p.status, abort_flag, HDIT_ERR_PEER_TIMEOUT, W_SM_ODONE, t);
        ok = false;
      }
      // Interleaved mode: half 1 hands its unnormalised partial result (O1, m1, l1) to half 0 through the
      // K / V rings, which no MMA reads any more once both halves are done.
      float* const xo = reinterpret_cast<float*>(smem_k);   // [D][128] fp32, column-major: conflict-free
      float* const xml = reinterpret_cast<float*>(smem_v);  // [2][128]: m, l
      float scale0 = 1.0f, scale1 = 0.0f;
      bool writes_result = true;
      if (il && t == 1) {
        writes_result = false;
        if (ok && !__all_sync(0xffffffffu, mbar_wait_bounded(&o_done[0], 0, abort_flag, kSpinLimit))) {
          report_failure(p.status, abort_flag, HDIT_ERR_PEER_TIMEOUT, W_SM_ODONE, 2);
          ok = false;
        }
        if (ok) {
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tmem_ld32(tm_o + c * 32, o);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) xo[(c * 32 + i) * 128 + row] = __uint_as_float(o[i]);
          }
          xml[row] = m_run;
          xml[128 + row] = l_run;
          __syncwarp();
          if (lane == 0) mbar_arrive(merge_bar);
        }
      } else if (il && half1_active) {
        if (ok && !__all_sync(0xffffffffu, mbar_wait_bounded(merge_bar, 0, abort_flag, kSpinLimit))) {
          report_failure(p.status, abort_flag, HDIT_ERR_PEER_TIMEOUT, W_SM_ODONE, 3);
          ok = false;
        }
        if (ok) {
          const float m1 = xml[row], l1 = xml[128 + row];
          const float m = fmaxf(m_run, m1);
          scale0 = ex2_approx(m_run - m);
          scale1 = ex2_approx(m1 - m);
          l_run = scale0 * l_run + scale1 * l1;
          m_run = m;
        }
      }
      if (ok && writes_result) {
        tc_fence_after();
        int seg, row0, orow0;
        tile_coords(p, tile0 + (il ? 0 : t), seg, row0, orow0);
        const bool row_valid = (row0 + row) < p.q_len[seg];
        const long long qpos = orow0 + row;
        const float blk_lse2 = m_run + log2f(l_run);  // log2 domain
        float w_blk = 1.0f / l_run;
        float w_prev = 0.f;
        float lse_out = blk_lse2 * kLn2;
        const long long acc_row = ((static_cast<long long>(b) * p.sq_total + qpos) * p.heads + h) * D;
        const long long lse_idx = (static_cast<long long>(b) * p.heads + h) * p.sq_total + qpos;
        const bool merge = (p.mode == HDIT_ATTN_PARTIAL_MERGE || p.mode == HDIT_ATTN_MERGE_FINAL);
        const bool to_acc = (p.mode == HDIT_ATTN_PARTIAL_FIRST || p.mode == HDIT_ATTN_PARTIAL_MERGE);
        if (merge && row_valid) {
          const float prev = acc_lse[lse_idx];
          const float blk = blk_lse2 * kLn2;
          const float mx = fmaxf(prev, blk);
          const float merged = mx + logf(expf(prev - mx) + expf(blk - mx));
          w_prev = expf(prev - merged);
          w_blk = expf(blk - merged) / l_run;
          lse_out = merged;
        }
        if (row_valid) {
          if (to_acc)
            acc_lse[lse_idx] = lse_out;
          else if (p.lse != nullptr)
            p.lse[lse_idx] = lse_out;
        }
        // where the 16-bit result row goes: `out`, or (reverse all-to-all) the buffer of the rank that owns the row
        int d_lo = 0, d_hi = 1;
        long long drow = qpos;
        if (p.n_dst > 0) {
          const long long r = row0 + row;  // row within its Q segment
          const long long rpd = p.seg_rows_per_dst[seg];
          if (rpd > 0) {
            d_lo = static_cast<int>(r / rpd);
            d_hi = d_lo + 1;
            drow = p.seg_dst_row0[seg] + (r - d_lo * rpd);
          } else {
            d_lo = 0;
            d_hi = p.n_dst;
            drow = p.seg_dst_row0[seg] + r;
          }
        }
        const float w0 = w_blk * scale0, w1 = w_blk * scale1;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          tmem_ld32(tm_o + c * 32, o);
          tc_wait_ld();
          if (row_valid) {
            float f[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(o[i]) * w0;
            if (il && half1_active) {
#pragma unroll
              for (int i = 0; i < 32; ++i) f[i] = fmaf(xo[(c * 32 + i) * 128 + row], w1, f[i]);
            }
            if (merge) {
              const float4* prev = reinterpret_cast<const float4*>(acc_out + acc_row + c * 32);
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const float4 v = prev[i];
                f[4 * i + 0] = fmaf(v.x, w_prev, f[4 * i + 0]);
                f[4 * i + 1] = fmaf(v.y, w_prev, f[4 * i + 1]);
                f[4 * i + 2] = fmaf(v.z, w_prev, f[4 * i + 2]);
                f[4 * i + 3] = fmaf(v.w, w_prev, f[4 * i + 3]);
              }
            }
            if (to_acc) {
              float4* dst = reinterpret_cast<float4*>(acc_out + acc_row + c * 32);
#pragma unroll
              for (int i = 0; i < 8; ++i) dst[i] = make_float4(f[4 * i], f[4 * i + 1], f[4 * i + 2], f[4 * i + 3]);
            } else {
              uint4 v[4];
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                v[i].x = pack2<FP16>(f[8 * i + 0], f[8 * i + 1]);
                v[i].y = pack2<FP16>(f[8 * i + 2], f[8 * i + 3]);
                v[i].z = pack2<FP16>(f[8 * i + 4], f[8 * i + 5]);
                v[i].w = pack2<FP16>(f[8 * i + 6], f[8 * i + 7]);
              }
              const long long off = static_cast<long long>(b) * p.out_sb + drow * p.out_ss +
                                    static_cast<long long>(h) * p.out_sh + c * 32;
              for (int d = d_lo; d < d_hi; ++d) {
                uint16_t* base = reinterpret_cast<uint16_t*>(p.n_dst > 0 ? p.dst[d] : p.out) + off;
                uint4* dst = reinterpret_cast<uint4*>(base);
#pragma unroll
                for (int i = 0; i < 4; ++i) dst[i] = v[i];
              }
            }
          }
        }
      }
    }
  }

  // ---- teardown ----------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0) {
    // Let anything this CTA still has in flight (TMA writes, MMAs) land before
    // its shared memory and TMEM go back to the SM.
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 9) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
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

// Descriptor over a (B, S, H, D) tensor, box = 64 elements x 128 rows of one head.
int encode_seg(CUtensorMap* map, unsigned char* swapped, const hdit_seg& seg, int dtype, int B, int H, int D) {
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return set_error(HDIT_ERR_CUDA, "cuTensorMapEncodeTiled entry point unavailable");
  if (seg.ptr == nullptr || seg.len <= 0) return set_error(HDIT_ERR_BAD_ARG, "segment with null pointer or len <= 0");
  if ((reinterpret_cast<uintptr_t>(seg.ptr) & 15) != 0)
    return set_error(HDIT_ERR_SHAPE, "segment pointer not 16-byte aligned");
  if (seg.stride_s % 8 != 0 || seg.stride_h % 8 != 0 || seg.stride_b % 8 != 0)
    return set_error(HDIT_ERR_SHAPE, "segment strides must be multiples of 8 elements");
  if (seg.stride_s < D || (H > 1 && seg.stride_h < D))
    return set_error(HDIT_ERR_SHAPE, "segment rows overlap (stride < head_dim)");
  const long long sh = (H > 1) ? seg.stride_h : D;
  long long sb = seg.stride_b;
  if (B == 1 || sb <= 0) {
    // Size-1 batch: any stride addresses the same data; give the descriptor a legal one.
    const long long span_s = seg.stride_s * seg.len;
    const long long span_h = sh * H;
    sb = span_s > span_h ? span_s : span_h;
  }
  const bool swap = sh > seg.stride_s;  // keep descriptor strides ascending
  cuuint64_t dims[4];
  cuuint64_t strides[3];
  cuuint32_t box[4];
  cuuint32_t estr[4] = {1, 1, 1, 1};
  dims[0] = static_cast<cuuint64_t>(D);
  box[0] = 64;
  if (!swap) {
    dims[1] = static_cast<cuuint64_t>(H);
    dims[2] = static_cast<cuuint64_t>(seg.len);
    strides[0] = static_cast<cuuint64_t>(sh) * 2;
    strides[1] = static_cast<cuuint64_t>(seg.stride_s) * 2;
    box[1] = 1;
    box[2] = kBlockN;
  } else {
    dims[1] = static_cast<cuuint64_t>(seg.len);
    dims[2] = static_cast<cuuint64_t>(H);
    strides[0] = static_cast<cuuint64_t>(seg.stride_s) * 2;
    strides[1] = static_cast<cuuint64_t>(sh) * 2;
    box[1] = kBlockN;
    box[2] = 1;
  }
  dims[3] = static_cast<cuuint64_t>(B);
  strides[2] = static_cast<cuuint64_t>(sb) * 2;
  box[3] = 1;
  const CUtensorMapDataType dt = (dtype == HDIT_FP16) ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const CUresult r = enc(map, dt, 4, const_cast<void*>(seg.ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return set_error(HDIT_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (len=%lld strides=%lld,%lld,%lld)",
                     static_cast<int>(r), static_cast<long long>(seg.len), static_cast<long long>(seg.stride_b),
                     static_cast<long long>(seg.stride_s), static_cast<long long>(seg.stride_h));
  *swapped = swap ? 1 : 0;
  return HDIT_OK;
}

template <int D, bool FP16, bool IL>
int launch(const AttnKernelParams& kp, int grid, int grid_y, cudaStream_t stream) {
  auto kernel = attn_fwd_kernel<D, FP16, IL>;
  // The attribute is per device: set it whenever this thread meets a new device.
  static thread_local int last_dev = -1;
  int dev = 0;
  HDIT_CUDA_OK(cudaGetDevice(&dev));
  if (dev != last_dev) {
    HDIT_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<D>::kSmemBytes));
    last_dev = dev;
  }
  kernel<<<dim3(grid, grid_y), kNumThreads, Cfg<D>::kSmemBytes, stream>>>(kp);
  HDIT_CUDA_OK(cudaGetLastError());
  return HDIT_OK;
}

// Result scatter of the split-KV merge pass (same meaning as in AttnKernelParams).
struct ScatterParams {
  int n_dst;
  long long q_len0;  // length of Q segment 0 (rows below it belong to segment 0)
  void* dst[8];
  long long seg_rows_per_dst[HDIT_MAX_Q_SEG];
  long long seg_dst_row0[HDIT_MAX_Q_SEG];
};

// Merges the partial results of a split-KV launch: out = sum_s w_s O_s with w_s = exp(lse_s - lse),
// lse = log sum_s exp(lse_s). One warp per (batch, query, head) row, one vector load per lane and split.
// NS > 0 fixes the split count at compile time: all partial rows and LSEs of a row are then requested
// before any of them is used (the kernel is latency-bound: 17 MB per call at the Flux shape).
template <int D, bool FP16, int NS>
__global__ void __launch_bounds__(256) attn_combine_kernel(const float* __restrict__ part_out,
                                                          const float* __restrict__ part_lse, int n_split,
                                                          long long acc_stride, long long lse_stride, int batch,
                                                          long long sq, int heads, void* out, long long out_sb,
                                                          long long out_ss, long long out_sh, float* lse,
                                                          const __grid_constant__ ScatterParams sc) {
  constexpr int E = D / 32;  // floats per lane: 4 (D = 128) or 2 (D = 64)
  constexpr int kMaxNs = NS > 0 ? NS : 1;
  const int lane = threadIdx.x & 31;
  const long long n_rows = static_cast<long long>(batch) * sq * heads;
  const long long warps = static_cast<long long>(gridDim.x) * 8;
  for (long long r = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5); r < n_rows; r += warps) {
    const int h = static_cast<int>(r % heads);
    const long long bq = r / heads;
    const long long q = bq % sq;
    const int b = static_cast<int>(bq / sq);
    const long long lse_idx = (static_cast<long long>(b) * heads + h) * sq + q;
    const float* src0 = part_out + r * D + lane * E;
    float acc[E];
    float mx = -INFINITY, wsum = 0.f;
    if constexpr (NS > 0) {
      float l[kMaxNs];
      float o[kMaxNs][E];
#pragma unroll
      for (int s = 0; s < NS; ++s) {
        l[s] = part_lse[s * lse_stride + lse_idx];
        if constexpr (E == 4) {
          const float4 v = *reinterpret_cast<const float4*>(src0 + s * acc_stride);
          o[s][0] = v.x, o[s][1] = v.y, o[s][2] = v.z, o[s][3] = v.w;
        } else {
          const float2 v = *reinterpret_cast<const float2*>(src0 + s * acc_stride);
          o[s][0] = v.x, o[s][1] = v.y;
        }
      }
#pragma unroll
      for (int s = 0; s < NS; ++s) mx = fmaxf(mx, l[s]);
#pragma unroll
      for (int i = 0; i < E; ++i) acc[i] = 0.f;
#pragma unroll
      for (int s = 0; s < NS; ++s) {
        const float w = expf(l[s] - mx);
        wsum += w;
#pragma unroll
        for (int i = 0; i < E; ++i) acc[i] = fmaf(w, o[s][i], acc[i]);
      }
    } else {
      for (int s = 0; s < n_split; ++s) mx = fmaxf(mx, part_lse[s * lse_stride + lse_idx]);
#pragma unroll
      for (int i = 0; i < E; ++i) acc[i] = 0.f;
      for (int s = 0; s < n_split; ++s) {
        const float w = expf(part_lse[s * lse_stride + lse_idx] - mx);
        wsum += w;
        const float* src = src0 + s * acc_stride;
#pragma unroll
        for (int i = 0; i < E; ++i) acc[i] = fmaf(w, src[i], acc[i]);
      }
    }
    const float inv = 1.0f / wsum;
    int d_lo = 0, d_hi = 1;
    long long drow = q;
    if (sc.n_dst > 0) {
      const int seg = (q >= sc.q_len0) ? 1 : 0;
      const long long r = seg ? q - sc.q_len0 : q;
      const long long rpd = sc.seg_rows_per_dst[seg];
      if (rpd > 0) {
        d_lo = static_cast<int>(r / rpd);
        d_hi = d_lo + 1;
        drow = sc.seg_dst_row0[seg] + (r - d_lo * rpd);
      } else {
        d_hi = sc.n_dst;
        drow = sc.seg_dst_row0[seg] + r;
      }
    }
    for (int d = d_lo; d < d_hi; ++d) {
      uint16_t* dst = reinterpret_cast<uint16_t*>(sc.n_dst > 0 ? sc.dst[d] : out) + b * out_sb + drow * out_ss +
                      static_cast<long long>(h) * out_sh + lane * E;
      if constexpr (E == 4) {
        uint2 v;
        v.x = pack2<FP16>(acc[0] * inv, acc[1] * inv);
        v.y = pack2<FP16>(acc[2] * inv, acc[3] * inv);
        *reinterpret_cast<uint2*>(dst) = v;
      } else {
        *reinterpret_cast<uint32_t*>(dst) = pack2<FP16>(acc[0] * inv, acc[1] * inv);
      }
    }
    if (lse != nullptr && lane == 0) lse[lse_idx] = mx + logf(wsum);
  }
}

int attn_fwd_impl(const hdit_attn_args* a, int n_split, float* split_out, float* split_lse);

}  // namespace
}  // namespace hdit

#ifdef HDIT_ATTN_TRACE
extern "C" __attribute__((visibility("default"))) int hdit_attn_trace_read(long long* softmax_out, long long* mma_out) {
  using namespace hdit;
  HDIT_CUDA_OK(cudaMemcpyFromSymbol(softmax_out, g_attn_trace, sizeof(long long) * 2 * 64 * 8));
  HDIT_CUDA_OK(cudaMemcpyFromSymbol(mma_out, g_attn_trace_mma, sizeof(long long) * 2 * 64 * 4));
  return HDIT_OK;
}
#endif

extern "C" int hdit_attn_fwd(const hdit_attn_args* a) { return hdit::attn_fwd_impl(a, 1, nullptr, nullptr); }

extern "C" int hdit_attn_fwd_splitkv(const hdit_attn_args* a, int32_t n_split, float* split_out, float* split_lse) {
  using namespace hdit;
  if (n_split < 1 || n_split > 16) return set_error(HDIT_ERR_BAD_ARG, "n_split must be 1..16");
  if (n_split == 1) return attn_fwd_impl(a, 1, nullptr, nullptr);
  if (a == nullptr) return set_error(HDIT_ERR_BAD_ARG, "args is null");
  if (a->mode != HDIT_ATTN_FINAL) return set_error(HDIT_ERR_BAD_ARG, "split-KV needs mode HDIT_ATTN_FINAL");
  if (split_out == nullptr || split_lse == nullptr || (reinterpret_cast<uintptr_t>(split_out) & 15) != 0)
    return set_error(HDIT_ERR_BAD_ARG, "split scratch missing or misaligned");
  return attn_fwd_impl(a, n_split, split_out, split_lse);
}

namespace hdit {
namespace {

int attn_fwd_impl(const hdit_attn_args* a, int n_split, float* split_out, float* split_lse) {
  if (a == nullptr) return set_error(HDIT_ERR_BAD_ARG, "args is null");
  if (a->dtype != HDIT_BF16 && a->dtype != HDIT_FP16) return set_error(HDIT_ERR_BAD_ARG, "dtype must be bf16 or fp16");
  if (a->head_dim != 64 && a->head_dim != 128) return set_error(HDIT_ERR_SHAPE, "head_dim must be 64 or 128");
  if (a->batch <= 0 || a->heads <= 0) return set_error(HDIT_ERR_BAD_ARG, "batch and heads must be positive");
  if (a->n_q_seg < 1 || a->n_q_seg > HDIT_MAX_Q_SEG) return set_error(HDIT_ERR_SHAPE, "n_q_seg out of range");
  if (a->n_kv_seg < 1 || a->n_kv_seg > HDIT_MAX_KV_SEG) return set_error(HDIT_ERR_SHAPE, "n_kv_seg out of range");
  if (a->mode < HDIT_ATTN_FINAL || a->mode > HDIT_ATTN_MERGE_FINAL) return set_error(HDIT_ERR_BAD_ARG, "unknown mode");
  const bool needs_acc = a->mode != HDIT_ATTN_FINAL;
  const bool needs_out = a->mode == HDIT_ATTN_FINAL || a->mode == HDIT_ATTN_MERGE_FINAL;
  if (needs_acc && (a->acc_out == nullptr || a->acc_lse == nullptr))
    return set_error(HDIT_ERR_BAD_ARG, "acc_out / acc_lse required for partial and merge modes");
  if (a->n_out_dst < 0 || a->n_out_dst > 8) return set_error(HDIT_ERR_BAD_ARG, "n_out_dst must be 0..8");
  if (a->kv_interleave < 0 || a->kv_interleave > 2) return set_error(HDIT_ERR_BAD_ARG, "kv_interleave must be 0, 1 or 2");
  if (needs_out) {
    if (a->n_out_dst == 0) {
      if (a->out == nullptr) return set_error(HDIT_ERR_BAD_ARG, "out is null");
      if ((reinterpret_cast<uintptr_t>(a->out) & 15) != 0)
        return set_error(HDIT_ERR_SHAPE, "out must be 16-byte aligned with strides multiple of 8 elements");
    }
    for (int i = 0; i < a->n_out_dst; ++i)
      if (a->out_dst[i] == nullptr || (reinterpret_cast<uintptr_t>(a->out_dst[i]) & 15) != 0)
        return set_error(HDIT_ERR_BAD_ARG, "out_dst[%d] is null or not 16-byte aligned", i);
    if (a->out_stride_s % 8 != 0 || a->out_stride_h % 8 != 0 || a->out_stride_b % 8 != 0)
      return set_error(HDIT_ERR_SHAPE, "out must be 16-byte aligned with strides multiple of 8 elements");
  }
  if (needs_acc && (reinterpret_cast<uintptr_t>(a->acc_out) & 15) != 0)
    return set_error(HDIT_ERR_SHAPE, "acc_out must be 16-byte aligned");

  AttnKernelParams kp;
  memset(&kp, 0, sizeof(kp));
  kp.batch = a->batch;
  kp.heads = a->heads;
  kp.mode = a->mode;

  // Drop empty segments so the kernel never sees a zero-length block list.
  long long sq = 0;
  int nq = 0;
  for (int i = 0; i < a->n_q_seg; ++i) {
    if (a->q[i].len < 0) return set_error(HDIT_ERR_BAD_ARG, "negative q segment length");
    if (a->q[i].len == 0) continue;
    if (a->q[i].len > 0x7fffff00LL) return set_error(HDIT_ERR_TOO_LARGE, "q segment too long");
    const int rc = encode_seg(&kp.q_map[nq], &kp.q_swap[nq], a->q[i], a->dtype, a->batch, a->heads, a->head_dim);
    if (rc != HDIT_OK) return rc;
    kp.q_len[nq] = static_cast<int>(a->q[i].len);
    sq += a->q[i].len;
    ++nq;
  }
  if (nq == 0) return HDIT_OK;  // nothing to compute
  int nkv = 0;
  int nblk = 0;
  for (int i = 0; i < a->n_kv_seg; ++i) {
    if (a->k[i].len != a->v[i].len) return set_error(HDIT_ERR_SHAPE, "k and v segment lengths differ");
    if (a->k[i].len < 0) return set_error(HDIT_ERR_BAD_ARG, "negative kv segment length");
    if (a->k[i].len == 0) continue;
    if (a->k[i].len > 0x7fffff00LL) return set_error(HDIT_ERR_TOO_LARGE, "kv segment too long");
    int rc = encode_seg(&kp.k_map[nkv], &kp.k_swap[nkv], a->k[i], a->dtype, a->batch, a->heads, a->head_dim);
    if (rc != HDIT_OK) return rc;
    rc = encode_seg(&kp.v_map[nkv], &kp.v_swap[nkv], a->v[i], a->dtype, a->batch, a->heads, a->head_dim);
    if (rc != HDIT_OK) return rc;
    kp.kv_len[nkv] = static_cast<int>(a->k[i].len);
    nblk += static_cast<int>((a->k[i].len + kBlockN - 1) / kBlockN);
    ++nkv;
  }
  if (nkv == 0) return set_error(HDIT_ERR_SHAPE, "attention over an empty key/value sequence");
  kp.n_q_seg = nq;
  kp.n_kv_seg = nkv;
  kp.n_kv_blocks = nblk;
  kp.n_tiles_seg0 = (kp.q_len[0] + kBlockM - 1) / kBlockM;
  kp.n_tiles = kp.n_tiles_seg0 + (nq > 1 ? (kp.q_len[1] + kBlockM - 1) / kBlockM : 0);
  kp.n_pairs = (kp.n_tiles + 1) / 2;
  kp.sq_total = sq;
  const float scale = a->softmax_scale > 0.f ? a->softmax_scale : 1.0f / sqrtf(static_cast<float>(a->head_dim));
  kp.scale_log2 = scale * 1.4426950408889634f;
  kp.out = a->out;
  kp.out_sb = a->out_stride_b;
  kp.out_ss = a->out_stride_s;
  kp.out_sh = a->out_stride_h;
  kp.lse = a->lse;
  kp.acc_out = a->acc_out;
  kp.acc_lse = a->acc_lse;
  kp.status = device_status_ptr();
  if (kp.status == nullptr) return HDIT_ERR_CUDA;
  ScatterParams sc;
  memset(&sc, 0, sizeof(sc));
  if (needs_out && a->n_out_dst > 0) {
    // the segment index of a row is its position in the caller's list; empty segments were dropped above, so
    // map the caller's per-segment values onto the kernel's compacted list
    int kq = 0;
    for (int i = 0; i < a->n_q_seg; ++i) {
      if (a->q[i].len == 0) continue;
      if (a->q_rows_per_dst[i] < 0 || a->q_dst_row0[i] < 0)
        return set_error(HDIT_ERR_BAD_ARG, "negative q_rows_per_dst / q_dst_row0");
      if (a->q_rows_per_dst[i] > 0 && (a->q[i].len + a->q_rows_per_dst[i] - 1) / a->q_rows_per_dst[i] > a->n_out_dst)
        return set_error(HDIT_ERR_SHAPE, "q segment %d: %lld rows at %lld per destination exceed %d destinations", i,
                         static_cast<long long>(a->q[i].len), static_cast<long long>(a->q_rows_per_dst[i]),
                         a->n_out_dst);
      kp.seg_rows_per_dst[kq] = sc.seg_rows_per_dst[kq] = a->q_rows_per_dst[i];
      kp.seg_dst_row0[kq] = sc.seg_dst_row0[kq] = a->q_dst_row0[i];
      ++kq;
    }
    kp.n_dst = sc.n_dst = a->n_out_dst;
    sc.q_len0 = kp.q_len[0];
    for (int i = 0; i < a->n_out_dst; ++i) kp.dst[i] = sc.dst[i] = a->out_dst[i];
  }

  if (a->n_wait < 0 || a->n_wait > 8) return set_error(HDIT_ERR_BAD_ARG, "n_wait must be 0..8");
  if (a->n_wait > 0) {
    if (a->wait_epoch == nullptr) return set_error(HDIT_ERR_BAD_ARG, "wait_epoch is null");
    kp.n_wait = a->n_wait;
    for (int i = 0; i < a->n_wait; ++i) kp.wait_slot[i] = a->wait_slots[i];
    kp.wait_epoch = a->wait_epoch;
    const long long spins = a->wait_spins > 0 ? a->wait_spins : 20000000LL;
    kp.wait_spins = static_cast<unsigned>(spins > 0xffffffffLL ? 0xffffffffLL : spins);
  }

  // Interleaved mode (one Q tile per CTA, its two halves on the even and odd KV blocks): taken when it cuts
  // the number of CTA waves, i.e. for grids smaller than the GPU. Costs are in KV blocks of one CTA.
  if (n_split <= 1 && a->kv_interleave != 1 && nblk >= 2) {
    const long long ctas_pair = static_cast<long long>(kp.n_pairs) * a->heads * a->batch;
    const long long ctas_il = static_cast<long long>(kp.n_tiles) * a->heads * a->batch;
    // measured at 3 heads x 4608 tokens, head_dim 128: an interleaved iteration (two KV blocks, each ring
    // effectively half as deep) costs 1.12 paired blocks; about 6 blocks' worth of fixed cost per CTA
    const double t_pair = static_cast<double>((ctas_pair + kSmCount - 1) / kSmCount) * (nblk + 6.0);
    const double t_il = static_cast<double>((ctas_il + kSmCount - 1) / kSmCount) * ((nblk + 1) / 2 * 1.12 + 6.0);
    if (a->kv_interleave == 2 || t_il * 1.05 < t_pair) {
      kp.interleave = 1;
      kp.n_pairs = kp.n_tiles;
    }
  }

  const long long grid = static_cast<long long>(kp.n_pairs) * a->heads * a->batch;
  if (grid > 0x7fffffffLL) return set_error(HDIT_ERR_TOO_LARGE, "grid too large");
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(a->stream);
  const bool fp16 = a->dtype == HDIT_FP16;
  int grid_y = 1;
  if (n_split > 1 && nblk >= 2) {
    // every split gets the same number of 128-row KV blocks (the last one possibly fewer, never zero)
    const int bps = (nblk + n_split - 1) / n_split;
    grid_y = (nblk + bps - 1) / bps;
    kp.kv_split_blocks = bps;
    kp.mode = HDIT_ATTN_PARTIAL_FIRST;
    kp.acc_out = split_out;
    kp.acc_lse = split_lse;
    kp.split_acc_stride = static_cast<long long>(a->batch) * sq * a->heads * a->head_dim;
    kp.split_lse_stride = static_cast<long long>(a->batch) * a->heads * sq;
  }
  int rc;
  const int g = static_cast<int>(grid);
  if (kp.interleave) {
    if (a->head_dim == 128)
      rc = fp16 ? launch<128, true, true>(kp, g, grid_y, stream) : launch<128, false, true>(kp, g, grid_y, stream);
    else
      rc = fp16 ? launch<64, true, true>(kp, g, grid_y, stream) : launch<64, false, true>(kp, g, grid_y, stream);
  } else {
    if (a->head_dim == 128)
      rc = fp16 ? launch<128, true, false>(kp, g, grid_y, stream) : launch<128, false, false>(kp, g, grid_y, stream);
    else
      rc = fp16 ? launch<64, true, false>(kp, g, grid_y, stream) : launch<64, false, false>(kp, g, grid_y, stream);
  }
  if (rc != HDIT_OK || grid_y == 1) return rc;
  const long long n_rows = static_cast<long long>(a->batch) * sq * a->heads;
  long long blocks = (n_rows + 7) / 8;
  if (blocks > 148LL * 8) blocks = 148LL * 8;
#define HDIT_COMBINE_NS(DD, FF, NN)                                                                                \
  attn_combine_kernel<DD, FF, NN><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(                               \
      split_out, split_lse, grid_y, kp.split_acc_stride, kp.split_lse_stride, a->batch, sq, a->heads, a->out,      \
      a->out_stride_b, a->out_stride_s, a->out_stride_h, a->lse, sc)
#define HDIT_COMBINE(DD, FF)                                                                                       \
  do {                                                                                                             \
    if (grid_y == 2) HDIT_COMBINE_NS(DD, FF, 2);                                                                   \
    else if (grid_y == 3) HDIT_COMBINE_NS(DD, FF, 3);                                                              \
    else if (grid_y == 4) HDIT_COMBINE_NS(DD, FF, 4);                                                              \
    else HDIT_COMBINE_NS(DD, FF, 0);                                                                               \
  } while (0)
  if (a->head_dim == 128) {
    if (fp16) HDIT_COMBINE(128, true); else HDIT_COMBINE(128, false);
  } else {
    if (fp16) HDIT_COMBINE(64, true); else HDIT_COMBINE(64, false);
  }
#undef HDIT_COMBINE_NS
#undef HDIT_COMBINE
  HDIT_CUDA_OK(cudaGetLastError());
  return HDIT_OK;
}

}  // namespace
}  // namespace hdit

// ---------------------------------------------------------------------------------------------
// Two-pass attention whose fp32 running result lives in a static device array.
//
// Some hosts of this library cannot allocate device memory around a call: a serving process whose HBM
// is wholly reserved by its own pool (so a raw cudaMalloc fails or fragments it), or a denoising loop
// that must not take the device-wide synchronisation cudaMalloc / cudaFree imply. For them the
// partial-result buffers of the PARTIAL_FIRST -> MERGE_FINAL sequence are carved out of the array
// below instead of being passed in. Every GPU that loads the library holds these 32.5 MiB until exit.
namespace hdit {
namespace {

constexpr size_t kStaticAccFloats = size_t(8) << 20;    // fp32 partial output, 32 MiB
constexpr size_t kStaticLseFloats = size_t(128) << 10;  // fp32 log-sum-exp, 512 KiB
static __device__ __align__(256) float g_static_attn_scratch[kStaticAccFloats + kStaticLseFloats];

// Host code must not hand the symbol itself to a kernel: on the host the name is only a stand-in.
// Its device address is looked up once per device, with that device current.
float* g_static_scratch_addr[64] = {nullptr};
std::mutex g_static_scratch_mutex;

int static_scratch_for_current_device(float** out) {
  int dev = 0;
  HDIT_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return set_error(HDIT_ERR_CUDA, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    HDIT_CUDA_OK(cudaGetSymbolAddress(&p, g_static_attn_scratch));
    g_static_scratch_addr[dev] = static_cast<float*>(p);
  }
  *out = g_static_scratch_addr[dev];
  return HDIT_OK;
}

}  // namespace
}  // namespace hdit

extern "C" int hdit_attn_fwd_split_static(const hdit_attn_args* a, int32_t first_pass_kv_segs) {
  using namespace hdit;
  if (a == nullptr) return set_error(HDIT_ERR_BAD_ARG, "args is null");
  if (a->mode != HDIT_ATTN_FINAL) return set_error(HDIT_ERR_BAD_ARG, "mode must be HDIT_ATTN_FINAL");
  if (a->n_kv_seg < 2 || a->n_kv_seg > HDIT_MAX_KV_SEG || first_pass_kv_segs < 1 || first_pass_kv_segs >= a->n_kv_seg)
    return set_error(HDIT_ERR_BAD_ARG, "need 1 <= first_pass_kv_segs (%d) < n_kv_seg (%d)", first_pass_kv_segs,
                     a->n_kv_seg);
  if (a->n_q_seg < 1 || a->n_q_seg > HDIT_MAX_Q_SEG || a->batch <= 0 || a->heads <= 0 || a->head_dim <= 0)
    return set_error(HDIT_ERR_BAD_ARG, "bad batch / heads / head_dim / n_q_seg");
  long long sq = 0;
  for (int i = 0; i < a->n_q_seg; ++i) {
    if (a->q[i].len < 0) return set_error(HDIT_ERR_BAD_ARG, "negative q segment length");
    sq += a->q[i].len;
  }
  long long kv_first = 0, kv_second = 0;
  for (int i = 0; i < a->n_kv_seg; ++i) {
    if (a->k[i].len < 0) return set_error(HDIT_ERR_BAD_ARG, "negative kv segment length");
    (i < first_pass_kv_segs ? kv_first : kv_second) += a->k[i].len;
  }
  if (sq == 0) return HDIT_OK;
  if (kv_first == 0 || kv_second == 0) return hdit_attn_fwd(a);  // one side is empty: a single pass is the answer
  const unsigned long long acc_need = 1ull * a->batch * sq * a->heads * a->head_dim;
  const unsigned long long lse_need = 1ull * a->batch * a->heads * sq;
  if (acc_need > kStaticAccFloats || lse_need > kStaticLseFloats)
    return set_error(HDIT_ERR_TOO_LARGE,
                     "static scratch too small: batch*Sq*heads*head_dim = %llu (max %llu), batch*heads*Sq = %llu "
                     "(max %llu); use hdit_attn_fwd with caller-provided acc_out / acc_lse instead",
                     acc_need, (unsigned long long)kStaticAccFloats, lse_need, (unsigned long long)kStaticLseFloats);
  float* scratch = nullptr;
  const int rc = static_scratch_for_current_device(&scratch);
  if (rc != HDIT_OK) return rc;

  hdit_attn_args first = *a;
  first.mode = HDIT_ATTN_PARTIAL_FIRST;
  first.n_kv_seg = first_pass_kv_segs;
  first.out = nullptr;
  first.lse = nullptr;
  first.acc_out = scratch;
  first.acc_lse = scratch + kStaticAccFloats;
  const int rc1 = hdit_attn_fwd(&first);
  if (rc1 != HDIT_OK) return rc1;

  hdit_attn_args second = *a;
  second.mode = HDIT_ATTN_MERGE_FINAL;
  second.n_kv_seg = a->n_kv_seg - first_pass_kv_segs;
  for (int i = 0; i < second.n_kv_seg; ++i) {
    second.k[i] = a->k[first_pass_kv_segs + i];
    second.v[i] = a->v[first_pass_kv_segs + i];
  }
  second.acc_out = scratch;
  second.acc_lse = scratch + kStaticAccFloats;
  return hdit_attn_fwd(&second);
}
