// Fused per-head RMSNorm + rotary embedding + (optional) Ulysses head scatter.
//
// One pass over Q, K (and V, copy only) of a layer: each thread owns 8
// consecutive elements (16 bytes) of one (token, head) row, the row's threads
// reduce the sum of squares with shuffles, and the result is written either in
// place, to a plain destination, or head-sliced into up to 8 destination
// buffers (one per Ulysses peer, mapped peer memory included) at a sequence
// offset -- which turns the head->sequence all-to-all into the epilogue of this
// kernel. HBM-bound: 2 bytes read + 2 bytes written per element plus the
// L2-resident cos/sin rows.
//
// Rounding follows the reference's eager sequence so results agree to the
// last bit wherever the fp32 reduction order does: normalise in fp32, round to
// the 16-bit type, multiply by the 16-bit weight and round, rotate in fp32 with
// separately rounded products, round once more.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "host_common.h"

namespace hdit {
namespace {

constexpr int kMaxDst = 8;
constexpr int kMaxTensors = 3;

struct NormRopeTensor {
  const void* x;
  long long xs_b, xs_s, xs_h;
  const void* weight;  // 16-bit (D) or null
  const void* bias;    // 16-bit (D) or null (LayerNorm mode only)
  int do_norm;         // 0 none, 1 RMSNorm, 2 LayerNorm
  int do_rope;
  void* dst[kMaxDst];
  long long ds_b, ds_s, ds_h;
  long long dst_seq_offset;
};

struct NormRopeParams {
  NormRopeTensor t[kMaxTensors];
  int n_tensors;
  int batch, seq, heads;
  int n_dst;           // heads are split evenly over n_dst destinations
  float eps;
  const float* cos_tab;  // (rope_rows, D) fp32
  const float* sin_tab;
  long long rope_seq_start;  // tokens below this index are not rotated
  long long rope_row0;       // table row of token rope_seq_start
  // second row range: tokens >= range2_start take these norm weights / rotary rows instead (seq = none)
  long long range2_start;
  const void* weight2[kMaxTensors];
  const void* bias2[kMaxTensors];
  int do_rope2[kMaxTensors];
  long long rope_row0_2;
  // after the last CTA: publish the next epoch to the peers' flag slots (0 = no signal)
  int n_signal;
  int signal_me;
  int32_t* signal_slot[kMaxDst];
  int32_t* epoch_counter;
  unsigned int* ticket;
};

__device__ __forceinline__ void nr_st_release_sys(int32_t* p, int32_t v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

template <bool FP16>
__device__ __forceinline__ float to_f(uint16_t v) {
  if constexpr (FP16)
    return __half2float(__ushort_as_half(v));
  else
    return __bfloat162float(__ushort_as_bfloat16(v));
}
template <bool FP16>
__device__ __forceinline__ uint16_t from_f(float f) {
  if constexpr (FP16)
    return __half_as_ushort(__float2half_rn(f));
  else
    return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}

// Grid size per SM. A CTA that handles a single pair of tokens lives for one load round trip, and the launch
// and retirement of thousands of such CTAs is what the kernel then spends its time on; a few CTAs per SM that
// loop over many token pairs keep their loads in flight back to back.
#ifndef HDIT_NR_CTAS_PER_SM
#define HDIT_NR_CTAS_PER_SM 32
#endif

// Resident CTAs per SM the register allocation aims for (bytes in flight per SM = CTAs x threads x 32). Measured at
// the Flux shape (4608 tokens, 24 x 128, Q and K): 2 -> 46.5 us, 3 (40 registers, small spills) -> 50.1 us.
#ifndef HDIT_NR_MIN_CTAS
#define HDIT_NR_MIN_CTAS 2
#endif

template <int D, bool FP16>
__global__ void __launch_bounds__(512, HDIT_NR_MIN_CTAS) norm_rope_kernel(const __grid_constant__ NormRopeParams p) {
  constexpr int TPR = D / 8;  // threads per (token, head) row
  const NormRopeTensor& t = p.t[blockIdx.y];
  const int rows_per_iter = blockDim.x / TPR;
  const int part = threadIdx.x % TPR;
  const int row_in_blk = threadIdx.x / TPR;
  const int heads_per_dst = p.heads / p.n_dst;
  const long long n_tok = static_cast<long long>(p.batch) * p.seq;

  // Two tokens per pass: both 16-byte loads of a thread are issued before either is used, which doubles the
  // bytes in flight per resident thread (the kernel is latency-bound: one short dependent chain per load).
  for (long long tok0 = blockIdx.x; tok0 < n_tok; tok0 += 2LL * gridDim.x) {
    const long long toks[2] = {tok0, tok0 + gridDim.x};
    const int n_here = toks[1] < n_tok ? 2 : 1;
    int bb_[2], ss_[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const long long tk = j < n_here ? toks[j] : toks[0];
      bb_[j] = static_cast<int>(tk / p.seq);
      ss_[j] = static_cast<int>(tk - static_cast<long long>(bb_[j]) * p.seq);
    }
    // All threads of a warp run the same number of iterations (heads is padded up), so the
    // shuffles below are always executed by full warps.
    for (int h0 = 0; h0 < p.heads; h0 += rows_per_iter) {
      const int h = h0 + row_in_blk;
      const bool live = h < p.heads;
      uint4 raws[2];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        raws[j] = make_uint4(0, 0, 0, 0);
        if (live && j < n_here) {
          const uint16_t* src =
              static_cast<const uint16_t*>(t.x) + bb_[j] * t.xs_b + ss_[j] * t.xs_s + h * t.xs_h + part * 8;
          raws[j] = *reinterpret_cast<const uint4*>(src);
        }
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        if (j >= n_here) break;  // uniform over the CTA
        const int b = bb_[j], s = ss_[j];
        const bool r2 = s >= p.range2_start;
        const bool rotate = r2 ? (p.do_rope2[blockIdx.y] != 0) : (t.do_rope && s >= p.rope_seq_start);
        const void* const weight = r2 ? p.weight2[blockIdx.y] : t.weight;
        const void* const bias = r2 ? p.bias2[blockIdx.y] : t.bias;
        float cs[8], sn[8];
        if (rotate) {
          const long long trow =
              (r2 ? (s - p.range2_start + p.rope_row0_2) : (s - p.rope_seq_start + p.rope_row0)) * D + part * 8;
          const float4 c0 = *reinterpret_cast<const float4*>(p.cos_tab + trow);
          const float4 c1 = *reinterpret_cast<const float4*>(p.cos_tab + trow + 4);
          const float4 s0 = *reinterpret_cast<const float4*>(p.sin_tab + trow);
          const float4 s1 = *reinterpret_cast<const float4*>(p.sin_tab + trow + 4);
          cs[0] = c0.x; cs[1] = c0.y; cs[2] = c0.z; cs[3] = c0.w; cs[4] = c1.x; cs[5] = c1.y; cs[6] = c1.z; cs[7] = c1.w;
          sn[0] = s0.x; sn[1] = s0.y; sn[2] = s0.z; sn[3] = s0.w; sn[4] = s1.x; sn[5] = s1.y; sn[6] = s1.z; sn[7] = s1.w;
        }
        const uint4 raw = raws[j];
        const uint16_t* e = reinterpret_cast<const uint16_t*>(&raw);
        float f[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = to_f<FP16>(e[i]);

        if (t.do_norm == 2) {
          // LayerNorm over the head dimension (CogVideoX-style QK norm): fp32 throughout, one rounding,
          // as torch's layer_norm does for 16-bit inputs
          float sum = 0.f;
#pragma unroll
          for (int i = 0; i < 8; ++i) sum += f[i];
#pragma unroll
          for (int off = TPR / 2; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
          const float mean = sum * (1.0f / D);
          float ss = 0.f;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            f[i] -= mean;
            ss = fmaf(f[i], f[i], ss);
          }
#pragma unroll
          for (int off = TPR / 2; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
          const float rstd = rsqrtf(ss * (1.0f / D) + p.eps);
          float w[8], bb[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) w[i] = 1.f, bb[i] = 0.f;
          if (weight != nullptr) {
            const uint4 wraw = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(weight) + part * 8);
            const uint16_t* wp = reinterpret_cast<const uint16_t*>(&wraw);
#pragma unroll
            for (int i = 0; i < 8; ++i) w[i] = to_f<FP16>(wp[i]);
          }
          if (bias != nullptr) {
            const uint4 braw = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(bias) + part * 8);
            const uint16_t* bp = reinterpret_cast<const uint16_t*>(&braw);
#pragma unroll
            for (int i = 0; i < 8; ++i) bb[i] = to_f<FP16>(bp[i]);
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) f[i] = to_f<FP16>(from_f<FP16>(fmaf(f[i] * rstd, w[i], bb[i])));
        } else if (t.do_norm) {
          float ss = 0.f;
#pragma unroll
          for (int i = 0; i < 8; ++i) ss = fmaf(f[i], f[i], ss);
#pragma unroll
          for (int off = TPR / 2; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
          const float rstd = rsqrtf(ss * (1.0f / D) + p.eps);
          if (weight != nullptr) {
            const uint4 wraw = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(weight) + part * 8);
            const uint16_t* w = reinterpret_cast<const uint16_t*>(&wraw);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float y = to_f<FP16>(from_f<FP16>(__fmul_rn(f[i], rstd)));
              f[i] = to_f<FP16>(from_f<FP16>(__fmul_rn(y, to_f<FP16>(w[i]))));
            }
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = to_f<FP16>(from_f<FP16>(__fmul_rn(f[i], rstd)));
          }
        }
        if (rotate) {
#pragma unroll
          for (int i = 0; i < 8; i += 2) {
            const float a = f[i], c = f[i + 1];
            f[i] = __fadd_rn(__fmul_rn(a, cs[i]), __fmul_rn(-c, sn[i]));
            f[i + 1] = __fadd_rn(__fmul_rn(c, cs[i + 1]), __fmul_rn(a, sn[i + 1]));
          }
        }
        if (live) {
          uint4 outv;
          uint16_t* o = reinterpret_cast<uint16_t*>(&outv);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = from_f<FP16>(f[i]);
          const int d_idx = h / heads_per_dst;
          const int hh = h - d_idx * heads_per_dst;
          uint16_t* dst = static_cast<uint16_t*>(t.dst[d_idx]) + b * t.ds_b + (s + t.dst_seq_offset) * t.ds_s +
                          hh * t.ds_h + part * 8;
          *reinterpret_cast<uint4*>(dst) = outv;
        }
      }
    }
  }
  if (p.n_signal > 0) {
    // The CTA that finishes last tells every peer that this rank's rows have landed in its buffers: the epoch
    // lives in device memory (a replayed CUDA graph advances it by itself), the ticket goes back to zero for
    // the next launch. Writes of the other threads are ordered before the ticket by the barrier + fence.
    __shared__ unsigned int last;
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();
      const unsigned int total = gridDim.x * gridDim.y;
      last = (atomicAdd(p.ticket, 1u) == total - 1) ? 1u : 0u;
    }
    __syncthreads();
    if (last && threadIdx.x < 32) {
      int32_t epoch = 0;
      if (threadIdx.x == 0) {
        __threadfence_system();
        epoch = *p.epoch_counter + 1;
        *p.epoch_counter = epoch;
        *p.ticket = 0;
      }
      epoch = __shfl_sync(0xffffffffu, epoch, 0);
      if (threadIdx.x < p.n_signal && static_cast<int>(threadIdx.x) != p.signal_me) {
        __threadfence_system();
        nr_st_release_sys(p.signal_slot[threadIdx.x], epoch);
      }
    }
  }
}

}  // namespace
}  // namespace hdit

extern "C" int hdit_qk_norm_rope(const hdit_norm_rope_args* a) {
  using namespace hdit;
  if (a == nullptr) return set_error(HDIT_ERR_BAD_ARG, "args is null");
  if (a->dtype != HDIT_BF16 && a->dtype != HDIT_FP16) return set_error(HDIT_ERR_BAD_ARG, "dtype must be bf16 or fp16");
  if (a->head_dim != 64 && a->head_dim != 128) return set_error(HDIT_ERR_SHAPE, "head_dim must be 64 or 128");
  if (a->n_tensors < 1 || a->n_tensors > kMaxTensors) return set_error(HDIT_ERR_SHAPE, "n_tensors must be 1..3");
  if (a->n_dst < 1 || a->n_dst > kMaxDst || a->heads % a->n_dst != 0)
    return set_error(HDIT_ERR_SHAPE, "heads (%d) must split evenly over n_dst (%d) <= 8", a->heads, a->n_dst);
  if (a->batch < 0 || a->seq < 0 || a->heads <= 0) return set_error(HDIT_ERR_BAD_ARG, "negative size");
  if (static_cast<long long>(a->batch) * a->seq == 0) return HDIT_OK;
  NormRopeParams p;
  memset(&p, 0, sizeof(p));
  bool any_rope = false;
  for (int i = 0; i < a->n_tensors; ++i) {
    const hdit_norm_rope_tensor& s = a->t[i];
    NormRopeTensor& d = p.t[i];
    if (s.x == nullptr) return set_error(HDIT_ERR_BAD_ARG, "tensor %d: x is null", i);
    if ((reinterpret_cast<uintptr_t>(s.x) & 15) || (s.x_stride_b % 8) || (s.x_stride_s % 8) || (s.x_stride_h % 8))
      return set_error(HDIT_ERR_SHAPE, "tensor %d: x must be 16-byte aligned with strides multiple of 8", i);
    if ((s.dst_stride_b % 8) || (s.dst_stride_s % 8) || (s.dst_stride_h % 8))
      return set_error(HDIT_ERR_SHAPE, "tensor %d: dst strides must be multiples of 8", i);
    if (s.norm_weight != nullptr && (reinterpret_cast<uintptr_t>(s.norm_weight) & 15))
      return set_error(HDIT_ERR_SHAPE, "tensor %d: norm weight must be 16-byte aligned", i);
    d.x = s.x;
    d.xs_b = s.x_stride_b;
    d.xs_s = s.x_stride_s;
    d.xs_h = s.x_stride_h;
    d.weight = s.norm_weight;
    d.bias = s.norm_bias;
    if (s.do_norm < 0 || s.do_norm > 2) return set_error(HDIT_ERR_BAD_ARG, "tensor %d: do_norm must be 0, 1 or 2", i);
    if (s.norm_bias != nullptr && (reinterpret_cast<uintptr_t>(s.norm_bias) & 15))
      return set_error(HDIT_ERR_SHAPE, "tensor %d: norm bias must be 16-byte aligned", i);
    d.do_norm = s.do_norm;
    d.do_rope = s.do_rope;
    any_rope |= s.do_rope != 0;
    for (int j = 0; j < a->n_dst; ++j) {
      if (s.dst[j] == nullptr || (reinterpret_cast<uintptr_t>(s.dst[j]) & 15))
        return set_error(HDIT_ERR_BAD_ARG, "tensor %d: dst[%d] null or misaligned", i, j);
      d.dst[j] = s.dst[j];
    }
    d.ds_b = s.dst_stride_b;
    d.ds_s = s.dst_stride_s;
    d.ds_h = s.dst_stride_h;
    d.dst_seq_offset = s.dst_seq_offset;
  }
  if (any_rope) {
    if (a->cos == nullptr || a->sin == nullptr) return set_error(HDIT_ERR_BAD_ARG, "rope requested without cos/sin tables");
    if ((reinterpret_cast<uintptr_t>(a->cos) & 15) || (reinterpret_cast<uintptr_t>(a->sin) & 15))
      return set_error(HDIT_ERR_SHAPE, "cos/sin tables must be 16-byte aligned");
    const long long first_end = (a->range2_start > 0 && a->range2_start < a->seq) ? a->range2_start : a->seq;
    if (a->rope_seq_start < 0 || a->rope_row0 < 0 ||
        (first_end > a->rope_seq_start && a->rope_row0 + (first_end - a->rope_seq_start) > a->rope_rows))
      return set_error(HDIT_ERR_SHAPE, "rope table of %lld rows does not cover tokens [%lld, %d)",
                       (long long)a->rope_rows, (long long)a->rope_seq_start, a->seq);
  }
  p.n_tensors = a->n_tensors;
  p.batch = a->batch;
  p.seq = a->seq;
  p.heads = a->heads;
  p.n_dst = a->n_dst;
  p.eps = a->eps;
  p.cos_tab = a->cos;
  p.sin_tab = a->sin;
  p.rope_seq_start = a->rope_seq_start;
  p.rope_row0 = a->rope_row0;
  p.range2_start = (a->range2_start > 0 && a->range2_start < a->seq) ? a->range2_start : a->seq;
  if (p.range2_start < a->seq) {
    bool rope2 = false;
    for (int i = 0; i < a->n_tensors; ++i) {
      p.weight2[i] = a->range2_norm_weight[i];
      p.bias2[i] = a->range2_norm_bias[i];
      p.do_rope2[i] = a->range2_do_rope[i];
      rope2 |= a->range2_do_rope[i] != 0;
      if ((reinterpret_cast<uintptr_t>(p.weight2[i]) | reinterpret_cast<uintptr_t>(p.bias2[i])) & 15)
        return set_error(HDIT_ERR_SHAPE, "tensor %d: second-range norm weight / bias must be 16-byte aligned", i);
    }
    p.rope_row0_2 = a->range2_rope_row0;
    if (rope2) {
      if (a->cos == nullptr || a->sin == nullptr) return set_error(HDIT_ERR_BAD_ARG, "rope requested without cos/sin tables");
      if (a->range2_rope_row0 < 0 || a->range2_rope_row0 + (a->seq - p.range2_start) > a->rope_rows)
        return set_error(HDIT_ERR_SHAPE, "rope table of %lld rows does not cover the second range", (long long)a->rope_rows);
    }
  }
  if (a->n_signal < 0 || a->n_signal > kMaxDst) return set_error(HDIT_ERR_BAD_ARG, "n_signal must be 0..8");
  if (a->n_signal > 0) {
    if (a->epoch_counter == nullptr || a->ticket == nullptr || a->signal_me < 0 || a->signal_me >= a->n_signal)
      return set_error(HDIT_ERR_BAD_ARG, "signal needs an epoch counter, a ticket word and this rank's index");
    for (int i = 0; i < a->n_signal; ++i) {
      if (i != a->signal_me && a->signal_slots[i] == nullptr)
        return set_error(HDIT_ERR_NOT_INITIALISED, "signal slot of peer %d is null", i);
      p.signal_slot[i] = a->signal_slots[i];
    }
    p.n_signal = a->n_signal;
    p.signal_me = a->signal_me;
    p.epoch_counter = a->epoch_counter;
    p.ticket = reinterpret_cast<unsigned int*>(a->ticket);
  }

  const int tpr = a->head_dim / 8;
  int threads = a->heads * tpr;
  threads = (threads + 31) / 32 * 32;
  if (threads > 512) threads = 512;
  const long long n_tok = static_cast<long long>(a->batch) * a->seq;
  const long long cap = 148LL * HDIT_NR_CTAS_PER_SM;
  const long long want = (n_tok + 1) / 2;  // a CTA takes two tokens per pass
  dim3 grid(static_cast<unsigned>(want < cap ? want : cap), static_cast<unsigned>(a->n_tensors));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(a->stream);
  const bool fp16 = a->dtype == HDIT_FP16;
  if (a->head_dim == 128) {
    if (fp16) norm_rope_kernel<128, true><<<grid, threads, 0, st>>>(p);
    else norm_rope_kernel<128, false><<<grid, threads, 0, st>>>(p);
  } else {
    if (fp16) norm_rope_kernel<64, true><<<grid, threads, 0, st>>>(p);
    else norm_rope_kernel<64, false><<<grid, threads, 0, st>>>(p);
  }
  HDIT_CUDA_OK(cudaGetLastError());
  return HDIT_OK;
}
