// adaLN-Zero glue of the DiT blocks as two HBM-bound kernels:
//   ln_modulate  : out = LayerNorm(x) * (1 + scale[b]) + shift[b]      (no affine, biased variance)
//   gate_residual: out = x + gate[b] * y
// Each replaces a chain of eager kernels (layer_norm, mul, add, add / mul, add) that re-reads and
// re-writes the (B, S, Dm) activation once per link; here every element is read once and written once,
// with fp32 arithmetic in between. One CTA normalises one token row held in registers (16-byte loads,
// consecutive threads on consecutive 16-byte chunks).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "host_common.h"

namespace hdit {
namespace {

constexpr int kLnThreads = 128;
constexpr int kMaxChunks = 8;  // 8-element chunks per thread -> rows of up to 8192 elements

template <bool FP16>
__device__ __forceinline__ float ew_to_f(uint16_t v) {
  if constexpr (FP16) return __half2float(__ushort_as_half(v));
  else return __bfloat162float(__ushort_as_bfloat16(v));
}
template <bool FP16>
__device__ __forceinline__ uint16_t ew_from_f(float f) {
  if constexpr (FP16) return __half_as_ushort(__float2half_rn(f));
  else return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}

// Sum of two values over the CTA with one shared-memory round trip.
__device__ __forceinline__ float2 block_sum2(float a, float b, float2* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    a += __shfl_xor_sync(0xffffffffu, a, o);
    b += __shfl_xor_sync(0xffffffffu, b, o);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // the previous row's readers are done with `red`
  if (lane == 0) red[warp] = make_float2(a, b);
  __syncthreads();
  float2 t = make_float2(0.f, 0.f);
#pragma unroll
  for (int w = 0; w < kLnThreads / 32; ++w) {
    t.x += red[w].x;
    t.y += red[w].y;
  }
  return t;
}

template <bool FP16, int NCH>
__global__ void __launch_bounds__(kLnThreads) ln_modulate_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ shift,
                                                                const uint16_t* __restrict__ scale, uint16_t* __restrict__ out,
                                                                long long rows, int dim, long long rows_per_batch,
                                                                long long x_row_stride, long long out_row_stride,
                                                                long long mod_batch_stride, float eps) {
  __shared__ float2 red[kLnThreads / 32];
  const int n_chunks = dim / 8;
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const long long b = row / rows_per_batch;
    const uint16_t* xr = x + row * x_row_stride;
    uint4 raw[NCH];
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int chunk = threadIdx.x + c * kLnThreads;
      if (chunk < n_chunks) raw[c] = *reinterpret_cast<const uint4*>(xr + chunk * 8);
    }
    float v[NCH][8];
    float s = 0.f, q = 0.f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int chunk = threadIdx.x + c * kLnThreads;
      if (chunk < n_chunks) {
        const uint16_t* e = reinterpret_cast<const uint16_t*>(&raw[c]);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          v[c][i] = ew_to_f<FP16>(e[i]);
          s += v[c][i];
          q = fmaf(v[c][i], v[c][i], q);
        }
      }
    }
    // one reduction for both moments: var = E[x^2] - mean^2 in fp32 (activations here are O(1..100))
    const float2 tot = block_sum2(s, q, red);
    const float mean = tot.x / dim;
    const float rstd = rsqrtf(fmaxf(tot.y / dim - mean * mean, 0.f) + eps);
    uint16_t* orow = out + row * out_row_stride;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int chunk = threadIdx.x + c * kLnThreads;
      if (chunk < n_chunks) {
        const uint4 sh = *reinterpret_cast<const uint4*>(shift + b * mod_batch_stride + chunk * 8);
        const uint4 sc = *reinterpret_cast<const uint4*>(scale + b * mod_batch_stride + chunk * 8);
        const uint16_t* she = reinterpret_cast<const uint16_t*>(&sh);
        const uint16_t* sce = reinterpret_cast<const uint16_t*>(&sc);
        uint4 o;
        uint16_t* oe = reinterpret_cast<uint16_t*>(&o);
#pragma unroll
        for (int i = 0; i < 8; ++i)
          oe[i] = ew_from_f<FP16>(fmaf((v[c][i] - mean) * rstd, 1.0f + ew_to_f<FP16>(sce[i]), ew_to_f<FP16>(she[i])));
        *reinterpret_cast<uint4*>(orow + chunk * 8) = o;
      }
    }
  }
}

// Warp-per-row variant for row lengths that are multiples of 256: a lane keeps its CH 16-byte chunks of the
// row in registers (all loads of a row in flight at once), reductions are warp shuffles only, and a CTA of
// 8 warps walks 8 rows at a time -- no __syncthreads on the critical path.
template <bool FP16, int CH>
__global__ void __launch_bounds__(256) ln_modulate_warp_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ shift,
                                                             const uint16_t* __restrict__ scale, uint16_t* __restrict__ out,
                                                             long long rows, int dim, long long rows_per_batch,
                                                             long long x_row_stride, long long out_row_stride,
                                                             long long mod_batch_stride, float eps) {
  const int lane = threadIdx.x & 31;
  const long long warp_global = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const long long n_warps = static_cast<long long>(gridDim.x) * 8;
  const float inv_dim = 1.0f / dim;
  for (long long row = warp_global; row < rows; row += n_warps) {
    const long long b = row / rows_per_batch;
    const uint16_t* xr = x + row * x_row_stride;
    uint4 raw[CH];
#pragma unroll
    for (int c = 0; c < CH; ++c) raw[c] = *reinterpret_cast<const uint4*>(xr + (c * 32 + lane) * 8);
    float v[CH][8];
    float s = 0.f;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const uint16_t* e = reinterpret_cast<const uint16_t*>(&raw[c]);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        v[c][i] = ew_to_f<FP16>(e[i]);
        s += v[c][i];
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float mean = s * inv_dim;
    float q = 0.f;
#pragma unroll
    for (int c = 0; c < CH; ++c)
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float d = v[c][i] - mean;
        q = fmaf(d, d, q);
      }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
    const float rstd = rsqrtf(q * inv_dim + eps);
    uint16_t* orow = out + row * out_row_stride;
    const uint16_t* shr = shift + b * mod_batch_stride;
    const uint16_t* scr = scale + b * mod_batch_stride;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int off = (c * 32 + lane) * 8;
      const uint4 sh = *reinterpret_cast<const uint4*>(shr + off);
      const uint4 sc = *reinterpret_cast<const uint4*>(scr + off);
      const uint16_t* she = reinterpret_cast<const uint16_t*>(&sh);
      const uint16_t* sce = reinterpret_cast<const uint16_t*>(&sc);
      uint4 o;
      uint16_t* oe = reinterpret_cast<uint16_t*>(&o);
#pragma unroll
      for (int i = 0; i < 8; ++i)
        oe[i] = ew_from_f<FP16>(fmaf((v[c][i] - mean) * rstd, 1.0f + ew_to_f<FP16>(sce[i]), ew_to_f<FP16>(she[i])));
      *reinterpret_cast<uint4*>(orow + off) = o;
    }
  }
}

template <bool FP16, int CH>
void launch_ln_warp(const uint16_t* x, const uint16_t* sh, const uint16_t* sc, uint16_t* out, long long rows, int dim,
                    long long rpb, long long xs, long long os, long long ms, float eps, cudaStream_t st) {
  long long blocks = (rows + 7) / 8;
  if (blocks > 148LL * 8) blocks = 148LL * 8;
  ln_modulate_warp_kernel<FP16, CH><<<static_cast<unsigned>(blocks), 256, 0, st>>>(x, sh, sc, out, rows, dim, rpb, xs, os,
                                                                                 ms, eps);
}

template <bool FP16>
bool try_ln_warp(const uint16_t* x, const uint16_t* sh, const uint16_t* sc, uint16_t* out, long long rows, int dim,
                 long long rpb, long long xs, long long os, long long ms, float eps, cudaStream_t st) {
  if (dim % 256 != 0) return false;
  switch (dim / 256) {
    case 1: launch_ln_warp<FP16, 1>(x, sh, sc, out, rows, dim, rpb, xs, os, ms, eps, st); return true;
    case 2: launch_ln_warp<FP16, 2>(x, sh, sc, out, rows, dim, rpb, xs, os, ms, eps, st); return true;
    case 4: launch_ln_warp<FP16, 4>(x, sh, sc, out, rows, dim, rpb, xs, os, ms, eps, st); return true;
    case 6: launch_ln_warp<FP16, 6>(x, sh, sc, out, rows, dim, rpb, xs, os, ms, eps, st); return true;
    default: return false;
  }
}

template <bool FP16>
__global__ void __launch_bounds__(256) gate_residual_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ gate,
                                                           const uint16_t* __restrict__ y, uint16_t* __restrict__ out,
                                                           long long rows, int dim, long long rows_per_batch,
                                                           long long x_row_stride, long long y_row_stride,
                                                           long long out_row_stride, long long gate_batch_stride) {
  const int chunks_per_row = dim / 8;
  const long long total = rows * chunks_per_row;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    // 32-bit division when the index fits (the host caps rows * dim / 8 there for the common shapes)
    const long long row = (total <= 0xffffffffLL) ? static_cast<long long>(static_cast<unsigned>(i) / static_cast<unsigned>(chunks_per_row))
                                                  : i / chunks_per_row;
    const int chunk = static_cast<int>(i - row * chunks_per_row);
    const long long b = (rows <= 0xffffffffLL && rows_per_batch <= 0xffffffffLL)
                            ? static_cast<long long>(static_cast<unsigned>(row) / static_cast<unsigned>(rows_per_batch))
                            : row / rows_per_batch;
    const uint4 xv = *reinterpret_cast<const uint4*>(x + row * x_row_stride + chunk * 8);
    const uint4 yv = *reinterpret_cast<const uint4*>(y + row * y_row_stride + chunk * 8);
    const uint4 gv = *reinterpret_cast<const uint4*>(gate + b * gate_batch_stride + chunk * 8);
    const uint16_t* xe = reinterpret_cast<const uint16_t*>(&xv);
    const uint16_t* ye = reinterpret_cast<const uint16_t*>(&yv);
    const uint16_t* ge = reinterpret_cast<const uint16_t*>(&gv);
    uint4 o;
    uint16_t* oe = reinterpret_cast<uint16_t*>(&o);
#pragma unroll
    for (int k = 0; k < 8; ++k)
      oe[k] = ew_from_f<FP16>(fmaf(ew_to_f<FP16>(ge[k]), ew_to_f<FP16>(ye[k]), ew_to_f<FP16>(xe[k])));
    *reinterpret_cast<uint4*>(out + row * out_row_stride + chunk * 8) = o;
  }
}

__device__ __forceinline__ float gelu_tanh_f(float x) {
  // 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))), tanh on the MUFU unit
  const float u = 0.7978845608028654f * fmaf(0.044715f * x, x * x, x);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  return 0.5f * x * (1.0f + t);
}

// out[r, :] = gelu_tanh(x[r, :]); rows may be strided on both sides (e.g. the output is a column block of
// a wider buffer). Two 16-byte loads in flight per thread.
template <bool FP16>
__global__ void __launch_bounds__(256) gelu_tanh_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ out,
                                                       long long rows, int dim, long long x_row_stride,
                                                       long long out_row_stride) {
  const unsigned chunks_per_row = static_cast<unsigned>(dim / 8);
  const long long total = rows * chunks_per_row;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total; i += 2 * stride) {
    const long long i1 = i + stride;
    const bool has1 = i1 < total;
    const long long r0 = i / chunks_per_row, r1 = has1 ? i1 / chunks_per_row : 0;
    const long long c0 = i - r0 * chunks_per_row, c1 = has1 ? i1 - r1 * chunks_per_row : 0;
    const uint4 a = *reinterpret_cast<const uint4*>(x + r0 * x_row_stride + c0 * 8);
    uint4 bq = make_uint4(0, 0, 0, 0);
    if (has1) bq = *reinterpret_cast<const uint4*>(x + r1 * x_row_stride + c1 * 8);
    uint4 oa, ob;
    const uint16_t* ae = reinterpret_cast<const uint16_t*>(&a);
    const uint16_t* be = reinterpret_cast<const uint16_t*>(&bq);
    uint16_t* oae = reinterpret_cast<uint16_t*>(&oa);
    uint16_t* obe = reinterpret_cast<uint16_t*>(&ob);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      oae[k] = ew_from_f<FP16>(gelu_tanh_f(ew_to_f<FP16>(ae[k])));
      obe[k] = ew_from_f<FP16>(gelu_tanh_f(ew_to_f<FP16>(be[k])));
    }
    *reinterpret_cast<uint4*>(out + r0 * out_row_stride + c0 * 8) = oa;
    if (has1) *reinterpret_cast<uint4*>(out + r1 * out_row_stride + c1 * 8) = ob;
  }
}

int check_common(int dtype, int64_t rows, int64_t dim, int64_t rows_per_batch) {
  if (dtype != HDIT_BF16 && dtype != HDIT_FP16) return set_error(HDIT_ERR_BAD_ARG, "dtype must be bf16 or fp16");
  if (rows < 0 || dim <= 0 || rows_per_batch <= 0) return set_error(HDIT_ERR_BAD_ARG, "bad sizes");
  if (dim % 8 != 0 || dim > 8 * kLnThreads * kMaxChunks)
    return set_error(HDIT_ERR_SHAPE, "row length must be a multiple of 8 and at most %d", 8 * kLnThreads * kMaxChunks);
  return HDIT_OK;
}

bool misaligned(const void* p, int64_t stride) { return (reinterpret_cast<uintptr_t>(p) & 15) != 0 || stride % 8 != 0; }

}  // namespace
}  // namespace hdit

namespace hdit {
namespace {

// Classifier-free guidance + flow-matching Euler step of a latent patch in one pass, with an optional second
// destination (the next pipeline stage's inbox). Rounding follows the eager sequence it replaces: the guidance
// combine runs in the 16-bit type, one rounding per operation (difference, scaled difference, sum); the step keeps
// the operation order of the reference's scheduler wrapper (prediction * sigma rounded to the 16-bit type; then in
// fp32 denoised = sample - product, derivative = (sample - denoised) / sigma, sample + derivative * dt, each
// operation rounded on its own) and is rounded to the 16-bit type once.
template <bool FP16>
__global__ void __launch_bounds__(256) cfg_euler_step_kernel(const uint16_t* __restrict__ uncond,
                                                            const uint16_t* __restrict__ cond,
                                                            const uint16_t* __restrict__ sample, uint16_t* __restrict__ out,
                                                            uint16_t* __restrict__ out2, long long n_vec, float guidance,
                                                            const float* __restrict__ sigmas, int step) {
  const float sigma = sigmas[step];
  const float dt = __fsub_rn(sigmas[step + 1], sigma);
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec; i += stride) {
    const uint4 u4 = reinterpret_cast<const uint4*>(uncond)[i];
    const uint4 s4 = reinterpret_cast<const uint4*>(sample)[i];
    uint4 c4 = u4;
    if (cond != nullptr) c4 = reinterpret_cast<const uint4*>(cond)[i];
    const uint16_t* u = reinterpret_cast<const uint16_t*>(&u4);
    const uint16_t* c = reinterpret_cast<const uint16_t*>(&c4);
    const uint16_t* sm = reinterpret_cast<const uint16_t*>(&s4);
    uint4 o4;
    uint16_t* o = reinterpret_cast<uint16_t*>(&o4);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float pred = ew_to_f<FP16>(u[k]);
      if (cond != nullptr) {
        const float d = ew_to_f<FP16>(ew_from_f<FP16>(ew_to_f<FP16>(c[k]) - pred));
        const float m = ew_to_f<FP16>(ew_from_f<FP16>(guidance * d));
        pred = ew_to_f<FP16>(ew_from_f<FP16>(pred + m));
      }
      const float x = ew_to_f<FP16>(sm[k]);
      const float product = ew_to_f<FP16>(ew_from_f<FP16>(__fmul_rn(pred, sigma)));
      const float denoised = __fsub_rn(x, product);
      const float derivative = __fdiv_rn(__fsub_rn(x, denoised), sigma);
      o[k] = ew_from_f<FP16>(__fadd_rn(x, __fmul_rn(derivative, dt)));
    }
    reinterpret_cast<uint4*>(out)[i] = o4;
    if (out2 != nullptr) reinterpret_cast<uint4*>(out2)[i] = o4;
  }
}

}  // namespace
}  // namespace hdit

extern "C" int hdit_cfg_euler_step(int32_t dtype, const void* uncond, const void* cond, const void* sample, void* out,
                                   void* out_peer, int64_t n_elems, float guidance_scale, const float* sigmas,
                                   int32_t step_index, void* stream) {
  using namespace hdit;
  if (dtype != HDIT_BF16 && dtype != HDIT_FP16) return set_error(HDIT_ERR_BAD_ARG, "dtype must be bf16 or fp16");
  if (uncond == nullptr || sample == nullptr || out == nullptr || sigmas == nullptr || n_elems < 0 || step_index < 0)
    return set_error(HDIT_ERR_BAD_ARG, "null pointer or negative size");
  if (n_elems == 0) return HDIT_OK;
  const uintptr_t bits = reinterpret_cast<uintptr_t>(uncond) | reinterpret_cast<uintptr_t>(cond) |
                         reinterpret_cast<uintptr_t>(sample) | reinterpret_cast<uintptr_t>(out) |
                         reinterpret_cast<uintptr_t>(out_peer);
  if ((bits & 15) != 0 || n_elems % 8 != 0)
    return set_error(HDIT_ERR_SHAPE, "pointers must be 16-byte aligned and n_elems a multiple of 8");
  const long long n_vec = n_elems / 8;
  long long blocks = (n_vec + 255) / 256;
  if (blocks > 148LL * 8) blocks = 148LL * 8;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == HDIT_FP16)
    cfg_euler_step_kernel<true><<<static_cast<unsigned>(blocks), 256, 0, st>>>(
        static_cast<const uint16_t*>(uncond), static_cast<const uint16_t*>(cond), static_cast<const uint16_t*>(sample),
        static_cast<uint16_t*>(out), static_cast<uint16_t*>(out_peer), n_vec, guidance_scale, sigmas, step_index);
  else
    cfg_euler_step_kernel<false><<<static_cast<unsigned>(blocks), 256, 0, st>>>(
        static_cast<const uint16_t*>(uncond), static_cast<const uint16_t*>(cond), static_cast<const uint16_t*>(sample),
        static_cast<uint16_t*>(out), static_cast<uint16_t*>(out_peer), n_vec, guidance_scale, sigmas, step_index);
  HDIT_CUDA_OK(cudaGetLastError());
  return HDIT_OK;
}

extern "C" int hdit_ln_modulate(int32_t dtype, const void* x, const void* shift, const void* scale, void* out,
                                int64_t rows, int64_t dim, int64_t rows_per_batch, int64_t x_row_stride,
                                int64_t out_row_stride, int64_t mod_batch_stride, float eps, void* stream) {
  using namespace hdit;
  const int rc = check_common(dtype, rows, dim, rows_per_batch);
  if (rc != HDIT_OK) return rc;
  if (rows == 0) return HDIT_OK;
  if (x == nullptr || shift == nullptr || scale == nullptr || out == nullptr) return set_error(HDIT_ERR_BAD_ARG, "null pointer");
  if (misaligned(x, x_row_stride) || misaligned(out, out_row_stride) || misaligned(shift, mod_batch_stride) ||
      misaligned(scale, mod_batch_stride))
    return set_error(HDIT_ERR_SHAPE, "pointers must be 16-byte aligned and strides multiples of 8 elements");
  const unsigned grid = static_cast<unsigned>(rows < 148LL * 16 ? rows : 148LL * 16);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  auto xp = static_cast<const uint16_t*>(x);
  auto sh = static_cast<const uint16_t*>(shift);
  auto sc = static_cast<const uint16_t*>(scale);
  auto op = static_cast<uint16_t*>(out);
  const bool fast = (dtype == HDIT_FP16)
                        ? try_ln_warp<true>(xp, sh, sc, op, rows, static_cast<int>(dim), rows_per_batch, x_row_stride,
                                            out_row_stride, mod_batch_stride, eps, st)
                        : try_ln_warp<false>(xp, sh, sc, op, rows, static_cast<int>(dim), rows_per_batch, x_row_stride,
                                             out_row_stride, mod_batch_stride, eps, st);
  if (fast) {
    HDIT_CUDA_OK(cudaGetLastError());
    return HDIT_OK;
  }
  const int nch = static_cast<int>((dim / 8 + kLnThreads - 1) / kLnThreads);
  const int d = static_cast<int>(dim);
#define HDIT_LN_CASE(N)                                                                                          \
  case N:                                                                                                        \
    if (dtype == HDIT_FP16)                                                                                      \
      ln_modulate_kernel<true, N><<<grid, kLnThreads, 0, st>>>(xp, sh, sc, op, rows, d, rows_per_batch,          \
                                                               x_row_stride, out_row_stride, mod_batch_stride, eps); \
    else                                                                                                         \
      ln_modulate_kernel<false, N><<<grid, kLnThreads, 0, st>>>(xp, sh, sc, op, rows, d, rows_per_batch,         \
                                                                x_row_stride, out_row_stride, mod_batch_stride, eps); \
    break;
  switch (nch) {
    HDIT_LN_CASE(1) HDIT_LN_CASE(2) HDIT_LN_CASE(3) HDIT_LN_CASE(4) HDIT_LN_CASE(5) HDIT_LN_CASE(6) HDIT_LN_CASE(7)
    HDIT_LN_CASE(8)
    default: return set_error(HDIT_ERR_SHAPE, "row too long");
  }
#undef HDIT_LN_CASE
  HDIT_CUDA_OK(cudaGetLastError());
  return HDIT_OK;
}

extern "C" int hdit_gate_residual(int32_t dtype, const void* x, const void* gate, const void* y, void* out, int64_t rows,
                                  int64_t dim, int64_t rows_per_batch, int64_t x_row_stride, int64_t y_row_stride,
                                  int64_t out_row_stride, int64_t gate_batch_stride, void* stream) {
  using namespace hdit;
  const int rc = check_common(dtype, rows, dim, rows_per_batch);
  if (rc != HDIT_OK) return rc;
  if (rows == 0) return HDIT_OK;
  if (x == nullptr || gate == nullptr || y == nullptr || out == nullptr) return set_error(HDIT_ERR_BAD_ARG, "null pointer");
  if (misaligned(x, x_row_stride) || misaligned(y, y_row_stride) || misaligned(out, out_row_stride) ||
      misaligned(gate, gate_batch_stride))
    return set_error(HDIT_ERR_SHAPE, "pointers must be 16-byte aligned and strides multiples of 8 elements");
  const long long total = rows * (dim / 8);
  long long blocks = (total + 255) / 256;
  if (blocks > 148LL * 16) blocks = 148LL * 16;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  auto xp = static_cast<const uint16_t*>(x);
  auto gp = static_cast<const uint16_t*>(gate);
  auto yp = static_cast<const uint16_t*>(y);
  auto op = static_cast<uint16_t*>(out);
  if (dtype == HDIT_FP16)
    gate_residual_kernel<true><<<static_cast<unsigned>(blocks), 256, 0, st>>>(
        xp, gp, yp, op, rows, static_cast<int>(dim), rows_per_batch, x_row_stride, y_row_stride, out_row_stride,
        gate_batch_stride);
  else
    gate_residual_kernel<false><<<static_cast<unsigned>(blocks), 256, 0, st>>>(
        xp, gp, yp, op, rows, static_cast<int>(dim), rows_per_batch, x_row_stride, y_row_stride, out_row_stride,
        gate_batch_stride);
  HDIT_CUDA_OK(cudaGetLastError());
  return HDIT_OK;
}

extern "C" int hdit_gelu_tanh(int32_t dtype, const void* x, void* out, int64_t rows, int64_t dim, int64_t x_row_stride,
                              int64_t out_row_stride, void* stream) {
  using namespace hdit;
  if (dtype != HDIT_BF16 && dtype != HDIT_FP16) return set_error(HDIT_ERR_BAD_ARG, "dtype must be bf16 or fp16");
  if (rows < 0 || dim <= 0 || dim % 8 != 0) return set_error(HDIT_ERR_SHAPE, "row length must be a positive multiple of 8");
  if (rows == 0) return HDIT_OK;
  if (x == nullptr || out == nullptr) return set_error(HDIT_ERR_BAD_ARG, "null pointer");
  if (misaligned(x, x_row_stride) || misaligned(out, out_row_stride))
    return set_error(HDIT_ERR_SHAPE, "pointers must be 16-byte aligned and strides multiples of 8 elements");
  const long long total = rows * (dim / 8);
  long long blocks = (total + 511) / 512;
  if (blocks > 148LL * 16) blocks = 148LL * 16;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == HDIT_FP16)
    gelu_tanh_kernel<true><<<static_cast<unsigned>(blocks), 256, 0, st>>>(
        static_cast<const uint16_t*>(x), static_cast<uint16_t*>(out), rows, static_cast<int>(dim), x_row_stride,
        out_row_stride);
  else
    gelu_tanh_kernel<false><<<static_cast<unsigned>(blocks), 256, 0, st>>>(
        static_cast<const uint16_t*>(x), static_cast<uint16_t*>(out), rows, static_cast<int>(dim), x_row_stride,
        out_row_stride);
  HDIT_CUDA_OK(cudaGetLastError());
  return HDIT_OK;
}
