// ln_mul: out = (LayerNorm(x) * gamma + beta) * u over the rows of fp32 [A, R] matrices, eps = 1e-5.
//
// The step that consumes the attention output in an HSTU layer (reference operator ops_rec::ln_mul,
// ascendc/activation/ln_mul/torch_extension/ln_mul_plugin.cpp:28-55; arithmetic in
// ascendc/activation/ln_mul/op_kernel/ln_mul_kernel.h:230-300: row sum -> mean, mean of (x - mean)^2 -> variance,
// rstd = 1 / sqrt(var + eps), (x - mean) * rstd * gamma + beta, times u; eps fixed by op_host/ln_mul.cpp:73).
//
// HBM-bound: 12 bytes per element (read x, read u, write out) plus gamma / beta from L2.  Every row is read once:
// it stays in registers between the two reductions (the exact two-pass mean / variance of the reference, no
// E[x^2] - mean^2 shortcut) and the final pass.
//   R <= 1024    one warp per row   (<= 32 values per lane), 8 rows per 256-thread CTA
//   R <= 8192    one CTA per row    (<= 32 values per thread)
//   larger       one CTA per row, three passes over x (the row does not fit the registers)
// Grid-stride over rows with a grid of a few CTAs per SM; loads are 16-byte vectors when R % 4 == 0 and the bases are
// aligned.
#include <cuda_runtime.h>
#include <stdint.h>

namespace hstu {

namespace {

constexpr int kLnThreads = 256;
constexpr int kLnMaxPerThread = 32;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// sum over the CTA; every thread gets the result.  `red` holds one float per warp.
__device__ __forceinline__ float cta_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();   // the previous use of `red` is over
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < kLnThreads / 32 ? red[lane] : 0.f;
  return warp_sum(t);
}

// One row by `kGroup` threads (32 = a warp, kLnThreads = the CTA), values cached in registers.
// kVec: 16-byte accesses (cols % 4 == 0, aligned bases).
template <int kGroup, bool kVec>
__global__ void __launch_bounds__(kLnThreads) ln_mul_rows_kernel(const float* __restrict__ x, const float* __restrict__ u,
                                                                const float* __restrict__ gamma,
                                                                const float* __restrict__ beta, float* __restrict__ out,
                                                                long long rows, int cols, float eps) {
  __shared__ float red[kLnThreads / 32];
  constexpr int kRowsPerCta = kLnThreads / kGroup;
  const int t = threadIdx.x % kGroup;        // position inside the group that owns the row
  const int g = threadIdx.x / kGroup;
  const float inv_n = 1.f / static_cast<float>(cols);
  constexpr int kStep = kVec ? 4 : 1;
  for (long long row = static_cast<long long>(blockIdx.x) * kRowsPerCta + g; row < rows;
       row += static_cast<long long>(gridDim.x) * kRowsPerCta) {
    const float* xr = x + row * cols;
    const float* ur = u + row * cols;
    float* orow = out + row * cols;
    float v[kLnMaxPerThread];
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < kLnMaxPerThread / kStep; ++i) {
      const int c = (i * kGroup + t) * kStep;
      if (kVec) {
        float4 q = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < cols) q = *reinterpret_cast<const float4*>(xr + c);
        v[4 * i] = q.x, v[4 * i + 1] = q.y, v[4 * i + 2] = q.z, v[4 * i + 3] = q.w;
        sum += (q.x + q.y) + (q.z + q.w);
      } else {
        v[i] = c < cols ? xr[c] : 0.f;
        sum += v[i];
      }
    }
    sum = kGroup == 32 ? warp_sum(sum) : cta_sum(sum, red);
    const float mean = sum * inv_n;
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < kLnMaxPerThread / kStep; ++i) {
      const int c = (i * kGroup + t) * kStep;
#pragma unroll
      for (int e = 0; e < kStep; ++e) {
        const float d = v[kStep * i + e] - mean;
        if (c + e < cols) sq = fmaf(d, d, sq);
      }
    }
    sq = kGroup == 32 ? warp_sum(sq) : cta_sum(sq, red);
    const float rstd = 1.f / sqrtf(sq * inv_n + eps);
#pragma unroll
    for (int i = 0; i < kLnMaxPerThread / kStep; ++i) {
      const int c = (i * kGroup + t) * kStep;
      if (c >= cols) continue;
      if (kVec) {
        const float4 uu = *reinterpret_cast<const float4*>(ur + c);
        const float4 gg = __ldg(reinterpret_cast<const float4*>(gamma + c));
        const float4 bb = __ldg(reinterpret_cast<const float4*>(beta + c));
        float4 o;
        o.x = fmaf((v[4 * i] - mean) * rstd, gg.x, bb.x) * uu.x;
        o.y = fmaf((v[4 * i + 1] - mean) * rstd, gg.y, bb.y) * uu.y;
        o.z = fmaf((v[4 * i + 2] - mean) * rstd, gg.z, bb.z) * uu.z;
        o.w = fmaf((v[4 * i + 3] - mean) * rstd, gg.w, bb.w) * uu.w;
        *reinterpret_cast<float4*>(orow + c) = o;
      } else {
        orow[c] = fmaf((v[i] - mean) * rstd, __ldg(gamma + c), __ldg(beta + c)) * ur[c];
      }
    }
  }
}

// Rows longer than the register cache: one CTA per row, x is read three times (the second and third mostly from L2).
__global__ void __launch_bounds__(kLnThreads) ln_mul_long_rows_kernel(const float* __restrict__ x,
                                                                     const float* __restrict__ u,
                                                                     const float* __restrict__ gamma,
                                                                     const float* __restrict__ beta,
                                                                     float* __restrict__ out, long long rows, int cols,
                                                                     float eps) {
  __shared__ float red[kLnThreads / 32];
  const float inv_n = 1.f / static_cast<float>(cols);
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const float* xr = x + row * cols;
    float sum = 0.f;
    for (int c = threadIdx.x; c < cols; c += kLnThreads) sum += xr[c];
    const float mean = cta_sum(sum, red) * inv_n;
    float sq = 0.f;
    for (int c = threadIdx.x; c < cols; c += kLnThreads) {
      const float d = xr[c] - mean;
      sq = fmaf(d, d, sq);
    }
    const float rstd = 1.f / sqrtf(cta_sum(sq, red) * inv_n + eps);
    for (int c = threadIdx.x; c < cols; c += kLnThreads)
      out[row * cols + c] = fmaf((xr[c] - mean) * rstd, __ldg(gamma + c), __ldg(beta + c)) * u[row * cols + c];
  }
}

}  // namespace

cudaError_t launch_ln_mul(const float* x, const float* u, const float* gamma, const float* beta, float* out,
                          long long rows, int cols, float eps, int num_sms, cudaStream_t stream) {
  if (rows == 0 || cols == 0) return cudaSuccess;
  const uintptr_t bases = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(u) |
                          reinterpret_cast<uintptr_t>(gamma) | reinterpret_cast<uintptr_t>(beta) |
                          reinterpret_cast<uintptr_t>(out);
  const bool vec = cols % 4 == 0 && (bases & 15u) == 0;
  const long long max_ctas = static_cast<long long>(num_sms) * 8;
  if (cols <= 32 * kLnMaxPerThread) {
    const long long ctas = (rows + 7) / 8;
    const unsigned grid = static_cast<unsigned>(ctas < max_ctas ? ctas : max_ctas);
    if (vec) ln_mul_rows_kernel<32, true><<<grid, kLnThreads, 0, stream>>>(x, u, gamma, beta, out, rows, cols, eps);
    else ln_mul_rows_kernel<32, false><<<grid, kLnThreads, 0, stream>>>(x, u, gamma, beta, out, rows, cols, eps);
  } else if (cols <= kLnThreads * kLnMaxPerThread) {
    const unsigned grid = static_cast<unsigned>(rows < max_ctas ? rows : max_ctas);
    if (vec) ln_mul_rows_kernel<kLnThreads, true><<<grid, kLnThreads, 0, stream>>>(x, u, gamma, beta, out, rows, cols, eps);
    else ln_mul_rows_kernel<kLnThreads, false><<<grid, kLnThreads, 0, stream>>>(x, u, gamma, beta, out, rows, cols, eps);
  } else {
    const unsigned grid = static_cast<unsigned>(rows < max_ctas ? rows : max_ctas);
    ln_mul_long_rows_kernel<<<grid, kLnThreads, 0, stream>>>(x, u, gamma, beta, out, rows, cols, eps);
  }
  return cudaGetLastError();
}

}  // namespace hstu
