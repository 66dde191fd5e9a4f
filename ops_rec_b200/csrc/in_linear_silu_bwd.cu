// in_linear_silu backward: gradients of  (user, value, query, key) = split(silu(x . weight^T + bias))  with respect
// to x, weight and bias, given the forward's saved linear_output.
//
// Reference operator ops_rec::in_linear_silu_backward
// (ascendc/activation/in_linear_silu/torch_extension/in_linear_silu_backward_plugin.cpp:118-152; definition of the
// result in in_linear_silu_backward/test/pytest/test_in_linear_silu_backward.py:125-171):
//     g   = cat(user_grad, value_grad, query_grad, key_grad)                    [m, n]
//     dL  = g * sig * (1 + lo * (1 - sig)),  sig = sigmoid(lo), lo = linear_output      fp32
//     bias_grad = column sums of dL (fp32);  dL is then rounded to the element type
//     x_grad = dL . weight  [m, k];   weight_grad = dL^T . x  [n, k]            fp32 accumulation, one rounding
//
// Three HBM-bound passes and two tensor-core products:
//   silu_grad_kernel   one read of g and linear_output -> dL [m, n] and its transpose dLT [n, m'] (through a shared-
//                      memory tile, so both are written with 16-byte stores) + per-row-block column sums of dL
//   transpose16_kernel weight -> weight^T [k, n], x -> x^T [k, m']  (m' = m rounded up to 8: TMA wants 16-byte pitches)
//   colsum_kernel      the row-block sums -> bias_grad, in a fixed order (bitwise reproducible; no atomics)
//   launch_gemm_abt    x_grad = dL . (weight^T)^T and weight_grad = dLT . (x^T)^T on the forward's tcgen05 pipeline
//                      (both operands K-major, which is why the transposes are materialised)
// All intermediates live in the caller's workspace.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "hstu_common.cuh"

namespace hstu {

cudaError_t launch_gemm_abt(const void* a, long long rows_a, long long lda, const void* b, int rows_b, long long ldb,
                            long long kdim, void* out, int dtype, uint32_t* status, cudaStream_t stream);

namespace {

constexpr int kBt = 64;          // tile edge of the element-wise and transpose passes
constexpr int kBtThreads = 256;

template <typename T> struct Cvt;
template <> struct Cvt<__nv_bfloat16> {
  static __device__ __forceinline__ float2 up(uint32_t u) { return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u)); }
  static __device__ __forceinline__ uint32_t down(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ float round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
};
template <> struct Cvt<__half> {
  static __device__ __forceinline__ float2 up(uint32_t u) { return __half22float2(*reinterpret_cast<__half2*>(&u)); }
  static __device__ __forceinline__ uint32_t down(float a, float b) {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ float round(float x) { return __half2float(__float2half_rn(x)); }
};

struct SiluGradParams {
  const void* grad[4];     // user / value / query / key gradients, [m, width[i]]
  int width[4], start[5];  // column range of each in the concatenated [m, n]
  const void* lo;          // linear_output [m, n]
  void* dl;                // [m, n]
  void* dlt;               // [n, ldm]
  float* partial;          // [ceil(m / 64), n] column sums per row block
  long long m, ldm;
  int n;
};

// One 64 x 64 tile of [m, n] per CTA; a thread owns two 8-column pieces (one row each) of it.
template <typename T>
__global__ void __launch_bounds__(kBtThreads) silu_grad_kernel(const SiluGradParams p) {
  __shared__ unsigned short s_t[kBt][kBt + 8];   // the tile of dL in the element type, for the transposed store
  const int tid = threadIdx.x;
  const int c0 = blockIdx.x * kBt;
  const long long r0 = static_cast<long long>(blockIdx.y) * kBt;
  const int piece = tid & 7;                     // columns c0 + 8 piece ..
  const int col = c0 + piece * 8;
  float csum[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int lr = (tid >> 3) + half * 32;       // row inside the tile
    const long long row = r0 + lr;
    uint4 out = make_uint4(0, 0, 0, 0);
    if (row < p.m && col < p.n) {
      const int which = (col >= p.start[1]) + (col >= p.start[2]) + (col >= p.start[3]);
      const T* g = static_cast<const T*>(which == 0 ? p.grad[0] : which == 1 ? p.grad[1] : which == 2 ? p.grad[2] : p.grad[3]);
      const int w = which == 0 ? p.width[0] : which == 1 ? p.width[1] : which == 2 ? p.width[2] : p.width[3];
      const int st = which == 0 ? p.start[0] : which == 1 ? p.start[1] : which == 2 ? p.start[2] : p.start[3];
      const uint4 gv = *reinterpret_cast<const uint4*>(g + row * w + (col - st));
      const uint4 lv = *reinterpret_cast<const uint4*>(static_cast<const T*>(p.lo) + row * p.n + col);
      const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, lw[4] = {lv.x, lv.y, lv.z, lv.w};
      uint32_t ow[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 g2 = Cvt<T>::up(gw[e]), l2 = Cvt<T>::up(lw[e]);
        const float s0 = 1.f / (1.f + __expf(-l2.x)), s1 = 1.f / (1.f + __expf(-l2.y));
        const float d0 = g2.x * (s0 * (1.f + l2.x * (1.f - s0))), d1 = g2.y * (s1 * (1.f + l2.y * (1.f - s1)));
        csum[2 * e] += d0;
        csum[2 * e + 1] += d1;
        ow[e] = Cvt<T>::down(d0, d1);
      }
      out = make_uint4(ow[0], ow[1], ow[2], ow[3]);
      *reinterpret_cast<uint4*>(static_cast<T*>(p.dl) + row * p.n + col) = out;
    }
    *reinterpret_cast<uint4*>(&s_t[lr][piece * 8]) = out;
  }
  // column sums: the 8 lanes that share `piece` across a warp's 4 rows, then the warps of a quarter ... kept simple and
  // deterministic: every thread adds its two rows, rows are combined through shared memory in a fixed order
  __shared__ float s_part[32][kBt];
#pragma unroll
  for (int e = 0; e < 8; ++e) s_part[tid >> 3][piece * 8 + e] = csum[e];
  __syncthreads();
  if (tid < kBt) {
    float acc = 0.f;
#pragma unroll 8
    for (int r = 0; r < 32; ++r) acc += s_part[r][tid];
    if (c0 + tid < p.n) p.partial[static_cast<long long>(blockIdx.y) * p.n + c0 + tid] = acc;
  }
  // transposed store: dLT[c][r0 .. r0 + 64) for the 64 columns of the tile, 16 bytes (8 rows) per store
  for (int i = tid; i < kBt * (kBt / 8); i += kBtThreads) {
    const int c = i >> 3, rp = (i & 7) * 8;
    if (c0 + c >= p.n || r0 + rp >= p.ldm) continue;
    uint32_t w4[4];
#pragma unroll
    for (int e = 0; e < 4; ++e)
      w4[e] = static_cast<uint32_t>(s_t[rp + 2 * e][c]) | (static_cast<uint32_t>(s_t[rp + 2 * e + 1][c]) << 16);
    *reinterpret_cast<uint4*>(static_cast<T*>(p.dlt) + static_cast<long long>(c0 + c) * p.ldm + r0 + rp) =
        make_uint4(w4[0], w4[1], w4[2], w4[3]);
  }
}

// dst [cols, ld_dst] = src [rows, cols]^T for 16-bit elements (cols a multiple of 8, ld_dst a multiple of 8 >= rows).
__global__ void __launch_bounds__(kBtThreads) transpose16_kernel(const unsigned short* __restrict__ src,
                                                                  unsigned short* __restrict__ dst, long long rows,
                                                                  int cols, long long ld_dst) {
  __shared__ unsigned short s_t[kBt][kBt + 8];
  const int tid = threadIdx.x;
  const int c0 = blockIdx.x * kBt;
  const long long r0 = static_cast<long long>(blockIdx.y) * kBt;
  for (int i = tid; i < kBt * (kBt / 8); i += kBtThreads) {
    const int lr = i >> 3, piece = i & 7;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r0 + lr < rows && c0 + piece * 8 < cols)
      v = *reinterpret_cast<const uint4*>(src + (r0 + lr) * cols + c0 + piece * 8);
    *reinterpret_cast<uint4*>(&s_t[lr][piece * 8]) = v;
  }
  __syncthreads();
  for (int i = tid; i < kBt * (kBt / 8); i += kBtThreads) {
    const int c = i >> 3, rp = (i & 7) * 8;
    if (c0 + c >= cols || r0 + rp >= ld_dst) continue;
    uint32_t w4[4];
#pragma unroll
    for (int e = 0; e < 4; ++e)
      w4[e] = static_cast<uint32_t>(s_t[rp + 2 * e][c]) | (static_cast<uint32_t>(s_t[rp + 2 * e + 1][c]) << 16);
    *reinterpret_cast<uint4*>(dst + static_cast<long long>(c0 + c) * ld_dst + r0 + rp) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
  }
}

// bias_grad[c] = sum over the row blocks, in block order
__global__ void colsum_kernel(const float* __restrict__ partial, float* __restrict__ out, long long blocks, int n) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= n) return;
  float acc = 0.f;
  for (long long b = 0; b < blocks; ++b) acc += partial[b * n + c];
  out[c] = acc;
}

inline uint64_t up256(uint64_t x) { return (x + 255) & ~static_cast<uint64_t>(255); }

}  // namespace

// Workspace bytes of the backward for an [m, k] x, [n, k] weight.
uint64_t in_linear_silu_bwd_workspace(long long m, int n, int k) {
  const uint64_t ldm = static_cast<uint64_t>((m + 7) / 8 * 8);
  return up256(static_cast<uint64_t>(m) * n * 2) + up256(static_cast<uint64_t>(n) * ldm * 2) +
         up256(static_cast<uint64_t>(k) * n * 2) + up256(static_cast<uint64_t>(k) * ldm * 2) +
         up256(static_cast<uint64_t>((m + kBt - 1) / kBt) * n * 4);
}

// grads: the four output gradients; lo: linear_output; every tensor 16-byte aligned; bias_grad fp32 [n] or null.
cudaError_t launch_in_linear_silu_bwd(const LinSiluParams& shape, const void* x, const void* weight,
                                      const void* const grads[4], const void* lo, void* x_grad, void* weight_grad,
                                      float* bias_grad, void* workspace, int dtype, uint32_t* status,
                                      cudaStream_t stream) {
  const long long m = shape.m;
  const int n = shape.n, k = shape.k;
  if (m == 0) return cudaSuccess;
  const long long ldm = (m + 7) / 8 * 8;
  char* ws = static_cast<char*>(workspace);
  void* dl = ws;
  ws += up256(static_cast<uint64_t>(m) * n * 2);
  void* dlt = ws;
  ws += up256(static_cast<uint64_t>(n) * ldm * 2);
  void* wt = ws;
  ws += up256(static_cast<uint64_t>(k) * n * 2);
  void* xt = ws;
  ws += up256(static_cast<uint64_t>(k) * ldm * 2);
  float* partial = reinterpret_cast<float*>(ws);
  const long long row_blocks = (m + kBt - 1) / kBt;

  SiluGradParams sp;
  for (int i = 0; i < 4; ++i) {
    sp.grad[i] = grads[i];
    sp.width[i] = shape.width[i];
  }
  for (int i = 0; i < 5; ++i) sp.start[i] = shape.start[i];
  sp.lo = lo;
  sp.dl = dl;
  sp.dlt = dlt;
  sp.partial = partial;
  sp.m = m;
  sp.ldm = ldm;
  sp.n = n;
  const dim3 grid_mn((n + kBt - 1) / kBt, static_cast<unsigned>(row_blocks));
  if (row_blocks > 65535) return cudaErrorInvalidConfiguration;  // m <= 4 194 240 rows per call
  if (dtype == HSTU_DTYPE_BF16)
    silu_grad_kernel<__nv_bfloat16><<<grid_mn, kBtThreads, 0, stream>>>(sp);
  else
    silu_grad_kernel<__half><<<grid_mn, kBtThreads, 0, stream>>>(sp);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  transpose16_kernel<<<dim3((k + kBt - 1) / kBt, (n + kBt - 1) / kBt), kBtThreads, 0, stream>>>(
      static_cast<const unsigned short*>(weight), static_cast<unsigned short*>(wt), n, k, n);
  transpose16_kernel<<<dim3((k + kBt - 1) / kBt, static_cast<unsigned>(row_blocks)), kBtThreads, 0, stream>>>(
      static_cast<const unsigned short*>(x), static_cast<unsigned short*>(xt), m, k, ldm);
  if (bias_grad) colsum_kernel<<<(n + 255) / 256, 256, 0, stream>>>(partial, bias_grad, row_blocks, n);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  // x_grad [m, k] = dL [m, n] . (weight^T [k, n])^T ;  weight_grad [n, k] = dLT [n, m] . (x^T [k, m])^T
  e = launch_gemm_abt(dl, m, n, wt, k, n, n, x_grad, dtype, status, stream);
  if (e != cudaSuccess) return e;
  return launch_gemm_abt(dlt, n, ldm, xt, k, ldm, m, weight_grad, dtype, status, stream);
}

}  // namespace hstu
