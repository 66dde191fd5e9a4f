// Generic HSTU jagged forward on CUDA cores: fp32 products and fp32 accumulation for every input type.
//
// This is the kernel behind fp32 inputs (the 1e-5 tolerance rules out TF32 tensor cores), behind head dims
// the tcgen05 kernel is not instantiated for, behind dim_qk != dim_v, and behind mask_type = custom.
// One CTA owns a 32-row q-tile of one (sequence, head), walks the K tiles the composite mask leaves visible
// (hstu_dense_forward_jagged_kernel.h:285-289 ends a row at the first fully masked tile; so does this),
// and writes its rows of the jagged output once - no atomics, no zero-initialised output.
//
// Reference arithmetic being reproduced (…/op_kernel/atlas950/hstu_dense_forward_kernel_patten_bsnd.h:258-326,
// regbase_silu.h:21-40): x = alpha * (S + bias); P = x / (1 + exp(-x)) * scale, exactly 0 where masked; P is
// rounded to the input type before P.V; the result is rounded to the input type.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "hstu_common.cuh"

namespace hstu {

namespace {

constexpr int GM = 32;       // q rows per CTA
constexpr int GN = 32;       // keys per tile
constexpr int GTHREADS = 256;
constexpr int GROWS = 4;     // rows per thread (GM / 8 warps)
constexpr int GMAXC = 16;    // dv <= 512 -> at most 16 output columns per thread

template <typename T> __device__ __forceinline__ float to_f(T x);
template <> __device__ __forceinline__ float to_f<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <> __device__ __forceinline__ float to_f<__half>(__half x) { return __half2float(x); }

template <typename T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ __half from_f<__half>(float x) { return __float2half_rn(x); }

template <typename T>
__global__ void __launch_bounds__(GTHREADS) hstu_generic_kernel(const KParams p) {
  extern __shared__ float smem[];
  const int bh = blockIdx.x;
  const int b = bh / p.hq;
  const int h = bh - b * p.hq;
  const int hk = h / p.gqa_ratio;
  const int r0 = blockIdx.y * GM;
  const SeqInfo s = load_seq(p, b);
  if (r0 >= s.lq) return;

  const int dq = p.dqk, dv = p.dv;
  const int ldq = dq + 1;  // +1 float of padding: conflict-free column reads
  float* Qs = smem;                     // [GM][ldq]
  float* Ks = Qs + GM * ldq;            // [GN][ldq]
  float* Vs = Ks + GN * ldq;            // [GN][dv]
  float* Ps = Vs + GN * dv;             // [GM][GN]

  const int tid = threadIdx.x;
  const int tx = tid & 31;
  const int ty = tid >> 5;

  const T* q = static_cast<const T*>(p.q);
  const T* k = static_cast<const T*>(p.k);
  const T* v = static_cast<const T*>(p.v);
  const T* bias = static_cast<const T*>(p.bias);
  const T* cmask = static_cast<const T*>(p.mask);

  for (int idx = tid; idx < GM * dq; idx += GTHREADS) {
    const int r = idx / dq, d = idx - r * dq;
    const int row = r0 + r;
    Qs[r * ldq + d] = row < s.lq ? to_f<T>(q[((s.q0 + row) * p.hq + h) * dq + d]) : 0.f;
  }

  RowBounds rb[GROWS];
#pragma unroll
  for (int r = 0; r < GROWS; ++r) rb[r] = row_bounds(s, r0 + ty * GROWS + r, p.mask_type, p.group);

  float acc[GROWS][GMAXC];
#pragma unroll
  for (int r = 0; r < GROWS; ++r)
#pragma unroll
    for (int c = 0; c < GMAXC; ++c) acc[r][c] = 0.f;

  const int ntiles = kv_tiles_for_rows(s, r0, GM, p.mask_type, GN);
  const int ncol = (dv + 31) >> 5;
  const bool alpha_first = (p.flags & HSTU_FLAG_ALPHA_BEFORE_BIAS) != 0;

  for (int t = 0; t < ntiles; ++t) {
    const int c0 = t * GN;
    __syncthreads();  // previous tile's Ks/Vs/Ps fully consumed (also orders the Qs fill on t == 0)
    for (int idx = tid; idx < GN * dq; idx += GTHREADS) {
      const int r = idx / dq, d = idx - r * dq;
      const int col = c0 + r;
      Ks[r * ldq + d] = col < s.lk ? to_f<T>(k[((s.k0 + col) * p.hk + hk) * dq + d]) : 0.f;
    }
    for (int idx = tid; idx < GN * dv; idx += GTHREADS) {
      const int r = idx / dv, d = idx - r * dv;
      const int col = c0 + r;
      Vs[idx] = col < s.lk ? to_f<T>(v[((s.k0 + col) * p.hk + hk) * dv + d]) : 0.f;
    }
    __syncthreads();

    float sc[GROWS] = {0.f, 0.f, 0.f, 0.f};
    const float* krow = Ks + tx * ldq;
    const float* qrow = Qs + ty * GROWS * ldq;
    for (int d = 0; d < dq; ++d) {
      const float kv = krow[d];
#pragma unroll
      for (int r = 0; r < GROWS; ++r) sc[r] = fmaf(qrow[r * ldq + d], kv, sc[r]);
    }
    const int j = c0 + tx;
#pragma unroll
    for (int r = 0; r < GROWS; ++r) {
      const int i = r0 + ty * GROWS + r;
      float pv = 0.f;
      if (i < s.lq && j < s.lk && allowed(rb[r], j)) {
        float x = sc[r];
        if (bias) {
          const long long boff = static_cast<long long>(b) * p.bias_bstride +
                                 (static_cast<long long>(h) * p.maxq + i) * p.maxk + j;
          const float bv = to_f<T>(bias[boff]);
          x = alpha_first ? fmaf(x, p.alpha, bv) : (x + bv) * p.alpha;
        } else {
          x *= p.alpha;
        }
        pv = x / (1.f + expf(-x)) * p.scale;
        if (p.mask_type == HSTU_MASK_CUSTOM) {
          const long long moff = ((static_cast<long long>(b) * p.hq + h) * p.maxq + i) * p.maxk + j;
          pv *= to_f<T>(cmask[moff]);
        }
        pv = to_f<T>(from_f<T>(pv));
      }
      Ps[(ty * GROWS + r) * GN + tx] = pv;
    }
    __syncthreads();

    const int kend = min(GN, s.lk - c0);
    for (int kk = 0; kk < kend; ++kk) {
      float pr[GROWS];
#pragma unroll
      for (int r = 0; r < GROWS; ++r) pr[r] = Ps[(ty * GROWS + r) * GN + kk];
      const float* vrow = Vs + kk * dv;
#pragma unroll
      for (int c = 0; c < GMAXC; ++c) {
        if (c < ncol) {
          const int col = tx + 32 * c;
          const float vv = col < dv ? vrow[col] : 0.f;
#pragma unroll
          for (int r = 0; r < GROWS; ++r) acc[r][c] = fmaf(pr[r], vv, acc[r][c]);
        }
      }
    }
  }

  T* out = static_cast<T*>(p.out);
#pragma unroll
  for (int r = 0; r < GROWS; ++r) {
    const int i = r0 + ty * GROWS + r;
    if (i >= s.lq) continue;
    T* orow = out + ((s.q0 + i) * p.hq + h) * dv;
#pragma unroll
    for (int c = 0; c < GMAXC; ++c) {
      const int col = tx + 32 * c;
      if (c < ncol && col < dv) orow[col] = from_f<T>(acc[r][c]);
    }
  }
}

size_t generic_smem_bytes(const KParams& p) {
  return sizeof(float) * (static_cast<size_t>(GM + GN) * (p.dqk + 1) + static_cast<size_t>(GN) * p.dv + GM * GN);
}

template <typename T>
cudaError_t launch_t(const KParams& p, cudaStream_t stream) {
  const size_t smem = generic_smem_bytes(p);
  cudaError_t e = cudaFuncSetAttribute(hstu_generic_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem));
  if (e != cudaSuccess) return e;
  dim3 grid(static_cast<unsigned>(p.batch) * p.hq, (p.maxq + GM - 1) / GM, 1);
  hstu_generic_kernel<T><<<grid, GTHREADS, smem, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_generic(const KParams& p, int dtype, cudaStream_t stream) {
  switch (dtype) {
    case HSTU_DTYPE_BF16: return launch_t<__nv_bfloat16>(p, stream);
    case HSTU_DTYPE_FP16: return launch_t<__half>(p, stream);
    default: return launch_t<float>(p, stream);
  }
}

}  // namespace hstu
