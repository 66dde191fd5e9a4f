// HSTU jagged backward on CUDA cores: fp32 products and fp32 accumulation for every input type, any head dims,
// every mask form.  Two kernels, both without atomics (bitwise reproducible):
//
//   hstu_bwd_dq_kernel    one CTA per (sequence, query head, 16-row q-tile): walks the visible K tiles, recomputes
//                         S = Q.K^T and dP = dO.V^T, forms dS, writes that tile of d_bias, accumulates dQ = dS.K.
//                         It also writes the zeros of its d_bias rows outside the visible region, so the caller
//                         need not clear d_bias (the reference adapter clears it with zeros_like,
//                         hstu_v1/torch_extension/hstu_jagged_plugin.cpp:113-118).
//   hstu_bwd_dkv_kernel   one CTA per (sequence, key/value head, 16-key tile): walks the query heads of the group
//                         and the q-tiles that can see the keys, recomputes S and dP, accumulates dV = P^T.dO and
//                         dK = dS^T.Q.
//
// Element-wise stage as in the reference kernel (hstu_backward_v1/op_kernel/vector_score.h:159-209):
//   x = alpha (S + bias);  sg = sigmoid(x) * M;  P = x * sg * scale;  dS = dP * scale * alpha * sg * (1 + x - x sg)
// with P and dS rounded to the input type before the products that consume them; d_bias = dS.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "hstu_common.cuh"

namespace hstu {

namespace {

constexpr int BT = 16;          // tile edge (rows and keys)
constexpr int BTHREADS = 256;   // BT x BT threads
constexpr int BMAXC = 32;       // dims <= 512 -> at most 32 columns per thread

template <typename T> __device__ __forceinline__ float ld_f(const T* p);
template <> __device__ __forceinline__ float ld_f<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ld_f<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <> __device__ __forceinline__ float ld_f<__half>(const __half* p) { return __half2float(*p); }

template <typename T> __device__ __forceinline__ T cvt_f(float x);
template <> __device__ __forceinline__ float cvt_f<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 cvt_f<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ __half cvt_f<__half>(float x) { return __float2half_rn(x); }

template <typename T> __device__ __forceinline__ float round_to(float x) {
  T t = cvt_f<T>(x);
  return ld_f<T>(&t);
}

// rows [r0, r0 + BT) of a [tokens, heads, dim] tensor, head h -> dst[BT][ld] (zeros past `len`)
template <typename T>
__device__ __forceinline__ void load_tile(float* dst, int ld, const T* src, long long tok0, int r0, int len, int heads,
                                          int h, int dim) {
  for (int idx = threadIdx.x; idx < BT * dim; idx += BTHREADS) {
    const int r = idx / dim, d = idx - r * dim;
    const int row = r0 + r;
    dst[r * ld + d] = row < len ? ld_f<T>(src + ((tok0 + row) * heads + h) * dim + d) : 0.f;
  }
}

// P (rounded) and dS (rounded) of element (i, j) from the raw dot products s = q_i.k_j and dp = dO_i.v_j.
// d_bias gets dS for the reference's x = alpha (S + bias) and dX for the alpha-before-bias variant.
template <typename T>
__device__ __forceinline__ void score_grad(const KParams& p, int b, int h, int i, int j, bool visible, float s, float dp,
                                           float* p_out, float* ds_out, float* dbias_out) {
  float pv = 0.f, ds = 0.f, db = 0.f;
  if (visible) {
    const bool alpha_first = (p.flags & HSTU_FLAG_ALPHA_BEFORE_BIAS) != 0;
    float x = s;
    if (p.bias) {
      const long long boff =
          static_cast<long long>(b) * p.bias_bstride + (static_cast<long long>(h) * p.maxq + i) * p.maxk + j;
      const float bv = ld_f<T>(static_cast<const T*>(p.bias) + boff);
      x = alpha_first ? fmaf(x, p.alpha, bv) : (x + bv) * p.alpha;
    } else {
      x *= p.alpha;
    }
    float m = 1.f;
    if (p.mask_type == HSTU_MASK_CUSTOM) {
      const long long moff = ((static_cast<long long>(b) * p.hq + h) * p.maxq + i) * p.maxk + j;
      m = ld_f<T>(static_cast<const T*>(p.mask) + moff);
    }
    const float sg = 1.f / (1.f + expf(-x));
    pv = round_to<T>(x * sg * p.scale * m);
    const float dx = dp * p.scale * m * sg * (1.f + x * (1.f - sg));
    ds = round_to<T>(dx * p.alpha);
    db = alpha_first ? round_to<T>(dx) : ds;
  }
  *p_out = pv;
  *ds_out = ds;
  *dbias_out = db;
}

template <typename T>
__global__ void __launch_bounds__(BTHREADS) hstu_bwd_dq_kernel(const BwdParams bp) {
  extern __shared__ float smem[];
  const KParams& p = bp.f;
  const int bh = blockIdx.x;
  const int b = bh / p.hq;
  const int h = bh - b * p.hq;
  const int hk = h / p.gqa_ratio;
  const int r0 = blockIdx.y * BT;
  const SeqInfo s = load_seq(p, b);
  const int tid = threadIdx.x;
  const int tx = tid & (BT - 1), ty = tid >> 4;
  T* dbias = static_cast<T*>(bp.dbias);
  const long long brow0 = (static_cast<long long>(b) * p.hq + h) * p.maxq;  // first bias row of (b, h)

  const int ntiles = kv_tiles_for_rows(s, r0, BT, p.mask_type, BT);
  if (dbias) {
    // zeros of this CTA's d_bias rows: everything right of the visited tiles (all columns when none is visited)
    const int first = ntiles * BT;
    const int width = p.maxk - first;
    if (width > 0) {
      for (int idx = tid; idx < BT * width; idx += BTHREADS) {
        const int r = idx / width, c = idx - r * width;
        if (r0 + r < p.maxq) dbias[(brow0 + r0 + r) * p.maxk + first + c] = cvt_f<T>(0.f);
      }
    }
  }
  if (ntiles == 0) return;

  const int dq = p.dqk, dv = p.dv;
  const int ldq = dq + 1, ldv = dv + 1;  // +1 float: conflict-free column reads
  float* Qs = smem;               // [BT][ldq]
  float* Gs = Qs + BT * ldq;      // [BT][ldv]   dO rows
  float* Ks = Gs + BT * ldv;      // [BT][ldq]
  float* Vs = Ks + BT * ldq;      // [BT][ldv]
  float* Ds = Vs + BT * ldv;      // [BT][BT]    dS

  load_tile<T>(Qs, ldq, static_cast<const T*>(p.q), s.q0, r0, s.lq, p.hq, h, dq);
  load_tile<T>(Gs, ldv, static_cast<const T*>(bp.dout), s.q0, r0, s.lq, p.hq, h, dv);

  const int i = r0 + ty;
  const RowBounds rb = row_bounds(s, i < s.lq ? i : s.lq - 1, p.mask_type, p.group);
  float acc[BMAXC];
#pragma unroll
  for (int c = 0; c < BMAXC; ++c) acc[c] = 0.f;
  const int ncol = (dq + BT - 1) / BT;

  for (int t = 0; t < ntiles; ++t) {
    const int c0 = t * BT;
    __syncthreads();  // the previous tile's Ks / Vs / Ds are consumed (and, for t == 0, Qs / Gs are filled)
    load_tile<T>(Ks, ldq, static_cast<const T*>(p.k), s.k0, c0, s.lk, p.hk, hk, dq);
    load_tile<T>(Vs, ldv, static_cast<const T*>(p.v), s.k0, c0, s.lk, p.hk, hk, dv);
    __syncthreads();
    float sc = 0.f, dp = 0.f;
    for (int d = 0; d < dq; ++d) sc = fmaf(Qs[ty * ldq + d], Ks[tx * ldq + d], sc);
    for (int d = 0; d < dv; ++d) dp = fmaf(Gs[ty * ldv + d], Vs[tx * ldv + d], dp);
    const int j = c0 + tx;
    const bool visible = i < s.lq && j < s.lk && allowed(rb, j);
    float pv, ds, db;
    score_grad<T>(p, b, h, i, j, visible, sc, dp, &pv, &ds, &db);
    Ds[ty * BT + tx] = ds;
    if (dbias && i < p.maxq && j < p.maxk) dbias[(brow0 + i) * p.maxk + j] = cvt_f<T>(db);
    __syncthreads();
    for (int kk = 0; kk < BT; ++kk) {
      const float d = Ds[ty * BT + kk];
#pragma unroll
      for (int c = 0; c < BMAXC; ++c) {
        if (c < ncol) {
          const int col = tx + BT * c;
          acc[c] = fmaf(d, col < dq ? Ks[kk * ldq + col] : 0.f, acc[c]);
        }
      }
    }
  }
  if (i < s.lq) {
    T* row = static_cast<T*>(bp.dq) + ((s.q0 + i) * p.hq + h) * dq;
#pragma unroll
    for (int c = 0; c < BMAXC; ++c) {
      const int col = tx + BT * c;
      if (c < ncol && col < dq) row[col] = cvt_f<T>(acc[c]);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(BTHREADS) hstu_bwd_dkv_kernel(const BwdParams bp) {
  extern __shared__ float smem[];
  const KParams& p = bp.f;
  const int bh = blockIdx.x;
  const int b = bh / p.hk;
  const int hk = bh - b * p.hk;
  const int c0 = blockIdx.y * BT;
  const SeqInfo s = load_seq(p, b);
  if (c0 >= s.lk) return;
  const int tid = threadIdx.x;
  const int tx = tid & (BT - 1), ty = tid >> 4;

  const int dq = p.dqk, dv = p.dv;
  const int ldq = dq + 1, ldv = dv + 1;
  float* Ks = smem;               // [BT][ldq]
  float* Vs = Ks + BT * ldq;      // [BT][ldv]
  float* Qs = Vs + BT * ldv;      // [BT][ldq]
  float* Gs = Qs + BT * ldq;      // [BT][ldv]
  float* Ps = Gs + BT * ldv;      // [BT][BT]  P  (row = query)
  float* Ds = Ps + BT * BT;       // [BT][BT]  dS (row = query)

  load_tile<T>(Ks, ldq, static_cast<const T*>(p.k), s.k0, c0, s.lk, p.hk, hk, dq);
  load_tile<T>(Vs, ldv, static_cast<const T*>(p.v), s.k0, c0, s.lk, p.hk, hk, dv);

  float acc_k[BMAXC], acc_v[BMAXC];
#pragma unroll
  for (int c = 0; c < BMAXC; ++c) acc_k[c] = acc_v[c] = 0.f;
  const int ncol_k = (dq + BT - 1) / BT, ncol_v = (dv + BT - 1) / BT;
  const int ktile = c0 / BT;
  const int j = c0 + tx;

  for (int hh = 0; hh < p.gqa_ratio; ++hh) {
    const int h = hk * p.gqa_ratio + hh;
    for (int r0 = 0; r0 < s.lq; r0 += BT) {
      if (kv_tiles_for_rows(s, r0, BT, p.mask_type, BT) <= ktile) continue;  // no row of this q-tile sees these keys
      __syncthreads();  // the previous Qs / Gs / Ps / Ds are consumed (and, first time, Ks / Vs are filled)
      load_tile<T>(Qs, ldq, static_cast<const T*>(p.q), s.q0, r0, s.lq, p.hq, h, dq);
      load_tile<T>(Gs, ldv, static_cast<const T*>(bp.dout), s.q0, r0, s.lq, p.hq, h, dv);
      __syncthreads();
      const int i = r0 + ty;
      const RowBounds rb = row_bounds(s, i < s.lq ? i : s.lq - 1, p.mask_type, p.group);
      float sc = 0.f, dp = 0.f;
      for (int d = 0; d < dq; ++d) sc = fmaf(Qs[ty * ldq + d], Ks[tx * ldq + d], sc);
      for (int d = 0; d < dv; ++d) dp = fmaf(Gs[ty * ldv + d], Vs[tx * ldv + d], dp);
      const bool visible = i < s.lq && j < s.lk && allowed(rb, j);
      float pv, ds, db;
      score_grad<T>(p, b, h, i, j, visible, sc, dp, &pv, &ds, &db);
      Ps[ty * BT + tx] = pv;
      Ds[ty * BT + tx] = ds;
      __syncthreads();
      // this thread now owns key `ty` and the columns tx, tx + 16, ...
      for (int ii = 0; ii < BT; ++ii) {
        const float pe = Ps[ii * BT + ty], de = Ds[ii * BT + ty];
#pragma unroll
        for (int c = 0; c < BMAXC; ++c) {
          const int col = tx + BT * c;
          if (c < ncol_v) acc_v[c] = fmaf(pe, col < dv ? Gs[ii * ldv + col] : 0.f, acc_v[c]);
          if (c < ncol_k) acc_k[c] = fmaf(de, col < dq ? Qs[ii * ldq + col] : 0.f, acc_k[c]);
        }
      }
    }
  }
  const int key = c0 + ty;
  if (key < s.lk) {
    T* krow = static_cast<T*>(bp.dk) + ((s.k0 + key) * p.hk + hk) * dq;
    T* vrow = static_cast<T*>(bp.dv) + ((s.k0 + key) * p.hk + hk) * dv;
#pragma unroll
    for (int c = 0; c < BMAXC; ++c) {
      const int col = tx + BT * c;
      if (c < ncol_k && col < dq) krow[col] = cvt_f<T>(acc_k[c]);
      if (c < ncol_v && col < dv) vrow[col] = cvt_f<T>(acc_v[c]);
    }
  }
}

template <typename T>
cudaError_t launch_bwd_t(const BwdParams& bp, cudaStream_t stream) {
  const KParams& p = bp.f;
  const size_t tile = static_cast<size_t>(BT) * (p.dqk + 1) + static_cast<size_t>(BT) * (p.dv + 1);
  const size_t smem_q = sizeof(float) * (2 * tile + BT * BT);
  const size_t smem_kv = sizeof(float) * (2 * tile + 2 * BT * BT);
  cudaError_t e = cudaFuncSetAttribute(hstu_bwd_dq_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem_q));
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(hstu_bwd_dkv_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem_kv));
  if (e != cudaSuccess) return e;
  dim3 grid_q(static_cast<unsigned>(p.batch) * p.hq, (p.maxq + BT - 1) / BT, 1);
  hstu_bwd_dq_kernel<T><<<grid_q, BTHREADS, smem_q, stream>>>(bp);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  dim3 grid_k(static_cast<unsigned>(p.batch) * p.hk, (p.maxk + BT - 1) / BT, 1);
  hstu_bwd_dkv_kernel<T><<<grid_k, BTHREADS, smem_kv, stream>>>(bp);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_bwd_generic(const BwdParams& bp, int dtype, cudaStream_t stream) {
  switch (dtype) {
    case HSTU_DTYPE_BF16: return launch_bwd_t<__nv_bfloat16>(bp, stream);
    case HSTU_DTYPE_FP16: return launch_bwd_t<__half>(bp, stream);
    default: return launch_bwd_t<float>(bp, stream);
  }
}

}  // namespace hstu
