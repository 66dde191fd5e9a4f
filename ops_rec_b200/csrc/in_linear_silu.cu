// in_linear_silu forward on Blackwell tensor cores: mixed = x . weight^T + bias;  linear_output = mixed;
// (user, value, query, key) = split(silu(mixed)) - the step that produces the attention's q / k / v in an HSTU layer.
//
// Reference operator ops_rec::distance_in_linear_silu
// (ascendc/activation/in_linear_silu/torch_extension/in_linear_silu_plugin.cpp:36-98; definition of the result in
// in_linear_silu_forward/test/pytest/test_in_linear_silu.py:36-50: addmm in the input type, SiLU of that ROUNDED
// value, split along the last dimension).  x [m, k] and weight [n, k] are bf16 / fp16, bias [n] fp32.
//
// One CTA per 128 x 128 tile of mixed (n-tiles fastest, so the CTAs that run together share their x rows; the weight
// stays in L2), two CTAs per SM so that one tile's epilogue overlaps the other's main loop:
//   warp 0   TMA producer: 64-wide K chunks of the x tile and the weight tile (both K-major) into a 3-stage ring
//   warp 1   MMA issuer: tcgen05.mma SS, M128 N128 K16, fp32 accumulator in TMEM (128 columns)
//   warp 2   TMEM allocation
//   warps 4-7 epilogue (thread = row): TMEM -> + bias -> round -> linear_output; SiLU of the rounded value -> the output
//            its 16-column group belongs to (the split sizes are multiples of 16)
// Rows / columns / K past the matrix edges are zero-filled by TMA and never stored.  Tensor bound: 2 m n k FLOPs.
// Every mbarrier wait is bounded (then: status bit in the caller's status word, CTA-wide abort flag).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../../include/hstu_b200.h"
#include "ptx_sm100.cuh"

namespace hstu {

bool make_matrix_map(CUtensorMap* m, const void* base, long long rows, long long cols, int dtype);

struct LinSiluParams {
  const float* bias;       // [n] or null
  void* out[4];            // user, value, query, key: [m, width[i]]
  void* linear;            // [m, n]
  int width[4];
  int start[5];            // first column of each output in mixed; start[4] = n
  long long m;
  int n, k;
  uint32_t* status;        // optional: HSTU_ST_PIPE_TIMEOUT is or-ed into it when a wait gives up
};

namespace {

constexpr int kLsThreads = 256;
constexpr int kLsTile = 128;
constexpr int kLsStages = 3;
constexpr int kLsChunkBytes = kLsTile * 128;   // 128 rows x 64 16-bit values
constexpr long long kLsWaitLimit = 2000000000ll;

struct LsBars {
  uint64_t full[kLsStages], empty[kLsStages];
  uint64_t acc_full;
  uint32_t tmem_base;
  int abort_flag;
};

template <typename T> struct LsPack;
template <> struct LsPack<__nv_bfloat16> {
  static constexpr int kFormat = 1;
  static __device__ __forceinline__ float round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
};
template <> struct LsPack<__half> {
  static constexpr int kFormat = 0;
  static __device__ __forceinline__ float round(float x) { return __half2float(__float2half_rn(x)); }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
};

__device__ __forceinline__ void ls_wait(LsBars* bars, uint32_t* status, uint32_t bar, uint32_t parity) {
  if (ptx::mbar_try_wait(bar, parity)) return;
  if (*reinterpret_cast<volatile int*>(&bars->abort_flag)) return;
  const long long t0 = clock64();
  unsigned spins = 0;
  while (!ptx::mbar_try_wait(bar, parity)) {
    if ((++spins & 0x3ffu) == 0) {
      if (*reinterpret_cast<volatile int*>(&bars->abort_flag)) return;
      if (clock64() - t0 > kLsWaitLimit) {
        *reinterpret_cast<volatile int*>(&bars->abort_flag) = 1;
        if (status) atomicOr(status, static_cast<uint32_t>(HSTU_ST_PIPE_TIMEOUT));
        return;
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kLsThreads, 2)
in_linear_silu_kernel(const LinSiluParams p, const __grid_constant__ CUtensorMap tm_x,
                      const __grid_constant__ CUtensorMap tm_w) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  LsBars* bars = reinterpret_cast<LsBars*>(base_ptr + kLsStages * 2 * kLsChunkBytes);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * kLsTile;
  const long long m0 = static_cast<long long>(blockIdx.y) * kLsTile;
  const int chunks = (p.k + 63) / 64;

  if (tid == 0) {
    ptx::prefetch_tensormap(&tm_x);
    ptx::prefetch_tensormap(&tm_w);
    for (int i = 0; i < kLsStages; ++i) {
      ptx::mbar_init(ptx::smem_u32(&bars->full[i]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->empty[i]), 1);
    }
    ptx::mbar_init(ptx::smem_u32(&bars->acc_full), 1);
    bars->abort_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == 2) {
    ptx::tmem_alloc(ptx::smem_u32(&bars->tmem_base), kLsTile);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);

  if (warp == 0) {
    if (lane == 0) {
      for (int c = 0; c < chunks; ++c) {
        const int s = c % kLsStages;
        ls_wait(bars, p.status, ptx::smem_u32(&bars->empty[s]), ((c / kLsStages) & 1) ^ 1);
        const uint32_t full = ptx::smem_u32(&bars->full[s]);
        ptx::mbar_expect_tx(full, 2 * kLsChunkBytes);
        ptx::tma_load_2d(base + s * 2 * kLsChunkBytes, &tm_x, full, c * 64, static_cast<int>(m0));
        ptx::tma_load_2d(base + s * 2 * kLsChunkBytes + kLsChunkBytes, &tm_w, full, c * 64, n0);
      }
      // drain (matters only after an abort): the last loads have landed before the CTA exits
      for (int back = 0; back < kLsStages && back < chunks; ++back) {
        const int c = chunks - 1 - back;
        const uint32_t bar = ptx::smem_u32(&bars->full[c % kLsStages]);
        for (int spin = 0; spin < (1 << 22) && !ptx::mbar_try_wait(bar, (c / kLsStages) & 1); ++spin) {}
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = ptx::umma_idesc_f16(LsPack<T>::kFormat, kLsTile, kLsTile, 0);
      constexpr uint64_t kDescK = ptx::umma_desc_sw128_hi(16, 1024);
      for (int c = 0; c < chunks; ++c) {
        const int s = c % kLsStages;
        ls_wait(bars, p.status, ptx::smem_u32(&bars->full[s]), (c / kLsStages) & 1);
        ptx::tc_fence_after();
        const uint64_t a = kDescK | static_cast<uint64_t>((base + s * 2 * kLsChunkBytes) >> 4);
        const uint64_t b = kDescK | static_cast<uint64_t>((base + s * 2 * kLsChunkBytes + kLsChunkBytes) >> 4);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          ptx::mma_ss(tmem, a + static_cast<uint64_t>((ks * 32) >> 4), b + static_cast<uint64_t>((ks * 32) >> 4), idesc,
                      (c > 0 || ks > 0) ? 1u : 0u);
        ptx::mma_commit(ptx::smem_u32(&bars->empty[s]));
      }
      ptx::mma_commit(ptx::smem_u32(&bars->acc_full));
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ epilogue (thread = row of the tile)
    const int row = tid - 128;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const long long gr = m0 + row;
    const bool row_ok = gr < p.m;
    ls_wait(bars, p.status, ptx::smem_u32(&bars->acc_full), 0);
    ptx::tc_fence_after();
    T* lin_row = static_cast<T*>(p.linear) + gr * p.n;
#pragma unroll 1
    for (int ch = 0; ch < kLsTile / 32; ++ch) {
      const int c0 = n0 + ch * 32;
      if (c0 >= p.n) break;   // uniform over the CTA
      uint32_t acc[32];
      ptx::tmem_ld32(tmem + lane_base + ch * 32, acc);
      ptx::tmem_wait_ld();
      if (!row_ok) continue;
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        const int cg = c0 + 16 * g;
        if (cg >= p.n) break;   // n is a multiple of 16
        float v[16];
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          float4 bb = make_float4(0.f, 0.f, 0.f, 0.f);
          if (p.bias) bb = __ldg(reinterpret_cast<const float4*>(p.bias + cg) + q4);
          v[4 * q4 + 0] = LsPack<T>::round(__uint_as_float(acc[16 * g + 4 * q4 + 0]) + bb.x);
          v[4 * q4 + 1] = LsPack<T>::round(__uint_as_float(acc[16 * g + 4 * q4 + 1]) + bb.y);
          v[4 * q4 + 2] = LsPack<T>::round(__uint_as_float(acc[16 * g + 4 * q4 + 2]) + bb.z);
          v[4 * q4 + 3] = LsPack<T>::round(__uint_as_float(acc[16 * g + 4 * q4 + 3]) + bb.w);
        }
        uint4* lin = reinterpret_cast<uint4*>(lin_row + cg);
        lin[0] = make_uint4(LsPack<T>::pack(v[0], v[1]), LsPack<T>::pack(v[2], v[3]), LsPack<T>::pack(v[4], v[5]),
                            LsPack<T>::pack(v[6], v[7]));
        lin[1] = make_uint4(LsPack<T>::pack(v[8], v[9]), LsPack<T>::pack(v[10], v[11]), LsPack<T>::pack(v[12], v[13]),
                            LsPack<T>::pack(v[14], v[15]));
        // SiLU of the rounded value, into the output this 16-column group belongs to
        const int which = (cg >= p.start[1]) + (cg >= p.start[2]) + (cg >= p.start[3]);
#pragma unroll
        for (int e = 0; e < 16; ++e) v[e] = v[e] / (1.f + __expf(-v[e]));
        void* obase = which == 0 ? p.out[0] : which == 1 ? p.out[1] : which == 2 ? p.out[2] : p.out[3];
        const int owidth = which == 0 ? p.width[0] : which == 1 ? p.width[1] : which == 2 ? p.width[2] : p.width[3];
        const int ostart = which == 0 ? p.start[0] : which == 1 ? p.start[1] : which == 2 ? p.start[2] : p.start[3];
        uint4* dst = reinterpret_cast<uint4*>(static_cast<T*>(obase) + gr * owidth + (cg - ostart));
        dst[0] = make_uint4(LsPack<T>::pack(v[0], v[1]), LsPack<T>::pack(v[2], v[3]), LsPack<T>::pack(v[4], v[5]),
                            LsPack<T>::pack(v[6], v[7]));
        dst[1] = make_uint4(LsPack<T>::pack(v[8], v[9]), LsPack<T>::pack(v[10], v[11]), LsPack<T>::pack(v[12], v[13]),
                            LsPack<T>::pack(v[14], v[15]));
      }
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, kLsTile);
  }
}

template <typename T>
cudaError_t launch_t(const LinSiluParams& p, const CUtensorMap& mx, const CUtensorMap& mw, cudaStream_t stream) {
  constexpr int smem = 1024 + kLsStages * 2 * kLsChunkBytes + 256;
  static_assert(sizeof(LsBars) <= 256, "barrier block too large");
  auto kern = in_linear_silu_kernel<T>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  dim3 grid((p.n + kLsTile - 1) / kLsTile, static_cast<unsigned>((p.m + kLsTile - 1) / kLsTile), 1);
  kern<<<grid, kLsThreads, smem, stream>>>(p, mx, mw);
  return cudaGetLastError();
}

}  // namespace

// Returns cudaSuccess, a CUDA error, or cudaErrorNotSupported when the tensor maps could not be encoded.
cudaError_t launch_in_linear_silu(const LinSiluParams& p, const void* x, const void* weight, int dtype,
                                  cudaStream_t stream) {
  if (p.m == 0) return cudaSuccess;
  CUtensorMap mx, mw;
  if (!make_matrix_map(&mx, x, p.m, p.k, dtype) || !make_matrix_map(&mw, weight, p.n, p.k, dtype))
    return cudaErrorNotSupported;
  return dtype == HSTU_DTYPE_BF16 ? launch_t<__nv_bfloat16>(p, mx, mw, stream) : launch_t<__half>(p, mx, mw, stream);
}

}  // namespace hstu
