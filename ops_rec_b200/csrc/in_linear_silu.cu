// in_linear_silu forward on Blackwell tensor cores: mixed = x . weight^T + bias;  linear_output = mixed;
// (user, value, query, key) = split(silu(mixed)) - the step that produces the attention's q / k / v in an HSTU layer.
//
// Reference operator ops_rec::distance_in_linear_silu
// (ascendc/activation/in_linear_silu/torch_extension/in_linear_silu_plugin.cpp:36-98; definition of the result in
// in_linear_silu_forward/test/pytest/test_in_linear_silu.py:36-50: addmm in the input type, SiLU of that ROUNDED
// value, split along the last dimension).  x [m, k] and weight [n, k] are bf16 / fp16, bias [n] fp32.
//
// One CTA per 256 x 256 tile of mixed (n-tiles fastest, so the CTAs that run together share their x rows; the weight
// stays in L2).  The tile size is set by the L2 -> shared-memory traffic: a 128 x 128 tile needs 1 byte per 64 FLOPs
// (measured: 531 TFLOP/s, the L2 limit), a 256 x 256 tile half of that.
//   warp 0   TMA producer: 64-wide K chunks of the x tile and the weight tile (both K-major, 256 rows each) into a
//            3-stage ring
//   warp 1   MMA issuer: tcgen05.mma SS, M128 N256 K16, two fp32 accumulators in TMEM (rows 0..127 and 128..255 of
//            the tile, 256 columns each)
//   warp 2   TMEM allocation
//   warps 4-7 / 8-11 epilogue of the first / second accumulator (thread = row): TMEM -> + bias -> round ->
//            linear_output; SiLU of the rounded value -> the output its 16-column group belongs to (the split sizes
//            are multiples of 16)
// Rows / columns / K past the matrix edges are zero-filled by TMA and never stored.  Tensor bound: 2 m n k FLOPs.
// Every mbarrier wait is bounded (then: status bit in the caller's status word, CTA-wide abort flag).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "hstu_common.cuh"
#include "ptx_sm100.cuh"

namespace hstu {

bool make_matrix_map(CUtensorMap* m, const void* base, long long rows, long long cols, int dtype, int box_rows);

namespace {

constexpr int kLsThreads = 384;
constexpr int kLsTile = 256;                    // tile edge (rows of x and rows of the weight per CTA)
constexpr int kLsStages = 3;
constexpr int kLsChunkBytes = kLsTile * 128;   // 256 rows x 64 16-bit values
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

// kPlain: the bare product  out = x . weight^T  rounded to the element type, written to p.linear ([m, n]) - the two
// matrix products of the backward (in_linear_silu_bwd.cu) run on this same pipeline.
template <typename T, bool kPlain>
__global__ void __launch_bounds__(kLsThreads, 1)
in_linear_silu_kernel(const LinSiluParams p, const __grid_constant__ CUtensorMap tm_x,
                      const __grid_constant__ CUtensorMap tm_w) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  LsBars* bars = reinterpret_cast<LsBars*>(base_ptr + kLsStages * 2 * kLsChunkBytes);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // tiles are numbered along the grid's x axis, the n tiles of one row block next to each other (so the CTAs that
  // run together share their rows of x): the row count may be far larger than a grid's y extent allows
  const int n_tiles = (p.n + kLsTile - 1) / kLsTile;
  const int n0 = static_cast<int>(blockIdx.x % n_tiles) * kLsTile;
  const long long m0 = static_cast<long long>(blockIdx.x / n_tiles) * kLsTile;
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
  // the bias values of this tile's columns (zeros without a bias / past the last column), read by every epilogue thread
  float* s_bias = reinterpret_cast<float*>(base_ptr + kLsStages * 2 * kLsChunkBytes + 256);
  if (tid < kLsTile) s_bias[tid] = (!kPlain && p.bias && n0 + tid < p.n) ? p.bias[n0 + tid] : 0.f;
  if (warp == 2) {
    ptx::tmem_alloc(ptx::smem_u32(&bars->tmem_base), 512);
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
    // (an elected thread, not `lane == 0`: the compiler then keeps descriptors and barrier addresses in uniform registers)
    if (ptx::elect_one()) {
      constexpr uint32_t idesc = ptx::umma_idesc_f16(LsPack<T>::kFormat, 128, kLsTile, 0);
      constexpr uint64_t kDescK = ptx::umma_desc_sw128_hi(16, 1024);
      for (int c = 0; c < chunks; ++c) {
        const int s = c % kLsStages;
        ls_wait(bars, p.status, ptx::smem_u32(&bars->full[s]), (c / kLsStages) & 1);
        ptx::tc_fence_after();
        const uint64_t a = kDescK | static_cast<uint64_t>((base + s * 2 * kLsChunkBytes) >> 4);
        const uint64_t b = kDescK | static_cast<uint64_t>((base + s * 2 * kLsChunkBytes + kLsChunkBytes) >> 4);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          const uint64_t off = static_cast<uint64_t>((ks * 32) >> 4);
          const uint32_t acc = (c > 0 || ks > 0) ? 1u : 0u;
          ptx::mma_ss(tmem, a + off, b + off, idesc, acc);                                          // rows 0..127
          ptx::mma_ss(tmem + kLsTile, a + static_cast<uint64_t>((128 * 128) >> 4) + off, b + off, idesc, acc);  // 128..255
        }
        ptx::mma_commit(ptx::smem_u32(&bars->empty[s]));
      }
      ptx::mma_commit(ptx::smem_u32(&bars->acc_full));
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ epilogue (thread = row of the tile)
    // Each warp turns 32 rows x 32 columns at a time: TMEM -> registers -> (+ bias, round, SiLU) -> a private staging
    // block in the (now idle) operand ring -> global, four lanes per row, so that every store instruction writes whole
    // 64-byte row pieces instead of 32 scattered 16-byte ones.
    const int half = (warp - 4) >> 2;          // which accumulator: rows [128 half, 128 half + 128) of the tile
    const uint32_t lane_base = (static_cast<uint32_t>((warp & 3) * 32) << 16) + half * kLsTile;
    const long long row0 = m0 + half * 128 + (warp & 3) * 32;   // first row of this warp
    constexpr int kPitch = 80;                                   // bytes per staged row (64 + 16: fewer bank conflicts)
    uint8_t* stage = base_ptr + (warp - 4) * (2 * 32 * kPitch);  // [lin | silu] x 32 rows
    ls_wait(bars, p.status, ptx::smem_u32(&bars->acc_full), 0);  // all MMAs are done: the ring is free
    ptx::tc_fence_after();
    // a wait gave up (status word set): the accumulators hold nothing valid, store nothing
    const bool give_up = *reinterpret_cast<volatile int*>(&bars->abort_flag) != 0;
    const int sub_row = lane >> 2, part = lane & 3;              // store phase: 8 rows per instruction, 4 lanes per row
#pragma unroll 1
    for (int ch = 0; ch < kLsTile / 32; ++ch) {
      const int c0 = n0 + ch * 32;
      if (c0 >= p.n || give_up) break;   // uniform over the CTA
      uint32_t acc[32];
      ptx::tmem_ld32(tmem + lane_base + ch * 32, acc);
      ptx::tmem_wait_ld();
      uint32_t lin[16], act[16];
#pragma unroll
      for (int e = 0; e < 16; ++e) {
        const float b0 = s_bias[ch * 32 + 2 * e], b1 = s_bias[ch * 32 + 2 * e + 1];
        const float v0 = LsPack<T>::round(__uint_as_float(acc[2 * e]) + b0);
        const float v1 = LsPack<T>::round(__uint_as_float(acc[2 * e + 1]) + b1);
        lin[e] = LsPack<T>::pack(v0, v1);
        // SiLU of the rounded value
        if (!kPlain) act[e] = LsPack<T>::pack(__fdividef(v0, 1.f + __expf(-v0)), __fdividef(v1, 1.f + __expf(-v1)));
      }
      __syncwarp();   // the previous chunk's staged rows have been read
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        *reinterpret_cast<uint4*>(stage + lane * kPitch + q4 * 16) =
            make_uint4(lin[4 * q4], lin[4 * q4 + 1], lin[4 * q4 + 2], lin[4 * q4 + 3]);
        if (!kPlain)
          *reinterpret_cast<uint4*>(stage + 32 * kPitch + lane * kPitch + q4 * 16) =
              make_uint4(act[4 * q4], act[4 * q4 + 1], act[4 * q4 + 2], act[4 * q4 + 3]);
      }
      __syncwarp();
      // this lane's 8 columns: c0 + 8 part .. ; their 16-column group decides the SiLU output tensor
      const int cg = c0 + 16 * (part >> 1);
      const bool col_ok = cg < p.n;   // n is a multiple of 16
      const int which = kPlain ? 0 : (cg >= p.start[1]) + (cg >= p.start[2]) + (cg >= p.start[3]);
      T* obase = static_cast<T*>(which == 0 ? p.out[0] : which == 1 ? p.out[1] : which == 2 ? p.out[2] : p.out[3]);
      const int owidth = which == 0 ? p.width[0] : which == 1 ? p.width[1] : which == 2 ? p.width[2] : p.width[3];
      const int ostart = which == 0 ? p.start[0] : which == 1 ? p.start[1] : which == 2 ? p.start[2] : p.start[3];
#pragma unroll
      for (int it = 0; it < 4; ++it) {
        const int r = it * 8 + sub_row;
        const long long gr = row0 + r;
        if (gr < p.m && col_ok) {
          const uint4 l = *reinterpret_cast<const uint4*>(stage + r * kPitch + part * 16);
          const uint4 a = *reinterpret_cast<const uint4*>(stage + 32 * kPitch + r * kPitch + part * 16);
          *reinterpret_cast<uint4*>(static_cast<T*>(p.linear) + gr * p.n + c0 + part * 8) = l;
          if (!kPlain) *reinterpret_cast<uint4*>(obase + gr * owidth + (cg - ostart) + (part & 1) * 8) = a;
        }
      }
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, 512);
  }
}

template <typename T, bool kPlain>
cudaError_t launch_t(const LinSiluParams& p, const CUtensorMap& mx, const CUtensorMap& mw, cudaStream_t stream) {
  constexpr int smem = 1024 + kLsStages * 2 * kLsChunkBytes + 256 + kLsTile * 4;
  static_assert(sizeof(LsBars) <= 256, "barrier block too large");
  auto kern = in_linear_silu_kernel<T, kPlain>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  const long long tiles = static_cast<long long>((p.n + kLsTile - 1) / kLsTile) * ((p.m + kLsTile - 1) / kLsTile);
  if (tiles > 0x7fffffffll) return cudaErrorInvalidConfiguration;  // (m <= 2^31 - 256 and n <= 32768 never get here)
  kern<<<dim3(static_cast<unsigned>(tiles)), kLsThreads, smem, stream>>>(p, mx, mw);
  return cudaGetLastError();
}

}  // namespace

// Returns cudaSuccess, a CUDA error, or cudaErrorNotSupported when the tensor maps could not be encoded.
cudaError_t launch_in_linear_silu(const LinSiluParams& p, const void* x, const void* weight, int dtype,
                                  cudaStream_t stream) {
  if (p.m == 0) return cudaSuccess;
  CUtensorMap mx, mw;
  if (!make_matrix_map(&mx, x, p.m, p.k, dtype, kLsTile) || !make_matrix_map(&mw, weight, p.n, p.k, dtype, kLsTile))
    return cudaErrorNotSupported;
  return dtype == HSTU_DTYPE_BF16 ? launch_t<__nv_bfloat16, false>(p, mx, mw, stream)
                                  : launch_t<__half, false>(p, mx, mw, stream);
}

bool make_matrix_map_ld(CUtensorMap* m, const void* base, long long rows, long long cols, long long ld, int dtype,
                        int box_rows);

// out [rows_a, rows_b] = a . b^T in the element type (fp32 accumulation, one rounding); a [rows_a, kdim] with row pitch
// lda, b [rows_b, kdim] with row pitch ldb (pitches multiples of 8 elements, bases 16-byte aligned, rows_b a multiple of
// 16, out contiguous).  kdim need not be a multiple of anything: what lies past it reads as zeros.
cudaError_t launch_gemm_abt(const void* a, long long rows_a, long long lda, const void* b, int rows_b, long long ldb,
                            long long kdim, void* out, int dtype, uint32_t* status, cudaStream_t stream) {
  if (rows_a == 0 || rows_b == 0) return cudaSuccess;
  CUtensorMap ma, mb;
  if (!make_matrix_map_ld(&ma, a, rows_a, kdim, lda, dtype, kLsTile) ||
      !make_matrix_map_ld(&mb, b, rows_b, kdim, ldb, dtype, kLsTile))
    return cudaErrorNotSupported;
  LinSiluParams p = {};
  p.linear = out;
  p.m = rows_a;
  p.n = rows_b;
  p.k = static_cast<int>(kdim);
  p.start[4] = rows_b;
  p.status = status;
  return dtype == HSTU_DTYPE_BF16 ? launch_t<__nv_bfloat16, true>(p, ma, mb, stream)
                                  : launch_t<__half, true>(p, ma, mb, stream);
}

}  // namespace hstu
