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
bool make_store_map(CUtensorMap* m, void* base, long long rows, long long cols, long long ld, int dtype, int box_cols);

namespace {

constexpr int kLsThreads = 384;
constexpr int kLsTile = 256;                    // tile edge (rows of x and rows of the weight per CTA)
constexpr int kLsStages = 3;
constexpr int kLsChunkBytes = kLsTile * 128;   // 256 rows x 64 16-bit values
constexpr long long kLsWaitLimit = 2000000000ll;

struct LsBars {
  uint64_t full[kLsStages], empty[kLsStages];
  uint64_t acc_full, acc_free;
  uint32_t tmem_base;
  int abort_flag;
  int epi_stop[2];   // the abort flag as the epilogue warps agree to have seen it (per tile parity)
};

template <typename T> struct LsPack;
template <> struct LsPack<__nv_bfloat16> {
  static constexpr int kFormat = 1;
  static __device__ __forceinline__ float round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) {
    return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
  }
  // SiLU in the tanh form, one SFU operation per element: v sigmoid(v) = h (1 + tanh h), h = v / 2.  The error of
  // tanh.approx (2^-11) stays below half a unit in the last place of the bf16 result wherever the result is not tiny.
  static __device__ __forceinline__ uint32_t silu2(float2 v) {
    const float2 h = __fmul2_rn(v, make_float2(0.5f, 0.5f));
    const float2 o = __ffma2_rn(h, make_float2(ptx::tanh_approx(h.x), ptx::tanh_approx(h.y)), h);
    return pack(o.x, o.y);
  }
};
template <> struct LsPack<__half> {
  static constexpr int kFormat = 0;
  static __device__ __forceinline__ float round(float x) { return __half2float(__float2half_rn(x)); }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) { return __half22float2(*reinterpret_cast<const __half2*>(&u)); }
  static __device__ __forceinline__ uint32_t silu2(float2 v) {
    return pack(__fdividef(v.x, 1.f + __expf(-v.x)), __fdividef(v.y, 1.f + __expf(-v.y)));
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

constexpr int kLsStageBytes = 8 * 2 * 2048;   // per epilogue warp: 32 rows x 32 columns of linear_output and of SiLU
constexpr int kLsRingBytes = kLsStages * 2 * kLsChunkBytes;

// kPlain: the bare product  out = x . weight^T  rounded to the element type, written to p.linear ([m, n]) - the two
// matrix products of the backward (in_linear_silu_bwd.cu) run on this same pipeline.
//
// Persistent: one CTA per SM walks the tiles blockIdx.x, blockIdx.x + gridDim.x, ...  The operand ring runs on across
// tiles, so while the epilogue warps turn a tile's accumulators into outputs the producer already fetches the first
// chunks of the next tile; the MMA issuer starts on them as soon as the epilogue has read the last accumulator
// column (acc_free).  Tensor memory holds one tile (2 x 256 columns), so the epilogue itself is not overlapped - but
// its stores are: the results leave through TMA stores from a staging block per warp, so the writes to HBM (1 GB per
// step at m = 65536, n = 4096: with the CTAs in lockstep, synchronous stores ran at the HBM write limit for a third
// of the step) drain while the next main loop runs.
template <typename T, bool kPlain>
__global__ void __launch_bounds__(kLsThreads, 1)
in_linear_silu_kernel(const LinSiluParams p, const __grid_constant__ CUtensorMap tm_x,
                      const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_lin,
                      const __grid_constant__ CUtensorMap tm_o0, const __grid_constant__ CUtensorMap tm_o1,
                      const __grid_constant__ CUtensorMap tm_o2, const __grid_constant__ CUtensorMap tm_o3,
                      const long long tiles) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  LsBars* bars = reinterpret_cast<LsBars*>(base_ptr + kLsRingBytes + kLsStageBytes);
  float* s_bias = reinterpret_cast<float*>(base_ptr + kLsRingBytes + kLsStageBytes + 256);   // [256]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // tiles are numbered with the n tiles of one row block next to each other (so the CTAs that run together share their
  // rows of x; the weight stays in L2)
  const int n_tiles = (p.n + kLsTile - 1) / kLsTile;
  const int chunks = (p.k + 63) / 64;

  if (tid == 0) {
    ptx::prefetch_tensormap(&tm_x);
    ptx::prefetch_tensormap(&tm_w);
    ptx::prefetch_tensormap(&tm_lin);
    if (!kPlain) {
      ptx::prefetch_tensormap(&tm_o0);
      ptx::prefetch_tensormap(&tm_o1);
      ptx::prefetch_tensormap(&tm_o2);
      ptx::prefetch_tensormap(&tm_o3);
    }
    for (int i = 0; i < kLsStages; ++i) {
      ptx::mbar_init(ptx::smem_u32(&bars->full[i]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->empty[i]), 1);
    }
    ptx::mbar_init(ptx::smem_u32(&bars->acc_full), 1);
    ptx::mbar_init(ptx::smem_u32(&bars->acc_free), 8 * 32);   // every epilogue thread
    bars->abort_flag = 0;
    ptx::fence_mbar_init();
  }
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
      uint32_t g = 0;   // chunks requested so far (over all tiles of this CTA)
      for (long long t = blockIdx.x; t < tiles; t += gridDim.x) {
        const int n0 = static_cast<int>(t % n_tiles) * kLsTile;
        const int m0 = static_cast<int>(t / n_tiles) * kLsTile;
        for (int c = 0; c < chunks; ++c, ++g) {
          const uint32_t s = g % kLsStages;
          ls_wait(bars, p.status, ptx::smem_u32(&bars->empty[s]), ((g / kLsStages) & 1u) ^ 1u);
          if (*reinterpret_cast<volatile int*>(&bars->abort_flag)) break;
          const uint32_t full = ptx::smem_u32(&bars->full[s]);
          ptx::mbar_expect_tx(full, 2 * kLsChunkBytes);
          ptx::tma_load_2d(base + s * 2 * kLsChunkBytes, &tm_x, full, c * 64, m0);
          ptx::tma_load_2d(base + s * 2 * kLsChunkBytes + kLsChunkBytes, &tm_w, full, c * 64, n0);
        }
        if (*reinterpret_cast<volatile int*>(&bars->abort_flag)) break;
      }
      // drain (matters only after an abort): the last loads have landed before the CTA exits
      for (uint32_t back = 0; back < kLsStages && back < g; ++back) {
        const uint32_t c = g - 1 - back;
        const uint32_t bar = ptx::smem_u32(&bars->full[c % kLsStages]);
        for (int spin = 0; spin < (1 << 22) && !ptx::mbar_try_wait(bar, (c / kLsStages) & 1u); ++spin) {}
      }
    }
  } else if (warp == 1) {
    // (an elected thread, not `lane == 0`: the compiler then keeps descriptors and barrier addresses in uniform registers)
    if (ptx::elect_one()) {
      constexpr uint32_t idesc = ptx::umma_idesc_f16(LsPack<T>::kFormat, 128, kLsTile, 0);
      constexpr uint64_t kDescK = ptx::umma_desc_sw128_hi(16, 1024);
      uint32_t g = 0, it = 0;
      for (long long t = blockIdx.x; t < tiles; t += gridDim.x, ++it) {
        // the epilogue has read the accumulators of the previous tile
        if (it > 0) ls_wait(bars, p.status, ptx::smem_u32(&bars->acc_free), (it - 1u) & 1u);
        for (int c = 0; c < chunks; ++c, ++g) {
          const uint32_t s = g % kLsStages;
          ls_wait(bars, p.status, ptx::smem_u32(&bars->full[s]), (g / kLsStages) & 1u);
          if (*reinterpret_cast<volatile int*>(&bars->abort_flag)) break;
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
        if (*reinterpret_cast<volatile int*>(&bars->abort_flag)) break;
        ptx::mma_commit(ptx::smem_u32(&bars->acc_full));
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ epilogue (thread = row of the tile)
    // Each warp turns 32 rows x 32 columns at a time: TMEM -> registers -> (+ bias, round, SiLU) -> its staging block
    // -> TMA stores (one 32-column box of linear_output, 64-byte swizzle; the SiLU values as two 16-column boxes,
    // because a split boundary may fall between them).  The TMEM load of the next 32 columns is in flight while the
    // current ones are computed; the staging block is reused once the stores of the previous round have read it.
    const int half = (warp - 4) >> 2;          // which accumulator: rows [128 half, 128 half + 128) of the tile
    const uint32_t lane_base = (static_cast<uint32_t>((warp & 3) * 32) << 16) + half * kLsTile;
    const uint32_t st_lin = base + kLsRingBytes + (warp - 4) * 4096;   // 32 rows x 64 bytes, 64-byte swizzle
    const uint32_t st_act = st_lin + 2048;                            // 2 x (32 rows x 32 bytes)
    const uint32_t swz = (lane >> 1) & 3;      // 64-byte swizzle: 16-byte chunk index ^ address bits [7, 9)
    const int etid = tid - 128;                // 0..255 among the epilogue threads
    uint32_t it = 0;
    for (long long t = blockIdx.x; t < tiles; t += gridDim.x, ++it) {
      const int n0 = static_cast<int>(t % n_tiles) * kLsTile;
      const long long m0 = (t / n_tiles) * kLsTile;
      const int row0 = static_cast<int>(m0) + half * 128 + (warp & 3) * 32;   // first row of this warp
      // The eight warps meet at barriers once per tile, so they must leave the loop together: one thread samples the
      // abort flag before the first barrier, everybody acts on that sample after it.
      if (etid == 0) bars->epi_stop[it & 1u] = *reinterpret_cast<volatile int*>(&bars->abort_flag);
      ptx::named_bar_sync(1, 8 * 32);   // (also: every warp has read the previous tile's bias values)
      if (*reinterpret_cast<volatile int*>(&bars->epi_stop[it & 1u])) break;
      // the bias values of this tile's columns (zeros without a bias / past the last column)
      s_bias[etid] = (!kPlain && p.bias && n0 + etid < p.n) ? p.bias[n0 + etid] : 0.f;
      ptx::named_bar_sync(1, 8 * 32);
      ls_wait(bars, p.status, ptx::smem_u32(&bars->acc_full), it & 1u);
      ptx::tc_fence_after();
      // a wait gave up (status word set) since the sample: the accumulators hold nothing valid - touch nothing, store
      // nothing, and leave at the next tile's barrier
      if (*reinterpret_cast<volatile int*>(&bars->abort_flag)) continue;
      const int nch = (p.n - n0 + 31) / 32 < kLsTile / 32 ? (p.n - n0 + 31) / 32 : kLsTile / 32;   // uniform over the CTA
      uint32_t acc[2][32];
      ptx::tmem_ld32(tmem + lane_base, acc[0]);
#pragma unroll 1
      for (int ch2 = 0; ch2 < kLsTile / 32; ch2 += 2) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int ch = ch2 + u;
          if (ch >= nch) break;
          const int c0 = n0 + ch * 32;
          ptx::tmem_wait_ld_dep(acc[u]);
          if (ch + 1 < nch) {
            ptx::tmem_ld32(tmem + lane_base + (ch + 1) * 32, acc[u ^ 1]);
          } else {
            // the last columns of this tile's accumulators are in registers: the next tile's products may overwrite them
            ptx::tc_fence_before();
            ptx::mbar_arrive(ptx::smem_u32(&bars->acc_free));
          }
          uint32_t lin[16], act[16];
          // packed f32x2 arithmetic; the rounded values come back out of the packed pair (one conversion each way)
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const float2 bb = *reinterpret_cast<const float2*>(&s_bias[ch * 32 + 2 * e]);
            const float2 sum = __fadd2_rn(make_float2(__uint_as_float(acc[u][2 * e]), __uint_as_float(acc[u][2 * e + 1])), bb);
            lin[e] = LsPack<T>::pack(sum.x, sum.y);
            if (!kPlain) act[e] = LsPack<T>::silu2(LsPack<T>::unpack(lin[e]));   // SiLU of the rounded value
          }
          // the stores of the previous round have read the staging block
          if (lane < 3) ptx::bulk_wait_read<0>();   // (lanes 0..2 issue one store each)
          __syncwarp();
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(st_lin + lane * 64 + ((q4 ^ swz) << 4)),
                         "r"(lin[4 * q4]), "r"(lin[4 * q4 + 1]), "r"(lin[4 * q4 + 2]), "r"(lin[4 * q4 + 3])
                         : "memory");
            if (!kPlain)   // columns 0..15 of the chunk in the first block, 16..31 in the second
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(st_act + (q4 >> 1) * 1024 + lane * 32 + (q4 & 1) * 16),
                           "r"(act[4 * q4]), "r"(act[4 * q4 + 1]), "r"(act[4 * q4 + 2]), "r"(act[4 * q4 + 3])
                           : "memory");
          }
          ptx::fence_proxy_async();
          __syncwarp();
          // three lanes issue one store each (an issue costs its thread ~100 cycles); rows and columns past the
          // matrix edge are clipped by the tensor maps
          if (row0 < p.m) {
            if (lane == 0) {
              ptx::tma_store_2d(&tm_lin, st_lin, c0, row0);
              ptx::bulk_commit();
            } else if (!kPlain && lane < 3) {
              const int hf = lane - 1;
              const int cg = c0 + 16 * hf;   // the 16-column group decides the SiLU output tensor (n, splits: multiples of 16)
              if (cg < p.n) {
                const int which = (cg >= p.start[1]) + (cg >= p.start[2]) + (cg >= p.start[3]);
                const CUtensorMap* tm = which == 0 ? &tm_o0 : which == 1 ? &tm_o1 : which == 2 ? &tm_o2 : &tm_o3;
                ptx::tma_store_2d(tm, st_act + hf * 1024, cg - p.start[which], row0);
                ptx::bulk_commit();
              }
            }
          }
        }
      }
    }
    if (lane < 3) ptx::bulk_wait<0>();   // this thread's TMA stores have completed
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, 512);
  }
}

template <typename T, bool kPlain>
cudaError_t launch_t(const LinSiluParams& p, const CUtensorMap& mx, const CUtensorMap& mw, int dtype,
                     cudaStream_t stream) {
  // store maps: linear_output [m, n], and the four SiLU outputs [m, width[i]] (a width of 0: never addressed)
  CUtensorMap ml, mo[4];
  if (!make_store_map(&ml, p.linear, p.m, p.n, p.n, dtype, 32)) return cudaErrorNotSupported;
  for (int i = 0; i < 4; ++i) {
    const bool used = !kPlain && p.width[i] > 0;
    if (!make_store_map(&mo[i], used ? p.out[i] : p.linear, p.m, used ? p.width[i] : p.n, used ? p.width[i] : p.n, dtype,
                        16))
      return cudaErrorNotSupported;
  }
  constexpr int smem = 1024 + kLsRingBytes + kLsStageBytes + 256 + kLsTile * 4;
  static_assert(smem <= 232448, "shared memory budget");
  static_assert(sizeof(LsBars) <= 256, "barrier block too large");
  auto kern = in_linear_silu_kernel<T, kPlain>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  const long long tiles = static_cast<long long>((p.n + kLsTile - 1) / kLsTile) * ((p.m + kLsTile - 1) / kLsTile);
  if ((p.m + kLsTile - 1) / kLsTile > 0x7fffffll) return cudaErrorInvalidConfiguration;   // (TMA row coordinates are int)
  int dev = 0, sms = 0;
  if ((e = cudaGetDevice(&dev)) != cudaSuccess) return e;
  if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
  const unsigned grid = static_cast<unsigned>(tiles < sms ? tiles : sms);
  kern<<<dim3(grid), kLsThreads, smem, stream>>>(p, mx, mw, ml, mo[0], mo[1], mo[2], mo[3], tiles);
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
  return dtype == HSTU_DTYPE_BF16 ? launch_t<__nv_bfloat16, false>(p, mx, mw, dtype, stream)
                                  : launch_t<__half, false>(p, mx, mw, dtype, stream);
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
  return dtype == HSTU_DTYPE_BF16 ? launch_t<__nv_bfloat16, true>(p, ma, mb, dtype, stream)
                                  : launch_t<__half, true>(p, ma, mb, dtype, stream);
}

}  // namespace hstu
