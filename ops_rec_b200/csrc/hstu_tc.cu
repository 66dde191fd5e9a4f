// HSTU jagged attention forward on the sm_100a tensor cores (tcgen05 + TMEM), bf16 / fp16, head dim 64 or 128.
//
// One persistent CTA per SM walks the scheduler's work list.  A work item is a (sequence, head, 256-row q-pair):
// two 128-row Q tiles that share every K/V tile fetched.  Per K tile and Q tile:
//
//     S = Q.K^T            tcgen05.mma, both operands from swizzled shared memory (TMA-filled), fp32 in TMEM
//     P = silu(alpha*(S + bias)) * scale, 0 where masked, rounded to the input type
//                          TMEM -> registers -> TMEM by a 128-thread group; P overwrites S in place
//     O += P.V             tcgen05.mma with P as the TMEM operand, V N-major from shared memory
//
// S and P never leave the SM; O stays in TMEM for the whole row of K tiles (there is no softmax, so no
// rescaling), then goes TMEM -> registers -> 16-byte stores into the jagged [tokens, heads, dim] output.
// Compare the reference kernel, which moves every S tile and every P tile through a global-memory ring
// between its matrix and vector cores and accumulates partial O rows with atomics
// (…/op_kernel/atlas950/hstu_dense_forward_kernel_patten_bsnd.h:156-176, 590-689,
//  hstu_dense_forward_jagged_kernel.h:257-398).
//
// Warp roles (384 threads): warp 0 = TMA producer, warp 1 = MMA issuer, warp 2 = TMEM allocator,
// warps 4-7 = P/O group of Q tile 0, warps 8-11 = P/O group of Q tile 1.
//
// Every wait on an mbarrier is bounded: after ~1 s without progress the waiter raises HSTU_ST_PIPE_TIMEOUT in
// the workspace status word and a CTA-wide abort flag that turns all later waits into no-ops, so the kernel
// always runs to its end, frees its tensor memory and returns (with garbage in `out` and the flag set).
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <mutex>

#include "hstu_common.cuh"
#include "ptx_sm100.cuh"

namespace hstu {

namespace {

constexpr int kThreads = 384;
constexpr int kTmemCols = 512;
constexpr int kColS0 = 0, kColS1 = 128, kColO0 = 256;
constexpr long long kWaitLimitCycles = 2000000000ll;  // ~1 s

template <int D>
struct Cfg {
  static constexpr int kHalves = D / 64;                 // 128-byte swizzle atoms along the head dim
  static constexpr int kHalfBytes = kTileM * 128;        // 128 rows x 128 B
  static constexpr int kTileBytes = kHalves * kHalfBytes;
  static constexpr int kStages = D == 128 ? 4 : 8;       // K/V ring slots (one tile each)
  static constexpr int kQBytes = 2 * kTileBytes;
  static constexpr int kRingBytes = kStages * kTileBytes;
  static constexpr int kBarBytes = 512;
  static constexpr int kSmemBytes = 1024 + kQBytes + kRingBytes + kBarBytes;
  static constexpr int kColO1 = kColO0 + D;
};

struct Barriers {
  uint64_t q_full[2], q_free[2];
  uint64_t s_full[2], p_full[2];
  uint64_t o_full[2], o_free[2];
  uint64_t done;
  uint64_t kv_full[8], kv_free[8];
  uint32_t tmem_base;
  int abort_flag;
};
static_assert(sizeof(Barriers) <= 512, "barrier block too large");

struct Waiter {
  int* abort_flag;
  uint32_t* status;
  __device__ __forceinline__ void wait(uint32_t bar, uint32_t parity) const {
    if (*reinterpret_cast<volatile int*>(abort_flag)) return;
    if (ptx::mbar_try_wait(bar, parity)) return;
    const long long t0 = clock64();
    unsigned spins = 0;
    while (!ptx::mbar_try_wait(bar, parity)) {
      if ((++spins & 0x3ffu) == 0) {
        if (*reinterpret_cast<volatile int*>(abort_flag)) return;
        if (clock64() - t0 > kWaitLimitCycles) {
          *reinterpret_cast<volatile int*>(abort_flag) = 1;
          atomicOr(status, static_cast<uint32_t>(HSTU_ST_PIPE_TIMEOUT));
          return;
        }
      }
    }
  }
};

struct Item {
  SeqInfo s;
  int b, h, hk, r0;
  int n[2];   // K tiles each Q tile visits
  int nmax;
};

__device__ __forceinline__ Item load_item(const KParams& p, long long idx) {
  Item it;
  it.b = static_cast<int>(p.items[2 * idx]);
  const uint32_t hp = p.items[2 * idx + 1];
  it.h = static_cast<int>(hp >> 16);
  it.hk = it.h / p.gqa_ratio;
  it.r0 = static_cast<int>(hp & 0xffffu) * kPairM;
  it.s = load_seq(p, it.b);
  it.n[0] = kv_tiles_for_rows(it.s, it.r0, kTileM, p.mask_type, kTileN);
  it.n[1] = kv_tiles_for_rows(it.s, it.r0 + kTileM, kTileM, p.mask_type, kTileN);
  it.nmax = it.n[0] > it.n[1] ? it.n[0] : it.n[1];
  return it;
}

template <typename T> struct Pack;
template <> struct Pack<__nv_bfloat16> {
  static constexpr int kFormat = 1;
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
  }
  static __device__ __forceinline__ float one(const void* p, long long i) {
    return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  }
};
template <> struct Pack<__half> {
  static constexpr int kFormat = 0;
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) {
    return __half22float2(*reinterpret_cast<__half2*>(&u));
  }
  static __device__ __forceinline__ float one(const void* p, long long i) {
    return __half2float(static_cast<const __half*>(p)[i]);
  }
};

// silu(y) * scale with a = y / 2:  a*scale*(1 + tanh(a))  (one MUFU op per element)
__device__ __forceinline__ float silu_scaled_tanh(float a, float scale) {
  const float r = a * scale;
  return fmaf(r, ptx::tanh_approx(a), r);
}
// silu(y) * scale = y*scale / (1 + 2^(-y*log2 e))  (two MUFU ops, ~1 ulp; used for fp16 inputs)
__device__ __forceinline__ float silu_scaled_exact(float y, float scale) {
  const float e = ptx::ex2_approx(-1.4426950408889634f * y);
  return y * scale * ptx::rcp_approx(1.f + e);
}

template <int D, typename T, bool kBias>
__global__ void __launch_bounds__(kThreads, 1)
hstu_tc_kernel(const KParams p, const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, const int bias_vec_ok) {
  using C = Cfg<D>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  const uint32_t sm_q = base;                    // 2 Q tiles
  const uint32_t sm_ring = base + C::kQBytes;    // K/V ring
  Barriers* bars = reinterpret_cast<Barriers*>(base_ptr + C::kQBytes + C::kRingBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const Waiter w{&bars->abort_flag, p.ws_header};

  if (threadIdx.x == 0) {
    ptx::prefetch_tensormap(&tm_q);
    ptx::prefetch_tensormap(&tm_k);
    ptx::prefetch_tensormap(&tm_v);
    for (int t = 0; t < 2; ++t) {
      ptx::mbar_init(ptx::smem_u32(&bars->q_full[t]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->q_free[t]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->s_full[t]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->p_full[t]), kTileM);
      ptx::mbar_init(ptx::smem_u32(&bars->o_full[t]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->o_free[t]), kTileM);
    }
    ptx::mbar_init(ptx::smem_u32(&bars->done), 1);
    for (int s = 0; s < C::kStages; ++s) {
      ptx::mbar_init(ptx::smem_u32(&bars->kv_full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->kv_free[s]), 1);
    }
    bars->abort_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == 2) {
    ptx::tmem_alloc(ptx::smem_u32(&bars->tmem_base), kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);

  const long long num_items = p.ws_header[1];
  const long long G = gridDim.x;
  const long long cta = blockIdx.x;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t q_uses[2] = {0, 0};
      uint32_t ring_pos = 0;
      long long round = 0;
      for (long long first = 0; first < num_items; first += G, ++round) {
        const long long idx = first + ((round & 1) ? (G - 1 - cta) : cta);
        if (idx >= num_items) continue;
        const Item it = load_item(p, idx);
        for (int t = 0; t < 2; ++t) {
          if (it.n[t] == 0) continue;
          const uint32_t full = ptx::smem_u32(&bars->q_full[t]);
          w.wait(ptx::smem_u32(&bars->q_free[t]), (q_uses[t] & 1u) ^ 1u);
          ptx::mbar_expect_tx(full, C::kTileBytes);
          const int row = static_cast<int>(it.s.q0) + it.r0 + t * kTileM;
#pragma unroll
          for (int hf = 0; hf < C::kHalves; ++hf)
            ptx::tma_load_3d(sm_q + t * C::kTileBytes + hf * C::kHalfBytes, &tm_q, full, hf * 64, it.h, row);
          ++q_uses[t];
        }
        for (int j = 0; j < it.nmax; ++j) {
          const int row = static_cast<int>(it.s.k0) + j * kTileN;
#pragma unroll
          for (int kv = 0; kv < 2; ++kv) {
            const uint32_t stage = ring_pos % C::kStages;
            const uint32_t use = ring_pos / C::kStages;
            const uint32_t full = ptx::smem_u32(&bars->kv_full[stage]);
            w.wait(ptx::smem_u32(&bars->kv_free[stage]), (use & 1u) ^ 1u);
            ptx::mbar_expect_tx(full, C::kTileBytes);
#pragma unroll
            for (int hf = 0; hf < C::kHalves; ++hf)
              ptx::tma_load_3d(sm_ring + stage * C::kTileBytes + hf * C::kHalfBytes, kv == 0 ? &tm_k : &tm_v, full,
                               hf * 64, it.hk, row);
            ++ring_pos;
          }
        }
      }
      // Drain: every load this thread issued must have landed before the CTA may exit (matters only after an
      // abort; otherwise the consumers have already waited for all of them).  Bounded, ignores the abort flag.
      for (int s = 0; s < C::kStages; ++s) {
        if (ring_pos <= static_cast<uint32_t>(s)) continue;
        const uint32_t last_use = (ring_pos - 1 - s) / C::kStages;
        const uint32_t bar = ptx::smem_u32(&bars->kv_full[s]);
        for (int spin = 0; spin < (1 << 22) && !ptx::mbar_try_wait(bar, last_use & 1u); ++spin) {}
      }
      for (int t = 0; t < 2; ++t) {
        if (q_uses[t] == 0) continue;
        const uint32_t bar = ptx::smem_u32(&bars->q_full[t]);
        for (int spin = 0; spin < (1 << 22) && !ptx::mbar_try_wait(bar, (q_uses[t] - 1) & 1u); ++spin) {}
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = ptx::umma_idesc_f16(Pack<T>::kFormat, kTileM, kTileN, 0);
      constexpr uint32_t idesc_pv = ptx::umma_idesc_f16(Pack<T>::kFormat, kTileM, D, 1);
      uint32_t q_uses[2] = {0, 0}, p_uses[2] = {0, 0}, o_uses[2] = {0, 0};
      uint32_t ring_base = 0;
      long long round = 0;
      for (long long first = 0; first < num_items; first += G, ++round) {
        const long long idx = first + ((round & 1) ? (G - 1 - cta) : cta);
        if (idx >= num_items) continue;
        const Item it = load_item(p, idx);
        for (int step = 0; step <= it.nmax; ++step) {
          const uint32_t pos_k = ring_base + 2u * step;            // K(step)
          const uint32_t pos_v = ring_base + 2u * (step - 1) + 1u;  // V(step - 1)
          if (step < it.nmax) w.wait(ptx::smem_u32(&bars->kv_full[pos_k % C::kStages]), (pos_k / C::kStages) & 1u);
          if (step >= 1) w.wait(ptx::smem_u32(&bars->kv_full[pos_v % C::kStages]), (pos_v / C::kStages) & 1u);
          ptx::tc_fence_after();
          const uint32_t sm_k = sm_ring + (pos_k % C::kStages) * C::kTileBytes;
          const uint32_t sm_v = sm_ring + (pos_v % C::kStages) * C::kTileBytes;
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            const uint32_t col_s = tmem + (t == 0 ? kColS0 : kColS1);
            const uint32_t col_o = tmem + (t == 0 ? kColO0 : C::kColO1);
            if (step >= 1 && step - 1 < it.n[t]) {
              // O_t (+)= P_t(step-1) . V(step-1)
              w.wait(ptx::smem_u32(&bars->p_full[t]), p_uses[t] & 1u);
              ++p_uses[t];
              if (step == 1) w.wait(ptx::smem_u32(&bars->o_free[t]), (o_uses[t] & 1u) ^ 1u);
              ptx::tc_fence_after();
#pragma unroll
              for (int ks = 0; ks < kTileN / 16; ++ks) {
                const uint64_t bdesc = ptx::umma_desc_sw128(sm_v + ks * 2048, C::kHalfBytes, 1024);
                ptx::mma_ts(col_o, col_s + ks * 8, bdesc, idesc_pv, (step > 1 || ks > 0) ? 1u : 0u);
              }
              if (step == it.n[t]) {
                ptx::mma_commit(ptx::smem_u32(&bars->o_full[t]));
                ++o_uses[t];
              }
            }
            if (step < it.n[t]) {
              // S_t = Q_t . K(step)^T
              if (step == 0) {
                w.wait(ptx::smem_u32(&bars->q_full[t]), q_uses[t] & 1u);
                ptx::tc_fence_after();
              }
              const uint32_t sm_qt = sm_q + t * C::kTileBytes;
#pragma unroll
              for (int ks = 0; ks < D / 16; ++ks) {
                const uint32_t off = (ks >> 2) * C::kHalfBytes + (ks & 3) * 32;
                const uint64_t adesc = ptx::umma_desc_sw128(sm_qt + off, 16, 1024);
                const uint64_t bdesc = ptx::umma_desc_sw128(sm_k + off, 16, 1024);
                ptx::mma_ss(col_s, adesc, bdesc, idesc_qk, ks > 0 ? 1u : 0u);
              }
              ptx::mma_commit(ptx::smem_u32(&bars->s_full[t]));
              if (step == it.n[t] - 1) {
                ptx::mma_commit(ptx::smem_u32(&bars->q_free[t]));
                ++q_uses[t];
              }
            }
          }
          if (step < it.nmax) ptx::mma_commit(ptx::smem_u32(&bars->kv_free[pos_k % C::kStages]));
          if (step >= 1) ptx::mma_commit(ptx::smem_u32(&bars->kv_free[pos_v % C::kStages]));
        }
        ring_base += 2u * it.nmax;
      }
      // all MMAs (and the mbarrier arrivals of their commits) complete before the CTA tears down
      ptx::mma_commit(ptx::smem_u32(&bars->done));
      w.wait(ptx::smem_u32(&bars->done), 0);
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ P / O groups (thread = row)
    const int t = (warp - 4) >> 2;                 // Q tile of this group
    const int row = (threadIdx.x - 128) & 127;     // row inside the tile == TMEM lane
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t t_s = tmem + lane_base + (t == 0 ? kColS0 : kColS1);
    const uint32_t t_o = tmem + lane_base + (t == 0 ? kColO0 : C::kColO1);
    const uint32_t bar_s = ptx::smem_u32(&bars->s_full[t]);
    const uint32_t bar_p = ptx::smem_u32(&bars->p_full[t]);
    const uint32_t bar_of = ptx::smem_u32(&bars->o_full[t]);
    const uint32_t bar_oe = ptx::smem_u32(&bars->o_free[t]);
    const bool alpha_first = (p.flags & HSTU_FLAG_ALPHA_BEFORE_BIAS) != 0;
    constexpr bool kExact = Pack<T>::kFormat == 0;  // fp16: two-MUFU sigmoid; bf16: one-MUFU tanh form
    const float c_in = kExact ? p.alpha : 0.5f * p.alpha;
    const float c_bias = alpha_first ? (kExact ? 1.f : 0.5f) : c_in;
    uint32_t s_uses = 0, o_uses = 0;
    long long round = 0;
    for (long long first = 0; first < num_items; first += G, ++round) {
      const long long idx = first + ((round & 1) ? (G - 1 - cta) : cta);
      if (idx >= num_items) continue;
      const Item it = load_item(p, idx);
      const int tile_r0 = it.r0 + t * kTileM;
      if (tile_r0 >= it.s.lq) continue;
      const int i = tile_r0 + row;
      const bool row_ok = i < it.s.lq;
      const RowBounds rb = row_bounds(it.s, row_ok ? i : it.s.lq - 1, p.mask_type, p.group);
      const long long bias_row = kBias ? static_cast<long long>(it.b) * p.bias_bstride +
                                             (static_cast<long long>(it.h) * p.maxq + i) * p.maxk
                                       : 0;
      for (int j = 0; j < it.n[t]; ++j) {
        const int c0 = j * kTileN;
        const bool full = tile_is_full(it.s, tile_r0, kTileM, c0, kTileN, p.mask_type, p.group);
        w.wait(bar_s, s_uses & 1u);
        ++s_uses;
        ptx::tc_fence_after();
#pragma unroll 1
        for (int ch = 0; ch < kTileN / 32; ++ch) {
          uint32_t sr[32];
          ptx::tmem_ld32(t_s + ch * 32, sr);
          float bv[32];
          if (kBias) {
            const int jb = c0 + ch * 32;
            if (row_ok && bias_vec_ok && jb + 32 <= p.maxk) {
              const uint4* src = reinterpret_cast<const uint4*>(static_cast<const T*>(p.bias) + bias_row + jb);
#pragma unroll
              for (int q4 = 0; q4 < 4; ++q4) {
                const uint4 u = __ldg(src + q4);
                const uint32_t uu[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float2 f = Pack<T>::unpack(uu[e]);
                  bv[q4 * 8 + e * 2] = f.x;
                  bv[q4 * 8 + e * 2 + 1] = f.y;
                }
              }
            } else {
#pragma unroll
              for (int e = 0; e < 32; ++e)
                bv[e] = (row_ok && jb + e < it.s.lk) ? Pack<T>::one(p.bias, bias_row + jb + e) : 0.f;
            }
          }
          ptx::tmem_wait_ld();
          uint32_t pr[16];
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            float x0 = __uint_as_float(sr[e]), x1 = __uint_as_float(sr[e + 1]);
            if (kBias) {
              if (alpha_first) {
                x0 = fmaf(x0, c_in, bv[e] * c_bias);
                x1 = fmaf(x1, c_in, bv[e + 1] * c_bias);
              } else {
                x0 = (x0 + bv[e]) * c_in;
                x1 = (x1 + bv[e + 1]) * c_in;
              }
            } else {
              x0 *= c_in;
              x1 *= c_in;
            }
            float p0, p1;
            if (kExact) {
              p0 = silu_scaled_exact(x0, p.scale);
              p1 = silu_scaled_exact(x1, p.scale);
            } else {
              p0 = silu_scaled_tanh(x0, p.scale);
              p1 = silu_scaled_tanh(x1, p.scale);
            }
            if (!full) {
              const int jc = c0 + ch * 32 + e;
              p0 = allowed(rb, jc) ? p0 : 0.f;
              p1 = allowed(rb, jc + 1) ? p1 : 0.f;
            }
            pr[e >> 1] = Pack<T>::pack(p0, p1);
          }
          ptx::tmem_st16(t_s + ch * 16, pr);
        }
        ptx::tmem_wait_st();
        ptx::tc_fence_before();
        ptx::mbar_arrive(bar_p);
      }
      T* orow = static_cast<T*>(p.out) + ((it.s.q0 + i) * p.hq + it.h) * D;
      if (it.n[t] > 0) {
        w.wait(bar_of, o_uses & 1u);
        ++o_uses;
        ptx::tc_fence_after();
#pragma unroll 1
        for (int ch = 0; ch < D / 32; ++ch) {
          uint32_t orr[32];
          ptx::tmem_ld32(t_o + ch * 32, orr);
          ptx::tmem_wait_ld();
          if (row_ok) {
            uint4* dst = reinterpret_cast<uint4*>(orow + ch * 32);
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint4 u;
              u.x = Pack<T>::pack(__uint_as_float(orr[q4 * 8 + 0]), __uint_as_float(orr[q4 * 8 + 1]));
              u.y = Pack<T>::pack(__uint_as_float(orr[q4 * 8 + 2]), __uint_as_float(orr[q4 * 8 + 3]));
              u.z = Pack<T>::pack(__uint_as_float(orr[q4 * 8 + 4]), __uint_as_float(orr[q4 * 8 + 5]));
              u.w = Pack<T>::pack(__uint_as_float(orr[q4 * 8 + 6]), __uint_as_float(orr[q4 * 8 + 7]));
              dst[q4] = u;
            }
          }
        }
        ptx::tc_fence_before();
        ptx::mbar_arrive(bar_oe);
      } else if (row_ok) {
        uint4* dst = reinterpret_cast<uint4*>(orow);
#pragma unroll
        for (int q4 = 0; q4 < D / 8; ++q4) dst[q4] = make_uint4(0, 0, 0, 0);
      }
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------- host side
PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
  });
  return fn;
}

// 3-D view (dim, heads, tokens) of a contiguous [tokens, heads, dim] tensor; box = 64 x 1 x 128, 128-byte swizzle.
bool make_map(CUtensorMap* m, const void* base, long long tokens, int heads, int dim, int dtype) {
  auto fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(dim), static_cast<cuuint64_t>(heads),
                        static_cast<cuuint64_t>(tokens > 0 ? tokens : 1)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(dim) * 2, static_cast<cuuint64_t>(dim) * 2 * heads};
  cuuint32_t box[3] = {64, 1, static_cast<cuuint32_t>(kTileM)};
  cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapDataType dt = dtype == HSTU_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                          : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUresult r = fn(m, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

template <int D, typename T, bool kBias>
cudaError_t launch_inst(const KParams& p, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                        int bias_vec_ok, int grid, cudaStream_t stream) {
  auto kern = hstu_tc_kernel<D, T, kBias>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<D>::kSmemBytes);
  if (e != cudaSuccess) return e;
  kern<<<grid, kThreads, Cfg<D>::kSmemBytes, stream>>>(p, mq, mk, mv, bias_vec_ok);
  return cudaGetLastError();
}

}  // namespace

bool tc_supported(const KParams& p, int dtype) {
  if (dtype != HSTU_DTYPE_BF16 && dtype != HSTU_DTYPE_FP16) return false;
  if (p.dqk != p.dv || (p.dqk != 64 && p.dqk != 128)) return false;
  if (p.mask_type != HSTU_MASK_TRIL && p.mask_type != HSTU_MASK_NONE) return false;
  if (p.hq > 0xffff || p.total_q > 0x7fffff00ll || p.total_k > 0x7fffff00ll) return false;
  const uintptr_t align = reinterpret_cast<uintptr_t>(p.q) | reinterpret_cast<uintptr_t>(p.k) |
                          reinterpret_cast<uintptr_t>(p.v) | reinterpret_cast<uintptr_t>(p.out);
  return (align & 15u) == 0;
}

// Returns cudaSuccess, a CUDA error, or cudaErrorNotSupported when the tensor maps could not be encoded.
cudaError_t launch_tc(const KParams& p, int dtype, int num_sms, cudaStream_t stream) {
  CUtensorMap mq, mk, mv;
  if (!make_map(&mq, p.q, p.total_q, p.hq, p.dqk, dtype) || !make_map(&mk, p.k, p.total_k, p.hk, p.dqk, dtype) ||
      !make_map(&mv, p.v, p.total_k, p.hk, p.dv, dtype))
    return cudaErrorNotSupported;
  long long grid = p.item_capacity < num_sms ? p.item_capacity : num_sms;
  if (grid < 1) grid = 1;
  const int g = static_cast<int>(grid);
  const int vec_ok = p.bias && (p.maxk % 8 == 0) && (p.bias_bstride % 8 == 0) &&
                     (reinterpret_cast<uintptr_t>(p.bias) & 15u) == 0;
  const bool bias = p.bias != nullptr;
#define HSTU_TC_CASE(DD, TT)                                                                 \
  return bias ? launch_inst<DD, TT, true>(p, mq, mk, mv, vec_ok, g, stream)                 \
              : launch_inst<DD, TT, false>(p, mq, mk, mv, vec_ok, g, stream)
  if (dtype == HSTU_DTYPE_BF16) {
    if (p.dqk == 128) { HSTU_TC_CASE(128, __nv_bfloat16); }
    HSTU_TC_CASE(64, __nv_bfloat16);
  }
  if (p.dqk == 128) { HSTU_TC_CASE(128, __half); }
  HSTU_TC_CASE(64, __half);
#undef HSTU_TC_CASE
}

}  // namespace hstu
