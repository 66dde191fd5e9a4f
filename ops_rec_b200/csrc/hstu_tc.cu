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
// rescaling), then goes TMEM -> registers -> shared memory -> TMA stores (a tile cut by the sequence end: 16-byte
// row stores that stop at the end) into the jagged [tokens, heads, dim] output.
// Compare the reference kernel, which moves every S tile and every P tile through a global-memory ring
// between its matrix and vector cores and accumulates partial O rows with atomics
// (…/op_kernel/atlas950/hstu_dense_forward_kernel_patten_bsnd.h:156-176, 590-689,
//  hstu_dense_forward_jagged_kernel.h:257-398).
//
// Warp roles (384 threads): warp 0 = TMA producer, warps 1 and 3 = MMA issuers (one per Q tile), warp 2 = TMEM
// allocator, work-item scheduler and TMA producer of the staged bias tiles, warps 4-7 and 8-11 = the two P/O groups:
// both work on both Q tiles, group g owning 64 of the 128 score columns and half of the output columns of each.
//
// Every wait on an mbarrier is bounded: after ~1 s without progress the waiter raises HSTU_ST_PIPE_TIMEOUT in
// the workspace status word and a CTA-wide abort flag that turns all later waits into no-ops, so the kernel
// always runs to its end, frees its tensor memory and returns (with garbage in `out` and the flag set).  Once the flag
// is up no role touches a barrier any more: a role that passed a wait only because of the flag leaves its loop.
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <mutex>

#include <type_traits>

#include "hstu_common.cuh"
#include "ptx_sm100.cuh"

namespace hstu {

namespace {

constexpr int kThreads = 384;
constexpr int kTmemCols = 512;
constexpr int kColS0 = 0, kColS1 = 128, kColO0 = 256;
constexpr long long kWaitLimitCycles = 2000000000ll;  // ~1 s
constexpr int kSchedStages = 8;                       // depth of the work-item ring between scheduler and roles
constexpr int kSchedReaders = 3 + 2 * 128;            // producer lane + two MMA lanes + every thread of both P/O groups
                                                      // (+ the two bias cursors of the scheduler thread, kBias == 2)

// kBias: 0 = no attn_bias, 1 = bias read by plain loads and added in registers (fallback when its rows are not
// 16-byte aligned, or with HSTU_FLAG_ALPHA_BEFORE_BIAS),
// 3 = no bias, but a custom mask (mask_type 3) read by plain loads through the same operand path: P *= mask,
// 2 = bias tiles staged in shared memory by TMA and added to S on the tensor cores: after S = Q.K^T the issuer
//     runs eight M128 N16 K16 products  S[:, 16s .. 16s+16) += bias[:, 16s .. 16s+16) . I16  (the staged tile is the
//     K-major A operand, a 16 x 16 identity the B operand), so the P/O groups never touch the bias and the
//     staging buffer is free again as soon as these products complete.
template <int D, int kBias = 0>
struct Cfg {
  static constexpr int kHalves = D / 64;                 // 128-byte swizzle atoms along the head dim
  static constexpr int kHalfBytes = kTileM * 128;        // 128 rows x 128 B
  static constexpr int kTileBytes = kHalves * kHalfBytes;
  static constexpr int kBiasBytes = kBias == 2 ? 2 * kTileM * kTileN * 2 : 0;  // one 128x128 16-bit tile per Q tile
  static constexpr int kStages = D == 128 ? (kBias == 2 ? 3 : 4) : 8;          // K/V ring slots (one tile each)
  static constexpr int kQBytes = 2 * kTileBytes;
  static constexpr int kRingBytes = kStages * kTileBytes;
  static constexpr int kBarBytes = 2048;
  // output staging for TMA stores: per P/O group two buffers of 128 rows x 32 columns (16 bit); not available
  // when the staged bias tiles already fill the shared memory
  static constexpr int kOutWarpBytes = 32 * 32 * 2;   // output staging: 32 rows x 32 columns per warp and buffer
  static constexpr int kOutBytes = kBias == 2 ? 0 : 8 * 2 * kOutWarpBytes;
  static constexpr int kSmemBytes = 1024 + kQBytes + kRingBytes + kBiasBytes + kOutBytes + kBarBytes;
  static constexpr int kColO1 = kColO0 + D;
};

// A decoded work item: (sequence, head, 256-row q-pair) with the sequence geometry and the number of K tiles each
// of the two Q tiles visits.  The scheduler warp decodes it once; the other roles read it from shared memory.
struct Item {
  SeqInfo s;
  int b, h, hk, r0;
  int n0, n1;
  int nmax;
  int valid;  // 0 = end of work
  // hstu_paged with direct page reads: the K / V tiles 0 .. full_pages - 1 are the cache pages
  // page_ids[first_slot + j], the others come from the staging tensors like any jagged K / V
  int full_pages;
  long long first_slot;
  __device__ __forceinline__ int n(int t) const { return t == 0 ? n0 : n1; }
};

// What the output store of one Q tile needs to know.
struct OutTile {
  long long q0;   // first token of the sequence
  int lq;         // its length (rows at or after it are never written)
  int tile_r0;    // first row of the tile inside the sequence
  int h;          // query head
  int n;          // K tiles the tile visited (0: its rows are zeros)
};

struct Barriers {
  uint64_t q_full[2], q_free[2];
  uint64_t s_full[2], p_full[2][2];  // P is handed over in two steps, each by all 256 P/O threads
  uint64_t o_full[2], o_free[2];
  uint64_t done[2];
  uint64_t bias_full[2], bias_free[2];
  uint64_t kv_full[8], kv_free[8];
  uint64_t sched_full[kSchedStages], sched_free[kSchedStages];
  Item sched_item[kSchedStages];
  uint32_t tmem_base;
  int abort_flag;
  // kBias == 2: the 16 x 16 identity the bias products multiply by, in the element type, as a K-major operand
  // without swizzle: four 8 x 8 core matrices of 128 bytes, element (n, k) at (n/8)*256 + (k/8)*128 + (n%8)*16 + (k%8)*2
  alignas(16) uint16_t ident[256];
};
static_assert(sizeof(Barriers) <= 2048, "barrier block too large");

// The waiting loop of Waiter::wait, one copy for every wait of the kernel (the fast path - the phase is already
// complete - stays inline): less code for the instruction caches, and the warps that spin all spin in the same lines.
__device__ __noinline__ void wait_slow(int* abort_flag, uint32_t* status, uint32_t bar, uint32_t parity) {
  if (*reinterpret_cast<volatile int*>(abort_flag)) return;
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

struct Waiter {
  int* abort_flag;
  uint32_t* status;
  // `polled` is the result of an earlier mbar_try_wait on the same phase (polls of several barriers are issued
  // back to back so that their latencies overlap); only an unsuccessful poll falls into the waiting loop.
  __device__ __forceinline__ void wait_polled(bool polled, uint32_t bar, uint32_t parity) const {
    if (!polled) wait(bar, parity);
  }
  __device__ __forceinline__ bool aborted() const { return *reinterpret_cast<volatile int*>(abort_flag) != 0; }
  __device__ __forceinline__ void wait(uint32_t bar, uint32_t parity) const {
    if (ptx::mbar_try_wait(bar, parity)) return;
    wait_slow(abort_flag, status, bar, parity);
  }
};

// Consumer side of the work-item ring: every role sees the same sequence of items, in the order the scheduler
// warp drew them from the global counter.
struct ItemFeed {
  Barriers* bars;
  const Waiter* w;
  uint32_t n;
  __device__ __forceinline__ bool next(Item& it) {
    const uint32_t slot = n % kSchedStages;
    w->wait(ptx::smem_u32(&bars->sched_full[slot]), (n / kSchedStages) & 1u);
    it = bars->sched_item[slot];
    if (*reinterpret_cast<volatile int*>(w->abort_flag)) it.valid = 0;  // a wait gave up: stop taking work
    ptx::mbar_arrive(ptx::smem_u32(&bars->sched_free[slot]));
    ++n;
    return it.valid != 0;
  }
};


__device__ __forceinline__ Item load_item(const KParams& p, long long idx) {
  Item it;
  it.b = static_cast<int>(p.items[2 * idx]);
  const uint32_t hp = p.items[2 * idx + 1];
  it.h = static_cast<int>(hp >> 16);
  it.r0 = static_cast<int>(hp & 0xffffu) * kPairM;
  // an entry that does not name a (sequence, head) of this call does nothing (the list is rebuilt by every call,
  // so this can only happen with inconsistent offsets; it must still never address anything out of range)
  if (it.b < 0 || it.b >= p.batch || it.h >= p.hq) {
    it.b = 0;
    it.h = 0;
    it.r0 = 0x40000000;
  }
  it.hk = it.h / p.gqa_ratio;
  it.s = load_seq(p, it.b);
  it.n0 = kv_tiles_for_rows(it.s, it.r0, kTileM, p.mask_type, kTileN);
  it.n1 = kv_tiles_for_rows(it.s, it.r0 + kTileM, kTileM, p.mask_type, kTileN);
  it.nmax = it.n0 > it.n1 ? it.n0 : it.n1;
  it.full_pages = 0;
  it.first_slot = 0;
  if (p.paged_direct)
    it.full_pages = paged_full_tiles(p.offq, p.offk, p.tgt, p.page_offsets, p.index_bytes, p.total_q, p.num_page_ids,
                                     it.b, &it.first_slot);
  it.valid = 1;
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

struct BiasRow {
  const void* base;     // attn_bias
  long long row;        // element offset of (b, h, i, 0)
  bool row_ok;          // row i exists in the sequence
  bool vec_ok;          // 16-byte loads are aligned
  int maxk, lk;
};

// 32 consecutive bias values of one row, starting at column jb, as 16 packed words (0 beyond the sequence).
template <typename T>
__device__ __forceinline__ void load_bias32(const BiasRow& br, int jb, uint32_t (&bv)[16]) {
  if (br.row_ok && br.vec_ok && jb + 32 <= br.maxk) {
    const uint4* src = reinterpret_cast<const uint4*>(static_cast<const T*>(br.base) + br.row + jb);
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) {
      const uint4 u = __ldg(src + q4);
      bv[q4 * 4] = u.x;
      bv[q4 * 4 + 1] = u.y;
      bv[q4 * 4 + 2] = u.z;
      bv[q4 * 4 + 3] = u.w;
    }
  } else {
    const unsigned short* src = static_cast<const unsigned short*>(br.base);
#pragma unroll
    for (int e = 0; e < 16; ++e) {
      const uint32_t lo = (br.row_ok && jb + 2 * e < br.lk) ? src[br.row + jb + 2 * e] : 0u;
      const uint32_t hi = (br.row_ok && jb + 2 * e + 1 < br.lk) ? src[br.row + jb + 2 * e + 1] : 0u;
      bv[e] = lo | (hi << 16);
    }
  }
}

// 32 scores of one row (fp32 bits in sr) -> 16 words of packed P.  Branch-free; the arithmetic runs on the
// packed f32x2 pipe.  x = c_in * s + c_bias * bias covers both orders of alpha and bias (c_bias = c_in gives
// alpha * (s + bias)).
// One tanh.approx per element is the SFU's whole budget (16 results/clk/SM = 1024 clk per 128 x 128 tile).  Moving
// half of the columns to an FMA-pipe polynomial was tried: it is faster only without a range check, and any
// data-dependent branch in this block costs more than it saves, so every element goes through the SFU.
template <typename T, int kBias, bool kMasked>
__device__ __forceinline__ void silu_chunk(const uint32_t (&sr)[32], const uint32_t (&bv)[16], uint32_t (&pr)[16],
                                           float c_in, float c_bias, float scale, uint32_t visible) {
  constexpr bool kExact = Pack<T>::kFormat == 0;  // fp16: exp2 + rcp (two MUFU ops); bf16: tanh form (one)
  const float2 cin2 = make_float2(c_in, c_in);
  const float2 cb2 = make_float2(c_bias, c_bias);
  const float2 sc2 = make_float2(scale, scale);
#pragma unroll
  for (int e = 0; e < 16; ++e) {
    float2 x = make_float2(__uint_as_float(sr[2 * e]), __uint_as_float(sr[2 * e + 1]));
    if (kBias == 1)
      x = __ffma2_rn(x, cin2, __fmul2_rn(Pack<T>::unpack(bv[e]), cb2));
    else
      x = __fmul2_rn(x, cin2);
    const float2 r = __fmul2_rn(x, sc2);
    float2 o;
    if (kExact) {
      // sigmoid form: o = y*scale / (1 + 2^(-y log2 e))
      const float2 ny = __fmul2_rn(x, make_float2(-1.4426950408889634f, -1.4426950408889634f));
      const float2 d = __fadd2_rn(make_float2(ptx::ex2_approx(ny.x), ptx::ex2_approx(ny.y)), make_float2(1.f, 1.f));
      o = __fmul2_rn(r, make_float2(ptx::rcp_approx(d.x), ptx::rcp_approx(d.y)));
    } else {
      // tanh form on x = y/2: o = x*scale*(1 + tanh x)
      o = __ffma2_rn(r, make_float2(ptx::tanh_approx(x.x), ptx::tanh_approx(x.y)), r);
    }
    if (kBias == 3) o = __fmul2_rn(o, Pack<T>::unpack(bv[e]));  // custom mask: its values multiply (fp32)
    if (kMasked) {  // a select, not a multiply: scores of rows past the sequence end may be Inf or NaN
      o.x = (visible & (1u << (2 * e))) ? o.x : 0.f;
      o.y = (visible & (2u << (2 * e))) ? o.y : 0.f;
    }
    pr[e] = Pack<T>::pack(o.x, o.y);
  }
}

// Bit e set <=> column j0 + e is visible to the row described by rb (columns j0 .. j0 + 31).
__device__ __forceinline__ uint32_t low_bits(int n) {  // n lowest bits set, n clamped to [0, 32]
  return n <= 0 ? 0u : (n >= 32 ? 0xffffffffu : ((1u << n) - 1u));
}
__device__ __forceinline__ uint32_t visible_bits(const RowBounds& rb, int j0) {
  return low_bits(rb.lim1 - j0) | (low_bits(rb.hi2 + 1 - j0) & ~low_bits(rb.lo2 - j0));
}

// kBias == 2, a sequence's last K tile: the 16-column slice that contains the sequence end is not added by the tensor
// cores - whatever lies in the bias buffer beyond column lk would reach the slice's visible columns through the
// identity product (0 x NaN).  The warps that own the slice add its n (< 16) in-sequence bias values of their rows to
// S in tensor memory before they compute P: load 16 columns, add, store back.  `bv` holds the slice as packed
// pairs, fetched from global memory before the wait for the scores (zeros for rows outside the sequence).  Called by
// whole warps (the tensor-memory accesses are warp-wide); kept out of p_half so that tiles without such a slice
// execute none of it.
template <typename T>
__device__ __forceinline__ void add_end_slice(uint32_t t_slice, const uint32_t (&bv)[8], int n) {
  uint32_t v[16];
  ptx::tmem_ld16(t_slice, v);
  ptx::tmem_wait_ld();
#pragma unroll
  for (int e = 0; e < 15; ++e) {
    const float2 b2 = Pack<T>::unpack(bv[e >> 1]);
    if (e < n) v[e] = __float_as_uint(__uint_as_float(v[e]) + ((e & 1) ? b2.y : b2.x));
  }
  ptx::tmem_st16(t_slice, v);
  ptx::tmem_wait_st();
}

// Zeroes `pieces` 16-byte pieces from shared-memory address `first` on, in each of `boxes` regions `box_bytes` apart
// (the rows of a V tile behind a sequence end); called by the 128 threads of a P/O group, `tid` = 0..127.
__device__ __noinline__ void zero_v_rows(uint32_t first, int pieces, int tid, int boxes, int box_bytes) {
  for (int i = tid; i < pieces; i += kTileM)
    for (int b = 0; b < boxes; ++b) ptx::st_shared_zero16(first + b * box_bytes + i * 16);
  ptx::fence_proxy_async();
}

// This thread's 64 columns of one 128 x 128 score tile, its row: S (TMEM, fp32) -> P (TMEM, packed 16-bit).
// Group g reads the S columns [64g, 64g+64) and writes its half of P inside its own column range (keys 0..63 at
// columns 0..31, keys 64..127 at columns 64..95), so neither group ever overwrites scores the other still has to
// read.  The TMEM load of the second 32 columns is in flight while the first 32 are computed.  In a tile the mask
// cuts through (kMasked) every warp classifies each 32 x 32 chunk of its rows: all visible -> plain path, nothing
// visible -> zeros without any arithmetic, mixed -> per-element select.
//
// kBias == 2: the bias is already inside S when this runs (added by the tensor cores, and for the one slice that
// holds a sequence's end by add_end_slice below).
template <typename T, int kBias, bool kMasked>
__device__ __forceinline__ void p_half(uint32_t t_s, int grp, int c0, const BiasRow& br, const RowBounds& rb,
                                       float c_in, float c_bias, float scale, uint32_t bar_p0) {
  uint32_t sbuf[2][32];
  uint32_t bv[16];
  uint32_t pr[16];
  const uint32_t s_col = t_s + 64 * grp;
  const uint32_t p_col = t_s + 64 * grp;
  const int j0 = c0 + 64 * grp;
  ptx::tmem_ld32(s_col, sbuf[0]);
#pragma unroll
  for (int ch = 0; ch < 2; ++ch) {
    uint32_t vis = 0xffffffffu;
    bool all_on = true, all_off = false;
    if (kMasked) {
      vis = visible_bits(rb, j0 + ch * 32);
      all_on = __all_sync(0xffffffffu, vis == 0xffffffffu);
      all_off = __all_sync(0xffffffffu, vis == 0u);
    }
    if ((kBias == 1 || kBias == 3) && !all_off) load_bias32<T>(br, j0 + ch * 32, bv);
    ptx::tmem_wait_ld_dep(sbuf[ch]);
    if (ch == 0) ptx::tmem_ld32(s_col + 32, sbuf[1]);
    if (all_on) {
      silu_chunk<T, kBias, false>(sbuf[ch], bv, pr, c_in, c_bias, scale, 0u);
    } else if (all_off) {
#pragma unroll
      for (int e = 0; e < 16; ++e) pr[e] = 0u;
    } else {
      silu_chunk<T, kBias, true>(sbuf[ch], bv, pr, c_in, c_bias, scale, vis);
    }
    ptx::tmem_st16(p_col + ch * 16, pr);
    // hand these 32 keys to the MMA issuer (bar_p0 and the 8 bytes after it: the two hand-over barriers of the tile)
    ptx::tmem_wait_st();
    ptx::tc_fence_before();
    ptx::mbar_arrive(bar_p0 + 8 * ch);
  }
}

// kRolled: the P/O groups run both Q tiles of an item through one copy of their code.  Their code is most of what the
// SM's instruction caches have to hold; on batches of many short items - where every item walks through every path:
// tiles with and without a mask, the end-of-sequence slice, both kinds of output store - instruction-cache misses
// were the largest stall (batch of 4096 sequences of mean length 270 with a bias: - 21 % time).  Long sequences spend
// their time in one path and prefer the unrolled form (+ 6 % time rolled), so both exist and the launcher chooses.
template <int D, typename T, int kBias, bool kRolled>
__global__ void __launch_bounds__(kThreads, 1)
hstu_tc_kernel(const KParams p, const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_bias,
               const __grid_constant__ CUtensorMap tm_out, const __grid_constant__ CUtensorMap tm_cache,
               const int bias_vec_ok) {
  using C = Cfg<D, kBias>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  const uint32_t sm_q = base;                    // 2 Q tiles
  const uint32_t sm_ring = base + C::kQBytes;    // K/V ring
  const uint32_t sm_bias = sm_ring + C::kRingBytes;  // kBias == 2: one staged bias tile per Q tile
  const uint32_t sm_out = sm_bias + C::kBiasBytes;   // kOutBytes > 0: output staging, two 2 KB buffers per P/O warp
  Barriers* bars = reinterpret_cast<Barriers*>(base_ptr + C::kQBytes + C::kRingBytes + C::kBiasBytes + C::kOutBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const Waiter w{&bars->abort_flag, p.ws_header};

  if (threadIdx.x == 0) {
    ptx::prefetch_tensormap(&tm_q);
    ptx::prefetch_tensormap(&tm_k);
    ptx::prefetch_tensormap(&tm_v);
    if (p.paged_direct) ptx::prefetch_tensormap(&tm_cache);
    if (kBias == 2) ptx::prefetch_tensormap(&tm_bias);
    if (C::kOutBytes > 0) ptx::prefetch_tensormap(&tm_out);
    for (int t = 0; t < 2; ++t) {
      ptx::mbar_init(ptx::smem_u32(&bars->q_full[t]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->q_free[t]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->s_full[t]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->p_full[t][0]), 2 * kTileM);
      ptx::mbar_init(ptx::smem_u32(&bars->p_full[t][1]), 2 * kTileM);
      ptx::mbar_init(ptx::smem_u32(&bars->o_full[t]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->o_free[t]), 2 * kTileM);
    }
    ptx::mbar_init(ptx::smem_u32(&bars->done[0]), 1);
    ptx::mbar_init(ptx::smem_u32(&bars->done[1]), 1);
    for (int t = 0; t < 2; ++t) {
      ptx::mbar_init(ptx::smem_u32(&bars->bias_full[t]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->bias_free[t]), 1);  // the commit of the bias products
    }
    for (int s = 0; s < C::kStages; ++s) {
      ptx::mbar_init(ptx::smem_u32(&bars->kv_full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->kv_free[s]), 2);  // one arrival from each MMA issuer
    }
    for (int s = 0; s < kSchedStages; ++s) {
      ptx::mbar_init(ptx::smem_u32(&bars->sched_full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->sched_free[s]), kSchedReaders + (kBias == 2 ? 2 : 0));
    }
    bars->abort_flag = 0;
    ptx::fence_mbar_init();
  }
  if (kBias == 2 && threadIdx.x >= 128) {
    // the identity operand of the bias products (1.0 in the element type on the diagonal)
    const int e = threadIdx.x - 128, n = e >> 4, k = e & 15;
    const uint16_t one = Pack<T>::kFormat == 1 ? 0x3F80 : 0x3C00;
    bars->ident[((n >> 3) * 256 + (k >> 3) * 128 + (n & 7) * 16 + (k & 7) * 2) >> 1] = n == k ? one : 0;
    ptx::fence_proxy_async();  // generic-proxy writes, read by the tensor cores through the async proxy
  }
  if (warp == 2) {
    ptx::tmem_alloc(ptx::smem_u32(&bars->tmem_base), kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);

  ItemFeed feed{bars, &w, 0};

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t q_uses[2] = {0, 0};
      uint32_t ring_pos = 0;
      for (Item it; feed.next(it);) {
        // Q tile t of this item, once the MMAs of the previous item have finished with the buffer
        auto load_q = [&](int t) {
          if (it.n(t) == 0) return;
          const uint32_t full = ptx::smem_u32(&bars->q_full[t]);
          w.wait(ptx::smem_u32(&bars->q_free[t]), (q_uses[t] & 1u) ^ 1u);
          if (w.aborted()) return;  // a wait gave up somewhere: request nothing more, touch no barrier
          ptx::mbar_expect_tx(full, C::kTileBytes);
          const int row = static_cast<int>(it.s.q0) + it.r0 + t * kTileM;
#pragma unroll
          for (int hf = 0; hf < C::kHalves; ++hf)
            ptx::tma_load_3d(sm_q + t * C::kTileBytes + hf * C::kHalfBytes, &tm_q, full, hf * 64, it.h, row);
          ++q_uses[t];
        };
        // Order: Q tile 0, K tile 0, Q tile 1, V tile 0, ...  Tile 1's buffer is released last by the previous
        // item (its chain ends one step later), and the first S tile of this item needs only Q tile 0 and K tile 0.
        load_q(0);
        for (int j = 0; j < it.nmax; ++j) {
          const int row = static_cast<int>(it.s.k0) + j * kTileN;
          // a whole cache page (hstu_paged): the cache is [pages, 2 (K, V), 128 rows, heads, dim]; a page id outside
          // the cache (flagged by the pre-pass) reads as zeros - the coordinate lies past the tensor
          const bool from_cache = j < it.full_pages;
          long long pid = 0;
          if (from_cache) {
            pid = load_index(p.page_ids, p.index_bytes, it.first_slot + j);
            if (pid < 0 || pid >= p.num_pages) pid = p.num_pages;
          }
#pragma unroll
          for (int kv = 0; kv < 2; ++kv) {
            const uint32_t stage = ring_pos % C::kStages;
            const uint32_t use = ring_pos / C::kStages;
            const uint32_t full = ptx::smem_u32(&bars->kv_full[stage]);
            w.wait(ptx::smem_u32(&bars->kv_free[stage]), (use & 1u) ^ 1u);
            if (w.aborted()) break;
            ptx::mbar_expect_tx(full, C::kTileBytes);
            const CUtensorMap* tm = from_cache ? &tm_cache : (kv == 0 ? &tm_k : &tm_v);
            const int trow = from_cache ? static_cast<int>((pid * 2 + kv) * kTileN) : row;
#pragma unroll
            for (int hf = 0; hf < C::kHalves; ++hf)
              ptx::tma_load_3d(sm_ring + stage * C::kTileBytes + hf * C::kHalfBytes, tm, full, hf * 64, it.hk, trow);
            ++ring_pos;
            if (j == 0 && kv == 0) load_q(1);
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
  } else if (warp == 1 || warp == 3) {
    // ------------------------------------------------------------------ MMA issuers, one per Q tile.
    // Each chain (S_t = Q_t.K^T, then O_t += P_t.V) is issued by its own thread: a barrier poll costs the
    // issuing thread ~130 cycles and the tensor pipe queues only a few instructions, so while one issuer
    // waits for its P tile the other keeps the pipe fed.  The chains share nothing but the read-only K/V tiles.
    // The thread is an elected one, not `lane == 0`: the compiler then knows that a single thread runs this code
    // and keeps the descriptors and barrier addresses in uniform registers (cfg5-shaped batches: -18 % time).
    // (The same for the producer and the scheduler was measured slower.)
    if (ptx::elect_one()) {
      const int t = warp == 1 ? 0 : 1;
      constexpr uint32_t idesc_qk = ptx::umma_idesc_f16(Pack<T>::kFormat, kTileM, kTileN, 0);
      constexpr uint32_t idesc_pv = ptx::umma_idesc_f16(Pack<T>::kFormat, kTileM, D, 1);
      // descriptor templates (everything but the start address): K-major Q / K tiles, N-major V tiles
      constexpr uint64_t kDescK = ptx::umma_desc_sw128_hi(16, 1024);
      constexpr uint64_t kDescV = ptx::umma_desc_sw128_hi(C::kHalfBytes, 1024);
      const uint32_t col_s = tmem + (t == 0 ? kColS0 : kColS1);
      const uint32_t col_o = tmem + (t == 0 ? kColO0 : C::kColO1);
      const uint64_t qbase = kDescK | static_cast<uint64_t>((sm_q + t * C::kTileBytes) >> 4);
      const uint32_t bar_q_full = ptx::smem_u32(&bars->q_full[t]), bar_q_free = ptx::smem_u32(&bars->q_free[t]);
      const uint32_t bar_s_full = ptx::smem_u32(&bars->s_full[t]);
      const uint32_t bar_p_full = ptx::smem_u32(&bars->p_full[t][0]), bar_p_half1 = ptx::smem_u32(&bars->p_full[t][1]);
      const uint32_t bar_o_full = ptx::smem_u32(&bars->o_full[t]), bar_o_free = ptx::smem_u32(&bars->o_free[t]);
      // kBias == 2: the staged bias tile of this Q tile as K-major A operand, the identity as B operand (no swizzle:
      // 128 bytes between the core matrices along K, 256 along N), 16 score columns per product
      constexpr uint32_t idesc_bias = ptx::umma_idesc_f16(Pack<T>::kFormat, kTileM, 16, 0);
      const uint64_t bias_base = kDescK | static_cast<uint64_t>((sm_bias + t * (kTileM * kTileN * 2)) >> 4);
      const uint64_t ident_desc = static_cast<uint64_t>((ptx::smem_u32(bars->ident) & 0x3FFFFu) >> 4) |
                                  (static_cast<uint64_t>(128 >> 4) << 16) | (static_cast<uint64_t>(256 >> 4) << 32) |
                                  (static_cast<uint64_t>(1) << 46);
      const uint32_t bar_bias_full = ptx::smem_u32(&bars->bias_full[t]);
      const uint32_t bar_bias_free = ptx::smem_u32(&bars->bias_free[t]);
      uint32_t q_uses = 0, p_uses = 0, o_uses = 0, b_uses = 0;
      uint32_t ring_base = 0;
      for (Item it; feed.next(it);) {
        const int n = it.n(t);
        for (int step = 0; step <= it.nmax; ++step) {
          const uint32_t pos_k = ring_base + 2u * step;             // K(step)
          const uint32_t pos_v = ring_base + 2u * (step - 1) + 1u;  // V(step - 1)
          const uint32_t st_k = pos_k % C::kStages, st_v = pos_v % C::kStages;
          const bool has_v = step >= 1, has_k = step < it.nmax;
          const bool do_pv = has_v && step - 1 < n, do_qk = has_k && step < n;
          const uint32_t bar_vf = ptx::smem_u32(&bars->kv_full[st_v]), par_vf = (pos_v / C::kStages) & 1u;
          const uint32_t bar_kf = ptx::smem_u32(&bars->kv_full[st_k]), par_kf = (pos_k / C::kStages) & 1u;
          // A V tile that is cut by its sequence's end is waited for a step early, together with its K tile: the
          // completion of S(step) then tells the P/O groups that V(step) has landed too (they zero the rows behind
          // the end in it without having to poll its barrier).  (Waiting early for every V tile costs ring depth:
          // -14 % on long sequences.)
          const bool cut_v = has_k && it.s.lk - step * kTileN < kTileN;
          const uint32_t bar_vc = ptx::smem_u32(&bars->kv_full[(pos_k + 1u) % C::kStages]);
          const uint32_t par_vc = ((pos_k + 1u) / C::kStages) & 1u;
          // The two issuers run free of each other: the P/O groups serve the tiles in a fixed order (tile 0,
          // tile 1, tile 0 ...), so the P tiles - and with them the MMA bursts - alternate by themselves.
          // poll everything this step needs at once
          const bool ok_v = has_v ? ptx::mbar_try_wait(bar_vf, par_vf) : true;
          const bool ok_k = has_k ? ptx::mbar_try_wait(bar_kf, par_kf) : true;
          const bool ok_p = do_pv ? ptx::mbar_try_wait(bar_p_full, p_uses & 1u) : true;
          const bool ok_b = (kBias == 2 && do_qk) ? ptx::mbar_try_wait(bar_bias_full, b_uses & 1u) : true;
          w.wait_polled(ok_v, bar_vf, par_vf);
          w.wait_polled(ok_k, bar_kf, par_kf);
          if (cut_v) w.wait(bar_vc, par_vc);
          if (kBias == 2 && do_qk) w.wait_polled(ok_b, bar_bias_full, b_uses & 1u);
          w.wait_polled(ok_p, bar_p_full, p_uses & 1u);
          if (do_pv && step == 1) w.wait(bar_o_free, (o_uses & 1u) ^ 1u);
          if (do_qk && step == 0) w.wait(bar_q_full, q_uses & 1u);
          if (w.aborted()) break;  // a wait gave up somewhere: issue nothing more, touch no barrier
          ptx::tc_fence_after();
          if (do_pv) {
            // O_t (+)= P_t(step-1) . V(step-1)
            const uint64_t vbase = kDescV | static_cast<uint64_t>((sm_ring + st_v * C::kTileBytes) >> 4);
            // P arrives in two steps: first the leading 32 keys of both 64-key halves (k-steps 0, 1, 4, 5), then,
            // while these MMAs run, the rest.  Keys 0..63 sit at columns 0..31 of the S tile, keys 64..127 at
            // columns 64..95.
            auto pv = [&](int ks, uint32_t acc) {
              ptx::mma_ts(col_o, col_s + (ks >> 2) * 64 + (ks & 3) * 8, vbase + static_cast<uint64_t>((ks * 2048) >> 4),
                          idesc_pv, acc);
            };
            pv(0, step > 1 ? 1u : 0u);
            pv(1, 1u);
            pv(4, 1u);
            pv(5, 1u);
            w.wait(bar_p_half1, p_uses & 1u);
            ptx::tc_fence_after();
            pv(2, 1u);
            pv(3, 1u);
            pv(6, 1u);
            pv(7, 1u);
            ++p_uses;
            if (step == n) {
              ptx::mma_commit(bar_o_full);
              ++o_uses;
            }
          }
          if (do_qk) {
            // S_t = Q_t . K(step)^T
            const uint64_t kbase = kDescK | static_cast<uint64_t>((sm_ring + st_k * C::kTileBytes) >> 4);
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
              const uint64_t off = static_cast<uint64_t>(((ks >> 2) * C::kHalfBytes + (ks & 3) * 32) >> 4);
              ptx::mma_ss(col_s, qbase + off, kbase + off, idesc_qk, ks > 0 ? 1u : 0u);
            }
            if (kBias == 2) {
              // S_t += bias tile, 16 columns per product; only the slices that lie wholly inside the sequence
              // (the slice that contains the sequence end is added by the P/O groups)
              const int inside = (it.s.lk - step * kTileN) >> 4;
              auto add_bias = [&](int sl) {
                const uint64_t off = static_cast<uint64_t>(((sl >> 2) * (kTileM * 128) + (sl & 3) * 32) >> 4);
                ptx::mma_ss(col_s + 16 * sl, bias_base + off, ident_desc, idesc_bias, 1u);
              };
              if (inside >= 8) {
#pragma unroll
                for (int sl = 0; sl < 8; ++sl) add_bias(sl);
              } else {
                for (int sl = 0; sl < inside; ++sl) add_bias(sl);
              }
              ptx::mma_commit(bar_bias_free);
              ++b_uses;
            }
            ptx::mma_commit(bar_s_full);
            if (step == n - 1) {
              ptx::mma_commit(bar_q_free);
              ++q_uses;
            }
          }
          // release the K/V tiles of this step: after this tile's MMAs that read them, or at once when this
          // tile does not visit them (the tile is loaded - waited above - so the arrival counts for its
          // current use)
          if (has_v) {
            if (do_pv) ptx::mma_commit(ptx::smem_u32(&bars->kv_free[st_v]));
            else ptx::mbar_arrive(ptx::smem_u32(&bars->kv_free[st_v]));
          }
          if (has_k) {
            if (do_qk) ptx::mma_commit(ptx::smem_u32(&bars->kv_free[st_k]));
            else ptx::mbar_arrive(ptx::smem_u32(&bars->kv_free[st_k]));
          }
        }
        if (w.aborted()) break;
        ring_base += 2u * it.nmax;
      }
      // all MMAs (and the mbarrier arrivals of their commits) complete before the CTA tears down
      ptx::mma_commit(ptx::smem_u32(&bars->done[t]));
      w.wait(ptx::smem_u32(&bars->done[t]), 0);
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------------ scheduler: draws items from the global
    // counter (the list is ordered heaviest sequences first, so this is greedy longest-first list scheduling)
    if (lane == 0) {
      // The kernel is launched with programmatic stream serialization: everything above overlapped the tail of
      // the scheduling pre-pass.  Only this thread reads what the pre-pass wrote (item count, work list, and the
      // offsets it validated), so only it has to wait for that grid to complete.
      asm volatile("griddepcontrol.wait;" ::: "memory");
      long long num_items = p.ws_header[1];
      if (num_items > p.item_capacity) num_items = p.item_capacity;  // never read past the list (inconsistent offsets)
      // Draw the next item from the global counter and publish it in ring slot n % kSchedStages.
      uint32_t q0_uses = 0;      // items published so far whose Q tile 0 visits at least one K tile
      bool last_has_q0 = false;  // ... the last one published among them
      auto publish = [&](uint32_t n) -> bool {
        const long long idx = static_cast<long long>(atomicAdd(&p.ws_header[2], 1u));
        const bool more = idx < num_items && !*reinterpret_cast<volatile int*>(&bars->abort_flag);
        Item it;
        if (more) it = load_item(p, idx);
        else it.valid = 0;
        last_has_q0 = more && it.n0 > 0;
        q0_uses += last_has_q0 ? 1u : 0u;
        bars->sched_item[n % kSchedStages] = it;
        ptx::mbar_arrive(ptx::smem_u32(&bars->sched_full[n % kSchedStages]));
        return more;
      };
      // How far this CTA draws ahead of the item its P/O groups have started: an item drawn is an item no other CTA
      // can take, so with few items per CTA a deep look-ahead hands the whole list to the CTAs that start first
      // (cfg2: 392 items, 148 CTAs, 8 slots - a third of the CTAs took everything).  One item of look-ahead is
      // what the loads need; more only pays when items are short and plentiful.
      // Long items (mean sequence length >= 1024: dozens of steps each) are taken one at a time as well: drawing ahead
      // buys nothing there (the next item's loads wait for the Q buffer anyway) and costs balance at the end of the
      // kernel (cfg4: + 5 %).
      const long long per_cta = num_items / (4 * static_cast<long long>(gridDim.x));
      const bool long_items = p.batch > 0 && p.total_q / p.batch >= 1024;
      const uint32_t ahead = static_cast<uint32_t>(
          per_cta < 1 || long_items ? 1 : (per_cta > kSchedStages ? kSchedStages : per_cta));
      if (kBias != 2) {
        for (uint32_t n = 0;; ++n) {
          w.wait(ptx::smem_u32(&bars->sched_free[n % kSchedStages]), ((n / kSchedStages) & 1u) ^ 1u);
          // (slot n - ahead has been read by every role: its P/O groups have started that item)
          if (ahead < kSchedStages && n >= ahead)
            w.wait(ptx::smem_u32(&bars->sched_free[(n - ahead) % kSchedStages]), ((n - ahead) / kSchedStages) & 1u);
          // With one item of look-ahead, draw the next item only when the last one is about to end (the Q tile 0
          // buffer is released with its last Q.K^T): the loads of the next item cannot start before that anyway,
          // and an item still in the list can go to a CTA that has run dry.
          if (ahead == 1 && n >= 1 && last_has_q0) w.wait(ptx::smem_u32(&bars->q_free[0]), (q0_uses - 1u) & 1u);
          if (!publish(n)) break;
        }
      } else {
        // With staged bias tiles this thread is also their TMA producer.  It polls instead of waiting: whenever a
        // ring slot is free it publishes the next item, and whenever the bias buffer of Q tile t is free (its bias
        // products have completed, early in the step) it requests that tile's next bias tile - so a bias tile has
        // a whole step to arrive, whatever the other loads are waiting for.  A cursor holds its item's ring slot
        // (it counts as one reader) until the item's last bias tile is requested.
        // (The loop exists twice, with and without the look-ahead limits: this thread's reaction time is the
        // latency of every bias tile, and the extra polls cost 5 % on batches of many short items.)
        uint32_t loads[2] = {0, 0};
        auto run = [&](auto limited) {
        constexpr bool kLimited = decltype(limited)::value;
        uint32_t n_pub = 0;
        bool sched_done = false;
        uint32_t cur_item[2] = {0, 0};
        int cur_j[2] = {0, 0};
        bool cur_done[2] = {false, false};
        long long t_progress = clock64();
        unsigned spins = 0;
        while (!(sched_done && cur_done[0] && cur_done[1])) {
          bool progress = false;
          // one poll per round: with a limit, the limit is the condition that binds (slots are released in item
          // order, so the ring slot itself - last used by item n - 8 - is free whenever item n - ahead has been read,
          // and the Q buffer of item n - 1 is released long after every role has read that item)
          bool may_draw = !sched_done;
          if (may_draw) {
            if (kLimited && ahead == 1 && n_pub >= 1 && last_has_q0)
              may_draw = ptx::mbar_try_wait(ptx::smem_u32(&bars->q_free[0]), (q0_uses - 1u) & 1u);
            else if (kLimited && n_pub >= ahead)
              may_draw = ptx::mbar_try_wait(ptx::smem_u32(&bars->sched_free[(n_pub - ahead) % kSchedStages]),
                                            ((n_pub - ahead) / kSchedStages) & 1u);
            else
              may_draw = ptx::mbar_try_wait(ptx::smem_u32(&bars->sched_free[n_pub % kSchedStages]),
                                            ((n_pub / kSchedStages) & 1u) ^ 1u);
          }
          if (may_draw) {
            if (!publish(n_pub)) sched_done = true;
            ++n_pub;
            progress = true;
          }
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            if (cur_done[t] || cur_item[t] >= n_pub) continue;
            const uint32_t slot = cur_item[t] % kSchedStages;
            const Item& of = bars->sched_item[slot];
            if (!of.valid) {
              cur_done[t] = true;
              continue;
            }
            if (cur_j[t] >= of.n(t)) {  // every bias tile of this item is requested: release the slot
              ptx::mbar_arrive(ptx::smem_u32(&bars->sched_free[slot]));
              ++cur_item[t];
              cur_j[t] = 0;
              progress = true;
              continue;
            }
            if (!ptx::mbar_try_wait(ptx::smem_u32(&bars->bias_free[t]), (loads[t] & 1u) ^ 1u)) continue;
            const uint32_t bfull = ptx::smem_u32(&bars->bias_full[t]);
            ptx::mbar_expect_tx(bfull, kTileM * kTileN * 2);
            const int brow = of.b * (p.bias_bstride ? p.hq * p.maxq : 0) + of.h * p.maxq + of.r0 + t * kTileM;
#pragma unroll
            for (int hf = 0; hf < 2; ++hf)
              ptx::tma_load_2d(sm_bias + t * (kTileM * kTileN * 2) + hf * (kTileM * 128), &tm_bias, bfull,
                               cur_j[t] * kTileN + hf * 64, brow);
            ++loads[t];
            ++cur_j[t];
            progress = true;
          }
          if (progress) {
            t_progress = clock64();
          } else if ((++spins & 0xffu) == 0) {
            // a wait gave up somewhere: every reader of the item ring stops by itself when it sees the flag
            if (*reinterpret_cast<volatile int*>(&bars->abort_flag)) break;
            if (clock64() - t_progress > kWaitLimitCycles) {
              *reinterpret_cast<volatile int*>(&bars->abort_flag) = 1;
              atomicOr(p.ws_header, static_cast<uint32_t>(HSTU_ST_PIPE_TIMEOUT));
            }
          }
        }
        };
        if (ahead < kSchedStages) run(std::true_type{});
        else run(std::false_type{});
        // the bias tiles this thread requested have landed (already true unless a wait gave up)
        for (int t = 0; t < 2; ++t) {
          if (loads[t] == 0) continue;
          const uint32_t bar = ptx::smem_u32(&bars->bias_full[t]);
          for (int spin = 0; spin < (1 << 22) && !ptx::mbar_try_wait(bar, (loads[t] - 1) & 1u); ++spin) {}
        }
      }
    }
    __syncwarp();
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ P / O groups (thread = row)
    // Both groups work on BOTH Q tiles: group g owns the score columns [64g, 64g+64) of every S tile and the
    // output columns [g*D/2, (g+1)*D/2) of every O tile.  A tile's P is therefore produced by two warps per SM
    // sub-partition at once (their SFU and FMA work overlaps), the halves of P become ready together, and the
    // groups are busy on one chain's tile while the other chain's MMAs run.
    const int grp = (warp - 4) >> 2;
    const int row = (threadIdx.x - 128) & 127;  // row inside a tile == TMEM lane
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const bool alpha_first = (p.flags & HSTU_FLAG_ALPHA_BEFORE_BIAS) != 0;
    constexpr bool kExact = Pack<T>::kFormat == 0;
    // bf16 works on a = y / 2 (tanh form), fp16 on y itself;  x = c_in * s + c_bias * bias
    const float c_in = kExact ? p.alpha : 0.5f * p.alpha;
    const float c_bias = alpha_first ? (kExact ? 1.f : 0.5f) : c_in;
    // (per Q tile, as scalars: the loop over the two tiles is not unrolled - this role's code is what the SM's
    // instruction caches have to hold, and on batches of short sequences their misses were the largest stall)
    uint32_t s_uses0 = 0, s_uses1 = 0, o_uses0 = 0, o_uses1 = 0;
    uint32_t out_chunks = 0;              // TMA-store chunks issued so far by this warp (selects the staging buffer)
    // O tiles: this group's half of the columns.  A Q tile that lies wholly inside its sequence leaves through
    // shared memory and TMA stores (32 rows x 32 columns per warp and store, double buffered); a tile cut by the
    // sequence end must not touch the rows after it and is written row by row.
    auto store_o = [&](const int t, const OutTile& ot) {
      const int tile_r0 = ot.tile_r0;
      if (tile_r0 >= ot.lq) return;
      const int col0 = grp * (D / 2);
      const bool row_ok_t = tile_r0 + row < ot.lq;
      T* orow = static_cast<T*>(p.out) + ((ot.q0 + tile_r0 + row) * p.hq + ot.h) * D + col0;
      if (ot.n > 0) {
        const uint32_t t_o = tmem + lane_base + (t == 0 ? kColO0 : C::kColO1) + col0;
        w.wait(ptx::smem_u32(&bars->o_full[t]), (t == 0 ? o_uses0 : o_uses1) & 1u);
        if (w.aborted()) return;  // nothing valid to store; the barriers are left alone
        if (t == 0) ++o_uses0;
        else ++o_uses1;
        ptx::tc_fence_after();
        const bool by_tma = C::kOutBytes > 0 && tile_r0 + kTileM <= ot.lq;
#pragma unroll 1
        for (int ch = 0; ch < D / 64; ++ch) {
          uint32_t orr[32];
          ptx::tmem_ld32(t_o + ch * 32, orr);
          ptx::tmem_wait_ld();
          if (by_tma) {
            // every warp stores its own 32 rows (its TMEM lane quarter) with its own TMA store: no CTA-level
            // barrier, only the warp's lanes meet
            const uint32_t buf = sm_out + ((warp - 4) * 2 + (out_chunks & 1u)) * C::kOutWarpBytes;
            ++out_chunks;
            // the store that last read this buffer (two stores ago) is done with it
            if (lane == 0) ptx::bulk_wait_read<1>();
            __syncwarp();
            const uint32_t dst_row = buf + lane * 64;
            const uint32_t swz = (lane >> 1) & 3;  // 64-byte swizzle: 16-byte chunk index ^ address bits [7,9)
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              const uint32_t u0 = Pack<T>::pack(__uint_as_float(orr[q4 * 8 + 0]), __uint_as_float(orr[q4 * 8 + 1]));
              const uint32_t u1 = Pack<T>::pack(__uint_as_float(orr[q4 * 8 + 2]), __uint_as_float(orr[q4 * 8 + 3]));
              const uint32_t u2 = Pack<T>::pack(__uint_as_float(orr[q4 * 8 + 4]), __uint_as_float(orr[q4 * 8 + 5]));
              const uint32_t u3 = Pack<T>::pack(__uint_as_float(orr[q4 * 8 + 6]), __uint_as_float(orr[q4 * 8 + 7]));
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst_row + ((q4 ^ swz) << 4)), "r"(u0),
                           "r"(u1), "r"(u2), "r"(u3)
                           : "memory");
            }
            ptx::fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
              ptx::tma_store_3d(&tm_out, buf, col0 + ch * 32, ot.h,
                                static_cast<int>(ot.q0) + tile_r0 + (warp & 3) * 32);
              ptx::bulk_commit();
            }
          } else if (row_ok_t) {
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
        ptx::mbar_arrive(ptx::smem_u32(&bars->o_free[t]));
      } else if (row_ok_t) {
        uint4* dst = reinterpret_cast<uint4*>(orow);
#pragma unroll
        for (int q4 = 0; q4 < D / 16; ++q4) dst[q4] = make_uint4(0, 0, 0, 0);
      }
    };
    // the S tiles arrive in the order the MMA issuers alternate: tile 0 step j, tile 1 step j, tile 0 step j+1 ..
    uint32_t ring_base = 0;   // position of the current item's first K tile in the K/V ring (as the issuers count it)
    for (Item it;;) {
      if (!feed.next(it)) break;
      // Step j of Q tile t: S -> P for this thread's row and its group's 64 columns.  False after an abort.
      auto tile = [&](const int t, const int j, const bool row_ok, const RowBounds& rb, const long long bias_row) -> bool {
        const int tile_r0 = it.r0 + t * kTileM;
        const int c0 = j * kTileN;
        const bool full = tile_is_full(it.s, tile_r0, kTileM, c0, kTileN, p.mask_type, p.group);
        const uint32_t t_s = tmem + lane_base + (t == 0 ? kColS0 : kColS1);
        const uint32_t bar_p = ptx::smem_u32(&bars->p_full[t][0]);
        // kBias == 2: the 16-column slice of the sequence's last K tile that holds the sequence end (if any) is
        // added here, not by the tensor cores; the group that owns it fetches it now, before it waits for the scores
        const int rem = it.s.lk - c0;
        const int fix_n = (kBias == 2 && rem < kTileN) ? (rem & 15) : 0;
        const int fix_col = rem & ~15;
        const bool fix_here = fix_n > 0 && (fix_col >> 6) == grp;   // the same for every thread of the group
        uint32_t fixv[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
        if (kBias == 2 && fix_here && row_ok) {
          const T* src = static_cast<const T*>(p.bias) + bias_row + c0 + fix_col;
          if (c0 + fix_col + 16 <= p.maxk) {  // 32-byte aligned: the rows are 16-byte aligned and c0 + fix_col is a multiple of 16
            const uint4 u0 = __ldg(reinterpret_cast<const uint4*>(src));
            const uint4 u1 = __ldg(reinterpret_cast<const uint4*>(src) + 1);
            fixv[0] = u0.x, fixv[1] = u0.y, fixv[2] = u0.z, fixv[3] = u0.w;
            fixv[4] = u1.x, fixv[5] = u1.y, fixv[6] = u1.z, fixv[7] = u1.w;
          } else {
            const unsigned short* s16 = reinterpret_cast<const unsigned short*>(src);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const uint32_t lo = 2 * e < fix_n ? s16[2 * e] : 0u;
              const uint32_t hi = 2 * e + 1 < fix_n ? s16[2 * e + 1] : 0u;
              fixv[e] = lo | (hi << 16);
            }
          }
        }
        w.wait(ptx::smem_u32(&bars->s_full[t]), (t == 0 ? s_uses0 : s_uses1) & 1u);
        if (w.aborted()) return false;  // (the item feed then ends the outer loops)
        if (t == 0) ++s_uses0;
        else ++s_uses1;
        ptx::tc_fence_after();
        // A sequence's last K/V tile holds rows of the NEXT sequence behind the sequence end.  P is 0 there, but
        // 0 x NaN is not, so group 1 zeroes those V rows in shared memory before it hands P over (generic-proxy
        // stores, proxy fence, arrive: ordered before this tile's P.V).  The tile has landed: the issuer waited for
        // it before it issued the S tile whose completion this thread has just seen.
        // (The stores sit in a function of their own, not inlined: inlined, their mere presence cost the P loop 5 %
        // on batches that hardly ever run them.)
        if (grp == 1 && rem < kTileN)
          zero_v_rows(sm_ring + ((ring_base + 2u * j + 1u) % C::kStages) * C::kTileBytes + rem * 128,
                      (kTileN - rem) * 8, row, C::kHalves, C::kHalfBytes);
        const BiasRow br{p.bias, bias_row, row_ok, bias_vec_ok != 0, p.maxk, it.s.lk};
        if (kBias == 2 && fix_here) add_end_slice<T>(t_s + fix_col, fixv, fix_n);
        if (full)
          p_half<T, kBias, false>(t_s, grp, c0, br, rb, c_in, c_bias, p.scale, bar_p);
        else
          p_half<T, kBias, true>(t_s, grp, c0, br, rb, c_in, c_bias, p.scale, bar_p);
        return true;
      };
      if constexpr (kRolled) {
        // Round j serves step j of both Q tiles through ONE copy of the code (the loop over the tiles is not unrolled,
        // the output store has one call site); a tile that has finished its last step - or visits nothing at all -
        // stores its output in the round after it.
        for (int j = 0; j <= it.nmax; ++j) {
#pragma unroll 1
          for (int t = 0; t < 2; ++t) {
            const int nt = it.n(t);
            const int tile_r0 = it.r0 + t * kTileM;
            if (j == nt) store_o(t, OutTile{it.s.q0, it.s.lq, tile_r0, it.h, nt});
            if (j >= nt) continue;
            const int i_row = tile_r0 + row;
            const bool row_ok = i_row < it.s.lq;
            const RowBounds rb = row_bounds(it.s, row_ok ? i_row : it.s.lq - 1, p.mask_type, p.group);
            const long long bias_row = kBias != 0 ? static_cast<long long>(it.b) * p.bias_bstride +
                                                        (static_cast<long long>(it.h) * p.maxq + i_row) * p.maxk
                                                  : 0;
            if (!tile(t, j, row_ok, rb, bias_row)) break;
          }
          if (w.aborted()) break;
        }
      } else {
        int i_row[2];
        bool row_ok[2];
        RowBounds rb[2];
        long long bias_row[2];
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          i_row[t] = it.r0 + t * kTileM + row;
          row_ok[t] = i_row[t] < it.s.lq;
          rb[t] = row_bounds(it.s, row_ok[t] ? i_row[t] : it.s.lq - 1, p.mask_type, p.group);
          bias_row[t] = kBias != 0 ? static_cast<long long>(it.b) * p.bias_bstride +
                                         (static_cast<long long>(it.h) * p.maxq + i_row[t]) * p.maxk
                                   : 0;
        }
        // Tile 0 usually ends one K tile before tile 1: its output leaves while tile 1's last S tile is computed.
        // (Keeping tile 1's output back until the next item's first score tile has been served was measured too:
        // slower on every workload.)
        const OutTile out0{it.s.q0, it.s.lq, it.r0, it.h, it.n0};
        bool o0_stored = false;
        for (int j = 0; j < it.nmax; ++j) {
          if (!o0_stored && j >= it.n(0)) {
            store_o(0, out0);
            o0_stored = true;
          }
          bool ok = true;
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            if (j >= it.n(t) || !ok) continue;
            ok = tile(t, j, row_ok[t], rb[t], bias_row[t]);
          }
          if (!ok) break;
        }
        if (!o0_stored) store_o(0, out0);
        store_o(1, OutTile{it.s.q0, it.s.lq, it.r0 + kTileM, it.h, it.n1});
      }
      ring_base += 2u * it.nmax;
    }
    if (C::kOutBytes > 0 && lane == 0) ptx::bulk_wait<0>();  // this thread's TMA stores have completed
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

// 2-D view (max_seq_len_k, all rows) of the bias; box = 64 x 128, 128-byte swizzle.
bool make_bias_map(CUtensorMap* m, const KParams& p, int dtype) {
  auto fn = encode_fn();
  if (!fn) return false;
  const long long rows = static_cast<long long>(p.bias_bstride ? p.batch : 1) * p.hq * p.maxq;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(p.maxk), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(p.maxk) * 2};
  cuuint32_t box[2] = {64, static_cast<cuuint32_t>(kTileM)};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = dtype == HSTU_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                          : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  return fn(m, dt, 2, const_cast<void*>(p.bias), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 3-D view (dim, heads, tokens) of the output for the epilogue's TMA stores; box = 32 x 1 x 128, 64-byte swizzle.
bool make_out_map(CUtensorMap* m, const KParams& p, int dtype) {
  auto fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(p.dv), static_cast<cuuint64_t>(p.hq),
                        static_cast<cuuint64_t>(p.total_q > 0 ? p.total_q : 1)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(p.dv) * 2, static_cast<cuuint64_t>(p.dv) * 2 * p.hq};
  cuuint32_t box[3] = {32, 1, 32};  // one warp's rows
  cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapDataType dt = dtype == HSTU_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                          : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  return fn(m, dt, 3, p.out, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
            CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int D, typename T, int kBias, bool kRolled>
cudaError_t launch_inst(const KParams& p, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                        const CUtensorMap& mb, const CUtensorMap& mo, const CUtensorMap& mc, int bias_vec_ok, int grid,
                        cudaStream_t stream) {
  auto kern = hstu_tc_kernel<D, T, kBias, kRolled>;
  constexpr int smem = Cfg<D, kBias>::kSmemBytes;
  static_assert(smem <= 232448, "shared memory budget of one CTA exceeded");
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // start while the pre-pass is still running
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, p, mq, mk, mv, mb, mo, mc, bias_vec_ok);
}

}  // namespace


// 2-D view (cols, rows) of a contiguous 16-bit [rows, cols] matrix; box = 64 x box_rows (<= 256), 128-byte swizzle
// (a K-major operand tile of 64 K values).  Reads past either edge give zeros.
bool make_matrix_map_ld(CUtensorMap* m, const void* base, long long rows, long long cols, long long ld, int dtype,
                        int box_rows);
bool make_matrix_map(CUtensorMap* m, const void* base, long long rows, long long cols, int dtype, int box_rows) {
  return make_matrix_map_ld(m, base, rows, cols, cols, dtype, box_rows);
}
// The same with a row pitch of `ld` elements (a multiple of 8: TMA wants 16-byte strides); columns at or past `cols`
// read as zeros whatever the padding holds.
bool make_matrix_map_ld(CUtensorMap* m, const void* base, long long rows, long long cols, long long ld, int dtype,
                        int box_rows) {
  auto fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows > 0 ? rows : 1)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  cuuint32_t box[2] = {64, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = dtype == HSTU_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                          : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  return fn(m, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 2-D view (cols, rows) of a 16-bit [rows, cols] matrix with row pitch `ld` for TMA stores of 32-row boxes:
// box_cols = 32 with the 64-byte swizzle (one 64-byte row piece per row), or 16 without swizzle.
bool make_store_map(CUtensorMap* m, void* base, long long rows, long long cols, long long ld, int dtype, int box_cols) {
  auto fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols > 0 ? cols : 1), static_cast<cuuint64_t>(rows > 0 ? rows : 1)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), 32};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = dtype == HSTU_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                          : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  return fn(m, dt, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            box_cols == 32 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The bias tile map (64 x 128 boxes, 128-byte swizzle) for other translation units (the backward kernels).
bool make_bias_tile_map(CUtensorMap* m, const KParams& p, int dtype) { return make_bias_map(m, p, dtype); }

// The q / k / v tile map for other translation units (the backward kernels).
bool make_tile_map(CUtensorMap* m, const void* base, long long tokens, int heads, int dim, int dtype) {
  return make_map(m, base, tokens, heads, dim, dtype);
}

bool tc_supported(const KParams& p, int dtype) {
  if (dtype != HSTU_DTYPE_BF16 && dtype != HSTU_DTYPE_FP16) return false;
  if (p.dqk != p.dv || (p.dqk != 64 && p.dqk != 128)) return false;
  // a custom mask takes the operand slot of the bias (plain loads), so the two together run on the generic kernel
  if (p.mask_type == HSTU_MASK_CUSTOM && (!p.mask || p.bias)) return false;
  if (p.hq > 0xffff || p.total_q > 0x7fffff00ll || p.total_k > 0x7fffff00ll) return false;
  const uintptr_t align = reinterpret_cast<uintptr_t>(p.q) | reinterpret_cast<uintptr_t>(p.k) |
                          reinterpret_cast<uintptr_t>(p.v) | reinterpret_cast<uintptr_t>(p.out);
  return (align & 15u) == 0;
}

// Returns cudaSuccess, a CUDA error, or cudaErrorNotSupported when the tensor maps could not be encoded.
cudaError_t launch_tc(const KParams& p_in, int dtype, int num_sms, cudaStream_t stream) {
  KParams p = p_in;
  const bool custom_mask = p.mask_type == HSTU_MASK_CUSTOM;
  if (custom_mask) {  // the kernel reads the mask [B, Hq, maxq, maxk] through its bias operand path (mode 3)
    p.bias = p.mask;
    p.bias_bstride = static_cast<long long>(p.hq) * p.maxq * p.maxk;
  }
  CUtensorMap mq, mk, mv;
  if (!make_map(&mq, p.q, p.total_q, p.hq, p.dqk, dtype) || !make_map(&mk, p.k, p.total_k, p.hk, p.dqk, dtype) ||
      !make_map(&mv, p.v, p.total_k, p.hk, p.dv, dtype))
    return cudaErrorNotSupported;
  long long grid = p.item_capacity < num_sms ? p.item_capacity : num_sms;
  if (grid < 1) grid = 1;
  const int g = static_cast<int>(grid);
  const int vec_ok = p.bias && (p.maxk % 8 == 0) && (p.bias_bstride % 8 == 0) &&
                     (reinterpret_cast<uintptr_t>(p.bias) & 15u) == 0;
  // bias staging by TMA needs 16-byte aligned rows and batch blocks laid out back to back (or one shared block);
  // the tensor cores then add the tile to S, which gives alpha * (S + bias) only
  int bias_mode = p.bias ? 1 : 0;
  CUtensorMap mb = mq;
  if (custom_mask) bias_mode = 3;
  if (!custom_mask && p.bias && vec_ok && !(p.flags & HSTU_FLAG_ALPHA_BEFORE_BIAS) &&
      (p.bias_bstride == 0 || p.bias_bstride == static_cast<long long>(p.hq) * p.maxq * p.maxk) &&
      make_bias_map(&mb, p, dtype))
    bias_mode = 2;
  CUtensorMap mo;
  if (!make_out_map(&mo, p, dtype)) return cudaErrorNotSupported;
  // hstu_paged with direct page reads: the cache as one K / V tensor of num_pages * 2 * 128 rows
  CUtensorMap mc = mk;
  if (p.paged_direct && !make_map(&mc, p.kv_cache, p.num_pages * 2 * kTileN, p.hk, p.dqk, dtype)) return cudaErrorNotSupported;
  // Which form of the P/O code (see the kernel): the rolled one for batches of short sequences, where every item
  // walks through every path of that code, the unrolled one where long sequences keep it in one path.  Measured
  // (B200, in-process A/B): mean length 270 with a bias - 21 % time rolled, without - 10 %; mean 640 with a bias - 4 %,
  // without + 3 %; mean 2400 + 6 %.
  const long long mean_len = p.batch > 0 ? p.total_q / p.batch : 0;
  const bool rolled = mean_len < 512 || (bias_mode == 2 && mean_len < 1024);
#define HSTU_TC_CASE(DD, TT)                                                                                       \
  if (rolled && bias_mode == 2) return launch_inst<DD, TT, 2, true>(p, mq, mk, mv, mb, mo, mc, vec_ok, g, stream);  \
  if (rolled && bias_mode == 0) return launch_inst<DD, TT, 0, true>(p, mq, mk, mv, mb, mo, mc, vec_ok, g, stream);  \
  return bias_mode == 3   ? launch_inst<DD, TT, 3, false>(p, mq, mk, mv, mb, mo, mc, vec_ok, g, stream)             \
         : bias_mode == 2 ? launch_inst<DD, TT, 2, false>(p, mq, mk, mv, mb, mo, mc, vec_ok, g, stream)             \
         : bias_mode == 1 ? launch_inst<DD, TT, 1, false>(p, mq, mk, mv, mb, mo, mc, vec_ok, g, stream)             \
                          : launch_inst<DD, TT, 0, false>(p, mq, mk, mv, mb, mo, mc, vec_ok, g, stream)
  if (dtype == HSTU_DTYPE_BF16) {
    if (p.dqk == 128) { HSTU_TC_CASE(128, __nv_bfloat16); }
    HSTU_TC_CASE(64, __nv_bfloat16);
  }
  if (p.dqk == 128) { HSTU_TC_CASE(128, __half); }
  HSTU_TC_CASE(64, __half);
#undef HSTU_TC_CASE
}

}  // namespace hstu
