// HSTU jagged backward on Blackwell tensor cores (tcgen05 + TMEM + TMA), bf16 / fp16, Dqk = Dv in {64, 128},
// mask tril / none, the reference's order x = alpha (S + bias).  Everything else runs on hstu_bwd_generic.cu.
//
// One kernel template, launched twice with one persistent CTA per SM (the tiles of a pass come from a list the
// pre-pass wrote - only tiles that exist - through a counter in the workspace; the producer thread draws them and
// runs ahead of the other warps across tile boundaries), no atomics on the data (bitwise reproducible):
//
//   dQ pass   (kDKV = false)  one tile of work per (sequence, query head, 128-row q-tile).  Resident: Q tile, dO tile.
//             Streamed over the visible K tiles j: K_j, V_j.   S = Q.K_j^T, dP = dO.V_j^T  ->  dS  ->  dQ += dS.K_j.
//             dS (rounded to the input type) is also this tile of d_bias; the CTA writes the zeros of its d_bias
//             rows right of the visited tiles, so d_bias needs no clearing.
//   dK/dV pass (kDKV = true)  one tile of work per (sequence, kv head, 128-key tile).  Resident: K tile, V tile.
//             Streamed over the query heads of the group and the q-tiles i that see the keys: Q_i, dO_i.
//             S^T = K.Q_i^T, dP^T = V.dO_i^T  ->  P^T, dS^T  ->  dV += P^T.dO_i, dK += dS^T.Q_i.
//
// Both passes are the same pipeline: two "T" products (SS form, both operands K-major from shared memory) into
// TMEM, an element-wise stage by 256 threads (thread = TMEM lane = row, two groups share the columns) that writes
// the 16-bit results in place over the fp32 ones, and accumulate products (A operand = those results in TMEM, B =
// the streamed tile again, read N-major).  TMEM: T1, T2 (128 columns each), Acc1, Acc2 (D columns each).
// A step's element-wise stage and the MMAs do not overlap yet (one chain per CTA); the element-wise math follows
// hstu_backward_v1/op_kernel/vector_score.h:159-209 with P and dS rounded to the input type.
//
// Every mbarrier wait is bounded; a wait that gives up sets HSTU_ST_PIPE_TIMEOUT and a CTA-wide abort flag, the
// kernel still drains its TMA loads, frees its tensor memory and returns.
#include <cuda.h>

#include <type_traits>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "hstu_common.cuh"
#include "ptx_sm100.cuh"

namespace hstu {

bool make_tile_map(CUtensorMap* m, const void* base, long long tokens, int heads, int dim, int dtype);
bool make_bias_tile_map(CUtensorMap* m, const KParams& p, int dtype);

namespace {

constexpr int kBwdThreads = 384;
constexpr long long kBwdWaitLimit = 2000000000ll;  // ~1 s of SM clock

template <typename T> struct BPack;
template <> struct BPack<__nv_bfloat16> {
  static constexpr int kFormat = 1;
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ float one(const void* p, long long i) {
    return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
  }
};
template <> struct BPack<__half> {
  static constexpr int kFormat = 0;
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ float one(const void* p, long long i) {
    return __half2float(static_cast<const __half*>(p)[i]);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) {
    return __half22float2(*reinterpret_cast<__half2*>(&u));
  }
};

struct BwdBars {
  uint64_t a_full;             // the resident pair has landed
  uint64_t b_full[2], b_free[2];
  uint64_t t_full;             // T1 and T2 of the current step are complete
  uint64_t u_full[2];          // their 16-bit replacements are written: first / second 32 values of each 64 (256 arrivals)
  uint64_t acc_full;           // every accumulate MMA is complete
  uint64_t bias_full, bias_free;   // dK/dV pass with a staged bias tile: landed / read by all 256 element-wise threads
  uint32_t tmem_base;
  int abort_flag;
  // the tiles this CTA has drawn, two slots used in turn:
  int item[2];                 // -1: no tile left; else the tile every thread of the CTA works on:
  int item_seq[2];             //   its sequence,
  uint32_t item_head_tile[2];  //   head << 16 | tile index (the pre-pass's list entry)
  uint64_t item_full[2];       // slot written by the producer thread / read by every other warp (11 arrivals)
  uint64_t item_free[2];
};

struct BwdWaiter {
  int* abort_flag;
  uint32_t* status;
  __device__ __forceinline__ void wait(uint32_t bar, uint32_t parity) const {
    if (ptx::mbar_try_wait(bar, parity)) return;
    if (*reinterpret_cast<volatile int*>(abort_flag)) return;
    const long long t0 = clock64();
    unsigned spins = 0;
    while (!ptx::mbar_try_wait(bar, parity)) {
      if ((++spins & 0x3ffu) == 0) {
        if (*reinterpret_cast<volatile int*>(abort_flag)) return;
        if (clock64() - t0 > kBwdWaitLimit) {
          *reinterpret_cast<volatile int*>(abort_flag) = 1;
          atomicOr(status, static_cast<uint32_t>(HSTU_ST_PIPE_TIMEOUT));
          return;
        }
      }
    }
  }
};

// The steps of one CTA, in the order every role walks them.  f(stream_head, stream_row0, query_head):
//   dQ pass:    stream = K/V tiles of kv head hk, rows stream_row0 = j * 128 (keys);   query_head = h
//   dK/dV pass: stream = Q/dO tiles of query head h, rows stream_row0 = r0 (queries);  query_head = h
template <bool kDKV, typename F>
__device__ __forceinline__ void for_each_step(const KParams& p, const SeqInfo& s, int tile0, int head, F&& f) {
  if (!kDKV) {
    const int n = kv_tiles_for_rows(s, tile0, kTileM, p.mask_type, kTileN);
    for (int j = 0; j < n; ++j) f(head / p.gqa_ratio, j * kTileN, head);
  } else {
    const int ktile = tile0 / kTileN;
    for (int hh = 0; hh < p.gqa_ratio; ++hh)
      for (int r0 = 0; r0 < s.lq; r0 += kTileM)
        if (kv_tiles_for_rows(s, r0, kTileM, p.mask_type, kTileN) > ktile) f(head * p.gqa_ratio + hh, r0, head * p.gqa_ratio + hh);
  }
}

// Bit e set <=> column j0 + e is visible to the row described by rb (columns j0 .. j0 + 31).
__device__ __forceinline__ uint32_t low_bits(int n) {  // n lowest bits set, n clamped to [0, 32]
  return n <= 0 ? 0u : (n >= 32 ? 0xffffffffu : ((1u << n) - 1u));
}
__device__ __forceinline__ uint32_t visible_bits(const RowBounds& rb, int j0) {
  return low_bits(rb.lim1 - j0) | (low_bits(rb.hi2 + 1 - j0) & ~low_bits(rb.lo2 - j0));
}

// P and dS of two neighbouring elements from s = q.k and dp = dO.v (vector_score.h:175-197) on the packed f32x2
// pipe:  x = alpha (s + bias),  sg = sigmoid(x),  P = x sg scale,  dS = dp scale alpha sg (1 + x - x sg).
// kSelect: zero the elements whose bit in `vis` (bits 0 and 1) is clear - a select, never a multiply: scores of
// rows past a sequence end may be Inf or NaN.
template <typename T, bool kBiasOn, bool kSelect>
__device__ __forceinline__ void score_grad2(float2 s, float2 dp, float2 bias, float alpha, float scale, uint32_t vis,
                                            uint32_t& p_out, uint32_t& ds_out) {
  const float2 al = make_float2(alpha, alpha);
  float2 x = kBiasOn ? __fmul2_rn(__fadd2_rn(s, bias), al) : __fmul2_rn(s, al);
  float2 sg;
  if (BPack<T>::kFormat == 0) {
    const float2 ny = __fmul2_rn(x, make_float2(-1.4426950408889634f, -1.4426950408889634f));
    const float2 d = __fadd2_rn(make_float2(ptx::ex2_approx(ny.x), ptx::ex2_approx(ny.y)), make_float2(1.f, 1.f));
    sg = make_float2(ptx::rcp_approx(d.x), ptx::rcp_approx(d.y));
  } else {
    const float2 hx = __fmul2_rn(x, make_float2(0.5f, 0.5f));
    sg = __ffma2_rn(make_float2(ptx::tanh_approx(hx.x), ptx::tanh_approx(hx.y)), make_float2(0.5f, 0.5f),
                    make_float2(0.5f, 0.5f));
  }
  const float2 xs = __fmul2_rn(x, sg);
  float2 pv = __fmul2_rn(xs, make_float2(scale, scale));
  const float2 wgt = __ffma2_rn(xs, make_float2(-1.f, -1.f), __fadd2_rn(x, make_float2(1.f, 1.f)));
  const float sa = scale * alpha;
  float2 ds = __fmul2_rn(__fmul2_rn(__fmul2_rn(dp, make_float2(sa, sa)), sg), wgt);
  if (kSelect) {
    pv.x = (vis & 1u) ? pv.x : 0.f;
    pv.y = (vis & 2u) ? pv.y : 0.f;
    ds.x = (vis & 1u) ? ds.x : 0.f;
    ds.y = (vis & 2u) ? ds.y : 0.f;
  }
  p_out = BPack<T>::pack(pv.x, pv.y);
  ds_out = BPack<T>::pack(ds.x, ds.y);
}

// kStaged (dK/dV pass with a bias that TMA can tile): a kernel of its own - the same code merely present in the
// bias-free kernel cost that one 4 %.
template <int D, typename T, bool kDKV, bool kStaged>
__global__ void __launch_bounds__(kBwdThreads, 1)
hstu_bwd_tc_kernel(const BwdParams bp, const __grid_constant__ CUtensorMap tm_a1,
                   const __grid_constant__ CUtensorMap tm_a2, const __grid_constant__ CUtensorMap tm_b1,
                   const __grid_constant__ CUtensorMap tm_b2, const __grid_constant__ CUtensorMap tm_bias) {
  constexpr int kHalves = D / 64;
  constexpr int kHalfBytes = kTileM * 128;
  constexpr int kTileBytes = kHalves * kHalfBytes;
  constexpr uint32_t kColT1 = 0, kColT2 = 128, kColAcc1 = 256, kColAcc2 = 256 + D;
  // dQ pass: Acc1 is not used, so T1 (the scores) has a second buffer in the free columns and alternates by step:
  // the scores of step c + 1 are computed while the element-wise stage of step c still runs, and only the dP
  // product (whose buffer the 16-bit dS of step c occupies until its accumulate products are done) stays behind them.
  constexpr uint32_t kColT1b = kDKV ? kColT1 : (D == 128 ? 256u : 384u);
  const KParams& p = bp.f;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  const uint32_t sm_a = base;                        // A1, A2
  const uint32_t sm_b = base + 2 * kTileBytes;       // ring: stage x {B1, B2}
  // With a bias that TMA can tile: the 128 x 128 bias tile of a step (rows = queries, columns = keys), staged by TMA.
  // dK/dV pass: a thread owns a key and reads its column, one value per query, from shared memory instead of 32
  // strided 2-byte loads from global memory per chunk; dQ pass: a thread owns a query and reads 64 bytes of its row
  const uint32_t sm_bias = base + 6 * kTileBytes;    // 2 boxes of 128 rows x 128 bytes, 128-byte swizzle
  constexpr bool staged = kStaged;
  BwdBars* bars = reinterpret_cast<BwdBars*>(base_ptr + 6 * kTileBytes + (staged ? 2 * kTileM * 128 : 0));
  const BwdWaiter w{&bars->abort_flag, p.ws_header};

  // The two passes do not depend on each other, only on the pre-pass before them.  The dK/dV pass is launched with
  // programmatic stream serialization behind the dQ pass, which lets it go at once: its CTAs take the SMs as the dQ
  // pass's CTAs leave them, so the end of the one pass (CTAs running dry) overlaps the start of the other.  The dK/dV
  // pass waits for the dQ pass's completion only at its very end, so that whatever follows in the stream finds both
  // complete.  The dQ pass itself is launched the same way behind the pre-pass (its set-up overlaps it): one thread
  // waits for the pre-pass to complete before the barrier that ends the set-up, and only behind that barrier do the
  // threads release the dK/dV pass - so the tile lists are complete before either pass reads them.
  if (tid == 0) {
    ptx::prefetch_tensormap(&tm_a1);
    ptx::prefetch_tensormap(&tm_a2);
    ptx::prefetch_tensormap(&tm_b1);
    ptx::prefetch_tensormap(&tm_b2);
    ptx::mbar_init(ptx::smem_u32(&bars->a_full), 1);
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(ptx::smem_u32(&bars->b_full[i]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->b_free[i]), 1);
    }
    ptx::mbar_init(ptx::smem_u32(&bars->t_full), 1);
    ptx::mbar_init(ptx::smem_u32(&bars->u_full[0]), 2 * kTileM);
    ptx::mbar_init(ptx::smem_u32(&bars->u_full[1]), 2 * kTileM);
    ptx::mbar_init(ptx::smem_u32(&bars->acc_full), 1);
    ptx::mbar_init(ptx::smem_u32(&bars->bias_full), 1);
    ptx::mbar_init(ptx::smem_u32(&bars->bias_free), 2 * kTileM);
    for (int sl = 0; sl < 2; ++sl) {
      ptx::mbar_init(ptx::smem_u32(&bars->item_full[sl]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->item_free[sl]), 11);
    }
    if (staged) ptx::prefetch_tensormap(&tm_bias);
    bars->abort_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == 2) {
    ptx::tmem_alloc(ptx::smem_u32(&bars->tmem_base), 512);
    ptx::tmem_relinquish();
  }
  if (!kDKV && tid == 0) asm volatile("griddepcontrol.wait;" ::: "memory");
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  if (!kDKV) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);

  // Persistent CTAs take tiles from the pre-pass's list of this pass through a counter in the workspace (zeroed by
  // the pre-pass).  Order of the list: all tiles of a (sequence, head) are neighbours, so the CTAs that run together
  // stream the same K/V (Q/dO) rows out of L2, and the tiles with the most steps of a sequence come first (dQ pass:
  // its last q-tile; dK/dV pass: its first keys).
  const int heads = kDKV ? p.hk : p.hq;
  const uint32_t* list = p.items + (kDKV ? 2 * p.bwd_cap_q : 0);
  uint32_t* counter = p.ws_header + (kDKV ? 3 : 2);
  uint32_t cnt = 0;          // steps so far (every role counts them alike): barrier phases run on across tiles
  uint32_t tiles_done = 0;   // tiles so far: phase of a_full / acc_full
  // Tiles are drawn by the producer thread, which runs ahead of the other warps across tile boundaries: when it has
  // requested the last loads of a tile it draws the next one, publishes it in one of two slots (item_full / item_free)
  // and - once the MMAs of the current tile are complete (acc_full: the resident pair's buffer is free) - requests
  // the next tile's loads, so that the draw (an atomic and a dependent load of the list entry) and the first loads
  // overlap the current tile's epilogue.  The draw comes a step or two before the current tile's end (the ring of
  // streamed tiles has two stages), which costs no balance worth the name; drawing at the START of the current tile
  // did (a tile drawn early is a tile that cannot go to a CTA that has run dry: - 7 % on a batch with four tiles per
  // CTA).
  // The other warps meet at a named barrier at the end of a tile (the producer warp takes no part in it).
  constexpr int kConsumers = kBwdThreads - 32;
  if (warp == 0) {
    if (lane == 0) {
      // ---------------------------------------------------------------- TMA producer (and tile drawer)
      const unsigned n_list = p.ws_header[kDKV ? 4 : 1];
      uint32_t draws = 0;
      for (;;) {
        const uint32_t slot = draws & 1u;
        // the slot's last tile (two draws ago) has been read by every warp
        if (draws >= 2) w.wait(ptx::smem_u32(&bars->item_free[slot]), ((draws >> 1) - 1u) & 1u);
        int found = -1, b = 0;
        uint32_t head_tile = 0;
        if (!*reinterpret_cast<volatile int*>(&bars->abort_flag)) {
          const unsigned idx = atomicAdd(counter, 1u);
          if (idx < n_list) {
            const uint2 e = *reinterpret_cast<const uint2*>(list + 2ull * idx);
            b = static_cast<int>(e.x);
            head_tile = e.y;
            found = 0;
          }
        }
        bars->item_seq[slot] = b;
        bars->item_head_tile[slot] = head_tile;
        bars->item[slot] = found;
        ptx::mbar_arrive(ptx::smem_u32(&bars->item_full[slot]));
        ++draws;
        if (found < 0) break;
        const int head = static_cast<int>(head_tile >> 16);
        const int tile0 = static_cast<int>(head_tile & 0xffffu) * kTileM;
        const SeqInfo s = load_seq(p, b);
        if (tile0 >= (kDKV ? s.lk : s.lq)) continue;   // (a q-tile past the sequence end: nothing to load)
        const long long a_row = (kDKV ? s.k0 : s.q0) + tile0;
        const long long b_row0 = kDKV ? s.q0 : s.k0;
        const int a_head = head;
        // the resident pair's buffer is free once the MMAs of the tile before are complete
        if (tiles_done > 0) w.wait(ptx::smem_u32(&bars->acc_full), (tiles_done - 1u) & 1u);
        if (*reinterpret_cast<volatile int*>(&bars->abort_flag)) break;
        const uint32_t afull = ptx::smem_u32(&bars->a_full);
        ptx::mbar_expect_tx(afull, 2 * kTileBytes);
#pragma unroll
        for (int hf = 0; hf < kHalves; ++hf) {
          ptx::tma_load_3d(sm_a + hf * kHalfBytes, &tm_a1, afull, hf * 64, a_head, static_cast<int>(a_row));
          ptx::tma_load_3d(sm_a + kTileBytes + hf * kHalfBytes, &tm_a2, afull, hf * 64, a_head, static_cast<int>(a_row));
        }
        for_each_step<kDKV>(p, s, tile0, head, [&](int sh, int srow0, int qh) {
          const uint32_t stage = cnt & 1u;
          const uint32_t full = ptx::smem_u32(&bars->b_full[stage]);
          if (staged) {
            // the bias tile of this step, once every element-wise thread has read the last one
            w.wait(ptx::smem_u32(&bars->bias_free), (cnt & 1u) ^ 1u);
            const uint32_t bfull = ptx::smem_u32(&bars->bias_full);
            ptx::mbar_expect_tx(bfull, 2 * kTileM * 128);
            // rows = queries, columns = keys: the streamed rows are queries in the dK/dV pass and keys in the dQ pass
            const int brow = (b * p.hq + qh) * p.maxq + (kDKV ? srow0 : tile0);
            const int bcol0 = kDKV ? tile0 : srow0;
#pragma unroll
            for (int hf = 0; hf < 2; ++hf)
              ptx::tma_load_2d(sm_bias + hf * (kTileM * 128), &tm_bias, bfull, bcol0 + hf * 64, brow);
          }
          w.wait(ptx::smem_u32(&bars->b_free[stage]), ((cnt >> 1) & 1u) ^ 1u);
          ptx::mbar_expect_tx(full, 2 * kTileBytes);
          const int row = static_cast<int>(b_row0) + srow0;
#pragma unroll
          for (int hf = 0; hf < kHalves; ++hf) {
            ptx::tma_load_3d(sm_b + stage * 2 * kTileBytes + hf * kHalfBytes, &tm_b1, full, hf * 64, sh, row);
            ptx::tma_load_3d(sm_b + stage * 2 * kTileBytes + kTileBytes + hf * kHalfBytes, &tm_b2, full, hf * 64, sh, row);
          }
          ++cnt;
        });
        ++tiles_done;
      }
      if (tiles_done > 0) {
        // drain (matters only after an abort: otherwise the consumers have waited for every load)
        for (int spin = 0; spin < (1 << 22) && !ptx::mbar_try_wait(ptx::smem_u32(&bars->a_full), (tiles_done - 1) & 1u); ++spin) {}
        for (uint32_t back = 0; back < 2 && back < cnt; ++back) {
          const uint32_t c = cnt - 1 - back;
          const uint32_t bar = ptx::smem_u32(&bars->b_full[c & 1u]);
          for (int spin = 0; spin < (1 << 22) && !ptx::mbar_try_wait(bar, (c >> 1) & 1u); ++spin) {}
        }
        if (staged && cnt > 0)
          for (int spin = 0; spin < (1 << 22) && !ptx::mbar_try_wait(ptx::smem_u32(&bars->bias_full), (cnt - 1) & 1u); ++spin) {}
      }
    }
  } else {
  uint32_t draws = 0;        // tiles read so far (every thread of these warps counts alike)
  for (;;) {
  const uint32_t slot = draws & 1u;
  w.wait(ptx::smem_u32(&bars->item_full[slot]), (draws >> 1) & 1u);
  const int found = *reinterpret_cast<volatile int*>(&bars->item[slot]);
  const int b = *reinterpret_cast<volatile int*>(&bars->item_seq[slot]);
  const uint32_t head_tile = *reinterpret_cast<volatile uint32_t*>(&bars->item_head_tile[slot]);
  __syncwarp();
  if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&bars->item_free[slot]));
  ++draws;
  if (found < 0 || *reinterpret_cast<volatile int*>(&bars->abort_flag)) break;
  const int head = static_cast<int>(head_tile >> 16);    // dQ pass: query head; dK/dV pass: kv head
  const int tile0 = static_cast<int>(head_tile & 0xffffu) * kTileM;   // first query row (dQ) / first key (dK/dV)
  const SeqInfo s = load_seq(p, b);
  const int len = kDKV ? s.lk : s.lq;
  const uint32_t first = cnt;

  if (!kDKV && bp.dbias) {
    // zeros of this tile's d_bias rows right of the visited K tiles (all columns when nothing is visited)
    const int first_col = kv_tiles_for_rows(s, tile0, kTileM, p.mask_type, kTileN) * kTileN;
    const int width = p.maxk - first_col;
    T* dbias = static_cast<T*>(bp.dbias);
    const long long brow0 = (static_cast<long long>(b) * p.hq + head) * p.maxq;
    if (width > 0) {
      if (p.maxk % 8 == 0 && (reinterpret_cast<uintptr_t>(bp.dbias) & 15u) == 0) {
        // 16-byte stores: first_col is a multiple of 128, so every row piece starts on a 16-byte boundary
        const int pieces = width / 8;
        for (int idx = tid - 32; idx < kTileM * pieces; idx += kConsumers) {
          const int r = idx / pieces, c = idx - r * pieces;
          if (tile0 + r < p.maxq)
            *reinterpret_cast<uint4*>(dbias + (brow0 + tile0 + r) * p.maxk + first_col + 8 * c) = make_uint4(0, 0, 0, 0);
        }
      } else {
        for (int idx = tid - 32; idx < kTileM * width; idx += kConsumers) {
          const int r = idx / width, c = idx - r * width;
          if (tile0 + r < p.maxq) dbias[(brow0 + tile0 + r) * p.maxk + first_col + c] = T(0.f);
        }
      }
    }
  }
  if (tile0 >= len) {   // uniform over these warps
    ptx::named_bar_sync(1, kConsumers);
    continue;
  }

  if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // (an elected thread, not `lane == 0`: the compiler then keeps descriptors and barrier addresses in uniform registers)
    if (ptx::elect_one()) {
      constexpr uint32_t idesc_t = ptx::umma_idesc_f16(BPack<T>::kFormat, kTileM, kTileN, 0);
      constexpr uint32_t idesc_acc = ptx::umma_idesc_f16(BPack<T>::kFormat, kTileM, D, 1);
      constexpr uint64_t kDescK = ptx::umma_desc_sw128_hi(16, 1024);           // K-major tiles
      constexpr uint64_t kDescN = ptx::umma_desc_sw128_hi(kHalfBytes, 1024);   // the same tiles read N-major
      const uint64_t a1 = kDescK | static_cast<uint64_t>(sm_a >> 4);
      const uint64_t a2 = kDescK | static_cast<uint64_t>((sm_a + kTileBytes) >> 4);
      // accumulate products of step c (its U1 / U2 are written): Acc1 += U1.B2, Acc2 += U2.B1
      // The element-wise groups hand their results over in two parts (values 0..31 and 64..95 of a tile row, then
      // the rest), so the first half of these MMAs runs while the second part is still being computed.
      auto accumulate = [&](uint32_t c, auto&& between) {
        const uint32_t stage = c & 1u;
        // dQ pass: the 16-bit dS of step c sits in the score buffer of step c (dead once the scores are read), so
        // the dP buffer is free for the next step as soon as the element-wise stage has read it
        const uint32_t col_u2 = kDKV ? kColT2 : ((c & 1u) ? kColT1b : kColT1);
        const uint64_t b1n = kDescN | static_cast<uint64_t>((sm_b + stage * 2 * kTileBytes) >> 4);
        const uint64_t b2n = kDescN | static_cast<uint64_t>((sm_b + stage * 2 * kTileBytes + kTileBytes) >> 4);
        auto part = [&](int ks, uint32_t acc) {
          const uint32_t ucol = (ks >> 2) * 64 + (ks & 3) * 8;
          const uint64_t off = static_cast<uint64_t>((ks * 2048) >> 4);
          if (kDKV) ptx::mma_ts(tmem + kColAcc1, tmem + kColT1 + ucol, b2n + off, idesc_acc, acc);
          ptx::mma_ts(tmem + kColAcc2, tmem + col_u2 + ucol, b1n + off, idesc_acc, acc);
        };
        w.wait(ptx::smem_u32(&bars->u_full[0]), c & 1u);
        ptx::tc_fence_after();
        part(0, c > first ? 1u : 0u);
        part(1, 1u);
        part(4, 1u);
        part(5, 1u);
        w.wait(ptx::smem_u32(&bars->u_full[1]), c & 1u);
        ptx::tc_fence_after();
        between();   // (dQ pass: the dP product of the next step - its buffer has been read completely by now)
        part(2, 1u);
        part(3, 1u);
        part(6, 1u);
        part(7, 1u);
        ptx::mma_commit(ptx::smem_u32(&bars->b_free[stage]));
      };
      w.wait(ptx::smem_u32(&bars->a_full), tiles_done & 1u);
      for_each_step<kDKV>(p, s, tile0, head, [&](int, int, int) {
        // dK/dV pass: the accumulate products of the last step must precede this step's T products (they overwrite
        // U1 / U2).  dQ pass: only U2 is in use, T1 goes to its other buffer first.
        if (kDKV && cnt > first) accumulate(cnt - 1, [] {});
        const uint32_t stage = cnt & 1u;
        w.wait(ptx::smem_u32(&bars->b_full[stage]), (cnt >> 1) & 1u);
        ptx::tc_fence_after();
        const uint64_t b1 = kDescK | static_cast<uint64_t>((sm_b + stage * 2 * kTileBytes) >> 4);
        const uint64_t b2 = kDescK | static_cast<uint64_t>((sm_b + stage * 2 * kTileBytes + kTileBytes) >> 4);
        const uint32_t col_t1 = (cnt & 1u) ? kColT1b : kColT1;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint64_t off = static_cast<uint64_t>(((ks >> 2) * kHalfBytes + (ks & 3) * 32) >> 4);
          ptx::mma_ss(tmem + col_t1, a1 + off, b1 + off, idesc_t, ks > 0 ? 1u : 0u);
        }
        auto t2_product = [&]() {
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const uint64_t off = static_cast<uint64_t>(((ks >> 2) * kHalfBytes + (ks & 3) * 32) >> 4);
            ptx::mma_ss(tmem + kColT2, a2 + off, b2 + off, idesc_t, ks > 0 ? 1u : 0u);
          }
          ptx::mma_commit(ptx::smem_u32(&bars->t_full));
        };
        // dQ pass: first half of the last step's accumulate products, this step's dP product, then the second half
        if (!kDKV && cnt > first) accumulate(cnt - 1, t2_product);
        else t2_product();
        ++cnt;
      });
      if (cnt > first) accumulate(cnt - 1, [] {});
      ptx::mma_commit(ptx::smem_u32(&bars->acc_full));
      w.wait(ptx::smem_u32(&bars->acc_full), tiles_done & 1u);   // all MMAs and their barrier arrivals are done before teardown
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ element-wise groups (thread = row)
    // Group g owns the columns [64g, 64g + 64) of T1 / T2 and the columns [g D/2, (g+1) D/2) of the accumulators.
    // The 16-bit results replace the fp32 values inside the group's own column range (values 0..63 of a tile
    // row at columns 0..31, values 64..127 at columns 64..95), so no group overwrites what the other still reads.
    const int grp = (warp - 4) >> 2;
    const int row = (tid - 128) & 127;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int mine = tile0 + row;                 // this thread's query row (dQ pass) / key (dK/dV pass)
    const bool mine_ok = mine < len;
    const RowBounds rb_mine = row_bounds(s, (mine_ok || kDKV) ? mine : s.lq - 1, p.mask_type, p.group);  // dQ pass
    T* dbias = static_cast<T*>(bp.dbias);
    const bool dbias_vec = dbias && (p.maxk % 8 == 0) && (reinterpret_cast<uintptr_t>(bp.dbias) & 15u) == 0;
    const bool bias_vec = p.bias && (p.maxk % 8 == 0) && (p.bias_bstride % 8 == 0) &&
                          (reinterpret_cast<uintptr_t>(p.bias) & 15u) == 0;
    // The dK/dV pass holds the score tile transposed (thread = key), so it needs the queries that see key `mine`:
    // history queries [c_lo, hq_end) by the causal rule, context rows [0, ctx_hi) for a history key, and the target
    // queries [t_lo, t_hi) - every target for a history key, else the targets of the key's own group from the key's
    // own position on (the transpose of row_bounds(); no mask: every query).
    const bool grouped = p.mask_type == HSTU_MASK_TRIL && s.tgt > 0 && p.group > 0;
    const int hq_end = grouped ? s.lq - s.tgt : s.lq;
    int c_lo = 0, ctx_hi = 0, t_lo = 0, t_hi = 0;
    if (kDKV && p.mask_type == HSTU_MASK_TRIL) {
      const int hist = s.lk - s.tgt;
      c_lo = mine - (s.lk - s.lq);
      if (s.ctx > 0 && mine < hist) ctx_hi = s.ctx < hq_end ? s.ctx : hq_end;
      if (grouped) {
        if (mine < hist) {
          t_lo = hq_end;
          t_hi = s.lq;
        } else {
          const int tj = mine - hist;
          const int gend = (tj / p.group + 1) * p.group;
          t_lo = hq_end + tj;
          t_hi = hq_end + (gend < s.tgt ? gend : s.tgt);
        }
      }
    }
    for_each_step<kDKV>(p, s, tile0, head, [&](int, int srow0, int qh) {
      w.wait(ptx::smem_u32(&bars->t_full), cnt & 1u);
      ptx::tc_fence_after();
      // rows of the score tile are queries, columns keys - in the dK/dV pass the tile is held transposed
      const int q_first = kDKV ? srow0 : tile0, k_first = kDKV ? tile0 : srow0;
      const bool full = tile_is_full(s, q_first, kTileM, k_first, kTileN, p.mask_type, p.group) &&
                        (!kDKV || q_first + kTileM <= s.lq);
      const long long bias_bh = static_cast<long long>(b) * p.bias_bstride + static_cast<long long>(qh) * p.maxq * p.maxk;
#pragma unroll 1
      for (int ch = 0; ch < 2; ++ch) {
        const int col = 64 * grp + 32 * ch;
        uint32_t t1[32], t2[32];
        ptx::tmem_ld32(tmem + lane_base + ((cnt & 1u) ? kColT1b : kColT1) + col, t1);
        ptx::tmem_ld32(tmem + lane_base + kColT2 + col, t2);
        // dK/dV pass: this key's bias values for the 32 queries of the chunk lie a row pitch apart - all 32 loads
        // are issued here, ahead of the wait for the products (addresses clamped into the plane: what lies outside
        // the sequence is never used)
        uint32_t bcol[16];
        if (staged && !kDKV) {
          if (ch == 0) w.wait(ptx::smem_u32(&bars->bias_full), cnt & 1u);
          // this query's 32 keys col .. col + 31: box col / 64 (= grp), row = query, four 16-byte chunks from
          // (col % 64) / 8 on, each ^ (query & 7)
          const uint32_t rowbase = sm_bias + grp * (kTileM * 128) + row * 128;
          const uint32_t c16 = static_cast<uint32_t>(col & 63) >> 3;
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4)
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(bcol[4 * q4]), "=r"(bcol[4 * q4 + 1]), "=r"(bcol[4 * q4 + 2]), "=r"(bcol[4 * q4 + 3])
                         : "r"(rowbase + (((c16 + q4) ^ (row & 7)) << 4)));
          if (ch == 1) ptx::mbar_arrive(ptx::smem_u32(&bars->bias_free));   // this thread has read its row
        } else if (staged) {
          if (ch == 0) {
            w.wait(ptx::smem_u32(&bars->bias_full), cnt & 1u);
          }
          // element (query col + e, key row): box row / 64, row = query, 16-byte chunk (key % 64) / 8 ^ (query & 7)
          const uint32_t box = sm_bias + (row >> 6) * (kTileM * 128) + (row & 7) * 2;
          const uint32_t kchunk = (row & 63) >> 3;
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const int q0l = col + 2 * e, q1l = q0l + 1;
            uint32_t lo, hi;
            asm volatile("ld.shared.u16 %0, [%1];" : "=r"(lo) : "r"(box + q0l * 128 + ((kchunk ^ (q0l & 7)) << 4)));
            asm volatile("ld.shared.u16 %0, [%1];" : "=r"(hi) : "r"(box + q1l * 128 + ((kchunk ^ (q1l & 7)) << 4)));
            bcol[e] = lo | (hi << 16);
          }
          if (ch == 1) ptx::mbar_arrive(ptx::smem_u32(&bars->bias_free));   // this thread has read its column
        } else if (kDKV && p.bias) {
          const int kk = mine < p.maxk ? mine : p.maxk - 1;
          const unsigned short* bsrc = static_cast<const unsigned short*>(p.bias) + bias_bh + kk;
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const int r0 = srow0 + col + 2 * e, r1 = r0 + 1;
            const uint32_t lo = __ldg(bsrc + static_cast<long long>(r0 < p.maxq ? r0 : p.maxq - 1) * p.maxk);
            const uint32_t hi = __ldg(bsrc + static_cast<long long>(r1 < p.maxq ? r1 : p.maxq - 1) * p.maxk);
            bcol[e] = lo | (hi << 16);
          }
        }
        ptx::tmem_wait_ld();
        // bit e of `bits`: element (this row, column col + e) of the tile is visible
        uint32_t bits;
        if (!kDKV) {
          bits = !mine_ok ? 0u : (full ? 0xffffffffu : visible_bits(rb_mine, srow0 + col));
        } else if (full) {
          bits = 0xffffffffu;
        } else if (mine >= s.lk) {
          bits = 0u;
        } else {
          const int i0 = srow0 + col;
          bits = (low_bits(hq_end - i0) & ~low_bits(c_lo - i0)) | low_bits(ctx_hi - i0) |
                 (low_bits(t_hi - i0) & ~low_bits(t_lo - i0));
        }
        uint32_t u1[16], u2[16];
        // per warp: every element visible -> no selects; nothing visible -> zeros without arithmetic; else selects
        const bool all_on = __all_sync(0xffffffffu, bits == 0xffffffffu);
        const bool all_off = __all_sync(0xffffffffu, bits == 0u);
        if (all_off) {
#pragma unroll
          for (int e = 0; e < 16; ++e) u1[e] = u2[e] = 0u;
        } else if (staged && !kDKV) {
          // (values of rows / keys outside the sequence are never used: their elements are not visible)
#pragma unroll
          for (int e = 0; e < 16; ++e)
            score_grad2<T, true, true>(make_float2(__uint_as_float(t1[2 * e]), __uint_as_float(t1[2 * e + 1])),
                                       make_float2(__uint_as_float(t2[2 * e]), __uint_as_float(t2[2 * e + 1])),
                                       BPack<T>::unpack(bcol[e]), p.alpha, p.scale, (bits >> (2 * e)) & 3u, u1[e], u2[e]);
        } else if (!kDKV && bias_vec && mine_ok && srow0 + col + 32 <= p.maxk) {
          // dQ pass: the 32 bias values of this row and chunk are contiguous - four 16-byte loads
          const uint4* src = reinterpret_cast<const uint4*>(static_cast<const T*>(p.bias) + bias_bh +
                                                            static_cast<long long>(mine) * p.maxk + srow0 + col);
          uint32_t bw[16];
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            const uint4 v4 = __ldg(src + q4);
            bw[4 * q4] = v4.x, bw[4 * q4 + 1] = v4.y, bw[4 * q4 + 2] = v4.z, bw[4 * q4 + 3] = v4.w;
          }
#pragma unroll
          for (int e = 0; e < 16; ++e)
            score_grad2<T, true, true>(make_float2(__uint_as_float(t1[2 * e]), __uint_as_float(t1[2 * e + 1])),
                                       make_float2(__uint_as_float(t2[2 * e]), __uint_as_float(t2[2 * e + 1])),
                                       BPack<T>::unpack(bw[e]), p.alpha, p.scale, (bits >> (2 * e)) & 3u, u1[e], u2[e]);
        } else if (p.bias) {
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const uint32_t v2 = (bits >> (2 * e)) & 3u;
            const int c = col + 2 * e;
            float2 bias;
            if (kDKV) {
              const float2 both = BPack<T>::unpack(bcol[e]);
              bias.x = (v2 & 1u) ? both.x : 0.f;
              bias.y = (v2 & 2u) ? both.y : 0.f;
            } else {
              const long long at = bias_bh + static_cast<long long>(mine) * p.maxk + srow0 + c;
              bias.x = (v2 & 1u) ? BPack<T>::one(p.bias, at) : 0.f;
              bias.y = (v2 & 2u) ? BPack<T>::one(p.bias, at + 1) : 0.f;
            }
            score_grad2<T, true, true>(make_float2(__uint_as_float(t1[2 * e]), __uint_as_float(t1[2 * e + 1])),
                                       make_float2(__uint_as_float(t2[2 * e]), __uint_as_float(t2[2 * e + 1])), bias,
                                       p.alpha, p.scale, v2, u1[e], u2[e]);
          }
        } else if (all_on) {
#pragma unroll
          for (int e = 0; e < 16; ++e)
            score_grad2<T, false, false>(make_float2(__uint_as_float(t1[2 * e]), __uint_as_float(t1[2 * e + 1])),
                                         make_float2(__uint_as_float(t2[2 * e]), __uint_as_float(t2[2 * e + 1])),
                                         make_float2(0.f, 0.f), p.alpha, p.scale, 3u, u1[e], u2[e]);
        } else {
#pragma unroll
          for (int e = 0; e < 16; ++e)
            score_grad2<T, false, true>(make_float2(__uint_as_float(t1[2 * e]), __uint_as_float(t1[2 * e + 1])),
                                        make_float2(__uint_as_float(t2[2 * e]), __uint_as_float(t2[2 * e + 1])),
                                        make_float2(0.f, 0.f), p.alpha, p.scale, (bits >> (2 * e)) & 3u, u1[e], u2[e]);
        }
        if (kDKV) ptx::tmem_st16(tmem + lane_base + kColT1 + 64 * grp + 16 * ch, u1);
        ptx::tmem_st16(tmem + lane_base + (kDKV ? kColT2 : ((cnt & 1u) ? kColT1b : kColT1)) + 64 * grp + 16 * ch, u2);
        ptx::tmem_wait_st();
        ptx::tc_fence_before();
        ptx::mbar_arrive(ptx::smem_u32(&bars->u_full[ch]));
        if (!kDKV && dbias && mine < p.maxq) {
          // this tile of d_bias = dS (already rounded), zeros where nothing is visible
          const int j0 = srow0 + col;
          T* dst = dbias + static_cast<long long>(b) * p.bias_bstride +
                   (static_cast<long long>(qh) * p.maxq + mine) * p.maxk + j0;
          if (dbias_vec && j0 + 32 <= p.maxk) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4)
              reinterpret_cast<uint4*>(dst)[q4] = make_uint4(u2[4 * q4], u2[4 * q4 + 1], u2[4 * q4 + 2], u2[4 * q4 + 3]);
          } else {
            unsigned short* d16 = reinterpret_cast<unsigned short*>(dst);
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              if (j0 + 2 * e < p.maxk) d16[2 * e] = static_cast<unsigned short>(u2[e] & 0xffffu);
              if (j0 + 2 * e + 1 < p.maxk) d16[2 * e + 1] = static_cast<unsigned short>(u2[e] >> 16);
            }
          }
        }
      }
      ++cnt;
    });
    // accumulators -> global (this group's half of the columns); rows past the sequence end are not written
    if (cnt > first) {
      w.wait(ptx::smem_u32(&bars->acc_full), tiles_done & 1u);
      ptx::tc_fence_after();
    }
    const int col0 = grp * (D / 2);
    const long long tok = (kDKV ? s.k0 : s.q0) + mine;
    T* out2 = static_cast<T*>(kDKV ? bp.dk : bp.dq) + (tok * heads + head) * D + col0;
    T* out1 = kDKV ? static_cast<T*>(bp.dv) + (tok * heads + head) * D + col0 : nullptr;
#pragma unroll 1
    for (int ch = 0; ch < D / 64; ++ch) {
#pragma unroll 1
      for (int which = kDKV ? 0 : 1; which < 2; ++which) {
        uint32_t acc[32];
        if (cnt > first) {
          ptx::tmem_ld32(tmem + lane_base + (which == 0 ? kColAcc1 : kColAcc2) + col0 + ch * 32, acc);
          ptx::tmem_wait_ld();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) acc[e] = 0u;   // nothing visible: zero gradient
        }
        if (mine_ok) {
          uint4* dst = reinterpret_cast<uint4*>((which == 0 ? out1 : out2) + ch * 32);
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint4 u;
            u.x = BPack<T>::pack(__uint_as_float(acc[q4 * 8 + 0]), __uint_as_float(acc[q4 * 8 + 1]));
            u.y = BPack<T>::pack(__uint_as_float(acc[q4 * 8 + 2]), __uint_as_float(acc[q4 * 8 + 3]));
            u.z = BPack<T>::pack(__uint_as_float(acc[q4 * 8 + 4]), __uint_as_float(acc[q4 * 8 + 5]));
            u.w = BPack<T>::pack(__uint_as_float(acc[q4 * 8 + 6]), __uint_as_float(acc[q4 * 8 + 7]));
            dst[q4] = u;
          }
        }
      }
    }
  }

  // everything of this tile is complete (MMAs, TMEM reads) before the next one reuses the tensor memory
  ++tiles_done;
  ptx::tc_fence_before();
  ptx::named_bar_sync(1, kConsumers);
  ptx::tc_fence_after();
  }  // tiles
  }  // warps 1 .. 11

  if (kDKV && tid == 0) asm volatile("griddepcontrol.wait;" ::: "memory");   // (no-op when launched the plain way)
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, 512);
  }
}

template <int D, typename T>
cudaError_t launch_bwd_tc_t(const BwdParams& bp, int dtype, int num_sms, cudaStream_t stream) {
  const KParams& p = bp.f;
  CUtensorMap mq, mg, mk, mv;
  if (!make_tile_map(&mq, p.q, p.total_q, p.hq, p.dqk, dtype) ||
      !make_tile_map(&mg, bp.dout, p.total_q, p.hq, p.dv, dtype) ||
      !make_tile_map(&mk, p.k, p.total_k, p.hk, p.dqk, dtype) || !make_tile_map(&mv, p.v, p.total_k, p.hk, p.dv, dtype))
    return cudaErrorNotSupported;
  constexpr int smem = 1024 + 6 * (D / 64) * kTileM * 128 + 256;
  constexpr int smem_kv = smem + 2 * kTileM * 128;   // + the staged bias tile of the dK/dV pass
  static_assert(smem_kv <= 232448, "shared memory budget of one CTA exceeded");
  static_assert(sizeof(BwdBars) <= 256, "barrier block too large");
  // the bias as TMA tiles: rows 16-byte aligned and batch blocks back to back (what the forward's staged mode needs)
  CUtensorMap mb = mq;
  const int bias_staged = p.bias && (p.maxk % 8 == 0) && (reinterpret_cast<uintptr_t>(p.bias) & 15u) == 0 &&
                          p.bias_bstride == static_cast<long long>(p.hq) * p.maxq * p.maxk &&
                          make_bias_tile_map(&mb, p, dtype);
  // one pass: the instantiation for (staged bias, tile look-ahead), its shared-memory size set, launched
  bool overlap = false;
  // one pass: the instantiation with or without a staged bias, its shared-memory size set, launched
  auto launch = [&](auto kdkv, long long tiles_bound, const CUtensorMap& a1, const CUtensorMap& a2,
                    const CUtensorMap& b1, const CUtensorMap& b2) -> cudaError_t {
    constexpr bool kDKV = decltype(kdkv)::value;
    const unsigned grid = static_cast<unsigned>(tiles_bound < num_sms ? tiles_bound : num_sms);
    auto go = [&](auto kern, int bytes) -> cudaError_t {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
      if (e != cudaSuccess) return e;
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(grid);
      cfg.blockDim = dim3(kBwdThreads);
      cfg.dynamicSmemBytes = bytes;
      cfg.stream = stream;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[0].val.programmaticStreamSerializationAllowed = 1;
      cfg.attrs = attr;
      // the dQ pass sets itself up while the pre-pass runs; the dK/dV pass may start while the dQ pass is still
      // running (when there is no dQ pass it follows the pre-pass in plain stream order)
      cfg.numAttrs = (!kDKV || overlap) ? 1 : 0;
      return cudaLaunchKernelEx(&cfg, kern, bp, a1, a2, b1, b2, mb);
    };
    return bias_staged ? go(hstu_bwd_tc_kernel<D, T, kDKV, true>, smem_kv) : go(hstu_bwd_tc_kernel<D, T, kDKV, false>, smem);
  };
  cudaError_t e = cudaSuccess;
  overlap = p.total_q > 0;   // (a dQ pass is launched in front of the dK/dV pass)
  if (p.total_q > 0)
    e = launch(std::false_type{}, static_cast<long long>(p.batch) * p.hq * ((p.maxq + kTileM - 1) / kTileM), mq, mg,
               mk, mv);
  if (e != cudaSuccess) return e;
  if (p.total_k > 0)
    e = launch(std::true_type{}, static_cast<long long>(p.batch) * p.hk * ((p.maxk + kTileN - 1) / kTileN), mk, mv,
               mq, mg);
  return e;
}

}  // namespace

bool bwd_tc_supported(const BwdParams& bp, int dtype) {
  const KParams& p = bp.f;
  if (dtype != HSTU_DTYPE_BF16 && dtype != HSTU_DTYPE_FP16) return false;
  if (p.dqk != p.dv || (p.dqk != 64 && p.dqk != 128)) return false;
  if (p.mask_type != HSTU_MASK_TRIL && p.mask_type != HSTU_MASK_NONE) return false;
  if (p.flags & (HSTU_FLAG_ALPHA_BEFORE_BIAS | HSTU_FLAG_FORCE_GENERIC)) return false;
  if (p.total_q > 0x7fffff00ll || p.total_k > 0x7fffff00ll) return false;
  const uintptr_t align = reinterpret_cast<uintptr_t>(p.q) | reinterpret_cast<uintptr_t>(p.k) |
                          reinterpret_cast<uintptr_t>(p.v) | reinterpret_cast<uintptr_t>(bp.dout) |
                          reinterpret_cast<uintptr_t>(bp.dq) | reinterpret_cast<uintptr_t>(bp.dk) |
                          reinterpret_cast<uintptr_t>(bp.dv);
  return (align & 15u) == 0;
}

// Returns cudaSuccess, a CUDA error, or cudaErrorNotSupported when the tensor maps could not be encoded.
cudaError_t launch_bwd_tc(const BwdParams& bp, int dtype, int num_sms, cudaStream_t stream) {
  const KParams& p = bp.f;
  if (dtype == HSTU_DTYPE_BF16)
    return p.dqk == 128 ? launch_bwd_tc_t<128, __nv_bfloat16>(bp, dtype, num_sms, stream)
                        : launch_bwd_tc_t<64, __nv_bfloat16>(bp, dtype, num_sms, stream);
  return p.dqk == 128 ? launch_bwd_tc_t<128, __half>(bp, dtype, num_sms, stream) : launch_bwd_tc_t<64, __half>(bp, dtype, num_sms, stream);
}

}  // namespace hstu
