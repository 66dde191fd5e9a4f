// Shared host/device definitions of the HSTU jagged forward: kernel parameter block, per-sequence
// geometry, the composite mask expressed as per-row column bounds, and the K-tile range of a q-tile.
//
// Mask semantics follow the reference golden create_causal_mask
// (ascendc/attention/hstu_v1/hstu_forward_v1/test/pytest/common.py:118-137) and the kernel-side tile
// classifier (ascendc/attention/hstu_v1/hstu_forward_v1/op_kernel/atlas950/hstu_dense_causal_mask.h:63-109).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/hstu_b200.h"

#define HSTU_HD __host__ __device__ __forceinline__

namespace hstu {

// Rows of Q handled by one work item of the tensor-core kernel (two 128-row tiles) and its K tile width.
constexpr int kTileM = 128;
constexpr int kPairM = 2 * kTileM;
constexpr int kTileN = 128;

// Workspace layout (all offsets in bytes from the 256-byte aligned base).
//   [0]   uint32 status bits (HSTU_ST_*)
//   [4]   uint32 number of work items
//   [8]   uint32 work counter (forward kernel; backward dQ pass)
//   [12]  uint32 work counter (backward dK/dV pass)
//   [256] uint32 items[2 * capacity]   {sequence, head << 16 | q_pair}
constexpr uint64_t kWsHeaderBytes = 256;
// Below this many work items (tiles) in a call - eight per SM of a B200 - a list is ordered by the items' step counts,
// longest first: with a few items per CTA the balance at the end of the kernel is what counts.  Above it the items of
// one (sequence, head) stay neighbours, so the CTAs that run together share K/V in L2.
constexpr long long kFewItems = 8 * 148;

struct KParams {
  const void* q;
  const void* k;
  const void* v;
  void* out;
  const void* bias;
  const void* mask;
  const void* offq;
  const void* offk;
  const void* ctx;
  const void* tgt;
  long long total_q, total_k;
  long long bias_bstride;
  int index_bytes;
  int batch;
  int hq, hk, dqk, dv;
  int gqa_ratio;
  int mask_type;
  int maxq, maxk;
  int group;
  float scale;
  float alpha;
  unsigned flags;
  uint32_t* ws_header;  // status, item count, counter
  uint32_t* items;      // work list
  long long item_capacity;
  // hstu_paged only (null / 0 otherwise): the page table the keys / values were gathered from, for the pre-pass's
  // consistency check
  const void* page_offsets;   // [batch + 1]
  const void* page_ids;       // [num_page_ids]
  const void* last_page_len;  // [batch]
  long long num_pages, num_page_ids;
  int page_size;
  // hstu_paged on the tensor-core kernel with 128-row pages: the K / V tiles that are whole cache pages are read
  // from the cache itself (one TMA box per page); only the rest of each sequence - its partial last page and the new
  // rows - goes through the staging tensors
  const void* kv_cache;       // [num_pages, 2, page_size, hk, d]
  int paged_direct;
  // backward on the tensor-core kernels only (0 otherwise): `items` holds two tile lists, bwd_cap_q entries for the
  // dQ pass followed by bwd_cap_k for the dK/dV pass; bwd_all_q_tiles: the dQ pass also visits the q-tiles past a
  // sequence's end (they hold rows of grad_bias that must be zeroed)
  long long bwd_cap_q, bwd_cap_k;
  int bwd_all_q_tiles;
  int bwd_by_steps;   // order the lists by the tiles' step counts (few tiles per CTA) instead of sequence by sequence
  int fwd_by_steps;   // the same for the forward's work list: all sequences' last q-pairs first, then the ones before
};

// Backward call: the forward's parameters plus the gradient tensors.
struct BwdParams {
  KParams f;          // the forward call (f.out unused)
  const void* dout;   // [total_q, hq, dv]
  void* dq;           // [total_q, hq, dqk]
  void* dk;           // [total_k, hk, dqk]
  void* dv;           // [total_k, hk, dv]
  void* dbias;        // [batch, hq, maxq, maxk] or null
};

// in_linear_silu call: the output tensors and the column ranges of mixed that go to each of them.
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

struct SeqInfo {
  long long q0, k0;  // first token of the sequence in q / k,v
  int lq, lk;        // lengths
  int ctx, tgt;      // num_context, num_target (0 when absent)
};

HSTU_HD long long load_index(const void* p, int index_bytes, long long i) {
  return index_bytes == 8 ? static_cast<const long long*>(p)[i]
                          : static_cast<long long>(static_cast<const int*>(p)[i]);
}

HSTU_HD SeqInfo load_seq(const KParams& p, int b) {
  SeqInfo s;
  s.q0 = load_index(p.offq, p.index_bytes, b);
  long long q1 = load_index(p.offq, p.index_bytes, b + 1);
  s.k0 = load_index(p.offk, p.index_bytes, b);
  long long k1 = load_index(p.offk, p.index_bytes, b + 1);
  long long lq = q1 - s.q0, lk = k1 - s.k0;
  // Inconsistent inputs (flagged by check_seq) are made harmless here: no row outside [0, total) and no
  // bias/mask element outside its [max_seq_len_q, max_seq_len_k] block is ever addressed.
  if (s.q0 < 0 || s.q0 > p.total_q) { s.q0 = 0; lq = 0; }
  if (s.k0 < 0 || s.k0 > p.total_k) { s.k0 = 0; lk = 0; }
  if (s.q0 + lq > p.total_q) lq = p.total_q - s.q0;
  if (s.k0 + lk > p.total_k) lk = p.total_k - s.k0;
  if (lq > p.maxq) lq = p.maxq;
  if (lk > p.maxk) lk = p.maxk;
  s.lq = lq < 0 ? 0 : static_cast<int>(lq);
  s.lk = lk < 0 ? 0 : static_cast<int>(lk);
  long long c = p.ctx ? load_index(p.ctx, p.index_bytes, b) : 0;
  long long t = p.tgt ? load_index(p.tgt, p.index_bytes, b) : 0;
  s.ctx = c < 0 ? 0 : (c > s.lq ? s.lq : static_cast<int>(c));
  s.tgt = t < 0 ? 0 : (t > s.lq ? s.lq : static_cast<int>(t));
  if (s.tgt > s.lk) s.tgt = s.lk;
  return s;
}

// Input consistency of one sequence (HSTU_ST_* bits).  The reference does not check these and would read
// out of bounds (the bias/mask row stride is max_seq_len_k).
HSTU_HD unsigned check_seq(const KParams& p, int b) {
  unsigned st = 0;
  long long q0 = load_index(p.offq, p.index_bytes, b), q1 = load_index(p.offq, p.index_bytes, b + 1);
  long long k0 = load_index(p.offk, p.index_bytes, b), k1 = load_index(p.offk, p.index_bytes, b + 1);
  if (q1 < q0 || k1 < k0 || q0 < 0 || k0 < 0 || q1 > p.total_q || k1 > p.total_k) st |= HSTU_ST_BAD_OFFSETS;
  if (q1 - q0 > p.maxq || k1 - k0 > p.maxk) st |= HSTU_ST_LEN_GT_MAX;
  long long c = p.ctx ? load_index(p.ctx, p.index_bytes, b) : 0;
  long long t = p.tgt ? load_index(p.tgt, p.index_bytes, b) : 0;
  if (c < 0 || t < 0 || c + t > q1 - q0 || t > k1 - k0) st |= HSTU_ST_BAD_CTX_TARGET;
  return st;
}

// hstu_paged, direct page reads: how many leading K / V tiles (128 keys each) of sequence b are whole cache pages the
// attention kernel reads from the cache itself, and the first slot of the sequence in page_ids.  The gather leaves
// exactly these rows out of the staging tensors, so both sides use this one rule (every index clamped: the
// result never names a page slot outside page_ids).
HSTU_HD int paged_full_tiles(const void* offq, const void* offk, const void* tgt, const void* page_offsets,
                             int index_bytes, long long total_q, long long num_page_ids, int b, long long* first_slot) {
  const long long k0 = load_index(offk, index_bytes, b), k1 = load_index(offk, index_bytes, b + 1);
  const long long q0 = load_index(offq, index_bytes, b);
  long long q1 = load_index(offq, index_bytes, b + 1);
  if (q1 > total_q) q1 = total_q;
  long long t = tgt ? load_index(tgt, index_bytes, b) : 0;
  if (t < 0) t = 0;
  if (t > q1 - q0) t = q1 - q0 > 0 ? q1 - q0 : 0;
  long long pg0 = load_index(page_offsets, index_bytes, b), pg1 = load_index(page_offsets, index_bytes, b + 1);
  if (pg0 < 0) pg0 = 0;
  if (pg1 > num_page_ids) pg1 = num_page_ids;
  long long n = ((k1 - k0) - t) / kTileN;   // whole pages of the cached part
  if (n > pg1 - pg0) n = pg1 - pg0;
  if (n < 0) n = 0;
  if (n > 0x7fff) n = 0x7fff;
  *first_slot = pg0;
  return static_cast<int>(n);
}

// hstu_paged: the page table of sequence b must describe exactly the cached part of its keys,
// (pages - 1) * page_size + last_page_len == len_k - num_target, with page ids inside the cache
// (the reference golden asserts the former, hstu_forward_v1/test/pytest/common.py:286).
HSTU_HD unsigned check_pages(const KParams& p, int b) {
  if (!p.page_offsets) return 0;
  const long long pg0 = load_index(p.page_offsets, p.index_bytes, b), pg1 = load_index(p.page_offsets, p.index_bytes, b + 1);
  if (pg0 < 0 || pg1 < pg0 || pg1 > p.num_page_ids) return HSTU_ST_BAD_PAGES;
  const long long last = p.last_page_len ? load_index(p.last_page_len, p.index_bytes, b) : p.page_size;
  const long long k0 = load_index(p.offk, p.index_bytes, b), k1 = load_index(p.offk, p.index_bytes, b + 1);
  long long t = p.tgt ? load_index(p.tgt, p.index_bytes, b) : 0;
  if (t < 0) t = 0;
  const long long pages = pg1 - pg0;
  const long long cached = pages > 0 ? (pages - 1) * p.page_size + last : 0;
  if (last < 0 || last > p.page_size || (pages > 0 && last == 0) || cached != (k1 - k0) - t) return HSTU_ST_BAD_PAGES;
  for (long long s = pg0; s < pg1; ++s) {
    const long long pid = load_index(p.page_ids, p.index_bytes, s);
    if (pid < 0 || pid >= p.num_pages) return HSTU_ST_BAD_PAGES;
  }
  return 0;
}

// Visibility of row i as column bounds:  allowed(j)  <=>  j < lim1  ||  (lo2 <= j && j <= hi2).
// Both already respect j < lk.
struct RowBounds {
  int lim1, lo2, hi2;
};

HSTU_HD RowBounds row_bounds(const SeqInfo& s, int i, int mask_type, int group) {
  RowBounds r;
  r.lo2 = 1;
  r.hi2 = 0;
  if (mask_type != HSTU_MASK_TRIL) {
    r.lim1 = s.lk;
    return r;
  }
  const int delta = s.lk - s.lq;
  const int hist = s.lk - s.tgt;
  if (s.tgt > 0 && group > 0 && i >= s.lq - s.tgt) {
    const int ti = i - (s.lq - s.tgt);
    r.lim1 = hist;
    r.lo2 = hist + (ti / group) * group;
    r.hi2 = hist + ti;
    if (r.hi2 > s.lk - 1) r.hi2 = s.lk - 1;
  } else {
    int lim = i + delta + 1;
    if (s.ctx > 0 && i < s.ctx && hist > lim) lim = hist;
    r.lim1 = lim;
  }
  if (r.lim1 < 0) r.lim1 = 0;
  if (r.lim1 > s.lk) r.lim1 = s.lk;
  return r;
}

HSTU_HD bool allowed(const RowBounds& r, int j) {
  return j < r.lim1 || (j >= r.lo2 && j <= r.hi2);
}

// Number of leading K tiles of width bn a q-tile of rows [r0, r0 + rows) has to visit (0 = nothing visible
// or tile out of range).  Tiles beyond it are fully masked for every row of the q-tile.
HSTU_HD int kv_tiles_for_rows(const SeqInfo& s, int r0, int rows, int mask_type, int bn) {
  if (r0 >= s.lq || s.lk <= 0) return 0;
  int r1 = r0 + rows - 1;
  if (r1 > s.lq - 1) r1 = s.lq - 1;
  int ub;
  if (mask_type != HSTU_MASK_TRIL) {
    ub = s.lk;
  } else {
    ub = r1 + (s.lk - s.lq) + 1;
    const int hist = s.lk - s.tgt;
    if (s.ctx > 0 && r0 < s.ctx && hist > ub) ub = hist;
    if (ub > s.lk) ub = s.lk;
  }
  if (ub <= 0) return 0;
  return (ub + bn - 1) / bn;
}

// True when every (row, col) of the tile rows [r0, r0+rows) x cols [c0, c0+bn) is visible, so the epilogue can
// skip the per-element predicate.  Conservative (may answer false for a full tile), never optimistic.
HSTU_HD bool tile_is_full(const SeqInfo& s, int r0, int rows, int c0, int bn, int mask_type, int group) {
  int lim = s.lk;
  if (mask_type == HSTU_MASK_TRIL) {
    const int causal = r0 + (s.lk - s.lq) + 1;
    if (causal < lim) lim = causal;
    int r1 = r0 + rows - 1;
    if (r1 > s.lq - 1) r1 = s.lq - 1;
    if (s.tgt > 0 && group > 0 && r1 >= s.lq - s.tgt) {
      const int hist = s.lk - s.tgt;
      if (hist < lim) lim = hist;
    }
  }
  return c0 + bn <= lim;
}

// Number of work items (q-pairs) of a sequence.
HSTU_HD int pairs_of(int lq) { return (lq + kPairM - 1) / kPairM; }

}  // namespace hstu
