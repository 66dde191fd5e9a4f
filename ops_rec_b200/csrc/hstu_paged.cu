// hstu_paged: the key / value gather that turns a paged KV cache plus the new target rows into the packed
// [tokens, heads, dim] layout the attention kernels read.
//
// The reference operator (ascendc/attention/hstu_v1/torch_extension/hstu_paged_plugin.cpp:21-72; kernel
// .../hstu_forward_v1/op_kernel/atlas950/hstu_paged_forward_kernel.h, FetchKvMayFromCache) attends, per sequence,
// over   K/V = [ page 0 | page 1 | ... | last page cut to last_page_len ]  ++  [ the target rows of the input k / v ]
// where the pages are kv_cache[page_ids[page_offsets[b] .. page_offsets[b + 1])] and the target rows are the last
// num_target[b] rows of the sequence's segment of the input k / v (the history rows of the input are not used).
// Here one HBM-bound pass writes exactly that into two staging tensors inside the caller's workspace, after which the
// call is an ordinary jagged forward in its `.delta` form (len_q = new history + targets <= len_k = cache + targets)
// on the same tcgen05 / generic kernels, scheduler and mask algebra.  A page of the cache is contiguous
// [page_size, heads, dim], so every page is one straight copy of page_size * heads * dim elements.
//
// Inconsistent page tables are flagged by the scheduling pre-pass (HSTU_ST_BAD_PAGES); this pass only makes them
// harmless: a row whose source does not exist (a page slot outside the sequence's range, a page id outside the cache)
// becomes zeros, and nothing outside the tensors is ever addressed.
#include "hstu_common.cuh"

namespace hstu {

namespace {

constexpr int kGatherThreads = 256;
constexpr int kGatherRows = 64;   // consecutive staging rows per CTA

struct GatherParams {
  const unsigned char* cache;   // [pages, 2, page_size, heads_k, dim]
  const unsigned char* k_in;    // [total_q, heads_k, dim]
  const unsigned char* v_in;
  unsigned char* k_out;         // [capacity, heads_k, dim]
  unsigned char* v_out;
  const void* offq;
  const void* offk;
  const void* tgt;
  const void* page_offsets;
  const void* page_ids;
  long long total_q, capacity, num_pages, num_page_ids;
  int index_bytes, batch, page_size;
  int row_bytes;                // heads_k * dim * element size
  int skip_full_pages;          // the attention kernel reads whole pages from the cache: stage only the rest
};

// One CTA per kGatherRows consecutive rows of a staging tensor (grid.y = 0: keys, 1: values).
//   phase 1  one thread per row finds the row's source: its sequence by bisection over seq_offset_k, then either a row
//            of a cache page or a target row of the input; rows behind the last sequence become zeros for one K/V
//            tile's worth (a tile that runs past the end of the data multiplies those rows by P = 0, which must not
//            meet the NaN bit patterns uninitialised memory may hold), the rest of the capacity is never read
//   phase 2  all threads copy: a warp takes four rows at a time and issues their loads before the first store
template <typename V>
__global__ void __launch_bounds__(kGatherThreads) hstu_paged_gather_kernel(const GatherParams p) {
  __shared__ const unsigned char* s_src[kGatherRows];
  __shared__ unsigned char s_mode[kGatherRows];   // 0: skip the row, 1: copy from s_src, 2: zeros
  __shared__ long long s_off[kGatherRows + 1];    // seq_offset_k[b0 .. b0 + 64], b0 = the sequence of the CTA's first row
  __shared__ int s_b0;
  __shared__ int s_skip_all;
  const bool is_v = blockIdx.y != 0;
  unsigned char* out = is_v ? p.v_out : p.k_out;
  const long long first = static_cast<long long>(blockIdx.x) * kGatherRows;
  // The rows of a CTA are consecutive, so their sequences are b0, b0 + 1, ...: warp 0 finds b0 with a 32-way search
  // (three rounds of loads for 32 768 sequences instead of fifteen dependent ones per row), the offsets from b0 on go
  // to shared memory, and every row finds its sequence there.  Offsets that are not monotone (flagged by the
  // pre-pass) may send a row to the wrong sequence; the range check below then gives it no source.
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    int lo = 0, hi = p.batch - 1;   // the last sequence whose first row is <= first lies in [lo, hi]
    while (hi > lo) {
      const int stride = (hi - lo + 31) >> 5;
      auto probe = [&](int l) { const int at = lo + (l + 1) * stride; return at < hi ? at : hi; };
      const bool le = load_index(p.offk, p.index_bytes, probe(lane)) <= first;
      const int c = __popc(__ballot_sync(0xffffffffu, le));
      if (c == 0) {
        hi = probe(0) - 1;
      } else {
        const int nlo = probe(c - 1);
        if (c < 32) hi = probe(c) - 1 > nlo ? probe(c) - 1 : nlo;
        lo = nlo;
      }
    }
    if (lane == 0) s_b0 = lo;
  }
  __syncthreads();
  const int b0 = s_b0;
  if (threadIdx.x <= kGatherRows) {
    const int at = b0 + static_cast<int>(threadIdx.x) < p.batch ? b0 + static_cast<int>(threadIdx.x) : p.batch;
    s_off[threadIdx.x] = load_index(p.offk, p.index_bytes, at);
  }
  __syncthreads();
  // Direct page reads: most CTAs lie wholly inside the whole pages of one sequence and have nothing to stage.
  if (p.skip_full_pages) {
    if (threadIdx.x == 0) {
      int all = 0;
      if (first >= s_off[0] && first + kGatherRows <= s_off[1]) {
        long long slot;
        const int n = paged_full_tiles(p.offq, p.offk, p.tgt, p.page_offsets, p.index_bytes, p.total_q, p.num_page_ids,
                                       b0, &slot);
        all = first + kGatherRows - s_off[0] <= static_cast<long long>(kTileN) * n ? 1 : 0;
      }
      s_skip_all = all;
    }
    __syncthreads();
    if (s_skip_all) return;
  }
  if (threadIdx.x < kGatherRows) {
    const long long row = first + threadIdx.x;
    const unsigned char* src = nullptr;
    unsigned char mode = 0;
    long long k_end = load_index(p.offk, p.index_bytes, p.batch);
    if (k_end < 0) k_end = 0;
    if (k_end > p.capacity) k_end = p.capacity;
    if (row < p.capacity && row >= k_end) {
      mode = row < k_end + kTileN ? 2 : 0;
    } else if (row < p.capacity) {
      // the last sequence whose first row is <= row (sequences of length 0 share their offset with the next one)
      int b;
      long long k0, k1;
      if (row < s_off[kGatherRows] || b0 + kGatherRows >= p.batch) {
        int lo = 0, hi = kGatherRows - 1;
        while (lo < hi) {
          const int mid = (lo + hi + 1) >> 1;
          if (s_off[mid] <= row) lo = mid; else hi = mid - 1;
        }
        b = b0 + lo < p.batch - 1 ? b0 + lo : p.batch - 1;
        k0 = s_off[b - b0];
        k1 = s_off[b - b0 + 1];
      } else {   // more than 64 sequences begin inside this CTA's rows (runs of empty ones): the long way
        int lo = b0, hi = p.batch - 1;
        while (lo < hi) {
          const int mid = (lo + hi + 1) >> 1;
          if (load_index(p.offk, p.index_bytes, mid) <= row) lo = mid; else hi = mid - 1;
        }
        b = lo;
        k0 = load_index(p.offk, p.index_bytes, b);
        k1 = load_index(p.offk, p.index_bytes, b + 1);
      }
      if (row >= k0 && row < k1) {   // (offsets that are not monotone, flagged by the pre-pass, leave rows uncovered)
        mode = 2;                    // zeros unless a source exists (an inconsistent table has none for this row)
        const long long q0 = load_index(p.offq, p.index_bytes, b);
        long long q1 = load_index(p.offq, p.index_bytes, b + 1);
        if (q1 > p.total_q) q1 = p.total_q;
        long long t = p.tgt ? load_index(p.tgt, p.index_bytes, b) : 0;
        if (t < 0) t = 0;
        if (t > q1 - q0) t = q1 - q0 > 0 ? q1 - q0 : 0;
        const long long r = row - k0, cache_len = (k1 - k0) - t;
        long long unused_slot;
        if (p.skip_full_pages &&
            r < static_cast<long long>(kTileN) * paged_full_tiles(p.offq, p.offk, p.tgt, p.page_offsets, p.index_bytes,
                                                                  p.total_q, p.num_page_ids, b, &unused_slot)) {
          mode = 0;   // a row of a whole page: never read from the staging tensor
        } else if (r < cache_len) {
          long long pg0 = load_index(p.page_offsets, p.index_bytes, b), pg1 = load_index(p.page_offsets, p.index_bytes, b + 1);
          if (pg0 < 0) pg0 = 0;
          if (pg1 > p.num_page_ids) pg1 = p.num_page_ids;
          const long long slot = pg0 + r / p.page_size;
          if (slot < pg1) {
            const long long pid = load_index(p.page_ids, p.index_bytes, slot);
            if (pid >= 0 && pid < p.num_pages) {
              src = p.cache + ((pid * 2 + (is_v ? 1 : 0)) * p.page_size + r % p.page_size) * p.row_bytes;
              mode = 1;
            }
          }
        } else {
          const long long at = q1 - t + (r - cache_len);
          if (at >= 0 && at < p.total_q) {
            src = (is_v ? p.v_in : p.k_in) + at * p.row_bytes;
            mode = 1;
          }
        }
      }
    }
    s_src[threadIdx.x] = src;
    s_mode[threadIdx.x] = mode;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int kWarps = kGatherThreads / 32;
  constexpr int kBatch = 4;   // rows in flight per warp
  for (int r0 = warp * kBatch; r0 < kGatherRows; r0 += kWarps * kBatch) {
    for (int i = lane * static_cast<int>(sizeof(V)); i < p.row_bytes; i += 32 * static_cast<int>(sizeof(V))) {
      V v[kBatch];
#pragma unroll
      for (int j = 0; j < kBatch; ++j) v[j] = s_mode[r0 + j] == 1 ? *reinterpret_cast<const V*>(s_src[r0 + j] + i) : V{};
#pragma unroll
      for (int j = 0; j < kBatch; ++j)
        if (s_mode[r0 + j]) *reinterpret_cast<V*>(out + (first + r0 + j) * p.row_bytes + i) = v[j];
    }
  }
}

}  // namespace

// Enqueues the gather.  All pointers are device pointers; capacity = rows of each staging tensor.
cudaError_t launch_paged_gather(const KParams& p, const void* kv_cache, const void* k_in, const void* v_in,
                                void* k_out, void* v_out, long long capacity, long long num_pages,
                                long long num_page_ids, int esize, cudaStream_t stream) {
  GatherParams g;
  g.cache = static_cast<const unsigned char*>(kv_cache);
  g.k_in = static_cast<const unsigned char*>(k_in);
  g.v_in = static_cast<const unsigned char*>(v_in);
  g.k_out = static_cast<unsigned char*>(k_out);
  g.v_out = static_cast<unsigned char*>(v_out);
  g.offq = p.offq;
  g.offk = p.offk;
  g.tgt = p.tgt;
  g.page_offsets = p.page_offsets;
  g.page_ids = p.page_ids;
  g.total_q = p.total_q;
  g.capacity = capacity;
  g.num_pages = num_pages;
  g.num_page_ids = num_page_ids;
  g.index_bytes = p.index_bytes;
  g.batch = p.batch;
  g.page_size = p.page_size;
  g.row_bytes = p.hk * p.dqk * esize;
  g.skip_full_pages = p.paged_direct;
  const dim3 grid(static_cast<unsigned>((capacity + kGatherRows - 1) / kGatherRows), 2, 1);
  const uintptr_t align = reinterpret_cast<uintptr_t>(kv_cache) | reinterpret_cast<uintptr_t>(k_in) |
                          reinterpret_cast<uintptr_t>(v_in) | reinterpret_cast<uintptr_t>(k_out) |
                          reinterpret_cast<uintptr_t>(v_out) | static_cast<uintptr_t>(g.row_bytes);
  if ((align & 15u) == 0)
    hstu_paged_gather_kernel<uint4><<<grid, kGatherThreads, 0, stream>>>(g);
  else if ((align & 3u) == 0)
    hstu_paged_gather_kernel<uint32_t><<<grid, kGatherThreads, 0, stream>>>(g);
  else
    hstu_paged_gather_kernel<uint16_t><<<grid, kGatherThreads, 0, stream>>>(g);
  return cudaGetLastError();
}

}  // namespace hstu
