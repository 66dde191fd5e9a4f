// Jagged tile scheduler: the device pre-pass that turns seq_offset into the work list of the tensor-core
// kernel, and its host mirror.
//
// The reference splits work inside the kernel: every core walks all B offsets and takes an equal share of
// the non-empty causal tiles, which can cut a q-block row between two cores and is why its output must be
// zero-filled and accumulated atomically (…/op_kernel/atlas950/hstu_split_core_policy.h:53-214,
// torch_extension/hstu_jagged_plugin.cpp:56-59).  Here a work item is a whole (sequence, head, 256-row q-pair):
// nothing is ever split, so the output needs neither zero-fill nor atomics.
//
// Order of the list: sequences by number of q-pairs, longest first (a counting sort, stable in the sequence
// index); inside a sequence head-major, and inside a head the q-pairs from the last (most K tiles) to the
// first.  Persistent CTAs draw items from a global atomic counter, so the order of the list is greedy
// longest-first scheduling, and the CTAs that run at the same time work on neighbouring q-pairs of the same few
// (sequence, head) - their K/V stays in L2.
// A call with few items (fewer than eight per SM) orders them by steps instead: q-pair number descending over all
// sequences - a q-pair's cost grows with its number, and with two or three items per CTA the balance at the end of
// the kernel counts for more than L2 reuse (such a call's K/V fits the L2 anyway).
#include "hstu_common.cuh"

namespace hstu {

constexpr int kMaxPairs = 20480 / kPairM;   // 80: max_seq_len is limited to 20480 like the reference
constexpr int kBuckets = kMaxPairs + 1;
constexpr int kPreThreads = 1024;

__global__ void __launch_bounds__(kPreThreads) hstu_prepass_kernel(const KParams p, const int build_items) {
  __shared__ unsigned s_count[kBuckets];        // sequences per bucket
  __shared__ unsigned s_start[kBuckets];        // first item of the bucket
  __shared__ unsigned s_seen[kBuckets];         // sequences of the bucket placed by earlier chunks
  __shared__ unsigned s_warp[32][kBuckets];     // per-warp counts of the current chunk, then exclusive prefix
  __shared__ unsigned s_status;
  __shared__ unsigned s_first[kPreThreads];     // first item of each sequence of the chunk
  __shared__ unsigned short s_key[kPreThreads]; // its number of q-pairs (0: nothing to write)
  __shared__ unsigned s_before[kBuckets];       // by steps: sequences with more q-pairs than the bucket's
  __shared__ unsigned s_class[kBuckets];        // by steps: first item of the class "q-pair number `index` - 1"
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  // Let the attention kernel (launched with programmatic stream serialization) begin its set-up now; it waits
  // for this grid to complete before it reads the work list.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // (this kernel's latency is part of every call: the attention kernel's first item waits for it.  Hence one
  // read of the offsets for the first 1024 sequences, and a warp-wide scan instead of a serial walk over the buckets.)
  for (int i = tid; i < kBuckets; i += kPreThreads) {
    s_count[i] = 0;
    s_seen[i] = 0;
  }
  for (int i = tid; i < 32 * kBuckets; i += kPreThreads) (&s_warp[0][0])[i] = 0;
  if (tid == 0) s_status = 0;
  __syncthreads();

  unsigned st = 0;
  int key_first = 0;   // bucket of sequence `tid` (the first chunk of the second pass)
  for (int b = tid; b < p.batch; b += kPreThreads) {
    st |= check_seq(p, b) | check_pages(p, b);
    if (build_items) {
      const SeqInfo s = load_seq(p, b);
      const int key = pairs_of(s.lq);
      if (b == tid) key_first = key;
      atomicAdd(&s_count[key], 1u);
    }
  }
  if (st) atomicOr(&s_status, st);
  __syncthreads();
  if (warp == 0) {
    // s_start[key] = items of all larger keys: an exclusive scan from the largest key down, three keys per lane
    // (lane 0 holds the largest)
    unsigned v[3], sum = 0;
#pragma unroll
    for (int i = 0; i < 3; ++i) {
      const int key = kMaxPairs - (3 * lane + i);
      v[i] = key >= 1 ? s_count[key] * static_cast<unsigned>(key) * static_cast<unsigned>(p.hq) : 0u;
      sum += v[i];
    }
    unsigned incl = sum;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const unsigned o = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += o;
    }
    unsigned run = incl - sum;
#pragma unroll
    for (int i = 0; i < 3; ++i) {
      const int key = kMaxPairs - (3 * lane + i);
      if (key >= 0) s_start[key] = run;
      run += v[i];
    }
    // Ordered by steps (p.fwd_by_steps, calls with few items): the last q-pairs of all sequences first, then the ones
    // before them - a q-pair's cost grows with its number, so this is longest-first list scheduling.  Q-pair number
    // s - 1 exists once per head in every sequence of at least s pairs, and these sequences are a prefix of the sorted
    // order: item = s_class[s] + (rank of the sequence in the sorted order) * heads + head.
    {
      unsigned c[3], csum = 0;
#pragma unroll
      for (int i = 0; i < 3; ++i) {
        const int key = kMaxPairs - (3 * lane + i);
        c[i] = key >= 1 ? s_count[key] : 0u;
        csum += c[i];
      }
      unsigned cincl = csum;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const unsigned o = __shfl_up_sync(0xffffffffu, cincl, d);
        if (lane >= d) cincl += o;
      }
      unsigned before = cincl - csum, g[3], gsum = 0;
#pragma unroll
      for (int i = 0; i < 3; ++i) {
        const int key = kMaxPairs - (3 * lane + i);
        if (key >= 0) s_before[key] = before;
        before += c[i];
        g[i] = key >= 1 ? before * static_cast<unsigned>(p.hq) : 0u;
        gsum += g[i];
      }
      unsigned gincl = gsum;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const unsigned o = __shfl_up_sync(0xffffffffu, gincl, d);
        if (lane >= d) gincl += o;
      }
      unsigned gstart = gincl - gsum;
#pragma unroll
      for (int i = 0; i < 3; ++i) {
        const int key = kMaxPairs - (3 * lane + i);
        if (key >= 0) s_class[key] = gstart;
        gstart += g[i];
      }
    }
    if (lane == 31) {
      // never more than the list holds: offsets that are not monotone can describe more q-pairs than total_q has
      // rows for (the host sizes the list from total_q); the surplus items are dropped, the status word says why
      unsigned total = incl;
      if (static_cast<long long>(total) > p.item_capacity) total = static_cast<unsigned>(p.item_capacity);
      p.ws_header[0] = s_status;
      p.ws_header[2] = 0;   // work counters (forward; backward dQ pass)
      p.ws_header[3] = 0;   // (backward dK/dV pass)
      p.ws_header[1] = build_items ? total : 0u;
    }
  }
  if (!build_items) return;
  __syncthreads();

  for (int base = 0; base < p.batch; base += kPreThreads) {
    if (base > 0) {
      for (int i = tid; i < 32 * kBuckets; i += kPreThreads) (&s_warp[0][0])[i] = 0;
      __syncthreads();
    }
    const int b = base + tid;
    const bool live = b < p.batch;
    int key = 0;
    if (live) key = base == 0 ? key_first : pairs_of(load_seq(p, b).lq);
    // rank among the lanes of this warp that hold the same key (idle lanes use key -1 and are ignored)
    const unsigned same = __match_any_sync(0xffffffffu, live ? key : -1);
    const unsigned rank_in_warp = __popc(same & ((1u << lane) - 1u));
    if (live && rank_in_warp == 0) s_warp[warp][key] = __popc(same);
    __syncthreads();
    if (tid < kBuckets) {
      unsigned acc = s_seen[tid];
      const int live_warps = p.batch - base >= kPreThreads ? 32 : (p.batch - base + 31) / 32;   // (the others hold zeros)
      for (int w = 0; w < live_warps; ++w) {
        const unsigned c = s_warp[w][tid];
        s_warp[w][tid] = acc;
        acc += c;
      }
      s_seen[tid] = acc;
    }
    __syncthreads();
    s_key[tid] = static_cast<unsigned short>(live ? key : 0);
    if (live && key > 0)
      s_first[tid] = p.fwd_by_steps ? (s_before[key] + s_warp[warp][key] + rank_in_warp) * p.hq   // rank * heads
                                    : s_start[key] + (s_warp[warp][key] + rank_in_warp) * key * p.hq;
    __syncthreads();
    // A chunk of few sequences: the items of a sequence are written by a whole warp (a long sequence has hundreds of
    // them, and this kernel's latency is part of every call); a full chunk: every thread writes its own sequence's.
    const int in_chunk = p.batch - base < kPreThreads ? p.batch - base : kPreThreads;
    const bool by_warp = in_chunk <= 256;
    for (int i = by_warp ? warp : tid; i < in_chunk; i += by_warp ? kPreThreads / 32 : kPreThreads) {
      const unsigned wkey = s_key[i];
      const long long first = s_first[i];
      for (unsigned e = by_warp ? lane : 0; e < wkey * p.hq; e += by_warp ? 32 : 1) {   // e = h * key + (key - 1 - pr)
        const unsigned h = e / wkey, pr = wkey - 1u - (e - h * wkey);
        const long long at = p.fwd_by_steps ? static_cast<long long>(s_class[pr + 1u]) + first + h : first + e;
        if (at < p.item_capacity) {
          *reinterpret_cast<uint2*>(p.items + 2 * at) = make_uint2(static_cast<uint32_t>(base + i), (h << 16) | pr);
        }
      }
    }
    __syncthreads();
  }
}

// Pre-pass of the tensor-core backward: input check, and the two tile lists its persistent kernels draw from - the
// (sequence, query head, 128-row q-tile) triples of the dQ pass and the (sequence, kv head, 128-key tile) triples of
// the dK/dV pass, only tiles that exist (a batch of short sequences under a large max_seq_len has few of the
// batch x heads x max_seq_len / 128 slots filled).  Order of a list, as in the forward's: sequences by their number of
// tiles, most first (a counting sort, stable in the sequence index) - the tiles drawn last, when the other CTAs run
// dry, are then the short ones of the shortest sequences; inside a sequence head-major, and inside a head the tiles
// with the most steps first (dQ: the last q-tile; dK/dV: the first keys) - the CTAs that run together then stream the
// same K/V (Q/dO) rows out of L2.  Entry: [sequence, head << 16 | tile].
// header[1] / header[4] = entries of the dQ / dK/dV list, header[2] / header[3] = the two work counters.
constexpr int kMaxTiles = 20480 / kTileM;   // 160
constexpr int kTBuckets = kMaxTiles + 1;

__global__ void __launch_bounds__(kPreThreads) hstu_bwd_prepass_kernel(const KParams p) {
  __shared__ unsigned s_count[kTBuckets];       // sequences per bucket (bucket = number of tiles)
  __shared__ unsigned s_start[kTBuckets];       // first entry of the bucket
  __shared__ unsigned s_before[kTBuckets];      // by steps: sequences with more tiles than the bucket's
  __shared__ unsigned s_class[kTBuckets];       // by steps: first entry of the tiles with `index` steps
  __shared__ unsigned s_seen[kTBuckets];        // sequences of the bucket placed by earlier chunks
  __shared__ unsigned s_warp[32][kTBuckets];    // per-warp counts of the current chunk, then exclusive prefix
  __shared__ unsigned s_first[kPreThreads];     // first entry of each sequence of the chunk
  __shared__ unsigned short s_key[kPreThreads]; // its number of tiles
  __shared__ unsigned s_status;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // (the dQ pass, launched with programmatic stream serialization, may begin its set-up now; it waits for this grid
  // to complete before it reads the lists)
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int all_q = (p.maxq + kTileM - 1) / kTileM;
  if (tid == 0) s_status = 0;
  unsigned st = 0;
#pragma unroll 1
  for (int which = 0; which < 2; ++which) {   // 0: dQ list, 1: dK/dV list
    const int heads = which ? p.hk : p.hq;
    uint32_t* list = which ? p.items + 2 * p.bwd_cap_q : p.items;
    const long long cap = which ? p.bwd_cap_k : p.bwd_cap_q;
    auto tiles_of = [&](int b) -> int {
      const SeqInfo s = load_seq(p, b);
      int n = which ? (s.lk + kTileN - 1) / kTileN : (p.bwd_all_q_tiles ? all_q : (s.lq + kTileM - 1) / kTileM);
      return n > kMaxTiles ? kMaxTiles : n;
    };
    for (int i = tid; i < kTBuckets; i += kPreThreads) {
      s_count[i] = 0;
      s_seen[i] = 0;
    }
    for (int i = tid; i < 32 * kTBuckets; i += kPreThreads) (&s_warp[0][0])[i] = 0;
    __syncthreads();
    int key_first = 0;   // bucket of sequence `tid` (the first chunk of the second pass)
    for (int b = tid; b < p.batch; b += kPreThreads) {
      if (which == 0) st |= check_seq(p, b) | check_pages(p, b);
      const int key = tiles_of(b);
      if (b == tid) key_first = key;
      atomicAdd(&s_count[key], 1u);
    }
    __syncthreads();
    if (warp == 0) {
      // s_start[key] = entries of all larger keys: an exclusive scan from the largest key down, six keys per lane
      unsigned v[6], sum = 0;
#pragma unroll
      for (int i = 0; i < 6; ++i) {
        const int key = kMaxTiles - (6 * lane + i);
        v[i] = key >= 1 ? s_count[key] * static_cast<unsigned>(key) * static_cast<unsigned>(heads) : 0u;
        sum += v[i];
      }
      unsigned incl = sum;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const unsigned o = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += o;
      }
      unsigned run = incl - sum;
#pragma unroll
      for (int i = 0; i < 6; ++i) {
        const int key = kMaxTiles - (6 * lane + i);
        if (key >= 0) s_start[key] = run;
        run += v[i];
      }
      // Ordered by steps (p.bwd_by_steps): the tiles of all sequences with the most steps first - with a few tiles per
      // CTA that is longest-first list scheduling.  A tile with s steps exists once per head in every sequence of at
      // least s tiles, and these sequences are a prefix of the sorted order: entry = s_class[s] + (rank of the
      // sequence in the sorted order) * heads + head.
      {
        unsigned c[6], csum = 0;
#pragma unroll
        for (int i = 0; i < 6; ++i) {
          const int key = kMaxTiles - (6 * lane + i);
          c[i] = key >= 1 ? s_count[key] : 0u;
          csum += c[i];
        }
        unsigned cincl = csum;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const unsigned o = __shfl_up_sync(0xffffffffu, cincl, d);
          if (lane >= d) cincl += o;
        }
        // before[key] = sequences with more tiles; ge = sequences with at least `key` tiles = tiles per head in class
        // `key`; class start = entries of all classes with more steps
        unsigned before = cincl - csum, g[6], gsum = 0;
#pragma unroll
        for (int i = 0; i < 6; ++i) {
          const int key = kMaxTiles - (6 * lane + i);
          if (key >= 0) s_before[key] = before;
          before += c[i];
          g[i] = key >= 1 ? before * static_cast<unsigned>(heads) : 0u;
          gsum += g[i];
        }
        unsigned gincl = gsum;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const unsigned o = __shfl_up_sync(0xffffffffu, gincl, d);
          if (lane >= d) gincl += o;
        }
        unsigned gstart = gincl - gsum;
#pragma unroll
        for (int i = 0; i < 6; ++i) {
          const int key = kMaxTiles - (6 * lane + i);
          if (key >= 0) s_class[key] = gstart;
          gstart += g[i];
        }
      }
      if (lane == 31) {
        // never more than the list holds: offsets that are not monotone can describe more tiles than the tensors have
        // rows for (the host sizes the lists from total_q / total_k); the surplus is dropped, the status word says why
        unsigned total = incl;
        if (static_cast<long long>(total) > cap) total = static_cast<unsigned>(cap);
        p.ws_header[which ? 4 : 1] = total;
        p.ws_header[2 + which] = 0;   // the pass's work counter
      }
    }
    __syncthreads();
    for (int base = 0; base < p.batch; base += kPreThreads) {
      if (base > 0) {
        for (int i = tid; i < 32 * kTBuckets; i += kPreThreads) (&s_warp[0][0])[i] = 0;
        __syncthreads();
      }
      const int b = base + tid;
      const bool live = b < p.batch;
      int key = 0;
      if (live) key = base == 0 ? key_first : tiles_of(b);
      // rank among the lanes of this warp that hold the same key (idle lanes use key -1 and are ignored)
      const unsigned same = __match_any_sync(0xffffffffu, live ? key : -1);
      const unsigned rank_in_warp = __popc(same & ((1u << lane) - 1u));
      if (live && rank_in_warp == 0) s_warp[warp][key] = __popc(same);
      __syncthreads();
      if (tid < kTBuckets) {
        unsigned acc = s_seen[tid];
        const int live_warps = p.batch - base >= kPreThreads ? 32 : (p.batch - base + 31) / 32;   // (the others hold zeros)
        for (int w = 0; w < live_warps; ++w) {
          const unsigned c = s_warp[w][tid];
          s_warp[w][tid] = acc;
          acc += c;
        }
        s_seen[tid] = acc;
      }
      __syncthreads();
      s_key[tid] = static_cast<unsigned short>(live ? key : 0);
      if (live && key > 0)
        s_first[tid] = p.bwd_by_steps ? (s_before[key] + s_warp[warp][key] + rank_in_warp) * heads   // rank * heads
                                      : s_start[key] + (s_warp[warp][key] + rank_in_warp) * key * heads;
      __syncthreads();
      // (few sequences: a warp per sequence - a long one has hundreds of entries; a full chunk: a thread per sequence)
      const int in_chunk = p.batch - base < kPreThreads ? p.batch - base : kPreThreads;
      const bool by_warp = in_chunk <= 256;
      for (int i = by_warp ? warp : tid; i < in_chunk; i += by_warp ? kPreThreads / 32 : kPreThreads) {
        const unsigned wkey = s_key[i];
        const long long first = s_first[i];
        for (unsigned e = by_warp ? lane : 0; e < wkey * heads; e += by_warp ? 32 : 1) {   // e = h * key + t
          const unsigned h = e / wkey, t = e - h * wkey;   // t-th heaviest tile of the head: key - t steps
          const long long at = p.bwd_by_steps ? static_cast<long long>(s_class[wkey - t]) + first + h : first + e;
          if (at < cap) {
            *reinterpret_cast<uint2*>(list + 2 * at) =
                make_uint2(static_cast<uint32_t>(base + i), (h << 16) | (which ? t : wkey - 1u - t));
          }
        }
      }
      __syncthreads();
    }
  }
  if (st) atomicOr(&s_status, st);
  __syncthreads();
  if (tid == 0) p.ws_header[0] = s_status;
}

cudaError_t launch_bwd_prepass(const KParams& p, cudaStream_t stream) {
  hstu_bwd_prepass_kernel<<<1, kPreThreads, 0, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_prepass(const KParams& p, bool build_items, cudaStream_t stream) {
  hstu_prepass_kernel<<<1, kPreThreads, 0, stream>>>(p, build_items ? 1 : 0);
  return cudaGetLastError();
}

// Host mirror of the ordering rule above, on host copies of the index arrays.
long long plan_host(const KParams& p, uint32_t* items, long long capacity, uint32_t* status) {
  unsigned st = 0;
  long long n = 0;
  for (int b = 0; b < p.batch; ++b) st |= check_seq(p, b) | check_pages(p, b);
  if (p.fwd_by_steps) {
    // q-pair number descending over all sequences; inside a number the sequences in the sorted order (most pairs
    // first, stable in the index), heads inside a sequence
    for (int pr = kMaxPairs - 1; pr >= 0; --pr)
      for (int key = kMaxPairs; key > pr; --key)
        for (int b = 0; b < p.batch; ++b) {
          if (pairs_of(load_seq(p, b).lq) != key) continue;
          for (int h = 0; h < p.hq; ++h) {
            if (n < capacity && items) {
              items[2 * n] = static_cast<uint32_t>(b);
              items[2 * n + 1] = (static_cast<uint32_t>(h) << 16) | static_cast<uint32_t>(pr);
            }
            ++n;
          }
        }
    if (status) *status = st;
    return n;
  }
  for (int key = kMaxPairs; key >= 1; --key) {
    for (int b = 0; b < p.batch; ++b) {
      const SeqInfo s = load_seq(p, b);
      if (pairs_of(s.lq) != key) continue;
      for (int h = 0; h < p.hq; ++h) {
        for (int pr = key - 1; pr >= 0; --pr) {
          if (n < capacity && items) {
            items[2 * n] = static_cast<uint32_t>(b);
            items[2 * n + 1] = (static_cast<uint32_t>(h) << 16) | static_cast<uint32_t>(pr);
          }
          ++n;
        }
      }
    }
  }
  if (status) *status = st;
  return n;
}

}  // namespace hstu
