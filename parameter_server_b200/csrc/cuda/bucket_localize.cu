// Skew-aware minibatch localisation without a full sort.
//
// Produces exactly what the sort-based path (radix_sort.cu + localize.cu)
// produces -- the sorted unique key list, CSC segment offsets, the CSR column
// remap, the CSC row index, the head bitmap and the owner slice offsets -- but
// groups the nonzeros instead of sorting them. It replaces the reference's
// Localizer::CountUniqIndex + RemapIndex (util/localizer.h:97-221) and the
// thread merge sort under it (util/parallel_sort.h:14-41) on the hot path.
//
// Why: a click-log minibatch is dominated by a few very frequent keys (under a
// Zipf law the thousand most frequent ids carry half of the nonzeros) while most
// distinct keys occur once or twice. An LSD radix sort moves every nonzero once
// per digit; here a nonzero is moved once.
//
//   1. sample     a strided sample of the keys is counted in a small global hash
//                 table; keys that occur often in it become "hot" (at most 2048).
//   2. count      every CTA walks a contiguous slice of the input and counts, in
//                 shared memory, its nonzeros per hot key and, for all others
//                 ("cold"), per bucket (bucket = top bits of the key, so buckets
//                 are ordered by key).
//   3. scan/plan  prefix sums give every CTA a private output cursor per bin (no
//                 look-back chain), every bucket its output range, every hot key
//                 its place in the hot stream.
//   4. scatter    the same walk again: a cold nonzero goes to its bucket as one
//                 64-bit word (key | position), a hot nonzero's position goes to
//                 its key's list.
//   5. bucket     one CTA per bucket: a shared-memory table de-duplicates the
//                 bucket's keys and counts them. The table is order preserving
//                 (home slot = leading bits of the key, linear probing without
//                 wrap-around), so the occupied slots read in address order are
//                 sorted up to a permutation inside each run of adjacent slots;
//                 a key's rank is a prefix count plus a look at its own run, and
//                 nothing is sorted. Hot keys that fall into the bucket are
//                 merged in, a chained scan over the buckets (decoupled
//                 look-back, in ticket order) gives the global index of the
//                 bucket's first unique key, and every nonzero is written to its
//                 final CSC position.
//   6. hot emit   the hot keys' position lists are written to the CSC ranges
//                 that step 5 reserved for them.
//
// Inside a key's CSC segment the nonzeros are in no particular order (the sort
// based path lists them by position).
//
// When the keys are not spread evenly over the key space (a bucket far above the
// average), or a bucket holds more distinct keys than its table can take, a
// device flag is raised, the remaining steps return at once, and the caller's
// gated sort-based path (psb_sort_pairs_gated + psb_localize2_gated) does the
// work instead. Every spin is bounded and reports through the status word.
#include "psb_common.cuh"
#include "psb_cuda.h"

namespace psb {

static constexpr u32 kSampSlots = 1u << 17;       // sample hash table (global memory)
static constexpr u32 kSampMax = 1u << 16;         // elements sampled
static constexpr u32 kHotSlots = 4096;            // hot-key lookup table (open addressing)
static constexpr u32 kHotMax = 2048;              // hot keys at most
static constexpr int kWalkThreads = 1024;         // count / scatter CTAs
static constexpr int kBucketThreads = 256;
static constexpr u32 kRunMax = 64;                // longest probe sequence / run of adjacent occupied slots
static constexpr u32 kMaxBuckets = 8192;
// A bucket's table comes in two sizes. 2^11 home slots (35 KB of shared memory, six CTAs per SM) serve
// minibatches in which keys repeat, the usual case; 2^12 (55 KB, four per SM) those in which nearly
// every nonzero has its own key. The sample decides (k_bl_plan), both kernels are launched and the
// one that was not chosen returns at once.
template <int kBits> struct BucketShape {
  static constexpr u32 kHs = 1u << kBits;                  // home slots
  static constexpr u32 kHsAll = kHs + 2 * kRunMax;         // plus the spill area behind the last home slot
  static constexpr u32 kHsWords = kHsAll / 32;             // occupancy bitmap words
  static constexpr u32 kDistinctMax = kHs / 2;             // distinct keys a bucket may hold
  static constexpr int kEntriesPerThread = kDistinctMax / kBucketThreads;
  static constexpr size_t smem_bytes(size_t key_bytes) {
    return kHsAll * (key_bytes + 4 + 2) + kDistinctMax * (4 + 2) + 2 * kHsWords * 4;
  }
};
static constexpr u32 kFlagAgg = 1u << 30;
static constexpr u32 kFlagIncl = 2u << 30;
static constexpr u32 kValMask = (1u << 30) - 1;

// control words
enum { kCtlNumHot = 0, kCtlTicket = 1, kCtlFallback = 2, kCtlHotElems = 3, kCtlSampleDistinct = 4, kCtlBigTables = 5,
       kCtlWords = 16 };

struct BLP {
  // input
  const void* in;
  int in_kind;            // 0 = uint64 keys, 1 = uint32 ids (hashed), 2 = uint64 ids (hashed)
  u64 seed;
  u32 n;
  int lo;                 // low key bits that are always zero (they carry the position when packed)
  int packed;
  int nb_bits;            // log2(number of buckets)
  u32 NB, NBINS;          // buckets; NB + kHotMax
  u32 G, chunk;           // walk CTAs and elements per CTA
  u32 samp_m, samp_stride, hot_thresh, cold_limit;
  // rows
  const u32* row_ptr; u32 n_rows, fixed_z;
  const float* vals;
  // scratch
  u64* samp_key; u32* samp_cnt;
  u64* hot_tab; unsigned short* hot_idx; u64* hot_key;
  u32* ctl;
  u32* part;              // [G][NBINS]
  u32* bin_total;         // [NBINS]
  u32* cold_base;         // [NB + 1]
  u32* pos_base;          // [NB + 1]
  u32* hot_base;          // [kHotMax + 1]
  u64* shot_key; u32* shot_h;       // hot keys sorted by key
  u32* bucket_hot_off;    // [NB + 1]
  u32* hot_u; u32* hot_seg;         // [kHotMax]
  u32* bstate;            // [NB]
  u64* cold_words; u32* cold_pos; u32* hot_pos;
  // outputs
  u64* ukeys; u32* seg_off; u32* csr_col; u32* csc_row; float* csc_val;
  u32* flagbits; u32* wordbase; u32* n_unique;
  u32* status;
};

__device__ __forceinline__ u64 bl_key_of(const BLP& p, u32 i) {
  if (p.in_kind == 0) return ((const u64*)p.in)[i];
  u64 id = p.in_kind == 1 ? (u64)((const u32*)p.in)[i] : ((const u64*)p.in)[i];
  return hash_id_to_key(id, p.seed);
}
__device__ __forceinline__ u32 hot_home(u64 key) {
  return (((u32)(key >> 32) ^ (u32)key) * 0x9E3779B1u) >> 20;   // 12 bits = kHotSlots
}
__device__ __forceinline__ u32 row_of_pos(const BLP& p, u32 pos, u32 zinv) {
  if (p.row_ptr == nullptr) {
    u32 r = __umulhi(pos, zinv);
    while (pos - r * p.fixed_z >= p.fixed_z) ++r;              // the estimate is at most two short
    return r;
  }
  u32 lo = 0, hi = p.n_rows;                                   // largest r with row_ptr[r] <= pos
  while (hi - lo > 1) {
    u32 mid = (lo + hi) >> 1;
    if (p.row_ptr[mid] <= pos) lo = mid; else hi = mid;
  }
  return lo;
}

// ---------------------------------------------------------------- 1. sample
__global__ void __launch_bounds__(256) k_bl_sample(const BLP p) {
  const u32 j = blockIdx.x * blockDim.x + threadIdx.x;
  const bool valid = j < p.samp_m;
  const u64 key = valid ? bl_key_of(p, j * p.samp_stride) : kEmptyKey;
  // equal keys of a warp count once (the most frequent key would otherwise take thousands of
  // atomics on one address)
  const u32 m = __match_any_sync(0xffffffffu, key);
  if (!valid || (int)(threadIdx.x & 31) != __ffs(m) - 1) return;
  u32 slot = (u32)(fmix64(key) & (kSampSlots - 1));
  for (u32 probe = 0; probe < kSampSlots; ++probe) {
    u64 old = atomicCAS(&p.samp_key[slot], kEmptyKey, key);
    if (old == kEmptyKey || old == key) { atomicAdd(&p.samp_cnt[slot], (u32)__popc(m)); return; }
    slot = (slot + 1) & (kSampSlots - 1);
  }
}

__global__ void __launch_bounds__(256) k_bl_hot(const BLP p) {
  const u32 s = blockIdx.x * blockDim.x + threadIdx.x;
  const u32 c = s < kSampSlots ? p.samp_cnt[s] : 0u;
  // distinct keys of the sample (how much keys repeat decides the size of the buckets' tables)
  const u32 occ = __ballot_sync(0xffffffffu, c > 0);
  if ((threadIdx.x & 31) == 0 && occ) atomicAdd(&p.ctl[kCtlSampleDistinct], (u32)__popc(occ));
  if (c < p.hot_thresh) return;
  const u64 key = p.samp_key[s];
  const u32 h = atomicAdd(&p.ctl[kCtlNumHot], 1u);
  if (h >= kHotMax) return;                                    // more candidates than places: the rest stay cold
  p.hot_key[h] = key;
  u32 slot = hot_home(key);
  for (u32 probe = 0; probe < kHotSlots; ++probe) {
    u64 old = atomicCAS(&p.hot_tab[slot], kEmptyKey, key);
    if (old == kEmptyKey) { p.hot_idx[slot] = (unsigned short)h; return; }
    slot = (slot + 1) & (kHotSlots - 1);
  }
}

// ---------------------------------------------------------------- 2./4. the two walks
// Shared-memory layout of a walk CTA: hot table keys | hot index per slot | one word per bin.
// kScatter = false: count. kScatter = true: the words start as this CTA's output cursors.
template <bool kScatter>
__global__ void __launch_bounds__(kWalkThreads) k_bl_walk(const BLP p) {
  extern __shared__ __align__(16) unsigned char smem[];
  u64* s_hot = reinterpret_cast<u64*>(smem);
  unsigned short* s_hidx = reinterpret_cast<unsigned short*>(smem + kHotSlots * 8);
  u32* s_bin = reinterpret_cast<u32*>(smem + kHotSlots * 8 + kHotSlots * 2);
  if (kScatter && p.ctl[kCtlFallback]) return;
  const u32 nh = min(p.ctl[kCtlNumHot], kHotMax);
  const int t = threadIdx.x, lane = t & 31;
  for (u32 i = t; i < kHotSlots; i += kWalkThreads) { s_hot[i] = p.hot_tab[i]; s_hidx[i] = p.hot_idx[i]; }
  u32* my_part = p.part + (size_t)blockIdx.x * p.NBINS;
  for (u32 i = t; i < p.NBINS; i += kWalkThreads) {
    u32 v = 0;
    if (kScatter) v = my_part[i] + (i < p.NB ? p.cold_base[i] : p.hot_base[i - p.NB]);
    s_bin[i] = v;
  }
  __syncthreads();
  const u32 begin = blockIdx.x * p.chunk;
  const u32 end = min(p.n, begin + p.chunk);
  const int bshift = 64 - p.nb_bits;
  // One element: look the key up among the hot keys, then count it (or, when scattering, take an
  // output place from the bin's cursor and store it).
  auto handle = [&](u64 key, u32 pos, bool valid) {
    bool hot = false;
    u32 bin = (u32)(key >> bshift);
    if (valid && nh) {
      u32 slot = hot_home(key);
      for (u32 probe = 0; probe < kHotSlots; ++probe) {
        const u64 k = s_hot[slot];
        if (k == key) { hot = true; bin = p.NB + s_hidx[slot]; break; }
        if (k == kEmptyKey) break;
        slot = (slot + 1) & (kHotSlots - 1);
      }
    }
    // plain shared-memory atomics, also for the hot keys: lanes that hit one address serialise
    // inside the instruction, which costs far less than finding the groups first
    u32 dst = 0;
    if (valid) dst = atomicAdd(&s_bin[bin], 1u);
    if (kScatter && valid) {
      if (hot) {
        p.hot_pos[dst] = pos;
      } else if (p.packed) {
        p.cold_words[dst] = key | (u64)pos;
      } else {
        p.cold_words[dst] = key;
        p.cold_pos[dst] = pos;
      }
    }
  };
  // Four consecutive elements per thread and trip; every lane of a warp makes the same number of trips.
  const u32 first = begin + 4u * (u32)(t - lane);
  const u32 step = 4u * kWalkThreads;
  if (p.in_kind == 1 && (((size_t)p.in) & 15) == 0) {
    // 32-bit ids: one 16-byte load per trip, the next trip's load in flight while this one is handled
    const u32* ids = (const u32*)p.in;
    uint4 cur = make_uint4(0, 0, 0, 0);
    {
      const u32 i = first + 4u * lane;
      if (first < end && i + 3 < end) cur = *reinterpret_cast<const uint4*>(ids + i);
    }
    for (u32 i0 = first; i0 < end; i0 += step) {
      const u32 i = i0 + 4u * lane;
      uint4 nxt = make_uint4(0, 0, 0, 0);
      const u32 in_ = i + step;
      if (i0 + step < end && in_ + 3 < end) nxt = *reinterpret_cast<const uint4*>(ids + in_);
      u32 id[4] = {cur.x, cur.y, cur.z, cur.w};
      if (!(i + 3 < end)) {
#pragma unroll
        for (int q = 0; q < 4; ++q) id[q] = (i + q < end) ? ids[i + q] : 0u;
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) handle(hash_id_to_key(id[q], p.seed), i + q, i + q < end);
      cur = nxt;
    }
  } else {
    for (u32 i0 = first; i0 < end; i0 += step) {
      const u32 i = i0 + 4u * lane;
      u64 key[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) key[q] = (i + q < end) ? bl_key_of(p, i + q) : 0;
#pragma unroll
      for (int q = 0; q < 4; ++q) handle(key[q], i + q, i + q < end);
    }
  }
  if (!kScatter) {
    __syncthreads();
    for (u32 i = t; i < p.NBINS; i += kWalkThreads) my_part[i] = s_bin[i];
  }
}

// ---------------------------------------------------------------- 3. scan + plan
// Per bin: exclusive prefix over the walk CTAs (in place) and the bin's total.
__global__ void __launch_bounds__(256) k_bl_scan(const BLP p) {
  const u32 bin = blockIdx.x * blockDim.x + threadIdx.x;
  if (bin >= p.NBINS) return;
  u32 run = 0;
  // sixteen CTAs' counts are fetched before the first prefix is stored
  for (u32 c0 = 0; c0 < p.G; c0 += 16) {
    u32 v[16];
#pragma unroll
    for (int k = 0; k < 16; ++k) v[k] = (c0 + k < p.G) ? p.part[(size_t)(c0 + k) * p.NBINS + bin] : 0u;
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      if (c0 + k < p.G) p.part[(size_t)(c0 + k) * p.NBINS + bin] = run;
      run += v[k];
    }
  }
  p.bin_total[bin] = run;
}

// Exclusive scan, in place, of the shared-memory array a[0..n) by one CTA of 1024 threads (n a multiple
// of 1024 or below it); returns the total to every thread.
__device__ u32 smem_scan_1024(u32* a, u32 n, u32* s_tmp /* 33 words */) {
  const int t = threadIdx.x, lane = t & 31, w = t >> 5;
  const u32 per = (n + 1023) / 1024;
  const u32 b = min(n, t * per), e = min(n, b + per);
  u32 sum = 0;
  for (u32 i = b; i < e; ++i) sum += a[i];
  u32 x = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    u32 y = __shfl_up_sync(0xffffffffu, x, o);
    if (lane >= o) x += y;
  }
  __syncthreads();          // s_tmp may still be read from the previous call
  if (lane == 31) s_tmp[w] = x;
  __syncthreads();
  if (w == 0) {
    u32 v = s_tmp[lane], xs = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      u32 y = __shfl_up_sync(0xffffffffu, xs, o);
      if (lane >= o) xs += y;
    }
    s_tmp[lane] = xs - v;
    if (lane == 31) s_tmp[32] = xs;
  }
  __syncthreads();
  u32 run = s_tmp[w] + x - sum;
  for (u32 i = b; i < e; ++i) { u32 v = a[i]; a[i] = run; run += v; }
  __syncthreads();
  return s_tmp[32];
}

// One CTA: the hot keys grouped by bucket, the hot stream's offsets, and per bucket the cold stream
// offset, the final output offset and its first hot key. All scans run in shared memory.
__global__ void __launch_bounds__(1024) k_bl_plan(const BLP p) {
  extern __shared__ __align__(16) unsigned char smem[];
  u32* s_a = reinterpret_cast<u32*>(smem);          // [NB] cold totals -> cold offsets -> cursors
  u32* s_b = s_a + p.NB;                            // [NB] hot nonzeros per bucket -> output offsets
  u32* s_c = s_b + p.NB;                            // [NB] hot keys per bucket -> first hot key
  __shared__ u32 s_ht[kHotMax];
  __shared__ u32 s_tmp[33];
  __shared__ u32 s_max;
  const int t = threadIdx.x;
  const u32 nh = min(p.ctl[kCtlNumHot], kHotMax);
  const int bshift = 64 - p.nb_bits;
  if (t == 0) s_max = 0;
  // all global loads first: this thread's hot keys and totals (two at most), then the cold totals
  u64 hk[kHotMax / 1024];
  u32 ht[kHotMax / 1024];
#pragma unroll
  for (int k = 0; k < (int)(kHotMax / 1024); ++k) {
    const u32 i = t + k * 1024;
    hk[k] = i < nh ? p.hot_key[i] : 0;
    ht[k] = i < nh ? p.bin_total[p.NB + i] : 0u;
  }
  u32 mx = 0;
  for (u32 b0 = t; b0 < p.NB; b0 += 4 * 1024) {
    u32 c[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) c[k] = (b0 + k * 1024 < p.NB) ? p.bin_total[b0 + k * 1024] : 0u;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const u32 b = b0 + k * 1024;
      if (b < p.NB) { s_a[b] = c[k]; s_b[b] = 0; s_c[b] = 0; mx = max(mx, c[k]); }
    }
  }
#pragma unroll
  for (int k = 0; k < (int)(kHotMax / 1024); ++k) s_ht[t + k * 1024] = ht[k];
  __syncthreads();
  atomicMax(&s_max, mx);
#pragma unroll
  for (int k = 0; k < (int)(kHotMax / 1024); ++k) {
    if (t + k * 1024 < (int)nh) {
      const u32 b = (u32)(hk[k] >> bshift);
      atomicAdd(&s_b[b], ht[k]);
      atomicAdd(&s_c[b], 1u);
    }
  }
  __syncthreads();
  for (u32 b = t; b < p.NB; b += 1024) s_b[b] += s_a[b];
  __syncthreads();
  const u32 cold_total = smem_scan_1024(s_a, p.NB, s_tmp);
  const u32 all_total = smem_scan_1024(s_b, p.NB, s_tmp);
  const u32 hk_total = smem_scan_1024(s_c, p.NB, s_tmp);
  for (u32 b = t; b < p.NB; b += 1024) {
    p.cold_base[b] = s_a[b]; p.pos_base[b] = s_b[b]; p.bucket_hot_off[b] = s_c[b];
    s_a[b] = 0;
  }
  if (t == 0) { p.cold_base[p.NB] = cold_total; p.pos_base[p.NB] = all_total; p.bucket_hot_off[p.NB] = hk_total; }
  __syncthreads();
  // hot keys grouped by bucket (any order inside a bucket: the bucket kernel puts them into its table)
#pragma unroll
  for (int k = 0; k < (int)(kHotMax / 1024); ++k) {
    const u32 i = t + k * 1024;
    if (i < nh) {
      const u32 b = (u32)(hk[k] >> bshift);
      const u32 at = s_c[b] + atomicAdd(&s_a[b], 1u);
      p.shot_key[at] = hk[k];
      p.shot_h[at] = i;
    }
  }
  // hot stream offsets, in hot-index order
  const u32 hot_total = smem_scan_1024(s_ht, kHotMax, s_tmp);
  for (u32 i = t; i < kHotMax; i += 1024) p.hot_base[i] = s_ht[i];
  if (t == 0) {
    p.hot_base[kHotMax] = hot_total;
    p.ctl[kCtlHotElems] = hot_total;
    if (s_max > p.cold_limit) p.ctl[kCtlFallback] = 1;   // keys are not spread evenly: use the sort
    // more than three quarters of the sampled nonzeros have a key of their own: the big tables
    p.ctl[kCtlBigTables] = (4ull * p.ctl[kCtlSampleDistinct] > 3ull * p.samp_m) ? 1u : 0u;
  }
}

// ---------------------------------------------------------------- 5. per-bucket grouping
template <typename CK> struct CkT;
template <> struct CkT<u32> { static constexpr u32 kEmpty = 0xFFFFFFFFu; };
template <> struct CkT<u64> { static constexpr u64 kEmpty = 0xFFFFFFFFFFFFFFFFull; };

// Home slot of a compact key with `rem` significant bits: its leading kBits bits (order preserving).
template <typename CK, int kBits>
__device__ __forceinline__ u32 bucket_home(CK ck, int rem) {
  return rem >= kBits ? (u32)(ck >> (rem - kBits)) : (u32)(ck << (kBits - rem));
}

template <typename CK, int kBits>
__device__ __forceinline__ int bucket_find(const CK* s_key, CK ck, int rem) {
  u32 slot = bucket_home<CK, kBits>(ck, rem);
  for (u32 probe = 0; probe < kRunMax; ++probe, ++slot) {
    const CK k = s_key[slot];
    if (k == ck) return (int)slot;
    if (k == CkT<CK>::kEmpty) return -1;
  }
  return -1;
}

// Finds or inserts ck; returns the slot, or -1 when the probe sequence got longer than kRunMax
// (keys that are not spread evenly inside the bucket). A new key sets its bit in the occupancy bitmap.
template <typename CK, int kBits>
__device__ __forceinline__ int bucket_insert(CK* s_key, u32* s_bits, CK ck, int rem) {
  u32 slot = bucket_home<CK, kBits>(ck, rem);
  for (u32 probe = 0; probe < kRunMax; ++probe, ++slot) {
    CK k = s_key[slot];
    if (k == ck) return (int)slot;
    if (k == CkT<CK>::kEmpty) {
      k = atomicCAS(&s_key[slot], CkT<CK>::kEmpty, ck);
      if (k == CkT<CK>::kEmpty) { atomicOr(&s_bits[slot >> 5], 1u << (slot & 31)); return (int)slot; }
      if (k == ck) return (int)slot;
    }
  }
  return -1;
}

// Exclusive block scan of one value per thread (kBucketThreads threads); total to every thread.
__device__ __forceinline__ u32 bucket_block_scan(u32 v, u32* s_warp /* 9 words */, u32* total) {
  const int t = threadIdx.x, lane = t & 31, w = t >> 5;
  u32 x = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    u32 y = __shfl_up_sync(0xffffffffu, x, o);
    if (lane >= o) x += y;
  }
  __syncthreads();
  if (lane == 31) s_warp[w] = x;
  __syncthreads();
  u32 pre = x - v, tot = 0;
#pragma unroll
  for (int i = 0; i < kBucketThreads / 32; ++i) { const u32 sw = s_warp[i]; if (i < w) pre += sw; tot += sw; }
  *total = tot;
  return pre;
}

template <typename CK, int kBits>
__global__ void __launch_bounds__(kBucketThreads) k_bl_bucket(const BLP p) {
  typedef BucketShape<kBits> Sh;
  constexpr u32 kHsAll = Sh::kHsAll, kHsWords = Sh::kHsWords, kDistinctMax = Sh::kDistinctMax;
  constexpr int kEntriesPerThread = Sh::kEntriesPerThread;
  extern __shared__ __align__(16) unsigned char smem[];
  CK* s_key = reinterpret_cast<CK*>(smem);                                     // table: compact keys
  u32* s_cnt = reinterpret_cast<u32*>(s_key + kHsAll);                         // per slot: count, then cursor
  u32* s_start = s_cnt + kHsAll;                                               // per distinct key, slot order
  u32* s_bits = s_start + kDistinctMax;                                        // occupancy bitmap
  u32* s_hbits = s_bits + kHsWords;                                            // slots that hold a hot key
  unsigned short* s_rank = reinterpret_cast<unsigned short*>(s_hbits + kHsWords);  // per slot: hot index, then rank
  unsigned short* s_dense = s_rank + kHsAll;                                   // occupied slots in slot order
  __shared__ u32 s_ovf, s_b, s_ubase, s_warp[kBucketThreads / 32 + 1];
  const int t = threadIdx.x, lane = t & 31, w = t >> 5;
  // A CTA takes buckets by ticket until none is left (a few CTAs per SM are launched, not one per bucket).
  for (;;) {
  if (t == 0) {
    // one thread reads the flags for the whole CTA: other CTAs may raise the fallback flag at any moment
    const bool mine = (p.ctl[kCtlBigTables] != 0) == (kBits == 12);
    s_b = (!mine || ld_relaxed_gpu(&p.ctl[kCtlFallback])) ? 0xFFFFFFFFu : atomicAdd(&p.ctl[kCtlTicket], 1u);
    s_ovf = 0;
  }
  {
    // keys = all ones, counts = 0, bitmaps = 0, with 16-byte stores (while the ticket is on its way)
    uint4* k4 = reinterpret_cast<uint4*>(s_key);
    const u32 nk4 = kHsAll * sizeof(CK) / 16;
    for (u32 i = t; i < nk4; i += kBucketThreads) k4[i] = make_uint4(~0u, ~0u, ~0u, ~0u);
    uint4* c4 = reinterpret_cast<uint4*>(s_cnt);
    for (u32 i = t; i < kHsAll / 4; i += kBucketThreads) c4[i] = make_uint4(0, 0, 0, 0);
    for (u32 i = t; i < 2 * kHsWords; i += kBucketThreads) s_bits[i] = 0;
  }
  __syncthreads();
  const u32 b = s_b;
  if (b >= p.NB) return;
  const u32 cb = p.cold_base[b], nb = p.cold_base[b + 1] - cb;
  const u32 pb = p.pos_base[b];
  const u32 h0 = p.bucket_hot_off[b], h1 = p.bucket_hot_off[b + 1];
  const int sh_l = p.nb_bits, sh_r = p.nb_bits + p.lo;
  const int rem = 64 - sh_r;                    // significant bits of a compact key
  const u64 posmask = p.packed ? ((1ull << p.lo) - 1) : 0ull;
  // The first four nonzeros of every thread stay in registers for both passes over the bucket
  // (a bucket of average size has no more), the rest is read again in pass 2.
  u64 w0[4];
  u32 p0[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const u32 j = t + q * kBucketThreads;
    w0[q] = j < nb ? p.cold_words[cb + j] : 0;
    p0[q] = (j < nb && !p.packed) ? p.cold_pos[cb + j] : 0;
  }
  // hot keys of this bucket enter the table with their total count
  for (u32 i = h0 + t; i < h1; i += kBucketThreads) {
    const u32 h = p.shot_h[i];
    const CK ck = (CK)((p.shot_key[i] << sh_l) >> sh_r);
    const int slot = bucket_insert<CK, kBits>(s_key, s_bits, ck, rem);
    if (slot < 0) { s_ovf = 1; continue; }
    s_cnt[slot] = p.bin_total[p.NB + h];
    s_rank[slot] = (unsigned short)h;
    atomicOr(&s_hbits[slot >> 5], 1u << (slot & 31));
  }
  // pass 1 over the bucket's nonzeros: distinct keys and their counts
  for (u32 j0 = t; j0 < nb; j0 += 4 * kBucketThreads) {
    u64 wd[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const u32 j = j0 + q * kBucketThreads;
      wd[q] = j0 == (u32)t ? w0[q] : (j < nb ? p.cold_words[cb + j] : 0);
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const u32 j = j0 + q * kBucketThreads;
      if (j >= nb) break;
      const CK ck = (CK)((wd[q] << sh_l) >> sh_r);
      const int slot = bucket_insert<CK, kBits>(s_key, s_bits, ck, rem);
      if (slot < 0) { s_ovf = 1; continue; }
      atomicAdd(&s_cnt[slot], 1u);
    }
  }
  __syncthreads();
  // occupied slots in slot order: prefix over the bitmap words, then one thread per word lists its slots
  u32 d = 0;
  const u32 myw = t < (int)kHsWords ? s_bits[t] : 0u;
  const u32 wpre = bucket_block_scan((u32)__popc(myw), s_warp, &d);
  if (d > kDistinctMax && t == 0) s_ovf = 1;
  __syncthreads();
  if (s_ovf) {
    // keys bunched inside the bucket (or too many of them): hand the whole minibatch to the sort-based path
    if (t == 0) { st_relaxed_gpu(&p.ctl[kCtlFallback], 1u); st_relaxed_gpu(&p.bstate[b], kFlagIncl); }
    return;
  }
  // the bucket's number of unique keys is known: publish it for the buckets behind
  if (t == 0) st_relaxed_gpu(&p.bstate[b], (b == 0 ? kFlagIncl : kFlagAgg) | d);
  {
    u32 wbits = myw, k = wpre;
    while (wbits) {
      const int bit = __ffs(wbits) - 1;
      s_dense[k++] = (unsigned short)(32 * t + bit);
      wbits &= wbits - 1;
    }
  }
  __syncthreads();
  // nonzeros before every distinct key, in slot order (a thread takes adjacent entries)
  const u32 ipt = (d + kBucketThreads - 1) / kBucketThreads;
  const u32 i0 = min(d, (u32)t * ipt), i1 = min(d, i0 + ipt);
  u32 sum = 0;
  for (u32 i = i0; i < i1; ++i) sum += s_cnt[s_dense[i]];
  u32 dummy;
  u32 run = bucket_block_scan(sum, s_warp, &dummy);
  for (u32 i = i0; i < i1; ++i) { s_start[i] = run; run += s_cnt[s_dense[i]]; }
  __syncthreads();
  // Rank and segment start of every distinct key: the prefix at the first entry of its run of adjacent
  // occupied slots, plus the smaller keys of that run (a run is a permutation of its sorted order).
  u32 my_rank[kEntriesPerThread], my_start[kEntriesPerThread];
  bool bad = false;
#pragma unroll
  for (int k = 0; k < kEntriesPerThread; ++k) {
    const u32 i = t + k * kBucketThreads;
    my_rank[k] = 0xFFFFFFFFu; my_start[k] = 0;
    if (i >= d) continue;
    const u32 slot = s_dense[i];
    const CK key = s_key[slot];
    u32 j = i;                                      // first entry of the run
    while (j > 0 && (u32)s_dense[j - 1] + 1 == (u32)s_dense[j]) {
      --j;
      if (i - j > 2 * kRunMax) { bad = true; break; }
    }
    u32 r = j, st = s_start[j];
    for (u32 q = j; q < d; ++q) {
      if (q > j && (u32)s_dense[q - 1] + 1 != (u32)s_dense[q]) break;
      if (q - j > 4 * kRunMax) { bad = true; break; }
      const u32 sq = s_dense[q];
      if (s_key[sq] < key) { ++r; st += s_cnt[sq]; }
    }
    my_rank[k] = r; my_start[k] = st;
  }
  if (bad) s_ovf = 1;
  // unique keys in all buckets before this one: look back over the published counts, 32 buckets per trip
  if (w == 0) {
    u32 ex = 0;
    if (b > 0) {
      long long q = (long long)b - 1;
      u32 spins = 0;
      bool done = false;
      while (!done && q >= 0) {
        const long long idx = q - lane;
        u32 v = kFlagIncl;
        if (idx >= 0) asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p.bstate + idx));
        const u32 f = v & ~kValMask;
        const u32 empty = __ballot_sync(0xffffffffu, f == 0);
        const u32 incl = __ballot_sync(0xffffffffu, f == kFlagIncl);
        const int first_empty = empty ? __ffs(empty) - 1 : 32;
        const int first_incl = incl ? __ffs(incl) - 1 : 32;
        const int upto = first_incl < first_empty ? first_incl + 1 : first_empty;   // lanes [0, upto) are usable
        u32 add = lane < upto ? (v & kValMask) : 0u;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) add += __shfl_xor_sync(0xffffffffu, add, o);
        ex += add;
        if (first_incl < first_empty) done = true;
        else {
          q -= upto;
          if (upto == 0) {
            // a bucket that gave up (or never started because of that) publishes nothing: stop waiting
            if (ld_relaxed_gpu(&p.ctl[kCtlFallback])) break;
            if (++spins > kGridWaitIters) { if (lane == 0) set_status(p.status, kLookbackTimeout); break; }
            __nanosleep(40);
          }
        }
      }
      if (lane == 0) st_relaxed_gpu(&p.bstate[b], kFlagIncl | ((ex + d) & kValMask));
    }
    if (lane == 0) {
      s_ubase = ex;
      if (b == p.NB - 1) *p.n_unique = ex + d;
    }
  }
  __syncthreads();
  if (s_ovf) {
    if (t == 0) st_relaxed_gpu(&p.ctl[kCtlFallback], 1u);
    return;
  }
  const u32 ub = s_ubase;
  const u64 bucket_bits = (u64)b << (64 - p.nb_bits);
#pragma unroll
  for (int k = 0; k < kEntriesPerThread; ++k) {
    if (my_rank[k] == 0xFFFFFFFFu) continue;
    const u32 slot = s_dense[t + k * kBucketThreads];
    const u32 c = s_cnt[slot];
    const bool is_hot = (s_hbits[slot >> 5] >> (slot & 31)) & 1u;
    const u32 hh = is_hot ? s_rank[slot] : 0u;
    const u32 start = my_start[k];
    s_cnt[slot] = start;
    s_rank[slot] = (unsigned short)my_rank[k];
    const u32 u = ub + my_rank[k], P = pb + start;
    p.ukeys[u] = bucket_bits | ((u64)s_key[slot] << p.lo);
    p.seg_off[u] = P;
    atomicOr(&p.flagbits[P >> 5], 1u << (P & 31));
    if (is_hot) {
      p.hot_u[hh] = u;          // the hot emit kernel fills this segment (and its wordbase words)
      p.hot_seg[hh] = P;
    } else {
      // number of segment heads before every 32-aligned position inside the segment
      for (u32 wd = (P + 31) >> 5; (wd << 5) < P + c; ++wd) p.wordbase[wd] = ((wd << 5) == P) ? u : u + 1;
    }
  }
  __syncthreads();
  // pass 2: every nonzero to its place
  const u32 zinv = p.fixed_z ? (u32)(0xffffffffu / p.fixed_z) : 0u;
  for (u32 j0 = t; j0 < nb; j0 += 4 * kBucketThreads) {
    u64 wd[4];
    u32 ps[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const u32 j = j0 + q * kBucketThreads;
      const bool first = j0 == (u32)t;
      wd[q] = first ? w0[q] : (j < nb ? p.cold_words[cb + j] : 0);
      ps[q] = first ? p0[q] : ((j < nb && !p.packed) ? p.cold_pos[cb + j] : 0);
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const u32 j = j0 + q * kBucketThreads;
      if (j >= nb) break;
      const CK ck = (CK)((wd[q] << sh_l) >> sh_r);
      const int slot = bucket_find<CK, kBits>(s_key, ck, rem);
      if (slot < 0) continue;                     // cannot happen: the key was inserted in pass 1
      const u32 pos = p.packed ? (u32)(wd[q] & posmask) : ps[q];
      const u32 P = pb + atomicAdd(&s_cnt[slot], 1u);
      const u32 u = ub + s_rank[slot];
      p.csc_row[P] = row_of_pos(p, pos, zinv);
      p.csr_col[pos] = u;
      if (p.csc_val) p.csc_val[P] = p.vals[pos];
    }
  }
  __syncthreads();       // the tables are rebuilt for the next bucket
  }
}

// ---------------------------------------------------------------- 6. hot keys' position lists
__global__ void __launch_bounds__(256) k_bl_hot_emit(const BLP p) {
  __shared__ u32 s_base[kHotMax + 1];
  __shared__ u32 s_u[kHotMax], s_seg[kHotMax];
  if (p.ctl[kCtlFallback]) return;
  const u32 nh = min(p.ctl[kCtlNumHot], kHotMax);
  if (nh == 0) return;
  for (u32 i = threadIdx.x; i <= nh; i += blockDim.x) s_base[i] = p.hot_base[i];
  for (u32 i = threadIdx.x; i < nh; i += blockDim.x) { s_u[i] = p.hot_u[i]; s_seg[i] = p.hot_seg[i]; }
  __syncthreads();
  const u32 total = s_base[nh];
  const u32 zinv = p.fixed_z ? (u32)(0xffffffffu / p.fixed_z) : 0u;
  // A warp walks one contiguous piece of the hot stream, 4 x 32 positions per trip. The stream is
  // grouped by hot key, so the key index only ever moves forward: one binary search at the start.
  const int lane = threadIdx.x & 31;
  const u32 nwarps = gridDim.x * (blockDim.x >> 5);
  const u32 gw = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const u32 piece = ((total + nwarps - 1) / nwarps + 127) & ~127u;
  const u32 begin = min(total, gw * piece), end = min(total, begin + piece);
  if (begin >= end) return;
  u32 h;
  {
    u32 lo = 0, hi = nh;                            // largest h with s_base[h] <= begin
    while (hi - lo > 1) {
      u32 mid = (lo + hi) >> 1;
      if (s_base[mid] <= begin) lo = mid; else hi = mid;
    }
    h = lo;
  }
  for (u32 j0 = begin + lane; j0 < end + lane; j0 += 128) {
    u32 pos[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const u32 j = j0 + q * 32;
      pos[q] = j < end ? __ldcs(&p.hot_pos[j]) : 0u;
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const u32 j = j0 + q * 32;
      if (j >= end) break;
      while (h + 1 < nh && s_base[h + 1] <= j) ++h;
      const u32 u = s_u[h];
      const u32 P = s_seg[h] + (j - s_base[h]);
      p.csc_row[P] = row_of_pos(p, pos[q], zinv);
      p.csr_col[pos[q]] = u;
      if (p.csc_val) p.csc_val[P] = p.vals[pos[q]];
      if ((P & 31u) == 0) p.wordbase[P >> 5] = (j == s_base[h]) ? u : u + 1;
    }
  }
}

__global__ void k_bl_gate(const u32* ctl, u32* gate) { *gate = ctl[kCtlFallback]; }

// scratch layout (bytes), shared by the size query and the launcher
struct BlLayout {
  size_t zero_begin, samp_cnt, ctl, bstate, zero_end;
  size_t ff_begin, samp_key, hot_tab, ff_end;
  size_t hot_idx, hot_key, part, bin_total, cold_base, pos_base, hot_base, shot_key, shot_h, bucket_hot_off,
      hot_u, hot_seg, total;
};
static size_t al(size_t x) { return (x + 255) & ~(size_t)255; }
static BlLayout bl_layout(u32 NB, u32 G) {
  BlLayout L;
  size_t o = 0;
  const u32 NBINS = NB + kHotMax;
  L.zero_begin = o;
  L.samp_cnt = o; o = al(o + kSampSlots * 4);
  L.ctl = o; o = al(o + kCtlWords * 4);
  L.bstate = o; o = al(o + (size_t)NB * 4);
  L.zero_end = o;
  L.ff_begin = o;
  L.samp_key = o; o = al(o + (size_t)kSampSlots * 8);
  L.hot_tab = o; o = al(o + (size_t)kHotSlots * 8);
  L.ff_end = o;
  L.hot_idx = o; o = al(o + kHotSlots * 2);
  L.hot_key = o; o = al(o + kHotMax * 8);
  L.part = o; o = al(o + (size_t)G * NBINS * 4);
  L.bin_total = o; o = al(o + (size_t)NBINS * 4);
  L.cold_base = o; o = al(o + (size_t)(NB + 1) * 4);
  L.pos_base = o; o = al(o + (size_t)(NB + 1) * 4);
  L.hot_base = o; o = al(o + (kHotMax + 1) * 4);
  L.shot_key = o; o = al(o + kHotMax * 8);
  L.shot_h = o; o = al(o + kHotMax * 4);
  L.bucket_hot_off = o; o = al(o + (size_t)(NB + 1) * 4);
  L.hot_u = o; o = al(o + kHotMax * 4);
  L.hot_seg = o; o = al(o + kHotMax * 4);
  L.total = o;
  return L;
}

static u32 bl_num_buckets(u32 n) {
  // about 1600 nonzeros per bucket at most on average: even a minibatch without any repeated key
  // fills a bucket's table to 40 % only, so runs of adjacent occupied slots stay short
  u32 nb = 64;
  while (nb < kMaxBuckets && (size_t)nb * 1600 < n) nb <<= 1;
  return nb;
}
static int bl_walk_ctas() {
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms > 0 ? sms : 1;
}

}  // namespace psb

using namespace psb;

extern "C" size_t psb_bucket_localize_scratch_bytes(uint32_t max_n) {
  (void)max_n;   // the layout is sized for the largest bucket count; the per-nonzero buffers are the caller's
  return bl_layout(kMaxBuckets, (u32)bl_walk_ctas()).total;
}

// Groups the n nonzeros of a minibatch by key. Inputs as for psb_sort_pairs (in, in_kind, seed);
// low_zero_bits = number of low key bits that are zero in every key (64 - significant bits of a
// narrow hashed key); when n - 1 fits in them the position rides in the key word (no cold_pos needed).
// cold_words (n x 8 bytes), cold_pos (n x 4 bytes, may be null when the positions fit) and hot_pos
// (n x 4 bytes) are work buffers. Outputs as for psb_localize2. *gate_out (device word) is set to 1
// when the caller must run the gated sort-based path instead (its outputs then replace these).
extern "C" int psb_bucket_localize(const void* in, int in_kind, psb_u64 seed, uint32_t n, int low_zero_bits,
                                   const uint32_t* row_ptr, uint32_t n_rows, uint32_t fixed_z,
                                   const float* vals, const psb_u64* bounds, int S,
                                   psb_u64* cold_words, uint32_t* cold_pos, uint32_t* hot_pos,
                                   psb_u64* ukeys, uint32_t* seg_off, uint32_t* csr_col, uint32_t* csc_row,
                                   float* csc_val, uint32_t* flagbits, uint32_t* wordbase,
                                   uint32_t* n_unique, uint32_t* own_off, void* scratch, uint32_t* status,
                                   uint32_t* gate_out, cudaStream_t stream) {
  if (S < 1 || S > 64) return -(int)cudaErrorInvalidValue;
  if (row_ptr == nullptr && fixed_z == 0) return -(int)cudaErrorInvalidValue;
  if (low_zero_bits < 0 || low_zero_bits > 48 || in_kind < 0 || in_kind > 2) return -(int)cudaErrorInvalidValue;
  if (n == 0) {
    cudaMemsetAsync(n_unique, 0, sizeof(u32), stream);
    cudaMemsetAsync(own_off, 0, sizeof(u32) * (S + 1), stream);
    cudaMemsetAsync(seg_off, 0, sizeof(u32), stream);
    cudaMemsetAsync(gate_out, 0, sizeof(u32), stream);
    return -(int)cudaGetLastError();
  }
  BLP p{};
  p.in = in; p.in_kind = in_kind; p.seed = seed; p.n = n;
  p.lo = low_zero_bits;
  p.packed = (low_zero_bits > 0 && (low_zero_bits >= 32 || ((n - 1) >> low_zero_bits) == 0)) ? 1 : 0;
  if (!p.packed && cold_pos == nullptr) return -(int)cudaErrorInvalidValue;
  p.NB = bl_num_buckets(n);
  p.nb_bits = 0;
  while ((1u << p.nb_bits) < p.NB) ++p.nb_bits;
  p.NBINS = p.NB + kHotMax;
  p.G = (u32)bl_walk_ctas();
  p.chunk = ((n + p.G - 1) / p.G + 3) & ~3u;
  p.samp_m = min(n, kSampMax);
  p.samp_stride = n / p.samp_m;
  // hot: about half an average bucket or more, judged from the sample
  p.hot_thresh = max(4u, p.samp_m / p.NB / 2);
  p.cold_limit = max(32768u, 16u * (n / p.NB));
  p.row_ptr = row_ptr; p.n_rows = n_rows; p.fixed_z = fixed_z; p.vals = vals;
  const BlLayout L = bl_layout(p.NB, p.G);
  unsigned char* sc = (unsigned char*)scratch;
  p.samp_key = (u64*)(sc + L.samp_key); p.samp_cnt = (u32*)(sc + L.samp_cnt);
  p.hot_tab = (u64*)(sc + L.hot_tab); p.hot_idx = (unsigned short*)(sc + L.hot_idx);
  p.hot_key = (u64*)(sc + L.hot_key);
  p.ctl = (u32*)(sc + L.ctl); p.part = (u32*)(sc + L.part); p.bin_total = (u32*)(sc + L.bin_total);
  p.cold_base = (u32*)(sc + L.cold_base); p.pos_base = (u32*)(sc + L.pos_base);
  p.hot_base = (u32*)(sc + L.hot_base); p.shot_key = (u64*)(sc + L.shot_key); p.shot_h = (u32*)(sc + L.shot_h);
  p.bucket_hot_off = (u32*)(sc + L.bucket_hot_off); p.hot_u = (u32*)(sc + L.hot_u);
  p.hot_seg = (u32*)(sc + L.hot_seg); p.bstate = (u32*)(sc + L.bstate);
  p.cold_words = (u64*)cold_words; p.cold_pos = cold_pos; p.hot_pos = hot_pos;
  p.ukeys = (u64*)ukeys; p.seg_off = seg_off; p.csr_col = csr_col; p.csc_row = csc_row; p.csc_val = csc_val;
  p.flagbits = flagbits; p.wordbase = wordbase; p.n_unique = n_unique; p.status = status;

  cudaMemsetAsync(sc + L.zero_begin, 0, L.zero_end - L.zero_begin, stream);
  cudaMemsetAsync(sc + L.ff_begin, 0xFF, L.ff_end - L.ff_begin, stream);
  cudaMemsetAsync(flagbits, 0, sizeof(u32) * ((n + 31) / 32), stream);
  k_bl_sample<<<(p.samp_m + 255) / 256, 256, 0, stream>>>(p);
  k_bl_hot<<<kSampSlots / 256, 256, 0, stream>>>(p);
  const size_t walk_smem = kHotSlots * 8 + kHotSlots * 2 + (size_t)p.NBINS * 4;
  static bool attr_set = false;
  const int remaining = 64 - p.nb_bits - p.lo;      // key bits that distinguish keys inside a bucket
  const bool ck32 = remaining <= 31;
  const size_t plan_smem = (size_t)p.NB * 12;
  if (!attr_set) {
    const size_t walk_max = kHotSlots * 10 + (size_t)(kMaxBuckets + kHotMax) * 4;
    cudaFuncSetAttribute((const void*)k_bl_plan, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(kMaxBuckets * 12));
    cudaFuncSetAttribute((const void*)k_bl_walk<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)walk_max);
    cudaFuncSetAttribute((const void*)k_bl_walk<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)walk_max);
    cudaFuncSetAttribute((const void*)k_bl_bucket<u32, 11>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)BucketShape<11>::smem_bytes(4));
    cudaFuncSetAttribute((const void*)k_bl_bucket<u32, 12>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)BucketShape<12>::smem_bytes(4));
    cudaFuncSetAttribute((const void*)k_bl_bucket<u64, 11>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)BucketShape<11>::smem_bytes(8));
    cudaFuncSetAttribute((const void*)k_bl_bucket<u64, 12>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)BucketShape<12>::smem_bytes(8));
    attr_set = true;
  }
  k_bl_walk<false><<<p.G, kWalkThreads, walk_smem, stream>>>(p);
  k_bl_scan<<<(p.NBINS + 255) / 256, 256, 0, stream>>>(p);
  k_bl_plan<<<1, 1024, plan_smem, stream>>>(p);
  k_bl_walk<true><<<p.G, kWalkThreads, walk_smem, stream>>>(p);
  const u32 g11 = min(p.NB, p.G * 6), g12 = min(p.NB, p.G * 4);
  if (ck32) {
    k_bl_bucket<u32, 11><<<g11, kBucketThreads, BucketShape<11>::smem_bytes(4), stream>>>(p);
    k_bl_bucket<u32, 12><<<g12, kBucketThreads, BucketShape<12>::smem_bytes(4), stream>>>(p);
  } else {
    k_bl_bucket<u64, 11><<<g11, kBucketThreads, BucketShape<11>::smem_bytes(8), stream>>>(p);
    k_bl_bucket<u64, 12><<<g12, kBucketThreads, BucketShape<12>::smem_bytes(8), stream>>>(p);
  }
  k_bl_hot_emit<<<p.G * 8, 256, 0, stream>>>(p);
  k_bl_gate<<<1, 1, 0, stream>>>(p.ctl, gate_out);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return -(int)e;
  return psb_owner_offsets_n(ukeys, n_unique, bounds, S, n, seg_off, own_off, gate_out, stream);
}
