// Single-pass-per-digit LSD radix sort of (uint64 key, uint32 payload) pairs.
//
// This is the device replacement for the recursive thread merge sort that the
// reference uses to localise a minibatch (util/parallel_sort.h:14-41, called
// from util/localizer.h:97-160). Design (B200: 148 SMs, 126 MB L2, 6.5 TB/s):
//
//   * one up-front kernel reads the keys once and builds the histograms of all
//     digits (and can hash raw feature ids to uint64 keys on the way in);
//   * each 8-bit digit pass is ONE kernel: a tile of 512 threads x 8 keys is
//     ranked with warp match-any, tile totals are chained with a decoupled
//     look-back over per-tile status words, and the tile is scattered through
//     shared memory so that global stores go out in digit runs;
//   * the look-back spin is bounded and reports through the status word.
//
// Traffic per pass is one read and one write of the pairs (24 B per element;
// 16 B when the position is packed into the key and there is no payload array).
#include "psb_common.cuh"
#include "psb_cuda.h"

namespace psb {

// 512 threads x 8 keys: the same 4096-key tile as 256 x 16, but half the
// registers per thread (two resident CTAs = 32 warps per SM) and a ranking chain
// of 8 dependent steps instead of 16.
static constexpr int kSortThreads = 512;
static constexpr int kSortWarps = kSortThreads / 32;
static constexpr int kSortItems = 8;
static constexpr int kSortTile = kSortThreads * kSortItems;  // 4096
static constexpr int kRadixBits = 8;
static constexpr int kRadix = 1 << kRadixBits;
static constexpr u32 kFlagAgg = 1u << 30;
static constexpr u32 kFlagIncl = 2u << 30;
static constexpr u32 kValMask = (1u << 30) - 1;

// Poll of a tile status word: an L2 load (L1 bypassed) that is re-issued on every
// call. Only the word itself is exchanged, so no ordering with other data is needed.
__device__ __forceinline__ u32 ld_status(const u32* p) {
  u32 v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}

// Launch gate: a device word decides whether the kernels of a call run at all (the sort-based
// localisation is enqueued behind the bucket-based one and only runs when that one gave up).
__device__ __forceinline__ bool gate_closed(const u32* gate) { return gate != nullptr && *gate == 0; }

__device__ __forceinline__ u32 digit_of(u64 k, int shift, u32 dmask) {
  return (u32)(k >> shift) & dmask;
}

// in_kind: 0 = uint64 keys (used as is), 1 = uint32 ids, 2 = uint64 ids; for
// 1 and 2 the key is hash_id_to_key(id, seed) and is written to keys_out.
// pack_bits > 0 (hashed input only): the element index is stored in the low
// pack_bits bits of the key, which the narrow hash leaves zero, so the pairs
// travel as single 64-bit words and need no payload array.
__global__ void __launch_bounds__(256) k_sort_histogram(
    const void* __restrict__ in, int in_kind, u64 seed, u64* __restrict__ keys_out, u32 n,
    int begin_bit, int end_bit, u32* __restrict__ ghist, int pack_bits, const u32* __restrict__ gate) {
  __shared__ u32 sh[8 * kRadix];
  if (gate_closed(gate)) return;
  const int npass = (end_bit - begin_bit + kRadixBits - 1) / kRadixBits;
  for (int i = threadIdx.x; i < npass * kRadix; i += blockDim.x) sh[i] = 0;
  __syncthreads();
  auto count = [&](u64 k) {
    for (int p = 0; p < npass; ++p) {
      int shift = begin_bit + p * kRadixBits;
      int bits = min(kRadixBits, end_bit - shift);
      atomicAdd(&sh[p * kRadix + digit_of(k, shift, (1u << bits) - 1)], 1u);
    }
  };
  const u32 gtid = blockIdx.x * blockDim.x + threadIdx.x, gsz = gridDim.x * blockDim.x;
  u32 done = 0;   // elements [0, done) are handled by the vector path
  if (in_kind == 1 && (((size_t)in | (size_t)keys_out) & 15) == 0) {
    // 32-bit ids: four per thread and trip (one 16-byte load, two 16-byte stores),
    // two trips in flight
    const u32 n4 = n / 4;
    const uint4* __restrict__ in4 = (const uint4*)in;
    ulonglong2* __restrict__ out2 = (ulonglong2*)keys_out;
    for (u32 i = gtid; i < n4; i += 2 * gsz) {
      const u32 j = i + gsz;
      uint4 a = in4[i], b = make_uint4(0, 0, 0, 0);
      if (j < n4) b = in4[j];
      u64 k[8];
      k[0] = hash_id_to_key(a.x, seed); k[1] = hash_id_to_key(a.y, seed);
      k[2] = hash_id_to_key(a.z, seed); k[3] = hash_id_to_key(a.w, seed);
      k[4] = hash_id_to_key(b.x, seed); k[5] = hash_id_to_key(b.y, seed);
      k[6] = hash_id_to_key(b.z, seed); k[7] = hash_id_to_key(b.w, seed);
      if (pack_bits) {
#pragma unroll
        for (int q = 0; q < 4; ++q) { k[q] |= (u64)(4 * i + q); k[4 + q] |= (u64)(4 * j + q); }
      }
      out2[2 * (size_t)i] = make_ulonglong2(k[0], k[1]);
      out2[2 * (size_t)i + 1] = make_ulonglong2(k[2], k[3]);
#pragma unroll
      for (int q = 0; q < 4; ++q) count(k[q]);
      if (j < n4) {
        out2[2 * (size_t)j] = make_ulonglong2(k[4], k[5]);
        out2[2 * (size_t)j + 1] = make_ulonglong2(k[6], k[7]);
#pragma unroll
        for (int q = 0; q < 4; ++q) count(k[4 + q]);
      }
    }
    done = n4 * 4;
  } else if (in_kind == 0 && (((size_t)in | (size_t)keys_out) & 15) == 0) {
    // plain 64-bit keys: two per thread and trip, two trips in flight
    const u32 n2 = n / 2;
    const ulonglong2* __restrict__ in2 = (const ulonglong2*)in;
    ulonglong2* __restrict__ out2 = (keys_out && keys_out != (const u64*)in) ? (ulonglong2*)keys_out : nullptr;
    for (u32 i = gtid; i < n2; i += 2 * gsz) {
      const u32 j = i + gsz;
      ulonglong2 a = in2[i], b = a;
      if (j < n2) b = in2[j];
      if (out2) { out2[i] = a; if (j < n2) out2[j] = b; }
      count(a.x); count(a.y);
      if (j < n2) { count(b.x); count(b.y); }
    }
    done = n2 * 2;
  }
  for (u32 i = done + gtid; i < n; i += gsz) {
    u64 k;
    if (in_kind == 0) {
      k = ((const u64*)in)[i];
      if (keys_out && keys_out != (const u64*)in) keys_out[i] = k;   // passes ping-pong between A and B
    } else {
      u64 id = in_kind == 1 ? (u64)((const u32*)in)[i] : ((const u64*)in)[i];
      k = hash_id_to_key(id, seed);
      if (pack_bits) k |= (u64)i;
      keys_out[i] = k;
    }
    count(k);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < npass * kRadix; i += blockDim.x)
    if (sh[i]) atomicAdd(&ghist[i], sh[i]);
}

// Pass plan. A digit position whose histogram has a single non-empty bin does
// not change the order, so its pass is skipped (keys with fewer significant bits
// than the sorted range, e.g. hashed 40-bit keys, cost proportionally less).
// plan[p]: bit 0 = skip, bit 1 = source buffer (0 = A, 1 = B), bit 2 = first
// executed pass (payload defaults to the element index); plan[16] = buffer that
// holds the result.
__global__ void __launch_bounds__(kRadix) k_sort_plan(const u32* __restrict__ ghist, int npass, u32 n,
                                                      u32* __restrict__ plan, u32* __restrict__ gpre,
                                                      const u32* __restrict__ gate) {
  __shared__ u32 s_skip[8];
  if (gate_closed(gate)) return;
  __shared__ u32 s_scan[kRadix];
  const int t = threadIdx.x;
  if (t < 8) s_skip[t] = 0;
  __syncthreads();
  for (int p = 0; p < npass; ++p) {
    // gpre[p][d] = number of keys whose digit p is below d (global start of digit d)
    const u32 c = ghist[p * kRadix + t];
    if (c == n) s_skip[p] = 1;
    s_scan[t] = c;
    __syncthreads();
    for (int o = 1; o < kRadix; o <<= 1) {
      u32 y = t >= o ? s_scan[t - o] : 0u;
      __syncthreads();
      s_scan[t] += y;
      __syncthreads();
    }
    gpre[p * kRadix + t] = s_scan[t] - c;
    __syncthreads();
  }
  if (t == 0) {
    u32 cur = 0, first = 1;
    for (int p = 0; p < npass; ++p) {
      u32 w = s_skip[p] | (cur << 1) | ((first && !s_skip[p]) ? 4u : 0u);
      plan[p] = w;
      if (!s_skip[p]) { cur ^= 1; first = 0; }
    }
    plan[16] = cur;
    plan[17] = first;   // 1: every pass was skipped (the input order is already sorted)
  }
}

// When every pass is skipped (the input is already in order) and no payload was
// given, the payload still has to become the element index.
__global__ void k_sort_identity_payload(const u32* __restrict__ plan, u32* __restrict__ vals_a, u32 n,
                                        const u32* __restrict__ gate) {
  if (gate_closed(gate) || plan[17] == 0) return;
  for (u32 i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) vals_a[i] = i;
}

// Optional per-phase cycle stamps (thread 0 of every tile) for tuning builds.
#ifdef PSB_SORT_TRACE
#define PSB_TRACE_PARAM , long long* trace
#define PSB_STAMP() do { if (threadIdx.x == 0 && nts < 10) ts[nts++] = clock64(); } while (0)
#else
#define PSB_TRACE_PARAM
#define PSB_STAMP() do { } while (0)
#endif

// One digit pass. `status` holds ntiles*256 zeroed words for this pass.
//
// A block takes its tile index from a per-pass ticket counter (one atomic per
// block), so the look-back of a tile only ever waits for tiles whose blocks are
// already running or finished, whatever order the hardware dispatches blocks in.
// The spin is bounded all the same and reports kLookbackTimeout.
//
// Order of work in a tile: rank -> digit totals (published as the tile's
// aggregate) -> keys scattered to shared memory in digit order -> look-back
// (the key registers are free by then, so 32 predecessors are fetched per L2
// round trip) -> coalesced global stores of the digit runs.
__global__ void __launch_bounds__(kSortThreads, 2) k_sort_onesweep(
    u64* __restrict__ keys_a, u32* __restrict__ vals_a, u64* __restrict__ keys_b, u32* __restrict__ vals_b,
    int vals_given, u32 n, int shift, u32 dmask, const u32* __restrict__ gpre,
    u32* __restrict__ status, u32* __restrict__ err, const u32* __restrict__ plan, int pass,
    u32* __restrict__ ticket, const u32* __restrict__ gate PSB_TRACE_PARAM) {
#ifdef PSB_SORT_TRACE
  long long ts[12] = {0}; int nts = 0;
#endif
  PSB_STAMP();
  if (gate_closed(gate)) return;
  // the plan word is the same for every tile: keep its line in L1 for the later tiles of this SM
  u32 pl;
  asm volatile("ld.global.nc.L1::evict_last.u32 %0, [%1];" : "=r"(pl) : "l"(plan + pass));
  if (pl & 1u) return;                                   // constant digit: nothing to do
  const bool from_b = (pl >> 1) & 1u;
  const u64* __restrict__ keys_in = from_b ? keys_b : keys_a;
  u64* __restrict__ keys_out = from_b ? keys_a : keys_b;
  const u32* __restrict__ vals_in = from_b ? vals_b : vals_a;
  u32* __restrict__ vals_out = from_b ? vals_a : vals_b;
  if ((pl & 4u) && !vals_given) vals_in = nullptr;       // first executed pass: payload = index
  __shared__ u64 s_keys[kSortTile];            // 32 KB, reused for payloads
  // per-warp digit counters (<= 256 each), two 16-bit counters per word so that the
  // ranking can use 32-bit shared atomics; read back as 16-bit values afterwards. 8 KB
  __shared__ u32 s_cnt32[kSortWarps * kRadix / 2];
  unsigned short* s_cnt = reinterpret_cast<unsigned short*>(s_cnt32);
  __shared__ u32 s_dstart[kRadix];             // tile-local start of each digit
  __shared__ u32 s_gbase[kRadix];              // global dst = s_gbase[d] + p
  __shared__ u32 s_warp[kRadix / 32];
  __shared__ u32 s_tile;

  const int t = threadIdx.x, lane = t & 31, w = t >> 5;
  if (t == 0) s_tile = atomicAdd(ticket, 1u);
  __syncthreads();
  const u32 tile = s_tile;
  const u32 tile_base = tile * (u32)kSortTile;
  const u32 nvalid = min((u32)kSortTile, n - tile_base);

  // ---- load (warp-striped: consecutive lanes read consecutive elements) ----
  u64 key[kSortItems];
  u32 off[kSortItems];
  const u32 wbase = w * (32 * kSortItems);
#pragma unroll
  for (int i = 0; i < kSortItems; ++i) {
    u32 idx = wbase + i * 32 + lane;
    key[i] = kEmptyKey;
    if (idx < nvalid)   // read once: do not displace the plan line in L1
      asm volatile("ld.global.L1::no_allocate.u64 %0, [%1];" : "=l"(key[i]) : "l"(keys_in + tile_base + idx));
  }
  // every warp clears its own counter row, so no block barrier is needed before the ranking
#pragma unroll
  for (int i = 0; i < kRadix / 2 / 32; ++i) s_cnt32[w * (kRadix / 2) + i * 32 + lane] = 0;
  __syncwarp();
  PSB_STAMP();
  // ---- rank inside the warp, in (item, lane) order ----
  // Three pipelined sweeps instead of one dependent chain per item: all match
  // masks first, then one shared-memory atomic per (item, distinct digit) by the
  // group's lowest lane, then the broadcasts of the returned counts. The warp
  // issues the atomics of item i before those of item i + 1, so the count that a
  // group reads covers exactly the earlier items: the ranking stays stable.
  const u32 lt = (1u << lane) - 1;
  u32 mask[kSortItems];
#pragma unroll
  for (int i = 0; i < kSortItems; ++i) mask[i] = __match_any_sync(0xffffffffu, digit_of(key[i], shift, dmask));
#ifdef PSB_SORT_TRACE
  if (mask[kSortItems - 1] == 0x12345u) ts[11] = 1;   // make the stamp wait for the loads
#endif
  PSB_STAMP();
#pragma unroll
  for (int i = 0; i < kSortItems; ++i) {
    u32 old = 0;
    const u32 d = digit_of(key[i], shift, dmask), sh16 = (d & 1u) * 16;
    if (lane == __ffs(mask[i]) - 1)
      old = (atomicAdd(&s_cnt32[w * (kRadix / 2) + (d >> 1)], (u32)__popc(mask[i]) << sh16) >> sh16) & 0xffffu;
    off[i] = old;
    __syncwarp();
  }
#pragma unroll
  for (int i = 0; i < kSortItems; ++i)
    off[i] = __shfl_sync(0xffffffffu, off[i], __ffs(mask[i]) - 1) + __popc(mask[i] & lt);
#ifdef PSB_SORT_TRACE
  if (off[kSortItems - 1] == 0x7777777u) ts[11] = 2;
#endif
  PSB_STAMP();
  __syncthreads();
  PSB_STAMP();
  // ---- per digit (thread t < 256 owns digit t): prefix over warps, tile total ----
  const bool owner = t < kRadix;
  u32 total = 0, dstart = 0;
  u32* my_status = status + (size_t)tile * kRadix;
  if (owner) {
#pragma unroll
    for (int ww = 0; ww < kSortWarps; ++ww) {
      u32 c = s_cnt[ww * kRadix + t];
      s_cnt[ww * kRadix + t] = (unsigned short)total;
      total += c;
    }
    // publish the tile aggregate early so successors can move on. The status word
    // itself is the only datum exchanged, so relaxed gpu-scope accesses suffice.
    st_relaxed_gpu(&my_status[t], (tile == 0 ? kFlagIncl : kFlagAgg) | total);
    // tile-local start of digit t: exclusive scan of the totals over the 256 owner threads
    u32 x = total;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      u32 y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += y;
    }
    if (lane == 31) s_warp[w] = x;
    asm volatile("bar.sync 1, %0;" ::"n"(kRadix) : "memory");   // the owner warps only
    u32 base = 0;
#pragma unroll
    for (int i = 0; i < kRadix / 32; ++i) base += (i < w) ? s_warp[i] : 0u;
    dstart = base + x - total;
    s_dstart[t] = dstart;
  }
  __syncthreads();
  PSB_STAMP();
  // ---- scatter keys into shared memory in digit order ----
#pragma unroll
  for (int i = 0; i < kSortItems; ++i) {
    u32 d = digit_of(key[i], shift, dmask);
    u32 p = s_dstart[d] + s_cnt[w * kRadix + d] + off[i];
    off[i] = p;
    s_keys[p] = key[i];
  }
  PSB_STAMP();
  // ---- decoupled look-back for digit t, kLookBatch predecessors per round trip ----
  // Many tiles run at once, so a tile usually has to walk over dozens of
  // predecessors that have only published aggregates; fetching them in batches of
  // independent loads hides the L2 latency of that walk.
  if (owner) {
    u32 ex = 0;
    if (tile > 0) {
      constexpr int kLookBatch = 16;
      long long p = (long long)tile - 1;
      u32 spins = 0;
      bool done = false;
#ifdef PSB_SORT_TRACE
      u32 trips = 0, stalls = 0;
      long long lb0 = clock64(), first_trip = 0;
#endif
      while (!done && p >= 0) {
        u32 sv[kLookBatch];
#pragma unroll
        for (int k = 0; k < kLookBatch; ++k)
          sv[k] = (p - k >= 0) ? ld_status(status + (size_t)(p - k) * kRadix + t) : kFlagIncl;
        int used = 0;
#pragma unroll
        for (int k = 0; k < kLookBatch; ++k) {
          if (done || used < k) continue;
          u32 f = sv[k] & ~kValMask;
          if (f == 0) continue;          // not published yet: stop consuming, re-poll from here
          ex += sv[k] & kValMask;
          used = k + 1;
          if (f == kFlagIncl) done = true;
        }
        p -= used;
#ifdef PSB_SORT_TRACE
        ++trips; if (!done && used < kLookBatch) ++stalls;
        if (trips == 1) first_trip = clock64() - lb0;
#endif
        if (!done && used < kLookBatch) {
          if (++spins > kGridWaitIters) { set_status(err, kLookbackTimeout); break; }
          if (used == 0) __nanosleep(20);
        }
      }
      st_relaxed_gpu(&my_status[t], kFlagIncl | ((ex + total) & kValMask));
#ifdef PSB_SORT_TRACE
      if (t == 0) { ts[10] = trips | ((long long)stalls << 32); ts[11] = ((long long)tile - 1 - p) | (first_trip << 32); }
#endif
    }
    s_gbase[t] = gpre[t] + ex - dstart;
  }
  PSB_STAMP();
  __syncthreads();
  PSB_STAMP();
  u32 dst[kSortItems];
#pragma unroll
  for (int j = 0; j < kSortItems; ++j) {
    u32 p = t + j * kSortThreads;
    u64 k = s_keys[p];
    u32 d = digit_of(k, shift, dmask);
    dst[j] = s_gbase[d] + p;
    if (p < nvalid) keys_out[dst[j]] = k;
  }
  PSB_STAMP();
#ifdef PSB_SORT_TRACE
  if (t == 0 && trace) {
    for (int q = 0; q < 12; ++q) trace[(size_t)tile * 12 + q] = ts[q];
  }
#endif
  if (vals_out == nullptr) return;
  __syncthreads();
  // ---- payloads through the same staging buffer ----
  u32* s_vals = reinterpret_cast<u32*>(s_keys);
#pragma unroll
  for (int i = 0; i < kSortItems; ++i) {
    u32 idx = wbase + i * 32 + lane;
    u32 v = 0;
    if (idx < nvalid) v = vals_in ? vals_in[tile_base + idx] : tile_base + idx;
    s_vals[off[i]] = v;
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < kSortItems; ++j) {
    u32 p = t + j * kSortThreads;
    if (p < nvalid) vals_out[dst[j]] = s_vals[p];
  }
}

}  // namespace psb

using namespace psb;

extern "C" size_t psb_sort_scratch_bytes(uint32_t n, int begin_bit, int end_bit) {
  int npass = (end_bit - begin_bit + kRadixBits - 1) / kRadixBits;
  size_t ntiles = (n + kSortTile - 1) / kSortTile;
  if (ntiles == 0) ntiles = 1;
  // ghist | gpre | reserved (16) | plan (32) | status
  return sizeof(u32) * (2 * (size_t)npass * kRadix + 48 + (size_t)npass * ntiles * kRadix);
}

// Sorts n pairs by key bits [begin_bit, end_bit), ping-ponging between buffers A
// (keys_a, vals_a) and B (keys_b, vals_b). The input is `in` (see k_sort_histogram
// for in_kind); plain keys (in_kind 0) that are not already in A are copied there.
// vals_given = 0 means payload = element index. Passes over digit positions that
// are constant across the batch are skipped, so which buffer holds the result is
// only known on the device: *where_out (device word) is 0 for A, 1 for B.
// With pack_pos_bits > 0 (see k_sort_histogram) pass null payload buffers.
static int sort_pairs_impl(const void* in, int in_kind, psb_u64 seed, psb_u64* keys_a,
                           uint32_t* vals_a, int vals_given, psb_u64* keys_b, uint32_t* vals_b,
                           uint32_t n, int begin_bit, int end_bit, void* scratch,
                           uint32_t* status, uint32_t* where_out, int pack_pos_bits, const uint32_t* gate,
                           cudaStream_t stream
#ifdef PSB_SORT_TRACE
                           , long long* trace, int trace_pass
#endif
                           ) {
  if (end_bit <= begin_bit || end_bit > 64 || begin_bit < 0) return -(int)cudaErrorInvalidValue;
  if (pack_pos_bits) {
    // packed mode: hashed input, index bits below the sorted range, and they must hold every index
    if (in_kind == 0 || pack_pos_bits > begin_bit || pack_pos_bits > 32 ||
        (pack_pos_bits < 32 && (n - 1) >> pack_pos_bits)) return -(int)cudaErrorInvalidValue;
  }
  if (n == 0) { cudaMemsetAsync(where_out, 0, sizeof(u32), stream); return -(int)cudaGetLastError(); }
  const int npass = (end_bit - begin_bit + kRadixBits - 1) / kRadixBits;
  const u32 ntiles = (n + kSortTile - 1) / kSortTile;
  u32* ghist = (u32*)scratch;
  u32* gpre = ghist + (size_t)npass * kRadix;
  u32* tickets = gpre + (size_t)npass * kRadix;   // one zeroed word per pass (16 reserved)
  u32* plan = tickets + 16;
  u32* st = plan + 32;
  cudaMemsetAsync(scratch, 0, psb_sort_scratch_bytes(n, begin_bit, end_bit), stream);
  int hb = (int)min((u32)(psb_device_sm_count() * 8), (n / 8 + 255) / 256 + 1);
  k_sort_histogram<<<hb, 256, 0, stream>>>(in, in_kind, seed, (u64*)keys_a, n, begin_bit, end_bit, ghist,
                                           pack_pos_bits, gate);
  k_sort_plan<<<1, kRadix, 0, stream>>>(ghist, npass, n, plan, gpre, gate);
  for (int p = 0; p < npass; ++p) {
    int shift = begin_bit + p * kRadixBits;
    int bits = min(kRadixBits, end_bit - shift);
    k_sort_onesweep<<<ntiles, kSortThreads, 0, stream>>>(
        (u64*)keys_a, vals_a, (u64*)keys_b, vals_b, vals_given, n, shift, (1u << bits) - 1,
        gpre + (size_t)p * kRadix, st + (size_t)p * ntiles * kRadix, status, plan, p, tickets + p, gate
#ifdef PSB_SORT_TRACE
        , p == trace_pass ? trace : nullptr
#endif
        );
  }
  if (!vals_given && vals_a && !pack_pos_bits) k_sort_identity_payload<<<hb, 256, 0, stream>>>(plan, vals_a, n, gate);
  cudaMemcpyAsync(where_out, plan + 16, sizeof(u32), cudaMemcpyDeviceToDevice, stream);
  return -(int)cudaGetLastError();
}

extern "C" int psb_sort_pairs(const void* in, int in_kind, psb_u64 seed, psb_u64* keys_a,
                              uint32_t* vals_a, int vals_given, psb_u64* keys_b, uint32_t* vals_b,
                              uint32_t n, int begin_bit, int end_bit, void* scratch,
                              uint32_t* status, uint32_t* where_out, int pack_pos_bits, cudaStream_t stream
#ifdef PSB_SORT_TRACE
                              , long long* trace, int trace_pass
#endif
                              ) {
  return sort_pairs_impl(in, in_kind, seed, keys_a, vals_a, vals_given, keys_b, vals_b, n, begin_bit, end_bit,
                         scratch, status, where_out, pack_pos_bits, nullptr, stream
#ifdef PSB_SORT_TRACE
                         , trace, trace_pass
#endif
                         );
}

// Same, but every kernel of the call returns at once unless the device word *gate is non-zero.
extern "C" int psb_sort_pairs_gated(const void* in, int in_kind, psb_u64 seed, psb_u64* keys_a,
                                    uint32_t* vals_a, int vals_given, psb_u64* keys_b, uint32_t* vals_b,
                                    uint32_t n, int begin_bit, int end_bit, void* scratch,
                                    uint32_t* status, uint32_t* where_out, int pack_pos_bits,
                                    const uint32_t* gate, cudaStream_t stream) {
  return sort_pairs_impl(in, in_kind, seed, keys_a, vals_a, vals_given, keys_b, vals_b, n, begin_bit, end_bit,
                         scratch, status, where_out, pack_pos_bits, gate, stream
#ifdef PSB_SORT_TRACE
                         , nullptr, -1
#endif
                         );
}
