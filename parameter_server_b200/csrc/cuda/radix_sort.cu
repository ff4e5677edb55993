// Single-pass-per-digit LSD radix sort of (uint64 key, uint32 payload) pairs.
//
// This is the device replacement for the recursive thread merge sort that the
// reference uses to localise a minibatch (util/parallel_sort.h:14-41, called
// from util/localizer.h:97-160). Design (B200: 148 SMs, 126 MB L2, 6.5 TB/s):
//
//   * one up-front kernel reads the keys once and builds the histograms of all
//     digits (and can hash raw feature ids to uint64 keys on the way in);
//   * each 8-bit digit pass is ONE kernel: a tile of 256 threads x 16 keys is
//     ranked with warp match-any, tile totals are chained with a decoupled
//     look-back over per-tile status words, and the tile is scattered through
//     shared memory so that global stores go out in digit runs;
//   * tiles take their index from an atomic ticket, so a predecessor tile is
//     always scheduled before its successor looks back at it; the look-back
//     spin is bounded and reports through the status word.
//
// Traffic per pass is one read and one write of the pairs (24 B per element).
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
    int begin_bit, int end_bit, u32* __restrict__ ghist, int pack_bits) {
  __shared__ u32 sh[8 * kRadix];
  const int npass = (end_bit - begin_bit + kRadixBits - 1) / kRadixBits;
  for (int i = threadIdx.x; i < npass * kRadix; i += blockDim.x) sh[i] = 0;
  __syncthreads();
  for (u32 i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
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
    for (int p = 0; p < npass; ++p) {
      int shift = begin_bit + p * kRadixBits;
      int bits = min(kRadixBits, end_bit - shift);
      atomicAdd(&sh[p * kRadix + digit_of(k, shift, (1u << bits) - 1)], 1u);
    }
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
__global__ void k_sort_plan(const u32* __restrict__ ghist, int npass, u32 n, u32* __restrict__ plan) {
  __shared__ u32 s_skip[8];
  if (threadIdx.x < 8) s_skip[threadIdx.x] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < npass * kRadix; i += blockDim.x)
    if (ghist[i] == n) s_skip[i / kRadix] = 1;
  __syncthreads();
  if (threadIdx.x == 0) {
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
__global__ void k_sort_identity_payload(const u32* __restrict__ plan, u32* __restrict__ vals_a, u32 n) {
  if (plan[17] == 0) return;
  for (u32 i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) vals_a[i] = i;
}

// Exclusive scan of one value per thread across the block (kSortWarps warps).
__device__ __forceinline__ u32 block_excl_scan_256(u32 v, u32* s_warp /*kSortWarps words*/, u32* total) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  u32 x = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    u32 y = __shfl_up_sync(0xffffffffu, x, o);
    if (lane >= o) x += y;
  }
  if (lane == 31) s_warp[w] = x;
  __syncthreads();
  u32 base = 0, tot = 0;
#pragma unroll
  for (int i = 0; i < kSortWarps; ++i) {
    u32 t = s_warp[i];
    if (i < w) base += t;
    tot += t;
  }
  if (total) *total = tot;
  __syncthreads();
  return base + x - v;
}

// One digit pass. `status` holds ntiles*256 zeroed words for this pass.
__global__ void __launch_bounds__(kSortThreads, 2) k_sort_onesweep(
    u64* __restrict__ keys_a, u32* __restrict__ vals_a, u64* __restrict__ keys_b, u32* __restrict__ vals_b,
    int vals_given, u32 n, int shift, u32 dmask, const u32* __restrict__ ghist, u32* __restrict__ ticket,
    u32* __restrict__ status, u32* __restrict__ err, const u32* __restrict__ plan, int pass) {
  const u32 pl = plan[pass];
  if (pl & 1u) return;                                   // constant digit: nothing to do
  const bool from_b = (pl >> 1) & 1u;
  const u64* __restrict__ keys_in = from_b ? keys_b : keys_a;
  u64* __restrict__ keys_out = from_b ? keys_a : keys_b;
  const u32* __restrict__ vals_in = from_b ? vals_b : vals_a;
  u32* __restrict__ vals_out = from_b ? vals_a : vals_b;
  if ((pl & 4u) && !vals_given) vals_in = nullptr;       // first executed pass: payload = index
  __shared__ u64 s_keys[kSortTile];            // 32 KB, reused for payloads
  __shared__ unsigned short s_cnt[kSortWarps * kRadix];  // per-warp digit counters (<= 256 each), 8 KB
  __shared__ u32 s_dstart[kRadix];             // tile-local start of each digit
  __shared__ u32 s_gbase[kRadix];              // global dst = s_gbase[d] + p
  __shared__ u32 s_warp[kSortWarps];
  __shared__ u32 s_tile;

  const int t = threadIdx.x, lane = t & 31, w = t >> 5;
  if (t == 0) s_tile = atomicAdd(ticket, 1u);
  for (int i = t; i < kSortWarps * kRadix; i += kSortThreads) s_cnt[i] = 0;
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
    key[i] = idx < nvalid ? keys_in[tile_base + idx] : kEmptyKey;
  }
  // ---- rank inside the warp, in (item, lane) order ----
  const u32 lt = (1u << lane) - 1;
#pragma unroll
  for (int i = 0; i < kSortItems; ++i) {
    u32 d = digit_of(key[i], shift, dmask);
    u32 m = __match_any_sync(0xffffffffu, d);
    int leader = __ffs(m) - 1;
    u32 old = 0;
    if (lane == leader) {
      old = s_cnt[w * kRadix + d];
      s_cnt[w * kRadix + d] = (unsigned short)(old + __popc(m));
    }
    old = __shfl_sync(0xffffffffu, old, leader);
    off[i] = old + __popc(m & lt);
    __syncwarp();
  }
  __syncthreads();
  // ---- per digit (thread t < 256 owns digit t): prefix over warps, tile total ----
  const bool owner = t < kRadix;
  u32 total = 0;
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
  }

  u32 dstart = block_excl_scan_256(total, s_warp, nullptr);
  if (owner) s_dstart[t] = dstart;
  // global exclusive base of digit t
  u32 gh = owner ? ghist[t] : 0u;
  u32 gex = block_excl_scan_256(gh, s_warp, nullptr);

  // ---- decoupled look-back for digit t, kLookBatch predecessors per round trip ----
  // All tiles of the first wave start together, so a tile may have to walk over
  // many predecessors that have only published aggregates; fetching them in
  // batches of independent loads hides the L2 latency of that walk.
  u32 ex = 0;
  if (tile > 0 && owner) {
    constexpr int kLookBatch = 8;
    long long p = (long long)tile - 1;
    u32 spins = 0;
    bool done = false;
    while (!done && p >= 0) {
      u32 sv[kLookBatch];
#pragma unroll
      for (int k = 0; k < kLookBatch; ++k)
        sv[k] = (p - k >= 0) ? ld_relaxed_gpu(status + (size_t)(p - k) * kRadix + t) : kFlagIncl;
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
      if (!done && used < kLookBatch) {
        if (++spins > kGridWaitIters) { set_status(err, kLookbackTimeout); break; }
        if (used == 0) __nanosleep(20);
      }
    }
    st_relaxed_gpu(&my_status[t], kFlagIncl | ((ex + total) & kValMask));
  }
  if (owner) s_gbase[t] = gex + ex - dstart;
  __syncthreads();

  // ---- scatter keys into shared memory in digit order ----
#pragma unroll
  for (int i = 0; i < kSortItems; ++i) {
    u32 d = digit_of(key[i], shift, dmask);
    u32 p = s_dstart[d] + s_cnt[w * kRadix + d] + off[i];
    off[i] = p;
    s_keys[p] = key[i];
  }
  __syncthreads();
  u32 dst[kSortItems];
#pragma unroll
  for (int j = 0; j < kSortItems; ++j) {
    u32 p = t + j * kSortThreads;
    u64 k = s_keys[p];
    u32 d = digit_of(k, shift, dmask);
    dst[j] = s_gbase[d] + p;
    if (p < nvalid) keys_out[dst[j]] = k;
  }
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
  // ghist | tickets (16) | plan (32) | status
  return sizeof(u32) * ((size_t)npass * kRadix + 48 + (size_t)npass * ntiles * kRadix);
}

// Sorts n pairs by key bits [begin_bit, end_bit), ping-ponging between buffers A
// (keys_a, vals_a) and B (keys_b, vals_b). The input is `in` (see k_sort_histogram
// for in_kind); plain keys (in_kind 0) that are not already in A are copied there.
// vals_given = 0 means payload = element index. Passes over digit positions that
// are constant across the batch are skipped, so which buffer holds the result is
// only known on the device: *where_out (device word) is 0 for A, 1 for B.
// With pack_pos_bits > 0 (see k_sort_histogram) pass null payload buffers.
extern "C" int psb_sort_pairs(const void* in, int in_kind, psb_u64 seed, psb_u64* keys_a,
                              uint32_t* vals_a, int vals_given, psb_u64* keys_b, uint32_t* vals_b,
                              uint32_t n, int begin_bit, int end_bit, void* scratch,
                              uint32_t* status, uint32_t* where_out, int pack_pos_bits, cudaStream_t stream) {
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
  u32* tickets = ghist + (size_t)npass * kRadix;
  u32* plan = tickets + 16;
  u32* st = plan + 32;
  cudaMemsetAsync(scratch, 0, psb_sort_scratch_bytes(n, begin_bit, end_bit), stream);
  int hb = (int)min((u32)(148 * 8), (n + 255) / 256);
  k_sort_histogram<<<hb, 256, 0, stream>>>(in, in_kind, seed, (u64*)keys_a, n, begin_bit, end_bit, ghist,
                                           pack_pos_bits);
  k_sort_plan<<<1, 256, 0, stream>>>(ghist, npass, n, plan);
  for (int p = 0; p < npass; ++p) {
    int shift = begin_bit + p * kRadixBits;
    int bits = min(kRadixBits, end_bit - shift);
    k_sort_onesweep<<<ntiles, kSortThreads, 0, stream>>>(
        (u64*)keys_a, vals_a, (u64*)keys_b, vals_b, vals_given, n, shift, (1u << bits) - 1,
        ghist + (size_t)p * kRadix, tickets + p, st + (size_t)p * ntiles * kRadix, status, plan, p);
  }
  if (!vals_given && vals_a && !pack_pos_bits) k_sort_identity_payload<<<hb, 256, 0, stream>>>(plan, vals_a, n);
  cudaMemcpyAsync(where_out, plan + 16, sizeof(u32), cudaMemcpyDeviceToDevice, stream);
  return -(int)cudaGetLastError();
}
