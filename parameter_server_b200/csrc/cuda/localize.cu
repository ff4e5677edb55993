// Minibatch localisation on the device: from the sorted (key, position) pairs
// produce the sorted unique key list, the CSC segment offsets, the CSR column
// remap and the per-owner slice offsets.
//
// Reference behaviour: Localizer::CountUniqIndex + RemapIndex
// (util/localizer.h:97-221) and the key-range slicing of
// SliceKOFVMessage (system/message.h:107-147). Here the sort already groups
// equal keys, so "unique + counts" is a head-flag scan, the remap is a scatter
// of the unique index back to each nonzero's original position, and slicing
// is S+1 binary searches over the unique keys.
//
// Kernels: k_uniq_count (heads per tile) -> k_uniq_scan (tile bases, U) ->
// k_uniq_emit (everything else) -> k_owner_offsets.
#include "psb_common.cuh"
#include "psb_cuda.h"

namespace psb {

static constexpr int kLocThreads = 256;
static constexpr int kLocItems = 16;
static constexpr int kLocTile = kLocThreads * kLocItems;  // 4096 = 128 flag words

// Launch gate: with a non-null gate word the kernel runs only when (*gate != 0) == want.
__device__ __forceinline__ bool gate_skips(const u32* gate, int want) {
  return gate != nullptr && ((*gate != 0) != (want != 0));
}

// Loads the warp's 16 x 32 consecutive keys starting at `base` (all requested
// before the first is used) and returns, per item, the ballot of segment heads.
// kmask selects the key bits (all ones, or without the packed position bits).
__device__ __forceinline__ void warp_heads(const u64* __restrict__ keys, u32 n, u32 base, int lane, u64 kmask,
                                           u64 (&k)[kLocItems], u32 (&bal)[kLocItems]) {
#pragma unroll
  for (int i = 0; i < kLocItems; ++i) {
    u32 g = base + i * 32 + lane;
    k[i] = g < n ? keys[g] : 0;
  }
  u64 before = (lane == 0 && base > 0 && base < n) ? keys[base - 1] : 0;   // last key before the warp's span
#pragma unroll
  for (int i = 0; i < kLocItems; ++i) {
    u32 g = base + i * 32 + lane;
    u64 prev = __shfl_up_sync(0xffffffffu, k[i], 1);
    u64 carry = __shfl_sync(0xffffffffu, i ? k[i ? i - 1 : 0] : before, i ? 31 : 0);
    if (lane == 0) prev = carry;
    bool head = g < n && (g == 0 || (k[i] & kmask) != (prev & kmask));
    bal[i] = __ballot_sync(0xffffffffu, head);
  }
}

__global__ void __launch_bounds__(kLocThreads) k_uniq_count(const u64* __restrict__ keys_a,
                                                            const u64* __restrict__ keys_b,
                                                            const u32* __restrict__ where, u32 n,
                                                            u32* __restrict__ tile_heads, u64 kmask,
                                                            const u32* __restrict__ gate) {
  __shared__ u32 s_w[8];
  if (gate_skips(gate, 1)) return;
  const u64* __restrict__ keys = (where && *where) ? keys_b : keys_a;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const u32 base = blockIdx.x * (u32)kLocTile + w * (32 * kLocItems);
  u64 k[kLocItems];
  u32 bal[kLocItems];
  warp_heads(keys, n, base, lane, kmask, k, bal);
  u32 cnt = 0;
#pragma unroll
  for (int i = 0; i < kLocItems; ++i) cnt += __popc(bal[i]);
  if (lane == 0) s_w[w] = cnt;
  __syncthreads();
  if (threadIdx.x == 0) {
    u32 t = 0;
    for (int i = 0; i < 8; ++i) t += s_w[i];
    tile_heads[blockIdx.x] = t;
  }
}

// One block: exclusive scan of tile_heads in place; writes U.
__global__ void __launch_bounds__(1024) k_uniq_scan(u32* __restrict__ tile_heads, u32 ntiles,
                                                    u32* __restrict__ n_unique, const u32* __restrict__ gate) {
  __shared__ u32 s_warp[32];
  __shared__ u32 s_carry;
  if (gate_skips(gate, 1)) return;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (threadIdx.x == 0) s_carry = 0;
  __syncthreads();
  for (u32 base = 0; base < ntiles; base += 1024) {
    u32 i = base + threadIdx.x;
    u32 v = i < ntiles ? tile_heads[i] : 0;
    u32 x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      u32 y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += y;
    }
    if (lane == 31) s_warp[w] = x;
    __syncthreads();
    if (w == 0) {
      u32 t = s_warp[lane];
      u32 xs = t;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        u32 y = __shfl_up_sync(0xffffffffu, xs, o);
        if (lane >= o) xs += y;
      }
      s_warp[lane] = xs - t;
    }
    __syncthreads();
    u32 carry = s_carry;
    if (i < ntiles) tile_heads[i] = carry + s_warp[w] + x - v;
    __syncthreads();
    if (threadIdx.x == 1023) s_carry = carry + s_warp[w] + x;
    __syncthreads();
  }
  if (threadIdx.x == 0) *n_unique = s_carry;
}

// Emits, for the sorted pairs (keys[i], pos[i]) held in buffer A or B (*where):
//   ukeys[u], seg_off[u] at segment heads (seg_off[U] = n),
//   csr_col[pos[i]] = u            (CSR remap to local column ids),
//   csc_row[i] = row of pos[i]     (the CSC row index),
//   csc_val[i] = vals[pos[i]]      (only when vals != null),
//   flagbits[i/32], wordbase[i/32] (head bitmap and heads before each word).
// Row of a position: pos / fixed_z when row_ptr is null, else the row whose
// [row_ptr[r], row_ptr[r+1]) contains it.
__global__ void __launch_bounds__(kLocThreads) k_uniq_emit(
    const u64* __restrict__ keys_a, const u64* __restrict__ keys_b, const u32* pos_a,
    const u32* pos_b, const u32* __restrict__ where, u32* csc_row /* may alias pos */, u32 n,
    const u32* __restrict__ tile_base,
    const u32* __restrict__ row_ptr, u32 n_rows, u32 fixed_z, const float* __restrict__ vals,
    u64* __restrict__ ukeys, u32* __restrict__ seg_off, u32* __restrict__ csr_col,
    float* __restrict__ csc_val, u32* __restrict__ flagbits, u32* __restrict__ wordbase, u64 kmask,
    const u32* __restrict__ gate) {
  __shared__ u32 s_w[8];
  if (gate_skips(gate, 1)) return;
  const bool in_b = where && *where;
  const u64* __restrict__ keys = in_b ? keys_b : keys_a;
  const u32* pos = in_b ? pos_b : pos_a;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const u32 base = blockIdx.x * (u32)kLocTile + w * (32 * kLocItems);
  u64 key[kLocItems];
  u32 bal[kLocItems];
  warp_heads(keys, n, base, lane, kmask, key, bal);
  u32 cnt = 0;
#pragma unroll
  for (int i = 0; i < kLocItems; ++i) cnt += __popc(bal[i]);
  if (lane == 0) s_w[w] = cnt;
  __syncthreads();
  u32 run = tile_base[blockIdx.x];
  for (int i = 0; i < w; ++i) run += s_w[i];
  const u32 zinv = fixed_z ? (u32)(0xffffffffu / fixed_z) : 0u;   // umulhi(p, zinv) <= p / fixed_z, short by at most 2
  const u32 le = 0xffffffffu >> (31 - lane);
#pragma unroll
  for (int i = 0; i < kLocItems; ++i) {
    u32 g = base + i * 32 + lane;
    if (g - lane < n && lane == 0) {
      flagbits[g >> 5] = bal[i];
      wordbase[g >> 5] = run;
    }
    if (g < n) {
      u32 u = run + __popc(bal[i] & le) - 1;
      if ((bal[i] >> lane) & 1u) {
        ukeys[u] = key[i] & kmask;
        seg_off[u] = g;
      }
      u32 p = pos ? pos[g] : (u32)(key[i] & ~kmask);   // packed: the position rides in the key's low bits
      csr_col[p] = u;
      if (csc_val) csc_val[g] = vals[p];
      u32 r;
      if (row_ptr == nullptr) {
        r = __umulhi(p, zinv);
        while (p - r * fixed_z >= fixed_z) ++r;   // the estimate is at most two short
      } else {
        u32 lo = 0, hi = n_rows;  // largest r with row_ptr[r] <= p
        while (hi - lo > 1) {
          u32 mid = (lo + hi) >> 1;
          if (row_ptr[mid] <= p) lo = mid; else hi = mid;
        }
        r = lo;
      }
      csc_row[g] = r;
    }
    run += __popc(bal[i]);
  }
}

// own_off[s] = lower_bound(ukeys[0..U), bounds[s]) for s in 0..S; own_off[S] = U.
// Also closes the CSC offsets with seg_off[U] = n.
__global__ void k_owner_offsets(const u64* __restrict__ ukeys, const u32* __restrict__ n_unique,
                                const u64* __restrict__ bounds, int S, u32 n,
                                u32* __restrict__ seg_off, u32* __restrict__ own_off,
                                const u32* __restrict__ gate, int want) {
  if (gate_skips(gate, want)) return;
  const u32 U = *n_unique;
  int s = threadIdx.x;
  if (s == 0 && seg_off) seg_off[U] = n;
  if (s > S) return;
  if (s == S) { own_off[S] = U; return; }
  u64 b = bounds[s];
  u32 lo = 0, hi = U;
  while (lo < hi) {
    u32 mid = (lo + hi) >> 1;
    if (ukeys[mid] < b) lo = mid + 1; else hi = mid;
  }
  own_off[s] = lo;
}

}  // namespace psb

using namespace psb;

// Owner slice offsets of an already sorted unique key list (generic Push/Pull
// path): own_off[s] = lower_bound(ukeys, bounds[s]), own_off[S] = *n_unique.
extern "C" int psb_owner_offsets(const psb_u64* ukeys, const uint32_t* n_unique, const psb_u64* bounds, int S,
                                 uint32_t* own_off, cudaStream_t stream) {
  if (S < 1 || S > 64) return -(int)cudaErrorInvalidValue;
  k_owner_offsets<<<1, 96, 0, stream>>>((const u64*)ukeys, n_unique, (const u64*)bounds, S, 0, nullptr, own_off, nullptr, 0);
  return -(int)cudaGetLastError();
}

extern "C" size_t psb_localize_scratch_bytes(uint32_t n) {
  size_t ntiles = (n + kLocTile - 1) / kLocTile;
  return sizeof(u32) * (ntiles + 16);
}

// The sorted pairs are in (keys_a, pos_a) when *where == 0 (or where is null) and
// in (keys_b, pos_b) otherwise. csc_row may alias the selected pos buffer.
static int localize2_impl(const psb_u64* keys_a, const psb_u64* keys_b, const uint32_t* pos_a,
                          const uint32_t* pos_b, const uint32_t* where, uint32_t* csc_row, uint32_t n,
                          const uint32_t* row_ptr, uint32_t n_rows, uint32_t fixed_z,
                          const float* vals, const psb_u64* bounds, int S, psb_u64* ukeys,
                          uint32_t* seg_off, uint32_t* csr_col, float* csc_val,
                          uint32_t* flagbits, uint32_t* wordbase, uint32_t* n_unique,
                          uint32_t* own_off, void* scratch, int pack_pos_bits, const uint32_t* gate,
                          cudaStream_t stream) {
  if (S < 1 || S > 64) return -(int)cudaErrorInvalidValue;
  if (row_ptr == nullptr && fixed_z == 0) return -(int)cudaErrorInvalidValue;
  if (pack_pos_bits < 0 || pack_pos_bits > 32) return -(int)cudaErrorInvalidValue;
  const u64 kmask = pack_pos_bits ? ~((1ull << pack_pos_bits) - 1) : ~0ull;
  if (pack_pos_bits) pos_a = pos_b = nullptr;
  u32 ntiles = (n + kLocTile - 1) / kLocTile;
  u32* tile_heads = (u32*)scratch;
  if (n == 0) {
    cudaMemsetAsync(n_unique, 0, sizeof(u32), stream);
    cudaMemsetAsync(own_off, 0, sizeof(u32) * (S + 1), stream);
    cudaMemsetAsync(seg_off, 0, sizeof(u32), stream);
    return -(int)cudaGetLastError();
  }
  k_uniq_count<<<ntiles, kLocThreads, 0, stream>>>((const u64*)keys_a, (const u64*)keys_b, where, n, tile_heads, kmask, gate);
  k_uniq_scan<<<1, 1024, 0, stream>>>(tile_heads, ntiles, n_unique, gate);
  k_uniq_emit<<<ntiles, kLocThreads, 0, stream>>>((const u64*)keys_a, (const u64*)keys_b, pos_a, pos_b, where, csc_row,
                                                  n, tile_heads, row_ptr, n_rows, fixed_z, vals, (u64*)ukeys, seg_off,
                                                  csr_col, csc_val, flagbits, wordbase, kmask, gate);
  k_owner_offsets<<<1, 96, 0, stream>>>((const u64*)ukeys, n_unique, (const u64*)bounds, S, n, seg_off, own_off, gate, 1);
  return -(int)cudaGetLastError();
}

extern "C" int psb_localize2(const psb_u64* keys_a, const psb_u64* keys_b, const uint32_t* pos_a,
                             const uint32_t* pos_b, const uint32_t* where, uint32_t* csc_row, uint32_t n,
                             const uint32_t* row_ptr, uint32_t n_rows, uint32_t fixed_z,
                             const float* vals, const psb_u64* bounds, int S, psb_u64* ukeys,
                             uint32_t* seg_off, uint32_t* csr_col, float* csc_val,
                             uint32_t* flagbits, uint32_t* wordbase, uint32_t* n_unique,
                             uint32_t* own_off, void* scratch, int pack_pos_bits, cudaStream_t stream) {
  return localize2_impl(keys_a, keys_b, pos_a, pos_b, where, csc_row, n, row_ptr, n_rows, fixed_z, vals, bounds, S,
                        ukeys, seg_off, csr_col, csc_val, flagbits, wordbase, n_unique, own_off, scratch,
                        pack_pos_bits, nullptr, stream);
}

// Same, but every kernel of the call returns at once unless the device word *gate is non-zero.
extern "C" int psb_localize2_gated(const psb_u64* keys_a, const psb_u64* keys_b, const uint32_t* pos_a,
                                   const uint32_t* pos_b, const uint32_t* where, uint32_t* csc_row, uint32_t n,
                                   const uint32_t* row_ptr, uint32_t n_rows, uint32_t fixed_z,
                                   const float* vals, const psb_u64* bounds, int S, psb_u64* ukeys,
                                   uint32_t* seg_off, uint32_t* csr_col, float* csc_val,
                                   uint32_t* flagbits, uint32_t* wordbase, uint32_t* n_unique,
                                   uint32_t* own_off, void* scratch, int pack_pos_bits, const uint32_t* gate,
                                   cudaStream_t stream) {
  return localize2_impl(keys_a, keys_b, pos_a, pos_b, where, csc_row, n, row_ptr, n_rows, fixed_z, vals, bounds, S,
                        ukeys, seg_off, csr_col, csc_val, flagbits, wordbase, n_unique, own_off, scratch,
                        pack_pos_bits, gate, stream);
}

// Owner offsets plus the closing CSC offset seg_off[U] = n; runs only while *skip_when_set is zero
// (the bucket-based localisation's last step).
extern "C" int psb_owner_offsets_n(const psb_u64* ukeys, const uint32_t* n_unique, const psb_u64* bounds, int S,
                                   uint32_t n, uint32_t* seg_off, uint32_t* own_off,
                                   const uint32_t* skip_when_set, cudaStream_t stream) {
  if (S < 1 || S > 64) return -(int)cudaErrorInvalidValue;
  k_owner_offsets<<<1, 96, 0, stream>>>((const u64*)ukeys, n_unique, (const u64*)bounds, S, n, seg_off, own_off,
                                        skip_when_set, 0);
  return -(int)cudaGetLastError();
}

// Sorted pairs in one buffer; sorted_pos is rewritten in place with the CSC row index.
extern "C" int psb_localize(const psb_u64* sorted_keys, uint32_t* sorted_pos, uint32_t n,
                            const uint32_t* row_ptr, uint32_t n_rows, uint32_t fixed_z,
                            const float* vals, const psb_u64* bounds, int S, psb_u64* ukeys,
                            uint32_t* seg_off, uint32_t* csr_col, float* csc_val,
                            uint32_t* flagbits, uint32_t* wordbase, uint32_t* n_unique,
                            uint32_t* own_off, void* scratch, cudaStream_t stream) {
  if (S < 1 || S > 64) return -(int)cudaErrorInvalidValue;
  if (row_ptr == nullptr && fixed_z == 0) return -(int)cudaErrorInvalidValue;
  u32 ntiles = (n + kLocTile - 1) / kLocTile;
  u32* tile_heads = (u32*)scratch;
  if (n == 0) {
    cudaMemsetAsync(n_unique, 0, sizeof(u32), stream);
    cudaMemsetAsync(own_off, 0, sizeof(u32) * (S + 1), stream);
    cudaMemsetAsync(seg_off, 0, sizeof(u32), stream);
    return -(int)cudaGetLastError();
  }
  k_uniq_count<<<ntiles, kLocThreads, 0, stream>>>((const u64*)sorted_keys, nullptr, nullptr, n, tile_heads, ~0ull, nullptr);
  k_uniq_scan<<<1, 1024, 0, stream>>>(tile_heads, ntiles, n_unique, nullptr);
  k_uniq_emit<<<ntiles, kLocThreads, 0, stream>>>((const u64*)sorted_keys, nullptr, sorted_pos, nullptr, nullptr,
                                                  sorted_pos, n, tile_heads, row_ptr, n_rows, fixed_z, vals,
                                                  (u64*)ukeys, seg_off, csr_col, csc_val, flagbits, wordbase, ~0ull, nullptr);
  k_owner_offsets<<<1, 96, 0, stream>>>((const u64*)ukeys, n_unique, (const u64*)bounds, S, n, seg_off, own_off, nullptr, 0);
  return -(int)cudaGetLastError();
}

// ---------------------------------------------------------------------------
// Allocation-free variant (declared in psb_noalloc.h; nothing like it exists in
// the reference). The per-tile head counts, which psb_localize keeps in a
// caller-provided scratch buffer, live in this fixed device array instead.
#include <mutex>
#include "psb_noalloc.h"

static __device__ __align__(256) unsigned int g_localize_static_scratch[PSB_LOCALIZE_STATIC_SCRATCH_WORDS];

namespace {
// In host code the array's name is only a handle for the runtime, not an
// address a kernel can use; the device address is looked up once per device,
// with that device current.
constexpr int kMaxDevices = 64;
std::mutex g_static_mu;
void* g_static_ptr[kMaxDevices] = {nullptr};

int localize_static_scratch(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return -(int)e;
  if (dev < 0 || dev >= kMaxDevices) return -(int)cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (g_static_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_localize_static_scratch);
    if (e != cudaSuccess) return -(int)e;
    g_static_ptr[dev] = p;
  }
  *out = g_static_ptr[dev];
  return 0;
}
}  // namespace

extern "C" int psb_localize_static(const psb_u64* sorted_keys, uint32_t* sorted_pos, uint32_t n,
                                   const uint32_t* row_ptr, uint32_t n_rows, uint32_t fixed_z,
                                   const float* vals, const psb_u64* bounds, int S, psb_u64* ukeys,
                                   uint32_t* seg_off, uint32_t* csr_col, float* csc_val,
                                   uint32_t* flagbits, uint32_t* wordbase, uint32_t* n_unique,
                                   uint32_t* own_off, cudaStream_t stream) {
  if (n > PSB_LOCALIZE_STATIC_MAX_N) return -(int)cudaErrorInvalidValue;  // beyond the built-in scratch
  if (S < 1 || S > 64) return -(int)cudaErrorInvalidValue;
  if (row_ptr == nullptr && fixed_z == 0) return -(int)cudaErrorInvalidValue;
  void* scratch = nullptr;
  int rc = localize_static_scratch(&scratch);
  if (rc != 0) return rc;
  u32* tile_heads = (u32*)scratch;
  if (n == 0) {
    cudaMemsetAsync(n_unique, 0, sizeof(u32), stream);
    cudaMemsetAsync(own_off, 0, sizeof(u32) * (S + 1), stream);
    cudaMemsetAsync(seg_off, 0, sizeof(u32), stream);
    return -(int)cudaGetLastError();
  }
  const u32 ntiles = (n + kLocTile - 1) / kLocTile;
  // every tile_heads word that the scan and the emit kernel read is written by
  // k_uniq_count first, so the array needs no clearing between calls
  k_uniq_count<<<ntiles, kLocThreads, 0, stream>>>((const u64*)sorted_keys, nullptr, nullptr, n, tile_heads, ~0ull, nullptr);
  k_uniq_scan<<<1, 1024, 0, stream>>>(tile_heads, ntiles, n_unique, nullptr);
  k_uniq_emit<<<ntiles, kLocThreads, 0, stream>>>((const u64*)sorted_keys, nullptr, sorted_pos, nullptr, nullptr,
                                                  sorted_pos, n, tile_heads, row_ptr, n_rows, fixed_z, vals,
                                                  (u64*)ukeys, seg_off, csr_col, csc_val, flagbits, wordbase, ~0ull, nullptr);
  k_owner_offsets<<<1, 96, 0, stream>>>((const u64*)ukeys, n_unique, (const u64*)bounds, S, n, seg_off,
                                        own_off, nullptr, 0);
  return -(int)cudaGetLastError();
}
