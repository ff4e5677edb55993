// Shared device-side building blocks for every sm_100a kernel in this library:
// key hashing, the server-shard hash-table entry, system-scope flag accessors,
// bounded waits and a bounded grid barrier.
//
// Rule for every wait in this library: it is a spin with an iteration limit.
// When the limit is hit the kernel records a code in a caller-supplied status
// word and returns; it never traps, asserts or loops forever.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace psb {

typedef unsigned long long u64;
typedef unsigned int u32;

// Largest uint64 is never a valid key (the key space is [0, 2^64-1)); it marks
// an empty hash-table slot.
static constexpr u64 kEmptyKey = 0xFFFFFFFFFFFFFFFFull;

// Status codes written (atomicMax) into the status word of a launch.
enum Status : u32 {
  kOk = 0,
  kTableFull = 1,        // linear probe wrapped without finding a free slot
  kInboxOverflow = 2,    // more records than the inbox capacity
  kWaitTimeout = 3,      // a bounded flag wait ran out
  kBarrierTimeout = 4,   // a bounded grid barrier ran out
  kLookbackTimeout = 5,  // decoupled look-back predecessor never published
  kBadArgument = 6,
};

__device__ __forceinline__ void set_status(u32* status, u32 code) {
  if (status) atomicMax(status, code);
}

// 64-bit finaliser of MurmurHash3 (public-domain mixing constants).
__host__ __device__ __forceinline__ u64 fmix64(u64 k) {
  k ^= k >> 33;
  k *= 0xff51afd7ed558ccdull;
  k ^= k >> 33;
  k *= 0xc4ceb9fe1a85ec53ull;
  k ^= k >> 33;
  return k;
}

// Feature id -> uint64 key. The low 56 bits of `seed_bits` are the seed, the top
// byte is the number of significant key bits B (0 means 64). For B = 64 the key is
// a 64-bit mix of the id (a bijection; the all-ones output is remapped). For
// B < 64 the id (which must be < 2^B) goes through a bijection of B-bit values
// (odd multiplications and right xor-shifts modulo 2^B) and the result is placed
// in the TOP B bits of the key: keys stay uniformly spread over the key space for
// range sharding, and a radix sort of them only needs ceil(B/8) digit passes.
__host__ __device__ __forceinline__ u64 hash_id_to_key(u64 id, u64 seed_bits) {
  const u64 seed = seed_bits & 0x00FFFFFFFFFFFFFFull;
  const int bits = (int)(seed_bits >> 56);
  if (bits == 0 || bits >= 64) {
    u64 k = fmix64(id + seed * 0x9E3779B97F4A7C15ull + 0x632BE59BD9B4E019ull);
    return k == kEmptyKey ? (kEmptyKey - 1) : k;
  }
  const u64 m = (1ull << bits) - 1;
  u64 h = (id + seed * 0x9E3779B97F4A7C15ull) & m;
  h = (h * 0xff51afd7ed558ccdull) & m;
  h ^= h >> (bits / 2);
  h = (h * 0xc4ceb9fe1a85ec53ull) & m;
  h ^= h >> (bits / 2 + 1);
  h = (h * 0x9E3779B97F4A7C15ull) & m;
  h ^= h >> (bits / 2);
  return h << (64 - bits);
}

// One slot of a server shard's open-addressing table for scalar (k=1) values.
// 32 bytes = one L2 sector / one NVLink read: a pull touches exactly one
// sector per key, an optimiser update reads and writes exactly one.
//   w     : the weight that Pull returns; {key, w} sit in the first 16 bytes so
//           a pull is a single 16-byte load
//   s0,s1 : optimiser state (FTRL: z, sqrt_n; AdaGrad: sum_sq_grad, unused)
//   gacc, gcnt : per-round accumulator of the duplicate-key reduce across sources: the sum of the
//           gradients pushed for the key in this round and how many sources pushed it. Both are
//           updated by ONE 8-byte vector atomic per pushed record (the source that finds gcnt == 0
//           becomes the key's leader) and both are zero between applies.
struct __align__(32) Entry {
  u64 key;
  float w;
  float s0;
  float s1;
  u32 pad;
  float gacc;     // 8-byte aligned together with gcnt
  float gcnt;
};
static_assert(sizeof(Entry) == 32, "Entry must be one 32-byte sector");

// ---- system-scope flag accessors (flags live in peer-mapped memory) ----
__device__ __forceinline__ u32 ld_acquire_sys(const u32* p) {
  u32 v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(u32* p, u32 v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ u32 ld_acquire_gpu(const u32* p) {
  u32 v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(u32* p, u32 v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ u32 ld_relaxed_gpu(const u32* p) {
  u32 v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_gpu(u32* p, u32 v) {
  asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// {a, b} += {x, y} as one 8-byte atomic on global memory (sm_90+ vector atomics); returns the old pair.
__device__ __forceinline__ float2 atomic_add_f32x2(float* addr8, float x, float y) {
  float2 old;
  asm volatile("atom.global.v2.f32.add {%0, %1}, [%2], {%3, %4};"
               : "=f"(old.x), "=f"(old.y) : "l"(addr8), "f"(x), "f"(y) : "memory");
  return old;
}
__device__ __forceinline__ u64 ld_relaxed_sys_u64(const u64* p) {
  u64 v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// Spin until *flag >= want (monotone counters), at most max_iters polls.
// Returns true on success. ~100 ns sleep between polls keeps the memory system
// quiet while a peer is still working.
__device__ __forceinline__ bool wait_flag_ge_sys(const u32* flag, u32 want, u32 max_iters) {
  for (u32 it = 0; it < max_iters; ++it) {
    if (ld_acquire_sys(flag) >= want) return true;
    __nanosleep(100);
  }
  return false;
}

// Default budgets, in polls. A cross-GPU poll is a 100 ns sleep plus a system-scope load (about 1.2 us
// in all), so 2^24 polls give a peer roughly 20 s (a rank may be held up by its data loader; a wait for
// S sources polls them one after another, so the worst case is S times that). An in-grid poll is a
// 40 ns sleep plus a load from L2 (under 1 us): 2^22 polls end a barrier that cannot complete after
// about 3 s. A wait that runs out sets the status word and the kernel carries on or returns; the host
// then clears the barrier and arrival words (check_status of the owning object) before the next launch.
static constexpr u32 kPeerWaitIters = 1u << 24;
static constexpr u32 kGridWaitIters = 1u << 22;

// Bounded grid-wide barrier for kernels launched cooperatively (all CTAs are
// co-resident). `bar` points at two zero-initialised u32 words {count, sense}
// that persist across launches (the barrier leaves count at 0). Returns false
// if the wait ran out; every thread of the CTA gets the same answer.
__device__ __forceinline__ bool grid_barrier(u32* bar, u32* status) {
  __shared__ u32 s_ok;
  __syncthreads();
  if (threadIdx.x == 0) {
    u32 ok = 1;
    u32 sense = ld_acquire_gpu(bar + 1);
    __threadfence();
    u32 arrived = atomicAdd(bar, 1u) + 1;
    if (arrived == gridDim.x * gridDim.y * gridDim.z) {
      atomicExch(bar, 0u);
      __threadfence();
      st_release_gpu(bar + 1, sense + 1);
    } else {
      u32 it = 0;
      while (ld_acquire_gpu(bar + 1) == sense) {
        if (++it > kGridWaitIters) { ok = 0; break; }
        __nanosleep(40);
      }
    }
    if (!ok) set_status(status, kBarrierTimeout);
    s_ok = ok;
  }
  __syncthreads();
  return s_ok != 0;
}

// How a key is mapped to its first probe slot. mult == 0: slot = fmix64(key) &
// mask (any key distribution). mult != 0: order-preserving map for keys that are
// already uniformly spread over the shard's range (hashed keys):
//   slot = floor((key - begin) * capacity / range_size) = umulhi(key - begin, mult),
// so that a sorted key list walks the table in address order (TLB- and
// DRAM-page-friendly for the pull and apply kernels, which see sorted keys).
struct SlotMap {
  u64 mask;
  u64 begin;
  u64 mult;
};
__device__ __forceinline__ u64 first_slot(const SlotMap& m, u64 key) {
  if (m.mult == 0) return fmix64(key) & m.mask;
  u64 s = __umul64hi(key - m.begin, m.mult);
  return s > m.mask ? m.mask : s;
}

// ---- open-addressing table probe (linear probing, power-of-two capacity) ----
// Returns the slot index of `key`, or -1 if absent (insert=false) / table full.
// `tab` may be a peer-mapped pointer: all accesses are plain loads plus one
// 64-bit CAS on insert, which NVLink carries natively.
template <bool kInsert>
__device__ __forceinline__ long long table_find(Entry* tab, const SlotMap& sm, u64 key, u32 max_probe) {
  const u64 mask = sm.mask;
  u64 slot = first_slot(sm, key);
  for (u32 p = 0; p < max_probe; ++p) {
    u64 k = ld_relaxed_sys_u64(&tab[slot].key);
    if (k == key) return (long long)slot;
    if (k == kEmptyKey) {
      if (!kInsert) return -1;
      u64 old = atomicCAS_system(&tab[slot].key, kEmptyKey, key);
      if (old == kEmptyKey || old == key) return (long long)slot;
    }
    slot = (slot + 1) & mask;
  }
  return -1;
}

// Pull-side probe: one 16-byte load per probed slot returns key and weight.
// Returns the slot (or -1) and writes the weight (0 when absent).
__device__ __forceinline__ long long table_lookup_w(const Entry* tab, const SlotMap& sm, u64 key,
                                                    u32 max_probe, float* w_out) {
  const u64 mask = sm.mask;
  u64 slot = first_slot(sm, key);
  for (u32 p = 0; p < max_probe; ++p) {
    u64 k, hi;
    asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];"
                 : "=l"(k), "=l"(hi) : "l"(&tab[slot]) : "memory");
    if (k == key) { *w_out = __uint_as_float((u32)hi); return (long long)slot; }
    if (k == kEmptyKey) break;
    slot = (slot + 1) & mask;
  }
  *w_out = 0.f;
  return -1;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Owner of a position in the sorted unique-key list: own_off[s] <= u < own_off[s+1].
__device__ __forceinline__ int owner_of(const u32* own_off, int S, u32 u) {
  int s = 0;
#pragma unroll 1
  while (s + 1 < S && u >= own_off[s + 1]) ++s;
  return s;
}

}  // namespace psb
