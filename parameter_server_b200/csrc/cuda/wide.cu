// Wide-value path (kernel family F4): tables whose values are 64-wide bf16
// vectors with fp32 AdaGrad accumulators on the server side.
//
//   k_wide_pull_gemm  worker: for a tile of 128 unique keys, locate each key in
//                     its owner's key table and fetch its 128-byte value row
//                     (plain loads; the owner may be a peer GPU) straight into
//                     shared memory in the 128-byte-swizzled K-major layout that
//                     the tensor core expects, then multiply the [128 x 64] tile
//                     by the batch's [64 x N] context matrix with tcgen05.mma
//                     (accumulator in TMEM), read the result back with tcgen05.ld
//                     and either store P[U x N] or, fused, add each product that a
//                     row needs straight into that row's margin: the tile's
//                     products are staged in shared memory and the CTA walks the
//                     CSC segments of the tile's keys (margin[row] += P[key,
//                     context(row)]), so the U x N matrix never reaches memory.
//                     The context matrix is brought in once
//                     per CTA by a TMA tiled load (cp.async.bulk.tensor.2d, no
//                     multicast) with the same swizzle.
//   k_wide_rowsum     worker: prediction per row = sum over its keys of
//                     P[key, context(row)], logistic loss and d loss / d margin
//                     (the unfused form, from a stored P).
//   k_wide_rowloss    worker: logistic loss and d loss / d margin from margins that
//                     the fused pull has accumulated.
//   k_wide_push       worker: gradient of every unique key,
//                     G[u,:] = sum_{rows containing u} gcoef[row] * C[:, ctx(row)],
//                     one warp per key over the CSC segment, written as bf16
//                     records into the owner's inbox by peer stores + release flag.
//   k_wide_apply      owner: bounded wait per source, then AdaGrad on the fp32
//                     accumulators and bf16 weights, sources applied in rank order
//                     (grid barrier between sources).
//
// Only loads/stores through peer pointers cross GPUs; the TMA load reads local
// memory and carries no multicast qualifier.
#include <cuda.h>
#include <cuda_bf16.h>
#include "psb_common.cuh"
#include "psb_cuda.h"

namespace psb {

static constexpr int kWide = 64;                 // values per key
static constexpr int kTileM = 128;               // keys per MMA tile
static constexpr u32 kWideProbe = 1u << 16;
static constexpr u32 kPullLongSeg = 512;         // fused margins: longer segments go to k_wide_long_margins

// ---------------------------------------------------------------- small PTX wrappers
__device__ __forceinline__ u32 smem_u32(const void* p) { return (u32)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(u64* bar, u32 count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(u64* bar, u32 bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// bounded wait on a phase parity; false if the budget ran out
__device__ __forceinline__ bool mbar_wait(u64* bar, u32 parity, u32 max_iters) {
  const u32 addr = smem_u32(bar);
  for (u32 it = 0; it < max_iters; ++it) {
    u32 ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
    if (ok) return true;
  }
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, u64* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_alloc(u32* smem_out, u32 ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_out)), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(u32 taddr, u32 ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// K-major operand tile in shared memory, rows of 128 bytes, 128-byte swizzle:
// 8-row groups are 1024 bytes apart (SBO); LBO is unused for this layout.
__device__ __forceinline__ u64 make_smem_desc(u32 smem_addr) {
  u64 d = 0;
  d |= (u64)((smem_addr & 0x3FFFF) >> 4);         // start address
  d |= (u64)(16 >> 4) << 16;                      // leading byte offset (ignored)
  d |= (u64)(1024 >> 4) << 32;                    // stride byte offset between 8-row groups
  d |= 1ull << 46;                                // descriptor version of this architecture
  d |= 2ull << 61;                                // 128-byte swizzle
  return d;
}
// kind::f16, bf16 x bf16 -> fp32, both operands K-major, M x N tile
__device__ __forceinline__ u32 make_idesc(int M, int N) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((u32)(N >> 3) << 17) | ((u32)(M >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(u32 tmem_d, u64 desc_a, u64 desc_b, u32 idesc, u32 accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(u64* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 32 lanes x 32 columns of 32-bit: thread i of the warp gets row (lane base + i)
__device__ __forceinline__ void tmem_ld_32x32(u32 taddr, u32* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---------------------------------------------------------------- key table of a wide shard
// keys[slot] (u64, kEmptyKey = free); values at vals + slot*64 (bf16), accumulators at acc + slot*64 (fp32)
template <bool kInsert>
__device__ __forceinline__ long long wide_find(u64* keys, const SlotMap& sm, u64 key) {
  u64 slot = first_slot(sm, key);
  for (u32 p = 0; p < kWideProbe; ++p) {
    u64 k = ld_relaxed_sys_u64(&keys[slot]);
    if (k == key) return (long long)slot;
    if (k == kEmptyKey) {
      if (!kInsert) return -1;
      u64 old = atomicCAS_system(&keys[slot], kEmptyKey, key);
      if (old == kEmptyKey || old == key) return (long long)slot;
    }
    slot = (slot + 1) & sm.mask;
  }
  return -1;
}

// ---------------------------------------------------------------- F4: pull + GEMM
struct WidePullArgs {
  int S;
  int N;                                  // contexts (columns of the result): 64 or 128
  psb_u64* keys[PSB_MAX_SHARDS];
  const __nv_bfloat16* vals[PSB_MAX_SHARDS];
  psb_u64 mask[PSB_MAX_SHARDS], key_begin[PSB_MAX_SHARDS], slot_mult[PSB_MAX_SHARDS];
  const psb_u64* ukeys;
  const uint32_t* n_unique;
  const uint32_t* own_off;
  float* P;                               // [U x N] fp32
  __nv_bfloat16* v_local;                 // nullable: gathered rows [U x 64]
  uint32_t* status;
  // fused margins (margin non-null; P may then be null): CSC of the batch and the rows' contexts
  const uint32_t* seg_off;
  const uint32_t* csc_row;
  const uint32_t* row_ctx;                // nullable -> row % N
  float* margin;                          // [n_rows], zero on entry
  // keys with long segments are only listed here (with their row of products); k_wide_long_margins adds them
  unsigned long long* plong_n;            // {count (low word), chunks (high word)}, zero on entry
  uint4* plong_list;                      // {unused, first chunk, first element, end element}
  float* plong_rows;                      // [plong_cap x N]
  uint32_t plong_cap;
};

// Exchange form of the pull (see k_wide_pull_xgemm): per-owner flags and buffers.
struct WideXArgs {
  int S, me;
  int N;
  uint32_t ts1, req_cap, wait_iters, phases;
  // my shard (owner role)
  psb_u64* keys;
  const __nv_bfloat16* vals;
  psb_u64 mask, key_begin, slot_mult;
  // requester role: where my keys go and who tells me that my rows have arrived
  psb_u64* req_keys[PSB_MAX_SHARDS];         // owner s's request buffer for source me
  uint32_t* req_hdr[PSB_MAX_SHARDS];         // {count, base} at owner s for source me
  uint32_t* req_ready[PSB_MAX_SHARDS];
  const uint32_t* my_resp_ready[PSB_MAX_SHARDS];   // set by owner s when my rows are in place
  const __nv_bfloat16* my_resp_rows;         // [pull_cap x 64] local
  // owner role: the sources' requests here, and their response buffers
  const psb_u64* my_req_keys[PSB_MAX_SHARDS];
  const uint32_t* my_req_hdr[PSB_MAX_SHARDS];
  const uint32_t* my_req_ready[PSB_MAX_SHARDS];
  __nv_bfloat16* resp_rows[PSB_MAX_SHARDS];  // source r's response buffer
  uint32_t* resp_ready[PSB_MAX_SHARDS];      // source r's flag for owner me
  uint8_t alive[PSB_MAX_SHARDS];
  const psb_u64* ukeys;
  const uint32_t* n_unique;
  const uint32_t* own_off;
  float* P;
  uint32_t* done;                            // 2 words, zero on entry, left zero
  uint32_t* status;
  // fused margins, as in WidePullArgs
  const uint32_t* seg_off;
  const uint32_t* csc_row;
  const uint32_t* row_ctx;
  float* margin;
  unsigned long long* plong_n;
  uint4* plong_list;
  float* plong_rows;
  uint32_t plong_cap;
};

// Shared state of the tensor-core tile loop.
struct WideTileCtx {
  unsigned char* sA;
  unsigned char* sB;
  u64* bar;        // 2 mbarriers: 0 = TMA, 1 = MMA
  u32 tmem_base;
  u32 idesc;
  u32 phase;
  u32* s_fail;
  // fused margins: staging of the tile's products [128 x (N + 1)] fp32 and of its 129 segment offsets
  float* sP;
  u32* s_seg;      // [129] segment offsets of the tile's keys
  u32* s_pre;      // [129] prefix of the short keys' lengths
  u32* s_wsum;     // [4]
  const u32* seg_off;
  const u32* csc_row;
  const u32* row_ctx;
  float* margin;
  unsigned long long* plong_n;
  uint4* plong_list;
  float* plong_rows;
  u32 plong_cap;
};

// One [128 x 64] x [64 x N] tile: `row` holds this thread's 128-byte value row (zeros when
// absent); the product goes to P[u, :].
__device__ __forceinline__ bool wide_tile_mma_store(WideTileCtx& c, const uint4 (&row)[8], u32 u, u32 U, int N, float* P,
                                                    u32* status) {
  const int tid = threadIdx.x, warp = tid >> 5;
#pragma unroll
  for (int q = 0; q < 8; ++q)   // 16-byte chunk q of row r lands at chunk (q ^ (r & 7))
    *reinterpret_cast<uint4*>(c.sA + tid * 128 + ((q ^ (tid & 7)) << 4)) = row[q];
  fence_async_smem();
  __syncthreads();
  // ---- MMA: one thread issues K = 64 as four K = 16 steps
  if (tid == 0) {
    tc_fence_after();
    const u64 da = make_smem_desc(smem_u32(c.sA)), db = make_smem_desc(smem_u32(c.sB));
#pragma unroll
    for (int k = 0; k < 4; ++k) umma_bf16(c.tmem_base, da + (u64)(2 * k), db + (u64)(2 * k), c.idesc, k > 0 ? 1u : 0u);
    umma_commit(&c.bar[1]);
  }
  if (!mbar_wait(&c.bar[1], c.phase, 1u << 22)) { if (tid == 0) { *c.s_fail = 1; set_status(status, kWaitTimeout); } }
  c.phase ^= 1;
  tc_fence_after();
  __syncthreads();
  if (*c.s_fail) return false;
  // ---- epilogue: warp w owns TMEM lanes [32w, 32w+32) = rows of the tile
  const int ldp = N + 1;                          // padded: thread = row, so a column is a bank stride apart
  for (int c0 = 0; c0 < N; c0 += 32) {
    u32 r[32];
    tmem_ld_32x32(c.tmem_base + ((u32)(warp * 32) << 16) + (u32)c0, r);
    if (P != nullptr && u < U) {
      float4* dst = reinterpret_cast<float4*>(P + (size_t)u * N + c0);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        dst[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                             __uint_as_float(r[4 * j + 3]));
    }
    if (c.margin != nullptr) {
#pragma unroll
      for (int j = 0; j < 32; ++j) c.sP[tid * ldp + c0 + j] = __uint_as_float(r[j]);
    }
  }
  tc_fence_before();
  if (c.margin != nullptr) {
    // The tile's keys own the contiguous nonzeros [seg_off[u0], seg_off[u0 + 128)): every nonzero adds the
    // product of its key and its row's context to the row's margin. A key with a long segment (under a
    // Zipf law one key can own a fifth of all nonzeros) is only listed, with its row of products, and
    // k_wide_long_margins spreads it over the whole grid; the others are walked here, all 128 threads
    // over the short keys' nonzeros laid end to end.
    const u32 u0 = u - (u32)tid;
    c.s_seg[tid] = c.seg_off[min(u0 + (u32)tid, U)];
    if (tid == 0) c.s_seg[kTileM] = c.seg_off[min(u0 + (u32)kTileM, U)];
    __syncthreads();
    const u32 i0 = c.s_seg[tid], len = c.s_seg[tid + 1] - i0;
    bool is_long = false;
    if (len > kPullLongSeg && c.plong_cap) {
      const u32 nch = (len + kPullLongSeg - 1) / kPullLongSeg;
      const unsigned long long old = atomicAdd(c.plong_n, 1ull | ((unsigned long long)nch << 32));
      const u32 k = (u32)old;
      if (k < c.plong_cap) {
        is_long = true;
        c.plong_list[k] = make_uint4(u, (u32)(old >> 32), i0, i0 + len);
        for (int j = 0; j < N; ++j) c.plong_rows[(size_t)k * N + j] = c.sP[tid * ldp + j];
      }                                            // a full list: the key is walked here after all
    }
    // exclusive prefix of the short keys' lengths (warp scans, then the four warp totals)
    const u32 mine = is_long ? 0u : len;
    u32 inc = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const u32 v = __shfl_up_sync(0xffffffffu, inc, o);
      if ((tid & 31) >= o) inc += v;
    }
    if ((tid & 31) == 31) c.s_wsum[warp] = inc;
    __syncthreads();
    u32 base = 0;
    for (int w = 0; w < warp; ++w) base += c.s_wsum[w];
    c.s_pre[tid] = base + inc - mine;
    if (tid == kTileM - 1) c.s_pre[kTileM] = base + inc;
    __syncthreads();
    const u32 total = c.s_pre[kTileM];
    for (u32 t = tid; t < total; t += kTileM) {
      int lo = 0, hi = kTileM - 1;                 // the last key whose share starts at or before t
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (c.s_pre[mid] <= t) lo = mid; else hi = mid - 1;
      }
      const u32 row = c.csc_row[c.s_seg[lo] + (t - c.s_pre[lo])];
      const u32 cx = c.row_ctx ? c.row_ctx[row] : row % (u32)N;
      atomicAdd(&c.margin[row], c.sP[lo * ldp + (int)cx]);
    }
  }
  __syncthreads();
  return true;
}

// Common prologue: mbarriers, TMEM allocation, context matrix by TMA. Returns false on a time-out.
__device__ __forceinline__ bool wide_tile_setup(WideTileCtx& c, const CUtensorMap* ctx_map, int N, u32* s_tmem, u32* status) {
  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid == 0) {
    *c.s_fail = 0;
    mbar_init(&c.bar[0], 1);
    mbar_init(&c.bar[1], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) tmem_alloc(s_tmem, (u32)N);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  c.tmem_base = *s_tmem;
  if (tid == 0) {
    mbar_expect_tx(&c.bar[0], (u32)N * 128u);
    tma_load_2d(c.sB, ctx_map, 0, 0, &c.bar[0]);
  }
  if (!mbar_wait(&c.bar[0], 0, 1u << 22)) { if (tid == 0) { *c.s_fail = 1; set_status(status, kWaitTimeout); } }
  __syncthreads();
  c.idesc = make_idesc(kTileM, N);
  c.phase = 0;
  return *c.s_fail == 0;
}

__global__ void __launch_bounds__(128) k_wide_pull_gemm(const __grid_constant__ CUtensorMap ctx_map, const WidePullArgs p) {
  // operand tiles: 1024-byte aligned because of the 128-byte swizzle
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ u64 s_bar[2];
  __shared__ u32 s_tmem;
  __shared__ u32 s_off[PSB_MAX_SHARDS + 1];
  __shared__ u32 s_fail;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int N = p.N;
  const u32 U = *p.n_unique;
  if (tid <= p.S) s_off[tid] = p.own_off[tid];
  __shared__ u32 s_seg[kTileM + 1], s_pre[kTileM + 1], s_wsum[4];
  WideTileCtx c{smem, smem + kTileM * 128, s_bar, 0, 0, 0, &s_fail,
                reinterpret_cast<float*>(smem + kTileM * 128 + N * 128), s_seg, s_pre, s_wsum,
                p.seg_off, p.csc_row, p.row_ctx, p.margin, p.plong_n, p.plong_list, p.plong_rows, p.plong_cap};
  wide_tile_setup(c, &ctx_map, N, &s_tmem, p.status);
  const u32 ntiles = (U + kTileM - 1) / kTileM;
  for (u32 t = blockIdx.x; t < ntiles && !s_fail; t += gridDim.x) {
    // ---- gather: thread = one key = one 128-byte row
    const u32 u = t * kTileM + tid;
    uint4 row[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) row[q] = make_uint4(0, 0, 0, 0);
    if (u < U) {
      int s = owner_of(s_off, p.S, u);
      const SlotMap sm{p.mask[s], p.key_begin[s], p.slot_mult[s]};
      long long slot = wide_find<false>((u64*)p.keys[s], sm, p.ukeys[u]);
      if (slot >= 0) {
        const uint4* src = reinterpret_cast<const uint4*>(p.vals[s] + (size_t)slot * kWide);
#pragma unroll
        for (int q = 0; q < 8; ++q) row[q] = src[q];
      }
      if (p.v_local) {
        uint4* dst = reinterpret_cast<uint4*>(p.v_local + (size_t)u * kWide);
#pragma unroll
        for (int q = 0; q < 8; ++q) dst[q] = row[q];
      }
    }
    if (!wide_tile_mma_store(c, row, u, U, N, p.P, p.status)) break;
  }
  __syncthreads();
  if (warp == 0) tmem_dealloc(c.tmem_base, (u32)N);
}

// Exchange form of the fused pull: three roles in one cooperative kernel.
//   (a) requester: my sorted unique keys go to their owners' request buffers in bulk;
//   (b) owner: for every source, look its keys up in my table and store the 128-byte
//       value rows into the source's response buffer (peer stores), then raise that
//       source's flag;
//   (c) requester: tile by tile, wait for the flags of the owners that cover the tile,
//       read the rows from the local response buffer and run the tcgen05 product.
// Only bulk stores cross NVLink (keys out, rows back); tiles of an owner that has
// answered are multiplied while other owners are still sending. `phases` (bit 0: a,
// bit 1: b, bit 2: c) lets ranks emulated on one GPU run the roles as separate launches.
__global__ void __launch_bounds__(128) k_wide_pull_xgemm(const __grid_constant__ CUtensorMap ctx_map, const WideXArgs p) {
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ u64 s_bar[2];
  __shared__ u32 s_tmem;
  __shared__ u32 s_off[PSB_MAX_SHARDS + 1];
  __shared__ u32 s_fail, s_last, s_n, s_base;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int S = p.S, N = p.N;
  const u32 U = *p.n_unique;
  const u32 iters = p.wait_iters ? p.wait_iters : kPeerWaitIters;
  const u32 gsize = gridDim.x * blockDim.x, gtid = blockIdx.x * blockDim.x + tid;
  if (tid <= S) s_off[tid] = p.own_off[tid];
  __syncthreads();
  // ---- (a)
  if (p.phases & 1) {
    for (u32 u = gtid; u < U; u += gsize) {
      int s = owner_of(s_off, S, u);
      u32 j = u - s_off[s];
      if (j < p.req_cap) p.req_keys[s][j] = p.ukeys[u];
    }
    __threadfence_system();
    __syncthreads();
    if (tid == 0) s_last = atomicAdd(&p.done[0], 1u) + 1 == gridDim.x;
    __syncthreads();
    if (s_last && tid < S) {
      int s = tid;
      u32 cnt = s_off[s + 1] - s_off[s];
      if (cnt > p.req_cap) { set_status(p.status, kInboxOverflow); cnt = p.req_cap; }
      __threadfence_system();
      p.req_hdr[s][0] = cnt;
      p.req_hdr[s][1] = s_off[s];
      __threadfence_system();
      st_release_sys(p.req_ready[s], p.ts1);
      if (s == 0) atomicExch(&p.done[0], 0u);
    }
  }
  // ---- (b)
  if (p.phases & 2) {
    const SlotMap sm{p.mask, p.key_begin, p.slot_mult};
    for (int r = 0; r < S; ++r) {
      if (!p.alive[r]) continue;
      __syncthreads();
      if (tid == 0) {
        u32 n = 0, base = 0;
        if (wait_flag_ge_sys(p.my_req_ready[r], p.ts1, iters)) {
          n = *((volatile const u32*)&p.my_req_hdr[r][0]);
          base = *((volatile const u32*)&p.my_req_hdr[r][1]);
        } else {
          set_status(p.status, kWaitTimeout);
        }
        s_n = min(n, p.req_cap);
        s_base = base;
      }
      __syncthreads();
      const u32 n = s_n, base = s_base;
      // Eight lanes per key: the look-up by the first of them, then one 16-byte chunk each. Four keys
      // per lane group and trip, every stage issued for all four before the next stage starts (key,
      // first probe, row chunk are a chain of dependent loads). The trip count is the same for every
      // lane of a warp: the shuffle needs all of them.
      const u32 n8 = (n * 8 + 31) & ~31u;
      for (u32 j8 = gtid; j8 < n8; j8 += 4 * gsize) {
        u64 key[4], k0[4], sl0[4];
        long long slot[4];
        bool act[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const u32 x = j8 + q * gsize;
          act[q] = x < n8;                          // the same for a whole warp
          key[q] = (act[q] && (x >> 3) < n && (x & 7) == 0) ? p.my_req_keys[r][x >> 3] : kEmptyKey;
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          sl0[q] = first_slot(sm, key[q]);
          k0[q] = key[q] != kEmptyKey ? ld_relaxed_sys_u64(&p.keys[sl0[q]]) : kEmptyKey;
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          slot[q] = -1;
          if (key[q] != kEmptyKey) slot[q] = k0[q] == key[q] ? (long long)sl0[q] : wide_find<false>(p.keys, sm, key[q]);
          if (act[q]) slot[q] = __shfl_sync(0xffffffffu, slot[q], (tid & 31) & ~7);
        }
        uint4 v[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const u32 x = j8 + q * gsize;
          v[q] = make_uint4(0, 0, 0, 0);
          if (act[q] && slot[q] >= 0) v[q] = reinterpret_cast<const uint4*>(p.vals + (size_t)slot[q] * kWide)[x & 7];
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const u32 x = j8 + q * gsize;
          if (act[q] && (x >> 3) < n) reinterpret_cast<uint4*>(p.resp_rows[r] + (size_t)(base + (x >> 3)) * kWide)[x & 7] = v[q];
        }
      }
    }
    __threadfence_system();
    __syncthreads();
    if (tid == 0) s_last = atomicAdd(&p.done[1], 1u) + 1 == gridDim.x;
    __syncthreads();
    if (s_last && tid < S && p.alive[tid]) {
      __threadfence_system();
      st_release_sys(p.resp_ready[tid], p.ts1);
    }
    if (s_last && tid == 0) atomicExch(&p.done[1], 0u);
  }
  if (!(p.phases & 4)) return;
  // ---- (c)
  __shared__ u32 s_seg[kTileM + 1], s_pre[kTileM + 1], s_wsum[4];
  WideTileCtx c{smem, smem + kTileM * 128, s_bar, 0, 0, 0, &s_fail,
                reinterpret_cast<float*>(smem + kTileM * 128 + N * 128), s_seg, s_pre, s_wsum,
                p.seg_off, p.csc_row, p.row_ctx, p.margin, p.plong_n, p.plong_list, p.plong_rows, p.plong_cap};
  wide_tile_setup(c, &ctx_map, N, &s_tmem, p.status);
  const u32 ntiles = (U + kTileM - 1) / kTileM;
  for (u32 t = blockIdx.x; t < ntiles && !s_fail; t += gridDim.x) {
    const u32 u0 = t * kTileM, u = u0 + tid;
    if (tid == 0) {
      const int sa = owner_of(s_off, S, u0), sb = owner_of(s_off, S, min(u0 + kTileM - 1, U - 1));
      for (int s = sa; s <= sb; ++s)
        if (p.alive[s] && !wait_flag_ge_sys(p.my_resp_ready[s], p.ts1, iters)) { s_fail = 1; set_status(p.status, kWaitTimeout); }
    }
    __syncthreads();
    if (s_fail) break;
    uint4 row[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) row[q] = make_uint4(0, 0, 0, 0);
    if (u < U) {
      const uint4* src = reinterpret_cast<const uint4*>(p.my_resp_rows + (size_t)u * kWide);
#pragma unroll
      for (int q = 0; q < 8; ++q) row[q] = src[q];
    }
    if (!wide_tile_mma_store(c, row, u, U, N, p.P, p.status)) break;
  }
  __syncthreads();
  if (warp == 0) tmem_dealloc(c.tmem_base, (u32)N);
}

// ---------------------------------------------------------------- rows: prediction, loss, gcoef
__global__ void __launch_bounds__(256) k_wide_rowsum(const float* __restrict__ P, int N, const u32* __restrict__ row_ptr,
                                                     u32 n_rows, u32 fixed_z, const u32* __restrict__ csr_col,
                                                     const u32* __restrict__ row_ctx, const float* __restrict__ y,
                                                     float* __restrict__ gcoef, float* __restrict__ margin,
                                                     double* __restrict__ stats) {
  const int lane = threadIdx.x & 31;
  const u32 gwarp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = (gridDim.x * blockDim.x) >> 5;
  double loss = 0, correct = 0, seen = 0;
  for (u32 r = gwarp; r < n_rows; r += nwarps) {
    u32 b = row_ptr ? row_ptr[r] : r * fixed_z, e = row_ptr ? row_ptr[r + 1] : b + fixed_z;
    u32 ctx = row_ctx ? row_ctx[r] : r % (u32)N;
    float acc = 0.f;
    for (u32 j = b + lane; j < e; j += 32) acc += P[(size_t)csr_col[j] * N + ctx];
    acc = warp_sum(acc);
    if (lane == 0) {
      float yy = y[r], ym = yy * acc;
      float en = expf(-fabsf(ym));
      float tau = ym > 0 ? en / (1.f + en) : 1.f / (1.f + en);
      gcoef[r] = -yy * tau;
      if (margin) margin[r] = acc;
      loss += log1pf(en) + fmaxf(-ym, 0.f);
      correct += ym > 0 ? 1 : 0;
      seen += 1;
    }
  }
  loss = warp_sum_d(loss); correct = warp_sum_d(correct); seen = warp_sum_d(seen);
  if (lane == 0 && stats && seen > 0) { atomicAdd(&stats[0], loss); atomicAdd(&stats[1], correct); atomicAdd(&stats[2], seen); }
}

// The long segments that the fused pull listed: chunks of kPullLongSeg nonzeros, one per warp and trip
// (the list is sorted by first chunk: one 64-bit atomic handed out position and chunk numbers together).
__global__ void __launch_bounds__(256) k_wide_long_margins(const unsigned long long* __restrict__ plong_n,
                                                           const uint4* __restrict__ list, const float* __restrict__ rows,
                                                           u32 cap, int N, const u32* __restrict__ csc_row,
                                                           const u32* __restrict__ row_ctx, float* __restrict__ margin) {
  const int lane = threadIdx.x & 31;
  const u32 gwarp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = (gridDim.x * blockDim.x) >> 5;
  const unsigned long long tot = *plong_n;
  const u32 n_long = min((u32)tot, cap);
  const u32 n_chunks = n_long ? (u32)(tot >> 32) : 0u;
  for (u32 c = gwarp; c < n_chunks; c += nwarps) {
    u32 lo = 0, hi = n_long;                       // the entry with the largest first chunk <= c
    while (hi - lo > 1) {
      const u32 mid = (lo + hi) >> 1;
      if (list[mid].y <= c) lo = mid; else hi = mid;
    }
    const uint4 e = list[lo];
    const u32 b0 = e.z + (c - e.y) * kPullLongSeg;
    if (b0 >= e.w) continue;                       // (a chunk number of a key that did not fit the list)
    const u32 b1 = min(e.w, b0 + kPullLongSeg);
    for (u32 i = b0 + lane; i < b1; i += 32) {
      const u32 row = csc_row[i];
      const u32 cx = row_ctx ? row_ctx[row] : row % (u32)N;
      atomicAdd(&margin[row], rows[(size_t)lo * N + cx]);
    }
  }
}

// margins are complete (the fused pull added every product): loss, accuracy and d loss / d margin per row
__global__ void __launch_bounds__(256) k_wide_rowloss(const float* __restrict__ margin, const float* __restrict__ y,
                                                      u32 n_rows, float* __restrict__ gcoef, double* __restrict__ stats,
                                                      unsigned long long* plong_n) {
  const int lane = threadIdx.x & 31;
  if (plong_n != nullptr && blockIdx.x == 0 && threadIdx.x == 0) *plong_n = 0ull;   // the list is used up
  double loss = 0, correct = 0, seen = 0;
  for (u32 r = blockIdx.x * blockDim.x + threadIdx.x; r < n_rows; r += gridDim.x * blockDim.x) {
    const float yy = y[r], ym = yy * margin[r];
    const float en = expf(-fabsf(ym));
    const float tau = ym > 0 ? en / (1.f + en) : 1.f / (1.f + en);
    gcoef[r] = -yy * tau;
    loss += log1pf(en) + fmaxf(-ym, 0.f);
    correct += ym > 0 ? 1 : 0;
    seen += 1;
  }
  loss = warp_sum_d(loss); correct = warp_sum_d(correct); seen = warp_sum_d(seen);
  if (lane == 0 && stats && seen > 0) { atomicAdd(&stats[0], loss); atomicAdd(&stats[1], correct); atomicAdd(&stats[2], seen); }
}

// ---------------------------------------------------------------- push: per-key gradient rows to the owners
struct WidePushArgs {
  int S;
  int N;
  uint32_t ts1, inbox_cap;
  psb_u64* inbox_keys[PSB_MAX_SHARDS];
  __nv_bfloat16* inbox_vals[PSB_MAX_SHARDS];   // [cap x 64]
  uint32_t* ready[PSB_MAX_SHARDS];
  uint32_t* count[PSB_MAX_SHARDS];
  const psb_u64* ukeys;
  const uint32_t* n_unique;
  const uint32_t* own_off;
  const uint32_t* seg_off;
  const uint32_t* csc_row;
  const float* gcoef;
  const uint32_t* row_ctx;                     // nullable -> row % N
  const __nv_bfloat16* ctx;                    // [N x 64] (context n in row n)
  uint32_t* done;
  uint32_t* status;
  uint32_t* bar;                               // 2 words (grid barrier), zero on first use
  unsigned long long* n_long;                  // {count (low word), chunks (high word)}, zero on entry, left zero
  uint4* long_list;                            // long_cap entries {key index, first chunk, first element, end element}
  float* long_acc;                             // long_cap x 64 floats, zero on entry, left zero
  uint32_t long_cap;
};

// Segments longer than this are reduced by many warps (under a Zipf law one key can
// own a fifth of all nonzeros; a single warp walking it would take milliseconds).
static constexpr u32 kWideLongSeg = 256;

// G += sum over the elements [i0, i1) of gcoef[row] * C[ctx(row), 2*lane .. 2*lane+1]; the row ids,
// coefficients and context ids of 32 elements are fetched by the lanes in parallel and then
// broadcast one by one, the context rows come from shared memory.
__device__ __forceinline__ void wide_seg_accumulate(const WidePushArgs& p, const __nv_bfloat162* s_ctx, u32 i0, u32 i1,
                                                    int lane, float& g0, float& g1) {
  for (u32 base = i0; base < i1; base += 32) {
    const u32 i = base + lane;
    float gc = 0.f;
    u32 n = 0;
    if (i < i1) {
      const u32 r = __ldcs(&p.csc_row[i]);
      gc = __ldg(&p.gcoef[r]);
      n = p.row_ctx ? p.row_ctx[r] : r % (u32)p.N;
    }
    const int cnt = (int)min(32u, i1 - base);
    for (int e = 0; e < cnt; ++e) {
      const float gce = __shfl_sync(0xffffffffu, gc, e);
      const u32 ne = __shfl_sync(0xffffffffu, n, e);
      const __nv_bfloat162 c2 = s_ctx[ne * (kWide / 2) + lane];
      g0 += gce * __bfloat162float(c2.x);
      g1 += gce * __bfloat162float(c2.y);
    }
  }
}

__global__ void __launch_bounds__(256) k_wide_push(const WidePushArgs p) {
  __shared__ u32 s_off[PSB_MAX_SHARDS + 1];
  __shared__ u32 s_last;
  __shared__ __nv_bfloat162 s_ctx[128 * kWide / 2];   // the context matrix, 16 KB at N = 128
  if (threadIdx.x <= p.S) s_off[threadIdx.x] = p.own_off[threadIdx.x];
  for (int i = threadIdx.x; i < p.N * kWide / 2; i += blockDim.x) s_ctx[i] = reinterpret_cast<const __nv_bfloat162*>(p.ctx)[i];
  __syncthreads();
  const u32 U = *p.n_unique;
  const int lane = threadIdx.x & 31;
  const u32 gwarp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = (gridDim.x * blockDim.x) >> 5;
  auto emit = [&](u32 u, float g0, float g1) {
    int s = owner_of(s_off, p.S, u);
    u32 j = u - s_off[s];
    if (j >= p.inbox_cap) { if (lane == 0) set_status(p.status, kInboxOverflow); return; }
    reinterpret_cast<__nv_bfloat162*>(p.inbox_vals[s] + (size_t)j * kWide)[lane] = __floats2bfloat162_rn(g0, g1);
    if (lane == 0) p.inbox_keys[s][j] = p.ukeys[u];
  };
  // ---- phase 1: one warp per key; long segments are only listed, with the number of their
  // first chunk (one 64-bit atomic hands out list position and chunk numbers together, so the
  // list is sorted by first chunk)
  for (u32 u = gwarp; u < U; u += nwarps) {
    const u32 i0 = p.seg_off[u], i1 = p.seg_off[u + 1];
    if (i1 - i0 > kWideLongSeg && p.long_cap) {
      if (lane == 0) {
        const u32 nch = (i1 - i0 + kWideLongSeg - 1) / kWideLongSeg;
        const unsigned long long old = atomicAdd(p.n_long, 1ull | ((unsigned long long)nch << 32));
        const u32 k = (u32)old;
        if (k < p.long_cap) p.long_list[k] = make_uint4(u, (u32)(old >> 32), i0, i1);
        else set_status(p.status, kInboxOverflow);
      }
      continue;
    }
    float g0 = 0.f, g1 = 0.f;   // lane handles dimensions 2*lane, 2*lane+1
    wide_seg_accumulate(p, s_ctx, i0, i1, lane, g0, g1);
    emit(u, g0, g1);
  }
  if (p.long_cap) {
    if (!grid_barrier(p.bar, p.status)) return;
    // ---- phase 2: all chunks of all long segments, one per warp and trip
    const unsigned long long tot = *((volatile unsigned long long*)p.n_long);
    const u32 n_long = min((u32)tot, p.long_cap);
    const u32 n_chunks = n_long ? (u32)(tot >> 32) : 0u;
    for (u32 c = gwarp; c < n_chunks; c += nwarps) {
      // the entry with the largest first chunk <= c
      u32 lo = 0, hi = n_long;
      while (hi - lo > 1) {
        const u32 mid = (lo + hi) >> 1;
        if (__ldcg(&p.long_list[mid].y) <= c) lo = mid; else hi = mid;
      }
      const uint4 e = __ldcg(&p.long_list[lo]);
      const u32 cc = c - e.y;
      const u32 b0 = e.z + cc * kWideLongSeg;
      if (b0 >= e.w) continue;                       // (only if the list overflowed)
      float g0 = 0.f, g1 = 0.f;
      wide_seg_accumulate(p, s_ctx, b0, min(e.w, b0 + kWideLongSeg), lane, g0, g1);
      atomicAdd(&p.long_acc[(size_t)lo * kWide + 2 * lane], g0);
      atomicAdd(&p.long_acc[(size_t)lo * kWide + 2 * lane + 1], g1);
    }
    if (!grid_barrier(p.bar, p.status)) return;
    // ---- phase 3: emit the long keys and leave the scratch zeroed
    for (u32 k = gwarp; k < n_long; k += nwarps) {
      float2* a = reinterpret_cast<float2*>(p.long_acc + (size_t)k * kWide) + lane;
      float2 g = __ldcg(a);
      *a = make_float2(0.f, 0.f);
      emit(__ldcg(&p.long_list[k].x), g.x, g.y);
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(p.done, 1u) + 1 == gridDim.x;
  __syncthreads();
  if (s_last && threadIdx.x == 0 && p.n_long) *p.n_long = 0ull;
  if (s_last && threadIdx.x < p.S) {
    int s = threadIdx.x;
    __threadfence_system();
    *p.count[s] = min(s_off[s + 1] - s_off[s], p.inbox_cap);
    __threadfence_system();
    st_release_sys(p.ready[s], p.ts1);
    if (s == 0) atomicExch(p.done, 0u);
  }
}

// ---------------------------------------------------------------- apply: AdaGrad per source, in rank order
struct WideApplyArgs {
  int S;
  uint32_t ts1, inbox_cap;
  psb_u64* keys;
  __nv_bfloat16* vals;
  float* acc;
  psb_u64 mask, key_begin, slot_mult;
  const psb_u64* inbox_keys[PSB_MAX_SHARDS];
  const __nv_bfloat16* inbox_vals[PSB_MAX_SHARDS];
  const uint32_t* ready[PSB_MAX_SHARDS];
  const uint32_t* count[PSB_MAX_SHARDS];
  uint8_t alive[PSB_MAX_SHARDS];
  float alpha, beta;
  uint32_t wait_iters;
  uint32_t* applied;
  uint32_t* bar;
  uint32_t* done;
  uint32_t* status;
};

__global__ void __launch_bounds__(256) k_wide_apply(const WideApplyArgs p) {
  __shared__ u32 s_cnt[PSB_MAX_SHARDS];
  __shared__ u32 s_last;
  if (threadIdx.x == 0) {
    const u32 iters = p.wait_iters ? p.wait_iters : kPeerWaitIters;
    for (int r = 0; r < p.S; ++r) {
      s_cnt[r] = 0;
      if (!p.alive[r]) continue;
      if (!wait_flag_ge_sys(p.ready[r], p.ts1, iters)) { set_status(p.status, kWaitTimeout); continue; }
      s_cnt[r] = min(*((volatile const u32*)p.count[r]), p.inbox_cap);
    }
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const u32 gwarp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = (gridDim.x * blockDim.x) >> 5;
  const SlotMap sm{p.mask, p.key_begin, p.slot_mult};
  int applied_sources = 0;
  for (int r = 0; r < p.S; ++r) {
    if (!p.alive[r]) continue;
    // a key pushed by two sources is updated twice, once per source: keep the passes apart
    if (applied_sources++ > 0) { if (!grid_barrier(p.bar, p.status)) return; }
    for (u32 j = gwarp; j < s_cnt[r]; j += nwarps) {
      long long slot = 0;
      if (lane == 0) slot = wide_find<true>((u64*)p.keys, sm, p.inbox_keys[r][j]);
      slot = __shfl_sync(0xffffffffu, slot, 0);
      if (slot < 0) { if (lane == 0) set_status(p.status, kTableFull); continue; }
      __nv_bfloat162 g2 = reinterpret_cast<const __nv_bfloat162*>(p.inbox_vals[r] + (size_t)j * kWide)[lane];
      float g0 = __bfloat162float(g2.x), g1 = __bfloat162float(g2.y);
      float2* ap = reinterpret_cast<float2*>(p.acc + (size_t)slot * kWide) + lane;
      __nv_bfloat162* wp = reinterpret_cast<__nv_bfloat162*>(p.vals + (size_t)slot * kWide) + lane;
      float2 a = *ap;
      __nv_bfloat162 w2 = *wp;
      a.x += g0 * g0; a.y += g1 * g1;
      float w0 = __bfloat162float(w2.x) - p.alpha / (sqrtf(a.x) + p.beta) * g0;
      float w1 = __bfloat162float(w2.y) - p.alpha / (sqrtf(a.y) + p.beta) * g1;
      *ap = a;
      *wp = __floats2bfloat162_rn(w0, w1);
    }
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(p.done, 1u) + 1 == gridDim.x;
  __syncthreads();
  if (s_last && threadIdx.x == 0) {
    __threadfence_system();
    st_release_sys(p.applied, p.ts1);
    atomicExch(p.done, 0u);
  }
}

__global__ void k_wide_init(u64* keys, __nv_bfloat16* vals, float* acc, u64 cap, u64 seed, float scale) {
  for (u64 i = blockIdx.x * (u64)blockDim.x + threadIdx.x; i < cap * kWide; i += (u64)gridDim.x * blockDim.x) {
    if (i < cap) keys[i] = kEmptyKey;
    vals[i] = __float2bfloat16(0.f);
    acc[i] = 0.f;
  }
  (void)seed; (void)scale;
}

// bulk load of (key, 64 values) rows: table initialisation / checkpoint restore
__global__ void k_wide_load(u64* keys, __nv_bfloat16* vals, SlotMap sm, const u64* in_keys, const __nv_bfloat16* in_vals,
                            u32 n, u32* status) {
  const int lane = threadIdx.x & 31;
  const u32 gwarp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = (gridDim.x * blockDim.x) >> 5;
  for (u32 i = gwarp; i < n; i += nwarps) {
    long long slot = 0;
    if (lane == 0) slot = wide_find<true>(keys, sm, in_keys[i]);
    slot = __shfl_sync(0xffffffffu, slot, 0);
    if (slot < 0) { if (lane == 0) set_status(status, kTableFull); continue; }
    reinterpret_cast<__nv_bfloat162*>(vals + (size_t)slot * kWide)[lane] =
        reinterpret_cast<const __nv_bfloat162*>(in_vals + (size_t)i * kWide)[lane];
  }
}

}  // namespace psb
using namespace psb;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) fn = (EncodeTiledFn)p;
  }
  return fn;
}

extern "C" int psb_wide_init(psb_u64* keys, void* vals, float* acc, psb_u64 cap, cudaStream_t stream) {
  k_wide_init<<<psb_device_sm_count() * 8, 256, 0, stream>>>((u64*)keys, (__nv_bfloat16*)vals, acc, cap, 0, 0.f);
  return -(int)cudaGetLastError();
}
extern "C" int psb_wide_load(psb_u64* keys, void* vals, psb_u64 mask, psb_u64 key_begin, psb_u64 slot_mult,
                             const psb_u64* in_keys, const void* in_vals, uint32_t n, uint32_t* status,
                             cudaStream_t stream) {
  if (n == 0) return 0;
  k_wide_load<<<psb_device_sm_count() * 4, 256, 0, stream>>>((u64*)keys, (__nv_bfloat16*)vals, SlotMap{mask, key_begin, slot_mult},
                                           (const u64*)in_keys, (const __nv_bfloat16*)in_vals, n, status);
  return -(int)cudaGetLastError();
}

// args: a WidePullArgs block (see psb_wide_args_size); ctx: [N x 64] bf16, 16-byte aligned, local memory
extern "C" int psb_wide_pull_gemm(const void* args, const void* ctx, uint32_t max_unique, cudaStream_t stream) {
  WidePullArgs a = *reinterpret_cast<const WidePullArgs*>(args);
  if (a.N != 64 && a.N != 128) return -(int)cudaErrorInvalidValue;
  if (a.S < 1 || a.S > PSB_MAX_SHARDS) return -(int)cudaErrorInvalidValue;
  EncodeTiledFn enc = encode_tiled();
  if (!enc) return -(int)cudaErrorNotSupported;
  CUtensorMap map;
  cuuint64_t dims[2] = {(cuuint64_t)kWide, (cuuint64_t)a.N};
  cuuint64_t strides[1] = {(cuuint64_t)kWide * 2};
  cuuint32_t box[2] = {(cuuint32_t)kWide, (cuuint32_t)a.N};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ctx), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -(int)cudaErrorInvalidValue;
  if (a.margin == nullptr && a.P == nullptr) return -(int)cudaErrorInvalidValue;
  size_t smem = (size_t)kTileM * 128 + (size_t)a.N * 128 + 1024 + (a.margin ? (size_t)kTileM * (a.N + 1) * 4 : 0);
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute((const void*)k_wide_pull_gemm, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024);
    attr_set = true;
  }
  int tiles = (int)((max_unique + kTileM - 1) / kTileM);
  const int grid_max = psb_device_sm_count() * 3;
  int grid = tiles < 1 ? 1 : (tiles > grid_max ? grid_max : tiles);
  k_wide_pull_gemm<<<grid, 128, smem, stream>>>(map, a);
  return -(int)cudaGetLastError();
}

// args: a WideXArgs block; ctx as above. Cooperative launch: the roles wait on one another.
extern "C" int psb_wide_pull_xgemm(const void* args, const void* ctx, uint32_t max_unique, cudaStream_t stream) {
  WideXArgs a = *reinterpret_cast<const WideXArgs*>(args);
  if (a.N != 64 && a.N != 128) return -(int)cudaErrorInvalidValue;
  if (a.S < 1 || a.S > PSB_MAX_SHARDS) return -(int)cudaErrorInvalidValue;
  EncodeTiledFn enc = encode_tiled();
  if (!enc) return -(int)cudaErrorNotSupported;
  CUtensorMap map;
  cuuint64_t dims[2] = {(cuuint64_t)kWide, (cuuint64_t)a.N};
  cuuint64_t strides[1] = {(cuuint64_t)kWide * 2};
  cuuint32_t box[2] = {(cuuint32_t)kWide, (cuuint32_t)a.N};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ctx), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -(int)cudaErrorInvalidValue;
  if ((a.phases & 4) && a.margin == nullptr && a.P == nullptr) return -(int)cudaErrorInvalidValue;
  size_t smem = (size_t)kTileM * 128 + (size_t)a.N * 128 + 1024 + (a.margin ? (size_t)kTileM * (a.N + 1) * 4 : 0);
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute((const void*)k_wide_pull_xgemm, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024);
    // several CTAs per SM must be resident at once: ask for the large shared-memory carve-out
    cudaFuncSetAttribute((const void*)k_wide_pull_xgemm, cudaFuncAttributePreferredSharedMemoryCarveout,
                         cudaSharedmemCarveoutMaxShared);
    attr_set = true;
  }
  // all CTAs must be co-resident: three per SM (each holds N <= 128 of the SM's 512 TMEM columns)
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  (void)max_unique;
  int per = 0;
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per, (const void*)k_wide_pull_xgemm, 128, smem);
  per = per < 1 ? 1 : (per > 3 ? 3 : per);
  void* params[] = {&map, &a};
  return -(int)cudaLaunchCooperativeKernel((const void*)k_wide_pull_xgemm, dim3(sms * per), dim3(128), params, smem, stream);
}

extern "C" int psb_wide_rowsum(const float* P, int N, const uint32_t* row_ptr, uint32_t n_rows, uint32_t fixed_z,
                               const uint32_t* csr_col, const uint32_t* row_ctx, const float* y, float* gcoef,
                               float* margin, double* stats, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  k_wide_rowsum<<<psb_device_sm_count() * 4, 256, 0, stream>>>(P, N, row_ptr, n_rows, fixed_z, csr_col, row_ctx, y, gcoef, margin, stats);
  return -(int)cudaGetLastError();
}
// After a fused pull: add the listed long segments into the margins, then loss and d loss / d margin per row.
extern "C" int psb_wide_rowloss(float* margin, const float* y, uint32_t n_rows, float* gcoef, double* stats,
                                unsigned long long* plong_n, const void* plong_list, const float* plong_rows,
                                uint32_t plong_cap, int N, const uint32_t* csc_row, const uint32_t* row_ctx,
                                cudaStream_t stream) {
  if (plong_n != nullptr && plong_cap > 0)
    k_wide_long_margins<<<psb_device_sm_count() * 4, 256, 0, stream>>>(plong_n, (const uint4*)plong_list, plong_rows, plong_cap,
                                                                       N, csc_row, row_ctx, margin);
  const int blocks = (int)((n_rows + 255) / 256);
  k_wide_rowloss<<<blocks < 1 ? 1 : (blocks > 1024 ? 1024 : blocks), 256, 0, stream>>>(margin, y, n_rows, gcoef, stats, plong_n);
  return -(int)cudaGetLastError();
}
extern "C" int psb_wide_push(const void* args, cudaStream_t stream) {
  WidePushArgs a = *reinterpret_cast<const WidePushArgs*>(args);
  if (a.S < 1 || a.S > PSB_MAX_SHARDS) return -(int)cudaErrorInvalidValue;
  // cooperative: the phases of the long-segment path are separated by grid barriers
  static int grid = 0;
  if (!grid) {
    int dev = 0, sms = 0, per = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per, (const void*)k_wide_push, 256, 0);
    grid = sms * (per < 1 ? 1 : (per > 4 ? 4 : per));
  }
  void* params[] = {&a};
  return -(int)cudaLaunchCooperativeKernel((const void*)k_wide_push, dim3(grid), dim3(256), params, 0, stream);
}
extern "C" int psb_wide_apply(const void* args, cudaStream_t stream) {
  WideApplyArgs a = *reinterpret_cast<const WideApplyArgs*>(args);
  if (a.S < 1 || a.S > PSB_MAX_SHARDS) return -(int)cudaErrorInvalidValue;
  static int grid = 0;
  if (!grid) {
    int dev = 0, sms = 0, per = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per, (const void*)k_wide_apply, 256, 0);
    grid = sms * (per < 1 ? 1 : (per > 4 ? 4 : per));
  }
  void* params[] = {&a};
  return -(int)cudaLaunchCooperativeKernel((const void*)k_wide_apply, dim3(grid), dim3(256), params, 0, stream);
}
extern "C" int psb_wide_args_size(int which) {
  return which == 0 ? (int)sizeof(WidePullArgs) : which == 1 ? (int)sizeof(WidePushArgs)
       : which == 2 ? (int)sizeof(WideApplyArgs) : (int)sizeof(WideXArgs);
}
