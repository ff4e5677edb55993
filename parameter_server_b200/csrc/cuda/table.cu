// Server-shard table and the three fused push/pull kernels for scalar values.
//
//   k_pull_margin  (F2)  worker: gather w for each unique key straight out of
//                        the owning shard's table through (peer) pointers,
//                        then X.w margins, loss, d loss/d margin and metrics.
//                        Replaces KVMap::GetValue (parameter/kv_map.h:69-77),
//                        the pull round trip (parameter/parameter.cc:5-49) and
//                        the worker SpMV + loss (app/linear_method/
//                        async_sgd.h:264-296, loss.h:81-93).
//   k_push         (F1a) worker: X^T g as a segmented reduction over the CSC
//                        order the sort produced, range partition, optional
//                        block-scaled quantisation (fixed-point filter), peer
//                        stores into the owners' inboxes, release flags.
//                        Replaces loss.h:91-92, SliceKOFVMessage
//                        (system/message.h:107-147) and the Van send path.
//   k_apply        (F1b) server: bounded wait on the sources' flags, duplicate
//                        key reduce across sources, one optimiser step per
//                        touched key (FTRLEntry::Set / AdaGradEntry::Set,
//                        app/linear_method/async_sgd.h:132-176), progress
//                        stats (SGDState::UpdateWeight, :104-114).
//
// All three are persistent kernels launched cooperatively (one wave, grid
// barrier between phases). Nothing here uses TMA or cluster multicast: remote
// data moves with plain loads/stores through peer-mapped pointers.
#include <cuda_fp16.h>
#include "psb_common.cuh"
#include "psb_cuda.h"

namespace psb {

static constexpr int kThreads = 256;
static constexpr int kMergeHashBits = 11;               // k_apply's per-part merge table: 2048 slots, half full at most
static constexpr int kMergeHash = 1 << kMergeHashBits;

// Optional per-phase cycle stamps (thread 0 of every CTA, 16 slots per CTA) for tuning builds.
#ifdef PSB_TRACE
__device__ long long* g_trace = nullptr;
#define PSB_TSTAMP(k) do { if (threadIdx.x == 0 && g_trace) g_trace[(size_t)blockIdx.x * 16 + (k)] = clock64(); } while (0)
#else
#define PSB_TSTAMP(k) do { } while (0)
#endif
static constexpr u32 kMaxProbe = 1u << 16;

// ------------------------------------------------------------------ optimiser
__device__ __forceinline__ float lr_eval(const PsbOptimizer& o, float x) {
  return o.lr_type == PSB_LR_CONSTANT ? o.alpha : o.alpha / (x + o.beta);
}
__device__ __forceinline__ float prox(const PsbOptimizer& o, float z, float eta) {
  float leta = o.l1 * eta;
  if (z <= leta && z >= -leta) return 0.f;
  return z > 0 ? (z - leta) / (1.f + o.l2 * eta) : (z + leta) / (1.f + o.l2 * eta);
}

// One optimiser step on (w, s0, s1) with gradient g; returns the new weight.
__device__ __forceinline__ float opt_step(const PsbOptimizer& o, float g, float& w, float& s0,
                                          float& s1) {
  if (o.algo == PSB_ALGO_FTRL) {
    // s0 = z, s1 = sqrt(n)
    float sn = sqrtf(s1 * s1 + g * g);
    float sigma = (sn - s1) / o.alpha;
    s0 += g - sigma * w;
    s1 = sn;
    float eta = lr_eval(o, sn);
    w = prox(o, -s0 * eta, eta);
  } else if (o.algo == PSB_ALGO_ADAGRAD) {
    s0 += g * g;  // sum of squared gradients
    float eta = lr_eval(o, sqrtf(s0));
    w = prox(o, w - eta * g, eta);
  } else if (o.algo == PSB_ALGO_SGD) {
    s0 += 1.f;    // number of updates of this key
    float eta = lr_eval(o, sqrtf(s0));
    w = prox(o, w - eta * g, eta);
  } else if (o.algo == PSB_ALGO_SUM) {   // plain accumulate (KVVector PLUS / custom "+=" entries)
    w += g;
  }                                       // PSB_ALGO_KEEP: the stored value stays
  return w;
}

struct StatAcc {
  double d_nnz = 0, w2 = 0, dw2 = 0, n = 0;
  __device__ __forceinline__ void add(float w_new, float w_old) {
    if (w_new == 0.f && w_old != 0.f) d_nnz -= 1;
    else if (w_new != 0.f && w_old == 0.f) d_nnz += 1;
    w2 += (double)w_new * w_new;
    double d = (double)w_new - w_old;
    dw2 += d * d;
    n += 1;
  }
};

__device__ __forceinline__ void block_add4(double a, double b, double c, double d, double* out) {
  __shared__ double s_acc[4];
  if (threadIdx.x < 4) s_acc[threadIdx.x] = 0;
  __syncthreads();
  a = warp_sum_d(a); b = warp_sum_d(b); c = warp_sum_d(c); d = warp_sum_d(d);
  if ((threadIdx.x & 31) == 0) {
    atomicAdd(&s_acc[0], a); atomicAdd(&s_acc[1], b);
    atomicAdd(&s_acc[2], c); atomicAdd(&s_acc[3], d);
  }
  __syncthreads();
  if (threadIdx.x < 4 && out && s_acc[threadIdx.x] != 0) atomicAdd(&out[threadIdx.x], s_acc[threadIdx.x]);
}

// ------------------------------------------------------------------ table init / io
__global__ void k_table_init(Entry* tab, u64 cap) {
  for (u64 i = blockIdx.x * (u64)blockDim.x + threadIdx.x; i < cap; i += (u64)gridDim.x * blockDim.x) {
    uint4* p = reinterpret_cast<uint4*>(&tab[i]);
    p[0] = make_uint4(0xFFFFFFFFu, 0xFFFFFFFFu, 0u, 0u);
    p[1] = make_uint4(0u, 0u, 0u, 0u);
  }
}

template <bool kAll>
__global__ void k_table_dump(const Entry* tab, u64 cap, u64* out_keys, float* out_s0, float* out_s1,
                             float* out_w, u64 out_cap, unsigned long long* out_n) {
  const int lane = threadIdx.x & 31;
  for (u64 base = (blockIdx.x * (u64)blockDim.x + threadIdx.x) - lane; base < cap;
       base += (u64)gridDim.x * blockDim.x) {
    u64 i = base + lane;
    bool take = false;
    Entry e;
    if (i < cap) {
      e = tab[i];
      take = e.key != kEmptyKey && (kAll || (e.w != 0.f && e.w == e.w));
    }
    u32 m = __ballot_sync(0xffffffffu, take);
    if (m == 0) continue;
    unsigned long long at = 0;
    if (lane == 0) at = atomicAdd(out_n, (unsigned long long)__popc(m));
    at = __shfl_sync(0xffffffffu, at, 0);
    if (take) {
      u64 o = at + __popc(m & ((1u << lane) - 1));
      if (o < out_cap) {
        out_keys[o] = e.key;
        out_w[o] = e.w;
        if (kAll) { out_s0[o] = e.s0; out_s1[o] = e.s1; }
      }
    }
  }
}

__global__ void k_table_load(Entry* tab, SlotMap sm, const u64* keys, const float* s0, const float* s1,
                             const float* w, u64 n, u32* status) {
  for (u64 i = blockIdx.x * (u64)blockDim.x + threadIdx.x; i < n; i += (u64)gridDim.x * blockDim.x) {
    long long slot = table_find<true>(tab, sm, keys[i], kMaxProbe);
    if (slot < 0) { set_status(status, kTableFull); continue; }
    tab[slot].w = w ? w[i] : 0.f;
    tab[slot].s0 = s0 ? s0[i] : 0.f;
    tab[slot].s1 = s1 ? s1[i] : 0.f;
  }
}

// ------------------------------------------------------------------ F2: pull + margins
__global__ void __launch_bounds__(kThreads) k_pull_margin(const PsbPullParams p) {
  __shared__ u32 s_off[PSB_MAX_SHARDS + 1];
  const int S = p.S;
  const u32 U = *p.n_unique;
  if (threadIdx.x <= S) s_off[threadIdx.x] = p.own_off[threadIdx.x];
  if (threadIdx.x == 0 && p.need_applied > 0) {
    for (int s = 0; s < S; ++s)
      if (!wait_flag_ge_sys(p.applied[s], p.need_applied, kPeerWaitIters))
        set_status(p.status, kWaitTimeout);
  }
  __syncthreads();
  const u32 gsize = gridDim.x * blockDim.x;
  const u32 gtid = blockIdx.x * blockDim.x + threadIdx.x;
  // phase 1: gather one weight per unique key from its owner's table
  // (insert == 2: w_local was filled by someone else, e.g. a collective; only clear grad)
  if (p.insert == 2) {
    if (p.grad_zero) for (u32 u = gtid; u < U; u += gsize) p.grad_zero[u] = 0.f;
  } else {
  const bool reuse = p.key_hit && p.slot_local && *p.key_hit;
  for (u32 u = gtid; u < U; u += gsize) {
    int s = owner_of(s_off, S, u);
    u64 key = p.ukeys[u];
    float w;
    long long slot;
    const SlotMap sm{p.mask[s], p.key_begin[s], p.slot_mult[s]};
    if (reuse && p.slot_local[u] >= 0) {
      // key-cache hit: the slot found last time is still this key's slot
      slot = p.slot_local[u];
      asm volatile("ld.relaxed.sys.global.f32 %0, [%1];"
                   : "=f"(w) : "l"(&((Entry*)p.table[s])[slot].w) : "memory");
    } else if (p.insert == 1) {
      slot = table_find<true>((Entry*)p.table[s], sm, key, kMaxProbe);
      w = 0.f;
      if (slot >= 0) {
        asm volatile("ld.relaxed.sys.global.f32 %0, [%1];"
                     : "=f"(w) : "l"(&((Entry*)p.table[s])[slot].w) : "memory");
      } else {
        set_status(p.status, kTableFull);
      }
    } else {
      slot = table_lookup_w((const Entry*)p.table[s], sm, key, kMaxProbe, &w);
    }
    p.w_local[u] = w;
    if (p.slot_local) p.slot_local[u] = (int32_t)slot;
    if (p.grad_zero) p.grad_zero[u] = 0.f;
  }
  }
  if (p.n_rows == 0) return;
  if (!grid_barrier(p.bar, p.status)) return;
  // phase 2: one warp per row
  const int lane = threadIdx.x & 31;
  const u32 gwarp = gtid >> 5, nwarps = gsize >> 5;
  double loss_sum = 0, n_correct = 0, n_seen = 0;
  for (u32 r = gwarp; r < p.n_rows; r += nwarps) {
    u32 b, e;
    if (p.row_ptr) { b = p.row_ptr[r]; e = p.row_ptr[r + 1]; }
    else { b = r * p.fixed_z; e = b + p.fixed_z; }
    float acc = 0.f;
    for (u32 j = b + lane; j < e; j += 32) {
      float w = __ldcg(&p.w_local[p.csr_col[j]]);
      acc += p.csr_val ? w * p.csr_val[j] : w;
    }
    acc = warp_sum(acc);
    if (lane == 0) {
      float y = p.y[r];
      float ym = y * acc;
      float g, l;
      if (p.loss == PSB_LOSS_LOGIT) {
        // tau = 1/(1+exp(y m)); loss = log(1+exp(-y m)), both evaluated stably
        float en = expf(-fabsf(ym));
        float tau = ym > 0 ? en / (1.f + en) : 1.f / (1.f + en);
        g = -y * tau;
        l = log1pf(en) + fmaxf(-ym, 0.f);
      } else {
        float h = fmaxf(1.f - ym, 0.f);
        g = -2.f * y * h;
        l = h * h;
      }
      p.gcoef[r] = g;
      if (p.margin) p.margin[r] = acc;
      loss_sum += l;
      n_correct += (ym > 0.f) ? 1.0 : 0.0;
      n_seen += 1.0;
      if (p.auc_hist) {
        float pr = 1.f / (1.f + expf(-acc));
        int bin = min(4095, max(0, (int)(pr * 4096.f)));
        atomicAdd(&p.auc_hist[(y > 0 ? 4096 : 0) + bin], 1u);
      }
    }
  }
  block_add4(loss_sum, n_correct, n_seen, 0.0, p.stats);
}

// ------------------------------------------------------------------ F2 (exchange form)
__global__ void __launch_bounds__(kThreads) k_pull_exchange(const PsbPullExchangeParams p) {
  __shared__ u32 s_off[PSB_MAX_SHARDS + 1];
  __shared__ u32 s_last;
  __shared__ u32 s_n, s_base;
  __shared__ u32 s_wslot[kThreads];                // slots of a tile of the k-wide owner path
  const int S = p.S;
  const u32 U = *p.n_unique;
  const u32 iters = p.wait_iters ? p.wait_iters : kPeerWaitIters;
  if (threadIdx.x <= S) s_off[threadIdx.x] = p.own_off[threadIdx.x];
  __syncthreads();
  const u32 gsize = gridDim.x * blockDim.x;
  const u32 gtid = blockIdx.x * blockDim.x + threadIdx.x;
  PSB_TSTAMP(0);
  // ---- (a) my keys to their owners
  if (p.phases & 1) {
  bool key_hit = false;
  if (p.key_cache) {
    // Key caching: fingerprint of the whole list (every key mixed with its position), summed over the
    // grid; all CTAs then take the same decision. The two accumulators alternate by round parity.
    const u32 par = (p.ts1 - 1) & 1u;
    unsigned long long fp = 0;
    for (u32 u = gtid; u < U; u += gsize) fp += fmix64(p.ukeys[u] ^ ((u64)u * 0x9E3779B97F4A7C15ull));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) fp += __shfl_xor_sync(0xffffffffu, fp, o);
    if ((threadIdx.x & 31) == 0 && fp) atomicAdd(&p.kc_state[2 * par], fp);
    if (gtid == 0) p.kc_state[2 * par + 1] = (u64)U + 1;
    __threadfence();
    if (!grid_barrier(p.bar, p.status)) return;
    const u64 cur = __ldcg(&p.kc_state[2 * par]), prev = __ldcg(&p.kc_state[2 * (par ^ 1)]);
    key_hit = p.ts1 > 1 && cur == prev && __ldcg(&p.kc_state[2 * (par ^ 1) + 1]) == (u64)U + 1;
  }
  // four independent keys per thread and trip, loads first
  // Every CTA takes the owners in its own order (CTA b starts with owner b mod S), each owner's part of the
  // key list divided over the whole grid: at any moment the grid's peer stores are spread over all owners
  // instead of all GPUs writing into the same one.
  for (int kk = 0; kk < S; ++kk) {
    const int s = (int)((blockIdx.x + (u32)kk) % (u32)S);
    const u32 b0 = s_off[s], cnt = s_off[s + 1] - b0;
    for (u32 j0 = gtid; j0 < cnt; j0 += 4 * gsize) {
      u64 k[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const u32 j = j0 + q * gsize;
        k[q] = j < cnt ? p.ukeys[b0 + j] : 0;
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const u32 j = j0 + q * gsize;
        if (j >= cnt) break;
        if (j < p.req_cap && !key_hit) p.req_keys[s][j] = k[q];
        if (p.grad_zero) p.grad_zero[b0 + j] = 0.f;
      }
    }
  }
  PSB_TSTAMP(1);
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(&p.done[0], 1u) + 1 == gridDim.x;
  __syncthreads();
  if (s_last && threadIdx.x < S) {
    int s = threadIdx.x;
    u32 c = s_off[s + 1] - s_off[s];
    if (c > p.req_cap) { set_status(p.status, kInboxOverflow); c = p.req_cap; }
    __threadfence_system();
    p.req_hdr[s][0] = c | (key_hit ? 0x80000000u : 0u);     // top bit: no keys, answer from the remembered slots
    p.req_hdr[s][1] = s_off[s];
    __threadfence_system();
    st_release_sys(p.req_ready[s], p.ts1);
    if (s == 0) {
      atomicExch(&p.done[0], 0u);
      // every CTA has read the other parity's fingerprint by now: clear it for the next round
      if (p.key_cache) p.kc_state[2 * (((p.ts1 - 1) & 1u) ^ 1)] = 0;
    }
  }
  }
  PSB_TSTAMP(2);
  // ---- (b) owner role: serve every source
  if (p.phases & 2) {
  if (threadIdx.x == 0 && p.need_applied > 0 && !wait_flag_ge_sys(p.applied, p.need_applied, iters))
    set_status(p.status, kWaitTimeout);
  Entry* tab = (Entry*)p.table;
  const SlotMap sm{p.mask, p.key_begin, p.slot_mult};
  for (int kk = 0; kk < S; ++kk) {
    const int r = (int)((blockIdx.x + (u32)kk) % (u32)S);   // sources in a per-CTA order: no source gets all answers at once
    if (!p.alive[r]) continue;
    __syncthreads();
    if (threadIdx.x == 0) {
      u32 n = 0, base = 0;
      if (wait_flag_ge_sys(p.my_req_ready[r], p.ts1, iters)) {
        n = *((volatile const u32*)&p.my_req_hdr[r][0]);
        base = *((volatile const u32*)&p.my_req_hdr[r][1]);
      } else {
        set_status(p.status, kWaitTimeout);
      }
      s_n = min(n & 0x7fffffffu, p.req_cap) | (n & 0x80000000u);
      s_base = base;
    }
    __syncthreads();
    PSB_TSTAMP(3);
    const u32 n = s_n & 0x7fffffffu, base = s_base;
    const int kw = p.width > 1 ? p.width : 1;
    if (p.tile_off != nullptr && S > 1) {
      // for the merge in k_apply: where each equal part of my key range starts in this source's list
      const u32 T = (u32)p.tiles;
      u32* to = p.tile_off + (size_t)r * (T + 1);
      if (s_n & 0x80000000u) {
        const u32* tp = p.tile_off_prev + (size_t)r * (T + 1);
        for (u32 k = gtid; k <= T; k += gsize) to[k] = tp[k];
      } else {
        const u64 range = p.key_end - p.key_begin;          // key_end 0 stands for 2^64
        const int sh = 64 - (31 - __clz(T));
        for (u32 k = gtid; k <= T; k += gsize) {
          u32 lo = 0, hi = n;
          if (k == T) lo = n;
          else if (k > 0) {
            const u64 bound = p.key_begin + __umul64hi(range, (u64)k << sh);
            while (lo < hi) {
              const u32 mid = (lo + hi) >> 1;
              if (p.my_req_keys[r][mid] < bound) lo = mid + 1; else hi = mid;
            }
          }
          to[k] = lo;
        }
      }
    }
    if (kw > 1) {
      // k values per key. A CTA takes tiles of blockDim.x keys: one thread per key finds the slot
      // (remembered slots on a key-cache hit at the source), then the whole CTA copies the tile's
      // k-wide rows with consecutive threads on consecutive values (16 bytes each when k % 4 == 0),
      // so that the peer stores of a warp form whole lines.
      const bool hit = (s_n & 0x80000000u) != 0;
      for (u32 t0 = blockIdx.x * blockDim.x; t0 < n; t0 += gridDim.x * blockDim.x) {
        const u32 j = t0 + threadIdx.x;
        if (j < n) {
          u32 sc;
          if (hit) {
            sc = p.slot_cache_prev[r][j] & 0x7fffffffu;
          } else {
            const long long sl = table_find<true>(tab, sm, p.my_req_keys[r][j], kMaxProbe);
            sc = sl >= 0 ? (u32)sl : 0x7fffffffu;
            if (sl < 0) set_status(p.status, kTableFull);
          }
          p.slot_cache[r][j] = sc;
          s_wslot[threadIdx.x] = sc;
        }
        __syncthreads();
        const u32 cnt = min((u32)blockDim.x, n - t0);
        float* dst = p.resp_w[r] + (size_t)(base + t0) * kw;
        if ((kw & 3) == 0) {
          const u32 q4 = (u32)kw >> 2;
          for (u32 idx = threadIdx.x; idx < cnt * q4; idx += blockDim.x) {
            const u32 jj = idx / q4, c4 = idx - jj * q4, sc = s_wslot[jj];
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (sc != 0x7fffffffu) v = __ldcg(reinterpret_cast<const float4*>(p.wide_vals + (size_t)sc * kw) + c4);
            reinterpret_cast<float4*>(dst)[idx] = v;
          }
        } else {
          for (u32 idx = threadIdx.x; idx < cnt * (u32)kw; idx += blockDim.x) {
            const u32 jj = idx / (u32)kw, c = idx - jj * (u32)kw, sc = s_wslot[jj];
            dst[idx] = sc != 0x7fffffffu ? __ldcg(&p.wide_vals[(size_t)sc * kw + c]) : 0.f;
          }
        }
        __syncthreads();
      }
      continue;
    }
    if (s_n & 0x80000000u) {
      // key-cache hit at the source: same keys as in the round before, so the same slots
      for (u32 j = gtid; j < n; j += gsize) {
        const u32 sc = p.slot_cache_prev[r][j] & 0x7fffffffu;
        p.slot_cache[r][j] = sc;
        float w = 0.f;
        if (sc != 0x7fffffffu) w = __ldcg(&tab[sc].w);
        p.resp_w[r][base + j] = w;
      }
      continue;
    }
    // Four keys per thread and trip. The first probe of each is one 16-byte load
    // that returns key and weight, issued for all four before any is examined;
    // only a miss on that slot (collision or new key) takes the probing path.
    for (u32 j0 = gtid; j0 < n; j0 += 4 * gsize) {
      u64 key[4], slot[4], k0[4], hi[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        u32 j = j0 + q * gsize;
        key[q] = j < n ? p.my_req_keys[r][j] : 0;
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        u32 j = j0 + q * gsize;
        slot[q] = first_slot(sm, key[q]);
        k0[q] = kEmptyKey; hi[q] = 0;
        if (j < n)
          asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];"
                       : "=l"(k0[q]), "=l"(hi[q]) : "l"(&tab[slot[q]]) : "memory");
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        u32 j = j0 + q * gsize;
        if (j >= n) break;
        float w = __uint_as_float((u32)hi[q]);
        u32 sc = (u32)slot[q];
        if (k0[q] != key[q]) {
          long long sl = table_find<true>(tab, sm, key[q], kMaxProbe);
          w = 0.f;
          sc = 0x7fffffffu;
          if (sl >= 0) { w = __ldcg(&tab[sl].w); sc = (u32)sl; }
          else set_status(p.status, kTableFull);
        }
        p.slot_cache[r][j] = sc;
        p.resp_w[r][base + j] = w;
      }
    }
  }
  PSB_TSTAMP(4);
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(&p.done[1], 1u) + 1 == gridDim.x;
  __syncthreads();
  if (s_last && threadIdx.x < S && p.alive[threadIdx.x]) {
    __threadfence_system();
    st_release_sys(p.resp_ready[threadIdx.x], p.ts1);
  }
  if (s_last && threadIdx.x == 0) atomicExch(&p.done[1], 0u);
  }
  if (!(p.phases & 4)) return;
  // ---- (c) worker: all owners have answered -> margins (none when n_rows == 0: the
  // caller then reads the weights from the response buffer after this kernel)
  PSB_TSTAMP(5);
  __syncthreads();
  if (threadIdx.x < S) {                           // one lane per owner: the polls run side by side
    const int s = threadIdx.x;
    if (p.alive[s] && !wait_flag_ge_sys(p.my_resp_ready[s], p.ts1, iters)) set_status(p.status, kWaitTimeout);
  }
  __syncthreads();
  if (p.n_rows == 0) return;
  PSB_TSTAMP(6);
  const int lane = threadIdx.x & 31;
  const u32 gwarp = gtid >> 5, nwarps = gsize >> 5;
  double loss_sum = 0, n_correct = 0, n_seen = 0;
  for (u32 r = gwarp; r < p.n_rows; r += nwarps) {
    u32 b, e;
    if (p.row_ptr) { b = p.row_ptr[r]; e = p.row_ptr[r + 1]; }
    else { b = r * p.fixed_z; e = b + p.fixed_z; }
    float acc = 0.f;
    // eight column ids per lane are fetched before the first weight is gathered
    for (u32 j0 = b + lane; j0 < e; j0 += 32 * 8) {
      u32 col[8];
      float xv[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        u32 j = j0 + q * 32;
        col[q] = j < e ? __ldcs(&p.csr_col[j]) : 0xffffffffu;   // column ids are streamed
        xv[q] = (p.csr_val && j < e) ? __ldcs(&p.csr_val[j]) : 1.f;
      }
#pragma unroll
      for (int q = 0; q < 8; ++q)
        // Plain (L1-cached) gathers: every weight was written before the flags that this
        // CTA has acquired, and frequent columns repeat within a few rows, so they hit L1.
        if (col[q] != 0xffffffffu) acc += p.my_resp_w[col[q]] * xv[q];
    }
    acc = warp_sum(acc);
    if (lane == 0) {
      float y = p.y[r];
      float ym = y * acc;
      float g, l;
      if (p.loss == PSB_LOSS_LOGIT) {
        float en = expf(-fabsf(ym));
        float tau = ym > 0 ? en / (1.f + en) : 1.f / (1.f + en);
        g = -y * tau;
        l = log1pf(en) + fmaxf(-ym, 0.f);
      } else {
        float h = fmaxf(1.f - ym, 0.f);
        g = -2.f * y * h;
        l = h * h;
      }
      p.gcoef[r] = g;
      if (p.margin) p.margin[r] = acc;
      loss_sum += l;
      n_correct += (ym > 0.f) ? 1.0 : 0.0;
      n_seen += 1.0;
      if (p.auc_hist) {
        float pr = 1.f / (1.f + expf(-acc));
        int bin = min(4095, max(0, (int)(pr * 4096.f)));
        atomicAdd(&p.auc_hist[(y > 0 ? 4096 : 0) + bin], 1u);
      }
    }
  }
  PSB_TSTAMP(7);
  block_add4(loss_sum, n_correct, n_seen, 0.0, p.stats);
  PSB_TSTAMP(8);
}

// ------------------------------------------------------------------ F1a: worker push
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Value region of one inbox, by quantisation mode (cap = records per inbox):
//   NONE : float v[cap]
//   INT8 : float scale[ceil(cap/32)] followed by int8 code[cap]
//   FP16 : float scale[ceil(cap/32)] followed by half  code[cap]
__device__ __forceinline__ u32 scale_words(u32 cap) { return (cap + 31) / 32; }

__global__ void __launch_bounds__(kThreads) k_push(const PsbPushParams p) {
  __shared__ u32 s_off[PSB_MAX_SHARDS + 1];
  __shared__ u32 s_gp[PSB_MAX_SHARDS + 1];  // group prefix per owner
  __shared__ u32 s_last;
  const int S = p.S;
  if (threadIdx.x <= S) s_off[threadIdx.x] = p.own_off[threadIdx.x];
  if (threadIdx.x == 0 && p.need_applied > 0) {
    for (int s = 0; s < S; ++s)
      if (!wait_flag_ge_sys(p.applied[s], p.need_applied, kPeerWaitIters))
        set_status(p.status, kWaitTimeout);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    u32 acc = 0;
    for (int s = 0; s < S; ++s) {
      s_gp[s] = acc;
      u32 c = s_off[s + 1] - s_off[s];
      if (c > p.inbox_cap) { set_status(p.status, kInboxOverflow); c = p.inbox_cap; }
      acc += (c + 31) / 32;
    }
    s_gp[S] = acc;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const u32 gsize = gridDim.x * blockDim.x;
  const u32 gtid = blockIdx.x * blockDim.x + threadIdx.x;
  const u32 gwarp = gtid >> 5, nwarps = gsize >> 5;
  const u32 le = 0xffffffffu >> (31 - lane);
  PSB_TSTAMP(0);

  if (p.nnz > 0) {
    // phase 1: segmented reduction of gcoef[row]*x over the key-sorted nonzeros
    const u32 nwords = (p.nnz + 31) / 32;
    // A warp takes chunks of kChunkWords consecutive 32-element words. Inside a chunk
    // the sum of a segment that runs over a word boundary is carried in a register
    // and added to grad once, so a frequent key (a segment of up to millions of
    // nonzeros) costs one atomic per chunk, not one per word: same-address atomics
    // serialise in L2. Four words are loaded per trip (row ids, then the gathers).
    // chunk length: up to 16 words, but no longer than what keeps every warp busy (small batches)
    const u32 kChunkWords = max(1u, min(16u, (nwords + nwarps - 1) / nwarps));
    const u32 nchunks = (nwords + kChunkWords - 1) / kChunkWords;
    for (u32 c = gwarp; c < nchunks; c += nwarps) {
      const u32 wend = min(nwords, (c + 1) * kChunkWords);
      float carry = 0.f;        // sum so far of the segment that is open at the word boundary
      u32 carry_id = 0;         // its unique-key index
      bool open = false;
      for (u32 w0 = c * kChunkWords; w0 < wend; w0 += 4) {
        u32 f[4], base[4], row[4];
        float x[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          u32 wi = w0 + q, i = wi * 32 + lane;
          bool okw = wi < wend;
          f[q] = okw ? p.flagbits[wi] : 0u;
          base[q] = okw ? p.wordbase[wi] : 0u;
          row[q] = (okw && i < p.nnz) ? __ldcs(&p.csc_row[i]) : 0xffffffffu;
          x[q] = (p.csc_val && okw && i < p.nnz) ? __ldcs(&p.csc_val[i]) : 1.f;
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) x[q] = row[q] != 0xffffffffu ? x[q] * __ldg(&p.gcoef[row[q]]) : 0.f;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const u32 wi = w0 + q, i = wi * 32 + lane;
          if (wi >= wend) break;                    // warp-uniform
          if (open && (f[q] & 1u)) {                // the open segment ended with the previous word
            if (lane == 0) atomicAdd(&p.grad[carry_id], carry);
            open = false; carry = 0.f;
          }
          u32 fle = f[q] & le;
          int start = fle ? 31 - __clz(fle) : 0;
          float xs = x[q];
#pragma unroll
          for (int o = 1; o < 32; o <<= 1) {
            float yv = __shfl_up_sync(0xffffffffu, xs, o);
            if (lane >= start + o) xs += yv;
          }
          if (fle == 0) xs += carry;                // lanes that continue the open segment (carry is 0 otherwise)
          const bool valid = i < p.nnz;
          const bool last_elem = i == p.nnz - 1;
          const bool tail = valid && ((lane == 31) || ((f[q] >> (lane + 1)) & 1u) || last_elem);
          // the word's last segment stays open unless this is the chunk's last word or the data ends here
          const bool keep = (wi + 1 < wend) && ((wi + 1) * 32 < p.nnz);
          const u32 id = base[q] + __popc(fle) - 1;
          if (tail && !(keep && lane == 31)) atomicAdd(&p.grad[id], xs);
          if (keep) {
            carry = __shfl_sync(0xffffffffu, xs, 31);
            carry_id = base[q] + __popc(f[q]) - 1;
            open = true;
          } else {
            open = false; carry = 0.f;
          }
        }
      }
    }
    PSB_TSTAMP(1);
    if (!grid_barrier(p.bar, p.status)) return;
  }
  PSB_TSTAMP(2);

  // phase 2: range partition + (quantise) + peer stores, 32 values per warp step. With value width k
  // an owner's slice is cnt keys and cnt * k values (key-major); the group prefix counts value groups.
  const bool omit_keys = !p.send_keys || (p.key_hit && *p.key_hit);
  const u32 kw = p.width > 1 ? (u32)p.width : 1u;
  if (kw > 1) {
    // group prefix over values instead of keys (recomputed by every CTA's thread 0)
    __syncthreads();
    if (threadIdx.x == 0) {
      u32 acc = 0;
      for (int s = 0; s < S; ++s) {
        s_gp[s] = acc;
        acc += (min(s_off[s + 1] - s_off[s], p.inbox_cap) * kw + 31) / 32;
      }
      s_gp[S] = acc;
    }
    __syncthreads();
    if (!omit_keys)
      for (u32 u = gtid; u < s_off[S]; u += gsize) {
        const int s = owner_of(s_off, S, u);
        const u32 j = u - s_off[s];
        if (j < p.inbox_cap) p.inbox_keys[s][j] = p.ukeys[u];
      }
  }
  // owners in a per-CTA order, each owner's groups divided over the whole grid (see k_pull_exchange)
  for (int kk = 0; kk < S; ++kk) {
  const int s = (int)((blockIdx.x + (u32)kk) % (u32)S);
  const u32 ng = s_gp[s + 1] - s_gp[s];
  for (u32 gi = gwarp; gi < ng; gi += nwarps) {
    const u32 g = s_gp[s] + gi;
    u32 cnt = min(s_off[s + 1] - s_off[s], p.inbox_cap) * kw;       // values of this owner's slice
    u32 j0 = (g - s_gp[s]) * 32, j = j0 + lane;
    bool valid = j < cnt;
    size_t u = (size_t)s_off[s] * kw + j;
    float v = valid ? __ldcg(&p.grad[u]) : 0.f;
    if (kw == 1 && !omit_keys && valid) p.inbox_keys[s][j] = p.ukeys[u];
    const u32 vcap = p.inbox_cap * kw;
    if (p.quant == PSB_QUANT_NONE) {
      if (valid) ((float*)p.inbox_vals[s])[j] = v;
    } else {
      float amax = warp_max(fabsf(v));
      float* scales = (float*)p.inbox_vals[s];
      if (p.quant == PSB_QUANT_INT8) {
        float scale = amax / 127.f;
        int code = amax > 0.f ? __float2int_rn(v / scale) : 0;
        signed char* codes = (signed char*)(scales + scale_words(vcap));
        if (valid) codes[j] = (signed char)max(-127, min(127, code));
        if (lane == 0) scales[j0 >> 5] = scale;
      } else {
        float scale = amax > 0.f ? amax : 1.f;
        __half* codes = (__half*)(scales + scale_words(vcap));
        if (valid) codes[j] = __float2half_rn(v / scale);
        if (lane == 0) scales[j0 >> 5] = scale;
      }
    }
  }
  }
  // signal: all of this CTA's peer stores are ordered before its arrival, the
  // last CTA to arrive publishes counts and the release flags
  PSB_TSTAMP(3);
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    u32 arrived = atomicAdd(p.done, 1u) + 1;
    s_last = (arrived == gridDim.x);
  }
  __syncthreads();
  if (s_last && threadIdx.x < S) {
    int s = threadIdx.x;
    __threadfence_system();
    *p.count[s] = min(s_off[s + 1] - s_off[s], p.inbox_cap);
    if (p.mode[s]) *p.mode[s] = omit_keys ? 1u : 0u;
    __threadfence_system();
    st_release_sys(p.ready[s], p.ts1);
    if (s == 0) atomicExch(p.done, 0u);
  }
  PSB_TSTAMP(4);
}

// ------------------------------------------------------------------ F1b: server apply
__device__ __forceinline__ float inbox_value(const void* vals, int quant, u32 cap, u32 j) {
  if (quant == PSB_QUANT_NONE) return ((const float*)vals)[j];
  const float* scales = (const float*)vals;
  float scale = scales[j >> 5];
  if (quant == PSB_QUANT_INT8)
    return scale * (float)((const signed char*)(scales + scale_words(cap)))[j];
  return scale * __half2float(((const __half*)(scales + scale_words(cap)))[j]);
}

__global__ void __launch_bounds__(kThreads) k_apply(const PsbApplyParams p) {
  __shared__ u32 s_wslot[kThreads], s_wsrc[kThreads], s_wrec[kThreads];   // a tile of the k-wide path
  __shared__ u32 s_pre[PSB_MAX_SHARDS + 1];
  __shared__ u32 s_cached[PSB_MAX_SHARDS];
  __shared__ u32 s_last;
  const int S = p.S;
  Entry* tab = (Entry*)p.table;
  PSB_TSTAMP(0);
  // the sources' flags are polled side by side (lane r of warp 0 waits for source r): a system-scope
  // poll costs about a microsecond even when the flag is already set, and eight in a row add up
  if (threadIdx.x < 32) {
    const int r = threadIdx.x;
    u32 mine = 0;
    if (r < S) {
      s_cached[r] = p.cached[r];
      if (p.alive[r]) {
        const u32 iters = p.wait_iters ? p.wait_iters : kPeerWaitIters;
        if (wait_flag_ge_sys(p.ready[r], p.ts1, iters)) {
          const u32 c = *((volatile const u32*)p.count[r]);
          if (p.mode[r] && *((volatile const u32*)p.mode[r])) s_cached[r] = 1;
          mine = min(c, p.inbox_cap);
        } else {
          set_status(p.status, kWaitTimeout);
        }
      }
    }
    u32 inc = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const u32 v = __shfl_up_sync(0xffffffffu, inc, o);
      if (r >= o) inc += v;
    }
    if (r < S) s_pre[r] = inc - mine;
    if (r == S - 1) s_pre[S] = inc;
  }
  __syncthreads();
  PSB_TSTAMP(1);
  const u32 total = s_pre[S];
  const u32 gsize = gridDim.x * blockDim.x;
  const u32 gtid = blockIdx.x * blockDim.x + threadIdx.x;
  int n_src = 0;
  bool all_cached = true;
  for (int r = 0; r < S; ++r) {
    n_src += p.alive[r] ? 1 : 0;
    if (p.alive[r] && !s_cached[r]) all_cached = false;
  }
  const bool single = n_src <= 1;
  const bool merge = !single && p.tile_off != nullptr && all_cached && p.width <= 1;
  const SlotMap sm{p.mask, p.key_begin, p.slot_mult};
  StatAcc st;

  if (p.width > 1) {
    // k values per key, sum entries: every record adds its k values to wide_vals[slot * k ..]. A CTA
    // takes tiles of blockDim.x records: one thread per record finds the slot, then the CTA adds the
    // tile's values with consecutive threads on consecutive values (coalesced inbox reads; 16 bytes
    // per thread where the inbox holds plain floats and k % 4 == 0). One source: plain
    // read-modify-write (a slot belongs to one record); several: atomic adds.
    const u32 kw = (u32)p.width, vcap = p.inbox_cap * kw;
    for (u32 t0 = blockIdx.x * blockDim.x; t0 < total; t0 += gridDim.x * blockDim.x) {
      const u32 i = t0 + threadIdx.x;
      if (i < total) {
        int r = 0;
        while (r + 1 < S && i >= s_pre[r + 1]) ++r;
        const u32 j = i - s_pre[r];
        u32 sc;
        if (s_cached[r]) {
          sc = p.slot_cache[r][j] & 0x7fffffffu;
        } else {
          const long long sl = table_find<true>(tab, sm, p.inbox_keys[r][j], kMaxProbe);
          sc = sl >= 0 ? (u32)sl : 0x7fffffffu;
          if (sl < 0) set_status(p.status, kTableFull);
        }
        s_wslot[threadIdx.x] = sc;
        s_wsrc[threadIdx.x] = (u32)r;
        s_wrec[threadIdx.x] = j;
        if (sc != 0x7fffffffu) st.n += 1;
      }
      __syncthreads();
      const u32 cnt = min((u32)blockDim.x, total - t0);
      if (p.opt.algo != PSB_ALGO_KEEP) {
        if ((kw & 3) == 0 && p.quant == PSB_QUANT_NONE) {
          const u32 q4 = kw >> 2;
          for (u32 idx = threadIdx.x; idx < cnt * q4; idx += blockDim.x) {
            const u32 jj = idx / q4, c4 = idx - jj * q4, sc = s_wslot[jj];
            if (sc == 0x7fffffffu) continue;
            const float4 g = reinterpret_cast<const float4*>((const float*)p.inbox_vals[s_wsrc[jj]] + (size_t)s_wrec[jj] * kw)[c4];
            float4* dst = reinterpret_cast<float4*>(p.wide_vals + (size_t)sc * kw) + c4;
            if (single) {
              float4 o = *dst;
              o.x += g.x; o.y += g.y; o.z += g.z; o.w += g.w;
              *dst = o;
            } else {
              atomicAdd(dst, g);
            }
          }
        } else {
          for (u32 idx = threadIdx.x; idx < cnt * kw; idx += blockDim.x) {
            const u32 jj = idx / kw, c = idx - jj * kw, sc = s_wslot[jj];
            if (sc == 0x7fffffffu) continue;
            const float g = inbox_value(p.inbox_vals[s_wsrc[jj]], p.quant, vcap, s_wrec[jj] * kw + c);
            float* dst = p.wide_vals + (size_t)sc * kw + c;
            if (single) *dst += g; else atomicAdd(dst, g);
          }
        }
      }
      __syncthreads();
    }
  } else if (merge) {
    // Several sources whose slots are all remembered: one key-range part at a time, the records of all
    // sources are summed per slot in a shared-memory hash table, then every slot gets one optimiser
    // step and one entry write. A part with more records than the table takes goes through the
    // accumulate-then-lead protocol below (phase B then runs for those records only).
    const u32 T = (u32)p.tiles;
    __shared__ u32 s_hslot[kMergeHash];
    __shared__ float s_hacc[kMergeHash];
    __shared__ u32 s_tlo[PSB_MAX_SHARDS], s_tpre[PSB_MAX_SHARDS + 1];
    // The notes divide the key range into T parts; neighbouring parts are taken together so that a
    // step covers about 400 records of this round (a third of what the merge table takes).
    u32 group = 1;
    while (group < T && (u64)total * group < (u64)400 * T) group <<= 1;
    const u32 n_tiles = T / group;
    for (u32 tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
      if (threadIdx.x < 32) {
        const int r = threadIdx.x;
        u32 lo = 0, len = 0;
        if (r < S) {
          const u32 nr = s_pre[r + 1] - s_pre[r];               // 0: dead or empty source
          lo = min(p.tile_off[(size_t)r * (T + 1) + (size_t)tile * group], nr);
          const u32 hi = min(p.tile_off[(size_t)r * (T + 1) + (size_t)(tile + 1) * group], nr);
          len = hi > lo ? hi - lo : 0;
        }
        u32 inc = len;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const u32 v = __shfl_up_sync(0xffffffffu, inc, o);
          if (r >= o) inc += v;
        }
        if (r < S) { s_tlo[r] = lo; s_tpre[r] = inc - len; }
        if (r == S - 1) s_tpre[S] = inc;
      }
      for (u32 h = threadIdx.x; h < kMergeHash; h += blockDim.x) { s_hslot[h] = 0xffffffffu; s_hacc[h] = 0.f; }
      __syncthreads();
      const u32 cnt = s_tpre[S];
      const bool fits = cnt <= kMergeHash / 2;
      if (!fits && threadIdx.x == 0) atomicExch(p.slow, 1u);
      for (u32 i = threadIdx.x; i < cnt; i += blockDim.x) {
        int r = 0;
        while (r + 1 < S && i >= s_tpre[r + 1]) ++r;
        const u32 j = s_tlo[r] + (i - s_tpre[r]);
        const u32 sc = p.slot_cache[r][j] & 0x7fffffffu;
        if (sc == 0x7fffffffu) continue;
        const float g = inbox_value(p.inbox_vals[r], p.quant, p.inbox_cap, j);
        if (fits) {
          u32 h = (sc * 2654435761u) >> (32 - kMergeHashBits);
          for (;;) {
            const u32 old = atomicCAS(&s_hslot[h], 0xffffffffu, sc);
            if (old == 0xffffffffu || old == sc) { atomicAdd(&s_hacc[h], g); break; }
            h = (h + 1) & (kMergeHash - 1);
          }
        } else {
          const float seen = atomic_add_f32x2(&tab[sc].gacc, g, 1.f).y;
          p.slot_cache[r][j] = sc | (seen == 0.f ? 0x80000000u : 0u);
        }
      }
      __syncthreads();
      if (fits) {
        for (u32 h = threadIdx.x; h < kMergeHash; h += blockDim.x) {
          const u32 sc = s_hslot[h];
          if (sc == 0xffffffffu) continue;
          Entry* e = &tab[sc];
          const float2 ws = *reinterpret_cast<const float2*>(&e->w);
          float w = ws.x, s0 = ws.y, t1 = e->s1, w_old = w;
          opt_step(p.opt, s_hacc[h], w, s0, t1);
          *reinterpret_cast<float2*>(&e->w) = make_float2(w, s0);
          e->s1 = t1;
          st.add(w, w_old);
        }
      }
      __syncthreads();
    }
  } else {
  // phase A: locate the slot of every record; single source -> update in place,
  // several sources -> accumulate into gacc and elect one leader per key
  // four records per thread and trip: values and slots first, then the entries
  for (u32 i0 = gtid; i0 < total; i0 += 4 * gsize) {
    long long slot[4];
    float g[4];
    int rr[4];
    u32 jj[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      u32 i = i0 + q * gsize;
      slot[q] = -1;
      g[q] = 0.f; rr[q] = 0; jj[q] = 0;
      if (i >= total) continue;
      int r = 0;
      while (r + 1 < S && i >= s_pre[r + 1]) ++r;
      u32 j = i - s_pre[r];
      rr[q] = r; jj[q] = j;
      g[q] = inbox_value(p.inbox_vals[r], p.quant, p.inbox_cap, j);
      if (s_cached[r]) {
        u32 sc = p.slot_cache[r][j] & 0x7fffffffu;
        if (sc != 0x7fffffffu) slot[q] = sc;
      } else {
        slot[q] = table_find<true>(tab, sm, p.inbox_keys[r][j], kMaxProbe);
        if (slot[q] < 0) { set_status(p.status, kTableFull); if (p.slot_cache[r]) p.slot_cache[r][j] = 0x7fffffffu; }
      }
    }
    if (single) {
      float2 ws[4];
      float s1[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        ws[q] = make_float2(0.f, 0.f); s1[q] = 0.f;
        if (slot[q] >= 0) {
          ws[q] = *reinterpret_cast<const float2*>(&tab[slot[q]].w);   // (w, s0): one 8-byte load
          s1[q] = tab[slot[q]].s1;
        }
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (slot[q] < 0) continue;
        float w = ws[q].x, s0 = ws[q].y, t1 = s1[q], w_old = w;
        opt_step(p.opt, g[q], w, s0, t1);
        Entry* e = &tab[slot[q]];
        *reinterpret_cast<float2*>(&e->w) = make_float2(w, s0);
        e->s1 = t1;
        st.add(w, w_old);
        if (p.slot_cache[rr[q]]) p.slot_cache[rr[q]][jj[q]] = (u32)slot[q];
      }
    } else {
      // one vector atomic per record: gradient into gacc, one into gcnt; the record that finds
      // gcnt == 0 is the key's leader in phase B
      float seen[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        seen[q] = 1.f;
        if (slot[q] >= 0) seen[q] = atomic_add_f32x2(&tab[slot[q]].gacc, g[q], 1.f).y;
      }
#pragma unroll
      for (int q = 0; q < 4; ++q)
        if (slot[q] >= 0) p.slot_cache[rr[q]][jj[q]] = (u32)slot[q] | (seen[q] == 0.f ? 0x80000000u : 0u);
    }
  }
  }
  PSB_TSTAMP(2);
  bool phase_b = !single && p.width <= 1;
  if (merge) {
    if (!grid_barrier(p.bar, p.status)) return;
    phase_b = __ldcg(p.slow) != 0;                 // only if a part went through the accumulators
  } else if (phase_b) {
    if (!grid_barrier(p.bar, p.status)) return;
  }
  if (phase_b) {
    PSB_TSTAMP(3);
    // phase B: the leader of each touched key runs the optimiser on the summed gradient
    for (u32 i0 = gtid; i0 < total; i0 += 4 * gsize) {
      u32 sc[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        u32 i = i0 + q * gsize;
        sc[q] = 0;
        if (i >= total) continue;
        int r = 0;
        while (r + 1 < S && i >= s_pre[r + 1]) ++r;
        sc[q] = __ldcg(&p.slot_cache[r][i - s_pre[r]]);
        if ((sc[q] & 0x7fffffffu) == 0x7fffffffu) sc[q] = 0;
      }
      float2 ws[4];
      float4 sg[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        ws[q] = make_float2(0.f, 0.f);
        sg[q] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (sc[q] & 0x80000000u) {
          const Entry* e = &tab[sc[q] & 0x7fffffffu];
          ws[q] = __ldcg(reinterpret_cast<const float2*>(&e->w));    // (w, s0)
          sg[q] = __ldcg(reinterpret_cast<const float4*>(&e->s1));   // (s1, pad, gacc, gcnt): the second half
        }
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (!(sc[q] & 0x80000000u)) continue;
        Entry* e = &tab[sc[q] & 0x7fffffffu];
        float w = ws[q].x, s0 = ws[q].y, s1 = sg[q].x, w_old = w;
        opt_step(p.opt, sg[q].z, w, s0, s1);
        *reinterpret_cast<float2*>(&e->w) = make_float2(w, s0);
        *reinterpret_cast<float4*>(&e->s1) = make_float4(s1, 0.f, 0.f, 0.f);   // accumulator and count back to zero
        st.add(w, w_old);
      }
    }
  }
  PSB_TSTAMP(4);
  block_add4(st.d_nnz, st.w2, st.dw2, st.n, p.stats);
  // publish "applied" once every CTA is done
  PSB_TSTAMP(5);
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    u32 arrived = atomicAdd(p.done, 1u) + 1;
    s_last = (arrived == gridDim.x);
  }
  __syncthreads();
  if (s_last && threadIdx.x == 0) {
    if (p.slow) atomicExch(p.slow, 0u);
    __threadfence_system();
    st_release_sys(p.applied, p.ts1);
    atomicExch(p.done, 0u);
  }
  PSB_TSTAMP(6);
}

static int coop_grid_for(const void* fn) {
  int dev = 0, sms = 0, per = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per, fn, kThreads, 0);
  if (per < 1) per = 1;
  if (per > 4) per = 4;
  return sms * per;
}

}  // namespace psb

using namespace psb;

extern "C" int psb_device_sm_count(void) {
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms;
}

extern "C" int psb_coop_grid(int which) {
  static int g[4] = {0, 0, 0, 0};
  if (which < 0 || which > 3) return 0;
  if (!g[which]) {
    const void* fn = which == 0 ? (const void*)k_pull_margin
                   : which == 1 ? (const void*)k_push
                   : which == 2 ? (const void*)k_apply : (const void*)k_pull_exchange;
    g[which] = coop_grid_for(fn);
  }
  return g[which];
}

extern "C" int psb_table_init(void* table, psb_u64 capacity, cudaStream_t stream) {
  k_table_init<<<psb_device_sm_count() * 8, 256, 0, stream>>>((Entry*)table, capacity);
  return -(int)cudaGetLastError();
}

extern "C" int psb_table_dump(const void* table, psb_u64 capacity, psb_u64* out_keys,
                              float* out_w, psb_u64 out_cap, unsigned long long* out_n,
                              cudaStream_t stream) {
  cudaMemsetAsync(out_n, 0, sizeof(unsigned long long), stream);
  k_table_dump<false><<<psb_device_sm_count() * 8, 256, 0, stream>>>((const Entry*)table, capacity, (u64*)out_keys,
                                                   nullptr, nullptr, out_w, out_cap, out_n);
  return -(int)cudaGetLastError();
}

extern "C" int psb_table_export(const void* table, psb_u64 capacity, psb_u64* out_keys,
                                float* out_s0, float* out_s1, float* out_w, psb_u64 out_cap,
                                unsigned long long* out_n, cudaStream_t stream) {
  cudaMemsetAsync(out_n, 0, sizeof(unsigned long long), stream);
  k_table_dump<true><<<psb_device_sm_count() * 8, 256, 0, stream>>>((const Entry*)table, capacity, (u64*)out_keys,
                                                  out_s0, out_s1, out_w, out_cap, out_n);
  return -(int)cudaGetLastError();
}

extern "C" int psb_table_load(void* table, psb_u64 mask, psb_u64 key_begin, psb_u64 slot_mult,
                              const psb_u64* keys, const float* s0, const float* s1, const float* w,
                              psb_u64 n, uint32_t* status, cudaStream_t stream) {
  if (n == 0) return 0;
  k_table_load<<<psb_device_sm_count() * 4, 256, 0, stream>>>((Entry*)table, SlotMap{mask, key_begin, slot_mult},
                                            (const u64*)keys, s0, s1, w, n, status);
  return -(int)cudaGetLastError();
}

template <typename P>
static int launch_coop(const void* fn, int which, const P* p, cudaStream_t stream) {
  P local = *p;
  void* args[] = {&local};
  cudaError_t e = cudaLaunchCooperativeKernel(fn, dim3(psb_coop_grid(which)), dim3(kThreads), args,
                                              0, stream);
  return -(int)e;
}

extern "C" int psb_pull_margin(const PsbPullParams* p, cudaStream_t stream) {
  if (p->S < 1 || p->S > PSB_MAX_SHARDS) return -(int)cudaErrorInvalidValue;
  return launch_coop((const void*)k_pull_margin, 0, p, stream);
}
extern "C" int psb_pull_exchange(const PsbPullExchangeParams* p, cudaStream_t stream) {
  if (p->S < 1 || p->S > PSB_MAX_SHARDS) return -(int)cudaErrorInvalidValue;
  return launch_coop((const void*)k_pull_exchange, 3, p, stream);
}
extern "C" int psb_push(const PsbPushParams* p, cudaStream_t stream) {
  if (p->S < 1 || p->S > PSB_MAX_SHARDS) return -(int)cudaErrorInvalidValue;
  return launch_coop((const void*)k_push, 1, p, stream);
}
extern "C" int psb_apply(const PsbApplyParams* p, cudaStream_t stream) {
  if (p->S < 1 || p->S > PSB_MAX_SHARDS) return -(int)cudaErrorInvalidValue;
  return launch_coop((const void*)k_apply, 2, p, stream);
}

// sizeof of the parameter blocks, so that a binding can verify its mirror structs
#ifdef PSB_TRACE
extern "C" int psb_trace_set(long long* buf) {
  return -(int)cudaMemcpyToSymbol(g_trace, &buf, sizeof(buf));
}
#endif

extern "C" int psb_struct_size(int which) {
  switch (which) {
    case 0: return (int)sizeof(PsbPullParams);
    case 1: return (int)sizeof(PsbPushParams);
    case 2: return (int)sizeof(PsbApplyParams);
    case 3: return (int)sizeof(PsbOptimizer);
    case 4: return (int)sizeof(PsbPullExchangeParams);
    default: return -1;
  }
}
