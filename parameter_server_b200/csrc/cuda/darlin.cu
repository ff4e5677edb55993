// Darlin (delayed block proximal gradient) on the device, kernel family F3.
//
//   k_darlin_grad    worker: per column of the block, first-order gradient g and
//                    the diagonal upper bound u of the second order, as a
//                    segmented reduction over the block's CSC nonzeros (balanced
//                    per 32 nonzeros, not per column); then the dense (G, U)
//                    slices go to the owning shards by peer stores + release flags.
//                    Replaces DarlinWorker::ComputeGradient and the push
//                    (app/linear_method/darlin.h:368-463).
//   k_darlin_update  owner: bounded wait for every worker's slice, sum over
//                    workers, Newton step with soft threshold inside the trust
//                    region, KKT filter; new weights are broadcast to every
//                    worker by peer stores (NaN marks a deactivated coordinate,
//                    filter/sparse_filter.h:8-20). Replaces
//                    DarlinServer::Update / UpdateWeight (darlin.h:200-304).
//   k_darlin_dual    worker: bounded wait for the owners' slices, margin update
//                    m_i += dw_j x_ij (the log of the reference's multiplicative
//                    dual update, darlin.h:507-588), then per-column state
//                    (weights, trust region, active set).
//
// The worker keeps margins m = Xw instead of dual = exp(y m): tau = 1/(1+exp(y m))
// is evaluated where it is used, and the dual update becomes an atomic add.
#include <cstdlib>
#include "psb_common.cuh"
#include "psb_cuda.h"

namespace psb {

static constexpr int kDThreads = 256;

__device__ __forceinline__ int shard_of_col(const u32* shard_col, int S, u32 c) {
  int s = 0;
#pragma unroll 1
  while (s + 1 < S && c >= shard_col[s + 1]) ++s;
  return s;
}

// Phase 1 of the gradient step: segmented reduction over the block's nonzeros into the staging area
// (zero on entry: phase 2 of the previous use of this area cleared what it read). A warp takes chunks of
// consecutive 32-element words and carries the sums of a column that runs over a word boundary in
// registers, so that a frequent feature (a column of millions of nonzeros under a Zipf law) costs two
// atomics per chunk instead of two per word: same-address atomics serialise in L2. The loads of
// kGradGroup words are issued together before the (sequential) scans, because every word costs a chain
// of three dependent gathers (word base -> column -> column state; row -> label, margin).
static constexpr int kGradGroup = 4;

// The CTAs that share a column pass: all of the grid, or a part of it when several passes run side
// by side (k_darlin_pass). index: this CTA's place among them.
struct Part { u32 index, count; };
__device__ __forceinline__ Part whole_grid() { return Part{blockIdx.x, gridDim.x}; }
__device__ void darlin_grad_p1(const PsbDarlinGrad& p) {
  if (p.u1 <= p.u0) return;
  const u32 gsize = gridDim.x * blockDim.x, gtid = blockIdx.x * blockDim.x + threadIdx.x;
  const int lane = threadIdx.x & 31;
  const u32 gwarp = gtid >> 5, nwarps = gsize >> 5;
  const u32 nz0 = p.nz0, nz1 = p.nz1;
  const u32 w0 = nz0 >> 5, w1 = (nz1 + 31) >> 5;
  const u32 le = 0xffffffffu >> (31 - lane);
  // chunk length: up to 16 words, but no longer than what keeps every warp busy
  const u32 kChunkWords = max(1u, min(16u, (w1 - w0 + nwarps - 1) / nwarps));
  const u32 nchunks = (w1 - w0 + kChunkWords - 1) / kChunkWords;
  auto flush = [&](u32 col, float gg, float hh) {
    const u32 c = col - p.c0;
    if (c < p.block_cap && (gg != 0.f || hh != 0.f)) {
      atomicAdd(&p.stage[c], gg);
      atomicAdd(&p.stage[p.block_cap + c], hh);
    }
  };
  for (u32 ch = gwarp; ch < nchunks; ch += nwarps) {
    const u32 wb = w0 + ch * kChunkWords, we = min(w1, wb + kChunkWords);
    float cg = 0.f, chh = 0.f;   // sums so far of the column that is open at the word boundary
    u32 ccol = 0;                // that column
    bool open = false;
    for (u32 gb = wb; gb < we; gb += kGradGroup) {
      u32 f[kGradGroup], col[kGradGroup], row[kGradGroup];
      float g[kGradGroup], h[kGradGroup], val[kGradGroup];
      bool in[kGradGroup];
#pragma unroll
      for (int k = 0; k < kGradGroup; ++k) {
        const u32 wi = gb + k;
        const bool valid = wi < we;
        f[k] = valid ? p.flagbits[wi] : 0u;
        const u32 i = wi * 32 + lane;
        in[k] = valid && i >= nz0 && i < nz1;
        if (p.csc_col != nullptr) {
          col[k] = in[k] ? p.csc_col[i] : 0u;                         // the column of every nonzero is at hand
        } else {
          const u32 base = valid ? p.wordbase[wi] : 0u;
          col[k] = in[k] ? p.gcol[base + __popc(f[k] & le) - 1] : 0u;   // local unique key -> global column
        }
        row[k] = in[k] ? p.csc_row[i] : 0u;
        val[k] = (in[k] && p.csc_val) ? p.csc_val[i] : 1.f;
      }
#pragma unroll
      for (int k = 0; k < kGradGroup; ++k) {
        g[k] = h[k] = 0.f;
        // every gather of this level is issued before the active flag is known
        const unsigned char act = in[k] ? p.active[col[k]] : (unsigned char)0;
        const float y = in[k] ? p.y[row[k]] : 0.f;
        const float mg = in[k] ? __ldcg(&p.margin[row[k]]) : 0.f;
        const float d = in[k] ? p.delta[col[k]] : 0.f;
        if (act) {
          const float ym = y * mg;
          // tau = 1/(1+exp(y m)) evaluated stably; the fast exponential and reciprocal are good to a few
          // ulp, far inside what the sums over a column carry
          const float en = __expf(-fabsf(ym));
          const float rc = __fdividef(1.f, 1.f + en);
          const float tau = ym > 0 ? en * rc : rc;
          const float v = val[k];
          g[k] = -y * tau * v;
          h[k] = fminf(tau * (1.f - tau) * __expf(fabsf(v) * d), 0.25f) * v * v;
        }
      }
#pragma unroll
      for (int k = 0; k < kGradGroup; ++k) {
        const u32 wi = gb + k;
        if (wi >= we) break;
        const u32 i = wi * 32 + lane;
        const u32 fw = f[k], fle = fw & le;
        float gg = g[k], hh = h[k];
        if (open && (fw & 1u)) {                     // the open column ended with the previous word
          if (lane == 0) flush(ccol, cg, chh);
          open = false; cg = chh = 0.f;
        }
        // segmented inclusive scan inside the word; segment = column
        const int start = fle ? 31 - __clz(fle) : 0;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const float g2 = __shfl_up_sync(0xffffffffu, gg, o);
          const float h2 = __shfl_up_sync(0xffffffffu, hh, o);
          if (lane >= start + o) { gg += g2; hh += h2; }
        }
        if (fle == 0) { gg += cg; hh += chh; }       // lanes that continue the open column (the carry is 0 otherwise)
        const bool tail = (lane == 31) || ((fw >> (lane + 1)) & 1u) || (i + 1 == nz1);
        // the word's last column stays open unless this is the chunk's last word or the block's data ends here
        const bool keep = (wi + 1 < we) && ((wi + 1) * 32 < nz1);
        if (in[k] && tail && !(keep && lane == 31)) flush(col[k], gg, hh);
        if (keep) {
          cg = __shfl_sync(0xffffffffu, gg, 31);
          chh = __shfl_sync(0xffffffffu, hh, 31);
          ccol = __shfl_sync(0xffffffffu, col[k], 31);
          open = true;
        } else {
          open = false; cg = chh = 0.f;
        }
      }
    }
  }
}

// Phase 2 of the gradient step (after a grid barrier): the dense (G, U) slices go to the owners; the
// last CTA to finish raises this source's flag at every owner.
__device__ void darlin_grad_p2(const PsbDarlinGrad& p, const Part part) {
  __shared__ u32 s_last;
  const u32 gsize = part.count * blockDim.x, gtid = part.index * blockDim.x + threadIdx.x;
  const u32 ncol = p.c1 - p.c0;
  for (u32 c = gtid; c < ncol; c += gsize) {
    int s = shard_of_col(p.shard_col, p.S, p.c0 + c);
    p.gu_inbox[s][c] = __ldcg(&p.stage[c]);
    p.gu_inbox[s][p.block_cap + c] = __ldcg(&p.stage[p.block_cap + c]);
    p.stage[c] = 0.f;                      // leave the staging area clean for its next block
    p.stage[p.block_cap + c] = 0.f;
  }
  // One system fence per CTA: the block barrier orders every thread's peer stores before
  // thread 0's fence (fences are cumulative), and that fence precedes the arrival count.
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    s_last = atomicAdd(p.done, 1u) + 1 == part.count;
  }
  __syncthreads();
  if (s_last && threadIdx.x < p.S) {
    __threadfence_system();
    st_release_sys(p.ready[threadIdx.x], p.ts1);
    if (threadIdx.x == 0) atomicExch(p.done, 0u);
  }
}

__device__ bool darlin_grad_body(const PsbDarlinGrad& p) {
  darlin_grad_p1(p);
  if (!grid_barrier(p.bar, p.status)) return false;
  darlin_grad_p2(p, whole_grid());
  return true;
}
__global__ void __launch_bounds__(kDThreads) k_darlin_grad(const PsbDarlinGrad p) { darlin_grad_body(p); }

__device__ void darlin_update_body(const PsbDarlinUpdate& p, const Part part) {
  __shared__ u32 s_last;
  __shared__ float s_vio;
  const int S = p.S;
  if (threadIdx.x == 0) s_vio = 0.f;
  if (threadIdx.x < S && p.alive[threadIdx.x]) {   // one lane per source: the polls run side by side
    const u32 iters = p.wait_iters ? p.wait_iters : kPeerWaitIters;
    if (!wait_flag_ge_sys(p.ready[threadIdx.x], p.ts1, iters)) set_status(p.status, kWaitTimeout);
  }
  __syncthreads();
  const u32 gsize = part.count * blockDim.x, gtid = part.index * blockDim.x + threadIdx.x;
  float vio_max = 0.f;
  const float nan = __int_as_float(0x7fffffff);
  for (u32 c = p.my0 + gtid; c < p.my1; c += gsize) {
    const u32 b = c - p.c0;
    float out;
    if (!p.active[c]) {
      out = nan;
    } else {
      float G = 0.f, U = 0.f;
      for (int r = 0; r < S; ++r) {
        if (!p.alive[r]) continue;
        G += p.gu_inbox[r][b];
        U += p.gu_inbox[r][p.block_cap + b];
      }
      float u = U / p.eta + 1e-10f;
      float g_pos = G + p.lambda, g_neg = G - p.lambda;
      float w = p.w[c];
      float d = -w, vio = 0.f;
      bool frozen = false;
      if (w == 0.f) {
        if (g_pos < 0.f) vio = -g_pos;
        else if (g_neg > 0.f) vio = g_neg;
        else if (g_pos > p.kkt_threshold && g_neg < -p.kkt_threshold) frozen = true;
      }
      if (frozen) {
        p.active[c] = 0;
        out = nan;
      } else {
        vio_max = fmaxf(vio_max, vio);
        if (g_pos <= u * w) d = -g_pos / u;
        else if (g_neg >= u * w) d = -g_neg / u;
        float dl = p.delta[c];
        d = fminf(dl, fmaxf(-dl, d));
        p.delta[c] = fminf(p.delta_max, 2.f * fabsf(d) + 0.1f);
        w += d;
        p.w[c] = w;
        out = w;
      }
    }
    for (int r = 0; r < S; ++r) if (p.alive[r]) p.wnew_inbox[r][b] = out;   // broadcast
  }
  // violation
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) vio_max = fmaxf(vio_max, __shfl_xor_sync(0xffffffffu, vio_max, o));
  if ((threadIdx.x & 31) == 0 && vio_max > 0.f) atomicMax((int*)&s_vio, __float_as_int(vio_max));
  __syncthreads();
  if (threadIdx.x == 0) {
    if (s_vio > 0.f && p.violation) atomicMax((int*)p.violation, __float_as_int(s_vio));
    __threadfence_system();   // one per CTA, after the block barrier (see darlin_grad_p2)
    s_last = atomicAdd(p.done, 1u) + 1 == part.count;
  }
  __syncthreads();
  if (s_last && threadIdx.x < S && p.alive[threadIdx.x]) {
    __threadfence_system();
    st_release_sys(p.wnew_ready[threadIdx.x], p.ts1);
  }
  if (s_last && threadIdx.x == 0) atomicExch(p.done, 0u);
}
__global__ void __launch_bounds__(kDThreads) k_darlin_update(const PsbDarlinUpdate p) { darlin_update_body(p, whole_grid()); }

// The margin step in three parts: bounded wait for the owners' slices; m_i += dw_j x_ij over the
// block's nonzeros; after a grid barrier the per-column state of the whole block.
__device__ void darlin_dual_wait(const PsbDarlinDual& p) {
  if (threadIdx.x == 0) {
    const u32 iters = p.wait_iters ? p.wait_iters : kPeerWaitIters;
    for (int s = 0; s < p.S; ++s) {
      // only owners that hold a part of this block publish a slice
      u32 lo = max(p.c0, p.shard_col[s]), hi = min(p.c1, p.shard_col[s + 1]);
      if (lo >= hi || !p.alive[s]) continue;
      if (!wait_flag_ge_sys(p.wnew_ready[s], p.ts1, iters)) set_status(p.status, kWaitTimeout);
    }
  }
  __syncthreads();
}
// The same wait by one warp for itself: lane s polls owner s's flag, so the flags are polled side by side.
__device__ void darlin_dual_wait_warp(const PsbDarlinDual& p) {
  const int s = threadIdx.x & 31;
  if (s < p.S) {
    const u32 lo = max(p.c0, p.shard_col[s]), hi = min(p.c1, p.shard_col[s + 1]);
    if (lo < hi && p.alive[s]) {
      const u32 iters = p.wait_iters ? p.wait_iters : kPeerWaitIters;
      if (!wait_flag_ge_sys(p.wnew_ready[s], p.ts1, iters)) set_status(p.status, kWaitTimeout);
    }
  }
  __syncwarp();
}
__device__ void darlin_dual_p1(const PsbDarlinDual& p) {
  if (p.u1 <= p.u0) return;
  const u32 gsize = gridDim.x * blockDim.x, gtid = blockIdx.x * blockDim.x + threadIdx.x;
  const int lane = threadIdx.x & 31;
  const u32 gwarp = gtid >> 5, nwarps = gsize >> 5;
  const u32 nz0 = p.nz0, nz1 = p.nz1;
  const u32 w0 = nz0 >> 5, w1 = (nz1 + 31) >> 5;
  const u32 le = 0xffffffffu >> (31 - lane);
  constexpr int kGroup = 4;                 // words whose gathers are in flight together
  for (u32 wa = w0 + gwarp; wa < w1; wa += nwarps * kGroup) {
    u32 col[kGroup], row[kGroup];
    float x[kGroup];
    bool in[kGroup];
#pragma unroll
    for (int k = 0; k < kGroup; ++k) {
      const u32 wi = wa + k * nwarps;
      const u32 i = wi * 32 + lane;
      in[k] = wi < w1 && i >= nz0 && i < nz1;
      if (p.csc_col != nullptr) col[k] = in[k] ? p.csc_col[i] : 0u;
      else col[k] = in[k] ? p.gcol[p.wordbase[wi] + __popc(p.flagbits[wi] & le) - 1] : 0u;
      row[k] = in[k] ? p.csc_row[i] : 0u;
      x[k] = (in[k] && p.csc_val) ? p.csc_val[i] : 1.f;
    }
#pragma unroll
    for (int k = 0; k < kGroup; ++k) {
      if (!in[k]) continue;
      // the three gathers are independent of each other: issue them together
      const unsigned char act = p.active[col[k]];
      const float nw = p.wnew[col[k] - p.c0];
      const float wc = p.w_cur[col[k]];
      const float dw = nw - wc;                     // NaN (deactivated by the owner) fails the test below
      if (act && dw == dw && dw != 0.f) atomicAdd(&p.margin[row[k]], dw * x[k]);
    }
  }
}
__device__ void darlin_dual_p2(const PsbDarlinDual& p, const Part part) {
  const u32 gsize = part.count * blockDim.x, gtid = part.index * blockDim.x + threadIdx.x;
  // per-column state of the whole block (also columns without local data)
  for (u32 c = p.c0 + gtid; c < p.c1; c += gsize) {
    if (!p.active[c]) continue;
    float nw = p.wnew[c - p.c0];
    if (nw != nw) { p.active[c] = 0; p.w_cur[c] = 0.f; continue; }
    float dw = nw - p.w_cur[c];
    p.delta[c] = fminf(p.delta_max, 2.f * fabsf(dw) + 0.1f);
    p.w_cur[c] = nw;
  }
}
__device__ bool darlin_dual_body(const PsbDarlinDual& p) {
  darlin_dual_wait(p);
  darlin_dual_p1(p);
  if (!grid_barrier(p.bar, p.status)) return false;
  darlin_dual_p2(p, whole_grid());
  return true;
}
__global__ void __launch_bounds__(kDThreads) k_darlin_dual(const PsbDarlinDual p) { darlin_dual_body(p); }

// ---------------------------------------------------------------- a whole pass in one launch
// The block schedule of a pass (darlin.h:56-85,157-164) as one persistent cooperative kernel. The
// per-block parameter blocks (one per block and ring slot) are prepared by the host once and read from
// device memory here; only the stamp and the KKT threshold change from pass to pass. Between GPUs the
// same release/acquire flags as in the single-block kernels are used.
//
// Without delay (tau = 0) a block's gradient, owner update and margin step run one after another with
// a grid barrier between the phases. With delay tau >= 1 the scheduler's wait_time window lets the
// gradient of block i run on margins that miss the weight changes of the last tau blocks, so step i is
// two phases with ONE grid barrier between them, and nothing in it waits for work of the same step
// unless tau == 1:
//
//   phase A   nonzero passes: gradient sums of block i into staging area i % ring; margin update of
//             block i - tau (its new weights were published during step i - 1)
//   ---- grid barrier
//   phase B   column passes: gradient slices of block i to the owners (+ flags); column state of block
//             i - tau; owner update of block i - tau + 1 (+ flags), whose slices arrived a step ago
//             when tau >= 2
//
// There is no barrier between phase B of step i and phase A of step i + 1: the two touch different
// staging areas, different blocks' column state, and the margins only by atomic adds and loads that
// the window allows to be stale; a CTA that runs ahead stops at the barrier of step i + 1.
template <typename P>
__device__ __forceinline__ void load_params(P* dst, const P* src) {
  static_assert(sizeof(P) % 4 == 0, "parameter blocks are copied word by word");
  const u32* s = reinterpret_cast<const u32*>(src);
  u32* d = reinterpret_cast<u32*>(dst);
  for (u32 i = threadIdx.x; i < sizeof(P) / 4; i += blockDim.x) d[i] = s[i];
}

static constexpr int kPassThreads = 1024;

__device__ __forceinline__ u64 globaltimer_ns() {
  u64 t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__global__ void __launch_bounds__(kPassThreads, 1) k_darlin_pass(const PsbDarlinPass q) {
  __shared__ PsbDarlinGrad s_g;
  __shared__ PsbDarlinUpdate s_u;
  __shared__ PsbDarlinDual s_d;
  const int R = q.ring;
  const u32 n = q.n_steps, tau = (u32)q.tau;
  if (tau == 0) {
    for (u32 i = 0; i < n; ++i) {
      const u32 ts = q.ts_base + i;
      const size_t at = (size_t)q.order[i] * R + ts % R;
      __syncthreads();                             // nobody still reads the previous step's blocks
      load_params(&s_g, &q.grad[at]);
      load_params(&s_u, &q.update[at]);
      load_params(&s_d, &q.dual[at]);
      __syncthreads();
      if (threadIdx.x == 0) {
        s_g.ts1 = s_u.ts1 = s_d.ts1 = ts + 1;
        s_u.kkt_threshold = q.kkt_threshold;
        s_u.wait_iters = s_d.wait_iters = q.wait_iters;
      }
      __syncthreads();
      darlin_grad_p1(s_g);
      if (!grid_barrier(q.bar, q.status)) return;
      darlin_grad_p2(s_g, whole_grid());
      if (s_u.S > 0) darlin_update_body(s_u, whole_grid());      // S == 0: none of the block's columns is mine
      darlin_dual_wait(s_d);
      darlin_dual_p1(s_d);
      if (!grid_barrier(q.bar, q.status)) return;
      darlin_dual_p2(s_d, whole_grid());
      // the next gradient reads trust regions and the active set that the column pass wrote
      if (!grid_barrier(q.bar, q.status)) return;
    }
    return;
  }
  // shares of the column passes: the owner update is the longest of the three, the column state the
  // shortest; with fewer than six CTAs (never on a real device) every CTA would need all three
  const u32 n_upd = gridDim.x / 2, n_out = gridDim.x / 3;
  // The parameter blocks of step i + 1 are fetched (one word per thread, into a register) right after the
  // barrier of step i, so that their global-memory latency runs under the column passes.
  constexpr u32 WG = sizeof(PsbDarlinGrad) / 4, WU = sizeof(PsbDarlinUpdate) / 4, WD = sizeof(PsbDarlinDual) / 4;
  static_assert(WG + WU + WD <= kPassThreads, "one word of the three parameter blocks per thread");
  auto fetch = [&](u32 i, u32& word) -> bool {
    const u32 t = threadIdx.x;
    if (t < WG) {
      if (i >= n) return false;
      word = reinterpret_cast<const u32*>(&q.grad[(size_t)q.order[i] * R + (q.ts_base + i) % R])[t];
    } else if (t < WG + WU) {
      if (i + 1 < tau || i + 1 - tau >= n) return false;
      const u32 k = i + 1 - tau;
      word = reinterpret_cast<const u32*>(&q.update[(size_t)q.order[k] * R + (q.ts_base + k) % R])[t - WG];
    } else if (t < WG + WU + WD) {
      if (i < tau || i - tau >= n) return false;
      const u32 j = i - tau;
      word = reinterpret_cast<const u32*>(&q.dual[(size_t)q.order[j] * R + (q.ts_base + j) % R])[t - WG - WU];
    } else {
      return false;
    }
    return true;
  };
  u32 pre = 0;
  bool pre_ok = fetch(0, pre);
  for (u32 i = 0; i < n + tau; ++i) {
    const bool has_g = i < n, has_d = i >= tau, has_u = i + 1 >= tau && i + 1 - tau < n;
    // With q.phase_ns, CTA 0 adds up where its time goes: {loading the parameter blocks, the two nonzero
    // passes, barrier, its column pass (the owner update)} in nanoseconds (the CTA is held together at
    // every mark).
    u64 t[5];
    auto mark = [&](int k) {
      if (q.phase_ns == nullptr || blockIdx.x != 0) return;
      __syncthreads();
      if (threadIdx.x == 0) t[k] = globaltimer_ns();
    };
    mark(0);
    __syncthreads();                               // nobody still reads the previous step's blocks
    if (pre_ok) {
      const u32 tt = threadIdx.x;
      if (tt < WG) reinterpret_cast<u32*>(&s_g)[tt] = pre;
      else if (tt < WG + WU) reinterpret_cast<u32*>(&s_u)[tt - WG] = pre;
      else reinterpret_cast<u32*>(&s_d)[tt - WG - WU] = pre;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      s_g.ts1 = q.ts_base + i + 1;
      s_d.ts1 = q.ts_base + i - tau + 1;
      s_u.ts1 = q.ts_base + i + 1 - tau + 1;
      s_u.kkt_threshold = q.kkt_threshold;
      s_u.wait_iters = s_d.wait_iters = q.wait_iters;
    }
    __syncthreads();
    // phase A. Both nonzero passes are a burst of gathers followed by arithmetic; odd warps take them in
    // the other order so that one half's arithmetic runs under the other half's memory latency.
    mark(1);
    if ((threadIdx.x >> 5) & 1) {
      if (has_d) { darlin_dual_wait_warp(s_d); darlin_dual_p1(s_d); }
      if (has_g) darlin_grad_p1(s_g);
    } else {
      if (has_g) darlin_grad_p1(s_g);
      if (has_d) { darlin_dual_wait_warp(s_d); darlin_dual_p1(s_d); }
    }
    mark(2);
    if (!grid_barrier(q.bar, q.status)) return;
    mark(3);
    pre_ok = fetch(i + 1, pre);
    // phase B: the three column passes side by side, each on its share of the CTAs
    if (blockIdx.x < n_upd) {
      if (has_u && s_u.S > 0) darlin_update_body(s_u, Part{blockIdx.x, n_upd});
    } else if (blockIdx.x < n_upd + n_out) {
      if (has_g) darlin_grad_p2(s_g, Part{blockIdx.x - n_upd, n_out});
    } else {
      if (has_d) darlin_dual_p2(s_d, Part{blockIdx.x - n_upd - n_out, gridDim.x - n_upd - n_out});
    }
    mark(4);
    if (q.phase_ns != nullptr && blockIdx.x == 0 && threadIdx.x == 0)
      for (int k = 0; k < 4; ++k) q.phase_ns[k] += t[k + 1] - t[k];
  }
}

__global__ void __launch_bounds__(256) k_darlin_eval(const float* __restrict__ y, const float* __restrict__ margin,
                                                     u32 n_rows, const float* __restrict__ w,
                                                     const unsigned char* __restrict__ active, u32 c0, u32 c1,
                                                     float lambda, double* __restrict__ out) {
  __shared__ double s_acc[4];
  if (threadIdx.x < 4) s_acc[threadIdx.x] = 0;
  __syncthreads();
  double loss = 0, l1 = 0, nnz = 0, act = 0;
  const u32 gsize = gridDim.x * blockDim.x, gtid = blockIdx.x * blockDim.x + threadIdx.x;
  for (u32 r = gtid; r < n_rows; r += gsize) {
    float ym = y[r] * margin[r];
    loss += log1pf(expf(-fabsf(ym))) + fmaxf(-ym, 0.f);
  }
  for (u32 c = c0 + gtid; c < c1; c += gsize) {
    float v = w[c];
    if (active[c]) act += 1;
    if (v == v && v != 0.f) { l1 += fabsf(v); nnz += 1; }
  }
  loss = warp_sum_d(loss); l1 = warp_sum_d(l1); nnz = warp_sum_d(nnz); act = warp_sum_d(act);
  if ((threadIdx.x & 31) == 0) {
    atomicAdd(&s_acc[0], loss); atomicAdd(&s_acc[1], l1 * lambda); atomicAdd(&s_acc[2], nnz); atomicAdd(&s_acc[3], act);
  }
  __syncthreads();
  if (threadIdx.x < 4 && s_acc[threadIdx.x] != 0) atomicAdd(&out[threadIdx.x], s_acc[threadIdx.x]);
}

static int darlin_grid(const void* fn) {
  int dev = 0, sms = 0, per = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per, fn, kDThreads, 0);
  // at most four co-resident CTAs per SM: more only lengthen the grid barriers of these short kernels
  const int want = 4;
  per = per < 1 ? 1 : (per > want ? want : per);
  return sms * per;
}

}  // namespace psb
using namespace psb;

template <typename P>
static int launch_darlin(const void* fn, const P* p, cudaStream_t stream) {
  static int grid = 0;  // one instantiation (and one cached grid) per kernel parameter type
  if (grid == 0) grid = darlin_grid(fn);
  P local = *p;
  void* args[] = {&local};
  return -(int)cudaLaunchCooperativeKernel(fn, dim3(grid), dim3(kDThreads), args, 0, stream);
}

extern "C" int psb_darlin_grad(const PsbDarlinGrad* p, cudaStream_t stream) {
  if (p->S < 1 || p->S > PSB_MAX_SHARDS || p->c1 - p->c0 > p->block_cap) return -(int)cudaErrorInvalidValue;
  return launch_darlin((const void*)k_darlin_grad, p, stream);
}
extern "C" int psb_darlin_update(const PsbDarlinUpdate* p, cudaStream_t stream) {
  if (p->S < 1 || p->S > PSB_MAX_SHARDS || p->c1 - p->c0 > p->block_cap) return -(int)cudaErrorInvalidValue;
  return launch_darlin((const void*)k_darlin_update, p, stream);
}
extern "C" int psb_darlin_dual(const PsbDarlinDual* p, cudaStream_t stream) {
  if (p->S < 1 || p->S > PSB_MAX_SHARDS || p->c1 - p->c0 > p->block_cap) return -(int)cudaErrorInvalidValue;
  return launch_darlin((const void*)k_darlin_dual, p, stream);
}
extern "C" int psb_darlin_pass(const PsbDarlinPass* p, cudaStream_t stream) {
  if (p->ring < 1 || p->tau < 0 || p->tau + 1 > p->ring) return -(int)cudaErrorInvalidValue;
  if (psb_device_sm_count() < 6) return -(int)cudaErrorInvalidValue;   // the column passes share the CTAs 3 : 2 : 1
  // one CTA of 1024 threads per SM: the grid barrier gets shorter with fewer arrivals, and the gathers
  // of the nonzero passes want every warp slot the register file allows
  PsbDarlinPass local = *p;
  void* args[] = {&local};
  return -(int)cudaLaunchCooperativeKernel((const void*)k_darlin_pass, dim3(psb_device_sm_count()), dim3(kPassThreads), args,
                                           0, stream);
}
extern "C" int psb_darlin_eval(const float* y, const float* margin, uint32_t n_rows, const float* w,
                               const unsigned char* active, uint32_t c0, uint32_t c1, float lambda, double* out,
                               cudaStream_t stream) {
  k_darlin_eval<<<psb_device_sm_count() * 2, 256, 0, stream>>>(y, margin, n_rows, w, active, c0, c1, lambda, out);
  return -(int)cudaGetLastError();
}
extern "C" int psb_darlin_struct_size(int which) {
  return which == 0 ? (int)sizeof(PsbDarlinGrad) : which == 1 ? (int)sizeof(PsbDarlinUpdate)
       : which == 2 ? (int)sizeof(PsbDarlinDual) : (int)sizeof(PsbDarlinPass);
}
