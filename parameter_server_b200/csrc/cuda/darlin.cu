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

__global__ void __launch_bounds__(kDThreads) k_darlin_grad(const PsbDarlinGrad p) {
  __shared__ u32 s_last;
  const u32 gsize = gridDim.x * blockDim.x, gtid = blockIdx.x * blockDim.x + threadIdx.x;
  const int lane = threadIdx.x & 31;
  const u32 gwarp = gtid >> 5, nwarps = gsize >> 5;
  const u32 ncol = p.c1 - p.c0;
  // The staging area is zero on entry: phase 2 of the previous call cleared what it read.
  // phase 1: segmented reduction over the block's nonzeros. A warp takes chunks of
  // kChunkWords consecutive 32-element words and carries the sums of a column that runs
  // over a word boundary in registers, so that a frequent feature (a column of millions of
  // nonzeros under a Zipf law) costs two atomics per chunk instead of two per word:
  // same-address atomics serialise in L2.
  if (p.u1 > p.u0) {
    const u32 nz0 = p.seg_off[p.u0], nz1 = p.seg_off[p.u1];
    const u32 w0 = nz0 >> 5, w1 = (nz1 + 31) >> 5;
    const u32 le = 0xffffffffu >> (31 - lane);
    // chunk length: up to 16 words, but no longer than what keeps every warp busy
    const u32 kChunkWords = max(1u, min(16u, (w1 - w0 + nwarps - 1) / nwarps));
    const u32 nchunks = (w1 - w0 + kChunkWords - 1) / kChunkWords;
    for (u32 ch = gwarp; ch < nchunks; ch += nwarps) {
      const u32 wb = w0 + ch * kChunkWords, we = min(w1, wb + kChunkWords);
      float cg = 0.f, chh = 0.f;   // sums so far of the column that is open at the word boundary
      u32 cu = 0;                  // its local unique-key index
      bool open = false;
      for (u32 wi = wb; wi < we; ++wi) {
        const u32 i = wi * 32 + lane;
        const u32 f = p.flagbits[wi];
        const u32 fle = f & le;
        const u32 u = p.wordbase[wi] + __popc(fle) - 1;     // local unique key of this nonzero
        const bool in = i >= nz0 && i < nz1;
        float g = 0.f, h = 0.f;
        if (in) {
          u32 c = p.gcol[u];
          if (p.active[c]) {
            u32 r = p.csc_row[i];
            float y = p.y[r];
            float ym = y * __ldcg(&p.margin[r]);
            // tau = 1/(1+exp(y m)) evaluated stably
            float en = expf(-fabsf(ym));
            float tau = ym > 0 ? en / (1.f + en) : 1.f / (1.f + en);
            float d = p.delta[c];
            if (p.csc_val) {
              float v = p.csc_val[i];
              g = -y * tau * v;
              h = fminf(tau * (1.f - tau) * expf(fabsf(v) * d), 0.25f) * v * v;
            } else {
              g = -y * tau;
              h = fminf(tau * (1.f - tau) * expf(d), 0.25f);
            }
          }
        }
        auto flush = [&](u32 uu, float gg, float hh) {
          u32 c = p.gcol[uu] - p.c0;
          if (c < p.block_cap && (gg != 0.f || hh != 0.f)) {
            atomicAdd(&p.stage[c], gg);
            atomicAdd(&p.stage[p.block_cap + c], hh);
          }
        };
        if (open && (f & 1u)) {                     // the open column ended with the previous word
          if (lane == 0) flush(cu, cg, chh);
          open = false; cg = chh = 0.f;
        }
        // segmented inclusive scan inside the word; segment = column
        int start = fle ? 31 - __clz(fle) : 0;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          float g2 = __shfl_up_sync(0xffffffffu, g, o);
          float h2 = __shfl_up_sync(0xffffffffu, h, o);
          if (lane >= start + o) { g += g2; h += h2; }
        }
        if (fle == 0) { g += cg; h += chh; }        // lanes that continue the open column (the carry is 0 otherwise)
        const bool tail = (lane == 31) || ((f >> (lane + 1)) & 1u) || (i + 1 == nz1);
        // the word's last column stays open unless this is the chunk's last word or the block's data ends here
        const bool keep = (wi + 1 < we) && ((wi + 1) * 32 < nz1);
        if (in && tail && !(keep && lane == 31)) flush(u, g, h);
        if (keep) {
          cg = __shfl_sync(0xffffffffu, g, 31);
          chh = __shfl_sync(0xffffffffu, h, 31);
          cu = p.wordbase[wi] + __popc(f) - 1;
          open = true;
        } else {
          open = false; cg = chh = 0.f;
        }
      }
    }
  }
  if (!grid_barrier(p.bar, p.status)) return;
  // phase 2: dense slices to the owners
  for (u32 c = gtid; c < ncol; c += gsize) {
    int s = shard_of_col(p.shard_col, p.S, p.c0 + c);
    p.gu_inbox[s][c] = __ldcg(&p.stage[c]);
    p.gu_inbox[s][p.block_cap + c] = __ldcg(&p.stage[p.block_cap + c]);
    p.stage[c] = 0.f;                      // leave the staging area clean for the next block
    p.stage[p.block_cap + c] = 0.f;
  }
  // One system fence per CTA: the block barrier orders every thread's peer stores before
  // thread 0's fence (fences are cumulative), and that fence precedes the arrival count.
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    s_last = atomicAdd(p.done, 1u) + 1 == gridDim.x;
  }
  __syncthreads();
  if (s_last && threadIdx.x < p.S) {
    __threadfence_system();
    st_release_sys(p.ready[threadIdx.x], p.ts1);
    if (threadIdx.x == 0) atomicExch(p.done, 0u);
  }
}

__global__ void __launch_bounds__(kDThreads) k_darlin_update(const PsbDarlinUpdate p) {
  __shared__ u32 s_last;
  __shared__ float s_vio;
  const int S = p.S;
  if (threadIdx.x == 0) {
    s_vio = 0.f;
    const u32 iters = p.wait_iters ? p.wait_iters : kPeerWaitIters;
    for (int r = 0; r < S; ++r) {
      if (!p.alive[r]) continue;
      if (!wait_flag_ge_sys(p.ready[r], p.ts1, iters)) set_status(p.status, kWaitTimeout);
    }
  }
  __syncthreads();
  const u32 gsize = gridDim.x * blockDim.x, gtid = blockIdx.x * blockDim.x + threadIdx.x;
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
    __threadfence_system();   // one per CTA, after the block barrier (see k_darlin_grad)
    s_last = atomicAdd(p.done, 1u) + 1 == gridDim.x;
  }
  __syncthreads();
  if (s_last && threadIdx.x < S && p.alive[threadIdx.x]) {
    __threadfence_system();
    st_release_sys(p.wnew_ready[threadIdx.x], p.ts1);
  }
  if (s_last && threadIdx.x == 0) atomicExch(p.done, 0u);
}

__global__ void __launch_bounds__(kDThreads) k_darlin_dual(const PsbDarlinDual p) {
  const int S = p.S;
  if (threadIdx.x == 0) {
    const u32 iters = p.wait_iters ? p.wait_iters : kPeerWaitIters;
    for (int s = 0; s < S; ++s) {
      // only owners that hold a part of this block publish a slice
      u32 lo = max(p.c0, p.shard_col[s]), hi = min(p.c1, p.shard_col[s + 1]);
      if (lo >= hi || !p.alive[s]) continue;
      if (!wait_flag_ge_sys(p.wnew_ready[s], p.ts1, iters)) set_status(p.status, kWaitTimeout);
    }
  }
  __syncthreads();
  const u32 gsize = gridDim.x * blockDim.x, gtid = blockIdx.x * blockDim.x + threadIdx.x;
  const int lane = threadIdx.x & 31;
  const u32 gwarp = gtid >> 5, nwarps = gsize >> 5;
  // phase 1: m_i += dw_j x_ij over the block's nonzeros
  if (p.u1 > p.u0) {
    const u32 nz0 = p.seg_off[p.u0], nz1 = p.seg_off[p.u1];
    const u32 w0 = nz0 >> 5, w1 = (nz1 + 31) >> 5;
    const u32 le = 0xffffffffu >> (31 - lane);
    for (u32 wi = w0 + gwarp; wi < w1; wi += nwarps) {
      u32 i = wi * 32 + lane;
      if (i < nz0 || i >= nz1) continue;
      u32 u = p.wordbase[wi] + __popc(p.flagbits[wi] & le) - 1;
      u32 c = p.gcol[u];
      if (!p.active[c]) continue;
      float nw = p.wnew[c - p.c0];
      if (nw != nw) continue;                       // deactivated by the owner
      float dw = nw - p.w_cur[c];
      if (dw == 0.f) continue;
      float x = p.csc_val ? p.csc_val[i] : 1.f;
      atomicAdd(&p.margin[p.csc_row[i]], dw * x);
    }
  }
  if (!grid_barrier(p.bar, p.status)) return;
  // phase 2: per-column state of the whole block (also columns without local data)
  for (u32 c = p.c0 + gtid; c < p.c1; c += gsize) {
    if (!p.active[c]) continue;
    float nw = p.wnew[c - p.c0];
    if (nw != nw) { p.active[c] = 0; p.w_cur[c] = 0.f; continue; }
    float dw = nw - p.w_cur[c];
    p.delta[c] = fminf(p.delta_max, 2.f * fabsf(dw) + 0.1f);
    p.w_cur[c] = nw;
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
extern "C" int psb_darlin_eval(const float* y, const float* margin, uint32_t n_rows, const float* w,
                               const unsigned char* active, uint32_t c0, uint32_t c1, float lambda, double* out,
                               cudaStream_t stream) {
  k_darlin_eval<<<psb_device_sm_count() * 2, 256, 0, stream>>>(y, margin, n_rows, w, active, c0, c1, lambda, out);
  return -(int)cudaGetLastError();
}
extern "C" int psb_darlin_struct_size(int which) {
  return which == 0 ? (int)sizeof(PsbDarlinGrad) : which == 1 ? (int)sizeof(PsbDarlinUpdate) : (int)sizeof(PsbDarlinDual);
}
