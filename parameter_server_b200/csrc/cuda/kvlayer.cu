// Dense "layer" parameters (kernel family K10): tensors keyed by a layer id,
// small ones stored whole on one shard, large ones split evenly by element range.
// Counterpart of KVLayer Slice / SetValue / GetValue (parameter/kv_layer.h:121-210);
// over NVLink a push is the scatter half of a reduce-scatter (every worker stores
// each owner's slice into that owner's inbox) and a pull is an all-gather done by
// the reader.
//
//   k_layer_push   worker: for every owner, wait (bounded) until that owner has
//                  applied the round that last used this ring slot, then copy the
//                  owner's element range into its inbox with 16-byte peer stores
//                  (one contiguous loop per owner), then a release flag.
//   k_layer_apply  owner: bounded wait for every source, sum the sources with
//                  16-byte loads and run the updater (assign / add / sgd step) on
//                  the owned segment, publish the applied counter.
//   k_layer_pull   worker: the owned segments are read back from the owners with
//                  16-byte system-scope peer loads.
//
// The inbox of a (layer, source) pair is a ring of slots indexed by round % ring:
// a worker may run up to `ring` rounds ahead of a slow owner and no further (the
// same rule as the sparse plane's inboxes). Segment boundaries are multiples of
// four elements, so every slice starts 16-byte aligned.
//
// Also here: the fabric probe (peer store / peer load bandwidth), the device
// counterpart of the reference's raw transport probe (test/network_perf_ps.cc:23-47).
#include "psb_common.cuh"
#include "psb_cuda.h"

namespace psb {

__device__ __forceinline__ float4 ld_sys_f4(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float ld_sys_f1(const float* p) {
  float v;
  asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}

struct LayerPushArgs {
  int S;
  uint32_t ts1;
  uint32_t need_applied;                   // owners must have applied this many rounds before the slot is reused
  uint32_t wait_iters;
  const float* data;                       // the whole layer on the worker
  psb_u64 seg_begin[PSB_MAX_SHARDS + 1];   // element range of shard s: [seg_begin[s], seg_begin[s+1])
  float* inbox[PSB_MAX_SHARDS];            // owner s: this source's inbox for this ring slot
  uint32_t* ready[PSB_MAX_SHARDS];         // owner s: this source's ready flag for this ring slot
  const uint32_t* applied[PSB_MAX_SHARDS]; // owner s: applied counter of the layer
  uint32_t* done;
  uint32_t* status;
};

__global__ void __launch_bounds__(256) k_layer_push(const LayerPushArgs p) {
  __shared__ u32 s_last;
  __shared__ u32 s_ok[PSB_MAX_SHARDS];
  if (threadIdx.x == 0) {
    const u32 iters = p.wait_iters ? p.wait_iters : kPeerWaitIters;
    for (int s = 0; s < p.S; ++s) {
      s_ok[s] = 1;
      if (p.need_applied && p.seg_begin[s + 1] > p.seg_begin[s] &&
          !wait_flag_ge_sys(p.applied[s], p.need_applied, iters)) {
        // the owner still needs the slot's previous round: leave it alone and report
        s_ok[s] = 0;
        set_status(p.status, kWaitTimeout);
      }
    }
  }
  __syncthreads();
  const u64 gsize = (u64)gridDim.x * blockDim.x, gtid = blockIdx.x * (u64)blockDim.x + threadIdx.x;
  // Every CTA takes the owners in its own order (CTA b starts with owner b mod S): at any moment the grid's
  // stores are spread over all owners. With every CTA on owner 0 first, all GPUs would write into the same
  // GPU at the same time and the other links would sit idle.
  for (int k = 0; k < p.S; ++k) {
    const int s = (int)((blockIdx.x + (u32)k) % (u32)p.S);
    if (!s_ok[s]) continue;
    const u64 b = p.seg_begin[s], n = p.seg_begin[s + 1] - b;
    const float* src = p.data + b;
    float* dst = p.inbox[s];
    const u64 n4 = ((((size_t)src | (size_t)dst) & 15) == 0) ? n / 4 : 0;
    // two 16-byte loads in flight per thread
    for (u64 i = gtid; i < n4; i += 2 * gsize) {
      const u64 j = i + gsize;
      const float4 a = __ldcs(reinterpret_cast<const float4*>(src) + i);
      float4 c = a;
      if (j < n4) c = __ldcs(reinterpret_cast<const float4*>(src) + j);
      reinterpret_cast<float4*>(dst)[i] = a;
      if (j < n4) reinterpret_cast<float4*>(dst)[j] = c;
    }
    for (u64 i = 4 * n4 + gtid; i < n; i += gsize) dst[i] = src[i];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(p.done, 1u) + 1 == gridDim.x;
  __syncthreads();
  if (s_last && threadIdx.x < p.S) {
    __threadfence_system();
    if (s_ok[threadIdx.x]) st_release_sys(p.ready[threadIdx.x], p.ts1);
    if (threadIdx.x == 0) atomicExch(p.done, 0u);
  }
}

struct LayerApplyArgs {
  int S;
  uint32_t ts1;
  int updater;                             // 0 assign sum, 1 add sum, 2 sgd: data -= lr * sum
  float lr;
  psb_u64 n;                               // elements of my segment
  float* data;                             // my segment
  const float* inbox[PSB_MAX_SHARDS];      // source r's inbox for this ring slot
  const uint32_t* ready[PSB_MAX_SHARDS];
  uint8_t alive[PSB_MAX_SHARDS];
  uint32_t wait_iters;
  uint32_t* applied;
  uint32_t* done;
  uint32_t* status;
};

__device__ __forceinline__ float layer_update(int updater, float lr, float d, float s) {
  return updater == 0 ? s : (updater == 1 ? d + s : d - lr * s);
}

__global__ void __launch_bounds__(256) k_layer_apply(const LayerApplyArgs p) {
  __shared__ u32 s_last;
  if (threadIdx.x == 0) {
    const u32 iters = p.wait_iters ? p.wait_iters : kPeerWaitIters;
    for (int r = 0; r < p.S; ++r)
      if (p.alive[r] && !wait_flag_ge_sys(p.ready[r], p.ts1, iters)) set_status(p.status, kWaitTimeout);
  }
  __syncthreads();
  const u64 gsize = (u64)gridDim.x * blockDim.x, gtid = blockIdx.x * (u64)blockDim.x + threadIdx.x;
  bool aligned = (((size_t)p.data) & 15) == 0;
  for (int r = 0; r < p.S; ++r) aligned = aligned && ((((size_t)p.inbox[r]) & 15) == 0);
  const u64 n4 = aligned ? p.n / 4 : 0;
  for (u64 i = gtid; i < n4; i += gsize) {
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < p.S; ++r)
      if (p.alive[r]) {
        // the inbox was filled by peer stores that the ready flag ordered: read past L1
        const float4 v = __ldcg(reinterpret_cast<const float4*>(p.inbox[r]) + i);
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
      }
    float4 d = reinterpret_cast<float4*>(p.data)[i];
    d.x = layer_update(p.updater, p.lr, d.x, s.x); d.y = layer_update(p.updater, p.lr, d.y, s.y);
    d.z = layer_update(p.updater, p.lr, d.z, s.z); d.w = layer_update(p.updater, p.lr, d.w, s.w);
    reinterpret_cast<float4*>(p.data)[i] = d;
  }
  for (u64 i = 4 * n4 + gtid; i < p.n; i += gsize) {
    float s = 0.f;
    for (int r = 0; r < p.S; ++r) if (p.alive[r]) s += __ldcg(&p.inbox[r][i]);
    p.data[i] = layer_update(p.updater, p.lr, p.data[i], s);
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

struct LayerPullArgs {
  int S;
  uint32_t need_applied;
  float* out;                              // the whole layer on the worker
  psb_u64 seg_begin[PSB_MAX_SHARDS + 1];
  const float* data[PSB_MAX_SHARDS];       // owner s: its segment (peer pointer)
  const uint32_t* applied[PSB_MAX_SHARDS];
  uint32_t wait_iters;
  uint32_t* status;
};

__global__ void __launch_bounds__(256) k_layer_pull(const LayerPullArgs p) {
  if (threadIdx.x == 0 && p.need_applied) {
    const u32 iters = p.wait_iters ? p.wait_iters : kPeerWaitIters;
    for (int s = 0; s < p.S; ++s)
      if (p.seg_begin[s + 1] > p.seg_begin[s] && !wait_flag_ge_sys(p.applied[s], p.need_applied, iters))
        set_status(p.status, kWaitTimeout);
  }
  __syncthreads();
  const u64 gsize = (u64)gridDim.x * blockDim.x, gtid = blockIdx.x * (u64)blockDim.x + threadIdx.x;
  for (int k = 0; k < p.S; ++k) {
    const int s = (int)((blockIdx.x + (u32)k) % (u32)p.S);   // owners in a per-CTA order, as in k_layer_push
    const u64 b = p.seg_begin[s], n = p.seg_begin[s + 1] - b;
    const float* src = p.data[s];
    float* dst = p.out + b;
    const u64 n4 = ((((size_t)src | (size_t)dst) & 15) == 0) ? n / 4 : 0;
    for (u64 i = gtid; i < n4; i += 2 * gsize) {
      const u64 j = i + gsize;
      const float4 a = ld_sys_f4(src + 4 * i);
      float4 c = a;
      if (j < n4) c = ld_sys_f4(src + 4 * j);
      __stcs(reinterpret_cast<float4*>(dst) + i, a);
      if (j < n4) __stcs(reinterpret_cast<float4*>(dst) + j, c);
    }
    for (u64 i = 4 * n4 + gtid; i < n; i += gsize) dst[i] = ld_sys_f1(src + i);
  }
}

// ---------------------------------------------------------------- fabric probe
// mode 0: dst[i] = src[i] with 16-byte accesses (peer store when dst is a peer's memory, peer load when
// src is); mode 1: read-only sum of src (peer load bandwidth without a local write).
__global__ void __launch_bounds__(256) k_fabric_copy(const float4* __restrict__ src, float4* __restrict__ dst,
                                                     psb_u64 n4, int mode, float* sink) {
  const u64 gsize = (u64)gridDim.x * blockDim.x, gtid = blockIdx.x * (u64)blockDim.x + threadIdx.x;
  float acc = 0.f;
  for (u64 i = gtid; i < n4; i += 4 * gsize) {
    float4 v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const u64 j = i + k * gsize;
      v[k] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (j < n4) v[k] = ld_sys_f4(reinterpret_cast<const float*>(src + j));
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const u64 j = i + k * gsize;
      if (j >= n4) break;
      if (mode == 0) dst[j] = v[k];
      else acc += v[k].x + v[k].y + v[k].z + v[k].w;
    }
  }
  if (mode == 1 && acc == 12345.678f) *sink = acc;   // keeps the loads alive
}

}  // namespace psb
using namespace psb;

static int layer_grid(psb_u64 n) {
  const psb_u64 b = (n / 4 + 255) / 256;
  const psb_u64 mx = (psb_u64)psb_device_sm_count() * 8;
  return (int)(b < 1 ? 1 : (b > mx ? mx : b));
}
extern "C" int psb_layer_push(const void* args, cudaStream_t stream) {
  LayerPushArgs a = *reinterpret_cast<const LayerPushArgs*>(args);
  if (a.S < 1 || a.S > PSB_MAX_SHARDS) return -(int)cudaErrorInvalidValue;
  k_layer_push<<<layer_grid(a.seg_begin[a.S]), 256, 0, stream>>>(a);
  return -(int)cudaGetLastError();
}
extern "C" int psb_layer_apply(const void* args, cudaStream_t stream) {
  LayerApplyArgs a = *reinterpret_cast<const LayerApplyArgs*>(args);
  if (a.S < 1 || a.S > PSB_MAX_SHARDS) return -(int)cudaErrorInvalidValue;
  k_layer_apply<<<layer_grid(a.n), 256, 0, stream>>>(a);
  return -(int)cudaGetLastError();
}
extern "C" int psb_layer_pull(const void* args, cudaStream_t stream) {
  LayerPullArgs a = *reinterpret_cast<const LayerPullArgs*>(args);
  if (a.S < 1 || a.S > PSB_MAX_SHARDS) return -(int)cudaErrorInvalidValue;
  k_layer_pull<<<layer_grid(a.seg_begin[a.S]), 256, 0, stream>>>(a);
  return -(int)cudaGetLastError();
}
extern "C" int psb_layer_args_size(int which) {
  return which == 0 ? (int)sizeof(LayerPushArgs) : which == 1 ? (int)sizeof(LayerApplyArgs) : (int)sizeof(LayerPullArgs);
}
// bytes must be a multiple of 16 and both pointers 16-byte aligned; either may be peer-mapped memory
extern "C" int psb_fabric_copy(const void* src, void* dst, psb_u64 bytes, int mode, float* sink, cudaStream_t stream) {
  if ((bytes & 15) || (((size_t)src | (size_t)dst) & 15)) return -(int)cudaErrorInvalidValue;
  k_fabric_copy<<<psb_device_sm_count() * 8, 256, 0, stream>>>((const float4*)src, (float4*)dst, bytes / 16, mode, sink);
  return -(int)cudaGetLastError();
}
