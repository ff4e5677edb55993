// Dense "layer" parameters (kernel family K10): tensors keyed by a layer id,
// small ones stored whole on one shard, large ones split evenly by element range.
// Counterpart of KVLayer Slice / SetValue / GetValue (parameter/kv_layer.h:121-210).
//
//   k_layer_push   worker: each shard's element range of the layer goes into that
//                  owner's per-source inbox by 16-byte peer stores, then a release flag.
//   k_layer_apply  owner: bounded wait for every source, sum the sources and run
//                  the updater (assign / add / sgd step) on the owned segment.
//   k_layer_pull   worker: the owned segments are read back from the owners by
//                  16-byte peer loads (an all-gather done by the reader).
#include "psb_common.cuh"
#include "psb_cuda.h"

namespace psb {

struct LayerPushArgs {
  int S;
  uint32_t ts1;
  const float* data;                       // the whole layer on the worker
  psb_u64 seg_begin[PSB_MAX_SHARDS + 1];   // element range of shard s: [seg_begin[s], seg_begin[s+1])
  float* inbox[PSB_MAX_SHARDS];            // owner s: inbox of this source, indexed from the segment start
  uint32_t* ready[PSB_MAX_SHARDS];
  uint32_t* done;
};

__global__ void __launch_bounds__(256) k_layer_push(const LayerPushArgs p) {
  __shared__ u32 s_last;
  const u64 gsize = (u64)gridDim.x * blockDim.x, gtid = blockIdx.x * (u64)blockDim.x + threadIdx.x;
  const u64 total = p.seg_begin[p.S];
  for (u64 i = gtid; i < total; i += gsize) {
    int s = 0;
    while (s + 1 < p.S && i >= p.seg_begin[s + 1]) ++s;
    p.inbox[s][i - p.seg_begin[s]] = p.data[i];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(p.done, 1u) + 1 == gridDim.x;
  __syncthreads();
  if (s_last && threadIdx.x < p.S) {
    __threadfence_system();
    st_release_sys(p.ready[threadIdx.x], p.ts1);
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
  const float* inbox[PSB_MAX_SHARDS];
  const uint32_t* ready[PSB_MAX_SHARDS];
  uint8_t alive[PSB_MAX_SHARDS];
  uint32_t wait_iters;
  uint32_t* applied;
  uint32_t* done;
  uint32_t* status;
};

__global__ void __launch_bounds__(256) k_layer_apply(const LayerApplyArgs p) {
  __shared__ u32 s_last;
  if (threadIdx.x == 0) {
    const u32 iters = p.wait_iters ? p.wait_iters : kPeerWaitIters;
    for (int r = 0; r < p.S; ++r)
      if (p.alive[r] && !wait_flag_ge_sys(p.ready[r], p.ts1, iters)) set_status(p.status, kWaitTimeout);
  }
  __syncthreads();
  const u64 gsize = (u64)gridDim.x * blockDim.x, gtid = blockIdx.x * (u64)blockDim.x + threadIdx.x;
  for (u64 i = gtid; i < p.n; i += gsize) {
    float s = 0.f;
    for (int r = 0; r < p.S; ++r) if (p.alive[r]) s += p.inbox[r][i];
    float d = p.data[i];
    p.data[i] = p.updater == 0 ? s : (p.updater == 1 ? d + s : d - p.lr * s);
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
  const u64 total = p.seg_begin[p.S];
  for (u64 i = gtid; i < total; i += gsize) {
    int s = 0;
    while (s + 1 < p.S && i >= p.seg_begin[s + 1]) ++s;
    float v;
    asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p.data[s] + (i - p.seg_begin[s])) : "memory");
    p.out[i] = v;
  }
}

}  // namespace psb
using namespace psb;

static int layer_grid(psb_u64 n) {
  psb_u64 b = (n + 255) / 256;
  return (int)(b < 1 ? 1 : (b > 148 * 8 ? 148 * 8 : b));
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
