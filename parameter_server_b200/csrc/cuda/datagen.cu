// Synthetic sparse logistic-regression data, generated on the device with a
// counter-based generator so that any (seed, batch, row, j) cell can be
// reproduced on the host. Shapes follow the benchmark configurations: rows
// with a fixed number of binary (or |N(0,1)|, row-normalised) nonzeros whose
// feature ids follow a Zipf-like law, labels y = sign(x.w* + logistic noise)
// with a sparse ground truth w* (1 % non-zeros ~ N(0,1)).
//
// The id law is the continuous inverse-CDF of x^-s on [1, N+1):
//   x = ((N+1)^(1-s) - 1) * u + 1) ^ (1/(1-s)),  id = floor(x) - 1,
// which matches Zipf(s) up to the discretisation of the first few ranks.
#include "psb_common.cuh"
#include "psb_cuda.h"

namespace psb {

__host__ __device__ __forceinline__ u64 cell_hash(u64 seed, u64 batch, u64 row, u64 j) {
  u64 h = fmix64(seed ^ 0xD1B54A32D192ED03ull);
  h = fmix64(h ^ (batch * 0x9E3779B97F4A7C15ull));
  h = fmix64(h ^ (row * 0xC2B2AE3D27D4EB4Full));
  h = fmix64(h ^ (j * 0x165667B19E3779F9ull));
  return h;
}
__host__ __device__ __forceinline__ double u01(u64 h) {  // (0,1)
  return ((double)(h >> 11) + 0.5) * (1.0 / 9007199254740992.0);
}
// ground-truth weight of a feature id: 1 % non-zero, standard normal
__device__ __forceinline__ float wstar(u64 id, u64 seed) {
  u64 h = fmix64(id * 0x9E3779B97F4A7C15ull + (seed ^ 0x5851F42D4C957F2Dull));
  if (h % 100 != 0) return 0.f;
  u64 h2 = fmix64(h ^ 0xA0761D6478BD642Full);
  float a = (float)u01(h2), b = (float)u01(fmix64(h2));
  return sqrtf(-2.f * logf(a)) * cospif(2.f * b);
}

__global__ void __launch_bounds__(256) k_gen_batch(u32* __restrict__ ids32, u64* __restrict__ ids64,
                                                   float* __restrict__ vals, float* __restrict__ y,
                                                   u32 n_rows, u32 z, u64 n_feat, double zipf_s,
                                                   u64 seed, u64 batch, int real_values) {
  const int lane = threadIdx.x & 31;
  const u32 gwarp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const u32 nwarps = (gridDim.x * blockDim.x) >> 5;
  const double one_m_s = 1.0 - zipf_s;
  const double span = pow((double)n_feat + 1.0, one_m_s) - 1.0;
  const double inv = 1.0 / one_m_s;
  for (u32 r = gwarp; r < n_rows; r += nwarps) {
    float dot = 0.f, nrm = 0.f;
    for (u32 j = lane; j < z; j += 32) {
      u64 h = cell_hash(seed, batch, r, j);
      double x = pow(span * u01(h) + 1.0, inv);
      u64 id = (u64)x;
      id = id < 1 ? 0 : id - 1;
      if (id >= n_feat) id = n_feat - 1;
      float v = 1.f;
      if (real_values) {
        u64 h2 = fmix64(h ^ 0x2545F4914F6CDD1Dull);
        float a = (float)u01(h2), b = (float)u01(fmix64(h2));
        v = fabsf(sqrtf(-2.f * logf(a)) * cospif(2.f * b)) + 1e-3f;
        nrm += v * v;
      }
      size_t o = (size_t)r * z + j;
      if (ids32) ids32[o] = (u32)id;
      if (ids64) ids64[o] = id;
      if (vals) vals[o] = v;
      dot += v * wstar(id, seed);
    }
    dot = warp_sum(dot);
    if (real_values) {
      nrm = sqrtf(warp_sum(nrm));
      for (u32 j = lane; j < z; j += 32) vals[(size_t)r * z + j] /= nrm;
      dot /= nrm;
    }
    if (lane == 0) {
      double u = u01(cell_hash(seed ^ 0x94D049BB133111EBull, batch, r, 0));
      float noise = (float)log(u / (1.0 - u));
      y[r] = (dot + noise) >= 0.f ? 1.f : -1.f;
    }
  }
}

__global__ void k_hash_ids(const u32* ids32, const u64* ids64, u64* keys, u64 n, u64 seed) {
  for (u64 i = blockIdx.x * (u64)blockDim.x + threadIdx.x; i < n; i += (u64)gridDim.x * blockDim.x)
    keys[i] = hash_id_to_key(ids32 ? (u64)ids32[i] : ids64[i], seed);
}

// Writes (1 + 2^-20) x 4-byte words over a buffer larger than L2; used by
// benchmarks to evict L2 between timed iterations.
__global__ void k_flush_l2(u32* buf, u64 n_words, u32 v) {
  for (u64 i = blockIdx.x * (u64)blockDim.x + threadIdx.x; i < n_words; i += (u64)gridDim.x * blockDim.x)
    buf[i] = v;
}

}  // namespace psb
using namespace psb;

extern "C" int psb_gen_batch(uint32_t* ids32, psb_u64* ids64, float* vals, float* y,
                             uint32_t n_rows, uint32_t z, psb_u64 n_feat, double zipf_s,
                             psb_u64 seed, psb_u64 batch, int real_values, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  if (zipf_s == 1.0) zipf_s = 1.0 + 1e-9;
  if (real_values && !vals) return -(int)cudaErrorInvalidValue;
  k_gen_batch<<<psb_device_sm_count() * 8, 256, 0, stream>>>(ids32, (u64*)ids64, vals, y, n_rows, z, n_feat, zipf_s,
                                           seed, batch, real_values);
  return -(int)cudaGetLastError();
}

extern "C" int psb_hash_ids(const uint32_t* ids32, const psb_u64* ids64, psb_u64* keys,
                            psb_u64 n, psb_u64 seed, cudaStream_t stream) {
  if (n == 0) return 0;
  k_hash_ids<<<psb_device_sm_count() * 8, 256, 0, stream>>>(ids32, (const u64*)ids64, (u64*)keys, n, seed);
  return -(int)cudaGetLastError();
}

// ---------------------------------------------------------------- random-access probes
// What a table walk can reach on this part: n look-ups of 32-byte entries at the given slot indices.
// mode 0: one 16-byte load per entry (what a pull does); mode 1: read 24 bytes, write 12 (what an
// optimiser update does). Four independent entries per thread and trip, as in the real kernels.
namespace psb {
__global__ void __launch_bounds__(256) k_probe_entries(Entry* __restrict__ tab, const u32* __restrict__ slots, u32 n,
                                                       int mode, float* __restrict__ out) {
  const u32 gsize = gridDim.x * blockDim.x, gtid = blockIdx.x * blockDim.x + threadIdx.x;
  for (u32 i0 = gtid; i0 < n; i0 += 4 * gsize) {
    u32 sl[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) sl[q] = (i0 + q * gsize < n) ? slots[i0 + q * gsize] : 0u;
    if (mode == 0) {
      u64 k[4], hi[4];
#pragma unroll
      for (int q = 0; q < 4; ++q)
        asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(k[q]), "=l"(hi[q]) : "l"(&tab[sl[q]]) : "memory");
#pragma unroll
      for (int q = 0; q < 4; ++q)
        if (i0 + q * gsize < n) out[i0 + q * gsize] = __uint_as_float((u32)hi[q]) + (k[q] == 1 ? 1.f : 0.f);
    } else {
      float2 ws[4];
      float s1[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        ws[q] = *reinterpret_cast<const float2*>(&tab[sl[q]].w);
        s1[q] = tab[sl[q]].s1;
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (i0 + q * gsize >= n) break;
        *reinterpret_cast<float2*>(&tab[sl[q]].w) = make_float2(ws[q].x + 1.f, ws[q].y + s1[q]);
        tab[sl[q]].s1 = s1[q] + 1.f;
      }
    }
  }
}
}  // namespace psb

extern "C" int psb_probe_entries(void* table, const uint32_t* slots, uint32_t n, int mode, float* out,
                                 cudaStream_t stream) {
  psb::k_probe_entries<<<psb_device_sm_count() * 4, 256, 0, stream>>>((psb::Entry*)table, slots, n, mode, out);
  return -(int)cudaGetLastError();
}

// Ids that arrive as a bit stream (`bits` per id, id i at bit offset i * bits of little-endian 32-bit
// words; the stream has a spare word after the last id) become 32-bit ids: two word loads, a funnel
// shift and a mask per id, neighbouring threads on neighbouring ids.
__global__ void __launch_bounds__(256) k_unpack_ids(const uint32_t* __restrict__ words, int bits, uint32_t n,
                                                    uint32_t* __restrict__ out) {
  const uint32_t mask = bits >= 32 ? 0xffffffffu : ((1u << bits) - 1u);
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const unsigned long long off = (unsigned long long)i * (unsigned)bits;
    const uint32_t w = (uint32_t)(off >> 5), sh = (uint32_t)(off & 31);
    out[i] = __funnelshift_r(words[w], words[w + 1], sh) & mask;
  }
}
extern "C" int psb_unpack_ids(const uint32_t* words, int bits, uint32_t n, uint32_t* out, cudaStream_t stream) {
  if (bits < 1 || bits > 32) return -(int)cudaErrorInvalidValue;
  if (n == 0) return 0;
  const uint32_t blocks = (n + 255) / 256, mx = (uint32_t)psb_device_sm_count() * 8;
  k_unpack_ids<<<blocks > mx ? mx : blocks, 256, 0, stream>>>(words, bits, n, out);
  return -(int)cudaGetLastError();
}

extern "C" int psb_flush_l2(uint32_t* buf, psb_u64 n_words, uint32_t v, cudaStream_t stream) {
  k_flush_l2<<<psb_device_sm_count() * 8, 256, 0, stream>>>(buf, n_words, v);
  return -(int)cudaGetLastError();
}
