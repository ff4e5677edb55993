// Device forms of the message filters and of the sorted-key utilities:
//
//   k_key_signature   key-caching filter (filter/key_caching.h:9-76): crc32c of
//                     the first 2 KiB of the key list (bit-compatible with the
//                     host crc32c) plus a fingerprint of the whole list; compares
//                     with the previous signature held in device memory and
//                     leaves a hit flag that the push / pull kernels read, so the
//                     decision never needs the host.
//   k_fixfloat_*      reference fixed-point codec (filter/fixing_float.h:51-102):
//                     clamp to [min,max], scale to an n-byte unsigned integer,
//                     random-bit rounding, little-endian bytes.
//   k_add_noise       NOISE filter (filter/add_noise.h:9-41).
//   k_countmin_*      count-min sketch with saturating uint8 cells and the same
//                     hash / probe sequence as util/countmin.h:21-41.
//   k_ordered_match   merge-join of two sorted key lists, dst op= src for k-wide
//                     values (util/parallel_ordered_match.h:7-83).
//   k_minmax          min / max of a float array (feeds the codec's range).
#include "psb_common.cuh"
#include "psb_cuda.h"

namespace psb {

// ---------------------------------------------------------------- crc32c + fingerprint
__device__ __forceinline__ u32 crc32c_byte(u32 c, u32 byte) {
  c ^= byte;
#pragma unroll
  for (int k = 0; k < 8; ++k) c = (c & 1) ? (c >> 1) ^ 0x82F63B78u : (c >> 1);
  return c;
}

// sig[0] = crc32c of the first min(8n, 2048) bytes, sig[1..2] = 64-bit
// fingerprint of (n, every key and its position). state = {prev sig[0..2], prev n};
// *hit = 1 iff all four match, then state is replaced by the new values.
__global__ void __launch_bounds__(256) k_key_signature(const u64* __restrict__ keys, const u32* __restrict__ n_ptr,
                                                       u32* __restrict__ partial, u32* __restrict__ state,
                                                       u32* __restrict__ hit, u32* __restrict__ sig_out,
                                                       u32* __restrict__ done) {
  __shared__ u64 s_red[8];
  __shared__ u32 s_last;
  const u32 n = *n_ptr;
  u64 acc = 0;
  for (u32 i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
    acc += fmix64(keys[i] ^ ((u64)i * 0x9E3779B97F4A7C15ull));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    u64 t = 0;
    for (int i = 0; i < 8; ++i) t += s_red[i];
    atomicAdd((unsigned long long*)partial, (unsigned long long)t);
    __threadfence();
    s_last = atomicAdd(done, 1u) + 1 == gridDim.x;
  }
  __syncthreads();
  if (!s_last || threadIdx.x != 0) return;
  __threadfence();
  // the last block finishes: crc of the head of the list (sequential, <= 2 KiB)
  u32 bytes = min(n * 8u, 2048u);
  u32 c = 0xffffffffu;
  const unsigned char* p = reinterpret_cast<const unsigned char*>(keys);
  for (u32 i = 0; i < bytes; ++i) c = crc32c_byte(c, p[i]);
  c ^= 0xffffffffu;
  u64 fp = *((volatile u64*)partial) + fmix64(n);
  u32 s1 = (u32)fp, s2 = (u32)(fp >> 32);
  u32 h = (state[0] == c && state[1] == s1 && state[2] == s2 && state[3] == n && n > 0) ? 1u : 0u;
  state[0] = c; state[1] = s1; state[2] = s2; state[3] = n;
  *hit = h;
  if (sig_out) { sig_out[0] = c; sig_out[1] = s1; sig_out[2] = s2; }
  *((volatile u64*)partial) = 0;
  *done = 0;
}

// ---------------------------------------------------------------- fixed point
__global__ void k_fixfloat_encode(const float* __restrict__ x, unsigned char* __restrict__ code, u64 n, int nbytes,
                                  float lo, float hi, u64 seed) {
  const double ratio = (double)(1ull << (nbytes * 8)) - 2.0;
  const double bin = (double)hi - (double)lo;
  for (u64 i = blockIdx.x * (u64)blockDim.x + threadIdx.x; i < n; i += (u64)gridDim.x * blockDim.x) {
    double v = x[i];
    v = v > hi ? hi : (v < lo ? lo : v);
    u64 r = (u64)floor((v - lo) / bin * ratio) + (fmix64(seed ^ (i * 0x9E3779B97F4A7C15ull)) & 1ull);
    for (int j = 0; j < nbytes; ++j) { code[i * nbytes + j] = (unsigned char)(r & 0xFF); r >>= 8; }
  }
}
__global__ void k_fixfloat_decode(const unsigned char* __restrict__ code, float* __restrict__ x, u64 n, int nbytes,
                                  float lo, float hi) {
  const double ratio = (double)(1ull << (nbytes * 8)) - 2.0;
  const double bin = (double)hi - (double)lo;
  for (u64 i = blockIdx.x * (u64)blockDim.x + threadIdx.x; i < n; i += (u64)gridDim.x * blockDim.x) {
    u64 r = 0;
    for (int j = 0; j < nbytes; ++j) r += (u64)code[i * nbytes + j] << (8 * j);
    x[i] = (float)((double)r / ratio * bin + lo);
  }
}

__global__ void k_minmax(const float* __restrict__ x, u64 n, float* __restrict__ out /*{min,max}, preset*/) {
  float lo = INFINITY, hi = -INFINITY;
  for (u64 i = blockIdx.x * (u64)blockDim.x + threadIdx.x; i < n; i += (u64)gridDim.x * blockDim.x) {
    float v = x[i];
    lo = fminf(lo, v); hi = fmaxf(hi, v);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
    hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
  }
  if ((threadIdx.x & 31) == 0) {
    // float atomics via the ordered-int trick
    auto amin = [](float* a, float v) {
      if (v >= 0) atomicMin((int*)a, __float_as_int(v)); else atomicMax((unsigned int*)a, __float_as_uint(v));
    };
    auto amax = [](float* a, float v) {
      if (v >= 0) atomicMax((int*)a, __float_as_int(v)); else atomicMin((unsigned int*)a, __float_as_uint(v));
    };
    amin(&out[0], lo); amax(&out[1], hi);
  }
}

__global__ void k_add_noise(float* __restrict__ x, u64 n, float mean, float stdv, u64 seed) {
  for (u64 i = blockIdx.x * (u64)blockDim.x + threadIdx.x; i < n; i += (u64)gridDim.x * blockDim.x) {
    u64 h = fmix64(seed ^ (i * 0xD1B54A32D192ED03ull));
    float a = ((float)(h >> 40) + 0.5f) * (1.f / 16777216.f);
    float b = ((float)((h >> 16) & 0xFFFFFF) + 0.5f) * (1.f / 16777216.f);
    x[i] += mean + stdv * sqrtf(-2.f * logf(a)) * cospif(2.f * b);
  }
}

// ---------------------------------------------------------------- count-min
__device__ __forceinline__ u32 sketch_hash(u64 key) {
  const u32 seed = 0xbc9f1d34u, m = 0xc6a4a793u, n = 8;
  u32 h = seed ^ (n * m);
  u32 w = (u32)key;
  h += w; h *= m; h ^= (h >> 16);
  w = (u32)(key >> 32);
  h += w; h *= m; h ^= (h >> 16);
  return h;
}
// cells are bytes packed four to a word; saturating add by CAS on the word
__device__ __forceinline__ void cell_add_sat(u32* words, u32 cell, u32 count) {
  u32* w = words + (cell >> 2);
  const u32 sh = (cell & 3) * 8;
  u32 old = *w;
  while (true) {
    u32 v = (old >> sh) & 0xFF;
    u32 nv = min(255u, v + count);
    if (nv == v) return;
    u32 assumed = old;
    old = atomicCAS(w, assumed, (assumed & ~(0xFFu << sh)) | (nv << sh));
    if (old == assumed) return;
  }
}
__global__ void k_countmin_insert(u32* __restrict__ cells, u32 n_cells, int k, const u64* __restrict__ keys,
                                  const unsigned char* __restrict__ counts, const u32* __restrict__ n_ptr, u32 n_fixed) {
  const u32 n = n_ptr ? *n_ptr : n_fixed;
  for (u32 i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    u32 h = sketch_hash(keys[i]);
    const u32 delta = (h >> 17) | (h << 15);
    u32 c = counts ? counts[i] : 1u;
    for (int j = 0; j < k; ++j) { cell_add_sat(cells, h % n_cells, c); h += delta; }
  }
}
__global__ void k_countmin_query(const u32* __restrict__ cells, u32 n_cells, int k, const u64* __restrict__ keys,
                                 unsigned char* __restrict__ out, const u32* __restrict__ n_ptr, u32 n_fixed) {
  const u32 n = n_ptr ? *n_ptr : n_fixed;
  for (u32 i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    u32 h = sketch_hash(keys[i]);
    const u32 delta = (h >> 17) | (h << 15);
    u32 res = 255;
    for (int j = 0; j < k; ++j) {
      u32 cell = h % n_cells;
      res = min(res, (cells[cell >> 2] >> ((cell & 3) * 8)) & 0xFF);
      h += delta;
    }
    out[i] = (unsigned char)res;
  }
}

// ---------------------------------------------------------------- ordered match
// op: 0 assign, 1 plus, 2 minus, 3 times, 4 divide. matched (nullable) counts hits.
__global__ void k_ordered_match(const u64* __restrict__ src_key, const float* __restrict__ src_val, u32 n_src,
                                const u64* __restrict__ dst_key, float* __restrict__ dst_val, u32 n_dst, int k, int op,
                                unsigned long long* __restrict__ matched) {
  u32 hits = 0;
  for (u32 i = blockIdx.x * blockDim.x + threadIdx.x; i < n_src; i += gridDim.x * blockDim.x) {
    u64 key = src_key[i];
    u32 lo = 0, hi = n_dst;
    while (lo < hi) { u32 mid = (lo + hi) >> 1; if (dst_key[mid] < key) lo = mid + 1; else hi = mid; }
    if (lo < n_dst && dst_key[lo] == key) {
      ++hits;
      for (int j = 0; j < k; ++j) {
        float s = src_val[(size_t)i * k + j];
        float* d = &dst_val[(size_t)lo * k + j];
        switch (op) {
          case 0: *d = s; break;
          case 1: *d += s; break;
          case 2: *d -= s; break;
          case 3: *d *= s; break;
          default: *d /= s; break;
        }
      }
    }
  }
  if (matched) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) hits += __shfl_xor_sync(0xffffffffu, hits, o);
    if ((threadIdx.x & 31) == 0 && hits) atomicAdd(matched, (unsigned long long)hits);
  }
}

}  // namespace psb
using namespace psb;

// scratch: 4 zeroed u32 words {partial lo, partial hi, done, pad}; state: 4 words kept between calls
extern "C" int psb_key_signature(const psb_u64* keys, const uint32_t* n_ptr, uint32_t max_n, uint32_t* scratch,
                                 uint32_t* state, uint32_t* hit, uint32_t* sig_out, cudaStream_t stream) {
  int blocks = (int)min((u32)(psb_device_sm_count() * 4), max(1u, (max_n + 255) / 256));
  k_key_signature<<<blocks, 256, 0, stream>>>((const u64*)keys, n_ptr, scratch, state, hit, sig_out, scratch + 2);
  return -(int)cudaGetLastError();
}
extern "C" int psb_fixfloat_encode(const float* x, void* code, psb_u64 n, int nbytes, float lo, float hi,
                                   psb_u64 seed, cudaStream_t stream) {
  if (nbytes < 1 || nbytes > 7 || !(hi > lo)) return -(int)cudaErrorInvalidValue;
  if (n == 0) return 0;
  k_fixfloat_encode<<<psb_device_sm_count() * 8, 256, 0, stream>>>(x, (unsigned char*)code, n, nbytes, lo, hi, seed);
  return -(int)cudaGetLastError();
}
extern "C" int psb_fixfloat_decode(const void* code, float* x, psb_u64 n, int nbytes, float lo, float hi,
                                   cudaStream_t stream) {
  if (nbytes < 1 || nbytes > 7 || !(hi > lo)) return -(int)cudaErrorInvalidValue;
  if (n == 0) return 0;
  k_fixfloat_decode<<<psb_device_sm_count() * 8, 256, 0, stream>>>((const unsigned char*)code, x, n, nbytes, lo, hi);
  return -(int)cudaGetLastError();
}
// out = {+inf, -inf} must be preset by the caller
extern "C" int psb_minmax(const float* x, psb_u64 n, float* out, cudaStream_t stream) {
  if (n == 0) return 0;
  k_minmax<<<psb_device_sm_count() * 4, 256, 0, stream>>>(x, n, out);
  return -(int)cudaGetLastError();
}
extern "C" int psb_add_noise(float* x, psb_u64 n, float mean, float stdv, psb_u64 seed, cudaStream_t stream) {
  if (n == 0) return 0;
  k_add_noise<<<psb_device_sm_count() * 8, 256, 0, stream>>>(x, n, mean, stdv, seed);
  return -(int)cudaGetLastError();
}
extern "C" int psb_countmin_insert(uint32_t* cells, uint32_t n_cells, int k, const psb_u64* keys,
                                   const unsigned char* counts, const uint32_t* n_ptr, uint32_t n,
                                   cudaStream_t stream) {
  k_countmin_insert<<<psb_device_sm_count() * 4, 256, 0, stream>>>(cells, n_cells, k, (const u64*)keys, counts, n_ptr, n);
  return -(int)cudaGetLastError();
}
extern "C" int psb_countmin_query(const uint32_t* cells, uint32_t n_cells, int k, const psb_u64* keys,
                                  unsigned char* out, const uint32_t* n_ptr, uint32_t n, cudaStream_t stream) {
  k_countmin_query<<<psb_device_sm_count() * 4, 256, 0, stream>>>(cells, n_cells, k, (const u64*)keys, out, n_ptr, n);
  return -(int)cudaGetLastError();
}
extern "C" int psb_ordered_match(const psb_u64* src_key, const float* src_val, uint32_t n_src,
                                 const psb_u64* dst_key, float* dst_val, uint32_t n_dst, int k, int op,
                                 unsigned long long* matched, cudaStream_t stream) {
  if (n_src == 0 || n_dst == 0) return 0;
  if (matched) cudaMemsetAsync(matched, 0, sizeof(unsigned long long), stream);
  k_ordered_match<<<psb_device_sm_count() * 4, 256, 0, stream>>>((const u64*)src_key, src_val, n_src, (const u64*)dst_key, dst_val,
                                               n_dst, k, op, matched);
  return -(int)cudaGetLastError();
}
