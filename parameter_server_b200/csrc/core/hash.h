// Hash functions used by the filters and parsers:
//  * crc32c (Castagnoli polynomial, reflected 0x82F63B78) with the
//    Extend/Value/Mask/Unmask interface of util/crc32c.h:10-42. The table is
//    generated at start-up (slicing-by-4) instead of being stored as literals.
//  * MurmurHash3 x86_32, x86_128 and x64_128 (public-domain algorithm by Austin
//    Appleby, util/murmurhash3.h:29-33), written from the published algorithm.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cstring>

namespace PS {
namespace crc32c {

struct Tables {
  uint32_t t[4][256];
  Tables() {
    for (uint32_t i = 0; i < 256; ++i) {
      uint32_t c = i;
      for (int k = 0; k < 8; ++k) c = (c & 1) ? (c >> 1) ^ 0x82F63B78u : (c >> 1);
      t[0][i] = c;
    }
    for (uint32_t i = 0; i < 256; ++i)
      for (int s = 1; s < 4; ++s) t[s][i] = (t[s - 1][i] >> 8) ^ t[0][t[s - 1][i] & 0xff];
  }
};
inline const Tables& tables() { static Tables tb; return tb; }

// crc of concat(A, data[0,n-1]) given init_crc = crc of A
inline uint32_t Extend(uint32_t init_crc, const char* data, size_t n) {
  const Tables& tb = tables();
  const uint8_t* p = reinterpret_cast<const uint8_t*>(data);
  uint32_t c = init_crc ^ 0xffffffffu;
  while (n && (reinterpret_cast<uintptr_t>(p) & 3)) { c = tb.t[0][(c ^ *p++) & 0xff] ^ (c >> 8); --n; }
  while (n >= 4) {
    uint32_t w; memcpy(&w, p, 4); c ^= w;
    c = tb.t[3][c & 0xff] ^ tb.t[2][(c >> 8) & 0xff] ^ tb.t[1][(c >> 16) & 0xff] ^ tb.t[0][c >> 24];
    p += 4; n -= 4;
  }
  while (n--) c = tb.t[0][(c ^ *p++) & 0xff] ^ (c >> 8);
  return c ^ 0xffffffffu;
}
inline uint32_t Value(const char* data, size_t n) { return Extend(0, data, n); }
static const uint32_t kMaskDelta = 0xa282ead8ul;
// masked form for crcs that are stored next to the data they cover
inline uint32_t Mask(uint32_t crc) { return ((crc >> 15) | (crc << 17)) + kMaskDelta; }
inline uint32_t Unmask(uint32_t masked) { uint32_t r = masked - kMaskDelta; return (r >> 17) | (r << 15); }

}  // namespace crc32c

// ---------------------------------------------------------------- MurmurHash3
namespace murmur {
inline uint32_t rotl32(uint32_t x, int8_t r) { return (x << r) | (x >> (32 - r)); }
inline uint64_t rotl64(uint64_t x, int8_t r) { return (x << r) | (x >> (64 - r)); }
inline uint32_t fmix32(uint32_t h) { h ^= h >> 16; h *= 0x85ebca6b; h ^= h >> 13; h *= 0xc2b2ae35; h ^= h >> 16; return h; }
inline uint64_t fmix64(uint64_t k) { k ^= k >> 33; k *= 0xff51afd7ed558ccdULL; k ^= k >> 33; k *= 0xc4ceb9fe1a85ec53ULL; k ^= k >> 33; return k; }
inline uint32_t blk32(const uint8_t* p, int i) { uint32_t v; memcpy(&v, p + 4 * i, 4); return v; }
inline uint64_t blk64(const uint8_t* p, int i) { uint64_t v; memcpy(&v, p + 8 * i, 8); return v; }
}  // namespace murmur

inline void MurmurHash3_x86_32(const void* key, int len, uint32_t seed, void* out) {
  using namespace murmur;
  const uint8_t* data = (const uint8_t*)key;
  const int nblocks = len / 4;
  uint32_t h1 = seed;
  const uint32_t c1 = 0xcc9e2d51, c2 = 0x1b873593;
  for (int i = 0; i < nblocks; ++i) {
    uint32_t k1 = blk32(data, i);
    k1 *= c1; k1 = rotl32(k1, 15); k1 *= c2;
    h1 ^= k1; h1 = rotl32(h1, 13); h1 = h1 * 5 + 0xe6546b64;
  }
  const uint8_t* tail = data + nblocks * 4;
  uint32_t k1 = 0;
  switch (len & 3) {
    case 3: k1 ^= tail[2] << 16;  // fallthrough
    case 2: k1 ^= tail[1] << 8;   // fallthrough
    case 1: k1 ^= tail[0]; k1 *= c1; k1 = rotl32(k1, 15); k1 *= c2; h1 ^= k1;
  }
  h1 ^= len;
  h1 = fmix32(h1);
  *(uint32_t*)out = h1;
}

inline void MurmurHash3_x86_128(const void* key, const int len, uint32_t seed, void* out) {
  using namespace murmur;
  const uint8_t* data = (const uint8_t*)key;
  const int nblocks = len / 16;
  uint32_t h1 = seed, h2 = seed, h3 = seed, h4 = seed;
  const uint32_t c1 = 0x239b961b, c2 = 0xab0e9789, c3 = 0x38b34ae5, c4 = 0xa1e38b93;
  for (int i = 0; i < nblocks; ++i) {
    uint32_t k1 = blk32(data, i * 4 + 0), k2 = blk32(data, i * 4 + 1);
    uint32_t k3 = blk32(data, i * 4 + 2), k4 = blk32(data, i * 4 + 3);
    k1 *= c1; k1 = rotl32(k1, 15); k1 *= c2; h1 ^= k1;
    h1 = rotl32(h1, 19); h1 += h2; h1 = h1 * 5 + 0x561ccd1b;
    k2 *= c2; k2 = rotl32(k2, 16); k2 *= c3; h2 ^= k2;
    h2 = rotl32(h2, 17); h2 += h3; h2 = h2 * 5 + 0x0bcaa747;
    k3 *= c3; k3 = rotl32(k3, 17); k3 *= c4; h3 ^= k3;
    h3 = rotl32(h3, 15); h3 += h4; h3 = h3 * 5 + 0x96cd1c35;
    k4 *= c4; k4 = rotl32(k4, 18); k4 *= c1; h4 ^= k4;
    h4 = rotl32(h4, 13); h4 += h1; h4 = h4 * 5 + 0x32ac3b17;
  }
  const uint8_t* tail = data + nblocks * 16;
  uint32_t k1 = 0, k2 = 0, k3 = 0, k4 = 0;
  switch (len & 15) {
    case 15: k4 ^= tail[14] << 16;  // fallthrough
    case 14: k4 ^= tail[13] << 8;   // fallthrough
    case 13: k4 ^= tail[12] << 0; k4 *= c4; k4 = rotl32(k4, 18); k4 *= c1; h4 ^= k4;  // fallthrough
    case 12: k3 ^= tail[11] << 24;  // fallthrough
    case 11: k3 ^= tail[10] << 16;  // fallthrough
    case 10: k3 ^= tail[9] << 8;    // fallthrough
    case 9: k3 ^= tail[8] << 0; k3 *= c3; k3 = rotl32(k3, 17); k3 *= c4; h3 ^= k3;    // fallthrough
    case 8: k2 ^= tail[7] << 24;    // fallthrough
    case 7: k2 ^= tail[6] << 16;    // fallthrough
    case 6: k2 ^= tail[5] << 8;     // fallthrough
    case 5: k2 ^= tail[4] << 0; k2 *= c2; k2 = rotl32(k2, 16); k2 *= c3; h2 ^= k2;    // fallthrough
    case 4: k1 ^= tail[3] << 24;    // fallthrough
    case 3: k1 ^= tail[2] << 16;    // fallthrough
    case 2: k1 ^= tail[1] << 8;     // fallthrough
    case 1: k1 ^= tail[0] << 0; k1 *= c1; k1 = rotl32(k1, 15); k1 *= c2; h1 ^= k1;
  }
  h1 ^= len; h2 ^= len; h3 ^= len; h4 ^= len;
  h1 += h2; h1 += h3; h1 += h4; h2 += h1; h3 += h1; h4 += h1;
  h1 = fmix32(h1); h2 = fmix32(h2); h3 = fmix32(h3); h4 = fmix32(h4);
  h1 += h2; h1 += h3; h1 += h4; h2 += h1; h3 += h1; h4 += h1;
  ((uint32_t*)out)[0] = h1; ((uint32_t*)out)[1] = h2; ((uint32_t*)out)[2] = h3; ((uint32_t*)out)[3] = h4;
}

inline void MurmurHash3_x64_128(const void* key, const int len, const uint32_t seed, void* out) {
  using namespace murmur;
  const uint8_t* data = (const uint8_t*)key;
  const int nblocks = len / 16;
  uint64_t h1 = seed, h2 = seed;
  const uint64_t c1 = 0x87c37b91114253d5ULL, c2 = 0x4cf5ad432745937fULL;
  for (int i = 0; i < nblocks; ++i) {
    uint64_t k1 = blk64(data, i * 2 + 0), k2 = blk64(data, i * 2 + 1);
    k1 *= c1; k1 = rotl64(k1, 31); k1 *= c2; h1 ^= k1;
    h1 = rotl64(h1, 27); h1 += h2; h1 = h1 * 5 + 0x52dce729;
    k2 *= c2; k2 = rotl64(k2, 33); k2 *= c1; h2 ^= k2;
    h2 = rotl64(h2, 31); h2 += h1; h2 = h2 * 5 + 0x38495ab5;
  }
  const uint8_t* tail = data + nblocks * 16;
  uint64_t k1 = 0, k2 = 0;
  switch (len & 15) {
    case 15: k2 ^= ((uint64_t)tail[14]) << 48;  // fallthrough
    case 14: k2 ^= ((uint64_t)tail[13]) << 40;  // fallthrough
    case 13: k2 ^= ((uint64_t)tail[12]) << 32;  // fallthrough
    case 12: k2 ^= ((uint64_t)tail[11]) << 24;  // fallthrough
    case 11: k2 ^= ((uint64_t)tail[10]) << 16;  // fallthrough
    case 10: k2 ^= ((uint64_t)tail[9]) << 8;    // fallthrough
    case 9: k2 ^= ((uint64_t)tail[8]) << 0; k2 *= c2; k2 = rotl64(k2, 33); k2 *= c1; h2 ^= k2;  // fallthrough
    case 8: k1 ^= ((uint64_t)tail[7]) << 56;    // fallthrough
    case 7: k1 ^= ((uint64_t)tail[6]) << 48;    // fallthrough
    case 6: k1 ^= ((uint64_t)tail[5]) << 40;    // fallthrough
    case 5: k1 ^= ((uint64_t)tail[4]) << 32;    // fallthrough
    case 4: k1 ^= ((uint64_t)tail[3]) << 24;    // fallthrough
    case 3: k1 ^= ((uint64_t)tail[2]) << 16;    // fallthrough
    case 2: k1 ^= ((uint64_t)tail[1]) << 8;     // fallthrough
    case 1: k1 ^= ((uint64_t)tail[0]) << 0; k1 *= c1; k1 = rotl64(k1, 31); k1 *= c2; h1 ^= k1;
  }
  h1 ^= len; h2 ^= len;
  h1 += h2; h2 += h1;
  h1 = fmix64(h1); h2 = fmix64(h2);
  h1 += h2; h2 += h1;
  ((uint64_t*)out)[0] = h1; ((uint64_t*)out)[1] = h2;
}

}  // namespace PS
