// Hash functions used by the filters and parsers:
//  * crc32c (Castagnoli polynomial, reflected 0x82F63B78) with the
//    Extend/Value/Mask/Unmask interface of util/crc32c.h:10-42. The table is
//    generated at start-up (slicing-by-4) instead of being stored as literals.
//  * MurmurHash3 x86_32, x86_128 and x64_128 (public-domain algorithm by Austin
//    Appleby, util/murmurhash3.h:29-33), written from the published algorithm.
#pragma once
#include <algorithm>
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
// The three variants share one shape: the input is cut into stripes of L lanes (L = 1, 4 words of 32 bits, or
// 2 words of 64 bits); lane j of a stripe is scrambled with its constants and folded into state word j, which
// is then rotated, chained to its neighbour and stepped; a last, partial stripe is zero-padded and only
// scrambled; the length is mixed in and the state words are cross-added around a finalising mix.
namespace murmur {
template <typename W> inline W rotl(W x, int r) { return (W)((x << r) | (x >> (int(sizeof(W)) * 8 - r))); }
inline uint32_t fmix(uint32_t h) { h ^= h >> 16; h *= 0x85ebca6b; h ^= h >> 13; h *= 0xc2b2ae35; h ^= h >> 16; return h; }
inline uint64_t fmix(uint64_t k) { k ^= k >> 33; k *= 0xff51afd7ed558ccdULL; k ^= k >> 33; k *= 0xc4ceb9fe1a85ec53ULL; k ^= k >> 33; return k; }

// little-endian word from `n` <= sizeof(W) bytes, the missing high bytes zero
template <typename W> inline W load_le(const uint8_t* p, size_t n) {
  W v = 0;
  for (size_t i = 0; i < n; ++i) v |= (W)p[i] << (8 * i);
  return v;
}
// a whole word (little-endian hosts)
template <typename W> inline W load_word(const uint8_t* p) { W v; memcpy(&v, p, sizeof(W)); return v; }

// W: state word; L: lanes. mul[j], mul[(j+1)%L] scramble lane j around a rotation by kr[j]; the state word is
// then rotated by hr[j] and stepped to h * 5 + add[j].
template <typename W, int L>
struct Variant {
  W mul[L];
  int kr[L], hr[L];
  uint32_t add[L];
  W scramble(W k, int j) const { return (W)(rotl<W>((W)(k * mul[j]), kr[j]) * mul[(j + 1) % L]); }
  void run(const void* key, int len, uint32_t seed, W* h) const {
    const uint8_t* p = (const uint8_t*)key;
    const size_t word = sizeof(W), stripe = word * L;
    for (int j = 0; j < L; ++j) h[j] = seed;
    size_t left = (size_t)len;
    for (; left >= stripe; left -= stripe, p += stripe) {
      for (int j = 0; j < L; ++j) {
        h[j] ^= scramble(load_word<W>(p + word * j), j);
        h[j] = rotl<W>(h[j], hr[j]);
        if (L > 1) h[j] += h[(j + 1) % L];
        h[j] = (W)(h[j] * 5 + add[j]);
      }
    }
    // the ragged end: highest lane first, as the state words are not chained here the order does not matter
    for (int j = L - 1; j >= 0; --j) {
      if (left <= word * j) continue;
      const size_t n = std::min(word, left - word * j);
      h[j] ^= scramble(load_le<W>(p + word * j, n), j);
    }
    for (int j = 0; j < L; ++j) h[j] ^= (W)len;
    for (int pass = 0; pass < 2; ++pass) {
      for (int j = 1; j < L; ++j) h[0] += h[j];
      for (int j = 1; j < L; ++j) h[j] += h[0];
      if (pass == 0) for (int j = 0; j < L; ++j) h[j] = fmix(h[j]);
    }
  }
};
}  // namespace murmur

inline void MurmurHash3_x86_32(const void* key, int len, uint32_t seed, void* out) {
  using namespace murmur;
  const uint32_t c1 = 0xcc9e2d51, c2 = 0x1b873593;
  auto scramble = [&](uint32_t k) { return (uint32_t)(rotl<uint32_t>(k * c1, 15) * c2); };
  const uint8_t* p = (const uint8_t*)key;
  uint32_t h = seed;
  size_t left = (size_t)len;
  for (; left >= 4; left -= 4, p += 4) h = rotl<uint32_t>(h ^ scramble(load_word<uint32_t>(p)), 13) * 5 + 0xe6546b64;
  if (left) h ^= scramble(load_le<uint32_t>(p, left));
  *(uint32_t*)out = fmix(h ^ (uint32_t)len);
}

inline void MurmurHash3_x86_128(const void* key, const int len, uint32_t seed, void* out) {
  static const murmur::Variant<uint32_t, 4> v = {{0x239b961b, 0xab0e9789, 0x38b34ae5, 0xa1e38b93},
                                                 {15, 16, 17, 18}, {19, 17, 15, 13},
                                                 {0x561ccd1b, 0x0bcaa747, 0x96cd1c35, 0x32ac3b17}};
  v.run(key, len, seed, (uint32_t*)out);
}

inline void MurmurHash3_x64_128(const void* key, const int len, const uint32_t seed, void* out) {
  static const murmur::Variant<uint64_t, 2> v = {{0x87c37b91114253d5ULL, 0x4cf5ad432745937fULL}, {31, 33}, {27, 31},
                                                 {0x52dce729, 0x38495ab5}};
  v.run(key, len, seed, (uint64_t*)out);
}

}  // namespace PS
