// Probabilistic sketches: the shared 64->32 bit hash, count-min sketch, Bloom
// filter, cache-line-blocked Bloom filter, and the uint16-word bitmap.
// Counterparts: util/sketch.h:7-34, util/countmin.h:7-48,
// util/bloom_filter.h:5-47, util/block_bloom_filter.h:10-69, util/bitmap.h:13-97.
#pragma once
#include "hash.h"
#include "sarray.h"

namespace PS {

class Sketch {
 public:
  // multiplicative 64->32 bit mix of the two key halves (same constants and
  // steps as the reference, so sketch contents agree)
  static uint32_t hash(const uint64_t& key) {
    const uint32_t seed = 0xbc9f1d34, m = 0xc6a4a793, n = 8;
    uint32_t h = seed ^ (n * m);
    uint32_t w = (uint32_t)key;
    h += w; h *= m; h ^= (h >> 16);
    w = (uint32_t)(key >> 32);
    h += w; h *= m; h ^= (h >> 16);
    return h;
  }
};

// Count-min sketch with saturating cells. A key touches `depth` cells of ONE row of `width` cells:
// cell j is (h + j * step) mod width with h = hash(key) and step = h rotated right by 17 bits (double
// hashing), which is also what the device kernels k_countmin_* compute.
template <typename K, typename V>
class CountMin : public Sketch {
 public:
  static constexpr int kMinWidth = 64, kMaxDepth = 30;
  bool empty() const { return width_ == 0; }
  void clear() { cells_.clear(); width_ = 0; }
  void resize(int width, int depth, V ceiling) {
    width_ = width < kMinWidth ? kMinWidth : width;
    depth_ = depth < 1 ? 1 : (depth > kMaxDepth ? kMaxDepth : depth);
    ceiling_ = ceiling;
    cells_.resize(width_);
    cells_.SetZero();
  }
  void insert(const K& key, const V& count) {
    for (Walk w(hash(key)); w.index < depth_; w.next()) {
      V& c = cells_[w.pos % width_];
      const V room = ceiling_ - c;
      c = count > room ? ceiling_ : (V)(c + count);
    }
  }
  V query(const K& key) const {
    V lowest = ceiling_;
    for (Walk w(hash(key)); w.index < depth_; w.next()) {
      const V c = cells_[w.pos % width_];
      if (c < lowest) lowest = c;
    }
    return lowest;
  }
  const SArray<V>& data() const { return cells_; }
 private:
  struct Walk {
    explicit Walk(uint32_t h) : pos(h), step((h >> 17) | (h << 15)) {}
    void next() { pos += step; ++index; }
    uint32_t pos, step;
    int index = 0;
  };
  SArray<V> cells_;
  int width_ = 0, depth_ = 1;
  V ceiling_ = 0;
};

template <typename K>
class BloomFilter : public Sketch {
 public:
  BloomFilter() {}
  BloomFilter(int m, int k) { resize(m, k); }
  void resize(int m, int k) {
    k_ = std::min(64, std::max(1, k));
    m_ = m;
    data_.assign((m + 7) / 8, 0);
  }
  bool operator[](K key) const { return query(key); }
  bool query(K key) const {
    uint32_t h = hash(key);
    const uint32_t delta = (h >> 17) | (h << 15);
    for (int j = 0; j < k_; ++j) {
      uint32_t pos = h % m_;
      if ((data_[pos / 8] & (1 << (pos % 8))) == 0) return false;
      h += delta;
    }
    return true;
  }
  void insert(K key) {
    uint32_t h = hash(key);
    const uint32_t delta = (h >> 17) | (h << 15);
    for (int j = 0; j < k_; ++j) { uint32_t pos = h % m_; data_[pos / 8] |= (1 << (pos % 8)); h += delta; }
  }
 private:
  std::vector<uint8_t> data_;
  uint32_t m_ = 0;
  int k_ = 0;
};

// All k probes of a key land in one 64-byte bin (one cache line).
template <typename K>
class BlockBloomFilter : public Sketch {
 public:
  BlockBloomFilter() {}
  BlockBloomFilter(size_t n, int k) { resize(n, k); }
  void resize(size_t n, int k) {
    k_ = std::min(64, std::max(1, k));
    num_bin_ = (n / 8 / kBinBytes) + 1;
    data_.assign(num_bin_ * kBinBytes, 0);
  }
  bool operator[](K key) const { return query(key); }
  bool query(K key) const {
    uint32_t h = hash(key);
    const uint8_t* bin = &data_[(size_t)(h % num_bin_) * kBinBytes];
    const uint32_t delta = (h >> 17) | (h << 15);
    for (int j = 0; j < k_; ++j) {
      h += delta;
      uint32_t pos = h % (kBinBytes * 8);
      if ((bin[pos / 8] & (1 << (pos % 8))) == 0) return false;
    }
    return true;
  }
  void insert(K key) {
    uint32_t h = hash(key);
    uint8_t* bin = &data_[(size_t)(h % num_bin_) * kBinBytes];
    const uint32_t delta = (h >> 17) | (h << 15);
    for (int j = 0; j < k_; ++j) { h += delta; uint32_t pos = h % (kBinBytes * 8); bin[pos / 8] |= (1 << (pos % 8)); }
  }
 private:
  static const uint32_t kBinBytes = 64;
  std::vector<uint8_t> data_;
  uint32_t num_bin_ = 0;
  int k_ = 0;
};

// Bit set over 16-bit words with a population-count table (Darlin active set).
class Bitmap {
 public:
  Bitmap() {}
  explicit Bitmap(uint32_t size, bool value = false) { resize(size, value); }
  void resize(uint32_t size, bool value = false) {
    size_ = size;
    map_.assign((size >> 4) + 1, value ? 0xFFFF : 0);
  }
  void clear() { map_.clear(); size_ = 0; }
  void set(uint32_t i) { map_[i >> 4] |= (uint16_t)(1u << (i & 15)); }
  void clear(uint32_t i) { map_[i >> 4] &= (uint16_t)~(1u << (i & 15)); }
  bool test(uint32_t i) const { return (map_[i >> 4] >> (i & 15)) & 1; }
  bool operator[](uint32_t i) const { return test(i); }
  void fill(bool value) { std::fill(map_.begin(), map_.end(), value ? 0xFFFF : 0); }
  uint32_t size() const { return size_; }
  size_t memSize() const { return map_.size() * 2; }
  uint32_t nnz() const {
    static const std::vector<uint8_t> lut = [] {
      std::vector<uint8_t> t(65536);
      for (uint32_t i = 0; i < 65536; ++i) t[i] = (uint8_t)__builtin_popcount(i);
      return t;
    }();
    if (size_ == 0) return 0;
    uint32_t v = 0, full = size_ >> 4;
    for (uint32_t i = 0; i < full; ++i) v += lut[map_[i]];
    uint32_t rem = size_ & 15;
    if (rem) v += lut[map_[full] & ((1u << rem) - 1)];
    return v;
  }
 private:
  std::vector<uint16_t> map_;
  uint32_t size_ = 0;
};

}  // namespace PS
