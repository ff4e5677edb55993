// Message filters: per-peer codecs applied in list order on send and in reverse
// order on receive. Counterparts: filter/filter.h:9-24, filter/filter.cc:9-31,
// filter/key_caching.h:9-76, filter/compressing.h:6-38,
// filter/fixing_float.h:6-103, filter/add_noise.h:9-41,
// filter/sparse_filter.h:5-24, filter/frequency_filter.h:11-65.
#pragma once
#include <cmath>
#include <limits>
#include <random>
#include "hash.h"
#include "message.h"
#include "sketch.h"

namespace PS {

class Filter {
 public:
  virtual ~Filter() {}
  static Filter* create(const FilterConfig& conf);
  virtual void encode(Message* msg) {}
  virtual void decode(Message* msg) {}
  // the mutable config of `type` inside the task header (filters stash runtime
  // fields there: signature, sizes, min/max), or null
  static FilterConfig* find(FilterConfig::Type type, Task* task) {
    for (auto& f : task->filter) if (f.type == type) return &f;
    return nullptr;
  }
  static FilterConfig* find(FilterConfig::Type type, Message* msg) { return find(type, &msg->task); }
};

// Key caching. One remembered key list per (key channel, key range) of a peer.
//   sending:   the list's signature always travels in the filter header; when the remembered list of
//              the slot has the same signature and byte length (and is not empty) the keys themselves
//              are left out of the message, otherwise the slot remembers the new list.
//   receiving: a message with keys refreshes the slot; one without takes the slot's keys back in.
// The signature is crc32c over the first kSignedBytes bytes of the list. With clear_cache_if_done
// a slot is dropped once the exchange it served is over (a response, or a push request).
class KeyCachingFilter : public Filter {
 public:
  static constexpr size_t kSignedBytes = 2048;

  void encode(Message* msg) override {
    FilterConfig* hdr = find(FilterConfig::KEY_CACHING, msg);
    if (hdr == nullptr) return;
    hdr->has_signature = msg->task.has_key;
    if (!msg->task.has_key) return;
    hdr->signature = Signature(msg->key);
    Lock l(mu_);
    const SlotId id = IdOf(msg->task);
    Slot& slot = slots_[id];
    if (!msg->key.empty() && slot.Matches(hdr->signature, msg->key.size())) msg->clear_key();
    else slot.Remember(hdr->signature, msg->key);
    Retire(*hdr, msg->task, id);
  }

  void decode(Message* msg) override {
    FilterConfig* hdr = find(FilterConfig::KEY_CACHING, msg);
    if (hdr == nullptr || !hdr->has_signature) return;
    Lock l(mu_);
    const SlotId id = IdOf(msg->task);
    Slot& slot = slots_[id];
    if (msg->task.has_key) {
      PS_CHECK_EQ(Signature(msg->key), hdr->signature);
      slot.Remember(hdr->signature, msg->key);
    } else {
      PS_CHECK_EQ(hdr->signature, slot.signature) << "key cache miss on " << msg->ShortDebugString();
      msg->key = slot.keys;
      msg->task.has_key = true;
    }
    Retire(*hdr, msg->task, id);
  }

  size_t cache_entries() const { return slots_.size(); }

 private:
  typedef std::pair<int, Range<Key>> SlotId;
  struct Slot {
    uint32_t signature = 0;
    SArray<char> keys;
    bool Matches(uint32_t sig, size_t bytes) const { return signature == sig && keys.size() == bytes; }
    void Remember(uint32_t sig, const SArray<char>& k) { signature = sig; keys = k; }
  };
  struct SlotIdHash {
    size_t operator()(const SlotId& k) const { return k.first * 7919u ^ k.second.Hash(); }
  };
  static uint32_t Signature(const SArray<char>& keys) {
    return crc32c::Value(keys.data(), keys.size() < kSignedBytes ? keys.size() : kSignedBytes);
  }
  static SlotId IdOf(const Task& t) { return SlotId(t.key_channel, t.key_range); }
  void Retire(const FilterConfig& hdr, const Task& t, const SlotId& id) {
    const bool exchange_over = !t.request || (t.has_param && t.param.push);
    if (hdr.clear_cache_if_done && exchange_over) slots_.erase(id);
  }
  std::unordered_map<SlotId, Slot, SlotIdHash> slots_;
  std::mutex mu_;
};

// Lossless byte compression of the key and every value array.
class CompressingFilter : public Filter {
 public:
  void encode(Message* msg) override {
    auto conf = find(FilterConfig::COMPRESSING, msg);
    if (!conf) return;
    conf->uncompressed_size.clear();
    if (msg->has_key()) {
      conf->uncompressed_size.push_back(msg->key.size());
      msg->key = msg->key.CompressTo();
    }
    for (auto& v : msg->value) {
      conf->uncompressed_size.push_back(v.size());
      if (!v.empty()) v = v.CompressTo();
    }
  }
  void decode(Message* msg) override {
    auto conf = find(FilterConfig::COMPRESSING, msg);
    if (!conf) return;
    size_t has_key = msg->has_key();
    PS_CHECK_EQ(conf->uncompressed_size.size(), msg->value.size() + has_key);
    if (has_key) {
      SArray<char> raw(conf->uncompressed_size[0]);
      raw.UncompressFrom(msg->key);
      msg->key = raw;
    }
    for (size_t i = 0; i < msg->value.size(); ++i) {
      SArray<char> raw(conf->uncompressed_size[i + has_key]);
      if (raw.size()) raw.UncompressFrom(msg->value[i]);
      msg->value[i] = raw;
    }
  }
};

// Lossy fixed-point codec of float/double value arrays: clamp into [min,max],
// map to an unsigned integer of num_bytes bytes with a random-bit rounding,
// little-endian. min/max come from the config or from the data.
class FixingFloatFilter : public Filter {
 public:
  void encode(Message* msg) override { convert(msg, true); }
  void decode(Message* msg) override { convert(msg, false); }
  // deterministic rounding source for tests
  void set_seed(unsigned s) { seed_ = s; fixed_seed_ = true; }
 private:
  // linear-congruential coin flip
  static int boolrand(unsigned* seed) {
    *seed = (214013u * *seed + 2531011u);
    return (*seed >> 16) & 0x1;
  }
  void convert(Message* msg, bool encode) {
    auto conf = find(FilterConfig::FIXING_FLOAT, msg);
    if (!conf) return;
    int n = (int)msg->value.size();
    PS_CHECK_EQ(n, (int)msg->task.value_type.size());
    int k = 0;
    for (int i = 0; i < n; ++i) {
      if (msg->value[i].empty()) continue;
      auto type = msg->task.value_type[i];
      if (type != DataType::FLOAT && type != DataType::DOUBLE) continue;
      if ((int)conf->fixed_point.size() <= k) conf->fixed_point.resize(k + 1);
      auto* fc = &conf->fixed_point[k++];
      if (type == DataType::FLOAT) msg->value[i] = codec<float>(msg->value[i], encode, conf->num_bytes, fc);
      else msg->value[i] = codec<double>(msg->value[i], encode, conf->num_bytes, fc);
    }
  }
  template <typename V>
  SArray<char> codec(const SArray<char>& array, bool encode, int nbytes, FilterConfig::FixedFloat* fc) {
    PS_CHECK_GT(nbytes, 0);
    PS_CHECK_LT(nbytes, 8);
    const double ratio = static_cast<double>(1ull << (nbytes * 8)) - 2;
    if (encode) {
      SArray<V> orig(array);
      if (!fc->has_min) { fc->min_value = (float)*std::min_element(orig.begin(), orig.end()); fc->has_min = true; }
      if (!fc->has_max) { fc->max_value = (float)(*std::max_element(orig.begin(), orig.end()) + 1e-6); fc->has_max = true; }
    }
    PS_CHECK(fc->has_min && fc->has_max);
    const double lo = fc->min_value, hi = fc->max_value, bin = hi - lo;
    PS_CHECK_GT(bin, 0.0);
    if (encode) {
      SArray<V> orig(array);
      SArray<uint8_t> code(orig.size() * nbytes);
      uint8_t* out = code.data();
      unsigned seed = fixed_seed_ ? seed_ : (unsigned)time(NULL);
      for (size_t i = 0; i < orig.size(); ++i) {
        double x = orig[i] > hi ? hi : (orig[i] < lo ? lo : (double)orig[i]);
        uint64_t r = static_cast<uint64_t>(std::floor((x - lo) / bin * ratio)) + boolrand(&seed);
        for (int j = 0; j < nbytes; ++j) { *out++ = (uint8_t)(r & 0xFF); r >>= 8; }
      }
      return SArray<char>(code);
    }
    SArray<uint8_t> code(array);
    SArray<V> orig(code.size() / nbytes);
    const uint8_t* in = code.data();
    for (size_t i = 0; i < orig.size(); ++i) {
      uint64_t r = 0;
      for (int j = 0; j < nbytes; ++j) r += (uint64_t)(*in++) << (8 * j);
      orig[i] = static_cast<V>((double)r / ratio * bin + lo);
    }
    return SArray<char>(orig);
  }
  unsigned seed_ = 0;
  bool fixed_seed_ = false;
};

// Adds N(mean, std) noise to float/double values on send.
class AddNoiseFilter : public Filter {
 public:
  void encode(Message* msg) override {
    auto conf = find(FilterConfig::NOISE, msg);
    if (!conf) return;
    int n = (int)msg->value.size();
    PS_CHECK_EQ(n, (int)msg->task.value_type.size());
    for (int i = 0; i < n; ++i) {
      if (msg->value[i].empty()) continue;
      auto type = msg->task.value_type[i];
      if (type == DataType::FLOAT) add<float>(msg->value[i], conf);
      else if (type == DataType::DOUBLE) add<double>(msg->value[i], conf);
    }
  }
 private:
  template <typename V>
  void add(const SArray<char>& array, FilterConfig* conf) {
    std::normal_distribution<V> dist((V)conf->mean, (V)conf->std);
    SArray<V> data(array);
    for (size_t i = 0; i < data.size(); ++i) data[i] += dist(gen_);
  }
  std::default_random_engine gen_;
};

inline Filter* Filter::create(const FilterConfig& conf) {
  switch (conf.type) {
    case FilterConfig::KEY_CACHING: return new KeyCachingFilter();
    case FilterConfig::COMPRESSING: return new CompressingFilter();
    case FilterConfig::FIXING_FLOAT: return new FixingFloatFilter();
    case FilterConfig::NOISE: return new AddNoiseFilter();
  }
  PS_CHECK(false) << "unknown filter type " << conf.type;
  return nullptr;
}

// Marks "this coordinate is inactive" inside value arrays with an all-ones bit
// pattern (a NaN), used by Darlin's KKT filter.
class SparseFilter {
 public:
  SparseFilter() { memset(&float_v_, 0xff, sizeof(float)); memset(&double_v_, 0xff, sizeof(double)); }
  void mark(float* v) const { *v = float_v_; }
  void mark(double* v) const { *v = double_v_; }
  bool marked(double v) const { return v != v; }
  bool marked(float v) const { return v != v; }
 private:
  float float_v_;
  double double_v_;
};

// Count-min based frequency filter (tail-feature filtering).
template <typename K, typename V>
class FreqencyFilter {
 public:
  void Resize(int n, int k) { cm_.resize(n, k, std::numeric_limits<V>::max()); }
  bool Empty() const { return cm_.empty(); }
  void Clear() { cm_.clear(); }
  void InsertKeys(const SArray<K>& key, const SArray<V>& count) {
    PS_CHECK_EQ(key.size(), count.size());
    for (size_t i = 0; i < key.size(); ++i) cm_.insert(key[i], count[i]);
  }
  // keys whose estimated count is greater than freq_thr
  SArray<K> QueryKeys(const SArray<K>& key, int freq_thr) const {
    PS_CHECK_LT(freq_thr, (int)std::numeric_limits<V>::max()) << "change V to a wider type";
    SArray<K> out;
    for (size_t i = 0; i < key.size(); ++i) if ((int)cm_.query(key[i]) > freq_thr) out.push_back(key[i]);
    return out;
  }
 private:
  CountMin<K, V> cm_;
};

}  // namespace PS
