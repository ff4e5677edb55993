// SArray<V>: reference-counted typed view of a byte buffer. Copies share memory;
// a view can be reinterpreted as another element type or cut into segments
// without copying, which is how message payloads travel through the runtime.
// Counterpart of util/shared_array.h:29-293 / shared_array_inl.h:10-263.
#pragma once
#include <zlib.h>
#include <algorithm>
#include <random>
#include "common.h"
#include "range.h"

namespace PS {

struct ParamInit {  // parameter/proto/param.proto ParamInitConfig
  enum Type { ZERO = 0, CONSTANT = 1, GAUSSIAN = 2, FILE = 3, CLONE = 4 };
  Type type = ZERO;
  double constant = 1.0;
  double mean = 0.0;
  double std = 1.0;
  std::string file_name;
};

template <typename V>
class SArray {
 public:
  SArray() {}
  explicit SArray(size_t n) { resize(n); }
  SArray(size_t n, V val) { resize(n); SetValue(val); }
  SArray(const std::initializer_list<V>& l) { CopyFrom(l.begin(), l.size()); }
  explicit SArray(const std::vector<V>& v) { CopyFrom(v.data(), v.size()); }
  // take ownership of `data` (freed with `deleter`, default delete[])
  SArray(V* data, size_t n, std::function<void(V*)> deleter = nullptr) { reset(data, n, deleter); }
  // zero-copy reinterpretation of another element type
  template <typename W>
  explicit SArray(const SArray<W>& o) { *this = o; }
  template <typename W>
  void operator=(const SArray<W>& o) {
    size_ = o.size() * sizeof(W) / sizeof(V);
    capacity_ = o.capacity() * sizeof(W) / sizeof(V);
    ptr_ = std::shared_ptr<char>(o.pointer(), reinterpret_cast<char*>(o.data()));
    data_ = reinterpret_cast<V*>(o.data());
  }

  void reset(V* data, size_t n, std::function<void(V*)> deleter = nullptr) {
    size_ = capacity_ = n;
    data_ = data;
    if (deleter) {
      ptr_ = std::shared_ptr<char>(reinterpret_cast<char*>(data),
                                   [deleter](char* p) { deleter(reinterpret_cast<V*>(p)); });
    } else {
      ptr_ = std::shared_ptr<char>(reinterpret_cast<char*>(data), [](char* p) { delete[] reinterpret_cast<V*>(p); });
    }
  }
  // view of memory owned elsewhere (no deletion)
  static SArray<V> Wrap(V* data, size_t n) {
    SArray<V> a;
    a.size_ = a.capacity_ = n;
    a.data_ = data;
    a.ptr_ = std::shared_ptr<char>(reinterpret_cast<char*>(data), [](char*) {});
    return a;
  }
  void CopyFrom(const V* src, size_t n) {
    resize(n);
    if (n) memcpy(data_, src, n * sizeof(V));
  }
  void CopyFrom(const SArray<V>& o) { if (this != &o) CopyFrom(o.data(), o.size()); }
  SArray<V> Clone() const { SArray<V> a; a.CopyFrom(*this); return a; }

  void resize(size_t n) {
    if (n <= capacity_) { size_ = n; return; }
    V* nd = new V[n + 5];
    if (size_) memcpy(nd, data_, size_ * sizeof(V));
    size_t old = size_;
    reset(nd, n);
    (void)old;
  }
  void reserve(size_t n) {
    if (n <= capacity_) return;
    size_t s = size_;
    resize(n);
    size_ = s;
  }
  void clear() { ptr_.reset(); data_ = nullptr; size_ = capacity_ = 0; }
  void push_back(const V& v) {
    if (size_ == capacity_) reserve(std::max<size_t>(16, size_ * 2));
    data_[size_++] = v;
  }
  void pop_back() { if (size_) --size_; }
  void append(const SArray<V>& o) {
    if (o.empty()) return;
    size_t s = size_;
    reserve(s + o.size());
    size_ = s + o.size();
    memcpy(data_ + s, o.data(), o.size() * sizeof(V));
  }

  bool empty() const { return size_ == 0; }
  size_t size() const { return size_; }
  size_t capacity() const { return capacity_; }
  size_t memSize() const { return size_ * sizeof(V); }
  V* data() const { return data_; }
  V* begin() const { return data_; }
  V* end() const { return data_ + size_; }
  const std::shared_ptr<char>& pointer() const { return ptr_; }
  V& operator[](size_t i) const { return data_[i]; }
  V& front() const { return data_[0]; }
  V& back() const { return data_[size_ - 1]; }

  // zero-copy slice [range.begin, range.end)
  SArray<V> Segment(const SizeR& range) const {
    PS_CHECK(range.valid());
    PS_CHECK_LE(range.end(), size_);
    SArray<V> a;
    a.ptr_ = std::shared_ptr<char>(ptr_, reinterpret_cast<char*>(data_ + range.begin()));
    a.data_ = data_ + range.begin();
    a.size_ = a.capacity_ = range.size();
    return a;
  }
  // index range of a *sorted* array whose values fall in `bound`
  template <typename K>
  SizeR FindRange(const Range<K>& bound) const {
    if (empty()) return SizeR(0, 0);
    PS_CHECK(bound.valid());
    auto lb = std::lower_bound(begin(), end(), static_cast<V>(bound.begin()));
    auto ub = std::lower_bound(begin(), end(), static_cast<V>(bound.end()));
    return SizeR(lb - begin(), ub - begin());
  }
  // sorted-set operations
  SArray<V> SetIntersection(const SArray<V>& o) const {
    SArray<V> r(std::min(size(), o.size()) + 1);
    V* e = std::set_intersection(begin(), end(), o.begin(), o.end(), r.begin());
    r.size_ = e - r.begin();
    return r;
  }
  SArray<V> SetUnion(const SArray<V>& o) const {
    SArray<V> r(size() + o.size() + 1);
    V* e = std::set_union(begin(), end(), o.begin(), o.end(), r.begin());
    r.size_ = e - r.begin();
    return r;
  }

  void SetValue(V v) { std::fill(begin(), end(), v); }
  void SetZero() { if (size_) memset(data_, 0, size_ * sizeof(V)); }
  void SetValue(const ParamInit& c) {
    if (c.type == ParamInit::ZERO) { SetZero(); }
    else if (c.type == ParamInit::CONSTANT) { SetValue(static_cast<V>(c.constant)); }
    else if (c.type == ParamInit::GAUSSIAN) {
      std::mt19937_64 gen(20141010);
      std::normal_distribution<double> d(c.mean, c.std);
      for (size_t i = 0; i < size_; ++i) data_[i] = static_cast<V>(d(gen));
    } else if (c.type == ParamInit::FILE) {
      PS_CHECK(ReadFromFile(c.file_name)) << "cannot read " << c.file_name;
    } else { PS_CHECK(false) << "unsupported init type " << c.type; }
  }
  size_t nnz() const { size_t n = 0; for (size_t i = 0; i < size_; ++i) n += data_[i] != 0; return n; }
  double Sum() const { double s = 0; for (size_t i = 0; i < size_; ++i) s += data_[i]; return s; }
  bool operator==(const SArray<V>& o) const {
    return size_ == o.size_ && (size_ == 0 || memcmp(data_, o.data_, size_ * sizeof(V)) == 0);
  }

  // lossless byte compression (zlib deflate); the wire-format of CompressingFilter
  SArray<char> CompressTo() const {
    uLongf cap = compressBound(memSize());
    SArray<char> out(cap);
    PS_CHECK_EQ(compress2(reinterpret_cast<Bytef*>(out.data()), &cap, reinterpret_cast<const Bytef*>(data_),
                          memSize(), Z_BEST_SPEED), Z_OK);
    out.resize(cap);
    return out;
  }
  void UncompressFrom(const char* src, size_t src_size) {
    uLongf dst = memSize();
    PS_CHECK_EQ(uncompress(reinterpret_cast<Bytef*>(data_), &dst, reinterpret_cast<const Bytef*>(src), src_size), Z_OK);
    PS_CHECK_EQ(dst, memSize());
  }
  void UncompressFrom(const SArray<char>& src) { UncompressFrom(src.data(), src.size()); }

  // raw binary file io
  bool WriteToFile(const std::string& file) const { return WriteToFile(SizeR(0, size_), file); }
  bool WriteToFile(SizeR range, const std::string& file) const {
    FILE* f = fopen(file.c_str(), "wb");
    if (!f) return false;
    size_t n = fwrite(data_ + range.begin(), sizeof(V), range.size(), f);
    fclose(f);
    return n == range.size();
  }
  bool ReadFromFile(const std::string& file) {
    FILE* f = fopen(file.c_str(), "rb");
    if (!f) return false;
    fseek(f, 0, SEEK_END);
    long bytes = ftell(f);
    fseek(f, 0, SEEK_SET);
    resize(bytes / sizeof(V));
    size_t n = fread(data_, sizeof(V), size_, f);
    fclose(f);
    return n == size_;
  }
  bool ReadFromFile(SizeR range, const std::string& file) {
    FILE* f = fopen(file.c_str(), "rb");
    if (!f) return false;
    fseek(f, range.begin() * sizeof(V), SEEK_SET);
    resize(range.size());
    size_t n = fread(data_, sizeof(V), size_, f);
    fclose(f);
    return n == size_;
  }
  std::vector<V> ToVector() const { return std::vector<V>(begin(), end()); }

 private:
  size_t size_ = 0, capacity_ = 0;
  V* data_ = nullptr;
  std::shared_ptr<char> ptr_;
};

template <typename V>
std::ostream& operator<<(std::ostream& os, const SArray<V>& a) {
  os << "[" << a.size() << "]{";
  for (size_t i = 0; i < std::min<size_t>(a.size(), 10); ++i) os << (i ? "," : "") << a[i];
  return os << (a.size() > 10 ? ",...}" : "}");
}

}  // namespace PS
