// Half-open interval [begin, end) over keys or indices.
// Counterpart of util/range.h:10-131; EvenDivide reproduces the reference's
// long-double arithmetic (util/range.h:99-107) because it defines which server
// owns which key.
#pragma once
#include "common.h"

namespace PS {

template <typename T>
class Range {
 public:
  Range() : begin_(0), end_(0) {}
  Range(T b, T e) : begin_(b), end_(e) {}
  template <typename U>
  explicit Range(const Range<U>& o) : begin_(static_cast<T>(o.begin())), end_(static_cast<T>(o.end())) {}
  static Range All() { return Range(0, static_cast<T>(-1)); }

  T begin() const { return begin_; }
  T end() const { return end_; }
  T& begin() { return begin_; }
  T& end() { return end_; }
  void Set(T b, T e) { begin_ = b; end_ = e; }
  size_t size() const { return static_cast<size_t>(end_ - begin_); }
  bool valid() const { return end_ >= begin_; }
  bool empty() const { return begin_ >= end_; }
  bool operator==(const Range& o) const { return begin_ == o.begin_ && end_ == o.end_; }
  bool operator!=(const Range& o) const { return !(*this == o); }
  Range operator+(T v) const { return Range(begin_ + v, end_ + v); }
  Range operator-(T v) const { return Range(begin_ - v, end_ - v); }
  Range operator*(T v) const { return Range(begin_ * v, end_ * v); }
  bool contains(T v) const { return begin_ <= v && v < end_; }
  bool contains(const Range& o) const { return begin_ <= o.begin_ && o.end_ <= end_; }
  bool InLeft(const Range& o) const { return begin_ <= o.begin_ && end_ <= o.end_; }
  bool InRight(const Range& o) const { return !InLeft(o); }
  // clamp v into [begin, end]
  T Project(T v) const { return v < begin_ ? begin_ : (v > end_ ? end_ : v); }
  Range SetIntersection(const Range& o) const {
    return Range(std::max(begin_, o.begin_), std::min(end_, o.end_));
  }
  Range SetUnion(const Range& o) const {
    return Range(std::min(begin_, o.begin_), std::max(end_, o.end_));
  }
  // i-th of n equal parts
  Range EvenDivide(size_t n, size_t i) const {
    PS_CHECK(valid());
    PS_CHECK_GT(n, (size_t)0);
    PS_CHECK_LT(i, n);
    long double step = static_cast<long double>(end_ - begin_) / static_cast<long double>(n);
    // the last part ends exactly at end_ (the rounded product may exceed the type's range)
    T hi = (i + 1 == n) ? end_ : static_cast<T>(begin_ + step * (i + 1));
    return Range(static_cast<T>(begin_ + step * i), hi);
  }
  std::string ToString() const {
    std::ostringstream ss;
    ss << "[" << begin_ << "," << end_ << ")";
    return ss.str();
  }
  size_t Hash() const { return std::hash<T>()(begin_) * 1000003u ^ std::hash<T>()(end_); }

 private:
  T begin_, end_;
};

typedef Range<size_t> SizeR;
template <typename T>
std::ostream& operator<<(std::ostream& os, const Range<T>& r) { return os << r.ToString(); }

}  // namespace PS

namespace std {
template <typename T>
struct hash<PS::Range<T>> {
  size_t operator()(const PS::Range<T>& r) const { return r.Hash(); }
};
}  // namespace std
