// AssignOp, ordered merge-join of sorted key arrays with value widths, parallel
// merge sort. Counterparts: util/assign_op.h:9-50,
// util/parallel_ordered_match.h:7-112, util/parallel_sort.h:14-41.
#pragma once
#include <algorithm>
#include "sarray.h"
#include "threading.h"

namespace PS {

enum class AssignOp : int { ASSIGN = 0, PLUS = 1, MINUS = 2, TIMES = 3, DIVIDE = 4, AND = 5, OR = 6, XOR = 7 };

template <typename T>
inline void AssignFunc(T& dst, const T& src, AssignOp op) {
  switch (op) {
    case AssignOp::ASSIGN: dst = src; break;
    case AssignOp::PLUS: dst += src; break;
    case AssignOp::MINUS: dst -= src; break;
    case AssignOp::TIMES: dst *= src; break;
    case AssignOp::DIVIDE: dst /= src; break;
    default:
      if constexpr (std::is_integral<T>::value) {
        if (op == AssignOp::AND) dst &= src;
        else if (op == AssignOp::OR) dst |= src;
        else if (op == AssignOp::XOR) dst ^= src;
      } else {
        PS_CHECK(false) << "bit operations need an integral type";
      }
  }
}

namespace detail {
// join src (keys+values) into dst by walking both sorted key lists; `grain` bounds
// the work below which no more threads are forked
template <typename K, typename V>
void MatchRange(const K* src_key, const K* src_key_end, const V* src_val, const K* dst_key,
                const K* dst_key_end, V* dst_val, int k, AssignOp op, size_t grain, size_t* n) {
  size_t src_len = src_key_end - src_key, dst_len = dst_key_end - dst_key;
  if (dst_len == 0 || src_len == 0) return;
  // clip src to the key span of dst
  src_key_end = std::upper_bound(src_key, src_key_end, *(dst_key_end - 1));
  const K* clipped = std::lower_bound(src_key, src_key_end, *dst_key);
  src_val += (clipped - src_key) * k;
  src_key = clipped;
  src_len = src_key_end - src_key;
  if (src_len == 0) return;
  if (grain >= dst_len + src_len || dst_len < 2) {
    size_t hits = 0;
    while (dst_key != dst_key_end && src_key != src_key_end) {
      if (*src_key < *dst_key) { ++src_key; src_val += k; }
      else {
        if (!(*dst_key < *src_key)) {
          for (int i = 0; i < k; ++i) AssignFunc(dst_val[i], src_val[i], op);
          ++src_key; src_val += k; ++hits;
        }
        ++dst_key; dst_val += k;
      }
    }
    *n += hits;
    return;
  }
  size_t half = dst_len / 2;
  size_t n_left = 0, n_right = 0;
  std::thread thr([&] {
    MatchRange(src_key, src_key_end, src_val, dst_key, dst_key + half, dst_val, k, op, grain, &n_left);
  });
  MatchRange(src_key, src_key_end, src_val, dst_key + half, dst_key_end, dst_val + half * k, k, op, grain, &n_right);
  thr.join();
  *n += n_left + n_right;
}
}  // namespace detail

// dst_val[j] op= src_val[i] for every pair with src_key[i] == dst_key[j]; both key
// arrays sorted and unique, values k wide. Returns the number of matched keys.
template <typename K, typename V>
size_t ParallelOrderedMatch(const SArray<K>& src_key, const SArray<V>& src_val, const SArray<K>& dst_key,
                            SArray<V>* dst_val, int k = 1, AssignOp op = AssignOp::ASSIGN, int num_threads = 2) {
  if (dst_key.empty()) return 0;
  PS_CHECK_GT(num_threads, 0);
  PS_CHECK_EQ(src_key.size() * k, src_val.size());
  if (dst_val->size() != dst_key.size() * k) {
    dst_val->resize(dst_key.size() * k);
    dst_val->SetZero();
  }
  SizeR range = dst_key.FindRange(Range<K>(src_key.empty() ? 0 : src_key.front(),
                                           src_key.empty() ? 0 : src_key.back() + 1));
  (void)range;
  size_t grain = std::max<size_t>((src_key.size() + dst_key.size()) / num_threads, 1 << 20);
  size_t n = 0;
  detail::MatchRange<K, V>(src_key.begin(), src_key.end(), src_val.begin(), dst_key.begin(), dst_key.end(),
                           dst_val->begin(), k, op, grain, &n);
  return n;
}

// union of two sorted key arrays with their values joined by `op`
template <typename K, typename V>
void ParallelUnion(const SArray<K>& key1, const SArray<V>& val1, const SArray<K>& key2, const SArray<V>& val2,
                   SArray<K>* joined_key, SArray<V>* joined_val, int k = 1, AssignOp op = AssignOp::PLUS,
                   int num_threads = 2) {
  *joined_key = key1.SetUnion(key2);
  joined_val->clear();
  ParallelOrderedMatch(key1, val1, *joined_key, joined_val, k, AssignOp::ASSIGN, num_threads);
  ParallelOrderedMatch(key2, val2, *joined_key, joined_val, k, op, num_threads);
}

namespace detail {
template <typename T, class Fn>
void MergeSortRange(T* data, size_t len, size_t grain, const Fn& cmp) {
  if (len <= grain) { std::sort(data, data + len, cmp); return; }
  std::thread thr([&] { MergeSortRange(data, len / 2, grain, cmp); });
  MergeSortRange(data + len / 2, len - len / 2, grain, cmp);
  thr.join();
  std::inplace_merge(data, data + len / 2, data + len, cmp);
}
}  // namespace detail

template <typename T, class Fn>
void ParallelSort(T* data, size_t len, size_t num_threads, const Fn& cmp) {
  size_t grain = std::max<size_t>(len / std::max<size_t>(num_threads, 1) + 5, 1024 * 16);
  detail::MergeSortRange(data, len, grain, cmp);
}
template <typename T, class Fn>
void ParallelSort(SArray<T>* arr, size_t num_threads, const Fn& cmp) {
  ParallelSort(arr->data(), arr->size(), num_threads, cmp);
}

}  // namespace PS
