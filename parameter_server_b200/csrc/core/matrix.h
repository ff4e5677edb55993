// Matrices of the CPU path: CSR/CSC sparse matrix (binary matrices carry no
// value array), dense matrix, and the minibatch localizer.
// Counterparts: util/matrix.h:29-125, util/sparse_matrix.h:23-241,
// util/dense_matrix.h:7-104, util/localizer.h:14-221, util/proto/matrix.proto:4-28.
#pragma once
#include <cmath>
#include <numeric>
#include "ordered_match.h"
#include "sarray.h"
#include "threading.h"

namespace PS {

struct MatrixInfo {
  enum Type { DENSE = 1, SPARSE = 2, SPARSE_BINARY = 3 };
  Type type = SPARSE;
  bool row_major = true;
  int id = 0;               // feature group
  SizeR row, col;           // global row / column ranges
  size_t nnz = 0;
  uint32_t sizeof_index = 0, sizeof_value = 0;
  double nnz_per_row = 0, nnz_per_col = 0;
  std::string DebugString() const {
    std::ostringstream ss;
    ss << (type == DENSE ? "DENSE" : type == SPARSE ? "SPARSE" : "SPARSE_BINARY") << (row_major ? " row-major" : " col-major")
       << " id " << id << " rows " << row.ToString() << " cols " << col.ToString() << " nnz " << nnz;
    return ss.str();
  }
};

template <typename V>
class Matrix {
 public:
  virtual ~Matrix() {}
  MatrixInfo& info() { return info_; }
  const MatrixInfo& info() const { return info_; }
  size_t rows() const { return info_.row.size(); }
  size_t cols() const { return info_.col.size(); }
  size_t nnz() const { return info_.nnz; }
  bool rowMajor() const { return info_.row_major; }
  bool colMajor() const { return !info_.row_major; }
  bool binary() const { return info_.type == MatrixInfo::SPARSE_BINARY; }
  bool empty() const { return nnz() == 0; }
  size_t innerSize() const { return rowMajor() ? cols() : rows(); }
  size_t outerSize() const { return rowMajor() ? rows() : cols(); }
  // header and the first entries, for logs (util/matrix.h:121, util/sparse_matrix.h:365-371)
  virtual std::string debugString() const { return info_.DebugString(); }
  // y = A x and y = A' x
  virtual void times(const V* x, V* y, int num_threads = 2) const = 0;
  virtual void transTimes(const V* x, V* y, int num_threads = 2) const = 0;
  SArray<V> times(const SArray<V>& x, int num_threads = 2) const {
    PS_CHECK_EQ(x.size(), cols());
    SArray<V> y(rows());
    times(x.data(), y.data(), num_threads);
    return y;
  }
  SArray<V> transTimes(const SArray<V>& x, int num_threads = 2) const {
    PS_CHECK_EQ(x.size(), rows());
    SArray<V> y(cols());
    transTimes(x.data(), y.data(), num_threads);
    return y;
  }
 protected:
  MatrixInfo info_;
};

template <typename V>
class DenseMatrix : public Matrix<V> {
 public:
  DenseMatrix() {}
  DenseMatrix(size_t rows, size_t cols, bool row_major = true) { resize(rows, cols, row_major); }
  void resize(size_t rows, size_t cols, bool row_major = true) {
    this->info_.type = MatrixInfo::DENSE;
    this->info_.row_major = row_major;
    this->info_.row = SizeR(0, rows);
    this->info_.col = SizeR(0, cols);
    this->info_.nnz = rows * cols;
    this->info_.sizeof_value = sizeof(V);
    value_.resize(rows * cols);
    value_.SetZero();
  }
  SArray<V>& value() { return value_; }
  const SArray<V>& value() const { return value_; }
  V& at(size_t r, size_t c) { return this->rowMajor() ? value_[r * this->cols() + c] : value_[c * this->rows() + r]; }
  std::string debugString() const override {
    std::ostringstream ss;
    ss << this->info_.DebugString() << "\nvalue: " << value_;
    return ss.str();
  }
  void times(const V* x, V* y, int = 2) const override {
    size_t R = this->rows(), C = this->cols();
    for (size_t r = 0; r < R; ++r) {
      V s = 0;
      for (size_t c = 0; c < C; ++c) s += (this->rowMajor() ? value_[r * C + c] : value_[c * R + r]) * x[c];
      y[r] = s;
    }
  }
  void transTimes(const V* x, V* y, int = 2) const override {
    size_t R = this->rows(), C = this->cols();
    for (size_t c = 0; c < C; ++c) y[c] = 0;
    for (size_t r = 0; r < R; ++r)
      for (size_t c = 0; c < C; ++c) y[c] += (this->rowMajor() ? value_[r * C + c] : value_[c * R + r]) * x[r];
  }
 private:
  SArray<V> value_;
};

// Compressed sparse storage; row-major = CSR, column-major = CSC.
template <typename I, typename V>
class SparseMatrix : public Matrix<V> {
 public:
  SparseMatrix() {}
  SparseMatrix(const MatrixInfo& info, SArray<size_t> offset, SArray<I> index, SArray<V> value)
      : offset_(offset), index_(index), value_(value) { this->info_ = info; }
  SArray<size_t>& offset() { return offset_; }
  SArray<I>& index() { return index_; }
  SArray<V>& value() { return value_; }
  const SArray<size_t>& offset() const { return offset_; }
  const SArray<I>& index() const { return index_; }
  const SArray<V>& value() const { return value_; }

  std::string debugString() const override {
    std::ostringstream ss;
    ss << this->info_.DebugString() << "\noffset: " << offset_ << "\nindex: " << index_;
    if (!this->binary()) ss << "\nvalue: " << value_;
    return ss.str();
  }

  using Matrix<V>::times;
  using Matrix<V>::transTimes;
  void times(const V* x, V* y, int num_threads = 2) const override { Mult(x, y, false, num_threads); }
  void transTimes(const V* x, V* y, int num_threads = 2) const override { Mult(x, y, true, num_threads); }

  // y[i] = sum_j A_ij^2 x_j (used for diagonal Hessians)
  void dotTimes(const V* x, V* y, bool trans) const {
    size_t outer = this->outerSize();
    bool gather = this->rowMajor() != trans;
    size_t ny = trans ? this->cols() : this->rows();
    if (!gather) for (size_t i = 0; i < ny; ++i) y[i] = 0;
    for (size_t o = 0; o < outer; ++o) {
      V s = 0;
      for (size_t j = offset_[o]; j < offset_[o + 1]; ++j) {
        V v = this->binary() ? 1 : value_[j];
        if (gather) s += v * v * x[index_[j]]; else y[index_[j]] += v * v * x[o];
      }
      if (gather) y[o] = s;
    }
  }

  // CSR <-> CSC by counting sort on the inner index
  std::shared_ptr<SparseMatrix<I, V>> alterStorage() const {
    size_t inner = this->innerSize(), outer = this->outerSize(), n = index_.size();
    SArray<size_t> off(inner + 1);
    off.SetZero();
    for (size_t j = 0; j < n; ++j) ++off[index_[j] + 1];
    for (size_t i = 0; i < inner; ++i) off[i + 1] += off[i];
    SArray<I> idx(n);
    SArray<V> val(this->binary() ? 0 : n);
    std::vector<size_t> cursor(off.begin(), off.begin() + inner);
    for (size_t o = 0; o < outer; ++o) {
      for (size_t j = offset_[o]; j < offset_[o + 1]; ++j) {
        size_t p = cursor[index_[j]]++;
        idx[p] = (I)o;
        if (!this->binary()) val[p] = value_[j];
      }
    }
    MatrixInfo info = this->info_;
    info.row_major = !info.row_major;
    return std::make_shared<SparseMatrix<I, V>>(info, off, idx, val);
  }
  std::shared_ptr<SparseMatrix<I, V>> toRowMajor() const {
    return this->rowMajor() ? std::make_shared<SparseMatrix<I, V>>(*this) : alterStorage();
  }
  std::shared_ptr<SparseMatrix<I, V>> toColMajor() const {
    return this->colMajor() ? std::make_shared<SparseMatrix<I, V>>(*this) : alterStorage();
  }
  // zero-copy block of outer slices [range)
  std::shared_ptr<SparseMatrix<I, V>> outerBlock(SizeR range) const {
    PS_CHECK_LE(range.end(), this->outerSize());
    MatrixInfo info = this->info_;
    (this->rowMajor() ? info.row : info.col) = range;
    size_t b = offset_[range.begin()], e = offset_[range.end()];
    info.nnz = e - b;
    // offsets stay absolute into the shared index/value arrays
    return std::make_shared<SparseMatrix<I, V>>(info, offset_.Segment(SizeR(range.begin(), range.end() + 1)),
                                                index_, value_);
  }
  std::shared_ptr<SparseMatrix<I, V>> rowBlock(SizeR range) const { PS_CHECK(this->rowMajor()); return outerBlock(range); }
  std::shared_ptr<SparseMatrix<I, V>> colBlock(SizeR range) const { PS_CHECK(this->colMajor()); return outerBlock(range); }

  bool writeToBinFile(const std::string& name) const {
    return offset_.WriteToFile(name + ".offset") && index_.WriteToFile(name + ".index") &&
           (this->binary() || value_.WriteToFile(name + ".value"));
  }

 private:
  void Mult(const V* x, V* y, bool trans, int num_threads) const {
    const bool gather = this->rowMajor() != trans;  // y[outer] = sum value * x[inner]
    const size_t outer = this->outerSize();
    const size_t ny = trans ? this->cols() : this->rows();
    num_threads = std::max(1, num_threads);
    if (gather) {
      auto work = [&](size_t b, size_t e) {
        for (size_t o = b; o < e; ++o) {
          V s = 0;
          if (this->binary()) for (size_t j = offset_[o]; j < offset_[o + 1]; ++j) s += x[index_[j]];
          else for (size_t j = offset_[o]; j < offset_[o + 1]; ++j) s += value_[j] * x[index_[j]];
          y[o] = s;
        }
      };
      RunRanges(outer, num_threads, work);
    } else {
      // scatter-add; every thread owns a range of y
      for (size_t i = 0; i < ny; ++i) y[i] = 0;
      auto work = [&](size_t b, size_t e) {
        for (size_t o = 0; o < outer; ++o) {
          V xo = x[o];
          if (xo == 0) continue;
          for (size_t j = offset_[o]; j < offset_[o + 1]; ++j) {
            size_t i = index_[j];
            if (i < b || i >= e) continue;
            y[i] += (this->binary() ? 1 : value_[j]) * xo;
          }
        }
      };
      RunRanges(ny, num_threads, work);
    }
  }
  template <class F>
  static void RunRanges(size_t n, int num_threads, const F& f) {
    if (num_threads <= 1 || n < 4096) { f(0, n); return; }
    std::vector<std::thread> ths;
    for (int t = 0; t < num_threads; ++t) {
      SizeR r = SizeR(0, n).EvenDivide(num_threads, t);
      ths.emplace_back([&f, r] { f(r.begin(), r.end()); });
    }
    for (auto& t : ths) t.join();
  }
  SArray<size_t> offset_;
  SArray<I> index_;
  SArray<V> value_;
};

// Maps the global (uint64) column ids of a minibatch to dense local ids.
template <typename I, typename V>
class Localizer {
 public:
  // sorted unique column ids of `mat`, and (optionally) their saturating counts
  template <typename C>
  void CountUniqIndex(const SparseMatrix<I, V>& mat, SArray<I>* uniq_idx, SArray<C>* idx_frq = nullptr, int num_threads = 2) {
    mat_ = &mat;
    const SArray<I>& idx = mat.index();
    size_t n = idx.size();
    pair_.resize(n);
    for (size_t i = 0; i < n; ++i) { pair_[i].k = idx[i]; pair_[i].i = (uint32_t)i; }
    ParallelSort(pair_.data(), n, num_threads, [](const Pair& a, const Pair& b) { return a.k < b.k; });
    uniq_idx->clear();
    if (idx_frq) idx_frq->clear();
    const C cmax = std::numeric_limits<C>::max();
    I cur = 0;
    C cnt = 0;
    for (size_t i = 0; i < n; ++i) {
      if (i == 0 || pair_[i].k != cur) {
        if (i && idx_frq) idx_frq->push_back(cnt);
        cur = pair_[i].k;
        uniq_idx->push_back(cur);
        cnt = 0;
      }
      if (cnt < cmax) ++cnt;
    }
    if (n && idx_frq) idx_frq->push_back(cnt);
  }
  void CountUniqIndex(const SparseMatrix<I, V>& mat, SArray<I>* uniq_idx) { CountUniqIndex<uint8_t>(mat, uniq_idx, nullptr); }

  // Rewrites the matrix with columns 0..|idx_dict|-1; entries whose id is not in
  // the (sorted) dictionary are dropped.
  std::shared_ptr<SparseMatrix<uint32_t, V>> RemapIndex(const SArray<I>& idx_dict) {
    PS_CHECK(mat_ != nullptr) << "call CountUniqIndex first";
    const SparseMatrix<I, V>& mat = *mat_;
    size_t n = pair_.size();
    std::vector<uint32_t> local(n, 0);  // 0 = dropped, else local id + 1
    size_t d = 0, kept = 0;
    for (size_t i = 0; i < n; ++i) {
      while (d < idx_dict.size() && idx_dict[d] < pair_[i].k) ++d;
      if (d < idx_dict.size() && idx_dict[d] == pair_[i].k) { local[pair_[i].i] = (uint32_t)d + 1; ++kept; }
    }
    size_t outer = mat.outerSize();
    SArray<size_t> off(outer + 1);
    SArray<uint32_t> idx(kept);
    SArray<V> val(mat.binary() ? 0 : kept);
    size_t p = 0;
    off[0] = 0;
    for (size_t o = 0; o < outer; ++o) {
      for (size_t j = mat.offset()[o]; j < mat.offset()[o + 1]; ++j) {
        if (!local[j]) continue;
        idx[p] = local[j] - 1;
        if (!mat.binary()) val[p] = mat.value()[j];
        ++p;
      }
      off[o + 1] = p;
    }
    MatrixInfo info = mat.info();
    info.col = SizeR(0, idx_dict.size());
    info.nnz = kept;
    info.sizeof_index = sizeof(uint32_t);
    return std::make_shared<SparseMatrix<uint32_t, V>>(info, off, idx, val);
  }
  void Clear() { pair_.clear(); mat_ = nullptr; }
  size_t memSize() const { return pair_.size() * sizeof(Pair); }
 private:
#pragma pack(push, 4)
  struct Pair { I k; uint32_t i; };
#pragma pack(pop)
  std::vector<Pair> pair_;
  const SparseMatrix<I, V>* mat_ = nullptr;
};

}  // namespace PS
