// Binary-classification metrics: exact AUC (rank statistic), accuracy, logloss;
// and a mergeable histogram AUC for distributed evaluation.
// Counterparts: util/evaluation.h:9-79, util/auc.h:8-103, util/proto/auc.proto:3-9.
// Also the timers of util/resource_usage.h:15-132.
#pragma once
#include <algorithm>
#include <cmath>
#include <fstream>
#include <map>
#include "sarray.h"

namespace PS {

template <typename V>
class Evaluation {
 public:
  // area under the ROC curve; labels > 0 are positive
  static V auc(const SArray<V>& label, const SArray<V>& predict) {
    size_t n = label.size();
    PS_CHECK_EQ(n, predict.size());
    std::vector<std::pair<V, V>> buf(n);
    for (size_t i = 0; i < n; ++i) buf[i] = std::make_pair(predict[i], label[i]);
    std::sort(buf.begin(), buf.end(), [](const std::pair<V, V>& a, const std::pair<V, V>& b) { return a.first < b.first; });
    double area = 0, cum_tp = 0;
    for (size_t i = 0; i < n; ++i) {
      if (buf[i].second > 0) cum_tp += 1;
      else area += cum_tp;
    }
    if (cum_tp == 0 || cum_tp == n) return 1;
    area /= cum_tp * (n - cum_tp);
    return (V)(area < 0.5 ? 1 - area : area);
  }
  static V accuracy(const SArray<V>& label, const SArray<V>& predict, V threshold = 0) {
    size_t n = label.size();
    PS_CHECK_EQ(n, predict.size());
    double correct = 0;
    for (size_t i = 0; i < n; ++i)
      if ((label[i] > 0 && predict[i] > threshold) || (label[i] <= 0 && predict[i] <= threshold)) correct += 1;
    V acc = (V)(correct / n);
    return acc > 0.5 ? acc : 1 - acc;
  }
  static V logloss(const SArray<V>& label, const SArray<V>& predict) {
    size_t n = label.size();
    PS_CHECK_EQ(n, predict.size());
    double loss = 0;
    for (size_t i = 0; i < n; ++i) {
      double y = label[i] > 0 ? 1 : 0;
      double p = 1.0 / (1.0 + std::exp(-(double)predict[i]));
      p = p < 1e-10 ? 1e-10 : p;
      loss += y * std::log(p) + (1 - y) * std::log(1 - p);
    }
    return (V)(-loss / n);
  }
};

// Histogram AUC: every node counts positives / negatives per quantised score;
// histograms merge by addition.
class AUC {
 public:
  void setGoodness(int64_t g) { goodness_ = g; }
  struct Data { std::map<int64_t, uint64_t> tp, fp; };
  template <typename V>
  void compute(const SArray<V>& label, const SArray<V>& predict, Data* out) const {
    PS_CHECK_EQ(label.size(), predict.size());
    for (size_t i = 0; i < label.size(); ++i) {
      int64_t k = (int64_t)(predict[i] * goodness_);
      if (label[i] > 0) ++out->tp[k]; else ++out->fp[k];
    }
  }
  void merge(const Data& d) {
    for (auto& kv : d.tp) data_.tp[kv.first] += kv.second;
    for (auto& kv : d.fp) data_.fp[kv.first] += kv.second;
  }
  double evaluate() const {
    if (data_.tp.empty() || data_.fp.empty()) return 0.5;
    double tp_sum = 0, fp_sum = 0;
    for (auto& kv : data_.tp) tp_sum += kv.second;
    for (auto& kv : data_.fp) fp_sum += kv.second;
    // walk thresholds from high to low accumulating the trapezoid area
    std::map<int64_t, std::pair<uint64_t, uint64_t>> all;
    for (auto& kv : data_.tp) all[kv.first].first += kv.second;
    for (auto& kv : data_.fp) all[kv.first].second += kv.second;
    double area = 0, tp = 0;
    for (auto it = all.rbegin(); it != all.rend(); ++it) {
      double dtp = it->second.first, dfp = it->second.second;
      area += dfp * (tp + dtp / 2);
      tp += dtp;
    }
    area /= tp_sum * fp_sum;
    return area < 0.5 ? 1 - area : area;
  }
  double accuracy(double threshold = 0) const {
    double correct = 0, total = 0;
    int64_t thr = (int64_t)(threshold * goodness_);
    for (auto& kv : data_.tp) { total += kv.second; if (kv.first > thr) correct += kv.second; }
    for (auto& kv : data_.fp) { total += kv.second; if (kv.first <= thr) correct += kv.second; }
    return total ? correct / total : 0;
  }
  void clear() { data_.tp.clear(); data_.fp.clear(); }
 private:
  int64_t goodness_ = 1000;
  Data data_;
};

// ---------------------------------------------------------------- timers
inline std::chrono::steady_clock::time_point tic() { return std::chrono::steady_clock::now(); }
inline double toc(std::chrono::steady_clock::time_point start) {
  return std::chrono::duration<double>(std::chrono::steady_clock::now() - start).count();
}
// Cycle-counter pair for very short sections (the reference's hwtic / hwtoc, util/resource_usage.h:33-50):
// hwtic() reads the time-stamp counter, hwtoc(start) the cycles since (0 where the target has no such counter).
inline uint64_t hwtic() {
#if defined(__x86_64__) || defined(__i386__)
  uint32_t lo, hi;
  __asm__ __volatile__("rdtsc" : "=a"(lo), "=d"(hi));
  return ((uint64_t)hi << 32) | lo;
#elif defined(__aarch64__)
  uint64_t v;
  __asm__ __volatile__("mrs %0, cntvct_el0" : "=r"(v));
  return v;
#else
  return 0;
#endif
}
inline uint64_t hwtoc(uint64_t start) { return hwtic() - start; }

class Timer {
 public:
  void start() { tp_ = tic(); }
  void restart() { reset(); start(); }
  void reset() { time_ = 0; }
  double stop() { time_ += toc(tp_); return time_; }
  double get() const { return time_; }
  double getAndRestart() { double t = get(); reset(); start(); return t; }
 private:
  std::chrono::steady_clock::time_point tp_ = tic();
  double time_ = 0;
};
class MilliTimer {
 public:
  void start() { tp_ = tic(); }
  void stop() { total_ms_ += (uint64_t)(toc(tp_) * 1e3); }
  uint64_t get() const { return total_ms_; }
  void reset() { total_ms_ = 0; }
 private:
  std::chrono::steady_clock::time_point tp_ = tic();
  uint64_t total_ms_ = 0;
};
class ScopedTimer {
 public:
  explicit ScopedTimer(double* aggregate) : aggregate_(aggregate), tp_(tic()) {}
  ~ScopedTimer() { *aggregate_ += toc(tp_); }
 private:
  double* aggregate_;
  std::chrono::steady_clock::time_point tp_;
};
// resident / virtual memory of this process in MB
class ResUsage {
 public:
  static double myPhyMem() { return Field(1) * 4096.0 / (1 << 20); }
  static double myVirMem() { return Field(0) * 4096.0 / (1 << 20); }
  // the machine's memory in MB: total, and in use (total - free - buffers - page cache)
  static double hostTotalMem() { return MemInfo("MemTotal:") / 1024.0; }
  static double hostInUseMem() {
    return (MemInfo("MemTotal:") - MemInfo("MemFree:") - MemInfo("Buffers:") - MemInfo("Cached:")) / 1024.0;
  }
 private:
  static double MemInfo(const char* name) {   // the kB figure of one /proc/meminfo line
    std::ifstream f("/proc/meminfo");
    std::string key;
    double kb = 0;
    while (f >> key) {
      if (key == name) { f >> kb; return kb; }
      f.ignore(256, '\n');
    }
    return 0;
  }
  static double Field(int i) {
    std::ifstream f("/proc/self/statm");
    double v[2] = {0, 0};
    f >> v[0] >> v[1];
    return v[i];
  }
};

}  // namespace PS
