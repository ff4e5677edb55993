// Learner skeletons shared by the applications: the workload pool, the SGD
// scheduler / compute-node bases with progress reporting, the prefetching
// minibatch reader, and the progress records.
// Counterparts: learner/workload_pool.h:8-39 (+.cc), learner/sgd.h:21-144 (+.cc),
// learner/proto/sgd.proto:5-26, learner/proto/bcd.proto:47-60.
#pragma once
#include <iomanip>
#include <set>
#include "data.h"
#include "filter.h"
#include "monitor.h"
#include "parameter.h"

namespace PS {

// ---------------------------------------------------------------- workload pool
// One workload per (file, replica); assigned to workers on request, put back
// when a worker dies, finished when the worker reports back.
class WorkloadPool {
 public:
  WorkloadPool() {}
  explicit WorkloadPool(const Workload& load) { set(load); }
  void set(const Workload& load) {
    Lock l(mu_);
    loads_.clear();
    num_finished_ = 0;
    DataConfig files = searchFiles(load.data);
    std::vector<std::string> list = files.file;
    int replica = std::max(1, load.replica);
    for (int r = 0; r < replica; ++r) {
      if (load.shuffle) { std::mt19937 g(1000 + r); std::shuffle(list.begin(), list.end(), g); }
      for (auto& f : list) {
        Item it;
        it.load = load;
        it.load.data.file = {f};
        it.load.id = {(int)loads_.size()};
        it.load.replica = 1;
        loads_.push_back(it);
      }
    }
  }
  // false if nothing is left to hand out
  bool assign(const NodeID& node, Workload* load) {
    Lock l(mu_);
    for (auto& it : loads_) {
      if (it.assigned || it.finished) continue;
      it.assigned = true;
      it.node = node;
      *load = it.load;
      return true;
    }
    return false;
  }
  // put the unfinished workloads of a dead node back
  void restore(const NodeID& node) {
    Lock l(mu_);
    for (auto& it : loads_) if (it.assigned && !it.finished && it.node == node) { it.assigned = false; it.node.clear(); }
    cv_.notify_all();
  }
  void finish(int id) {
    {
      Lock l(mu_);
      PS_CHECK_LT((size_t)id, loads_.size());
      if (!loads_[id].finished) { loads_[id].finished = true; ++num_finished_; }
    }
    cv_.notify_all();
  }
  void waitUtilDone() {
    ULock l(mu_);
    cv_.wait(l, [this] { return num_finished_ >= loads_.size(); });
  }
  size_t size() { Lock l(mu_); return loads_.size(); }
  size_t num_finished() { Lock l(mu_); return num_finished_; }
 private:
  struct Item { Workload load; NodeID node; bool assigned = false, finished = false; };
  std::vector<Item> loads_;
  size_t num_finished_ = 0;
  std::mutex mu_;
  std::condition_variable cv_;
};

// ---------------------------------------------------------------- progress records
struct SGDProgress {
  std::vector<double> objective, accuracy, auc;
  uint64_t num_examples_processed = 0;
  uint64_t nnz = 0;
  double weight_sum = 0, delta_sum = 0;
  uint64_t round = 0;      // lock-step device workers: push/pull rounds submitted so far
  std::string Serialize() const {
    Writer w;
    auto vec = [&w](const std::vector<double>& v) { w.U64(v.size()); for (double x : v) w.F64(x); };
    vec(objective); vec(accuracy); vec(auc);
    w.U64(num_examples_processed); w.U64(nnz); w.F64(weight_sum); w.F64(delta_sum); w.U64(round);
    return w.str();
  }
  bool Parse(const std::string& s) {
    Reader r(s.data(), s.size());
    auto vec = [&r](std::vector<double>* v) { uint64_t n = r.U64(); v->clear(); for (uint64_t i = 0; i < n && r.ok(); ++i) v->push_back(r.F64()); };
    vec(&objective); vec(&accuracy); vec(&auc);
    num_examples_processed = r.U64(); nnz = r.U64(); weight_sum = r.F64(); delta_sum = r.F64(); round = r.U64();
    return r.ok();
  }
};

struct BCDProgress {
  double objective = 0, relative_obj = 0, violation = 0, total_time = 0;
  uint64_t nnz_w = 0, nnz_active_set = 0;
  std::vector<double> busy_time;
  std::string Serialize() const {
    Writer w;
    w.F64(objective); w.F64(relative_obj); w.F64(violation); w.F64(total_time); w.U64(nnz_w); w.U64(nnz_active_set);
    w.U64(busy_time.size()); for (double b : busy_time) w.F64(b);
    return w.str();
  }
  bool Parse(const std::string& s) {
    Reader r(s.data(), s.size());
    objective = r.F64(); relative_obj = r.F64(); violation = r.F64(); total_time = r.F64(); nnz_w = r.U64(); nnz_active_set = r.U64();
    uint64_t n = r.U64(); busy_time.clear(); for (uint64_t i = 0; i < n && r.ok(); ++i) busy_time.push_back(r.F64());
    return r.ok();
  }
};

// ---------------------------------------------------------------- SGD scheduler / nodes
static const int kMonitorCustomerID = 90;   // the progress monitor's customer id on every node

class ISGDScheduler : public App {
 public:
  explicit ISGDScheduler(Postoffice* po = nullptr) : App(po), monitor_(kMonitorCustomerID, po) {}
  virtual ~ISGDScheduler() {}
  void Run() override;
  void ProcessRequest(Message* request) override;
  void ProcessResponse(Message* response) override;
  // "sec examples loss auc accuracy |w|_0 updt-ratio" table
  static std::string ProgressHeader();
  std::string ProgressLine(double time, std::unordered_map<NodeID, SGDProgress>* progress);
  size_t num_examples_processed() const { return num_ex_processed_; }
 protected:
  // false when the pool had nothing to hand out
  virtual bool SendWorkload(const NodeID& recver);
  WorkloadPool* workload_pool_ = nullptr;
  MonitorMaster<SGDProgress> monitor_;
  std::atomic<size_t> num_ex_processed_{0};
  bool show_progress_ = true;
  bool printed_header_ = false;
};

// Scheduler of workers that run their push/pull rounds in lock step (one device shard and one
// worker per GPU: round t of every worker is aggregated at the owners, so every worker has to run
// every round, with an empty minibatch when it has no data). Files are handed out one at a time as
// in ISGDScheduler; in addition the scheduler grants rounds in leases: a worker may run round t
// only while t < round_limit. Workers report their round counter with their progress, the limit
// stays `lease` rounds ahead of the largest one reported, and when the last file is finished the
// limit that is in force becomes final: every worker stops at exactly that round, without any
// per-round agreement between the workers.
class LockstepSGDScheduler : public ISGDScheduler {
 public:
  LockstepSGDScheduler(const Workload& load, int lease, Postoffice* po = nullptr)
      : ISGDScheduler(po), lease_(std::max(4, lease)) {
    pool_.set(load);
    workload_pool_ = &pool_;
  }
  void Run() override;
  uint64_t round_limit() { Lock l(lease_mu_); return limit_; }
  WorkloadPool& pool() { return pool_; }
 protected:
  // remembers the workers that asked when the pool was empty: the files of a lost worker go to them
  bool SendWorkload(const NodeID& recver) override;
 private:
  void Grant(bool final_round);
  void NodeLost(const NodeID& id);
  WorkloadPool pool_;
  std::mutex idle_mu_;
  std::set<NodeID> idle_;
  const int lease_;
  std::mutex lease_mu_;
  uint64_t max_round_ = 0, limit_ = 0;
  bool final_sent_ = false;
};

class ISGDCompNode : public App {
 public:
  explicit ISGDCompNode(Postoffice* po = nullptr)
      : App(po), reporter_(sys_->manager().van().scheduler().id, kMonitorCustomerID, po) {}
  virtual ~ISGDCompNode() {}
 protected:
  MonitorSlaver<SGDProgress> reporter_;
};

// Reads minibatches on a background thread and localises them: unique column
// ids, optional tail-feature filter by count-min, remap to local ids.
template <typename V>
class MinibatchReader {
 public:
  MinibatchReader() {}
  void InitReader(const DataConfig& file, int minibatch_size, int data_buf_mb = 1000) {
    reader_.init(file);
    mb_size_ = minibatch_size;
    data_prefetcher_.setCapacity(data_buf_mb);
  }
  // keys seen fewer than `freq` times (estimated) are dropped; n, k size the sketch
  void InitFilter(size_t n, int k, int freq) { filter_.Resize((int)std::min<size_t>(n, 1u << 30), k); key_freq_ = freq; }
  void Start() {
    data_prefetcher_.startProducer([this](Batch* data, size_t* size) -> bool {
      data->mats.clear();
      bool ok = reader_.readMatrices(mb_size_, &data->label, &data->mats);
      *size = 1;
      if (ok) for (auto& m : data->mats) *size += m->index().memSize() + m->value().memSize() + m->offset().memSize();
      data->valid = ok;
      return ok;
    });
  }
  // labels Y, localized X (uint32 columns) and the global keys of those columns
  bool Read(SArray<V>* Y, std::shared_ptr<SparseMatrix<uint32_t, V>>* X, SArray<Key>* key) {
    Batch data;
    while (true) {
      if (!data_prefetcher_.pop(&data)) return false;
      if (data.valid && !data.mats.empty()) break;
      if (!data.valid) return false;
    }
    *Y = data.label;
    // feature groups are merged into one matrix by the parser option ignore_feature_group
    auto& mat = *data.mats[0];
    SArray<Key> uniq;
    SArray<uint8_t> cnt;
    Localizer<Key, V> localizer;
    localizer.template CountUniqIndex<uint8_t>(mat, &uniq, &cnt);
    if (key_freq_ > 0) {
      filter_.InsertKeys(uniq, cnt);
      *key = filter_.QueryKeys(uniq, key_freq_);
    } else {
      *key = uniq;
    }
    *X = localizer.RemapIndex(*key);
    return true;
  }
 private:
  struct Batch {
    SArray<V> label;
    std::vector<std::shared_ptr<SparseMatrix<uint64_t, V>>> mats;
    bool valid = false;
  };
  int mb_size_ = 1000;
  StreamReader<V> reader_;
  FreqencyFilter<Key, uint8_t> filter_;
  int key_freq_ = 0;
  ProducerConsumer<Batch> data_prefetcher_;
};

}  // namespace PS
