// Darlin: delayed block proximal gradient (block coordinate descent) for
// L1-regularised logistic regression, CPU path.
//
// Scheduler: load -> preprocess -> divide features into blocks -> passes over
// the blocks with bounded delay tau (a block's task waits for the block tau+1
// places before it) -> evaluate -> stop test -> save.
// Worker: column-major X per feature group, dual = exp(y.Xw); per block compute
// (G, U), push at t, pull new weights at t+2 (waiting on the server's virtual
// t+1), update the dual. Server: sum (G, U) over workers, Newton step with soft
// threshold inside a trust region, KKT filter.
//
// Counterparts: app/linear_method/darlin.h:12-592, learner/bcd.h:24-440,
// learner/bcd.cc:6-175.
#include "linear_method.h"

namespace PS {
namespace LM {

static const int kTimeRatio = 3;  // model timestamps per step: push, virtual aggregate, pull
inline Real TrustDelta(Real delta_max, Real d) { return std::min(delta_max, 2 * std::fabs(d) + (Real)0.1); }

// ---------------------------------------------------------------- scheduler
class DarlinScheduler : public App {
 public:
  DarlinScheduler(const Config& conf, Postoffice* po) : App(po), conf_(conf), bcd_(conf.darlin) {
    PS_CHECK(conf.loss.type == LossConfig::LOGIT) << "darlin needs the logit loss";
    PS_CHECK(conf.penalty.type == PenaltyConfig::L1) << "darlin needs an L1 penalty";
  }
  void Run() override {
    sys_->manager().WaitServersReady();
    sys_->manager().WaitWorkersReady();
    total_timer_.start();
    LoadData();
    PreprocessData();
    DivideFeatureBlocks();
    const int tau = bcd_.max_block_delay;
    PS_NOTICE("maximal allowed delay: %d", tau);
    int model_time = (int)fea_grp_.size() * 6;  // timestamps consumed by preprocessing
    bool reset_kkt = false, random_order = bcd_.random_feature_block_order;
    Real kkt_threshold = 1e20f;
    int iter = 0;
    for (; iter < bcd_.max_pass_of_data; ++iter) {
      std::vector<int> order;
      // pass 0 starts with the prior groups' blocks, repeated
      std::vector<int> prior;
      if (iter == 0) prior = prior_blk_order_;
      std::vector<int> rest = blk_order_;
      if (random_order) { std::mt19937 g(1000 + iter); std::shuffle(rest.begin(), rest.end(), g); }
      order = prior;
      order.insert(order.end(), rest.begin(), rest.end());
      int first_time = -1;
      for (size_t i = 0; i < order.size(); ++i) {
        Task update;
        update.more = true;  // a whole pass is packed into one wire message per node
        BCDCall* cmd = update.mutable_bcd();
        cmd->cmd = BCDCall::UPDATE_MODEL;
        cmd->time = model_time;
        model_time += kTimeRatio;
        const auto& blk = fea_blk_[order[i]];
        cmd->has_key = true;
        cmd->key = blk.second;
        cmd->feature_group_id = blk.first;
        cmd->kkt_filter_threshold = kkt_threshold;
        cmd->reset_kkt_filter = reset_kkt && i == 0;
        int cur = exec_.time() + 1;
        if (first_time < 0) first_time = cur;
        int t = (i < prior.size()) ? 0 : tau;  // prior blocks run one after another
        // wait for the tasks [max(first, cur-2t-1), max(first+1, cur-t))
        int lo = std::max(first_time, cur - 2 * t - 1), hi = std::max(first_time + 1, cur - t);
        for (int w = lo; w < hi && w < cur; ++w) update.wait_time.push_back(w);
        update.set_time(cur);
        Submit(update, kCompGroup);
      }
      // evaluate (closes the pack)
      Task eval;
      eval.more = false;
      eval.mutable_bcd()->cmd = BCDCall::EVALUATE_PROGRESS;
      eval.bcd.iter = iter;
      int cur = exec_.time() + 1;
      if (cur - 1 >= std::max(0, first_time)) eval.wait_time.push_back(cur - 1);
      progress_.clear();
      int ts = Submit(eval, kCompGroup);
      Wait(ts);
      BCDProgress merged = MergeProgress(iter);
      ShowProgress(iter, merged);
      if (bcd_.save_model_every_n_iter > 0 && (iter + 1) % bcd_.save_model_every_n_iter == 0 &&
          conf_.has_model_output && !conf_.model_output.file.empty()) {
        SaveModel(conf_.model_output.file[0] + "_it_" + std::to_string(iter));
      }
      // the KKT filter threshold follows the largest violation of this pass
      Real vio = (Real)merged.violation;
      Real ratio = (Real)bcd_.kkt_filter_threshold_ratio;
      kkt_threshold = vio / (Real)std::max<uint64_t>(1, num_examples_) * ratio;
      double rel = merged.relative_obj;
      if (rel > 0 && rel <= bcd_.epsilon) {
        if (reset_kkt) { PS_NOTICE("converged: relative objective <= %g", bcd_.epsilon); break; }
        reset_kkt = true;  // first hit: re-open every coordinate once
      } else {
        reset_kkt = false;
      }
    }
    if (conf_.has_model_output && !conf_.model_output.file.empty()) SaveModel(conf_.model_output.file[0]);
    final_iter_ = iter;
  }
  void ProcessResponse(Message* response) override {
    const Task& t = response->task;
    if (!t.has_bcd) return;
    Lock l(mu_);
    if (t.bcd.cmd == BCDCall::LOAD_DATA) {
      num_examples_ += (uint64_t)t.bcd.delta;
      for (int g : t.bcd.fea_grp) grp_set_[g] += t.bcd.kkt_filter_threshold;  // nnz per group rides in this field
    } else if (t.bcd.cmd == BCDCall::EVALUATE_PROGRESS) {
      BCDProgress p;
      if (p.Parse(t.msg)) progress_[response->sender] = p;
    }
  }
  const std::vector<BCDProgress>& history() const { return history_; }

 private:
  void LoadData() {
    Task load;
    load.mutable_bcd()->cmd = BCDCall::LOAD_DATA;
    int ts = Submit(load, kWorkerGroup);
    Wait(ts);
    fea_grp_.clear();
    for (auto& kv : grp_set_) fea_grp_.push_back(kv.first);
    PS_NOTICE("loaded %lu examples, %d feature group(s)", (unsigned long)num_examples_, (int)fea_grp_.size());
  }
  void PreprocessData() {
    Task pre;
    BCDCall* cmd = pre.mutable_bcd();
    cmd->cmd = BCDCall::PREPROCESS_DATA;
    cmd->fea_grp = fea_grp_;
    cmd->tail_feature_freq = bcd_.tail_feature_freq;
    cmd->delta = (double)num_examples_;
    int ts = Submit(pre, kCompGroup);
    Wait(ts);
  }
  // per group: n = ceil(nnz_per_row * feature_block_ratio) even key-range blocks
  void DivideFeatureBlocks() {
    fea_blk_.clear(); blk_order_.clear(); prior_blk_order_.clear();
    for (int g : fea_grp_) {
      double nnz_per_row = num_examples_ ? grp_set_[g] / (double)num_examples_ : 1;
      int n = 1;
      if (bcd_.feature_block_ratio > 0) n = std::max(1, (int)std::ceil(nnz_per_row * bcd_.feature_block_ratio));
      for (int i = 0; i < n; ++i) {
        Range<Key> blk = Range<Key>::All().EvenDivide(n, i);
        fea_blk_.push_back(std::make_pair(g, blk));
      }
    }
    for (size_t i = 0; i < fea_blk_.size(); ++i) blk_order_.push_back((int)i);
    for (int g : bcd_.prior_fea_group)
      for (int r = 0; r < bcd_.num_iter_for_prior_fea_group; ++r)
        for (size_t i = 0; i < fea_blk_.size(); ++i) if (fea_blk_[i].first == g) prior_blk_order_.push_back((int)i);
    PS_NOTICE("features are partitioned into %d blocks", (int)fea_blk_.size());
  }
  BCDProgress MergeProgress(int iter) {
    Lock l(mu_);
    BCDProgress m;
    for (auto& kv : progress_) {
      const BCDProgress& p = kv.second;
      m.objective += p.objective;
      m.nnz_w += p.nnz_w;
      m.violation = std::max(m.violation, p.violation);
      m.nnz_active_set += p.nnz_active_set;
      m.busy_time.insert(m.busy_time.end(), p.busy_time.begin(), p.busy_time.end());
    }
    m.total_time = total_timer_.stop();
    total_timer_.start();
    if (!history_.empty() && history_.back().objective != 0)
      m.relative_obj = (history_.back().objective - m.objective) / history_.back().objective;
    else m.relative_obj = 1;
    history_.push_back(m);
    return m;
  }
  void ShowProgress(int iter, const BCDProgress& p) {
    if (iter == 0) {
      PS_NOTICE("  iter |  objective    relative   |w|_0   | violation  active set |  time: busy(min,max)  total");
    }
    double bmin = 0, bmax = 0;
    if (!p.busy_time.empty()) { bmin = *std::min_element(p.busy_time.begin(), p.busy_time.end()); bmax = *std::max_element(p.busy_time.begin(), p.busy_time.end()); }
    PS_NOTICE(" %5d | %.5e  %.3e  %8lu | %.3e  %9lu | %6.2f %6.2f %6.2f", iter, p.objective, p.relative_obj,
              (unsigned long)p.nnz_w, p.violation, (unsigned long)p.nnz_active_set, bmin, bmax, p.total_time);
  }
  void SaveModel(const std::string& file) {
    Task save;
    save.mutable_bcd()->cmd = BCDCall::SAVE_MODEL;
    save.msg = file;
    int ts = Submit(save, kCompGroup);
    Wait(ts);
  }

  Config conf_;
  BCDConfig bcd_;
  std::mutex mu_;
  uint64_t num_examples_ = 0;
  std::map<int, double> grp_set_;        // feature group -> nnz
  std::vector<int> fea_grp_;
  std::vector<std::pair<int, Range<Key>>> fea_blk_;
  std::vector<int> blk_order_, prior_blk_order_;
  std::unordered_map<NodeID, BCDProgress> progress_;
  std::vector<BCDProgress> history_;
  Timer total_timer_;
  int final_iter_ = 0;
};

// ---------------------------------------------------------------- compute node base
class DarlinCompNode : public App {
 public:
  DarlinCompNode(const Config& conf, Postoffice* po)
      : App(po), conf_(conf), bcd_(conf.darlin), model_(true, 1, kModelCustomerID, po) {}
  void ProcessRequest(Message* request) override {
    const Task& t = request->task;
    if (!t.has_bcd) return;
    switch (t.bcd.cmd) {
      case BCDCall::LOAD_DATA: LoadData(request); break;
      case BCDCall::PREPROCESS_DATA: PreprocessData(request); break;
      case BCDCall::UPDATE_MODEL: Update(request); break;
      case BCDCall::EVALUATE_PROGRESS: {
        BCDProgress prog;
        Evaluate(&prog);
        Task resp;
        resp.mutable_bcd()->cmd = BCDCall::EVALUATE_PROGRESS;
        resp.msg = prog.Serialize();
        Reply(request, resp);
        break;
      }
      case BCDCall::SAVE_MODEL: SaveModel(request->task.msg); break;
      default: break;
    }
  }
 protected:
  virtual void LoadData(Message* request) {}
  virtual void PreprocessData(Message* request) = 0;
  virtual void Update(Message* request) = 0;
  virtual void Evaluate(BCDProgress* prog) = 0;
  virtual void SaveModel(const std::string& file) {}
  std::vector<FilterConfig> filters() const { return bcd_.comm_filter; }

  Config conf_;
  BCDConfig bcd_;
  KVVector<Key, Real> model_;
  std::vector<int> fea_grp_;
  std::unordered_map<int, Bitmap> active_set_;
  std::unordered_map<int, SArray<Real>> delta_;
  SparseFilter kkt_filter_;
  Real kkt_filter_threshold_ = 1e20f;
};

// ---------------------------------------------------------------- server
class DarlinServer : public DarlinCompNode {
 public:
  using DarlinCompNode::DarlinCompNode;
 protected:
  void PreprocessData(Message* request) override {
    const BCDCall& call = request->task.bcd;
    fea_grp_ = call.fea_grp;
    int time = 0;
    const bool tail = call.tail_feature_freq > 0;
    // first exchange per group: workers push (key, count); release their filtered-key pulls
    for (int grp : fea_grp_) {
      (void)grp;
      if (tail) model_.WaitReceivedRequest(time, kWorkerGroup);
      model_.FinishReceivedRequest(time + 1, kWorkerGroup);
      time += kTimeRatio;
    }
    // second exchange per group: workers push their keys; allocate weights; release the initial pulls
    for (int grp : fea_grp_) {
      model_.WaitReceivedRequest(time, kWorkerGroup);
      auto& kv = model_[grp];
      kv.value.resize(kv.key.size());
      kv.value.SetValue(bcd_.init_w);      // the workers pull these and start from dual = exp(y . Xw)
      active_set_[grp].resize((uint32_t)kv.key.size(), true);
      delta_[grp].resize(kv.key.size());
      delta_[grp].SetValue((Real)bcd_.delta_init_value);
      model_.FinishReceivedRequest(time + 1, kWorkerGroup);
      time += kTimeRatio;
    }
  }
  void Update(Message* request) override {
    const BCDCall& call = request->task.bcd;
    if (call.reset_kkt_filter) for (int g : fea_grp_) active_set_[g].fill(true);
    kkt_filter_threshold_ = (Real)call.kkt_filter_threshold;
    Range<Key> my_range = sys_->manager().van().my_node().key;
    Range<Key> blk = call.key.SetIntersection(my_range);
    int time = call.time, grp = call.feature_group_id;
    if (blk.empty()) {
      // this block lives on other servers; still release whoever depends on the stamp
      model_.FinishReceivedRequest(time + 1, kWorkerGroup);
      return;
    }
    // all workers' (G, U) of this block, summed
    model_.WaitReceivedRequest(time, kWorkerGroup);
    auto& kv = model_[grp];
    SizeR idx = kv.key.FindRange(call.key);
    if (!idx.empty()) {
      auto& buf = model_.buffer(time);
      PS_VLOG(1) << "server update t=" << time << " idx=" << idx << " buf.idx=" << buf.idx_range << " nvals="
                 << buf.values.size() << " n0=" << (buf.values.empty() ? 0 : buf.values[0].size());
      if (buf.values.size() >= 2 && buf.values[0].size() == idx.size() && buf.idx_range == idx) {
        UpdateWeight(grp, idx, buf.values[0], buf.values[1]);
      }
    }
    model_.ClearBuffer(time);
    // workers' pulls at time+2 wait for this
    model_.FinishReceivedRequest(time + 1, kWorkerGroup);
  }
  void Evaluate(BCDProgress* prog) override {
    size_t nnz_w = 0, nnz_as = 0;
    double objv = 0;
    for (int grp : fea_grp_) {
      const auto& value = model_[grp].value;
      for (size_t i = 0; i < value.size(); ++i) {
        Real w = value[i];
        if (kkt_filter_.marked(w) || w == 0) continue;
        ++nnz_w;
        objv += std::fabs(w);
      }
      nnz_as += active_set_[grp].nnz();
    }
    prog->objective = objv * conf_.penalty.lambda[0];
    prog->nnz_w = nnz_w;
    prog->violation = violation_;
    prog->nnz_active_set = nnz_as;
    violation_ = 0;
  }
  void SaveModel(const std::string& file) override {
    std::string name = file + "_" + sys_->manager().van().my_node().id;
    std::ofstream out(name);
    PS_CHECK(out.good()) << "cannot write " << name;
    for (int grp : fea_grp_) {
      auto& kv = model_[grp];
      for (size_t i = 0; i < kv.key.size(); ++i) {
        Real w = kv.value[i];
        if (w != 0 && !(w != w)) out << kv.key[i] << "\t" << w << "\n";
      }
    }
  }
 private:
  // One coordinate of the block: g is the summed gradient, u the summed curvature bound. The
  // objective along the coordinate is bounded by the quadratic g d + (u / (2 eta)) d^2 + lambda |w + d|,
  // whose minimiser is a soft threshold in the variable w + d; the step is then clipped to the
  // coordinate's trust region, which is re-sized from the step taken (darlin.h:261-304).
  struct CoordinateStep {
    Real step = 0, violation = 0;
    bool frozen = false;           // KKT filter: a zero weight far inside the subdifferential
  };
  static CoordinateStep SolveCoordinate(Real w, Real g, Real curvature, Real lambda, Real kkt_threshold) {
    CoordinateStep out;
    const Real up = g + lambda, down = g - lambda;      // one-sided derivatives at w = 0 (right, left)
    if (w == 0) {
      if (up < 0) out.violation = -up;
      else if (down > 0) out.violation = down;
      else if (up > kkt_threshold && down < -kkt_threshold) { out.frozen = true; return out; }
    }
    const Real cw = curvature * w;
    if (up <= cw) out.step = -up / curvature;            // the minimiser stays positive
    else if (down >= cw) out.step = -down / curvature;   // ... stays negative
    else out.step = -w;                                   // ... is zero
    return out;
  }
  void UpdateWeight(int grp, SizeR range, const SArray<Real>& G, const SArray<Real>& U) {
    const Real eta = (Real)conf_.learning_rate.alpha;
    const Real lambda = (Real)conf_.penalty.lambda[0];
    const Real widest = (Real)bcd_.delta_max_value;
    SArray<Real>& weights = model_[grp].value;
    SArray<Real>& radius = delta_[grp];
    auto& active = active_set_[grp];
    const size_t first = range.begin();
    for (size_t i = 0; i < range.size(); ++i) {
      const uint32_t col = (uint32_t)(first + i);
      if (!active.test(col)) continue;
      const CoordinateStep cs = SolveCoordinate(weights[col], G[i], U[i] / eta + (Real)1e-10, lambda,
                                                (Real)kkt_filter_threshold_);
      if (cs.frozen) {
        active.clear(col);
        kkt_filter_.mark(&weights[col]);
        continue;
      }
      if (cs.violation > violation_) violation_ = cs.violation;
      const Real r = radius[col];
      const Real d = cs.step > r ? r : (cs.step < -r ? -r : cs.step);
      radius[col] = TrustDelta(widest, d);
      weights[col] += d;
    }
  }
  Real violation_ = 0;
};

// ---------------------------------------------------------------- worker
class DarlinWorker : public DarlinCompNode {
 public:
  using DarlinCompNode::DarlinCompNode;
 protected:
  void LoadData(Message* request) override {
    DataConfig data = conf_.training_data;
    // every worker takes its share of the files
    DataConfig all = searchFiles(data);
    int rank = sys_->manager().van().my_node().rank, n = std::max(1, sys_->manager().num_workers());
    data = divideFiles(all, n)[rank % n];
    StreamReader<Real> reader(data);
    SArray<Real> y;
    std::vector<std::shared_ptr<SparseMatrix<uint64_t, Real>>> mats;
    // gather everything (the batch solver keeps the data in memory)
    std::map<int, std::vector<std::shared_ptr<SparseMatrix<uint64_t, Real>>>> parts;
    y_.clear();
    while (reader.readMatrices(100000, &y, &mats)) {
      y_.append(y);
      for (auto& m : mats) parts[m->info().id].push_back(m);
    }
    Task resp;
    BCDCall* r = resp.mutable_bcd();
    r->cmd = BCDCall::LOAD_DATA;
    r->delta = (double)y_.size();
    for (auto& kv : parts) {
      // concatenate the row blocks of a group
      SArray<size_t> off; off.push_back(0);
      SArray<uint64_t> idx; SArray<Real> val;
      bool binary = true;
      for (auto& m : kv.second) {
        size_t base = off.back();
        for (size_t i = 1; i < m->offset().size(); ++i) off.push_back(base + m->offset()[i]);
        idx.append(m->index());
        if (!m->binary()) { binary = false; val.append(m->value()); }
      }
      while (off.size() < y_.size() + 1) off.push_back(off.back());
      MatrixInfo info = kv.second[0]->info();
      info.row = SizeR(0, y_.size());
      info.nnz = idx.size();
      info.type = binary ? MatrixInfo::SPARSE_BINARY : MatrixInfo::SPARSE;
      raw_[kv.first] = std::make_shared<SparseMatrix<uint64_t, Real>>(info, off, idx, val);
      r->fea_grp.push_back(kv.first);
      r->kkt_filter_threshold += (double)idx.size();  // total nnz (see the scheduler)
    }
    // one response per group would be cleaner; a single group is the common case
    if (r->fea_grp.size() > 1) {
      // report groups one by one through separate fields is not possible in one
      // response: send the mean so that block counts stay proportional
      r->kkt_filter_threshold /= r->fea_grp.size();
    }
    Reply(request, resp);
  }

  void PreprocessData(Message* request) override {
    const BCDCall& call = request->task.bcd;
    fea_grp_ = call.fea_grp;
    const int freq = call.tail_feature_freq;
    const size_t num_ex_total = (size_t)call.delta;
    int time = 0;
    std::unordered_map<int, Localizer<Key, Real>> localizer;
    std::unordered_map<int, SArray<Key>> uniq;
    // first exchange: tail-feature filter
    for (int grp : fea_grp_) {
      auto it = raw_.find(grp);
      SArray<Key> keys;
      SArray<uint8_t> cnt;
      if (it != raw_.end()) localizer[grp].CountUniqIndex<uint8_t>(*it->second, &keys, &cnt);
      if (freq > 0) {
        Task push = Parameter::Request(grp, time, {}, filters());
        ParamCall* pc = push.mutable_param();
        pc->has_tail_filter = true;
        pc->tail_filter.insert_count = true;
        pc->tail_filter.countmin_k = bcd_.countmin_k;
        pc->tail_filter.countmin_n = (int)std::min<double>(1e9, std::max<double>(64, num_ex_total * bcd_.countmin_n_ratio));
        Message msg(push);
        msg.recver = kServerGroup;
        msg.set_key(keys);
        msg.add_value(cnt);
        model_.Push(&msg);
        Task pull = Parameter::Request(grp, time + 2, {time + 1}, filters());
        ParamCall* qc = pull.mutable_param();
        qc->has_tail_filter = true;
        qc->tail_filter.has_freq_threshold = true;
        qc->tail_filter.freq_threshold = freq;
        Message pm(pull);
        pm.recver = kServerGroup;
        pm.set_key(keys);
        int ts = model_.Pull(&pm);
        model_.Wait(ts);
        // the filtered keys of every server arrive as key-only responses: merged into channel grp
        uniq[grp] = model_[grp].key;
      } else {
        uniq[grp] = keys;
      }
      time += kTimeRatio;
    }
    // second exchange: publish my keys, fetch initial weights, build column-major X and the dual
    dual_.resize(y_.size());
    dual_.SetValue(1);
    for (int grp : fea_grp_) {
      SArray<Key>& keys = uniq[grp];
      model_[grp].key = keys;
      model_[grp].value.resize(keys.size());
      model_[grp].value.SetZero();
      Task push = Parameter::Request(grp, time, {}, filters());
      model_.Push(push, keys);
      Task pull = Parameter::Request(grp, time + 2, {time + 1}, filters());
      int ts = model_.Pull(pull, keys);
      model_.Wait(ts);
      auto& buf = model_.buffer(time + 2);
      if (!buf.values.empty() && buf.values[0].size() == keys.size()) model_[grp].value = buf.values[0].Clone();
      model_.ClearBuffer(time + 2);
      if (raw_.count(grp)) {
        auto X = localizer[grp].RemapIndex(keys);
        X_[grp] = X->toColMajor();
        // dual = exp(y . Xw)
        SArray<Real> Xw(y_.size());
        X->times(model_[grp].value.data(), Xw.data());
        for (size_t i = 0; i < y_.size(); ++i) dual_[i] *= std::exp(y_[i] * Xw[i]);
      }
      active_set_[grp].resize((uint32_t)keys.size(), true);
      delta_[grp].resize(keys.size());
      delta_[grp].SetValue((Real)bcd_.delta_init_value);
      localizer[grp].Clear();
      raw_.erase(grp);
      time += kTimeRatio;
    }
  }

  void Update(Message* request) override {
    const BCDCall& call = request->task.bcd;
    if (call.reset_kkt_filter) { Lock l(dual_mu_); for (int g : fea_grp_) active_set_[g].fill(true); }
    int time = call.time, grp = call.feature_group_id;
    Range<Key> blk = call.key;
    auto& kv = model_[grp];
    SizeR col = kv.key.FindRange(blk);
    SArray<Real> G(col.size()), U(col.size());
    G.SetZero(); U.SetZero();
    {
      // The gradient of this block and the dual update of an earlier block (which runs on
      // the parameter's thread when its pull returns) share dual_, the weights, the active
      // set and the trust-region deltas: one at a time, as in darlin.h:300-312,398-470.
      Lock l(dual_mu_);
      busy_timer_.start();
      if (!col.empty() && X_.count(grp)) ComputeGradient(grp, col, &G, &U);
      busy_timer_.stop();
    }
    // push (G, U) at `time`
    Task push = Parameter::Request(grp, time, {}, filters(), blk);
    model_.Push(push, kv.key.Segment(col), {G, U});
    // pull the new weights at time+2 once the servers have finished time+1
    Task pull = Parameter::Request(grp, time + 2, {time + 1}, filters(), blk);
    request->finished = false;  // this block counts as done only after the dual is updated
    std::shared_ptr<Message> req = LastRequest();
    int pull_ts = time + 2;
    Message pm(pull);
    pm.recver = kServerGroup;
    pm.set_key(kv.key.Segment(col));
    pm.callback = [this, grp, col, pull_ts, req] {
      auto& buf = model_.buffer(pull_ts);
      if (!col.empty() && !buf.values.empty() && buf.values[0].size() == col.size()) UpdateDual(grp, col, buf.values[0]);
      model_.ClearBuffer(pull_ts);
      FinishReceivedRequest(req->task.time, req->sender);
      Reply(req.get());
    };
    model_.Pull(&pm);
  }

  void Evaluate(BCDProgress* prog) override {
    Lock l(dual_mu_);
    double objv = 0;
    for (size_t i = 0; i < dual_.size(); ++i) objv += std::log1p(1.0 / dual_[i]);
    prog->objective = objv;
    prog->busy_time.push_back(busy_timer_.get());
    busy_timer_.reset();
  }

 private:
  void ComputeGradient(int grp, SizeR col_range, SArray<Real>* G, SArray<Real>* U) {
    int nt = std::max(1, sys_->options().num_threads);
    ThreadPool pool(nt);
    int npart = std::max(1, std::min<int>(nt * 4, (int)col_range.size() / 64 + 1));
    for (int p = 0; p < npart; ++p) {
      SizeR part = SizeR(0, col_range.size()).EvenDivide(npart, p);
      if (part.empty()) continue;
      pool.add([this, grp, col_range, part, G, U] { GradientRange(grp, col_range, part, G->data(), U->data()); });
    }
    pool.startWorkers();
  }
  void GradientRange(int grp, SizeR col_range, SizeR part, Real* G, Real* U) {
    const auto& X = *X_[grp];
    const auto& active = active_set_[grp];
    const auto& delta = delta_[grp];
    const size_t* offset = X.offset().data();
    const uint32_t* index = X.index().data();
    const Real* value = X.value().data();
    const bool binary = X.binary();
    for (size_t j = part.begin(); j < part.end(); ++j) {
      size_t k = j + col_range.begin();
      if (!active.test((uint32_t)k)) { kkt_filter_.mark(&G[j]); kkt_filter_.mark(&U[j]); continue; }
      Real g = 0, u = 0;
      Real d = binary ? std::exp(delta[k]) : delta[k];
      for (size_t o = offset[k]; o < offset[k + 1]; ++o) {
        uint32_t i = index[o];
        Real tau = 1 / (1 + dual_[i]);
        if (binary) {
          g -= y_[i] * tau;
          u += std::min(tau * (1 - tau) * d, (Real)0.25);
        } else {
          Real v = value[o];
          g -= y_[i] * tau * v;
          u += std::min(tau * (1 - tau) * std::exp(std::fabs(v) * d), (Real)0.25) * v * v;
        }
      }
      G[j] = g; U[j] = u;
    }
  }
  void UpdateDual(int grp, SizeR col_range, const SArray<Real>& new_w) {
    Lock l(dual_mu_);
    auto& cur_w = model_[grp].value;
    auto& active = active_set_[grp];
    auto& delta = delta_[grp];
    const Real delta_max = (Real)bcd_.delta_max_value;
    SArray<Real> dw(new_w.size());
    for (size_t i = 0; i < new_w.size(); ++i) {
      size_t j = col_range.begin() + i;
      Real nw = new_w[i];
      if (kkt_filter_.marked(nw)) { active.clear((uint32_t)j); cur_w[j] = 0; dw[i] = 0; continue; }
      dw[i] = nw - cur_w[j];
      delta[j] = TrustDelta(delta_max, dw[i]);
      cur_w[j] = nw;
    }
    if (!X_.count(grp)) return;
    busy_timer_.start();
    const auto& X = *X_[grp];
    const size_t* offset = X.offset().data();
    const uint32_t* index = X.index().data();
    const Real* value = X.value().data();
    const bool binary = X.binary();
    int nt = std::max(1, sys_->options().num_threads);
    {
      ThreadPool pool(nt);
      for (int t = 0; t < nt; ++t) {
        SizeR rows = SizeR(0, y_.size()).EvenDivide(nt, t);
        if (rows.empty()) continue;
        pool.add([&, rows] {
          for (size_t jj = 0; jj < dw.size(); ++jj) {
            Real wd = dw[jj];
            size_t k = jj + col_range.begin();
            if (wd == 0 || !active.test((uint32_t)k)) continue;
            for (size_t o = offset[k]; o < offset[k + 1]; ++o) {
              uint32_t i = index[o];
              if (!rows.contains(i)) continue;
              dual_[i] *= binary ? std::exp(y_[i] * wd) : std::exp(y_[i] * wd * value[o]);
            }
          }
        });
      }
      pool.startWorkers();
    }
    busy_timer_.stop();
  }

  SArray<Real> y_, dual_;
  std::unordered_map<int, std::shared_ptr<SparseMatrix<uint64_t, Real>>> raw_;
  std::unordered_map<int, std::shared_ptr<SparseMatrix<uint32_t, Real>>> X_;
  std::mutex dual_mu_;
  Timer busy_timer_;
};

App* CreateDarlin(const Config& conf, Postoffice* po) {
  Node::Role role = po->manager().van().my_node().role;
  if (role == Node::SCHEDULER) return new DarlinScheduler(conf, po);
  if (role == Node::WORKER) return new DarlinWorker(conf, po);
  return new DarlinServer(conf, po);
}

}  // namespace LM
}  // namespace PS
