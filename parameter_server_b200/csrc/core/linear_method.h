// The linear-method application on the CPU path: loss, penalty and learning-rate
// objects, asynchronous SGD (FTRL-proximal / AdaGrad / plain SGD entries),
// Darlin block coordinate descent, model evaluation, and the factory that picks
// one from a text configuration.
// Counterparts: app/linear_method/{main.cc:7-46, async_sgd.h:22-310,
// darlin.h:12-592, loss.h:10-129, penalty.h:11-91, learning_rate.h:6-29,
// model_evaluation.h:17-107}, learner/bcd.h:24-440, learner/bcd.cc:6-175.
#pragma once
#include "evaluation.h"
#include "learner.h"
#include "lm_config.h"

namespace PS {
namespace LM {

typedef float Real;

// ---------------------------------------------------------------- learning rate / penalty / loss
template <typename V>
class LearningRate {
 public:
  LearningRate() {}
  explicit LearningRate(const LearningRateConfig& conf) : conf_(conf) {
    PS_CHECK_GT(conf.alpha, 0.0);
    PS_CHECK_GE(conf.beta, 0.0);
  }
  // alpha, or alpha / (x + beta)
  V eval(V x = 0) const { return conf_.type == LearningRateConfig::CONSTANT ? alpha() : alpha() / (x + beta()); }
  V alpha() const { return (V)conf_.alpha; }
  V beta() const { return (V)conf_.beta; }
 private:
  LearningRateConfig conf_;
};

template <typename T>
class Penalty {
 public:
  virtual ~Penalty() {}
  virtual T eval(const SArray<T>& model) = 0;
  // argmin_x 1/(2 eta) (x - z)^2 + h(x)
  virtual T proximal(T z, T eta) = 0;
};

// lambda1 |x|_1 + lambda2 |x|_2^2
template <typename T>
class ElasticNet : public Penalty<T> {
 public:
  ElasticNet(T lambda1, T lambda2) : lambda1_(lambda1), lambda2_(lambda2) {
    PS_CHECK_GE(lambda1, (T)0);
    PS_CHECK_GE(lambda2, (T)0);
  }
  T eval(const SArray<T>& w) override {
    double l1 = 0, l2 = 0;
    for (size_t i = 0; i < w.size(); ++i) { l1 += std::fabs(w[i]); l2 += (double)w[i] * w[i]; }
    return (T)(lambda1_ * l1 + lambda2_ * l2);
  }
  T proximal(T z, T eta) override {
    T leta = lambda1_ * eta;
    if (z <= leta && z >= -leta) return 0;
    return z > 0 ? (z - leta) / (1 + lambda2_ * eta) : (z + leta) / (1 + lambda2_ * eta);
  }
  T lambda1() const { return lambda1_; }
  T lambda2() const { return lambda2_; }
 private:
  T lambda1_, lambda2_;
};

template <typename T>
std::shared_ptr<Penalty<T>> createPenalty(const PenaltyConfig& conf) {
  PS_CHECK_GE(conf.lambda.size(), (size_t)1) << "penalty needs at least one lambda";
  if (conf.type == PenaltyConfig::L1)
    return std::make_shared<ElasticNet<T>>((T)conf.lambda[0], conf.lambda.size() > 1 ? (T)conf.lambda[1] : (T)0);
  return std::make_shared<ElasticNet<T>>((T)0, (T)conf.lambda[0]);
}

template <typename T>
class Loss {
 public:
  virtual ~Loss() {}
  // objective value given labels and margins Xw
  virtual T evaluate(const SArray<T>& y, const SArray<T>& Xw) = 0;
  // gradient X'(dl/dm) and (optionally) the diagonal Hessian (X.X)'(d2l/dm2)
  virtual void compute(const SArray<T>& y, const Matrix<T>& X, const SArray<T>& Xw, SArray<T>* gradient,
                       SArray<T>* diag_hessian = nullptr) = 0;
};

template <typename T>
class LogitLoss : public Loss<T> {
 public:
  T evaluate(const SArray<T>& y, const SArray<T>& Xw) override {
    double s = 0;
    for (size_t i = 0; i < y.size(); ++i) {
      double ym = (double)y[i] * Xw[i];
      s += ym > 0 ? std::log1p(std::exp(-ym)) : -ym + std::log1p(std::exp(ym));
    }
    return (T)s;
  }
  void compute(const SArray<T>& y, const Matrix<T>& X, const SArray<T>& Xw, SArray<T>* gradient,
               SArray<T>* diag_hessian = nullptr) override {
    size_t n = y.size();
    SArray<T> coef(n), h(diag_hessian ? n : 0);
    for (size_t i = 0; i < n; ++i) {
      T tau = 1 / (1 + std::exp(y[i] * Xw[i]));
      coef[i] = -y[i] * tau;
      if (diag_hessian) h[i] = tau * (1 - tau);
    }
    if (gradient) { gradient->resize(X.cols()); X.transTimes(coef.data(), gradient->data()); }
    if (diag_hessian) {
      diag_hessian->resize(X.cols());
      auto* sp = dynamic_cast<const SparseMatrix<uint32_t, T>*>(&X);
      PS_CHECK(sp != nullptr);
      sp->dotTimes(h.data(), diag_hessian->data(), true);
    }
  }
};

template <typename T>
class SquareHingeLoss : public Loss<T> {
 public:
  T evaluate(const SArray<T>& y, const SArray<T>& Xw) override {
    double s = 0;
    for (size_t i = 0; i < y.size(); ++i) { double h = std::max(0.0, 1.0 - (double)y[i] * Xw[i]); s += h * h; }
    return (T)s;
  }
  void compute(const SArray<T>& y, const Matrix<T>& X, const SArray<T>& Xw, SArray<T>* gradient,
               SArray<T>* diag_hessian = nullptr) override {
    size_t n = y.size();
    SArray<T> coef(n);
    for (size_t i = 0; i < n; ++i) coef[i] = -2 * y[i] * std::max((T)0, 1 - y[i] * Xw[i]);
    if (gradient) { gradient->resize(X.cols()); X.transTimes(coef.data(), gradient->data()); }
    (void)diag_hessian;
  }
};

template <typename T>
std::shared_ptr<Loss<T>> createLoss(const LossConfig& conf) {
  if (conf.type == LossConfig::LOGIT) return std::make_shared<LogitLoss<T>>();
  if (conf.type == LossConfig::SQUARE_HINGE) return std::make_shared<SquareHingeLoss<T>>();
  PS_CHECK(false) << "unsupported loss type " << conf.type;
  return nullptr;
}

// ================================================================= async SGD
class AsyncSGDScheduler : public ISGDScheduler {
 public:
  AsyncSGDScheduler(const Config& conf, Postoffice* po) : ISGDScheduler(po), conf_(conf) {
    Workload load;
    load.data = conf.training_data;
    load.data.ignore_feature_group = true;
    load.replica = conf.async_sgd.num_data_pass;
    load.shuffle = true;
    pool_.set(load);
    workload_pool_ = &pool_;
  }
 private:
  Config conf_;
  WorkloadPool pool_;
};

// per-server optimiser state shared by all entries + progress counters
template <typename V>
struct SGDState {
  SGDState() {}
  SGDState(const PenaltyConfig& h_conf, const LearningRateConfig& lr_conf)
      : lr(std::make_shared<LearningRate<V>>(lr_conf)), h(createPenalty<V>(h_conf)) {}
  // called once per push message: send the counters to the scheduler
  void Update() {
    if (!reporter) return;
    SGDProgress prog;
    prog.nnz = nnz;
    prog.weight_sum = weight_sum; weight_sum = 0;
    prog.delta_sum = delta_sum; delta_sum = 0;
    reporter->Report(prog);
  }
  void UpdateWeight(V new_w, V old_w) {
    if (new_w == 0 && old_w != 0) --nnz;
    else if (new_w != 0 && old_w == 0) ++nnz;
    weight_sum += (double)new_w * new_w;
    double d = (double)new_w - old_w;
    delta_sum += d * d;
  }
  std::shared_ptr<LearningRate<V>> lr;
  std::shared_ptr<Penalty<V>> h;
  size_t nnz = 0;
  double weight_sum = 0, delta_sum = 0;
  MonitorSlaver<SGDProgress>* reporter = nullptr;
};

// The per-key update rules of the server. An entry is three numbers (the weight and two rule
// specific accumulators) plus a rule; the step functions below are the same arithmetic, in the same
// order of operations, as the device table's opt_step (csrc/cuda/table.cu), so the CPU application
// can serve as the oracle of the GPU one.
//   FTRL-proximal (McMahan et al.): acc0 = z, acc1 = sqrt(n);  sigma = (sqrt(n + g^2) - sqrt(n)) / alpha,
//       z += g - sigma * w,  w = prox(-z * eta, eta) with eta = lr(sqrt(n))
//   AdaGrad:  acc0 = sum of g^2;  w = prox(w - eta * g, eta) with eta = lr(sqrt(acc0))
//   SGD:      acc0 = number of updates of the key;  w = prox(w - eta * g, eta) with eta = lr(sqrt(acc0))
enum class UpdateRule { kFtrl, kAdaGrad, kSgd };

template <typename V>
struct EntryCells { V w = 0, acc0 = 0, acc1 = 0; };

template <typename V>
inline void StepFtrl(EntryCells<V>* e, V g, LearningRate<V>& lr, Penalty<V>& h) {
  const V root_after = std::sqrt(e->acc1 * e->acc1 + g * g);
  e->acc0 += g - (root_after - e->acc1) / lr.alpha() * e->w;
  e->acc1 = root_after;
  const V eta = lr.eval(root_after);
  e->w = h.proximal(-e->acc0 * eta, eta);
}
template <typename V>
inline void StepAdaGrad(EntryCells<V>* e, V g, LearningRate<V>& lr, Penalty<V>& h) {
  e->acc0 += g * g;
  const V eta = lr.eval(std::sqrt(e->acc0));
  e->w = h.proximal(e->w - eta * g, eta);
}
template <typename V>
inline void StepSgd(EntryCells<V>* e, V g, LearningRate<V>& lr, Penalty<V>& h) {
  e->acc0 += 1;
  const V eta = lr.eval(std::sqrt(e->acc0));
  e->w = h.proximal(e->w - eta * g, eta);
}

// KVMap entry (Get / Set as parameter/kv_map.h:43-59 asks for) applying one rule.
template <typename V, UpdateRule R>
struct RuleEntry {
  EntryCells<V> cells;
  void Set(const V* grad, void* state) {
    auto* st = static_cast<SGDState<V>*>(state);
    const V before = cells.w;
    switch (R) {
      case UpdateRule::kFtrl: StepFtrl(&cells, *grad, *st->lr, *st->h); break;
      case UpdateRule::kAdaGrad: StepAdaGrad(&cells, *grad, *st->lr, *st->h); break;
      case UpdateRule::kSgd: StepSgd(&cells, *grad, *st->lr, *st->h); break;
    }
    st->UpdateWeight(cells.w, before);
  }
  void Get(V* out, void*) { *out = cells.w; }
};
template <typename V> using FTRLEntry = RuleEntry<V, UpdateRule::kFtrl>;
template <typename V> using AdaGradEntry = RuleEntry<V, UpdateRule::kAdaGrad>;
template <typename V> using SGDEntry = RuleEntry<V, UpdateRule::kSgd>;

static const int kModelCustomerID = 20;

template <typename V>
class AsyncSGDServer : public ISGDCompNode {
 public:
  AsyncSGDServer(const Config& conf, Postoffice* po) : ISGDCompNode(po), conf_(conf) {
    SGDState<V> state(conf.penalty, conf.learning_rate);
    state.reporter = &reporter_;
    if (conf.async_sgd.algo == SGDConfig::FTRL) {
      auto m = new KVMap<Key, V, FTRLEntry<V>, SGDState<V>>(1, kModelCustomerID, po);
      m->set_state(state);
      model_.reset(m);
    } else if (conf.async_sgd.ada_grad) {
      auto m = new KVMap<Key, V, AdaGradEntry<V>, SGDState<V>>(1, kModelCustomerID, po);
      m->set_state(state);
      model_.reset(m);
    } else {
      auto m = new KVMap<Key, V, SGDEntry<V>, SGDState<V>>(1, kModelCustomerID, po);
      m->set_state(state);
      model_.reset(m);
    }
  }
  void ProcessRequest(Message* request) override {
    if (request->task.has_sgd && request->task.sgd.cmd == SGDCall::SAVE_MODEL) {
      PS_CHECK(conf_.has_model_output && !conf_.model_output.file.empty()) << "no model_output in the configuration";
      std::string file = conf_.model_output.file[0] + "_" + sys_->manager().van().my_node().id;
      model_->WriteToFile(file);
      PS_VLOG(1) << "model written to " << file;
    }
  }
 private:
  Config conf_;
  std::unique_ptr<Parameter> model_;
};

template <typename V>
class AsyncSGDWorker : public ISGDCompNode {
 public:
  AsyncSGDWorker(const Config& conf, Postoffice* po)
      : ISGDCompNode(po), conf_(conf), model_(false, 1, kModelCustomerID, po), loss_(createLoss<V>(conf.loss)) {}
  void Run() override {
    // ask for the first workload
    Task task;
    task.mutable_sgd()->cmd = SGDCall::REQUEST_WORKLOAD;
    Submit(task, sys_->manager().van().scheduler().id);
  }
  void ProcessRequest(Message* request) override {
    const Task& t = request->task;
    if (t.has_sgd && t.sgd.cmd == SGDCall::UPDATE_MODEL) {
      UpdateModel(t.sgd.load);
      // the response tells the scheduler which workload is done
      Task done;
      done.mutable_sgd()->cmd = SGDCall::UPDATE_MODEL;
      done.sgd.has_load = true;
      done.sgd.load.id = t.sgd.load.id;
      done.sgd.load.finished = true;
      Reply(request, done);
    }
  }
  size_t minibatches_processed() const { return processed_batch_; }
 private:
  struct Batch { SArray<V> y; std::shared_ptr<SparseMatrix<uint32_t, V>> X; SArray<Key> key; };

  void UpdateModel(const Workload& load) {
    const SGDConfig& sgd = conf_.async_sgd;
    MinibatchReader<V> reader;
    reader.InitReader(load.data, sgd.minibatch, sgd.data_buf);
    if (sgd.tail_feature_freq > 0) reader.InitFilter((size_t)sgd.countmin_n, sgd.countmin_k, sgd.tail_feature_freq);
    reader.Start();
    processed_batch_ = 0;
    int id = 0;
    const int tau = sgd.max_delay;
    for (;; ++id) {
      auto b = std::make_shared<Batch>();
      if (!reader.Read(&b->y, &b->X, &b->key)) break;
      { Lock l(mu_); batch_[id] = b; }
      // bounded delay: at most tau+1 minibatches without an acknowledged push (0 = unbounded)
      if (tau > 0) {
        ULock l(mu_);
        cv_.wait(l, [this, id, tau] { return (int)processed_batch_ + tau >= id; });
      }
      Task pull = Parameter::Request(id, -1, {}, sgd.pull_filter);
      model_[id].key = b->key;
      model_.Pull(pull, b->key, [this, id] { ComputeGradient(id); });
    }
    // wait until every push has been acknowledged
    ULock l(mu_);
    cv_.wait(l, [this, id] { return (int)processed_batch_ >= id; });
  }

  // runs on the model's executor thread when the pulled weights have arrived
  void ComputeGradient(int id) {
    std::shared_ptr<Batch> b;
    { Lock l(mu_); b = batch_[id]; batch_.erase(id); }
    SArray<V> w = model_[id].value;
    if (w.size() != b->key.size()) { w.resize(b->key.size()); w.SetZero(); }
    SArray<V> Xw(b->y.size());
    b->X->times(w.data(), Xw.data());
    // progress
    SGDProgress prog;
    prog.objective.push_back(loss_->evaluate(b->y, Xw));
    prog.auc.push_back(Evaluation<V>::auc(b->y, Xw));
    prog.accuracy.push_back(Evaluation<V>::accuracy(b->y, Xw));
    prog.num_examples_processed = b->y.size();
    reporter_.Report(prog);
    // minibatch *sum* of the gradients
    SArray<V> grad(b->X->cols());
    loss_->compute(b->y, *b->X, Xw, &grad);
    Task push = Parameter::Request(id, -1, {}, conf_.async_sgd.push_filter);
    model_.Push(push, b->key, {grad}, [this] { { Lock l(mu_); ++processed_batch_; } cv_.notify_all(); });
    model_.Clear(id);
  }

  Config conf_;
  KVVector<Key, V> model_;
  std::shared_ptr<Loss<V>> loss_;
  std::unordered_map<int, std::shared_ptr<Batch>> batch_;
  std::mutex mu_;
  std::condition_variable cv_;
  size_t processed_batch_ = 0;
};

// ================================================================= model evaluation
class ModelEvaluation : public App {
 public:
  ModelEvaluation(const Config& conf, Postoffice* po) : App(po), conf_(conf) {}
  void Run() override;
  double auc = 0, accuracy = 0, logloss = 0;
  size_t num_examples = 0, num_weights = 0;
 private:
  Config conf_;
};

// ================================================================= Darlin (see darlin.cc)
App* CreateDarlin(const Config& conf, Postoffice* po);

// role-dependent application object for a configuration text
App* CreateLinearMethod(const std::string& conf_text, Postoffice* po);

}  // namespace LM
}  // namespace PS
